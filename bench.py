#!/usr/bin/env python
"""Benchmark of the ternary / binary conv hot path (quantise+pack+im2row -> bitwise GEMM + PReLU).

    python bench.py --gpus N --steps K --warmup W            # this library, one rank per GPU
    python bench.py --impl reference --gpus N --steps K ...   # the reference's CPU code path
    python bench.py --workload tnn_stack | tbn_conv_56 | e2e_resnet18 | ...

Default workload: the large single TNN conv layer -- batch 64, 512 channels, 32x32, 512 kernels
3x3, stride 1, pad 1 (M=65536, K=4608, N=512), activations uniform in [-1,1), thresholds +-0.25,
ternary weights, PReLU alpha 0.5.  Rows of the im2row matrix are independent, so the layer is
partitioned by batch index with the weights replicated and no collective on the data path.
Default "scaling": "strong": the job is the configured batch at every N, each rank owns batch/N of
its images; the weak figure (every rank processes the configured batch) is reported alongside, and
--scaling weak makes it the headline.  One "step" is one pass of the job's batch.
Metric: GOPS = 2*M*N*K / time (unpadded K).

Prints ONE JSON line on rank 0.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import sys
import threading
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))

import numpy as np  # noqa: E402

from fastertnn_b200 import synth  # noqa: E402
from fastertnn_b200.shard import batch_slice  # noqa: E402
from fastertnn_b200.workloads import (CONV_LARGE, CONV_56, FC_GEMM, RESNET18_STACK, RESNET18_STACK_BATCH,  # noqa: E402
                                      REFERENCE_MODEL_BATCH, Layer, model_layers, model_names)

TNN, TBN, BTN, BNN = 0, 1, 2, 3
TYPE_NAMES = {TNN: "tnn", TBN: "tbn", BTN: "btn", BNN: "bnn"}
METRIC = "ternary conv GOPS (2*M*N*K/s)"
L2_BYTES = 126 * 1024 * 1024
SEED_X, SEED_W = 0xC0FFEE40, 0xC0FFEE41

# name -> (kind, network type, batch, layer or list of layers)
WORKLOADS = {
    "tnn_conv_large": ("layer", TNN, *CONV_LARGE),   # batch 64, 512x32x32 -> 512, 3x3 s1 p1
    "tnn_conv_56": ("layer", TNN, *CONV_56),         # batch 1, 256x56x56 -> 256
    "tbn_conv_56": ("layer", TBN, *CONV_56),         # ternary activations x binary weights
    "btn_conv_56": ("layer", BTN, *CONV_56),         # binary activations x ternary weights
    "tnn_fc": ("layer", TNN, *FC_GEMM),              # 1024 x 4096 -> 1024
    "tnn_stack": ("stack", TNN, RESNET18_STACK_BATCH, RESNET18_STACK),  # 11 layers, batch 256
}
for _m in model_names():  # the reference's end-to-end model tables, batch 8 as in its driver
    WORKLOADS["e2e_" + _m] = ("stack", TNN, REFERENCE_MODEL_BATCH, model_layers(_m))


def act_ternary(t):
    return t in (TNN, TBN)


def wgt_ternary(t):
    return t in (TNN, BTN)


def peaks():
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        d = json.loads(p.read_text())
        return {"hbm_gbs": d["hbm_gbs"], "bf16_tflops": d["bf16_tflops"], "bf16_tflops_sustained": d["bf16_tflops_sustained"],
                "source": "measured"}
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0, "source": "fallback"}


def ncu_traffic(workload: str, kernel_key: str):
    """dram__bytes_read.sum + dram__bytes_write.sum per processed image, from the ncu captures
    summarised under profiles/ (profiles/dram_traffic.json is written by
    `python -m fastertnn_b200.profile_summary` from a capture)."""
    p = ROOT / "profiles" / "dram_traffic.json"
    if not p.exists():
        return None
    e = json.loads(p.read_text()).get(workload, {}).get(kernel_key)
    return e["dram_bytes_per_image"] if e else None


def layer_weights(type_: int, layer: Layer, seed: int = SEED_W):
    shape_w = (layer.KN, layer.C, layer.KH, layer.KW)
    w = synth.ternary_values(seed, shape_w) if wgt_ternary(type_) else synth.binary_values(seed, shape_w)
    return w, np.full(layer.KN, 0.5 if wgt_ternary(type_) else 0.0, np.float32)


def layer_inputs(type_: int, layer: Layer, n0: int, n1: int):
    """Images n0..n1 of the seeded batch and their thresholds."""
    per = layer.C * layer.H * layer.W
    x = synth.uniform_pm1(SEED_X, (n1 - n0, layer.C, layer.H, layer.W), offset=n0 * per)
    thr = np.full(n1 - n0, 0.25 if act_ternary(type_) else 0.0, np.float32)
    return x, thr


def common_config(name, kind, type_, batch, layers, scaling, layout="nchw"):
    """The keys both arms print, with the same values: what is computed, not how."""
    L = layers[0]
    cfg = {"workload": name, "type": TYPE_NAMES[type_], "batch": batch, "layout": layout.upper(), "scaling": scaling}
    if kind == "layer":
        cfg.update({"layer": str(L), "M": batch * L.OH * L.OW, "K": L.C * L.KH * L.KW, "N": L.KN})
    else:
        cfg.update({"layers": len(layers), "first_layer": str(layers[0]), "last_layer": str(layers[-1]),
                    "giga_ops": sum(x.ops(batch) for x in layers) / 1e9})
    return cfg


# ------------------------------------------------------------------------------------------------
# clocks sampled during the timed regions
# ------------------------------------------------------------------------------------------------
class ClockSampler:
    REASONS = {0x8: "hw_slowdown", 0x40: "hw_thermal_slowdown", 0x20: "sw_thermal_slowdown", 0x4: "sw_power_cap",
               0x80: "hw_power_brake_slowdown"}

    def __init__(self, uuid: str | None, period: float = 0.01):
        self.samples, self.reasons, self.max_mhz, self.period = [], set(), None, period
        self._stop = threading.Event()
        self._thread = None
        self._h = None
        try:
            import pynvml
            pynvml.nvmlInit()
            self._nv = pynvml
            h = None
            if uuid:
                for cand in (uuid, "GPU-" + uuid):
                    try:
                        h = pynvml.nvmlDeviceGetHandleByUUID(cand.encode() if isinstance(cand, str) else cand)
                        break
                    except Exception:
                        continue
            self._h = h or pynvml.nvmlDeviceGetHandleByIndex(0)
            self.max_mhz = pynvml.nvmlDeviceGetMaxClockInfo(self._h, pynvml.NVML_CLOCK_SM)
        except Exception:
            self._h = None

    def _run(self):
        nv = self._nv
        while not self._stop.is_set():
            try:
                self.samples.append(nv.nvmlDeviceGetClockInfo(self._h, nv.NVML_CLOCK_SM))
                r = nv.nvmlDeviceGetCurrentClocksEventReasons(self._h)
                for bit, name in self.REASONS.items():
                    if r & bit:
                        self.reasons.add(name)
            except Exception:
                pass
            self._stop.wait(self.period)

    def start(self):
        if self._h is not None and self._thread is None:
            self._stop.clear()
            self._thread = threading.Thread(target=self._run, daemon=True)
            self._thread.start()

    def stop(self):
        if self._thread is not None:
            self._stop.set()
            self._thread.join()
            self._thread = None

    def mark(self) -> int:
        return len(self.samples)

    def median_since(self, mark: int):
        s = self.samples[mark:]
        return statistics.median(s) if s else None

    def summary(self):
        if not self.samples:
            return {"sm_mhz": None, "sm_max_mhz": self.max_mhz, "reasons": sorted(self.reasons), "samples": 0}
        return {"sm_mhz": statistics.median(self.samples), "sm_max_mhz": self.max_mhz, "reasons": sorted(self.reasons),
                "samples": len(self.samples)}


# ------------------------------------------------------------------------------------------------
# CPU reference (the reference's own AVX2 objects when built, else the restatement)
# ------------------------------------------------------------------------------------------------
def cpu_conv(chk, type_, x, thr, wp, layer: Layer, threads: int):
    """One layer over the batch, images spread over `threads` host threads (the reference code is
    single-threaded and re-entrant; the binding releases the GIL during the call)."""
    from concurrent.futures import ThreadPoolExecutor
    N = x.shape[0]
    T = max(1, min(threads, N))
    bounds = [batch_slice(N, r, T) for r in range(T)]

    def run(b):
        a, e = b
        return chk.conv(type_, x[a:e], thr[a:e], wp, (layer.KH, layer.KW), (layer.P, layer.P), (layer.S, layer.S), 0.5)

    if T == 1:
        return run(bounds[0])
    with ThreadPoolExecutor(T) as ex:
        return np.concatenate(list(ex.map(run, bounds)), axis=0)


def cpu_chain(chk, type_, x, thr, pws, layers, threads: int):
    """The reference's end-to-end protocol (src/timing_layers.c:186-202 of the reference): every layer's
    output buffer is the next layer's input, read with the next layer's shape."""
    N = x.shape[0]
    cur = x
    for L, pw in zip(layers, pws):
        need = N * L.C * L.H * L.W
        if cur.shape != (N, L.C, L.H, L.W):
            cur = np.ascontiguousarray(cur.reshape(-1)[:need]).reshape(N, L.C, L.H, L.W)
        cur = cpu_conv(chk, type_, cur, thr, pw, L, threads)
    return cur


class CpuWorkload:
    """The workload (or a bounded sample of it) for the CPU legs: cpu_baseline and --impl reference."""

    def __init__(self, kind, type_, batch, layers, sample_batch):
        from oracle import binding
        self.chk = binding.best()
        self.kind, self.type, self.layers = kind, type_, layers
        self.N = min(batch, sample_batch)
        self.full_batch = batch
        L0 = layers[0]
        if kind == "layer":
            self.x, self.thr = layer_inputs(type_, L0, 0, self.N)
        else:
            self.x = synth.uniform_pm1(SEED_X + 0x10, (self.N, L0.C, L0.H, L0.W))
            self.thr = np.full(self.N, 0.25 if act_ternary(type_) else 0.0, np.float32)
        self.pws = []
        for i, L in enumerate(layers):
            w, wt = layer_weights(type_, L, SEED_W + (0x10 + i if kind == "stack" else 0))
            self.pws.append(self.chk.pack_weights(wgt_ternary(type_), w, wt))
        self.ops = sum(L.ops(self.N) for L in layers)

    def run(self, threads: int):
        t0 = time.perf_counter()
        cpu_chain(self.chk, self.type, self.x, self.thr, self.pws, self.layers, threads)
        return time.perf_counter() - t0

    def describe(self, threads: int) -> str:
        what = "layer" if self.kind == "layer" else f"{len(self.layers)}-layer chain"
        part = "the full" if self.N == self.full_batch else f"a {self.N}-image sample of the"
        return f"one pass of the {what} over {part} {self.full_batch}-image batch, images split over {min(threads, self.N)} host threads"


def cpu_baseline(kind, type_, batch, layers, passes: int):
    threads = os.cpu_count() or 1
    ops_full = sum(L.ops(batch) for L in layers)
    # bound the sample to a few seconds of CPU work at ~2 TOP/s over all threads
    sample = batch if ops_full < 6e12 else max(threads, int(batch * 6e12 / ops_full))
    wl = CpuWorkload(kind, type_, batch, layers, sample)
    wl.run(threads)  # warm-up
    t = statistics.mean(wl.run(threads) for _ in range(passes))
    # the reference's design point: ONE pinned core (its Makefile runs every binary under taskset -c 0)
    one_n = max(1, min(wl.N, int(wl.N * 1.0e11 / max(wl.ops, 1)) or 1))   # about 0.5 s at ~200 GOPS
    one = CpuWorkload(kind, type_, batch, layers, one_n)
    one.run(1)
    t1 = statistics.mean(one.run(1) for _ in range(max(2, passes // 2)))
    return {"value": wl.ops / t / 1e9, "unit": "GOPS", "cores": min(threads, wl.N), "kind": wl.chk.kind,
            "sample": f"{passes} x {wl.describe(threads)}, mean {t * 1e3:.1f} ms per pass",
            "one_core": {"value": one.ops / t1 / 1e9, "unit": "GOPS", "cores": 1,
                         "sample": f"{one.describe(1)} on one host thread, mean {t1 * 1e3:.1f} ms per pass "
                                   "(the reference's own design point: single-threaded, pinned to one core)"}}


def run_reference(args, name, kind, type_, batch, layers):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return  # the reference is a CPU code path: rank 0 alone runs it
    threads = os.cpu_count() or 1
    N_job = batch * (args.gpus if args.scaling == "weak" else 1)
    ops_full = sum(L.ops(N_job) for L in layers)
    sample = N_job if ops_full < 1.5e12 else max(threads, int(N_job * 1.5e12 / ops_full))
    wl = CpuWorkload(kind, type_, N_job, layers, sample)
    for _ in range(args.warmup):
        wl.run(threads)
    t = statistics.mean(wl.run(threads) for _ in range(args.steps))
    val = wl.ops / t / 1e9
    used = min(threads, wl.N)
    line = {
        "impl": "reference", "metric": METRIC, "value": val, "unit": "GOPS", "n_gpus": args.gpus, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": t * 1e3, "higher_is_better": True, "scaling": args.scaling, "vs_baseline": None,
        "dtype": "int (64-bit popcount lanes)", "data": "synthetic",
        "config": common_config(name, kind, type_, N_job, layers, args.scaling, args.layout if kind == "layer" else "nchw"),
        "impl_config": {"batch_timed_per_step": wl.N, "host_threads": used, "code": wl.chk.kind,
                        "note": "GOPS = operations of the images actually processed per step / time; the CPU path has no GPUs to "
                                "shard over, so n_gpus only names the run it is compared with"},
        "cpu_baseline": {"value": val, "unit": "GOPS", "cores": used, "kind": wl.chk.kind, "sample": "each step = " + wl.describe(threads)},
        "e2e": {"value": val, "unit": "GOPS", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    print(json.dumps(line), flush=True)


# ------------------------------------------------------------------------------------------------
# this library
# ------------------------------------------------------------------------------------------------
class Dist:
    def __init__(self, args):
        import torch
        self.torch = torch
        self.rank = int(os.environ.get("RANK", "0"))
        self.world = int(os.environ.get("WORLD_SIZE", "1"))
        self.local = int(os.environ.get("LOCAL_RANK", "0"))
        if self.world != args.gpus:
            raise SystemExit(f"--gpus {args.gpus} but WORLD_SIZE={self.world}: launch with torch.distributed.run --nproc-per-node {args.gpus}")
        if not torch.cuda.is_available():
            raise SystemExit("no CUDA device: this benchmark has no CPU fallback")
        torch.cuda.set_device(self.local)
        self.dist = None
        if self.world > 1:
            import torch.distributed as dist
            dist.init_process_group("nccl", device_id=torch.device("cuda", self.local))
            self.dist = dist

    def barrier(self):
        if self.dist:
            self.dist.barrier()
        self.torch.cuda.synchronize()

    def max_over_ranks(self, v: float) -> float:
        if not self.dist:
            return v
        t = self.torch.tensor([v], device="cuda", dtype=self.torch.float64)
        self.dist.all_reduce(t, op=self.dist.ReduceOp.MAX)
        return float(t.item())

    def host_signal(self, key: str):
        """Rank 0 tells the other ranks, through the rendezvous store, that it is done with `key`."""
        if self.dist:
            self.dist.distributed_c10d._get_default_store().set(key, "1")

    def host_wait(self, key: str):
        """Waits on the HOST for host_signal(key): unlike a NCCL barrier no kernel spins on this
        rank's GPU meanwhile, so rank 0 can use every GPU of the run undisturbed."""
        if self.dist:
            self.dist.distributed_c10d._get_default_store().wait([key])

    def all_true(self, ok: bool) -> bool:
        return self.max_over_ranks(0.0 if ok else 1.0) == 0.0

    def close(self):
        if self.dist:
            self.dist.destroy_process_group()


def timed_region(D: Dist, stream, step, steps: int, first: int = 0):
    """K steps between two events on the launching stream; ms in total, max over ranks."""
    torch = D.torch
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    D.barrier()
    e0.record(stream)
    for i in range(steps):
        step(first + i)
    e1.record(stream)
    stream.synchronize()
    D.barrier()
    return D.max_over_ranks(e0.elapsed_time(e1))


def sustained_regions(D: Dist, stream, step, steps: int, ms_step: float, sampler, seconds: float = 1.0):
    """The K-step region repeated back to back for about `seconds` of GPU time: the burst figure of
    a 2 ms run says nothing about what the part holds under its power cap."""
    torch = D.torch
    R = max(3, min(4000, int(seconds * 1e3 / max(ms_step * steps, 1e-3)) + 1))
    evs = [torch.cuda.Event(enable_timing=True) for _ in range(R + 1)]
    mark = sampler.mark() if sampler else 0
    D.barrier()
    t0 = time.perf_counter()
    evs[0].record(stream)
    for r in range(R):
        for i in range(steps):
            step(r * steps + i)
        evs[r + 1].record(stream)
    stream.synchronize()
    wall = time.perf_counter() - t0
    D.barrier()
    per = sorted(evs[r].elapsed_time(evs[r + 1]) / steps for r in range(R))
    med = D.max_over_ranks(per[R // 2])
    mhz = sampler.median_since(mark) if sampler else None
    return {"seconds": wall, "regions": R, "steps_per_region": steps, "ms_per_step_median": med, "ms_per_step_min": per[0],
            "ms_per_step_p10": per[R // 10], "ms_per_step_p90": per[(9 * R) // 10], "ms_per_step_max": per[-1],
            "sm_mhz_median": mhz, "clock_samples": (sampler.mark() - mark) if sampler else 0,
            "ms_x_mhz": (med * mhz) if mhz else None}


def pcie_floor(torch, devices, in_bytes_each, out_bytes_each, reps=3):
    """Plain page-locked copies, up and down at once, on every device of the run: the time no
    host-buffer layer call can beat.  One upload and one download of a device's share per device."""
    bufs = []
    for d, bi, bo in zip(devices, in_bytes_each, out_bytes_each):
        with torch.cuda.device(d):
            bufs.append((torch.empty(max(bi, 4), dtype=torch.uint8).pin_memory(), torch.empty(max(bi, 4), dtype=torch.uint8, device=f"cuda:{d}"),
                         torch.empty(max(bo, 4), dtype=torch.uint8).pin_memory(), torch.empty(max(bo, 4), dtype=torch.uint8, device=f"cuda:{d}"),
                         torch.cuda.Stream(device=d), torch.cuda.Stream(device=d)))
    best = None
    for _ in range(reps + 1):
        for d in devices:
            torch.cuda.synchronize(d)
        t0 = time.perf_counter()
        for (hi, di, ho, do, s_up, s_dn) in bufs:
            with torch.cuda.stream(s_up):
                di.copy_(hi, non_blocking=True)
            with torch.cuda.stream(s_dn):
                ho.copy_(do, non_blocking=True)
        for d in devices:
            torch.cuda.synchronize(d)
        t = (time.perf_counter() - t0) * 1e3
        best = t if best is None else min(best, t)
    return best


class LayerRun:
    """One rank's share of a layer workload: a ring of distinct buffer sets (so consecutive steps
    never find their data in L2) and the launches of one step."""

    def __init__(self, D: Dist, ft, ctx, w, type_, layer: Layer, x_h, thr_h, nloc: int, args):
        torch = D.torch
        self.ft, self.ctx, self.w, self.type, self.layer, self.nloc, self.args = ft, ctx, w, type_, layer, nloc, args
        self.tern = act_ternary(type_)
        self.shape = layer.shape(nloc)
        OH, OW = layer.OH, layer.OW
        self.nhwc = getattr(args, "layout", "nchw") == "nhwc"
        self.layout = LO = ft.NHWC if self.nhwc else ft.NCHW
        self.in_bytes = nloc * layer.C * layer.H * layer.W * 4
        self.out_bytes = nloc * layer.KN * OH * OW * 4
        tc4 = args.gemm in ("auto", "f4tc")
        # the slab-fed route (stride-1 layers from a bordered 4-bit image): on request, or where the library's own rule takes it
        self.slab = tc4 and (args.route in ("slab", "slab_fused") or (args.route == "auto" and ctx.slab_auto(w, self.shape, 4096, LO) > 0))
        if self.slab and not ctx.slab_supported(w, self.shape):
            raise SystemExit("bench: this workload does not qualify for the slab-fed route")
        self.im2col = tc4 and not self.slab and args.route in ("auto", "im2col", "fused") and ctx.im2col_supported(w, self.shape)
        if args.route in ("im2col", "fused") and not self.im2col:
            raise SystemExit("bench: this workload does not qualify for the im2col tensor-copy route")
        self.implicit = tc4 and (self.slab or self.im2col or args.route in ("auto", "implicit"))
        self.fused = False
        if self.slab:
            self.fused = args.route == "slab_fused" or (args.route == "auto" and ctx.slab_auto(w, self.shape, 4096, LO) == 2)
        elif self.im2col and args.route in ("auto", "fused"):
            # the pointer only stands for the input's alignment here (torch allocations are 512-byte aligned)
            self.fused = (ctx.conv_fused_supported(w, self.shape, 4096, LO) if args.route == "fused"
                          else ctx.conv_fused_preferred(w, self.shape, 4096, LO))
        self.pack_bytes = (ft.api.slab_workspace_bytes(nloc, layer.C, layer.H, layer.W, layer.P, layer.P) if self.slab else
                           ft.api.fused_workspace_bytes(nloc, layer.C, layer.H, layer.W) if self.im2col else
                           ft.api.packed_image_bytes(self.tern, nloc, layer.C, layer.H, layer.W) if self.implicit
                           else ft.packed_bytes(type_, self.shape))
        self.step_bytes = self.in_bytes + self.out_bytes + self.pack_bytes
        self.ring = max(2, -(-3 * L2_BYTES // max(self.step_bytes, 1)))
        if self.nhwc and (args.route == "slab_fused" or not tc4):
            raise SystemExit("bench: NHWC input is measured on the tensor-core routes (not the one-launch slab form)")
        x0 = torch.from_numpy(x_h[:nloc]).cuda()
        if self.nhwc:
            x0 = x0.permute(0, 2, 3, 1).contiguous()
        self.xs, self.ys, self.ps = [], [], []
        for r in range(self.ring):
            # distinct data per ring slot: the images rotated
            self.xs.append(x0 if r == 0 else torch.roll(x0, shifts=r, dims=0))
            self.ys.append(torch.empty((nloc, OH, OW, layer.KN) if self.nhwc else (nloc, layer.KN, OH, OW), dtype=torch.float32, device="cuda"))
            self.ps.append(torch.empty(self.pack_bytes // 8 + 32, dtype=torch.int64, device="cuda"))
        self.thr_d = torch.from_numpy(thr_h[:nloc].copy()).cuda()
        self.stream = torch.cuda.Stream()
        self.sp = self.stream.cuda_stream
        self.gemm_algo = {"auto": ft.GEMM_AUTO, "popc": ft.GEMM_POPC_TILED, "i8tc": ft.GEMM_I8_TC, "f4tc": ft.GEMM_F4_TC}[args.gemm]
        self.launches_per_step = 1 if self.fused else 2
        # default route and default GEMM: the timed step is ONE call of the library's layer entry point
        # (tnns_cuda_conv_ws), which takes the same route by its own rule; the two halves are called
        # separately only in the instrumented pass that times them
        self.auto_call = args.route == "auto" and args.gemm == "auto"

    @staticmethod
    def _aligned(t):
        return (t.data_ptr() + 127) & ~127

    def quantise(self, r):
        ft, L = self.ft, self.layer
        if self.slab:
            self.ctx.quantise_e2m1_bordered(self.tern, self.xs[r].data_ptr(), self.thr_d.data_ptr(), self._aligned(self.ps[r]), self.nloc, L.C, L.H, L.W,
                                            L.P, L.P, self.layout, self.sp)
        elif self.im2col:
            self.ctx.quantise_e2m1(self.xs[r].data_ptr(), self.thr_d.data_ptr(), self._aligned(self.ps[r]), self.nloc, L.C, L.H, L.W, self.layout, self.sp)
        else:
            self.ctx.quantise(self.tern, self.xs[r].data_ptr(), self.thr_d.data_ptr(), self._aligned(self.ps[r]), self.nloc, L.C, L.H, L.W, self.layout, self.sp)

    def step(self, i, ev=None):
        ft, L, r = self.ft, self.layer, i % self.ring
        x, y, p = self.xs[r].data_ptr(), self.ys[r].data_ptr(), self._aligned(self.ps[r])
        if ev is None and self.auto_call:
            # the library's own layer call: one call into the library per step, its own choice of route
            self.ctx.conv_ws(self.w, x, self.thr_d.data_ptr(), y, p, self.pack_bytes, self.shape, 0.5, self.layout, ft.PACK_AUTO, ft.GEMM_AUTO, self.sp)
            return
        if ev:
            ev[0].record(self.stream)
        if self.fused:
            pass
        elif self.implicit:
            self.quantise(r)
        else:
            self.ctx.pack(self.tern, x, self.thr_d.data_ptr(), p, self.shape, self.layout, ft.PACK_AUTO, self.sp)
        if ev:
            ev[1].record(self.stream)
        if self.slab and self.fused:
            self.ctx.conv_slab(self.w, x, self.thr_d.data_ptr(), y, p, self.pack_bytes, self.shape, 0.5, 0, self.sp)
        elif self.slab:
            self.ctx.gemm_slab(self.w, p, y, self.shape, 0.5, self.layout, self.sp)
        elif self.fused:
            self.ctx.conv_ws(self.w, x, self.thr_d.data_ptr(), y, p, self.pack_bytes, self.shape, 0.5, self.layout, ft.PACK_AUTO, ft.GEMM_F4_FUSED, self.sp)
        elif self.im2col:
            self.ctx.gemm_im2col(self.w, p, y, self.shape, 0.5, self.layout, self.sp)
        elif self.implicit:
            self.ctx.gemm_implicit(self.w, p, y, self.shape, 0.5, self.layout, self.sp)
        else:
            self.ctx.gemm(self.w, p, y, self.nloc, L.OH, L.OW, 0.5, self.layout, self.gemm_algo, self.sp)
        if ev:
            ev[2].record(self.stream)

    def route_name(self):
        if self.slab:
            return ("one launch: quantise to a bordered 4-bit image inside the GEMM kernel, GEMM fed by one slab of pixels per tile for all filter taps"
                    if self.fused else "quantise to a bordered 4-bit image -> GEMM fed by one slab of pixels per tile for all filter taps")
        return ("one launch: quantise to a 4-bit image inside the GEMM kernel, GEMM fed by im2col tensor copies" if self.fused else
                "quantise to a 4-bit image -> GEMM fed by im2col tensor copies" if self.im2col else
                "quantise to bit planes -> GEMM with implicit im2row" if self.implicit else "pack (im2row matrix) -> GEMM")

    def kernel_key(self):
        if self.slab and self.args.gemm in ("auto", "f4tc"):
            return "f4_slab_fused" if self.fused else "f4_slab"
        return {"popc": "popc", "i8tc": "tc"}.get(self.args.gemm, "f4_fused" if self.fused else "f4_im2col" if self.im2col else
                                                 "f4" if self.implicit else "f4_explicit")

    def free(self):
        self.xs = self.ys = self.ps = None
        self.thr_d = None


def check_rank_slice(D: Dist, run: LayerRun, type_, layer, x_h, thr_h, wp):
    """Every rank compares the first and the last image of its own slice with the CPU checker."""
    from oracle import binding
    chk = binding.best()
    run.step(0)
    D.torch.cuda.synchronize()
    ok = True
    for n in sorted({0, run.nloc - 1}):
        want = chk.conv(type_, x_h[n:n + 1], thr_h[n:n + 1], wp, (layer.KH, layer.KW), (layer.P, layer.P), (layer.S, layer.S), 0.5)
        got = run.ys[0][n:n + 1]
        if run.nhwc:
            got = got.permute(0, 3, 1, 2).contiguous()
        ok = ok and got.cpu().numpy().tobytes() == want.tobytes()
    return ok


def run_layer(args, name, type_, N_cfg, layer: Layer):
    D = Dist(args)
    torch = D.torch
    import fastertnn_b200 as ft
    rank, world, local = D.rank, D.world, D.local
    strong = args.scaling == "strong"
    N_total = N_cfg if strong else N_cfg * world
    if N_total < world:
        raise SystemExit(f"bench: {N_total} images cannot be split over {world} ranks (use --scaling weak for batch-1 workloads)")
    n0, n1 = batch_slice(N_total, rank, world)
    nloc = n1 - n0
    # the rank's images of the seeded stream; the alongside measurement (the other scaling mode) needs
    # N_cfg (weak) or N_cfg / world (strong) images per rank, taken from the same place
    n_other = N_cfg if strong else batch_slice(N_cfg, rank, world)[1] - batch_slice(N_cfg, rank, world)[0]
    n_have = max(nloc, n_other)
    x_h, thr_h = layer_inputs(type_, layer, n0, n0 + n_have)
    w_f, w_thr = layer_weights(type_, layer)
    wp = (ft.pack_weights_ternary if wgt_ternary(type_) else ft.pack_weights_binary)(w_f, w_thr)
    ctx = ft.Context(local)
    w = ctx.upload_weights(type_, wp, layer.C, layer.KH, layer.KW)
    OH, OW = layer.OH, layer.OW

    run = LayerRun(D, ft, ctx, w, type_, layer, x_h, thr_h, nloc, args)
    stream = run.stream

    # correctness gate on every rank, on images of its own slice (not timed)
    if not args.no_check:
        ok = check_rank_slice(D, run, type_, layer, x_h, thr_h, wp)
        if not D.all_true(ok):
            raise SystemExit("bench: GPU output differs from the CPU checker on some rank; refusing to time a wrong kernel")

    sampler = ClockSampler(str(torch.cuda.get_device_properties(local).uuid)) if rank == 0 else None

    # ---- device-resident timing -----------------------------------------------------------
    for i in range(args.warmup):
        run.step(i)
    launches0 = ft.api.launch_count()
    if sampler:
        sampler.start()
    ms_total = timed_region(D, stream, run.step, args.steps, args.warmup)
    launches = ft.api.launch_count() - launches0
    ms_step = ms_total / args.steps
    # per-kernel times: the same K steps once more with events between the launches (kept out of the
    # timed region above: three event records per step cost several microseconds of a 90 us step)
    evs = [[torch.cuda.Event(enable_timing=True) for _ in range(3)] for _ in range(args.steps)]
    for i in range(args.steps):
        run.step(args.warmup + i, evs[i])
    stream.synchronize()
    D.barrier()
    t_pack = statistics.mean(e[0].elapsed_time(e[1]) for e in evs)
    t_gemm = statistics.mean(e[1].elapsed_time(e[2]) for e in evs)
    t_gemm_instrumented = t_gemm
    if run.fused:
        t_gemm = ms_step  # one launch per step: its average duration over the timed region is the step time itself
    sustained = None if args.no_sustained else sustained_regions(D, stream, run.step, args.steps, ms_step, sampler, args.sustain_seconds)
    # The first kernel of a step also pays for the previous GEMM's output still draining from L2 to
    # HBM.  Timed by itself (same ring of inputs, larger than L2) it shows what the kernel alone reaches.
    t_pack_alone = None
    if run.implicit and rank == 0:
        for i in range(3):
            run.quantise(i % run.ring)
        stream.synchronize()
        a0, a1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a0.record(stream)
        for i in range(args.steps):
            run.quantise(i % run.ring)
        a1.record(stream)
        stream.synchronize()
        t_pack_alone = a0.elapsed_time(a1) / args.steps
    if sampler:
        sampler.stop()
    ctx_lop3_rate = ctx.pipe_rate(0) if args.gemm == "popc" else 0.0
    # issue-bound tcgen05.mma loop (no loads, no epilogue) on this GPU, 1e9 operations per second
    ctx_mma_rate = ctx.pipe_rate(3 if args.gemm == "i8tc" else 4) if args.gemm != "popc" else 0.0
    ctx.sync()
    info = {"route": run.route_name(), "key": run.kernel_key(), "fused": run.fused, "im2col": run.im2col, "implicit": run.implicit, "slab": run.slab,
            "ring": run.ring, "step_bytes": run.step_bytes, "in_bytes": run.in_bytes, "out_bytes": run.out_bytes,
            "pack_bytes": run.pack_bytes}
    y0_dev = run.ys[0][:1].cpu()
    run.free()
    del run
    torch.cuda.empty_cache()

    # ---- the other scaling mode alongside (multi-GPU runs only) --------------------------------
    other = None
    if world > 1 and n_other > 0:
        run2 = LayerRun(D, ft, ctx, w, type_, layer, x_h, thr_h, n_other, args)
        for i in range(args.warmup):
            run2.step(i)
        o_ms = timed_region(D, run2.stream, run2.step, args.steps, args.warmup) / args.steps
        N_other_total = N_cfg * world if strong else N_cfg
        other = {"scaling": "weak" if strong else "strong", "batch": N_other_total, "batch_per_gpu": n_other, "ms_per_step": o_ms,
                 "value": layer.ops(N_other_total) / (o_ms * 1e-3) / 1e9, "unit": "GOPS", "route": run2.route_name()}
        run2.free()
        del run2
        torch.cuda.empty_cache()

    # ---- the same job in the other memory layout alongside (default route only): the layer configurations are worded
    # for pixel-major (NHWC) tensors, the reference's C API takes NCHW; both go through the same kernels
    other_layout = None
    if args.route == "auto" and args.gemm == "auto" and layer.C % 4 == 0:
        args2 = argparse.Namespace(**vars(args))
        args2.layout = "nhwc" if args.layout == "nchw" else "nchw"
        run3 = LayerRun(D, ft, ctx, w, type_, layer, x_h, thr_h, nloc, args2)
        ok3 = True if args.no_check else check_rank_slice(D, run3, type_, layer, x_h, thr_h, wp)
        if not D.all_true(ok3):
            raise SystemExit("bench: GPU output in the other layout differs from the CPU checker on some rank")
        for i in range(args.warmup):
            run3.step(i)
        l_ms = timed_region(D, run3.stream, run3.step, args.steps, args.warmup) / args.steps
        other_layout = {"layout": args2.layout.upper(), "ms_per_step": l_ms, "value": layer.ops(N_total) / (l_ms * 1e-3) / 1e9, "unit": "GOPS",
                        "route": run3.route_name()}
        run3.free()
        del run3
        torch.cuda.empty_cache()

    # ---- end to end: ONE host batch in, host buffers out, copies inside the timed region --------
    # through the library call that takes a host batch: tnns_cuda_conv_host on one GPU,
    # tnns_cuda_multi_conv_host (one host thread per device behind one call) on several; rank 0 makes
    # the call for the whole job, the other ranks' processes stay idle meanwhile
    e2e = None
    D.barrier()
    if rank == 0:
        xj, tj = layer_inputs(type_, layer, 0, N_total)
        nhwc = args.layout == "nhwc"
        LO = ft.NHWC if nhwc else ft.NCHW
        x_pin = torch.from_numpy(np.ascontiguousarray(xj.transpose(0, 2, 3, 1)) if nhwc else xj).pin_memory()
        t_pin = torch.from_numpy(tj).pin_memory()
        y_pin = torch.empty((N_total, OH, OW, layer.KN) if nhwc else (N_total, layer.KN, OH, OW), dtype=torch.float32).pin_memory()
        shape_job = layer.shape(N_total)
        if world == 1:
            def call():
                ctx.conv_host(w, x_pin.data_ptr(), t_pin.data_ptr(), y_pin.data_ptr(), shape_job, 0.5, LO)
            grp = None
        else:
            grp = ft.MultiContext(list(range(world)))
            gw = grp.upload_weights(type_, wp, layer.C, layer.KH, layer.KW)

            def call():
                grp.conv_host(gw, x_pin.data_ptr(), t_pin.data_ptr(), y_pin.data_ptr(), shape_job, 0.5, LO)
        for _ in range(3):
            call()
        e2e_steps = max(3, min(args.steps, 10))
        if sampler:
            sampler.start()
        l0 = ft.api.launch_count()
        t0 = time.perf_counter()
        for _ in range(e2e_steps):
            call()
        e2e_ms = (time.perf_counter() - t0) * 1e3 / e2e_steps
        e2e_launches = (ft.api.launch_count() - l0) // e2e_steps
        if sampler:
            sampler.stop()
        e2e_ok = bool(torch.equal(y_pin[:1], y0_dev))
        in_each = [(batch_slice(N_total, g, world)[1] - batch_slice(N_total, g, world)[0]) * layer.C * layer.H * layer.W * 4 for g in range(world)]
        out_each = [(batch_slice(N_total, g, world)[1] - batch_slice(N_total, g, world)[0]) * layer.KN * OH * OW * 4 for g in range(world)]
        floor_ms = pcie_floor(torch, list(range(world)), in_each, out_each)
        e2e = {"value": layer.ops(N_total) / (e2e_ms * 1e-3) / 1e9, "unit": "GOPS", "ms_per_step": e2e_ms, "steps": e2e_steps,
               "h2d_bytes_per_step": int(xj.nbytes + tj.nbytes), "d2h_bytes_per_step": int(y_pin.numel() * 4),
               "call": "tnns_cuda_conv_host" if world == 1 else f"tnns_cuda_multi_conv_host over {world} devices (one host thread per device)",
               "kernel_launches_per_step": int(e2e_launches), "matches_device_path": e2e_ok,
               "copy_floor_ms": floor_ms, "frac_of_copy_floor": floor_ms / e2e_ms,
               "copy_floor": "plain page-locked cudaMemcpyAsync of every device's share, upload and download at once on all devices of the run"}
        if grp:
            gw.free()
            grp.close()
        D.host_signal("e2e_done")
    else:
        D.host_wait("e2e_done")
    D.barrier()

    if rank == 0:
        pk = peaks()
        ops = layer.ops(N_total)
        ops_loc = layer.ops(nloc)
        in_bytes, out_bytes, pack_bytes = info["in_bytes"], info["out_bytes"], info["pack_bytes"]
        fused, im2col, implicit, slab = info["fused"], info["im2col"], info["implicit"], info["slab"]
        pack_alg_bytes = in_bytes + (ft.api.bordered_image_bytes(nloc, layer.C, layer.H, layer.W, layer.P, layer.P) if slab else
                                     ft.api.e2m1_image_bytes(nloc, layer.C, layer.H, layer.W) if im2col else pack_bytes)
        t_pack_eff = t_pack_alone if fused else t_pack
        gemm_tops = ops_loc / (t_gemm * 1e-3) / 1e12
        per_img = ncu_traffic(name, info["key"])
        gemm_traffic = per_img * nloc if per_img else None
        pack_key = "quantise_e2m1_bordered" if slab else "quantise_e2m1" if im2col else "quantise" if implicit else "pack"
        per_img = (ncu_traffic(name, pack_key + "_nhwc") if args.layout == "nhwc" else None) or ncu_traffic(name, pack_key)
        pack_traffic = per_img * nloc if per_img else None
        if args.gemm == "popc":
            # integer-pipe kernel: 5.5 LOP3 per 32-bit lane and output, LOP3 issues 64 lanes/clk/SM
            gemm_kernel_name, gemm_bound = "gemm_popc_tiled_kernel (LOP3 carry-save popcount GEMM + PReLU)", "int"
            gemm_peak = ctx_lop3_rate * 1e9 * 64.0 / 5.5 / 1e12
            gemm_peak_source = "measured LOP3 issue rate x 64 ops per lane / 5.5 LOP3 per lane"
        elif args.gemm == "i8tc":
            gemm_kernel_name, gemm_bound = "gemm_tc_kernel<F4=false> (tcgen05.mma kind::i8 GEMM + PReLU)", "tensor"
            gemm_peak = 2.0 * pk["bf16_tflops"]
            gemm_peak_source = f"2 x {pk['source']} bf16 burst figure (int8 dense rate = 2 x bf16)"
        else:
            gemm_kernel_name, gemm_bound = ("gemm_slab_kernel<QF=true> (whole layer in one launch: quantiser warps write the bordered 4-bit image, tcgen05.mma kind::mxf4 GEMM fed by one slab of pixels per tile, unit scales, + PReLU)" if slab and fused else
                                            "gemm_slab_kernel (tcgen05.mma kind::mxf4 GEMM fed by one slab of pixels per tile from a bordered 4-bit image, unit scales, + PReLU)" if slab else
                                            "gemm_tc_kernel<F4=true, ATMA=true, QF=true> (whole layer in one launch: quantiser warps write the 4-bit image, tcgen05.mma kind::mxf4 GEMM fed by im2col tensor copies, unit scales, + PReLU)" if fused else
                                            "gemm_tc_kernel<F4=true, ATMA=true> (tcgen05.mma kind::mxf4 GEMM fed by im2col tensor copies, unit scales, + PReLU)" if im2col else
                                            "gemm_tc_kernel<F4=true> (tcgen05.mma kind::mxf4 GEMM, unit scales, + PReLU)"), "tensor"
            gemm_peak = 4.0 * pk["bf16_tflops"]
            gemm_peak_source = f"4 x {pk['source']} bf16 burst figure (4-bit dense rate = 4 x bf16)"
        line = {
            "metric": METRIC, "value": ops / (ms_step * 1e-3) / 1e9, "unit": "GOPS", "n_gpus": world, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": ms_step, "higher_is_better": True, "scaling": args.scaling, "vs_baseline": None,
            "dtype": (("e2m1 (4-bit) operands quantised from fp32, unit block scales, fp32 accumulate (exact), fp32 PReLU" if im2col else
                       "e2m1 operands expanded from 2-bit planes, unit block scales, fp32 accumulate (exact), fp32 PReLU") if args.gemm in ("auto", "f4tc") else "int8 operands expanded from 2-bit planes, int32 accumulate, fp32 PReLU") if args.gemm != "popc" else "u32 bit-plane lanes, int32 popcount accumulate, fp32 PReLU",
            "data": "synthetic",
            "config": common_config(name, "layer", type_, N_total, [layer], args.scaling, args.layout),
            "impl_config": {"batch_per_gpu": nloc, "gemm": args.gemm, "route": info["route"],
                            "l2": f"ring of {info['ring']} distinct input/workspace/output buffer sets ({info['ring'] * info['step_bytes'] >> 20} MiB) cycled "
                                  f"between steps; one set alone is {info['step_bytes'] >> 20} MiB",
                            "check": "skipped" if args.no_check else "every rank compared the first and the last image of its slice with the CPU checker before timing"},
            "gpu_launches": int(launches * world),
            "kernels_ms": ({"quantise+gemm (one launch)": t_gemm, "same, with event records around every launch": t_gemm_instrumented} if fused
                           else {("quantise" if implicit else "pack"): t_pack, "gemm": t_gemm,
                                 "note": "from a second, instrumented pass (event records between the launches); ms_per_step is the uninstrumented pass"}),
            # dominant kernel: the GEMM.  Its roof is the tensor pipe; the 4-bit (int8) rate of this part
            # is four times (twice) its bf16 rate, and bf16 is what MEASURED_PEAKS.json holds (cuBLAS, burst
            # figure for a kernel timed alone)
            "roofline": {
                "kernel": gemm_kernel_name, "bound": gemm_bound, "achieved": gemm_tops, "peak": gemm_peak, "unit": "TFLOP/s",
                "frac": gemm_tops / gemm_peak, "traffic": gemm_traffic, "peak_source": gemm_peak_source,
                "algorithmic_ops_per_launch": ops_loc, "ms_per_launch": t_gemm,
                # second denominator, measured live: the rate of a bare tcgen05.mma loop of the same
                # kind and tile shape (operands resident in shared memory, no loads, no epilogue)
                "pipe_peak": ctx_mma_rate / 1e3 if ctx_mma_rate else None,
                "frac_of_pipe_peak": gemm_tops / (ctx_mma_rate / 1e3) if ctx_mma_rate else None,
                # the fused launch also streams the fp32 input and output through HBM
                "hbm_algorithmic_bytes_per_launch": (in_bytes + out_bytes) if fused else None,
                "hbm_frac": ((in_bytes + out_bytes) / (t_gemm * 1e-3) / 1e9 / pk["hbm_gbs"]) if fused else None},
            "roofline_pack": {
                "kernel": ("quantise_tma_kernel<e2m1> (tensor-copy fed quantise to a bordered 4-bit operand image)" if slab else
                           "quantise_tma_kernel<e2m1> (tensor-copy fed quantise to a 4-bit operand image)" if im2col else
                           "pack_staged_kernel<IMG_OUT> (quantise + bit-pack to a packed image)" if implicit else "pack_staged_kernel (quantise + bit-pack + im2row)"), "bound": "hbm",
                "achieved": pack_alg_bytes / (t_pack_eff * 1e-3) / 1e9 if t_pack_eff else None, "peak": pk["hbm_gbs"], "unit": "GB/s",
                "frac": pack_alg_bytes / (t_pack_eff * 1e-3) / 1e9 / pk["hbm_gbs"] if t_pack_eff else None, "traffic": pack_traffic, "peak_source": pk["source"],
                "algorithmic_bytes_per_launch": pack_alg_bytes, "ms_per_launch": t_pack_eff,
                "note": ("not launched in the timed step (the quantise step runs inside the GEMM launch there); timed back to back by itself"
                         if fused else None),
                # the same kernel launched back to back without the GEMM in between
                "ms_per_launch_alone": t_pack_alone,
                "frac_alone": (pack_alg_bytes / (t_pack_alone * 1e-3) / 1e9 / pk["hbm_gbs"]) if t_pack_alone else None},
            "sustained": sustained,
            "e2e": e2e,
            "clocks": sampler.summary() if sampler else None,
        }
        if sustained:
            line["sustained"]["value_median"] = ops / (sustained["ms_per_step_median"] * 1e-3) / 1e9
            line["sustained"]["frac_of_sustained_peak"] = (ops_loc / (sustained["ms_per_step_median"] * 1e-3) / 1e12) / (4.0 * pk["bf16_tflops_sustained"]) if args.gemm in ("auto", "f4tc") else None
        if other:
            line["weak_scaling" if strong else "fixed_total_batch"] = other
        if other_layout:
            line["other_layout"] = other_layout
        if world == 1 and not args.no_cpu:
            line["cpu_baseline"] = cpu_baseline("layer", type_, N_total, [layer], passes=args.cpu_passes)
        print(json.dumps(line), flush=True)
    w.free()
    ctx.close()
    D.close()


def run_stack(args, name, type_, N_cfg, layers):
    """A chain of layers on the device (ConvStack): 4-bit images between layers by default, one kernel
    per layer.  Multi-GPU: the batch is split over the ranks, every rank runs the whole chain."""
    D = Dist(args)
    torch = D.torch
    import fastertnn_b200 as ft
    from fastertnn_b200.stack import ConvStack
    rank, world, local = D.rank, D.world, D.local
    strong = args.scaling == "strong"
    N_total = N_cfg if strong else N_cfg * world
    n0, n1 = batch_slice(N_total, rank, world)
    nloc = n1 - n0
    if nloc <= 0:
        raise SystemExit("bench: fewer images than ranks")
    L0, Ll = layers[0], layers[-1]
    per = L0.C * L0.H * L0.W
    x_h = synth.uniform_pm1(SEED_X + 0x10, (nloc, L0.C, L0.H, L0.W), offset=n0 * per)
    thr_val = 0.25 if act_ternary(type_) else 0.0
    pws = []
    for i, L in enumerate(layers):
        w_f, w_thr = layer_weights(type_, L, SEED_W + 0x10 + i)
        pws.append((ft.pack_weights_ternary if wgt_ternary(type_) else ft.pack_weights_binary)(w_f, w_thr))
    ctx = ft.Context(local)
    chain = args.chain if act_ternary(type_) else ("packed" if args.chain == "image" else args.chain)
    st = ConvStack(ctx, type_, layers, pws, nloc, thr_val, chain=chain, reinterpret_links=True)
    stream = torch.cuda.Stream()
    sp = stream.cuda_stream
    x_pin = torch.from_numpy(x_h).pin_memory()
    out_shape = (nloc, Ll.KN, Ll.OH, Ll.OW)
    y_pin = torch.empty(out_shape, dtype=torch.float32).pin_memory()
    in_bytes, out_bytes = x_h.nbytes, int(np.prod(out_shape)) * 4
    ctx.lib.tnns_cuda_memcpy_h2d(ctx.handle, st.input_ptr(), x_h.ctypes.data, x_h.nbytes)

    # correctness gate: the first image of the rank's slice, chained on the host (not timed)
    if not args.no_check:
        from oracle import binding
        chk = binding.best()
        st.run(sp)
        ctx.sync()
        got = ctx.to_host(st.output_ptr(), out_shape, np.float32)
        if nloc * Ll.KN * Ll.OH * Ll.OW == 0:
            ok = True
        else:
            # a reinterpreted link mixes images, so the check chains the whole (small) batch where the model has one
            nchk = nloc if not all(st.link_ok) else 1
            want = cpu_chain(chk, type_, x_h[:nchk], np.full(nchk, thr_val, np.float32), pws, layers, os.cpu_count() or 1)
            ok = got[:nchk].tobytes() == want.tobytes()
        if not D.all_true(ok):
            raise SystemExit("bench: GPU output of the chain differs from the CPU checker on some rank; refusing to time it")
        ctx.lib.tnns_cuda_memcpy_h2d(ctx.handle, st.input_ptr(), x_h.ctypes.data, x_h.nbytes)

    sampler = ClockSampler(str(torch.cuda.get_device_properties(local).uuid)) if rank == 0 else None

    def step(i):
        st.run(sp)

    for i in range(args.warmup):
        step(i)
    launches0 = ft.api.launch_count()
    if sampler:
        sampler.start()
    ms_step = timed_region(D, stream, step, args.steps) / args.steps
    launches = ft.api.launch_count() - launches0
    sustained = None if args.no_sustained else sustained_regions(D, stream, step, args.steps, ms_step, sampler, args.sustain_seconds)
    if sampler:
        sampler.stop()

    # per-layer times: every layer alone, on its own buffers, back to back (a chain run gives no
    # place to put events: the stack enqueues all of its kernels in one call)
    per_layer = []
    if rank == 0:
        for i, (L, pw) in enumerate(zip(layers, pws)):
            one = ConvStack(ctx, type_, [L], [pw], nloc, thr_val, chain="fp32")
            for _ in range(2):
                one.run(sp)
            a0, a1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            reps = max(3, args.steps // 2)
            a0.record(stream)
            for _ in range(reps):
                one.run(sp)
            a1.record(stream)
            stream.synchronize()
            ms = a0.elapsed_time(a1) / reps
            per_layer.append({"layer": str(L), "ms": ms, "giga_ops": L.ops(nloc) / 1e9, "tops": L.ops(nloc) / (ms * 1e-3) / 1e12,
                              "hbm_bytes": nloc * (L.C * L.H * L.W + L.KN * L.OH * L.OW) * 4})
            one.close()
    ctx.sync()

    # ---- end to end: host input in, chain, host output out ----------------------------------------
    D.barrier()
    e2e_steps = max(3, min(args.steps, 10))

    def e2e_step():
        ctx.lib.tnns_cuda_memcpy_h2d(ctx.handle, st.input_ptr(), x_pin.data_ptr(), in_bytes)
        st.run(sp)
        stream.synchronize()
        ctx.lib.tnns_cuda_memcpy_d2h(ctx.handle, y_pin.data_ptr(), st.output_ptr(), out_bytes)

    e2e_step()
    D.barrier()
    t0 = time.perf_counter()
    for _ in range(e2e_steps):
        e2e_step()
    e2e_ms = D.max_over_ranks((time.perf_counter() - t0) * 1e3) / e2e_steps
    D.barrier()

    if rank == 0:
        pk = peaks()
        ops = sum(L.ops(N_total) for L in layers)
        slow = max(per_layer, key=lambda d: d["ms"])
        peak = 4.0 * pk["bf16_tflops"]
        line = {
            "metric": METRIC, "value": ops / (ms_step * 1e-3) / 1e9, "unit": "GOPS", "n_gpus": world, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": ms_step, "higher_is_better": True, "scaling": args.scaling, "vs_baseline": None,
            "dtype": "e2m1 (4-bit) operands, unit block scales, fp32 accumulate (exact), fp32 PReLU; 4-bit images between layers",
            "data": "synthetic",
            "config": common_config(name, "stack", type_, N_total, layers, args.scaling),
            "impl_config": {"batch_per_gpu": nloc, "chain": chain,
                            "routes": ([m + (" (one launch with its quantise step)" if f else "") for m, f in zip(st.mode, st.fuse)] if chain == "image" else None),
                            "l2": "the chain's activations (hundreds of MB at this batch) pass through the same ping-pong buffers every step; "
                                  "each layer's input was written by its predecessor, as in any chained run",
                            "check": "skipped" if args.no_check else "every rank compared its chain output with the CPU checker chained on the host before timing"},
            "gpu_launches": int(launches * world),
            "kernels_ms": {f"L{i}": d["ms"] for i, d in enumerate(per_layer)},
            "layers": per_layer,
            "roofline": {"kernel": f"slowest layer alone, fp32 in and out (tnns_cuda_conv): {slow['layer']}", "bound": "tensor",
                         "achieved": slow["tops"], "peak": peak, "unit": "TFLOP/s", "frac": slow["tops"] / peak, "traffic": None,
                         "peak_source": f"4 x {pk['source']} bf16 burst figure", "ms_per_launch": slow["ms"],
                         "hbm_algorithmic_bytes_per_launch": slow["hbm_bytes"],
                         "hbm_frac": slow["hbm_bytes"] / (slow["ms"] * 1e-3) / 1e9 / pk["hbm_gbs"],
                         "whole_chain_frac": (ops / world / (ms_step * 1e-3) / 1e12) / peak},
            "sustained": sustained,
            "e2e": {"value": ops / (e2e_ms * 1e-3) / 1e9, "unit": "GOPS", "ms_per_step": e2e_ms, "steps": e2e_steps,
                    "h2d_bytes_per_step": int(in_bytes * world), "d2h_bytes_per_step": int(out_bytes * world),
                    "call": "host input -> device, ConvStack.run, final output -> host; one process per GPU"},
            "clocks": sampler.summary() if sampler else None,
        }
        if sustained:
            line["sustained"]["value_median"] = ops / (sustained["ms_per_step_median"] * 1e-3) / 1e9
        if world == 1 and not args.no_cpu:
            line["cpu_baseline"] = cpu_baseline("stack", type_, N_total, layers, passes=max(2, args.cpu_passes // 2))
        print(json.dumps(line), flush=True)
    st.close()
    ctx.close()
    D.close()


def main():
    # stdout carries exactly one JSON line: whatever libraries print there on the way (NCCL's version
    # banner, for one) goes to stderr instead, and print() writes to the saved descriptor
    sys.stdout.flush()
    saved = os.dup(1)
    os.dup2(2, 1)
    sys.stdout = os.fdopen(saved, "w", buffering=1)
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", choices=["ours", "reference"], default="ours")
    ap.add_argument("--workload", choices=sorted(WORKLOADS), default="tnn_conv_large")
    ap.add_argument("--gemm", choices=["auto", "popc", "i8tc", "f4tc"], default="auto")
    ap.add_argument("--route", choices=["auto", "slab", "slab_fused", "fused", "im2col", "implicit", "explicit"], default="auto",
                    help="auto: the library's default layer route (fused where the layer qualifies and is large enough, "
                         "else im2col where it qualifies, else implicit); "
                         "slab / slab_fused: stride-1 layers from a bordered 4-bit image, one slab of pixels per tile for all taps (two launches / one); "
                         "fused: quantise + GEMM fed by im2col tensor copies in ONE launch; "
                         "im2col: quantise to a 4-bit image + GEMM fed by im2col tensor copies; "
                         "implicit: quantise to bit planes + GEMM whose warps gather and expand their im2row rows; "
                         "explicit: pack to the im2row matrix, then GEMM")
    ap.add_argument("--layout", choices=["nchw", "nhwc"], default="nchw", help="layer workloads: memory layout of the fp32 input and output")
    ap.add_argument("--chain", choices=["image", "packed", "fp32"], default="image", help="stack workloads: what travels between two layers")
    ap.add_argument("--scaling", choices=["weak", "strong"], default="strong",
                    help="strong: the configured batch is split over the ranks; weak: every rank processes the configured batch")
    ap.add_argument("--no-check", action="store_true", help="skip the pre-timing comparison with the CPU checker")
    ap.add_argument("--no-cpu", action="store_true", help="skip the CPU baseline leg")
    ap.add_argument("--no-sustained", action="store_true", help="skip the one-second sustained measurement")
    ap.add_argument("--sustain-seconds", type=float, default=1.0)
    ap.add_argument("--cpu-passes", type=int, default=5)
    args = ap.parse_args()
    if args.warmup < 3 and args.impl == "ours":
        args.warmup = 3
    kind, type_, batch, what = WORKLOADS[args.workload]
    layers = [what] if kind == "layer" else list(what)
    if kind == "layer" and batch < args.gpus and args.scaling == "strong":
        args.scaling = "weak"  # a batch-1 layer cannot be split by image
    if args.impl == "reference":
        run_reference(args, args.workload, kind, type_, batch, layers)
    elif kind == "layer":
        run_layer(args, args.workload, type_, batch, layers[0])
    else:
        run_stack(args, args.workload, type_, batch, layers)


if __name__ == "__main__":
    main()
