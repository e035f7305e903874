#!/usr/bin/env python
"""Benchmark of the ternary conv hot path (quantise+pack+im2row -> bitwise GEMM + PReLU).

    python bench.py --gpus N --steps K --warmup W            # this library, one rank per GPU
    python bench.py --impl reference --gpus N --steps K ...   # the reference's CPU code path

Workload: the large single TNN conv layer -- batch 64, 512 channels, 32x32, 512 kernels
3x3, stride 1, pad 1 (M=65536, K=4608, N=512), activations uniform in [-1,1), thresholds
+-0.25, ternary weights, PReLU alpha 0.5.  Rows of the im2row matrix are independent, so the
layer is partitioned by batch index with the weights replicated and no collective on the data
path.  By default every rank processes one full 64-image batch of the seeded stream (rank r
owns images 64r .. 64r+63; the job's batch is 64*N, "scaling": "weak"); --scaling strong keeps
the job at 64 images and gives each rank 64/N of them.  The default run also reports the
fixed-64-image figure as "fixed_total_batch".  One "step" is one pass of the job's batch.
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
from fastertnn_b200.workloads import CONV_LARGE, CONV_56, FC_GEMM, Layer  # noqa: E402

METRIC = "ternary conv GOPS (2*M*N*K/s)"
# dram__bytes_read.sum + dram__bytes_write.sum per launch from the ncu captures summarised under
# profiles/ (large layer, 64 images per launch), kept per image so that a rank's share scales.
NCU_TRAFFIC_PER_IMAGE = {
    ("tnn_conv_large", "f4_fused"): 226.1e6 / 64,  # quantise + GEMM in one launch: fp32 input read once, output partly still in L2
    ("tnn_conv_large", "f4_im2col"): 91.5e6 / 64,  # im2col tensor copies from the 16.8 MB 4-bit image (block pairs)
    ("tnn_conv_large", "quantise_e2m1"): 143.1e6 / 64,
    ("tnn_conv_large", "f4"): 85.2e6 / 64,        # implicit im2row: reads the 8.4 MB image, not the im2row matrix
    ("tnn_conv_large", "f4_explicit"): 150.9e6 / 64,
    ("tnn_conv_large", "quantise"): 138.7e6 / 64,
    ("tnn_conv_large", "tc"): 153.8e6 / 64,
    ("tnn_conv_large", "popc"): 419.3e6 / 64,
    ("tnn_conv_large", "pack"): 155.8e6 / 64,
}
L2_BYTES = 126 * 1024 * 1024
SEED_X, SEED_W = 0xC0FFEE40, 0xC0FFEE41
WORKLOADS = {
    "tnn_conv_large": CONV_LARGE,   # batch 64, 512x32x32 -> 512, 3x3 s1 p1
    "tnn_conv_56": CONV_56,         # batch 1, 256x56x56 -> 256
    "tnn_fc": FC_GEMM,              # 1024 x 4096 -> 1024
}


def peaks():
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        d = json.loads(p.read_text())
        return {"hbm_gbs": d["hbm_gbs"], "bf16_tflops": d["bf16_tflops"], "bf16_tflops_sustained": d["bf16_tflops_sustained"],
                "source": "measured"}
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0, "source": "fallback"}


def make_inputs(N_total: int, layer: Layer, n0: int, n1: int):
    """Images n0..n1 of the seeded batch, the thresholds and the packed ternary weights."""
    per = layer.C * layer.H * layer.W
    x = synth.uniform_pm1(SEED_X, (n1 - n0, layer.C, layer.H, layer.W), offset=n0 * per)
    thr = np.full(n1 - n0, 0.25, np.float32)
    w = synth.ternary_values(SEED_W, (layer.KN, layer.C, layer.KH, layer.KW))
    return x, thr, w


# ------------------------------------------------------------------------------------------------
# clocks sampled during the timed regions
# ------------------------------------------------------------------------------------------------
class ClockSampler:
    REASONS = {0x8: "hw_slowdown", 0x40: "hw_thermal_slowdown", 0x20: "sw_thermal_slowdown", 0x4: "sw_power_cap",
               0x80: "hw_power_brake_slowdown"}

    def __init__(self, uuid: str | None):
        self.samples, self.reasons, self.max_mhz = [], set(), None
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
            self._stop.wait(0.02)

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

    def summary(self):
        if not self.samples:
            return {"sm_mhz": None, "sm_max_mhz": self.max_mhz, "reasons": sorted(self.reasons), "samples": 0}
        return {"sm_mhz": statistics.median(self.samples), "sm_max_mhz": self.max_mhz, "reasons": sorted(self.reasons),
                "samples": len(self.samples)}


# ------------------------------------------------------------------------------------------------
# CPU reference (the reference's own AVX2 objects when built, else the restatement)
# ------------------------------------------------------------------------------------------------
def cpu_layer_pass(chk, x, thr, wp, layer: Layer, threads: int):
    """One pass over the batch, images spread over `threads` host threads (the reference code
    is single-threaded and re-entrant; ctypes releases the GIL during the call)."""
    from concurrent.futures import ThreadPoolExecutor
    N = x.shape[0]
    bounds = [batch_slice(N, r, min(threads, N)) for r in range(min(threads, N))]

    def run(b):
        a, e = b
        return chk.conv(0, x[a:e], thr[a:e], wp, (layer.KH, layer.KW), (layer.P, layer.P), (layer.S, layer.S), 0.5)

    t0 = time.perf_counter()
    with ThreadPoolExecutor(len(bounds)) as ex:
        outs = list(ex.map(run, bounds))
    return time.perf_counter() - t0, outs


def cpu_baseline(layer: Layer, N_total: int, passes: int):
    from oracle import binding
    chk = binding.best()
    threads = os.cpu_count() or 1
    x, thr, w = make_inputs(N_total, layer, 0, N_total)
    wp = chk.pack_weights(True, w, np.full(layer.KN, 0.5, np.float32))
    cpu_layer_pass(chk, x[:threads], thr[:threads], wp, layer, threads)  # warm-up
    times = [cpu_layer_pass(chk, x, thr, wp, layer, threads)[0] for _ in range(passes)]
    t = statistics.mean(times)
    return {"value": layer.ops(N_total) / t / 1e9, "unit": "GOPS", "cores": min(threads, N_total), "kind": chk.kind,
            "sample": f"{passes} passes over the full {N_total}-image batch, images split over {min(threads, N_total)} host threads, "
                      f"mean {t * 1e3:.1f} ms per pass"}


def run_reference(args, layer: Layer, N_total: int, name: str):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return  # the reference is a CPU code path: rank 0 alone runs it
    from oracle import binding
    chk = binding.best()
    threads = os.cpu_count() or 1
    x, thr, w = make_inputs(N_total, layer, 0, N_total)
    wp = chk.pack_weights(True, w, np.full(layer.KN, 0.5, np.float32))
    for _ in range(args.warmup):
        cpu_layer_pass(chk, x, thr, wp, layer, threads)
    t0 = time.perf_counter()
    for _ in range(args.steps):
        cpu_layer_pass(chk, x, thr, wp, layer, threads)
    t = (time.perf_counter() - t0) / args.steps
    val = layer.ops(N_total) / t / 1e9
    used = min(threads, N_total)
    line = {
        "impl": "reference", "metric": METRIC, "value": val, "unit": "GOPS", "n_gpus": args.gpus, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": t * 1e3, "higher_is_better": True, "scaling": args.scaling, "vs_baseline": None,
        "dtype": "int (64-bit popcount lanes)", "data": "synthetic",
        "config": {"workload": name, "batch": N_total, "layer": str(layer), "layout": "NCHW"},
        "cpu_baseline": {"value": val, "unit": "GOPS", "cores": used, "kind": chk.kind,
                         "sample": f"each step = one pass over the full {N_total}-image batch split over {used} host threads"},
        "e2e": {"value": val, "unit": "GOPS", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    print(json.dumps(line), flush=True)


# ------------------------------------------------------------------------------------------------
# this library
# ------------------------------------------------------------------------------------------------
def run_ours(args, layer: Layer, N_total: int, name: str):
    import torch
    import torch.distributed as dist
    import fastertnn_b200 as ft

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if world != args.gpus:
        raise SystemExit(f"--gpus {args.gpus} but WORLD_SIZE={world}: launch with torch.distributed.run --nproc-per-node {args.gpus}")
    if not torch.cuda.is_available():
        raise SystemExit("no CUDA device: this benchmark has no CPU fallback")
    torch.cuda.set_device(local)
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def max_over_ranks(v: float) -> float:
        if world == 1:
            return v
        t = torch.tensor([v], device="cuda", dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    N_cfg = N_total
    if args.scaling == "weak":
        N_total = N_cfg * world
    n0, n1 = batch_slice(N_total, rank, world)
    nloc = n1 - n0
    x_h, thr_h, w_f = make_inputs(N_total, layer, n0, n1)
    wp = ft.pack_weights_ternary(w_f, np.full(layer.KN, 0.5, np.float32))
    ctx = ft.Context(local)
    w = ctx.upload_weights(ft.TNN, wp, layer.C, layer.KH, layer.KW)
    shape = layer.shape(nloc)
    OH, OW = layer.OH, layer.OW
    in_bytes, out_bytes = x_h.nbytes, nloc * layer.KN * OH * OW * 4
    # default route (what tnns_cuda_conv does): quantise to a packed image, GEMM gathers its im2row
    # rows itself; --route explicit: pack to the im2row matrix (t2r_p2_opt's job), then GEMM
    # "auto" is what tnns_cuda_conv picks: the copy-engine (im2col tensor copy) form where the layer qualifies
    tc4 = args.gemm in ("auto", "f4tc")
    im2col = tc4 and args.route in ("auto", "im2col", "fused") and ctx.im2col_supported(w, shape)
    if args.route in ("im2col", "fused") and not im2col:
        raise SystemExit("bench: this workload does not qualify for the im2col tensor-copy route")
    implicit = tc4 and (im2col or args.route in ("auto", "implicit"))

    def fused_for(n):
        """One launch with the quantise step inside the GEMM kernel: on request, else where the
        library's own rule (tnns_cuda_conv with TNNS_GEMM_AUTO) takes that route.  The pointer only
        stands for the input's alignment here (torch allocations are 512-byte aligned)."""
        if not (im2col and args.route in ("auto", "fused")):
            return False
        if args.route == "fused":
            return ctx.conv_fused_supported(w, layer.shape(n), 4096, ft.NCHW)
        return ctx.conv_fused_preferred(w, layer.shape(n), 4096, ft.NCHW)

    fused = fused_for(nloc)
    pack_bytes = (ft.api.fused_workspace_bytes(nloc, layer.C, layer.H, layer.W) if im2col else
                  ft.api.packed_image_bytes(True, nloc, layer.C, layer.H, layer.W) if implicit else ft.packed_bytes(ft.TNN, shape))

    def run_quantise(xp, pp, n, strm):
        if im2col:
            ctx.quantise_e2m1(xp, thr_d.data_ptr(), pp, n, layer.C, layer.H, layer.W, layout, strm)
        else:
            ctx.quantise(True, xp, thr_d.data_ptr(), pp, n, layer.C, layer.H, layer.W, layout, strm)

    def run_fused(xp, pp, yp, shp, strm):
        ctx.conv_fused(w, xp, thr_d.data_ptr(), yp, pp, pack_bytes, shp, 0.5, 0, strm)

    def run_gemm_image(pp, yp, shp, strm):
        if im2col:
            ctx.gemm_im2col(w, pp, yp, shp, 0.5, layout, strm)
        else:
            ctx.gemm_implicit(w, pp, yp, shp, 0.5, layout, strm)

    # ring of distinct buffer sets so that consecutive steps never find their data in L2
    step_bytes = in_bytes + out_bytes + pack_bytes
    ring = max(2, -(-3 * L2_BYTES // max(step_bytes, 1)))
    x_pin = torch.from_numpy(x_h).pin_memory()
    thr_pin = torch.from_numpy(thr_h).pin_memory()
    xs, ys, ps = [], [], []
    for r in range(ring):
        xd = torch.empty(x_h.shape, dtype=torch.float32, device="cuda")
        xd.copy_(x_pin)
        if r:  # distinct data per ring slot: rotate the images
            xd.copy_(torch.roll(xd, shifts=r, dims=0))
        xs.append(xd)
        ys.append(torch.empty((nloc, layer.KN, OH, OW), dtype=torch.float32, device="cuda"))
        ps.append(torch.empty(pack_bytes // 8 + 32, dtype=torch.int64, device="cuda"))
    thr_d = torch.from_numpy(thr_h).cuda()
    stream = torch.cuda.Stream()
    sp = stream.cuda_stream
    layout = ft.NCHW
    gemm_algo = {"auto": ft.GEMM_AUTO, "popc": ft.GEMM_POPC_TILED, "i8tc": ft.GEMM_I8_TC, "f4tc": ft.GEMM_F4_TC}[args.gemm]

    def aligned(t):
        return (t.data_ptr() + 127) & ~127

    def step(i, ev=None):
        r = i % ring
        if ev:
            ev[0].record(stream)
        if fused:
            pass
        elif implicit:
            run_quantise(xs[r].data_ptr(), ps[r].data_ptr(), nloc, sp)
        else:
            ctx.pack(True, xs[r].data_ptr(), thr_d.data_ptr(), ps[r].data_ptr(), shape, layout, ft.PACK_AUTO, sp)
        if ev:
            ev[1].record(stream)
        if fused:
            run_fused(xs[r].data_ptr(), aligned(ps[r]), ys[r].data_ptr(), shape, sp)
        elif implicit:
            run_gemm_image(ps[r].data_ptr(), ys[r].data_ptr(), shape, sp)
        else:
            ctx.gemm(w, ps[r].data_ptr(), ys[r].data_ptr(), nloc, OH, OW, 0.5, layout, gemm_algo, sp)
        if ev:
            ev[2].record(stream)

    # correctness gate on a slice small enough for the CPU checker (not timed)
    if rank == 0 and not args.no_check:
        from oracle import binding
        chk = binding.best()
        step(0)
        torch.cuda.synchronize()
        want = chk.conv(0, x_h[:1], thr_h[:1], wp, (layer.KH, layer.KW), (layer.P, layer.P), (layer.S, layer.S), 0.5)
        if ys[0][:1].cpu().numpy().tobytes() != want.tobytes():
            raise SystemExit("bench: GPU output differs from the CPU checker; refusing to time a wrong kernel")

    sampler = ClockSampler(str(torch.cuda.get_device_properties(local).uuid)) if rank == 0 else None

    # ---- device-resident timing -----------------------------------------------------------
    for i in range(args.warmup):
        step(i)
    barrier()
    evs = [[torch.cuda.Event(enable_timing=True) for _ in range(3)] for _ in range(args.steps)]
    e_start, e_end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    launches0 = ft.api.launch_count()
    if sampler:
        sampler.start()
    e_start.record(stream)
    for i in range(args.steps):
        step(args.warmup + i)
    e_end.record(stream)
    stream.synchronize()
    barrier()
    launches = ft.api.launch_count() - launches0
    ms_total = max_over_ranks(e_start.elapsed_time(e_end))
    # per-kernel times: the same K steps once more with events between the launches (kept out of the
    # timed region above: three event records per step cost several microseconds of a 90 us step)
    for i in range(args.steps):
        step(args.warmup + i, evs[i])
    stream.synchronize()
    barrier()
    if sampler:
        sampler.stop()

    # the same layer with the job fixed at the configured batch, partitioned over the ranks
    fixed = None
    if args.scaling == "weak" and world > 1:
        f0, f1 = batch_slice(N_cfg, rank, world)
        nfix = f1 - f0
        fshape = layer.shape(nfix)

        def fstep(i):
            r = i % ring
            if fused_for(nfix):
                run_fused(xs[r].data_ptr(), aligned(ps[r]), ys[r].data_ptr(), fshape, sp)
            elif implicit:
                run_quantise(xs[r].data_ptr(), ps[r].data_ptr(), nfix, sp)
                run_gemm_image(ps[r].data_ptr(), ys[r].data_ptr(), fshape, sp)
            else:
                ctx.pack(True, xs[r].data_ptr(), thr_d.data_ptr(), ps[r].data_ptr(), fshape, layout, ft.PACK_AUTO, sp)
                ctx.gemm(w, ps[r].data_ptr(), ys[r].data_ptr(), nfix, OH, OW, 0.5, layout, gemm_algo, sp)

        for i in range(args.warmup):
            fstep(i)
        barrier()
        f_start, f_end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        f_start.record(stream)
        for i in range(args.steps):
            fstep(i)
        f_end.record(stream)
        stream.synchronize()
        barrier()
        f_ms = max_over_ranks(f_start.elapsed_time(f_end)) / args.steps
        fixed = {"batch": N_cfg, "batch_per_gpu": nfix, "ms_per_step": f_ms, "value": layer.ops(N_cfg) / (f_ms * 1e-3) / 1e9,
                 "unit": "GOPS", "scaling": "strong",
                 "note": "per-GPU working set is below L2 size at this split; buffers still rotate through the ring"}
    ms_step = ms_total / args.steps
    t_pack = statistics.mean(e[0].elapsed_time(e[1]) for e in evs)
    t_gemm = statistics.mean(e[1].elapsed_time(e[2]) for e in evs)
    t_gemm_instrumented = t_gemm
    if fused:
        # one launch per step: its average duration over the timed region is the step time itself
        t_gemm = ms_total / args.steps
    # The first kernel of a step also pays for the previous GEMM's output still draining from L2 to
    # HBM.  Timed by itself (same ring of inputs, larger than L2) it shows what the kernel alone reaches.
    t_pack_alone = None
    if implicit and rank == 0:
        for i in range(3):
            run_quantise(xs[i % ring].data_ptr(), ps[i % ring].data_ptr(), nloc, sp)
        stream.synchronize()
        a0, a1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a0.record(stream)
        for i in range(args.steps):
            run_quantise(xs[i % ring].data_ptr(), ps[i % ring].data_ptr(), nloc, sp)
        a1.record(stream)
        stream.synchronize()
        t_pack_alone = a0.elapsed_time(a1) / args.steps
    ctx_lop3_rate = ctx.pipe_rate(0) if args.gemm == "popc" else 0.0
    # issue-bound tcgen05.mma loop (no loads, no epilogue) on this GPU, 1e9 operations per second
    ctx_mma_rate = ctx.pipe_rate(3 if args.gemm == "i8tc" else 4) if args.gemm != "popc" else 0.0
    ctx.sync()

    # ---- end to end: pinned host buffers in, host buffers out, copies inside the timed region ----
    y_pin = torch.empty((nloc, layer.KN, OH, OW), dtype=torch.float32).pin_memory()
    for _ in range(max(1, min(args.warmup, 3))):
        ctx.conv_host(w, x_pin.data_ptr(), thr_pin.data_ptr(), y_pin.data_ptr(), shape, 0.5, layout)
    e2e_steps = max(3, min(args.steps, 10))
    barrier()
    if sampler:
        sampler.start()
    t0 = time.perf_counter()
    for _ in range(e2e_steps):
        ctx.conv_host(w, x_pin.data_ptr(), thr_pin.data_ptr(), y_pin.data_ptr(), shape, 0.5, layout)
    torch.cuda.synchronize()
    e2e_ms = max_over_ranks((time.perf_counter() - t0) * 1e3) / e2e_steps
    barrier()
    if sampler:
        sampler.stop()
    e2e_ok = bool(torch.equal(y_pin[:1], ys[0][:1].cpu())) if ring and args.warmup + args.steps > 0 else True

    if rank == 0:
        pk = peaks()
        ops = layer.ops(N_total)
        ops_loc = layer.ops(nloc)
        pack_alg_bytes = in_bytes + (ft.api.e2m1_image_bytes(nloc, layer.C, layer.H, layer.W) if im2col else pack_bytes)
        t_pack_eff = t_pack_alone if fused else t_pack
        gemm_tops = ops_loc / (t_gemm * 1e-3) / 1e12
        per_img = NCU_TRAFFIC_PER_IMAGE.get((name, {"popc": "popc", "i8tc": "tc"}.get(args.gemm, "f4_fused" if fused else "f4_im2col" if im2col else "f4" if implicit else "f4_explicit")))
        gemm_traffic = per_img * nloc if per_img else None
        per_img = NCU_TRAFFIC_PER_IMAGE.get((name, "quantise_e2m1" if im2col else "quantise" if implicit else "pack"))
        pack_traffic = per_img * nloc if per_img else None
        if args.gemm == "popc":
            # integer-pipe kernel: 5.5 LOP3 per 32-bit lane and output, LOP3 issues 64 lanes/clk/SM
            # (measured with tnns_cuda_pipe_rate: 18.5e12 thread-instructions/s on this part)
            lop3 = ctx_lop3_rate
            gemm_kernel_name, gemm_bound = "gemm_popc_tiled_kernel (LOP3 carry-save popcount GEMM + PReLU)", "int"
            gemm_peak = lop3 * 1e9 * 64.0 / 5.5 / 1e12
            gemm_peak_source = "measured LOP3 issue rate x 64 ops per lane / 5.5 LOP3 per lane"
        elif args.gemm == "i8tc":
            gemm_kernel_name, gemm_bound = "gemm_tc_kernel<F4=false> (tcgen05.mma kind::i8 GEMM + PReLU)", "tensor"
            gemm_peak = 2.0 * pk["bf16_tflops"]
            gemm_peak_source = f"2 x {pk['source']} bf16 burst figure (int8 dense rate = 2 x bf16)"
        else:
            gemm_kernel_name, gemm_bound = ("gemm_tc_kernel<F4=true, ATMA=true, QF=true> (whole layer in one launch: quantiser warps write the 4-bit image, tcgen05.mma kind::mxf4 GEMM fed by im2col tensor copies, unit scales, + PReLU)" if fused else
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
            "config": {"workload": name, "batch": N_total, "batch_per_gpu": nloc, "layer": str(layer), "layout": "NCHW",
                       "M": N_total * OH * OW, "K": layer.C * layer.KH * layer.KW, "N": layer.KN, "gemm": args.gemm,
                       "route": ("one launch: quantise to a 4-bit image inside the GEMM kernel, GEMM fed by im2col tensor copies" if fused else
                                 "quantise to a 4-bit image -> GEMM fed by im2col tensor copies" if im2col else
                                 "quantise to bit planes -> GEMM with implicit im2row" if implicit else "pack (im2row matrix) -> GEMM"),
                       "l2": f"ring of {ring} distinct input/workspace/output buffer sets ({ring * step_bytes >> 20} MiB) cycled "
                             f"between steps; one set alone is {step_bytes >> 20} MiB"},
            "gpu_launches": int(launches * world),
            "kernels_ms": ({"quantise+gemm (one launch)": t_gemm, "same, with event records around every launch": t_gemm_instrumented} if fused
                           else {("quantise" if implicit else "pack"): t_pack, "gemm": t_gemm,
                                 "note": "from a second, instrumented pass (event records between the launches); ms_per_step is the uninstrumented pass"}),
            # dominant kernel: the GEMM.  Its roof is the tensor pipe; the int8 rate of this part is
            # twice its bf16 rate, and bf16 is what MEASURED_PEAKS.json holds (cuBLAS, burst figure
            # for a kernel timed alone), so peak = 2 x measured bf16.
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
                "kernel": ("quantise_tma_kernel<e2m1> (tensor-copy fed quantise to a 4-bit operand image)" if im2col else
                           "pack_staged_kernel<IMG_OUT> (quantise + bit-pack to a packed image)" if implicit else "pack_staged_kernel (quantise + bit-pack + im2row)"), "bound": "hbm",
                "achieved": pack_alg_bytes / (t_pack_eff * 1e-3) / 1e9, "peak": pk["hbm_gbs"], "unit": "GB/s",
                "frac": pack_alg_bytes / (t_pack_eff * 1e-3) / 1e9 / pk["hbm_gbs"], "traffic": pack_traffic, "peak_source": pk["source"],
                "algorithmic_bytes_per_launch": pack_alg_bytes, "ms_per_launch": t_pack_eff,
                "note": ("not launched in the timed step (the quantise step runs inside the GEMM launch there); timed back to back by itself"
                         if fused else None),
                # the same kernel launched back to back without the GEMM in between
                "ms_per_launch_alone": t_pack_alone,
                "frac_alone": (pack_alg_bytes / (t_pack_alone * 1e-3) / 1e9 / pk["hbm_gbs"]) if t_pack_alone else None},
            "e2e": {"value": ops / (e2e_ms * 1e-3) / 1e9, "unit": "GOPS", "ms_per_step": e2e_ms, "steps": e2e_steps,
                    "h2d_bytes_per_step": int((in_bytes + thr_h.nbytes) * world), "d2h_bytes_per_step": int(out_bytes * world),
                    "matches_device_path": e2e_ok},
            "clocks": sampler.summary() if sampler else None,
        }
        if fixed:
            line["fixed_total_batch"] = fixed
        if world == 1 and not args.no_cpu:
            line["cpu_baseline"] = cpu_baseline(layer, N_total, passes=args.cpu_passes)
        print(json.dumps(line), flush=True)
    w.free()
    ctx.close()
    if world > 1:
        dist.destroy_process_group()


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
    ap.add_argument("--route", choices=["auto", "fused", "im2col", "implicit", "explicit"], default="auto",
                    help="auto: the library's default layer route (fused where the layer qualifies and is large enough, "
                         "else im2col where it qualifies, else implicit); "
                         "fused: quantise + GEMM fed by im2col tensor copies in ONE launch; "
                         "im2col: quantise to a 4-bit image + GEMM fed by im2col tensor copies; "
                         "implicit: quantise to bit planes + GEMM whose warps gather and expand their im2row rows; "
                         "explicit: pack to the im2row matrix, then GEMM")
    ap.add_argument("--scaling", choices=["weak", "strong"], default="weak",
                    help="weak: every rank processes the configured batch; strong: the configured batch is split over the ranks")
    ap.add_argument("--no-check", action="store_true", help="skip the pre-timing comparison with the CPU checker")
    ap.add_argument("--no-cpu", action="store_true", help="skip the CPU baseline leg")
    ap.add_argument("--cpu-passes", type=int, default=5)
    args = ap.parse_args()
    if args.warmup < 3 and args.impl == "ours":
        args.warmup = 3
    N_total, layer = WORKLOADS[args.workload]
    if args.impl == "reference":
        run_reference(args, layer, N_total, args.workload)
    else:
        run_ours(args, layer, N_total, args.workload)


if __name__ == "__main__":
    main()
