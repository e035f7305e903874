"""CPU suite: the multi-GPU path is a partition of the batch with no collective on the
data path.  Two gloo ranks each process their slice (the oracle stands in for the GPU
here) and the concatenation must equal the unsharded result."""
import os
import sys
from pathlib import Path

import numpy as np
import pytest

from fastertnn_b200.shard import all_slices, batch_slice

ROOT = Path(__file__).resolve().parents[1]


def test_slices_partition_the_batch():
    for N in (0, 1, 5, 8, 64, 257):
        for world in (1, 2, 3, 4, 8):
            sl = all_slices(N, world)
            assert sl[0][0] == 0 and sl[-1][1] == N
            assert all(a[1] == b[0] for a, b in zip(sl, sl[1:]))
            sizes = [b - a for a, b in sl]
            assert max(sizes) - min(sizes) <= 1
    with pytest.raises(ValueError):
        batch_slice(8, 2, 2)


def test_shard_run_completes_the_other_shards_when_one_leaves_early(port_oracle):
    """Host-side failure form: one shard's worker returns early with an error (as a rank that
    lost its device would); the call must still complete every other shard, say which shard is
    missing, and leave the missing slice untouched."""
    import fastertnn_b200 as ft
    from cases import make_case, TNN
    from fastertnn_b200.workloads import Layer

    c = make_case(TNN, Layer(64, 6, 6, 16, 3, 3, 1, 1), 7, 78, "uniform")
    P = port_oracle
    wp = P.pack_weights(True, c.w, c.w_thr)
    full = P.conv(TNN, c.x, c.thr, wp, c.kernel_hw, c.padding, c.stride, c.alpha)
    out = np.full_like(full, np.nan)
    started = []

    def worker(g, G, n0, n1):
        started.append(g)
        if g == 2:
            return 2  # TNNS_ERR_CUDA: this shard leaves before doing any work
        out[n0:n1] = P.conv(TNN, c.x[n0:n1], c.thr[n0:n1], wp, c.kernel_hw, c.padding, c.stride, c.alpha)
        return 0

    rc, st = ft.shard_run(4, c.N, worker)
    assert sorted(started) == [0, 1, 2, 3]
    assert rc == 2 and st == [0, 0, 2, 0]
    detail = ft.load_library().tnns_cuda_error_detail().decode()
    assert "1 of 4 shards failed" in detail and "shards 2;" in detail
    n0, n1 = batch_slice(c.N, 2, 4)
    assert np.isnan(out[n0:n1]).all()
    ok = np.ones(c.N, bool)
    ok[n0:n1] = False
    assert out[ok].tobytes() == full[ok].tobytes()
    # and with every shard healthy the pieces are the whole
    rc, st = ft.shard_run(3, c.N, lambda g, G, a, b: (out.__setitem__(slice(a, b), P.conv(TNN, c.x[a:b], c.thr[a:b], wp, c.kernel_hw, c.padding, c.stride, c.alpha)), 0)[1])
    assert rc == 0 and st == [0, 0, 0]
    assert out.tobytes() == full.tobytes()
    # more shards than images: the surplus shards own nothing and succeed
    assert ft.shard_run(5, 2, lambda g, G, a, b: 0 if b - a in (0, 1) else 1) == (0, [0] * 5)


def _worker(rank, world, port, tmp):
    sys.path.insert(0, str(ROOT))
    sys.path.insert(0, str(ROOT / "tests"))
    import torch
    import torch.distributed as dist
    from cases import make_case, TNN
    from fastertnn_b200.workloads import Layer
    from oracle import binding

    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    c = make_case(TNN, Layer(64, 6, 6, 16, 3, 3, 1, 1), 5, 77, "uniform")
    P = binding.port()
    wp = P.pack_weights(True, c.w, c.w_thr)
    n0, n1 = batch_slice(c.N, rank, world)
    y = P.conv(TNN, c.x[n0:n1], c.thr[n0:n1], wp, c.kernel_hw, c.padding, c.stride, c.alpha)
    np.save(Path(tmp) / f"y{rank}.npy", y)
    # the only cross-rank traffic: the max-over-ranks reduction of the step time
    t = torch.tensor([float(rank + 1)])
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    assert t.item() == world
    dist.barrier()
    if rank == 0:
        full = P.conv(TNN, c.x, c.thr, wp, c.kernel_hw, c.padding, c.stride, c.alpha)
        parts = np.concatenate([np.load(Path(tmp) / f"y{r}.npy") for r in range(world)], axis=0)
        assert parts.tobytes() == full.tobytes()
    dist.destroy_process_group()


def test_two_rank_sharding_reassembles(tmp_path):
    import torch.multiprocessing as mp
    port = 29500 + (os.getpid() % 500)
    mp.spawn(_worker, args=(2, port, str(tmp_path)), nprocs=2, join=True)
