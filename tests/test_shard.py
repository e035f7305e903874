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
