"""Row sharding across GPUs.

Rows of the im2row matrix are independent and an image's rows depend only on that image,
so a layer is partitioned by batch index: rank r of `world` owns a contiguous slice of
images (contiguous in both NCHW and NHWC input and output).  Packed weights are
replicated; the data path needs no collective.
"""
from __future__ import annotations


def batch_slice(N: int, rank: int, world: int) -> tuple[int, int]:
    """[n0, n1) of the images rank `rank` owns; the first N % world ranks get one extra."""
    if world <= 0 or not (0 <= rank < world) or N < 0:
        raise ValueError(f"bad shard request N={N} rank={rank} world={world}")
    base, extra = divmod(N, world)
    n0 = rank * base + min(rank, extra)
    return n0, n0 + base + (1 if rank < extra else 0)


def all_slices(N: int, world: int) -> list[tuple[int, int]]:
    return [batch_slice(N, r, world) for r in range(world)]
