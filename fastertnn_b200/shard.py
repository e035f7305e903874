"""Row sharding across GPUs.

Rows of the im2row matrix are independent and an image's rows depend only on that image,
so a layer is partitioned by batch index: shard r of `world` owns a contiguous slice of
images (contiguous in both NCHW and NHWC input and output).  Packed weights are
replicated; the data path needs no collective.  The partition itself is the library's
(``tnns_shard_range``), so one-process-per-GPU callers and the in-library device group
(``tnns_cuda_multi_conv_host``) cut a batch at the same places.
"""
from __future__ import annotations

from .api import shard_range


def batch_slice(N: int, rank: int, world: int) -> tuple[int, int]:
    """[n0, n1) of the images rank `rank` owns; the first N % world ranks get one extra."""
    if world <= 0 or not (0 <= rank < world) or N < 0:
        raise ValueError(f"bad shard request N={N} rank={rank} world={world}")
    return shard_range(N, rank, world)


def all_slices(N: int, world: int) -> list[tuple[int, int]]:
    return [batch_slice(N, r, world) for r in range(world)]
