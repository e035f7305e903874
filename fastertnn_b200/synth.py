"""Seeded synthetic inputs.

The reference measures on no dataset: its drivers fill arrays with ``rand()``
(src/utils.c:8-32 of the reference).  Here a counter-based splitmix64 stream is used so
that element i of a tensor depends only on (seed, i): the same values can be produced in
slices, on any rank, in numpy.
"""
from __future__ import annotations

import numpy as np

_GAMMA = np.uint64(0x9E3779B97F4A7C15)
_M1 = np.uint64(0xBF58476D1CE4E5B9)
_M2 = np.uint64(0x94D049BB133111EB)


def splitmix64(seed: int, count: int, offset: int = 0) -> np.ndarray:
    """Elements offset .. offset+count-1 of the stream for `seed` (uint64)."""
    with np.errstate(over="ignore"):
        i = np.arange(offset + 1, offset + count + 1, dtype=np.uint64)
        z = np.uint64(seed & 0xFFFFFFFFFFFFFFFF) + i * _GAMMA
        z = (z ^ (z >> np.uint64(30))) * _M1
        z = (z ^ (z >> np.uint64(27))) * _M2
        return z ^ (z >> np.uint64(31))


def uniform_pm1(seed: int, shape, offset: int = 0) -> np.ndarray:
    """fp32 uniform in [-1, 1): 24 random bits scaled by 2^-23, minus one."""
    n = int(np.prod(shape))
    r = (splitmix64(seed, n, offset) >> np.uint64(40)).astype(np.float32)
    return (r * np.float32(2.0 ** -23) - np.float32(1.0)).reshape(shape)


def ternary_values(seed: int, shape, offset: int = 0) -> np.ndarray:
    """fp32 values i.i.d. uniform in {-1, 0, +1}."""
    n = int(np.prod(shape))
    r = (splitmix64(seed, n, offset) >> np.uint64(33)) % np.uint64(3)
    return (r.astype(np.float32) - np.float32(1.0)).reshape(shape)


def binary_values(seed: int, shape, offset: int = 0) -> np.ndarray:
    """fp32 values i.i.d. uniform in {-1, +1}."""
    n = int(np.prod(shape))
    r = (splitmix64(seed, n, offset) >> np.uint64(33)) & np.uint64(1)
    return (np.float32(2.0) * r.astype(np.float32) - np.float32(1.0)).reshape(shape)
