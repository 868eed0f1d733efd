"""A counter-based generator of approximately normal values: element i of a tensor is a function of
(seed, tensor name, i) alone, made of integer operations and two exactly rounded float32 operations, so
that numpy on the host and the fill kernel on the device (csrc/elementwise.cu, fill_normal_kernel) give
the same bits, in any order and for any part of a tensor.

    h_j = mix64(key + (3 i + j) * GOLDEN), j = 0, 1, 2          (splitmix64's finalizer, 64-bit wrap-around)
    x   = (the sum of the twelve 16-bit fields of h_0, h_1, h_2 - 6 * 65535) / 65536
    value = mean + std * x                                      (float32: one product, one sum)

x is a sum of twelve uniform variables: mean 0, variance 1, no value beyond 6 in size.  The reference has no
generator in its engine (its tests write a seeded fixture, tests/regression/mk_tiny_st.py:21-45).
"""
from __future__ import annotations

import zlib

import numpy as np

GOLDEN = 0x9E3779B97F4A7C15
_M1, _M2 = 0xBF58476D1CE4E5B9, 0x94D049BB133111EB
_MASK = (1 << 64) - 1


def tensor_key(seed: int, name: str) -> int:
    """The 64-bit key of a tensor's values."""
    z = (int(seed) * GOLDEN + zlib.crc32(name.encode()) * _M2 + len(name)) & _MASK
    z = ((z ^ (z >> 30)) * _M1) & _MASK
    z = ((z ^ (z >> 27)) * _M2) & _MASK
    return z ^ (z >> 31)


def _mix64(z: np.ndarray) -> np.ndarray:
    z = (z ^ (z >> np.uint64(30))) * np.uint64(_M1)
    z = (z ^ (z >> np.uint64(27))) * np.uint64(_M2)
    return z ^ (z >> np.uint64(31))


def standard(key: int, n: int, start: int = 0) -> np.ndarray:
    """x of the elements start .. start + n - 1 as float32."""
    with np.errstate(over="ignore"):
        i = np.arange(start, start + n, dtype=np.uint64)
        total = np.zeros(n, dtype=np.int64)
        f = np.uint64(0xFFFF)
        for j in range(3):
            h = _mix64(np.uint64(key) + (i * np.uint64(3) + np.uint64(j)) * np.uint64(GOLDEN))
            total += ((h & f) + ((h >> np.uint64(16)) & f) + ((h >> np.uint64(32)) & f) + (h >> np.uint64(48))).astype(np.int64)
    return (total - 6 * 65535).astype(np.float32) * np.float32(1.0 / 65536.0)


def normal(key: int, n: int, mean: float, std: float, start: int = 0) -> np.ndarray:
    """mean + std * x as float32, rounded after the product and after the sum."""
    return np.float32(mean) + np.float32(std) * standard(key, n, start)
