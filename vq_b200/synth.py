"""Seeded synthetic inputs with the shapes and value distributions of the
reference's evaluation data (src/bin/utils.rs:31-41: i.i.d. uniform [0,1) rows)
and of the benchmark configurations.  The reference generates them with
``StdRng``, which cannot be reproduced here; a counter-based SplitMix64 mixer
stands in.  Values: u = (mix(seed, index) >> 40) * 2^-24, i.e. 24-bit floats in [0,1).
"""
from __future__ import annotations

import numpy as np


def _mix(seed: int, idx: np.ndarray) -> np.ndarray:
    with np.errstate(over="ignore"):
        z = idx.astype(np.uint64) * np.uint64(0x9E3779B97F4A7C15) + np.uint64((seed * 0xD1342543DE82EF95 + 0x2545F4914F6CDD1D) & ((1 << 64) - 1))
        z = (z ^ (z >> np.uint64(30))) * np.uint64(0xBF58476D1CE4E5B9)
        z = (z ^ (z >> np.uint64(27))) * np.uint64(0x94D049BB133111EB)
        return z ^ (z >> np.uint64(31))


def uniform01(n: int, dim: int, seed: int, chunk_rows: int = 1 << 16, out: np.ndarray | None = None,
              row0: int = 0) -> np.ndarray:
    """Rows [row0, row0 + n) of the seeded n_total x dim float32 matrix of i.i.d. uniform [0, 1) values."""
    if out is None:
        out = np.empty((n, dim), dtype=np.float32)
    flat = out.reshape(-1)
    step = chunk_rows * dim
    base = row0 * dim
    for a in range(0, n * dim, step):
        b = min(n * dim, a + step)
        bits = _mix(seed, np.arange(base + a, base + b, dtype=np.uint64)) >> np.uint64(40)
        flat[a:b] = bits.astype(np.float32) * np.float32(2.0 ** -24)
    return out


def uniform(n: int, dim: int, seed: int, lo: float, hi: float) -> np.ndarray:
    """n x dim float32, i.i.d. uniform on [lo, hi)."""
    x = uniform01(n, dim, seed)
    x *= np.float32(hi - lo)
    x += np.float32(lo)
    return x


def normal(n: int, dim: int, seed: int) -> np.ndarray:
    """n x dim float32 standard normal (Box-Muller on two uniform streams)."""
    u1 = uniform01(n, dim, seed * 2 + 1).astype(np.float64)
    u2 = uniform01(n, dim, seed * 2 + 2).astype(np.float64)
    r = np.sqrt(-2.0 * np.log(1.0 - u1))
    return (r * np.cos(2.0 * np.pi * u2)).astype(np.float32)


def gaussian_mixture(n: int, dim: int, seed: int, components: int = 64, sigma: float = 0.05) -> np.ndarray:
    """Rows from a `components`-component isotropic Gaussian mixture, means uniform in [0,1)^dim."""
    means = uniform01(components, dim, seed)
    which = (_mix(seed + 7919, np.arange(n, dtype=np.uint64)) % np.uint64(components)).astype(np.int64)
    return (means[which] + np.float32(sigma) * normal(n, dim, seed + 1)).astype(np.float32)


def correlated(n: int, dim: int, seed: int) -> np.ndarray:
    """x = A z with z ~ N(0, I) and A a fixed dim x dim matrix with N(0, 1/dim) entries."""
    a = normal(dim, dim, seed) / np.float32(np.sqrt(dim))
    z = normal(n, dim, seed + 1)
    return (z @ a.T).astype(np.float32)
