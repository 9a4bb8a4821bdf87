"""Seeded row sampling for codebook initialisation and empty-cluster re-seeding.

The reference draws with ``rand`` 0.9's ``StdRng::seed_from_u64(seed)``:
``choose_multiple(k)`` once (src/utils.rs:52-54) and ``choose`` per empty
cluster (src/utils.rs:100).  That crate's source is not available to this
project, so the generator below is a documented STAND-IN with the same call
pattern (one stream per LBG call, seeded ``seed + i``); it does not reproduce
``StdRng``'s actual draws.  The native library never draws by itself: it takes
row indices and a draw callback, so a Rust host can supply true ``StdRng``
draws without touching the library.

Stand-in definition (must stay identical in every host language):
  state  <- seed (u64)
  next() : state += 0x9E3779B97F4A7C15; z = state;
           z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9; z = (z ^ (z >> 27)) * 0x94D049BB133111EB;
           return z ^ (z >> 31)                                    (SplitMix64)
  below(n)            = (next() * n) >> 64
  choose_multiple(n,k): partial Fisher-Yates over 0..n-1: for i in 0..k: j = i + below(n - i); swap(a[i], a[j]); emit a[i]
  choose(n)           = below(n)
"""
from __future__ import annotations

import numpy as np

_MASK = (1 << 64) - 1


class StandInRng:
    def __init__(self, seed: int):
        self.state = int(seed) & _MASK

    def next_u64(self) -> int:
        self.state = (self.state + 0x9E3779B97F4A7C15) & _MASK
        z = self.state
        z = ((z ^ (z >> 30)) * 0xBF58476D1CE4E5B9) & _MASK
        z = ((z ^ (z >> 27)) * 0x94D049BB133111EB) & _MASK
        return z ^ (z >> 31)

    def below(self, n: int) -> int:
        return (self.next_u64() * int(n)) >> 64

    def choose_multiple(self, n: int, k: int) -> np.ndarray:
        swapped = {}
        out = np.empty(k, dtype=np.uint64)
        for i in range(k):
            j = i + self.below(n - i)
            vi = swapped.get(i, i)
            vj = swapped.get(j, j)
            swapped[i], swapped[j] = vj, vi
            out[i] = vj
        return out

    def choose(self, n: int) -> int:
        return self.below(n)


class LbgSeeder:
    """One RNG stream per LBG call, seeded ``seed + stream`` like the reference
    (src/pq.rs:119, src/rvq.rs:107, src/opq.rs:140)."""

    def __init__(self, seed: int):
        self.seed = int(seed)
        self.rngs = {}

    def init_indices(self, stream: int, n: int, k: int) -> np.ndarray:
        rng = StandInRng(self.seed + stream)
        self.rngs[stream] = rng
        return rng.choose_multiple(n, k)

    def draw(self, stream: int, n: int) -> int:
        rng = self.rngs.get(stream)
        if rng is None:
            rng = self.rngs[stream] = StandInRng(self.seed + stream)
        return rng.choose(n)
