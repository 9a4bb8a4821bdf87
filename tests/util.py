"""Shared helpers of the GPU parity tests: identical seeded inputs for the oracle and the CUDA library."""
import numpy as np

from vq_b200.seeding import LbgSeeder

METRICS = {"SquaredEuclidean": 0, "Euclidean": 1, "CosineDistance": 2, "Manhattan": 3, "Chebyshev": 4, "Hamming": 6}


class RecordingSeeder:
    """LbgSeeder that also records every draw, so the oracle's and the library's draw sequences can be compared."""

    def __init__(self, seed):
        self.seed = seed
        self._pq_args = None
        self.reset()

    def reset(self):
        """Fresh RNG streams, re-consuming the initial sample if one was drawn (the reference re-creates
        StdRng(seed + i) at every OPQ outer iteration, src/opq.rs:140)."""
        self.s = LbgSeeder(self.seed)
        self.draws = []
        if getattr(self, "_pq_args", None):
            n, m, k = self._pq_args
            for i in range(m):
                self.s.init_indices(i, n, k)

    def __call__(self, stream, n):
        return self.draw(stream, n)

    def init_pq(self, n, m, k):
        self._pq_args = (n, m, k)
        return np.stack([self.s.init_indices(i, n, k) for i in range(m)])

    def init_stage(self, stage, n, k):
        return self.s.init_indices(stage, n, k)

    def draw(self, stream, n):
        r = self.s.draw(stream, n)
        self.draws.append((stream, r))
        return r


def by_stream(draws):
    """Per-stream draw sequences: the oracle finishes one subspace before the next while the library advances all
    subspaces together, so only the order WITHIN a stream (one reference RNG each) is comparable."""
    out = {}
    for stream, r in draws:
        out.setdefault(stream, []).append(r)
    return out


def near_tie_mismatches(oracle, codebooks, x, codes_a, codes_b, metric, p=0.0):
    """Split code mismatches into near-ties (relative gap of the two distances below 1e-6) and real ones."""
    bad = np.argwhere(codes_a != codes_b)
    m, k, sd = codebooks.shape
    near = real = 0
    for i, s in bad:
        sub = x[i, s * sd:(s + 1) * sd]
        da = oracle.distance(metric, sub, codebooks[s, codes_a[i, s]], p)
        db = oracle.distance(metric, sub, codebooks[s, codes_b[i, s]], p)
        gap = abs(da - db) / max(abs(da), abs(db), 1e-30)
        if gap < 1e-6:
            near += 1
        else:
            real += 1
    return near, real
