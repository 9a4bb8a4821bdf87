"""The split-TF32 tensor-core kernel of the product quantizer: accuracy of the raw scores against f64 (the margin of the
decision is built on it), codes identical to the oracle's, and the share of pairs left to the exact scan."""
import ctypes as C

import numpy as np
import pytest

import vq_b200 as vq
from tests.golden import reference_known_answers as ka
from vq_b200 import _lib, synth

pytestmark = pytest.mark.gpu


def _scores(ctx, x, cb, want_scores=True):
    n = x.shape[0]
    m, k, _ = cb.shape
    scores = np.zeros((n, m, 256), np.float32) if want_scores else None
    codes = np.zeros((n, m), np.uint32)
    marked = C.c_ulonglong(0)
    rc = _lib.load().vqb_pq_tensor_scores(ctx.handle, x.ctypes.data, n, m, cb.ctypes.data, k,
                                          scores.ctypes.data if want_scores else None, codes.ctypes.data, C.byref(marked))
    assert rc == 0, _lib.load().vqb_last_error(ctx.handle).decode()
    return scores, codes, int(marked.value)


def _exact_scores(x, cb):
    n = x.shape[0]
    m, k, sd = cb.shape
    xs = x.astype(np.float64).reshape(n, m, sd)
    c = cb.astype(np.float64)
    hn = 0.5 * (c * c).sum(-1)                      # m x k
    return hn[None] - np.einsum("nmd,mkd->nmk", xs, c), 0.5 * (xs * xs).sum(-1), hn


@pytest.mark.parametrize("n,m,k,scale", [(1000, 16, 256, 1.0), (777, 4, 100, 1.0), (4097, 8, 256, 37.0), (300, 12, 17, 1e-3),
                                          (50000, 16, 256, 1.0)])
def test_split_tf32_scores_are_within_a_quarter_of_the_assumed_error(ctx, oracle, n, m, k, scale):
    rng = np.random.default_rng(n + m)
    x = (rng.normal(size=(n, m * 8)) * scale).astype(np.float32)
    cb = (rng.normal(size=(m, k, 8)) * scale).astype(np.float32)
    scores, codes, marked = _scores(ctx, x, cb)
    exact, xh2, hn = _exact_scores(x, cb)
    bound = 2.4e-6 * (xh2[:, :, None] + 2.0 * hn.max(-1)[None, :, None])   # E of the kernel's margin
    err = np.abs(scores[:, :, :k] - exact)
    assert (err <= 0.25 * bound).all(), float((err / bound).max())
    assert (scores[:, :, k:32 * ((k + 31) // 32)] > 1e29).all()             # padding columns can never be chosen
    # the codes are the oracle's, and only a small share of the pairs needed the exact scan
    _, codes_o = oracle.pq_quantize(cb, x, ka.SQ)
    assert np.array_equal(codes, codes_o)
    assert marked <= 0.01 * n * m + 8, marked


def test_ties_duplicates_and_specials_go_to_the_exact_scan(ctx, oracle):
    rng = np.random.default_rng(5)
    m, k = 8, 64
    cb = rng.normal(size=(m, k, 8)).astype(np.float32)
    cb[:, 9] = cb[:, 3]            # duplicate centroids: exact ties, the lower index must win
    cb[2, 5, 1] = np.nan           # a NaN centroid never wins ...
    cb[3, 0, 0] = np.nan           # ... unless it is centroid 0, where the reference's scan starts
    cb[4, 7] = np.inf
    x = rng.normal(size=(2000, m * 8)).astype(np.float32)
    x[:64] = cb[:, 3].reshape(-1)[None]      # rows sitting exactly on the duplicated centroid
    x[100, 5] = np.nan
    x[101, 17] = np.inf
    x[102] = 0.0
    x[103] = 1e-25                 # too small to scale: ranked by the exact scan
    x[104] = 3e18                  # squares overflow
    x[105, :8] = 0.0
    x[105, 0] = 1.3e19             # scores stay finite but the true distance to centroid 20 overflows f32
    cb[0, 20] = 0.0
    cb[0, 20, 0] = -1.3e19
    _, codes, marked = _scores(ctx, x, cb, want_scores=False)
    _, codes_o = oracle.pq_quantize(cb, x, ka.SQ)
    assert np.array_equal(codes, codes_o)
    assert marked >= 64


def test_marked_share_on_the_benchmark_distribution(ctx):
    x = synth.uniform01(100000, 128, 1)
    cb = synth.uniform01(16 * 256, 8, 2).reshape(16, 256, 8)
    _, _, marked = _scores(ctx, x, cb, want_scores=False)
    assert marked < 0.005 * x.shape[0] * 16, marked


@pytest.mark.parametrize("n", [1, 5, 127, 128, 129, 257])
@pytest.mark.parametrize("m,k", [(4, 2), (8, 3), (64, 256)])
def test_tiny_and_ragged_row_counts(ctx, oracle, n, m, k):
    rng = np.random.default_rng(n * 1000 + m)
    x = rng.normal(size=(n, m * 8)).astype(np.float32)
    cb = rng.normal(size=(m, k, 8)).astype(np.float32)
    _, codes, _ = _scores(ctx, x, cb, want_scores=False)
    _, codes_o = oracle.pq_quantize(cb, x, ka.SQ)
    assert np.array_equal(codes, codes_o)


def test_fit_with_retiring_subspaces_matches_oracle(oracle):
    """Sub-spaces converge at different iterations, so later passes run with some of a group's four sub-spaces inactive."""
    from tests.util import RecordingSeeder, by_stream

    x = synth.gaussian_mixture(3000, 64, 5, components=4, sigma=0.01)   # few tight clusters: quick, uneven convergence
    so, sg = RecordingSeeder(9), RecordingSeeder(9)
    init = so.init_pq(3000, 8, 8)
    sg.init_pq(3000, 8, 8)
    cb_o, iters_o = oracle.pq_fit(x, 8, 8, 25, init, so.draw)
    pq = vq.ProductQuantizer.fit(x, 8, 8, 25, vq.Distance.Euclidean, 9, init_idx=init, draw=sg.draw, accumulate=vq.ACCUM_ORDERED)
    assert np.array_equal(pq.codebooks, cb_o)
    assert np.array_equal(pq.iterations, iters_o)
    assert len(set(int(v) for v in iters_o)) > 1 or int(iters_o[0]) < 25
    assert by_stream(so.draws) == by_stream(sg.draws)
