"""The CUDA library (through the C ABI) against the known answers of the reference's own tests."""
import numpy as np
import pytest

import vq_b200 as vq
from tests.golden import reference_known_answers as ka

pytestmark = pytest.mark.gpu


def _dist(metric, p):
    return vq.Distance(metric, p)


@pytest.mark.parametrize("case", ka.DISTANCE_CASES, ids=[c[0] for c in ka.DISTANCE_CASES])
def test_distance_known_answers(case, oracle):
    _src, metric, p, a, b, expected, tol = case
    got = _dist(metric, p).compute(np.asarray(a, np.float32), np.asarray(b, np.float32))
    assert abs(got - expected) < tol
    if metric != ka.MINKOWSKI:  # powf differs between libm and CUDA in the last place
        assert got == oracle.distance(metric, np.asarray(a, np.float32), np.asarray(b, np.float32), p)


def test_distance_rows_bit_exact_vs_oracle(oracle, ctx):
    rng = np.random.default_rng(3)
    for d in (1, 3, 8, 128, 1034):
        a = rng.uniform(-10, 10, (64, d)).astype(np.float32)
        b = rng.uniform(-10, 10, (64, d)).astype(np.float32)
        b[5] = a[5]
        a[7] = 0
        for metric in (0, 1, 2, 3, 4, 6):
            out = np.empty(64, np.float32)
            from vq_b200 import _lib
            rc = _lib.load().vqb_distance_rows(ctx.handle, metric, 0.0, a.ctypes.data, d, b.ctypes.data, d, 64, out.ctypes.data)
            assert rc == 0
            want = np.array([oracle.distance(metric, a[i], b[i]) for i in range(64)], np.float32)
            assert np.array_equal(out, want), (metric, d)


def test_distance_mismatch_and_minkowski_errors():
    with pytest.raises(vq.DimensionMismatch) as e:
        vq.Distance.Euclidean.compute([1.0, 2.0], [1.0])
    assert str(e.value) == "Dimension mismatch: expected 2, got 1"
    with pytest.raises(vq.InvalidMetricParameter) as e:
        vq.Distance.Minkowski(0.0).compute([1.0], [2.0])
    assert str(e.value) == ka.ERROR_TEXTS["minkowski_p"]


def test_lbg_single_point():
    _src, data, k, iters, expected = ka.LBG_SINGLE_POINT
    cent, _ = vq.lbg_quantize(data, k, iters, 42)
    assert np.array_equal(cent, np.asarray(expected, np.float32))


@pytest.mark.parametrize("case", ka.LBG_PANICS, ids=[c[0] for c in ka.LBG_PANICS])
def test_lbg_panics(case):
    _src, data, k, text = case
    with pytest.raises(vq.InvalidParameter, match=text):
        vq.lbg_quantize(data, k, 10, 42)


@pytest.mark.parametrize("iters", [10, 100])
def test_lbg_basic(iters, oracle):
    cent, _ = vq.lbg_quantize(ka.LBG_BASIC, 2, iters, 42, init_idx=[0, 3])
    want, _, _ = oracle.lbg(ka.LBG_BASIC, 2, iters, [0, 3])
    assert cent.shape == (2, 2) and np.array_equal(cent, want)


def test_lbg_identical_rows_one_iteration(oracle):
    data = np.tile(np.arange(64, dtype=np.float32), (100, 1))
    draws = []

    def draw(stream, n):
        draws.append((stream, n))
        return 7

    cent, iters = vq.lbg_quantize(data, 8, 10, 0, init_idx=np.arange(8), draw=draw)
    assert iters == 1 and len(draws) == 7
    assert np.array_equal(cent, np.tile(data[0], (8, 1)))


def test_bq_doc_and_large(oracle):
    _src, thr, low, high, x, expected = ka.BQ_DOC
    assert vq.BinaryQuantizer.fit(thr, low, high).quantize(np.asarray(x, np.float32)).tolist() == expected
    _src, thr, low, high, dim = ka.BQ_LARGE
    x = np.random.default_rng(42).uniform(-1000, 1000, dim).astype(np.float32)
    assert np.array_equal(vq.BinaryQuantizer.fit(thr, low, high).quantize(x), (x >= 0).astype(np.uint8))


def test_sq_scalars_and_large(oracle):
    _src, vmin, vmax, levels, values = ka.SQ_SCALARS
    q = vq.ScalarQuantizer.fit(vmin, vmax, levels)
    for v in values:  # one-element vectors, like the reference test
        idx = q.quantize(np.array([v], np.float32))
        recon = q.min + float(idx[0]) * q.step
        assert abs(recon - min(max(v, vmin), vmax)) <= q.step / 2 + 1e-6
    _src, vmin, vmax, levels, shape = ka.SQ_LARGE
    x = np.random.default_rng(42).uniform(-1000, 1000, shape).astype(np.float32)
    q = vq.ScalarQuantizer.fit(vmin, vmax, levels)
    idx = q.quantize(x)
    assert idx.shape == x.shape
    assert np.array_equal(idx, oracle.sq_quantize(vmin, vmax, levels, q.step, x))


def test_f16_exact_round_trip():
    # identical vectors come back exactly through the f16 output (tests/test_tsvq.rs:11-22 pins this for f16 outputs)
    vals = np.asarray(ka.F16_EXACT[:8], np.float32)
    data = np.tile(vals, (10, 1))
    pq = vq.ProductQuantizer.fit(data, 2, 1, 5, vq.Distance.Euclidean, 0)
    out = pq.quantize(data[0])
    assert out.dtype == np.float16 and np.array_equal(out.astype(np.float32), vals)
