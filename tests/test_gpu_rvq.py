"""ResidualQuantizer on the GPU against the CPU oracle."""
import numpy as np
import pytest

import vq_b200 as vq
from tests.golden import reference_known_answers as ka
from tests.util import METRICS, RecordingSeeder, by_stream
from vq_b200 import synth

pytestmark = pytest.mark.gpu


def _fit_both(oracle, x, stages, k, iters, eps, name, seed=42, accumulate=vq.ACCUM_ORDERED):
    so, sg = RecordingSeeder(seed), RecordingSeeder(seed)
    cb_o, res_o, norms_o = oracle.rvq_fit(x, stages, k, iters, eps, METRICS[name], so.init_stage, so.draw)
    rq = vq.ResidualQuantizer.fit(x, stages, k, iters, eps, getattr(vq.Distance, name), seed, init=sg.init_stage,
                                  draw=sg.draw, accumulate=accumulate)
    return cb_o, so, rq, sg


def test_reference_test_shape(oracle):
    """tests/test_rvq.rs:10-62: 1000 x 10 in [-1000,1000), 2 stages (m=2), k=2, 50 iterations, epsilon 1e-6."""
    x = synth.uniform(1000, 10, 42, -1000.0, 1000.0)
    cb_o, so, rq, sg = _fit_both(oracle, x, 2, 2, 50, 1e-6, "SquaredEuclidean")
    assert rq.shape() == (2, 2, 10)
    assert np.array_equal(rq.codebooks, cb_o) and by_stream(so.draws) == by_stream(sg.draws)
    for v in x[:10]:
        q = rq.quantize(v)
        assert q.shape == (10,) and np.isfinite(q.astype(np.float32)).all()
    out, codes = rq.quantize(x, return_codes=True)
    out_o, codes_o, _ = oracle.rvq_quantize(cb_o, 1e-6, x, ka.SQ)
    assert np.array_equal(codes, codes_o) and np.array_equal(out.view(np.uint16), out_o)


@pytest.mark.parametrize("n,dim,stages,k,name", [(2000, 128, 3, 32, "Euclidean"), (777, 20, 4, 9, "Manhattan"),
                                                  (500, 7, 2, 5, "CosineDistance"), (300, 33, 2, 1, "Euclidean"),
                                                  (1200, 64, 2, 300, "SquaredEuclidean")])
def test_fit_and_quantize_bit_exact(oracle, n, dim, stages, k, name):
    x = synth.gaussian_mixture(n, dim, 11, components=8)
    cb_o, so, rq, sg = _fit_both(oracle, x, stages, k, 5, 0.01, name)
    assert rq.shape()[0] == cb_o.shape[0]
    assert np.array_equal(rq.codebooks, cb_o) and by_stream(so.draws) == by_stream(sg.draws)
    out, codes = rq.quantize(x, return_codes=True)
    out_o, codes_o, _ = oracle.rvq_quantize(cb_o, 0.01, x, METRICS[name])
    assert np.array_equal(codes, codes_o)
    assert np.array_equal(out.view(np.uint16), out_o)


@pytest.mark.parametrize("name", sorted(METRICS))
def test_encode_with_every_metric_given_identical_codebooks(oracle, name):
    """src/rvq.rs:186-199 takes whatever Distance the quantizer was built with (src/distances.rs:115-172)."""
    rng = np.random.default_rng(21)
    cb = rng.normal(size=(3, 11, 24)).astype(np.float32)
    cb[1, 4] = cb[1, 2]                      # duplicate centroid: the lower index wins
    x = rng.normal(size=(900, 24)).astype(np.float32)
    x[5] = 0.0
    if name == "Hamming":
        x, cb = np.round(x), np.round(cb)
    rq = vq.ResidualQuantizer.from_codebooks(cb, 0.01, getattr(vq.Distance, name))
    out, codes = rq.quantize(x, return_codes=True)
    out_o, codes_o, _ = oracle.rvq_quantize(cb, 0.01, x, METRICS[name])
    assert np.array_equal(codes, codes_o)
    assert np.array_equal(out.view(np.uint16), out_o)


@pytest.mark.parametrize("name", ["Chebyshev", "Hamming"])
def test_fit_with_the_rarer_metrics(oracle, name):
    """The residual update of a stage (src/rvq.rs:111-128) uses the quantizer's metric; the k-means itself is Euclidean."""
    x = synth.gaussian_mixture(600, 12, 3, components=5)
    if name == "Hamming":
        x = np.round(x * 4.0).astype(np.float32)
    cb_o, so, rq, sg = _fit_both(oracle, x, 3, 7, 4, 0.01, name)
    assert np.array_equal(rq.codebooks, cb_o) and by_stream(so.draws) == by_stream(sg.draws)


def test_minkowski_codes_within_near_ties(oracle):
    rng = np.random.default_rng(22)
    cb = rng.normal(size=(2, 9, 16)).astype(np.float32)
    x = rng.normal(size=(500, 16)).astype(np.float32)
    rq = vq.ResidualQuantizer.from_codebooks(cb, 0.01, vq.Distance.Minkowski(3.0))
    _, codes = rq.quantize(x, return_codes=True)
    _, codes_o, _ = oracle.rvq_quantize(cb, 0.01, x, ka.MINKOWSKI, 3.0)
    # powf differs in the last place between libm and CUDA: a first-stage near-tie changes the later stages of that row too
    assert int((codes != codes_o).any(axis=1).sum()) <= 5


def test_training_stops_when_the_mean_residual_norm_drops_below_epsilon(oracle):
    """src/rvq.rs:131-148: with every row equal to one of k points the first stage leaves zero residuals, so only one
    codebook is produced although more stages were asked for."""
    base = synth.uniform01(4, 16, 3)
    x = np.repeat(base, 50, axis=0)
    so = RecordingSeeder(1)
    # initial sample = one row of each distinct point, so stage 0 reproduces the data exactly
    init = lambda stage, n, k: np.array([0, 50, 100, 150], np.uint64)  # noqa: E731
    cb_o, _res, _norms = oracle.rvq_fit(x, 5, 4, 10, 0.01, ka.EUCLID, init, so.draw)
    rq = vq.ResidualQuantizer.fit(x, 5, 4, 10, 0.01, vq.Distance.Euclidean, 1, init=init)
    assert cb_o.shape[0] == 1 and rq.shape()[0] == 1
    assert np.array_equal(rq.codebooks, cb_o)


def test_per_row_early_exit_in_quantize(oracle):
    """src/rvq.rs:204-207: a row whose residual norm falls below epsilon stops consuming stages."""
    rng = np.random.default_rng(4)
    cb = rng.normal(size=(3, 6, 12)).astype(np.float32)
    x = rng.normal(size=(50, 12)).astype(np.float32)
    x[7] = cb[0, 2]                      # exact hit in stage 0: residual 0 -> stop after one stage
    x[9] = cb[0, 1] + cb[1, 4]           # residual after stage 0 may or may not pick (1,4); the oracle decides
    rq = vq.ResidualQuantizer.from_codebooks(cb, 0.05, vq.Distance.Euclidean)
    out, codes = rq.quantize(x, return_codes=True)
    out_o, codes_o, _ = oracle.rvq_quantize(cb, 0.05, x, ka.EUCLID)
    assert codes_o[7, 1] == 0xFFFFFFFF  # the case exercises the early exit
    assert np.array_equal(codes, codes_o) and np.array_equal(out.view(np.uint16), out_o)


def test_zero_stages_gives_zero_output():
    x = synth.uniform01(10, 8, 1)
    rq = vq.ResidualQuantizer.fit(x, 0, 4, 5, 0.01, vq.Distance.Euclidean, 0)
    assert rq.shape()[0] == 0
    out = rq.quantize(x)
    assert out.shape == (10, 8) and not out.astype(np.float32).any()


def test_errors():
    with pytest.raises(vq.EmptyInput) as e:
        vq.ResidualQuantizer.fit(np.zeros((0, 4), np.float32), 2, 2, 5, 0.01, vq.Distance.Euclidean, 0)
    assert str(e.value) == ka.ERROR_TEXTS["pq_empty"]
    x = synth.uniform01(10, 4, 1)
    with pytest.raises(vq.InvalidParameter) as e:
        vq.ResidualQuantizer.fit(x, 2, 11, 5, 0.01, vq.Distance.Euclidean, 0)
    assert str(e.value) == ka.ERROR_TEXTS["n_lt_k"]
    rq = vq.ResidualQuantizer.fit(x, 2, 2, 5, 0.01, vq.Distance.Euclidean, 0)
    with pytest.raises(vq.DimensionMismatch) as e:
        rq.quantize(np.zeros(5, np.float32))
    assert str(e.value) == "Dimension mismatch: expected 4, got 5"


def test_mixture_config_scaled_down(oracle):
    """The mixture benchmark configuration scaled to 20,000 rows: 64-component mixture in 128-d, 8 stages, k=256, Euclidean.
    Fast (unordered) accumulation: codebooks within tolerance after the first stage, final error within 1 %."""
    x = synth.gaussian_mixture(20000, 128, 11)
    so, sg = RecordingSeeder(5), RecordingSeeder(5)
    cb_o, _res, _n = oracle.rvq_fit(x, 3, 256, 4, 0.01, ka.EUCLID, so.init_stage, so.draw)
    rq = vq.ResidualQuantizer.fit(x, 3, 256, 4, 0.01, vq.Distance.Euclidean, 5, init=sg.init_stage, draw=sg.draw,
                                  accumulate=vq.ACCUM_FAST)
    assert rq.shape()[0] == cb_o.shape[0]
    out = rq.quantize(x)
    out_o, _c, _s = oracle.rvq_quantize(cb_o, 0.01, x, ka.EUCLID)
    mse_g, mse_o = oracle.mse_f16(x, out.view(np.uint16)), oracle.mse_f16(x, out_o)
    assert abs(mse_g - mse_o) <= 0.01 * mse_o
