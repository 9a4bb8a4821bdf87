"""OptimizedProductQuantizer on the GPU against the CPU oracle (rotation agrees to rounding: the reference's SVD and
matrix products come from nalgebra, whose operation order is not pinned)."""
import numpy as np
import pytest

import vq_b200 as vq
from tests.golden import reference_known_answers as ka
from tests.util import RecordingSeeder
from vq_b200 import synth

pytestmark = pytest.mark.gpu


def test_reference_test_shape(oracle):
    """tests/test_opq.rs:10-80: 1000 x 10 in [-1000,1000), m=2, k=2, 50 LBG iterations, 5 outer iterations."""
    x = synth.uniform(1000, 10, 42, -1000.0, 1000.0)
    oq = vq.OptimizedProductQuantizer.fit(x, 2, 2, 50, 5, vq.Distance.SquaredEuclidean, 42)
    rot = oq.rotation
    assert rot.shape == (10, 10)
    assert np.allclose(rot @ rot.T, np.eye(10), atol=1e-5)
    for v in x[:10]:
        q = oq.quantize(v)
        assert q.shape == (10,) and np.isfinite(q.astype(np.float32)).all()


def test_quantize_given_identical_parts_is_bit_exact_after_rotation(oracle):
    """Given the same rotation and codebooks, codes match the oracle except where the rotated value differs in the last
    place (the rotation product's order is unspecified); such rows are near-ties and are counted."""
    rng = np.random.default_rng(6)
    dim, m, k = 32, 4, 16
    qmat, _ = np.linalg.qr(rng.normal(size=(dim, dim)))
    rot = qmat.astype(np.float32)
    cb = rng.normal(size=(m, k, dim // m)).astype(np.float32)
    x = rng.normal(size=(3000, dim)).astype(np.float32)
    oq = vq.OptimizedProductQuantizer.from_parts(rot, cb, vq.Distance.Euclidean)
    out, codes = oq.quantize(x, return_codes=True)
    out_o, codes_o = oracle.opq_quantize(rot, cb, x, ka.EUCLID)
    mism = int((codes != codes_o).sum())
    assert mism <= 3, mism
    same = (codes == codes_o).all(axis=1)
    assert np.array_equal(out.view(np.uint16)[same], out_o[same])


@pytest.mark.parametrize("name", ["SquaredEuclidean", "CosineDistance", "Manhattan", "Chebyshev", "Hamming"])
def test_quantize_with_every_metric_given_identical_parts(oracle, name):
    """src/opq.rs:246-261 compares with the quantizer's Distance.  A permutation matrix as rotation keeps the rotated rows
    exact, so the codes must equal the oracle's bit for bit."""
    from tests.util import METRICS
    rng = np.random.default_rng(16)
    dim, m, k = 24, 3, 13
    rot = np.eye(dim, dtype=np.float32)[rng.permutation(dim)]
    cb = rng.normal(size=(m, k, dim // m)).astype(np.float32)
    x = rng.normal(size=(1200, dim)).astype(np.float32)
    if name == "Hamming":
        x, cb = np.round(x), np.round(cb)
    oq = vq.OptimizedProductQuantizer.from_parts(rot, cb, getattr(vq.Distance, name))
    out, codes = oq.quantize(x, return_codes=True)
    out_o, codes_o = oracle.opq_quantize(rot, cb, x, METRICS[name])
    assert np.array_equal(codes, codes_o)
    assert np.array_equal(out.view(np.uint16), out_o)


def test_one_outer_iteration_matches_the_oracle(oracle):
    """First outer iteration starts from the identity, so codebooks are bit-exact; the rotation agrees to 1e-4."""
    x = synth.correlated(4000, 16, 3)
    n, m, k = 4000, 4, 16
    so = RecordingSeeder(7)
    init = so.init_pq(n, m, k)
    rot_o, cb_o = oracle.opq_fit(x, m, k, 5, 1, ka.EUCLID, init, so.draw)
    oq = vq.OptimizedProductQuantizer.fit(x, m, k, 5, 1, vq.Distance.Euclidean, 7, init_idx=init, accumulate=vq.ACCUM_ORDERED)
    assert np.array_equal(oq.codebooks, cb_o)
    assert np.allclose(oq.rotation, rot_o, atol=2e-4)
    assert np.allclose(oq.rotation @ oq.rotation.T, np.eye(16), atol=1e-5)


def test_full_fit_improves_error_like_the_oracle(oracle):
    """Several outer iterations on correlated data: reconstruction error of the rotated data within 1 % + rounding of the
    oracle's, orthogonal rotation."""
    x = synth.correlated(6000, 32, 3)
    n, m, k = 6000, 8, 16
    so = RecordingSeeder(9)
    init = so.init_pq(n, m, k)
    rot_o, cb_o = oracle.opq_fit(x, m, k, 5, 4, ka.EUCLID, init, so)
    oq = vq.OptimizedProductQuantizer.fit(x, m, k, 5, 4, vq.Distance.Euclidean, 9, init_idx=init, accumulate=vq.ACCUM_ORDERED)
    rot = oq.rotation
    assert np.allclose(rot @ rot.T, np.eye(32), atol=1e-5)
    out = oq.quantize(x)
    out_o, _ = oracle.opq_quantize(rot_o, cb_o, x, ka.EUCLID)
    err_g = oracle.mse_f16(oracle.rotate_rows(rot, x), out.view(np.uint16))
    err_o = oracle.mse_f16(oracle.rotate_rows(rot_o, x), out_o)
    assert abs(err_g - err_o) <= 0.02 * err_o


def test_zero_outer_iterations_gives_identity_and_empty_output():
    x = synth.uniform01(100, 8, 1)
    oq = vq.OptimizedProductQuantizer.fit(x, 2, 4, 5, 0, vq.Distance.Euclidean, 0)
    assert np.array_equal(oq.rotation, np.eye(8, dtype=np.float32))
    assert oq.quantize(x[0]).shape == (0,)


def test_errors():
    x = synth.uniform01(10, 3, 1)
    with pytest.raises(vq.EmptyInput):
        vq.OptimizedProductQuantizer.fit(np.zeros((0, 4), np.float32), 2, 2, 5, 2, vq.Distance.Euclidean, 0)
    with pytest.raises(vq.InvalidParameter) as e:
        vq.OptimizedProductQuantizer.fit(x, 4, 2, 5, 2, vq.Distance.Euclidean, 0)
    assert str(e.value) == ka.ERROR_TEXTS["opq_dim_lt_m"]
    with pytest.raises(vq.InvalidParameter) as e:
        vq.OptimizedProductQuantizer.fit(x, 2, 2, 5, 2, vq.Distance.Euclidean, 0)
    assert str(e.value) == ka.ERROR_TEXTS["opq_dim_mod_m"]
    oq = vq.OptimizedProductQuantizer.fit(x, 3, 2, 5, 2, vq.Distance.Euclidean, 0)
    with pytest.raises(vq.DimensionMismatch) as e:
        oq.quantize(np.zeros(4, np.float32))
    assert str(e.value) == "Dimension mismatch: expected 3, got 4"
