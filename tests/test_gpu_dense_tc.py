"""The tensor-core (tcgen05) shortlist of the full-width nearest-centroid search: dot products within the proven
TF32 error bound, and the final choice (after the exact resolve) identical to the CUDA-core / oracle result."""
import ctypes as C

import numpy as np
import pytest

import vq_b200 as vq
from tests.golden import reference_known_answers as ka
from tests.util import RecordingSeeder, by_stream
from vq_b200 import _lib, synth

pytestmark = pytest.mark.gpu


def _dots(ctx, x, cb):
    n, dim = x.shape
    k = cb.shape[0]
    dots = np.zeros((n, 256), np.float32)
    stats = (C.c_ulonglong * 3)()
    rc = _lib.load().vqb_dense_dots(ctx.handle, x.ctypes.data, n, dim, cb.ctypes.data, k, dots.ctypes.data, stats)
    assert rc == 0, _lib.load().vqb_last_error(ctx.handle).decode()
    return dots, [int(v) for v in stats]


@pytest.mark.parametrize("n,dim,k", [(128, 128, 256), (1000, 128, 256), (333, 64, 100), (4097, 32, 2), (5000, 96, 17)])
def test_tf32_dot_products_within_the_bound(ctx, n, dim, k):
    rng = np.random.default_rng(n + dim)
    x = rng.normal(size=(n, dim)).astype(np.float32)
    cb = rng.normal(size=(k, dim)).astype(np.float32)
    dots, stats = _dots(ctx, x, cb)
    exact = x.astype(np.float64) @ cb.astype(np.float64).T
    scale = np.linalg.norm(x, axis=1)[:, None] * np.linalg.norm(cb, axis=1)[None, :]
    rel = np.abs(dots[:, :k] - exact) / scale
    assert rel.max() < 2.1e-3, rel.max()       # the bound the shortlist margin is built on
    assert rel.max() > 1e-7                    # TF32 really is in use (not an f32 fallback)
    assert not dots[:, k:].any()
    assert stats[0] == n


def test_rvq_fit_and_quantize_tensor_path_bit_exact(oracle):
    """128-d mixture rows: training (k-means per stage), residual update and encode all go through the tensor-core
    shortlist; codebooks, codes and f16 output must still equal the oracle's bit for bit (ordered sums, n <= 65536)."""
    x = synth.gaussian_mixture(6000, 128, 11, components=16)
    so, sg = RecordingSeeder(3), RecordingSeeder(3)
    cb_o, _res, _norms = oracle.rvq_fit(x, 3, 64, 5, 0.01, ka.EUCLID, so.init_stage, so.draw)
    rq = vq.ResidualQuantizer.fit(x, 3, 64, 5, 0.01, vq.Distance.Euclidean, 3, init=sg.init_stage, draw=sg.draw,
                                  accumulate=vq.ACCUM_ORDERED)
    assert np.array_equal(rq.codebooks, cb_o) and by_stream(so.draws) == by_stream(sg.draws)
    out, codes = rq.quantize(x, return_codes=True)
    out_o, codes_o, _ = oracle.rvq_quantize(cb_o, 0.01, x, ka.EUCLID)
    assert np.array_equal(codes, codes_o)
    assert np.array_equal(out.view(np.uint16), out_o)


def test_lbg_full_width_with_duplicates_and_specials(oracle):
    """Duplicate rows (exact ties between centroids), a NaN row and an infinite row: the shortlist must hand these to the
    exact scan so that the reference's tie-breaking and NaN behaviour survive."""
    base = synth.uniform01(50, 64, 2)
    x = np.repeat(base, 20, axis=0)
    x[7, 3] = np.nan
    x[11, 5] = np.inf
    so = RecordingSeeder(8)
    init = so.init_stage(0, 1000, 32)
    cent_o, assign_o, it_o = oracle.lbg(x, 32, 4, init, so.draw)
    sg = RecordingSeeder(8)
    sg.init_stage(0, 1000, 32)
    cent, it = vq.lbg_quantize(x, 32, 4, 8, init_idx=init, draw=sg.draw, accumulate=vq.ACCUM_ORDERED)
    assert it == it_o
    assert np.array_equal(cent, cent_o, equal_nan=True)


def test_pq_filter_kernel_matches_the_default_path(oracle):
    """The CUDA-core filter kernel of the product quantizer (VQB_PQ_TENSOR=0) in a child process: codebooks and codes must
    be bit-identical to the oracle's, like the default tcgen05 path."""
    import os
    import subprocess
    import sys
    import tempfile
    code = r"""
import sys, numpy as np
sys.path.insert(0, %r)
import vq_b200 as vq
from vq_b200 import synth
from vq_b200.seeding import LbgSeeder
x = synth.uniform01(20000, 128, 42)
s = LbgSeeder(42)
init = np.stack([s.init_indices(i, 20000, 256) for i in range(16)])
pq = vq.ProductQuantizer.fit(x, 16, 256, 4, vq.Distance.Euclidean, 42, init_idx=init, draw=s.draw, accumulate=vq.ACCUM_ORDERED)
out, codes = pq.quantize(x, return_codes=True)
np.savez(sys.argv[1], cb=pq.codebooks, codes=codes, out=out.view(np.uint16))
""" % os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    from vq_b200 import synth
    from vq_b200.seeding import LbgSeeder
    with tempfile.TemporaryDirectory() as d:
        path = os.path.join(d, "r.npz")
        res = subprocess.run([sys.executable, "-c", code, path], env=dict(os.environ, VQB_PQ_TENSOR="0"), stdout=subprocess.PIPE,
                             stderr=subprocess.STDOUT, timeout=600)
        assert res.returncode == 0, res.stdout.decode()[-2000:]
        got = np.load(path)
        x = synth.uniform01(20000, 128, 42)
        s = LbgSeeder(42)
        init = np.stack([s.init_indices(i, 20000, 256) for i in range(16)])
        cb_o, _ = oracle.pq_fit(x, 16, 256, 4, init, s.draw)
        out_o, codes_o = oracle.pq_quantize(cb_o, x, ka.EUCLID)
        assert np.array_equal(got["cb"], cb_o)
        assert np.array_equal(got["codes"], codes_o) and np.array_equal(got["out"], out_o)
