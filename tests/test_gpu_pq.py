"""ProductQuantizer on the GPU (through the C ABI) against the CPU oracle on identical seeded inputs."""
import numpy as np
import pytest

import vq_b200 as vq
from tests.golden import reference_known_answers as ka
from tests.util import METRICS, RecordingSeeder, by_stream, near_tie_mismatches
from vq_b200 import synth

pytestmark = pytest.mark.gpu


def _fit_both(oracle, x, m, k, iters, seed, accumulate=vq.ACCUM_ORDERED, metric=vq.Distance.Euclidean):
    n = x.shape[0]
    so, sg = RecordingSeeder(seed), RecordingSeeder(seed)
    init = so.init_pq(n, m, k)
    sg.init_pq(n, m, k)
    cb_o, it_o = oracle.pq_fit(x, m, k, iters, init, so.draw)
    pq = vq.ProductQuantizer.fit(x, m, k, iters, metric, seed, init_idx=init, draw=sg.draw, accumulate=accumulate)
    return cb_o, it_o, so, pq, sg


def test_10k_shape_bit_exact_training_and_encode(oracle):
    """10,000 x 128 uniform [0,1), m=16, k=256, 10 iterations, Euclidean: every cluster stays under 1025 members,
    so the reference is deterministic and the whole trajectory must match bit for bit."""
    x = synth.uniform01(10000, 128, 42)
    cb_o, it_o, so, pq, sg = _fit_both(oracle, x, 16, 256, 10, 42)
    assert np.array_equal(pq.iterations, it_o)
    assert by_stream(so.draws) == by_stream(sg.draws)
    assert np.array_equal(pq.codebooks, cb_o)
    out, codes = pq.quantize(x, return_codes=True)
    out_o, codes_o = oracle.pq_quantize(cb_o, x, ka.EUCLID)
    assert np.array_equal(codes, codes_o)
    assert np.array_equal(out.view(np.uint16), out_o)
    mse = oracle.mse_f16(x, out.view(np.uint16))
    assert 0.015 < mse < 0.025  # the reference publishes 0.0196 at n = 10k (notebooks/performance_analysis.ipynb)


def test_reference_test_shape(oracle):
    """tests/test_pq.rs:10-45: 1000 x 10 in [-1000, 1000), m=2, k=2, 50 iterations, SquaredEuclidean."""
    x = synth.uniform(1000, 10, 42, -1000.0, 1000.0)
    cb_o, it_o, so, pq, sg = _fit_both(oracle, x, 2, 2, 50, 42, metric=vq.Distance.SquaredEuclidean)
    assert np.array_equal(pq.codebooks, cb_o) and np.array_equal(pq.iterations, it_o)
    for v in x[:20]:  # one vector per call, like the reference API
        q = pq.quantize(v)
        assert q.shape == (10,) and np.isfinite(q.astype(np.float32)).all()
    out, codes = pq.quantize(x, return_codes=True)
    out_o, codes_o = oracle.pq_quantize(cb_o, x, ka.SQ)
    assert np.array_equal(codes, codes_o) and np.array_equal(out.view(np.uint16), out_o)


@pytest.mark.parametrize("n,dim,m,k", [(777, 16, 4, 16), (1, 8, 2, 1), (33, 32, 2, 7), (2049, 24, 3, 30), (500, 10, 2, 9),
                                        (600, 7, 7, 5), (3000, 16, 2, 300), (400, 260, 1, 6)])
def test_shapes_bit_exact(oracle, n, dim, m, k):
    """Sub-space widths 4/8/16 (register kernel), 5/1/260 (generic kernel), k not a multiple of 4, k > 256 (16-bit codes),
    row counts that are not a multiple of the tile."""
    x = synth.uniform01(n, dim, 1000 + n)
    cb_o, it_o, so, pq, sg = _fit_both(oracle, x, m, k, 6, 9)
    assert np.array_equal(pq.iterations, it_o) and by_stream(so.draws) == by_stream(sg.draws)
    assert np.array_equal(pq.codebooks, cb_o)
    out, codes = pq.quantize(x, return_codes=True)
    out_o, codes_o = oracle.pq_quantize(cb_o, x, ka.EUCLID)
    assert np.array_equal(codes, codes_o) and np.array_equal(out.view(np.uint16), out_o)


@pytest.mark.parametrize("name", sorted(METRICS))
@pytest.mark.parametrize("dim,m", [(32, 4), (20, 4)])
def test_encode_metrics_given_identical_codebooks(oracle, name, dim, m):
    rng = np.random.default_rng(11)
    k = 37
    cb = rng.normal(size=(m, k, dim // m)).astype(np.float32)
    cb[1, 5] = cb[1, 3]          # duplicate centroid: the lower index must win
    cb[2, 0] = 0.0               # zero-norm centroid: cosine distance 1 (src/distances.rs:146-147)
    x = rng.normal(size=(1500, dim)).astype(np.float32)
    x[3] = 0.0
    x[10, : dim // m] = cb[0, 7]  # exact hit
    if name == "Hamming":
        x = np.round(x)
        cb = np.round(cb)
    metric = METRICS[name]
    pq = vq.ProductQuantizer.from_codebooks(cb, getattr(vq.Distance, name))
    out, codes = pq.quantize(x, return_codes=True)
    out_o, codes_o = oracle.pq_quantize(cb, x, metric)
    assert np.array_equal(codes, codes_o)
    assert np.array_equal(out.view(np.uint16), out_o)


def test_minkowski_codes_within_near_ties(oracle):
    rng = np.random.default_rng(12)
    cb = rng.normal(size=(4, 16, 8)).astype(np.float32)
    x = rng.normal(size=(800, 32)).astype(np.float32)
    pq = vq.ProductQuantizer.from_codebooks(cb, vq.Distance.Minkowski(3.0))
    _, codes = pq.quantize(x, return_codes=True)
    _, codes_o = oracle.pq_quantize(cb, x, ka.MINKOWSKI, 3.0)
    near, real = near_tie_mismatches(oracle, cb, x, codes, codes_o, ka.MINKOWSKI, 3.0)
    assert real == 0 and near <= 8


def sqrt_merge_case():
    """Codebook where centroid 2 has the smaller SQUARED distance to the origin but the same f32 square root as
    centroid 0 (values found by search; the premises are re-checked here in f32)."""
    f = np.float32
    a, u, t = f(1.500100016593933), f(1.500099778175354), f(0.000699999975040555)
    s0 = f(a * a)
    s2 = f(f(u * u) + f(t * t))
    assert s2 < s0 and np.sqrt(s2) == np.sqrt(s0)
    cb = np.zeros((1, 4, 8), np.float32)
    cb[0, 0, 0] = a
    cb[0, 1] = 50.0
    cb[0, 2, 0], cb[0, 2, 1] = u, t
    cb[0, 3] = 60.0
    return cb


def test_euclidean_sqrt_merged_ties_pick_the_lower_index(oracle):
    """The reference compares square roots (src/distances.rs:134-140): when two different squared sums round to the
    same root, the LOWER index keeps the win even though its squared sum is larger."""
    cb = sqrt_merge_case()
    x = np.zeros((70, 8), np.float32)
    pq_e = vq.ProductQuantizer.from_codebooks(cb, vq.Distance.Euclidean)
    pq_s = vq.ProductQuantizer.from_codebooks(cb, vq.Distance.SquaredEuclidean)
    _, ce = pq_e.quantize(x, return_codes=True)
    _, cs = pq_s.quantize(x, return_codes=True)
    _, ce_o = oracle.pq_quantize(cb, x, ka.EUCLID)
    _, cs_o = oracle.pq_quantize(cb, x, ka.SQ)
    assert ce_o[0, 0] == 0 and cs_o[0, 0] == 2  # the case really separates the two metrics
    assert np.array_equal(ce, ce_o) and np.array_equal(cs, cs_o)


def test_nan_and_inf_inputs_follow_strict_less_than(oracle):
    rng = np.random.default_rng(13)
    cb = rng.normal(size=(2, 9, 8)).astype(np.float32)
    x = rng.normal(size=(40, 16)).astype(np.float32)
    x[0, 0] = np.nan
    x[1, 9] = np.inf
    x[2, :] = -np.inf
    cb2 = cb.copy()
    cb2[0, 0, 0] = np.nan  # centroid 0 gives NaN: nothing can replace it (src/pq.rs:166-174)
    for c in (cb, cb2):
        for name in ("Euclidean", "SquaredEuclidean", "Manhattan", "CosineDistance"):
            pq = vq.ProductQuantizer.from_codebooks(c, getattr(vq.Distance, name))
            _, codes = pq.quantize(x, return_codes=True)
            _, codes_o = oracle.pq_quantize(c, x, METRICS[name])
            assert np.array_equal(codes, codes_o), name


def test_empty_clusters_are_reseeded_in_reference_order(oracle):
    """Many duplicate rows make duplicate centroids; the higher index never wins a tie, goes empty and is re-seeded
    from the draw callback, ascending cluster index, one draw each (src/utils.rs:95-101)."""
    base = synth.uniform01(40, 16, 5)
    x = np.repeat(base, 25, axis=0)  # 1000 rows, 40 distinct
    cb_o, it_o, so, pq, sg = _fit_both(oracle, x, 2, 64, 8, 21)
    assert len(so.draws) > 0
    assert by_stream(so.draws) == by_stream(sg.draws)
    assert np.array_equal(pq.iterations, it_o)
    assert np.array_equal(pq.codebooks, cb_o)


def test_max_iters_zero_keeps_the_initial_sample(oracle):
    x = synth.uniform01(100, 8, 2)
    cb_o, it_o, so, pq, sg = _fit_both(oracle, x, 2, 5, 0, 3)
    assert np.array_equal(pq.codebooks, cb_o) and not pq.iterations.any()


def test_fast_accumulation_within_reference_tolerance(oracle):
    """Unordered (atomic) cluster sums: per-centroid relative error <= 1e-3 after the first iteration and the final
    reconstruction error within 1 % of the ordered result (the reference's own >1024-member sums are unordered too)."""
    x = synth.uniform01(60000, 32, 77)
    n, m, k = x.shape[0], 4, 16  # ~3750 members per cluster
    so = RecordingSeeder(5)
    init = so.init_pq(n, m, k)
    cb1_o, _ = oracle.pq_fit(x, m, k, 1, init, so.draw)
    pq1 = vq.ProductQuantizer.fit(x, m, k, 1, vq.Distance.Euclidean, 5, init_idx=init, accumulate=vq.ACCUM_FAST)
    rel = np.linalg.norm(pq1.codebooks - cb1_o, axis=2) / np.linalg.norm(cb1_o, axis=2)
    assert rel.max() <= 1e-3
    cb_o, _ = oracle.pq_fit(x, m, k, 10, init, so.draw)
    pq = vq.ProductQuantizer.fit(x, m, k, 10, vq.Distance.Euclidean, 5, init_idx=init, accumulate=vq.ACCUM_FAST)
    mse_g = oracle.mse_f16(x, pq.quantize(x).view(np.uint16))
    mse_o = oracle.mse_f16(x, oracle.pq_quantize(cb_o, x, ka.EUCLID)[0])
    assert abs(mse_g - mse_o) <= 0.01 * mse_o


def test_errors_match_the_reference(oracle):
    x = synth.uniform01(10, 3, 1)
    with pytest.raises(vq.EmptyInput) as e:
        vq.ProductQuantizer.fit(np.zeros((0, 4), np.float32), 2, 2, 5, vq.Distance.Euclidean, 0)
    assert str(e.value) == ka.ERROR_TEXTS["pq_empty"]
    with pytest.raises(vq.EmptyInput):
        vq.ProductQuantizer.fit([], 2, 2, 5, vq.Distance.Euclidean, 0)
    with pytest.raises(vq.InvalidParameter) as e:
        vq.ProductQuantizer.fit(x, 4, 2, 5, vq.Distance.Euclidean, 0)
    assert str(e.value) == ka.ERROR_TEXTS["pq_dim_lt_m"]
    with pytest.raises(vq.InvalidParameter) as e:
        vq.ProductQuantizer.fit(x, 2, 2, 5, vq.Distance.Euclidean, 0)
    assert str(e.value) == ka.ERROR_TEXTS["pq_dim_mod_m"]
    with pytest.raises(vq.InvalidParameter) as e:
        vq.ProductQuantizer.fit(x, 3, 0, 5, vq.Distance.Euclidean, 0)
    assert str(e.value) == ka.ERROR_TEXTS["k_zero"]
    with pytest.raises(vq.InvalidParameter) as e:
        vq.ProductQuantizer.fit(x, 3, 11, 5, vq.Distance.Euclidean, 0)
    assert str(e.value) == ka.ERROR_TEXTS["n_lt_k"]
    pq = vq.ProductQuantizer.fit(x, 3, 2, 5, vq.Distance.Euclidean, 0)
    with pytest.raises(vq.DimensionMismatch) as e:
        pq.quantize(np.zeros(4, np.float32))
    assert str(e.value) == "Dimension mismatch: expected 3, got 4"
    pqm = vq.ProductQuantizer.fit(x, 3, 2, 5, vq.Distance.Minkowski(-1.0), 0)  # fit never evaluates the metric
    with pytest.raises(vq.InvalidMetricParameter) as e:
        pqm.quantize(x[0])
    assert str(e.value) == ka.ERROR_TEXTS["minkowski_p"]


def test_device_resident_tensors(oracle):
    import torch
    x = synth.uniform01(5000, 32, 8)
    xt = torch.from_numpy(x).cuda()
    so = RecordingSeeder(4)
    init = so.init_pq(5000, 4, 32)
    cb_o, _ = oracle.pq_fit(x, 4, 32, 5, init, so.draw)
    pq = vq.ProductQuantizer.fit(xt, 4, 32, 5, vq.Distance.Euclidean, 4, init_idx=init, accumulate=vq.ACCUM_ORDERED)
    assert np.array_equal(pq.codebooks, cb_o)
    out, codes = pq.quantize(xt, return_codes=True)
    assert out.is_cuda and out.dtype == torch.float16
    out_o, codes_o = oracle.pq_quantize(cb_o, x, ka.EUCLID)
    assert np.array_equal(out.cpu().numpy().view(np.uint16), out_o)
    assert np.array_equal(codes.cpu().numpy().astype(np.uint32), codes_o)
    # an unaligned view (row offset by one float) takes the scalar-load path and must agree too
    flat = torch.empty(5000 * 32 + 1, device="cuda")
    flat[1:] = xt.reshape(-1)
    out2 = pq.quantize(flat[1:].view(5000, 32))
    assert torch.equal(out2, out)


@pytest.mark.parametrize("mode", ["ordered", "fast"])
@pytest.mark.parametrize("n,iters", [(150_000, 4), (70_001, 2), (150_000, 0)])
def test_fit_from_a_host_buffer_follows_the_copy_and_equals_the_device_resident_fit(mode, n, iters):
    """A large host buffer is copied in pieces while the first iteration already assigns (and, unordered, adds up) the
    rows that have arrived, and the initial centroids are taken from the host copy.  Integer data make every sum exact,
    so the result must equal the fit on device-resident rows bit for bit in both accumulation modes; with no iterations
    the codebooks are the initial rows."""
    import torch
    m, k = 16, 64
    x = np.random.default_rng(n).integers(0, 16, (n, 128)).astype(np.float32)
    acc = vq.ACCUM_ORDERED if mode == "ordered" else vq.ACCUM_FAST
    sh, sd = RecordingSeeder(5), RecordingSeeder(5)
    init = sh.init_pq(n, m, k)
    sd.init_pq(n, m, k)
    pq_h = vq.ProductQuantizer.fit(x, m, k, iters, vq.Distance.Euclidean, 5, init_idx=init, draw=sh.draw, accumulate=acc)
    pq_d = vq.ProductQuantizer.fit(torch.from_numpy(x).cuda(), m, k, iters, vq.Distance.Euclidean, 5, init_idx=init, draw=sd.draw,
                                   accumulate=acc)
    assert np.array_equal(pq_h.iterations, pq_d.iterations)
    assert np.array_equal(pq_h.codebooks, pq_d.codebooks)
    assert by_stream(sh.draws) == by_stream(sd.draws)
    if iters == 0:
        want = x[init.reshape(-1)].reshape(m, k, m, 8)[np.arange(m), :, np.arange(m), :]
        assert np.array_equal(pq_h.codebooks.reshape(m, k, 8), want)


def test_quantize_into_a_callers_buffer():
    """`out=` takes the result where the caller wants it (page-locked host memory, or a CUDA tensor for device input): same
    bits as a fresh result, and a buffer of the wrong shape, type or side is refused."""
    import torch
    x = synth.uniform01(3000, 32, 3)
    pq = vq.ProductQuantizer.fit(x, 4, 16, 3, vq.Distance.Euclidean, 1)
    want = pq.quantize(x)
    buf = torch.empty((3000, 32), dtype=torch.float16, pin_memory=True)
    got = pq.quantize(x, out=buf.numpy())
    assert got is not None and np.array_equal(buf.numpy().view(np.uint16), want.view(np.uint16))
    dev = torch.empty((3000, 32), dtype=torch.float16, device="cuda")
    pq.quantize(torch.from_numpy(x).cuda(), out=dev)
    assert np.array_equal(dev.cpu().numpy().view(np.uint16), want.view(np.uint16))
    for bad in (np.empty((3000, 31), np.float16), np.empty((3000, 32), np.float32), dev):
        with pytest.raises(ValueError):
            pq.quantize(x, out=bad)
    sq = vq.ScalarQuantizer.fit(0.0, 1.0, 256)
    b8 = np.empty((3000, 32), np.uint8)
    sq.quantize(x, out=b8)
    assert np.array_equal(b8, sq.quantize(x))
    t = vq.TSVQ(x, 3, vq.Distance.Euclidean)
    bt = np.empty((3000, 32), np.float16)
    t.quantize(x, out=bt)
    assert np.array_equal(bt.view(np.uint16), t.quantize(x).view(np.uint16))


def test_full_size_properties_1m(oracle):
    """README scale (1,000,000 x 128, m=16, k=256): size-independent properties at full size plus an oracle
    comparison on a row sample."""
    import torch
    n = 1_000_000
    x = synth.uniform01(n, 128, 7)
    xt = torch.from_numpy(x).cuda()
    seeder = RecordingSeeder(42)
    init = seeder.init_pq(n, 16, 256)
    pq = vq.ProductQuantizer.fit(xt, 16, 256, 3, vq.Distance.Euclidean, 42, init_idx=init)
    cb = pq.codebooks
    assert np.isfinite(cb).all()
    out, codes = pq.quantize(xt, return_codes=True)
    codes_h = codes.cpu().numpy().astype(np.int64)
    out_h = out.cpu().numpy()
    # (1) the f16 output is exactly the f16 image of the chosen centroids
    recon = cb[np.arange(16)[None, :], codes_h].reshape(n, 128).astype(np.float16)
    assert np.array_equal(out_h.view(np.uint16), recon.view(np.uint16))
    # (2) every centroid is used by at least one row after training on the same rows, and codes are in range
    assert codes_h.min() >= 0 and codes_h.max() < 256
    # (3) sample of rows against the oracle, identical codebooks: bit-exact
    idx = np.random.default_rng(0).choice(n, 4000, replace=False)
    _, codes_o = oracle.pq_quantize(cb, x[idx], ka.EUCLID)
    assert np.array_equal(codes_h[idx].astype(np.uint32), codes_o)
    # (4) idempotence: the f32 reconstruction quantizes to itself
    rec32 = torch.from_numpy(cb[np.arange(16)[None, :], codes_h[:20000]].reshape(20000, 128)).cuda()
    out2 = pq.quantize(rec32)
    assert torch.equal(out2, out[:20000])
    # (5) first-iteration centroids within 1e-3 of the oracle on a subsample of subspaces is covered by
    #     test_fast_accumulation_within_reference_tolerance; here: reconstruction error in the published range
    mse = float(((xt - out.float()) ** 2).mean())
    assert 0.015 < mse < 0.03


def test_large_host_batch_goes_through_the_chunked_pipeline(oracle):
    """Host arrays of >= 131072 rows are encoded in 65536-row chunks with copies and kernels overlapped; the result
    must not depend on the chunking (row count deliberately not a multiple of the chunk)."""
    n = 200_003
    x = synth.uniform01(n, 16, 77)
    rng = np.random.default_rng(2)
    cb = rng.uniform(0, 1, (2, 32, 8)).astype(np.float32)
    pq = vq.ProductQuantizer.from_codebooks(cb, vq.Distance.Euclidean)
    out, codes = pq.quantize(x, return_codes=True)
    out_o, codes_o = oracle.pq_quantize(cb, x, ka.EUCLID)
    assert np.array_equal(codes, codes_o) and np.array_equal(out.view(np.uint16), out_o)
    only_f16 = pq.quantize(x)
    assert np.array_equal(only_f16.view(np.uint16), out_o)


@pytest.mark.parametrize("n,m,dim", [(70_000, 16, 128), (500_000, 16, 128), (90_000, 4, 32), (80_000, 2, 128)])
def test_unordered_accumulation_moves_only_changed_rows_and_stays_exact_on_integers(oracle, n, m, dim):
    """From the second iteration on the unordered accumulation adds and subtracts only the rows whose assignment changed
    (three kernels: 64-bit code words with 128-bit atomics for small shards, per-CTA sums for large ones, whole rows for wide
    sub-spaces).  Small integers make every f32 sum exact whatever the order, so the codebooks, the iteration counts and the
    draws must equal the oracle's bit for bit; any slip in the bookkeeping (a row added twice, a count off by one) shows."""
    oracle.use_all_host_threads()
    k, iters = 64, 6
    x = np.random.default_rng(n + m).integers(0, 16, (n, dim)).astype(np.float32)
    so, sg = RecordingSeeder(13), RecordingSeeder(13)
    init = so.init_pq(n, m, k)
    sg.init_pq(n, m, k)
    cb_o, it_o = oracle.pq_fit(x, m, k, iters, init, so.draw)
    pq = vq.ProductQuantizer.fit(x, m, k, iters, vq.Distance.Euclidean, 13, init_idx=init, draw=sg.draw, accumulate=vq.ACCUM_FAST)
    assert np.array_equal(pq.iterations, it_o)
    assert np.array_equal(pq.codebooks, cb_o)
    assert by_stream(so.draws) == by_stream(sg.draws)
