"""The CPU oracle against every known answer the reference's own tests hold for the hot path."""
import numpy as np
import pytest

from tests.golden import reference_known_answers as ka


@pytest.mark.parametrize("case", ka.DISTANCE_CASES, ids=[c[0] for c in ka.DISTANCE_CASES])
def test_distance_known_answers(oracle, case):
    _src, metric, p, a, b, expected, tol = case
    got = oracle.distance(metric, np.asarray(a, np.float32), np.asarray(b, np.float32), p)
    assert abs(got - expected) < tol


def test_distance_mismatch(oracle):
    _src, metric, a, b, text = ka.DISTANCE_MISMATCH
    with pytest.raises(oracle.OracleError, match=text) as e:
        oracle.distance(metric, a, b)
    assert str(e.value) == "Dimension mismatch: expected 2, got 1"


def test_minkowski_p_must_be_positive(oracle):
    with pytest.raises(oracle.OracleError) as e:
        oracle.distance(ka.MINKOWSKI, [1, 2], [3, 4], 0.0)
    assert str(e.value) == ka.ERROR_TEXTS["minkowski_p"]


def test_distance2(oracle):
    _src, a, b, expected, tol = ka.DISTANCE2_CASE
    assert abs(oracle.distance2(a, b) - expected) < tol


@pytest.mark.parametrize("case", ka.MEAN_CASES, ids=[c[0] for c in ka.MEAN_CASES])
def test_mean_vector(oracle, case):
    _src, rows, expected, tol = case
    assert np.all(np.abs(oracle.mean_vector(rows) - np.asarray(expected, np.float32)) < tol)


def test_cosine_zero_norm_is_one(oracle):
    # src/distances.rs:146-147
    assert oracle.distance(ka.COSINE, [0, 0, 0], [1, 2, 3]) == 1.0
    assert oracle.distance(ka.COSINE, [1, 2, 3], [0, 0, 0]) == 1.0


def test_lbg_single_point(oracle):
    _src, data, k, iters, expected = ka.LBG_SINGLE_POINT
    cent, assign, _ = oracle.lbg(data, k, iters, [0])
    assert np.array_equal(cent, np.asarray(expected, np.float32))
    assert assign.tolist() == [0]


@pytest.mark.parametrize("case", ka.LBG_PANICS, ids=[c[0] for c in ka.LBG_PANICS])
def test_lbg_panics(oracle, case):
    _src, data, k, text = case
    with pytest.raises(oracle.OracleError, match=text):
        oracle.lbg(data, k, 10, np.zeros(max(k, 1), np.uint64))


def test_lbg_k_checked_before_n(oracle):
    # k == 0 and n == 0 together: the k check comes first (src/utils.rs:39-50)
    with pytest.raises(oracle.OracleError, match="k must be greater than 0"):
        oracle.lbg(np.zeros((0, 2), np.float32), 0, 10, [0])


@pytest.mark.parametrize("iters", [10, 100])
def test_lbg_basic(oracle, iters):
    cent, assign, _ = oracle.lbg(ka.LBG_BASIC, 2, iters, [0, 3])
    assert cent.shape == (2, 2)
    # two clusters on a line: {p0,p1} and {p2,p3}
    assert np.allclose(cent, [[1.5, 2.5], [3.5, 4.5]])
    assert assign.tolist() == [0, 0, 1, 1]


def test_lbg_identical_rows_stops_after_one_iteration(oracle):
    # benches/utils.rs:14-21: 100 identical vectors; iteration 1 assigns everything to centroid 0, which equals
    # the initial all-zero assignment, so the loop ends after one update with k-1 clusters re-seeded.
    data = np.tile(np.arange(64, dtype=np.float32), (100, 1))
    draws = []

    def draw(stream, n):
        draws.append((stream, n))
        return 7

    cent, assign, iters = oracle.lbg(data, 8, 10, np.arange(8), draw=draw)
    assert iters == 1
    assert len(draws) == 7 and all(d == (0, 100) for d in draws)
    assert np.array_equal(cent, np.tile(data[0], (8, 1)))
    assert not assign.any()


def test_lbg_max_iters_zero_returns_initial_sample(oracle):
    data = np.arange(20, dtype=np.float32).reshape(10, 2)
    cent, _, iters = oracle.lbg(data, 3, 0, [4, 1, 9])
    assert iters == 0 and np.array_equal(cent, data[[4, 1, 9]])


def test_bq_doc_example(oracle):
    _src, thr, low, high, x, expected = ka.BQ_DOC
    assert oracle.bq_quantize(thr, low, high, np.asarray(x, np.float32)).tolist() == expected


def test_bq_large(oracle):
    _src, thr, low, high, dim = ka.BQ_LARGE
    x = np.random.default_rng(42).uniform(-1000, 1000, dim).astype(np.float32)
    assert np.array_equal(oracle.bq_quantize(thr, low, high, x), (x >= 0).astype(np.uint8))


def test_bq_nan_is_low(oracle):
    assert oracle.bq_quantize(0.0, 3, 9, np.array([np.nan, np.inf, -np.inf, -0.0], np.float32)).tolist() == [3, 9, 3, 9]


def _sq_bound(oracle, vmin, vmax, levels, x):
    # The reference asserts error <= step/2 + 1e-6 on its own seeded data; for arbitrary data the f32 rounding of
    # `min + i*step` near |x| ~ 1000 (ulp 6e-5) can exceed 1e-6, so the slack here is two ulps of the range end.
    step = oracle.sq_fit(vmin, vmax, levels)
    idx = oracle.sq_quantize(vmin, vmax, levels, step, x)
    recon = np.float32(vmin) + idx.astype(np.float32) * np.float32(step)
    clamped = np.clip(x, np.float32(vmin), np.float32(vmax))
    slack = max(1e-6, 2 * float(np.spacing(np.float32(max(abs(vmin), abs(vmax))))))
    assert np.all(np.abs(recon - clamped) <= np.float32(step) / 2 + slack)
    return idx


def test_sq_scalars(oracle):
    _src, vmin, vmax, levels, values = ka.SQ_SCALARS
    idx = _sq_bound(oracle, vmin, vmax, levels, np.asarray(values, np.float32))
    assert idx.tolist() == [0, 0, 0, 1, 2, 3, 3, 4, 4]


def test_sq_large(oracle):
    _src, vmin, vmax, levels, shape = ka.SQ_LARGE
    x = np.random.default_rng(42).uniform(-1000, 1000, shape).astype(np.float32)
    _sq_bound(oracle, vmin, vmax, levels, x)


def test_sq_specials(oracle):
    # NaN passes the clamp and `as usize` turns it into 0; infinities clamp to the range ends (src/sq.rs:117-127)
    step = oracle.sq_fit(0.0, 1.0, 256)
    x = np.array([np.nan, np.inf, -np.inf, 0.501, 1.0, 0.0], np.float32)
    assert oracle.sq_quantize(0.0, 1.0, 256, step, x).tolist() == [0, 255, 0, 128, 255, 0]


def test_sq_round_half_away_from_zero(oracle):
    # f32::round: 0.5 -> 1, 1.5 -> 2, 2.5 -> 3 (numpy's rint would give 0, 2, 2)
    step = oracle.sq_fit(0.0, 4.0, 5)
    assert step == 1.0
    assert oracle.sq_quantize(0.0, 4.0, 5, step, np.array([0.5, 1.5, 2.5, 3.5], np.float32)).tolist() == [1, 2, 3, 4]


@pytest.mark.parametrize("args,key", [((1.0, 1.0, 4), "sq_max_le_min"), ((0.0, 1.0, 1), "sq_levels_lt_2"),
                                      ((0.0, 1.0, 257), "sq_levels_gt_256")])
def test_sq_fit_errors(oracle, args, key):
    with pytest.raises(oracle.OracleError) as e:
        oracle.sq_fit(*args)
    assert str(e.value) == ka.ERROR_TEXTS[key]


def test_bq_fit_error(oracle):
    with pytest.raises(oracle.OracleError) as e:
        oracle.bq_fit(1, 1)
    assert str(e.value) == ka.ERROR_TEXTS["bq_low_ge_high"]


def test_f16_exact_values_and_numpy_agreement(oracle):
    exact = np.asarray(ka.F16_EXACT, np.float32)
    assert np.array_equal(oracle.f32_to_f16_bits(exact).view(np.float16).astype(np.float32), exact)
    rng = np.random.default_rng(0)
    bits = rng.integers(0, 2 ** 32, 20000, dtype=np.uint64).astype(np.uint32)
    vals = np.concatenate([bits.view(np.float32), rng.uniform(-70000, 70000, 5000).astype(np.float32),
                           (rng.uniform(-1, 1, 5000) * 1e-6).astype(np.float32),
                           np.array([65504.0, 65519.99, 65520.0, 5.96e-8, 2.98e-8, 2.9802322e-8, 6.1e-5], np.float32)])
    vals = vals[~np.isnan(vals)]
    with np.errstate(over="ignore"):
        want = vals.astype(np.float16).view(np.uint16)
    assert np.array_equal(oracle.f32_to_f16_bits(vals), want)


def test_pq_validation_order_and_texts(oracle):
    with pytest.raises(oracle.OracleError) as e:
        oracle.pq_fit(np.zeros((0, 4), np.float32), 2, 2, 5, np.zeros((2, 2)))
    assert str(e.value) == ka.ERROR_TEXTS["pq_empty"]
    x = np.zeros((10, 3), np.float32)
    with pytest.raises(oracle.OracleError) as e:
        oracle.pq_fit(x, 4, 2, 5, np.zeros((4, 2)))
    assert str(e.value) == ka.ERROR_TEXTS["pq_dim_lt_m"]
    with pytest.raises(oracle.OracleError) as e:
        oracle.pq_fit(x, 2, 2, 5, np.zeros((2, 2)))
    assert str(e.value) == ka.ERROR_TEXTS["pq_dim_mod_m"]


def test_pq_matches_independent_numpy_restatement(oracle):
    """The C oracle against a direct numpy transcription of src/utils.rs:32-109 + src/pq.rs:146-187 on a small case."""
    rng = np.random.default_rng(5)
    n, dim, m, k = 300, 8, 2, 5
    sd = dim // m
    x = rng.uniform(-1000, 1000, (n, dim)).astype(np.float32)  # tests/utils.rs:8-25 value range
    init = np.stack([rng.choice(n, k, replace=False) for _ in range(m)]).astype(np.uint64)
    cb, iters = oracle.pq_fit(x, m, k, 50, init)

    def dist2(a, c):  # serial f32 fold, separate roundings (src/vector.rs:198-201,214-220)
        acc = np.float32(0)
        for t in range(len(a)):
            d = np.float32(a[t] - c[t])
            acc = np.float32(acc + np.float32(d * d))
        return acc

    for s in range(m):
        sub = x[:, s * sd:(s + 1) * sd]
        cent = sub[init[s].astype(int)].copy()
        assign = np.zeros(n, int)
        done = 0
        for _ in range(50):
            done += 1
            new = np.zeros(n, int)
            for i in range(n):
                best, bd = 0, dist2(sub[i], cent[0])
                for j in range(1, k):
                    d = dist2(sub[i], cent[j])
                    if d < bd:
                        best, bd = j, d
                new[i] = best
            changed = bool(np.any(new != assign))
            assign = new
            for j in range(k):
                members = sub[assign == j]
                assert len(members) > 0  # no empty cluster on this data, so no draw is needed
                acc = np.zeros(sd, np.float32)
                for r in members:
                    acc = (acc + r).astype(np.float32)
                cent[j] = acc / np.float32(len(members))
            if not changed:
                break
        assert done == iters[s]
        assert np.array_equal(cent, cb[s])
    out, codes = oracle.pq_quantize(cb, x[:50], ka.EUCLID)
    for i in range(50):
        for s in range(m):
            d = [np.sqrt(dist2(x[i, s * sd:(s + 1) * sd], cb[s, j])) for j in range(k)]
            best = 0
            for j in range(1, k):
                if d[j] < d[best]:
                    best = j
            assert codes[i, s] == best
            assert np.array_equal(out[i, s * sd:(s + 1) * sd], cb[s, best].astype(np.float16).view(np.uint16))


def test_faithful_timing_variant_gives_the_same_codebooks(oracle):
    """The "faithful" CPU baseline (per-row allocations, an allocation per distance2, O(n k) gather: the reference's memory
    behaviour, src/pq.rs:110-117, src/vector.rs:214-220,259-265, src/utils.rs:83-92) only differs in speed."""
    import numpy as np
    from tests.util import RecordingSeeder
    from vq_b200 import synth
    x = synth.uniform01(900, 12, 4)
    a, b = RecordingSeeder(3), RecordingSeeder(3)
    init = a.init_pq(900, 3, 20)
    b.init_pq(900, 3, 20)
    cb, _ = oracle.pq_fit(x, 3, 20, 7, init, a.draw)
    cbf = oracle.pq_fit_faithful(x, 3, 20, 7, init, b.draw)
    assert np.array_equal(cb, cbf)
