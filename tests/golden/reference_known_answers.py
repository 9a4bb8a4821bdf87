"""Known answers held by the reference's own tests, transcribed as data.

Each entry names the reference test it comes from (file:line inside the
reference tree).  Both the CPU oracle (tests/test_oracle_known_answers.py) and
the CUDA library (tests/test_gpu_known_answers.py) are checked against them.
PARALLEL_THRESHOLD is 1024 (src/vector.rs:16).
"""
import numpy as np

PARALLEL_THRESHOLD = 1024
_LEN = PARALLEL_THRESHOLD + 10
_I = np.arange(_LEN, dtype=np.float32)

SQ, EUCLID, COSINE, MANHATTAN, CHEBYSHEV, MINKOWSKI, HAMMING = range(7)

_cheb_a = _I.copy()
_cheb_b = _I.copy()
_cheb_a[-1] = 1000.0
_cheb_b[-1] = 0.0

# (source, metric, p, a, b, expected, tolerance)
DISTANCE_CASES = [
    ("tests/test_distances.rs:16-23", SQ, 0.0, [1, 2, 3], [4, 6, 8], 50.0, 1e-6),
    ("tests/test_distances.rs:26-34", SQ, 0.0, _I, _I + 1, float(_LEN), 1e-6),
    ("tests/test_distances.rs:40-48", EUCLID, 0.0, [1, 2, 3], [4, 6, 8], float(np.sqrt(np.float32(50.0))), 1e-6),
    ("tests/test_distances.rs:51-60", EUCLID, 0.0, _I, _I + 1, float(np.sqrt(np.float32(_LEN))), 1e-6),
    ("tests/test_distances.rs:66-73", COSINE, 0.0, [1, 0], [0, 1], 1.0, 1e-6),
    ("tests/test_distances.rs:75-78", COSINE, 0.0, [1, 1], [1, 1], 0.0, 1e-6),
    ("tests/test_distances.rs:82-90", COSINE, 0.0, np.ones(_LEN), np.ones(_LEN), 0.0, 1e-6),
    ("tests/test_distances.rs:96-103", MANHATTAN, 0.0, [1, 2, 3], [4, 6, 8], 12.0, 1e-6),
    ("tests/test_distances.rs:106-115", MANHATTAN, 0.0, _I, _I + 2, 2.0 * _LEN, 1e-6),
    ("tests/test_distances.rs:121-128", CHEBYSHEV, 0.0, [1, 5, 3], [4, 2, 9], 6.0, 1e-6),
    ("tests/test_distances.rs:131-142", CHEBYSHEV, 0.0, _cheb_a, _cheb_b, 1000.0, 1e-6),
    ("tests/test_distances.rs:148-156", MINKOWSKI, 3.0, [1, 2, 3], [4, 6, 8], 6.0, 1e-6),
    # the reference's own tolerance here is 1e-6 on a powf result; libm differences allow a few ulp
    ("tests/test_distances.rs:159-169", MINKOWSKI, 3.0, _I, _I + 1, float(np.float32(_LEN) ** np.float32(1.0 / 3.0)), 1e-5),
    ("tests/test_distances.rs:175-182", HAMMING, 0.0, [1, 2, 3, 4], [1, 0, 3, 0], 2.0, 1e-6),
    ("tests/test_distances.rs:185-201", HAMMING, 0.0, np.ones(_LEN), (np.arange(_LEN) % 2 == 0).astype(np.float32),
     float(_LEN // 2), 1e-6),
]

# tests/test_distances.rs:206-213 -- mismatched lengths panic with "Dimension mismatch"
DISTANCE_MISMATCH = ("tests/test_distances.rs:206-213", EUCLID, [1.0, 2.0], [1.0], "Dimension mismatch")

# tests/test_vector.rs:67-75
DISTANCE2_CASE = ("tests/test_vector.rs:67-75", [1, 2, 3], [4, 5, 6], 27.0, 1e-6)
# tests/test_vector.rs:77-89 and 91-105
MEAN_CASES = [
    ("tests/test_vector.rs:77-89", np.array([[1, 2, 3], [4, 5, 6], [7, 8, 9]], np.float32), [4, 5, 6], 1e-6),
    ("tests/test_vector.rs:91-105", np.tile(np.arange(5, dtype=np.float32), (_LEN, 1)), [0, 1, 2, 3, 4], 1e-6),
]
# src/utils.rs:147-153 -- one point, k = 1: the centroid is the point
LBG_SINGLE_POINT = ("src/utils.rs:147-153", np.array([[1.0, 2.0]], np.float32), 1, 10, [[1.0, 2.0]])
# src/utils.rs:133-145 -- panic substrings, k checked before n
LBG_PANICS = [
    ("src/utils.rs:133-138", np.array([[1.0, 2.0], [2.0, 3.0]], np.float32), 0, "k must be greater than 0"),
    ("src/utils.rs:140-145", np.array([[1.0, 2.0]], np.float32), 2, "Not enough data points for k clusters"),
]
# src/utils.rs:113-131,155-160 -- four 2-d points, k = 2: two centroids come back
LBG_BASIC = np.array([[1, 2], [2, 3], [3, 4], [4, 5]], np.float32)
# src/bq.rs:16-19 doc-test: fit(0.0, 0, 1) on [-1.0, 0.0, 1.0] -> [0, 1, 1]
BQ_DOC = ("src/bq.rs:12-20", 0.0, 0, 1, [-1.0, 0.0, 1.0], [0, 1, 1])
# tests/test_sq.rs:9-33 -- fit(-1, 1, 5): reconstruction error <= step/2 + 1e-6 after clamping
SQ_SCALARS = ("tests/test_sq.rs:9-33", -1.0, 1.0, 5, [-1.2, -1.0, -0.8, -0.3, 0.0, 0.3, 0.6, 1.0, 1.2])
# tests/test_sq.rs:36-77 -- fit(-1000, 1000, 256) on 100 x 1024 values in [-1000, 1000): same bound
SQ_LARGE = ("tests/test_sq.rs:36-77", -1000.0, 1000.0, 256, (100, 1024))
# tests/test_bq.rs:9-32 -- fit(0.0, 0, 1) on 1024 values in [-1000, 1000): out == (x >= 0)
BQ_LARGE = ("tests/test_bq.rs:9-32", 0.0, 0, 1, 1024)
# f16 conversion of exactly representable values round-trips (tests/test_tsvq.rs:11-22, tests/test_vector.rs:185-202)
F16_EXACT = [0.0, 1.0, 2.0, 3.0, 4.0, 5.0, 6.0, -1.5, 0.5, 0.25, 1024.0, 65504.0]
# error texts (src/exceptions.rs:11-24 with the detail strings of each call site)
ERROR_TEXTS = {
    "pq_empty": "Empty input: at least one vector is required.",                       # src/pq.rs:87-89
    "pq_dim_lt_m": "Invalid parameter: Data dimension must be at least m",             # src/pq.rs:91-96
    "pq_dim_mod_m": "Invalid parameter: Data dimension must be divisible by m",        # src/pq.rs:97-102
    "opq_dim_lt_m": "Invalid parameter: Dimension must be at least m",                 # src/opq.rs:103-108
    "opq_dim_mod_m": "Invalid parameter: Dimension must be divisible by m",            # src/opq.rs:109-114
    "sq_max_le_min": "Invalid parameter: max must be greater than min",                # src/sq.rs:51-56
    "sq_levels_lt_2": "Invalid parameter: levels must be at least 2",                  # src/sq.rs:57-62
    "sq_levels_gt_256": "Invalid parameter: levels must be no more than 256",          # src/sq.rs:63-68
    "bq_low_ge_high": "Invalid parameter: Low quantization level must be less than high quantization level",  # src/bq.rs:47-54
    "minkowski_p": "Invalid metric parameter for Minkowski: p must be positive",       # src/distances.rs:155-163
    "k_zero": "Invalid parameter: k must be greater than 0",                           # src/utils.rs:39-44
    "n_lt_k": "Invalid parameter: Not enough data points for k clusters",              # src/utils.rs:45-50
}
