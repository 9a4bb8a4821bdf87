"""CPU oracle for the quantizer hot path -- TEST INFRASTRUCTURE ONLY.

ctypes front end to ``libvq_oracle.so`` (built from ``vq_oracle.c`` by the
Makefile beside it).  Only the test-suite, the smoke check and the CPU-baseline
leg of the benchmark may import this package; the product package never does.

Parity status: arithmetic is pinned against the reference's own known-answer
tests; which rows the seeded RNG draws and the OPQ rotation are PARITY UNPINNED
(third-party crates whose sources are not available), so row indices are
inputs everywhere and the rotation is compared with a tolerance.
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB_PATH = os.path.join(_HERE, "libvq_oracle.so")

SQUARED_EUCLIDEAN, EUCLIDEAN, COSINE, MANHATTAN, CHEBYSHEV, MINKOWSKI, HAMMING = range(7)

DRAW_FN = C.CFUNCTYPE(C.c_uint64, C.c_void_p, C.c_size_t, C.c_uint64)
INIT_FN = C.CFUNCTYPE(None, C.c_void_p, C.c_size_t, C.c_uint64, C.c_size_t, C.POINTER(C.c_uint64))


class OracleError(Exception):
    def __init__(self, code: int, message: str):
        super().__init__(message)
        self.code = code


def build(force: bool = False) -> str:
    """Compile the oracle if the shared object is missing or older than its source."""
    src = os.path.join(_HERE, "vq_oracle.c")
    if force or not os.path.exists(_LIB_PATH) or os.path.getmtime(_LIB_PATH) < os.path.getmtime(src):
        subprocess.check_call(["make", "-C", _HERE, "-s"])
    return _LIB_PATH


_lib = None


def lib():
    global _lib
    if _lib is None:
        if not os.path.exists(_LIB_PATH):
            build()
        L = C.CDLL(_LIB_PATH)
        L.vqo_last_error.restype = C.c_char_p
        L.vqo_f32_to_f16.restype = C.c_uint16
        L.vqo_f32_to_f16.argtypes = [C.c_float]
        L.vqo_distance2.restype = C.c_float
        L.vqo_distance2.argtypes = [C.c_void_p, C.c_void_p, C.c_size_t]
        L.vqo_distance.argtypes = [C.c_int, C.c_double, C.c_void_p, C.c_size_t, C.c_void_p, C.c_size_t,
                                   C.POINTER(C.c_float)]
        L.vqo_mean_rows.argtypes = [C.c_void_p, C.c_size_t, C.c_size_t, C.c_size_t, C.c_void_p]
        L.vqo_lbg.argtypes = [C.c_void_p, C.c_size_t, C.c_size_t, C.c_size_t, C.c_size_t, C.c_size_t,
                              C.c_size_t, C.c_void_p, DRAW_FN, C.c_void_p, C.c_size_t, C.c_void_p,
                              C.c_void_p, C.POINTER(C.c_size_t)]
        L.vqo_pq_fit.argtypes = [C.c_void_p, C.c_size_t, C.c_size_t, C.c_size_t, C.c_size_t, C.c_size_t,
                                 C.c_void_p, DRAW_FN, C.c_void_p, C.c_void_p, C.c_void_p]
        L.vqo_pq_quantize.argtypes = [C.c_void_p, C.c_size_t, C.c_size_t, C.c_size_t, C.c_int, C.c_double,
                                      C.c_void_p, C.c_size_t, C.c_void_p, C.c_void_p, C.c_void_p]
        L.vqo_rvq_fit.argtypes = [C.c_void_p, C.c_size_t, C.c_size_t, C.c_size_t, C.c_size_t, C.c_size_t,
                                  C.c_float, C.c_int, C.c_double, INIT_FN, DRAW_FN, C.c_void_p, C.c_void_p,
                                  C.POINTER(C.c_size_t), C.c_void_p]
        L.vqo_rvq_quantize.argtypes = [C.c_void_p, C.c_size_t, C.c_size_t, C.c_size_t, C.c_float, C.c_int,
                                       C.c_double, C.c_void_p, C.c_size_t, C.c_void_p, C.c_void_p, C.c_void_p]
        L.vqo_rotate_rows.restype = None
        L.vqo_rotate_rows.argtypes = [C.c_void_p, C.c_size_t, C.c_void_p, C.c_size_t, C.c_void_p]
        L.vqo_cross_cov.restype = None
        L.vqo_cross_cov.argtypes = [C.c_void_p, C.c_void_p, C.c_size_t, C.c_size_t, C.c_void_p]
        L.vqo_sq_fit.argtypes = [C.c_float, C.c_float, C.c_size_t, C.POINTER(C.c_float)]
        L.vqo_sq_quantize.restype = None
        L.vqo_sq_quantize.argtypes = [C.c_float, C.c_float, C.c_size_t, C.c_float, C.c_void_p, C.c_size_t,
                                      C.c_void_p]
        L.vqo_bq_fit.argtypes = [C.c_uint8, C.c_uint8]
        L.vqo_bq_quantize.restype = None
        L.vqo_bq_quantize.argtypes = [C.c_float, C.c_uint8, C.c_uint8, C.c_void_p, C.c_size_t, C.c_void_p]
        L.vqo_mse_f16.restype = C.c_double
        L.vqo_mse_f16.argtypes = [C.c_void_p, C.c_void_p, C.c_size_t, C.c_size_t]
        L.vqo_tsvq_fit.argtypes = [C.c_void_p, C.c_size_t, C.c_size_t, C.c_size_t, C.c_size_t, C.c_void_p, C.c_void_p,
                                   C.c_void_p, C.POINTER(C.c_size_t)]
        L.vqo_tsvq_quantize.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p, C.c_size_t, C.c_int, C.c_double, C.c_void_p,
                                        C.c_size_t, C.c_void_p, C.c_void_p]
        L.vqo_num_threads.restype = C.c_int
        L.vqo_set_num_threads.restype = None
        L.vqo_set_num_threads.argtypes = [C.c_int]
        _lib = L
    return _lib


def _check(rc: int):
    if rc != 0:
        raise OracleError(rc, lib().vqo_last_error().decode())


def _f32(a) -> np.ndarray:
    return np.ascontiguousarray(a, dtype=np.float32)


def _ptr(a: np.ndarray):
    return a.ctypes.data_as(C.c_void_p)


def num_threads() -> int:
    return int(lib().vqo_num_threads())


def use_all_host_threads() -> int:
    """Undo a launcher's OMP_NUM_THREADS=1 (torchrun sets it): one thread per CPU this process may run on."""
    n = len(os.sched_getaffinity(0)) if hasattr(os, "sched_getaffinity") else (os.cpu_count() or 1)
    lib().vqo_set_num_threads(int(n))
    return num_threads()


def f32_to_f16_bits(x) -> np.ndarray:
    x = _f32(x).ravel()
    return np.array([lib().vqo_f32_to_f16(float(v)) for v in x], dtype=np.uint16)


def distance2(a, b) -> float:
    a, b = _f32(a), _f32(b)
    if a.size != b.size:
        raise OracleError(3, f"Dimension mismatch: expected {a.size}, got {b.size}")
    return float(lib().vqo_distance2(_ptr(a), _ptr(b), a.size))


def distance(metric: int, a, b, p: float = 0.0) -> float:
    a, b = _f32(a), _f32(b)
    out = C.c_float()
    _check(lib().vqo_distance(metric, p, _ptr(a), a.size, _ptr(b), b.size, C.byref(out)))
    return float(out.value)


def mean_vector(rows) -> np.ndarray:
    rows = _f32(rows)
    if rows.ndim != 2 or rows.shape[0] == 0:
        raise OracleError(1, "Empty input: at least one vector is required.")
    out = np.empty(rows.shape[1], np.float32)
    _check(lib().vqo_mean_rows(_ptr(rows), rows.shape[0], rows.shape[1], rows.shape[1], _ptr(out)))
    return out


def _draw_cb(draw):
    """Wrap ``draw(stream, n) -> int`` into the C callback (kept alive by the caller)."""
    if draw is None:
        return DRAW_FN(lambda user, stream, n: 0)
    return DRAW_FN(lambda user, stream, n: int(draw(int(stream), int(n))))


def lbg(data, k: int, max_iters: int, init_idx, draw=None, stream: int = 0, col0: int = 0, d=None):
    """src/utils.rs:32-109.  Returns (centroids k x d, assignments n, iterations)."""
    data = _f32(data)
    if data.ndim != 2:
        raise ValueError("data must be 2-D")
    n, ld = data.shape
    d = ld - col0 if d is None else d
    idx = np.ascontiguousarray(init_idx, dtype=np.uint64)
    cent = np.empty((k, d), np.float32)
    assign = np.empty(n, np.uint32)
    iters = C.c_size_t(0)
    cb = _draw_cb(draw)
    _check(lib().vqo_lbg(_ptr(data), n, ld, col0, d, k, max_iters, _ptr(idx), cb, None, stream,
                         _ptr(cent), _ptr(assign), C.byref(iters)))
    return cent, assign, int(iters.value)


def pq_fit(data, m: int, k: int, max_iters: int, init_idx, draw=None):
    """src/pq.rs:79-129.  init_idx is m x k.  Returns (codebooks m x k x sub_dim, iterations per subspace)."""
    data = _f32(data)
    if data.ndim != 2 or data.shape[0] == 0:
        raise OracleError(1, "Empty input: at least one vector is required.")
    n, dim = data.shape
    idx = np.ascontiguousarray(init_idx, dtype=np.uint64)
    sd = dim // m if m and dim % m == 0 else 1
    cb = np.zeros((max(m, 1), k, sd), np.float32)
    iters = np.zeros(max(m, 1), dtype=np.uintp)
    fn = _draw_cb(draw)
    _check(lib().vqo_pq_fit(_ptr(data), n, dim, m, k, max_iters, _ptr(idx), fn, None, _ptr(cb), _ptr(iters)))
    return cb, iters


def pq_fit_faithful(data, m: int, k: int, max_iters: int, init_idx, draw=None):
    """vqo_pq_fit with the reference's memory behaviour (a heap allocation per row and per distance2, an O(n k) gather with
    cloned members): same codebooks, much slower; exists only to be timed as the "faithful" CPU baseline."""
    data = _f32(data)
    n, dim = data.shape
    idx = np.ascontiguousarray(init_idx, dtype=np.uint64)
    cb = np.zeros((m, k, dim // m), np.float32)
    L = lib()
    L.vqo_pq_fit_faithful.restype = C.c_int
    L.vqo_pq_fit_faithful.argtypes = [C.c_void_p, C.c_size_t, C.c_size_t, C.c_size_t, C.c_size_t, C.c_size_t, C.c_void_p, DRAW_FN,
                                      C.c_void_p, C.c_void_p]
    fn = _draw_cb(draw)
    _check(L.vqo_pq_fit_faithful(_ptr(data), n, dim, m, k, max_iters, _ptr(idx), fn, None, _ptr(cb)))
    return cb


def pq_quantize(codebooks, x, metric: int = EUCLIDEAN, p: float = 0.0):
    """src/pq.rs:146-187 per row.  Returns (f16 bits n x dim, codes n x m)."""
    cb = _f32(codebooks)
    m, k, sd = cb.shape
    x = _f32(x)
    n = x.shape[0]
    out = np.empty((n, m * sd), np.uint16)
    codes = np.empty((n, m), np.uint32)
    _check(lib().vqo_pq_quantize(_ptr(cb), m, k, sd, metric, p, _ptr(x), n, _ptr(out), _ptr(codes), None))
    return out, codes


def pq_reconstruct_f32(codebooks, x, metric: int = EUCLIDEAN, p: float = 0.0) -> np.ndarray:
    """f32 reconstruction used inside OPQ training (src/opq.rs:146-168)."""
    cb = _f32(codebooks)
    m, k, sd = cb.shape
    x = _f32(x)
    n = x.shape[0]
    rec = np.empty((n, m * sd), np.float32)
    _check(lib().vqo_pq_quantize(_ptr(cb), m, k, sd, metric, p, _ptr(x), n, None, None, _ptr(rec)))
    return rec


def rvq_fit(data, stages: int, k: int, max_iters: int, epsilon: float, metric: int, init, draw=None,
            p: float = 0.0):
    """src/rvq.rs:87-154.  ``init(stage, n, k) -> k indices``.  Returns (codebooks, residuals, avg norms)."""
    data = _f32(data)
    if data.ndim != 2 or data.shape[0] == 0:
        raise OracleError(1, "Empty input: at least one vector is required.")
    n, dim = data.shape
    res = data.copy()
    cb = np.zeros((max(stages, 1), max(k, 1), dim), np.float32)
    norms = np.zeros(max(stages, 1), np.float32)
    done = C.c_size_t(0)

    def _init(user, stage, n_, k_, out):
        idx = np.asarray(init(int(stage), int(n_), int(k_)), dtype=np.uint64)
        for j in range(int(k_)):
            out[j] = int(idx[j])

    icb = INIT_FN(_init)
    dcb = _draw_cb(draw)
    _check(lib().vqo_rvq_fit(_ptr(res), n, dim, stages, k, max_iters, epsilon, metric, p, icb, dcb, None,
                             _ptr(cb), C.byref(done), _ptr(norms)))
    s = int(done.value)
    return cb[:s].copy(), res, norms[:s].copy()


def rvq_quantize(codebooks, epsilon: float, x, metric: int = EUCLIDEAN, p: float = 0.0):
    """src/rvq.rs:171-215 per row.  Returns (f16 bits, codes n x stages, f32 sums)."""
    cb = _f32(codebooks)
    x = _f32(x)
    n, dim = x.shape
    if cb.size == 0:
        return np.zeros((n, dim), np.uint16), np.zeros((n, 0), np.uint32), np.zeros((n, dim), np.float32)
    stages, k, _ = cb.shape
    out = np.empty((n, dim), np.uint16)
    codes = np.empty((n, stages), np.uint32)
    sums = np.empty((n, dim), np.float32)
    _check(lib().vqo_rvq_quantize(_ptr(cb), stages, k, dim, epsilon, metric, p, _ptr(x), n, _ptr(out),
                                  _ptr(codes), _ptr(sums)))
    return out, codes, sums


def rotate_rows(rot, x) -> np.ndarray:
    rot, x = _f32(rot), _f32(x)
    y = np.empty_like(x)
    lib().vqo_rotate_rows(_ptr(rot), rot.shape[0], _ptr(x), x.shape[0], _ptr(y))
    return y


def cross_cov(y, x) -> np.ndarray:
    y, x = _f32(y), _f32(x)
    a = np.empty((x.shape[1], x.shape[1]), np.float64)
    lib().vqo_cross_cov(_ptr(y), _ptr(x), x.shape[0], x.shape[1], _ptr(a))
    return a


def opq_fit(data, m: int, k: int, max_iters: int, opq_iters: int, metric: int, init_idx, draw=None,
            p: float = 0.0):
    """src/opq.rs:90-205.  Returns (rotation dim x dim, codebooks m x k x sub_dim).

    The SVD (opq.rs:180-183) is numpy's; ``rotation = V * U^T`` exactly as the
    reference writes it.  ``draw(stream, n)`` is called with a fresh per-subspace
    stream every outer iteration because the reference re-seeds with ``seed + i``
    each time (opq.rs:140); callers that need that behaviour pass a factory via
    ``draw.reset()`` if the object has one.
    """
    data = _f32(data)
    if data.ndim != 2 or data.shape[0] == 0:
        raise OracleError(1, "Empty input: at least one vector is required.")
    n, dim = data.shape
    if dim < m:
        raise OracleError(2, "Invalid parameter: Dimension must be at least m")
    if dim % m != 0:
        raise OracleError(2, "Invalid parameter: Dimension must be divisible by m")
    rot = np.eye(dim, dtype=np.float32)
    rotated = data.copy()
    cb = np.zeros((0, k, dim // m), np.float32)
    for _ in range(opq_iters):
        if draw is not None and hasattr(draw, "reset"):
            draw.reset()
        cb, _it = pq_fit(rotated, m, k, max_iters, init_idx, draw)
        rec = pq_reconstruct_f32(cb, rotated, metric, p)
        a = cross_cov(rec, rotated)
        u, _s, vt = np.linalg.svd(a)
        rot = (vt.T @ u.T).astype(np.float32)
        rotated = rotate_rows(rot, data)
    return rot, cb


def opq_quantize(rot, codebooks, x, metric: int = EUCLIDEAN, p: float = 0.0):
    """src/opq.rs:222-264 per row."""
    cb = _f32(codebooks)
    x = _f32(x)
    if cb.shape[0] == 0:
        return np.zeros((x.shape[0], 0), np.uint16), np.zeros((x.shape[0], 0), np.uint32)
    y = rotate_rows(rot, x)
    return pq_quantize(cb, y, metric, p)


def sq_fit(vmin: float, vmax: float, levels: int) -> float:
    step = C.c_float()
    _check(lib().vqo_sq_fit(vmin, vmax, levels, C.byref(step)))
    return float(step.value)


def sq_quantize(vmin: float, vmax: float, levels: int, step: float, x) -> np.ndarray:
    x = _f32(x)
    out = np.empty(x.shape, np.uint8)
    lib().vqo_sq_quantize(vmin, vmax, levels, step, _ptr(x), x.size, _ptr(out))
    return out


def bq_fit(low: int, high: int) -> None:
    _check(lib().vqo_bq_fit(low, high))


def bq_quantize(threshold: float, low: int, high: int, x) -> np.ndarray:
    x = _f32(x)
    out = np.empty(x.shape, np.uint8)
    lib().vqo_bq_quantize(threshold, low, high, _ptr(x), x.size, _ptr(out))
    return out


def tsvq_fit(x, max_depth: int):
    """TSVQ::new / TSVQNode::fit (src/tsvq.rs:71-148,205-211).  Returns (centroids nodes x dim, left, right), nodes numbered
    breadth-first, -1 = no child."""
    x = _f32(x)
    n, dim = x.shape if x.ndim == 2 else (0, 0)
    cap = max(1, min(2 ** (max_depth + 1) - 1 if max_depth < 40 else 2 * n, 2 * max(n, 1)))
    cent = np.zeros((cap, max(dim, 1)), np.float32)
    left = np.full(cap, -1, np.int32)
    right = np.full(cap, -1, np.int32)
    nn = C.c_size_t(0)
    _check(lib().vqo_tsvq_fit(_ptr(x), n, dim, max_depth, cap, _ptr(cent), _ptr(left), _ptr(right), C.byref(nn)))
    k = int(nn.value)
    return cent[:k, :dim].copy(), left[:k].copy(), right[:k].copy()


def tsvq_quantize(centroids, left, right, x, metric: int = EUCLIDEAN, p: float = 0.0):
    """TSVQ::quantize (src/tsvq.rs:231-249).  Returns (f16 bits n x dim, leaf node per row)."""
    cent, x = _f32(centroids), _f32(x)
    left = np.ascontiguousarray(left, np.int32)
    right = np.ascontiguousarray(right, np.int32)
    n, dim = x.shape
    out = np.empty((n, dim), np.uint16)
    leaf = np.empty(n, np.uint32)
    _check(lib().vqo_tsvq_quantize(_ptr(cent), _ptr(left), _ptr(right), dim, metric, p, _ptr(x), n, _ptr(out), _ptr(leaf)))
    return out, leaf


def recall_at_k(original, approx, k: int = 10) -> float:
    """calculate_recall, src/bin/utils.rs:70-127 (approx = the f16 reconstruction converted back to f32)."""
    original, approx = _f32(original), _f32(approx)
    n = original.shape[0]
    eval_samples = min(n, 1000)
    step = n // eval_samples if n // eval_samples > 0 else 1
    total = np.float32(0.0)

    def knn(data, i, start, end):
        rows, q = data[start:end], data[i]
        acc = np.zeros(end - start, np.float32)
        for t in range(data.shape[1]):  # serial f32 fold over the dimensions, as Vector::distance2 does
            diff = q[t] - rows[:, t]
            acc = acc + diff * diff
        d = np.sqrt(acc)
        order = [start + t for t in np.argsort(d, kind="stable") if start + t != i]
        return order[:k]

    for i in range(0, n, step):
        window = 5000 if n > 10_000 else n
        start = i - window // 2 if i > window // 2 else 0
        end = min(i + window // 2, n)
        true_nn = knn(original, i, start, end)
        approx_nn = set(knn(approx, i, start, end))
        total = np.float32(total + np.float32(sum(1 for j in true_nn if j in approx_nn)) / np.float32(k))
    return float(total / np.float32(n // step))


def mse_f16(x, q_bits) -> float:
    """src/bin/utils.rs:50-67 (f64 accumulation)."""
    x = _f32(x)
    q = np.ascontiguousarray(q_bits, dtype=np.uint16)
    return float(lib().vqo_mse_f16(_ptr(x), _ptr(q), x.shape[0], x.shape[1]))
