"""ctypes binding of libvqb.so (the C ABI in include/vqb.h).

There is no fallback: if the shared library is missing or cannot be loaded,
importing fails with instructions to build it.
"""
from __future__ import annotations

import ctypes as C
import os

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "libvqb.so")

DRAW_FN = C.CFUNCTYPE(C.c_uint64, C.c_void_p, C.c_size_t, C.c_uint64)
INIT_FN = C.CFUNCTYPE(None, C.c_void_p, C.c_size_t, C.c_uint64, C.c_size_t, C.POINTER(C.c_uint64))
RESTART_FN = C.CFUNCTYPE(None, C.c_void_p)

UNIQUE_ID_BYTES = 128
ACCUM_AUTO, ACCUM_ORDERED, ACCUM_FAST = 0, 1, 2

_P = C.c_void_p
_SZ = C.c_size_t

# name -> (restype, argtypes); every symbol include/vqb.h declares
SIGNATURES = {
    "vqb_version": (C.c_char_p, []),
    "vqb_ctx_create": (C.c_int, [C.c_int, C.POINTER(_P)]),
    "vqb_ctx_destroy": (C.c_int, [_P]),
    "vqb_last_error": (C.c_char_p, [_P]),
    "vqb_ctx_set_stream": (C.c_int, [_P, _P]),
    "vqb_ctx_reset_stream": (C.c_int, [_P]),
    "vqb_ctx_synchronize": (C.c_int, [_P]),
    "vqb_ctx_launch_count": (C.c_int, [_P, C.POINTER(C.c_uint64)]),
    "vqb_ctx_alloc_count": (C.c_int, [_P, C.POINTER(C.c_uint64)]),
    "vqb_ctx_timing": (C.c_int, [_P, C.c_int]),
    "vqb_ctx_timing_report": (C.c_int, [_P, C.c_char_p, _SZ]),
    "vqb_comm_unique_id": (C.c_int, [_P]),
    "vqb_comm_init": (C.c_int, [_P, _P, C.c_int, C.c_int]),
    "vqb_comm_destroy": (C.c_int, [_P]),
    "vqb_comm_exchange_count": (C.c_int, [_P, C.POINTER(C.c_uint64)]),
    "vqb_distance_rows": (C.c_int, [_P, C.c_int, C.c_double, _P, _SZ, _P, _SZ, _SZ, _P]),
    "vqb_tsvq_fit": (C.c_int, [_P, _P, _SZ, _SZ, _SZ, C.c_int, C.c_double, C.POINTER(_P)]),
    "vqb_tsvq_quantize": (C.c_int, [_P, _P, _SZ, _SZ, _P, _P]),
    "vqb_tsvq_shape": (C.c_int, [_P, C.POINTER(_SZ), C.POINTER(_SZ)]),
    "vqb_tsvq_tree": (C.c_int, [_P, _P, _P, _P]),
    "vqb_tsvq_destroy": (C.c_int, [_P]),
    "vqb_evaluate_f16": (C.c_int, [_P, _P, _P, _SZ, _SZ, _SZ, C.POINTER(C.c_float), C.POINTER(C.c_float)]),
    "vqb_pq_tensor_scores": (C.c_int, [_P, _P, _SZ, _SZ, _P, _SZ, _P, _P, _P]),
    "vqb_dense_dots": (C.c_int, [_P, _P, _SZ, _SZ, _P, _SZ, _P, _P]),
    "vqb_opq_rotate_rows": (C.c_int, [_P, _P, _SZ, _P, _SZ, _P]),
    "vqb_opq_cross_cov": (C.c_int, [_P, _P, _P, _SZ, _SZ, _P]),
    "vqb_lbg_fit": (C.c_int, [_P, _P, _SZ, _SZ, _SZ, _SZ, _P, DRAW_FN, _P, C.c_int, _P, C.POINTER(_SZ)]),
    "vqb_pq_fit": (C.c_int, [_P, _P, _SZ, _SZ, _SZ, _SZ, _SZ, C.c_int, C.c_double, _P, DRAW_FN, _P, C.c_int,
                             C.POINTER(_P)]),
    "vqb_pq_from_codebooks": (C.c_int, [_P, _P, _SZ, _SZ, _SZ, C.c_int, C.c_double, C.POINTER(_P)]),
    "vqb_pq_quantize": (C.c_int, [_P, _P, _SZ, _SZ, _P, _P]),
    "vqb_pq_shape": (C.c_int, [_P, C.POINTER(_SZ), C.POINTER(_SZ), C.POINTER(_SZ)]),
    "vqb_pq_codebooks": (C.c_int, [_P, _P]),
    "vqb_pq_iterations": (C.c_int, [_P, _P]),
    "vqb_pq_destroy": (C.c_int, [_P]),
    "vqb_rvq_fit": (C.c_int, [_P, _P, _SZ, _SZ, _SZ, _SZ, _SZ, C.c_float, C.c_int, C.c_double, INIT_FN, DRAW_FN, _P,
                              C.c_int, C.POINTER(_P)]),
    "vqb_rvq_from_codebooks": (C.c_int, [_P, _P, _SZ, _SZ, _SZ, C.c_float, C.c_int, C.c_double, C.POINTER(_P)]),
    "vqb_rvq_quantize": (C.c_int, [_P, _P, _SZ, _SZ, _P, _P]),
    "vqb_rvq_shape": (C.c_int, [_P, C.POINTER(_SZ), C.POINTER(_SZ), C.POINTER(_SZ)]),
    "vqb_rvq_codebooks": (C.c_int, [_P, _P]),
    "vqb_rvq_destroy": (C.c_int, [_P]),
    "vqb_opq_fit": (C.c_int, [_P, _P, _SZ, _SZ, _SZ, _SZ, _SZ, _SZ, C.c_int, C.c_double, _P, DRAW_FN, RESTART_FN, _P,
                              C.c_int, C.POINTER(_P)]),
    "vqb_opq_from_parts": (C.c_int, [_P, _P, _P, _SZ, _SZ, _SZ, C.c_int, C.c_double, C.POINTER(_P)]),
    "vqb_opq_quantize": (C.c_int, [_P, _P, _SZ, _SZ, _P, _P]),
    "vqb_opq_quantize_static": (C.c_int, [_P, _P, _SZ, _SZ, _P, _P]),
    "vqb_opq_shape": (C.c_int, [_P, C.POINTER(_SZ), C.POINTER(_SZ), C.POINTER(_SZ)]),
    "vqb_opq_rotation": (C.c_int, [_P, _P]),
    "vqb_opq_codebooks": (C.c_int, [_P, _P]),
    "vqb_opq_destroy": (C.c_int, [_P]),
    "vqb_sq_fit": (C.c_int, [C.c_float, C.c_float, _SZ, C.POINTER(C.c_float)]),
    "vqb_sq_quantize": (C.c_int, [_P, C.c_float, C.c_float, _SZ, C.c_float, _P, _SZ, _P]),
    "vqb_bq_fit": (C.c_int, [C.c_float, C.c_uint8, C.c_uint8]),
    "vqb_bq_quantize": (C.c_int, [_P, C.c_float, C.c_uint8, C.c_uint8, _P, _SZ, _P]),
}

_lib = None


def load():
    """Load libvqb.so and attach the signatures.  Raises if it is not built."""
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(LIB_PATH):
        raise ImportError(
            f"{LIB_PATH} is missing: build it with `make -C vq_b200/csrc` (or `python -c 'import "
            "__graft_entry__ as g; g.build()'`).  vq_b200 has no fallback path.")
    L = C.CDLL(LIB_PATH)
    for name, (res, args) in SIGNATURES.items():
        fn = getattr(L, name)  # AttributeError here means header and library disagree
        fn.restype = res
        fn.argtypes = args
    _lib = L
    return L
