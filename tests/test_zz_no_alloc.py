"""vqb_opq_quantize_static: the OPQ encode for embedders that cannot let the library allocate device memory
(all HBM already belongs to their own pool, or the CUDA allocator must stay out of their request loop).

Called through the C ABI with device pointers and checked against vqb_opq_quantize on the same inputs, twice in
a row (the static scratch keeps the previous call's rows, so the second call, with fewer and different rows, would
show stale data if the entry point relied on the array's old contents).  This file sorts last on purpose.
"""
import ctypes as C

import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def _quantize(fn, handle, x, dim, m):
    import torch
    n = x.shape[0]
    out = torch.zeros((n, dim), dtype=torch.float16, device="cuda")
    codes = torch.zeros((n, m), dtype=torch.int32, device="cuda")
    rc = fn(handle, C.c_void_p(x.data_ptr()), n, dim, C.c_void_p(out.data_ptr()), C.c_void_p(codes.data_ptr()))
    torch.cuda.synchronize()
    return rc, out, codes


def test_static_scratch_variant_matches_the_allocating_entry_point():
    import torch

    import vq_b200 as vq
    from vq_b200 import _lib

    lib = _lib.load()
    ctx = vq.Context(torch.cuda.current_device())
    ctx.use_stream(torch.cuda.current_stream().cuda_stream)
    rng = np.random.default_rng(17)
    dim, m, k = 64, 8, 32
    q, _ = np.linalg.qr(rng.normal(size=(dim, dim)))
    oq = vq.OptimizedProductQuantizer.from_parts(q.astype(np.float32), rng.normal(size=(m, k, dim // m)).astype(np.float32),
                                                 vq.Distance.Euclidean, ctx=ctx)
    max_floats = 1 << 20
    for n in (5000, 777):  # two calls in a row, the second smaller and on other data
        x = torch.from_numpy(rng.normal(size=(n, dim)).astype(np.float32)).cuda()
        rc_a, out_a, codes_a = _quantize(lib.vqb_opq_quantize, oq._h, x, dim, m)
        rc_s, out_s, codes_s = _quantize(lib.vqb_opq_quantize_static, oq._h, x, dim, m)
        assert rc_a == 0 and rc_s == 0, lib.vqb_last_error(ctx.handle)
        assert torch.equal(codes_s, codes_a)
        assert torch.equal(out_s.view(torch.int16), out_a.view(torch.int16))  # bit-identical, tolerance 0 like the other tests
        assert int(codes_s.max()) < k and float(out_s.float().abs().sum()) > 0

    # beyond the stated maximum: refused with a clear message, nothing written
    n_big = max_floats // dim + 1
    xb = torch.zeros((n_big, dim), device="cuda")
    rc, out_b, _ = _quantize(lib.vqb_opq_quantize_static, oq._h, xb, dim, m)
    assert rc == 103
    msg = lib.vqb_last_error(ctx.handle).decode()
    assert "exceeds the static scratch" in msg and str(max_floats) in msg
    assert not out_b.any()
    # exactly at the maximum is accepted
    xm = torch.from_numpy(rng.normal(size=(max_floats // dim, dim)).astype(np.float32)).cuda()
    rc_a, out_a, codes_a = _quantize(lib.vqb_opq_quantize, oq._h, xm, dim, m)
    rc_s, out_s, codes_s = _quantize(lib.vqb_opq_quantize_static, oq._h, xm, dim, m)
    assert rc_a == 0 and rc_s == 0
    assert torch.equal(codes_s, codes_a) and torch.equal(out_s.view(torch.int16), out_a.view(torch.int16))

    # host pointers are refused (staging them would need an allocation); the wrong width keeps the reference's error
    xh = np.zeros((4, dim), np.float32)
    oh = np.zeros((4, dim), np.uint16)
    rc = lib.vqb_opq_quantize_static(oq._h, xh.ctypes.data, 4, dim, oh.ctypes.data, None)
    assert rc == 90 and "device pointers only" in lib.vqb_last_error(ctx.handle).decode()
    rc = lib.vqb_opq_quantize_static(oq._h, C.c_void_p(xm.data_ptr()), 4, dim + 1, C.c_void_p(out_s.data_ptr()), None)
    assert rc == 3 and lib.vqb_last_error(ctx.handle).decode() == f"Dimension mismatch: expected {dim}, got {dim + 1}"
