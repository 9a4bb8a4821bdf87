"""vqb_opq_quantize_static: the OPQ encode for embedders that cannot let the library allocate device memory
(all HBM already belongs to their own pool, or the CUDA allocator must stay out of their request loop).

Two things are checked, both through the C ABI with device pointers:

* that the call really allocates nothing.  This runs in a child process with a fresh context whose FIRST encode is the
  static one, so nothing an earlier call provisioned can hide an allocation: the library's own allocation counter, the
  reserved size of the device's stream-ordered memory pool and the free device memory are read before and after three
  calls with growing row counts, and must not move;
* that the result equals vqb_opq_quantize on the same inputs, bit for bit, twice in a row (the static scratch keeps the
  previous call's rows, so the second call, with fewer and different rows, would show stale data if the entry point
  relied on the array's old contents).

This file sorts last on purpose.
"""
import ctypes as C
import os
import subprocess
import sys

import numpy as np
import pytest

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _quantize(fn, handle, x, dim, m):
    import torch
    n = x.shape[0]
    out = torch.zeros((n, dim), dtype=torch.float16, device="cuda")
    codes = torch.zeros((n, m), dtype=torch.int32, device="cuda")
    rc = fn(handle, C.c_void_p(x.data_ptr()), n, dim, C.c_void_p(out.data_ptr()), C.c_void_p(codes.data_ptr()))
    torch.cuda.synchronize()
    return rc, out, codes


CHILD = r"""
import ctypes as C, json, sys
import numpy as np, torch
sys.path.insert(0, sys.argv[1])
import vq_b200 as vq
from vq_b200 import _lib

lib = _lib.load()
torch.cuda.init()
ctx = vq.Context(torch.cuda.current_device())
ctx.use_stream(torch.cuda.current_stream().cuda_stream)
rng = np.random.default_rng(5)
report = {}
for dim, m, k in ((128, 16, 256), (64, 8, 32)):   # both are shapes the allocating entry point runs on its tensor-core kernel
    q, _ = np.linalg.qr(rng.normal(size=(dim, dim)))
    oq = vq.OptimizedProductQuantizer.from_parts(q.astype(np.float32), rng.normal(size=(m, k, dim // m)).astype(np.float32),
                                                 vq.Distance.Euclidean, ctx=ctx)
    sizes = (700, 3000, (1 << 20) // dim)       # growing: a scratch buffer sized by an earlier call would have to grow
    xs = [torch.from_numpy(rng.normal(size=(n, dim)).astype(np.float32)).cuda() for n in sizes]
    outs = [torch.zeros((n, dim), dtype=torch.float16, device="cuda") for n in sizes]
    codes = [torch.zeros((n, m), dtype=torch.int32, device="cuda") for n in sizes]
    ref_outs = [torch.zeros_like(o) for o in outs]
    ref_codes = [torch.zeros_like(c) for c in codes]
    torch.cuda.synchronize()
    def snapshot():
        free, _total = torch.cuda.mem_get_info()
        return {"allocs": ctx.alloc_count(), "free": int(free)}
    before = snapshot()
    rcs = []
    for x, o, c in zip(xs, outs, codes):
        rcs.append(lib.vqb_opq_quantize_static(oq._h, C.c_void_p(x.data_ptr()), x.shape[0], dim, C.c_void_p(o.data_ptr()), C.c_void_p(c.data_ptr())))
        rcs.append(lib.vqb_ctx_synchronize(ctx.handle))
    torch.cuda.synchronize()
    after = snapshot()
    # only now the allocating entry point, for the comparison
    for x, o, c in zip(xs, ref_outs, ref_codes):
        rcs.append(lib.vqb_opq_quantize(oq._h, C.c_void_p(x.data_ptr()), x.shape[0], dim, C.c_void_p(o.data_ptr()), C.c_void_p(c.data_ptr())))
    torch.cuda.synchronize()
    later = snapshot()
    report[f"{dim}x{m}x{k}"] = {
        "rcs": rcs, "before": before, "after": after, "later": later,
        "equal": all(torch.equal(a, b) for a, b in zip(codes, ref_codes)) and
                 all(torch.equal(a.view(torch.int16), b.view(torch.int16)) for a, b in zip(outs, ref_outs)),
        "nonzero": all(float(o.float().abs().sum()) > 0 for o in outs),
    }
print("REPORT " + json.dumps(report))
"""


def test_static_entry_point_allocates_nothing_on_a_fresh_context():
    # every kernel image is loaded when the context is created, so that loading one cannot pass for an allocation
    env = dict(os.environ, CUDA_MODULE_LOADING="EAGER")
    proc = subprocess.run([sys.executable, "-c", CHILD, ROOT], env=env, capture_output=True, text=True, timeout=600)
    assert proc.returncode == 0, proc.stdout[-2000:] + proc.stderr[-3000:]
    import json
    line = [ln for ln in proc.stdout.splitlines() if ln.startswith("REPORT ")][-1]
    report = json.loads(line[len("REPORT "):])
    assert len(report) == 2
    for shape, r in report.items():
        assert all(rc == 0 for rc in r["rcs"]), (shape, r["rcs"])
        assert r["after"]["allocs"] == r["before"]["allocs"], (shape, r)      # the library asked CUDA for no memory
        assert r["after"]["free"] == r["before"]["free"], (shape, r)          # and the device's free memory did not move
        assert r["later"]["allocs"] > r["after"]["allocs"], (shape, r)        # the counter does see the allocating entry point
        assert r["equal"] and r["nonzero"], shape


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
        allocs = ctx.alloc_count()
        rc_s, out_s, codes_s = _quantize(lib.vqb_opq_quantize_static, oq._h, x, dim, m)
        assert ctx.alloc_count() == allocs
        rc_a, out_a, codes_a = _quantize(lib.vqb_opq_quantize, oq._h, x, dim, m)
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
    rc_s, out_s, codes_s = _quantize(lib.vqb_opq_quantize_static, oq._h, xm, dim, m)
    rc_a, out_a, codes_a = _quantize(lib.vqb_opq_quantize, oq._h, xm, dim, m)
    assert rc_a == 0 and rc_s == 0
    assert torch.equal(codes_s, codes_a) and torch.equal(out_s.view(torch.int16), out_a.view(torch.int16))

    # host pointers are refused (staging them would need an allocation); the wrong width keeps the reference's error
    xh = np.zeros((4, dim), np.float32)
    oh = np.zeros((4, dim), np.uint16)
    rc = lib.vqb_opq_quantize_static(oq._h, xh.ctypes.data, 4, dim, oh.ctypes.data, None)
    assert rc == 90 and "device pointers only" in lib.vqb_last_error(ctx.handle).decode()
    rc = lib.vqb_opq_quantize_static(oq._h, C.c_void_p(xm.data_ptr()), 4, dim + 1, C.c_void_p(out_s.data_ptr()), None)
    assert rc == 3 and lib.vqb_last_error(ctx.handle).decode() == f"Dimension mismatch: expected {dim}, got {dim + 1}"
