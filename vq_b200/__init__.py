"""vq_b200 -- host-side mirror of the reference's quantizer API over libvqb.so.

Same names, argument meaning and error text as the Rust crate ``vq``
(src/pq.rs, src/rvq.rs, src/opq.rs, src/sq.rs, src/bq.rs, src/distances.rs,
src/exceptions.rs); the compute runs in hand-written sm_100a kernels behind
the C ABI of include/vqb.h.  Inputs may be numpy arrays (host memory, copied
by the library) or CUDA ``torch`` tensors (used in place); the output lives
where the input lives.  ``quantize`` accepts one vector (1-D, like the
reference) or a batch (2-D, one vector per row).

There is no CPU path: every call fails if the library or a B200 is missing.
"""
from __future__ import annotations

import ctypes as C
import threading

import numpy as np

from . import _lib
from .seeding import LbgSeeder, StandInRng  # noqa: F401

ACCUM_AUTO, ACCUM_ORDERED, ACCUM_FAST = _lib.ACCUM_AUTO, _lib.ACCUM_ORDERED, _lib.ACCUM_FAST


# ---- errors (src/exceptions.rs:9-25) ------------------------------------------------------------
class VqError(Exception):
    """Base of the reference's error kinds; ``str(e)`` is the reference's Display text."""
    code = 0


class EmptyInput(VqError):
    code = 1


class InvalidParameter(VqError):
    code = 2


class DimensionMismatch(VqError):
    code = 3


class InvalidMetricParameter(VqError):
    code = 4


class BackendError(VqError):
    """CUDA / NCCL / argument failures below the reference's API (codes >= 90)."""


_ERRORS = {1: EmptyInput, 2: InvalidParameter, 3: DimensionMismatch, 4: InvalidMetricParameter}


def _raise(code: int, ctx_handle=None):
    msg = _lib.load().vqb_last_error(ctx_handle).decode()
    cls = _ERRORS.get(code, BackendError)
    err = cls(msg)
    err.code = code
    raise err


# ---- Distance (src/distances.rs:73-88) ----------------------------------------------------------
class Distance:
    """One of the reference's metrics; ``Distance.Minkowski(p)`` carries its parameter."""

    def __init__(self, metric: int, p: float = 0.0, name: str = ""):
        self.metric, self.p, self.name = metric, float(p), name

    def __repr__(self):
        return f"Distance.{self.name}" + (f"({self.p})" if self.metric == 5 else "")

    @staticmethod
    def Minkowski(p: float) -> "Distance":
        return Distance(5, p, "Minkowski")

    def compute(self, a, b, ctx: "Context | None" = None) -> float:
        """Distance::compute (src/distances.rs:115-172) for one pair, evaluated on the GPU."""
        a = np.ascontiguousarray(a, dtype=np.float32).ravel()
        b = np.ascontiguousarray(b, dtype=np.float32).ravel()
        ctx = ctx or default_context()
        out = np.empty(1, np.float32)
        rc = _lib.load().vqb_distance_rows(ctx.handle, self.metric, self.p, a.ctypes.data, a.size, b.ctypes.data,
                                           b.size, 1, out.ctypes.data)
        if rc:
            _raise(rc, ctx.handle)
        return float(out[0])


Distance.SquaredEuclidean = Distance(0, name="SquaredEuclidean")
Distance.Euclidean = Distance(1, name="Euclidean")
Distance.CosineDistance = Distance(2, name="CosineDistance")
Distance.Manhattan = Distance(3, name="Manhattan")
Distance.Chebyshev = Distance(4, name="Chebyshev")
Distance.Hamming = Distance(6, name="Hamming")


class Vector:
    """Thin stand-in for the reference's ``Vector<T>`` (src/vector.rs:149-176): ``data`` is a 1-D numpy array."""

    def __init__(self, data):
        self.data = np.asarray(data)

    def __len__(self):
        return int(self.data.shape[0])

    def len(self):
        return len(self)

    def is_empty(self):
        return len(self) == 0


# ---- context ------------------------------------------------------------------------------------
class Context:
    """One per (process, GPU): owns the library's stream, scratch and (optionally) the NCCL communicator."""

    def __init__(self, device: int = 0):
        L = _lib.load()
        h = C.c_void_p()
        rc = L.vqb_ctx_create(int(device), C.byref(h))
        if rc:
            _raise(rc, None)
        self.handle = h
        self.device = int(device)
        self.rank, self.world = 0, 1

    def close(self):
        if getattr(self, "handle", None):
            _lib.load().vqb_ctx_destroy(self.handle)
            self.handle = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def set_stream(self, cuda_stream: int | None):
        """Run on the given cudaStream_t handle (0 = the CUDA default stream); None = the context's own stream."""
        L = _lib.load()
        rc = L.vqb_ctx_reset_stream(self.handle) if cuda_stream is None else L.vqb_ctx_set_stream(self.handle, C.c_void_p(cuda_stream))
        if rc:
            _raise(rc, self.handle)

    def synchronize(self):
        rc = _lib.load().vqb_ctx_synchronize(self.handle)
        if rc:
            _raise(rc, self.handle)

    def launch_count(self) -> int:
        n = C.c_uint64(0)
        _lib.load().vqb_ctx_launch_count(self.handle, C.byref(n))
        return int(n.value)

    def alloc_count(self) -> int:
        """How often this context has asked CUDA for device or pinned memory so far."""
        n = C.c_uint64(0)
        _lib.load().vqb_ctx_alloc_count(self.handle, C.byref(n))
        return int(n.value)

    def timing(self, enable: bool):
        rc = _lib.load().vqb_ctx_timing(self.handle, 1 if enable else 0)
        if rc:
            _raise(rc, self.handle)

    def timing_report(self) -> dict:
        import json
        buf = C.create_string_buffer(1 << 16)
        rc = _lib.load().vqb_ctx_timing_report(self.handle, buf, len(buf))
        if rc:
            _raise(rc, self.handle)
        return json.loads(buf.value.decode())

    def use_stream(self, cuda_stream: int | None):
        """Pin all work of this context to `cuda_stream` (e.g. torch.cuda.current_stream().cuda_stream), also for
        host-memory inputs; None returns to the default behaviour (caller's torch stream for CUDA tensors, the
        context's own stream for host arrays)."""
        self._sticky = cuda_stream
        self._pinned = cuda_stream is not None
        self.set_stream(cuda_stream)

    def init_comm(self, unique_id: bytes, rank: int, world: int):
        """Join the NCCL communicator of a one-process-per-GPU job (see vq_b200.distributed)."""
        buf = (C.c_uint8 * _lib.UNIQUE_ID_BYTES).from_buffer_copy(unique_id)
        rc = _lib.load().vqb_comm_init(self.handle, buf, int(rank), int(world))
        if rc:
            _raise(rc, self.handle)
        self.rank, self.world = int(rank), int(world)

    def exchange_count(self) -> int:
        """Iterations so far whose per-rank parts were added by the centroid-update kernel over peer memory (0: NCCL)."""
        n = C.c_uint64(0)
        _lib.load().vqb_comm_exchange_count(self.handle, C.byref(n))
        return int(n.value)

    def destroy_comm(self):
        _lib.load().vqb_comm_destroy(self.handle)
        self.rank, self.world = 0, 1


_default = {}
_default_lock = threading.Lock()


def default_context(device: int | None = None) -> Context:
    if device is None:
        device = 0
        try:
            import torch
            if torch.cuda.is_available():
                device = torch.cuda.current_device()
        except Exception:
            pass
    with _default_lock:
        ctx = _default.get(device)
        if ctx is None:
            ctx = _default[device] = Context(device)
        return ctx


def unique_id() -> bytes:
    buf = (C.c_uint8 * _lib.UNIQUE_ID_BYTES)()
    rc = _lib.load().vqb_comm_unique_id(buf)
    if rc:
        _raise(rc, None)
    return bytes(buf)


# ---- array plumbing -----------------------------------------------------------------------------
def _is_torch(x) -> bool:
    return type(x).__module__.startswith("torch")


class _Arr:
    """A float32 C-contiguous view of the caller's data plus where outputs should live."""

    def __init__(self, x, ctx: Context, want_2d=True):
        self.torch = None
        if isinstance(x, Vector):
            x = x.data
        if _is_torch(x) and x.is_cuda:
            import torch
            self.torch = torch
            t = x.detach()
            if t.dtype != torch.float32 or not t.is_contiguous():
                t = t.to(torch.float32).contiguous()
            self.keep = t
            self.shape = tuple(t.shape)
            self.ptr = t.data_ptr()
            self.device = t.device
            if not getattr(ctx, "_pinned", False):
                ctx.set_stream(torch.cuda.current_stream(t.device).cuda_stream)
        else:
            if _is_torch(x):
                x = x.detach().cpu().numpy()
            a = np.ascontiguousarray(x, dtype=np.float32)
            self.keep = a
            self.shape = a.shape
            self.ptr = a.ctypes.data
            if not getattr(ctx, "_pinned", False):
                ctx.set_stream(None)
        self.single = len(self.shape) == 1
        if want_2d:
            if len(self.shape) == 1:
                self.n, self.dim = 1, self.shape[0]
            elif len(self.shape) == 2:
                self.n, self.dim = self.shape
            else:
                raise ValueError("expected a vector or a matrix of row vectors")
        self.size = int(np.prod(self.shape)) if len(self.shape) else 1

    def empty(self, shape, np_dtype, out=None):
        """A fresh result of the input's kind, or the caller's `out`: a C-contiguous array of this shape and dtype that
        lives where the input lives (numpy or CPU tensor for host input -- page-locked memory makes the copy back run at the
        link's rate -- CUDA tensor for device input)."""
        if out is not None:
            want = tuple(int(v) for v in shape)
            if _is_torch(out):
                tdt = {np.float16: "float16", np.uint8: "uint8", np.uint32: "int32", np.float32: "float32"}[np_dtype]
                on_device = bool(out.is_cuda)
                ok = tuple(out.shape) == want and str(out.dtype) == "torch." + tdt and out.is_contiguous()
                ptr = out.data_ptr()
            else:
                on_device = False
                ok = isinstance(out, np.ndarray) and out.shape == want and out.dtype == np.dtype(np_dtype) and out.flags.c_contiguous \
                    and out.flags.writeable
                ptr = out.ctypes.data if ok else 0
            if not ok or on_device != (self.torch is not None):
                raise ValueError(f"out must be a contiguous {np.dtype(np_dtype).name} array of shape {want} on the input's side")
            return out, ptr
        if self.torch is not None:
            tdt = {np.float16: self.torch.float16, np.uint8: self.torch.uint8, np.uint32: self.torch.int32,
                   np.float32: self.torch.float32}[np_dtype]
            t = self.torch.empty(shape, dtype=tdt, device=self.device)
            return t, t.data_ptr()
        a = np.empty(shape, dtype=np_dtype)
        return a, a.ctypes.data


def _rows(training_data, ctx):
    """Pack the reference's ``&[Vector<f32>]`` (list of rows) or take an n x dim array as is."""
    if isinstance(training_data, (list, tuple)):
        if len(training_data) == 0:
            return _Arr(np.zeros((0, 0), np.float32), ctx)
        training_data = np.stack([v.data if isinstance(v, Vector) else np.asarray(v) for v in training_data])
    arr = _Arr(training_data, ctx)
    return arr


def _make_draw(seeder: LbgSeeder):
    return _lib.DRAW_FN(lambda user, stream, n: seeder.draw(int(stream), int(n)))


def _global_rows(n_local: int, ctx: Context) -> int:
    if ctx.world <= 1:
        return n_local
    import torch
    import torch.distributed as dist
    t = torch.tensor([n_local], dtype=torch.int64)
    if dist.get_backend() == "nccl":
        t = t.cuda(ctx.device)
    dist.all_reduce(t)
    return int(t.item())


# ---- ProductQuantizer (src/pq.rs) ---------------------------------------------------------------
class ProductQuantizer:
    def __init__(self, handle, ctx: Context, distance: Distance):
        self._h, self._ctx, self.distance = handle, ctx, distance

    @classmethod
    def fit(cls, training_data, m: int, k: int, max_iters: int, distance: Distance, seed: int, *,
            ctx: Context | None = None, accumulate: int = ACCUM_AUTO, init_idx=None, draw=None):
        """ProductQuantizer::fit (src/pq.rs:79-129).  In a multi-GPU job ``training_data`` is this rank's
        shard.  ``init_idx`` (m x k global row indices) and ``draw(stream, n)`` override the seeded stand-in."""
        ctx = ctx or default_context()
        L = _lib.load()
        x = _rows(training_data, ctx)
        n_global = _global_rows(x.n, ctx)
        seeder = LbgSeeder(seed)
        if init_idx is None:
            ok = m > 0 and 0 < k <= n_global
            init_idx = (np.stack([seeder.init_indices(i, n_global, k) for i in range(m)]) if ok
                        else np.zeros((max(m, 1), max(k, 1)), np.uint64))
        init_idx = np.ascontiguousarray(init_idx, dtype=np.uint64)
        cb = _lib.DRAW_FN(lambda user, stream, n: int(draw(int(stream), int(n)))) if draw else _make_draw(seeder)
        h = C.c_void_p()
        rc = L.vqb_pq_fit(ctx.handle, x.ptr, x.n, x.dim, m, k, max_iters, distance.metric, distance.p,
                          init_idx.ctypes.data, cb, None, accumulate, C.byref(h))
        if rc:
            _raise(rc, ctx.handle)
        return cls(h, ctx, distance)

    @classmethod
    def from_codebooks(cls, codebooks, distance: Distance, *, ctx: Context | None = None):
        ctx = ctx or default_context()
        cbk = np.ascontiguousarray(codebooks, dtype=np.float32)
        m, k, sd = cbk.shape
        h = C.c_void_p()
        rc = _lib.load().vqb_pq_from_codebooks(ctx.handle, cbk.ctypes.data, m, k, sd, distance.metric, distance.p,
                                                C.byref(h))
        if rc:
            _raise(rc, ctx.handle)
        return cls(h, ctx, distance)

    def shape(self):
        m, k, sd = C.c_size_t(), C.c_size_t(), C.c_size_t()
        _lib.load().vqb_pq_shape(self._h, C.byref(m), C.byref(k), C.byref(sd))
        return int(m.value), int(k.value), int(sd.value)

    @property
    def codebooks(self) -> np.ndarray:
        m, k, sd = self.shape()
        out = np.empty((m, k, sd), np.float32)
        rc = _lib.load().vqb_pq_codebooks(self._h, out.ctypes.data)
        if rc:
            _raise(rc, self._ctx.handle)
        return out

    @property
    def iterations(self) -> np.ndarray:
        m = self.shape()[0]
        out = np.zeros(m, dtype=np.uintp)
        _lib.load().vqb_pq_iterations(self._h, out.ctypes.data)
        return out

    def quantize(self, vector, return_codes: bool = False, out=None):
        """ProductQuantizer::quantize (src/pq.rs:146-187): f16 reconstruction, one row per input vector (written to `out`
        when given: n x dim float16)."""
        x = _Arr(vector, self._ctx)
        out, optr = x.empty((x.n, x.dim), np.float16, out)
        codes, cptr = (x.empty((x.n, self.shape()[0]), np.uint32) if return_codes else (None, None))
        rc = _lib.load().vqb_pq_quantize(self._h, x.ptr, x.n, x.dim, optr, cptr)
        if rc:
            _raise(rc, self._ctx.handle)
        if x.single:
            out = out[0]
            codes = codes[0] if codes is not None else None
        return (out, codes) if return_codes else out

    def __del__(self):
        try:
            if self._h:
                _lib.load().vqb_pq_destroy(self._h)
                self._h = None
        except Exception:
            pass


# ---- ResidualQuantizer (src/rvq.rs) -------------------------------------------------------------
class ResidualQuantizer:
    def __init__(self, handle, ctx: Context, distance: Distance):
        self._h, self._ctx, self.distance = handle, ctx, distance

    @classmethod
    def fit(cls, training_data, stages: int, k: int, max_iters: int, epsilon: float, distance: Distance, seed: int, *,
            ctx: Context | None = None, accumulate: int = ACCUM_AUTO, init=None, draw=None):
        """ResidualQuantizer::fit (src/rvq.rs:87-154).  ``init(stage, n, k)`` overrides the seeded stand-in."""
        ctx = ctx or default_context()
        x = _rows(training_data, ctx)
        seeder = LbgSeeder(seed)

        def _init(user, stage, n, kk, out):
            idx = init(int(stage), int(n), int(kk)) if init else seeder.init_indices(int(stage), int(n), int(kk))
            for j in range(int(kk)):
                out[j] = int(idx[j])

        icb = _lib.INIT_FN(_init)
        dcb = _lib.DRAW_FN(lambda user, stream, n: int(draw(int(stream), int(n)))) if draw else _make_draw(seeder)
        h = C.c_void_p()
        rc = _lib.load().vqb_rvq_fit(ctx.handle, x.ptr, x.n, x.dim, stages, k, max_iters, float(epsilon),
                                     distance.metric, distance.p, icb, dcb, None, accumulate, C.byref(h))
        if rc:
            _raise(rc, ctx.handle)
        return cls(h, ctx, distance)

    @classmethod
    def from_codebooks(cls, codebooks, epsilon: float, distance: Distance, *, ctx: Context | None = None):
        ctx = ctx or default_context()
        cbk = np.ascontiguousarray(codebooks, dtype=np.float32)
        stages, k, dim = cbk.shape
        h = C.c_void_p()
        rc = _lib.load().vqb_rvq_from_codebooks(ctx.handle, cbk.ctypes.data, stages, k, dim, float(epsilon),
                                                 distance.metric, distance.p, C.byref(h))
        if rc:
            _raise(rc, ctx.handle)
        return cls(h, ctx, distance)

    def shape(self):
        s, k, d = C.c_size_t(), C.c_size_t(), C.c_size_t()
        _lib.load().vqb_rvq_shape(self._h, C.byref(s), C.byref(k), C.byref(d))
        return int(s.value), int(k.value), int(d.value)

    @property
    def codebooks(self) -> np.ndarray:
        s, k, d = self.shape()
        out = np.empty((s, k, d), np.float32)
        if out.size:
            rc = _lib.load().vqb_rvq_codebooks(self._h, out.ctypes.data)
            if rc:
                _raise(rc, self._ctx.handle)
        return out

    def quantize(self, vector, return_codes: bool = False, out=None):
        """ResidualQuantizer::quantize (src/rvq.rs:171-215); `out` as in ProductQuantizer.quantize."""
        x = _Arr(vector, self._ctx)
        out, optr = x.empty((x.n, x.dim), np.float16, out)
        codes, cptr = (x.empty((x.n, self.shape()[0]), np.uint32) if return_codes else (None, None))
        rc = _lib.load().vqb_rvq_quantize(self._h, x.ptr, x.n, x.dim, optr, cptr)
        if rc:
            _raise(rc, self._ctx.handle)
        if x.single:
            out = out[0]
            codes = codes[0] if codes is not None else None
        return (out, codes) if return_codes else out

    def __del__(self):
        try:
            if self._h:
                _lib.load().vqb_rvq_destroy(self._h)
                self._h = None
        except Exception:
            pass


# ---- OptimizedProductQuantizer (src/opq.rs) -----------------------------------------------------
class OptimizedProductQuantizer:
    def __init__(self, handle, ctx: Context, distance: Distance, dim: int):
        self._h, self._ctx, self.distance, self.dim = handle, ctx, distance, dim

    @classmethod
    def fit(cls, training_data, m: int, k: int, max_iters: int, opq_iters: int, distance: Distance, seed: int, *,
            ctx: Context | None = None, accumulate: int = ACCUM_AUTO, init_idx=None):
        """OptimizedProductQuantizer::fit (src/opq.rs:90-205)."""
        ctx = ctx or default_context()
        x = _rows(training_data, ctx)
        n_global = _global_rows(x.n, ctx)
        state = {"seeder": LbgSeeder(seed)}
        ok = m > 0 and 0 < k <= n_global
        user_idx = init_idx is not None
        if init_idx is None:
            init_idx = (np.stack([state["seeder"].init_indices(i, n_global, k) for i in range(m)]) if ok
                        else np.zeros((max(m, 1), max(k, 1)), np.uint64))
        init_idx = np.ascontiguousarray(init_idx, dtype=np.uint64)

        # every outer iteration re-creates StdRng(seed + i) (src/opq.rs:140): same sample, same draws.  The streams' states
        # right after the initial sample are the same every time, so they are recorded once and restored (drawing the
        # 16 x 256 sample again in Python cost 2.4 ms per outer iteration of the benchmark configuration).
        after_init = {st: r.state for st, r in state["seeder"].rngs.items()} if ok and not user_idx else {}

        def _restart(user):
            state["seeder"] = LbgSeeder(seed)
            for st, value in after_init.items():
                rng = StandInRng(0)
                rng.state = value
                state["seeder"].rngs[st] = rng

        rcb = _lib.RESTART_FN(_restart)
        dcb = _lib.DRAW_FN(lambda user, stream, n: state["seeder"].draw(int(stream), int(n)))
        h = C.c_void_p()
        rc = _lib.load().vqb_opq_fit(ctx.handle, x.ptr, x.n, x.dim, m, k, max_iters, opq_iters, distance.metric,
                                     distance.p, init_idx.ctypes.data, dcb, rcb, None, accumulate, C.byref(h))
        if rc:
            _raise(rc, ctx.handle)
        return cls(h, ctx, distance, x.dim)

    @classmethod
    def from_parts(cls, rotation, codebooks, distance: Distance, *, ctx: Context | None = None):
        ctx = ctx or default_context()
        rot = np.ascontiguousarray(rotation, dtype=np.float32)
        cbk = np.ascontiguousarray(codebooks, dtype=np.float32)
        m, k, sd = cbk.shape
        h = C.c_void_p()
        rc = _lib.load().vqb_opq_from_parts(ctx.handle, rot.ctypes.data, cbk.ctypes.data, m, k, sd, distance.metric,
                                             distance.p, C.byref(h))
        if rc:
            _raise(rc, ctx.handle)
        return cls(h, ctx, distance, m * sd)

    def shape(self):
        m, k, sd = C.c_size_t(), C.c_size_t(), C.c_size_t()
        _lib.load().vqb_opq_shape(self._h, C.byref(m), C.byref(k), C.byref(sd))
        return int(m.value), int(k.value), int(sd.value)

    @property
    def rotation(self) -> np.ndarray:
        out = np.empty((self.dim, self.dim), np.float32)
        rc = _lib.load().vqb_opq_rotation(self._h, out.ctypes.data)
        if rc:
            _raise(rc, self._ctx.handle)
        return out

    @property
    def codebooks(self) -> np.ndarray:
        m, k, sd = self.shape()
        out = np.empty((m, k, sd), np.float32)
        if out.size:
            rc = _lib.load().vqb_opq_codebooks(self._h, out.ctypes.data)
            if rc:
                _raise(rc, self._ctx.handle)
        return out

    def quantize(self, vector, return_codes: bool = False, out=None):
        """OptimizedProductQuantizer::quantize (src/opq.rs:222-264).  Without codebooks (opq_iters == 0)
        the result is empty, as in the reference.  `out` as in ProductQuantizer.quantize."""
        x = _Arr(vector, self._ctx)
        m = self.shape()[0]
        width = x.dim if m else 0
        out, optr = x.empty((x.n, width), np.float16, out)
        codes, cptr = (x.empty((x.n, m), np.uint32) if return_codes else (None, None))
        rc = _lib.load().vqb_opq_quantize(self._h, x.ptr, x.n, x.dim, optr if width else None,
                                           cptr if (return_codes and m) else None)
        if rc:
            _raise(rc, self._ctx.handle)
        if x.single:
            out = out[0]
            codes = codes[0] if codes is not None else None
        return (out, codes) if return_codes else out

    def __del__(self):
        try:
            if self._h:
                _lib.load().vqb_opq_destroy(self._h)
                self._h = None
        except Exception:
            pass


# ---- ScalarQuantizer / BinaryQuantizer (src/sq.rs, src/bq.rs) -----------------------------------
class ScalarQuantizer:
    def __init__(self, vmin, vmax, levels, step, ctx):
        self.min, self.max, self.levels, self.step, self._ctx = vmin, vmax, levels, step, ctx

    @classmethod
    def fit(cls, min: float, max: float, levels: int, *, ctx: Context | None = None):
        """ScalarQuantizer::fit (src/sq.rs:50-76)."""
        step = C.c_float()
        rc = _lib.load().vqb_sq_fit(float(min), float(max), int(levels), C.byref(step))
        if rc:
            _raise(rc, None)
        return cls(float(np.float32(min)), float(np.float32(max)), int(levels), float(step.value), ctx)

    def quantize(self, vector, out=None):
        """ScalarQuantizer::quantize (src/sq.rs:89-106); any shape, element-wise (into `out` when given: uint8, the input's shape)."""
        ctx = self._ctx or default_context()
        x = _Arr(vector, ctx, want_2d=False)
        out, optr = x.empty(x.shape, np.uint8, out)
        rc = _lib.load().vqb_sq_quantize(ctx.handle, self.min, self.max, self.levels, self.step, x.ptr, x.size, optr)
        if rc:
            _raise(rc, ctx.handle)
        return out


class BinaryQuantizer:
    def __init__(self, threshold, low, high, ctx):
        self.threshold, self.low, self.high, self._ctx = threshold, low, high, ctx

    @classmethod
    def fit(cls, threshold: float, low: int, high: int, *, ctx: Context | None = None):
        """BinaryQuantizer::fit (src/bq.rs:46-60)."""
        rc = _lib.load().vqb_bq_fit(float(threshold), int(low), int(high))
        if rc:
            _raise(rc, None)
        return cls(float(np.float32(threshold)), int(low), int(high), ctx)

    def quantize(self, vector, out=None):
        """BinaryQuantizer::quantize (src/bq.rs:75-104); any shape, element-wise (into `out` when given: uint8, the input's shape)."""
        ctx = self._ctx or default_context()
        x = _Arr(vector, ctx, want_2d=False)
        out, optr = x.empty(x.shape, np.uint8, out)
        rc = _lib.load().vqb_bq_quantize(ctx.handle, self.threshold, self.low, self.high, x.ptr, x.size, optr)
        if rc:
            _raise(rc, ctx.handle)
        return out


class TSVQ:
    """TSVQ (src/tsvq.rs:189-250): ``TSVQ(training_data, max_depth, distance)`` builds the tree, ``quantize`` returns the
    leaf centroid as f16.  ``tree()`` gives (centroids, left, right) with nodes numbered breadth-first."""

    def __init__(self, training_data, max_depth: int, distance: Distance, *, ctx: Context | None = None):
        ctx = ctx or default_context()
        x = _rows(training_data, ctx)
        h = C.c_void_p()
        rc = _lib.load().vqb_tsvq_fit(ctx.handle, x.ptr, x.n, x.dim, int(max_depth), distance.metric, distance.p, C.byref(h))
        if rc:
            _raise(rc, ctx.handle)
        self._h, self._ctx, self.distance = h, ctx, distance

    def shape(self):
        nodes, dim = C.c_size_t(), C.c_size_t()
        _lib.load().vqb_tsvq_shape(self._h, C.byref(nodes), C.byref(dim))
        return int(nodes.value), int(dim.value)

    def tree(self):
        nodes, dim = self.shape()
        cent = np.empty((nodes, dim), np.float32)
        left = np.empty(nodes, np.int32)
        right = np.empty(nodes, np.int32)
        rc = _lib.load().vqb_tsvq_tree(self._h, cent.ctypes.data, left.ctypes.data, right.ctypes.data)
        if rc:
            _raise(rc, self._ctx.handle)
        return cent, left, right

    def quantize(self, vector, return_leaf: bool = False, out=None):
        """TSVQ::quantize (src/tsvq.rs:231-249): one f16 row per input vector; `out` as in ProductQuantizer.quantize."""
        x = _Arr(vector, self._ctx)
        out, optr = x.empty((x.n, x.dim), np.float16, out)
        leaf, lptr = (x.empty((x.n,), np.uint32) if return_leaf else (None, None))
        rc = _lib.load().vqb_tsvq_quantize(self._h, x.ptr, x.n, x.dim, optr, lptr)
        if rc:
            _raise(rc, self._ctx.handle)
        if x.single:
            out = out[0]
            leaf = leaf[0] if leaf is not None else None
        return (out, leaf) if return_leaf else out

    def __del__(self):
        try:
            if self._h:
                _lib.load().vqb_tsvq_destroy(self._h)
                self._h = None
        except Exception:
            pass


def evaluate(original, quantized_f16, k: int = 10, *, ctx: Context | None = None):
    """The reference harness's quality metrics on the device: (reconstruction error, recall@k), i.e.
    calculate_reconstruction_error and calculate_recall of src/bin/utils.rs:50-127 applied to the f16 output of a
    ``quantize`` call (numpy float16 array or CUDA float16 tensor, one row per vector)."""
    ctx = ctx or default_context()
    x = _Arr(original, ctx)
    if _is_torch(quantized_f16) and quantized_f16.is_cuda:
        qk = quantized_f16.contiguous()
        qptr = qk.data_ptr()
    else:
        qk = np.ascontiguousarray(quantized_f16, dtype=np.float16)
        qptr = qk.ctypes.data
    mse, rec = C.c_float(), C.c_float()
    rc = _lib.load().vqb_evaluate_f16(ctx.handle, x.ptr, qptr, x.n, x.dim, int(k), C.byref(mse), C.byref(rec))
    if rc:
        _raise(rc, ctx.handle)
    return float(mse.value), float(rec.value)


def lbg_quantize(data, k: int, max_iters: int, seed: int, *, ctx: Context | None = None, accumulate: int = ACCUM_AUTO,
                 init_idx=None, draw=None):
    """lbg_quantize (src/utils.rs:32-109) on n x d rows.  Returns (centroids k x d, iterations)."""
    ctx = ctx or default_context()
    x = _rows(data, ctx)
    seeder = LbgSeeder(seed)
    if init_idx is None:
        init_idx = seeder.init_indices(0, x.n, k) if 0 < k <= x.n else np.zeros(max(k, 1), np.uint64)
    init_idx = np.ascontiguousarray(init_idx, dtype=np.uint64)
    cb = _lib.DRAW_FN(lambda user, stream, n: int(draw(int(stream), int(n)))) if draw else _make_draw(seeder)
    out = np.empty((k, x.dim), np.float32)
    iters = C.c_size_t(0)
    rc = _lib.load().vqb_lbg_fit(ctx.handle, x.ptr, x.n, x.dim, k, max_iters, init_idx.ctypes.data, cb, None,
                                 accumulate, out.ctypes.data if out.size else None, C.byref(iters))
    if rc:
        _raise(rc, ctx.handle)
    return out, int(iters.value)
