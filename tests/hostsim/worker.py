"""One CPU rank of the host-loop simulation (TEST INFRASTRUCTURE; see hostsim.cpp).

usage: worker.py <case.npz> <out_prefix>   with RANK / WORLD_SIZE / MASTER_ADDR / MASTER_PORT in the environment.
The all-reduces the training loops ask for are carried by torch.distributed with the gloo backend.
"""
import ctypes as C
import os
import sys

import numpy as np
import torch
import torch.distributed as dist

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, ROOT)

from vq_b200.distributed import shard_bounds  # noqa: E402
from vq_b200.seeding import LbgSeeder  # noqa: E402

DRAW_FN = C.CFUNCTYPE(C.c_uint64, C.c_void_p, C.c_size_t, C.c_uint64)
INIT_FN = C.CFUNCTYPE(None, C.c_void_p, C.c_size_t, C.c_uint64, C.c_size_t, C.POINTER(C.c_uint64))
RESTART_FN = C.CFUNCTYPE(None, C.c_void_p)
AR_FN = C.CFUNCTYPE(None, C.c_void_p, C.c_int, C.c_void_p, C.c_size_t)
KINDS = {0: (np.float32, dist.ReduceOp.SUM), 1: (np.float64, dist.ReduceOp.SUM), 2: (np.int32, dist.ReduceOp.SUM),
         3: (np.int64, dist.ReduceOp.MAX), 4: (np.int64, dist.ReduceOp.SUM)}


def main():
    case = np.load(sys.argv[1], allow_pickle=True)
    out_prefix = sys.argv[2]
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    if world > 1:
        dist.init_process_group("gloo", rank=rank, world_size=world)
    lib = C.CDLL(os.path.join(HERE, "libhostsim.so"))
    lib.hs_last_error.restype = C.c_char_p
    calls = []

    def allreduce(user, kind, buf, n):
        calls.append((int(kind), int(n)))
        if kind == 3:  # max over u32 bit patterns: widen so the comparison is unsigned
            a = np.ctypeslib.as_array(C.cast(buf, C.POINTER(C.c_uint32)), shape=(n,))
            t = torch.from_numpy(a.astype(np.int64))
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            a[:] = t.numpy().astype(np.uint32)
            return
        ctype = {0: C.c_float, 1: C.c_double, 2: C.c_int32, 4: C.c_int64}[kind]
        a = np.ctypeslib.as_array(C.cast(buf, C.POINTER(ctype)), shape=(n,))
        t = torch.from_numpy(a)
        dist.all_reduce(t, op=dist.ReduceOp.SUM)

    ar = AR_FN(allreduce)
    x = np.ascontiguousarray(case["x"], dtype=np.float32)
    n, dim = x.shape
    begin, end = shard_bounds(n, rank, world)
    xs = np.ascontiguousarray(x[begin:end])
    kind = str(case["kind"])
    seed = int(case["seed"])
    k, iters = int(case["k"]), int(case["iters"])
    seeder = LbgSeeder(seed)
    draws = []

    def draw(user, stream, nn):
        r = seeder.draw(int(stream), int(nn))
        draws.append((int(stream), int(r)))
        return r

    dcb = DRAW_FN(draw)
    result = {}
    if kind == "pq":
        m = int(case["m"])
        init = np.stack([seeder.init_indices(i, n, k) for i in range(m)]) if 0 < k <= n else np.zeros((m, max(k, 1)), np.uint64)
        init = np.ascontiguousarray(init, dtype=np.uint64)
        cb = np.zeros((m, max(k, 1), dim // m), np.float32)
        its = np.zeros(m, dtype=np.uintp)
        rc = lib.hs_pq_fit(C.c_void_p(xs.ctypes.data), C.c_size_t(xs.shape[0]), C.c_size_t(dim), C.c_size_t(m), C.c_size_t(k),
                           C.c_size_t(iters), C.c_void_p(init.ctypes.data), dcb, None, ar, None, rank, world,
                           C.c_void_p(cb.ctypes.data), C.c_void_p(its.ctypes.data))
        lib.hs_moved_passes.restype = C.c_size_t
        lib.hs_pieces_walked.restype = C.c_size_t
        result = {"codebooks": cb, "iterations": its, "moved_passes": np.array(int(lib.hs_moved_passes())),
                  "pieces_walked": np.array(int(lib.hs_pieces_walked()))}
    elif kind == "rvq":
        stages = int(case["stages"])

        def init_fn(user, stage, nn, kk, out):
            idx = seeder.init_indices(int(stage), int(nn), int(kk))
            for j in range(int(kk)):
                out[j] = int(idx[j])

        icb = INIT_FN(init_fn)
        cb = np.zeros((stages, k, dim), np.float32)
        done = C.c_size_t(0)
        rc = lib.hs_rvq_fit(C.c_void_p(xs.ctypes.data), C.c_size_t(xs.shape[0]), C.c_size_t(dim), C.c_size_t(stages), C.c_size_t(k),
                            C.c_size_t(iters), C.c_float(float(case["epsilon"])), icb, dcb, None, ar, None, rank, world,
                            C.c_void_p(cb.ctypes.data), C.byref(done))
        result = {"codebooks": cb[: int(done.value)], "stages": np.array(int(done.value))}
    else:  # opq
        m = int(case["m"])
        outer = int(case["outer"])
        init = np.ascontiguousarray(np.stack([seeder.init_indices(i, n, k) for i in range(m)]), dtype=np.uint64)

        def restart(user):
            nonlocal seeder
            seeder = LbgSeeder(seed)
            for i in range(m):
                seeder.init_indices(i, n, k)

        rcb = RESTART_FN(restart)
        rot = np.zeros((dim, dim), np.float32)
        cb = np.zeros((m, k, dim // m), np.float32)
        rc = lib.hs_opq_fit(C.c_void_p(xs.ctypes.data), C.c_size_t(xs.shape[0]), C.c_size_t(dim), C.c_size_t(m), C.c_size_t(k),
                            C.c_size_t(iters), C.c_size_t(outer), C.c_void_p(init.ctypes.data), dcb, rcb, None, ar, None, rank, world,
                            C.c_void_p(rot.ctypes.data), C.c_void_p(cb.ctypes.data))
        result = {"rotation": rot, "codebooks": cb}
    np.savez(f"{out_prefix}.rank{rank}.npz", rc=np.array(rc), error=np.array(lib.hs_last_error().decode()),
             draws=np.array(draws, dtype=np.int64).reshape(-1, 2), allreduce_calls=np.array(calls, dtype=np.int64).reshape(-1, 2), **result)
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
