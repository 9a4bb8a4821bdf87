"""The multi-rank path of the training loops on CPU: world_size 2 (and 3) over torch.distributed/gloo.

The product's host loops (vq_b200/csrc/driver.cpp) are compiled against a CPU stand-in of the device interface
(tests/hostsim/, test infrastructure) and run as separate rank processes; results are compared with the single-process
oracle.  Integer-valued rows make every cluster sum exact in f32 whatever the order, so sharded runs must then
reproduce the oracle bit for bit, including re-seeded clusters whose rows live on another rank.
"""
import ctypes as C
import os
import socket
import subprocess
import sys

import numpy as np
import pytest

from tests.util import RecordingSeeder, by_stream

HERE = os.path.dirname(os.path.abspath(__file__))
SIM = os.path.join(HERE, "hostsim")


@pytest.fixture(scope="module")
def hostsim():
    subprocess.check_call(["make", "-C", SIM, "-s"])
    return os.path.join(SIM, "libhostsim.so")


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    return port


def run_ranks(tmp_path, world, extra_env=None, **case):
    path = os.path.join(tmp_path, "case.npz")
    np.savez(path, **case)
    prefix = os.path.join(tmp_path, "out")
    env = dict(os.environ, MASTER_ADDR="127.0.0.1", MASTER_PORT=str(_free_port()), WORLD_SIZE=str(world), OMP_NUM_THREADS="1")
    env.update(extra_env or {})
    procs = [subprocess.Popen([sys.executable, os.path.join(SIM, "worker.py"), path, prefix], env=dict(env, RANK=str(r)),
                              stdout=subprocess.PIPE, stderr=subprocess.STDOUT) for r in range(world)]
    for p in procs:
        out, _ = p.communicate(timeout=300)
        assert p.returncode == 0, out.decode()[-2000:]
    return [np.load(f"{prefix}.rank{r}.npz", allow_pickle=True) for r in range(world)]


def _draw_pairs(res):
    return [tuple(int(v) for v in row) for row in res["draws"]]


def _int_rows(n, dim, seed, hi=50, distinct=None):
    rng = np.random.default_rng(seed)
    if distinct:
        base = rng.integers(0, hi, (distinct, dim)).astype(np.float32)
        return base[rng.integers(0, distinct, n)]
    return rng.integers(0, hi, (n, dim)).astype(np.float32)


@pytest.mark.parametrize("world", [1, 2, 3])
def test_pq_fit_sharded_equals_oracle_on_exact_sums(hostsim, oracle, tmp_path, world):
    n, dim, m, k, iters, seed = 1001, 8, 2, 24, 12, 5
    x = _int_rows(n, dim, 3, distinct=60)  # duplicates force empty clusters -> re-seeds, some from the other rank's rows
    so = RecordingSeeder(seed)
    cb_o, it_o = oracle.pq_fit(x, m, k, iters, so.init_pq(n, m, k), so.draw)
    assert len(so.draws) > 0
    res = run_ranks(str(tmp_path), world, kind="pq", x=x, m=m, k=k, iters=iters, seed=seed)
    for r in res:
        assert int(r["rc"]) == 0, str(r["error"])
        assert np.array_equal(r["codebooks"], cb_o)
        assert np.array_equal(r["iterations"], it_o)
        assert by_stream(_draw_pairs(r)) == by_stream(so.draws)  # every rank evaluates the same draws
    if world > 1:
        calls = res[0]["allreduce_calls"]
        # per iteration ONE f32 all-reduce carries sums, counts and flags (fewer than 2^24 rows: counts are exact in f32);
        # plus the row-count exchange (u64, once) and the row patches (max): no u32 sums at all
        assert (calls[:, 0] == 0).sum() >= 1 and (calls[:, 0] == 2).sum() == 0
        f32_sizes = calls[calls[:, 0] == 0, 1]
        assert (f32_sizes == m * k * (dim // m) + m * k + m).all()
        assert (calls[:, 0] == 4).sum() == 1 and (calls[:, 0] == 3).sum() >= 1
        assert all(np.array_equal(res[0]["allreduce_calls"], r["allreduce_calls"]) for r in res[1:])


@pytest.mark.parametrize("world", [1, 2])
def test_unordered_mode_keeps_running_sums_and_moves_only_changed_rows(hostsim, oracle, tmp_path, world):
    """Unordered accumulation: after the first iteration every rank updates its running sums by the rows whose assignment
    changed and copies them into the exchange buffer (driver.cpp::lbg_fit).  On integer rows the sums are exact, so the
    sharded result must equal the oracle's bit for bit, re-seeded clusters included; the exchange stays one f32 all-reduce."""
    n, dim, m, k, iters, seed = 1501, 8, 2, 24, 12, 7
    x = _int_rows(n, dim, 4, distinct=70)
    so = RecordingSeeder(seed)
    cb_o, it_o = oracle.pq_fit(x, m, k, iters, so.init_pq(n, m, k), so.draw)
    res = run_ranks(str(tmp_path), world, extra_env={"HOSTSIM_ACCUM": "2"}, kind="pq", x=x, m=m, k=k, iters=iters, seed=seed)
    for r in res:
        assert int(r["rc"]) == 0, str(r["error"])
        assert np.array_equal(r["codebooks"], cb_o) and np.array_equal(r["iterations"], it_o)
        assert by_stream(_draw_pairs(r)) == by_stream(so.draws)
        assert int(r["moved_passes"]) >= 2          # the short cut ran (every iteration but the first)
    if world > 1:
        calls = res[0]["allreduce_calls"]
        assert ((calls[calls[:, 0] == 0, 1]) == m * k * (dim // m) + m * k + m).all() and (calls[:, 0] == 2).sum() == 0


@pytest.mark.parametrize("world,accum", [(1, "1"), (1, "2"), (2, "2")])
def test_first_iteration_follows_rows_that_arrive_in_pieces(hostsim, oracle, tmp_path, world, accum):
    """A fit handed a host buffer starts while the rows are still being copied in: the first iteration of lbg_fit assigns
    (and, unordered, adds up) one piece at a time (Device::arriving_pieces / await_piece).  Here the pieces are only a way of
    walking the rows (seven of them, the last one short), so the result must be the oracle's bit for bit in both
    accumulation modes, sharded or not, and every piece must have been awaited exactly once."""
    n, dim, m, k, iters, seed = 1501, 8, 2, 24, 6, 7
    x = _int_rows(n, dim, 4, distinct=70)
    so = RecordingSeeder(seed)
    cb_o, it_o = oracle.pq_fit(x, m, k, iters, so.init_pq(n, m, k), so.draw)
    res = run_ranks(str(tmp_path), world, extra_env={"HOSTSIM_ACCUM": accum, "HOSTSIM_PIECES": "7"}, kind="pq", x=x, m=m, k=k,
                    iters=iters, seed=seed)
    for r in res:
        assert int(r["rc"]) == 0, str(r["error"])
        assert np.array_equal(r["codebooks"], cb_o) and np.array_equal(r["iterations"], it_o)
        assert by_stream(_draw_pairs(r)) == by_stream(so.draws)
        assert int(r["pieces_walked"]) == 7


def test_single_rank_host_loop_equals_oracle_on_float_rows(hostsim, oracle, tmp_path):
    """world = 1: the product's loop (ordered sums) against the oracle on ordinary float data, bit for bit."""
    from vq_b200 import synth
    x = synth.uniform01(700, 12, 9)
    so = RecordingSeeder(11)
    cb_o, it_o = oracle.pq_fit(x, 3, 16, 9, so.init_pq(700, 3, 16), so.draw)
    (r,) = run_ranks(str(tmp_path), 1, kind="pq", x=x, m=3, k=16, iters=9, seed=11)
    assert np.array_equal(r["codebooks"], cb_o) and np.array_equal(r["iterations"], it_o)


def test_pq_fit_sharded_float_rows_within_tolerance(hostsim, oracle, tmp_path):
    """Float rows: per-rank partial sums are added in a different order than the single-process sum, so the codebooks
    agree to rounding (<= 1e-3 relative per centroid after the first iteration, the accepted tolerance)."""
    from vq_b200 import synth
    x = synth.uniform01(4001, 8, 21)
    so = RecordingSeeder(2)
    init = so.init_pq(4001, 2, 8)
    cb_o, _ = oracle.pq_fit(x, 2, 8, 1, init, so.draw)
    res = run_ranks(str(tmp_path), 2, kind="pq", x=x, m=2, k=8, iters=1, seed=2)
    for r in res:
        rel = np.linalg.norm(r["codebooks"] - cb_o, axis=2) / np.linalg.norm(cb_o, axis=2)
        assert rel.max() <= 1e-3
    assert np.array_equal(res[0]["codebooks"], res[1]["codebooks"])  # ranks agree exactly with each other


def test_too_few_rows_is_reported_on_every_rank(hostsim, tmp_path):
    x = _int_rows(5, 4, 1)
    res = run_ranks(str(tmp_path), 2, kind="pq", x=x, m=2, k=9, iters=3, seed=0)
    for r in res:
        assert int(r["rc"]) == 2 and str(r["error"]) == "Invalid parameter: Not enough data points for k clusters"


def test_rvq_fit_sharded(hostsim, oracle, tmp_path):
    n, dim, stages, k = 600, 6, 3, 8
    x = _int_rows(n, dim, 8, hi=30)
    so = RecordingSeeder(4)
    cb_o, _res, _norms = oracle.rvq_fit(x, stages, k, 6, 0.01, oracle.EUCLIDEAN, so.init_stage, so.draw)
    res = run_ranks(str(tmp_path), 2, kind="rvq", x=x, stages=stages, k=k, iters=6, seed=4, epsilon=0.01)
    for r in res:
        assert int(r["rc"]) == 0 and int(r["stages"]) == cb_o.shape[0]
        assert np.array_equal(r["codebooks"][0], cb_o[0])          # stage 0 sums integer rows: exact
        assert np.allclose(r["codebooks"], cb_o, rtol=1e-3, atol=1e-3)  # later stages sum residuals: rounding only
    assert np.array_equal(res[0]["codebooks"], res[1]["codebooks"])


def test_opq_fit_sharded(hostsim, oracle, tmp_path):
    from vq_b200 import synth
    x = synth.correlated(900, 8, 3)
    so = RecordingSeeder(6)
    init = so.init_pq(900, 2, 8)
    rot_o, cb_o = oracle.opq_fit(x, 2, 8, 4, 2, oracle.EUCLIDEAN, init, so)
    res = run_ranks(str(tmp_path), 2, kind="opq", x=x, m=2, k=8, iters=4, outer=2, seed=6)
    for r in res:
        assert int(r["rc"]) == 0
        rot = r["rotation"]
        assert np.allclose(rot @ rot.T, np.eye(8), atol=1e-5)
        assert np.allclose(rot, rot_o, atol=5e-3)
    assert np.array_equal(res[0]["rotation"], res[1]["rotation"])


def test_jacobi_svd_against_numpy(hostsim):
    lib = C.CDLL(hostsim)
    rng = np.random.default_rng(0)
    for n, rank_def in ((1, False), (5, False), (32, False), (128, False), (16, True)):
        a = rng.normal(size=(n, n))
        if rank_def:
            a[:, 3] = a[:, 1]
            a[7] = 0
        u, s, v = np.zeros((n, n)), np.zeros(n), np.zeros((n, n))
        lib.hs_jacobi_svd(C.c_void_p(a.ctypes.data), C.c_size_t(n), C.c_void_p(u.ctypes.data), C.c_void_p(s.ctypes.data),
                          C.c_void_p(v.ctypes.data))
        assert np.allclose(u @ np.diag(s) @ v.T, a, atol=1e-10)
        assert np.allclose(u.T @ u, np.eye(n), atol=1e-10) and np.allclose(v.T @ v, np.eye(n), atol=1e-10)
        assert np.allclose(np.sort(s)[::-1], np.linalg.svd(a, compute_uv=False), atol=1e-10)
        if not rank_def:  # V U^T is invariant to the SVD's sign/ordering choices when singular values are distinct
            un, _sn, vtn = np.linalg.svd(a)
            assert np.allclose(v @ u.T, vtn.T @ un.T, atol=1e-8)
