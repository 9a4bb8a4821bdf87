#!/usr/bin/env python
"""Benchmark of the quantizer hot path: product-quantizer training + encode at README scale.

Workload (the reference README's scale): 1,000,000 x 128 f32 rows, i.i.d. uniform [0,1) from seed 7 (synthetic
stand-in for the reference's StdRng-generated evaluation data, src/bin/utils.rs:31-41), m=16, k=256,
10 LBG iterations on all rows, then encode all rows to f16 (src/bin/eval_pq.rs:40-60 is what is timed).
One step = one fit + one encode.  With N > 1 the same 1M rows are sharded over the ranks (strong scaling),
one NCCL all-reduce of centroid sums/counts per LBG iteration.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--rows R]

Prints ONE JSON line (rank 0).  `value` is timed with CUDA events on device-resident inputs; `e2e` goes through
the same public API with pinned HOST buffers (copies inside the timed region).  `--impl reference` times the
CPU restatement of the reference (oracle/, all host threads) on a bounded row sample of the same workload.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

N_ROWS, DIM, M, K, ITERS = 1_000_000, 128, 16, 256, 10
DATA_SEED, FIT_SEED = 7, 42
METRIC_NAME, UNIT = "pq_fit_plus_encode_throughput", "Mvec/s"
# algorithmic bytes per vector (what must cross HBM): training pass = 512 B row + 16 B old codes + 16 B new codes;
# encode = 512 B row + 256 B f16 output.
TRAIN_BYTES_PER_VEC, ENCODE_BYTES_PER_VEC = 544, 768
# DRAM traffic per launch measured with ncu (dram__bytes_read.sum + dram__bytes_write.sum): assign_train = pq_tc_kernel,
# 530.6 B read + 27 B written per row on a 262144-row capture, scaled to 1M rows (traffic grows with the rows: every row
# is read once); the encode launch was not captured.
NCU_TRAFFIC_BYTES = {"assign_train": 558.0e6, "pq_encode": None}


def workload_config(rows: int, world: int) -> dict:
    """The workload both arms report: same keys, same values."""
    return {"workload": "pq_1m_x128_m16_k256_10iters_fit_plus_encode", "rows": rows, "dim": DIM, "m": M, "k": K,
            "lbg_iters": ITERS, "distance": "Euclidean", "parallelism": f"rows sharded over {world} GPU(s)",
            "l2": "256 MiB flush write before every step; the 512 MB row matrix exceeds L2 at N=1"}


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            d = json.load(f)
        return float(d["hbm_gbs"]), "measured"
    return 6650.0, "fallback"


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""

    FIELDS = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index, self.proc, self.lines = index, None, []

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--id={self.index}", f"--query-gpu={self.FIELDS}",
                                          "--format=csv,noheader,nounits", "-lms", "200"],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._pump, daemon=True)
            self.thread.start()
        except Exception:
            self.proc = None

    def _pump(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def stop(self) -> dict:
        if not self.proc:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.25)
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            self.proc.kill()
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for line in self.lines:
            parts = [p.strip() for p in line.split(",")]
            if len(parts) < 6:
                continue
            try:
                sm.append(float(parts[0]))
                mx.append(float(parts[1]))
            except ValueError:
                continue
            for name, val in zip(names, parts[2:6]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": sorted(reasons), "samples": len(sm)}


def cpu_reference(rows: int, steps: int, warmup: int, x=None):
    """The reference's algorithm on the host cores: oracle/ (C restatement, OpenMP over points, all threads)."""
    import oracle
    from vq_b200 import synth
    from vq_b200.seeding import LbgSeeder
    oracle.build()
    oracle.use_all_host_threads()
    if x is None:
        x = synth.uniform01(rows, DIM, DATA_SEED)
    times = []
    for it in range(warmup + steps):
        seeder = LbgSeeder(FIT_SEED)
        init = np.stack([seeder.init_indices(i, rows, K) for i in range(M)])
        t0 = time.perf_counter()
        cb, _ = oracle.pq_fit(x, M, K, ITERS, init, seeder.draw)
        t1 = time.perf_counter()
        oracle.pq_quantize(cb, x, oracle.EUCLIDEAN)
        t2 = time.perf_counter()
        if it >= warmup:
            times.append((t1 - t0, t2 - t1))
    fit_s = sum(t[0] for t in times) / len(times)
    enc_s = sum(t[1] for t in times) / len(times)
    return {"value": rows / (fit_s + enc_s) / 1e6, "unit": UNIT, "cores": oracle.num_threads(), "kind": "port",
            "sample": (f"all {rows} rows, full algorithm (10 LBG iterations + encode), {len(times)} run(s)" if rows == N_ROWS else
                       f"{rows} of {N_ROWS} rows, full algorithm (10 LBG iterations + encode), scaled per vector"),
            "train_s_per_1m_rows": fit_s * N_ROWS / rows, "encode_mvec_per_s": rows / enc_s / 1e6}


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    rows = args.rows or N_ROWS  # the whole workload: about 6 s per step on 16 host threads
    cb = cpu_reference(rows, max(1, args.steps), max(0, min(args.warmup, 1)))
    step_s = rows / (cb["value"] * 1e6)
    line = {"impl": "reference", "metric": METRIC_NAME, "value": cb["value"], "unit": UNIT, "n_gpus": args.gpus,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": step_s * 1e3, "higher_is_better": True,
            "scaling": "strong", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": workload_config(N_ROWS, args.gpus), "rows_timed": rows,
            "cpu_baseline": cb,
            "e2e": {"value": cb["value"], "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
            "gpu_launches": 0}
    print(json.dumps(line), flush=True)


def full_size_parity(vq, ctx, dist, rank, world, x_dev, x_host, begin, n_local, n_global, init, pq10, out10):
    """The parity figures at the benchmark's own size, outside every timed region (reported, never timed):
    centroid error after one iteration against the oracle on all rows, final-MSE ratio with 10-iteration codebooks, code
    mismatches and near-ties on >= 100,000 rows given identical codebooks, and (N > 1) bit-identical codebooks on all ranks.
    Rank 0 also times the oracle's full-size fit + encode it needs for this: that is the CPU baseline."""
    import torch
    from vq_b200 import synth
    from vq_b200.seeding import LbgSeeder

    # every rank: one library iteration from the same initial rows (a collective when sharded)
    seeder = LbgSeeder(FIT_SEED)
    for i in range(M):
        seeder.init_indices(i, n_global, K)
    pq1 = vq.ProductQuantizer.fit(x_dev, M, K, 1, vq.Distance.Euclidean, FIT_SEED, ctx=ctx, init_idx=init, draw=seeder.draw)
    cb1, cb10 = pq1.codebooks, pq10.codebooks
    identical = None
    if world > 1:  # every rank must hold the same bits
        digest = torch.tensor([int(np.frombuffer(cb10.tobytes(), dtype=np.uint32).astype(np.uint64).sum() & 0x7FFFFFFFFFFFFFFF),
                               int(np.bitwise_xor.reduce(np.frombuffer(cb10.tobytes(), dtype=np.uint32)))], dtype=torch.int64, device="cuda")
        lo, hi = digest.clone(), digest.clone()
        dist.all_reduce(lo, op=dist.ReduceOp.MIN)
        dist.all_reduce(hi, op=dist.ReduceOp.MAX)
        identical = bool(torch.equal(lo, hi))
    if rank != 0:
        return None, None
    try:
        import oracle
        oracle.build()
        oracle.use_all_host_threads()
        x_all = x_host.numpy() if world == 1 else synth.uniform01(n_global, DIM, DATA_SEED)
        s1 = LbgSeeder(FIT_SEED)
        for i in range(M):
            s1.init_indices(i, n_global, K)
        ocb1, _ = oracle.pq_fit(x_all, M, K, 1, init, s1.draw)
        rel = np.linalg.norm(cb1.astype(np.float64) - ocb1, axis=2) / np.maximum(np.linalg.norm(ocb1.astype(np.float64), axis=2), 1e-30)
        s10 = LbgSeeder(FIT_SEED)
        for i in range(M):
            s10.init_indices(i, n_global, K)
        t0 = time.perf_counter()
        ocb10, _ = oracle.pq_fit(x_all, M, K, ITERS, init, s10.draw)
        t1 = time.perf_counter()
        o16_all, _codes_all = oracle.pq_quantize(ocb10, x_all, oracle.EUCLIDEAN)
        t2 = time.perf_counter()
        shard = x_all[begin:begin + n_local]
        mse_oracle = oracle.mse_f16(shard, o16_all[begin:begin + n_local])
        lib16 = out10.cpu().numpy() if hasattr(out10, "cpu") else np.asarray(out10)
        mse_lib = oracle.mse_f16(shard, lib16.view(np.uint16))
        # identical codebooks (the library's), >= 100,000 rows: codes must agree outside near-ties
        rows = min(n_local, 131072)
        sample = shard[:rows]
        _o, codes_o = oracle.pq_quantize(cb10, sample, oracle.EUCLIDEAN)
        _g, codes_g = pq10.quantize(sample, return_codes=True)
        mism = int((codes_o != np.asarray(codes_g)).sum())
        near = 0
        sd = DIM // M
        for s_ in range(M):  # the oracle's two smallest distances per (row, sub-space), relative gap < 1e-6
            xs = sample[:, s_ * sd:(s_ + 1) * sd].astype(np.float64)
            cs = cb10[s_].astype(np.float64)
            d = (xs * xs).sum(1)[:, None] - 2.0 * xs @ cs.T + (cs * cs).sum(1)[None, :]
            two = np.partition(d, 1, axis=1)[:, :2]
            near += int(((two[:, 1] - two[:, 0]) < 1e-6 * np.maximum(two[:, 1], 1e-30)).sum())
        parity = {"centroid_rel_err_iter1": float(rel.max()), "centroid_rel_err_bar": 1e-3,
                  "mse_library": float(mse_lib), "mse_oracle": float(mse_oracle), "mse_ratio": float(mse_lib / mse_oracle), "mse_ratio_bar": "within 1 %",
                  "code_rows": rows, "code_mismatches": mism, "near_ties": near,
                  "codebooks_identical_on_all_ranks": identical, "rows_fitted_by_oracle": int(n_global)}
        cpu = {"value": n_global / ((t1 - t0) + (t2 - t1)) / 1e6, "unit": UNIT, "cores": oracle.num_threads(), "kind": "port",
               "variant": "tight (contiguous rows, no allocation per distance, one-pass gather)",
               "sample": f"all {n_global} rows, full algorithm (10 LBG iterations + encode), one run",
               "train_s_per_1m_rows": (t1 - t0) * N_ROWS / n_global, "encode_mvec_per_s": n_global / (t2 - t1) / 1e6}
        if world == 1:  # the same fit with the reference's memory behaviour, on a bounded sample (it is several times slower)
            fr = 16384
            sf = LbgSeeder(FIT_SEED)
            init_f = np.stack([sf.init_indices(i, fr, K) for i in range(M)])
            tf0 = time.perf_counter()
            oracle.pq_fit_faithful(x_all[:fr], M, K, ITERS, init_f, sf.draw)
            tf = time.perf_counter() - tf0
            cpu["faithful"] = {"variant": "faithful (a heap allocation per row and per distance2, O(n k) gather with cloned members)",
                               "sample": f"{fr} of {n_global} rows, 10 LBG iterations, scaled per vector",
                               "train_s_per_1m_rows": tf * N_ROWS / fr}
        return parity, cpu
    except Exception as exc:  # the oracle is only a checker; the bench line survives without it
        return {"error": f"{type(exc).__name__}: {exc}"[:200], "codebooks_identical_on_all_ranks": identical}, None


def run_ours(args):
    import torch
    import torch.distributed as dist

    import vq_b200 as vq
    from vq_b200 import synth
    from vq_b200.distributed import init_comm, shard_bounds
    from vq_b200.seeding import LbgSeeder

    rank, world = int(os.environ.get("RANK", "0")), int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: vq_b200 has no CPU path (use --impl reference for the CPU baseline)")
    torch.cuda.set_device(local)
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    n_global = args.rows or N_ROWS
    begin, end = shard_bounds(n_global, rank, world)
    n_local = end - begin

    # inputs: this rank's shard in pinned host memory (for the end-to-end leg) and resident in HBM (for `value`)
    x_host = torch.empty((n_local, DIM), dtype=torch.float32, pin_memory=True)
    synth.uniform01(n_local, DIM, DATA_SEED, out=x_host.numpy(), row0=begin)
    x_dev = x_host.cuda(non_blocking=False)
    out_host = torch.empty((n_local, DIM), dtype=torch.float16, pin_memory=True)

    ctx = vq.Context(local)
    init_comm(ctx)
    stream = torch.cuda.current_stream()
    ctx.use_stream(stream.cuda_stream)
    seeder0 = LbgSeeder(FIT_SEED)
    init = np.stack([seeder0.init_indices(i, n_global, K) for i in range(M)])
    flush = torch.empty(256 << 20, dtype=torch.uint8, device="cuda")  # > 126 MB L2

    def one_step(x, timed):
        seeder = LbgSeeder(FIT_SEED)
        for i in range(M):
            seeder.init_indices(i, n_global, K)
        flush.fill_(1)
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()
        e0, e1, e2 = (torch.cuda.Event(enable_timing=True) for _ in range(3))
        e0.record(stream)
        pq = vq.ProductQuantizer.fit(x, M, K, ITERS, vq.Distance.Euclidean, FIT_SEED, ctx=ctx, init_idx=init,
                                     draw=seeder.draw)
        e1.record(stream)
        if isinstance(x, np.ndarray):
            lib_out = out_host.numpy()
            rc = vq._lib.load().vqb_pq_quantize(pq._h, x.ctypes.data, n_local, DIM, lib_out.ctypes.data, None)
            assert rc == 0
            out = out_host
        else:
            out = pq.quantize(x)
        e2.record(stream)
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        return e0.elapsed_time(e1) / 1e3, e1.elapsed_time(e2) / 1e3, pq, out

    def max_over_ranks(v):
        if world == 1:
            return v
        t = torch.tensor([v], dtype=torch.float64, device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    pq = out = None
    for _ in range(max(3, args.warmup)):
        # results are held exactly as in the timed loop, so that the caller-side allocator (torch's cache: two 256 MB
        # output blocks alternate) is warm as well and no cudaMalloc lands inside a timed step
        _f, _e, pq, out = one_step(x_dev, False)

    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
    launches0 = ctx.launch_count()
    fit_s, enc_s = [], []
    for _ in range(args.steps):  # the loop behind `value`: no per-kernel events in it
        f, e, pq, out = one_step(x_dev, True)
        fit_s.append(max_over_ranks(f))
        enc_s.append(max_over_ranks(e))
        if os.environ.get("VQB_BENCH_DEBUG"):
            print(f"[rank {rank}] fit {f * 1e3:.3f} ms encode {e * 1e3:.3f} ms", file=sys.stderr, flush=True)
    launches = ctx.launch_count() - launches0
    clocks = sampler.stop() if rank == 0 else {}

    # per-kernel breakdown (roofline inputs): the same steps again with CUDA events around every launch
    ctx.timing(True)
    ctx.timing_report()
    breakdown_steps = max(1, min(5, args.steps))
    for _ in range(breakdown_steps):
        one_step(x_dev, True)
    kernels = ctx.timing_report()
    ctx.timing(False)
    for v in kernels.values():
        v["launches_per_step"] = v["launches"] / breakdown_steps
        v["ms_per_step"] = v["ms"] / breakdown_steps

    # end to end: same public API, pinned host buffers in, host f16 out; copies inside the timed region
    e2e_s = []
    for i in range(0 if args.kernels_only else 1 + min(3, args.steps)):
        f, e, _pq, _o = one_step(x_host.numpy(), True)
        if i > 0:
            e2e_s.append(max_over_ranks(f + e))

    parity, cpu = None, None
    if not args.kernels_only:
        parity, cpu = full_size_parity(vq, ctx, dist, rank, world, x_dev, x_host, begin, n_local, n_global, init, pq, out)

    if rank != 0:
        if world > 1:
            dist.destroy_process_group()
        return

    train_s = sum(fit_s) / len(fit_s)
    encode_s = sum(enc_s) / len(enc_s)
    step_s = train_s + encode_s
    value = n_global / step_s / 1e6
    peak, peak_kind = measured_peaks()

    def roof(name, bytes_per_vec):
        k = kernels.get(name)
        if not k or not k["launches"]:
            return None
        avg_s = k["ms"] / k["launches"] / 1e3
        achieved = bytes_per_vec * n_local / avg_s / 1e9
        return {"bound": "hbm", "kernel": name, "achieved": achieved, "peak": peak, "peak_kind": peak_kind, "unit": "GB/s",
                "frac": achieved / peak,
                "traffic": (NCU_TRAFFIC_BYTES[name] * n_local / N_ROWS) if NCU_TRAFFIC_BYTES.get(name) else None,  # scales with the rows of this rank
                "launches": k["launches"],
                "avg_ms": avg_s * 1e3, "algorithmic_bytes_per_launch": bytes_per_vec * n_local,
                "fp32_ops_per_launch": n_local * M * K * (DIM // M) * 3}

    dominant = max(kernels, key=lambda kname: kernels[kname]["ms"]) if kernels else None
    roofline = roof("assign_train", TRAIN_BYTES_PER_VEC)
    if world > 1:
        cpu = None  # the CPU baseline is reported by rank 0 at N=1 only
    e2e_step = sum(e2e_s) / len(e2e_s) if e2e_s else float("nan")
    line = {
        "metric": METRIC_NAME, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps, "warmup": max(3, args.warmup),
        "ms_per_step": step_s * 1e3, "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
        "dtype": "f32", "data": "synthetic",
        "config": workload_config(n_global, world),
        "train_s": train_s, "encode_s": encode_s, "encode_mvec_per_s": n_global / encode_s / 1e6,
        "roofline": roofline, "roofline_encode": roof("pq_encode", ENCODE_BYTES_PER_VEC),
        "dominant_kernel": dominant, "kernels": kernels, "kernels_note": f"separate pass of {breakdown_steps} step(s) with CUDA events around every launch",
        "cpu_baseline": cpu,
        "e2e": {"value": n_global / e2e_step / 1e6, "unit": UNIT,
                "h2d_bytes_per_step": 2 * n_local * DIM * 4 + int(init.nbytes), "d2h_bytes_per_step": n_local * DIM * 2 + ITERS * (M * K + M) * 4,
                "ms_per_step": e2e_step * 1e3},
        "gpu_launches": launches, "clocks": clocks, "parity": parity,
        "exchange": (None if world == 1 else
                     "per-rank sums added inside the centroid-update kernel over peer memory" if ctx.exchange_count() > 0 else
                     "one NCCL all-reduce per iteration"),
        "published_reference": {"train_s": 232.5, "encode_s": 34.1, "hardware": "i7-1355U laptop (README)"},
    }
    print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


def run_secondary(args):
    """The other benchmark configurations on one GPU (measurement aid; the headline line is the default workload).
    sq / bq: 10,000,000 x 128 values in [-1,1), SQ [0,1] x 256 levels, BQ threshold 0.
    rvq: 1,000,000 x 128 Gaussian mixture (64 components, sigma 0.05), 8 stages, k=256, 10 iterations, Euclidean.
    opq: 1,000,000 x 128 correlated rows, m=16, k=256, 10 outer x 5 LBG iterations.
    tsvq: 1,000,000 x 128 uniform rows, depth 10, Euclidean (build + lookup of every row)."""
    import torch

    import vq_b200 as vq
    from vq_b200 import synth

    torch.cuda.set_device(0)
    ctx = vq.Context(0)
    stream = torch.cuda.current_stream()
    ctx.use_stream(stream.cuda_stream)
    peak, peak_kind = measured_peaks()
    flush = torch.empty(256 << 20, dtype=torch.uint8, device="cuda")
    w = args.workload
    rows = args.rows or (10_000_000 if w in ("sq", "bq") else 1_000_000)

    def timed(fn):
        flush.fill_(1)
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(stream)
        out = fn()
        e1.record(stream)
        torch.cuda.synchronize()
        return e0.elapsed_time(e1) / 1e3, out

    sampler = ClockSampler(0)
    extra = {}
    if w in ("sq", "bq"):
        g = torch.Generator(device="cuda")
        g.manual_seed(1)
        x = torch.empty((rows, DIM), device="cuda", dtype=torch.float32)
        x.uniform_(-1.0, 1.0, generator=g)
        q = vq.ScalarQuantizer.fit(0.0, 1.0, 256, ctx=ctx) if w == "sq" else vq.BinaryQuantizer.fit(0.0, 0, 1, ctx=ctx)
        step = lambda: q.quantize(x)  # noqa: E731
        kname, bytes_per_vec, cfg = f"{w}_quantize", 5 * DIM, f"{w}_10m_x128"
        host = synth.uniform(1 << 20, DIM, 1, -1.0, 1.0)
        import oracle
        oracle.use_all_host_threads()
        t0 = time.perf_counter()
        for _ in range(3):
            (oracle.sq_quantize(0.0, 1.0, 256, q.step, host) if w == "sq" else oracle.bq_quantize(0.0, 0, 1, host))
        cpu = {"value": 3 * host.shape[0] / (time.perf_counter() - t0) / 1e6, "unit": UNIT, "cores": oracle.num_threads(),
               "kind": "port", "variant": "rows in parallel (benches/bench_sq.rs:91-94)", "sample": f"{host.shape[0]} rows x 128, 3 passes"}
        # the reference's evaluation binary walks the rows in a serial loop (src/bin/eval_sq.rs:45-46): one host thread
        oracle.lib().vqo_set_num_threads(1)
        t0 = time.perf_counter()
        (oracle.sq_quantize(0.0, 1.0, 256, q.step, host) if w == "sq" else oracle.bq_quantize(0.0, 0, 1, host))
        cpu["serial_outer_loop"] = {"value": host.shape[0] / (time.perf_counter() - t0) / 1e6, "unit": UNIT, "cores": 1,
                                    "sample": f"{host.shape[0]} rows x 128, 1 pass"}
        oracle.use_all_host_threads()
        xp = torch.empty((min(rows, 2_000_000), DIM), dtype=torch.float32, pin_memory=True)
        xp.copy_(x[: xp.shape[0]])
        out_pinned = torch.empty(tuple(xp.shape), dtype=torch.uint8, pin_memory=True)
        e2e_fn = lambda: q.quantize(xp.numpy(), out=out_pinned.numpy())  # noqa: E731  (page-locked buffers in and out)
        e2e_rows, h2d, d2h = xp.shape[0], xp.numel() * 4, xp.numel()
    else:
        import oracle
        from vq_b200.seeding import LbgSeeder
        oracle.use_all_host_threads()
        sample_rows = min(rows, 65536)  # bounded CPU sample, scaled per vector (the cost per vector does not depend on n)
        if w == "rvq":
            xh = synth.gaussian_mixture(rows, DIM, 11)
            fit = lambda xx: vq.ResidualQuantizer.fit(xx, 8, K, ITERS, 0.01, vq.Distance.Euclidean, FIT_SEED, ctx=ctx)  # noqa: E731
            # full-width passes: the shortlist kernel reads every row once (512 B) plus its norm and writes the candidate mask
            kname, bytes_per_vec, cfg = "dense_shortlist", 512 + 4 + 32, "rvq_1m_x128_8stages_k256_10iters_fit_plus_encode"

            def cpu_run(xs):
                sd_ = LbgSeeder(FIT_SEED)
                t0 = time.perf_counter()
                cb, _r, _n = oracle.rvq_fit(xs, 8, K, ITERS, 0.01, oracle.EUCLIDEAN, sd_.init_indices, sd_.draw)
                t1 = time.perf_counter()
                oracle.rvq_quantize(cb, 0.01, xs, oracle.EUCLIDEAN)
                return t1 - t0, time.perf_counter() - t1
        elif w == "tsvq":
            xh = synth.uniform01(rows, DIM, 1)
            fit = lambda xx: vq.TSVQ(xx, 10, vq.Distance.Euclidean, ctx=ctx)  # noqa: E731  (depth 10: benches/bench_tsvq.rs:11)
            kname, bytes_per_vec, cfg = "tsvq_node_spreads", 512, "tsvq_1m_x128_depth10_fit_plus_encode"

            def cpu_run(xs):
                t0 = time.perf_counter()
                cen, left, right = oracle.tsvq_fit(xs, 10)
                t1 = time.perf_counter()
                oracle.tsvq_quantize(cen, left, right, xs, oracle.EUCLIDEAN)
                return t1 - t0, time.perf_counter() - t1
        else:
            xh = synth.correlated(rows, DIM, 3)
            fit = lambda xx: vq.OptimizedProductQuantizer.fit(xx, M, K, 5, 10, vq.Distance.Euclidean, FIT_SEED, ctx=ctx)  # noqa: E731
            kname, bytes_per_vec, cfg = "assign_train", TRAIN_BYTES_PER_VEC, "opq_1m_x128_m16_k256_10outer_x_5iters_fit_plus_encode"

            def cpu_run(xs):
                sd_ = LbgSeeder(FIT_SEED)
                init_ = np.stack([sd_.init_indices(i, xs.shape[0], K) for i in range(M)])
                t0 = time.perf_counter()
                rot, cb = oracle.opq_fit(xs, M, K, 5, 10, oracle.EUCLIDEAN, init_, sd_.draw)
                t1 = time.perf_counter()
                oracle.opq_quantize(rot, cb, xs, oracle.EUCLIDEAN)
                return t1 - t0, time.perf_counter() - t1
        x = torch.from_numpy(xh).cuda()
        xp = torch.empty((rows, DIM), dtype=torch.float32, pin_memory=True)
        xp.copy_(torch.from_numpy(xh))

        def step():
            t_fit, qz = timed(lambda: fit(x))
            t_enc, out = timed(lambda: qz.quantize(x))
            extra["train_s"], extra["encode_s"] = t_fit, t_enc
            return out

        out_pinned = torch.empty((rows, DIM), dtype=torch.float16, pin_memory=True)

        def e2e_fn():  # page-locked host rows in, page-locked host f16 out, through the same public calls
            qz = fit(xp.numpy())
            return qz.quantize(xp.numpy(), out=out_pinned.numpy())
        cpu_fit, cpu_enc = cpu_run(np.ascontiguousarray(xh[:sample_rows]))
        cpu = {"value": sample_rows / (cpu_fit + cpu_enc) / 1e6, "unit": UNIT, "cores": oracle.num_threads(), "kind": "port",
               "sample": f"{sample_rows} of {rows} rows, full algorithm, scaled per vector",
               "train_s_per_1m_rows": cpu_fit * 1e6 / sample_rows, "encode_mvec_per_s": sample_rows / cpu_enc / 1e6}
        e2e_rows, h2d, d2h = rows, 2 * rows * DIM * 4, rows * DIM * 2

    heavy = w in ("rvq", "opq", "tsvq")
    for _ in range(max(1, min(3, args.warmup)) if heavy else max(3, args.warmup)):
        step()
    sampler.start()
    l0 = ctx.launch_count()
    times = []
    for _ in range(args.steps):  # the loop behind `value`: no per-kernel events in it
        if not heavy:
            t, _o = timed(step)
        else:
            step()
            t = extra["train_s"] + extra["encode_s"]
        times.append(t)
    launches = ctx.launch_count() - l0
    clocks = sampler.stop()
    ctx.timing(True)  # per-kernel breakdown in a pass of its own
    ctx.timing_report()
    timed(step) if not heavy else step()
    kernels = ctx.timing_report()
    ctx.timing(False)
    step_s = sum(times) / len(times)
    e2e = None
    if e2e_fn is not None and not args.kernels_only:
        ts = [timed(e2e_fn)[0] for _ in range(2 if heavy else 4)][1:]
        e2e = {"value": e2e_rows / (sum(ts) / len(ts)) / 1e6, "unit": UNIT, "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
               "rows": e2e_rows}
    kk = kernels.get(kname)
    roofline = None
    if kk and kk["launches"]:
        avg = kk["ms"] / kk["launches"] / 1e3
        ach = bytes_per_vec * rows / avg / 1e9
        roofline = {"bound": "hbm", "kernel": kname, "achieved": ach, "peak": peak, "peak_kind": peak_kind, "unit": "GB/s",
                    "frac": ach / peak, "traffic": None, "launches": kk["launches"], "avg_ms": avg * 1e3}
    line = {"metric": f"{w}_throughput", "value": rows / step_s / 1e6, "unit": UNIT, "n_gpus": 1, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": step_s * 1e3, "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "f32",
            "data": "synthetic", "config": {"workload": cfg, "rows": rows, "dim": DIM, "l2": "256 MiB flush write before every timed call"},
            "roofline": roofline, "kernels": kernels, "cpu_baseline": cpu, "e2e": e2e, "gpu_launches": launches, "clocks": clocks, **extra}
    print(json.dumps(line), flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--workload", default="pq", choices=["pq", "sq", "bq", "rvq", "opq", "tsvq"],
                    help="pq (default) is the headline benchmark; the others measure the remaining configurations on one GPU")
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--kernels-only", action="store_true",
                    help="skip the end-to-end and CPU-baseline legs (for profiler captures; not a valid bench line)")
    ap.add_argument("--rows", type=int, default=0, help="override the row count (default: 1,000,000; reference arm: 32768-row sample)")
    args = ap.parse_args()
    if args.workload != "pq":
        run_secondary(args)
    elif args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
