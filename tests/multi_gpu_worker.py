"""One rank of the 2-GPU product-quantizer test (launched by tests/test_gpu_multi.py with torchrun-style environment)."""
import os
import sys

import numpy as np
import torch
import torch.distributed as dist

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)

import vq_b200 as vq  # noqa: E402
from vq_b200 import synth  # noqa: E402
from vq_b200.distributed import init_comm, shard_bounds  # noqa: E402


def main():
    out_prefix = sys.argv[1]
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", device_id=torch.device("cuda", rank))
    ctx = init_comm(vq.Context(rank))
    n, dim, m, k = 40001, 32, 4, 64
    rng = np.random.default_rng(3)
    x_int = rng.integers(0, 40, (n, dim)).astype(np.float32)      # exact sums: sharded == single process, bit for bit
    x_flt = synth.uniform01(n, dim, 5)
    begin, end = shard_bounds(n, rank, world)
    res = {}
    for name, x, iters in (("int", x_int, 6), ("flt", x_flt, 1)):
        pq = vq.ProductQuantizer.fit(torch.from_numpy(x[begin:end]).cuda(), m, k, iters, vq.Distance.Euclidean, 9, ctx=ctx,
                                     accumulate=vq.ACCUM_FAST)
        res[f"cb_{name}"] = pq.codebooks
        res[f"it_{name}"] = pq.iterations
        out, codes = pq.quantize(torch.from_numpy(x[begin:end]).cuda(), return_codes=True)
        res[f"codes_{name}"] = codes.cpu().numpy()
    # 16-wide sub-spaces take the general assignment and update kernels
    pqw = vq.ProductQuantizer.fit(torch.from_numpy(x_int[begin:end]).cuda(), 2, k, 4, vq.Distance.Euclidean, 9, ctx=ctx, accumulate=vq.ACCUM_FAST)
    res["cb_wide"] = pqw.codebooks
    res["it_wide"] = pqw.iterations
    res["exchanges"] = np.int64(ctx.exchange_count())
    np.savez(f"{out_prefix}.rank{rank}.npz", begin=begin, end=end, **res)
    ctx.destroy_comm()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
