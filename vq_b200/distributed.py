"""One-process-per-GPU plumbing: torch.distributed carries the rendezvous, NCCL (inside libvqb.so)
carries the per-iteration all-reduce of centroid sums and counts over NVLink."""
from __future__ import annotations

import os

from . import Context, unique_id


def shard_bounds(n_global: int, rank: int, world: int) -> tuple[int, int]:
    """Contiguous row block of `rank`: the first n % world ranks hold one extra row."""
    base, extra = divmod(int(n_global), int(world))
    begin = rank * base + min(rank, extra)
    return begin, begin + base + (1 if rank < extra else 0)


def owner_of(row: int, n_global: int, world: int) -> int:
    """Rank whose shard holds global row `row` under shard_bounds."""
    base, extra = divmod(int(n_global), int(world))
    edge = extra * (base + 1)
    if row < edge:
        return row // (base + 1)
    return extra + (row - edge) // base if base else world - 1


def init_comm(ctx: Context, group=None) -> Context:
    """Create the library's NCCL communicator across the ranks of an initialised torch.distributed job."""
    import torch.distributed as dist
    if not dist.is_initialized() or dist.get_world_size(group) == 1:
        return ctx
    rank, world = dist.get_rank(group), dist.get_world_size(group)
    box = [unique_id() if rank == 0 else None]
    dist.broadcast_object_list(box, src=0, group=group)
    ctx.init_comm(box[0], rank, world)
    return ctx


def env_rank_world() -> tuple[int, int, int]:
    return int(os.environ.get("RANK", "0")), int(os.environ.get("WORLD_SIZE", "1")), int(os.environ.get("LOCAL_RANK", "0"))
