"""Trajectory sharding across the GPUs of one box.

Every rank holds a full weight replica and decodes a contiguous slice of the
trajectories of every series; trajectories never interact, so the data path has
no collective.  The only exchange is one all-gather of the sampled token streams
at the end (NCCL over NVLink on GPUs, gloo in the CPU tests).  Because the random
stream is keyed by the GLOBAL trajectory index, the gathered result is the same
for every world size.
"""

from __future__ import annotations

import torch
import torch.distributed as dist


def shard_range(n_items: int, rank: int, world: int) -> tuple[int, int]:
    """(first, count) of the contiguous slice of `n_items` owned by `rank`; slices differ by at most one."""
    assert 0 <= rank < world
    base, extra = divmod(n_items, world)
    first = rank * base + min(rank, extra)
    return first, base + (1 if rank < extra else 0)


def gather_trajectories(local: torch.Tensor, n_total: int, group=None) -> torch.Tensor:
    """All-gather per-rank token blocks (S, n_local, G) into (S, n_total, G), in rank order.

    Ranks may own slices that differ by one trajectory; blocks are padded to a common
    size for the collective and trimmed afterwards.
    """
    if not dist.is_available() or not dist.is_initialized():
        assert local.shape[1] == n_total
        return local
    world = dist.get_world_size(group)
    rank = dist.get_rank(group)
    S, n_local, G = local.shape
    assert n_local == shard_range(n_total, rank, world)[1]
    width = -(-n_total // world)
    block = local
    if n_local < width:
        pad = torch.zeros((S, width - n_local, G), dtype=local.dtype, device=local.device)
        block = torch.cat([local, pad], dim=1)
    out = [torch.empty((S, width, G), dtype=local.dtype, device=local.device) for _ in range(world)]
    dist.all_gather(out, block.contiguous(), group=group)
    parts = [out[r][:, : shard_range(n_total, r, world)[1]] for r in range(world)]
    return torch.cat(parts, dim=1)


def decode_sharded(engine, prompts, num_samples: int, group=None, **kwargs):
    """`Engine.generate_many` with the trajectories of every series split over the ranks of `group`.

    Returns (tokens, masks) of shape (S, num_samples, G) on every rank.
    """
    if dist.is_available() and dist.is_initialized():
        world, rank = dist.get_world_size(group), dist.get_rank(group)
    else:
        world, rank = 1, 0
    first, count = shard_range(num_samples, rank, world)
    toks, masks = engine.generate_many(prompts, count, traj_offset=first, **kwargs)
    return gather_trajectories(toks, num_samples, group), gather_trajectories(masks, num_samples, group)
