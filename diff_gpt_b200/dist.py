"""Trajectory sharding across the GPUs of one box.

Every rank holds a full weight replica and decodes a contiguous slice of the
trajectories of every series; trajectories never interact, so the data path has
no collective.  The only exchange is one all-gather of the sampled token streams
at the end (NCCL over NVLink on GPUs, gloo in the CPU tests).  Because the random
stream is keyed by the GLOBAL trajectory index, the gathered result is the same
for every world size.

Failure handling is host-side only.  A rank whose decode raised, or that is gone, must not leave the others
inside a collective: with a `store` (any torch.distributed key-value store shared by the ranks) every rank posts
"ready" or "failed" for the step after its local decode and reads the others' posts BEFORE the all-gather is
launched; a missing post within the time limit, or a "failed" post, raises `ShardFailure` on the healthy ranks,
which then have no kernel and no collective in flight.  No device-side wait is involved.
"""

from __future__ import annotations

import time

import torch
import torch.distributed as dist


class ShardFailure(RuntimeError):
    """Another rank reported a failure, or did not report at all within the time limit."""

    def __init__(self, message: str, ranks: list[int]) -> None:
        super().__init__(message)
        self.ranks = ranks


def post_failure(store, step_id: int, rank: int, message: str) -> None:
    """Tell the other ranks that this rank cannot take part in the gather of `step_id`."""
    store.set(f"dgpt/{step_id}/failed/{rank}", message[:500])


def rendezvous(store, step_id: int, rank: int, world: int, timeout_s: float = 60.0, poll_s: float = 0.02) -> None:
    """Post "ready" for `step_id` and return once every rank has; raise `ShardFailure` as soon as a rank has posted
    a failure, or when the time limit passes with ranks still silent.  Host code only: it reads and writes the store."""
    store.set(f"dgpt/{step_id}/ready/{rank}", "1")
    waiting = [r for r in range(world) if r != rank]
    deadline = time.monotonic() + timeout_s
    while waiting:
        for r in list(waiting):
            if store.check([f"dgpt/{step_id}/failed/{r}"]):
                why = store.get(f"dgpt/{step_id}/failed/{r}").decode(errors="replace")
                raise ShardFailure(f"rank {r} failed in step {step_id}: {why}", [r])
            if store.check([f"dgpt/{step_id}/ready/{r}"]):
                waiting.remove(r)
        if waiting:
            if time.monotonic() > deadline:
                raise ShardFailure(f"ranks {waiting} did not reach step {step_id} within {timeout_s} s", list(waiting))
            time.sleep(poll_s)


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
    width = max(1, -(-n_total // world))
    block = local
    if n_local < width:
        pad = torch.zeros((S, width - n_local, G), dtype=local.dtype, device=local.device)
        block = torch.cat([local, pad], dim=1)
    out = [torch.empty((S, width, G), dtype=local.dtype, device=local.device) for _ in range(world)]
    dist.all_gather(out, block.contiguous(), group=group)
    parts = [out[r][:, : shard_range(n_total, r, world)[1]] for r in range(world)]
    return torch.cat(parts, dim=1)


def decode_sharded(engine, prompts, num_samples: int, group=None, store=None, step_id: int = 0,
                   timeout_s: float = 60.0, **kwargs):
    """`Engine.generate_many` with the trajectories of every series split over the ranks of `group`.

    Returns (tokens, masks) of shape (S, num_samples, G) on every rank.  With a `store`, the ranks meet on the host
    (`rendezvous`) between the local decode and the all-gather: a rank whose decode raised posts the failure and
    re-raises, the others raise `ShardFailure` instead of entering the collective.  Use a fresh `step_id` per call.
    """
    if dist.is_available() and dist.is_initialized():
        world, rank = dist.get_world_size(group), dist.get_rank(group)
    else:
        world, rank = 1, 0
    first, count = shard_range(num_samples, rank, world)
    # every rank takes the attention path the unsharded job would take, whatever its own share is (the two paths
    # round differently, so the choice must not depend on the world size)
    from .model.engine import SHARED_PREFIX_MIN_ROWS

    kwargs.setdefault("shared_prefix", num_samples >= SHARED_PREFIX_MIN_ROWS)
    # every rank decodes other trajectories of the same prompts: prefill each prompt on one rank only and exchange the
    # prompt K/V (needs every rank in the call, so only when none of them is left without trajectories)
    if world > 1 and num_samples >= world and len(prompts) % world == 0:
        kwargs.setdefault("prefill_group", group if group is not None else dist.group.WORLD)
    if store is None or world == 1:
        toks, masks = engine.generate_many(prompts, count, traj_offset=first, **kwargs)
    else:
        try:
            toks, masks = engine.generate_many(prompts, count, traj_offset=first, **kwargs)
            if toks.is_cuda:
                torch.cuda.synchronize(toks.device)  # device-side problems surface here, before the others are told "ready"
        except Exception as exc:
            post_failure(store, step_id, rank, f"{type(exc).__name__}: {exc}")
            raise
        rendezvous(store, step_id, rank, world, timeout_s)
    return gather_trajectories(toks, num_samples, group), gather_trajectories(masks, num_samples, group)
