"""World-size-2 gloo run of the trajectory sharding helpers (host logic; no GPU)."""

import os
import socket

import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from diff_gpt_b200.dist import gather_trajectories, shard_range


def test_shard_range_partitions_everything():
    for n in (1, 7, 100, 4096):
        for world in (1, 2, 3, 8):
            spans = [shard_range(n, r, world) for r in range(world)]
            assert spans[0][0] == 0 and sum(c for _, c in spans) == n
            for (a, c), (b, _) in zip(spans, spans[1:]):
                assert a + c == b
            assert max(c for _, c in spans) - min(c for _, c in spans) <= 1


def _fake_tokens(n_series, first, count, horizon):
    """Tokens that depend only on (series, GLOBAL trajectory id, step), like the keyed random stream."""
    s = torch.arange(n_series)[:, None, None]
    t = (first + torch.arange(count))[None, :, None]
    g = torch.arange(horizon)[None, None, :]
    return ((s * 1000003 + t * 7919 + g * 31) % 4096).to(torch.int32)


def _worker(rank, world, port, n_total, q):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        first, count = shard_range(n_total, rank, world)
        local = _fake_tokens(3, first, count, 5)
        full = gather_trajectories(local, n_total)
        q.put((rank, full.clone()))
        dist.barrier()
    finally:
        dist.destroy_process_group()


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def test_gathered_result_is_independent_of_world_size():
    for n_total in (8, 7):  # even split and a split that differs by one trajectory
        ctx = mp.get_context("spawn")
        q = ctx.Queue()
        port = _free_port()
        procs = [ctx.Process(target=_worker, args=(r, 2, port, n_total, q)) for r in range(2)]
        for p in procs:
            p.start()
        got = dict(q.get(timeout=120) for _ in range(2))
        for p in procs:
            p.join(timeout=60)
            assert p.exitcode == 0
        want = _fake_tokens(3, 0, n_total, 5)
        assert torch.equal(got[0], want) and torch.equal(got[1], want)


def test_single_process_passthrough():
    x = _fake_tokens(2, 0, 6, 4)
    assert gather_trajectories(x, 6) is x
