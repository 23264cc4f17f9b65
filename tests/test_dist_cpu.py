"""World-size-2 gloo run of the trajectory sharding helpers (host logic; no GPU)."""

import os
import socket

import torch
import torch.distributed as dist
import torch.multiprocessing as mp

import datetime
import time

import pytest

from diff_gpt_b200.dist import ShardFailure, decode_sharded, gather_trajectories, rendezvous, shard_range


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
    try:
        dist.init_process_group("gloo", rank=rank, world_size=world, timeout=datetime.timedelta(seconds=60))
    except Exception as e:  # the port was taken between choosing it and binding it: the test picks another
        q.put((rank, repr(e)))
        return
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
        for attempt in range(3):
            q = ctx.Queue()
            port = _free_port()
            procs = [ctx.Process(target=_worker, args=(r, 2, port, n_total, q)) for r in range(2)]
            for p in procs:
                p.start()
            got = dict(q.get(timeout=180) for _ in range(2))
            for p in procs:
                p.join(timeout=120)
                assert p.exitcode == 0, (p.exitcode, got)
            if not any(isinstance(v, str) for v in got.values()):
                break
        want = _fake_tokens(3, 0, n_total, 5)
        assert torch.equal(got[0], want) and torch.equal(got[1], want)


def test_single_process_passthrough():
    x = _fake_tokens(2, 0, 6, 4)
    assert gather_trajectories(x, 6) is x


# ---- failures, made on the host: a rank that raises, a rank that leaves, a collective whose peer never comes ----
class _FakeEngine:
    """Stands in for Engine.generate_many on CPU: tokens keyed by global trajectory id, or an exception."""

    def __init__(self, fail: bool) -> None:
        self.fail = fail
        self.calls = []

    def generate_many(self, prompts, count, traj_offset=0, **kwargs):
        self.calls.append((count, traj_offset, kwargs.get("shared_prefix")))
        self.prefill_group = kwargs.get("prefill_group")
        if self.fail:
            raise RuntimeError("device-side status 2: a bounded wait ran out")
        t = _fake_tokens(len(prompts), traj_offset, count, 4)
        return t, torch.ones_like(t)


def _failure_worker(rank, world, port, mode, q):
    store = dist.TCPStore("127.0.0.1", port, world, is_master=(rank == 0), timeout=datetime.timedelta(seconds=30))
    dist.init_process_group("gloo", store=store, rank=rank, world_size=world, timeout=datetime.timedelta(seconds=4))
    out = ("ok", None)
    try:
        t0 = time.monotonic()
        try:
            if mode == "raises":  # rank 1's decode raises: it posts the failure; rank 0 must not enter the gather
                eng = _FakeEngine(fail=(rank == 1))
                toks, _ = decode_sharded(eng, [[1, 2], [3]], 24, store=store, step_id=7, timeout_s=20.0)
                out = ("gathered", toks.shape)
            elif mode == "leaves":  # step 0 completes on both; rank 1 then leaves between steps without a word
                eng = _FakeEngine(fail=False)
                toks, _ = decode_sharded(eng, [[1, 2]], 10, store=store, step_id=0, timeout_s=20.0)
                assert torch.equal(toks, _fake_tokens(1, 0, 10, 4))
                if rank == 1:
                    q.put((rank, ("left", None), 0.0))
                    return
                decode_sharded(eng, [[1, 2]], 10, store=store, step_id=1, timeout_s=1.5)
                out = ("gathered", None)
            elif mode == "collective":  # no store: the peer never joins the all-gather, the group's timeout ends it
                if rank == 1:
                    time.sleep(8.0)
                    q.put((rank, ("skipped", None), 0.0))
                    return
                gather_trajectories(_fake_tokens(1, 0, 5, 4), 10)
                out = ("gathered", None)
        except ShardFailure as e:
            out = ("shard_failure", (e.ranks, str(e)))
        except Exception as e:  # noqa: BLE001
            out = ("error", f"{type(e).__name__}: {e}"[:200])
        q.put((rank, out, time.monotonic() - t0))
    finally:
        try:
            dist.destroy_process_group()
        except Exception:  # noqa: BLE001 - a group whose collective timed out may refuse a clean shutdown
            pass


def _run_failure(mode):
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_failure_worker, args=(r, 2, port, mode, q)) for r in range(2)]
    for p in procs:
        p.start()
    got = {}
    for _ in range(2):
        r, out, dt = q.get(timeout=120)
        got[r] = (out, dt)
    for p in procs:
        p.join(timeout=60)
    return got


def test_rank_that_raises_is_reported_before_the_gather():
    got = _run_failure("raises")
    assert got[1][0][0] == "error" and "bounded wait ran out" in got[1][0][1]  # the failing rank re-raises its own error
    kind, (ranks, text) = got[0][0]
    assert kind == "shard_failure" and ranks == [1] and "bounded wait ran out" in text
    assert got[0][1] < 10.0  # learnt from the store, not from a collective timing out


def test_rank_that_leaves_between_steps_times_out_on_the_host():
    got = _run_failure("leaves")
    assert got[1][0][0] == "left"
    kind, (ranks, text) = got[0][0]
    assert kind == "shard_failure" and ranks == [1] and "did not reach step 1" in text
    assert 1.0 < got[0][1] < 15.0


def test_collective_without_its_peer_ends_with_an_error_after_the_group_timeout():
    got = _run_failure("collective")
    assert got[0][0][0] == "error", got  # gloo raises once the 4 s group timeout has passed
    assert got[0][1] < 30.0


def test_shard_of_zero_trajectories_and_path_choice_follow_the_whole_job():
    """world > num_samples leaves ranks without work; every rank is told the attention path of the WHOLE job."""
    assert shard_range(2, 3, 4) == (2, 0)
    eng = _FakeEngine(fail=False)
    toks, _ = decode_sharded(eng, [[1]], 24)  # one process: the whole job
    assert eng.calls == [(24, 0, True)] and toks.shape == (1, 24, 4)
    eng = _FakeEngine(fail=False)
    decode_sharded(eng, [[1]], 12)
    assert eng.calls == [(12, 0, False)]
