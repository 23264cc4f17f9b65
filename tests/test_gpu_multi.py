"""Two ranks on two GPUs (NCCL): trajectories split over the ranks, each prompt prefilled on one rank only and its K/V
exchanged, token streams gathered - against the same job decoded by one process.  Skipped on a box with one GPU."""

import os
import socket

import pytest
import torch

pytestmark = pytest.mark.gpu


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, q):
    import torch.distributed as dist

    from conftest import golden_weights, load_golden
    from diff_gpt_b200 import GPT, Engine, NucleusSampler, TemperatureSampler
    from diff_gpt_b200.dist import decode_sharded

    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    try:
        g = load_golden("small_bf16_d64")
        V, C, H, L, block = (int(x) for x in g["meta"][:5])
        m = GPT(vocab_size=V, n_embd=C, block_size=block, n_head=H, n_layer=L).eval()
        sd = dict(golden_weights(g, torch.float32))
        sd["lm_head.weight"] = sd["token_embedding_table.weight"]
        m.load_state_dict(sd)
        m = m.to(torch.bfloat16).cuda()
        prompts = [g["idx"][0].tolist(), g["idx"][1].tolist()]
        s = NucleusSampler(0.9, TemperatureSampler(1.0))
        eng = Engine(m)
        toks, masks = decode_sharded(eng, prompts, 40, max_tokens=10, sampler=s, seed=5)
        shared = eng._run.prefill_group is not None and len(eng._run.prefills) == 1 and eng._run.prefills[0][1] == [rank]
        whole, _ = Engine(m).generate_many(prompts, 40, 10, s, seed=5)
        q.put((rank, bool(torch.equal(toks, whole)), bool((masks == 1).all()), shared, tuple(toks.shape)))
        dist.barrier()
    finally:
        dist.destroy_process_group()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_two_ranks_share_the_prompt_prefill_and_reproduce_the_whole_job():
    import torch.multiprocessing as mp

    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, 2, port, q)) for r in range(2)]
    for p in procs:
        p.start()
    got = {}
    for _ in range(2):
        r, same, sampled, shared, shape = q.get(timeout=300)
        got[r] = (same, sampled, shared, shape)
    for p in procs:
        p.join(timeout=120)
        assert p.exitcode == 0
    for r in range(2):
        assert got[r] == (True, True, True, (2, 40, 10)), got
