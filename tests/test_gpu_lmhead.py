"""The model's head as one call (`dgpt_lmhead_sample`): tied-embedding GEMM on the tcgen05 kernel, soft-cap, draw."""

import pytest
import torch

from conftest import golden_weights, load_golden

pytestmark = pytest.mark.gpu


def _ops():
    from diff_gpt_b200 import ops

    return ops


def _inputs(R, C, V, seed, scale=1.0):
    g = torch.Generator().manual_seed(seed)
    xn = torch.randn(R, C, generator=g).to(torch.bfloat16).cuda()
    emb = (torch.randn(V, C, generator=g) * scale / C**0.5).to(torch.bfloat16).cuda()
    return xn, emb


@pytest.mark.parametrize("R,C,V", [(300, 128, 512), (5, 64, 64), (1000, 768, 4096)])
def test_argmax_in_the_epilogue_equals_gemm_then_sampling_kernel(R, C, V):
    """Temperature 0: the token kept by the GEMM's epilogue is the one the sampling kernel picks from the stored logits
    (same GEMM, same soft-cap, ties to the lower token), and it is the arg-max of the fp32 logits wherever their top
    two are further apart than bf16 rounding."""
    ops = _ops()
    xn, emb = _inputs(R, C, V, seed=R + V, scale=4.0)
    logits = torch.empty(R, V, dtype=torch.bfloat16, device="cuda")
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    two = torch.empty(R, dtype=torch.int32, device="cuda")
    ops.lmhead_sample(xn, emb, two, cap=15.0, temperature=0.0, logits_out=logits, status=status)
    ws = torch.empty(ops.lmhead_workspace_bytes(R) // 8, dtype=torch.int64, device="cuda")
    one = torch.full((R,), -1, dtype=torch.int32, device="cuda")
    ops.lmhead_sample(xn, emb, one, cap=15.0, temperature=0.0, workspace=ws, status=status)
    assert status.item() == 0
    assert torch.equal(one, two)
    ref = xn.float() @ emb.float().T
    assert (logits.float() - ref).abs().max().item() <= 1e-2 * ref.abs().max().item()
    top2 = ref.topk(2, dim=-1).values
    clear = (top2[:, 0] - top2[:, 1]) > 2e-2 * ref.abs().max()
    assert bool(clear.any())
    assert torch.equal(one[clear].long(), ref.argmax(dim=-1)[clear])


@pytest.mark.parametrize("temperature", [1.0, 0.6])
def test_draws_in_the_epilogue_follow_softmax(temperature):
    """60 000 rows holding the same vector, each with its own trajectory id: token frequencies against
    softmax(cap(logits) / T) within 0.01 (the bar of the reference's tests/diff_gpt/sampler/test_temperature_sampler.py:95-122)."""
    ops = _ops()
    R, C, V = 60000, 64, 64
    xn1, emb = _inputs(1, C, V, seed=3, scale=6.0)
    xn = xn1.expand(R, C).contiguous()
    ws = torch.empty(ops.lmhead_workspace_bytes(R) // 8, dtype=torch.int64, device="cuda")
    tok = torch.empty(R, dtype=torch.int32, device="cuda")
    ops.lmhead_sample(xn, emb, tok, cap=15.0, temperature=temperature, seed=11, traj_id0=1000, workspace=ws)
    logits = torch.empty(1, V, dtype=torch.bfloat16, device="cuda")
    ops.linear(xn1, emb, logits)
    z = 15.0 * torch.tanh(logits.float() / 15.0)
    want = torch.softmax(z[0] / temperature, dim=-1).cpu()
    got = torch.bincount(tok.long().cpu(), minlength=V).float() / R
    assert int(tok.min()) >= 0 and int(tok.max()) < V
    assert (got - want).abs().max().item() <= 0.01
    # the stream depends on (seed, trajectory id, step) only: another launch shape, same ids, same tokens
    tok2 = torch.empty(777, dtype=torch.int32, device="cuda")
    ids = torch.arange(1000 + 123, 1000 + 123 + 777, dtype=torch.int64, device="cuda")
    ops.lmhead_sample(xn[:777], emb, tok2, cap=15.0, temperature=temperature, seed=11, traj_ids=ids, workspace=ws)
    assert torch.equal(tok2, tok[123 : 123 + 777])
    other = torch.empty(R, dtype=torch.int32, device="cuda")
    ops.lmhead_sample(xn, emb, other, cap=15.0, temperature=temperature, seed=12, traj_id0=1000, workspace=ws)
    assert not torch.equal(other, tok)


def test_forcing_history_and_masks_through_the_epilogue_form():
    ops = _ops()
    R, C, V, G = 12, 64, 128, 5
    xn, emb = _inputs(R, C, V, seed=9, scale=4.0)
    ws = torch.empty(ops.lmhead_workspace_bytes(R) // 8, dtype=torch.int64, device="cuda")
    tok = torch.empty(R, dtype=torch.int32, device="cuda")
    masks = torch.empty(R, dtype=torch.int32, device="cuda")
    hist = torch.full((R, G), -1, dtype=torch.int32, device="cuda")
    hmask = torch.full((R, G), -1, dtype=torch.int32, device="cuda")
    force = torch.tensor([[-1, 7, -1, -1, -1], [-1, -1, -1, -1, -1], [3, 3, 3, 3, 3]], dtype=torch.int32, device="cuda")
    step = torch.tensor([1], dtype=torch.int32, device="cuda")
    ops.lmhead_sample(xn, emb, tok, cap=15.0, temperature=0.0, step=step, force_schedule=force, force_group_rows=4,
                      force_group_stride=G, out_masks=masks, history_tokens=hist, history_masks=hmask, workspace=ws)
    free = torch.empty(R, dtype=torch.int32, device="cuda")
    ops.lmhead_sample(xn, emb, free, cap=15.0, temperature=0.0, workspace=ws)
    want = free.clone()
    want[:4], want[8:] = 7, 3
    assert torch.equal(tok, want)
    assert masks.tolist() == [0] * 4 + [1] * 4 + [0] * 4
    assert torch.equal(hist[:, 1], tok) and torch.equal(hmask[:, 1], masks)
    assert bool((hist[:, [0, 2, 3, 4]] == -1).all())


def test_refusals():
    from diff_gpt_b200 import _lib

    ops = _ops()
    xn, emb = _inputs(4, 64, 64, seed=1)
    tok = torch.empty(4, dtype=torch.int32, device="cuda")
    with pytest.raises(_lib.DgptError, match="logits buffer"):
        ops.lmhead_sample(xn, emb, tok, temperature=1.0, top_p=0.9)
    with pytest.raises(_lib.DgptError, match="workspace"):
        ops.lmhead_sample(xn, emb, tok, temperature=1.0)
    with pytest.raises(_lib.DgptError, match="bf16"):
        ops.lmhead_sample(xn.float(), emb.float(), tok, temperature=0.0)


def test_engine_tokens_do_not_depend_on_where_the_draw_happens():
    """Arg-max decode of 40 trajectories, bf16: the draw inside the head GEMM's epilogue (logits never stored) against
    the head GEMM followed by the sampling kernel, eager and as a replayed graph; with temperature the two forms use
    different random streams, so only shape, range and the forced steps are compared."""
    from diff_gpt_b200 import GPT, TemperatureSampler
    from diff_gpt_b200.model.engine import DecodeRun

    g = load_golden("small_bf16_d64")
    V, C, H, L, block = (int(x) for x in g["meta"][:5])
    m = GPT(vocab_size=V, n_embd=C, block_size=block, n_head=H, n_layer=L).eval()
    sd = dict(golden_weights(g, torch.float32))
    sd["lm_head.weight"] = sd["token_embedding_table.weight"]
    m.load_state_dict(sd)
    m = m.to(torch.bfloat16).cuda()
    prompt = g["idx"][0].tolist()
    G = 12
    outs = []
    for fused in (False, True):
        for graph in (False, True):
            run = DecodeRun(m, [prompt], 40, G, TemperatureSampler(0.0), 42, None, use_graph=graph, fused_head=fused)
            assert run.lmhead and (run.head_ws is not None) == fused and (run.logits is None) == fused
            run.start()
            run.advance(G)
            run.check_status()
            outs.append(run.history[:, :G].clone())
    assert all(torch.equal(outs[0], o) for o in outs[1:])
    sched = [None, 5, None, None, 9, None, None, None, None, None, None, None]
    run = DecodeRun(m, [prompt], 40, G, TemperatureSampler(1.0), 42, [sched])
    run.start()
    run.advance(G)
    run.check_status()
    t = run.history[:, :G]
    assert int(t.min()) >= 0 and int(t.max()) < V and bool((t[:, 1] == 5).all()) and bool((t[:, 4] == 9).all())
    assert len({tuple(r) for r in t.cpu().tolist()}) > 1
