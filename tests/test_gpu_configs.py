"""Reduced-size versions of the BASELINE configurations 2, 3 and 5 against the CPU oracle (same code paths as full size)."""

import numpy as np
import pytest
import torch

from oracle import ref_decode, ref_math

pytestmark = pytest.mark.gpu


def _gpu_model(shape, w, dtype):
    from diff_gpt_b200 import GPT

    m = GPT(vocab_size=shape.vocab_size, n_embd=shape.n_embd, block_size=shape.block_size, n_head=shape.n_head,
            n_layer=shape.n_layer).eval()
    sd = dict(w)
    sd["lm_head.weight"] = sd["token_embedding_table.weight"]
    m.load_state_dict(sd)
    return m.to(dtype).cuda()


def test_config2_shape_batched_forward_bf16_head_dim_32():
    """Config 2 narrowed (n_embd 128, 4 heads of 32, 2 layers, vocab 512, T = 96, batch 6): full causal forward
    with soft-cap in bf16 through the warp-level attention kernel; logits within 2e-2 of the oracle."""
    shape = ref_math.Shape(vocab_size=512, n_embd=128, n_head=4, n_layer=2, block_size=96)
    w = ref_math.random_weights(shape, seed=2, dtype=torch.bfloat16, std=0.08)
    idx = torch.randint(0, 512, (6, 96), generator=torch.Generator().manual_seed(2))
    want = ref_math.forward(shape, w, idx).float()
    got = _gpu_model(shape, w, torch.bfloat16)(idx.cuda())[0].float().cpu()
    assert got.shape == (6, 96, 512)
    assert (got - want).abs().max().item() <= 2e-2 * want.abs().max().item()


def test_config2_full_shape_on_the_tensor_core_attention():
    """Config 2 as BASELINE states it (V512 C256 H8 of 32, L4, bf16, N(0, 0.02) seed 2; 256 sequences x 512 tokens):
    head_dim 32 takes the tensor-core attention kernel; sequences do not interact, so four of the 256 rows of the
    full-batch result are compared with the oracle's forward of those four sequences."""
    from diff_gpt_b200 import _lib

    shape = ref_math.Shape(vocab_size=512, n_embd=256, n_head=8, n_layer=4, block_size=512)
    w = ref_math.random_weights(shape, seed=2, dtype=torch.bfloat16)
    idx = torch.randint(0, 512, (256, 512), generator=torch.Generator().manual_seed(2))
    rows = [0, 77, 130, 255]
    want = ref_math.forward(shape, w, idx[rows]).float()
    model = _gpu_model(shape, w, torch.bfloat16)
    timer = _lib.KernelTimer()
    with _lib.timed(timer):
        got = model(idx.cuda())[0]
    torch.cuda.synchronize()
    assert got.shape == (256, 512, 512)
    err = (got[rows].float().cpu() - want).abs().max().item() / want.abs().max().item()
    assert err <= 2e-2, err
    assert timer.summary()["dgpt_fmha_prefill"]["launches"] == 4


def test_config3_shape_many_series_one_trajectory_teacher_forced():
    """Config 3 narrowed: 5 series x 1 trajectory, 7 channels of which 2 are forced from a schedule, head_dim 64.
    One trajectory per series takes the per-row path with the prompt split along the keys (no shared-prompt phase).
    fp32 so that argmax streams can be compared token for token with the oracle."""
    from diff_gpt_b200 import Engine, TemperatureSampler

    shape = ref_math.Shape(vocab_size=128, n_embd=128, n_head=2, n_layer=2, block_size=1024)
    w = ref_math.random_weights(shape, seed=3, dtype=torch.float32, std=0.2)
    g = torch.Generator().manual_seed(3)
    F, P, G = 7, 7 * 90, 7 * 6  # prompt long enough (630 keys) for the split-K policy to engage
    prompts = [torch.randint(0, 128, (P,), generator=g).tolist() for _ in range(5)]
    cov = [torch.randint(0, 128, (G,), generator=g).tolist() for _ in range(5)]
    scheds = [[c[p] if (p % F) >= 5 else None for p in range(G)] for c in cov]
    eng = Engine(_gpu_model(shape, w, torch.float32))
    toks, masks = eng.generate_many(prompts, 1, G, TemperatureSampler(0.0), force_schedules=scheds)
    assert toks.shape == (5, 1, G)
    for s in range(5):
        ref, ref_m, _ = ref_decode.mc_decode(shape, w, prompts[s], 1, G, temperature=0.0, force_schedule=scheds[s])
        assert toks[s, 0].cpu().tolist() == ref[0].tolist(), s
        assert masks[s, 0].cpu().tolist() == ref_m[0].tolist()


@pytest.mark.parametrize("S", [200, 384])
def test_config5_shape_attention_layer_bf16_head_dim_128(S):
    """Config 5 narrowed (batch 2, 4 heads of 128, S = 200 / 384): RoPE + QK-norm + causal attention on the
    tcgen05 kernel + output projection, inputs injected after the projections; within 2e-2 of the oracle."""
    from diff_gpt_b200 import ops

    B, H, D = 2, 4, 128
    C = H * D
    g = torch.Generator().manual_seed(5)
    q = torch.randn(B, S, H, D, generator=g).to(torch.bfloat16)
    k = torch.randn(B, S, H, D, generator=g).to(torch.bfloat16)
    v = torch.randn(B, S, H, D, generator=g).to(torch.bfloat16)
    wp = (torch.randn(C, C, generator=g) * 0.02).to(torch.bfloat16)
    table = ref_math.rope_table(D, 512).to(torch.bfloat16)
    want = ref_math.attention_only(q, k, v, table, wp).float()

    cap = -(-S // 128) * 128
    cache = torch.zeros(B, 2, H, cap, D, dtype=torch.bfloat16, device="cuda")
    lay = ops.kv_layout(cache[0, 0], cache[0, 1], 2 * H * cap * D, cap * D, cap)
    qkv = torch.cat([q.reshape(B * S, C), k.reshape(B * S, C), v.reshape(B * S, C)], dim=1).cuda()
    q_rot = torch.empty(B * S, C, dtype=torch.bfloat16, device="cuda")
    zero = torch.zeros(B, dtype=torch.int32, device="cuda")
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    ops.rope_qknorm_kvappend(qkv[:, :C], qkv[:, C : 2 * C], qkv[:, 2 * C :], q_rot, table.cuda(), lay, zero, zero, None,
                             B, S, H, D, status)
    y = torch.empty(B * S, C, dtype=torch.bfloat16, device="cuda")
    ops.fmha_prefill(q_rot, lay, y, B=B, H=H, Tq=S, D=D, q_batch_stride=S * C, q_row_stride=C, o_batch_stride=S * C,
                     o_row_stride=C, kv_len_all=S, causal=True, impl=2, status=status)
    out = torch.mm(y, wp.cuda().t()).view(B, S, C).float().cpu()
    assert status.item() == 0
    assert (out - want).abs().max().item() <= 2e-2 * want.abs().max().item()


# ---- full BASELINE sizes, checked through properties that do not need the CPU oracle -------------------
def test_config4_full_size_shards_reproduce_the_whole_and_argmax_rows_agree():
    """One series of config 4 at full size (12 layers, 12 heads of 64, 1024-token prompt, 4096 trajectories,
    horizon 32 to keep the test short): (a) decoding trajectories [0, 2048) and [2048, 4096) separately gives
    exactly the tokens of the whole run (the random stream is keyed by trajectory id, and no kernel's result
    may depend on which rows share a launch); (b) under argmax all 4096 rows produce one and the same stream;
    (c) forced steps are honoured in every row; (d) nucleus draws stay inside the nucleus of their row."""
    import workloads
    from diff_gpt_b200 import Engine, NucleusSampler, TemperatureSampler

    m = workloads.gpu_model(workloads.CFG4, workloads.weights(workloads.CFG4, 4, torch.bfloat16), torch.bfloat16)
    prompt = workloads.cfg4_prompts(1)[0]
    assert len(prompt) == 1024
    N, G = 4096, 32
    s = NucleusSampler(0.9, TemperatureSampler(1.0))
    eng = Engine(m)
    whole, _ = eng.generate_many([prompt], N, G, s, seed=42)
    lo, _ = eng.generate_many([prompt], N // 2, G, s, seed=42, traj_offset=0)
    hi, _ = eng.generate_many([prompt], N // 2, G, s, seed=42, traj_offset=N // 2)
    assert torch.equal(whole[:, : N // 2], lo) and torch.equal(whole[:, N // 2 :], hi)
    assert int(whole.min()) >= 0 and int(whole.max()) < workloads.CFG4["vocab_size"]
    assert len({tuple(r) for r in whole[0, :64].cpu().tolist()}) > 32  # trajectories differ
    sched = [None] * G
    sched[3], sched[17] = 7, 4000
    greedy, masks = eng.generate_many([prompt], N, G, TemperatureSampler(0.0), force_schedules=[sched])
    assert bool((greedy[0] == greedy[0, :1]).all())
    assert bool((greedy[0, :, 3] == 7).all()) and bool((greedy[0, :, 17] == 4000).all())
    assert masks[0, 0].cpu().tolist() == [0 if i in (3, 17) else 1 for i in range(G)]
    eng.release()


@pytest.mark.parametrize("S", [4096, 8192])
def test_config5_full_size_the_two_tensor_core_kernels_agree_and_attention_is_linear_in_v(S):
    """Config 5 at full size (batch 8, 16 heads of 128, causal): the warp-specialised kernel and the
    two-CTAs-per-SM kernel are different programs and must agree within bf16 rounding; the output is linear
    in V (att(q, k, 2 v1 - v2) = 2 att(v1) - att(v2)); row 0 of every sequence sees one key, so it returns v[0]."""
    from diff_gpt_b200 import ops

    B, H, D = 8, 16, 128
    g = torch.Generator(device="cuda").manual_seed(5)
    q = torch.randn((B, S, H, D), device="cuda", dtype=torch.bfloat16, generator=g)
    k = torch.randn((B, H, S, D), device="cuda", dtype=torch.bfloat16, generator=g)
    v1 = torch.randn((B, H, S, D), device="cuda", dtype=torch.bfloat16, generator=g)
    v2 = torch.randn((B, H, S, D), device="cuda", dtype=torch.bfloat16, generator=g)
    status = torch.zeros(1, dtype=torch.int32, device="cuda")

    def att(v, impl):
        o = torch.empty_like(q)
        lay = ops.kv_layout(k, v, page_stride=H * S * D, head_stride=S * D, page_tokens=S)
        ops.fmha_prefill(q, lay, o, B=B, H=H, Tq=S, D=D, q_batch_stride=S * H * D, q_row_stride=H * D,
                         o_batch_stride=S * H * D, o_row_stride=H * D, kv_len_all=S, causal=True, impl=impl, status=status)
        return o.float()

    a2, a3 = att(v1, 2), att(v1, 3)
    assert status.item() == 0
    scale = a2.abs().max().item()
    # two (batch, head) slices of the warp-specialised kernel against fp32 softmax attention on the host (reference
    # mha.py:64): every 29th query row plus the whole last tile, against all the keys each may see
    rows = torch.unique(torch.cat([torch.arange(0, S, 29), torch.arange(S - 130, S)]))
    for b, h in ((0, 0), (B - 1, 7)):
        qs = q[b, rows, h].float().cpu()
        ks, vs = k[b, h].float().cpu(), v1[b, h].float().cpu()
        sc = (qs @ ks.T) / D**0.5
        sc = sc.masked_fill(torch.arange(S)[None, :] > rows[:, None], float("-inf"))
        want = torch.softmax(sc, dim=-1) @ vs
        for got in (a2, a3):
            err = (got[b, rows, h].cpu() - want).abs().max().item() / want.abs().max().item()
            assert err <= 1e-2, (b, h, err)
    assert (a2 - a3).abs().max().item() <= 1.5e-2 * scale
    # every row of every (batch, head) pair against fp64 softmax attention on the device: late rows average thousands
    # of values and are small, so the bound follows the value (bf16 output rounding) plus a floor for the rounding of
    # the probabilities; and a second launch must repeat the first bit for bit (nothing in the kernels depends on timing)
    key_ix = torch.arange(S, device="cuda")
    future = key_ix[None, :] > key_ix[:, None]
    for b in range(B):
        for h in range(H):
            sc = (q[b, :, h].double() @ k[b, h].double().T) / D**0.5
            want = (torch.softmax(sc.masked_fill(future, float("-inf")), dim=-1) @ v1[b, h].double()).float()
            for got in (a2, a3):
                excess = (got[b, :, h] - want).abs() - (2.0**-8 * want.abs() + 4e-3)
                assert excess.max().item() <= 0.0, (b, h, excess.argmax().item() // D)
    assert torch.equal(att(v1, 2), a2) and torch.equal(att(v1, 3), a3)
    assert torch.equal(a2[:, 0], v1[:, :, 0].float()) and torch.equal(a3[:, 0], v1[:, :, 0].float())
    mix = (2 * v1.float() - v2.float()).bfloat16()
    lin = 2 * a2 - att(v2, 2)
    got = att(mix, 2)
    assert (got - lin).abs().max().item() <= 4e-2 * lin.abs().max().item()
    # late rows average many values: their magnitude shrinks like 1/sqrt(keys) for these random inputs
    assert a2[:, -64:].abs().mean().item() < 0.25 * a2[:, :4].abs().mean().item()
