"""tcgen05 prefill-attention kernels (bf16, head_dim 32/64/128) against the CPU oracle.  head_dim 32 runs on the
64-wide kernels with TMA boxes that reach past the tensor and are zero-filled there."""

import math

import pytest
import torch

from oracle import ref_math

pytestmark = pytest.mark.gpu


def _run(D, B, H, Tq, Tk, pt, causal, q_offset, use_table, o_f32, impl=2, seed=0):
    from diff_gpt_b200 import ops

    gen = torch.Generator().manual_seed(seed + D + Tq)
    dt = torch.bfloat16
    cap = -(-max(Tk) // pt) * pt if use_table else pt
    q = torch.randn(B, Tq, H, D, generator=gen).to(dt)
    k = torch.randn(B, H, cap, D, generator=gen).to(dt)
    v = torch.randn(B, H, cap, D, generator=gen).to(dt)
    if use_table:
        pages = cap // pt
        perm = torch.randperm(B * pages, generator=gen).to(torch.int32).view(B, pages)
        pool = torch.full((B * pages + 1, 2, H, pt, D), float("nan"), dtype=dt, device="cuda")
        for b in range(B):
            for p in range(pages):
                pool[perm[b, p], 0] = k[b, :, p * pt : (p + 1) * pt].cuda()
                pool[perm[b, p], 1] = v[b, :, p * pt : (p + 1) * pt].cuda()
        lay = ops.kv_layout(pool[0, 0], pool[0, 1], 2 * H * pt * D, pt * D, pt, perm.cuda(), n_pages=pool.shape[0])
    else:
        pool = torch.stack([k, v], dim=1).cuda().contiguous()  # (B, 2, H, cap, D): one page per sequence
        lay = ops.kv_layout(pool[0, 0], pool[0, 1], 2 * H * cap * D, cap * D, cap)
    o = torch.full((B, Tq, H, D), float("nan"), dtype=torch.float32 if o_f32 else dt, device="cuda")
    lse = torch.empty(B, Tq, H, dtype=torch.float32, device="cuda")
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    ops.fmha_prefill(
        q.cuda(), lay, o, B=B, H=H, Tq=Tq, D=D, q_batch_stride=Tq * H * D, q_row_stride=H * D,
        o_batch_stride=Tq * H * D, o_row_stride=H * D, kv_len=torch.tensor(Tk, dtype=torch.int32, device="cuda"),
        q_offset=q_offset, causal=causal, lse=lse, impl=impl, status=status,
    )
    torch.cuda.synchronize()
    assert status.item() == 0
    for b in range(B):
        qh = q[b : b + 1].transpose(1, 2)
        kk, vv = k[b : b + 1, :, : Tk[b]], v[b : b + 1, :, : Tk[b]]
        want = ref_math.sdpa(qh.float(), kk.float(), vv.float(), q_offset=q_offset if causal else 10**7).transpose(1, 2)
        got = o[b : b + 1].float().cpu()
        err = (got - want).abs().max().item() / want.abs().max().item()
        assert err <= 1.5e-2, (b, err)
        s = torch.matmul(qh.float(), kk.float().transpose(-1, -2)) / math.sqrt(D)
        if causal:
            i = torch.arange(Tq)[:, None]
            j = torch.arange(Tk[b])[None, :]
            s = s.masked_fill(j > q_offset + i, float("-inf"))
        want_lse = torch.logsumexp(s, dim=-1).transpose(1, 2)
        assert (lse[b : b + 1].cpu() - want_lse).abs().max().item() <= 2e-2


IMPLS = [2, 3, 4]  # 2 = warp-specialised kernel, 3 = two CTAs per SM, 4 = two query tiles per CTA


@pytest.mark.parametrize("impl", IMPLS)
@pytest.mark.parametrize("D", [32, 64, 128])
def test_single_tile(D, impl):
    _run(D, B=1, H=1, Tq=128, Tk=[128], pt=128, causal=False, q_offset=0, use_table=False, o_f32=False, impl=impl)


@pytest.mark.parametrize("D", [32, 64, 128])
@pytest.mark.parametrize("causal", [False, True])
@pytest.mark.parametrize("impl", IMPLS)
def test_multi_tile_dense(D, causal, impl):
    _run(D, B=2, H=2, Tq=300, Tk=[384, 300] if not causal else [300, 300], pt=384, causal=causal, q_offset=0,
         use_table=False, o_f32=False, impl=impl)


@pytest.mark.parametrize("D", [32, 64, 128])
@pytest.mark.parametrize("pt", [16, 64, 128])
@pytest.mark.parametrize("impl", IMPLS)
def test_paged_ragged_offset(D, pt, impl):
    _run(D, B=2, H=3, Tq=37, Tk=[48, 43], pt=pt, causal=True, q_offset=11, use_table=True, o_f32=False, impl=impl)
    _run(D, B=2, H=2, Tq=200, Tk=[700, 513], pt=pt, causal=False, q_offset=0, use_table=True, o_f32=True, impl=impl)


@pytest.mark.parametrize("impl", IMPLS + [0])
def test_matches_warp_level_kernel_on_a_long_causal_case(impl):
    _run(128, B=1, H=2, Tq=1024, Tk=[1024], pt=1024, causal=True, q_offset=0, use_table=False, o_f32=False, impl=impl)
    _run(64, B=1, H=2, Tq=640, Tk=[1024], pt=64, causal=True, q_offset=384, use_table=True, o_f32=False, impl=impl)


@pytest.mark.parametrize("D", [64, 128])
@pytest.mark.parametrize("causal", [False, True])
@pytest.mark.parametrize("impl", IMPLS)
def test_capped_grid_loops_over_query_tiles_with_identical_results(D, causal, impl):
    """max_ctas below the number of (query tile, head, batch) items: every CTA walks several items (barriers
    re-initialised in between) and the output is bit-identical to one CTA per item, for both tensor-core kernels."""
    from diff_gpt_b200 import ops

    B, H, Tq, Tk, pt = 2, 3, 600, 700, 64
    g = torch.Generator(device="cuda").manual_seed(D + causal)
    q = torch.randn((B, Tq, H, D), device="cuda", dtype=torch.bfloat16, generator=g)
    pages = -(-Tk // pt)
    pool = torch.randn((B * pages, 2, H, pt, D), device="cuda", dtype=torch.bfloat16, generator=g)
    table = torch.randperm(B * pages, generator=torch.Generator().manual_seed(1)).to(torch.int32).view(B, pages).cuda()
    lay = ops.kv_layout(pool[0, 0], pool[0, 1], 2 * H * pt * D, pt * D, pt, table, n_pages=B * pages)
    klen = torch.tensor([Tk, Tk - 77], dtype=torch.int32, device="cuda")
    outs = []
    for cap in (0, 1, 7, 1000):
        o = torch.full((B, Tq, H, D), float("nan"), device="cuda", dtype=torch.float32)
        lse = torch.full((B, Tq, H), float("nan"), device="cuda", dtype=torch.float32)
        status = torch.zeros(1, dtype=torch.int32, device="cuda")
        ops.fmha_prefill(q, lay, o, B=B, H=H, Tq=Tq, D=D, q_batch_stride=Tq * H * D, q_row_stride=H * D,
                         o_batch_stride=Tq * H * D, o_row_stride=H * D, kv_len=klen, q_offset=Tk - 77 - Tq if causal else 0,
                         causal=causal, lse=lse, impl=impl, status=status, max_ctas=cap)
        assert status.item() == 0 and torch.isfinite(o).all() and torch.isfinite(lse).all()
        outs.append((o, lse))
    for o, lse in outs[1:]:
        assert torch.equal(o, outs[0][0]) and torch.equal(lse, outs[0][1])


@pytest.mark.parametrize("impl", [2, 4])
@pytest.mark.parametrize("D,pt", [(64, 64), (128, 128), (32, 4096)])
def test_long_causal_rows_stay_within_rounding_of_fp64_and_repeat_bit_for_bit(D, pt, impl):
    """4096 keys per sequence (32 key tiles per work item, many items per CTA) through a shuffled page table: every row
    against fp64 attention on the device with a bound that follows the value (bf16 output rounding) plus a floor for
    the rounding of the probabilities, and three more launches that must reproduce the first bit for bit - the
    persistent kernels hand buffers between their roles, and a hand-over that is a tile early shows up as a few
    wrong elements in one launch out of several."""
    from diff_gpt_b200 import ops

    B, H, S = 2, 8, 4096
    g = torch.Generator(device="cuda").manual_seed(11 * D + impl)
    q = torch.randn((B, S, H, D), device="cuda", dtype=torch.bfloat16, generator=g)
    pages = S // pt
    pool = torch.randn((B * pages, 2, H, pt, D), device="cuda", dtype=torch.bfloat16, generator=g)
    table = torch.randperm(B * pages, generator=torch.Generator().manual_seed(2)).to(torch.int32).view(B, pages).cuda()
    lay = ops.kv_layout(pool[0, 0], pool[0, 1], 2 * H * pt * D, pt * D, pt, table, n_pages=B * pages)
    status = torch.zeros(1, dtype=torch.int32, device="cuda")

    def att():
        o = torch.empty_like(q)
        ops.fmha_prefill(q, lay, o, B=B, H=H, Tq=S, D=D, q_batch_stride=S * H * D, q_row_stride=H * D,
                         o_batch_stride=S * H * D, o_row_stride=H * D, kv_len_all=S, causal=True, impl=impl, status=status)
        return o

    first = att()
    assert status.item() == 0
    ix = torch.arange(S, device="cuda")
    future = ix[None, :] > ix[:, None]
    for b in range(B):
        kv = pool[table[b].long()]  # (pages, 2, H, pt, D) in logical order
        for h in range(H):
            kk = kv[:, 0, h].reshape(S, D).double()
            vv = kv[:, 1, h].reshape(S, D).double()
            sc = (q[b, :, h].double() @ kk.T) / D**0.5
            want = (torch.softmax(sc.masked_fill(future, float("-inf")), dim=-1) @ vv).float()
            excess = (first[b, :, h].float() - want).abs() - (2.0**-8 * want.abs() + 4e-3)
            assert excess.max().item() <= 0.0, (b, h, excess.argmax().item() // D)
    for _ in range(3):
        assert torch.equal(att(), first)
