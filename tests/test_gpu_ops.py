"""Kernel-level parity: each C-ABI entry point against the CPU oracle on seeded inputs."""

import math

import numpy as np
import pytest
import torch

from conftest import load_golden
from oracle import ref_decode, ref_math

pytestmark = pytest.mark.gpu

DT = [(torch.float32, 2e-6, "f32"), (torch.bfloat16, 1e-2, "bf16")]


def _ops():
    from diff_gpt_b200 import ops

    return ops


def _rel(a: torch.Tensor, b: torch.Tensor) -> float:
    return (a.float().cpu() - b.float().cpu()).abs().max().item() / max(b.float().abs().max().item(), 1e-30)


@pytest.mark.parametrize("dtype,tol,tag", DT)
def test_rmsnorm_and_golden(dtype, tol, tag):
    from diff_gpt_b200.model.rms_norm import rms_norm

    g = load_golden("ops")
    x = torch.from_numpy(g[f"rope_x_{tag}"]).to(dtype)
    got = rms_norm(x.cuda())
    assert got.dtype == dtype and got.shape == x.shape
    assert _rel(got, torch.from_numpy(g[f"rn_y_{tag}"])) <= tol * 4
    # scale invariance and odd widths (reference tests/diff_gpt/model/test_rms_norm.py)
    y = torch.randn(7, 100, generator=torch.Generator().manual_seed(0)).to(dtype)
    a, b = rms_norm(y.cuda()), rms_norm((y * 8).cuda())
    assert _rel(a, b) <= 1e-2
    assert _rel(a, ref_math.rms_norm(y)) <= tol * 4


@pytest.mark.parametrize("dtype,tol,tag", DT)
def test_depthmix_golden_and_random(dtype, tol, tag):
    ops = _ops()
    g = load_golden("ops")
    c = torch.from_numpy(g[f"mix_c_{tag}"]).to(dtype).cuda()
    w = torch.from_numpy(g[f"mix_w_{tag}"]).to(dtype).cuda().reshape(-1)
    cands = [c[i].contiguous() for i in range(4)]
    h = torch.empty_like(cands[0])
    rn = torch.empty_like(cands[0])
    ops.depthmix(cands, w, h, rn)
    want = torch.from_numpy(g[f"mix_h_{tag}"])
    assert _rel(h, want) <= (1e-5 if dtype == torch.float32 else 2e-2)
    assert _rel(rn, ref_math.rms_norm(h.cpu())) <= tol * 8
    # wide rows, many candidates with a duplicate (the committed embedding appears twice)
    gen = torch.Generator().manual_seed(3)
    for C in (64, 768, 2048):
        cs = [(torch.randn(9, C, generator=gen) * (1 + i)).to(dtype) for i in range(6)]
        cs.insert(1, cs[0])
        wv = (torch.randn(C, generator=gen) * 0.2).to(dtype)
        want = ref_math.depth_mix(cs, wv)
        out = torch.empty(9, C, dtype=dtype, device="cuda")
        ops.depthmix([t.cuda() for t in cs], wv.cuda(), out, None)
        assert _rel(out, want) <= (2e-5 if dtype == torch.float32 else 3e-2), C
    # the same device buffer listed twice (read once, weight doubled) against two separate copies of it;
    # and a list that is one buffer repeated: the mix is that buffer
    base = [(torch.randn(10, 768, generator=gen) * (1 + i)).to(dtype).cuda() for i in range(4)]
    wv = (torch.randn(768, generator=gen) * 0.2).to(dtype).cuda()
    o_same, o_copy, o_one = (torch.empty(10, 768, dtype=dtype, device="cuda") for _ in range(3))
    ops.depthmix([base[0], base[0], base[1], base[2], base[0], base[3]], wv, o_same, None)
    ops.depthmix([base[0], base[0].clone(), base[1], base[2], base[0].clone(), base[3]], wv, o_copy, None)
    assert _rel(o_same, o_copy) <= (1e-6 if dtype == torch.float32 else 8e-3)
    ops.depthmix([base[1], base[1], base[1]], wv, o_one, None)
    assert torch.equal(o_one, base[1])
    # norm factors carried between mixes: written by one call, read by the next, same bits as without them
    rows = 37
    pool = [(torch.randn(rows, 768, generator=gen) * (1 + i)).to(dtype).cuda() for i in range(5)]
    wv = (torch.randn(768, generator=gen) * 0.2).to(dtype).cuda()
    plain, first, second = (torch.empty(rows, 768, dtype=dtype, device="cuda") for _ in range(3))
    lst = [pool[0], pool[0], pool[1], pool[2], pool[3], pool[4]]
    ops.depthmix(lst, wv, None, plain)
    inv = [torch.full((rows,), float("nan"), device="cuda") for _ in range(3)]
    ops.depthmix_cached(lst, [None] * 6, wv, None, first, inv[0], 0)      # writes the factor of pool[0]
    ops.depthmix_cached(lst, [inv[0], inv[0], None, None, None, None], wv, None, second, inv[1], 2)  # reads it, writes pool[1]'s
    assert torch.equal(first, plain) and torch.equal(second, plain)
    want_inv = torch.rsqrt(pool[1].float().pow(2).mean(-1) + 1.1920928955078125e-07)
    assert torch.isfinite(inv[0]).all() and (inv[1] - want_inv).abs().max().item() <= 1e-6 * want_inv.abs().max().item()
    third = torch.empty_like(plain)
    ops.depthmix_cached(lst, [inv[0], inv[0], inv[1], None, None, None], wv, None, third)
    assert torch.equal(third, plain)
    # candidate counts on both sides of the shared-memory-staged kernel's limit (32), odd row count
    for n_c in (2, 3, 13, 17, 32, 33):
        cs = [(torch.randn(11, 768, generator=gen) * (1 + 0.3 * i)).to(dtype) for i in range(n_c)]
        wv = (torch.randn(768, generator=gen) * 0.2).to(dtype)
        want = ref_math.depth_mix(cs, wv)
        out = torch.empty(11, 768, dtype=dtype, device="cuda")
        rn = torch.empty_like(out)
        ops.depthmix([t.cuda() for t in cs], wv.cuda(), out, rn)
        assert _rel(out, want) <= (2e-5 if dtype == torch.float32 else 3e-2), n_c
        assert _rel(rn, ref_math.rms_norm(out.cpu())) <= tol * 8, n_c


@pytest.mark.parametrize("dtype,tol,tag", DT)
def test_swiglu_golden(dtype, tol, tag):
    ops = _ops()
    g = load_golden("ops")
    u = torch.from_numpy(g[f"glu_u_{tag}"]).to(dtype).cuda()
    out = torch.empty(u.shape[0], u.shape[1] // 2, dtype=dtype, device="cuda")
    ops.swiglu(u, out, 1.702, 7.0)
    assert _rel(out, torch.from_numpy(g[f"glu_y_{tag}"])) <= (1e-6 if dtype == torch.float32 else 1e-2)
    # ragged tail of the vectorised bf16 path
    x = (torch.randn(3, 2 * 37, generator=torch.Generator().manual_seed(1)) * 4).to(dtype)
    o = torch.empty(3, 37, dtype=dtype, device="cuda")
    ops.swiglu(x.cuda(), o, 1.702, 7.0)
    assert _rel(o, ref_math.swiglu(x, 1.702, 7.0)) <= (1e-6 if dtype == torch.float32 else 1e-2)


@pytest.mark.parametrize("dtype,tol,tag", DT)
def test_softcap(dtype, tol, tag):
    ops = _ops()
    x = (torch.randn(5, 64, generator=torch.Generator().manual_seed(2)) * 20).to(dtype)
    y = x.clone().cuda()
    ops.softcap_(y, 15.0)
    want = 15.0 * torch.tanh(x / 15.0)
    assert _rel(y, want) <= (1e-6 if dtype == torch.float32 else 1e-2)
    assert y.float().abs().max().item() <= 15.0


def _dense_cache(L, B, H, T, D, dtype):
    return torch.zeros(L, 2, B, H, T, D, dtype=dtype, device="cuda")


@pytest.mark.parametrize("dtype,tol,tag", DT)
@pytest.mark.parametrize("D", [8, 16, 64, 128])
def test_rope_qknorm_kvappend_dense(dtype, tol, tag, D):
    """RoPE + QK-norm + append into the reference's dense layout, at a non-zero position."""
    ops = _ops()
    B, T, H = 2, 5, 3
    C = H * D
    gen = torch.Generator().manual_seed(D)
    qkvg = (torch.randn(B * T, 4 * C, generator=gen) * 1.5).to(dtype)
    table = ref_math.rope_table(D, 64).to(dtype)
    t0, cap = 7, 16
    cache = _dense_cache(1, B, H, cap, D, dtype)
    lay = ops.kv_layout(cache[0, 0], cache[0, 1], page_stride=H * cap * D, head_stride=cap * D, page_tokens=cap)
    dq = qkvg.cuda()
    q_out = torch.empty(B * T, C, dtype=dtype, device="cuda")
    start = torch.full((B,), t0, dtype=torch.int32, device="cuda")
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    ops.rope_qknorm_kvappend(
        dq[:, :C], dq[:, C : 2 * C], dq[:, 2 * C : 3 * C], q_out, table.cuda(), lay, start, start, None, B, T, H, D, status
    )
    assert status.item() == 0
    cs = table[t0 : t0 + T]
    q = qkvg[:, :C].view(B, T, H, D)
    k = qkvg[:, C : 2 * C].view(B, T, H, D)
    v = qkvg[:, 2 * C : 3 * C].view(B, T, H, D)
    want_q = ref_math.rms_norm(ref_math.rope(q, cs))
    want_k = ref_math.rms_norm(ref_math.rope(k, cs)).transpose(1, 2)
    assert _rel(q_out.view(B, T, H, D), want_q) <= tol * 4
    assert _rel(cache[0, 0, :, :, t0 : t0 + T], want_k) <= tol * 4
    assert torch.equal(cache[0, 1, :, :, t0 : t0 + T].cpu(), v.transpose(1, 2))
    assert cache[0, :, :, :, :t0].abs().max().item() == 0 and cache[0, :, :, :, t0 + T :].abs().max().item() == 0
    # out-of-range slot: flagged, nothing written
    status.zero_()
    far = torch.full((B,), cap - 2, dtype=torch.int32, device="cuda")
    before = cache.clone()
    ops.rope_qknorm_kvappend(
        dq[:, :C], dq[:, C : 2 * C], dq[:, 2 * C : 3 * C], q_out, table.cuda(), lay, far, far, None, B, T, H, D, status
    )
    assert status.item() == 1
    assert torch.equal(cache[..., : cap - 2, :], before[..., : cap - 2, :])


def _paged(ops, n_pages, H, pt, D, dtype, table):
    pool = torch.zeros(n_pages, 2, H, pt, D, dtype=dtype, device="cuda")
    lay = ops.kv_layout(pool[0, 0], pool[0, 1], page_stride=2 * H * pt * D, head_stride=pt * D, page_tokens=pt, page_table=table)
    return pool, lay


@pytest.mark.parametrize("dtype,tol,tag", DT)
@pytest.mark.parametrize("D,impl", [(16, 1), (32, 1), (64, 1), (128, 1)])
@pytest.mark.parametrize("causal", [True, False])
def test_fmha_prefill_paged(dtype, tol, tag, D, impl, causal):
    """Attention over a scrambled page table with ragged lengths, a query offset, LSE output."""
    ops = _ops()
    B, H, Tq, pt = 2, 3, 37, 16
    q_offset = 11 if causal else 0
    Tk = [Tq + q_offset, Tq + q_offset - 5] if causal else [50, 23]
    gen = torch.Generator().manual_seed(17 + D)
    q = torch.randn(B, Tq, H, D, generator=gen).to(dtype)
    k = torch.randn(B, H, 64, D, generator=gen).to(dtype)
    v = torch.randn(B, H, 64, D, generator=gen).to(dtype)
    pages = 4
    perm = torch.randperm(B * pages, generator=gen).to(torch.int32).view(B, pages)
    pool, lay = _paged(ops, B * pages, H, pt, D, dtype, perm.cuda())
    pool.fill_(float("nan"))  # an out-of-range read would poison the result
    for b in range(B):
        for p in range(pages):
            pool[perm[b, p], 0] = k[b, :, p * pt : (p + 1) * pt].cuda()
            pool[perm[b, p], 1] = v[b, :, p * pt : (p + 1) * pt].cuda()
    o = torch.empty(B, Tq, H, D, dtype=dtype, device="cuda")
    lse = torch.empty(B, Tq, H, dtype=torch.float32, device="cuda")
    kv_len = torch.tensor(Tk, dtype=torch.int32, device="cuda")
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    ops.fmha_prefill(
        q.cuda(), lay, o, B=B, H=H, Tq=Tq, D=D, q_batch_stride=Tq * H * D, q_row_stride=H * D,
        o_batch_stride=Tq * H * D, o_row_stride=H * D, kv_len=kv_len, q_offset=q_offset, causal=causal, lse=lse,
        impl=impl, status=status,
    )
    for b in range(B):
        qh = q[b : b + 1].transpose(1, 2)
        kk, vv = k[b : b + 1, :, : Tk[b]], v[b : b + 1, :, : Tk[b]]
        off = q_offset if causal else 10**6
        want = ref_math.sdpa(qh, kk, vv, q_offset=off).transpose(1, 2)
        assert _rel(o[b : b + 1], want) <= (2e-5 if dtype == torch.float32 else 1e-2)
        s = torch.matmul(qh.float(), kk.float().transpose(-1, -2)) / math.sqrt(D)
        if causal:
            i = torch.arange(Tq)[:, None]
            j = torch.arange(Tk[b])[None, :]
            s = s.masked_fill(j > q_offset + i, float("-inf"))
        want_lse = torch.logsumexp(s, dim=-1).transpose(1, 2)  # (1, Tq, H)
        assert (lse[b : b + 1].cpu() - want_lse).abs().max().item() <= 1e-4
    assert status.item() == 0


@pytest.mark.parametrize("dtype,tol,tag", DT)
@pytest.mark.parametrize("D", [16, 64, 128])
@pytest.mark.parametrize("n_splits", [1, 3])
@pytest.mark.parametrize("with_prefix", [False, True])
def test_decode_attn_two_ranges(dtype, tol, tag, D, n_splits, with_prefix):
    """One query per row over a shared prompt range plus a private range, optional split-K,
    optional merge with a prompt partial computed by the prefill kernel, sigmoid gate in the epilogue."""
    ops = _ops()
    S, N, H, pt = 2, 3, 2, 8
    R = S * N
    P = [13, 21]
    own = [5, 1, 9, 2, 7, 16]  # generated tokens so far per row (includes the new one)
    gen = torch.Generator().manual_seed(5 + D)
    pp, op = 3, 2
    n_pages = S * pp + R * op
    pool = torch.full((n_pages, 2, H, pt, D), float("nan"), dtype=dtype, device="cuda")
    pre_tab = torch.arange(S * pp, dtype=torch.int32).view(S, pp)
    own_tab = S * pp + torch.arange(R * op, dtype=torch.int32).view(R, op)
    row_tab = torch.cat([pre_tab.repeat_interleave(N, 0), own_tab], 1).cuda()
    lay_row = ops.kv_layout(pool[0, 0], pool[0, 1], 2 * H * pt * D, pt * D, pt, row_tab)
    lay_pre = ops.kv_layout(pool[0, 0], pool[0, 1], 2 * H * pt * D, pt * D, pt, pre_tab.cuda())
    kp = [torch.randn(H, P[s], D, generator=gen).to(dtype) for s in range(S)]
    vp = [torch.randn(H, P[s], D, generator=gen).to(dtype) for s in range(S)]
    ko = [torch.randn(H, own[r], D, generator=gen).to(dtype) for r in range(R)]
    vo = [torch.randn(H, own[r], D, generator=gen).to(dtype) for r in range(R)]

    def put(table_row, base_slot, kk, vv):
        for t in range(kk.shape[1]):
            slot = base_slot + t
            pg = int(table_row[slot // pt])
            pool[pg, 0, :, slot % pt] = kk[:, t].cuda()
            pool[pg, 1, :, slot % pt] = vv[:, t].cuda()

    for s in range(S):
        put(pre_tab[s], 0, kp[s], vp[s])
    for r in range(R):
        put(row_tab[r].cpu(), pp * pt, ko[r], vo[r])
    q = torch.randn(R, H * D, generator=gen).to(dtype)
    gate = torch.randn(R, H * D, generator=gen).to(dtype)
    len0 = torch.tensor([P[r // N] for r in range(R)], dtype=torch.int32, device="cuda")
    start1 = torch.full((R,), pp * pt, dtype=torch.int32, device="cuda")
    step = torch.tensor([2], dtype=torch.int32, device="cuda")
    len1 = torch.tensor([o - 2 for o in own], dtype=torch.int32, device="cuda")  # kernel adds the step
    y = torch.empty(R, H * D, dtype=dtype, device="cuda")
    ws = None
    if n_splits > 1:
        ws = torch.empty(ops.decode_attn_workspace_bytes(R, H, D, n_splits) // 4, dtype=torch.float32, device="cuda")
    po = pl = None
    if with_prefix:
        po = torch.empty(R, H, D, dtype=torch.float32, device="cuda")
        pl = torch.empty(R, H, dtype=torch.float32, device="cuda")
        ops.fmha_prefill(
            q.cuda(), lay_pre, po, B=S, H=H, Tq=N, D=D, q_batch_stride=N * H * D, q_row_stride=H * D,
            o_batch_stride=N * H * D, o_row_stride=H * D, kv_len=torch.tensor(P, dtype=torch.int32, device="cuda"),
            causal=False, lse=pl, impl=1,
        )
    ops.decode_attn(
        q.cuda(), lay_row, len0, start1, len1, step, y, H=H, D=D, gate=gate.cuda(), prefix_o=po, prefix_lse=pl,
        workspace=ws, n_splits=n_splits,
    )
    for r in range(R):
        s = r // N
        kk = torch.cat([kp[s], ko[r]], 1)[None]
        vv = torch.cat([vp[s], vo[r]], 1)[None]
        qh = q[r].view(1, 1, H, D).transpose(1, 2)
        att = ref_math.sdpa(qh, kk, vv, q_offset=10**6).transpose(1, 2).reshape(H * D)
        want = att * torch.sigmoid(gate[r])
        assert _rel(y[r], want) <= (2e-5 if dtype == torch.float32 else 1.5e-2), r
    if n_splits > 1:
        return
    # the same result from the two-launch form: per-row partial, then merge with the other partial
    part_o = torch.full((R, H, D), float("nan"), dtype=torch.float32, device="cuda")
    part_lse = torch.full((R, H), float("nan"), dtype=torch.float32, device="cuda")
    y2 = torch.empty_like(y)
    if with_prefix:  # prompt partial from the prefill kernel, own tokens from the partial kernel
        ops.decode_attn_partial(q.cuda(), lay_row, None, start1, len1, step, part_o, part_lse, H=H, D=D)
        ops.attn_merge(po, pl, part_o, part_lse, y2, H=H, D=D, gate=gate.cuda())
    else:  # both ranges in the partial kernel, merged with an empty partial
        ops.decode_attn_partial(q.cuda(), lay_row, len0, start1, len1, step, part_o, part_lse, H=H, D=D)
        zo = torch.zeros_like(part_o)
        zl = torch.full_like(part_lse, float("-inf"))
        ops.attn_merge(zo, zl, part_o, part_lse, y2, H=H, D=D, gate=gate.cuda())
    assert torch.isfinite(part_lse).all()
    assert _rel(y2, y) <= (2e-6 if dtype == torch.float32 else 8e-3)


def _philox_u(seed: int, traj: int, step: int, attempt: int = 0) -> float:
    """Host Philox4x32-10, first output word -> 24-bit uniform (the generator the kernel documents)."""
    M0, M1, W0, W1 = 0xD2511F53, 0xCD9E8D57, 0x9E3779B9, 0xBB67AE85
    c = [traj & 0xFFFFFFFF, (traj >> 32) & 0xFFFFFFFF, step & 0xFFFFFFFF, attempt]
    k0, k1 = seed & 0xFFFFFFFF, (seed >> 32) & 0xFFFFFFFF
    for _ in range(10):
        p0, p1 = M0 * c[0], M1 * c[2]
        c = [(p1 >> 32) ^ c[1] ^ k0, p1 & 0xFFFFFFFF, (p0 >> 32) ^ c[3] ^ k1, p0 & 0xFFFFFFFF]
        k0, k1 = (k0 + W0) & 0xFFFFFFFF, (k1 + W1) & 0xFFFFFFFF
    return (c[0] >> 8) / 16777216.0


def test_nucleus_filter_matches_reference_masks():
    ops = _ops()
    g = load_golden("samplers")
    logits = torch.from_numpy(g["logits"]).cuda()
    for p in (0.3, 0.5, 0.9, 0.99):
        got = torch.isfinite(ops.nucleus_filter(logits, p)).cpu().numpy()
        assert np.array_equal(got, g[f"mask_p{p}"]), p
    ka = torch.from_numpy(g["known_logits"]).cuda()
    assert torch.isfinite(ops.nucleus_filter(ka, 0.9)).cpu().tolist() == [[True, True, True, False]]
    # p -> 0 keeps only the top token; p >= 1 keeps everything
    assert torch.isfinite(ops.nucleus_filter(logits, 0.0)).sum(-1).cpu().tolist() == [1] * logits.shape[0]
    assert bool(torch.isfinite(ops.nucleus_filter(logits, 1.0)).all())
    # large vocabulary against the oracle's sort-based rule
    big = torch.randn(4, 4096, generator=torch.Generator().manual_seed(9)) * 1.5
    got = torch.isfinite(ops.nucleus_filter(big.cuda(), 0.9)).cpu()
    assert torch.equal(got, ref_decode.nucleus_mask(big, 0.9))


def test_nucleus_ties_keep_lowest_ids():
    ops = _ops()
    # 8 equal tokens: p = 0.30 needs 3 of them (mass before the third is 0.25 < 0.3) -> ids 0, 1, 2
    logits = torch.zeros(1, 8, device="cuda")
    kept = torch.isfinite(ops.nucleus_filter(logits, 0.30)).cpu().tolist()
    assert kept == [[True, True, True, False, False, False, False, False]]


@pytest.mark.parametrize("top_p", [1.0, 0.7])
@pytest.mark.parametrize("V,dtype", [(300, torch.float32), (1024, torch.float32), (4096, torch.bfloat16), (1000, torch.bfloat16)])
def test_sample_inverse_cdf_with_host_philox(top_p, V, dtype):
    """V = 300 and 1000 take the scalar loads, 1024 and 4096 the 16-byte loads of the warp-per-row kernel."""
    ops = _ops()
    R, seed, step0 = 64, 0x1234_5678_9ABC, 5
    logits = (torch.randn(R, V, generator=torch.Generator().manual_seed(4)) * 2).to(dtype).float()
    out = torch.empty(R, dtype=torch.int32, device="cuda")
    step = torch.tensor([step0], dtype=torch.int32, device="cuda")
    T = 0.8
    ops.sample(logits.to(dtype).cuda(), out, temperature=T, top_p=top_p, seed=seed, traj_id0=1000, step=step)
    got = out.cpu().tolist()
    # The kernel draws from softmax(l / T) over all tokens (attempt a uses Philox counter word 3 = a) and
    # accepts the first draw that lies in the nucleus; accepted draws follow the restricted distribution.
    mask = ref_decode.nucleus_mask(logits, top_p) if top_p < 1 else torch.ones_like(logits, dtype=torch.bool)
    w = torch.exp((logits.double() - logits.double().max(-1, keepdim=True).values) / T)
    cdf = torch.cumsum(w, -1) / w.sum(-1, keepdim=True)
    checked = 0
    for r in range(R):
        t = got[r]
        assert mask[r, t]
        for a in range(8):
            u = _philox_u(seed, 1000 + r, step0, a)
            cand = int(torch.searchsorted(cdf[r], torch.tensor(u, dtype=torch.float64), right=True).clamp(max=V - 1))
            edge = min(abs(u - cdf[r, cand].item()), abs(u - (cdf[r, cand - 1].item() if cand else 0.0)))
            if edge < 1e-5:
                break  # too close to a bin edge to predict in float32: skip this row
            if mask[r, cand]:
                assert cand == t, (r, a, cand, t)
                checked += 1
                break
    assert checked >= R * 3 // 4


def test_sample_argmax_cap_force_and_history():
    ops = _ops()
    R, V = 6, 128
    logits = torch.randn(R, V, generator=torch.Generator().manual_seed(8)) * 30
    out = torch.empty(R, dtype=torch.int32, device="cuda")
    masks = torch.empty(R, dtype=torch.int32, device="cuda")
    hist = torch.full((R, 4), -7, dtype=torch.int32, device="cuda")
    step = torch.tensor([1], dtype=torch.int32, device="cuda")
    ops.sample(logits.cuda(), out, cap=15.0, temperature=0.0, step=step, out_masks=masks, history_tokens=hist)
    assert out.cpu().tolist() == torch.argmax(15 * torch.tanh(logits / 15), -1).tolist()
    assert masks.cpu().tolist() == [1] * R and hist[:, 1].cpu().tolist() == out.cpu().tolist()
    assert hist[:, 0].cpu().tolist() == [-7] * R
    # bf16 rows wide enough for the 16-byte loads: the soft cap is rounded to bf16 after every operation, as in
    # the reference; the chosen token must carry the maximal capped value (ties are common at 8 bits)
    xb = (torch.randn(5, 1024, generator=torch.Generator().manual_seed(9)) * 30).bfloat16()
    ob = torch.empty(5, dtype=torch.int32, device="cuda")
    ops.sample(xb.cuda(), ob, cap=15.0, temperature=0.0)
    th = torch.tanh((xb.float() / 15).bfloat16().float()).bfloat16()
    zb = (15 * th.float()).bfloat16().float()
    picked = zb[torch.arange(5), ob.cpu().long()]
    assert torch.equal(picked, zb.max(-1).values)
    # two groups of rows with their own schedule; step 1 forces group 0 only
    force = torch.tensor([[-1, 42, -1, -1], [-1, -1, 3, -1]], dtype=torch.int32, device="cuda")
    ops.sample(
        logits.cuda(), out, temperature=0.0, step=step, force_schedule=force, force_group_rows=3, force_group_stride=4,
        out_masks=masks,
    )
    want = torch.argmax(logits, -1).tolist()
    assert out.cpu().tolist() == [42, 42, 42] + want[3:]
    assert masks.cpu().tolist() == [0, 0, 0, 1, 1, 1]


def test_sample_frequencies_follow_softmax():
    """50k draws from one row: empirical frequencies within 0.01 of softmax(l / T)
    (mirrors reference tests/diff_gpt/sampler/test_temperature_sampler.py:95-122)."""
    ops = _ops()
    logits = torch.tensor([[2.0, 1.0, 0.5, -1.0, 0.0, 3.0]])
    n = 50_000
    out = torch.empty(n, dtype=torch.int32, device="cuda")
    for T in (0.5, 1.0, 2.0):
        ops.sample(logits.cuda(), out, R=n, row_stride=0, temperature=T, seed=7)
        freq = torch.bincount(out.cpu().long(), minlength=6).double() / n
        want = torch.softmax(logits[0].double() / T, -1)
        assert (freq - want).abs().max().item() < 0.01, T


@pytest.mark.parametrize("dtype,tol,tag", DT)
@pytest.mark.parametrize("R,H,D,n_splits", [(3, 1, 64, 3), (1, 3, 64, 3), (5, 3, 16, 7), (1, 1, 128, 5)])
def test_decode_attn_split_with_odd_slot_counts(dtype, tol, tag, R, H, D, n_splits):
    """Split-K with an odd R*H*n_splits (odd head counts are legal: reference mha.py:18-20 only asks that
    n_embd % n_head == 0) against the oracle's single-query attention, through a caller workspace and through the
    library's own scratch array."""
    ops = _ops()
    gen = torch.Generator().manual_seed(R * 100 + H * 10 + n_splits)
    pt = 16
    lens = [int(x) for x in torch.randint(1, 900, (R,), generator=gen)]
    lens[0] = 800
    pages = -(-max(lens) // pt)
    k = torch.randn(R, H, pages * pt, D, generator=gen).to(dtype)
    v = torch.randn(R, H, pages * pt, D, generator=gen).to(dtype)
    pool = torch.full((R * pages + 1, 2, H, pt, D), float("nan"), dtype=dtype)
    table = torch.randperm(R * pages, generator=gen).to(torch.int32).view(R, pages)
    for r in range(R):
        for p in range(pages):
            pool[table[r, p], 0] = k[r, :, p * pt : (p + 1) * pt]
            pool[table[r, p], 1] = v[r, :, p * pt : (p + 1) * pt]
    pool = pool.cuda()
    lay = ops.kv_layout(pool[0, 0], pool[0, 1], 2 * H * pt * D, pt * D, pt, table.cuda(), n_pages=R * pages)
    q = torch.randn(R, H * D, generator=gen).to(dtype)
    gate = torch.randn(R, H * D, generator=gen).to(dtype)
    zero = torch.zeros(R, dtype=torch.int32, device="cuda")
    n = torch.tensor(lens, dtype=torch.int32, device="cuda")
    nbytes = ops.decode_attn_workspace_bytes(R, H, D, n_splits)
    assert nbytes % 16 == 0
    ws = torch.empty(nbytes // 4, dtype=torch.float32, device="cuda")
    y = torch.full((R, H * D), float("nan"), dtype=dtype, device="cuda")
    ops.decode_attn(q.cuda(), lay, zero, zero, n, None, y, H=H, D=D, gate=gate.cuda(), workspace=ws, n_splits=n_splits)
    y2 = torch.full_like(y, float("nan"))
    ops.decode_attn_static(q.cuda(), lay, zero, zero, n, None, y2, H=H, D=D, gate=gate.cuda(), n_splits=n_splits)
    torch.cuda.synchronize()
    assert torch.equal(y, y2)
    for r in range(R):
        qh = q[r].view(1, 1, H, D).transpose(1, 2)
        att = ref_math.sdpa(qh, k[r : r + 1, :, : lens[r]], v[r : r + 1, :, : lens[r]], q_offset=10**6)
        want = att.transpose(1, 2).reshape(H * D) * torch.sigmoid(gate[r])
        assert _rel(y[r], want) <= (2e-5 if dtype == torch.float32 else 1.5e-2), r


def test_decode_attn_never_reads_past_the_cache_capacity():
    """Lengths that run past the page table are cut at the capacity: with NaN in every page the row does not own,
    the output stays finite and equals attention over the slots that exist."""
    ops = _ops()
    R, H, D, pt, pages = 3, 2, 64, 8, 4
    gen = torch.Generator().manual_seed(11)
    pool = torch.full((R * pages + 2, 2, H, pt, D), float("nan"), dtype=torch.float32)
    table = (1 + torch.arange(R * pages, dtype=torch.int32)).view(R, pages)
    k = torch.randn(R, H, pages * pt, D, generator=gen)
    v = torch.randn(R, H, pages * pt, D, generator=gen)
    for r in range(R):
        for p in range(pages):
            pool[table[r, p], 0] = k[r, :, p * pt : (p + 1) * pt]
            pool[table[r, p], 1] = v[r, :, p * pt : (p + 1) * pt]
    pool = pool.cuda()
    lay = ops.kv_layout(pool[0, 0], pool[0, 1], 2 * H * pt * D, pt * D, pt, table.cuda(), n_pages=R * pages + 2)
    q = torch.randn(R, H * D, generator=gen)
    zero = torch.zeros(R, dtype=torch.int32, device="cuda")
    n = torch.tensor([pages * pt + 9, pages * pt, 5], dtype=torch.int32, device="cuda")
    for n_splits in (1, 3):
        ws = torch.empty(max(ops.decode_attn_workspace_bytes(R, H, D, n_splits) // 4, 4), dtype=torch.float32, device="cuda")
        y = torch.full((R, H * D), float("nan"), device="cuda")
        ops.decode_attn(q.cuda(), lay, zero, zero, n, None, y, H=H, D=D, workspace=ws, n_splits=n_splits)
        assert torch.isfinite(y).all()
        for r, ln in enumerate([pages * pt, pages * pt, 5]):
            qh = q[r].view(1, 1, H, D).transpose(1, 2)
            want = ref_math.sdpa(qh, k[r : r + 1, :, :ln], v[r : r + 1, :, :ln], q_offset=10**6).transpose(1, 2).reshape(-1)
            assert _rel(y[r], want) <= 2e-5
