"""Split-K decode attention without a caller workspace (`dgpt_decode_attn_static`).

Some hosts cannot allocate device memory at the point where they launch: a server whose memory is
handed out once at start-up, a plugin that owns nothing but its input and output buffers.  For them the
library keeps the split-K partials in a fixed array of its own.  This file checks, through the C ABI,
that the variant gives the same numbers as `dgpt_decode_attn` with a caller workspace — twice in a
row with different inputs, since both calls reuse the same array and it keeps the earlier contents —
and that a request larger than the array is refused.  It is collected last so that a failure here
cannot hide the result of any other test.
"""

import pytest
import torch

pytestmark = pytest.mark.gpu


def _case(ops, seed, dtype, R, H, D, pt, lens):
    gen = torch.Generator().manual_seed(seed)
    pages = -(-max(lens) // pt)
    pool = (torch.randn(R * pages, 2, H, pt, D, generator=gen) * 0.7).to(dtype).cuda()
    table = torch.randperm(R * pages, generator=gen).to(torch.int32).view(R, pages).cuda()
    lay = ops.kv_layout(pool[0, 0], pool[0, 1], 2 * H * pt * D, pt * D, pt, table, n_pages=R * pages)
    q = torch.randn(R, H * D, generator=gen).to(dtype).cuda()
    gate = torch.randn(R, H * D, generator=gen).to(dtype).cuda()
    zero = torch.zeros(R, dtype=torch.int32, device="cuda")
    n = torch.tensor(lens, dtype=torch.int32, device="cuda")
    return lay, q, gate, zero, n


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("H,n_splits", [(4, 5), (3, 3)])
def test_static_scratch_matches_caller_workspace_twice(dtype, H, n_splits):
    from diff_gpt_b200 import ops

    R, D, pt = (6, 64, 16) if H == 4 else (5, 64, 16)  # the second shape has an odd number of (split, row, head) slots
    for seed, lens in ((1, [200, 37, 1, 129, 64, 333][:R]), (2, [5, 400, 77, 16, 250, 31][:R])):
        lay, q, gate, zero, n = _case(ops, seed, dtype, R, H, D, pt, lens)
        want = torch.empty_like(q)
        ws = torch.empty(ops.decode_attn_workspace_bytes(R, H, D, n_splits) // 4, dtype=torch.float32, device="cuda")
        ops.decode_attn(q, lay, zero, zero, n, None, want, H=H, D=D, gate=gate, workspace=ws, n_splits=n_splits)
        got = torch.full_like(q, float("nan"))
        ops.decode_attn_static(q, lay, zero, zero, n, None, got, H=H, D=D, gate=gate, n_splits=n_splits)
        torch.cuda.synchronize()
        assert torch.equal(got, want), (seed, (got.float() - want.float()).abs().max().item())
        single = torch.empty_like(q)
        ops.decode_attn(q, lay, zero, zero, n, None, single, H=H, D=D, gate=gate)
        tol = 2e-5 if dtype == torch.float32 else 1.5e-2
        assert (got.float() - single.float()).abs().max().item() <= tol * single.float().abs().max().item()


def test_static_scratch_refuses_what_does_not_fit():
    from diff_gpt_b200 import _lib, ops

    cap = ops.decode_attn_static_capacity_bytes()
    assert cap == 16 << 20
    R, H, D, pt = 4096, 12, 64, 16
    n_splits = cap // (R * H * (D + 2) * 4) + 1
    lay, q, gate, zero, n = _case(ops, 3, torch.bfloat16, 2, H, D, pt, [8, 8])
    big_q = torch.zeros(R, H * D, dtype=torch.bfloat16, device="cuda")
    y = torch.empty_like(big_q)
    z = torch.zeros(R, dtype=torch.int32, device="cuda")
    with pytest.raises(_lib.DgptError, match="built-in scratch"):
        ops.decode_attn_static(big_q, lay, z, z, z, None, y, H=H, D=D, n_splits=n_splits)
