"""dgpt_linear (tcgen05 GEMM with the SwiGLU epilogue) against an exact matmul of the same bf16 operands."""

import pytest
import torch

from oracle import ref_math

pytestmark = pytest.mark.gpu


def _operands(M, N, K, seed):
    g = torch.Generator().manual_seed(seed)
    a = torch.randn(M, K, generator=g).bfloat16()
    w = (torch.randn(N, K, generator=g) * 0.05).bfloat16()
    return a, w


@pytest.mark.parametrize(
    "M,N,K",
    [(128, 256, 64), (4096, 3072, 768), (300, 272, 200), (1, 16, 8), (129, 528, 1000), (2048, 768, 1536)],
)
def test_plain_store(M, N, K):
    """Full tiles, ragged edges in every dimension (zero-filled by TMA), one row, more tiles than SMs."""
    from diff_gpt_b200 import ops

    a, w = _operands(M, N, K, M + N + K)
    out = torch.full((M, N), float("nan"), dtype=torch.bfloat16, device="cuda")
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    ops.linear(a.cuda(), w.cuda(), out, status=status)
    want = a.double() @ w.double().T
    assert status.item() == 0
    assert torch.isfinite(out).all()
    err = (out.cpu().double() - want).abs().max().item()
    assert err <= 6e-3 * want.abs().max().item(), (err, want.abs().max().item())


@pytest.mark.parametrize("M,N,K", [(128, 256, 64), (4096, 3072, 768), (77, 96, 136)])
def test_swiglu_epilogue_equals_gemm_then_swiglu(M, N, K):
    """Epilogue 1 = the library's own SwiGLU kernel applied to epilogue 0's output, bit for bit; and the oracle's
    SwiGLU of the exact product within bf16 rounding."""
    from diff_gpt_b200 import ops

    a, w = _operands(M, N, K, 7 * M + K)
    w = w * 8  # reach the clamp at 7 in a few places
    plain = torch.empty((M, N), dtype=torch.bfloat16, device="cuda")
    ops.linear(a.cuda(), w.cuda(), plain)
    two_step = torch.empty((M, N // 2), dtype=torch.bfloat16, device="cuda")
    ops.swiglu(plain, two_step, 1.702, 7.0)
    fused = torch.full((M, N // 2), float("nan"), dtype=torch.bfloat16, device="cuda")
    ops.linear(a.cuda(), w.cuda(), fused, swiglu=(1.702, 7.0))
    assert torch.equal(fused, two_step)
    want = ref_math.swiglu((a.double() @ w.double().T).bfloat16(), 1.702, 7.0).float()
    err = (fused.cpu().float() - want).abs().max().item()
    assert err <= 3e-2 * want.abs().max().item()


def test_strided_operands_and_back_to_back_launches():
    """Row slices of wider buffers (as the fused QKVG buffer is used) and repeated launches on one stream."""
    from diff_gpt_b200 import ops

    g = torch.Generator().manual_seed(3)
    big_a = torch.randn(500, 4 * 128, generator=g).bfloat16().cuda()
    w = (torch.randn(256, 128, generator=g) * 0.1).bfloat16().cuda()
    big_out = torch.zeros(500, 3 * 256, dtype=torch.bfloat16, device="cuda")
    a = big_a[:, 128:256]
    for _ in range(3):
        ops.linear(a, w, big_out[:, 256:512])
    want = a.double().cpu() @ w.double().cpu().T
    assert (big_out[:, 256:512].cpu().double() - want).abs().max().item() <= 6e-3 * want.abs().max().item()
    assert big_out[:, :256].abs().max().item() == 0 and big_out[:, 512:].abs().max().item() == 0


def test_rejects_what_it_cannot_tile():
    from diff_gpt_b200 import ops
    from diff_gpt_b200._lib import DgptError

    a = torch.zeros(8, 12, dtype=torch.bfloat16, device="cuda")  # K = 12 is not a multiple of 8
    w = torch.zeros(16, 12, dtype=torch.bfloat16, device="cuda")
    with pytest.raises(DgptError):
        ops.linear(a, w, torch.zeros(8, 16, dtype=torch.bfloat16, device="cuda"))
    with pytest.raises(DgptError):  # fp32 is not built
        ops.linear(a.float()[:, :8].contiguous(), w.float()[:, :8].contiguous(), torch.zeros(8, 16, device="cuda"))


@pytest.mark.parametrize("M,N,K", [(4096, 768, 768), (4096, 768, 1536), (300, 400, 136), (2048, 128, 64)])
def test_add_epilogue_in_place_and_narrow_tiles(M, N, K):
    """out = resid + a @ w.T with one rounding, in place and into another buffer; N = 768 / 400 / 128 pick the
    192- and 128-wide tiles."""
    from diff_gpt_b200 import ops

    a, w = _operands(M, N, K, 3 * M + N)
    g = torch.Generator().manual_seed(5)
    resid = torch.randn(M, N, generator=g).bfloat16()
    want = (resid.double() + a.double() @ w.double().T)
    other = torch.full((M, N), float("nan"), dtype=torch.bfloat16, device="cuda")
    r_dev = resid.cuda()
    ops.linear(a.cuda(), w.cuda(), other, add=r_dev)
    assert torch.equal(r_dev.cpu(), resid)  # the addend is only read
    in_place = resid.cuda()
    ops.linear(a.cuda(), w.cuda(), in_place, add=in_place)
    assert torch.equal(in_place, other)
    err = (other.cpu().double() - want).abs().max().item()
    assert err <= 6e-3 * want.abs().max().item()
    ref = torch.addmm(resid.cuda(), a.cuda(), w.cuda().t())  # cuBLAS: same single rounding, other summation order
    assert (other.float() - ref.float()).abs().max().item() <= 2e-2 * want.abs().max().item()


@pytest.mark.parametrize("mode", ["plain", "swiglu", "add"])
def test_every_output_within_one_bf16_step_of_the_exact_product_and_repeats_bit_for_bit(mode):
    """The decode step's shape (4096 x 768 -> 3072, 384 tiles over 148 persistent CTAs, two accumulators in turn): every
    element against the fp64 product of the same bf16 operands, with a bound of one bf16 rounding step of the value
    plus the fp32 accumulation error, and five more launches that must reproduce the first bit for bit - an epilogue
    that reads an accumulator a tile late or early shows up as a few wrong elements in one launch out of several."""
    from diff_gpt_b200 import ops

    M, N, K = 4096, 3072, 768
    a, w = _operands(M, N, K, 99)
    a, w = a.cuda(), w.cuda()
    resid = torch.randn((M, N), device="cuda", generator=torch.Generator(device="cuda").manual_seed(5)).bfloat16()
    status = torch.zeros(1, dtype=torch.int32, device="cuda")

    def run():
        if mode == "swiglu":
            out = torch.full((M, N // 2), float("nan"), dtype=torch.bfloat16, device="cuda")
            ops.linear(a, w * 8, out, swiglu=(1.702, 7.0), status=status)
        elif mode == "add":
            out = torch.full((M, N), float("nan"), dtype=torch.bfloat16, device="cuda")
            ops.linear(a, w, out, add=resid, status=status)
        else:
            out = torch.full((M, N), float("nan"), dtype=torch.bfloat16, device="cuda")
            ops.linear(a, w, out, status=status)
        return out

    first = run()
    assert status.item() == 0 and torch.isfinite(first).all()
    if mode != "swiglu":  # (the SwiGLU form is pinned bit for bit to the plain form + the SwiGLU kernel by the test above)
        want = a.double() @ w.double().T
        if mode == "add":
            want = want + resid.double()
        excess = (first.double() - want).abs() - (2.0**-8 * want.abs() + 1e-4)
        assert excess.max().item() <= 0.0, excess.argmax().item()
    for _ in range(5):
        assert torch.equal(run(), first)
