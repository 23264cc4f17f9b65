"""The mbarrier wait used by the tcgen05 kernels gives up after its cycle limit and reports which wait it was.

The failure is made by NOT arriving on a barrier (nothing faults, traps or spins without a limit): the kernel
returns normally and the context stays usable, which the last lines check by running real work afterwards."""

import pytest
import torch

pytestmark = pytest.mark.gpu


def test_wait_succeeds_when_the_arrival_comes_and_gives_up_when_it_does_not():
    from diff_gpt_b200 import _lib, ops

    out = torch.full((4,), -1, dtype=torch.int32, device="cuda")
    stream = torch.cuda.current_stream().cuda_stream
    _lib.check(_lib.lib.dgpt_bounded_wait_probe(1, 100_000_000, out.data_ptr(), stream))
    ok0, ok1, flag, cycles = out.cpu().tolist()
    assert (ok0, ok1, flag) == (1, 1, 0) and cycles < 1_000_000

    limit = 50_000_000  # about 25 ms
    _lib.check(_lib.lib.dgpt_bounded_wait_probe(0, limit, out.data_ptr(), stream))
    ok0, ok1, flag, cycles = out.cpu().tolist()
    assert (ok0, ok1) == (0, 0)
    assert flag == 40  # the first thread's wait is the one that ran out; the second left on seeing the flag
    assert limit <= cycles < 3 * limit

    with pytest.raises(_lib.DgptError):
        _lib.check(_lib.lib.dgpt_bounded_wait_probe(0, 0, out.data_ptr(), stream))
    # the context is intact: a tensor-core kernel with the same waits runs and reports no problem
    a = torch.randn(256, 128, device="cuda").bfloat16()
    w = torch.randn(256, 128, device="cuda").bfloat16()
    o = torch.empty(256, 256, device="cuda", dtype=torch.bfloat16)
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    ops.linear(a, w, o, status=status)
    assert status.item() == 0
    assert (o.float() - a.float() @ w.float().T).abs().max().item() <= 0.02 * (a.float() @ w.float().T).abs().max().item()
