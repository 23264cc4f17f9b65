"""Weight-free RMSNorm over the last axis (reference: src/diff_gpt/model/rms_norm.py:5-7)."""

from __future__ import annotations

import torch

from .. import ops


def rms_norm(x: torch.Tensor) -> torch.Tensor:
    """x * rsqrt(mean(x^2) + FLT_EPSILON), fp32 accumulation, output in x.dtype (CUDA only)."""
    src = x.contiguous()
    out = torch.empty_like(src)
    ops.depthmix([src.view(-1, src.shape[-1])], None, None, out.view(-1, src.shape[-1]))
    return out
