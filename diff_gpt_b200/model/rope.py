"""Rotary-embedding table and a stand-alone rotation helper.

The decode and prefill paths never call `apply_rotary_emb`: the rotation is
fused with the QK RMSNorm and the cache append in one kernel
(dgpt_rope_qknorm_kvappend).  The helper exists for callers that used the
reference's function of the same name (src/diff_gpt/model/rope.py:4-27).
"""

from __future__ import annotations

import torch


def precompute_freqs_cis(dim: int, end: int, theta: float) -> torch.Tensor:
    """fp32 table (end, dim/2, 2): [m, j] = (cos, sin)(m * theta**(-2j/dim))  (rope.py:30-44)."""
    exponent = torch.arange(0, dim, 2, dtype=torch.float32)[: dim // 2] / dim
    inv_freq = torch.reciprocal(torch.pow(torch.tensor(float(theta)), exponent))
    angle = torch.arange(end, dtype=torch.float32)[:, None] * inv_freq[None, :]
    return torch.stack((torch.cos(angle), torch.sin(angle)), dim=-1)


def apply_rotary_emb(x: torch.Tensor, freqs_cis: torch.Tensor) -> torch.Tensor:
    """Rotate pairs (2j, 2j+1) of the last axis of x by the (cos, sin) pairs of freqs_cis, in fp32."""
    pairs = x.float().unflatten(-1, (-1, 2))
    cos, sin = freqs_cis[..., 0].float(), freqs_cis[..., 1].float()
    even, odd = pairs[..., 0], pairs[..., 1]
    rotated = torch.stack((even * cos - odd * sin, even * sin + odd * cos), dim=-1)
    return rotated.flatten(-2).to(x.dtype)
