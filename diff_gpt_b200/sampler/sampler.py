"""Sampler protocol (reference: src/diff_gpt/sampler/sampler.py:4-11)."""

from __future__ import annotations

import torch


class Sampler:
    """Maps logits [..., n_tokens] to token ids [..., 1] (int64)."""

    def __call__(self, logits: torch.Tensor, rng: torch.Generator | None = None) -> torch.Tensor:
        raise NotImplementedError()

    def native_spec(self) -> tuple[float, float] | None:
        """(temperature, top_p) if the fused sampling kernel can stand in for this object, else None."""
        return None


def draw_seed(rng: torch.Generator | None) -> int:
    """A 63-bit seed for the counter-based generator, advancing `rng` so successive calls differ."""
    if rng is None:
        return int(torch.randint(0, 2**62, (1,)).item())
    cpu = rng if rng.device.type == "cpu" else None
    if cpu is not None:
        return int(torch.randint(0, 2**62, (1,), generator=cpu).item())
    return int(torch.randint(0, 2**62, (1,), generator=rng, device=rng.device).item())
