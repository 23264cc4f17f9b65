"""Temperature sampler on the fused sampling kernel.

Same constructor and call contract as the reference
(src/diff_gpt/sampler/temperature.py:6-26): temperature 0 is argmax, otherwise a
draw from softmax(logits / T).  The draw uses the library's counter-based Philox
stream seeded from `rng`, so equal generator states give equal tokens, but the
stream is not bit-identical to torch.multinomial's.
"""

from __future__ import annotations

import torch

from .. import ops
from .sampler import Sampler, draw_seed


class TemperatureSampler(Sampler):
    __slots__ = "temperature"

    def __init__(self, temperature: float = 1.0) -> None:
        self.temperature = temperature

    def native_spec(self) -> tuple[float, float] | None:
        return (float(self.temperature), 1.0)

    def __call__(self, logits: torch.Tensor, rng: torch.Generator | None = None) -> torch.Tensor:
        return _native_sample(logits, float(self.temperature), 1.0, rng)


def _native_sample(logits: torch.Tensor, temperature: float, top_p: float, rng) -> torch.Tensor:
    lead = logits.shape[:-1]
    flat = logits.reshape(-1, logits.shape[-1])
    if flat.stride(-1) != 1:
        flat = flat.contiguous()
    out = torch.empty(flat.shape[0], dtype=torch.int32, device=logits.device)
    seed = 0 if temperature == 0 else draw_seed(rng)
    ops.sample(flat, out, R=flat.shape[0], row_stride=flat.stride(0), temperature=temperature, top_p=top_p, seed=seed)
    return out.to(torch.int64).view(*lead, 1)
