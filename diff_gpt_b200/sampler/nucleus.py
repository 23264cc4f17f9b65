"""Top-p (nucleus) sampler on the fused kernels.

Same constructor and call contract as the reference
(src/diff_gpt/sampler/nucleus.py:7-40): the nucleus is decided at temperature 1
on the logits it is given — tokens in descending probability order are kept
while the mass before them is below p — and the inner sampler then draws from
the kept tokens.  With a `TemperatureSampler` inside, filter and draw are one
kernel; any other inner sampler receives logits with -inf outside the nucleus.
"""

from __future__ import annotations

import torch

from .. import ops
from .sampler import Sampler
from .temperature import TemperatureSampler, _native_sample


class NucleusSampler(Sampler):
    __slots__ = ("p", "sampler")

    def __init__(self, p: float, sampler: Sampler) -> None:
        self.p = p
        self.sampler = sampler

    def native_spec(self) -> tuple[float, float] | None:
        if type(self.sampler) is TemperatureSampler:
            return (float(self.sampler.temperature), float(self.p))
        return None

    def __call__(self, logits: torch.Tensor, rng: torch.Generator | None = None) -> torch.Tensor:
        spec = self.native_spec()
        if spec is not None:
            return _native_sample(logits, spec[0], spec[1], rng)
        return self.sampler(ops.nucleus_filter(logits, float(self.p)), rng=rng)
