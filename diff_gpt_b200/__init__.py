"""B200-native attention forward and KV-cache Monte-Carlo decode for diff-gpt.

Mirrors the reference's import surface for this path:

    from diff_gpt_b200 import GPT, KVCache, Engine, TemperatureSampler, NucleusSampler

The CUDA library (libdgpt_b200.so, built by `python diff_gpt_b200/build.py`) is
required at import time; there is no CPU or PyTorch fallback.
"""

from . import _lib  # noqa: F401  (raises if the shared object is missing)
from .model.engine import Engine
from .model.gpt import GPT, BaseGPT
from .model.kv_cache import KVCache, PagedKVCache
from .sampler.nucleus import NucleusSampler
from .sampler.sampler import Sampler
from .sampler.temperature import TemperatureSampler

__all__ = [
    "GPT", "BaseGPT", "KVCache", "PagedKVCache", "Engine", "Sampler", "TemperatureSampler", "NucleusSampler",
]
