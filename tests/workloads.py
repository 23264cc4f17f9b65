"""Seeded synthetic inputs of the BASELINE configurations, shared by the GPU tests.

Weights come from `oracle.ref_math.random_weights` (one torch.Generator per seed, tensors drawn in a fixed
order), prompts from the series below run through the host tokeniser.
"""

from __future__ import annotations

import numpy as np
import torch

from oracle import ref_math

CFG3 = dict(vocab_size=1024, n_embd=512, n_head=8, n_layer=6, block_size=4096)
CFG4 = dict(vocab_size=4096, n_embd=768, n_head=12, n_layer=12, block_size=2048)


def weights(cfg: dict, seed: int, dtype: torch.dtype, std: float = 0.02) -> dict:
    return ref_math.random_weights(ref_math.Shape(**cfg), seed=seed, dtype=dtype, std=std)


def gpu_model(cfg: dict, w: dict, dtype: torch.dtype):
    from diff_gpt_b200 import GPT

    m = GPT(**cfg).eval()
    sd = dict(w)
    sd["lm_head.weight"] = sd["token_embedding_table.weight"]
    m.load_state_dict(sd)
    return m.to(dtype).cuda()


def cfg4_prompts(n_series: int, points: int = 1025) -> list[list[int]]:
    """Config 4's series: random walk (step sd 0.5) + sin(2 pi t / 24), order-1 tokens (points - 1 per series)."""
    from diff_gpt_b200.encoder_decoder import encode, get_domain_of_definition

    rng = np.random.default_rng(4)
    t = np.arange(points)
    out = []
    for _ in range(n_series):
        x = (np.cumsum(rng.normal(0.0, 0.5, t.size)) + np.sin(2 * np.pi * t / 24.0)).reshape(-1, 1)
        dom = get_domain_of_definition(x, 1, use_decimal=False)
        _, _, tok = encode(inp=x, vocab_size=CFG4["vocab_size"], domain_of_definition=dom, order_of_derivative=1,
                           use_decimal=False)
        out.append(tok.reshape(-1).astype(np.int64).tolist())
    return out


def cfg3_frames(n_series: int, rows: int, seed: int = 3) -> list[np.ndarray]:
    """Config 3's series: 7 channels, each the sum of 3 sinusoids (periods 12..168, amplitudes U(0.5, 2)) plus
    AR(1) noise (phi 0.8, sd 0.1)."""
    rng = np.random.default_rng(seed)
    out = []
    for _ in range(n_series):
        t = np.arange(rows)[:, None]
        periods = rng.integers(12, 169, size=(3, 7))
        amps = rng.uniform(0.5, 2.0, size=(3, 7))
        x = sum(amps[i] * np.sin(2 * np.pi * t / periods[i]) for i in range(3))
        e = rng.normal(0, 0.1, size=(rows, 7))
        noise = np.zeros((rows, 7))
        for i in range(1, rows):
            noise[i] = 0.8 * noise[i - 1] + e[i]
        out.append((x + noise).astype(np.float64))
    return out


CFG3_ORDERS = np.array([0, 1, 1, 2, 2, 1, 0])


def cfg3_tokens(frame: np.ndarray) -> list[int]:
    """A config-3 frame as row-major (time, channel) tokens with the per-column orders of the config."""
    from diff_gpt_b200.encoder_decoder import encode, get_domain_of_definition

    dom = get_domain_of_definition(frame, CFG3_ORDERS, use_decimal=False)
    _, _, tok = encode(inp=frame, vocab_size=CFG3["vocab_size"], domain_of_definition=dom,
                       order_of_derivative=CFG3_ORDERS, use_decimal=False)
    return tok.reshape(-1).astype(np.int64).tolist()
