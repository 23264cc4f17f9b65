"""CPU restatement of diff-gpt's samplers and Monte-Carlo decode loop (test infrastructure).

ORACLE code: used only by tests, the smoke run and the benchmark's CPU legs.
Pinned against fixtures generated from the unmodified reference
(`tests/golden/make_golden.py`, checked in `tests/test_oracle_golden.py`).

Reference call sites followed:
  * `src/diff_gpt/sampler/temperature.py:17-26` -> `sample_temperature`
  * `src/diff_gpt/sampler/nucleus.py:25-40`     -> `nucleus_mask`, `sample`
  * `src/diff_gpt/model/engine.py:29-169`       -> `mc_decode`
"""

from __future__ import annotations

import torch

from .ref_math import DenseKV, Shape, forward, rope_table


def nucleus_mask(logits: torch.Tensor, p: float) -> torch.Tensor:
    """True where a token is in the top-p set (`nucleus.py:29-37`).

    Probabilities at temperature 1, sorted descending; token i of the sorted
    order is kept iff the cumulative mass BEFORE it is < p (so the first is
    always kept).
    """
    probs = torch.softmax(logits, dim=-1)
    sp, order = torch.sort(probs, dim=-1, descending=True)
    keep_sorted = torch.cumsum(sp, dim=-1) < p
    keep_sorted = torch.cat([torch.ones_like(keep_sorted[..., :1]), keep_sorted[..., :-1]], dim=-1)
    mask = torch.zeros_like(keep_sorted)
    mask.scatter_(-1, order, keep_sorted)
    return mask


def sample_temperature(logits: torch.Tensor, temperature: float, gen: torch.Generator | None) -> torch.Tensor:
    """(B,1) int64: argmax at T == 0, else multinomial(softmax(logits / T)) (`temperature.py:21-25`)."""
    if temperature == 0:
        return torch.argmax(logits, dim=-1, keepdim=True)
    return torch.multinomial(torch.softmax(logits / temperature, dim=-1), 1, generator=gen)


def sample(
    logits: torch.Tensor, temperature: float, top_p: float | None, gen: torch.Generator | None
) -> torch.Tensor:
    """Temperature sampling, optionally restricted to the top-p set decided at T = 1."""
    if top_p is not None:
        logits = logits.masked_fill(~nucleus_mask(logits, top_p), float("-inf"))
    return sample_temperature(logits, temperature, gen)


def mc_decode(
    shape: Shape,
    w: dict[str, torch.Tensor],
    prompt: list[int],
    num_samples: int,
    max_tokens: int,
    temperature: float = 1.0,
    top_p: float | None = None,
    seed: int = 42,
    force_schedule: list[int | None] | None = None,
    keep_logits: bool = False,
):
    """Prefill once, replicate the cache, then sample-or-force step by step (`engine.py:29-154`).

    Returns (tokens [N,G] int64, masks [N,G] int64, logits [G,N,V] or None).
    `logits[g]` are the logits token g was drawn from.  The forward after the
    last token is skipped (its result is never used by the reference either).
    """
    dtype = w["token_embedding_table.weight"].dtype
    table = rope_table(shape.head_dim, 2 * shape.block_size, shape.rope_theta).to(dtype)
    P = len(prompt)
    G = min(max_tokens, max(0, 2 * shape.block_size - P))
    tokens = torch.zeros(num_samples, G, dtype=torch.int64)
    masks = torch.zeros(num_samples, G, dtype=torch.int64)
    if G == 0:
        return tokens, masks, None
    if force_schedule is not None:
        assert len(force_schedule) >= G, "force_schedule must cover all generation steps"
    gen = torch.Generator().manual_seed(seed)
    H, D, L = shape.n_head, shape.head_dim, shape.n_layer
    pre = DenseKV(L, 1, H, P, D)
    logits = forward(shape, w, torch.tensor([prompt]), kv=pre, table=table)[:, -1, :]
    logits = logits.expand(num_samples, -1)
    kv = DenseKV(L, num_samples, H, P + G, D)
    kv.broadcast_from(pre)
    kept = [] if keep_logits else None
    for g in range(G):
        if kept is not None:
            kept.append(logits.float().clone())
        forced = None if force_schedule is None else force_schedule[g]
        if forced is None:
            nxt = sample(logits, temperature, top_p, gen)[:, 0]
            masks[:, g] = 1
        else:
            nxt = torch.full((num_samples,), int(forced), dtype=torch.int64)
        tokens[:, g] = nxt
        if g + 1 < G:
            logits = forward(shape, w, nxt[:, None], kv=kv, table=table)[:, -1, :]
    return tokens, masks, (torch.stack(kept) if kept is not None else None)


def token_nll(shape: Shape, w: dict, tokens: torch.Tensor) -> torch.Tensor:
    """-log p(token_t | tokens before t) for t = 1..N-1 from one forward of the N tokens
    (src/diff_gpt/diff_gpt.py:347-356): log_softmax of the soft-capped logits, gathered at the next token."""
    logits = forward(shape, w, tokens.view(1, -1))[0]
    logp = torch.log_softmax(logits[:-1], dim=-1)
    return -logp.gather(-1, tokens.view(-1)[1:].unsqueeze(-1)).squeeze(-1)
