"""CPU restatement of diff-gpt's GPT inference forward (test infrastructure).

This file is the ORACLE: a functional, weight-dict based restatement of the
reference's PyTorch inference branch, run on CPU.  It exists only so that the
parity tests, the smoke run and the benchmark's CPU-baseline leg have something
to check the CUDA path against; the product never imports it.

Parity is PINNED: `tests/test_oracle_golden.py` checks every function here
against fixtures under `tests/golden/` that were produced by importing and
running the unmodified reference (`tests/golden/make_golden.py`).

The arithmetic itself lives in PyTorch (a third-party dependency of the
reference, pinned to torch 2.8.0 in its `uv.lock`; this image carries 2.11.0).
The restatement keeps the reference's rounding points: every intermediate that
the reference materialises in the model dtype is materialised in that dtype
here too, so a bf16 run rounds where the reference rounds.

Reference call sites followed (paths inside the reference project):
  * `src/diff_gpt/model/rms_norm.py:5-7`       -> `rms_norm`
  * `src/diff_gpt/model/rope.py:4-44`          -> `rope_table`, `rope`
  * `src/diff_gpt/model/block.py:10-44`        -> `depth_mix`
  * `src/diff_gpt/model/mha.py:31-85`          -> `attention_layer`
  * `src/diff_gpt/model/swi_glu.py:11-19`      -> `swiglu`
  * `src/diff_gpt/model/feed_forward.py:10-18` -> `feed_forward`
  * `src/diff_gpt/model/block.py:87-107`       -> loop body of `forward`
  * `src/diff_gpt/model/gpt.py:140-186`        -> `forward`
  * `src/diff_gpt/model/kv_cache.py:83-116`    -> `DenseKV`
"""

from __future__ import annotations

import math
from dataclasses import dataclass, field

import torch

FLT_EPS = 1.1920928955078125e-07  # torch.finfo(float32).eps, the F.rms_norm default


# ----------------------------------------------------------------------------
# elementary ops
# ----------------------------------------------------------------------------
def rms_norm(x: torch.Tensor) -> torch.Tensor:
    """x * rsqrt(mean(x^2, last dim) + FLT_EPS); fp32 accumulate, output in x.dtype.

    Follows `rms_norm.py:5-7` (F.rms_norm with no weight and eps=None).
    """
    xf = x.float()
    inv = torch.rsqrt(xf.pow(2).mean(dim=-1, keepdim=True) + FLT_EPS)
    return (xf * inv).to(x.dtype)


def rope_table(head_dim: int, length: int, theta: float = 10000.0) -> torch.Tensor:
    """(length, head_dim/2, 2) table of (cos, sin)(m * theta^(-2j/D)), fp32.

    Follows `rope.py:30-44`.
    """
    j = torch.arange(0, head_dim, 2, dtype=torch.float32)[: head_dim // 2]
    inv_freq = 1.0 / (theta ** (j / head_dim))
    m = torch.arange(length, dtype=torch.float32)
    ang = torch.outer(m, inv_freq)
    return torch.stack([ang.cos(), ang.sin()], dim=-1)


def rope(x: torch.Tensor, cs: torch.Tensor) -> torch.Tensor:
    """Rotate interleaved pairs (2j, 2j+1) of x (B,T,H,D) by cs (T,D/2,2).

    Math in fp32 (the table is upcast from whatever dtype it is stored in),
    result rounded back to x.dtype.  Follows `rope.py:20-27`.
    """
    xf = x.float()
    a, b = xf[..., 0::2], xf[..., 1::2]
    c = cs[None, :, None, :, 0].float()
    s = cs[None, :, None, :, 1].float()
    out = torch.empty_like(xf)
    out[..., 0::2] = a * c - b * s
    out[..., 1::2] = a * s + b * c
    return out.to(x.dtype)


def depth_mix(cands: list[torch.Tensor], w: torch.Tensor) -> torch.Tensor:
    """Block Attention Residual: softmax over candidates of rn(v_n).w, then sum a_n v_n.

    Every intermediate stays in the candidates' dtype, as in `block.py:30-43`.
    """
    v = torch.stack(cands, dim=0)
    score = rms_norm(v).matmul(w.reshape(-1))
    a = score.softmax(dim=0).unsqueeze(-1)
    return (a * v).sum(dim=0)


def swiglu(u: torch.Tensor, alpha: float, limit: float) -> torch.Tensor:
    """Interleaved even/odd gated unit with clamps (`swi_glu.py:11-19`)."""
    g = u[..., 0::2].clamp(max=limit)
    lin = u[..., 1::2].clamp(min=-limit, max=limit)
    return g * torch.sigmoid(alpha * g) * (lin + 1)


def sdpa(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, q_offset: int) -> torch.Tensor:
    """softmax(q k^T / sqrt(D) + mask) v with q (B,H,Tq,D), k/v (B,H,Tk,D).

    Key j is visible to query i iff j <= q_offset + i, which covers the three
    branches of `mha.py:61-81`: full causal (q_offset 0, Tq == Tk), one query
    against the whole cache (q_offset Tk-1) and a chunk behind a visible prefix.
    Scores and probabilities are fp32; the output is rounded to q.dtype.
    """
    Tq, Tk, D = q.shape[-2], k.shape[-2], q.shape[-1]
    s = torch.matmul(q.float(), k.float().transpose(-1, -2)) / math.sqrt(D)
    i = torch.arange(Tq)[:, None]
    j = torch.arange(Tk)[None, :]
    s = s.masked_fill(j > (q_offset + i), float("-inf"))
    p = s.softmax(dim=-1)
    return torch.matmul(p, v.float()).to(q.dtype)


# ----------------------------------------------------------------------------
# dense replicated KV store (the reference layout)
# ----------------------------------------------------------------------------
@dataclass
class DenseKV:
    """(L, 2, B, H, T, D) store with a single write cursor (`kv_cache.py:4-116`)."""

    n_layer: int
    batch: int
    n_head: int
    capacity: int
    head_dim: int
    pos: int = 0
    data: torch.Tensor | None = field(default=None, repr=False)

    def append(self, layer: int, k: torch.Tensor, v: torch.Tensor):
        if self.data is None:
            self.data = torch.zeros(
                self.n_layer, 2, self.batch, self.n_head, self.capacity, self.head_dim, dtype=k.dtype
            )
        t0, t1 = self.pos, self.pos + k.shape[2]
        assert t1 <= self.capacity
        self.data[layer, 0, :, :, t0:t1] = k
        self.data[layer, 1, :, :, t0:t1] = v
        if layer == self.n_layer - 1:
            self.pos = t1
        return self.data[layer, 0, :, :, :t1], self.data[layer, 1, :, :, :t1]

    def broadcast_from(self, other: "DenseKV") -> None:
        """Replicate a batch-1 prompt store into every row (`kv_cache.py:35-81`)."""
        assert other.data is not None and self.data is None
        self.data = torch.zeros(
            self.n_layer, 2, self.batch, self.n_head, self.capacity, self.head_dim, dtype=other.data.dtype
        )
        self.data[:, :, :, :, : other.pos] = other.data[:, :, :, :, : other.pos]
        self.pos = other.pos


# ----------------------------------------------------------------------------
# the model
# ----------------------------------------------------------------------------
@dataclass
class Shape:
    vocab_size: int
    n_embd: int
    n_head: int
    n_layer: int
    block_size: int
    rope_theta: float = 10000.0
    swiglu_alpha: float = 1.702
    swiglu_limit: float = 7.0
    logit_softcap: float = 15.0

    @property
    def head_dim(self) -> int:
        return self.n_embd // self.n_head


def random_weights(shape: Shape, seed: int, dtype: torch.dtype, std: float = 0.02) -> dict[str, torch.Tensor]:
    """Every parameter ~ N(0, std) from torch.Generator(seed); names as in the reference state_dict."""
    g = torch.Generator().manual_seed(seed)
    C, V = shape.n_embd, shape.vocab_size

    def n(*s):
        return (torch.randn(*s, generator=g) * std).to(dtype)

    w = {"token_embedding_table.weight": n(V, C)}
    for i in range(shape.n_layer):
        p = f"blocks.{i}."
        for name in ("c_q", "c_k", "c_v", "c_g", "c_proj"):
            w[p + f"sa.{name}.weight"] = n(C, C)
        w[p + "ffwd.net.0.weight"] = n(4 * C, C)
        w[p + "ffwd.net.2.weight"] = n(C, 2 * C)
        w[p + "attn_res_proj.weight"] = n(1, C)
        w[p + "mlp_res_proj.weight"] = n(1, C)
    return w


def attention_layer(
    shape: Shape,
    w: dict[str, torch.Tensor],
    layer: int,
    u: torch.Tensor,
    cs: torch.Tensor,
    kv: DenseKV | None,
) -> torch.Tensor:
    """QKVG projections, RoPE, QK-norm, cache append, SDPA, sigmoid gate, out-proj (`mha.py:31-85`)."""
    B, T, C = u.shape
    H, D = shape.n_head, shape.head_dim
    p = f"blocks.{layer}.sa."
    q = (u @ w[p + "c_q.weight"].T).view(B, T, H, D)
    k = (u @ w[p + "c_k.weight"].T).view(B, T, H, D)
    v = (u @ w[p + "c_v.weight"].T).view(B, T, H, D)
    g = u @ w[p + "c_g.weight"].T
    q = rms_norm(rope(q, cs)).transpose(1, 2)
    k = rms_norm(rope(k, cs)).transpose(1, 2)
    v = v.transpose(1, 2)
    if kv is not None:
        k, v = kv.append(layer, k, v)
    y = sdpa(q, k, v, q_offset=k.shape[2] - T)
    y = y.transpose(1, 2).reshape(B, T, C)
    y = y * torch.sigmoid(g)
    return y @ w[p + "c_proj.weight"].T


def feed_forward(shape: Shape, w: dict[str, torch.Tensor], layer: int, u: torch.Tensor) -> torch.Tensor:
    p = f"blocks.{layer}.ffwd."
    hidden = swiglu(u @ w[p + "net.0.weight"].T, shape.swiglu_alpha, shape.swiglu_limit)
    return hidden @ w[p + "net.2.weight"].T


def forward(
    shape: Shape,
    w: dict[str, torch.Tensor],
    idx: torch.Tensor,
    kv: DenseKV | None = None,
    table: torch.Tensor | None = None,
    last_only: bool = False,
) -> torch.Tensor:
    """Logits (B,T,V) of the inference branch, layers_per_block = 1 (`gpt.py:140-186`).

    `table` is the (2*block_size, D/2, 2) RoPE table in the MODEL dtype (the
    reference's `.to(bfloat16)` rounds its non-persistent buffer as well).
    """
    B, T = idx.shape
    dtype = w["token_embedding_table.weight"].dtype
    if table is None:
        table = rope_table(shape.head_dim, 2 * shape.block_size, shape.rope_theta).to(dtype)
    t0 = 0 if kv is None else kv.pos
    assert t0 + T <= table.shape[0]
    cs = table[t0 : t0 + T]
    x = rms_norm(w["token_embedding_table.weight"][idx])
    committed = [x]
    partial = x
    for i in range(shape.n_layer):
        pre = f"blocks.{i}."
        # first mix of layer 0 has a single distinct candidate -> identity (block.py:27-28)
        h = x if i == 0 else depth_mix(committed + [partial], w[pre + "attn_res_proj.weight"])
        committed = committed + [partial]  # commit at every layer; (x, x) after layer 0
        attn_out = attention_layer(shape, w, i, rms_norm(h), cs, kv)
        partial = attn_out
        h2 = depth_mix(committed + [partial], w[pre + "mlp_res_proj.weight"])
        partial = partial + feed_forward(shape, w, i, rms_norm(h2))
    if last_only:
        partial = partial[:, -1:, :]
    logits = rms_norm(partial) @ w["token_embedding_table.weight"].T
    if shape.logit_softcap > 0:
        logits = shape.logit_softcap * torch.tanh(logits / shape.logit_softcap)
    return logits


def attention_only(
    q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, table: torch.Tensor, w_proj: torch.Tensor | None
) -> torch.Tensor:
    """Long-context prefill attention with inputs injected after the projections.

    q, k, v are (B,T,H,D); RoPE + QK-norm, causal SDPA, optional out-proj;
    i.e. `mha.py:44-48,64,83,85` without gate.
    """
    B, T, H, D = q.shape
    cs = table[:T]
    qh = rms_norm(rope(q, cs)).transpose(1, 2)
    kh = rms_norm(rope(k, cs)).transpose(1, 2)
    y = sdpa(qh, kh, v.transpose(1, 2), q_offset=0).transpose(1, 2).reshape(B, T, H * D)
    return y if w_proj is None else y @ w_proj.T
