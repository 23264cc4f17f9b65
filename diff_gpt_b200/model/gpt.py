"""Drop-in `GPT` whose inference forward runs on the libdgpt_b200 kernels.

Same constructor keywords, attributes and state_dict keys as the reference
module (src/diff_gpt/model/gpt.py:79-136), so checkpoints move both ways, and
the same `forward(idx, targets=None, kv_cache=None) -> (logits, loss)` contract
that the reference Engine and DiffGPT facade rely on (gpt.py:140-200).

The sub-modules below are parameter containers: they give the parameters their
reference names and shapes; the arithmetic of a forward pass is enqueued by
`ForwardPlan.run`, which walks the layers and launches

    embed+rmsnorm -> [depth-mix+rmsnorm -> QKVG GEMM -> rope/qk-norm/kv-append ->
    attention (+gate) -> out-proj GEMM -> depth-mix+rmsnorm -> FFN GEMM -> swiglu ->
    FFN GEMM (+residual)] x L -> rmsnorm -> tied-embedding GEMM -> soft-cap

with the GEMMs on cuBLAS (torch.mm / addmm_) and everything else in this
library.  There is no CPU implementation: CPU tensors raise.
"""

from __future__ import annotations

from abc import ABC, abstractmethod
from dataclasses import dataclass

import torch
import torch.nn as nn
import torch.nn.functional as F

from .. import ops
from .._lib import region
from ..sampler.sampler import Sampler
from .kv_cache import KVCache, PagedKVCache
from .rope import precompute_freqs_cis


class BaseGPT(nn.Module, ABC):
    """The seam the Engine and the DiffGPT facade program against (gpt.py:38-76)."""

    def __init__(self, block_size: int, vocab_size: int, n_embd: int, n_head: int, n_layer: int) -> None:
        super().__init__()
        self.block_size = block_size
        self.vocab_size = vocab_size
        self.n_embd = n_embd
        self.n_head = n_head
        self.n_layer = n_layer

    @abstractmethod
    def forward(self, idx, targets=None, kv_cache=None):
        ...

    @abstractmethod
    def generate(self, idx, max_new_tokens, sampler, seed=None):
        ...

    @property
    @abstractmethod
    def device_type(self) -> str:
        ...


# ---- parameter containers (names and shapes of the reference state_dict) -------
class SwiGLU(nn.Module):
    def __init__(self, alpha: float, limit: float) -> None:
        super().__init__()
        self.alpha = alpha
        self.limit = limit

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        out = torch.empty((*x.shape[:-1], x.shape[-1] // 2), dtype=x.dtype, device=x.device)
        ops.swiglu(x.contiguous(), out, self.alpha, self.limit)
        return out


class FeedForward(nn.Module):
    def __init__(self, n_embd: int, swiglu_alpha: float, swiglu_limit: float) -> None:
        super().__init__()
        self.net = nn.Sequential(
            nn.Linear(n_embd, 4 * n_embd, bias=False),
            SwiGLU(alpha=swiglu_alpha, limit=swiglu_limit),
            nn.Linear(2 * n_embd, n_embd, bias=False),
        )


class MultiHeadAttention(nn.Module):
    def __init__(self, n_embd: int, n_head: int, layer_idx: int) -> None:
        super().__init__()
        assert n_embd % n_head == 0
        assert (n_embd // n_head) % 2 == 0  # RoPE rotates pairs
        self.n_embd, self.n_head, self.layer_idx = n_embd, n_head, layer_idx
        self.head_dim = n_embd // n_head
        for name in ("c_q", "c_k", "c_v", "c_g", "c_proj"):
            setattr(self, name, nn.Linear(n_embd, n_embd, bias=False))


class Block(nn.Module):
    def __init__(self, n_embd, n_head, swiglu_alpha, swiglu_limit, layer_idx, layers_per_block=1) -> None:
        super().__init__()
        assert layers_per_block >= 1
        self.layer_idx = layer_idx
        self.layers_per_block = layers_per_block
        self.sa = MultiHeadAttention(n_embd=n_embd, n_head=n_head, layer_idx=layer_idx)
        self.ffwd = FeedForward(n_embd=n_embd, swiglu_alpha=swiglu_alpha, swiglu_limit=swiglu_limit)
        self.attn_res_proj = nn.Linear(n_embd, 1, bias=False)
        self.mlp_res_proj = nn.Linear(n_embd, 1, bias=False)


CACHE_NORMS = True  # depth mix: reuse the norm factors of committed candidates instead of recomputing them
FUSED_FFN = True  # first feed-forward GEMM on the library's tcgen05 kernel with the SwiGLU fused (bf16 only)
FUSED_FFN_MIN_ROWS = 256
# The shared-prompt attention phase while it runs beside the per-row phase: which kernel (an `impl` of
# dgpt_fmha_prefill) and on how many SMs.  Measured per 255 config-4 steps, one process, alternating: the persistent
# kernel with two query tiles per CTA on 64 SMs, which it owns outright (it fills an SM's shared memory and TMEM)
# while the HBM-bound per-row kernel has the other 84 to itself, 1249-1259 ms; on 48 or 80 SMs 1256-1262; the small
# kernel (impl 3) on every SM, one CTA each, sharing the SMs with the per-row kernel, 1271-1275; the persistent kernel
# with one query tile per CTA on 64 SMs 1267-1271, on 40 SMs 1288 (the phase becomes the longer one).
PREFIX_CTAS = 64
PREFIX_IMPL = 4
SIDE_PRIORITY = -1  # stream of the shared-prompt attention phase: ahead of the per-row phase it runs beside


# ---- how one forward call is bound to K/V storage ----------------------------------
@dataclass
class KvBinding:
    """Where the new K/V go and which cached keys each query sees.

    layouts[l]    storage of layer l; its sequence index is the row of `pos0`
    pos0, slot0   int32 [n_seq]: RoPE position / cache slot of the first new token
    step          int32 device scalar added to both (None = 0)
    Prefill / chunk (T >= 1, `decode` False): keys [0, kv_len) with the causal rule j <= q_offset + i.
    Decode (T == 1, `decode` True): row r sees slots [0, len0[r]) and [start1[r], start1[r] + len1[r] + step).
    shared_*      optional shared-prefix phase: rows are grouped `rows_per_series` to a series whose
                  prompt keys live in `shared_layouts[l]` (sequence index = series), lengths `shared_len`.
    """

    layouts: list
    pos0: torch.Tensor
    slot0: torch.Tensor
    step: torch.Tensor | None = None
    decode: bool = False
    kv_len: int = 0
    q_offset: int = 0
    len0: torch.Tensor | None = None
    start1: torch.Tensor | None = None
    len1: torch.Tensor | None = None
    n_splits: int = 1
    shared_layouts: list | None = None
    shared_len: torch.Tensor | None = None
    rows_per_series: int = 0
    fmha_impl: int = 0
    overlap_prefix: bool = False  # run the shared-prompt phase on a second stream beside the per-row phase


class ForwardPlan:
    """Buffers for one (n_seq, T) forward and the launch sequence that fills them.

    `run` only enqueues work on the current stream and reuses the same buffers
    every time, so a plan can be captured into a CUDA graph and replayed.
    """

    def __init__(self, model: "GPT", n_seq: int, T: int, last_only: bool = False, want_logits: bool = True) -> None:
        emb = model.token_embedding_table.weight
        dev, dt = emb.device, emb.dtype
        C, V, L = model.n_embd, model.vocab_size, model.n_layer
        n = n_seq * T
        self.model, self.n_seq, self.T, self.n, self.last_only = model, n_seq, T, n, last_only

        def buf(*shape, dtype=dt):
            return torch.empty(shape, dtype=dtype, device=dev)

        self.x, self.u, self.q, self.y = buf(n, C), buf(n, C), buf(n, C), buf(n, C)
        self.qkvg = buf(n, 4 * C)
        self.parts = [buf(n, C) for _ in range(L)]
        self.act = buf(n, 2 * C)
        n_out = n_seq if last_only else n
        self.xn = buf(n_out, C)
        self.last = buf(n_out, C) if (last_only and T > 1) else None
        self.logits = buf(n_out, V) if want_logits else None
        # the tied-embedding head on the library's tcgen05 GEMM (bf16 with tileable sizes); fp32 stays on cuBLAS
        self.own_head = dt == torch.bfloat16 and C % 8 == 0 and V % 16 == 0
        self.status = torch.zeros(1, dtype=torch.int32, device=dev)
        # tcgen05 GEMM + SwiGLU epilogue: bf16 with tileable sizes, and enough rows to fill the tensor cores
        self.fused_ffn = FUSED_FFN and dt == torch.bfloat16 and C % 8 == 0 and n >= FUSED_FFN_MIN_ROWS
        self.f = None if self.fused_ffn else buf(n, 4 * C)
        # norm factors of committed depth-mix candidates, carried from mix to mix (16-byte rows needed)
        self.cache_norms = CACHE_NORMS and (C * emb.element_size()) % 16 == 0
        self.norm_cache: dict[int, torch.Tensor] = {}
        self.prefix_o = None
        self.prefix_lse = None
        self.part_o = None
        self.part_lse = None
        self.side = None
        self.prefix_on_tc = False
        self.prefix_ctas = 0
        self.workspace = None

    def _mix(self, cands: list, partial: torch.Tensor, w: torch.Tensor, known: set) -> None:
        """Depth mix of the committed candidates and the running block sum into self.u.  A committed candidate no
        longer changes, so the first mix that sees it writes its per-row norm factor and the later ones read it."""
        if not self.cache_norms:
            ops.depthmix(cands + [partial], w, None, self.u)
            return
        inv_in, inv_out, out_index = [], None, -1
        for idx, t in enumerate(cands):
            key = t.data_ptr()
            if key in known:
                inv_in.append(self.norm_cache[key])
            else:
                inv_in.append(None)
                if inv_out is None and not any(c.data_ptr() == key for c in cands[:idx]):
                    buf = self.norm_cache.get(key)
                    if buf is None:
                        buf = self.norm_cache[key] = torch.empty(self.n, dtype=torch.float32, device=t.device)
                    inv_out, out_index = buf, idx
        ops.depthmix_cached(cands + [partial], inv_in + [None], w, None, self.u, inv_out, out_index)
        if inv_out is not None:
            known.add(cands[out_index].data_ptr())

    def _decode_extras(self, b: KvBinding) -> None:
        m = self.model
        H, D = m.n_head, m.n_embd // m.n_head
        dev = self.x.device
        if b.shared_layouts is not None and self.prefix_o is None:
            self.prefix_o = torch.empty((self.n, H, D), dtype=torch.float32, device=dev)
            self.prefix_lse = torch.empty((self.n, H), dtype=torch.float32, device=dev)
        if b.shared_layouts is not None and b.overlap_prefix and b.n_splits == 1 and self.part_o is None:
            self.part_o = torch.empty((self.n, H, D), dtype=torch.float32, device=dev)
            self.part_lse = torch.empty((self.n, H), dtype=torch.float32, device=dev)
            self.side = torch.cuda.Stream(device=dev, priority=SIDE_PRIORITY)
            n_sm = torch.cuda.get_device_properties(dev).multi_processor_count
            self.prefix_ctas = n_sm if PREFIX_CTAS is None else min(PREFIX_CTAS, n_sm)
            # the persistent tensor-core kernel covers bf16 heads of 32, 64 or 128 in pages that tile its 128-key
            # blocks; other models leave the choice to the library (its warp-level kernel)
            pt = int(b.shared_layouts[0].page_tokens)
            self.prefix_on_tc = (
                self.q.dtype == torch.bfloat16 and D in (32, 64, 128) and pt >= 8 and (pt % 128 == 0 or 128 % pt == 0)
            )
        if b.n_splits > 1 and self.workspace is None:
            nbytes = ops.decode_attn_workspace_bytes(self.n, H, D, b.n_splits)
            self.workspace = torch.empty(nbytes // 4, dtype=torch.float32, device=dev)

    def run(self, ids32: torch.Tensor, b: KvBinding) -> torch.Tensor | None:
        m = self.model
        C, H, L = m.n_embd, m.n_head, m.n_layer
        D = C // H
        T, n_seq = self.T, self.n_seq
        W = m.packed_weights()
        if b.decode:
            assert T == 1
            self._decode_extras(b)
        ops.embed_rmsnorm(ids32, W.emb, self.x)
        cands = [self.x]
        partial = self.x
        known: set[int] = set()  # committed candidates whose norm factor has been written during this forward
        for i in range(L):
            lw = W.layers[i]
            if i == 0:
                ops.depthmix([self.x], None, None, self.u)  # single candidate: mix is the identity
            else:
                self._mix(cands, partial, lw.w_attn, known)
            if (i + 1) % m.attn_res_layers_per_block == 0:
                cands = cands + [partial]
                partial = None
            with region("gemm_qkvg"):
                torch.mm(self.u, lw.wqkvg_t, out=self.qkvg)
            qv, kv_, vv, gv = (self.qkvg[:, j * C : (j + 1) * C] for j in range(4))
            ops.rope_qknorm_kvappend(
                qv, kv_, vv, self.q, W.freqs_cis, b.layouts[i], b.pos0, b.slot0, b.step, n_seq, T, H, D, self.status
            )
            if b.decode:
                po = pl = None
                if b.shared_layouts is not None:
                    N = b.rows_per_series
                    prefix_phase = lambda: ops.fmha_prefill(  # noqa: E731
                        self.q, b.shared_layouts[i], self.prefix_o, B=n_seq // N, H=H, Tq=N, D=D,
                        q_batch_stride=N * C, q_row_stride=C, o_batch_stride=N * C, o_row_stride=C,
                        kv_len=b.shared_len, causal=False, lse=self.prefix_lse,
                        impl=PREFIX_IMPL if (self.side is not None and PREFIX_IMPL and self.prefix_on_tc) else b.fmha_impl,
                        status=self.status,
                        max_ctas=self.prefix_ctas if self.side is not None else 0,
                    )
                    po, pl = self.prefix_o, self.prefix_lse
                if po is not None and self.side is not None:
                    # The tensor-core contraction over the shared prompt and the HBM-bound pass over each
                    # row's own tokens need different parts of the SM: run them side by side, then merge.
                    main = torch.cuda.current_stream()
                    self.side.wait_stream(main)
                    with torch.cuda.stream(self.side):
                        prefix_phase()
                    ops.decode_attn_partial(
                        self.q, b.layouts[i], None, b.start1, b.len1, b.step, self.part_o, self.part_lse, H=H, D=D
                    )
                    main.wait_stream(self.side)
                    ops.attn_merge(po, pl, self.part_o, self.part_lse, self.y, H=H, D=D, gate=gv)
                else:
                    if po is not None:
                        prefix_phase()
                    ops.decode_attn(
                        self.q, b.layouts[i], b.len0, b.start1, b.len1, b.step, self.y, H=H, D=D, gate=gv,
                        prefix_o=po, prefix_lse=pl, workspace=self.workspace, n_splits=b.n_splits,
                    )
            else:
                ops.fmha_prefill(
                    self.q, b.layouts[i], self.y, B=n_seq, H=H, Tq=T, D=D, q_batch_stride=T * C, q_row_stride=C,
                    o_batch_stride=T * C, o_row_stride=C, kv_len_all=b.kv_len, q_offset=b.q_offset, causal=True,
                    impl=b.fmha_impl, status=self.status,
                )
                ops.sigmoid_gate(self.y, gv)
            part = self.parts[i]
            with region("gemm_proj"):
                if partial is None:
                    torch.mm(self.y, lw.wproj_t, out=part)
                else:  # layers_per_block > 1: the running block sum keeps accumulating
                    torch.addmm(partial, self.y, lw.wproj_t, out=part)
            partial = part
            self._mix(cands, partial, lw.w_mlp, known)
            if self.fused_ffn:  # first FFN GEMM with the SwiGLU in its epilogue (the [n, 4C] product never reaches HBM)
                ops.linear(self.u, lw.w1, self.act, swiglu=(m.swiglu_alpha, m.swiglu_limit), status=self.status)
            else:
                with region("gemm_ffn1"):
                    torch.mm(self.u, lw.w1_t, out=self.f)
                ops.swiglu(self.f, self.act, m.swiglu_alpha, m.swiglu_limit)
            with region("gemm_ffn2"):  # cuBLAS: 6.6 / 9.8 us for the two n_embd-wide GEMMs against 10.4 / 14.4 us for dgpt_linear
                partial.addmm_(self.act, lw.w2_t)
        final = partial
        if self.last is not None:
            self.last.copy_(partial.view(n_seq, T, C)[:, T - 1, :])
            final = self.last
        ops.depthmix([final], None, None, self.xn)
        if self.logits is None:
            return None
        if self.own_head:
            ops.linear(self.xn, W.emb, self.logits, status=self.status)
        else:
            with region("gemm_logits"):
                torch.mm(self.xn, W.emb.t(), out=self.logits)
        return self.logits


@dataclass
class _LayerWeights:
    w1: torch.Tensor
    wqkvg_t: torch.Tensor
    wproj_t: torch.Tensor
    w1_t: torch.Tensor
    w2_t: torch.Tensor
    w_attn: torch.Tensor
    w_mlp: torch.Tensor


@dataclass
class _Packed:
    emb: torch.Tensor
    freqs_cis: torch.Tensor
    layers: list
    stamp: tuple


class GPT(BaseGPT):
    def __init__(
        self,
        vocab_size: int,
        n_embd: int = 64,
        block_size: int = 32,
        n_head: int = 4,
        n_layer: int = 4,
        rope_theta: float = 10000,
        swiglu_alpha: float = 1.702,
        swiglu_limit: float = 7.0,
        use_checkpoint: bool = True,
        logit_softcap: float = 15.0,
        pad_vocab_size_to: int = 64,
        attn_res_layers_per_block: int = 1,
        label_smoothing_sigma: float = 0.0,
    ) -> None:
        super().__init__(block_size=block_size, vocab_size=vocab_size, n_embd=n_embd, n_head=n_head, n_layer=n_layer)
        assert logit_softcap >= 0, "logit_softcap must be non-negative (0 disables it)"
        assert label_smoothing_sigma >= 0, "label_smoothing_sigma must be non-negative (0 disables it)"
        assert pad_vocab_size_to >= 1, "pad_vocab_size_to must be >= 1"
        assert attn_res_layers_per_block >= 1, "attn_res_layers_per_block must be >= 1"
        assert vocab_size % pad_vocab_size_to == 0, (
            f"vocab_size ({vocab_size}) must be a multiple of "
            f"pad_vocab_size_to ({pad_vocab_size_to}); pad it in the encoder"
        )
        self.token_embedding_table = nn.Embedding(vocab_size, n_embd)
        self.blocks = nn.ModuleList(
            Block(n_embd, n_head, swiglu_alpha, swiglu_limit, layer_idx=i, layers_per_block=attn_res_layers_per_block)
            for i in range(n_layer)
        )
        self.lm_head = nn.Linear(n_embd, vocab_size, bias=False)
        self.lm_head.weight = self.token_embedding_table.weight  # tied
        self.register_buffer(
            "freqs_cis", precompute_freqs_cis(n_embd // n_head, block_size * 2, theta=rope_theta), persistent=False
        )
        self.use_checkpoint = use_checkpoint
        self.logit_softcap = logit_softcap
        self.label_smoothing_sigma = label_smoothing_sigma
        self.swiglu_alpha = swiglu_alpha
        self.swiglu_limit = swiglu_limit
        self.attn_res_layers_per_block = attn_res_layers_per_block
        self._packed: _Packed | None = None

    # ---- weights as the kernels want them -------------------------------------------
    def packed_weights(self) -> _Packed:
        """Fused QKVG weight and transposed views, rebuilt when a parameter was modified or moved."""
        params = [p for p in self.parameters()]
        stamp = tuple((p.data_ptr(), p._version, p.dtype) for p in params) + (self.freqs_cis.data_ptr(),)
        if self._packed is not None and self._packed.stamp == stamp:
            return self._packed
        layers = []
        with torch.no_grad():
            for blk in self.blocks:
                a = blk.sa
                wqkvg = torch.cat([a.c_q.weight, a.c_k.weight, a.c_v.weight, a.c_g.weight], dim=0).contiguous()
                layers.append(
                    _LayerWeights(
                        w1=blk.ffwd.net[0].weight.detach(),
                        wqkvg_t=wqkvg.t(),
                        wproj_t=a.c_proj.weight.detach().t(),
                        w1_t=blk.ffwd.net[0].weight.detach().t(),
                        w2_t=blk.ffwd.net[2].weight.detach().t(),
                        w_attn=blk.attn_res_proj.weight.detach().reshape(-1),
                        w_mlp=blk.mlp_res_proj.weight.detach().reshape(-1),
                    )
                )
            emb = self.token_embedding_table.weight.detach()
            table = self.freqs_cis.to(emb.dtype).contiguous()
        self._packed = _Packed(emb=emb, freqs_cis=table, layers=layers, stamp=stamp)
        return self._packed

    # ---- the reference contract --------------------------------------------------------
    def forward(
        self,
        idx: torch.Tensor,
        targets: torch.Tensor | None = None,
        kv_cache: KVCache | None = None,
    ) -> tuple[torch.Tensor, torch.Tensor | None]:
        if not idx.is_cuda:
            raise RuntimeError("diff_gpt_b200.GPT runs on CUDA only; there is no CPU path")
        if torch.is_grad_enabled() and any(p.requires_grad for p in self.parameters()) and self.training:
            raise NotImplementedError("training (backward) is outside this build; use the reference module to train")
        with torch.no_grad():
            logits = self._infer(idx, kv_cache)
        loss = None
        if targets is not None:
            flat, tgt = logits.view(-1, logits.shape[-1]).float(), targets.view(-1)
            if self.label_smoothing_sigma > 0:
                loss = _ordinal_soft_ce(flat, tgt, self.label_smoothing_sigma)
            else:
                loss = F.cross_entropy(flat, tgt)
        return logits, loss

    def _infer(self, idx: torch.Tensor, kv_cache: KVCache | None) -> torch.Tensor:
        B, T = idx.shape
        C, H, L, V = self.n_embd, self.n_head, self.n_layer, self.vocab_size
        D = C // H
        dev = idx.device
        dt = self.token_embedding_table.weight.dtype
        t0 = 0 if kv_cache is None else kv_cache.get_pos()
        assert t0 + T <= self.freqs_cis.shape[0]
        if kv_cache is None:
            scratch = KVCache(batch_size=B, num_heads=H, seq_len=T, head_dim=D, num_layers=1)
            scratch.ensure(T, dt, dev)
            layouts = [scratch.layer_layout(0)] * L  # every layer reuses the same scratch K/V
            store = scratch
        else:
            assert not isinstance(kv_cache, PagedKVCache), "PagedKVCache is driven by the Engine"
            kv_cache.ensure(t0 + T, dt, dev)
            layouts = [kv_cache.layer_layout(i) for i in range(L)]
            store = kv_cache
        del store
        start = torch.full((B,), t0, dtype=torch.int32, device=dev)
        bind = KvBinding(layouts=layouts, pos0=start, slot0=start, kv_len=t0 + T, q_offset=t0)
        if T == 1 and t0 > 0:
            zeros = torch.zeros(B, dtype=torch.int32, device=dev)
            bind.decode = True
            bind.len0, bind.start1 = zeros, zeros
            bind.len1 = torch.full((B,), t0 + 1, dtype=torch.int32, device=dev)
            n_keys = t0 + 1
            bind.n_splits = _pick_splits(B * H, n_keys)
        plan = ForwardPlan(self, B, T)
        logits = plan.run(idx.reshape(-1).to(torch.int32), bind)
        if self.logit_softcap > 0:
            ops.softcap_(logits, self.logit_softcap)
        if kv_cache is not None:
            kv_cache.pos = t0 + T
        return logits.view(B, T, V)

    @torch.inference_mode()
    def generate(self, idx: torch.Tensor, max_new_tokens: int, sampler: Sampler | None, seed: int | None = None):
        """Naive sliding-window generation without a cache (gpt.py:202-237); kept for API parity."""
        rng = None
        if seed is not None:
            rng = torch.Generator(device=idx.device)
            rng.manual_seed(seed)
        B, T = idx.shape
        out = torch.zeros((B, T + max_new_tokens), dtype=torch.int64, device=idx.device)
        out[:, :T] = idx
        for cur in range(T, T + max_new_tokens):
            window = out[:, max(0, cur - self.block_size) : cur]
            logits = self(window)[0][:, -1]
            if sampler is not None:
                nxt = sampler(logits, rng=rng)
            else:
                nxt = torch.multinomial(F.softmax(logits.float(), dim=-1), num_samples=1, generator=rng)
            out[:, cur] = nxt.reshape(-1)
        return out

    @property
    def device_type(self) -> str:
        return str(self.freqs_cis.device.type)


_SM_COUNT: dict[int, int] = {}


def _sm_count() -> int:
    """Multiprocessors of the current CUDA device (148 on a B200); that figure is assumed where no device is present,
    so the split policy can be examined on a CPU box."""
    if not torch.cuda.is_available():
        return 148
    dev = torch.cuda.current_device()
    if dev not in _SM_COUNT:
        _SM_COUNT[dev] = torch.cuda.get_device_properties(dev).multi_processor_count
    return _SM_COUNT[dev]


def _pick_splits(n_pairs: int, n_keys: int) -> int:
    """Split the keys when (row, head) pairs alone cannot fill the GPU (16 warps on every multiprocessor)."""
    target_warps = _sm_count() * 16
    if n_pairs <= 0 or n_pairs >= target_warps or n_keys < 512:
        return 1
    return max(1, min(-(-target_warps // n_pairs), n_keys // 256, 64))


def _ordinal_soft_ce(logits: torch.Tensor, targets: torch.Tensor, sigma: float, ignore_index: int = -100):
    """Cross entropy against a Gaussian bump of width sigma (in bins) centred on the target bin."""
    keep = targets != ignore_index
    if not bool(keep.any()):
        return logits.sum() * 0.0
    lg, tg = logits[keep], targets[keep]
    bins = torch.arange(lg.shape[-1], device=lg.device, dtype=lg.dtype)
    soft = F.softmax(-((bins[None, :] - tg[:, None].to(lg.dtype)) ** 2) / (2.0 * sigma * sigma), dim=-1)
    return -(soft * F.log_softmax(lg, dim=-1)).sum(dim=-1).mean()
