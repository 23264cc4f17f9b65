"""Tensor-level wrappers over the C ABI (include/dgpt.h).

Each function takes CUDA torch tensors, extracts raw device pointers, strides
and the current stream, and enqueues one library call.  Nothing here computes
on the host and nothing falls back to torch ops: a CPU tensor is an error.
"""

from __future__ import annotations

import ctypes as C
import math

import torch

from . import _lib
from ._lib import KvLayout, check, lib

_DT = {torch.float32: _lib.F32, torch.bfloat16: _lib.BF16}


def dtype_code(t: torch.Tensor) -> int:
    try:
        return _DT[t.dtype]
    except KeyError:
        raise TypeError(f"unsupported dtype {t.dtype}: float32 and bfloat16 are built") from None


def _cuda(*ts: torch.Tensor | None) -> None:
    for t in ts:
        if t is not None and not t.is_cuda:
            raise RuntimeError("diff_gpt_b200 kernels run on CUDA tensors only (no CPU path)")


def _ptr(t: torch.Tensor | None) -> int | None:
    return None if t is None else t.data_ptr()


def _stream() -> int:
    return torch.cuda.current_stream().cuda_stream


def kv_layout(
    k: torch.Tensor,
    v: torch.Tensor,
    page_stride: int,
    head_stride: int,
    page_tokens: int,
    page_table: torch.Tensor | None = None,
    n_pages: int = 0,
) -> KvLayout:
    """Descriptor of one layer's K/V storage; `k`/`v` are views whose first element is the base."""
    _cuda(k, v, page_table)
    lay = KvLayout()
    lay.n_pages = n_pages
    lay.k_base = k.data_ptr()
    lay.v_base = v.data_ptr()
    lay.page_stride = page_stride
    lay.head_stride = head_stride
    lay.page_table = _ptr(page_table)
    lay.page_tokens = page_tokens
    lay.max_pages = 0 if page_table is None else page_table.shape[-1]
    lay._keep = (k, v, page_table)  # the struct holds raw addresses: keep their owners alive with it
    return lay


def embed_rmsnorm(ids: torch.Tensor, emb: torch.Tensor, out: torch.Tensor) -> None:
    _cuda(ids, emb, out)
    assert ids.dtype == torch.int32 and ids.is_contiguous() and emb.is_contiguous() and out.is_contiguous()
    V, Cdim = emb.shape
    check(lib.dgpt_embed_rmsnorm(ids.data_ptr(), emb.data_ptr(), out.data_ptr(), ids.numel(), Cdim, V, dtype_code(emb), _stream()))


def depthmix(
    cands: list[torch.Tensor],
    w: torch.Tensor | None,
    out_h: torch.Tensor | None,
    out_rn: torch.Tensor | None,
) -> None:
    _cuda(*cands, w, out_h, out_rn)
    c0 = cands[0]
    Cdim = c0.shape[-1]
    rows = c0.numel() // Cdim
    for c in cands:
        assert c.is_contiguous() and c.shape == c0.shape and c.dtype == c0.dtype
    arr = (C.c_void_p * len(cands))(*[c.data_ptr() for c in cands])
    check(lib.dgpt_depthmix(arr, len(cands), _ptr(w), _ptr(out_h), _ptr(out_rn), rows, Cdim, dtype_code(c0), _stream()))


def depthmix_cached(
    cands: list[torch.Tensor],
    cand_inv: list[torch.Tensor | None],
    w: torch.Tensor | None,
    out_h: torch.Tensor | None,
    out_rn: torch.Tensor | None,
    inv_out: torch.Tensor | None = None,
    inv_out_index: int = -1,
) -> None:
    """`depthmix` that reads the norm factors in `cand_inv` (fp32 [rows] each, None = compute) and writes the one it
    computes for candidate `inv_out_index` into `inv_out`."""
    _cuda(*cands, *[t for t in cand_inv if t is not None], w, out_h, out_rn, inv_out)
    c0 = cands[0]
    Cdim = c0.shape[-1]
    rows = c0.numel() // Cdim
    assert len(cand_inv) == len(cands)
    for c in cands:
        assert c.is_contiguous() and c.shape == c0.shape and c.dtype == c0.dtype
    for t in [*cand_inv, inv_out]:
        assert t is None or (t.dtype == torch.float32 and t.numel() == rows and t.is_contiguous())
    arr = (C.c_void_p * len(cands))(*[c.data_ptr() for c in cands])
    inv = (C.c_void_p * len(cands))(*[None if t is None else t.data_ptr() for t in cand_inv])
    check(
        lib.dgpt_depthmix_cached(
            arr, inv, len(cands), _ptr(w), _ptr(out_h), _ptr(out_rn), _ptr(inv_out), inv_out_index, rows, Cdim,
            dtype_code(c0), _stream(),
        )
    )


def rope_qknorm_kvappend(
    q: torch.Tensor,
    k: torch.Tensor,
    v: torch.Tensor,
    q_out: torch.Tensor,
    cs_table: torch.Tensor,
    kv: KvLayout,
    seq_pos0: torch.Tensor,
    seq_slot0: torch.Tensor,
    step: torch.Tensor | None,
    n_seq: int,
    T: int,
    H: int,
    D: int,
    status: torch.Tensor,
) -> None:
    """q, k, v: 2-D views [n_seq*T, H*D] sharing one row stride (slices of a fused projection)."""
    _cuda(q, k, v, q_out, cs_table, seq_pos0, seq_slot0, step, status)
    assert q.stride(0) == k.stride(0) == v.stride(0) and q.stride(1) == 1
    assert cs_table.is_contiguous() and cs_table.dtype == q.dtype
    assert seq_pos0.dtype == torch.int32 and seq_slot0.dtype == torch.int32
    check(
        lib.dgpt_rope_qknorm_kvappend(
            q.data_ptr(), k.data_ptr(), v.data_ptr(), q.stride(0), q_out.data_ptr(), q_out.stride(0),
            cs_table.data_ptr(), cs_table.shape[0], C.byref(kv), seq_pos0.data_ptr(), seq_slot0.data_ptr(),
            _ptr(step), n_seq, T, H, D, dtype_code(q), status.data_ptr(), _stream(),
        )
    )


def fmha_prefill(
    q: torch.Tensor,
    kv: KvLayout,
    o: torch.Tensor,
    *,
    B: int,
    H: int,
    Tq: int,
    D: int,
    q_batch_stride: int,
    q_row_stride: int,
    o_batch_stride: int,
    o_row_stride: int,
    kv_len: torch.Tensor | None = None,
    kv_len_all: int = -1,
    q_offset: int = 0,
    causal: bool = True,
    lse: torch.Tensor | None = None,
    impl: int = 0,
    status: torch.Tensor | None = None,
    max_ctas: int = 0,
) -> None:
    _cuda(q, o, kv_len, lse, status)
    o_f32 = int(o.dtype == torch.float32 and q.dtype != torch.float32)
    check(
        lib.dgpt_fmha_prefill(
            q.data_ptr(), q_batch_stride, q_row_stride, C.byref(kv), _ptr(kv_len), kv_len_all, o.data_ptr(),
            o_batch_stride, o_row_stride, o_f32, _ptr(lse), B, H, Tq, D, q_offset, int(causal), dtype_code(q),
            impl, max_ctas, _ptr(status), _stream(),
        )
    )


def decode_attn_workspace_bytes(R: int, H: int, D: int, n_splits: int) -> int:
    return int(lib.dgpt_decode_attn_workspace_bytes(R, H, D, n_splits))


def decode_attn(
    q: torch.Tensor,
    kv: KvLayout,
    len0: torch.Tensor,
    start1: torch.Tensor,
    len1: torch.Tensor,
    step: torch.Tensor | None,
    y: torch.Tensor,
    *,
    H: int,
    D: int,
    gate: torch.Tensor | None = None,
    prefix_o: torch.Tensor | None = None,
    prefix_lse: torch.Tensor | None = None,
    workspace: torch.Tensor | None = None,
    n_splits: int = 1,
) -> None:
    _cuda(q, len0, start1, len1, step, y, gate, prefix_o, prefix_lse, workspace)
    R = q.shape[0]
    ws_bytes = 0 if workspace is None else workspace.numel() * workspace.element_size()
    check(
        lib.dgpt_decode_attn(
            q.data_ptr(), q.stride(0), C.byref(kv), len0.data_ptr(), start1.data_ptr(), len1.data_ptr(), _ptr(step),
            _ptr(prefix_o), _ptr(prefix_lse), _ptr(gate), 0 if gate is None else gate.stride(0), y.data_ptr(),
            y.stride(0), _ptr(workspace), ws_bytes, n_splits, R, H, D, dtype_code(q), _stream(),
        )
    )


def decode_attn_partial(
    q: torch.Tensor,
    kv: KvLayout,
    len0: torch.Tensor | None,
    start1: torch.Tensor,
    len1: torch.Tensor,
    step: torch.Tensor | None,
    part_o: torch.Tensor,
    part_lse: torch.Tensor,
    *,
    H: int,
    D: int,
) -> None:
    """Per-row half of `decode_attn`: normalised fp32 result and log-sum-exp, to be merged by `attn_merge`."""
    _cuda(q, len0, start1, len1, step, part_o, part_lse)
    assert part_o.dtype == torch.float32 and part_lse.dtype == torch.float32
    assert part_o.is_contiguous() and part_lse.is_contiguous()
    check(
        lib.dgpt_decode_attn_partial(
            q.data_ptr(), q.stride(0), C.byref(kv), _ptr(len0), start1.data_ptr(), len1.data_ptr(), _ptr(step),
            part_o.data_ptr(), part_lse.data_ptr(), q.shape[0], H, D, dtype_code(q), _stream(),
        )
    )


def attn_merge(
    o_a: torch.Tensor,
    lse_a: torch.Tensor,
    o_b: torch.Tensor,
    lse_b: torch.Tensor,
    y: torch.Tensor,
    *,
    H: int,
    D: int,
    gate: torch.Tensor | None = None,
) -> None:
    """y = merge of two normalised attention partials, times sigmoid(gate)."""
    _cuda(o_a, lse_a, o_b, lse_b, y, gate)
    for t in (o_a, lse_a, o_b, lse_b):
        assert t.dtype == torch.float32 and t.is_contiguous()
    check(
        lib.dgpt_attn_merge(
            o_a.data_ptr(), lse_a.data_ptr(), o_b.data_ptr(), lse_b.data_ptr(), _ptr(gate),
            0 if gate is None else gate.stride(0), y.data_ptr(), y.stride(0), y.shape[0], H, D, dtype_code(y), _stream(),
        )
    )


def linear(
    a: torch.Tensor,
    w: torch.Tensor,
    out: torch.Tensor,
    *,
    swiglu: tuple[float, float] | None = None,
    add: torch.Tensor | None = None,
    status: torch.Tensor | None = None,
) -> None:
    """out = a @ w.T on the tcgen05 kernel (bf16).  swiglu=(alpha, limit): the SwiGLU of interleaved column pairs is
    applied in the epilogue and `out` has half as many columns as `w` has rows.  add=r: out = r + a @ w.T, rounded
    once (r may be `out`)."""
    _cuda(a, w, out, add, status)
    assert not (swiglu and add is not None)
    M, K = a.shape
    N = w.shape[0]
    assert w.shape[1] == K and a.stride(1) == 1 and w.stride(1) == 1 and out.stride(1) == 1
    assert out.shape == (M, N // 2 if swiglu else N) and a.dtype == w.dtype == out.dtype
    if add is not None:
        assert add.shape == out.shape and add.dtype == out.dtype and add.stride(1) == 1
    alpha, limit = swiglu if swiglu else (0.0, 0.0)
    check(
        lib.dgpt_linear(
            a.data_ptr(), a.stride(0), w.data_ptr(), w.stride(0), out.data_ptr(), out.stride(0), _ptr(add),
            0 if add is None else add.stride(0), M, N, K, 1 if swiglu else (2 if add is not None else 0), alpha, limit,
            dtype_code(a), _ptr(status), _stream(),
        )
    )


def integrate_tokens(
    tokens: torch.Tensor, n_chan: int, vocab_size: int, scale: torch.Tensor, order: torch.Tensor, state: torch.Tensor
) -> torch.Tensor:
    """(token - V/2) / scale followed by order[c] cumulative sums continued from `state`: int32 [N, H * F] -> f64 [N, H, F]."""
    _cuda(tokens, scale, order, state)
    assert tokens.dtype == torch.int32 and tokens.dim() == 2 and tokens.stride(1) == 1 and tokens.shape[1] % n_chan == 0
    assert scale.dtype == torch.float64 and state.dtype == torch.float64 and order.dtype == torch.int32
    assert scale.shape == (n_chan,) and order.shape == (n_chan,) and state.dim() == 2 and state.shape[0] == n_chan
    assert scale.is_contiguous() and order.is_contiguous() and state.is_contiguous()
    N, horizon = tokens.shape[0], tokens.shape[1] // n_chan
    out = torch.empty((N, horizon, n_chan), dtype=torch.float64, device=tokens.device)
    check(
        lib.dgpt_integrate_tokens(
            tokens.data_ptr(), tokens.stride(0), N, horizon, n_chan, vocab_size, scale.data_ptr(), order.data_ptr(),
            state.data_ptr(), state.shape[1], out.data_ptr(), _stream(),
        )
    )
    return out


def encode_series(
    values: torch.Tensor, vocab_size: int, scale: torch.Tensor, order: torch.Tensor, max_order: int, scalar_order: bool
) -> tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    """Tokenise many series at once: f64 [S, rows, F] -> (tokens int32 [S, rows - max_order, F],
    start f64 [S, max_order, F], end state of the decoder's running sums f64 [S, F, max(max_order, 1)])."""
    _cuda(values, scale, order)
    assert values.dtype == torch.float64 and values.dim() == 3
    S, rows, F = values.shape
    assert S == 0 or values[0].is_contiguous()
    assert scale.dtype == torch.float64 and order.dtype == torch.int32
    assert scale.shape == (F,) and order.shape == (F,) and scale.is_contiguous() and order.is_contiguous()
    assert 0 <= max_order <= rows
    dev = values.device
    tokens = torch.empty((S, rows - max_order, F), dtype=torch.int32, device=dev)
    start = torch.empty((S, max_order, F), dtype=torch.float64, device=dev)
    state = torch.empty((S, F, max(max_order, 1)), dtype=torch.float64, device=dev)
    if S == 0:
        return tokens, start, state
    check(
        lib.dgpt_encode_series(
            values.data_ptr(), values.stride(0) if S > 1 else rows * F, S, rows, F, vocab_size, order.data_ptr(),
            max_order, 1 if scalar_order else 0, scale.data_ptr(), tokens.data_ptr(), start.data_ptr(),
            state.data_ptr(), _stream(),
        )
    )
    return tokens, start, state


def token_nll(logits: torch.Tensor, targets: torch.Tensor, status: torch.Tensor | None = None) -> torch.Tensor:
    """-log softmax(logits)[r, targets[r]] per row as fp32 [R]; logits [R, V] (last dim contiguous), targets int32 [R]."""
    _cuda(logits, targets, status)
    assert logits.dim() == 2 and logits.stride(1) == 1 and targets.dtype == torch.int32 and targets.is_contiguous()
    R, V = logits.shape
    assert targets.numel() == R
    out = torch.empty(R, dtype=torch.float32, device=logits.device)
    check(
        lib.dgpt_token_nll(
            logits.data_ptr(), logits.stride(0), targets.data_ptr(), out.data_ptr(), R, V, dtype_code(logits),
            _ptr(status), _stream(),
        )
    )
    return out


def decode_attn_static_capacity_bytes() -> int:
    return int(lib.dgpt_decode_attn_static_capacity_bytes())


def decode_attn_static(
    q: torch.Tensor,
    kv: KvLayout,
    len0: torch.Tensor,
    start1: torch.Tensor,
    len1: torch.Tensor,
    step: torch.Tensor | None,
    y: torch.Tensor,
    *,
    H: int,
    D: int,
    gate: torch.Tensor | None = None,
    prefix_o: torch.Tensor | None = None,
    prefix_lse: torch.Tensor | None = None,
    n_splits: int = 1,
) -> None:
    """`decode_attn` with the split-K partials kept in the library's built-in 16 MiB array.

    For hosts that may not allocate device memory where they launch (memory handed out once at start-up,
    plugins that own only their inputs and outputs).  Raises `DgptError` when the partials would not fit.
    Calls share the array: do not let two of them overlap on the GPU.  Make the first call on a device
    outside stream capture.
    """
    _cuda(q, len0, start1, len1, step, y, gate, prefix_o, prefix_lse)
    check(
        lib.dgpt_decode_attn_static(
            q.data_ptr(), q.stride(0), C.byref(kv), len0.data_ptr(), start1.data_ptr(), len1.data_ptr(), _ptr(step),
            _ptr(prefix_o), _ptr(prefix_lse), _ptr(gate), 0 if gate is None else gate.stride(0), y.data_ptr(),
            y.stride(0), n_splits, q.shape[0], H, D, dtype_code(q), _stream(),
        )
    )


def swiglu(x: torch.Tensor, out: torch.Tensor, alpha: float, limit: float) -> None:
    _cuda(x, out)
    assert x.is_contiguous() and out.is_contiguous() and x.shape[-1] == 2 * out.shape[-1]
    rows = out.numel() // out.shape[-1]
    check(lib.dgpt_swiglu(x.data_ptr(), out.data_ptr(), rows, out.shape[-1], alpha, limit, dtype_code(x), _stream()))


def sigmoid_gate(y: torch.Tensor, gate: torch.Tensor) -> None:
    """y[r, :] *= sigmoid(gate[r, :]) in place; 2-D views with unit inner stride."""
    _cuda(y, gate)
    assert y.dim() == 2 and gate.shape == y.shape and y.stride(1) == 1 and gate.stride(1) == 1
    check(lib.dgpt_sigmoid_gate(y.data_ptr(), y.stride(0), gate.data_ptr(), gate.stride(0), y.shape[0], y.shape[1], dtype_code(y), _stream()))


def softcap_(logits: torch.Tensor, cap: float) -> None:
    _cuda(logits)
    assert logits.is_contiguous()
    check(lib.dgpt_softcap(logits.data_ptr(), logits.numel(), cap, dtype_code(logits), _stream()))


def step_advance(step: torch.Tensor, delta: int = 1) -> None:
    _cuda(step)
    check(lib.dgpt_step_advance(step.data_ptr(), delta, _stream()))


def sample(
    logits: torch.Tensor,
    out_tokens: torch.Tensor,
    *,
    R: int | None = None,
    row_stride: int | None = None,
    cap: float = 0.0,
    temperature: float = 1.0,
    top_p: float = 1.0,
    seed: int = 0,
    traj_id0: int = 0,
    traj_ids: torch.Tensor | None = None,
    step_base: int = 0,
    step: torch.Tensor | None = None,
    force_schedule: torch.Tensor | None = None,
    force_group_rows: int = 1,
    force_group_stride: int = 0,
    out_masks: torch.Tensor | None = None,
    history_tokens: torch.Tensor | None = None,
    history_masks: torch.Tensor | None = None,
) -> None:
    """One token per row.  `row_stride=0` with `R` rows samples R times from a single logits row."""
    _cuda(logits, out_tokens, traj_ids, step, force_schedule, out_masks, history_tokens, history_masks)
    V = logits.shape[-1]
    if R is None:
        R = logits.numel() // V
    if row_stride is None:
        row_stride = logits.stride(-2) if logits.dim() > 1 else V
    assert out_tokens.dtype == torch.int32 and out_tokens.numel() >= R
    hs = 0 if history_tokens is None else history_tokens.stride(0)
    if history_masks is not None and history_tokens is not None:
        assert history_masks.stride(0) == hs
    check(
        lib.dgpt_sample(
            logits.data_ptr(), row_stride, R, V, cap, temperature, top_p, seed & 0xFFFFFFFFFFFFFFFF, traj_id0,
            _ptr(traj_ids), step_base, _ptr(step), _ptr(force_schedule), force_group_rows, force_group_stride,
            out_tokens.data_ptr(), _ptr(out_masks),
            _ptr(history_tokens), _ptr(history_masks), hs, dtype_code(logits), _stream(),
        )
    )


def nucleus_filter(logits: torch.Tensor, top_p: float) -> torch.Tensor:
    _cuda(logits)
    x = logits.reshape(-1, logits.shape[-1])
    if x.stride(-1) != 1:
        x = x.contiguous()
    out = torch.empty(x.shape, dtype=x.dtype, device=x.device)
    check(lib.dgpt_nucleus_filter(x.data_ptr(), x.stride(0), out.data_ptr(), out.stride(0), x.shape[0], x.shape[1], top_p, dtype_code(x), _stream()))
    return out.view(logits.shape)


def attn_scale(D: int) -> float:
    return 1.0 / math.sqrt(D)


def lmhead_workspace_bytes(R: int) -> int:
    return int(lib.dgpt_lmhead_workspace_bytes(R))


def lmhead_sample(
    xn: torch.Tensor,
    emb: torch.Tensor,
    out_tokens: torch.Tensor,
    *,
    cap: float = 0.0,
    temperature: float = 1.0,
    top_p: float = 1.0,
    seed: int = 0,
    traj_id0: int = 0,
    traj_ids: torch.Tensor | None = None,
    step_base: int = 0,
    step: torch.Tensor | None = None,
    force_schedule: torch.Tensor | None = None,
    force_group_rows: int = 1,
    force_group_stride: int = 0,
    out_masks: torch.Tensor | None = None,
    history_tokens: torch.Tensor | None = None,
    history_masks: torch.Tensor | None = None,
    logits_out: torch.Tensor | None = None,
    workspace: torch.Tensor | None = None,
    status: torch.Tensor | None = None,
) -> None:
    """Head GEMM + soft-cap + draw in one call (`dgpt_lmhead_sample`).  With `logits_out`, or a top-p filter, the
    logits are written and sampled by the sampling kernel; otherwise they never leave the chip (needs `workspace`)."""
    _cuda(xn, emb, out_tokens, traj_ids, step, force_schedule, out_masks, history_tokens, history_masks, logits_out, workspace, status)
    R, Cdim = xn.shape
    V = emb.shape[0]
    assert emb.shape[1] == Cdim and xn.stride(1) == 1 and emb.stride(1) == 1
    assert out_tokens.dtype == torch.int32 and out_tokens.numel() >= R
    hs = 0 if history_tokens is None else history_tokens.stride(0)
    check(
        lib.dgpt_lmhead_sample(
            xn.data_ptr(), xn.stride(0), emb.data_ptr(), emb.stride(0), cap, temperature, top_p,
            seed & 0xFFFFFFFFFFFFFFFF, traj_id0, _ptr(traj_ids), step_base, _ptr(step), _ptr(force_schedule),
            force_group_rows, force_group_stride, out_tokens.data_ptr(), _ptr(out_masks), _ptr(history_tokens),
            _ptr(history_masks), hs, _ptr(logits_out), 0 if logits_out is None else logits_out.stride(0), _ptr(workspace),
            0 if workspace is None else workspace.numel() * workspace.element_size(), R, Cdim, V, dtype_code(xn),
            _ptr(status), _stream(),
        )
    )
