"""KV storage for the decode path.

`KVCache` keeps the reference's public surface (constructor, `insert_kv`,
`prefill`, `get_pos`, `reset`, attributes `kv_shape`, `kv_cache`, `pos`;
reference: src/diff_gpt/model/kv_cache.py:4-116) so code written against the
reference — including its Engine — keeps working; the CUDA kernels read and
write its dense (L, 2, B, H, T, D) tensor in place through `layer_layout`.

`PagedKVCache` is the layout the Monte-Carlo engine uses instead of replicating
the prompt (the reference's `prefill` broadcast, kv_cache.py:79): K/V live in
fixed-size pages, every trajectory of a series points at the SAME prompt pages,
and each trajectory owns a contiguous run of pages for the tokens it generates.
"""

from __future__ import annotations

import torch

from .. import ops


class KVCache:
    """Dense cache, one tensor (n_layer, 2, batch, n_head, seq_len, head_dim).

    `.pos` advances when the last layer has inserted (kv_cache.py:113-115).
    """

    __slots__ = ("kv_shape", "kv_cache", "pos")

    def __init__(self, batch_size: int, num_heads: int, seq_len: int, head_dim: int, num_layers: int) -> None:
        self.kv_shape = (num_layers, 2, batch_size, num_heads, seq_len, head_dim)
        self.kv_cache = torch.zeros(0)
        self.pos = 0

    # -- reference API ---------------------------------------------------------
    def reset(self) -> None:
        self.pos = 0

    def get_pos(self) -> int:
        return self.pos

    def prefill(self, other: "KVCache") -> None:
        """Take over `other`'s first `other.pos` tokens, broadcasting a batch of 1 to this batch."""
        assert self.kv_cache.size(0) == 0, "Cannot prefill a non-empty KV cache"
        assert other.kv_cache.size(0) != 0, "Cannot prefill with a None KV cache"
        mine, theirs = self.kv_shape, other.kv_shape
        names = ("Layer count", "K/V dimension", None, "Head count", None, "Head dim")
        for axis, label in enumerate(names):
            if label is not None:
                assert mine[axis] == theirs[axis], f"{label} mismatch: {mine[axis]} != {theirs[axis]}"
        assert mine[2] == theirs[2] or theirs[2] == 1, (
            f"Batch size mismatch: {mine[2]} vs {theirs[2]} (other must be 1 or equal)"
        )
        assert mine[4] >= theirs[4], f"Sequence length mismatch: {mine[4]} < {theirs[4]}"
        src = other.kv_cache
        self.kv_cache = torch.empty(self.kv_shape, dtype=src.dtype, device=src.device)
        n = other.pos
        self.kv_cache[:, :, :, :, :n].copy_(src[:, :, :, :, :n])
        self.pos = n

    def insert_kv(self, layer_idx: int, k: torch.Tensor, v: torch.Tensor) -> tuple[torch.Tensor, torch.Tensor]:
        """Write k, v (B, H, T_add, D) at the cursor; return views of everything cached so far."""
        t_add = k.size(2)
        t_end = self.pos + t_add
        self.ensure(t_end, k.dtype, k.device)
        store = self.kv_cache
        store[layer_idx, 0, :, :, self.pos : t_end].copy_(k)
        store[layer_idx, 1, :, :, self.pos : t_end].copy_(v)
        keys = store[layer_idx, 0, :, :, :t_end]
        values = store[layer_idx, 1, :, :, :t_end]
        if layer_idx == store.size(0) - 1:
            self.pos = t_end
        return keys, values

    # -- what the kernels need ---------------------------------------------------
    def ensure(self, t_end: int, dtype: torch.dtype, device: torch.device) -> None:
        """Allocate lazily; grow to (t_end + 1024) rounded up to 1024 when full (kv_cache.py:87-106)."""
        if self.kv_cache.size(0) == 0:
            self.kv_cache = torch.empty(self.kv_shape, dtype=dtype, device=device)
        have = self.kv_cache.size(4)
        if t_end > have:
            want = (t_end + 1024 + 1023) & ~1023
            grown = torch.empty(
                (*self.kv_cache.shape[:4], want, self.kv_cache.shape[5]), dtype=dtype, device=device
            )
            grown[:, :, :, :, :have].copy_(self.kv_cache)
            self.kv_cache = grown
            self.kv_shape = self.kv_cache.shape

    def layer_layout(self, layer: int) -> ops.KvLayout:
        _, _, _, H, T, D = self.kv_cache.shape
        c = self.kv_cache
        return ops.kv_layout(c[layer, 0], c[layer, 1], page_stride=H * T * D, head_stride=T * D, page_tokens=T)


class PagedKVCache:
    """Paged K/V with one shared prompt per series and private pages per trajectory.

    pool            (n_layer, n_pages, 2, n_head, page_tokens, head_dim)
    prefix_table    (n_series, prefix_pages)            int32  -> prompt pages of a series
    row_table       (n_rows, prefix_pages + own_pages)  int32  -> same prompt pages, then the row's own run
    Rows are series-major: row = series * rows_per_series + trajectory.
    A row's generated token g sits at logical slot prefix_pages * page_tokens + g.
    """

    def __init__(
        self,
        n_layer: int,
        n_head: int,
        head_dim: int,
        n_series: int,
        rows_per_series: int,
        prefix_len: int,
        max_new: int,
        dtype: torch.dtype,
        device: torch.device | str,
        page_tokens: int = 64,
        pool: torch.Tensor | None = None,
    ) -> None:
        pt = page_tokens
        self.page_tokens = pt
        self.n_layer, self.n_head, self.head_dim = n_layer, n_head, head_dim
        self.n_series, self.rows_per_series = n_series, rows_per_series
        self.n_rows = n_series * rows_per_series
        self.prefix_len = prefix_len
        self.prefix_pages = max(1, -(-prefix_len // pt))
        self.own_pages = max(1, -(-max_new // pt))
        self.max_new = max_new
        n_pages = n_series * self.prefix_pages + self.n_rows * self.own_pages
        shape = (n_layer, n_pages, 2, n_head, pt, head_dim)
        if pool is not None:  # storage handed in by the caller (e.g. kept across calls); contents need not be cleared
            assert tuple(pool.shape) == shape and pool.dtype == dtype and pool.is_contiguous(), "pool does not fit this cache"
            self.pool = pool
        else:
            self.pool = torch.empty(shape, dtype=dtype, device=device)
        pre = torch.arange(n_series * self.prefix_pages, dtype=torch.int32).view(n_series, self.prefix_pages)
        own = n_series * self.prefix_pages + torch.arange(self.n_rows * self.own_pages, dtype=torch.int32).view(
            self.n_rows, self.own_pages
        )
        row = torch.cat([pre.repeat_interleave(rows_per_series, dim=0), own], dim=1)
        self.prefix_table = pre.contiguous().to(device)
        self.row_table = row.contiguous().to(device)
        self.suffix_slot0 = self.prefix_pages * pt

    @property
    def bytes(self) -> int:
        return self.pool.numel() * self.pool.element_size()

    def _layout(self, layer: int, table: torch.Tensor) -> ops.KvLayout:
        H, pt, D = self.n_head, self.page_tokens, self.head_dim
        p = self.pool[layer]
        return ops.kv_layout(
            p[0, 0], p[0, 1], page_stride=2 * H * pt * D, head_stride=pt * D, page_tokens=pt, page_table=table,
            n_pages=p.shape[0],
        )

    def prefix_layout(self, layer: int) -> ops.KvLayout:
        """Sequence index = series (prompt prefill and the shared-prefix attention phase)."""
        return self._layout(layer, self.prefix_table)

    def row_layout(self, layer: int) -> ops.KvLayout:
        """Sequence index = row (append and per-trajectory attention)."""
        return self._layout(layer, self.row_table)
