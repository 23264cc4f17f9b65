"""Derivative + sigma-delta tokeniser used on both sides of the decode path (float64).

Restates the reference codec's arithmetic (src/diff_gpt/encoder_decoder.py:36-427)
column by column so that tokens, `start` and `scale` are identical to the
reference's for float64 input; the arbitrary-precision `Decimal` mode of the
reference is not carried over (`use_decimal=True` raises).  It runs on the host:
it is O(rows x columns) once per call and is not part of the GPU hot path, but the
facade needs it to turn frames into prompts and trajectories back into values.

Conventions kept from the reference:
  * scalar order k: `start` has k rows, row i = first value of the i-th difference;
    per-column orders: `start` is the raw prefix `inp[:max_k]`.
  * a column is MASH-coded iff k >= 2 and vocab_size > 2**k + 2; its scale leaves
    2**k bins of headroom.  Otherwise the first-order carry scheme is used — except
    that with PER-COLUMN orders a k = 0 column is plainly rounded.
"""

from __future__ import annotations

import math

import numpy as np


def _scalar(order) -> bool:
    return isinstance(order, (int, np.integer))


def _orders(order, n_cols: int) -> np.ndarray:
    if _scalar(order):
        assert int(order) >= 0
        return np.full(n_cols, int(order), dtype=np.int64)
    arr = np.asarray(order, dtype=np.int64)
    assert arr.shape == (n_cols,) and (arr >= 0).all()
    return arr


def _no_decimal(use_decimal: bool) -> None:
    if use_decimal:
        raise NotImplementedError("the Decimal code path of the reference codec is not part of this build")


def _uses_mash(k: int, vocab_size: int) -> bool:
    return k >= 2 and vocab_size > 2**k + 2


def get_domain_of_definition(inp: np.ndarray, order_of_derivative, use_decimal: bool) -> np.ndarray:
    """max |k-th difference| per column (encoder_decoder.py:400-427)."""
    _no_decimal(use_decimal)
    assert inp.dtype == np.float64
    orders = _orders(order_of_derivative, inp.shape[1])
    out = np.zeros(inp.shape[1], dtype=np.float64)
    for c, k in enumerate(orders):
        d = np.diff(inp[:, c], n=int(k))
        if d.size:
            out[c] = np.max(np.abs(d))
    return out


def differentiate(inp: np.ndarray, order_of_derivative, use_decimal: bool = False):
    """(start, diff): k-th finite differences, all columns trimmed to rows - max_k (encoder_decoder.py:36-94)."""
    _no_decimal(use_decimal)
    assert inp.dtype == np.float64
    rows, n_cols = inp.shape
    orders = _orders(order_of_derivative, n_cols)
    max_k = int(orders.max()) if n_cols else 0
    assert max_k <= rows
    n = rows - max_k
    diff = np.zeros((n, n_cols), dtype=np.float64)
    for c, k in enumerate(orders):
        d = np.diff(inp[:, c], n=int(k)) if k else inp[:, c]
        diff[:, c] = d[len(d) - n :] if n > 0 else d[:0]
    if _scalar(order_of_derivative):
        k = int(order_of_derivative)
        start = np.zeros((k, n_cols), dtype=np.float64)
        level = inp
        for i in range(k):
            start[i] = level[0]
            level = np.diff(level, axis=0)
    else:
        start = inp[:max_k].copy()
    return start, diff


def integrate(start: np.ndarray, diff: np.ndarray, order_of_derivative, use_decimal: bool = False) -> np.ndarray:
    """Inverse of `differentiate` over the trailing axis pair (time, column).

    `diff` may carry leading batch axes: (..., N, F) -> (..., N + max_k, F); every
    trajectory is integrated with the same sequence of float64 additions the
    reference performs for a single one (encoder_decoder.py:97-152).
    """
    _no_decimal(use_decimal)
    n_cols = diff.shape[-1]
    lead = diff.shape[:-2]
    orders = _orders(order_of_derivative, n_cols)
    scalar = _scalar(order_of_derivative)
    max_k = start.shape[0]
    if scalar:
        assert int(order_of_derivative) == max_k
    else:
        assert (orders <= max_k).all()
    out = np.zeros((*lead, diff.shape[-2] + max_k, n_cols), dtype=np.float64)
    for c, k in enumerate(orders):
        k = int(k)
        if scalar:
            firsts = [start[i, c] for i in range(k)]
        else:
            firsts, level = [], start[max_k - k : max_k, c]
            for _ in range(k):
                firsts.append(level[0])
                level = np.diff(level)
        col = diff[..., c]
        for i in range(k):
            head = np.full((*lead, 1), firsts[k - 1 - i], dtype=np.float64)
            col = np.cumsum(np.concatenate([head, col], axis=-1), axis=-1)
        if max_k > k:
            head = np.broadcast_to(start[: max_k - k, c], (*lead, max_k - k))
            col = np.concatenate([head, col], axis=-1)
        out[..., c] = col
    return out


def integrate_end_state(start: np.ndarray, diff: np.ndarray, order_of_derivative) -> np.ndarray:
    """Running sums that `integrate` has reached after the last row of `diff` (N, F), per column and level:
    result[c, m] = last element of the (m + 1)-th cumulative sum of column c, zeros beyond the column's order.
    Continuing the sums from this state reproduces `integrate` over a longer sequence addition for addition."""
    n_cols = diff.shape[-1]
    orders = _orders(order_of_derivative, n_cols)
    scalar = _scalar(order_of_derivative)
    max_k = start.shape[0]
    state = np.zeros((n_cols, max(max_k, 1)), dtype=np.float64)
    for c, k in enumerate(orders):
        k = int(k)
        if scalar:
            firsts = [start[i, c] for i in range(k)]
        else:
            firsts, level = [], start[max_k - k : max_k, c]
            for _ in range(k):
                firsts.append(level[0])
                level = np.diff(level)
        col = diff[:, c]
        for i in range(k):
            col = np.cumsum(np.concatenate([np.array([firsts[k - 1 - i]], dtype=np.float64), col]))
            state[c, i] = col[-1]
    return state


def _carry_sigma_delta(x: np.ndarray, vocab_size: int) -> np.ndarray:
    """First-order scheme: integer part plus the increments of the rounded running fraction."""
    whole = np.trunc(x)
    carried = np.rint(np.cumsum(x - whole, axis=0))
    step = np.diff(np.concatenate([np.zeros((1, x.shape[1])), carried], axis=0), axis=0)
    tok = whole + vocab_size // 2 + step
    return np.clip(tok, 0, vocab_size - 1).astype(np.int64)


def _mash(x: np.ndarray, k: int, vocab_size: int) -> np.ndarray:
    """k cascaded first-order loops combined through (1 - z^-1)^i (encoder_decoder.py:155-226)."""
    rows, n_cols = x.shape
    stage_out = np.zeros((k, rows, n_cols), dtype=np.float64)
    err = np.zeros((k, n_cols), dtype=np.float64)
    for t in range(rows):
        feed = x[t]
        for i in range(k):
            eff = feed - err[i]
            q = np.rint(eff)
            stage_out[i, t] = q
            err[i] = q - eff
            feed = -err[i]
    total = np.zeros((rows, n_cols), dtype=np.float64)
    for i in range(k):
        for j in range(i + 1):
            coef = float((-1) ** j * math.comb(i, j))
            if j == 0:
                total = total + coef * stage_out[i]
            else:
                total[j:] = total[j:] + coef * stage_out[i, : rows - j]
    tok = np.rint(total).astype(np.int64) + vocab_size // 2
    return np.clip(tok, 0, vocab_size - 1)


def column_scales(vocab_size: int, domain_of_definition: np.ndarray, orders: np.ndarray) -> np.ndarray:
    """Tokens per unit of the k-th difference, per column: the largest difference lands one token inside the
    vocabulary's edge, less the 2^k headroom the cascaded quantiser needs (encoder_decoder.py:311-325)."""
    scale = np.ones(len(orders), dtype=np.float64)
    for c, k in enumerate(orders):
        if abs(domain_of_definition[c]) > np.finfo(np.float64).eps:
            room = vocab_size - 2 - (2 ** int(k) if _uses_mash(int(k), vocab_size) else 0)
            scale[c] = room / domain_of_definition[c] / 2
    return scale


def encode(inp: np.ndarray, vocab_size: int, domain_of_definition: np.ndarray, order_of_derivative, use_decimal: bool):
    """-> (start, scale, tokens[rows - max_k, F] int64) (encoder_decoder.py:278-370)."""
    _no_decimal(use_decimal)
    assert vocab_size % 2 == 0 and vocab_size >= 4
    assert inp.dtype == np.float64 and domain_of_definition.dtype == np.float64
    n_cols = inp.shape[1]
    assert domain_of_definition.shape[0] == n_cols
    orders = _orders(order_of_derivative, n_cols)
    scale = column_scales(vocab_size, domain_of_definition, orders)
    start, diff = differentiate(inp, order_of_derivative)
    scaled = diff * scale
    tokens = np.zeros(scaled.shape, dtype=np.int64)
    scalar = _scalar(order_of_derivative)
    for c, k in enumerate(orders):
        k = int(k)
        col = scaled[:, c : c + 1]
        if _uses_mash(k, vocab_size):
            tokens[:, c] = _mash(col, k, vocab_size)[:, 0]
        elif k == 0 and not scalar:
            tokens[:, c] = np.clip(np.rint(col).astype(np.int64) + vocab_size // 2, 0, vocab_size - 1)[:, 0]
        else:
            tokens[:, c] = _carry_sigma_delta(col, vocab_size)[:, 0]
    return start, scale, tokens


def decode(start: np.ndarray, scale: np.ndarray, inp: np.ndarray, vocab_size: int, order_of_derivative, use_decimal: bool):
    """tokens (..., N, F) int64 -> values (..., N + max_k, F) float64 (encoder_decoder.py:373-397)."""
    _no_decimal(use_decimal)
    assert vocab_size % 2 == 0 and vocab_size >= 4
    assert start.dtype == np.float64 and scale.dtype == np.float64 and inp.dtype == np.int64
    return integrate(start, (inp - vocab_size // 2) / scale, order_of_derivative)
