"""The host tokeniser reproduces the reference codec bit for bit (float64) on reference-made fixtures."""

import numpy as np
import pytest

from conftest import load_golden
from diff_gpt_b200.encoder_decoder import decode, encode, get_domain_of_definition

CASES = ["k0", "k1", "k2", "k3", "k2_v6", "mixed"]


@pytest.mark.parametrize("tag", CASES)
def test_encode_decode_identical_to_reference(tag):
    g = load_golden("codec")
    x, V = g[f"{tag}:x"], int(g[f"{tag}:V"])
    order = g[f"{tag}:order"]
    order = int(order) if order.ndim == 0 else order
    dom = get_domain_of_definition(x, order, use_decimal=False)
    assert np.array_equal(dom, g[f"{tag}:dom"])
    start, scale, tok = encode(inp=x, vocab_size=V, domain_of_definition=dom, order_of_derivative=order, use_decimal=False)
    assert np.array_equal(start, g[f"{tag}:start"]) and np.array_equal(scale, g[f"{tag}:scale"])
    assert tok.dtype == np.int64 and np.array_equal(tok, g[f"{tag}:tok"])
    dec = decode(start=start, scale=scale, inp=tok, vocab_size=V, order_of_derivative=order, use_decimal=False)
    assert np.array_equal(dec, g[f"{tag}:dec"])
    # a batch of trajectories decodes exactly like each one alone
    batch = np.stack([tok, np.clip(tok + 1, 0, V - 1), tok[::-1].copy()])
    many = decode(start=start, scale=scale, inp=batch, vocab_size=V, order_of_derivative=order, use_decimal=False)
    for i in range(3):
        one = decode(start=start, scale=scale, inp=batch[i], vocab_size=V, order_of_derivative=order, use_decimal=False)
        assert np.array_equal(many[i], one)


def test_round_trip_error_bound_order1():
    """|decoded - x| stays within one quantisation bin (cf. reference test_encoder_decoder.py:11-45)."""
    rng = np.random.default_rng(0)
    x = np.cumsum(rng.normal(0, 1, (200, 2)), axis=0)
    dom = get_domain_of_definition(x, 1, use_decimal=False)
    start, scale, tok = encode(inp=x, vocab_size=256, domain_of_definition=dom, order_of_derivative=1, use_decimal=False)
    dec = decode(start=start, scale=scale, inp=tok, vocab_size=256, order_of_derivative=1, use_decimal=False)
    assert np.abs(dec - x).max() <= (1.0 / scale).max()


def test_decimal_mode_is_refused():
    x = np.zeros((4, 1))
    with pytest.raises(NotImplementedError):
        get_domain_of_definition(x, 1, use_decimal=True)


def test_cumulative_sums_can_be_continued_from_their_end_state():
    """integrate_end_state + one addition per level and step reproduces integrate over the longer sequence
    bit for bit (what the device-side decode of the generated horizon relies on)."""
    from diff_gpt_b200.encoder_decoder import _orders, integrate, integrate_end_state

    rng = np.random.default_rng(0)
    for order in (0, 1, 2, 3, np.array([0, 1, 2, 2, 1])):
        F, Tp, H = 5, 17, 9
        max_k = int(np.max(order))
        start = rng.normal(size=(max_k, F))
        head, tail = rng.normal(size=(Tp, F)), rng.normal(size=(H, F))
        whole = integrate(start, np.concatenate([head, tail], 0), order)
        state = integrate_end_state(start, head, order)
        got = np.zeros((H, F))
        for c, k in enumerate(_orders(order, F)):
            x = state[c].copy()
            for t in range(H):
                v = tail[t, c]
                for m in range(int(k)):
                    x[m] = x[m] + v
                    v = x[m]
                got[t, c] = v
        assert np.array_equal(got, whole[max_k + Tp :])


def test_quantile_of_sorted_equals_numpy_linear_quantile():
    import torch

    from diff_gpt_b200.diff_gpt import _quantile_of_sorted

    rng = np.random.default_rng(1)
    for n in (1, 2, 7, 100, 4096):
        x = rng.normal(size=(n, 6, 3)) * 1e3
        ordered = torch.sort(torch.from_numpy(x), dim=0).values
        for q in (0.1, 0.25, 0.5, 0.9, 0.999):
            assert np.array_equal(_quantile_of_sorted(ordered, q).numpy(), np.quantile(x, q, axis=0)), (n, q)
