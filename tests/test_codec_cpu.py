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
