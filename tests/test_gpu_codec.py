"""dgpt_encode_series against the reference-made codec fixtures and the host codec, bit for bit."""

import numpy as np
import pytest
import torch

from conftest import load_golden

pytestmark = pytest.mark.gpu

CASES = ["k0", "k1", "k2", "k3", "k2_v6", "mixed"]


def _device_encode(x, V, dom, order):
    """x f64 [S, rows, F] -> numpy (tokens, start, state) through the C ABI."""
    from diff_gpt_b200 import ops
    from diff_gpt_b200.encoder_decoder import _orders, _scalar, column_scales

    orders = _orders(order, x.shape[2])
    scale = column_scales(V, dom, orders)
    tok, start, state = ops.encode_series(
        torch.from_numpy(x).cuda(), V, torch.from_numpy(scale).cuda(), torch.from_numpy(orders.astype(np.int32)).cuda(),
        int(orders.max()), _scalar(order),
    )
    torch.cuda.synchronize()
    return tok.cpu().numpy(), start.cpu().numpy(), state.cpu().numpy(), scale


@pytest.mark.parametrize("tag", CASES)
def test_reference_fixtures(tag):
    """Tokens, start rows and scales the reference produced for scalar orders 0..3, a vocabulary too small
    for the cascade, and per-column orders."""
    from diff_gpt_b200.encoder_decoder import integrate_end_state

    g = load_golden("codec")
    x, dom, V = g[f"{tag}:x"], g[f"{tag}:dom"], int(g[f"{tag}:V"])
    order = g[f"{tag}:order"]
    order = int(order) if order.ndim == 0 else order
    tok, start, state, scale = _device_encode(x[None], V, dom, order)
    assert np.array_equal(scale, np.broadcast_to(g[f"{tag}:scale"], scale.shape))
    assert np.array_equal(tok[0], g[f"{tag}:tok"])
    assert np.array_equal(start[0].view(np.int64), g[f"{tag}:start"].view(np.int64))
    want = integrate_end_state(g[f"{tag}:start"], (g[f"{tag}:tok"] - V // 2) / scale, order)
    assert np.array_equal(state[0].view(np.int64), want.view(np.int64))


@pytest.mark.parametrize(
    "order,V,F",
    [(0, 256, 3), (1, 1024, 4), (2, 1024, 2), (3, 4096, 3), (4, 64, 2), (2, 6, 2), (np.array([0, 3, 1, 2, 0, 1]), 512, 6)],
)
def test_many_series_equal_host_codec(order, V, F):
    """41 series in one launch against the host codec one series at a time; values large enough that tokens
    reach both ends of the vocabulary (the domain is taken from the first series only)."""
    from diff_gpt_b200.encoder_decoder import encode, get_domain_of_definition, integrate_end_state

    rng = np.random.default_rng(5 + V + F)
    S, rows = 41, 150
    x = np.cumsum(rng.normal(0, 1, (S, rows, F)), axis=1) * rng.uniform(0.2, 3.0, (S, 1, 1))
    dom = get_domain_of_definition(x[0], order, use_decimal=False)
    tok, start, state, scale = _device_encode(x, V, dom, order)
    seen = set()
    for s in range(S):
        h_start, h_scale, h_tok = encode(x[s], V, dom, order, use_decimal=False)
        assert np.array_equal(tok[s], h_tok), s
        assert np.array_equal(start[s].view(np.int64), np.asarray(h_start, dtype=np.float64).view(np.int64)), s
        want = integrate_end_state(h_start, (h_tok - V // 2) / h_scale, order)
        assert np.array_equal(state[s].view(np.int64), want.view(np.int64)), s
        seen.update((int(h_tok.min()), int(h_tok.max())))
    assert 0 in seen and V - 1 in seen  # the clip at both ends was exercised


def test_shortest_series_and_rejections():
    """rows == max order leaves no tokens; rows < max order and an odd vocabulary are refused."""
    from diff_gpt_b200 import ops
    from diff_gpt_b200._lib import DgptError

    x = torch.arange(6, dtype=torch.float64, device="cuda").reshape(1, 2, 3)
    scale = torch.ones(3, dtype=torch.float64, device="cuda")
    order = torch.full((3,), 2, dtype=torch.int32, device="cuda")
    tok, start, state = ops.encode_series(x, 64, scale, order, 2, True)
    assert tok.shape == (1, 0, 3)
    assert torch.equal(start[0, 0], x[0, 0]) and torch.equal(start[0, 1], x[0, 1] - x[0, 0])
    with pytest.raises((DgptError, AssertionError)):
        ops.encode_series(x, 64, scale, order, 3, True)
    with pytest.raises(DgptError):
        ops.encode_series(x, 63, scale, order, 2, True)


def test_predict_samples_many_matches_single_frames():
    """Two different frames decoded together under argmax give each frame's own predict_samples."""
    import pandas as pd

    from diff_gpt_b200.diff_gpt import DiffGPT
    from diff_gpt_b200.encoder_decoder import get_domain_of_definition
    from diff_gpt_b200.model.gpt import GPT
    from diff_gpt_b200.sampler.temperature import TemperatureSampler

    torch.manual_seed(3)
    m = GPT(vocab_size=64, n_embd=32, block_size=96, n_head=4, n_layer=2).cuda().eval()
    with torch.no_grad():
        for p in m.parameters():
            p.normal_(0, 0.3)
    rng = np.random.default_rng(8)
    x = np.cumsum(rng.normal(0, 1, (2, 20, 3)), axis=1)
    order = np.array([0, 1, 2])
    dom = get_domain_of_definition(x.reshape(-1, 3), order, use_decimal=False)
    dg = DiffGPT(model=m, order_of_derivative=order, domain_of_definition=dom, use_decimal=False)
    frames = [pd.DataFrame(x[s], columns=list("abc")) for s in range(2)]
    many = dg.predict_samples_many(frames, max_new_points=5, num_samples=3, sampler=TemperatureSampler(0.0))
    assert many.shape == (2, 3, 5, 3)
    for s in range(2):
        single = dg.predict_samples(frames[s], max_new_points=5, num_samples=3, sampler=TemperatureSampler(0.0))
        assert np.array_equal(many[s].view(np.int64), single.view(np.int64)), s
