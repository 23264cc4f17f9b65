"""Pins the CPU oracle against fixtures produced by the unmodified reference."""

import numpy as np
import pytest
import torch

from conftest import golden_weights, load_golden
from oracle import ref_decode, ref_math


def _shape(meta, **kw):
    V, C, H, L, block = (int(x) for x in meta[:5])
    return ref_math.Shape(vocab_size=V, n_embd=C, n_head=H, n_layer=L, block_size=block, **kw)


@pytest.mark.parametrize(
    "name,dtype,tol",
    [
        ("small_fp32", torch.float32, 2e-5),
        ("small_bf16_d64", torch.bfloat16, 2e-2),
        ("small_bf16_d32", torch.bfloat16, 2e-2),
    ],
)
def test_forward_full_serial_chunked(name, dtype, tol):
    g = load_golden(name)
    shape = _shape(g["meta"])
    w = golden_weights(g, dtype)
    idx = torch.from_numpy(g["idx"])
    B, T = idx.shape
    table = torch.from_numpy(g["freqs_cis"]).to(dtype)
    full = ref_math.forward(shape, w, idx, table=table).float().numpy()
    scale = np.abs(g["logits_full"]).max()
    assert np.abs(full - g["logits_full"]).max() <= tol * scale
    kv = ref_math.DenseKV(shape.n_layer, B, shape.n_head, T, shape.head_dim)
    serial = torch.cat(
        [ref_math.forward(shape, w, idx[:, t : t + 1], kv=kv, table=table) for t in range(T)], dim=1
    )
    assert np.abs(serial.float().numpy() - g["logits_serial"]).max() <= tol * scale
    cut = int(g["meta"][7])
    kv2 = ref_math.DenseKV(shape.n_layer, B, shape.n_head, T, shape.head_dim)
    a = ref_math.forward(shape, w, idx[:, :cut], kv=kv2, table=table)
    b = ref_math.forward(shape, w, idx[:, cut:], kv=kv2, table=table)
    chunked = torch.cat([a, b], dim=1).float().numpy()
    assert np.abs(chunked - g["logits_chunked"]).max() <= tol * scale
    # K is cached after RoPE + QK-norm, V raw
    kscale = np.abs(g["kv_cache"]).max()
    assert np.abs(kv2.data.float().numpy() - g["kv_cache"]).max() <= (1e-5 if dtype == torch.float32 else 2e-2) * kscale


def test_rope_table_matches_reference_buffer():
    g = load_golden("ops")
    t = ref_math.rope_table(16, 32).numpy()
    assert np.abs(t - g["table_16_32"]).max() < 1e-6


@pytest.mark.parametrize("tag,dtype,tol", [("f32", torch.float32, 1e-6), ("bf16", torch.bfloat16, 1e-2)])
def test_unit_ops(tag, dtype, tol):
    g = load_golden("ops")
    x = torch.from_numpy(g[f"rope_x_{tag}"]).to(dtype)
    cs = torch.from_numpy(g[f"rope_cs_{tag}"]).to(dtype)
    assert np.abs(ref_math.rope(x, cs).float().numpy() - g[f"rope_y_{tag}"]).max() <= tol * 8
    assert np.abs(ref_math.rms_norm(x).float().numpy() - g[f"rn_y_{tag}"]).max() <= tol * 8
    c = torch.from_numpy(g[f"mix_c_{tag}"]).to(dtype)
    w = torch.from_numpy(g[f"mix_w_{tag}"]).to(dtype)
    h = ref_math.depth_mix([c[i] for i in range(4)], w).float().numpy()
    assert np.abs(h - g[f"mix_h_{tag}"]).max() <= tol * 16
    u = torch.from_numpy(g[f"glu_u_{tag}"]).to(dtype)
    assert np.abs(ref_math.swiglu(u, 1.702, 7.0).float().numpy() - g[f"glu_y_{tag}"]).max() <= tol * 64


def test_nucleus_masks_exact():
    g = load_golden("samplers")
    logits = torch.from_numpy(g["logits"])
    for p in (0.3, 0.5, 0.9, 0.99):
        assert np.array_equal(ref_decode.nucleus_mask(logits, p).numpy(), g[f"mask_p{p}"])
    ka = torch.from_numpy(g["known_logits"])
    m = ref_decode.nucleus_mask(ka, 0.9).numpy()
    assert np.array_equal(m, g["known_mask_p0.9"])
    assert m.tolist() == [[True, True, True, False]]  # reference test_nucleus_sampler.py:55-87


def test_config1_argmax_stream_and_step_logits():
    g = load_golden("cfg1_fp32")
    shape = _shape(g["meta"])
    w = golden_weights(g, torch.float32)
    prompt = g["prompt"].tolist()
    toks, masks, logits = ref_decode.mc_decode(
        shape, w, prompt, num_samples=2, max_tokens=48, temperature=0.0, keep_logits=True
    )
    assert toks.shape == (2, 48) and masks.min() == 1
    ref_logits = g["step_logits"]
    got = logits[:, 0].numpy()
    # compare under the reference's own stream as long as streams agree; argmax streams must agree
    # wherever the reference's top-2 gap exceeds the fp32 tolerance
    assert np.array_equal(toks[0].numpy(), g["argmax_stream"])
    assert np.abs(got - ref_logits).max() <= 1e-4 * np.abs(ref_logits).max()


def test_engine_force_schedule():
    g = load_golden("engine_force")
    shape = _shape(g["meta"])
    w = golden_weights(g, torch.float32)
    sched = [None if s < 0 else int(s) for s in g["sched"]]
    prompt = g["prompt"].tolist()
    toks, masks, _ = ref_decode.mc_decode(
        shape, w, prompt, num_samples=3, max_tokens=10, temperature=0.0, force_schedule=sched
    )
    P = len(prompt)
    assert np.array_equal(toks.numpy(), g["results"][:, P:])
    assert np.array_equal(masks.numpy(), g["masks"][:, P:])


def test_anomaly_scores_restatement():
    """Token negative log-likelihoods of the oracle against DiffGPT.anomaly_scores of the reference."""
    from diff_gpt_b200.encoder_decoder import encode

    g = load_golden("anomaly")
    shape = _shape(g["meta"])
    w = golden_weights(g, torch.float32)
    for order, dom, key in ((g["order"], g["dom"], "scores_fp32"), (1, g["dom_k1"], "scores_fp32_k1")):
        _, _, tok = encode(inp=g["x"], vocab_size=shape.vocab_size, domain_of_definition=dom, order_of_derivative=order,
                           use_decimal=False)
        nll = ref_decode.token_nll(shape, w, torch.from_numpy(tok.reshape(-1).astype(np.int64))).numpy()
        want = g[key]
        k = int(np.max(order))
        flat = want[k:].reshape(-1)
        assert np.isnan(want[:k]).all() and np.isnan(flat[0]) and not np.isnan(flat[1:]).any()
        assert np.abs(nll - flat[1:]).max() <= 1e-4
