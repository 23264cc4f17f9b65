"""Generate the golden fixtures in this directory by RUNNING THE UNMODIFIED REFERENCE.

Usage (in a container that has the reference checked out):

    python tests/golden/make_golden.py /path/to/reference

The reference's `src/` is put on `sys.path`, its own `GPT`, `KVCache`,
`Engine`, samplers and `DiffGPT` are run on CPU with fixed seeds and the
inputs, weights and outputs are written as `.npz` files next to this script.
bf16 tensors are stored as float32 (exactly representable).  The fixtures are
small (a few hundred KB each) so they can be committed; the test-suite never
needs the reference itself.
"""

from __future__ import annotations

import os
import sys

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))


def _np(t: torch.Tensor) -> np.ndarray:
    return t.detach().float().numpy() if t.is_floating_point() else t.detach().numpy()


def _weights(model) -> dict[str, np.ndarray]:
    return {"w:" + k: _np(v) for k, v in model.state_dict().items() if k != "lm_head.weight"}


def _init(model, seed: int, std: float) -> None:
    torch.manual_seed(seed)
    with torch.no_grad():
        for p in model.parameters():
            p.normal_(0.0, std)


def small_forward(GPT, KVCache, name, dtype, V, C, H, L, block, std, seed, B, T):
    m = GPT(vocab_size=V, n_embd=C, block_size=block, n_head=H, n_layer=L).eval()
    _init(m, seed, std)
    m = m.to(dtype)
    g = torch.Generator().manual_seed(seed + 100)
    idx = torch.randint(0, V, (B, T), generator=g)
    with torch.inference_mode():
        full, _ = m(idx)
        kv = KVCache(batch_size=B, num_heads=H, seq_len=T, head_dim=C // H, num_layers=L)
        serial = torch.cat([m(idx[:, t : t + 1], kv_cache=kv)[0] for t in range(T)], dim=1)
        kv2 = KVCache(batch_size=B, num_heads=H, seq_len=T, head_dim=C // H, num_layers=L)
        cut = T // 2 + 1
        a, _ = m(idx[:, :cut], kv_cache=kv2)
        b, _ = m(idx[:, cut:], kv_cache=kv2)
        chunked = torch.cat([a, b], dim=1)
        kcache = kv2.kv_cache.clone()
    np.savez_compressed(
        os.path.join(HERE, name + ".npz"),
        meta=np.array([V, C, H, L, block, B, T, cut], dtype=np.int64),
        idx=_np(idx),
        logits_full=_np(full),
        logits_serial=_np(serial),
        logits_chunked=_np(chunked),
        kv_cache=_np(kcache),
        freqs_cis=_np(m.freqs_cis),
        **_weights(m),
    )
    print(name, "max|full-serial|", (full.float() - serial.float()).abs().max().item())


class _Capture:
    """Sampler that records the logits it is handed and answers with argmax."""

    def __init__(self):
        self.seen = []

    def __call__(self, logits, rng=None):
        self.seen.append(logits.detach().float().clone())
        return torch.argmax(logits, dim=-1, keepdim=True)


def config1(ref):
    """BASELINE config 1: V256 C64 H4 L2 block 138, fp32, weights N(0,0.02) seed 0, walk seed 1."""
    from diff_gpt.diff_gpt import DiffGPT
    from diff_gpt.encoder_decoder import encode, get_domain_of_definition
    from diff_gpt.model.engine import Engine
    from diff_gpt.model.gpt import GPT
    from diff_gpt.sampler.temperature import TemperatureSampler
    import pandas as pd

    V, C, H, L, block = 256, 64, 4, 2, 138
    m = GPT(vocab_size=V, n_embd=C, block_size=block, n_head=H, n_layer=L).eval()
    _init(m, 0, 0.02)
    walk = np.cumsum(np.random.default_rng(1).normal(0.0, 1.0, 96))
    ctx = walk[-90:].reshape(-1, 1)
    domain = get_domain_of_definition(walk.reshape(-1, 1), 1, use_decimal=False)
    start, scale, toks = encode(
        inp=ctx, vocab_size=V, domain_of_definition=domain, order_of_derivative=1, use_decimal=False
    )
    prompt = toks.reshape(-1).astype(np.int64).tolist()
    cap = _Capture()
    res, masks = Engine(m).generate_batch(prompt, num_samples=3, max_tokens=48, sampler=cap)
    stream = np.asarray(res[0][len(prompt) :], dtype=np.int64)
    step_logits = torch.stack([s[0] for s in cap.seen]).numpy()  # (48, V)
    dg = DiffGPT(model=m, order_of_derivative=1, domain_of_definition=domain, use_decimal=False)
    df = pd.DataFrame(ctx, columns=["y"])
    fut0 = dg.predict_samples(df, max_new_points=48, num_samples=4, sampler=TemperatureSampler(0.0))
    pred = dg.predict(df, max_new_points=48, sampler=TemperatureSampler(0.0)).to_numpy()
    q = dg.predict_quantiles(df, 48, quantiles=(0.1, 0.5, 0.9), num_samples=4, sampler=TemperatureSampler(0.0))
    np.savez_compressed(
        os.path.join(HERE, "cfg1_fp32.npz"),
        meta=np.array([V, C, H, L, block], dtype=np.int64),
        walk=walk,
        ctx=ctx,
        domain=np.asarray(domain, dtype=np.float64),
        start=np.asarray(start, dtype=np.float64),
        scale=np.asarray(scale, dtype=np.float64),
        prompt=np.asarray(prompt, dtype=np.int64),
        argmax_stream=stream,
        step_logits=step_logits,
        futures_t0=fut0,
        predict_t0=pred,
        q50_t0=q[0.5].to_numpy(),
        **_weights(m),
    )
    print("cfg1 prompt", len(prompt), "stream head", stream[:8])


def samplers(ref):
    from diff_gpt.sampler.nucleus import NucleusSampler

    g = torch.Generator().manual_seed(7)
    logits = torch.randn(16, 96, generator=g) * 2.0
    out = {"logits": _np(logits)}
    for p in (0.3, 0.5, 0.9, 0.99):
        cap = _Capture()
        NucleusSampler(p=p, sampler=cap)(logits)
        out[f"mask_p{p}"] = torch.isfinite(cap.seen[0]).numpy()
    ka = torch.log(torch.tensor([[0.6, 0.25, 0.1, 0.05]]))
    cap = _Capture()
    NucleusSampler(p=0.9, sampler=cap)(ka)
    out["known_logits"] = _np(ka)
    out["known_mask_p0.9"] = torch.isfinite(cap.seen[0]).numpy()
    np.savez_compressed(os.path.join(HERE, "samplers.npz"), **out)


def ops(ref):
    from diff_gpt.model.block import block_attn_res
    from diff_gpt.model.rms_norm import rms_norm
    from diff_gpt.model.rope import apply_rotary_emb, precompute_freqs_cis
    from diff_gpt.model.swi_glu import SwiGLU

    g = torch.Generator().manual_seed(11)
    out = {}
    for tag, dt in (("f32", torch.float32), ("bf16", torch.bfloat16)):
        x = (torch.randn(3, 5, 4, 16, generator=g) * 1.7).to(dt)
        cs = precompute_freqs_cis(16, 32, 10000.0).to(dt)[7:12].view(1, 5, 1, 8, 2)
        out[f"rope_x_{tag}"] = _np(x)
        out[f"rope_cs_{tag}"] = _np(cs.view(5, 8, 2))
        out[f"rope_y_{tag}"] = _np(apply_rotary_emb(x, cs))
        out[f"rn_y_{tag}"] = _np(rms_norm(x))
        cands = [(torch.randn(2, 3, 48, generator=g) * (0.5 + i)).to(dt) for i in range(4)]
        proj = torch.nn.Linear(48, 1, bias=False)
        with torch.no_grad():
            proj.weight.copy_(torch.randn(1, 48, generator=g) * 0.3)
        proj = proj.to(dt)
        with torch.no_grad():
            h = block_attn_res(tuple(cands[:3]), cands[3], proj)
        out[f"mix_c_{tag}"] = np.stack([_np(c) for c in cands])
        out[f"mix_w_{tag}"] = _np(proj.weight)
        out[f"mix_h_{tag}"] = _np(h)
        u = (torch.randn(4, 64, generator=g) * 5.0).to(dt)
        out[f"glu_u_{tag}"] = _np(u)
        out[f"glu_y_{tag}"] = _np(SwiGLU(alpha=1.702, limit=7.0)(u))
    out["table_16_32"] = _np(precompute_freqs_cis(16, 32, 10000.0))
    np.savez_compressed(os.path.join(HERE, "ops.npz"), **out)


def engine_force(ref):
    """Engine with a force schedule on a tiny fp32 model, argmax elsewhere."""
    from diff_gpt.model.engine import Engine
    from diff_gpt.model.gpt import GPT
    from diff_gpt.sampler.temperature import TemperatureSampler

    V, C, H, L, block = 64, 32, 4, 2, 24
    m = GPT(vocab_size=V, n_embd=C, block_size=block, n_head=H, n_layer=L).eval()
    _init(m, 5, 0.3)
    prompt = [3, 17, 42, 8, 8, 61, 0]
    sched = [None, 5, None, None, 9, 9, None, 1, None, None]
    res, masks = Engine(m).generate_batch(
        prompt, num_samples=3, max_tokens=10, sampler=TemperatureSampler(0.0), force_schedule=sched
    )
    np.savez_compressed(
        os.path.join(HERE, "engine_force.npz"),
        meta=np.array([V, C, H, L, block], dtype=np.int64),
        prompt=np.asarray(prompt, dtype=np.int64),
        sched=np.asarray([-1 if s is None else s for s in sched], dtype=np.int64),
        results=np.asarray(res, dtype=np.int64),
        masks=np.asarray(masks, dtype=np.int64),
        **_weights(m),
    )


def _series(rng, rows, cols):
    t = np.arange(rows)[:, None]
    periods = rng.integers(12, 169, size=(3, cols))
    amps = rng.uniform(0.5, 2.0, size=(3, cols))
    x = sum(amps[i] * np.sin(2 * np.pi * t / periods[i]) for i in range(3))
    noise = np.zeros((rows, cols))
    e = rng.normal(0, 0.1, size=(rows, cols))
    for i in range(1, rows):
        noise[i] = 0.8 * noise[i - 1] + e[i]
    return (x + noise).astype(np.float64)


def codec(ref):
    """Tokeniser round trips: scalar orders 0..3, per-column orders, a vocabulary too small for MASH."""
    from diff_gpt.encoder_decoder import decode, encode, get_domain_of_definition

    rng = np.random.default_rng(21)
    out = {}
    cases = [("k0", 0, 256, 3), ("k1", 1, 256, 3), ("k2", 2, 256, 3), ("k3", 3, 256, 2), ("k2_v6", 2, 6, 2),
             ("mixed", np.array([0, 1, 1, 2, 2, 1, 0]), 1024, 7)]
    for tag, order, V, cols in cases:
        x = _series(rng, 60, cols) if tag == "mixed" else np.cumsum(rng.normal(0, 1, (40, cols)), axis=0)
        dom = get_domain_of_definition(x, order, use_decimal=False)
        start, scale, tok = encode(inp=x, vocab_size=V, domain_of_definition=dom, order_of_derivative=order, use_decimal=False)
        dec = decode(start=start, scale=scale, inp=tok, vocab_size=V, order_of_derivative=order, use_decimal=False)
        out[f"{tag}:x"], out[f"{tag}:dom"], out[f"{tag}:start"] = x, np.asarray(dom, dtype=np.float64), np.asarray(start, dtype=np.float64)
        out[f"{tag}:scale"], out[f"{tag}:tok"], out[f"{tag}:dec"] = np.asarray(scale, dtype=np.float64), tok, np.asarray(dec, dtype=np.float64)
        out[f"{tag}:order"] = np.asarray(order, dtype=np.int64)
        out[f"{tag}:V"] = np.asarray(V, dtype=np.int64)
    np.savez_compressed(os.path.join(HERE, "codec.npz"), **out)


def teacher_forced(ref):
    """DiffGPT.predict with future covariates (3 channels, orders [0,1,2], channel 0 is the target) and
    predict_samples / predict on the same tiny fp32 model, all under argmax."""
    from diff_gpt.diff_gpt import DiffGPT
    from diff_gpt.encoder_decoder import get_domain_of_definition
    from diff_gpt.model.gpt import GPT
    from diff_gpt.sampler.temperature import TemperatureSampler
    import pandas as pd

    V, C, H, L, block = 64, 32, 4, 2, 96
    m = GPT(vocab_size=V, n_embd=C, block_size=block, n_head=H, n_layer=L).eval()
    _init(m, 9, 0.3)
    rng = np.random.default_rng(33)
    x = _series(rng, 26, 3)
    order = np.array([0, 1, 2])
    dom = get_domain_of_definition(x, order, use_decimal=False)
    dg = DiffGPT(model=m, order_of_derivative=order, domain_of_definition=dom, use_decimal=False)
    ctx = pd.DataFrame(x[:20], columns=["a", "b", "c"])
    fut = pd.DataFrame(x[20:], columns=["a", "b", "c"])
    tf = dg.predict(ctx, future_covariates_df=fut, target_columns=["a"], sampler=TemperatureSampler(0.0))
    ar = dg.predict(ctx, max_new_points=6, sampler=TemperatureSampler(0.0))
    ps = dg.predict_samples(ctx, max_new_points=6, num_samples=3, sampler=TemperatureSampler(0.0))
    np.savez_compressed(
        os.path.join(HERE, "teacher_forced.npz"),
        meta=np.array([V, C, H, L, block], dtype=np.int64),
        x=x, order=order, dom=np.asarray(dom, dtype=np.float64),
        teacher_forced=tf.to_numpy(), autoregressive=ar.to_numpy(), samples=ps,
        **_weights(m),
    )


def anomaly(ref):
    """DiffGPT.anomaly_scores on a three-channel signal (orders [0, 1, 2]) with a tiny fp32 model, per-column and scalar order."""
    from diff_gpt.diff_gpt import DiffGPT
    from diff_gpt.encoder_decoder import get_domain_of_definition
    from diff_gpt.model.gpt import GPT
    import pandas as pd

    V, C, H, L, block = 64, 32, 4, 2, 96
    m = GPT(vocab_size=V, n_embd=C, block_size=block, n_head=H, n_layer=L).eval()
    _init(m, 12, 0.3)
    rng = np.random.default_rng(34)
    x = _series(rng, 30, 3)
    order = np.array([0, 1, 2])
    dom = get_domain_of_definition(x, order, use_decimal=False)
    df = pd.DataFrame(x, columns=["a", "b", "c"])
    weights = _weights(m)
    dg = DiffGPT(model=m, order_of_derivative=order, domain_of_definition=dom, use_decimal=False)
    s32 = dg.anomaly_scores(df).to_numpy()
    dg1 = DiffGPT(model=m, order_of_derivative=1, domain_of_definition=get_domain_of_definition(x, 1, use_decimal=False), use_decimal=False)
    s32_k1 = dg1.anomaly_scores(df).to_numpy()
    dom1 = np.asarray(dg1.domain_of_definition, dtype=np.float64)
    # (a bf16 module cannot be scored by the reference: its .numpy() call rejects bfloat16)
    np.savez_compressed(
        os.path.join(HERE, "anomaly.npz"),
        meta=np.array([V, C, H, L, block], dtype=np.int64),
        x=x, order=order, dom=np.asarray(dom, dtype=np.float64), dom_k1=dom1,
        scores_fp32=s32, scores_fp32_k1=s32_k1,
        **weights,
    )


def _seeded_state_dict(V, C, L, seed, std, dtype):
    """The weights `oracle.ref_math.random_weights` draws: one torch.Generator(seed), tensors in a fixed order.
    A test regenerates them from the seed, so a fixture made from these needs to store no weights."""
    g = torch.Generator().manual_seed(seed)

    def n(*s):
        return (torch.randn(*s, generator=g) * std).to(dtype)

    w = {"token_embedding_table.weight": n(V, C)}
    for i in range(L):
        p = f"blocks.{i}."
        for name in ("c_q", "c_k", "c_v", "c_g", "c_proj"):
            w[p + f"sa.{name}.weight"] = n(C, C)
        w[p + "ffwd.net.0.weight"] = n(4 * C, C)
        w[p + "ffwd.net.2.weight"] = n(C, 2 * C)
        w[p + "attn_res_proj.weight"] = n(1, C)
        w[p + "mlp_res_proj.weight"] = n(1, C)
    w["lm_head.weight"] = w["token_embedding_table.weight"]
    return w


def _forced_logits(m, prompt, G):
    """Per-step logits of the reference Engine under its own argmax stream (one trajectory)."""
    from diff_gpt.model.engine import Engine

    cap = _Capture()
    res, _ = Engine(m).generate_batch(prompt, num_samples=1, max_tokens=G, sampler=cap)
    stream = np.asarray(res[0][len(prompt) :], dtype=np.int64)
    return stream, torch.stack([s[0] for s in cap.seen]).numpy()


def cfg4_bf16_init002(ref):
    """BASELINE config 4 at full architecture (V4096 C768 H12 L12 block 2048), weights N(0, 0.02) seed 4 rounded to
    bf16, a 300-token seeded prompt, 6 argmax steps: per-step logits of the reference in bf16 and, on the same
    (bf16-valued) weights, in fp32.  Weights are not stored: they are regenerated from the seed."""
    from diff_gpt.model.gpt import GPT

    V, C, H, L, block = 4096, 768, 12, 12, 2048
    sd = _seeded_state_dict(V, C, L, 4, 0.02, torch.bfloat16)
    prompt = torch.randint(0, V, (300,), generator=torch.Generator().manual_seed(44)).tolist()
    G = 6
    out = {}
    m = GPT(vocab_size=V, n_embd=C, block_size=block, n_head=H, n_layer=L).eval()
    m.load_state_dict({k: v.float() for k, v in sd.items()})
    out["stream"], out["logits_bf16"] = _forced_logits(m.to(torch.bfloat16), prompt, G)
    # fp32 on the same (bf16-valued) weights and the same token stream: one causal forward over prompt + stream
    m32 = GPT(vocab_size=V, n_embd=C, block_size=block, n_head=H, n_layer=L).eval()
    m32.load_state_dict({k: v.float() for k, v in sd.items()})
    ids = torch.tensor([prompt + out["stream"].tolist()[:-1]])
    with torch.inference_mode():
        full, _ = m32(ids)
    out["logits_fp32"] = _np(full[0, len(prompt) - 1 :])
    np.savez_compressed(
        os.path.join(HERE, "cfg4_bf16_init002.npz"),
        meta=np.array([V, C, H, L, block, 4, G], dtype=np.int64),
        prompt=np.asarray(prompt, dtype=np.int64), stream=out["stream"],
        logits_bf16=out["logits_bf16"], logits_fp32=out["logits_fp32"],
    )
    d = np.abs(out["logits_bf16"] - out["logits_fp32"]).max() / np.abs(out["logits_fp32"]).max()
    print("cfg4_bf16_init002: reference bf16 vs fp32 rel err", d, "max|logit|", np.abs(out["logits_fp32"]).max())


def bf16_wide_init(ref):
    """A small bf16 model with N(0, 0.15) weights: the reference's logits in bf16 and in fp32 on the same weights.
    On such weights the reference's own bf16 arithmetic strays furthest from exact arithmetic."""
    from diff_gpt.model.gpt import GPT

    V, C, H, L, block, B, T = 128, 128, 2, 2, 32, 2, 13
    sd = _seeded_state_dict(V, C, L, 6, 0.15, torch.bfloat16)
    idx = torch.randint(0, V, (B, T), generator=torch.Generator().manual_seed(106))
    out = {}
    for tag, dt in (("bf16", torch.bfloat16), ("fp32", torch.float32)):
        m = GPT(vocab_size=V, n_embd=C, block_size=block, n_head=H, n_layer=L).eval()
        m.load_state_dict({k: v.float() for k, v in sd.items()})
        m = m.to(dt)
        with torch.inference_mode():
            out[tag] = _np(m(idx)[0])
    np.savez_compressed(
        os.path.join(HERE, "bf16_wide_init.npz"),
        meta=np.array([V, C, H, L, block, 6], dtype=np.int64), idx=_np(idx),
        logits_bf16=out["bf16"], logits_fp32=out["fp32"],
    )
    print("bf16_wide_init: reference bf16 vs fp32 rel err", np.abs(out["bf16"] - out["fp32"]).max() / np.abs(out["fp32"]).max())


def main():
    if len(sys.argv) < 2:
        raise SystemExit("usage: python tests/golden/make_golden.py /path/to/reference [fixture ...]")
    ref = sys.argv[1]
    sys.path.insert(0, os.path.join(ref, "src"))
    sys.dont_write_bytecode = True
    torch.set_num_threads(4)
    from diff_gpt.model.gpt import GPT
    from diff_gpt.model.kv_cache import KVCache

    only = set(sys.argv[2:])  # no names: every fixture

    def want(name: str) -> bool:
        return not only or name in only

    if want("small_fp32"):
        small_forward(GPT, KVCache, "small_fp32", torch.float32, 64, 32, 4, 3, 16, 0.3, 0, 2, 9)
    if want("small_bf16_d64"):
        small_forward(GPT, KVCache, "small_bf16_d64", torch.bfloat16, 128, 128, 2, 2, 32, 0.08, 1, 2, 13)
    if want("small_bf16_d32"):
        small_forward(GPT, KVCache, "small_bf16_d32", torch.bfloat16, 64, 64, 2, 3, 24, 0.1, 2, 3, 11)
    for fn in (config1, samplers, ops, engine_force, codec, teacher_forced, anomaly, cfg4_bf16_init002, bf16_wide_init):
        if want(fn.__name__):
            fn(ref)


if __name__ == "__main__":
    main()
