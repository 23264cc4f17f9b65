"""Model- and engine-level parity on the GPU against reference-generated fixtures and the CPU oracle."""

import numpy as np
import pytest
import torch

from conftest import golden_weights, load_golden
from oracle import ref_decode, ref_math

pytestmark = pytest.mark.gpu


def _model(meta, weights, dtype, **kw):
    from diff_gpt_b200 import GPT

    V, C, H, L, block = (int(x) for x in meta[:5])
    m = GPT(vocab_size=V, n_embd=C, block_size=block, n_head=H, n_layer=L, **kw).eval()
    sd = dict(weights)
    sd["lm_head.weight"] = sd["token_embedding_table.weight"]
    m.load_state_dict(sd)
    return m.to(dtype).cuda()


def _shape(meta, **kw):
    V, C, H, L, block = (int(x) for x in meta[:5])
    return ref_math.Shape(vocab_size=V, n_embd=C, n_head=H, n_layer=L, block_size=block, **kw)


CASES = [
    ("small_fp32", torch.float32, 1e-4),
    ("small_bf16_d64", torch.bfloat16, 2e-2),
    ("small_bf16_d32", torch.bfloat16, 2e-2),
]


@pytest.mark.parametrize("name,dtype,tol", CASES)
def test_forward_full_serial_chunked_vs_reference(name, dtype, tol):
    """Full causal forward, token-by-token decode through a KVCache and chunked prefill all
    reproduce the reference's logits (cf. reference tests test_gpt.py:34-76, test_mha.py:80-158)."""
    from diff_gpt_b200 import KVCache

    g = load_golden(name)
    m = _model(g["meta"], golden_weights(g, torch.float32), dtype)
    idx = torch.from_numpy(g["idx"]).cuda()
    B, T = idx.shape
    H, L, D = m.n_head, m.n_layer, m.n_embd // m.n_head
    scale = np.abs(g["logits_full"]).max()
    full, loss = m(idx)
    assert loss is None and full.shape == g["logits_full"].shape and full.dtype == dtype
    assert np.abs(full.float().cpu().numpy() - g["logits_full"]).max() <= tol * scale
    kv = KVCache(batch_size=B, num_heads=H, seq_len=T, head_dim=D, num_layers=L)
    serial = torch.cat([m(idx[:, t : t + 1], kv_cache=kv)[0] for t in range(T)], dim=1)
    assert kv.get_pos() == T
    assert np.abs(serial.float().cpu().numpy() - g["logits_serial"]).max() <= tol * scale
    cut = int(g["meta"][7])
    kv2 = KVCache(batch_size=B, num_heads=H, seq_len=T, head_dim=D, num_layers=L)
    a, _ = m(idx[:, :cut], kv_cache=kv2)
    b, _ = m(idx[:, cut:], kv_cache=kv2)
    chunked = torch.cat([a, b], dim=1).float().cpu().numpy()
    assert np.abs(chunked - g["logits_chunked"]).max() <= tol * scale
    # cache contents: K after RoPE + QK-norm, V raw, reference layout (L, 2, B, H, T, D)
    assert kv2.kv_cache.shape == g["kv_cache"].shape
    kscale = np.abs(g["kv_cache"]).max()
    assert np.abs(kv2.kv_cache.float().cpu().numpy() - g["kv_cache"]).max() <= (1e-5 if dtype == torch.float32 else 2e-2) * kscale


def test_state_dict_keys_and_tying():
    from diff_gpt_b200 import GPT

    g = load_golden("small_fp32")
    m = GPT(vocab_size=64, n_embd=32, block_size=16, n_head=4, n_layer=3)
    ref_keys = {k[2:] for k in g if k.startswith("w:")} | {"lm_head.weight"}
    assert set(m.state_dict().keys()) == ref_keys
    assert m.lm_head.weight is m.token_embedding_table.weight
    assert m.freqs_cis.shape == (32, 4, 2)
    with pytest.raises(AssertionError):
        GPT(vocab_size=100)  # not a multiple of pad_vocab_size_to


def test_softcap_bounds_and_disable():
    g = load_golden("small_fp32")
    w = golden_weights(g, torch.float32)
    idx = torch.from_numpy(g["idx"]).cuda()
    m = _model(g["meta"], w, torch.float32, logit_softcap=2.0)
    assert m(idx)[0].abs().max().item() <= 2.0
    raw = _model(g["meta"], w, torch.float32, logit_softcap=0.0)(idx)[0]
    want = ref_math.forward(_shape(g["meta"], logit_softcap=0.0), w, idx.cpu())
    assert (raw.cpu() - want).abs().max().item() <= 1e-4 * want.abs().max().item()


def test_layers_per_block_two_matches_oracle_generalisation():
    """Commit every second layer: compare with a direct restatement of block.py:74-107."""
    g = load_golden("small_fp32")
    w = golden_weights(g, torch.float32)
    shape = _shape(g["meta"])
    idx = torch.from_numpy(g["idx"])
    m = _model(g["meta"], w, torch.float32, attn_res_layers_per_block=2)
    got = m(idx.cuda())[0].cpu()
    # restatement with a commit schedule
    table = ref_math.rope_table(shape.head_dim, 2 * shape.block_size)
    cs = table[: idx.shape[1]]
    x = ref_math.rms_norm(w["token_embedding_table.weight"][idx])
    blocks, partial = [x], x
    for i in range(shape.n_layer):
        pre = f"blocks.{i}."
        h = x if (len(blocks) == 1 and partial is x) else ref_math.depth_mix(blocks + [partial], w[pre + "attn_res_proj.weight"])
        if (i + 1) % 2 == 0:
            blocks, partial = blocks + [partial], None
        a = ref_math.attention_layer(shape, w, i, ref_math.rms_norm(h), cs, None)
        partial = a if partial is None else partial + a
        h2 = ref_math.depth_mix(blocks + [partial], w[pre + "mlp_res_proj.weight"])
        partial = partial + ref_math.feed_forward(shape, w, i, ref_math.rms_norm(h2))
    want = 15 * torch.tanh(ref_math.rms_norm(partial) @ w["token_embedding_table.weight"].T / 15)
    assert (got - want).abs().max().item() <= 1e-4 * want.abs().max().item()


def test_config1_teacher_forced_logits_and_argmax_stream():
    """BASELINE config 1: drive the engine with the reference's own argmax stream as a force
    schedule and compare every step's logits; then free-run argmax and compare the streams."""
    from diff_gpt_b200 import Engine, TemperatureSampler
    from diff_gpt_b200.model.engine import DecodeRun

    g = load_golden("cfg1_fp32")
    m = _model(g["meta"], golden_weights(g, torch.float32), torch.float32)
    prompt = g["prompt"].tolist()
    stream = g["argmax_stream"].tolist()
    ref_logits = g["step_logits"]
    G = len(stream)
    run = DecodeRun(m, [prompt], 4, G, TemperatureSampler(0.0), 42, [stream], use_graph=False)
    run.start()
    got = [15 * torch.tanh(run.logits0[0].float() / 15).cpu().numpy()]
    for _ in range(G - 1):
        run.advance(1)
        lg = run.logits[0].float()
        got.append((15 * torch.tanh(lg / 15)).cpu().numpy())
    got = np.stack(got)
    assert np.abs(got - ref_logits).max() <= 1e-4 * np.abs(ref_logits).max()
    assert run.history.cpu()[:, :G].tolist() == [stream] * 4
    # free-running argmax: identical stream (the fixture's top-2 gaps are far above 1e-4 relative)
    top2 = np.sort(ref_logits, axis=-1)[:, -2:]
    assert (top2[:, 1] - top2[:, 0]).min() > 1e-4 * np.abs(ref_logits).max()
    res, masks = Engine(m).generate_batch(prompt, num_samples=3, max_tokens=G, sampler=TemperatureSampler(0.0))
    assert all(r[: len(prompt)] == prompt and r[len(prompt) :] == stream for r in res)
    assert all(mk == [0] * len(prompt) + [1] * G for mk in masks)


def test_engine_force_schedule_fixture():
    from diff_gpt_b200 import Engine, TemperatureSampler

    g = load_golden("engine_force")
    m = _model(g["meta"], golden_weights(g, torch.float32), torch.float32)
    sched = [None if s < 0 else int(s) for s in g["sched"]]
    res, masks = Engine(m).generate_batch(
        g["prompt"].tolist(), num_samples=3, max_tokens=10, sampler=TemperatureSampler(0.0), force_schedule=sched
    )
    assert np.array_equal(np.asarray(res), g["results"])
    assert np.array_equal(np.asarray(masks), g["masks"])


def test_engine_streaming_equals_batch_and_graph_equals_eager():
    from diff_gpt_b200 import Engine, NucleusSampler, TemperatureSampler

    g = load_golden("small_bf16_d64")
    m = _model(g["meta"], golden_weights(g, torch.float32), torch.bfloat16)
    prompt = g["idx"][0].tolist()
    s = NucleusSampler(0.9, TemperatureSampler(1.0))
    eng = Engine(m)
    res, _ = eng.generate_batch(prompt, num_samples=40, max_tokens=19, sampler=s, seed=7)
    cols = list(eng.generate(prompt, num_samples=40, max_tokens=19, sampler=s, seed=7))
    assert len(cols) == 19
    streamed = np.asarray([c[0] for c in cols]).T
    assert np.array_equal(streamed, np.asarray(res)[:, len(prompt) :])
    t_graph, _ = eng.generate_many([prompt], 40, 19, s, seed=7, use_graph=True)
    t_eager, _ = eng.generate_many([prompt], 40, 19, s, seed=7, use_graph=False)
    assert torch.equal(t_graph, t_eager)
    assert torch.equal(t_graph[0].cpu(), torch.tensor(res)[:, len(prompt) :].int())
    other, _ = eng.generate_many([prompt], 40, 19, s, seed=8)
    assert not torch.equal(other, t_graph)
    assert len({tuple(r) for r in t_graph[0].cpu().tolist()}) > 1


def test_engine_validation_and_ceiling():
    from diff_gpt_b200 import Engine, TemperatureSampler

    g = load_golden("small_fp32")
    m = _model(g["meta"], golden_weights(g, torch.float32), torch.float32)  # block_size 16 -> ceiling 32
    eng = Engine(m)
    with pytest.raises(AssertionError, match="non-empty"):
        eng.generate_batch([], num_samples=1, max_tokens=2)
    with pytest.raises(AssertionError, match="list of ints"):
        eng.generate_batch([1.5, 2], num_samples=1, max_tokens=2)
    with pytest.raises(AssertionError, match="force_schedule must cover"):
        eng.generate_batch([1, 2, 3], num_samples=1, max_tokens=5, force_schedule=[None, 1])
    res, _ = eng.generate_batch(list(range(30)), num_samples=2, max_tokens=10, sampler=TemperatureSampler(0.0))
    assert all(len(r) == 32 for r in res)  # clamped to 2 * block_size
    res, _ = eng.generate_batch(list(range(32)), num_samples=2, max_tokens=10)
    assert all(len(r) == 32 for r in res)  # nothing to generate


def test_prefill_once_equals_independent_runs_and_shared_prefix_phase():
    """N trajectories from one prefill equal N single runs under argmax (reference test_engine.py:301-347);
    with >= 16 trajectories the shared-prefix phase is active and must give the same tokens."""
    from diff_gpt_b200 import Engine, TemperatureSampler

    g = load_golden("small_bf16_d32")
    w = golden_weights(g, torch.float32)
    m = _model(g["meta"], w, torch.float32)
    prompt = g["idx"][1].tolist()
    eng = Engine(m)
    one, _ = eng.generate_batch(prompt, num_samples=1, max_tokens=12, sampler=TemperatureSampler(0.0))
    many, _ = eng.generate_batch(prompt, num_samples=20, max_tokens=12, sampler=TemperatureSampler(0.0))
    assert all(r == one[0] for r in many)
    shape = _shape(g["meta"])
    ref, _, _ = ref_decode.mc_decode(shape, w, prompt, 1, 12, temperature=0.0)
    assert one[0][len(prompt) :] == ref[0].tolist()


def test_multi_series_batch_equals_single_series_runs():
    from diff_gpt_b200 import Engine, NucleusSampler, TemperatureSampler

    g = load_golden("small_bf16_d32")
    m = _model(g["meta"], golden_weights(g, torch.float32), torch.float32)
    prompts = [g["idx"][0].tolist(), g["idx"][1].tolist()[:7], g["idx"][2].tolist()]
    s = NucleusSampler(0.8, TemperatureSampler(1.3))
    eng = Engine(m)
    toks, masks = eng.generate_many(prompts, 18, 9, s, seed=3)
    assert toks.shape == (3, 18, 9) and bool((masks == 1).all())
    for i, p in enumerate(prompts):
        solo, _ = eng.generate_many([p], 18, 9, s, seed=3, series_offset=i)
        assert torch.equal(solo[0], toks[i]), i
    # a shard of the trajectories reproduces its slice of the full run
    part, _ = eng.generate_many(prompts, 6, 9, s, seed=3, traj_offset=12)
    assert torch.equal(part, toks[:, 12:18])
    # per-series force schedules
    sch = [[None, 5, None] + [None] * 6, [7, None, None] + [None] * 6, [None] * 9]
    ft, fm = eng.generate_many(prompts, 18, 9, s, seed=3, force_schedules=sch)
    assert bool((ft[0, :, 1] == 5).all()) and bool((ft[1, :, 0] == 7).all())
    assert fm[0, 0].tolist() == [1, 0, 1, 1, 1, 1, 1, 1, 1] and fm[2, 0].tolist() == [1] * 9


def test_engine_reuses_decode_state_across_calls_of_one_shape():
    """A second call of the same shape reloads prompts into the cached pool, plans and graph; its tokens
    equal those of a fresh engine, with and without teacher forcing, and after the weights changed."""
    from diff_gpt_b200 import Engine, NucleusSampler, TemperatureSampler

    g = load_golden("small_bf16_d32")
    m = _model(g["meta"], golden_weights(g, torch.float32), torch.float32)
    s = NucleusSampler(0.9, TemperatureSampler(1.1))
    a = [g["idx"][0].tolist(), g["idx"][1].tolist()]
    b = [g["idx"][2].tolist(), g["idx"][0].tolist()[::-1]]
    eng = Engine(m)
    first, _ = eng.generate_many(a, 20, 10, s, seed=5)
    run = eng._run
    second, _ = eng.generate_many(b, 20, 10, s, seed=5, series_offset=2, traj_offset=3)
    assert eng._run is run and run.graph is not None  # same state, same captured graph
    fresh, _ = Engine(m).generate_many(b, 20, 10, s, seed=5, series_offset=2, traj_offset=3)
    assert torch.equal(second, fresh)
    again, _ = eng.generate_many(a, 20, 10, s, seed=5)
    assert torch.equal(again, first)
    # forcing: schedules are reloaded too
    sch1 = [[None, 4] + [None] * 8, [None] * 10]
    sch2 = [[9] + [None] * 9, [None, None, 3] + [None] * 7]
    eng.generate_many(a, 20, 10, s, seed=5, force_schedules=sch1)
    run = eng._run
    f2, m2 = eng.generate_many(b, 20, 10, s, seed=5, force_schedules=sch2)
    assert eng._run is run
    w2, wm2 = Engine(m).generate_many(b, 20, 10, s, seed=5, force_schedules=sch2)
    assert torch.equal(f2, w2) and torch.equal(m2, wm2) and bool((f2[0, :, 0] == 9).all())
    # another shape, or new weights, rebuild instead of replaying a stale graph
    eng.generate_many(a, 20, 7, s, seed=5)
    assert eng._run is not run
    run = eng._run
    with torch.no_grad():
        m.token_embedding_table.weight.mul_(1.5)
    changed, _ = eng.generate_many(a, 20, 7, s, seed=5)
    assert eng._run is not run
    want, _ = Engine(m).generate_many(a, 20, 7, s, seed=5)
    assert torch.equal(changed, want)
    eng.release()
    assert eng._run is None


def test_overlapped_prefix_phase_equals_sequential():
    """Shared-prompt phase beside the per-row phase on a second stream (then a merge launch) against the
    one-stream form whose per-row kernel merges in its epilogue: same tokens, eager and graph."""
    from diff_gpt_b200 import Engine, TemperatureSampler

    g = load_golden("small_bf16_d32")
    w = golden_weights(g, torch.float32)
    m = _model(g["meta"], w, torch.float32)
    prompts = [g["idx"][0].tolist(), g["idx"][2].tolist()]
    s = TemperatureSampler(0.0)
    outs = []
    for overlap in (False, True):
        for graph in (False, True):
            t, _ = Engine(m).generate_many(prompts, 24, 12, s, seed=1, overlap_prefix=overlap, use_graph=graph)
            outs.append(t)
    assert all(torch.equal(outs[0], o) for o in outs[1:])
    ref, _, _ = ref_decode.mc_decode(_shape(g["meta"]), w, prompts[0], 1, 12, temperature=0.0)
    assert outs[3][0, 0].tolist() == ref[0].tolist()


def test_python_callable_sampler_sees_device_logits():
    from diff_gpt_b200 import Engine

    g = load_golden("small_fp32")
    w = golden_weights(g, torch.float32)
    m = _model(g["meta"], w, torch.float32)
    seen = []

    def pick(logits, rng=None):
        assert logits.is_cuda and logits.shape == (3, 64)
        seen.append(logits.float().cpu())
        return torch.argmax(logits, dim=-1, keepdim=True)

    prompt = [3, 1, 4, 1, 5]
    res, masks = Engine(m).generate_batch(prompt, num_samples=3, max_tokens=6, sampler=pick)
    ref, _, ref_logits = ref_decode.mc_decode(_shape(g["meta"]), w, prompt, 3, 6, temperature=0.0, keep_logits=True)
    assert torch.tensor(res)[:, 5:].tolist() == ref.tolist()
    got = torch.stack(seen)
    assert (got - ref_logits).abs().max().item() <= 1e-4 * ref_logits.abs().max().item()


def test_samplers_standalone_contract():
    """Shape (B,1) int64, seeded determinism, T=0 == argmax, p -> 0 == argmax, p = 1 == inner sampler
    (reference tests/diff_gpt/sampler/*.py)."""
    from diff_gpt_b200 import NucleusSampler, TemperatureSampler

    logits = torch.randn(4, 50, generator=torch.Generator().manual_seed(0)).cuda()
    for s in (TemperatureSampler(1.0), NucleusSampler(0.9, TemperatureSampler(1.5))):
        out = s(logits)
        assert out.shape == (4, 1) and out.dtype == torch.int64
        a = s(logits, rng=torch.Generator(device="cuda").manual_seed(42))
        b = s(logits, rng=torch.Generator(device="cuda").manual_seed(42))
        assert torch.equal(a, b)
        many = [s(logits, rng=torch.Generator().manual_seed(k)) for k in range(12)]
        assert any(not torch.equal(many[0], x) for x in many[1:])
    am = torch.argmax(logits, -1, keepdim=True)
    assert torch.equal(TemperatureSampler(0.0)(logits), am)
    assert torch.equal(NucleusSampler(1e-9, TemperatureSampler(1.0))(logits), am)
    assert torch.equal(NucleusSampler(0.5, TemperatureSampler(0.0))(logits), am)
    r1 = NucleusSampler(1.0, TemperatureSampler(1.0))(logits, rng=torch.Generator().manual_seed(5))
    r2 = TemperatureSampler(1.0)(logits, rng=torch.Generator().manual_seed(5))
    assert torch.equal(r1, r2)
    # a foreign inner sampler receives -inf outside the nucleus
    probs = torch.tensor([[0.6, 0.25, 0.1, 0.05]]).log().cuda()

    class Inner:
        def __call__(self, lg, rng=None):
            self.lg = lg
            return torch.argmax(lg, -1, keepdim=True)

    inner = Inner()
    NucleusSampler(0.9, inner)(probs)
    assert torch.isfinite(inner.lg).cpu().tolist() == [[True, True, True, False]]


def test_diffgpt_facade_config1_and_teacher_forced():
    """predict / predict_samples / predict_quantiles / teacher-forced predict reproduce the reference's
    frames under argmax (values are decoded from identical token streams, so they match to the bit)."""
    import pandas as pd

    from diff_gpt_b200 import TemperatureSampler
    from diff_gpt_b200.diff_gpt import DiffGPT

    g = load_golden("cfg1_fp32")
    m = _model(g["meta"], golden_weights(g, torch.float32), torch.float32)
    dg = DiffGPT(model=m, order_of_derivative=1, domain_of_definition=g["domain"], use_decimal=False)
    df = pd.DataFrame(g["ctx"], columns=["y"])
    fut = dg.predict_samples(df, max_new_points=48, num_samples=4, sampler=TemperatureSampler(0.0))
    assert fut.shape == (4, 48, 1) and np.array_equal(fut, g["futures_t0"])
    pred = dg.predict(df, max_new_points=48, sampler=TemperatureSampler(0.0))
    assert list(pred.columns) == ["y"] and np.array_equal(pred.to_numpy(), g["predict_t0"])
    q = dg.predict_quantiles(df, 48, quantiles=(0.1, 0.5, 0.9), num_samples=4, sampler=TemperatureSampler(0.0))
    assert np.array_equal(q[0.5].to_numpy(), g["q50_t0"])
    # stochastic bands are ordered (reference test_diff_gpt.py:295-317)
    qs = dg.predict_quantiles(df, 48, quantiles=(0.1, 0.5, 0.9), num_samples=64, sampler=TemperatureSampler(1.0))
    assert (qs[0.1].to_numpy() <= qs[0.5].to_numpy()).all() and (qs[0.5].to_numpy() <= qs[0.9].to_numpy()).all()
    with pytest.raises(AssertionError, match="block_size"):
        dg.predict_samples(pd.DataFrame(g["walk"].reshape(-1, 1), columns=["y"]), 48, 2)  # 96 + 48 - 1 > 138

    t = load_golden("teacher_forced")
    m2 = _model(t["meta"], golden_weights(t, torch.float32), torch.float32)
    dg2 = DiffGPT(model=m2, order_of_derivative=t["order"], domain_of_definition=t["dom"], use_decimal=False)
    ctx = pd.DataFrame(t["x"][:20], columns=["a", "b", "c"])
    future = pd.DataFrame(t["x"][20:], columns=["a", "b", "c"])
    tf = dg2.predict(ctx, future_covariates_df=future, target_columns=["a"], sampler=TemperatureSampler(0.0))
    assert np.array_equal(tf.to_numpy(), t["teacher_forced"])
    ar = dg2.predict(ctx, max_new_points=6, sampler=TemperatureSampler(0.0))
    assert np.array_equal(ar.to_numpy(), t["autoregressive"])
    ps = dg2.predict_samples(ctx, max_new_points=6, num_samples=3, sampler=TemperatureSampler(0.0))
    assert np.array_equal(ps, t["samples"])


def test_anomaly_scores_match_reference_and_bf16_runs():
    """DiffGPT.anomaly_scores (one prefill + dgpt_token_nll) against the reference's frames, NaN pattern included;
    a bf16 module (which the reference cannot score) stays close to the fp32 scores."""
    import pandas as pd

    from diff_gpt_b200.diff_gpt import DiffGPT

    g = load_golden("anomaly")
    w = golden_weights(g, torch.float32)
    m = _model(g["meta"], w, torch.float32)
    df = pd.DataFrame(g["x"], columns=["a", "b", "c"], index=np.arange(100, 100 + len(g["x"])))
    for order, dom, key in ((g["order"], g["dom"], "scores_fp32"), (1, g["dom_k1"], "scores_fp32_k1")):
        got = DiffGPT(model=m, order_of_derivative=order, domain_of_definition=dom, use_decimal=False).anomaly_scores(df)
        assert list(got.columns) == ["a", "b", "c"] and got.index.equals(df.index)
        want = g[key]
        assert np.array_equal(np.isnan(got.to_numpy()), np.isnan(want))
        assert np.nanmax(np.abs(got.to_numpy() - want)) <= 1e-4 * np.nanmax(np.abs(want))
    mb = _model(g["meta"], w, torch.bfloat16)
    sb = DiffGPT(model=mb, order_of_derivative=g["order"], domain_of_definition=g["dom"], use_decimal=False).anomaly_scores(df)
    assert np.array_equal(np.isnan(sb.to_numpy()), np.isnan(g["scores_fp32"]))
    assert np.nanmax(np.abs(sb.to_numpy() - g["scores_fp32"])) <= 0.15  # bf16 logits of |z| <= 15 carry ~0.06 of rounding
    with pytest.raises(AssertionError, match="block_size"):
        big = pd.DataFrame(np.tile(g["x"], (2, 1)), columns=["a", "b", "c"])  # 58 x 3 tokens > block 96
        DiffGPT(model=m, order_of_derivative=g["order"], domain_of_definition=g["dom"], use_decimal=False).anomaly_scores(big)


def test_token_nll_kernel_against_torch():
    from diff_gpt_b200 import ops

    gen = torch.Generator().manual_seed(11)
    for dtype, tol in ((torch.float32, 2e-6), (torch.bfloat16, 8e-3)):
        for V in (7, 64, 1000, 4096):
            x = (torch.randn(37, V, generator=gen) * 4).to(dtype)
            t = torch.randint(0, V, (37,), generator=gen)
            status = torch.zeros(1, dtype=torch.int32, device="cuda")
            got = ops.token_nll(x.cuda(), t.to(torch.int32).cuda(), status).cpu()
            want = -torch.log_softmax(x.float(), -1).gather(-1, t[:, None])[:, 0]
            assert (got - want).abs().max().item() <= tol * max(1.0, want.abs().max().item()), (dtype, V)
            assert status.item() == 0
    # a row slice with a stride, and a target outside the vocabulary: NaN for that row and a status bit
    x = torch.randn(5, 3, 32, generator=gen).cuda()
    t = torch.tensor([1, 2, 40, 0, 31], dtype=torch.int32).cuda()
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    got = ops.token_nll(x[:, 1], t, status).cpu()
    want = -torch.log_softmax(x[:, 1].cpu(), -1)
    assert torch.isnan(got[2]) and status.item() == 4
    for r in (0, 1, 3, 4):
        assert abs(got[r].item() - want[r, int(t[r])].item()) <= 1e-5


def test_kv_cache_reference_surface():
    """Lazy allocation, growth in multiples of 1024, pos on the last layer only, batch broadcast, reset
    (reference tests/diff_gpt/model/test_kv_cache.py)."""
    from diff_gpt_b200 import KVCache

    c = KVCache(batch_size=2, num_heads=2, seq_len=4, head_dim=8, num_layers=2)
    assert c.kv_cache.numel() == 0 and c.get_pos() == 0
    k = torch.randn(2, 2, 3, 8, device="cuda")
    kk, vv = c.insert_kv(0, k, k * 2)
    assert c.get_pos() == 0 and kk.shape == (2, 2, 3, 8)
    c.insert_kv(1, k, k)
    assert c.get_pos() == 3
    c.insert_kv(0, k, k)  # 6 > 4: grow to (6 + 1024) rounded up to 1024 = 2048
    assert c.kv_cache.shape[4] == 2048 and c.kv_shape[4] == 2048
    assert torch.equal(c.kv_cache[0, 0, :, :, :3], k) and torch.equal(c.kv_cache[0, 1, :, :, :3], k * 2)
    one = KVCache(batch_size=1, num_heads=2, seq_len=3, head_dim=8, num_layers=2)
    one.insert_kv(0, k[:1], k[:1])
    one.insert_kv(1, k[:1], k[:1])
    wide = KVCache(batch_size=5, num_heads=2, seq_len=9, head_dim=8, num_layers=2)
    wide.prefill(one)
    assert wide.get_pos() == 3 and torch.equal(wide.kv_cache[1, 0, 4, :, :3], k[0])
    wide.reset()
    assert wide.get_pos() == 0


def test_device_side_decode_and_quantiles_equal_the_host_path():
    """dgpt_integrate_tokens against the host decode of whole sequences (mixed orders, bit for bit), and the
    device-side quantiles of DiffGPT.predict_quantiles against np.quantile over predict_samples."""
    import pandas as pd

    from diff_gpt_b200 import TemperatureSampler, ops
    from diff_gpt_b200.diff_gpt import DiffGPT, _quantile_of_sorted
    from diff_gpt_b200.encoder_decoder import _orders, decode, encode, get_domain_of_definition, integrate_end_state

    rng = np.random.default_rng(7)
    V, F, rows, H, N = 256, 5, 40, 12, 33
    order = np.array([0, 1, 2, 3, 1])
    x = np.cumsum(rng.normal(size=(rows, F)), axis=0)
    dom = get_domain_of_definition(x, order, use_decimal=False)
    start, scale, enc = encode(inp=x, vocab_size=V, domain_of_definition=dom, order_of_derivative=order, use_decimal=False)
    gen = rng.integers(0, V, size=(N, H * F))
    whole = np.concatenate([np.broadcast_to(enc.reshape(1, -1), (N, enc.size)), gen], axis=1).reshape(N, -1, F)
    want = decode(start=start, scale=scale, inp=whole.astype(np.int64), vocab_size=V, order_of_derivative=order,
                  use_decimal=False)[:, rows:]
    state = integrate_end_state(start, (enc - V // 2) / scale, order)
    sc = np.array(np.broadcast_to(np.asarray(scale, dtype=np.float64).reshape(-1), (F,)))
    got = ops.integrate_tokens(
        torch.from_numpy(gen.astype(np.int32)).cuda(), F, V, torch.from_numpy(sc).cuda(),
        torch.from_numpy(_orders(order, F).astype(np.int32)).cuda(), torch.from_numpy(state).cuda(),
    )
    assert got.shape == (N, H, F) and np.array_equal(got.cpu().numpy(), want)
    srt = torch.sort(got, dim=0).values
    for q in (0.1, 0.5, 0.9):
        assert np.array_equal(_quantile_of_sorted(srt, q).cpu().numpy(), np.quantile(want, q, axis=0))
    # through the facade: same trajectories from predict_samples and inside predict_quantiles (seeded stream)
    g = load_golden("cfg1_fp32")
    m = _model(g["meta"], golden_weights(g, torch.float32), torch.float32)
    dg = DiffGPT(model=m, order_of_derivative=1, domain_of_definition=g["domain"], use_decimal=False)
    df = pd.DataFrame(g["ctx"], columns=["y"])
    s = TemperatureSampler(1.0)
    fut = dg.predict_samples(df, max_new_points=24, num_samples=50, sampler=s)
    qs = dg.predict_quantiles(df, 24, quantiles=(0.1, 0.5, 0.9), num_samples=50, sampler=s)
    for q in (0.1, 0.5, 0.9):
        assert np.array_equal(qs[q].to_numpy(), np.quantile(fut, q, axis=0))


def test_gpt_generate_without_cache_matches_the_engine_under_argmax():
    """GPT.generate (the reference's cache-free sliding-window loop, gpt.py:202-237) and the KV-cache engine produce
    the same argmax continuation while the window has not started to slide; beyond block_size it keeps going."""
    from diff_gpt_b200 import Engine, TemperatureSampler

    g = load_golden("small_bf16_d32")
    w = golden_weights(g, torch.float32)
    m = _model(g["meta"], w, torch.float32)
    prompt = g["idx"][0].tolist()
    room = m.block_size - len(prompt)
    out = m.generate(torch.tensor([prompt], device="cuda"), room, TemperatureSampler(0.0))
    assert out.shape == (1, m.block_size) and out[0, : len(prompt)].tolist() == prompt
    res, _ = Engine(m).generate_batch(prompt, num_samples=1, max_tokens=room, sampler=TemperatureSampler(0.0))
    assert out[0].tolist() == res[0]
    ref, _, _ = ref_decode.mc_decode(_shape(g["meta"]), w, prompt, 1, room, temperature=0.0)
    assert out[0, len(prompt) :].tolist() == ref[0].tolist()
    longer = m.generate(torch.tensor([prompt], device="cuda"), room + 5, TemperatureSampler(1.0), seed=3)
    assert longer.shape == (1, m.block_size + 5) and int(longer.min()) >= 0 and int(longer.max()) < m.vocab_size


def test_generate_batch_rejects_unknown_keywords():
    """The reference forwards **kwargs to generate(), so a misspelt keyword is a TypeError there (engine.py:156-169)."""
    from diff_gpt_b200 import Engine

    g = load_golden("small_fp32")
    m = _model(g["meta"], golden_weights(g, torch.float32), torch.float32)
    with pytest.raises(TypeError, match="max_token"):
        Engine(m).generate_batch([1, 2, 3], num_samples=2, max_token=4)


def test_shards_below_the_sharing_threshold_follow_the_whole_jobs_path():
    """24 trajectories decoded as 12 + 12 (each below the 16-row threshold of the shared-prompt phase) with the
    whole job's path handed down equal the 24 decoded at once, token for token; an empty shard returns empty tensors."""
    from diff_gpt_b200 import Engine, NucleusSampler, TemperatureSampler

    g = load_golden("small_bf16_d64")
    m = _model(g["meta"], golden_weights(g, torch.float32), torch.bfloat16)
    prompts = [g["idx"][0].tolist(), g["idx"][1].tolist()]
    s = NucleusSampler(0.9, TemperatureSampler(1.0))
    eng = Engine(m)
    whole, _ = eng.generate_many(prompts, 24, 10, s, seed=11)
    lo, _ = eng.generate_many(prompts, 12, 10, s, seed=11, traj_offset=0, shared_prefix=True)
    hi, _ = eng.generate_many(prompts, 12, 10, s, seed=11, traj_offset=12, shared_prefix=True)
    assert torch.equal(torch.cat([lo, hi], dim=1), whole)
    none, masks = eng.generate_many(prompts, 0, 10, s, seed=11, traj_offset=24)
    assert none.shape == (2, 0, 10) and masks.shape == (2, 0, 10)


def test_difference_order_above_the_device_codec_takes_the_host_codec():
    """Order 9 (the reference accepts any order in float64): predict_samples tokenises and decodes on the host and
    still decodes the trajectories on the device; under argmax every trajectory equals the host-side restatement."""
    import pandas as pd

    from diff_gpt_b200 import TemperatureSampler
    from diff_gpt_b200.diff_gpt import DiffGPT
    from diff_gpt_b200.encoder_decoder import decode, encode, get_domain_of_definition

    g = load_golden("small_fp32")
    w = golden_weights(g, torch.float32)
    m = _model(g["meta"], w, torch.float32)  # block_size 16
    x = np.cumsum(np.random.default_rng(5).normal(0, 1, (14, 1)), axis=0)
    dom = get_domain_of_definition(x, 9, use_decimal=False)
    dg = DiffGPT(model=m, order_of_derivative=9, domain_of_definition=dom, use_decimal=False)
    df = pd.DataFrame(x, columns=["y"])
    fut = dg.predict_samples(df, max_new_points=4, num_samples=3, sampler=TemperatureSampler(0.0))
    assert fut.shape == (3, 4, 1) and np.isfinite(fut).all()
    start, scale, tok = encode(inp=x, vocab_size=64, domain_of_definition=dom, order_of_derivative=9, use_decimal=False)
    prompt = tok.reshape(-1).astype(np.int64).tolist()
    ref, _, _ = ref_decode.mc_decode(_shape(g["meta"]), w, prompt, 1, 4, temperature=0.0)
    full = np.asarray(prompt + ref[0].tolist(), dtype=np.int64).reshape(1, -1, 1)
    want = decode(start=start, scale=scale, inp=full, vocab_size=64, order_of_derivative=9, use_decimal=False)[0, 14:18]
    assert np.array_equal(fut[0], want) and np.array_equal(fut[1], want)
