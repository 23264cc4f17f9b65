"""Benchmark of the Monte-Carlo decode path (BASELINE config 4) on 1..8 B200s of one box.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N ... bench.py --gpus N ...

Workload ("step"): W = n_gpus series are decoded per step; each rank prefills the
1024-token prompt of one series of the step, the ranks exchange the prompt K/V (one
all-gather), and each decodes its contiguous slice of
4096 / W of every series' 4096 trajectories for 256 tokens with top-p 0.9 /
temperature 1 sampling, then the token streams are all-gathered.  Every rank
therefore carries 4096 trajectories per step whatever N is (weak scaling), and at
N = 1 a step is exactly one series of config 4.  Model: vocab 4096, n_embd 768,
12 heads (head_dim 64), 12 layers, block 2048, bf16, weights N(0, 0.02) seed 4.
Inputs are seeded synthetic random-walk + seasonal series tokenised with the
order-1 sigma-delta encoder; nothing is read from disk.

One JSON line is printed by rank 0.  `value` is device-timed with the prompts
already resident in HBM; `e2e` goes through `Engine.generate_many` with host
prompts and a device->host copy of all tokens inside the timed region, and at N = 1
`e2e.predict_samples` times the reference's own call, `DiffGPT.predict_samples`, from a
float64 host frame to the float64 host array of forecasts.  The KV
pool (38.7 GB per rank) is far larger than L2, so no explicit L2 flush is needed.
"""

from __future__ import annotations

import argparse
import json
import os
import statistics
import sys
import time

import numpy as np
import torch

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

CFG4 = dict(vocab_size=4096, n_embd=768, n_head=12, n_layer=12, block_size=2048)
PROMPT_TOKENS, HORIZON, TRAJECTORIES, N_SERIES = 1024, 256, 4096, 32
TOP_P, TEMPERATURE, WEIGHT_SEED = 0.9, 1.0, 4


_RESULT_OUT = None


def claim_stdout() -> None:
    """Keep stdout for the one JSON line: libraries that print there (NCCL's version banner) are sent to stderr."""
    global _RESULT_OUT
    if _RESULT_OUT is None:
        sys.stdout.flush()
        _RESULT_OUT = os.fdopen(os.dup(1), "w")
        os.dup2(2, 1)


def emit(line: dict) -> None:
    out = _RESULT_OUT if _RESULT_OUT is not None else sys.stdout
    print(json.dumps(line), file=out, flush=True)


def peaks() -> dict:
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        p = json.load(open(path))
        return {"hbm_gbs": p["hbm_gbs"], "bf16_tflops": p["bf16_tflops"], "bf16_tflops_sustained": p["bf16_tflops_sustained"], "source": "measured"}
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0, "source": "fallback"}


def synthetic_series(n_series: int) -> list[np.ndarray]:
    """Random walk (step sd 0.5) + sin(2 pi t / 24), 1025 points per series, float64 [1025, 1]."""
    rng = np.random.default_rng(4)
    t = np.arange(PROMPT_TOKENS + 1)
    return [(np.cumsum(rng.normal(0.0, 0.5, t.size)) + np.sin(2 * np.pi * t / 24.0)).reshape(-1, 1) for _ in range(n_series)]


def host_codec():
    """The host tokeniser (plain numpy), loaded from its file so that a process which only needs prompts (the
    reference arm) does not import the package and so never maps the CUDA library."""
    import importlib.util

    name = "_dgpt_host_codec"
    if name in sys.modules:
        return sys.modules[name]
    spec = importlib.util.spec_from_file_location(name, os.path.join(ROOT, "diff_gpt_b200", "encoder_decoder.py"))
    mod = importlib.util.module_from_spec(spec)
    sys.modules[name] = mod
    spec.loader.exec_module(mod)
    return mod


def synthetic_prompts(n_series: int, vocab: int) -> list[list[int]]:
    """The synthetic series as 1024 order-1 tokens each."""
    encode, get_domain_of_definition = host_codec().encode, host_codec().get_domain_of_definition

    out = []
    for x in synthetic_series(n_series):
        dom = get_domain_of_definition(x, 1, use_decimal=False)
        _, _, tok = encode(inp=x, vocab_size=vocab, domain_of_definition=dom, order_of_derivative=1, use_decimal=False)
        out.append(tok.reshape(-1).astype(np.int64).tolist())
    return out


def seeded_weights(cfg: dict, seed: int, dtype, std: float = 0.02) -> dict:
    """state_dict of a model of shape `cfg`: every parameter ~ N(0, std) from one torch.Generator(seed), drawn in a
    fixed order (embedding, then per layer q, k, v, g, proj, the two feed-forward matrices, the two depth-mix queries)."""
    g = torch.Generator().manual_seed(seed)
    C, V = cfg["n_embd"], cfg["vocab_size"]

    def n(*s):
        return (torch.randn(*s, generator=g) * std).to(dtype)

    w = {"token_embedding_table.weight": n(V, C)}
    for i in range(cfg["n_layer"]):
        p = f"blocks.{i}."
        for name in ("c_q", "c_k", "c_v", "c_g", "c_proj"):
            w[p + f"sa.{name}.weight"] = n(C, C)
        w[p + "ffwd.net.0.weight"] = n(4 * C, C)
        w[p + "ffwd.net.2.weight"] = n(C, 2 * C)
        w[p + "attn_res_proj.weight"] = n(1, C)
        w[p + "mlp_res_proj.weight"] = n(1, C)
    return w


def cfg4_weights(dtype) -> dict:
    """Config 4: N(0, 0.02), seed 4."""
    return seeded_weights(CFG4, WEIGHT_SEED, dtype)


def load_into(model, w: dict, dtype, device=None):
    """Weights into a module with the reference's parameter names (the reference's GPT or this package's)."""
    sd = {k: v.float() for k, v in w.items()}
    sd["lm_head.weight"] = sd["token_embedding_table.weight"]
    model.load_state_dict(sd)
    model = model.to(dtype)
    return (model.to(device) if device is not None else model).eval()


def oracle_shape():
    from oracle import ref_math  # CPU legs only

    return ref_math.Shape(**CFG4)


class ClockSampler:
    """SM clock and throttle reasons of one GPU, polled through NVML from a thread while the timed region runs.

    (Polling with an `nvidia-smi -lms 200` child process perturbed the measurement by up to 30 %; NVML reads of
    one device every 250 ms do not.)  Only reads settings; never changes any.
    """

    REASONS = {
        "hw_slowdown": 0x8, "sw_power_cap": 0x4, "sw_thermal_slowdown": 0x20, "hw_thermal_slowdown": 0x40,
    }

    def __init__(self, index: int) -> None:
        import threading

        self.sm, self.mask, self.max_mhz, self.err = [], 0, None, None
        self._stop = threading.Event()
        try:
            import pynvml

            pynvml.nvmlInit()
            visible = os.environ.get("CUDA_VISIBLE_DEVICES")
            phys = int(visible.split(",")[index]) if visible and visible.split(",")[index].isdigit() else index
            self.h = pynvml.nvmlDeviceGetHandleByIndex(phys)
            self.nv = pynvml
            self.max_mhz = float(pynvml.nvmlDeviceGetMaxClockInfo(self.h, pynvml.NVML_CLOCK_SM))
        except Exception as e:  # noqa: BLE001 - NVML missing or not permitted: report it, do not fail the benchmark
            self.err = f"nvml unavailable: {e}"
            self.t = None
            return
        self.t = threading.Thread(target=self._loop, daemon=True)
        self.t.start()

    def _loop(self) -> None:
        while not self._stop.is_set():
            try:
                self.sm.append(float(self.nv.nvmlDeviceGetClockInfo(self.h, self.nv.NVML_CLOCK_SM)))
                self.mask |= int(self.nv.nvmlDeviceGetCurrentClocksEventReasons(self.h))
            except Exception as e:  # noqa: BLE001
                self.err = str(e)
                return
            self._stop.wait(0.25)

    def stop(self) -> dict:
        if self.t is not None:
            self._stop.set()
            self.t.join()
        reasons = sorted(k for k, bit in self.REASONS.items() if self.mask & bit)
        if self.err:
            reasons.append(self.err)
        return {
            "sm_mhz": statistics.median(self.sm) if self.sm else None,
            "sm_max_mhz": self.max_mhz,
            "samples": len(self.sm),
            "reasons": reasons,
        }


# ---------------------------------------------------------------------------------------
# CPU legs: the reference itself when it is installed under baseline/_ref (pip install --target),
# else the oracle port of the same path; all host threads
# ---------------------------------------------------------------------------------------
CPU_SAMPLE = dict(series=1, trajectories=64, steps=32)


def host_threads() -> int:
    """Use every core this process may run on (a launcher may have set OMP_NUM_THREADS=1) and say how many."""
    n = len(os.sched_getaffinity(0))
    torch.set_num_threads(n)
    return torch.get_num_threads()


class ReferenceSide:
    """The reference's own classes, imported from baseline/_ref; `available` is False when it is not installed."""

    def __init__(self) -> None:
        path = os.path.join(ROOT, "baseline", "_ref")
        self.available = os.path.isdir(os.path.join(path, "diff_gpt"))
        if not self.available:
            return
        if path not in sys.path:
            sys.path.insert(0, path)
        from diff_gpt.diff_gpt import DiffGPT
        from diff_gpt.model.engine import Engine
        from diff_gpt.model.gpt import GPT
        from diff_gpt.sampler.nucleus import NucleusSampler
        from diff_gpt.sampler.temperature import TemperatureSampler

        self.GPT, self.Engine, self.DiffGPT = GPT, Engine, DiffGPT
        self.NucleusSampler, self.TemperatureSampler = NucleusSampler, TemperatureSampler

    def model(self, cfg: dict, w: dict, dtype, device=None):
        return load_into(self.GPT(**cfg), w, dtype, device)


_REF = None


def reference_side() -> ReferenceSide:
    global _REF
    if _REF is None:
        _REF = ReferenceSide()
    return _REF


def cpu_decoder(cfg: dict, w: dict, dtype, top_p, temperature):
    """decode(prompt, num_samples, max_tokens, force_schedule=None) -> tokens generated, on the host cores, by the
    reference's Engine.generate_batch (kind "reference") or by the oracle port (kind "port")."""
    ref = reference_side()
    if ref.available:
        model = ref.model(cfg, w, dtype)
        inner = ref.TemperatureSampler(temperature)
        sampler = inner if top_p is None else ref.NucleusSampler(top_p, inner)

        def decode(prompt, num_samples, max_tokens, force_schedule=None) -> int:
            with torch.inference_mode():
                res, _ = ref.Engine(model).generate_batch(prompt, num_samples=num_samples, max_tokens=max_tokens, sampler=sampler,
                                                          force_schedule=force_schedule)
            return sum(len(r) - len(prompt) for r in res)

        return decode, "reference"
    from oracle import ref_decode, ref_math  # CPU legs only

    shape = ref_math.Shape(**cfg)
    wd = {k: v.to(dtype) for k, v in w.items()}

    def decode(prompt, num_samples, max_tokens, force_schedule=None) -> int:
        toks, _, _ = ref_decode.mc_decode(shape, wd, prompt, num_samples=num_samples, max_tokens=max_tokens,
                                          temperature=temperature, top_p=top_p, seed=42, force_schedule=force_schedule)
        return toks.numel()

    return decode, "port"


def cpu_sample_text() -> str:
    return (
        f"config 4 model and 1024-token prompt, {CPU_SAMPLE['series']} series x {CPU_SAMPLE['trajectories']} trajectories x "
        f"{CPU_SAMPLE['steps']} decode steps (prefill included), replicated dense KV cache as in the reference"
    )


def sample_config() -> dict:
    """What one step of the CPU arm actually runs: the config-4 model and prompt, a bounded number of trajectories and steps."""
    return {
        "workload": "BASELINE config 4, bounded sample for the host cores: one series, 64 of its 4096 trajectories, "
                    "32 of its 256 decode steps, 1024-token prefill included in every step",
        **CFG4, "prompt_tokens": PROMPT_TOKENS, "horizon": CPU_SAMPLE["steps"], "trajectories_per_series": CPU_SAMPLE["trajectories"],
        "series_per_step": CPU_SAMPLE["series"], "sampler": f"nucleus p={TOP_P}, temperature {TEMPERATURE}",
        "sample_of": "BASELINE config 4: large Monte-Carlo decode sharded by trajectory (4096 trajectories x 256 steps per series)",
        "device": "cpu",
    }


def run_reference(args) -> None:
    """The reference arm: the reference's own code path on the host cores (rank 0 only; other ranks do nothing)."""
    if int(os.environ.get("RANK", "0")) != 0:
        return
    cores = host_threads()
    decode, kind = cpu_decoder(CFG4, cfg4_weights(torch.bfloat16), torch.bfloat16, TOP_P, TEMPERATURE)
    prompt = synthetic_prompts(1, CFG4["vocab_size"])[0]
    for _ in range(args.warmup):
        decode(prompt, CPU_SAMPLE["trajectories"], CPU_SAMPLE["steps"])
    t0 = time.perf_counter()
    n = 0
    for _ in range(args.steps):
        n += decode(prompt, CPU_SAMPLE["trajectories"], CPU_SAMPLE["steps"])
    dt = time.perf_counter() - t0
    v = n / dt
    emit({
        "impl": "reference", "metric": "mc_decode_tokens_per_s", "value": v, "unit": "tokens/s", "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": 1e3 * dt / args.steps, "higher_is_better": True,
        "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": sample_config(),
        "cpu_baseline": {"value": v, "unit": "tokens/s", "cores": cores, "kind": kind, "sample": cpu_sample_text()},
        "e2e": {"value": v, "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "native_library_loaded": "diff_gpt_b200" in sys.modules,
    })


def workload_config(n_gpus: int) -> dict:
    return {
        "workload": "BASELINE config 4: large Monte-Carlo decode sharded by trajectory",
        **CFG4, "prompt_tokens": PROMPT_TOKENS, "horizon": HORIZON, "trajectories_per_series": TRAJECTORIES,
        "series_per_step": n_gpus, "trajectories_per_rank_per_series": TRAJECTORIES // n_gpus,
        "sampler": f"nucleus p={TOP_P}, temperature {TEMPERATURE}", "parallelism": f"trajectory-sharded x{n_gpus}, weight replicas",
        "l2": "inputs (38.7 GB KV pool per rank) are larger than L2; no flush",
    }


# ---------------------------------------------------------------------------------------
# our arm
# ---------------------------------------------------------------------------------------
def run_ours(args) -> None:
    import torch.distributed as dist

    from diff_gpt_b200 import GPT, Engine, NucleusSampler, TemperatureSampler, _lib
    from diff_gpt_b200.dist import gather_trajectories
    from diff_gpt_b200.model.engine import DecodeRun

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    assert world == args.gpus, f"--gpus {args.gpus} but WORLD_SIZE={world}: launch with torch.distributed.run for N > 1"
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        import datetime

        # a step takes seconds: a collective that has not completed after three minutes never will
        dist.init_process_group("nccl", device_id=dev, timeout=datetime.timedelta(minutes=3))
    assert TRAJECTORIES % world == 0
    n_local = TRAJECTORIES // world
    series_per_step = world

    w = cfg4_weights(torch.bfloat16)
    model = GPT(**CFG4).eval()
    sd = dict(w)
    sd["lm_head.weight"] = sd["token_embedding_table.weight"]
    model.load_state_dict(sd)
    model = model.to(torch.bfloat16).to(dev)
    prompts = synthetic_prompts(N_SERIES, CFG4["vocab_size"])
    prompts_dev = torch.tensor(prompts, dtype=torch.int32, device=dev)
    sampler = NucleusSampler(TOP_P, TemperatureSampler(TEMPERATURE))
    engine = Engine(model)
    tokens_per_step = series_per_step * TRAJECTORIES * HORIZON

    def series_of(step_idx: int) -> list[int]:
        return [(step_idx * series_per_step + j) % N_SERIES for j in range(series_per_step)]

    # The 38.7 GB page pool, the forward plans and the captured decode-step graph depend only on the shape
    # of a step: they are built by the first step and reused by the following ones (what a server that
    # decodes one batch after another keeps alive between requests).
    kv_pool = None
    runs: dict[tuple, DecodeRun] = {}

    def device_step(step_idx: int, use_graph: bool = not args.no_graph, gather: bool = True, collective: bool = True):
        """`collective` False: a step that one rank runs alone (the instrumented pass) - it prefills every prompt itself."""
        nonlocal kv_pool
        ids = series_of(step_idx)
        batch = prompts_dev[torch.tensor(ids, device=dev)]
        run = runs.get((use_graph, collective))
        if run is None:
            run = runs[(use_graph, collective)] = DecodeRun(
                model, batch, n_local, HORIZON, sampler, 42, None, traj_offset=rank * n_local, series_offset=ids[0],
                use_graph=use_graph, kv_pool=kv_pool, overlap_prefix=not args.no_overlap,
                prefill_group=dist.group.WORLD if (world > 1 and collective) else None,  # one rank prefills a prompt, K/V exchanged
            )
            kv_pool = run.cache.pool
        else:
            run.load(batch, None, traj_offset=rank * n_local, series_offset=ids[0])
        run.start()
        run.advance(HORIZON)
        toks = run.history.view(series_per_step, n_local, HORIZON)
        return (gather_trajectories(toks, TRAJECTORIES) if gather else toks), run

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize(dev)

    for i in range(args.warmup):
        device_step(i)
    barrier()
    clocks = ClockSampler(local)
    _lib.stats.launches = 0
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    statuses = []
    for i in range(args.steps):
        out, run = device_step(args.warmup + i)
        statuses.append(run.plan.status.clone())  # device-side status words, read after the timed region
    e1.record()
    barrier()
    launches = _lib.stats.launches
    ms = e0.elapsed_time(e1)
    clock_info = clocks.stop()
    status_ok = all(int(t.item()) == 0 for t in statuses)
    assert status_ok, "a kernel reported a device-side failure (slot out of range or a bounded wait ran out)"
    if world > 1:
        t = torch.tensor([ms], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms = float(t.item())
    value = args.steps * tokens_per_step / (ms / 1e3)
    assert out.shape == (series_per_step, TRAJECTORIES, HORIZON) and int(out.min()) >= 0 and int(out.max()) < CFG4["vocab_size"]

    # ---- world-size invariance: every N decodes series 0 .. N-1 once more, untimed; the gathered tokens of series 0
    # (all 4096 trajectories x 256 steps) must be the same bytes whatever N is, so their digest is printed ----
    import hashlib

    inv_out, _ = device_step(0)
    invariance = {"series": 0, "shape": list(inv_out[0].shape),
                  "tokens_sha256": hashlib.sha256(inv_out[0].cpu().numpy().tobytes()).hexdigest()}

    # ---- end to end: host prompts in, host tokens out, through the public engine call ----
    # The engine keeps its decode state between calls of one shape, so one untimed call comes first (as the
    # device-timed loop has its warm-up steps); every timed call still uploads its prompts from the host,
    # prefills them, decodes, gathers and copies the tokens back to pinned host memory.
    e2e_steps = 0 if args.no_e2e else args.steps
    pinned = torch.empty((series_per_step, TRAJECTORIES, HORIZON), dtype=torch.int32).pin_memory()

    def e2e_step(i: int) -> None:
        ids = series_of(i)
        toks, _ = engine.generate_many(
            [prompts[s] for s in ids], n_local, HORIZON, sampler, seed=42, traj_offset=rank * n_local,
            series_offset=ids[0], overlap_prefix=not args.no_overlap, prefill_group=dist.group.WORLD if world > 1 else None,
        )
        full = gather_trajectories(toks, TRAJECTORIES)
        pinned.copy_(full, non_blocking=False)

    if e2e_steps:
        e2e_step(0)
    barrier()
    t0 = time.perf_counter()
    for i in range(e2e_steps):
        e2e_step(1 + i)
    barrier()
    e2e_s = time.perf_counter() - t0
    if world > 1:
        t = torch.tensor([e2e_s], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        e2e_s = float(t.item())
    e2e = None if e2e_steps == 0 else {
        "value": e2e_steps * tokens_per_step / e2e_s, "unit": "tokens/s",
        "h2d_bytes_per_step": series_per_step * PROMPT_TOKENS * 4,
        "d2h_bytes_per_step": series_per_step * TRAJECTORIES * HORIZON * 4,
        "steps": e2e_steps, "api": "Engine.generate_many(host prompts) -> pinned host int32 tokens",
    }

    # ---- the same through the reference's own call: DiffGPT.predict_samples, values in, values out ----
    # One series of 4096 trajectories per step (the tokens of a 1-GPU step above; measured on one GPU only): a
    # float64 frame goes in from the host, is tokenised on the device, decoded, turned back into values and
    # comes back as a float64 host array.
    e2e_api = None
    if e2e is not None and world == 1:
        try:
            import pandas as pd

            from diff_gpt_b200.diff_gpt import DiffGPT
            from diff_gpt_b200.encoder_decoder import get_domain_of_definition

            engine.release()
            series = synthetic_series(N_SERIES)
            doms = [get_domain_of_definition(x, 1, use_decimal=False) for x in series]
            frames = [pd.DataFrame(x, columns=["y"]) for x in series]
            dg = DiffGPT(model=model, order_of_derivative=1, domain_of_definition=doms[0], use_decimal=False)

            def api_step(i: int) -> np.ndarray:
                sidx = (i * world + rank) % N_SERIES
                dg.domain_of_definition = doms[sidx]
                return dg.predict_samples(frames[sidx], max_new_points=HORIZON, num_samples=TRAJECTORIES, sampler=sampler)

            fut = api_step(0)
            assert fut.shape == (TRAJECTORIES, HORIZON, 1) and np.isfinite(fut).all()
            barrier()
            t0 = time.perf_counter()
            for i in range(e2e_steps):
                api_step(1 + i)
            barrier()
            api_s = time.perf_counter() - t0
            e2e_api = {
                "value": e2e_steps * world * TRAJECTORIES * HORIZON / api_s, "unit": "tokens/s",
                "h2d_bytes_per_step": world * (PROMPT_TOKENS + 1) * 8, "d2h_bytes_per_step": world * TRAJECTORIES * HORIZON * 8,
                "api": "DiffGPT.predict_samples(host float64 frame) -> host float64 [4096, 256, 1], one series per step",
            }
            dg._get_engine().release()
            del dg
        except Exception as exc:  # the headline figures above do not depend on this leg
            e2e_api = {"error": f"{type(exc).__name__}: {exc}"[:300]}

    # ---- per-kernel device time: one more step, launched eagerly with events around every call ----
    roof, kernels = None, None
    if rank == 0 and not args.no_kernel_pass:
        timer = _lib.KernelTimer()
        with _lib.timed(timer):
            _, run = device_step(args.warmup + args.steps, use_graph=False, gather=False, collective=False)  # rank 0 alone
        torch.cuda.synchronize(dev)
        del run
        kernels = {k: {kk: round(vv, 4) if isinstance(vv, float) else vv for kk, vv in v.items()} for k, v in timer.summary().items()}
        roof = roofline(kernels, n_local * series_per_step, series_per_step)
    if world > 1:
        barrier()

    ref_cuda = None
    if rank == 0 and world == 1 and not args.no_reference_cuda:
        engine.release()
        runs.clear()
        kv_pool = None
        torch.cuda.empty_cache()
        ref_cuda = reference_torch_cuda(model, w, prompts[0], dev)

    prefill = None if args.no_prefill else prefill_attention(world, rank, dev)
    if world > 1:
        barrier()

    cpu = None
    if rank == 0 and world == 1 and not args.no_cpu:
        cores = host_threads()
        decode, kind = cpu_decoder(CFG4, w, torch.bfloat16, TOP_P, TEMPERATURE)
        decode(prompts[0], CPU_SAMPLE["trajectories"], 2)  # warm
        t0 = time.perf_counter()
        n = decode(prompts[0], CPU_SAMPLE["trajectories"], CPU_SAMPLE["steps"])
        dt = time.perf_counter() - t0
        cpu = {"value": n / dt, "unit": "tokens/s", "cores": cores, "kind": kind, "sample": cpu_sample_text()}

    others = None
    if rank == 0 and world == 1 and not args.no_other_configs:
        others = other_configs(dev, cpu=not args.no_cpu)

    if rank == 0:
        pk = peaks()
        bytes_per_token = 4.82e6  # unique HBM bytes per generated token at this config (weights, shared prompt, own K/V)
        line = {
            "metric": "mc_decode_tokens_per_s", "value": value, "unit": "tokens/s", "n_gpus": world, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": ms / args.steps, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "bf16", "data": "synthetic", "config": workload_config(world),
            "clocks": clock_info, "e2e": e2e, "e2e_predict_samples": e2e_api, "gpu_launches": launches, "roofline": roof,
            "cpu_baseline": cpu, "invariance": invariance, "reference_torch_cuda": ref_cuda, "other_configs": others,
            "decode_hbm": {
                "algorithmic_bytes_per_token": bytes_per_token,
                "achieved_gbs_per_gpu": value / world * bytes_per_token / 1e9,
                "frac_of_peak": value / world * bytes_per_token / 1e9 / pk["hbm_gbs"], "peak_source": pk["source"],
            },
            "prefill_attention": prefill, "kernels": kernels, "status_ok": status_ok,
        }
        emit(line)
    if world > 1:
        dist.destroy_process_group()


def _wall(fn, dev, repeat: int = 1) -> float:
    """Seconds per call of fn(), host clock between two device synchronisations."""
    torch.cuda.synchronize(dev)
    t0 = time.perf_counter()
    for _ in range(repeat):
        fn()
    torch.cuda.synchronize(dev)
    return (time.perf_counter() - t0) / repeat


def reference_torch_cuda(model, w: dict, prompt: list[int], dev) -> dict:
    """The reference's own decode (its Engine, KVCache, samplers and GPT, unmodified, torch kernels) on this GPU in
    bf16, next to this library through the same call, `Engine.generate_batch(list prompt) -> python lists`, at a
    trajectory count whose replicated cache fits the reference (it copies the prompt K/V into every row)."""
    ref = reference_side()
    if not ref.available:
        return {"unavailable": "the reference is not installed under baseline/_ref"}
    from diff_gpt_b200 import Engine, NucleusSampler, TemperatureSampler

    n, horizon = 256, HORIZON
    out = {"trajectories": n, "horizon": horizon, "prompt_tokens": len(prompt), "unit": "tokens/s",
           "api": "Engine.generate_batch(python list prompt) -> python lists of tokens and masks"}
    try:
        ref_model = ref.model(CFG4, w, torch.bfloat16, dev)
        ref_sampler = ref.NucleusSampler(TOP_P, ref.TemperatureSampler(TEMPERATURE))
        with torch.inference_mode():
            ref.Engine(ref_model).generate_batch(prompt, num_samples=8, max_tokens=4, sampler=ref_sampler)
            t_ref = _wall(lambda: ref.Engine(ref_model).generate_batch(prompt, num_samples=n, max_tokens=horizon, sampler=ref_sampler), dev)
        del ref_model
        torch.cuda.empty_cache()
        sampler = NucleusSampler(TOP_P, TemperatureSampler(TEMPERATURE))
        eng = Engine(model)
        eng.generate_batch(prompt, num_samples=n, max_tokens=horizon, sampler=sampler)
        t_ours = _wall(lambda: eng.generate_batch(prompt, num_samples=n, max_tokens=horizon, sampler=sampler), dev, repeat=3)
        eng.release()
        out.update({"reference_value": n * horizon / t_ref, "reference_s": t_ref, "ours_value": n * horizon / t_ours,
                    "ours_s": t_ours, "ours_over_reference": t_ref / t_ours})
    except Exception as exc:  # noqa: BLE001 - the headline figures do not depend on this leg
        out["error"] = f"{type(exc).__name__}: {exc}"[:300]
    return out


def other_configs(dev, cpu: bool = True) -> dict:
    """One timed line each for BASELINE configs 1, 2 and 3 on one GPU, with a bounded run of the same call on the host cores."""
    out = {}
    for name, fn in (("config1", _config1), ("config2", _config2), ("config3", _config3)):
        try:
            out[name] = fn(dev, cpu)
        except Exception as exc:  # noqa: BLE001 - these lines are additions; the headline does not depend on them
            out[name] = {"error": f"{type(exc).__name__}: {exc}"[:300]}
        torch.cuda.empty_cache()
    return out


def _config1(dev, cpu: bool) -> dict:
    """Config 1: V256 C64 H4 L2 block 138, fp32, weights N(0, 0.02) seed 0; Gaussian random walk (seed 1, 96 points, the
    last 90 as context so that 89 + 48 positions fit the block), order 1; predict_samples(100 trajectories, 48 points)."""
    import pandas as pd

    from diff_gpt_b200 import GPT, TemperatureSampler
    from diff_gpt_b200.diff_gpt import DiffGPT

    cfg = dict(vocab_size=256, n_embd=64, n_head=4, n_layer=2, block_size=138)
    w = seeded_weights(cfg, 0, torch.float32)
    walk = np.cumsum(np.random.default_rng(1).normal(0.0, 1.0, 96))
    dom = host_codec().get_domain_of_definition(walk.reshape(-1, 1), 1, use_decimal=False)
    df = pd.DataFrame(walk[-90:].reshape(-1, 1), columns=["y"])
    n, h = 100, 48
    dg = DiffGPT(model=load_into(GPT(**cfg), w, torch.float32, dev), order_of_derivative=1, domain_of_definition=dom, use_decimal=False)
    fut = dg.predict_samples(df, max_new_points=h, num_samples=n, sampler=TemperatureSampler(1.0))
    assert fut.shape == (n, h, 1) and np.isfinite(fut).all()
    t = _wall(lambda: dg.predict_samples(df, max_new_points=h, num_samples=n, sampler=TemperatureSampler(1.0)), dev, repeat=10)
    line = {"workload": "BASELINE config 1: DiffGPT.predict_samples, 100 trajectories x 48 points, fp32, 89-token prompt",
            "value": n * h / t, "unit": "tokens/s", "ms_per_call": 1e3 * t, "us_per_decode_step": 1e6 * t / h, "dtype": "f32",
            "bound": "launch latency (0.43 MB of weights, 137 cached positions): one graph replay per step",
            "api": "DiffGPT.predict_samples(host frame) -> host float64 [100, 48, 1]"}
    ref = reference_side()
    if cpu and ref.available:
        rdg = ref.DiffGPT(model=ref.model(cfg, w, torch.float32), order_of_derivative=1, domain_of_definition=dom, use_decimal=False)
        rs = ref.TemperatureSampler(1.0)
        rdg.predict_samples(df, max_new_points=h, num_samples=n, sampler=rs)
        t0 = time.perf_counter()
        for _ in range(3):
            rdg.predict_samples(df, max_new_points=h, num_samples=n, sampler=rs)
        tc = (time.perf_counter() - t0) / 3
        line["cpu"] = {"value": n * h / tc, "unit": "tokens/s", "kind": "reference", "cores": torch.get_num_threads(), "sample": "the same call, full size"}
    return line


def _config2(dev, cpu: bool) -> dict:
    """Config 2: V512 C256 H8 (head_dim 32) L4 block 512, bf16, weights N(0, 0.02) seed 2; one causal forward of
    256 sequences x 512 uniform-random tokens (seed 2) with the logit soft-cap."""
    from diff_gpt_b200 import GPT, _lib

    cfg = dict(vocab_size=512, n_embd=256, n_head=8, n_layer=4, block_size=512)
    w = seeded_weights(cfg, 2, torch.bfloat16)
    B, T, C, L, V = 256, 512, 256, 4, 512
    idx = torch.randint(0, V, (B, T), generator=torch.Generator().manual_seed(2)).to(dev)
    model = load_into(GPT(**cfg), w, torch.bfloat16, dev)
    for _ in range(3):
        logits = model(idx)[0]
    assert logits.shape == (B, T, V)
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    torch.cuda.synchronize(dev)
    a.record()
    for _ in range(5):
        model(idx)
    b.record()
    torch.cuda.synchronize(dev)
    ms = a.elapsed_time(b) / 5
    timer = _lib.KernelTimer()
    with _lib.timed(timer):
        model(idx)
    torch.cuda.synchronize(dev)
    attn_ms = timer.summary()["dgpt_fmha_prefill"]["total_ms"]
    attn_flops = 2.0 * B * T * T * C * L  # causal QK^T and PV over all layers
    gemm_flops = 2.0 * B * T * (11 * C * C * L + C * V)
    pk = peaks()
    line = {"workload": "BASELINE config 2: batched causal forward, 256 x 512 tokens, bf16, head_dim 32", "value": ms, "unit": "ms per forward",
            "tokens_per_s": B * T / ms * 1e3, "forward_tflops": (attn_flops + gemm_flops) / ms / 1e9,
            "attention_ms": attn_ms, "attention_tflops": attn_flops / attn_ms / 1e9,
            "attention_frac_of_bf16_peak": attn_flops / attn_ms / 1e9 / pk["bf16_tflops_sustained"], "peak": pk["bf16_tflops_sustained"],
            "peak_source": pk["source"], "dtype": "bf16", "api": "GPT.forward(idx) -> logits [256, 512, 512]"}
    del model, logits
    ref = reference_side()
    if cpu and ref.available:
        rm = ref.model(cfg, w, torch.bfloat16)
        small = idx[:8].cpu()
        with torch.inference_mode():
            rm(small)
            t0 = time.perf_counter()
            rm(small)
            tc = time.perf_counter() - t0
        line["cpu"] = {"value": 1e3 * tc * (B / 8), "unit": "ms per forward", "kind": "reference", "cores": torch.get_num_threads(),
                       "sample": f"8 of the 256 sequences ({1e3 * tc:.0f} ms), scaled by 32"}
    return line


def cfg3_series(n_series: int, rows: int = 608) -> list[np.ndarray]:
    """Config 3's frames: 7 channels, sum of 3 sinusoids (periods 12..168, amplitudes U(0.5, 2)) + AR(1) noise (phi 0.8, sd 0.1), seed 3."""
    rng = np.random.default_rng(3)
    out = []
    for _ in range(n_series):
        t = np.arange(rows)[:, None]
        periods = rng.integers(12, 169, size=(3, 7))
        amps = rng.uniform(0.5, 2.0, size=(3, 7))
        x = sum(amps[i] * np.sin(2 * np.pi * t / periods[i]) for i in range(3))
        e = rng.normal(0, 0.1, size=(rows, 7))
        noise = np.zeros((rows, 7))
        for i in range(1, rows):
            noise[i] = 0.8 * noise[i - 1] + e[i]
        out.append((x + noise).astype(np.float64))
    return out


def _config3(dev, cpu: bool) -> dict:
    """Config 3: V1024 C512 H8 (head_dim 64) L6 block 4096, bf16, weights N(0, 0.02) seed 3; 64 series of 7 channels with
    per-column orders [0,1,1,2,2,1,0], 512 context rows (3570 tokens) + 96 rows (672 steps), channels 5 and 6 forced
    from the known future, argmax elsewhere; one trajectory per series, all 64 series in one decode."""
    from diff_gpt_b200 import GPT, Engine, TemperatureSampler

    cfg = dict(vocab_size=1024, n_embd=512, n_head=8, n_layer=6, block_size=4096)
    w = seeded_weights(cfg, 3, torch.bfloat16)
    orders = np.array([0, 1, 1, 2, 2, 1, 0])
    codec = host_codec()
    S, F, P, G = 64, 7, 3570, 672
    prompts, scheds = [], []
    for x in cfg3_series(S):
        dom = codec.get_domain_of_definition(x, orders, use_decimal=False)
        _, _, tok = codec.encode(inp=x, vocab_size=cfg["vocab_size"], domain_of_definition=dom, order_of_derivative=orders, use_decimal=False)
        flat = tok.reshape(-1).astype(np.int64).tolist()
        assert len(flat) == P + G
        prompts.append(flat[:P])
        scheds.append([flat[P + p] if (p % F) >= 5 else None for p in range(G)])
    eng = Engine(load_into(GPT(**cfg), w, torch.bfloat16, dev))
    sampler = TemperatureSampler(0.0)
    toks, masks = eng.generate_many(prompts, 1, G, sampler, force_schedules=scheds)
    assert toks.shape == (S, 1, G) and int(masks.sum()) == S * G * 5 // 7
    t = _wall(lambda: eng.generate_many(prompts, 1, G, sampler, force_schedules=scheds), dev, repeat=2)
    C, L = cfg["n_embd"], cfg["n_layer"]
    params = L * (11 * C * C + 2 * C) + cfg["vocab_size"] * C
    # every decode step reads each series' whole cache (no sharing across series): 2 (K, V) * L * C * 2 B per cached token
    kv_bytes = sum(S * 2 * L * C * 2 * (P + g) for g in range(1, G))
    algo = kv_bytes + (G - 1) * 2 * params
    pk = peaks()
    line = {"workload": "BASELINE config 3: 64 series x 1 trajectory, 3570-token prompts, 672 steps, channels 5-6 teacher-forced, bf16",
            "value": S * G / t, "unit": "tokens/s", "ms_per_call": 1e3 * t, "dtype": "bf16",
            "hbm": {"algorithmic_bytes_per_call": algo, "achieved_gbs": algo / t / 1e9, "frac_of_peak": algo / t / 1e9 / pk["hbm_gbs"],
                    "peak": pk["hbm_gbs"], "peak_source": pk["source"], "note": "prefill of the 64 prompts is inside the timed call; its bytes and FLOPs are not counted"},
            "api": "Engine.generate_many(64 host prompts, force_schedules) -> device tokens [64, 1, 672]"}
    eng.release()
    del eng
    if cpu:
        steps = 7
        decode, kind = cpu_decoder(cfg, w, torch.bfloat16, None, 0.0)
        t0 = time.perf_counter()
        n = decode(prompts[0], 1, steps, scheds[0][:steps])
        tc = time.perf_counter() - t0
        line["cpu"] = {"value": n / tc, "unit": "tokens/s", "kind": kind, "cores": torch.get_num_threads(),
                       "sample": f"one of the 64 series, prefill of 3570 tokens + {steps} of the 672 steps ({tc:.1f} s)"}
    return line


def prefill_attention(world: int, rank: int, dev, lengths=(4096, 8192, 16384, 32768)) -> list:
    """BASELINE config 5: one attention layer (RoPE + QK-norm + causal attention + output projection) on
    Q, K, V ~ N(0, 1), 16 heads of 128, batch 8 split over the ranks; TFLOP/s counts 2 B H S^2 D for the attention kernel."""
    import torch.distributed as dist

    from diff_gpt_b200 import ops

    B, H, D = max(1, 8 // world), 16, 128
    C = H * D
    pk = peaks()
    g = torch.Generator(device=dev).manual_seed(5 + rank)
    wp = (torch.randn((C, C), device=dev, generator=g) * 0.02).to(torch.bfloat16)
    out = []
    for S in lengths:
        j = torch.arange(0, D, 2, dtype=torch.float32, device=dev) / D
        ang = torch.outer(torch.arange(S, dtype=torch.float32, device=dev), 1.0 / (10000.0 ** j))
        table = torch.stack([ang.cos(), ang.sin()], dim=-1).to(torch.bfloat16).contiguous()
        qkv = torch.randn((B * S, 3 * C), device=dev, generator=g, dtype=torch.float32).to(torch.bfloat16)
        cache = torch.empty((B, 2, H, S, D), device=dev, dtype=torch.bfloat16)
        lay = ops.kv_layout(cache[0, 0], cache[0, 1], 2 * H * S * D, S * D, S)
        q_rot = torch.empty((B * S, C), device=dev, dtype=torch.bfloat16)
        y = torch.empty_like(q_rot)
        proj = torch.empty_like(q_rot)
        zero = torch.zeros(B, dtype=torch.int32, device=dev)
        status = torch.zeros(1, dtype=torch.int32, device=dev)
        ev = [torch.cuda.Event(enable_timing=True) for _ in range(4)]

        def layer(timed: bool):
            if timed:
                ev[0].record()
            ops.rope_qknorm_kvappend(qkv[:, :C], qkv[:, C : 2 * C], qkv[:, 2 * C :], q_rot, table, lay, zero, zero, None,
                                     B, S, H, D, status)
            if timed:
                ev[1].record()
            ops.fmha_prefill(q_rot, lay, y, B=B, H=H, Tq=S, D=D, q_batch_stride=S * C, q_row_stride=C,
                             o_batch_stride=S * C, o_row_stride=C, kv_len_all=S, causal=True,
                             impl=2, status=status)  # the library's own choice from 1024 keys on, made explicit so that it cannot fall back
            if timed:
                ev[2].record()
            torch.mm(y, wp.t(), out=proj)
            if timed:
                ev[3].record()

        layer(False)
        layer(False)
        torch.cuda.synchronize(dev)
        t_attn, t_layer = [], []
        for _ in range(3):
            layer(True)
            torch.cuda.synchronize(dev)
            t_attn.append(ev[1].elapsed_time(ev[2]))
            t_layer.append(ev[0].elapsed_time(ev[3]))
        assert int(status.item()) == 0, "the attention kernel reported a device-side failure"
        ta, tl = min(t_attn), min(t_layer)
        if world > 1:
            t = torch.tensor([ta, tl], device=dev)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            ta, tl = float(t[0]), float(t[1])
        flops = 2.0 * B * world * H * S * S * D
        sdpa = sdpa_reference(q_rot.view(B, S, H, D).transpose(1, 2), cache[:, 0], cache[:, 1], y.view(B, S, H, D), flops / world) if rank == 0 else None
        out.append({"S": S, "batch": B * world, "attn_ms": ta, "layer_ms": tl, "attn_tflops": flops / ta / 1e9,
                    "sdpa": sdpa,
                    "attn_tflops_per_gpu": flops / ta / 1e9 / world,
                    "frac_of_bf16_peak": flops / ta / 1e9 / world / pk["bf16_tflops"], "peak": pk["bf16_tflops"],
                    "peak_source": pk["source"]})
        del qkv, cache, q_rot, y, proj
    return out


def sdpa_reference(q, k, v, ours, flops: float) -> dict:
    """`F.scaled_dot_product_attention(q, k, v, is_causal=True)` (the reference's call, mha.py:64) on the tensors the
    attention kernel just read - q after RoPE and QK-norm [B, H, S, D] strided, K and V as cached - with torch's own
    backend choice and with the cuDNN backend forced; TFLOP/s on this rank and the largest difference from `ours`."""
    import torch.nn.functional as F
    from torch.nn.attention import SDPBackend, sdpa_kernel

    out = {}
    for tag, backends in (("default", None), ("cudnn", [SDPBackend.CUDNN_ATTENTION])):
        try:
            def call():
                if backends is None:
                    return F.scaled_dot_product_attention(q, k, v, is_causal=True)
                with sdpa_kernel(backends):
                    return F.scaled_dot_product_attention(q, k, v, is_causal=True)

            o = call()
            call()
            torch.cuda.synchronize()
            ts = []
            for _ in range(3):
                a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                a.record()
                call()
                b.record()
                torch.cuda.synchronize()
                ts.append(a.elapsed_time(b))
            diff = (o.transpose(1, 2).float() - ours.float()).abs().max().item()
            out[tag] = {"ms": min(ts), "tflops": flops / min(ts) / 1e9, "max_abs_diff_from_ours": diff}
            del o
        except Exception as exc:  # noqa: BLE001 - a backend that refuses these strides is reported, not fatal
            out[tag] = {"error": f"{type(exc).__name__}: {exc}"[:200]}
    return out


def roofline(kernels: dict, rows: int, n_series: int) -> dict:
    """Roofline of the library kernel with the largest share of device time in the instrumented step."""
    pk = peaks()
    C, L, H = CFG4["n_embd"], CFG4["n_layer"], CFG4["n_head"]
    mine = {k: v for k, v in kernels.items() if k.startswith("dgpt_")}
    top = max(mine, key=lambda k: mine[k]["total_ms"])
    k = mine[top]
    total_s = k["total_ms"] / 1e3
    steps = HORIZON - 1  # decode forwards (the forward after the last token is skipped)
    if top in ("dgpt_decode_attn", "dgpt_decode_attn_partial"):
        # per launch (one layer, decode forward g = 1..255): every row reads its g own K and V vectors (C bf16 each), plus
        # q (bf16); the one-stream form also reads gate (bf16) and the prompt partial (fp32 o + lse) and writes y (bf16),
        # the two-stream form writes its own fp32 partial (o + lse) instead
        kv_bytes = sum(rows * 2 * C * 2 * g for g in range(1, steps + 1)) * L
        per_row = (3 * C * 2 + C * 4 + H * 4) if top == "dgpt_decode_attn" else (C * 2 + C * 4 + H * 4)
        io_bytes = steps * L * rows * per_row
        achieved = (kv_bytes + io_bytes) / total_s / 1e9
        # DRAM traffic per launch: the ncu capture of this kernel at decode step 128 (profiles/) read and wrote 1.002 x
        # its algorithmic bytes; the traffic is proportional to the keys read, so the ratio is applied to the mean launch
        out = {"kernel": top, "bound": "hbm", "achieved": achieved, "peak": pk["hbm_gbs"], "unit": "GB/s",
               "frac": achieved / pk["hbm_gbs"], "traffic": 1.002 * (kv_bytes + io_bytes) / k["launches"],
               "traffic_source": "ncu capture at decode step 128 scaled by keys read", "peak_source": pk["source"],
               "launches": k["launches"], "avg_launch_ms": k["avg_ms"], "algorithmic_bytes_per_launch": (kv_bytes + io_bytes) / k["launches"]}
        if top == "dgpt_decode_attn_partial":
            out["note"] = ("each launch shares the GPU with the prompt-phase tensor-core kernel running on a second stream, "
                           "so its duration is longer than alone (python bench.py --kernel-case decode_attn times it alone)")
        return out
    if top == "dgpt_fmha_prefill":
        # shared-prompt phase per launch: QK^T and PV over rows x 1024 prompt keys, all heads: 4 * rows * P * C flops
        decode_flops = steps * L * 4 * rows * PROMPT_TOKENS * C
        prefill_flops = L * 2 * n_series * PROMPT_TOKENS * PROMPT_TOKENS * C  # causal prompt prefill
        achieved = (decode_flops + prefill_flops) / total_s / 1e12
        return {"kernel": top, "bound": "tensor", "achieved": achieved, "peak": pk["bf16_tflops_sustained"], "unit": "TFLOP/s",
                "frac": achieved / pk["bf16_tflops_sustained"], "traffic": None, "peak_source": pk["source"],
                "launches": k["launches"], "avg_launch_ms": k["avg_ms"]}
    return {"kernel": top, "bound": "hbm", "achieved": None, "peak": pk["hbm_gbs"], "unit": "GB/s", "frac": None,
            "traffic": None, "launches": k["launches"], "avg_launch_ms": k["avg_ms"]}


def kernel_case(name: str, iters: int = 8) -> None:
    """One kernel alone on a case sized for an `ncu --set full` capture (a few launches, < 2 GB touched).

    decode_attn: config-4 shapes at decode step 128 — 4096 trajectories x 12 heads, head_dim 64, 128 own
                 tokens per trajectory in 64-token pages, prompt partial merged, gate applied.
    fmha:        config-5 shapes at S = 4096 — batch 8, 16 heads, head_dim 128, causal, dense K/V (two CTAs per SM).
    fmha_long:   the same at S = 8192 on the warp-specialised kernel.
    sample:      config-4 logits, 4096 rows x 4096 tokens, nucleus 0.9.
    depthmix:    config-4 rows, 8 candidates (mid-stack).
    fmha_prefix: shared-prompt phase of a config-4 decode step (4096 rows x 1024 prompt keys, 12 heads x 64).
    linear:      first feed-forward GEMM of a config-4 decode step with the SwiGLU epilogue.
    Prints one JSON line with the CUDA-event time per launch and the achieved rate.
    """
    from diff_gpt_b200 import ops

    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    g = torch.Generator(device=dev).manual_seed(0)
    pk = peaks()
    if name == "decode_attn":
        R, H, D, pt, own = TRAJECTORIES, CFG4["n_head"], 64, 64, 128
        C = H * D
        pages = own // pt
        pool = torch.randn((R * pages, 2, H, pt, D), device=dev, dtype=torch.bfloat16, generator=g)
        table = torch.arange(R * pages, dtype=torch.int32, device=dev).view(R, pages)
        lay = ops.kv_layout(pool[0, 0], pool[0, 1], 2 * H * pt * D, pt * D, pt, table, n_pages=R * pages)
        q = torch.randn((R, C), device=dev, dtype=torch.bfloat16, generator=g)
        gate = torch.randn((R, C), device=dev, dtype=torch.bfloat16, generator=g)
        y = torch.empty_like(q)
        po = torch.randn((R, H, D), device=dev, dtype=torch.float32, generator=g)
        pl = torch.randn((R, H), device=dev, dtype=torch.float32, generator=g)
        zero = torch.zeros(R, dtype=torch.int32, device=dev)
        n1 = torch.full((R,), own, dtype=torch.int32, device=dev)

        def launch():
            ops.decode_attn(q, lay, zero, zero, n1, None, y, H=H, D=D, gate=gate, prefix_o=po, prefix_lse=pl)

        work = R * (2 * C * 2 * own + 3 * C * 2 + C * 4 + H * 4)
        unit, peak = "GB/s", pk["hbm_gbs"]
    elif name in ("fmha", "fmha_long", "fmha_pair"):
        # config-5 shapes; "fmha" = S 4096 on the two-CTAs-per-SM kernel (the one used below 1024 keys and for the
        # shared-prompt phase), "fmha_long" = S 8192 on the warp-specialised one, "fmha_pair" = S 8192 on the kernel
        # with two query tiles per CTA
        B, H, S, D = 8, 16, (4096 if name == "fmha" else 8192), 128
        which = {"fmha": 3, "fmha_long": 2, "fmha_pair": 4}[name]
        q = torch.randn((B, S, H, D), device=dev, dtype=torch.bfloat16, generator=g)
        kv = torch.randn((B, 2, H, S, D), device=dev, dtype=torch.bfloat16, generator=g)
        lay = ops.kv_layout(kv[0, 0], kv[0, 1], 2 * H * S * D, S * D, S)
        o = torch.empty_like(q)
        st = torch.zeros(1, dtype=torch.int32, device=dev)

        def launch():
            ops.fmha_prefill(q, lay, o, B=B, H=H, Tq=S, D=D, q_batch_stride=S * H * D, q_row_stride=H * D,
                             o_batch_stride=S * H * D, o_row_stride=H * D, kv_len_all=S, causal=True, impl=which, status=st)

        work = 2 * B * H * S * S * D
        unit, peak = "TFLOP/s", pk["bf16_tflops"]
    elif name == "fmha_prefix":
        # shared-prompt phase of one config-4 decode step: 4096 trajectories of one series against the
        # 1024 prompt keys, 12 heads x 64, not causal, fp32 output + log-sum-exp for the later merge
        R, H, D, P, pt = TRAJECTORIES, CFG4["n_head"], 64, PROMPT_TOKENS, 64
        C = H * D
        pages = P // pt
        pool = torch.randn((pages, 2, H, pt, D), device=dev, dtype=torch.bfloat16, generator=g)
        table = torch.arange(pages, dtype=torch.int32, device=dev).view(1, pages)
        lay = ops.kv_layout(pool[0, 0], pool[0, 1], 2 * H * pt * D, pt * D, pt, table, n_pages=pages)
        q = torch.randn((R, C), device=dev, dtype=torch.bfloat16, generator=g)
        o = torch.empty((R, H, D), device=dev, dtype=torch.float32)
        lse = torch.empty((R, H), device=dev, dtype=torch.float32)
        klen = torch.full((1,), P, dtype=torch.int32, device=dev)
        st = torch.zeros(1, dtype=torch.int32, device=dev)

        def launch():
            ops.fmha_prefill(q, lay, o, B=1, H=H, Tq=R, D=D, q_batch_stride=R * C, q_row_stride=C,
                             o_batch_stride=R * C, o_row_stride=C, kv_len=klen, causal=False, lse=lse, impl=3, status=st)

        work = 4 * R * P * C
        unit, peak = "TFLOP/s", pk["bf16_tflops"]
    elif name == "linear":
        # first feed-forward GEMM of a config-4 decode step with the SwiGLU epilogue: [4096, 768] x [3072, 768]^T -> [4096, 1536]
        M, K, N = TRAJECTORIES, CFG4["n_embd"], 4 * CFG4["n_embd"]
        a = torch.randn((M, K), device=dev, dtype=torch.bfloat16, generator=g)
        wgt = torch.randn((N, K), device=dev, dtype=torch.bfloat16, generator=g) * 0.05
        act = torch.empty((M, N // 2), device=dev, dtype=torch.bfloat16)
        st = torch.zeros(1, dtype=torch.int32, device=dev)

        def launch():
            ops.linear(a, wgt, act, swiglu=(1.702, 7.0), status=st)

        work = 2 * M * N * K
        unit, peak = "TFLOP/s", pk["bf16_tflops"]
    elif name == "sample":
        R, V = TRAJECTORIES, CFG4["vocab_size"]
        logits = (torch.randn((R, V), device=dev, generator=g) * 0.05).to(torch.bfloat16)  # near-flat, as at random init
        out = torch.empty(R, dtype=torch.int32, device=dev)

        def launch():
            ops.sample(logits, out, cap=15.0, temperature=TEMPERATURE, top_p=TOP_P, seed=42)

        work = R * V * 2
        unit, peak = "GB/s", pk["hbm_gbs"]
    elif name == "depthmix":
        # config-4 shapes in the middle of the stack: 4096 rows x 768 channels, 8 candidates.  Four sets of
        # candidates (201 MB) are rotated so that consecutive launches do not find their inputs in L2.
        R, C, n_c, sets = TRAJECTORIES, CFG4["n_embd"], 8, 4
        cands = [[torch.randn((R, C), device=dev, dtype=torch.bfloat16, generator=g) for _ in range(n_c)] for _ in range(sets)]
        wmix = torch.randn((C,), device=dev, dtype=torch.bfloat16, generator=g) * 0.1
        out = torch.empty((R, C), device=dev, dtype=torch.bfloat16)
        turn = [0]

        def launch():
            ops.depthmix(cands[turn[0] % sets], wmix, None, out)
            turn[0] += 1

        work = R * C * 2 * (n_c + 1)
        unit, peak = "GB/s", pk["hbm_gbs"]
    else:
        raise SystemExit(f"unknown kernel case {name}")
    for _ in range(3):
        launch()
    torch.cuda.synchronize()
    # The launches are replayed from a CUDA graph so that the time is the device's, not the host's
    # (a Python call costs more than some of these kernels run).
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        for _ in range(iters):
            launch()
    graph.replay()
    torch.cuda.synchronize()
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a.record()
    graph.replay()
    b.record()
    torch.cuda.synchronize()
    ms = a.elapsed_time(b) / iters
    rate = work / (ms / 1e3) / (1e9 if unit == "GB/s" else 1e12)
    print(json.dumps({"kernel_case": name, "ms_per_launch": ms, "achieved": rate, "unit": unit, "peak": peak,
                      "frac": rate / peak, "algorithmic_work_per_launch": work, "peak_source": pk["source"]}), flush=True)


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--kernel-case", default=None, choices=["decode_attn", "fmha", "fmha_long", "fmha_pair", "sample", "depthmix", "fmha_prefix", "linear"],
                    help="run one kernel alone on a small case (for ncu) and exit")
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=3)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--no-cpu", action="store_true", help="skip the CPU baseline leg")
    ap.add_argument("--no-kernel-pass", action="store_true", help="skip the per-kernel timing step")
    ap.add_argument("--no-e2e", action="store_true", help="skip the end-to-end leg")
    ap.add_argument("--no-prefill", action="store_true", help="skip the config-5 prefill-attention sweep")
    ap.add_argument("--no-other-configs", action="store_true", help="skip the lines for BASELINE configs 1, 2 and 3")
    ap.add_argument("--no-reference-cuda", action="store_true", help="skip the reference's own torch-CUDA decode leg")
    ap.add_argument("--no-overlap", action="store_true",
                    help="run the shared-prompt attention phase before the per-row phase instead of beside it")
    ap.add_argument("--no-graph", action="store_true", help="launch the decode steps eagerly (for profilers)")
    ap.add_argument("--small", action="store_true",
                    help="profiling case: 2048 trajectories x 64 steps (4.8 GB of KV), same model and prompt")
    args = ap.parse_args()
    if args.small:
        globals().update(TRAJECTORIES=2048, HORIZON=64)
    if args.kernel_case:
        kernel_case(args.kernel_case)
        return
    claim_stdout()
    if args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
