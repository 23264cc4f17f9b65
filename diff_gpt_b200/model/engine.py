"""Monte-Carlo decode engine: prefill once per series, share the prompt K/V, decode on device.

Public surface of the reference Engine (src/diff_gpt/model/engine.py:23-169):
`Engine(model)`, `generate(...)` yielding `(token_column, token_masks)` per
step, `generate_batch(...) -> (results, masks)`, the same assertions and the
same RoPE-ceiling clamp.  What differs is where the work happens:

  * the prompt is prefilled into shared pages; trajectories are not given copies
    (the reference replicates the cache, engine.py:92-99);
  * sampling, teacher forcing, the next embedding lookup and the position
    counter stay on the device; one decode step is a CUDA graph that is replayed,
    so there is no per-step host synchronisation (the reference reads the tokens
    back and re-uploads them every step, engine.py:121,150);
  * `generate_many` (additive API) decodes several series in one batch and can
    take a trajectory offset, which is what the multi-GPU sharding uses;
  * the page pool, the forward plans and the captured step graph are kept on the
    engine and reused by the next call of the same shape (`Engine.release()` frees them).

A sampler that is not one of the library's (any callable `f(logits, rng)`) is
honoured by running the same forward eagerly and handing it the device logits.
"""

from __future__ import annotations

from typing import Callable, Generator

import torch
import torch.distributed as dist

from .. import _lib, ops
from ..sampler.sampler import Sampler
from .gpt import GPT, BaseGPT, ForwardPlan, KvBinding, _pick_splits  # noqa: F401
from .kv_cache import KVCache, PagedKVCache

SHARED_PREFIX_MIN_ROWS = 16  # below this the prompt is read by the per-row kernel (split along keys)


def _effective_max_tokens(block_size: int, prompt_len: int, max_tokens: int | None) -> int:
    ceiling = max(0, block_size * 2 - prompt_len)  # RoPE table length (engine.py:55-64)
    return ceiling if max_tokens is None else min(max_tokens, ceiling)


class DecodeRun:
    """State of one batched Monte-Carlo decode: S series x N trajectories, G steps.

    Everything that depends only on the SHAPE of the job (page pool, tables, forward plans, the captured
    decode-step graph) is built once; `load` brings in a new set of prompts of the same lengths and rewinds,
    so a server decoding batch after batch of equally shaped requests pays for construction and graph
    capture once.  `key` identifies the shape; two jobs with equal keys can share a DecodeRun.
    """

    @staticmethod
    def key_for(model, prompt_lens, num_samples, max_tokens, sampler, seed, has_force, page_tokens, use_graph,
                fmha_impl, overlap_prefix, shared_prefix=None, fused_head=True, prefill_shared=False) -> tuple:
        spec = (1.0, 1.0) if sampler is None else (sampler.native_spec() if isinstance(sampler, Sampler) else None)
        emb = model.token_embedding_table.weight
        return (
            id(model), str(emb.device), emb.dtype, tuple(prompt_lens), num_samples, max_tokens, spec,
            None if spec is not None else id(sampler), seed, has_force, page_tokens, use_graph, fmha_impl,
            overlap_prefix, shared_prefix, fused_head, prefill_shared,
        )

    def __init__(
        self,
        model: GPT,
        prompts: list[list[int]],
        num_samples: int,
        max_tokens: int,
        sampler: Sampler | Callable | None,
        seed: int,
        force_schedules: list[list[int | None]] | None,
        traj_offset: int = 0,
        series_offset: int = 0,
        page_tokens: int = 64,
        use_graph: bool = True,
        fmha_impl: int = 0,
        kv_pool: torch.Tensor | None = None,
        overlap_prefix: bool = True,
        shared_prefix: bool | None = None,
        fused_head: bool = True,
        prefill_group=None,
    ) -> None:
        self.model = model
        emb = model.token_embedding_table.weight
        if not emb.is_cuda:
            raise RuntimeError("diff_gpt_b200.Engine runs on CUDA only; there is no CPU path")
        dev, dt = emb.device, emb.dtype
        self.dev = dev
        S, N, G = len(prompts), num_samples, max_tokens
        self.S, self.N, self.G, self.R = S, N, G, S * N
        H, L = model.n_head, model.n_layer
        D = model.n_embd // H
        self.cap = float(model.logit_softcap)
        self.seed = seed
        self.use_graph = use_graph

        spec = (1.0, 1.0) if sampler is None else (sampler.native_spec() if isinstance(sampler, Sampler) else None)
        self.native = spec is not None
        self.temperature, self.top_p = spec if spec is not None else (1.0, 1.0)
        self.sampler = sampler

        on_device = isinstance(prompts, torch.Tensor)  # [S, P] int32, already on the GPU
        lens = [int(prompts.shape[1])] * S if on_device else [len(p) for p in prompts]
        self.prompt_lens = lens
        self.key = self.key_for(
            model, lens, N, G, sampler, seed, force_schedules is not None, page_tokens, use_graph, fmha_impl,
            overlap_prefix, shared_prefix, fused_head, prefill_group is not None,
        )
        self.packed = model.packed_weights()  # the graph holds these tensors' addresses
        self.cache = PagedKVCache(L, H, D, S, N, max(lens), G, dt, dev, page_tokens=page_tokens, pool=kv_pool)
        self.prefix_lens = torch.tensor(lens, dtype=torch.int32, device=dev)
        row_len = self.prefix_lens.repeat_interleave(N)
        self.tokens = torch.zeros(self.R, dtype=torch.int32, device=dev)
        self.history = torch.zeros((self.R, max(G, 1)), dtype=torch.int32, device=dev)
        self.step = torch.zeros(1, dtype=torch.int32, device=dev)
        self.traj_ids = torch.zeros(self.R, dtype=torch.int64, device=dev)
        self.force = None
        self.force_host = None
        if force_schedules is not None:
            self.force = torch.zeros((S, G), dtype=torch.int32, device=dev)

        # ---- who prefills which prompt ----
        # Ranks that decode different trajectories of the SAME series (dist.decode_sharded) all need every prompt's
        # K/V.  With a process group each rank prefills a contiguous block of S / W series only and the ranks exchange
        # the prompt pages and the last-position logits with one all-gather each (NCCL; each rank's own memory only).
        self.prefill_group, self.prefill_world, self.prefill_rank = None, 1, 0
        if prefill_group is not None and dist.is_available() and dist.is_initialized():
            w = dist.get_world_size(prefill_group)
            if w > 1 and S % w == 0:
                self.prefill_group, self.prefill_world, self.prefill_rank = prefill_group, w, dist.get_rank(prefill_group)
        per_rank = S // self.prefill_world
        mine = range(self.prefill_rank * per_rank, (self.prefill_rank + 1) * per_rank)

        # ---- prefill plans, one per distinct prompt length; only the last position's logits are needed ----
        self.logits0 = torch.empty((S, model.vocab_size), dtype=dt, device=dev)
        groups: dict[int, list[int]] = {}
        for s, n in enumerate(lens):
            if s in mine:
                groups.setdefault(n, []).append(s)
        zero = torch.zeros(S, dtype=torch.int32, device=dev)
        self.prefills = []
        for P, members in groups.items():
            idx = torch.tensor(members, device=dev)
            table = self.cache.prefix_table[idx].contiguous()
            layouts = [self.cache._layout(l, table) for l in range(L)]
            bind = KvBinding(
                layouts=layouts, pos0=zero[: len(members)], slot0=zero[: len(members)], kv_len=P, q_offset=0,
                fmha_impl=fmha_impl,
            )
            plan = ForwardPlan(model, len(members), P, last_only=True)
            self.prefills.append((P, members, idx, bind, plan, table))

        # ---- decode plan ----
        # A shard of a larger job takes the path the whole job would take (the two paths round differently), so the
        # caller may decide; by default the prompt is shared from SHARED_PREFIX_MIN_ROWS trajectories per series on.
        shared = (N >= SHARED_PREFIX_MIN_ROWS) if shared_prefix is None else bool(shared_prefix)
        slot0 = torch.full((self.R,), self.cache.suffix_slot0, dtype=torch.int32, device=dev)
        self.bind = KvBinding(
            layouts=[self.cache.row_layout(l) for l in range(L)],
            pos0=row_len.contiguous(),
            slot0=slot0,
            step=self.step,
            decode=True,
            len0=row_len.contiguous(),
            start1=slot0,
            len1=torch.ones(self.R, dtype=torch.int32, device=dev),
            n_splits=1 if shared else _pick_splits(self.R * H, max(lens) + G),
            shared_layouts=[self.cache.prefix_layout(l) for l in range(L)] if shared else None,
            shared_len=self.prefix_lens if shared else None,
            rows_per_series=N,
            fmha_impl=fmha_impl,
            overlap_prefix=overlap_prefix and shared,
        )
        # The head of a decode step.  With one of the library's samplers and a bf16 model it is one call,
        # dgpt_lmhead_sample: without a top-p filter the logits are sampled inside the GEMM's epilogue and never
        # stored (`fused_head`); with one, or when a caller wants to see them, the GEMM writes them for the
        # sampling kernel.  Other samplers and fp32 models get the logits from the forward plan.
        C, V = model.n_embd, model.vocab_size
        self.lmhead = self.native and dt == torch.bfloat16 and C % 8 == 0 and V % 16 == 0
        nucleus = self.top_p < 1.0 and self.temperature > 0.0
        self.head_logits = None
        self.head_ws = None
        if self.lmhead:
            if nucleus or not fused_head:
                self.head_logits = torch.empty((self.R, V), dtype=dt, device=dev)
            else:
                self.head_ws = torch.empty(max(1, ops.lmhead_workspace_bytes(self.R) // 8), dtype=torch.int64, device=dev)
        self.plan = ForwardPlan(model, self.R, 1, want_logits=not self.lmhead)
        self.graph = None
        self.done = 0  # tokens produced so far per row
        self.rng = None
        self.load(prompts, force_schedules, traj_offset, series_offset)

    def reusable(self) -> bool:
        """False once the model's weights have been repacked (the captured graph points at the old ones)."""
        return self.model.packed_weights() is self.packed

    def load(self, prompts, force_schedules=None, traj_offset: int = 0, series_offset: int = 0) -> None:
        """Prefill a new set of prompts (same lengths as the first) and rewind to step 0."""
        S, N, G, dev = self.S, self.N, self.G, self.dev
        on_device = isinstance(prompts, torch.Tensor)
        lens = [int(prompts.shape[1])] * len(prompts) if on_device else [len(p) for p in prompts]
        assert lens == self.prompt_lens, "load() needs prompts of the lengths this run was built for"
        assert (force_schedules is not None) == (self.force is not None)
        ids = (torch.arange(S, dtype=torch.int64) + series_offset).repeat_interleave(N) * (1 << 32)
        ids += (torch.arange(N, dtype=torch.int64) + traj_offset).repeat(S)
        self.traj_ids.copy_(ids)
        if force_schedules is not None:
            f = torch.tensor(
                [[-1 if t is None else int(t) for t in sch[:G]] for sch in force_schedules], dtype=torch.int32
            )
            self.force_host = f
            self.force.copy_(f)
        self.step.zero_()
        self.plan.status.zero_()
        for P, members, idx, bind, plan, _table in self.prefills:
            if on_device:
                ids32 = prompts.reshape(-1) if len(members) == S else prompts[idx].reshape(-1)
            else:
                ids32 = torch.tensor([prompts[s] for s in members], dtype=torch.int32).reshape(-1).to(dev)
            out = plan.run(ids32, bind)
            if len(members) == S:
                self.logits0.copy_(out)
            else:
                self.logits0[idx] = out
        if self.prefill_group is not None:
            self._exchange_prompts()
        self.done = 0
        self.rng = None

    def _exchange_prompts(self) -> None:
        """Every rank has prefilled its block of series: all-gather the prompt pages (they are the first pages of the
        pool, series-major, so a block of series is one run of pages per layer) and the last-position logits."""
        W, r, S = self.prefill_world, self.prefill_rank, self.S
        n = (S // W) * self.cache.prefix_pages
        pool = self.cache.pool
        if getattr(self, "_stage", None) is None:
            self._stage = torch.empty((W, pool.shape[0], n) + tuple(pool.shape[2:]), dtype=pool.dtype, device=pool.device)
            self._stage_logits = torch.empty_like(self.logits0)
        local = pool[:, r * n : (r + 1) * n].contiguous()
        dist.all_gather_into_tensor(self._stage.view(-1), local.view(-1), group=self.prefill_group)
        for other in range(W):
            if other != r:
                pool[:, other * n : (other + 1) * n].copy_(self._stage[other])
        mine = self.logits0[r * (S // W) : (r + 1) * (S // W)].contiguous()
        dist.all_gather_into_tensor(self._stage_logits.view(-1), mine.view(-1), group=self.prefill_group)
        self.logits0.copy_(self._stage_logits)

    # -- sampling ---------------------------------------------------------------------
    def _sample_first(self) -> None:
        """Token 0 of every trajectory comes from its series' prefill logits (engine.py:89)."""
        N = self.N
        for s in range(self.S):
            sl = slice(s * N, (s + 1) * N)
            self._sample(self.logits0[s : s + 1], sl, row_stride=0)

    def _sample(self, logits: torch.Tensor, rows: slice, row_stride: int | None) -> None:
        n = rows.stop - rows.start
        if self.native:
            force = None
            if self.force is not None:
                force = self.force[rows.start // self.N :]
            ops.sample(
                logits, self.tokens[rows], R=n, row_stride=row_stride, cap=self.cap, temperature=self.temperature,
                top_p=self.top_p, seed=self.seed, traj_ids=self.traj_ids[rows], step=self.step, force_schedule=force,
                force_group_rows=self.N, force_group_stride=self.G if force is not None else 0,
                history_tokens=self.history[rows],
            )
            return
        # arbitrary Python sampler: give it soft-capped device logits, honour the schedule on the host
        g = self.done
        col = None
        if self.force_host is not None:
            sched = self.force_host[rows.start // self.N : (rows.stop - 1) // self.N + 1, g]
            if bool((sched >= 0).all()):
                col = sched.to(self.dev).repeat_interleave(self.N)[:n]
            else:
                assert bool((sched < 0).all()), "series in one batch must force the same steps with a Python sampler"
        if col is None:
            lg = logits.expand(n, -1).clone() if row_stride == 0 else logits.clone()
            if self.cap > 0:
                ops.softcap_(lg, self.cap)
            if self.rng is None:
                self.rng = torch.Generator(device=self.dev)
                self.rng.manual_seed(self.seed)
            col = self.sampler(lg, rng=self.rng).reshape(-1).to(torch.int32)
        self.tokens[rows] = col
        self.history[rows, g] = col

    # -- stepping ------------------------------------------------------------------------
    @property
    def logits(self) -> torch.Tensor | None:
        """Raw (not yet soft-capped) logits of the last decode step, or None when they were never stored."""
        return self.head_logits if self.lmhead else self.plan.logits

    def _body(self) -> None:
        """One decode step: forward of the current tokens, advance the position, draw the next tokens."""
        logits = self.plan.run(self.tokens, self.bind)
        ops.step_advance(self.step, 1)
        if self.lmhead:
            ops.lmhead_sample(
                self.plan.xn, self.packed.emb, self.tokens, cap=self.cap, temperature=self.temperature, top_p=self.top_p,
                seed=self.seed, traj_ids=self.traj_ids, step=self.step, force_schedule=self.force,
                force_group_rows=self.N, force_group_stride=self.G if self.force is not None else 0,
                history_tokens=self.history, logits_out=self.head_logits, workspace=self.head_ws, status=self.plan.status,
            )
        elif self.native:
            self._sample(logits, slice(0, self.R), row_stride=logits.stride(0))

    def start(self) -> None:
        if self.G == 0:
            return
        self._sample_first()
        self.done = 1

    def advance(self, n_steps: int) -> None:
        """Produce up to `n_steps` more tokens per row (no host synchronisation on the native path)."""
        n_steps = min(n_steps, self.G - self.done)
        if n_steps <= 0:
            return
        if not self.native:
            for _ in range(n_steps):
                logits = self.plan.run(self.tokens, self.bind)
                ops.step_advance(self.step, 1)
                self._sample(logits, slice(0, self.R), row_stride=logits.stride(0))
                self.done += 1
            return
        if self.use_graph and self.graph is None:
            # warm the forward (cuBLAS handles, lazy module loads) without touching tokens or the counter
            self.plan.run(self.tokens, self.bind)
            if self.lmhead:  # and the head GEMM (function attributes, tensor-map encoder) into a scratch token buffer
                ops.lmhead_sample(
                    self.plan.xn, self.packed.emb, torch.empty_like(self.tokens), cap=self.cap, temperature=self.temperature,
                    top_p=self.top_p, seed=self.seed, traj_ids=self.traj_ids, step=self.step, logits_out=self.head_logits,
                    workspace=self.head_ws, status=self.plan.status,
                )
            ops.step_advance(self.step, 0)
            torch.cuda.synchronize(self.dev)
            self.graph = torch.cuda.CUDAGraph()
            before = _lib.stats.launches
            with torch.cuda.graph(self.graph):
                self._body()
            # capture does not execute: nothing has advanced yet
            self.graph_launches = _lib.stats.launches - before
            _lib.stats.launches = before
        for _ in range(n_steps):
            if self.graph is not None:
                self.graph.replay()
                _lib.stats.launches += self.graph_launches
            else:
                self._body()
        self.done += n_steps

    def check_status(self) -> None:
        bad = int(self.plan.status.item())
        for entry in self.prefills:
            bad = bad or int(entry[4].status.item())
        if bad:
            raise RuntimeError(f"device-side status {bad}: a cache slot or position was out of range, or a bounded wait ran out")

    def tokens_so_far(self) -> torch.Tensor:
        return self.history[:, : self.done]


class Engine:
    __slots__ = ("model", "_run")

    def __init__(self, model: BaseGPT) -> None:
        self.model = model
        self._run = None  # the last DecodeRun: reused when the next job has the same shape

    def release(self) -> None:
        """Drop the cached decode state (page pool, plans, captured graph)."""
        self._run = None

    # ---- additive, device-level API -----------------------------------------------------
    @torch.inference_mode()
    def generate_many(
        self,
        prompts: list[list[int]],
        num_samples: int = 1,
        max_tokens: int | None = None,
        sampler: Sampler | Callable | None = None,
        seed: int = 42,
        force_schedules: list[list[int | None]] | None = None,
        traj_offset: int = 0,
        series_offset: int = 0,
        page_tokens: int = 64,
        use_graph: bool = True,
        fmha_impl: int = 0,
        overlap_prefix: bool = True,
        shared_prefix: bool | None = None,
        prefill_group=None,
    ) -> tuple[torch.Tensor, torch.Tensor]:
        """Decode every prompt `num_samples` times.

        `prompts` is a list of token lists, or an int32 device tensor [S, P] of equally long prompts.
        The decode state (page pool, plans, captured step graph) is kept on the engine and reused when the
        next call has the same shape; `release()` frees it.

        Returns (tokens, masks): int32 device tensors of shape (S, num_samples, G); masks are 1 where a
        token was sampled and 0 where it was forced.  `traj_offset`/`series_offset` shift the ids that key
        the random stream, so a shard of the trajectories reproduces exactly its part of the full run;
        `shared_prefix` (None = decide from `num_samples`) fixes whether the prompt's keys are read once per series
        by the tensor-core phase or per row, so that a shard can take the path the whole job takes.
        `num_samples == 0` (a rank without work) returns empty tensors.  `prefill_group`: a process group whose ranks
        decode different trajectories of these same prompts; each rank then prefills only its share of the prompts
        and the ranks exchange the prompt K/V (every rank of the group must make the call).
        """
        assert isinstance(self.model, GPT), "generate_many needs the diff_gpt_b200 GPT"
        assert len(prompts) > 0 and all(len(p) > 0 for p in prompts), "tokens must be non-empty"
        if isinstance(prompts, torch.Tensor):
            assert prompts.is_cuda and prompts.dtype == torch.int32 and prompts.dim() == 2 and prompts.is_contiguous()
        G = min(_effective_max_tokens(self.model.block_size, len(p), max_tokens) for p in prompts)
        S = len(prompts)
        dev = self.model.token_embedding_table.weight.device
        if G == 0 or num_samples == 0:
            z = torch.zeros((S, num_samples, G), dtype=torch.int32, device=dev)
            return z, z.clone()
        if force_schedules is not None:
            assert len(force_schedules) == S
            for sch in force_schedules:
                assert len(sch) >= G, (
                    f"force_schedule must cover all generation steps (len={len(sch)} < {G})"
                )
        on_device = isinstance(prompts, torch.Tensor)
        lens = [int(prompts.shape[1])] * S if on_device else [len(p) for p in prompts]
        key = DecodeRun.key_for(
            self.model, lens, num_samples, G, sampler, seed, force_schedules is not None, page_tokens, use_graph,
            fmha_impl, overlap_prefix, shared_prefix, True, prefill_group is not None,
        )
        run = self._run
        if run is not None and run.key == key and run.reusable():
            run.load(prompts, force_schedules, traj_offset, series_offset)
        else:
            self._run = run = None  # free the old pool before the new one is allocated
            run = DecodeRun(
                self.model, prompts, num_samples, G, sampler, seed, force_schedules, traj_offset=traj_offset,
                series_offset=series_offset, page_tokens=page_tokens, use_graph=use_graph, fmha_impl=fmha_impl,
                overlap_prefix=overlap_prefix, shared_prefix=shared_prefix, prefill_group=prefill_group,
            )
            self._run = run
        run.start()
        run.advance(G)
        toks = run.history.view(S, num_samples, -1)[:, :, :G].clone()  # the run's buffer is reused by the next call
        if run.force is not None:
            masks = (run.force[:, None, :G] < 0).to(torch.int32).expand(S, num_samples, G).contiguous()
        else:
            masks = torch.ones_like(toks)
        run.check_status()
        return toks, masks

    # ---- reference API --------------------------------------------------------------------
    @torch.inference_mode()
    def generate(
        self,
        tokens: list[int],
        num_samples: int = 1,
        max_tokens: int | None = None,
        sampler: Sampler | None = None,
        seed: int = 42,
        force_schedule: list[int | None] | None = None,
    ) -> Generator[tuple[list[int], list[int]], None, None]:
        """Stream `(token_column, token_masks)` per generated position (engine.py:29-154).

        The device runs ahead in chunks of steps; each chunk is read back once.
        """
        assert isinstance(tokens, list), "tokens must be a list of ints"
        assert len(tokens) > 0, "tokens must be non-empty"
        assert all(isinstance(t, int) for t in tokens), "tokens must be a list of ints"
        G = _effective_max_tokens(self.model.block_size, len(tokens), max_tokens)
        if G == 0:
            return
        if force_schedule is not None:
            assert len(force_schedule) >= G, (
                f"force_schedule must cover all generation steps (len={len(force_schedule)} < {G})"
            )
        if not isinstance(self.model, GPT):
            yield from _generate_generic(self.model, tokens, num_samples, G, sampler, seed, force_schedule)
            return
        run = DecodeRun(
            self.model, [tokens], num_samples, G, sampler, seed,
            None if force_schedule is None else [force_schedule],
        )
        run.start()
        emitted = 0
        target = 1  # the first column is available right after the prefill
        while emitted < G:
            run.advance(target - run.done)
            block = run.history[:, emitted : run.done].cpu()  # one read-back per chunk
            for j in range(block.shape[1]):
                g = emitted + j
                forced = force_schedule is not None and force_schedule[g] is not None
                yield block[:, j].tolist(), [0 if forced else 1] * num_samples
            emitted = run.done
            target = min(G, max(16, 2 * run.done))
        run.check_status()

    def generate_batch(
        self, tokens: list[int], num_samples: int = 1, **kwargs
    ) -> tuple[list[list[int]], list[list[int]]]:
        """All trajectories at once: (results, masks), prompt included, masks 0 on prompt/forced positions."""
        unknown = set(kwargs) - {"max_tokens", "sampler", "seed", "force_schedule"}
        if unknown:  # the reference forwards **kwargs to generate(), whose signature rejects anything else
            raise TypeError(f"generate() got an unexpected keyword argument {sorted(unknown)[0]!r}")
        results = [list(tokens) for _ in range(num_samples)]
        masks = [[0] * len(tokens) for _ in range(num_samples)]
        if isinstance(self.model, GPT) and isinstance(tokens, list) and len(tokens) > 0 and all(
            isinstance(t, int) for t in tokens
        ):
            sched = kwargs.get("force_schedule")
            toks, mk = self.generate_many(
                [tokens], num_samples, kwargs.get("max_tokens"), kwargs.get("sampler"), kwargs.get("seed", 42),
                None if sched is None else [sched],
            )
            toks, mk = toks[0].cpu().tolist(), mk[0].cpu().tolist()  # the only read-back
            for i in range(num_samples):
                results[i].extend(toks[i])
                masks[i].extend(mk[i])
            return results, masks
        for column, column_masks in self.generate(tokens, num_samples, **kwargs):
            for i in range(num_samples):
                results[i].append(column[i])
                masks[i].append(column_masks[i])
        return results, masks


def _generate_generic(model, tokens, num_samples, G, sampler, seed, force_schedule):
    """Any other BaseGPT: forward + dense KVCache, tokens kept on the device between steps."""
    device = model.device_type
    rng = torch.Generator(device=device)
    rng.manual_seed(seed)
    H, D, L = model.n_head, model.n_embd // model.n_head, model.n_layer
    first = KVCache(batch_size=1, num_heads=H, seq_len=len(tokens), head_dim=D, num_layers=L)
    logits = model.forward(torch.tensor([tokens], dtype=torch.long, device=device), kv_cache=first)[0]
    logits = logits[:, -1, :].expand(num_samples, -1)
    cache = KVCache(batch_size=num_samples, num_heads=H, seq_len=len(tokens) + G, head_dim=D, num_layers=L)
    cache.prefill(first)
    for g in range(G):
        forced = None if force_schedule is None else force_schedule[g]
        if forced is not None:
            ids = torch.full((num_samples, 1), int(forced), dtype=torch.long, device=device)
        elif sampler is not None:
            ids = sampler(logits, rng=rng)
        else:
            ids = torch.multinomial(torch.softmax(logits.float(), dim=-1), num_samples=1, generator=rng)
        yield ids[:, 0].tolist(), [1 if forced is None else 0] * num_samples
        if g + 1 < G:
            logits = model.forward(ids, kv_cache=cache)[0][:, -1, :]
