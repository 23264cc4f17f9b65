"""`DiffGPT` forecasting facade over the device engine.

Keeps the reference's inference surface (src/diff_gpt/diff_gpt.py:15-37,127-293,365-505):
`predict` (autoregressive and teacher-forced), `predict_samples`, `predict_quantiles`,
`save`, `load`, with the same assertions and return types.  Differences are internal:
the Monte-Carlo trajectories come from one device-resident decode, and all
trajectories are turned back into values by one vectorised integration instead of a
Python loop over samples (diff_gpt.py:239-252).

`anomaly_scores` (diff_gpt.py:295-363) is provided too: one prefill and a fused log-softmax +
gather.  Training (`train`, `train_numa`) belongs to another part of the reference and is not
provided here.
"""

from __future__ import annotations

import numpy as np
import pandas as pd
import torch

from .encoder_decoder import decode, encode
from .model.engine import Engine
from .model.gpt import GPT, BaseGPT
from .sampler.sampler import Sampler


def _quantile_of_sorted(ordered: torch.Tensor, q: float) -> torch.Tensor:
    """np.quantile(x, q, axis=0) with its default linear method, on values already sorted along axis 0, with the
    same float64 operations numpy performs (its _lerp): a + (b - a) t, and b - (b - a)(1 - t) where t >= 0.5.
    Every product and sum is a separate rounded operation, as in numpy."""
    n = ordered.shape[0]
    virtual = (n - 1) * q
    lo = int(np.floor(virtual))
    hi = min(lo + 1, n - 1)
    t = virtual - lo
    a, b = ordered[lo], ordered[hi]
    diff = b - a
    if t >= 0.5:
        return b - diff * (1 - t)
    return a + diff * t


DEVICE_CODEC_MAX_ORDER = 8  # dgpt_encode_series / dgpt_integrate_tokens keep this many difference levels per column


class DiffGPT:
    __slots__ = ("model", "order_of_derivative", "domain_of_definition", "use_decimal", "_engine")

    def __init__(self, model: BaseGPT, order_of_derivative, domain_of_definition: np.ndarray, use_decimal: bool) -> None:
        self.model = model
        self.order_of_derivative = order_of_derivative
        self.domain_of_definition = domain_of_definition
        self.use_decimal = use_decimal
        self._engine = None

    def _get_engine(self) -> Engine:
        """One Engine per DiffGPT (the reference builds one per call, diff_gpt.py:229,479): the engine keeps its
        decode state, so repeated forecasts of one shape reuse the page pool and the captured step graph."""
        if self._engine is None or self._engine.model is not self.model:
            self._engine = Engine(model=self.model)
        return self._engine

    # ---- helpers ---------------------------------------------------------------------
    def _max_order(self, n_cols: int, label: str) -> int:
        order = self.order_of_derivative
        if isinstance(order, (int, np.integer)):
            return int(order)
        arr = np.asarray(order)
        assert arr.shape == (n_cols,), f"order_of_derivative shape {arr.shape} must match {label} {n_cols}"
        return int(arr.max())

    def _device_codec(self, n_cols: int) -> bool:
        """True when values <-> tokens can run on the device: this package's GPT, and difference orders the device
        codec covers.  Higher orders take the host codec (any order), then the same device decode of the tokens."""
        return isinstance(self.model, GPT) and self._max_order(n_cols, "columns") <= DEVICE_CODEC_MAX_ORDER

    def _encode(self, values: np.ndarray):
        return encode(
            inp=values,
            vocab_size=self.model.vocab_size,
            domain_of_definition=self.domain_of_definition,
            order_of_derivative=self.order_of_derivative,
            use_decimal=self.use_decimal,
        )

    def _decode(self, start, scale, tokens: np.ndarray) -> np.ndarray:
        return decode(
            start=start,
            scale=scale,
            inp=tokens,
            vocab_size=self.model.vocab_size,
            order_of_derivative=self.order_of_derivative,
            use_decimal=self.use_decimal,
        )

    # ---- Monte-Carlo futures ---------------------------------------------------------
    def _check_future_request(self, df: pd.DataFrame, max_new_points: int, num_samples: int) -> None:
        assert num_samples >= 1
        rows, columns = df.shape
        max_order = self._max_order(columns, "columns")
        assert max_order <= rows, (
            f"max order {max_order} > context length {rows}: "
            f"not enough history to compute the k-th derivative prefix"
        )
        total_positions = (rows + max_new_points - max_order) * columns
        assert total_positions <= self.model.block_size, (
            f"prompt rows ({rows}) + new points ({max_new_points}) with "
            f"{columns} columns (max_order={max_order}) require {total_positions} "
            f"context positions, but block_size is {self.model.block_size}"
        )

    def _encode_on_device(self, values: np.ndarray):
        """values f64 [S, rows, F] -> (tokens int32 [S, rows - max_k, F], end state f64 [S, F, max(max_k, 1)], scale,
        orders), all on the model's device: one `dgpt_encode_series` launch tokenises every series and leaves the
        running sums the decoder continues from."""
        from . import ops
        from .encoder_decoder import _orders, _scalar, column_scales

        assert not self.use_decimal, "the Decimal code path of the reference codec is not part of this build"
        assert values.dtype == np.float64 and values.ndim == 3
        columns = values.shape[2]
        dev = self.model.token_embedding_table.weight.device
        orders = _orders(self.order_of_derivative, columns)
        scale = torch.from_numpy(column_scales(self.model.vocab_size, self.domain_of_definition, orders)).to(dev)
        orders_dev = torch.from_numpy(orders.astype(np.int32)).to(dev)
        tokens, _start, state = ops.encode_series(
            torch.from_numpy(np.array(values, dtype=np.float64, order="C")).to(dev), self.model.vocab_size, scale, orders_dev,
            int(orders.max()) if columns else 0, _scalar(self.order_of_derivative),
        )
        return tokens, state, scale, orders_dev

    def _future_samples_on_device(self, df: pd.DataFrame, max_new_points: int, sampler: Sampler | None, num_samples: int) -> torch.Tensor:
        """(num_samples, max_new_points, n_features) float64 ON THE DEVICE."""
        values = df.to_numpy(dtype=np.float64)
        return self._many_futures_on_device(values[None], max_new_points, sampler, num_samples)[0]

    def _many_futures_on_device(self, values: np.ndarray, max_new_points: int, sampler: Sampler | None, num_samples: int) -> torch.Tensor:
        """(S, num_samples, max_new_points, n_features) float64 ON THE DEVICE for S equally shaped series: the
        series are tokenised where the model lives (`dgpt_encode_series`), all prompts are decoded together, and
        the tokens are turned back into values where they were sampled (`dgpt_integrate_tokens`), continuing the
        cumulative sums from the state each context leaves."""
        from . import ops

        S, _rows, columns = values.shape
        tokens, state, scale, orders_dev = self._encode_on_device(values)
        prompts = tokens.reshape(S, -1)  # row-major: (time, channel)
        generated, _ = self._get_engine().generate_many(prompts, num_samples, max_new_points * columns, sampler)
        V = self.model.vocab_size
        out = torch.empty((S, num_samples, max_new_points, columns), dtype=torch.float64, device=generated.device)
        for s in range(S):
            out[s] = ops.integrate_tokens(generated[s], columns, V, scale, orders_dev, state[s])
        return out

    @torch.inference_mode()
    def predict_samples_many(self, dfs, max_new_points: int, num_samples: int, sampler: Sampler | None = None) -> np.ndarray:
        """`predict_samples` for several equally shaped frames in one decode: (S, num_samples, max_new_points, F).
        The reference loops over series on the host (benchmarks/prob_m4_bench.py:174-182).  Trajectory n of
        series s draws the random stream keyed by (s, n); `predict_samples` is the case S = 1."""
        assert isinstance(self.model, GPT), "predict_samples_many needs the diff_gpt_b200 GPT"
        assert len(dfs) > 0
        assert self._device_codec(dfs[0].shape[1]), f"difference orders above {DEVICE_CODEC_MAX_ORDER}: call predict_samples per frame"
        shape = dfs[0].shape
        for df in dfs:
            assert df.shape == shape, "all frames must have the same shape"
            self._check_future_request(df, max_new_points, num_samples)
        values = np.stack([df.to_numpy(dtype=np.float64) for df in dfs])
        return self._many_futures_on_device(values, max_new_points, sampler, num_samples).cpu().numpy()

    def _generate_future_samples(self, df: pd.DataFrame, max_new_points: int, sampler: Sampler | None, num_samples: int) -> np.ndarray:
        """(num_samples, max_new_points, n_features) float64: the forecast rows only."""
        self._check_future_request(df, max_new_points, num_samples)
        rows, columns = df.shape
        if self._device_codec(columns):
            return self._future_samples_on_device(df, max_new_points, sampler, num_samples).cpu().numpy()
        start, scale, encoded = self._encode(df.to_numpy(dtype=np.float64))
        prompt = encoded.reshape(-1).astype(np.int64).tolist()  # row-major: (time, channel)
        results, _ = self._get_engine().generate_batch(
            tokens=prompt, num_samples=num_samples, max_tokens=max_new_points * columns, sampler=sampler
        )
        tokens = np.asarray(results, dtype=np.int64).reshape(num_samples, -1, columns)
        values = self._decode(start, scale, tokens)  # (N, rows + new, F), all trajectories at once
        return np.ascontiguousarray(values[:, rows : rows + max_new_points, :])

    @torch.inference_mode()
    def predict_samples(self, df: pd.DataFrame, max_new_points: int, num_samples: int, sampler: Sampler | None = None) -> np.ndarray:
        return self._generate_future_samples(df=df, max_new_points=max_new_points, sampler=sampler, num_samples=num_samples)

    @torch.inference_mode()
    def predict_quantiles(
        self,
        df: pd.DataFrame,
        max_new_points: int,
        quantiles=(0.1, 0.5, 0.9),
        num_samples: int = 100,
        sampler: Sampler | None = None,
    ) -> dict[float, pd.DataFrame]:
        for q in quantiles:
            assert 0.0 < q < 1.0, f"quantile {q} must be in (0, 1)"
        if self._device_codec(df.shape[1]):
            self._check_future_request(df, max_new_points, num_samples)
            futures = self._future_samples_on_device(df, max_new_points, sampler, num_samples)
            ordered = torch.sort(futures, dim=0).values  # (N, H, F) sorted over the trajectories
            return {
                float(q): pd.DataFrame(_quantile_of_sorted(ordered, float(q)).cpu().numpy(), columns=df.columns)
                for q in quantiles
            }
        futures = self._generate_future_samples(df=df, max_new_points=max_new_points, sampler=sampler, num_samples=num_samples)
        return {float(q): pd.DataFrame(np.quantile(futures, q, axis=0), columns=df.columns) for q in quantiles}

    # ---- point forecasts ---------------------------------------------------------------
    @torch.inference_mode()
    def predict(
        self,
        df: pd.DataFrame,
        max_new_points: int | None = None,
        future_covariates_df: pd.DataFrame | None = None,
        target_columns=None,
        sampler: Sampler | None = None,
    ) -> pd.DataFrame:
        if future_covariates_df is None:
            assert target_columns is None, "target_columns is only meaningful with future_covariates_df"
            assert max_new_points is not None, "max_new_points is required when future_covariates_df is None"
            future = self._generate_future_samples(df=df, max_new_points=max_new_points, sampler=sampler, num_samples=1)[0]
            return pd.DataFrame(np.concatenate([df.to_numpy(dtype=np.float64), future], axis=0), columns=df.columns)
        assert target_columns is not None and len(target_columns) > 0, (
            "target_columns must be non-empty when future_covariates_df is given"
        )
        pred_len = len(future_covariates_df)
        assert max_new_points is None or max_new_points == pred_len, (
            f"max_new_points ({max_new_points}) must equal len(future_covariates_df) ({pred_len})"
        )
        return self._predict_teacher_forced(df, future_covariates_df, target_columns, sampler)

    def _predict_teacher_forced(self, context_df, future_covariates_df, target_columns, sampler) -> pd.DataFrame:
        """Known future columns are forced token by token, target columns are sampled (diff_gpt.py:396-498)."""
        names = list(context_df.columns)
        assert list(future_covariates_df.columns) == names, "context and future must have the same columns"
        n_features = len(names)
        targets: set[int] = set()
        for c in target_columns:
            if isinstance(c, str):
                assert c in names, f"target column {c!r} not found in {names}"
                targets.add(names.index(c))
            else:
                targets.add(int(c))
        ctx_len, pred_len = len(context_df), len(future_covariates_df)
        max_order = self._max_order(n_features, "n_features")
        assert max_order <= ctx_len, (
            f"max order {max_order} > context length {ctx_len}: "
            f"not enough history to compute the k-th derivative prefix"
        )
        total_tokens = (ctx_len + pred_len - max_order) * n_features
        assert total_tokens <= self.model.block_size, (
            f"ctx={ctx_len} pred={pred_len} cols={n_features} (max_order={max_order}) "
            f"need {total_tokens} tokens but block_size={self.model.block_size}"
        )
        frame = pd.concat([context_df, future_covariates_df], ignore_index=True).copy()
        for c in targets:
            frame.iloc[ctx_len:, c] = 0.0  # placeholders; these positions are generated
        start, scale, encoded = self._encode(frame.to_numpy(dtype=np.float64))
        flat = encoded.reshape(-1).astype(np.int64)
        n_prompt = (ctx_len - max_order) * n_features
        schedule = [None if (p % n_features) in targets else int(flat[p]) for p in range(n_prompt, total_tokens)]
        results, _ = self._get_engine().generate_batch(
            tokens=flat[:n_prompt].tolist(), num_samples=1, max_tokens=total_tokens - n_prompt, sampler=sampler,
            force_schedule=schedule,
        )
        tokens = np.asarray(results[0], dtype=np.int64).reshape(-1, n_features)
        return pd.DataFrame(self._decode(start, scale, tokens), columns=names)

    # ---- anomaly scores --------------------------------------------------------------------
    @torch.inference_mode()
    def anomaly_scores(self, df: pd.DataFrame) -> pd.DataFrame:
        """-log p(token_t | tokens before t) per (time, channel), NaN where nothing can be scored
        (the first max-order rows and the very first token); diff_gpt.py:295-363.

        One prefill forward of the encoded signal; the negative log-likelihood of each next token is
        taken from the logits on the device (`dgpt_token_nll`) without building the log-probability table.
        """
        from . import ops

        columns, T = df.shape[1], df.shape[0]
        max_order = self._max_order(columns, "columns")
        assert max_order <= T, f"max order {max_order} > signal length {T}"
        inp = df.to_numpy(dtype=np.float64)
        N = (T - max_order) * columns
        assert N <= self.model.block_size, (
            f"signal has {N} tokens but block_size is {self.model.block_size}; "
            f"chunk the input manually for longer sequences"
        )
        device = torch.device(self.model.device_type)
        if self._device_codec(columns):  # tokenised where the model lives
            tokens = self._encode_on_device(inp[None])[0].reshape(1, N).to(torch.int64)
        else:
            _, _, encoded = self._encode(inp)
            tokens = torch.as_tensor(encoded.reshape(-1).astype(np.int64), dtype=torch.int64, device=device).unsqueeze(0)
        was_training = self.model.training
        self.model.eval()
        logits, _ = self.model.forward(tokens)  # (1, N, V); row i predicts token i + 1
        if was_training:
            self.model.train()
        flat = np.full(N, np.nan, dtype=np.float64)
        if N > 1:
            status = torch.zeros(1, dtype=torch.int32, device=device)
            nll = ops.token_nll(logits[0, :-1], tokens[0, 1:].to(torch.int32).contiguous(), status)
            flat[1:] = nll.cpu().numpy().astype(np.float64)
            assert int(status.item()) == 0, "a token id was outside the vocabulary"
        out = np.full((T, columns), np.nan, dtype=np.float64)
        out[max_order:] = flat.reshape(T - max_order, columns)
        return pd.DataFrame(out, columns=df.columns, index=df.index)

    # ---- checkpoints --------------------------------------------------------------------
    def save(self, path: str = "diff-gpt.bin") -> None:
        torch.save(self.model.state_dict(), path)

    def load(self, path: str = "diff-gpt.bin") -> None:
        self.model.load_state_dict(torch.load(path, weights_only=True))
        self.model.eval()
