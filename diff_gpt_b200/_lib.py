"""ctypes binding of libdgpt_b200.so (the C ABI declared in include/dgpt.h).

The library is mandatory: importing this module raises if the shared object has
not been built, and every wrapper raises `DgptError` on a non-zero status.
There is no fallback path.

`stats.launches` counts the library calls that enqueued kernels (eagerly or into a
graph being captured); `KernelTimer` brackets each such call with CUDA events on the
current stream, which is how the benchmark attributes device time to kernels.
"""

from __future__ import annotations

import contextlib
import ctypes as C
import os

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "libdgpt_b200.so")

F32, BF16 = 0, 1


class DgptError(RuntimeError):
    pass


class KvLayout(C.Structure):
    _fields_ = [
        ("k_base", C.c_void_p),
        ("v_base", C.c_void_p),
        ("page_stride", C.c_int64),
        ("head_stride", C.c_int64),
        ("page_table", C.c_void_p),
        ("page_tokens", C.c_int32),
        ("max_pages", C.c_int32),
        ("n_pages", C.c_int64),
    ]


_p, _i32, _i64, _f32, _u64, _sz = C.c_void_p, C.c_int32, C.c_int64, C.c_float, C.c_uint64, C.c_size_t
_kvp = C.POINTER(KvLayout)

# name -> (restype, argtypes); mirrors include/dgpt.h one to one
PROTOTYPES = {
    "dgpt_last_error": (C.c_int, [C.c_char_p, _sz]),
    "dgpt_version": (C.c_int, []),
    "dgpt_embed_rmsnorm": (C.c_int, [_p, _p, _p, _i64, _i32, _i32, _i32, _p]),
    "dgpt_depthmix": (C.c_int, [C.POINTER(_p), _i32, _p, _p, _p, _i64, _i32, _i32, _p]),
    "dgpt_depthmix_cached": (C.c_int, [C.POINTER(_p), C.POINTER(_p), _i32, _p, _p, _p, _p, _i32, _i64, _i32, _i32, _p]),
    "dgpt_rope_qknorm_kvappend": (
        C.c_int,
        [_p, _p, _p, _i64, _p, _i64, _p, _i32, _kvp, _p, _p, _p, _i32, _i32, _i32, _i32, _i32, _p, _p],
    ),
    "dgpt_fmha_prefill": (
        C.c_int,
        [_p, _i64, _i64, _kvp, _p, _i32, _p, _i64, _i64, _i32, _p, _i32, _i32, _i32, _i32, _i32, _i32, _i32, _i32, _i32, _p, _p],
    ),
    "dgpt_decode_attn_workspace_bytes": (_sz, [_i32, _i32, _i32, _i32]),
    "dgpt_decode_attn": (
        C.c_int,
        [_p, _i64, _kvp, _p, _p, _p, _p, _p, _p, _p, _i64, _p, _i64, _p, _sz, _i32, _i32, _i32, _i32, _i32, _p],
    ),
    "dgpt_decode_attn_partial": (C.c_int, [_p, _i64, _kvp, _p, _p, _p, _p, _p, _p, _i32, _i32, _i32, _i32, _p]),
    "dgpt_attn_merge": (C.c_int, [_p, _p, _p, _p, _p, _i64, _p, _i64, _i32, _i32, _i32, _i32, _p]),
    "dgpt_decode_attn_static_capacity_bytes": (_sz, []),
    "dgpt_decode_attn_static": (
        C.c_int,
        [_p, _i64, _kvp, _p, _p, _p, _p, _p, _p, _p, _i64, _p, _i64, _i32, _i32, _i32, _i32, _i32, _p],
    ),
    "dgpt_swiglu": (C.c_int, [_p, _p, _i64, _i32, _f32, _f32, _i32, _p]),
    "dgpt_sigmoid_gate": (C.c_int, [_p, _i64, _p, _i64, _i64, _i32, _i32, _p]),
    "dgpt_softcap": (C.c_int, [_p, _i64, _f32, _i32, _p]),
    "dgpt_step_advance": (C.c_int, [_p, _i32, _p]),
    "dgpt_linear": (C.c_int, [_p, _i64, _p, _i64, _p, _i64, _p, _i64, _i32, _i32, _i32, _i32, _f32, _f32, _i32, _p, _p]),
    "dgpt_integrate_tokens": (C.c_int, [_p, _i64, _i32, _i32, _i32, _i32, _p, _p, _p, _i32, _p, _p]),
    "dgpt_encode_series": (C.c_int, [_p, _i64, _i32, _i32, _i32, _i32, _p, _i32, _i32, _p, _p, _p, _p, _p]),
    "dgpt_bounded_wait_probe": (C.c_int, [_i32, _i64, _p, _p]),
    "dgpt_token_nll": (C.c_int, [_p, _i64, _p, _p, _i32, _i32, _i32, _p, _p]),
    "dgpt_sample": (
        C.c_int,
        [_p, _i64, _i32, _i32, _f32, _f32, _f32, _u64, _i64, _p, _i32, _p, _p, _i32, _i64, _p, _p, _p, _p, _i64, _i32, _p],
    ),
    "dgpt_nucleus_filter": (C.c_int, [_p, _i64, _p, _i64, _i32, _i32, _f32, _i32, _p]),
    "dgpt_lmhead_workspace_bytes": (_sz, [_i32]),
    "dgpt_lmhead_sample": (
        C.c_int,
        [_p, _i64, _p, _i64, _f32, _f32, _f32, _u64, _i64, _p, _i32, _p, _p, _i32, _i64, _p, _p, _p, _p, _i64, _p, _i64, _p,
         _sz, _i32, _i32, _i32, _i32, _p, _p],
    ),
}
_NOT_LAUNCHING = {
    "dgpt_last_error", "dgpt_version", "dgpt_decode_attn_workspace_bytes", "dgpt_decode_attn_static_capacity_bytes",
    "dgpt_lmhead_workspace_bytes",
}


class Stats:
    launches = 0
    timer = None


stats = Stats()


class KernelTimer:
    """Per-entry-point device time from CUDA events recorded around each call on the current stream."""

    def __init__(self) -> None:
        self.events: dict[str, list] = {}

    def run(self, name, fn, args):
        import torch

        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        rc = fn(*args)
        b.record()
        self.events.setdefault(name, []).append((a, b))
        return rc

    @contextlib.contextmanager
    def region(self, name):
        import torch

        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        yield
        b.record()
        self.events.setdefault(name, []).append((a, b))

    def summary(self) -> dict[str, dict]:
        """{name: {"launches", "total_ms", "avg_ms"}} (synchronise before calling)."""
        out = {}
        for name, evs in self.events.items():
            ms = [a.elapsed_time(b) for a, b in evs]
            out[name] = {"launches": len(ms), "total_ms": sum(ms), "avg_ms": sum(ms) / len(ms)}
        return out


@contextlib.contextmanager
def timed(timer: KernelTimer):
    stats.timer = timer
    try:
        yield timer
    finally:
        stats.timer = None


@contextlib.contextmanager
def region(name: str):
    """Bracket non-library work (the cuBLAS GEMMs) when a timer is active; free otherwise."""
    t = stats.timer
    if t is None:
        yield
    else:
        with t.region(name):
            yield


class _Lib:
    def __init__(self, raw: C.CDLL) -> None:
        self._raw = raw
        for name, (res, args) in PROTOTYPES.items():
            fn = getattr(raw, name)  # AttributeError if the symbol is not exported
            fn.restype = res
            fn.argtypes = args
            setattr(self, name, fn if name in _NOT_LAUNCHING else self._wrap(name, fn))

    @staticmethod
    def _wrap(name, fn):
        def call(*args):
            t = stats.timer
            rc = fn(*args) if t is None else t.run(name, fn, args)
            if rc == 0:
                stats.launches += 1
            return rc

        call.__name__ = name
        return call


def _load() -> _Lib:
    if not os.path.exists(LIB_PATH):
        raise ImportError(
            f"{LIB_PATH} is missing: build it with `python diff_gpt_b200/build.py` "
            "(there is no fallback implementation)"
        )
    return _Lib(C.CDLL(LIB_PATH))


lib = _load()


def last_error() -> str:
    buf = C.create_string_buffer(512)
    lib.dgpt_last_error(buf, 512)
    return buf.value.decode()


def check(rc: int) -> None:
    if rc != 0:
        raise DgptError(f"libdgpt_b200 status {rc}: {last_error()}")
