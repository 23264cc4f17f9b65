"""ctypes binding of libdgpt_b200.so (the C ABI declared in include/dgpt.h).

The library is mandatory: importing this module raises if the shared object has
not been built, and every wrapper raises `DgptError` on a non-zero status.
There is no fallback path.
"""

from __future__ import annotations

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
    ]


_p, _i32, _i64, _f32, _u64, _sz = C.c_void_p, C.c_int32, C.c_int64, C.c_float, C.c_uint64, C.c_size_t
_kvp = C.POINTER(KvLayout)

# name -> (restype, argtypes); mirrors include/dgpt.h one to one
PROTOTYPES = {
    "dgpt_last_error": (C.c_int, [C.c_char_p, _sz]),
    "dgpt_version": (C.c_int, []),
    "dgpt_embed_rmsnorm": (C.c_int, [_p, _p, _p, _i64, _i32, _i32, _i32, _p]),
    "dgpt_depthmix": (C.c_int, [C.POINTER(_p), _i32, _p, _p, _p, _i64, _i32, _i32, _p]),
    "dgpt_rope_qknorm_kvappend": (
        C.c_int,
        [_p, _p, _p, _i64, _p, _i64, _p, _i32, _kvp, _p, _p, _p, _i32, _i32, _i32, _i32, _i32, _p, _p],
    ),
    "dgpt_fmha_prefill": (
        C.c_int,
        [_p, _i64, _i64, _kvp, _p, _i32, _p, _i64, _i64, _i32, _p, _i32, _i32, _i32, _i32, _i32, _i32, _i32, _i32, _p, _p],
    ),
    "dgpt_decode_attn_workspace_bytes": (_sz, [_i32, _i32, _i32, _i32]),
    "dgpt_decode_attn": (
        C.c_int,
        [_p, _i64, _kvp, _p, _p, _p, _p, _p, _p, _p, _i64, _p, _i64, _p, _sz, _i32, _i32, _i32, _i32, _i32, _p],
    ),
    "dgpt_swiglu": (C.c_int, [_p, _p, _i64, _i32, _f32, _f32, _i32, _p]),
    "dgpt_sigmoid_gate": (C.c_int, [_p, _i64, _p, _i64, _i64, _i32, _i32, _p]),
    "dgpt_softcap": (C.c_int, [_p, _i64, _f32, _i32, _p]),
    "dgpt_step_advance": (C.c_int, [_p, _i32, _p]),
    "dgpt_sample": (
        C.c_int,
        [_p, _i64, _i32, _i32, _f32, _f32, _f32, _u64, _i64, _p, _i32, _p, _p, _i32, _i64, _p, _p, _p, _p, _i64, _i32, _p],
    ),
    "dgpt_nucleus_filter": (C.c_int, [_p, _i64, _p, _i64, _i32, _i32, _f32, _i32, _p]),
}


def _load() -> C.CDLL:
    if not os.path.exists(LIB_PATH):
        raise ImportError(
            f"{LIB_PATH} is missing: build it with `python -m diff_gpt_b200.build` "
            "(there is no fallback implementation)"
        )
    lib = C.CDLL(LIB_PATH)
    for name, (res, args) in PROTOTYPES.items():
        fn = getattr(lib, name)  # AttributeError if the symbol is not exported
        fn.restype = res
        fn.argtypes = args
    return lib


lib = _load()


def last_error() -> str:
    buf = C.create_string_buffer(512)
    lib.dgpt_last_error(buf, 512)
    return buf.value.decode()


def check(rc: int) -> None:
    if rc != 0:
        raise DgptError(f"libdgpt_b200 status {rc}: {last_error()}")
