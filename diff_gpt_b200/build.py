"""Compile the CUDA sources under csrc/ into libdgpt_b200.so (sm_100a only).

    python diff_gpt_b200/build.py [--force] [--verbose]

Run it as a script: the package itself refuses to import until the library exists.

nvcc cross-compiles without a GPU.  Objects are cached next to the sources and
rebuilt when a source or header is newer; the shared object lands in this
package directory so it travels with the tree.
"""

from __future__ import annotations

import os
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor

PKG = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(PKG, "csrc")
INCLUDE = os.path.join(os.path.dirname(PKG), "include")
LIB = os.path.join(PKG, "libdgpt_b200.so")
NVCC = os.environ.get("NVCC", "/usr/local/cuda/bin/nvcc")
FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-O3", "-std=c++17", "-lineinfo", "-Xcompiler", "-fPIC",
    "-Xptxas", "-v" if os.environ.get("DGPT_PTXAS_V") else "-O3",
]


def _sources() -> list[str]:
    return sorted(os.path.join(CSRC, f) for f in os.listdir(CSRC) if f.endswith(".cu"))


def _headers() -> list[str]:
    hs = [os.path.join(CSRC, f) for f in os.listdir(CSRC) if f.endswith(".cuh")]
    hs += [os.path.join(INCLUDE, f) for f in os.listdir(INCLUDE) if f.endswith(".h")]
    return hs


def _stale(target: str, deps: list[str]) -> bool:
    if not os.path.exists(target):
        return True
    t = os.path.getmtime(target)
    return any(os.path.getmtime(d) > t for d in deps)


def _flags_changed() -> bool:
    """True (and the record is rewritten) when the objects on disk were built with other flags."""
    record = os.path.join(CSRC, ".build_flags")
    now = " ".join(FLAGS)
    try:
        same = open(record).read() == now
    except OSError:
        same = False
    if not same:
        with open(record, "w") as f:
            f.write(now)
    return not same


def _compile(src: str, verbose: bool) -> str:
    obj = src[:-3] + ".o"
    if _stale(obj, [src] + _headers() + [os.path.abspath(__file__)]):
        cmd = [NVCC, *FLAGS, "-I", INCLUDE, "-c", src, "-o", obj]
        if verbose:
            print(" ".join(cmd), flush=True)
        r = subprocess.run(cmd, capture_output=True, text=True)
        if verbose or r.returncode != 0:
            sys.stderr.write(r.stdout + r.stderr)
        if r.returncode != 0:
            raise RuntimeError(f"nvcc failed on {os.path.basename(src)}")
    return obj


def build(force: bool = False, verbose: bool = False) -> str:
    """Build (if stale) and return the path of libdgpt_b200.so."""
    srcs = _sources()
    force = force or _flags_changed()
    if force:
        for s in srcs:
            o = s[:-3] + ".o"
            if os.path.exists(o):
                os.remove(o)
    with ThreadPoolExecutor(max_workers=min(8, len(srcs))) as ex:
        objs = list(ex.map(lambda s: _compile(s, verbose), srcs))
    if force or _stale(LIB, objs):
        cmd = [NVCC, "-shared", "-o", LIB, *objs]
        if verbose:
            print(" ".join(cmd), flush=True)
        r = subprocess.run(cmd, capture_output=True, text=True)
        if r.returncode != 0:
            sys.stderr.write(r.stdout + r.stderr)
            raise RuntimeError("link failed")
    return LIB


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose="--verbose" in sys.argv))
