"""The reference's own skeleton algorithms as plain CUDA for sm_100a (refskel.cu), built into
librefskel.so and called through ctypes on torch device tensors.

A baseline for bench.py only: nothing in the library imports this package.
"""
from __future__ import annotations

import ctypes as C
import os
import shutil
import subprocess

HERE = os.path.dirname(os.path.abspath(__file__))
SRC = os.path.join(HERE, "refskel.cu")
LIB = os.path.join(HERE, "librefskel.so")

_lib = None


def build(force: bool = False) -> str:
    """nvcc -> librefskel.so (cross-compiles without a GPU)."""
    if not force and os.path.exists(LIB) and os.path.getmtime(LIB) >= os.path.getmtime(SRC):
        return LIB
    nvcc = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    # -use_fast_math as for the library's Black-Scholes functor, so that only the skeleton differs
    subprocess.run([nvcc, "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
                    "-use_fast_math", "-Xcompiler", "-fPIC", "-shared", "-cudart", "static", SRC, "-o", LIB],
                   check=True)
    return LIB


def lib() -> C.CDLL:
    global _lib
    if _lib is None:
        if not os.path.exists(LIB):
            raise RuntimeError(f"{LIB} is missing: run `python __graft_entry__.py` (or refskel.build()) first")
        _lib = C.CDLL(LIB)
        P, I, F = C.c_void_p, C.c_int, C.c_float
        _lib.refskel_map_blackscholes.argtypes = [P, P, P, P, P, I, P]
        _lib.refskel_dot.argtypes = [P, P, I, F, P, P, P]
        _lib.refskel_fold_rows.argtypes = [P, I, I, F, P, P]
        _lib.refskel_scanl.argtypes = [P, I, I, P, P, P]
        _lib.refskel_histogram.argtypes = [P, I, P, I, P, P, P, P]
        _lib.refskel_stencil_blur.argtypes = [P, P, I, I, P]
        _lib.refskel_config.argtypes = [I, C.POINTER(C.c_int), C.POINTER(C.c_int)]
    return _lib


def _check(rc: int, what: str) -> None:
    if rc != 0:
        raise RuntimeError(f"refskel {what} failed (see stderr)")


def _stream() -> int:
    import torch
    return torch.cuda.current_stream().cuda_stream


def map_blackscholes(spot, strike, years, call, put) -> None:
    _check(lib().refskel_map_blackscholes(spot.data_ptr(), strike.data_ptr(), years.data_ptr(), call.data_ptr(),
                                          put.data_ptr(), spot.numel(), _stream()), "map")


def dot(xs, ys, seed, partials, out) -> None:
    _check(lib().refskel_dot(xs.data_ptr(), ys.data_ptr(), xs.numel(), float(seed), partials.data_ptr(),
                             out.data_ptr(), _stream()), "foldAll")


def fold_rows(m, seed, out) -> None:
    _check(lib().refskel_fold_rows(m.data_ptr(), m.shape[0], m.shape[1], float(seed), out.data_ptr(), _stream()), "fold")


def scanl(x, seed, out, blk) -> None:
    _check(lib().refskel_scanl(x.data_ptr(), x.numel(), int(seed), out.data_ptr(), blk.data_ptr(), _stream()), "scanl")


def histogram(keys, defaults, out, lock, err) -> None:
    _check(lib().refskel_histogram(keys.data_ptr(), keys.numel(), defaults.data_ptr(), defaults.numel(),
                                   out.data_ptr(), lock.data_ptr(), err.data_ptr(), _stream()), "permute")


def stencil_blur(a, b) -> None:
    _check(lib().refskel_stencil_blur(a.data_ptr(), b.data_ptr(), a.shape[0], a.shape[1], _stream()), "stencil")


def config(which: int):
    cta, per_sm = C.c_int(), C.c_int()
    _check(lib().refskel_config(which, C.byref(cta), C.byref(per_sm)), "config")
    return cta.value, per_sm.value


def scratch_elems(sm_count: int) -> int:
    """Elements of scratch (partials / interval totals) any of the calls above may need."""
    return 2 * sm_count * 32
