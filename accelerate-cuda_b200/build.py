"""Build step of the accelerate-b200 package.

Compiles ``libaccb200.so`` (host runtime + the kernels that are part of the
library binary) with nvcc for sm_100a, then pre-seeds the in-tree kernel cache
``kcache/sm_100a/`` with the benchmark programs of ``programs.py`` through the
library's own compile path (``accb_kernel_precompile``), so that a fresh GPU
box finds them as disk-cache hits instead of running nvcc on first use.

nvcc cross-compiles, so all of this works on a machine without a GPU.
Run as ``python accelerate-cuda_b200/build.py`` or through ``__graft_entry__.build()``.
"""
from __future__ import annotations

import ctypes as C
import glob
import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(HERE, "csrc")
LIB = os.path.join(HERE, "libaccb200.so")
NVCC = os.environ.get("ACCB_NVCC", "/usr/local/cuda/bin/nvcc" if os.path.exists("/usr/local/cuda/bin/nvcc") else "nvcc")


def _newest(paths):
    return max(os.path.getmtime(p) for p in paths)


def build_library(force: bool = False, verbose: bool = False) -> str:
    srcs = sorted(glob.glob(os.path.join(CSRC, "runtime", "*.cc")) + glob.glob(os.path.join(CSRC, "runtime", "*.cu")))
    deps = srcs + glob.glob(os.path.join(CSRC, "runtime", "*.h")) + glob.glob(os.path.join(CSRC, "cubits", "*")) + [
        os.path.join(HERE, "..", "include", "accb200.h")]
    if not force and os.path.exists(LIB) and os.path.getmtime(LIB) >= _newest(deps):
        return LIB
    cmd = [NVCC, "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
           "-Xcompiler", "-fPIC,-fvisibility=hidden,-Wall", "-shared", "-cudart", "static",
           "-x", "cu", *srcs, "-o", LIB, "-ldl", "-lpthread"]
    if verbose:
        cmd.insert(1, "-Xptxas")
        cmd.insert(2, "-v")
    subprocess.run(cmd, check=True)
    return LIB


def preseed_cache(verbose: bool = False) -> int:
    """Compile every program of programs.py, and the kernels the embedded language prints for the example
    programs of examples.py, into kcache/ (skips cache hits)."""
    sys.path.insert(0, os.path.dirname(HERE))
    import importlib
    import types
    hand = importlib.import_module("accelerate-cuda_b200.programs")
    generated = importlib.import_module("accelerate-cuda_b200.examples").generated_specs()
    programs = types.SimpleNamespace(ALL={**hand.ALL, **{"lang:" + k: s for k, s in generated.items()}})
    lib = C.CDLL(LIB)
    lib.accb_kernel_precompile.argtypes = [C.c_char_p, C.c_char_p, C.c_char_p, C.c_char_p, C.c_char_p, C.c_char_p, C.c_size_t]
    lib.accb_last_error.restype = C.c_char_p
    lib.accb_last_error.argtypes = [C.c_void_p]
    cache = os.path.join(HERE, "kcache")
    arch_dir = os.path.join(cache, "sm_100a")
    before = set(os.listdir(arch_dir)) if os.path.isdir(arch_dir) else set()
    started = __import__("time").time()

    def one(item):
        name, spec = item
        log = C.create_string_buffer(1 << 16)
        st = lib.accb_kernel_precompile(spec.skeleton.encode(), spec.source.encode(), spec.functor.encode(),
                                        spec.flags.encode() if spec.flags else None, cache.encode(), log, len(log))
        if st != 0:
            raise RuntimeError(f"precompile of {name} failed:\n{log.value.decode(errors='replace')}")
        if verbose:
            print(f"[build] {name}: ok")
        return name

    # nvcc runs in child processes and ctypes drops the GIL: compile in parallel
    from concurrent.futures import ThreadPoolExecutor
    with ThreadPoolExecutor(max_workers=os.cpu_count() or 4) as ex:
        done = list(ex.map(one, programs.ALL.items()))
    # cubins of older skeleton headers are unreachable (the key hashes the headers): drop them
    for f in before:
        p = os.path.join(arch_dir, f)
        if os.path.getmtime(p) < started - 1 and not _is_current(lib, programs, f):
            os.unlink(p)
    return len(done)


def _is_current(lib, programs, filename: str) -> bool:
    if not hasattr(_is_current, "keys"):
        lib.accb_kernel_key.argtypes = [C.c_char_p, C.c_char_p, C.c_char_p, C.c_char_p, C.c_char_p, C.c_size_t]
        keys = set()
        for spec in programs.ALL.values():
            buf = C.create_string_buffer(64)
            lib.accb_kernel_key(spec.skeleton.encode(), spec.source.encode(), spec.functor.encode(),
                                spec.flags.encode() if spec.flags else None, buf, len(buf))
            keys.add(buf.value.decode() + ".cubin")
        _is_current.keys = keys
    return filename in _is_current.keys


def main():
    build_library(force="--force" in sys.argv, verbose="-v" in sys.argv)
    n = preseed_cache(verbose=True)
    print(f"built {LIB}; {n} programs in the kernel cache")


if __name__ == "__main__":
    main()
