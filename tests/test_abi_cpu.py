"""What can be checked of the C-ABI library without a GPU: it loads, exports every
symbol the header declares, fails loudly without a CUDA driver, and its kernel
cache compiles, keys, persists and reports compiler errors.  No compute calls."""
import ctypes as C
import os
import re
import subprocess
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
HEADER = os.path.join(ROOT, "include", "accb200.h")
PKG = os.path.join(ROOT, "accelerate-cuda_b200")


def declared_symbols():
    text = open(HEADER).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    text = "\n".join(l for l in text.splitlines() if not l.lstrip().startswith("#"))
    return sorted(set(re.findall(r"ACCB_API\s+[^;(]*?\b(\w+)\s*\(", text)))


def test_header_declares_the_expected_surface():
    syms = declared_symbols()
    for name in ("accb_map", "accb_fold_all", "accb_fold_dim", "accb_fold_seg", "accb_scan", "accb_permute",
                 "accb_stencil", "accb_stencil2", "accb_kernel_get", "accb_malloc", "accb_insert_unmanaged",
                 "accelerateCreate", "runProgram", "freeOutput", "freeProgram", "accelerateDestroy",
                 "accb_scanl_add_i32_noalloc"):
        assert name in syms
    assert len(syms) >= 60


def test_library_loads_and_exports_every_declared_symbol(accb):
    L = accb.lib()
    missing = [s for s in declared_symbols() if not hasattr(L, s)]
    assert not missing, missing


def test_struct_layouts_match_accffi_h(accb):
    """InputArray {int*; void**}, OutputArray {int*; void**; stable pointer} (include/AccFFI.h:10-19)."""
    p = C.sizeof(C.c_void_p)
    assert C.sizeof(accb.InputArray) == 2 * p and C.sizeof(accb.OutputArray) == 3 * p
    assert accb.OutputArray.stable_ptr.offset == 2 * p


def test_no_cpu_fallback_without_a_driver(accb):
    import torch
    if torch.cuda.is_available():
        pytest.skip("a GPU is present")
    L = accb.lib()
    assert L.accb_init() == accb.ENODRIVER
    assert b"libcuda" in L.accb_last_error(None)
    with pytest.raises(accb.AccbError) as e:
        accb.Context(0)
    assert e.value.status == accb.ENODRIVER
    assert L.accelerateCreate(0, None) is None
    with pytest.raises(accb.AccbError) as e:
        accb.Group([0, 0])
    assert e.value.status == accb.ENODRIVER


def test_header_is_plain_c_and_the_library_links_from_c(tmp_path):
    """What a cgo / hsc2hs stub needs: `include/accb200.h` under -std=c99 -pedantic, and -laccb200 from a C program."""
    exe = tmp_path / "abi_smoke"
    subprocess.run(["gcc", "-std=c99", "-pedantic", "-Wall", "-Werror", "-I", os.path.join(ROOT, "include"),
                    os.path.join(ROOT, "tests", "cpp", "abi_smoke.c"), "-L", PKG, "-laccb200",
                    f"-Wl,-rpath,{PKG}", "-o", str(exe)], check=True)
    out = subprocess.run([str(exe)], capture_output=True, text=True)
    assert out.returncode == 0 and out.stdout.strip() == "OK", out.stdout + out.stderr


def test_product_never_touches_the_oracle():
    for dirpath, _, files in os.walk(PKG):
        for f in files:
            if f.endswith((".py", ".cc", ".cu", ".cuh", ".h")):
                src = open(os.path.join(dirpath, f), errors="replace").read()
                # prose may mention "the float64 oracle"; code must not import, load or call it
                for needle in ("import oracle", "from oracle", 'import_module("oracle', "liborc", "orc_"):
                    assert needle not in src, f"{f} refers to the oracle: {needle}"


def _key(L, spec, flags=None):
    buf = C.create_string_buffer(64)
    L.accb_kernel_key.argtypes = [C.c_char_p] * 4 + [C.c_char_p, C.c_size_t]
    assert L.accb_kernel_key(spec.skeleton.encode(), spec.source.encode(), spec.functor.encode(),
                             flags.encode() if flags else None, buf, len(buf)) == 0
    return buf.value.decode()


def test_kernel_keys_depend_on_source_and_flags(accb, P):
    L = accb.lib()
    k1, k2 = _key(L, P.SCAN_ADD_I32), _key(L, P.SCAN_ADD_I32)
    assert k1 == k2 and re.fullmatch(r"[0-9a-f]{32}", k1)
    assert _key(L, P.SCAN_ADD_I32, "-DACCB_SCAN_TMA=0") != k1
    assert _key(L, P.SCAN_ADD_I64) != k1


def test_every_shipped_program_is_in_the_preseeded_cache(accb, P):
    L = accb.lib()
    cache = os.path.join(PKG, "kcache", "sm_100a")
    missing = [n for n, s in P.ALL.items() if not os.path.exists(os.path.join(cache, _key(L, s, s.flags or None) + ".cubin"))]
    assert not missing, f"run `python accelerate-cuda_b200/build.py`: {missing}"


def _precompile(L, spec, cache_dir):
    L.accb_kernel_precompile.argtypes = [C.c_char_p] * 5 + [C.c_char_p, C.c_size_t]
    log = C.create_string_buffer(1 << 16)
    st = L.accb_kernel_precompile(spec.skeleton.encode(), spec.source.encode(), spec.functor.encode(),
                                  spec.flags.encode() if spec.flags else None, str(cache_dir).encode(), log, len(log))
    return st, log.value.decode(errors="replace")


def test_precompile_persists_a_cubin_under_its_key(accb, P, tmp_path):
    """nvcc cross-compiles without a GPU; the cubin lands in <dir>/sm_100a/<key>.cubin, written atomically."""
    L = accb.lib()
    spec = accb.KernelSpec("map", "Twice", """
struct Twice { using In = accb::types<int>; using Out = accb::types<int>;
  static __device__ void apply(const accb::Env&, long long, int x, int& o) { o = 2 * x; } };""")
    st, log = _precompile(L, spec, tmp_path)
    assert st == 0, log
    path = tmp_path / "sm_100a" / (_key(L, spec) + ".cubin")
    assert path.exists() and path.stat().st_size > 1000
    assert not list((tmp_path / "sm_100a").glob("*.part.*"))


def test_compiler_errors_come_back_as_a_status_with_the_nvcc_log(accb, tmp_path):
    L = accb.lib()
    bad = accb.KernelSpec("map", "Broken", "struct Broken { this is not C++ };")
    st, log = _precompile(L, bad, tmp_path)
    assert st == accb.ECOMPILE and "error" in log.lower()
    assert b"failed" in L.accb_last_error(None)
    unknown = accb.KernelSpec("no_such_skeleton", "X", "struct X {};")
    st, _ = _precompile(L, unknown, tmp_path)
    assert st == accb.EINVAL


def test_injected_compiler_failure(accb, tmp_path):
    """ACCB_FAIL=nvcc: the compiler 'fails' without running; checked in a child process so the
    injection counter of this process is untouched."""
    code = f"""
import sys, importlib, ctypes as C
sys.path.insert(0, {ROOT!r})
accb = importlib.import_module("accelerate-cuda_b200")
L = accb.lib()
L.accb_kernel_precompile.argtypes = [C.c_char_p] * 5 + [C.c_char_p, C.c_size_t]
src = b"struct F {{ using In = accb::types<int>; using Out = accb::types<int>; static __device__ void apply(const accb::Env&, long long, int x, int& o) {{ o = x + 12345; }} }};"
log = C.create_string_buffer(4096)
st = L.accb_kernel_precompile(b"map", src, b"F", None, {str(tmp_path)!r}.encode(), log, 4096)
print(st, log.value.decode())
"""
    env = dict(os.environ, ACCB_FAIL="nvcc")
    out = subprocess.run([sys.executable, "-c", code], env=env, capture_output=True, text=True, timeout=120)
    assert out.returncode == 0, out.stderr
    assert out.stdout.startswith("4 ") and "injected" in out.stdout


def test_memory_table_logic_with_a_fake_device(tmp_path):
    """LRU write-back eviction, pinning, unmanaged entries (Array/Remote.hs:91-202) through a fake allocator."""
    exe = tmp_path / "memtable_harness"
    subprocess.run(["g++", "-std=c++17", "-O1", "-I", os.path.join(PKG, "csrc", "runtime"), "-o", str(exe),
                    os.path.join(ROOT, "tests", "cpp", "memtable_harness.cc")], check=True)
    out = subprocess.run([str(exe)], capture_output=True, text=True)
    assert out.returncode == 0 and out.stdout.strip() == "OK", out.stdout + out.stderr
