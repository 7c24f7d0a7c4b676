"""CPU oracle for the accelerate-b200 skeleton library -- TEST INFRASTRUCTURE ONLY.

This package is the checker: it is imported by ``tests/``, by
``__graft_entry__.smoke()`` and by the ``cpu_baseline`` / ``--impl reference``
legs of ``bench.py``.  The product (the ``accelerate-cuda_b200`` package and
``libaccb200.so``) never imports, links or executes anything in here.

PARITY UNPINNED: accelerate-cuda ships no test-suite; the only known-answer
vectors in its tree are the worked scan examples in
``Data/Array/Accelerate/CUDA/CodeGen/PrefixSum.hs:149-153,162-166,176-180``
(checked in ``tests/test_oracle.py``).  The CPU semantics proper belong to the
un-vendored ``accelerate`` 1.0 package (``stack-8.0.yaml:8-11``); what is
restated here is its published denotational semantics, anchored on the call
sites cited beside each function in ``accb_oracle.c``.

Two layers:
  * ``liborc.so`` (``accb_oracle.c``, built by ``make -C oracle``): the five
    benchmark configurations and the integer skeletons, sequential and OpenMP;
  * numpy restatements below for small generic cases (any combiner, all
    boundary modes, tuples).
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB = None


def build(force: bool = False) -> str:
    """Compile ``liborc.so`` with the Makefile beside this file."""
    so = os.path.join(_HERE, "liborc.so")
    src = os.path.join(_HERE, "accb_oracle.c")
    if force or not os.path.exists(so) or os.path.getmtime(so) < os.path.getmtime(src):
        subprocess.run(["make", "-C", _HERE, "-B" if force else "-s"], check=True,
                       stdout=subprocess.DEVNULL)
    return so


def lib() -> C.CDLL:
    global _LIB
    if _LIB is None:
        _LIB = C.CDLL(build())
        _LIB.orc_dot_f32.restype = C.c_double
        _LIB.orc_dot_f32_seq32.restype = C.c_float
        _LIB.orc_sum_f32.restype = C.c_double
        _LIB.orc_max_threads.restype = C.c_int
    return _LIB


def _p(a: np.ndarray):
    assert a.flags["C_CONTIGUOUS"]
    return a.ctypes.data_as(C.c_void_p)


def max_threads() -> int:
    return int(lib().orc_max_threads())


# --------------------------------------------------------------------------
# C-backed oracles
# --------------------------------------------------------------------------
def dot_f32(xs, ys, seed=0.0, nthreads=1) -> float:
    xs = np.ascontiguousarray(xs, np.float32); ys = np.ascontiguousarray(ys, np.float32)
    return float(lib().orc_dot_f32(_p(xs), _p(ys), C.c_int64(xs.size), C.c_double(seed), C.c_int(nthreads)))


def dot_f32_seq32(xs, ys, seed=0.0) -> float:
    xs = np.ascontiguousarray(xs, np.float32); ys = np.ascontiguousarray(ys, np.float32)
    return float(lib().orc_dot_f32_seq32(_p(xs), _p(ys), C.c_int64(xs.size), C.c_float(seed)))


def fold_rows_f32(m, seed=0.0, nthreads=1) -> np.ndarray:
    m = np.ascontiguousarray(m, np.float32)
    rows, cols = m.shape
    out = np.empty(rows, np.float64)
    lib().orc_fold_rows_f32(_p(m), C.c_int64(rows), C.c_int64(cols), C.c_double(seed), _p(out), C.c_int(nthreads))
    return out


def fold_rows_i32(m, seed=0) -> np.ndarray:
    m = np.ascontiguousarray(m, np.int32)
    rows, cols = m.shape
    out = np.empty(rows, np.int32)
    lib().orc_fold_rows_i32(_p(m), C.c_int64(rows), C.c_int64(cols), C.c_int32(seed), _p(out))
    return out


def fold_seg_i32(xs, offs, seed=0) -> np.ndarray:
    xs = np.ascontiguousarray(xs, np.int32); offs = np.ascontiguousarray(offs, np.int32)
    out = np.empty(offs.size - 1, np.int32)
    lib().orc_fold_seg_i32(_p(xs), _p(offs), C.c_int64(offs.size - 1), C.c_int32(seed), _p(out))
    return out


def fold_seg_f32(xs, offs, seed=0.0) -> np.ndarray:
    xs = np.ascontiguousarray(xs, np.float32); offs = np.ascontiguousarray(offs, np.int32)
    out = np.empty(offs.size - 1, np.float64)
    lib().orc_fold_seg_f32(_p(xs), _p(offs), C.c_int64(offs.size - 1), C.c_double(seed), _p(out))
    return out


def scanl_i32(xs, z=0, nthreads=1) -> np.ndarray:
    xs = np.ascontiguousarray(xs, np.int32)
    out = np.empty(xs.size + 1, np.int32)
    if nthreads > 1:
        lib().orc_scanl_i32_par(_p(xs), C.c_int64(xs.size), C.c_int32(z), _p(out), C.c_int(nthreads))
    else:
        lib().orc_scanl_i32(_p(xs), C.c_int64(xs.size), C.c_int32(z), _p(out))
    return out


def scanl1_i32(xs) -> np.ndarray:
    xs = np.ascontiguousarray(xs, np.int32)
    out = np.empty(xs.size, np.int32)
    lib().orc_scanl1_i32(_p(xs), C.c_int64(xs.size), _p(out))
    return out


def scanl_prime_i32(xs, z=0):
    xs = np.ascontiguousarray(xs, np.int32)
    out = np.empty(xs.size, np.int32)
    tot = np.zeros(1, np.int32)
    lib().orc_scanl_prime_i32(_p(xs), C.c_int64(xs.size), C.c_int32(z), _p(out), _p(tot))
    return out, int(tot[0])


def scanr_i32(xs, z=0) -> np.ndarray:
    xs = np.ascontiguousarray(xs, np.int32)
    out = np.empty(xs.size + 1, np.int32)
    lib().orc_scanr_i32(_p(xs), C.c_int64(xs.size), C.c_int32(z), _p(out))
    return out


def scanr1_i32(xs) -> np.ndarray:
    xs = np.ascontiguousarray(xs, np.int32)
    out = np.empty(xs.size, np.int32)
    lib().orc_scanr1_i32(_p(xs), C.c_int64(xs.size), _p(out))
    return out


def scanr_prime_i32(xs, z=0):
    xs = np.ascontiguousarray(xs, np.int32)
    out = np.empty(xs.size, np.int32)
    tot = np.zeros(1, np.int32)
    lib().orc_scanr_prime_i32(_p(xs), C.c_int64(xs.size), C.c_int32(z), _p(out), _p(tot))
    return out, int(tot[0])


def scanl_f32(xs, z=0.0) -> np.ndarray:
    xs = np.ascontiguousarray(xs, np.float32)
    out = np.empty(xs.size + 1, np.float64)
    lib().orc_scanl_f32(_p(xs), C.c_int64(xs.size), C.c_double(z), _p(out))
    return out


def permute_add_i32(keys, nbins, defaults=None, weights=None, nthreads=1) -> np.ndarray:
    keys = np.ascontiguousarray(keys, np.int32)
    defaults = np.zeros(nbins, np.int32) if defaults is None else np.ascontiguousarray(defaults, np.int32)
    w = None if weights is None else np.ascontiguousarray(weights, np.int32)
    out = np.empty(nbins, np.int32)
    lib().orc_permute_add_i32(_p(keys), None if w is None else _p(w), C.c_int64(keys.size), _p(defaults),
                              C.c_int64(nbins), _p(out), C.c_int(nthreads))
    return out


BOUNDARY = {"clamp": 0, "mirror": 1, "wrap": 2, "constant": 3}


def stencil2d(a, weights, boundary="clamp", cval=0.0, nthreads=1) -> np.ndarray:
    """One stencil application on a float32 (or float64) grid; float64 result."""
    wt = np.ascontiguousarray(weights, np.float64)
    ry, rx = wt.shape[0] // 2, wt.shape[1] // 2
    h, w = a.shape
    out = np.empty((h, w), np.float64)
    if a.dtype == np.float64:
        a = np.ascontiguousarray(a)
        lib().orc_stencil2d_f64(_p(a), C.c_int64(h), C.c_int64(w), _p(wt), ry, rx, BOUNDARY[boundary],
                                C.c_double(cval), _p(out), C.c_int(nthreads))
    else:
        a = np.ascontiguousarray(a, np.float32)
        lib().orc_stencil2d_f32in(_p(a), C.c_int64(h), C.c_int64(w), _p(wt), ry, rx, BOUNDARY[boundary],
                                  C.c_double(cval), _p(out), C.c_int(nthreads))
    return out


def stencil2d_iter(a, weights, iters, boundary="clamp", cval=0.0, nthreads=1) -> np.ndarray:
    a = np.ascontiguousarray(a, np.float32)
    wt = np.ascontiguousarray(weights, np.float64)
    ry, rx = wt.shape[0] // 2, wt.shape[1] // 2
    h, w = a.shape
    out = np.empty((h, w), np.float64)
    tmp = np.empty((h, w), np.float64)
    lib().orc_stencil2d_iter(_p(a), C.c_int64(h), C.c_int64(w), _p(wt), ry, rx, BOUNDARY[boundary],
                             C.c_double(cval), C.c_int(iters), _p(tmp), _p(out), C.c_int(nthreads))
    return out


def stencil2d_f32(a, weights, boundary="clamp", cval=0.0, nthreads=1) -> np.ndarray:
    a = np.ascontiguousarray(a, np.float32)
    wt = np.ascontiguousarray(weights, np.float32)
    ry, rx = wt.shape[0] // 2, wt.shape[1] // 2
    h, w = a.shape
    out = np.empty((h, w), np.float32)
    lib().orc_stencil2d_f32(_p(a), C.c_int64(h), C.c_int64(w), _p(wt), ry, rx, BOUNDARY[boundary],
                            C.c_float(cval), _p(out), C.c_int(nthreads))
    return out


def stencil2_2d(a, b, w1, w2, boundary="clamp", cval=0.0) -> np.ndarray:
    a = np.ascontiguousarray(a, np.float32); b = np.ascontiguousarray(b, np.float32)
    w1 = np.ascontiguousarray(w1, np.float64); w2 = np.ascontiguousarray(w2, np.float64)
    ry, rx = w1.shape[0] // 2, w1.shape[1] // 2
    h, w = min(a.shape[0], b.shape[0]), min(a.shape[1], b.shape[1])
    out = np.empty((h, w), np.float64)
    lib().orc_stencil2_2d(_p(a), C.c_int64(a.shape[0]), C.c_int64(a.shape[1]), _p(b), C.c_int64(b.shape[0]),
                          C.c_int64(b.shape[1]), _p(w1), _p(w2), ry, rx, BOUNDARY[boundary], C.c_double(cval),
                          _p(out))
    return out


def blackscholes(spot, strike, years, r=0.02, v=0.30, nthreads=1):
    spot = np.ascontiguousarray(spot, np.float32); strike = np.ascontiguousarray(strike, np.float32)
    years = np.ascontiguousarray(years, np.float32)
    call = np.empty(spot.size, np.float64); put = np.empty(spot.size, np.float64)
    lib().orc_blackscholes(_p(spot), _p(strike), _p(years), C.c_int64(spot.size), C.c_double(r), C.c_double(v),
                           _p(call), _p(put), C.c_int(nthreads))
    return call, put


def blackscholes_f32(spot, strike, years, r=0.02, v=0.30, nthreads=1):
    spot = np.ascontiguousarray(spot, np.float32); strike = np.ascontiguousarray(strike, np.float32)
    years = np.ascontiguousarray(years, np.float32)
    call = np.empty(spot.size, np.float32); put = np.empty(spot.size, np.float32)
    lib().orc_blackscholes_f32(_p(spot), _p(strike), _p(years), C.c_int64(spot.size), C.c_float(r), C.c_float(v),
                               _p(call), _p(put), C.c_int(nthreads))
    return call, put


def backpermute_i32(src, idx) -> np.ndarray:
    src = np.ascontiguousarray(src, np.int32); idx = np.ascontiguousarray(idx, np.int32)
    out = np.empty(idx.size, np.int32)
    lib().orc_backpermute_i32(_p(src), _p(idx), C.c_int64(idx.size), _p(out))
    return out


# --------------------------------------------------------------------------
# numpy restatements for small generic cases (pure-Python loops: small n only)
# --------------------------------------------------------------------------
def scan_generic(xs, f, z=None, direction="l", kind="excl"):
    """Data.List-style scans with an arbitrary associative ``f`` (CodeGen/PrefixSum.hs:137-198).

    kind: "excl" -> scanl/scanr (length n+1), "incl" -> scanl1/scanr1 (length n),
    "prime" -> scanl'/scanr' ((length n), total).  For right scans the new
    element is the LEFT argument: out[i] = f(xs[i], out[i+1]) (Data.List.scanr).
    """
    xs = list(xs)
    n = len(xs)
    if direction == "l":
        if kind == "incl":
            out, acc = [], None
            for x in xs:
                acc = x if acc is None else f(acc, x)
                out.append(acc)
            return out
        out, acc = [z], z
        for x in xs:
            acc = f(acc, x)
            out.append(acc)
        return out if kind == "excl" else (out[:-1], out[-1])
    if kind == "incl":
        out, acc = [None] * n, None
        for i in range(n - 1, -1, -1):
            acc = xs[i] if acc is None else f(xs[i], acc)
            out[i] = acc
        return out
    out, acc = [None] * (n + 1), z
    out[n] = z
    for i in range(n - 1, -1, -1):
        acc = f(xs[i], acc)
        out[i] = acc
    return out if kind == "excl" else (out[1:], out[0])


def fold_generic(xs, f, z=None):
    """fold / fold1 with seed on the right, f(acc, seed) (CodeGen/Reduction.hs:203-215)."""
    acc = None
    for x in xs:
        acc = x if acc is None else f(acc, x)
    if z is None:
        if acc is None:
            raise IndexError("fold1: empty array")  # Execute.hs:283-285
        return acc
    return z if acc is None else f(acc, z)


def permute_generic(defaults, dst_index, src, f):
    """Forward permutation: out[p(i)] = f(src[i], out[p(i)]) with the new value
    as FIRST argument (CodeGen/IndexSpace.hs:203-208); p(i) < 0 is `ignore`."""
    out = list(defaults)
    for i, x in enumerate(src):
        j = dst_index(i)
        if j is None or j < 0:
            continue
        out[j] = f(x, out[j])
    return out


def bound_index(i, sz, mode):
    """One coordinate through a stencil boundary (CodeGen/Stencil/Extra.hs:200-226)."""
    if mode == "clamp":
        return max(0, min(i, sz - 1))
    if mode == "mirror":
        return -i if i < 0 else (sz - (i - sz + 2) if i >= sz else i)
    if mode == "wrap":
        return sz + i if i < 0 else (i - sz if i >= sz else i)
    return i if 0 <= i < sz else None


def stencil3d(a, weights, boundary="clamp", cval=0.0) -> np.ndarray:
    """Linear stencil over a rank-3 array in float64: out[z,y,x] = sum of weights[dz][dy][dx] * a at offset
    (dz-rz, dy-ry, dx-rx), every coordinate through its boundary on its own and, with Constant, the whole tap
    replaced as soon as one coordinate is outside (CodeGen/Stencil/Extra.hs:122-128,191-226; the pattern nests
    outermost dimension first, Stencil.hs:97-98).  numpy's padding modes are the same maps: edge = Clamp,
    reflect = Mirror (-i, sz-(i-sz+2)), wrap = Wrap; tests/test_oracle.py checks that against bound_index."""
    a = np.asarray(a, np.float64)
    wt = np.asarray(weights, np.float64)
    rz, ry, rx = (s // 2 for s in wt.shape)
    mode = {"clamp": "edge", "mirror": "reflect", "wrap": "wrap", "constant": "constant"}[boundary]
    kw = {"constant_values": cval} if boundary == "constant" else {}
    pad = np.pad(a, ((rz, rz), (ry, ry), (rx, rx)), mode=mode, **kw)
    d, h, w = a.shape
    out = np.zeros((d, h, w), np.float64)
    for dz in range(wt.shape[0]):
        for dy in range(wt.shape[1]):
            for dx in range(wt.shape[2]):
                out += wt[dz, dy, dx] * pad[dz:dz + d, dy:dy + h, dx:dx + w]
    return out


def stencil3d_generic(a, fn, rz, ry, rx, boundary="clamp", cval=0.0):
    """Generic rank-3 stencil by loops over bound_index (small arrays only): ``fn`` receives the neighbourhood
    as nested lists t[dz][dy][dx]."""
    a = np.asarray(a)
    d, h, w = a.shape
    out = np.empty((d, h, w), np.float64)
    for z in range(d):
        for y in range(h):
            for x in range(w):
                nb = []
                for dz in range(-rz, rz + 1):
                    plane = []
                    for dy in range(-ry, ry + 1):
                        row = []
                        for dx in range(-rx, rx + 1):
                            zz, yy, xx = bound_index(z + dz, d, boundary), bound_index(y + dy, h, boundary), bound_index(x + dx, w, boundary)
                            row.append(cval if (zz is None or yy is None or xx is None) else float(a[zz, yy, xx]))
                        plane.append(row)
                    nb.append(plane)
                out[z, y, x] = fn(nb)
    return out


def stencil_generic(a, fn, ry, rx, boundary="clamp", cval=0.0):
    """Generic 2-D stencil: ``fn`` receives the (2ry+1)x(2rx+1) neighbourhood as a
    nested list, row-major (CodeGen/Stencil.hs:34-44,97-98)."""
    a = np.asarray(a)
    h, w = a.shape
    out = np.empty((h, w), np.float64)
    for y in range(h):
        for x in range(w):
            nb = []
            for dy in range(-ry, ry + 1):
                row = []
                for dx in range(-rx, rx + 1):
                    yy, xx = bound_index(y + dy, h, boundary), bound_index(x + dx, w, boundary)
                    row.append(cval if (yy is None or xx is None) else float(a[yy, xx]))
                nb.append(row)
            out[y, x] = fn(nb)
    return out
