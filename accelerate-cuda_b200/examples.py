"""The benchmark programs of this repository written in the embedded array language (lang.py), the way an
Accelerate user would write them.  ``generated_specs()`` gives the kernels they compile to, under the names of
the hand-written functors of programs.py they correspond to; bench.py can run its workloads with either set
(``--functors lang``), and the build pre-compiles both.
"""
from __future__ import annotations

import dataclasses
import importlib

import numpy as np

A = importlib.import_module(__name__.rsplit(".", 1)[0] + ".lang")
f32, i32, i64 = np.float32, np.int32, np.int64

add = lambda a, b: a + b  # noqa: E731


def dotp(xs, ys):
    """foldAll (+) 0 (zipWith (*) xs ys)"""
    return A.fold(add, 0.0, A.zipWith(lambda a, b: a * b, xs, ys))


def prefix_sum(v):
    """scanl (+) 0 v"""
    return A.scanl(add, 0, v)


def histogram(keys, bins=4096):
    """permute (+) (fill bins 0) (\\i -> index1 (keys ! i)) (fill n 1)"""
    return A.permute(add, A.fill(bins, 0, i32), lambda i: keys[i], A.fill(A.shape_of(keys), 1, i32))


def blur(grid, iterate=1):
    """stencil with the 3x3 binomial weights 1/16 [1 2 1; 2 4 2; 1 2 1], Clamp boundary"""
    w = [[0.0625, 0.125, 0.0625], [0.125, 0.25, 0.125], [0.0625, 0.125, 0.0625]]

    def f(t):
        acc = t[0][0] * w[0][0]
        for y in range(3):
            for x in range(3):
                if (y, x) != (0, 0):
                    acc = acc + t[y][x] * w[y][x]
        return acc
    return A.stencil(f, "clamp", grid, iterate=iterate)


def blackscholes(spot, strike, years):
    """map over (spot, strike, years) -> (call, put); r = 0.02, sigma = 0.30; the normal CDF through erf, which the
    reference can only reach as a foreign CUDA function (Foreign/Import.hs:107-111)"""
    def price(s, k, t):
        r, v = 0.02, 0.30
        vsq = v * A.sqrt(t)
        d1 = (A.log(s / k) + (r + 0.5 * v * v) * t) / vsq
        d2 = d1 - vsq
        kexp = k * A.exp(-r * t)
        n1, n2 = 0.5 + 0.5 * A.erf(0.70710678 * d1), 0.5 + 0.5 * A.erf(0.70710678 * d2)
        return s * n1 - kexp * n2, kexp * (1.0 - n2) - s * (1.0 - n1)
    return A.zipWith(price, spot, strike, years)


def row_sums(m):
    """fold (+) 0 m"""
    return A.fold(add, 0.0, m)


def smvm(vals, cols, vec, seglens):
    """foldSeg (+) 0 (zipWith (*) vals (gather cols vec)) seglens"""
    return A.foldSeg(add, 0.0, A.zipWith(lambda v, c: v * vec[c], vals, cols), seglens)


def prefix_sum64(v):
    return A.scanl(add, 0, v)


def smooth(v):
    """rank-1 stencil 1/4 [1 2 1], Clamp"""
    return A.stencil(lambda t: 0.25 * t[0] + 0.5 * t[1] + 0.25 * t[2], "clamp", v)


_specs = None


def generated_specs():
    """{name of the functor in programs.py: the KernelSpec the language prints for the same program}."""
    global _specs
    if _specs is None:
        v = A.vector
        bs = A.specs(blackscholes, v(f32), v(f32), v(f32))[0]
        _specs = {
            "DOT": A.specs(dotp, v(f32), v(f32))[0],
            "SCAN_ADD_I32": A.specs(prefix_sum, v(i32))[0],
            "HIST": A.specs(histogram, v(i32))[1],          # [0] generates the defaults
            "BLUR": A.specs(blur, A.matrix(f32))[0],
            # the hand-written functor is compiled with the fast math library; so is this one
            "BLACKSCHOLES": dataclasses.replace(bs, flags="-use_fast_math"),
            "ROWSUM": A.specs(row_sums, A.matrix(f32))[0],
            "SMVM": A.specs(smvm, v(f32), v(i32), v(f32), v(i32))[1],   # [0] scans the segment lengths
            "SCAN_ADD_I64": A.specs(prefix_sum64, v(i64))[0],
            "SMOOTH1D": A.specs(smooth, v(f32))[0],
            "TRANSPOSE_TILED": A.specs(lambda a: A.transpose(a), A.matrix(f32))[0],  # launched with map_transposed
        }
    return _specs
