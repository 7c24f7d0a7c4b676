"""Generates tests/golden/golden.npz: small seeded inputs of every benchmark
configuration with the CPU oracle's outputs.

The reference (accelerate-cuda) cannot run here and ships no fixtures, so these
vectors come from the oracle restatement, not from the reference: they pin the
oracle against accidental change and give the GPU tests a fixed target, but
they do not pin parity with the reference itself.

    python tests/golden/make_golden.py
"""
import importlib
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)
oracle = importlib.import_module("oracle")
W = importlib.import_module("accelerate-cuda_b200.workloads")


def main():
    g = {}
    n = 5003
    x = W.uniform_i32(W.SEED, W.S_SCAN, n, 16)
    g["scan_x"] = x
    g["scanl"] = oracle.scanl_i32(x, 0)
    g["scanl1"] = oracle.scanl1_i32(x)
    b, t = oracle.scanl_prime_i32(x, 5)
    g["scanl_prime_body"], g["scanl_prime_total"] = b, np.int32(t)
    g["scanr"] = oracle.scanr_i32(x, 0)
    g["scanr1"] = oracle.scanr1_i32(x)
    b, t = oracle.scanr_prime_i32(x, 5)
    g["scanr_prime_body"], g["scanr_prime_total"] = b, np.int32(t)

    xs = W.uniform_f32(W.SEED, W.S_XS, 4099, -1, 1)
    ys = W.uniform_f32(W.SEED, W.S_YS, 4099, -1, 1)
    g["dot_xs"], g["dot_ys"], g["dot"] = xs, ys, np.float64(oracle.dot_f32(xs, ys))

    cdf = W.zipf_cdf()
    keys = W.zipf_mix_keys(W.SEED, 30011, cdf)
    g["hist_keys"] = keys
    g["hist"] = oracle.permute_add_i32(keys, W.HIST_BINS)

    grid = W.uniform_f32(W.SEED, W.S_GRID, 48 * 76, 0, 1).reshape(48, 76)
    g["grid"] = grid
    for mode in ("clamp", "mirror", "wrap", "constant"):
        g[f"blur_{mode}"] = oracle.stencil2d(grid, W.BLUR_WEIGHTS, mode, 0.5)
    g["blur_clamp_x10"] = oracle.stencil2d_iter(grid, W.BLUR_WEIGHTS, 10, "clamp")

    s = W.uniform_f32(W.SEED, W.S_SPOT, 2048, 5, 30)
    k = W.uniform_f32(W.SEED, W.S_STRIKE, 2048, 1, 100)
    y = W.uniform_f32(W.SEED, W.S_YEARS, 2048, 0.25, 10)
    c, p = oracle.blackscholes(s, k, y)
    g["bs_spot"], g["bs_strike"], g["bs_years"], g["bs_call"], g["bs_put"] = s, k, y, c, p

    m = W.uniform_f32(W.SEED, W.S_MATRIX, 37 * 2051, -1, 1).reshape(37, 2051)
    g["matrix"], g["rowsum"] = m, oracle.fold_rows_f32(m)

    np.savez_compressed(os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden.npz"), **g)
    print("wrote golden.npz with", len(g), "arrays")


if __name__ == "__main__":
    main()
