"""The CPU oracle against the only known-answer vectors the reference holds
(worked examples in CodeGen/PrefixSum.hs doc comments), against the committed
fixtures, and its C and numpy layers against each other.  No GPU needed."""
import os

import numpy as np
import pytest

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "golden.npz")


@pytest.fixture(scope="module")
def golden():
    return np.load(GOLDEN)


# ---- known-answer vectors from the reference's documentation ----
def test_scanl_doc_example(oracle):
    """scanl (+) 10 (ten ones) ==> [10..20]   (CodeGen/PrefixSum.hs:149-153)"""
    assert oracle.scanl_i32(np.ones(10, np.int32), 10).tolist() == list(range(10, 21))


def test_scanl1_doc_example(oracle):
    """scanl1 (+) (ten ones) ==> [1..10]   (CodeGen/PrefixSum.hs:162-166)"""
    assert oracle.scanl1_i32(np.ones(10, np.int32)).tolist() == list(range(1, 11))


def test_scanl_prime_doc_law(oracle, rng):
    """scanl' f z xs = (init res, last res) where res = scanl f z xs   (CodeGen/PrefixSum.hs:176-180)"""
    x = rng.integers(-100, 100, 1000).astype(np.int32)
    res = oracle.scanl_i32(x, 7)
    body, total = oracle.scanl_prime_i32(x, 7)
    assert np.array_equal(body, res[:-1]) and total == res[-1]


# ---- the C layer against the generic numpy layer ----
@pytest.mark.parametrize("n", [0, 1, 2, 33, 1000])
def test_c_scans_match_generic_scans(oracle, rng, n):
    x = rng.integers(-2**31, 2**31 - 1, n).astype(np.int32)
    add = lambda a, b: int(np.int32(np.uint32((a + b) & 0xffffffff)))
    xs = [int(v) for v in x]
    assert oracle.scanl_i32(x, 3).tolist() == oracle.scan_generic(xs, add, 3, "l", "excl")
    assert oracle.scanr_i32(x, 3).tolist() == oracle.scan_generic(xs, add, 3, "r", "excl")
    assert oracle.scanl1_i32(x).tolist() == oracle.scan_generic(xs, add, None, "l", "incl")
    assert oracle.scanr1_i32(x).tolist() == oracle.scan_generic(xs, add, None, "r", "incl")
    body, tot = oracle.scanr_prime_i32(x, 3)
    gb, gt = oracle.scan_generic(xs, add, 3, "r", "prime")
    assert body.tolist() == gb and tot == gt


def test_right_scan_puts_the_new_element_on_the_left(oracle):
    """Data.List.scanr: out[i] = f(xs[i], out[i+1]); visible with a non-commutative f."""
    sub = lambda a, b: a - b
    assert oracle.scan_generic([1, 2, 3], sub, 0, "r", "excl") == [2, -1, 3, 0]
    assert oracle.scan_generic([1, 2, 3], sub, 0, "l", "excl") == [0, -1, -3, -6]


def test_parallel_scan_equals_sequential(oracle, rng):
    x = rng.integers(0, 16, 1 << 18).astype(np.int32)
    assert np.array_equal(oracle.scanl_i32(x, 5, nthreads=4), oracle.scanl_i32(x, 5))


def test_fold_seed_on_the_right_and_empty_input(oracle):
    """f(acc, seed) (CodeGen/Reduction.hs:203-215); empty input yields the seed (:204-214); fold1 of
    an empty array is a bounds error (Execute.hs:283-285)."""
    sub = lambda a, b: a - b
    assert oracle.fold_generic([10, 1, 2], sub, 100) == (10 - 1 - 2) - 100
    assert oracle.fold_generic([], sub, 42) == 42
    with pytest.raises(IndexError):
        oracle.fold_generic([], sub)


def test_permute_new_value_is_first_argument_and_ignore_is_skipped(oracle):
    """combine x y with y the old value (CodeGen/IndexSpace.hs:203-208); ignore drops the element (:200,229-233)."""
    out = oracle.permute_generic([100, 200], lambda i: [0, -1, 1, 0][i], [1, 2, 3, 4], lambda x, y: x - y)
    assert out == [4 - (1 - 100), 3 - 200]
    keys = np.array([0, 5, -1, 2, 2, 7], np.int32)
    assert oracle.permute_add_i32(keys, 4).tolist() == [1, 0, 2, 0]


@pytest.mark.parametrize("mode,expect", [("clamp", [0, 0, 3, 3]), ("mirror", [1, 2, 2, 1]), ("wrap", [3, 2, 0, 1]),
                                          ("constant", [None, None, None, None])])
def test_boundary_functions(oracle, mode, expect):
    """cclamp / cmirror / cwrap / inRange (CodeGen/Stencil/Extra.hs:191-226) on a size-4 axis at -1, -2, 4, 5."""
    got = [oracle.bound_index(i, 4, mode) for i in (-1, -2, 4, 5)]
    assert got == expect


@pytest.mark.parametrize("mode", ["clamp", "mirror", "wrap", "constant"])
def test_c_stencil_matches_generic_stencil(oracle, workloads, rng, mode):
    a = rng.uniform(0, 1, (6, 7)).astype(np.float32)
    w = workloads.BLUR_WEIGHTS
    fn = lambda nb: sum(w[y][x] * nb[y][x] for y in range(3) for x in range(3))
    assert np.allclose(oracle.stencil2d(a, w, mode, 0.25), oracle.stencil_generic(a, fn, 1, 1, mode, 0.25), rtol=0, atol=1e-15)


def test_iterated_stencil_is_repeated_application_in_double(oracle, workloads, rng):
    a = rng.uniform(0, 1, (9, 11)).astype(np.float32)
    ref = a.astype(np.float64)
    for _ in range(3):
        ref = oracle.stencil2d(ref, workloads.BLUR_WEIGHTS, "clamp")
    assert np.array_equal(oracle.stencil2d_iter(a, workloads.BLUR_WEIGHTS, 3, "clamp"), ref)


def test_blackscholes_put_call_parity(oracle, rng):
    s = rng.uniform(5, 30, 1000).astype(np.float32)
    k = rng.uniform(1, 100, 1000).astype(np.float32)
    t = rng.uniform(0.25, 10, 1000).astype(np.float32)
    c, p = oracle.blackscholes(s, k, t)
    assert np.allclose(c - p, s - k * np.exp(-0.02 * t.astype(np.float64)), rtol=1e-12, atol=1e-12)


# ---- committed fixtures ----
def test_oracle_reproduces_the_committed_fixtures(oracle, workloads, golden):
    g, W = golden, workloads
    x = g["scan_x"]
    assert np.array_equal(x, W.uniform_i32(W.SEED, W.S_SCAN, x.size, 16))
    assert np.array_equal(oracle.scanl_i32(x, 0), g["scanl"])
    assert np.array_equal(oracle.scanl1_i32(x), g["scanl1"])
    assert np.array_equal(oracle.scanr_i32(x, 0), g["scanr"])
    assert np.array_equal(oracle.scanr1_i32(x), g["scanr1"])
    b, t = oracle.scanl_prime_i32(x, 5)
    assert np.array_equal(b, g["scanl_prime_body"]) and t == g["scanl_prime_total"]
    assert oracle.dot_f32(g["dot_xs"], g["dot_ys"]) == float(g["dot"])
    assert np.array_equal(oracle.permute_add_i32(g["hist_keys"], W.HIST_BINS), g["hist"])
    for mode in ("clamp", "mirror", "wrap", "constant"):
        assert np.array_equal(oracle.stencil2d(g["grid"], W.BLUR_WEIGHTS, mode, 0.5), g[f"blur_{mode}"])
    assert np.array_equal(oracle.stencil2d_iter(g["grid"], W.BLUR_WEIGHTS, 10, "clamp"), g["blur_clamp_x10"])
    c, p = oracle.blackscholes(g["bs_spot"], g["bs_strike"], g["bs_years"])
    assert np.allclose(c, g["bs_call"], rtol=1e-13, atol=0) and np.allclose(p, g["bs_put"], rtol=1e-13, atol=1e-15)
    assert np.array_equal(oracle.fold_rows_f32(g["matrix"]), g["rowsum"])


@pytest.mark.parametrize("boundary", ["clamp", "mirror", "wrap", "constant"])
def test_rank3_stencil_oracle_by_padding_equals_the_boundary_functions(oracle, boundary):
    """The padded-array form used at size against the loop over bound_index (Stencil/Extra.hs:200-226), with 27
    different weights so that the orientation of the pattern matters."""
    rng = np.random.default_rng(3)
    a = rng.uniform(-1, 1, (4, 5, 6)).astype(np.float32)
    w = (np.arange(27, dtype=np.float64).reshape(3, 3, 3) + 1) / 378.0
    fn = lambda t: sum(w[z, y, x] * t[z][y][x] for z in range(3) for y in range(3) for x in range(3))  # noqa: E731
    ref = oracle.stencil3d_generic(a, fn, 1, 1, 1, boundary, 0.5)
    assert np.allclose(oracle.stencil3d(a, w, boundary, 0.5), ref, rtol=0, atol=1e-12)
