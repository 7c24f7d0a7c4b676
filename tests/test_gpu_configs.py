"""Parity at the FULL size of every benchmark configuration, through the C ABI.

Each test runs one configuration at the size it is timed at (dot product 2^24
and 2^28, scanl and scanl' over 2^28 Int32, histogram of 2^28 keys, ten blur
applications on 8192 x 8192, Black-Scholes over 2^26 options, row sums of
16384 x 16384) and compares the whole result with TWO checkers that share no
code:

  * the C oracle (``oracle/accb_oracle.c``, OpenMP over the host's cores), which
    restates the reference's semantics (Execute.hs:326-362 for the scans,
    :396-408 for permute, :413-425 and Stencil/Extra.hs:200-203 for the Clamp
    stencil, Reduction.hs:203-215 for the folds);
  * plain torch operators in float64 / int64 (cumsum, bincount, weighted shifted
    slices of a replicate-padded grid, special.erfc, sum), written here without looking at
    the oracle, so that a misreading shared by oracle and kernels cannot pass.

The inputs come from the device generators; the numpy generator of
``workloads.py`` is compared with them on slices at both ends and in the
middle, so the oracle's input does not rest on the device code alone.

Bit-exact for the integer configurations; |got - ref| <= 1e-5 |ref| + atol for
float32 results against the float64 checkers, atol stated per test.
"""
import os

import numpy as np
import pytest

pytestmark = pytest.mark.gpu

RTOL = 1e-5


def _threads(oracle):
    try:
        cores = len(os.sched_getaffinity(0))
    except AttributeError:
        cores = os.cpu_count() or 1
    return max(1, min(max(oracle.max_threads(), cores), 64))


def _close(got, ref, atol, what):
    got = np.asarray(got, np.float64)
    ref = np.asarray(ref, np.float64)
    excess = np.abs(got - ref) - (RTOL * np.abs(ref) + atol)
    worst = int(np.argmax(excess))
    assert excess.flat[worst] <= 0, f"{what}: |{got.flat[worst]} - {ref.flat[worst]}| exceeds the tolerance at {worst}"


def _same_as_numpy_generator(dev_tensor, host_slice_fn, n):
    """The device generator against the numpy one on three slices of 4096 elements."""
    for first in (0, n // 2 - 2048, n - 4096):
        got = dev_tensor.reshape(-1)[first:first + 4096].cpu().numpy()
        assert np.array_equal(got, host_slice_fn(4096, first)), f"generators differ at {first}"


# ---------------------------------------------------------------- config 1
@pytest.mark.parametrize("log2n", [24, 28])
def test_dot_product_full_size(ctx, P, workloads, oracle, torch_cuda, log2n):
    t, W = torch_cuda, workloads
    n = 1 << log2n
    x = t.empty(n, dtype=t.float32, device="cuda")
    y = t.empty(n, dtype=t.float32, device="cuda")
    ctx.gen_uniform_f32(x, n, 0, W.SEED, W.S_XS, -1.0, 1.0)
    ctx.gen_uniform_f32(y, n, 0, W.SEED, W.S_YS, -1.0, 1.0)
    _same_as_numpy_generator(x, lambda m, f: W.uniform_f32(W.SEED, W.S_XS, m, -1.0, 1.0, f), n)
    out = t.zeros(1, dtype=t.float32, device="cuda")
    ctx.fold_all(P.DOT, [x, y], n, out, seed=np.float32(0))
    ctx.sync()
    got = float(out[0])
    ref = oracle.dot_f32(x.cpu().numpy(), y.cpu().numpy(), nthreads=_threads(oracle))
    second = float((x.double() * y.double()).sum())
    # the sum of 2^28 products of mean zero is small against its terms: one float32 rounding of the result
    # is the floor, plus what float64 accumulation in another order may differ by
    atol = 1e-9 * n ** 0.5
    assert abs(ref - second) <= 1e-9 * abs(ref) + atol, "the two checkers disagree"
    assert abs(got - ref) <= RTOL * abs(ref) + atol, (got, ref)


# ---------------------------------------------------------------- config 2
def test_scanl_and_scanl_prime_full_size(accb, ctx, P, workloads, oracle, torch_cuda):
    t, W = torch_cuda, workloads
    n = W.N28
    x = t.empty(n, dtype=t.int32, device="cuda")
    ctx.gen_uniform_i32(x, n, 0, W.SEED, W.S_SCAN, 16)
    _same_as_numpy_generator(x, lambda m, f: W.uniform_i32(W.SEED, W.S_SCAN, m, 16, f), n)
    ref = t.from_numpy(oracle.scanl_i32(x.cpu().numpy(), 0, nthreads=_threads(oracle))).cuda()
    # second checker: int64 cumulative sum wrapped to 32 bits
    second = t.zeros(n + 1, dtype=t.int64, device="cuda")
    t.cumsum(x, 0, dtype=t.int64, out=second[1:])
    assert t.equal(second.int(), ref), "the two checkers disagree"
    del second
    out = t.empty(n + 1, dtype=t.int32, device="cuda")
    ctx.scan(P.SCAN_ADD_I32, [x], n, out, seed=np.int32(0))
    ctx.sync()
    assert t.equal(out, ref), "scanl differs from the oracle"
    # scanl': the body has n elements, the total is a separate scalar (Execute.hs:352-362)
    out.fill_(-1)
    total = t.full((1,), -1, dtype=t.int32, device="cuda")
    ctx.scan(P.SCAN_ADD_I32, [x], n, out[:n], kind=accb.SCAN_PRIME, seed=np.int32(0), total=total)
    ctx.sync()
    assert t.equal(out[:n], ref[:n]) and int(total[0]) == int(ref[n]), "scanl' differs from the oracle"
    assert int(out[n]) == -1, "scanl' wrote past its n-element body"


# ---------------------------------------------------------------- config 3
def test_histogram_full_size(ctx, P, workloads, oracle, torch_cuda):
    t, W = torch_cuda, workloads
    n = W.N28
    cdf = W.zipf_cdf()
    keys = t.empty(n, dtype=t.int32, device="cuda")
    ctx.gen_zipf_mix_i32(keys, n, 0, W.SEED, t.from_numpy(cdf).cuda(), W.HIST_BINS)
    _same_as_numpy_generator(keys, lambda m, f: W.zipf_mix_keys(W.SEED, m, cdf, f), n)
    out = t.full((W.HIST_BINS,), 12345, dtype=t.int32, device="cuda")
    ctx.permute(P.HIST, [keys], n, out, defaults=t.zeros(W.HIST_BINS, dtype=t.int32, device="cuda"))
    ctx.sync()
    ref = oracle.permute_add_i32(keys.cpu().numpy(), W.HIST_BINS, nthreads=_threads(oracle))
    second = t.bincount(keys.long(), minlength=W.HIST_BINS).int().cpu().numpy()
    assert np.array_equal(ref, second), "the two checkers disagree"
    got = out.cpu().numpy()
    assert np.array_equal(got, ref) and int(got.astype(np.int64).sum()) == n


# ---------------------------------------------------------------- config 4
def test_ten_blur_applications_full_size(ctx, P, workloads, oracle, torch_cuda):
    t, W = torch_cuda, workloads
    h = w = 8192
    src = t.empty((h, w), dtype=t.float32, device="cuda")
    ctx.gen_uniform_f32(src, h * w, 0, W.SEED, W.S_GRID, 0.0, 1.0)
    _same_as_numpy_generator(src, lambda m, f: W.uniform_f32(W.SEED, W.S_GRID, m, 0.0, 1.0, f), h * w)
    a, b = t.empty_like(src), t.empty_like(src)
    ctx.stencil(P.BLUR, src, a, boundary="clamp")
    res = ctx.stencil_iterate(P.BLUR, a, b, 9, boundary="clamp")
    ctx.sync()
    # oracle: the same ten-step recurrence with its state in float64
    ref = oracle.stencil2d_iter(src.cpu().numpy(), W.BLUR_WEIGHTS, 10, "clamp", nthreads=_threads(oracle))
    # second checker: float64 weighted sum of shifted views of a grid padded by replicating its edge (Clamp moves every
    # out-of-range coordinate to the nearest valid one, Stencil/Extra.hs:200-203)
    F = t.nn.functional
    wts = [[1.0, 2.0, 1.0], [2.0, 4.0, 2.0], [1.0, 2.0, 1.0]]
    cur = src.double().reshape(1, 1, h, w)
    for _ in range(10):
        pad = F.pad(cur, (1, 1, 1, 1), mode="replicate")
        cur = t.zeros_like(cur)
        for dy in range(3):
            for dx in range(3):
                cur += (wts[dy][dx] / 16.0) * pad[:, :, dy:dy + h, dx:dx + w]
        del pad
    second = cur.reshape(h, w).cpu().numpy()
    del cur
    assert np.max(np.abs(ref - second)) <= 1e-12, "the two checkers disagree"
    _close(res.cpu().numpy(), ref, 1e-6, "10 x blur")


# --------------------------------------------------------------- config 5a
def test_black_scholes_full_size(ctx, P, workloads, oracle, torch_cuda):
    t, W = torch_cuda, workloads
    n = W.N26
    mk = lambda: t.empty(n, dtype=t.float32, device="cuda")  # noqa: E731
    s, k, y, call, put = mk(), mk(), mk(), mk(), mk()
    ctx.gen_uniform_f32(s, n, 0, W.SEED, W.S_SPOT, 5.0, 30.0)
    ctx.gen_uniform_f32(k, n, 0, W.SEED, W.S_STRIKE, 1.0, 100.0)
    ctx.gen_uniform_f32(y, n, 0, W.SEED, W.S_YEARS, 0.25, 10.0)
    _same_as_numpy_generator(k, lambda m, f: W.uniform_f32(W.SEED, W.S_STRIKE, m, 1.0, 100.0, f), n)
    ctx.map(P.BLACKSCHOLES, [(s, k, y)], (call, put))
    ctx.sync()
    rc, rp = oracle.blackscholes(s.cpu().numpy(), k.cpu().numpy(), y.cpu().numpy(), nthreads=_threads(oracle))
    # second checker: the closed form in float64 torch operators
    S, K, T = s.double(), k.double(), y.double()
    r, v = 0.02, 0.30
    d1 = (t.log(S / K) + (r + 0.5 * v * v) * T) / (v * t.sqrt(T))
    d2 = d1 - v * t.sqrt(T)
    cnd = lambda d: 0.5 * t.special.erfc(-d / 2.0 ** 0.5)  # noqa: E731
    kexp = K * t.exp(-r * T)
    c2 = (S * cnd(d1) - kexp * cnd(d2)).cpu().numpy()
    p2 = (kexp * cnd(-d2) - S * cnd(-d1)).cpu().numpy()
    assert np.max(np.abs(rc - c2)) <= 1e-9 and np.max(np.abs(rp - p2)) <= 1e-9, "the two checkers disagree"
    # prices reach 100; float32 rounding of d1 alone moves them by ~1e-5
    _close(call.cpu().numpy(), rc, 2e-5, "call")
    _close(put.cpu().numpy(), rp, 2e-5, "put")


# --------------------------------------------------------------- config 5b
def test_row_sums_full_size(ctx, P, workloads, oracle, torch_cuda):
    t, W = torch_cuda, workloads
    rows = cols = 16384
    m = t.empty((rows, cols), dtype=t.float32, device="cuda")
    ctx.gen_uniform_f32(m, rows * cols, 0, W.SEED, W.S_MATRIX, -1.0, 1.0)
    _same_as_numpy_generator(m, lambda k, f: W.uniform_f32(W.SEED, W.S_MATRIX, k, -1.0, 1.0, f), rows * cols)
    out = t.zeros(rows, dtype=t.float32, device="cuda")
    ctx.fold_dim(P.ROWSUM, [m], rows, cols, out, seed=np.float32(0))
    ctx.sync()
    ref = oracle.fold_rows_f32(m.cpu().numpy(), nthreads=_threads(oracle))
    second = m.double().sum(dim=1).cpu().numpy()
    assert np.max(np.abs(ref - second)) <= 1e-9, "the two checkers disagree"
    # a row of 16384 terms of mean zero sums to ~74; a sum near zero keeps one float32 rounding of a term-sized value
    _close(out.cpu().numpy(), ref, 1e-6, "row sums")
