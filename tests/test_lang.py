"""The embedded array language (accelerate-cuda_b200/lang.py): what it prints (no device needed), that
what it prints compiles for sm_100a, and -- on a GPU -- that whole programs written like Accelerate programs
compute what numpy computes."""
import ctypes as C
import importlib

import numpy as np
import pytest

A = importlib.import_module("accelerate-cuda_b200.lang")
f32, f64, i32, i64, u32 = np.float32, np.float64, np.int32, np.int64, np.uint32

add = lambda a, b: a + b  # noqa: E731


# ------------------------------------------------------------------ programs shared by the tests
def dotp(xs, ys):
    return A.fold(add, 0.0, A.zipWith(lambda a, b: a * b, xs, ys))


def histogram(keys):
    return A.permute(add, A.fill(4096, 0, i32), lambda i: keys[i], A.fill(A.shape_of(keys), 1, i32))


def blur(g):
    w = [[1, 2, 1], [2, 4, 2], [1, 2, 1]]
    return A.stencil(lambda t: sum((t[y][x] * (w[y][x] / 16.0) for y in range(3) for x in range(3)), A.constant(0, f32)),
                     "clamp", g)


def blackscholes(spot, strike, years):
    def price(s, k, t):
        r, v = 0.02, 0.30
        vsq = v * A.sqrt(t)
        d1 = (A.log(s / k) + (r + 0.5 * v * v) * t) / vsq
        d2 = d1 - vsq
        cnd = lambda d: 0.5 + 0.5 * A.erf(0.70710678 * d)  # noqa: E731
        kexp = k * A.exp(-r * t)
        return s * cnd(d1) - kexp * cnd(d2), kexp * (1.0 - cnd(d2)) - s * (1.0 - cnd(d1))
    return A.zipWith(price, spot, strike, years)


def smvm(vals, cols, vec, seglens):
    return A.foldSeg(add, 0.0, A.zipWith(lambda v, c: v * vec[c], vals, cols), seglens)


def argmax(xs):
    pairs = A.generate(A.shape_of(xs), lambda i: (xs[i], i))
    return A.fold1(lambda a, b: A.cond((b[0] > a[0]) | ((b[0] == a[0]) & (b[1] < a[1])), b, a), pairs)


# ------------------------------------------------------------------ what is printed (CPU)
def test_a_fold_over_a_zipwith_is_one_kernel_reading_both_vectors_elementwise():
    specs = A.specs(dotp, A.vector(f32), A.vector(f32))
    assert [s.skeleton for s in specs] == ["fold_all"]
    src = specs[0].source
    assert "using In = accb::types<float, float>;" in src and "in0 * in1" in src
    assert "accb::Fold<float, double>" in src  # a recognised (+) on Float accumulates in double


def test_fill_sources_cost_no_traffic_and_the_combiner_picks_the_atomic():
    specs = A.specs(histogram, A.vector(i32))
    assert [s.skeleton for s in specs] == ["map", "permute_smem"]  # the defaults are generated, the ones are fused
    src = specs[1].source
    assert "accb::Atomic::Add" in src and "using In = accb::types<int>;" in src and "identity()" in src
    mx = A.specs(lambda k, v: A.permute(A.maximum, A.fill(16, 0.0, f32), lambda i: k[i], v), A.vector(i32), A.vector(f32))
    assert "accb::Atomic::Cas" in mx[-1].source and mx[-1].skeleton == "permute"
    last = A.specs(lambda k, v: A.permute(lambda x, y: x, A.fill(16, 0, i32), lambda i: k[i], v), A.vector(i32), A.vector(i32))
    assert "accb::Atomic::None" in last[-1].source


def test_integer_arithmetic_follows_the_reference_c_forms():
    def f(x):
        return A.map(lambda a: (a // 3, a % 3, A.quot(a, 3), A.rem(a, 3), -a, abs(a), a << 2), x)
    src = A.specs(f, A.vector(i32))[0].source
    for piece in ["accb::idiv<int>(in0, 3)", "accb::imod<int>(in0, 3)", "in0 / 3", "in0 % 3",
                  "(int)(0 - (unsigned int)in0)", "(int)(in0 << 2)"]:
        assert piece in src, piece
    g = A.specs(lambda x: A.map(lambda a: (A.round_(a), A.floor(a), A.minimum(a, 2.0), a ** 2.0), x), A.vector(f32))[0].source
    for piece in ["(int)roundf(in0)", "(int)floorf(in0)", "fminf(in0, 2.0f)", "powf(in0, 2.0f)"]:
        assert piece in g, piece


def test_cube_stencil_functors_declare_the_taps_they_read():
    """The functor printed for a rank-3 stencil carries `uses`: true exactly for the taps the function reads, so
    that the skeleton can skip the rows and halo columns nobody reads."""
    seven = lambda t: (t[0][1][1] + t[2][1][1] + t[1][0][1] + t[1][2][1] + t[1][1][0] + t[1][1][2]) - 6.0 * t[1][1][1]  # noqa: E731
    spec = A.specs(lambda a: A.stencil(seven, "clamp", a), A.array(3, f32))[0]
    assert spec.skeleton == "stencil3" and "static constexpr bool uses(int z, int y, int x)" in spec.source
    table = spec.source.split("constexpr bool read[3][3][3] = ")[1].split(";")[0]
    assert table.count("true") == 7 and table.count("false") == 20
    flat = [w == "true" for w in table.replace("{", " ").replace("}", " ").replace(",", " ").split()]
    assert [i for i, u in enumerate(flat) if u] == [4, 10, 12, 13, 14, 16, 22]  # (z * 3 + y) * 3 + x
    every = lambda t: sum((t[z][y][x] for z in range(3) for y in range(3) for x in range(3)), A.constant(0, f32))  # noqa: E731
    full = A.specs(lambda a: A.stencil(every, "clamp", a), A.array(3, f32))[0].source
    assert full.split("constexpr bool read[3][3][3] = ")[1].split(";")[0].count("false") == 0


def test_the_language_is_typed_like_accelerate():
    with pytest.raises(TypeError):
        A.specs(lambda x, y: A.zipWith(add, x, y), A.vector(f32), A.vector(i32))  # Float + Int
    with pytest.raises(TypeError):
        A.specs(lambda x: A.map(lambda a: a + 0.5, x), A.vector(i32))  # fractional literal at Int
    with pytest.raises(TypeError):
        A.specs(lambda x: A.map(lambda a: a / 2, x), A.vector(i32))  # (/) on Int
    with pytest.raises(TypeError):
        A.specs(lambda x: A.map(lambda a: 1 if a > 0 else 0, x), A.vector(i32))  # Python `if` on an Exp
    ok = A.specs(lambda x, y: A.zipWith(lambda a, b: a + A.fromIntegral(b, f32), x, y), A.vector(f32), A.vector(i32))
    assert "(float)in1" in ok[0].source


def test_backpermute_is_a_gather_and_indices_are_row_major():
    src = A.specs(lambda m: A.backpermute((4, 6), lambda ix: (ix[1], ix[0]), m), A.matrix(f32))[0].source
    assert "using In = accb::types<>;" in src and "env.in<float>(0)" in src
    assert "accb::from_index2(6, i," in src and "* env.dim(0, 0) +" in src


def test_an_array_read_at_its_own_index_and_elsewhere_appears_twice():
    f = lambda v: A.generate(A.shape_of(v), lambda i: v[i] - v[A.maximum(i - 1, 0)])  # noqa: E731
    src = A.specs(f, A.vector(i32))[0].source
    assert "using In = accb::types<int>;" in src and "env.in<int>(1)" in src


def test_tuples_become_structs_with_soa_outputs():
    specs = A.specs(argmax, A.vector(f32))
    assert [s.skeleton for s in specs] == ["fold_all"]
    src = specs[0].source
    assert "struct E { float c0; int c1; };" in src and "using Out = accb::types<float, int>;" in src
    assert "void put(E r, float &o0, int &o1)" in src


def test_segments_are_lengths_scanned_to_offsets_as_in_the_reference():
    specs = A.specs(smvm, A.vector(f32), A.vector(i32), A.vector(f32), A.vector(i32))
    assert [s.skeleton for s in specs] == ["scan", "fold_seg"]
    assert "using In = accb::types<float, int>;" in specs[1].source and "env.in<float>(2)" in specs[1].source


def test_row_scans_and_segmented_scans_are_scans_of_value_flag_pairs():
    """What the reference rejects (PrefixSum.hs:39-46): the scan skeleton over (value, restart flag)."""
    rows = A.specs(lambda m: A.scanl1(add, m), A.matrix(i32))
    assert [s.skeleton for s in rows] == ["scan"]
    src = rows[0].source
    assert "struct E { int c0; unsigned char c1; };" in src and "using Out = accb::types<int>;" in src
    assert "accb::from_index2(" in src  # the flag is "first column", from the index
    seg = A.specs(lambda v, lens: A.scanl1Seg(add, v, lens), A.vector(f32), A.vector(i32))
    assert [s.skeleton for s in seg] == ["scan", "map", "permute", "scan"]  # offsets, cleared flags, heads, the scan
    assert "accb::Atomic::None" in seg[2].source and "using In = accb::types<float, unsigned char>;" in seg[3].source


def mvm(mat, vec):
    """matrix x vector the Accelerate way: replicate the vector over the rows, zip, fold the rows"""
    return A.fold(add, 0.0, A.zipWith(lambda a, b: a * b, mat, A.replicate(vec, A.dim(mat, 0), axis=0)))


def test_shapes_computed_from_other_arrays():
    specs = A.specs(mvm, A.matrix(f32), A.vector(f32))
    assert [s.skeleton for s in specs] == ["fold_dim"]  # replicate is fused: the matrix element-wise, the vector gathered
    assert "using In = accb::types<float>;" in specs[0].source and "env.in<float>(1)" in specs[0].source
    t = A.specs(lambda m: A.transpose(m), A.matrix(i32))
    # a transpose made manifest is the plain map functor launched over shared-memory tiles, not a gather
    assert [s.skeleton for s in t] == ["map"] and "using In = accb::types<int>;" in t[0].source
    g = A.specs(lambda m: A.fold(add, 0, A.transpose(m)), A.matrix(i32))  # column sums: tiled transpose, then row sums
    assert [s.skeleton for s in g] == ["map", "fold_dim"]
    r = A.specs(lambda m: A.map(lambda x: x + 1, A.reshape((A.dim(m, 1), A.dim(m, 0)), m)), A.matrix(i32))
    assert "using In = accb::types<int>;" in r[0].source  # same row-major position: still element-wise
    ex = A.specs(lambda m: A.scanl(add, 0, m), A.matrix(i32))
    assert [s.skeleton for s in ex] == ["map", "scan"]  # rows widened by the seed, then the row scan


def test_everything_printed_compiles_for_sm_100a(accb):
    """nvcc -arch=sm_100a on a sample of generated functors (no device needed)."""
    import os
    import tempfile
    lib = accb.lib()
    programs = [
        (dotp, [A.vector(f32), A.vector(f32)]), (histogram, [A.vector(i32)]), (blur, [A.matrix(f32)]),
        (blackscholes, [A.vector(f32)] * 3), (smvm, [A.vector(f32), A.vector(i32), A.vector(f32), A.vector(i32)]),
        (argmax, [A.vector(f32)]),
        (lambda m: A.backpermute((4, 6), lambda ix: (ix[1], ix[0]), m), [A.matrix(f32)]),
        (lambda a, b: A.stencil2(lambda s, t: s[1][1] + 0.5 * (t[0][1] + t[2][1]), ("constant", 0.0), a, b),
         [A.matrix(f32), A.matrix(f32)]),
        (lambda ab: A.scanl1(lambda f, g: (g[0] * f[0], g[0] * f[1] + g[1]), ab), [A.vector(u32, u32)]),
        (lambda x: A.map(lambda a: (a // 3, a % 3, A.cast(a, i64) * 5, A.cast(a, f64) / 3.0, a > 2), x), [A.vector(i32)]),
        (lambda m: A.scanr1(add, m), [A.matrix(f32)]),
        (mvm, [A.matrix(f32), A.vector(f32)]), (lambda m: A.scanr(A.maximum, 0, m), [A.matrix(i32)]),
        (lambda m: (A.transpose(m), A.slice(m, 0, 2), A.reshape((A.dim(m, 1), A.dim(m, 0)), m)), [A.matrix(i32)]),
        (lambda v: (A.reverse(v), A.init(v), A.tail(v), A.take(3, v), A.drop(2, v), A.enumFromN(A.dim(v, 0), 5)), [A.vector(i32)]),
        (lambda v, lens: A.scanl1Seg(add, v, lens), [A.vector(f32), A.vector(i32)]),
        (lambda v, lens: A.scanr1Seg(A.maximum, v, lens), [A.vector(i64), A.vector(i32)]),
        (lambda k, v: A.permute(lambda x, y: (x[0] + y[0], x[1] + y[1]), A.zip(A.fill(64, 0, i32), A.fill(64, 0, i32)),
                                lambda i: k[i], A.zip(v, A.fill(A.shape_of(v), 1, i32))),
         [A.vector(i32), A.vector(i32)]),
    ]
    specs = {}
    for f, ts in programs:
        for s in A.specs(f, *ts):
            specs[s.functor] = s
    from concurrent.futures import ThreadPoolExecutor
    with tempfile.TemporaryDirectory() as cache:
        def one(s):
            log = C.create_string_buffer(1 << 16)
            st = lib.accb_kernel_precompile(s.skeleton.encode(), s.source.encode(), s.functor.encode(), None,
                                            cache.encode(), log, len(log))
            return st, s, log.value.decode(errors="replace")
        with ThreadPoolExecutor(max_workers=os.cpu_count() or 4) as ex:
            for st, s, log in ex.map(one, specs.values()):
                assert st == 0, f"{s.skeleton} {s.functor}:\n{s.source}\n{log}"


# ------------------------------------------------------------------ whole programs on a GPU
def close(got, ref, atol, rtol=1e-5):
    got, ref = np.asarray(got, f64), np.asarray(ref, f64)
    assert np.all(np.abs(got - ref) <= rtol * np.abs(ref) + atol), float(np.max(np.abs(got - ref)))


@pytest.mark.gpu
def test_dot_product_and_row_sums(ctx, rng):
    x, y = rng.uniform(-1, 1, 300001).astype(f32), rng.uniform(-1, 1, 300001).astype(f32)
    close(A.runWith(ctx, dotp, x, y), np.dot(x.astype(f64), y.astype(f64)), 1e-6)
    m = rng.uniform(-1, 1, (700, 1300)).astype(f32)
    close(A.runWith(ctx, lambda a: A.fold(add, 0.0, a), m), m.astype(f64).sum(axis=1), 1e-6)
    close(A.runWith(ctx, lambda a: A.foldAll(A.maximum, -1e30, a), m), m.max(), 0)
    with pytest.raises(ValueError):
        A.runWith(ctx, dotp, x, y[:-1])  # zipped arrays of different length


@pytest.mark.gpu
def test_the_six_scans(ctx, rng):
    x = rng.integers(-100, 100, 100003).astype(i32)
    c = np.cumsum(x.astype(i64)).astype(i32)
    assert np.array_equal(A.runWith(ctx, lambda v: A.scanl(add, 7, v), x), np.concatenate([[7], c + 7]).astype(i32))
    assert np.array_equal(A.runWith(ctx, lambda v: A.scanl1(add, v), x), c)
    body, tot = A.runWith(ctx, lambda v: A.scanl_(add, 0, v), x)
    assert np.array_equal(body, np.concatenate([[0], c[:-1]]).astype(i32)) and tot == c[-1]
    r = np.cumsum(x[::-1].astype(i64))[::-1].astype(i32)
    assert np.array_equal(A.runWith(ctx, lambda v: A.scanr1(add, v), x), r)
    assert np.array_equal(A.runWith(ctx, lambda v: A.scanr(add, 0, v), x), np.concatenate([r, [0]]).astype(i32))
    body, tot = A.runWith(ctx, lambda v: A.scanr_(add, 0, v), x)
    assert np.array_equal(body, np.concatenate([r[1:], [0]]).astype(i32)) and tot == r[0]
    # a scan over a fused producer and a non-commutative tuple combiner (composition of affine maps)
    a, b = rng.integers(1, 5, 5000).astype(u32), rng.integers(0, 9, 5000).astype(u32)
    ga, gb = A.runWith(ctx, lambda ab: A.scanl1(lambda f, g: (g[0] * f[0], g[0] * f[1] + g[1]), ab), (a, b))
    ra, rb = np.empty_like(a), np.empty_like(b)
    fa, fb = np.uint32(1), np.uint32(0)
    with np.errstate(over="ignore"):
        for i in range(a.size):
            fa, fb = a[i] * fa, a[i] * fb + b[i]
            ra[i], rb[i] = fa, fb
    assert np.array_equal(ga, ra) and np.array_equal(gb, rb)


@pytest.mark.gpu
def test_scans_along_rows_and_inside_segments(ctx, rng):
    m = rng.integers(-100, 100, (300, 1237)).astype(i32)
    assert np.array_equal(A.runWith(ctx, lambda a: A.scanl1(add, a), m), np.cumsum(m, axis=1, dtype=i64).astype(i32))
    assert np.array_equal(A.runWith(ctx, lambda a: A.scanr1(add, a), m),
                          np.cumsum(m[:, ::-1], axis=1, dtype=i64)[:, ::-1].astype(i32))
    wide = rng.integers(-9, 9, (3, 40000)).astype(i32)  # rows longer than a tile: the restart crosses tiles
    assert np.array_equal(A.runWith(ctx, lambda a: A.scanl1(A.maximum, a), wide), np.maximum.accumulate(wide, axis=1))
    lens = rng.integers(0, 50, 4000).astype(i32)
    lens[100:140] = 0
    lens[7] = 30000
    v = rng.uniform(-1, 1, int(lens.sum())).astype(f32)
    offs = np.concatenate([[0], np.cumsum(lens)])
    refl, refr = np.empty_like(v, dtype=f64), np.empty_like(v, dtype=f64)
    for s in range(lens.size):
        seg = v[offs[s]:offs[s + 1]].astype(f64)
        refl[offs[s]:offs[s + 1]] = np.cumsum(seg)
        refr[offs[s]:offs[s + 1]] = np.cumsum(seg[::-1])[::-1]
    close(A.runWith(ctx, lambda a, l: A.scanl1Seg(add, a, l), v, lens), refl, 2e-3)  # float32 sums of up to 30000 terms
    close(A.runWith(ctx, lambda a, l: A.scanr1Seg(add, a, l), v, lens), refr, 2e-3)
    # scanl'Seg / scanr'Seg: the exclusive scan inside every segment plus one total per segment (empty ones: the seed)
    w = rng.integers(-100, 100, int(lens.sum())).astype(i32)
    exl, exr, tot = np.empty_like(w), np.empty_like(w), np.empty(lens.size, i32)
    for s in range(lens.size):
        seg = w[offs[s]:offs[s + 1]].astype(i64)
        exl[offs[s]:offs[s + 1]] = 5 + np.concatenate([[0], np.cumsum(seg)])[:seg.size]
        exr[offs[s]:offs[s + 1]] = 5 + np.concatenate([np.cumsum(seg[::-1])[::-1], [0]])[1:]
        tot[s] = 5 + seg.sum()
    body, totals = A.runWith(ctx, lambda a, l: A.scanl_Seg(add, 5, a, l), w, lens)
    assert np.array_equal(body, exl) and np.array_equal(totals, tot)
    body, totals = A.runWith(ctx, lambda a, l: A.scanr_Seg(add, 5, a, l), w, lens)
    assert np.array_equal(body, exr) and np.array_equal(totals, tot)
    # scanlSeg / scanrSeg: every segment one element longer, the seed first (last); length = data + segments
    refl, refr = [], []
    for s in range(lens.size):
        seg = w[offs[s]:offs[s + 1]].astype(i64)
        refl.append(5 + np.concatenate([[0], np.cumsum(seg)]))
        refr.append(5 + np.concatenate([np.cumsum(seg[::-1])[::-1], [0]]))
    assert np.array_equal(A.runWith(ctx, lambda a, l: A.scanlSeg(add, 5, a, l), w, lens), np.concatenate(refl).astype(i32))
    assert np.array_equal(A.runWith(ctx, lambda a, l: A.scanrSeg(add, 5, a, l), w, lens), np.concatenate(refr).astype(i32))
    # (++): the extent of the result is the sum of two arrays' extents
    assert np.array_equal(A.runWith(ctx, lambda a, b: A.concat(A.map(lambda e: e + 1, a), b), w, lens),
                          np.concatenate([w + 1, lens]))


@pytest.mark.gpu
def test_every_scalar_operator_against_numpy(ctx, rng):
    """The C forms of CodeGen/Arithmetic.hs, operator by operator, on negative and positive operands."""
    a = rng.integers(-1000, 1000, 4096).astype(i32)
    b = rng.integers(1, 50, 4096).astype(i32) * rng.choice([-1, 1], 4096).astype(i32)
    with np.errstate(over="ignore"):
        got = A.runWith(ctx, lambda x, y: A.zipWith(lambda p, q: (p + q, p - q, p * q, p // q, p % q, A.quot(p, q), A.rem(p, q), -p), x, y), a, b)
        tq = np.trunc(a / b).astype(i32)
        for g, r in zip(got, [a + b, a - b, a * b, a // b, a % b, tq, a - tq * b, -a]):
            assert np.array_equal(g, r)
        got = A.runWith(ctx, lambda x, y: A.zipWith(lambda p, q: (abs(p), A.signum(p), A.minimum(p, q), A.maximum(p, q), p & q, p | q, p ^ q, ~p), x, y), a, b)
        for g, r in zip(got, [np.abs(a), np.sign(a), np.minimum(a, b), np.maximum(a, b), a & b, a | b, a ^ b, ~a]):
            assert np.array_equal(g, r)
        got = A.runWith(ctx, lambda x, y: A.zipWith(lambda p, q: (p << 3, p >> 2, p < q, p <= q, p == q, p != q, (p > 0) & (q > 0), (p > 0) | ~(q > 0)), x, y), a, b)
        for g, r in zip(got, [a << 3, a >> 2, a < b, a <= b, a == b, a != b, (a > 0) & (b > 0), (a > 0) | ~(b > 0)]):
            assert np.array_equal(g.astype(r.dtype), r)
        # wrapping: Int32 arithmetic is modulo 2^32, unsigned division and shifts are logical
        big = rng.integers(-2**31, 2**31 - 1, 4096).astype(i32)
        w1, w2 = A.runWith(ctx, lambda x: A.map(lambda p: (p * p + p, A.cast(A.cast(p, u32) >> 1, i32)), x), big)
        assert np.array_equal(w1, big * big + big) and np.array_equal(w2, (big.astype(u32) >> 1).astype(i32))
    x = rng.uniform(-4, 4, 4096).astype(f32)
    y = rng.uniform(0.1, 4, 4096).astype(f32)
    got = A.runWith(ctx, lambda p, q: A.zipWith(lambda s, t: (s / t, s ** 2.0, A.sqrt(t), A.exp(s), A.log(t), A.sin(s), A.cos(s), A.atan2(s, t)), p, q), x, y)
    for g, r in zip(got, [x / y, x ** 2, np.sqrt(y), np.exp(x), np.log(y), np.sin(x), np.cos(x), np.arctan2(x, y)]):
        close(g, r.astype(f64), 1e-6, rtol=2e-6)
    got = A.runWith(ctx, lambda p: A.map(lambda s: (A.floor(s), A.ceiling(s), A.round_(s), A.truncate(s), abs(s), A.signum(s), A.tanh(s), A.isnan(s / s)), p),
                    np.concatenate([x, np.array([0.0, 0.5, 1.5, 2.5, -0.5, -1.5, -2.5], f32)]))
    xx = np.concatenate([x, np.array([0.0, 0.5, 1.5, 2.5, -0.5, -1.5, -2.5], f32)])
    half_away = np.where(xx >= 0, np.floor(xx + 0.5), np.ceil(xx - 0.5)).astype(i32)  # C round, not banker's
    with np.errstate(invalid="ignore"):
        refs = [np.floor(xx).astype(i32), np.ceil(xx).astype(i32), half_away, np.trunc(xx).astype(i32), np.abs(xx), np.sign(xx), np.tanh(xx), np.isnan(xx / xx)]
    for k, (g, r) in enumerate(zip(got, refs)):
        if r.dtype.kind == "f":
            close(g, r.astype(f64), 1e-6, rtol=2e-6)
        else:
            assert np.array_equal(g.astype(r.dtype), r), k
    # conversions and double precision
    d = A.runWith(ctx, lambda p: A.map(lambda s: (A.cast(s, f64) * 1.0000000001, A.cast(A.cast(s, f64) * 1e10, i64), A.cond(s > 0.0, A.toFloating(A.floor(s), f32), s)), p), x)
    assert np.array_equal(d[0], x.astype(f64) * 1.0000000001) and np.array_equal(d[1], (x.astype(f64) * 1e10).astype(i64))
    assert np.array_equal(d[2], np.where(x > 0, np.floor(x), x))


@pytest.mark.gpu
def test_replicate_slice_reshape_and_friends(ctx, rng):
    m = rng.uniform(-1, 1, (301, 517)).astype(f32)
    v = rng.uniform(-1, 1, 517).astype(f32)
    close(A.runWith(ctx, mvm, m, v), m.astype(f64) @ v.astype(f64), 1e-5)
    with pytest.raises(ValueError):
        A.runWith(ctx, mvm, m, v[:-1])
    mi = rng.integers(-99, 99, (37, 53)).astype(i32)
    t, row, col, rs = A.runWith(ctx, lambda a: (A.transpose(a), A.slice(a, 0, 5), A.slice(a, 1, 7),
                                                A.reshape((A.dim(a, 1), A.dim(a, 0)), a)), mi)
    assert np.array_equal(t, mi.T) and np.array_equal(row, mi[5]) and np.array_equal(col, mi[:, 7])
    assert np.array_equal(rs, mi.reshape(53, 37))
    x = rng.integers(-99, 99, 10001).astype(i32)
    rv, ini, tl, tk, dr, en = A.runWith(ctx, lambda a: (A.reverse(a), A.init(a), A.tail(a), A.take(3, a), A.drop(2, a),
                                                        A.enumFromN(A.dim(a, 0), 5)), x)
    assert np.array_equal(rv, x[::-1]) and np.array_equal(ini, x[:-1]) and np.array_equal(tl, x[1:])
    assert np.array_equal(tk, x[:3]) and np.array_equal(dr, x[2:]) and np.array_equal(en, np.arange(5, 5 + x.size, dtype=i32))
    for shp in [(1, 1), (33, 1000), (1025, 257)]:  # tiled transposes: maps and zips over them, wide and tuple elements
        a, b = rng.uniform(-1, 1, shp), rng.integers(-9, 9, shp).astype(i32)
        t1, t2, t3 = A.runWith(ctx, lambda p, q: (A.map(lambda e: e * 2.0, A.transpose(p)),
                                                  A.zipWith(lambda e, k: e + A.cast(k, f64), A.transpose(p), A.transpose(q)),
                                                  A.transpose(A.compute(A.zip(p, q)))), a, b)
        assert np.array_equal(t1, 2 * a.T) and np.array_equal(t2, a.T + b.T)
        assert np.array_equal(t3[0], a.T) and np.array_equal(t3[1], b.T)
    rep = A.runWith(ctx, lambda a: A.replicate(a, 4, axis=1), x[:9])
    assert np.array_equal(rep, np.repeat(x[:9, None], 4, axis=1))
    # exclusive scans along rows: one element longer per row, seed first (scanl) or last (scanr)
    ex = A.runWith(ctx, lambda a: A.scanl(add, 10, a), mi)
    assert np.array_equal(ex, np.concatenate([np.full((37, 1), 10), 10 + np.cumsum(mi, axis=1)], axis=1).astype(i32))
    er = A.runWith(ctx, lambda a: A.scanr(add, 10, a), mi)
    assert np.array_equal(er, np.concatenate([10 + np.cumsum(mi[:, ::-1], axis=1)[:, ::-1], np.full((37, 1), 10)], axis=1).astype(i32))


@pytest.mark.gpu
def test_histogram_and_scatter_with_ignore(ctx, rng):
    keys = rng.integers(0, 4096, 200000).astype(i32)
    assert np.array_equal(A.runWith(ctx, histogram, keys), np.bincount(keys, minlength=4096).astype(i32))
    vals = rng.uniform(0, 1, keys.size).astype(f32)
    got = A.runWith(ctx, lambda k, v: A.permute(A.maximum, A.fill(4096, -1.0, f32),
                                                lambda i: A.cond_index(k[i] % 2 == 0, k[i]), v), keys, vals)
    ref = np.full(4096, -1.0, f32)
    even = keys % 2 == 0
    np.maximum.at(ref, keys[even], vals[even])
    assert np.array_equal(got, ref)
    # stream compaction (the core of `filter`): kept elements in order at the front, and how many there are
    front, count = A.runWith(ctx, lambda v: A.compact(lambda e: e > 0.5, v), vals)
    kept = vals[vals > 0.5]
    assert int(count) == kept.size and np.array_equal(front[:kept.size], kept) and not front[kept.size:].any()
    pairs, count = A.runWith(ctx, lambda kv: A.compact(lambda e: e[0] % 3 == 0, kv), (keys, vals))
    sel = keys % 3 == 0
    assert int(count) == sel.sum() and np.array_equal(pairs[0][:sel.sum()], keys[sel]) and np.array_equal(pairs[1][:sel.sum()], vals[sel])


@pytest.mark.gpu
@pytest.mark.parametrize("boundary", ["clamp", "mirror", "wrap", ("constant", 0.5)])
def test_stencils(ctx, oracle, rng, boundary):
    g = rng.uniform(0, 1, (300, 520)).astype(f32)
    w = np.array([[1, 2, 1], [2, 4, 2], [1, 2, 1]]) / 16.0
    f = lambda a: A.stencil(lambda t: sum((t[y][x] * float(w[y][x]) for y in range(3) for x in range(3)),  # noqa: E731
                                          A.constant(0, f32)), boundary, a)
    mode, cval = boundary if isinstance(boundary, tuple) else (boundary, 0.0)
    close(A.runWith(ctx, f, g), oracle.stencil2d(g, w, mode, cval), 1e-6)
    v = rng.uniform(0, 1, 10007).astype(f32)
    s1 = A.runWith(ctx, lambda a: A.stencil(lambda t: 0.25 * t[0] + 0.5 * t[1] + 0.25 * t[2], boundary, a), v)
    close(s1, oracle.stencil2d(v.reshape(1, -1), np.array([[0.25, 0.5, 0.25]]), mode, cval).reshape(-1), 1e-6)


@pytest.mark.gpu
@pytest.mark.parametrize("boundary,padmode", [("clamp", "edge"), ("mirror", "reflect"), ("wrap", "wrap"),
                                              (("constant", 2.0), "constant")])
def test_stencil_over_a_cube_and_over_pairs(ctx, rng, boundary, padmode):
    """A cube of one 4-byte component runs on the rank-3 stencil skeleton; pairs gather through the boundary function."""
    c = rng.uniform(0, 1, (9, 20, 33)).astype(f32)
    mean27 = lambda t: sum((t[z][y][x] for z in range(3) for y in range(3) for x in range(3)), A.constant(0, f32)) / 27.0  # noqa: E731
    got = A.runWith(ctx, lambda a: A.stencil(mean27, boundary, a), c)
    kw = {"constant_values": 2.0} if padmode == "constant" else {}
    p = np.pad(c.astype(f64), 1, mode=padmode, **kw)
    ref = sum(p[z:z + 9, y:y + 20, x:x + 33] for z in range(3) for y in range(3) for x in range(3)) / 27.0
    close(got, ref, 1e-6)
    # elements that are pairs: the neighbourhood of a vector of (value, weight)
    v, w = rng.uniform(0, 1, 5000).astype(f32), rng.uniform(1, 2, 5000).astype(f32)
    sv, sw = A.runWith(ctx, lambda a: A.stencil(lambda t: (t[0][0] * t[0][1] + t[1][0] * t[1][1] + t[2][0] * t[2][1],
                                                           t[0][1] + t[1][1] + t[2][1]), "clamp", a), (v, w))
    pv, pw = np.pad(v.astype(f64), 1, mode="edge"), np.pad(w.astype(f64), 1, mode="edge")
    close(sv, pv[:-2] * pw[:-2] + pv[1:-1] * pw[1:-1] + pv[2:] * pw[2:], 1e-6)
    close(sw, pw[:-2] + pw[1:-1] + pw[2:], 1e-6)


@pytest.mark.gpu
@pytest.mark.parametrize("taps", [[(1, 1, 1), (0, 1, 1), (2, 1, 1), (1, 0, 1), (1, 2, 1), (1, 1, 0), (1, 1, 2)],  # 7-point
                                  [(1, 1, 0), (0, 2, 1)],   # a left halo column in one row, centre columns in another
                                  [(2, 0, 2)],              # one corner: a right halo column only
                                  [(0, 0, 0), (2, 2, 2), (1, 1, 1)],
                                  [(1, 1, 1)]])
@pytest.mark.parametrize("boundary,padmode", [("clamp", "edge"), (("constant", -1.5), "constant")])
def test_cube_stencils_that_read_some_of_their_taps(ctx, rng, taps, boundary, padmode):
    """The functor printed for a rank-3 stencil tells the skeleton which taps the function reads; rows and halo
    columns that nobody reads are skipped.  The cube is wider than one tile (128 columns, 32 rows) and ragged."""
    d, h, w = 5, 37, (260 if boundary == "clamp" else 261)  # 16-byte copies of whole vectors, and the element-wise fill
    c = rng.uniform(0, 1, (d, h, w)).astype(f32)
    wts = {t: float(i + 1) for i, t in enumerate(taps)}
    fn = lambda t: sum((wts[(z, y, x)] * t[z][y][x] for z, y, x in taps), A.constant(0, f32))  # noqa: E731
    got = A.runWith(ctx, lambda a: A.stencil(fn, boundary, a), c)
    kw = {"constant_values": -1.5} if padmode == "constant" else {}
    p = np.pad(c.astype(f64), 1, mode=padmode, **kw)
    ref = sum(wts[(z, y, x)] * p[z:z + d, y:y + h, x:x + w] for z, y, x in taps)
    close(got, ref, 1e-6)


@pytest.mark.gpu
def test_iterated_stencil_and_stencil2(ctx, rng):
    g = rng.uniform(0, 1, (64, 128)).astype(f32)
    five = lambda t: 0.2 * (t[0][1] + t[1][0] + t[1][1] + t[1][2] + t[2][1])  # noqa: E731
    once = A.run1With(ctx, lambda a: A.stencil(five, "clamp", a), A.matrix(f32))
    ref = g
    for _ in range(4):
        ref = once(ref)
    close(A.runWith(ctx, lambda a: A.stencil(five, "clamp", a, iterate=4), g), ref, 1e-6)
    h = rng.uniform(0, 1, (60, 128)).astype(f32)  # the result covers the intersection: 60 rows
    got = A.runWith(ctx, lambda a, b: A.stencil2(lambda s, t: s[1][1] - t[1][1] + 0.5 * t[0][1], "clamp", a, b), g, h)
    up = np.vstack([h[:1], h[:-1]])
    close(got, g[:60] - h + 0.5 * up, 1e-6)


@pytest.mark.gpu
def test_black_scholes_is_one_map_with_two_outputs(ctx, workloads, oracle):
    n = 50000
    W = workloads
    s, k, t = W.uniform_f32(W.SEED, W.S_SPOT, n, 5, 30), W.uniform_f32(W.SEED, W.S_STRIKE, n, 1, 100), \
        W.uniform_f32(W.SEED, W.S_YEARS, n, 0.25, 10)
    assert [x.skeleton for x in A.specs(blackscholes, *[A.vector(f32)] * 3)] == ["map"]
    call, put = A.runWith(ctx, blackscholes, s, k, t)
    rc, rp = oracle.blackscholes(s, k, t)
    close(call, rc, 2e-5)
    close(put, rp, 2e-5)


@pytest.mark.gpu
def test_sparse_matrix_vector_product(ctx, rng):
    nrows, ncols = 20000, 3000
    nnz = rng.integers(0, 13, nrows).astype(i32)
    vals = rng.uniform(-1, 1, int(nnz.sum())).astype(f32)
    cols = rng.integers(0, ncols, vals.size).astype(i32)
    vec = rng.uniform(-1, 1, ncols).astype(f32)
    got = A.runWith(ctx, smvm, vals, cols, vec, nnz)
    offs = np.concatenate([[0], np.cumsum(nnz)])
    prod = np.concatenate([(vals * vec[cols]).astype(f64), [0.0]])
    close(got, np.add.reduceat(prod, offs[:-1]) * (nnz > 0), 1e-6)


@pytest.mark.gpu
def test_generate_backpermute_tuples_and_index_arithmetic(ctx, rng):
    m = rng.uniform(-1, 1, (37, 53)).astype(f32)
    assert np.array_equal(A.runWith(ctx, lambda a: A.backpermute((53, 37), lambda ix: (ix[1], ix[0]), a), m), m.T)
    x = rng.uniform(-1, 1, 100001).astype(f32)
    v, i = A.runWith(ctx, argmax, x)
    assert i == int(np.argmax(x)) and v == x.max()
    a = rng.integers(-50, 50, 10000).astype(i32)
    d, r, q, t, big, frac, pos = A.runWith(
        ctx, lambda z: A.map(lambda e: (e // 7, e % 7, A.quot(e, 7), A.rem(e, 7), A.cast(e, i64) * (1 << 33),
                                        A.cast(e, f64) / 3.0, e > 2), z), a)
    assert np.array_equal(d, a // 7) and np.array_equal(r, a % 7)  # numpy's // and % floor like Haskell's div and mod
    assert np.array_equal(q, np.trunc(a / 7).astype(i32)) and np.array_equal(t, a - 7 * np.trunc(a / 7).astype(i32))
    assert np.array_equal(big, a.astype(i64) << 33) and np.array_equal(frac, a / 3.0) and np.array_equal(pos.astype(bool), a > 2)
    iota = A.runWith(ctx, lambda z: A.generate((3, 5), lambda ix: ix[0] * 10 + ix[1] + A.the(A.fold(add, 0, z))), a)
    assert np.array_equal(iota, np.arange(3)[:, None] * 10 + np.arange(5)[None, :] + a.sum(dtype=i64).astype(i32))
    f = A.run1With(ctx, lambda z: A.map(lambda e: A.cond(e < 0.0, -e, A.sqrt(e)), z), A.vector(f32))
    for n in (5, 70000):  # one compiled function, several shapes
        y = rng.uniform(-1, 1, n).astype(f32)
        close(f(y), np.where(y < 0, -y, np.sqrt(np.abs(y))), 1e-7)


@pytest.mark.gpu
@pytest.mark.parametrize("device", [False, True])
def test_awhile_keeps_the_loop_on_the_device(ctx, accb, rng, device):
    """awhile: doubling until the largest element passes a bound (the trip count depends on the data), and a
    smoothing loop that carries a counter as a second state array.  The device-resident loop (a conditional
    WHILE node) and the host-driven one agree with the same loop written in numpy."""
    x = rng.integers(1, 50, 10001).astype(i32)
    small = lambda v: A.map(lambda m: m < 100000, A.foldAll(A.maximum, 0, v))  # noqa: E731
    got, n = A.awhile(small, lambda v: A.map(lambda e: e * 2 + 1, v), x, ctx=ctx, device=device)
    ref, k = x.copy(), 0
    while ref.max() < 100000:
        ref, k = ref * 2 + 1, k + 1
    assert n == k and k > 5 and np.array_equal(got, ref)

    g = rng.uniform(0, 1, 4099).astype(f32)
    three = lambda t: (t[0] + t[1] + t[2]) / 3.0  # noqa: E731
    (gg, kk), n = A.awhile(lambda a, c: A.map(lambda v: v < 9, c),
                           lambda a, c: (A.stencil(three, "clamp", a), A.map(lambda v: v + 1, c)),
                           g, np.array(0, i32), ctx=ctx, device=device)
    ref = g.astype(f64)
    for _ in range(9):
        p = np.concatenate([ref[:1], ref, ref[-1:]])
        ref = (p[:-2] + p[1:-1] + p[2:]) / 3.0
    assert n == 9 and int(kk) == 9
    close(gg, ref, 1e-6)
    # a condition that is false from the start: the body never runs and the state comes back untouched
    got, n = A.awhile(lambda v: A.map(lambda m: m < 0, A.foldAll(A.maximum, 0, v)), lambda v: A.map(lambda e: e + 1, v),
                      x, ctx=ctx, device=device)
    assert n == 0 and np.array_equal(got, x)
    # a condition that never turns false is stopped by the iteration limit, on the device as well
    with pytest.raises(accb.AccbError) as e:
        A.awhile(lambda v: A.map(lambda m: m > -1, A.foldAll(A.maximum, 0, v)), lambda v: A.map(lambda e: e // 2, v),
                 x, ctx=ctx, device=device, max_iters=6)
    assert e.value.status == accb.ETIMEOUT
