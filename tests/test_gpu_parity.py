"""Parity of every skeleton against the CPU oracle, through the C ABI.

Integer results are compared bit-exactly; float32 results against the float64
oracle with |got - ref| <= RTOL*|ref| + ATOL where RTOL = 1e-5 and the
absolute floor is stated per test.
"""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu

RTOL = 1e-5

# ragged sizes around the vector width (4), the warp (32), the map/fold trip
# (2048 / 4096) and the scan tile (8192)
SIZES = [1, 3, 4, 5, 31, 32, 33, 127, 1000, 2047, 2048, 2049, 4095, 4097, 8191, 8192, 8193, 16385, 100003,
         (1 << 20) + 7]


def dev(torch, a):
    return torch.from_numpy(np.ascontiguousarray(a)).cuda()


def close(got, ref, atol):
    got = np.asarray(got, np.float64)
    ref = np.asarray(ref, np.float64)
    err = np.abs(got - ref)
    tol = RTOL * np.abs(ref) + atol
    assert np.all(err <= tol), f"max excess {np.max(err - tol)} at {np.argmax(err - tol)}"


# ------------------------------------------------------------------- map
@pytest.mark.parametrize("n", [0] + SIZES)
def test_map_saxpy(ctx, P, torch_cuda, rng, n):
    t = torch_cuda
    x, y = rng.standard_normal(n).astype(np.float32), rng.standard_normal(n).astype(np.float32)
    out = t.empty(max(n, 1), dtype=t.float32, device="cuda")[:n]  # an empty array still has an allocation (Prim.hs:167)
    pad = lambda a: dev(t, np.concatenate([a, np.zeros(1, a.dtype)]))[:n]
    ctx.map(P.SAXPY, [pad(x), pad(y)], out, scalars=np.float32(2.5))
    ctx.sync()
    ref = np.float32(2.5) * x + y  # one rounding per op, fma contraction aside
    close(out.cpu().numpy(), ref.astype(np.float64), 1e-6)


def test_map_unaligned_falls_back_to_scalar_path(ctx, P, torch_cuda, rng):
    t = torch_cuda
    n = 10001
    x, y = rng.standard_normal(n + 1).astype(np.float32), rng.standard_normal(n).astype(np.float32)
    xd = dev(t, x)[1:]  # 4-byte aligned only
    out = t.empty(n, dtype=t.float32, device="cuda")
    ctx.map(P.SAXPY, [xd, dev(t, y)], out, scalars=np.float32(-1.0))
    ctx.sync()
    close(out.cpu().numpy(), (-x[1:].astype(np.float64) + y), 1e-6)


@pytest.mark.parametrize("n", [1, 1000, 65537])
def test_generate_from_index(ctx, P, torch_cuda, n):
    t = torch_cuda
    out = t.empty(n, dtype=t.int32, device="cuda")
    ctx.map(P.IOTA_SQ, [], out)
    ctx.sync()
    i = np.arange(n, dtype=np.int64)
    assert np.array_equal(out.cpu().numpy(), (i * i + 1).astype(np.int32))


@pytest.mark.parametrize("n", [5, 4096, 70001])
def test_backpermute_gather(ctx, P, torch_cuda, oracle, rng, n):
    t = torch_cuda
    src = rng.integers(-1000, 1000, 3000).astype(np.int32)
    idx = rng.integers(0, src.size, n).astype(np.int32)
    out = t.empty(n, dtype=t.int32, device="cuda")
    ctx.map(P.GATHER, [dev(t, idx), dev(t, src)], out)
    ctx.sync()
    assert np.array_equal(out.cpu().numpy(), oracle.backpermute_i32(src, idx))


def test_transpose_by_index_arithmetic(ctx, P, torch_cuda, rng):
    t = torch_cuda
    a = rng.standard_normal((37, 53)).astype(np.float32)
    out = t.empty((53, 37), dtype=t.float32, device="cuda")
    ctx.map(P.TRANSPOSE, [dev(t, a)], out)
    ctx.sync()
    assert np.array_equal(out.cpu().numpy(), a.T)


@pytest.mark.parametrize("h,w", [(1, 1), (3, 70), (64, 64), (65, 127), (128, 192), (1000, 36), (257, 1028)])
def test_map_over_transposed_inputs_through_shared_memory_tiles(ctx, P, accb, torch_cuda, rng, h, w):
    """accb_map_transposed: the functor of `map f m` launched as `map f (transpose m)`; full 64x64 tiles take the
    vector path, ragged edges and widths that are not multiples of 4 the scalar one."""
    t = torch_cuda
    x, y = rng.standard_normal((h, w)).astype(np.float32), rng.standard_normal((h, w)).astype(np.float32)
    out = t.empty((w, h), dtype=t.float32, device="cuda")
    ctx.map_transposed(P.SAXPY, [dev(t, x), dev(t, y)], out, scalars=np.float32(2.5))
    ctx.sync()
    close(out.cpu().numpy(), (np.float32(2.5) * x + y).T.astype(np.float64), 1e-6)
    a = rng.integers(-128, 128, (h, w)).astype(np.int8)
    b = rng.integers(-30000, 30000, (h, w)).astype(np.int16)
    c = rng.standard_normal((h, w)) * 1000
    o = t.empty((w, h), dtype=t.int64, device="cuda")
    f = t.empty((w, h), dtype=t.uint8, device="cuda")
    ctx.map_transposed(P.WIDEN, [(dev(t, a), dev(t, b), dev(t, c))], (o, f))  # components of 1, 2 and 8 bytes
    ctx.sync()
    assert np.array_equal(o.cpu().numpy(), (a.astype(np.int64) * b + c.astype(np.int64)).T)
    assert np.array_equal(f.cpu().numpy(), (a > 0).astype(np.uint8).T)
    with pytest.raises(accb.AccbError):
        ctx.map_transposed(P.SAXPY, [dev(t, x), dev(t, y)], t.empty((h + 1, w), device="cuda"), scalars=np.float32(1))


@pytest.mark.parametrize("h,w", [(4, 4), (64, 64), (68, 132), (128, 192), (1000, 36), (256, 1028), (257, 1028), (2048, 4100)])
def test_map_over_one_transposed_input_through_tensor_map_copies(ctx, P, accb, torch_cuda, rng, monkeypatch, h, w):
    """One 4-byte value in and one out: the copy engine moves the 64x64 tiles through tensor maps (extents that are
    multiples of 4; tiles that hang over the edge are clipped by the engine), every other shape takes the
    load / store form.  Both against numpy, with the element index the functor is told, and against each other."""
    t = torch_cuda
    x = rng.standard_normal((h, w)).astype(np.float32)
    out = t.full((w, h), np.nan, dtype=t.float32, device="cuda")
    ctx.map_transposed(P.SCALE_PLUS_INDEX, [dev(t, x)], out)
    ctx.sync()
    ref = 2.0 * x.T.astype(np.float64) + (np.arange(h * w).reshape(w, h) % 5)
    close(out.cpu().numpy(), ref, 1e-6)
    monkeypatch.setenv("ACCB_TRANSPOSE_TMA", "0")  # read when a context is created
    plain = accb.Context(0)
    out2 = t.full((w, h), np.nan, dtype=t.float32, device="cuda")
    plain.map_transposed(P.SCALE_PLUS_INDEX, [dev(t, x)], out2)
    plain.sync()
    assert t.equal(out, out2)
    plain.destroy()


@pytest.mark.parametrize("n", [7, 4096, 12345])
def test_map_mixed_widths(ctx, P, torch_cuda, rng, n):
    t = torch_cuda
    a = rng.integers(-128, 128, n).astype(np.int8)
    b = rng.integers(-30000, 30000, n).astype(np.int16)
    c = rng.standard_normal(n) * 1000
    o = t.empty(n, dtype=t.int64, device="cuda")
    f = t.empty(n, dtype=t.uint8, device="cuda")
    ctx.map(P.WIDEN, [(dev(t, a), dev(t, b), dev(t, c))], (o, f))
    ctx.sync()
    assert np.array_equal(o.cpu().numpy(), a.astype(np.int64) * b + c.astype(np.int64))
    assert np.array_equal(f.cpu().numpy(), (a > 0).astype(np.uint8))


def test_blackscholes(ctx, P, torch_cuda, oracle, workloads):
    t = torch_cuda
    n = 1 << 20
    W = workloads
    s = W.uniform_f32(W.SEED, W.S_SPOT, n, 5, 30)
    k = W.uniform_f32(W.SEED, W.S_STRIKE, n, 1, 100)
    y = W.uniform_f32(W.SEED, W.S_YEARS, n, 0.25, 10)
    call = t.empty(n, dtype=t.float32, device="cuda")
    put = t.empty(n, dtype=t.float32, device="cuda")
    ctx.map(P.BLACKSCHOLES, [(dev(t, s), dev(t, k), dev(t, y))], (call, put))
    ctx.sync()
    rc, rp = oracle.blackscholes(s, k, y)
    # absolute floor: prices reach 100 and float32 rounding of d1 alone moves them by ~1e-5
    close(call.cpu().numpy(), rc, 2e-5)
    close(put.cpu().numpy(), rp, 2e-5)


# ------------------------------------------------------------------ folds
@pytest.mark.parametrize("n", SIZES)
def test_fold_all_dot(ctx, P, torch_cuda, oracle, rng, n):
    t = torch_cuda
    x = rng.uniform(-1, 1, n).astype(np.float32)
    y = rng.uniform(-1, 1, n).astype(np.float32)
    out = t.zeros(1, dtype=t.float32, device="cuda")
    ctx.fold_all(P.DOT, [dev(t, x), dev(t, y)], n, out, seed=np.float32(0))
    ctx.sync()
    # double accumulation: the result is the correctly rounded float32 of the exact sum
    close(out.cpu().numpy()[0], oracle.dot_f32(x, y), 0.0 if n > 64 else 1e-7)


def test_fold_all_float32_accumulator_is_within_tolerance_of_sum_of_magnitudes(ctx, P, torch_cuda, oracle, rng):
    t = torch_cuda
    n = 1 << 22
    x = rng.uniform(-1, 1, n).astype(np.float32)
    y = rng.uniform(-1, 1, n).astype(np.float32)
    out = t.zeros(1, dtype=t.float32, device="cuda")
    ctx.fold_all(P.DOT_F32ACC, [dev(t, x), dev(t, y)], n, out, seed=np.float32(0))
    ctx.sync()
    ref = oracle.dot_f32(x, y)
    assert abs(out.cpu().numpy()[0] - ref) <= 1e-5 * float(np.sum(np.abs(x.astype(np.float64) * y)))


@pytest.mark.parametrize("n", [0, 1, 33, 5000, 300001])
def test_fold_all_int_with_seed(ctx, P, torch_cuda, rng, n):
    t = torch_cuda
    x = rng.integers(-2**31, 2**31 - 1, n).astype(np.int32)
    out = t.zeros(1, dtype=t.int32, device="cuda")
    ctx.fold_all(P.SUM_I32, [dev(t, x)], n, out, seed=np.int32(17))
    ctx.sync()
    assert out.cpu().numpy()[0] == np.array((int(x.astype(np.int64).sum()) + 17) & 0xffffffff, np.uint32).astype(np.int32)


def test_fold1_all_max_and_empty_is_a_bounds_error(ctx, P, accb, torch_cuda, rng):
    t = torch_cuda
    x = rng.integers(-10**6, 10**6, 77777).astype(np.int32)
    out = t.zeros(1, dtype=t.int32, device="cuda")
    ctx.fold_all(P.MAX_I32, [dev(t, x)], x.size, out)  # no seed: fold1All
    ctx.sync()
    assert out.cpu().numpy()[0] == x.max()
    with pytest.raises(accb.AccbError) as e:
        ctx.fold_all(P.MAX_I32, [dev(t, x)], 0, out)
    assert e.value.status == accb.EBOUNDS


def test_fold_all_tuple_argmax(ctx, P, torch_cuda, rng):
    t = torch_cuda
    x = rng.standard_normal(123457).astype(np.float32)
    v = t.zeros(1, dtype=t.float32, device="cuda")
    i = t.zeros(1, dtype=t.int32, device="cuda")
    ctx.fold_all(P.ARGMAX, [dev(t, x)], x.size, (v, i))
    ctx.sync()
    assert i.cpu().numpy()[0] == int(np.argmax(x)) and v.cpu().numpy()[0] == x.max()


@pytest.mark.parametrize("rows,cols", [(1, 1), (7, 3), (5, 31), (100, 32), (33, 100), (64, 1000), (9, 2048),
                                       (17, 4099), (3, 16384), (300, 516),
                                       # many short rows: groups of 4 / 8 / 16 / 32 lanes per row
                                       (20000, 8), (20001, 20), (9000, 48), (9000, 200), (10000, 516), (8200, 2052),
                                       # ... of which rows up to 128 elements go thread-per-row out of shared memory
                                       (70000, 1), (40001, 3), (5003, 100), (600, 128), (3000, 127),
                                       # few long rows: every row cut into pieces across the SMs
                                       (3, 200000), (2, 70001), (5, 1 << 20), (40, 140000)])
def test_fold_rows(ctx, P, torch_cuda, oracle, rng, rows, cols):
    t = torch_cuda
    m = rng.uniform(-1, 1, (rows, cols)).astype(np.float32)
    out = t.zeros(rows, dtype=t.float32, device="cuda")
    ctx.fold_dim(P.ROWSUM, [dev(t, m)], rows, cols, out, seed=np.float32(0))
    ctx.sync()
    close(out.cpu().numpy(), oracle.fold_rows_f32(m), 1e-7)
    mi = rng.integers(-2**31, 2**31 - 1, (rows, cols)).astype(np.int32)
    oi = t.zeros(rows, dtype=t.int32, device="cuda")
    ctx.fold_dim(P.ROWSUM_I32, [dev(t, mi)], rows, cols, oi, seed=np.int32(-5))
    ctx.sync()
    assert np.array_equal(oi.cpu().numpy(), oracle.fold_rows_i32(mi, -5))


def test_fold_rows_empty_inner_dimension_yields_seed(ctx, P, accb, torch_cuda):
    t = torch_cuda
    out = t.zeros(6, dtype=t.int32, device="cuda")
    empty = t.zeros(1, dtype=t.int32, device="cuda")
    ctx.fold_dim(P.ROWSUM_I32, [empty], 6, 0, out, seed=np.int32(42))
    ctx.sync()
    assert np.array_equal(out.cpu().numpy(), np.full(6, 42, np.int32))
    with pytest.raises(accb.AccbError) as e:
        ctx.fold_dim(P.ROWMIN_I32, [empty], 6, 0, out)  # fold1 of empty rows
    assert e.value.status == accb.EBOUNDS


@pytest.mark.parametrize("rows,cols", [(50, 777), (30000, 12), (3, 300000)])
def test_fold1_rows_min(ctx, P, torch_cuda, rng, rows, cols):
    t = torch_cuda
    m = rng.integers(-10**6, 10**6, (rows, cols)).astype(np.int32)
    out = t.zeros(rows, dtype=t.int32, device="cuda")
    ctx.fold_dim(P.ROWMIN_I32, [dev(t, m)], rows, cols, out)
    ctx.sync()
    assert np.array_equal(out.cpu().numpy(), m.min(axis=1))


def test_fold_seg(ctx, P, torch_cuda, oracle, rng):
    t = torch_cuda
    lens = rng.integers(0, 200, 500)
    lens[::7] = 0  # empty segments yield the seed
    offs = np.concatenate([[0], np.cumsum(lens)]).astype(np.int32)
    x = rng.integers(-1000, 1000, int(offs[-1])).astype(np.int32)
    out = t.zeros(lens.size, dtype=t.int32, device="cuda")
    ctx.fold_seg(P.SEGSUM_I32, [dev(t, x)], 1, x.size, dev(t, offs), lens.size, out, seed=np.int32(3))
    ctx.sync()
    assert np.array_equal(out.cpu().numpy(), oracle.fold_seg_i32(x, offs, 3))
    xf = rng.uniform(-1, 1, x.size).astype(np.float32)
    of = t.zeros(lens.size, dtype=t.float32, device="cuda")
    ctx.fold_seg(P.SEGSUM_F32, [dev(t, xf)], 1, x.size, dev(t, offs), lens.size, of, seed=np.float32(0))
    ctx.sync()
    close(of.cpu().numpy(), oracle.fold_seg_f32(xf, offs), 1e-7)


@pytest.mark.parametrize("nseg,mean", [(60000, 3), (30000, 12), (9000, 40), (9000, 100), (300, 3000), (12, 20000),
                                       (20000, 150), (6000, 300), (5000, 1000)])  # staged with 8 lanes per segment; groups
def test_fold_seg_by_segment_length(ctx, P, torch_cuda, oracle, rng, nseg, mean):
    """4, 8, 16 and 32 lanes or a whole block per segment, chosen by the average segment length."""
    t = torch_cuda
    lens = rng.integers(0, 2 * mean + 1, nseg)
    offs = np.concatenate([[0], np.cumsum(lens)]).astype(np.int32)
    x = rng.integers(-1000, 1000, int(offs[-1])).astype(np.int32)
    out = t.zeros(nseg, dtype=t.int32, device="cuda")
    ctx.fold_seg(P.SEGSUM_I32, [dev(t, x)], 1, x.size, dev(t, offs), nseg, out, seed=np.int32(-9))
    ctx.sync()
    assert np.array_equal(out.cpu().numpy(), oracle.fold_seg_i32(x, offs, -9))


def test_fold_seg_short_segments_with_outliers(ctx, P, torch_cuda, oracle, rng):
    """The windowed form: mostly short segments, runs of empty ones, a few that span several windows,
    a source length that is not a multiple of 4, and trailing empty segments."""
    t = torch_cuda
    lens = rng.integers(0, 9, 50000)
    lens[1000:1400] = 0
    lens[[5, 20000, 49990]] = [30000, 70, 9001]
    lens[-3:] = 0
    lens[7] += (-int(lens.sum())) % 4 + 1  # total = 1 (mod 4)
    offs = np.concatenate([[0], np.cumsum(lens)]).astype(np.int32)
    x = rng.integers(-1000, 1000, int(offs[-1])).astype(np.int32)
    out = t.full((lens.size,), 77, dtype=t.int32, device="cuda")
    ctx.fold_seg(P.SEGSUM_I32, [dev(t, x)], 1, x.size, dev(t, offs), lens.size, out, seed=np.int32(5))
    ctx.sync()
    assert np.array_equal(out.cpu().numpy(), oracle.fold_seg_i32(x, offs, 5))
    xf = rng.uniform(-1, 1, x.size).astype(np.float32)
    of = t.zeros(lens.size, dtype=t.float32, device="cuda")
    ctx.fold_seg(P.SEGSUM_F32, [dev(t, xf)], 1, x.size, dev(t, offs), lens.size, of, seed=np.float32(0))
    ctx.sync()
    ref = np.array([xf[offs[s]:offs[s + 1]].astype(np.float64).sum() for s in range(lens.size)])
    close(of.cpu().numpy(), ref, 1e-5)


@pytest.mark.parametrize("nrows,mean_nnz", [(300, 7), (40000, 5), (20000, 30), (3000, 400)])
def test_fold_seg_sparse_matrix_vector_product(ctx, P, torch_cuda, rng, nrows, mean_nnz):
    """CSR smvm: two zipped inputs of different types plus a gathered free array variable."""
    t = torch_cuda
    ncols = 5000
    nnz = rng.integers(0, 2 * mean_nnz + 1, nrows)
    offs = np.concatenate([[0], np.cumsum(nnz)]).astype(np.int32)
    vals = rng.uniform(-1, 1, int(offs[-1])).astype(np.float32)
    cols = rng.integers(0, ncols, int(offs[-1])).astype(np.int32)
    vec = rng.uniform(-1, 1, ncols).astype(np.float32)
    out = t.zeros(nrows, dtype=t.float32, device="cuda")
    ctx.fold_seg(P.SMVM, [(dev(t, vals), dev(t, cols)), dev(t, vec)], 1, vals.size, dev(t, offs), nrows, out,
                 seed=np.float32(0))
    ctx.sync()
    prod = np.concatenate([(vals * vec[cols]).astype(np.float64), [0.0]])  # products rounded to float32 as on the device
    ref = np.add.reduceat(prod, offs[:-1]) * (nnz > 0)
    close(out.cpu().numpy(), ref, 1e-6)


@pytest.mark.parametrize("rows,cols", [(30000, 10), (900, 3000)])
def test_fold_rows_of_two_zipped_inputs(ctx, P, torch_cuda, rng, rows, cols):
    t = torch_cuda
    a = rng.uniform(-1, 1, (rows, cols)).astype(np.float32)
    b = rng.uniform(-1, 1, (rows, cols)).astype(np.float32)
    out = t.zeros(rows, dtype=t.float32, device="cuda")
    ctx.fold_dim(P.ROWDOT, [(dev(t, a), dev(t, b))], rows, cols, out, seed=np.float32(0))
    ctx.sync()
    close(out.cpu().numpy(), ((a * b).astype(np.float64)).sum(axis=1), 1e-6)


def test_fold_seg_short_segments_rank2(ctx, P, torch_cuda, rng):
    t = torch_cuda
    lens = rng.integers(0, 13, 3000)
    lens[0] += (-int(lens.sum())) % 16  # row length a multiple of 16: the windowed form applies per row
    offs = np.concatenate([[0], np.cumsum(lens)]).astype(np.int32)
    m = rng.integers(-50, 50, (3, int(offs[-1]))).astype(np.int32)
    out = t.zeros((3, lens.size), dtype=t.int32, device="cuda")
    ctx.fold_seg(P.SEGSUM_I32, [dev(t, m)], 3, m.shape[1], dev(t, offs), lens.size, out, seed=np.int32(0))
    ctx.sync()
    ref = np.stack([np.add.reduceat(np.concatenate([m[r], [0]]), offs[:-1])[:lens.size] * (lens > 0) for r in range(3)])
    assert np.array_equal(out.cpu().numpy(), ref.astype(np.int32))


def test_fold_seg_rank2(ctx, P, torch_cuda, rng):
    t = torch_cuda
    lens = np.array([3, 0, 10, 40, 1])
    offs = np.concatenate([[0], np.cumsum(lens)]).astype(np.int32)
    m = rng.integers(-50, 50, (4, int(offs[-1]))).astype(np.int32)
    out = t.zeros((4, lens.size), dtype=t.int32, device="cuda")
    ctx.fold_seg(P.SEGSUM_I32, [dev(t, m)], 4, m.shape[1], dev(t, offs), lens.size, out, seed=np.int32(0))
    ctx.sync()
    ref = np.stack([[m[r, offs[s]:offs[s + 1]].sum() for s in range(lens.size)] for r in range(4)]).astype(np.int32)
    assert np.array_equal(out.cpu().numpy(), ref)


def _seg_ref(x, offs, seed):
    tot = np.concatenate([[0], np.cumsum(x.astype(np.int64))])
    return (tot[offs[1:]] - tot[offs[:-1]] + seed).astype(np.int64)


@pytest.mark.parametrize("case", ["tile_edges", "one_giant", "giant_among_short", "offsets_inside", "leading_empty",
                                  "all_empty", "ragged_tail", "many_empty_runs"])
def test_fold_seg_segments_of_any_length(ctx, P, torch_cuda, rng, case):
    """Segments that end exactly on multiples of 32 and 4096 elements, one segment of 4.5 M elements, segments of
    a million and more elements among 2.6 million short ones (sources of 2^24 elements and more hand segments
    longer than 65536 elements over to a second launch that splits them over all blocks), offsets that cover only
    the middle of the source, empty segments first, last and in runs, no elements at all."""
    t = torch_cuda
    T, V = 4096, 32
    pad_front = pad_back = 0
    if case == "tile_edges":
        lens = np.array([T, V, V, T - 2 * V, 1, T - 1, 2 * T, 0, 0, 3, T - 3, V - 1, 1, 5 * T + 17, 40])
    elif case == "one_giant":
        lens = np.array([0, 1100 * T + 5, 0])
    elif case == "giant_among_short":
        lens = rng.integers(0, 12, 2600000)
        lens[[100, 20000, 2599999]] = [450 * T + 1, 3 * T, 390 * T - 7]
    elif case == "offsets_inside":
        lens = rng.integers(0, 30, 3000)
        pad_front, pad_back = 5000, 7003
    elif case == "leading_empty":
        lens = np.concatenate([np.zeros(2000, np.int64), rng.integers(1, 20, 2000), np.zeros(1500, np.int64)])
        pad_front = 4099
    elif case == "all_empty":
        lens = np.zeros(3000, np.int64)
        pad_front, pad_back = 3, 9000
    elif case == "ragged_tail":
        lens = rng.integers(0, 64, 1000)
        lens[-1] += (1 - int(lens.sum())) % 4  # the source ends one element into a 16-byte unit
    else:
        lens = rng.integers(1, 9, 30000)
        for first in range(0, 30000, 700):
            lens[first:first + 300] = 0
    offs = (pad_front + np.concatenate([[0], np.cumsum(lens)])).astype(np.int32)
    n = int(offs[-1]) + pad_back
    x = rng.integers(-1000, 1000, n).astype(np.int32)
    out = t.full((lens.size,), 77, dtype=t.int32, device="cuda")
    ctx.fold_seg(P.SEGSUM_I32, [dev(t, x)], 1, n, dev(t, offs), lens.size, out, seed=np.int32(5))
    ctx.sync()
    assert np.array_equal(out.cpu().numpy().astype(np.int64), _seg_ref(x, offs, 5))
    # fold1Seg: no seed, empty segments are left alone
    out.fill_(77)
    ctx.fold_seg(P.SEGSUM_I32, [dev(t, x)], 1, n, dev(t, offs), lens.size, out)
    ctx.sync()
    ref = np.where(lens > 0, _seg_ref(x, offs, 0), 77)
    assert np.array_equal(out.cpu().numpy().astype(np.int64), ref)


def test_fold_seg_long_segments_in_rows_and_with_two_inputs(ctx, P, torch_cuda, rng):
    """Rank 2 (every row cut by the same offsets; one segment of 1.1 M elements per row is handed to the second
    launch) and a functor with two zipped inputs of float32 and Int32 plus a gathered vector, accumulating in
    float64, with a segment of 900000 elements among short ones."""
    t = torch_cuda
    lens = rng.integers(0, 16000, 400)
    lens[17] = 1100000
    lens[0] += (-int(lens.sum())) % 16
    offs = np.concatenate([[0], np.cumsum(lens)]).astype(np.int32)
    m = rng.integers(-50, 50, (3, int(offs[-1]))).astype(np.int32)
    out = t.zeros((3, lens.size), dtype=t.int32, device="cuda")
    ctx.fold_seg(P.SEGSUM_I32, [dev(t, m)], 3, m.shape[1], dev(t, offs), lens.size, out, seed=np.int32(1))
    ctx.sync()
    ref = np.stack([_seg_ref(m[r], offs, 1) for r in range(3)])
    assert np.array_equal(out.cpu().numpy().astype(np.int64), ref)
    nnz = rng.integers(0, 120, 270000)
    nnz[[5, 3000]] = [900000, 70001]
    offs = np.concatenate([[0], np.cumsum(nnz)]).astype(np.int32)
    vals = rng.uniform(-1, 1, int(offs[-1])).astype(np.float32)
    cols = rng.integers(0, 5000, int(offs[-1])).astype(np.int32)
    vec = rng.uniform(-1, 1, 5000).astype(np.float32)
    of = t.zeros(nnz.size, dtype=t.float32, device="cuda")
    ctx.fold_seg(P.SMVM, [(dev(t, vals), dev(t, cols)), dev(t, vec)], 1, vals.size, dev(t, offs), nnz.size, of,
                 seed=np.float32(0))
    ctx.sync()
    prod = np.concatenate([(vals * vec[cols]).astype(np.float64), [0.0]])
    close(of.cpu().numpy(), np.add.reduceat(prod, offs[:-1]) * (nnz > 0), 1e-6)


@pytest.fixture(scope="module")
def ctx_one_application_per_launch(accb, torch_cuda):
    """A context whose iterated stencils never fuse two applications into one launch (tuning is read when a
    context is made)."""
    import os
    os.environ["ACCB_STENCIL_NO_FUSE"] = "1"
    try:
        c = accb.Context(0)
    finally:
        del os.environ["ACCB_STENCIL_NO_FUSE"]
    yield c
    c.sync()


@pytest.mark.parametrize("shape", [(16, 256), (33, 260), (100, 516), (257, 1024), (64, 252)])
@pytest.mark.parametrize("boundary", ["clamp", "mirror", "constant", "wrap"])
@pytest.mark.parametrize("prog,iters", [("BLUR", 2), ("BLUR", 7), ("LAPLACE", 4), ("BOX5", 3)])
def test_two_applications_per_launch_equal_one_by_one(ctx, ctx_one_application_per_launch, P, torch_cuda, rng, shape, boundary,
                                                      prog, iters):
    """An iterated stencil runs two applications per launch where it can (the intermediate grid of a block stays
    in shared memory): bit-identical to one application per launch, for tiles along every edge and corner, widths
    that are not whole tiles, odd counts (the last application goes alone) and a 5x5 neighbourhood (radius 2)."""
    t = torch_cuda
    g = rng.uniform(-1, 1, shape).astype(np.float32)
    const = np.float32(0.5)
    outs = []
    for c in (ctx, ctx_one_application_per_launch):
        a, b = dev(t, g), t.empty(shape, dtype=t.float32, device="cuda")
        before = c.launch_count()
        r = c.stencil_iterate(getattr(P, prog), a, b, iters, boundary=boundary, constant=const)
        c.sync()
        outs.append((r.cpu().numpy(), c.launch_count() - before))
    assert np.array_equal(outs[0][0], outs[1][0])
    assert outs[1][1] == iters
    if boundary != "wrap" and shape[1] % 4 == 0:
        assert outs[0][1] == (iters + 1) // 2  # pairs, and the odd one out


# ------------------------------------------------------------------ scans
def test_scan_known_answers_from_the_reference_docs(ctx, P, accb, torch_cuda):
    """CodeGen/PrefixSum.hs:149-153, 162-166, 176-180."""
    t = torch_cuda
    ones = t.ones(10, dtype=t.int32, device="cuda")
    out = t.zeros(11, dtype=t.int32, device="cuda")
    ctx.scan(P.SCAN_ADD_I32, [ones], 10, out, seed=np.int32(10))
    ctx.sync()
    assert out.cpu().tolist() == [10, 11, 12, 13, 14, 15, 16, 17, 18, 19, 20]
    out1 = t.zeros(10, dtype=t.int32, device="cuda")
    ctx.scan(P.SCAN_ADD_I32, [ones], 10, out1, kind=accb.SCAN_INCLUSIVE)
    ctx.sync()
    assert out1.cpu().tolist() == [1, 2, 3, 4, 5, 6, 7, 8, 9, 10]
    body = t.zeros(10, dtype=t.int32, device="cuda")
    tot = t.zeros(1, dtype=t.int32, device="cuda")
    ctx.scan(P.SCAN_ADD_I32, [ones], 10, body, kind=accb.SCAN_PRIME, seed=np.int32(10), total=tot)
    ctx.sync()
    assert body.cpu().tolist() == [10, 11, 12, 13, 14, 15, 16, 17, 18, 19] and tot.cpu().tolist() == [20]


@pytest.mark.parametrize("n", [0] + SIZES)
def test_scan_all_six_variants_int32(ctx, P, accb, torch_cuda, oracle, rng, n):
    t = torch_cuda
    x = rng.integers(-2**31, 2**31 - 1, n).astype(np.int32)  # wraps: addition is modulo 2^32
    xd = dev(t, x) if n else t.zeros(1, dtype=t.int32, device="cuda")
    z = np.int32(-7)
    out = t.zeros(n + 1, dtype=t.int32, device="cuda")
    ctx.scan(P.SCAN_ADD_I32, [xd], n, out, seed=z)
    ctx.sync()
    assert np.array_equal(out.cpu().numpy(), oracle.scanl_i32(x, z))
    ctx.scan(P.SCAN_ADD_I32, [xd], n, out, direction=accb.SCAN_RIGHT, seed=z)
    ctx.sync()
    assert np.array_equal(out.cpu().numpy(), oracle.scanr_i32(x, z))
    body = t.zeros(max(n, 1), dtype=t.int32, device="cuda")
    tot = t.zeros(1, dtype=t.int32, device="cuda")
    for direction, ref in ((accb.SCAN_LEFT, oracle.scanl_prime_i32), (accb.SCAN_RIGHT, oracle.scanr_prime_i32)):
        ctx.scan(P.SCAN_ADD_I32, [xd], n, body, direction=direction, kind=accb.SCAN_PRIME, seed=z, total=tot)
        ctx.sync()
        rb, rt = ref(x, z)
        assert np.array_equal(body.cpu().numpy()[:n], rb) and tot.cpu().numpy()[0] == rt
    if n:
        for direction, ref in ((accb.SCAN_LEFT, oracle.scanl1_i32), (accb.SCAN_RIGHT, oracle.scanr1_i32)):
            ctx.scan(P.SCAN_ADD_I32, [xd], n, body, direction=direction, kind=accb.SCAN_INCLUSIVE)
            ctx.sync()
            assert np.array_equal(body.cpu().numpy()[:n], ref(x))


@pytest.mark.parametrize("n", [1, 100, 8193, 250007])
def test_scan_non_commutative_pairs_keeps_order(ctx, P, accb, torch_cuda, oracle, rng, n):
    """Affine-map composition: associative, not commutative, two SoA components."""
    t = torch_cuda
    a = rng.integers(0, 2**32, n, dtype=np.uint64).astype(np.uint32) | np.uint32(1)
    b = rng.integers(0, 2**32, n, dtype=np.uint64).astype(np.uint32)
    M = 1 << 32
    f = lambda p, q: ((q[0] * p[0]) % M, (q[0] * p[1] + q[1]) % M)  # p then q
    items = list(zip(a.tolist(), b.tolist()))
    ad, bd = dev(t, a.view(np.int32)), dev(t, b.view(np.int32))
    oa = t.zeros(n + 1, dtype=t.int32, device="cuda")
    ob = t.zeros(n + 1, dtype=t.int32, device="cuda")
    seed = (np.uint32(3), np.uint32(5))
    for direction, dname in ((accb.SCAN_LEFT, "l"), (accb.SCAN_RIGHT, "r")):
        ctx.scan(P.SCAN_AFFINE, [(ad, bd)], n, (oa, ob), direction=direction, seed=seed)
        ctx.sync()
        ref = oracle.scan_generic(items, f, (3, 5), direction=dname, kind="excl") if n <= 8193 else None
        if ref is not None:
            got = list(zip(oa.cpu().numpy().view(np.uint32).tolist(), ob.cpu().numpy().view(np.uint32).tolist()))
            assert got == ref
    if n > 8193:  # large case: check the recurrence out[i+1] = f(out[i], x[i]) everywhere (left scan)
        ctx.scan(P.SCAN_AFFINE, [(ad, bd)], n, (oa, ob), seed=seed)
        ctx.sync()
        ga = oa.cpu().numpy().view(np.uint32).astype(np.uint64)
        gb = ob.cpu().numpy().view(np.uint32).astype(np.uint64)
        A, B = a.astype(np.uint64), b.astype(np.uint64)
        assert ga[0] == 3 and gb[0] == 5
        assert np.array_equal(ga[1:], (A * ga[:-1]) % M) and np.array_equal(gb[1:], (A * gb[:-1] + B) % M)


@pytest.mark.parametrize("n", [5, 8192, 100001])
def test_scan_int64_and_float(ctx, P, accb, torch_cuda, oracle, rng, n):
    t = torch_cuda
    x = rng.integers(-2**40, 2**40, n).astype(np.int64)
    out = t.zeros(n + 1, dtype=t.int64, device="cuda")
    ctx.scan(P.SCAN_ADD_I64, [dev(t, x)], n, out, seed=np.int64(1))
    ctx.sync()
    assert np.array_equal(out.cpu().numpy(), np.concatenate([[1], 1 + np.cumsum(x)]))
    xf = rng.uniform(0, 1, n).astype(np.float32)
    of = t.zeros(n + 1, dtype=t.float32, device="cuda")
    ctx.scan(P.SCAN_ADD_F32, [dev(t, xf)], n, of, seed=np.float32(0))
    ctx.sync()
    # float32 running sums of positive terms: error grows with the prefix, bound it by eps*log2(n)*prefix
    ref = oracle.scanl_f32(xf)
    assert np.all(np.abs(of.cpu().numpy() - ref) <= 1e-5 * np.abs(ref) + 1e-6)
    xm = rng.integers(-10**9, 10**9, n).astype(np.int32)
    om = t.zeros(n, dtype=t.int32, device="cuda")
    ctx.scan(P.SCAN_MAX_I32, [dev(t, xm)], n, om, kind=accb.SCAN_INCLUSIVE)
    ctx.sync()
    assert np.array_equal(om.cpu().numpy(), np.maximum.accumulate(xm))


def test_scan_back_to_back_launches_share_scratch(ctx, P, accb, torch_cuda, oracle, rng):
    """Status words are never cleared between launches: epochs must keep them apart."""
    t = torch_cuda
    for n in (100000, 30, 250000, 8192, 77):
        x = rng.integers(0, 16, n).astype(np.int32)
        out = t.zeros(n + 1, dtype=t.int32, device="cuda")
        ctx.scan(P.SCAN_ADD_I32, [dev(t, x)], n, out, seed=np.int32(0))
        a = rng.integers(0, 100, n).astype(np.int64)
        o64 = t.zeros(n + 1, dtype=t.int64, device="cuda")
        ctx.scan(P.SCAN_ADD_I64, [dev(t, a)], n, o64, seed=np.int64(0))  # other record layout, same scratch
        ctx.sync()
        assert np.array_equal(out.cpu().numpy(), oracle.scanl_i32(x, 0))
        assert np.array_equal(o64.cpu().numpy()[1:], np.cumsum(a))


# ---------------------------------------------------------------- permute
@pytest.mark.parametrize("n", [0, 1, 33, 4097, 1 << 20])
def test_histogram(ctx, P, torch_cuda, oracle, workloads, n):
    t = torch_cuda
    W = workloads
    cdf = W.zipf_cdf()
    keys = W.zipf_mix_keys(W.SEED, n, cdf) if n else np.zeros(0, np.int32)
    kd = dev(t, keys) if n else t.zeros(1, dtype=t.int32, device="cuda")
    defaults = t.arange(W.HIST_BINS, dtype=t.int32, device="cuda")  # non-zero defaults must survive
    ref = oracle.permute_add_i32(keys, W.HIST_BINS, defaults=np.arange(W.HIST_BINS, dtype=np.int32))
    for spec in (P.HIST, P.HIST_GLOBAL):
        out = t.zeros(W.HIST_BINS, dtype=t.int32, device="cuda")
        ctx.permute(spec, [kd], n, out, defaults=defaults)
        ctx.sync()
        assert np.array_equal(out.cpu().numpy(), ref)


def test_permute_ignores_out_of_range_and_negative_destinations(ctx, P, torch_cuda, oracle, rng):
    t = torch_cuda
    keys = rng.integers(-5, 40, 10000).astype(np.int32)  # bins are [0, 32)
    w = rng.integers(-9, 9, keys.size).astype(np.int32)
    out = t.zeros(32, dtype=t.int32, device="cuda")
    ctx.permute(P.HIST_WEIGHTED, [(dev(t, keys), dev(t, w))], keys.size, out, defaults=t.zeros(32, dtype=t.int32, device="cuda"))
    ctx.sync()
    assert np.array_equal(out.cpu().numpy(), oracle.permute_add_i32(keys, 32, weights=w))


def test_permute_cas_float_max(ctx, P, torch_cuda, rng):
    t = torch_cuda
    keys = rng.integers(0, 50, 100000).astype(np.int32)
    v = rng.standard_normal(keys.size).astype(np.float32)
    dfl = np.full(50, -1e30, np.float32)
    out = t.zeros(50, dtype=t.float32, device="cuda")
    ctx.permute(P.SCATTER_MAX_F32, [(dev(t, keys), dev(t, v))], keys.size, out, defaults=dev(t, dfl))
    ctx.sync()
    ref = dfl.copy()
    np.maximum.at(ref, keys, v)
    assert np.array_equal(out.cpu().numpy(), ref)


def test_permute_plain_scatter_is_a_permutation(ctx, P, torch_cuda, rng):
    t = torch_cuda
    n = 50000
    perm = rng.permutation(n).astype(np.int32)
    v = rng.integers(-10**6, 10**6, n).astype(np.int32)
    out = t.zeros(n, dtype=t.int32, device="cuda")
    ctx.permute(P.SCATTER, [(dev(t, perm), dev(t, v))], n, out, defaults=t.zeros(n, dtype=t.int32, device="cuda"))
    ctx.sync()
    ref = np.zeros(n, np.int32)
    ref[perm] = v
    assert np.array_equal(out.cpu().numpy(), ref)


def test_permute_tuple_value_under_lock(ctx, P, torch_cuda, rng):
    t = torch_cuda
    keys = rng.integers(0, 97, 20000).astype(np.int32)
    v = rng.integers(-100, 100, keys.size).astype(np.int32)
    s = t.zeros(97, dtype=t.int32, device="cuda")
    c = t.zeros(97, dtype=t.int32, device="cuda")
    z = t.zeros(97, dtype=t.int32, device="cuda")
    ctx.permute(P.SCATTER_PAIR, [(dev(t, keys), dev(t, v))], keys.size, (s, c), defaults=(z, z))
    ctx.sync()
    rs, rc = np.zeros(97, np.int64), np.zeros(97, np.int64)
    np.add.at(rs, keys, v)
    np.add.at(rc, keys, 1)
    assert np.array_equal(s.cpu().numpy(), rs.astype(np.int32)) and np.array_equal(c.cpu().numpy(), rc.astype(np.int32))


# ---------------------------------------------------------------- stencil
@pytest.mark.parametrize("boundary", ["clamp", "mirror", "wrap", "constant"])
@pytest.mark.parametrize("shape", [(3, 3), (5, 7), (32, 128), (33, 130), (70, 1031), (257, 64)])
def test_stencil_blur_all_boundaries(ctx, P, torch_cuda, oracle, workloads, rng, boundary, shape):
    t = torch_cuda
    a = rng.uniform(0, 1, shape).astype(np.float32)
    out = t.zeros(shape, dtype=t.float32, device="cuda")
    ctx.stencil(P.BLUR, dev(t, a), out, boundary=boundary, constant=np.float32(0.5))
    ctx.sync()
    close(out.cpu().numpy(), oracle.stencil2d(a, workloads.BLUR_WEIGHTS, boundary, 0.5), 1e-6)


@pytest.mark.parametrize("boundary", ["clamp", "mirror", "wrap", "constant"])
@pytest.mark.parametrize("shape", [(16, 8), (17, 260), (64, 1024), (100, 516), (33, 256), (300, 252)])
def test_stencil_tile_form_shapes(ctx, P, torch_cuda, oracle, workloads, rng, boundary, shape):
    """Widths that are multiples of 4 with at least 16 rows take the TMA-staged tile kernel: one and
    several column tiles, ragged last tiles in both directions, radius 1 and 2."""
    t = torch_cuda
    a = rng.uniform(0, 1, shape).astype(np.float32)
    out = t.zeros(shape, dtype=t.float32, device="cuda")
    ctx.stencil(P.BLUR, dev(t, a), out, boundary=boundary, constant=np.float32(-1.5))
    ctx.sync()
    close(out.cpu().numpy(), oracle.stencil2d(a, workloads.BLUR_WEIGHTS, boundary, -1.5), 1e-6)
    ctx.stencil(P.BOX5, dev(t, a), out, boundary=boundary, constant=np.float32(0.25))
    ctx.sync()
    close(out.cpu().numpy(), oracle.stencil2d(a, np.full((5, 5), 0.04), boundary, 0.25), 2e-6)


def test_stencil_tile_and_register_forms_agree_bit_for_bit(ctx, P, torch_cuda, rng, monkeypatch):
    t = torch_cuda
    a = dev(t, rng.uniform(0, 1, (200, 1028)).astype(np.float32))
    tiled, plain = t.zeros_like(a), t.zeros_like(a)
    ctx.stencil(P.BLUR, a, tiled, boundary="mirror")
    monkeypatch.setenv("ACCB_STENCIL_NO_TILE", "1")
    ctx.stencil(P.BLUR, a, plain, boundary="mirror")
    ctx.sync()
    assert t.equal(tiled, plain)


@pytest.mark.parametrize("boundary", ["clamp", "mirror", "wrap", "constant"])
def test_stencil_radius2_and_laplace(ctx, P, torch_cuda, oracle, rng, boundary):
    t = torch_cuda
    a = rng.uniform(-1, 1, (61, 203)).astype(np.float32)
    out = t.zeros(a.shape, dtype=t.float32, device="cuda")
    ctx.stencil(P.BOX5, dev(t, a), out, boundary=boundary, constant=np.float32(-2.0))
    ctx.sync()
    close(out.cpu().numpy(), oracle.stencil2d(a, np.full((5, 5), 0.04), boundary, -2.0), 2e-6)
    lap = np.array([[0, 1, 0], [1, -4, 1], [0, 1, 0]], np.float64)
    ctx.stencil(P.LAPLACE, dev(t, a), out, boundary=boundary, constant=np.float32(0.0))
    ctx.sync()
    close(out.cpu().numpy(), oracle.stencil2d(a, lap, boundary, 0.0), 2e-6)


@pytest.mark.parametrize("n", [1, 2, 5, 129, 10007,
                               4096, 8192, 8196, 100000, 1 << 20])  # multiples of 4 from 4096 up: the staged line form
@pytest.mark.parametrize("boundary", ["clamp", "mirror", "wrap", "constant"])
def test_stencil_rank1(ctx, P, torch_cuda, oracle, rng, n, boundary):
    t = torch_cuda
    if boundary in ("wrap", "mirror") and n < 2:
        pytest.skip("wrap and mirror need an array larger than the stencil radius")
    a = rng.uniform(0, 1, n).astype(np.float32)
    out = t.zeros(n, dtype=t.float32, device="cuda")
    ctx.stencil(P.SMOOTH1D, dev(t, a), out, boundary=boundary, constant=np.float32(1.0))
    ctx.sync()
    ref = oracle.stencil2d(a.reshape(1, n), np.array([[0.25, 0.5, 0.25]]), boundary, 1.0).reshape(n)
    close(out.cpu().numpy(), ref, 1e-6)


def test_stencil_iterated_blur_matches_float64_recurrence(ctx, P, torch_cuda, oracle, workloads, rng):
    t = torch_cuda
    a = rng.uniform(0, 1, (256, 512)).astype(np.float32)
    A, B = dev(t, a), t.zeros(a.shape, dtype=t.float32, device="cuda")
    res = ctx.stencil_iterate(P.BLUR, A, B, 10, boundary="clamp")
    ctx.sync()
    close(res.cpu().numpy(), oracle.stencil2d_iter(a, workloads.BLUR_WEIGHTS, 10, "clamp"), 1e-6)


@pytest.mark.parametrize("boundary", ["clamp", "mirror", "wrap", "constant"])
@pytest.mark.parametrize("shape", [(3, 3, 4), (5, 7, 9), (19, 33, 260), (40, 16, 128), (9, 50, 131)])
def test_stencil_rank3(ctx, P, torch_cuda, oracle, rng, boundary, shape):
    """Stencils over cubes (mkStencil is rank-polymorphic, Stencil.hs:55-114): 27 different weights against the
    float64 oracle, ragged and aligned extents, all four boundaries; and the 7-point Laplacian."""
    t = torch_cuda
    a = rng.uniform(-1, 1, shape).astype(np.float32)
    out = t.empty(shape, dtype=t.float32, device="cuda")
    const = np.float32(0.25) if boundary == "constant" else None
    ctx.stencil(P.WEIGHTED27, dev(t, a), out, boundary=boundary, constant=const)
    ctx.sync()
    w = (np.arange(27, dtype=np.float64).reshape(3, 3, 3) + 1) / 378.0
    close(out.cpu().numpy(), oracle.stencil3d(a, w, boundary, 0.25), 1e-6)
    ctx.stencil(P.LAPLACE3, dev(t, a), out, boundary=boundary, constant=const)
    ctx.sync()
    lap = np.zeros((3, 3, 3))
    lap[1, 1, 1] = -6
    for z, y, x in ((0, 1, 1), (2, 1, 1), (1, 0, 1), (1, 2, 1), (1, 1, 0), (1, 1, 2)):
        lap[z, y, x] = 1
    close(out.cpu().numpy(), oracle.stencil3d(a, lap, boundary, 0.25), 1e-5)


def test_stencil_rank3_unaligned_source_and_iteration(ctx, P, torch_cuda, oracle, rng):
    t = torch_cuda
    shape = (12, 20, 64)
    a = rng.uniform(-1, 1, shape).astype(np.float32)
    flat = t.empty(a.size + 1, dtype=t.float32, device="cuda")
    src = flat[1:].view(shape)  # 4-byte aligned only: scalar loads
    src.copy_(dev(t, a))
    out, tmp = t.empty(shape, dtype=t.float32, device="cuda"), t.empty(shape, dtype=t.float32, device="cuda")
    ctx.stencil(P.WEIGHTED27, src, out, boundary="clamp")
    ctx.sync()
    w = (np.arange(27, dtype=np.float64).reshape(3, 3, 3) + 1) / 378.0
    ref = oracle.stencil3d(a, w, "clamp")
    close(out.cpu().numpy(), ref, 1e-6)
    res = ctx.stencil_iterate(P.WEIGHTED27, out, tmp, 2, boundary="clamp")  # three applications in all
    ctx.sync()
    for _ in range(2):
        ref = oracle.stencil3d(ref, w, "clamp")
    close(res.cpu().numpy(), ref, 1e-5)
    with pytest.raises(Exception):  # a rank-2 kernel on a cube
        ctx.stencil(P.BLUR, src, out, boundary="clamp")


def test_stencil2_on_different_extents_uses_the_intersection(ctx, P, torch_cuda, oracle, rng):
    t = torch_cuda
    a = rng.uniform(0, 1, (40, 100)).astype(np.float32)
    b = rng.uniform(0, 1, (37, 120)).astype(np.float32)
    out = t.zeros((37, 100), dtype=t.float32, device="cuda")
    ctx.stencil2(P.STENCIL2_SUM, dev(t, a), dev(t, b), out, boundary="clamp")
    ctx.sync()
    w1 = np.array([[0, 0, 0], [0.5, 1, 0.5], [0, 0, 0]], np.float64)
    w2 = np.array([[0, 0.25, 0], [0, -1, 0], [0, 0.25, 0]], np.float64)
    close(out.cpu().numpy(), oracle.stencil2_2d(a, b, w1, w2, "clamp"), 1e-6)


# ------------------------------------------------- generators and programs
def test_device_generators_match_the_host_definition(ctx, torch_cuda, workloads):
    t = torch_cuda
    W = workloads
    n, first = 100003, 12345
    f = t.empty(n, dtype=t.float32, device="cuda")
    ctx.gen_uniform_f32(f, n, first, W.SEED, W.S_SPOT, 5.0, 30.0)
    i = t.empty(n, dtype=t.int32, device="cuda")
    ctx.gen_uniform_i32(i, n, first, W.SEED, W.S_SCAN, 16)
    cdf = W.zipf_cdf()
    k = t.empty(n, dtype=t.int32, device="cuda")
    ctx.gen_zipf_mix_i32(k, n, first, W.SEED, dev(t, cdf), cdf.size)
    ctx.sync()
    assert np.array_equal(f.cpu().numpy(), W.uniform_f32(W.SEED, W.S_SPOT, n, 5.0, 30.0, first))
    assert np.array_equal(i.cpu().numpy(), W.uniform_i32(W.SEED, W.S_SCAN, n, 16, first))
    assert np.array_equal(k.cpu().numpy(), W.zipf_mix_keys(W.SEED, n, cdf, first))


# ------------------------------------------------------------------ maximum sizes
def test_arrays_of_the_largest_size_the_abi_can_describe(ctx, P, torch_cuda):
    """Extents are C ints: 2^31 - 2 elements is the largest vector whose scanl result (one longer) still has
    an Int32 extent.  Positions inside the kernels are 64-bit (the reference's are 32-bit ints,
    CodeGen/Base.hs:144-145)."""
    t = torch_cuda
    if t.cuda.mem_get_info()[0] < 40 << 30:
        pytest.skip("needs 40 GB of free device memory")
    n = (1 << 31) - 2
    x = t.ones(n, dtype=t.int32, device="cuda")
    x[12345] = 7
    out = t.empty(n + 1, dtype=t.int32, device="cuda")
    ctx.scan(P.SCAN_ADD_I32, [x], n, out, seed=np.int32(0))
    tot = t.zeros(1, dtype=t.int32, device="cuda")
    ctx.fold_all(P.SUM_I32, [x], n, tot, seed=np.int32(0))
    ctx.sync()
    wrapped = np.array((n + 6) & 0xffffffff, np.uint32).astype(np.int32)  # the sum wraps past 2^31
    assert (int(out[0]), int(out[12345]), int(out[12346]), int(out[-1])) == (0, 12345, 12352, int(wrapped))
    assert int(tot[0]) == int(wrapped)
    del out
    y = t.empty(n, dtype=t.int32, device="cuda")
    ctx.map(P.IOTA_SQ, [], y)  # o = (int)(i * i + 1) with a 64-bit i
    ctx.sync()
    assert (int(y[0]), int(y[3]), int(y[-1])) == (1, 10, int(np.array(((n - 1) ** 2 + 1) & 0xffffffff, np.uint32).astype(np.int32)))
    del y
    keys = (t.arange(n, dtype=t.int64, device="cuda") % 4096).int()
    h, z = t.zeros(4096, dtype=t.int32, device="cuda"), t.zeros(4096, dtype=t.int32, device="cuda")
    ctx.permute(P.HIST, [keys], n, h, defaults=z)
    ctx.sync()
    assert int(h.sum(dtype=t.int64)) == n and int(h[0]) == 524288 and int(h[4095]) == 524287
