"""Whole programs: run / run1 / runWith on host arrays (upload, launch, download) and the
AccFFI.h surface (accelerateCreate, runProgram, freeOutput, freeProgram) on device arrays."""
import ctypes as C

import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def test_run1_scan_small_and_pipelined(accb, P, ctx, oracle, rng):
    """run1 compiles once and is applied to several host arrays (CUDA.hs:307-330); inputs of at
    least two 2^24-element chunks take the pipelined upload / scan / download path."""
    scan = accb.run1With(ctx, lambda v: accb.scan(P.SCAN_ADD_I32, [v], np.int32, seed=np.int32(3)),
                         accb.ArrayType(1, np.int32))
    for n in (10, 100003, (1 << 25) + 12345):
        x = rng.integers(0, 16, n).astype(np.int32)
        assert np.array_equal(scan(x), oracle.scanl_i32(x, 3))
    scan.destroy()


def test_run1_scan_prime_returns_body_and_total(accb, P, ctx, oracle, rng):
    f = accb.run1With(ctx, lambda v: accb.scan(P.SCAN_ADD_I32, [v], np.int32, kind=accb.SCAN_PRIME, seed=np.int32(0)),
                      accb.ArrayType(1, np.int32))
    x = rng.integers(-50, 50, 70001).astype(np.int32)
    body, total = f(x)
    rb, rt = oracle.scanl_prime_i32(x, 0)
    assert np.array_equal(body, rb) and total.shape == () and int(total) == rt
    f.destroy()


def test_runWith_dot_product_program(accb, P, ctx, oracle, rng):
    """foldAll (+) 0 (zipWith (*) xs ys) arrives as ONE fold over a fused producer (CodeGen.hs:104)."""
    xs = rng.uniform(-1, 1, 1 << 20).astype(np.float32)
    ys = rng.uniform(-1, 1, 1 << 20).astype(np.float32)
    r = accb.runWith(ctx, lambda a, b: accb.fold(P.DOT, [a, b], np.float32, seed=np.float32(0), all=True), xs, ys)
    ref = oracle.dot_f32(xs, ys)
    assert r.shape == () and abs(float(r) - ref) <= 1e-5 * abs(ref)


def test_program_chain_map_then_row_fold(accb, P, ctx, oracle, rng):
    """let-bound chain: an intermediate array lives on the device only."""
    def prog(x, y):
        z = accb.map_(P.SAXPY, [x, y], accb.ArrayType(2, np.float32), scalars=np.float32(2.0))
        return accb.fold(P.ROWSUM, [z], np.float32, seed=np.float32(0))
    x = rng.uniform(-1, 1, (33, 2100)).astype(np.float32)
    y = rng.uniform(-1, 1, (33, 2100)).astype(np.float32)
    r = accb.runWith(ctx, prog, x, y)
    ref = oracle.fold_rows_f32((np.float32(2.0) * x + y).astype(np.float32))
    assert r.shape == (33,) and np.all(np.abs(r - ref) <= 1e-5 * np.abs(ref) + 1e-5)


def test_program_histogram_and_iterated_stencil(accb, P, ctx, oracle, workloads, rng):
    W = workloads
    keys = W.zipf_mix_keys(W.SEED, 200001, W.zipf_cdf())
    zeros = np.zeros(W.HIST_BINS, np.int32)
    h = accb.runWith(ctx, lambda k, d: accb.permute(P.HIST, [k], d), keys, zeros)
    assert np.array_equal(h, oracle.permute_add_i32(keys, W.HIST_BINS))
    g = rng.uniform(0, 1, (96, 260)).astype(np.float32)
    for iters in (1, 2, 5):
        r = accb.runWith(ctx, lambda a: accb.stencil(P.BLUR, a, boundary="clamp", iters=iters), g)
        ref = oracle.stencil2d_iter(g, W.BLUR_WEIGHTS, iters, "clamp")
        assert np.all(np.abs(r - ref) <= 1e-5 * np.abs(ref) + 1e-6)


def test_blackscholes_program_with_tuple_input_and_output(accb, P, ctx, oracle, workloads):
    W = workloads
    n = 50000
    s = W.uniform_f32(W.SEED, W.S_SPOT, n, 5, 30)
    k = W.uniform_f32(W.SEED, W.S_STRIKE, n, 1, 100)
    y = W.uniform_f32(W.SEED, W.S_YEARS, n, 0.25, 10)
    f = accb.run1With(ctx, lambda o: accb.map_(P.BLACKSCHOLES, [o], accb.ArrayType(1, [np.float32, np.float32])),
                      accb.ArrayType(1, [np.float32] * 3))
    call, put = f((s, k, y))
    rc, rp = oracle.blackscholes(s, k, y)
    assert np.all(np.abs(call - rc) <= 1e-5 * np.abs(rc) + 2e-5) and np.all(np.abs(put - rp) <= 1e-5 * np.abs(rp) + 2e-5)
    ca, pa = accb.runWith(ctx, lambda o: accb.map_(P.BLACKSCHOLES_ACCURATE, [o], accb.ArrayType(1, [np.float32] * 2)), (s, k, y))
    assert np.all(np.abs(ca - rc) <= 1e-5 * np.abs(rc) + 2e-5) and np.all(np.abs(pa - rp) <= 1e-5 * np.abs(rp) + 2e-5)
    f.destroy()


def test_accffi_surface_runProgram_on_device_arrays(accb, P, torch_cuda, oracle, rng):
    """accelerateCreate / runProgram / freeOutput / freeProgram / accelerateDestroy with the struct
    layouts of include/AccFFI.h:10-19: borrowed input pointers, library-owned outputs."""
    t = torch_cuda
    L = accb.lib()
    h = L.accelerateCreate(0, None)
    assert h
    cctx = L.accelerateContext(h)
    shim = accb.Context.__new__(accb.Context)  # a Context object around the handle's context
    shim.handle, shim.device, shim._kernels = C.c_void_p(cctx), 0, {}
    prog = accb.run1With(shim, lambda v: accb.scan(P.SCAN_ADD_I32, [v], np.int32, seed=np.int32(0)),
                         accb.ArrayType(1, np.int32))
    n = 123457
    x = rng.integers(0, 16, n).astype(np.int32)
    xd = t.from_numpy(x).cuda()
    shape = (C.c_int * 1)(n)
    ptrs = (C.c_void_p * 1)(xd.data_ptr())
    inp = accb.InputArray(C.cast(shape, C.POINTER(C.c_int)), C.cast(ptrs, C.POINTER(C.c_void_p)))
    out = accb.OutputArray()
    L.runProgram(h, prog.handle, C.byref(inp), C.byref(out))
    assert L.accelerateStatus(h) == accb.OK
    assert out.shape[0] == n + 1
    host = np.empty(n + 1, np.int32)
    acc = accb.lib()
    # read the library-owned result through the memory table API: register the pointer as
    # unmanaged (insertUnmanaged, Array/Remote.hs:168-184), then peek
    key = 0xABCDEF
    assert acc.accb_insert_unmanaged(cctx, key, C.c_void_p(out.adata[0]), (n + 1) * 4) == accb.OK
    assert acc.accb_peek(cctx, key, 0, host.ctypes.data_as(C.c_void_p), (n + 1) * 4, None) == accb.OK
    assert acc.accb_context_sync(cctx) == accb.OK
    assert acc.accb_free(cctx, key) == accb.OK
    assert np.array_equal(host, oracle.scanl_i32(x, 0))
    L.freeOutput(C.byref(out))
    assert not out.adata
    L.freeProgram(prog.handle)
    prog.handle = None
    L.accelerateDestroy(h)


class _DevView:
    """A device pointer as something torch.as_tensor understands."""

    def __init__(self, a, typestr):
        shape = tuple(a.shape[d] for d in reversed(range(a.rank)))
        self.__cuda_array_interface__ = {"shape": shape, "typestr": typestr, "data": (int(a.ptr[0]), False), "version": 2}


def test_program_as_one_cuda_graph_replays_on_new_contents(accb, ctx, torch_cuda, rng):
    """accb_program_run_graph: recorded once per set of input arrays, replayed on whatever they contain;
    the scan inside clears its tile status words in every replay."""
    import importlib
    t = torch_cuda
    A = importlib.import_module("accelerate-cuda_b200.lang")
    add = lambda a, b: a + b  # noqa: E731

    def prog(v):
        return (A.scanl1(add, A.map(lambda x: x * 2, v)), A.fold(add, 0, v),
                A.permute(add, A.fill(64, 0, np.int32), lambda i: v[i] & 63, A.fill(A.shape_of(v), 1, np.int32)))
    f = A.run1With(ctx, prog, A.vector(np.int32))
    n = 300001
    v = t.from_numpy(rng.integers(0, 1000, n).astype(np.int32)).cuda()
    s = t.cuda.Stream()
    launches = []
    for rep in range(4):
        if rep:
            v.add_(rep)  # new contents, same array
        t.cuda.synchronize()
        before = ctx.launch_count()
        outs = f.run_device([v], stream=s.cuda_stream, graph=True)
        s.synchronize()
        launches.append(ctx.launch_count() - before)
        h = v.cpu().numpy()
        got = [t.as_tensor(_DevView(o, "<i4"), device="cuda").cpu().numpy() for o in outs]
        assert np.array_equal(got[0], np.cumsum(2 * h.astype(np.int64)).astype(np.int32))
        assert got[1].reshape(-1)[0] == h.sum(dtype=np.int64).astype(np.int32)
        assert np.array_equal(got[2], np.bincount(h & 63, minlength=64).astype(np.int32))
    assert launches[0] > 0 and launches[1:] == [0, 0, 0]  # replays issue no launches of their own
    # another array: recorded again; and the ordinary path still agrees
    w = t.from_numpy(rng.integers(0, 1000, n).astype(np.int32)).cuda()
    o1 = f.run_device([w], stream=s.cuda_stream, graph=True)
    s.synchronize()
    a = t.as_tensor(_DevView(o1[0], "<i4"), device="cuda").clone()
    o2 = f.run_device([w], stream=s.cuda_stream)
    s.synchronize()
    assert t.equal(a, t.as_tensor(_DevView(o2[0], "<i4"), device="cuda"))
    # a larger run replaces the pooled intermediates and the scan scratch the recording names: recorded again
    big = t.from_numpy(rng.integers(0, 1000, 40 * n).astype(np.int32)).cuda()
    f.run_device([big], stream=s.cuda_stream)
    s.synchronize()
    before = ctx.launch_count()
    o3 = f.run_device([w], stream=s.cuda_stream, graph=True)
    s.synchronize()
    assert ctx.launch_count() > before and t.equal(a, t.as_tensor(_DevView(o3[0], "<i4"), device="cuda"))
    with pytest.raises(accb.AccbError):
        f.run_device([w], stream=None, graph=True)  # the default stream cannot be captured
    f.destroy()


def test_fold_seg_with_a_long_segment_inside_a_cuda_graph(accb, P, ctx, torch_cuda, rng):
    """A foldSeg over 18 M elements records two launches (the second one splits the segments that the first one put
    on its list over all blocks); replays follow the arrays' new contents, also when another segment becomes the
    long one."""
    t = torch_cuda
    nseg = 300000
    f = accb.run1With(ctx, lambda v, o: accb.fold_seg(P.SEGSUM_I32, [v], o, np.int32, seed=np.int32(2)),
                      accb.ArrayType(1, np.int32), accb.ArrayType(1, np.int32))
    lens = rng.integers(0, 100, nseg)
    lens[777] = 3_000_000
    n = int(lens.sum())
    x = t.from_numpy(rng.integers(-50, 50, n).astype(np.int32)).cuda()
    offs = t.from_numpy(np.concatenate([[0], np.cumsum(lens)]).astype(np.int32)).cuda()
    s = t.cuda.Stream()
    for rep in range(3):
        if rep == 1:
            x.add_(1)
        if rep == 2:  # the long segment moves: same arrays, other contents
            lens2 = lens.copy()
            lens2[777], lens2[231000] = lens[231000], lens[777]
            offs.copy_(t.from_numpy(np.concatenate([[0], np.cumsum(lens2)]).astype(np.int32)))
        t.cuda.synchronize()
        before = ctx.launch_count()
        outs = f.run_device([x, offs], stream=s.cuda_stream, graph=True)
        s.synchronize()
        assert (ctx.launch_count() - before == 0) == (rep > 0)
        got = t.as_tensor(_DevView(outs[0], "<i4"), device="cuda").cpu().numpy()
        h, o = x.cpu().numpy().astype(np.int64), offs.cpu().numpy()
        tot = np.concatenate([[0], np.cumsum(h)])
        assert np.array_equal(got, (tot[o[1:]] - tot[o[:-1]] + 2).astype(np.int32))
    ctx.sync()
    f.destroy()


# ------------------------------------------------------------- streamed host runs
_D = "static __device__ __forceinline__"


def _index_specs(accb):
    KS = accb.KernelSpec
    add_index = KS("map", "AddIndex", f"""
struct AddIndex {{
    using In = accb::types<int>;
    using Out = accb::types<int>;
    {_D} void apply(const accb::Env &, long long i, int x, int &o) {{ o = x + (int)(i % 1000003); }}
}};
""")
    weighted = KS("fold_all", "IndexWeighted", f"""
struct IndexWeighted : accb::Fold<int> {{
    using In = accb::types<int>;
    {_D} int get(const accb::Env &, long long i, int x) {{ return x * (int)(i % 7); }}
    {_D} int combine(int a, int b) {{ return (int)((unsigned)a + (unsigned)b); }}
}};
""")
    scatter = KS("permute", "IndexScatter", f"""
struct IndexScatter : accb::Permute<int, accb::Atomic::Add> {{
    using In = accb::types<int>;
    {_D} long long index(const accb::Env &, long long i, int) {{ return i % 977; }}
    {_D} int get(const accb::Env &, long long i, int x) {{ return x + (int)(i & 3); }}
    {_D} int combine(int x, int y) {{ return (int)((unsigned)x + (unsigned)y); }}
}};
""")
    return add_index, weighted, scatter


def _both_ways(accb, ctx, build, types, inputs, piece):
    """The same program run whole (the reference's upload / run / download) and in pieces of `piece` elements."""
    f = accb.run1With(ctx, build, *types)
    whole = f.stream_chunk(0)(*inputs)
    pieces = f.stream_chunk(piece)(*inputs)
    f.destroy()
    return whole, pieces


@pytest.mark.parametrize("n,piece", [(100003, 4096), (65536, 16384), (1 << 20, 100000), (33, 16)])
def test_streamed_runs_give_the_results_of_whole_runs(accb, P, ctx, oracle, workloads, rng, n, piece):
    """Maps, folds, the three left scans and permutes on host arrays, cut into many small pieces: bit-identical to
    the run that uploads everything first for integers, and the functor sees the same element indices."""
    add_index, weighted, scatter = _index_specs(accb)
    i32 = accb.ArrayType(1, np.int32)
    x = rng.integers(-100, 100, n).astype(np.int32)
    y = rng.integers(-100, 100, n).astype(np.int32)
    # map with the element index; zipWith of two streamed inputs
    w, s = _both_ways(accb, ctx, lambda a: accb.map_(add_index, [a], i32), [i32], [x], piece)
    assert np.array_equal(w, s) and np.array_equal(w, x + (np.arange(n) % 1000003).astype(np.int32))
    f32 = accb.ArrayType(1, np.float32)
    xf, yf = x.astype(np.float32) / 7, y.astype(np.float32) / 3
    w, s = _both_ways(accb, ctx, lambda a, b: accb.map_(P.SAXPY, [a, b], f32, scalars=np.float32(2.5)), [f32, f32], [xf, yf], piece)
    assert np.array_equal(w, s) and np.allclose(s, np.float32(2.5) * xf + yf, rtol=1e-6, atol=1e-4)
    # foldAll: index-dependent, with a seed; fold1 (no seed).  (Folds hand a thread every G-th element, as the
    # reference's do, so their combiners commute; only scans keep the order of the values.)
    w, s = _both_ways(accb, ctx, lambda a: accb.fold(weighted, [a], np.int32, seed=np.int32(11), all=True), [i32], [x], piece)
    assert int(w) == int(s) == int(np.int32((x.astype(np.int64) * (np.arange(n) % 7)).sum() + 11))
    w, s = _both_ways(accb, ctx, lambda a: accb.fold(P.MAX_I32, [a], np.int32, all=True), [i32], [x], piece)
    assert int(w) == int(s) == int(x.max())
    # scans
    for kind, ref in ((accb.SCAN_EXCLUSIVE, oracle.scanl_i32(x, 5)), (accb.SCAN_INCLUSIVE, oracle.scanl1_i32(x))):
        seed = None if kind == accb.SCAN_INCLUSIVE else np.int32(5)
        w, s = _both_ways(accb, ctx, lambda a: accb.scan(P.SCAN_ADD_I32, [a], np.int32, kind=kind, seed=seed), [i32], [x], piece)
        assert np.array_equal(w, ref) and np.array_equal(s, ref)
    w, s = _both_ways(accb, ctx, lambda a: accb.scan(P.SCAN_ADD_I32, [a], np.int32, kind=accb.SCAN_PRIME, seed=np.int32(-2)),
                      [i32], [x], piece)
    body, total = oracle.scanl_prime_i32(x, -2)
    assert np.array_equal(s[0], body) and int(s[1]) == total and np.array_equal(w[0], body) and int(w[1]) == total
    # permute: index-dependent scatter onto defaults that are uploaded once
    d = rng.integers(-5, 5, 977).astype(np.int32)
    w, s = _both_ways(accb, ctx, lambda a, dfl: accb.permute(scatter, [a], dfl), [i32, i32], [x, d], piece)
    ref = d.astype(np.int64).copy()
    np.add.at(ref, np.arange(n) % 977, x.astype(np.int64) + (np.arange(n) & 3))
    assert np.array_equal(w, s) and np.array_equal(s, ref.astype(np.int32))
    # a chain: the intermediate array never leaves the device
    w, s = _both_ways(accb, ctx, lambda a: accb.fold(weighted, [accb.map_(add_index, [a], i32)], np.int32, seed=np.int32(0), all=True),
                      [i32], [x], piece)
    assert int(w) == int(s)


def test_streamed_row_folds_and_tuple_maps(accb, P, ctx, oracle, workloads, rng):
    W = workloads
    m = rng.uniform(-1, 1, (4099, 260)).astype(np.float32)
    mt = accb.ArrayType(2, np.float32)
    w, s = _both_ways(accb, ctx, lambda a: accb.fold(P.ROWSUM, [a], np.float32, seed=np.float32(0)), [mt], [m], 260 * 64)
    ref = oracle.fold_rows_f32(m)
    assert s.shape == (4099,) and np.array_equal(w, s) and np.all(np.abs(s - ref) <= 1e-5 * np.abs(ref) + 1e-6)
    n = 70001
    opts = tuple(W.uniform_f32(W.SEED, st, n, lo, hi) for st, lo, hi in ((W.S_SPOT, 5, 30), (W.S_STRIKE, 1, 100), (W.S_YEARS, 0.25, 10)))
    w, s = _both_ways(accb, ctx, lambda o: accb.map_(P.BLACKSCHOLES, [o], accb.ArrayType(1, [np.float32, np.float32])),
                      [accb.ArrayType(1, [np.float32] * 3)], [opts], 8192)
    assert np.array_equal(w[0], s[0]) and np.array_equal(w[1], s[1])
    rc, _ = oracle.blackscholes(*opts)
    assert np.all(np.abs(s[0] - rc) <= 1e-5 * np.abs(rc) + 2e-5)
    # the dot product: float results of the two ways differ by the rounding of the carry between pieces only
    xs, ys = rng.uniform(-1, 1, 1 << 18).astype(np.float32), rng.uniform(-1, 1, 1 << 18).astype(np.float32)
    v = accb.ArrayType(1, np.float32)
    w, s = _both_ways(accb, ctx, lambda a, b: accb.fold(P.DOT, [a, b], np.float32, seed=np.float32(0), all=True), [v, v], [xs, ys], 1 << 14)
    ref = oracle.dot_f32(xs, ys)
    assert abs(float(w) - ref) <= 1e-5 * abs(ref) + 1e-5 and abs(float(s) - ref) <= 1e-5 * abs(ref) + 1e-5


@pytest.mark.parametrize("shape,boundary,iters,chunk", [((512, 260), "clamp", 3, 4096), ((1000, 256), "mirror", 5, 20000),
                                                        ((333, 1024), "constant", 2, 30000), ((2048, 130), "clamp", 10, 8000)])
def test_stencil_chains_run_slab_by_slab(accb, P, ctx, oracle, workloads, rng, shape, boundary, iters, chunk):
    """An iterated stencil on a host grid goes up, through the kernels and down in row slabs with a margin of
    iters rows either side: bit-identical to the run that uploads the whole grid first, and equal to the oracle's
    recurrence.  Then a chain of two different stencil nodes."""
    W = workloads
    g = rng.uniform(0, 1, shape).astype(np.float32)
    gt = accb.ArrayType(2, np.float32)
    const = np.float32(0.25) if boundary == "constant" else None
    w, s = _both_ways(accb, ctx, lambda a: accb.stencil(P.BLUR, a, boundary=boundary, iters=iters, constant=const), [gt], [g], chunk)
    assert s.shape == shape and np.array_equal(w, s)
    ref = oracle.stencil2d_iter(g, W.BLUR_WEIGHTS, iters, boundary, cval=0.25)
    assert np.all(np.abs(s - ref) <= 1e-5 * np.abs(ref) + 1e-6)
    w, s = _both_ways(accb, ctx, lambda a: accb.stencil(P.BLUR, accb.stencil(P.BLUR, a, boundary=boundary, iters=2, constant=const),
                                                          boundary="clamp", iters=1), [gt], [g], chunk)
    assert np.array_equal(w, s)


@pytest.mark.parametrize("boundary", ["clamp", "mirror", "constant"])
def test_cube_stencils_run_in_slabs_of_planes(accb, P, ctx, oracle, rng, boundary):
    """Rank 3 from host arrays: slabs of planes, each with the planes above and below that the applications reach;
    bit-identical to the whole-cube run."""
    c = rng.uniform(0, 1, (70, 24, 132)).astype(np.float32)
    ct = accb.ArrayType(3, np.float32)
    const = np.float32(0.25) if boundary == "constant" else None
    w, s = _both_ways(accb, ctx, lambda a: accb.stencil(P.WEIGHTED27, a, boundary=boundary, iters=2, constant=const), [ct], [c],
                      8 * 24 * 132)
    assert s.shape == c.shape and np.array_equal(w, s)
    w27 = (np.arange(27, dtype=np.float64).reshape(3, 3, 3) + 1) / 378.0
    ref = oracle.stencil3d(oracle.stencil3d(c, w27, boundary, 0.25).astype(np.float32), w27, boundary, 0.25)
    assert np.all(np.abs(s - ref) <= 1e-5 * np.abs(ref) + 1e-6)


def test_programs_that_do_not_fit_run_whole(accb, P, ctx, oracle, workloads, rng):
    """A Wrap stencil reaches across the whole grid and a right scan starts at the far end: such programs are not cut
    into pieces or slabs, whatever the piece size, and give the same results as before."""
    W = workloads
    g = rng.uniform(0, 1, (512, 260)).astype(np.float32)
    f = accb.run1With(ctx, lambda a: accb.stencil(P.BLUR, a, boundary="wrap", iters=3), accb.ArrayType(2, np.float32))
    r = f.stream_chunk(4096)(g)
    ref = oracle.stencil2d_iter(g, W.BLUR_WEIGHTS, 3, "wrap")
    assert np.all(np.abs(r - ref) <= 1e-5 * np.abs(ref) + 1e-6)
    f.destroy()
    x = rng.integers(-9, 9, 100003).astype(np.int32)
    f = accb.run1With(ctx, lambda a: accb.scan(P.SCAN_ADD_I32, [a], np.int32, direction=accb.SCAN_RIGHT, seed=np.int32(1)),
                      accb.ArrayType(1, np.int32))
    assert np.array_equal(f.stream_chunk(4096)(x), oracle.scanr_i32(x, 1))
    f.destroy()
