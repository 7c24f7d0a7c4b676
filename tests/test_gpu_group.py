"""Several GPUs from one process (accb_group_*): the joined result of the slabs equals the oracle's result on the
whole array.  A device may be listed more than once, so the exchange logic (totals, carries, merged destinations,
halo rows) is exercised on a single GPU as well; with two or more GPUs the same cases run across devices."""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu

RTOL = 1e-5


def device_lists(torch):
    lists = [[0], [0, 0], [0, 0, 0]]
    n = torch.cuda.device_count()
    if n >= 2:
        lists.append([0, 1])
    return lists


@pytest.fixture(scope="module", params=range(4))
def group(request, accb, torch_cuda):
    lists = device_lists(torch_cuda)
    if request.param >= len(lists):
        pytest.skip("needs more GPUs")
    g = accb.Group(lists[request.param])
    yield g
    g.sync()
    g.destroy()


def cuts(n, parts, rng, align=1):
    """Uneven slab boundaries, every slab non-empty."""
    if parts == 1:
        return [0, n]
    inner = np.sort(rng.choice(np.arange(1, n // align), parts - 1, replace=False)) * align
    return [0] + [int(c) for c in inner] + [n]


def put(torch, a, device):
    return torch.from_numpy(np.ascontiguousarray(a)).to(f"cuda:{device}")


def sync_all(torch):
    for d in range(torch.cuda.device_count()):
        torch.cuda.synchronize(d)


def close(got, ref, atol):
    got, ref = np.asarray(got, np.float64), np.asarray(ref, np.float64)
    assert np.all(np.abs(got - ref) <= RTOL * np.abs(ref) + atol)


def test_group_map_and_row_folds(group, P, torch_cuda, oracle, rng):
    t, G = torch_cuda, group.size
    n = 50001
    x, y = rng.standard_normal(n).astype(np.float32), rng.standard_normal(n).astype(np.float32)
    c = cuts(n, G, rng)
    env = [[put(t, x[c[r]:c[r + 1]], group.devices[r]), put(t, y[c[r]:c[r + 1]], group.devices[r])] for r in range(G)]
    out = [t.empty(c[r + 1] - c[r], dtype=t.float32, device=f"cuda:{group.devices[r]}") for r in range(G)]
    sync_all(t)
    group.map(P.SAXPY, env, out, scalars=np.float32(0.5))
    group.sync()
    close(np.concatenate([o.cpu().numpy() for o in out]), np.float32(0.5) * x + y, 1e-6)

    rows, cols = 301, 517
    m = rng.standard_normal((rows, cols)).astype(np.float32)
    c = cuts(rows, G, rng)
    env = [[put(t, m[c[r]:c[r + 1]], group.devices[r])] for r in range(G)]
    out = [t.empty(c[r + 1] - c[r], dtype=t.float32, device=f"cuda:{group.devices[r]}") for r in range(G)]
    sync_all(t)
    group.fold_dim(P.ROWSUM, env, [c[r + 1] - c[r] for r in range(G)], cols, out, seed=np.float32(0))
    group.sync()
    close(np.concatenate([o.cpu().numpy() for o in out]), oracle.fold_rows_f32(m), 1e-5)


@pytest.mark.parametrize("n", [7, 100003, (1 << 21) + 5])
def test_group_dot_product(group, P, torch_cuda, oracle, rng, n):
    t, G = torch_cuda, group.size
    if n < G:
        pytest.skip("fewer elements than ranks")
    x, y = rng.uniform(-1, 1, n).astype(np.float32), rng.uniform(-1, 1, n).astype(np.float32)
    c = cuts(n, G, rng)
    env = [[put(t, x[c[r]:c[r + 1]], group.devices[r]), put(t, y[c[r]:c[r + 1]], group.devices[r])] for r in range(G)]
    out = [t.zeros(1, dtype=t.float32, device=f"cuda:{group.devices[r]}") for r in range(G)]
    sync_all(t)
    for _ in range(2):  # twice: the second call reuses the exchange areas behind the first
        group.fold_all(P.DOT, P.SUM_F32, env, [c[r + 1] - c[r] for r in range(G)], out, seed=np.float32(1.5))
    group.sync()
    ref = oracle.dot_f32(x, y, 1.5)
    scale = float(np.sum(np.abs(x.astype(np.float64) * y))) + 1.5
    for o in out:  # every rank holds the result
        assert abs(float(o.cpu()[0]) - ref) <= 1e-6 * scale
    assert len({float(o.cpu()[0]) for o in out}) == 1


SCANS = [("l", "excl"), ("l", "incl"), ("l", "prime"), ("r", "excl"), ("r", "incl"), ("r", "prime")]


@pytest.mark.parametrize("direction,kind", SCANS)
@pytest.mark.parametrize("n", [5, 40000, (1 << 20) + 3])
def test_group_scans_match_the_scan_of_the_whole_vector(group, accb, P, torch_cuda, oracle, rng, direction, kind, n):
    t, G = torch_cuda, group.size
    if n < G:
        pytest.skip("fewer elements than ranks")
    x = rng.integers(-50, 50, n).astype(np.int32)
    seed = 7
    c = cuts(n, G, rng)
    lens = [c[r + 1] - c[r] for r in range(G)]
    env = [[put(t, x[c[r]:c[r + 1]], group.devices[r])] for r in range(G)]
    extra = [1 if (kind == "excl" and r == G - 1) else 0 for r in range(G)]
    out = [t.full((lens[r] + extra[r],), -1, dtype=t.int32, device=f"cuda:{group.devices[r]}") for r in range(G)]
    tot = [t.full((1,), -1, dtype=t.int32, device=f"cuda:{group.devices[r]}") for r in range(G)]
    sync_all(t)
    k = {"excl": accb.SCAN_EXCLUSIVE, "incl": accb.SCAN_INCLUSIVE, "prime": accb.SCAN_PRIME}[kind]
    d = accb.SCAN_LEFT if direction == "l" else accb.SCAN_RIGHT
    group.scan(P.SCAN_ADD_I32, P.SUM_I32, P.SCAN_ADD_I32, env, lens, out, direction=d, kind=k,
               seed=None if kind == "incl" else np.int32(seed), total=tot if kind == "prime" else None)
    group.sync()
    got = np.concatenate([o.cpu().numpy() for o in out])
    if kind == "excl":
        ref = oracle.scanl_i32(x, seed) if direction == "l" else oracle.scanr_i32(x, seed)
    elif kind == "incl":
        ref = oracle.scanl1_i32(x) if direction == "l" else oracle.scanr1_i32(x)
    else:
        ref, total = oracle.scanl_prime_i32(x, seed) if direction == "l" else oracle.scanr_prime_i32(x, seed)
        assert int(tot[G - 1 if direction == "l" else 0].cpu()[0]) == np.int32(total)
    assert np.array_equal(got, ref)


def test_group_scan_refuses_what_it_cannot_shard(group, accb, P, torch_cuda):
    t, G = torch_cuda, group.size
    env = [[t.zeros(4, dtype=t.int32, device=f"cuda:{group.devices[r]}")] for r in range(G)]
    out = [t.zeros(5, dtype=t.int32, device=f"cuda:{group.devices[r]}") for r in range(G)]
    with pytest.raises(accb.AccbError):  # an empty slab
        group.scan(P.SCAN_ADD_I32, P.SUM_I32, P.SCAN_ADD_I32, env, [4] * (G - 1) + [0], out, seed=np.int32(0))
    with pytest.raises(accb.AccbError):  # scanl1 takes no seed
        group.scan(P.SCAN_ADD_I32, P.SUM_I32, P.SCAN_ADD_I32, env, [4] * G, out, kind=accb.SCAN_INCLUSIVE,
                   seed=np.int32(0))
    group.sync()


@pytest.mark.parametrize("n,bins", [(100, 16), (300007, 4096), (1 << 21, 4096)])
def test_group_histogram(group, P, torch_cuda, oracle, rng, n, bins):
    t, G = torch_cuda, group.size
    if n < G:
        pytest.skip("fewer elements than ranks")
    keys = rng.integers(0, bins, n).astype(np.int32)
    defaults = rng.integers(0, 100, bins).astype(np.int32)
    c = cuts(n, G, rng)
    env = [[put(t, keys[c[r]:c[r + 1]], group.devices[r])] for r in range(G)]
    out = [put(t, defaults if r == 0 else np.zeros(bins, np.int32), group.devices[r]) for r in range(G)]
    sync_all(t)
    group.permute(P.HIST, P.ZIP_ADD_I32, env, [c[r + 1] - c[r] for r in range(G)], out, broadcast=True)
    group.sync()
    ref = oracle.permute_add_i32(keys, bins, defaults)
    for o in out:
        assert np.array_equal(o.cpu().numpy(), ref)


@pytest.mark.parametrize("boundary", ["clamp", "mirror", "wrap", "constant"])
@pytest.mark.parametrize("iters", [1, 4])
def test_group_iterated_blur_with_one_halo_exchange(group, P, torch_cuda, oracle, workloads, rng, boundary, iters):
    t, G = torch_cuda, group.size
    h, w = 64 * G + 11, 256
    a = rng.uniform(0, 1, (h, w)).astype(np.float32)
    c = cuts(h, G, rng)
    if min(c[r + 1] - c[r] for r in range(G)) < iters:  # a slab must own at least the halo it sends
        c = [r * (h // G) for r in range(G)] + [h]
    rows = [c[r + 1] - c[r] for r in range(G)]
    pads = [group.stencil_layout(r, iters, 1, boundary) for r in range(G)]
    A, B = [], []
    for r in range(G):
        pt, pb = pads[r]
        slab = np.full((pt + rows[r] + pb, w), np.nan, np.float32)  # halos start as garbage
        slab[pt:pt + rows[r]] = a[c[r]:c[r + 1]]
        A.append(put(t, slab, group.devices[r]))
        B.append(t.empty_like(A[-1]))
    sync_all(t)
    res = group.stencil_iterate(P.BLUR, A, B, rows, iters, 1, boundary, constant=np.float32(0.25))
    group.sync()
    got = np.concatenate([res[r].cpu().numpy()[pads[r][0]:pads[r][0] + rows[r]] for r in range(G)])
    close(got, oracle.stencil2d_iter(a, workloads.BLUR_WEIGHTS, iters, boundary, 0.25), 1e-6)


def test_group_stencil_slabs_that_take_different_numbers_of_launches(group, P, torch_cuda, oracle, workloads, rng):
    """A slab of 16 rows and more runs two applications per launch, a thinner one runs them one by one, so the ranks
    end in different buffers of their pairs: the answer is still the same-named buffer on every rank."""
    t, G = torch_cuda, group.size
    if G < 2:
        pytest.skip("one rank has one slab")
    iters, w = 3, 256
    rows = [24] + [9] * (G - 1)  # rank 0: 24 + 3 halo rows; the others 3 + 9 (+ 3): fewer than 16 only for the last
    h = sum(rows)
    a = rng.uniform(0, 1, (h, w)).astype(np.float32)
    c = np.concatenate([[0], np.cumsum(rows)])
    pads = [group.stencil_layout(r, iters, 1, "clamp") for r in range(G)]
    A, B = [], []
    for r in range(G):
        pt, pb = pads[r]
        slab = np.full((pt + rows[r] + pb, w), np.nan, np.float32)
        slab[pt:pt + rows[r]] = a[c[r]:c[r + 1]]
        A.append(put(t, slab, group.devices[r]))
        B.append(t.empty_like(A[-1]))
    assert A[0].shape[0] >= 16 and A[-1].shape[0] < 16
    sync_all(t)
    res = group.stencil_iterate(P.BLUR, A, B, rows, iters, 1, "clamp")
    group.sync()
    got = np.concatenate([res[r].cpu().numpy()[pads[r][0]:pads[r][0] + rows[r]] for r in range(G)])
    close(got, oracle.stencil2d_iter(a, workloads.BLUR_WEIGHTS, iters, "clamp"), 1e-6)


@pytest.mark.parametrize("boundary", ["clamp", "mirror", "wrap", "constant"])
@pytest.mark.parametrize("iters", [1, 3])
def test_group_iterated_stencil_over_a_cube_cut_into_slabs_of_planes(group, P, torch_cuda, oracle, rng, boundary, iters):
    """Rank 3: the slabs are runs of planes, a halo "row" is a whole plane (the 27-tap weighted stencil of the rank-3
    skeleton, applied iters times with one halo exchange)."""
    t, G = torch_cuda, group.size
    d, h, w = 12 * G + 5, 21, 132
    a = rng.uniform(0, 1, (d, h, w)).astype(np.float32)
    c = [r * (d // G) for r in range(G)] + [d]
    planes = [c[r + 1] - c[r] for r in range(G)]
    pads = [group.stencil_layout(r, iters, 1, boundary) for r in range(G)]
    A, B = [], []
    for r in range(G):
        pt, pb = pads[r]
        slab = np.full((pt + planes[r] + pb, h, w), np.nan, np.float32)
        slab[pt:pt + planes[r]] = a[c[r]:c[r + 1]]
        A.append(put(t, slab, group.devices[r]))
        B.append(t.empty_like(A[-1]))
    sync_all(t)
    res = group.stencil_iterate(P.WEIGHTED27, A, B, planes, iters, 1, boundary, constant=np.float32(0.25))
    group.sync()
    got = np.concatenate([res[r].cpu().numpy()[pads[r][0]:pads[r][0] + planes[r]] for r in range(G)])
    w27 = (np.arange(27, dtype=np.float64).reshape(3, 3, 3) + 1) / 378.0
    ref = a.astype(np.float64)
    for _ in range(iters):
        ref = oracle.stencil3d(ref.astype(np.float32), w27, boundary, 0.25)
    close(got, ref, 1e-5)


@pytest.mark.parametrize("boundary", ["clamp", "mirror", "wrap", "constant"])
def test_group_stencil2_on_row_slabs(group, P, torch_cuda, oracle, rng, boundary):
    """stencil2 over two matrices dealt out as row slabs: both sources' halo rows come from the neighbours
    (Execute.hs:427-450 on one device)."""
    t, G = torch_cuda, group.size
    h, w = 40 * G + 7, 128
    a, b = rng.uniform(0, 1, (h, w)).astype(np.float32), rng.uniform(0, 1, (h, w)).astype(np.float32)
    c = cuts(h, G, rng)
    rows = [c[r + 1] - c[r] for r in range(G)]
    pads = [group.stencil_layout(r, 1, 1, boundary) for r in range(G)]
    A, B, O = [], [], []
    for r in range(G):
        pt, pb = pads[r]
        for src, dst in ((a, A), (b, B)):
            slab = np.full((pt + rows[r] + pb, w), np.nan, np.float32)
            slab[pt:pt + rows[r]] = src[c[r]:c[r + 1]]
            dst.append(put(t, slab, group.devices[r]))
        O.append(t.empty_like(A[-1]))
    sync_all(t)
    group.stencil2(P.STENCIL2_SUM, A, B, O, rows, 1, boundary, constant=np.float32(0.25))
    group.sync()
    got = np.concatenate([O[r].cpu().numpy()[pads[r][0]:pads[r][0] + rows[r]] for r in range(G)])
    w1 = np.zeros((3, 3)); w1[1, 1] = 1; w1[1, 0] = w1[1, 2] = 0.5
    w2 = np.zeros((3, 3)); w2[0, 1] = w2[2, 1] = 0.25; w2[1, 1] = -1
    close(got, oracle.stencil2_2d(a, b, w1, w2, boundary, 0.25), 1e-6)


@pytest.mark.parametrize("nseg,mean", [(1, 5), (10, 3), (5000, 7), (300, 900)])
def test_group_fold_seg_split_between_segments(group, accb, P, torch_cuda, oracle, rng, nseg, mean):
    """foldSeg over a vector split BETWEEN segments: every rank gets a run of whole segments holding about the same
    number of elements, its offsets rebased on the device (Execute.hs:320-324 on one device)."""
    t, G = torch_cuda, group.size
    lens = rng.integers(0, 2 * mean + 1, nseg).astype(np.int32)
    offs = np.concatenate([[0], np.cumsum(lens)]).astype(np.int32)
    n = int(offs[-1])
    x = rng.integers(-50, 50, max(n, 1)).astype(np.int32)[:n]
    first = accb.seg_partition(offs, G)
    sh = __import__("importlib").import_module("accelerate-cuda_b200.sharded")
    assert first == sh.segment_partition(offs, G) and first[0] == 0 and first[-1] == nseg and sorted(first) == first
    env, runs, out, cnt, segs = [], [], [], [], []
    for r in range(G):
        s0, s1 = first[r], first[r + 1]
        lo, hi = int(offs[s0]), int(offs[s1])
        dev = group.devices[r]
        env.append([put(t, np.concatenate([x[lo:hi], np.zeros(1, np.int32)]), dev)[:hi - lo]])
        runs.append(put(t, offs[s0:s1 + 1], dev))  # as they stand in the whole array: not starting at zero
        out.append(t.full((max(s1 - s0, 1),), -99, dtype=t.int32, device=f"cuda:{dev}")[:s1 - s0])
        cnt.append(hi - lo)
        segs.append(s1 - s0)
    sync_all(t)
    group.fold_seg(P.SEGSUM_I32, env, cnt, runs, segs, out, seed=np.int32(3))
    group.sync()
    got = np.concatenate([o.cpu().numpy() for o in out])
    assert np.array_equal(got, oracle.fold_seg_i32(x, offs, 3))
    if G > 1 and nseg >= 300:  # the cuts balance elements, not segments
        assert max(cnt) <= 1.5 * n / G + 2 * (2 * mean + 1)


def test_group_stencil_refuses_a_slab_smaller_than_its_halo(group, accb, P, torch_cuda):
    t, G = torch_cuda, group.size
    if G == 1:
        pytest.skip("one rank exchanges nothing")
    iters, rows = 8, [4] * G
    A = []
    for r in range(G):
        pt, pb = group.stencil_layout(r, iters, 1, "clamp")
        A.append(t.zeros((pt + rows[r] + pb, 64), dtype=t.float32, device=f"cuda:{group.devices[r]}"))
    B = [t.empty_like(x) for x in A]
    with pytest.raises(accb.AccbError):
        group.stencil_iterate(P.BLUR, A, B, rows, iters, 1, "clamp")
    group.sync()


_D = "static __device__ __forceinline__"
MINMAX_BODY = f"""
    typedef LH elem; typedef LH acc;
    using Out = accb::types<float, float>;
    {_D} LH lift(LH x) {{ return x; }}
    {_D} LH lower(LH x) {{ return x; }}
    {_D} LH combine(LH a, LH b) {{ LH r; r.lo = fminf(a.lo, b.lo); r.hi = fmaxf(a.hi, b.hi); return r; }}
    {_D} void put(LH r, float &lo, float &hi) {{ lo = r.lo; hi = r.hi; }}
"""


def test_group_fold_of_pairs_and_permute_with_max(group, accb, P, torch_cuda, rng):
    """A two-component value (min, max) through the partial exchange, and a permute whose combiner is not (+):
    partial destinations start from the combiner's neutral element and are merged with a zipWith of the combiner."""
    t, G = torch_cuda, group.size
    minmax = accb.KernelSpec("fold_all", "MinMax", f"""
struct LH {{ float lo, hi; }};
struct MinMax {{
    using In = accb::types<float>;
    {_D} LH get(const accb::Env &, long long, float x) {{ LH r; r.lo = x; r.hi = x; return r; }}
{MINMAX_BODY}}};
""")
    minmax_pairs = accb.KernelSpec("fold_all", "MinMaxP", f"""
struct LH {{ float lo, hi; }};
struct MinMaxP {{
    using In = accb::types<float, float>;
    {_D} LH get(const accb::Env &, long long, float lo, float hi) {{ LH r; r.lo = lo; r.hi = hi; return r; }}
{MINMAX_BODY}}};
""")
    n = 200003
    x = rng.standard_normal(n).astype(np.float32)
    c = cuts(n, G, rng)
    env = [[put(t, x[c[r]:c[r + 1]], group.devices[r])] for r in range(G)]
    out = [(t.zeros(1, device=f"cuda:{group.devices[r]}"), t.zeros(1, device=f"cuda:{group.devices[r]}")) for r in range(G)]
    sync_all(t)
    group.fold_all(minmax, minmax_pairs, env, [c[r + 1] - c[r] for r in range(G)], out)  # fold1All: no seed
    group.sync()
    for lo, hi in out:
        assert float(lo.cpu()[0]) == x.min() and float(hi.cpu()[0]) == x.max()

    zip_max = accb.KernelSpec("map", "ZipMaxF", f"""
struct ZipMaxF {{
    using In = accb::types<float, float>;
    using Out = accb::types<float>;
    {_D} void apply(const accb::Env &, long long, float a, float b, float &o) {{ o = fmaxf(a, b); }}
}};
""")
    bins = 1000
    keys = rng.integers(0, bins, n).astype(np.int32)
    defaults = rng.standard_normal(bins).astype(np.float32)
    env = [[(put(t, keys[c[r]:c[r + 1]], group.devices[r]), put(t, x[c[r]:c[r + 1]], group.devices[r]))] for r in range(G)]
    dst = [put(t, defaults if r == 0 else np.full(bins, -np.inf, np.float32), group.devices[r]) for r in range(G)]
    sync_all(t)
    group.permute(P.SCATTER_MAX_F32, zip_max, env, [c[r + 1] - c[r] for r in range(G)], dst)
    group.sync()
    ref = defaults.copy()
    np.maximum.at(ref, keys, x)
    assert np.array_equal(dst[0].cpu().numpy(), ref)
