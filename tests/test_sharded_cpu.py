"""The multi-GPU host logic (slab partitioning, scan carry, histogram all-reduce,
stencil halo exchange) run as gloo ranks on CPU tensors.  The local work is done
by the CPU oracle here -- on a GPU it is the skeleton launches."""
import importlib
import os
import socket
import sys

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, case, ret):
    sys.path.insert(0, ROOT)
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        sh = importlib.import_module("accelerate-cuda_b200.sharded")
        W = importlib.import_module("accelerate-cuda_b200.workloads")
        oracle = importlib.import_module("oracle")
        ok = True
        if case == "scan":
            n = 100003
            x = W.uniform_i32(W.SEED, W.S_SCAN, n, 16)
            lo, hi = sh.slab(n, rank, world)
            # each rank generates only its slab: the generator is index-addressable
            xl = torch.from_numpy(W.uniform_i32(W.SEED, W.S_SCAN, hi - lo, 16, first=lo))
            total = lambda t: torch.tensor([int(t.sum(dtype=torch.int64)) & 0xffffffff], dtype=torch.int64).to(torch.int32)
            scan = lambda t, seed: torch.from_numpy(oracle.scanl_i32(t.numpy(), int(seed[0])))
            out = sh.sharded_scanl(xl, 7, total, scan)
            ref = oracle.scanl_i32(x, 7)
            hi_ref = hi + 1 if rank == world - 1 else hi
            ok = np.array_equal(out.numpy(), ref[lo:hi_ref])
        elif case == "hist":
            n = 50001
            cdf = W.zipf_cdf()
            lo, hi = sh.slab(n, rank, world)
            keys = W.zipf_mix_keys(W.SEED, hi - lo, cdf, first=lo)
            part = torch.from_numpy(oracle.permute_add_i32(keys, W.HIST_BINS))
            defaults = torch.arange(W.HIST_BINS, dtype=torch.int32)
            got = sh.sharded_histogram(part, defaults)
            ref = oracle.permute_add_i32(W.zipf_mix_keys(W.SEED, n, cdf), W.HIST_BINS, defaults=defaults.numpy())
            ok = np.array_equal(got.numpy(), ref)
        elif case == "dot":
            n = 70001
            lo, hi = sh.slab(n, rank, world)
            xs = W.uniform_f32(W.SEED, W.S_XS, hi - lo, -1, 1, first=lo)
            ys = W.uniform_f32(W.SEED, W.S_YS, hi - lo, -1, 1, first=lo)
            part = torch.tensor([oracle.dot_f32(xs, ys)], dtype=torch.float64)
            got = sh.sharded_fold_all(part, lambda a, b: a + b)
            ref = oracle.dot_f32(W.uniform_f32(W.SEED, W.S_XS, n, -1, 1), W.uniform_f32(W.SEED, W.S_YS, n, -1, 1))
            ok = abs(float(got[0]) - ref) <= 1e-12 * abs(ref)
        elif case == "foldseg":
            # split between segments: every rank folds a run of whole segments with its offsets rebased
            rng = np.random.default_rng(5)
            lens = rng.integers(0, 40, 2000).astype(np.int32)
            offs = np.concatenate([[0], np.cumsum(lens)]).astype(np.int32)
            x = rng.integers(-9, 9, int(offs[-1])).astype(np.int32)
            first = sh.segment_partition(offs, world)
            s0, s1 = first[rank], first[rank + 1]
            fold = lambda v, o: torch.from_numpy(oracle.fold_seg_i32(v.numpy(), o.numpy().astype(np.int32), 2))
            got = sh.sharded_fold_seg(torch.from_numpy(x[offs[s0]:offs[s1]]), torch.from_numpy(offs[s0:s1 + 1]), fold)
            ok = np.array_equal(got.numpy(), oracle.fold_seg_i32(x, offs, 2)[s0:s1])
            sizes = [int(offs[first[r + 1]] - offs[first[r]]) for r in range(world)]
            ok = ok and max(sizes) - min(sizes) <= 2 * 40  # the runs hold about the same number of elements
        elif case.startswith("stencil2"):
            mode = case.split("-")[1]
            h, w = 9 * world + 4, 24
            a = W.uniform_f32(W.SEED, W.S_GRID, h * w, 0, 1).reshape(h, w)
            b = W.uniform_f32(W.SEED, W.S_MATRIX, h * w, 0, 1).reshape(h, w)
            lo, hi = (rank * (h // world), (rank + 1) * (h // world) if rank < world - 1 else h)
            w1 = np.array([[0, 1, 0], [2, 3, 4], [0, 5, 0]], np.float64) / 15
            w2 = np.array([[1, 0, 2], [0, -1, 0], [3, 0, 4]], np.float64) / 9
            apply2 = lambda p, q: torch.from_numpy(oracle.stencil2_2d(p.numpy(), q.numpy(), w1, w2, mode))  # noqa: E731
            got = sh.sharded_stencil2(torch.from_numpy(a[lo:hi].copy()), torch.from_numpy(b[lo:hi].copy()), 1, apply2, boundary=mode)
            ok = np.allclose(got.numpy(), oracle.stencil2_2d(a, b, w1, w2, mode)[lo:hi], rtol=0, atol=1e-14)
        elif case.startswith("cube"):
            # rank 3: slabs of planes, a halo "row" is a plane
            mode = case.split("-")[1]
            d, h, w, iters = 6 * world + 3, 7, 12, 3
            g = W.uniform_f32(W.SEED, W.S_GRID, d * h * w, 0, 1).reshape(d, h, w).astype(np.float64)
            lo, hi = (rank * (d // world), (rank + 1) * (d // world) if rank < world - 1 else d)
            w27 = (np.arange(27, dtype=np.float64).reshape(3, 3, 3) + 1) / 378.0
            apply3 = lambda a: torch.from_numpy(oracle.stencil3d(a.numpy(), w27, mode))  # noqa: E731
            got = sh.sharded_stencil_iterate(torch.from_numpy(g[lo:hi].copy()), iters, 1, apply3, boundary=mode)
            ref = g
            for _ in range(iters):
                ref = oracle.stencil3d(ref, w27, mode)
            ok = np.allclose(got.numpy(), ref[lo:hi], rtol=0, atol=1e-14)
        elif case.startswith("stencil"):
            mode = case.split("-")[1]
            h, w, iters = 12 * world + 5, 40, 4
            g = W.uniform_f32(W.SEED, W.S_GRID, h * w, 0, 1).reshape(h, w).astype(np.float64)
            lo, hi = (rank * (h // world), (rank + 1) * (h // world) if rank < world - 1 else h)
            def apply(a, mode=mode):
                # the boundary in x is the kernel's; in y the halo rows already hold the right neighbours, so
                # what the kernel does beyond them only lands in halo rows, which the next exchange overwrites
                return torch.from_numpy(oracle.stencil2d(a.numpy(), W.BLUR_WEIGHTS, mode))
            def iterate(a, times):
                for _ in range(times):
                    a = apply(a)
                return a
            if case.startswith("stencilwide"):  # one exchange of iters rows each way, then iters applications
                got = sh.sharded_stencil_iterate_blocked(torch.from_numpy(g[lo:hi].copy()), iters, 1, iterate, boundary=mode)
            elif case.startswith("stencilshort"):  # slabs shorter than the wide halo: one exchange per application
                iters = 14
                got = sh.sharded_stencil_iterate_blocked(torch.from_numpy(g[lo:hi].copy()), iters, 1, iterate, boundary=mode)
            else:
                got = sh.sharded_stencil_iterate(torch.from_numpy(g[lo:hi].copy()), iters, 1, apply, boundary=mode)
            ref = g
            for _ in range(iters):
                ref = oracle.stencil2d(ref, W.BLUR_WEIGHTS, mode)
            ok = np.allclose(got.numpy(), ref[lo:hi], rtol=0, atol=1e-14)
        ret[rank] = bool(ok)
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world", [2, 3])
@pytest.mark.parametrize("case", ["scan", "hist", "dot", "stencil-clamp", "stencil-mirror", "stencil-wrap",
                                  "stencilwide-clamp", "stencilwide-mirror", "stencilwide-wrap", "stencilshort-clamp",
                                  "foldseg", "stencil2-clamp", "stencil2-mirror", "stencil2-wrap",
                                  "cube-clamp", "cube-mirror", "cube-wrap"])
def test_sharded_paths_match_the_single_device_oracle(case, world):
    mgr = mp.Manager()
    ret = mgr.dict()
    mp.spawn(_worker, args=(world, _free_port(), case, ret), nprocs=world, join=True)
    assert all(ret.get(r) for r in range(world)), dict(ret)


def test_slabs_partition_the_index_space_and_stay_aligned():
    sh = importlib.import_module("accelerate-cuda_b200.sharded")
    for n in (0, 1, 7, 1000, 1 << 20, (1 << 20) + 3):
        for world in (1, 2, 3, 8):
            edges = [sh.slab(n, r, world) for r in range(world)]
            assert edges[0][0] == 0 and edges[-1][1] == n
            assert all(edges[i][1] == edges[i + 1][0] for i in range(world - 1))
            assert all(lo % 4 == 0 for lo, _ in edges)


class _FakePeers:
    """The exchange buffers of all ranks as numpy arrays in one process: what peer_wide_halos asks of accb_peer_*
    (barrier, pull) replayed on the CPU, so that the offsets it computes can be checked without GPUs."""

    def __init__(self, world, nbytes):
        self.world, self.bufs = world, [np.zeros(nbytes, np.uint8) for _ in range(world)]
        self.base = [1 << 20] * world  # pretend device address of every rank's data area

    def view(self, rank):
        outer = self

        class Peer:
            world, data_ptr = outer.world, outer.base[rank]

            def __init__(self):
                self.rank, self.barriers, self.pulls = rank, 0, []

            def barrier(self):
                self.barriers += 1

            def pull(self, from_rank, offset, nbytes, dst_ptr):
                self.pulls.append((from_rank, offset, nbytes, dst_ptr - outer.base[rank]))
        return Peer()


@pytest.mark.parametrize("world", [2, 3, 4])
@pytest.mark.parametrize("boundary", ["clamp", "wrap"])
def test_peer_halo_pulls_name_the_neighbours_own_rows(world, boundary):
    """peer_wide_halos on fake exchange buffers: after replaying the pulls every halo row holds the row of the global
    grid it stands for (clamp: ranks at the global edges have no halo there; wrap: the ranks form a ring)."""
    sh = importlib.import_module("accelerate-cuda_b200.sharded")
    rows, w, reach = 6, 4, 2
    row_bytes = 4 * w
    ring = boundary == "wrap"
    pads = [((reach if (r > 0 or ring) else 0), (reach if (r < world - 1 or ring) else 0)) for r in range(world)]
    fake = _FakePeers(world, (rows + 2 * reach) * row_bytes)
    grid = np.arange(world * rows * w, dtype=np.float32).reshape(world * rows, w)
    slabs = []
    for r in range(world):  # own rows in the middle of the padded slab, halos marked -1
        pt, pb = pads[r]
        slab = fake.bufs[r][:(pt + rows + pb) * row_bytes].view(np.float32).reshape(pt + rows + pb, w)
        slab[:] = -1
        slab[pt:pt + rows] = grid[r * rows:(r + 1) * rows]
        slabs.append(slab)
    peers = [fake.view(r) for r in range(world)]
    for r in range(world):
        assert sh.peer_wide_halos(peers[r], 0, rows, row_bytes, reach, boundary) == pads[r]
        assert peers[r].barriers == 2  # before the pulls, and after them
    for r in range(world):
        for src, off, n, dst in peers[r].pulls:
            fake.bufs[r][dst:dst + n] = fake.bufs[src][off:off + n]
    total = world * rows
    for r in range(world):
        pt, pb = pads[r]
        want = [(r * rows - pt + i) % total for i in range(pt + rows + pb)]
        assert np.array_equal(slabs[r], grid[want])


@pytest.mark.parametrize("world", [1, 2, 3, 8])
@pytest.mark.parametrize("n,block", [(0, 8), (1, 8), (8, 8), (9, 8), (63, 8), (64, 8), (65, 8), (1000, 16), (12345, 32)])
def test_block_cyclic_layout_of_the_sharded_scan(world, n, block):
    """accb_peer_scan_layout (no device needed) against the Python helpers, and take/put as inverses: block j
    lives on rank j mod world, only the last block may be short, and that block's owner holds the total."""
    sys.path.insert(0, ROOT)
    accb = importlib.import_module("accelerate-cuda_b200")
    sh = importlib.import_module("accelerate-cuda_b200.sharded")
    counts = sh.block_cyclic_counts(n, world, block)
    assert sum(counts) == n
    x = torch.arange(n, dtype=torch.int32)
    back = torch.full((n,), -1, dtype=torch.int32)
    nblocks = -(-n // block)
    for r in range(world):
        n_local, owner, scratch = accb.scan_layout(world, r, n, block)
        mine = sh.block_cyclic_take(x, r, world, block)
        assert n_local == counts[r] == mine.numel()
        assert owner == ((nblocks - 1) % world if nblocks else 0)
        assert scratch >= 2 * 128 * max(1, nblocks) and scratch % 256 == 0
        # the rank's k-th element of local block b is element (b * world + r) * block + k of the whole vector
        for b in range(0, mine.numel(), block):
            assert int(mine[b]) == (b // block * world + r) * block
        sh.block_cyclic_put(back, mine, r, world, block)
    assert torch.equal(back, x)
