"""accb_peer_*: exchanges between processes (one per GPU) by the library's own kernels over NVLink peer mappings.
With one GPU only the single-rank forms run; with two or more, tests/peer_ranks.py runs under torchrun with one
rank per GPU (never several ranks on one GPU: their kernels wait for one another) and is checked against NCCL."""
import os
import subprocess
import sys

import numpy as np
import pytest

pytestmark = pytest.mark.gpu

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_peer_single_rank_forms(accb, ctx, torch_cuda, rng):
    t = torch_cuda
    peer = accb.Peer(ctx, 0, 1, 1 << 16, lambda b: [b])
    x = rng.integers(-50, 50, 1000).astype(np.int32)
    view = t.as_tensor(peer.array(256, (1000,), np.int32), device="cuda")  # the buffer seen as a tensor, no copy
    view.copy_(t.from_numpy(x).cuda())
    got = t.zeros(1000, dtype=t.int32, device="cuda")
    peer.allreduce(256, 1000, np.int32, "add", got)
    peer.gather(256, 64, got[:16])
    peer.barrier()
    peer.status()
    assert np.array_equal(got.cpu().numpy(), x)
    with pytest.raises(accb.AccbError):
        peer.gather(1 << 20, 64, got)  # outside the buffer
    with pytest.raises(accb.AccbError):
        peer.allreduce(256, 10, np.float32, "xor", got)  # bitwise combination of floats
    peer.destroy()


TILE = 9216  # elements of a tile of the block-cyclic scan for 4-byte values (4608 for 8-byte values)


@pytest.mark.parametrize("n,tiles_per_block", [(1, 1), (TILE, 1), (5 * TILE, 1), (5 * TILE + 17, 2), (40 * TILE, 8),
                                               (100 * TILE + 4099, 32), (3 * TILE - 1, 4), (777, 2)])
@pytest.mark.parametrize("kind", ["scanl", "scanl1", "scanl'"])
def test_block_chained_scan_on_one_gpu(accb, ctx, P, oracle, torch_cuda, rng, n, tiles_per_block, kind):
    """The scan over several GPUs with a world of one: every block record is written and read by the same GPU in
    ONE launch (nothing waits for another launch), which exercises the chain of blocks -- aggregates published by
    a block's last tile, prefixes taken up by the next block's first tile -- without a second GPU."""
    t = torch_cuda
    assert ctx.scan_tile(P.SCAN_ADD_I32) == TILE
    block = tiles_per_block * TILE
    n_local, owner, scratch = accb.scan_layout(1, 0, n, block)
    assert (n_local, owner) == (n, 0)
    peer = accb.Peer(ctx, 0, 1, scratch + 256, lambda b: [b])
    x = rng.integers(-9, 10, n).astype(np.int32)
    xd = t.from_numpy(x).cuda()
    for _ in range(3):  # launches alternate between the two sets of block records
        out = t.full((n + 1,), -77, dtype=t.int32, device="cuda")
        if kind == "scanl":
            peer.scan(P.SCAN_ADD_I32, [xd], n, out, seed=np.int32(5), block_elems=block, scratch_offset=256)
            ctx.sync()
            assert np.array_equal(out.cpu().numpy(), oracle.scanl_i32(x, 5))
        elif kind == "scanl1":
            peer.scan(P.SCAN_ADD_I32, [xd], n, out[:n], kind=accb.SCAN_INCLUSIVE, block_elems=block, scratch_offset=256)
            ctx.sync()
            assert np.array_equal(out[:n].cpu().numpy(), oracle.scanl1_i32(x)) and int(out[n]) == -77
        else:
            tot = t.zeros(1, dtype=t.int32, device="cuda")
            peer.scan(P.SCAN_ADD_I32, [xd], n, out[:n], kind=accb.SCAN_PRIME, seed=np.int32(-3), total=tot,
                      block_elems=block, scratch_offset=256)
            ctx.sync()
            body, total = oracle.scanl_prime_i32(x, -3)
            assert np.array_equal(out[:n].cpu().numpy(), body) and int(tot[0]) == total and int(out[n]) == -77
    peer.status()
    peer.destroy()


def test_block_chained_scan_of_eight_byte_values_and_floats(accb, ctx, P, torch_cuda, rng):
    t = torch_cuda
    tile = ctx.scan_tile(P.SCAN_ADD_I64)  # half as many 8-byte values
    assert tile == TILE // 2
    n = 9 * tile + 5
    n_local, owner, scratch = accb.scan_layout(1, 0, n, 2 * tile)
    peer = accb.Peer(ctx, 0, 1, scratch, lambda b: [b])
    x = rng.integers(-(1 << 40), 1 << 40, n).astype(np.int64)
    out = t.empty(n + 1, dtype=t.int64, device="cuda")
    peer.scan(P.SCAN_ADD_I64, [t.from_numpy(x).cuda()], n, out, seed=np.int64(1), block_elems=2 * tile)
    ctx.sync()
    assert np.array_equal(out.cpu().numpy(), np.concatenate([[1], 1 + np.cumsum(x)]))
    with pytest.raises(accb.AccbError):  # a result array shorter than this rank's share of the vector
        peer.scan(P.SCAN_ADD_I64, [t.from_numpy(x).cuda()], n, out[:n], seed=np.int64(1), block_elems=2 * tile)
    with pytest.raises(accb.AccbError):  # blocks are whole tiles
        peer.scan(P.SCAN_ADD_I64, [t.from_numpy(x).cuda()], n, out, seed=np.int64(1), block_elems=1000)
    with pytest.raises(accb.AccbError):  # right scans are not dealt in blocks
        peer.scan(P.SCAN_ADD_I64, [t.from_numpy(x).cuda()], n, out, kind=accb.SCAN_INCLUSIVE_SEEDED, seed=np.int64(1))
    peer.destroy()


@pytest.mark.parametrize("n,tiles_per_block,per", [(50 * TILE + 77, 2, 3), (7 * TILE, 1, 1), (33 * TILE, 4, 100)])
def test_scan_launched_piece_by_piece_from_host_arrays(accb, ctx, P, oracle, torch_cuda, rng, n, tiles_per_block, per):
    """PeerScanFromHost with a world of one: pinned host arrays in and out, the scan launched in pieces of `per`
    blocks that find the records of the pieces before them; uploads, launches and downloads overlap."""
    t = torch_cuda
    sh = __import__("importlib").import_module("accelerate-cuda_b200.sharded")
    block = tiles_per_block * TILE
    _, _, scratch = accb.scan_layout(1, 0, n, block)
    peer = accb.Peer(ctx, 0, 1, scratch, lambda b: [b])
    run = sh.PeerScanFromHost(ctx, peer, P.SCAN_ADD_I32, n, block, t.int32, np.int32(9), blocks_per_piece=per)
    for _ in range(2):
        x = rng.integers(-9, 10, n).astype(np.int32)
        hin = t.from_numpy(x).pin_memory()
        hout = t.full((n + 1,), -1, dtype=t.int32).pin_memory()
        run(hin, hout)
        assert np.array_equal(hout.numpy(), oracle.scanl_i32(x, 9))
    ctx.sync()
    with pytest.raises(accb.AccbError):  # a piece out of order
        peer.scan(P.SCAN_ADD_I32, [run.x], n, run.out, seed=np.int32(9), block_elems=block, first_block=5, blocks=1)
    peer.destroy()


def test_block_chained_scan_of_nothing(accb, ctx, P, torch_cuda):
    t = torch_cuda
    peer = accb.Peer(ctx, 0, 1, 4096, lambda b: [b])
    out = t.full((1,), -1, dtype=t.int32, device="cuda")
    peer.scan(P.SCAN_ADD_I32, [t.empty(1, dtype=t.int32, device="cuda")[:0]], 0, out, seed=np.int32(42))
    ctx.sync()
    assert int(out[0]) == 42  # scanl f z [] = [z]
    peer.destroy()


def test_a_rank_that_never_arrives_runs_the_wait_into_its_limit(accb, ctx, torch_cuda, monkeypatch):
    """The failure is made on the host: this process claims to be rank 0 of 2 and nobody plays rank 1, so rank 1's
    flag is never set.  The barrier kernel gives up after its limit (one second here), finishes normally, and the
    status call reports ETIMEOUT; the context stays usable."""
    t = torch_cuda
    monkeypatch.setenv("ACCB_PEER_TIMEOUT_MS", "1000")
    peer = accb.Peer(ctx, 0, 2, 4096, None)
    peer.barrier()
    with pytest.raises(accb.AccbError) as e:
        peer.status()
    assert e.value.status == accb.ETIMEOUT
    peer.status()  # the error word was cleared
    x = t.arange(10, device="cuda")
    assert int(x.sum()) == 45  # the device still answers
    peer.destroy()


def test_a_scan_whose_other_rank_never_publishes_gives_up(accb, ctx, P, torch_cuda, monkeypatch):
    """Rank 0 of a pretended world of two holds blocks 0, 2, 4, ..; block 2 needs block 1's record, which nobody
    writes.  The failure is made on the host (no second rank exists); the kernel's waits run into the time limit,
    the launch finishes, accb_context_sync reports ETIMEOUT and the device still answers."""
    t = torch_cuda
    monkeypatch.setenv("ACCB_PEER_TIMEOUT_MS", "500")
    n_g = 6 * TILE
    n_local, owner, scratch = accb.scan_layout(2, 0, n_g, TILE)
    peer = accb.Peer(ctx, 0, 2, scratch, None)
    x = t.ones(n_local, dtype=t.int32, device="cuda")
    out = t.empty(n_local + 1, dtype=t.int32, device="cuda")
    peer.scan(P.SCAN_ADD_I32, [x], n_g, out, seed=np.int32(0), block_elems=TILE)
    with pytest.raises(accb.AccbError) as e:
        ctx.sync()
    assert e.value.status == accb.ETIMEOUT
    assert int(out[TILE - 1]) == TILE - 1  # block 0 needed nobody and is right
    ctx.sync()  # the error word was cleared
    assert int(t.arange(10, device="cuda").sum()) == 45
    try:
        peer.status()
    except accb.AccbError:
        pass  # the barrier ahead of a scan with few blocks gave up as well
    peer.destroy()


def test_peer_exchanges_match_nccl_on_two_or_more_gpus(torch_cuda):
    n = torch_cuda.cuda.device_count()
    if n < 2:
        pytest.skip("needs two GPUs: ranks that wait for one another never share a GPU")
    world = 4 if n >= 4 else 2
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    out = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={world}",
                          "--master-addr", "127.0.0.1", "--master-port", "29577",
                          os.path.join(ROOT, "tests", "peer_ranks.py")], capture_output=True, text=True, env=env, timeout=600)
    assert out.returncode == 0, out.stdout[-2000:] + out.stderr[-4000:]
    assert out.stdout.count("PEER-OK") == world, out.stdout[-2000:] + out.stderr[-2000:]
