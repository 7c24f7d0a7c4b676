"""Child program of tests/test_gpu_peer.py: run under torchrun with one rank per GPU.  Every exchange kernel of
accb_peer_* is compared with the corresponding NCCL collective over many rounds, regions alternating as the API
asks; prints PEER-OK on every rank that saw no difference."""
import importlib
import os
import sys

import numpy as np
import torch
import torch.distributed as dist

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)


def main():
    local = int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local)
    dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    rank, world = dist.get_rank(), dist.get_world_size()
    accb = importlib.import_module("accelerate-cuda_b200")
    sh = importlib.import_module("accelerate-cuda_b200.sharded")
    ctx = accb.Context(local)
    n = 4096
    pitch = 4 * n
    peer = sh.peer_buffer(ctx, 2 * pitch + 1024 * 1024)
    views = [torch.as_tensor(peer.array(o, (n,), np.int32), device="cuda") for o in (0, pitch)]
    big = torch.as_tensor(peer.array(2 * pitch, (262144,), np.float32), device="cuda")  # pulled by the next rank
    gen = torch.Generator(device="cuda").manual_seed(1234 + rank)
    ok = True
    for it in range(40):
        p = it & 1
        views[p].copy_(torch.randint(-1000, 1000, (n,), generator=gen, device="cuda", dtype=torch.int32))
        # all-reduce (+) in rank order against NCCL
        got = torch.empty(n, dtype=torch.int32, device="cuda")
        peer.allreduce((0, pitch)[p], n, np.int32, "add", got)
        ref = views[p].clone()
        dist.all_reduce(ref)
        ok = ok and bool(torch.equal(got, ref))
        # max
        peer.allreduce((0, pitch)[p], n, np.int32, "max", got)
        ref = views[p].clone()
        dist.all_reduce(ref, op=dist.ReduceOp.MAX)
        ok = ok and bool(torch.equal(got, ref))
        # gather of the first 4 elements of every rank
        g = torch.empty(4 * world, dtype=torch.int32, device="cuda")
        peer.gather((0, pitch)[p], 16, g)
        ref = torch.empty(4 * world, dtype=torch.int32, device="cuda")
        dist.all_gather_into_tensor(ref, views[p][:4].contiguous())
        ok = ok and bool(torch.equal(g, ref))
        carry = sh.peer_scan_carry(peer, (0, pitch)[p], torch.empty(world, dtype=torch.int32, device="cuda"))
        ok = ok and int(carry[0]) == int(ref[0::4][:rank].sum())
        seed, c2 = torch.full((4,), 7, dtype=torch.int32, device="cuda"), torch.empty(4, dtype=torch.int32, device="cuda")
        peer.exscan((0, pitch)[p], 4, np.int32, "add", seed, c2)  # 7 + the lower ranks' elements, in one kernel
        ok = ok and bool(torch.equal(c2, 7 + ref.view(world, 4)[:rank].sum(dim=0, dtype=torch.int32)))
    # pull: every rank fetches the previous rank's block between two barriers
    big.copy_(torch.rand(262144, generator=gen, device="cuda"))
    mine = torch.empty_like(big)
    peer.barrier()
    peer.pull((rank - 1) % world, 2 * pitch, big.numel() * 4, mine.data_ptr())
    peer.barrier()
    blocks = [torch.empty_like(big) for _ in range(world)]
    dist.all_gather(blocks, big)
    ok = ok and bool(torch.equal(mine, blocks[(rank - 1) % world]))
    # the scan over a vector dealt to the ranks in blocks, against a cumulative sum of the whole vector
    P = importlib.import_module("accelerate-cuda_b200.programs")
    tile = ctx.scan_tile(P.SCAN_ADD_I32)
    cases = ((world * 64 * tile + 12345, 4), (world * 8 * tile, 2), (3 * tile + 5, 1), (5, 1), (world * 300 * tile, 32))
    host_case = (world * 40 * tile + 999, 2)  # scanned from host arrays further down
    scratch_max = max(accb.scan_layout(world, rank, n_g, tpb * tile)[2] for n_g, tpb in cases + (host_case,))
    peer2 = sh.peer_buffer(ctx, scratch_max)
    for n_g, tpb in cases:
        block = tpb * tile
        n_local, owner, _ = accb.scan_layout(world, rank, n_g, block)
        same = torch.Generator(device="cuda").manual_seed(4321)  # every rank draws the same whole vector
        whole = torch.randint(-9, 10, (n_g,), generator=same, device="cuda", dtype=torch.int32)
        mine = sh.block_cyclic_take(whole, rank, world, block).contiguous()
        ok = ok and mine.numel() == n_local == sh.block_cyclic_counts(n_g, world, block)[rank]
        ref = torch.cat([torch.zeros(1, dtype=torch.int64, device="cuda"), torch.cumsum(whole, 0, dtype=torch.int64)]) + 3
        ref = ref.int()  # wraps as the kernel's addition does
        for rep in range(3):
            out = torch.full((n_local + 1,), -77, dtype=torch.int32, device="cuda")
            peer2.scan(P.SCAN_ADD_I32, [mine], n_g, out, seed=np.int32(3), block_elems=block)
            ctx.sync()
            ok = ok and bool(torch.equal(out[:n_local], sh.block_cyclic_take(ref[:n_g], rank, world, block)))
            ok = ok and int(out[n_local]) == (int(ref[n_g]) if rank == owner else -77)
            out.fill_(-77)
            peer2.scan(P.SCAN_ADD_I32, [mine], n_g, out[:n_local], kind=accb.SCAN_INCLUSIVE, block_elems=block)
            ctx.sync()
            ok = ok and bool(torch.equal(out[:n_local], sh.block_cyclic_take(ref[1:] - 3, rank, world, block)))
            ok = ok and int(out[n_local]) == -77
    # the same from pinned host arrays, the scan launched in pieces that overlap with the copies
    n_g, block = host_case[0], host_case[1] * tile
    n_local, owner, _ = accb.scan_layout(world, rank, n_g, block)
    same = torch.Generator(device="cuda").manual_seed(777)
    whole = torch.randint(-9, 10, (n_g,), generator=same, device="cuda", dtype=torch.int32)
    ref = (torch.cat([torch.zeros(1, dtype=torch.int64, device="cuda"), torch.cumsum(whole, 0, dtype=torch.int64)]) + 3).int()
    run = sh.PeerScanFromHost(ctx, peer2, P.SCAN_ADD_I32, n_g, block, torch.int32, np.int32(3), blocks_per_piece=3)
    hin = sh.block_cyclic_take(whole, rank, world, block).cpu().pin_memory()
    hout = torch.full((n_local + 1,), -77, dtype=torch.int32).pin_memory()
    for rep in range(2):
        run(hin, hout)
        ok = ok and bool(torch.equal(hout[:n_local], sh.block_cyclic_take(ref[:n_g], rank, world, block).cpu()))
        ok = ok and int(hout[n_local]) == (int(ref[n_g]) if rank == owner else -77)
    ctx.sync()
    peer2.status()
    peer.status()
    flag = torch.tensor([int(ok)], device="cuda")
    dist.all_reduce(flag, op=dist.ReduceOp.MIN)
    dist.barrier()
    peer.destroy()
    peer2.destroy()
    dist.barrier()
    if int(flag[0]) == 1:
        print(f"PEER-OK rank {rank} of {world}", flush=True)
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
