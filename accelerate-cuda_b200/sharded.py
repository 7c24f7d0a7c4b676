"""Multi-GPU execution of the skeletons: one process per GPU, ``torch.distributed``
for the exchange steps (NCCL on GPUs; the same code runs on CPU tensors with
the gloo backend, which is how it is tested without GPUs).

The reference has no multi-device code; its only primitive is an uncalled peer
copy (``Data/Array/Accelerate/CUDA/Array/Prim.hs:306-335``).  Here every
collective operation shards by contiguous slabs of the outermost index space:

* map, fold over rows  -- no exchange, results stay sharded;
* foldAll              -- one partial per rank, all-gathered and combined in rank order;
* scan                 -- slab totals all-gathered; each rank continues from the
                          exclusive sum of the lower ranks' totals (the carry);
                          or, without the extra pass over the data that the slab
                          total costs, dealt to the ranks in blocks (block j on rank
                          j mod world) and scanned by ``Peer.scan`` in one pass;
* permute (+)          -- full-size partial destinations, one all-reduce;
* iterated stencil     -- row slabs with halo rows towards each neighbour, refreshed
                          by neighbour send/recv into the rank's OWN halo rows (no
                          kernel reads a peer's memory): either RY rows before every
                          application, or iters*RY rows ONCE, after which all the
                          applications run on the padded slab (a few rows are
                          computed twice instead of exchanging iters times).

Only the partitioning and exchange logic lives here; the local work is done by
whatever ``local_*`` callables the caller passes (the skeleton launches of
``Context`` on a GPU).
"""
from __future__ import annotations

from typing import Callable, Tuple

import torch
import torch.distributed as dist


def slab(n: int, rank: int, world: int) -> Tuple[int, int]:
    """[lo, hi) of rank's contiguous slab of n items; sizes differ by at most one
    and are multiples of 4 wherever possible so that slabs stay 16-byte aligned."""
    q = (n // 4) // world * 4  # aligned base size
    lo = rank * q
    hi = (rank + 1) * q if rank < world - 1 else n
    return lo, hi


def block_cyclic_counts(n: int, world: int, block: int):
    """Elements per rank when a vector of n elements is dealt in blocks of ``block``: block j goes to rank
    j mod world; only the last block may be short.  The same arithmetic as ``accb_peer_scan_layout``."""
    full, rem = divmod(n, block)
    counts = [(full // world + (1 if r < full % world else 0)) * block for r in range(world)]
    if rem:
        counts[full % world] += rem
    return counts


def block_cyclic_take(x: torch.Tensor, rank: int, world: int, block: int) -> torch.Tensor:
    """This rank's share of the vector x, its blocks one after the other."""
    n = x.shape[0]
    parts = [x[lo:min(lo + block, n)] for lo in range(rank * block, n, world * block)]
    return torch.cat(parts) if parts else x[:0]


def block_cyclic_put(dst: torch.Tensor, local: torch.Tensor, rank: int, world: int, block: int) -> torch.Tensor:
    """The inverse of ``block_cyclic_take``: writes this rank's blocks to their places in the whole vector."""
    n, at = dst.shape[0], 0
    for lo in range(rank * block, n, world * block):
        m = min(block, n - lo)
        dst[lo:lo + m] = local[at:at + m]
        at += m
    return dst


def scan_carry(local_total: torch.Tensor, group=None) -> torch.Tensor:
    """Exclusive sum over the lower ranks of each rank's slab total (wrapping
    integer addition): the seed the rank's local scan continues from."""
    world, rank = dist.get_world_size(group), dist.get_rank(group)
    gathered = torch.empty(world, dtype=local_total.dtype, device=local_total.device)
    dist.all_gather_into_tensor(gathered, local_total.reshape(1), group=group)
    carry = gathered[:rank].sum(dtype=local_total.dtype) if rank else torch.zeros((), dtype=local_total.dtype,
                                                                                  device=local_total.device)
    return carry.reshape(1)


def sharded_scanl(x_local: torch.Tensor, seed: int, local_total: Callable, local_scan: Callable, group=None):
    """scanl (+) seed over the concatenation of the ranks' slabs.

    ``local_total(x) -> 1-element tensor`` and ``local_scan(x, seed_tensor) ->
    tensor of len(x)+1`` (exclusive body + running total) do the local work.
    Returns the rank's part of the result: len(x) values (len(x)+1 on the last
    rank, whose final element is the grand total)."""
    world, rank = dist.get_world_size(group), dist.get_rank(group)
    carry = scan_carry(local_total(x_local), group) + seed
    out = local_scan(x_local, carry.to(x_local.dtype))
    return out if rank == world - 1 else out[:-1]


def sharded_fold_all(local_partial: torch.Tensor, combine: Callable, group=None) -> torch.Tensor:
    """All ranks get the combination of the per-rank partials, taken in rank order
    so that the result does not depend on arrival order."""
    world = dist.get_world_size(group)
    gathered = torch.empty(world, dtype=local_partial.dtype, device=local_partial.device)
    dist.all_gather_into_tensor(gathered, local_partial.reshape(1), group=group)
    acc = gathered[0]
    for r in range(1, world):
        acc = combine(acc, gathered[r])
    return acc.reshape(1)


def sharded_histogram(local_hist: torch.Tensor, defaults: torch.Tensor, group=None) -> torch.Tensor:
    """permute (+): each rank scattered its slab of keys into a zero-initialised
    full-size partial; the partials are summed by one all-reduce and the
    defaults added once."""
    total = local_hist.clone()
    dist.all_reduce(total, op=dist.ReduceOp.SUM, group=group)
    return total + defaults


def exchange_halos(grid: torch.Tensor, ry: int, boundary: str = "clamp", group=None):
    """Refresh the halo rows of a row-slab (of a matrix; for a cube cut along its outermost dimension a "row" is
    a plane).

    ``grid`` has ry halo rows above and below the rank's interior rows.  Interior
    edge rows go to the neighbours' halos; at the global top and bottom the halo
    is filled locally according to the boundary mode (clamp: replicate the edge
    row; wrap: taken from the other end of the ring; constant: left untouched,
    the caller keeps the constant there; mirror: reflected interior rows)."""
    world, rank = dist.get_world_size(group), dist.get_rank(group)
    interior = grid[ry:grid.shape[0] - ry]
    # row blocks of a contiguous grid are contiguous: sent from and received into place, no staging copies
    top, bottom = interior[:ry], interior[-ry:]
    up, down = rank - 1, rank + 1
    ring = boundary == "wrap"
    if ring:
        up, down = up % world, down % world
    ops, recv_top, recv_bot = [], grid[:ry], grid[grid.shape[0] - ry:]
    has_up, has_down = up >= 0, down < world
    if world > 1:
        # Rows travelling up carry tag 0, rows travelling down tag 1.  NCCL matches the messages
        # between two ranks by order, not by tag, so the order matters when both neighbours are the
        # same rank (a ring of two): each side sends [up, down] and receives [from below, from above].
        if has_up:
            ops.append(dist.P2POp(dist.isend, top, up, group, 0))
        if has_down:
            ops.append(dist.P2POp(dist.isend, bottom, down, group, 1))
        if has_down:
            ops.append(dist.P2POp(dist.irecv, recv_bot, down, group, 0))
        if has_up:
            ops.append(dist.P2POp(dist.irecv, recv_top, up, group, 1))
    if ops:
        for w in dist.batch_isend_irecv(ops):
            w.wait()
    if world == 1 and ring:
        grid[:ry] = bottom
        grid[-ry:] = top
        return grid
    if has_up:
        pass  # received in place
    elif boundary == "clamp":
        grid[:ry] = interior[:1].expand(ry, *interior.shape[1:])
    elif boundary == "mirror":
        grid[:ry] = interior[1:ry + 1].flip(0)
    if has_down:
        pass  # received in place
    elif boundary == "clamp":
        grid[-ry:] = interior[-1:].expand(ry, *interior.shape[1:])
    elif boundary == "mirror":
        grid[-ry:] = interior[-ry - 1:-1].flip(0)
    return grid


def sharded_stencil_iterate_blocked(grid_local: torch.Tensor, iters: int, ry: int, local_iterate: Callable,
                                    boundary: str = "clamp", group=None) -> torch.Tensor:
    """``iters`` stencil applications on a row-slab with ONE exchange: the halo is iters*ry rows wide, the
    applications run on the whole padded slab, and what the kernel's own boundary treatment does at the padded
    edges creeps inwards by ry rows per application -- exactly as far as the halo reaches.  About iters^2*ry/2 rows
    per side are computed redundantly instead of exchanging ry rows iters times.  Ranks at the global top and bottom
    get no halo on that side (the kernel's boundary IS the global one there); with Wrap every rank has both.
    ``local_iterate(padded, iters) -> padded`` applies the stencil iters times.  Falls back to one exchange per
    application when some slab has fewer than iters*ry rows."""
    world, rank = dist.get_world_size(group), dist.get_rank(group)
    k = iters * ry
    h = grid_local.shape[0]
    hmin = grid_local.new_tensor([float(h)])
    if world > 1:
        dist.all_reduce(hmin, op=dist.ReduceOp.MIN, group=group)
    if world == 1:
        return local_iterate(grid_local, iters)
    if int(hmin[0]) < k:  # every rank takes the same path: the exchange is collective
        out = grid_local
        return sharded_stencil_iterate(out, iters, ry, lambda a: local_iterate(a, 1), boundary, group)
    pt, pb = wide_halo_layout(k, boundary, group)
    a = torch.empty((pt + h + pb, grid_local.shape[1]), dtype=grid_local.dtype, device=grid_local.device)
    a[pt:pt + h] = grid_local
    exchange_wide_halos(a, pt, pb, group)
    return local_iterate(a, iters)[pt:pt + h]


def wide_halo_layout(k: int, boundary: str = "clamp", group=None) -> Tuple[int, int]:
    """Halo rows (above, below) of this rank's slab for k rows of reach: none at the global top and bottom, where
    the kernel's boundary is the global one, except with Wrap, where the ranks form a ring."""
    world, rank = dist.get_world_size(group), dist.get_rank(group)
    ring = boundary == "wrap" and world > 1
    return (k if (rank > 0 or ring) else 0), (k if (rank < world - 1 or ring) else 0)


def exchange_wide_halos(a: torch.Tensor, pt: int, pb: int, group=None) -> torch.Tensor:
    """Fill the pt halo rows above and the pb halo rows below the interior of a padded slab from the neighbours'
    interiors, in place (a caller that keeps its data in such a slab exchanges without any copy)."""
    world, rank = dist.get_world_size(group), dist.get_rank(group)
    h = a.shape[0] - pt - pb
    interior = a[pt:pt + h]
    up, down = (rank - 1) % world, (rank + 1) % world
    ops = []
    # rows travelling up carry tag 0, rows travelling down tag 1; between two ranks messages match by order, which
    # matters when both neighbours are the same rank (a ring of two): send [up, down], receive [from below, from above]
    if pt:
        ops.append(dist.P2POp(dist.isend, interior[:pt], up, group, 0))
    if pb:
        ops.append(dist.P2POp(dist.isend, interior[h - pb:], down, group, 1))
    if pb:
        ops.append(dist.P2POp(dist.irecv, a[pt + h:], down, group, 0))
    if pt:
        ops.append(dist.P2POp(dist.irecv, a[:pt], up, group, 1))
    if ops:
        for wk in dist.batch_isend_irecv(ops):
            wk.wait()
    return a


def sharded_stencil_iterate(grid_local: torch.Tensor, iters: int, ry: int, local_apply: Callable,
                            boundary: str = "clamp", group=None) -> torch.Tensor:
    """``iters`` stencil applications on a row-slab.  ``grid_local`` holds only the
    rank's interior rows; ``local_apply(padded) -> padded`` applies the stencil
    to a slab with halo rows (any boundary treatment in x is the kernel's; rows
    beyond the halo are never read because the halo already carries the
    boundary)."""
    h = grid_local.shape[0]
    a = torch.empty((h + 2 * ry, *grid_local.shape[1:]), dtype=grid_local.dtype, device=grid_local.device)
    a[ry:ry + h] = grid_local
    for _ in range(iters):
        exchange_halos(a, ry, boundary, group)
        a = local_apply(a)
    return a[ry:ry + h]


def segment_partition(offsets, parts: int):
    """Cuts between segments for ``parts`` ranks: run p holds the segments from the first one whose offset reaches
    p/parts of all elements, so the runs hold about the same number of elements and no segment is cut.  The
    arithmetic of ``accb_seg_partition``.  Returns parts + 1 segment numbers."""
    offs = torch.as_tensor(offsets).to(torch.int64).cpu()
    nseg = offs.numel() - 1
    total = int(offs[nseg] - offs[0])
    first = [0]
    for p in range(1, parts):
        want = int(offs[0]) + total * p // parts
        cut = int(torch.searchsorted(offs, torch.tensor(want), right=False))
        first.append(max(first[-1], min(cut, nseg)))
    return first + [nseg]


def sharded_fold_seg(values_local: torch.Tensor, offsets_run: torch.Tensor, local_fold_seg: Callable) -> torch.Tensor:
    """foldSeg split between segments (no exchange): ``offsets_run`` is this rank's run of the whole array's offsets
    (its segments + 1 values); rebased to start at zero it indexes the rank's own slice ``values_local``.
    ``local_fold_seg(values, offsets) -> one result per segment``."""
    return local_fold_seg(values_local, offsets_run - offsets_run[:1])


def sharded_stencil2(a_local: torch.Tensor, b_local: torch.Tensor, ry: int, local_apply: Callable, boundary: str = "clamp",
                     group=None) -> torch.Tensor:
    """stencil2 on row slabs: both sources get ry halo rows from the neighbours (``exchange_halos``), then
    ``local_apply(a_padded, b_padded) -> padded result``; returns the rank's own rows.  Sources of different extents
    are cut to their intersection before they are dealt out (CUDA/Execute.hs:433-435)."""
    h, w = a_local.shape
    pa = torch.empty((h + 2 * ry, w), dtype=a_local.dtype, device=a_local.device)
    pb = torch.empty((h + 2 * ry, w), dtype=b_local.dtype, device=b_local.device)
    pa[ry:ry + h], pb[ry:ry + h] = a_local, b_local
    exchange_halos(pa, ry, boundary, group)
    exchange_halos(pb, ry, boundary, group)
    return local_apply(pa, pb)[ry:ry + h]


# ------------------------------------------------------------------ exchanges by the library's own kernels
def peer_buffer(ctx, nbytes: int, group=None):
    """This rank's exchange buffer, connected to the other ranks' buffers (``Peer``): the 64-byte IPC handles travel
    through the process group once; afterwards the exchanges below are single kernels over NVLink peer mappings and
    involve neither the collective library nor the host."""
    from . import AccbError, ECUDA, Peer
    world, rank = dist.get_world_size(group), dist.get_rank(group)
    gathered = [False]

    def all_gather_bytes(b):
        out = [None] * world
        gathered[0] = True
        dist.all_gather_object(out, b, group=group)
        if any(h is None for h in out):
            raise AccbError(ECUDA, "a rank could not create its exchange buffer")
        return out
    try:
        return Peer(ctx, rank, world, nbytes, all_gather_bytes)
    except AccbError:
        if not gathered[0]:  # failed before the handles were exchanged: the other ranks are waiting in the gather
            dist.all_gather_object([None] * world, None, group=group)
        raise


class PeerScanFromHost:
    """``scanl`` over one vector dealt to the ranks in blocks, from HOST arrays to HOST arrays: the counterpart of
    ``run1`` (upload, run, download: CUDA.hs:307-330,382-389) for one process per GPU.  Every rank passes its own
    blocks (pinned host memory) and receives its share of the result.  The scan is launched piece by piece
    (``Peer.scan`` with ``first_block`` / ``blocks``): while piece k is scanned, piece k+1 is on its way to the
    device and the result of piece k-1 on its way back, so both directions of every rank's host link and the GPUs
    work at the same time."""

    def __init__(self, ctx, peer, kernel, n_global: int, block_elems: int, dtype, seed, blocks_per_piece: int = 32,
                 scratch_offset: int = 0):
        from . import scan_layout
        self.ctx, self.peer, self.kernel, self.seed = ctx, peer, kernel, seed
        self.n_global, self.block, self.per, self.scratch_offset = n_global, block_elems, blocks_per_piece, scratch_offset
        self.n_local, self.owner, _ = scan_layout(peer.world, peer.rank, n_global, block_elems)
        self.has_total = peer.rank == self.owner
        # every rank launches the same number of pieces: as many as the rank with the most blocks needs
        most = -(-(-(-n_global // block_elems)) // peer.world)
        self.pieces = max(1, -(-most // blocks_per_piece))
        self.x = torch.empty(max(1, self.n_local), dtype=dtype, device="cuda")
        self.out = torch.empty(self.n_local + 1, dtype=dtype, device="cuda")
        self.up, self.comp, self.down = torch.cuda.Stream(), torch.cuda.Stream(), torch.cuda.Stream()

    def __call__(self, host_in: torch.Tensor, host_out: torch.Tensor):
        """host_in: this rank's n_local elements; host_out: n_local elements (+ 1 on the rank that owns the last
        block: the total).  Returns when the result has arrived."""
        n, blk = self.n_local, self.block
        for k in range(self.pieces):
            first = k * self.per
            lo, hi = min(n, first * blk), min(n, (first + self.per) * blk)
            arrived, scanned = torch.cuda.Event(), torch.cuda.Event()
            with torch.cuda.stream(self.up):
                if hi > lo:
                    self.x[lo:hi].copy_(host_in[lo:hi], non_blocking=True)
                arrived.record()
            self.comp.wait_event(arrived)
            self.peer.scan(self.kernel, [self.x[:max(1, n)]], self.n_global, self.out, seed=self.seed, block_elems=blk,
                           scratch_offset=self.scratch_offset, stream=self.comp.cuda_stream, first_block=first,
                           blocks=self.per)
            scanned.record(self.comp)
            self.down.wait_event(scanned)
            with torch.cuda.stream(self.down):
                top = hi + (1 if (hi == n and self.has_total and k == self.pieces - 1) else 0)
                if top > lo:
                    host_out[lo:top].copy_(self.out[lo:top], non_blocking=True)
        self.down.synchronize()
        return host_out


def peer_scan_carry(peer, offset: int, gathered: torch.Tensor) -> torch.Tensor:
    """The carry of a sharded scan when the slab total was written at ``offset`` of the rank's exchange buffer: one
    kernel synchronises the ranks and gathers the totals; the exclusive sum of the lower ranks follows."""
    peer.gather(offset, gathered.element_size(), gathered)
    r = peer.rank
    return gathered[:r].sum(dtype=gathered.dtype).reshape(1) if r else torch.zeros(1, dtype=gathered.dtype,
                                                                                  device=gathered.device)


def peer_wide_halos(peer, slab_offset: int, rows: int, row_bytes: int, reach: int, boundary: str = "clamp"):
    """Fill the halo rows of a padded slab that lives at ``slab_offset`` of the exchange buffer (every rank: the same
    offset and ``rows`` own rows) from the neighbours' own rows: barrier, two pulls over NVLink, barrier -- the
    second so that no rank overwrites rows a neighbour is still reading."""
    world, rank = peer.world, peer.rank
    ring = boundary == "wrap" and world > 1
    pads = [((reach if (r > 0 or ring) else 0), (reach if (r < world - 1 or ring) else 0)) for r in range(world)]
    pt, pb = pads[rank]
    up, down = (rank - 1) % world, (rank + 1) % world
    peer.barrier()
    if pt:  # the last rows of the rank above
        peer.pull(up, slab_offset + (pads[up][0] + rows - reach) * row_bytes, reach * row_bytes,
                  peer.data_ptr + slab_offset)
    if pb:  # the first rows of the rank below
        peer.pull(down, slab_offset + pads[down][0] * row_bytes, reach * row_bytes,
                  peer.data_ptr + slab_offset + (pt + rows) * row_bytes)
    peer.barrier()
    return pt, pb
