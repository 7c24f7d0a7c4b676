#!/usr/bin/env python
"""Benchmark of the B200 skeleton library on BASELINE.json's metric:
effective HBM GB/s per skeleton.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload scan] [--impl reference]

A step is one pass of one skeleton over its synthetic input.  The default
workload is the prefix sum ``scanl (+) 0`` over 2^28 Int32 per GPU; the other
configurations are measured after the timed region and reported under
``skeletons`` (N = 1 only).  With N > 1 (under torchrun) every rank scans its
own 2^28-element slab of one N*2^28-element vector and the slabs are joined by
a carry: weak scaling.

One JSON line on stdout (rank 0):
  value      algorithmic bytes of all ranks / device time of the K timed steps
             (CUDA events on the launching stream, max over ranks), GB/s;
  roofline   the same for the dominant kernel against the measured HBM copy
             bandwidth of MEASURED_PEAKS.json;
  e2e        the metric through run1 on pinned HOST arrays: upload, launch,
             download inside the timed region;
  cpu_baseline  the CPU oracle (a port: the reference's own interpreter
             cannot be built here) on a bounded sample, one core.
``--impl reference`` times that oracle with all host threads instead.
"""
from __future__ import annotations

import argparse
import importlib
import json
import os
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

METRIC = "effective HBM GB/s per skeleton at 2^28 elems"

# DRAM traffic (dram__bytes_read.sum + dram__bytes_write.sum) per unit of work, from the ncu captures
# summarised under profiles/: (kernel, bytes per unit).  A unit is an element (scan, dot, hist,
# rowsum), an option (blackscholes) or a grid point of one application (stencil).  Dirty lines still
# in L2 when a kernel ends are not counted as DRAM writes by the profiler.
NCU_TRAFFIC = {
    "scan": ("scanl", 480.0e6 / (1 << 26)),
    "dot": ("foldAll", 541.0e6 / (1 << 26)),
    "hist": ("permute_smem", 274.9e6 / (1 << 26)),
    "stencil": ("stencil_tile2", 250.2e6 / (6144 * 6144) / 2),  # one launch = two applications (one alone: 245.4e6)
    "blackscholes": ("map", 292.9e6 / (1 << 24)),
    "rowsum": ("fold", 276.4e6 / (8192 * 8192)),
}
# algorithmic bytes per unit (see accelerate-cuda_b200/workloads.py)
BYTES_PER_UNIT = {"scan": 8, "dot": 8, "hist": 4, "stencil": 8, "blackscholes": 20, "rowsum": 4}
SPEC_PEAK_GBS = 8000.0
FALLBACK_PEAK_GBS = 6650.0


def measured_peak():
    try:
        with open(os.path.join(ROOT, "MEASURED_PEAKS.json")) as f:
            return float(json.load(f)["hbm_gbs"]), "measured"
    except Exception:
        return FALLBACK_PEAK_GBS, "fallback"


# ----------------------------------------------------------------- clocks
class ClockSampler:
    """Samples SM clock and throttle reasons through NVML while the timed region runs (read-only)."""

    def __init__(self, device: int):
        self.samples, self.reasons, self.max_mhz = [], set(), None
        self._stop = threading.Event()
        self._thr = None
        try:
            import pynvml as nv
            nv.nvmlInit()
            self.nv = nv
            self.h = nv.nvmlDeviceGetHandleByIndex(device)
            self.max_mhz = nv.nvmlDeviceGetMaxClockInfo(self.h, nv.NVML_CLOCK_SM)
        except Exception:
            self.nv = None

    def _loop(self):
        nv = self.nv
        names = {
            getattr(nv, "nvmlClocksEventReasonHwSlowdown", 0x8): "hw_slowdown",
            getattr(nv, "nvmlClocksEventReasonHwThermalSlowdown", 0x40): "hw_thermal_slowdown",
            getattr(nv, "nvmlClocksEventReasonSwThermalSlowdown", 0x20): "sw_thermal_slowdown",
            getattr(nv, "nvmlClocksEventReasonSwPowerCap", 0x4): "sw_power_cap",
        }
        while not self._stop.is_set():
            try:
                self.samples.append(nv.nvmlDeviceGetClockInfo(self.h, nv.NVML_CLOCK_SM))
                try:
                    mask = nv.nvmlDeviceGetCurrentClocksEventReasons(self.h)
                except Exception:
                    mask = nv.nvmlDeviceGetCurrentClocksThrottleReasons(self.h)
                for bit, name in names.items():
                    if mask & bit:
                        self.reasons.add(name)
            except Exception:
                pass
            self._stop.wait(0.001)  # the timed region of the default run lasts only a few milliseconds

    def __enter__(self):
        if self.nv:
            self._thr = threading.Thread(target=self._loop, daemon=True)
            self._thr.start()
        return self

    def __exit__(self, *a):
        self._stop.set()
        if self._thr:
            self._thr.join()

    def summary(self):
        return {"sm_mhz": float(np.median(self.samples)) if self.samples else None, "sm_max_mhz": self.max_mhz,
                "reasons": sorted(self.reasons), "samples": len(self.samples)}


def host_threads():
    """All the host threads this process may use (torchrun sets OMP_NUM_THREADS=1, which is not a property of the
    host), bounded by the container's CPU quota where there is one."""
    oracle = importlib.import_module("oracle")
    try:
        cores = len(os.sched_getaffinity(0))
    except AttributeError:
        cores = os.cpu_count() or 1
    try:
        quota, period = open("/sys/fs/cgroup/cpu.max").read().split()
        if quota != "max":
            cores = min(cores, max(1, int(quota) // int(period)))
    except (OSError, ValueError):
        pass
    return max(oracle.max_threads(), cores)


def pinned(torch, dev, fill=True):
    """A pinned host array with the shape and type of a device array (and, unless fill is False, its contents)."""
    h = torch.empty(dev.shape, dtype=dev.dtype).pin_memory()
    if fill:
        h.copy_(dev)
    return h


def close_to(got, ref, atol, rtol=1e-5):
    got, ref = np.asarray(got, np.float64), np.asarray(ref, np.float64)
    return bool(np.all(np.abs(got - ref) <= rtol * np.abs(ref) + atol))


# -------------------------------------------------------------- workloads
class Workload:
    name = ""
    dtype = ""

    def __init__(self, accb, ctx, torch, rank, world):
        self.accb, self.ctx, self.t, self.rank, self.world = accb, ctx, torch, rank, world
        self.P = importlib.import_module("accelerate-cuda_b200.programs")
        self.W = importlib.import_module("accelerate-cuda_b200.workloads")

    functors = "hand"  # "lang": the kernels the embedded language prints for the same programs (examples.py)
    exchange = "peer"  # several GPUs: "peer" = the library's own exchange kernels over NVLink, "nccl" = collectives

    def make_peer(self, nbytes):
        """This rank's exchange buffer connected to the others', or None when the exchanges go through NCCL: by
        request, or because some rank could not map the buffers (all ranks then agree to fall back)."""
        if self.world == 1 or Workload.exchange != "peer":
            return None
        import torch.distributed as dist
        sh = importlib.import_module("accelerate-cuda_b200.sharded")
        peer, why = None, ""
        try:
            peer = sh.peer_buffer(self.ctx, nbytes)
        except self.accb.AccbError as e:
            why = str(e)
        ok = self.t.tensor([int(peer is not None)], device="cuda")
        dist.all_reduce(ok, op=dist.ReduceOp.MIN)
        if int(ok[0]) == 0:
            if peer is not None:
                peer.destroy()
            Workload.exchange = "nccl (peer mapping unavailable" + (": " + why.splitlines()[0][:80] if why else "") + ")"
            return None
        return peer

    def peer_views(self, nbytes_each, shape, dtype):
        """Two regions of a fresh exchange buffer as torch tensors (used alternately: a rank may overwrite what it
        exchanged only after the next exchange) -- or None when the exchanges go through NCCL."""
        pitch = (nbytes_each + 255) // 256 * 256
        self.peer = self.make_peer(2 * pitch)
        if self.peer is None:
            return None
        self.parity = 0
        self.peer_offsets = (0, pitch)
        return [self.t.as_tensor(self.peer.array(o, shape, dtype), device="cuda") for o in self.peer_offsets]

    def functor(self, name):
        if self.functors == "lang":
            return importlib.import_module("accelerate-cuda_b200.examples").generated_specs()[name]
        return getattr(self.P, name)


class ScanWorkload(Workload):
    """scanl (+) 0 over Int32, values uniform in [0,16); 2^28 elements per GPU.

    Several GPUs scan ONE vector of world * 2^28 elements.  By default it is dealt to the GPUs in blocks of 1 MiB
    (block j on GPU j mod world) and scanned in one pass per GPU (accb_peer_scan); ``distribution = "slabs"``
    gives every GPU a contiguous slab instead, which costs a second read of the slab for its total."""
    name, dtype = "scanl (+) 0, Int32, 2^28 per GPU", "int32"
    distribution = "block-cyclic"  # or "slabs"
    tiles_per_block = 32            # blocks of the block-cyclic distribution: 32 tiles (1.1 MiB); 16 at eight GPUs

    def setup(self, n=None):
        t, W = self.t, self.W
        self.n = n or W.N28
        self.x = t.empty(self.n, dtype=t.int32, device="cuda")
        self.cyclic = self.world > 1 and self.distribution == "block-cyclic" and Workload.exchange == "peer"
        if self.world > 1 and not self.cyclic:
            self.distribution = "contiguous slabs"
        # rank r writes its share of the global result; the owner of the last element also holds out[n_total]
        self.out = t.empty(self.n + 1, dtype=t.int32, device="cuda")
        self.k = self.ctx.kernel(self.functor("SCAN_ADD_I32")).wait()
        self.bytes = W.bytes_scan(self.n)
        self.peer = None
        if self.world > 1:
            import torch.distributed as dist
            self.dist = dist
            self.sh = importlib.import_module("accelerate-cuda_b200.sharded")
        if self.cyclic:
            # every GPU holds the same number of whole blocks; what is left of its 2^28 elements (less than a block)
            # stays outside the scan, and the algorithmic bytes count only what is scanned
            # measured at eight GPUs: 8 / 16 / 24 / 32 / 64 tiles per block 0.396 / 0.388 / 0.392 / 0.396 / 0.409 ms
            # (at four GPUs 16 and 32 are level, at two 32 is ahead)
            tpb = self.tiles_per_block if self.world < 8 else self.tiles_per_block // 2
            self.block = tpb * self.ctx.scan_tile(self.k)
            self.n = self.n // self.block * self.block
            self.x, self.out = self.x[:self.n], self.out[:self.n + 1]
            self.bytes = W.bytes_scan(self.n)
            self.n_global = self.n * self.world
            n_local, self.owner, scratch = self.accb.scan_layout(self.world, self.rank, self.n_global, self.block)
            assert n_local == self.n
            self.peer = self.make_peer(scratch)
            self.cyclic = self.peer is not None
        if self.cyclic:
            # local block b is global block b * world + rank: generated in place from the index-addressable generator
            for b in range(self.n // self.block):
                self.ctx.gen_uniform_i32(self.x[b * self.block:(b + 1) * self.block], self.block,
                                         (b * self.world + self.rank) * self.block, W.SEED, W.S_SCAN, 16)
        else:
            self.ctx.gen_uniform_i32(self.x, self.n, self.rank * self.n, W.SEED, W.S_SCAN, 16)
        if self.world > 1 and not self.cyclic:
            self.distribution = "contiguous slabs"
            self.ksum = self.ctx.kernel(self.P.SUM_I32).wait()
            self.total = t.zeros(1, dtype=t.int32, device="cuda")
            self.gathered = t.zeros(self.world, dtype=t.int32, device="cuda")
            self.carry = t.zeros(1, dtype=t.int32, device="cuda")
            self.totals = self.peer_views(4, (1,), np.int32)
            self.zero = t.zeros(1, dtype=t.int32, device="cuda")  # the seed of the whole scan
        self.ctx.sync()

    def step(self):
        if self.world == 1:
            self.ctx.scan(self.k, [self.x], self.n, self.out, seed=np.int32(0))
            return 1
        if self.cyclic:  # one pass: block records travel between the GPUs inside the scan kernel itself
            self.peer.scan(self.k, [self.x], self.n_global, self.out, seed=np.int32(0), block_elems=self.block)
            return 1
        # carry pass: slab totals -> gathered -> exclusive sum of the lower ranks -> seeded local scan
        if self.peer is not None:  # the total goes straight into the exchange buffer; one kernel syncs and gathers
            p = self.parity
            self.parity ^= 1
            self.ctx.fold_all(self.ksum, [self.x], self.n, self.totals[p], seed=np.int32(0))
            self.peer.exscan(self.peer_offsets[p], 1, np.int32, "add", self.zero, self.carry)  # sync + carry: one kernel
            self.ctx.scan(self.k, [self.x], self.n, self.out, seed=self.carry)
            return 3
        self.ctx.fold_all(self.ksum, [self.x], self.n, self.total, seed=np.int32(0))
        self.dist.all_gather_into_tensor(self.gathered, self.total)
        self.carry.copy_(self.gathered[: self.rank].sum(dtype=self.t.int32).reshape(1)) if self.rank else self.carry.zero_()
        self.ctx.scan(self.k, [self.x], self.n, self.out, seed=self.carry)
        return 2

    def verify(self):
        """One GPU: the whole result against the oracle.  Contiguous slabs: out[i+1] - out[i] == x[i] everywhere,
        out[0] == the wrapped sum of the lower ranks' slabs and out[n] == out[0] + this slab's sum, which pins every
        element.  Block-cyclic: the whole local result against torch operators -- every block's exclusive prefix from
        the all-gathered block sums (int64, wrapped) plus the cumulative sum inside the block."""
        t = self.t
        wrap = lambda v: int(np.array(v & 0xffffffff, np.uint32).astype(np.int32))  # noqa: E731
        if self.world > 1 and self.cyclic:
            nb = self.n // self.block
            xb = self.x.view(nb, self.block)
            sums = xb.sum(dim=1, dtype=t.int64)
            every = t.empty(self.world * nb, dtype=t.int64, device="cuda")
            self.dist.all_gather_into_tensor(every, sums)
            in_order = every.view(self.world, nb).t().reshape(-1)  # global block j = b * world + rank
            before = t.cumsum(in_order, 0) - in_order
            mine = before.view(nb, self.world)[:, self.rank]
            inside = t.cumsum(xb, 1, dtype=t.int64)
            inside -= xb
            inside += mine[:, None]
            ok = bool(t.equal(self.out[:self.n], inside.int().view(-1)))
            if self.rank == self.owner:
                ok = ok and int(self.out[self.n]) == wrap(int(in_order.sum()))
            return ok
        d = self.out[1:] - self.out[:-1]
        ok = bool(t.equal(d, self.x))
        mine = self.x.sum(dtype=t.int64).reshape(1)
        lower = 0
        if self.world > 1:
            totals = t.zeros(self.world, dtype=t.int64, device="cuda")
            self.dist.all_gather_into_tensor(totals, mine)
            lower = int(totals[: self.rank].sum())
        ok = ok and int(self.out[0]) == wrap(lower) and int(self.out[-1]) == wrap(lower + int(mine[0]))
        if self.world == 1 and self.functors == "hand":
            oracle = importlib.import_module("oracle")
            ref = oracle.scanl_i32(self.x.cpu().numpy(), 0, nthreads=host_threads())
            ok = ok and bool(t.equal(self.out, t.from_numpy(ref).cuda()))
        return ok

    def host_program(self):
        """The same operation as a run1 function on host arrays: (program, inputs, result buffers, check)."""
        accb, P, t = self.accb, self.P, self.t
        prog = accb.run1With(self.ctx, lambda v: accb.scan(P.SCAN_ADD_I32, [v], np.int32, seed=np.int32(0)),
                             accb.ArrayType(1, np.int32))
        hin, hout = pinned(t, self.x), pinned(t, self.out, fill=False)
        return prog, [hin.numpy()], [[hout.numpy()]], lambda: bool(t.equal(hout, self.out.cpu()))


class DotWorkload(Workload):
    name, dtype = "foldAll (+) 0 (zipWith (*) xs ys), Float32, 2^28", "f32"
    sets = 1  # buffer sets the steps rotate through (inputs smaller than L2 need several)

    def setup(self, n=None):
        t, W = self.t, self.W
        self.n = n or W.N28
        first = self.rank * self.n  # each rank holds its own slab of one world*n vector
        self.pairs = []
        for _ in range(self.sets):  # every set holds the same values: one reference serves all of them
            x = t.empty(self.n, dtype=t.float32, device="cuda")
            y = t.empty(self.n, dtype=t.float32, device="cuda")
            self.ctx.gen_uniform_f32(x, self.n, first, W.SEED, W.S_XS, -1.0, 1.0)
            self.ctx.gen_uniform_f32(y, self.n, first, W.SEED, W.S_YS, -1.0, 1.0)
            self.pairs.append((x, y))
        self.turn = 0
        self.x, self.y = self.pairs[0]
        self.out = t.zeros(1, dtype=t.float32, device="cuda")
        self.k = self.ctx.kernel(self.functor("DOT")).wait()
        self.bytes = W.bytes_dot(self.n)
        if self.world > 1:
            self.sh = importlib.import_module("accelerate-cuda_b200.sharded")
            self.partials = self.peer_views(4, (1,), np.float32)
            self.result = t.zeros(1, dtype=t.float32, device="cuda")
        self.ctx.sync()

    def step(self):
        if self.sets > 1:
            self.turn = (self.turn + 1) % self.sets
            self.x, self.y = self.pairs[self.turn]
        if self.world > 1 and self.peer is not None:  # partials combined in rank order by one kernel over NVLink
            p = self.parity
            self.parity ^= 1
            self.out = self.partials[p]
            self.ctx.fold_all(self.k, [self.x, self.y], self.n, self.out, seed=np.float32(0))
            self.peer.allreduce(self.peer_offsets[p], 1, np.float32, "add", self.result)
            return 2
        self.ctx.fold_all(self.k, [self.x, self.y], self.n, self.out, seed=np.float32(0))
        if self.world > 1:  # partials all-gathered and combined in rank order
            self.result = self.sh.sharded_fold_all(self.out, lambda a, b: a + b)
        return 1

    def host_program(self):
        accb, P, t = self.accb, self.P, self.t
        v = accb.ArrayType(1, np.float32)
        prog = accb.run1With(self.ctx, lambda a, b: accb.fold(P.DOT, [a, b], np.float32, seed=np.float32(0), all=True), v, v)
        hx, hy, hout = pinned(t, self.x), pinned(t, self.y), t.zeros((), dtype=t.float32).pin_memory()
        dev = float(self.out[0])
        # the streamed run rounds the running sum to Float once per piece; the device-resident run once in all
        return prog, [hx.numpy(), hy.numpy()], [[hout.numpy()]], lambda: abs(float(hout) - dev) <= 1e-5 * abs(dev) + 1e-9 * self.n ** 0.5

    def verify(self):
        ref = float((self.x.double() * self.y.double()).sum())
        atol = 1e-9 * self.n ** 0.5  # the sum of mean-zero products may land near zero
        ok = abs(float(self.out[0]) - ref) <= 1e-5 * abs(ref) + atol
        if self.world == 1:
            oracle = importlib.import_module("oracle")
            ref2 = oracle.dot_f32(self.x.cpu().numpy(), self.y.cpu().numpy(), nthreads=host_threads())
            ok = ok and abs(float(self.out[0]) - ref2) <= 1e-5 * abs(ref2) + atol
        if self.world > 1:
            tot = self.t.tensor([ref], dtype=self.t.float64, device="cuda")
            self.sh.dist.all_reduce(tot)
            ok = ok and abs(float(self.result[0]) - float(tot[0])) <= 1e-5 * abs(float(tot[0]))
        return ok


class Dot24Workload(DotWorkload):
    """Configuration 1 at its own size: 128 MiB of input per step is about the size of L2, so the steps rotate
    through four disjoint buffer sets (512 MiB)."""
    name, dtype = "foldAll (+) 0 (zipWith (*) xs ys), Float32, 2^24, 4 rotating buffer sets", "f32"
    sets = 4

    def setup(self, n=None):
        super().setup(n or self.W.N24)


class HistWorkload(Workload):
    name, dtype = "permute (+) histogram, 2^28 Int32 keys, 4096 bins", "int32"

    def setup(self, n=None):
        t, W = self.t, self.W
        self.n = n or W.N28
        self.keys = t.empty(self.n, dtype=t.int32, device="cuda")
        cdf = t.from_numpy(W.zipf_cdf()).cuda()
        self.ctx.gen_zipf_mix_i32(self.keys, self.n, self.rank * self.n, W.SEED, cdf, W.HIST_BINS)
        self.defaults = t.zeros(W.HIST_BINS, dtype=t.int32, device="cuda")
        self.out = t.zeros(W.HIST_BINS, dtype=t.int32, device="cuda")
        self.k = self.ctx.kernel(self.functor("HIST")).wait()
        self.bytes = W.bytes_hist(self.n)
        if self.world > 1:
            self.sh = importlib.import_module("accelerate-cuda_b200.sharded")
            self.parts = self.peer_views(4 * W.HIST_BINS, (W.HIST_BINS,), np.int32)
            self.result = t.zeros(W.HIST_BINS, dtype=t.int32, device="cuda")
        self.ctx.sync()

    def step(self):
        if self.world > 1 and self.peer is not None:  # partial histograms summed in rank order by one kernel over NVLink
            p = self.parity
            self.parity ^= 1
            self.out = self.parts[p]
            self.ctx.permute(self.k, [self.keys], self.n, self.out, defaults=self.defaults)
            self.peer.allreduce(self.peer_offsets[p], self.W.HIST_BINS, np.int32, "add", self.result)
            return 2
        self.ctx.permute(self.k, [self.keys], self.n, self.out, defaults=self.defaults)
        if self.world > 1:  # per-GPU partial histograms, one all-reduce of 16 KiB
            self.result = self.sh.sharded_histogram(self.out, self.defaults)
        return 1

    def host_program(self):
        accb, P, t = self.accb, self.P, self.t
        i32 = accb.ArrayType(1, np.int32)
        prog = accb.run1With(self.ctx, lambda k, d: accb.permute(P.HIST, [k], d), i32, i32)
        hk, hd, hout = pinned(t, self.keys), pinned(t, self.defaults), pinned(t, self.out, fill=False)
        return prog, [hk.numpy(), hd.numpy()], [[hout.numpy()]], lambda: bool(t.equal(hout, self.out.cpu()))

    def verify(self):
        t = self.t
        ref = t.bincount(self.keys.long(), minlength=self.W.HIST_BINS).int()
        ok = bool(t.equal(ref, self.out)) and int(self.out.sum()) == self.n
        if self.world == 1:
            oracle = importlib.import_module("oracle")
            ref2 = oracle.permute_add_i32(self.keys.cpu().numpy(), self.W.HIST_BINS, nthreads=host_threads())
            ok = ok and bool(np.array_equal(self.out.cpu().numpy(), ref2))
        if self.world > 1:
            self.sh.dist.all_reduce(ref)
            ok = ok and bool(t.equal(ref, self.result)) and int(self.result.sum()) == self.n * self.world
        return ok


class StencilWorkload(Workload):
    name, dtype = "10 x stencil 3x3 blur Clamp, Float32 8192x8192", "f32"

    def setup(self, n=None):
        t, W = self.t, self.W
        self.h = self.w = n or 8192
        self.iters = 10
        # With several GPUs each rank owns a slab of h rows of a (world*h) x w grid, plus `iters` halo rows towards
        # each neighbour that ONE exchange per step refreshes (320 KiB each way): the ten applications then run on
        # the padded slab, and what the kernel's Clamp does at the padded edges creeps in by a row per application,
        # exactly as far as the halo reaches.
        if self.world > 1:
            self.sh = importlib.import_module("accelerate-cuda_b200.sharded")
            self.pt, self.pb = self.sh.wide_halo_layout(self.iters, "clamp")
        else:
            self.pt = self.pb = 0
        rows = self.pt + self.h + self.pb
        self.a = t.empty((rows, self.w), dtype=t.float32, device="cuda")
        self.b = t.empty_like(self.a)
        self.peer = None
        self.peer = self.make_peer(rows * self.w * 4)
        if self.peer is not None:
            # the source slab lives in the exchange buffer: the neighbours pull their halo rows out of it
            self.src = t.as_tensor(self.peer.array(0, (rows, self.w), np.float32), device="cuda")
            self.src.zero_()
        else:
            self.src = t.zeros_like(self.a)
        self.ctx.gen_uniform_f32(self.src[self.pt:self.pt + self.h], self.h * self.w, self.rank * self.h * self.w, W.SEED,
                                 W.S_GRID, 0.0, 1.0)
        self.k = self.ctx.kernel(self.functor("BLUR")).wait()
        self.bytes = W.bytes_stencil(self.h, self.w, self.iters)
        if self.world > 1:
            self.sh = importlib.import_module("accelerate-cuda_b200.sharded")
        self.ctx.sync()

    def step(self):
        if self.world == 1:
            # the source is only read, so every step does identical work; two applications per launch
            before = self.ctx.launch_count()
            self.res = self.ctx.stencil_iterate(self.k, self.a, self.b, self.iters, boundary="clamp", src=self.src)
            self.dom_launches = self.ctx.launch_count() - before  # 5: every launch does two applications
            return self.dom_launches
        if self.peer is not None:  # barrier, two pulls over NVLink, barrier: the library's own kernels
            self.sh.peer_wide_halos(self.peer, 0, self.h, self.w * 4, self.iters, "clamp")
        else:
            self.sh.exchange_wide_halos(self.src, self.pt, self.pb)  # in place: the data lives in the padded slab
        before = self.ctx.launch_count()
        res = self.ctx.stencil_iterate(self.k, self.a, self.b, self.iters, boundary="clamp", src=self.src)
        self.res = res[self.pt:self.pt + self.h]
        return self.ctx.launch_count() - before + (2 + bool(self.pt) + bool(self.pb) if self.peer is not None else 0)

    def host_program(self):
        accb, P, t = self.accb, self.P, self.t
        g = accb.ArrayType(2, np.float32)
        prog = accb.run1With(self.ctx, lambda a: accb.stencil(P.BLUR, a, boundary="clamp", iters=self.iters), g)
        hin, hout = pinned(t, self.src), pinned(t, self.res, fill=False)
        return prog, [hin.numpy()], [[hout.numpy()]], lambda: bool(t.equal(hout, self.res.cpu()))

    def verify(self):
        """Bands of 48 result rows at the top, the middle and the bottom of this rank's slab against the oracle's
        ten-step recurrence (float64 state).  The oracle's input is a band of the GLOBAL (world*h) x w grid widened
        by ten rows each way, made on the host by the numpy generator: it shares neither the device generator nor
        the halo exchange with what it checks.  Where the widened band is cut inside the grid the oracle's Clamp
        is wrong there, which reaches ten rows inwards: exactly the widening."""
        r, t, W = self.res, self.t, self.W
        oracle = importlib.import_module("oracle")
        H, band, reach = self.h * self.world, 48, self.iters
        ok = True
        for local0 in (0, self.h // 2 - band // 2, self.h - band):
            g0 = self.rank * self.h + local0  # first global row of the band
            lo, hi = max(0, g0 - reach), min(H, g0 + band + reach)
            src = W.uniform_f32(W.SEED, W.S_GRID, (hi - lo) * self.w, 0.0, 1.0, first=lo * self.w).reshape(hi - lo, self.w)
            ref = oracle.stencil2d_iter(src, W.BLUR_WEIGHTS, self.iters, "clamp", nthreads=host_threads())
            ok = ok and close_to(r[local0:local0 + band].cpu().numpy(), ref[g0 - lo:g0 - lo + band], 1e-6)
        # everywhere: blur with Clamp keeps values inside [min, max] of the source
        interior = self.src[self.pt:self.pt + self.h]
        ok = ok and bool(r.min() >= interior.min() - 1e-6) and bool(r.max() <= interior.max() + 1e-6)
        if self.world == 1:
            return ok and abs(float(r.mean()) - float(interior.mean())) < 1e-3
        # several GPUs: the wide-halo scheme against one exchange of a single row per application, bit for bit
        cur = t.zeros((self.h + 2, self.w), dtype=t.float32, device="cuda")
        cur[1:-1] = interior
        nxt = t.empty_like(cur)
        for _ in range(self.iters):
            self.sh.exchange_halos(cur, 1, "clamp")
            self.ctx.stencil(self.k, cur, nxt, boundary="clamp")
            cur, nxt = nxt, cur
        self.ctx.sync()
        return ok and bool(t.equal(cur[1:-1], r))


class BlackScholesWorkload(Workload):
    name, dtype = "map Black-Scholes, 2^26 options, Float32", "f32"

    def setup(self, n=None):
        t, W = self.t, self.W
        self.n = n or W.N26
        mk = lambda: t.empty(self.n, dtype=t.float32, device="cuda")
        self.s, self.k_, self.y, self.call, self.put = mk(), mk(), mk(), mk(), mk()
        self.first = self.rank * self.n  # each rank prices its own slice of world*n options: no exchange
        self.ctx.gen_uniform_f32(self.s, self.n, self.first, W.SEED, W.S_SPOT, 5.0, 30.0)
        self.ctx.gen_uniform_f32(self.k_, self.n, self.first, W.SEED, W.S_STRIKE, 1.0, 100.0)
        self.ctx.gen_uniform_f32(self.y, self.n, self.first, W.SEED, W.S_YEARS, 0.25, 10.0)
        self.k = self.ctx.kernel(self.functor("BLACKSCHOLES")).wait()
        self.bytes = W.bytes_blackscholes(self.n)
        self.ctx.sync()

    def step(self):
        self.ctx.map(self.k, [(self.s, self.k_, self.y)], (self.call, self.put))
        return 1

    def host_program(self):
        accb, P, t = self.accb, self.P, self.t
        prog = accb.run1With(self.ctx, lambda o: accb.map_(P.BLACKSCHOLES, [o], accb.ArrayType(1, [np.float32, np.float32])),
                             accb.ArrayType(1, [np.float32] * 3))
        hs, hk, hy = pinned(t, self.s), pinned(t, self.k_), pinned(t, self.y)
        hc, hp = pinned(t, self.call, fill=False), pinned(t, self.put, fill=False)
        return (prog, [(hs.numpy(), hk.numpy(), hy.numpy())], [[hc.numpy(), hp.numpy()]],
                lambda: bool(t.equal(hc, self.call.cpu())) and bool(t.equal(hp, self.put.cpu())))

    def verify(self):
        """Every option: put-call parity, call - put = S - K exp(-rT).  Every 1024th option (2^16 of them): both
        prices against the oracle's float64 closed form on inputs made by the numpy generator."""
        t, W = self.t, self.W
        lhs = (self.call - self.put).double()
        rhs = self.s.double() - self.k_.double() * t.exp(-0.02 * self.y.double())
        ok = bool(((lhs - rhs).abs() <= 1e-5 * rhs.abs() + 1e-4).all())
        oracle = importlib.import_module("oracle")
        stride = max(1, self.n >> 16)
        idx = np.arange(0, self.n, stride)
        gen = lambda stream, lo, hi: np.concatenate(  # noqa: E731
            [W.uniform_f32(W.SEED, stream, 1, lo, hi, first=self.first + int(i)) for i in idx[:64]])
        # the strided sample comes from the device arrays; its first 64 entries are also regenerated on the host
        pick = t.from_numpy(idx).cuda()
        s, k, y = (a[pick].cpu().numpy() for a in (self.s, self.k_, self.y))
        ok = ok and np.array_equal(s[:64], gen(W.S_SPOT, 5.0, 30.0)) and np.array_equal(k[:64], gen(W.S_STRIKE, 1.0, 100.0))
        rc, rp = oracle.blackscholes(s, k, y, nthreads=host_threads())
        return ok and close_to(self.call[pick].cpu().numpy(), rc, 2e-5) and close_to(self.put[pick].cpu().numpy(), rp, 2e-5)


class RowSumWorkload(Workload):
    name, dtype = "fold (+) 0 over rows, Float32 16384x16384", "f32"

    def setup(self, n=None):
        t, W = self.t, self.W
        self.rows = self.cols = n or 16384
        self.m = t.empty((self.rows, self.cols), dtype=t.float32, device="cuda")
        # each rank sums its own slab of rows of a (world*rows) x cols matrix: no exchange, results stay sharded
        self.ctx.gen_uniform_f32(self.m, self.rows * self.cols, self.rank * self.rows * self.cols, W.SEED, W.S_MATRIX,
                                 -1.0, 1.0)
        self.out = t.zeros(self.rows, dtype=t.float32, device="cuda")
        self.k = self.ctx.kernel(self.functor("ROWSUM")).wait()
        self.bytes = W.bytes_rowsum(self.rows, self.cols)
        self.ctx.sync()

    def step(self):
        self.ctx.fold_dim(self.k, [self.m], self.rows, self.cols, self.out, seed=np.float32(0))
        return 1

    def host_program(self):
        accb, P, t = self.accb, self.P, self.t
        prog = accb.run1With(self.ctx, lambda a: accb.fold(P.ROWSUM, [a], np.float32, seed=np.float32(0)),
                             accb.ArrayType(2, np.float32))
        hm, hout = pinned(t, self.m), pinned(t, self.out, fill=False)
        return prog, [hm.numpy()], [[hout.numpy()]], lambda: bool(t.equal(hout, self.out.cpu()))

    def verify(self):
        ref = self.m.double().sum(dim=1)
        ok = bool(((self.out.double() - ref).abs() <= 1e-5 * ref.abs() + 1e-6).all())
        # every 64th row against the oracle's float64 row sums
        oracle = importlib.import_module("oracle")
        rows = self.m[::64].contiguous().cpu().numpy()
        return ok and close_to(self.out[::64].cpu().numpy(), oracle.fold_rows_f32(rows, nthreads=host_threads()), 1e-6)


class ScanPrimeWorkload(Workload):
    """scanl' (+) 0: the n-element body plus the total as a separate scalar (the second half of configuration 2)."""
    name, dtype = "scanl' (+) 0, Int32, 2^28", "int32"

    def setup(self, n=None):
        t, W = self.t, self.W
        self.n = n or W.N28
        self.x = t.empty(self.n, dtype=t.int32, device="cuda")
        self.ctx.gen_uniform_i32(self.x, self.n, 0, W.SEED, W.S_SCAN, 16)
        self.out = t.empty(self.n, dtype=t.int32, device="cuda")
        self.total = t.zeros(1, dtype=t.int32, device="cuda")
        self.k = self.ctx.kernel(self.functor("SCAN_ADD_I32")).wait()
        self.bytes = W.bytes_scan(self.n)
        self.ctx.sync()

    def step(self):
        self.ctx.scan(self.k, [self.x], self.n, self.out, kind=self.accb.SCAN_PRIME, seed=np.int32(0), total=self.total)
        return 1

    def verify(self):
        t = self.t
        oracle = importlib.import_module("oracle")
        ref = oracle.scanl_i32(self.x.cpu().numpy(), 0, nthreads=host_threads())
        return bool(t.equal(self.out, t.from_numpy(ref[:-1]).cuda())) and int(self.total[0]) == int(ref[-1])


# ---- secondary shapes and types of the same skeletons (not BASELINE configurations; --workload selects them
# ---- for profiling, and the default run reports them in a table of their own)
class Scan64Workload(Workload):
    """Accelerate's Int is 64 bits wide: the default integer scan."""
    name, dtype = "scanl (+) 0, Int64, 2^27", "int64"

    def setup(self, n=None):
        t = self.t
        self.n = n or (1 << 27)
        x32 = t.empty(self.n, dtype=t.int32, device="cuda")
        self.ctx.gen_uniform_i32(x32, self.n, 0, self.W.SEED, self.W.S_SCAN, 16)
        self.x = x32.long()
        del x32
        self.out = t.empty(self.n + 1, dtype=t.int64, device="cuda")
        self.k = self.ctx.kernel(self.functor("SCAN_ADD_I64")).wait()
        self.bytes = 16 * self.n + 8
        self.ctx.sync()

    def step(self):
        self.ctx.scan(self.k, [self.x], self.n, self.out, seed=np.int64(0))
        return 1

    def verify(self):
        return bool(self.t.equal(self.out[1:] - self.out[:-1], self.x)) and int(self.out[0]) == 0


class ShortRowsWorkload(Workload):
    name, dtype = "fold (+) 0 over rows, Float32 2^24 x 16", "f32"

    def setup(self, n=None):
        t, W = self.t, self.W
        self.rows, self.cols = n or (1 << 24), 16
        self.m = t.empty((self.rows, self.cols), dtype=t.float32, device="cuda")
        self.ctx.gen_uniform_f32(self.m, self.rows * self.cols, 0, W.SEED, W.S_MATRIX, -1.0, 1.0)
        self.out = t.zeros(self.rows, dtype=t.float32, device="cuda")
        self.k = self.ctx.kernel(self.functor("ROWSUM")).wait()
        self.bytes = W.bytes_rowsum(self.rows, self.cols)
        self.ctx.sync()

    def step(self):
        self.ctx.fold_dim(self.k, [self.m], self.rows, self.cols, self.out, seed=np.float32(0))
        return 1

    def verify(self):
        ref = self.m.double().sum(dim=1)
        return bool(((self.out.double() - ref).abs() <= 1e-5 * ref.abs() + 1e-6).all())


class SmvmWorkload(Workload):
    """Sparse matrix x dense vector, CSR: foldSeg (+) 0 (zipWith (*) vals (gather cols vec)) offsets; 2^24 rows of
    0..16 non-zeros (mean 8), 2^20 columns."""
    name, dtype = "smvm: foldSeg over 2^24 rows, mean 8 non-zeros, Float32", "f32"

    def setup(self, n=None):
        t, W = self.t, self.W
        self.rows, self.ncols = n or (1 << 24), 1 << 20
        lens = t.empty(self.rows, dtype=t.int32, device="cuda")
        self.ctx.gen_uniform_i32(lens, self.rows, 0, W.SEED, W.S_SCAN, 17)
        self.offs = t.zeros(self.rows + 1, dtype=t.int32, device="cuda")
        self.offs[1:] = t.cumsum(lens, 0)
        self.nnz = int(self.offs[-1])
        self.vals = t.empty(self.nnz, dtype=t.float32, device="cuda")
        self.colidx = t.empty(self.nnz, dtype=t.int32, device="cuda")
        self.vec = t.empty(self.ncols, dtype=t.float32, device="cuda")
        self.ctx.gen_uniform_f32(self.vals, self.nnz, 0, W.SEED, W.S_XS, -1.0, 1.0)
        self.ctx.gen_uniform_i32(self.colidx, self.nnz, 0, W.SEED, W.S_YS, self.ncols)
        self.ctx.gen_uniform_f32(self.vec, self.ncols, 0, W.SEED, W.S_MATRIX, -1.0, 1.0)
        self.out = t.zeros(self.rows, dtype=t.float32, device="cuda")
        self.k = self.ctx.kernel(self.functor("SMVM")).wait()
        # values + column indices + offsets in, one Float per row out; the gathered vector (4 MiB) lives in L2
        self.bytes = 8 * self.nnz + 4 * (self.rows + 1) + 4 * self.rows
        self.ctx.sync()

    def step(self):
        self.ctx.fold_seg(self.k, [(self.vals, self.colidx), self.vec], 1, self.nnz, self.offs, self.rows, self.out,
                          seed=np.float32(0))
        return 2 if self.nnz >= (1 << 24) else 1  # sources of 2^24 elements and more get the second launch

    def verify(self):
        t = self.t
        prod = (self.vals * self.vec[self.colidx.long()]).double()
        csum = t.cat([t.zeros(1, dtype=t.float64, device="cuda"), t.cumsum(prod, 0)])
        ref = csum[self.offs[1:].long()] - csum[self.offs[:-1].long()]
        return bool(((self.out.double() - ref).abs() <= 1e-5 * ref.abs() + 1e-4).all())


class SmvmBandedWorkload(SmvmWorkload):
    """The same product with the non-zeros of row r in columns (r mod 2^20) .. + 63: the gathers of neighbouring rows
    share cache lines, as they do for matrices that come from meshes and grids."""
    name = "smvm: foldSeg over 2^24 rows, mean 8 non-zeros within 64 columns of a diagonal, Float32"

    def setup(self, n=None):
        super().setup(n)
        t = self.t
        row_of = t.repeat_interleave(t.arange(self.rows, device="cuda"), (self.offs[1:] - self.offs[:-1]).long())
        self.colidx = ((row_of + self.colidx.long() % 64) % self.ncols).int()
        del row_of
        self.ctx.sync()


class FoldSegWorkload(Workload):
    """foldSeg (+) 0 over 2^27 Int32 cut into segments of random length, mean 50 (0..100)."""
    name, dtype = "foldSeg (+) 0, Int32, 2^27 elements, segment lengths uniform in 0..100", "int32"
    mean = 50

    def lengths(self, n):
        t, W = self.t, self.W
        lens = t.empty(int(n * 0.95) // self.mean, dtype=t.int32, device="cuda")
        self.ctx.gen_uniform_i32(lens, lens.numel(), 0, W.SEED, W.S_SCAN, 2 * self.mean + 1)
        return lens

    def setup(self, n=None):
        t, W = self.t, self.W
        n = n or (1 << 27)
        lens = self.lengths(n)
        self.nseg = lens.numel()
        self.offs = t.zeros(self.nseg + 1, dtype=t.int32, device="cuda")
        self.offs[1:] = t.cumsum(lens.long(), 0).int()
        self.n = int(self.offs[-1])
        self.x = t.empty(self.n, dtype=t.int32, device="cuda")
        self.ctx.gen_uniform_i32(self.x, self.n, 0, W.SEED, W.S_XS, 16)
        self.out = t.zeros(self.nseg, dtype=t.int32, device="cuda")
        self.k = self.ctx.kernel(self.functor("SEGSUM_I32")).wait()
        self.bytes = 4 * self.n + 4 * (self.nseg + 1) + 4 * self.nseg
        self.ctx.sync()

    def step(self):
        self.ctx.fold_seg(self.k, [self.x], 1, self.n, self.offs, self.nseg, self.out, seed=np.int32(0))
        return 2 if self.n >= (1 << 24) else 1  # sources of 2^24 elements and more get the second launch

    def verify(self):
        t = self.t
        csum = t.cat([t.zeros(1, dtype=t.int64, device="cuda"), t.cumsum(self.x, 0, dtype=t.int64)])
        ref = csum[self.offs[1:].long()] - csum[self.offs[:-1].long()]
        return bool(t.equal(self.out, ref.int()))


class FoldSegGiantsWorkload(FoldSegWorkload):
    """Short segments (0..16 elements) with three of 20 M, 9 M and 3 M elements among them: the long ones are handed
    to the second launch, which splits them over all blocks."""
    name = "foldSeg (+) 0, Int32, 8 M segments of 0..16 elements and three of 20 M, 9 M and 3 M"
    mean = 8

    def lengths(self, n):
        t, W = self.t, self.W
        lens = t.empty(8_000_000, dtype=t.int32, device="cuda")
        self.ctx.gen_uniform_i32(lens, lens.numel(), 0, W.SEED, W.S_SCAN, 17)
        lens[[5, 4_000_000, 7_999_999]] = t.tensor([20_000_000, 9_000_000, 3_000_001], dtype=t.int32, device="cuda")
        return lens


class FoldSegLongWorkload(FoldSegWorkload):
    """Eight segments of 2^24 elements: every one goes to the second launch."""
    name = "foldSeg (+) 0, Int32, 8 segments of 2^24 elements"

    def lengths(self, n):
        return self.t.full((8,), 1 << 24, dtype=self.t.int32, device="cuda")


class Smooth1dWorkload(Workload):
    name, dtype = "stencil 3-tap smoothing Clamp, Float32 vector of 2^28", "f32"

    def setup(self, n=None):
        t, W = self.t, self.W
        self.n = n or W.N28
        self.v = t.empty(self.n, dtype=t.float32, device="cuda")
        self.ctx.gen_uniform_f32(self.v, self.n, 0, W.SEED, W.S_GRID, 0.0, 1.0)
        self.out = t.empty_like(self.v)
        self.k = self.ctx.kernel(self.functor("SMOOTH1D")).wait()
        self.bytes = 8 * self.n
        self.ctx.sync()

    def step(self):
        self.ctx.stencil(self.k, self.v, self.out, boundary="clamp")
        return 1

    def verify(self):
        v, o = self.v, self.out
        ref = 0.25 * v[:-2] + 0.5 * v[1:-1] + 0.25 * v[2:]
        edge = abs(float(o[0]) - (0.75 * float(v[0]) + 0.25 * float(v[1]))) <= 1e-6
        return bool(((o[1:-1] - ref).abs() <= 1e-6).all()) and edge


class TransposeWorkload(Workload):
    """`transpose m` made manifest: the map skeleton over 64x64 shared-memory tiles (the reference runs a transpose
    as a backpermute, i.e. a gather)."""
    name, dtype = "transpose, Float32 8192 x 8192 (tiles moved by the copy engine through tensor maps)", "f32"

    def setup(self, n=None):
        t, W = self.t, self.W
        self.side = n or 8192
        self.m = t.empty((self.side, self.side), dtype=t.float32, device="cuda")
        self.ctx.gen_uniform_f32(self.m, self.side * self.side, 0, W.SEED, W.S_MATRIX, -1.0, 1.0)
        self.out = t.empty_like(self.m)
        # the plain map functor (out = in) that the embedded language prints for `transpose`
        spec = importlib.import_module("accelerate-cuda_b200.examples").generated_specs()["TRANSPOSE_TILED"]
        self.k = self.ctx.kernel(spec).wait()
        self.bytes = 8 * self.side * self.side
        self.ctx.sync()

    def step(self):
        self.ctx.map_transposed(self.k, [self.m], self.out)
        return 1

    def verify(self):
        return bool(self.t.equal(self.out, self.m.T))


class HistEqualWorkload(HistWorkload):
    """The adversarial histogram: every key is the same, so every update of a warp meets in one bin."""
    name = "permute (+) histogram, 2^28 Int32 keys, all keys equal"

    def setup(self, n=None):
        super().setup(n)
        self.keys.fill_(1234)
        self.ctx.sync()


class HistHotWorkload(HistWorkload):
    """Sixteen hot bins (uniform over bins 0, 256, 512, ..): a warp's 32 updates fall on 16 addresses."""
    name = "permute (+) histogram, 2^28 Int32 keys, 16 hot bins"

    def setup(self, n=None):
        super().setup(n)
        self.ctx.gen_uniform_i32(self.keys, self.n, 0, self.W.SEED, self.W.S_UNIF, 16)
        self.keys.mul_(256)
        self.ctx.sync()


class ScanChainedWorkload(Workload):
    """The kernel of the scan over several GPUs on ONE GPU (a world of one): the vector in blocks of 32 tiles, block
    records written and read by the same GPU.  What the chain of blocks costs without any NVLink latency."""
    name, dtype = "scanl (+) 0, Int32, 2^28, block-chained kernel of the multi-GPU scan (world of one)", "int32"

    def setup(self, n=None):
        t, W = self.t, self.W
        self.k = self.ctx.kernel(self.functor("SCAN_ADD_I32")).wait()
        self.block = 32 * self.ctx.scan_tile(self.k)
        self.n = (n or W.N28) // self.block * self.block
        self.x = t.empty(self.n, dtype=t.int32, device="cuda")
        self.ctx.gen_uniform_i32(self.x, self.n, 0, W.SEED, W.S_SCAN, 16)
        self.out = t.empty(self.n + 1, dtype=t.int32, device="cuda")
        _, _, scratch = self.accb.scan_layout(1, 0, self.n, self.block)
        self.chain = self.accb.Peer(self.ctx, 0, 1, scratch, lambda b: [b])
        self.bytes = W.bytes_scan(self.n)
        self.ctx.sync()

    def step(self):
        self.chain.scan(self.k, [self.x], self.n, self.out, seed=np.int32(0), block_elems=self.block)
        return 1

    def verify(self):
        t = self.t
        ok = bool(t.equal(self.out[1:] - self.out[:-1], self.x)) and int(self.out[0]) == 0
        return ok and int(self.out[-1]) == int(np.array(int(self.x.sum(dtype=t.int64)) & 0xffffffff, np.uint32).astype(np.int32))


class TransposeLoadStoreWorkload(TransposeWorkload):
    """The same transpose with the tiles moved by load and store instructions (a context created with
    ACCB_TRANSPOSE_TMA=0) instead of the copy engine."""
    name = "transpose, Float32 8192 x 8192 (tiles moved by loads and stores)"

    def setup(self, n=None):
        old = os.environ.get("ACCB_TRANSPOSE_TMA")
        os.environ["ACCB_TRANSPOSE_TMA"] = "0"  # read when a context is created
        try:
            self.ctx = self.accb.Context(self.ctx.device)
        finally:
            if old is None:
                del os.environ["ACCB_TRANSPOSE_TMA"]
            else:
                os.environ["ACCB_TRANSPOSE_TMA"] = old
        super().setup(n)


class Stencil3dWorkload(Workload):
    """27-point weighted stencil over a 512^3 cube (rank 3): a block marches along z with three plane tiles in
    shared memory."""
    name, dtype = "stencil 3x3x3 Clamp, Float32 512^3", "f32"

    def setup(self, n=None):
        t, W = self.t, self.W
        self.side = n or 512
        shape = (self.side,) * 3
        self.v = t.empty(shape, dtype=t.float32, device="cuda")
        self.ctx.gen_uniform_f32(self.v, self.side ** 3, 0, W.SEED, W.S_GRID, 0.0, 1.0)
        self.out = t.empty_like(self.v)
        self.k = self.ctx.kernel(self.P.WEIGHTED27).wait()
        self.bytes = 8 * self.side ** 3
        self.ctx.sync()

    def step(self):
        self.ctx.stencil(self.k, self.v, self.out, boundary="clamp")
        return 1

    def verify(self):
        # the first 12 planes against the oracle (clamped at the cut: the last plane compared is two away from it)
        oracle = importlib.import_module("oracle")
        w = (np.arange(27, dtype=np.float64).reshape(3, 3, 3) + 1) / 378.0
        ref = oracle.stencil3d(self.v[:12].cpu().numpy(), w, "clamp")
        return close_to(self.out[:10].cpu().numpy(), ref[:10], 1e-6)


class Stencil3dLaplaceWorkload(Stencil3dWorkload):
    """The 7-point Laplacian over the same cube: the taps a functor does not use are never read."""
    name = "stencil 7-point Laplacian Clamp, Float32 512^3"

    def setup(self, n=None):
        super().setup(n)
        self.k = self.ctx.kernel(self.P.LAPLACE3).wait()

    def verify(self):
        oracle = importlib.import_module("oracle")
        w = np.zeros((3, 3, 3))
        w[1, 1, 1] = -6
        for z, y, x in ((0, 1, 1), (2, 1, 1), (1, 0, 1), (1, 2, 1), (1, 1, 0), (1, 1, 2)):
            w[z, y, x] = 1
        ref = oracle.stencil3d(self.v[:12].cpu().numpy(), w, "clamp")
        return close_to(self.out[:10].cpu().numpy(), ref[:10], 1e-5)


SECONDARY_KERNEL = {"scan_chained": "scanl_bc", "hist_equal": "permute_smem", "hist_hot16": "permute_smem", "scan64": "scanl", "shortrows": "fold_staged", "smvm": "foldSeg_staged", "smooth1d": "stencil_line",
                    "smvm_banded": "foldSeg_staged", "foldseg_irregular": "foldSeg_staged", "foldseg_giants": "foldSeg_staged", "foldseg_long": "foldSeg_deferred",
                    "transpose": "map_transposed_tma", "transpose_loadstore": "map_transposed", "stencil3d": "stencil3", "stencil3d_laplace": "stencil3"}
SECONDARY = {"scan_chained": ScanChainedWorkload, "hist_equal": HistEqualWorkload, "hist_hot16": HistHotWorkload, "scan64": Scan64Workload, "shortrows": ShortRowsWorkload, "smvm": SmvmWorkload, "smooth1d": Smooth1dWorkload,
             "smvm_banded": SmvmBandedWorkload, "foldseg_irregular": FoldSegWorkload, "foldseg_giants": FoldSegGiantsWorkload, "foldseg_long": FoldSegLongWorkload,
             "transpose": TransposeWorkload, "transpose_loadstore": TransposeLoadStoreWorkload, "stencil3d": Stencil3dWorkload, "stencil3d_laplace": Stencil3dLaplaceWorkload}


# ---- the reference's own algorithms on the same GPU and the same device inputs (baseline/refskel)
def ref_algorithm(torch, wl, sm_count):
    """Times the reference's algorithm for wl's program; returns {"GB/s", "ms", "check", "note"}.
    Call after wl has run and verified: its result is what the baseline's result is checked against."""
    R = importlib.import_module("baseline.refskel")
    t = torch
    scratch = R.scratch_elems(sm_count)
    nbytes, note = wl.bytes, None
    if isinstance(wl, ScanWorkload):
        out2, blk = t.empty_like(wl.out), t.empty(scratch, dtype=t.int32, device="cuda")
        fn = lambda: R.scanl(wl.x, 0, out2, blk)
        check = lambda: bool(t.equal(out2, wl.out))
        note = "3 launches: interval totals, scan of totals, second pass over the input"
    elif isinstance(wl, DotWorkload):
        out2, part = t.zeros(1, device="cuda"), t.empty(scratch, dtype=t.float32, device="cuda")
        fn = lambda: R.dot(wl.x, wl.y, 0.0, part, out2)
        check = lambda: abs(float(out2[0]) - float(wl.out[0])) <= 1e-6 * wl.n  # float32 accumulation, as the reference
        note = "foldAll relaunched on the partials until one block is left; float32 accumulator"
    elif type(wl) is HistWorkload:  # not the adversarial variants: a lock that every key shares serialises the whole sample
        # Every update of a hot bin is serialised by its lock while hundreds of thousands of threads
        # spin on it (measured: ~0.2 ms per update of one shared bin), so a small bounded sample.
        m = min(wl.n, 1 << 16)
        keys = wl.keys[:m]
        out2, lock = t.zeros_like(wl.out), t.zeros_like(wl.out)
        err = t.zeros(1, dtype=t.int32, device="cuda")
        fn = lambda: R.histogram(keys, wl.defaults, out2, lock, err)
        check = lambda: bool(t.equal(out2, t.bincount(keys.long(), minlength=out2.numel()).int())) and int(err[0]) == 0
        nbytes = wl.W.bytes_hist(m)
        note = "spin lock per destination element; first 2^16 of the keys"
    elif isinstance(wl, StencilWorkload):
        a2, b2 = t.empty_like(wl.a), t.empty_like(wl.a)
        def fn():
            R.stencil_blur(wl.src, a2)
            cur, nxt = a2, b2
            for _ in range(wl.iters - 1):
                R.stencil_blur(cur, nxt)
                cur, nxt = nxt, cur
            fn.res = cur
        check = lambda: bool(((fn.res - wl.res).abs() <= 1e-5).all())
        note = "one element per thread, nine global loads; one launch per application (the reference launches each twice)"
    elif isinstance(wl, BlackScholesWorkload):
        c2, p2 = t.empty_like(wl.call), t.empty_like(wl.put)
        fn = lambda: R.map_blackscholes(wl.s, wl.k_, wl.y, c2, p2)
        check = lambda: bool(((c2 - wl.call).abs() <= 1e-4).all()) and bool(((p2 - wl.put).abs() <= 1e-4).all())
        note = "one element per thread per trip, scalar accesses; same functor and math flags"
    elif isinstance(wl, RowSumWorkload):
        out2 = t.empty_like(wl.out)
        fn = lambda: R.fold_rows(wl.m, 0.0, out2)
        check = lambda: bool(((out2 - wl.out).abs() <= 1e-2).all())  # float32 accumulation, as the reference
        note = "one block per row, shared-memory tree"
    else:
        return None
    fn()
    t.cuda.synchronize()
    e0, e1 = t.cuda.Event(enable_timing=True), t.cuda.Event(enable_timing=True)
    steps = 3
    e0.record()
    for _ in range(steps):
        fn()
    e1.record()
    t.cuda.synchronize()
    ms = e0.elapsed_time(e1) / steps
    return {"GB/s": nbytes / (ms * 1e-3) / 1e9, "ms": ms, "check": check(), "note": note}


WORKLOADS = {"scan": ScanWorkload, "dot": DotWorkload, "hist": HistWorkload, "stencil": StencilWorkload,
             "blackscholes": BlackScholesWorkload, "rowsum": RowSumWorkload}
# the configurations' own sizes and forms where they differ from the 2^28 headline (one GPU)
CONFIG_EXTRAS = {"dot_n24": Dot24Workload, "scan_prime": ScanPrimeWorkload}


def awhile_sample(accb, ctx, torch, side=128, iters=200):
    """`awhile` around a 5-point stencil and a counter, the loop driven from the host (the flag read back every
    iteration, as the reference does) and resident on the device (one graph launch with a conditional WHILE
    node): wall-clock microseconds per iteration, the host being part of what is measured."""
    A = importlib.import_module("accelerate-cuda_b200.lang")
    f32, i32 = np.float32, np.int32
    five = lambda t: 0.2 * (t[0][1] + t[1][0] + t[1][1] + t[1][2] + t[2][1])  # noqa: E731
    types = (A.matrix(f32), A.scalar(i32))
    cond = A.run1With(ctx, lambda a, c: A.map(lambda v: v < iters, c), *types)
    body = A.run1With(ctx, lambda a, c: (A.stencil(five, "clamp", a), A.map(lambda v: v + 1, c)), *types)
    grid = torch.rand((side, side), device="cuda")
    count = torch.zeros((), dtype=torch.int32, device="cuda")
    stream = torch.cuda.Stream()
    out = {"program": f"{iters} x 5-point stencil on {side}x{side} Float32 + counter", "unit": "us per iteration"}
    for mode, device in (("host_loop", False), ("device_loop", True)):
        best = None
        for _ in range(4):
            count.zero_()
            torch.cuda.synchronize()
            t0 = time.perf_counter()
            n = accb.awhile(cond, body, [grid, count], device=device, max_iters=10 * iters, stream=stream.cuda_stream,
                            count=True)
            dt = time.perf_counter() - t0
            best = dt if best is None else min(best, dt)
        out[mode] = best / max(n, 1) * 1e6
        out["iterations_ok"] = out.get("iterations_ok", True) and n == iters
    cond.destroy()
    body.destroy()
    return out


def time_steps(torch, wl, steps, warmup):
    """K steps between two CUDA events on the launching (current) stream; returns (ms total, launches)."""
    for _ in range(warmup):
        wl.step()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    launches = 0
    e0.record()
    for _ in range(steps):
        launches += wl.step()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1), launches


# --------------------------------------------------------- CPU reference arm
def cpu_scan_sample(threads: int, n: int, repeats: int):
    oracle = importlib.import_module("oracle")
    W = importlib.import_module("accelerate-cuda_b200.workloads")
    x = W.uniform_i32(W.SEED, W.S_SCAN, n, 16)
    best = float("inf")
    for _ in range(repeats):
        t0 = time.perf_counter()
        out = oracle.scanl_i32(x, 0, nthreads=threads)
        best = min(best, time.perf_counter() - t0)
    assert int(out[-1]) == int(x.astype(np.int64).sum() & 0xffffffff)
    return W.bytes_scan(n) / best / 1e9, best


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    oracle = importlib.import_module("oracle")
    threads = host_threads()
    # the GPU arm's size: 2^28 elements per step (1 GiB in, 1 GiB out; a step takes tens of milliseconds).  The
    # values repeat with period 2^24 -- the time of an integer prefix sum does not depend on them -- so that
    # generating the input does not take longer than the measurement.
    n = 1 << 28
    W = importlib.import_module("accelerate-cuda_b200.workloads")
    x = np.tile(W.uniform_i32(W.SEED, W.S_SCAN, 1 << 24, 16), n >> 24)
    for _ in range(args.warmup):
        oracle.scanl_i32(x, 0, nthreads=threads)
    t0 = time.perf_counter()
    for _ in range(args.steps):
        out = oracle.scanl_i32(x, 0, nthreads=threads)
    dt = time.perf_counter() - t0
    assert int(out[-1]) == int(x.astype(np.int64).sum() & 0xffffffff)
    gbs = W.bytes_scan(n) * args.steps / dt / 1e9
    line = {
        "impl": "reference", "metric": METRIC, "value": gbs, "unit": "GB/s", "n_gpus": args.gpus, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": dt / args.steps * 1e3, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "int32", "data": "synthetic",
        "config": {"workload": ScanWorkload.name, "threads": threads,
                   "sample": "the full 2^28 elements per step (one GPU's share; the values repeat with period 2^24)"},
        "cpu_baseline": {"value": gbs, "unit": "GB/s", "cores": threads, "kind": "port",
                         "sample": "scanl (+) 0 over 2^28 Int32 per step, blocked two-pass OpenMP scan on %d threads" % threads},
        "e2e": {"value": gbs, "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "note": "the reference's own CPU path (Accelerate's interpreter) cannot be built here (no GHC); this is the C oracle port",
    }
    print(json.dumps(line), flush=True)


def measure(torch, dist, wl, steps, warmup):
    """(ms per step as the max over ranks, launches per step, parity as the min over ranks) of a workload that has
    been set up; every rank calls this."""
    if dist:
        dist.barrier()
    torch.cuda.synchronize()
    ms, launches = time_steps(torch, wl, steps, warmup)
    if dist:
        tm = torch.tensor([ms], device="cuda", dtype=torch.float64)
        dist.all_reduce(tm, op=dist.ReduceOp.MAX)
        ms = float(tm[0])
        dist.barrier()
    ok = bool(wl.verify())
    if dist:
        okt = torch.tensor([int(ok)], device="cuda")
        dist.all_reduce(okt, op=dist.ReduceOp.MIN)
        ok = bool(okt[0])
    return ms / steps, launches // steps, ok


def release(torch, dist, wl):
    """Frees a workload; with several ranks its exchange buffer only after every rank is done with the others'."""
    peer = getattr(wl, "peer", None)
    if dist:
        dist.barrier()
    if peer is not None:
        peer.status()
        peer.destroy()
        dist.barrier()
    torch.cuda.empty_cache()


def e2e_single(torch, wl, steps):
    """A workload's program through run1 on pinned HOST arrays: uploads, launches and downloads inside the timed
    region (wall clock around the calls)."""
    prog, ins, outs, check = wl.host_program()
    for _ in range(2):
        prog(*ins, out=outs)
    reps = max(3, min(steps, 5))
    t0 = time.perf_counter()
    for _ in range(reps):
        prog(*ins, out=outs)
    dt = (time.perf_counter() - t0) / reps
    ok = bool(check())
    prog.destroy()
    nbytes = lambda arrays: int(sum(a.nbytes for x in arrays for a in (x if isinstance(x, (tuple, list)) else [x])))  # noqa: E731
    return {"value": wl.bytes / dt / 1e9, "unit": "GB/s", "h2d_bytes_per_step": nbytes(ins), "d2h_bytes_per_step": nbytes(outs),
            "ms_per_step": dt * 1e3, "steps": reps, "parity_check": ok}


def e2e_sharded(torch, dist, wl, world):
    """The scan end to end on N GPUs: every rank uploads its share from pinned host memory, takes part in the
    exchange, scans, and downloads its part of the result; wall clock between barriers, max over ranks.  With the
    vector dealt in blocks the three overlap, piece by piece (sharded.PeerScanFromHost)."""
    n = wl.n
    hin = pinned(torch, wl.x)
    hout = torch.empty(n + 1, dtype=torch.int32).pin_memory()
    note = "upload, exchange, scan, download per rank; not pipelined"
    if getattr(wl, "cyclic", False):
        run = wl.sh.PeerScanFromHost(wl.ctx, wl.peer, wl.k, wl.n_global, wl.block, torch.int32, np.int32(0))
        step = lambda: run(hin, hout)  # noqa: E731
        result = run.out
        note = "per rank: upload, scan and download overlap piece by piece (36 MiB pieces)"
    else:
        def step():
            wl.x.copy_(hin, non_blocking=True)
            wl.step()
            hout.copy_(wl.out, non_blocking=True)
            torch.cuda.synchronize()
        result = wl.out
    wl.step()  # the reference result, device-resident
    torch.cuda.synchronize()
    expect = wl.out.clone()
    step()
    reps = 3
    dist.barrier()
    t0 = time.perf_counter()
    for _ in range(reps):
        step()
    dt = torch.tensor([(time.perf_counter() - t0) / reps], device="cuda", dtype=torch.float64)
    dist.all_reduce(dt, op=dist.ReduceOp.MAX)
    valid = n + (1 if (not getattr(wl, "cyclic", False) or wl.rank == wl.owner) else 0)
    ok = bool(torch.equal(hout[:valid], expect[:valid].cpu())) and bool(torch.equal(result[:valid], expect[:valid])) and bool(wl.verify())
    okt = torch.tensor([int(ok)], device="cuda")
    dist.all_reduce(okt, op=dist.ReduceOp.MIN)
    return {"value": wl.bytes * world / float(dt[0]) / 1e9, "unit": "GB/s", "h2d_bytes_per_step": 4 * n * world,
            "d2h_bytes_per_step": 4 * (n + 1) * world, "ms_per_step": float(dt[0]) * 1e3, "steps": reps,
            "parity_check": bool(okt[0]), "note": note}


# -------------------------------------------------------------------- main
def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--workload", default="scan", choices=sorted(WORKLOADS) + sorted(SECONDARY) + sorted(CONFIG_EXTRAS))
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--functors", default="hand", choices=["hand", "lang"],
                    help="hand-written functor snippets (programs.py) or the ones the embedded language prints (examples.py)")
    ap.add_argument("--exchange", default="peer", choices=["peer", "nccl"],
                    help="several GPUs: the library's own exchange kernels over NVLink peer mappings, or NCCL collectives")
    ap.add_argument("--scan-distribution", default="block-cyclic", choices=["block-cyclic", "slabs"],
                    help="several GPUs: the vector dealt in 1 MiB blocks and scanned in one pass, or contiguous slabs "
                         "joined by a carry (one more read of every slab)")
    ap.add_argument("--size", type=int, default=None, help="override the problem size (profiling small cases)")
    ap.add_argument("--no-extras", action="store_true", help="skip the per-skeleton table, e2e and CPU baseline")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3) if args.impl == "b200" else args.warmup

    if args.impl == "reference":
        return run_reference(args)

    import torch
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device; there is no CPU fallback")
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dist = None
    if world > 1:
        import torch.distributed as dist
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    accb = importlib.import_module("accelerate-cuda_b200")
    ctx = accb.Context(local)
    peak, peak_kind = measured_peak()

    everything = {**WORKLOADS, **SECONDARY, **CONFIG_EXTRAS}
    if args.workload not in WORKLOADS and world > 1:
        raise SystemExit("the secondary workloads run on one GPU")
    Workload.functors = args.functors
    Workload.exchange = args.exchange
    ScanWorkload.distribution = args.scan_distribution
    wl = everything[args.workload](accb, ctx, torch, rank, world)
    wl.setup(args.size)
    if dist:
        dist.barrier()
    torch.cuda.synchronize()
    with ClockSampler(local) as clocks:
        ms, launches = time_steps(torch, wl, args.steps, args.warmup)
    if dist:
        tm = torch.tensor([ms], device="cuda", dtype=torch.float64)
        dist.all_reduce(tm, op=dist.ReduceOp.MAX)
        ms = float(tm[0])
        dist.barrier()
    ok = wl.verify()
    if dist:
        okt = torch.tensor([int(ok)], device="cuda")
        dist.all_reduce(okt, op=dist.ReduceOp.MIN)
        ok = bool(okt[0])
    ms_step = ms / args.steps
    total_bytes = wl.bytes * world
    value = total_bytes / (ms_step * 1e-3) / 1e9
    per_gpu = wl.bytes / (ms_step * 1e-3) / 1e9

    line = {
        "metric": METRIC, "value": value, "unit": "GB/s", "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": ms_step, "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": wl.dtype,
        "data": "synthetic",
        "config": {"workload": wl.name, "l2": "inputs larger than L2 (1 GiB read per step)", "parity_check": ok,
                   "elements_per_gpu": getattr(wl, "n", None), "seed": hex(wl.W.SEED), "functors": args.functors,
                   **({"exchange": Workload.exchange, "distribution": getattr(wl, "distribution", "contiguous slabs")}
                      if world > 1 else {})},
        "gpu_launches": launches,
        "clocks": clocks.summary(),
        "pct_of_spec_peak_8TBs": 100.0 * per_gpu / SPEC_PEAK_GBS,
    }
    # dominant kernel = the skeleton's kernel; its launches in a step move the algorithmic bytes of the step.
    # traffic: DRAM bytes per launch from one ncu capture of the same kernel on a smaller case (profiles/),
    # scaled by the number of units a full launch processes (traffic grows in proportion to them).
    dom = getattr(wl, 'dom_launches', getattr(wl, 'iters', 1))  # launches of the dominant kernel per step (the iterated stencil: 5)
    if args.workload in NCU_TRAFFIC:
        kernel_name, traffic_per_unit = NCU_TRAFFIC[args.workload]
        traffic = traffic_per_unit * wl.bytes / BYTES_PER_UNIT[args.workload] / dom
    else:  # secondary workloads: no scaled ncu figure
        kernel_name, traffic = SECONDARY_KERNEL.get(args.workload, args.workload), None
    line["roofline"] = {"bound": "hbm", "achieved": per_gpu, "peak": peak, "unit": "GB/s", "frac": per_gpu / peak,
                        "traffic": traffic, "peak_kind": peak_kind, "kernel": kernel_name,
                        "algorithmic_bytes_per_launch": wl.bytes / dom}

    def entry_of(w, ms1, ok1):
        g = w.bytes / (ms1 * 1e-3) / 1e9
        return {"GB/s": g, "frac_of_measured": g / peak, "ms": ms1, "parity_check": ok1, "workload": w.name}

    if world == 1 and not args.no_extras:
        # ---- e2e: run1 on pinned host arrays (upload + launch + download inside the timed region)
        line["e2e"] = e2e_single(torch, wl, args.steps) if hasattr(wl, "host_program") else None
        # ---- CPU baseline on a bounded sample, one core
        gbs, secs = cpu_scan_sample(1, 1 << 26, 3)
        line["cpu_baseline"] = {"value": gbs, "unit": "GB/s", "cores": 1, "kind": "port",
                                "sample": "sequential scanl (+) 0 over a 2^26-element Int32 slice, best of 3"}
        # ---- the reference's own algorithm for the same program on this GPU (baseline/refskel), then
        # ---- the other skeletons, each on its configuration
        def with_ref(entry, w):
            try:
                ra = ref_algorithm(torch, w, ctx.sm_count)
            except (OSError, RuntimeError) as e:  # baseline library not built
                ra = {"unavailable": str(e)}
            if ra and "GB/s" in ra:
                ra["speedup"] = entry["GB/s"] / ra["GB/s"]
            entry["ref_algorithm"] = ra
            return entry

        table = {args.workload: with_ref(entry_of(wl, ms_step, ok), wl)}
        table[args.workload]["e2e"] = line["e2e"]
        line["ref_algorithm"] = table[args.workload]["ref_algorithm"]
        del wl
        torch.cuda.empty_cache()
        for name, cls in everything.items():
            if name == args.workload:
                continue
            w2 = cls(accb, ctx, torch, 0, 1)
            w2.setup(None)
            ms2, _, ok2 = measure(torch, None, w2, 10, 3)
            table[name] = with_ref(entry_of(w2, ms2, ok2), w2)
            if name in WORKLOADS:  # end to end from pinned host arrays, like the headline's e2e
                table[name]["e2e"] = e2e_single(torch, w2, 3)
            del w2
            torch.cuda.empty_cache()
        line["skeletons"] = {k: v for k, v in table.items() if k in WORKLOADS or k in CONFIG_EXTRAS}  # the BASELINE configurations
        line["secondary"] = {k: v for k, v in table.items() if k in SECONDARY}                       # other shapes and types
        # ---- the same programs written in the embedded language: the kernels it prints against the hand-written ones
        if args.functors == "hand":
            Workload.functors = "lang"
            gen = {}
            for name, cls in WORKLOADS.items():
                w3 = cls(accb, ctx, torch, 0, 1)
                w3.setup(None)
                ms3, _, ok3 = measure(torch, None, w3, 10, 3)
                g = w3.bytes / (ms3 * 1e-3) / 1e9
                gen[name] = {"GB/s": g, "frac_of_measured": g / peak, "vs_hand_written": g / table[name]["GB/s"],
                             "parity_check": ok3}
                del w3
                torch.cuda.empty_cache()
            Workload.functors = "hand"
            line["generated_functors"] = gen
        if not os.environ.get("ACCB_BENCH_SKIP_AWHILE"):  # set for profiler runs: the loop is a graph with a WHILE node
            line["awhile"] = awhile_sample(accb, ctx, torch)
    elif world > 1 and not args.no_extras:
        # ---- e2e of the timed workload at N GPUs
        line["e2e"] = e2e_sharded(torch, dist, wl, world) if isinstance(wl, ScanWorkload) else None
        # ---- every skeleton through its sharded path: aggregate GB/s, parity, and efficiency against the SAME
        # ---- program run unsharded on every GPU at once in this run (no exchange: what N independent GPUs give)
        table = {args.workload: entry_of(wl, ms_step, ok)}
        release(torch, dist, wl)
        del wl
        torch.cuda.empty_cache()
        for name, cls in WORKLOADS.items():
            if name != args.workload:
                w2 = cls(accb, ctx, torch, rank, world)
                w2.setup(None)
                ms2, _, ok2 = measure(torch, dist, w2, 10, 3)
                table[name] = entry_of(w2, ms2, ok2)
                release(torch, dist, w2)
                del w2
                torch.cuda.empty_cache()
            w1 = cls(accb, ctx, torch, 0, 1)  # unsharded, on every rank at the same time
            w1.setup(None)
            ms1, _, ok1 = measure(torch, dist, w1, 10, 3)
            del w1
            torch.cuda.empty_cache()
            e = table[name]
            e["GB/s_per_gpu"] = e["GB/s"]
            e["GB/s"] = e["GB/s_per_gpu"] * world
            e["unsharded_ms"] = ms1
            e["efficiency"] = ms1 / e["ms"]
            e["parity_check"] = e["parity_check"] and ok1
        # ---- the scan over contiguous slabs joined by a carry, for comparison: one more read of every slab
        if ScanWorkload.distribution == "block-cyclic" and "scan" in table:
            ScanWorkload.distribution = "slabs"
            w2 = ScanWorkload(accb, ctx, torch, rank, world)
            w2.setup(None)
            ms2, _, ok2 = measure(torch, dist, w2, 10, 3)
            e = entry_of(w2, ms2, ok2)
            e.update({"GB/s_per_gpu": e["GB/s"], "GB/s": e["GB/s"] * world, "unsharded_ms": table["scan"]["unsharded_ms"],
                      "efficiency": table["scan"]["unsharded_ms"] / ms2, "distribution": "contiguous slabs"})
            table["scan_slabs"] = e
            release(torch, dist, w2)
            del w2
            torch.cuda.empty_cache()
            ScanWorkload.distribution = "block-cyclic"
            # ---- strong scaling: ONE vector of 2^28 elements dealt over all GPUs (the headline's own size), against
            # ---- one GPU scanning all of it in this run
            w2 = ScanWorkload(accb, ctx, torch, rank, world)
            w2.setup(w2.W.N28 // world)
            if w2.cyclic:
                ms2, _, ok2 = measure(torch, dist, w2, 10, 3)
                one = table["scan"]["unsharded_ms"]
                g = w2.bytes * world / (ms2 * 1e-3) / 1e9
                table["scan_strong"] = {"GB/s": g, "ms": ms2, "parity_check": ok2, "elements_total": w2.n_global,
                                        "one_gpu_ms": one, "speedup": one / ms2, "efficiency": one / ms2 / world,
                                        "workload": "scanl (+) 0, Int32, 2^28 elements over all GPUs"}
            release(torch, dist, w2)
            del w2
            torch.cuda.empty_cache()
        line["skeletons"] = table
    elif rank == 0:
        line["e2e"] = None
    ctx.sync()
    if rank == 0:
        print(json.dumps(line), flush=True)
    if dist:
        try:
            release(torch, dist, wl)
        except NameError:
            dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
