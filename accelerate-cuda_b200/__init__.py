"""accelerate-b200: host-side mirror of ``Data.Array.Accelerate.CUDA`` over libaccb200.so.

The reference exposes ``run``, ``run1``, ``runWith``, ``run1With``, ``stream``,
``runAsync`` ..., ``create`` / ``destroy``, ``unsafeFree`` and ``performGC``
(``Data/Array/Accelerate/CUDA.hs:184-200,232-353,421-441``).  Its host language
(Haskell) has no toolchain on this machine, so the same surface is offered here
in Python on top of the C ABI of ``include/accb200.h``; everything below the
ABI (memory table, kernel cache, launch logic, kernels) is native code.

Two levels:

* **programs** -- ``run1(f, *input_types)`` traces ``f`` over symbolic arrays
  into an op list (the role of ``convertAfunWith`` + ``compileAfun``,
  ``CUDA.hs:326-329``) and returns a callable from host arrays to host
  arrays: upload, launch, download, exactly what ``run1`` does
  (``CUDA.hs:307-330,382-389``).
* **launches** -- ``Context.map`` / ``fold_all`` / ``fold_dim`` / ``fold_seg`` /
  ``scan`` / ``permute`` / ``stencil`` / ``stencil2`` on device arrays: the
  per-skeleton drivers of ``CUDA/Execute.hs:264-450``.

The module never falls back to a CPU implementation: without the compiled
library or without a GPU every call raises.
"""
from __future__ import annotations

import ctypes as C
import os
from typing import Callable, Sequence

import numpy as np

from .programs import KernelSpec  # noqa: F401  (re-export)
from . import programs  # noqa: F401

_HERE = os.path.dirname(os.path.abspath(__file__))
LIBRARY_PATH = os.path.join(_HERE, "libaccb200.so")

OK, EINVAL, ECUDA, ENOMEM, ECOMPILE, EIO, EBOUNDS, ETIMEOUT, ENOTFOUND, ENODRIVER = range(10)
_STATUS = ["OK", "EINVAL", "ECUDA", "ENOMEM", "ECOMPILE", "EIO", "EBOUNDS", "ETIMEOUT", "ENOTFOUND", "ENODRIVER"]

SCAN_LEFT, SCAN_RIGHT = 0, 1
SCAN_EXCLUSIVE, SCAN_INCLUSIVE, SCAN_PRIME, SCAN_INCLUSIVE_SEEDED = 0, 1, 2, 3
SEED_ON_DEVICE = 0x100
CLAMP, MIRROR, WRAP, CONSTANT = 0, 1, 2, 3
BOUNDARY = {"clamp": CLAMP, "mirror": MIRROR, "wrap": WRAP, "constant": CONSTANT}

MAX_RANK, MAX_COMP = 4, 8


class AccbError(RuntimeError):
    def __init__(self, status: int, message: str):
        super().__init__(f"[{_STATUS[status] if 0 <= status < len(_STATUS) else status}] {message}")
        self.status = status


class accb_array(C.Structure):
    _fields_ = [("rank", C.c_int), ("shape", C.c_int * MAX_RANK), ("ncomp", C.c_int),
                ("ptr", C.c_void_p * MAX_COMP)]


class accb_value_type(C.Structure):
    _fields_ = [("rank", C.c_int), ("ncomp", C.c_int), ("comp_bytes", C.c_int * MAX_COMP)]


class InputArray(C.Structure):
    _fields_ = [("shape", C.POINTER(C.c_int)), ("adata", C.POINTER(C.c_void_p))]


class OutputArray(C.Structure):
    _fields_ = [("shape", C.POINTER(C.c_int)), ("adata", C.POINTER(C.c_void_p)), ("stable_ptr", C.c_void_p)]


_lib = None


def lib() -> C.CDLL:
    """The C-ABI library.  Raises if it has not been built (no fallback)."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIBRARY_PATH):
            raise AccbError(ENOTFOUND, f"{LIBRARY_PATH} is missing: run `python accelerate-cuda_b200/build.py`")
        L = C.CDLL(LIBRARY_PATH)
        vp, ll, i32, u64, sz = C.c_void_p, C.c_longlong, C.c_int, C.c_uint64, C.c_size_t
        arrp = C.POINTER(accb_array)
        sigs = {
            "accb_init": [],
            "accb_device_count": [C.POINTER(i32)],
            "accb_context_create": [i32, vp, C.POINTER(vp)],
            "accb_context_destroy": [vp],
            "accb_context_sync": [vp],
            "accb_device_info": [vp, C.POINTER(i32), C.POINTER(sz), C.POINTER(i32), C.POINTER(i32)],
            "accb_stream_acquire": [vp, C.POINTER(vp)],
            "accb_stream_release": [vp, vp],
            "accb_stream_sync": [vp, vp],
            "accb_event_record": [vp, vp, C.POINTER(vp)],
            "accb_stream_wait_event": [vp, vp, vp],
            "accb_event_sync": [vp, vp],
            "accb_event_query": [vp, vp, C.POINTER(i32)],
            "accb_event_release": [vp, vp],
            "accb_malloc": [vp, u64, sz, C.POINTER(vp)],
            "accb_use": [vp, u64, vp, sz, vp, C.POINTER(vp)],
            "accb_insert_unmanaged": [vp, u64, vp, sz],
            "accb_with_ptr": [vp, u64, C.POINTER(vp), C.POINTER(sz)],
            "accb_release": [vp, u64],
            "accb_release_after": [vp, u64, vp],
            "accb_peek": [vp, u64, sz, vp, sz, vp],
            "accb_poke": [vp, u64, sz, vp, sz, vp],
            "accb_copy": [vp, u64, u64, sz, vp],
            "accb_copy_peer": [vp, u64, vp, u64, sz, vp],
            "accb_index": [vp, u64, sz, sz, vp],
            "accb_free": [vp, u64],
            "accb_reclaim": [vp],
            "accb_memory_stats": [vp, C.POINTER(sz), C.POINTER(sz), C.POINTER(sz)],
            "accb_kernel_get": [vp, C.c_char_p, C.c_char_p, C.c_char_p, C.c_char_p, C.POINTER(vp)],
            "accb_kernel_wait": [vp, vp],
            "accb_kernel_info": [vp, vp, C.c_char_p] + [C.POINTER(i32)] * 4,
            "accb_kernel_release": [vp, vp],
            "accb_kernel_precompile": [C.c_char_p] * 5 + [C.c_char_p, sz],
            "accb_cache_flush": [vp],
            "accb_cache_stats": [vp, C.POINTER(sz), C.POINTER(sz), C.POINTER(sz)],
            "accb_launch_config": [vp, vp, C.c_char_p, ll, C.POINTER(i32), C.POINTER(i32), C.POINTER(i32)],
            "accb_launch_count": [vp, C.POINTER(C.c_ulonglong)],
            "accb_map": [vp, vp, vp, arrp, i32, vp, sz, arrp],
            "accb_map_transposed": [vp, vp, vp, arrp, i32, vp, sz, arrp],
            "accb_fold_all": [vp, vp, vp, arrp, i32, ll, vp, sz, arrp],
            "accb_fold_dim": [vp, vp, vp, arrp, i32, ll, ll, vp, sz, arrp],
            "accb_fold_seg": [vp, vp, vp, arrp, i32, ll, ll, vp, ll, vp, sz, arrp],
            "accb_scan": [vp, vp, vp, arrp, i32, ll, i32, i32, vp, sz, arrp, arrp],
            "accb_permute_defaults": [vp, vp, arrp, arrp, C.POINTER(i32)],
            "accb_permute": [vp, vp, vp, arrp, i32, ll, vp, sz, arrp],
            "accb_stencil": [vp, vp, vp, arrp, i32, vp, sz, arrp],
            "accb_stencil2": [vp, vp, vp, arrp, arrp, i32, vp, sz, arrp],
            "accb_stencil_iterate": [vp, vp, vp, arrp, arrp, i32, i32, vp, sz, C.POINTER(i32)],
            "accb_stencil_iterate_from": [vp, vp, vp, arrp, arrp, arrp, i32, i32, vp, sz, C.POINTER(i32)],
            "accb_program_create": [vp, i32, C.POINTER(accb_value_type), C.POINTER(vp)],
            "accb_program_map": [vp, vp, C.POINTER(i32), i32, i32, C.POINTER(accb_value_type), vp, sz],
            "accb_program_fold": [vp, vp, C.POINTER(i32), i32, i32, i32, vp, sz, C.POINTER(accb_value_type)],
            "accb_program_scan": [vp, vp, C.POINTER(i32), i32, i32, i32, i32, vp, sz, C.POINTER(accb_value_type)],
            "accb_program_permute": [vp, vp, C.POINTER(i32), i32, i32, i32, C.POINTER(accb_value_type)],
            "accb_program_stencil": [vp, vp, i32, i32, vp, sz, i32, C.POINTER(accb_value_type)],
            "accb_program_map_transposed": [vp, vp, C.POINTER(i32), i32, i32, C.POINTER(accb_value_type), vp, sz],
            "accb_program_generate": [vp, vp, C.POINTER(i32), i32, i32, C.POINTER(i32), C.POINTER(accb_value_type), vp, sz],
            "accb_program_generate_dims": [vp, vp, C.POINTER(i32), i32, i32, C.POINTER(i32), C.POINTER(i32), C.POINTER(i32),
                                           C.POINTER(accb_value_type), vp, sz],
            "accb_program_generate_dims2": [vp, vp, C.POINTER(i32), i32, i32] + [C.POINTER(i32)] * 5 +
                                           [C.POINTER(accb_value_type), vp, sz],
            "accb_program_fold_seg": [vp, vp, C.POINTER(i32), i32, i32, i32, vp, sz, C.POINTER(accb_value_type)],
            "accb_program_stencil2": [vp, vp, i32, i32, i32, vp, sz, C.POINTER(accb_value_type)],
            "accb_program_outputs": [vp, C.POINTER(i32), i32],
            "accb_program_run": [vp, vp, arrp, arrp],
            "accb_program_run_graph": [vp, vp, arrp, arrp],
            "accb_program_run_host": [vp, arrp, arrp],
            "accb_program_stream_chunk": [vp, ll],
            "accb_program_destroy": [vp],
            "accb_awhile": [vp, vp, vp, arrp, i32, ll, C.POINTER(ll)],
            "accb_group_create": [C.POINTER(i32), i32, C.POINTER(vp)],
            "accb_group_destroy": [vp],
            "accb_group_size": [vp, C.POINTER(i32)],
            "accb_group_context": [vp, i32, C.POINTER(vp)],
            "accb_group_stream": [vp, i32, C.POINTER(vp)],
            "accb_group_sync": [vp],
            "accb_group_map": [vp, vp, arrp, i32, vp, sz, arrp],
            "accb_group_fold_dim": [vp, vp, arrp, i32, C.POINTER(ll), ll, vp, sz, arrp],
            "accb_group_fold_all": [vp, vp, vp, arrp, i32, C.POINTER(ll), vp, sz, C.POINTER(i32), arrp],
            "accb_group_scan": [vp, vp, vp, vp, arrp, i32, C.POINTER(ll), i32, i32, vp, sz, sz, arrp, arrp],
            "accb_group_permute": [vp, vp, vp, arrp, i32, C.POINTER(ll), vp, sz, C.POINTER(i32), arrp, i32],
            "accb_group_stencil_layout": [vp, i32, i32, i32, i32, C.POINTER(i32), C.POINTER(i32)],
            "accb_group_stencil2": [vp, vp, arrp, arrp, arrp, C.POINTER(i32), i32, i32, vp, sz, C.POINTER(i32)],
            "accb_seg_partition": [C.POINTER(i32), ll, i32, C.POINTER(ll)],
            "accb_group_fold_seg": [vp, vp, arrp, i32, C.POINTER(ll), C.POINTER(vp), C.POINTER(ll), vp, sz, arrp],
            "accb_group_stencil_iterate": [vp, vp, arrp, arrp, C.POINTER(i32), i32, i32, i32, vp, sz,
                                           C.POINTER(i32), C.POINTER(i32)],
            "accb_peer_create": [vp, i32, i32, sz, C.POINTER(vp)],
            "accb_peer_handle": [vp, vp],
            "accb_peer_connect": [vp, vp],
            "accb_peer_loopback": [vp],
            "accb_peer_data": [vp, C.POINTER(vp), C.POINTER(sz)],
            "accb_peer_barrier": [vp, vp],
            "accb_peer_gather": [vp, vp, sz, sz, vp],
            "accb_peer_allreduce": [vp, vp, sz, ll, i32, i32, vp],
            "accb_peer_exscan": [vp, vp, sz, ll, i32, i32, vp, vp],
            "accb_peer_pull": [vp, vp, i32, sz, sz, vp],
            "accb_peer_scan_tile": [vp, vp, C.POINTER(ll)],
            "accb_peer_scan_layout": [i32, i32, ll, ll, C.POINTER(ll), C.POINTER(i32), C.POINTER(sz)],
            "accb_peer_scan": [vp, vp, vp, arrp, i32, ll, ll, i32, vp, sz, sz, arrp, arrp],
            "accb_peer_scan_piece": [vp, vp, vp, arrp, i32, ll, ll, i32, vp, sz, sz, arrp, arrp, ll, ll],
            "accb_peer_status": [vp, vp, C.POINTER(i32)],
            "accb_peer_destroy": [vp],
            "accb_gen_uniform_f32": [vp, vp, vp, ll, ll, u64, u64, C.c_float, C.c_float],
            "accb_gen_uniform_i32": [vp, vp, vp, ll, ll, u64, u64, i32],
            "accb_gen_zipf_mix_i32": [vp, vp, vp, ll, ll, u64, vp, i32],
            "accb_flush_l2": [vp, vp],
            "accelerateDestroy": [vp],
            "runProgram": [vp, vp, C.POINTER(InputArray), C.POINTER(OutputArray)],
            "freeOutput": [C.POINTER(OutputArray)],
            "freeProgram": [vp],
            "accelerateStatus": [vp],
        }
        for name, args in sigs.items():
            fn = getattr(L, name)
            fn.argtypes = args
            fn.restype = C.c_int
        for name in ("accelerateDestroy", "runProgram", "freeOutput", "freeProgram"):
            getattr(L, name).restype = None
        L.accb_last_error.argtypes = [vp]
        L.accb_last_error.restype = C.c_char_p
        L.accb_group_last_error.argtypes = [vp]
        L.accb_group_last_error.restype = C.c_char_p
        L.accb_version.restype = C.c_char_p
        L.accelerateCreate.argtypes = [C.c_int32, vp]
        L.accelerateCreate.restype = vp
        L.accelerateContext.argtypes = [vp]
        L.accelerateContext.restype = vp
        _lib = L
    return _lib


def _check(status: int, ctx=None):
    if status != OK:
        msg = lib().accb_last_error(ctx)
        raise AccbError(status, msg.decode(errors="replace") if msg else "")


# --------------------------------------------------------------- marshalling
def _components(x):
    """A device array is a tensor-like (``data_ptr()``, ``shape``) or a tuple of
    them for an array of tuples (structure of arrays)."""
    return list(x) if isinstance(x, (tuple, list)) else [x]


def _ptr(t) -> int:
    if hasattr(t, "data_ptr"):
        return int(t.data_ptr())
    if isinstance(t, DeviceArray):
        return t.ptr
    raise TypeError(f"not a device array: {type(t)!r}")


def to_accb_array(x, shape=None) -> accb_array:
    comps = _components(x)
    a = accb_array()
    shp = tuple(shape if shape is not None else comps[0].shape)
    if len(shp) > MAX_RANK or len(comps) > MAX_COMP:
        raise AccbError(EINVAL, "rank or component count too large")
    a.rank = len(shp)
    for d, e in enumerate(reversed(shp)):  # innermost extent first
        a.shape[d] = int(e)
    a.ncomp = len(comps)
    for c, t in enumerate(comps):
        if hasattr(t, "is_contiguous") and not t.is_contiguous():
            raise AccbError(EINVAL, "device arrays must be contiguous")
        a.ptr[c] = _ptr(t)
    return a


def _arr_list(xs):
    arr = (accb_array * max(1, len(xs)))()
    for i, x in enumerate(xs):
        arr[i] = to_accb_array(x)
    return arr


def _bytes_of(value, dtype=None):
    """Pack a seed / scalar (numpy scalar, or tuple of them) into bytes."""
    if value is None:
        return None, 0
    if isinstance(value, (bytes, bytearray)):
        b = bytes(value)
    elif isinstance(value, (tuple, list)):
        b = b"".join(np.asarray(v).tobytes() for v in value)
    else:
        b = (np.asarray(value, dtype=dtype) if dtype is not None else np.asarray(value)).tobytes()
    return C.create_string_buffer(b, len(b)), len(b)


class DeviceArray:
    """A raw device allocation (for callers without torch)."""

    def __init__(self, ptr: int, shape, dtype):
        self.ptr, self.shape, self.dtype = int(ptr), tuple(shape), np.dtype(dtype)

    def element_size(self) -> int:
        return self.dtype.itemsize

    @property
    def __cuda_array_interface__(self):
        """Lets ``torch.as_tensor(device_array, device="cuda")`` (or cupy) view the memory without a copy."""
        return {"shape": self.shape, "typestr": self.dtype.str, "data": (self.ptr, False), "version": 3, "strides": None}


PEER_TYPES = {np.dtype(np.int32): 0, np.dtype(np.uint32): 1, np.dtype(np.int64): 2, np.dtype(np.float32): 3,
              np.dtype(np.float64): 4}
PEER_OPS = {"add": 0, "min": 1, "max": 2, "and": 3, "or": 4, "xor": 5}


class Peer:
    """This rank's exchange buffer and its mappings of the other ranks' buffers (``accb_peer_*``): exchanges
    between processes, one per GPU, done by the library's own kernels over NVLink.  ``all_gather_bytes(b)`` is the
    host's way to hand every rank's 64-byte handle to every rank, e.g. built on ``torch.distributed``."""

    def __init__(self, ctx: "Context", rank: int, world: int, nbytes: int, all_gather_bytes: Callable):
        self.ctx, self.rank, self.world = ctx, rank, world
        h = C.c_void_p()
        _check(lib().accb_peer_create(ctx.handle, rank, world, nbytes, C.byref(h)), ctx.handle)
        self.handle = h
        if all_gather_bytes is None:  # tests of the time limit: the other ranks never arrive
            self._check(lib().accb_peer_loopback(h))
        else:
            mine = C.create_string_buffer(64)
            self._check(lib().accb_peer_handle(h, mine))
            handles = all_gather_bytes(mine.raw)  # list of `world` bytes objects, in rank order
            blob = C.create_string_buffer(b"".join(handles), 64 * world)
            self._check(lib().accb_peer_connect(h, blob))
        p, n = C.c_void_p(), C.c_size_t()
        self._check(lib().accb_peer_data(h, C.byref(p), C.byref(n)))
        self.data_ptr, self.nbytes = p.value, n.value

    def _check(self, status: int):
        _check(status, self.ctx.handle)

    def array(self, offset: int, shape, dtype) -> "DeviceArray":
        """A region of this rank's own buffer as a device array that skeleton launches can write."""
        return DeviceArray(self.data_ptr + offset, shape, dtype)

    def barrier(self, stream=None):
        self._check(lib().accb_peer_barrier(self.handle, Context._stream(stream)))

    def gather(self, offset: int, nbytes: int, dst, stream=None):
        self._check(lib().accb_peer_gather(self.handle, Context._stream(stream), offset, nbytes, C.c_void_p(_ptr(dst))))

    def allreduce(self, offset: int, count: int, dtype, op: str, dst, stream=None):
        self._check(lib().accb_peer_allreduce(self.handle, Context._stream(stream), offset, count,
                                              PEER_TYPES[np.dtype(dtype)], PEER_OPS[op], C.c_void_p(_ptr(dst))))

    def exscan(self, offset: int, count: int, dtype, op: str, first, dst, stream=None):
        """dst = first (op) the data of every LOWER rank, in rank order: the carry of a sharded scan."""
        self._check(lib().accb_peer_exscan(self.handle, Context._stream(stream), offset, count,
                                           PEER_TYPES[np.dtype(dtype)], PEER_OPS[op], C.c_void_p(_ptr(first)),
                                           C.c_void_p(_ptr(dst))))

    def pull(self, from_rank: int, offset: int, nbytes: int, dst_ptr: int, stream=None):
        self._check(lib().accb_peer_pull(self.handle, Context._stream(stream), from_rank, offset, nbytes,
                                         C.c_void_p(int(dst_ptr))))

    def scan(self, kernel, env: Sequence, n_global: int, out, kind=SCAN_EXCLUSIVE, seed=None, total=None,
             block_elems: int = 0, scratch_offset: int = 0, stream=None, first_block: int = 0, blocks: int = -1):
        """scanl / scanl1 / scanl' over one vector dealt to the ranks in blocks (``accb_peer_scan``): ``env`` and
        ``out`` are this rank's blocks, one after the other (``scan_layout`` gives their length).  ``first_block`` /
        ``blocks`` launch only a piece of it (``accb_peer_scan_piece``): pieces follow one another on one stream."""
        sb, sn = _bytes_of(seed)
        o = to_accb_array(out)
        t = to_accb_array(total, shape=()) if total is not None else None
        self._check(lib().accb_peer_scan_piece(self.handle, self.ctx._k(kernel), Context._stream(stream), _arr_list(env),
                                               len(env), n_global, block_elems, kind, sb, sn, scratch_offset, C.byref(o),
                                               C.byref(t) if t is not None else None, first_block, blocks))

    def status(self, stream=None):
        """Waits for the stream; raises ETIMEOUT if a rank did not reach some exchange in time."""
        t = C.c_int()
        self._check(lib().accb_peer_status(self.handle, Context._stream(stream), C.byref(t)))

    def destroy(self):
        if self.handle:
            lib().accb_peer_destroy(self.handle)
            self.handle = None


def seg_partition(offsets, parts: int):
    """Cuts between segments so that ``parts`` runs of whole segments hold about the same number of elements
    (``accb_seg_partition``): returns parts + 1 segment numbers."""
    offs = np.ascontiguousarray(offsets, np.int32)
    first = (C.c_longlong * (parts + 1))()
    _check(lib().accb_seg_partition(offs.ctypes.data_as(C.POINTER(C.c_int)), offs.size - 1, parts, first))
    return list(first)


def scan_layout(world: int, rank: int, n_global: int, block_elems: int):
    """(elements this rank holds, rank that owns the last block and with it the total, bytes of exchange-buffer
    scratch) of a block-cyclic scan (``accb_peer_scan_layout``)."""
    n, owner, scratch = C.c_longlong(), C.c_int(), C.c_size_t()
    _check(lib().accb_peer_scan_layout(world, rank, n_global, block_elems, C.byref(n), C.byref(owner), C.byref(scratch)))
    return n.value, owner.value, scratch.value


class Kernel:
    def __init__(self, ctx: "Context", spec: KernelSpec, handle):
        self.ctx, self.spec, self.handle = ctx, spec, handle

    def wait(self):
        _check(lib().accb_kernel_wait(self.ctx.handle, self.handle), self.ctx.handle)
        return self

    def info(self, entry: str):
        r, s, b, o = C.c_int(), C.c_int(), C.c_int(), C.c_int()
        _check(lib().accb_kernel_info(self.ctx.handle, self.handle, entry.encode(), C.byref(r), C.byref(s),
                                      C.byref(b), C.byref(o)), self.ctx.handle)
        return {"regs": r.value, "static_smem": s.value, "block": b.value, "blocks_per_sm": o.value}


class Context:
    """One execution context per GPU (``Context.create``, CUDA/Context.hs:55-71)."""

    def __init__(self, device: int = 0, cu_context=None):
        h = C.c_void_p()
        _check(lib().accb_context_create(device, cu_context, C.byref(h)))
        self.handle = h
        self.device = device
        self._kernels = {}
        sm, mem, maj, mnr = C.c_int(), C.c_size_t(), C.c_int(), C.c_int()
        _check(lib().accb_device_info(h, C.byref(sm), C.byref(mem), C.byref(maj), C.byref(mnr)), h)
        self.sm_count, self.total_mem, self.cc = sm.value, mem.value, (maj.value, mnr.value)

    # -- lifetime
    def destroy(self):
        if self.handle:
            lib().accb_context_destroy(self.handle)
            self.handle = None

    def sync(self):
        _check(lib().accb_context_sync(self.handle), self.handle)

    @staticmethod
    def _stream(stream):
        if stream is not None:
            return C.c_void_p(int(stream))
        try:
            import torch
            return C.c_void_p(int(torch.cuda.current_stream().cuda_stream))
        except Exception:
            return C.c_void_p(0)

    # -- kernel cache
    def kernel(self, spec: KernelSpec) -> Kernel:
        k = self._kernels.get(spec)
        if k is None:
            h = C.c_void_p()
            _check(lib().accb_kernel_get(self.handle, spec.skeleton.encode(), spec.source.encode(),
                                         spec.functor.encode(), spec.flags.encode() if spec.flags else None,
                                         C.byref(h)), self.handle)
            k = self._kernels[spec] = Kernel(self, spec, h)
        return k

    def scan_tile(self, kernel) -> int:
        """Elements of one tile of the kernel's block-cyclic scan entries (``accb_peer_scan_tile``)."""
        n = C.c_longlong()
        _check(lib().accb_peer_scan_tile(self.handle, self._k(kernel), C.byref(n)), self.handle)
        return n.value

    def cache_stats(self):
        a, b, c = C.c_size_t(), C.c_size_t(), C.c_size_t()
        _check(lib().accb_cache_stats(self.handle, C.byref(a), C.byref(b), C.byref(c)), self.handle)
        return {"memory_hits": a.value, "disk_hits": b.value, "compiles": c.value}

    def launch_count(self) -> int:
        n = C.c_ulonglong()
        _check(lib().accb_launch_count(self.handle, C.byref(n)), self.handle)
        return n.value

    def _k(self, k):
        return (k if isinstance(k, Kernel) else self.kernel(k)).handle

    # -- skeleton launches on device arrays
    def map(self, kernel, env: Sequence, out, scalars=None, stream=None):
        sb, sn = _bytes_of(scalars)
        o = to_accb_array(out)
        _check(lib().accb_map(self.handle, self._k(kernel), self._stream(stream), _arr_list(env), len(env), sb, sn,
                              C.byref(o)), self.handle)

    def map_transposed(self, kernel, env: Sequence, out, scalars=None, stream=None):
        """``map f (transpose m)``: the element-wise inputs have the transposed shape of ``out``."""
        sb, sn = _bytes_of(scalars)
        o = to_accb_array(out)
        _check(lib().accb_map_transposed(self.handle, self._k(kernel), self._stream(stream), _arr_list(env), len(env),
                                         sb, sn, C.byref(o)), self.handle)

    def fold_all(self, kernel, env: Sequence, n: int, out, seed=None, stream=None):
        sb, sn = _bytes_of(seed)
        o = to_accb_array(out, shape=())
        _check(lib().accb_fold_all(self.handle, self._k(kernel), self._stream(stream), _arr_list(env), len(env), n,
                                   sb, sn, C.byref(o)), self.handle)

    def fold_dim(self, kernel, env: Sequence, rows: int, cols: int, out, seed=None, stream=None):
        sb, sn = _bytes_of(seed)
        o = to_accb_array(out)
        _check(lib().accb_fold_dim(self.handle, self._k(kernel), self._stream(stream), _arr_list(env), len(env),
                                   rows, cols, sb, sn, C.byref(o)), self.handle)

    def fold_seg(self, kernel, env: Sequence, rows: int, cols: int, offsets, nseg: int, out, seed=None, stream=None):
        sb, sn = _bytes_of(seed)
        o = to_accb_array(out)
        _check(lib().accb_fold_seg(self.handle, self._k(kernel), self._stream(stream), _arr_list(env), len(env),
                                   rows, cols, C.c_void_p(_ptr(offsets)), nseg, sb, sn, C.byref(o)), self.handle)

    def scan(self, kernel, env: Sequence, n: int, out, direction=SCAN_LEFT, kind=SCAN_EXCLUSIVE, seed=None,
             total=None, stream=None):
        if hasattr(seed, "data_ptr"):  # a device scalar: the carry of a sharded scan
            sb, sn, kind = C.c_void_p(int(seed.data_ptr())), seed.element_size(), kind | SEED_ON_DEVICE
        else:
            sb, sn = _bytes_of(seed)
        o = to_accb_array(out)
        t = to_accb_array(total, shape=()) if total is not None else None
        _check(lib().accb_scan(self.handle, self._k(kernel), self._stream(stream), _arr_list(env), len(env), n,
                               direction, kind, sb, sn, C.byref(o), C.byref(t) if t is not None else None),
               self.handle)

    def permute(self, kernel, env: Sequence, n_src: int, out, defaults=None, comp_bytes=None, scalars=None,
                stream=None):
        o = to_accb_array(out)
        s = self._stream(stream)
        if defaults is not None:
            d = to_accb_array(defaults)
            cb = comp_bytes or [c.element_size() for c in _components(out)]
            _check(lib().accb_permute_defaults(self.handle, s, C.byref(d), C.byref(o), (C.c_int * len(cb))(*cb)),
                   self.handle)
        sb, sn = _bytes_of(scalars)
        _check(lib().accb_permute(self.handle, self._k(kernel), s, _arr_list(env), len(env), n_src, sb, sn,
                                  C.byref(o)), self.handle)

    def stencil(self, kernel, src, out, boundary="clamp", constant=None, stream=None):
        cb, cn = _bytes_of(constant)
        a, o = to_accb_array(src), to_accb_array(out)
        _check(lib().accb_stencil(self.handle, self._k(kernel), self._stream(stream), C.byref(a),
                                  BOUNDARY[boundary], cb, cn, C.byref(o)), self.handle)

    def stencil2(self, kernel, src1, src2, out, boundary="clamp", constant=None, stream=None):
        cb, cn = _bytes_of(constant)
        a, b, o = to_accb_array(src1), to_accb_array(src2), to_accb_array(out)
        _check(lib().accb_stencil2(self.handle, self._k(kernel), self._stream(stream), C.byref(a), C.byref(b),
                                   BOUNDARY[boundary], cb, cn, C.byref(o)), self.handle)

    def stencil_iterate(self, kernel, a, b, iters: int, boundary="clamp", constant=None, stream=None, src=None):
        """``iters`` applications ping-ponging between ``a`` and ``b`` (starting from ``src``, which is only read, if
        one is given); returns the array holding the result."""
        cb, cn = _bytes_of(constant)
        aa, bb = to_accb_array(a), to_accb_array(b)
        ss = to_accb_array(src) if src is not None else None
        in_b = C.c_int()
        _check(lib().accb_stencil_iterate_from(self.handle, self._k(kernel), self._stream(stream),
                                               C.byref(ss) if ss is not None else None, C.byref(aa), C.byref(bb), iters,
                                               BOUNDARY[boundary], cb, cn, C.byref(in_b)), self.handle)
        return b if in_b.value else a

    # -- synthetic inputs
    def gen_uniform_f32(self, dst, n, first, seed, stream_id, lo, hi, stream=None):
        _check(lib().accb_gen_uniform_f32(self.handle, self._stream(stream), C.c_void_p(_ptr(dst)), n, first, seed,
                                          stream_id, lo, hi), self.handle)

    def gen_uniform_i32(self, dst, n, first, seed, stream_id, m, stream=None):
        _check(lib().accb_gen_uniform_i32(self.handle, self._stream(stream), C.c_void_p(_ptr(dst)), n, first, seed,
                                          stream_id, m), self.handle)

    def gen_zipf_mix_i32(self, dst, n, first, seed, cdf, nbins, stream=None):
        _check(lib().accb_gen_zipf_mix_i32(self.handle, self._stream(stream), C.c_void_p(_ptr(dst)), n, first, seed,
                                           C.c_void_p(_ptr(cdf)), nbins), self.handle)

    def flush_l2(self, stream=None):
        _check(lib().accb_flush_l2(self.handle, self._stream(stream)), self.handle)


class Group:
    """Several GPUs driven from one process (``accb_group_*``): rank r owns the r-th contiguous slab of every
    array.  Per-rank arguments are lists with one entry per rank.  The reference has no multi-device execution
    (its peer copy, CUDA/Array/Prim.hs:306-335, is never called)."""

    def __init__(self, devices: Sequence[int]):
        h = C.c_void_p()
        devs = (C.c_int * len(devices))(*devices)
        st = lib().accb_group_create(devs, len(devices), C.byref(h))
        if st != OK:
            _check(st)
        self.handle, self.devices, self.size = h, list(devices), len(devices)
        self.contexts, self.streams = [], []
        for r in range(self.size):
            c, s = C.c_void_p(), C.c_void_p()
            self._check(lib().accb_group_context(h, r, C.byref(c)))
            self._check(lib().accb_group_stream(h, r, C.byref(s)))
            ctx = Context.__new__(Context)  # borrowed: destroyed with the group
            ctx.handle, ctx.device, ctx._kernels = c, devices[r], {}
            self.contexts.append(ctx)
            self.streams.append(s.value)

    def _check(self, status: int):
        if status != OK:
            msg = lib().accb_group_last_error(self.handle)
            raise AccbError(status, msg.decode(errors="replace") if msg else "")

    def destroy(self):
        if self.handle:
            lib().accb_group_destroy(self.handle)
            self.handle = None

    def sync(self):
        self._check(lib().accb_group_sync(self.handle))

    def _k(self, k):
        return self.contexts[0]._k(k)  # one kernel object serves every context

    def _env(self, env):
        flat = [a for rank_env in env for a in rank_env]
        return _arr_list(flat), (len(env[0]) if env else 0)

    def _lls(self, xs):
        return (C.c_longlong * len(xs))(*[int(x) for x in xs])

    @staticmethod
    def _cb(arr):
        cb = [c.element_size() for c in _components(arr)]
        return (C.c_int * len(cb))(*cb)

    def map(self, kernel, env, out, scalars=None):
        sb, sn = _bytes_of(scalars)
        e, nenv = self._env(env)
        self._check(lib().accb_group_map(self.handle, self._k(kernel), e, nenv, sb, sn, _arr_list(out)))

    def fold_dim(self, kernel, env, rows, cols: int, out, seed=None):
        sb, sn = _bytes_of(seed)
        e, nenv = self._env(env)
        self._check(lib().accb_group_fold_dim(self.handle, self._k(kernel), e, nenv, self._lls(rows), cols, sb, sn,
                                              _arr_list(out)))

    def fold_all(self, kernel, combine_kernel, env, n, out, seed=None):
        sb, sn = _bytes_of(seed)
        e, nenv = self._env(env)
        outs = (accb_array * self.size)(*[to_accb_array(o, shape=()) for o in out])
        self._check(lib().accb_group_fold_all(self.handle, self._k(kernel), self._k(combine_kernel), e, nenv,
                                              self._lls(n), sb, sn, self._cb(out[0]), outs))

    def scan(self, kernel, total_kernel, carry_kernel, env, n, out, direction=SCAN_LEFT, kind=SCAN_EXCLUSIVE,
             seed=None, total=None):
        sb, sn = _bytes_of(seed)
        e, nenv = self._env(env)
        tot = (accb_array * self.size)(*[to_accb_array(t, shape=()) for t in total]) if total is not None else None
        self._check(lib().accb_group_scan(self.handle, self._k(kernel), self._k(total_kernel), self._k(carry_kernel),
                                          e, nenv, self._lls(n), direction, kind, sb, sn,
                                          _components(out[0])[0].element_size(), _arr_list(out), tot))

    def permute(self, kernel, merge_kernel, env, n_src, out, scalars=None, broadcast=False):
        sb, sn = _bytes_of(scalars)
        e, nenv = self._env(env)
        self._check(lib().accb_group_permute(self.handle, self._k(kernel), self._k(merge_kernel), e, nenv,
                                             self._lls(n_src), sb, sn, self._cb(out[0]), _arr_list(out),
                                             1 if broadcast else 0))

    def stencil_layout(self, rank: int, iters: int, ry: int, boundary="clamp"):
        t, b = C.c_int(), C.c_int()
        self._check(lib().accb_group_stencil_layout(self.handle, rank, iters, ry, BOUNDARY[boundary], C.byref(t),
                                                    C.byref(b)))
        return t.value, b.value

    def stencil2(self, kernel, a, b, out, rows, ry: int, boundary="clamp", constant=None):
        """stencil2 on row slabs padded by ``stencil_layout(rank, 1, ry, boundary)``: the halo rows of both sources
        are filled from the neighbours; the own rows of ``out`` hold the result."""
        cb, cn = _bytes_of(constant)
        self._check(lib().accb_group_stencil2(self.handle, self._k(kernel), _arr_list(a), _arr_list(b), _arr_list(out),
                                              (C.c_int * len(rows))(*rows), ry, BOUNDARY[boundary], cb, cn, self._cb(a[0])))

    def fold_seg(self, kernel, env, n, offsets, nseg, out, seed=None):
        """foldSeg split between segments: ``offsets[r]`` is rank r's run of the whole array's offsets (a device
        array of nseg[r] + 1 Int32 on that rank), rebased by the call."""
        sb, sn = _bytes_of(seed)
        e, nenv = self._env(env)
        ptrs = (C.c_void_p * self.size)(*[_ptr(o) if nseg[r] > 0 else None for r, o in enumerate(offsets)])
        self._check(lib().accb_group_fold_seg(self.handle, self._k(kernel), e, nenv, self._lls(n), ptrs, self._lls(nseg),
                                              sb, sn, _arr_list(out)))

    def stencil_iterate(self, kernel, a, b, rows, iters: int, ry: int, boundary="clamp", constant=None):
        """Returns the list of slabs (``a`` or ``b``) that hold the result in their own rows."""
        cb, cn = _bytes_of(constant)
        in_b = C.c_int()
        self._check(lib().accb_group_stencil_iterate(self.handle, self._k(kernel), _arr_list(a), _arr_list(b),
                                                     (C.c_int * len(rows))(*rows), iters, ry, BOUNDARY[boundary],
                                                     cb, cn, self._cb(a[0]), C.byref(in_b)))
        return b if in_b.value else a


# ------------------------------------------------------------------ programs
class ArrayType:
    """Shape rank and element type of an array: dtypes lists one numpy dtype per
    flattened tuple component (``Elt`` representation, CodeGen/Type.hs:101-104)."""

    def __init__(self, rank: int, dtypes):
        self.rank = rank
        self.dtypes = [np.dtype(d) for d in (dtypes if isinstance(dtypes, (tuple, list)) else [dtypes])]

    def ctype(self) -> accb_value_type:
        t = accb_value_type()
        t.rank, t.ncomp = self.rank, len(self.dtypes)
        for i, d in enumerate(self.dtypes):
            t.comp_bytes[i] = d.itemsize
        return t


class Acc:
    """A symbolic array inside a traced program."""

    def __init__(self, prog: "Afun", vid: int, atype: ArrayType):
        self.prog, self.id, self.type = prog, vid, atype


def _seed_bytes(seed, atype: ArrayType):
    if seed is None:
        return None, 0
    vals = seed if isinstance(seed, (tuple, list)) else [seed]
    b = b"".join(np.asarray(v, dtype=d).tobytes() for v, d in zip(vals, atype.dtypes))
    return C.create_string_buffer(b, len(b)), len(b)


class Afun:
    """A compiled array function: the counterpart of ``ExecAfun`` (CUDA/AST.hs:118-126)."""

    def __init__(self, ctx: Context, input_types: Sequence[ArrayType]):
        self.ctx = ctx
        self.input_types = list(input_types)
        types = (accb_value_type * max(1, len(input_types)))(*[t.ctype() for t in input_types])
        h = C.c_void_p()
        _check(lib().accb_program_create(ctx.handle, len(input_types), types, C.byref(h)), ctx.handle)
        self.handle = h
        self.inputs = [Acc(self, i, t) for i, t in enumerate(input_types)]
        self.output_types = []

    def _ids(self, env):
        return (C.c_int * max(1, len(env)))(*[e.id for e in env]), len(env)

    def _new(self, vid: int, t: ArrayType) -> Acc:
        if vid < 0:
            _check(-vid, self.ctx.handle)
        return Acc(self, vid, t)

    def set_outputs(self, outs: Sequence[Acc]):
        ids = (C.c_int * len(outs))(*[o.id for o in outs])
        _check(lib().accb_program_outputs(self.handle, ids, len(outs)), self.ctx.handle)
        self.output_types = [o.type for o in outs]

    # device arrays in, device arrays out (library-owned until the next run)
    def run_device(self, inputs: Sequence, stream=None, graph: bool = False):
        """graph=True: the whole op list as one CUDA graph launch, recorded at the first call for these
        input arrays on this stream (which must not be the default stream) and replayed afterwards."""
        ins = _arr_list(inputs)
        outs = (accb_array * len(self.output_types))()
        run = lib().accb_program_run_graph if graph else lib().accb_program_run
        _check(run(self.handle, Context._stream(stream), ins, outs), self.ctx.handle)
        return list(outs)

    # host arrays in, host arrays out: run1
    def __call__(self, *host_inputs, out=None):
        ins = (accb_array * max(1, len(host_inputs)))()
        keep = []
        for i, (x, t) in enumerate(zip(host_inputs, self.input_types)):
            comps = [np.ascontiguousarray(c, dtype=d) for c, d in zip(_components(x), t.dtypes)]
            keep.append(comps)
            a = ins[i]
            a.rank, a.ncomp = comps[0].ndim, len(comps)
            for d, e in enumerate(reversed(comps[0].shape)):
                a.shape[d] = e
            for c, arr in enumerate(comps):
                a.ptr[c] = arr.ctypes.data
        shapes = self._result_shapes([k[0].shape for k in keep])
        outs = (accb_array * len(self.output_types))()
        results = []
        for j, (t, shp) in enumerate(zip(self.output_types, shapes)):
            comps = out[j] if out is not None else [np.empty(shp, d) for d in t.dtypes]
            comps = _components(comps)
            results.append(comps)
            for c, arr in enumerate(comps):
                outs[j].ptr[c] = arr.ctypes.data
        _check(lib().accb_program_run_host(self.handle, ins, outs), self.ctx.handle)
        res = [r[0] if len(r) == 1 else tuple(r) for r in results]
        return res[0] if len(res) == 1 else tuple(res)

    def stream_chunk(self, elements: int):
        """Piece size, in elements, of the streamed host run (``accb_program_stream_chunk``): -1 the default,
        0 never run in pieces."""
        _check(lib().accb_program_stream_chunk(self.handle, elements), self.ctx.handle)
        return self

    def _result_shapes(self, in_shapes):
        return [fn(in_shapes) for fn in self._shape_fns]

    def destroy(self):
        if self.handle:
            lib().accb_program_destroy(self.handle)
            self.handle = None


def awhile(cond: Afun, body: Afun, state: Sequence, device: bool = True, max_iters: int = 1 << 20, stream=None,
           count: bool = False):
    """``awhile cond body`` on device arrays, in place: while ``cond(*state)`` (one Scalar Bool) holds, ``state``
    is replaced by ``body(*state)``.  ``device=True`` runs the whole loop as one CUDA graph with a conditional
    WHILE node -- the flag never reaches the host and the call returns at once; ``device=False`` is the
    reference's scheme, one read-back of the flag per iteration (Awhile, CUDA/Execute.hs:236-244).
    ``count=True`` waits and returns how often the body ran."""
    it = C.c_longlong(0)
    _check(lib().accb_awhile(cond.handle, body.handle, Context._stream(stream), _arr_list(state),
                             1 if device else 0, max_iters, C.byref(it) if (count or not device) else None),
           body.ctx.handle)
    return it.value if (count or not device) else None


# builder functions used inside a traced function --------------------------------
def _prog(*accs) -> Afun:
    return accs[0].prog


def map_(spec: KernelSpec, env: Sequence[Acc], out_type: ArrayType, shape_like: Acc = None, scalars=None) -> Acc:
    """map / zipWith / generate / backpermute node (Execute.hs:194-197)."""
    p = _prog(*env)
    like = shape_like or env[0]
    ids, n = p._ids(env)
    sb, sn = _bytes_of(scalars)
    t = out_type.ctype()
    vid = lib().accb_program_map(p.handle, p.ctx._k(spec), ids, n, like.id, C.byref(t), sb, sn)
    r = p._new(vid, out_type)
    r.shape_fn = like.shape_fn
    return r


def fold(spec: KernelSpec, env: Sequence[Acc], out_dtypes, seed=None, all=False, shape_like: Acc = None) -> Acc:
    """fold / fold1 / foldAll / fold1All node (Execute.hs:201-202,282-318)."""
    p = _prog(*env)
    like = shape_like or env[0]
    rank = 0 if (all or like.type.rank <= 1) else like.type.rank - 1
    out_type = ArrayType(rank, out_dtypes)
    ids, n = p._ids(env)
    sb, sn = _seed_bytes(seed, out_type)
    t = out_type.ctype()
    vid = lib().accb_program_fold(p.handle, p.ctx._k(spec), ids, n, like.id, int(all), sb, sn, C.byref(t))
    r = p._new(vid, out_type)
    seeded = seed is not None
    r.shape_fn = (lambda s, f=like.shape_fn: ()) if rank == 0 else (
        lambda s, f=like.shape_fn: tuple(max(1, e) if seeded else e for e in f(s)[:-1]))
    return r


def scan(spec: KernelSpec, env: Sequence[Acc], out_dtypes, direction=SCAN_LEFT, kind=SCAN_EXCLUSIVE, seed=None,
         shape_like: Acc = None):
    """scanl / scanl1 / scanl' / scanr / scanr1 / scanr' node (Execute.hs:205-210,328-392).
    Returns the result array, or (body, total) for the primed forms."""
    p = _prog(*env)
    like = shape_like or env[0]
    # an inclusive scan over the row-major sequence of a matrix keeps its shape (segmented / row scans)
    out_type = ArrayType(like.type.rank if kind == SCAN_INCLUSIVE else 1, out_dtypes)
    ids, n = p._ids(env)
    sb, sn = _seed_bytes(seed, out_type)
    t = out_type.ctype()
    vid = lib().accb_program_scan(p.handle, p.ctx._k(spec), ids, n, like.id, direction, kind, sb, sn, C.byref(t))
    r = p._new(vid, out_type)
    extra = 1 if kind == SCAN_EXCLUSIVE else 0
    r.shape_fn = (lambda s, f=like.shape_fn: tuple(f(s))) if kind == SCAN_INCLUSIVE else (
        lambda s, f=like.shape_fn: (f(s)[0] + extra,))
    if kind == SCAN_PRIME:
        tot = Acc(p, vid + 1, ArrayType(0, out_dtypes))
        tot.shape_fn = lambda s: ()
        return r, tot
    return r


def permute(spec: KernelSpec, env: Sequence[Acc], defaults: Acc, shape_like: Acc = None) -> Acc:
    """permute node: defaults copied first, then the scatter-combine (Execute.hs:211,396-408)."""
    p = _prog(*env)
    ids, n = p._ids(env)
    t = defaults.type.ctype()
    vid = lib().accb_program_permute(p.handle, p.ctx._k(spec), ids, n, (shape_like or env[0]).id, defaults.id, C.byref(t))
    r = p._new(vid, defaults.type)
    r.shape_fn = defaults.shape_fn
    return r


def stencil(spec: KernelSpec, src: Acc, out_dtype=None, boundary="clamp", constant=None, iters=1) -> Acc:
    """stencil node, optionally iterated in place of a chain of identical nodes (Execute.hs:212,413-425)."""
    p = src.prog
    out_type = ArrayType(src.type.rank, out_dtype or src.type.dtypes)
    cb, cn = _bytes_of(constant)
    t = out_type.ctype()
    vid = lib().accb_program_stencil(p.handle, p.ctx._k(spec), src.id, BOUNDARY[boundary], cb, cn, iters, C.byref(t))
    r = p._new(vid, out_type)
    r.shape_fn = src.shape_fn
    return r


def map_transposed(spec: KernelSpec, env: Sequence[Acc], src: Acc, out_type: ArrayType, scalars=None) -> Acc:
    """map over transposed matrices: the result has the transposed shape of ``src`` (one of the element-wise inputs)."""
    p = src.prog
    ids, n = p._ids(env)
    sb, sn = _bytes_of(scalars)
    t = out_type.ctype()
    vid = lib().accb_program_map_transposed(p.handle, p.ctx._k(spec), ids, n, src.id, C.byref(t), sb, sn)
    r = p._new(vid, out_type)
    r.shape_fn = lambda s, f=src.shape_fn: tuple(reversed(f(s)))
    return r


def generate(prog: Afun, spec: KernelSpec, env: Sequence[Acc], shape, out_type: ArrayType, scalars=None) -> Acc:
    """generate node with a literal shape (outermost extent first, as numpy writes shapes)."""
    shape = tuple(int(e) for e in shape)
    ids, n = prog._ids(env)
    sb, sn = _bytes_of(scalars)
    t = out_type.ctype()
    inner_first = (C.c_int * max(1, len(shape)))(*reversed(shape))
    vid = lib().accb_program_generate(prog.handle, prog.ctx._k(spec), ids, n, len(shape), inner_first, C.byref(t), sb, sn)
    r = prog._new(vid, out_type)
    r.shape_fn = lambda s: shape
    return r


def generate_dims(prog: Afun, spec: KernelSpec, env: Sequence[Acc], dims, out_type: ArrayType, scalars=None) -> Acc:
    """generate node whose shape is computed when the program runs.  dims lists, outermost first, one
    (source, dim, add) per extent: ``add`` plus -- when source is an Acc -- extent ``dim`` (outermost first) of it."""
    # an entry may name a second source, (source, dim, add, source2, dim2): the extents of both are added
    dims = [(e[0], int(e[1]), int(e[2]), e[3] if len(e) > 3 else None, int(e[4]) if len(e) > 3 else 0) for e in dims]
    ids, n = prog._ids(env)
    sb, sn = _bytes_of(scalars)
    t = out_type.ctype()
    r = len(dims)
    inner = list(reversed(dims))  # the C side counts extents innermost first
    ints = lambda xs: (C.c_int * max(1, r))(*xs)  # noqa: E731
    src = ints([(e[0].id if e[0] is not None else -1) for e in inner])
    sdim = ints([((e[0].type.rank - 1 - e[1]) if e[0] is not None else 0) for e in inner])
    src2 = ints([(e[3].id if e[3] is not None else -1) for e in inner])
    sdim2 = ints([((e[3].type.rank - 1 - e[4]) if e[3] is not None else 0) for e in inner])
    add = ints([e[2] for e in inner])
    vid = lib().accb_program_generate_dims2(prog.handle, prog.ctx._k(spec), ids, n, r, src, sdim, src2, sdim2, add,
                                            C.byref(t), sb, sn)
    node = prog._new(vid, out_type)
    node.shape_fn = lambda s: tuple((a.shape_fn(s)[d] if a is not None else 0) + k + (b.shape_fn(s)[d2] if b is not None else 0)
                                    for a, d, k, b, d2 in dims)
    return node


def fold_seg(spec: KernelSpec, env: Sequence[Acc], offsets: Acc, out_dtypes, seed=None, shape_like: Acc = None) -> Acc:
    """foldSeg / fold1Seg node; ``offsets`` is the Int32 vector of segments + 1 offsets (Execute.hs:320-324)."""
    p = _prog(*env)
    like = shape_like or env[0]
    out_type = ArrayType(like.type.rank, out_dtypes)
    ids, n = p._ids(env)
    sb, sn = _seed_bytes(seed, out_type)
    t = out_type.ctype()
    vid = lib().accb_program_fold_seg(p.handle, p.ctx._k(spec), ids, n, like.id, offsets.id, sb, sn, C.byref(t))
    r = p._new(vid, out_type)
    r.shape_fn = lambda s, f=like.shape_fn, g=offsets.shape_fn: tuple(f(s)[:-1]) + (g(s)[0] - 1,)
    return r


def stencil2(spec: KernelSpec, src1: Acc, src2: Acc, out_dtype, boundary="clamp", constant=None) -> Acc:
    """stencil2 node: result over the intersection of the sources (Execute.hs:427-450)."""
    p = src1.prog
    out_type = ArrayType(src1.type.rank, out_dtype)
    cb, cn = _bytes_of(constant)
    t = out_type.ctype()
    vid = lib().accb_program_stencil2(p.handle, p.ctx._k(spec), src1.id, src2.id, BOUNDARY[boundary], cb, cn, C.byref(t))
    r = p._new(vid, out_type)
    r.shape_fn = lambda s, f=src1.shape_fn, g=src2.shape_fn: tuple(min(a, b) for a, b in zip(f(s), g(s)))
    return r


_default_context = None


def default_context() -> Context:
    """The process-wide context on device 0 (``defaultContext``, CUDA/State.hs:111-132)."""
    global _default_context
    if _default_context is None:
        _default_context = Context(0)
    return _default_context


def create(device: int = 0, cu_context=None) -> Context:
    return Context(device, cu_context)


def destroy(ctx: Context):
    ctx.destroy()


def run1With(ctx: Context, f: Callable, *input_types: ArrayType) -> Afun:
    """Compile an array function once; the result maps host arrays to host arrays
    and can be applied many times (``run1With``, CUDA.hs:312-330)."""
    prog = Afun(ctx, input_types)
    for i, a in enumerate(prog.inputs):
        a.shape_fn = lambda s, i=i: tuple(s[i])
    outs = f(*prog.inputs)
    outs = list(outs) if isinstance(outs, (tuple, list)) else [outs]
    prog.set_outputs(outs)
    prog._shape_fns = [o.shape_fn for o in outs]
    return prog


def run1(f: Callable, *input_types: ArrayType) -> Afun:
    return run1With(default_context(), f, *input_types)


def _types_of(arrays):
    ts = []
    for x in arrays:
        comps = _components(x)
        ts.append(ArrayType(np.asarray(comps[0]).ndim, [np.asarray(c).dtype for c in comps]))
    return ts


def runWith(ctx: Context, f: Callable, *arrays):
    """Compile and run once on the given host arrays (``runWith``, CUDA.hs:248-251)."""
    prog = run1With(ctx, f, *_types_of(arrays))
    try:
        return prog(*arrays)
    finally:
        prog.destroy()


def run(f: Callable, *arrays):
    return runWith(default_context(), f, *arrays)


def stream(f: Callable, input_types: Sequence[ArrayType], inputs):
    """Apply one compiled function to a sequence of inputs (``stream``, CUDA.hs:333-347)."""
    prog = run1(f, *input_types)
    for x in inputs:
        yield prog(*(x if isinstance(x, (tuple, list)) else (x,)))


def runAsync(f: Callable, *arrays):
    """``runAsync`` (CUDA.hs:258-266): returns a future of the result."""
    from concurrent.futures import ThreadPoolExecutor
    ex = ThreadPoolExecutor(max_workers=1)
    fut = ex.submit(run, f, *arrays)
    ex.shutdown(wait=False)
    return fut


def unsafeFree(ctx: Context, key: int):
    """Release the device copy of a host array now (``unsafeFreeWith``, CUDA.hs:421-431)."""
    _check(lib().accb_free(ctx.handle, key), ctx.handle)


def performGC(ctx: Context = None):
    """Evict every unpinned array that has a host copy (``performGCWith``, CUDA.hs:433-441)."""
    ctx = ctx or default_context()
    _check(lib().accb_reclaim(ctx.handle), ctx.handle)
