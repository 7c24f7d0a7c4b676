"""The host runtime on a GPU: run-time compilation and the kernel cache, launch configuration,
the device memory table, streams and events, and the bounded device-side waits."""
import ctypes as C
import os
import time

import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def _fresh_map_spec(accb, tag):
    """A functor nobody compiled before (the tag goes into the source, hence into the cache key)."""
    return accb.KernelSpec("map", "Jit", f"""
struct Jit {{
    using In = accb::types<int>; using Out = accb::types<int>;
    static __device__ __forceinline__ void apply(const accb::Env &, long long i, int x, int &o) {{ o = 3 * x + {tag}; }}
}};""")


def test_run_time_compile_then_memory_and_disk_cache(accb, torch_cuda, tmp_path, monkeypatch):
    """nvcc -arch=sm_100a at run time on a miss; the second context finds the cubin in the process-wide
    table; a later process would find it on disk under <cache>/sm_100a/<key>.cubin (Persistent.hs:218-228)."""
    t = torch_cuda
    monkeypatch.setenv("ACCB_CACHE_DIR", str(tmp_path))
    tag = int(time.time() * 1000) % 1000003
    spec = _fresh_map_spec(accb, tag)
    ctx1 = accb.Context(0)
    x = t.arange(10000, dtype=t.int32, device="cuda")
    out = t.zeros_like(x)
    ctx1.map(spec, [x], out)  # returns at once; the launch waits for the compiler (lazy link, Compile.hs:444-459)
    ctx1.sync()
    assert t.equal(out, 3 * x + tag)
    assert ctx1.cache_stats()["compiles"] == 1
    files = list((tmp_path / "sm_100a").glob("*.cubin"))
    assert len(files) == 1 and files[0].stat().st_size > 1000
    ctx2 = accb.Context(0)
    out.zero_()
    ctx2.map(spec, [x], out)
    ctx2.sync()
    assert t.equal(out, 3 * x + tag)
    ctx1.destroy()
    ctx2.destroy()


def test_compile_error_surfaces_at_first_use(accb, ctx, torch_cuda):
    t = torch_cuda
    bad = accb.KernelSpec("map", "Bad", "struct Bad { using In = accb::types<int>; using Out = accb::types<int>; "
                          f"static __device__ void apply(const accb::Env&, long long, int x, int& o) {{ o = undefined_{os.getpid()}; }} }};")
    x = t.zeros(16, dtype=t.int32, device="cuda")
    with pytest.raises(accb.AccbError) as e:
        ctx.map(bad, [x], x.clone())
    assert e.value.status == accb.ECOMPILE and "undefined_" in str(e.value)


def test_kernel_info_and_launch_config(accb, P, ctx):
    """registers / shared memory / resident blocks from the driver (determineOccupancy, Launch.hs:62-74);
    grid = min(SMs x resident blocks, work) (launchConfig, Launch.hs:42-55)."""
    k = ctx.kernel(P.DOT).wait()
    info = k.info("foldAll")
    assert 16 <= info["regs"] <= 128 and info["block"] == 256 and 1 <= info["blocks_per_sm"] <= 8
    L = accb.lib()
    b, g, s = C.c_int(), C.c_int(), C.c_int()
    assert L.accb_launch_config(ctx.handle, k.handle, b"foldAll", 1 << 28, C.byref(b), C.byref(g), C.byref(s)) == 0
    assert b.value == 256 and g.value == ctx.sm_count * info["blocks_per_sm"]
    assert L.accb_launch_config(ctx.handle, k.handle, b"foldAll", 1000, C.byref(b), C.byref(g), C.byref(s)) == 0
    assert g.value == 1
    with pytest.raises(accb.AccbError) as e:
        k.info("no_such_entry")
    assert e.value.status == accb.ENOTFOUND


def test_wrong_skeleton_and_bad_arguments_are_rejected(accb, P, ctx, torch_cuda):
    t = torch_cuda
    x = t.zeros(64, dtype=t.int32, device="cuda")
    with pytest.raises(accb.AccbError) as e:
        ctx.map(P.SCAN_ADD_I32, [x], x.clone())
    assert e.value.status == accb.EINVAL
    with pytest.raises(accb.AccbError):
        ctx.scan(P.SCAN_ADD_I32, [x], 64, t.zeros(65, dtype=t.int32, device="cuda"))  # exclusive scan without a seed
    with pytest.raises(accb.AccbError):
        ctx.stencil(P.BLUR, t.zeros((8, 8), device="cuda"), t.zeros((8, 8), device="cuda"), boundary="constant")


def test_memory_table_on_the_device(accb, torch_cuda):
    """malloc / use / peek / poke / copy / index / with_ptr / free (Array/Remote.hs, Array/Prim.hs)."""
    L = accb.lib()
    ctx = accb.Context(0)
    h = ctx.handle
    a = np.arange(1000, dtype=np.int32)
    d = C.c_void_p()
    assert L.accb_use(h, 1, a.ctypes.data_as(C.c_void_p), a.nbytes, None, C.byref(d)) == 0
    d2 = C.c_void_p()
    assert L.accb_use(h, 1, a.ctypes.data_as(C.c_void_p), a.nbytes, None, C.byref(d2)) == 0 and d2.value == d.value  # resident: no second upload
    assert L.accb_malloc(h, 2, a.nbytes, C.byref(d2)) == 0
    assert L.accb_copy(h, 1, 2, a.nbytes, None) == 0
    patch = np.array([-7, -8], np.int32)
    assert L.accb_poke(h, 2, 40, patch.ctypes.data_as(C.c_void_p), patch.nbytes, None) == 0
    back = np.zeros(1000, np.int32)
    assert L.accb_peek(h, 2, 0, back.ctypes.data_as(C.c_void_p), back.nbytes, None) == 0
    ctx.sync()
    ref = a.copy(); ref[10:12] = patch
    assert np.array_equal(back, ref)
    one = C.c_int32()
    assert L.accb_index(h, 2, 11, 4, C.byref(one)) == 0 and one.value == -8
    assert L.accb_peek(h, 2, 3990, back.ctypes.data_as(C.c_void_p), 100, None) == accb.EBOUNDS
    n, b, ev = C.c_size_t(), C.c_size_t(), C.c_size_t()
    assert L.accb_memory_stats(h, C.byref(n), C.byref(b), C.byref(ev)) == 0 and n.value == 2 and b.value == 2 * 4096
    # pinned arrays survive a reclaim, unpinned ones with a host copy are written back and evicted
    sz = C.c_size_t()
    assert L.accb_with_ptr(h, 1, C.byref(d), C.byref(sz)) == 0 and sz.value == a.nbytes
    assert L.accb_reclaim(h) == 0
    assert L.accb_memory_stats(h, C.byref(n), C.byref(b), C.byref(ev)) == 0 and ev.value == 0
    assert L.accb_release(h, 1) == 0
    assert L.accb_reclaim(h) == 0
    assert L.accb_memory_stats(h, C.byref(n), C.byref(b), C.byref(ev)) == 0 and ev.value == 1
    # ... and come back on the next use
    assert L.accb_index(h, 1, 999, 4, C.byref(one)) == 0 and one.value == 999
    assert L.accb_free(h, 1) == 0 and L.accb_free(h, 2) == 0 and L.accb_free(h, 2) == accb.ENOTFOUND
    ctx.destroy()


def test_eviction_waits_for_work_that_still_uses_an_array(accb, P, torch_cuda):
    """An array released while a kernel on another stream still writes it: accb_release_after leaves a waypoint
    behind that kernel, and the write-back of an eviction waits for it (Array/Remote.hs:113-134), so the host copy
    receives the finished result."""
    t = torch_cuda
    L = accb.lib()
    ctx = accb.Context(0)
    h = ctx.handle
    n = 1 << 24
    host = np.zeros(n, np.int32)
    d, sz = C.c_void_p(), C.c_size_t()
    assert L.accb_use(h, 7, host.ctypes.data_as(C.c_void_p), host.nbytes, None, C.byref(d)) == 0
    assert L.accb_with_ptr(h, 7, C.byref(d), C.byref(sz)) == 0
    stream = t.cuda.Stream()
    out = t.as_tensor(accb.DeviceArray(d.value, (n,), np.int32), device="cuda")
    x = t.ones(n, dtype=t.int32, device="cuda")
    t.cuda.synchronize()
    for _ in range(20):  # enough queued work that the last launch is still pending when the eviction starts
        ctx.scan(P.SCAN_ADD_I32, [x], n - 1, out, seed=np.int32(1), stream=stream.cuda_stream)
    assert L.accb_release_after(h, 7, C.c_void_p(stream.cuda_stream)) == 0
    assert L.accb_reclaim(h) == 0  # writes key 7 back to `host` and frees it
    ev, nn, b = C.c_size_t(), C.c_size_t(), C.c_size_t()
    assert L.accb_memory_stats(h, C.byref(nn), C.byref(b), C.byref(ev)) == 0 and ev.value == 1
    assert np.array_equal(host, np.arange(1, n + 1, dtype=np.int32))
    assert L.accb_release_after(h, 12345, None) == accb.ENOTFOUND
    t.cuda.synchronize()
    ctx.destroy()


def test_streams_and_events(accb, P, torch_cuda):
    """A producer on one stream, a consumer on another, joined by an event (Execute/Stream.hs:66-74,
    Execute/Event.hs:112-115); streams and events are recycled through the reservoirs."""
    t = torch_cuda
    L = accb.lib()
    ctx = accb.Context(0)
    s1, s2 = C.c_void_p(), C.c_void_p()
    assert L.accb_stream_acquire(ctx.handle, C.byref(s1)) == 0 and L.accb_stream_acquire(ctx.handle, C.byref(s2)) == 0
    n = 1 << 22
    x = t.ones(n, dtype=t.int32, device="cuda")
    mid = t.zeros(n + 1, dtype=t.int32, device="cuda")
    tot = t.zeros(1, dtype=t.int32, device="cuda")
    t.cuda.synchronize()
    ctx.scan(P.SCAN_ADD_I32, [x], n, mid, seed=np.int32(0), stream=s1.value)
    ev = C.c_void_p()
    assert L.accb_event_record(ctx.handle, s1, C.byref(ev)) == 0
    assert L.accb_stream_wait_event(ctx.handle, s2, ev) == 0
    ctx.fold_all(P.MAX_I32, [mid], n + 1, tot, stream=s2.value)
    assert L.accb_stream_sync(ctx.handle, s2) == 0
    done = C.c_int()
    assert L.accb_event_query(ctx.handle, ev, C.byref(done)) == 0 and done.value == 1
    assert int(tot[0]) == n
    assert L.accb_event_release(ctx.handle, ev) == 0
    assert L.accb_stream_release(ctx.handle, s1) == 0 and L.accb_stream_release(ctx.handle, s2) == 0
    s3 = C.c_void_p()
    assert L.accb_stream_acquire(ctx.handle, C.byref(s3)) == 0 and s3.value in (s1.value, s2.value)  # reused
    L.accb_stream_release(ctx.handle, s3)
    ctx.destroy()


def test_a_device_side_wait_that_runs_out_is_reported_not_hung(accb, P, torch_cuda):
    """Bounded look-back: with the first tile never publishing, its successors give up after their poll
    limit, raise the error word and finish; the host sees ACCB_ETIMEOUT at the next sync and the
    context stays usable.  Nothing faults and nothing spins forever."""
    t = torch_cuda
    ctx = accb.Context(0)
    broken = accb.KernelSpec("scan", "AddI", P.SCAN_ADD_I32.source, "-DACCB_SCAN_TEST_DROP_TILE0 -DACCB_SCAN_SPIN_LIMIT=64")
    n = 100000
    x = t.ones(n, dtype=t.int32, device="cuda")
    out = t.zeros(n + 1, dtype=t.int32, device="cuda")
    ctx.scan(broken, [x], n, out, seed=np.int32(0))
    with pytest.raises(accb.AccbError) as e:
        ctx.sync()
    assert e.value.status == accb.ETIMEOUT
    # the error word was cleared and the context still works
    ctx.scan(P.SCAN_ADD_I32, [x], n, out, seed=np.int32(0))
    ctx.sync()
    assert int(out[-1]) == n
    ctx.destroy()


def test_injected_allocation_failure_is_an_error_not_a_crash(accb, torch_cuda):
    """ACCB_FAIL=malloc: the allocator reports out-of-memory once; with nothing to evict the call
    fails with ACCB_ENOMEM and the next call succeeds.  Run in a child process (the injection counter
    is per process)."""
    import subprocess, sys
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    code = f"""
import sys, importlib, ctypes as C
sys.path.insert(0, {root!r})
accb = importlib.import_module("accelerate-cuda_b200")
L = accb.lib(); ctx = accb.Context(0); d = C.c_void_p()
print(L.accb_malloc(ctx.handle, 1, 4096, C.byref(d)), L.accb_malloc(ctx.handle, 2, 4096, C.byref(d)))
"""
    out = subprocess.run([sys.executable, "-c", code], env=dict(os.environ, ACCB_FAIL="malloc"), capture_output=True,
                         text=True, timeout=300)
    assert out.returncode == 0, out.stderr
    assert out.stdout.split() == [str(accb.ENOMEM), "0"]
