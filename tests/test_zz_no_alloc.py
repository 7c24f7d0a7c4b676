"""The allocation-free scan entry point against the regular one.

``accb_scanl_add_i32_noalloc`` is for callers that cannot allocate device
memory at the point of the call (a fixed memory budget, a callback that must
not touch the allocator).  It keeps its tile status words in an array that is
part of the library image, shared by all calls and never cleared behind the
caller's back, so the test makes two calls in a row on different inputs and
checks both bit-for-bit against ``accb_scan``.  The file name sorts last on
purpose: with ``-x`` every other test has run before this one.
"""
import ctypes as C

import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def _noalloc(accb, torch, x, seed, out, status):
    L = accb.lib()
    fn = L.accb_scanl_add_i32_noalloc
    fn.argtypes = [C.c_int, C.c_void_p, C.c_void_p, C.c_longlong, C.c_int32, C.c_void_p, C.c_void_p]
    fn.restype = C.c_int
    st = fn(0, C.c_void_p(int(torch.cuda.current_stream().cuda_stream)), C.c_void_p(x.data_ptr()), x.numel(),
            int(seed), C.c_void_p(out.data_ptr()), C.c_void_p(status.data_ptr()))
    return st


def test_noalloc_scan_matches_regular_scan_on_two_calls_in_a_row(accb, P, ctx, torch_cuda):
    t = torch_cuda
    rng = np.random.default_rng(7)
    status = t.ones(1, dtype=t.int32, device="cuda")
    # second call is smaller and ragged: it must not see the first call's status words
    for n, seed in (((1 << 21) + 12345, -3), (70001, 11)):
        x = t.from_numpy(rng.integers(-2**31, 2**31 - 1, n).astype(np.int32)).cuda()
        ref = t.zeros(n + 1, dtype=t.int32, device="cuda")
        got = t.full((n + 1,), 0x55555555, dtype=t.int32, device="cuda")
        ctx.scan(P.SCAN_ADD_I32, [x], n, ref, seed=np.int32(seed))
        assert _noalloc(accb, t, x, seed, got, status) == accb.OK
        ctx.sync()
        t.cuda.synchronize()
        assert int(status[0]) == 0
        assert t.equal(got, ref)  # integer work: bit-exact


def test_noalloc_scan_rejects_inputs_beyond_its_fixed_scratch(accb, torch_cuda):
    t = torch_cuda
    x = t.zeros(16, dtype=t.int32, device="cuda")
    L = accb.lib()
    fn = L.accb_scanl_add_i32_noalloc
    fn.argtypes = [C.c_int, C.c_void_p, C.c_void_p, C.c_longlong, C.c_int32, C.c_void_p, C.c_void_p]
    fn.restype = C.c_int
    st = fn(0, None, C.c_void_p(x.data_ptr()), (1 << 28) + 1, 0, C.c_void_p(x.data_ptr()), None)
    assert st == accb.EINVAL
    assert b"exceed" in L.accb_last_error(None)
