"""baseline/refskel: the reference's own algorithms as CUDA, used by bench.py as a GPU baseline.
They must compute what the library computes, or the comparison means nothing."""
import ctypes as C
import importlib

import numpy as np
import pytest

SYMBOLS = ["refskel_map_blackscholes", "refskel_dot", "refskel_fold_rows", "refskel_scanl", "refskel_histogram",
           "refskel_stencil_blur", "refskel_config"]


def test_library_builds_and_exports_its_entry_points():
    R = importlib.import_module("baseline.refskel")
    lib = C.CDLL(R.build())
    for s in SYMBOLS:
        assert hasattr(lib, s), s


@pytest.fixture(scope="module")
def R(torch_cuda):
    mod = importlib.import_module("baseline.refskel")
    mod.build()
    return mod


@pytest.mark.gpu
@pytest.mark.parametrize("n", [1, 1000, 300001])
def test_scan_and_dot_and_histogram(R, torch_cuda, n):
    t = torch_cuda
    scratch = R.scratch_elems(t.cuda.get_device_properties(0).multi_processor_count)
    x = t.randint(0, 16, (n,), dtype=t.int32, device="cuda")
    out = t.zeros(n + 1, dtype=t.int32, device="cuda")
    R.scanl(x, 5, out, t.zeros(scratch, dtype=t.int32, device="cuda"))
    ref = t.cat([t.tensor([5], device="cuda"), 5 + t.cumsum(x.long(), 0)]).int()
    assert t.equal(out, ref)

    a, b = t.rand(n, device="cuda") - 0.5, t.rand(n, device="cuda") - 0.5
    o = t.zeros(1, device="cuda")
    R.dot(a, b, 1.0, t.zeros(scratch, device="cuda"), o)
    assert abs(float(o[0]) - (float((a.double() * b.double()).sum()) + 1.0)) <= 1e-6 * n + 1e-5

    keys = t.randint(0, 4096, (n,), dtype=t.int32, device="cuda")  # spread keys: little lock contention
    d = t.full((4096,), 2, dtype=t.int32, device="cuda")
    h, lock, err = t.zeros_like(d), t.zeros_like(d), t.zeros(1, dtype=t.int32, device="cuda")
    R.histogram(keys, d, h, lock, err)
    assert t.equal(h, t.bincount(keys.long(), minlength=4096).int() + 2) and int(err[0]) == 0


@pytest.mark.gpu
@pytest.mark.parametrize("h,w", [(3, 5), (100, 257), (512, 1024)])
def test_stencil_and_row_fold(R, torch_cuda, h, w):
    t = torch_cuda
    F = t.nn.functional
    g = t.rand((h, w), device="cuda")
    o = t.empty_like(g)
    R.stencil_blur(g, o)
    k = t.tensor([[1, 2, 1], [2, 4, 2], [1, 2, 1]], device="cuda", dtype=t.float32)[None, None] / 16
    ref = F.conv2d(F.pad(g[None, None], (1, 1, 1, 1), mode="replicate"), k)[0, 0]
    assert float((o - ref).abs().max()) <= 1e-6
    ro = t.empty(h, device="cuda")
    R.fold_rows(g, 1.0, ro)
    assert float((ro.double() - (g.double().sum(1) + 1)).abs().max()) <= 1e-4 * w / 100 + 1e-5


@pytest.mark.gpu
def test_map_blackscholes_put_call_parity(R, torch_cuda):
    t = torch_cuda
    n = 100000
    s, k, y = t.rand(n, device="cuda") * 25 + 5, t.rand(n, device="cuda") * 99 + 1, t.rand(n, device="cuda") * 9.75 + 0.25
    c, p = t.empty(n, device="cuda"), t.empty(n, device="cuda")
    R.map_blackscholes(s, k, y, c, p)
    assert float(((c - p) - (s - k * t.exp(-0.02 * y))).abs().max()) <= 1e-4
