"""The synthetic input generators: index-addressable (a shard reproduces its slice),
within range, and with the stated distributions."""
import numpy as np


def test_generators_are_index_addressable(workloads):
    W = workloads
    full = W.uniform_f32(W.SEED, W.S_XS, 10000, -1, 1)
    assert np.array_equal(full[1234:5678], W.uniform_f32(W.SEED, W.S_XS, 5678 - 1234, -1, 1, first=1234))
    ints = W.uniform_i32(W.SEED, W.S_SCAN, 10000, 16)
    assert np.array_equal(ints[9000:], W.uniform_i32(W.SEED, W.S_SCAN, 1000, 16, first=9000))
    cdf = W.zipf_cdf()
    keys = W.zipf_mix_keys(W.SEED, 10000, cdf)
    assert np.array_equal(keys[77:4001], W.zipf_mix_keys(W.SEED, 4001 - 77, cdf, first=77))


def test_ranges_and_streams_differ(workloads):
    W = workloads
    a = W.uniform_f32(W.SEED, W.S_SPOT, 100000, 5, 30)
    assert a.dtype == np.float32 and a.min() >= 5 and a.max() < 30 and abs(a.mean() - 17.5) < 0.1
    b = W.uniform_f32(W.SEED, W.S_STRIKE, 100000, 5, 30)
    assert not np.array_equal(a, b)
    i = W.uniform_i32(W.SEED, W.S_SCAN, 100000, 16)
    assert i.min() == 0 and i.max() == 15 and abs(i.mean() - 7.5) < 0.1


def test_zipf_mix_puts_about_eight_percent_of_the_keys_in_bin_zero(workloads):
    """50 % Zipf(1.1) over 4096 bins + 50 % uniform: P(bin 0) = 0.5/H(4096,1.1) + 0.5/4096 = 8.04 %."""
    W = workloads
    cdf = W.zipf_cdf()
    assert cdf.size == 4096 and abs(cdf[-1] - 1) < 1e-12 and np.all(np.diff(cdf) > 0)
    keys = W.zipf_mix_keys(W.SEED, 400000, cdf)
    assert keys.min() >= 0 and keys.max() < 4096
    assert abs((keys == 0).mean() - 0.0804) < 0.003


def test_algorithmic_bytes(workloads):
    W = workloads
    assert W.bytes_dot(W.N24) == 134217732 and W.bytes_scan(W.N28) == 2147483652
    assert W.bytes_hist(W.N28) == 1073774592 and W.bytes_stencil(8192, 8192, 10) == 5368709120
    assert W.bytes_blackscholes(W.N26) == 1342177280 and W.bytes_rowsum(16384, 16384) == 1073807360


def test_bench_workloads_have_the_methods_the_driver_loop_calls():
    """bench.py only runs on a GPU; this catches a workload class that lost a method in an edit."""
    import importlib
    bench = importlib.import_module("bench")
    classes = list(bench.WORKLOADS.values()) + list(bench.SECONDARY.values())
    assert len(classes) >= 10
    for cls in classes:
        for m in ("setup", "step", "verify", "functor", "make_peer", "peer_views"):
            assert callable(getattr(cls, m, None)), f"{cls.__name__}.{m}"
