"""Synthetic inputs of the five benchmark configurations.

One index-addressable generator defines every input, so that the numpy code
below, the device generators in ``csrc/runtime/util_kernels.cu`` and every
shard of a multi-GPU run produce the same element ``i`` from ``(seed,
stream, i)``:

    mix(z):  z ^= z >> 30; z *= 0xbf58476d1ce4e5b9; z ^= z >> 27;
             z *= 0x94d049bb133111eb; z ^= z >> 31           (64-bit wrap)
    key    = mix(seed ^ (stream * 0x9E3779B97F4A7C15))
    h(i)   = mix(key + (i + 1) * 0x9E3779B97F4A7C15)
    float in [lo, hi):  fma(hi - lo, (h >> 40) * 2**-24, lo)  in float32
    int in [0, m):      ((h >> 32) * m) >> 32
    double in [0, 1):   (h >> 11) * 2**-53

No public dataset is involved: the configurations are defined by their
distributions (uniform ranges, a 50/50 mix of Zipf(1.1) and uniform keys).
"""
from __future__ import annotations

import numpy as np

SEED = 0x5EEDB200
GOLDEN = np.uint64(0x9E3779B97F4A7C15)

# stream ids
S_XS, S_YS, S_COIN, S_ZIPF, S_UNIF, S_SCAN, S_GRID, S_SPOT, S_STRIKE, S_YEARS, S_MATRIX = range(11)

N24, N26, N28 = 1 << 24, 1 << 26, 1 << 28
HIST_BINS = 4096
BLUR_WEIGHTS = np.array([[1, 2, 1], [2, 4, 2], [1, 2, 1]], np.float64) / 16.0


def _mix(z: np.ndarray) -> np.ndarray:
    z = z.astype(np.uint64, copy=True)
    z ^= z >> np.uint64(30)
    z *= np.uint64(0xbf58476d1ce4e5b9)
    z ^= z >> np.uint64(27)
    z *= np.uint64(0x94d049bb133111eb)
    z ^= z >> np.uint64(31)
    return z


def stream_key(seed: int, stream: int) -> np.uint64:
    with np.errstate(over="ignore"):
        return _mix(np.array([np.uint64(seed) ^ (np.uint64(stream) * GOLDEN)], np.uint64))[0]


def hashes(seed: int, stream: int, n: int, first: int = 0) -> np.ndarray:
    with np.errstate(over="ignore"):
        i = np.arange(first + 1, first + n + 1, dtype=np.uint64)
        return _mix(stream_key(seed, stream) + i * GOLDEN)


def uniform_f32(seed, stream, n, lo, hi, first=0) -> np.ndarray:
    h = hashes(seed, stream, n, first)
    u = (h >> np.uint64(40)).astype(np.float64) * 2.0 ** -24
    lo32, hi32 = np.float32(lo), np.float32(hi)
    span = np.float64(np.float32(hi32 - lo32))
    # exact in double for the ranges used here, so one rounding == fmaf
    return (span * u + np.float64(lo32)).astype(np.float32)


def uniform_i32(seed, stream, n, m, first=0) -> np.ndarray:
    h = hashes(seed, stream, n, first)
    return (((h >> np.uint64(32)) * np.uint64(m)) >> np.uint64(32)).astype(np.int32)


def zipf_cdf(nbins: int = HIST_BINS, s: float = 1.1) -> np.ndarray:
    """Inverse-CDF table of Zipf(s) over [0, nbins): built on the host in
    float64 and handed to the device generator as data."""
    w = 1.0 / np.arange(1, nbins + 1, dtype=np.float64) ** s
    return np.cumsum(w) / w.sum()


def zipf_mix_keys(seed, n, cdf: np.ndarray, first=0) -> np.ndarray:
    nbins = cdf.size
    coin = (hashes(seed, S_COIN, n, first) >> np.uint64(63)).astype(bool)
    u = (hashes(seed, S_ZIPF, n, first) >> np.uint64(11)).astype(np.float64) * 2.0 ** -53
    zk = np.minimum(np.searchsorted(cdf, u, side="right"), nbins - 1).astype(np.int32)
    uk = (((hashes(seed, S_UNIF, n, first) >> np.uint64(32)) * np.uint64(nbins)) >> np.uint64(32)).astype(np.int32)
    return np.where(coin, zk, uk).astype(np.int32)


# ---- algorithmic bytes per configuration: the numerator of the roofline ----
def bytes_dot(n):          # two Float vectors in, one Float out
    return 2 * 4 * n + 4


def bytes_scan(n):         # Int32 in, n+1 Int32 out
    return 4 * n + 4 * (n + 1)


def bytes_hist(n, bins=HIST_BINS):   # keys in, defaults in + result out
    return 4 * n + 2 * 4 * bins


def bytes_stencil(h, w, iters):      # one read and one write of the grid per iteration
    return 2 * 4 * h * w * iters


def bytes_blackscholes(n):           # 3 Float in, 2 Float out
    return 5 * 4 * n


def bytes_rowsum(rows, cols):
    return 4 * rows * cols + 4 * rows
