/*
 * util_kernels.cu -- kernels that are part of the library binary itself:
 * index-addressable generators for the synthetic benchmark inputs and the L2
 * flush used between timed iterations.
 *
 * Generator definition (shared with the numpy restatement in
 * accelerate-cuda_b200/workloads.py, which the tests compare against):
 *   mix(z): z ^= z>>30; z *= 0xbf58476d1ce4e5b9; z ^= z>>27;
 *           z *= 0x94d049bb133111eb; z ^= z>>31
 *   key    = mix(seed ^ (stream * 0x9E3779B97F4A7C15))
 *   h(i)   = mix(key + (i+1) * 0x9E3779B97F4A7C15)
 *   uniform float in [lo,hi): fma(hi-lo, (h>>40) * 2^-24, lo)
 *   uniform int in [0,m):     ((h>>32) * m) >> 32
 *   uniform double in [0,1):  (h>>11) * 2^-53
 * Element i depends only on (seed, stream, i), so any shard of any GPU can
 * produce its own slice.
 */
#include <algorithm>

#include "common.h"

namespace {

__host__ __device__ inline unsigned long long mix64(unsigned long long z) {
    z ^= z >> 30;
    z *= 0xbf58476d1ce4e5b9ull;
    z ^= z >> 27;
    z *= 0x94d049bb133111ebull;
    z ^= z >> 31;
    return z;
}
constexpr unsigned long long kGolden = 0x9E3779B97F4A7C15ull;

__device__ inline unsigned long long hash_at(unsigned long long key, long long i) {
    return mix64(key + (unsigned long long)(i + 1) * kGolden);
}

__global__ void gen_uniform_f32(float *dst, long long n, long long first, unsigned long long key, float lo, float hi) {
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x) {
        const unsigned long long h = hash_at(key, first + i);
        const float u = (float)(h >> 40) * 0x1p-24f;
        dst[i] = __fmaf_rn(hi - lo, u, lo);
    }
}

__global__ void gen_uniform_i32(int *dst, long long n, long long first, unsigned long long key, unsigned m) {
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x) {
        const unsigned long long h = hash_at(key, first + i);
        dst[i] = (int)(((h >> 32) * (unsigned long long)m) >> 32);
    }
}

/* dst[i] = src[i] - src[0]: a run of segment offsets of a larger array, made to start at zero */
__global__ void rebase_i32(int *dst, const int *src, long long n) {
    const int base = src[0];
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x)
        dst[i] = src[i] - base;
}

/* streams: 2 = coin, 3 = Zipf draw, 4 = uniform draw */
__global__ void gen_zipf_mix(int *dst, long long n, long long first, unsigned long long k_coin,
                             unsigned long long k_zipf, unsigned long long k_unif, const double *cdf, int nbins) {
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (long long)gridDim.x * blockDim.x) {
        const bool zipf = (hash_at(k_coin, first + i) >> 63) != 0;
        int key;
        if (zipf) {
            const double u = (double)(hash_at(k_zipf, first + i) >> 11) * 0x1p-53;
            /* number of table entries <= u (searchsorted, side = right) */
            int lo = 0, hi = nbins;
            while (lo < hi) {
                const int mid = (lo + hi) >> 1;
                if (cdf[mid] <= u)
                    lo = mid + 1;
                else
                    hi = mid;
            }
            key = lo < nbins ? lo : nbins - 1;
        } else {
            key = (int)(((hash_at(k_unif, first + i) >> 32) * (unsigned long long)nbins) >> 32);
        }
        dst[i] = key;
    }
}

__global__ void flush_l2_kernel(uint4 *buf, long long nvec, unsigned tag) {
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < nvec; i += (long long)gridDim.x * blockDim.x)
        buf[i] = make_uint4(tag, tag, tag, tag);
}

unsigned long long stream_key(unsigned long long seed, unsigned long long stream) {
    return mix64(seed ^ (stream * kGolden));
}

}  // namespace

using namespace accb_rt;

#define LOCK(ctx)                                                   \
    if (!(ctx)) return fail(nullptr, ACCB_EINVAL, "null context"); \
    std::lock_guard<std::recursive_mutex> lock_((ctx)->mu);         \
    CtxGuard guard_(ctx)

static int gen_grid(accb_context *ctx, long long n) {
    const long long blocks = (n + 255) / 256;
    return (int)std::max<long long>(1, std::min<long long>(blocks, (long long)ctx->sm_count * 16));
}

extern "C" {

int accb_gen_uniform_f32(accb_context *ctx, accb_stream stream, float *dst, long long n, long long first_index,
                         uint64_t seed, uint64_t stream_id, float lo, float hi) {
    LOCK(ctx);
    if (!dst || n < 0) return fail(ctx, ACCB_EINVAL, "bad argument");
    if (n == 0) return ACCB_OK;
    gen_uniform_f32<<<gen_grid(ctx, n), 256, 0, (cudaStream_t)stream>>>(dst, n, first_index, stream_key(seed, stream_id), lo, hi);
    ctx->launches++;
    return check_cuda(ctx, cudaGetLastError(), "gen_uniform_f32");
}

int accb_gen_uniform_i32(accb_context *ctx, accb_stream stream, int32_t *dst, long long n, long long first_index,
                         uint64_t seed, uint64_t stream_id, int32_t m) {
    LOCK(ctx);
    if (!dst || n < 0 || m <= 0) return fail(ctx, ACCB_EINVAL, "bad argument");
    if (n == 0) return ACCB_OK;
    gen_uniform_i32<<<gen_grid(ctx, n), 256, 0, (cudaStream_t)stream>>>(dst, n, first_index, stream_key(seed, stream_id), (unsigned)m);
    ctx->launches++;
    return check_cuda(ctx, cudaGetLastError(), "gen_uniform_i32");
}

int accb_gen_zipf_mix_i32(accb_context *ctx, accb_stream stream, int32_t *dst, long long n, long long first_index,
                          uint64_t seed, const double *cdf, int nbins) {
    LOCK(ctx);
    if (!dst || !cdf || n < 0 || nbins <= 0) return fail(ctx, ACCB_EINVAL, "bad argument");
    if (n == 0) return ACCB_OK;
    gen_zipf_mix<<<gen_grid(ctx, n), 256, 0, (cudaStream_t)stream>>>(dst, n, first_index, stream_key(seed, 2),
                                                                    stream_key(seed, 3), stream_key(seed, 4), cdf, nbins);
    ctx->launches++;
    return check_cuda(ctx, cudaGetLastError(), "gen_zipf_mix");
}

int accb_flush_l2(accb_context *ctx, accb_stream stream) {
    LOCK(ctx);
    if (!ctx->l2_flush) {
        ctx->l2_flush_bytes = (size_t)256 << 20; /* twice the 126 MB L2 */
        ctx->l2_flush = ctx->mem.alloc_raw(ctx->l2_flush_bytes);
        if (!ctx->l2_flush) return fail(ctx, ACCB_ENOMEM, "cannot allocate the L2 flush buffer");
    }
    static unsigned tag = 0;
    flush_l2_kernel<<<ctx->sm_count * 8, 256, 0, (cudaStream_t)stream>>>((uint4 *)ctx->l2_flush,
                                                                        (long long)(ctx->l2_flush_bytes / 16), ++tag);
    return check_cuda(ctx, cudaGetLastError(), "flush_l2");
}

} /* extern "C" */

namespace accb_rt {
int rebase_offsets(accb_context *ctx, cudaStream_t s, int *dst, const int *src, long long n) {
    if (n <= 0) return ACCB_OK;
    const int grid = (int)std::min<long long>((n + 255) / 256, 1024);
    rebase_i32<<<grid, 256, 0, s>>>(dst, src, n);
    ctx->launches++;
    return check_cuda(ctx, cudaGetLastError(), "rebase_i32");
}
}  // namespace accb_rt
