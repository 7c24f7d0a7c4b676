/*
 * refskel.cu -- the reference's OWN skeleton algorithms, restated as plain CUDA
 * for sm_100a, as a like-for-like GPU baseline.
 *
 * accelerate-cuda cannot be built or run here (no GHC; its device headers do
 * not compile under CUDA 12), so "how fast would the reference's design be on
 * this GPU" is answered by writing out what its code generator would emit for
 * the six benchmark programs, with the scalar functions fixed:
 *
 *   map            one element per thread per trip, grid-stride, scalar 4-byte
 *                  accesses (CodeGen/Mapping.hs:39-78)
 *   foldAll        strided per-thread accumulation in the element type, a
 *                  shared-memory tree per block, then the SAME kernel relaunched
 *                  on the partials until one block remains, the seed applied by
 *                  the last launch (CodeGen/Reduction.hs:87-215, 648-699;
 *                  Execute.hs:291-318)
 *   fold (rows)    one block per row, block-strided scalar loads, shared-memory
 *                  tree per row (CodeGen/Reduction.hs:221-367)
 *   scanl          three launches: per-interval totals with a Hillis-Steele
 *                  block scan per chunk, a one-block scan of the totals, and a
 *                  second pass over the input that carries the interval prefix
 *                  (CodeGen/PrefixSum.hs:200-533; Execute.hs:364-392)
 *   permute        scatter-combine under one spin lock per destination element:
 *                  atomicExch to take and release, __threadfence after every
 *                  attempt (CodeGen/IndexSpace.hs:160-303; lock array cleared
 *                  and defaults copied per call, Execute.hs:396-408)
 *   stencil        one output element per thread per trip, div/mod index
 *                  recovery, nine scalar global loads, a warp vote choosing the
 *                  unclamped path for interior warps (CodeGen/Stencil.hs:55-114)
 *
 * Launch geometry follows Analysis/Launch.hs:42-128: the block size of best
 * occupancy (a power of two for folds, the largest for scans), the grid capped
 * at SMs x resident blocks, one element per thread per trip.
 *
 * What is deliberately modern, because the original forms are not valid on
 * this architecture: warp-level steps use __syncwarp / __all_sync instead of
 * relying on lock-step warps; the locked read-modify-write goes through
 * volatile accesses; the lock spin is bounded (an error word is raised if it
 * ever runs out).  None of this code is used by the library; bench.py times it
 * beside the library's kernels.
 */
#include <cuda_runtime.h>

#include <algorithm>
#include <cstdint>
#include <cstdio>

namespace {

int g_sms = 0;

int sms() {
    if (!g_sms) {
        int dev = 0;
        cudaGetDevice(&dev);
        cudaDeviceGetAttribute(&g_sms, cudaDevAttrMultiProcessorCount, dev);
    }
    return g_sms;
}

enum Strategy { DEC_WARP, INC_POW2, LARGEST };

/* block size and resident blocks per SM in the manner of blockSize / determineOccupancy */
template <class K>
void configure(K kernel, Strategy how, size_t smem_per_thread, int *cta, int *per_sm) {
    int best_cta = 32, best_threads = 0, best_blocks = 1;
    /* the reference keeps the LAST candidate of maximal occupancy in list order: the smallest block
     * for the decreasing list, the largest for the increasing ones */
    auto consider = [&](int c) {
        int nb = 0;
        if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&nb, kernel, c, smem_per_thread * c) != cudaSuccess) return;
        const int threads = nb * c;
        if (nb > 0 && threads >= best_threads) {
            best_threads = threads;
            best_cta = c;
            best_blocks = nb;
        }
    };
    if (how == INC_POW2) {
        for (int c = 32; c <= 1024; c *= 2) consider(c);
    } else if (how == LARGEST) {
        for (int c = 32; c <= 1024; c += 32) consider(c);
    } else {
        for (int c = 1024; c >= 32; c -= 32) consider(c);
    }
    *cta = best_cta;
    *per_sm = best_blocks;
}

int grid_for(long long n, int cta, int per_sm) {
    const long long want = std::max(1LL, (n + cta - 1) / cta);
    return (int)std::min<long long>(want, (long long)sms() * per_sm);
}

/* -------------------------------------------------------------------- map */
__device__ __forceinline__ float cnd(float d) { return 0.5f + 0.5f * erff(0.70710678f * d); }

__global__ void map_blackscholes(const float *__restrict__ spot, const float *__restrict__ strike,
                                 const float *__restrict__ years, float *__restrict__ call, float *__restrict__ put,
                                 int shapeSize) {
    const int gridSize = blockDim.x * gridDim.x;
    for (int ix = blockDim.x * blockIdx.x + threadIdx.x; ix < shapeSize; ix += gridSize) {
        const float s = spot[ix], k = strike[ix], t = years[ix];
        const float r = 0.02f, v = 0.30f;
        const float sq = sqrtf(t), vsq = v * sq;
        const float d1 = (logf(s / k) + (r + 0.5f * v * v) * t) / vsq;
        const float d2 = d1 - vsq;
        const float kexp = k * expf(-r * t);
        const float n1 = cnd(d1), n2 = cnd(d2);
        call[ix] = s * n1 - kexp * n2;
        put[ix] = kexp * (1.0f - n2) - s * (1.0f - n1);
    }
}

/* ------------------------------------------------------------------ folds */
/* tree reduction of sdata[0..n) (n <= blockDim.x); the result ends in y of thread 0 */
__device__ __forceinline__ void reduce_block_tree(float *sdata, float &y, int n) {
    for (int i = 512; i > 32; i >>= 1) {
        if (blockDim.x > i) { /* the reference unrolls these steps over the largest block size */
            __syncthreads();
            if (threadIdx.x + i < n) y = y + sdata[threadIdx.x + i];
            __syncthreads();
            sdata[threadIdx.x] = y;
        }
    }
    __syncthreads();
    if (threadIdx.x < 32) {
        for (int i = 32; i > 0; i >>= 1) {
            if (threadIdx.x + i < n) y = y + sdata[threadIdx.x + i];
            __syncwarp();
            sdata[threadIdx.x] = y;
            __syncwarp();
        }
    }
}

/* foldAll (+) seed (zipWith (*) xs ys) when ys != null, else over xs alone (the recursive step) */
__global__ void fold_all(const float *__restrict__ xs, const float *__restrict__ ys, float *__restrict__ out,
                         int shapeSize, float seed) {
    extern __shared__ float sdata[];
    const int gridSize = blockDim.x * gridDim.x;
    int ix = blockDim.x * blockIdx.x + threadIdx.x;
    float y = 0.0f;
    if (ix < shapeSize) {
        y = ys ? xs[ix] * ys[ix] : xs[ix];
        for (ix += gridSize; ix < shapeSize; ix += gridSize) y = y + (ys ? xs[ix] * ys[ix] : xs[ix]);
    }
    sdata[threadIdx.x] = y;
    ix = min(shapeSize - (int)(blockIdx.x * blockDim.x), (int)blockDim.x);
    reduce_block_tree(sdata, y, ix);
    if (threadIdx.x == 0) {
        if (shapeSize > 0) {
            if (gridDim.x == 1) y = y + seed;
            out[blockIdx.x] = y;
        } else {
            out[blockIdx.x] = seed;
        }
    }
}

/* fold (+) seed over the rows of a matrix: one block per row */
__global__ void fold_rows(const float *__restrict__ in, float *__restrict__ out, int numIntervals, int intervalSize,
                          float seed) {
    extern __shared__ float sdata[];
    for (int seg = blockIdx.x; seg < numIntervals; seg += gridDim.x) {
        const int start = seg * intervalSize, end = start + intervalSize;
        const int n = min(end - start, (int)blockDim.x);
        if ((int)threadIdx.x >= n) return;
        float y = 0.0f;
        int ix = start - (start & 31);
        if (ix == start || intervalSize > (int)blockDim.x) {
            ix += threadIdx.x;
            if (ix >= start) y = in[ix];
            if (ix + (int)blockDim.x < end) {
                const float x = in[ix + blockDim.x];
                y = ix >= start ? y + x : x;
            }
            for (ix += 2 * blockDim.x; ix < end; ix += blockDim.x) y = y + in[ix];
        } else {
            y = in[start + threadIdx.x];
        }
        sdata[threadIdx.x] = y;
        reduce_block_tree(sdata, y, n);
        if (threadIdx.x == 0) out[seg] = y + seed;
        __syncthreads(); /* sdata is reused by the next row */
    }
}

/* ------------------------------------------------------------------- scan */
/* Hillis-Steele inclusive scan of one value per thread through shared memory */
__device__ __forceinline__ void scan_block_tree(int *sdata, int &x) {
    for (int n = 1; n <= 1024; n <<= 1) {
        if ((int)blockDim.x > n) {
            if ((int)threadIdx.x >= n) x = sdata[threadIdx.x - n] + x;
            __syncthreads();
            sdata[threadIdx.x] = x;
            __syncthreads();
        }
    }
}

/* up-sweep: the total of every interval */
__global__ void scanl_up(const int *__restrict__ in, int *__restrict__ blk, int shapeSize) {
    extern __shared__ int sscan[];
    const int intervalSize = (shapeSize + gridDim.x - 1) / gridDim.x;
    const int start = blockIdx.x * intervalSize;
    const int end = min(start + intervalSize, shapeSize);
    const int numElements = end - start;
    int carryIn = 0, y = 0;
    for (int seg = threadIdx.x; seg < numElements; seg += blockDim.x) {
        int x = in[start + seg];
        if (threadIdx.x == 0 && carryIn) x = y + x;
        sscan[threadIdx.x] = x;
        __syncthreads();
        scan_block_tree(sscan, x);
        if (threadIdx.x == 0) {
            const int last = min(numElements - seg, (int)blockDim.x) - 1;
            y = sscan[last];
        }
        carryIn = 1;
        __syncthreads(); /* sscan is rewritten by the next chunk */
    }
    if (threadIdx.x == 0) blk[blockIdx.x] = y;
}

/* exclusive scan with a seed: the totals pass (one block, in place over blk) and the final pass
 * (carry-in from blk when there is more than one block) are the same kernel in the reference */
__global__ void scanl_main(const int *in, int *out, const int *blk, int *sum, int shapeSize, int seed) {
    extern __shared__ int sscan[];
    const int intervalSize = (shapeSize + gridDim.x - 1) / gridDim.x;
    int z = 0;
    if (threadIdx.x == 0) z = gridDim.x > 1 ? blk[blockIdx.x] : seed;
    const int start = blockIdx.x * intervalSize;
    const int end = min(start + intervalSize, shapeSize);
    const int numElements = end - start;
    for (int seg = threadIdx.x; seg < numElements; seg += blockDim.x) {
        const int ix = start + seg;
        int x = in[ix];
        if (threadIdx.x == 0) x = z + x;
        sscan[threadIdx.x] = x;
        __syncthreads();
        scan_block_tree(sscan, x);
        x = threadIdx.x == 0 ? z : sscan[threadIdx.x - 1];
        out[ix] = x;
        if (threadIdx.x == 0) {
            const int last = min(numElements - seg, (int)blockDim.x) - 1;
            z = sscan[last];
        }
        __syncthreads();
    }
    if (threadIdx.x == 0 && blockIdx.x == gridDim.x - 1) sum[0] = z;
}

/* ---------------------------------------------------------------- permute */
#define REFSKEL_LOCK_SPIN_LIMIT (1 << 24)

/* out[keys[ix]] += 1 under a spin lock per destination element */
__global__ void permute_histogram(const int *__restrict__ keys, int *out, int *lock, int shapeSize, unsigned *err) {
    const int gridSize = blockDim.x * gridDim.x;
    for (int ix = blockDim.x * blockIdx.x + threadIdx.x; ix < shapeSize; ix += gridSize) {
        const int jx = keys[ix];
        if (jx == -1) continue; /* the `ignore` index */
        const int x = 1;
        int done = 0, tries = 0;
        do {
            int *addr = &lock[jx];
            if (atomicExch(addr, 1) == 0) {
                volatile int *slot = out + jx;
                const int y = *slot;
                *slot = x + y;
                done = 1;
                __threadfence(); /* the update is visible before the lock is seen free */
                atomicExch(addr, 0);
            }
            __threadfence();
            if (!done && ++tries > REFSKEL_LOCK_SPIN_LIMIT) { /* bounded: give up and say so */
                atomicExch(err, 1u);
                done = 1;
            }
        } while (done == 0);
    }
}

/* ---------------------------------------------------------------- stencil */
__device__ __forceinline__ int clampi(int i, int sz) { return max(0, min(i, sz - 1)); }

/* 3x3 blur, Clamp boundary, one element per thread per trip */
__global__ void stencil_blur(const float *__restrict__ in, float *__restrict__ out, int h, int w) {
    const int shapeSize = h * w;
    const int gridSize = blockDim.x * gridDim.x;
    /* the trip count is the same for every lane of a warp except in the last trip, where the
     * vote below is restricted to the lanes still in range */
    for (int ix = blockDim.x * blockIdx.x + threadIdx.x; ix < shapeSize; ix += gridSize) {
        const int y = ix / w, x = ix - y * w;
        const bool inside = y >= 1 && y < h - 1 && x >= 1 && x < w - 1;
        float t[3][3];
        if (__all_sync(__activemask(), inside)) {
#pragma unroll
            for (int dy = -1; dy <= 1; ++dy)
#pragma unroll
                for (int dx = -1; dx <= 1; ++dx) t[dy + 1][dx + 1] = in[(y + dy) * w + (x + dx)];
        } else {
#pragma unroll
            for (int dy = -1; dy <= 1; ++dy)
#pragma unroll
                for (int dx = -1; dx <= 1; ++dx) t[dy + 1][dx + 1] = in[clampi(y + dy, h) * w + clampi(x + dx, w)];
        }
        out[ix] = 0.0625f * t[0][0] + 0.125f * t[0][1] + 0.0625f * t[0][2] + 0.125f * t[1][0] + 0.25f * t[1][1] +
                  0.125f * t[1][2] + 0.0625f * t[2][0] + 0.125f * t[2][1] + 0.0625f * t[2][2];
    }
}

int last_error(const char *what) {
    const cudaError_t e = cudaGetLastError();
    if (e == cudaSuccess) return 0;
    fprintf(stderr, "refskel: %s: %s\n", what, cudaGetErrorString(e));
    return 1;
}

}  // namespace

extern "C" {

/* Every function enqueues its launches on `stream` and returns 0, or 1 after printing a CUDA error.
 * Sizes are C ints as in the reference's kernels (array sizes below 2^31). */

int refskel_map_blackscholes(const float *spot, const float *strike, const float *years, float *call, float *put,
                             int n, cudaStream_t stream) {
    static int cta = 0, per_sm = 0;
    if (!cta) configure(map_blackscholes, DEC_WARP, 0, &cta, &per_sm);
    map_blackscholes<<<grid_for(n, cta, per_sm), cta, 0, stream>>>(spot, strike, years, call, put, n);
    return last_error("map");
}

/* partials: scratch of at least 2 x SMs x 32 floats; launches until one block is left */
int refskel_dot(const float *xs, const float *ys, int n, float seed, float *partials, float *out,
                cudaStream_t stream) {
    static int cta = 0, per_sm = 0;
    if (!cta) configure(fold_all, INC_POW2, sizeof(float), &cta, &per_sm);
    int size = n;
    const float *a = xs, *b = ys;
    float *bufs[2] = {partials, partials + (size_t)sms() * 32};
    int flip = 0;
    for (;;) {
        const int grid = grid_for(size, cta, per_sm);
        float *dst = grid == 1 ? out : bufs[flip];
        fold_all<<<grid, cta, cta * sizeof(float), stream>>>(a, b, dst, size, seed);
        if (last_error("foldAll")) return 1;
        if (grid == 1) return 0;
        a = dst;
        b = nullptr;
        size = grid;
        flip ^= 1;
    }
}

int refskel_fold_rows(const float *in, int rows, int cols, float seed, float *out, cudaStream_t stream) {
    static int cta = 0, per_sm = 0;
    if (!cta) configure(fold_rows, INC_POW2, sizeof(float), &cta, &per_sm);
    const int grid = (int)std::min<long long>(std::max(1, rows), (long long)sms() * per_sm);
    fold_rows<<<grid, cta, cta * sizeof(float), stream>>>(in, out, rows, cols, seed);
    return last_error("fold");
}

/* out has n + 1 elements (the total goes last); blk: scratch of at least SMs x 32 ints */
int refskel_scanl(const int *in, int n, int seed, int *out, int *blk, cudaStream_t stream) {
    static int cta = 0, per_sm = 0;
    if (!cta) configure(scanl_main, LARGEST, sizeof(int), &cta, &per_sm);
    const int intervals = grid_for(n, cta, per_sm);
    if (intervals > 1) {
        if (intervals > cta) { /* the totals must fit one block, as in the reference */
            fprintf(stderr, "refskel: %d intervals do not fit a block of %d\n", intervals, cta);
            return 1;
        }
        scanl_up<<<intervals, cta, cta * sizeof(int), stream>>>(in, blk, n);
        if (last_error("scanlUp")) return 1;
        /* the totals are scanned in place by one block; their sum lands in out[n] and is
         * overwritten with the same value by the final pass */
        scanl_main<<<grid_for(intervals, cta, per_sm), cta, cta * sizeof(int), stream>>>(blk, blk, blk, out + n,
                                                                                         intervals, seed);
        if (last_error("scanlUp2")) return 1;
    }
    scanl_main<<<intervals, cta, cta * sizeof(int), stream>>>(in, out, blk, out + n, n, seed);
    return last_error("scanl");
}

/* out: nbins ints; lock: nbins ints of scratch; err: one word, raised if a lock wait ran out */
int refskel_histogram(const int *keys, int n, const int *defaults, int nbins, int *out, int *lock, unsigned *err,
                      cudaStream_t stream) {
    static int cta = 0, per_sm = 0;
    if (!cta) configure(permute_histogram, DEC_WARP, 0, &cta, &per_sm);
    if (cudaMemsetAsync(lock, 0, (size_t)nbins * sizeof(int), stream) != cudaSuccess) return last_error("memset");
    if (cudaMemcpyAsync(out, defaults, (size_t)nbins * sizeof(int), cudaMemcpyDeviceToDevice, stream) != cudaSuccess)
        return last_error("copy defaults");
    permute_histogram<<<grid_for(n, cta, per_sm), cta, 0, stream>>>(keys, out, lock, n, err);
    return last_error("permute");
}

int refskel_stencil_blur(const float *in, float *out, int h, int w, cudaStream_t stream) {
    static int cta = 0, per_sm = 0;
    if (!cta) configure(stencil_blur, DEC_WARP, 0, &cta, &per_sm);
    stencil_blur<<<grid_for((long long)h * w, cta, per_sm), cta, 0, stream>>>(in, out, h, w);
    return last_error("stencil");
}

/* launch geometry actually used, for the report: which = 0 map, 1 foldAll, 2 fold, 3 scan, 4 permute, 5 stencil */
int refskel_config(int which, int *cta, int *per_sm) {
    switch (which) {
        case 0: configure(map_blackscholes, DEC_WARP, 0, cta, per_sm); return 0;
        case 1: configure(fold_all, INC_POW2, sizeof(float), cta, per_sm); return 0;
        case 2: configure(fold_rows, INC_POW2, sizeof(float), cta, per_sm); return 0;
        case 3: configure(scanl_main, LARGEST, sizeof(int), cta, per_sm); return 0;
        case 4: configure(permute_histogram, DEC_WARP, 0, cta, per_sm); return 0;
        case 5: configure(stencil_blur, DEC_WARP, 0, cta, per_sm); return 0;
    }
    return 1;
}

}  // extern "C"
