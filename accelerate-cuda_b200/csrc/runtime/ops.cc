/*
 * ops.cc -- launch analysis and the per-skeleton host drivers.
 *
 * Replaces Data/Array/Accelerate/CUDA/Analysis/Launch.hs:42-172 (block size,
 * grid size, shared memory) and the drivers executeOp, foldCore/foldRec,
 * foldSegOp, scanOp/scan1Op/scan'Op/scanCore, permuteOp, stencilOp and
 * stencil2Op of Data/Array/Accelerate/CUDA/Execute.hs:264-450 with the
 * marshalling and launch code of Execute.hs:823-982.
 *
 * Launch policy.  The reference picks the block size from an occupancy
 * search and caps the grid at SMs x resident blocks (Launch.hs:42-55) with one
 * element per thread per trip.  Here the block size is fixed by each skeleton
 * (it fixes the tile shape), the grid is SMs x resident blocks for the
 * persistent kernels (map, folds, permute) and one block per tile for the
 * ticketed scan and the stencil, and the resident-block count comes from the
 * driver's occupancy calculator for the compiled kernel.
 */
#include <algorithm>
#include <cstdlib>

#include "common.h"

namespace accb_rt {

int occupancy(accb_context *ctx, CUfunction fn, int block, size_t smem, int *blocks_per_sm) {
    /* asked on every launch: remember the answer per (entry point, block size, dynamic shared memory), as
     * the reference keeps the occupancy with each compiled kernel (CUDA/AST.hs:51-59) */
    const auto key = std::make_tuple(fn, block, smem);
    auto it = ctx->occupancy_cache.find(key);
    if (it != ctx->occupancy_cache.end()) {
        *blocks_per_sm = it->second;
        return ACCB_OK;
    }
    int n = 0;
    int st = check_cu(ctx, driver().OccupancyMaxActiveBlocksPerMultiprocessor(&n, fn, block, smem),
                      "cuOccupancyMaxActiveBlocksPerMultiprocessor");
    if (st != ACCB_OK) return st;
    *blocks_per_sm = std::max(1, n);
    ctx->occupancy_cache[key] = *blocks_per_sm;
    return ACCB_OK;
}

int launch(accb_context *ctx, CUfunction fn, const char *name, int grid, int block, size_t smem, cudaStream_t stream,
           const accb_kparams &p, bool prefer_smem, void *extra1, void *extra2) {
    void *args[] = {const_cast<accb_kparams *>(&p), extra1, extra2}; /* entries with tensor maps take them after the block */
    if (ctx->trace_exec)
        fprintf(stderr, "[accb exec] %s<<<%d,%d,%zu>>> n=%lld\n", name, grid, block, smem, p.n);
    /* an entry that stages tiles in dynamic shared memory wants several of them per SM at the
     * expense of L1; the other entries of the same module keep the default split */
    if (smem > 0 && prefer_smem && ctx->carveout_set.insert(fn).second)
        driver().FuncSetAttribute(fn, CU_FUNC_ATTRIBUTE_PREFERRED_SHARED_MEMORY_CARVEOUT, 100);
    int st = check_cu(ctx, driver().LaunchKernel(fn, (unsigned)grid, 1, 1, (unsigned)block, 1, 1, (unsigned)smem,
                                                 (CUstream)stream, args, nullptr),
                      name);
    if (st == ACCB_OK) ctx->launches++;
    return st;
}

int launch_dependent(accb_context *ctx, CUfunction fn, const char *name, int grid, int block, cudaStream_t stream,
                     const accb_kparams &p) {
    cudaStreamCaptureStatus cap = cudaStreamCaptureStatusNone;
    cudaStreamIsCapturing(stream, &cap);
    if (!driver().LaunchKernelEx || cap != cudaStreamCaptureStatusNone) return launch(ctx, fn, name, grid, block, 0, stream, p);
    void *args[] = {const_cast<accb_kparams *>(&p)};
    if (ctx->trace_exec) fprintf(stderr, "[accb exec] %s<<<%d,%d>>> (dependent) n=%lld\n", name, grid, block, p.n);
    CUlaunchAttribute attr;
    memset(&attr, 0, sizeof attr);
    attr.id = CU_LAUNCH_ATTRIBUTE_PROGRAMMATIC_STREAM_SERIALIZATION;
    attr.value.programmaticStreamSerializationAllowed = 1;
    CUlaunchConfig cfg;
    memset(&cfg, 0, sizeof cfg);
    cfg.gridDimX = (unsigned)grid;
    cfg.gridDimY = cfg.gridDimZ = 1;
    cfg.blockDimX = (unsigned)block;
    cfg.blockDimY = cfg.blockDimZ = 1;
    cfg.hStream = (CUstream)stream;
    cfg.attrs = &attr;
    cfg.numAttrs = 1;
    int st = check_cu(ctx, driver().LaunchKernelEx(&cfg, fn, args, nullptr), name);
    if (st == ACCB_OK) ctx->launches++;
    return st;
}

static bool aligned16(const void *p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

/* environment arrays -> slots, shapes, alignment flag */
static int fill_env(accb_context *ctx, accb_kparams &p, const accb_array *env, int nenv) {
    if (nenv < 0 || nenv > ACCB_MAX_ARR) return fail(ctx, ACCB_EINVAL, "too many environment arrays (%d)", nenv);
    if (nenv > 0 && !env) return fail(ctx, ACCB_EINVAL, "null environment");
    int slot = 0;
    bool vec = true;
    for (int a = 0; a < nenv; ++a) {
        if (env[a].rank < 0 || env[a].rank > ACCB_MAX_RANK || env[a].ncomp < 0 || env[a].ncomp > ACCB_ARRAY_MAX_COMP)
            return fail(ctx, ACCB_EINVAL, "environment array %d: bad rank or component count", a);
        p.in_first[a] = slot;
        for (int d = 0; d < env[a].rank; ++d) p.in_shape[a][d] = env[a].shape[d];
        for (int c = 0; c < env[a].ncomp; ++c) {
            if (slot >= ACCB_MAX_IN) return fail(ctx, ACCB_EINVAL, "more than %d input components", ACCB_MAX_IN);
            p.in[slot++] = env[a].ptr[c];
            vec = vec && aligned16(env[a].ptr[c]);
        }
    }
    if (vec) p.flags |= ACCB_F_VEC;
    return ACCB_OK;
}

static int fill_out(accb_context *ctx, accb_kparams &p, const accb_array *out, int first_slot = 0) {
    if (!out) return fail(ctx, ACCB_EINVAL, "null output array");
    if (out->ncomp < 1 || first_slot + out->ncomp > ACCB_MAX_OUT)
        return fail(ctx, ACCB_EINVAL, "bad output component count %d", out->ncomp);
    for (int c = 0; c < out->ncomp; ++c) {
        if (!out->ptr[c]) return fail(ctx, ACCB_EINVAL, "null output pointer");
        p.out[first_slot + c] = out->ptr[c];
        if (first_slot == 0 && !aligned16(out->ptr[c])) p.flags &= ~ACCB_F_VEC;
    }
    if (first_slot == 0)
        for (int d = 0; d < out->rank && d < ACCB_MAX_RANK; ++d) p.out_shape[d] = out->shape[d];
    return ACCB_OK;
}

static long long array_size(const accb_array *a) {
    long long n = 1;
    for (int d = 0; d < a->rank; ++d) n *= a->shape[d];
    return n;
}

static int fill_scalars(accb_context *ctx, accb_kparams &p, const void *s, size_t bytes) {
    if (bytes > ACCB_SCALAR_BYTES) return fail(ctx, ACCB_EINVAL, "scalar block of %zu bytes exceeds %d", bytes, ACCB_SCALAR_BYTES);
    if (bytes && !s) return fail(ctx, ACCB_EINVAL, "null scalar block");
    if (bytes) memcpy(p.scalars, s, bytes);
    return ACCB_OK;
}

static int grow(accb_context *ctx, void **buf, size_t *have, size_t want, cudaStream_t stream, bool zero) {
    if (*have >= want) return ACCB_OK;
    /* the old buffer may still be read by work enqueued earlier on this stream */
    int st = check_cuda(ctx, cudaStreamSynchronize(stream), "cudaStreamSynchronize");
    if (st != ACCB_OK) return st;
    ctx->buffer_generation++; /* recorded graphs that name the old buffer are stale now */
    if (*buf) cudaFree(*buf);
    *buf = nullptr;
    *have = 0;
    const size_t bytes = std::max(want, (size_t)1 << 20);
    void *p = ctx->mem.alloc_raw(bytes);
    if (!p) return fail(ctx, ACCB_ENOMEM, "device out of memory allocating %zu bytes of scratch", bytes);
    *buf = p;
    *have = bytes;
    if (zero) return check_cuda(ctx, cudaMemsetAsync(p, 0, bytes, stream), "cudaMemsetAsync");
    return ACCB_OK;
}

struct Prep {
    CUfunction fn = nullptr;
    KernelMeta meta;
    int block = 0;
    int per_sm = 1;
};

static int prepare(accb_context *ctx, accb_kernel *k, const char *entry, size_t smem, Prep *pr) {
    if (!k) return fail(ctx, ACCB_EINVAL, "null kernel");
    int st = get_function(ctx, k, entry, &pr->fn, &pr->meta);
    if (st != ACCB_OK) return st;
    pr->block = pr->meta.v[1];
    if (pr->block <= 0) return fail(ctx, ACCB_EINVAL, "kernel %s carries no launch metadata", k->key.c_str());
    return occupancy(ctx, pr->fn, pr->block, smem, &pr->per_sm);
}

static int check_skeleton(accb_context *ctx, accb_kernel *k, std::initializer_list<int> ids, const char *what) {
    if (!k) return fail(ctx, ACCB_EINVAL, "null kernel");
    for (int id : ids)
        if (k->skeleton == id) return ACCB_OK;
    return fail(ctx, ACCB_EINVAL, "kernel %s was not built for the %s skeleton", k->key.c_str(), what);
}

static long long ceil_div(long long a, long long b) { return (a + b - 1) / b; }

/* Threads that share one range of `items` loads (vectors or scalars) when `units` ranges are
 * reduced: 4, 8, 16 or 32 lanes, or 256 (a block) once a range has at least `block_from` loads or
 * there are too few ranges to fill the GPU with warps. */
static int pick_group(long long items, long long units, long long block_from) {
    if (items >= block_from || (items >= 512 && units < 8192)) return 256;
    int g = 4;
    while (g < 32 && (long long)g * 8 < items) g *= 2;
    return g;
}

}  // namespace accb_rt

using namespace accb_rt;

#define LOCK(ctx)                                                   \
    if (!(ctx)) return fail(nullptr, ACCB_EINVAL, "null context"); \
    std::lock_guard<std::recursive_mutex> lock_((ctx)->mu);         \
    CtxGuard guard_(ctx)
#define TRY(expr)                     \
    do {                              \
        int st_ = (expr);             \
        if (st_ != ACCB_OK) return st_; \
    } while (0)

extern "C" {

int accb_launch_count(accb_context *ctx, unsigned long long *launches) {
    LOCK(ctx);
    if (launches) *launches = ctx->launches;
    return ACCB_OK;
}

int accb_launch_config(accb_context *ctx, accb_kernel *k, const char *entry, long long n, int *block, int *grid,
                       int *dynamic_smem) {
    LOCK(ctx);
    Prep pr;
    TRY(prepare(ctx, k, entry, 0, &pr));
    const long long per_block = (long long)pr.block * std::max(1, pr.meta.v[4]) * 4;
    const long long units = std::max(1LL, ceil_div(n, per_block));
    if (block) *block = pr.block;
    if (grid) *grid = (int)std::min<long long>(units, (long long)ctx->sm_count * pr.per_sm);
    if (dynamic_smem) *dynamic_smem = 0;
    return ACCB_OK;
}

/* ------------------------------------------------------------------ map */
int accb_map(accb_context *ctx, accb_kernel *k, accb_stream stream, const accb_array *env, int nenv,
             const void *scalars, size_t scalar_bytes, const accb_array *out) {
    return accb_map_at(ctx, k, stream, env, nenv, scalars, scalar_bytes, out, 0);
}

int accb_map_at(accb_context *ctx, accb_kernel *k, accb_stream stream, const accb_array *env, int nenv,
                const void *scalars, size_t scalar_bytes, const accb_array *out, long long index_base) {
    LOCK(ctx);
    TRY(check_skeleton(ctx, k, {SK_MAP}, "map"));
    if (!out) return fail(ctx, ACCB_EINVAL, "null output array");
    if (array_size(out) == 0) return ACCB_OK; /* nothing to compute; an empty array may have no storage */
    accb_kparams p;
    memset(&p, 0, sizeof p);
    TRY(fill_env(ctx, p, env, nenv));
    TRY(fill_out(ctx, p, out));
    TRY(fill_scalars(ctx, p, scalars, scalar_bytes));
    p.n = array_size(out);
    p.base = index_base;
    if (p.n == 0) return ACCB_OK;
    Prep pr;
    TRY(prepare(ctx, k, "map", 0, &pr));
    const long long units = ceil_div(p.n, (long long)pr.block * pr.meta.v[4] * 4);
    const int grid = (int)std::min<long long>(std::max(1LL, units), (long long)ctx->sm_count * pr.per_sm);
    return launch(ctx, pr.fn, "map", grid, pr.block, 0, (cudaStream_t)stream, p);
}

int accb_map_transposed(accb_context *ctx, accb_kernel *k, accb_stream stream, const accb_array *env, int nenv,
                        const void *scalars, size_t scalar_bytes, const accb_array *out) {
    LOCK(ctx);
    TRY(check_skeleton(ctx, k, {SK_MAP}, "map"));
    if (!out || out->rank != 2) return fail(ctx, ACCB_EINVAL, "the result of a transposed map is a matrix");
    if (array_size(out) == 0) return ACCB_OK;
    accb_kparams p;
    memset(&p, 0, sizeof p);
    TRY(fill_env(ctx, p, env, nenv));
    TRY(fill_out(ctx, p, out));
    TRY(fill_scalars(ctx, p, scalars, scalar_bytes));
    p.n = array_size(out);
    Prep pr;
    TRY(prepare(ctx, k, "map_transposed", 0, &pr));
    const size_t smem = (size_t)pr.meta.v[6];
    if (smem == 0) return fail(ctx, ACCB_EINVAL, "kernel %s reads no array element-wise: nothing to transpose", k->key.c_str());
    /* the element-wise inputs are out's shape transposed: out has shape[1] rows of shape[0] columns */
    const int H = out->shape[0], W = out->shape[1]; /* rows and columns of the sources */
    /* the arrays that hold the first In::size components (metadata slot 5) are the element-wise ones */
    for (int a = 0, slot = 0; a < nenv && slot < pr.meta.v[5]; slot += env[a].ncomp, ++a)
        if (env[a].rank != 2 || env[a].shape[0] != W || env[a].shape[1] != H)
            return fail(ctx, ACCB_EINVAL, "environment array %d is not the transposed shape of the result", a);
    p.ip[0] = H;
    p.ip[1] = W;
    if (ctx->tune.transpose_tma && driver().TensorMapEncodeTiled && pr.meta.v[8] == 1 && (p.flags & ACCB_F_VEC) && W % 4 == 0 && H % 4 == 0 && nenv >= 1 &&
        env[0].ncomp == 1 && out->ncomp == 1) {
        /* one 4-byte value in, one out: the copy engine moves the tiles, through a tensor map of either matrix
         * (64x64 tiles as two boxes of 32 columns, the hardware's 128-byte swizzle) */
        alignas(64) CUtensorMap tin, tout;
        const cuuint32_t box[2] = {32, 64}, ones[2] = {1, 1};
        const cuuint64_t din[2] = {(cuuint64_t)W, (cuuint64_t)H}, sin[1] = {(cuuint64_t)W * 4};
        const cuuint64_t dout[2] = {(cuuint64_t)H, (cuuint64_t)W}, sout[1] = {(cuuint64_t)H * 4};
        const Driver &d = driver();
        CUresult e1 = d.TensorMapEncodeTiled(&tin, CU_TENSOR_MAP_DATA_TYPE_UINT32, 2, env[0].ptr[0], din, sin, box, ones,
                                             CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                                             CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
        CUresult e2 = d.TensorMapEncodeTiled(&tout, CU_TENSOR_MAP_DATA_TYPE_UINT32, 2, out->ptr[0], dout, sout, box, ones,
                                             CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                                             CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
        if (e1 == CUDA_SUCCESS && e2 == CUDA_SUCCESS) {
            Prep pt;
            TRY(prepare(ctx, k, "map_transposed_tma", 0, &pt));
            StreamScratch *sc = scratch_for(ctx, (cudaStream_t)stream);
            if (!sc) return fail(ctx, ACCB_ENOMEM, "cannot allocate stream scratch");
            p.aux[1] = sc->words + 2; /* error word of the bounded wait for the copy */
            const long long tiles_tma = ceil_div(W, 64) * ceil_div(H, 64);
            if (tiles_tma > 0x7fffffffLL) return fail(ctx, ACCB_EINVAL, "matrix too large for one launch");
            return launch(ctx, pt.fn, "map_transposed_tma", (int)tiles_tma, pt.block, (size_t)pr.meta.v[9], (cudaStream_t)stream, p,
                          true, &tin, &tout);
        }
        /* a map the driver refuses (extents beyond its limits): the other form takes it */
    }
    const long long tiles = ceil_div(W, 64) * ceil_div(H, 64); /* kTransTile of map.cuh */
    TRY(occupancy(ctx, pr.fn, pr.block, smem, &pr.per_sm));
    const int grid = (int)std::min<long long>(tiles, (long long)ctx->sm_count * pr.per_sm);
    return launch(ctx, pr.fn, "map_transposed", grid, pr.block, smem, (cudaStream_t)stream, p);
}

/* ---------------------------------------------------------------- folds */
static int set_seed(accb_context *ctx, accb_kparams &p, const void *seed, size_t seed_bytes) {
    if (!seed) return ACCB_OK;
    TRY(fill_scalars(ctx, p, seed, seed_bytes));
    p.flags |= ACCB_F_HAS_SEED;
    return ACCB_OK;
}

int accb_fold_all(accb_context *ctx, accb_kernel *k, accb_stream stream, const accb_array *env, int nenv,
                  long long n, const void *seed, size_t seed_bytes, const accb_array *out) {
    return accb_fold_all_at(ctx, k, stream, env, nenv, n, seed, seed_bytes, out, 0, nullptr);
}

int accb_fold_all_at(accb_context *ctx, accb_kernel *k, accb_stream stream, const accb_array *env, int nenv,
                     long long n, const void *seed, size_t seed_bytes, const accb_array *out, long long index_base,
                     const void *carry) {
    LOCK(ctx);
    TRY(check_skeleton(ctx, k, {SK_FOLD_ALL}, "fold_all"));
    if (n < 0) return fail(ctx, ACCB_EINVAL, "negative size");
    if (n == 0 && !seed && !carry) return fail(ctx, ACCB_EBOUNDS, "fold1: empty array");
    accb_kparams p;
    memset(&p, 0, sizeof p);
    TRY(fill_env(ctx, p, env, nenv));
    TRY(fill_out(ctx, p, out));
    TRY(set_seed(ctx, p, seed, seed_bytes));
    p.n = n;
    Prep pr;
    TRY(prepare(ctx, k, "foldAll", 0, &pr));
    const long long quantum = (long long)pr.block * pr.meta.v[4] * 4;
    const int grid = (int)std::min<long long>(std::max(1LL, ceil_div(n, quantum)), (long long)ctx->sm_count * pr.per_sm);
    cudaStream_t s = (cudaStream_t)stream;
    StreamScratch *sc = scratch_for(ctx, s);
    if (!sc) return fail(ctx, ACCB_ENOMEM, "cannot allocate stream scratch");
    TRY(grow(ctx, &sc->partial, &sc->partial_bytes, (size_t)grid * std::max(8, pr.meta.v[2]), s, false));
    p.aux[0] = sc->partial;
    p.aux[1] = sc->words + 0;
    p.base = index_base;
    if (carry) {
        p.aux[2] = const_cast<void *>(carry);
        p.flags |= ACCB_F_CARRY;
    }
    return launch(ctx, pr.fn, "foldAll", grid, pr.block, 0, s, p);
}

int accb_fold_dim(accb_context *ctx, accb_kernel *k, accb_stream stream, const accb_array *env, int nenv,
                  long long rows, long long cols, const void *seed, size_t seed_bytes, const accb_array *out) {
    return accb_fold_dim_at(ctx, k, stream, env, nenv, rows, cols, seed, seed_bytes, out, 0);
}

int accb_fold_dim_at(accb_context *ctx, accb_kernel *k, accb_stream stream, const accb_array *env, int nenv,
                     long long rows, long long cols, const void *seed, size_t seed_bytes, const accb_array *out,
                     long long index_base) {
    LOCK(ctx);
    TRY(check_skeleton(ctx, k, {SK_FOLD_DIM}, "fold_dim"));
    if (rows < 0 || cols < 0) return fail(ctx, ACCB_EINVAL, "negative extent");
    if (cols == 0 && !seed) return fail(ctx, ACCB_EBOUNDS, "fold1: empty array");
    if (rows == 0) return ACCB_OK;
    accb_kparams p;
    memset(&p, 0, sizeof p);
    TRY(fill_env(ctx, p, env, nenv));
    TRY(fill_out(ctx, p, out));
    TRY(set_seed(ctx, p, seed, seed_bytes));
    p.n = rows * cols;
    p.base = index_base;
    p.ip[0] = rows;
    p.ip[1] = cols;
    /* threads per row (the reference always uses one block per row, Launch.hs:120): a whole block
     * for long rows, else an aligned group of 32 / 16 / 8 / 4 lanes sized so that a lane gets
     * about 8 vectors of the row */
    const int group = pick_group(cols % 4 == 0 ? cols / 4 : cols, rows, 2048);
    const char *entry = group > 32 ? "fold" : group == 32 ? "fold_warp" : group == 16 ? "fold_g16" : group == 8 ? "fold_g8" : "fold_g4";
    Prep pr;
    TRY(prepare(ctx, k, entry, 0, &pr));
    if (cols >= 1 && cols <= ctx->tune.fold_stage_max && rows * cols >= (1 << 16) && rows * cols < (1LL << 40) && pr.meta.v[6] > 0 &&
        (p.flags & ACCB_F_VEC) && !ctx->tune.fold_no_stage) {
        /* many short rows: a block stages a run of whole rows (the matrix read as one long
         * vector) in shared memory and every thread reduces whole rows */
        const size_t smem = (size_t)pr.meta.v[6];
        Prep ps;
        TRY(get_function(ctx, k, "fold_staged", &ps.fn, &ps.meta)); /* its block size is meta.v[5] */
        StreamScratch *sc = scratch_for(ctx, (cudaStream_t)stream);
        if (!sc) return fail(ctx, ACCB_ENOMEM, "cannot allocate stream scratch");
        const long long run = std::max(1LL, (ps.meta.v[3] - 16) / cols); /* rows per block */
        p.ip[0] = 1;
        p.ip[1] = rows * cols;
        p.ip[2] = rows;
        p.ip[3] = cols;
        p.ip[4] = run;
        p.aux[1] = sc->words + 2;
        return launch(ctx, ps.fn, "fold_staged", (int)ceil_div(rows, run), ps.meta.v[5], smem, (cudaStream_t)stream, p);
    }
    const long long resident = (long long)ctx->sm_count * pr.per_sm;
    const long long quantum = (long long)pr.block * pr.meta.v[4] * 4; /* elements a block takes per trip */
    if (group > 32 && rows <= kRowCounters && rows < 4 * resident && cols >= 8 * quantum) {
        /* too few rows to occupy the GPU evenly: cut every row into pieces, one block each, so
         * that there are many more pieces than resident blocks */
        long long pieces = std::min<long long>(ceil_div(16 * resident, rows), cols / (4 * quantum));
        const long long chunk = ceil_div(ceil_div(cols, pieces), quantum) * quantum;
        pieces = ceil_div(cols, chunk);
        TRY(prepare(ctx, k, "fold_split", 0, &pr));
        cudaStream_t s = (cudaStream_t)stream;
        StreamScratch *sc = scratch_for(ctx, s);
        if (!sc) return fail(ctx, ACCB_ENOMEM, "cannot allocate stream scratch");
        TRY(grow(ctx, &sc->partial, &sc->partial_bytes, (size_t)(rows * pieces) * std::max(8, pr.meta.v[2]), s, false));
        p.ip[2] = pieces;
        p.ip[3] = chunk;
        p.aux[0] = sc->partial;
        p.aux[1] = sc->words + kRowCounterBase;
        const int grid = (int)std::min<long long>(rows * pieces, (long long)ctx->sm_count * pr.per_sm);
        return launch(ctx, pr.fn, "fold_split", grid, pr.block, 0, s, p);
    }
    const long long units = ceil_div(rows, pr.block / std::min(group, pr.block));
    const int grid = (int)std::min<long long>(std::max(1LL, units), (long long)ctx->sm_count * pr.per_sm);
    return launch(ctx, pr.fn, entry, grid, pr.block, 0, (cudaStream_t)stream, p);
}

int accb_fold_seg(accb_context *ctx, accb_kernel *k, accb_stream stream, const accb_array *env, int nenv,
                  long long rows, long long cols, const int *offsets, long long nseg, const void *seed,
                  size_t seed_bytes, const accb_array *out) {
    LOCK(ctx);
    TRY(check_skeleton(ctx, k, {SK_FOLD_SEG}, "fold_seg"));
    if (rows < 0 || cols < 0 || nseg < 0) return fail(ctx, ACCB_EINVAL, "negative extent");
    if (!offsets) return fail(ctx, ACCB_EINVAL, "null segment offsets");
    if (rows * nseg == 0) return ACCB_OK;
    accb_kparams p;
    memset(&p, 0, sizeof p);
    TRY(fill_env(ctx, p, env, nenv));
    TRY(fill_out(ctx, p, out));
    TRY(set_seed(ctx, p, seed, seed_bytes));
    p.n = rows * cols;
    p.ip[0] = rows;
    p.ip[1] = cols;
    p.ip[2] = nseg;
    p.aux[0] = const_cast<int *>(offsets);
    /* the reference gives every segment one warp (Launch.hs:118); here the group follows the
     * average segment length (accesses are scalar, so a lane should get about 8 elements) */
    const long long avg = cols / std::max(1LL, nseg);
    const int group = pick_group(avg, rows * nseg, 8192);
    const char *entry = group > 32 ? "foldSeg_block" : group == 32 ? "foldSeg" : group == 16 ? "foldSeg_g16" : group == 8 ? "foldSeg_g8" : "foldSeg_g4";
    Prep pr;
    TRY(prepare(ctx, k, entry, 0, &pr));
    /* Segments far longer than the rest (64 K elements where a thread, a warp or a few lanes own a segment, 1 M
     * where a block does) go on a list, and a second launch reduces them with all blocks; without it one such
     * segment keeps a single warp or block busy long after the launch would have ended.  Only sources of 16 M
     * elements and more get the second launch (it costs about three microseconds when the list stays empty), and
     * smaller ones of at least 1 M when a block owns a segment and there are too few segments to fill the GPU. */
    cudaStream_t s = (cudaStream_t)stream;
    StreamScratch *sc = scratch_for(ctx, s);
    if (!sc) return fail(ctx, ACCB_ENOMEM, "cannot allocate stream scratch");
    const long long piece = pr.meta.v[7];
    /* few segments under the block-per-segment form: the blocks cannot fill the GPU, every long segment is worth handing over */
    const bool starved = group > 32 && rows * nseg < 4LL * ctx->sm_count * pr.per_sm;
    const bool defer = !ctx->tune.foldseg_no_defer && piece > 0 && (cols >= (1LL << 24) || (starved && cols >= (1LL << 20)));
    /* everything that can fail is done before the first launch: a list left behind by a launch whose second half
     * never ran would be reduced, with the wrong arrays, by the next foldSeg on this stream */
    Prep pd;
    if (defer) {
        TRY(prepare(ctx, k, "foldSeg_deferred", 0, &pd));
        /* a listed segment of n elements has at most n / piece + 1 pieces */
        const size_t parts = (size_t)(rows * cols / piece) + ACCB_FOLD_DEFER_MAX;
        TRY(grow(ctx, &sc->partial, &sc->partial_bytes, parts * std::max(8, pr.meta.v[2]), s, false));
    }
    auto second_launch = [&](int st) {
        if (st != ACCB_OK || !defer) return st;
        accb_kparams q = p;
        q.aux[1] = sc->partial;
        st = launch_dependent(ctx, pd.fn, "foldSeg_deferred", ctx->sm_count * pd.per_sm, pd.block, s, q);
        if (st != ACCB_OK) cudaMemsetAsync(sc->words + kDeferredBase, 0, 2 * sizeof(unsigned), s); /* drop the list */
        return st;
    };
    if (defer) {
        p.ip[6] = (group > 32 && !starved) ? (1LL << 20) : (1LL << 16);
        p.aux[2] = sc->words + kDeferredBase;
    }
    if (avg <= ctx->tune.foldseg_stage_max && rows * nseg >= 4096 && (rows == 1 || cols % 16 == 0) && pr.meta.v[6] > 0 &&
        (p.flags & ACCB_F_VEC)) {
        /* short segments: a block stages a run of consecutive segments in shared memory and every
         * thread reduces whole segments; the run is sized to fill 3/4 of the window on average */
        const size_t smem = (size_t)pr.meta.v[6];
        Prep ps;
        TRY(get_function(ctx, k, "foldSeg_staged", &ps.fn, &ps.meta)); /* its block size is meta.v[5] */
        if (defer) p.ip[6] = 1LL << 16;
        /* a run that overflows the window reads its last segments from global memory, so aim high */
        const long long fill = ctx->tune.foldseg_fill8;
        const long long run =
            std::min<long long>(std::max(1LL, (ps.meta.v[3] - 32) * fill / 8 / std::max(1LL, avg)), 16LL * ps.meta.v[5]);
        /* lanes per segment: a thread takes whole segments of up to ~100 elements; longer ones are shared by
         * 8 lanes so that the few segments of a window still occupy the block */
        const long long lanes = ctx->tune.foldseg_lanes > 0 ? ctx->tune.foldseg_lanes : (avg <= 112 ? 1 : 8);
        p.ip[4] = run;
        p.ip[5] = lanes;
        p.aux[1] = sc->words + 2;
        const long long blocks = rows * ceil_div(nseg, run);
        if (blocks > 0x7fffffffLL) return fail(ctx, ACCB_EINVAL, "array too large for one foldSeg launch");
        return second_launch(launch(ctx, ps.fn, "foldSeg_staged", (int)blocks, ps.meta.v[5], smem, s, p));
    }
    const long long units = ceil_div(rows * nseg, pr.block / std::min(group, pr.block));
    const int grid = (int)std::min<long long>(std::max(1LL, units), (long long)ctx->sm_count * pr.per_sm);
    return second_launch(launch(ctx, pr.fn, entry, grid, pr.block, 0, s, p));
}

/* ----------------------------------------------------------------- scan */
/* Tile status records of a scan on stream s: sized for ntiles records of rec bytes, and the epoch that marks
 * this launch's records (records of earlier launches read as "not ready", so nothing is cleared between
 * launches). */
static int scan_scratch(accb_context *ctx, cudaStream_t s, long long ntiles, int rec, StreamScratch **out, unsigned *epoch_out) {
    StreamScratch *sc = scratch_for(ctx, s);
    if (!sc) return fail(ctx, ACCB_ENOMEM, "cannot allocate stream scratch");
    const size_t need = (size_t)std::max(1LL, ntiles) * rec;
    const bool regrow = sc->status_bytes < need;
    cudaStreamCaptureStatus cap = cudaStreamCaptureStatusNone;
    cudaStreamIsCapturing(s, &cap);
    unsigned epoch;
    if (cap == cudaStreamCaptureStatusActive) {
        /* Inside a stream capture the launch will be replayed with the epoch recorded now, so every replay
         * clears the status words it uses first (a memset node), and takes its epoch from a range of
         * its own (2^29 ..) that launches outside captures never reach. */
        if (regrow) return fail(ctx, ACCB_EINVAL, "scan scratch must be sized by a run before the stream capture");
        TRY(check_cuda(ctx, cudaMemsetAsync(sc->status, 0, need, s), "cudaMemsetAsync"));
        epoch = (1u << 29) + (sc->graph_epoch++ & ((1u << 29) - 1u));
    } else {
        TRY(grow(ctx, &sc->status, &sc->status_bytes, need, s, true));
        if (!regrow && (sc->status_layout != rec || sc->epoch >= (1u << 29) - 2)) {
            /* another record layout or an exhausted epoch counter: old words could alias new flags */
            TRY(check_cuda(ctx, cudaMemsetAsync(sc->status, 0, sc->status_bytes, s), "cudaMemsetAsync"));
            if (sc->epoch >= (1u << 29) - 2) sc->epoch = 0;
        }
        sc->status_layout = rec;
        epoch = ++sc->epoch;
    }
    *out = sc;
    *epoch_out = epoch;
    return ACCB_OK;
}

int accb_scan(accb_context *ctx, accb_kernel *k, accb_stream stream, const accb_array *env, int nenv, long long n,
              int direction, int kind, const void *seed, size_t seed_bytes, const accb_array *out,
              const accb_array *total) {
    return accb_scan_at(ctx, k, stream, env, nenv, n, direction, kind, seed, seed_bytes, out, total, 0);
}

int accb_scan_at(accb_context *ctx, accb_kernel *k, accb_stream stream, const accb_array *env, int nenv, long long n,
                 int direction, int kind, const void *seed, size_t seed_bytes, const accb_array *out,
                 const accb_array *total, long long index_base) {
    LOCK(ctx);
    TRY(check_skeleton(ctx, k, {SK_SCAN}, "scan"));
    if (n < 0) return fail(ctx, ACCB_EINVAL, "negative size");
    const bool right = direction == ACCB_SCAN_RIGHT;
    const bool seed_on_device = (kind & ACCB_SEED_ON_DEVICE) != 0;
    kind &= ~ACCB_SEED_ON_DEVICE;
    if (kind < ACCB_SCAN_EXCLUSIVE || kind > ACCB_SCAN_INCLUSIVE_SEEDED) return fail(ctx, ACCB_EINVAL, "unknown scan kind %d", kind);
    if (kind != ACCB_SCAN_INCLUSIVE && !seed) return fail(ctx, ACCB_EINVAL, "scanl/scanr/scan' need a seed");
    if (kind == ACCB_SCAN_INCLUSIVE && seed) return fail(ctx, ACCB_EINVAL, "scanl1/scanr1 take no seed");
    if (kind == ACCB_SCAN_PRIME && !total) return fail(ctx, ACCB_EINVAL, "scan' needs a total array");
    accb_kparams p;
    memset(&p, 0, sizeof p);
    TRY(fill_env(ctx, p, env, nenv));
    TRY(fill_out(ctx, p, out));
    if (seed_on_device) {
        /* the seed is produced by earlier work on this stream: pass its address */
        TRY(fill_scalars(ctx, p, &seed, sizeof(void *)));
        p.flags |= ACCB_F_HAS_SEED | ACCB_F_SEED_PTR;
    } else {
        TRY(set_seed(ctx, p, seed, seed_bytes));
    }
    p.n = n;
    p.base = index_base;
    p.ip[3] = -1;
    p.ip[4] = -1;
    const char *entry;
    if (kind == ACCB_SCAN_INCLUSIVE || kind == ACCB_SCAN_INCLUSIVE_SEEDED) {
        entry = right ? "scanr1" : "scanl1"; /* with a seed: the look-back of the first tile starts from it */
    } else if (kind == ACCB_SCAN_PRIME) {
        entry = right ? "scanr" : "scanl";
        TRY(fill_out(ctx, p, total, out->ncomp));
        p.ip[3] = 0;
    } else if (!right) { /* scanl: exclusive body aligned with the input, total at out[n] */
        entry = "scanl";
        TRY(fill_out(ctx, p, out, out->ncomp));
        p.ip[3] = n;
    } else { /* scanr: seeded inclusive body, the seed itself at out[n] */
        entry = "scanr1";
        TRY(fill_out(ctx, p, out, out->ncomp));
        p.ip[4] = n;
    }
    Prep pr;
    TRY(prepare(ctx, k, entry, 0, &pr));
    const int rec = pr.meta.v[2];
    const long long tile = pr.meta.v[3];
    if (rec <= 0 || tile <= 0) return fail(ctx, ACCB_EINVAL, "kernel %s carries no scan metadata", k->key.c_str());
    const long long ntiles = ceil_div(n, tile);
    if (ntiles > 0x7fffffffLL) return fail(ctx, ACCB_EINVAL, "array too large for one scan launch");
    cudaStream_t s = (cudaStream_t)stream;
    StreamScratch *sc = nullptr;
    unsigned epoch = 0;
    TRY(scan_scratch(ctx, s, ntiles, rec, &sc, &epoch));
    p.ip[0] = ntiles;
    p.ip[1] = sc->scan_ticket;
    p.ip[2] = epoch;
    p.aux[0] = sc->status;
    p.aux[1] = sc->words + 1;
    p.aux[2] = sc->words + 2;
    /* how the kernel assigns tiles: 0 = by block index, 2 = one ticket per block */
    const int mode = pr.meta.v[5];
    const int grid = (int)std::max(1LL, ntiles);
    /* keep the host's copy of the ticket counter in step with what the launch will draw */
    if (n > 0 && mode == 2) sc->scan_ticket += (unsigned)grid;
    /* full tiles are staged in dynamic shared memory by the TMA engine */
    const size_t smem = (size_t)pr.meta.v[6];
    return launch(ctx, pr.fn, entry, grid, pr.block, smem, s, p);
}

/* ----------------------------------------- scan over several GPUs, block-cyclic */
static int bc_layout(int world, int rank, long long n_global, long long block_elems, long long *n_local, int *total_owner) {
    if (world < 1 || rank < 0 || rank >= world || n_global < 0 || block_elems < 1) return ACCB_EINVAL;
    const long long full = n_global / block_elems, rem = n_global % block_elems;
    const long long mine = full / world + (rank < full % world ? 1 : 0);
    const long long blocks = full + (rem ? 1 : 0);
    if (n_local) *n_local = mine * block_elems + ((rem && full % world == rank) ? rem : 0);
    if (total_owner) *total_owner = blocks ? (int)((blocks - 1) % world) : 0;
    return ACCB_OK;
}

int accb_peer_scan_layout(int world, int rank, long long n_global, long long block_elems, long long *n_local,
                          int *total_owner, size_t *scratch_bytes) {
    if (bc_layout(world, rank, n_global, block_elems, n_local, total_owner) != ACCB_OK)
        return fail(nullptr, ACCB_EINVAL, "block-cyclic layout: rank %d of %d, %lld elements in blocks of %lld", rank, world,
                    n_global, block_elems);
    /* two sets of block records (launches alternate between them), one 128-byte line per block
     * (ACCB_SCAN_BLOCK_RECORD of scan.cuh) */
    if (scratch_bytes) *scratch_bytes = (size_t)(2 * std::max(1LL, ceil_div(n_global, block_elems)) * 128);
    return ACCB_OK;
}

int accb_peer_scan_tile(accb_context *ctx, accb_kernel *k, long long *tile_elems) {
    LOCK(ctx);
    TRY(check_skeleton(ctx, k, {SK_SCAN}, "scan"));
    Prep pr;
    TRY(prepare(ctx, k, "scanl_bc", 0, &pr));
    if (pr.meta.v[9] <= 0) return fail(ctx, ACCB_EINVAL, "kernel %s carries no scan metadata", k->key.c_str());
    if (tile_elems) *tile_elems = pr.meta.v[9];
    return ACCB_OK;
}

int accb_peer_scan(accb_peer *peer, accb_kernel *k, accb_stream stream, const accb_array *env, int nenv,
                   long long n_global, long long block_elems, int kind, const void *seed, size_t seed_bytes,
                   size_t scratch_offset, const accb_array *out, const accb_array *total) {
    return accb_peer_scan_piece(peer, k, stream, env, nenv, n_global, block_elems, kind, seed, seed_bytes, scratch_offset, out,
                                total, 0, -1);
}

int accb_peer_scan_piece(accb_peer *peer, accb_kernel *k, accb_stream stream, const accb_array *env, int nenv,
                         long long n_global, long long block_elems, int kind, const void *seed, size_t seed_bytes,
                         size_t scratch_offset, const accb_array *out, const accb_array *total,
                         long long first_local_block, long long local_blocks) {
    accb_context *ctx = peer_context(peer);
    LOCK(ctx);
    TRY(check_skeleton(ctx, k, {SK_SCAN}, "scan"));
    if (kind != ACCB_SCAN_EXCLUSIVE && kind != ACCB_SCAN_INCLUSIVE && kind != ACCB_SCAN_PRIME)
        return fail(ctx, ACCB_EINVAL, "the block-cyclic scan serves scanl, scanl1 and scanl' (kind %d)", kind);
    if (kind != ACCB_SCAN_INCLUSIVE && !seed) return fail(ctx, ACCB_EINVAL, "scanl / scanl' need a seed");
    if (kind == ACCB_SCAN_INCLUSIVE && seed) return fail(ctx, ACCB_EINVAL, "scanl1 takes no seed");
    if (kind == ACCB_SCAN_PRIME && !total) return fail(ctx, ACCB_EINVAL, "scanl' needs a total array");
    if (first_local_block < 0) return fail(ctx, ACCB_EINVAL, "negative block number");
    const char *entry = kind == ACCB_SCAN_INCLUSIVE ? "scanl1_bc" : "scanl_bc";
    Prep pr;
    TRY(prepare(ctx, k, entry, 0, &pr));
    const int rec = pr.meta.v[2];
    const long long tile = pr.meta.v[9]; /* the block-cyclic entries have a tile shape of their own */
    pr.block = pr.meta.v[8];
    if (rec <= 0 || tile <= 0 || pr.block <= 0) return fail(ctx, ACCB_EINVAL, "kernel %s carries no scan metadata", k->key.c_str());
    if (pr.meta.v[7] < 1 || pr.meta.v[7] > 8)
        return fail(ctx, ACCB_EINVAL, "the block-cyclic scan carries values of up to 8 bytes between GPUs (this kernel's have %d)",
                    pr.meta.v[7]);
    if (block_elems == 0) block_elems = 32 * tile; /* 1.1 MiB of input */
    if (n_global < 0 || block_elems < tile || block_elems % tile)
        return fail(ctx, ACCB_EINVAL, "blocks are whole multiples of the kernel's tile of %lld elements", tile);
    cudaStream_t s = (cudaStream_t)stream;
    cudaStreamCaptureStatus cap = cudaStreamCaptureStatusNone;
    cudaStreamIsCapturing(s, &cap);
    if (cap == cudaStreamCaptureStatusActive) return fail(ctx, ACCB_EINVAL, "a scan over several GPUs cannot be recorded in a stream capture");

    const long long blocks = ceil_div(n_global, block_elems);
    size_t scratch = 0;
    TRY(accb_peer_scan_layout(1, 0, n_global, block_elems, nullptr, nullptr, &scratch));
    PeerScanInfo info;
    TRY(peer_scan_begin(peer, scratch_offset, scratch, &info, false));
    long long n_local = 0;
    int owner = 0;
    bc_layout(info.world, info.rank, n_global, block_elems, &n_local, &owner);
    /* the caller's arrays must be as long as the layout says: a result array sized for another distribution
     * would be written out of bounds */
    const long long need_out = n_local + ((kind == ACCB_SCAN_EXCLUSIVE && info.rank == owner) ? 1 : 0);
    if (n_global > 0 && n_local > 0 && (!out || array_size(out) < need_out))
        return fail(ctx, ACCB_EINVAL, "rank %d holds %lld elements of this scan: the result array needs %lld elements, it has %lld",
                    info.rank, n_local, need_out, out ? array_size(out) : 0LL);
    PieceState &piece = *info.piece;
    const bool begin = first_local_block == 0;
    if (!begin) {
        const bool same = piece.n_global == n_global && piece.block_elems == block_elems && piece.stream == s;
        /* a rank that holds fewer blocks than the others is done earlier: its later pieces are empty */
        if (same && !piece.open && first_local_block >= piece.next_block) return ACCB_OK;
        if (!(same && piece.open && piece.next_block == first_local_block))
            return fail(ctx, ACCB_EINVAL, "piece %lld does not continue the scan begun on this stream (next block %lld)",
                        first_local_block, piece.open ? piece.next_block : -1LL);
    }
    const long long ntiles = ceil_div(n_local, tile);
    if (ntiles > 0x7fffffffLL) return fail(ctx, ACCB_EINVAL, "array too large for one scan launch");
    StreamScratch *sc = nullptr;
    if (begin) {
        TRY(peer_scan_begin(peer, scratch_offset, scratch, &info, true)); /* counts the scan: every rank calls, with or without data */
        /* With fewer than two blocks per GPU a rank could finish this scan and start the one after the next while a
         * slower rank still reads this scan's block records (they alternate between two sets only): line the ranks
         * up first.  With two or more blocks per GPU no rank can finish scan e+1 before every rank has begun it,
         * i.e. has finished scan e. */
        if (info.world > 1 && blocks < 2LL * info.world) TRY(accb_peer_barrier(peer, stream));
        if (n_global == 0) { /* only the seed survives: scanl's single element and the total, on rank 0 */
            if (info.rank != 0) return ACCB_OK;
            return accb_scan(ctx, k, stream, env, nenv, 0, ACCB_SCAN_LEFT, kind, seed, seed_bytes, out, total);
        }
        piece = PieceState();
        piece.count = info.count;
        piece.n_global = n_global;
        piece.block_elems = block_elems;
        piece.stream = s;
        piece.open = true;
        if (n_local > 0) TRY(scan_scratch(ctx, s, ntiles, rec, &sc, &piece.epoch));
    } else if (n_local > 0) {
        sc = scratch_for(ctx, s);
        if (!sc || sc->epoch != piece.epoch)
            return fail(ctx, ACCB_EINVAL, "another scan ran on this stream between the pieces of this one");
    }
    const long long tpb = block_elems / tile;
    const long long local_all = ceil_div(n_local, block_elems);
    const long long last_block = local_blocks < 0 ? local_all : std::min(local_all, first_local_block + local_blocks);
    piece.next_block = last_block;
    if (last_block >= local_all) piece.open = false;
    if (n_local == 0 || last_block <= first_local_block) return ACCB_OK;

    accb_kparams p;
    memset(&p, 0, sizeof p);
    TRY(fill_env(ctx, p, env, nenv));
    TRY(fill_out(ctx, p, out));
    TRY(set_seed(ctx, p, seed, seed_bytes));
    p.n = n_local;
    p.ip[3] = -1;
    p.ip[4] = -1;
    if (info.rank == owner) {
        if (kind == ACCB_SCAN_PRIME) {
            TRY(fill_out(ctx, p, total, out->ncomp));
            p.ip[3] = 0;
        } else if (kind == ACCB_SCAN_EXCLUSIVE) { /* the total follows this rank's last element */
            TRY(fill_out(ctx, p, out, out->ncomp));
            p.ip[3] = n_local;
        }
    }
    const long long tile_first = first_local_block * tpb, tile_end = std::min(ntiles, last_block * tpb);
    p.ip[0] = ntiles;
    p.ip[1] = sc->scan_ticket;
    p.ip[2] = piece.epoch;
    p.ip[5] = tpb;
    p.ip[6] = info.world;
    p.ip[7] = info.rank;
    p.ip[8] = piece.count & 0x3fffffffu;
    p.ip[9] = (long long)info.timeout_ns;
    p.ip[10] = (long long)(info.header_bytes + scratch_offset + (piece.count & 1u) * (scratch / 2));
    p.ip[11] = tile_first;
    p.aux[0] = sc->status;
    p.aux[1] = sc->words + 1;
    p.aux[2] = sc->words + 2;
    p.aux[3] = info.dev_bases;
    const int grid = (int)(tile_end - tile_first);
    if (pr.meta.v[5] == 2) sc->scan_ticket += (unsigned)grid;
    return launch(ctx, pr.fn, entry, grid, pr.block, (size_t)pr.meta.v[10], s, p);
}

/* -------------------------------------------------------------- permute */
int accb_permute_defaults(accb_context *ctx, accb_stream stream, const accb_array *defaults, const accb_array *out,
                          const int *comp_bytes) {
    LOCK(ctx);
    if (!defaults || !out || !comp_bytes || defaults->ncomp != out->ncomp)
        return fail(ctx, ACCB_EINVAL, "defaults / result mismatch");
    const long long n = array_size(out);
    if (array_size(defaults) != n) return fail(ctx, ACCB_EINVAL, "defaults and result differ in size");
    /* device-to-device copy on the same stream, ahead of the kernel (Execute.hs:405-407) */
    for (int c = 0; c < out->ncomp; ++c)
        TRY(check_cuda(ctx,
                       cudaMemcpyAsync(out->ptr[c], defaults->ptr[c], (size_t)n * comp_bytes[c],
                                       cudaMemcpyDeviceToDevice, (cudaStream_t)stream),
                       "copying permute defaults"));
    return ACCB_OK;
}

int accb_permute(accb_context *ctx, accb_kernel *k, accb_stream stream, const accb_array *env, int nenv,
                 long long n_src, const void *scalars, size_t scalar_bytes, const accb_array *out) {
    return accb_permute_at(ctx, k, stream, env, nenv, n_src, scalars, scalar_bytes, out, 0);
}

int accb_permute_at(accb_context *ctx, accb_kernel *k, accb_stream stream, const accb_array *env, int nenv,
                    long long n_src, const void *scalars, size_t scalar_bytes, const accb_array *out,
                    long long index_base) {
    LOCK(ctx);
    TRY(check_skeleton(ctx, k, {SK_PERMUTE, SK_PERMUTE_SMEM}, "permute"));
    if (n_src < 0) return fail(ctx, ACCB_EINVAL, "negative size");
    if (!out || out->rank < 1) return fail(ctx, ACCB_EINVAL, "permute into a rank-0 array is not supported"); /* IndexSpace.hs:230 */
    accb_kparams p;
    memset(&p, 0, sizeof p);
    TRY(fill_env(ctx, p, env, nenv));
    const unsigned vec = p.flags & ACCB_F_VEC; /* only the inputs are read as vectors */
    TRY(fill_out(ctx, p, out));
    p.flags |= vec;
    TRY(fill_scalars(ctx, p, scalars, scalar_bytes));
    p.n = n_src;
    p.base = index_base;
    const long long nout = array_size(out);
    p.ip[0] = nout;
    if (n_src == 0 || nout == 0) return ACCB_OK;
    cudaStream_t s = (cudaStream_t)stream;
    StreamScratch *sc = scratch_for(ctx, s);
    if (!sc) return fail(ctx, ACCB_ENOMEM, "cannot allocate stream scratch");
    p.aux[1] = sc->words + 2;

    Prep pr;
    TRY(prepare(ctx, k, "permute", 0, &pr));
    const int elem = pr.meta.v[2];
    const bool needs_lock = pr.meta.v[5] != 0;
    /* privatise in shared memory when R skewed copies of the destination fit */
    if (k->skeleton == SK_PERMUTE_SMEM && (nout + 1) * elem <= 96 * 1024) {
        int R = ctx->tune.permute_replicas;
        while (R > 1 && (R & (R - 1))) R &= R - 1; /* power of two */
        while (R > 1 && (long long)R * (nout + 1) * elem > 200 * 1024) R >>= 1;
        const size_t smem = (size_t)R * (nout + 1) * elem;
        Prep ps;
        TRY(prepare(ctx, k, "permute_smem", smem, &ps));
        p.ip[1] = R;
        const long long units = ceil_div(n_src, (long long)ps.block * ps.meta.v[4] * 4);
        const int grid = (int)std::min<long long>(std::max(1LL, units), (long long)ctx->sm_count * ps.per_sm);
        /* the replicas take what they need; the driver's own split measured faster than the maximum */
        return launch(ctx, ps.fn, "permute_smem", grid, ps.block, smem, s, p, false);
    }
    if (needs_lock) {
        /* one lock word per destination element, cleared for every launch (Execute.hs:402-405) */
        TRY(grow(ctx, &sc->partial, &sc->partial_bytes, (size_t)nout * sizeof(int), s, false));
        TRY(check_cuda(ctx, cudaMemsetAsync(sc->partial, 0, (size_t)nout * sizeof(int), s), "cudaMemsetAsync"));
        p.aux[0] = sc->partial;
    }
    const long long units = ceil_div(n_src, (long long)pr.block * pr.meta.v[4] * 4);
    const int grid = (int)std::min<long long>(std::max(1LL, units), (long long)ctx->sm_count * pr.per_sm);
    return launch(ctx, pr.fn, "permute", grid, pr.block, 0, s, p);
}

/* -------------------------------------------------------------- stencil */
/* rank 3: a block owns a column of the cube and marches along z (skeletons/stencil3.cuh) */
static int stencil3_launch(accb_context *ctx, accb_kernel *k, cudaStream_t s, const accb_array *src, int boundary,
                           const void *constant, size_t constant_bytes, const accb_array *out) {
    if (k->skeleton != SK_STENCIL3) return fail(ctx, ACCB_EINVAL, "kernel %s was not built for the stencil3 skeleton (rank-3 arrays)", k->key.c_str());
    if (!src || src->rank != 3 || src->ncomp != 1 || !src->ptr[0]) return fail(ctx, ACCB_EINVAL, "stencil source: rank / component mismatch");
    if (boundary < ACCB_CLAMP || boundary > ACCB_CONSTANT) return fail(ctx, ACCB_EINVAL, "unknown boundary %d", boundary);
    if (boundary == ACCB_CONSTANT && !constant) return fail(ctx, ACCB_EINVAL, "Constant boundary needs a value");
    for (int d = 0; d < 3; ++d)
        if (src->shape[d] != out->shape[d]) return fail(ctx, ACCB_EINVAL, "a stencil's result has the shape of its source");
    accb_kparams p;
    memset(&p, 0, sizeof p);
    p.flags |= ACCB_F_VEC;
    p.in[0] = src->ptr[0];
    if (!aligned16(src->ptr[0])) p.flags &= ~ACCB_F_VEC;
    TRY(fill_out(ctx, p, out));
    if (constant) TRY(fill_scalars(ctx, p, constant, constant_bytes));
    const long long W = out->shape[0], H = out->shape[1], D = out->shape[2];
    p.n = W * H * D;
    if (p.n == 0) return ACCB_OK;
    Prep pr;
    TRY(prepare(ctx, k, "stencil3", 0, &pr));
    if (pr.meta.v[2] != 4) return fail(ctx, ACCB_EINVAL, "the rank-3 stencil skeleton takes 4-byte elements");
    const size_t smem = (size_t)pr.meta.v[6];
    TRY(occupancy(ctx, pr.fn, pr.block, smem, &pr.per_sm));
    const long long columns = ceil_div(W, pr.meta.v[4]) * ceil_div(H, pr.meta.v[3]);
    const long long resident = (long long)ctx->sm_count * pr.per_sm;
    /* cut z so that there are a few times more tasks than resident blocks, but keep runs long: every run
     * re-reads 2*RZ planes of its neighbours */
    const long long min_run = std::max(8LL, 8LL * pr.meta.v[5]);
    long long zchunks = std::max(1LL, std::min(ceil_div(D, min_run), ceil_div(4 * resident, columns)));
    const long long zrun = ceil_div(D, zchunks);
    zchunks = ceil_div(D, zrun);
    p.ip[0] = D;
    p.ip[1] = H;
    p.ip[2] = W;
    p.ip[3] = zrun;
    p.ip[4] = boundary;
    const int grid = (int)std::min(columns * zchunks, resident);
    return launch(ctx, pr.fn, "stencil3", grid, pr.block, smem, s, p);
}

/* `twice`, if not null: the caller would like TWO applications of the stencil from src[0] to out in this one launch;
 * *twice says whether that is what was launched (the two-application tile form: one source, rank 2, 4-byte elements
 * of one type, 16-byte aligned rows, any boundary but Wrap) or one application as usual. */
static int stencil_launch(accb_context *ctx, accb_kernel *k, const char *entry, cudaStream_t s,
                          const accb_array *const *src, int nsrc, int boundary, const void *constant,
                          size_t constant_bytes, const accb_array *out, bool *twice = nullptr) {
    const bool want_twice = twice && *twice;
    if (twice) *twice = false;
    if (out && out->rank == 3 && nsrc == 1) return stencil3_launch(ctx, k, s, src[0], boundary, constant, constant_bytes, out);
    if (k->skeleton == SK_STENCIL3) return fail(ctx, ACCB_EINVAL, "kernel %s was built for rank-3 arrays", k->key.c_str());
    if (!out || out->rank < 1 || out->rank > 2) return fail(ctx, ACCB_EINVAL, "stencil2 supports rank 1 and 2, stencil rank 1 to 3");
    if (boundary < ACCB_CLAMP || boundary > ACCB_CONSTANT) return fail(ctx, ACCB_EINVAL, "unknown boundary %d", boundary);
    if (boundary == ACCB_CONSTANT && !constant) return fail(ctx, ACCB_EINVAL, "Constant boundary needs a value");
    accb_kparams p;
    memset(&p, 0, sizeof p);
    p.flags |= ACCB_F_VEC;
    for (int a = 0; a < nsrc; ++a) {
        if (!src[a] || src[a]->rank != out->rank || src[a]->ncomp != 1 || !src[a]->ptr[0])
            return fail(ctx, ACCB_EINVAL, "stencil source %d: rank / component mismatch", a);
        p.in[a] = src[a]->ptr[0];
        if (!aligned16(src[a]->ptr[0])) p.flags &= ~ACCB_F_VEC;
        p.ip[5 + 2 * a] = out->rank == 2 ? src[a]->shape[1] : 1;
        p.ip[6 + 2 * a] = src[a]->shape[0];
    }
    TRY(fill_out(ctx, p, out));
    if (constant) TRY(fill_scalars(ctx, p, constant, constant_bytes));
    const int W = out->shape[0], H = out->rank == 2 ? out->shape[1] : 1;
    p.n = (long long)W * H;
    if (p.n == 0) return ACCB_OK;
    for (int a = 0; a < nsrc; ++a)
        if (p.ip[5 + 2 * a] < H || p.ip[6 + 2 * a] < W)
            return fail(ctx, ACCB_EINVAL, "stencil result larger than source %d", a);
    Prep pr;
    TRY(prepare(ctx, k, entry, 0, &pr));
    StreamScratch *sc = scratch_for(ctx, s);
    if (!sc) return fail(ctx, ACCB_ENOMEM, "cannot allocate stream scratch");
    p.aux[1] = sc->words + 2; /* error word of the bounded waits */
    p.ip[4] = boundary;
    /* Tile form (input tile staged in shared memory by TMA): needs 4-byte elements (the kernel
     * reports 0 bytes of shared memory otherwise), 16-byte aligned arrays, widths that are
     * multiples of 4 and enough rows to fill a tile. */
    bool staged = (p.flags & ACCB_F_VEC) && W % 4 == 0 && !ctx->tune.stencil_no_tile;
    for (int a = 0; a < nsrc; ++a) staged = staged && p.ip[6 + 2 * a] % 4 == 0;
    const bool tiled = staged && pr.meta.v[6] > 0 && H >= 16;
    if (staged && out->rank == 1 && pr.meta.v[5] > 0 && W >= 4096) {
        /* line form: one bulk copy of (tile + 8 halo elements) x 4 bytes per source */
        const std::string lentry = std::string(entry) + "_line";
        const size_t smem = (size_t)nsrc * (pr.meta.v[5] + 8) * 4;
        Prep pl;
        TRY(prepare(ctx, k, lentry.c_str(), smem, &pl));
        p.ip[0] = 1;
        p.ip[1] = W;
        return launch(ctx, pl.fn, lentry.c_str(), (int)ceil_div(W, pl.meta.v[5]), pl.block, smem, s, p);
    }
    if (tiled && want_twice && nsrc == 1 && boundary != ACCB_WRAP && pr.meta.v[8] > 0 && !ctx->tune.stencil_no_fuse) {
        const size_t smem = (size_t)pr.meta.v[8];
        Prep pt;
        TRY(prepare(ctx, k, "stencil_tile2", smem, &pt));
        p.ip[0] = H;
        p.ip[1] = W;
        const long long tiles = ceil_div(W, pr.meta.v[4]) * ceil_div(H, pr.meta.v[9]);
        if (tiles > 0x7fffffffLL) return fail(ctx, ACCB_EINVAL, "array too large for one stencil launch");
        *twice = true;
        return launch(ctx, pt.fn, "stencil_tile2", (int)tiles, pt.block, smem, s, p);
    }
    if (tiled) {
        const std::string tentry = std::string(entry) + "_tile";
        const size_t smem = (size_t)pr.meta.v[6];
        Prep pt;
        TRY(prepare(ctx, k, tentry.c_str(), smem, &pt));
        p.ip[0] = H;
        p.ip[1] = W;
        const long long tiles = ceil_div(W, pt.meta.v[4]) * ceil_div(H, pt.meta.v[3]);
        if (tiles > 0x7fffffffLL) return fail(ctx, ACCB_EINVAL, "array too large for one stencil launch");
        return launch(ctx, pt.fn, tentry.c_str(), (int)tiles, pt.block, smem, s, p);
    }
    int txw = 32;
    while (txw < pr.block && txw * 4 < W) txw *= 2;
    const int rb = ctx->tune.stencil_rows;
    const int ty = pr.block / txw;
    p.ip[0] = H;
    p.ip[1] = W;
    p.ip[2] = rb;
    p.ip[3] = txw;
    p.ip[4] = boundary;
    const long long tasks = ceil_div(W, (long long)txw * 4) * ceil_div(H, (long long)rb * ty);
    const int grid = (int)std::min<long long>(tasks, 1 << 20);
    return launch(ctx, pr.fn, entry, grid, pr.block, 0, s, p);
}

int accb_stencil(accb_context *ctx, accb_kernel *k, accb_stream stream, const accb_array *src, int boundary,
                 const void *constant, size_t constant_bytes, const accb_array *out) {
    LOCK(ctx);
    TRY(check_skeleton(ctx, k, {SK_STENCIL, SK_STENCIL3}, "stencil"));
    const accb_array *srcs[1] = {src};
    return stencil_launch(ctx, k, "stencil", (cudaStream_t)stream, srcs, 1, boundary, constant, constant_bytes, out);
}

int accb_stencil2(accb_context *ctx, accb_kernel *k, accb_stream stream, const accb_array *src1,
                  const accb_array *src2, int boundary, const void *constant, size_t constant_bytes,
                  const accb_array *out) {
    LOCK(ctx);
    TRY(check_skeleton(ctx, k, {SK_STENCIL2}, "stencil2"));
    const accb_array *srcs[2] = {src1, src2};
    return stencil_launch(ctx, k, "stencil2", (cudaStream_t)stream, srcs, 2, boundary, constant, constant_bytes, out);
}

int accb_stencil_iterate(accb_context *ctx, accb_kernel *k, accb_stream stream, const accb_array *a,
                         const accb_array *b, int iters, int boundary, const void *constant, size_t constant_bytes,
                         int *result_in_b) {
    return accb_stencil_iterate_from(ctx, k, stream, nullptr, a, b, iters, boundary, constant, constant_bytes, result_in_b);
}

int accb_stencil_iterate_from(accb_context *ctx, accb_kernel *k, accb_stream stream, const accb_array *src,
                              const accb_array *a, const accb_array *b, int iters, int boundary, const void *constant,
                              size_t constant_bytes, int *result_in_b) {
    LOCK(ctx);
    TRY(check_skeleton(ctx, k, {SK_STENCIL, SK_STENCIL3}, "stencil"));
    if (!a || !b || iters < 0 || (src && iters < 1)) return fail(ctx, ACCB_EINVAL, "bad argument");
    /* with a separate source the first launch reads it and writes a; cur is always what the next launch reads */
    const accb_array *cur = src ? src : a, *nxt = src ? a : b, *spare = src ? b : nullptr;
    for (int left = iters; left > 0;) {
        const accb_array *srcs[1] = {cur};
        bool twice = left >= 2; /* two applications per launch where the kernel has that form: half the traffic */
        TRY(stencil_launch(ctx, k, "stencil", (cudaStream_t)stream, srcs, 1, boundary, constant, constant_bytes, nxt, &twice));
        left -= twice ? 2 : 1;
        if (spare) { /* the source is never written: from now on ping-pong between a and b */
            cur = nxt;
            nxt = spare;
            spare = nullptr;
        } else {
            std::swap(cur, nxt);
        }
    }
    if (result_in_b) *result_in_b = (cur == b);
    return ACCB_OK;
}

} /* extern "C" */
