/*
 * peer.cu -- the small exchanges of the sharded skeletons done by the library's own kernels over NVLink, one
 * process per GPU: every rank owns an exchange buffer that the other ranks map (CUDA IPC, plain peer mappings,
 * no multicast objects), and a kernel that first synchronises the ranks through flags in those buffers and
 * then moves or combines the data with peer loads.
 *
 *   scan      slab totals       barrier + gather of one element per rank          (accb_peer_gather)
 *   foldAll   partials          the same
 *   permute   partial results   barrier + element-wise combination in rank order   (accb_peer_allreduce)
 *   stencil   halo rows         barrier, pull from the neighbours' slabs, barrier   (accb_peer_barrier / _pull)
 *
 * The reference has no multi-device execution; its peer copy (CUDA/Array/Prim.hs:306-335) is never called.
 *
 * Flags: rank r's buffer starts with one 32-bit word per rank.  Barrier number e: every rank stores e into word
 * [own rank] of EVERY rank's buffer (release, system scope), then waits until all words of its own buffer have
 * reached e (acquire).  The ranks run on different GPUs; a wait gives up after five seconds (or
 * ACCB_PEER_TIMEOUT_MS), sets the buffer's error word and lets the kernel finish, so a rank that never arrives
 * cannot hang the others.
 */
#include <type_traits>

#include "common.h"

using namespace accb_rt;

namespace {
constexpr int kMaxWorld = 64;
constexpr size_t kHeader = 1024;           /* flags [0..64), error word at [64], padding */
constexpr int kErrorWord = kMaxWorld;
constexpr unsigned kSpinLimit = 1u << 24;  /* polls (some 15 s); a second bound should the timer misbehave */

struct PeerPtrs {
    unsigned char *base[kMaxWorld];
    unsigned long long timeout_ns; /* how long a rank waits for the others */
};

__device__ __forceinline__ unsigned long long global_ns() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}

__device__ __forceinline__ void st_release_sys(unsigned *p, unsigned v) {
    asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ unsigned ld_acquire_sys(const unsigned *p) {
    unsigned v;
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}
template <class T>
__device__ __forceinline__ T ld_peer(const T *p) { /* not through this GPU's L1 */
    return __ldcg(p);
}

/* all threads of ONE block call this; threads 0..world-1 do the signalling */
__device__ void block_barrier(const PeerPtrs &pp, int rank, int world, unsigned epoch) {
    __syncthreads();
    const int r = threadIdx.x;
    if (r < world) {
        __threadfence_system();
        st_release_sys(reinterpret_cast<unsigned *>(pp.base[r]) + rank, epoch);
        const unsigned *mine = reinterpret_cast<const unsigned *>(pp.base[rank]) + r;
        unsigned spins = 0;
        const unsigned long long t0 = global_ns();
        while ((int)(ld_acquire_sys(mine) - epoch) < 0) {
            __nanosleep(250);
            if (++spins > kSpinLimit || ((spins & 63u) == 0 && global_ns() - t0 > pp.timeout_ns)) {
                atomicExch(reinterpret_cast<unsigned *>(pp.base[rank]) + kErrorWord, 1u);
                break;
            }
        }
    }
    __syncthreads();
}

__global__ void peer_barrier_kernel(PeerPtrs pp, int rank, int world, unsigned epoch) { block_barrier(pp, rank, world, epoch); }

/* dst[r * bytes ..] = rank r's data[offset .. offset + bytes), bytes a multiple of 4 */
__global__ void peer_gather_kernel(PeerPtrs pp, int rank, int world, unsigned epoch, size_t offset, size_t bytes,
                                   unsigned *dst) {
    block_barrier(pp, rank, world, epoch);
    const size_t words = bytes / 4;
    for (size_t i = threadIdx.x; i < words * world; i += blockDim.x) {
        const int r = (int)(i / words);
        const unsigned *src = reinterpret_cast<const unsigned *>(pp.base[r] + kHeader + offset);
        dst[i] = ld_peer(src + i % words);
    }
}

enum { OP_ADD = 0, OP_MIN = 1, OP_MAX = 2, OP_AND = 3, OP_OR = 4, OP_XOR = 5 };

template <class T>
__device__ __forceinline__ T combine(int op, T a, T b) {
    if (op == OP_MIN) return b < a ? b : a;
    if (op == OP_MAX) return b > a ? b : a;
    if constexpr (std::is_integral<T>::value) {
        typedef typename std::make_unsigned<T>::type U;
        if (op == OP_AND) return a & b;
        if (op == OP_OR) return a | b;
        if (op == OP_XOR) return a ^ b;
        return (T)((U)a + (U)b); /* wrapping, as the skeletons add */
    } else {
        return a + b;
    }
}

/* dst[i] = data_0[i] (op) data_1[i] (op) ... in rank order: every rank computes the same bits.  A thread takes
 * 16 bytes of every rank's data at a time and issues the loads of up to eight ranks before it combines any of
 * them: the loads cross NVLink, and one after the other their latencies would add up. */
template <class T>
__global__ void peer_allreduce_kernel(PeerPtrs pp, int rank, int world, unsigned epoch, size_t offset, long long count,
                                      int op, T *dst) {
    block_barrier(pp, rank, world, epoch);
    constexpr int VEC = 16 / sizeof(T), BATCH = 8;
    const bool vec_ok = (reinterpret_cast<uintptr_t>(dst) & 15u) == 0; /* `offset` is a multiple of 16 */
    const long long nvec = vec_ok ? count / VEC : 0;
    for (long long i = threadIdx.x; i < nvec; i += blockDim.x) {
        __align__(16) T acc[VEC];
        for (int r0 = 0; r0 < world; r0 += BATCH) {
            uint4 v[BATCH];
#pragma unroll
            for (int j = 0; j < BATCH; ++j)
                if (r0 + j < world) v[j] = ld_peer(reinterpret_cast<const uint4 *>(pp.base[r0 + j] + kHeader + offset) + i);
#pragma unroll
            for (int j = 0; j < BATCH; ++j)
                if (r0 + j < world) {
                    const T *e = reinterpret_cast<const T *>(&v[j]);
#pragma unroll
                    for (int k = 0; k < VEC; ++k) acc[k] = (r0 + j == 0) ? e[k] : combine<T>(op, acc[k], e[k]);
                }
        }
        reinterpret_cast<uint4 *>(dst)[i] = *reinterpret_cast<const uint4 *>(acc);
    }
    for (long long i = nvec * VEC + threadIdx.x; i < count; i += blockDim.x) {
        T acc = ld_peer(reinterpret_cast<const T *>(pp.base[0] + kHeader + offset) + i);
        for (int r = 1; r < world; ++r)
            acc = combine<T>(op, acc, ld_peer(reinterpret_cast<const T *>(pp.base[r] + kHeader + offset) + i));
        dst[i] = acc;
    }
}

/* dst[i] = first[i] (op) data_0[i] (op) .. (op) data_{rank-1}[i]: what the slabs before this rank's add up to, the
 * carry its scan continues from (`first` = the seed of the whole scan, in this rank's memory) */
template <class T>
__global__ void peer_exscan_kernel(PeerPtrs pp, int rank, int world, unsigned epoch, size_t offset, long long count,
                                   int op, const T *first, T *dst) {
    block_barrier(pp, rank, world, epoch);
    for (long long i = threadIdx.x; i < count; i += blockDim.x) {
        T acc = first[i];
        for (int r0 = 0; r0 < rank; r0 += 8) {
            T v[8];
#pragma unroll
            for (int j = 0; j < 8; ++j)
                if (r0 + j < rank) v[j] = ld_peer(reinterpret_cast<const T *>(pp.base[r0 + j] + kHeader + offset) + i);
#pragma unroll
            for (int j = 0; j < 8; ++j)
                if (r0 + j < rank) acc = combine<T>(op, acc, v[j]);
        }
        dst[i] = acc;
    }
}

/* dst[0 .. bytes) = rank `from`'s data[offset ..), 16 bytes per thread and trip; no barrier of its own */
__global__ void peer_pull_kernel(PeerPtrs pp, int from, size_t offset, size_t bytes, uint4 *dst) {
    const uint4 *src = reinterpret_cast<const uint4 *>(pp.base[from] + kHeader + offset);
    const size_t n = bytes / 16;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x)
        dst[i] = ld_peer(src + i);
}

}  // namespace

struct accb_peer {
    accb_context *ctx = nullptr;
    int rank = 0, world = 1;
    size_t bytes = 0;              /* of the data area */
    unsigned char *local = nullptr;
    PeerPtrs pp;
    bool connected = false;
    unsigned epoch = 0;
    unsigned char **dev_bases = nullptr; /* the buffers' addresses in device memory, for kernels that take a table */
    unsigned scans = 0;                  /* block-cyclic scans so far: the epoch of their block records */
    PieceState piece;                    /* a scan that is being launched piece by piece */
};

extern "C" {
static int make_table(accb_peer *p);
}

#define PLOCKP(p)                                                   \
    if (!(p)) return fail(nullptr, ACCB_EINVAL, "null peer object"); \
    std::lock_guard<std::recursive_mutex> lock_((p)->ctx->mu);      \
    CtxGuard guard_((p)->ctx)

extern "C" {

int accb_peer_create(accb_context *ctx, int rank, int world, size_t bytes, accb_peer **out) {
    if (!ctx || !out) return fail(ctx, ACCB_EINVAL, "null argument");
    *out = nullptr;
    if (world < 1 || world > kMaxWorld || rank < 0 || rank >= world) return fail(ctx, ACCB_EINVAL, "rank %d of %d", rank, world);
    std::lock_guard<std::recursive_mutex> lock_(ctx->mu);
    CtxGuard guard_(ctx);
    accb_peer *p = new accb_peer;
    p->ctx = ctx;
    p->rank = rank;
    p->world = world;
    p->bytes = (bytes + 255) / 256 * 256;
    memset(&p->pp, 0, sizeof p->pp);
    /* a plain cudaMalloc block of its own: that is what an IPC handle names */
    int st = check_cuda(ctx, cudaMalloc((void **)&p->local, kHeader + p->bytes), "cudaMalloc");
    /* flags, error word and data all start at zero (records that kernels validate by an epoch must not hold
     * leftovers of whoever owned the memory before), and the clearing is finished before any rank can learn
     * this buffer's handle and write into it */
    if (st == ACCB_OK) st = check_cuda(ctx, cudaMemset(p->local, 0, kHeader + p->bytes), "cudaMemset");
    if (st == ACCB_OK) st = check_cuda(ctx, cudaDeviceSynchronize(), "cudaDeviceSynchronize");
    if (st != ACCB_OK) {
        if (p->local) cudaFree(p->local);
        delete p;
        return st;
    }
    p->pp.base[rank] = p->local;
    const char *ms = getenv("ACCB_PEER_TIMEOUT_MS");
    p->pp.timeout_ns = (unsigned long long)(ms && atoll(ms) > 0 ? atoll(ms) : 5000) * 1000000ull;
    p->connected = world == 1;
    *out = p;
    return ACCB_OK;
}

int accb_peer_handle(accb_peer *p, unsigned char *handle) {
    PLOCKP(p);
    if (!handle) return fail(p->ctx, ACCB_EINVAL, "null handle buffer");
    static_assert(sizeof(cudaIpcMemHandle_t) == ACCB_PEER_HANDLE_BYTES, "handle size");
    cudaIpcMemHandle_t h;
    int st = check_cuda(p->ctx, cudaIpcGetMemHandle(&h, p->local), "cudaIpcGetMemHandle");
    if (st == ACCB_OK) memcpy(handle, &h, sizeof h);
    return st;
}

int accb_peer_connect(accb_peer *p, const unsigned char *handles) {
    PLOCKP(p);
    if (!handles) return fail(p->ctx, ACCB_EINVAL, "null handles");
    for (int r = 0; r < p->world; ++r) {
        if (r == p->rank || p->pp.base[r]) continue;
        cudaIpcMemHandle_t h;
        memcpy(&h, handles + (size_t)r * sizeof h, sizeof h);
        void *q = nullptr;
        int st = check_cuda(p->ctx, cudaIpcOpenMemHandle(&q, h, cudaIpcMemLazyEnablePeerAccess), "cudaIpcOpenMemHandle");
        if (st != ACCB_OK) return st;
        p->pp.base[r] = static_cast<unsigned char *>(q);
    }
    p->connected = true;
    return make_table(p);
}

/* Every other rank is stood in for by this rank's own buffer: nobody ever sets their flags, so the next
 * synchronising call runs into its time limit.  How the bounded wait is tested without a second process. */
int accb_peer_loopback(accb_peer *p) {
    PLOCKP(p);
    for (int r = 0; r < p->world; ++r)
        if (!p->pp.base[r]) p->pp.base[r] = p->local;
    p->connected = true;
    return make_table(p);
}

int accb_peer_data(accb_peer *p, void **data, size_t *bytes) {
    PLOCKP(p);
    if (data) *data = p->local + kHeader;
    if (bytes) *bytes = p->bytes;
    return ACCB_OK;
}

/* 1 when a wait of some earlier exchange gave up (the word is cleared); waits for the stream */
int accb_peer_status(accb_peer *p, accb_stream stream, int *timed_out) {
    PLOCKP(p);
    unsigned w = 0;
    int st = check_cuda(p->ctx, cudaStreamSynchronize((cudaStream_t)stream), "cudaStreamSynchronize");
    if (st == ACCB_OK)
        st = check_cuda(p->ctx, cudaMemcpy(&w, p->local + kErrorWord * 4, 4, cudaMemcpyDeviceToHost), "cudaMemcpy");
    if (st != ACCB_OK) return st;
    if (w) cudaMemset(p->local + kErrorWord * 4, 0, 4);
    if (timed_out) *timed_out = w != 0;
    return w ? fail(p->ctx, ACCB_ETIMEOUT, "a rank did not reach an exchange in time") : ACCB_OK;
}

/* the table of buffer addresses that kernels index by rank, built once all buffers are mapped */
static int make_table(accb_peer *p) {
    if (p->dev_bases) return ACCB_OK;
    int st = check_cuda(p->ctx, cudaMalloc((void **)&p->dev_bases, sizeof(unsigned char *) * kMaxWorld), "cudaMalloc");
    if (st == ACCB_OK)
        st = check_cuda(p->ctx, cudaMemcpy(p->dev_bases, p->pp.base, sizeof(unsigned char *) * kMaxWorld, cudaMemcpyHostToDevice),
                        "cudaMemcpy");
    return st;
}

static int ready(accb_peer *p, size_t offset, size_t bytes) {
    if (!p->connected) return fail(p->ctx, ACCB_EINVAL, "peer buffers are not connected yet");
    if (offset % 16 || offset + bytes > p->bytes) return fail(p->ctx, ACCB_EINVAL, "range outside the exchange buffer");
    return ACCB_OK;
}

int accb_peer_barrier(accb_peer *p, accb_stream stream) {
    PLOCKP(p);
    int st = ready(p, 0, 0);
    if (st != ACCB_OK) return st;
    if (p->world == 1) return ACCB_OK;
    peer_barrier_kernel<<<1, 64, 0, (cudaStream_t)stream>>>(p->pp, p->rank, p->world, ++p->epoch);
    p->ctx->launches++;
    return check_cuda(p->ctx, cudaGetLastError(), "peer barrier");
}

int accb_peer_gather(accb_peer *p, accb_stream stream, size_t offset, size_t bytes, void *dst) {
    PLOCKP(p);
    int st = ready(p, offset, bytes);
    if (st != ACCB_OK) return st;
    if (!dst || bytes % 4) return fail(p->ctx, ACCB_EINVAL, "gather moves multiples of 4 bytes");
    peer_gather_kernel<<<1, 256, 0, (cudaStream_t)stream>>>(p->pp, p->rank, p->world, ++p->epoch, offset, bytes,
                                                           static_cast<unsigned *>(dst));
    p->ctx->launches++;
    return check_cuda(p->ctx, cudaGetLastError(), "peer gather");
}

int accb_peer_allreduce(accb_peer *p, accb_stream stream, size_t offset, long long count, int type, int op, void *dst) {
    PLOCKP(p);
    const size_t eb = (type == ACCB_PEER_I64 || type == ACCB_PEER_F64) ? 8 : 4;
    int st = ready(p, offset, (size_t)count * eb);
    if (st != ACCB_OK) return st;
    if (!dst || count < 0 || op < OP_ADD || op > OP_XOR) return fail(p->ctx, ACCB_EINVAL, "bad all-reduce arguments");
    const bool real = type == ACCB_PEER_F32 || type == ACCB_PEER_F64;
    if (real && op > OP_MAX) return fail(p->ctx, ACCB_EINVAL, "bitwise combination of floating-point values");
    cudaStream_t s = (cudaStream_t)stream;
    if (type < ACCB_PEER_I32 || type > ACCB_PEER_F64) return fail(p->ctx, ACCB_EINVAL, "unknown element type %d", type);
    const unsigned e = ++p->epoch;
#define ACCB_PEER_LAUNCH(T) \
    peer_allreduce_kernel<T><<<1, 1024, 0, s>>>(p->pp, p->rank, p->world, e, offset, count, op, static_cast<T *>(dst))
    switch (type) {
        case ACCB_PEER_I32: ACCB_PEER_LAUNCH(int); break;
        case ACCB_PEER_U32: ACCB_PEER_LAUNCH(unsigned); break;
        case ACCB_PEER_I64: ACCB_PEER_LAUNCH(long long); break;
        case ACCB_PEER_F32: ACCB_PEER_LAUNCH(float); break;
        case ACCB_PEER_F64: ACCB_PEER_LAUNCH(double); break;
        default: return fail(p->ctx, ACCB_EINVAL, "unknown element type %d", type);
    }
#undef ACCB_PEER_LAUNCH
    p->ctx->launches++;
    return check_cuda(p->ctx, cudaGetLastError(), "peer all-reduce");
}

int accb_peer_exscan(accb_peer *p, accb_stream stream, size_t offset, long long count, int type, int op,
                     const void *first, void *dst) {
    PLOCKP(p);
    if (type < ACCB_PEER_I32 || type > ACCB_PEER_F64) return fail(p->ctx, ACCB_EINVAL, "unknown element type %d", type);
    const size_t eb = (type == ACCB_PEER_I64 || type == ACCB_PEER_F64) ? 8 : 4;
    int st = ready(p, offset, (size_t)count * eb);
    if (st != ACCB_OK) return st;
    if (!dst || !first || count < 0 || op < OP_ADD || op > OP_XOR) return fail(p->ctx, ACCB_EINVAL, "bad scan arguments");
    if ((type == ACCB_PEER_F32 || type == ACCB_PEER_F64) && op > OP_MAX)
        return fail(p->ctx, ACCB_EINVAL, "bitwise combination of floating-point values");
    cudaStream_t s = (cudaStream_t)stream;
    const unsigned e = ++p->epoch;
#define ACCB_PEER_LAUNCH(T)                                                                                      \
    peer_exscan_kernel<T><<<1, 256, 0, s>>>(p->pp, p->rank, p->world, e, offset, count, op, static_cast<const T *>(first), \
                                            static_cast<T *>(dst))
    switch (type) {
        case ACCB_PEER_I32: ACCB_PEER_LAUNCH(int); break;
        case ACCB_PEER_U32: ACCB_PEER_LAUNCH(unsigned); break;
        case ACCB_PEER_I64: ACCB_PEER_LAUNCH(long long); break;
        case ACCB_PEER_F32: ACCB_PEER_LAUNCH(float); break;
        default: ACCB_PEER_LAUNCH(double); break;
    }
#undef ACCB_PEER_LAUNCH
    p->ctx->launches++;
    return check_cuda(p->ctx, cudaGetLastError(), "peer exclusive scan");
}

int accb_peer_pull(accb_peer *p, accb_stream stream, int from_rank, size_t offset, size_t bytes, void *dst) {
    PLOCKP(p);
    int st = ready(p, offset, bytes);
    if (st != ACCB_OK) return st;
    if (from_rank < 0 || from_rank >= p->world || !dst || bytes % 16 || (reinterpret_cast<uintptr_t>(dst) & 15))
        return fail(p->ctx, ACCB_EINVAL, "pull moves 16-byte aligned multiples of 16 bytes from an existing rank");
    if (bytes == 0) return ACCB_OK;
    const int grid = (int)std::min<size_t>((bytes / 16 + 255) / 256, (size_t)p->ctx->sm_count * 4);
    peer_pull_kernel<<<grid, 256, 0, (cudaStream_t)stream>>>(p->pp, from_rank, offset, bytes, static_cast<uint4 *>(dst));
    p->ctx->launches++;
    return check_cuda(p->ctx, cudaGetLastError(), "peer pull");
}

}  // extern "C"

namespace accb_rt {
/* what the block-cyclic scan driver (ops.cc) needs to know about an exchange buffer; `count` makes this call
 * the next scan on the buffer */
int peer_scan_begin(accb_peer *p, size_t offset, size_t bytes, PeerScanInfo *info, bool count) {
    if (!p || !info) return fail(nullptr, ACCB_EINVAL, "null peer object");
    int st = ready(p, offset, bytes);
    if (st != ACCB_OK) return st;
    if (p->world > 1 && !p->dev_bases) return fail(p->ctx, ACCB_EINVAL, "peer buffers are not connected yet");
    if (!p->dev_bases) {
        st = make_table(p);
        if (st != ACCB_OK) return st;
    }
    info->ctx = p->ctx;
    info->rank = p->rank;
    info->world = p->world;
    info->dev_bases = p->dev_bases;
    info->header_bytes = kHeader;
    info->timeout_ns = p->pp.timeout_ns;
    info->count = count ? ++p->scans : p->scans;
    info->piece = &p->piece;
    return ACCB_OK;
}
accb_context *peer_context(accb_peer *p) { return p ? p->ctx : nullptr; }
}  // namespace accb_rt

extern "C" {

int accb_peer_destroy(accb_peer *p) {
    if (!p) return ACCB_OK;
    {
        std::lock_guard<std::recursive_mutex> lock_(p->ctx->mu);
        CtxGuard guard_(p->ctx);
        cudaDeviceSynchronize();
        for (int r = 0; r < p->world; ++r)
            if (r != p->rank && p->pp.base[r] && p->pp.base[r] != p->local) cudaIpcCloseMemHandle(p->pp.base[r]);
        if (p->local) cudaFree(p->local);
        if (p->dev_bases) cudaFree(p->dev_bases);
    }
    delete p;
    return ACCB_OK;
}

}  // extern "C"
