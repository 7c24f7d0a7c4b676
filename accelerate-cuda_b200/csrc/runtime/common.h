/*
 * common.h -- shared declarations of the host runtime behind accb200.h.
 *
 * The runtime is the C++ counterpart of accelerate-cuda's Haskell host code:
 * State/Context (Data/Array/Accelerate/CUDA/State.hs, Context.hs), the memory
 * table (Array/Remote.hs, Array/Prim.hs), the kernel table (Compile.hs,
 * Persistent.hs), launch analysis (Analysis/Launch.hs) and the per-skeleton
 * drivers of Execute.hs.
 */
#pragma once
#include <cuda.h>
#include <cuda_runtime_api.h>

#include <atomic>
#include <condition_variable>
#include <cstdarg>
#include <cstdint>
#include <cstdio>
#include <cstring>
#include <future>
#include <map>
#include <memory>
#include <mutex>
#include <set>
#include <string>
#include <unordered_map>
#include <vector>

#include "../../../include/accb200.h"
#include "../cubits/accb_params.h"
#include "memtable.h"

namespace accb_rt {

/* ---- driver API, resolved at run time so that the library loads (and its
 * symbol table can be inspected) on a machine without libcuda ---- */
struct Driver {
    bool ok = false;
    std::string why;
    CUresult (*ModuleLoadData)(CUmodule *, const void *) = nullptr;
    CUresult (*ModuleUnload)(CUmodule) = nullptr;
    CUresult (*ModuleGetFunction)(CUfunction *, CUmodule, const char *) = nullptr;
    CUresult (*ModuleGetGlobal)(CUdeviceptr *, size_t *, CUmodule, const char *) = nullptr;
    CUresult (*FuncGetAttribute)(int *, CUfunction_attribute, CUfunction) = nullptr;
    CUresult (*FuncSetAttribute)(CUfunction, CUfunction_attribute, int) = nullptr;
    CUresult (*OccupancyMaxActiveBlocksPerMultiprocessor)(int *, CUfunction, int, size_t) = nullptr;
    CUresult (*LaunchKernel)(CUfunction, unsigned, unsigned, unsigned, unsigned, unsigned, unsigned, unsigned,
                             CUstream, void **, void **) = nullptr;
    CUresult (*LaunchKernelEx)(const CUlaunchConfig *, CUfunction, void **, void **) = nullptr; /* optional */
    CUresult (*CtxPushCurrent)(CUcontext) = nullptr;
    CUresult (*CtxPopCurrent)(CUcontext *) = nullptr;
    CUresult (*GetErrorString)(CUresult, const char **) = nullptr;
    CUresult (*MemcpyDtoH)(void *, CUdeviceptr, size_t) = nullptr;
    CUresult (*DevicePrimaryCtxGetState)(CUdevice, unsigned *, int *) = nullptr;
    CUresult (*TensorMapEncodeTiled)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *, const cuuint64_t *,
                                     const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave, CUtensorMapSwizzle,
                                     CUtensorMapL2promotion, CUtensorMapFloatOOBfill) = nullptr;
};
const Driver &driver();

/* ---- kernel table ---- */
struct SkeletonDesc {
    const char *name;     /* C-ABI name */
    const char *header;   /* file under skeletons/ */
    const char *macro;    /* instantiation macro */
    int id;
};
enum SkeletonId { SK_MAP = 1, SK_FOLD_ALL, SK_FOLD_DIM, SK_FOLD_SEG, SK_SCAN, SK_PERMUTE, SK_PERMUTE_SMEM,
                  SK_STENCIL, SK_STENCIL2, SK_STENCIL3 };
const SkeletonDesc *find_skeleton(const char *name);

struct CompileResult {
    int status = ACCB_OK;
    std::string log;
    std::string cubin; /* bytes */
    int source = 0;    /* 1 memory, 2 disk, 3 compiled */
};

struct KernelMeta {
    int v[12] = {0}; /* what accb_meta_query of the module reports (ACCB_META12 of cubits/accb_types.cuh) */
};

struct LoadedModule {
    CUmodule mod = nullptr;
    KernelMeta meta;
    std::unordered_map<std::string, CUfunction> fn;
};

}  // namespace accb_rt

struct accb_kernel {
    std::string key;  /* hex hash */
    int skeleton = 0;
    std::shared_future<accb_rt::CompileResult> result;
    std::mutex mu;
    std::map<accb_context *, accb_rt::LoadedModule> loaded; /* one module per context */
    std::atomic<int> refs{1};
};

struct accb_event {
    cudaEvent_t ev = nullptr;
};

namespace accb_rt {

constexpr int kRowCounterBase = 16; /* first row counter in StreamScratch::words */
constexpr int kRowCounters = 4096;  /* most rows a split fold takes */
constexpr int kDeferredBase = kRowCounterBase + kRowCounters; /* accb_deferred_segments of foldSeg (8-byte aligned) */
constexpr int kDeferredWords = (int)(sizeof(accb_deferred_segments) / sizeof(unsigned));

struct StreamScratch {
    void *status = nullptr;       /* scan tile status */
    size_t status_bytes = 0;
    int status_layout = 0;        /* bytes per tile record of the last scan */
    void *partial = nullptr;      /* fold partials */
    size_t partial_bytes = 0;
    unsigned *words = nullptr;    /* [0] fold ticket, [1] scan ticket, [2] error word,
                                     [kRowCounterBase..] per-row arrival counters of a split fold,
                                     [kDeferredBase..] the list of segments a foldSeg hands to its second launch */
    unsigned scan_ticket = 0;     /* host mirror of words[1] */
    unsigned epoch = 0;           /* scan launches so far (below 2^29) */
    unsigned graph_epoch = 0;     /* scan launches recorded inside stream captures (offset by 2^29) */
};

struct CudaAllocator : DeviceAllocator {
    void *alloc(size_t bytes) override;
    void release(void *p) override;
    bool copy_to_host(void *host, const void *dev, size_t bytes) override;
    void wait_token(void *token) override;    /* tokens are CUDA events */
    void release_token(void *token) override;
};

}  // namespace accb_rt

namespace accb_rt {
/* Tuning knobs, read from the environment ONCE when a context is created (never on the launch path):
 *   ACCB_FOLD_STAGE_MAX, ACCB_FOLD_NO_STAGE, ACCB_FOLDSEG_STAGE_MAX, ACCB_FOLDSEG_STAGE_FILL8,
 *   ACCB_FOLDSEG_STAGE_LANES, ACCB_FOLDSEG_NO_DEFER, ACCB_PERMUTE_REPLICAS, ACCB_STENCIL_NO_TILE, ACCB_STENCIL_NO_FUSE, ACCB_STENCIL_ROWS,
 *   ACCB_PIPELINE_CHUNK_LOG2, ACCB_NO_PIPELINE, ACCB_TRANSPOSE_TMA (0 or 1). */
struct Tuning {
    long long fold_stage_max = 128;    /* longest row the staged thread-per-row fold takes */
    bool fold_no_stage = false;
    long long foldseg_stage_max = 384; /* longest average segment the staged foldSeg takes */
    int foldseg_fill8 = 6;             /* eighths of the shared-memory window a run of segments aims to fill */
    int foldseg_lanes = 0;             /* lanes per segment of the staged foldSeg; 0: by segment length */
    bool foldseg_no_defer = false;     /* never hand long segments over to a second launch */
    int permute_replicas = 4;          /* shared-memory copies of a privatised permute destination */
    bool stencil_no_tile = false;
    bool stencil_no_fuse = false;      /* iterated stencils: never two applications per launch */
    int stencil_rows = 64;             /* band height of the register-form stencil */
    bool transpose_tma = true;         /* transposed maps of one 4-byte value through tensor-map copies */
    int pipeline_chunk_log2 = 0;       /* chunk of the host pipeline; 0: default */
    bool no_pipeline = false;
    void read_environment();
};
}  // namespace accb_rt

struct accb_context {
    int device = 0;
    CUcontext foreign = nullptr; /* non-null: a context the caller owns */
    int sm_count = 0, cc_major = 0, cc_minor = 0;
    size_t total_mem = 0;
    std::recursive_mutex mu;
    std::string last_error;
    accb_rt::CudaAllocator allocator;
    accb_rt::MemTable mem{&allocator};
    std::vector<cudaStream_t> stream_pool;     /* idle streams (reservoir) */
    std::vector<cudaEvent_t> event_pool;       /* idle events */
    std::map<cudaStream_t, accb_rt::StreamScratch> scratch;
    void *l2_flush = nullptr;
    size_t l2_flush_bytes = 0;
    unsigned long long launches = 0;
    unsigned long long buffer_generation = 0; /* bumped whenever a scratch or pooled buffer is replaced */
    std::set<CUfunction> carveout_set; /* entries already told to prefer shared memory over L1 */
    std::map<std::tuple<CUfunction, int, size_t>, int> occupancy_cache; /* resident blocks per SM */
    size_t mem_hits = 0, disk_hits = 0, compiles = 0;
    bool trace_exec = false, trace_gc = false, trace_cc = false;
    accb_rt::Tuning tune;
    std::set<void *> loops_unchecked; /* counter words of device-resident awhile loops whose overrun flag nobody has read yet */
};

namespace accb_rt {

/* makes the context's device (or foreign CUcontext) current for a scope */
struct CtxGuard {
    accb_context *c;
    bool pushed = false;
    int previous = -1; /* the device to make current again when the scope ends, or -1 */
    explicit CtxGuard(accb_context *ctx);
    ~CtxGuard();
};

int fail(accb_context *ctx, int code, const char *fmt, ...);
int check_cuda(accb_context *ctx, cudaError_t e, const char *what);
int check_cu(accb_context *ctx, CUresult e, const char *what);
void set_global_error(const std::string &s);

StreamScratch *scratch_for(accb_context *ctx, cudaStream_t s);

/* kernel cache */
std::string cache_key(const SkeletonDesc *sk, const char *src, const char *name, const char *flags);
std::string make_source(const SkeletonDesc *sk, const char *src, const char *name);
CompileResult compile_or_load(const std::string &key, const std::string &source, const char *flags,
                              const char *cache_dir_override);
std::string default_cache_dir();
std::string preseed_cache_dir();
std::string include_dir();
bool trace_enabled(const char *family);

/* launching */
int get_function(accb_context *ctx, accb_kernel *k, const char *entry, CUfunction *fn, KernelMeta *meta);
void forget_context(accb_context *ctx); /* unload the modules loaded for a context that is being destroyed */
int occupancy(accb_context *ctx, CUfunction fn, int block, size_t smem, int *blocks_per_sm);
int launch(accb_context *ctx, CUfunction fn, const char *name, int grid, int block, size_t smem,
           cudaStream_t stream, const accb_kparams &p, bool prefer_smem = true, void *extra1 = nullptr, void *extra2 = nullptr);
/* a launch whose blocks may be scheduled while the launch before it on the stream drains; its kernel waits for
 * that launch's results itself (griddepcontrol.wait) before it reads them */
int launch_dependent(accb_context *ctx, CUfunction fn, const char *name, int grid, int block, cudaStream_t stream,
                     const accb_kparams &p);

/* exchange buffers (peer.cu), as the block-cyclic scan driver sees them */
struct PieceState;
struct PeerScanInfo {
    accb_context *ctx = nullptr;
    int rank = 0, world = 1;
    void *dev_bases = nullptr;         /* device table: address of every rank's buffer */
    size_t header_bytes = 0;           /* the data area starts this far into a buffer */
    unsigned long long timeout_ns = 0; /* how long a rank waits for the others */
    unsigned count = 0;                /* number of this scan on the buffer (the same on every rank) */
    struct PieceState *piece = nullptr; /* the scan that is being launched piece by piece, if any */
};
/* a block-cyclic scan launched in pieces keeps its epochs from piece to piece */
struct PieceState {
    bool open = false;
    unsigned count = 0, epoch = 0;
    long long n_global = 0, block_elems = 0, next_block = 0;
    cudaStream_t stream = nullptr;
};
int peer_scan_begin(accb_peer *p, size_t offset, size_t bytes, PeerScanInfo *info, bool count);
accb_context *peer_context(accb_peer *p);

/* dst[i] = src[i] - src[0] for n values on the device: segment offsets of a slice made to start at zero */
int rebase_offsets(accb_context *ctx, cudaStream_t s, int *dst, const int *src, long long n);

/* host fault injection: ACCB_FAIL=<site>[:N] makes the N-th call at <site>
 * fail (sites: malloc, nvcc, cache_io) */
bool inject_failure(const char *site);

}  // namespace accb_rt
