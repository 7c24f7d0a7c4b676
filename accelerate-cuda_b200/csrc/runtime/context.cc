/*
 * context.cc -- contexts, error reporting, stream / event reservoirs and the
 * C-ABI face of the device memory table.
 *
 * Replaces Data/Array/Accelerate/CUDA/Context.hs:44-127, State.hs:61-132,
 * Execute/Stream.hs:52-140, Execute/Event.hs:38-140 and the transfer
 * functions of Array/Prim.hs:189-391.
 */
#include <dlfcn.h>

#include <algorithm>
#include <cstdlib>

#include "common.h"

namespace accb_rt {

static thread_local std::string g_error;
void set_global_error(const std::string &s) { g_error = s; }

const Driver &driver() {
    static Driver d;
    static std::once_flag once;
    std::call_once(once, [] {
        void *h = dlopen("libcuda.so.1", RTLD_NOW | RTLD_GLOBAL);
        if (!h) {
            d.why = std::string("cannot load libcuda.so.1: ") + dlerror();
            return;
        }
        bool ok = true;
        auto sym = [&](const char *name) {
            void *p = dlsym(h, name);
            if (!p) {
                ok = false;
                d.why = std::string("missing driver symbol ") + name;
            }
            return p;
        };
        d.ModuleLoadData = (decltype(d.ModuleLoadData))sym("cuModuleLoadData");
        d.ModuleUnload = (decltype(d.ModuleUnload))sym("cuModuleUnload");
        d.ModuleGetFunction = (decltype(d.ModuleGetFunction))sym("cuModuleGetFunction");
        d.ModuleGetGlobal = (decltype(d.ModuleGetGlobal))sym("cuModuleGetGlobal_v2");
        d.FuncGetAttribute = (decltype(d.FuncGetAttribute))sym("cuFuncGetAttribute");
        d.FuncSetAttribute = (decltype(d.FuncSetAttribute))sym("cuFuncSetAttribute");
        d.OccupancyMaxActiveBlocksPerMultiprocessor =
            (decltype(d.OccupancyMaxActiveBlocksPerMultiprocessor))sym("cuOccupancyMaxActiveBlocksPerMultiprocessor");
        d.LaunchKernel = (decltype(d.LaunchKernel))sym("cuLaunchKernel");
        d.CtxPushCurrent = (decltype(d.CtxPushCurrent))sym("cuCtxPushCurrent_v2");
        d.CtxPopCurrent = (decltype(d.CtxPopCurrent))sym("cuCtxPopCurrent_v2");
        d.GetErrorString = (decltype(d.GetErrorString))sym("cuGetErrorString");
        d.MemcpyDtoH = (decltype(d.MemcpyDtoH))sym("cuMemcpyDtoH_v2");
        d.DevicePrimaryCtxGetState = (decltype(d.DevicePrimaryCtxGetState))sym("cuDevicePrimaryCtxGetState");
        /* optional: lets a second launch be scheduled while its predecessor drains */
        d.LaunchKernelEx = (decltype(d.LaunchKernelEx))dlsym(h, "cuLaunchKernelEx");
        /* optional: only the tensor-map form of the transposed map needs it */
        d.TensorMapEncodeTiled = (decltype(d.TensorMapEncodeTiled))dlsym(h, "cuTensorMapEncodeTiled");
        d.ok = ok;
    });
    return d;
}

int fail(accb_context *ctx, int code, const char *fmt, ...) {
    char buf[4096];
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(buf, sizeof buf, fmt, ap);
    va_end(ap);
    if (ctx)
        ctx->last_error = buf;
    else
        g_error = buf;
    return code;
}

int check_cuda(accb_context *ctx, cudaError_t e, const char *what) {
    if (e == cudaSuccess) return ACCB_OK;
    return fail(ctx, e == cudaErrorMemoryAllocation ? ACCB_ENOMEM : ACCB_ECUDA, "%s: %s (%s)", what,
                cudaGetErrorString(e), cudaGetErrorName(e));
}

int check_cu(accb_context *ctx, CUresult e, const char *what) {
    if (e == CUDA_SUCCESS) return ACCB_OK;
    const char *s = nullptr;
    if (driver().GetErrorString) driver().GetErrorString(e, &s);
    return fail(ctx, ACCB_ECUDA, "%s: %s (CUresult %d)", what, s ? s : "?", (int)e);
}

bool trace_enabled(const char *family) {
    const char *t = getenv("ACCB_TRACE");
    return t && strstr(t, family) != nullptr;
}

bool inject_failure(const char *site) {
    /* ACCB_FAIL=<site>[:N]: the N-th call (1-based, default 1) at <site> fails */
    static std::mutex mu;
    static std::map<std::string, int> counts;
    const char *spec = getenv("ACCB_FAIL");
    if (!spec) return false;
    const size_t len = strlen(site);
    if (strncmp(spec, site, len) != 0 || (spec[len] != 0 && spec[len] != ':')) return false;
    const int nth = spec[len] == ':' ? atoi(spec + len + 1) : 1;
    std::lock_guard<std::mutex> g(mu);
    return ++counts[site] == nth;
}

void Tuning::read_environment() {
    auto num = [](const char *name, long long dflt) {
        const char *e = getenv(name);
        return e ? atoll(e) : dflt;
    };
    fold_stage_max = num("ACCB_FOLD_STAGE_MAX", fold_stage_max);
    fold_no_stage = getenv("ACCB_FOLD_NO_STAGE") != nullptr;
    foldseg_stage_max = num("ACCB_FOLDSEG_STAGE_MAX", foldseg_stage_max);
    foldseg_fill8 = (int)std::min(8LL, std::max(1LL, num("ACCB_FOLDSEG_STAGE_FILL8", foldseg_fill8)));
    foldseg_lanes = (int)std::max(0LL, num("ACCB_FOLDSEG_STAGE_LANES", 0));
    foldseg_no_defer = getenv("ACCB_FOLDSEG_NO_DEFER") != nullptr;
    permute_replicas = (int)std::max(1LL, num("ACCB_PERMUTE_REPLICAS", permute_replicas));
    stencil_no_tile = getenv("ACCB_STENCIL_NO_TILE") != nullptr;
    stencil_no_fuse = getenv("ACCB_STENCIL_NO_FUSE") != nullptr;
    stencil_rows = (int)std::max(1LL, num("ACCB_STENCIL_ROWS", stencil_rows));
    transpose_tma = num("ACCB_TRANSPOSE_TMA", 1) != 0;
    pipeline_chunk_log2 = (int)num("ACCB_PIPELINE_CHUNK_LOG2", 0);
    no_pipeline = getenv("ACCB_NO_PIPELINE") != nullptr;
}

CtxGuard::CtxGuard(accb_context *ctx) : c(ctx) {
    if (!c) return;
    if (c->foreign) {
        pushed = driver().CtxPushCurrent(c->foreign) == CUDA_SUCCESS;
    } else {
        /* the caller's current device comes back when the scope ends -- but only if that device already has a
         * primary context: making a device current creates one, and a process that never touched, say,
         * device 0 must not start holding memory there because a library call passed through */
        int cur = -1;
        if (cudaGetDevice(&cur) == cudaSuccess && cur != c->device) {
            unsigned flags = 0;
            int active = 0;
            if (driver().DevicePrimaryCtxGetState((CUdevice)cur, &flags, &active) == CUDA_SUCCESS && active) previous = cur;
        }
        if (cur != c->device) cudaSetDevice(c->device);
    }
}
CtxGuard::~CtxGuard() {
    if (pushed) {
        CUcontext old;
        driver().CtxPopCurrent(&old);
    }
    if (previous >= 0) cudaSetDevice(previous);
}

void *CudaAllocator::alloc(size_t bytes) {
    if (inject_failure("malloc")) return nullptr;
    void *p = nullptr;
    cudaError_t e = cudaMalloc(&p, bytes);
    if (e != cudaSuccess) {
        cudaGetLastError(); /* out of memory is the signal to evict, not a sticky error */
        return nullptr;
    }
    return p;
}
void CudaAllocator::release(void *p) { cudaFree(p); }
bool CudaAllocator::copy_to_host(void *host, const void *dev, size_t bytes) {
    return cudaMemcpy(host, dev, bytes, cudaMemcpyDeviceToHost) == cudaSuccess;
}

void CudaAllocator::wait_token(void *token) { cudaEventSynchronize(static_cast<cudaEvent_t>(token)); }
void CudaAllocator::release_token(void *token) { cudaEventDestroy(static_cast<cudaEvent_t>(token)); }

/* an event recorded behind everything enqueued on `s` so far, as a memory-table waypoint */
static void *waypoint_after(cudaStream_t s) {
    cudaEvent_t ev = nullptr;
    if (cudaEventCreateWithFlags(&ev, cudaEventDisableTiming) != cudaSuccess) return nullptr;
    if (cudaEventRecord(ev, s) != cudaSuccess) {
        cudaEventDestroy(ev);
        return nullptr;
    }
    return ev;
}

StreamScratch *scratch_for(accb_context *ctx, cudaStream_t s) {
    auto it = ctx->scratch.find(s);
    if (it != ctx->scratch.end()) return &it->second;
    StreamScratch sc;
    const size_t bytes = (kDeferredBase + kDeferredWords) * sizeof(unsigned);
    if (cudaMalloc((void **)&sc.words, bytes) != cudaSuccess) return nullptr;
    if (cudaMemsetAsync(sc.words, 0, bytes, s) != cudaSuccess) return nullptr;
    return &(ctx->scratch[s] = sc);
}

}  // namespace accb_rt

using namespace accb_rt;

#define LOCK(ctx)                                        \
    if (!(ctx)) return fail(nullptr, ACCB_EINVAL, "null context"); \
    std::lock_guard<std::recursive_mutex> lock_((ctx)->mu);        \
    CtxGuard guard_(ctx)

extern "C" {

const char *accb_version(void) { return "0.1.0"; }

int accb_init(void) {
    const Driver &d = driver();
    if (!d.ok) return fail(nullptr, ACCB_ENODRIVER, "%s", d.why.c_str());
    int n = 0;
    return check_cuda(nullptr, cudaGetDeviceCount(&n), "cudaGetDeviceCount");
}

int accb_device_count(int *count) {
    if (!count) return fail(nullptr, ACCB_EINVAL, "null count");
    return check_cuda(nullptr, cudaGetDeviceCount(count), "cudaGetDeviceCount");
}

const char *accb_last_error(accb_context *ctx) { return ctx ? ctx->last_error.c_str() : g_error.c_str(); }

int accb_context_create(int device, void *cu_context, accb_context **out) {
    if (!out) return fail(nullptr, ACCB_EINVAL, "null out pointer");
    *out = nullptr;
    int st = accb_init();
    if (st != ACCB_OK) return st;
    int n = 0;
    cudaGetDeviceCount(&n);
    if (device < 0 || device >= n) return fail(nullptr, ACCB_EINVAL, "device %d out of range (%d devices)", device, n);
    std::unique_ptr<accb_context> c(new accb_context);
    c->device = device;
    c->foreign = (CUcontext)cu_context;
    CtxGuard g(c.get());
    if (!c->foreign) {
        st = check_cuda(nullptr, cudaFree(0), "initialising the primary context");
        if (st != ACCB_OK) return st;
    }
    cudaDeviceProp prop;
    st = check_cuda(nullptr, cudaGetDeviceProperties(&prop, device), "cudaGetDeviceProperties");
    if (st != ACCB_OK) return st;
    c->sm_count = prop.multiProcessorCount;
    c->cc_major = prop.major;
    c->cc_minor = prop.minor;
    c->total_mem = prop.totalGlobalMem;
    c->trace_exec = trace_enabled("exec");
    c->trace_gc = trace_enabled("gc");
    c->trace_cc = trace_enabled("cc");
    c->tune.read_environment();
    if (c->cc_major != 10)
        return fail(nullptr, ACCB_EINVAL, "device %d is sm_%d%d; this library only carries sm_100a code", device,
                    prop.major, prop.minor);
    *out = c.release();
    return ACCB_OK;
}

int accb_context_destroy(accb_context *ctx) {
    if (!ctx) return ACCB_OK;
    {
        std::lock_guard<std::recursive_mutex> lock_(ctx->mu);
        CtxGuard g(ctx);
        cudaDeviceSynchronize();
        forget_context(ctx);
        ctx->mem.clear();
        for (auto &kv : ctx->scratch) {
            cudaFree(kv.second.status);
            cudaFree(kv.second.partial);
            cudaFree(kv.second.words);
        }
        for (auto s : ctx->stream_pool) cudaStreamDestroy(s);
        for (auto e : ctx->event_pool) cudaEventDestroy(e);
        if (ctx->l2_flush) cudaFree(ctx->l2_flush);
    }
    delete ctx;
    return ACCB_OK;
}

int accb_context_sync(accb_context *ctx) {
    LOCK(ctx);
    int st = check_cuda(ctx, cudaDeviceSynchronize(), "cudaDeviceSynchronize");
    if (st != ACCB_OK) return st;
    for (auto &kv : ctx->scratch) {
        unsigned w[3] = {0, 0, 0};
        st = check_cuda(ctx, cudaMemcpy(w, kv.second.words, sizeof w, cudaMemcpyDeviceToHost), "reading status words");
        if (st != ACCB_OK) return st;
        if (w[2] != 0) {
            cudaMemset(kv.second.words + 2, 0, sizeof(unsigned));
            return fail(ctx, ACCB_ETIMEOUT, "a bounded device-side wait (scan look-back or permute lock) gave up");
        }
    }
    /* device-resident awhile loops started without an iteration count: were they cut off at max_iters? */
    std::set<void *> loops;
    loops.swap(ctx->loops_unchecked);
    for (void *words : loops) {
        unsigned long long w[2] = {0, 0};
        st = check_cuda(ctx, cudaMemcpy(w, words, sizeof w, cudaMemcpyDeviceToHost), "reading loop words");
        if (st != ACCB_OK) return st;
        if (w[1]) return fail(ctx, ACCB_ETIMEOUT, "awhile: still true after %lld iterations", (long long)w[0]);
    }
    return ACCB_OK;
}

int accb_device_info(accb_context *ctx, int *sm_count, size_t *total_mem, int *cc_major, int *cc_minor) {
    LOCK(ctx);
    if (sm_count) *sm_count = ctx->sm_count;
    if (total_mem) *total_mem = ctx->total_mem;
    if (cc_major) *cc_major = ctx->cc_major;
    if (cc_minor) *cc_minor = ctx->cc_minor;
    return ACCB_OK;
}

/* ------------------------------------------------------ streams / events */
int accb_stream_acquire(accb_context *ctx, accb_stream *stream) {
    LOCK(ctx);
    if (!stream) return fail(ctx, ACCB_EINVAL, "null stream pointer");
    if (!ctx->stream_pool.empty()) {
        *stream = ctx->stream_pool.back();
        ctx->stream_pool.pop_back();
        return ACCB_OK;
    }
    cudaStream_t s;
    int st = check_cuda(ctx, cudaStreamCreateWithFlags(&s, cudaStreamNonBlocking), "cudaStreamCreate");
    if (st == ACCB_OK) *stream = s;
    return st;
}

int accb_stream_release(accb_context *ctx, accb_stream stream) {
    LOCK(ctx);
    if (stream) ctx->stream_pool.push_back((cudaStream_t)stream); /* reused once its work has drained */
    return ACCB_OK;
}

int accb_stream_sync(accb_context *ctx, accb_stream stream) {
    LOCK(ctx);
    return check_cuda(ctx, cudaStreamSynchronize((cudaStream_t)stream), "cudaStreamSynchronize");
}

int accb_event_record(accb_context *ctx, accb_stream stream, accb_event **event) {
    LOCK(ctx);
    if (!event) return fail(ctx, ACCB_EINVAL, "null event pointer");
    cudaEvent_t ev;
    if (!ctx->event_pool.empty()) {
        ev = ctx->event_pool.back();
        ctx->event_pool.pop_back();
    } else {
        int st = check_cuda(ctx, cudaEventCreateWithFlags(&ev, cudaEventDisableTiming), "cudaEventCreate");
        if (st != ACCB_OK) return st;
    }
    int st = check_cuda(ctx, cudaEventRecord(ev, (cudaStream_t)stream), "cudaEventRecord");
    if (st != ACCB_OK) return st;
    *event = new accb_event{ev};
    return ACCB_OK;
}

int accb_stream_wait_event(accb_context *ctx, accb_stream stream, accb_event *event) {
    LOCK(ctx);
    if (!event) return fail(ctx, ACCB_EINVAL, "null event");
    return check_cuda(ctx, cudaStreamWaitEvent((cudaStream_t)stream, event->ev, 0), "cudaStreamWaitEvent");
}

int accb_event_sync(accb_context *ctx, accb_event *event) {
    LOCK(ctx);
    if (!event) return fail(ctx, ACCB_EINVAL, "null event");
    return check_cuda(ctx, cudaEventSynchronize(event->ev), "cudaEventSynchronize");
}

int accb_event_query(accb_context *ctx, accb_event *event, int *done) {
    LOCK(ctx);
    if (!event || !done) return fail(ctx, ACCB_EINVAL, "null argument");
    cudaError_t e = cudaEventQuery(event->ev);
    if (e == cudaSuccess) {
        *done = 1;
        return ACCB_OK;
    }
    if (e == cudaErrorNotReady) {
        cudaGetLastError();
        *done = 0;
        return ACCB_OK;
    }
    return check_cuda(ctx, e, "cudaEventQuery");
}

int accb_event_release(accb_context *ctx, accb_event *event) {
    LOCK(ctx);
    if (!event) return ACCB_OK;
    ctx->event_pool.push_back(event->ev);
    delete event;
    return ACCB_OK;
}

/* --------------------------------------------------------- memory table */
int accb_malloc(accb_context *ctx, uint64_t key, size_t bytes, void **dptr) {
    LOCK(ctx);
    if (!dptr) return fail(ctx, ACCB_EINVAL, "null dptr");
    MemTable::Entry *e = ctx->mem.insert(key, bytes, nullptr);
    if (!e) return fail(ctx, ACCB_ENOMEM, "device out of memory allocating %zu bytes (nothing left to evict)", bytes);
    if (ctx->trace_gc) fprintf(stderr, "[accb gc] malloc key=%llx %zu B\n", (unsigned long long)key, bytes);
    *dptr = e->dptr;
    return ACCB_OK;
}

int accb_use(accb_context *ctx, uint64_t key, const void *host, size_t bytes, accb_stream stream, void **dptr) {
    LOCK(ctx);
    if (!dptr || !host) return fail(ctx, ACCB_EINVAL, "null argument");
    bool upload = false;
    MemTable::Entry *e = ctx->mem.find(key);
    if (e) {
        e = ctx->mem.ensure_resident(key, &upload);
        if (!e) return fail(ctx, ACCB_ENOMEM, "device out of memory restoring key %llx", (unsigned long long)key);
    } else {
        e = ctx->mem.insert(key, bytes, const_cast<void *>(host));
        if (!e) return fail(ctx, ACCB_ENOMEM, "device out of memory allocating %zu bytes", bytes);
        upload = true;
    }
    if (upload) {
        if (ctx->trace_gc) fprintf(stderr, "[accb gc] upload key=%llx %zu B\n", (unsigned long long)key, bytes);
        int st = check_cuda(ctx, cudaMemcpyAsync(e->dptr, host, bytes, cudaMemcpyHostToDevice, (cudaStream_t)stream),
                            "upload");
        if (st != ACCB_OK) return st;
        /* the copy is asynchronous: eviction must not free the destination under it */
        if (void *w = waypoint_after((cudaStream_t)stream)) ctx->mem.set_waypoint(key, w);
    }
    *dptr = e->dptr;
    return ACCB_OK;
}

int accb_insert_unmanaged(accb_context *ctx, uint64_t key, void *dptr, size_t bytes) {
    LOCK(ctx);
    if (!dptr) return fail(ctx, ACCB_EINVAL, "null dptr");
    ctx->mem.insert_unmanaged(key, dptr, bytes);
    return ACCB_OK;
}

int accb_with_ptr(accb_context *ctx, uint64_t key, void **dptr, size_t *bytes) {
    LOCK(ctx);
    bool upload = false;
    MemTable::Entry *e = ctx->mem.ensure_resident(key, &upload);
    if (!e) return fail(ctx, ACCB_ENOTFOUND, "unknown or unrestorable key %llx", (unsigned long long)key);
    if (upload) {
        int st = check_cuda(ctx, cudaMemcpy(e->dptr, e->host, e->bytes, cudaMemcpyHostToDevice), "re-upload");
        if (st != ACCB_OK) return st;
    }
    ctx->mem.pin(key);
    if (dptr) *dptr = e->dptr;
    if (bytes) *bytes = e->bytes;
    return ACCB_OK;
}

int accb_release(accb_context *ctx, uint64_t key) {
    LOCK(ctx);
    if (!ctx->mem.unpin(key)) return fail(ctx, ACCB_ENOTFOUND, "key %llx is not pinned", (unsigned long long)key);
    return ACCB_OK;
}

int accb_release_after(accb_context *ctx, uint64_t key, accb_stream stream) {
    LOCK(ctx);
    if (!ctx->mem.peek(key)) return fail(ctx, ACCB_ENOTFOUND, "unknown key %llx", (unsigned long long)key);
    /* the waypoint first: once unpinned the entry may be chosen for eviction at any time */
    void *w = waypoint_after((cudaStream_t)stream);
    if (!w) return fail(ctx, ACCB_ECUDA, "cannot record an event on the stream");
    ctx->mem.set_waypoint(key, w);
    if (!ctx->mem.unpin(key)) return fail(ctx, ACCB_ENOTFOUND, "key %llx is not pinned", (unsigned long long)key);
    return ACCB_OK;
}

static int resolve(accb_context *ctx, uint64_t key, size_t offset, size_t bytes, char **p) {
    bool upload = false;
    MemTable::Entry *e = ctx->mem.ensure_resident(key, &upload);
    if (!e) return fail(ctx, ACCB_ENOTFOUND, "unknown key %llx", (unsigned long long)key);
    if (upload) {
        int st = check_cuda(ctx, cudaMemcpy(e->dptr, e->host, e->bytes, cudaMemcpyHostToDevice), "re-upload");
        if (st != ACCB_OK) return st;
    }
    if (offset + bytes > e->bytes)
        return fail(ctx, ACCB_EBOUNDS, "range [%zu, %zu) outside an array of %zu bytes", offset, offset + bytes, e->bytes);
    *p = static_cast<char *>(e->dptr) + offset;
    return ACCB_OK;
}

int accb_peek(accb_context *ctx, uint64_t key, size_t offset, void *host, size_t bytes, accb_stream stream) {
    LOCK(ctx);
    char *p;
    int st = resolve(ctx, key, offset, bytes, &p);
    if (st != ACCB_OK) return st;
    return check_cuda(ctx, cudaMemcpyAsync(host, p, bytes, cudaMemcpyDeviceToHost, (cudaStream_t)stream), "peek");
}

int accb_poke(accb_context *ctx, uint64_t key, size_t offset, const void *host, size_t bytes, accb_stream stream) {
    LOCK(ctx);
    char *p;
    int st = resolve(ctx, key, offset, bytes, &p);
    if (st != ACCB_OK) return st;
    return check_cuda(ctx, cudaMemcpyAsync(p, host, bytes, cudaMemcpyHostToDevice, (cudaStream_t)stream), "poke");
}

int accb_copy(accb_context *ctx, uint64_t src_key, uint64_t dst_key, size_t bytes, accb_stream stream) {
    LOCK(ctx);
    char *s, *d;
    int st = resolve(ctx, src_key, 0, bytes, &s);
    if (st != ACCB_OK) return st;
    st = resolve(ctx, dst_key, 0, bytes, &d);
    if (st != ACCB_OK) return st;
    return check_cuda(ctx, cudaMemcpyAsync(d, s, bytes, cudaMemcpyDeviceToDevice, (cudaStream_t)stream), "copy");
}

int accb_copy_peer(accb_context *src_ctx, uint64_t src_key, accb_context *dst_ctx, uint64_t dst_key, size_t bytes,
                   accb_stream stream) {
    if (!src_ctx || !dst_ctx) return fail(nullptr, ACCB_EINVAL, "null context");
    char *s, *d;
    {
        std::lock_guard<std::recursive_mutex> l(src_ctx->mu);
        CtxGuard g(src_ctx);
        int st = resolve(src_ctx, src_key, 0, bytes, &s);
        if (st != ACCB_OK) return st;
    }
    std::lock_guard<std::recursive_mutex> l(dst_ctx->mu);
    CtxGuard g(dst_ctx);
    int st = resolve(dst_ctx, dst_key, 0, bytes, &d);
    if (st != ACCB_OK) return st;
    return check_cuda(dst_ctx,
                      cudaMemcpyPeerAsync(d, dst_ctx->device, s, src_ctx->device, bytes, (cudaStream_t)stream),
                      "peer copy");
}

int accb_index(accb_context *ctx, uint64_t key, size_t index, size_t elt_bytes, void *out) {
    LOCK(ctx);
    char *p;
    int st = resolve(ctx, key, index * elt_bytes, elt_bytes, &p);
    if (st != ACCB_OK) return st;
    return check_cuda(ctx, cudaMemcpy(out, p, elt_bytes, cudaMemcpyDeviceToHost), "index");
}

int accb_free(accb_context *ctx, uint64_t key) {
    LOCK(ctx);
    if (!ctx->mem.remove(key)) return fail(ctx, ACCB_ENOTFOUND, "unknown key %llx", (unsigned long long)key);
    return ACCB_OK;
}

int accb_reclaim(accb_context *ctx) {
    LOCK(ctx);
    int st = check_cuda(ctx, cudaDeviceSynchronize(), "cudaDeviceSynchronize");
    if (st != ACCB_OK) return st;
    size_t n = ctx->mem.reclaim();
    if (ctx->trace_gc) fprintf(stderr, "[accb gc] reclaim evicted %zu arrays\n", n);
    return ACCB_OK;
}

int accb_memory_stats(accb_context *ctx, size_t *entries, size_t *bytes_resident, size_t *evictions) {
    LOCK(ctx);
    if (entries) *entries = ctx->mem.entries();
    if (bytes_resident) *bytes_resident = ctx->mem.resident_bytes();
    if (evictions) *evictions = ctx->mem.evictions();
    return ACCB_OK;
}

} /* extern "C" */
