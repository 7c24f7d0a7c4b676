/*
 * accb200.h -- C ABI of the B200 execution backend for Accelerate's collective
 * operations (libaccb200.so).
 *
 * This header is the successor of accelerate-cuda's include/AccFFI.h:7-30 and
 * of the Haskell-internal interfaces behind it.  Each group below names the
 * reference interface it replaces (paths are relative to the accelerate-cuda
 * source tree).  Conventions:
 *   - every function returns an int status (ACCB_OK == 0); no exception and no
 *     process exit crosses this boundary (the reference's functions are void
 *     and a CUDA error terminates the process, Data/Array/Accelerate/CUDA/State.hs:84-92);
 *     accb_last_error() gives the message of the last failure on a context;
 *   - plain pointers and sizes only; device pointers are ordinary CUDA device
 *     pointers of the context's device; streams are cudaStream_t / CUstream
 *     passed as void*;
 *   - arrays of tuples are structure-of-arrays, one device pointer per
 *     flattened scalar component (CUDA/CodeGen/Base.hs:69-79);
 *   - shapes list the INNERMOST extent first, like the shape buffers of
 *     AccFFI.h (CUDA/Foreign/Export.hs:210-214,274-275);
 *   - all functions are thread-safe; calls on one context are serialised by an
 *     internal mutex except for the asynchronous device work they enqueue.
 */
#ifndef ACCB200_H
#define ACCB200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define ACCB_API __attribute__((visibility("default")))

/* ---------------------------------------------------------------- status */
enum {
    ACCB_OK = 0,
    ACCB_EINVAL = 1,    /* bad argument */
    ACCB_ECUDA = 2,     /* a CUDA runtime / driver call failed */
    ACCB_ENOMEM = 3,    /* device memory exhausted even after eviction */
    ACCB_ECOMPILE = 4,  /* nvcc failed; the log is in accb_last_error() */
    ACCB_EIO = 5,       /* kernel cache I/O */
    ACCB_EBOUNDS = 6,   /* e.g. fold1 of an empty array (CUDA/Execute.hs:283-285) */
    ACCB_ETIMEOUT = 7,  /* a bounded device-side wait gave up */
    ACCB_ENOTFOUND = 8, /* unknown key / entry point */
    ACCB_ENODRIVER = 9  /* libcuda.so.1 is not available */
};

typedef struct accb_context accb_context;
typedef struct accb_kernel accb_kernel;
typedef struct accb_event accb_event;
typedef void *accb_stream;

#define ACCB_ARRAY_MAX_RANK 4
#define ACCB_ARRAY_MAX_COMP 8

/* One array as the launch functions see it: replaces the Marshalable
 * instance for arrays (shape ints followed by one pointer per component,
 * CUDA/Execute.hs:823-873). */
typedef struct accb_array {
    int rank;                          /* 0 for a scalar */
    int shape[ACCB_ARRAY_MAX_RANK];    /* innermost extent first */
    int ncomp;                         /* flattened tuple components */
    void *ptr[ACCB_ARRAY_MAX_COMP];    /* device pointers, leftmost field first */
} accb_array;

/* ------------------------------------------------- runtime and contexts
 * replaces accelerateCreate / accelerateDestroy (include/AccFFI.h:21-30,
 * CUDA/Foreign/Export.hs:146-153), Context.create / destroy
 * (CUDA/Context.hs:55-93) and the global state of CUDA/State.hs:61-132.   */
ACCB_API int accb_init(void);
ACCB_API int accb_device_count(int *count);
ACCB_API const char *accb_version(void);
/* cu_context: NULL to use the device's primary context (shared with the CUDA
 * runtime and with PyTorch), or a CUcontext the caller owns. */
ACCB_API int accb_context_create(int device, void *cu_context, accb_context **ctx);
ACCB_API int accb_context_destroy(accb_context *ctx);
/* Waits for all work enqueued through this context and reports device-side
 * bounded-wait failures (ACCB_ETIMEOUT). */
ACCB_API int accb_context_sync(accb_context *ctx);
ACCB_API const char *accb_last_error(accb_context *ctx); /* ctx may be NULL */
ACCB_API int accb_device_info(accb_context *ctx, int *sm_count, size_t *total_mem, int *cc_major,
                              int *cc_minor);

/* ----------------------------------------------------- streams and events
 * replaces the stream reservoir and event table, CUDA/Execute/Stream.hs:52-140
 * and CUDA/Execute/Event.hs:38-140.                                        */
ACCB_API int accb_stream_acquire(accb_context *ctx, accb_stream *stream);
ACCB_API int accb_stream_release(accb_context *ctx, accb_stream stream);
ACCB_API int accb_stream_sync(accb_context *ctx, accb_stream stream);
ACCB_API int accb_event_record(accb_context *ctx, accb_stream stream, accb_event **event);
ACCB_API int accb_stream_wait_event(accb_context *ctx, accb_stream stream, accb_event *event);
ACCB_API int accb_event_sync(accb_context *ctx, accb_event *event);
ACCB_API int accb_event_query(accb_context *ctx, accb_event *event, int *done);
ACCB_API int accb_event_release(accb_context *ctx, accb_event *event);

/* ------------------------------------------------- device memory table
 * replaces CUDA/Array/Remote.hs:91-202 (malloc, withRemote, free,
 * insertUnmanaged, reclaim) and the typed transfer functions of
 * CUDA/Array/Prim.hs:159-472.  `key` identifies a host array (the reference
 * uses the host array's stable name).  Allocation sizes are rounded up to
 * 1024 bytes (Remote.hs:60-80).  When the device is full, least recently
 * used unpinned entries with a host copy are written back and evicted.    */
ACCB_API int accb_malloc(accb_context *ctx, uint64_t key, size_t bytes, void **dptr);
/* upload-if-absent of a host array (useArrayAsync, Prim.hs:226-234) */
ACCB_API int accb_use(accb_context *ctx, uint64_t key, const void *host, size_t bytes, accb_stream stream,
                      void **dptr);
/* register memory the caller owns; never freed by the table (Remote.hs:168-184) */
ACCB_API int accb_insert_unmanaged(accb_context *ctx, uint64_t key, void *dptr, size_t bytes);
/* pin / unpin an entry while device work uses it (withRemote, Remote.hs:113-134) */
ACCB_API int accb_with_ptr(accb_context *ctx, uint64_t key, void **dptr, size_t *bytes);
ACCB_API int accb_release(accb_context *ctx, uint64_t key);
/* unpin, and remember that work enqueued on `stream` so far still uses the entry: the table waits for that work
 * before it writes the entry back to the host, frees it or forgets it -- the waypoint event that withRemote
 * attaches to every use (Remote.hs:127-134).  accb_release alone is for callers that have synchronised. */
ACCB_API int accb_release_after(accb_context *ctx, uint64_t key, accb_stream stream);
ACCB_API int accb_peek(accb_context *ctx, uint64_t key, size_t offset, void *host, size_t bytes,
                       accb_stream stream); /* device -> host (peekArrayAsync) */
ACCB_API int accb_poke(accb_context *ctx, uint64_t key, size_t offset, const void *host, size_t bytes,
                       accb_stream stream); /* host -> device (pokeArrayAsync) */
ACCB_API int accb_copy(accb_context *ctx, uint64_t src_key, uint64_t dst_key, size_t bytes,
                       accb_stream stream); /* device -> device (copyArrayAsync) */
ACCB_API int accb_copy_peer(accb_context *src_ctx, uint64_t src_key, accb_context *dst_ctx, uint64_t dst_key,
                            size_t bytes, accb_stream stream); /* copyArrayPeerAsync, Prim.hs:306-335 */
/* read one element synchronously (indexArray, Prim.hs:189-211) */
ACCB_API int accb_index(accb_context *ctx, uint64_t key, size_t index, size_t elt_bytes, void *out);
ACCB_API int accb_free(accb_context *ctx, uint64_t key);    /* unsafeFree, CUDA.hs:421-431 */
ACCB_API int accb_reclaim(accb_context *ctx);               /* performGC, CUDA.hs:433-441 */
ACCB_API int accb_memory_stats(accb_context *ctx, size_t *entries, size_t *bytes_resident, size_t *evictions);

/* ---------------------------------------------------- kernel cache (JIT)
 * replaces build / compile / link of CUDA/Compile.hs:439-660 and the
 * two-level KernelTable of CUDA/Persistent.hs:77-378.
 * `skeleton` is one of "map", "fold_all", "fold_dim", "fold_seg", "scan",
 * "permute", "permute_smem", "stencil", "stencil2"; `functor_src` is C++
 * source defining a struct (what the scalar code generator CUDA/CodeGen.hs
 * prints for the user's functions); `functor_name` is that struct's name;
 * `nvcc_flags` may add -D options or NULL.  The result is looked up by
 * hash(arch, skeleton library, source, flags) in memory, then on disk, and
 * only then compiled with nvcc -arch=sm_100a -cubin in a worker thread; the
 * call returns at once and the first launch waits for the compiler
 * (the reference's lazy link, Compile.hs:444-459).                          */
ACCB_API int accb_kernel_get(accb_context *ctx, const char *skeleton, const char *functor_src,
                             const char *functor_name, const char *nvcc_flags, accb_kernel **kernel);
ACCB_API int accb_kernel_wait(accb_context *ctx, accb_kernel *kernel); /* block until linked */
/* registers, static shared memory, block size and resident blocks per SM of
 * an entry point (determineOccupancy, CUDA/Analysis/Launch.hs:62-74) */
ACCB_API int accb_kernel_info(accb_context *ctx, accb_kernel *kernel, const char *entry, int *regs,
                              int *static_smem, int *block, int *blocks_per_sm);
ACCB_API int accb_kernel_release(accb_context *ctx, accb_kernel *kernel);
/* Compile into a cache directory without a GPU (build-time pre-seeding). */
ACCB_API int accb_kernel_precompile(const char *skeleton, const char *functor_src, const char *functor_name,
                                    const char *nvcc_flags, const char *cache_dir, char *log, size_t log_bytes);
/* the cache key (32 hex digits) the library derives for a kernel: the name of
 * its cubin in the cache directories (Compile.hs:565, Persistent.hs:218-228) */
ACCB_API int accb_kernel_key(const char *skeleton, const char *functor_src, const char *functor_name,
                             const char *nvcc_flags, char *key, size_t key_bytes);
ACCB_API int accb_cache_flush(accb_context *ctx); /* -fflush-cache, Persistent.hs:305-344 */
ACCB_API int accb_cache_stats(accb_context *ctx, size_t *mem_hits, size_t *disk_hits, size_t *compiles);
/* grid the runtime would use for `n` elements (launchConfig, Launch.hs:42-55) */
ACCB_API int accb_launch_config(accb_context *ctx, accb_kernel *kernel, const char *entry, long long n,
                                int *block, int *grid, int *dynamic_smem);
ACCB_API int accb_launch_count(accb_context *ctx, unsigned long long *launches);

/* ------------------------------------------- skeleton launches (Execute)
 * replace executeOp, foldCore/foldRec, foldSegOp, scanOp/scan1Op/scan'Op,
 * permuteOp, stencilOp and stencil2Op of CUDA/Execute.hs:264-450 together
 * with configure/execute/launch (:930-982).  `env` are the free array
 * variables of the functor in Gamma order (CUDA/AST.hs:72-112); `scalars` is
 * a packed block of user scalars the functor reads with env.scalar<T>(off).
 * All launches are asynchronous on `stream`.                               */
ACCB_API int accb_map(accb_context *ctx, accb_kernel *k, accb_stream stream, const accb_array *env, int nenv,
                      const void *scalars, size_t scalar_bytes, const accb_array *out);
/* `map f (transpose m)` with the same kernel object as `map f m`: the environment arrays that the functor
 * reads element-wise are matrices of the transposed shape of `out` and go through 64x64 shared-memory tiles, so
 * that loads and stores are both contiguous.  In the reference a transpose is a backpermute, i.e. a gather
 * (mkTransform, CUDA/CodeGen/IndexSpace.hs:96-141). */
ACCB_API int accb_map_transposed(accb_context *ctx, accb_kernel *k, accb_stream stream, const accb_array *env,
                                 int nenv, const void *scalars, size_t scalar_bytes, const accb_array *out);

/* seed == NULL selects fold1 / fold1All (no seed) */
ACCB_API int accb_fold_all(accb_context *ctx, accb_kernel *k, accb_stream stream, const accb_array *env,
                           int nenv, long long n, const void *seed, size_t seed_bytes, const accb_array *out);
ACCB_API int accb_fold_dim(accb_context *ctx, accb_kernel *k, accb_stream stream, const accb_array *env,
                           int nenv, long long rows, long long cols, const void *seed, size_t seed_bytes,
                           const accb_array *out);
/* offsets: Int32 device array of nseg+1 exclusive-scanned segment lengths.  Segments may have any length: where a
 * thread, a warp or a block owns a segment, one that is far longer than the rest (65536 elements, or 2^20 under a
 * block) is put on a device-side list instead, and for sources of 2^24 elements and more (2^20 when there are too
 * few segments to fill the GPU with a block each) a second launch cuts the listed segments into pieces for all
 * blocks -- about three microseconds when the list stays empty. */
ACCB_API int accb_fold_seg(accb_context *ctx, accb_kernel *k, accb_stream stream, const accb_array *env,
                           int nenv, long long rows, long long cols, const int *offsets, long long nseg,
                           const void *seed, size_t seed_bytes, const accb_array *out);

enum { ACCB_SCAN_LEFT = 0, ACCB_SCAN_RIGHT = 1 };
enum {
    ACCB_SCAN_EXCLUSIVE = 0, /* scanl / scanr : out has n+1 elements            */
    ACCB_SCAN_INCLUSIVE = 1, /* scanl1 / scanr1: out has n elements, no seed    */
    ACCB_SCAN_PRIME = 2,     /* scanl' / scanr': out has n elements + `total`   */
    /* scanl1 / scanr1 continuing from a seed: out[i] = seed (+) x0 (+) .. (+) xi,
     * n elements.  How a later slab of a sharded scan1 continues from the carry
     * of the earlier slabs; the reference has no such form. */
    ACCB_SCAN_INCLUSIVE_SEEDED = 3
};
/* OR into `kind`: `seed` is a DEVICE pointer to the seed value, written by
 * earlier work on the same stream (the carry of a sharded scan). */
#define ACCB_SEED_ON_DEVICE 0x100
ACCB_API int accb_scan(accb_context *ctx, accb_kernel *k, accb_stream stream, const accb_array *env, int nenv,
                       long long n, int direction, int kind, const void *seed, size_t seed_bytes,
                       const accb_array *out, const accb_array *total);

/* The same launches over a PIECE of a larger array: `env` and `out` describe the piece, and the functor is told
 * index_base + position, i.e. the element's index in the whole array.  This is how a program whose input does
 * not fit, or has not arrived yet, is run piece by piece (accb_program_run_host streams host arrays this way:
 * while piece k is computed, piece k+1 is on its way to the device and the result of piece k-1 on its way back).
 *   fold_all  `carry` is NULL or a device pointer to what the pieces before this one came to (one value of the
 *             result type): the result is carry (f) fold of this piece [(f) seed], the carry on the LEFT.  Pass
 *             the seed with the last piece only.
 *   scan      continue from the previous piece with ACCB_SEED_ON_DEVICE (and ACCB_SCAN_INCLUSIVE_SEEDED for scanl1).
 *   permute   every piece combines into the same `out`; copy the defaults once, before the first piece.
 * No counterpart in the reference, which uploads whole arrays before the first launch (CUDA.hs:307-330). */
ACCB_API int accb_map_at(accb_context *ctx, accb_kernel *k, accb_stream stream, const accb_array *env, int nenv,
                         const void *scalars, size_t scalar_bytes, const accb_array *out, long long index_base);
ACCB_API int accb_fold_all_at(accb_context *ctx, accb_kernel *k, accb_stream stream, const accb_array *env,
                              int nenv, long long n, const void *seed, size_t seed_bytes, const accb_array *out,
                              long long index_base, const void *carry);
ACCB_API int accb_fold_dim_at(accb_context *ctx, accb_kernel *k, accb_stream stream, const accb_array *env,
                              int nenv, long long rows, long long cols, const void *seed, size_t seed_bytes,
                              const accb_array *out, long long index_base);
ACCB_API int accb_scan_at(accb_context *ctx, accb_kernel *k, accb_stream stream, const accb_array *env, int nenv,
                          long long n, int direction, int kind, const void *seed, size_t seed_bytes,
                          const accb_array *out, const accb_array *total, long long index_base);
ACCB_API int accb_permute_at(accb_context *ctx, accb_kernel *k, accb_stream stream, const accb_array *env,
                             int nenv, long long n_src, const void *scalars, size_t scalar_bytes,
                             const accb_array *out, long long index_base);

/* Int32 `scanl (+) seed` for callers that cannot allocate device memory.  It has
 * no counterpart in the reference, whose every scan allocates its block-sum
 * array (scanCore, CUDA/Execute.hs:364-392).  Meant for code that runs with a
 * memory budget fixed in advance or in a place where touching the allocator is
 * forbidden (a real-time loop, a callback of another library, a process whose
 * pool is fully handed out): the call performs no cudaMalloc / cudaFree and
 * needs no accb_context.  The tile status words live in a 1 MiB array that is
 * part of the library image and stays resident on every GPU that loads the
 * library until the process exits.
 *   - `in` (n elements) and `out` (n + 1 elements: out[0] = seed, out[n] = the
 *     total) are device pointers on `device`; the launch is asynchronous on
 *     `stream`.
 *   - n may be at most 2^28 (268 435 456) elements; larger inputs are refused
 *     with ACCB_EINVAL and a message in accb_last_error(NULL).
 *   - `status` is NULL or a device word the caller owns: it is cleared on the
 *     stream and set to 1 if a bounded device-side wait gave up.  With
 *     status == NULL such a failure cannot be observed: the output is then
 *     wrong without any signal, so pass a word unless the result is checked
 *     by other means.
 *   - Every call looks up the array's device address in the current CUDA
 *     context.  The first call on a device makes the CUDA runtime load the
 *     library's code there; make that first call before any stream capture
 *     begins.
 *   - All calls on a device share the one array, which keeps the previous
 *     call's contents; each call clears on `stream` what it will read.  Two
 *     calls that overlap on the GPU (different streams, no dependency between
 *     them) race on it: order them. */
ACCB_API int accb_scanl_add_i32_noalloc(int device, accb_stream stream, const int32_t *in, long long n,
                                        int32_t seed, int32_t *out, unsigned int *status);

/* out must already hold the default values (the reference copies them first,
 * Execute.hs:405-407); use accb_permute_defaults to do that copy. */
ACCB_API int accb_permute_defaults(accb_context *ctx, accb_stream stream, const accb_array *defaults,
                                   const accb_array *out, const int *comp_bytes);
ACCB_API int accb_permute(accb_context *ctx, accb_kernel *k, accb_stream stream, const accb_array *env,
                          int nenv, long long n_src, const void *scalars, size_t scalar_bytes,
                          const accb_array *out);

enum { ACCB_CLAMP = 0, ACCB_MIRROR = 1, ACCB_WRAP = 2, ACCB_CONSTANT = 3 };
ACCB_API int accb_stencil(accb_context *ctx, accb_kernel *k, accb_stream stream, const accb_array *src,
                          int boundary, const void *constant, size_t constant_bytes, const accb_array *out);
ACCB_API int accb_stencil2(accb_context *ctx, accb_kernel *k, accb_stream stream, const accb_array *src1,
                           const accb_array *src2, int boundary, const void *constant, size_t constant_bytes,
                           const accb_array *out);
/* `iters` applications ping-ponging between a and b; *result tells which of
 * the two holds the final grid.  Replaces a chain of Stencil nodes, each of
 * which allocates a fresh array in the reference (Execute.hs:413-425). */
ACCB_API int accb_stencil_iterate(accb_context *ctx, accb_kernel *k, accb_stream stream, const accb_array *a,
                                  const accb_array *b, int iters, int boundary, const void *constant,
                                  size_t constant_bytes, int *result_in_b);
/* The same with a source of its own that is only read: the first launch goes from `src` to a, the rest ping-pong
 * between a and b (iters >= 1).  Where the kernel has the form (rank 2, one 4-byte element type, 16-byte aligned
 * rows of a multiple of 4 elements, any boundary but Wrap), a launch does TWO applications -- the intermediate grid
 * of a block never leaves shared memory -- so an iterated stencil reads and writes the grid once per two
 * applications; the results are those of one application per launch bit for bit.  accb_stencil_iterate does the
 * same from a. */
ACCB_API int accb_stencil_iterate_from(accb_context *ctx, accb_kernel *k, accb_stream stream, const accb_array *src,
                                       const accb_array *a, const accb_array *b, int iters, int boundary,
                                       const void *constant, size_t constant_bytes, int *result_in_b);

/* -------------------------------------- whole programs (AccFFI.h surface)
 * Same struct layouts and entry points as include/AccFFI.h:10-30.  An
 * AccProgram is an op list built with accb_program_* instead of a Haskell
 * closure exported by Template Haskell (CUDA/Foreign/Export.hs:231-265).   */
typedef void *AccHandle;
typedef void *AccProgram;
typedef struct {
    int *shape;
    void **adata;
} InputArray;
typedef struct {
    int *shape;
    void **adata;
    void *stable_ptr;
} OutputArray;

ACCB_API AccHandle accelerateCreate(int32_t device, void *cu_context);
/* AccFFI.h:27-30 defines accelerateInit in the header itself: it starts the Haskell run-time system (hs_init) and
 * calls accelerateCreate.  There is no run-time system to start here, so argc / argv are ignored; C code written
 * against AccFFI.h compiles unchanged. */
static inline AccHandle accelerateInit(int argc, char **argv, int device, void *cu_context) {
    (void)argc;
    (void)argv;
    return accelerateCreate((int32_t)device, cu_context);
}
ACCB_API void accelerateDestroy(AccHandle hndl);
ACCB_API void runProgram(AccHandle hndl, AccProgram p, InputArray *in, OutputArray *out);
ACCB_API void freeOutput(OutputArray *out);
ACCB_API void freeProgram(AccProgram p);
/* status of the last runProgram on this handle (the reference has none) */
ACCB_API int accelerateStatus(AccHandle hndl);
ACCB_API accb_context *accelerateContext(AccHandle hndl);

/* Program construction.  Values are numbered: 0..ninputs-1 are the program
 * inputs, each added node returns the id of its result (scan' returns the
 * body id; the total is id+1).  Shapes of results follow Execute.hs:264-450. */
typedef struct accb_program accb_program;
typedef struct accb_value_type {
    int rank;
    int ncomp;
    int comp_bytes[ACCB_ARRAY_MAX_COMP];
} accb_value_type;
ACCB_API int accb_program_create(accb_context *ctx, int ninputs, const accb_value_type *input_types,
                                 accb_program **prog);
ACCB_API int accb_program_map(accb_program *p, accb_kernel *k, const int *env_ids, int nenv, int shape_like,
                              const accb_value_type *out_type, const void *scalars, size_t scalar_bytes);
ACCB_API int accb_program_fold(accb_program *p, accb_kernel *k, const int *env_ids, int nenv, int shape_like,
                               int all, const void *seed, size_t seed_bytes, const accb_value_type *out_type);
ACCB_API int accb_program_scan(accb_program *p, accb_kernel *k, const int *env_ids, int nenv, int shape_like,
                               int direction, int kind, const void *seed, size_t seed_bytes,
                               const accb_value_type *out_type);
ACCB_API int accb_program_permute(accb_program *p, accb_kernel *k, const int *env_ids, int nenv, int shape_like,
                                  int defaults_id, const accb_value_type *out_type);
ACCB_API int accb_program_stencil(accb_program *p, accb_kernel *k, int src_id, int boundary,
                                  const void *constant, size_t constant_bytes, int iters,
                                  const accb_value_type *out_type);
/* map over transposed matrices (accb_map_transposed): the result has the transposed shape of value src_id */
ACCB_API int accb_program_map_transposed(accb_program *p, accb_kernel *k, const int *env_ids, int nenv, int src_id,
                                         const accb_value_type *out_type, const void *scalars, size_t scalar_bytes);
/* generate: a map node whose result shape is given literally, innermost extent first
 * (`generate (constant sh) f`, CUDA/Execute.hs:194-195) */
ACCB_API int accb_program_generate(accb_program *p, accb_kernel *k, const int *env_ids, int nenv, int rank,
                                   const int *shape, const accb_value_type *out_type, const void *scalars,
                                   size_t scalar_bytes);
/* generate whose shape is computed from other values when the program runs: extent d (innermost first) is
 * add[d], plus extent src_dim[d] of value src_value[d] where src_value[d] >= 0.  What the reference gets by
 * evaluating the shape expression of a Generate / Backpermute on the host (executeOpenAcc, CUDA/Execute.hs:194-199). */
ACCB_API int accb_program_generate_dims(accb_program *p, accb_kernel *k, const int *env_ids, int nenv, int rank,
                                        const int *src_value, const int *src_dim, const int *add,
                                        const accb_value_type *out_type, const void *scalars, size_t scalar_bytes);
/* the same with up to two sources per extent: add[d] + extent src_dim[d] of src_value[d] + extent src_dim2[d] of
 * src_value2[d] (each where the value id is >= 0): the shape of `xs ++ ys` and of segmented scans whose segments
 * grow by one element. */
ACCB_API int accb_program_generate_dims2(accb_program *p, accb_kernel *k, const int *env_ids, int nenv, int rank,
                                         const int *src_value, const int *src_dim, const int *src_value2,
                                         const int *src_dim2, const int *add, const accb_value_type *out_type,
                                         const void *scalars, size_t scalar_bytes);
/* foldSeg / fold1Seg: offsets_id names an Int32 vector of segments + 1 offsets, the exclusive scan of the
 * segment lengths (foldSegOp, CUDA/Execute.hs:320-324); the innermost extent of the result is the segment count */
ACCB_API int accb_program_fold_seg(accb_program *p, accb_kernel *k, const int *env_ids, int nenv, int shape_like,
                                   int offsets_id, const void *seed, size_t seed_bytes,
                                   const accb_value_type *out_type);
/* stencil2: the result covers the intersection of the two sources (stencil2Op, CUDA/Execute.hs:427-450) */
ACCB_API int accb_program_stencil2(accb_program *p, accb_kernel *k, int src1_id, int src2_id, int boundary,
                                   const void *constant, size_t constant_bytes, const accb_value_type *out_type);
ACCB_API int accb_program_outputs(accb_program *p, const int *ids, int nout);
/* run with DEVICE arrays (what runProgram does) */
ACCB_API int accb_program_run(accb_program *p, accb_stream stream, const accb_array *inputs,
                              accb_array *outputs);
/* The same as ONE CUDA graph launch: the first call for a set of input arrays (pointers and shapes) on a
 * stream runs the program once, records a second run by stream capture and instantiates the graph; later
 * calls with the same arrays replay it on whatever the arrays then contain.  `stream` must not be the default
 * stream.  No counterpart in the reference, whose executeOpenAcc launches node by node
 * (CUDA/Execute.hs:164-219). */
ACCB_API int accb_program_run_graph(accb_program *p, accb_stream stream, const accb_array *inputs,
                                    accb_array *outputs);
/* awhile: while `cond` holds of the state, replace the state by `body` of it.  `cond` takes the state arrays as
 * its inputs and has ONE output, a Scalar of one 1-byte component (Bool); `body` takes the same inputs and has one
 * output per input, of the same type and -- when it runs -- the same shape.  `state` are body's-input-many device
 * arrays that hold the initial state and receive the final one (each iteration's results are copied back into
 * them on the stream).
 *   ACCB_AWHILE_HOST    the reference's scheme (Awhile of executeOpenAcc, CUDA/Execute.hs:236-244): the flag is
 *                       copied to the host and the stream synchronised once per iteration.
 *   ACCB_AWHILE_DEVICE  the whole loop is ONE CUDA graph launch: a conditional WHILE node whose body holds the
 *                       launches of `body`, the copies and `cond`; the flag never leaves the device and the call
 *                       returns without waiting.  Recorded at the first call for these arrays on this stream
 *                       (not the default stream) and replayed afterwards.
 * max_iters > 0 bounds the loop on the device as well.  When it stops the loop, ACCB_ETIMEOUT is returned by the
 * call itself in host mode; in device mode by the call itself when `iterations` is not NULL (the call then waits
 * for the stream), otherwise by the next accb_context_sync.  `iterations`, if not NULL, receives the number of
 * times the body ran. */
enum { ACCB_AWHILE_HOST = 0, ACCB_AWHILE_DEVICE = 1 };
ACCB_API int accb_awhile(accb_program *cond, accb_program *body, accb_stream stream, const accb_array *state,
                         int mode, long long max_iters, long long *iterations);
/* run1 with HOST arrays: upload, execute, download (CUDA.hs:307-330,382-389).
 * host_in[i] / host_out[j] point to one host buffer per component.  A program made of maps, folds, left scans
 * and permutes over inputs of one outermost extent is run in pieces (see accb_map_at), so that both directions
 * of the host link and the GPU work at the same time; accb_program_stream_chunk sets the piece size in elements
 * (-1: the default of 2^23, 0: never run in pieces).  A chain of stencils over one grid or cube (Clamp, Mirror or
 * Constant boundaries) is run in row slabs (slabs of planes) instead, each uploaded with as many rows above and
 * below as the chain reaches; the results are bit-identical to the whole-grid run.  Use pinned host memory for the copies to overlap. */
ACCB_API int accb_program_stream_chunk(accb_program *p, long long elements);
ACCB_API int accb_program_run_host(accb_program *p, const accb_array *host_in, accb_array *host_out);
ACCB_API int accb_program_destroy(accb_program *p);

/* ------------------------------------------ several GPUs from one process
 * A group is an ordered list of devices ("ranks"), each with its own context
 * and stream.  Arrays are sharded by contiguous slabs of the outermost index
 * space, rank 0 holding the first slab.  Every accb_group_* launch enqueues
 * work on all ranks' streams and returns; ordering between devices is done
 * with events; exchanged data is copied into the receiving device's OWN memory
 * (peer copy) before a kernel reads it, and no kernel waits for another device.
 * The reference drives one device per context; its only multi-device primitive
 * is the peer copy of CUDA/Array/Prim.hs:306-335, which nothing calls.
 * Per-rank arguments are rank-major: env[r * nenv + j], out[r], n[r].  A device
 * may appear more than once in the list (its ranks then share that GPU).  The
 * caller orders its own work against the group's streams (accb_group_stream,
 * accb_group_sync).                                                         */
typedef struct accb_group accb_group;
ACCB_API int accb_group_create(const int *devices, int n, accb_group **grp);
ACCB_API int accb_group_destroy(accb_group *grp);
ACCB_API int accb_group_size(accb_group *grp, int *n);
ACCB_API int accb_group_context(accb_group *grp, int rank, accb_context **ctx); /* borrowed */
ACCB_API int accb_group_stream(accb_group *grp, int rank, accb_stream *stream); /* borrowed */
ACCB_API int accb_group_sync(accb_group *grp); /* waits for every rank; reports bounded-wait failures */
ACCB_API const char *accb_group_last_error(accb_group *grp);
/* map / generate / transform over slabs: no exchange */
ACCB_API int accb_group_map(accb_group *grp, accb_kernel *k, const accb_array *env, int nenv, const void *scalars,
                            size_t scalar_bytes, const accb_array *out);
/* fold over the innermost dimension, rows[r] rows on rank r: no exchange */
ACCB_API int accb_group_fold_dim(accb_group *grp, accb_kernel *k, const accb_array *env, int nenv,
                                 const long long *rows, long long cols, const void *seed, size_t seed_bytes,
                                 const accb_array *out);
/* foldAll / fold1All (seed NULL): each rank reduces its n[r] >= 1 elements with `k`; the partials are copied to
 * rank 0 and reduced IN RANK ORDER, with the seed, by `k_combine` -- a fold_all kernel with the same combiner whose
 * functor reads one plain array of elements; every out[r] (a Scalar on rank r) receives the result. */
ACCB_API int accb_group_fold_all(accb_group *grp, accb_kernel *k, accb_kernel *k_combine, const accb_array *env,
                                 int nenv, const long long *n, const void *seed, size_t seed_bytes,
                                 const int *comp_bytes, const accb_array *out);
/* All six scans over the concatenation of the slabs (n[r] >= 1 elements on rank r; one-component elements of
 * elt_bytes).  `k` scans a slab; `k_total` is the fold_all kernel of the same producer and combiner (the slab
 * totals: one extra read of the slab); `k_carry` a scan kernel with the same combiner over a plain array, run on
 * rank 0 over the totals.  Each rank then continues from the carry of the slabs before it (after it, for right
 * scans), read from its own memory.  out[r] has n[r] elements; for ACCB_SCAN_EXCLUSIVE the LAST rank's has
 * n[r] + 1 (scanl: the total; scanr: the seed).  total[r] (needed for ACCB_SCAN_PRIME, else may be NULL) receives
 * the running total at the end of rank r's slab: the grand total is on the last rank (left) or rank 0 (right). */
ACCB_API int accb_group_scan(accb_group *grp, accb_kernel *k, accb_kernel *k_total, accb_kernel *k_carry,
                             const accb_array *env, int nenv, const long long *n, int direction, int kind,
                             const void *seed, size_t seed_bytes, size_t elt_bytes, const accb_array *out,
                             const accb_array *total);
/* permute with an associative and commutative combiner: every out[r] is a full-size destination; out[0] must hold
 * the defaults and out[r > 0] the combiner's neutral element.  Each rank scatters its n_src[r] source elements;
 * the partial destinations are copied to rank 0 one after another and merged into out[0] by `k_merge`, a map
 * kernel computing combine(a, b) of two plain arrays.  With `broadcast` every out[r] then receives the result. */
ACCB_API int accb_group_permute(accb_group *grp, accb_kernel *k, accb_kernel *k_merge, const accb_array *env,
                                int nenv, const long long *n_src, const void *scalars, size_t scalar_bytes,
                                const int *comp_bytes, const accb_array *out, int broadcast);
/* `iters` applications of a stencil on row slabs with ONE exchange: a[r] and b[r] are slabs of
 * pad_top + rows[r] + pad_bottom rows (accb_group_stencil_layout: iters * ry rows towards each neighbouring
 * rank, none at the global top and bottom unless the boundary is ACCB_WRAP), the rank's rows[r] >= iters * ry
 * own rows in the middle of a[r].  The halos are filled from the neighbours' rows by peer copies, then all
 * applications run on the padded slab: what the kernel's boundary treatment does at a padded edge creeps inwards
 * by ry rows per application, exactly as far as the halo reaches.  *result_in_b tells which buffer holds the
 * result (own rows only; the halos hold garbage).  `ry` is the stencil's reach along the outermost dimension.
 * Vectors, matrices and cubes: the slabs are cut along the outermost dimension, so a "row" of a cube is a plane. */
ACCB_API int accb_group_stencil_layout(accb_group *grp, int rank, int iters, int ry, int boundary, int *pad_top,
                                       int *pad_bottom);
ACCB_API int accb_group_stencil_iterate(accb_group *grp, accb_kernel *k, const accb_array *a, const accb_array *b,
                                        const int *rows, int iters, int ry, int boundary, const void *constant,
                                        size_t constant_bytes, const int *comp_bytes, int *result_in_b);
/* stencil2 on the same row slabs: a[r], b[r] and out[r] are slabs of pad_top + rows[r] + pad_bottom rows
 * (accb_group_stencil_layout with iters = 1); the halo rows of BOTH sources are filled from the neighbours, then every
 * rank applies the stencil to its padded slabs.  The result's own rows are final; its halo rows are not (they
 * belong to the neighbours).  Sources of different extents, whose result covers the intersection
 * (CUDA/Execute.hs:433-435), are cut to the intersection by the caller before they are dealt out. */
ACCB_API int accb_group_stencil2(accb_group *grp, accb_kernel *k, const accb_array *a, const accb_array *b,
                                 const accb_array *out, const int *rows, int ry, int boundary, const void *constant,
                                 size_t constant_bytes, const int *comp_bytes);
/* foldSeg over a vector, split BETWEEN segments: rank r owns nseg[r] consecutive segments and the n[r] elements they
 * cover (env[r]: its slice of the sources; out[r]: nseg[r] results).  offsets[r] is a device pointer on rank r to
 * the nseg[r] + 1 offsets of its segments as they stand in the WHOLE offsets array (CUDA/Execute.hs:320-324); the
 * call rebases them to the slice and folds.  No exchange.  accb_seg_partition picks the cuts from a host copy of
 * the offsets: first_seg[0..parts] with runs of whole segments that hold about the same number of elements. */
ACCB_API int accb_seg_partition(const int *offsets_host, long long nseg, int parts, long long *first_seg);
ACCB_API int accb_group_fold_seg(accb_group *grp, accb_kernel *k, const accb_array *env, int nenv, const long long *n,
                                 const int *const *offsets, const long long *nseg, const void *seed,
                                 size_t seed_bytes, const accb_array *out);

/* ------------------------- exchanges between processes, one per GPU
 * For hosts that run one process per GPU (torchrun, MPI): the small exchanges of the sharded skeletons -- slab
 * totals of a scan, partials of a foldAll, partial destinations of a permute, halo rows of a stencil -- done by
 * the library's own kernels over NVLink instead of a collective library.  Every rank creates an exchange buffer
 * of the same size, passes its 64-byte handle to the others by whatever channel the host has (the Python mirror
 * uses torch.distributed), and connects; the buffers are plain CUDA IPC peer mappings (no multicast objects).
 * Ranks write what they want to exchange into their OWN buffer (accb_peer_data: a device pointer any skeleton
 * launch can write to) and then call, all of them and in the same order:
 *   accb_peer_gather     one kernel: synchronise the ranks, then dst[r * bytes ..] = rank r's data[offset ..]
 *   accb_peer_allreduce  one kernel: synchronise, then dst[i] = data_0[i] (op) data_1[i] (op) .., in rank order,
 *                        so that every rank gets the same bits
 *   accb_peer_barrier    synchronise only;  accb_peer_pull copies from ONE rank's buffer without synchronising
 * The synchronisation is a flag per rank in every buffer (release stores to the peers, acquire polling of the own
 * buffer); a wait gives up after five seconds (ACCB_PEER_TIMEOUT_MS, read when the buffer is created, changes that)
 * and accb_peer_status then reports ACCB_ETIMEOUT.  A rank may
 * overwrite data it exchanged only after the NEXT synchronising call has returned on its stream, since slower
 * ranks may still be reading: callers alternate between two offsets.  No counterpart in the reference. */
typedef struct accb_peer accb_peer;
#define ACCB_PEER_HANDLE_BYTES 64
enum { ACCB_PEER_I32 = 0, ACCB_PEER_U32 = 1, ACCB_PEER_I64 = 2, ACCB_PEER_F32 = 3, ACCB_PEER_F64 = 4 };
enum { ACCB_PEER_ADD = 0, ACCB_PEER_MIN = 1, ACCB_PEER_MAX = 2, ACCB_PEER_AND = 3, ACCB_PEER_OR = 4, ACCB_PEER_XOR = 5 };
ACCB_API int accb_peer_create(accb_context *ctx, int rank, int world, size_t bytes, accb_peer **peer);
ACCB_API int accb_peer_handle(accb_peer *peer, unsigned char *handle /* ACCB_PEER_HANDLE_BYTES */);
ACCB_API int accb_peer_connect(accb_peer *peer, const unsigned char *handles /* world x ACCB_PEER_HANDLE_BYTES */);
/* instead of accb_peer_connect, for tests of the time limit: the other ranks never arrive */
ACCB_API int accb_peer_loopback(accb_peer *peer);
ACCB_API int accb_peer_data(accb_peer *peer, void **data, size_t *bytes);
ACCB_API int accb_peer_barrier(accb_peer *peer, accb_stream stream);
ACCB_API int accb_peer_gather(accb_peer *peer, accb_stream stream, size_t offset, size_t bytes, void *dst);
ACCB_API int accb_peer_allreduce(accb_peer *peer, accb_stream stream, size_t offset, long long count, int type,
                                 int op, void *dst);
/* one kernel: synchronise, then dst[i] = first[i] (op) data_0[i] (op) .. (op) data_{rank-1}[i] -- the carry a
 * sharded scan continues from on this rank (`first`: the seed of the whole scan, a device pointer on this rank) */
ACCB_API int accb_peer_exscan(accb_peer *peer, accb_stream stream, size_t offset, long long count, int type, int op,
                              const void *first, void *dst);
ACCB_API int accb_peer_pull(accb_peer *peer, accb_stream stream, int from_rank, size_t offset, size_t bytes,
                            void *dst);
/* scanl / scanl1 / scanl' over ONE vector of n_global elements that is dealt to the ranks in blocks: global block j
 * (block_elems elements, a multiple of the kernel's tile, see accb_peer_scan_tile; 0 picks 32 tiles) lives on rank j mod world, and every
 * rank stores its blocks one after the other (accb_peer_scan_layout tells how many elements that is; only the last
 * global block may be short).  `env` and `out` are the rank's own arrays in that layout.  One launch per rank of the
 * same single-pass kernel as accb_scan: every element is read and written once, the ranks run at the same time, and
 * what crosses NVLink is one 16-byte store per block and rank (the block's aggregate, later its prefix), stored
 * into every rank's exchange buffer with plain peer stores -- `scratch_offset` names scratch_bytes of the data area
 * (16-byte aligned, the same on every rank) that this call owns.  A scan over contiguous slabs must know a slab's
 * total before it starts and therefore reads every element twice; the reference's scan reads twice on ONE GPU
 * (CUDA/CodeGen/PrefixSum.hs:59-120).
 *   ACCB_SCAN_EXCLUSIVE  out has n_local elements; the rank that owns the last block (total_owner) has one more:
 *                        the total, right after its last element.  With n_global == 0 rank 0 writes the seed.
 *   ACCB_SCAN_INCLUSIVE  scanl1, no seed.      ACCB_SCAN_PRIME  `total` is written on total_owner only.
 * Values of up to 8 bytes (one component).  Every rank must call, in the same order, also one that holds no element.
 * Waits on other ranks give up after the buffer's time limit; accb_context_sync then returns ACCB_ETIMEOUT. */
/* elements of one tile of kernel k's block-cyclic entries (blocks are whole multiples of it) */
ACCB_API int accb_peer_scan_tile(accb_context *ctx, accb_kernel *k, long long *tile_elems);
ACCB_API int accb_peer_scan_layout(int world, int rank, long long n_global, long long block_elems, long long *n_local,
                                   int *total_owner, size_t *scratch_bytes);
ACCB_API int accb_peer_scan(accb_peer *peer, accb_kernel *k, accb_stream stream, const accb_array *env, int nenv,
                            long long n_global, long long block_elems, int kind, const void *seed, size_t seed_bytes,
                            size_t scratch_offset, const accb_array *out, const accb_array *total);
/* The same scan launched piece by piece: this call covers the rank's blocks first_local_block .. first_local_block +
 * local_blocks - 1 (local_blocks < 0: all the rest); `env`, `out` and every other argument are those of the whole
 * scan in every call.  Piece 0 begins the scan, later pieces must follow in order on the same stream, with no other
 * scan on that stream in between; every rank cuts its blocks at the same places.  A later piece finds the
 * records of the earlier ones, so a rank can scan what has arrived while the rest of its input is still on its way
 * from the host, and send results back while later pieces run. */
ACCB_API int accb_peer_scan_piece(accb_peer *peer, accb_kernel *k, accb_stream stream, const accb_array *env, int nenv,
                                  long long n_global, long long block_elems, int kind, const void *seed,
                                  size_t seed_bytes, size_t scratch_offset, const accb_array *out,
                                  const accb_array *total, long long first_local_block, long long local_blocks);
ACCB_API int accb_peer_status(accb_peer *peer, accb_stream stream, int *timed_out);
ACCB_API int accb_peer_destroy(accb_peer *peer); /* after every rank has finished using the buffers */

/* -------------------------------------------- synthetic benchmark inputs
 * Index-addressable generators (any shard can produce its own slice).      */
ACCB_API int accb_gen_uniform_f32(accb_context *ctx, accb_stream stream, float *dst, long long n,
                                  long long first_index, uint64_t seed, uint64_t stream_id, float lo, float hi);
ACCB_API int accb_gen_uniform_i32(accb_context *ctx, accb_stream stream, int32_t *dst, long long n,
                                  long long first_index, uint64_t seed, uint64_t stream_id, int32_t m);
/* 50 % Zipf (inverse CDF table of `nbins` doubles on the device) / 50 % uniform */
ACCB_API int accb_gen_zipf_mix_i32(accb_context *ctx, accb_stream stream, int32_t *dst, long long n,
                                   long long first_index, uint64_t seed, const double *cdf, int nbins);
/* writes `bytes` of a private buffer larger than L2 to evict cached lines */
ACCB_API int accb_flush_l2(accb_context *ctx, accb_stream stream);

#ifdef __cplusplus
}
#endif
#endif /* ACCB200_H */
