/*
 * program.cc -- whole programs: the AccFFI.h surface (accelerateCreate,
 * runProgram, freeOutput, freeProgram, accelerateDestroy) and the op list
 * that stands in for a compiled Accelerate function.
 *
 * Replaces Data/Array/Accelerate/CUDA/Foreign/Export.hs:100-283 and the
 * execute phase executeAfun1 / executeOpenAcc of
 * Data/Array/Accelerate/CUDA/Execute.hs:143-219 for straight-line programs
 * (a let-bound chain of collective operations).  In the reference an
 * AccProgram is a StablePtr to a Haskell closure `run1With ctx f`
 * (Export.hs:255-265); here it is a list of nodes, each naming a compiled
 * kernel, the values it reads and how the shape of its result follows from
 * them (Execute.hs:264-450).
 *
 * Intermediate arrays are kept in a per-program pool and reused from run to
 * run when large enough, instead of one cuMemAlloc per intermediate per run
 * (Array/Sugar.hs:40-44 via Execute.hs:264-268).
 */
#include <algorithm>
#include <cstdlib>

#include "common.h"

using namespace accb_rt;

namespace {

enum NodeKind { N_MAP, N_FOLD, N_SCAN, N_PERMUTE, N_STENCIL, N_FOLDSEG, N_STENCIL2 };

struct Node {
    NodeKind kind;
    accb_kernel *k = nullptr;
    std::vector<int> env;
    int shape_like = 0;   /* value whose shape the result takes; -1: the shape described below (generate) */
    int lit_rank = 0;
    int lit_shape[ACCB_MAX_RANK] = {0};           /* extent d = lit_shape[d] ... */
    int dim_src[ACCB_MAX_RANK] = {-1, -1, -1, -1}; /* ... + extent dim_of[d] of value dim_src[d], if >= 0 */
    int dim_of[ACCB_MAX_RANK] = {0};
    int dim_src2[ACCB_MAX_RANK] = {-1, -1, -1, -1}; /* ... + a second such extent, if >= 0 (appended arrays) */
    int dim_of2[ACCB_MAX_RANK] = {0};
    int offsets_id = -1;  /* foldSeg: Int32 vector of segment offsets, length segments + 1 */
    bool transposed = false; /* map: the element-wise inputs are read transposed; the result has shape_like's shape transposed */
    int all = 0;          /* fold: reduce everything */
    int direction = 0, scan_kind = 0;
    int defaults_id = -1; /* permute */
    int boundary = 0, iters = 1;
    bool has_seed = false;
    std::vector<unsigned char> scalars; /* map scalars / fold+scan seed / stencil constant */
    int out_id = -1;      /* first value id produced */
    accb_value_type out_type;
};

struct PoolBuf {
    void *ptr = nullptr;
    size_t bytes = 0;
};

}  // namespace

struct accb_program {
    accb_context *ctx = nullptr;
    int ninputs = 0;
    std::vector<accb_value_type> types; /* per value id */
    std::vector<Node> nodes;
    std::vector<int> outputs;
    std::vector<std::vector<PoolBuf>> pool; /* per value id, per component (stencil uses 2x) */
    std::vector<std::vector<PoolBuf>> in_pool;
    PoolBuf slab_pool[4];               /* work grids of a stencil chain run slab by slab: two sets of two */
    cudaStream_t host_stream = nullptr;
    cudaStream_t pipe_stream[3] = {nullptr, nullptr, nullptr}; /* upload, compute, download */
    std::vector<cudaEvent_t> pipe_events;
    int status = ACCB_OK;
    long long stream_chunk = -1; /* elements per piece of a streamed host run: -1 the default, 0 never stream */
    /* the op list recorded as a CUDA graph for one set of input arrays on one stream */
    cudaGraphExec_t graph_exec = nullptr;
    cudaStream_t graph_stream = nullptr;
    unsigned long long graph_generation = 0; /* the context's buffer_generation when it was recorded */
    std::vector<accb_array> graph_inputs, graph_outputs;
    /* awhile with this program as the body, recorded as a graph with a conditional WHILE node */
    cudaGraphExec_t loop_exec = nullptr;
    cudaStream_t loop_stream = nullptr;
    accb_program *loop_cond = nullptr;
    unsigned long long loop_generation = 0;
    long long loop_max_iters = 0;
    std::vector<accb_array> loop_state;
    unsigned long long *loop_words = nullptr; /* device: [0] times the body ran, [1] stopped by the limit */
};

namespace {

long long size_of(const accb_array &a) {
    long long n = 1;
    for (int d = 0; d < a.rank; ++d) n *= a.shape[d];
    return n;
}

int pool_get(accb_program *p, PoolBuf &b, size_t bytes, void **out) {
    bytes = std::max<size_t>(bytes, 16);
    if (b.bytes < bytes) {
        p->ctx->buffer_generation++; /* a recorded graph of this program names the old buffer */
        if (b.ptr) {
            cudaDeviceSynchronize(); /* earlier runs may still read it */
            cudaFree(b.ptr);
            b.ptr = nullptr;
            b.bytes = 0;
        }
        void *q = p->ctx->mem.alloc_raw(bytes);
        if (!q) return fail(p->ctx, ACCB_ENOMEM, "device out of memory allocating %zu bytes for an intermediate", bytes);
        b.ptr = q;
        b.bytes = MemTable::round_up(bytes);
    }
    *out = b.ptr;
    return ACCB_OK;
}

/* allocate the components of value `id` with shape already set in `a` */
int alloc_value(accb_program *p, int id, accb_array &a, bool fresh, int pool_slot = 0) {
    const accb_value_type &t = p->types[id];
    a.ncomp = t.ncomp;
    const long long n = std::max(1LL, size_of(a)); /* at least one element (Prim.hs:167,186) */
    for (int c = 0; c < t.ncomp; ++c) {
        const size_t bytes = (size_t)n * t.comp_bytes[c];
        if (fresh) {
            a.ptr[c] = p->ctx->mem.alloc_raw(bytes);
            if (!a.ptr[c]) return fail(p->ctx, ACCB_ENOMEM, "device out of memory allocating %zu bytes for a result", bytes);
        } else {
            auto &slots = p->pool[id];
            const size_t idx = (size_t)pool_slot * ACCB_ARRAY_MAX_COMP + c;
            if (slots.size() <= idx) slots.resize(idx + 1);
            int st = pool_get(p, slots[idx], bytes, &a.ptr[c]);
            if (st != ACCB_OK) return st;
        }
    }
    return ACCB_OK;
}

#define TRY(expr)                       \
    do {                                \
        int st_ = (expr);               \
        if (st_ != ACCB_OK) return st_; \
    } while (0)

int run_internal(accb_program *p, cudaStream_t s, const accb_array *inputs, accb_array *outputs, bool fresh_outputs) {
    accb_context *ctx = p->ctx;
    std::vector<accb_array> val(p->types.size());
    for (int i = 0; i < p->ninputs; ++i) val[i] = inputs[i];
    auto is_output = [&](int id) { return std::find(p->outputs.begin(), p->outputs.end(), id) != p->outputs.end(); };

    for (Node &nd : p->nodes) {
        std::vector<accb_array> env;
        for (int e : nd.env) env.push_back(val[e]);
        accb_array literal;
        memset(&literal, 0, sizeof literal);
        literal.rank = nd.lit_rank;
        for (int d = 0; d < nd.lit_rank && nd.shape_like < 0; ++d) {
            long long e = nd.lit_shape[d];
            if (nd.dim_src[d] >= 0) {
                const accb_array &src = val[nd.dim_src[d]];
                if (nd.dim_of[d] >= src.rank) return fail(ctx, ACCB_EINVAL, "shape refers to a dimension its source lacks");
                e += src.shape[nd.dim_of[d]];
            }
            if (nd.dim_src2[d] >= 0) {
                const accb_array &src = val[nd.dim_src2[d]];
                if (nd.dim_of2[d] >= src.rank) return fail(ctx, ACCB_EINVAL, "shape refers to a dimension its source lacks");
                e += src.shape[nd.dim_of2[d]];
            }
            if (e < 0 || e > 0x7fffffffLL) return fail(ctx, ACCB_EBOUNDS, "computed extent %lld is out of range", e);
            literal.shape[d] = (int)e;
        }
        const accb_array &like = nd.shape_like >= 0 ? val[nd.shape_like] : literal;
        accb_array out;
        memset(&out, 0, sizeof out);
        const bool fresh = fresh_outputs && is_output(nd.out_id);
        const void *sc = nd.scalars.empty() ? nullptr : nd.scalars.data();
        switch (nd.kind) {
            case N_MAP: {
                out.rank = like.rank;
                memcpy(out.shape, like.shape, sizeof out.shape);
                if (nd.transposed) {
                    if (like.rank != 2) return fail(ctx, ACCB_EINVAL, "transpose of an array of rank %d", like.rank);
                    std::swap(out.shape[0], out.shape[1]);
                }
                TRY(alloc_value(p, nd.out_id, out, fresh));
                if (nd.transposed)
                    TRY(accb_map_transposed(ctx, nd.k, s, env.data(), (int)env.size(), sc, nd.scalars.size(), &out));
                else
                    TRY(accb_map(ctx, nd.k, s, env.data(), (int)env.size(), sc, nd.scalars.size(), &out));
                break;
            }
            case N_FOLD: {
                const void *seed = nd.has_seed ? sc : nullptr;
                if (nd.all || like.rank <= 1) {
                    out.rank = 0;
                    TRY(alloc_value(p, nd.out_id, out, fresh));
                    TRY(accb_fold_all(ctx, nd.k, s, env.data(), (int)env.size(), size_of(like), seed, nd.scalars.size(), &out));
                } else {
                    /* result drops the innermost extent; zero outer extents become 1 (Execute.hs:287-289) */
                    out.rank = like.rank - 1;
                    long long rows = 1;
                    for (int d = 1; d < like.rank; ++d) {
                        out.shape[d - 1] = nd.has_seed ? std::max(1, like.shape[d]) : like.shape[d];
                        rows *= out.shape[d - 1];
                    }
                    TRY(alloc_value(p, nd.out_id, out, fresh));
                    TRY(accb_fold_dim(ctx, nd.k, s, env.data(), (int)env.size(), rows, like.shape[0], seed,
                                      nd.scalars.size(), &out));
                }
                break;
            }
            case N_SCAN: {
                /* The reference scans vectors only (PrefixSum.hs:39-46).  An INCLUSIVE scan is also taken over
                 * the row-major sequence of an array of higher rank: the result keeps the shape, and a
                 * combiner that restarts at row or segment heads makes it a scan along the innermost
                 * dimension or a segmented scan. */
                if (like.rank != 1 && !(like.rank > 1 && nd.scan_kind == ACCB_SCAN_INCLUSIVE))
                    return fail(ctx, ACCB_EINVAL, "exclusive scans are defined on vectors only");
                const long long n = size_of(like);
                if (n > 0x7fffffffLL - 1) return fail(ctx, ACCB_EINVAL, "array too large for one scan");
                out.rank = like.rank;
                memcpy(out.shape, like.shape, sizeof out.shape);
                if (like.rank == 1) out.shape[0] = (int)(nd.scan_kind == ACCB_SCAN_EXCLUSIVE ? n + 1 : n);
                TRY(alloc_value(p, nd.out_id, out, fresh));
                accb_array total;
                memset(&total, 0, sizeof total);
                if (nd.scan_kind == ACCB_SCAN_PRIME)
                    TRY(alloc_value(p, nd.out_id + 1, total, fresh_outputs && is_output(nd.out_id + 1)));
                TRY(accb_scan(ctx, nd.k, s, env.data(), (int)env.size(), n, nd.direction, nd.scan_kind,
                              nd.has_seed ? sc : nullptr, nd.scalars.size(), &out,
                              nd.scan_kind == ACCB_SCAN_PRIME ? &total : nullptr));
                if (nd.scan_kind == ACCB_SCAN_PRIME) val[nd.out_id + 1] = total;
                break;
            }
            case N_PERMUTE: {
                const accb_array &dfl = val[nd.defaults_id];
                out.rank = dfl.rank;
                memcpy(out.shape, dfl.shape, sizeof out.shape);
                TRY(alloc_value(p, nd.out_id, out, fresh));
                TRY(accb_permute_defaults(ctx, s, &dfl, &out, p->types[nd.out_id].comp_bytes));
                TRY(accb_permute(ctx, nd.k, s, env.data(), (int)env.size(), size_of(like), nullptr, 0, &out));
                break;
            }
            case N_FOLDSEG: {
                /* the innermost extent becomes the number of segments (Execute.hs:320-324) */
                const accb_array &offs = val[nd.offsets_id];
                if (offs.rank != 1 || offs.shape[0] < 1 || like.rank < 1)
                    return fail(ctx, ACCB_EINVAL, "foldSeg needs a vector of segments + 1 offsets and a source of rank >= 1");
                const long long nseg = offs.shape[0] - 1;
                out.rank = like.rank;
                out.shape[0] = (int)nseg;
                long long rows = 1;
                for (int d = 1; d < like.rank; ++d) {
                    out.shape[d] = like.shape[d];
                    rows *= like.shape[d];
                }
                TRY(alloc_value(p, nd.out_id, out, fresh));
                TRY(accb_fold_seg(ctx, nd.k, s, env.data(), (int)env.size(), rows, like.shape[0],
                                  static_cast<const int *>(offs.ptr[0]), nseg, nd.has_seed ? sc : nullptr,
                                  nd.scalars.size(), &out));
                break;
            }
            case N_STENCIL2: {
                /* the result covers the intersection of the two sources (Execute.hs:433-435) */
                const accb_array &a = val[nd.env[0]], &b = val[nd.env[1]];
                if (a.rank != b.rank) return fail(ctx, ACCB_EINVAL, "stencil2 sources differ in rank");
                out.rank = a.rank;
                for (int d = 0; d < a.rank; ++d) out.shape[d] = std::min(a.shape[d], b.shape[d]);
                TRY(alloc_value(p, nd.out_id, out, fresh));
                TRY(accb_stencil2(ctx, nd.k, s, &a, &b, nd.boundary, sc, nd.scalars.size(), &out));
                break;
            }
            case N_STENCIL: {
                out.rank = like.rank;
                memcpy(out.shape, like.shape, sizeof out.shape);
                if (nd.iters <= 1) {
                    TRY(alloc_value(p, nd.out_id, out, fresh));
                    TRY(accb_stencil(ctx, nd.k, s, &like, nd.boundary, sc, nd.scalars.size(), &out));
                } else {
                    /* ping-pong between the value's two pooled grids; whichever holds the final grid is the value */
                    accb_array tmp = out;
                    TRY(alloc_value(p, nd.out_id, out, fresh, 0));
                    TRY(alloc_value(p, nd.out_id, tmp, false, 1));
                    int in_b = 0;
                    TRY(accb_stencil_iterate_from(ctx, nd.k, s, &like, &out, &tmp, nd.iters, nd.boundary, sc, nd.scalars.size(), &in_b));
                    if (in_b) out = tmp;
                }
                break;
            }
        }
        val[nd.out_id] = out;
    }
    for (size_t j = 0; j < p->outputs.size(); ++j) outputs[j] = val[p->outputs[j]];
    return ACCB_OK;
}

int add_node(accb_program *p, Node &nd, const accb_value_type *out_type, int nvalues) {
    if (!out_type || out_type->ncomp < 1 || out_type->ncomp > ACCB_ARRAY_MAX_COMP)
        return -fail(p->ctx, ACCB_EINVAL, "bad result type");
    for (int e : nd.env)
        if (e < 0 || e >= (int)p->types.size()) return -fail(p->ctx, ACCB_EINVAL, "unknown value id %d", e);
    if (nd.shape_like >= (int)p->types.size() || (nd.shape_like < 0 && !(nd.kind == N_MAP && nd.shape_like == -1)))
        return -fail(p->ctx, ACCB_EINVAL, "unknown value id");
    nd.out_id = (int)p->types.size();
    nd.out_type = *out_type;
    p->types.push_back(*out_type);
    if (nvalues == 2) { /* scan': the total is a scalar of the same element type */
        accb_value_type t = *out_type;
        t.rank = 0;
        p->types.push_back(t);
    }
    p->pool.resize(p->types.size());
    p->nodes.push_back(nd);
    return nd.out_id;
}

struct Handle {
    accb_context *ctx = nullptr;
    int status = ACCB_OK;
};

struct OutputOwner {
    accb_context *ctx;
    std::vector<void *> ptrs;
};

}  // namespace

#define PLOCK(p)                                                      \
    if (!(p)) return fail(nullptr, ACCB_EINVAL, "null program");      \
    std::lock_guard<std::recursive_mutex> lock_((p)->ctx->mu);        \
    CtxGuard guard_((p)->ctx)

extern "C" {

int accb_program_create(accb_context *ctx, int ninputs, const accb_value_type *input_types, accb_program **prog) {
    if (!ctx || !prog || ninputs < 0 || (ninputs > 0 && !input_types)) return fail(ctx, ACCB_EINVAL, "bad argument");
    accb_program *p = new accb_program;
    p->ctx = ctx;
    p->ninputs = ninputs;
    p->types.assign(input_types, input_types + ninputs);
    p->pool.resize(ninputs);
    p->in_pool.resize(ninputs);
    *prog = p;
    return ACCB_OK;
}

/* the add functions return the new value id (>= 0) or minus a status code */
int accb_program_map(accb_program *p, accb_kernel *k, const int *env_ids, int nenv, int shape_like,
                     const accb_value_type *out_type, const void *scalars, size_t scalar_bytes) {
    if (!p || !k) return -ACCB_EINVAL;
    Node nd;
    nd.kind = N_MAP;
    nd.k = k;
    nd.env.assign(env_ids, env_ids + nenv);
    nd.shape_like = shape_like;
    if (scalars) nd.scalars.assign((const unsigned char *)scalars, (const unsigned char *)scalars + scalar_bytes);
    return add_node(p, nd, out_type, 1);
}

int accb_program_fold(accb_program *p, accb_kernel *k, const int *env_ids, int nenv, int shape_like, int all,
                      const void *seed, size_t seed_bytes, const accb_value_type *out_type) {
    if (!p || !k) return -ACCB_EINVAL;
    Node nd;
    nd.kind = N_FOLD;
    nd.k = k;
    nd.env.assign(env_ids, env_ids + nenv);
    nd.shape_like = shape_like;
    nd.all = all;
    nd.has_seed = seed != nullptr;
    if (seed) nd.scalars.assign((const unsigned char *)seed, (const unsigned char *)seed + seed_bytes);
    return add_node(p, nd, out_type, 1);
}

int accb_program_scan(accb_program *p, accb_kernel *k, const int *env_ids, int nenv, int shape_like, int direction,
                      int kind, const void *seed, size_t seed_bytes, const accb_value_type *out_type) {
    if (!p || !k) return -ACCB_EINVAL;
    Node nd;
    nd.kind = N_SCAN;
    nd.k = k;
    nd.env.assign(env_ids, env_ids + nenv);
    nd.shape_like = shape_like;
    nd.direction = direction;
    nd.scan_kind = kind;
    nd.has_seed = seed != nullptr;
    if (seed) nd.scalars.assign((const unsigned char *)seed, (const unsigned char *)seed + seed_bytes);
    return add_node(p, nd, out_type, kind == ACCB_SCAN_PRIME ? 2 : 1);
}

int accb_program_permute(accb_program *p, accb_kernel *k, const int *env_ids, int nenv, int shape_like,
                         int defaults_id, const accb_value_type *out_type) {
    if (!p || !k) return -ACCB_EINVAL;
    if (defaults_id < 0 || defaults_id >= (int)p->types.size()) return -fail(p->ctx, ACCB_EINVAL, "unknown defaults id");
    Node nd;
    nd.kind = N_PERMUTE;
    nd.k = k;
    nd.env.assign(env_ids, env_ids + nenv);
    nd.shape_like = shape_like;
    nd.defaults_id = defaults_id;
    return add_node(p, nd, out_type, 1);
}

int accb_program_stencil(accb_program *p, accb_kernel *k, int src_id, int boundary, const void *constant,
                         size_t constant_bytes, int iters, const accb_value_type *out_type) {
    if (!p || !k) return -ACCB_EINVAL;
    Node nd;
    nd.kind = N_STENCIL;
    nd.k = k;
    nd.env.push_back(src_id);
    nd.shape_like = src_id;
    nd.boundary = boundary;
    nd.iters = std::max(1, iters);
    if (constant) nd.scalars.assign((const unsigned char *)constant, (const unsigned char *)constant + constant_bytes);
    return add_node(p, nd, out_type, 1);
}

int accb_program_map_transposed(accb_program *p, accb_kernel *k, const int *env_ids, int nenv, int src_id,
                                const accb_value_type *out_type, const void *scalars, size_t scalar_bytes) {
    if (!p || !k) return -ACCB_EINVAL;
    if (src_id < 0) return -fail(p->ctx, ACCB_EINVAL, "unknown value id");
    Node nd;
    nd.kind = N_MAP;
    nd.k = k;
    nd.env.assign(env_ids, env_ids + nenv);
    nd.shape_like = src_id;
    nd.transposed = true;
    if (scalars) nd.scalars.assign((const unsigned char *)scalars, (const unsigned char *)scalars + scalar_bytes);
    return add_node(p, nd, out_type, 1);
}

/* generate: a map whose result shape is given literally (innermost extent first) */
int accb_program_generate(accb_program *p, accb_kernel *k, const int *env_ids, int nenv, int rank, const int *shape,
                          const accb_value_type *out_type, const void *scalars, size_t scalar_bytes) {
    if (!p || !k) return -ACCB_EINVAL;
    if (rank < 0 || rank > ACCB_ARRAY_MAX_RANK || (rank > 0 && !shape)) return -fail(p->ctx, ACCB_EINVAL, "bad shape");
    Node nd;
    nd.kind = N_MAP;
    nd.k = k;
    if (nenv > 0) nd.env.assign(env_ids, env_ids + nenv);
    nd.shape_like = -1;
    nd.lit_rank = rank;
    for (int d = 0; d < rank; ++d) {
        if (shape[d] < 0) return -fail(p->ctx, ACCB_EINVAL, "negative extent");
        nd.lit_shape[d] = shape[d];
    }
    if (scalars) nd.scalars.assign((const unsigned char *)scalars, (const unsigned char *)scalars + scalar_bytes);
    return add_node(p, nd, out_type, 1);
}

/* generate whose extents are taken from other values: extent d (innermost first) of the result is
 * add[d], plus extent src_dim[d] of value src_value[d] when src_value[d] >= 0 */
int accb_program_generate_dims2(accb_program *p, accb_kernel *k, const int *env_ids, int nenv, int rank,
                                const int *src_value, const int *src_dim, const int *src_value2, const int *src_dim2,
                                const int *add, const accb_value_type *out_type, const void *scalars,
                                size_t scalar_bytes) {
    if (!p || !k) return -ACCB_EINVAL;
    if (rank < 0 || rank > ACCB_ARRAY_MAX_RANK || (rank > 0 && (!src_value || !src_dim || !add)) ||
        ((src_value2 == nullptr) != (src_dim2 == nullptr)))
        return -fail(p->ctx, ACCB_EINVAL, "bad shape description");
    Node nd;
    nd.kind = N_MAP;
    nd.k = k;
    if (nenv > 0) nd.env.assign(env_ids, env_ids + nenv);
    nd.shape_like = -1;
    nd.lit_rank = rank;
    auto known = [&](int v, int d) { return v < (int)p->types.size() && (v < 0 || (d >= 0 && d < ACCB_ARRAY_MAX_RANK)); };
    for (int d = 0; d < rank; ++d) {
        if (!known(src_value[d], src_dim[d]) || (src_value2 && !known(src_value2[d], src_dim2[d])))
            return -fail(p->ctx, ACCB_EINVAL, "shape refers to an unknown value or dimension");
        nd.dim_src[d] = src_value[d] < 0 ? -1 : src_value[d];
        nd.dim_of[d] = src_dim[d];
        if (src_value2) {
            nd.dim_src2[d] = src_value2[d] < 0 ? -1 : src_value2[d];
            nd.dim_of2[d] = src_dim2[d];
        }
        nd.lit_shape[d] = add[d];
    }
    if (scalars) nd.scalars.assign((const unsigned char *)scalars, (const unsigned char *)scalars + scalar_bytes);
    return add_node(p, nd, out_type, 1);
}

int accb_program_generate_dims(accb_program *p, accb_kernel *k, const int *env_ids, int nenv, int rank,
                               const int *src_value, const int *src_dim, const int *add,
                               const accb_value_type *out_type, const void *scalars, size_t scalar_bytes) {
    return accb_program_generate_dims2(p, k, env_ids, nenv, rank, src_value, src_dim, nullptr, nullptr, add, out_type,
                                       scalars, scalar_bytes);
}

int accb_program_fold_seg(accb_program *p, accb_kernel *k, const int *env_ids, int nenv, int shape_like, int offsets_id,
                          const void *seed, size_t seed_bytes, const accb_value_type *out_type) {
    if (!p || !k) return -ACCB_EINVAL;
    if (offsets_id < 0 || offsets_id >= (int)p->types.size()) return -fail(p->ctx, ACCB_EINVAL, "unknown offsets id");
    if (p->types[offsets_id].ncomp != 1 || p->types[offsets_id].comp_bytes[0] != 4)
        return -fail(p->ctx, ACCB_EINVAL, "segment offsets are Int32");
    Node nd;
    nd.kind = N_FOLDSEG;
    nd.k = k;
    nd.env.assign(env_ids, env_ids + nenv);
    nd.shape_like = shape_like;
    nd.offsets_id = offsets_id;
    nd.has_seed = seed != nullptr;
    if (seed) nd.scalars.assign((const unsigned char *)seed, (const unsigned char *)seed + seed_bytes);
    return add_node(p, nd, out_type, 1);
}

int accb_program_stencil2(accb_program *p, accb_kernel *k, int src1_id, int src2_id, int boundary, const void *constant,
                          size_t constant_bytes, const accb_value_type *out_type) {
    if (!p || !k) return -ACCB_EINVAL;
    Node nd;
    nd.kind = N_STENCIL2;
    nd.k = k;
    nd.env.push_back(src1_id);
    nd.env.push_back(src2_id);
    nd.shape_like = src1_id;
    nd.boundary = boundary;
    if (constant) nd.scalars.assign((const unsigned char *)constant, (const unsigned char *)constant + constant_bytes);
    return add_node(p, nd, out_type, 1);
}

int accb_program_outputs(accb_program *p, const int *ids, int nout) {
    if (!p || !ids || nout < 1) return fail(p ? p->ctx : nullptr, ACCB_EINVAL, "bad argument");
    for (int i = 0; i < nout; ++i)
        if (ids[i] < 0 || ids[i] >= (int)p->types.size()) return fail(p->ctx, ACCB_EINVAL, "unknown value id %d", ids[i]);
    p->outputs.assign(ids, ids + nout);
    return ACCB_OK;
}

int accb_program_run(accb_program *p, accb_stream stream, const accb_array *inputs, accb_array *outputs) {
    PLOCK(p);
    if ((p->ninputs && !inputs) || !outputs || p->outputs.empty()) return fail(p->ctx, ACCB_EINVAL, "bad argument");
    return run_internal(p, (cudaStream_t)stream, inputs, outputs, false);
}

/* ------------------------------------------------------------------------------------------------------
 * Streamed host runs.  The reference uploads every input, runs, and downloads every result, one after the
 * other (useArrayAsync / collect, CUDA.hs:307-330,382-389), so the host link idles while the kernels run and
 * one direction idles while the other is used.  A program whose nodes work on their input piece by piece is
 * run in pieces instead: while piece k is computed, piece k+1 is on its way up and the results of piece k-1 on
 * their way down.  What makes a node fit:
 *   map / zipWith   element-wise inputs are cut into the same pieces as the result (accb_map_at);
 *   fold over rows  a piece is a run of rows (accb_fold_dim_at);
 *   foldAll         every piece continues from what the pieces before it came to (accb_fold_all_at);
 *   scanl, scanl1, scanl'   every piece continues from the previous piece's last value (seed on the device);
 *   permute         every piece combines into the one result (accb_permute_at).
 * Values are classed as STREAM (cut into pieces along the outermost dimension), WHOLE (an input that is not
 * read element-wise -- a table that is gathered from, the defaults of a permute: uploaded once, ahead of the
 * first piece) or ACC (built up over all pieces: a fold's scalar, a permute's result, a scan' total; downloaded
 * at the end).  Stencils, transposed maps, right scans, segmented folds and nodes that read an ACC value do not
 * fit; such programs run the reference's way. */
enum StreamClass { SC_UNKNOWN = 0, SC_STREAM, SC_WHOLE, SC_ACC };

struct StreamValue {
    int cls = SC_UNKNOWN;
    long long per_unit = 1; /* elements per unit of the outermost dimension */
    int tail = 0;           /* elements beyond units * per_unit (the total of an exclusive scan) */
    accb_array whole;       /* the device array (all pieces) */
};

/* number of leading components the kernel reads element-wise (In::size of its functor) */
static int elementwise_components(accb_context *ctx, accb_kernel *k, const char *entry, int *n) {
    CUfunction fn;
    KernelMeta meta;
    int st = get_function(ctx, k, entry, &fn, &meta);
    if (st == ACCB_OK) *n = meta.v[11];
    return st;
}

static long long outer_extent(const accb_array &a) { return a.rank >= 1 ? a.shape[a.rank - 1] : 1; }
static long long inner_elems(const accb_array &a) {
    long long n = 1;
    for (int d = 0; d + 1 < a.rank; ++d) n *= a.shape[d];
    return n;
}

/* A chain of stencils over ONE host grid or cube (a blur applied ten times, say) does not stream element by
 * element, but it does by ROW SLABS (slabs of planes for a cube): a slab of the result depends on the slab of the
 * source plus as many rows above and below as the whole chain reaches (the sum over its stencils of applications
 * x reach along the outermost dimension).  Every slab is
 * uploaded with that margin, the chain is applied to the widened slab as if it were a whole grid -- rows next to a
 * cut are wrong by one more row per application, which is what the margin is for, while at the grid's real top and
 * bottom the slab's edge IS the grid's edge and the boundary condition applies as always -- and the slab's own rows
 * are downloaded while the next slab is worked on.  Clamp, Mirror and Constant only (Wrap reaches across the grid).
 * The results are those of the whole-grid run, bit for bit: the same kernels see the same neighbourhoods.
 * Returns 1 if it handled the run (status in *status), 0 if the program does not fit. */
static int run_host_slabbed(accb_program *p, const accb_array *host_in, accb_array *host_out, int *status) {
    *status = ACCB_OK;
    accb_context *ctx = p->ctx;
    if (ctx->tune.no_pipeline || p->stream_chunk == 0 || p->ninputs != 1 || p->outputs.size() != 1 || p->nodes.empty()) return 0;
    const int rank = host_in[0].rank;
    if ((rank != 2 && rank != 3) || p->types[0].ncomp != 1) return 0;
    long long reach = 0;
    size_t widest = p->types[0].comp_bytes[0];
    int prev = 0;
    for (Node &nd : p->nodes) {
        if (nd.kind != N_STENCIL || nd.shape_like != prev || nd.boundary == ACCB_WRAP || nd.iters < 1) return 0;
        if (nd.out_type.ncomp != 1 || nd.out_type.rank != rank) return 0;
        CUfunction fn;
        KernelMeta meta;
        /* how far the stencil reaches along the outermost dimension: rows for a matrix, planes for a cube */
        if (rank == 2) {
            if (nd.k->skeleton != SK_STENCIL || get_function(ctx, nd.k, "stencil", &fn, &meta) != ACCB_OK) return 0;
            reach += (long long)nd.iters * meta.v[7];
        } else {
            if (nd.k->skeleton != SK_STENCIL3 || get_function(ctx, nd.k, "stencil3", &fn, &meta) != ACCB_OK) return 0;
            reach += (long long)nd.iters * (meta.v[5] / 2);
        }
        widest = std::max<size_t>(widest, nd.out_type.comp_bytes[0]);
        prev = nd.out_id;
    }
    if (p->outputs[0] != prev) return 0;
    /* a "row" is everything below the outermost dimension: a row of a matrix, a plane of a cube */
    const long long W = rank == 2 ? host_in[0].shape[0] : (long long)host_in[0].shape[0] * host_in[0].shape[1];
    const long long H = host_in[0].shape[rank - 1];
    if (W < 1 || reach < 1) return 0;
    /* slabs of about 32 MiB, at least eight times the margin, a multiple of 16 rows */
    long long rows = p->stream_chunk > 0 ? p->stream_chunk / W : (32LL << 20) / (W * (long long)widest);
    rows = std::max(rows, 8 * reach);
    if (rank == 2) rows = std::max(rows, 16LL) / 16 * 16;
    if (H < 2 * rows) return 0;
    const long long nslabs = (H + rows - 1) / rows;
    const size_t in_bytes = p->types[0].comp_bytes[0], out_bytes = p->types[prev].comp_bytes[0];
    if (!host_out[0].ptr[0]) {
        *status = fail(ctx, ACCB_EINVAL, "null host buffer for the result");
        return 1;
    }

    auto run = [&]() -> int {
        for (int i = 0; i < 3; ++i)
            if (!p->pipe_stream[i])
                TRY(check_cuda(ctx, cudaStreamCreateWithFlags(&p->pipe_stream[i], cudaStreamNonBlocking), "cudaStreamCreate"));
        cudaStream_t up = p->pipe_stream[0], comp = p->pipe_stream[1], down = p->pipe_stream[2];
        while ((long long)p->pipe_events.size() < 3 * nslabs) {
            cudaEvent_t e;
            TRY(check_cuda(ctx, cudaEventCreateWithFlags(&e, cudaEventDisableTiming), "cudaEventCreate"));
            p->pipe_events.push_back(e);
        }
        auto &slots = p->in_pool[0];
        if (slots.empty()) slots.resize(1);
        void *dev_in = nullptr;
        TRY(pool_get(p, slots[0], (size_t)(H * W) * in_bytes, &dev_in));
        void *work[4];
        for (int i = 0; i < 4; ++i) TRY(pool_get(p, p->slab_pool[i], (size_t)((rows + 2 * reach) * W) * widest, &work[i]));
        long long uploaded = 0; /* rows of the source on the device so far */
        for (long long sl = 0; sl < nslabs; ++sl) {
            const long long r0 = sl * rows, r1 = std::min(H, r0 + rows);
            const long long e0 = std::max(0LL, r0 - reach), e1 = std::min(H, r1 + reach);
            cudaEvent_t ev_up = p->pipe_events[3 * sl], ev_comp = p->pipe_events[3 * sl + 1], ev_down = p->pipe_events[3 * sl + 2];
            if (uploaded < e1) {
                TRY(check_cuda(ctx, cudaMemcpyAsync(static_cast<char *>(dev_in) + uploaded * W * in_bytes,
                                                    static_cast<const char *>(host_in[0].ptr[0]) + uploaded * W * in_bytes,
                                                    (size_t)((e1 - uploaded) * W) * in_bytes, cudaMemcpyHostToDevice, up), "upload"));
                uploaded = e1;
            }
            TRY(check_cuda(ctx, cudaEventRecord(ev_up, up), "cudaEventRecord"));
            TRY(check_cuda(ctx, cudaStreamWaitEvent(comp, ev_up, 0), "cudaStreamWaitEvent"));
            /* this slab's pair of work grids was last read by the download of the slab before the previous one */
            if (sl >= 2) TRY(check_cuda(ctx, cudaStreamWaitEvent(comp, p->pipe_events[3 * (sl - 2) + 2], 0), "cudaStreamWaitEvent"));
            accb_array cur = host_in[0];
            cur.shape[rank - 1] = (int)(e1 - e0);
            cur.ptr[0] = static_cast<char *>(dev_in) + e0 * W * in_bytes;
            int next_work = 0;
            for (Node &nd : p->nodes) {
                const void *sc = nd.scalars.empty() ? nullptr : nd.scalars.data();
                accb_array a = cur, b = cur;
                a.ptr[0] = work[2 * (sl & 1) + next_work];
                b.ptr[0] = work[2 * (sl & 1) + (next_work ^ 1)];
                int in_b = 0;
                TRY(accb_stencil_iterate_from(ctx, nd.k, (accb_stream)comp, &cur, &a, &b, nd.iters, nd.boundary, sc, nd.scalars.size(), &in_b));
                cur = in_b ? b : a;
                next_work = in_b ? next_work : next_work ^ 1; /* the next stencil writes to the grid `cur` is not in */
            }
            TRY(check_cuda(ctx, cudaEventRecord(ev_comp, comp), "cudaEventRecord"));
            TRY(check_cuda(ctx, cudaStreamWaitEvent(down, ev_comp, 0), "cudaStreamWaitEvent"));
            TRY(check_cuda(ctx, cudaMemcpyAsync(static_cast<char *>(host_out[0].ptr[0]) + r0 * W * out_bytes,
                                                static_cast<const char *>(cur.ptr[0]) + (r0 - e0) * W * out_bytes,
                                                (size_t)((r1 - r0) * W) * out_bytes, cudaMemcpyDeviceToHost, down), "download"));
            TRY(check_cuda(ctx, cudaEventRecord(ev_down, down), "cudaEventRecord"));
        }
        TRY(check_cuda(ctx, cudaStreamSynchronize(down), "cudaStreamSynchronize"));
        host_out[0].rank = rank;
        for (int d = 0; d < rank; ++d) host_out[0].shape[d] = host_in[0].shape[d];
        host_out[0].ncomp = 1;
        return ACCB_OK;
    };
    *status = run();
    return 1;
}

/* Returns 1 if it handled the run (status in *status), 0 if the program does not fit. */
static int run_host_streamed(accb_program *p, const accb_array *host_in, accb_array *host_out, int *status) {
    *status = ACCB_OK;
    accb_context *ctx = p->ctx;
    if (ctx->tune.no_pipeline || p->stream_chunk == 0 || p->ninputs < 1) return 0;
    const size_t nvalues = p->types.size();
    std::vector<StreamValue> val(nvalues);
    std::vector<int> first_ew(p->nodes.size(), 0); /* element-wise components per node */

    /* ---- does every node fit, and which inputs are cut into pieces? ---- */
    auto want = [&](int id, int cls) { /* an input takes the class its first reader needs; others must agree */
        if (val[id].cls == SC_UNKNOWN && id < p->ninputs) val[id].cls = cls;
        return val[id].cls == cls;
    };
    for (size_t ni = 0; ni < p->nodes.size(); ++ni) {
        Node &nd = p->nodes[ni];
        const char *entry = nullptr;
        switch (nd.kind) {
            case N_MAP: entry = nd.transposed ? nullptr : "map"; break;
            case N_FOLD: entry = nullptr; break; /* decided below: foldAll or fold over rows */
            case N_SCAN: entry = nd.direction == ACCB_SCAN_LEFT ? "scanl" : nullptr; break;
            case N_PERMUTE: entry = "permute"; break;
            default: return 0;
        }
        if (!entry && nd.kind != N_FOLD) return 0;
        if (nd.shape_like < 0) return 0;
        if (nd.kind == N_FOLD) entry = (nd.all || p->types[nd.shape_like].rank <= 1) ? "foldAll" : "fold";
        int ew = 0;
        if (elementwise_components(ctx, nd.k, entry, &ew) != ACCB_OK) return 0;
        first_ew[ni] = ew;
        int slot = 0;
        for (int e : nd.env) { /* the arrays that hold the first `ew` components are read element-wise */
            const bool elementwise = slot < ew;
            slot += p->types[e].ncomp;
            if (!want(e, elementwise ? SC_STREAM : SC_WHOLE)) return 0;
        }
        if (!want(nd.shape_like, SC_STREAM)) return 0;
        const accb_value_type &to = p->types[nd.out_id];
        switch (nd.kind) {
            case N_MAP: val[nd.out_id].cls = SC_STREAM; break;
            case N_FOLD:
                if (!strcmp(entry, "foldAll")) {
                    if (to.ncomp != 1) return 0; /* the carry between pieces is one value */
                    val[nd.out_id].cls = SC_ACC;
                } else {
                    val[nd.out_id].cls = SC_STREAM;
                }
                break;
            case N_SCAN:
                if (to.ncomp != 1 || p->types[nd.shape_like].rank != 1) return 0;
                if (nd.scan_kind != ACCB_SCAN_EXCLUSIVE && nd.scan_kind != ACCB_SCAN_INCLUSIVE && nd.scan_kind != ACCB_SCAN_PRIME) return 0;
                val[nd.out_id].cls = SC_STREAM;
                val[nd.out_id].tail = nd.scan_kind == ACCB_SCAN_EXCLUSIVE ? 1 : 0;
                if (nd.scan_kind == ACCB_SCAN_PRIME) val[nd.out_id + 1].cls = SC_ACC;
                break;
            case N_PERMUTE:
                if (!want(nd.defaults_id, SC_WHOLE)) return 0;
                val[nd.out_id].cls = SC_ACC;
                break;
            default: return 0;
        }
    }
    for (int id : p->outputs)
        if (val[id].cls != SC_STREAM && val[id].cls != SC_ACC) return 0;

    /* ---- the pieces: all streamed inputs share the outermost extent ---- */
    long long units = -1, widest = 1;
    for (int i = 0; i < p->ninputs; ++i) {
        if (val[i].cls == SC_UNKNOWN) val[i].cls = SC_WHOLE; /* an input nobody reads */
        if (val[i].cls != SC_STREAM) continue;
        if (host_in[i].rank < 1) return 0;
        if (units < 0) units = outer_extent(host_in[i]);
        if (outer_extent(host_in[i]) != units) return 0;
        val[i].per_unit = inner_elems(host_in[i]);
        widest = std::max(widest, val[i].per_unit);
    }
    if (units < 0) return 0;
    long long chunk_elems = 1LL << 23; /* long enough for the copy engines, short ramps at both ends */
    if (ctx->tune.pipeline_chunk_log2 > 0) chunk_elems = 1LL << std::min(28, std::max(10, ctx->tune.pipeline_chunk_log2));
    if (p->stream_chunk > 0) chunk_elems = p->stream_chunk;
    /* pieces start on multiples of 16 units, so that every component of every piece stays 16-byte aligned */
    const long long per_piece = std::max(16LL, chunk_elems / widest / 16 * 16);
    if (units < 2 * per_piece) return 0;
    const long long npieces = (units + per_piece - 1) / per_piece;

    auto run = [&]() -> int {
        for (int i = 0; i < 3; ++i)
            if (!p->pipe_stream[i])
                TRY(check_cuda(ctx, cudaStreamCreateWithFlags(&p->pipe_stream[i], cudaStreamNonBlocking), "cudaStreamCreate"));
        cudaStream_t up = p->pipe_stream[0], comp = p->pipe_stream[1], down = p->pipe_stream[2];
        while ((long long)p->pipe_events.size() < 2 * npieces + 1) {
            cudaEvent_t e;
            TRY(check_cuda(ctx, cudaEventCreateWithFlags(&e, cudaEventDisableTiming), "cudaEventCreate"));
            p->pipe_events.push_back(e);
        }
        /* device arrays of the inputs (whole size); WHOLE inputs go up first */
        for (int i = 0; i < p->ninputs; ++i) {
            accb_array &d = val[i].whole;
            d = host_in[i];
            const accb_value_type &t = p->types[i];
            auto &slots = p->in_pool[i];
            if ((int)slots.size() < t.ncomp) slots.resize(t.ncomp);
            const long long n = size_of(host_in[i]);
            for (int c = 0; c < t.ncomp; ++c) {
                TRY(pool_get(p, slots[c], (size_t)std::max(1LL, n) * t.comp_bytes[c], &d.ptr[c]));
                if (val[i].cls == SC_WHOLE && n > 0)
                    TRY(check_cuda(ctx, cudaMemcpyAsync(d.ptr[c], host_in[i].ptr[c], (size_t)n * t.comp_bytes[c],
                                                        cudaMemcpyHostToDevice, up), "upload"));
            }
        }
        TRY(check_cuda(ctx, cudaEventRecord(p->pipe_events[2 * npieces], up), "cudaEventRecord"));
        TRY(check_cuda(ctx, cudaStreamWaitEvent(comp, p->pipe_events[2 * npieces], 0), "cudaStreamWaitEvent"));

        /* a piece [u0, u0 + len) of a streamed value */
        auto piece = [&](int id, long long u0, long long len, int extra) {
            const StreamValue &v = val[id];
            accb_array a = v.whole;
            a.shape[a.rank - 1] = (int)(len + (a.rank == 1 ? extra : 0));
            for (int c = 0; c < a.ncomp; ++c)
                a.ptr[c] = static_cast<char *>(v.whole.ptr[c]) + u0 * v.per_unit * p->types[id].comp_bytes[c];
            return a;
        };

        for (long long k = 0; k < npieces; ++k) {
            const long long u0 = k * per_piece, len = std::min(per_piece, units - u0);
            const bool first = k == 0, last = k == npieces - 1;
            for (int i = 0; i < p->ninputs; ++i) {
                if (val[i].cls != SC_STREAM) continue;
                const accb_value_type &t = p->types[i];
                for (int c = 0; c < t.ncomp; ++c) {
                    const size_t off = (size_t)(u0 * val[i].per_unit) * t.comp_bytes[c];
                    TRY(check_cuda(ctx, cudaMemcpyAsync(static_cast<char *>(val[i].whole.ptr[c]) + off,
                                                        static_cast<const char *>(host_in[i].ptr[c]) + off,
                                                        (size_t)(len * val[i].per_unit) * t.comp_bytes[c], cudaMemcpyHostToDevice, up),
                                   "upload"));
                }
            }
            TRY(check_cuda(ctx, cudaEventRecord(p->pipe_events[2 * k], up), "cudaEventRecord"));
            TRY(check_cuda(ctx, cudaStreamWaitEvent(comp, p->pipe_events[2 * k], 0), "cudaStreamWaitEvent"));

            for (size_t ni = 0; ni < p->nodes.size(); ++ni) {
                Node &nd = p->nodes[ni];
                const StreamValue &like = val[nd.shape_like];
                const void *sc = nd.scalars.empty() ? nullptr : nd.scalars.data();
                std::vector<accb_array> env;
                for (int e : nd.env) env.push_back(val[e].cls == SC_STREAM ? piece(e, u0, len, 0) : val[e].whole);
                const long long base = u0 * like.per_unit; /* index of the piece's first element in the whole array */
                StreamValue &ov = val[nd.out_id];
                if (first) { /* size the result from the whole input */
                    accb_array &o = ov.whole;
                    memset(&o, 0, sizeof o);
                    const accb_array &lw = like.whole;
                    switch (nd.kind) {
                        case N_MAP:
                            o.rank = lw.rank;
                            memcpy(o.shape, lw.shape, sizeof o.shape);
                            ov.per_unit = like.per_unit;
                            break;
                        case N_FOLD:
                            if (ov.cls == SC_ACC) {
                                o.rank = 0;
                            } else { /* the innermost extent goes */
                                o.rank = lw.rank - 1;
                                for (int d = 1; d < lw.rank; ++d) o.shape[d - 1] = lw.shape[d];
                                ov.per_unit = lw.shape[0] ? like.per_unit / lw.shape[0] : 0;
                            }
                            break;
                        case N_SCAN:
                            o.rank = 1;
                            o.shape[0] = (int)(units + ov.tail);
                            ov.per_unit = 1;
                            break;
                        case N_PERMUTE: {
                            const accb_array &dfl = val[nd.defaults_id].whole;
                            o.rank = dfl.rank;
                            memcpy(o.shape, dfl.shape, sizeof o.shape);
                            break;
                        }
                        default: break;
                    }
                    if (nd.kind == N_SCAN && units + ov.tail > 0x7fffffffLL) return fail(ctx, ACCB_EINVAL, "array too large for one scan");
                    TRY(alloc_value(p, nd.out_id, o, false));
                    if (nd.kind == N_SCAN && nd.scan_kind == ACCB_SCAN_PRIME) {
                        accb_array &t = val[nd.out_id + 1].whole;
                        memset(&t, 0, sizeof t);
                        TRY(alloc_value(p, nd.out_id + 1, t, false));
                    }
                    if (nd.kind == N_PERMUTE)
                        TRY(accb_permute_defaults(ctx, comp, &val[nd.defaults_id].whole, &o, p->types[nd.out_id].comp_bytes));
                }
                switch (nd.kind) {
                    case N_MAP: {
                        accb_array o = piece(nd.out_id, u0, len, 0);
                        TRY(accb_map_at(ctx, nd.k, comp, env.data(), (int)env.size(), sc, nd.scalars.size(), &o, base));
                        break;
                    }
                    case N_FOLD: {
                        if (ov.cls == SC_ACC) {
                            const bool seed_now = nd.has_seed && last; /* f(.., seed) closes the fold: with the last piece */
                            TRY(accb_fold_all_at(ctx, nd.k, comp, env.data(), (int)env.size(), len * like.per_unit,
                                                 seed_now ? sc : nullptr, nd.scalars.size(), &ov.whole, base,
                                                 first ? nullptr : ov.whole.ptr[0]));
                        } else {
                            accb_array o = piece(nd.out_id, u0, len, 0);
                            const long long cols = like.whole.shape[0];
                            TRY(accb_fold_dim_at(ctx, nd.k, comp, env.data(), (int)env.size(), cols ? len * like.per_unit / cols : 0,
                                                 cols, nd.has_seed ? sc : nullptr, nd.scalars.size(), &o, base));
                        }
                        break;
                    }
                    case N_SCAN: {
                        const int eb = p->types[nd.out_id].comp_bytes[0];
                        accb_array o = piece(nd.out_id, u0, len, last ? ov.tail : ov.tail); /* every piece writes its running total behind itself */
                        char *optr = static_cast<char *>(o.ptr[0]);
                        if (nd.scan_kind == ACCB_SCAN_EXCLUSIVE) {
                            /* piece k continues from the total piece k-1 left in the element it also starts with */
                            TRY(accb_scan_at(ctx, nd.k, comp, env.data(), (int)env.size(), len, ACCB_SCAN_LEFT,
                                             first ? ACCB_SCAN_EXCLUSIVE : (ACCB_SCAN_EXCLUSIVE | ACCB_SEED_ON_DEVICE),
                                             first ? sc : static_cast<const void *>(optr), first ? nd.scalars.size() : (size_t)eb, &o,
                                             nullptr, base));
                        } else if (nd.scan_kind == ACCB_SCAN_INCLUSIVE) {
                            TRY(accb_scan_at(ctx, nd.k, comp, env.data(), (int)env.size(), len, ACCB_SCAN_LEFT,
                                             first ? ACCB_SCAN_INCLUSIVE : (ACCB_SCAN_INCLUSIVE_SEEDED | ACCB_SEED_ON_DEVICE),
                                             first ? nullptr : static_cast<const void *>(optr - eb), first ? 0 : (size_t)eb, &o, nullptr,
                                             base));
                        } else { /* scanl': the total so far is the next piece's seed */
                            accb_array &tot = val[nd.out_id + 1].whole;
                            TRY(accb_scan_at(ctx, nd.k, comp, env.data(), (int)env.size(), len, ACCB_SCAN_LEFT,
                                             first ? ACCB_SCAN_PRIME : (ACCB_SCAN_PRIME | ACCB_SEED_ON_DEVICE),
                                             first ? sc : static_cast<const void *>(tot.ptr[0]), first ? nd.scalars.size() : (size_t)eb, &o,
                                             &tot, base));
                        }
                        break;
                    }
                    case N_PERMUTE:
                        TRY(accb_permute_at(ctx, nd.k, comp, env.data(), (int)env.size(), len * like.per_unit, nullptr, 0,
                                            &ov.whole, base));
                        break;
                    default: break;
                }
            }
            TRY(check_cuda(ctx, cudaEventRecord(p->pipe_events[2 * k + 1], comp), "cudaEventRecord"));
            TRY(check_cuda(ctx, cudaStreamWaitEvent(down, p->pipe_events[2 * k + 1], 0), "cudaStreamWaitEvent"));
            /* the piece's share of every streamed result goes down while the next piece is computed */
            for (size_t j = 0; j < p->outputs.size(); ++j) {
                const int id = p->outputs[j];
                const StreamValue &v = val[id];
                if (v.cls != SC_STREAM) continue;
                const accb_value_type &t = p->types[id];
                const long long take = len * v.per_unit + (last ? v.tail : 0);
                for (int c = 0; c < t.ncomp; ++c) {
                    const size_t off = (size_t)(u0 * v.per_unit) * t.comp_bytes[c];
                    if (take > 0)
                        TRY(check_cuda(ctx, cudaMemcpyAsync(static_cast<char *>(host_out[j].ptr[c]) + off,
                                                            static_cast<const char *>(v.whole.ptr[c]) + off,
                                                            (size_t)take * t.comp_bytes[c], cudaMemcpyDeviceToHost, down), "download"));
                }
            }
        }
        /* results built up over all pieces */
        for (size_t j = 0; j < p->outputs.size(); ++j) {
            const int id = p->outputs[j];
            const StreamValue &v = val[id];
            const accb_value_type &t = p->types[id];
            void *host_ptr[ACCB_ARRAY_MAX_COMP];
            for (int c = 0; c < t.ncomp; ++c) host_ptr[c] = host_out[j].ptr[c];
            if (v.cls == SC_ACC) {
                const long long n = size_of(v.whole);
                for (int c = 0; c < t.ncomp; ++c)
                    if (n > 0)
                        TRY(check_cuda(ctx, cudaMemcpyAsync(host_ptr[c], v.whole.ptr[c], (size_t)n * t.comp_bytes[c],
                                                            cudaMemcpyDeviceToHost, down), "download"));
            }
            host_out[j] = v.whole; /* rank and shape of the result */
            for (int c = 0; c < t.ncomp; ++c) host_out[j].ptr[c] = host_ptr[c];
        }
        TRY(check_cuda(ctx, cudaStreamSynchronize(down), "cudaStreamSynchronize"));
        return ACCB_OK;
    };
    *status = run();
    return 1;
}

int accb_program_stream_chunk(accb_program *p, long long elements) {
    PLOCK(p);
    if (elements < -1) return fail(p->ctx, ACCB_EINVAL, "piece size %lld", elements);
    p->stream_chunk = elements;
    return ACCB_OK;
}

int accb_program_run_host(accb_program *p, const accb_array *host_in, accb_array *host_out) {
    PLOCK(p);
    if ((p->ninputs && !host_in) || !host_out || p->outputs.empty()) return fail(p->ctx, ACCB_EINVAL, "bad argument");
    accb_context *ctx = p->ctx;
    {
        int st = ACCB_OK;
        if (run_host_streamed(p, host_in, host_out, &st)) return st;
        if (run_host_slabbed(p, host_in, host_out, &st)) return st;
    }
    if (!p->host_stream) TRY(check_cuda(ctx, cudaStreamCreateWithFlags(&p->host_stream, cudaStreamNonBlocking), "cudaStreamCreate"));
    cudaStream_t s = p->host_stream;
    /* upload (useArrayAsync, Execute.hs:151-154) */
    std::vector<accb_array> dev_in(p->ninputs);
    for (int i = 0; i < p->ninputs; ++i) {
        dev_in[i] = host_in[i];
        const long long n = std::max(1LL, size_of(host_in[i]));
        auto &slots = p->in_pool[i];
        if ((int)slots.size() < p->types[i].ncomp) slots.resize(p->types[i].ncomp);
        for (int c = 0; c < p->types[i].ncomp; ++c) {
            const size_t bytes = (size_t)n * p->types[i].comp_bytes[c];
            TRY(pool_get(p, slots[c], bytes, &dev_in[i].ptr[c]));
            TRY(check_cuda(ctx, cudaMemcpyAsync(dev_in[i].ptr[c], host_in[i].ptr[c], (size_t)size_of(host_in[i]) * p->types[i].comp_bytes[c],
                                                cudaMemcpyHostToDevice, s), "upload"));
        }
    }
    std::vector<accb_array> dev_out(p->outputs.size());
    TRY(run_internal(p, s, dev_in.data(), dev_out.data(), false));
    /* collect: every result goes back to the host (CUDA.hs:382-389) */
    for (size_t j = 0; j < p->outputs.size(); ++j) {
        const accb_value_type &t = p->types[p->outputs[j]];
        void *host_ptr[ACCB_ARRAY_MAX_COMP];
        for (int c = 0; c < t.ncomp; ++c) host_ptr[c] = host_out[j].ptr[c];
        host_out[j].rank = dev_out[j].rank;
        memcpy(host_out[j].shape, dev_out[j].shape, sizeof dev_out[j].shape);
        host_out[j].ncomp = t.ncomp;
        for (int c = 0; c < t.ncomp; ++c) {
            if (!host_ptr[c]) return fail(ctx, ACCB_EINVAL, "null host buffer for result %zu", j);
            TRY(check_cuda(ctx, cudaMemcpyAsync(host_ptr[c], dev_out[j].ptr[c], (size_t)size_of(dev_out[j]) * t.comp_bytes[c],
                                                cudaMemcpyDeviceToHost, s), "download"));
        }
    }
    TRY(check_cuda(ctx, cudaStreamSynchronize(s), "cudaStreamSynchronize"));
    return ACCB_OK;
}

/* Run the op list as ONE CUDA graph launch.  The first call for a given set of input arrays (pointers and
 * shapes) on a given stream runs the program once the ordinary way -- which sizes every intermediate and
 * scratch buffer and loads every kernel --, records a second run with stream capture and instantiates the
 * graph; later calls with the same arrays replay it, whatever the arrays now contain.  The outputs are the
 * program's pooled result arrays, as for accb_program_run.  Replaces the per-node launch loop of
 * executeOpenAcc (CUDA/Execute.hs:164-219) for programs that are applied again and again to arrays in place. */
int accb_program_run_graph(accb_program *p, accb_stream stream, const accb_array *inputs, accb_array *outputs) {
    PLOCK(p);
    if ((p->ninputs && !inputs) || !outputs || p->outputs.empty()) return fail(p->ctx, ACCB_EINVAL, "bad argument");
    accb_context *ctx = p->ctx;
    cudaStream_t s = (cudaStream_t)stream;
    if (!s) return fail(ctx, ACCB_EINVAL, "graph runs need a stream of their own (the default stream cannot be captured)");
    /* a scratch or pooled buffer replaced since the recording (by any launch of this context) makes it stale */
    bool same = p->graph_exec && p->graph_stream == s && (int)p->graph_inputs.size() == p->ninputs &&
                p->graph_generation == ctx->buffer_generation;
    for (int i = 0; same && i < p->ninputs; ++i) {
        const accb_array &a = p->graph_inputs[i], &b = inputs[i];
        same = a.rank == b.rank && a.ncomp == b.ncomp;
        for (int d = 0; same && d < a.rank; ++d) same = a.shape[d] == b.shape[d];
        for (int c = 0; same && c < a.ncomp; ++c) same = a.ptr[c] == b.ptr[c];
    }
    if (!same) {
        if (p->graph_exec) {
            cudaGraphExecDestroy(p->graph_exec);
            p->graph_exec = nullptr;
        }
        std::vector<accb_array> outs(p->outputs.size());
        TRY(run_internal(p, s, inputs, outs.data(), false));
        TRY(check_cuda(ctx, cudaStreamSynchronize(s), "cudaStreamSynchronize"));
        TRY(check_cuda(ctx, cudaStreamBeginCapture(s, cudaStreamCaptureModeRelaxed), "cudaStreamBeginCapture"));
        const int st = run_internal(p, s, inputs, outs.data(), false);
        cudaGraph_t g = nullptr;
        const cudaError_t ce = cudaStreamEndCapture(s, &g);
        if (st != ACCB_OK) {
            if (g) cudaGraphDestroy(g);
            return st;
        }
        TRY(check_cuda(ctx, ce, "cudaStreamEndCapture"));
        const cudaError_t ci = cudaGraphInstantiate(&p->graph_exec, g, 0);
        cudaGraphDestroy(g);
        if (ci != cudaSuccess) p->graph_exec = nullptr;
        TRY(check_cuda(ctx, ci, "cudaGraphInstantiate"));
        p->graph_stream = s;
        p->graph_generation = ctx->buffer_generation;
        p->graph_inputs.assign(inputs, inputs + p->ninputs);
        p->graph_outputs = outs;
    }
    TRY(check_cuda(ctx, cudaGraphLaunch(p->graph_exec, s), "cudaGraphLaunch"));
    for (size_t j = 0; j < p->graph_outputs.size(); ++j) outputs[j] = p->graph_outputs[j];
    return ACCB_OK;
}

}  // extern "C"

/* ---------------------------------------------------------------- awhile */
namespace {

/* Decides whether the loop goes on.  Runs once ahead of the WHILE node (in_body = 0: resets the counters) and
 * once at the end of every pass through its body.  The limit keeps a loop whose condition never turns false
 * from occupying the GPU for ever. */
__global__ void awhile_step(cudaGraphConditionalHandle handle, const unsigned char *flag, unsigned long long *words,
                            unsigned long long max_iters, int in_body) {
    unsigned long long done = 0;
    if (in_body) {
        done = words[0] + 1;
        words[0] = done;
    } else {
        words[0] = 0;
        words[1] = 0;
    }
    unsigned go = *flag != 0;
    if (go && done >= max_iters) {
        go = 0;
        words[1] = 1;
    }
    cudaGraphSetConditional(handle, go);
}

bool same_shape(const accb_array &a, const accb_array &b) {
    if (a.rank != b.rank || a.ncomp != b.ncomp) return false;
    for (int d = 0; d < a.rank; ++d)
        if (a.shape[d] != b.shape[d]) return false;
    return true;
}

/* state <- the body's results, on the stream */
int copy_back(accb_program *body, cudaStream_t s, const accb_array *state, const std::vector<accb_array> &outs) {
    accb_context *ctx = body->ctx;
    for (int i = 0; i < body->ninputs; ++i) {
        if (!same_shape(state[i], outs[i]))
            return fail(ctx, ACCB_EINVAL, "awhile: result %d of the body differs in shape from the state it replaces", i);
        const accb_value_type &t = body->types[body->outputs[i]];
        const long long n = size_of(state[i]);
        for (int c = 0; c < t.ncomp; ++c) {
            if (outs[i].ptr[c] == state[i].ptr[c] || n == 0) continue; /* passed through unchanged */
            TRY(check_cuda(ctx, cudaMemcpyAsync(state[i].ptr[c], outs[i].ptr[c], (size_t)n * t.comp_bytes[c],
                                                cudaMemcpyDeviceToDevice, s), "cudaMemcpyAsync"));
        }
    }
    return ACCB_OK;
}

int awhile_check(accb_program *cond, accb_program *body, const accb_array *state, long long max_iters) {
    accb_context *ctx = body->ctx;
    if (cond->ctx != ctx) return fail(ctx, ACCB_EINVAL, "awhile: condition and body belong to different contexts");
    if (!state || body->ninputs < 1 || cond->ninputs != body->ninputs || (int)body->outputs.size() != body->ninputs)
        return fail(ctx, ACCB_EINVAL, "awhile: the condition takes, and the body takes and returns, the state arrays");
    if (cond->outputs.size() != 1) return fail(ctx, ACCB_EINVAL, "awhile: the condition has one result");
    const accb_value_type &ft = cond->types[cond->outputs[0]];
    if (ft.ncomp != 1 || ft.comp_bytes[0] != 1) return fail(ctx, ACCB_EINVAL, "awhile: the condition yields a Scalar Bool");
    for (int i = 0; i < body->ninputs; ++i) {
        const accb_value_type &a = body->types[i], &b = body->types[body->outputs[i]], &c = cond->types[i];
        bool ok = a.ncomp == b.ncomp && a.ncomp == c.ncomp && a.rank == b.rank;
        for (int k = 0; ok && k < a.ncomp; ++k) ok = a.comp_bytes[k] == b.comp_bytes[k] && a.comp_bytes[k] == c.comp_bytes[k];
        if (!ok) return fail(ctx, ACCB_EINVAL, "awhile: state array %d changes type", i);
    }
    if (max_iters < 1) return fail(ctx, ACCB_EINVAL, "awhile: max_iters must be positive");
    return ACCB_OK;
}

/* one graph: [cond, decide] -> WHILE { body, copy back, cond, decide } */
int awhile_record(accb_program *cond, accb_program *body, cudaStream_t s, const accb_array *state, long long max_iters) {
    accb_context *ctx = body->ctx;
    if (body->loop_exec) {
        cudaGraphExecDestroy(body->loop_exec);
        body->loop_exec = nullptr;
    }
    if (!body->loop_words)
        TRY(check_cuda(ctx, cudaMalloc((void **)&body->loop_words, 2 * sizeof(unsigned long long)), "cudaMalloc"));
    /* a run outside any capture sizes every pooled and scratch buffer and loads the kernels; the body's results
     * are not copied back, so the state is untouched */
    accb_array flag;
    std::vector<accb_array> outs(body->outputs.size());
    TRY(run_internal(cond, s, state, &flag, false));
    TRY(run_internal(body, s, state, outs.data(), false));
    TRY(check_cuda(ctx, cudaStreamSynchronize(s), "cudaStreamSynchronize"));

    cudaGraph_t g = nullptr;
    TRY(check_cuda(ctx, cudaGraphCreate(&g, 0), "cudaGraphCreate"));
    struct Guard {
        cudaGraph_t g;
        ~Guard() { cudaGraphDestroy(g); }
    } guard{g};
    cudaGraphConditionalHandle handle;
    TRY(check_cuda(ctx, cudaGraphConditionalHandleCreate(&handle, g, 0, cudaGraphCondAssignDefault),
                   "cudaGraphConditionalHandleCreate"));
    /* ahead of the loop */
    TRY(check_cuda(ctx, cudaStreamBeginCaptureToGraph(s, g, nullptr, nullptr, 0, cudaStreamCaptureModeRelaxed),
                   "cudaStreamBeginCaptureToGraph"));
    int st = run_internal(cond, s, state, &flag, false);
    std::vector<cudaGraphNode_t> deps;
    if (st == ACCB_OK) {
        awhile_step<<<1, 1, 0, s>>>(handle, static_cast<const unsigned char *>(flag.ptr[0]), body->loop_words,
                                    (unsigned long long)max_iters, 0);
        cudaStreamCaptureStatus cs;
        const cudaGraphNode_t *d = nullptr;
        size_t nd = 0;
        st = check_cuda(ctx, cudaStreamGetCaptureInfo(s, &cs, nullptr, nullptr, &d, &nd), "cudaStreamGetCaptureInfo");
        if (st == ACCB_OK) deps.assign(d, d + nd);
    }
    cudaGraph_t ended = nullptr;
    cudaError_t ce = cudaStreamEndCapture(s, &ended);
    TRY(st);
    TRY(check_cuda(ctx, ce, "cudaStreamEndCapture"));
    /* the loop */
    cudaGraphNodeParams params = {cudaGraphNodeTypeConditional}; /* the remaining members zero */
    params.type = cudaGraphNodeTypeConditional;
    params.conditional.handle = handle;
    params.conditional.type = cudaGraphCondTypeWhile;
    params.conditional.size = 1;
    cudaGraphNode_t loop;
    TRY(check_cuda(ctx, cudaGraphAddNode(&loop, g, deps.data(), deps.size(), &params), "cudaGraphAddNode (while)"));
    cudaGraph_t inside = params.conditional.phGraph_out[0];
    TRY(check_cuda(ctx, cudaStreamBeginCaptureToGraph(s, inside, nullptr, nullptr, 0, cudaStreamCaptureModeRelaxed),
                   "cudaStreamBeginCaptureToGraph"));
    st = run_internal(body, s, state, outs.data(), false);
    if (st == ACCB_OK) st = copy_back(body, s, state, outs);
    if (st == ACCB_OK) st = run_internal(cond, s, state, &flag, false);
    if (st == ACCB_OK)
        awhile_step<<<1, 1, 0, s>>>(handle, static_cast<const unsigned char *>(flag.ptr[0]), body->loop_words,
                                    (unsigned long long)max_iters, 1);
    ce = cudaStreamEndCapture(s, &ended);
    TRY(st);
    TRY(check_cuda(ctx, ce, "cudaStreamEndCapture"));
    const cudaError_t ci = cudaGraphInstantiate(&body->loop_exec, g, 0);
    if (ci != cudaSuccess) body->loop_exec = nullptr;
    TRY(check_cuda(ctx, ci, "cudaGraphInstantiate"));
    body->loop_stream = s;
    body->loop_cond = cond;
    body->loop_generation = ctx->buffer_generation;
    body->loop_max_iters = max_iters;
    body->loop_state.assign(state, state + body->ninputs);
    return ACCB_OK;
}

}  // namespace

extern "C" {

int accb_awhile(accb_program *cond, accb_program *body, accb_stream stream, const accb_array *state, int mode,
                long long max_iters, long long *iterations) {
    if (!cond) return fail(nullptr, ACCB_EINVAL, "null program");
    PLOCK(body);
    accb_context *ctx = body->ctx;
    TRY(awhile_check(cond, body, state, max_iters));
    cudaStream_t s = (cudaStream_t)stream;
    if (mode == ACCB_AWHILE_HOST) {
        long long done = 0;
        accb_array flag;
        std::vector<accb_array> outs(body->outputs.size());
        for (;;) {
            TRY(run_internal(cond, s, state, &flag, false));
            unsigned char go = 0;
            TRY(check_cuda(ctx, cudaMemcpyAsync(&go, flag.ptr[0], 1, cudaMemcpyDeviceToHost, s), "cudaMemcpyAsync"));
            TRY(check_cuda(ctx, cudaStreamSynchronize(s), "cudaStreamSynchronize"));
            if (!go) break;
            if (done >= max_iters) {
                if (iterations) *iterations = done;
                return fail(ctx, ACCB_ETIMEOUT, "awhile: still true after %lld iterations", done);
            }
            TRY(run_internal(body, s, state, outs.data(), false));
            TRY(copy_back(body, s, state, outs));
            ++done;
        }
        if (iterations) *iterations = done;
        return ACCB_OK;
    }
    if (mode != ACCB_AWHILE_DEVICE) return fail(ctx, ACCB_EINVAL, "awhile: unknown mode %d", mode);
    if (!s) return fail(ctx, ACCB_EINVAL, "a device-resident loop needs a stream of its own (the default stream cannot be captured)");
    bool same = body->loop_exec && body->loop_stream == s && body->loop_cond == cond &&
                body->loop_generation == ctx->buffer_generation && body->loop_max_iters == max_iters;
    for (int i = 0; same && i < body->ninputs; ++i) {
        same = same_shape(body->loop_state[i], state[i]);
        for (int c = 0; same && c < state[i].ncomp; ++c) same = body->loop_state[i].ptr[c] == state[i].ptr[c];
    }
    if (!same) TRY(awhile_record(cond, body, s, state, max_iters));
    TRY(check_cuda(ctx, cudaGraphLaunch(body->loop_exec, s), "cudaGraphLaunch"));
    if (iterations) {
        unsigned long long w[2] = {0, 0};
        TRY(check_cuda(ctx, cudaMemcpyAsync(w, body->loop_words, sizeof w, cudaMemcpyDeviceToHost, s), "cudaMemcpyAsync"));
        TRY(check_cuda(ctx, cudaStreamSynchronize(s), "cudaStreamSynchronize"));
        *iterations = (long long)w[0];
        if (w[1]) return fail(ctx, ACCB_ETIMEOUT, "awhile: still true after %lld iterations", (long long)w[0]);
    } else {
        /* nobody waits here: a loop cut off at max_iters is reported by the next accb_context_sync, as the
         * bounded waits of scans and permutes are */
        ctx->loops_unchecked.insert(body->loop_words);
    }
    return ACCB_OK;
}

int accb_program_destroy(accb_program *p) {
    if (!p) return ACCB_OK;
    {
        std::lock_guard<std::recursive_mutex> lock_(p->ctx->mu);
        CtxGuard g(p->ctx);
        cudaDeviceSynchronize();
        if (p->graph_exec) cudaGraphExecDestroy(p->graph_exec);
        if (p->loop_exec) cudaGraphExecDestroy(p->loop_exec);
        if (p->loop_words) {
            p->ctx->loops_unchecked.erase(p->loop_words);
            cudaFree(p->loop_words);
        }
        for (auto &v : p->pool)
            for (auto &b : v)
                if (b.ptr) cudaFree(b.ptr);
        for (auto &v : p->in_pool)
            for (auto &b : v)
                if (b.ptr) cudaFree(b.ptr);
        for (auto &b : p->slab_pool)
            if (b.ptr) cudaFree(b.ptr);
        if (p->host_stream) cudaStreamDestroy(p->host_stream);
        for (auto s : p->pipe_stream)
            if (s) cudaStreamDestroy(s);
        for (auto e : p->pipe_events) cudaEventDestroy(e);
    }
    delete p;
    return ACCB_OK;
}

/* ----------------------------------------------------- AccFFI.h surface */
AccHandle accelerateCreate(int32_t device, void *cu_context) {
    accb_context *ctx = nullptr;
    if (accb_context_create(device, cu_context, &ctx) != ACCB_OK) return nullptr;
    Handle *h = new Handle;
    h->ctx = ctx;
    return h;
}

void accelerateDestroy(AccHandle hndl) {
    Handle *h = static_cast<Handle *>(hndl);
    if (!h) return;
    accb_context_destroy(h->ctx);
    delete h;
}

int accelerateStatus(AccHandle hndl) {
    Handle *h = static_cast<Handle *>(hndl);
    return h ? h->status : ACCB_EINVAL;
}

accb_context *accelerateContext(AccHandle hndl) {
    Handle *h = static_cast<Handle *>(hndl);
    return h ? h->ctx : nullptr;
}

/* in: ninputs consecutive InputArray structs (device pointers, borrowed);
 * out: one OutputArray per program output, filled with malloc'ed shape and
 * pointer buffers that freeOutput releases (Export.hs:155-166,203-226). */
void runProgram(AccHandle hndl, AccProgram prog, InputArray *in, OutputArray *out) {
    Handle *h = static_cast<Handle *>(hndl);
    accb_program *p = static_cast<accb_program *>(prog);
    if (!h || !p || !out) {
        if (h) h->status = ACCB_EINVAL;
        return;
    }
    std::lock_guard<std::recursive_mutex> lock_(p->ctx->mu);
    CtxGuard g(p->ctx);
    std::vector<accb_array> inputs(p->ninputs);
    for (int i = 0; i < p->ninputs; ++i) {
        accb_array &a = inputs[i];
        memset(&a, 0, sizeof a);
        a.rank = p->types[i].rank;
        a.ncomp = p->types[i].ncomp;
        for (int d = 0; d < a.rank; ++d) a.shape[d] = in[i].shape[d];
        for (int c = 0; c < a.ncomp; ++c) a.ptr[c] = in[i].adata[c];
    }
    std::vector<accb_array> outputs(p->outputs.size());
    h->status = run_internal(p, nullptr, inputs.data(), outputs.data(), true);
    if (h->status == ACCB_OK) h->status = check_cuda(p->ctx, cudaStreamSynchronize(nullptr), "cudaStreamSynchronize");
    for (size_t j = 0; j < outputs.size(); ++j) {
        out[j].shape = nullptr;
        out[j].adata = nullptr;
        out[j].stable_ptr = nullptr;
        if (h->status != ACCB_OK) continue;
        const accb_array &a = outputs[j];
        out[j].shape = (int *)malloc(sizeof(int) * std::max(1, a.rank));
        out[j].adata = (void **)malloc(sizeof(void *) * a.ncomp);
        OutputOwner *own = new OutputOwner;
        own->ctx = p->ctx;
        for (int d = 0; d < a.rank; ++d) out[j].shape[d] = a.shape[d];
        for (int c = 0; c < a.ncomp; ++c) {
            out[j].adata[c] = a.ptr[c];
            own->ptrs.push_back(a.ptr[c]);
        }
        out[j].stable_ptr = own;
    }
}

void freeOutput(OutputArray *out) {
    if (!out) return;
    free(out->shape);
    free(out->adata);
    if (OutputOwner *own = static_cast<OutputOwner *>(out->stable_ptr)) {
        std::lock_guard<std::recursive_mutex> lock_(own->ctx->mu);
        CtxGuard g(own->ctx);
        for (void *q : own->ptrs) cudaFree(q);
        delete own;
    }
    out->shape = nullptr;
    out->adata = nullptr;
    out->stable_ptr = nullptr;
}

void freeProgram(AccProgram p) { accb_program_destroy(static_cast<accb_program *>(p)); }

} /* extern "C" */
