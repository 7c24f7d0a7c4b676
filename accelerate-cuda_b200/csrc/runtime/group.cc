/*
 * group.cc -- the skeletons over several GPUs driven from one process.
 *
 * The reference executes on one device per context (CUDA/State.hs:61-132);
 * its only multi-device primitive is the peer copy of
 * CUDA/Array/Prim.hs:306-335.  A group shards every array by contiguous slabs
 * of the outermost index space and joins the slabs with the smallest exchange
 * each skeleton allows:
 *
 *   map, fold over rows   none
 *   foldAll               one partial per rank -> rank 0 -> combined in rank order -> every rank
 *   scan                  slab totals -> rank 0 -> scan of the totals -> one carry per rank
 *   permute               partial destinations -> rank 0, merged one after another
 *   iterated stencil      iters*ry halo rows from each neighbour, once
 *   stencil2              ry halo rows of both sources from each neighbour
 *   foldSeg               none: split between segments, every rank's offsets rebased to its slice
 *
 * Exchanged data is copied into the receiving device's own memory before a
 * kernel reads it; devices are ordered with events only, so no kernel ever
 * waits for a kernel on another device.
 */
#include <algorithm>

#include "common.h"

using namespace accb_rt;

namespace {
constexpr size_t kSlot = 64;            /* bytes per component in the small per-rank areas */
constexpr size_t kPartialOff = 0;       /* this rank's partial / slab total */
constexpr size_t kCarryOff = 1024;      /* carry this rank's scan continues from */
constexpr size_t kDummyOff = 2048;      /* running totals nobody asked for */
constexpr size_t kSmallBytes = 4096;
}  // namespace

struct accb_group {
    int n = 0;
    std::vector<int> dev;
    std::vector<accb_context *> ctx;
    std::vector<cudaStream_t> st;
    std::vector<cudaEvent_t> ev_a, ev_b, ev_end; /* per rank: phase 1 done, phase 2 done, operation enqueued */
    std::vector<char *> small;                    /* kSmallBytes per rank, on the rank's device */
    char *gather = nullptr;                       /* rank 0: gathered partials, then the carries */
    size_t gather_comp = 0;                       /* bytes reserved per component in `gather` */
    char *stage = nullptr;                        /* rank 0: a peer's partial destination */
    size_t stage_bytes = 0;
    std::vector<int *> seg_offsets;               /* per rank: a slice's segment offsets, rebased to start at zero */
    std::vector<size_t> seg_capacity;             /* ... and how many values fit */
    std::mutex mu;
    std::string last_error;
};

namespace {

int gfail(accb_group *g, int code, const char *fmt, ...) {
    char buf[512];
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(buf, sizeof buf, fmt, ap);
    va_end(ap);
    if (g) g->last_error = buf;
    set_global_error(buf);
    return code;
}

/* an accb_* call on rank r failed: keep its message */
int inner(accb_group *g, int r, int st) {
    if (st != ACCB_OK) {
        const char *m = accb_last_error(g->ctx[r]);
        g->last_error = std::string("rank ") + std::to_string(r) + ": " + (m ? m : "");
        set_global_error(g->last_error);
    }
    return st;
}

int cuda(accb_group *g, cudaError_t e, const char *what) {
    if (e == cudaSuccess) return ACCB_OK;
    return gfail(g, ACCB_ECUDA, "%s: %s", what, cudaGetErrorString(e));
}

#define GTRY(expr)                        \
    do {                                  \
        int st_ = (expr);                 \
        if (st_ != ACCB_OK) return st_;   \
    } while (0)
#define GLOCK(g)                                                          \
    if (!(g)) return gfail(nullptr, ACCB_EINVAL, "null group");           \
    std::lock_guard<std::mutex> glock_((g)->mu)

/* enqueue on rank `dst`'s stream a copy from rank `src`'s memory */
int copy_between(accb_group *g, int dst, void *to, int src, const void *from, size_t bytes) {
    if (bytes == 0) return ACCB_OK;
    CtxGuard guard(g->ctx[dst]);
    if (g->dev[dst] == g->dev[src])
        return cuda(g, cudaMemcpyAsync(to, from, bytes, cudaMemcpyDeviceToDevice, g->st[dst]), "cudaMemcpyAsync");
    return cuda(g, cudaMemcpyPeerAsync(to, g->dev[dst], from, g->dev[src], bytes, g->st[dst]), "cudaMemcpyPeerAsync");
}

int record(accb_group *g, std::vector<cudaEvent_t> &ev, int r) {
    CtxGuard guard(g->ctx[r]);
    return cuda(g, cudaEventRecord(ev[r], g->st[r]), "cudaEventRecord");
}

/* rank r's stream waits for what rank `of` had enqueued when it recorded ev[of] */
int wait_for(accb_group *g, int r, std::vector<cudaEvent_t> &ev, int of) {
    if (r == of) return ACCB_OK; /* stream order */
    CtxGuard guard(g->ctx[r]);
    return cuda(g, cudaStreamWaitEvent(g->st[r], ev[of], 0), "cudaStreamWaitEvent");
}

/* Start of an operation that exchanges through rank 0: rank 0 must not overwrite its gather area while a rank still
 * copies the previous operation's result out of it, and no rank may overwrite its small area while rank 0 still
 * copies from it. */
int op_begin(accb_group *g) {
    for (int r = 1; r < g->n; ++r) GTRY(wait_for(g, 0, g->ev_end, r));
    for (int r = 1; r < g->n; ++r) GTRY(wait_for(g, r, g->ev_end, 0));
    return ACCB_OK;
}

int op_end(accb_group *g) {
    for (int r = 0; r < g->n; ++r) GTRY(record(g, g->ev_end, r));
    return ACCB_OK;
}

accb_array scalar_at(char *base, int ncomp) {
    accb_array a;
    memset(&a, 0, sizeof a);
    a.rank = 0;
    a.ncomp = ncomp;
    for (int c = 0; c < ncomp; ++c) a.ptr[c] = base + c * kSlot;
    return a;
}

int check_comp(accb_group *g, int ncomp, const int *comp_bytes) {
    if (ncomp < 1 || ncomp > ACCB_ARRAY_MAX_COMP) return gfail(g, ACCB_EINVAL, "bad component count %d", ncomp);
    if (!comp_bytes) return gfail(g, ACCB_EINVAL, "null comp_bytes");
    for (int c = 0; c < ncomp; ++c)
        if (comp_bytes[c] < 1 || (size_t)comp_bytes[c] > kSlot / 4)
            return gfail(g, ACCB_EINVAL, "component %d of %d bytes", c, comp_bytes[c]);
    return ACCB_OK;
}

long long elements(const accb_array &a) {
    long long n = 1;
    for (int d = 0; d < a.rank; ++d) n *= a.shape[d];
    return n;
}

}  // namespace

extern "C" {

int accb_group_create(const int *devices, int n, accb_group **out) {
    if (!out) return gfail(nullptr, ACCB_EINVAL, "null out pointer");
    *out = nullptr;
    if (!devices || n < 1 || n > 64) return gfail(nullptr, ACCB_EINVAL, "a group has 1..64 ranks");
    std::unique_ptr<accb_group> g(new accb_group);
    g->n = n;
    int st = ACCB_OK;
    for (int r = 0; r < n && st == ACCB_OK; ++r) {
        accb_context *c = nullptr;
        st = accb_context_create(devices[r], nullptr, &c);
        if (st != ACCB_OK) {
            g->last_error = accb_last_error(nullptr);
            break;
        }
        g->dev.push_back(devices[r]);
        g->ctx.push_back(c);
        accb_stream s = nullptr;
        st = accb_stream_acquire(c, &s);
        if (st != ACCB_OK) break;
        g->st.push_back((cudaStream_t)s);
        CtxGuard guard(c);
        cudaEvent_t e[3] = {nullptr, nullptr, nullptr};
        for (int i = 0; i < 3 && st == ACCB_OK; ++i)
            st = cuda(g.get(), cudaEventCreateWithFlags(&e[i], cudaEventDisableTiming), "cudaEventCreate");
        g->ev_a.push_back(e[0]);
        g->ev_b.push_back(e[1]);
        g->ev_end.push_back(e[2]);
        char *p = nullptr;
        if (st == ACCB_OK) st = cuda(g.get(), cudaMalloc((void **)&p, kSmallBytes), "cudaMalloc");
        g->small.push_back(p);
    }
    if (st == ACCB_OK) {
        CtxGuard guard(g->ctx[0]);
        g->gather_comp = ((size_t)(n + 1) * (kSlot / 4) + 255) / 256 * 256;
        st = cuda(g.get(), cudaMalloc((void **)&g->gather, 2 * ACCB_ARRAY_MAX_COMP * g->gather_comp), "cudaMalloc");
    }
    /* direct peer copies where the devices allow it; otherwise the copies are staged by the driver */
    for (int i = 0; i < n && st == ACCB_OK; ++i)
        for (int j = 0; j < n; ++j) {
            if (g->dev[i] == g->dev[j]) continue;
            int can = 0;
            if (cudaDeviceCanAccessPeer(&can, g->dev[i], g->dev[j]) != cudaSuccess || !can) {
                cudaGetLastError();
                continue;
            }
            CtxGuard on_i(g->ctx[i]); /* makes dev[i] current and hands the caller's device back afterwards */
            if (cudaDeviceEnablePeerAccess(g->dev[j], 0) != cudaSuccess) cudaGetLastError(); /* already enabled */
        }
    if (st != ACCB_OK) {
        set_global_error(g->last_error);
        accb_group_destroy(g.release());
        return st;
    }
    *out = g.release();
    return ACCB_OK;
}

int accb_group_destroy(accb_group *g) {
    if (!g) return ACCB_OK;
    for (size_t r = 0; r < g->ctx.size(); ++r) {
        CtxGuard guard(g->ctx[r]);
        if (r < g->st.size()) cudaStreamSynchronize(g->st[r]);
        if (r < g->ev_a.size() && g->ev_a[r]) cudaEventDestroy(g->ev_a[r]);
        if (r < g->ev_b.size() && g->ev_b[r]) cudaEventDestroy(g->ev_b[r]);
        if (r < g->ev_end.size() && g->ev_end[r]) cudaEventDestroy(g->ev_end[r]);
        if (r < g->small.size() && g->small[r]) cudaFree(g->small[r]);
        if (r < g->seg_offsets.size() && g->seg_offsets[r]) cudaFree(g->seg_offsets[r]);
        if (r == 0) {
            if (g->gather) cudaFree(g->gather);
            if (g->stage) cudaFree(g->stage);
        }
        if (r < g->st.size()) accb_stream_release(g->ctx[r], g->st[r]);
    }
    for (accb_context *c : g->ctx) accb_context_destroy(c);
    delete g;
    return ACCB_OK;
}

int accb_group_size(accb_group *g, int *n) {
    GLOCK(g);
    if (!n) return gfail(g, ACCB_EINVAL, "null pointer");
    *n = g->n;
    return ACCB_OK;
}

int accb_group_context(accb_group *g, int rank, accb_context **ctx) {
    GLOCK(g);
    if (!ctx || rank < 0 || rank >= g->n) return gfail(g, ACCB_EINVAL, "no rank %d", rank);
    *ctx = g->ctx[rank];
    return ACCB_OK;
}

int accb_group_stream(accb_group *g, int rank, accb_stream *stream) {
    GLOCK(g);
    if (!stream || rank < 0 || rank >= g->n) return gfail(g, ACCB_EINVAL, "no rank %d", rank);
    *stream = g->st[rank];
    return ACCB_OK;
}

int accb_group_sync(accb_group *g) {
    GLOCK(g);
    for (int r = 0; r < g->n; ++r) GTRY(inner(g, r, accb_stream_sync(g->ctx[r], g->st[r])));
    for (int r = 0; r < g->n; ++r) GTRY(inner(g, r, accb_context_sync(g->ctx[r])));
    return ACCB_OK;
}

const char *accb_group_last_error(accb_group *g) { return g ? g->last_error.c_str() : accb_last_error(nullptr); }

/* ------------------------------------------------------ no exchange */
int accb_group_map(accb_group *g, accb_kernel *k, const accb_array *env, int nenv, const void *scalars,
                   size_t scalar_bytes, const accb_array *out) {
    GLOCK(g);
    if (!out || (nenv > 0 && !env)) return gfail(g, ACCB_EINVAL, "null arrays");
    for (int r = 0; r < g->n; ++r)
        GTRY(inner(g, r, accb_map(g->ctx[r], k, g->st[r], env + (size_t)r * nenv, nenv, scalars, scalar_bytes, &out[r])));
    return ACCB_OK;
}

int accb_group_fold_dim(accb_group *g, accb_kernel *k, const accb_array *env, int nenv, const long long *rows,
                        long long cols, const void *seed, size_t seed_bytes, const accb_array *out) {
    GLOCK(g);
    if (!out || !rows || (nenv > 0 && !env)) return gfail(g, ACCB_EINVAL, "null arrays");
    for (int r = 0; r < g->n; ++r)
        GTRY(inner(g, r, accb_fold_dim(g->ctx[r], k, g->st[r], env + (size_t)r * nenv, nenv, rows[r], cols, seed,
                                       seed_bytes, &out[r])));
    return ACCB_OK;
}

/* ---------------------------------------------------------- foldAll */
int accb_group_fold_all(accb_group *g, accb_kernel *k, accb_kernel *k_combine, const accb_array *env, int nenv,
                        const long long *n, const void *seed, size_t seed_bytes, const int *comp_bytes,
                        const accb_array *out) {
    GLOCK(g);
    if (!out || !n || (nenv > 0 && !env)) return gfail(g, ACCB_EINVAL, "null arrays");
    const int nc = out[0].ncomp;
    GTRY(check_comp(g, nc, comp_bytes));
    for (int r = 0; r < g->n; ++r)
        if (n[r] < 1) return gfail(g, ACCB_EINVAL, "rank %d has an empty slab", r);
    if (g->n == 1) return inner(g, 0, accb_fold_all(g->ctx[0], k, g->st[0], env, nenv, n[0], seed, seed_bytes, &out[0]));
    GTRY(op_begin(g));
    for (int r = 0; r < g->n; ++r) {
        const accb_array part = scalar_at(g->small[r] + kPartialOff, nc);
        GTRY(inner(g, r, accb_fold_all(g->ctx[r], k, g->st[r], env + (size_t)r * nenv, nenv, n[r], nullptr, 0, &part)));
        GTRY(record(g, g->ev_a, r));
    }
    accb_array all;
    memset(&all, 0, sizeof all);
    all.rank = 1;
    all.shape[0] = g->n;
    all.ncomp = nc;
    for (int c = 0; c < nc; ++c) all.ptr[c] = g->gather + c * g->gather_comp;
    for (int r = 0; r < g->n; ++r) {
        GTRY(wait_for(g, 0, g->ev_a, r));
        for (int c = 0; c < nc; ++c)
            GTRY(copy_between(g, 0, (char *)all.ptr[c] + (size_t)r * comp_bytes[c], r,
                              g->small[r] + kPartialOff + c * kSlot, comp_bytes[c]));
    }
    GTRY(inner(g, 0, accb_fold_all(g->ctx[0], k_combine, g->st[0], &all, 1, g->n, seed, seed_bytes, &out[0])));
    GTRY(record(g, g->ev_b, 0));
    for (int r = 1; r < g->n; ++r) {
        GTRY(wait_for(g, r, g->ev_b, 0));
        for (int c = 0; c < nc; ++c) GTRY(copy_between(g, r, out[r].ptr[c], 0, out[0].ptr[c], comp_bytes[c]));
    }
    return op_end(g);
}

/* ------------------------------------------------------------- scan */
int accb_group_scan(accb_group *g, accb_kernel *k, accb_kernel *k_total, accb_kernel *k_carry, const accb_array *env,
                    int nenv, const long long *n, int direction, int kind, const void *seed, size_t seed_bytes,
                    size_t elt_bytes, const accb_array *out, const accb_array *total) {
    GLOCK(g);
    if (!out || !n || (nenv > 0 && !env)) return gfail(g, ACCB_EINVAL, "null arrays");
    if (kind != ACCB_SCAN_EXCLUSIVE && kind != ACCB_SCAN_INCLUSIVE && kind != ACCB_SCAN_PRIME)
        return gfail(g, ACCB_EINVAL, "scan kind %d", kind);
    if (kind == ACCB_SCAN_PRIME && !total) return gfail(g, ACCB_EINVAL, "scan' needs the total arrays");
    if ((kind == ACCB_SCAN_INCLUSIVE) != (seed == nullptr))
        return gfail(g, ACCB_EINVAL, "scanl/scanr/scan' need a seed, scanl1/scanr1 take none");
    if (out[0].ncomp != 1) return gfail(g, ACCB_EINVAL, "group scans take one-component elements");
    if (elt_bytes < 1 || elt_bytes > kSlot / 4) return gfail(g, ACCB_EINVAL, "element of %zu bytes", elt_bytes);
    if (seed && seed_bytes != elt_bytes) return gfail(g, ACCB_EINVAL, "seed and element sizes differ");
    const int G = g->n, last = G - 1;
    for (int r = 0; r < G; ++r)
        if (n[r] < 1) return gfail(g, ACCB_EINVAL, "rank %d has an empty slab", r);
    if (G == 1)
        return inner(g, 0, accb_scan(g->ctx[0], k, g->st[0], env, nenv, n[0], direction, kind, seed, seed_bytes, &out[0],
                                     total ? &total[0] : nullptr));
    const bool right = direction == ACCB_SCAN_RIGHT;
    const int m = G - 1;             /* totals that some carry needs */
    const int first_total = right ? 1 : 0; /* left: ranks 0..G-2; right: ranks 1..G-1 */
    GTRY(op_begin(g));
    for (int i = 0; i < m; ++i) {
        const int r = first_total + i;
        const accb_array part = scalar_at(g->small[r] + kPartialOff, 1);
        GTRY(inner(g, r, accb_fold_all(g->ctx[r], k_total, g->st[r], env + (size_t)r * nenv, nenv, n[r], nullptr, 0, &part)));
        GTRY(record(g, g->ev_a, r));
    }
    /* rank 0: totals T[0..m), carries C = scan of T */
    char *T = g->gather, *Cc = g->gather + ACCB_ARRAY_MAX_COMP * g->gather_comp;
    for (int i = 0; i < m; ++i) {
        const int r = first_total + i;
        GTRY(wait_for(g, 0, g->ev_a, r));
        GTRY(copy_between(g, 0, T + (size_t)i * elt_bytes, r, g->small[r] + kPartialOff, elt_bytes));
    }
    accb_array tarr, carr;
    memset(&tarr, 0, sizeof tarr);
    tarr.rank = 1;
    tarr.shape[0] = m;
    tarr.ncomp = 1;
    tarr.ptr[0] = T;
    carr = tarr;
    carr.shape[0] = seed ? m + 1 : m;
    carr.ptr[0] = Cc;
    GTRY(inner(g, 0, accb_scan(g->ctx[0], k_carry, g->st[0], &tarr, 1, m, direction,
                               seed ? ACCB_SCAN_EXCLUSIVE : ACCB_SCAN_INCLUSIVE, seed, seed_bytes, &carr, nullptr)));
    GTRY(record(g, g->ev_b, 0));
    /* Where rank r's carry sits in C.  With a seed C has m+1 entries and C[r] is the carry of rank r in both
     * directions (left: seed and the totals before r; right: the totals after r and the seed).  Without one, the
     * first (left) or last (right) rank has no carry and the others read C[r-1] (left) or C[r] (right). */
    for (int r = 0; r < G; ++r) {
        int idx;
        if (seed) idx = r;
        else if (!right) idx = r - 1;
        else idx = r < last ? r : -1;
        GTRY(wait_for(g, r, g->ev_b, 0));
        char *carry = g->small[r] + kCarryOff;
        if (idx >= 0) GTRY(copy_between(g, r, carry, 0, Cc + (size_t)idx * elt_bytes, elt_bytes));
        accb_array dummy = scalar_at(g->small[r] + kDummyOff, 1);
        const accb_array *tot = (total && total[r].ncomp == 1 && total[r].ptr[0]) ? &total[r] : &dummy;
        int local;
        if (kind == ACCB_SCAN_PRIME) {
            local = ACCB_SCAN_PRIME;
        } else if (kind == ACCB_SCAN_EXCLUSIVE) {
            /* the last rank writes the extra element; earlier ranks the exclusive (left) or inclusive (right) body */
            local = r == last ? ACCB_SCAN_EXCLUSIVE : (right ? ACCB_SCAN_INCLUSIVE_SEEDED : ACCB_SCAN_PRIME);
        } else {
            local = idx >= 0 ? ACCB_SCAN_INCLUSIVE_SEEDED : ACCB_SCAN_INCLUSIVE;
        }
        const bool seeded = local != ACCB_SCAN_INCLUSIVE;
        GTRY(inner(g, r, accb_scan(g->ctx[r], k, g->st[r], env + (size_t)r * nenv, nenv, n[r], direction,
                                   seeded ? (local | ACCB_SEED_ON_DEVICE) : local, seeded ? (const void *)carry : nullptr,
                                   seeded ? elt_bytes : 0, &out[r], local == ACCB_SCAN_PRIME ? tot : nullptr)));
    }
    return op_end(g);
}

/* ---------------------------------------------------------- permute */
int accb_group_permute(accb_group *g, accb_kernel *k, accb_kernel *k_merge, const accb_array *env, int nenv,
                       const long long *n_src, const void *scalars, size_t scalar_bytes, const int *comp_bytes,
                       const accb_array *out, int broadcast) {
    GLOCK(g);
    if (!out || !n_src || (nenv > 0 && !env)) return gfail(g, ACCB_EINVAL, "null arrays");
    const int nc = out[0].ncomp;
    GTRY(check_comp(g, nc, comp_bytes));
    const long long cells = elements(out[0]);
    for (int r = 1; r < g->n; ++r)
        if (elements(out[r]) != cells || out[r].ncomp != nc)
            return gfail(g, ACCB_EINVAL, "rank %d: destination differs from rank 0's", r);
    GTRY(op_begin(g));
    for (int r = 0; r < g->n; ++r) {
        GTRY(inner(g, r, accb_permute(g->ctx[r], k, g->st[r], env + (size_t)r * nenv, nenv, n_src[r], scalars,
                                      scalar_bytes, &out[r])));
        GTRY(record(g, g->ev_a, r));
    }
    if (g->n > 1) {
        /* staging area on rank 0: one component after another, each 256-byte aligned */
        size_t off[ACCB_ARRAY_MAX_COMP + 1] = {0};
        for (int c = 0; c < nc; ++c) off[c + 1] = off[c] + ((size_t)cells * comp_bytes[c] + 255) / 256 * 256;
        if (g->stage_bytes < off[nc]) {
            CtxGuard guard(g->ctx[0]);
            GTRY(cuda(g, cudaStreamSynchronize(g->st[0]), "cudaStreamSynchronize"));
            if (g->stage) cudaFree(g->stage);
            g->stage = nullptr;
            g->stage_bytes = 0;
            GTRY(cuda(g, cudaMalloc((void **)&g->stage, off[nc]), "cudaMalloc"));
            g->stage_bytes = off[nc];
        }
        accb_array pair[2];
        pair[0] = out[0];
        for (int c = 0; c < nc; ++c) pair[0].ptr[c] = g->stage + off[c];
        pair[1] = out[0];
        for (int r = 1; r < g->n; ++r) {
            GTRY(wait_for(g, 0, g->ev_a, r));
            for (int c = 0; c < nc; ++c)
                GTRY(copy_between(g, 0, pair[0].ptr[c], r, out[r].ptr[c], (size_t)cells * comp_bytes[c]));
            /* element-wise and in place: every thread reads the cells it then writes */
            GTRY(inner(g, 0, accb_map(g->ctx[0], k_merge, g->st[0], pair, 2, nullptr, 0, &out[0])));
        }
        if (broadcast) {
            GTRY(record(g, g->ev_b, 0));
            for (int r = 1; r < g->n; ++r) {
                GTRY(wait_for(g, r, g->ev_b, 0));
                for (int c = 0; c < nc; ++c)
                    GTRY(copy_between(g, r, out[r].ptr[c], 0, out[0].ptr[c], (size_t)cells * comp_bytes[c]));
            }
        }
    }
    return op_end(g);
}

/* ---------------------------------------------------------- stencil */
/* elements of one "row" of a slab: the slabs are cut along the outermost dimension, so a row of a matrix is a row
 * and a row of a cube is a plane */
static size_t slab_row_elems(const accb_array &a) {
    size_t n = 1;
    for (int d = 0; d + 1 < a.rank; ++d) n *= (size_t)a.shape[d];
    return n;
}

static void halo_rows(const accb_group *g, int rank, int reach, int boundary, int *top, int *bottom) {
    const bool ring = boundary == ACCB_WRAP && g->n > 1;
    *top = (rank > 0 || ring) ? reach : 0;
    *bottom = (rank < g->n - 1 || ring) ? reach : 0;
}

int accb_group_stencil_layout(accb_group *g, int rank, int iters, int ry, int boundary, int *pad_top, int *pad_bottom) {
    GLOCK(g);
    if (rank < 0 || rank >= g->n || iters < 0 || ry < 0 || !pad_top || !pad_bottom)
        return gfail(g, ACCB_EINVAL, "bad stencil layout query");
    halo_rows(g, rank, iters * ry, boundary, pad_top, pad_bottom);
    return ACCB_OK;
}

/* Fill the `reach` halo rows of every rank's padded slab a[r] (pt[r] + rows[r] + pb[r] rows) from the neighbours' own
 * rows by peer copies; afterwards ev_b[r] marks that rank r has read its neighbours. */
static int fill_halos(accb_group *g, const accb_array *a, const int *rows, const std::vector<int> &pt, const std::vector<int> &pb,
                      const std::vector<size_t> &row_elems, int reach, int nc, const int *comp_bytes) {
    const int G = g->n;
    for (int r = 0; r < G; ++r) GTRY(record(g, g->ev_a, r)); /* the slab's own rows are final */
    for (int r = 0; r < G; ++r) {
        const int up = (r + G - 1) % G, down = (r + 1) % G;
        for (int c = 0; c < nc; ++c) {
            const size_t rb = row_elems[r] * comp_bytes[c];
            if (pt[r]) { /* the last rows of the rank above */
                GTRY(wait_for(g, r, g->ev_a, up));
                GTRY(copy_between(g, r, a[r].ptr[c], up, (const char *)a[up].ptr[c] + (size_t)(pt[up] + rows[up] - reach) * rb,
                                  (size_t)reach * rb));
            }
            if (pb[r]) { /* the first rows of the rank below */
                GTRY(wait_for(g, r, g->ev_a, down));
                GTRY(copy_between(g, r, (char *)a[r].ptr[c] + (size_t)(pt[r] + rows[r]) * rb, down,
                                  (const char *)a[down].ptr[c] + (size_t)pt[down] * rb, (size_t)reach * rb));
            }
        }
        GTRY(record(g, g->ev_b, r));
    }
    return ACCB_OK;
}

/* padded row slabs of one array per rank: shapes against the layout, elements per row */
static int check_slabs(accb_group *g, const accb_array *a, const int *rows, const std::vector<int> &pt, const std::vector<int> &pb,
                       int nc, std::vector<size_t> &row_elems) {
    for (int r = 0; r < g->n; ++r) {
        if (a[r].rank < 1 || a[r].rank > 3 || a[r].ncomp != nc)
            return gfail(g, ACCB_EINVAL, "rank %d: slabs must be vectors, matrices or cubes of the same type", r);
        const int outer = a[r].shape[a[r].rank - 1];
        row_elems[r] = slab_row_elems(a[r]);
        if (outer != pt[r] + rows[r] + pb[r] || row_elems[r] != row_elems[0])
            return gfail(g, ACCB_EINVAL, "rank %d: slab of %d rows, expected %d + %d + %d", r, outer, pt[r], rows[r], pb[r]);
    }
    return ACCB_OK;
}

int accb_group_stencil2(accb_group *g, accb_kernel *k, const accb_array *a, const accb_array *b, const accb_array *out,
                        const int *rows, int ry, int boundary, const void *constant, size_t constant_bytes,
                        const int *comp_bytes) {
    GLOCK(g);
    if (!a || !b || !out || !rows) return gfail(g, ACCB_EINVAL, "null arrays");
    if (ry < 0) return gfail(g, ACCB_EINVAL, "negative reach");
    const int G = g->n, nc = a[0].ncomp;
    GTRY(check_comp(g, nc, comp_bytes));
    std::vector<int> pt(G), pb(G);
    std::vector<size_t> re_a(G), re_b(G);
    for (int r = 0; r < G; ++r) {
        halo_rows(g, r, ry, boundary, &pt[r], &pb[r]);
        if (G > 1 && rows[r] < ry) return gfail(g, ACCB_EINVAL, "rank %d owns %d rows, fewer than the halo of %d", r, rows[r], ry);
    }
    GTRY(check_slabs(g, a, rows, pt, pb, nc, re_a));
    GTRY(check_slabs(g, b, rows, pt, pb, nc, re_b));
    if (G > 1 && ry > 0) {
        GTRY(fill_halos(g, a, rows, pt, pb, re_a, ry, nc, comp_bytes));
        /* the second source reuses the events: rank r's copies are ordered on its stream, the neighbours' rows of b
         * were final before this call as well */
        GTRY(fill_halos(g, b, rows, pt, pb, re_b, ry, nc, comp_bytes));
        /* whatever a rank enqueues next may overwrite its sources: the neighbours must have read them by then */
        for (int r = 0; r < G; ++r) {
            if (pt[r]) GTRY(wait_for(g, r, g->ev_b, (r + G - 1) % G));
            if (pb[r]) GTRY(wait_for(g, r, g->ev_b, (r + 1) % G));
        }
    }
    /* every rank applies the stencil to its padded slabs: the result's own rows are right, its halo rows (computed
     * from rows the rank does not have) are not and belong to the neighbours anyway */
    for (int r = 0; r < G; ++r)
        GTRY(inner(g, r, accb_stencil2(g->ctx[r], k, g->st[r], &a[r], &b[r], boundary, constant, constant_bytes, &out[r])));
    return ACCB_OK;
}

/* ------------------------------------------------------------ foldSeg */
int accb_seg_partition(const int *offsets, long long nseg, int parts, long long *first_seg) {
    if (!offsets || !first_seg || nseg < 0 || parts < 1) return gfail(nullptr, ACCB_EINVAL, "bad segment partition request");
    /* part p starts at the first segment whose offset reaches p/parts of all elements: runs of whole segments
     * holding about the same number of elements (a segment is never cut) */
    const long long total = (long long)offsets[nseg] - offsets[0];
    first_seg[0] = 0;
    for (int p = 1; p < parts; ++p) {
        const long long want = offsets[0] + total * p / parts;
        const int *it = std::lower_bound(offsets, offsets + nseg + 1, (int)std::min<long long>(want, 0x7fffffffLL));
        first_seg[p] = std::max(first_seg[p - 1], std::min<long long>(it - offsets, nseg));
    }
    first_seg[parts] = nseg;
    return ACCB_OK;
}

int accb_group_fold_seg(accb_group *g, accb_kernel *k, const accb_array *env, int nenv, const long long *n,
                        const int *const *offsets, const long long *nseg, const void *seed, size_t seed_bytes,
                        const accb_array *out) {
    GLOCK(g);
    if (!out || !n || !offsets || !nseg || (nenv > 0 && !env)) return gfail(g, ACCB_EINVAL, "null arrays");
    if (g->seg_offsets.empty()) {
        g->seg_offsets.assign(g->n, nullptr);
        g->seg_capacity.assign(g->n, 0);
    }
    for (int r = 0; r < g->n; ++r) {
        if (nseg[r] < 0 || n[r] < 0) return gfail(g, ACCB_EINVAL, "rank %d: negative extent", r);
        if (nseg[r] == 0) continue;
        if (!offsets[r]) return gfail(g, ACCB_EINVAL, "rank %d: null segment offsets", r);
        CtxGuard guard(g->ctx[r]);
        const size_t need = (size_t)nseg[r] + 1;
        if (g->seg_capacity[r] < need) {
            GTRY(cuda(g, cudaStreamSynchronize(g->st[r]), "cudaStreamSynchronize")); /* earlier folds may still read it */
            if (g->seg_offsets[r]) cudaFree(g->seg_offsets[r]);
            g->seg_offsets[r] = nullptr;
            g->seg_capacity[r] = 0;
            GTRY(cuda(g, cudaMalloc((void **)&g->seg_offsets[r], need * sizeof(int)), "cudaMalloc"));
            g->seg_capacity[r] = need;
        }
        /* the rank's offsets are a run of the whole array's: made to start at zero, they index its own slice */
        GTRY(inner(g, r, rebase_offsets(g->ctx[r], g->st[r], g->seg_offsets[r], offsets[r], (long long)need)));
        GTRY(inner(g, r, accb_fold_seg(g->ctx[r], k, g->st[r], env + (size_t)r * nenv, nenv, 1, n[r], g->seg_offsets[r], nseg[r],
                                       seed, seed_bytes, &out[r])));
    }
    return ACCB_OK;
}

int accb_group_stencil_iterate(accb_group *g, accb_kernel *k, const accb_array *a, const accb_array *b, const int *rows,
                               int iters, int ry, int boundary, const void *constant, size_t constant_bytes,
                               const int *comp_bytes, int *result_in_b) {
    GLOCK(g);
    if (!a || !b || !rows || !result_in_b) return gfail(g, ACCB_EINVAL, "null arrays");
    if (iters < 0 || ry < 0) return gfail(g, ACCB_EINVAL, "negative iteration count or reach");
    const int G = g->n, reach = iters * ry, nc = a[0].ncomp;
    GTRY(check_comp(g, nc, comp_bytes));
    std::vector<int> pt(G), pb(G);
    std::vector<size_t> row_elems(G);
    for (int r = 0; r < G; ++r) {
        halo_rows(g, r, reach, boundary, &pt[r], &pb[r]);
        if (a[r].rank < 1 || a[r].rank > 3 || b[r].rank != a[r].rank || a[r].ncomp != nc || b[r].ncomp != nc)
            return gfail(g, ACCB_EINVAL, "rank %d: slabs must be vectors, matrices or cubes of the same type", r);
        const int outer = a[r].shape[a[r].rank - 1];
        row_elems[r] = slab_row_elems(a[r]);
        if (outer != pt[r] + rows[r] + pb[r] || b[r].shape[b[r].rank - 1] != outer || row_elems[r] != row_elems[0])
            return gfail(g, ACCB_EINVAL, "rank %d: slab of %d rows, expected %d + %d + %d", r, outer, pt[r], rows[r], pb[r]);
        if (G > 1 && rows[r] < reach)
            return gfail(g, ACCB_EINVAL, "rank %d owns %d rows, fewer than the halo of %d: use fewer iterations per call",
                         r, rows[r], reach);
    }
    if (G > 1 && reach > 0) {
        GTRY(fill_halos(g, a, rows, pt, pb, row_elems, reach, nc, comp_bytes));
        /* a rank's second application overwrites a[r]: the neighbours must have read it by then */
        for (int r = 0; r < G; ++r) {
            if (pt[r]) GTRY(wait_for(g, r, g->ev_b, (r + G - 1) % G));
            if (pb[r]) GTRY(wait_for(g, r, g->ev_b, (r + 1) % G));
        }
    }
    std::vector<int> in_b(G, 0);
    for (int r = 0; r < G; ++r)
        GTRY(inner(g, r, accb_stencil_iterate(g->ctx[r], k, g->st[r], &a[r], &b[r], iters, boundary, constant,
                                              constant_bytes, &in_b[r])));
    /* a rank whose slab took another number of launches (a very thin slab runs one application per launch, the
     * others two) ends in the other buffer: copy, so that the answer is the same buffer on every rank */
    for (int r = 1; r < G; ++r) {
        if (in_b[r] == in_b[0]) continue;
        const accb_array &from = in_b[r] ? b[r] : a[r], &to = in_b[r] ? a[r] : b[r];
        const size_t n = row_elems[r] * (size_t)from.shape[from.rank - 1];
        for (int c = 0; c < nc; ++c) GTRY(copy_between(g, r, to.ptr[c], r, from.ptr[c], n * comp_bytes[c]));
    }
    *result_in_b = in_b[0];
    return ACCB_OK;
}

}  // extern "C"
