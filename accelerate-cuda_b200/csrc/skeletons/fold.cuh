/*
 * fold.cuh -- reductions: foldAll / fold1All, fold / fold1 over the innermost
 * dimension, foldSeg / fold1Seg.
 *
 * Replaces mkFoldAll' (two kernels relaunched until one value is left,
 * Data/Array/Accelerate/CUDA/CodeGen/Reduction.hs:87-215 with the host
 * recursion foldCore/foldRec, Execute.hs:291-318), mkFoldDim (one block per
 * row, Reduction.hs:221-367) and mkFoldSeg' (one warp per segment,
 * Reduction.hs:421-574).  Semantics kept from there:
 *   - the seed is combined on the right, f(acc, seed) (Reduction.hs:203-215,
 *     364-367, 567-574); an empty input yields the seed (:204-214, :351-362);
 *   - like the reference's strided accumulation (:160-165) the combiner is
 *     assumed associative AND commutative.
 *
 * Functor contract (derive from accb::Fold<T[, Acc]> for the defaults):
 *   using In  = accb::types<...>;          element-wise inputs of the producer
 *   typedef T  elem;  typedef Acc acc;     value type / accumulator type
 *   static T   get(env, i, in-values...);  the fused producer
 *   static Acc lift(T);  static T lower(Acc);
 *   static Acc combine(Acc, Acc);
 *   using Out = accb::types<...>;  static void put(T, out-references...);
 * `Acc` wider than `T` (double for a recognised (+) on Float) keeps a float32
 * sum within one rounding of the exact result.
 *
 * foldAll is ONE launch: persistent blocks accumulate with 128-bit streaming
 * loads, write one partial each, and the block that finishes last (ticket
 * counter) combines the partials in block order and applies the seed.  The
 * partials and the ticket live in runtime-owned scratch (aux[0], aux[1]);
 * the last block resets the ticket, so no memset is needed between launches.
 */
#pragma once
#include "../cubits/accb_vec.cuh"
#include "../cubits/accb_warp.cuh"
#include "../cubits/accb_tma.cuh"

#ifndef ACCB_FOLD_SCALAR_UNROLL
#define ACCB_FOLD_SCALAR_UNROLL 4 /* scalar loads in flight per lane where vector loads do not apply (segments) */
#endif

namespace accb {

template <class T, class A = T>
struct Fold {
    typedef T elem;
    typedef A acc;
    typedef types<T> Out;
    static __device__ __forceinline__ A lift(T x) { return static_cast<A>(x); }
    static __device__ __forceinline__ T lower(A a) { return static_cast<T>(a); }
    static __device__ __forceinline__ void put(T r, T &o) { o = r; }
};

/* (have, value) pairs: a reduction without an identity element */
template <class A>
struct Opt {
    A v;
    int have;
};
template <class Fn>
struct OptCombine {
    typedef typename Fn::acc A;
    __device__ __forceinline__ Opt<A> operator()(Opt<A> a, Opt<A> b) const {
        Opt<A> r;
        r.have = a.have | b.have;
        r.v = (a.have && b.have) ? Fn::combine(a.v, b.v) : (a.have ? a.v : b.v);
        return r;
    }
};

template <class Fn, int N, int... I>
__device__ __forceinline__ void fold_get(const Env &env, long long i0, regs<N, typename Fn::In> &a,
                                         typename Fn::elem (&x)[N], std::integer_sequence<int, I...>) {
#pragma unroll
    for (int k = 0; k < N; ++k) x[k] = Fn::get(env, env.p.base + i0 + k, comp<I>(a)[k]...);
}

template <class Fn, int... O>
__device__ __forceinline__ void fold_put(const accb_kparams &p, long long j, typename Fn::elem r,
                                         std::integer_sequence<int, O...>) {
    regs<1, typename Fn::Out> b;
    Fn::put(r, comp<O>(b)[0]...);
    store_one(p.out, j, b);
}

template <class Fn>
__device__ __forceinline__ typename Fn::elem fold_seed(const accb_kparams &p) {
    typedef typename Fn::elem T;
    if (p.flags & ACCB_F_SEED_PTR) {
        /* the scalar block holds a device pointer to the seed (a carry produced
         * by earlier device work, e.g. the totals of lower-ranked shards) */
        const T *q = Env(p).scalar<const T *>(0);
        return *q;
    }
    return Env(p).scalar<T>(0);
}

/* foldSeg: hand segment `unit` (row * segments + segment) over to the second launch.  False when the list is
 * full: the caller then reduces the segment itself. */
__device__ __forceinline__ bool fold_defer(const accb_kparams &p, long long unit) {
    accb_deferred_segments *dl = static_cast<accb_deferred_segments *>(p.aux[2]);
    const unsigned idx = atomicAdd(&dl->count, 1u);
    if (idx >= ACCB_FOLD_DEFER_MAX) return false;
    dl->unit[idx] = unit;
    return true;
}

/* Accumulate elements [lo, lo+len) of the producer into `acc`, all threads of
 * a group of G threads (rank `g`) cooperating; vec_ok says lo and the slots
 * are vector aligned. */
template <class Fn, int U>
__device__ __forceinline__ void fold_range(const accb_kparams &p, const Env &env, long long lo, long long len,
                                           int g, int G, bool vec_ok, Opt<typename Fn::acc> &acc) {
    typedef typename Fn::In In;
    typedef typename Fn::elem T;
    typedef typename Fn::acc A;
    const auto iseq = std::make_integer_sequence<int, In::size>();
    const long long nvec = vec_ok ? len / V : 0;
    const long long v_lo = lo / V; /* lo is a multiple of V when vec_ok */
    const long long TRIP = (long long)G * U;
    const long long ntrip = nvec / TRIP;
    for (long long t = 0; t < ntrip; ++t) {
        const long long v0 = v_lo + t * TRIP + g;
        regs<V, In> a[U];
#pragma unroll
        for (int u = 0; u < U; ++u) load_all(p.in, v0 + (long long)u * G, a[u]);
        A part;
#pragma unroll
        for (int u = 0; u < U; ++u) {
            T x[V];
            fold_get<Fn>(env, (v0 + (long long)u * G) * V, a[u], x, iseq);
            A s = Fn::combine(Fn::combine(Fn::lift(x[0]), Fn::lift(x[1])),
                              Fn::combine(Fn::lift(x[2]), Fn::lift(x[3])));
            part = (u == 0) ? s : Fn::combine(part, s);
        }
        acc.v = acc.have ? Fn::combine(acc.v, part) : part;
        acc.have = 1;
    }
    for (long long v = v_lo + ntrip * TRIP + g; v < v_lo + nvec; v += G) {
        regs<V, In> a;
        T x[V];
        load_all(p.in, v, a);
        fold_get<Fn>(env, v * V, a, x, iseq);
        A s = Fn::combine(Fn::combine(Fn::lift(x[0]), Fn::lift(x[1])),
                          Fn::combine(Fn::lift(x[2]), Fn::lift(x[3])));
        acc.v = acc.have ? Fn::combine(acc.v, s) : s;
        acc.have = 1;
    }
    constexpr int kScalarUnroll = ACCB_FOLD_SCALAR_UNROLL;
#pragma unroll kScalarUnroll
    for (long long i = lo + nvec * V + g; i < lo + len; i += G) {
        regs<1, In> a;
        T x[1];
        load_one(p.in, i, a);
        fold_get<Fn>(env, i, a, x, iseq);
        A s = Fn::lift(x[0]);
        acc.v = acc.have ? Fn::combine(acc.v, s) : s;
        acc.have = 1;
    }
}

/* ------------------------------------------------------------------ foldAll */
template <class Fn, int CTA, int U>
__device__ __forceinline__ void fold_all_body(const accb_kparams &p) {
    typedef typename Fn::acc A;
    typedef Opt<A> O;
    __shared__ O s_red[CTA / 32];
    __shared__ int s_last;
    const Env env(p);
    const OptCombine<Fn> oc;
    const auto oseq = std::make_integer_sequence<int, Fn::Out::size>();
    const long long n = p.n;
    const bool vec_ok = (p.flags & ACCB_F_VEC) != 0;

    /* contiguous slab per block, boundaries on multiples of CTA*U*V */
    const long long quantum = (long long)CTA * U * V;
    const long long nq = (n + quantum - 1) / quantum;
    const long long q_per = (nq + gridDim.x - 1) / gridDim.x;
    long long lo = (long long)blockIdx.x * q_per * quantum;
    long long hi = lo + q_per * quantum;
    if (lo > n) lo = n;
    if (hi > n) hi = n;

    O acc;
    acc.have = 0;
    fold_range<Fn, U>(p, env, lo, hi - lo, threadIdx.x, CTA, vec_ok, acc);
    acc = block_reduce<CTA>(acc, oc, s_red);

    O *partial = static_cast<O *>(p.aux[0]);
    unsigned int *ticket = static_cast<unsigned int *>(p.aux[1]);
    if (threadIdx.x == 0) {
        partial[blockIdx.x] = acc;
        __threadfence();
        const unsigned int t = atomicAdd(ticket, 1u);
        s_last = (t == gridDim.x - 1);
    }
    __syncthreads();
    if (!s_last) return;

    /* last block: combine the partials in block order */
    __threadfence();
    O tot;
    tot.have = 0;
    for (unsigned int b = threadIdx.x; b < gridDim.x; b += CTA) {
        O x = ld_cg(partial + b);
        tot = oc(tot, x);
    }
    tot = block_reduce<CTA>(tot, oc, s_red);
    if (threadIdx.x == 0) {
        *ticket = 0u;
        if (p.flags & ACCB_F_CARRY) {
            /* this launch folds a later piece of a larger array: what the pieces before it came to stands on
             * the LEFT (the combiner need not commute) */
            const A c = Fn::lift(*static_cast<const typename Fn::elem *>(p.aux[2]));
            tot.v = tot.have ? Fn::combine(c, tot.v) : c;
            tot.have = 1;
        }
        if (p.flags & ACCB_F_HAS_SEED) {
            const A z = Fn::lift(fold_seed<Fn>(p));
            tot.v = tot.have ? Fn::combine(tot.v, z) : z;
            tot.have = 1;
        }
        if (tot.have) fold_put<Fn>(p, 0, Fn::lower(tot.v), oseq);
    }
}

/* ---------------------------------------- fold over inner dim and foldSeg */
/* Both reduce many independent ranges ("units": a row, or a segment of a row).
 * GROUP threads cooperate on one unit: the whole block (long ranges), a warp,
 * or an aligned sub-warp group of 16 / 8 / 4 lanes (short ranges, so that the
 * lanes of a warp still read one contiguous stretch of memory).  A group
 * takes KR units per trip so that short ranges still leave several loads in
 * flight per lane.  `range(w, lo, len, vec)` describes unit w. */
/* fold_range for a range that starts anywhere: the elements up to the first 16-byte boundary one by one, the rest
 * with 128-bit loads (`aligned`: the arrays themselves are 16-byte aligned and the range is worth the split) */
template <class Fn, int U>
__device__ __forceinline__ void fold_range_from_anywhere(const accb_kparams &p, const Env &env, long long lo, long long len,
                                                         int g, int G, bool aligned, Opt<typename Fn::acc> &acc) {
    if (aligned && len >= 2LL * G * V) {
        const long long head = (V - lo % V) % V;
        fold_range<Fn, U>(p, env, lo, head, g, G, false, acc);
        fold_range<Fn, U>(p, env, lo + head, len - head, g, G, true, acc);
    } else {
        fold_range<Fn, U>(p, env, lo, len, g, G, false, acc);
    }
}

template <class Fn, int CTA, int GROUP, int U, int KR, class Range>
__device__ __forceinline__ void fold_units(const accb_kparams &p, long long units, Range range, long long defer_above = 0,
                                           bool split_unaligned = false) {
    typedef typename Fn::acc A;
    typedef Opt<A> O;
    __shared__ O s_red[CTA / 32];
    __shared__ int s_deferred;
    const Env env(p);
    const OptCombine<Fn> oc;
    const auto oseq = std::make_integer_sequence<int, Fn::Out::size>();
    const bool seeded = (p.flags & ACCB_F_HAS_SEED) != 0;
    auto finish = [&](long long w, O acc) {
        if (seeded) {
            const A z = Fn::lift(fold_seed<Fn>(p));
            acc.v = acc.have ? Fn::combine(acc.v, z) : z;
            acc.have = 1;
        }
        if (acc.have) fold_put<Fn>(p, w, Fn::lower(acc.v), oseq);
    };

    if constexpr (GROUP == CTA) {
        for (long long w = blockIdx.x; w < units; w += gridDim.x) {
            long long lo, len;
            bool vec;
            range(w, lo, len, vec);
            if (defer_above > 0 && len > defer_above) { /* the same for the whole block */
                if (threadIdx.x == 0) s_deferred = fold_defer(p, w);
                __syncthreads();
                const int d = s_deferred;
                __syncthreads();
                if (d) continue;
            }
            O acc;
            acc.have = 0;
            if (vec || !split_unaligned)
                fold_range<Fn, U>(p, env, lo, len, threadIdx.x, CTA, vec, acc);
            else
                fold_range_from_anywhere<Fn, U>(p, env, lo, len, threadIdx.x, CTA, true, acc);
            acc = block_reduce<CTA>(acc, oc, s_red);
            if (threadIdx.x == 0) finish(w, acc);
        }
    } else {
        constexpr int PER = CTA / GROUP; /* units per block per sweep */
        const int g = threadIdx.x % GROUP;
        const long long sweep = (long long)gridDim.x * PER;
        /* the lanes of a group share their unit, so they leave the loops together */
        const unsigned gmask = GROUP == 32 ? FULL : (((1u << GROUP) - 1u) << ((threadIdx.x & 31) / GROUP * GROUP));
        for (long long w0 = (long long)blockIdx.x * PER + threadIdx.x / GROUP; w0 < units; w0 += sweep * KR) {
            O acc[KR];
            bool deferred[KR];
#pragma unroll
            for (int k = 0; k < KR; ++k) {
                acc[k].have = 0;
                deferred[k] = false;
                const long long w = w0 + k * sweep;
                if (w < units) { /* the same for all lanes of the group */
                    long long lo, len;
                    bool vec;
                    range(w, lo, len, vec);
                    if (defer_above > 0 && len > defer_above) {
                        const int d = g == 0 ? (int)fold_defer(p, w) : 0;
                        deferred[k] = __shfl_sync(gmask, d, (threadIdx.x & 31) / GROUP * GROUP) != 0;
                    }
                    if (deferred[k]) {
                    } else if (vec || !split_unaligned) {
                        fold_range<Fn, U>(p, env, lo, len, g, GROUP, vec, acc[k]);
                    } else {
                        fold_range_from_anywhere<Fn, U>(p, env, lo, len, g, GROUP, true, acc[k]);
                    }
                }
            }
#pragma unroll
            for (int k = 0; k < KR; ++k) {
                const long long w = w0 + k * sweep;
                if (w < units && !deferred[k]) {
#pragma unroll
                    for (int m = GROUP / 2; m > 0; m >>= 1) {
                        O o;
                        o.have = __shfl_xor_sync(gmask, acc[k].have, m);
                        constexpr int W = (sizeof(A) + 3) / 4;
                        unsigned wd[W] = {};
                        memcpy(wd, &acc[k].v, sizeof(A));
#pragma unroll
                        for (int q = 0; q < W; ++q) wd[q] = __shfl_xor_sync(gmask, wd[q], m);
                        memcpy(&o.v, wd, sizeof(A));
                        acc[k] = oc(acc[k], o);
                    }
                    if (g == 0) finish(w, acc[k]);
                }
            }
        }
    }
}

/* fold / fold1 over the innermost dimension: ip[0] = rows (outer size),
 * ip[1] = cols (innermost extent); unit = row. */
template <class Fn, int CTA, int GROUP, int U, int KR>
__device__ __forceinline__ void fold_dim_body(const accb_kparams &p) {
    const long long rows = p.ip[0], cols = p.ip[1];
    const bool vec_ok = (p.flags & ACCB_F_VEC) != 0 && (cols % V) == 0;
    fold_units<Fn, CTA, GROUP, U, KR>(p, rows, [&](long long w, long long &lo, long long &len, bool &vec) {
        lo = w * cols;
        len = cols;
        vec = vec_ok;
    });
}

/* Few, very long rows: a row is cut into ip[2] pieces of ip[3] elements (a
 * multiple of V; the last piece is shorter) so that all SMs get work.  One
 * block per (row, piece); the block that completes a row last (arrival counter
 * per row in aux[1], which it resets) combines the row's partials from aux[0]
 * in piece order and applies the seed -- the scheme of foldAll, per row. */
template <class Fn, int CTA, int U>
__device__ __forceinline__ void fold_split_body(const accb_kparams &p) {
    typedef typename Fn::acc A;
    typedef Opt<A> O;
    __shared__ O s_red[CTA / 32];
    __shared__ int s_last;
    const Env env(p);
    const OptCombine<Fn> oc;
    const auto oseq = std::make_integer_sequence<int, Fn::Out::size>();
    const long long rows = p.ip[0], cols = p.ip[1], pieces = p.ip[2], chunk = p.ip[3];
    const bool vec_ok = (p.flags & ACCB_F_VEC) != 0 && (cols % V) == 0;
    O *partial = static_cast<O *>(p.aux[0]);
    unsigned int *arrived = static_cast<unsigned int *>(p.aux[1]);
    for (long long w = blockIdx.x; w < rows * pieces; w += gridDim.x) {
        const long long r = w / pieces, pc = w - r * pieces;
        const long long lo = pc * chunk, len = min(chunk, cols - lo);
        O acc;
        acc.have = 0;
        fold_range<Fn, U>(p, env, r * cols + lo, len, threadIdx.x, CTA, vec_ok, acc);
        acc = block_reduce<CTA>(acc, oc, s_red);
        if (threadIdx.x == 0) {
            partial[w] = acc;
            __threadfence();
            s_last = atomicAdd(arrived + r, 1u) == (unsigned)pieces - 1u;
        }
        __syncthreads();
        if (s_last) { /* uniform over the block */
            __threadfence();
            O tot;
            tot.have = 0;
            for (long long b = threadIdx.x; b < pieces; b += CTA) tot = oc(tot, ld_cg(partial + r * pieces + b));
            tot = block_reduce<CTA>(tot, oc, s_red);
            if (threadIdx.x == 0) {
                arrived[r] = 0u;
                if (p.flags & ACCB_F_HAS_SEED) {
                    const A z = Fn::lift(fold_seed<Fn>(p));
                    tot.v = tot.have ? Fn::combine(tot.v, z) : z;
                    tot.have = 1;
                }
                if (tot.have) fold_put<Fn>(p, r, Fn::lower(tot.v), oseq);
            }
        }
        __syncthreads(); /* s_last and s_red are reused by the next unit */
    }
}

/* foldSeg / fold1Seg: unit = (row, segment).  aux[0] = Int32 offsets, length
 * nseg+1: the exclusive scan of the segment lengths (Execute.hs:320-324).
 * ip[0] = rows, ip[1] = cols (innermost extent of the source), ip[2] = nseg.
 * Segments start anywhere: one that is long enough is read with 128-bit loads from its first 16-byte
 * boundary on, the others element by element. */
template <class Fn, int CTA, int GROUP, int KR>
__device__ __forceinline__ void fold_seg_body(const accb_kparams &p) {
    const long long rows = p.ip[0], cols = p.ip[1], nseg = p.ip[2];
    const int *offs = static_cast<const int *>(p.aux[0]);
    /* once every block is running, the blocks of the second launch may take the places of those that finish */
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    fold_units<Fn, CTA, GROUP, 1, KR>(p, rows * nseg, [&](long long w, long long &lo, long long &len, bool &vec) {
        /* a 64-bit division per segment would cost more than a short segment's loads */
        long long r = 0, sgm = w;
        if (rows != 1) {
            if (rows * nseg <= 0xffffffffLL) {
                r = (unsigned)w / (unsigned)nseg;
                sgm = w - r * nseg;
            } else {
                r = w / nseg;
                sgm = w - r * nseg;
            }
        }
        const long long b = offs[sgm];
        lo = r * cols + b;
        len = offs[sgm + 1] - b;
        vec = false;
    }, p.ip[6], (p.flags & ACCB_F_VEC) != 0);
}

/* The second launch of a foldSeg: the segments that the first launch put on the list (longer than ip[6]
 * elements), each cut into pieces of ACCB_FOLD_DEFER_PIECE elements that the blocks take in turn -- the scheme
 * of fold_split, per listed segment: partial results in aux[0] (one per piece, in list order), the block that
 * completes a segment last combines its pieces in order and applies the seed.  The last block to leave clears
 * the list.  With an empty list (the usual case) a block reads one word and leaves. */
#ifndef ACCB_FOLD_DEFER_PIECE
#define ACCB_FOLD_DEFER_PIECE (1 << 16)
#endif
template <class Fn, int CTA, int U>
__device__ __forceinline__ void fold_deferred_body(const accb_kparams &p) {
    typedef typename Fn::acc A;
    typedef Opt<A> O;
    __shared__ O s_red[CTA / 32];
    __shared__ int s_last;
    __shared__ long long s_first[ACCB_FOLD_DEFER_MAX + 1]; /* first piece of every listed segment */
    const Env env(p);
    const OptCombine<Fn> oc;
    const auto oseq = std::make_integer_sequence<int, Fn::Out::size>();
    const long long cols = p.ip[1], nseg = p.ip[2];
    constexpr long long PIECE = ACCB_FOLD_DEFER_PIECE;
    const int *offs = static_cast<const int *>(p.aux[0]);
    O *partial = static_cast<O *>(p.aux[1]);
    accb_deferred_segments *dl = static_cast<accb_deferred_segments *>(p.aux[2]);
    const bool vec_ok = (p.flags & ACCB_F_VEC) != 0;
    /* the host launches this kernel so that its blocks may be scheduled while the first launch drains: wait
     * until that launch is complete and its list visible (no effect on an ordinary launch) */
    asm volatile("griddepcontrol.wait;" ::: "memory");
    const int listed = (int)min(*static_cast<volatile unsigned int *>(&dl->count), (unsigned)ACCB_FOLD_DEFER_MAX);
    if (listed == 0) return; /* nothing was deferred: the list is clear already */
    for (int g = threadIdx.x; g < listed; g += CTA) {
        const long long sgm = dl->unit[g] % nseg;
        s_first[g + 1] = ((long long)offs[sgm + 1] - offs[sgm] + PIECE - 1) / PIECE;
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        s_first[0] = 0;
        for (int g = 0; g < listed; ++g) s_first[g + 1] += s_first[g];
    }
    __syncthreads();
    const long long pieces = s_first[listed];
    for (long long it = blockIdx.x; it < pieces; it += gridDim.x) {
        int g = 0, h = listed; /* s_first[g] <= it < s_first[h] */
        while (h - g > 1) {
            const int m = (g + h) >> 1;
            if (s_first[m] <= it)
                g = m;
            else
                h = m;
        }
        const long long w = dl->unit[g], r = w / nseg, sgm = w - r * nseg;
        const long long pc = it - s_first[g], np = s_first[g + 1] - s_first[g];
        const long long b = offs[sgm], e = offs[sgm + 1];
        const long long lo = r * cols + b + pc * PIECE, len = min(PIECE, e - b - pc * PIECE);
        O acc;
        acc.have = 0;
        fold_range_from_anywhere<Fn, U>(p, env, lo, len, threadIdx.x, CTA, vec_ok, acc);
        acc = block_reduce<CTA>(acc, oc, s_red);
        if (threadIdx.x == 0) {
            partial[it] = acc;
            __threadfence();
            s_last = atomicAdd(&dl->arrived[g], 1u) == (unsigned)np - 1u;
        }
        __syncthreads();
        if (s_last) { /* uniform over the block */
            __threadfence();
            O tot;
            tot.have = 0;
            for (long long q = threadIdx.x; q < np; q += CTA) tot = oc(tot, ld_cg(partial + s_first[g] + q));
            tot = block_reduce<CTA>(tot, oc, s_red);
            if (threadIdx.x == 0) {
                dl->arrived[g] = 0u;
                if (p.flags & ACCB_F_HAS_SEED) {
                    const A z = Fn::lift(fold_seed<Fn>(p));
                    tot.v = tot.have ? Fn::combine(tot.v, z) : z;
                    tot.have = 1;
                }
                if (tot.have) fold_put<Fn>(p, w, Fn::lower(tot.v), oseq);
            }
        }
        __syncthreads(); /* s_last and s_red are reused by the next piece */
    }
    if (threadIdx.x == 0) {
        __threadfence();
        if (atomicAdd(&dl->finished, 1u) == gridDim.x - 1u) { /* every block has read the list */
            dl->finished = 0u;
            dl->count = 0u;
        }
    }
}

}  // namespace accb

#include "fold_staged.cuh" /* short rows and segments */

#define ACCB_FOLD_CTA 256
#define ACCB_FOLD_U 4

/* Entry points named after the reference's kernels (Reduction.hs:111,229,430);
 * the seeded and seedless forms share a kernel (flag ACCB_F_HAS_SEED). */
#define ACCB_INSTANTIATE_FOLD_ALL(Fn)                                                   \
    ACCB_META12(2, ACCB_FOLD_CTA, sizeof(accb::Opt<Fn::acc>), 0, ACCB_FOLD_U, 0, 0, 0, 0, 0, 0, Fn::In::size) \
    extern "C" __global__ void __launch_bounds__(ACCB_FOLD_CTA)                         \
        foldAll(const __grid_constant__ accb_kparams p) {                               \
        accb::fold_all_body<Fn, ACCB_FOLD_CTA, ACCB_FOLD_U>(p);                         \
    }

#define ACCB_FOLD_DIM_ENTRY(Fn, name, group, u, kr)                                      \
    extern "C" __global__ void __launch_bounds__(ACCB_FOLD_CTA)                         \
        name(const __grid_constant__ accb_kparams p) {                                  \
        accb::fold_dim_body<Fn, ACCB_FOLD_CTA, group, u, kr>(p);                        \
    }

#define ACCB_FOLD_STAGED_ENTRY(Fn, name, seg)                                           \
    extern "C" __global__ void __launch_bounds__(ACCB_FOLD_STAGE_CTA, 12)               \
        name(const __grid_constant__ accb_kparams p) {                                  \
        accb::fold_staged_or_nothing<Fn, seg>(p);                                       \
    }

/* One entry per group size; the host picks by row length.
 * Metadata: {.., bytes of a partial, elements per window of the staged form, U, block size of the
 * staged form, its shared memory} */
#define ACCB_INSTANTIATE_FOLD_DIM(Fn)                                                   \
    ACCB_META12(3, ACCB_FOLD_CTA, sizeof(accb::Opt<Fn::acc>),                           \
                accb::fold_stage_window<Fn::In>::value, ACCB_FOLD_U, ACCB_FOLD_STAGE_CTA, \
                (accb::fold_stage_smem<Fn>()), 0, 0, 0, 0, Fn::In::size)                \
    ACCB_FOLD_STAGED_ENTRY(Fn, fold_staged, false)                                      \
    ACCB_FOLD_DIM_ENTRY(Fn, fold, ACCB_FOLD_CTA, ACCB_FOLD_U, 1)                        \
    ACCB_FOLD_DIM_ENTRY(Fn, fold_warp, 32, 4, 1)                                        \
    ACCB_FOLD_DIM_ENTRY(Fn, fold_g16, 16, 4, 1)                                         \
    ACCB_FOLD_DIM_ENTRY(Fn, fold_g8, 8, 4, 2)                                           \
    ACCB_FOLD_DIM_ENTRY(Fn, fold_g4, 4, 4, 4)                                           \
    extern "C" __global__ void __launch_bounds__(ACCB_FOLD_CTA)                         \
        fold_split(const __grid_constant__ accb_kparams p) {                            \
        accb::fold_split_body<Fn, ACCB_FOLD_CTA, ACCB_FOLD_U>(p);                       \
    }

#define ACCB_FOLD_SEG_ENTRY(Fn, name, group, kr)                                        \
    extern "C" __global__ void __launch_bounds__(ACCB_FOLD_CTA)                         \
        name(const __grid_constant__ accb_kparams p) {                                  \
        accb::fold_seg_body<Fn, ACCB_FOLD_CTA, group, kr>(p);                           \
    }

/* `foldSeg` is the reference's warp-per-segment form (Reduction.hs:430); the
 * others serve shorter and longer segments; foldSeg_deferred is the second launch for the segments the first one
 * handed over */
#define ACCB_INSTANTIATE_FOLD_SEG(Fn)                                                   \
    ACCB_META12(4, ACCB_FOLD_CTA, sizeof(accb::Opt<Fn::acc>),                           \
                accb::fold_stage_window<Fn::In>::value, 1, ACCB_FOLD_STAGE_CTA,         \
                (accb::fold_stage_smem<Fn>()), ACCB_FOLD_DEFER_PIECE, 0, 0, 0, Fn::In::size) \
    ACCB_FOLD_STAGED_ENTRY(Fn, foldSeg_staged, true)                                    \
    ACCB_FOLD_SEG_ENTRY(Fn, foldSeg, 32, 1)                                             \
    ACCB_FOLD_SEG_ENTRY(Fn, foldSeg_g16, 16, 2)                                         \
    ACCB_FOLD_SEG_ENTRY(Fn, foldSeg_g8, 8, 2)                                           \
    ACCB_FOLD_SEG_ENTRY(Fn, foldSeg_g4, 4, 4)                                           \
    ACCB_FOLD_SEG_ENTRY(Fn, foldSeg_block, ACCB_FOLD_CTA, 1)                            \
    extern "C" __global__ void __launch_bounds__(ACCB_FOLD_CTA)                         \
        foldSeg_deferred(const __grid_constant__ accb_kparams p) {                      \
        accb::fold_deferred_body<Fn, ACCB_FOLD_CTA, ACCB_FOLD_U>(p);                    \
    }
