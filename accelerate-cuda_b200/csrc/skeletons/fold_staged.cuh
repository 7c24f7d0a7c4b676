/*
 * fold_staged.cuh -- fold over the innermost dimension and foldSeg for SHORT
 * rows and segments (a few elements to a few dozen).
 *
 * The reference gives a row a whole block (mkFoldDim,
 * Data/Array/Accelerate/CUDA/CodeGen/Reduction.hs:221-367) and a segment a
 * whole warp (mkFoldSeg', :421-574; its own comment at :391-393 notes that the
 * warp idles on short segments).  Groups of 4 to 32 lanes per unit (fold.cuh)
 * keep memory accesses contiguous but spend more instructions on bookkeeping
 * than on data once a unit is shorter than a few vectors.
 *
 * Here a block owns a run of S consecutive units.  Their elements are one
 * contiguous stretch of the source, which ONE bulk copy per input component
 * brings into shared memory (TMA, completion on an mbarrier) while the threads
 * fetch the bounds of their own units; then every thread reduces whole units
 * out of shared memory.  A thread starts (lane * len / 32) elements into its
 * unit and wraps around, so that neighbours with equal lengths read different
 * banks (folds assume a commutative combiner throughout).  Outliers longer than
 * ACCB_FOLD_STAGE_COOP elements are taken by the whole warp, lane-strided.  The host sizes S so
 * that a run normally fits the window; a run that does not (a few very long
 * segments among the short ones) is read from global memory directly by the
 * same code.
 *
 *   ip[0] rows, ip[1] cols (elements per row of the source), ip[2] units per
 *   row, ip[3] uniform unit length (fold over rows: the host passes the matrix
 *   as ONE row of rows x cols elements) or, with SEG, aux[0] = Int32 offsets of
 *   length units + 1; ip[4] = S; ip[5] = lanes per unit (1, or a power of two up to 32 for units of a few
 *   hundred elements: then consecutive lanes read consecutive elements of their unit and combine by
 *   shuffles).  aux[1] = error word of the bounded wait.  With SEG and ip[6] > 0, segments longer than ip[6]
 *   elements are handed over to the second launch (aux[2], see fold_defer).
 * Segment offsets are Int32 (Execute.hs:320-324), so positions inside a row
 * are held in 32-bit registers.
 */
#pragma once
#include "../cubits/accb_tma.cuh"

#ifndef ACCB_FOLD_STAGE_SPIN_LIMIT
#define ACCB_FOLD_STAGE_SPIN_LIMIT (1 << 16)
#endif
#ifndef ACCB_FOLD_STAGE_CTA
#define ACCB_FOLD_STAGE_CTA 128
#endif
#ifndef ACCB_FOLD_STAGE_COOP
#define ACCB_FOLD_STAGE_COOP 512 /* where a thread owns whole units, longer ones are reduced by the whole warp */
#endif
#ifndef ACCB_FOLD_STAGE_BYTES
#define ACCB_FOLD_STAGE_BYTES 16384 /* window size over all input components */
#endif

namespace accb {

/* elements per window */
template <class L>
struct fold_stage_window {
    static constexpr int bpe = L::size == 0 ? 0 : smem_offset<L, L::size, 128>::value / 128;
    static constexpr int value = bpe == 0 ? 0 : (ACCB_FOLD_STAGE_BYTES / bpe) / 128 * 128;
};

template <class Fn, int WIN, int... I>
__device__ __forceinline__ typename Fn::elem stage_get(const Env &env, const unsigned char *s, int j, long long i,
                                                       std::integer_sequence<int, I...>) {
    typedef typename Fn::In In;
    return Fn::get(env, env.p.base + i,
                   reinterpret_cast<const typename type_at<I, In>::type *>(s + smem_offset<In, I, WIN>::value)[j]...);
}
template <class Fn, int... I>
__device__ __forceinline__ typename Fn::elem global_get(const accb_kparams &p, const Env &env, long long i,
                                                        std::integer_sequence<int, I...>) {
    typedef typename Fn::In In;
    return Fn::get(env, p.base + i, static_cast<const typename type_at<I, In>::type *>(p.in[I])[i]...);
}

/* bulk copy of `len` elements of every component starting at element `g` (a multiple of 16); the
 * last len*size % 16 bytes of a component are left to stage_copy_tail */
template <class L, int WIN, int... I>
__device__ __forceinline__ void stage_issue(unsigned char *s, const void *const *slots, long long g, int len,
                                            unsigned long long *bar, std::integer_sequence<int, I...>) {
    const unsigned total = (unsigned)(((len * (int)sizeof(typename type_at<I, L>::type)) & ~15) + ... + 0);
    mbar_expect_tx(bar, total);
    ((((len * (int)sizeof(typename type_at<I, L>::type)) & ~15) != 0
          ? bulk_g2s(s + smem_offset<L, I, WIN>::value, static_cast<const typename type_at<I, L>::type *>(slots[I]) + g,
                     (unsigned)((len * (int)sizeof(typename type_at<I, L>::type)) & ~15), bar)
          : (void)0),
     ...);
}
template <class T>
__device__ __forceinline__ void stage_copy_tail_one(T *dst, const T *src, int len, int tid) {
    const int done = ((len * (int)sizeof(T)) & ~15) / (int)sizeof(T);
    if (done + tid < len) dst[done + tid] = src[done + tid]; /* fewer than 16 elements */
}
template <class L, int WIN, int... I>
__device__ __forceinline__ void stage_copy_tail(unsigned char *s, const void *const *slots, long long g, int len,
                                                int tid, std::integer_sequence<int, I...>) {
    (stage_copy_tail_one(reinterpret_cast<typename type_at<I, L>::type *>(s + smem_offset<L, I, WIN>::value),
                         static_cast<const typename type_at<I, L>::type *>(slots[I]) + g, len, tid),
     ...);
}

/* any block size that is a multiple of 32 (the host launches ACCB_FOLD_STAGE_CTA threads) */
template <class Fn, bool SEG>
__device__ __forceinline__ void fold_staged_body(const accb_kparams &p) {
    typedef typename Fn::In In;
    typedef typename Fn::acc A;
    typedef Opt<A> O;
    constexpr int WIN = fold_stage_window<In>::value;
    extern __shared__ __align__(128) unsigned char s_raw[];
    __shared__ __align__(8) unsigned long long s_bar;
    const Env env(p);
    const OptCombine<Fn> oc;
    const auto iseq = std::make_integer_sequence<int, In::size>();
    const auto oseq = std::make_integer_sequence<int, Fn::Out::size>();
    const long long cols = p.ip[1], nseg = p.ip[2];
    const int ulen = (int)p.ip[3], S = (int)p.ip[4];
    const int *offs = static_cast<const int *>(p.aux[0]);
    unsigned int *err = static_cast<unsigned int *>(p.aux[1]);
    const bool seeded = (p.flags & ACCB_F_HAS_SEED) != 0;
    const int defer_above = SEG ? (int)min(p.ip[6], 0x7fffffffLL) : 0; /* 0: never */
    if constexpr (SEG) /* once every block is running, the second launch's blocks may take the places of those that finish */
        asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    const int lane = lane_id(), warp = warp_id();

    /* the block's run of units, of row r */
    const long long runs = (nseg + S - 1) / S;
    const long long r = blockIdx.x / runs;
    const long long s_lo = (blockIdx.x - r * runs) * S;
    const int cnt = (int)min((long long)S, nseg - s_lo);
    const long long row0 = r * cols;
    /* Positions are relative to `org`: the row start for segments (Int32 offsets); for uniform
     * units the start of the run, so that they stay small however long the matrix is. */
    long long org;
    int d0, d1;
    if constexpr (SEG) {
        org = row0;
        d0 = offs[s_lo];
        d1 = offs[s_lo + cnt];
    } else {
        org = row0 + s_lo * ulen;
        d0 = 0;
        d1 = cnt * ulen;
    }
    /* the window starts at the 16-element boundary below the run (16-byte aligned for every
     * component size; the host checked that row starts are) */
    const int mis = (int)((org + d0) & 15);
    const int a0 = d0 - mis;
    /* elements to stage: whole 16-byte units, never beyond the end of the row, and as much of the run as the
     * window holds (what does not fit -- a run with a few long segments -- is read from global memory) */
    const long long row_left = row0 + cols - (org + a0);
    const int wlen = (int)min(min((long long)(d1 - a0 + 15) & ~15LL, (long long)WIN), row_left);
    const int w1 = a0 + wlen; /* positions in [a0, w1) are in shared memory */

    if (threadIdx.x == 0) {
        mbar_init(&s_bar, 1);
        fence_mbar_init();
        stage_issue<In, WIN>(s_raw, p.in, org + a0, wlen, &s_bar, iseq);
    }
    stage_copy_tail<In, WIN>(s_raw, p.in, org + a0, wlen, threadIdx.x, iseq);

    auto add = [&](O &acc, typename Fn::elem x) {
        const A s = Fn::lift(x);
        acc.v = acc.have ? Fn::combine(acc.v, s) : s;
        acc.have = 1;
    };
    auto at = [&](int i) {
        return (i >= a0 && i < w1) ? stage_get<Fn, WIN>(env, s_raw, i - a0, org + i, iseq)
                                   : global_get<Fn>(p, env, org + i, iseq);
    };
    /* G lanes share a unit (ip[5]: 1 for short units, a power of two up to 32 for longer ones): lane g of the
     * group takes elements g, g + G, ... -- consecutive lanes, consecutive words -- and the group's partial
     * results are combined by shuffles.  With G = 1 a thread owns whole units and rotates its start. */
    const int G = max(1, (int)p.ip[5]);
    const int upw = 32 / G, g = lane % G, slot = lane / G; /* units per warp and pass; place in the group; group */
    int b = 0, e = 0;
    auto bounds = [&](int k) { /* of unit k of the run; (0, 0) beyond it */
        b = e = 0;
        if (k < cnt) {
            if constexpr (SEG) {
                b = offs[s_lo + k];
                e = offs[s_lo + k + 1];
            } else {
                b = k * ulen;
                e = b + ulen;
            }
        }
    };
    bounds(warp * upw + slot); /* fetched while the copy is in flight */
    __syncthreads();           /* barrier initialised, tail elements written */
    {
        int tries = 0;
        while (!mbar_try_wait(&s_bar, 0)) {
            if (++tries > ACCB_FOLD_STAGE_SPIN_LIMIT) { /* bounded: flag the result invalid and go on */
                atomicExch(err, 1u);
                break;
            }
        }
    }
    const int per_pass = (blockDim.x / 32) * upw;
    for (int k0 = warp * upw; k0 < cnt; k0 += per_pass) {
        const int k = k0 + slot;
        const bool valid = k < cnt;
        if (k0 != warp * upw) bounds(k);
        const int len = e - b;
        O acc;
        acc.have = 0;
        /* a segment far longer than the rest goes to the second launch (its owner puts it on the list; all lanes that
         * share it learn the outcome: a full list leaves it here) */
        bool deferred = false;
        if constexpr (SEG) {
            const bool far = defer_above > 0 && valid && len > defer_above;
            const int d = (far && g == 0) ? (int)fold_defer(p, r * nseg + s_lo + k) : 0;
            deferred = __shfl_sync(FULL, d, lane - g) != 0;
        }
        if (G == 1) {
            const bool coop = len > ACCB_FOLD_STAGE_COOP && !deferred;
            if (valid && !coop && !deferred && len > 0) {
                /* one loop of len trips for every lane (two loops, before and after the wrap, would
                 * have different trip counts per lane and run one after the other) */
                int i = b + ((lane * len) >> 5);
                if (b >= a0 && e <= w1) {
#pragma unroll 4
                    for (int j = 0; j < len; ++j) {
                        add(acc, stage_get<Fn, WIN>(env, s_raw, i - a0, org + i, iseq));
                        if (++i == e) i = b;
                    }
                } else {
                    for (int j = 0; j < len; ++j) {
                        add(acc, at(i));
                        if (++i == e) i = b;
                    }
                }
            }
            unsigned m = __ballot_sync(FULL, valid && coop);
            while (m) { /* outliers: the whole warp, lane-strided */
                const int src = __ffs(m) - 1;
                m &= m - 1;
                const int bb = __shfl_sync(FULL, b, src), ee = __shfl_sync(FULL, e, src);
                O part;
                part.have = 0;
#pragma unroll 4
                for (int i = bb + lane; i < ee; i += 32) add(part, at(i));
                part = warp_reduce_xor(part, oc);
                if (lane == src) acc = part;
            }
        } else {
            /* (units whose length is a multiple of 32 G put the groups of a warp on the same banks; walking
             * them in rotated chunks of 32 elements cost more instructions than the conflicts do) */
            if (deferred) {
            } else if (valid && b >= a0 && e <= w1) {
#pragma unroll 4
                for (int i = b + g; i < e; i += G) add(acc, stage_get<Fn, WIN>(env, s_raw, i - a0, org + i, iseq));
            } else if (valid) {
                for (int i = b + g; i < e; i += G) add(acc, at(i));
            }
            for (int m = G >> 1; m > 0; m >>= 1) acc = oc(acc, shfl_xor(acc, m)); /* stays inside the aligned group */
        }
        if (valid && g == 0 && !deferred) {
            if (seeded) {
                const A z = Fn::lift(fold_seed<Fn>(p));
                acc.v = acc.have ? Fn::combine(acc.v, z) : z;
                acc.have = 1;
            }
            if (acc.have) fold_put<Fn>(p, r * nseg + s_lo + k, Fn::lower(acc.v), oseq);
        }
    }
}

template <class Fn, bool SEG>
__device__ __forceinline__ void fold_staged_or_nothing(const accb_kparams &p) {
    if constexpr (fold_stage_window<typename Fn::In>::value > 0) fold_staged_body<Fn, SEG>(p);
}
/* dynamic shared memory of the staged form; 0 when the fold has no array input */
template <class Fn>
__host__ __device__ constexpr int fold_stage_smem() {
    typedef typename Fn::In In;
    if constexpr (fold_stage_window<In>::value > 0)
        return smem_offset<In, In::size, fold_stage_window<In>::value>::value;
    else
        return 0;
}

}  // namespace accb
