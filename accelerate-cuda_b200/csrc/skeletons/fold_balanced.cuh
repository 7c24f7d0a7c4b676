/*
 * fold_balanced.cuh -- foldSeg / fold1Seg with the work divided by ELEMENTS,
 * not by segments.
 *
 * The reference gives every segment one warp (mkFoldSeg',
 * Data/Array/Accelerate/CUDA/CodeGen/Reduction.hs:421-574): lanes idle on short
 * segments (its own note at :391-393) and one long segment keeps a single warp
 * busy while the rest of the GPU waits.  The staged form (fold_staged.cuh)
 * gives a thread whole segments, so a warp takes as long as its longest one.
 * Here neither the length of a segment nor the spread of the lengths matters:
 *
 *   - the source row is cut into tiles of T = CTA x V consecutive elements, one
 *     per block, whatever the segments are; thread t of a tile owns the V
 *     consecutive elements starting at t x V;
 *   - every thread's V elements are brought into shared memory by one bulk copy
 *     per input component (cp.async.bulk, completion on an mbarrier), into rows
 *     that are 16 bytes longer than their data, so that the threads' 128-bit
 *     reads of their own rows fall into different banks;
 *   - while the copies are in flight the block finds the segment that contains
 *     its first element by a CTA-ary search over the offsets (four rounds for
 *     2^24 segments) and stages the offsets of the segments that follow;
 *   - a thread walks its elements in order, writes every segment that starts
 *     and ends inside its chunk, and is left with at most two partial results:
 *     of the segment that was open when its chunk began (head) and of the one
 *     still open where it ends (tail);
 *   - a segmented scan over the threads' tails (shuffles, then four warp
 *     totals) gives every thread what precedes its chunk inside the tile; the
 *     ONE thread in which the tile's first segment ends may also need what
 *     precedes the tile;
 *   - across tiles: a tile that contains a segment boundary publishes its open
 *     tail as a finished prefix at once, without looking at anybody (for short
 *     segments that is every tile, so no chain of waits forms); a tile that
 *     lies inside one long segment publishes its sum as an aggregate, looks
 *     back over its predecessors' records as the scans do (accb_status.cuh) and
 *     then publishes the prefix.  The tile in which a long segment ENDS writes
 *     its result.  A segment of any length is therefore reduced by as many
 *     blocks as it has tiles.
 *
 * Value order is preserved (only associativity is needed by this form).
 * Empty segments receive the seed from the thread that finishes the segment
 * before them (leading ones from the thread that owns the first element).
 *
 *   ip[0] rows, ip[1] cols, ip[2] segments, ip[3] epoch of the status records,
 *   ip[4] tiles per row; aux[0] Int32 offsets (segments + 1), aux[1] error word
 *   of the bounded waits, aux[2] status records (one per tile and row).
 * Requires 16-byte aligned arrays and row starts (the host checks).
 */
#pragma once
#include "../cubits/accb_status.cuh"

#ifndef ACCB_FOLD_BAL_CTA
#define ACCB_FOLD_BAL_CTA 128
#endif
#ifndef ACCB_FOLD_BAL_BYTES
#define ACCB_FOLD_BAL_BYTES 16384 /* data per tile over all input components */
#endif
#ifndef ACCB_FOLD_BAL_OFFS
#define ACCB_FOLD_BAL_OFFS 1023 /* segments whose offsets a tile's window holds; later ones read theirs from global memory */
#endif
#ifndef ACCB_FOLD_BAL_SPIN_LIMIT
#define ACCB_FOLD_BAL_SPIN_LIMIT (1 << 20)
#endif
#ifndef ACCB_FOLD_BAL_MINB
#define ACCB_FOLD_BAL_MINB 5
#endif

namespace accb {

enum : unsigned { ST_PREFIX_NONE = 3u }; /* a finished prefix with nothing in it: no segment is open at the tile's end */

template <class L>
struct fold_bal_shape {
    static constexpr int bpe = L::size == 0 ? 0 : smem_offset<L, L::size, 128>::value / 128;
    static constexpr int raw = bpe == 0 ? 0 : ACCB_FOLD_BAL_BYTES / bpe / ACCB_FOLD_BAL_CTA / 16 * 16;
    static constexpr int V = bpe == 0 ? 0 : (raw < 16 ? 16 : raw); /* elements per thread: a multiple of 16 */
    static constexpr int T = V * ACCB_FOLD_BAL_CTA;
};
/* bytes from one thread's row of component I to the next thread's */
template <class L, int I>
struct fold_bal_pitch {
    static constexpr int value = fold_bal_shape<L>::V * (int)sizeof(typename type_at<I, L>::type) + 16;
};
template <class L, int I>
struct fold_bal_offset {
    static constexpr int value = fold_bal_offset<L, I - 1>::value + ACCB_FOLD_BAL_CTA * fold_bal_pitch<L, I - 1>::value;
};
template <class L>
struct fold_bal_offset<L, 0> {
    static constexpr int value = 0;
};
template <class A>
constexpr bool fold_bal_record_ok() {
    return sizeof(A) <= 4 || sizeof(A) == 8 || (sizeof(A) % 4 == 0 && sizeof(A) <= 32);
}
template <class Fn>
__host__ __device__ constexpr int fold_bal_tile() {
    typedef typename Fn::In In;
    if constexpr (In::size > 0 && fold_bal_record_ok<typename Fn::acc>())
        return fold_bal_shape<In>::T;
    else
        return 0;
}
template <class Fn>
__host__ __device__ constexpr int fold_bal_smem() {
    typedef typename Fn::In In;
    if constexpr (In::size > 0)
        return 2 * fold_bal_offset<In, In::size>::value + 2 * (ACCB_FOLD_BAL_OFFS + 1) * 4;
    else
        return 0;
}
template <class Fn>
__host__ __device__ constexpr int fold_bal_record() {
    if constexpr (fold_bal_record_ok<typename Fn::acc>())
        return TileStatus<typename Fn::acc>::kBytes;
    else
        return 0;
}

/* thread t's copies of a full tile */
template <class L, int... I>
__device__ __forceinline__ void bal_issue(unsigned char *s, const void *const *slots, long long g, int t,
                                          unsigned long long *bar, std::integer_sequence<int, I...>) {
    constexpr int V = fold_bal_shape<L>::V;
    constexpr unsigned total = (unsigned)((V * (int)sizeof(typename type_at<I, L>::type)) + ... + 0);
    mbar_expect_tx(bar, total);
    (bulk_g2s(s + fold_bal_offset<L, I>::value + t * fold_bal_pitch<L, I>::value,
              static_cast<const typename type_at<I, L>::type *>(slots[I]) + g + (long long)t * V,
              (unsigned)(V * (int)sizeof(typename type_at<I, L>::type)), bar),
     ...);
}
/* a ragged tile (the last of a row): plain loads, element e of the tile to its place in the padded rows */
template <class L, int I>
__device__ __forceinline__ void bal_fill_one(unsigned char *s, const void *const *slots, long long g, int valid, int tid) {
    typedef typename type_at<I, L>::type T;
    constexpr int V = fold_bal_shape<L>::V;
    const T *src = static_cast<const T *>(slots[I]) + g;
    for (int e = tid; e < valid; e += ACCB_FOLD_BAL_CTA)
        *reinterpret_cast<T *>(s + fold_bal_offset<L, I>::value + (e / V) * fold_bal_pitch<L, I>::value + (e % V) * (int)sizeof(T)) =
            src[e];
}
template <class L, int... I>
__device__ __forceinline__ void bal_fill(unsigned char *s, const void *const *slots, long long g, int valid, int tid,
                                         std::integer_sequence<int, I...>) {
    (bal_fill_one<L, I>(s, slots, g, valid, tid), ...);
}

/* four consecutive elements of one component out of a thread's row, by the widest load their size allows */
template <class T>
__device__ __forceinline__ void bal_load4(const unsigned char *row, int j, T (&v)[4]) {
    const unsigned char *src = row + j * (int)sizeof(T);
    if constexpr (sizeof(T) * 4 == 16) {
        const uint4 q = *reinterpret_cast<const uint4 *>(src);
        memcpy(v, &q, 16);
    } else if constexpr (sizeof(T) * 4 == 32) {
        const uint4 q0 = *reinterpret_cast<const uint4 *>(src), q1 = *reinterpret_cast<const uint4 *>(src + 16);
        memcpy(v, &q0, 16);
        memcpy(reinterpret_cast<unsigned char *>(v) + 16, &q1, 16);
    } else if constexpr (sizeof(T) * 4 == 8) {
        const uint2 q = *reinterpret_cast<const uint2 *>(src);
        memcpy(v, &q, 8);
    } else if constexpr (sizeof(T) * 4 == 4) {
        const unsigned q = *reinterpret_cast<const unsigned *>(src);
        memcpy(v, &q, 4);
    } else {
#pragma unroll
        for (int u = 0; u < 4; ++u) v[u] = reinterpret_cast<const T *>(src)[u];
    }
}
template <class Fn, int... I>
__device__ __forceinline__ void bal_get4(const Env &env, const unsigned char *s, int t, int j, long long i0,
                                         typename Fn::elem (&x)[4], std::integer_sequence<int, I...>) {
    typedef typename Fn::In In;
    regs<4, In> a;
    (bal_load4(s + fold_bal_offset<In, I>::value + t * fold_bal_pitch<In, I>::value, j, comp<I>(a)), ...);
#pragma unroll
    for (int u = 0; u < 4; ++u) x[u] = Fn::get(env, env.p.base + i0 + u, comp<I>(a)[u]...);
}

template <class Fn>
__device__ __forceinline__ void fold_balanced_body(const accb_kparams &p) {
    typedef typename Fn::In In;
    typedef typename Fn::acc A;
    typedef Opt<A> O;
    constexpr int CTA = ACCB_FOLD_BAL_CTA;
    constexpr int V = fold_bal_shape<In>::V;
    constexpr int T = fold_bal_shape<In>::T;
    constexpr int NOFF = ACCB_FOLD_BAL_OFFS; /* a window holds the offsets of NOFF segments: NOFF + 1 values */
    constexpr int NPRE = (NOFF + CTA) / CTA; /* values of the next window a thread fetches ahead */
    constexpr int WARPS = CTA / 32;
    constexpr int BEYOND = T + 1; /* "after the end of the tile" in tile-relative positions */
    constexpr int DATA = fold_bal_offset<In, In::size>::value;
    extern __shared__ __align__(128) unsigned char s_raw[];
    __shared__ __align__(8) unsigned long long s_bar[2];
    __shared__ O s_wv[WARPS];
    __shared__ int s_wf[WARPS];
    __shared__ O s_first; /* the block's first segment up to its end, when it began before the block */
    __shared__ long long s_first_seg;
    __shared__ int s_have_first;
    int *s_off = reinterpret_cast<int *>(s_raw + 2 * DATA);

    const Env env(p);
    const OptCombine<Fn> oc;
    const auto iseq = std::make_integer_sequence<int, In::size>();
    const auto oseq = std::make_integer_sequence<int, Fn::Out::size>();
    const long long cols = p.ip[1], nseg = p.ip[2], tpr = p.ip[4], K = p.ip[5];
    const unsigned epoch = (unsigned)p.ip[3];
    const int *offs = static_cast<const int *>(p.aux[0]);
    unsigned int *err = static_cast<unsigned int *>(p.aux[1]);
    const TileStatus<A> status(p.aux[2]);
    const bool seeded = (p.flags & ACCB_F_HAS_SEED) != 0;
    const int tid = threadIdx.x, lane = lane_id(), warp = warp_id();

    const long long spans = (tpr + K - 1) / K; /* blocks per row */
    const long long blk = blockIdx.x;
    const long long r = blk / spans, sp = blk - r * spans;
    const long long t_first = sp * K;
    const int kt = (int)min(K, tpr - t_first); /* tiles of this block */
    const long long row0 = r * cols, out0 = r * nseg;
    auto finish = [&](long long k, O acc) { /* segment k is complete */
        if (seeded) {
            const A z = Fn::lift(fold_seed<Fn>(p));
            acc.v = acc.have ? Fn::combine(acc.v, z) : z;
            acc.have = 1;
        }
        if (acc.have) fold_put<Fn>(p, out0 + k, Fn::lower(acc.v), oseq);
    };
    O none;
    none.have = 0;

    const long long first_off = offs[0], last_off = offs[nseg];
    if (first_off >= last_off) { /* no elements at all: every segment is empty */
        if (sp == 0 && seeded)
            for (long long k = tid; k < nseg; k += CTA) finish(k, none);
        return;
    }
    if (t_first * T >= last_off || min(cols, (t_first + kt) * T) <= first_off) return; /* no segment reaches this block */

    if (tid == 0) {
        mbar_init(&s_bar[0], CTA);
        mbar_init(&s_bar[1], CTA);
        fence_mbar_init();
        s_have_first = 0;
    }
    __syncthreads();
    /* tile i of the block goes to buffer i & 1; full tiles by bulk copies that complete on that buffer's barrier */
    auto start_tile = [&](int i) {
        const long long tl = (t_first + i) * T;
        const int valid = (int)min((long long)T, cols - tl);
        unsigned char *buf = s_raw + (i & 1) * DATA;
        if (valid == T)
            bal_issue<In>(buf, p.in, row0 + tl, tid, &s_bar[i & 1], iseq);
        else
            bal_fill<In>(buf, p.in, row0 + tl, valid, tid, iseq);
    };
    start_tile(0);
    if (kt > 1) start_tile(1);

    /* the segment that contains position x of the row (the last k whose offset is <= x; 0 when x lies before
     * the first segment) by a (2 CTA)-ary search: every round narrows [lo, hi) by that factor and all threads
     * follow the same path.  Four rounds of an L2 access each for 2^24 segments, hidden behind the copies. */
    auto find_segment = [&](long long x) {
        long long lo = 0, hi = nseg + 1;
        while (hi > lo) {
            const long long step = (hi - lo + 2 * CTA - 1) / (2 * CTA);
            const long long i0 = lo + (2 * tid) * step, i1 = i0 + step;
            const int v0 = i0 < hi ? offs[i0] : 0, v1 = i1 < hi ? offs[i1] : 0;
            /* offsets ascend, so the probes at or below x are the first c of the 2 CTA */
            const int c = __syncthreads_count(i0 < hi && (long long)v0 <= x) +
                          __syncthreads_count(i1 < hi && (long long)v1 <= x);
            if (c == 0) {
                hi = lo;
            } else {
                hi = min(hi, lo + c * step);
                lo = lo + (c - 1) * step + 1;
            }
        }
        return max(lo - 1, 0LL);
    };
    /* an offset relative to a tile that starts at `base`, clamped to [-1, BEYOND] */
    auto rel = [&](int o, long long base) {
        const long long d = (long long)o - base;
        return (int)max(-1LL, min(d, (long long)BEYOND));
    };
    long long kb = find_segment(t_first * T);
    for (int j = tid; j <= NOFF; j += CTA)
        if (kb + j <= nseg) s_off[j] = rel(offs[kb + j], t_first * T);
    __syncthreads();

    int cf = 0;    /* a segment boundary lies in the tiles done so far */
    O cv = none;   /* the open segment's part in them (since that boundary, if there is one) */
    for (int i = 0; i < kt; ++i) {
        const long long tile_lo = (t_first + i) * T;
        const int valid = (int)min((long long)T, cols - tile_lo);
        const unsigned char *buf = s_raw + (i & 1) * DATA;
        const int *so = s_off + (i & 1) * (NOFF + 1);
        const int nstaged = (int)min((long long)NOFF, nseg - kb); /* so[0 .. nstaged] are valid */
        auto off = [&](long long k) { return k - kb <= nstaged ? so[k - kb] : rel(offs[k], tile_lo); };

        /* ---- the next tile's first segment, found in this tile's window where that reaches far enough, and
         * its offsets fetched into registers while this tile is worked on */
        const bool more = i + 1 < kt;
        bool covered = false;
        long long kb_next = kb;
        int pre[NPRE];
        if (more) {
            covered = so[nstaged] > T || kb + nstaged >= nseg;
            if (covered) {
                if (so[0] <= T) {
                    int l = 0, h = nstaged + 1; /* so[l] <= T, and so[h] > T or h is past the window */
                    while (h - l > 1) {
                        const int m = (l + h) >> 1;
                        if (so[m] <= T)
                            l = m;
                        else
                            h = m;
                    }
                    kb_next = min(kb + l, max(nseg - 1, 0LL));
                }
#pragma unroll
                for (int q = 0; q < NPRE; ++q) {
                    const long long k = kb_next + tid + q * CTA;
                    pre[q] = (tid + q * CTA <= NOFF && k <= nseg) ? offs[k] : 0;
                }
            }
        }

        if (valid == T) {
            int tries = 0;
            while (!mbar_try_wait(&s_bar[i & 1], (unsigned)(i >> 1) & 1u)) {
                if (++tries > ACCB_FOLD_STAGE_SPIN_LIMIT) { /* bounded: flag the result invalid and go on */
                    atomicExch(err, 1u);
                    break;
                }
            }
        }

        /* ---- this thread's elements: tile-relative positions [a, b) */
        const int t_lo = (int)max(0LL, min((long long)T, first_off - tile_lo));
        const int t_hi = (int)max(0LL, min((long long)valid, last_off - tile_lo));
        const int c_lo = tid * V;
        const int a = max(c_lo, t_lo), b = min(c_lo + V, t_hi);
        O acc = none, head = none;
        long long head_seg = 0;
        int flag = 0;
        bool have_head = false;
        if (a < b) {
            /* segment of position a: the last k with off(k) <= a */
            long long seg;
            if (so[nstaged] > a) {
                int l = 0, h = nstaged; /* so[l] <= a < so[h] */
                while (h - l > 1) {
                    const int m = (l + h) >> 1;
                    if (so[m] <= a)
                        l = m;
                    else
                        h = m;
                }
                seg = kb + l;
            } else {
                long long l = kb + nstaged, h = nseg; /* off(l) <= a < off(h): a < last_off */
                while (h - l > 1) {
                    const long long m = (l + h) >> 1;
                    if (rel(offs[m], tile_lo) <= a)
                        l = m;
                    else
                        h = m;
                }
                seg = l;
            }
            bool open_before = off(seg) < a; /* the segment began in an earlier chunk */
            flag = !open_before;
            int segend = off(seg + 1);
            if ((long long)a == first_off - tile_lo && seeded) /* empty segments before the first element */
                for (long long k = 0; k < seg; ++k) finish(k, none);
            auto boundary = [&](int pos1) { /* segment `seg` ends before position pos1 */
                if (open_before) {
                    head = acc;
                    head_seg = seg;
                    have_head = true;
                    open_before = false;
                } else {
                    finish(seg, acc);
                }
                flag = 1;
                acc.have = 0;
                ++seg;
                segend = BEYOND;
                while (seg < nseg) { /* empty segments that begin here */
                    segend = off(seg + 1);
                    if (segend != pos1) break;
                    finish(seg, none);
                    ++seg;
                    segend = BEYOND;
                }
            };
            auto add = [&](typename Fn::elem x) {
                const A s = Fn::lift(x);
                acc.v = acc.have ? Fn::combine(acc.v, s) : s;
                acc.have = 1;
            };
#pragma unroll 1
            for (int j = 0; j < V; j += 4) {
                const int p0 = c_lo + j;
                if (p0 + 4 <= a || p0 >= b) continue;
                typename Fn::elem x[4];
                bal_get4<Fn>(env, buf, tid, j, row0 + tile_lo + p0, x, iseq);
                if (p0 >= a && p0 + 4 <= b && segend > p0 + 4) { /* no boundary among these four */
#pragma unroll
                    for (int u = 0; u < 4; ++u) add(x[u]);
                } else {
#pragma unroll
                    for (int u = 0; u < 4; ++u) {
                        const int pos = p0 + u;
                        if (pos >= a && pos < b) {
                            add(x[u]);
                            if (pos + 1 == segend) boundary(pos + 1);
                        }
                    }
                }
            }
        }

        /* ---- segmented scan of (flag, tail) over the block: what precedes each chunk inside the tile */
        int f = flag;
        O v = acc;
#pragma unroll
        for (int d = 1; d < 32; d <<= 1) {
            const int f2 = __shfl_up_sync(FULL, f, d);
            const O v2 = shfl_up(v, d);
            if (lane >= d) {
                if (!f) v = oc(v2, v);
                f |= f2;
            }
        }
        int ef = __shfl_up_sync(FULL, f, 1);
        O ev = shfl_up(v, 1);
        if (lane == 0) {
            ef = 0;
            ev = none;
        }
        if (lane == 31) {
            s_wf[warp] = f;
            s_wv[warp] = v;
        }
        __syncthreads();
        int tf = 0; /* the whole tile, known to every thread */
        O tv = none;
#pragma unroll
        for (int w = 0; w < WARPS; ++w) {
            if (w == warp) { /* what precedes this warp */
                if (!ef) ev = oc(tv, ev);
                ef |= tf;
            }
            if (s_wf[w]) {
                tv = s_wv[w];
                tf = 1;
            } else {
                tv = oc(tv, s_wv[w]);
            }
        }
        if (have_head) { /* the segment that was open when this chunk began ends here */
            O part = oc(ev, head);
            if (!ef) part = oc(cv, part); /* it began in an earlier tile */
            if (ef || cf) {
                finish(head_seg, part);
            } else { /* .. before the block: completed after the look-back */
                s_first = part;
                s_first_seg = head_seg;
                s_have_first = 1;
            }
        }
        if (tf) {
            cv = tv;
            cf = 1;
        } else {
            cv = oc(cv, tv);
        }

        /* ---- the next tile's window */
        if (more) {
            int *sn = s_off + ((i + 1) & 1) * (NOFF + 1);
            const long long next_lo = tile_lo + T;
            if (covered) {
#pragma unroll
                for (int q = 0; q < NPRE; ++q)
                    if (tid + q * CTA <= NOFF) sn[tid + q * CTA] = rel(pre[q], next_lo);
            } else { /* more than NOFF segments begin in this tile (runs of empty ones): search again */
                kb_next = find_segment(next_lo);
                for (int j = tid; j <= NOFF; j += CTA)
                    if (kb_next + j <= nseg) sn[j] = rel(offs[kb_next + j], next_lo);
            }
        }
        __syncthreads(); /* this tile's buffer and window are free; the next window is complete */
        if (i + 2 < kt) start_tile(i + 2);
        kb = kb_next;
    }

    /* ---- across blocks (warp 0).  A block with a boundary knows its open tail without anybody's help and
     * publishes it as a finished prefix; a block inside one long segment publishes an aggregate, looks back over
     * its predecessors' records as the scans do, then publishes the prefix.  The look-back also completes the
     * block's first segment when that began in an earlier block. */
    if (warp != 0) return;
    const bool pass = !cf, need = s_have_first != 0;
    if (!pass && lane == 0) status.publish(blk, (epoch << 2) | (cv.have ? ST_PREFIX : ST_PREFIX_NONE), cv.v);
    if (!(pass || need)) return;
    O pre = none;
    if (sp > 0) {
        if (pass && lane == 0) status.publish(blk, (epoch << 2) | ST_AGG, cv.v);
        long long look = blk - 1; /* lane l examines block look - l, never before the row's first */
        const long long row_first = blk - sp;
        int spins = 0;
        bool done = false;
        while (!done) {
            const long long idx = look - lane;
            A val;
            unsigned fl = 0;
            bool ready = idx < row_first;
            while (true) {
                if (!ready) {
                    fl = status.peek(idx, val);
                    ready = (fl >> 2) == epoch && (fl & 3u) != 0;
                }
                if (__all_sync(FULL, ready)) break;
                if (++spins > ACCB_FOLD_BAL_SPIN_LIMIT ||
                    ((spins & 255) == 0 && *static_cast<volatile unsigned int *>(err) != 0u)) {
                    if (lane == 0) atomicExch(err, 1u);
                    if (!ready) fl = (epoch << 2) | ST_PREFIX_NONE; /* the result is flagged invalid */
                    ready = true;
                }
            }
            const bool in_row = idx >= row_first;
            const bool is_pre = in_row && (fl & 3u) != ST_AGG;
            const unsigned pm = __ballot_sync(FULL, is_pre);
            const int first = pm ? __ffs(pm) - 1 : 32; /* nearest block with a finished prefix */
            O win;
            win.v = val;
            win.have = in_row && lane <= first && (fl & 3u) != ST_PREFIX_NONE;
#pragma unroll
            for (int d = 1; d < 32; d <<= 1) { /* lanes hold ever earlier blocks: combine far to near */
                O o = shfl_down(win, d);
                if (lane + d < 32) win = oc(o, win);
            }
            win = shfl_idx(win, 0);
            pre = oc(win, pre);
            done = pm != 0 || look - 32 < row_first;
            look -= 32;
        }
    }
    if (lane == 0) {
        if (pass) {
            const O incl = oc(pre, cv);
            status.publish(blk, (epoch << 2) | (incl.have ? ST_PREFIX : ST_PREFIX_NONE), incl.v);
        } else {
            finish(s_first_seg, oc(pre, s_first));
        }
    }
}

template <class Fn>
__device__ __forceinline__ void fold_balanced_or_nothing(const accb_kparams &p) {
    if constexpr (fold_bal_tile<Fn>() > 0) fold_balanced_body<Fn>(p);
}

}  // namespace accb
