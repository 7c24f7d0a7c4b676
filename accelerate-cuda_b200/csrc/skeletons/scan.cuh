/*
 * scan.cuh -- prefix sums: scanl, scanl1, scanl', scanr, scanr1, scanr'.
 *
 * Replaces the three-kernel reduce-then-scan of
 * Data/Array/Accelerate/CUDA/CodeGen/PrefixSum.hs:59-120,200-480 (up-sweep of
 * interval totals, scan of the totals, down-sweep that reads the input a
 * second time; host side scanOp/scan1Op/scan'Op/scanCore, Execute.hs:328-392)
 * by ONE single-pass kernel with decoupled look-back: every element is read
 * once and written once (8 bytes per Int32 element instead of 12).
 *
 * Semantics (PrefixSum.hs:137-198, Execute.hs:326-362), with all body writes
 * aligned to the input index so that 128-bit stores stay aligned:
 *   scanl  f z : out[i] = z (+) x0 .. x(i-1)  for i in [0,n), out[n] = total
 *   scanl1 f   : out[i] = x0 .. xi
 *   scanl' f z : body as scanl, total written to a separate scalar
 *   scanr  f z : out[i] = xi .. x(n-1) (+) z  (inclusive, seeded), out[n] = z
 *   scanr1 f   : out[i] = xi .. x(n-1)
 *   scanr' f z : out[i] = x(i+1) .. x(n-1) (+) z, total separate
 * Right scans follow Data.List.scanr: the new element is the LEFT argument.
 * (The reference applies the combiner with the same argument order in both
 * directions, PrefixSum.hs:264,525-527; that only matters for a
 * non-commutative combiner and is not reproduced.)
 * Only an associative combiner is required; value order is preserved.
 *
 * Functor contract: as for folds (see fold.cuh) with a single value type:
 *   using In = accb::types<...>;  typedef T elem;
 *   static T get(env, i, in-values...);  static T combine(T, T);
 *   using Out = accb::types<...>;  static void put(T, out-references...);
 *
 * Tile = CTA * ROWS * 4 elements.  A warp owns ROWS "rows" of 128 consecutive
 * elements; lane l of row j holds the 4 elements at 128*j + 4*l, so every
 * load and store instruction of a warp covers 512 contiguous bytes.
 * Tiles are handed out by an atomic ticket (never by blockIdx) so a tile's
 * predecessors are always already running: look-back cannot deadlock however
 * the hardware orders blocks.  The wait on a predecessor is nevertheless
 * bounded: after ACCB_SCAN_SPIN_LIMIT polls the kernel raises the error word
 * and carries on, so the launch always terminates.
 *
 * Runtime-owned scratch (never cleared between launches):
 *   aux[0] tile status words, aux[1] ticket counter, aux[2] error word.
 * Status words carry the launch epoch (ip[2]); words of earlier launches read
 * as "not ready".  The ticket counter only ever grows; ip[1] is its value at
 * launch.
 *   ip[0] tiles, ip[1] ticket base, ip[2] epoch, ip[3] index of the total in
 *   the "sum" slots out[Out::size..] (or -1), ip[4] index at which the seed is
 *   stored in the sum slots (or -1).
 */
#pragma once
#include "../cubits/accb_vec.cuh"
#include "../cubits/accb_warp.cuh"
#include "fold.cuh"

#ifndef ACCB_SCAN_CTA
#define ACCB_SCAN_CTA 512
#endif
#ifndef ACCB_SCAN_ROWS
#define ACCB_SCAN_ROWS 4
#endif
#ifndef ACCB_SCAN_SPIN_LIMIT
#define ACCB_SCAN_SPIN_LIMIT (1 << 20)
#endif

namespace accb {

template <class T>
struct Scan {
    typedef T elem;
    typedef T acc;
    typedef types<T> Out;
    static __device__ __forceinline__ void put(T r, T &o) { o = r; }
};

enum : unsigned { ST_AGG = 1u, ST_PREFIX = 2u };

/* ---- tile status: one 64-bit word {flag, value} when the value fits 32 bits,
 * otherwise {flag | aggregate | prefix} records published with release /
 * acquire ordering. ---- */
template <class T, bool PACKED = (sizeof(T) <= 4)>
struct TileStatus;

template <class T>
struct TileStatus<T, true> {
    static constexpr int kBytes = 8;
    unsigned long long *w;
    __device__ __forceinline__ explicit TileStatus(void *base) : w(static_cast<unsigned long long *>(base)) {}
    __device__ __forceinline__ void publish(long long t, unsigned flag, T v) const {
        unsigned bits = 0;
        memcpy(&bits, &v, sizeof(T));
        const unsigned long long word = ((unsigned long long)flag << 32) | bits;
        asm volatile("st.relaxed.gpu.global.u64 [%0], %1;" ::"l"(w + t), "l"(word) : "memory");
    }
    /* returns the flag word; value valid when the flag's epoch matches */
    __device__ __forceinline__ unsigned peek(long long t, T &v) const {
        unsigned long long word;
        asm volatile("ld.relaxed.gpu.global.u64 %0, [%1];" : "=l"(word) : "l"(w + t) : "memory");
        const unsigned bits = (unsigned)word;
        memcpy(&v, &bits, sizeof(T));
        return (unsigned)(word >> 32);
    }
};

template <class T>
struct TileStatus<T, false> {
    static_assert(sizeof(T) % 4 == 0 && sizeof(T) <= 32, "scan value types are at most 32 bytes");
    struct Rec {
        unsigned flag;
        unsigned pad;
        T agg;
        T pre;
    };
    static constexpr int kBytes = sizeof(Rec);
    Rec *r;
    __device__ __forceinline__ explicit TileStatus(void *base) : r(static_cast<Rec *>(base)) {}
    __device__ __forceinline__ void publish(long long t, unsigned flag, T v) const {
        T *dst = ((flag & 3u) == ST_AGG) ? &r[t].agg : &r[t].pre;
        constexpr int W = sizeof(T) / 4;
        unsigned wv[W];
        memcpy(wv, &v, sizeof(T));
#pragma unroll
        for (int i = 0; i < W; ++i) __stcg(reinterpret_cast<unsigned *>(dst) + i, wv[i]);
        asm volatile("st.release.gpu.global.u32 [%0], %1;" ::"l"(&r[t].flag), "r"(flag) : "memory");
    }
    __device__ __forceinline__ unsigned peek(long long t, T &v) const {
        unsigned flag;
        asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(flag) : "l"(&r[t].flag) : "memory");
        const T *src = ((flag & 3u) == ST_AGG) ? &r[t].agg : &r[t].pre;
        v = ld_cg(src);
        return flag;
    }
};

template <class Fn, bool RIGHT>
struct ScanOp {
    typedef typename Fn::elem T;
    /* a precedes b in scan order */
    __device__ __forceinline__ T operator()(T a, T b) const {
        if constexpr (RIGHT)
            return Fn::combine(b, a);
        else
            return Fn::combine(a, b);
    }
};

template <class Fn, int... O>
__device__ __forceinline__ void scan_put_sum(const accb_kparams &p, long long j, typename Fn::elem r,
                                             std::integer_sequence<int, O...>) {
    regs<1, typename Fn::Out> b;
    Fn::put(r, comp<O>(b)[0]...);
    store_one(p.out + Fn::Out::size, j, b);
}

template <class Fn, int N, int... O>
__device__ __forceinline__ void scan_put_vec(typename Fn::elem (&y)[N], regs<N, typename Fn::Out> &b,
                                             std::integer_sequence<int, O...>) {
#pragma unroll
    for (int k = 0; k < N; ++k) Fn::put(y[k], comp<O>(b)[k]...);
}

/* One tile, from load to store.  FT: the tile is full and vector-aligned, so
 * every "have" flag below is known at compile time and the warp scans run on
 * bare values. */
template <class Fn, int CTA, int ROWS, bool RIGHT, bool INCL, bool FT>
__device__ __forceinline__ void scan_tile(const accb_kparams &p, long long t, long long ntiles, long long base,
                                          long long len, typename Fn::elem *s_warp,
                                          Opt<typename Fn::elem> *s_prefix) {
    typedef typename Fn::elem T;
    typedef typename Fn::In In;
    typedef typename Fn::Out Out;
    typedef Opt<T> O;
    constexpr int NW = CTA / 32;
    constexpr int TILE = CTA * ROWS * V;
    constexpr int TILE_VECS = CTA * ROWS;
    const ScanOp<Fn, RIGHT> op;
    const Env env(p);
    const auto iseq = std::make_integer_sequence<int, In::size>();
    const auto oseq = std::make_integer_sequence<int, Out::size>();
    const bool seeded = (p.flags & ACCB_F_HAS_SEED) != 0;
    const unsigned epoch = (unsigned)p.ip[2];
    const TileStatus<T> status(p.aux[0]);
    unsigned int *err = static_cast<unsigned int *>(p.aux[2]);
    const int lane = lane_id(), w = warp_id();
    auto oc = [&](O a, O b) {
        O r;
        r.have = a.have | b.have;
        r.v = (a.have && b.have) ? op(a.v, b.v) : (a.have ? a.v : b.v);
        return r;
    };

    /* ---- load: x[j][k] is logical element (w*ROWS*128 + j*128 + lane*4 + k) of the tile ---- */
    T x[ROWS][V];
    int valid[ROWS][V];
    if constexpr (FT) {
        regs<V, In> a[ROWS];
#pragma unroll
        for (int j = 0; j < ROWS; ++j) {
            const int lv = w * (ROWS * 32) + j * 32 + lane;
            const long long pv = base / V + (RIGHT ? (TILE_VECS - 1 - lv) : lv);
            load_all(p.in, pv, a[j]);
        }
#pragma unroll
        for (int j = 0; j < ROWS; ++j) {
            const int lv = w * (ROWS * 32) + j * 32 + lane;
            const long long pv = base / V + (RIGHT ? (TILE_VECS - 1 - lv) : lv);
            T tmp[V];
            fold_get<Fn>(env, pv * V, a[j], tmp, iseq);
#pragma unroll
            for (int k = 0; k < V; ++k) {
                x[j][k] = RIGHT ? tmp[V - 1 - k] : tmp[k];
                valid[j][k] = 1;
            }
        }
    } else {
#pragma unroll
        for (int j = 0; j < ROWS; ++j)
#pragma unroll
            for (int k = 0; k < V; ++k) {
                const int q = (w * (ROWS * 32) + j * 32 + lane) * V + k;
                /* right scans walk the tile backwards; a ragged tile is then
                 * the first in scan order and its valid part sits at the low
                 * physical offsets */
                const long long off = RIGHT ? (long long)(TILE - 1 - q) : (long long)q;
                valid[j][k] = off < len;
                if (valid[j][k]) {
                    regs<1, In> a;
                    T tmp[1];
                    load_one(p.in, base + off, a);
                    fold_get<Fn>(env, base + off, a, tmp, iseq);
                    x[j][k] = tmp[0];
                }
            }
    }

    /* ---- thread-local sums, then a warp scan per row ---- */
    O ex[ROWS]; /* exclusive prefix of this thread's vector inside the warp chunk */
    O wtot;     /* total of the warp chunk */
    wtot.have = 0;
#pragma unroll
    for (int j = 0; j < ROWS; ++j) {
        if constexpr (FT) {
            const T s = op(op(x[j][0], x[j][1]), op(x[j][2], x[j][3]));
            const T inc = warp_scan_inclusive(s, op);
            const T up = shfl_up(inc, 1);
            const T last = shfl_idx(inc, 31);
            if (j == 0) {
                ex[j].v = up;
                ex[j].have = lane > 0;
                wtot.v = last;
            } else {
                ex[j].v = lane > 0 ? op(wtot.v, up) : wtot.v;
                ex[j].have = 1;
                wtot.v = op(wtot.v, last);
            }
            wtot.have = 1;
        } else {
            O s;
            s.have = 0;
#pragma unroll
            for (int k = 0; k < V; ++k) {
                O e;
                e.v = x[j][k];
                e.have = valid[j][k];
                s = oc(s, e);
            }
            O inc = warp_scan_inclusive(s, oc);
            O up = shfl_up(inc, 1);
            if (lane == 0) up.have = 0;
            ex[j] = oc(wtot, up);
            wtot = oc(wtot, shfl_idx(inc, 31));
        }
    }

    /* ---- block level ---- */
    if (lane == 0) s_warp[w] = wtot.v;
    __syncthreads();
    /* warps holding data: the first nwv for a left scan; for a right scan of
     * a ragged tile the EARLY logical positions are the empty ones */
    const int nwv = FT ? NW : (int)((len + ROWS * 128 - 1) / (ROWS * 128));
    const int w_lo = RIGHT ? NW - nwv : 0, w_hi = RIGHT ? NW : nwv;
    O wpre, agg;
    wpre.have = 0;
    agg.have = 0;
#pragma unroll
    for (int k = 0; k < NW; ++k) {
        O e;
        e.v = s_warp[k];
        e.have = FT ? 1 : (k >= w_lo && k < w_hi);
        if (k < w) wpre = oc(wpre, e);
        agg = oc(agg, e);
    }

    /* ---- decoupled look-back (warp 0) ---- */
    if (w == 0) {
        O pre;
        pre.have = 0;
        if (t == 0) {
            if (seeded) {
                pre.v = fold_seed<Fn>(p);
                pre.have = 1;
            }
            if (lane == 0) status.publish(0, (epoch << 2) | ST_PREFIX, oc(pre, agg).v);
        } else {
            if (lane == 0) status.publish(t, (epoch << 2) | ST_AGG, agg.v);
            long long look = t - 1;
            int spins = 0;
            bool done = false;
            while (!done) {
                const long long idx = look - lane;
                T v;
                unsigned flag = 0;
                bool ready = idx < 0;
                /* every lane polls its own predecessor until it is published */
                while (true) {
                    if (!ready) {
                        flag = status.peek(idx, v);
                        ready = (flag >> 2) == epoch && (flag & 3u) != 0;
                    }
                    if (__all_sync(FULL, ready)) break;
                    /* give up after the limit, or at once when another tile already gave up */
                    if (++spins > ACCB_SCAN_SPIN_LIMIT ||
                        ((spins & 255) == 0 && *static_cast<volatile unsigned int *>(err) != 0u)) {
                        if (lane == 0) atomicExch(err, 1u);
                        if (!ready) flag = (epoch << 2) | ST_PREFIX; /* give up; the result is flagged invalid */
                        ready = true;
                    }
                }
                const bool is_pre = idx >= 0 && (flag & 3u) == ST_PREFIX;
                const unsigned pm = __ballot_sync(FULL, is_pre);
                const int first = pm ? __ffs(pm) - 1 : 32; /* nearest tile with a full prefix */
                O win;
                win.v = v;
                win.have = (idx >= 0) && (lane <= first);
                /* lanes hold tiles look, look-1, ...: combine far-to-near */
#pragma unroll
                for (int d = 1; d < 32; d <<= 1) {
                    O o = shfl_down(win, d);
                    if (lane + d < 32) win = oc(o, win);
                }
                win = shfl_idx(win, 0);
                pre = oc(win, pre);
                done = pm != 0 || look < 32;
                look -= 32;
            }
            if (lane == 0) status.publish(t, (epoch << 2) | ST_PREFIX, oc(pre, agg).v);
        }
        if (lane == 0) {
            *s_prefix = pre;
            if (t == ntiles - 1 && p.ip[3] >= 0) scan_put_sum<Fn>(p, p.ip[3], oc(pre, agg).v, oseq);
            if (t == 0 && p.ip[4] >= 0 && seeded) scan_put_sum<Fn>(p, p.ip[4], fold_seed<Fn>(p), oseq);
        }
    }
    __syncthreads();
    const O tile_pre = oc(*s_prefix, wpre);

    /* ---- final values and store ---- */
#pragma unroll
    for (int j = 0; j < ROWS; ++j) {
        O run = oc(tile_pre, ex[j]);
        if constexpr (FT) {
            T y[V];
#pragma unroll
            for (int k = 0; k < V; ++k) {
                const T nxt = run.have ? op(run.v, x[j][k]) : x[j][k];
                y[RIGHT ? V - 1 - k : k] = INCL ? nxt : run.v;
                run.v = nxt;
                run.have = 1;
            }
            regs<V, Out> b;
            scan_put_vec<Fn>(y, b, oseq);
            const int lv = w * (ROWS * 32) + j * 32 + lane;
            const long long pv = base / V + (RIGHT ? (TILE_VECS - 1 - lv) : lv);
            store_all(p.out, pv, b);
        } else {
#pragma unroll
            for (int k = 0; k < V; ++k) {
                const int q = (w * (ROWS * 32) + j * 32 + lane) * V + k;
                const long long off = RIGHT ? (long long)(TILE - 1 - q) : (long long)q;
                if (valid[j][k]) {
                    const T nxt = run.have ? op(run.v, x[j][k]) : x[j][k];
                    regs<1, Out> b;
                    T y[1] = {INCL ? nxt : run.v};
                    scan_put_vec<Fn>(y, b, oseq);
                    store_one(p.out, base + off, b);
                    run.v = nxt;
                    run.have = 1;
                }
            }
        }
    }
}

template <class Fn, int CTA, int ROWS, bool RIGHT, bool INCL>
__device__ __forceinline__ void scan_body(const accb_kparams &p) {
    typedef typename Fn::elem T;
    constexpr int NW = CTA / 32;
    constexpr int TILE = CTA * ROWS * V;
    const auto oseq = std::make_integer_sequence<int, Fn::Out::size>();
    __shared__ T s_warp[NW];
    __shared__ Opt<T> s_prefix;
    __shared__ long long s_tile;

    const long long n = p.n;
    const long long ntiles = p.ip[0];
    unsigned int *ticket = static_cast<unsigned int *>(p.aux[1]);

    if (n == 0) { /* empty input: only the seed survives */
        if (blockIdx.x == 0 && threadIdx.x == 0 && (p.flags & ACCB_F_HAS_SEED)) {
            const T z = fold_seed<Fn>(p);
            if (p.ip[3] >= 0) scan_put_sum<Fn>(p, p.ip[3], z, oseq);
            if (p.ip[4] >= 0) scan_put_sum<Fn>(p, p.ip[4], z, oseq);
        }
        return;
    }

    if (threadIdx.x == 0) s_tile = (long long)(unsigned)(atomicAdd(ticket, 1u) - (unsigned)p.ip[1]);
    __syncthreads();
    const long long t = s_tile; /* position in scan order */
    if (t >= ntiles) return;
    const long long pt = RIGHT ? ntiles - 1 - t : t; /* position in memory */
    const long long base = pt * TILE;
    const long long len = (n - base) < TILE ? (n - base) : TILE;
    if ((p.flags & ACCB_F_VEC) && len == TILE)
        scan_tile<Fn, CTA, ROWS, RIGHT, INCL, true>(p, t, ntiles, base, len, s_warp, &s_prefix);
    else
        scan_tile<Fn, CTA, ROWS, RIGHT, INCL, false>(p, t, ntiles, base, len, s_warp, &s_prefix);
}

}  // namespace accb

/* Entry points named after the reference's kernels (PrefixSum.hs:208,313):
 * exclusive and inclusive, left and right. */
#define ACCB_INSTANTIATE_SCAN(Fn)                                                              \
    ACCB_META(5, ACCB_SCAN_CTA, accb::TileStatus<Fn::elem>::kBytes,                            \
              ACCB_SCAN_CTA * ACCB_SCAN_ROWS * 4, ACCB_SCAN_ROWS, 0)                           \
    extern "C" __global__ void __launch_bounds__(ACCB_SCAN_CTA)                                \
        scanl(const __grid_constant__ accb_kparams p) {                                        \
        accb::scan_body<Fn, ACCB_SCAN_CTA, ACCB_SCAN_ROWS, false, false>(p);                   \
    }                                                                                          \
    extern "C" __global__ void __launch_bounds__(ACCB_SCAN_CTA)                                \
        scanl1(const __grid_constant__ accb_kparams p) {                                       \
        accb::scan_body<Fn, ACCB_SCAN_CTA, ACCB_SCAN_ROWS, false, true>(p);                    \
    }                                                                                          \
    extern "C" __global__ void __launch_bounds__(ACCB_SCAN_CTA)                                \
        scanr(const __grid_constant__ accb_kparams p) {                                        \
        accb::scan_body<Fn, ACCB_SCAN_CTA, ACCB_SCAN_ROWS, true, false>(p);                    \
    }                                                                                          \
    extern "C" __global__ void __launch_bounds__(ACCB_SCAN_CTA)                                \
        scanr1(const __grid_constant__ accb_kparams p) {                                       \
        accb::scan_body<Fn, ACCB_SCAN_CTA, ACCB_SCAN_ROWS, true, true>(p);                     \
    }
