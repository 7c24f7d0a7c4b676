/*
 * stencil.cuh -- stencil and stencil2 over rank-1 and rank-2 arrays with
 * Clamp / Mirror / Wrap / Constant boundaries.
 *
 * Replaces mkStencil / mkStencil2
 * (Data/Array/Accelerate/CUDA/CodeGen/Stencil.hs:55-114,131-228), the tap
 * access and boundary code in CodeGen/Stencil/Extra.hs:53-128,191-226 and the
 * host drivers stencilOp / stencil2Op (Execute.hs:413-450).  The reference
 * gathers every tap from global memory per output point and decides interior
 * vs border per warp with __all; it also launches the kernel twice
 * (Execute.hs:422-423), which is not reproduced.
 *
 * Two forms.  The TILE form (second half of this file, `stencil_tile`) stages
 * each block's input tile in shared memory with the TMA engine and is what
 * runs for 4-byte elements on aligned arrays whose width is a multiple of 4.
 * The REGISTER form below takes every other case (any element size, ragged
 * widths, rank 1): each thread owns 4 adjacent columns and walks down a band
 * of rows keeping the (2*RY+1) x (4+2*RX) window in registers: per output row it
 * issues ONE 128-bit load, gets the RX halo columns from the neighbouring
 * lanes with shuffles (only the lanes at a warp edge or at the array edge
 * read the halo from memory, through the boundary function) and writes one
 * 128-bit store.  Every element is therefore requested from DRAM once per
 * band; the 2*RY halo rows of a band are shared with the neighbouring bands,
 * which run next to it in block order, so they come from L2.
 * Boundary semantics (Extra.hs:200-226): each coordinate is mapped on its
 * own; with Constant the whole tap is the constant when any coordinate is
 * outside (:122-128,191-196).
 *
 * Functor contract (derive from accb::Stencil<Tin, Tout, RY, RX>):
 *   static Tout apply(env, const Tin (&t)[2*RY+1][2*RX+1]);              stencil
 *   static Tout apply(env, const Tin (&a)[..][..], const Tin (&b)[..][..]); stencil2
 * A rank-1 array is a single row (RY = 0).
 *
 *   in[0] (and in[1] for stencil2) source, out[0] result
 *   ip[0] H, ip[1] W of the result; ip[2] rows per band; ip[3] threads along x
 *   (a multiple of 32); ip[4] boundary (0 clamp 1 mirror 2 wrap 3 constant);
 *   ip[5], ip[6] = H, W of source 1; ip[7], ip[8] = H, W of source 2;
 *   scalars[0..] the constant of the Constant boundary.
 */
#pragma once
#include "../cubits/accb_vec.cuh"
#include "../cubits/accb_warp.cuh"
#include "../cubits/accb_tma.cuh"

#ifndef ACCB_STENCIL_TILE_RPT
#define ACCB_STENCIL_TILE_RPT 8 /* tile form: output rows per thread */
#endif
/* tile form: resident blocks per SM to leave registers for.  The register window of a thread is
 * arrays x (2RY+1) x (4+2RX) values: six blocks (40 registers) hold a 3x3 window, larger windows
 * get four (64) or three (80) so that they do not spill. */
#ifdef ACCB_STENCIL_TILE_MINB
#define ACCB_STENCIL_TILE_MINB_FOR(Fn, narr) ACCB_STENCIL_TILE_MINB
#else
#define ACCB_STENCIL_TILE_MINB_FOR(Fn, narr)                                   \
    ((narr) * (2 * Fn::RY + 1) * (4 + 2 * Fn::RX) <= 20 ? 6                    \
                                                        : ((narr) * (2 * Fn::RY + 1) * (4 + 2 * Fn::RX) <= 40 ? 4 : 3))
#endif
#ifndef ACCB_STENCIL_TILE2_RPT
#define ACCB_STENCIL_TILE2_RPT 6 /* two-application tile form: output rows per thread */
#endif
#ifndef ACCB_STENCIL_TILE2_MINB
#define ACCB_STENCIL_TILE2_MINB 4 /* .. resident blocks per SM to leave registers for */
#endif
#ifndef ACCB_STENCIL_TMA_SPIN_LIMIT
#define ACCB_STENCIL_TMA_SPIN_LIMIT (1 << 16)
#endif
#ifndef ACCB_STENCIL_CTA
#define ACCB_STENCIL_CTA 256
#endif
#ifndef ACCB_STENCIL_MINB
#define ACCB_STENCIL_MINB 4 /* resident blocks per SM the compiler must leave registers for */
#endif
#ifndef ACCB_STENCIL_ROWS_IN_FLIGHT
#define ACCB_STENCIL_ROWS_IN_FLIGHT 2 /* rows whose loads are issued before the first is used */
#endif

namespace accb {

template <class Tin, class Tout, int RY_, int RX_>
struct Stencil {
    typedef Tin in_t;
    typedef Tout out_t;
    static constexpr int RY = RY_, RX = RX_;
};

enum : int { B_CLAMP = 0, B_MIRROR = 1, B_WRAP = 2, B_CONSTANT = 3 };

/* one coordinate through the boundary; -1 = outside (Constant only) */
__device__ __forceinline__ int bound_coord(int i, int sz, int mode) {
    if (i >= 0 && i < sz) return i;
    int r;
    switch (mode) {
        case B_CLAMP: r = i < 0 ? 0 : sz - 1; break;
        case B_MIRROR: r = i < 0 ? -i : sz - (i - sz + 2); break;
        case B_WRAP: r = i < 0 ? sz + i : i - sz; break;
        default: return -1;
    }
    /* Mirror and Wrap assume an array at least as large as the stencil
     * (Extra.hs:206-207); never index outside a smaller one */
    return max(0, min(r, sz - 1));
}

/* A source array seen through its boundary condition. */
template <class T>
struct Source {
    const T *base;
    int h, w, mode;
    T cval;
    bool vec_ok;
    /* element (yy, x) where yy is already mapped (or -1) and x is raw */
    __device__ __forceinline__ T at(int yy, int x) const {
        const int xx = bound_coord(x, w, mode);
        if (yy < 0 || xx < 0) return cval;
        return base[(long long)yy * w + xx];
    }
};

/* What a thread reads from memory for one row: its 4 centre columns and, only
 * for lanes whose neighbour cannot supply them (warp edge, array edge), the
 * halo columns.  Issuing is kept apart from using so that the loads of several
 * rows can be in flight at once. */
template <class T, int RX>
struct RowRaw {
    T c[V];
    T l[RX > 0 ? RX : 1], r[RX > 0 ? RX : 1];
};

/* A thread's columns, fixed for a whole band: where its halo columns come
 * from is decided once here (boundary mapping in x included), not per row. */
template <int RX>
struct Cols {
    int x0;
    bool active;  /* x0 < w */
    bool vec;     /* the 4 centre columns are one aligned 16-byte load */
    bool l_ok;    /* left halo comes from lane-1 */
    bool r_ok;    /* right halo comes from lane+1 */
    int xl[RX > 0 ? RX : 1], xr[RX > 0 ? RX : 1]; /* mapped halo columns when read from memory (-1: constant) */
    int xc[V];    /* mapped centre columns for a ragged or unaligned vector */
};

template <class T, int RX>
__device__ __forceinline__ Cols<RX> make_cols(const Source<T> &s, int x0) {
    Cols<RX> c;
    const int lane = lane_id();
    c.x0 = x0;
    c.active = x0 < s.w;
    c.vec = s.vec_ok && x0 + V <= s.w;
    c.l_ok = lane > 0 && x0 > 0;
    c.r_ok = lane < 31 && x0 + 2 * V <= s.w;
#pragma unroll
    for (int k = 0; k < V; ++k) c.xc[k] = bound_coord(x0 + k, s.w, s.mode);
#pragma unroll
    for (int d = 0; d < RX; ++d) {
        c.xl[d] = bound_coord(x0 - RX + d, s.w, s.mode);
        c.xr[d] = bound_coord(x0 + V + d, s.w, s.mode);
    }
    return c;
}

template <class T, int RX>
__device__ __forceinline__ void issue_row(const Source<T> &s, int y, const Cols<RX> &c, RowRaw<T, RX> &raw) {
    const int yy = bound_coord(y, s.h, s.mode);
    const T *row = s.base + (long long)(yy < 0 ? 0 : yy) * s.w;
    if (yy >= 0 && c.vec) {
        load4<Cache::Default>(row, c.x0 / V, raw.c);
    } else {
#pragma unroll
        for (int k = 0; k < V; ++k) raw.c[k] = (c.active && yy >= 0 && c.xc[k] >= 0) ? row[c.xc[k]] : s.cval;
    }
    if constexpr (RX > 0) {
        if (c.active && !(c.l_ok && c.r_ok)) { /* only warp-edge and array-edge lanes */
#pragma unroll
            for (int d = 0; d < RX; ++d) {
                if (!c.l_ok) raw.l[d] = (yy >= 0 && c.xl[d] >= 0) ? row[c.xl[d]] : s.cval;
                if (!c.r_ok) raw.r[d] = (yy >= 0 && c.xr[d] >= 0) ? row[c.xr[d]] : s.cval;
            }
        }
    }
}

/* Complete a row: centre columns x0..x0+3 in r[RX..RX+3], halos in r[0..RX)
 * and r[RX+4..], taken from the neighbouring lanes where they hold them.
 * Every lane of the warp takes part in the shuffles. */
template <class T, int RX>
__device__ __forceinline__ void finish_row(const Cols<RX> &c, const RowRaw<T, RX> &raw, T (&r)[4 + 2 * RX]) {
#pragma unroll
    for (int k = 0; k < V; ++k) r[RX + k] = raw.c[k];
    if constexpr (RX > 0) {
#pragma unroll
        for (int d = 0; d < RX; ++d) {
            const T lf = shfl_up(raw.c[V - RX + d], 1); /* columns x0-RX+d */
            const T rt = shfl_down(raw.c[d], 1);        /* columns x0+4+d */
            r[d] = c.l_ok ? lf : raw.l[d];
            r[RX + V + d] = c.r_ok ? rt : raw.r[d];
        }
    }
}

/* One thread's walk down a band of rows [y_begin, y_end). */
template <class Fn, int NARR, bool FAST>
__device__ __forceinline__ void stencil_band(const Env &env, const Source<typename Fn::in_t> (&src)[NARR],
                                             const Cols<Fn::RX> (&cols)[NARR], typename Fn::out_t *out, int W,
                                             int x0, int y_begin, int y_end, bool out_vec) {
    typedef typename Fn::in_t Tin;
    typedef typename Fn::out_t Tout;
    constexpr int RY = Fn::RY, RX = Fn::RX;
    constexpr int WIN = 2 * RY + 1;
    constexpr int RW = 4 + 2 * RX;
    constexpr int CH = WIN * ((ACCB_STENCIL_ROWS_IN_FLIGHT + WIN - 1) / WIN);

    /* FAST: pointers to this thread's vector in the next row to load / store */
    const Tin *rp[NARR];
#pragma unroll
    for (int a = 0; a < NARR; ++a)
        rp[a] = src[a].base + (FAST ? ((long long)(y_begin - RY) * src[a].w + x0) : 0LL);
    Tout *op = out + (FAST ? ((long long)y_begin * W + x0) : 0LL);

    auto issue = [&](int a, int y, RowRaw<Tin, RX> &raw) {
        if constexpr (FAST) {
            load4<Cache::Default>(rp[a], 0, raw.c);
            if constexpr (RX > 0) {
#pragma unroll
                for (int d = 0; d < RX; ++d) {
                    if (!cols[a].l_ok) raw.l[d] = cols[a].xl[d] >= 0 ? rp[a][cols[a].xl[d] - x0] : src[a].cval;
                    if (!cols[a].r_ok) raw.r[d] = cols[a].xr[d] >= 0 ? rp[a][cols[a].xr[d] - x0] : src[a].cval;
                }
            }
            rp[a] += src[a].w;
        } else {
            issue_row<Tin, RX>(src[a], y, cols[a], raw);
        }
    };

    Tin win[NARR][WIN][RW];
    /* preload rows y_begin-RY .. y_begin+RY-1 into slots 0 .. 2RY-1 */
    if constexpr (WIN > 1) {
        RowRaw<Tin, RX> pre[NARR][WIN - 1];
#pragma unroll
        for (int s = 0; s < WIN - 1; ++s)
#pragma unroll
            for (int a = 0; a < NARR; ++a) issue(a, y_begin - RY + s, pre[a][s]);
#pragma unroll
        for (int a = 0; a < NARR; ++a)
#pragma unroll
            for (int s = 0; s < WIN - 1; ++s) finish_row<Tin, RX>(cols[a], pre[a][s], win[a][s]);
    }

    /* CH output rows per trip (a multiple of WIN, so window slots are
     * compile-time): first issue the loads of all CH new rows, then complete
     * and use them one by one */
    for (int y = y_begin; y < y_end; y += CH) {
        RowRaw<Tin, RX> raw[NARR][CH];
#pragma unroll
        for (int u = 0; u < CH; ++u)
            if (y + u < y_end) {
#pragma unroll
                for (int a = 0; a < NARR; ++a) issue(a, y + u + RY, raw[a][u]);
            }
#pragma unroll
        for (int u = 0; u < CH; ++u) {
            const int s = u % WIN; /* (yo - y_begin) % WIN */
            const int yo = y + u;  /* output row */
            if (yo < y_end) {
                /* newest row yo+RY goes to slot (s + 2RY) % WIN */
#pragma unroll
                for (int a = 0; a < NARR; ++a)
                    finish_row<Tin, RX>(cols[a], raw[a][u], win[a][(s + 2 * RY) % WIN]);
                if (FAST || x0 < W) {
                    Tout o[V];
#pragma unroll
                    for (int k = 0; k < V; ++k) {
                        Tin t[NARR][WIN][2 * RX + 1];
#pragma unroll
                        for (int a = 0; a < NARR; ++a)
#pragma unroll
                            for (int dy = 0; dy < WIN; ++dy)
#pragma unroll
                                for (int dx = 0; dx < 2 * RX + 1; ++dx)
                                    t[a][dy][dx] = win[a][(s + dy) % WIN][k + dx];
                        if constexpr (NARR == 1)
                            o[k] = Fn::apply(env, t[0]);
                        else
                            o[k] = Fn::apply(env, t[0], t[1]);
                    }
                    if constexpr (FAST) {
                        store4<Cache::Stream>(op, 0, o);
                        op += W;
                    } else if (out_vec && x0 + V <= W) {
                        store4<Cache::Stream>(out, ((long long)yo * W + x0) / V, o);
                    } else {
#pragma unroll
                        for (int k = 0; k < V; ++k)
                            if (x0 + k < W) out[(long long)yo * W + x0 + k] = o[k];
                    }
                }
            }
        }
    }
}

template <class Fn, int NARR, int CTA>
__device__ __forceinline__ void stencil_body(const accb_kparams &p) {
    typedef typename Fn::in_t Tin;
    typedef typename Fn::out_t Tout;
    constexpr int RY = Fn::RY, RX = Fn::RX;
    const Env env(p);
    const int H = (int)p.ip[0], W = (int)p.ip[1];
    const int RB = (int)p.ip[2], TXW = (int)p.ip[3];
    const int mode = (int)p.ip[4];
    const bool vec_ok = (p.flags & ACCB_F_VEC) != 0;

    Source<Tin> src[NARR];
#pragma unroll
    for (int a = 0; a < NARR; ++a) {
        src[a].base = static_cast<const Tin *>(p.in[a]);
        src[a].h = (int)p.ip[5 + 2 * a];
        src[a].w = (int)p.ip[6 + 2 * a];
        src[a].mode = mode;
        src[a].cval = env.scalar<Tin>(0);
        src[a].vec_ok = vec_ok && (src[a].w % V) == 0;
    }
    Tout *out = static_cast<Tout *>(p.out[0]);
    const bool out_vec = vec_ok && (W % V) == 0;

    const int tx = threadIdx.x % TXW, ty = threadIdx.x / TXW;
    const int TY = CTA / TXW;
    const int ncg = (W + TXW * V - 1) / (TXW * V);          /* column groups */
    const int nbands = (H + RB * TY - 1) / (RB * TY);       /* block-level bands */
    for (long long b = blockIdx.x; b < (long long)ncg * nbands; b += gridDim.x) {
        const int cg = (int)(b % ncg), band = (int)(b / ncg);
        const int x0 = (cg * TXW + tx) * V;
        Cols<RX> cols[NARR];
#pragma unroll
        for (int a = 0; a < NARR; ++a) cols[a] = make_cols<Tin, RX>(src[a], x0);
        const int y_begin = (band * TY + ty) * RB;
        const int y_end = min(H, y_begin + RB);
        if (y_begin >= H) continue; /* whole warps share ty, so a warp leaves together */

        /* Fast band: every row the band touches is inside every source and the
         * whole warp moves aligned vectors, so rows are reached by pointer
         * increments and no per-row boundary test is needed. */
        bool fast = out_vec && x0 + V <= W && y_begin - RY >= 0;
#pragma unroll
        for (int a = 0; a < NARR; ++a) fast = fast && cols[a].vec && y_end + RY <= src[a].h;
        if (__all_sync(FULL, fast))
            stencil_band<Fn, NARR, true>(env, src, cols, out, W, x0, y_begin, y_end, out_vec);
        else
            stencil_band<Fn, NARR, false>(env, src, cols, out, W, x0, y_begin, y_end, out_vec);
    }
}

/* ------------------------------------------------------------------------
 * Tile form: the (RB + 2RY) x (TW + 8) input tile of a block is brought into
 * shared memory by the TMA engine, one cp.async.bulk per tile row, all
 * completing on one mbarrier.  Nothing holds registers while the copies are
 * in flight, so the bytes in flight per SM are bounded by shared memory (six
 * 36 KB tiles), not by the register file -- the same reason as in scan.cuh.
 * Rows outside the array are fetched from their boundary-mapped row; the few
 * halo columns that fall outside the array (first / last column tile only)
 * and the rows of a Constant boundary are patched by the threads afterwards.
 * Then each thread walks RPT rows of 4 columns with the usual register
 * window, reading shared memory only.
 * Needs 4-byte elements, source widths that are multiples of 4 and 16-byte
 * aligned arrays (checked by the host, which otherwise launches `stencil`).
 * ---------------------------------------------------------------------- */
template <class Fn, int NARR, int CTA>
struct StencilTile {
    static constexpr int RY = Fn::RY, RX = Fn::RX;
    static constexpr int TXW = 64;                     /* threads along x */
    static constexpr int TY = CTA / TXW;               /* thread rows */
    static constexpr int RPT = ACCB_STENCIL_TILE_RPT;  /* output rows per thread */
    static constexpr int RB = TY * RPT;                /* output rows per tile */
    static constexpr int TW = TXW * V;                 /* output columns per tile */
    static constexpr int HX = 4;                       /* halo columns kept each side (16 bytes) */
    static constexpr int PW = TW + 2 * HX;             /* pitch of a tile row in elements */
    static constexpr int SR = RB + 2 * RY;             /* tile rows */
    static constexpr int kSmemBytes = NARR * SR * PW * 4;
    static_assert(RX <= HX, "stencil radius in x is at most 4 in the tile form");
};

template <class Fn, int NARR, int CTA>
__device__ __forceinline__ void stencil_tile_body(const accb_kparams &p) {
    typedef typename Fn::in_t Tin;
    typedef typename Fn::out_t Tout;
    typedef StencilTile<Fn, NARR, CTA> G;
    static_assert(sizeof(Tin) == 4 && sizeof(Tout) == 4, "tile form: 4-byte elements");
    constexpr int RY = G::RY, RX = G::RX, WIN = 2 * RY + 1, RW = 4 + 2 * RX;
    extern __shared__ __align__(128) unsigned char s_raw[];
    __shared__ __align__(8) unsigned long long s_bar;
    Tin(*tile)[G::SR][G::PW] = reinterpret_cast<Tin(*)[G::SR][G::PW]>(s_raw);

    const Env env(p);
    const int H = (int)p.ip[0], W = (int)p.ip[1];
    const int mode = (int)p.ip[4];
    Source<Tin> src[NARR];
#pragma unroll
    for (int a = 0; a < NARR; ++a) {
        src[a].base = static_cast<const Tin *>(p.in[a]);
        src[a].h = (int)p.ip[5 + 2 * a];
        src[a].w = (int)p.ip[6 + 2 * a];
        src[a].mode = mode;
        src[a].cval = env.scalar<Tin>(0);
        src[a].vec_ok = true;
    }
    Tout *out = static_cast<Tout *>(p.out[0]);
    unsigned int *err = static_cast<unsigned int *>(p.aux[1]);

    const int ncg = (W + G::TW - 1) / G::TW;
    const int x0t = (int)(blockIdx.x % ncg) * G::TW, y0t = (int)(blockIdx.x / ncg) * G::RB;
    /* columns [xs, xe) of source a are copied to tile columns [xs - (x0t - HX), ...) */
    auto col_range = [&](int a, int &xs, int &xe) {
        xs = max(0, x0t - G::HX);
        xe = min(src[a].w, x0t + G::TW + G::HX);
    };

    if (threadIdx.x == 0) {
        mbar_init(&s_bar, 1);
        fence_mbar_init();
    }
    __syncthreads();
    if (warp_id() == 0) {
        if (lane_id() == 0) {
            unsigned total = 0;
#pragma unroll
            for (int a = 0; a < NARR; ++a) {
                int xs, xe;
                col_range(a, xs, xe);
                for (int r = 0; r < G::SR; ++r)
                    if (bound_coord(y0t - RY + r, src[a].h, mode) >= 0) total += (unsigned)(xe - xs) * 4u;
            }
            mbar_expect_tx(&s_bar, total);
        }
        __syncwarp();
#pragma unroll
        for (int a = 0; a < NARR; ++a) {
            int xs, xe;
            col_range(a, xs, xe);
            for (int r = lane_id(); r < G::SR; r += 32) {
                const int yy = bound_coord(y0t - RY + r, src[a].h, mode);
                if (yy >= 0)
                    bulk_g2s(&tile[a][r][xs - (x0t - G::HX)], src[a].base + (long long)yy * src[a].w + xs,
                             (unsigned)(xe - xs) * 4u, &s_bar);
            }
        }
    }
    int tries = 0;
    while (!mbar_try_wait(&s_bar, 0)) {
        if (++tries > ACCB_STENCIL_TMA_SPIN_LIMIT) { /* bounded: flag the result invalid and go on */
            atomicExch(err, 1u);
            break;
        }
    }
    /* patch what the copies could not bring: columns outside the array, rows of a Constant boundary */
#pragma unroll
    for (int a = 0; a < NARR; ++a) {
        int xs, xe;
        col_range(a, xs, xe);
        const int lo = x0t - RX, hi = min(x0t + G::TW, W) + RX; /* columns any tap of this tile may touch */
        const int nleft = max(0, xs - lo), nright = max(0, hi - xe);
        const int per_row = nleft + nright;
        for (int i = threadIdx.x; i < G::SR * per_row; i += CTA) {
            const int r = i / per_row, j = i - r * per_row;
            const int c = j < nleft ? lo + j : xe + (j - nleft);
            const int yy = bound_coord(y0t - RY + r, src[a].h, mode);
            tile[a][r][c - (x0t - G::HX)] = src[a].at(yy, c);
        }
        if (mode == B_CONSTANT) {
            for (int r = 0; r < G::SR; ++r) {
                if (bound_coord(y0t - RY + r, src[a].h, mode) >= 0) continue; /* uniform per block */
                for (int c = threadIdx.x; c < G::PW; c += CTA) tile[a][r][c] = src[a].cval;
            }
        }
    }
    __syncthreads();

    /* each thread: 4 columns, RPT rows, window in registers, shared-memory reads only */
    const int tx = threadIdx.x % G::TXW, ty = threadIdx.x / G::TXW;
    const int x = x0t + tx * V;
    if (x >= W) return;
    const int sc = G::HX + tx * V; /* tile column of the thread's first centre column */
    auto row = [&](int a, int r, Tin(&d)[RW]) {
        const Tin *q = &tile[a][r][sc];
        Tin c[V];
        load4<Cache::Default>(q, 0, c);
#pragma unroll
        for (int k = 0; k < V; ++k) d[RX + k] = c[k];
#pragma unroll
        for (int k = 0; k < RX; ++k) {
            d[k] = q[k - RX];
            d[RX + V + k] = q[V + k];
        }
    };
    Tin win[NARR][WIN][RW];
#pragma unroll
    for (int a = 0; a < NARR; ++a)
#pragma unroll
        for (int s = 0; s < WIN - 1; ++s) row(a, ty * G::RPT + s, win[a][s]);
    const bool vec_store = x + V <= W;
#pragma unroll
    for (int u = 0; u < G::RPT; ++u) {
        const int yo = y0t + ty * G::RPT + u;
        if (yo >= H) break;
#pragma unroll
        for (int a = 0; a < NARR; ++a) row(a, ty * G::RPT + u + 2 * RY, win[a][(u + 2 * RY) % WIN]);
        Tout o[V];
#pragma unroll
        for (int k = 0; k < V; ++k) {
            Tin t[NARR][WIN][2 * RX + 1];
#pragma unroll
            for (int a = 0; a < NARR; ++a)
#pragma unroll
                for (int dy = 0; dy < WIN; ++dy)
#pragma unroll
                    for (int dx = 0; dx < 2 * RX + 1; ++dx) t[a][dy][dx] = win[a][(u + dy) % WIN][k + dx];
            if constexpr (NARR == 1)
                o[k] = Fn::apply(env, t[0]);
            else
                o[k] = Fn::apply(env, t[0], t[1]);
        }
        if (vec_store) {
            store4<Cache::Stream>(out + (long long)yo * W + x, 0, o);
        } else {
#pragma unroll
            for (int k = 0; k < V; ++k)
                if (x + k < W) out[(long long)yo * W + x + k] = o[k];
        }
    }
}

/* ------------------------------------------------------------------------
 * Two applications in one launch (an iterated stencil: the same functor applied again and again, e.g. ten
 * blurs).  Applied one by one, every application reads and writes the whole grid: 8 bytes per point and
 * application.  Here a block brings in its tile with TWICE the halo, applies the stencil to it into a second
 * shared-memory tile (the intermediate grid of the block: its output rows and columns plus one halo), and applies
 * it again from there: one read and one write of the grid for two applications.
 * The intermediate tile must look to the second application as the whole intermediate grid would: what lies
 * outside the array is replaced through the boundary function -- by the intermediate value at the mapped
 * coordinate for Clamp and Mirror (always inside the same tile), by the constant for Constant.  Wrap maps to the
 * far side of the grid and is not done this way.  The results are those of two separate applications bit for
 * bit: the same arithmetic on the same float values, the intermediate rounded to 4 bytes in both cases.
 * One source, 4-byte elements of one type, radius in x of at most 2.
 * ---------------------------------------------------------------------- */
template <class Fn, int CTA>
struct StencilTile2 {
    static constexpr int RY = Fn::RY, RX = Fn::RX;
    static constexpr int TXW = 64, TY = CTA / TXW, RPT = ACCB_STENCIL_TILE2_RPT;
    static constexpr int RB = TY * RPT, TW = TXW * V, HX = 4, PW = TW + 2 * HX;
    static constexpr int SRI = RB + 4 * RY; /* rows of the source tile */
    static constexpr int SRM = RB + 2 * RY; /* rows of the intermediate tile */
    static constexpr int kSmemBytes = (SRI + SRM) * PW * 4;
};

/* One tile per block, as in the tile form: the blocks resident on an SM overlap one another's copies and
 * arithmetic.  (Tried: persistent blocks that walk through tiles with the next tile's copies in flight into a
 * second source buffer.  Ten applications on 8192 x 8192 took 0.74 ms instead of 0.68 ms: the third tile per block
 * costs a resident block, and the hardware's block scheduling already overlaps what the loop overlapped by hand.) */
template <class Fn, int CTA>
__device__ __forceinline__ void stencil_tile2_body(const accb_kparams &p) {
    typedef typename Fn::in_t T;
    typedef StencilTile2<Fn, CTA> G;
    static_assert(sizeof(T) == 4 && 2 * Fn::RX <= G::HX, "4-byte elements, radius in x of at most 2");
    constexpr int RY = G::RY, RX = G::RX, WIN = 2 * RY + 1, RW = 4 + 2 * RX;
    extern __shared__ __align__(128) unsigned char s_raw[];
    __shared__ __align__(8) unsigned long long s_bar;
    T(*tin)[G::PW] = reinterpret_cast<T(*)[G::PW]>(s_raw);
    T(*mid)[G::PW] = reinterpret_cast<T(*)[G::PW]>(s_raw + G::SRI * G::PW * 4);

    const Env env(p);
    const int H = (int)p.ip[0], W = (int)p.ip[1];
    const int mode = (int)p.ip[4];
    Source<T> src;
    src.base = static_cast<const T *>(p.in[0]);
    src.h = H;
    src.w = W;
    src.mode = mode;
    src.cval = env.scalar<T>(0);
    src.vec_ok = true;
    T *out = static_cast<T *>(p.out[0]);
    unsigned int *err = static_cast<unsigned int *>(p.aux[1]);

    const int ncg = (W + G::TW - 1) / G::TW;
    const int x0t = (int)(blockIdx.x % ncg) * G::TW, y0t = (int)(blockIdx.x / ncg) * G::RB;
    /* source rows y0t - 2RY .. (SRI of them), columns [xs, xe) to tile columns [xs - (x0t - HX), ...) */
    const int xs = max(0, x0t - G::HX), xe = min(W, x0t + G::TW + G::HX);
    if (threadIdx.x == 0) {
        mbar_init(&s_bar, 1);
        fence_mbar_init();
    }
    __syncthreads();
    if (warp_id() == 0) {
        if (lane_id() == 0) {
            unsigned total = 0;
            for (int r = 0; r < G::SRI; ++r)
                if (bound_coord(y0t - 2 * RY + r, H, mode) >= 0) total += (unsigned)(xe - xs) * 4u;
            mbar_expect_tx(&s_bar, total);
        }
        __syncwarp();
        for (int r = lane_id(); r < G::SRI; r += 32) {
            const int yy = bound_coord(y0t - 2 * RY + r, H, mode);
            if (yy >= 0)
                bulk_g2s(&tin[r][xs - (x0t - G::HX)], src.base + (long long)yy * W + xs, (unsigned)(xe - xs) * 4u, &s_bar);
        }
    }
    int tries = 0;
    while (!mbar_try_wait(&s_bar, 0)) {
        if (++tries > ACCB_STENCIL_TMA_SPIN_LIMIT) { /* bounded: flag the result invalid and go on */
            atomicExch(err, 1u);
            break;
        }
    }
    /* patch what the copies could not bring: columns outside the array, rows of a Constant boundary */
    {
        const int lo = x0t - 2 * RX, hi = min(x0t + G::TW, W) + 2 * RX; /* columns any tap of the first application may touch */
        const int nleft = max(0, xs - lo), nright = max(0, hi - xe);
        const int per_row = nleft + nright;
        for (int i = threadIdx.x; i < G::SRI * per_row; i += CTA) {
            const int r = i / per_row, j = i - r * per_row;
            const int c = j < nleft ? lo + j : xe + (j - nleft);
            tin[r][c - (x0t - G::HX)] = src.at(bound_coord(y0t - 2 * RY + r, H, mode), c);
        }
        if (mode == B_CONSTANT) {
            for (int r = 0; r < G::SRI; ++r) {
                if (bound_coord(y0t - 2 * RY + r, H, mode) >= 0) continue; /* uniform per block */
                for (int c = threadIdx.x; c < G::PW; c += CTA) tin[r][c] = src.cval;
            }
        }
    }
    __syncthreads();

    const int tx = threadIdx.x % G::TXW, ty = threadIdx.x / G::TXW;
    const int sc = G::HX + tx * V; /* tile column of the thread's first centre column */
    /* a thread's part of tile row r: its own 4 columns by one 16-byte read, the RX columns either side by 4-byte
     * reads (taking them from the neighbouring lanes by shuffle instead measured slower here: 0.72 ms against
     * 0.69 ms for ten applications on 8192 x 8192 -- the kernel is bound by instruction issue) */
    auto row = [&](const T(*tile)[G::PW], int r, T(&d)[RW]) {
        const T *q = &tile[r][sc];
        T c[V];
        load4<Cache::Default>(q, 0, c);
#pragma unroll
        for (int k = 0; k < V; ++k) d[RX + k] = c[k];
#pragma unroll
        for (int k = 0; k < RX; ++k) {
            d[k] = q[k - RX];
            d[RX + V + k] = q[V + k];
        }
    };
    auto apply4 = [&](T(&win)[WIN][RW], int first, T(&o)[V]) { /* window row dy is win[(first + dy) % WIN] */
#pragma unroll
        for (int k = 0; k < V; ++k) {
            T t[WIN][2 * RX + 1];
#pragma unroll
            for (int dy = 0; dy < WIN; ++dy)
#pragma unroll
                for (int dx = 0; dx < 2 * RX + 1; ++dx) t[dy][dx] = win[(first + dy) % WIN][k + dx];
            o[k] = Fn::apply(env, t);
        }
    };

    /* ---- first application: intermediate row m is row y0t - RY + m of the grid and reads source tile rows
     * m .. m + 2RY; the threads' own 4 columns each, the intermediate rows dealt to the TY thread rows */
    {
        constexpr int R1 = (G::SRM + G::TY - 1) / G::TY;
        const int m0 = ty * R1;
        T win[WIN][RW];
#pragma unroll
        for (int s2 = 0; s2 < WIN - 1; ++s2)
            if (m0 + s2 < G::SRI) row(tin, m0 + s2, win[s2]);
#pragma unroll
        for (int u = 0; u < R1; ++u) {
            const int m = m0 + u;
            if (m >= G::SRM) break;
            row(tin, m + 2 * RY, win[(u + 2 * RY) % WIN]);
            T o[V];
            apply4(win, u, o);
            store4<Cache::Default>(&mid[m][sc], 0, o);
        }
        /* the RX columns either side of the tile's own */
        if constexpr (RX > 0) {
            for (int i = threadIdx.x; i < G::SRM * 2 * RX; i += CTA) {
                const int m = i / (2 * RX), h = i - m * (2 * RX);
                const int c = h < RX ? G::HX - RX + h : G::HX + G::TW + (h - RX); /* tile column */
                T t[WIN][2 * RX + 1];
#pragma unroll
                for (int dy = 0; dy < WIN; ++dy)
#pragma unroll
                    for (int dx = 0; dx < 2 * RX + 1; ++dx) t[dy][dx] = tin[m + dy][c + dx - RX];
                mid[m][c] = Fn::apply(env, t);
            }
        }
    }
    __syncthreads();
    /* intermediate values at coordinates outside the array (tiles along the array's edges only): what the
     * boundary function makes of them */
    if (y0t - RY < 0 || y0t + G::RB + RY > H || x0t - RX < 0 || x0t + G::TW + RX > W) { /* the same for the whole block */
        constexpr int MW = G::TW + 2 * RX;
        for (int i = threadIdx.x; i < G::SRM * MW; i += CTA) {
            const int m = i / MW, cc = i - m * MW;
            const int y = y0t - RY + m, c = x0t - RX + cc;
            if (y >= 0 && y < H && c >= 0 && c < W) continue;
            if (y < -RY || y >= H + RY || c < -RX || c >= W + RX) continue; /* nothing reads it */
            const int yy = bound_coord(y, H, mode), xx = bound_coord(c, W, mode);
            /* the mapped coordinate is inside the array and inside this tile: computed above, never patched here */
            const bool inside = yy >= 0 && yy < H && xx >= 0 && xx < W;
            mid[m][cc + G::HX - RX] = inside ? mid[yy - (y0t - RY)][xx - (x0t - G::HX)] : src.cval;
        }
        __syncthreads();
    }

    /* ---- second application: as the tile form, out of the intermediate tile */
    const int x = x0t + tx * V;
    if (x >= W) return;
    T win[WIN][RW];
#pragma unroll
    for (int s2 = 0; s2 < WIN - 1; ++s2) row(mid, ty * G::RPT + s2, win[s2]);
    const bool vec_store = x + V <= W;
#pragma unroll
    for (int u = 0; u < G::RPT; ++u) {
        const int yo = y0t + ty * G::RPT + u;
        if (yo >= H) break;
        row(mid, ty * G::RPT + u + 2 * RY, win[(u + 2 * RY) % WIN]);
        T o[V];
        apply4(win, u, o);
        if (vec_store) {
            store4<Cache::Stream>(out + (long long)yo * W + x, 0, o);
        } else {
#pragma unroll
            for (int k = 0; k < V; ++k)
                if (x + k < W) out[(long long)yo * W + x + k] = o[k];
        }
    }
}

template <class Fn, int CTA>
__host__ __device__ constexpr bool stencil_tile2_ok() {
    return sizeof(typename Fn::in_t) == 4 && std::is_same<typename Fn::in_t, typename Fn::out_t>::value && 2 * Fn::RX <= 4;
}
template <class Fn, int CTA>
__device__ __forceinline__ void stencil_tile2_or_nothing(const accb_kparams &p) {
    if constexpr (stencil_tile2_ok<Fn, CTA>()) stencil_tile2_body<Fn, CTA>(p);
}
template <class Fn, int CTA>
__host__ __device__ constexpr int stencil_tile2_smem() {
    if constexpr (stencil_tile2_ok<Fn, CTA>())
        return StencilTile2<Fn, CTA>::kSmemBytes;
    else
        return 0;
}

/* ----------------------------------------------------------------------
 * Line form: rank-1 arrays.  A block's tile is a run of CTA * 4 * RPT
 * elements plus 4 halo elements each side, brought into shared memory by ONE
 * bulk copy per source; a warp then walks RPT rows of 128 consecutive
 * elements (lane l takes 4 of them), as in the scan.  Same conditions as the
 * tile form: 4-byte elements, aligned arrays, lengths that are multiples of 4.
 * ---------------------------------------------------------------------- */
#ifndef ACCB_STENCIL_LINE_RPT
#define ACCB_STENCIL_LINE_RPT 8
#endif
template <int CTA>
struct StencilLine {
    static constexpr int HX = 4;
    static constexpr int L = CTA * V * ACCB_STENCIL_LINE_RPT; /* outputs per tile */
    static constexpr int PW = L + 2 * HX;
};

template <class Fn, int NARR, int CTA>
__device__ __forceinline__ void stencil_line_body(const accb_kparams &p) {
    typedef typename Fn::in_t Tin;
    typedef typename Fn::out_t Tout;
    typedef StencilLine<CTA> G;
    static_assert(Fn::RY == 0 && Fn::RX <= G::HX, "line form: rank-1 stencil of radius at most 4");
    constexpr int RX = Fn::RX, RW = V + 2 * RX, RPT = ACCB_STENCIL_LINE_RPT;
    extern __shared__ __align__(128) unsigned char s_raw[];
    __shared__ __align__(8) unsigned long long s_bar;
    Tin(*tile)[G::PW] = reinterpret_cast<Tin(*)[G::PW]>(s_raw);

    const Env env(p);
    const int W = (int)p.ip[1], mode = (int)p.ip[4];
    Source<Tin> src[NARR];
#pragma unroll
    for (int a = 0; a < NARR; ++a) {
        src[a].base = static_cast<const Tin *>(p.in[a]);
        src[a].h = 1;
        src[a].w = (int)p.ip[6 + 2 * a];
        src[a].mode = mode;
        src[a].cval = env.scalar<Tin>(0);
        src[a].vec_ok = true;
    }
    Tout *out = static_cast<Tout *>(p.out[0]);
    unsigned int *err = static_cast<unsigned int *>(p.aux[1]);
    const long long x0t = (long long)blockIdx.x * G::L;
    auto col_range = [&](int a, long long &xs, long long &xe) {
        xs = max(0LL, x0t - G::HX);
        xe = min((long long)src[a].w, x0t + G::L + G::HX);
    };

    if (threadIdx.x == 0) {
        mbar_init(&s_bar, 1);
        fence_mbar_init();
        unsigned total = 0;
#pragma unroll
        for (int a = 0; a < NARR; ++a) {
            long long xs, xe;
            col_range(a, xs, xe);
            total += (unsigned)(xe - xs) * 4u;
        }
        mbar_expect_tx(&s_bar, total);
#pragma unroll
        for (int a = 0; a < NARR; ++a) {
            long long xs, xe;
            col_range(a, xs, xe);
            bulk_g2s(&tile[a][xs - (x0t - G::HX)], src[a].base + xs, (unsigned)(xe - xs) * 4u, &s_bar);
        }
    }
    __syncthreads(); /* the barrier is initialised before anybody polls it */
    int tries = 0;
    while (!mbar_try_wait(&s_bar, 0)) {
        if (++tries > ACCB_STENCIL_TMA_SPIN_LIMIT) { /* bounded: flag the result invalid and go on */
            atomicExch(err, 1u);
            break;
        }
    }
    /* halo elements outside the array: at most RX each side, first / last tile only */
    if (threadIdx.x < 2 * RX) {
#pragma unroll
        for (int a = 0; a < NARR; ++a) {
            long long xs, xe;
            col_range(a, xs, xe);
            const long long hi = min(x0t + G::L, (long long)W);
            const long long c = threadIdx.x < RX ? x0t - RX + threadIdx.x : hi + (threadIdx.x - RX);
            if (c < xs || c >= xe) tile[a][c - (x0t - G::HX)] = src[a].at(0, (int)c);
        }
    }
    __syncthreads();

    const int base = warp_id() * (RPT * 32 * V) + lane_id() * V;
#pragma unroll
    for (int j = 0; j < RPT; ++j) {
        const int e = base + j * 32 * V;
        const long long x = x0t + e;
        if (x >= W) break;
        Tout o[V];
        Tin d[NARR][RW];
#pragma unroll
        for (int a = 0; a < NARR; ++a) {
            const Tin *q = &tile[a][G::HX + e];
            Tin c[V];
            load4<Cache::Default>(q, 0, c);
#pragma unroll
            for (int k = 0; k < V; ++k) d[a][RX + k] = c[k];
#pragma unroll
            for (int k = 0; k < RX; ++k) {
                d[a][k] = q[k - RX];
                d[a][RX + V + k] = q[V + k];
            }
        }
#pragma unroll
        for (int k = 0; k < V; ++k) {
            Tin t[NARR][1][2 * RX + 1];
#pragma unroll
            for (int a = 0; a < NARR; ++a)
#pragma unroll
                for (int dx = 0; dx < 2 * RX + 1; ++dx) t[a][0][dx] = d[a][k + dx];
            if constexpr (NARR == 1)
                o[k] = Fn::apply(env, t[0]);
            else
                o[k] = Fn::apply(env, t[0], t[1]);
        }
        if (x + V <= W) {
            store4<Cache::Stream>(out + x, 0, o);
        } else {
#pragma unroll
            for (int k = 0; k < V; ++k)
                if (x + k < W) out[x + k] = o[k];
        }
    }
}

template <class Fn, int NARR, int CTA>
__device__ __forceinline__ void stencil_line_or_nothing(const accb_kparams &p) {
    if constexpr (sizeof(typename Fn::in_t) == 4 && sizeof(typename Fn::out_t) == 4 && Fn::RY == 0 && Fn::RX <= 4)
        stencil_line_body<Fn, NARR, CTA>(p);
}
/* outputs per tile of the line form; 0 when it does not apply */
template <class Fn, int CTA>
__host__ __device__ constexpr int stencil_line_len() {
    return (sizeof(typename Fn::in_t) == 4 && sizeof(typename Fn::out_t) == 4 && Fn::RY == 0 && Fn::RX <= 4)
               ? StencilLine<CTA>::L
               : 0;
}

/* element types the tile form does not take still need a body to instantiate */
template <class Fn, int NARR, int CTA>
__device__ __forceinline__ void stencil_tile_or_nothing(const accb_kparams &p) {
    if constexpr (sizeof(typename Fn::in_t) == 4 && sizeof(typename Fn::out_t) == 4 && Fn::RX <= 4)
        stencil_tile_body<Fn, NARR, CTA>(p);
}
/* which: 0 dynamic shared memory, 1 rows per tile, 2 columns per tile; 0 when the tile form does not apply */
template <class Fn, int NARR, int CTA>
__host__ __device__ constexpr int stencil_tile_dim(int which) {
    if constexpr (sizeof(typename Fn::in_t) == 4 && sizeof(typename Fn::out_t) == 4 && Fn::RX <= 4) {
        typedef StencilTile<Fn, NARR, CTA> G;
        return which == 0 ? G::kSmemBytes : (which == 1 ? G::RB : G::TW);
    } else {
        return 0;
    }
}

}  // namespace accb

/* Entry points: `stencil` / `stencil2` as in the reference (Stencil.hs:67,158)
 * are the register form, which takes any shape and element type; the host
 * launches `stencil_tile` / `stencil2_tile` (rank 2) or `stencil_line` /
 * `stencil2_line` (rank 1) instead when their conditions hold.
 * Metadata: {.., element bytes, rows per tile, columns per tile, outputs per
 * tile of the line form, dynamic shared memory of the tile form, rows the stencil reaches up and down,
 * dynamic shared memory of the two-application form (0: not available), its rows per tile}. */
#define ACCB_STENCIL_ENTRIES(Fn, id, narr, name, tname, lname)                                 \
    ACCB_META12(id, ACCB_STENCIL_CTA, sizeof(Fn::in_t),                                        \
                (accb::stencil_tile_dim<Fn, narr, ACCB_STENCIL_CTA>(1)),                       \
                (accb::stencil_tile_dim<Fn, narr, ACCB_STENCIL_CTA>(2)),                       \
                (accb::stencil_line_len<Fn, ACCB_STENCIL_CTA>()),                              \
                (accb::stencil_tile_dim<Fn, narr, ACCB_STENCIL_CTA>(0)), Fn::RY,               \
                ((narr) == 1 ? accb::stencil_tile2_smem<Fn, ACCB_STENCIL_CTA>() : 0),          \
                (ACCB_STENCIL_CTA / 64 * ACCB_STENCIL_TILE2_RPT), 0, 0)                        \
    extern "C" __global__ void __launch_bounds__(ACCB_STENCIL_CTA, ACCB_STENCIL_MINB)          \
        name(const __grid_constant__ accb_kparams p) {                                         \
        accb::stencil_body<Fn, narr, ACCB_STENCIL_CTA>(p);                                     \
    }                                                                                          \
    extern "C" __global__ void __launch_bounds__(ACCB_STENCIL_CTA, ACCB_STENCIL_TILE_MINB_FOR(Fn, narr)) \
        tname(const __grid_constant__ accb_kparams p) {                                        \
        accb::stencil_tile_or_nothing<Fn, narr, ACCB_STENCIL_CTA>(p);                          \
    }                                                                                          \
    extern "C" __global__ void __launch_bounds__(ACCB_STENCIL_CTA, 6)                          \
        lname(const __grid_constant__ accb_kparams p) {                                        \
        accb::stencil_line_or_nothing<Fn, narr, ACCB_STENCIL_CTA>(p);                          \
    }

#define ACCB_INSTANTIATE_STENCIL(Fn)                                                           \
    ACCB_STENCIL_ENTRIES(Fn, 8, 1, stencil, stencil_tile, stencil_line)                        \
    extern "C" __global__ void __launch_bounds__(ACCB_STENCIL_CTA, ACCB_STENCIL_TILE2_MINB)    \
        stencil_tile2(const __grid_constant__ accb_kparams p) {                                \
        accb::stencil_tile2_or_nothing<Fn, ACCB_STENCIL_CTA>(p);                               \
    }
#define ACCB_INSTANTIATE_STENCIL2(Fn) ACCB_STENCIL_ENTRIES(Fn, 9, 2, stencil2, stencil2_tile, stencil2_line)
