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
 * Here each thread owns 4 adjacent columns and walks down a band of rows
 * keeping the (2*RY+1) x (4+2*RX) window in registers: per output row it
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

#ifndef ACCB_STENCIL_CTA
#define ACCB_STENCIL_CTA 256
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

/* Load this thread's piece of row y (raw index) of `src`: the 4 centre columns
 * x0..x0+3 in r[RX..RX+3], halos in r[0..RX) and r[RX+4..]. */
template <class T, int RX>
__device__ __forceinline__ void load_row(const Source<T> &s, int y, int x0, T (&r)[4 + 2 * RX]) {
    const int yy = bound_coord(y, s.h, s.mode);
    T c[V];
    const bool inside = x0 + V <= s.w;
    if (yy >= 0 && inside && s.vec_ok) {
        load4<Cache::Default>(s.base, ((long long)yy * s.w + x0) / V, c);
    } else {
#pragma unroll
        for (int k = 0; k < V; ++k) c[k] = x0 < s.w ? s.at(yy, x0 + k) : s.cval;
    }
#pragma unroll
    for (int k = 0; k < V; ++k) r[RX + k] = c[k];
    if constexpr (RX > 0) {
        const int lane = lane_id();
        /* neighbours' centre vectors; every lane takes part in the shuffles */
        T lf[RX], rt[RX];
#pragma unroll
        for (int d = 0; d < RX; ++d) {
            lf[d] = shfl_up(c[V - RX + d], 1);   /* columns x0-RX+d */
            rt[d] = shfl_down(c[d], 1);          /* columns x0+4+d */
        }
        const bool l_ok = lane > 0 && x0 > 0;
        const bool r_ok = lane < 31 && x0 + 2 * V <= s.w;
        if (x0 < s.w) {
#pragma unroll
            for (int d = 0; d < RX; ++d) {
                r[d] = l_ok ? lf[d] : s.at(yy, x0 - RX + d);
                r[RX + V + d] = r_ok ? rt[d] : s.at(yy, x0 + V + d);
            }
        }
    }
}

template <class Fn, int NARR, int CTA>
__device__ __forceinline__ void stencil_body(const accb_kparams &p) {
    typedef typename Fn::in_t Tin;
    typedef typename Fn::out_t Tout;
    constexpr int RY = Fn::RY, RX = Fn::RX;
    constexpr int WIN = 2 * RY + 1;
    constexpr int RW = 4 + 2 * RX;
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
        const int y_begin = (band * TY + ty) * RB;
        const int y_end = min(H, y_begin + RB);
        if (y_begin >= H) continue; /* whole warps share ty, so a warp leaves together */

        Tin win[NARR][WIN][RW];
        /* preload rows y_begin-RY .. y_begin+RY-1 into slots 0 .. 2RY-1 */
#pragma unroll
        for (int a = 0; a < NARR; ++a)
#pragma unroll
            for (int s = 0; s < WIN - 1; ++s) load_row<Tin, RX>(src[a], y_begin - RY + s, x0, win[a][s]);

        for (int y = y_begin; y < y_end; y += WIN) {
#pragma unroll
            for (int s = 0; s < WIN; ++s) {
                const int yo = y + s; /* output row; (yo - y_begin) % WIN == s */
                if (yo < y_end) {
                    /* newest row yo+RY goes to slot (s + 2RY) % WIN */
#pragma unroll
                    for (int a = 0; a < NARR; ++a)
                        load_row<Tin, RX>(src[a], yo + RY, x0, win[a][(s + 2 * RY) % WIN]);
                    if (x0 < W) {
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
                        if (out_vec && x0 + V <= W) {
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
}

}  // namespace accb

/* Entry points named after the reference's kernels (Stencil.hs:67,158). */
#define ACCB_INSTANTIATE_STENCIL(Fn)                                                           \
    ACCB_META(8, ACCB_STENCIL_CTA, sizeof(Fn::in_t), 0, 1, 0)                                  \
    extern "C" __global__ void __launch_bounds__(ACCB_STENCIL_CTA)                             \
        stencil(const __grid_constant__ accb_kparams p) {                                      \
        accb::stencil_body<Fn, 1, ACCB_STENCIL_CTA>(p);                                        \
    }

#define ACCB_INSTANTIATE_STENCIL2(Fn)                                                          \
    ACCB_META(9, ACCB_STENCIL_CTA, sizeof(Fn::in_t), 0, 1, 0)                                  \
    extern "C" __global__ void __launch_bounds__(ACCB_STENCIL_CTA)                             \
        stencil2(const __grid_constant__ accb_kparams p) {                                     \
        accb::stencil_body<Fn, 2, ACCB_STENCIL_CTA>(p);                                        \
    }
