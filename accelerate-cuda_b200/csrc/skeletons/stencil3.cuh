/*
 * stencil3.cuh -- stencil over rank-3 arrays (cubes) with Clamp / Mirror /
 * Wrap / Constant boundaries.
 *
 * The reference's mkStencil is rank-polymorphic
 * (Data/Array/Accelerate/CUDA/CodeGen/Stencil.hs:55-114): whatever the rank,
 * every output point gathers all its taps from global memory through
 * stencilAccess (CodeGen/Stencil/Extra.hs:53-128), i.e. 27 loads with three
 * boundary tests each for a 3x3x3 neighbourhood.  Here a block owns a column
 * of the cube -- TY x TX points in (y, x), a run of planes in z -- and marches
 * along z: the 2*RZ+1 input planes a z-step needs sit in a ring of tiles in
 * shared memory, every z-step brings in ONE new plane tile (with its halo in
 * y and x) and retires the oldest, so an input element is requested from
 * memory once per block that needs it instead of once per tap.  The new
 * plane is fetched with asynchronous 16-byte copies (cp.async) one z-step
 * ahead, into a spare slot of the ring, while the current step is computed.
 * The threads of a warp read and write 512 contiguous bytes per row; a thread
 * computes 4 adjacent x per row from 16-byte shared-memory reads, its halo
 * columns handed over by the neighbouring lanes.
 *
 * Tried and dropped: a thread that owns one row for the whole run and keeps
 * the 2*RZ+1 planes of its neighbourhood in registers, reading only the new
 * plane per z-step.  Shared-memory traffic fell to a third (ncu: l1tex 84 % ->
 * 30 % busy), the time did not (0.56 ms against 0.45 ms on 512^3): a 3x3x3
 * window of 54 values plus the functor's temporaries spill at three blocks per
 * SM, and with one row per warp and step the blocks spend their time at the
 * barrier.  The kernel is bound by instruction issue (27 multiply-adds per
 * output for a full 3x3x3 functor), not by shared memory or DRAM.
 *
 * Boundary semantics as for the lower ranks (Extra.hs:200-226): every
 * coordinate is mapped on its own; with Constant the whole tap is the constant
 * as soon as one coordinate is outside (:122-128,191-196).  The mapping is
 * done once, when a plane tile is filled, not per tap.
 *
 * Functor contract (derive from accb::Stencil3<Tin, Tout, RZ, RY, RX>; 4-byte
 * Tin):
 *   static Tout apply(env, const Tin (&t)[2*RZ+1][2*RY+1][2*RX+1]);
 *   static constexpr bool uses(int dz, int dy, int dx);   optional: the taps apply() reads (default: all)
 * with t[dz][dy][dx] the element at offset (dz-RZ, dy-RY, dx-RX), the order
 * in which Accelerate's stencil patterns nest (outermost dimension first); taps that uses() denies read as zero.
 *
 *   in[0] source, out[0] result; ip[0] D, ip[1] H, ip[2] W (planes, rows,
 *   columns); ip[3] planes per block; ip[4] boundary; scalars[0..] the constant.
 */
#pragma once
#include "../cubits/accb_vec.cuh"
#include "../cubits/accb_warp.cuh"
#include "../cubits/accb_tma.cuh"
#include "stencil.cuh"

#ifndef ACCB_STENCIL3_CTA
#define ACCB_STENCIL3_CTA 256
#endif
#ifndef ACCB_STENCIL3_TY
#define ACCB_STENCIL3_TY 32 /* rows of a block's column: four per warp (512^3, 27 taps: 0.45 ms against 0.53 ms with 16) */
#endif
#define ACCB_STENCIL3_TX 128 /* columns of a block's column: one warp row */
#ifndef ACCB_STENCIL3_AHEAD
#define ACCB_STENCIL3_AHEAD 1 /* z-steps between the request for a plane and its first use.  Two or three steps cost a
                                 resident block per SM and bought nothing (512^3, 7-point: 0.335 ms at one step, 0.42 ms
                                 at two or three; with 16-row tiles 0.37-0.40 ms at one to three) */
#endif
#ifndef ACCB_STENCIL3_MINB
#define ACCB_STENCIL3_MINB 3 /* resident blocks per SM the compiler must leave registers for */
#endif

namespace accb {

template <class Tin, class Tout, int RZ_, int RY_, int RX_>
struct Stencil3 {
    typedef Tin in_t;
    typedef Tout out_t;
    static constexpr int RZ = RZ_, RY = RY_, RX = RX_;
    /* does apply() read t[dz][dy][dx]?  A functor that reads only some taps (a 7-point Laplacian reads 7 of 27) says
     * so by overriding this, and the rows and halo columns nobody reads are then neither loaded nor shuffled (a
     * warp shuffle whose result is unused is not removed by the compiler). */
    static constexpr bool uses(int, int, int) { return true; }
};

/* which parts of row (DZ, DY) of the neighbourhood a functor needs */
template <class Fn, int DZ, int DY>
struct Stencil3Row {
    static constexpr bool some(int lo, int hi) {
        for (int dx = lo; dx < hi; ++dx)
            if (Fn::uses(DZ, DY, dx)) return true;
        return false;
    }
    static constexpr bool any = some(0, 2 * Fn::RX + 1);
    static constexpr bool left = some(0, Fn::RX);                  /* columns left of the thread's own four */
    static constexpr bool right = some(Fn::RX + 1, 2 * Fn::RX + 1); /* columns right of them */
};

/* geometry of one plane tile in shared memory: TY + 2*RY rows of PITCH values; the TX centre columns start
 * at value PAD (a multiple of 4, so that a thread's 4 columns are one aligned 16-byte read) */
template <class Fn>
struct Stencil3Tile {
    static constexpr int TY = ACCB_STENCIL3_TY, TX = ACCB_STENCIL3_TX;
    static constexpr int PAD = (Fn::RX + 3) / 4 * 4;
    static constexpr int PITCH = TX + 2 * PAD;
    static constexpr int ROWS = TY + 2 * Fn::RY;
    static constexpr int PLANE = ROWS * PITCH;     /* values per plane tile */
    static constexpr int AHEAD = ACCB_STENCIL3_AHEAD;
    static constexpr int RING = 2 * Fn::RZ + 1 + AHEAD; /* plane tiles resident: the 2*RZ+1 in use and those on their way */
    static constexpr int BYTES = RING * PLANE * 4;
};

/* Fill one plane tile: input plane `z` (already mapped through the boundary, or -1: all constant), rows
 * y0 - RY .. y0 + TY + RY - 1, columns x0 - PAD .. x0 + TX + PAD - 1 (only RX of the PAD columns are used). */
template <class Fn, int CTA>
__device__ __forceinline__ void stencil3_fill(typename Fn::in_t *tile, const typename Fn::in_t *src, int zz, int y0, int x0,
                                              int H, int W, int mode, typename Fn::in_t cval, bool vec_ok) {
    typedef typename Fn::in_t T;
    typedef Stencil3Tile<Fn> G;
    const T *plane = src + (long long)(zz < 0 ? 0 : zz) * H * W;
    /* centre columns: 16-byte loads where the whole vector is inside the row and aligned.  A thread keeps its
     * column of vectors and walks down the rows, CTA / VPR of them per pass */
    constexpr int VPR = G::TX / 4; /* vectors per row */
    static_assert(CTA % VPR == 0, "whole rows of vectors per pass");
    constexpr int RPP = CTA / VPR;
    const int v = threadIdx.x % VPR;
    const int x = x0 + 4 * v;
    const bool whole = zz >= 0 && vec_ok && x + 3 < W;
    T *dst = tile + (threadIdx.x / VPR) * G::PITCH + G::PAD + 4 * v;
    if (whole && y0 - Fn::RY >= 0 && y0 - Fn::RY + G::ROWS <= H) {
        /* all rows of the tile are rows of the cube (every tile but those along two faces): no boundary map */
        const T *from = plane + (long long)(y0 - Fn::RY + (int)(threadIdx.x / VPR)) * W + x;
        for (int r = threadIdx.x / VPR; r < G::ROWS; r += RPP, dst += RPP * G::PITCH, from += (long long)RPP * W)
            asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(smem_addr(dst)), "l"(from) : "memory");
    } else {
        for (int r = threadIdx.x / VPR; r < G::ROWS; r += RPP, dst += RPP * G::PITCH) {
            const int yy = bound_coord(y0 - Fn::RY + r, H, mode);
            if (whole && yy >= 0) {
                /* asynchronous: no register holds the data, the caller waits for the group before the tile is read */
                asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(smem_addr(dst)), "l"(plane + (long long)yy * W + x)
                             : "memory");
            } else {
#pragma unroll
                for (int k = 0; k < 4; ++k) {
                    const int xx = bound_coord(x + k, W, mode);
                    dst[k] = (zz < 0 || yy < 0 || xx < 0) ? cval : plane[(long long)yy * W + xx];
                }
            }
        }
    }
    /* halo columns, RX on either side */
    if constexpr (Fn::RX > 0) {
        for (int i = threadIdx.x; i < G::ROWS * 2 * Fn::RX; i += CTA) {
            const int r = i / (2 * Fn::RX), h = i - r * (2 * Fn::RX);
            const int dx = h < Fn::RX ? h - Fn::RX : G::TX + (h - Fn::RX); /* relative to x0 */
            const int yy = bound_coord(y0 - Fn::RY + r, H, mode);
            const int xx = bound_coord(x0 + dx, W, mode);
            tile[r * G::PITCH + G::PAD + dx] = (zz < 0 || yy < 0 || xx < 0) ? cval : plane[(long long)yy * W + xx];
        }
    }
}

/* Row (DZ, DY) of a thread's window: its own 4 columns by one 16-byte read, the RX halo columns either side from
 * the neighbouring lanes' centre columns by shuffles (instead of 4-byte reads 16 bytes apart: a four-way bank
 * conflict each); the two lanes at the ends of the row take the tile's own halo, which every lane reads from the
 * same address (a broadcast).  Parts the functor does not read are skipped. */
template <class Fn, int DZ, int DY>
__device__ __forceinline__ void stencil3_row(const typename Fn::in_t *ring, int at, int lane,
                                             typename Fn::in_t (&w)[4 + 2 * Fn::RX]) {
    typedef typename Fn::in_t T;
    typedef Stencil3Tile<Fn> G;
    typedef Stencil3Row<Fn, DZ, DY> R;
    constexpr int RX = Fn::RX;
    if constexpr (R::any) {
        const T *trow = ring + at + DY * G::PITCH; /* column x0 of this tile row; `at`: column x0 of window row 0 */
        const uint4 c = *reinterpret_cast<const uint4 *>(trow + 4 * lane);
        memcpy(&w[RX], &c, 16);
        if constexpr (R::left) {
#pragma unroll
            for (int h = 0; h < RX; ++h) {
                const T from_left = shfl_up(w[4 + h], 1); /* lane - 1's last RX columns */
                const T tile_left = trow[h - RX];
                w[h] = lane == 0 ? tile_left : from_left;
            }
        }
        if constexpr (R::right) {
#pragma unroll
            for (int h = 0; h < RX; ++h) {
                const T from_right = shfl_down(w[RX + h], 1); /* lane + 1's first RX columns */
                const T tile_right = trow[G::TX + h];
                w[RX + 4 + h] = lane == 31 ? tile_right : from_right;
            }
        }
    }
}
/* all rows of a thread's window: planes[dz] is where the plane tile of input plane z + dz - RZ starts in the ring,
 * row the offset of column x0 of the window's first row inside a plane tile (both worked out once, not per row) */
template <class Fn, int... ZY>
__device__ __forceinline__ void stencil3_window(const typename Fn::in_t *ring, const int (&planes)[2 * Fn::RZ + 1], int row, int lane,
                                                typename Fn::in_t (&win)[2 * Fn::RZ + 1][2 * Fn::RY + 1][4 + 2 * Fn::RX],
                                                std::integer_sequence<int, ZY...>) {
    constexpr int NY = 2 * Fn::RY + 1;
    (stencil3_row<Fn, ZY / NY, ZY % NY>(ring, planes[ZY / NY] + row, lane, win[ZY / NY][ZY % NY]), ...);
}

template <class Fn, int CTA>
__device__ __forceinline__ void stencil3_body(const accb_kparams &p) {
    typedef typename Fn::in_t T;
    typedef typename Fn::out_t U;
    typedef Stencil3Tile<Fn> G;
    static_assert(sizeof(T) == 4, "the rank-3 stencil skeleton stages 4-byte elements");
    static_assert(CTA == 256 && G::TX == 128, "eight warps, one row of 128 columns per warp and step");
    constexpr int RZ = Fn::RZ, RY = Fn::RY, RX = Fn::RX;
    extern __shared__ __align__(16) unsigned char s_raw[];
    T *ring = reinterpret_cast<T *>(s_raw);
    const Env env(p);
    const int D = (int)p.ip[0], H = (int)p.ip[1], W = (int)p.ip[2];
    const int zrun = (int)p.ip[3], mode = (int)p.ip[4];
    const T *src = static_cast<const T *>(p.in[0]);
    U *out = static_cast<U *>(p.out[0]);
    const T cval = mode == B_CONSTANT ? env.scalar<T>(0) : T();
    const bool vec_ok = (p.flags & ACCB_F_VEC) != 0 && W % 4 == 0;

    const int tiles_x = (W + G::TX - 1) / G::TX, tiles_y = (H + G::TY - 1) / G::TY;
    const int zchunks = (D + zrun - 1) / zrun;
    const long long ntask = (long long)tiles_x * tiles_y * zchunks;
    const int lane = lane_id(), w = warp_id();

    /* plane z of the cube lives in ring slot (z + RZ) mod RING (z >= -RZ) */
    auto slot = [&](int z) { return ring + ((z + RZ) % G::RING) * G::PLANE; };
    auto fetch = [&](int z, int y0, int x0) {
        stencil3_fill<Fn, CTA>(slot(z), src, bound_coord(z, D, mode), y0, x0, H, W, mode, cval, vec_ok);
        asm volatile("cp.async.commit_group;" ::: "memory");
    };

    for (long long task = blockIdx.x; task < ntask; task += gridDim.x) {
        /* x fastest, then y, then the z-chunk: blocks that run together share halo rows and planes in L2 */
        const int tx = (int)(task % tiles_x);
        const int ty = (int)((task / tiles_x) % tiles_y);
        const int tz = (int)(task / ((long long)tiles_x * tiles_y));
        const int x0 = tx * G::TX, y0 = ty * G::TY, z0 = tz * zrun;
        const int z1 = min(D, z0 + zrun);
        __syncthreads(); /* the previous task's last reads of the ring */
        /* planes z0 - RZ .. z0 + RZ are needed by the first step; AHEAD - 1 more are requested with them.  One
         * group of copies per plane, also for planes beyond the run (empty groups keep the count below exact) */
        for (int dz = -RZ; dz <= RZ + G::AHEAD - 1; ++dz) {
            if (dz <= RZ || z0 + dz - RZ < z1)
                fetch(z0 + dz, y0, x0);
            else
                asm volatile("cp.async.commit_group;" ::: "memory");
        }
        for (int z = z0; z < z1; ++z) {
            /* all but the newest AHEAD - 1 planes have landed; then start on the plane that step z + AHEAD adds,
             * into the slot that the step before this one read last */
            asm volatile("cp.async.wait_group %0;" ::"n"(G::AHEAD - 1) : "memory");
            __syncthreads();
            if (z + G::AHEAD < z1)
                fetch(z + G::AHEAD + RZ, y0, x0);
            else
                asm volatile("cp.async.commit_group;" ::: "memory");
            int planes[2 * RZ + 1]; /* input plane z + dz - RZ lives in ring slot (z + dz) mod RING */
#pragma unroll
            for (int dz = 0; dz <= 2 * RZ; ++dz) planes[dz] = (int)((unsigned)(z + dz) % (unsigned)G::RING) * G::PLANE;
            U *zout = out + (long long)z * H * W;
            /* warp w computes rows w, w + 8, ..: lane l the columns 4l .. 4l + 3 */
            for (int r = w; r < G::TY; r += CTA / 32) {
                const int y = y0 + r, x = x0 + 4 * lane;
                if (y < H) { /* the same for every lane of the warp: the shuffles below see all 32 */
                    T win[2 * RZ + 1][2 * RY + 1][4 + 2 * RX] = {};
                    stencil3_window<Fn>(ring, planes, r * G::PITCH + G::PAD, lane, win,
                                        std::make_integer_sequence<int, (2 * RZ + 1) * (2 * RY + 1)>());
                    U o[4];
#pragma unroll
                    for (int k = 0; k < 4; ++k) {
                        T t[2 * RZ + 1][2 * RY + 1][2 * RX + 1];
#pragma unroll
                        for (int dz = 0; dz <= 2 * RZ; ++dz)
#pragma unroll
                            for (int dy = 0; dy <= 2 * RY; ++dy)
#pragma unroll
                                for (int dx = 0; dx <= 2 * RX; ++dx) t[dz][dy][dx] = win[dz][dy][k + dx];
                        o[k] = Fn::apply(env, t);
                    }
                    U *dst = zout + (long long)y * W + x;
                    if (x >= W) {
                        /* beyond the last column: nothing to store */
                    } else if (vec_ok && sizeof(U) == 4 && x + 3 < W) {
                        uint4 q;
                        memcpy(&q, o, 16);
                        __stcs(reinterpret_cast<uint4 *>(dst), q);
                    } else {
#pragma unroll
                        for (int k = 0; k < 4; ++k)
                            if (x + k < W) dst[k] = o[k];
                    }
                }
            }
        }
    }
    asm volatile("cp.async.wait_group 0;" ::: "memory");
}

}  // namespace accb

/* metadata: element bytes, tile rows, tile columns, -, dynamic shared memory, 2*RZ */
#define ACCB_INSTANTIATE_STENCIL3(Fn)                                                          \
    ACCB_META7(10, ACCB_STENCIL3_CTA, sizeof(Fn::in_t), ACCB_STENCIL3_TY, ACCB_STENCIL3_TX, 2 * Fn::RZ, \
               accb::Stencil3Tile<Fn>::BYTES)                                                  \
    extern "C" __global__ void __launch_bounds__(ACCB_STENCIL3_CTA, ACCB_STENCIL3_MINB)        \
        stencil3(const __grid_constant__ accb_kparams p) {                                     \
        accb::stencil3_body<Fn, ACCB_STENCIL3_CTA>(p);                                         \
    }
