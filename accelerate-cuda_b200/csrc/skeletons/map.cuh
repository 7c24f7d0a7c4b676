/*
 * map.cuh -- element-wise skeletons: map / zipWith / generate / transform
 * (backpermute).
 *
 * Replaces the kernels made by mkMap
 * (Data/Array/Accelerate/CUDA/CodeGen/Mapping.hs:39-78), mkGenerate and
 * mkTransform (CodeGen/IndexSpace.hs:47-141) and their host driver executeOp
 * (Execute.hs:264-268).  One kernel covers all of them because in every case
 * the result at linear index i is a function of i and of the environment:
 *
 *   struct Fn {
 *     using In  = accb::types<...>;  // components read at the SAME linear index i
 *                                    // (slots 0..In::size-1 of the environment)
 *     using Out = accb::types<...>;  // components of the result
 *     static __device__ void apply(const accb::Env&, long long i,
 *                                  in-values..., out-references...);
 *   };
 *
 * `In` lists what the fused producer reads element-wise (map over a zip of
 * manifest arrays); those loads are 128-bit and streaming.  A producer that
 * gathers (backpermute, generate from an index) leaves `In` empty and reads
 * the environment through `env.in<T>(slot)[j]` itself.
 *
 * Work distribution: a persistent grid of SMs x resident blocks; a block
 * takes CTA*U vectors (CTA*U*4 elements) per trip with all U loads per input
 * issued before the first use, so each thread keeps U*In::size 16-byte loads
 * in flight.
 */
#pragma once
#include "../cubits/accb_vec.cuh"
#include "../cubits/accb_tma.cuh"

namespace accb {

template <class Fn, int N, int... I, int... O>
__device__ __forceinline__ void map_apply(const Env &env, long long i0, regs<N, typename Fn::In> &a,
                                          regs<N, typename Fn::Out> &b, std::integer_sequence<int, I...>,
                                          std::integer_sequence<int, O...>) {
#pragma unroll
    for (int k = 0; k < N; ++k) Fn::apply(env, env.p.base + i0 + k, comp<I>(a)[k]..., comp<O>(b)[k]...);
}

template <class Fn, int CTA, int U>
__device__ __forceinline__ void map_body(const accb_kparams &p) {
    typedef typename Fn::In In;
    typedef typename Fn::Out Out;
    const Env env(p);
    const auto iseq = std::make_integer_sequence<int, In::size>();
    const auto oseq = std::make_integer_sequence<int, Out::size>();
    const long long n = p.n;
    const long long nvec = (p.flags & ACCB_F_VEC) ? n / V : 0;
    constexpr long long TRIP = (long long)CTA * U;
    const long long ntrip = nvec / TRIP; /* trips made of full vectors only */

    for (long long t = blockIdx.x; t < ntrip; t += gridDim.x) {
        const long long v0 = t * TRIP + threadIdx.x;
        regs<V, In> a[U];
        regs<V, Out> b[U];
#pragma unroll
        for (int u = 0; u < U; ++u) load_all(p.in, v0 + (long long)u * CTA, a[u]);
#pragma unroll
        for (int u = 0; u < U; ++u) {
            map_apply<Fn>(env, (v0 + (long long)u * CTA) * V, a[u], b[u], iseq, oseq);
            store_all(p.out, v0 + (long long)u * CTA, b[u]);
        }
    }
    /* leftover full vectors */
    for (long long v = ntrip * TRIP + (long long)blockIdx.x * CTA + threadIdx.x; v < nvec;
         v += (long long)gridDim.x * CTA) {
        regs<V, In> a;
        regs<V, Out> b;
        load_all(p.in, v, a);
        map_apply<Fn>(env, v * V, a, b, iseq, oseq);
        store_all(p.out, v, b);
    }
    /* ragged tail, or everything when an array is not 16-byte aligned */
    for (long long i = nvec * V + (long long)blockIdx.x * CTA + threadIdx.x; i < n;
         i += (long long)gridDim.x * CTA) {
        regs<1, In> a;
        regs<1, Out> b;
        load_one(p.in, i, a);
        map_apply<Fn>(env, i, a, b, iseq, oseq);
        store_one(p.out, i, b);
    }
}

/* ----------------------------------------------------------------------
 * map over a TRANSPOSED matrix: `map f (transpose m)`.  Through the generic
 * kernel a transpose is a gather whose reads are a whole row apart between
 * neighbouring threads (the reference's backpermute, IndexSpace.hs:96-141, has
 * the same access pattern).  Here the element-wise inputs -- matrices of
 * ip[0] rows and ip[1] columns -- go through shared memory in tiles of 64x64:
 * read along their rows with 16-byte loads, handed to the functor along their
 * columns four at a time, so that loads and stores are both contiguous
 * vectors.  Ragged edge tiles and unaligned arrays take scalar accesses.  The functor is the one of the plain
 * map: apply(env, i, in-values..., out-references...) with i the OUTPUT
 * position, in an array of ip[1] rows and ip[0] columns.
 * ---------------------------------------------------------------------- */
#ifndef ACCB_TRANS_TILE_4B
#define ACCB_TRANS_TILE_4B 64 /* tile edge when every element-wise input is 4 bytes wide (64 or 128) */
#endif
constexpr int kTransTileAny = 64; /* tile edge otherwise */

template <class L, int... I>
__host__ __device__ constexpr bool trans_all4(std::integer_sequence<int, I...>) {
    return ((sizeof(typename type_at<I, L>::type) == 4) && ...);
}
/* tile edge in elements; the scalar layout pads every row by one element (odd pitch: the columns of a tile fall
 * into different banks) and the vector layout below fits into the same space */
template <class L>
__host__ __device__ constexpr int trans_tile() {
    return trans_all4<L>(std::make_integer_sequence<int, L::size>()) ? ACCB_TRANS_TILE_4B : kTransTileAny;
}
template <class L>
__host__ __device__ constexpr int trans_elems() {
    return trans_tile<L>() * (trans_tile<L>() + 1);
}

template <class L, int I>
__device__ __forceinline__ typename type_at<I, L>::type *trans_plane(unsigned char *s) {
    return reinterpret_cast<typename type_at<I, L>::type *>(s + smem_offset<L, I, trans_elems<L>()>::value);
}
/* N consecutive elements of every component into row `row` of the tile, from column `col` */
template <class L, int N, int... I>
__device__ __forceinline__ void trans_put(unsigned char *s, int row, int col, regs<N, L> &r,
                                          std::integer_sequence<int, I...>) {
#pragma unroll
    for (int k = 0; k < N; ++k) ((trans_plane<L, I>(s)[row * (trans_tile<L>() + 1) + col + k] = comp<I>(r)[k]), ...);
}
/* N elements of every component down column `col` of the tile, from row `row` */
template <class L, int N, int... I>
__device__ __forceinline__ void trans_take(unsigned char *s, int row, int col, regs<N, L> &r,
                                           std::integer_sequence<int, I...>) {
#pragma unroll
    for (int k = 0; k < N; ++k) ((comp<I>(r)[k] = trans_plane<L, I>(s)[(row + k) * (trans_tile<L>() + 1) + col]), ...);
}

/* Tiles of 4-byte components take a second layout, in which every shared-memory access is a 16-byte vector: a
 * thread that holds a 4x4 block (four consecutive rows, four consecutive columns) transposes it in registers and
 * stores each column piece as one vector into the TRANSPOSED tile (row = source column, T/4 vectors of 4 source
 * rows each); the result rows are then read back as vectors.  Vector j of row c sits at position j ^ ((c >> 2) & 7),
 * which spreads the eight lanes of a quarter warp over all banks both when they store (consecutive column
 * groups, one row group) and when they load (one row, consecutive vectors).  With scalar accesses the kernel
 * spent its time waiting for the shared-memory instruction queue (32 instructions per thread and tile, half of
 * them replayed for bank conflicts). */
template <class E>
__device__ __forceinline__ unsigned trans_bits(E v) {
    return *reinterpret_cast<const unsigned *>(&v);
}
template <class E>
__device__ __forceinline__ E trans_unbits(unsigned u) {
    return *reinterpret_cast<const E *>(&u);
}
/* the 4x4 block of row group `j` and column group `tx` */
template <class L, int I>
__device__ __forceinline__ void trans_put4_one(unsigned char *s, int j, int tx, regs<V, L> (&a)[4]) {
    uint4 *plane = reinterpret_cast<uint4 *>(trans_plane<L, I>(s));
#pragma unroll
    for (int k = 0; k < 4; ++k) {
        uint4 w;
        w.x = trans_bits(comp<I>(a[0])[k]);
        w.y = trans_bits(comp<I>(a[1])[k]);
        w.z = trans_bits(comp<I>(a[2])[k]);
        w.w = trans_bits(comp<I>(a[3])[k]);
        plane[(4 * tx + k) * (trans_tile<L>() / 4) + (j ^ (tx & 7))] = w;
    }
}
template <class L, int... I>
__device__ __forceinline__ void trans_put4(unsigned char *s, int j, int tx, regs<V, L> (&a)[4],
                                           std::integer_sequence<int, I...>) {
    (trans_put4_one<L, I>(s, j, tx, a), ...);
}
template <class L, int I>
__device__ __forceinline__ void trans_take4_one(unsigned char *s, int r, int tx, regs<V, L> &c) {
    typedef typename type_at<I, L>::type E;
    const uint4 w =
        reinterpret_cast<const uint4 *>(trans_plane<L, I>(s))[r * (trans_tile<L>() / 4) + (tx ^ ((r >> 2) & 7))];
    comp<I>(c)[0] = trans_unbits<E>(w.x);
    comp<I>(c)[1] = trans_unbits<E>(w.y);
    comp<I>(c)[2] = trans_unbits<E>(w.z);
    comp<I>(c)[3] = trans_unbits<E>(w.w);
}
template <class L, int... I>
__device__ __forceinline__ void trans_take4(unsigned char *s, int r, int tx, regs<V, L> &c, std::integer_sequence<int, I...>) {
    (trans_take4_one<L, I>(s, r, tx, c), ...);
}

template <class Fn, int CTA>
__device__ __forceinline__ void map_transposed_body(const accb_kparams &p) {
    typedef typename Fn::In In;
    typedef typename Fn::Out Out;
    constexpr int T = trans_tile<In>(), VX = T / V, RY = CTA / VX; /* threads along a row, rows per pass */
    /* all components 4 bytes wide and 4-element vectors: the all-vector tile layout, T/4 x T/4 blocks of 4x4 */
    constexpr bool fast = trans_all4<In>(std::make_integer_sequence<int, In::size>()) && V == 4 && (T / 4) % RY == 0;
    extern __shared__ __align__(128) unsigned char s_tile[];
    const Env env(p);
    const auto iseq = std::make_integer_sequence<int, In::size>();
    const auto oseq = std::make_integer_sequence<int, Out::size>();
    const int H = (int)p.ip[0], W = (int)p.ip[1]; /* of the sources; the result has W rows of H columns */
    const int tx = threadIdx.x % VX, ty = threadIdx.x / VX;
    const bool vec = (p.flags & ACCB_F_VEC) != 0 && W % V == 0 && H % V == 0;
    const long long tiles_x = (W + T - 1) / T, tiles_y = (H + T - 1) / T;
    for (long long t = blockIdx.x; t < tiles_x * tiles_y; t += gridDim.x) {
        const int y0 = (int)(t / tiles_x) * T, x0 = (int)(t % tiles_x) * T; /* source tile */
        const bool full = vec && y0 + T <= H && x0 + T <= W;
        if (full) {
            if constexpr (fast) { /* four consecutive rows at a time: a 4x4 block per thread and pass */
#pragma unroll
                for (int s = 0; s < (T / 4) / RY; ++s) {
                    const int j = ty + s * RY;
                    regs<V, In> a[4];
#pragma unroll
                    for (int q = 0; q < 4; ++q) load_all(p.in, ((long long)(y0 + 4 * j + q) * W + x0) / V + tx, a[q]);
                    trans_put4<In>(s_tile, j, tx, a, iseq);
                }
            } else { /* T / RY rows x one 16-byte vector per component and thread in flight */
                regs<V, In> a[T / RY];
#pragma unroll
                for (int q = 0; q < T / RY; ++q)
                    load_all(p.in, ((long long)(y0 + ty + q * RY) * W + x0) / V + tx, a[q]);
#pragma unroll
                for (int q = 0; q < T / RY; ++q) trans_put<In, V>(s_tile, ty + q * RY, tx * V, a[q], iseq);
            }
        } else {
            for (int r = ty; r < T; r += RY)
                for (int k = 0; k < V; ++k)
                    if (y0 + r < H && x0 + tx * V + k < W) {
                        regs<1, In> a;
                        load_one(p.in, (long long)(y0 + r) * W + x0 + tx * V + k, a);
                        trans_put<In, 1>(s_tile, r, tx * V + k, a, iseq);
                    }
        }
        __syncthreads();
        /* result row x0 + r holds source column x0 + r: elements y0 + 4 tx .. + 3 come from 4 tile rows */
        if (full) {
#pragma unroll 4
            for (int q = 0; q < T / RY; ++q) {
                const int r = ty + q * RY;
                regs<V, In> a;
                regs<V, Out> b;
                if constexpr (fast)
                    trans_take4<In>(s_tile, r, tx, a, iseq);
                else
                    trans_take<In, V>(s_tile, tx * V, r, a, iseq);
                const long long i = (long long)(x0 + r) * H + y0 + tx * V;
                map_apply<Fn>(env, i, a, b, iseq, oseq);
                store_all(p.out, i / V, b);
            }
        } else {
            for (int r = ty; r < T; r += RY)
                for (int k = 0; k < V; ++k)
                    if (x0 + r < W && y0 + tx * V + k < H) {
                        regs<1, In> a;
                        regs<1, Out> b;
                        trans_take<In, 1>(s_tile, tx * V + k, r, a, iseq);
                        const long long i = (long long)(x0 + r) * H + y0 + tx * V + k;
                        map_apply<Fn>(env, i, a, b, iseq, oseq);
                        store_one(p.out, i, b);
                    }
        }
        __syncthreads(); /* the tile is overwritten by the next trip */
    }
}

/* ---- the transposed form with the copy engine on both sides (one 4-byte input, one 4-byte output): a block
 * owns one 64x64 tile.  One thread asks for the tile as two boxes of 32 columns x 64 rows through a tensor map
 * with the hardware's 128-byte swizzle (a row of 32 values is 128 bytes; its 16-byte piece j lands at position
 * j ^ (row & 7)); every thread then takes one 4x4 block -- four 16-byte reads --, transposes it in registers,
 * applies the functor and writes four 16-byte pieces into the transposed tile, laid out the same way; one
 * thread hands that tile to the engine as two boxes of the result.  No load or store instruction touches global
 * memory, and the engine clips tiles that hang over the edge of the matrices (reads outside give zeros).
 * The 8 threads that share a shared-memory transaction take blocks (br, bc) = (8A + (u + s) mod 8, 8B + u),
 * u = 0..7: then both their reads (piece bc, rows 4 br + i) and their writes (piece br, rows 4 bc + k) fall
 * into 8 different 16-byte columns of the banks. ---- */
template <class Fn>
__host__ __device__ constexpr bool trans_tma_ok() {
    typedef typename Fn::In In;
    typedef typename Fn::Out Out;
    if constexpr (In::size == 1 && Out::size == 1)
        return sizeof(typename type_at<0, In>::type) == 4 && sizeof(typename type_at<0, Out>::type) == 4;
    else
        return false;
}
constexpr int kTransTmaSmem = 4 * 8192 + 1024; /* two boxes in, two boxes out, room to align to 1024 bytes */

template <class Fn, int CTA>
__device__ __forceinline__ void map_transposed_tma_body(const accb_kparams &p, const TensorMap *tin, const TensorMap *tout) {
    if constexpr (trans_tma_ok<Fn>()) {
        static_assert(CTA == 256, "one 4x4 block of the 64x64 tile per thread");
        typedef typename type_at<0, typename Fn::In>::type E;
        typedef typename type_at<0, typename Fn::Out>::type U;
        extern __shared__ __align__(128) unsigned char s_dyn[];
        __shared__ __align__(8) unsigned long long s_bar;
        /* the swizzle works on address bits: the boxes start on multiples of 1024 bytes */
        unsigned char *s_in = s_dyn + ((1024u - (smem_addr(s_dyn) & 1023u)) & 1023u);
        unsigned char *s_out = s_in + 2 * 8192;
        const Env env(p);
        const int H = (int)p.ip[0], W = (int)p.ip[1]; /* of the source; the result has W rows of H columns */
        const int tiles_x = (W + 63) / 64;
        const int y0 = (int)(blockIdx.x / tiles_x) * 64, x0 = (int)(blockIdx.x % tiles_x) * 64;
        unsigned int *err = static_cast<unsigned int *>(p.aux[1]);
        if (threadIdx.x == 0) {
            mbar_init(&s_bar, 1);
            fence_mbar_init();
        }
        __syncthreads();
        if (threadIdx.x == 0) {
            mbar_expect_tx(&s_bar, 2 * 8192);
            tensor_g2s_2d(s_in, tin, x0, y0, &s_bar);
            tensor_g2s_2d(s_in + 8192, tin, x0 + 32, y0, &s_bar);
        }
        int tries = 0;
        while (!mbar_try_wait(&s_bar, 0)) {
            if (++tries > (1 << 16)) { /* bounded: flag the result invalid and go on */
                atomicExch(err, 1u);
                break;
            }
        }
        const int u = threadIdx.x & 7, g = threadIdx.x >> 3;
        const int br = 8 * ((g >> 3) & 1) + ((u + (g & 7)) & 7), bc = 8 * (g >> 4) + u;
        uint4 a[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const int r = 4 * br + i;
            a[i] = *reinterpret_cast<const uint4 *>(s_in + (bc >> 3) * 8192 + r * 128 + (((bc & 7) ^ (r & 7)) << 4));
        }
#pragma unroll
        for (int k = 0; k < 4; ++k) {
            const int r = 4 * bc + k; /* row of the transposed tile = column of the source */
            const unsigned in4[4] = {k == 0 ? a[0].x : k == 1 ? a[0].y : k == 2 ? a[0].z : a[0].w,
                                     k == 0 ? a[1].x : k == 1 ? a[1].y : k == 2 ? a[1].z : a[1].w,
                                     k == 0 ? a[2].x : k == 1 ? a[2].y : k == 2 ? a[2].z : a[2].w,
                                     k == 0 ? a[3].x : k == 1 ? a[3].y : k == 2 ? a[3].z : a[3].w};
            unsigned o4[4];
            const long long i0 = (long long)(x0 + r) * H + y0 + 4 * br; /* position in the result */
#pragma unroll
            for (int q = 0; q < 4; ++q) {
                U o;
                Fn::apply(env, env.p.base + i0 + q, trans_unbits<E>(in4[q]), o);
                o4[q] = trans_bits(o);
            }
            *reinterpret_cast<uint4 *>(s_out + (br >> 3) * 8192 + r * 128 + (((br & 7) ^ (r & 7)) << 4)) =
                make_uint4(o4[0], o4[1], o4[2], o4[3]);
        }
        fence_async_shared();
        __syncthreads();
        if (threadIdx.x == 0) {
            tensor_s2g_2d(tout, y0, x0, s_out);
            tensor_s2g_2d(tout, y0 + 32, x0, s_out + 8192);
            bulk_commit();
            bulk_wait_read(); /* the shared memory must outlive the engine's reads */
        }
    }
}

/* the transposed form needs element-wise inputs; without any it has nothing to do */
template <class Fn, int CTA>
__device__ __forceinline__ void map_transposed_or_nothing(const accb_kparams &p) {
    if constexpr (Fn::In::size > 0) map_transposed_body<Fn, CTA>(p);
}
template <class Fn>
__host__ __device__ constexpr int map_transposed_smem() {
    typedef typename Fn::In In;
    if constexpr (In::size > 0)
        return smem_offset<In, In::size, trans_elems<In>()>::value;
    else
        return 0;
}

}  // namespace accb

#ifndef ACCB_MAP_CTA
#define ACCB_MAP_CTA 256
#endif
#ifndef ACCB_TRANS_MINB
#define ACCB_TRANS_MINB 8 /* resident blocks per SM the transposed form is compiled for: one 16 KB tile each */
#endif
#ifndef ACCB_MAP_U
#define ACCB_MAP_U 2 /* vectors per input per thread per trip */
#endif

/* Entry point named after the reference's kernel (Mapping.hs:53), and the form for transposed
 * inputs.  Metadata: {.., 0, 0, U, element-wise input components, shared memory of the transposed form, -,
 * whether the tensor-map transposed form exists, its shared memory}. */
#define ACCB_INSTANTIATE_MAP(Fn)                                                        \
    ACCB_META12(1, ACCB_MAP_CTA, 0, 0, ACCB_MAP_U, Fn::In::size,                        \
                (accb::map_transposed_smem<Fn>()), 0, accb::trans_tma_ok<Fn>() ? 1 : 0, \
                accb::kTransTmaSmem, 0, Fn::In::size)                                   \
    extern "C" __global__ void __launch_bounds__(ACCB_MAP_CTA)                          \
        map(const __grid_constant__ accb_kparams p) {                                   \
        accb::map_body<Fn, ACCB_MAP_CTA, ACCB_MAP_U>(p);                                \
    }                                                                                   \
    extern "C" __global__ void __launch_bounds__(ACCB_MAP_CTA, ACCB_TRANS_MINB)         \
        map_transposed(const __grid_constant__ accb_kparams p) {                        \
        accb::map_transposed_or_nothing<Fn, ACCB_MAP_CTA>(p);                           \
    }                                                                                   \
    extern "C" __global__ void __launch_bounds__(ACCB_MAP_CTA, 6)                       \
        map_transposed_tma(const __grid_constant__ accb_kparams p, const __grid_constant__ accb::TensorMap tin, \
                           const __grid_constant__ accb::TensorMap tout) {              \
        accb::map_transposed_tma_body<Fn, ACCB_MAP_CTA>(p, &tin, &tout);                \
    }
