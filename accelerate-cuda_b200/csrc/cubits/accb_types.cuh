/*
 * accb_types.cuh -- scalar type names, type lists and the environment view
 * that user functors see.
 *
 * Successor of cubits/accelerate_cuda_type.h:22-30 (Int8..Word64) and of the
 * C type table in Data/Array/Accelerate/CUDA/CodeGen/Type.hs:106-146
 * (Bool is one byte, Char is a 32-bit code point).
 */
#pragma once
#include <stdint.h>
#include <utility>
#include "accb_params.h"

namespace accb {

typedef int8_t Int8;
typedef int16_t Int16;
typedef int32_t Int32;
typedef int64_t Int64;
typedef uint8_t Word8;
typedef uint16_t Word16;
typedef uint32_t Word32;
typedef uint64_t Word64;
typedef float Float;
typedef double Double;
typedef uint8_t Bool;
typedef uint32_t Char;
typedef long long Int; /* Accelerate's Int is the 64-bit host word (Type.hs:131) */

/* ---- compile-time list of scalar types: one entry per SoA component ---- */
template <class... Ts>
struct types {
    static constexpr int size = sizeof...(Ts);
};

template <int I, class L>
struct type_at;
template <int I, class T, class... Ts>
struct type_at<I, types<T, Ts...>> : type_at<I - 1, types<Ts...>> {};
template <class T, class... Ts>
struct type_at<0, types<T, Ts...>> {
    typedef T type;
};

/* byte offset of component I when TILE elements of every component of a type list are staged in
 * shared memory one after the other, each component starting on a 128-byte boundary;
 * smem_offset<L, L::size, TILE> is the total */
template <class L, int I, int TILE>
struct smem_offset {
    static constexpr int value = smem_offset<L, I - 1, TILE>::value +
                                 ((TILE * (int)sizeof(typename type_at<I - 1, L>::type) + 127) / 128) * 128;
};
template <class L, int TILE>
struct smem_offset<L, 0, TILE> {
    static constexpr int value = 0;
};

/* registers for V consecutive elements of every component in a type list */
template <int V, class L>
struct regs;
template <int V>
struct regs<V, types<>> {};
template <int V, class T, class... Ts>
struct regs<V, types<T, Ts...>> {
    T v[V];
    regs<V, types<Ts...>> rest;
};

template <int I, int V, class T, class... Ts>
__device__ __forceinline__ auto &comp(regs<V, types<T, Ts...>> &r) {
    if constexpr (I == 0)
        return r.v;
    else
        return comp<I - 1>(r.rest);
}

/* ---- what a functor sees of the kernel arguments ---- */
struct Env {
    const accb_kparams &p;
    __device__ __forceinline__ explicit Env(const accb_kparams &q) : p(q) {}

    /* pointer to component `slot` of the environment, typed by the functor */
    template <class T>
    __device__ __forceinline__ const T *in(int slot) const {
        return static_cast<const T *>(p.in[slot]);
    }
    /* extent `d` (0 = innermost) of environment array `arr` */
    __device__ __forceinline__ int dim(int arr, int d) const { return p.in_shape[arr][d]; }
    __device__ __forceinline__ int out_dim(int d) const { return p.out_shape[d]; }
    /* user scalar stored at byte offset `off` of the scalar block */
    template <class T>
    __device__ __forceinline__ T scalar(int off) const {
        T t;
        const unsigned char *s = p.scalars + off;
        unsigned char *d = reinterpret_cast<unsigned char *>(&t);
#pragma unroll
        for (int i = 0; i < (int)sizeof(T); ++i) d[i] = s[i];
        return t;
    }
    __device__ __forceinline__ long long size() const { return p.n; }
};

/* ---- row-major index arithmetic (CodeGen/Base.hs:195-218), 64-bit ---- */
__device__ __forceinline__ long long to_index2(int sh0 /*inner extent*/, int y, int x) {
    return (long long)y * sh0 + x;
}
__device__ __forceinline__ long long to_index3(int sh1, int sh0, int z, int y, int x) {
    return ((long long)z * sh1 + y) * sh0 + x;
}
__device__ __forceinline__ void from_index2(int sh0, long long i, int &y, int &x) {
    y = (int)(i / sh0);
    x = (int)(i - (long long)y * sh0);
}
__device__ __forceinline__ void from_index3(int sh1, int sh0, long long i, int &z, int &y, int &x) {
    long long q = i / sh0;
    x = (int)(i - q * sh0);
    z = (int)(q / sh1);
    y = (int)(q - (long long)z * sh1);
}

/* Haskell-style integer division and modulus (round towards -inf),
 * CodeGen/Arithmetic.hs:103-134 */
template <class T>
__device__ __forceinline__ T idiv(T a, T b) {
    T q = a / b, r = a % b;
    return (r != 0 && ((r < 0) != (b < 0))) ? q - 1 : q;
}
template <class T>
__device__ __forceinline__ T imod(T a, T b) {
    T r = a % b;
    return (r != 0 && ((r < 0) != (b < 0))) ? r + b : r;
}

}  // namespace accb

/* Launch metadata the host asks the loaded module for (one single-thread
 * launch when the module is first loaded): {skeleton id, block size, record
 * bytes, tile elements, vectors per thread per trip, skeleton-specific flag,
 * 0, 0}.  It stands in for the (entry name, occupancy, block size, shared
 * memory) record the reference keeps per kernel
 * (Data/Array/Accelerate/CUDA/AST.hs:51-59). */
#define ACCB_META12(id, cta, rec, tile, u, extra, smem, last, m8, m9, m10, m11)     \
    extern "C" __global__ void accb_meta_query(int *out) {                     \
        const int m[12] = {(id), (cta), (int)(rec), (int)(tile), (u), (extra), (int)(smem), (int)(last), \
                           (int)(m8), (int)(m9), (int)(m10), (int)(m11)};      \
        for (int i = 0; i < 12; ++i) out[i] = m[i];                            \
    }
#define ACCB_META8(id, cta, rec, tile, u, extra, smem, last) ACCB_META12(id, cta, rec, tile, u, extra, smem, last, 0, 0, 0, 0)
#define ACCB_META7(id, cta, rec, tile, u, extra, smem) ACCB_META8(id, cta, rec, tile, u, extra, smem, 0)
#define ACCB_META(id, cta, rec, tile, u, extra) ACCB_META7(id, cta, rec, tile, u, extra, 0)
