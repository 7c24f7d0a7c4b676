/*
 * accb_warp.cuh -- warp-level data exchange and block-level reductions.
 *
 * Successor of cubits/accelerate_cuda_function.h:127-193 (shfl_up32/64,
 * shfl_xor32/64 built on the pre-Volta __shfl intrinsics, which no longer
 * exist) and of the shared-memory trees reduceWarpTree/reduceBlockTree in
 * Data/Array/Accelerate/CUDA/CodeGen/Reduction.hs:616-699, which rely on
 * implicit warp-synchronous execution.  Everything here uses the *_sync
 * forms with explicit masks; nothing assumes lock-step execution.
 */
#pragma once
#include <string.h>
#include "accb_types.cuh"

namespace accb {

constexpr unsigned FULL = 0xffffffffu;

template <class T>
__device__ __forceinline__ T shfl_down(T v, int d) {
    constexpr int W = (sizeof(T) + 3) / 4;
    unsigned w[W] = {};
    memcpy(w, &v, sizeof(T));
#pragma unroll
    for (int i = 0; i < W; ++i) w[i] = __shfl_down_sync(FULL, w[i], d);
    memcpy(&v, w, sizeof(T));
    return v;
}
template <class T>
__device__ __forceinline__ T shfl_up(T v, int d) {
    constexpr int W = (sizeof(T) + 3) / 4;
    unsigned w[W] = {};
    memcpy(w, &v, sizeof(T));
#pragma unroll
    for (int i = 0; i < W; ++i) w[i] = __shfl_up_sync(FULL, w[i], d);
    memcpy(&v, w, sizeof(T));
    return v;
}
template <class T>
__device__ __forceinline__ T shfl_xor(T v, int m) {
    constexpr int W = (sizeof(T) + 3) / 4;
    unsigned w[W] = {};
    memcpy(w, &v, sizeof(T));
#pragma unroll
    for (int i = 0; i < W; ++i) w[i] = __shfl_xor_sync(FULL, w[i], m);
    memcpy(&v, w, sizeof(T));
    return v;
}
template <class T>
__device__ __forceinline__ T shfl_idx(T v, int lane) {
    constexpr int W = (sizeof(T) + 3) / 4;
    unsigned w[W] = {};
    memcpy(w, &v, sizeof(T));
#pragma unroll
    for (int i = 0; i < W; ++i) w[i] = __shfl_sync(FULL, w[i], lane);
    memcpy(&v, w, sizeof(T));
    return v;
}

/* L2-coherent (L1-bypassing) load of a small struct written by another block */
template <class T>
__device__ __forceinline__ T ld_cg(const T *p) {
    static_assert(sizeof(T) % 4 == 0, "word-sized structs only");
    constexpr int W = sizeof(T) / 4;
    unsigned w[W];
    const unsigned *q = reinterpret_cast<const unsigned *>(p);
#pragma unroll
    for (int i = 0; i < W; ++i) w[i] = __ldcg(q + i);
    T t;
    memcpy(&t, w, sizeof(T));
    return t;
}

__device__ __forceinline__ int lane_id() { return threadIdx.x & 31; }
__device__ __forceinline__ int warp_id() { return threadIdx.x >> 5; }

/* Reduce over the whole warp; every lane gets the result.  The operator need
 * not be commutative for the *value order* lane 0, 1, ..., 31 only when the
 * down-shuffle form below is used; the butterfly is for commutative use. */
template <class T, class F>
__device__ __forceinline__ T warp_reduce_xor(T v, F f) {
#pragma unroll
    for (int m = 16; m > 0; m >>= 1) v = f(v, shfl_xor(v, m));
    return v;
}

/* Ordered reduction: result (valid in lane 0) = v0 (+) v1 (+) ... (+) v31. */
template <class T, class F>
__device__ __forceinline__ T warp_reduce_ordered(T v, F f) {
#pragma unroll
    for (int d = 1; d < 32; d <<= 1) {
        T o = shfl_down(v, d);
        if (lane_id() + d < 32) v = f(v, o);
    }
    return v;
}

/* Inclusive scan across the warp in lane order. */
template <class T, class F>
__device__ __forceinline__ T warp_scan_inclusive(T v, F f) {
    const int lane = lane_id();
#pragma unroll
    for (int d = 1; d < 32; d <<= 1) {
        T o = shfl_up(v, d);
        if (lane >= d) v = f(o, v);
    }
    return v;
}

/* Block reduction through one shared slot per warp.  `smem` holds at least
 * (CTA/32) values of T.  Result valid in thread 0.  Operator assumed
 * commutative (the same assumption as the strided accumulation of the
 * reference's foldAll, Reduction.hs:160-165). */
template <int CTA, class T, class F>
__device__ __forceinline__ T block_reduce(T v, F f, T *smem) {
    constexpr int NW = CTA / 32;
    v = warp_reduce_xor(v, f);
    if constexpr (NW == 1) return v;
    if (lane_id() == 0) smem[warp_id()] = v;
    __syncthreads();
    if (warp_id() == 0) {
        T w = smem[lane_id() < NW ? lane_id() : 0];
#pragma unroll
        for (int m = 16; m > 0; m >>= 1) {
            T o = shfl_xor(w, m);
            /* lanes >= NW hold a duplicate of slot 0: combine only real slots */
            if (m < NW) w = f(w, o);
        }
        v = w;
    }
    __syncthreads();
    return v;
}

}  // namespace accb
