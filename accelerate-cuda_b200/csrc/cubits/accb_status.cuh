/*
 * accb_status.cuh -- status records of single-pass kernels whose tiles wait for
 * their predecessors' results (the scans' decoupled look-back, the balanced
 * segmented fold): one record per tile, carrying a launch epoch, a state and a
 * value in a form that one store publishes and one load reads.
 */
#pragma once
#include <cstring>
#include "accb_warp.cuh"

#ifndef ACCB_SCAN_STATUS_STRIDE
#define ACCB_SCAN_STATUS_STRIDE 16 /* distance between tile status words, in 8-byte units */
#endif

namespace accb {

enum : unsigned { ST_AGG = 1u, ST_PREFIX = 2u };

/* ---- tile status.  A tile's record is kBytes long and starts with a 64-bit
 * head whose upper half is the flag {epoch << 2 | state} in every layout, so a
 * record left behind by a scan of another value type reads as an earlier
 * epoch, i.e. "not ready".
 *   values up to 4 bytes : the value sits in the lower half of the head; one
 *                          relaxed 64-bit store / load carries flag and value;
 *   values of 8 bytes    : {head, value} as one 128-bit store / load;
 *   larger values        : {head, aggregate, prefix}, the flag published with
 *                          release and read with acquire ordering.
 * Neighbouring tiles' records are at least ACCB_SCAN_STATUS_STRIDE * 8 bytes
 * apart. ---- */
template <class T, int LAYOUT = (sizeof(T) <= 4 ? 0 : (sizeof(T) == 8 ? 1 : 2))>
struct TileStatus;

template <class T>
struct TileStatus<T, 0> {
    static constexpr int kBytes = 8 * ACCB_SCAN_STATUS_STRIDE;
    unsigned long long *w;
    __device__ __forceinline__ explicit TileStatus(void *base) : w(static_cast<unsigned long long *>(base)) {}
    __device__ __forceinline__ void publish(long long t, unsigned flag, T v) const {
        unsigned bits = 0;
        memcpy(&bits, &v, sizeof(T));
        const unsigned long long word = ((unsigned long long)flag << 32) | bits;
        asm volatile("st.relaxed.gpu.global.u64 [%0], %1;" ::"l"(w + t * ACCB_SCAN_STATUS_STRIDE), "l"(word)
                     : "memory");
    }
    /* returns the flag word; value valid when the flag's epoch matches */
    __device__ __forceinline__ unsigned peek(long long t, T &v) const {
        unsigned long long word;
        asm volatile("ld.relaxed.gpu.global.u64 %0, [%1];"
                     : "=l"(word)
                     : "l"(w + t * ACCB_SCAN_STATUS_STRIDE)
                     : "memory");
        const unsigned bits = (unsigned)word;
        memcpy(&v, &bits, sizeof(T));
        return (unsigned)(word >> 32);
    }
};

template <class T>
struct TileStatus<T, 1> {
    static constexpr int kStride = ACCB_SCAN_STATUS_STRIDE < 2 ? 2 : (ACCB_SCAN_STATUS_STRIDE + 1) / 2 * 2;
    static constexpr int kBytes = 8 * kStride; /* 16-byte aligned records */
    unsigned long long *w;
    __device__ __forceinline__ explicit TileStatus(void *base) : w(static_cast<unsigned long long *>(base)) {}
    __device__ __forceinline__ void publish(long long t, unsigned flag, T v) const {
        unsigned long long bits;
        memcpy(&bits, &v, 8);
        const unsigned long long head = (unsigned long long)flag << 32;
        asm volatile("{ .reg .b128 q; mov.b128 q, {%1, %2}; st.relaxed.gpu.global.b128 [%0], q; }" ::"l"(w + t * kStride),
                     "l"(head), "l"(bits)
                     : "memory");
    }
    __device__ __forceinline__ unsigned peek(long long t, T &v) const {
        unsigned long long head, bits;
        asm volatile("{ .reg .b128 q; ld.relaxed.gpu.global.b128 q, [%2]; mov.b128 {%0, %1}, q; }"
                     : "=l"(head), "=l"(bits)
                     : "l"(w + t * kStride)
                     : "memory");
        memcpy(&v, &bits, 8);
        return (unsigned)(head >> 32);
    }
};

template <class T>
struct TileStatus<T, 2> {
    static_assert(sizeof(T) % 4 == 0 && sizeof(T) <= 32, "scan value types are at most 32 bytes");
    struct alignas(128) Rec {
        unsigned pad;
        unsigned flag;
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

}  // namespace accb
