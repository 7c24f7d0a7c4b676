/*
 * accb_vec.cuh -- 128-bit coalesced global loads and stores.
 *
 * accelerate-cuda reads one scalar (<= 8 bytes) per array per loop trip
 * (Data/Array/Accelerate/CUDA/CodeGen/Mapping.hs:65-71, Analysis/Launch.hs:124-128
 * "eltsPerThread = 1").  Here a thread always moves V = 4 consecutive elements
 * of a component: 16 bytes for 4-byte types (one LDG.128), 2 x 16 bytes for
 * 8-byte types, 8 / 4 bytes for 2- / 1-byte types.  The pointer must be
 * aligned to min(16, 4*sizeof(T)); the host checks that and falls back to the
 * scalar path otherwise.
 *
 * Streaming variants (ld.global.cs / st.global.cs) mark data that is touched
 * once so that it does not displace reusable lines in the 126 MB L2.
 */
#pragma once
#include <string.h>
#include "accb_types.cuh"

namespace accb {

constexpr int V = 4; /* elements per thread per vector access */

enum class Cache { Default, Stream };

template <int BYTES>
struct raw;
template <>
struct raw<4> {
    typedef unsigned int type;
};
template <>
struct raw<8> {
    typedef uint2 type;
};
template <>
struct raw<16> {
    typedef uint4 type;
};

template <Cache C, class R>
__device__ __forceinline__ R ld_raw(const R *p) {
    if constexpr (C == Cache::Stream)
        return __ldcs(p);
    else
        return *p;
}
template <Cache C, class R>
__device__ __forceinline__ void st_raw(R *p, R v) {
    if constexpr (C == Cache::Stream)
        __stcs(p, v);
    else
        *p = v;
}

/* load elements [4*vi, 4*vi+4) of `base` */
template <Cache C = Cache::Stream, class T>
__device__ __forceinline__ void load4(const T *base, long long vi, T (&r)[V]) {
    constexpr int B = V * (int)sizeof(T);
    if constexpr (B <= 16) {
        typedef typename raw<B>::type R;
        R x = ld_raw<C>(reinterpret_cast<const R *>(base) + vi);
        memcpy(&r[0], &x, B);
    } else {
        static_assert(B == 32, "component types are 1, 2, 4 or 8 bytes wide");
        const uint4 *p = reinterpret_cast<const uint4 *>(base) + 2 * vi;
        uint4 a = ld_raw<C>(p), b = ld_raw<C>(p + 1);
        memcpy(&r[0], &a, 16);
        memcpy(&r[2], &b, 16);
    }
}

template <Cache C = Cache::Stream, class T>
__device__ __forceinline__ void store4(T *base, long long vi, const T (&r)[V]) {
    constexpr int B = V * (int)sizeof(T);
    if constexpr (B <= 16) {
        typedef typename raw<B>::type R;
        R x;
        memcpy(&x, &r[0], B);
        st_raw<C>(reinterpret_cast<R *>(base) + vi, x);
    } else {
        uint4 *p = reinterpret_cast<uint4 *>(base) + 2 * vi;
        uint4 a, b;
        memcpy(&a, &r[0], 16);
        memcpy(&b, &r[2], 16);
        st_raw<C>(p, a);
        st_raw<C>(p + 1, b);
    }
}

/* ---- whole type lists at once: component I lives in slot (first + I) ---- */
template <Cache C, int V_, class L, int... I>
__device__ __forceinline__ void load_all_impl(const void *const *slots, long long vi, regs<V_, L> &r,
                                              std::integer_sequence<int, I...>) {
    (load4<C>(static_cast<const typename type_at<I, L>::type *>(slots[I]), vi, comp<I>(r)), ...);
}
template <Cache C = Cache::Stream, class L>
__device__ __forceinline__ void load_all(const void *const *slots, long long vi, regs<V, L> &r) {
    load_all_impl<C>(slots, vi, r, std::make_integer_sequence<int, L::size>());
}

template <Cache C, class L, int... I>
__device__ __forceinline__ void store_all_impl(void *const *slots, long long vi, regs<V, L> &r,
                                               std::integer_sequence<int, I...>) {
    (store4<C>(static_cast<typename type_at<I, L>::type *>(slots[I]), vi, comp<I>(r)), ...);
}
template <Cache C = Cache::Stream, class L>
__device__ __forceinline__ void store_all(void *const *slots, long long vi, regs<V, L> &r) {
    store_all_impl<C>(slots, vi, r, std::make_integer_sequence<int, L::size>());
}

/* scalar (one element) forms used for ragged tails and unaligned arrays */
template <class L, int... I>
__device__ __forceinline__ void load_one_impl(const void *const *slots, long long i, regs<1, L> &r,
                                              std::integer_sequence<int, I...>) {
    ((comp<I>(r)[0] = static_cast<const typename type_at<I, L>::type *>(slots[I])[i]), ...);
}
template <class L>
__device__ __forceinline__ void load_one(const void *const *slots, long long i, regs<1, L> &r) {
    load_one_impl(slots, i, r, std::make_integer_sequence<int, L::size>());
}
template <class L, int... I>
__device__ __forceinline__ void store_one_impl(void *const *slots, long long i, regs<1, L> &r,
                                               std::integer_sequence<int, I...>) {
    ((static_cast<typename type_at<I, L>::type *>(slots[I])[i] = comp<I>(r)[0]), ...);
}
template <class L>
__device__ __forceinline__ void store_one(void *const *slots, long long i, regs<1, L> &r) {
    store_one_impl(slots, i, r, std::make_integer_sequence<int, L::size>());
}

}  // namespace accb
