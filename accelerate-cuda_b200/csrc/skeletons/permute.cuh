/*
 * permute.cuh -- forward permutation with a combination function
 * (scatter-combine): out[p(i)] = f(src[i], out[p(i)]).
 *
 * Replaces mkPermute (Data/Array/Accelerate/CUDA/CodeGen/IndexSpace.hs:160-303)
 * and its host driver permuteOp (Execute.hs:396-408).  Kept from there: the
 * defaults are copied into the result before the kernel runs; a destination
 * equal to `ignore` drops the element (IndexSpace.hs:200,229-233; here: a
 * negative linear index); the NEW value is the first argument of the
 * combiner (:203-208); the result is only defined for an associative and
 * commutative combiner.
 *
 * The reference serialises every update through a per-destination spin lock
 * in global memory (atomicExch + __threadfence, :285-303).  Here the functor
 * names how its combiner can be made atomic:
 *   Atomic::Add / Min / Max / And / Or / Xor -- native red.global / red.shared
 *   Atomic::Cas   -- compare-and-swap loop on a 4- or 8-byte value
 *   Atomic::None  -- the combiner ignores the old value: plain store (:242,287)
 *   Atomic::Lock  -- anything else (tuples): bounded per-element try-lock
 * and, when the whole destination fits in shared memory and the operation is
 * native, the block accumulates into privatised shared-memory copies (one per
 * group of lanes, so equal keys inside a warp rarely meet) and flushes them
 * with one global reduction per non-identity bin.
 *
 * Functor contract (derive from accb::Permute<T, Atomic>):
 *   using In = accb::types<...>;   element-wise inputs shared by index and get
 *   static long long index(env, i, in-values...);   < 0 means ignore
 *   static T get(env, i, in-values...);
 *   static T combine(T fresh, T old);
 *   static T identity();           only for the shared-memory path
 *
 *   aux[0] lock array (Lock only), aux[1] error word
 *   ip[0] destination size, ip[1] shared-memory replicas
 */
#pragma once
#include <type_traits>
#include "../cubits/accb_vec.cuh"
#include "../cubits/accb_warp.cuh"

#ifndef ACCB_PERMUTE_CTA
#define ACCB_PERMUTE_CTA 512
#endif
#ifndef ACCB_PERMUTE_U
#define ACCB_PERMUTE_U 4
#endif
#ifndef ACCB_LOCK_SPIN_LIMIT
#define ACCB_LOCK_SPIN_LIMIT (1 << 20)
#endif

namespace accb {

enum class Atomic { None, Add, Min, Max, And, Or, Xor, Cas, Lock };

template <class T, Atomic A>
struct Permute {
    typedef T elem;
    static constexpr Atomic atomic = A;
    typedef types<T> Out;
    static __device__ __forceinline__ void put(T r, T &o) { o = r; }
    static __device__ __forceinline__ T take(const T &o) { return o; }
    static __device__ __forceinline__ T identity() { return T(); }
};

template <class T>
__device__ __forceinline__ bool bits_equal(const T &a, const T &b) {
    const unsigned char *x = reinterpret_cast<const unsigned char *>(&a);
    const unsigned char *y = reinterpret_cast<const unsigned char *>(&b);
    bool eq = true;
#pragma unroll
    for (int i = 0; i < (int)sizeof(T); ++i) eq = eq && (x[i] == y[i]);
    return eq;
}

/* atomic combine into any address space reachable by a generic pointer */
template <class Fn>
__device__ __forceinline__ void atomic_combine(typename Fn::elem *addr, typename Fn::elem x) {
    typedef typename Fn::elem T;
    constexpr Atomic A = Fn::atomic;
    if constexpr (A == Atomic::None) {
        *addr = x;
    } else if constexpr (A == Atomic::Add) {
        if constexpr (sizeof(T) == 8 && !std::is_floating_point<T>::value)
            atomicAdd(reinterpret_cast<unsigned long long *>(addr), (unsigned long long)x);
        else if constexpr (sizeof(T) == 4 && !std::is_floating_point<T>::value)
            atomicAdd(reinterpret_cast<unsigned int *>(addr), (unsigned int)x);
        else
            atomicAdd(addr, x);
    } else if constexpr (A == Atomic::Min && std::is_integral<T>::value) {
        atomicMin(addr, x);
    } else if constexpr (A == Atomic::Max && std::is_integral<T>::value) {
        atomicMax(addr, x);
    } else if constexpr (A == Atomic::And) {
        atomicAnd(addr, x);
    } else if constexpr (A == Atomic::Or) {
        atomicOr(addr, x);
    } else if constexpr (A == Atomic::Xor) {
        atomicXor(addr, x);
    } else {
        /* compare-and-swap loop with the user's combiner */
        static_assert(sizeof(T) == 4 || sizeof(T) == 8, "CAS combine needs a 4- or 8-byte value");
        if constexpr (sizeof(T) == 4) {
            unsigned int *a = reinterpret_cast<unsigned int *>(addr);
            unsigned int old = *a, assumed;
            do {
                assumed = old;
                T o;
                memcpy(&o, &assumed, 4);
                T r = Fn::combine(x, o);
                unsigned int rb;
                memcpy(&rb, &r, 4);
                old = atomicCAS(a, assumed, rb);
            } while (old != assumed);
        } else {
            unsigned long long *a = reinterpret_cast<unsigned long long *>(addr);
            unsigned long long old = *a, assumed;
            do {
                assumed = old;
                T o;
                memcpy(&o, &assumed, 8);
                T r = Fn::combine(x, o);
                unsigned long long rb;
                memcpy(&rb, &r, 8);
                old = atomicCAS(a, assumed, rb);
            } while (old != assumed);
        }
    }
}

template <class Fn, int... O>
__device__ __forceinline__ void permute_locked(const accb_kparams &p, long long j, typename Fn::elem x,
                                               std::integer_sequence<int, O...>) {
    /* try-lock form that lets every lane of a warp make progress
     * (IndexSpace.hs:262-303), with a bound on the number of attempts */
    int *lock = static_cast<int *>(p.aux[0]) + j;
    bool done = false;
    volatile unsigned int *err = static_cast<volatile unsigned int *>(p.aux[1]);
    for (int spin = 0; !done && spin < ACCB_LOCK_SPIN_LIMIT; ++spin) {
        if ((spin & 1023) == 1023 && *err != 0u) break; /* somebody already gave up: do not queue behind them */
        if (atomicCAS(lock, 0, 1) == 0) {
            __threadfence();
            regs<1, typename Fn::Out> b;
            ((comp<O>(b)[0] = static_cast<volatile typename type_at<O, typename Fn::Out>::type *>(p.out[O])[j]), ...);
            typename Fn::elem r = Fn::combine(x, Fn::take(comp<O>(b)[0]...));
            Fn::put(r, comp<O>(b)[0]...);
            ((static_cast<volatile typename type_at<O, typename Fn::Out>::type *>(p.out[O])[j] = comp<O>(b)[0]), ...);
            __threadfence();
            atomicExch(lock, 0);
            done = true;
        }
    }
    if (!done) atomicExch(static_cast<unsigned int *>(p.aux[1]), 1u);
}

template <class Fn, int N, int... I>
__device__ __forceinline__ void permute_elems(const accb_kparams &p, const Env &env, long long i0,
                                              regs<N, typename Fn::In> &a, std::integer_sequence<int, I...>) {
    typedef typename Fn::elem T;
    const long long nout = p.ip[0];
#pragma unroll
    for (int k = 0; k < N; ++k) {
        const long long j = Fn::index(env, env.p.base + i0 + k, comp<I>(a)[k]...);
        if (j >= 0 && j < nout) {
            const T x = Fn::get(env, env.p.base + i0 + k, comp<I>(a)[k]...);
            if constexpr (Fn::atomic == Atomic::Lock)
                permute_locked<Fn>(p, j, x, std::make_integer_sequence<int, Fn::Out::size>());
            else
                atomic_combine<Fn>(static_cast<T *>(p.out[0]) + j, x);
        }
    }
}

/* ---- general form: combine straight into global memory ---- */
template <class Fn, int CTA, int U>
__device__ __forceinline__ void permute_body(const accb_kparams &p) {
    typedef typename Fn::In In;
    const Env env(p);
    const auto iseq = std::make_integer_sequence<int, In::size>();
    const long long n = p.n;
    const long long nvec = (p.flags & ACCB_F_VEC) ? n / V : 0;
    constexpr long long TRIP = (long long)CTA * U;
    const long long ntrip = nvec / TRIP;
    for (long long t = blockIdx.x; t < ntrip; t += gridDim.x) {
        const long long v0 = t * TRIP + threadIdx.x;
        regs<V, In> a[U];
#pragma unroll
        for (int u = 0; u < U; ++u) load_all(p.in, v0 + (long long)u * CTA, a[u]);
#pragma unroll
        for (int u = 0; u < U; ++u) permute_elems<Fn>(p, env, (v0 + (long long)u * CTA) * V, a[u], iseq);
    }
    for (long long v = ntrip * TRIP + (long long)blockIdx.x * CTA + threadIdx.x; v < nvec;
         v += (long long)gridDim.x * CTA) {
        regs<V, In> a;
        load_all(p.in, v, a);
        permute_elems<Fn>(p, env, v * V, a, iseq);
    }
    for (long long i = nvec * V + (long long)blockIdx.x * CTA + threadIdx.x; i < n;
         i += (long long)gridDim.x * CTA) {
        regs<1, In> a;
        load_one(p.in, i, a);
        permute_elems<Fn>(p, env, i, a, iseq);
    }
}

/* ---- privatised form: the whole destination lives in shared memory ----
 * (Tried: a bank permutation of the slots, j ^ ((j >> 5 ^ j >> 10) & 31), so that hot destinations a multiple of
 * 32 elements apart stop sharing a bank.  16 hot bins 256 apart went from 60 % to 81 % of copy rate, and the
 * Zipf-distributed keys of the benchmark from 95 % to 81 %: four more integer instructions per element are not
 * free in a kernel that issues about ten.  Left out.) */
template <class Fn, int N, int... I>
__device__ __forceinline__ void permute_elems_smem(const accb_kparams &p, const Env &env, long long i0,
                                                   regs<N, typename Fn::In> &a, typename Fn::elem *mine,
                                                   std::integer_sequence<int, I...>) {
    typedef typename Fn::elem T;
    const long long nout = p.ip[0];
#pragma unroll
    for (int k = 0; k < N; ++k) {
        const long long j = Fn::index(env, env.p.base + i0 + k, comp<I>(a)[k]...);
        if (j >= 0 && j < nout) {
            const T x = Fn::get(env, env.p.base + i0 + k, comp<I>(a)[k]...);
            atomic_combine<Fn>(mine + j, x);
        }
    }
}

template <class Fn, int CTA, int U>
__device__ __forceinline__ void permute_smem_body(const accb_kparams &p) {
    typedef typename Fn::In In;
    typedef typename Fn::elem T;
    static_assert(Fn::atomic != Atomic::Lock && Fn::atomic != Atomic::Cas && Fn::atomic != Atomic::None,
                  "shared-memory privatisation needs a native atomic");
    extern __shared__ __align__(16) unsigned char s_raw[];
    T *priv = reinterpret_cast<T *>(s_raw);
    const Env env(p);
    const auto iseq = std::make_integer_sequence<int, In::size>();
    const long long n = p.n;
    const int nout = (int)p.ip[0];
    const int R = (int)p.ip[1];
    const int stride = nout + 1; /* skew the replicas across banks */
    for (int i = threadIdx.x; i < R * stride; i += CTA) priv[i] = Fn::identity();
    __syncthreads();
    T *mine = priv + (threadIdx.x & (R - 1)) * stride; /* R is a power of two */

    const long long nvec = (p.flags & ACCB_F_VEC) ? n / V : 0;
    constexpr long long TRIP = (long long)CTA * U;
    const long long ntrip = nvec / TRIP;
    for (long long t = blockIdx.x; t < ntrip; t += gridDim.x) {
        const long long v0 = t * TRIP + threadIdx.x;
        regs<V, In> a[U];
#pragma unroll
        for (int u = 0; u < U; ++u) load_all(p.in, v0 + (long long)u * CTA, a[u]);
#pragma unroll
        for (int u = 0; u < U; ++u)
            permute_elems_smem<Fn>(p, env, (v0 + (long long)u * CTA) * V, a[u], mine, iseq);
    }
    for (long long v = ntrip * TRIP + (long long)blockIdx.x * CTA + threadIdx.x; v < nvec;
         v += (long long)gridDim.x * CTA) {
        regs<V, In> a;
        load_all(p.in, v, a);
        permute_elems_smem<Fn>(p, env, v * V, a, mine, iseq);
    }
    for (long long i = nvec * V + (long long)blockIdx.x * CTA + threadIdx.x; i < n;
         i += (long long)gridDim.x * CTA) {
        regs<1, In> a;
        load_one(p.in, i, a);
        permute_elems_smem<Fn>(p, env, i, a, mine, iseq);
    }
    __syncthreads();
    /* flush: fold the replicas of a bin, then one global reduction per touched bin */
    T *out = static_cast<T *>(p.out[0]);
    const T id = Fn::identity();
    for (int b = threadIdx.x; b < nout; b += CTA) {
        T acc = priv[b];
        for (int r = 1; r < R; ++r) acc = Fn::combine(priv[r * stride + b], acc);
        if (!bits_equal(acc, id)) atomic_combine<Fn>(out + b, acc);
    }
}

}  // namespace accb

/* Entry points: `permute` as in the reference (IndexSpace.hs:172); the
 * privatised form is selected by the host when the destination is small. */
#define ACCB_INSTANTIATE_PERMUTE(Fn)                                                           \
    ACCB_META12(6, ACCB_PERMUTE_CTA, sizeof(Fn::elem), 0, ACCB_PERMUTE_U,                      \
                Fn::atomic == accb::Atomic::Lock ? 1 : 0, 0, 0, 0, 0, 0, Fn::In::size)         \
    extern "C" __global__ void __launch_bounds__(ACCB_PERMUTE_CTA)                             \
        permute(const __grid_constant__ accb_kparams p) {                                      \
        accb::permute_body<Fn, ACCB_PERMUTE_CTA, ACCB_PERMUTE_U>(p);                           \
    }

#define ACCB_INSTANTIATE_PERMUTE_SMEM(Fn)                                                      \
    ACCB_INSTANTIATE_PERMUTE(Fn)                                                               \
    extern "C" __global__ void __launch_bounds__(ACCB_PERMUTE_CTA)                             \
        permute_smem(const __grid_constant__ accb_kparams p) {                                 \
        accb::permute_smem_body<Fn, ACCB_PERMUTE_CTA, ACCB_PERMUTE_U>(p);                      \
    }
