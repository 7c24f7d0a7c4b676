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

namespace accb {

template <class Fn, int N, int... I, int... O>
__device__ __forceinline__ void map_apply(const Env &env, long long i0, regs<N, typename Fn::In> &a,
                                          regs<N, typename Fn::Out> &b, std::integer_sequence<int, I...>,
                                          std::integer_sequence<int, O...>) {
#pragma unroll
    for (int k = 0; k < N; ++k) Fn::apply(env, i0 + k, comp<I>(a)[k]..., comp<O>(b)[k]...);
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

}  // namespace accb

#ifndef ACCB_MAP_CTA
#define ACCB_MAP_CTA 256
#endif
#ifndef ACCB_MAP_U
#define ACCB_MAP_U 2 /* vectors per input per thread per trip */
#endif

/* Entry point named after the reference's kernel (Mapping.hs:53). */
#define ACCB_INSTANTIATE_MAP(Fn)                                                        \
    ACCB_META(1, ACCB_MAP_CTA, 0, 0, ACCB_MAP_U, 0)                                     \
    extern "C" __global__ void __launch_bounds__(ACCB_MAP_CTA)                          \
        map(const __grid_constant__ accb_kparams p) {                                   \
        accb::map_body<Fn, ACCB_MAP_CTA, ACCB_MAP_U>(p);                                \
    }
