/*
 * accb_tma.cuh -- bulk asynchronous copies global -> shared memory through the
 * TMA engine (cp.async.bulk) with completion on an mbarrier.
 *
 * accelerate-cuda has nothing comparable: its kernels read one scalar per
 * thread per trip (Data/Array/Accelerate/CUDA/CodeGen/Base.hs:262-305).  Here
 * one thread hands a whole tile to the copy engine; no register holds data
 * while the copy is in flight, and the bytes in flight per SM are bounded by
 * shared memory (227 KB) instead of by the register file.
 *
 * Rules the callers keep: source and destination 16-byte aligned, size a
 * multiple of 16 bytes, at most 2^20 - 1 bytes pending on one mbarrier, and
 * the source is always this GPU's own memory (no cluster multicast is used).
 */
#pragma once

namespace accb {

__device__ __forceinline__ unsigned smem_addr(const void *p) {
    return (unsigned)__cvta_generic_to_shared(p);
}

__device__ __forceinline__ void mbar_init(unsigned long long *bar, unsigned arrivals) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_addr(bar)), "r"(arrivals) : "memory");
}

/* makes the initialised barrier visible to the asynchronous proxy */
__device__ __forceinline__ void fence_mbar_init() {
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}

/* one arrival that also announces `bytes` of pending asynchronous writes */
__device__ __forceinline__ void mbar_expect_tx(unsigned long long *bar, unsigned bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_addr(bar)), "r"(bytes)
                 : "memory");
}

/* dst: shared memory of this block; src: global memory; completes `bytes` on `bar` */
__device__ __forceinline__ void bulk_g2s(void *dst, const void *src, unsigned bytes, unsigned long long *bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
                     smem_addr(dst)),
                 "l"(src), "r"(bytes), "r"(smem_addr(bar))
                 : "memory");
}

/* one bounded try: true once the phase with the given parity has completed */
__device__ __forceinline__ bool mbar_try_wait(unsigned long long *bar, unsigned parity) {
    unsigned ok;
    asm volatile(
        "{\n"
        ".reg .pred p;\n"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n"
        "selp.u32 %0, 1, 0, p;\n"
        "}\n"
        : "=r"(ok)
        : "r"(smem_addr(bar)), "r"(parity)
        : "memory");
    return ok != 0;
}

}  // namespace accb
