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

/* ---- tiled copies through a tensor map (cp.async.bulk.tensor): the host encodes the map (cuTensorMapEncodeTiled)
 * and passes it as a __grid_constant__ kernel parameter; the kernel only needs its address.  Always this GPU's
 * own memory, never with cluster multicast.  The innermost coordinate times the element size must be a multiple
 * of 16 bytes. ---- */
struct alignas(64) TensorMap {
    unsigned long long opaque[16]; /* the 128 bytes of a CUtensorMap */
};

/* global -> shared: the box at (x, y) of the tensor, completion counted in bytes on `bar` */
__device__ __forceinline__ void tensor_g2s_2d(void *dst, const TensorMap *map, int x, int y, unsigned long long *bar) {
    asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];" ::"r"(
                     smem_addr(dst)),
                 "l"(map), "r"(smem_addr(bar)), "r"(x), "r"(y)
                 : "memory");
}

/* shared -> global: the box at (x, y); what lies outside the tensor is not written */
__device__ __forceinline__ void tensor_s2g_2d(const TensorMap *map, int x, int y, const void *src) {
    asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.bulk_group [%0, {%2, %3}], [%1];" ::"l"(map), "r"(smem_addr(src)),
                 "r"(x), "r"(y)
                 : "memory");
}

/* writes of this thread to shared memory become visible to the copy engine */
__device__ __forceinline__ void fence_async_shared() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }

/* closes the group of stores issued so far; wait until the engine has READ their shared memory */
__device__ __forceinline__ void bulk_commit() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
__device__ __forceinline__ void bulk_wait_read() { asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory"); }

}  // namespace accb
