/*
 * noalloc_scan.cu -- accb_scanl_add_i32_noalloc: the Int32 prefix sum
 * `scanl (+) seed` for callers that must not allocate device memory.
 *
 * Who needs this: code that runs where cudaMalloc is not an option -- inside
 * a latency-critical loop whose memory was sized up front, inside a library
 * callback that is forbidden to touch the allocator (an allocation may
 * synchronise the whole device), or in a process whose memory pool is owned
 * by somebody else and fully handed out.  The regular accb_scan entry point
 * keeps its tile status words in runtime-owned scratch that it allocates (and
 * grows) on demand; this entry point keeps them in a fixed array that is part
 * of the library image instead, so a call performs no allocation of any kind:
 * no cudaMalloc, no cudaFree, no stream-ordered pool, no host-side context
 * object.  The price is a hard size limit and one array per GPU that stays
 * resident from the moment the library is loaded on that GPU until exit.
 *
 * The array's name is only meaningful in device code; on the host it is a
 * stand-in symbol, so the address the kernel gets is looked up with
 * cudaGetSymbolAddress with that device current (on every call: the answer
 * belongs to the current CUDA context, not to the device ordinal).
 */
#include "common.h"

/* 32-byte status records instead of 128-byte ones keep the resident array at
 * 1 MiB for the largest supported input */
#define ACCB_SCAN_STATUS_STRIDE 4
#include "../skeletons/scan.cuh"

namespace {

constexpr long long kMaxElements = 1LL << 28; /* largest input this entry point accepts */
constexpr int kCta = 256, kRows = 8;
constexpr long long kTile = (long long)kCta * kRows * 4;
constexpr long long kMaxTiles = kMaxElements / kTile;
constexpr size_t kStatusBytes = (size_t)kMaxTiles * 8 * ACCB_SCAN_STATUS_STRIDE;
constexpr size_t kWordsOffset = kStatusBytes; /* ticket word, error word follow the status records */

/* tile status records + two control words; every GPU that loads the library holds one copy */
static __device__ __align__(256) unsigned char g_noalloc_scratch[kStatusBytes + 256];

struct AddI32 : accb::Scan<int> {
    using In = accb::types<int>;
    static __device__ __forceinline__ int get(const accb::Env &, long long, int x) { return x; }
    static __device__ __forceinline__ int combine(int a, int b) { return (int)((unsigned)a + (unsigned)b); }
};

__global__ void __launch_bounds__(kCta, 6) noalloc_scanl_add_i32(const __grid_constant__ accb_kparams p) {
    accb::scan_body<AddI32, kCta, kRows, false, false, true>(p);
}

}  // namespace

using namespace accb_rt;

extern "C" int accb_scanl_add_i32_noalloc(int device, accb_stream stream, const int32_t *in, long long n,
                                          int32_t seed, int32_t *out, unsigned int *status) {
    if (n < 0 || !out || (n > 0 && !in)) return fail(nullptr, ACCB_EINVAL, "accb_scanl_add_i32_noalloc: bad argument");
    if (n > kMaxElements)
        return fail(nullptr, ACCB_EINVAL,
                    "accb_scanl_add_i32_noalloc: %lld elements exceed the fixed scratch of this entry point "
                    "(at most %lld elements); use accb_scan for larger inputs",
                    n, kMaxElements);
    if (device < 0 || device >= 64) return fail(nullptr, ACCB_EINVAL, "accb_scanl_add_i32_noalloc: bad device %d", device);

    int previous = -1;
    int st = check_cuda(nullptr, cudaGetDevice(&previous), "cudaGetDevice");
    if (st != ACCB_OK) return st;
    if (previous != device) {
        st = check_cuda(nullptr, cudaSetDevice(device), "cudaSetDevice");
        if (st != ACCB_OK) return st;
    }
    auto restore = [&]() {
        if (previous != device) cudaSetDevice(previous);
    };

    /* The device address of the resident scratch array, asked for on EVERY call with `device` current.  The
     * array has one instance per CUDA context, so an address remembered per device ordinal would be wrong for a
     * caller that switches between the primary context and a context of its own on the same GPU, or that
     * resets the device.  Only the first call on a device does real work here (it loads the library's
     * image onto that device, which is why that call belongs before any stream capture); later calls are a
     * table look-up and allocate nothing. */
    void *scratch = nullptr;
    st = check_cuda(nullptr, cudaGetSymbolAddress(&scratch, g_noalloc_scratch), "cudaGetSymbolAddress(scratch)");
    if (st != ACCB_OK) {
        restore();
        return st;
    }

    cudaStream_t s = (cudaStream_t)stream;
    const long long ntiles = (n + kTile - 1) / kTile;
    unsigned char *base = static_cast<unsigned char *>(scratch);
    /* The array keeps what the previous call left in it.  Status records that this call
     * will read must start as "not published" and the control words at zero. */
    const size_t used = (size_t)(ntiles > 0 ? ntiles : 1) * 8 * ACCB_SCAN_STATUS_STRIDE;
    st = check_cuda(nullptr, cudaMemsetAsync(base, 0, used, s), "clearing status records");
    if (st == ACCB_OK) st = check_cuda(nullptr, cudaMemsetAsync(base + kWordsOffset, 0, 256, s), "clearing control words");
    if (st == ACCB_OK && status) st = check_cuda(nullptr, cudaMemsetAsync(status, 0, sizeof(unsigned), s), "clearing status");
    if (st != ACCB_OK) {
        restore();
        return st;
    }

    accb_kparams p;
    memset(&p, 0, sizeof p);
    p.in[0] = in;
    p.out[0] = out;
    p.out[1] = out; /* "sum" slot: the total lands at out[n] */
    p.n = n;
    p.ip[0] = ntiles;
    p.ip[1] = 0;
    p.ip[2] = 1; /* epoch: the records were just cleared, any non-zero value works */
    p.ip[3] = n;
    p.ip[4] = -1;
    p.aux[0] = base;
    p.aux[1] = base + kWordsOffset;
    p.aux[2] = status ? static_cast<void *>(status) : static_cast<void *>(base + kWordsOffset + 8);
    p.flags = ACCB_F_HAS_SEED;
    const bool aligned = ((reinterpret_cast<uintptr_t>(in) | reinterpret_cast<uintptr_t>(out)) & 15u) == 0;
    if (aligned) p.flags |= ACCB_F_VEC;
    memcpy(p.scalars, &seed, sizeof seed);

    const int grid = (int)(ntiles > 0 ? ntiles : 1);
    const size_t smem = accb::smem_offset<AddI32::In, 1, (int)kTile>::value; /* 32 KB: below the 48 KB default limit */
    noalloc_scanl_add_i32<<<grid, kCta, smem, s>>>(p);
    st = check_cuda(nullptr, cudaGetLastError(), "noalloc_scanl_add_i32 launch");
    restore();
    return st;
}
