/*
 * scan.cuh -- prefix sums: scanl, scanl1, scanl', scanr, scanr1, scanr'.
 *
 * Replaces the three-kernel reduce-then-scan of
 * Data/Array/Accelerate/CUDA/CodeGen/PrefixSum.hs:59-120,200-480 (up-sweep of
 * interval totals, scan of the totals, down-sweep that reads the input a
 * second time; host side scanOp/scan1Op/scan'Op/scanCore, Execute.hs:328-392)
 * by ONE single-pass kernel with decoupled look-back: every element is read
 * from DRAM once and written once (8 bytes per Int32 element instead of 12).
 *
 * Semantics (PrefixSum.hs:137-198, Execute.hs:326-362), with all body writes
 * aligned to the input index so that 128-bit stores stay aligned:
 *   scanl  f z : out[i] = z (+) x0 .. x(i-1)  for i in [0,n), out[n] = total
 *   scanl1 f   : out[i] = x0 .. xi
 *   scanl' f z : body as scanl, total written to a separate scalar
 *   scanr  f z : out[i] = xi .. x(n-1) (+) z  (inclusive, seeded), out[n] = z
 *   scanr1 f   : out[i] = xi .. x(n-1)
 *   scanr' f z : out[i] = x(i+1) .. x(n-1) (+) z, total separate
 * Right scans follow Data.List.scanr: the new element is the LEFT argument.
 * (The reference applies the combiner with the same argument order in both
 * directions, PrefixSum.hs:264,525-527; that only matters for a
 * non-commutative combiner and is not reproduced.)
 * Only an associative combiner is required; value order is preserved.
 *
 * Functor contract: as for folds (see fold.cuh) with a single value type:
 *   using In = accb::types<...>;  typedef T elem;
 *   static T get(env, i, in-values...);  static T combine(T, T);
 *   using Out = accb::types<...>;  static void put(T, out-references...);
 *
 * One tile of CTA * ROWS * 4 elements per block.  What bounds the kernel is
 * not the arithmetic but the wait for the predecessors' totals (without it
 * the same kernel runs at copy speed), so the design keeps as many bytes as
 * possible in flight per SM while tiles wait:
 *   - a full, 16-byte aligned tile is brought into SHARED memory by the TMA
 *     engine (cp.async.bulk, completion on an mbarrier) as the block's first
 *     action; no registers hold data while the copy or the look-back is
 *     pending, so six 32 KB tiles are resident per SM;
 *   - pass 1 over shared memory: thread sums, warp scans, block aggregate,
 *     which warp 0 publishes at once;
 *   - warp 0 looks back over its predecessors' status words (each in its own
 *     128-byte line: hundreds of warps poll them while their owners write);
 *   - pass 2 over shared memory: final values, 128-bit streaming stores.
 * A warp owns ROWS "rows" of 128 consecutive elements; lane l of row j holds
 * the 4 elements at 128*j + 4*l, so shared-memory accesses are conflict-free
 * and every global store instruction of a warp covers 512 contiguous bytes.
 * The ragged last tile (first for right scans) and unaligned arrays take a
 * slower block-scan path with scalar accesses.
 *
 * A tile only ever waits for tiles earlier in scan order.  A block's tile is
 * its block index (blocks of a 1-D grid are dispatched in index order, so the
 * tiles waited for are resident or done); with ACCB_SCAN_TICKET tiles are
 * drawn from an atomic counter instead, which makes that order explicit at
 * the price of an L2 round trip per tile.  Every wait is bounded: after
 * ACCB_SCAN_SPIN_LIMIT polls (look-back) or ACCB_SCAN_TMA_SPIN_LIMIT tries
 * (mbarrier) the kernel raises the error word and carries on, so a launch
 * always terminates.
 *
 * Several GPUs (entries scanl_bc, scanl1_bc; host side accb_peer_scan).  The
 * vector is dealt to the G GPUs in blocks of TPB tiles: global block j lives
 * on GPU j mod G, which holds its blocks one after the other.  Every GPU runs
 * this same single-pass kernel over its own blocks, so every element still
 * crosses DRAM twice (a scan over contiguous slabs needs each slab's total
 * before it can start, i.e. a third pass).  Inside a block the look-back is
 * the one above, stopped at the block's first tile.  That first tile takes its
 * exclusive prefix from a second, much shorter chain: one status record per
 * BLOCK, of which every GPU keeps a full copy in memory the other GPUs can
 * write.  The last tile of a block stores the block's aggregate -- and later
 * its inclusive prefix -- into every GPU's copy with plain peer stores over
 * NVLink (no multicast); the first tile of a block polls only its own GPU's
 * copy.  All blocks of one round (one per GPU) publish their aggregates at
 * about the same time and independently of one another, so a round costs one
 * NVLink store latency, not G of them, and several blocks per GPU are in
 * flight to hide it.  Waits that depend on another GPU are bounded by the
 * global timer (ip[9] nanoseconds).
 *
 * Runtime-owned scratch (never cleared between launches):
 *   aux[0] tile status words, aux[1] ticket counter, aux[2] error word.
 * Status words carry the launch epoch (ip[2]); words of earlier launches read
 * as "not ready".  The ticket counter only ever grows; ip[1] is its value at
 * launch.
 *   ip[0] tiles, ip[1] ticket base, ip[2] epoch, ip[3] index of the total in
 *   the "sum" slots out[Out::size..] (or -1), ip[4] index at which the seed is
 *   stored in the sum slots (or -1).
 * Block-cyclic entries in addition: ip[5] tiles per block, ip[6] number of GPUs,
 * ip[7] this GPU's rank, ip[8] epoch of the block records (the same on every
 * GPU), ip[9] time limit in ns, ip[10] byte offset of the block records in
 * every GPU's exchange buffer, ip[11] first tile of this launch (the scan may be
 * launched piece by piece, all pieces with the same epochs, so that a later
 * piece finds the records of the earlier ones); aux[3] device table of the G
 * buffers' addresses.
 */
#pragma once
#include "../cubits/accb_vec.cuh"
#include "../cubits/accb_warp.cuh"
#include "../cubits/accb_tma.cuh"
#include "../cubits/accb_status.cuh"
#include "fold.cuh"

#ifndef ACCB_SCAN_TMA
#define ACCB_SCAN_TMA 1 /* 0: hold the tile in registers instead of shared memory */
#endif
/* threads per block.  With the tile in shared memory: 256, except that elements of more than 4 bytes (over all
 * input components) take 128 threads and 9 rows -- 36 KB tiles, six per SM: Int64 2^27 at 5716 GB/s against
 * 5510 with 256 threads x 4 rows */
#ifdef ACCB_SCAN_CTA
#define ACCB_SCAN_CTA_FOR(Fn) ACCB_SCAN_CTA
#elif ACCB_SCAN_TMA
#define ACCB_SCAN_CTA_FOR(Fn) (accb::scan_cta_for<Fn::In>::value)
#else
#define ACCB_SCAN_CTA_FOR(Fn) 128
#endif
/* rows of CTA x 4 elements per tile.  With the tile in shared memory the row count follows the bytes
 * of one element over all input components, so that a tile stays at 32 KB and six blocks fit an SM */
#ifdef ACCB_SCAN_ROWS
#define ACCB_SCAN_ROWS_FOR(Fn) ACCB_SCAN_ROWS
#elif ACCB_SCAN_TMA
#define ACCB_SCAN_ROWS_FOR(Fn) (accb::scan_rows_for<Fn::In>::value)
#else
#define ACCB_SCAN_ROWS_FOR(Fn) 4
#endif
#ifndef ACCB_SCAN_TICKET
#define ACCB_SCAN_TICKET 0 /* 1: draw tiles from an atomic counter instead of the block index */
#endif
#ifndef ACCB_SCAN_DELAY_NS
#define ACCB_SCAN_DELAY_NS 0 /* pause between two polls of a tile that is not published yet */
#endif
/* resident blocks per SM the compiler must leave registers for */
#ifdef ACCB_SCAN_MINB
#define ACCB_SCAN_MINB_FOR(Fn) ACCB_SCAN_MINB
#elif ACCB_SCAN_TMA
#define ACCB_SCAN_MINB_FOR(Fn) (sizeof(Fn::elem) <= 8 ? 6 : 3)
#else
#define ACCB_SCAN_MINB_FOR(Fn) (sizeof(Fn::elem) <= 4 ? 12 : (sizeof(Fn::elem) <= 8 ? 6 : 3))
#endif
/* The block-cyclic entries (several GPUs) take tiles of 36 KB from 128 threads: six of them fill an SM's shared
 * memory (216 KB in flight instead of 192), which buys back the longer wait of a tile whose predecessors sit on
 * another GPU.  Measured on two GPUs, 2^28 Int32 each: 0.368 ms against 0.385 ms with the 32 KB tiles. */
#ifndef ACCB_SCAN_BC_CTA
#define ACCB_SCAN_BC_CTA 128
#endif
#ifdef ACCB_SCAN_BC_ROWS
#define ACCB_SCAN_BC_ROWS_FOR(Fn) ACCB_SCAN_BC_ROWS
#else
#define ACCB_SCAN_BC_ROWS_FOR(Fn) (accb::scan_bc_rows_for<Fn::In>::value)
#endif
#ifndef ACCB_SCAN_BC_MINB
#define ACCB_SCAN_BC_MINB 6
#endif
#ifndef ACCB_SCAN_SPIN_LIMIT
#define ACCB_SCAN_SPIN_LIMIT (1 << 20)
#endif
#ifndef ACCB_SCAN_TMA_SPIN_LIMIT
#define ACCB_SCAN_TMA_SPIN_LIMIT (1 << 16)
#endif

namespace accb {

template <class T>
struct Scan {
    typedef T elem;
    typedef T acc;
    typedef types<T> Out;
    static __device__ __forceinline__ void put(T r, T &o) { o = r; }
};

template <class Fn, bool RIGHT>
struct ScanOp {
    typedef typename Fn::elem T;
    /* a precedes b in scan order */
    __device__ __forceinline__ T operator()(T a, T b) const {
        if constexpr (RIGHT)
            return Fn::combine(b, a);
        else
            return Fn::combine(a, b);
    }
    __device__ __forceinline__ Opt<T> operator()(Opt<T> a, Opt<T> b) const {
        Opt<T> r;
        r.have = a.have | b.have;
        r.v = (a.have && b.have) ? (*this)(a.v, b.v) : (a.have ? a.v : b.v);
        return r;
    }
};

template <class Fn, int... O>
__device__ __forceinline__ void scan_put_sum(const accb_kparams &p, long long j, typename Fn::elem r,
                                             std::integer_sequence<int, O...>) {
    regs<1, typename Fn::Out> b;
    Fn::put(r, comp<O>(b)[0]...);
    store_one(p.out + Fn::Out::size, j, b);
}

template <class Fn, int N, int... O>
__device__ __forceinline__ void scan_put_vec(typename Fn::elem (&y)[N], regs<N, typename Fn::Out> &b,
                                             std::integer_sequence<int, O...>) {
#pragma unroll
    for (int k = 0; k < N; ++k) Fn::put(y[k], comp<O>(b)[k]...);
}

/* ---- decoupled look-back, run by warp 0 of the block that owns tile t.
 * `agg` is the tile's aggregate.  Publishes the aggregate, gathers the
 * exclusive prefix of the tile from its predecessors, publishes the inclusive
 * prefix, writes the total / seed where the host asked for them, and returns
 * the exclusive prefix (have == 0: the first tile of an unseeded scan). ---- */
template <class Fn, bool RIGHT>
__device__ __forceinline__ Opt<typename Fn::elem> scan_lookback(const accb_kparams &p, long long t,
                                                                long long ntiles, typename Fn::elem agg) {
    typedef typename Fn::elem T;
    typedef Opt<T> O;
    const ScanOp<Fn, RIGHT> op;
    const auto oseq = std::make_integer_sequence<int, Fn::Out::size>();
    const bool seeded = (p.flags & ACCB_F_HAS_SEED) != 0;
    const unsigned epoch = (unsigned)p.ip[2];
    const TileStatus<T> status(p.aux[0]);
    unsigned int *err = static_cast<unsigned int *>(p.aux[2]);
    const int lane = lane_id();
    O pre;
    pre.have = 0;
    if (t == 0) {
        if (seeded) {
            pre.v = fold_seed<Fn>(p);
            pre.have = 1;
        }
    } else {
        if (lane == 0) status.publish(t, (epoch << 2) | ST_AGG, agg);
        long long look = t - 1; /* lane l examines tile look - l */
        int spins = 0;
        bool done = false;
        while (!done) {
            const long long idx = look - lane;
            T v;
            unsigned flag = 0;
            bool ready = idx < 0;
            /* every lane polls its own predecessor until it is published */
            while (true) {
                if (!ready) {
                    flag = status.peek(idx, v);
                    ready = (flag >> 2) == epoch && (flag & 3u) != 0;
                }
                if (__all_sync(FULL, ready)) break;
                __nanosleep(ACCB_SCAN_DELAY_NS);
                /* give up after the limit, or at once when another tile already gave up */
                if (++spins > ACCB_SCAN_SPIN_LIMIT ||
                    ((spins & 255) == 0 && *static_cast<volatile unsigned int *>(err) != 0u)) {
                    if (lane == 0) atomicExch(err, 1u);
                    if (!ready) flag = (epoch << 2) | ST_PREFIX; /* the result is flagged invalid */
                    ready = true;
                }
            }
            const bool is_pre = idx >= 0 && (flag & 3u) == ST_PREFIX;
            const unsigned pm = __ballot_sync(FULL, is_pre);
            const int first = pm ? __ffs(pm) - 1 : 32; /* nearest tile with a full prefix */
            O win;
            win.v = v;
            win.have = (idx >= 0) && (lane <= first);
            /* lanes hold ever earlier tiles: combine far-to-near */
#pragma unroll
            for (int d = 1; d < 32; d <<= 1) {
                O o = shfl_down(win, d);
                if (lane + d < 32) win = op(o, win);
            }
            win = shfl_idx(win, 0);
            pre = op(win, pre);
            done = pm != 0 || look < 32;
            look -= 32;
        }
    }
    if (lane == 0) {
        const T incl = pre.have ? op(pre.v, agg) : agg;
#ifdef ACCB_SCAN_TEST_DROP_TILE0
        /* test hook: the first tile never publishes, so every other tile's wait runs
         * into its bound; used to check that the error word is raised and the launch
         * still terminates */
        if (t != 0)
#endif
            status.publish(t, (epoch << 2) | ST_PREFIX, incl);
        if (t == ntiles - 1 && p.ip[3] >= 0) scan_put_sum<Fn>(p, p.ip[3], incl, oseq);
        if (t == 0 && p.ip[4] >= 0 && seeded) scan_put_sum<Fn>(p, p.ip[4], fold_seed<Fn>(p), oseq);
    }
    return pre;
}

/* ---- block records of the block-cyclic scan: one per global block, dense, read and written with system
 * scope because the writers are other GPUs.  Flag {epoch << 2 | state} and value travel in one store: a 64-bit
 * word for values up to 4 bytes, a 128-bit word for 8-byte values.  Records are ACCB_SCAN_BLOCK_RECORD bytes apart. ---- */
#ifndef ACCB_SCAN_BLOCK_RECORD
#define ACCB_SCAN_BLOCK_RECORD 128 /* bytes from one block record to the next: a line of its own (the host sizes the scratch for this) */
#endif
#ifndef ACCB_SCAN_BLOCK_DELAY_NS
#define ACCB_SCAN_BLOCK_DELAY_NS 100 /* pause between two polls of a block record that is not published yet */
#endif
constexpr int kBlockRecordBytes = ACCB_SCAN_BLOCK_RECORD;

template <class T>
struct BlockStatus {
    static_assert(sizeof(T) <= 8, "block records carry values of up to 8 bytes");
    static __device__ __forceinline__ void publish(unsigned char *base, long long j, unsigned flag, T v) {
        unsigned char *rec = base + j * kBlockRecordBytes;
        if constexpr (sizeof(T) <= 4) {
            unsigned bits = 0;
            memcpy(&bits, &v, sizeof(T));
            const unsigned long long word = ((unsigned long long)flag << 32) | bits;
            asm volatile("st.relaxed.sys.global.u64 [%0], %1;" ::"l"(rec), "l"(word) : "memory");
        } else {
            unsigned long long bits;
            memcpy(&bits, &v, 8);
            const unsigned long long head = (unsigned long long)flag << 32;
            asm volatile("{ .reg .b128 q; mov.b128 q, {%1, %2}; st.relaxed.sys.global.b128 [%0], q; }" ::"l"(rec), "l"(head),
                         "l"(bits)
                         : "memory");
        }
    }
    static __device__ __forceinline__ unsigned peek(const unsigned char *base, long long j, T &v) {
        const unsigned char *rec = base + j * kBlockRecordBytes;
        if constexpr (sizeof(T) <= 4) {
            unsigned long long word;
            asm volatile("ld.relaxed.sys.global.u64 %0, [%1];" : "=l"(word) : "l"(rec) : "memory");
            const unsigned bits = (unsigned)word;
            memcpy(&v, &bits, sizeof(T));
            return (unsigned)(word >> 32);
        } else {
            unsigned long long head, bits;
            asm volatile("{ .reg .b128 q; ld.relaxed.sys.global.b128 q, [%2]; mov.b128 {%0, %1}, q; }"
                         : "=l"(head), "=l"(bits)
                         : "l"(rec)
                         : "memory");
            memcpy(&v, &bits, 8);
            return (unsigned)(head >> 32);
        }
    }
};

__device__ __forceinline__ unsigned long long scan_global_ns() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}

/* combines a look-back window: lane l holds the record of the (l+1)-th nearest predecessor, `first` is the
 * nearest lane whose record is a full prefix (32: none); returns, in every lane, the combination of the
 * records up to and including that one, far to near */
template <class Fn>
__device__ __forceinline__ Opt<typename Fn::elem> scan_window(typename Fn::elem v, bool inside, int first) {
    const ScanOp<Fn, false> op;
    const int lane = lane_id();
    Opt<typename Fn::elem> win;
    win.v = v;
    win.have = inside && (lane <= first);
#pragma unroll
    for (int d = 1; d < 32; d <<= 1) {
        Opt<typename Fn::elem> o = shfl_down(win, d);
        if (lane + d < 32) win = op(o, win);
    }
    return shfl_idx(win, 0);
}

/* ---- look-back of the block-cyclic scan (left scans), run by warp 0 of the block that owns LOCAL tile t.
 * Tile t is tile k = t mod TPB of local block t / TPB, i.e. of global block j = (t / TPB) * G + g.  Its
 * predecessors in scan order are the earlier tiles of its own block and then the blocks j - 1, j - 2, ..:
 *   1. the look-back above over the tile records t - 1 .. t - k (this GPU's); it ends early at a tile that
 *      already knows its inclusive prefix (which contains everything before the block);
 *   2. otherwise it goes on over the BLOCK records j - 1, j - 2, .. of this GPU's copy: aggregates until a
 *      prefix (block 0 only ever publishes a prefix, which contains the seed).
 * Every tile walks both chains by itself, so nobody waits for the block's first tile: a tile is two dependent
 * polls behind the moment its predecessors' aggregates exist, wherever in the block it sits.  The LAST tile of
 * a block knows the block's aggregate once step 1 has reached the block's first tile and stores it into every
 * GPU's block records before step 2; at the end it stores the block's inclusive prefix there. ---- */
template <class Fn>
__device__ __forceinline__ Opt<typename Fn::elem> scan_lookback_bc(const accb_kparams &p, long long t,
                                                                   long long ntiles, typename Fn::elem agg) {
    typedef typename Fn::elem T;
    typedef Opt<T> O;
    const ScanOp<Fn, false> op;
    const auto oseq = std::make_integer_sequence<int, Fn::Out::size>();
    O pre;
    pre.have = 0;
    if constexpr (sizeof(T) <= 8) {
        const bool seeded = (p.flags & ACCB_F_HAS_SEED) != 0;
        const unsigned epoch = (unsigned)p.ip[2]; /* of this GPU's tile records */
        const unsigned pe = (unsigned)p.ip[8];    /* of the block records */
        const TileStatus<T> status(p.aux[0]);
        unsigned int *err = static_cast<unsigned int *>(p.aux[2]);
        const int lane = lane_id();
        const long long TPB = p.ip[5];
        const int G = (int)p.ip[6], g = (int)p.ip[7];
        const unsigned long long limit_ns = (unsigned long long)p.ip[9];
        const long long k = t % TPB, t0 = t - k;
        const long long j = (t / TPB) * G + g;
        const bool last_of_block = (k == TPB - 1) || (t == ntiles - 1);
        unsigned char *const *bases = static_cast<unsigned char *const *>(p.aux[3]);
        const long long boff = p.ip[10];
        /* all lanes hold the same flag and value: lane l stores into GPU l's copy (l + 32, ...) */
        auto publish_block = [&](unsigned state, T v) {
            for (int r = lane; r < G; r += 32) BlockStatus<T>::publish(bases[r] + boff, j, (pe << 2) | state, v);
        };
        const unsigned long long t_start = scan_global_ns();
        unsigned spins = 0;
        /* bounded waits: true once the time limit has passed, another tile has given up, or the poll count
         * says the timer itself cannot be trusted (called by all lanes alike) */
        auto expired = [&]() -> bool {
            if ((++spins & 63u) != 0) return false;
            return spins > (1u << 24) || *static_cast<volatile unsigned int *>(err) != 0u ||
                   scan_global_ns() - t_start > limit_ns;
        };

        bool resolved = false; /* `pre` is the exclusive prefix of the tile */
        if (t == 0 && j == 0) { /* nothing precedes the very first tile but the seed */
            if (seeded) {
                pre.v = fold_seed<Fn>(p);
                pre.have = 1;
            }
            resolved = true;
        } else if (lane == 0) {
            status.publish(t, (epoch << 2) | ST_AGG, agg);
        }
        /* step 1: the earlier tiles of this block */
        long long look = t - 1; /* lane l examines tile look - l */
        while (!resolved && look >= t0) {
            const long long idx = look - lane;
            const bool inside = idx >= t0;
            T v;
            unsigned flag = 0;
            bool ready = !inside;
            while (true) {
                if (!ready) {
                    flag = status.peek(idx, v);
                    ready = (flag >> 2) == epoch && (flag & 3u) != 0;
                }
                if (__all_sync(FULL, ready)) break;
                __nanosleep(ACCB_SCAN_DELAY_NS);
                if (expired()) {
                    if (lane == 0) atomicExch(err, 1u);
                    if (!ready) flag = (epoch << 2) | ST_PREFIX; /* the result is flagged invalid */
                    ready = true;
                }
            }
            const unsigned pm = __ballot_sync(FULL, inside && (flag & 3u) == ST_PREFIX);
            pre = op(scan_window<Fn>(v, inside, pm ? __ffs(pm) - 1 : 32), pre);
            resolved = pm != 0;
            look -= 32;
        }
        if (!resolved) {
            /* `pre` is what the block holds ahead of this tile.  The last tile now knows the block's aggregate,
             * ahead of its prefix: the blocks behind it, on the other GPUs, can use it at once. */
            if (last_of_block) publish_block(ST_AGG, pre.have ? op(pre.v, agg) : agg);
            /* step 2: the blocks before this one (j > 0: block 0 starts with the very first tile, whose record is
             * a prefix from the start, so step 1 cannot end here for it unless a wait gave up) */
            const unsigned char *mine = bases[g] + boff;
            look = j - 1; /* lane l examines block look - l */
            while (!resolved && look >= 0) {
                const long long idx = look - lane;
                T v;
                unsigned flag = 0;
                bool ready = idx < 0;
                while (true) {
                    if (!ready) {
                        flag = BlockStatus<T>::peek(mine, idx, v);
                        ready = (flag >> 2) == pe && (flag & 3u) != 0;
                    }
                    if (__all_sync(FULL, ready)) break;
                    __nanosleep(ACCB_SCAN_BLOCK_DELAY_NS);
                    if (expired()) {
                        if (lane == 0) atomicExch(err, 1u);
                        if (!ready) flag = (pe << 2) | ST_PREFIX;
                        ready = true;
                    }
                }
                const unsigned pm = __ballot_sync(FULL, idx >= 0 && (flag & 3u) == ST_PREFIX);
                pre = op(scan_window<Fn>(v, idx >= 0, pm ? __ffs(pm) - 1 : 32), pre);
                resolved = pm != 0;
                look -= 32;
            }
        }
        const T incl = pre.have ? op(pre.v, agg) : agg;
        if (lane == 0) status.publish(t, (epoch << 2) | ST_PREFIX, incl);
        if (last_of_block) publish_block(ST_PREFIX, incl);
        /* the host passes a total index only to the GPU that owns the last block */
        if (lane == 0 && t == ntiles - 1 && p.ip[3] >= 0) scan_put_sum<Fn>(p, p.ip[3], incl, oseq);
    }
    return pre;
}

/* warp prefix and block aggregate from the per-warp totals in shared memory
 * (all NW warps hold data) */
template <class Fn, bool RIGHT, int NW>
__device__ __forceinline__ void scan_block_level(const typename Fn::elem *s_warp, int w,
                                                 Opt<typename Fn::elem> &wpre, typename Fn::elem &agg) {
    const ScanOp<Fn, RIGHT> op;
    wpre.have = 0;
    agg = s_warp[0];
#pragma unroll
    for (int k = 0; k < NW; ++k) {
        if (k < w) {
            wpre.v = wpre.have ? op(wpre.v, s_warp[k]) : s_warp[k];
            wpre.have = 1;
        }
        if (k > 0) agg = op(agg, s_warp[k]);
    }
}

/* ---- full, aligned tile.  SMEM: the raw inputs sit in shared memory (put
 * there by the TMA engine) and are read twice; otherwise they are loaded into
 * registers once and kept there. ---- */
/* tile shape: 256 threads x 8 rows (32 KB) for up to 4 bytes per element (all components), 128 threads x 9 rows
 * (36 KB) up to 8, else 256 x 2 */
template <class L>
struct scan_rows_for {
    static constexpr int bpe = smem_offset<L, L::size, 128>::value / 128;
    static constexpr int value = bpe <= 4 ? 8 : (bpe <= 8 ? 9 : 2);
};
template <class L>
struct scan_cta_for {
    static constexpr int bpe = smem_offset<L, L::size, 128>::value / 128;
    static constexpr int value = (bpe > 4 && bpe <= 8) ? 128 : 256;
};

/* tile rows of the block-cyclic entries, 128 threads: 36 KB of input per tile */
template <class L>
struct scan_bc_rows_for {
    static constexpr int bpe = smem_offset<L, L::size, 128>::value / 128;
    static constexpr int value = bpe <= 4 ? 18 : (bpe <= 8 ? 9 : 4);
};

/* 4 consecutive values of one component from shared memory.  8-byte values make 32 bytes per
 * thread: read as two 16-byte halves at a 32-byte thread stride, threads l and l+4 of a quarter warp
 * would hit the same banks, so every other group of 4 threads takes its halves in the opposite
 * order (and swaps them back in registers). */
template <class T>
__device__ __forceinline__ void smem_load4(const T *base, int vi, T (&r)[V]) {
    if constexpr (sizeof(T) == 8) {
        const uint4 *q = reinterpret_cast<const uint4 *>(base) + 2 * vi;
        const int flip = (vi >> 2) & 1;
        const uint4 a = q[flip], b = q[flip ^ 1];
        const uint4 lo = flip ? b : a, hi = flip ? a : b;
        memcpy(&r[0], &lo, 16);
        memcpy(&r[2], &hi, 16);
    } else {
        load4<Cache::Default>(base, vi, r);
    }
}

template <class L, int TILE, int... I>
__device__ __forceinline__ void smem_load_row(const unsigned char *s, int vi, regs<V, L> &r,
                                              std::integer_sequence<int, I...>) {
    (smem_load4(reinterpret_cast<const typename type_at<I, L>::type *>(s + smem_offset<L, I, TILE>::value), vi,
                comp<I>(r)),
     ...);
}

template <class L, int TILE, int... I>
__device__ __forceinline__ void smem_issue_tma(unsigned char *s, const void *const *slots, long long base,
                                               unsigned long long *bar, std::integer_sequence<int, I...>) {
    constexpr unsigned total = (unsigned)((TILE * (int)sizeof(typename type_at<I, L>::type)) + ... + 0);
    mbar_expect_tx(bar, total);
    (bulk_g2s(s + smem_offset<L, I, TILE>::value,
              static_cast<const typename type_at<I, L>::type *>(slots[I]) + base,
              (unsigned)(TILE * sizeof(typename type_at<I, L>::type)), bar),
     ...);
}

template <class Fn, int CTA, int ROWS, bool RIGHT, bool INCL, bool SMEM, bool BC = false>
__device__ __forceinline__ void scan_tile_full(const accb_kparams &p, long long t, long long ntiles, long long base,
                                               typename Fn::elem *s_warp, Opt<typename Fn::elem> *s_prefix,
                                               const unsigned char *s_data) {
    typedef typename Fn::elem T;
    typedef typename Fn::In In;
    typedef typename Fn::Out Out;
    typedef Opt<T> O;
    constexpr int NW = CTA / 32;
    constexpr int TILE = CTA * ROWS * V;
    constexpr int TILE_VECS = CTA * ROWS;
    const ScanOp<Fn, RIGHT> op;
    const Env env(p);
    const auto iseq = std::make_integer_sequence<int, In::size>();
    const auto oseq = std::make_integer_sequence<int, Out::size>();
    const int lane = lane_id(), w = warp_id();

    /* x(j) = the 4 values of row j in scan order: logical element
     * (w*ROWS*128 + j*128 + lane*4 + k) of the tile */
    regs<V, In> a[SMEM ? 1 : ROWS];
    if constexpr (!SMEM) {
#pragma unroll
        for (int j = 0; j < ROWS; ++j) {
            const int lv = w * (ROWS * 32) + j * 32 + lane;
            load_all(p.in, base / V + (RIGHT ? (TILE_VECS - 1 - lv) : lv), a[j]);
        }
    }
    auto row = [&](int j, T (&x)[V]) {
        const int lv = w * (ROWS * 32) + j * 32 + lane;
        const int tv = RIGHT ? (TILE_VECS - 1 - lv) : lv; /* vector index inside the tile, in memory order */
        T tmp[V];
        if constexpr (SMEM) {
            smem_load_row<In, TILE>(s_data, tv, a[0], iseq);
            fold_get<Fn>(env, base + (long long)tv * V, a[0], tmp, iseq);
        } else {
            fold_get<Fn>(env, base + (long long)tv * V, a[j], tmp, iseq);
        }
#pragma unroll
        for (int k = 0; k < V; ++k) x[k] = RIGHT ? tmp[V - 1 - k] : tmp[k];
    };

    /* ---- pass 1: thread sums, a warp scan per row ---- */
    T ex[ROWS]; /* exclusive prefix of this thread's vector inside the warp chunk; none for (j, lane) == (0, 0) */
    T wtot;     /* total of the warp chunk */
#pragma unroll
    for (int j = 0; j < ROWS; ++j) {
        T x[V];
        row(j, x);
        const T s = op(op(x[0], x[1]), op(x[2], x[3]));
        const T inc = warp_scan_inclusive(s, op);
        const T up = shfl_up(inc, 1);
        const T last = shfl_idx(inc, 31);
        if (j == 0) {
            ex[j] = up;
            wtot = last;
        } else {
            ex[j] = lane > 0 ? op(wtot, up) : wtot;
            wtot = op(wtot, last);
        }
    }

    /* ---- block level, look-back ---- */
    if (lane == 0) s_warp[w] = wtot;
    __syncthreads();
    O wpre;
    T agg;
    scan_block_level<Fn, RIGHT, NW>(s_warp, w, wpre, agg);
    if (w == 0) {
        O pre;
        if constexpr (BC)
            pre = scan_lookback_bc<Fn>(p, t, ntiles, agg);
        else
            pre = scan_lookback<Fn, RIGHT>(p, t, ntiles, agg);
        if (lane == 0) *s_prefix = pre;
    }
    __syncthreads();
    const O tile_pre = op(*s_prefix, wpre);

    /* ---- pass 2: final values and store ---- */
#pragma unroll
    for (int j = 0; j < ROWS; ++j) {
        T x[V];
        row(j, x);
        O run = tile_pre;
        if (j > 0 || lane > 0) {
            run.v = run.have ? op(run.v, ex[j]) : ex[j];
            run.have = 1;
        }
        T y[V];
#pragma unroll
        for (int k = 0; k < V; ++k) {
            const T nxt = run.have ? op(run.v, x[k]) : x[k];
            y[RIGHT ? V - 1 - k : k] = INCL ? nxt : run.v;
            run.v = nxt;
            run.have = 1;
        }
        regs<V, Out> b;
        scan_put_vec<Fn>(y, b, oseq);
        const int lv = w * (ROWS * 32) + j * 32 + lane;
        store_all(p.out, base / V + (RIGHT ? (TILE_VECS - 1 - lv) : lv), b);
    }
}

/* ---- ragged tile (len <= TILE valid elements at `base`) or unaligned
 * arrays: scalar accesses, the tile walked twice in chunks of CTA elements
 * (once for the aggregate, once -- after the look-back -- for the values). ---- */
template <class Fn, int CTA, int ROWS, bool RIGHT, bool INCL, bool BC = false>
__device__ __forceinline__ void scan_tile_ragged(const accb_kparams &p, long long t, long long ntiles,
                                                 long long base, long long len,
                                                 Opt<typename Fn::elem> *s_opt /* CTA/32 + 1 slots */) {
    typedef typename Fn::elem T;
    typedef typename Fn::In In;
    typedef typename Fn::Out Out;
    typedef Opt<T> O;
    constexpr int NW = CTA / 32;
    const ScanOp<Fn, RIGHT> op;
    const Env env(p);
    const auto iseq = std::make_integer_sequence<int, In::size>();
    const auto oseq = std::make_integer_sequence<int, Out::size>();
    const int lane = lane_id(), w = warp_id();
    /* logical position q (scan order) <-> memory offset */
    auto fetch = [&](long long q) {
        O e;
        e.have = q < len;
        if (e.have) {
            const long long i = base + (RIGHT ? len - 1 - q : q);
            regs<1, In> a;
            T tmp[1];
            load_one(p.in, i, a);
            fold_get<Fn>(env, i, a, tmp, iseq);
            e.v = tmp[0];
        }
        return e;
    };

    /* aggregate of the tile, chunk by chunk so that value order is kept */
    O carry;
    carry.have = 0;
    const long long nchunk = (len + CTA - 1) / CTA;
    for (long long c = 0; c < nchunk; ++c) {
        O e = fetch(c * CTA + threadIdx.x);
        O inc = warp_scan_inclusive(e, op);
        if (lane == 31) s_opt[w] = inc;
        __syncthreads();
        O tot;
        tot.have = 0;
#pragma unroll
        for (int k = 0; k < NW; ++k) tot = op(tot, s_opt[k]);
        carry = op(carry, tot);
        __syncthreads();
    }
    if (w == 0) {
        O pre; /* len >= 1, so carry.have */
        if constexpr (BC)
            pre = scan_lookback_bc<Fn>(p, t, ntiles, carry.v);
        else
            pre = scan_lookback<Fn, RIGHT>(p, t, ntiles, carry.v);
        if (lane == 0) s_opt[NW] = pre;
    }
    __syncthreads();
    O run = s_opt[NW]; /* exclusive prefix of the chunk being written */
    __syncthreads();
    for (long long c = 0; c < nchunk; ++c) {
        const long long q = c * CTA + threadIdx.x;
        O e = fetch(q);
        O inc = warp_scan_inclusive(e, op);
        if (lane == 31) s_opt[w] = inc;
        __syncthreads();
        O before = run; /* everything ahead of this warp */
        O tot;
        tot.have = 0;
#pragma unroll
        for (int k = 0; k < NW; ++k) {
            if (k < w) before = op(before, s_opt[k]);
            tot = op(tot, s_opt[k]);
        }
        O up = shfl_up(inc, 1);
        if (lane == 0) up.have = 0;
        const O excl = op(before, up);
        if (e.have) {
            const T incl = excl.have ? op(excl.v, e.v) : e.v;
            T y[1] = {INCL ? incl : excl.v};
            regs<1, Out> b;
            scan_put_vec<Fn>(y, b, oseq);
            store_one(p.out, base + (RIGHT ? len - 1 - q : q), b);
        }
        run = op(run, tot);
        __syncthreads();
    }
}

template <class Fn, int CTA, int ROWS, bool RIGHT, bool INCL, bool SMEM, bool BC = false>
__device__ __forceinline__ void scan_body(const accb_kparams &p) {
    static_assert(!(BC && RIGHT), "the block-cyclic form serves left scans");
    typedef typename Fn::elem T;
    typedef typename Fn::In In;
    constexpr int NW = CTA / 32;
    constexpr int TILE = CTA * ROWS * V;
    const auto iseq = std::make_integer_sequence<int, In::size>();
    const auto oseq = std::make_integer_sequence<int, Fn::Out::size>();
    __shared__ T s_warp[NW];
    __shared__ Opt<T> s_opt[NW + 1];
    __shared__ long long s_tile;
    __shared__ __align__(8) unsigned long long s_bar;
    extern __shared__ __align__(128) unsigned char s_data[];

    const long long n = p.n;
    const long long ntiles = p.ip[0];

    if (n == 0) { /* empty input: only the seed survives */
        if (blockIdx.x == 0 && threadIdx.x == 0 && (p.flags & ACCB_F_HAS_SEED)) {
            const T z = fold_seed<Fn>(p);
            if (p.ip[3] >= 0) scan_put_sum<Fn>(p, p.ip[3], z, oseq);
            if (p.ip[4] >= 0) scan_put_sum<Fn>(p, p.ip[4], z, oseq);
        }
        return;
    }

    long long t; /* position in scan order */
    if constexpr (ACCB_SCAN_TICKET != 0) {
        unsigned int *ticket = static_cast<unsigned int *>(p.aux[1]);
        if (threadIdx.x == 0) s_tile = (long long)(unsigned)(atomicAdd(ticket, 1u) - (unsigned)p.ip[1]);
        __syncthreads();
        t = s_tile;
    } else {
        t = blockIdx.x;
    }
    if constexpr (BC) t += p.ip[11]; /* a launch may cover the tiles from ip[11] on: the scan launched piece by piece */
    if (t >= ntiles) return;
    const long long base = (RIGHT ? ntiles - 1 - t : t) * TILE; /* position in memory */
    const long long len = (n - base) < TILE ? (n - base) : (long long)TILE;
    const bool full = (p.flags & ACCB_F_VEC) != 0 && len == TILE;

    if (!full) {
        scan_tile_ragged<Fn, CTA, ROWS, RIGHT, INCL, BC>(p, t, ntiles, base, len, s_opt);
        return;
    }
    if constexpr (SMEM) {
        unsigned int *err = static_cast<unsigned int *>(p.aux[2]);
        /* the whole tile by TMA, completion counted in bytes on the mbarrier */
        if (threadIdx.x == 0) {
            mbar_init(&s_bar, 1);
            fence_mbar_init();
        }
        __syncthreads();
        if (threadIdx.x == 0) smem_issue_tma<In, TILE>(s_data, p.in, base, &s_bar, iseq);
        int tries = 0;
        while (!mbar_try_wait(&s_bar, 0)) {
            if (++tries > ACCB_SCAN_TMA_SPIN_LIMIT) { /* bounded: flag the result invalid and go on */
                atomicExch(err, 1u);
                break;
            }
        }
    }
    scan_tile_full<Fn, CTA, ROWS, RIGHT, INCL, SMEM, BC>(p, t, ntiles, base, s_warp, &s_opt[NW], s_data);
}

}  // namespace accb

/* Entry points named after the reference's kernels (PrefixSum.hs:208,313):
 * exclusive and inclusive, left and right. */
#define ACCB_SCAN_ENTRY(Fn, name, right, incl)                                                 \
    extern "C" __global__ void __launch_bounds__(ACCB_SCAN_CTA_FOR(Fn), ACCB_SCAN_MINB_FOR(Fn)) \
        name(const __grid_constant__ accb_kparams p) {                                         \
        accb::scan_body<Fn, ACCB_SCAN_CTA_FOR(Fn), ACCB_SCAN_ROWS_FOR(Fn), right, incl, ACCB_SCAN_TMA != 0, false>(p); \
    }
#define ACCB_SCAN_BC_ENTRY(Fn, name, incl)                                                     \
    extern "C" __global__ void __launch_bounds__(ACCB_SCAN_BC_CTA, ACCB_SCAN_BC_MINB)          \
        name(const __grid_constant__ accb_kparams p) {                                         \
        accb::scan_body<Fn, ACCB_SCAN_BC_CTA, ACCB_SCAN_BC_ROWS_FOR(Fn), false, incl, true, true>(p); \
    }

/* metadata: record bytes, tile elements, rows, ticket mode, dynamic shared memory, bytes of a value; of the
 * block-cyclic entries: threads, tile elements, dynamic shared memory */
#define ACCB_INSTANTIATE_SCAN(Fn)                                                              \
    ACCB_META12(5, ACCB_SCAN_CTA_FOR(Fn), accb::TileStatus<Fn::elem>::kBytes,                  \
               ACCB_SCAN_CTA_FOR(Fn) * ACCB_SCAN_ROWS_FOR(Fn) * 4, ACCB_SCAN_ROWS_FOR(Fn), ACCB_SCAN_TICKET ? 2 : 0,   \
               ACCB_SCAN_TMA ? (accb::smem_offset<Fn::In, Fn::In::size,                        \
                                                  ACCB_SCAN_CTA_FOR(Fn) * ACCB_SCAN_ROWS_FOR(Fn) * 4>::value)  \
                             : 0,                                                              \
               sizeof(Fn::elem), ACCB_SCAN_BC_CTA, ACCB_SCAN_BC_CTA * ACCB_SCAN_BC_ROWS_FOR(Fn) * 4,  \
               (accb::smem_offset<Fn::In, Fn::In::size, ACCB_SCAN_BC_CTA * ACCB_SCAN_BC_ROWS_FOR(Fn) * 4>::value), Fn::In::size) \
    ACCB_SCAN_ENTRY(Fn, scanl, false, false)                                                   \
    ACCB_SCAN_ENTRY(Fn, scanl1, false, true)                                                   \
    ACCB_SCAN_ENTRY(Fn, scanr, true, false)                                                    \
    ACCB_SCAN_ENTRY(Fn, scanr1, true, true)                                                    \
    ACCB_SCAN_BC_ENTRY(Fn, scanl_bc, false)                                                    \
    ACCB_SCAN_BC_ENTRY(Fn, scanl1_bc, true)
