// BCSR SpMM, tcgen05 path (sm_100a): C[W*16, N] = A_bcsr * B[K, N] for fp16/bf16, N % 128 == 0.
//
// Replaces tcspmm_base_kernel (core/include/spmm_tc.cuh:40-195).  Every 16x8 BCSR tile is a small
// dense contraction, so the product is run transposed on the 5th-generation tensor cores:
//
//     D^T[128 features x 16 window rows] += Hg^T[128 x 16 slots] * A^T[16 slots x 16 rows]
//
// i.e. one tcgen05.mma (M = 128, N = 16, K = 16) per pair of tiles and 128-feature slab:
//   * the B operand of the instruction is the raw pair of BCSR tiles: an fp16 [16][8] tile is two
//     8x16-byte core matrices, consecutive tiles are 256 bytes apart, so the tiles are streamed
//     from HBM by TMA bulk copies (cp.async.bulk) straight into a K-major, no-swizzle operand;
//   * the A operand is the gathered rows of the dense matrix, MN-major with the 128-byte swizzle:
//     a gathered row is two 128-byte lines, fetched from L2 by the TMA unit in gather mode
//     (cp.async.bulk.tensor ... tile::gather4: four rows by 64 features per copy, no registers, no
//     per-thread address arithmetic); a column id of -1 is out of bounds and reads zeros;
//   * accumulators live in tensor memory (16 fp32 columns per slab), four deep, so the epilogue
//     of one window overlaps the MMAs of the next.
//
// Persistent CTAs each own a contiguous range of the global tile array (equal tile counts, so
// power-law window lengths do not matter); the pieces of a window cut by a range boundary go to
// scratch as fp32 partial tiles and the CTA that finishes its piece last sums them in CTA order.
//
// Windows without tiles are zero-filled by all CTAs at the start and skipped by the window walk.
//
// Warp roles: 0-3 epilogue (TMEM -> registers -> global), 4 MMA issuer, 5 TMA producer for tile
// values and column ids, 6.. gather producers (one per ring slot).  The role index is read from
// lane 0 and every TMA copy / MMA is issued by one elected lane, which keeps descriptors and
// barrier addresses in uniform registers (the roles are chains of dependent instructions on
// single warps: their instruction count is what the kernel's run time follows).  Every mbarrier
// wait is bounded: on time-out the kernel raises the status word at the start of scratch and all
// roles drain and return.
#include <cuda.h>      // CUtensorMap and the cuTensorMapEncodeTiled prototype (resolved at run time)
#include <stdlib.h>

#include "grws_common.cuh"

namespace grws {

namespace tc5 {

#ifndef GRWS_TC5_STAGE_TILES
#define GRWS_TC5_STAGE_TILES 8
#endif
#ifndef GRWS_TC5_STAGES
#define GRWS_TC5_STAGES 5
#endif
constexpr int STAGE_TILES = GRWS_TC5_STAGE_TILES;    // tiles per pipeline stage (two per MMA K-step)
constexpr int STAGE_SLOTS = STAGE_TILES * TILE_COLS; // gathered rows per stage
constexpr int MMAS_PER_STAGE = STAGE_TILES / 2;
constexpr int SLAB = 128;                            // features per MMA (its M dimension)
// A operand of one K-step (16 slots x 128 features), MN-major with the 128-byte swizzle: four
// 1024-byte atoms [slot half][feature half], an atom holds 8 slots x 64 features, slot k at
// k * 128 bytes, its 16-byte piece c stored at piece c ^ k.  A gathered row therefore lands as
// two contiguous (permuted) 128-byte lines, which the TMA gather writes as whole lines.
constexpr int A_ATOM_BYTES = 1024;
constexpr int A_LBO = A_ATOM_BYTES;                  // between the two 64-feature halves
constexpr int A_SBO = 2 * A_ATOM_BYTES;              // between the two 8-slot halves
constexpr int A_MMA_BYTES = 4 * A_ATOM_BYTES;        // one K-step of one slab
constexpr int TILE_BYTES = TILE_ELEMS * 2;           // 256
constexpr int META_TILE_BYTES = STAGE_TILES * TILE_BYTES;
constexpr int META_COL_BYTES = STAGE_TILES * TILE_COLS * 4;
constexpr int META_CMD_BYTES = 16;                   // per-stage command word, copied from the stage's descriptor
constexpr int META_BYTES = META_TILE_BYTES + META_COL_BYTES + META_CMD_BYTES;
// command word: bits 0-4 tile count, bit 8 first stage of a window segment, bit 9 last stage,
// bit 10 end of this CTA's work
constexpr uint32_t CMD_COUNT = 31u, CMD_FIRST = 1u << 8, CMD_LAST = 1u << 9, CMD_END = 1u << 10;
static_assert(STAGE_TILES <= (int)CMD_COUNT && STAGE_TILES % 4 == 0, "count field of the command word; K-steps are issued in pairs");
#ifndef GRWS_TC5_NACC
#define GRWS_TC5_NACC 4
#endif
constexpr int NACC = GRWS_TC5_NACC;                  // accumulator buffers in tensor memory
constexpr int NUM_EPILOGUE = 128;
constexpr int EPILOGUE_WARP0 = 0;                    // four warps; warp % 4 is its TMEM lane quarter
constexpr int MMA_WARP = EPILOGUE_WARP0 + 4;
constexpr int WALK_WARP = MMA_WARP + 1;
constexpr int PRODUCER_WARP0 = WALK_WARP + 1;
constexpr int NUM_PRODUCER_WARPS = GRWS_TC5_STAGES;  // one per ring slot
constexpr int NUM_THREADS = (PRODUCER_WARP0 + NUM_PRODUCER_WARPS) * 32;
static_assert(EPILOGUE_WARP0 % 4 == 0, "epilogue warps must start at a multiple of four");
constexpr int64_t SPLIT256_OPERAND_BYTES = 8ll << 20;   // dense operand size above which width 256 runs as two 128-column passes
// A cut of the tile array that falls inside a window of at most min(chunk / 2, LONG_WINDOW_TILES)
// tiles moves back to the window's first tile: finishing a window that is split between two CTAs
// costs about as much as 100 tiles of work (partial tiles through global memory, a counter, the
// sum), so only windows well above that are worth splitting; the cap keeps the imbalance this
// causes at a few per cent of a large CTA range.
#ifndef GRWS_TC5_LW_TILES
#define GRWS_TC5_LW_TILES 512
#endif
#ifndef GRWS_TC5_AUTO_MIN_N
#define GRWS_TC5_AUTO_MIN_N 16
#endif
#ifndef GRWS_TC5_AUTO_MIN_TILES
#define GRWS_TC5_AUTO_MIN_TILES 512
#endif
constexpr int PLAN_MAGIC = 0x504c4e31;                                    // first word of a valid plan
constexpr int PLAN_LONG_WINDOW_STAGES = 16;                               // planned ranges: a window of more stages may be split
constexpr int64_t LONG_WINDOW_TILES = GRWS_TC5_LW_TILES;                 // a cut inside a window of at most chunk >> 4 tiles moves to the window start
constexpr long long WAIT_LIMIT_CYCLES = 3000000000ll;   // default: a wait gives up after about 1.5-2.5 s of SM clocks

// status codes: which wait ran out (the first four) / an injected failure of the self-test build
enum : int { ST_OK = 0, ST_TIMEOUT_FULL = 1, ST_TIMEOUT_EMPTY = 2, ST_TIMEOUT_ACC = 3, ST_TIMEOUT_META = 4 };

// experiment knobs of the profiling build (GRWS_TC5_SKIP); the product kernel compiles them out
enum : int { SKIP_MMA = 1, SKIP_GATHER = 2, SKIP_STORE = 4, SKIP_TILES = 8, SKIP_ONE_ARRIVE = 16 };

struct Params {
    const int64_t *window_offset;
    const int32_t *cols;
    const void *vals;
    const void *B;
    void *C;
    float *partial;
    int *status;      // this call's status word (start of scratch)
    int *sticky;      // per-device word that keeps the worst status since it was last read (may be null)
    int *split_count; // [grid]: pieces of the split window that starts in CTA k which are finished (zeroed before the launch)
    const int4 *plan; // tile ranges of the CTAs computed once per graph (spmm_plan_kernel), or null: every CTA searches its range
    int64_t W, N, ldb, ldc;   // N: width of the pass as the kernel lays it out (128 or 256)
    int n_valid;      // features of the pass that exist in B and C (a multiple of 8, <= N); the rest is computed on zeros and dropped
    int c_dtype;
    int is_bf16;
    int skip;         // profiling build only
    long long wait_limit;   // SM clocks after which a barrier wait gives up
    long long *dbg;   // profiling build: [grid][16] cycle counters (wait time per role) + a stage timeline
};

// ---------------------------------------------------------------------------------------------
// PTX wrappers
// ---------------------------------------------------------------------------------------------
__device__ __forceinline__ uint32_t smem_u32(const void *p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ uint32_t mbar_try_wait(uint32_t bar, uint32_t parity) {
    uint32_t ok;
#ifdef GRWS_TC5_WAIT_HINT_NS
    // the hint lets the hardware keep the thread suspended for up to that long before it reports failure
    asm volatile("{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n\tselp.u32 %0, 1, 0, p;\n\t}"
                 : "=r"(ok) : "r"(bar), "r"(parity), "r"((uint32_t)GRWS_TC5_WAIT_HINT_NS) : "memory");
#else
    asm volatile("{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}"
                 : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
#endif
    return ok;
}
// bounded wait: gives up after `limit` SM clocks or when another role already aborted.
// (The SM clock is used because reading %globaltimer costs about a microsecond per read.)
template <bool SLEEPY = false>
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile int *abort_flag, long long limit) {
    if (mbar_try_wait(bar, parity)) return true;
    long long t0 = 0;
    for (uint32_t i = 0;; ++i) {
        if (mbar_try_wait(bar, parity)) return true;
#ifdef GRWS_TC5_SLEEP_NS
        if (SLEEPY) __nanosleep(GRWS_TC5_SLEEP_NS);
#endif
        if ((i & 63u) == 63u) {
            if (*abort_flag) return false;
            const long long now = clock64();
            if (t0 == 0) t0 = now;
            if (now - t0 > limit) return false;
        }
    }
}
// the same wait without the abort test: used while draining after an abort
__device__ __forceinline__ bool mbar_wait_drain(uint32_t bar, uint32_t parity, long long limit) {
    const long long t0 = clock64();
    for (uint32_t i = 0;; ++i) {
        if (mbar_try_wait(bar, parity)) return true;
        if ((i & 63u) == 63u && clock64() - t0 > limit) return false;
    }
}
// wait that adds its duration to `acc` in the profiling build of the kernel
template <bool PROF>
__device__ __forceinline__ bool mbar_wait_t(uint32_t bar, uint32_t parity, volatile int *abort_flag, long long limit, long long &acc, int role = 0) {
    if constexpr (PROF) {
        // (a try_wait may itself suspend the thread until the phase completes, so even a wait whose
        // first try succeeds has to be timed)
        const long long t0 = clock64();
        const bool ok = mbar_wait(bar, parity, abort_flag, limit);
        acc += clock64() - t0;
        return ok;
    } else {
        (void)acc;
        // (experiment builds let the roles with slack -- a producer waiting for its slot, the
        // epilogue, the walker -- sleep between polls)
        if (role == 2 || role == 4 || role == 5) return mbar_wait<true>(bar, parity, abort_flag, limit);
        return mbar_wait<false>(bar, parity, abort_flag, limit);
    }
}
// timeline of the first stages of CTA 0 (profiling build): event e of stage `it`
template <bool PROF> __device__ __forceinline__ void prof_mark(long long *dbg, uint32_t it, int e) {
#ifdef GRWS_TC5_TIMELINE
    if constexpr (PROF) { if (dbg && blockIdx.x == 0 && it < 64) dbg[12288 + it * 8 + e] = clock64(); }
#else
    (void)dbg; (void)it; (void)e;
#endif
}
template <bool PROF> __device__ __forceinline__ long long prof_clock() {
    if constexpr (PROF) return clock64(); else return 0;
}
// wall-clock timestamp (ns) of the profiling build: comparable across SMs
template <bool PROF> __device__ __forceinline__ void prof_stamp(long long *dbg, int slot) {
    if constexpr (PROF) {
        if (dbg) {
            unsigned long long t;
            asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
            dbg[8192 + (size_t)blockIdx.x * 8 + slot] = (long long)t;
        }
    }
}
// clock reads inside the per-stage loops: only in the timeline build (they slow the loops down)
template <bool PROF> __device__ __forceinline__ long long prof_fine() {
#ifdef GRWS_TC5_TIMELINE
    if constexpr (PROF) return clock64();
#endif
    return 0;
}
__device__ __forceinline__ void bulk_g2s(uint32_t dst, const void *src, uint32_t bytes, uint32_t bar, uint64_t pol) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes.L2::cache_hint [%0], [%1], %2, [%3], %4;"
                 ::"r"(dst), "l"(src), "r"(bytes), "r"(bar), "l"(pol) : "memory");
}
// bulk store of a contiguous piece of shared memory to global memory (both 16-byte aligned)
__device__ __forceinline__ void bulk_s2g(void *dst, uint32_t src, uint32_t bytes, uint64_t pol) {
    asm volatile("cp.async.bulk.global.shared::cta.bulk_group.L2::cache_hint [%0], [%1], %2, %3;"
                 ::"l"(dst), "r"(src), "r"(bytes), "l"(pol) : "memory");
}
__device__ __forceinline__ void bulk_commit() { asm volatile("cp.async.bulk.commit_group;" ::: "memory"); }
__device__ __forceinline__ void bulk_wait_read0() { asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory"); }
__device__ __forceinline__ void bulk_wait0() { asm volatile("cp.async.bulk.wait_group 0;" ::: "memory"); }
// TMA gather of four rows of the dense operand (tile::gather4): 64 features of rows r0..r3 land as
// four consecutive 128-byte lines, already permuted for the 128-byte-swizzle operand layout.  A
// negative or too large row id is out of bounds and reads zeros.
__device__ __forceinline__ void tma_gather4(uint32_t dst, const CUtensorMap *map, uint32_t bar, int x, int r0, int r1,
                                            int r2, int r3, uint64_t pol) {
    asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.tile::gather4.mbarrier::complete_tx::bytes.L2::cache_hint"
                 " [%0], [%1, {%3, %4, %5, %6, %7}], [%2], %8;"
                 ::"r"(dst), "l"(map), "r"(bar), "r"(x), "r"(r0), "r"(r1), "r"(r2), "r"(r3), "l"(pol) : "memory");
}
// true in exactly one lane of a converged warp
__device__ __forceinline__ bool elect_one() {
    uint32_t e;
    asm volatile("{\n\t.reg .pred p;\n\telect.sync _|p, 0xffffffff;\n\tselp.u32 %0, 1, 0, p;\n\t}" : "=r"(e));
    return e != 0;
}
__device__ __forceinline__ uint64_t policy_keep() {
    uint64_t p;
    asm volatile("createpolicy.fractional.L2::evict_last.b64 %0, 1.0;" : "=l"(p));
    return p;
}
__device__ __forceinline__ uint64_t policy_stream() {
    uint64_t p;
    asm volatile("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;" : "=l"(p));
    return p;
}
__device__ __forceinline__ void tmem_alloc(uint32_t smem_dst, uint32_t ncols) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_dst), "r"(ncols) : "memory");
}
__device__ __forceinline__ void tmem_relinquish() {
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t ncols) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void fence_async_smem() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }
// barrier 1 of the CTA for the 128 epilogue threads
__device__ __forceinline__ void epilogue_sync() { asm volatile("bar.sync 1, 128;" ::: "memory"); }
// the same barrier with an OR over every thread's flag: all 128 threads get the same answer
__device__ __forceinline__ bool epilogue_sync_or(bool flag) {
    uint32_t r;
    asm volatile("{\n\t.reg .pred p, q;\n\tsetp.ne.u32 q, %1, 0;\n\tbar.red.or.pred p, 1, 128, q;\n\tselp.u32 %0, 1, 0, p;\n\t}"
                 : "=r"(r) : "r"(flag ? 1u : 0u) : "memory");
    return r != 0;
}

__device__ __forceinline__ void umma_f16(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t accumulate) {
    asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
                 "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
                 ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate) : "memory");
}
// the same with the accumulate flag fixed to "add to the accumulator" (no predicate to compute)
__device__ __forceinline__ void umma_f16_acc(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc) {
    asm volatile("{\n\t.reg .pred p;\n\tsetp.eq.u32 p, 0, 0;\n\t"
                 "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
                 ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc) : "memory");
}
__device__ __forceinline__ void umma_commit(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void tmem_ld16(uint32_t taddr, uint32_t (&r)[16]) {
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
                   "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
                 : "r"(taddr) : "memory");
}
__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

// shared-memory matrix descriptor (version 1); layout 0 = no swizzle, 2 = 128-byte swizzle
__device__ __forceinline__ uint64_t smem_desc(uint32_t addr, uint32_t lbo_bytes, uint32_t sbo_bytes, uint32_t layout) {
    return (uint64_t)((addr & 0x3FFFFu) >> 4) | ((uint64_t)(lbo_bytes >> 4) << 16) |
           ((uint64_t)(sbo_bytes >> 4) << 32) | (1ull << 46) | ((uint64_t)layout << 61);
}

// ---------------------------------------------------------------------------------------------
// window offsets streamed through registers: every lane of a warp holds one of 32 consecutive
// entries; all lanes must call get() together with a non-decreasing index
// ---------------------------------------------------------------------------------------------
struct OffsetStream {
    const int64_t *off;
    int64_t W, base;
    int64_t cur, nxt;
    __device__ __forceinline__ void init(const int64_t *o, int64_t w_total, int64_t start, int lane) {
        off = o; W = w_total; base = start;
        cur = __ldg(off + min(base + lane, W));
        nxt = __ldg(off + min(base + 32 + lane, W));
    }
    __device__ __forceinline__ int64_t get(int64_t idx, int lane) {
        while (idx >= base + 32) {
            base += 32;
            cur = nxt;
            nxt = __ldg(off + min(base + 32 + lane, W));
        }
        return __shfl_sync(0xffffffffu, cur, (int)(idx - base));
    }
};

// The sequence of window segments and stages of one CTA; every role walks it identically.
struct Walker {
    OffsetStream os;
    int64_t W, s, e, w;
    int64_t a, b, seg_s, seg_e;
    __device__ __forceinline__ void init(const int64_t *off, int64_t w_total, int64_t s_, int64_t e_, int64_t w0, int lane) {
        W = w_total; s = s_; e = e_; w = w0;
        os.init(off, w_total, w0, lane);
    }
    // advances to the next window owned or touched by this CTA
    __device__ __forceinline__ bool next_segment(int lane) {
        if (w >= W) return false;
        a = os.get(w, lane);
        b = os.get(w + 1, lane);
        // A run of windows without tiles is jumped 32 offsets at a time (nobody has to visit them:
        // all CTAs zero-fill them at start): the next window with tiles is the one before the
        // first offset above `a`.
        while (b == a) {
            const int64_t idx = os.base + lane;
            const unsigned m = __ballot_sync(0xffffffffu, idx > w && idx <= W && os.cur > a);
            if (m) {
                w = os.base + (__ffs(m) - 1) - 1;
                b = os.get(w + 1, lane);
            } else if (os.base + 32 <= W) {
                w = os.base + 31;                   // offsets up to base + 31 all equal `a`
                (void)os.get(os.base + 32, lane);   // slide the register window
            } else {
                w = W;
                return false;
            }
        }
        // Windows without tiles need no owner (all CTAs zero-fill them at start), so the walk ends at
        // the first window that starts at or behind the range end: a run of empty windows there
        // (padded blocks) would otherwise cost hundreds of cycles each on this dependent chain.
        if (a >= e) return false;
        seg_s = a > s ? a : s;
        seg_e = b < e ? b : e;
        ++w;
        return true;
    }
    __device__ __forceinline__ int64_t window() const { return w - 1; }
    __device__ __forceinline__ bool head() const { return seg_s > a; }
    __device__ __forceinline__ bool tail() const { return !(seg_s > a) && seg_e < b; }
};

// What the walker warp tells the producers about one stage: its first tile and its command word.
struct __align__(16) StageDesc {
    int64_t t0;
    uint32_t cmd, pad;
};
constexpr int DESC_BATCHES = 8;                      // descriptor ring: batches of one descriptor per producer

struct SharedStorage {
    uint64_t full_g[16], empty_g[16], full_m[48], desc_full[DESC_BATCHES], desc_empty[DESC_BATCHES], acc_full[NACC], acc_empty[NACC], drain;
    StageDesc desc[DESC_BATCHES * GRWS_TC5_STAGES];
    uint32_t tmem_base;
    int abort_flag;
    int last_piece;       // epilogue: this CTA finished the last piece of a split window
};

template <int NH> struct Cfg {
    // two CTAs per SM for one slab (their MMA-issuing threads overlap each other's latency),
    // one CTA per SM for two slabs (a stage is twice as large)
#ifndef GRWS_TC5_CTAS_PER_SM
#define GRWS_TC5_CTAS_PER_SM 2
#endif
    static constexpr int kCtasPerSm = (NH == 1) ? GRWS_TC5_CTAS_PER_SM : 1;
    static constexpr int kStages = GRWS_TC5_STAGES;
    // tile / column-id slots per producer: the tiles of a producer's stage n + kMetaDepth - 1 are
    // requested while it gathers for stage n, i.e. (kMetaDepth - 1) * kStages stages ahead of the
    // MMAs, which has to cover the HBM latency of the tile stream
#ifndef GRWS_TC5_META_DEPTH
#define GRWS_TC5_META_DEPTH 2
#endif
    static constexpr int kMetaDepth = (NH == 1) ? GRWS_TC5_META_DEPTH : 3;
    static constexpr int kMeta = kStages * kMetaDepth;
    static constexpr int kStageBytes = MMAS_PER_STAGE * NH * A_MMA_BYTES;
    static constexpr int kAccCols = 16 * NH;
    static constexpr int kTmemCols = (NACC * kAccCols) < 32 ? 32 : NACC * kAccCols;   // 64 or 128: powers of two
    // one window of 16-bit output rows, staged for the bulk store: [16 rows][128 * NH features]
    static constexpr int kStagingBytes = TILE_ROWS * SLAB * NH * 2;
    static_assert(kStages <= 16 && kMeta <= 48, "barrier arrays in SharedStorage");
    static constexpr size_t kSmem = 1024 + sizeof(SharedStorage) + 16 + (size_t)kStages * kStageBytes + (size_t)kMeta * META_BYTES + kStagingBytes;
};

// The launch is a programmatic dependent of the small kernel that zeroes the status word and the
// split-window counters: this kernel may start before that one has finished, and whoever is about
// to touch those words waits for it here (a no-op when the launch was an ordinary one).
__device__ __forceinline__ void wait_for_zeroed_scratch() { asm volatile("griddepcontrol.wait;" ::: "memory"); }

__device__ __forceinline__ void raise(Params const &prm, SharedStorage *ss, int code) {
    ss->abort_flag = 1;
    wait_for_zeroed_scratch();
    atomicMax(prm.status, code);
    if (prm.sticky) atomicMax(prm.sticky, code);
}

// The two rare paths of the epilogue live in functions of their own (not inlined), so that their
// registers do not count against the per-window path of the kernel.

// Rows of the windows without tiles in this CTA's share of the window list (a contiguous run,
// 32 offsets per coalesced load); warp quarter q writes features 32q .. 32q+31 of every slab.
template <int NH>
__device__ __noinline__ void zero_fill_empty_windows(const int64_t *__restrict__ window_offset, void *C, int64_t ldc, int c_dtype,
                                                    int64_t W, int n_valid, int q, int lane) {
    const int64_t per = (W + gridDim.x - 1) / gridDim.x;
    const int64_t w_lo = (int64_t)blockIdx.x * per, w_hi = min(W, w_lo + per);
    for (int64_t wb = w_lo; wb < w_hi; wb += 32) {
        const int64_t wl = wb + lane;
        const bool empty = wl < w_hi && __ldg(window_offset + wl) == __ldg(window_offset + wl + 1);
        unsigned m = __ballot_sync(0xffffffffu, empty);
        while (m) {
            const int64_t w0 = wb + (__ffs(m) - 1);
            m &= m - 1;
#pragma unroll
            for (int h = 0; h < NH; ++h) {
                if (h * SLAB + 32 * q + lane >= n_valid) continue;
                const int64_t o0 = (w0 * TILE_ROWS) * ldc + h * SLAB + 32 * q + lane;
                for (int r = 0; r < 16; ++r) {
                    const int64_t o = o0 + r * ldc;
                    if (c_dtype == GRWS_F32) static_cast<float *>(C)[o] = 0.0f;
                    else static_cast<uint16_t *>(C)[o] = 0;
                }
            }
        }
    }
}

// Sum of the pieces of split window w (held by CTAs k0 .. k_last, the first one in its tail slot,
// the others in their head slots), in CTA order, written to the window's rows.
template <int NH>
__device__ __noinline__ void sum_pieces(const float *partial, int64_t N, int n_valid, void *C, int64_t ldc, int c_dtype, int64_t w, int64_t k0,
                                       int64_t k_last, int q, int lane) {
    __threadfence();
    const int64_t elems = TILE_ROWS * N;
#pragma unroll
    for (int h = 0; h < NH; ++h) {
        const int64_t f = h * SLAB + 32 * q + lane;
        if (f >= n_valid) continue;
        float acc[16];
        const float *p0 = partial + (2 * k0 + 1) * elems + f;
#pragma unroll
        for (int r = 0; r < 16; ++r) acc[r] = __ldcg(p0 + (int64_t)r * N);
        for (int64_t kq = k0 + 1; kq <= k_last; ++kq) {
            const float *pq = partial + (2 * kq) * elems + f;
#pragma unroll
            for (int r = 0; r < 16; ++r) acc[r] += __ldcg(pq + (int64_t)r * N);
        }
        const int64_t base = (w * TILE_ROWS) * ldc + f;
#pragma unroll
        for (int r = 0; r < 16; ++r) {
            const int64_t o = base + r * ldc;
            if (c_dtype == GRWS_F32) static_cast<float *>(C)[o] = acc[r];
            else if (c_dtype == GRWS_F16) static_cast<__half *>(C)[o] = __float2half_rn(acc[r]);
            else static_cast<__nv_bfloat16 *>(C)[o] = __float2bfloat16_rn(acc[r]);
        }
    }
}

// NARROW: the operand has fewer features than the pass is wide (prm.n_valid < 128, one slab); the
// full-width kernel carries none of the tests that needs.
template <int NH, bool PROF, bool NARROW = false>
__global__ void __launch_bounds__(NUM_THREADS, Cfg<NH>::kCtasPerSm)
spmm_tc5_kernel(const Params prm, const __grid_constant__ CUtensorMap b_map) {
    using C = Cfg<NH>;
    static_assert(!NARROW || NH == 1, "narrow operands run as one slab");
    const int n_valid = NARROW ? prm.n_valid : SLAB * NH;
    extern __shared__ uint8_t smem_raw[];
    // the swizzled operand atoms must start on 1024-byte boundaries
    uint8_t *ring_g = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint8_t *ring_m = ring_g + (size_t)C::kStages * C::kStageBytes;
    uint8_t *staging = ring_m + (size_t)C::kMeta * META_BYTES;
    SharedStorage *ss = reinterpret_cast<SharedStorage *>(staging + C::kStagingBytes);

    // the warp index is taken from lane 0 so that the compiler knows it is the same in all lanes:
    // everything derived from it (role, barrier and ring addresses) can live in uniform registers
    const int warp = __shfl_sync(0xffffffffu, (int)(threadIdx.x >> 5), 0), lane = threadIdx.x & 31;
    const int64_t W = prm.W;
#ifndef GRWS_TC5_BUILD_SKIP
#define GRWS_TC5_BUILD_SKIP 0                      // experiment builds leave parts of the work out (SKIP_* bits)
#endif
    const int skip = PROF ? prm.skip : GRWS_TC5_BUILD_SKIP;   // folds to zero in the product kernel
    const long long limit = prm.wait_limit;
    if (threadIdx.x == 0) prof_stamp<PROF>(prm.dbg, 0);           // kernel entry

    if (threadIdx.x == 0) {
        for (int i = 0; i < C::kStages; ++i) { mbar_init(smem_u32(&ss->full_g[i]), 1); mbar_init(smem_u32(&ss->empty_g[i]), 1); }
        for (int i = 0; i < C::kMeta; ++i) mbar_init(smem_u32(&ss->full_m[i]), 1);
        for (int i = 0; i < DESC_BATCHES; ++i) { mbar_init(smem_u32(&ss->desc_full[i]), 1); mbar_init(smem_u32(&ss->desc_empty[i]), C::kStages); }
        for (int i = 0; i < NACC; ++i) { mbar_init(smem_u32(&ss->acc_full[i]), 1); mbar_init(smem_u32(&ss->acc_empty[i]), NUM_EPILOGUE / 32); }
        mbar_init(smem_u32(&ss->drain), 1);
        ss->abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == MMA_WARP) {
        tmem_alloc(smem_u32(&ss->tmem_base), C::kTmemCols);
        tmem_relinquish();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = ss->tmem_base;
    volatile int *abort_flag = &ss->abort_flag;
    if (threadIdx.x == 0) prof_stamp<PROF>(prm.dbg, 1);           // barriers and tensor memory set up

    if (warp == WALK_WARP || (warp >= EPILOGUE_WARP0 && warp < MMA_WARP)) {
        // ---- the two roles that walk the window structure: this CTA's tile range [s, e)
        const int64_t T = __ldg(prm.window_offset + W);
        const int64_t G = gridDim.x;
        int64_t chunk = (T + G - 1) / G;
        chunk = (chunk + 1) & ~int64_t(1);
        if (chunk < 2) chunk = 2;
        // a cut inside a short window moves back to that window's start: only long windows are
        // ever split between CTAs
        const int64_t long_window = min(chunk >> 1, LONG_WINDOW_TILES);
        int64_t w_first, s, e;
        // holders of the pieces of the windows this CTA's range starts / ends in (planned ranges only)
        int plan_head_k0 = 0, plan_head_klast = 0, plan_tail_klast = 0;
        bool planned = false;
        if (prm.plan != nullptr) {
            // ranges balanced by stage count, computed once per graph: header and the two cuts
            // arrive in one round trip (the search below needs three dependent ones)
            const int4 h0 = __ldg(prm.plan), h1 = __ldg(prm.plan + 1);
            const int4 c0 = __ldg(prm.plan + 2 + 2 * blockIdx.x), c1 = __ldg(prm.plan + 3 + 2 * blockIdx.x);
            const int4 n0 = __ldg(prm.plan + 4 + 2 * blockIdx.x);
            const int64_t plan_w = ((int64_t)(uint32_t)h0.w << 32) | (uint32_t)h0.z;
            const int64_t plan_t = ((int64_t)(uint32_t)h1.y << 32) | (uint32_t)h1.x;
            // a plan made for another grid or another graph size is ignored
            planned = h0.x == PLAN_MAGIC && h0.y == (int)G && plan_w == W && plan_t == T;
            if (planned) {
                s = ((int64_t)(uint32_t)c0.y << 32) | (uint32_t)c0.x;
                w_first = ((int64_t)(uint32_t)c0.w << 32) | (uint32_t)c0.z;
                e = ((int64_t)(uint32_t)n0.y << 32) | (uint32_t)n0.x;
                plan_head_k0 = c1.x; plan_head_klast = c1.y; plan_tail_klast = c1.z;
            }
        }
        if (!planned) warp_cut_pair(prm.window_offset, W, T, blockIdx.x, G, chunk, long_window, lane, &s, &e, &w_first);
        Walker wk;
        wk.init(prm.window_offset, W, s, e, blockIdx.x == 0 ? 0 : w_first, lane);
        if (warp == WALK_WARP && lane == 0) prof_stamp<PROF>(prm.dbg, 2);     // tile range found

        if (warp == WALK_WARP) {
            // -------------------------------------------------------------- walker
            // Walks this CTA's windows and writes one descriptor per stage (first tile, tile count,
            // first / last stage of its window segment) into a small ring; the producers, which
            // take the stages round-robin, fetch tiles, column ids and rows from the descriptors.
            // A batch is one descriptor per producer and is published with one barrier arrive.
            uint32_t it = 0;
            bool ok = true;
            long long w_desc = 0, t_walk = 0;
            const long long t_start = prof_clock<PROF>();
            // all lanes call; lane 0 writes
            auto push = [&](int64_t t0, uint32_t cmd) {
                const uint32_t pos = it % C::kStages, batch = it / C::kStages, bslot = batch % DESC_BATCHES;
                if (pos == 0) {
                    if (lane == 0) ok = mbar_wait_t<PROF>(smem_u32(&ss->desc_empty[bslot]), ((batch / DESC_BATCHES) & 1u) ^ 1u, abort_flag, limit, w_desc, 5);
                    ok = __shfl_sync(0xffffffffu, ok ? 1 : 0, 0) != 0;
                    if (!ok) { if (lane == 0) raise(prm, ss, ST_TIMEOUT_META); return; }
                }
                if (lane == 0) {
                    StageDesc *d = &ss->desc[bslot * C::kStages + pos];
                    d->t0 = t0;
                    d->cmd = cmd;
                    if (pos == C::kStages - 1) {
                        // self-test of the bounded waits (profiling build): one batch is never
                        // published; nothing was copied for it, so every role runs into its limit
                        if (!(PROF && (skip & SKIP_ONE_ARRIVE) && batch == 1 && blockIdx.x == 0))
                            mbar_arrive(smem_u32(&ss->desc_full[bslot]));    // release: publishes the batch
                    }
                }
                ++it;
            };
            for (;;) {
                const long long tw0 = prof_fine<PROF>();
                const bool more = ok && wk.next_segment(lane);
                t_walk += prof_fine<PROF>() - tw0;
                if (!more) break;
                for (int64_t t0 = wk.seg_s; ok && t0 < wk.seg_e; t0 += STAGE_TILES) {
                    const int ntiles = (int)min((int64_t)STAGE_TILES, wk.seg_e - t0);
                    push(t0, (uint32_t)ntiles | (t0 == wk.seg_s ? CMD_FIRST : 0u) | (t0 + STAGE_TILES >= wk.seg_e ? CMD_LAST : 0u));
                }
            }
            // one end marker per producer (the MMA warp stops at the first), then the rest of the batch
            for (int j = 0; ok && (j < C::kStages || it % C::kStages != 0); ++j) push(0, CMD_END);
            if (PROF && prm.dbg && lane == 0) {
                prm.dbg[blockIdx.x * 16 + 0] = w_desc; prm.dbg[blockIdx.x * 16 + 1] = prof_clock<PROF>() - t_start;
                prm.dbg[blockIdx.x * 16 + 15] = t_walk;
            }
        } else {
            // -------------------------------------------------------------- epilogue warps
            const uint64_t pol = policy_stream();
            const int q = warp & 3;                        // TMEM lane quarter this warp may read
            uint32_t ai = 0;
            long long w_af = 0;
            const long long t_epi0 = prof_clock<PROF>();
            // 16-bit outputs go through shared memory: every thread holds one feature of the 16 rows
            // (a tensor-memory lane), the window's rows are assembled in `staging` and leave as
            // 16-byte vector stores, 256 contiguous bytes per 16 threads
            const bool staged = prm.c_dtype != GRWS_F32 && !(skip & SKIP_STORE);
            // Windows without tiles produce zero rows.  They are dealt to all CTAs here, while the
            // pipeline fills, instead of being written by whichever CTA's tile range they border:
            // a run of empty windows (padded blocks, isolated nodes) would serialise on that one CTA.
            if (!(skip & SKIP_STORE)) zero_fill_empty_windows<NH>(prm.window_offset, prm.C, prm.ldc, prm.c_dtype, W, n_valid, q, lane);
            for (;;) {
                const bool more = wk.next_segment(lane);
                if (!more) break;                          // the same in all four warps: they walk the same ranges
                const int64_t w = wk.window();
                if (wk.seg_e <= wk.seg_s) continue;        // zero rows were written above
                uint32_t v[NH][16];
                const uint32_t buf = ai % NACC, aph = (ai / NACC) & 1u;
                ++ai;
                // One thread polls for all four warps (threads spinning on a barrier slow every other
                // barrier operation of the SM down).  All four warps then meet and leave together
                // when the wait ran out or another role gave up: none may be left alone at a later
                // barrier.  The barrier also orders the previous window's reads of `staging` before
                // this window's writes.
                bool ok = true;
                if (threadIdx.x == EPILOGUE_WARP0 * 32) {
                    ok = mbar_wait_t<PROF>(smem_u32(&ss->acc_full[buf]), aph, abort_flag, limit, w_af, 4);
                    if (!ok) raise(prm, ss, ST_TIMEOUT_ACC);
                }
                if (epilogue_sync_or(!ok || *abort_flag != 0)) break;
                tc_fence_after();
#pragma unroll
                for (int h = 0; h < NH; ++h)
                    tmem_ld16(tmem_base + ((uint32_t)(32 * q) << 16) + buf * C::kAccCols + h * 16, v[h]);
                tmem_ld_wait();
                tc_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive(smem_u32(&ss->acc_empty[buf]));
                const bool partial = wk.head() || wk.tail();
                if (skip & SKIP_STORE) {
                } else if (!partial && staged) {
#pragma unroll
                    for (int h = 0; h < NH; ++h) {
                        uint16_t *st = reinterpret_cast<uint16_t *>(staging) + h * SLAB + 32 * q + lane;
#pragma unroll
                        for (int r = 0; r < 16; ++r) {
                            const float x = __uint_as_float(v[h][r]);
                            st[r * (SLAB * NH)] = prm.c_dtype == GRWS_F16 ? __half_as_ushort(__float2half_rn(x))
                                                                         : __bfloat16_as_ushort(__float2bfloat16_rn(x));
                        }
                    }
                    epilogue_sync();
                    // 16 threads per 256-byte row: whole rows leave as 16-byte vector stores.  (A bulk
                    // store from shared memory would queue behind the gathers in the TMA unit and
                    // hold the staging buffer, and with it the accumulators, for thousands of cycles.)
                    {
                        constexpr int CPR = SLAB * NH * 2 / 16;            // 16-byte pieces per row
                        char *dst = static_cast<char *>(prm.C) + (w * TILE_ROWS) * prm.ldc * 2;
                        if (!NARROW) {
#pragma unroll
                            for (int c = threadIdx.x; c < TILE_ROWS * CPR; c += NUM_EPILOGUE) {
                                const int r = c / CPR, k = c % CPR;
                                const uint4 val = *reinterpret_cast<const uint4 *>(staging + r * (SLAB * NH * 2) + k * 16);
                                asm volatile("st.global.L2::cache_hint.v4.b32 [%0], {%1, %2, %3, %4}, %5;"
                                             ::"l"(dst + (int64_t)r * prm.ldc * 2 + k * 16), "r"(val.x), "r"(val.y), "r"(val.z), "r"(val.w), "l"(pol) : "memory");
                            }
                        } else {
                            const int cpr = n_valid / 8;               // a narrow operand: the row's first n_valid features
                            for (int c = threadIdx.x; c < TILE_ROWS * cpr; c += NUM_EPILOGUE) {
                                const int r = c / cpr, k = c % cpr;
                                const uint4 val = *reinterpret_cast<const uint4 *>(staging + r * (SLAB * NH * 2) + k * 16);
                                asm volatile("st.global.L2::cache_hint.v4.b32 [%0], {%1, %2, %3, %4}, %5;"
                                             ::"l"(dst + (int64_t)r * prm.ldc * 2 + k * 16), "r"(val.x), "r"(val.y), "r"(val.z), "r"(val.w), "l"(pol) : "memory");
                            }
                        }
                    }
                } else if (!partial) {
#pragma unroll
                    for (int h = 0; h < NH; ++h) {
                        if (h * SLAB + 32 * q + lane >= n_valid) continue;
                        const int64_t base = (w * TILE_ROWS) * prm.ldc + h * SLAB + 32 * q + lane;
#pragma unroll
                        for (int r = 0; r < 16; ++r)
                            asm volatile("st.global.L2::cache_hint.f32 [%0], %1, %2;"
                                         ::"l"(static_cast<float *>(prm.C) + base + r * prm.ldc), "f"(__uint_as_float(v[h][r])), "l"(pol) : "memory");
                    }
                } else {
#pragma unroll
                    for (int h = 0; h < NH; ++h) {
                        float *slot = prm.partial + (2 * (int64_t)blockIdx.x + (wk.tail() ? 1 : 0)) * (TILE_ROWS * prm.N) + h * SLAB + 32 * q + lane;
#pragma unroll
                        for (int r = 0; r < 16; ++r) slot[(int64_t)r * prm.N] = __uint_as_float(v[h][r]);
                    }
                    // A window cut between CTAs: every holder of a piece counts itself on the counter of
                    // the CTA that holds the window's first tile, and the one that arrives last sums the
                    // pieces in CTA order (the same order whoever is last) and writes the rows.  Cuts
                    // inside a split window are never moved, so its pieces are exactly the CTAs
                    // a / chunk .. (b - 1) / chunk (planned ranges: the plan names the first and the last).  A holder that finds all the others already counted
                    // is the last one for sure and goes straight to the sum (its own piece was written by
                    // the very threads that read it back: no fence, no atomic).
                    const int64_t k0 = planned ? (wk.head() ? plan_head_k0 : (int)blockIdx.x) : wk.a / chunk;
                    const int64_t k_last = planned ? (wk.head() ? plan_head_klast : plan_tail_klast) : (wk.b - 1) / chunk;
                    if (threadIdx.x == EPILOGUE_WARP0 * 32) {
                        wait_for_zeroed_scratch();
                        int seen;
                        asm volatile("ld.acquire.gpu.global.s32 %0, [%1];" : "=r"(seen) : "l"(prm.split_count + k0) : "memory");
                        ss->last_piece = (seen == (int)(k_last - k0)) ? 2 : 0;
                    }
                    epilogue_sync();
                    if (*reinterpret_cast<volatile int *>(&ss->last_piece) != 2) {
                        __threadfence();
                        epilogue_sync();
                        if (threadIdx.x == EPILOGUE_WARP0 * 32) {
                            const int old = atomicAdd(prm.split_count + k0, 1);
                            ss->last_piece = (old == (int)(k_last - k0)) ? 1 : 0;
                        }
                        epilogue_sync();
                    }
                    if (*reinterpret_cast<volatile int *>(&ss->last_piece)) sum_pieces<NH>(prm.partial, prm.N, n_valid, prm.C, prm.ldc, prm.c_dtype, w, k0, k_last, q, lane);
                }
            }
            if (threadIdx.x == EPILOGUE_WARP0 * 32) prof_stamp<PROF>(prm.dbg, 5);      // last rows written
            if (PROF && prm.dbg && threadIdx.x == EPILOGUE_WARP0 * 32) { prm.dbg[blockIdx.x * 16 + 7] = w_af; prm.dbg[blockIdx.x * 16 + 14] = prof_clock<PROF>() - t_epi0; }
        }
    } else if (warp >= PRODUCER_WARP0) {
        // ------------------------------------------------------------------ gather producers
        // Producer warp w owns ring slot w and fills every kStages-th stage, so the barrier polls
        // and column-id reads of kStages stages overlap.  The rows are fetched by the TMA unit
        // (tile::gather4: four consecutive slots x 64 features per copy, 32 copies per stage and
        // slab).  The whole role runs on one elected lane: a copy issued per lane costs its warp
        // ~220 cycles (the copies of different lanes go one after the other and each marshals its
        // operands into uniform registers).  The column ids of two K-steps are loaded into
        // registers before their 16 copies are issued -- a shared-memory load between two copies
        // cannot be moved across them and costs the chain ~45 cycles per copy instead of ~20 -- and
        // the first batch is loaded while the ring slot is still being waited for.
        const uint32_t gs = (uint32_t)(warp - PRODUCER_WARP0);
        // An operand of at most 64 features (one slab, NH = 1): only the first 64-feature half of a row
        // is fetched; the MMAs still multiply the whole slot, the other half's results are never read.
        const bool narrow = NARROW && n_valid <= 64;
        if (elect_one()) {
            constexpr uint32_t D = (uint32_t)C::kMetaDepth;
            const uint64_t keep = policy_keep(), stream_pol = policy_stream();
            long long w_full_m = 0, w_empty_g = 0, w_desc = 0, t_meta = 0;
            const long long t_prod0 = prof_clock<PROF>();
            const uint32_t full_bar = smem_u32(&ss->full_g[gs]), empty_bar = smem_u32(&ss->empty_g[gs]);
            const uint32_t dst_slot = smem_u32(ring_g + (size_t)gs * C::kStageBytes);
            uint32_t gph = 0, armed_ph = 0;
            bool armed = false;               // phase armed_ph of full_bar waits for copies of this warp
            bool failed = false, seen_end = false;
            uint32_t n_meta = 0;              // this producer's next stage whose tiles have not been requested yet
            // Requests tiles and column ids of this producer's stage n_meta (descriptor batch n_meta)
            // into its meta slot n_meta % D, and copies the command word there for the MMA thread.
            auto request_tiles = [&]() {
                const uint32_t bslot = n_meta % DESC_BATCHES;
                if (!mbar_wait_t<PROF>(smem_u32(&ss->desc_full[bslot]), (n_meta / DESC_BATCHES) & 1u, abort_flag, limit, w_desc, 5)) {
                    raise(prm, ss, ST_TIMEOUT_META);
                    failed = true;
                    return;
                }
                const long long tm0 = prof_fine<PROF>();
                StageDesc d;
                {
                    const int4 raw = *reinterpret_cast<const int4 *>(&ss->desc[bslot * C::kStages + gs]);
                    d.t0 = (int64_t)(((uint64_t)(uint32_t)raw.y << 32) | (uint32_t)raw.x);
                    d.cmd = (uint32_t)raw.z;
                }
                mbar_arrive(smem_u32(&ss->desc_empty[bslot]));
                const uint32_t mslot = gs * D + n_meta % D;
                uint8_t *dst = ring_m + (size_t)mslot * META_BYTES;
                const uint32_t bar = smem_u32(&ss->full_m[mslot]);
                *reinterpret_cast<volatile uint32_t *>(dst + META_TILE_BYTES + META_COL_BYTES) = d.cmd;
                ++n_meta;
                if (d.cmd & CMD_END) {
                    seen_end = true;
                    mbar_arrive(bar);
                    return;
                }
                const uint32_t ntiles = d.cmd & CMD_COUNT;
                if (ntiles & 1u) {
                    // An odd tile count leaves the second tile of the last K-step without data: its
                    // values become zeros (the MMA multiplies them with zero rows, which must not
                    // meet NaNs) and its column ids -1 (their rows are fetched as zeros).
#pragma unroll
                    for (int i = 0; i < TILE_BYTES / 16; ++i)
                        *reinterpret_cast<uint4 *>(dst + (size_t)ntiles * TILE_BYTES + i * 16) = make_uint4(0u, 0u, 0u, 0u);
                    *reinterpret_cast<int4 *>(dst + META_TILE_BYTES + (size_t)ntiles * TILE_COLS * 4) = make_int4(-1, -1, -1, -1);
                    *reinterpret_cast<int4 *>(dst + META_TILE_BYTES + (size_t)ntiles * TILE_COLS * 4 + 16) = make_int4(-1, -1, -1, -1);
                    fence_async_smem();
                }
                if (skip & SKIP_TILES) {
                    mbar_arrive(bar);
                } else {
                    mbar_expect_tx(bar, ntiles * (TILE_BYTES + TILE_COLS * 4));
                    bulk_g2s(smem_u32(dst), static_cast<const uint8_t *>(prm.vals) + d.t0 * TILE_BYTES, ntiles * TILE_BYTES, bar, stream_pol);
                    bulk_g2s(smem_u32(dst + META_TILE_BYTES), prm.cols + d.t0 * TILE_COLS, ntiles * TILE_COLS * 4, bar, stream_pol);
                }
                t_meta += prof_fine<PROF>() - tm0;
                prof_mark<PROF>(prm.dbg, gs + (n_meta - 1) * C::kStages, 0);
            };
            for (uint32_t j = 0; j < D && !seen_end && !failed; ++j) request_tiles();
            for (uint32_t n = 0; !failed; ++n, gph ^= 1u) {
                const uint32_t it = gs + n * C::kStages;
                const uint32_t mslot = gs * D + n % D;
                // tile values, column ids and the command have landed
                if (!mbar_wait_t<PROF>(smem_u32(&ss->full_m[mslot]), (n / D) & 1u, abort_flag, limit, w_full_m, 3)) { raise(prm, ss, ST_TIMEOUT_META); break; }
                prof_mark<PROF>(prm.dbg, it, 1);
                const uint8_t *meta = ring_m + (size_t)mslot * META_BYTES;
                const uint32_t cmd = *reinterpret_cast<const volatile uint32_t *>(meta + META_TILE_BYTES + META_COL_BYTES);
                const bool end = (cmd & CMD_END) != 0;
                const int nmma = end ? 0 : (int)((cmd & CMD_COUNT) + 1u) >> 1;
                const int4 *ids = reinterpret_cast<const int4 *>(meta + META_TILE_BYTES);
                int4 r[8];                                // slots of K-steps 0 and 1 (stale ids past the stage's last K-step are never used)
#pragma unroll
                for (int g = 0; g < 8; ++g) r[g] = ids[g];
                // The MMA warp has finished this producer's previous stage: its gather slot is free,
                // and so is the meta slot that stage's tiles were in.
                if (!mbar_wait_t<PROF>(empty_bar, gph ^ 1u, abort_flag, limit, w_empty_g, 2)) { raise(prm, ss, ST_TIMEOUT_EMPTY); break; }
                armed = false;
                prof_mark<PROF>(prm.dbg, it, 2);
                if (end) {                      // pass the end marker on to the MMA warp
                    mbar_arrive(full_bar);
                    break;
                }
                if (skip & SKIP_GATHER) {       // experiment: nothing to wait for
                    mbar_arrive(full_bar);
                } else {
                    // bytes the K-steps of this stage bring in: 16 slots x 128 features x NH slabs each
                    mbar_expect_tx(full_bar, (uint32_t)(nmma * 16 * SLAB * 2 * NH) >> (narrow ? 1 : 0));
                    armed = true;
                    armed_ph = gph;
                    // copy (K-step m, slot group g, feature half oh): slots 4g .. 4g+3 of K-step m land in
                    // slot half g / 2, lines (4g) % 8 .. +3 of the atom
#pragma unroll
                    for (int m0 = 0; m0 < MMAS_PER_STAGE; m0 += 2) {
                        if (m0 > 0) {
                            if (m0 >= nmma) break;
#pragma unroll
                            for (int g = 0; g < 8; ++g) r[g] = ids[m0 * 4 + g];
                        }
#pragma unroll
                        for (int mm = 0; mm < 2; ++mm) {
                            if (m0 + mm < nmma) {
#pragma unroll
                                for (int g = 0; g < 4; ++g) {
                                    const int4 rr = r[mm * 4 + g];
#pragma unroll
                                    for (int oh = 0; oh < 2; ++oh) {
                                        if (oh == 1 && narrow) break;      // features 64 .. 127 do not exist: nothing to fetch
                                        const uint32_t off = (uint32_t)((m0 + mm) * NH * A_MMA_BYTES + (g >> 1) * A_SBO + oh * A_LBO + ((4 * g) & 7) * 128);
#pragma unroll
                                        for (int h = 0; h < NH; ++h)
                                            tma_gather4(dst_slot + off + (uint32_t)(h * A_MMA_BYTES), &b_map, full_bar, h * SLAB + oh * 64, rr.x, rr.y, rr.z, rr.w, keep);
                                    }
                                }
                            }
                        }
                    }
                }
                prof_mark<PROF>(prm.dbg, it, 3);
                // the meta slot of stage n - 1 takes the tiles of stage n - 1 + D
                if (n >= 1 && !seen_end) request_tiles();
            }
            if (*abort_flag) {
                // aborted with copies of this thread possibly in flight: wait (bounded) until they
                // have landed, the CTA is about to give its shared memory back
                if (armed) (void)mbar_wait_drain(full_bar, armed_ph, limit);
                for (uint32_t j = 1; j <= D && j <= n_meta; ++j) {
                    const uint32_t nj = n_meta - j;
                    (void)mbar_wait_drain(smem_u32(&ss->full_m[gs * D + nj % D]), (nj / D) & 1u, limit);
                }
            }
            if (PROF && prm.dbg && gs == 0) { prm.dbg[blockIdx.x * 16 + 2] = w_full_m; prm.dbg[blockIdx.x * 16 + 3] = w_empty_g; prm.dbg[blockIdx.x * 16 + 13] = w_desc; prm.dbg[blockIdx.x * 16 + 5] = prof_clock<PROF>() - t_prod0; (void)t_meta; }
        }
        __syncwarp();
    } else if (warp == MMA_WARP) {
        // ------------------------------------------------------------------ MMA issuer (one thread)
        if (elect_one()) {
            const uint32_t idesc = (1u << 4) | ((uint32_t)prm.is_bf16 << 7) | ((uint32_t)prm.is_bf16 << 10) |
                                   (1u << 15) | ((16u >> 3) << 17) | ((128u >> 4) << 24);
            // descriptors of stage 0 / meta slot 0; other stages add their byte offset >> 4 to the low word
            const uint64_t a_desc0 = smem_desc(smem_u32(ring_g), A_LBO, A_SBO, 2);
            const uint64_t b_desc0 = smem_desc(smem_u32(ring_m), TILE_BYTES, 128, 0);
            uint32_t ai = 0, buf = 0;
            long long w_acc = 0, w_fg = 0;
            const long long t_mark = prof_clock<PROF>();
            constexpr uint32_t D = (uint32_t)C::kMetaDepth;
            uint32_t it = 0, gph = 0, nd = 0;              // stage it = gs + n * kStages, nd = n % D
            bool issued = false, stop = false;
            // The loop over the ring slots is unrolled, so that the slot's barrier addresses and
            // operand descriptors are constants of the code: this thread's instruction count per
            // stage is what bounds the kernel once the gathers keep up.
            while (!stop) {
#pragma unroll
                for (int gs = 0; gs < C::kStages; ++gs) {
                    // The producers arrive on full_g only after they have seen full_m of the same stage,
                    // so this one wait also covers the tile values and the command word.
                    if (!mbar_wait_t<PROF>(smem_u32(&ss->full_g[gs]), gph, abort_flag, limit, w_fg, 1)) { raise(prm, ss, ST_TIMEOUT_FULL); stop = true; break; }
                    prof_mark<PROF>(prm.dbg, it, 5);
                    if (it == 0) prof_stamp<PROF>(prm.dbg, 3);     // first stage ready for the MMAs
                    const uint32_t ms = (uint32_t)gs * D + nd;     // the stage's meta slot
                    const uint32_t cmd = *reinterpret_cast<const volatile uint32_t *>(ring_m + ms * META_BYTES + META_TILE_BYTES + META_COL_BYTES);
                    if (cmd & CMD_END) { stop = true; break; }
                    if (cmd & CMD_FIRST) {
                        buf = ai % NACC;
                        const uint32_t aph = (ai / NACC) & 1u;
                        ++ai;
                        if (!mbar_wait_t<PROF>(smem_u32(&ss->acc_empty[buf]), aph ^ 1u, abort_flag, limit, w_acc)) { raise(prm, ss, ST_TIMEOUT_ACC); stop = true; break; }
                        tc_fence_after();              // the epilogue's tcgen05.ld of this buffer happened before
                    }
                    // (the copied data is handed over by the mbarrier its bytes complete on: no fence)
                    const uint32_t d_tmem = tmem_base + buf * C::kAccCols;
                    const uint64_t ad = a_desc0 + (uint64_t)(gs * (C::kStageBytes >> 4));
                    const uint64_t bd = b_desc0 + (uint64_t)(ms * (META_BYTES >> 4));
                    const uint32_t first = (cmd & CMD_FIRST) ? 0u : 1u;
                    if (!(skip & SKIP_MMA)) {
                        if ((cmd & CMD_COUNT) == (uint32_t)STAGE_TILES) {       // a full stage: no per-K-step tests
#pragma unroll
                            for (int m = 0; m < MMAS_PER_STAGE; ++m)
#pragma unroll
                                for (int h = 0; h < NH; ++h) {
                                    const uint64_t am = ad + (uint64_t)(((m * NH + h) * A_MMA_BYTES) >> 4), bm = bd + (uint64_t)((m * 2 * TILE_BYTES) >> 4);
                                    if (m == 0) umma_f16(d_tmem + h * 16, am, bm, idesc, first);
                                    else umma_f16_acc(d_tmem + h * 16, am, bm, idesc);
                                }
                        } else {
                            const int nmma = (int)((cmd & CMD_COUNT) + 1u) >> 1;
#pragma unroll
                            for (int m = 0; m < MMAS_PER_STAGE; ++m)
                                if (m < nmma) {
#pragma unroll
                                    for (int h = 0; h < NH; ++h)
                                        umma_f16(d_tmem + h * 16, ad + (uint64_t)(((m * NH + h) * A_MMA_BYTES) >> 4),
                                                 bd + (uint64_t)((m * 2 * TILE_BYTES) >> 4), idesc, m > 0 ? 1u : first);
                                }
                        }
                    }
                    issued = true;
                    umma_commit(smem_u32(&ss->empty_g[gs]));
                    if (cmd & CMD_LAST) umma_commit(smem_u32(&ss->acc_full[buf]));
                    prof_mark<PROF>(prm.dbg, it, 6);
                    ++it;
                }
                gph ^= 1u;
                if (++nd == D) nd = 0;
            }
            prof_stamp<PROF>(prm.dbg, 4);                          // last MMA issued
            if (issued && *abort_flag) {
                // aborted: tensor memory is freed below, so the MMAs still in the pipe must finish first
                umma_commit(smem_u32(&ss->drain));
                (void)mbar_wait_drain(smem_u32(&ss->drain), 0u, limit);
            }
            if (PROF && prm.dbg) {
                long long *d = prm.dbg + blockIdx.x * 16;
                d[4] = w_acc; d[6] = w_fg; d[10] = prof_clock<PROF>() - t_mark; d[11] = it;
            }
        }
        __syncwarp();
    }

    // teardown: everybody meets, then the allocating warp frees tensor memory
    tc_fence_before();
    __syncthreads();
    if (warp == MMA_WARP) {
        tc_fence_after();
        tmem_dealloc(tmem_base, C::kTmemCols);
    }
    if (threadIdx.x == 0) prof_stamp<PROF>(prm.dbg, 6);           // CTA done
}

// ---------------------------------------------------------------------------------------------
// host side
// ---------------------------------------------------------------------------------------------
constexpr size_t STATUS_BYTES = 256;
constexpr size_t DEBUG_BYTES = 1024 * 16 * sizeof(long long);   // profiling counters (unused by the product kernel, kept in the layout)
constexpr size_t FIX_BYTES = 1024 * 4 * sizeof(int64_t);      // per-CTA counters of finished pieces of split windows
constexpr int64_t MIN_TILES_PER_CTA = 64;
constexpr int SCRATCH_CTAS_PER_SM = 4;                        // partial-tile slots are sized for up to this many CTAs per SM
static_assert(GRWS_TC5_CTAS_PER_SM <= SCRATCH_CTAS_PER_SM, "scratch sizing");

// Worst status any SpMM launch on this device has reported since the word was last cleared
// (grws_spmm_last_status / grws_spmm_check read it): callers that never look at the status word
// of their scratch buffer, or that use the built-in scratch, learn of a timed-out pipeline here.
static __device__ int g_sticky_status;

// What the host keeps per device: properties read once, the kernels' shared-memory opt-in, and the
// device addresses of the library's __device__ variables (their names are host-side handles only).
struct DeviceState {
    int ready;                 // 0 = not set up, 1 = set up (release / acquire)
    int sms;
    int *sticky;               // device address of g_sticky_status
    void *static_scratch;      // device address of the built-in scratch array (looked up on first use)
};
constexpr int MAX_DEVICES = 64;
static DeviceState g_devices[MAX_DEVICES];
static long long g_wait_limit = WAIT_LIMIT_CYCLES;

template <int NH>
static cudaError_t opt_in_smem() {
    cudaError_t e = cudaFuncSetAttribute(spmm_tc5_kernel<NH, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)Cfg<NH>::kSmem);
    if (NH == 1 && e == cudaSuccess)
        e = cudaFuncSetAttribute(spmm_tc5_kernel<1, false, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)Cfg<1>::kSmem);
#ifdef GRWS_TC5_PROFILING
    if (e == cudaSuccess) e = cudaFuncSetAttribute(spmm_tc5_kernel<NH, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)Cfg<NH>::kSmem);
    if (NH == 1 && e == cudaSuccess)
        e = cudaFuncSetAttribute(spmm_tc5_kernel<1, true, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)Cfg<1>::kSmem);
#endif
    return e;
}

// state of the current device; the first call on a device sets it up (with that device current)
static int device_state(DeviceState **out) {
    int dev = 0;
    GRWS_CUDA_TRY(cudaGetDevice(&dev));
    if (dev < 0 || dev >= MAX_DEVICES) return fail(GRWS_ERR_UNSUPPORTED, "device ordinal %d beyond %d", dev, MAX_DEVICES);
    DeviceState *d = &g_devices[dev];
    if (!__atomic_load_n(&d->ready, __ATOMIC_ACQUIRE)) {
        // two threads may both get here: they compute the same values, the stores are idempotent
        int sms = 0;
        GRWS_CUDA_TRY(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev));
        if (sms <= 0) return fail(GRWS_ERR_CUDA, "device %d reports %d SMs", dev, sms);
        GRWS_CUDA_TRY(opt_in_smem<1>());
        GRWS_CUDA_TRY(opt_in_smem<2>());
        void *p = nullptr;
        GRWS_CUDA_TRY(cudaGetSymbolAddress(&p, g_sticky_status));
        if (p == nullptr) return fail(GRWS_ERR_CUDA, "cudaGetSymbolAddress returned a null address");
        d->sms = sms;
        d->sticky = static_cast<int *>(p);
        __atomic_store_n(&d->ready, 1, __ATOMIC_RELEASE);
    }
    *out = d;
    return GRWS_OK;
}

#ifdef GRWS_TC5_PROFILING
static int profile_env(const char *name) {
    const char *e = getenv(name);
    return e ? atoi(e) : 0;
}
#endif

// Zeroes `n` 32-bit words (status word, split-window counters) and lets the SpMM kernel queued
// behind it start at once: that kernel's set-up and first stages overlap this one, and it waits
// (griddepcontrol.wait) only where it first touches these words.
__global__ void zero_words_kernel(int *p, int n) {
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    for (int i = threadIdx.x; i < n; i += blockDim.x) p[i] = 0;
}

template <int NH, bool PROF, bool NARROW>
static cudaError_t launch_dependent(const Params &prm, const CUtensorMap &b_map, int G, cudaStream_t stream) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((unsigned)G);
    cfg.blockDim = dim3(NUM_THREADS);
    cfg.dynamicSmemBytes = Cfg<NH>::kSmem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
#ifdef GRWS_TC5_NO_PDL
    cfg.numAttrs = 0;
#else
    cfg.numAttrs = 1;
#endif
    return cudaLaunchKernelEx(&cfg, spmm_tc5_kernel<NH, PROF, NARROW>, prm, b_map);
}

template <int NH, bool NARROW = false>
static cudaError_t launch_kernel(const Params &prm, const CUtensorMap &b_map, int G, cudaStream_t stream) {
#ifdef GRWS_TC5_PROFILING
    if (prm.dbg) return launch_dependent<NH, true, NARROW>(prm, b_map, G, stream);
#endif
    return launch_dependent<NH, false, NARROW>(prm, b_map, G, stream);
}

// Tensor map of the dense operand for the row gathers: 2-D [K rows][N features], box of one row
// by 64 features (128 bytes), 128-byte swizzle, zero fill outside the tensor.
static int encode_b_map(CUtensorMap *map, const void *B, int is_bf16, int64_t K, int64_t N, int64_t ldb) {
    typedef CUresult (*EncodeFn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *,
                                 const cuuint64_t *, const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave,
                                 CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
    static EncodeFn encode = [] {
        void *fn = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &q) != cudaSuccess ||
            q != cudaDriverEntryPointSuccess)
            fn = nullptr;
        return reinterpret_cast<EncodeFn>(fn);
    }();
    if (!encode) return fail(GRWS_ERR_CUDA, "cuTensorMapEncodeTiled is not available from this driver");
    const cuuint64_t dims[2] = {(cuuint64_t)N, (cuuint64_t)K};
    const cuuint64_t strides[1] = {(cuuint64_t)ldb * 2};
    const cuuint32_t box[2] = {64, 1};
    const cuuint32_t estr[2] = {1, 1};
    const CUresult r = encode(map, is_bf16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2,
                              const_cast<void *>(B), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                              CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                              CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return fail(GRWS_ERR_CUDA, "cuTensorMapEncodeTiled failed with CUresult %d", (int)r);
    return GRWS_OK;
}

// ---------------------------------------------------------------------------------------------
// Tile ranges computed once per graph.
//
// A CTA's run time follows its number of stages (a window of n tiles takes ceil(n / 8) stages; the
// last one of a window is padded), not its number of tiles: equal tile counts leave the stage counts
// of the CTAs 10-12 % apart on a power-law graph, and the slowest CTA sets the kernel's time.  The
// plan cuts the prefix sum of the windows' stage counts into equal parts instead.  A cut that falls
// into a window of at most PLAN_LONG_WINDOW_STAGES stages moves to the nearer end of that window; a
// longer window is cut at a stage boundary and its pieces are put together as for searched ranges.
// The search for the ranges (three dependent rounds of loads at the start of every launch) is
// replaced by one load.
//
// Layout (int4 units): [0] magic, grid, W lo, W hi; [1] T lo, T hi, 0, 0; then per cut k = 0..grid:
// [2 + 2k] first tile lo, hi, first window lo, hi; [3 + 2k] first / last holder of the window the range
// starts in, last holder of the window it ends in, 0; behind them the stage prefix sums [W + 1].
// ---------------------------------------------------------------------------------------------
__device__ __forceinline__ int64_t plan_cut_tile(const int4 *plan, int k) {
    const int4 c = plan[2 + 2 * k];
    return ((int64_t)(uint32_t)c.y << 32) | (uint32_t)c.x;
}

__global__ void __launch_bounds__(1024) spmm_plan_kernel(const int64_t *__restrict__ off, int64_t W, int G, int4 *plan, int64_t *sp) {
    __shared__ int64_t part[1024];
    const int t = threadIdx.x;
    const int64_t per = (W + 1023) / 1024;
    const int64_t w0 = min(W, (int64_t)t * per), w1 = min(W, w0 + per);
    int64_t sum = 0;
    for (int64_t w = w0; w < w1; ++w) sum += (off[w + 1] - off[w] + STAGE_TILES - 1) / STAGE_TILES;
    part[t] = sum;
    __syncthreads();
    for (int d = 1; d < 1024; d <<= 1) {
        const int64_t v = t >= d ? part[t - d] : 0;
        __syncthreads();
        part[t] += v;
        __syncthreads();
    }
    int64_t run = part[t] - sum;
    for (int64_t w = w0; w < w1; ++w) {
        sp[w] = run;
        run += (off[w + 1] - off[w] + STAGE_TILES - 1) / STAGE_TILES;
    }
    const int64_t S = part[1023], T = off[W];
    if (t == 1023) sp[W] = S;
    __syncthreads();
    // with fewer than 8 stages per CTA nothing is split: the pieces of a split window must all be
    // non-empty, which equal stage shares guarantee only when there are at least as many stages as CTAs
    const int64_t long_stages = S >= 8 * (int64_t)G ? PLAN_LONG_WINDOW_STAGES : INT64_MAX;
    for (int k = t; k <= G; k += 1024) {
        int64_t s, wf;
        if (k == 0) { s = 0; wf = 0; }
        else if (k == G || S == 0) { s = T; wf = W; }
        else {
            const int64_t tgt = ((int64_t)k * S) / G;          // S < 2^40 stages, k < 2^12
            int64_t lo = 0, hi = W - 1;                        // last window whose prefix is <= tgt (it has stages)
            while (lo < hi) {
                const int64_t mid = (lo + hi + 1) >> 1;
                if (sp[mid] <= tgt) lo = mid; else hi = mid - 1;
            }
            const int64_t a = off[lo], b = off[lo + 1], before = tgt - sp[lo], after = sp[lo + 1] - tgt;
            if (before == 0) { s = a; wf = lo; }
            else if (before + after <= long_stages) {
                if (after < before) { s = b; wf = lo + 1; } else { s = a; wf = lo; }
            } else { s = a + before * STAGE_TILES; wf = lo; }
        }
        plan[2 + 2 * k] = make_int4((int)(uint32_t)s, (int)(s >> 32), (int)(uint32_t)wf, (int)(wf >> 32));
    }
    __syncthreads();
    for (int k = t; k <= G; k += 1024) {
        int4 h = make_int4(k, k, k, 0);
        if (k < G) {
            const int4 c = plan[2 + 2 * k];
            const int64_t s = plan_cut_tile(plan, k), e = plan_cut_tile(plan, k + 1);
            const int64_t wf = ((int64_t)(uint32_t)c.w << 32) | (uint32_t)c.z;
            if (s < e && wf < W && s > off[wf]) {
                // the range starts inside window wf = [a, b): its pieces are held by the CTA whose range
                // holds tile a up to the one whose range holds tile b - 1
                const int64_t a = off[wf], b = off[wf + 1];
                int j = k;
                while (j > 0 && plan_cut_tile(plan, j) > a) --j;
                h.x = j;
                j = k;
                while (j + 1 < G && plan_cut_tile(plan, j + 1) < b) ++j;
                h.y = j;
            }
            if (s < e && e < T) {
                const int4 n = plan[2 + 2 * (k + 1)];
                const int64_t we = ((int64_t)(uint32_t)n.w << 32) | (uint32_t)n.z;
                if (we < W && e > off[we] && off[we] >= s) {
                    const int64_t b = off[we + 1];
                    int j = k + 1;
                    while (j + 1 < G && plan_cut_tile(plan, j + 1) < b) ++j;
                    h.z = j;
                }
            }
        }
        plan[3 + 2 * k] = h;
    }
    if (t == 0) {
        plan[0] = make_int4(PLAN_MAGIC, G, (int)(uint32_t)W, (int)(W >> 32));
        plan[1] = make_int4((int)(uint32_t)T, (int)(T >> 32), 0, 0);
    }
}

// number of persistent CTAs of one pass and the width of a pass, as the launch chooses them
static void launch_shape(int sms, int64_t num_tiles_bound, int64_t K, int64_t N, int *G_out, int64_t *pass_n_out) {
    // Width 256: one pass with two slabs per stage (one CTA per SM), or two passes of 128 columns.
    // Two passes read the tiles twice but gather from half as many bytes of the dense operand,
    // which then stays in L2 next to the tile stream, and they run two CTAs per SM: measured 4 %
    // faster at 86 MB of operand, 20 % at 119 MB.  Small operands keep the single pass (half the
    // launches).
    const bool split = N == 256 && K * 512 > SPLIT256_OPERAND_BYTES;
    const int64_t pass_n = (N <= 128 || split) ? 128 : 256;     // widths below 128 run as one pass over a zero-extended operand
    // one persistent CTA per SM slot, fewer for small products: a CTA range below ~64 tiles is mostly
    // cuts through windows, whose pieces then cost more to put together than the tiles to multiply
    int G = sms * (pass_n == 128 ? Cfg<1>::kCtasPerSm : Cfg<2>::kCtasPerSm);
    const int64_t g_small = num_tiles_bound / MIN_TILES_PER_CTA;
    if (g_small < G) G = g_small < 1 ? 1 : (int)g_small;
    *G_out = G;
    *pass_n_out = pass_n;
}

static size_t plan_bytes_for(int G, int64_t W) {
    return sizeof(int4) * (2 + 2 * ((size_t)G + 1)) + sizeof(int64_t) * ((size_t)W + 1);
}
}  // namespace tc5

// fp16 / bf16 operands of width 256, or of any multiple of 8 up to 128 (narrower operands are
// multiplied as 128 features of which the missing ones are zeros)
bool spmm_tc5_supported(int dtype, int64_t N) {
    return (dtype == GRWS_F16 || dtype == GRWS_BF16) && (N == 256 || (N >= 8 && N <= 128 && N % 8 == 0));
}

// What GRWS_SPMM_AUTO picks the tcgen05 kernel for: widths 128 and 256 always; narrower operands from
// 16 features and 512 tiles on (the kernel costs the same for every width up to 64 and up to 128, so
// it wins by 25-35 % on large graphs -- measured on a 114 M-entry graph and on a power-law graph of
// 2.5 M entries -- and the blocks of a sampled step, a few hundred to a few thousand tiles, take it
// 10-13 us against 35-120 us on the warp-MMA kernel, whose few warps walk such a block serially).
bool spmm_tc5_preferred(int dtype, int64_t N, int64_t num_tiles_bound) {
    if (!spmm_tc5_supported(dtype, N)) return false;
    return N >= 128 || (N >= GRWS_TC5_AUTO_MIN_N && num_tiles_bound >= GRWS_TC5_AUTO_MIN_TILES);
}

// Scratch of one call: status word | split-window counters | profiling counters | two fp32 partial
// tiles per CTA.  0 when the device cannot be queried (the launch then reports the error).
size_t spmm_tc5_scratch_bytes(int64_t num_tiles_bound, int64_t N) {
    (void)num_tiles_bound;
    tc5::DeviceState *d = nullptr;
    if (tc5::device_state(&d) != GRWS_OK) return 0;
    if (N < 128) N = 128;                     // partial tiles are laid out at the width of a pass
    return tc5::STATUS_BYTES + tc5::DEBUG_BYTES + tc5::FIX_BYTES +
           (size_t)d->sms * tc5::SCRATCH_CTAS_PER_SM * 2 * TILE_ROWS * (size_t)N * sizeof(float);
}

// Bytes of the plan of one graph (0 when the device cannot be queried).
size_t spmm_tc5_plan_bytes(int64_t W, int64_t num_tiles_bound, int64_t K, int64_t N) {
    tc5::DeviceState *d = nullptr;
    if (tc5::device_state(&d) != GRWS_OK) return 0;
    int G = 0;
    int64_t pass_n = 0;
    tc5::launch_shape(d->sms, num_tiles_bound, K, N, &G, &pass_n);
    return tc5::plan_bytes_for(G, W);
}

int spmm_tc5_plan_build(const int64_t *window_offset, int64_t W, int64_t num_tiles_bound, int64_t K, int64_t N,
                        void *plan, size_t plan_bytes, cudaStream_t stream) {
    using namespace tc5;
    DeviceState *dev = nullptr;
    if (int st = device_state(&dev)) return st;
    int G = 0;
    int64_t pass_n = 0;
    launch_shape(dev->sms, num_tiles_bound, K, N, &G, &pass_n);
    if (plan == nullptr || plan_bytes < plan_bytes_for(G, W))
        return fail(GRWS_ERR_SCRATCH, "spmm plan too small: %zu < %zu bytes", plan_bytes, plan_bytes_for(G, W));
    int4 *p = static_cast<int4 *>(plan);
    spmm_plan_kernel<<<1, 1024, 0, stream>>>(window_offset, W, G, p, reinterpret_cast<int64_t *>(p + 2 + 2 * ((size_t)G + 1)));
    GRWS_CUDA_TRY(cudaGetLastError());
    return GRWS_OK;
}

__global__ void spmm_zero_rows_kernel(void *C, int64_t rows, int64_t row_bytes16, int64_t ld_bytes16) {
    // 16-byte pieces of `rows` rows of C (rows are 16-byte aligned)
    const int64_t n = rows * row_bytes16;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x)
        reinterpret_cast<uint4 *>(C)[(i / row_bytes16) * ld_bytes16 + i % row_bytes16] = make_uint4(0u, 0u, 0u, 0u);
}

// C = 0 for a product without tiles or without dense rows (the kernels never run on it)
int spmm_zero_output(void *C, int c_dtype, int64_t ldc, int64_t W, int64_t N, cudaStream_t stream) {
    const int64_t rows = W * TILE_ROWS, esz = (int64_t)dtype_bytes(c_dtype);
    if (rows == 0) return GRWS_OK;
    const int64_t pieces = rows * (N * esz / 16);
    int64_t blocks = ceil_div(pieces, 256);
    if (blocks > 4096) blocks = 4096;
    spmm_zero_rows_kernel<<<(unsigned)blocks, 256, 0, stream>>>(C, rows, N * esz / 16, ldc * esz / 16);
    GRWS_CUDA_TRY(cudaGetLastError());
    return GRWS_OK;
}

int spmm_tc5_launch(const int64_t *window_offset, const int32_t *cols, const void *vals, int dtype,
                    const void *B, int64_t ldb, void *C, int c_dtype, int64_t ldc, int64_t W,
                    int64_t num_tiles_bound, int64_t K, int64_t N, void *scratch, size_t scratch_bytes,
                    const void *plan, size_t plan_bytes, cudaStream_t stream) {
    using namespace tc5;
    DeviceState *dev = nullptr;
    if (int st = device_state(&dev)) return st;
    const size_t need = spmm_tc5_scratch_bytes(num_tiles_bound, N);
    if (scratch_bytes < need || scratch == nullptr)
        return fail(GRWS_ERR_SCRATCH, "spmm scratch too small: %zu < %zu bytes", scratch_bytes, need);
    Params prm;
    prm.window_offset = window_offset; prm.cols = cols; prm.vals = vals; prm.B = B; prm.C = C;
    prm.status = static_cast<int *>(scratch);
    prm.sticky = dev->sticky;
    prm.skip = 0;
    prm.dbg = nullptr;
    prm.wait_limit = __atomic_load_n(&g_wait_limit, __ATOMIC_RELAXED);
#ifdef GRWS_TC5_PROFILING
    // profiling build only: GRWS_TC5_PROFILE=1 records wait times and a stage timeline behind the
    // split-window counters, GRWS_TC5_SKIP leaves parts of the work out (see the SKIP_* bits)
    if (profile_env("GRWS_TC5_PROFILE")) {
        prm.dbg = reinterpret_cast<long long *>(static_cast<char *>(scratch) + STATUS_BYTES + FIX_BYTES);
        prm.skip = profile_env("GRWS_TC5_SKIP");
    }
#endif
    // layout: status word | split-window counters | profiling counters | partial tiles; the first two are zeroed together
    prm.split_count = reinterpret_cast<int *>(static_cast<char *>(scratch) + STATUS_BYTES);
    prm.partial = reinterpret_cast<float *>(static_cast<char *>(scratch) + STATUS_BYTES + DEBUG_BYTES + FIX_BYTES);
    prm.W = W; prm.N = N; prm.ldb = ldb; prm.ldc = ldc; prm.c_dtype = c_dtype;
    prm.is_bf16 = dtype == GRWS_BF16 ? 1 : 0;
    int G = 0;
    int64_t pass_n = 0;
    launch_shape(dev->sms, num_tiles_bound, K, N, &G, &pass_n);
    prm.plan = nullptr;
    if (plan != nullptr) {
        if (plan_bytes < plan_bytes_for(G, W))
            return fail(GRWS_ERR_SCRATCH, "spmm plan too small: %zu < %zu bytes", plan_bytes, plan_bytes_for(G, W));
        prm.plan = static_cast<const int4 *>(plan);
    }
    if ((size_t)G * sizeof(int) > FIX_BYTES) return fail(GRWS_ERR_UNSUPPORTED, "more CTAs (%d) than split-window counters", G);
    const size_t c_elem = c_dtype == GRWS_F32 ? 4 : 2;
    for (int64_t col0 = 0; col0 < N; col0 += pass_n) {
        prm.B = static_cast<const char *>(B) + col0 * 2;
        prm.C = static_cast<char *>(C) + col0 * c_elem;
        prm.N = pass_n;
        prm.n_valid = (int)(N - col0 < pass_n ? N - col0 : pass_n);
        // the tensor map covers the features that exist: the TMA unit fills the rest of a 64-feature box with zeros
        alignas(64) CUtensorMap b_map;
        if (int st = encode_b_map(&b_map, prm.B, prm.is_bf16, K, prm.n_valid, ldb)) return st;
        // the status word is cleared once per call, the split-window counters before every pass
        if (col0 == 0) zero_words_kernel<<<1, 256, 0, stream>>>(static_cast<int *>(scratch), (int)(STATUS_BYTES / sizeof(int)) + G);
        else zero_words_kernel<<<1, 256, 0, stream>>>(prm.split_count, G);
        GRWS_CUDA_TRY(cudaGetLastError());
        GRWS_CUDA_TRY((pass_n == 256 ? launch_kernel<2>(prm, b_map, G, stream)
                       : prm.n_valid < 128 ? launch_kernel<1, true>(prm, b_map, G, stream) : launch_kernel<1>(prm, b_map, G, stream)));
        GRWS_CUDA_TRY(cudaGetLastError());
    }
    return GRWS_OK;
}

}  // namespace grws

// ---------------------------------------------------------------------------------------------
// Status of the tcgen05 SpMM launches of the current device.
// ---------------------------------------------------------------------------------------------
extern "C" __attribute__((visibility("default")))
int grws_spmm_last_status(int *out_status, int reset, void *stream) {
    using namespace grws;
    GRWS_REQUIRE(out_status != nullptr, "null pointer");
    tc5::DeviceState *d = nullptr;
    if (int st = tc5::device_state(&d)) return st;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    GRWS_CUDA_TRY(cudaMemcpyAsync(out_status, d->sticky, sizeof(int), cudaMemcpyDefault, s));
    if (reset) GRWS_CUDA_TRY(cudaMemsetAsync(d->sticky, 0, sizeof(int), s));
    return GRWS_OK;
}

extern "C" __attribute__((visibility("default")))
int grws_spmm_check(void *stream) {
    using namespace grws;
    tc5::DeviceState *d = nullptr;
    if (int st = tc5::device_state(&d)) return st;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    int status = 0;
    GRWS_CUDA_TRY(cudaMemcpyAsync(&status, d->sticky, sizeof(int), cudaMemcpyDeviceToHost, s));
    GRWS_CUDA_TRY(cudaStreamSynchronize(s));
    if (status == 0) return GRWS_OK;
    GRWS_CUDA_TRY(cudaMemsetAsync(d->sticky, 0, sizeof(int), s));
    static const char *const what[] = {"", "gathered rows never arrived (full_g)", "a gather slot was never released (empty_g)",
                                       "an accumulator hand-over never happened (acc)", "tiles / column ids never arrived (meta)"};
    return fail(GRWS_ERR_DEVICE, "a tcgen05 SpMM launch on this device gave up waiting: %s (code %d); its output is incomplete",
                status >= 1 && status <= 4 ? what[status] : "unknown wait", status);
}

extern "C" __attribute__((visibility("default")))
int grws_spmm_set_wait_limit(long long sm_clocks) {
    using namespace grws;
    GRWS_REQUIRE(sm_clocks >= 0, "negative limit");
    __atomic_store_n(&tc5::g_wait_limit, sm_clocks > 0 ? sm_clocks : tc5::WAIT_LIMIT_CYCLES, __ATOMIC_RELAXED);
    return GRWS_OK;
}

// ---------------------------------------------------------------------------------------------
// Forward SpMM for callers that must not allocate device memory.
//
// Some hosts of this library cannot call cudaMalloc around an SpMM: a plugin that runs inside
// another framework's stream-ordered or pooled allocator and is handed only its input and output
// buffers, a real-time inference loop whose memory was frozen at start-up, a caller that is in
// the middle of capturing work it does not own.  For them the scratch of the tcgen05 kernel (its
// status word, the per-CTA split-window counters and the fp32 partial tiles of windows that were split
// between CTAs) lives in the fixed array below instead of a caller-provided buffer.
//
//   * The array is STATIC_SCRATCH_BYTES (about 21 MB) and every GPU that loads the library keeps
//     it until the process exits.  It is sized for dense widths up to 256 on a device with up to
//     160 SMs; anything that would need more is rejected with GRWS_ERR_SCRATCH.
//   * In host code the array's name is only a host-side handle, not a device address.  The device
//     address is looked up with cudaGetSymbolAddress, once per device, with that device current,
//     on the first call made on that device -- so make that first call before any stream capture.
//   * All calls share the array and it keeps the last call's contents: the status word is cleared
//     on the stream before each launch, everything else is written before it is read within a
//     call.  Two calls that overlap on the GPU (different streams, or one device used from two
//     threads) race on it; serialise them or use grws_spmm_fwd with separate scratch buffers.
//   * The call's status word lives inside the array, out of the caller's reach: a pipeline wait
//     that ran out is reported through grws_spmm_last_status / grws_spmm_check instead.
//   * No cudaMalloc, cudaFree or allocating library routine is called.
// ---------------------------------------------------------------------------------------------
namespace grws {
namespace tc5 {

constexpr int STATIC_MAX_SMS = 160;
constexpr int STATIC_MAX_N = 256;
constexpr size_t STATIC_SCRATCH_BYTES =
    STATUS_BYTES + DEBUG_BYTES + FIX_BYTES + (size_t)STATIC_MAX_SMS * SCRATCH_CTAS_PER_SM * 2 * TILE_ROWS * STATIC_MAX_N * sizeof(float);
static_assert(STATIC_SCRATCH_BYTES == GRWS_SPMM_STATIC_SCRATCH_BYTES, "the header states the size of the built-in scratch");

static __device__ __align__(256) unsigned char static_scratch[STATIC_SCRATCH_BYTES];

// device address of static_scratch on the current device (looked up once per device)
static int static_scratch_address(void **out) {
    DeviceState *d = nullptr;
    if (int st = device_state(&d)) return st;
    void *p = __atomic_load_n(&d->static_scratch, __ATOMIC_ACQUIRE);
    if (p == nullptr) {
        GRWS_CUDA_TRY(cudaGetSymbolAddress(&p, static_scratch));
        if (p == nullptr) return fail(GRWS_ERR_CUDA, "cudaGetSymbolAddress returned a null address");
        __atomic_store_n(&d->static_scratch, p, __ATOMIC_RELEASE);      // every thread resolves the same address
    }
    *out = p;
    return GRWS_OK;
}

}  // namespace tc5
}  // namespace grws

extern "C" __attribute__((visibility("default")))
int grws_spmm_fwd_static(const int64_t *window_offset, const int32_t *cols, const void *vals, int val_dtype,
                         const void *B, int b_dtype, int64_t ldb, void *C, int c_dtype, int64_t ldc,
                         int64_t num_windows, int64_t num_tiles_bound, int64_t K, int64_t N, void *stream) {
    using namespace grws;
    GRWS_REQUIRE(num_windows >= 0 && num_tiles_bound >= 0 && K >= 0 && N > 0, "negative size");
    if (num_windows == 0) return GRWS_OK;
    GRWS_REQUIRE(window_offset && C && (num_tiles_bound == 0 || K == 0 || (cols && vals && B)), "null pointer");
    GRWS_REQUIRE(c_dtype >= GRWS_F32 && c_dtype <= GRWS_BF16, "bad output dtype %d", c_dtype);
    if (val_dtype != b_dtype || !(val_dtype == GRWS_F16 || val_dtype == GRWS_BF16) || !(N == 128 || N == 256))
        return fail(GRWS_ERR_UNSUPPORTED,
                    "the allocation-free SpMM covers fp16/bf16 operands with N = 128 or 256 (got dtypes %d/%d, N = %lld); "
                    "other shapes need grws_spmm_fwd with caller scratch", val_dtype, b_dtype, (long long)N);
    GRWS_REQUIRE(ldb >= N && ldc >= N, "leading dimension smaller than N");
    GRWS_REQUIRE((ldb * 2) % 16 == 0 && (ldc * dtype_bytes(c_dtype)) % 16 == 0, "rows of B and C must be 16-byte aligned");
    GRWS_REQUIRE(aligned16(B) && aligned16(C) && aligned16(vals) && aligned16(cols), "B, C, values and column ids must be 16-byte aligned");
    if (num_tiles_bound == 0 || K == 0)      // nothing to multiply: the rows are zeros
        return spmm_zero_output(C, c_dtype, ldc, num_windows, N, static_cast<cudaStream_t>(stream));
    const size_t need = spmm_tc5_scratch_bytes(num_tiles_bound, N);
    if (need == 0) return GRWS_ERR_CUDA;
    if (need > tc5::STATIC_SCRATCH_BYTES)
        return fail(GRWS_ERR_SCRATCH, "this device needs %zu bytes of SpMM scratch, the built-in array holds %zu "
                    "(more than %d SMs?); use grws_spmm_fwd with caller scratch", need, tc5::STATIC_SCRATCH_BYTES, tc5::STATIC_MAX_SMS);
    void *scratch = nullptr;
    if (int st = tc5::static_scratch_address(&scratch)) return st;
    return spmm_tc5_launch(window_offset, cols, vals, val_dtype, B, ldb, C, c_dtype, ldc, num_windows, num_tiles_bound,
                           K, N, scratch, tc5::STATIC_SCRATCH_BYTES, nullptr, 0, static_cast<cudaStream_t>(stream));
}
