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
constexpr int META_CMD_BYTES = 16;                   // per-stage command word written by the TMA warp
constexpr int META_BYTES = META_TILE_BYTES + META_COL_BYTES + META_CMD_BYTES;
// command word: bits 0-4 tile count, bit 8 first stage of a window segment, bit 9 last stage,
// bit 10 end of this CTA's work
#ifndef GRWS_TC5_SPAN
#define GRWS_TC5_SPAN 0
#endif
#if GRWS_TC5_SPAN
// Stages that span windows: a stage is MMAS_PER_STAGE K-steps (tile pairs), each of which belongs
// to one window segment.  Command word: bits 0-2 number of K-steps, bits 4+3i .. 6+3i the flags of
// K-step i (first of its segment, last of its segment, second tile absent), bit 31 end of work.
constexpr uint32_t CMD_COUNT = 7u, CMD_END = 1u << 31;
constexpr uint32_t KS_FIRST = 1u, KS_LAST = 2u, KS_SINGLE = 4u;
__device__ __forceinline__ uint32_t kstep_flags(uint32_t cmd, int i) { return (cmd >> (4 + 3 * i)) & 7u; }
constexpr uint32_t CMD_FIRST = 0, CMD_LAST = 0;      // unused in this mode
#else
constexpr uint32_t CMD_COUNT = 31u, CMD_FIRST = 1u << 8, CMD_LAST = 1u << 9, CMD_END = 1u << 10;
#endif
static_assert((GRWS_TC5_SPAN ? MMAS_PER_STAGE : STAGE_TILES) <= (int)CMD_COUNT && STAGE_TILES % 2 == 0, "count field of the command word");
static_assert(!GRWS_TC5_SPAN || MMAS_PER_STAGE <= 9, "K-step flags of the command word");
#ifndef GRWS_TC5_NACC
#define GRWS_TC5_NACC 4
#endif
constexpr int NACC = GRWS_TC5_NACC;                              // accumulator buffers in tensor memory
#ifndef GRWS_TC5_PRODUCER_WARPS
#define GRWS_TC5_PRODUCER_WARPS 5
#endif
constexpr int NUM_PRODUCER_WARPS = GRWS_TC5_PRODUCER_WARPS;   // a multiple of the stage count
constexpr int NUM_EPILOGUE = 128;
constexpr int EPILOGUE_WARP0 = 0;                        // four warps; warp % 4 is its TMEM lane quarter
constexpr int MMA_WARP = EPILOGUE_WARP0 + 4;
constexpr int TMA_WARP = MMA_WARP + 1;
#ifndef GRWS_TC5_META_WARPS
#define GRWS_TC5_META_WARPS 1
#endif
constexpr int NUM_META_WARPS = GRWS_TC5_META_WARPS;     // they take the stages round-robin
constexpr int PRODUCER_WARP0 = TMA_WARP + NUM_META_WARPS;
#ifndef GRWS_TC5_MMA_PHYS_WARP
#define GRWS_TC5_MMA_PHYS_WARP 4
#endif
static_assert(GRWS_TC5_MMA_PHYS_WARP >= 4, "warps 0-3 are the epilogue (their index is their TMEM lane quarter)");
constexpr int NUM_THREADS = (PRODUCER_WARP0 + NUM_PRODUCER_WARPS) * 32;
static_assert(EPILOGUE_WARP0 % 4 == 0, "epilogue warps must start at a multiple of four");
constexpr int64_t SPLIT256_OPERAND_BYTES = 8ll << 20;   // dense operand size above which width 256 runs as two 128-column passes
constexpr long long WAIT_LIMIT_CYCLES = 3000000000ll; // a wait gives up after about 1.5-2.5 s of SM clocks

enum : int { ST_OK = 0, ST_TIMEOUT_FULL = 1, ST_TIMEOUT_EMPTY = 2, ST_TIMEOUT_ACC = 3, ST_TIMEOUT_META = 4 };

struct Params {
    const int64_t *window_offset;
    const int32_t *cols;
    const void *vals;
    const void *B;
    void *C;
    float *partial;
    int *status;
    int *split_count; // [grid]: pieces of the split window that starts in CTA k which are finished (zeroed before the launch)
    int64_t W, N, ldb, ldc;
    int c_dtype;
    int is_bf16;
    int lw_shift;     // a cut inside a window of at most chunk >> lw_shift tiles moves to the window start
    int skip;         // experiment knob (GRWS_TC5_SKIP): 1 = issue no MMAs, 2 = gather nothing, 4 = no output stores
    long long *dbg;   // optional [grid][16] cycle counters (wait time per role), null when not profiling
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
// adds to the bytes the current phase waits for, without arriving
__device__ __forceinline__ void mbar_expect_tx_only(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.expect_tx.relaxed.cta.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
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
// bounded wait: gives up after WAIT_LIMIT_CYCLES SM clocks or when another role already aborted.
// (The SM clock is used because reading %globaltimer costs about a microsecond per read.)
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile int *abort_flag) {
    if (mbar_try_wait(bar, parity)) return true;
    long long t0 = 0;
    for (uint32_t i = 0;; ++i) {
        if (mbar_try_wait(bar, parity)) return true;
#ifdef GRWS_TC5_BACKOFF
        __nanosleep(GRWS_TC5_BACKOFF);
#endif
        if ((i & 63u) == 63u) {
            if (*abort_flag) return false;
            const long long now = clock64();
            if (t0 == 0) t0 = now;
            if (now - t0 > WAIT_LIMIT_CYCLES) return false;
        }
    }
}
// wait that adds its duration to `acc` in the profiling build of the kernel
__device__ unsigned long long g_prof_tries[8];     // profiling build: failed try_waits per role
template <bool PROF>
__device__ __forceinline__ bool mbar_wait_t(uint32_t bar, uint32_t parity, volatile int *abort_flag, long long &acc, int role = 0) {
    if constexpr (PROF) {
        const long long t0 = clock64();
        unsigned long long tries = 0;
        bool ok = false;
        for (; tries < 100000000ull; ++tries) {
            if (mbar_try_wait(bar, parity)) { ok = true; break; }
#ifdef GRWS_TC5_BACKOFF
            __nanosleep(GRWS_TC5_BACKOFF);
#endif
        }
        acc += clock64() - t0;
        if (tries) atomicAdd(&g_prof_tries[role], tries);
        (void)abort_flag;
        return ok;
    } else {
        return mbar_wait(bar, parity, abort_flag);
    }
}
// timeline of the first stages of CTA 0 (profiling build): event e of stage `it`
template <bool PROF> __device__ __forceinline__ void prof_mark(long long *dbg, uint32_t it, int e) {
    if constexpr (PROF) { if (dbg && blockIdx.x == 0 && it < 64) dbg[12288 + it * 8 + e] = clock64(); }
}
template <bool PROF> __device__ __forceinline__ long long prof_clock() {
    if constexpr (PROF) return clock64(); else return 0;
}
__device__ __forceinline__ void bulk_g2s(uint32_t dst, const void *src, uint32_t bytes, uint32_t bar, uint64_t pol) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes.L2::cache_hint [%0], [%1], %2, [%3], %4;"
                 ::"r"(dst), "l"(src), "r"(bytes), "r"(bar), "l"(pol) : "memory");
}
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

__device__ __forceinline__ void umma_f16(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t accumulate) {
    asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
                 "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
                 ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate) : "memory");
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

struct SharedStorage {
    uint64_t full_g[16], empty_g[16], full_m[64], empty_m[64], acc_full[NACC], acc_empty[NACC];
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
    // tile / column-id slots: the TMA warp runs kMeta - kStages stages ahead of the data it has
    // already landed, which has to cover the HBM latency of the tile stream
#ifndef GRWS_TC5_META_AHEAD
#define GRWS_TC5_META_AHEAD 6
#endif
    static constexpr int kMeta = kStages + ((NH == 1) ? GRWS_TC5_META_AHEAD : 16) * 8 / STAGE_TILES;
    static constexpr int kStageBytes = MMAS_PER_STAGE * NH * A_MMA_BYTES;
    static constexpr int kAccCols = 16 * NH;
    static constexpr int kTmemCols = (NACC * kAccCols) < 32 ? 32 : NACC * kAccCols;   // 64 or 128: powers of two
    static_assert(kStages <= 16 && kMeta <= 64, "barrier arrays in SharedStorage");
    static constexpr size_t kSmem = 1024 + sizeof(SharedStorage) + 16 + (size_t)kStages * kStageBytes + (size_t)kMeta * META_BYTES;
};

__device__ __forceinline__ void raise(Params const &prm, SharedStorage *ss, int code) {
    ss->abort_flag = 1;
    atomicMax(prm.status, code);
}

// The two rare paths of the epilogue live in functions of their own (not inlined), so that their
// registers do not count against the per-window path of the kernel.

// Rows of the windows without tiles in this CTA's share of the window list (a contiguous run,
// 32 offsets per coalesced load); warp quarter q writes features 32q .. 32q+31 of every slab.
template <int NH>
__device__ __noinline__ void zero_fill_empty_windows(const int64_t *__restrict__ window_offset, void *C, int64_t ldc, int c_dtype,
                                                    int64_t W, int q, int lane) {
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
__device__ __noinline__ void sum_pieces(const float *partial, int64_t N, void *C, int64_t ldc, int c_dtype, int64_t w, int64_t k0,
                                       int64_t k_last, int q, int lane) {
    __threadfence();
    const int64_t elems = TILE_ROWS * N;
#pragma unroll
    for (int h = 0; h < NH; ++h) {
        const int64_t f = h * SLAB + 32 * q + lane;
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

template <int NH, bool PROF>
__global__ void __launch_bounds__(NUM_THREADS, Cfg<NH>::kCtasPerSm)
spmm_tc5_kernel(const Params prm, const __grid_constant__ CUtensorMap b_map) {
    using C = Cfg<NH>;
    extern __shared__ uint8_t smem_raw[];
    // the swizzled operand atoms must start on 1024-byte boundaries
    uint8_t *ring_g = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint8_t *ring_m = ring_g + (size_t)C::kStages * C::kStageBytes;
    SharedStorage *ss = reinterpret_cast<SharedStorage *>(ring_m + (size_t)C::kMeta * META_BYTES);

    // role index of this warp: the hardware warp GRWS_TC5_MMA_PHYS_WARP trades places with the
    // MMA role's default slot, which decides which other roles share a scheduler with the MMA issuer
    // the warp index is taken from lane 0 so that the compiler knows it is the same in all lanes:
    // everything derived from it (role, barrier and ring addresses) can live in uniform registers
    const int phys_warp = __shfl_sync(0xffffffffu, (int)(threadIdx.x >> 5), 0), lane = threadIdx.x & 31;
    const int warp = phys_warp == GRWS_TC5_MMA_PHYS_WARP ? MMA_WARP : (phys_warp == MMA_WARP ? GRWS_TC5_MMA_PHYS_WARP : phys_warp);
    const int64_t W = prm.W;

    if (threadIdx.x == 0) {
        for (int i = 0; i < C::kStages; ++i) { mbar_init(smem_u32(&ss->full_g[i]), 1); mbar_init(smem_u32(&ss->empty_g[i]), 1); }
        for (int i = 0; i < C::kMeta; ++i) { mbar_init(smem_u32(&ss->full_m[i]), 1); mbar_init(smem_u32(&ss->empty_m[i]), 1); }
        for (int i = 0; i < NACC; ++i) { mbar_init(smem_u32(&ss->acc_full[i]), 1); mbar_init(smem_u32(&ss->acc_empty[i]), NUM_EPILOGUE / 32); }
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

    const bool is_meta = warp >= TMA_WARP && warp < TMA_WARP + NUM_META_WARPS;
    if (is_meta || (warp >= EPILOGUE_WARP0 && warp < MMA_WARP)) {
        // ---- the two roles that walk the window structure: this CTA's tile range [s, e)
        const int64_t T = __ldg(prm.window_offset + W);
        const int64_t G = gridDim.x;
        int64_t chunk = (T + G - 1) / G;
        chunk = (chunk + 1) & ~int64_t(1);
        if (chunk < 2) chunk = 2;
        // a cut inside a window of at most chunk/16 tiles moves back to that window's start, so
        // only long windows are ever split between CTAs (tile counts stay balanced within chunk >> lw_shift)
        const int64_t long_window = chunk >> prm.lw_shift;
        int64_t w_first, s, e;
        warp_cut_pair(prm.window_offset, W, T, blockIdx.x, G, chunk, long_window, lane, &s, &e, &w_first);
        Walker wk;
        wk.init(prm.window_offset, W, s, e, blockIdx.x == 0 ? 0 : w_first, lane);

        if (is_meta) {
            // -------------------------------------------------------------- TMA producer
            const uint32_t meta_id = (uint32_t)(warp - TMA_WARP);
            // streams tile values and column ids of every stage and tells the other roles, through
            // the command word of the stage, what the stage holds
            const uint64_t pol = policy_stream();
            uint32_t it = 0;
            bool ok = true;
            long long w_empty_m = 0;
            const long long t_start = prof_clock<PROF>();
#if GRWS_TC5_SPAN
            static_assert(NUM_META_WARPS == 1, "stages that span windows are packed by one warp");
            // K-steps are packed into stages across window segments; a stage is published (command
            // word written, barrier arrived on) when it is full or the CTA's range ends
            uint32_t cmdw = 0, slot = 0;
            int stage_k = 0;
            while (ok && wk.next_segment(lane)) {
                int64_t t0 = wk.seg_s;
                bool first = true;
                while (ok && t0 < wk.seg_e) {
                    if (stage_k == 0) {
                        slot = it % C::kMeta;
                        const uint32_t ph = (it / C::kMeta) & 1u;
                        if (lane == 0) ok = mbar_wait_t<PROF>(smem_u32(&ss->empty_m[slot]), ph ^ 1u, abort_flag, w_empty_m, 5);
                        ok = __shfl_sync(0xffffffffu, ok ? 1 : 0, 0) != 0;
                        if (!ok) { if (lane == 0) raise(prm, ss, ST_TIMEOUT_META); break; }
                    }
                    const int n = (int)min(wk.seg_e - t0, (int64_t)(MMAS_PER_STAGE - stage_k) * 2);    // tiles placed now
                    const int ks = (n + 1) >> 1;
                    uint8_t *dst = ring_m + (size_t)slot * META_BYTES;
                    const uint32_t bar = smem_u32(&ss->full_m[slot]);
                    if (n & 1) {        // the segment ends on a first tile: the K-step's second tile multiplies as zeros
                        if (lane < 16)
                            *reinterpret_cast<uint4 *>(dst + (size_t)(stage_k * 2 + n) * TILE_BYTES + lane * 16) = make_uint4(0u, 0u, 0u, 0u);
                        fence_async_smem();
                        __syncwarp();
                    }
                    // flags: the piece's first K-step opens the segment, its last one may close it
                    cmdw |= (first ? KS_FIRST : 0u) << (4 + 3 * stage_k);
                    cmdw |= ((t0 + n == wk.seg_e ? KS_LAST : 0u) | ((n & 1) ? KS_SINGLE : 0u)) << (4 + 3 * (stage_k + ks - 1));
                    const bool full = stage_k + ks == MMAS_PER_STAGE;
                    if (elect_one()) {
                        if (!(prm.skip & 8)) {
                            mbar_expect_tx_only(bar, (uint32_t)n * (TILE_BYTES + TILE_COLS * 4));
                            bulk_g2s(smem_u32(dst + (size_t)stage_k * 2 * TILE_BYTES), static_cast<const uint8_t *>(prm.vals) + t0 * TILE_BYTES,
                                     (uint32_t)n * TILE_BYTES, bar, pol);
                            bulk_g2s(smem_u32(dst + META_TILE_BYTES + (size_t)stage_k * 2 * TILE_COLS * 4), prm.cols + t0 * TILE_COLS,
                                     (uint32_t)n * TILE_COLS * 4, bar, pol);
                        }
                        if (full) {                                // publish the stage
                            *reinterpret_cast<volatile uint32_t *>(dst + META_TILE_BYTES + META_COL_BYTES) = (uint32_t)MMAS_PER_STAGE | cmdw;
                            mbar_arrive(bar);                      // release: publishes the command
                            prof_mark<PROF>(prm.dbg, it, 0);
                        }
                    }
                    stage_k += ks;
                    t0 += n;
                    first = false;
                    if (full) {
                        ++it;
                        stage_k = 0;
                        cmdw = 0;
                    }
                }
            }
            if (ok && stage_k > 0) {                               // the last, partly filled stage
                __syncwarp();
                if (elect_one()) {
                    *reinterpret_cast<volatile uint32_t *>(ring_m + (size_t)slot * META_BYTES + META_TILE_BYTES + META_COL_BYTES) = (uint32_t)stage_k | cmdw;
                    mbar_arrive(smem_u32(&ss->full_m[slot]));
                }
                ++it;
            }
#else
            while (ok && wk.next_segment(lane)) {
                for (int64_t t0 = wk.seg_s; ok && t0 < wk.seg_e; t0 += STAGE_TILES, ++it) {
                    if (it % NUM_META_WARPS != meta_id) continue;      // another meta warp's stage
                    const uint32_t slot = it % C::kMeta, ph = (it / C::kMeta) & 1u;
                    const int ntiles = (int)min((int64_t)STAGE_TILES, wk.seg_e - t0);
                    if (lane == 0) ok = mbar_wait_t<PROF>(smem_u32(&ss->empty_m[slot]), ph ^ 1u, abort_flag, w_empty_m, 5);
                    ok = __shfl_sync(0xffffffffu, ok ? 1 : 0, 0) != 0;
                    if (ok && (ntiles & 1)) {
                        // an odd tile count leaves the second tile of the last K-step without data:
                        // zero it (the MMA multiplies it with zero rows, which must not meet NaNs)
                        if (lane < 16)
                            *reinterpret_cast<uint4 *>(ring_m + (size_t)slot * META_BYTES + (size_t)ntiles * TILE_BYTES + lane * 16) = make_uint4(0u, 0u, 0u, 0u);
                        fence_async_smem();
                        __syncwarp();
                    }
                    __syncwarp();
                    if (elect_one()) {
                        if (ok) {
                            const uint32_t bar = smem_u32(&ss->full_m[slot]);
                            uint8_t *dst = ring_m + (size_t)slot * META_BYTES;
                            *reinterpret_cast<volatile uint32_t *>(dst + META_TILE_BYTES + META_COL_BYTES) =
                                (uint32_t)ntiles | (t0 == wk.seg_s ? CMD_FIRST : 0u) | (t0 + STAGE_TILES >= wk.seg_e ? CMD_LAST : 0u);
                            if (prm.skip & 8) {
                                mbar_arrive(bar);
                            } else {
                            mbar_expect_tx(bar, (uint32_t)ntiles * (TILE_BYTES + TILE_COLS * 4));   // release: publishes the command
                            bulk_g2s(smem_u32(dst), static_cast<const uint8_t *>(prm.vals) + t0 * TILE_BYTES,
                                     (uint32_t)ntiles * TILE_BYTES, bar, pol);
                            bulk_g2s(smem_u32(dst + META_TILE_BYTES), prm.cols + t0 * TILE_COLS,
                                     (uint32_t)ntiles * TILE_COLS * 4, bar, pol);
                            }
                            prof_mark<PROF>(prm.dbg, it, 0);
                        } else {
                            raise(prm, ss, ST_TIMEOUT_META);
                        }
                    }
                    ok = __shfl_sync(0xffffffffu, ok ? 1 : 0, 0) != 0;
                }
            }
#endif
            if (lane == 0 && meta_id == 0) {   // one end marker per gather slot; the MMA warp stops at the first
                for (int j = 0; ok && j < C::kStages; ++j, ++it) {
                    const uint32_t slot = it % C::kMeta, ph = (it / C::kMeta) & 1u;
                    ok = mbar_wait_t<PROF>(smem_u32(&ss->empty_m[slot]), ph ^ 1u, abort_flag, w_empty_m);
                    if (ok) {
                        *reinterpret_cast<volatile uint32_t *>(ring_m + (size_t)slot * META_BYTES + META_TILE_BYTES + META_COL_BYTES) = CMD_END;
                        mbar_arrive(smem_u32(&ss->full_m[slot]));
                    } else {
                        raise(prm, ss, ST_TIMEOUT_META);
                    }
                }
            }
            if (PROF && prm.dbg && lane == 0 && meta_id == 0) { prm.dbg[blockIdx.x * 16 + 0] = w_empty_m; prm.dbg[blockIdx.x * 16 + 1] = prof_clock<PROF>() - t_start; }
        } else {
            // -------------------------------------------------------------- epilogue warps
            const uint64_t pol = policy_stream();
            const int q = warp & 3;                        // TMEM lane quarter this warp may read
            uint32_t ai = 0;
            bool ok = true;
            long long w_af = 0;
            // Windows without tiles produce zero rows.  They are dealt to all CTAs here, while the
            // pipeline fills, instead of being written by whichever CTA's tile range they border:
            // a run of empty windows (padded blocks, isolated nodes) would serialise on that one CTA.
            if (!(prm.skip & 4)) zero_fill_empty_windows<NH>(prm.window_offset, prm.C, prm.ldc, prm.c_dtype, W, q, lane);
            while (ok && wk.next_segment(lane)) {
                const int64_t w = wk.window();
                const bool nonempty = wk.seg_e > wk.seg_s;
                if (!nonempty) continue;                   // zero rows were written above
                uint32_t v[NH][16];
                if (nonempty) {
                    const uint32_t buf = ai % NACC, aph = (ai / NACC) & 1u;
                    ++ai;
                    // one polling lane per warp: threads spinning on a barrier slow every other
                    // barrier operation of the SM down
                    if (lane == 0) ok = mbar_wait_t<PROF>(smem_u32(&ss->acc_full[buf]), aph, abort_flag, w_af, 4);
                    ok = __shfl_sync(0xffffffffu, ok ? 1 : 0, 0) != 0;
                    if (!ok) { if (lane == 0) raise(prm, ss, ST_TIMEOUT_ACC); break; }
                    tc_fence_after();
#pragma unroll
                    for (int h = 0; h < NH; ++h)
                        tmem_ld16(tmem_base + ((uint32_t)(32 * q) << 16) + buf * C::kAccCols + h * 16, v[h]);
                    tmem_ld_wait();
                    tc_fence_before();
                    __syncwarp();
                    if (lane == 0) mbar_arrive(smem_u32(&ss->acc_empty[buf]));
                } else {
#pragma unroll
                    for (int h = 0; h < NH; ++h)
#pragma unroll
                        for (int r = 0; r < 16; ++r) v[h][r] = 0u;
                }
                const bool partial = wk.head() || wk.tail();
#pragma unroll
                for (int h = 0; h < NH; ++h) {
                    const int64_t f = h * SLAB + 32 * q + lane;
                    if (prm.skip & 4) {
                    } else if (!partial) {
                        const int64_t base = (w * TILE_ROWS) * prm.ldc + f;
#pragma unroll
                        for (int r = 0; r < 16; ++r) {
                            const float x = __uint_as_float(v[h][r]);
                            const int64_t o = base + r * prm.ldc;
                            if (prm.c_dtype == GRWS_F32) {
                                asm volatile("st.global.L2::cache_hint.f32 [%0], %1, %2;" ::"l"(static_cast<float *>(prm.C) + o), "f"(x), "l"(pol) : "memory");
                            } else {
                                const uint16_t hbits = prm.c_dtype == GRWS_F16 ? __half_as_ushort(__float2half_rn(x))
                                                                               : __bfloat16_as_ushort(__float2bfloat16_rn(x));
                                asm volatile("st.global.L2::cache_hint.u16 [%0], %1, %2;" ::"l"(static_cast<uint16_t *>(prm.C) + o), "h"(hbits), "l"(pol) : "memory");
                            }
                        }
                    } else {
                        float *slot = prm.partial + (2 * (int64_t)blockIdx.x + (wk.tail() ? 1 : 0)) * (TILE_ROWS * prm.N);
#pragma unroll
                        for (int r = 0; r < 16; ++r) slot[(int64_t)r * prm.N + f] = __uint_as_float(v[h][r]);
                    }
                }
                if (partial && !(prm.skip & 4)) {
                    // A window cut between CTAs: every holder of a piece counts itself on the counter of
                    // the CTA that holds the window's first tile, and the one that arrives last sums the
                    // pieces in CTA order (the same order whoever is last) and writes the rows.  Cuts
                    // inside a split window are never moved, so its pieces are exactly the CTAs
                    // a / chunk .. (b - 1) / chunk.
                    __threadfence();
                    asm volatile("bar.sync 1, 128;" ::: "memory");
                    const int64_t k0 = wk.a / chunk, k_last = (wk.b - 1) / chunk;
                    if (threadIdx.x == 0) {
                        const int old = atomicAdd(prm.split_count + k0, 1);
                        ss->last_piece = (old == (int)(k_last - k0)) ? 1 : 0;
                    }
                    asm volatile("bar.sync 1, 128;" ::: "memory");
                    if (*reinterpret_cast<volatile int *>(&ss->last_piece)) sum_pieces<NH>(prm.partial, prm.N, prm.C, prm.ldc, prm.c_dtype, w, k0, k_last, q, lane);
                }
            }
            if (PROF && prm.dbg && threadIdx.x == EPILOGUE_WARP0 * 32) prm.dbg[blockIdx.x * 16 + 7] = w_af;
        }
    } else if (warp >= PRODUCER_WARP0) {
        // ------------------------------------------------------------------ gather producers
        // Producer warps k*w .. k*w+k-1 own ring slot w (k = 1 by default) and fill every kStages-th
        // stage, so the barrier polls and column-id reads of kStages stages overlap.  The rows are
        // fetched by the TMA unit (tile::gather4: four consecutive slots x 64 features per copy,
        // 32 copies per stage and slab), all issued by one elected lane in an unrolled loop: a copy
        // issued per lane costs its warp ~220 cycles (the copies of different lanes go one after
        // the other and each marshals its operands into uniform registers), a copy from the elected
        // lane with warp-uniform operands ~70.  The copies complete on the stage's barrier.
        constexpr int WARPS_PER_SLOT = NUM_PRODUCER_WARPS / Cfg<NH>::kStages;
        constexpr int STAGE_OPS = MMAS_PER_STAGE * 8;                          // gather4 copies per stage and slab
        static_assert(WARPS_PER_SLOT >= 1 && WARPS_PER_SLOT * Cfg<NH>::kStages == NUM_PRODUCER_WARPS, "producer warps per slot");
        const uint64_t keep = policy_keep();
        const int pwarp = warp - PRODUCER_WARP0;
        const int member = pwarp % WARPS_PER_SLOT;            // the copies of a stage are dealt round-robin to the slot's warps
        long long w_full_m = 0, w_empty_g = 0;
        const uint32_t gs = (uint32_t)(pwarp / WARPS_PER_SLOT);
        const uint32_t full_bar = smem_u32(&ss->full_g[gs]), empty_bar = smem_u32(&ss->empty_g[gs]);
        const uint32_t dst_slot = smem_u32(ring_g + (size_t)gs * C::kStageBytes);
        uint32_t gph = 0;
        for (uint32_t it = gs;; it += C::kStages, gph ^= 1u) {
            const uint32_t ms = it % C::kMeta, mph = (it / C::kMeta) & 1u;
            // column ids and the command have landed
            bool ok = true;
            if (lane == 0) ok = mbar_wait_t<PROF>(smem_u32(&ss->full_m[ms]), mph, abort_flag, w_full_m, 3);
            ok = __shfl_sync(0xffffffffu, ok ? 1 : 0, 0) != 0;
            if (!ok) { if (lane == 0) raise(prm, ss, ST_TIMEOUT_META); break; }
            if (lane == 0) prof_mark<PROF>(prm.dbg, it, 1);
            const uint8_t *meta = ring_m + (size_t)ms * META_BYTES;
            const uint32_t cmd = *reinterpret_cast<const volatile uint32_t *>(meta + META_TILE_BYTES + META_COL_BYTES);
            const bool end = (cmd & CMD_END) != 0;
#if GRWS_TC5_SPAN
            const int nmma = end ? 0 : (int)(cmd & CMD_COUNT);   // K-steps of the stage
#else
            const int ntiles = end ? 0 : (int)(cmd & CMD_COUNT);
            const int nvalid = ntiles * TILE_COLS;               // slots that carry a column id
            const int nmma = (ntiles + 1) >> 1;
#endif
            // the gather slot has been released by the MMA warp (it finished stage it - kStages)
            if (lane == 0) ok = mbar_wait_t<PROF>(empty_bar, gph ^ 1u, abort_flag, w_empty_g, 2);
            ok = __shfl_sync(0xffffffffu, ok ? 1 : 0, 0) != 0;
            if (!ok) { if (lane == 0) raise(prm, ss, ST_TIMEOUT_EMPTY); break; }
            if (lane == 0) prof_mark<PROF>(prm.dbg, it, 2);
            // ... which also frees the tile / column slot of that older stage for the TMA warp
            if (lane == 0 && member == 0 && it >= (uint32_t)C::kStages) mbar_arrive(smem_u32(&ss->empty_m[(it - C::kStages) % C::kMeta]));
            if (end) {                      // pass the end marker on to the MMA warp
                if (lane == 0 && member == 0) mbar_arrive(full_bar);
                break;
            }
            // bytes the K-steps of this stage bring in: 16 slots x 128 features x NH slabs each
            if (lane == 0 && member == 0) {
                if (prm.skip & 2) mbar_arrive(full_bar);          // experiment: no gathers, nothing to wait for
                else mbar_expect_tx(full_bar, (uint32_t)(nmma * 16 * SLAB * 2 * NH));
            }
            // (K-step om, slot group og, feature half oh) of copy o: slots 4*og .. 4*og+3 of K-step om
            // land in slot half og / 2, lines (4*og) % 8 .. +3 of the atom; slots past the last tile
            // carry no column id and fetch row -1, which is out of bounds and reads zeros
            __syncwarp();
            if (elect_one() && !(prm.skip & 2)) {
                constexpr int MAX_OPS = (STAGE_OPS + WARPS_PER_SLOT - 1) / WARPS_PER_SLOT;
#pragma unroll
                for (int j = 0; j < MAX_OPS; ++j) {
                    const int o = member + j * WARPS_PER_SLOT;
                    const int om = o >> 3, og = (o >> 1) & 3, oh = o & 1;
                    if (o < STAGE_OPS && om < nmma) {
                        const int s0 = 16 * om + 4 * og;
                        int4 r = *reinterpret_cast<const int4 *>(meta + META_TILE_BYTES + s0 * 4);
#if GRWS_TC5_SPAN
                        if ((kstep_flags(cmd, om) & KS_SINGLE) && og >= 2) r = make_int4(-1, -1, -1, -1);
#else
                        if (s0 >= nvalid) r = make_int4(-1, -1, -1, -1);
#endif
                        const uint32_t off = (uint32_t)(om * NH * A_MMA_BYTES + (og >> 1) * A_SBO + oh * A_LBO + ((4 * og) & 7) * 128);
#pragma unroll
                        for (int h = 0; h < NH; ++h)
                            tma_gather4(dst_slot + off + (uint32_t)(h * A_MMA_BYTES), &b_map, full_bar, h * SLAB + oh * 64, r.x, r.y, r.z, r.w, keep);
                    }
                }
            }
            __syncwarp();
            if (lane == 0) prof_mark<PROF>(prm.dbg, it, 3);
        }
        if (PROF && prm.dbg && threadIdx.x == PRODUCER_WARP0 * 32) { prm.dbg[blockIdx.x * 16 + 2] = w_full_m; prm.dbg[blockIdx.x * 16 + 3] = w_empty_g; }
    } else if (warp == MMA_WARP) {
        // ------------------------------------------------------------------ MMA issuer (one thread)
        if (elect_one()) {
            const uint32_t idesc = (1u << 4) | ((uint32_t)prm.is_bf16 << 7) | ((uint32_t)prm.is_bf16 << 10) |
                                   (1u << 15) | ((16u >> 3) << 17) | ((128u >> 4) << 24);
            // descriptors of stage 0 / meta slot 0; other stages add their byte offset >> 4 to the low word
            const uint64_t a_desc0 = smem_desc(smem_u32(ring_g), A_LBO, A_SBO, 2);
            const uint64_t b_desc0 = smem_desc(smem_u32(ring_m), TILE_BYTES, 128, 0);
            uint32_t ai = 0, buf = 0;
            long long w_acc = 0, w_fm = 0, w_fg = 0, t_issue = 0, t_commit = 0, t_cmd = 0, t_fence = 0;
            const long long t_mark = prof_clock<PROF>();
            uint32_t it = 0, gs = 0, gph = 0, ms = 0;
            for (;; ++it) {
                // The producers arrive on full_g only after they have seen full_m of the same stage,
                // so this one wait also covers the tile values and the command word.
                if (!mbar_wait_t<PROF>(smem_u32(&ss->full_g[gs]), gph, abort_flag, w_fg, 1)) { raise(prm, ss, ST_TIMEOUT_FULL); break; }
                prof_mark<PROF>(prm.dbg, it, 5);
                const long long tc0 = prof_clock<PROF>();
                const uint32_t cmd = *reinterpret_cast<const volatile uint32_t *>(ring_m + ms * META_BYTES + META_TILE_BYTES + META_COL_BYTES);
                if (cmd & CMD_END) break;
                if (PROF) t_cmd += prof_clock<PROF>() - tc0 + (long long)(cmd & 0);
#if GRWS_TC5_SPAN
                const int nmma = (int)(cmd & CMD_COUNT);
                const long long tf0 = prof_clock<PROF>();
                tc_fence_after();
                const long long ti0 = prof_clock<PROF>();
                t_fence += ti0 - tf0;
                const uint64_t ad = a_desc0 + (uint64_t)(gs * (C::kStageBytes >> 4));
                const uint64_t bd = b_desc0 + (uint64_t)(ms * (META_BYTES >> 4));
                // first pass: take the accumulator buffers of the segments that start in this stage
                // (at most four, and the buffer of the fourth was released by a segment that ended in an
                // earlier stage, so waiting for all of them up front cannot block on this stage's own
                // MMAs); second pass: the MMAs and commits as one straight-line sequence
                bool alive = true;
                uint32_t dt[MMAS_PER_STAGE], kbuf[MMAS_PER_STAGE];
#pragma unroll
                for (int m = 0; m < MMAS_PER_STAGE; ++m) {
                    if (m < nmma && alive && (kstep_flags(cmd, m) & KS_FIRST)) {
                        buf = ai % NACC;
                        const uint32_t aph = (ai / NACC) & 1u;
                        ++ai;
                        if (!mbar_wait_t<PROF>(smem_u32(&ss->acc_empty[buf]), aph ^ 1u, abort_flag, w_acc)) { raise(prm, ss, ST_TIMEOUT_ACC); alive = false; }
                    }
                    kbuf[m] = buf;
                    dt[m] = tmem_base + buf * C::kAccCols;
                }
                if (!alive) break;
                tc_fence_after();
#pragma unroll
                for (int m = 0; m < MMAS_PER_STAGE; ++m) {
                    if (m < nmma) {
                        const uint32_t f = kstep_flags(cmd, m);
                        if (!(prm.skip & 1)) {
#pragma unroll
                            for (int h = 0; h < NH; ++h)
                                umma_f16(dt[m] + h * 16, ad + (uint64_t)(((m * NH + h) * A_MMA_BYTES) >> 4),
                                         bd + (uint64_t)((m * 2 * TILE_BYTES) >> 4), idesc, (f & KS_FIRST) ? 0u : 1u);
                        }
                        if (f & KS_LAST) umma_commit(smem_u32(&ss->acc_full[kbuf[m]]));
                    }
                }
#else
                const int nmma = (int)((cmd & CMD_COUNT) + 1u) >> 1;
                if (cmd & CMD_FIRST) {
                    buf = ai % NACC;
                    const uint32_t aph = (ai / NACC) & 1u;
                    ++ai;
                    if (!mbar_wait_t<PROF>(smem_u32(&ss->acc_empty[buf]), aph ^ 1u, abort_flag, w_acc)) { raise(prm, ss, ST_TIMEOUT_ACC); break; }
                }
                // cp.async data is handed over by the mbarrier the producers arrive on after their
                // copies have landed; no generic->async proxy fence is issued here (it would also
                // wait for every younger gather in flight)
                const long long tf0 = prof_clock<PROF>();
                tc_fence_after();
                const long long ti0 = prof_clock<PROF>();
                t_fence += ti0 - tf0;
                const uint32_t d_tmem = tmem_base + buf * C::kAccCols;
                const uint64_t ad = a_desc0 + (uint64_t)(gs * (C::kStageBytes >> 4));
                const uint64_t bd = b_desc0 + (uint64_t)(ms * (META_BYTES >> 4));
                const uint32_t first = (cmd & CMD_FIRST) ? 0u : 1u;
#pragma unroll
                for (int m = 0; m < MMAS_PER_STAGE; ++m) {
                    if (m < nmma && !(prm.skip & 1)) {
#pragma unroll
                        for (int h = 0; h < NH; ++h)
                            umma_f16(d_tmem + h * 16, ad + (uint64_t)(((m * NH + h) * A_MMA_BYTES) >> 4),
                                     bd + (uint64_t)((m * 2 * TILE_BYTES) >> 4), idesc, m > 0 ? 1u : first);
                    }
                }
#endif
                const long long ti1 = prof_clock<PROF>();
                umma_commit(smem_u32(&ss->empty_g[gs]));
#if !GRWS_TC5_SPAN
                if (cmd & CMD_LAST) umma_commit(smem_u32(&ss->acc_full[buf]));
#endif
                const long long ti2 = prof_clock<PROF>();
                t_issue += ti1 - ti0;
                t_commit += ti2 - ti1;
                prof_mark<PROF>(prm.dbg, it, 6);
                if (++gs == (uint32_t)C::kStages) { gs = 0; gph ^= 1u; }
                if (++ms == (uint32_t)C::kMeta) ms = 0;
            }
            if (PROF && prm.dbg) {
                long long *d = prm.dbg + blockIdx.x * 16;
                d[4] = w_acc; d[5] = w_fm; d[6] = w_fg; d[8] = t_issue; d[9] = t_commit; d[10] = prof_clock<PROF>() - t_mark; d[11] = it; d[12] = t_cmd; d[13] = t_fence;
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
}

static int grid_size() {
    static const int sms = [] {
        int dev = 0, n = 0;
        if (cudaGetDevice(&dev) != cudaSuccess) return 148;
        if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) return 148;
        return n;
    }();
    return sms;
}

constexpr size_t STATUS_BYTES = 256;
constexpr size_t DEBUG_BYTES = 1024 * 16 * sizeof(long long);
constexpr size_t FIX_BYTES = 1024 * 4 * sizeof(int64_t);      // per-CTA counters of finished pieces of split windows

static bool profile_waits() {
    static const int v = [] { const char *e = getenv("GRWS_TC5_PROFILE"); return e ? atoi(e) : 0; }();
    return v != 0;
}

}  // namespace tc5

namespace tc5 {
template <int NH>
static cudaError_t launch_kernel(const Params &prm, const CUtensorMap &b_map, int G, cudaStream_t stream) {
    static const cudaError_t attr = [] {
        cudaError_t e = cudaFuncSetAttribute(spmm_tc5_kernel<NH, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)Cfg<NH>::kSmem);
        if (e != cudaSuccess) return e;
        return cudaFuncSetAttribute(spmm_tc5_kernel<NH, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)Cfg<NH>::kSmem);
    }();
    if (attr != cudaSuccess) return attr;
    if (prm.dbg) spmm_tc5_kernel<NH, true><<<G, NUM_THREADS, Cfg<NH>::kSmem, stream>>>(prm, b_map);
    else spmm_tc5_kernel<NH, false><<<G, NUM_THREADS, Cfg<NH>::kSmem, stream>>>(prm, b_map);
    return cudaSuccess;
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
    const cuuint64_t dims[2] = {(cuuint64_t)N, (cuuint64_t)(K > 0 ? K : 1)};
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
}  // namespace tc5

bool spmm_tc5_supported(int dtype, int64_t N) {
    static const int disabled = [] { const char *e = getenv("GRWS_DISABLE_TCGEN05"); return e ? atoi(e) : 0; }();
    return !disabled && (dtype == GRWS_F16 || dtype == GRWS_BF16) && (N == 128 || N == 256);
}

size_t spmm_tc5_scratch_bytes(int64_t num_tiles_bound, int64_t N) {
    (void)num_tiles_bound;
    return tc5::STATUS_BYTES + tc5::DEBUG_BYTES + tc5::FIX_BYTES + (size_t)tc5::grid_size() * 4 /* CTAs per SM, at most */ * 2 * TILE_ROWS * (size_t)N * sizeof(float);
}

int spmm_tc5_launch(const int64_t *window_offset, const int32_t *cols, const void *vals, int dtype,
                    const void *B, int64_t ldb, void *C, int c_dtype, int64_t ldc, int64_t W,
                    int64_t num_tiles_bound, int64_t K, int64_t N, void *scratch, size_t scratch_bytes,
                    cudaStream_t stream) {
    using namespace tc5;
    const size_t need = spmm_tc5_scratch_bytes(num_tiles_bound, N);
    if (scratch_bytes < need || scratch == nullptr)
        return fail(GRWS_ERR_SCRATCH, "spmm scratch too small: %zu < %zu bytes", scratch_bytes, need);
    Params prm;
    prm.window_offset = window_offset; prm.cols = cols; prm.vals = vals; prm.B = B; prm.C = C;
    prm.status = static_cast<int *>(scratch);
    { static const int sk = [] { const char *e = getenv("GRWS_TC5_SKIP"); return e ? atoi(e) : 0; }(); prm.skip = sk; }
    { static const int lw = [] { const char *e = getenv("GRWS_TC5_LW_SHIFT"); return e ? atoi(e) : 4; }(); prm.lw_shift = lw; }
    // layout: status word | split-window counters | profiling counters | partial tiles; the first two are zeroed together
    prm.dbg = profile_waits() ? reinterpret_cast<long long *>(static_cast<char *>(scratch) + STATUS_BYTES + FIX_BYTES) : nullptr;
    prm.split_count = reinterpret_cast<int *>(static_cast<char *>(scratch) + STATUS_BYTES);
    prm.partial = reinterpret_cast<float *>(static_cast<char *>(scratch) + STATUS_BYTES + DEBUG_BYTES + FIX_BYTES);
    prm.W = W; prm.N = N; prm.ldb = ldb; prm.ldc = ldc; prm.c_dtype = c_dtype;
    prm.is_bf16 = dtype == GRWS_BF16 ? 1 : 0;
    // Width 256: one pass with two slabs per stage (one CTA per SM), or two passes of 128 columns.
    // Two passes read the tiles twice but gather from half as many bytes of the dense operand,
    // which then stays in L2 next to the tile stream, and they run two CTAs per SM: measured 4 %
    // faster at 86 MB of operand, 20 % at 119 MB.  Small operands keep the single pass (half the
    // launches).  GRWS_TC5_SPLIT256 = 0 / 1 forces one way.
    static const int split_env = [] { const char *e = getenv("GRWS_TC5_SPLIT256"); return e ? atoi(e) : -1; }();
    const bool split = N == 256 && (split_env >= 0 ? split_env != 0 : K * 512 > SPLIT256_OPERAND_BYTES);
    const int64_t pass_n = (N == 128 || split) ? 128 : 256;
    const int G = grid_size() * (pass_n == 128 ? Cfg<1>::kCtasPerSm : Cfg<2>::kCtasPerSm);
    const size_t c_elem = c_dtype == GRWS_F32 ? 4 : 2;
    for (int64_t col0 = 0; col0 < N; col0 += pass_n) {
        prm.B = static_cast<const char *>(B) + col0 * 2;
        prm.C = static_cast<char *>(C) + col0 * c_elem;
        prm.N = pass_n;
        alignas(64) CUtensorMap b_map;
        if (int st = encode_b_map(&b_map, prm.B, prm.is_bf16, K, pass_n, ldb)) return st;
        // the status word is cleared once per call, the split-window counters before every pass
        if (col0 == 0) GRWS_CUDA_TRY(cudaMemsetAsync(scratch, 0, STATUS_BYTES + sizeof(int) * (size_t)G, stream));
        else GRWS_CUDA_TRY(cudaMemsetAsync(prm.split_count, 0, sizeof(int) * (size_t)G, stream));
        GRWS_CUDA_TRY((pass_n == 128 ? launch_kernel<1>(prm, b_map, G, stream) : launch_kernel<2>(prm, b_map, G, stream)));
        GRWS_CUDA_TRY(cudaGetLastError());
    }
    if (prm.dbg) {      // profiling build: failed try_waits per role since the last call, behind the timeline
        GRWS_CUDA_TRY(cudaMemcpyFromSymbolAsync(prm.dbg + 12288 + 64 * 8, g_prof_tries, sizeof(g_prof_tries), 0, cudaMemcpyDeviceToDevice, stream));
        static const unsigned long long zeros[8] = {0, 0, 0, 0, 0, 0, 0, 0};
        GRWS_CUDA_TRY(cudaMemcpyToSymbolAsync(g_prof_tries, zeros, sizeof(zeros), 0, cudaMemcpyHostToDevice, stream));
    }
    return GRWS_OK;
}

}  // namespace grws

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
//   * No cudaMalloc, cudaFree or allocating library routine is called.
// ---------------------------------------------------------------------------------------------
namespace grws {
namespace tc5 {

constexpr int STATIC_MAX_SMS = 160;
constexpr int STATIC_MAX_N = 256;
constexpr size_t STATIC_SCRATCH_BYTES =
    STATUS_BYTES + DEBUG_BYTES + FIX_BYTES + (size_t)STATIC_MAX_SMS * 4 * 2 * TILE_ROWS * STATIC_MAX_N * sizeof(float);
static_assert(STATIC_SCRATCH_BYTES == GRWS_SPMM_STATIC_SCRATCH_BYTES, "the header states the size of the built-in scratch");

static __device__ __align__(256) unsigned char static_scratch[STATIC_SCRATCH_BYTES];

// device address of static_scratch on the current device (looked up once per device)
static int static_scratch_address(void **out) {
    constexpr int MAX_DEVICES = 64;
    static void *cached[MAX_DEVICES] = {nullptr};
    int dev = 0;
    GRWS_CUDA_TRY(cudaGetDevice(&dev));
    if (dev < 0 || dev >= MAX_DEVICES) return fail(GRWS_ERR_UNSUPPORTED, "device ordinal %d beyond %d", dev, MAX_DEVICES);
    void *p = __atomic_load_n(&cached[dev], __ATOMIC_ACQUIRE);
    if (p == nullptr) {
        GRWS_CUDA_TRY(cudaGetSymbolAddress(&p, static_scratch));
        if (p == nullptr) return fail(GRWS_ERR_CUDA, "cudaGetSymbolAddress returned a null address");
        __atomic_store_n(&cached[dev], p, __ATOMIC_RELEASE);      // every thread resolves the same address
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
    GRWS_REQUIRE(window_offset && C && (num_tiles_bound == 0 || (cols && vals && B)), "null pointer");
    GRWS_REQUIRE(c_dtype >= GRWS_F32 && c_dtype <= GRWS_BF16, "bad output dtype %d", c_dtype);
    if (val_dtype != b_dtype || !(val_dtype == GRWS_F16 || val_dtype == GRWS_BF16) || !(N == 128 || N == 256))
        return fail(GRWS_ERR_UNSUPPORTED,
                    "the allocation-free SpMM covers fp16/bf16 operands with N = 128 or 256 (got dtypes %d/%d, N = %lld); "
                    "other shapes need grws_spmm_fwd with caller scratch", val_dtype, b_dtype, (long long)N);
    GRWS_REQUIRE(ldb >= N && ldc >= N, "leading dimension smaller than N");
    GRWS_REQUIRE((ldb * 2) % 16 == 0 && (ldc * dtype_bytes(c_dtype)) % 16 == 0, "rows of B and C must be 16-byte aligned");
    GRWS_REQUIRE(aligned16(B) && aligned16(C) && aligned16(vals) && aligned16(cols), "B, C, values and column ids must be 16-byte aligned");
    const size_t need = spmm_tc5_scratch_bytes(num_tiles_bound, N);
    if (need > tc5::STATIC_SCRATCH_BYTES)
        return fail(GRWS_ERR_SCRATCH, "this device needs %zu bytes of SpMM scratch, the built-in array holds %zu "
                    "(more than %d SMs?); use grws_spmm_fwd with caller scratch", need, tc5::STATIC_SCRATCH_BYTES, tc5::STATIC_MAX_SMS);
    void *scratch = nullptr;
    if (int st = tc5::static_scratch_address(&scratch)) return st;
    return spmm_tc5_launch(window_offset, cols, vals, val_dtype, B, ldb, C, c_dtype, ldc, num_windows, num_tiles_bound,
                           K, N, scratch, tc5::STATIC_SCRATCH_BYTES, static_cast<cudaStream_t>(stream));
}
