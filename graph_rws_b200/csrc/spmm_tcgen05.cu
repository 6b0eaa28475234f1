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
//   * the A operand is the gathered rows of the dense matrix, MN-major: each 16-byte piece of a
//     gathered row is written to its core-matrix slot by cp.async (L2 -> shared memory, no
//     registers), rows whose column id is -1 are zero-filled;
//   * accumulators live in tensor memory (16 fp32 columns per slab), four deep, so the epilogue
//     of one window overlaps the MMAs of the next.
//
// One persistent CTA per SM owns a contiguous range of the global tile array (equal tile counts,
// so power-law window lengths do not matter); a window cut by a range boundary is finished by the
// fix-up kernel from fp32 partial tiles in scratch, in a fixed order.
//
// Warp roles: 0-3 gather producers, 4-7 epilogue (TMEM -> registers -> global), 8 MMA issuer,
// 9 TMA producer for tile values and column ids.  Every mbarrier wait is bounded: on time-out the
// kernel raises the status word at the start of scratch and all roles drain and return.
#include <stdlib.h>

#include "grws_common.cuh"

namespace grws {

namespace tc5 {

constexpr int STAGE_TILES = 8;                       // tiles per pipeline stage (4 MMA K-steps)
constexpr int STAGE_SLOTS = STAGE_TILES * TILE_COLS; // gathered rows per stage
constexpr int MMAS_PER_STAGE = STAGE_TILES / 2;
constexpr int SLAB = 128;                            // features per MMA (its M dimension)
constexpr int CHUNKS = SLAB * 2 / 16;                // 16-byte pieces of a 128-feature row
constexpr int A_SBO = 272;                           // bytes between 8-feature core-matrix columns (odd
                                                     // multiple of 16: conflict-free cp.async writes)
constexpr int A_LBO = 128;                           // bytes between the two 8-slot halves of a K-step
constexpr int A_MMA_BYTES = CHUNKS * A_SBO;          // one K-step of one slab
constexpr int TILE_BYTES = TILE_ELEMS * 2;           // 256
constexpr int META_TILE_BYTES = STAGE_TILES * TILE_BYTES;
constexpr int META_COL_BYTES = STAGE_TILES * TILE_COLS * 4;
constexpr int META_BYTES = META_TILE_BYTES + META_COL_BYTES;
constexpr int NACC = 4;                              // accumulator buffers in tensor memory
constexpr int NUM_PRODUCERS = 128;
constexpr int NUM_EPILOGUE = 128;
constexpr int NUM_THREADS = 320;
constexpr uint64_t WAIT_LIMIT_NS = 2000000000ull;    // a wait gives up after two seconds

enum : int { ST_OK = 0, ST_TIMEOUT_FULL = 1, ST_TIMEOUT_EMPTY = 2, ST_TIMEOUT_ACC = 3, ST_TIMEOUT_META = 4 };

struct Params {
    const int64_t *window_offset;
    const int32_t *cols;
    const void *vals;
    const void *B;
    void *C;
    float *partial;
    int *status;
    int64_t W, N, ldb, ldc;
    int c_dtype;
    int is_bf16;
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
    asm volatile("{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}"
                 : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
    return ok;
}
__device__ __forceinline__ uint64_t global_ns() {
    uint64_t t;
    asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
    return t;
}
// bounded wait: gives up after WAIT_LIMIT_NS or when another role already aborted
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile int *abort_flag) {
    if (mbar_try_wait(bar, parity)) return true;
    const uint64_t t0 = global_ns();
    for (uint32_t i = 0;; ++i) {
        if (mbar_try_wait(bar, parity)) return true;
        if ((i & 31u) == 31u) {
            if (*abort_flag) return false;
            if (global_ns() - t0 > WAIT_LIMIT_NS) return false;
        }
    }
}
__device__ __forceinline__ void cp_async16(uint32_t dst, const void *src, uint32_t src_bytes, uint64_t pol) {
    asm volatile("cp.async.cg.shared.global.L2::cache_hint [%0], [%1], 16, %2, %3;"
                 ::"r"(dst), "l"(src), "r"(src_bytes), "l"(pol) : "memory");
}
__device__ __forceinline__ void cp_async_arrive_noinc(uint32_t bar) {
    asm volatile("cp.async.mbarrier.arrive.noinc.shared::cta.b64 [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void cp_async_wait_all() { asm volatile("cp.async.wait_all;" ::: "memory"); }
__device__ __forceinline__ void bulk_g2s(uint32_t dst, const void *src, uint32_t bytes, uint32_t bar, uint64_t pol) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes.L2::cache_hint [%0], [%1], %2, [%3], %4;"
                 ::"r"(dst), "l"(src), "r"(bytes), "r"(bar), "l"(pol) : "memory");
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

// shared-memory matrix descriptor, no swizzle (layout type 0), descriptor version 1
__device__ __forceinline__ uint64_t smem_desc(uint32_t addr, uint32_t lbo_bytes, uint32_t sbo_bytes) {
    return (uint64_t)((addr & 0x3FFFFu) >> 4) | ((uint64_t)(lbo_bytes >> 4) << 16) |
           ((uint64_t)(sbo_bytes >> 4) << 32) | (1ull << 46);
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
        if (!(b <= e || a < e)) return false;
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
    uint64_t full_g[16], empty_g[16], full_m[32], empty_m[32], acc_full[NACC], acc_empty[NACC];
    uint32_t tmem_base;
    int abort_flag;
};

template <int NH> struct Cfg {
    // shared-memory budget: one CTA per SM
    static constexpr int kStages = (NH == 1) ? 8 : 4;
    static constexpr int kMeta = 2 * kStages;
    static constexpr int kStageBytes = MMAS_PER_STAGE * NH * A_MMA_BYTES;
    static constexpr int kAccCols = 16 * NH;
    static constexpr int kTmemCols = (NACC * kAccCols) < 32 ? 32 : NACC * kAccCols;   // 64 or 128: powers of two
    static constexpr size_t kSmem = 1024 + sizeof(SharedStorage) + (size_t)kStages * kStageBytes + (size_t)kMeta * META_BYTES;
};

__device__ __forceinline__ void raise(Params const &prm, SharedStorage *ss, int code) {
    ss->abort_flag = 1;
    atomicMax(prm.status, code);
}

template <int NH>
__global__ void __launch_bounds__(NUM_THREADS, 1)
spmm_tc5_kernel(const Params prm) {
    using C = Cfg<NH>;
    extern __shared__ uint8_t smem_raw[];
    // 1024-byte alignment is not required by the no-swizzle layouts; 128 is kept for the bulk copies
    uint8_t *smem = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(smem_raw) + 127) & ~uintptr_t(127));
    SharedStorage *ss = reinterpret_cast<SharedStorage *>(smem);
    uint8_t *ring_g = smem + ((sizeof(SharedStorage) + 127) & ~size_t(127));
    uint8_t *ring_m = ring_g + (size_t)C::kStages * C::kStageBytes;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int64_t W = prm.W;
    const int64_t T = __ldg(prm.window_offset + W);
    const int64_t G = gridDim.x;
    int64_t chunk = (T + G - 1) / G;
    chunk = (chunk + 1) & ~int64_t(1);
    if (chunk < 2) chunk = 2;

    if (threadIdx.x == 0) {
        for (int i = 0; i < C::kStages; ++i) { mbar_init(smem_u32(&ss->full_g[i]), NUM_PRODUCERS); mbar_init(smem_u32(&ss->empty_g[i]), 1); }
        for (int i = 0; i < C::kMeta; ++i) { mbar_init(smem_u32(&ss->full_m[i]), 1); mbar_init(smem_u32(&ss->empty_m[i]), 1); }
        for (int i = 0; i < NACC; ++i) { mbar_init(smem_u32(&ss->acc_full[i]), 1); mbar_init(smem_u32(&ss->acc_empty[i]), NUM_EPILOGUE); }
        ss->abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 8) {
        tmem_alloc(smem_u32(&ss->tmem_base), C::kTmemCols);
        tmem_relinquish();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = ss->tmem_base;
    volatile int *abort_flag = &ss->abort_flag;

    // this CTA's tile range (no cut is moved: long_window = 0 splits any window a cut falls into)
    int64_t w_first, w_unused;
    const int64_t s = warp_cut(prm.window_offset, W, T, blockIdx.x, G, chunk, 0, lane, &w_first);
    const int64_t e = warp_cut(prm.window_offset, W, T, (int64_t)blockIdx.x + 1, G, chunk, 0, lane, &w_unused);
    Walker wk;
    wk.init(prm.window_offset, W, s, e, blockIdx.x == 0 ? 0 : w_first, lane);

    if (warp == 9) {
        // ------------------------------------------------------------------ TMA producer
        const uint64_t pol = policy_stream();
        uint32_t it = 0;
        bool ok = true;
        while (ok && wk.next_segment(lane)) {
            for (int64_t t0 = wk.seg_s; ok && t0 < wk.seg_e; t0 += STAGE_TILES, ++it) {
                const uint32_t slot = it % C::kMeta, ph = (it / C::kMeta) & 1u;
                const int ntiles = (int)min((int64_t)STAGE_TILES, wk.seg_e - t0);
                if (lane == 0) {
                    ok = mbar_wait(smem_u32(&ss->empty_m[slot]), ph ^ 1u, abort_flag);
                    if (ok) {
                        const uint32_t bar = smem_u32(&ss->full_m[slot]);
                        uint8_t *dst = ring_m + (size_t)slot * META_BYTES;
                        mbar_expect_tx(bar, (uint32_t)ntiles * (TILE_BYTES + TILE_COLS * 4));
                        bulk_g2s(smem_u32(dst), static_cast<const uint8_t *>(prm.vals) + t0 * TILE_BYTES,
                                 (uint32_t)ntiles * TILE_BYTES, bar, pol);
                        bulk_g2s(smem_u32(dst + META_TILE_BYTES), prm.cols + t0 * TILE_COLS,
                                 (uint32_t)ntiles * TILE_COLS * 4, bar, pol);
                    } else {
                        raise(prm, ss, ST_TIMEOUT_META);
                    }
                }
                ok = __shfl_sync(0xffffffffu, ok ? 1 : 0, 0) != 0;
            }
        }
    } else if (warp < 4) {
        // ------------------------------------------------------------------ gather producers
        const uint64_t keep = policy_keep();
        const int p = threadIdx.x;                 // 0..127
        const int prow = p >> 4, pchunk = p & 15;  // row inside a group of 8, 16-byte piece of the slab
        const char *Bb = static_cast<const char *>(prm.B);
        uint32_t it = 0;
        bool ok = true;
        while (ok && wk.next_segment(lane)) {
            for (int64_t t0 = wk.seg_s; ok && t0 < wk.seg_e; t0 += STAGE_TILES, ++it) {
                const uint32_t gs = it % C::kStages, gph = (it / C::kStages) & 1u;
                const uint32_t ms = it % C::kMeta, mph = (it / C::kMeta) & 1u;
                const int ntiles = (int)min((int64_t)STAGE_TILES, wk.seg_e - t0);
                const int nrows = ((ntiles + 1) >> 1) * 16;        // rows the MMAs of this stage read
                // column ids have landed; the gather slot has been released by the MMA warp
                ok = mbar_wait(smem_u32(&ss->full_m[ms]), mph, abort_flag);
                if (ok) ok = mbar_wait(smem_u32(&ss->empty_g[gs]), gph ^ 1u, abort_flag);
                ok = __all_sync(0xffffffffu, ok) != 0;          // keep the warp together
                if (!ok) { raise(prm, ss, ST_TIMEOUT_EMPTY); break; }
                const int32_t *scol = reinterpret_cast<const int32_t *>(ring_m + (size_t)ms * META_BYTES + META_TILE_BYTES);
                const uint32_t stage_base = smem_u32(ring_g + (size_t)gs * C::kStageBytes);
#pragma unroll
                for (int j = 0; j < STAGE_SLOTS / 8; ++j) {
                    const int row = 8 * j + prow;
                    if (row < nrows) {
                        const int32_t col = (row < ntiles * TILE_COLS) ? scol[row] : -1;
                        const int m = row >> 4, slot16 = row & 15;
                        const char *src = Bb + ((int64_t)(col >= 0 ? col : 0) * prm.ldb) * 2 + pchunk * 16;
                        const uint32_t nbytes = col >= 0 ? 16u : 0u;
#pragma unroll
                        for (int h = 0; h < NH; ++h) {
                            const uint32_t dst = stage_base + (uint32_t)((m * NH + h) * A_MMA_BYTES + pchunk * A_SBO +
                                                                         (slot16 >> 3) * A_LBO + (slot16 & 7) * 16);
                            cp_async16(dst, src + h * (SLAB * 2), nbytes, keep);
                        }
                    }
                }
                // an odd tile count leaves the second tile of the last K-step unwritten: zero it
                if ((ntiles & 1) && p < 16) {
                    const uint32_t dst = smem_u32(ring_m + (size_t)ms * META_BYTES + (size_t)ntiles * TILE_BYTES) + p * 16;
                    cp_async16(dst, Bb, 0u, keep);
                }
                cp_async_arrive_noinc(smem_u32(&ss->full_g[gs]));
            }
        }
        cp_async_wait_all();
    } else if (warp == 8) {
        // ------------------------------------------------------------------ MMA issuer
        const uint32_t idesc = (1u << 4) | ((uint32_t)prm.is_bf16 << 7) | ((uint32_t)prm.is_bf16 << 10) |
                               (1u << 15) | ((16u >> 3) << 17) | ((128u >> 4) << 24);
        uint32_t it = 0, ai = 0;
        bool ok = true;
        while (ok && wk.next_segment(lane)) {
            if (wk.seg_e <= wk.seg_s) continue;            // empty window: the epilogue writes zeros
            const uint32_t buf = ai % NACC, aph = (ai / NACC) & 1u;
            ++ai;
            if (lane == 0) {
                ok = mbar_wait(smem_u32(&ss->acc_empty[buf]), aph ^ 1u, abort_flag);
                if (!ok) raise(prm, ss, ST_TIMEOUT_ACC);
            }
            ok = __shfl_sync(0xffffffffu, ok ? 1 : 0, 0) != 0;
            for (int64_t t0 = wk.seg_s; ok && t0 < wk.seg_e; t0 += STAGE_TILES, ++it) {
                const uint32_t gs = it % C::kStages, gph = (it / C::kStages) & 1u;
                const uint32_t ms = it % C::kMeta, mph = (it / C::kMeta) & 1u;
                const int ntiles = (int)min((int64_t)STAGE_TILES, wk.seg_e - t0);
                const int nmma = (ntiles + 1) >> 1;
                if (lane == 0) {
                    ok = mbar_wait(smem_u32(&ss->full_m[ms]), mph, abort_flag);
                    if (ok) ok = mbar_wait(smem_u32(&ss->full_g[gs]), gph, abort_flag);
                    if (ok) {
                        fence_async_smem();
                        tc_fence_after();
                        const uint32_t a_base = smem_u32(ring_g + (size_t)gs * C::kStageBytes);
                        const uint32_t b_base = smem_u32(ring_m + (size_t)ms * META_BYTES);
                        for (int m = 0; m < nmma; ++m) {
                            const uint64_t bd = smem_desc(b_base + m * 2 * TILE_BYTES, TILE_BYTES, 128);
#pragma unroll
                            for (int h = 0; h < NH; ++h) {
                                const uint64_t ad = smem_desc(a_base + (m * NH + h) * A_MMA_BYTES, A_LBO, A_SBO);
                                umma_f16(tmem_base + buf * C::kAccCols + h * 16, ad, bd, idesc,
                                         (t0 > wk.seg_s || m > 0) ? 1u : 0u);
                            }
                        }
                        umma_commit(smem_u32(&ss->empty_g[gs]));
                        umma_commit(smem_u32(&ss->empty_m[ms]));
                        if (t0 + STAGE_TILES >= wk.seg_e) umma_commit(smem_u32(&ss->acc_full[buf]));
                    } else {
                        raise(prm, ss, ST_TIMEOUT_FULL);
                    }
                }
                ok = __shfl_sync(0xffffffffu, ok ? 1 : 0, 0) != 0;
            }
        }
    } else {
        // ------------------------------------------------------------------ epilogue (warps 4-7)
        const uint64_t pol = policy_stream();
        const int q = warp & 3;                        // TMEM lane quarter this warp may read
        uint32_t ai = 0;
        bool ok = true;
        while (ok && wk.next_segment(lane)) {
            const int64_t w = wk.window();
            const bool nonempty = wk.seg_e > wk.seg_s;
            uint32_t v[NH][16];
            if (nonempty) {
                const uint32_t buf = ai % NACC, aph = (ai / NACC) & 1u;
                ++ai;
                ok = mbar_wait(smem_u32(&ss->acc_full[buf]), aph, abort_flag);
                ok = __all_sync(0xffffffffu, ok) != 0;
                if (!ok) { raise(prm, ss, ST_TIMEOUT_ACC); break; }
                tc_fence_after();
#pragma unroll
                for (int h = 0; h < NH; ++h)
                    tmem_ld16(tmem_base + ((uint32_t)(32 * q) << 16) + buf * C::kAccCols + h * 16, v[h]);
                tmem_ld_wait();
                tc_fence_before();
                mbar_arrive(smem_u32(&ss->acc_empty[buf]));
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
                if (!partial) {
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
        }
    }

    // teardown: everybody meets, then the allocating warp frees tensor memory
    tc_fence_before();
    __syncthreads();
    if (warp == 8) {
        tc_fence_after();
        tmem_dealloc(tmem_base, C::kTmemCols);
    }
}

// Sums the partial tiles of windows cut by a CTA boundary (same rule as the warp path's fix-up,
// with the chunk derived from the live tile count and the grid size).
__global__ void __launch_bounds__(128)
spmm_tc5_fixup_kernel(const Params prm, int64_t G) {
    __shared__ int64_t sh[3];
    const int64_t k = (int64_t)blockIdx.x + 1;
    const int64_t W = prm.W, N = prm.N;
    const int64_t T = __ldg(prm.window_offset + W);
    int64_t chunk = (T + G - 1) / G;
    chunk = (chunk + 1) & ~int64_t(1);
    if (chunk < 2) chunk = 2;
    const int64_t x = k * chunk;
    if (x >= T) return;
    if (threadIdx.x < 32) {
        int64_t w = warp_count_ends_le(prm.window_offset, W, x, threadIdx.x);
        if (threadIdx.x == 0) {
            sh[0] = w;
            sh[1] = __ldg(prm.window_offset + w);
            sh[2] = __ldg(prm.window_offset + w + 1);
        }
    }
    __syncthreads();
    const int64_t w = sh[0], a = sh[1], b = sh[2];
    if (x <= a) return;                       // the cut coincides with the window start
    if (a / chunk + 1 != k) return;           // an earlier cut inside this window sums it
    const int64_t k_last = (b - 1) / chunk;
    const int64_t elems = TILE_ROWS * N;
    for (int64_t i = threadIdx.x; i < elems; i += blockDim.x) {
        float v = prm.partial[(2 * (k - 1) + 1) * elems + i];
        for (int64_t q = k; q <= k_last; ++q) v += prm.partial[(2 * q) * elems + i];
        const int64_t r = i / N, f = i % N;
        const int64_t o = (w * TILE_ROWS + r) * prm.ldc + f;
        if (prm.c_dtype == GRWS_F32) static_cast<float *>(prm.C)[o] = v;
        else if (prm.c_dtype == GRWS_F16) static_cast<__half *>(prm.C)[o] = __float2half_rn(v);
        else static_cast<__nv_bfloat16 *>(prm.C)[o] = __float2bfloat16_rn(v);
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

}  // namespace tc5

bool spmm_tc5_supported(int dtype, int64_t N) {
    static const int disabled = [] { const char *e = getenv("GRWS_DISABLE_TCGEN05"); return e ? atoi(e) : 0; }();
    return !disabled && (dtype == GRWS_F16 || dtype == GRWS_BF16) && (N == 128 || N == 256);
}

size_t spmm_tc5_scratch_bytes(int64_t num_tiles_bound, int64_t N) {
    (void)num_tiles_bound;
    return tc5::STATUS_BYTES + (size_t)tc5::grid_size() * 2 * TILE_ROWS * (size_t)N * sizeof(float);
}

int spmm_tc5_launch(const int64_t *window_offset, const int32_t *cols, const void *vals, int dtype,
                    const void *B, int64_t ldb, void *C, int c_dtype, int64_t ldc, int64_t W,
                    int64_t num_tiles_bound, int64_t K, int64_t N, void *scratch, size_t scratch_bytes,
                    cudaStream_t stream) {
    using namespace tc5;
    (void)K;
    const size_t need = spmm_tc5_scratch_bytes(num_tiles_bound, N);
    if (scratch_bytes < need || scratch == nullptr)
        return fail(GRWS_ERR_SCRATCH, "spmm scratch too small: %zu < %zu bytes", scratch_bytes, need);
    Params prm;
    prm.window_offset = window_offset; prm.cols = cols; prm.vals = vals; prm.B = B; prm.C = C;
    prm.status = static_cast<int *>(scratch);
    prm.partial = reinterpret_cast<float *>(static_cast<char *>(scratch) + STATUS_BYTES);
    prm.W = W; prm.N = N; prm.ldb = ldb; prm.ldc = ldc; prm.c_dtype = c_dtype;
    prm.is_bf16 = dtype == GRWS_BF16 ? 1 : 0;
    const int G = grid_size();
    GRWS_CUDA_TRY(cudaMemsetAsync(scratch, 0, STATUS_BYTES, stream));
    if (N == 128) {
        static const cudaError_t attr = cudaFuncSetAttribute(spmm_tc5_kernel<1>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)Cfg<1>::kSmem);
        GRWS_CUDA_TRY(attr);
        spmm_tc5_kernel<1><<<G, NUM_THREADS, Cfg<1>::kSmem, stream>>>(prm);
    } else {
        static const cudaError_t attr = cudaFuncSetAttribute(spmm_tc5_kernel<2>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)Cfg<2>::kSmem);
        GRWS_CUDA_TRY(attr);
        spmm_tc5_kernel<2><<<G, NUM_THREADS, Cfg<2>::kSmem, stream>>>(prm);
    }
    GRWS_CUDA_TRY(cudaGetLastError());
    if (G > 1) {
        spmm_tc5_fixup_kernel<<<G - 1, 128, 0, stream>>>(prm, (int64_t)G);
        GRWS_CUDA_TRY(cudaGetLastError());
    }
    return GRWS_OK;
}

}  // namespace grws
