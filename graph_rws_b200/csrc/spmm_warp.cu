// BCSR SpMM, warp-MMA path: C[W*16, N] = A_bcsr * B[K, N].
//
// Replaces tcspmm_base_kernel (core/include/spmm_tc.cuh:40-195) for every dtype/shape, and is the
// fallback of the tcgen05 path.  Design (all of it differs from the reference kernel):
//   - work is cut over the global tile array, not one CTA per window, so hub windows of a
//     power-law graph are shared between warps (see grws_common.cuh);
//   - one warp owns a work item and a slab of features; the gathered rows of B go from L2
//     straight into MMA fragments with 128-bit loads and never touch shared memory.  This works
//     because the n index of an MMA is free to be permuted: slab j of a 64-feature group takes
//     feature 8*n + j, so the eight slabs a lane feeds are eight consecutive features of one row;
//   - fp16/bf16 use m16n8k16 over a pair of tiles, fp32 is rounded to TF32 (cvt.rna, as
//     spmm_tc.cuh:118-121,144-145 does) and uses m16n8k8 over one tile; accumulation is fp32;
//   - loads of the next two steps are in flight while the current one is multiplied.
#include <stdlib.h>

#include "grws_common.cuh"

namespace grws {

struct SpmmWarpParams {
    const int64_t *window_offset;
    const int32_t *cols;
    const void *vals;
    const void *B;
    void *C;
    float *partial;
    int64_t W, K, N, ldb, ldc;
    int64_t n_items, chunk, long_window;
    int c_dtype;
};

constexpr int WARPS_PER_CTA = 8;

// L2 residency hints: the gathered rows of B are re-read by many windows and should stay in L2
// (evict_last); tile values, column ids and the output are touched once (evict_first).
__device__ __forceinline__ uint64_t l2_policy_keep() {
    uint64_t p;
    asm volatile("createpolicy.fractional.L2::evict_last.b64 %0, 1.0;" : "=l"(p));
    return p;
}
__device__ __forceinline__ uint64_t l2_policy_stream() {
    uint64_t p;
    asm volatile("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;" : "=l"(p));
    return p;
}
__device__ __forceinline__ uint4 ldg128_hint(const void *p, uint64_t pol) {
    uint4 v;
    asm volatile("ld.global.nc.L1::no_allocate.L2::cache_hint.v4.u32 {%0,%1,%2,%3}, [%4], %5;"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p), "l"(pol));
    return v;
}
__device__ __forceinline__ uint32_t ldg32_hint(const void *p, uint64_t pol) {
    uint32_t v;
    asm volatile("ld.global.nc.L1::no_allocate.L2::cache_hint.u32 %0, [%1], %2;" : "=r"(v) : "l"(p), "l"(pol));
    return v;
}
__device__ __forceinline__ int2 ldg64_hint(const void *p, uint64_t pol) {
    int2 v;
    asm volatile("ld.global.nc.L1::no_allocate.L2::cache_hint.v2.s32 {%0,%1}, [%2], %3;" : "=r"(v.x), "=r"(v.y) : "l"(p), "l"(pol));
    return v;
}
__device__ __forceinline__ void stg128_hint(void *p, uint4 v, uint64_t pol) {
    asm volatile("st.global.L2::cache_hint.v4.u32 [%0], {%1,%2,%3,%4}, %5;"
                 :: "l"(p), "r"(v.x), "r"(v.y), "r"(v.z), "r"(v.w), "l"(pol) : "memory");
}

__device__ __forceinline__ uint32_t to_tf32(uint32_t f32_bits) {
    uint32_t r;
    asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(r) : "f"(__uint_as_float(f32_bits)));
    return r;
}

template <int DT>
__device__ __forceinline__ void mma_tile(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    if constexpr (DT == GRWS_F16) {
        asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                     : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                     : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
    } else if constexpr (DT == GRWS_BF16) {
        asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                     : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                     : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
    } else {
        asm volatile("mma.sync.aligned.m16n8k8.row.col.f32.tf32.tf32.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                     : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                     : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
    }
}

// Per-dtype geometry of one multiply step.
template <int DT> struct StepGeom {
    static constexpr bool kHalf = (DT != GRWS_F32);
    static constexpr int kTiles = kHalf ? 2 : 1;     // tiles consumed per step
    static constexpr int kRows = kHalf ? 4 : 2;      // gathered rows a lane loads per step
    static constexpr int kGroup = kHalf ? 64 : 32;   // features per group (8 lanes x 16 bytes)
    static constexpr int kSlabs = kHalf ? 8 : 4;     // MMA n-slabs per group
    static constexpr int kElem = kHalf ? 2 : 4;      // bytes per element
};

template <int DT, int NG> struct StepData {
    uint4 h[StepGeom<DT>::kRows * NG];   // gathered rows, [row][group]
    uint32_t a[4];                       // A fragment of the tile (pair)
};

struct StepCols {
    int c[4];   // column ids of the rows this lane gathers (-1: none)
};

// column ids of step `p` of the segment starting at tile `seg_s` (tiles [seg_s, seg_e))
template <int DT>
__device__ __forceinline__ StepCols load_cols(const int32_t *__restrict__ cols, int64_t seg_s,
                                              int64_t seg_e, int64_t p, int t, uint64_t pol) {
    using G = StepGeom<DT>;
    StepCols sc;
    const int64_t tile0 = seg_s + p * G::kTiles;
    if constexpr (G::kHalf) {
        // rows k = 2t, 2t+1 (first tile) and 8+2t, 9+2t (second tile)
        int2 lo = make_int2(-1, -1), hi = make_int2(-1, -1);
        if (tile0 < seg_e) lo = ldg64_hint(cols + tile0 * TILE_COLS + 2 * t, pol);
        if (tile0 + 1 < seg_e) hi = ldg64_hint(cols + (tile0 + 1) * TILE_COLS + 2 * t, pol);
        sc.c[0] = lo.x; sc.c[1] = lo.y; sc.c[2] = hi.x; sc.c[3] = hi.y;
    } else {
        // rows k = t and t + 4 of the single tile
        sc.c[0] = sc.c[1] = sc.c[2] = sc.c[3] = -1;
        if (tile0 < seg_e) {
            sc.c[0] = (int)ldg32_hint(cols + tile0 * TILE_COLS + t, pol);
            sc.c[1] = (int)ldg32_hint(cols + tile0 * TILE_COLS + t + 4, pol);
        }
    }
    return sc;
}

template <int DT, int NG>
__device__ __forceinline__ void load_step(StepData<DT, NG> &d, const StepCols &sc,
                                          const void *__restrict__ vals, const void *__restrict__ B,
                                          int64_t ldb, int64_t K, int64_t N, int64_t n0, int64_t seg_s,
                                          int64_t seg_e, int64_t p, int g, int t, uint64_t keep,
                                          uint64_t stream) {
    using G = StepGeom<DT>;
    const char *Bb = static_cast<const char *>(B);
#pragma unroll
    for (int r = 0; r < G::kRows; ++r) {
#pragma unroll
        for (int gi = 0; gi < NG; ++gi) {
            const int64_t feat = n0 + gi * G::kGroup + g * (16 / G::kElem);
            uint4 v = make_uint4(0u, 0u, 0u, 0u);
            // ids outside [0, K) -- the -1 padding, an id past the operand -- contribute nothing
            if ((uint64_t)(int64_t)sc.c[r] < (uint64_t)K && feat < N) v = ldg128_hint(Bb + ((int64_t)sc.c[r] * ldb + feat) * G::kElem, keep);
            d.h[r * NG + gi] = v;
        }
    }
    const int64_t tile0 = seg_s + p * G::kTiles;
    const uint32_t *v32 = static_cast<const uint32_t *>(vals);
    d.a[0] = d.a[1] = d.a[2] = d.a[3] = 0u;
    if constexpr (G::kHalf) {
        // 16-bit tile: row r is 16 bytes = 4 words; a0 = (row g, k 2t..2t+1), a1 = (row g+8, same k)
        if (tile0 < seg_e) {
            d.a[0] = ldg32_hint(v32 + tile0 * (TILE_ELEMS / 2) + g * 4 + t, stream);
            d.a[1] = ldg32_hint(v32 + tile0 * (TILE_ELEMS / 2) + (g + 8) * 4 + t, stream);
        }
        if (tile0 + 1 < seg_e) {
            d.a[2] = ldg32_hint(v32 + (tile0 + 1) * (TILE_ELEMS / 2) + g * 4 + t, stream);
            d.a[3] = ldg32_hint(v32 + (tile0 + 1) * (TILE_ELEMS / 2) + (g + 8) * 4 + t, stream);
        }
    } else {
        if (tile0 < seg_e) {
            d.a[0] = ldg32_hint(v32 + tile0 * TILE_ELEMS + g * 8 + t, stream);
            d.a[1] = ldg32_hint(v32 + tile0 * TILE_ELEMS + (g + 8) * 8 + t, stream);
            d.a[2] = ldg32_hint(v32 + tile0 * TILE_ELEMS + g * 8 + t + 4, stream);
            d.a[3] = ldg32_hint(v32 + tile0 * TILE_ELEMS + (g + 8) * 8 + t + 4, stream);
        }
    }
}

__device__ __forceinline__ uint32_t word_of(const uint4 &v, int i) {
    return i == 0 ? v.x : (i == 1 ? v.y : (i == 2 ? v.z : v.w));
}

template <int DT, int NG>
__device__ __forceinline__ void mma_step(float (&acc)[NG][StepGeom<DT>::kSlabs][4],
                                         const StepData<DT, NG> &d) {
    using G = StepGeom<DT>;
    uint32_t a[4];
    if constexpr (G::kHalf) {
#pragma unroll
        for (int i = 0; i < 4; ++i) a[i] = d.a[i];
    } else {
#pragma unroll
        for (int i = 0; i < 4; ++i) a[i] = to_tf32(d.a[i]);
    }
#pragma unroll
    for (int gi = 0; gi < NG; ++gi) {
#pragma unroll
        for (int j = 0; j < G::kSlabs; ++j) {
            uint32_t b0, b1;
            if constexpr (G::kHalf) {
                // feature j of the lane's 8: halves j of rows (2t, 2t+1) and of rows (8+2t, 9+2t)
                const uint32_t sel = (j & 1) ? 0x7632u : 0x5410u;
                b0 = __byte_perm(word_of(d.h[0 * NG + gi], j >> 1), word_of(d.h[1 * NG + gi], j >> 1), sel);
                b1 = __byte_perm(word_of(d.h[2 * NG + gi], j >> 1), word_of(d.h[3 * NG + gi], j >> 1), sel);
            } else {
                b0 = to_tf32(word_of(d.h[0 * NG + gi], j));
                b1 = to_tf32(word_of(d.h[1 * NG + gi], j));
            }
            mma_tile<DT>(acc[gi][j], a, b0, b1);
        }
    }
}

__device__ __forceinline__ uint32_t pack_f16(float a, float b) {
    __half2 h = __floats2half2_rn(a, b);
    return *reinterpret_cast<uint32_t *>(&h);
}
__device__ __forceinline__ uint32_t pack_bf16(float a, float b) {
    __nv_bfloat162 h = __floats2bfloat162_rn(a, b);
    return *reinterpret_cast<uint32_t *>(&h);
}

// store `count` consecutive outputs (count = 2 * kSlabs) of one row; v[i] is feature feat0 + i
template <int COUNT>
__device__ __forceinline__ void store_row(void *C, int c_dtype, int64_t elem_off, int64_t feat0,
                                          int64_t N, const float (&v)[COUNT], uint64_t pol) {
    if (feat0 >= N) return;   // N is a multiple of 8 and feat0 of COUNT (8 or 16): all or nothing per 8
    if (c_dtype == GRWS_F32) {
        float4 *p = reinterpret_cast<float4 *>(static_cast<float *>(C) + elem_off);
#pragma unroll
        for (int i = 0; i < COUNT / 4; ++i)
            if (feat0 + 4 * i < N)
                stg128_hint(p + i, make_uint4(__float_as_uint(v[4 * i]), __float_as_uint(v[4 * i + 1]),
                                              __float_as_uint(v[4 * i + 2]), __float_as_uint(v[4 * i + 3])), pol);
    } else {
        uint4 *p = reinterpret_cast<uint4 *>(static_cast<uint16_t *>(C) + elem_off);
#pragma unroll
        for (int i = 0; i < COUNT / 8; ++i) {
            if (feat0 + 8 * i >= N) break;
            uint4 o;
            if (c_dtype == GRWS_F16) {
                o.x = pack_f16(v[8 * i], v[8 * i + 1]); o.y = pack_f16(v[8 * i + 2], v[8 * i + 3]);
                o.z = pack_f16(v[8 * i + 4], v[8 * i + 5]); o.w = pack_f16(v[8 * i + 6], v[8 * i + 7]);
            } else {
                o.x = pack_bf16(v[8 * i], v[8 * i + 1]); o.y = pack_bf16(v[8 * i + 2], v[8 * i + 3]);
                o.z = pack_bf16(v[8 * i + 4], v[8 * i + 5]); o.w = pack_bf16(v[8 * i + 6], v[8 * i + 7]);
            }
            stg128_hint(p + i, o, pol);
        }
    }
}

template <int DT, int NG>
__global__ void __launch_bounds__(WARPS_PER_CTA * 32)
spmm_warp_kernel(const SpmmWarpParams prm) {
    using G = StepGeom<DT>;
    // the warp index is read from lane 0 so that the compiler knows it (and the work item, window and tile
    // indices derived from it) to be the same in all lanes and can keep them in uniform registers
    const int lane = threadIdx.x & 31, warp = __shfl_sync(0xffffffffu, (int)(threadIdx.x >> 5), 0);
    const int g = lane >> 2, t = lane & 3;
    const int64_t item = (int64_t)blockIdx.x * WARPS_PER_CTA + warp;
    if (item >= prm.n_items) return;
    const int64_t n0 = (int64_t)blockIdx.y * (NG * G::kGroup);
    const int64_t W = prm.W, N = prm.N;
    const int64_t T = __ldg(prm.window_offset + W);
    const uint64_t keep = l2_policy_keep(), stream = l2_policy_stream();

    int64_t w_first, w_unused;
    const int64_t s = warp_cut(prm.window_offset, W, T, item, prm.n_items, prm.chunk, prm.long_window, lane, &w_first);
    const int64_t e = warp_cut(prm.window_offset, W, T, item + 1, prm.n_items, prm.chunk, prm.long_window, lane, &w_unused);

    for (int64_t w = (item == 0) ? 0 : w_first; w < W; ++w) {
        const int64_t a = __ldg(prm.window_offset + w), b = __ldg(prm.window_offset + w + 1);
        if (!(b <= e || a < e)) break;
        const int64_t seg_s = a > s ? a : s, seg_e = b < e ? b : e;
        const int64_t nsteps = seg_e > seg_s ? (seg_e - seg_s + G::kTiles - 1) / G::kTiles : 0;

        float acc[NG][G::kSlabs][4];
#pragma unroll
        for (int gi = 0; gi < NG; ++gi)
#pragma unroll
            for (int j = 0; j < G::kSlabs; ++j)
#pragma unroll
                for (int i = 0; i < 4; ++i) acc[gi][j][i] = 0.f;

        if (nsteps > 0) {
            StepCols c2 = load_cols<DT>(prm.cols, seg_s, seg_e, 2, t, stream);
            StepCols c3 = load_cols<DT>(prm.cols, seg_s, seg_e, 3, t, stream);
            StepData<DT, NG> d0, d1;
            {
                StepCols c0 = load_cols<DT>(prm.cols, seg_s, seg_e, 0, t, stream);
                StepCols c1 = load_cols<DT>(prm.cols, seg_s, seg_e, 1, t, stream);
                load_step<DT, NG>(d0, c0, prm.vals, prm.B, prm.ldb, prm.K, N, n0, seg_s, seg_e, 0, g, t, keep, stream);
                load_step<DT, NG>(d1, c1, prm.vals, prm.B, prm.ldb, prm.K, N, n0, seg_s, seg_e, 1, g, t, keep, stream);
            }
            for (int64_t p = 0; p < nsteps; p += 2) {
                StepCols c4 = load_cols<DT>(prm.cols, seg_s, seg_e, p + 4, t, stream);
                StepCols c5 = load_cols<DT>(prm.cols, seg_s, seg_e, p + 5, t, stream);
                mma_step<DT, NG>(acc, d0);
                load_step<DT, NG>(d0, c2, prm.vals, prm.B, prm.ldb, prm.K, N, n0, seg_s, seg_e, p + 2, g, t, keep, stream);
                if (p + 1 < nsteps) mma_step<DT, NG>(acc, d1);
                load_step<DT, NG>(d1, c3, prm.vals, prm.B, prm.ldb, prm.K, N, n0, seg_s, seg_e, p + 3, g, t, keep, stream);
                c2 = c4;
                c3 = c5;
            }
        }

        // acc[gi][j][0..1] = row g, features base + 16t + j and base + 16t + 8 + j (half) or
        // base + 8t + j and base + 8t + 4 + j (tf32); [2..3] the same for row g + 8.
        const bool head = seg_s > a, tail = !head && seg_e < b;
#pragma unroll
        for (int gi = 0; gi < NG; ++gi) {
            float lo[2 * G::kSlabs], hi[2 * G::kSlabs];
#pragma unroll
            for (int j = 0; j < G::kSlabs; ++j) {
                lo[j] = acc[gi][j][0]; lo[G::kSlabs + j] = acc[gi][j][1];
                hi[j] = acc[gi][j][2]; hi[G::kSlabs + j] = acc[gi][j][3];
            }
            const int64_t feat0 = n0 + gi * G::kGroup + t * (2 * G::kSlabs);
            if (!head && !tail) {
                store_row<2 * G::kSlabs>(prm.C, prm.c_dtype, (w * TILE_ROWS + g) * prm.ldc + feat0, feat0, N, lo, stream);
                store_row<2 * G::kSlabs>(prm.C, prm.c_dtype, (w * TILE_ROWS + g + 8) * prm.ldc + feat0, feat0, N, hi, stream);
            } else {
                float *slot = prm.partial + (2 * item + (tail ? 1 : 0)) * (TILE_ROWS * N);
                store_row<2 * G::kSlabs>(slot, GRWS_F32, (int64_t)g * N + feat0, feat0, N, lo, stream);
                store_row<2 * G::kSlabs>(slot, GRWS_F32, (int64_t)(g + 8) * N + feat0, feat0, N, hi, stream);
            }
        }
    }
}

// Sums the partial tiles of every window that was split between work items, in item order.
// One CTA per interior cut; only the first cut inside a window does the work.
__global__ void __launch_bounds__(128)
spmm_fixup_kernel(const SpmmWarpParams prm) {
    __shared__ int64_t sh[3];
    const int64_t k = (int64_t)blockIdx.x + 1;
    const int64_t W = prm.W, N = prm.N;
    const int64_t T = __ldg(prm.window_offset + W);
    const int64_t x = k * prm.chunk;
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
    if (b - a <= prm.long_window || x <= a) return;     // cut was moved to the window start / not inside
    if (a / prm.chunk + 1 != k) return;                 // an earlier cut inside this window sums it
    const int64_t k_last = (b - 1) / prm.chunk;
    const int64_t elems = TILE_ROWS * N;
    for (int64_t i = threadIdx.x; i < elems; i += blockDim.x) {
        float v = prm.partial[(2 * (k - 1) + 1) * elems + i];               // tail piece of item k-1
        for (int64_t q = k; q <= k_last; ++q) v += prm.partial[(2 * q) * elems + i];   // head pieces
        const int64_t r = i / N, f = i % N;
        const int64_t o = (w * TILE_ROWS + r) * prm.ldc + f;
        if (prm.c_dtype == GRWS_F32) static_cast<float *>(prm.C)[o] = v;
        else if (prm.c_dtype == GRWS_F16) static_cast<__half *>(prm.C)[o] = __float2half_rn(v);
        else static_cast<__nv_bfloat16 *>(prm.C)[o] = __float2bfloat16_rn(v);
    }
}

// ---------------------------------------------------------------------------------------------
// host side
// ---------------------------------------------------------------------------------------------
void spmm_warp_plan(int64_t num_tiles_bound, int64_t *n_items, int64_t *chunk, int64_t *long_window) {
    // work items (one warp each): 112 per SM, i.e. 14 waves of the 8-warp CTAs -- enough for the
    // power-law tail to even out, few enough that the per-item partial tiles stay small
    int dev = 0, sms = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || sms <= 0)
        sms = 148;
    const int64_t target_items = (int64_t)sms * 112;
    int64_t c = ceil_div(num_tiles_bound > 0 ? num_tiles_bound : 1, target_items);
    // at least 64 tiles per item, 16 for a small product: a warp walks its tiles one after the other
    // (~0.5 us per tile), so a block of a thousand tiles wants a hundred warps, not sixteen
    const int64_t c_min = num_tiles_bound <= 65536 ? 16 : 64;
    if (c < c_min) c = c_min;
    c = (c + 1) & ~int64_t(1);
    *chunk = c;
    *long_window = 2 * c;
    int64_t n = ceil_div(num_tiles_bound, c);
    *n_items = n > 0 ? n : 1;
}

size_t spmm_warp_scratch_bytes(int64_t num_tiles_bound, int64_t N) {
    int64_t n_items, chunk, lw;
    spmm_warp_plan(num_tiles_bound, &n_items, &chunk, &lw);
    return (size_t)n_items * 2 * TILE_ROWS * (size_t)N * sizeof(float);
}

// experiment builds (-DGRWS_WARP_NARROW=1) give every warp a single feature group (more warps per
// SM, the A fragments read once per group)
static bool narrow_slabs() {
#ifdef GRWS_WARP_NARROW
    return GRWS_WARP_NARROW != 0;
#else
    return false;
#endif
}

template <int DT>
static int launch_warp(const SpmmWarpParams &prm, cudaStream_t stream) {
    using G = StepGeom<DT>;
    const int64_t N = prm.N;
    dim3 block(WARPS_PER_CTA * 32);
    const unsigned gx = (unsigned)ceil_div(prm.n_items, WARPS_PER_CTA);
    // features per warp: at most two groups (128 features of a 16-bit type, 64 of fp32).  Four groups of
    // fp32 need 202 registers, one CTA per SM: 584 us on the 2.5 M-entry graph against 375 us with two.
    if (N <= G::kGroup || narrow_slabs()) {
        const unsigned gy = (unsigned)ceil_div(N, G::kGroup);
        spmm_warp_kernel<DT, 1><<<dim3(gx, gy), block, 0, stream>>>(prm);
    } else {
        const unsigned gy = (unsigned)ceil_div(N, 2 * G::kGroup);
        spmm_warp_kernel<DT, 2><<<dim3(gx, gy), block, 0, stream>>>(prm);
    }
    GRWS_CUDA_TRY(cudaGetLastError());
    if (prm.n_items > 1) {
        spmm_fixup_kernel<<<(unsigned)(prm.n_items - 1), 128, 0, stream>>>(prm);
        GRWS_CUDA_TRY(cudaGetLastError());
    }
    return GRWS_OK;
}

int spmm_warp_launch(const int64_t *window_offset, const int32_t *cols, const void *vals, int dtype,
                     const void *B, int64_t ldb, void *C, int c_dtype, int64_t ldc, int64_t W,
                     int64_t num_tiles_bound, int64_t K, int64_t N, void *scratch,
                     size_t scratch_bytes, cudaStream_t stream) {
    SpmmWarpParams prm;
    prm.window_offset = window_offset; prm.cols = cols; prm.vals = vals; prm.B = B; prm.C = C;
    prm.partial = static_cast<float *>(scratch);
    prm.W = W; prm.K = K; prm.N = N; prm.ldb = ldb; prm.ldc = ldc; prm.c_dtype = c_dtype;
    spmm_warp_plan(num_tiles_bound, &prm.n_items, &prm.chunk, &prm.long_window);
    const size_t need = spmm_warp_scratch_bytes(num_tiles_bound, N);
    if (scratch_bytes < need || (need > 0 && scratch == nullptr))
        return fail(GRWS_ERR_SCRATCH, "spmm scratch too small: %zu < %zu bytes", scratch_bytes, need);
    if (prm.n_items > 0x7fffffffLL * WARPS_PER_CTA) return fail(GRWS_ERR_UNSUPPORTED, "too many work items");
    switch (dtype) {
        case GRWS_F32: return launch_warp<GRWS_F32>(prm, stream);
        case GRWS_F16: return launch_warp<GRWS_F16>(prm, stream);
        case GRWS_BF16: return launch_warp<GRWS_BF16>(prm, stream);
    }
    return fail(GRWS_ERR_UNSUPPORTED, "unknown dtype %d", dtype);
}

}  // namespace grws
