// GPU neighbour sampling, dedup / reindex, and the column reindex of sampled blocks.
//
// Replaces the sampling half of the reference's extension.  The reference samples per 16-row
// window and keeps the top-K columns by edge weight (core/include/sampling.cuh:65-448, driven by
// core/wrapper/sampling_wrapper.cu:58-438); it has no random generator.  Here a hop is
//   1. sample_hop_kernel   one warp per frontier node: uniform sampling without replacement on a
//                          counter-based Philox4x32-10 stream keyed by (seed, node, hop), so a
//                          node's list does not depend on batch composition, launch shape or GPU
//                          count (Floyd's subset algorithm; degree <= fanout takes every
//                          neighbour in CSR order);
//   2. dedup / reindex     a global-memory hash set of the destination nodes plus the sampled
//                          neighbours: the source list of the hop is the destination nodes
//                          followed by the new nodes in ascending id order (radix sort), and every
//                          sampled edge gets the position of its endpoint in that list;
//   3. compaction          the fixed-stride neighbour lists become a local CSR, which the
//                          device BCSR builder (bcsr_build.cu) turns into the hop's block.
// reindex_and_prune_kernel (core/include/reindex.cuh:33-102) is kept as well, with the same
// integer arithmetic, for graphs that carry the reference's window-level `active_windows`.
#include <cub/cub.cuh>

#include "grws_common.cuh"

namespace grws {

constexpr int MAX_FANOUT = 256;          // the reference's dispatch stops at 256 too (core/helper/macros.h:60-71)
constexpr int SAMPLE_WARPS = 8;

// ---------------------------------------------------------------------------------------------
// Philox4x32-10 (Salmon et al., SC'11)
// ---------------------------------------------------------------------------------------------
__host__ __device__ __forceinline__ void philox4x32_10(uint32_t c0, uint32_t c1, uint32_t c2, uint32_t c3,
                                                       uint32_t k0, uint32_t k1, uint32_t (&out)[4]) {
#pragma unroll
    for (int r = 0; r < 10; ++r) {
        const uint64_t p0 = (uint64_t)0xD2511F53u * c0;
        const uint64_t p1 = (uint64_t)0xCD9E8D57u * c2;
        const uint32_t n0 = (uint32_t)(p1 >> 32) ^ c1 ^ k0;
        const uint32_t n1 = (uint32_t)p1;
        const uint32_t n2 = (uint32_t)(p0 >> 32) ^ c3 ^ k1;
        const uint32_t n3 = (uint32_t)p0;
        c0 = n0; c1 = n1; c2 = n2; c3 = n3;
        k0 += 0x9E3779B9u; k1 += 0xBB67AE85u;
    }
    out[0] = c0; out[1] = c1; out[2] = c2; out[3] = c3;
}

// j-th 64-bit draw of the stream (seed, node, hop): counter {node, hop, j >> 1, 0}, key = seed;
// words (2*(j&1)+1 : 2*(j&1)) of the block
__device__ __forceinline__ uint64_t sample_draw64(uint64_t seed, uint32_t node, uint32_t hop, uint32_t j) {
    uint32_t o[4];
    philox4x32_10(node, hop, j >> 1, 0u, (uint32_t)seed, (uint32_t)(seed >> 32), o);
    const uint32_t lo = (j & 1) ? o[2] : o[0], hi = (j & 1) ? o[3] : o[1];
    return ((uint64_t)hi << 32) | lo;
}

// One warp per frontier node.  Output slots have a fixed stride of `fanout`; unused slots hold
// -1 / 0.  For degree d > fanout f, pick j is floor(draw_j * (d - f + j + 1) / 2^64) unless an
// earlier pick has that value, in which case it is d - f + j (Floyd); picks are emitted in j order.
__global__ void __launch_bounds__(SAMPLE_WARPS * 32)
sample_hop_kernel(const int64_t *__restrict__ row_ptr, const int32_t *__restrict__ col_idx,
                  const float *__restrict__ values, const int32_t *__restrict__ nodes, int64_t n,
                  int fanout, uint64_t seed, const uint64_t *__restrict__ seed_dev, uint32_t hop,
                  int32_t *__restrict__ out_nbr, float *__restrict__ out_w, int32_t *__restrict__ out_cnt) {
    __shared__ int64_t picks[SAMPLE_WARPS][MAX_FANOUT];
    if (seed_dev) seed = *seed_dev;          // a seed that changes between replays of one captured launch
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int64_t i = (int64_t)blockIdx.x * SAMPLE_WARPS + warp;
    if (i >= n) return;
    const int32_t v = nodes[i];
    int32_t *nb = out_nbr + i * fanout;
    float *ww = out_w + i * fanout;
    int64_t e0 = 0, d = 0;
    if (v >= 0) {
        e0 = __ldg(row_ptr + v);
        d = __ldg(row_ptr + v + 1) - e0;
    }
    if (d <= fanout) {
        for (int j = lane; j < fanout; j += 32) {
            const bool in = j < d;
            nb[j] = in ? __ldg(col_idx + e0 + j) : -1;
            ww[j] = in ? (values ? __ldg(values + e0 + j) : 1.0f) : 0.0f;
        }
        if (lane == 0 && out_cnt) out_cnt[i] = (int32_t)d;
        return;
    }
    int64_t *pk = picks[warp];
    // all draws first (independent), then the sequential duplicate resolution
    for (int j = lane; j < fanout; j += 32)
        pk[j] = (int64_t)__umul64hi(sample_draw64(seed, (uint32_t)v, hop, (uint32_t)j), (uint64_t)(d - fanout + j + 1));
    __syncwarp();
    for (int j = 1; j < fanout; ++j) {
        const int64_t t = pk[j];
        bool dup = false;
        for (int q = lane; q < j; q += 32) dup |= (pk[q] == t);
        if (__any_sync(0xffffffffu, dup)) {
            if (lane == 0) pk[j] = d - fanout + j;
        }
        __syncwarp();
    }
    for (int j = lane; j < fanout; j += 32) {
        const int64_t e = e0 + pk[j];
        nb[j] = __ldg(col_idx + e);
        ww[j] = values ? __ldg(values + e) : 1.0f;
    }
    if (lane == 0 && out_cnt) out_cnt[i] = fanout;
}

// ---------------------------------------------------------------------------------------------
// dedup / reindex
// ---------------------------------------------------------------------------------------------
constexpr int32_t EMPTY_KEY = -1;
constexpr int32_t NEW_NODE = 0x7fffffff;     // value of a neighbour that is not a destination node (rank not yet known)

__device__ __forceinline__ uint32_t hash_node(int32_t k) {
    uint32_t x = (uint32_t)k * 0x9E3779B1u;
    return x ^ (x >> 15);
}

// inserts `key`; returns the slot.  `fresh` tells whether this call created the entry.
__device__ __forceinline__ uint32_t table_insert(int32_t *keys, uint32_t mask, int32_t key, bool &fresh) {
    uint32_t h = hash_node(key) & mask;
    for (;;) {
        // a plain read first: a slot that already holds this key (a hub sampled from many rows) or
        // another one needs no atomic
        const int32_t cur = *reinterpret_cast<const volatile int32_t *>(keys + h);
        if (cur == key) { fresh = false; return h; }
        if (cur == EMPTY_KEY) {
            const int32_t prev = atomicCAS(keys + h, EMPTY_KEY, key);
            if (prev == EMPTY_KEY) { fresh = true; return h; }
            if (prev == key) { fresh = false; return h; }
        }
        h = (h + 1) & mask;
    }
}

__device__ __forceinline__ int32_t table_lookup(const int32_t *keys, const int32_t *vals, uint32_t mask, int32_t key) {
    uint32_t h = hash_node(key) & mask;
    for (;;) {
        const int32_t k = keys[h];
        if (k == key) return vals[h];
        if (k == EMPTY_KEY) return -1;
        h = (h + 1) & mask;
    }
}

__global__ void insert_dst_kernel(const int32_t *__restrict__ dst, int64_t n_dst, int32_t *keys, int32_t *vals,
                                  uint32_t mask, int32_t *__restrict__ out_src) {
    const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n_dst) return;
    const int32_t v = dst[i];
    out_src[i] = v;
    if (v < 0) return;
    bool fresh;
    const uint32_t h = table_insert(keys, mask, v, fresh);
    atomicMin(vals + h, (int32_t)i);             // a repeated destination node keeps its first position
}

__global__ void insert_nbr_kernel(const int32_t *__restrict__ nbr, int64_t n_edges, int32_t *keys, int32_t *vals,
                                  uint32_t mask, int32_t *__restrict__ cand, int32_t *__restrict__ n_new) {
    const int64_t e = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    const int32_t u = e < n_edges ? nbr[e] : -1;
    bool fresh = false;
    if (u >= 0) table_insert(keys, mask, u, fresh);
    // one atomic on the shared counter per warp, not per new node (the order of `cand` does not
    // matter: it is sorted before the ranks are given out); vals[h] stays NEW_NODE until then
    const unsigned m = __ballot_sync(0xffffffffu, fresh);
    if (m) {
        const int lane = threadIdx.x & 31, leader = __ffs(m) - 1;
        int base = 0;
        if (lane == leader) base = atomicAdd(n_new, __popc(m));
        base = __shfl_sync(0xffffffffu, base, leader);
        if (fresh) cand[base + __popc(m & ((1u << lane) - 1u))] = u;
    }
}

__global__ void rank_new_kernel(const int32_t *__restrict__ cand_sorted, const int32_t *__restrict__ n_new,
                                int64_t n_dst, const int32_t *keys, int32_t *vals, uint32_t mask,
                                int32_t *__restrict__ out_src) {
    const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= *n_new) return;
    const int32_t u = cand_sorted[i];
    out_src[n_dst + i] = u;
    uint32_t h = hash_node(u) & mask;
    while (keys[h] != u) h = (h + 1) & mask;
    vals[h] = (int32_t)(n_dst + i);
}

// local ids of the sampled neighbours, and the number of valid entries of every destination row
__global__ void localize_kernel(const int32_t *__restrict__ nbr, int64_t n_dst, int fanout, const int32_t *keys,
                                const int32_t *vals, uint32_t mask, int32_t *__restrict__ out_local,
                                int64_t *__restrict__ row_cnt) {
    const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;   // one thread per destination row
    if (i >= n_dst) return;
    int cnt = 0;
    for (int j = 0; j < fanout; ++j) {
        const int32_t u = nbr[i * fanout + j];
        int32_t l = -1;
        if (u >= 0) { l = table_lookup(keys, vals, mask, u); ++cnt; }
        out_local[i * fanout + j] = l;
    }
    row_cnt[i + 1] = cnt;
    if (i == 0) row_cnt[0] = 0;
}

__global__ void finish_counts_kernel(const int32_t *__restrict__ n_new, int64_t n_dst, const int64_t *__restrict__ row_ptr,
                                     int64_t *__restrict__ out_counts) {
    out_counts[0] = n_dst + *n_new;      // number of source nodes
    out_counts[1] = row_ptr[n_dst];      // number of sampled edges
}

__global__ void compact_kernel(const int32_t *__restrict__ local, const float *__restrict__ w, int64_t n_dst, int fanout,
                               const int64_t *__restrict__ row_ptr, int32_t *__restrict__ out_col, float *__restrict__ out_val) {
    const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n_dst) return;
    int64_t o = row_ptr[i];
    for (int j = 0; j < fanout; ++j) {
        const int32_t l = local[i * fanout + j];
        if (l >= 0) { out_col[o] = l; out_val[o] = w[i * fanout + j]; ++o; }
    }
}

__global__ void fill_i32(int32_t *p, int64_t n, int32_t v) {
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x) p[i] = v;
}

// same integer arithmetic as reindex_and_prune_kernel (core/include/reindex.cuh:33-102): the window
// of a column is col / tile_rows with C division, so a -1 padding id is looked up as window 0
template <typename T>
__global__ void reindex_kernel(const int32_t *__restrict__ in_cols, T *__restrict__ values,
                               const int32_t *__restrict__ active_windows, int64_t num_indices, int num_active,
                               int tile_rows, int tile_cols, int32_t *__restrict__ out_cols) {
    const int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= num_indices) return;
    const int g = in_cols[idx];
    const int target = g / tile_rows;
    int left = 0, right = num_active - 1, found = -1;
    while (left <= right) {
        const int mid = (left + right) / 2;
        const int win = __ldg(active_windows + mid);
        if (win == target) { found = mid; break; }
        if (win < target) left = mid + 1; else right = mid - 1;
    }
    if (found != -1) {
        out_cols[idx] = found * tile_rows + (g % tile_rows);
    } else {
        out_cols[idx] = 0;
        const int64_t base = (idx / tile_cols) * tile_rows * tile_cols;
        const int cit = (int)(idx % tile_cols);
        for (int r = 0; r < tile_rows; ++r) values[base + r * tile_cols + cit] = T(0.0f);
    }
}

// one launch instead of four fills: empty hash table, candidate list of sentinels, zero counter,
// and the part of the source list behind the destination nodes set to -1
__global__ void dedup_init_kernel(int32_t *keys, int32_t *vals, int64_t slots, int32_t *cand, int64_t n_cand,
                                  int32_t *n_new, int32_t *src_tail, int64_t n_tail) {
    const int64_t stride = (int64_t)gridDim.x * blockDim.x, i0 = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    for (int64_t i = i0; i < slots; i += stride) { keys[i] = EMPTY_KEY; vals[i] = NEW_NODE; }
    for (int64_t i = i0; i < n_cand; i += stride) cand[i] = NEW_NODE;
    for (int64_t i = i0; i < n_tail; i += stride) src_tail[i] = -1;
    if (i0 == 0) *n_new = 0;
}

// local id of every sampled neighbour (one thread per list slot)
__global__ void localize_flat_kernel(const int32_t *__restrict__ nbr, int64_t n_entries, const int32_t *keys,
                                     const int32_t *vals, uint32_t mask, int32_t *__restrict__ out_local) {
    const int64_t e = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (e >= n_entries) return;
    const int32_t u = nbr[e];
    out_local[e] = u >= 0 ? table_lookup(keys, vals, mask, u) : -1;
}

// per-hop figures for the caller: {source nodes (padded destinations + new nodes), sampled edges,
// tiles of the block, real (non-padding) frontier nodes}
__global__ void hop_counts_kernel(const int32_t *__restrict__ n_new, const int32_t *__restrict__ dst, int64_t n_dst,
                                  const int32_t *__restrict__ cnt, const int64_t *__restrict__ window_offset, int64_t W,
                                  int64_t *__restrict__ out) {
    __shared__ unsigned long long s_edges, s_real;
    if (threadIdx.x == 0) { s_edges = 0; s_real = 0; }
    __syncthreads();
    unsigned long long e = 0, r = 0;
    for (int64_t i = threadIdx.x; i < n_dst; i += blockDim.x) { e += (unsigned long long)cnt[i]; r += dst[i] >= 0 ? 1 : 0; }
    atomicAdd(&s_edges, e);
    atomicAdd(&s_real, r);
    __syncthreads();
    if (threadIdx.x == 0) {
        out[0] = n_dst + *n_new;
        out[1] = (int64_t)s_edges;
        out[2] = window_offset[W];
        out[3] = (int64_t)s_real;
    }
}

static inline size_t up256(size_t x) { return (x + 255) / 256 * 256; }
static inline unsigned nblocks(int64_t n, int t) { int64_t b = (n + t - 1) / t; return (unsigned)(b < 1 ? 1 : b); }

struct DedupScratch {
    int32_t *keys, *vals, *cand, *cand_sorted, *n_new;
    void *cub_tmp;
    size_t cub_bytes, total;
    uint32_t slots;
};

static DedupScratch carve_dedup(void *base, int64_t n_dst, int fanout) {
    DedupScratch s;
    const int64_t n_edges = n_dst * fanout;
    uint64_t want = 2ull * (uint64_t)(n_dst + n_edges) + 16, slots = 64;
    while (slots < want) slots <<= 1;
    s.slots = (uint32_t)slots;
    char *p = static_cast<char *>(base);
    size_t off = 0;
    auto take = [&](size_t bytes) { char *q = p ? p + off : nullptr; off += up256(bytes); return (void *)q; };
    s.keys = (int32_t *)take(slots * 4);
    s.vals = (int32_t *)take(slots * 4);
    s.cand = (int32_t *)take((size_t)(n_edges + 1) * 4);
    s.cand_sorted = (int32_t *)take((size_t)(n_edges + 1) * 4);
    s.n_new = (int32_t *)take(256);
    size_t c1 = 0, c2 = 0;
    cub::DeviceRadixSort::SortKeys(nullptr, c1, (const int32_t *)nullptr, (int32_t *)nullptr, (int)(n_edges > 0 ? n_edges : 1));
    cub::DeviceScan::InclusiveSum(nullptr, c2, (const int64_t *)nullptr, (int64_t *)nullptr, (int)(n_dst + 1));
    s.cub_bytes = c1 > c2 ? c1 : c2;
    s.cub_tmp = take(s.cub_bytes);
    s.total = off;
    return s;
}

}  // namespace grws

using namespace grws;

extern "C" {

__attribute__((visibility("default")))
int grws_sample_hop(const int64_t *row_ptr, const int32_t *col_idx, const float *values, const int32_t *nodes,
                    int64_t num_nodes, int fanout, uint64_t seed, uint32_t hop, int32_t *out_nbr, float *out_w,
                    int32_t *out_cnt, void *stream) {
    GRWS_REQUIRE(num_nodes >= 0, "negative size");
    GRWS_REQUIRE(fanout > 0 && fanout <= MAX_FANOUT, "fanout %d outside [1, %d]", fanout, MAX_FANOUT);
    if (num_nodes == 0) return GRWS_OK;
    GRWS_REQUIRE(row_ptr && col_idx && nodes && out_nbr && out_w, "null pointer");
    sample_hop_kernel<<<nblocks(num_nodes, SAMPLE_WARPS), SAMPLE_WARPS * 32, 0, static_cast<cudaStream_t>(stream)>>>(
        row_ptr, col_idx, values, nodes, num_nodes, fanout, seed, nullptr, hop, out_nbr, out_w, out_cnt);
    GRWS_CUDA_TRY(cudaGetLastError());
    return GRWS_OK;
}

__attribute__((visibility("default")))
size_t grws_dedup_scratch_bytes(int64_t n_dst, int fanout) {
    if (n_dst < 0 || fanout <= 0) return 0;
    return carve_dedup(nullptr, n_dst, fanout).total;
}

__attribute__((visibility("default")))
int grws_dedup_reindex(const int32_t *dst, int64_t n_dst, const int32_t *nbr, int fanout, int32_t *out_src,
                       int32_t *out_local, int64_t *out_row_ptr, int64_t *out_counts, void *scratch,
                       size_t scratch_bytes, void *stream) {
    GRWS_REQUIRE(n_dst >= 0 && fanout > 0, "bad size");
    GRWS_REQUIRE(n_dst * (int64_t)fanout < 0x7fffffffLL, "hop too large");
    GRWS_REQUIRE(out_src && out_local && out_row_ptr && out_counts && scratch, "null pointer");
    DedupScratch s = carve_dedup(scratch, n_dst, fanout);
    if (scratch_bytes < s.total) return fail(GRWS_ERR_SCRATCH, "dedup scratch too small: %zu < %zu", scratch_bytes, s.total);
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    const int64_t n_edges = n_dst * fanout;
    const uint32_t mask = s.slots - 1;
    GRWS_CUDA_TRY(cudaMemsetAsync(s.keys, 0xff, (size_t)s.slots * 4, st));                 // EMPTY_KEY
    fill_i32<<<nblocks(s.slots, 256) > 2048 ? 2048 : nblocks(s.slots, 256), 256, 0, st>>>(s.vals, s.slots, NEW_NODE);
    fill_i32<<<nblocks(n_edges + 1, 256) > 2048 ? 2048 : nblocks(n_edges + 1, 256), 256, 0, st>>>(s.cand, n_edges + 1, NEW_NODE);
    GRWS_CUDA_TRY(cudaMemsetAsync(s.n_new, 0, 256, st));
    if (n_dst > 0) {
        GRWS_REQUIRE(dst && nbr, "null pointer");
        insert_dst_kernel<<<nblocks(n_dst, 256), 256, 0, st>>>(dst, n_dst, s.keys, s.vals, mask, out_src);
        insert_nbr_kernel<<<nblocks(n_edges, 256), 256, 0, st>>>(nbr, n_edges, s.keys, s.vals, mask, s.cand, s.n_new);
        size_t tmp = s.cub_bytes;
        GRWS_CUDA_TRY(cub::DeviceRadixSort::SortKeys(s.cub_tmp, tmp, s.cand, s.cand_sorted, (int)n_edges, 0, 32, st));
        rank_new_kernel<<<nblocks(n_edges, 256), 256, 0, st>>>(s.cand_sorted, s.n_new, n_dst, s.keys, s.vals, mask, out_src);
        localize_kernel<<<nblocks(n_dst, 128), 128, 0, st>>>(nbr, n_dst, fanout, s.keys, s.vals, mask, out_local, out_row_ptr);
        tmp = s.cub_bytes;
        GRWS_CUDA_TRY(cub::DeviceScan::InclusiveSum(s.cub_tmp, tmp, out_row_ptr, out_row_ptr, (int)(n_dst + 1), st));
    } else {
        GRWS_CUDA_TRY(cudaMemsetAsync(out_row_ptr, 0, 8, st));
    }
    finish_counts_kernel<<<1, 1, 0, st>>>(s.n_new, n_dst, out_row_ptr, out_counts);
    GRWS_CUDA_TRY(cudaGetLastError());
    return GRWS_OK;
}

__attribute__((visibility("default")))
int grws_block_compact(const int32_t *local, const float *w, int64_t n_dst, int fanout, const int64_t *row_ptr,
                       int32_t *out_col, float *out_val, void *stream) {
    GRWS_REQUIRE(n_dst >= 0 && fanout > 0, "bad size");
    if (n_dst == 0) return GRWS_OK;
    GRWS_REQUIRE(local && w && row_ptr, "null pointer");
    compact_kernel<<<nblocks(n_dst, 128), 128, 0, static_cast<cudaStream_t>(stream)>>>(local, w, n_dst, fanout, row_ptr, out_col, out_val);
    GRWS_CUDA_TRY(cudaGetLastError());
    return GRWS_OK;
}

__attribute__((visibility("default")))
int grws_reindex_bcsr(const int32_t *in_cols, void *values, int val_dtype, const int32_t *active_windows,
                      int64_t num_indices, int64_t num_active, int tile_rows, int tile_cols, int32_t *out_cols,
                      void *stream) {
    GRWS_REQUIRE(num_indices >= 0 && num_active >= 0 && tile_rows > 0 && tile_cols > 0, "bad size");
    GRWS_REQUIRE(num_active < 0x7fffffffLL, "too many active windows");
    if (num_indices == 0) return GRWS_OK;
    GRWS_REQUIRE(in_cols && values && out_cols && (num_active == 0 || active_windows), "null pointer");
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    const unsigned nb = nblocks(num_indices, 256);
    if (val_dtype == GRWS_F32)
        reindex_kernel<float><<<nb, 256, 0, st>>>(in_cols, (float *)values, active_windows, num_indices, (int)num_active, tile_rows, tile_cols, out_cols);
    else if (val_dtype == GRWS_F16)
        reindex_kernel<__half><<<nb, 256, 0, st>>>(in_cols, (__half *)values, active_windows, num_indices, (int)num_active, tile_rows, tile_cols, out_cols);
    else if (val_dtype == GRWS_BF16)
        reindex_kernel<__nv_bfloat16><<<nb, 256, 0, st>>>(in_cols, (__nv_bfloat16 *)values, active_windows, num_indices, (int)num_active, tile_rows, tile_cols, out_cols);
    else
        return fail(GRWS_ERR_UNSUPPORTED, "bad value dtype %d", val_dtype);
    GRWS_CUDA_TRY(cudaGetLastError());
    return GRWS_OK;
}

// ---------------------------------------------------------------------------------------------
// All hops of one mini-batch in one call: sample, dedup / reindex, block build, per hop, with
// every buffer sized by a bound that the host knows from (num_seeds, fanouts) alone, so nothing
// is read back between the hops.
// ---------------------------------------------------------------------------------------------
__attribute__((visibility("default")))
int grws_sample_layers_sizes(int64_t num_seeds, const int *fanouts, int num_hops, int64_t pad_to,
                             int64_t *n_dst, int64_t *n_src, int64_t *tiles_bound) {
    GRWS_REQUIRE(num_seeds >= 0 && num_hops >= 1 && num_hops <= 16 && fanouts && pad_to >= 0, "bad argument");
    int64_t d = num_seeds;
    for (int h = 0; h < num_hops; ++h) {
        GRWS_REQUIRE(fanouts[h] > 0 && fanouts[h] <= MAX_FANOUT, "fanout %d outside [1, %d]", fanouts[h], MAX_FANOUT);
        int64_t s = d * (1 + (int64_t)fanouts[h]);
        if (pad_to > 1) s = ceil_div(s, pad_to) * pad_to;
        GRWS_REQUIRE(s < 0x7fffffffLL, "hop %d too large", h);
        if (n_dst) n_dst[h] = d;
        if (n_src) n_src[h] = s;
        if (tiles_bound) tiles_bound[h] = d * fanouts[h] / TILE_COLS + ceil_div(d, TILE_ROWS);
        d = s;
    }
    return GRWS_OK;
}

// builder scratch, defined in bcsr_build.cu
size_t grws_csr_to_bcsr_scratch_bytes(int64_t num_rows, int64_t nnz);
int grws_block_build_count(const int32_t *local, const float *w, int64_t n_dst, int fanout, int64_t num_cols_bound,
                           int64_t *window_offset, void *scratch, size_t scratch_bytes, void *stream);
int grws_csr_to_bcsr_fill(int64_t num_rows, int64_t nnz, const int64_t *window_offset, int64_t num_tiles,
                          int32_t *out_cols, void *out_vals, int val_dtype, void *scratch, size_t scratch_bytes,
                          void *stream);

struct LayersScratch {
    int32_t *nbr, *local, *cnt;
    float *w;
    void *dedup, *build;
    size_t dedup_bytes, build_bytes, total;
};

static int carve_layers(void *base, int64_t num_seeds, const int *fanouts, int num_hops, int64_t pad_to, LayersScratch *out) {
    int64_t n_dst[16], n_src[16];
    if (int st = grws_sample_layers_sizes(num_seeds, fanouts, num_hops, pad_to, n_dst, n_src, nullptr)) return st;
    size_t entries = 1, rows = 1, dedup = 0, build = 0;
    for (int h = 0; h < num_hops; ++h) {
        const size_t e = (size_t)n_dst[h] * fanouts[h];
        if (e > entries) entries = e;
        if ((size_t)n_dst[h] > rows) rows = (size_t)n_dst[h];
        const size_t d = carve_dedup(nullptr, n_dst[h], fanouts[h]).total, b = grws_csr_to_bcsr_scratch_bytes(n_dst[h], (int64_t)e);
        if (d > dedup) dedup = d;
        if (b > build) build = b;
    }
    char *p = static_cast<char *>(base);
    size_t off = 0;
    auto take = [&](size_t bytes) { char *q = p ? p + off : nullptr; off += up256(bytes); return (void *)q; };
    out->nbr = (int32_t *)take(entries * 4);
    out->w = (float *)take(entries * 4);
    out->local = (int32_t *)take(entries * 4);
    out->cnt = (int32_t *)take(rows * 4);
    out->dedup = take(dedup);
    out->build = take(build);
    out->dedup_bytes = dedup;
    out->build_bytes = build;
    out->total = off;
    return GRWS_OK;
}

__attribute__((visibility("default")))
size_t grws_sample_layers_scratch_bytes(int64_t num_seeds, const int *fanouts, int num_hops, int64_t pad_to) {
    LayersScratch s;
    if (carve_layers(nullptr, num_seeds, fanouts, num_hops, pad_to, &s) != GRWS_OK) return 0;
    return s.total;
}

__attribute__((visibility("default")))
int grws_sample_layers(const int64_t *row_ptr, const int32_t *col_idx, const float *values, const int32_t *seeds,
                       int64_t num_seeds, const int *fanouts, int num_hops, uint64_t seed, const uint64_t *seed_dev,
                       int64_t pad_to, int val_dtype, int32_t *const *out_src, int64_t *const *out_window_offset,
                       int32_t *const *out_cols, void *const *out_vals, int64_t *out_counts, void *scratch,
                       size_t scratch_bytes, void *stream) {
    GRWS_REQUIRE(row_ptr && col_idx && (seeds || num_seeds == 0) && out_src && out_window_offset && out_cols && out_vals && scratch,
                 "null pointer");
    GRWS_REQUIRE(val_dtype >= GRWS_F32 && val_dtype <= GRWS_BF16, "bad value dtype %d", val_dtype);
    int64_t n_dst[16], n_src[16], tiles[16];
    if (int st = grws_sample_layers_sizes(num_seeds, fanouts, num_hops, pad_to, n_dst, n_src, tiles)) return st;
    LayersScratch s;
    if (int st = carve_layers(scratch, num_seeds, fanouts, num_hops, pad_to, &s)) return st;
    if (scratch_bytes < s.total) return fail(GRWS_ERR_SCRATCH, "sample_layers scratch too small: %zu < %zu", scratch_bytes, s.total);
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    const int32_t *dst = seeds;
    for (int h = 0; h < num_hops; ++h) {
        const int64_t nd = n_dst[h], f = fanouts[h], n_entries = nd * f, W = ceil_div(nd, (int64_t)TILE_ROWS);
        GRWS_REQUIRE(out_src[h] && out_window_offset[h] && (tiles[h] == 0 || (out_cols[h] && out_vals[h])), "null output of hop %d", h);
        if (nd == 0) {
            GRWS_CUDA_TRY(cudaMemsetAsync(out_window_offset[h], 0, 8, st));
            if (n_src[h] > 0) GRWS_CUDA_TRY(cudaMemsetAsync(out_src[h], 0xff, (size_t)n_src[h] * 4, st));
            if (out_counts) GRWS_CUDA_TRY(cudaMemsetAsync(out_counts + 4 * h, 0, 32, st));
            dst = out_src[h];
            continue;
        }
        // 1. neighbours of every frontier node (padding entries of the frontier, -1, get empty lists)
        sample_hop_kernel<<<nblocks(nd, SAMPLE_WARPS), SAMPLE_WARPS * 32, 0, st>>>(
            row_ptr, col_idx, values, dst, nd, (int)f, seed, seed_dev, (uint32_t)h, s.nbr, s.w, s.cnt);
        // 2. source list = frontier ++ ascending new nodes ++ -1 padding; local id of every neighbour
        DedupScratch d = carve_dedup(s.dedup, nd, (int)f);
        const uint32_t mask = d.slots - 1;
        const int64_t init_n = (int64_t)d.slots > n_src[h] ? (int64_t)d.slots : n_src[h];
        dedup_init_kernel<<<nblocks(init_n, 256) > 1184 ? 1184 : nblocks(init_n, 256), 256, 0, st>>>(
            d.keys, d.vals, d.slots, d.cand, n_entries + 1, d.n_new, out_src[h] + nd, n_src[h] - nd);
        insert_dst_kernel<<<nblocks(nd, 256), 256, 0, st>>>(dst, nd, d.keys, d.vals, mask, out_src[h]);
        insert_nbr_kernel<<<nblocks(n_entries, 256), 256, 0, st>>>(s.nbr, n_entries, d.keys, d.vals, mask, d.cand, d.n_new);
        size_t tmp = d.cub_bytes;
        GRWS_CUDA_TRY(cub::DeviceRadixSort::SortKeys(d.cub_tmp, tmp, d.cand, d.cand_sorted, (int)n_entries, 0, 32, st));
        rank_new_kernel<<<nblocks(n_entries, 256), 256, 0, st>>>(d.cand_sorted, d.n_new, nd, d.keys, d.vals, mask, out_src[h]);
        localize_flat_kernel<<<nblocks(n_entries, 256), 256, 0, st>>>(s.nbr, n_entries, d.keys, d.vals, mask, s.local);
        // 3. the hop's BCSR block straight from the fixed-stride lists
        if (int e = grws_block_build_count(s.local, s.w, nd, (int)f, n_src[h], out_window_offset[h], s.build, s.build_bytes, stream)) return e;
        if (int e = grws_csr_to_bcsr_fill(nd, n_entries, out_window_offset[h], tiles[h], out_cols[h], out_vals[h], val_dtype,
                                          s.build, s.build_bytes, stream)) return e;
        if (out_counts)
            hop_counts_kernel<<<1, 1024, 0, st>>>(d.n_new, dst, nd, s.cnt, out_window_offset[h], W, out_counts + 4 * h);
        GRWS_CUDA_TRY(cudaGetLastError());
        dst = out_src[h];
    }
    return GRWS_OK;
}

}  // extern "C"
