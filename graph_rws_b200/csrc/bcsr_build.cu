// Device-side BCSR construction.
//
//   CSR -> BCSR: the layout contract of csr_to_bcsr_cpu (core/wrapper/convert_wrapper.cpp:27-180),
//   built with one stable radix sort instead of per-window std::sort on the host: every edge
//   gets the key (window, column, row-in-window); sorted, equal (window, column) runs become one
//   column slot, slot / 8 is the tile, and the last duplicate of a (row, column) pair wins
//   (convert_wrapper.cpp:174).
//
//   BCSR -> transposed CSR: extracts the non-zero entries of the tiles as (column, row, value)
//   so that the transposed adjacency can be built once, cached and multiplied with the forward
//   kernel; this replaces the per-call atomic scatter of spmm_bcsr_transpose_atomic_kernel
//   (core/include/spmm_tc.cuh:211-270).
//
// cub::DeviceRadixSort / DeviceScan (CUDA toolkit) do the sort and the prefix sums; this is
// graph preparation, not the per-step hot loop.
#include <cub/cub.cuh>

#include "grws_common.cuh"

namespace grws {

constexpr int ROW_BITS = 4;   // row inside a 16-row window
// Key of an entry that does not exist (a padding slot of a fixed-stride neighbour list, the unused
// tail of a CSR array sized by a bound).  Real keys are below it (fewer than 2^28 windows), so such
// entries sort to the end; they open no column slot and write nothing.
constexpr uint64_t INVALID_KEY = ~0ull;

static inline size_t align_up(size_t x, size_t a = 256) { return (x + a - 1) / a * a; }

// layout of the scratch buffer shared by the count and fill phases of csr_to_bcsr
struct BuildScratch {
    uint64_t *keys_a, *keys_b;
    float *vals_a, *vals_b;
    int32_t *flags;         // per sorted entry: 1 when it opens a new (window, column) run
    int32_t *uidx;          // per sorted entry: 1 + global index of its (window, column) slot (inclusive scan of flags)
    int32_t *nuniq;         // [W+2] unique columns per window
    int32_t *ufirst;        // [W+2] exclusive scan of nuniq
    int64_t *tiles;         // [W+2] tiles per window, shifted by one
    int32_t *col_bits;      // bits of the column field of the keys (the count phase leaves it for the fill phase)
    void *cub_tmp;
    size_t cub_bytes;
    size_t total;
};

static size_t cub_temp_bytes(int64_t nnz, int64_t W) {
    size_t s1 = 0, s2 = 0, s3 = 0;
    cub::DeviceRadixSort::SortPairs(nullptr, s1, (const uint64_t *)nullptr, (uint64_t *)nullptr,
                                    (const float *)nullptr, (float *)nullptr, (int)nnz, 0, 64);
    cub::DeviceScan::InclusiveSum(nullptr, s2, (const int32_t *)nullptr, (int32_t *)nullptr, (int)nnz);
    cub::DeviceScan::InclusiveSum(nullptr, s3, (const int64_t *)nullptr, (int64_t *)nullptr, (int)(W + 1));
    size_t m = s1 > s2 ? s1 : s2;
    return m > s3 ? m : s3;
}

static BuildScratch carve(void *base, int64_t nnz, int64_t W) {
    BuildScratch s;
    char *p = static_cast<char *>(base);
    size_t off = 0;
    auto take = [&](size_t bytes) { char *q = p ? p + off : nullptr; off += align_up(bytes); return (void *)q; };
    const size_t n = (size_t)(nnz > 0 ? nnz : 1);
    s.keys_a = (uint64_t *)take(n * 8);
    s.keys_b = (uint64_t *)take(n * 8);
    s.vals_a = (float *)take(n * 4);
    s.vals_b = (float *)take(n * 4);
    s.flags = (int32_t *)take(n * 4);
    s.uidx = (int32_t *)take(n * 4);
    s.nuniq = (int32_t *)take((size_t)(W + 2) * 4);
    s.ufirst = (int32_t *)take((size_t)(W + 2) * 4);
    s.tiles = (int64_t *)take((size_t)(W + 2) * 8);
    s.col_bits = (int32_t *)take(64);
    s.cub_bytes = cub_temp_bytes(nnz, W);
    s.cub_tmp = take(s.cub_bytes);
    s.total = off;
    return s;
}

// Sort key of an entry: window | column | row-in-window.  The column field has as many bits as the
// caller's bound on the column ids needs (32 without a bound), so that the radix sort, which runs one
// pass per 8 key bits, has fewer passes to make: the blocks of a sampled step have 2^13 windows and 2^21
// columns at most, 38 key bits instead of 49.  A column field of b bits holds ids below 2^b - 1 only,
// which keeps the invalid key (all ones) apart from every real key within the sorted bits.
__host__ __device__ __forceinline__ uint64_t make_key(int64_t row, int32_t col, int col_bits) {
    return ((uint64_t)(row / TILE_ROWS) << (col_bits + ROW_BITS)) | ((uint64_t)(uint32_t)col << ROW_BITS) | (uint64_t)(row % TILE_ROWS);
}

static int column_bits(int64_t num_cols_bound) {
    if (num_cols_bound <= 0 || num_cols_bound >= (1LL << 31)) return 32;
    int b = 0;
    for (int64_t x = num_cols_bound; x > 0; x >>= 1) ++b;      // ids < bound <= 2^b - 1
    return b;
}

__global__ void make_keys_kernel(int64_t num_rows, const int64_t *__restrict__ row_ptr,
                                 const int32_t *__restrict__ col_idx, uint64_t *__restrict__ keys, int col_bits) {
    // one warp per row
    const int64_t row = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    const int lane = threadIdx.x & 31;
    if (row >= num_rows) return;
    const int64_t e0 = row_ptr[row], e1 = row_ptr[row + 1];
    for (int64_t e = e0 + lane; e < e1; e += 32)
        keys[e] = make_key(row, col_idx[e], col_bits);
}

// keys of a hop's fixed-stride neighbour lists: entry (row i, slot j) holds local column id
// local[i * fanout + j], or -1 when the slot is empty
__global__ void make_keys_lists_kernel(int64_t n_entries, int fanout, const int32_t *__restrict__ local,
                                       uint64_t *__restrict__ keys, int col_bits) {
    const int64_t e = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (e >= n_entries) return;
    const int32_t c = local[e];
    const int64_t row = e / fanout;
    keys[e] = c < 0 ? INVALID_KEY : make_key(row, c, col_bits);
}

__global__ void head_flags_kernel(int64_t nnz, const uint64_t *__restrict__ keys,
                                  int32_t *__restrict__ flags, int32_t *__restrict__ nuniq, int col_bits,
                                  int32_t *__restrict__ col_bits_out) {
    const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    bool head = false;
    uint64_t window = 0;
    if (i < nnz) {
        if (i == 0) *col_bits_out = col_bits;              // the fill phase decodes the keys with it
        const uint64_t key = keys[i];
        if (key != INVALID_KEY) {
            const uint64_t k = key >> ROW_BITS;
            head = (i == 0) || ((keys[i - 1] >> ROW_BITS) != k);
            window = k >> col_bits;
        }
        flags[i] = head ? 1 : 0;
    }
    // The keys are sorted, so the heads a warp sees belong to one or two windows almost always: one
    // atomic per window and warp instead of one per head (a window's counter otherwise takes
    // hundreds of atomics from neighbouring threads).
    const unsigned heads = __ballot_sync(0xffffffffu, head);
    if (head) {
        const unsigned same = __match_any_sync(heads, window);
        if ((threadIdx.x & 31) == __ffs(same) - 1) atomicAdd(nuniq + window, __popc(same));
    }
}

__global__ void tiles_kernel(int64_t W, const int32_t *__restrict__ nuniq, int64_t *__restrict__ tiles) {
    const int64_t w = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (w > W) return;
    tiles[w] = (w == 0) ? 0 : (nuniq[w - 1] + TILE_COLS - 1) / TILE_COLS;   // shifted by one for an inclusive scan
}

template <typename T> __device__ __forceinline__ T from_float(float v);
template <> __device__ __forceinline__ float from_float<float>(float v) { return v; }
template <> __device__ __forceinline__ __half from_float<__half>(float v) { return __float2half_rn(v); }
template <> __device__ __forceinline__ __nv_bfloat16 from_float<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }

template <typename T>
__global__ void fill_kernel(int64_t nnz, const uint64_t *__restrict__ keys, const float *__restrict__ vals,
                            const int32_t *__restrict__ uidx, const int32_t *__restrict__ ufirst,
                            const int64_t *__restrict__ window_offset, int32_t *__restrict__ out_cols,
                            T *__restrict__ out_vals, const int32_t *__restrict__ col_bits_in) {
    const int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= nnz) return;
    const uint64_t key = keys[i];
    if (key == INVALID_KEY) return;
    if (i + 1 < nnz && keys[i + 1] == key) return;          // an identical (row, column) follows: it wins
    const int col_bits = *col_bits_in;
    const int64_t w = (int64_t)(key >> (col_bits + ROW_BITS));
    const int32_t col = (int32_t)((key >> ROW_BITS) & ((1ull << col_bits) - 1ull));
    const int r = (int)(key & (TILE_ROWS - 1));
    const int32_t slot = uidx[i] - 1 - ufirst[w];
    const int64_t tile = window_offset[w] + slot / TILE_COLS;
    const int ic = slot % TILE_COLS;
    out_cols[tile * TILE_COLS + ic] = col;                    // every entry of the run writes the same id
    out_vals[tile * TILE_ELEMS + r * TILE_COLS + ic] = from_float<T>(vals[i]);
}

__global__ void fill_i32_kernel(int32_t *p, int64_t n, int32_t v) {
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x) p[i] = v;
}

static inline unsigned blocks_for(int64_t n, int threads) {
    int64_t b = ceil_div(n > 0 ? n : 1, threads);
    return (unsigned)(b > 0x7fffffff ? 0x7fffffff : b);
}

// ------------------------------- BCSR -> transposed CSR -------------------------------------
template <typename T> __device__ __forceinline__ float to_float(T v);
template <> __device__ __forceinline__ float to_float<float>(float v) { return v; }
template <> __device__ __forceinline__ float to_float<__half>(__half v) { return __half2float(v); }
template <> __device__ __forceinline__ float to_float<__nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }

// one thread per tile element; MODE 0 counts entries per column, MODE 1 scatters them
template <typename T, int MODE>
__global__ void transpose_entries_kernel(int64_t W, const int64_t *__restrict__ window_offset,
                                         const int32_t *__restrict__ cols, const T *__restrict__ vals,
                                         int64_t num_cols, int64_t *__restrict__ counts_or_cursor,
                                         int32_t *__restrict__ out_col, float *__restrict__ out_val) {
    // one warp per (window, tile): lane handles 4 elements
    const int64_t w = blockIdx.x;
    const int64_t t0 = window_offset[w], t1 = window_offset[w + 1];
    for (int64_t tile = t0 + (threadIdx.x >> 5); tile < t1; tile += blockDim.x >> 5) {
        const int lane = threadIdx.x & 31;
#pragma unroll
        for (int q = 0; q < 4; ++q) {
            const int el = lane + 32 * q;                // element of the 16x8 tile
            const int r = el >> 3, c = el & 7;
            const int32_t col = cols[tile * TILE_COLS + c];
            if (col < 0 || col >= num_cols) continue;
            const float v = to_float<T>(vals[tile * TILE_ELEMS + el]);
            if (v == 0.0f) continue;
            if (MODE == 0) {
                atomicAdd(reinterpret_cast<unsigned long long *>(counts_or_cursor + col + 1), 1ull);
            } else {
                const int64_t pos = (int64_t)atomicAdd(reinterpret_cast<unsigned long long *>(counts_or_cursor + col), 1ull);
                out_col[pos] = (int32_t)(w * TILE_ROWS + r);
                out_val[pos] = v;
            }
        }
    }
}

// BCSR -> CSR (not transposed): one warp per window, lane r < 16 walks row r of every tile in
// order.  Column ids are ascending inside a window, so every CSR row comes out ascending.
// MODE 0 counts the non-zero entries of each row, MODE 1 writes them.
template <typename T, int MODE>
__global__ void bcsr_rows_kernel(int64_t W, int64_t num_rows, const int64_t *__restrict__ window_offset,
                                 const int32_t *__restrict__ cols, const T *__restrict__ vals,
                                 int64_t *__restrict__ row_ptr, int32_t *__restrict__ out_col,
                                 float *__restrict__ out_val) {
    const int64_t w = ((int64_t)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    const int r = threadIdx.x & 31;
    if (w >= W || r >= TILE_ROWS) return;
    const int64_t row = w * TILE_ROWS + r;
    if (row >= num_rows) return;
    int64_t o = (MODE == 1) ? row_ptr[row] : 0;
    for (int64_t t = window_offset[w]; t < window_offset[w + 1]; ++t) {
#pragma unroll
        for (int c = 0; c < TILE_COLS; ++c) {
            const int32_t col = cols[t * TILE_COLS + c];
            const float v = to_float<T>(vals[t * TILE_ELEMS + r * TILE_COLS + c]);
            if (col < 0 || v == 0.0f) continue;
            if (MODE == 1) { out_col[o] = col; out_val[o] = v; }
            ++o;
        }
    }
    if (MODE == 0) row_ptr[row + 1] = o;
}

}  // namespace grws

using namespace grws;

// Second half of the count phase, shared by the CSR and the neighbour-list front ends: sorts the
// keys in s.keys_a (values alongside), flags the first entry of every (window, column) run and
// turns the unique-column counts into window_offset.
static int count_from_keys(const BuildScratch &s, int64_t nnz, int64_t W, const float *values,
                           int64_t *window_offset, int col_bits, cudaStream_t st) {
    GRWS_CUDA_TRY(cudaMemsetAsync(s.nuniq, 0, (size_t)(W + 2) * 4, st));
    if (nnz > 0) {
        size_t tmp = s.cub_bytes;
        // only the bits a key can use are sorted; the invalid key is all ones there too, so it
        // still sorts behind every real key (no column id fills its field with ones)
        int end_bit = col_bits + ROW_BITS;
        for (int64_t x = W; x > 0; x >>= 1) ++end_bit;
        if (end_bit > 64) end_bit = 64;
        GRWS_CUDA_TRY(cub::DeviceRadixSort::SortPairs(s.cub_tmp, tmp, s.keys_a, s.keys_b, values, s.vals_b,
                                                      (int)nnz, 0, end_bit, st));
        head_flags_kernel<<<blocks_for(nnz, 256), 256, 0, st>>>(nnz, s.keys_b, s.flags, s.nuniq, col_bits, s.col_bits);
        tmp = s.cub_bytes;
        GRWS_CUDA_TRY(cub::DeviceScan::InclusiveSum(s.cub_tmp, tmp, s.flags, s.uidx, (int)nnz, st));
    }
    tiles_kernel<<<blocks_for(W + 1, 256), 256, 0, st>>>(W, s.nuniq, s.tiles);
    size_t tmp = s.cub_bytes;
    GRWS_CUDA_TRY(cub::DeviceScan::InclusiveSum(s.cub_tmp, tmp, s.tiles, window_offset, (int)(W + 1), st));
    tmp = s.cub_bytes;
    GRWS_CUDA_TRY(cub::DeviceScan::ExclusiveSum(s.cub_tmp, tmp, s.nuniq, s.ufirst, (int)(W + 1), st));
    GRWS_CUDA_TRY(cudaGetLastError());
    return GRWS_OK;
}

template <typename T>
static int transpose_count(const int64_t *wo, const int32_t *cols, const void *vals, int64_t W, int64_t num_cols,
                           int64_t *row_ptr_t, void *scratch, cudaStream_t st) {
    int64_t *counts = static_cast<int64_t *>(scratch);
    void *cub_tmp = static_cast<char *>(scratch) + align_up((size_t)(num_cols + 1) * 8);
    size_t tmp = 0;
    cub::DeviceScan::InclusiveSum(nullptr, tmp, (const int64_t *)nullptr, (int64_t *)nullptr, (int)(num_cols + 1));
    GRWS_CUDA_TRY(cudaMemsetAsync(counts, 0, (size_t)(num_cols + 1) * 8, st));
    if (W > 0)
        transpose_entries_kernel<T, 0><<<(unsigned)W, 128, 0, st>>>(W, wo, cols, (const T *)vals, num_cols, counts, nullptr, nullptr);
    GRWS_CUDA_TRY(cub::DeviceScan::InclusiveSum(cub_tmp, tmp, counts, row_ptr_t, (int)(num_cols + 1), st));
    GRWS_CUDA_TRY(cudaGetLastError());
    return GRWS_OK;
}


extern "C" {

__attribute__((visibility("default")))
size_t grws_csr_to_bcsr_scratch_bytes(int64_t num_rows, int64_t nnz) {
    if (num_rows < 0 || nnz < 0) return 0;
    return carve(nullptr, nnz, ceil_div(num_rows, TILE_ROWS)).total;
}

static int csr_count(int64_t num_rows, const int64_t *row_ptr, const int32_t *col_idx, const float *values,
                     int64_t nnz, bool nnz_is_bound, int64_t num_cols_bound, int64_t *window_offset, void *scratch,
                     size_t scratch_bytes, void *stream) {
    GRWS_REQUIRE(num_rows >= 0 && nnz >= 0, "negative size");
    GRWS_REQUIRE(nnz < 0x7fffffffLL, "csr_to_bcsr handles fewer than 2^31 entries");
    const int64_t W = ceil_div(num_rows, TILE_ROWS);
    GRWS_REQUIRE(W < (1LL << 28), "too many windows");
    GRWS_REQUIRE(row_ptr && window_offset && scratch, "null pointer");
    GRWS_REQUIRE(nnz == 0 || (col_idx && values), "null CSR arrays");
    BuildScratch s = carve(scratch, nnz, W);
    if (scratch_bytes < s.total) return fail(GRWS_ERR_SCRATCH, "csr_to_bcsr scratch too small: %zu < %zu", scratch_bytes, s.total);
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    const int col_bits = column_bits(num_cols_bound);
    if (nnz > 0) {
        // entries of the arrays past row_ptr[num_rows] (a CSR sized by a bound) keep the invalid key
        if (nnz_is_bound) GRWS_CUDA_TRY(cudaMemsetAsync(s.keys_a, 0xff, (size_t)nnz * 8, st));
        make_keys_kernel<<<blocks_for(num_rows * 32, 256), 256, 0, st>>>(num_rows, row_ptr, col_idx, s.keys_a, col_bits);
    }
    return count_from_keys(s, nnz, W, values, window_offset, col_bits, st);
}

__attribute__((visibility("default")))
int grws_csr_to_bcsr_count(int64_t num_rows, const int64_t *row_ptr, const int32_t *col_idx,
                           const float *values, int64_t nnz, int64_t *window_offset, void *scratch,
                           size_t scratch_bytes, void *stream) {
    return csr_count(num_rows, row_ptr, col_idx, values, nnz, false, 0, window_offset, scratch, scratch_bytes, stream);
}

__attribute__((visibility("default")))
int grws_csr_to_bcsr_count_bounded(int64_t num_rows, const int64_t *row_ptr, const int32_t *col_idx,
                                   const float *values, int64_t nnz_bound, int64_t num_cols_bound,
                                   int64_t *window_offset, void *scratch, size_t scratch_bytes, void *stream) {
    GRWS_REQUIRE(num_cols_bound >= 0, "negative size");
    return csr_count(num_rows, row_ptr, col_idx, values, nnz_bound, true, num_cols_bound, window_offset, scratch, scratch_bytes,
                     stream);
}

__attribute__((visibility("default")))
int grws_block_build_count(const int32_t *local, const float *w, int64_t n_dst, int fanout, int64_t num_cols_bound,
                           int64_t *window_offset, void *scratch, size_t scratch_bytes, void *stream) {
    GRWS_REQUIRE(n_dst >= 0 && fanout > 0 && num_cols_bound >= 0, "bad size");
    const int64_t n_entries = n_dst * fanout;
    GRWS_REQUIRE(n_entries < 0x7fffffffLL, "hop too large");
    const int64_t W = ceil_div(n_dst, TILE_ROWS);
    GRWS_REQUIRE(window_offset && scratch && (n_entries == 0 || (local && w)), "null pointer");
    BuildScratch s = carve(scratch, n_entries, W);
    if (scratch_bytes < s.total) return fail(GRWS_ERR_SCRATCH, "block build scratch too small: %zu < %zu", scratch_bytes, s.total);
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    const int col_bits = column_bits(num_cols_bound);
    if (n_entries > 0)
        make_keys_lists_kernel<<<blocks_for(n_entries, 256), 256, 0, st>>>(n_entries, fanout, local, s.keys_a, col_bits);
    return count_from_keys(s, n_entries, W, w, window_offset, col_bits, st);
}

__attribute__((visibility("default")))
int grws_csr_to_bcsr_fill(int64_t num_rows, int64_t nnz, const int64_t *window_offset, int64_t num_tiles,
                          int32_t *out_cols, void *out_vals, int val_dtype, void *scratch,
                          size_t scratch_bytes, void *stream) {
    GRWS_REQUIRE(num_rows >= 0 && nnz >= 0 && num_tiles >= 0, "negative size");
    const int64_t W = ceil_div(num_rows, TILE_ROWS);
    BuildScratch s = carve(scratch, nnz, W);
    if (scratch_bytes < s.total) return fail(GRWS_ERR_SCRATCH, "csr_to_bcsr scratch too small");
    if (num_tiles == 0) return GRWS_OK;
    GRWS_REQUIRE(window_offset && out_cols && out_vals && scratch, "null pointer");
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    const unsigned fill_blocks = blocks_for(num_tiles * TILE_COLS, 256);
    fill_i32_kernel<<<fill_blocks > 4096 ? 4096 : fill_blocks, 256, 0, st>>>(out_cols, num_tiles * TILE_COLS, -1);
    GRWS_CUDA_TRY(cudaMemsetAsync(out_vals, 0, (size_t)num_tiles * TILE_ELEMS * dtype_bytes(val_dtype), st));
    if (nnz > 0) {
        const unsigned nb = blocks_for(nnz, 256);
        if (val_dtype == GRWS_F32)
            fill_kernel<float><<<nb, 256, 0, st>>>(nnz, s.keys_b, s.vals_b, s.uidx, s.ufirst, window_offset, out_cols, (float *)out_vals, s.col_bits);
        else if (val_dtype == GRWS_F16)
            fill_kernel<__half><<<nb, 256, 0, st>>>(nnz, s.keys_b, s.vals_b, s.uidx, s.ufirst, window_offset, out_cols, (__half *)out_vals, s.col_bits);
        else if (val_dtype == GRWS_BF16)
            fill_kernel<__nv_bfloat16><<<nb, 256, 0, st>>>(nnz, s.keys_b, s.vals_b, s.uidx, s.ufirst, window_offset, out_cols, (__nv_bfloat16 *)out_vals, s.col_bits);
        else
            return fail(GRWS_ERR_UNSUPPORTED, "bad value dtype %d", val_dtype);
    }
    GRWS_CUDA_TRY(cudaGetLastError());
    return GRWS_OK;
}

// counts[0] = 0, counts[c + 1] = non-zero entries in column c; then inclusive scan -> row_ptr of A^T
__attribute__((visibility("default")))
size_t grws_bcsr_transpose_scratch_bytes(int64_t num_cols) {
    size_t s3 = 0;
    cub::DeviceScan::InclusiveSum(nullptr, s3, (const int64_t *)nullptr, (int64_t *)nullptr, (int)(num_cols + 1));
    return align_up((size_t)(num_cols + 1) * 8) + align_up(s3);
}

__attribute__((visibility("default")))
int grws_bcsr_transpose_count(const int64_t *window_offset, const int32_t *cols, const void *vals, int val_dtype,
                              int64_t num_windows, int64_t num_cols, int64_t *row_ptr_t, void *scratch,
                              size_t scratch_bytes, void *stream) {
    GRWS_REQUIRE(num_windows >= 0 && num_cols >= 0, "negative size");
    GRWS_REQUIRE(num_windows < 0x7fffffffLL && num_cols < 0x7fffffffLL, "size beyond 2^31");
    GRWS_REQUIRE(window_offset && row_ptr_t && scratch, "null pointer");
    if (scratch_bytes < grws_bcsr_transpose_scratch_bytes(num_cols)) return fail(GRWS_ERR_SCRATCH, "transpose scratch too small");
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    switch (val_dtype) {
        case GRWS_F32: return transpose_count<float>(window_offset, cols, vals, num_windows, num_cols, row_ptr_t, scratch, st);
        case GRWS_F16: return transpose_count<__half>(window_offset, cols, vals, num_windows, num_cols, row_ptr_t, scratch, st);
        case GRWS_BF16: return transpose_count<__nv_bfloat16>(window_offset, cols, vals, num_windows, num_cols, row_ptr_t, scratch, st);
    }
    return fail(GRWS_ERR_UNSUPPORTED, "bad value dtype %d", val_dtype);
}

// scatters the entries; `scratch` must still hold what the count call left (it is reused as cursors)
__attribute__((visibility("default")))
int grws_bcsr_transpose_fill(const int64_t *window_offset, const int32_t *cols, const void *vals, int val_dtype,
                             int64_t num_windows, int64_t num_cols, const int64_t *row_ptr_t, int32_t *out_col,
                             float *out_val, void *scratch, size_t scratch_bytes, void *stream) {
    GRWS_REQUIRE(num_windows >= 0 && num_cols >= 0, "negative size");
    GRWS_REQUIRE(window_offset && row_ptr_t && scratch, "null pointer");
    if (scratch_bytes < grws_bcsr_transpose_scratch_bytes(num_cols)) return fail(GRWS_ERR_SCRATCH, "transpose scratch too small");
    if (num_windows == 0) return GRWS_OK;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    int64_t *cursor = static_cast<int64_t *>(scratch);
    GRWS_CUDA_TRY(cudaMemcpyAsync(cursor, row_ptr_t, (size_t)(num_cols + 1) * 8, cudaMemcpyDeviceToDevice, st));
    const unsigned W = (unsigned)num_windows;
    if (val_dtype == GRWS_F32)
        transpose_entries_kernel<float, 1><<<W, 128, 0, st>>>(num_windows, window_offset, cols, (const float *)vals, num_cols, cursor, out_col, out_val);
    else if (val_dtype == GRWS_F16)
        transpose_entries_kernel<__half, 1><<<W, 128, 0, st>>>(num_windows, window_offset, cols, (const __half *)vals, num_cols, cursor, out_col, out_val);
    else if (val_dtype == GRWS_BF16)
        transpose_entries_kernel<__nv_bfloat16, 1><<<W, 128, 0, st>>>(num_windows, window_offset, cols, (const __nv_bfloat16 *)vals, num_cols, cursor, out_col, out_val);
    else
        return fail(GRWS_ERR_UNSUPPORTED, "bad value dtype %d", val_dtype);
    GRWS_CUDA_TRY(cudaGetLastError());
    return GRWS_OK;
}

// BCSR -> CSR of the same matrix, two phases like the other builders.
__attribute__((visibility("default")))
size_t grws_bcsr_to_csr_scratch_bytes(int64_t num_rows) {
    size_t s3 = 0;
    cub::DeviceScan::InclusiveSum(nullptr, s3, (const int64_t *)nullptr, (int64_t *)nullptr, (int)(num_rows + 1));
    return align_up(s3);
}

__attribute__((visibility("default")))
int grws_bcsr_to_csr_count(const int64_t *window_offset, const int32_t *cols, const void *vals, int val_dtype,
                           int64_t num_windows, int64_t num_rows, int64_t *row_ptr, void *scratch,
                           size_t scratch_bytes, void *stream) {
    GRWS_REQUIRE(num_windows >= 0 && num_rows >= 0 && num_rows <= num_windows * TILE_ROWS, "bad size");
    GRWS_REQUIRE(num_rows < 0x7fffffffLL, "size beyond 2^31");
    GRWS_REQUIRE(window_offset && row_ptr && scratch, "null pointer");
    if (scratch_bytes < grws_bcsr_to_csr_scratch_bytes(num_rows)) return fail(GRWS_ERR_SCRATCH, "bcsr_to_csr scratch too small");
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    GRWS_CUDA_TRY(cudaMemsetAsync(row_ptr, 0, (size_t)(num_rows + 1) * 8, st));
    if (num_windows > 0) {
        const unsigned nb = blocks_for(num_windows * 32, 256);
        if (val_dtype == GRWS_F32) bcsr_rows_kernel<float, 0><<<nb, 256, 0, st>>>(num_windows, num_rows, window_offset, cols, (const float *)vals, row_ptr, nullptr, nullptr);
        else if (val_dtype == GRWS_F16) bcsr_rows_kernel<__half, 0><<<nb, 256, 0, st>>>(num_windows, num_rows, window_offset, cols, (const __half *)vals, row_ptr, nullptr, nullptr);
        else if (val_dtype == GRWS_BF16) bcsr_rows_kernel<__nv_bfloat16, 0><<<nb, 256, 0, st>>>(num_windows, num_rows, window_offset, cols, (const __nv_bfloat16 *)vals, row_ptr, nullptr, nullptr);
        else return fail(GRWS_ERR_UNSUPPORTED, "bad value dtype %d", val_dtype);
    }
    size_t tmp = scratch_bytes;
    GRWS_CUDA_TRY(cub::DeviceScan::InclusiveSum(scratch, tmp, row_ptr, row_ptr, (int)(num_rows + 1), st));
    GRWS_CUDA_TRY(cudaGetLastError());
    return GRWS_OK;
}

__attribute__((visibility("default")))
int grws_bcsr_to_csr_fill(const int64_t *window_offset, const int32_t *cols, const void *vals, int val_dtype,
                          int64_t num_windows, int64_t num_rows, const int64_t *row_ptr, int32_t *out_col,
                          float *out_val, void *stream) {
    GRWS_REQUIRE(num_windows >= 0 && num_rows >= 0, "bad size");
    if (num_windows == 0) return GRWS_OK;
    GRWS_REQUIRE(window_offset && row_ptr, "null pointer");
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    int64_t *rp = const_cast<int64_t *>(row_ptr);
    const unsigned nb = blocks_for(num_windows * 32, 256);
    if (val_dtype == GRWS_F32) bcsr_rows_kernel<float, 1><<<nb, 256, 0, st>>>(num_windows, num_rows, window_offset, cols, (const float *)vals, rp, out_col, out_val);
    else if (val_dtype == GRWS_F16) bcsr_rows_kernel<__half, 1><<<nb, 256, 0, st>>>(num_windows, num_rows, window_offset, cols, (const __half *)vals, rp, out_col, out_val);
    else if (val_dtype == GRWS_BF16) bcsr_rows_kernel<__nv_bfloat16, 1><<<nb, 256, 0, st>>>(num_windows, num_rows, window_offset, cols, (const __nv_bfloat16 *)vals, rp, out_col, out_val);
    else return fail(GRWS_ERR_UNSUPPORTED, "bad value dtype %d", val_dtype);
    GRWS_CUDA_TRY(cudaGetLastError());
    return GRWS_OK;
}

}  // extern "C"
