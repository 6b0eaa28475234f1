// extern "C" surface of libgrws_b200.so: argument checking, kernel selection, error text.
#include "grws_common.cuh"

namespace grws {

char *error_buffer() {
    static thread_local char buf[ERROR_BUFFER_BYTES] = {0};
    return buf;
}

// spmm_warp.cu
int spmm_warp_launch(const int64_t *, const int32_t *, const void *, int, const void *, int64_t,
                     void *, int, int64_t, int64_t, int64_t, int64_t, int64_t, void *, size_t,
                     cudaStream_t);
size_t spmm_warp_scratch_bytes(int64_t num_tiles_bound, int64_t N);
// spmm_tcgen05.cu
bool spmm_tc5_supported(int dtype, int64_t N);
bool spmm_tc5_preferred(int dtype, int64_t N, int64_t num_tiles_bound);
int spmm_tc5_launch(const int64_t *, const int32_t *, const void *, int, const void *, int64_t,
                    void *, int, int64_t, int64_t, int64_t, int64_t, int64_t, void *, size_t,
                    const void *, size_t, cudaStream_t);
size_t spmm_tc5_scratch_bytes(int64_t num_tiles_bound, int64_t N);
size_t spmm_tc5_plan_bytes(int64_t W, int64_t num_tiles_bound, int64_t K, int64_t N);
int spmm_tc5_plan_build(const int64_t *, int64_t, int64_t, int64_t, int64_t, void *, size_t, cudaStream_t);
int spmm_zero_output(void *C, int c_dtype, int64_t ldc, int64_t W, int64_t N, cudaStream_t stream);

}  // namespace grws

using namespace grws;

extern "C" {

__attribute__((visibility("default"))) const char *grws_last_error(void) { return error_buffer(); }

__attribute__((visibility("default"))) int grws_version(void) { return 100; }

__attribute__((visibility("default")))
size_t grws_spmm_scratch_bytes(int64_t num_windows, int64_t num_tiles_bound, int64_t N, int algo) {
    (void)num_windows;
    if (num_tiles_bound < 0 || N <= 0) return 0;
    size_t a = spmm_warp_scratch_bytes(num_tiles_bound, N);
    size_t b = spmm_tc5_scratch_bytes(num_tiles_bound, N);
    if (algo == GRWS_SPMM_WARP_MMA) return a;
    if (algo == GRWS_SPMM_TCGEN05) return b;
    return a > b ? a : b;
}

__attribute__((visibility("default")))
int grws_spmm_resolve_algo(int dtype, int64_t N, int algo) {
    // (for a width below 128 the answer assumes a large product: small ones stay on the warp-MMA kernel)
    if (algo == GRWS_SPMM_AUTO) return spmm_tc5_preferred(dtype, N, INT64_MAX) ? GRWS_SPMM_TCGEN05 : GRWS_SPMM_WARP_MMA;
    return algo;
}

static int spmm_fwd_any(const int64_t *window_offset, const int32_t *cols, const void *vals,
                        int val_dtype, const void *B, int b_dtype, int64_t ldb, void *C, int c_dtype,
                        int64_t ldc, int64_t num_windows, int64_t num_tiles_bound, int64_t K, int64_t N,
                        void *scratch, size_t scratch_bytes, int algo, const void *plan, size_t plan_bytes, void *stream) {
    GRWS_REQUIRE(num_windows >= 0 && num_tiles_bound >= 0 && K >= 0 && N > 0, "negative size");
    if (num_windows == 0) return GRWS_OK;
    GRWS_REQUIRE(window_offset && C, "null pointer");
    GRWS_REQUIRE(num_tiles_bound == 0 || (cols && vals), "null BCSR arrays");
    GRWS_REQUIRE(num_tiles_bound == 0 || K == 0 || B, "null dense operand");
    GRWS_REQUIRE(val_dtype >= GRWS_F32 && val_dtype <= GRWS_BF16, "bad value dtype %d", val_dtype);
    GRWS_REQUIRE(c_dtype >= GRWS_F32 && c_dtype <= GRWS_BF16, "bad output dtype %d", c_dtype);
    if (val_dtype != b_dtype)
        return fail(GRWS_ERR_UNSUPPORTED, "values dtype %d and dense dtype %d must match", val_dtype, b_dtype);
    GRWS_REQUIRE(N % 8 == 0, "N = %lld must be a multiple of 8 (pad the dense operand)", (long long)N);
    GRWS_REQUIRE(ldb >= N && ldc >= N, "leading dimension smaller than N");
    GRWS_REQUIRE((ldb * dtype_bytes(b_dtype)) % 16 == 0 && (ldc * dtype_bytes(c_dtype)) % 16 == 0,
                 "rows of B and C must be 16-byte aligned");
    GRWS_REQUIRE(aligned16(B) && aligned16(C) && aligned16(vals) && aligned16(cols) && aligned16(scratch),
                 "B, C, values, column ids and scratch must be 16-byte aligned");
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    // no tiles, or no dense rows (every column id is then out of range): the product is zero rows
    if (num_tiles_bound == 0 || K == 0) return spmm_zero_output(C, c_dtype, ldc, num_windows, N, st);
    bool tc5 = false;
    if (algo == GRWS_SPMM_TCGEN05) {
        if (!spmm_tc5_supported(val_dtype, N))
            return fail(GRWS_ERR_UNSUPPORTED, "tcgen05 path needs fp16/bf16 and N = 256 or a multiple of 8 up to 128 (N=%lld)", (long long)N);
        tc5 = true;
    } else if (algo == GRWS_SPMM_AUTO) {
        tc5 = spmm_tc5_preferred(val_dtype, N, num_tiles_bound);
    } else if (algo != GRWS_SPMM_WARP_MMA) {
        return fail(GRWS_ERR_INVALID, "unknown algo %d", algo);
    }
    if (tc5)
        return spmm_tc5_launch(window_offset, cols, vals, val_dtype, B, ldb, C, c_dtype, ldc, num_windows,
                               num_tiles_bound, K, N, scratch, scratch_bytes, plan, plan_bytes, st);
    return spmm_warp_launch(window_offset, cols, vals, val_dtype, B, ldb, C, c_dtype, ldc, num_windows,
                            num_tiles_bound, K, N, scratch, scratch_bytes, st);
}

__attribute__((visibility("default")))
int grws_spmm_fwd(const int64_t *window_offset, const int32_t *cols, const void *vals,
                  int val_dtype, const void *B, int b_dtype, int64_t ldb, void *C, int c_dtype,
                  int64_t ldc, int64_t num_windows, int64_t num_tiles_bound, int64_t K, int64_t N,
                  void *scratch, size_t scratch_bytes, int algo, void *stream) {
    return spmm_fwd_any(window_offset, cols, vals, val_dtype, B, b_dtype, ldb, C, c_dtype, ldc, num_windows,
                        num_tiles_bound, K, N, scratch, scratch_bytes, algo, nullptr, 0, stream);
}

// The same product with the CTAs' tile ranges taken from a plan of this graph (grws_spmm_plan_build)
// instead of searched at the start of the launch.  The plan only matters to the tcgen05 kernel; the
// other paths ignore it, and so does that kernel when the plan was made for another shape.
__attribute__((visibility("default")))
int grws_spmm_fwd_planned(const int64_t *window_offset, const int32_t *cols, const void *vals,
                          int val_dtype, const void *B, int b_dtype, int64_t ldb, void *C, int c_dtype,
                          int64_t ldc, int64_t num_windows, int64_t num_tiles_bound, int64_t K, int64_t N,
                          void *scratch, size_t scratch_bytes, int algo, const void *plan, size_t plan_bytes,
                          void *stream) {
    GRWS_REQUIRE(plan == nullptr || aligned16(plan), "the plan must be 16-byte aligned");
    return spmm_fwd_any(window_offset, cols, vals, val_dtype, B, b_dtype, ldb, C, c_dtype, ldc, num_windows,
                        num_tiles_bound, K, N, scratch, scratch_bytes, algo, plan, plan_bytes, stream);
}

__attribute__((visibility("default")))
size_t grws_spmm_plan_bytes(int64_t num_windows, int64_t num_tiles_bound, int64_t K, int64_t N) {
    if (num_windows < 0 || num_tiles_bound < 0 || K < 0 || N <= 0) return 0;
    return spmm_tc5_plan_bytes(num_windows, num_tiles_bound, K, N);
}

__attribute__((visibility("default")))
int grws_spmm_plan_build(const int64_t *window_offset, int64_t num_windows, int64_t num_tiles_bound, int64_t K,
                         int64_t N, void *plan, size_t plan_bytes, void *stream) {
    GRWS_REQUIRE(num_windows >= 0 && num_tiles_bound >= 0 && K >= 0 && N > 0, "negative size");
    GRWS_REQUIRE(window_offset && plan, "null pointer");
    GRWS_REQUIRE(aligned16(plan), "the plan must be 16-byte aligned");
    return spmm_tc5_plan_build(window_offset, num_windows, num_tiles_bound, K, N, plan, plan_bytes,
                               static_cast<cudaStream_t>(stream));
}

}  // extern "C"
