// placeholder until the tcgen05 kernel lands
#include "grws_common.cuh"
namespace grws {
bool spmm_tc5_supported(int, int64_t) { return false; }
size_t spmm_tc5_scratch_bytes(int64_t, int64_t) { return 0; }
int spmm_tc5_launch(const int64_t *, const int32_t *, const void *, int, const void *, int64_t,
                    void *, int, int64_t, int64_t, int64_t, int64_t, int64_t, void *, size_t,
                    cudaStream_t) { return fail(GRWS_ERR_UNSUPPORTED, "tcgen05 path not built"); }
}
