// Feature-row gather from a matrix whose rows are sharded over the GPUs of one node.
//
// The reference keeps features that do not fit one GPU in pinned host memory and gathers the rows
// of a step's input nodes on the CPU (helper/engine.py:135-147, data/data_loader.py:1513-1564).
// Here every GPU holds a contiguous block of rows in memory its peers can address (NVLink 5 through
// NVSwitch: every peer at full bandwidth), and a step's rows are read straight from their owners:
// one warp per row, plain 16-byte loads -- no TMA, no multicast, nothing the owner has to do --
// into a local matrix the first layer's product then reads.  No host round trip (an all-to-all of
// indices and rows needs the split sizes on the host) and nothing but loads crosses the links.
#include "grws_common.cuh"

namespace grws {

constexpr int GATHER_WARPS = 8;

// shards[r] = base of rank r's block (rows r * rows_per_shard ...); ids < 0 give zero rows
__global__ void __launch_bounds__(GATHER_WARPS * 32)
gather_rows_sharded_kernel(const uint4 *const *__restrict__ shards, int world, int64_t rows_per_shard, int row_vec16,
                           int64_t src_stride_vec16, const int32_t *__restrict__ ids, int64_t n, uint4 *__restrict__ out) {
    const int lane = threadIdx.x & 31;
    for (int64_t i = (int64_t)blockIdx.x * GATHER_WARPS + (threadIdx.x >> 5); i < n; i += (int64_t)gridDim.x * GATHER_WARPS) {
        const int32_t id = ids[i];
        uint4 *dst = out + i * row_vec16;
        if (id < 0) {
            for (int c = lane; c < row_vec16; c += 32) dst[c] = make_uint4(0u, 0u, 0u, 0u);
            continue;
        }
        int64_t owner = id / rows_per_shard;
        if (owner >= world) owner = world - 1;
        const uint4 *src = shards[owner] + ((int64_t)id - owner * rows_per_shard) * src_stride_vec16;
        for (int c = lane; c < row_vec16; c += 32) dst[c] = src[c];
    }
}

}  // namespace grws

using namespace grws;

extern "C" __attribute__((visibility("default")))
int grws_gather_rows_sharded(const void *const *shards, int world, int64_t rows_per_shard, int64_t row_bytes,
                             int64_t src_stride_bytes, const int32_t *ids, int64_t n, void *out, void *stream) {
    GRWS_REQUIRE(world >= 1 && rows_per_shard > 0 && n >= 0, "bad size");
    GRWS_REQUIRE(row_bytes > 0 && row_bytes % 16 == 0 && src_stride_bytes % 16 == 0 && src_stride_bytes >= row_bytes,
                 "rows must be multiples of 16 bytes");
    if (n == 0) return GRWS_OK;
    GRWS_REQUIRE(shards && ids && out && aligned16(out), "null or misaligned pointer");
    int64_t blocks = ceil_div(n, (int64_t)GATHER_WARPS);
    if (blocks > 148 * 16) blocks = 148 * 16;
    gather_rows_sharded_kernel<<<(unsigned)blocks, GATHER_WARPS * 32, 0, static_cast<cudaStream_t>(stream)>>>(
        reinterpret_cast<const uint4 *const *>(shards), world, rows_per_shard, (int)(row_bytes / 16), src_stride_bytes / 16,
        ids, n, static_cast<uint4 *>(out));
    GRWS_CUDA_TRY(cudaGetLastError());
    return GRWS_OK;
}
