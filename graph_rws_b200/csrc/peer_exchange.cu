// All-gather of row shards over NVLink with this library's own kernels.
//
// The row-partitioned product needs the whole dense operand on every GPU: each rank owns a block of
// rows and reads everybody else's before its local SpMM (the reference is single-GPU and has no
// counterpart).  Every rank keeps a staging block in memory its peers can address (one symmetric
// allocation per rank, mapped into all ranks of the node).  An exchange is two kernels per rank:
//
//   publish : waits until every peer has finished reading the previous exchange, copies this
//             rank's rows into its staging block, then raises its `ready` flag on every rank;
//   pull    : waits until every rank's `ready` flag shows this exchange, copies all staging blocks
//             into the local operand with plain 16-byte loads (peers' blocks over NVLink), then
//             raises its `done` flag on every rank.
//
// The push form does without the second pass: every rank owns an inbox with one slot per rank;
// `push` tells the peers that this rank is done with the previous contents of its inbox, waits for
// the same word from every peer, stores its rows into slot `rank` of every inbox (stores over NVLink
// run at about twice the rate of loads here) and raises `ready`; `arrive` waits for every rank's
// `ready`, after which the inbox IS the gathered operand -- valid until this rank's next exchange.
//
// Nothing but loads, stores and two flags per rank crosses the links: no TMA, no multicast, no
// library kernel is given a peer's memory, and the owner of a block does nothing while it is read.
// All state lives on the device (an exchange counter per rank, flags that hold exchange numbers),
// so a recorded launch sequence can be replayed.  Flags are written with release semantics at
// system scope after a system-wide fence and polled with acquire loads; peers' blocks are read with
// cache-bypassing loads, since the same addresses carry new data in every exchange.  Every wait is
// bounded: a rank whose peers do not show up within `wait_limit` SM clocks records a status, skips
// the copy and returns (the context stays usable; the output of that exchange is undefined).
#include "grws_common.cuh"

namespace grws {
namespace peer {

constexpr int CTRL_READY = 0;        // int32 index of ready[0] in a rank's control block
constexpr int CTRL_DONE = 64;        // int32 index of done[0]
constexpr int MAX_WORLD = 64;
// local state words
constexpr int ST_EPOCH = 0, ST_COUNT_PUBLISH = 1, ST_COUNT_PULL = 2, ST_STATUS = 3;
constexpr int STATUS_PEERS_STILL_READING = 1, STATUS_PEERS_NOT_READY = 2;

__device__ __forceinline__ int ld_acquire_sys(const int *p) {
    int v;
    asm volatile("ld.acquire.sys.global.s32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ void st_release_sys(int *p, int v) {
    asm volatile("st.release.sys.global.s32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}

// waits until flags[p] has reached `target` for every rank p (exchange numbers, compared modulo 2^32)
__device__ __forceinline__ bool wait_flags(const int *flags, int world, int target, long long limit) {
    const long long t0 = clock64();
    for (int p = 0; p < world; ++p) {
        for (uint32_t i = 0;; ++i) {
            if (ld_acquire_sys(flags + p) - target >= 0) break;
            if ((i & 63u) == 63u && clock64() - t0 > limit) return false;
        }
    }
    return true;
}

// ctrl[r] = base of rank r's control block (this rank's own included)
__global__ void __launch_bounds__(256)
publish_kernel(const uint4 *__restrict__ src, int64_t n_vec16, uint4 *__restrict__ stage, int64_t stage_vec16, int *const *ctrl,
               int world, int rank, int *state, long long limit) {
    __shared__ int s_ok;
    const int e = *reinterpret_cast<volatile int *>(state + ST_EPOCH) + 1;      // this exchange
    if (threadIdx.x == 0) {
        // the staging block still holds the previous exchange until every peer has pulled it
        s_ok = wait_flags(ctrl[rank] + CTRL_DONE, world, e - 1, limit) ? 1 : 0;
        if (!s_ok) atomicMax(state + ST_STATUS, STATUS_PEERS_STILL_READING);
    }
    __syncthreads();
    if (s_ok) {
        const int64_t stride = (int64_t)gridDim.x * blockDim.x;
        for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < stage_vec16; i += stride)
            stage[i] = i < n_vec16 ? src[i] : make_uint4(0u, 0u, 0u, 0u);
    }
    // the CTA that finishes last publishes the block
    __threadfence_system();
    __syncthreads();
    if (threadIdx.x == 0) {
        const int arrived = atomicAdd(state + ST_COUNT_PUBLISH, 1);
        if (arrived == (int)gridDim.x - 1) {
            state[ST_COUNT_PUBLISH] = 0;
            __threadfence_system();
            if (*reinterpret_cast<volatile int *>(state + ST_STATUS) == 0)
                for (int p = 0; p < world; ++p) st_release_sys(ctrl[p] + CTRL_READY + rank, e);
            *reinterpret_cast<volatile int *>(state + ST_EPOCH) = e;
        }
    }
}

// stages[r] = base of rank r's staging block; out = [world][stage_vec16]
__global__ void __launch_bounds__(256)
pull_kernel(const uint4 *const *__restrict__ stages, int64_t stage_vec16, uint4 *__restrict__ out, int *const *ctrl, int world,
            int rank, int *state, long long limit) {
    __shared__ int s_ok;
    const int e = *reinterpret_cast<volatile int *>(state + ST_EPOCH);          // the exchange this rank just published
    if (threadIdx.x == 0) {
        s_ok = wait_flags(ctrl[rank] + CTRL_READY, world, e, limit) ? 1 : 0;
        if (!s_ok) atomicMax(state + ST_STATUS, STATUS_PEERS_NOT_READY);
    }
    __syncthreads();
    if (s_ok) {
        const int64_t stride = (int64_t)gridDim.x * blockDim.x;
        for (int k = 0; k < world; ++k) {
            const int p = (rank + 1 + k) % world;                  // every rank starts at another peer; its own block comes last
            const uint4 *src = stages[p];
            uint4 *dst = out + (int64_t)p * stage_vec16;
            int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
            // eight loads in flight per thread: a round trip over NVLink is a few microseconds
            for (; i + 7 * stride < stage_vec16; i += 8 * stride) {
                uint4 v[8];
#pragma unroll
                for (int u = 0; u < 8; ++u) v[u] = __ldcv(src + i + u * stride);
#pragma unroll
                for (int u = 0; u < 8; ++u) dst[i + u * stride] = v[u];
            }
            for (; i < stage_vec16; i += stride) dst[i] = __ldcv(src + i);
        }
    }
    __threadfence_system();
    __syncthreads();
    if (threadIdx.x == 0) {
        const int arrived = atomicAdd(state + ST_COUNT_PULL, 1);
        if (arrived == (int)gridDim.x - 1) {
            state[ST_COUNT_PULL] = 0;
            __threadfence_system();
            // (also after a wait that ran out: the peers must not wait for this rank in turn)
            for (int p = 0; p < world; ++p) st_release_sys(ctrl[p] + CTRL_DONE + rank, e);
        }
    }
}


// inboxes[r] = base of rank r's inbox ([world][stage_vec16]); this rank's rows go into slot `rank` of each
__global__ void __launch_bounds__(256)
push_kernel(const uint4 *__restrict__ src, int64_t n_vec16, uint4 *const *__restrict__ inboxes, int64_t stage_vec16,
            int *const *ctrl, int world, int rank, int *state, long long limit) {
    __shared__ int s_ok;
    const int e = *reinterpret_cast<volatile int *>(state + ST_EPOCH) + 1;      // this exchange
    if (threadIdx.x == 0) {
        // everything queued behind the previous exchange has run: this rank's inbox may be overwritten
        if (blockIdx.x == 0)
            for (int p = 0; p < world; ++p) st_release_sys(ctrl[p] + CTRL_DONE + rank, e - 1);
        s_ok = wait_flags(ctrl[rank] + CTRL_DONE, world, e - 1, limit) ? 1 : 0;
        if (!s_ok) atomicMax(state + ST_STATUS, STATUS_PEERS_STILL_READING);
    }
    __syncthreads();
    if (s_ok) {
        const int64_t stride = (int64_t)gridDim.x * blockDim.x;
        for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < stage_vec16; i += stride) {
            const uint4 v = i < n_vec16 ? src[i] : make_uint4(0u, 0u, 0u, 0u);
            for (int k = 0; k < world; ++k) {
                const int p = (rank + 1 + k) % world;              // every rank starts at another peer
                inboxes[p][(int64_t)rank * stage_vec16 + i] = v;
            }
        }
    }
    __threadfence_system();
    __syncthreads();
    if (threadIdx.x == 0) {
        const int arrived = atomicAdd(state + ST_COUNT_PUBLISH, 1);
        if (arrived == (int)gridDim.x - 1) {
            state[ST_COUNT_PUBLISH] = 0;
            __threadfence_system();
            if (*reinterpret_cast<volatile int *>(state + ST_STATUS) == 0)
                for (int p = 0; p < world; ++p) st_release_sys(ctrl[p] + CTRL_READY + rank, e);
            *reinterpret_cast<volatile int *>(state + ST_EPOCH) = e;
        }
    }
}

// one thread: every rank's rows of this exchange have landed in this rank's inbox
__global__ void arrive_kernel(int *const *ctrl, int world, int rank, int *state, long long limit) {
    const int e = *reinterpret_cast<volatile int *>(state + ST_EPOCH);
    if (!wait_flags(ctrl[rank] + CTRL_READY, world, e, limit)) atomicMax(state + ST_STATUS, STATUS_PEERS_NOT_READY);
}

}  // namespace peer
}  // namespace grws

using namespace grws;

extern "C" {

// Bytes of a rank's control block (ready / done flags of up to 64 ranks) and of its local state.
__attribute__((visibility("default")))
size_t grws_peer_ctrl_bytes(void) { return 2 * peer::MAX_WORLD * sizeof(int); }

__attribute__((visibility("default")))
size_t grws_peer_state_bytes(void) { return 16 * sizeof(int); }

__attribute__((visibility("default")))
int grws_peer_all_gather(const void *local, int64_t local_bytes, void *my_stage, int64_t stage_bytes,
                         const void *const *stages, void *const *ctrl, int world, int rank, void *state, void *out,
                         long long wait_limit, void *stream) {
    GRWS_REQUIRE(world >= 1 && world <= peer::MAX_WORLD && rank >= 0 && rank < world, "bad rank / world");
    GRWS_REQUIRE(local_bytes >= 0 && stage_bytes > 0 && local_bytes <= stage_bytes, "bad size");
    GRWS_REQUIRE(local_bytes % 16 == 0 && stage_bytes % 16 == 0, "sizes must be multiples of 16 bytes");
    GRWS_REQUIRE(my_stage && stages && ctrl && state && out && (local || local_bytes == 0), "null pointer");
    GRWS_REQUIRE(aligned16(local) && aligned16(out) && aligned16(my_stage), "operands must be 16-byte aligned");
    GRWS_REQUIRE(wait_limit > 0, "the wait limit must be positive");
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    int dev = 0, sms = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || sms <= 0)
        sms = 148;
    const int64_t vec = stage_bytes / 16;
    int64_t blocks = ceil_div(vec, (int64_t)256);
    if (blocks > (int64_t)sms * 8) blocks = (int64_t)sms * 8;
    // ctrl / stages are device arrays of pointers (one per rank, this rank's own included)
    peer::publish_kernel<<<(unsigned)blocks, 256, 0, st>>>(static_cast<const uint4 *>(local), local_bytes / 16,
                                                           static_cast<uint4 *>(my_stage), vec, reinterpret_cast<int *const *>(ctrl), world, rank,
                                                           static_cast<int *>(state), wait_limit);
    GRWS_CUDA_TRY(cudaGetLastError());
    peer::pull_kernel<<<(unsigned)blocks, 256, 0, st>>>(reinterpret_cast<const uint4 *const *>(stages), vec, static_cast<uint4 *>(out),
                                                        reinterpret_cast<int *const *>(ctrl), world, rank, static_cast<int *>(state),
                                                        wait_limit);
    GRWS_CUDA_TRY(cudaGetLastError());
    return GRWS_OK;
}

// The push form: `inboxes` is a device array of `world` pointers to the ranks' inboxes
// ([world][stage_bytes] each, symmetric memory); when the call's kernels have run, this rank's inbox
// holds the gathered operand, until the next call.
__attribute__((visibility("default")))
int grws_peer_all_gather_push(const void *local, int64_t local_bytes, int64_t stage_bytes, void *const *inboxes,
                              void *const *ctrl, int world, int rank, void *state, long long wait_limit, void *stream) {
    GRWS_REQUIRE(world >= 1 && world <= peer::MAX_WORLD && rank >= 0 && rank < world, "bad rank / world");
    GRWS_REQUIRE(local_bytes >= 0 && stage_bytes > 0 && local_bytes <= stage_bytes, "bad size");
    GRWS_REQUIRE(local_bytes % 16 == 0 && stage_bytes % 16 == 0, "sizes must be multiples of 16 bytes");
    GRWS_REQUIRE(inboxes && ctrl && state && (local || local_bytes == 0), "null pointer");
    GRWS_REQUIRE(aligned16(local), "operands must be 16-byte aligned");
    GRWS_REQUIRE(wait_limit > 0, "the wait limit must be positive");
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    int dev = 0, sms = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || sms <= 0)
        sms = 148;
    const int64_t vec = stage_bytes / 16;
    int64_t blocks = ceil_div(vec, (int64_t)256);
    if (blocks > (int64_t)sms * 8) blocks = (int64_t)sms * 8;
    peer::push_kernel<<<(unsigned)blocks, 256, 0, st>>>(static_cast<const uint4 *>(local), local_bytes / 16,
                                                        reinterpret_cast<uint4 *const *>(inboxes), vec,
                                                        reinterpret_cast<int *const *>(ctrl), world, rank, static_cast<int *>(state),
                                                        wait_limit);
    GRWS_CUDA_TRY(cudaGetLastError());
    peer::arrive_kernel<<<1, 1, 0, st>>>(reinterpret_cast<int *const *>(ctrl), world, rank, static_cast<int *>(state), wait_limit);
    GRWS_CUDA_TRY(cudaGetLastError());
    return GRWS_OK;
}

}  // extern "C"
