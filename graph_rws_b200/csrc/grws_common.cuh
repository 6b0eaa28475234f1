// Shared device/host helpers of libgrws_b200.so (sm_100a only).
#pragma once

#include <cuda_runtime.h>
#include <cuda_fp16.h>
#include <cuda_bf16.h>
#include <stdint.h>
#include <stdio.h>
#include <stdarg.h>

#include "../../include/grws_b200.h"

namespace grws {

constexpr int TILE_ROWS = GRWS_TILE_ROWS;   // rows of a window / of a tile
constexpr int TILE_COLS = GRWS_TILE_COLS;   // column slots of a tile
constexpr int TILE_ELEMS = TILE_ROWS * TILE_COLS;

// ---------------------------------------------------------------------------------------------
// error reporting: one message per host thread, returned by grws_last_error()
// ---------------------------------------------------------------------------------------------
char *error_buffer();
constexpr size_t ERROR_BUFFER_BYTES = 512;

inline int fail(int status, const char *fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(error_buffer(), ERROR_BUFFER_BYTES, fmt, ap);
    va_end(ap);
    return status;
}

#define GRWS_CUDA_TRY(call)                                                                     \
    do {                                                                                        \
        cudaError_t e__ = (call);                                                               \
        if (e__ != cudaSuccess)                                                                 \
            return ::grws::fail(GRWS_ERR_CUDA, "%s failed: %s", #call, cudaGetErrorString(e__)); \
    } while (0)

#define GRWS_REQUIRE(cond, ...)                                                                 \
    do {                                                                                        \
        if (!(cond)) return ::grws::fail(GRWS_ERR_INVALID, __VA_ARGS__);                        \
    } while (0)

inline size_t dtype_bytes(int dt) { return dt == GRWS_F32 ? 4 : 2; }
inline bool aligned16(const void *p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }
inline int64_t ceil_div(int64_t a, int64_t b) { return (a + b - 1) / b; }

// ---------------------------------------------------------------------------------------------
// work partition of one SpMM over the global tile array
//
// The tile array [0, T) is cut at multiples of `chunk`; a cut that falls inside a window of at
// most `long_window` tiles is moved back to that window's first tile, so only long windows are
// ever split between two work items.  Item k covers tiles [cut(k), cut(k+1)) and owns every
// window whose last tile lies in that range (plus, for item 0, leading empty windows).
// A split window's pieces are written as fp32 partial tiles to scratch and summed in item order
// (by a fix-up kernel, or by the item that finishes last), so results do not depend on scheduling.
// ---------------------------------------------------------------------------------------------

// number of windows w in [0, W) with window_offset[w + 1] <= x, found by one warp with a 32-ary
// search (every lane must call it with the same arguments)
__device__ __forceinline__ int64_t warp_count_ends_le(const int64_t *__restrict__ window_offset,
                                                      int64_t W, int64_t x, int lane) {
    int64_t lo = 0, hi = W;   // answer in [lo, hi]
    while (hi - lo > 0) {
        int64_t span = hi - lo;
        int64_t step = (span + 31) / 32;
        int64_t probe = lo + (int64_t)lane * step;           // window index probed by this lane
        bool le = (probe < hi) && (__ldg(window_offset + probe + 1) <= x);
        unsigned m = __ballot_sync(0xffffffffu, le);
        int cnt = __popc(m);                                  // ends are sorted: `le` is a prefix
        // lanes [0, cnt) satisfy end <= x: the answer lies in (probe(cnt-1), probe(cnt)]
        int64_t new_lo = (cnt == 0) ? lo : min(hi, lo + (int64_t)(cnt - 1) * step + 1);
        int64_t new_hi = (cnt == 32) ? hi : min(hi, lo + (int64_t)cnt * step);
        lo = new_lo;
        hi = new_hi;
    }
    return lo;
}

// The same count for two values at once with a 128-ary search (four probes per lane): the two
// searches' loads are all in flight together, so a pair of cuts costs two or three rounds of
// memory latency instead of eight (W = 10^4 .. 10^6).  Every lane must call it with the same arguments.
__device__ __forceinline__ void warp_count_ends_le_pair(const int64_t *__restrict__ window_offset, int64_t W,
                                                        int64_t x0, int64_t x1, int lane, int64_t *r0, int64_t *r1) {
    int64_t lo[2] = {0, 0}, hi[2] = {W, W};
    const int64_t x[2] = {x0, x1};
    while (hi[0] > lo[0] || hi[1] > lo[1]) {
        int64_t step[2];
        bool le[2][4];
#pragma unroll
        for (int s = 0; s < 2; ++s) {
            step[s] = (hi[s] - lo[s] + 127) / 128;
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const int64_t probe = lo[s] + (int64_t)(lane * 4 + j) * step[s];
                le[s][j] = (probe < hi[s]) && (__ldg(window_offset + probe + 1) <= x[s]);
            }
        }
#pragma unroll
        for (int s = 0; s < 2; ++s) {
            int cnt = 0;                                      // ends are sorted: `le` is a prefix in probe order
#pragma unroll
            for (int j = 0; j < 4; ++j) cnt += __popc(__ballot_sync(0xffffffffu, le[s][j]));
            const int64_t new_lo = (cnt == 0) ? lo[s] : min(hi[s], lo[s] + (int64_t)(cnt - 1) * step[s] + 1);
            const int64_t new_hi = (cnt == 128) ? hi[s] : min(hi[s], lo[s] + (int64_t)cnt * step[s]);
            lo[s] = new_lo;
            hi[s] = new_hi;
        }
    }
    *r0 = lo[0];
    *r1 = lo[1];
}

// cut positions of boundaries k and k + 1 at once (see warp_cut below for one boundary)
__device__ __forceinline__ void warp_cut_pair(const int64_t *__restrict__ window_offset, int64_t W, int64_t T,
                                              int64_t k, int64_t n_items, int64_t chunk, int64_t long_window,
                                              int lane, int64_t *s_out, int64_t *e_out, int64_t *w_first) {
    const int64_t xs = k * chunk, xe = (k + 1) * chunk;
    const bool s_end = k >= n_items || xs >= T, e_end = k + 1 >= n_items || xe >= T;
    int64_t ws, we;
    warp_count_ends_le_pair(window_offset, W, s_end ? 0 : xs, e_end ? 0 : xe, lane, &ws, &we);   // window containing the tile
    // (a boundary at or behind the last tile loads nothing: its window index may be W)
    const int64_t as = s_end ? 0 : __ldg(window_offset + ws), bs = s_end ? 0 : __ldg(window_offset + ws + 1);
    const int64_t ae = e_end ? 0 : __ldg(window_offset + we), be = e_end ? 0 : __ldg(window_offset + we + 1);
    *s_out = s_end ? T : ((bs - as <= long_window) ? as : xs);
    *e_out = e_end ? T : ((be - ae <= long_window) ? ae : xe);
    *w_first = s_end ? W : ws;
}

struct ItemRange {
    int64_t s, e;      // tile range [s, e)
    int64_t w_lo;      // first window owned (or touched) by this item
};

// cut position of boundary k (k in [0, n_items]); all lanes of the warp participate
__device__ __forceinline__ int64_t warp_cut(const int64_t *__restrict__ window_offset, int64_t W,
                                            int64_t T, int64_t k, int64_t n_items, int64_t chunk,
                                            int64_t long_window, int lane, int64_t *w_at) {
    int64_t x = k * chunk;
    if (k >= n_items || x >= T) {
        *w_at = W;
        return T;
    }
    int64_t w = warp_count_ends_le(window_offset, W, x, lane);   // window containing tile x
    int64_t a = __ldg(window_offset + w), b = __ldg(window_offset + w + 1);
    *w_at = w;
    return (b - a <= long_window) ? a : x;
}

}  // namespace grws
