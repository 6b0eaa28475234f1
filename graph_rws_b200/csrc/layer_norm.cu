// Row normalisation of the GCN's hidden activations: y = LayerNorm(act(x)) * gamma + beta, act =
// identity or ReLU, and its backward pass.  The model applies activation and LayerNorm between its
// graph convolutions (models/model.py:117-121 of the reference, through torch.nn.LayerNorm); on the
// row counts of full-graph training (2.3e5 rows x 256) the library kernels spend 0.35 ms forward
// and 0.9 ms backward, most of it in the column reduction for the gamma / beta gradients, where
// one pass over the operands is 0.04 / 0.06 ms of HBM time.
//
// A warp owns a row: every lane holds 8 consecutive features per 256-feature chunk (one 16-byte load
// for 16-bit types), the row statistics are two shuffle reductions (mean, then the centred sum of
// squares), nothing goes through shared memory.  Backward: the same walk computes dx and keeps the
// gamma / beta gradient contributions of the rows a warp visits in registers; the warps of a CTA
// add theirs up in shared memory, every CTA writes one partial row, and a second small kernel adds
// the partial rows in CTA order (deterministic, no atomics).
#include "grws_common.cuh"

#include <cuda_bf16.h>
#include <cuda_fp16.h>

namespace grws {
namespace ln {

constexpr int WARPS = 8;
constexpr int MAX_CHUNKS = 4;          // up to 1024 features
constexpr int MAX_PARTIAL_CTAS = 1024;

template <typename T> struct Vec8;
template <> struct Vec8<float> {
    static __device__ __forceinline__ void load(const float *p, float (&v)[8]) {
        const float4 a = *reinterpret_cast<const float4 *>(p), b = *reinterpret_cast<const float4 *>(p + 4);
        v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w; v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
    }
    static __device__ __forceinline__ void store(float *p, const float (&v)[8]) {
        *reinterpret_cast<float4 *>(p) = make_float4(v[0], v[1], v[2], v[3]);
        *reinterpret_cast<float4 *>(p + 4) = make_float4(v[4], v[5], v[6], v[7]);
    }
};
template <> struct Vec8<__half> {
    static __device__ __forceinline__ void load(const __half *p, float (&v)[8]) {
        const uint4 u = *reinterpret_cast<const uint4 *>(p);
        const __half2 *h = reinterpret_cast<const __half2 *>(&u);
#pragma unroll
        for (int i = 0; i < 4; ++i) { const float2 f = __half22float2(h[i]); v[2 * i] = f.x; v[2 * i + 1] = f.y; }
    }
    static __device__ __forceinline__ void store(__half *p, const float (&v)[8]) {
        uint4 u;
        __half2 *h = reinterpret_cast<__half2 *>(&u);
#pragma unroll
        for (int i = 0; i < 4; ++i) h[i] = __floats2half2_rn(v[2 * i], v[2 * i + 1]);
        *reinterpret_cast<uint4 *>(p) = u;
    }
};
template <> struct Vec8<__nv_bfloat16> {
    static __device__ __forceinline__ void load(const __nv_bfloat16 *p, float (&v)[8]) {
        const uint4 u = *reinterpret_cast<const uint4 *>(p);
        const __nv_bfloat162 *h = reinterpret_cast<const __nv_bfloat162 *>(&u);
#pragma unroll
        for (int i = 0; i < 4; ++i) { const float2 f = __bfloat1622float2(h[i]); v[2 * i] = f.x; v[2 * i + 1] = f.y; }
    }
    static __device__ __forceinline__ void store(__nv_bfloat16 *p, const float (&v)[8]) {
        uint4 u;
        __nv_bfloat162 *h = reinterpret_cast<__nv_bfloat162 *>(&u);
#pragma unroll
        for (int i = 0; i < 4; ++i) h[i] = __floats2bfloat162_rn(v[2 * i], v[2 * i + 1]);
        *reinterpret_cast<uint4 *>(p) = u;
    }
};

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}

// features 8 * (32 * j + lane) .. + 7 of chunk j belong to this lane
template <typename T, int NCH, bool RELU>
__global__ void __launch_bounds__(WARPS * 32) layer_norm_fwd_kernel(const T *__restrict__ x, const T *__restrict__ gamma,
                                                                    const T *__restrict__ beta, T *__restrict__ y,
                                                                    float *__restrict__ mean_out, float *__restrict__ rstd_out,
                                                                    int64_t rows, int C, float eps) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    float g[NCH][8], b[NCH][8];
#pragma unroll
    for (int j = 0; j < NCH; ++j) {
        const int c0 = 8 * (32 * j + lane);
        if (c0 < C) { Vec8<T>::load(gamma + c0, g[j]); Vec8<T>::load(beta + c0, b[j]); }
    }
    const float inv_c = 1.0f / (float)C;
    for (int64_t row = (int64_t)blockIdx.x * WARPS + warp; row < rows; row += (int64_t)gridDim.x * WARPS) {
        float v[NCH][8];
        float s = 0.0f;
#pragma unroll
        for (int j = 0; j < NCH; ++j) {
            const int c0 = 8 * (32 * j + lane);
            if (c0 < C) {
                Vec8<T>::load(x + row * C + c0, v[j]);
#pragma unroll
                for (int i = 0; i < 8; ++i) { if (RELU) v[j][i] = fmaxf(v[j][i], 0.0f); s += v[j][i]; }
            }
        }
        const float mean = warp_sum(s) * inv_c;
        float q = 0.0f;
#pragma unroll
        for (int j = 0; j < NCH; ++j)
            if (8 * (32 * j + lane) < C) {
#pragma unroll
                for (int i = 0; i < 8; ++i) { const float d = v[j][i] - mean; q += d * d; }
            }
        const float rstd = rsqrtf(warp_sum(q) * inv_c + eps);
#pragma unroll
        for (int j = 0; j < NCH; ++j) {
            const int c0 = 8 * (32 * j + lane);
            if (c0 < C) {
                float o[8];
#pragma unroll
                for (int i = 0; i < 8; ++i) o[i] = (v[j][i] - mean) * rstd * g[j][i] + b[j][i];
                Vec8<T>::store(y + row * C + c0, o);
            }
        }
        if (lane == 0) { mean_out[row] = mean; rstd_out[row] = rstd; }
    }
}

template <typename T, int NCH, bool RELU>
__global__ void __launch_bounds__(WARPS * 32) layer_norm_bwd_kernel(const T *__restrict__ x, const T *__restrict__ gamma,
                                                                    const T *__restrict__ dy, const float *__restrict__ mean_in,
                                                                    const float *__restrict__ rstd_in, T *__restrict__ dx,
                                                                    float *__restrict__ partial, int64_t rows, int C) {
    extern __shared__ float red[];          // [WARPS][2][C]
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    float g[NCH][8], dg[NCH][8], db[NCH][8];
#pragma unroll
    for (int j = 0; j < NCH; ++j) {
        const int c0 = 8 * (32 * j + lane);
        if (c0 < C) Vec8<T>::load(gamma + c0, g[j]);
#pragma unroll
        for (int i = 0; i < 8; ++i) { dg[j][i] = 0.0f; db[j][i] = 0.0f; }
    }
    const float inv_c = 1.0f / (float)C;
    for (int64_t row = (int64_t)blockIdx.x * WARPS + warp; row < rows; row += (int64_t)gridDim.x * WARPS) {
        const float mean = mean_in[row], rstd = rstd_in[row];
        float xh[NCH][8], gy[NCH][8];
        bool pos[NCH][8];
        float s1 = 0.0f, s2 = 0.0f;
#pragma unroll
        for (int j = 0; j < NCH; ++j) {
            const int c0 = 8 * (32 * j + lane);
            if (c0 < C) {
                float xv[8], dv[8];
                Vec8<T>::load(x + row * C + c0, xv);
                Vec8<T>::load(dy + row * C + c0, dv);
#pragma unroll
                for (int i = 0; i < 8; ++i) {
                    pos[j][i] = !RELU || xv[i] > 0.0f;
                    const float a = RELU ? fmaxf(xv[i], 0.0f) : xv[i];
                    xh[j][i] = (a - mean) * rstd;
                    gy[j][i] = dv[i] * g[j][i];
                    s1 += gy[j][i];
                    s2 += gy[j][i] * xh[j][i];
                    dg[j][i] += dv[i] * xh[j][i];
                    db[j][i] += dv[i];
                }
            }
        }
        s1 = warp_sum(s1) * inv_c;
        s2 = warp_sum(s2) * inv_c;
#pragma unroll
        for (int j = 0; j < NCH; ++j) {
            const int c0 = 8 * (32 * j + lane);
            if (c0 < C) {
                float o[8];
#pragma unroll
                for (int i = 0; i < 8; ++i) {
                    const float d = rstd * (gy[j][i] - s1 - xh[j][i] * s2);
                    o[i] = pos[j][i] ? d : 0.0f;
                }
                Vec8<T>::store(dx + row * C + c0, o);
            }
        }
    }
    // the CTA's contribution to the gamma / beta gradients: warps in order, then one partial row
#pragma unroll
    for (int j = 0; j < NCH; ++j) {
        const int c0 = 8 * (32 * j + lane);
        if (c0 < C) {
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                red[(warp * 2 + 0) * C + c0 + i] = dg[j][i];
                red[(warp * 2 + 1) * C + c0 + i] = db[j][i];
            }
        }
    }
    __syncthreads();
    for (int c = threadIdx.x; c < 2 * C; c += blockDim.x) {
        const int which = c / C, col = c % C;
        float s = 0.0f;
#pragma unroll
        for (int w = 0; w < WARPS; ++w) s += red[(w * 2 + which) * C + col];
        partial[(size_t)blockIdx.x * 2 * C + c] = s;
    }
}

// Adds the CTAs' partial rows: a block owns 32 of the 2 C columns, its 32 x 32 threads each take every
// 32nd partial row (coalesced along the columns), then the 32 sums of a column are added in a fixed
// order.
__global__ void __launch_bounds__(1024) layer_norm_param_grad_kernel(const float *__restrict__ partial, int n_partial, int C,
                                                                      float *__restrict__ dgamma, float *__restrict__ dbeta) {
    __shared__ float red[32][33];
    const int cx = threadIdx.x & 31, py = threadIdx.x >> 5;
    const int c = blockIdx.x * 32 + cx;
    float s = 0.0f;
    if (c < 2 * C)
        for (int p = py; p < n_partial; p += 32) s += partial[(size_t)p * 2 * C + c];
    red[py][cx] = s;
    __syncthreads();
    if (py == 0 && c < 2 * C) {
        float t = 0.0f;
#pragma unroll
        for (int k = 0; k < 32; ++k) t += red[k][cx];
        if (c < C) dgamma[c] = t; else dbeta[c - C] = t;
    }
}

static int grid_for(int64_t rows) {
    int dev = 0, sms = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || sms <= 0)
        sms = 148;
    int64_t g = ceil_div(rows, (int64_t)WARPS);
    const int64_t cap = (int64_t)sms * 4 < MAX_PARTIAL_CTAS ? (int64_t)sms * 4 : MAX_PARTIAL_CTAS;
    if (g > cap) g = cap;
    return g < 1 ? 1 : (int)g;
}

template <typename T, int NCH>
static int launch_fwd(const void *x, const void *gamma, const void *beta, void *y, float *mean, float *rstd, int64_t rows,
                      int C, float eps, int relu, cudaStream_t st) {
    const int g = grid_for(rows);
    if (relu) layer_norm_fwd_kernel<T, NCH, true><<<g, WARPS * 32, 0, st>>>((const T *)x, (const T *)gamma, (const T *)beta, (T *)y, mean, rstd, rows, C, eps);
    else layer_norm_fwd_kernel<T, NCH, false><<<g, WARPS * 32, 0, st>>>((const T *)x, (const T *)gamma, (const T *)beta, (T *)y, mean, rstd, rows, C, eps);
    GRWS_CUDA_TRY(cudaGetLastError());
    return GRWS_OK;
}

template <typename T, int NCH>
static int launch_bwd(const void *x, const void *gamma, const void *dy, const float *mean, const float *rstd, void *dx,
                      float *dgamma, float *dbeta, float *partial, int64_t rows, int C, int relu, cudaStream_t st) {
    const int g = grid_for(rows);
    const size_t smem = (size_t)WARPS * 2 * C * sizeof(float);
    if (relu) {
        if (smem > 48 * 1024) GRWS_CUDA_TRY(cudaFuncSetAttribute(layer_norm_bwd_kernel<T, NCH, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
        layer_norm_bwd_kernel<T, NCH, true><<<g, WARPS * 32, smem, st>>>((const T *)x, (const T *)gamma, (const T *)dy, mean, rstd, (T *)dx, partial, rows, C);
    } else {
        if (smem > 48 * 1024) GRWS_CUDA_TRY(cudaFuncSetAttribute(layer_norm_bwd_kernel<T, NCH, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
        layer_norm_bwd_kernel<T, NCH, false><<<g, WARPS * 32, smem, st>>>((const T *)x, (const T *)gamma, (const T *)dy, mean, rstd, (T *)dx, partial, rows, C);
    }
    GRWS_CUDA_TRY(cudaGetLastError());
    layer_norm_param_grad_kernel<<<(unsigned)ceil_div((int64_t)2 * C, (int64_t)32), 1024, 0, st>>>(partial, g, C, dgamma, dbeta);
    GRWS_CUDA_TRY(cudaGetLastError());
    return GRWS_OK;
}

template <typename T>
static int dispatch_fwd(int nch, const void *x, const void *gamma, const void *beta, void *y, float *mean, float *rstd,
                        int64_t rows, int C, float eps, int relu, cudaStream_t st) {
    switch (nch) {
        case 1: return launch_fwd<T, 1>(x, gamma, beta, y, mean, rstd, rows, C, eps, relu, st);
        case 2: return launch_fwd<T, 2>(x, gamma, beta, y, mean, rstd, rows, C, eps, relu, st);
        case 3: return launch_fwd<T, 3>(x, gamma, beta, y, mean, rstd, rows, C, eps, relu, st);
        default: return launch_fwd<T, 4>(x, gamma, beta, y, mean, rstd, rows, C, eps, relu, st);
    }
}

template <typename T>
static int dispatch_bwd(int nch, const void *x, const void *gamma, const void *dy, const float *mean, const float *rstd,
                        void *dx, float *dgamma, float *dbeta, float *partial, int64_t rows, int C, int relu, cudaStream_t st) {
    switch (nch) {
        case 1: return launch_bwd<T, 1>(x, gamma, dy, mean, rstd, dx, dgamma, dbeta, partial, rows, C, relu, st);
        case 2: return launch_bwd<T, 2>(x, gamma, dy, mean, rstd, dx, dgamma, dbeta, partial, rows, C, relu, st);
        case 3: return launch_bwd<T, 3>(x, gamma, dy, mean, rstd, dx, dgamma, dbeta, partial, rows, C, relu, st);
        default: return launch_bwd<T, 4>(x, gamma, dy, mean, rstd, dx, dgamma, dbeta, partial, rows, C, relu, st);
    }
}

}  // namespace ln
}  // namespace grws

using namespace grws;

extern "C" {

__attribute__((visibility("default")))
size_t grws_layer_norm_scratch_bytes(int64_t C) {
    if (C <= 0) return 0;
    return (size_t)ln::MAX_PARTIAL_CTAS * 2 * (size_t)C * sizeof(float);
}

__attribute__((visibility("default")))
int grws_layer_norm_fwd(const void *x, const void *gamma, const void *beta, void *y, float *mean, float *rstd,
                        int64_t rows, int64_t C, int dtype, int relu_input, float eps, void *stream) {
    GRWS_REQUIRE(rows >= 0 && C > 0, "bad size");
    GRWS_REQUIRE(C % 8 == 0 && C <= 256 * ln::MAX_CHUNKS, "layer norm handles widths that are multiples of 8 up to %d (C = %lld)",
                 256 * ln::MAX_CHUNKS, (long long)C);
    if (rows == 0) return GRWS_OK;
    GRWS_REQUIRE(x && gamma && beta && y && mean && rstd, "null pointer");
    GRWS_REQUIRE(aligned16(x) && aligned16(y) && aligned16(gamma) && aligned16(beta), "operands must be 16-byte aligned");
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    const int nch = (int)ceil_div(C, (int64_t)256);
    switch (dtype) {
        case GRWS_F32: return ln::dispatch_fwd<float>(nch, x, gamma, beta, y, mean, rstd, rows, (int)C, eps, relu_input, st);
        case GRWS_F16: return ln::dispatch_fwd<__half>(nch, x, gamma, beta, y, mean, rstd, rows, (int)C, eps, relu_input, st);
        case GRWS_BF16: return ln::dispatch_fwd<__nv_bfloat16>(nch, x, gamma, beta, y, mean, rstd, rows, (int)C, eps, relu_input, st);
    }
    return fail(GRWS_ERR_UNSUPPORTED, "bad dtype %d", dtype);
}

__attribute__((visibility("default")))
int grws_layer_norm_bwd(const void *x, const void *gamma, const void *dy, const float *mean, const float *rstd, void *dx,
                        float *dgamma, float *dbeta, int64_t rows, int64_t C, int dtype, int relu_input, void *scratch,
                        size_t scratch_bytes, void *stream) {
    GRWS_REQUIRE(rows >= 0 && C > 0, "bad size");
    GRWS_REQUIRE(C % 8 == 0 && C <= 256 * ln::MAX_CHUNKS, "layer norm handles widths that are multiples of 8 up to %d (C = %lld)",
                 256 * ln::MAX_CHUNKS, (long long)C);
    GRWS_REQUIRE(dgamma && dbeta && scratch, "null pointer");
    if (scratch_bytes < grws_layer_norm_scratch_bytes(C)) return fail(GRWS_ERR_SCRATCH, "layer norm scratch too small");
    GRWS_REQUIRE(rows == 0 || (x && gamma && dy && mean && rstd && dx), "null pointer");
    GRWS_REQUIRE(aligned16(x) && aligned16(dy) && aligned16(dx) && aligned16(gamma), "operands must be 16-byte aligned");
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    const int nch = (int)ceil_div(C, (int64_t)256);
    float *partial = static_cast<float *>(scratch);
    switch (dtype) {
        case GRWS_F32: return ln::dispatch_bwd<float>(nch, x, gamma, dy, mean, rstd, dx, dgamma, dbeta, partial, rows, (int)C, relu_input, st);
        case GRWS_F16: return ln::dispatch_bwd<__half>(nch, x, gamma, dy, mean, rstd, dx, dgamma, dbeta, partial, rows, (int)C, relu_input, st);
        case GRWS_BF16: return ln::dispatch_bwd<__nv_bfloat16>(nch, x, gamma, dy, mean, rstd, dx, dgamma, dbeta, partial, rows, (int)C, relu_input, st);
    }
    return fail(GRWS_ERR_UNSUPPORTED, "bad dtype %d", dtype);
}

}  // extern "C"
