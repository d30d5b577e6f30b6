// Device-side helpers shared by the kernels: storage-type rounding, activations and their
// derivatives.  The formulas follow source/standard-modules/neural/activations.slang:8-228 and the
// max tie rule of source/slang/diff.meta.slang:2268-2273; GELU (tanh form) is written in the same style.
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <stdint.h>

#include "../../include/slang_b200_mlp.h"

namespace mlpb200 {

__host__ __device__ inline int dtype_size(int dtype) { return dtype == MLP_F32 ? 4 : 2; }

__device__ __forceinline__ float round_to(int dtype, float v)
{
    if (dtype == MLP_F16) return __half2float(__float2half_rn(v));
    if (dtype == MLP_BF16) return __bfloat162float(__float2bfloat16_rn(v));
    return v;
}

__device__ __forceinline__ float load_as_f32(int dtype, const void* base, int64_t idx)
{
    if (dtype == MLP_F16) return __half2float(((const __half*)base)[idx]);
    if (dtype == MLP_BF16) return __bfloat162float(((const __nv_bfloat16*)base)[idx]);
    return ((const float*)base)[idx];
}

__device__ __forceinline__ void store_from_f32(int dtype, void* base, int64_t idx, float v)
{
    if (dtype == MLP_F16) ((__half*)base)[idx] = __float2half_rn(v);
    else if (dtype == MLP_BF16) ((__nv_bfloat16*)base)[idx] = __float2bfloat16_rn(v);
    else ((float*)base)[idx] = v;
}

// Element index of weight (output o, input i) of a layer behind MlpLayerPointers.weights.  OptimalLayout
// (source/standard-modules/neural/network-parameter-layout-converter.slang:54-68, 176-181): 16x16 tiles,
// tile (input tile, output tile) at (input_tile * tile_cols + output_tile) * 256, inside a tile the register
// order of a tensor-core B fragment (lane = 4 * (output % 8) + (input % 8) / 2, then the output half, the
// input half and the parity of the input).
__host__ __device__ inline int64_t weight_index(int layout, int in, int out, int o, int i)
{
    if (layout != MLP_PARAMS_OPTIMAL) return int64_t(o) * in + i;
    const int tile_cols = (out + 15) / 16;
    const int row = i & 15, col = o & 15;
    const int pos = (((col & 7) * 4 + ((row & 7) >> 1)) * 8) + (col >> 3) * 4 + (row >> 3) * 2 + (row & 1);
    return int64_t((i >> 4) * tile_cols + (o >> 4)) * 256 + pos;
}

#define MLPB200_SQRT_2_OVER_PI 0.7978845608028654f
#define MLPB200_GELU_C 0.044715f

__device__ __forceinline__ float sigmoid_stable(float x)
{
    float ex = expf(x >= 0.0f ? -x : x);
    return x >= 0.0f ? __fdiv_rn(1.0f, 1.0f + ex) : __fdiv_rn(ex, 1.0f + ex);
}

__device__ __forceinline__ float act_value(int act, float alpha, float x)
{
    switch (act) {
    case MLP_ACT_RELU: return x > 0.0f ? x : 0.0f;
    case MLP_ACT_LEAKY_RELU: return x < 0.0f ? __fmul_rn(alpha, x) : x;
    case MLP_ACT_LEAKY_MAX: { float y = __fmul_rn(x, alpha); return x > y ? x : y; }
    case MLP_ACT_SIGMOID: return sigmoid_stable(x);
    case MLP_ACT_TANH: return tanhf(x);
    case MLP_ACT_EXP: return expf(x);
    case MLP_ACT_SINE: return sinf(x);
    case MLP_ACT_SILU: {
        float ex = expf(x >= 0.0f ? -x : x);
        return x >= 0.0f ? __fdiv_rn(x, 1.0f + ex) : __fdiv_rn(x * ex, 1.0f + ex);
    }
    case MLP_ACT_QUICK_GELU: {
        float sx = 1.702f * x;
        float ex = expf(sx >= 0.0f ? -sx : sx);
        return sx >= 0.0f ? __fdiv_rn(x, 1.0f + ex) : __fdiv_rn(x * ex, 1.0f + ex);
    }
    case MLP_ACT_GELU_TANH: {
        float u = MLPB200_SQRT_2_OVER_PI * (x + MLPB200_GELU_C * x * x * x);
        return 0.5f * x * (1.0f + tanhf(u));
    }
    default: return x;
    }
}

__device__ __forceinline__ float act_deriv(int act, float alpha, float x)
{
    switch (act) {
    case MLP_ACT_RELU: return x > 0.0f ? 1.0f : (x == 0.0f ? 0.5f : 0.0f);
    case MLP_ACT_LEAKY_RELU: return x < 0.0f ? alpha : 1.0f;
    case MLP_ACT_LEAKY_MAX: {
        float y = __fmul_rn(x, alpha);
        if (x > y) return 1.0f;
        if (x < y) return alpha;
        return 0.5f * (1.0f + alpha);
    }
    case MLP_ACT_SIGMOID: { float s = sigmoid_stable(x); return s * (1.0f - s); }
    case MLP_ACT_TANH: { float t = tanhf(x); return 1.0f - t * t; }
    case MLP_ACT_EXP: return expf(x);
    case MLP_ACT_SINE: return cosf(x);
    case MLP_ACT_SILU: { float s = sigmoid_stable(x); return s * (1.0f + x * (1.0f - s)); }
    case MLP_ACT_QUICK_GELU: {
        float s = sigmoid_stable(1.702f * x);
        return s * (1.0f + 1.702f * x * (1.0f - s));
    }
    case MLP_ACT_GELU_TANH: {
        float x2 = x * x;
        float u = MLPB200_SQRT_2_OVER_PI * (x + MLPB200_GELU_C * x * x2);
        float t = tanhf(u);
        float du = MLPB200_SQRT_2_OVER_PI * (1.0f + 3.0f * MLPB200_GELU_C * x2);
        return 0.5f * (1.0f + t) + 0.5f * x * (1.0f - t * t) * du;
    }
    default: return 1.0f;
    }
}

// Integer power by repeated squaring with separately rounded multiplies: the same on every machine.
__host__ __device__ inline float pow_int(float base, int32_t e)
{
    float r = 1.0f, b = base;
    while (e > 0) {
#ifdef __CUDA_ARCH__
        if (e & 1) r = __fmul_rn(r, b);
        b = __fmul_rn(b, b);
#else
        if (e & 1) r = r * b;
        b = b * b;
#endif
        e >>= 1;
    }
    return r;
}

struct Layout {
    int64_t w[MLP_MAX_LAYERS];
    int64_t b[MLP_MAX_LAYERS];
    int64_t total;
};

inline Layout make_layout(const MlpConfig& c)
{
    Layout L{};
    int64_t off = 0;
    if (c.param_layout == MLP_PARAMS_OPTIMAL) {
        // FFLayer's storage (source/standard-modules/neural/layers.slang:53-71): per layer align16(in) x align16(out)
        // weights in 16x16 tiles, then align16(out) bias slots
        for (int l = 0; l < c.n_layers; ++l) {
            const int64_t in16 = (int64_t(c.dims[l]) + 15) / 16 * 16, out16 = (int64_t(c.dims[l + 1]) + 15) / 16 * 16;
            L.w[l] = off; off += in16 * out16;
            L.b[l] = off; off += out16;
        }
        L.total = off;
        return L;
    }
    const int64_t align = 64 / dtype_size(c.dtype);
    for (int l = 0; l < c.n_layers; ++l) {
        int64_t nw = int64_t(c.dims[l]) * c.dims[l + 1];
        L.w[l] = off; off += (nw + align - 1) / align * align;
        L.b[l] = off; off += (int64_t(c.dims[l + 1]) + align - 1) / align * align;
    }
    L.total = off;
    return L;
}

}  // namespace mlpb200
