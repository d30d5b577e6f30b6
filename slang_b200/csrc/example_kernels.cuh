// The literal example entry points (learnGradient, adjustParameters) of the 4 -> 16 -> 4 half network.
//
// Kept in a header so that the same source builds twice: into the shared library (launched through
// the C ABI) and into a stand-alone sm_100a cubin whose two extern "C" entry points carry exactly the
// launch parameters a CUDA module built from examples/mlp-training/kernels.slang:8-41 exports
// (compute-stage uniforms stay launch parameters in declaration order; thread id =
// blockIdx * blockDim + threadIdx; block (256,1,1), grid (ceil(count/256),1,1)).
// Compile with -fmad=false: every half and float operation rounds on its own.
#pragma once
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/slang_b200_mlp_config.h"

namespace mlpb200 {

// ------------------------------------------------------------------------------------------------
// The literal example: 4 -> 16 -> 4 in half (examples/mlp-training/{kernels,network,mlp_sw,mlvec_sw}.slang).
// Every half operation is rounded on its own, as IEEE half arithmetic does.
// ------------------------------------------------------------------------------------------------
__device__ __forceinline__ __half hmul_(__half a, __half b) { return __float2half_rn(__half2float(a) * __half2float(b)); }
__device__ __forceinline__ __half hadd_(__half a, __half b) { return __float2half_rn(__half2float(a) + __half2float(b)); }
__device__ __forceinline__ __half hsub_(__half a, __half b) { return __float2half_rn(__half2float(a) - __half2float(b)); }
__device__ __forceinline__ __half hdiv_(__half a, __half b) { return __float2half_rn(__fdiv_rn(__half2float(a), __half2float(b))); }
__device__ __forceinline__ bool hneg_(__half a) { return __half2float(a) < 0.0f; }

template <int In, int Out>
__device__ void ex_layer_eval(const MlpLayerPointers& lp, const __half* x, __half* y)
{
    const __half* W = (const __half*)lp.weights;
    const __half* B = (const __half*)lp.biases;
    for (int i = 0; i < Out; ++i) {
        __half r = B[i];
        for (int j = 0; j < In; ++j) r = hadd_(r, hmul_(W[i * In + j], x[j]));
        y[i] = r;
    }
    const __half slope = __float2half_rn(0.001f);
    for (int i = 0; i < Out; ++i)
        if (hneg_(y[i])) y[i] = hmul_(y[i], slope);
}

// Backward of one layer for one sample.  The per-sample weight- and bias-gradient terms are left in
// shared memory (g and x) for the ordered block-level sum; dx = W^T g.
template <int In, int Out>
__device__ void ex_layer_bwd(const MlpLayerPointers& lp, const __half* x, __half* g, __half* dx)
{
    __half fwd[Out];
    ex_layer_eval<In, Out>(lp, x, fwd);
    const __half slope = __float2half_rn(0.01f);
    for (int i = 0; i < Out; ++i)
        if (hneg_(fwd[i])) g[i] = hmul_(g[i], slope);
    const __half* W = (const __half*)lp.weights;
    for (int i = 0; i < In; ++i) {
        __half r = __float2half_rn(0.0f);
        for (int j = 0; j < Out; ++j) r = hadd_(r, hmul_(W[j * In + i], g[j]));
        dx[i] = r;
    }
}

// Atomic half add through a 32-bit compare-and-swap on the containing word
// (the job of InterlockedAddF16Emulated, source/slang/hlsl.meta.slang:34654-34667).
__device__ inline void atomic_add_half(__half* addr, __half v)
{
    unsigned int* word = (unsigned int*)((uintptr_t)addr & ~(uintptr_t)3);
    const bool hi = ((uintptr_t)addr & 2) != 0;
    unsigned int old = *word, assumed;
    do {
        assumed = old;
        unsigned short cur = hi ? (unsigned short)(assumed >> 16) : (unsigned short)(assumed & 0xffffu);
        __half sum = hadd_(__ushort_as_half(cur), v);
        unsigned int repl = hi ? ((assumed & 0x0000ffffu) | ((unsigned int)__half_as_ushort(sum) << 16))
                               : ((assumed & 0xffff0000u) | (unsigned int)__half_as_ushort(sum));
        old = atomicCAS(word, assumed, repl);
    } while (old != assumed);
}

// Ordered sum over the block's samples of g[s][i] * x[s][j] (half, one rounding per multiply and per
// add, ascending sample order), then one atomic per element per block.  With a single block (the
// example runs 16 samples) the result is what a sequential machine produces.
template <int In, int Out>
__device__ void ex_accumulate(const MlpLayerPointers& lp, const __half* sg, const __half* sx, int n_valid, int gstride,
                              int xstride)
{
    __half* dW = (__half*)lp.weightsGrad;
    __half* dB = (__half*)lp.biasesGrad;
    const bool single = gridDim.x == 1;
    for (int p = threadIdx.x; p < In * Out + Out; p += blockDim.x) {
        const bool is_w = p < In * Out;
        const int i = is_w ? p / In : p - In * Out, j = is_w ? p % In : 0;
        __half* dst = is_w ? dW + p : dB + i;
        // A single block continues from the stored value, like the sequential machine; several
        // blocks each sum their own samples first and then add once.
        __half acc = single ? *dst : __float2half_rn(0.0f);
        bool first = !single;
        for (int s = 0; s < n_valid; ++s) {
            const __half term = is_w ? hmul_(sg[s * gstride + i], sx[s * xstride + j]) : sg[s * gstride + i];
            acc = first ? term : hadd_(acc, term);
            first = false;
        }
        if (single) *dst = acc;
        else if (n_valid > 0) atomic_add_half(dst, acc);
    }
}

extern "C" __global__ void __launch_bounds__(256)
learnGradient(const MlpLayerPointers* __restrict__ network, uint32_t* lossBuffer, const float2* __restrict__ inputs,
              uint32_t count)
{
    // Per-sample vectors staged for the ordered sums: encoding (4), layer-1 output (16), g2 (4), g1 (16).
    __shared__ __half s_enc[256 * 4];
    __shared__ __half s_h1[256 * 16];
    __shared__ __half s_g2[256 * 4];
    __shared__ __half s_g1[256 * 16];

    const uint32_t tid = blockIdx.x * blockDim.x + threadIdx.x;
    const bool valid = tid < count;
    const MlpLayerPointers L1 = network[0], L2 = network[1];
    float this_loss = 0.0f;
    if (valid) {
        const float2 in = inputs[tid];
        const __half x = __float2half_rn(in.x), y = __float2half_rn(in.y);
        __half enc[4] = {x, y, hmul_(x, x), hmul_(y, y)};
        __half h1[16], out[4], g2[4], g1[16], dead[4];
        ex_layer_eval<4, 16>(L1, enc, h1);
        ex_layer_eval<16, 4>(L2, h1, out);
        const __half one = __float2half_rn(1.0f), half_ = __float2half_rn(0.5f);
        __half gt[4];
        gt[0] = hdiv_(hadd_(x, y), hadd_(one, hmul_(y, y)));
        gt[1] = hadd_(hmul_(__float2half_rn(2.0f), x), y);
        gt[2] = hadd_(hmul_(hmul_(half_, x), x), hmul_(__float2half_rn(1.2f), y));
        gt[3] = hadd_(x, hmul_(hmul_(half_, y), y));
        __half l = __float2half_rn(0.0f);
        for (int k = 0; k < 4; ++k) {
            const __half d = hsub_(out[k], gt[k]);
            g2[k] = hadd_(hmul_(d, one), hmul_(d, one));
            l = hadd_(l, hmul_(d, d));
        }
        this_loss = __half2float(l);
        ex_layer_bwd<16, 4>(L2, h1, g2, g1);
        ex_layer_bwd<4, 16>(L1, enc, g1, dead);
        for (int k = 0; k < 4; ++k) { s_enc[threadIdx.x * 4 + k] = enc[k]; s_g2[threadIdx.x * 4 + k] = g2[k]; }
        for (int k = 0; k < 16; ++k) { s_h1[threadIdx.x * 16 + k] = h1[k]; s_g1[threadIdx.x * 16 + k] = g1[k]; }
    }
    __syncthreads();
    const int first = blockIdx.x * blockDim.x;
    const int n_valid = count > (uint32_t)first ? min((int)blockDim.x, (int)(count - first)) : 0;
    ex_accumulate<16, 4>(L2, s_g2, s_h1, n_valid, 4, 16);
    ex_accumulate<4, 16>(L1, s_g1, s_enc, n_valid, 16, 4);

    // WaveActiveMax, then the first lane folds the wave's value into the loss word.
    float m = this_loss;
    for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
    if ((threadIdx.x & 31) == 0 && first + (int)(threadIdx.x) < (int)count) atomicMax(lossBuffer, __float_as_uint(m));
}

// ------------------------------------------------------------------------------------------------
// The cooperative-vector flavour of the same example (examples/mlp-training-coopvec/{kernels,network,
// fflayer}.slang).  Differences from the software flavour above: a layer's sums start from zero and
// the bias is added last (the matrix-vector fallback, source/slang/hlsl.meta.slang:32858-32912 and the
// bias loop that follows it); the activation is max(o, o * 0.001h) and its derivative comes from the
// derivative of max (1 above, 0.001 below, the mean of both at a tie, source/slang/diff.meta.slang:
// 2268-2273), applied to the pre-activation sums; the weight gradient is accumulated into a matrix in
// the training-optimal layout (here: 16x16 tiles, tile-major, row-major inside a tile, zero padded;
// both of the example's matrices fit one tile, element (i, j) at i * 16 + j), which the host converts
// to row-major afterwards (mlp-training-coopvec.cpp:201-236); the bias gradient goes straight to the
// row-major gradient segment (coopVecReduceSumAccumulate, hlsl.meta.slang:33344-33351).
// ------------------------------------------------------------------------------------------------
template <int In, int Out>
__device__ void cv_layer_sums(const MlpLayerPointers& lp, const __half* x, __half* o)
{
    const __half* W = (const __half*)lp.weights;
    const __half* B = (const __half*)lp.biases;
    for (int i = 0; i < Out; ++i) {
        __half r = __float2half_rn(0.0f);
        for (int j = 0; j < In; ++j) r = hadd_(r, hmul_(W[i * In + j], x[j]));
        o[i] = hadd_(r, B[i]);
    }
}

template <int N>
__device__ void cv_activation(const __half* o, __half* y)
{
    const __half slope = __float2half_rn(0.001f);
    for (int i = 0; i < N; ++i) {
        const __half scaled = hmul_(o[i], slope);
        y[i] = __half2float(o[i]) > __half2float(scaled) ? o[i] : (__half2float(o[i]) < __half2float(scaled) ? scaled : o[i]);
    }
}

// g <- gradient with respect to the pre-activation sums o; dx = W^T g with sums starting from zero.
template <int In, int Out>
__device__ void cv_layer_bwd(const MlpLayerPointers& lp, const __half* o, __half* g, __half* dx)
{
    const __half slope = __float2half_rn(0.001f), half_ = __float2half_rn(0.5f);
    for (int i = 0; i < Out; ++i) {
        const float a = __half2float(o[i]), b = __half2float(hmul_(o[i], slope));
        if (a > b) { /* whole gradient to the first argument */ }
        else if (a < b) g[i] = hmul_(g[i], slope);
        else { const __half h = hmul_(half_, g[i]); g[i] = hadd_(h, hmul_(h, slope)); }
    }
    const __half* W = (const __half*)lp.weights;
    for (int i = 0; i < In; ++i) {
        __half r = __float2half_rn(0.0f);
        for (int j = 0; j < Out; ++j) r = hadd_(r, hmul_(W[j * In + i], g[j]));
        dx[i] = r;
    }
}

// Like ex_accumulate, with the weight gradient in the one-tile training-optimal layout.
template <int In, int Out>
__device__ void cv_accumulate(const MlpLayerPointers& lp, const __half* sg, const __half* sx, int n_valid, int gstride,
                              int xstride)
{
    __half* dW = (__half*)lp.weightsGrad;
    __half* dB = (__half*)lp.biasesGrad;
    const bool single = gridDim.x == 1;
    for (int p = threadIdx.x; p < In * Out + Out; p += blockDim.x) {
        const bool is_w = p < In * Out;
        const int i = is_w ? p / In : p - In * Out, j = is_w ? p % In : 0;
        __half* dst = is_w ? dW + i * 16 + j : dB + i;
        __half acc = single ? *dst : __float2half_rn(0.0f);
        bool first = !single;
        for (int s = 0; s < n_valid; ++s) {
            const __half term = is_w ? hmul_(sg[s * gstride + i], sx[s * xstride + j]) : sg[s * gstride + i];
            acc = first ? term : hadd_(acc, term);
            first = false;
        }
        if (single) *dst = acc;
        else if (n_valid > 0) atomic_add_half(dst, acc);
    }
}

extern "C" __global__ void __launch_bounds__(256)
learnGradient_coopvec(const MlpLayerPointers* __restrict__ network, uint32_t* lossBuffer,
                      const float2* __restrict__ inputs, uint32_t count)
{
    __shared__ __half s_enc[256 * 4];
    __shared__ __half s_h1[256 * 16];
    __shared__ __half s_g2[256 * 4];
    __shared__ __half s_g1[256 * 16];

    const uint32_t tid = blockIdx.x * blockDim.x + threadIdx.x;
    const bool valid = tid < count;
    const MlpLayerPointers L1 = network[0], L2 = network[1];
    float this_loss = 0.0f;
    if (valid) {
        const float2 in = inputs[tid];
        const __half x = __float2half_rn(in.x), y = __float2half_rn(in.y);
        __half enc[4] = {x, y, hmul_(x, x), hmul_(y, y)};
        __half o1[16], h1[16], o2[4], out[4], g2[4], g1[16], dead[4];
        cv_layer_sums<4, 16>(L1, enc, o1);
        cv_activation<16>(o1, h1);
        cv_layer_sums<16, 4>(L2, h1, o2);
        cv_activation<4>(o2, out);
        const __half one = __float2half_rn(1.0f), half_ = __float2half_rn(0.5f);
        __half gt[4];
        gt[0] = hdiv_(hadd_(x, y), hadd_(one, hmul_(y, y)));
        gt[1] = hadd_(hmul_(__float2half_rn(2.0f), x), y);
        gt[2] = hadd_(hmul_(hmul_(half_, x), x), hmul_(__float2half_rn(1.2f), y));
        gt[3] = hadd_(x, hmul_(hmul_(half_, y), y));
        __half l = __float2half_rn(0.0f);
        for (int k = 0; k < 4; ++k) {
            const __half d = hsub_(out[k], gt[k]);
            g2[k] = hadd_(hmul_(d, one), hmul_(d, one));
            l = hadd_(l, hmul_(d, d));
        }
        this_loss = __half2float(l);
        cv_layer_bwd<16, 4>(L2, o2, g2, g1);
        cv_layer_bwd<4, 16>(L1, o1, g1, dead);
        for (int k = 0; k < 4; ++k) { s_enc[threadIdx.x * 4 + k] = enc[k]; s_g2[threadIdx.x * 4 + k] = g2[k]; }
        for (int k = 0; k < 16; ++k) { s_h1[threadIdx.x * 16 + k] = h1[k]; s_g1[threadIdx.x * 16 + k] = g1[k]; }
    }
    __syncthreads();
    const int first = blockIdx.x * blockDim.x;
    const int n_valid = count > (uint32_t)first ? min((int)blockDim.x, (int)(count - first)) : 0;
    cv_accumulate<16, 4>(L2, s_g2, s_h1, n_valid, 4, 16);
    cv_accumulate<4, 16>(L1, s_g1, s_enc, n_valid, 16, 4);

    float m = this_loss;
    for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
    if ((threadIdx.x & 31) == 0 && first + (int)(threadIdx.x) < (int)count) atomicMax(lossBuffer, __float_as_uint(m));
}

extern "C" __global__ void __launch_bounds__(256)
adjustParameters(MlpExampleAdamState* states, __half* params, __half* gradients, uint32_t count)
{
    const uint32_t tid = blockIdx.x * blockDim.x + threadIdx.x;
    if (tid >= count) return;
    __half g = gradients[tid];
    if (__hisnan(g)) { gradients[tid] = __float2half_rn(0.0f); return; }
    const __half beta1 = __float2half_rn(0.9f), beta2 = __float2half_rn(0.999f);
    const __half eps = __float2half_rn(1e-7f), lr = __float2half_rn(0.01f), one = __float2half_rn(1.0f);
    MlpExampleAdamState st = states[tid];
    st.iteration++;
    if (__hisinf(g)) g = __float2half_rn(__half2float(g) > 0.0f ? 10000.0f : -10000.0f);
    __half m = __ushort_as_half(st.mean), v = __ushort_as_half(st.variance);
    m = hadd_(hmul_(beta1, m), hmul_(hsub_(one, beta1), g));
    v = hadd_(hmul_(beta2, v), hmul_(hmul_(hsub_(one, beta2), g), g));
    const __half it = __float2half_rn((float)st.iteration);
    const __half p1 = __float2half_rn(powf(__half2float(beta1), __half2float(it)));
    const __half p2 = __float2half_rn(powf(__half2float(beta2), __half2float(it)));
    const __half mean_hat = hdiv_(m, hsub_(one, p1));
    const __half var_hat = hdiv_(v, hsub_(one, p2));
    const __half mx = __half2float(var_hat) > 0.0f ? var_hat : __float2half_rn(0.0f);
    const __half den = __float2half_rn(__fsqrt_rn(__half2float(hadd_(mx, eps))));
    __half p = params[tid];
    p = hsub_(p, hdiv_(hmul_(lr, mean_hat), den));
    params[tid] = p;
    st.mean = __half_as_ushort(m);
    st.variance = __half_as_ushort(v);
    states[tid] = st;
    gradients[tid] = __float2half_rn(0.0f);
}

}  // namespace mlpb200
