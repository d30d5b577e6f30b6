// One-thread-per-sample kernels: the literal example entry points and the shape-generic path.
//
// These keep the reference's dispatch contract exactly: [numthreads(256,1,1)], thread id =
// blockIdx.x * blockDim.x + threadIdx.x, grid = ceil(count / 256)
// (examples/mlp-training/kernels.slang:8-41, examples/mlp-training/mlp-training.cpp:181-204).
// They serve every shape and number format; the tensor-core kernels take over for the shapes they
// are built for.  This file is compiled with -fmad=false: every multiply and add is separately
// rounded unless fmaf is written out, so fp32 results match a sequential CPU bit for bit.
#include <cuda_runtime.h>

#include <algorithm>
#include <cstdio>
#include <string>

#include "mlp_common.cuh"
#include "launchers.h"

#include "example_kernels.cuh"

namespace mlpb200 {

// ------------------------------------------------------------------------------------------------
// Shape-generic path: any MlpConfig within the scratch limits, one thread per sample.
// ------------------------------------------------------------------------------------------------
constexpr int kMaxActFloats = 768;  // sum of all layer widths a thread may hold

struct SimtNet {
    MlpConfig cfg;
    int a_off[MLP_MAX_LAYERS + 2];  // offset of the vector entering layer l in the per-thread arrays
};

// The type products read their operands in: the storage type, or MlpConfig.operand_dtype (fp32 storage whose
// weights and inter-layer vectors are converted to a 16-bit type where a product reads them).
__device__ __forceinline__ int operand_type(const MlpConfig& c) { return c.operand_dtype ? c.operand_dtype : c.dtype; }
__device__ __forceinline__ float load_weight(const MlpConfig& c, const void* W, int64_t idx)
{
    const float w = load_as_f32(c.dtype, W, idx);
    return c.operand_dtype ? round_to(c.operand_dtype, w) : w;
}

__device__ __forceinline__ void encode_input(const MlpConfig& c, const void* inputs, int64_t s, float* a0)
{
    const int opd = operand_type(c);
    if (c.encoding == MLP_ENC_FREQ2D) {
        for (int u = 0; u < 2; ++u) {
            const float v = load_as_f32(c.input_dtype, inputs, s * 2 + u);
            for (int k = 0; k < 8; ++k) {
                const float arg = ldexpf(3.14159265358979323846f, k) * v;
                a0[u * 16 + k * 2 + 0] = round_to(opd, sinf(arg));
                a0[u * 16 + k * 2 + 1] = round_to(opd, cosf(arg));
            }
        }
    } else {
        for (int i = 0; i < c.dims[0]; ++i)
            a0[i] = round_to(opd, load_as_f32(c.input_dtype, inputs, s * c.dims[0] + i));
    }
}

// One term of a scalar sum in the order MlpConfig.sum_order names: a fused multiply-add, or a rounded
// product followed by a rounded add (this file is compiled with -fmad=false, so `acc + a * b` is two
// roundings).
__device__ __forceinline__ float mac(float a, float b, float acc, bool fused)
{
    return fused ? fmaf(a, b, acc) : acc + __fmul_rn(a, b);
}

// Forward of one sample; a holds every layer's input vector, z every pre-activation (both rounded to
// the storage type); the last slot of a holds the fp32 outputs.
__device__ void simt_forward(const SimtNet& net, const MlpLayerPointers* __restrict__ lp, const void* inputs, int64_t s,
                             float* a, float* z)
{
    const MlpConfig& c = net.cfg;
    const bool fused = c.sum_order == MLP_SUM_BIAS_FIRST_FUSED;
    encode_input(c, inputs, s, a);
    for (int l = 0; l < c.n_layers; ++l) {
        const int in = c.dims[l], out = c.dims[l + 1];
        const bool last = (l == c.n_layers - 1);
        const float* ain = a + net.a_off[l];
        float* aout = a + net.a_off[l + 1];
        float* zl = z + net.a_off[l + 1] - net.a_off[1];
        const void* W = (const void*)lp[l].weights;
        const void* B = (const void*)lp[l].biases;
        for (int j = 0; j < out; ++j) {
            const float bias = load_as_f32(c.dtype, B, j);
            float r;
            if (fused) {
                r = bias;
                for (int i = 0; i < in; ++i) r = fmaf(load_weight(c, W, weight_index(c.param_layout, in, out, j, i)), ain[i], r);
            } else {
                r = 0.0f;
                for (int i = 0; i < in; ++i) r = mac(load_weight(c, W, weight_index(c.param_layout, in, out, j, i)), ain[i], r, false);
                r = r + bias;
            }
            const float zs = round_to(c.dtype, r);
            zl[j] = zs;
            aout[j] = last ? act_value(c.output_act, c.act_alpha, zs)
                           : round_to(operand_type(c), act_value(c.hidden_act, c.act_alpha, zs));
        }
    }
}

__global__ void __launch_bounds__(256)
forward_simt_kernel(SimtNet net, const MlpLayerPointers* __restrict__ lp, const void* __restrict__ inputs,
                    float* __restrict__ outputs, uint32_t count)
{
    const uint32_t tid = blockIdx.x * blockDim.x + threadIdx.x;
    if (tid >= count) return;
    float a[kMaxActFloats], z[kMaxActFloats];
    simt_forward(net, lp, inputs, tid, a, z);
    const int od = net.cfg.dims[net.cfg.n_layers];
    const float* o = a + net.a_off[net.cfg.n_layers];
    for (int j = 0; j < od; ++j) outputs[int64_t(tid) * od + j] = o[j];
}

// learnGradient, generic.  Phase A (per thread): forward, loss, backward; every layer's input vector
// a_l and output gradient dz_l stay in the per-thread arrays.  Phase B (per block): for each layer the
// block stages `group` samples' (dz_l, a_l) in shared memory and each thread owns a strided set of
// parameters, summing its terms over the staged samples in ascending order before one atomic add per
// parameter per group.  With MLP_FLAG_SEQUENTIAL_SUM the per-sample vectors go to a global scratch
// area instead and a second kernel adds them one sample at a time.
__global__ void __launch_bounds__(256)
learn_gradient_simt_kernel(SimtNet net, const MlpLayerPointers* __restrict__ lp, uint32_t* lossBuffer,
                           const void* __restrict__ inputs, const void* __restrict__ targets, uint32_t count,
                           int group, float* __restrict__ seq_scratch, float* __restrict__ input_grads)
{
    extern __shared__ float smem[];
    const MlpConfig& c = net.cfg;
    const int nl = c.n_layers;
    const uint32_t tid = blockIdx.x * blockDim.x + threadIdx.x;
    const bool valid = tid < count;
    float a[kMaxActFloats];   // inputs of every layer; outputs in the last slot
    float zd[kMaxActFloats];  // pre-activations going forward, overwritten by dz going backward
    float loss = 0.0f;
    const int od = c.dims[nl];
    const bool fused = c.sum_order == MLP_SUM_BIAS_FIRST_FUSED;
    if (valid) {
        simt_forward(net, lp, inputs, tid, a, zd);
        const float scale = (c.loss == MLP_LOSS_MSE_MEAN) ? 1.0f / float(od) : 1.0f;
        const float* o = a + net.a_off[nl];
        float* dzl = zd + net.a_off[nl] - net.a_off[1];
        for (int j = 0; j < od; ++j) {
            const float t = load_as_f32(c.target_dtype, targets, int64_t(tid) * od + j);
            const float diff = o[j] - t;
            loss = fmaf(diff * scale, diff, loss);
            const float dout = (2.0f * scale) * diff;
            const float d = act_deriv(c.output_act, c.act_alpha, dzl[j]);
            dzl[j] = round_to(operand_type(c), dout * d);
        }
        for (int l = nl - 1; l >= 1; --l) {
            const int in = c.dims[l], out = c.dims[l + 1];
            const float* dz = zd + net.a_off[l + 1] - net.a_off[1];
            float* zprev = zd + net.a_off[l] - net.a_off[1];
            const void* W = (const void*)lp[l].weights;
            for (int i = 0; i < in; ++i) {
                float r = 0.0f;
                for (int j = 0; j < out; ++j) r = mac(load_weight(c, W, weight_index(c.param_layout, in, out, j, i)), dz[j], r, fused);
                const float d = round_to(operand_type(c), act_deriv(c.hidden_act, c.act_alpha, zprev[i]));
                zprev[i] = round_to(operand_type(c), r * d);
            }
        }
        if (input_grads) {
            // dx = W_0^T dz_0: dead in the example (its inputs are no_diff), wanted by an encoder in front
            const int in = c.dims[0], out = c.dims[1];
            const float* dz = zd;
            const void* W = (const void*)lp[0].weights;
            for (int i = 0; i < in; ++i) {
                float r = 0.0f;
                for (int j = 0; j < out; ++j) r = mac(load_weight(c, W, weight_index(c.param_layout, in, out, j, i)), dz[j], r, fused);
                input_grads[int64_t(tid) * in + i] = round_to(c.dtype, r);
            }
        }
    }

    // Loss words: wave max folded in by the first lane; block sum added once.
    {
        float m = loss;
        for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
        float sum = loss;
        for (int o = 16; o > 0; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
        if ((threadIdx.x & 31) == 0) {
            if (blockIdx.x * blockDim.x + (threadIdx.x & ~31u) < count) atomicMax(lossBuffer, __float_as_uint(m));
            atomicAdd((float*)(lossBuffer + 1), sum);
        }
    }

    if (seq_scratch) {
        // Layout per sample: [a of all layers (a_off[nl] floats)][dz of all layers (a_off[nl+1]-a_off[1] floats)].
        if (valid) {
            const int na = net.a_off[nl], nz = net.a_off[nl + 1] - net.a_off[1];
            float* dst = seq_scratch + int64_t(tid) * (na + nz);
            for (int i = 0; i < na; ++i) dst[i] = a[i];
            for (int i = 0; i < nz; ++i) dst[na + i] = zd[i];
        }
        return;
    }

    const int first = blockIdx.x * blockDim.x;
    const int n_block = count > (uint32_t)first ? min((int)blockDim.x, (int)(count - first)) : 0;
    for (int l = 0; l < nl; ++l) {
        const int in = c.dims[l], out = c.dims[l + 1];
        const float* al = a + net.a_off[l];
        const float* dz = zd + net.a_off[l + 1] - net.a_off[1];
        float* dW = (float*)lp[l].weightsGrad;
        float* dB = (float*)lp[l].biasesGrad;
        const int stride = in + out;
        for (int g0 = 0; g0 < n_block; g0 += group) {
            const int gn = min(group, n_block - g0);
            __syncthreads();
            const int local = (int)threadIdx.x - g0;
            if (local >= 0 && local < gn) {
                float* row = smem + local * stride;
                for (int i = 0; i < in; ++i) row[i] = al[i];
                for (int j = 0; j < out; ++j) row[in + j] = dz[j];
            }
            __syncthreads();
            for (int p = threadIdx.x; p < in * out + out; p += blockDim.x) {
                float acc = 0.0f;
                if (p < in * out) {
                    const int j = p / in, i = p % in;
                    for (int s = 0; s < gn; ++s) acc = mac(smem[s * stride + in + j], smem[s * stride + i], acc, fused);
                    atomicAdd(dW + weight_index(c.param_layout, in, out, j, i), acc);
                } else {
                    const int j = p - in * out;
                    for (int s = 0; s < gn; ++s) acc += smem[s * stride + in + j];
                    atomicAdd(dB + j, acc);
                }
            }
        }
    }
}

// Second pass of the sequential mode: one thread per parameter walks the samples in ascending order,
// exactly the adds a sequential machine performs (load, fused multiply-add, store).
__global__ void __launch_bounds__(256)
sequential_sum_kernel(SimtNet net, const MlpLayerPointers* __restrict__ lp, const float* __restrict__ scratch,
                      uint32_t count, int layer)
{
    const MlpConfig& c = net.cfg;
    const bool fused = c.sum_order == MLP_SUM_BIAS_FIRST_FUSED;
    const int in = c.dims[layer], out = c.dims[layer + 1];
    const int p = blockIdx.x * blockDim.x + threadIdx.x;
    if (p >= in * out + out) return;
    const int nl = c.n_layers;
    const int na = net.a_off[nl], nz = net.a_off[nl + 1] - net.a_off[1];
    const int64_t stride = na + nz;
    const float* abase = scratch + net.a_off[layer];
    const float* zbase = scratch + na + net.a_off[layer + 1] - net.a_off[1];
    if (p < in * out) {
        const int j = p / in, i = p % in;
        float* dst = (float*)lp[layer].weightsGrad + weight_index(c.param_layout, in, out, j, i);
        float acc = *dst;
        for (uint32_t s = 0; s < count; ++s) acc = mac(zbase[s * stride + j], abase[s * stride + i], acc, fused);
        *dst = acc;
    } else {
        const int j = p - in * out;
        float* dst = (float*)lp[layer].biasesGrad + j;
        float acc = *dst;
        for (uint32_t s = 0; s < count; ++s) acc += zbase[s * stride + j];
        *dst = acc;
    }
}

// adjustParameters, fp32 state (examples/mlp-training/adam.slang:21-37 widened to float):
// NaN gradient -> zero it and skip; +-inf -> +-10000; eps inside the square root; gradient zeroed.
__global__ void __launch_bounds__(256)
adjust_parameters_kernel(MlpConfig c, MlpAdamState* __restrict__ states, void* __restrict__ params,
                         float* __restrict__ grads, uint32_t count)
{
    const uint32_t i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= count) return;
    float g = grads[i];
    if (isnan(g)) { grads[i] = 0.0f; return; }
    float4 raw = reinterpret_cast<float4*>(states)[i];
    float mean = raw.x, var = raw.y;
    int32_t it = __float_as_int(raw.z) + 1;
    if (isinf(g)) g = g > 0.0f ? 10000.0f : -10000.0f;
    mean = c.beta1 * mean + (1.0f - c.beta1) * g;
    var = c.beta2 * var + ((1.0f - c.beta2) * g) * g;
    const float mean_hat = __fdiv_rn(mean, 1.0f - pow_int(c.beta1, it));
    const float var_hat = __fdiv_rn(var, 1.0f - pow_int(c.beta2, it));
    float p = c.adam_master ? raw.w : load_as_f32(c.dtype, params, i);
    const float denom = __fsqrt_rn(fmaxf(0.0f, var_hat) + c.eps);
    p = p - __fdiv_rn(c.lr * mean_hat, denom);
    reinterpret_cast<float4*>(states)[i] = make_float4(mean, var, __int_as_float(it), p);
    store_from_f32(c.dtype, params, i, p);
    grads[i] = 0.0f;
}

// ------------------------------------------------------------------------------------------------
// Host launchers
// ------------------------------------------------------------------------------------------------
static bool make_simt_net(const MlpConfig& c, SimtNet* net, std::string* err)
{
    net->cfg = c;
    int off = 0;
    for (int l = 0; l <= c.n_layers; ++l) { net->a_off[l] = off; off += c.dims[l]; }
    net->a_off[c.n_layers + 1] = off;
    if (off > kMaxActFloats) {
        if (err) *err = "sum of layer widths exceeds the per-thread limit of the one-thread-per-sample kernels";
        return false;
    }
    return true;
}

cudaError_t launch_example_learn_gradient(cudaStream_t st, const MlpLearnGradParams& a, uint32_t grid)
{
    learnGradient<<<grid, 256, 0, st>>>((const MlpLayerPointers*)a.networkBuffer, (uint32_t*)a.lossBuffer,
                                        (const float2*)a.inputs, a.count);
    return cudaGetLastError();
}

cudaError_t launch_example_learn_gradient_coopvec(cudaStream_t st, const MlpLearnGradParams& a, uint32_t grid)
{
    learnGradient_coopvec<<<grid, 256, 0, st>>>((const MlpLayerPointers*)a.networkBuffer, (uint32_t*)a.lossBuffer,
                                                (const float2*)a.inputs, a.count);
    return cudaGetLastError();
}

cudaError_t launch_example_adjust_parameters(cudaStream_t st, const MlpAdjustParamsParams& a, uint32_t grid)
{
    adjustParameters<<<grid, 256, 0, st>>>((MlpExampleAdamState*)a.adamStates, (__half*)a.params, (__half*)a.gradients,
                                           a.count);
    return cudaGetLastError();
}

cudaError_t launch_forward_simt(cudaStream_t st, const MlpConfig& c, const MlpForwardParams& a, int* launches,
                                std::string* err)
{
    SimtNet net;
    if (!make_simt_net(c, &net, err)) return cudaErrorInvalidValue;
    if (a.count == 0) return cudaSuccess;
    const uint32_t grid = (a.count + 255) / 256;
    forward_simt_kernel<<<grid, 256, 0, st>>>(net, (const MlpLayerPointers*)a.networkBuffer, (const void*)a.inputs,
                                              (float*)a.outputs, a.count);
    *launches += 1;
    return cudaGetLastError();
}

cudaError_t launch_learn_gradient_simt(cudaStream_t st, const MlpConfig& c, const MlpLearnGradParamsEx& a,
                                       float* seq_scratch, int* launches, std::string* err, float* input_grads)
{
    SimtNet net;
    if (!make_simt_net(c, &net, err)) return cudaErrorInvalidValue;
    if (a.count == 0) return cudaSuccess;
    int max_stride = 0;
    for (int l = 0; l < c.n_layers; ++l) max_stride = std::max(max_stride, c.dims[l] + c.dims[l + 1]);
    const int budget = 96 * 1024;
    int group = budget / (max_stride * 4);
    group = std::min(256, group / 32 * 32);
    if (group < 32) {
        if (err) *err = "layer too wide for the one-thread-per-sample kernel's staging buffer";
        return cudaErrorInvalidValue;
    }
    const size_t smem = size_t(group) * max_stride * 4;
    {
        cudaError_t e = cudaFuncSetAttribute(learn_gradient_simt_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, budget);
        if (e != cudaSuccess) return e;
    }
    const uint32_t grid = (a.count + 255) / 256;
    const bool seq = (a.flags & MLP_FLAG_SEQUENTIAL_SUM) != 0;
    learn_gradient_simt_kernel<<<grid, 256, smem, st>>>(net, (const MlpLayerPointers*)a.networkBuffer,
                                                        (uint32_t*)a.lossBuffer, (const void*)a.inputs,
                                                        (const void*)a.targets, a.count, group,
                                                        seq ? seq_scratch : nullptr, input_grads);
    *launches += 1;
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess || !seq) return e;
    for (int l = 0; l < c.n_layers; ++l) {
        const int np = c.dims[l] * c.dims[l + 1] + c.dims[l + 1];
        sequential_sum_kernel<<<(np + 255) / 256, 256, 0, st>>>(net, (const MlpLayerPointers*)a.networkBuffer,
                                                                seq_scratch, a.count, l);
        *launches += 1;
    }
    return cudaGetLastError();
}

size_t sequential_scratch_floats_per_sample(const MlpConfig& c)
{
    size_t n = 0;
    for (int l = 0; l < c.n_layers; ++l) n += size_t(c.dims[l]) + size_t(c.dims[l + 1]);
    return n;
}

cudaError_t launch_adjust_parameters(cudaStream_t st, const MlpConfig& c, const MlpAdjustParamsParams& a, int* launches)
{
    if (a.count == 0) return cudaSuccess;
    adjust_parameters_kernel<<<(a.count + 255) / 256, 256, 0, st>>>(c, (MlpAdamState*)a.adamStates, (void*)a.params,
                                                                   (float*)a.gradients, a.count);
    *launches += 1;
    return cudaGetLastError();
}

// ------------------------------------------------------------------------------------------------
// learnGradient with ordered sums and no allocation
// ------------------------------------------------------------------------------------------------
// The ordered-sum mode parks every sample's layer inputs and output gradients in global memory
// between its two passes.  The variant below keeps that parking area inside the library image
// instead of asking the CUDA allocator for it: 4 MiB per GPU that has loaded the library, resident
// until the process exits.
constexpr size_t kStaticScratchFloats = size_t(1) << 20;
static __device__ __align__(256) float g_static_scratch[kStaticScratchFloats];

// In host code `g_static_scratch` is only a handle for the symbol; the address a kernel may
// dereference differs per device and comes from cudaGetSymbolAddress with that device current.
constexpr int kMaxDevices = 64;
static float* g_static_scratch_addr[kMaxDevices] = {};

void set_last_error(const char* text);                    // abi.cu
bool config_ok(const MlpConfig* c, std::string* why);     // abi.cu

}  // namespace mlpb200

using namespace mlpb200;

extern "C" int32_t mlp_learn_gradient_ordered_noalloc(int32_t device_ordinal, void* cuda_stream, const MlpConfig* config,
                                                      const MlpLearnGradParamsEx* args)
{
    // Everything that can be refused is refused here, before the first CUDA call.
    if (!config || !args) { set_last_error("null argument"); return MLP_E_INVALID_ARG; }
    if (device_ordinal < 0 || device_ordinal >= kMaxDevices) { set_last_error("device ordinal out of range"); return MLP_E_INVALID_ARG; }
    {
        std::string why;
        if (!config_ok(config, &why)) { set_last_error(("bad config: " + why).c_str()); return MLP_E_INVALID_ARG; }
    }
    const MlpConfig& c = *config;
    if (c.param_layout != MLP_PARAMS_ROW_MAJOR) { set_last_error("learnGradient takes row-major parameters"); return MLP_E_NOT_AVAILABLE; }
    if (args->flags & MLP_FLAG_INPUT_GRADIENT) {
        set_last_error("this entry point takes MlpLearnGradParamsEx, which has no input-gradient address: MLP_FLAG_INPUT_GRADIENT is not available here");
        return MLP_E_NOT_AVAILABLE;
    }
    if (args->flags & ~MLP_FLAG_SEQUENTIAL_SUM) { set_last_error("unknown flag bits"); return MLP_E_INVALID_ARG; }
    if (!args->networkBuffer || !args->lossBuffer || (args->count && (!args->inputs || !args->targets))) {
        set_last_error("null device address in the argument struct");
        return MLP_E_INVALID_ARG;
    }
    const size_t need = sequential_scratch_floats_per_sample(c) * size_t(args->count);
    if (need > kStaticScratchFloats) {
        char buf[256];
        snprintf(buf, sizeof buf,
                 "%u samples need %zu scratch floats; the built-in scratch area holds %zu (at most %zu samples of this network)",
                 args->count, need, (size_t)kStaticScratchFloats,
                 (size_t)kStaticScratchFloats / sequential_scratch_floats_per_sample(c));
        set_last_error(buf);
        return MLP_E_INVALID_ARG;
    }
    // The work runs with device_ordinal current; the caller's current device is put back on return.
    int prev_device = -1;
    cudaError_t e = cudaGetDevice(&prev_device);
    if (e == cudaSuccess && prev_device != device_ordinal) e = cudaSetDevice(device_ordinal);
    if (e == cudaSuccess && !g_static_scratch_addr[device_ordinal]) {
        // First call on this device: look the array's device address up once and keep it.
        float* addr = nullptr;
        e = cudaGetSymbolAddress((void**)&addr, g_static_scratch);
        if (e == cudaSuccess) g_static_scratch_addr[device_ordinal] = addr;
    }
    int32_t rc = MLP_OK;
    if (e != cudaSuccess) {
        std::string msg = std::string("CUDA set-up for the built-in scratch area failed: ") + cudaGetErrorString(e);
        set_last_error(msg.c_str());
        rc = MLP_E_CUDA;
    } else if (args->count != 0) {
        MlpLearnGradParamsEx a = *args;
        a.flags |= MLP_FLAG_SEQUENTIAL_SUM;
        int launches = 0;
        std::string err;
        e = launch_learn_gradient_simt((cudaStream_t)cuda_stream, c, a, g_static_scratch_addr[device_ordinal], &launches, &err);
        if (e != cudaSuccess) {
            if (err.empty()) err = std::string("kernel launch failed: ") + cudaGetErrorString(e);
            set_last_error(err.c_str());
            rc = e == cudaErrorInvalidValue ? MLP_E_NOT_AVAILABLE : MLP_E_CUDA;
        }
    }
    if (prev_device >= 0 && prev_device != device_ordinal) cudaSetDevice(prev_device);
    return rc;
}
