// The C ABI: devices, buffers, kernel handles and dispatch over the CUDA runtime.
// One function per call the reference's example host loop makes through slang-rhi
// (examples/mlp-training/mlp-training.cpp:92-312); see include/slang_b200_mlp.h.
#include <cuda.h>
#include <cuda_runtime.h>

#include <cstdarg>
#include <cstdio>
#include <cstring>
#include <string>

#include "abi_internal.h"
#include "launchers.h"
#include "mlp_common.cuh"

using namespace mlpb200;

namespace {

thread_local std::string g_last_error;

int32_t fail(int32_t code, const char* fmt, ...)
{
    char buf[512];
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(buf, sizeof buf, fmt, ap);
    va_end(ap);
    g_last_error = buf;
    return code;
}

#define CUDA_TRY(expr)                                                                                   \
    do {                                                                                                 \
        cudaError_t e_ = (expr);                                                                         \
        if (e_ != cudaSuccess) return fail(MLP_E_CUDA, "%s failed: %s", #expr, cudaGetErrorString(e_)); \
    } while (0)

enum class Entry { ExampleLearn, ExampleLearnCoopVec, ExampleAdjust, Learn, LearnSimt, Adjust, Forward, ForwardNarrow, ForwardWide, ForwardSimt, Module };

// Driver entry points for caller-supplied device modules, resolved through the runtime so that the
// library carries no link-time dependency on the driver library.
struct DriverApi {
    CUresult (*moduleLoadData)(CUmodule*, const void*) = nullptr;
    CUresult (*moduleUnload)(CUmodule) = nullptr;
    CUresult (*moduleGetFunction)(CUfunction*, CUmodule, const char*) = nullptr;
    CUresult (*launchKernel)(CUfunction, unsigned, unsigned, unsigned, unsigned, unsigned, unsigned, unsigned, CUstream,
                             void**, void**) = nullptr;
    CUresult (*getErrorString)(CUresult, const char**) = nullptr;
    CUresult (*funcGetParamInfo)(CUfunction, size_t, size_t*, size_t*) = nullptr;  // optional
    bool ok = false;
};

const DriverApi& driver_api()
{
    static DriverApi api = [] {
        DriverApi a;
        auto get = [](const char* name, void** fn) {
            cudaDriverEntryPointQueryResult q;
            return cudaGetDriverEntryPoint(name, fn, cudaEnableDefault, &q) == cudaSuccess && q == cudaDriverEntryPointSuccess && *fn;
        };
        a.ok = get("cuModuleLoadData", (void**)&a.moduleLoadData) && get("cuModuleUnload", (void**)&a.moduleUnload) &&
               get("cuModuleGetFunction", (void**)&a.moduleGetFunction) && get("cuLaunchKernel", (void**)&a.launchKernel) &&
               get("cuGetErrorString", (void**)&a.getErrorString);
        if (!get("cuFuncGetParamInfo", (void**)&a.funcGetParamInfo)) a.funcGetParamInfo = nullptr;
        return a;
    }();
    return api;
}

const char* cu_error(CUresult r)
{
    const char* s = nullptr;
    if (driver_api().getErrorString && driver_api().getErrorString(r, &s) == CUDA_SUCCESS && s) return s;
    return "unknown driver error";
}

}  // namespace

namespace mlpb200 {
// Lets the other translation units report through mlp_last_error_string().
void set_last_error(const char* text) { g_last_error = text ? text : ""; }

// The one validity check of a problem description; every entry point that takes an MlpConfig runs it.
bool config_ok(const MlpConfig* c, std::string* why)
{
    if (!c) { *why = "null config"; return false; }
    if (c->n_layers < 1 || c->n_layers > MLP_MAX_LAYERS) { *why = "n_layers out of range"; return false; }
    for (int l = 0; l <= c->n_layers; ++l)
        if (c->dims[l] < 1 || c->dims[l] > 1024) { *why = "layer width out of range"; return false; }
    if (c->dtype < MLP_F32 || c->dtype > MLP_BF16 || c->input_dtype < MLP_F32 || c->input_dtype > MLP_BF16 ||
        c->target_dtype < MLP_F32 || c->target_dtype > MLP_BF16) { *why = "unknown dtype"; return false; }
    if (c->hidden_act < MLP_ACT_IDENTITY || c->hidden_act > MLP_ACT_LEAKY_MAX || c->output_act < MLP_ACT_IDENTITY ||
        c->output_act > MLP_ACT_LEAKY_MAX) { *why = "unknown activation"; return false; }
    if (c->loss != MLP_LOSS_MSE_MEAN && c->loss != MLP_LOSS_L2_SUM) { *why = "unknown loss"; return false; }
    if (c->sum_order != MLP_SUM_NEURAL && c->sum_order != MLP_SUM_BIAS_FIRST_FUSED) { *why = "unknown sum_order"; return false; }
    if (c->param_layout != MLP_PARAMS_ROW_MAJOR && c->param_layout != MLP_PARAMS_OPTIMAL) { *why = "unknown param_layout"; return false; }
    if (c->operand_dtype != 0 && !(c->dtype == MLP_F32 && (c->operand_dtype == MLP_F16 || c->operand_dtype == MLP_BF16))) {
        *why = "operand_dtype must be 0, or MLP_F16 / MLP_BF16 with dtype = MLP_F32"; return false;
    }
    if (c->encoding == MLP_ENC_FREQ2D && (c->dims[0] != 32 || c->input_width != 2)) {
        *why = "frequency encoding needs dims[0] = 32 and input_width = 2"; return false;
    }
    if (c->encoding == MLP_ENC_NONE && c->input_width != c->dims[0]) { *why = "input_width must equal dims[0]"; return false; }
    if (c->encoding != MLP_ENC_NONE && c->encoding != MLP_ENC_FREQ2D) { *why = "unknown encoding"; return false; }
    return true;
}
}  // namespace mlpb200

struct MlpBuffer {
    int ordinal = 0;
    void* ptr = nullptr;
    size_t size = 0;
    bool owned = false;
};

struct MlpKernel {
    Entry entry;
    MlpConfig cfg;
    const char* impl;
    int ordinal = 0;
    CUmodule module = nullptr;     // Entry::Module only
    CUfunction function = nullptr;
    size_t param_bytes = 0;        // end of the last launch parameter; 0 = unknown
};

extern "C" {

const char* mlp_last_error_string(void) { return g_last_error.c_str(); }

static int32_t device_create(int32_t ordinal, bool borrow_stream, void* cuda_stream, MlpDevice** out_device)
{
    if (!out_device) return fail(MLP_E_INVALID_ARG, "out_device is null");
    *out_device = nullptr;
    int n = 0;
    cudaError_t e = cudaGetDeviceCount(&n);
    if (e != cudaSuccess || n == 0)
        return fail(MLP_E_CUDA, "no CUDA device: %s (this library has no CPU fallback)", cudaGetErrorString(e));
    if (ordinal < 0 || ordinal >= n) return fail(MLP_E_INVALID_ARG, "device ordinal %d out of range (0..%d)", ordinal, n - 1);
    CUDA_TRY(cudaSetDevice(ordinal));
    cudaDeviceProp prop;
    CUDA_TRY(cudaGetDeviceProperties(&prop, ordinal));
    if (prop.major != 10)
        return fail(MLP_E_NOT_AVAILABLE, "device %d is sm_%d%d; the kernels are built for sm_100a only", ordinal, prop.major, prop.minor);
    MlpDevice* d = new MlpDevice();
    d->ordinal = ordinal;
    if (borrow_stream) {
        d->stream = (cudaStream_t)cuda_stream;  // a null handle is the legacy default stream
    } else {
        cudaError_t se = cudaStreamCreateWithFlags(&d->stream, cudaStreamNonBlocking);
        if (se != cudaSuccess) { delete d; return fail(MLP_E_CUDA, "cudaStreamCreate failed: %s", cudaGetErrorString(se)); }
        d->owns_stream = true;
    }
    std::string err;
    d->tc = tc_workspace_create(ordinal, &err);
    if (!d->tc) {
        if (d->owns_stream) cudaStreamDestroy(d->stream);
        delete d;
        return fail(MLP_E_CUDA, "tensor-core workspace: %s", err.c_str());
    }
    *out_device = d;
    return MLP_OK;
}

int32_t mlp_device_create(int32_t ordinal, MlpDevice** out_device)
{
    return device_create(ordinal, false, nullptr, out_device);
}

int32_t mlp_device_create_on_stream(int32_t ordinal, void* cuda_stream, MlpDevice** out_device)
{
    return device_create(ordinal, true, cuda_stream, out_device);
}

int32_t mlp_device_destroy(MlpDevice* d)
{
    if (!d) return MLP_OK;
    cudaSetDevice(d->ordinal);
    cudaStreamSynchronize(d->stream);
    if (d->seq_scratch) cudaFree(d->seq_scratch);
    tc_workspace_destroy(d->tc);
    if (d->owns_stream) cudaStreamDestroy(d->stream);
    delete d;
    return MLP_OK;
}

int32_t mlp_wait(MlpDevice* d)
{
    if (!d) return fail(MLP_E_INVALID_ARG, "device is null");
    CUDA_TRY(cudaSetDevice(d->ordinal));
    uint32_t status = 0;
    CUDA_TRY(tc_read_status(d->stream, d->tc, &status));
    CUDA_TRY(cudaStreamSynchronize(d->stream));
    if (status != 0) return fail(MLP_E_DEVICE_STATUS, "a kernel gave up on a bounded wait (status word 0x%08x)", status);
    return MLP_OK;
}

uint64_t mlp_device_launch_count(const MlpDevice* d) { return d ? d->launches : 0; }

int32_t mlp_buffer_create(MlpDevice* d, size_t size, const void* init_data, MlpBuffer** out_buffer)
{
    if (!d || !out_buffer) return fail(MLP_E_INVALID_ARG, "null argument");
    *out_buffer = nullptr;
    CUDA_TRY(cudaSetDevice(d->ordinal));
    void* p = nullptr;
    CUDA_TRY(cudaMalloc(&p, size ? size : 1));
    if (init_data) {
        cudaError_t e = cudaMemcpyAsync(p, init_data, size, cudaMemcpyHostToDevice, d->stream);
        if (e == cudaSuccess) e = cudaStreamSynchronize(d->stream);
        if (e != cudaSuccess) { cudaFree(p); return fail(MLP_E_CUDA, "initial upload failed: %s", cudaGetErrorString(e)); }
    }
    MlpBuffer* b = new MlpBuffer();
    b->ordinal = d->ordinal; b->ptr = p; b->size = size; b->owned = true;
    *out_buffer = b;
    return MLP_OK;
}

int32_t mlp_buffer_wrap(MlpDevice* d, uint64_t device_address, size_t size, MlpBuffer** out_buffer)
{
    if (!d || !out_buffer || !device_address) return fail(MLP_E_INVALID_ARG, "null argument");
    MlpBuffer* b = new MlpBuffer();
    b->ordinal = d->ordinal; b->ptr = (void*)device_address; b->size = size; b->owned = false;
    *out_buffer = b;
    return MLP_OK;
}

int32_t mlp_buffer_destroy(MlpBuffer* b)
{
    if (!b) return MLP_OK;
    if (b->owned) { cudaSetDevice(b->ordinal); cudaFree(b->ptr); }
    delete b;
    return MLP_OK;
}

uint64_t mlp_buffer_address(const MlpBuffer* b) { return b ? (uint64_t)b->ptr : 0; }

int32_t mlp_buffer_clear(MlpDevice* d, MlpBuffer* b, size_t offset, size_t size)
{
    if (!d || !b) return fail(MLP_E_INVALID_ARG, "null argument");
    if (offset > b->size || size > b->size - offset) return fail(MLP_E_INVALID_ARG, "clear range outside the buffer");
    CUDA_TRY(cudaSetDevice(d->ordinal));
    CUDA_TRY(cudaMemsetAsync((char*)b->ptr + offset, 0, size, d->stream));
    return MLP_OK;
}

int32_t mlp_buffer_read(MlpDevice* d, const MlpBuffer* b, size_t offset, size_t size, void* dst)
{
    if (!d || !b || !dst) return fail(MLP_E_INVALID_ARG, "null argument");
    if (offset > b->size || size > b->size - offset) return fail(MLP_E_INVALID_ARG, "read range outside the buffer");
    CUDA_TRY(cudaSetDevice(d->ordinal));
    CUDA_TRY(cudaMemcpyAsync(dst, (const char*)b->ptr + offset, size, cudaMemcpyDeviceToHost, d->stream));
    CUDA_TRY(cudaStreamSynchronize(d->stream));
    return MLP_OK;
}

int32_t mlp_buffer_write(MlpDevice* d, MlpBuffer* b, size_t offset, size_t size, const void* src)
{
    if (!d || !b || !src) return fail(MLP_E_INVALID_ARG, "null argument");
    if (offset > b->size || size > b->size - offset) return fail(MLP_E_INVALID_ARG, "write range outside the buffer");
    CUDA_TRY(cudaSetDevice(d->ordinal));
    CUDA_TRY(cudaMemcpyAsync((char*)b->ptr + offset, src, size, cudaMemcpyHostToDevice, d->stream));
    return MLP_OK;
}

int32_t mlp_kernel_get(MlpDevice* d, const char* entry_point, MlpKernel** out_kernel)
{
    if (!d || !entry_point || !out_kernel) return fail(MLP_E_INVALID_ARG, "null argument");
    *out_kernel = nullptr;
    MlpKernel* k = new MlpKernel();
    std::memset(&k->cfg, 0, sizeof k->cfg);
    k->impl = "simt";
    if (!std::strcmp(entry_point, "learnGradient")) k->entry = Entry::ExampleLearn;
    else if (!std::strcmp(entry_point, "learnGradient_coopvec")) k->entry = Entry::ExampleLearnCoopVec;
    else if (!std::strcmp(entry_point, "adjustParameters")) k->entry = Entry::ExampleAdjust;
    else { delete k; return fail(MLP_E_NOT_AVAILABLE, "no entry point named '%s'", entry_point); }
    *out_kernel = k;
    return MLP_OK;
}

int32_t mlp_kernel_get_for_config(MlpDevice* d, const MlpConfig* config, const char* entry_point, MlpKernel** out_kernel)
{
    if (!d || !entry_point || !out_kernel) return fail(MLP_E_INVALID_ARG, "null argument");
    *out_kernel = nullptr;
    std::string why;
    if (!config_ok(config, &why)) return fail(MLP_E_INVALID_ARG, "bad config: %s", why.c_str());
    MlpKernel* k = new MlpKernel();
    k->cfg = *config;
    k->impl = "simt";
    if (!std::strcmp(entry_point, "learnGradient")) {
        if (tc_train_supported(*config)) { k->entry = Entry::Learn; k->impl = "tcgen05"; }
        else k->entry = Entry::LearnSimt;
    } else if (!std::strcmp(entry_point, "learnGradient_simt")) k->entry = Entry::LearnSimt;
    else if (!std::strcmp(entry_point, "adjustParameters")) k->entry = Entry::Adjust;
    else if (!std::strcmp(entry_point, "forward")) {
        if (tc_forward_supported(*config)) { k->entry = Entry::Forward; k->impl = "tcgen05"; }
        else if (tc_train_narrow_supported(*config)) { k->entry = Entry::ForwardNarrow; k->impl = "tcgen05"; }
        else if (tc_forward_wide_supported(*config)) { k->entry = Entry::ForwardWide; k->impl = "tcgen05"; }
        else k->entry = Entry::ForwardSimt;
    } else if (!std::strcmp(entry_point, "forward_simt")) k->entry = Entry::ForwardSimt;
    else { delete k; return fail(MLP_E_NOT_AVAILABLE, "no entry point named '%s'", entry_point); }
    *out_kernel = k;
    return MLP_OK;
}

int32_t mlp_kernel_load(MlpDevice* d, const void* image, size_t image_size, const char* entry_point, MlpKernel** out_kernel)
{
    if (!d || !image || !entry_point || !out_kernel) return fail(MLP_E_INVALID_ARG, "null argument");
    *out_kernel = nullptr;
    if (image_size < 4) return fail(MLP_E_INVALID_ARG, "device module image of %zu bytes is too small", image_size);
    const DriverApi& api = driver_api();
    if (!api.ok) return fail(MLP_E_NOT_AVAILABLE, "the CUDA driver's module entry points could not be resolved");
    CUDA_TRY(cudaSetDevice(d->ordinal));
    CUDA_TRY(cudaFree(nullptr));  // makes the device's primary context current for the driver calls
    // cuModuleLoadData reads a cubin by its header and PTX up to its terminating zero; copy the image so
    // that a text image is terminated whatever the caller passed.
    std::string copy((const char*)image, image_size);
    CUmodule mod = nullptr;
    CUresult r = api.moduleLoadData(&mod, copy.c_str());
    if (r != CUDA_SUCCESS) return fail(MLP_E_CUDA, "cuModuleLoadData failed: %s", cu_error(r));
    CUfunction fn = nullptr;
    r = api.moduleGetFunction(&fn, mod, entry_point);
    if (r != CUDA_SUCCESS) {
        api.moduleUnload(mod);
        return fail(MLP_E_NOT_AVAILABLE, "no entry point named '%s' in the module: %s", entry_point, cu_error(r));
    }
    MlpKernel* k = new MlpKernel();
    std::memset(&k->cfg, 0, sizeof k->cfg);
    k->entry = Entry::Module;
    k->impl = "module";
    k->ordinal = d->ordinal;
    k->module = mod;
    k->function = fn;
    if (api.funcGetParamInfo) {
        size_t off = 0, sz = 0;
        for (size_t i = 0; i < 4096 && api.funcGetParamInfo(fn, i, &off, &sz) == CUDA_SUCCESS; ++i)
            k->param_bytes = off + sz > k->param_bytes ? off + sz : k->param_bytes;
    }
    *out_kernel = k;
    return MLP_OK;
}

int32_t mlp_kernel_destroy(MlpKernel* k)
{
    if (k && k->module) {
        cudaSetDevice(k->ordinal);
        driver_api().moduleUnload(k->module);
    }
    delete k;
    return MLP_OK;
}
const char* mlp_kernel_implementation(const MlpKernel* k) { return k ? k->impl : ""; }

int32_t mlp_dispatch(MlpDevice* d, MlpKernel* k, const void* args, size_t args_size, uint32_t gx, uint32_t gy, uint32_t gz)
{
    if (!d || !k || !args) return fail(MLP_E_INVALID_ARG, "null argument");
    if (k->entry == Entry::Module) {
        // A loaded module's entry point: the packed argument bytes are the kernel's parameter buffer,
        // block (256,1,1) as [numthreads(256,1,1)] declares (tools/gfx/cuda/cuda-command-queue.cpp:122-147).
        if (k->ordinal != d->ordinal) return fail(MLP_E_INVALID_ARG, "the kernel was loaded on device %d, not %d", k->ordinal, d->ordinal);
        if (gx == 0 || gy == 0 || gz == 0) return MLP_OK;
        CUDA_TRY(cudaSetDevice(d->ordinal));
        // A host struct ends with padding up to its alignment (28 bytes of fields become 32); the launch
        // wants exactly the bytes up to the end of the last parameter (tests/cuda/cuda-kernel-param-layout.slang:1-8).
        size_t size = args_size;
        if (k->param_bytes) {
            if (args_size < k->param_bytes)
                return fail(MLP_E_INVALID_ARG, "the entry point takes %zu parameter bytes, got %zu", k->param_bytes, args_size);
            if (args_size - k->param_bytes >= 16)
                return fail(MLP_E_INVALID_ARG, "the entry point takes %zu parameter bytes, got %zu", k->param_bytes, args_size);
            size = k->param_bytes;
        }
        void* extra[] = {CU_LAUNCH_PARAM_BUFFER_POINTER, const_cast<void*>(args), CU_LAUNCH_PARAM_BUFFER_SIZE, &size, CU_LAUNCH_PARAM_END};
        CUresult r = driver_api().launchKernel(k->function, gx, gy, gz, 256, 1, 1, 0, (CUstream)d->stream, nullptr, extra);
        if (r != CUDA_SUCCESS) return fail(MLP_E_CUDA, "cuLaunchKernel failed: %s", cu_error(r));
        d->launches += 1;
        return MLP_OK;
    }
    if (gy != 1 || gz != 1) return fail(MLP_E_INVALID_ARG, "the entry points are one-dimensional: grid must be (n,1,1)");
    CUDA_TRY(cudaSetDevice(d->ordinal));
    int launches = 0;
    std::string err;
    cudaError_t e = cudaSuccess;
    switch (k->entry) {
    case Entry::ExampleLearnCoopVec:
    case Entry::ExampleLearn: {
        // The struct is 28 bytes of fields; hosts pass 28 or the padded 32 (tests/cuda/cuda-kernel-param-layout.slang).
        if (args_size != 28 && args_size != sizeof(MlpLearnGradParams)) return fail(MLP_E_INVALID_ARG, "learnGradient expects 28 or 32 argument bytes, got %zu", args_size);
        MlpLearnGradParams a; std::memset(&a, 0, sizeof a); std::memcpy(&a, args, 28);
        if ((uint64_t)gx * 256 < a.count) return fail(MLP_E_INVALID_ARG, "grid of %u groups does not cover %u samples", gx, a.count);
        if (a.count == 0 || gx == 0) return MLP_OK;
        e = k->entry == Entry::ExampleLearn ? launch_example_learn_gradient(d->stream, a, gx)
                                            : launch_example_learn_gradient_coopvec(d->stream, a, gx);
        launches = 1;
        break;
    }
    case Entry::ExampleAdjust: {
        if (args_size != 28 && args_size != sizeof(MlpAdjustParamsParams)) return fail(MLP_E_INVALID_ARG, "adjustParameters expects 28 or 32 argument bytes, got %zu", args_size);
        MlpAdjustParamsParams a; std::memset(&a, 0, sizeof a); std::memcpy(&a, args, 28);
        if ((uint64_t)gx * 256 < a.count) return fail(MLP_E_INVALID_ARG, "grid of %u groups does not cover %u elements", gx, a.count);
        if (a.count == 0 || gx == 0) return MLP_OK;
        e = launch_example_adjust_parameters(d->stream, a, gx); launches = 1;
        break;
    }
    case Entry::Adjust: {
        if (args_size != 28 && args_size != sizeof(MlpAdjustParamsParams)) return fail(MLP_E_INVALID_ARG, "adjustParameters expects 28 or 32 argument bytes, got %zu", args_size);
        MlpAdjustParamsParams a; std::memset(&a, 0, sizeof a); std::memcpy(&a, args, 28);
        if ((uint64_t)gx * 256 < a.count) return fail(MLP_E_INVALID_ARG, "grid of %u groups does not cover %u elements", gx, a.count);
        e = launch_adjust_parameters(d->stream, k->cfg, a, &launches);
        break;
    }
    case Entry::Learn:
    case Entry::LearnSimt: {
        if (args_size != sizeof(MlpLearnGradParamsEx) && args_size != sizeof(MlpLearnGradParamsEx2))
            return fail(MLP_E_INVALID_ARG, "learnGradient expects %zu or %zu argument bytes, got %zu", sizeof(MlpLearnGradParamsEx),
                        sizeof(MlpLearnGradParamsEx2), args_size);
        MlpLearnGradParamsEx a; std::memcpy(&a, args, sizeof a);
        float* input_grads = nullptr;
        if (a.flags & MLP_FLAG_INPUT_GRADIENT) {
            if (args_size != sizeof(MlpLearnGradParamsEx2)) return fail(MLP_E_INVALID_ARG, "MLP_FLAG_INPUT_GRADIENT needs MlpLearnGradParamsEx2");
            MlpLearnGradParamsEx2 a2; std::memcpy(&a2, args, sizeof a2);
            if (!a2.inputGradients) return fail(MLP_E_INVALID_ARG, "null input-gradient address");
            if (k->cfg.encoding != MLP_ENC_NONE) return fail(MLP_E_NOT_AVAILABLE, "input gradients are not defined through the frequency encoding");
            input_grads = (float*)a2.inputGradients;
        }
        if ((uint64_t)gx * 256 < a.count) return fail(MLP_E_INVALID_ARG, "grid of %u groups does not cover %u samples", gx, a.count);
        if (!a.networkBuffer || !a.lossBuffer || (a.count && (!a.inputs || !a.targets))) return fail(MLP_E_INVALID_ARG, "null device address in the argument struct");
        const bool seq = (a.flags & MLP_FLAG_SEQUENTIAL_SUM) != 0;
        if (k->entry == Entry::Learn && !seq) {
            // both tensor-core kernels also write the input gradients when asked
            e = launch_learn_gradient_tc(d->stream, d->tc, k->cfg, a, &launches, &err, input_grads);
        } else {
            if (seq) {
                const size_t need = sequential_scratch_floats_per_sample(k->cfg) * size_t(a.count);
                if (need > d->seq_scratch_floats) {
                    CUDA_TRY(cudaStreamSynchronize(d->stream));
                    if (d->seq_scratch) CUDA_TRY(cudaFree(d->seq_scratch));
                    d->seq_scratch = nullptr; d->seq_scratch_floats = 0;
                    CUDA_TRY(cudaMalloc((void**)&d->seq_scratch, need * sizeof(float)));
                    d->seq_scratch_floats = need;
                }
            }
            e = launch_learn_gradient_simt(d->stream, k->cfg, a, d->seq_scratch, &launches, &err, input_grads);
        }
        break;
    }
    case Entry::Forward:
    case Entry::ForwardNarrow:
    case Entry::ForwardWide:
    case Entry::ForwardSimt: {
        if (args_size != sizeof(MlpForwardParams)) return fail(MLP_E_INVALID_ARG, "forward expects %zu argument bytes, got %zu", sizeof(MlpForwardParams), args_size);
        MlpForwardParams a; std::memcpy(&a, args, sizeof a);
        if ((uint64_t)gx * 256 < a.count) return fail(MLP_E_INVALID_ARG, "grid of %u groups does not cover %u samples", gx, a.count);
        if (!a.networkBuffer || (a.count && (!a.inputs || !a.outputs))) return fail(MLP_E_INVALID_ARG, "null device address in the argument struct");
        if ((a.flags & MLP_FLAG_OUTPUT_STORAGE_TYPE) && k->entry != Entry::Forward)
            return fail(MLP_E_NOT_AVAILABLE, "MLP_FLAG_OUTPUT_STORAGE_TYPE needs the constant-width tensor-core forward kernel");
        if (k->entry == Entry::Forward) e = launch_forward_tc(d->stream, d->tc, k->cfg, a, &launches, &err);
        else if (k->entry == Entry::ForwardNarrow) e = launch_forward_narrow(d->stream, d->tc, k->cfg, a, &launches, &err);
        else if (k->entry == Entry::ForwardWide) e = launch_forward_wide(d->stream, d->tc, k->cfg, a, &launches, &err);
        else e = launch_forward_simt(d->stream, k->cfg, a, &launches, &err);
        break;
    }
    case Entry::Module: break;  // handled above
    }
    d->launches += (uint64_t)launches;
    if (e != cudaSuccess) {
        if (!err.empty()) return fail(e == cudaErrorInvalidValue ? MLP_E_NOT_AVAILABLE : MLP_E_CUDA, "%s", err.c_str());
        return fail(MLP_E_CUDA, "kernel launch failed: %s", cudaGetErrorString(e));
    }
    return MLP_OK;
}

int32_t mlp_matrix_size(uint32_t rows, uint32_t cols, int32_t component_type, int32_t layout, uint64_t row_col_stride,
                        uint64_t* out_size)
{
    if (!out_size) return fail(MLP_E_INVALID_ARG, "null argument");
    std::string err;
    size_t sz = 0;
    if (!matrix_size(rows, cols, component_type, layout, (size_t)row_col_stride, &sz, &err)) return fail(MLP_E_INVALID_ARG, "%s", err.c_str());
    *out_size = sz;
    return MLP_OK;
}

int32_t mlp_matrix_convert(MlpDevice* d, uint64_t dst_address, const MlpMatrixDesc* dst_descs, uint64_t src_address,
                           const MlpMatrixDesc* src_descs, uint32_t count)
{
    if (!d || !dst_address || !src_address || (count && (!dst_descs || !src_descs))) return fail(MLP_E_INVALID_ARG, "null argument");
    CUDA_TRY(cudaSetDevice(d->ordinal));
    std::string err;
    int launches = 0;
    cudaError_t e = launch_matrix_convert(d->stream, dst_address, dst_descs, src_address, src_descs, count, &launches, &err);
    d->launches += (uint64_t)launches;
    if (e != cudaSuccess) {
        if (!err.empty()) return fail(MLP_E_INVALID_ARG, "%s", err.c_str());
        return fail(MLP_E_CUDA, "kernel launch failed: %s", cudaGetErrorString(e));
    }
    return MLP_OK;
}

int32_t mlp_layout_sizes(const MlpNetworkShape* shape, int64_t* logical_elements, int64_t* physical_elements)
{
    if (!shape || !logical_elements || !physical_elements) return fail(MLP_E_INVALID_ARG, "null argument");
    std::string err;
    long long lo = 0, po = 0;
    if (!layout_sizes(*shape, &lo, &po, &err)) return fail(MLP_E_INVALID_ARG, "bad network shape: %s", err.c_str());
    *logical_elements = lo;
    *physical_elements = po;
    return MLP_OK;
}

static int32_t layout_convert(MlpDevice* d, const MlpNetworkShape* shape, bool to_optimal, uint64_t src, uint64_t dst)
{
    if (!d || !shape || !src || !dst) return fail(MLP_E_INVALID_ARG, "null argument");
    CUDA_TRY(cudaSetDevice(d->ordinal));
    std::string err;
    int launches = 0;
    cudaError_t e = launch_layout_convert(d->stream, *shape, to_optimal, (const void*)src, (void*)dst, &launches, &err);
    d->launches += (uint64_t)launches;
    if (e != cudaSuccess) {
        if (!err.empty()) return fail(MLP_E_INVALID_ARG, "bad network shape: %s", err.c_str());
        return fail(MLP_E_CUDA, "kernel launch failed: %s", cudaGetErrorString(e));
    }
    return MLP_OK;
}

int32_t mlp_layout_to_optimal(MlpDevice* d, const MlpNetworkShape* shape, uint64_t portable, uint64_t optimal)
{
    return layout_convert(d, shape, true, portable, optimal);
}

int32_t mlp_layout_to_portable(MlpDevice* d, const MlpNetworkShape* shape, uint64_t optimal, uint64_t portable)
{
    return layout_convert(d, shape, false, optimal, portable);
}

#ifdef MLPB200_TRACE
// Developer builds only: the time stamps CTA 0 of the last wide tensor-core learnGradient recorded.
int32_t mlpb200_debug_tc_timing(MlpDevice* d, unsigned long long* out256)
{
    if (!d || !out256) return fail(MLP_E_INVALID_ARG, "null argument");
    CUDA_TRY(cudaSetDevice(d->ordinal));
    CUDA_TRY(tc_read_timing(d->stream, d->tc, out256));
    return MLP_OK;
}
#endif

int32_t mlp_param_layout(const MlpConfig* config, int64_t* w_off, int64_t* b_off, int64_t* total)
{
    std::string why;
    if (!config_ok(config, &why)) return fail(MLP_E_INVALID_ARG, "bad config: %s", why.c_str());
    if (!w_off || !b_off || !total) return fail(MLP_E_INVALID_ARG, "null argument");
    Layout L = make_layout(*config);
    for (int l = 0; l < config->n_layers; ++l) { w_off[l] = L.w[l]; b_off[l] = L.b[l]; }
    *total = L.total;
    return MLP_OK;
}

}  // extern "C"
