// Gradient exchange between the GPUs of a data-parallel run, bound directly to NCCL.
//
// The training step shards by samples; the only exchange is the sum of the flat fp32 gradient
// segment (and of the two loss words) after learnGradient.  NCCL is resolved with dlopen at first
// use, so the library loads and every other entry point works where NCCL is not installed.
#include <cuda_runtime.h>
#include <dlfcn.h>
#include <nccl.h>  // types and enumerators only; the functions are resolved at run time

#include <chrono>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <mutex>
#include <string>
#include <thread>

#include "abi_internal.h"

using namespace mlpb200;

namespace {

struct NcclApi {
    ncclResult_t (*getUniqueId)(ncclUniqueId*) = nullptr;
    ncclResult_t (*commInitRank)(ncclComm_t*, int, ncclUniqueId, int) = nullptr;
    ncclResult_t (*commDestroy)(ncclComm_t) = nullptr;
    ncclResult_t (*allReduce)(const void*, void*, size_t, ncclDataType_t, ncclRedOp_t, ncclComm_t, cudaStream_t) = nullptr;
    ncclResult_t (*allGather)(const void*, void*, size_t, ncclDataType_t, ncclComm_t, cudaStream_t) = nullptr;
    ncclResult_t (*groupStart)() = nullptr;
    ncclResult_t (*groupEnd)() = nullptr;
    const char* (*getErrorString)(ncclResult_t) = nullptr;
    ncclResult_t (*commGetAsyncError)(ncclComm_t, ncclResult_t*) = nullptr;  // optional
    ncclResult_t (*commAbort)(ncclComm_t) = nullptr;                         // optional
    bool ok = false;
    std::string why;
};

const NcclApi& nccl_api()
{
    static NcclApi api;
    static std::once_flag once;
    std::call_once(once, [] {
        // SLANG_B200_NCCL_LIBRARY names the library file to bind instead of the default search.
        // A process that already holds an NCCL (a host framework's bundled copy) gets that one back.
        const char* override_path = getenv("SLANG_B200_NCCL_LIBRARY");
        void* h = nullptr;
        if (override_path && *override_path) {
            h = dlopen(override_path, RTLD_NOW | RTLD_GLOBAL);
            if (!h) { api.why = std::string(override_path) + " could not be loaded: " + dlerror(); return; }
        } else {
            h = dlopen("libnccl.so.2", RTLD_NOW | RTLD_GLOBAL);
            if (!h) h = dlopen("libnccl.so", RTLD_NOW | RTLD_GLOBAL);
            if (!h) { api.why = std::string("libnccl.so.2 could not be loaded: ") + dlerror(); return; }
        }
        bool all = true;
        auto get = [&](const char* name, void** fn) { *fn = dlsym(h, name); if (!*fn) { all = false; api.why = std::string("missing NCCL symbol ") + name; } };
        get("ncclGetUniqueId", (void**)&api.getUniqueId);
        get("ncclCommInitRank", (void**)&api.commInitRank);
        get("ncclCommDestroy", (void**)&api.commDestroy);
        get("ncclAllReduce", (void**)&api.allReduce);
        get("ncclAllGather", (void**)&api.allGather);
        get("ncclGroupStart", (void**)&api.groupStart);
        get("ncclGroupEnd", (void**)&api.groupEnd);
        get("ncclGetErrorString", (void**)&api.getErrorString);
        api.ok = all;
        api.commGetAsyncError = (ncclResult_t (*)(ncclComm_t, ncclResult_t*))dlsym(h, "ncclCommGetAsyncError");
        api.commAbort = (ncclResult_t (*)(ncclComm_t))dlsym(h, "ncclCommAbort");
    });
    return api;
}

int32_t comm_fail(int32_t code, const std::string& text)
{
    set_last_error(text.c_str());
    return code;
}

// out[i] = part[0][i] + part[1][i] + ... in ascending rank order (one rounding per add), so that the
// sum does not depend on the collective's algorithm.
__global__ void rank_ordered_sum_kernel(const float* __restrict__ parts, float* __restrict__ out, size_t count, int nranks)
{
    const size_t i = size_t(blockIdx.x) * blockDim.x + threadIdx.x;
    if (i >= count) return;
    float acc = parts[i];
    for (int r = 1; r < nranks; ++r) acc = __fadd_rn(acc, parts[size_t(r) * count + i]);
    out[i] = acc;
}

}  // namespace

struct MlpComm {
    int ordinal = 0;
    int nranks = 1, rank = 0;
    ncclComm_t comm = nullptr;
    float* gather = nullptr;      // nranks x count floats for the rank-ordered sum
    size_t gather_floats = 0;
    float* loss_tmp = nullptr;    // two floats: the loss words leave through here
    cudaEvent_t done = nullptr;   // recorded by mlp_comm_wait behind the collectives it watches
    bool aborted = false;         // mlp_comm_wait gave up on it: only mlp_comm_destroy is valid now
};

#define NCCL_TRY(expr)                                                                                     \
    do {                                                                                                   \
        ncclResult_t r_ = (expr);                                                                          \
        if (r_ != ncclSuccess) return comm_fail(MLP_E_CUDA, std::string(#expr " failed: ") + api.getErrorString(r_)); \
    } while (0)
#define CU_TRY(expr)                                                                                       \
    do {                                                                                                   \
        cudaError_t e_ = (expr);                                                                           \
        if (e_ != cudaSuccess) return comm_fail(MLP_E_CUDA, std::string(#expr " failed: ") + cudaGetErrorString(e_)); \
    } while (0)

extern "C" {

int32_t mlp_comm_unique_id(void* id_out, size_t id_bytes)
{
    if (!id_out) return comm_fail(MLP_E_INVALID_ARG, "null argument");
    if (id_bytes != MLP_COMM_ID_BYTES) return comm_fail(MLP_E_INVALID_ARG, "the id buffer must hold MLP_COMM_ID_BYTES bytes");
    static_assert(sizeof(ncclUniqueId) == MLP_COMM_ID_BYTES, "id size");
    const NcclApi& api = nccl_api();
    if (!api.ok) return comm_fail(MLP_E_NOT_AVAILABLE, api.why);
    ncclUniqueId id;
    NCCL_TRY(api.getUniqueId(&id));
    std::memcpy(id_out, &id, sizeof id);
    return MLP_OK;
}

int32_t mlp_comm_init(MlpDevice* d, int32_t nranks, int32_t rank, const void* id, size_t id_bytes, MlpComm** out_comm)
{
    if (!d || !id || !out_comm) return comm_fail(MLP_E_INVALID_ARG, "null argument");
    *out_comm = nullptr;
    if (id_bytes != MLP_COMM_ID_BYTES) return comm_fail(MLP_E_INVALID_ARG, "the id must be MLP_COMM_ID_BYTES bytes");
    if (nranks < 1 || rank < 0 || rank >= nranks) return comm_fail(MLP_E_INVALID_ARG, "rank outside [0, nranks)");
    const NcclApi& api = nccl_api();
    if (!api.ok) return comm_fail(MLP_E_NOT_AVAILABLE, api.why);
    CU_TRY(cudaSetDevice(d->ordinal));
    ncclUniqueId uid;
    std::memcpy(&uid, id, sizeof uid);
    MlpComm* c = new MlpComm();
    c->ordinal = d->ordinal; c->nranks = nranks; c->rank = rank;
    ncclResult_t r = api.commInitRank(&c->comm, nranks, uid, rank);
    if (r != ncclSuccess) { delete c; return comm_fail(MLP_E_CUDA, std::string("ncclCommInitRank failed: ") + api.getErrorString(r)); }
    cudaError_t e = cudaMalloc((void**)&c->loss_tmp, 2 * sizeof(float));
    if (e != cudaSuccess) { api.commDestroy(c->comm); delete c; return comm_fail(MLP_E_CUDA, std::string("cudaMalloc failed: ") + cudaGetErrorString(e)); }
    *out_comm = c;
    return MLP_OK;
}

int32_t mlp_comm_destroy(MlpComm* c)
{
    if (!c) return MLP_OK;
    cudaSetDevice(c->ordinal);
    if (c->comm && !c->aborted) nccl_api().commDestroy(c->comm);
    if (c->done) cudaEventDestroy(c->done);
    if (c->gather) cudaFree(c->gather);
    if (c->loss_tmp) cudaFree(c->loss_tmp);
    delete c;
    return MLP_OK;
}

int32_t mlp_allreduce_grads(MlpDevice* d, MlpComm* c, uint64_t gradients, size_t count, uint64_t loss_words, uint32_t flags)
{
    if (!d || !c) return comm_fail(MLP_E_INVALID_ARG, "null argument");
    if (d->ordinal != c->ordinal) return comm_fail(MLP_E_INVALID_ARG, "the communicator belongs to another device");
    if (count && !gradients) return comm_fail(MLP_E_INVALID_ARG, "null gradient address");
    if (flags & ~uint32_t(MLP_COMM_RANK_ORDERED_SUM)) return comm_fail(MLP_E_INVALID_ARG, "unknown flag");
    if (c->aborted) return comm_fail(MLP_E_COMM, "the communicator was aborted after an earlier failure");
    const NcclApi& api = nccl_api();
    CU_TRY(cudaSetDevice(d->ordinal));
    float* g = (float*)gradients;
    float* lw = (float*)loss_words;
    const bool ordered = (flags & MLP_COMM_RANK_ORDERED_SUM) != 0 && c->nranks > 1;
    if (ordered && count * size_t(c->nranks) > c->gather_floats) {
        CU_TRY(cudaStreamSynchronize(d->stream));
        if (c->gather) CU_TRY(cudaFree(c->gather));
        c->gather = nullptr; c->gather_floats = 0;
        CU_TRY(cudaMalloc((void**)&c->gather, count * size_t(c->nranks) * sizeof(float)));
        c->gather_floats = count * size_t(c->nranks);
    }
    NCCL_TRY(api.groupStart());
    ncclResult_t r = ncclSuccess;
    if (count) {
        if (ordered) r = api.allGather(g, c->gather, count, ncclFloat32, c->comm, d->stream);
        else r = api.allReduce(g, g, count, ncclFloat32, ncclSum, c->comm, d->stream);
    }
    // The loss words are non-negative floats: word 0 combines by max, word 1 by sum
    // (examples/mlp-training/kernels.slang:22-27 keeps the max; the mean loss needs the sum).
    if (r == ncclSuccess && lw) r = api.allReduce(lw, c->loss_tmp, 1, ncclFloat32, ncclMax, c->comm, d->stream);
    if (r == ncclSuccess && lw) r = api.allReduce(lw + 1, c->loss_tmp + 1, 1, ncclFloat32, ncclSum, c->comm, d->stream);
    ncclResult_t re = api.groupEnd();
    if (r != ncclSuccess) return comm_fail(MLP_E_CUDA, std::string("NCCL collective failed: ") + api.getErrorString(r));
    if (re != ncclSuccess) return comm_fail(MLP_E_CUDA, std::string("ncclGroupEnd failed: ") + api.getErrorString(re));
    if (ordered && count) {
        const unsigned blocks = (unsigned)((count + 255) / 256);
        rank_ordered_sum_kernel<<<blocks, 256, 0, d->stream>>>(c->gather, g, count, c->nranks);
        CU_TRY(cudaGetLastError());
        d->launches += 1;
    }
    if (lw) CU_TRY(cudaMemcpyAsync(lw, c->loss_tmp, 2 * sizeof(float), cudaMemcpyDeviceToDevice, d->stream));
    return MLP_OK;
}

// Host-side watch over the collectives queued so far: returns when the stream has drained, when the
// collective library reports an asynchronous error (a peer died, a link failed), or when the time limit
// passes.  In the last two cases the communicator is aborted, which releases kernels of the library that
// would otherwise wait for the missing peer, and the handle is good for mlp_comm_destroy only.
int32_t mlp_comm_wait(MlpDevice* d, MlpComm* c, uint32_t timeout_ms)
{
    if (!d || !c) return comm_fail(MLP_E_INVALID_ARG, "null argument");
    if (d->ordinal != c->ordinal) return comm_fail(MLP_E_INVALID_ARG, "the communicator belongs to another device");
    if (c->aborted) return comm_fail(MLP_E_COMM, "the communicator was aborted after an earlier failure");
    const NcclApi& api = nccl_api();
    CU_TRY(cudaSetDevice(d->ordinal));
    if (!c->done) CU_TRY(cudaEventCreateWithFlags(&c->done, cudaEventDisableTiming));
    CU_TRY(cudaEventRecord(c->done, d->stream));
    const auto t0 = std::chrono::steady_clock::now();
    std::string why;
    for (;;) {
        const cudaError_t q = cudaEventQuery(c->done);
        ncclResult_t async = ncclSuccess;
        if (api.commGetAsyncError) {
            const ncclResult_t r = api.commGetAsyncError(c->comm, &async);
            if (r != ncclSuccess) async = r;
        }
        if (async != ncclSuccess && async != ncclInProgress) {
            why = std::string("the collective library reported an asynchronous error: ") + api.getErrorString(async);
            break;
        }
        if (q == cudaSuccess) return MLP_OK;
        if (q != cudaErrorNotReady) return comm_fail(MLP_E_CUDA, std::string("cudaEventQuery failed: ") + cudaGetErrorString(q));
        const auto ms = std::chrono::duration_cast<std::chrono::milliseconds>(std::chrono::steady_clock::now() - t0).count();
        if (ms > (long long)timeout_ms) {
            why = "the collectives did not finish within the time limit of " + std::to_string(timeout_ms) + " ms";
            break;
        }
        std::this_thread::sleep_for(std::chrono::microseconds(50));
    }
    if (api.commAbort) api.commAbort(c->comm);
    c->aborted = true;
    return comm_fail(MLP_E_COMM, why + "; the communicator was aborted");
}

}  // extern "C"
