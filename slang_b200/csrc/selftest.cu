// Self-test of the bounded-wait reporting path that every tensor-core kernel of this library relies on.
//
// The kernels never spin without a limit: a wait on an mbarrier gives up after a fixed number of polls,
// raises the CTA's abort flag, records a code in the device status word and lets the CTA tear down
// (tensor memory freed, normal exit); mlp_wait() then reports MLP_E_DEVICE_STATUS once and clears the
// word.  In production that path only runs when something is already wrong.  The kernel below makes it
// run on purpose and harmlessly: one CTA allocates tensor memory, initialises an mbarrier that nobody
// ever arrives on, waits on it with a small poll limit, sees the wait run out, checks that a second
// wait returns at once because the CTA is aborting, frees its tensor memory and exits.  Nothing faults,
// traps or hangs; the context stays usable.
#include <cuda_runtime.h>

#include <string>

#include "abi_internal.h"
#include "tc_host.h"
#include "tc_ptx.cuh"

namespace mlpb200 {

constexpr uint32_t kStatusSelfTest = 0x40000000u;       // the first wait ran out, as intended
constexpr uint32_t kStatusSelfTestLate = 0x20000000u;   // the second wait did not return at once (a defect)

__global__ void __launch_bounds__(64, 1) bounded_wait_selftest_kernel(uint32_t* status, uint32_t max_polls)
{
    using namespace ptx;
    __shared__ __align__(8) uint64_t bar;
    __shared__ uint32_t tmem_ptr;
    __shared__ uint32_t abort_word;
    volatile uint32_t* abort_flag = &abort_word;
    const int warp = threadIdx.x >> 5;
    if (threadIdx.x == 0) {
        mbar_init(&bar, 1);
        abort_word = 0u;
        fence_mbar_init();
    }
    if (warp == 1) {
        tmem_alloc(&tmem_ptr, 32);
        tmem_relinquish();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    if (threadIdx.x == 0) {
        // Nobody arrives on `bar`: this wait runs out after max_polls polls.
        const bool ok = mbar_wait_limited(&bar, 0u, abort_flag, status, kStatusSelfTest, max_polls);
        // The CTA is aborting now: a production-limit wait must come back after at most 64 polls.
        const long long t0 = clock64();
        const bool ok2 = mbar_wait(&bar, 0u, abort_flag, status, kStatusSelfTestLate);
        const long long dt = clock64() - t0;
        if (ok || ok2 || dt > 50000000ll) atomicOr(status, kStatusSelfTestLate);
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        tmem_dealloc(tmem_ptr, 32);
    }
}

}  // namespace mlpb200

using namespace mlpb200;

extern "C" int32_t mlp_selftest_bounded_wait(MlpDevice* d, uint32_t max_polls)
{
    if (!d) { set_last_error("device is null"); return MLP_E_INVALID_ARG; }
    if (max_polls == 0 || max_polls > 100000u) { set_last_error("max_polls must be in 1..100000"); return MLP_E_INVALID_ARG; }
    cudaError_t e = cudaSetDevice(d->ordinal);
    if (e == cudaSuccess) {
        bounded_wait_selftest_kernel<<<1, 64, 0, d->stream>>>(d->tc->status, max_polls);
        e = cudaGetLastError();
    }
    if (e != cudaSuccess) {
        set_last_error((std::string("self-test launch failed: ") + cudaGetErrorString(e)).c_str());
        return MLP_E_CUDA;
    }
    d->launches += 1;
    return MLP_OK;
}
