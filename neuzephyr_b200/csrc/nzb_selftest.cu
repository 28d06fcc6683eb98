// Self-test of the give-up path every kernel of this library shares: a bounded wait on an mbarrier
// that nothing ever arrives at must END -- raise the CTA's abort flag, let every role leave, report
// NZB_ERR_DEVICE_TIMEOUT through the mapped status word -- and leave the context usable. The kernel
// below goes through the same helpers (mbar_wait_bounded_limit, the abort flag, the status write)
// as the GEMM and convolution kernels, with a caller-chosen cycle budget instead of their fixed one,
// no copy in flight and no tensor memory held, so letting the wait run out costs a millisecond and
// cannot hang or fault the GPU.
#include "nzb_internal.h"
#include "nzb_ptx.cuh"

namespace nzb {

__global__ void __launch_bounds__(64, 1) wait_timeout_selftest_kernel(int* status, long long limit, int* roles_left) {
    using namespace ptx;
    __shared__ uint64_t bar;
    __shared__ int abort_word;
    volatile int* abort_flag = &abort_word;
    if (threadIdx.x == 0) {
        mbar_init(&bar, 1);  // one arrival expected; nobody arrives
        abort_word = 0;
        fence_mbar_init();
    }
    __syncthreads();
    const int warp = threadIdx.x >> 5;
    bool ok;
    if (warp == 0) {
        ok = mbar_wait_warp(&bar, 0, abort_flag) ;  // fixed budget: would spin for seconds ...
    } else {
        ok = __all_sync(0xffffffffu, mbar_wait_bounded_limit(&bar, 0, abort_flag, limit));  // ... this one gives up first
    }
    // warp 0 polls the abort flag inside its own wait and leaves as soon as warp 1 has raised it
    if (!ok && (threadIdx.x & 31) == 0) atomicAdd(roles_left, 1);
    __syncthreads();
    if (threadIdx.x == 0 && *abort_flag) {
        *status = NZB_ERR_DEVICE_TIMEOUT;
        __threadfence_system();
    }
}

}  // namespace nzb

using namespace nzb;

extern "C" int nzb_selftest_wait_timeout(long long limit_cycles, int* roles_left_dev, void* stream) {
    if (limit_cycles < 1 || limit_cycles > (1ll << 28))
        return fail(NZB_ERR_BAD_ARG, "limit_cycles must be in [1, 2^28] (about 0.15 s at most)");
    if (!roles_left_dev) return fail(NZB_ERR_BAD_ARG, "roles_left_dev is null");
    DeviceState* ds;
    int rc = get_device_state(&ds);
    if (rc != NZB_OK) return rc;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    NZB_CUDA_TRY(cudaMemsetAsync(roles_left_dev, 0, sizeof(int), s));
    wait_timeout_selftest_kernel<<<1, 64, 0, s>>>(ds->status_dev, limit_cycles, roles_left_dev);
    NZB_CUDA_TRY(cudaGetLastError());
    return NZB_OK;
}
