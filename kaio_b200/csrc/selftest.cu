// A one-CTA kernel that makes a bounded wait run out on purpose: it waits on an mbarrier that
// nothing arrives at, with a budget of a few microseconds, and then leaves the way every kernel
// of the library leaves after a wait gave up -- abort flag raised, {DEV_TIMEOUT, block, site,
// kernel} recorded in the status block, normal return.  No trap, no assert, no unbounded loop:
// the context stays usable and the host reads the outcome with kaio_b200_device_status().
#include "common.cuh"
#include "kernels.h"

namespace kaio {

constexpr uint32_t SITE_SELFTEST = 99;

__global__ void __launch_bounds__(32, 1)
selftest_bounded_wait_kernel(uint32_t* status, unsigned long long max_cycles)
{
    __shared__ uint64_t bar;
    __shared__ uint32_t abort_flag;
    if (threadIdx.x == 0) {
        mbar_init(smem_u32(&bar), 1);
        abort_flag = 0;
        fence_barrier_init();
    }
    __syncwarp();
    // phase 0 of a fresh barrier never completes without an arrival
    const bool ok = mbar_wait_lane_budget(smem_u32(&bar), 0, &abort_flag, status, SITE_SELFTEST,
                                          KERNEL_SELFTEST, max_cycles);
    (void)__all_sync(0xffffffffu, ok);
}

cudaError_t launch_selftest_bounded_wait(const DeviceCtx& ctx, uint32_t budget_us,
                                         cudaStream_t stream)
{
    selftest_bounded_wait_kernel<<<1, 32, 0, stream>>>(ctx.status,
                                                       (unsigned long long)budget_us * 2000ull);
    return cudaGetLastError();
}

}  // namespace kaio
