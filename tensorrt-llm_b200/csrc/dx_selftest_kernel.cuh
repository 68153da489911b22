// Self-test of the device-side failure reporting: a wait that nothing ever satisfies.
//
// Every wait in this library is bounded; when one runs out the kernel records STATUS_TIMEOUT in the handle's
// status word and returns, and the host reads that as DX_ERR_TIMEOUT.  This kernel makes exactly that happen, on
// purpose and harmlessly: one warp waits, with a caller-chosen poll limit, on an mbarrier of its own that no
// thread arrives on and no copy is bound to, then reports the time-out through the same helper the attention
// kernels use.  Nothing is in flight into its shared memory at any point.
#pragma once

#include "dx_common.cuh"

namespace dx
{

__global__ void __launch_bounds__(32) wait_timeout_selftest_kernel(int32_t* status, const int poll_limit)
{
    __shared__ __align__(8) uint64_t bar;
    if (threadIdx.x == 0)
    {
        mbar_init(&bar, 1);
        fence_mbar_init();
    }
    __syncwarp();
    // CHECK_STATUS off: the limit alone ends the wait, whatever the status word holds already
    const bool ok = mbar_wait_limit<false>(&bar, 0, status, poll_limit);
    if (!ok && threadIdx.x == 0)
        report_status(status, STATUS_TIMEOUT);
}

} // namespace dx
