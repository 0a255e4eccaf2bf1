// selftest.cu - makes the give-up path of the bounded waits run, without a stuck kernel.
//
// Every wait of the tensor-core kernels is an mbar_wait with a time limit: when the limit
// passes, the waiting thread records a role code in the kernel status word and the kernel
// returns; the host sees the code at its next synchronisation.  In a healthy run that path
// never executes, so this file gives the host a way to execute it on purpose: a one-block
// kernel that initialises a barrier for two arrivals, arrives once and waits with a limit
// of the caller's choosing.  Nothing else is in flight - no TMA copy, no MMA, no tensor
// memory - so giving up has nothing to clean up and the kernel ends normally.
#include "tc_common.cuh"

namespace boatcu {
namespace {

__global__ void wait_timeout_kernel(unsigned int* status, unsigned long long limit_ns) {
    __shared__ uint64_t bar;
    if (threadIdx.x == 0) {
        tc::mbar_init(&bar, 2);
        tc::fence_barrier_init();
        tc::mbar_arrive(&bar);               // one of the two arrivals: the phase cannot complete
        tc::mbar_wait_limit(&bar, 0, status, tc::kTimeoutSelfTest, limit_ns);
    }
}

}  // namespace
}  // namespace boatcu

using namespace boatcu;

extern "C" int boat_cuda_selftest_wait_timeout(uint64_t limit_ns) {
    if (int rc = ensure_init()) return rc;
    if (limit_ns == 0 || limit_ns > 1000000000ull)
        return set_error(11, "boat_cuda_selftest_wait_timeout: limit must be between 1 ns and 1 s");
    wait_timeout_kernel<<<1, 32, 0, stream()>>>(kernel_status_ptr(), (unsigned long long)limit_ns);
    BOATCU_LAUNCH_OK("wait_timeout_selftest");
    return 0;
}
