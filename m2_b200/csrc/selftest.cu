// Self-test of the failure path every tensor-core kernel of this library shares: a bounded mbarrier wait
// that runs out, the device status word it sets, and a context that stays usable afterwards.  Nothing
// faults, traps or spins without bound: one thread waits, for at most the given time, on a barrier that
// nothing ever arrives at.
#include "tc_common.cuh"

namespace m2 {
__global__ void wait_timeout_kernel(unsigned long long limit_ns) {
  __shared__ uint64_t bar;
  __shared__ int abort_flag;
  if (threadIdx.x == 0) {
    tc::mbar_init(&bar, 1);
    abort_flag = 0;
    tc::mbar_fence_init();
  }
  __syncthreads();
  if (threadIdx.x == 0) tc::mbar_wait_ns(&bar, 0, &abort_flag, tc::ST_TIMEOUT_TMA, limit_ns);
  __syncthreads();
}
}  // namespace m2

extern "C" int m2_selftest_wait_timeout(unsigned long long limit_ns, void* stream) {
  M2_REQUIRE(limit_ns > 0 && limit_ns <= 1000000000ull, M2_ERR_ARG,
             "m2_selftest_wait_timeout: limit must be between 1 ns and 1 s");
  m2::wait_timeout_kernel<<<1, 32, 0, static_cast<cudaStream_t>(stream)>>>(limit_ns);
  M2_LAUNCH_CHECK("wait_timeout_kernel");
  return M2_OK;
}
