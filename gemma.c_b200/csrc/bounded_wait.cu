// Self-test of the bounded wait. Every spin in this library goes through
// mbar_wait_bounded() (common.cuh) or the peer kernel's flag poll, gives up
// after a clock limit and reports B200KV_STATUS_WAIT_TIMEOUT through the
// caller's status word instead of hanging the GPU. In normal operation no wait
// runs out, so that path would never be exercised; this kernel makes one run
// out on purpose and harmlessly: one warp arms an mbarrier that nothing will
// ever arrive at, waits for `clock_limit` SM clocks with the same helper, and
// records the outcome with the same set_status(). Nothing faults or traps; the
// kernel returns normally and the context stays usable.
#include "common.cuh"
#include "kernels.cuh"

namespace b200kv {
namespace {

__global__ void bounded_wait_selftest_kernel(long long clock_limit,
                                             int32_t *status,
                                             long long *waited_clocks) {
  __shared__ __align__(8) unsigned long long bar;
  const uint32_t addr = smem_u32(&bar);
  if (threadIdx.x == 0) {
    mbar_init(addr, 1);
    mbar_fence_init();
  }
  __syncwarp();
  const long long start = clock64();
  const bool arrived = mbar_wait_bounded(addr, 0u, clock_limit);
  const long long waited = clock64() - start;
  if (threadIdx.x == 0) {
    if (!arrived) set_status(status, B200KV_STATUS_WAIT_TIMEOUT);
    if (waited_clocks != nullptr) *waited_clocks = waited;
  }
}

}  // namespace

cudaError_t bounded_wait_selftest(long long clock_limit, int32_t *status,
                                  long long *waited_clocks,
                                  cudaStream_t stream) {
  // at most about a tenth of a second: this is a test of the give-up path
  if (clock_limit <= 0 || clock_limit > (1ll << 28)) return cudaErrorInvalidValue;
  bounded_wait_selftest_kernel<<<1, 32, 0, stream>>>(clock_limit, status,
                                                     waited_clocks);
  return cudaGetLastError();
}

}  // namespace b200kv
