// Self-test of the bounded wait every role of the attention kernel uses (wait_bar, common.cuh): one CTA waits, with
// a SHORT poll limit, on an mbarrier phase that nothing will ever complete.  The wait must run out, record its code
// in the status word and let the kernel return normally - no trap, no fault, no hang - which is how a protocol
// error inside the attention kernel surfaces as SAGE3_ERR_DEVICE_WAIT on the host.  No counterpart in the
// reference (its kernel waits without bounds).
#include "common.cuh"
#include "kernels.h"

namespace sage3 {

namespace {

__global__ void __launch_bounds__(32) bounded_wait_selftest_kernel(int* status, int code) {
  __shared__ __align__(8) unsigned long long bar_mem;
  __shared__ int abort_flag;
  const uint32_t bar = smem_u32(&bar_mem);
  if (threadIdx.x == 0) {
    abort_flag = 0;
    mbar_init(bar, 1);                  // one arrival expected, none will come
    fence_mbar_init();
  }
  __syncwarp();
  if (threadIdx.x == 0) {
    // 2048 polls of about 1.5 us: gives up after a few milliseconds
    const bool done = wait_bar<false, 2048>(bar, 0, &abort_flag, status, code);
    if (done) atomicCAS(status, 0, -1);  // cannot happen; would mean the wait saw a phase nobody completed
  }
}

}  // namespace

cudaError_t launch_bounded_wait_selftest(int* status, int code, cudaStream_t stream) {
  bounded_wait_selftest_kernel<<<1, 32, 0, stream>>>(status, code);
  return cudaGetLastError();
}

}  // namespace sage3
