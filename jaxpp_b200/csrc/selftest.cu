// Self-test kernels for the bounded waits: each one waits for something that never happens, so that a test can
// check that the wait runs out, the kernel returns, and the status word says why.  The waits are the library's
// own (common.cuh), with whatever budget jpb_set_wait_budget_ns() has set; nothing here traps or faults.
#include "common.cuh"

namespace jpb {

// One warp waits on an mbarrier that nobody arrives on.  out[0] = 1 if the wait reported a time-out (returned
// false), out[1] = nanoseconds spent in the wait.
__global__ void selftest_mbar_timeout_kernel(int* status, long long* out) {
  __shared__ uint64_t bar;
  __shared__ int abort_flag;
  if (threadIdx.x == 0) {
    mbar_init(&bar, 1);
    abort_flag = 0;
    fence_barrier_init();
  }
  __syncthreads();
  const uint64_t t0 = globaltimer_ns();
  const bool ok = mbar_wait_bounded_warp(&bar, 0, &abort_flag, status, JPB_ERR_WAIT_TIMEOUT);
  const uint64_t t1 = globaltimer_ns();
  if (threadIdx.x == 0) {
    out[0] = ok ? 0 : 1;
    out[1] = (long long)(t1 - t0);
  }
}

}  // namespace jpb

// Launches the kernel above on `stream`; `out` points to two int64 in device memory.
JPB_API int jpb_selftest_mbar_timeout(long long* out, void* stream) {
  jpb::selftest_mbar_timeout_kernel<<<1, 32, 0, static_cast<cudaStream_t>(stream)>>>(jpb_status_device_ptr(), out);
  return int(cudaGetLastError());
}
