// Self-test of the bounded waits the attention kernels are built on: a wait that nothing will ever
// satisfy has to run out, report through the status word and leave by the ordinary end of the
// kernel, with the context usable afterwards.  One CTA, two warps; no tensor memory, no TMA.
#include "host_common.h"
#include "sm100_ptx.cuh"

namespace bsa {

__global__ void __launch_bounds__(64, 1) wait_selftest_kernel(int32_t* status, int32_t* report) {
  __shared__ uint64_t bar;
  __shared__ int abort_flag;
  const int warp = uniform_warp_index();
  const int lane = threadIdx.x & 31;
  if (threadIdx.x == 0) {
    mbar_init(smem_u32(&bar), 1);  // one arrival expected; none is ever made
    abort_flag = 0;
    mbar_fence_init();
  }
  __syncthreads();
  volatile int* flag = &abort_flag;
  const uint64_t t0 = global_timer_ns();
  if (warp == 0) {
    // runs out after the wait limit, then raises the CTA's flag like a role of a kernel does
    const bool ok = mbar_wait_warp(smem_u32(&bar), 0, flag);
    if (!ok && lane == 0) {
      abort_flag = 1;
      report_status(status, 99);
    }
    if (lane == 0) report[0] = ok ? 1 : 0;
  } else {
    // the sleeping form of the wait: leaves because the other warp raised the flag (or by its own
    // limit, whichever comes first)
    const bool ok = mbar_wait_warp_idle(smem_u32(&bar), 0, flag, 256);
    if (lane == 0) report[1] = ok ? 1 : 0;
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    report[2] = 1;  // both warps reached the end of the kernel
    report[3] = static_cast<int32_t>((global_timer_ns() - t0) / 1000000ull);  // milliseconds waited
  }
}

}  // namespace bsa

extern "C" int bsa_selftest_bounded_wait(int32_t* status, int32_t* report, void* stream) {
  if (!report) return BSA_ERR_BAD_POINTER;
  int rc;
  if ((rc = bsa::check_device_sm100()) != BSA_OK) return rc;
  bsa::wait_selftest_kernel<<<1, 64, 0, static_cast<cudaStream_t>(stream)>>>(status, report);
  return cudaGetLastError() == cudaSuccess ? BSA_OK : BSA_ERR_CUDA;
}
