// Exercise of the bounded device-side wait, for tests of the failure path.
//
// Every kernel of this library waits on mbarriers through mbar_wait(): after a time limit the wait
// gives up, raises the CTA's error flag, records (code << 8) | where in the device status word and
// the kernel unwinds through its normal teardown.  In a healthy run that branch never executes, so
// this file provides the one situation in which it does, on purpose and harmlessly: a single small
// CTA initialises a barrier that nothing ever arrives on and waits for it with a SHORT limit given
// by the caller.  The wait runs out, the kernel records the status and returns by itself: nothing
// traps, faults or spins without a bound, and the context stays usable.
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/sparseflow_b200.h"
#include "device_state.h"
#include "kernels.h"
#include "sm100_ptx.cuh"

namespace sfb200 {
namespace {

__global__ void __launch_bounds__(64, 1) wait_probe_kernel(int* status, int where, unsigned long long limit_ns) {
  __shared__ __align__(8) uint64_t bar;
  __shared__ int err_flag;
  volatile int* err = &err_flag;
  const uint32_t bar_addr = smem_u32(&bar);
  if (threadIdx.x == 0) {
    *err = 0;
    mbar_init(bar_addr, 1);      // one arrival expected; none will come
    mbar_fence_init();
  }
  __syncthreads();
  bool ok = true;
  if (threadIdx.x == 0) ok = mbar_wait_limit(bar_addr, 0, err, status, where, limit_ns);
  // a second role notices the failure through the CTA-shared flag, as the GEMM kernels' warps do:
  // its own wait is given a long limit and must end early because `err` is set
  if (threadIdx.x == 32) ok = mbar_wait_limit(bar_addr, 0, err, status, 63, kWaitLimitNs);
  (void)ok;
  __syncthreads();               // normal teardown: every thread reaches the end
}

}  // namespace
}  // namespace sfb200

using namespace sfb200;

extern "C" int sfb200_debug_wait_timeout(unsigned limit_us, int where, int noalloc_word, void* stream) {
  int err = kOk;
  DeviceState* s = device_state(&err);
  if (!s) return err;
  if (limit_us == 0 || limit_us > 100000u || where < 0 || where > 255) return kErrInvalid;   // at most 0.1 s
  int* word = noalloc_word ? noalloc_status_word() : s->status;
  if (!word) return kErrCuda;
  wait_probe_kernel<<<1, 64, 0, static_cast<cudaStream_t>(stream)>>>(word, where,
                                                                      static_cast<unsigned long long>(limit_us) * 1000ull);
  return cudaGetLastError() == cudaSuccess ? kOk : kErrCuda;
}
