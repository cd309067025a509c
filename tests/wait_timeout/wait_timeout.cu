// Test helper, not part of the library: a one-block kernel that waits, with the library's own bounded-wait helper
// and a small poll limit, on an mbarrier that nobody ever arrives at.  The wait gives up, the kernel records a code in
// the caller's status word and returns normally: the same hand-over the attention kernels use when one of their
// waits runs out (there the limit is ptx::WAIT_POLLS), exercised without making any real kernel misbehave.
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../flashmla_b200/csrc/sm100_ptx.cuh"

namespace {

constexpr uint32_t TEST_POLLS = 4096;     // the kernels' limit is ptx::WAIT_POLLS (4 Mi polls)
constexpr int TEST_CODE = 77;

__global__ void __launch_bounds__(64, 1) wait_timeout_kernel(int* status, int arrive_first) {
  __shared__ __align__(8) unsigned long long bar;
  __shared__ int abort_flag;
  using namespace fmla::ptx;
  const uint32_t bar_addr = smem_u32(&bar);
  if (threadIdx.x == 0) {
    abort_flag = 0;
    mbar_init(bar_addr, 1);
    mbar_init_fence();
  }
  __syncthreads();
  // arrive_first != 0: the barrier completes and the wait succeeds (the control case)
  if (arrive_first && threadIdx.x == 32) mbar_arrive(bar_addr);
  if (threadIdx.x < 32) {
    const bool ok = mbar_wait_abortable<TEST_POLLS>(bar_addr, 0, &abort_flag);
    if (!ok && threadIdx.x == 0) {
      abort_flag = TEST_CODE;                    // what raise_abort does: tell the other roles, then the host
      atomicCAS(status, 0, TEST_CODE);
    }
  }
  __syncthreads();
  // the second warp plays "another role": it sees the flag instead of waiting out its own limit
  if (threadIdx.x == 32 && !arrive_first && abort_flag != TEST_CODE) atomicCAS(status, TEST_CODE, -1);
}

}  // namespace

extern "C" int wait_timeout_probe(int* status_device_word, int arrive_first, void* cuda_stream) {
  wait_timeout_kernel<<<1, 64, 0, static_cast<cudaStream_t>(cuda_stream)>>>(status_device_word, arrive_first);
  return (int)cudaGetLastError();
}
extern "C" int wait_timeout_code(void) { return TEST_CODE; }
