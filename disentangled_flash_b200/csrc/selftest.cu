// Diagnostic for the bounded-wait path of the tcgen05 kernels: a wait that nobody satisfies must run out, leave
// the CTA through its normal teardown (tensor memory freed) and report its code through the status word.
#include "dfl_common.cuh"
#include "tcgen05_ptx.cuh"

namespace dfl {
namespace {

constexpr int kSelftestCode = 99;

__global__ void __launch_bounds__(128, 1) selftest_bounded_wait_kernel(int* status_word, uint32_t limit_ns) {
  __shared__ uint64_t never_completes;   // one arrival expected, none ever made
  __shared__ uint32_t tmem_holder;
  __shared__ int abort_word;
  volatile int* abort_flag = &abort_word;
  const int warp = threadIdx.x >> 5;
  if (threadIdx.x == 0) {
    ptx::mbar_init(&never_completes, 1);
    abort_word = 0;
    ptx::fence_mbar_init();
  }
  if (warp == 0) {
    ptx::tmem_alloc(&tmem_holder, 32);
    ptx::tmem_relinquish();
  }
  ptx::tc_fence_before();
  __syncthreads();
  ptx::tc_fence_after();
  int fail_code = 0;
  // every thread waits, like the roles of the real kernels: the first to run out raises the abort flag, the
  // others leave at their next look at it
  ptx::mbar_wait_inline(&never_completes, 0, abort_flag, fail_code, kSelftestCode, limit_ns);
  if (fail_code != 0) atomicCAS(status_word, 0, fail_code);
  ptx::tc_fence_before();
  __syncthreads();
  if (warp == 0) ptx::tmem_dealloc(tmem_holder, 32);
}

}  // namespace

int launch_selftest_bounded_wait(int* status, uint32_t limit_us, cudaStream_t stream) {
  selftest_bounded_wait_kernel<<<1, 128, 0, stream>>>(status, limit_us * 1000u);
  return check_launch("selftest_bounded_wait_kernel");
}

}  // namespace dfl
