// Self-test of the bounded-wait error path.
//
// Every device-side wait of this library (mbarrier waits in the GEMM and attention kernels)
// gives up after a number of SM clocks, records the wait site in an error word and makes its
// kernel return.  rt_selftest_bounded_wait exercises exactly that path without involving any
// real work: one CTA waits on a barrier that nothing ever arrives on, with a caller-chosen,
// short limit.  The kernel returns normally (no trap, no fault); the host then sees
// RT_ERR_DEVICE_WAIT with site 901 from rt_check_device(), and the device stays usable.
#include <cuda_runtime.h>

#include "common.h"
#include "device_error.h"
#include "launch_count.h"
#include "sm100_ptx.cuh"

namespace rt {
int* static_scratch_status_word();  // no_alloc.cu: status word of rt_sparse_attention_static (this device)

namespace {
using namespace ptx;

constexpr int kSelfTestSite = 901;

__global__ void bounded_wait_selftest_kernel(int* error_flag, long long limit_cycles, int* gave_up_out) {
  __shared__ uint64_t bar;
  __shared__ int abort_flag;
  if (threadIdx.x == 0) {
    mbar_init(&bar, 1);
    abort_flag = 0;
    fence_barrier_init();
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    AbortCtx ab{&abort_flag, error_flag, limit_cycles};
    const bool completed = mbar_wait(&bar, 0, ab, kSelfTestSite);  // nothing arrives: runs out after limit_cycles
    if (gave_up_out) *gave_up_out = completed ? 0 : 1;
  }
  __syncthreads();
}

}  // namespace
}  // namespace rt

using namespace rt;

extern "C" rt_status rt_selftest_bounded_wait(int64_t limit_cycles, int target, void* stream) {
  RT_REQUIRE(limit_cycles > 0 && limit_cycles <= 200000000ll, RT_ERR_INVALID,
             "selftest_bounded_wait: limit must be in (0, 2e8] SM clocks (about 0.1 s)");
  RT_REQUIRE(target == 0 || target == 1, RT_ERR_INVALID, "selftest_bounded_wait: target must be 0 or 1");
  int* word = target == 0 ? device_error_word() : static_scratch_status_word();
  RT_REQUIRE(word != nullptr, RT_ERR_CUDA, "selftest_bounded_wait: no error word on this device");
  bounded_wait_selftest_kernel<<<1, 32, 0, static_cast<cudaStream_t>(stream)>>>(word, limit_cycles, nullptr);
  count_launch();
  RT_CHECK_CUDA(cudaGetLastError());
  return RT_OK;
}
