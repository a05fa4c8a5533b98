// Self-test of the bounded-wait machinery: one thread waits on a flag in global memory with a
// caller-given time limit.  When the flag never reaches the value the wait gives up, the
// kernel returns normally and the device status word holds {KST_FLAG_TIMEOUT, 900, block,
// wanted value}; the context stays usable.  This is how the framework's failure detection is
// exercised on a GPU without faulting, trapping or hanging it.
#include "host_common.h"
#include "sm100.cuh"
#include "cogito_kernels.h"

namespace {
using namespace cgk;
__global__ void bounded_wait_kernel(const int* flag, int want, int* status, unsigned long long budget_ns, int* reached) {
  if (threadIdx.x == 0) {
    const bool ok = flag_wait_ge_sys(flag, want, status, 900, budget_ns);
    if (reached) *reached = ok ? 1 : 0;
  }
}
}  // namespace

CGK_API int cgk_selftest_bounded_wait(const int* flag, int want, unsigned long long budget_ns, int* reached, void* stream) {
  CGK_REQUIRE(flag != nullptr, "cgk_selftest_bounded_wait: null flag");
  CGK_REQUIRE(budget_ns <= 5000000000ull, "cgk_selftest_bounded_wait: the limit must not exceed 5 s");
  int dev = 0;
  CGK_CUDA_CHECK(cudaGetDevice(&dev));
  bounded_wait_kernel<<<1, 32, 0, (cudaStream_t)stream>>>(flag, want, cgk::device_status(dev), budget_ns, reached);
  CGK_LAUNCH_CHECK();
  return 0;
}
