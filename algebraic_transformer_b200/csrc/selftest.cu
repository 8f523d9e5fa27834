// Self-test of the bounded-wait mechanism all tcgen05/TMA kernels of this library use for
// their mbarrier waits (sm100_ptx.cuh: BoundedWait).  The kernel waits on a barrier that
// nothing ever arrives on; the wait must give up after the budget, raise the CTA-wide abort
// flag so that every other thread leaves its wait too, report ALG_DEV_TIMEOUT through the
// status word, and return normally — leaving the context usable.
#include "common.cuh"
#include "sm100_ptx.cuh"

namespace alg {
namespace {

__global__ void bounded_wait_selftest_kernel(int* status, unsigned long long budget_ns, unsigned long long* waited_ns) {
  __shared__ uint64_t never;
  __shared__ int abort_flag;
  if (threadIdx.x == 0) {
    sm100::mbar_init(&never, 1);
    abort_flag = 0;
    sm100::fence_barrier_init();
  }
  __syncthreads();
  const sm100::BoundedWait bw{&abort_flag, budget_ns};
  const uint64_t t0 = sm100::global_timer_ns();
  const bool completed = bw.wait(&never, 0);        // every thread waits; the first timeout releases all
  const uint64_t t1 = sm100::global_timer_ns();
  __syncthreads();
  if (threadIdx.x == 0) {
    *status = (completed || abort_flag == 0) ? ALG_DEV_BAD_STATE : ALG_DEV_TIMEOUT;
    if (waited_ns != nullptr) *waited_ns = t1 - t0;
  }
}

}  // namespace
}  // namespace alg

extern "C" int alg_selftest_bounded_wait(int* status, unsigned long long budget_ns, unsigned long long* waited_ns,
                                         void* stream) {
  using namespace alg;
  if (status == nullptr) { set_error("selftest: status word required"); return ALG_ERR_INVALID; }
  if (budget_ns == 0 || budget_ns > 1000000000ull) { set_error("selftest: budget must be in (0, 1 s]"); return ALG_ERR_INVALID; }
  bounded_wait_selftest_kernel<<<1, 128, 0, static_cast<cudaStream_t>(stream)>>>(status, budget_ns, waited_ns);
  ALG_CUDA_TRY(cudaGetLastError());
  count_launch();
  return ALG_OK;
}
