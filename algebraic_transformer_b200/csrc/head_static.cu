// alg_head_fwd_static: the fused Alg-CE head for callers that must not allocate.
//
// alg_head_fwd needs scratch for its per-split partial sums and expects the caller to
// bring it.  Some callers have no way to do that: a custom-call handler running under a
// runtime that owns all device memory (it is handed operand and result buffers, nothing
// else, and a cudaMalloc of its own would bypass that runtime's allocator and stall the
// device), or a serving loop whose memory was laid out once at start-up.  For them this
// entry point keeps the scratch inside the library image, in the fixed-size device array
// below.  Each GPU that loads the library holds those ALG_HEAD_STATIC_SCRATCH_BYTES
// until the process exits, whether or not the entry point is ever called.
#include <mutex>

#include "common.cuh"
#include "launchers.h"

// Device-resident scratch.  In host code this name is only a handle for the runtime's
// symbol lookup, never a pointer a kernel may be given: the device address comes from
// cudaGetSymbolAddress below.
static __device__ __align__(256) float g_head_scratch[ALG_HEAD_STATIC_SCRATCH_BYTES / sizeof(float)];

namespace alg {
namespace {

constexpr size_t kScratchFloats = ALG_HEAD_STATIC_SCRATCH_BYTES / sizeof(float);

constexpr int kMaxDevices = 64;
std::mutex g_mu;
float* g_scratch_addr[kMaxDevices] = {};

// Device address of g_head_scratch on the current device, looked up once per device with
// that device current.
int scratch_address(float** out) {
  int dev = -1;
  ALG_CUDA_TRY(cudaGetDevice(&dev));
  if (dev < 0 || dev >= kMaxDevices) {
    set_error("alg_head_fwd_static: device ordinal %d is outside the supported range", dev);
    return ALG_ERR_UNSUPPORTED;
  }
  std::lock_guard<std::mutex> lock(g_mu);
  if (g_scratch_addr[dev] == nullptr) {
    float* ptr = nullptr;
    ALG_CUDA_TRY(cudaGetSymbolAddress(reinterpret_cast<void**>(&ptr), g_head_scratch));
    if (ptr == nullptr) {
      set_error("alg_head_fwd_static: the scratch symbol resolved to a null address");
      return ALG_ERR_CUDA;
    }
    g_scratch_addr[dev] = ptr;
  }
  *out = g_scratch_addr[dev];
  return ALG_OK;
}

}  // namespace
}  // namespace alg

using namespace alg;

extern "C" int alg_head_fwd_static(const alg_head_args* a, void* stream_) {
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  HeadParams p{};
  bool fast = false;
  if (int rc = head_fill(a, &p, &fast)) return rc;
  if (p.kind != ALG_HEAD_ALG_CE) { set_error("alg_head_fwd_static: only the alg_ce kind"); return ALG_ERR_UNSUPPORTED; }
  if (a->N == 0) return ALG_OK;
  const size_t need = size_t(2) * size_t(p.splits) * size_t(a->N);      // floats: l and zt partials
  if (need > kScratchFloats) {
    set_error("alg_head_fwd_static: this problem needs %zu bytes of scratch (N=%d, %d partial slots), more than the "
              "built-in %zu bytes; call alg_head_fwd with a caller-provided workspace instead",
              need * sizeof(float), a->N, p.splits, size_t(ALG_HEAD_STATIC_SCRATCH_BYTES));
    return ALG_ERR_WORKSPACE;
  }
  float* scratch = nullptr;
  if (int rc = scratch_address(&scratch)) return rc;
  // Every partial slot the reduction reads is written by the head kernel of this same call
  // (all token blocks x all splits), so nothing in the array has to start at zero and the
  // previous call's contents are simply overwritten.
  p.l_part = scratch;
  p.zt_part = scratch + size_t(p.splits) * a->N;
  if (int rc = fast ? launch_head_tcgen05(p, stream) : launch_head_mma(p, stream)) return rc;
  return launch_head_reduce(p, stream);
}
