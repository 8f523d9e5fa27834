// Shared device helpers: the algebraic scalar functions (rho, integer powers, inverse
// roots — only + - * / rsqrt and comparisons, as in src/algebraic/algebraic.py of the
// reference), warp reductions, and host-side error plumbing.
#pragma once

#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <cstdlib>
#include <stdint.h>

#include <atomic>

#include "../../include/alg_b200.h"

namespace alg {

// ---- host-side error plumbing -------------------------------------------------------
void set_error(const char* fmt, ...);
int cuda_fail(cudaError_t e, const char* what);
void count_launch(int n = 1);   // bumps the process-wide kernel-launch counter (alg_kernel_launches)

#define ALG_CUDA_TRY(expr)                                     \
  do {                                                         \
    cudaError_t _e = (expr);                                   \
    if (_e != cudaSuccess) return ::alg::cuda_fail(_e, #expr); \
  } while (0)

// Number of SMs of the current device (cached per device ordinal).  Grids and split counts are
// sized from it; 148 (B200) stands in when no device can be queried, which only happens when a
// workspace-size function is called on a machine without a GPU.
int sm_count();

// One-time per-DEVICE set-up of a kernel: function attributes such as the dynamic shared-memory
// opt-in belong to the device that was current when they were set, so a process that drives
// several GPUs has to repeat them on each.  `run` performs `setup` once for the current device
// and reports that device's SM count.
struct PerDeviceOnce {
  static constexpr int kMaxDevices = 64;
  std::atomic<int> done[kMaxDevices];
  template <class F>
  int run(F&& setup, int* sms = nullptr) {
    int dev = 0;
    ALG_CUDA_TRY(cudaGetDevice(&dev));
    if (dev < 0 || dev >= kMaxDevices) {
      set_error("device ordinal %d is outside the supported range [0, %d)", dev, kMaxDevices);
      return ALG_ERR_UNSUPPORTED;
    }
    if (done[dev].load(std::memory_order_acquire) == 0) {   // idempotent: a race repeats it harmlessly
      ALG_CUDA_TRY(setup());
      done[dev].store(1, std::memory_order_release);
    }
    if (sms != nullptr) *sms = sm_count();
    return ALG_OK;
  }
};

struct Strides3 {
  int64_t b, h, t;
};

inline Strides3 strides_or_dense(const int64_t s[3], int H, int T, int D) {
  if (s[0] == 0 && s[1] == 0 && s[2] == 0) return {int64_t(H) * T * D, int64_t(T) * D, int64_t(D)};
  return {s[0], s[1], s[2]};
}

// ---- scalar math --------------------------------------------------------------------
__device__ __forceinline__ float rsqrt_approx(float x) {
  float y;
  asm("rsqrt.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

// 2^x on the special-function unit (the softmax cross-entropy head only; the algebraic paths use
// no exponential)
__device__ __forceinline__ float exp2_approx(float x) {
  float y;
  asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
  return y;
}

// rho(x) = x + sqrt(1 + x^2), summation form (relative cancellation O(eps x^2) for x << 0).
// src/algebraic/kernels/flash.py:84-88.
__device__ __forceinline__ float rho_fast(float x) {
  float rad = fmaf(x, x, 1.0f);
  return fmaf(rad, rsqrt_approx(rad), x);
}

// Cancellation-free form: t = |x| + sqrt(1+x^2) >= 1, rho = x >= 0 ? t : 1/t.
// src/algebraic/algebraic.py:31-35.
__device__ __forceinline__ float rho_stable(float x) {
  float rad = fmaf(x, x, 1.0f);
  float t = fmaf(rad, rsqrt_approx(rad), fabsf(x));
  return x >= 0.0f ? t : __fdividef(1.0f, t);
}

// x^(2^LOG2N) by repeated squaring (n is a power of two on every kernel path).
template <int LOG2N>
__device__ __forceinline__ float pow2n(float x) {
#pragma unroll
  for (int i = 0; i < LOG2N; ++i) x *= x;
  return x;
}
__device__ __forceinline__ float pow2n_rt(float x, int log2n) {
  for (int i = 0; i < log2n; ++i) x *= x;
  return x;
}

// l^(-1/n), n = 2^log2n: rsqrt then square roots y <- y * rsqrt(y).
// src/algebraic/kernels/flash.py:95-104.
__device__ __forceinline__ float inv_root_rt(float l, int log2n) {
  float y = rsqrtf(l);
  for (int i = 1; i < log2n; ++i) y = y * rsqrtf(y);
  return y;
}

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}

__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
  __nv_bfloat162 p = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<uint32_t*>(&p);
}

inline int ilog2_exact(int n) {
  int k = 0;
  while ((1 << k) < n) ++k;
  return ((1 << k) == n) ? k : -1;
}

// Guard scratch: three non-negative floats kept as uint bit patterns so that atomicMax
// orders them: max |q_scaled|^2, max |k|^2, max |v|.
struct GuardWords {
  unsigned q2, k2, vmax, pad;
};

// The reference's range guard (src/algebraic/kernels/flash.py:834-849) evaluated from the
// three maxima: in range => unshifted accumulation is safe in fp32.
__device__ __forceinline__ bool guard_in_range(const GuardWords* g, float bound_sq, float vmax_limit) {
  float q2 = __uint_as_float(g->q2), k2 = __uint_as_float(g->k2), vm = __uint_as_float(g->vmax);
  return (q2 * k2 <= bound_sq) && (vm <= vmax_limit);
}

// Programmatic dependent launch.  A kernel launched with the programmatic-serialization attribute is
// placed on an SM as soon as the CTAs of the kernel before it in the stream have left it, instead of
// after that whole kernel has drained; griddep_wait() in it returns once that kernel has finished
// and its writes are visible (a no-op in a kernel launched the plain way).  So a kernel's set-up
// (barriers, tensor memory, descriptor prefetch) and its launch latency overlap the tail of the one
// before.  The earlier kernels do not announce themselves early (griddepcontrol.launch_dependents):
// measured on the prefill step, CTAs that sit waiting beside a running kernel cost a long step 1-2 %,
// while leaving it to each CTA's exit keeps the whole gain of the short steps (3 % at 2048 tokens).
__device__ __forceinline__ void griddep_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }

// Launch `kern` so that it may start before the kernel ahead of it in `stream` has finished
// (programmatic dependent launch); the kernel itself calls griddep_wait() before it touches
// anything the earlier kernel writes.
template <typename... Formal, typename... Actual>
inline cudaError_t launch_dependent(void (*kern)(Formal...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream,
                                    Actual&&... args) {
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = grid; cfg.blockDim = block; cfg.dynamicSmemBytes = smem; cfg.stream = stream;
  cudaLaunchAttribute attr[1];
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  static const bool plain = getenv("ALG_NO_PDL") != nullptr;      // measurement aid: ordinary stream order
  cfg.attrs = attr; cfg.numAttrs = plain ? 0 : 1;
  return cudaLaunchKernelEx(&cfg, kern, static_cast<Formal>(args)...);
}

}  // namespace alg
