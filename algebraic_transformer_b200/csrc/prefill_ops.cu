// The two elementwise stages of the prefill body that sit between the GEMMs:
//   rms_norm over d_model rows   y = x rsqrt(mean(x^2) + eps) gain     src/algebraic/algebraic.py:76-83
//                                (model._norm, src/algebraic/model.py:141-143)
//   ALU-GLU                      out = gate * alu_beta(up)             src/algebraic/algebraic.py:86-105
//                                (model._block, src/algebraic/model.py:184-193)
// Both are HBM-bound, bf16 in / bf16 out with fp32 math and the reference's rounding points
// (alu rounds to bf16 before the product with the gate, which rounds again).
#include "common.cuh"
#include "launchers.h"

namespace alg {
namespace {

__device__ __forceinline__ void unpack8(const uint4& r, float* v) {
  const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&r);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    float2 f = __bfloat1622float2(h[i]);
    v[2 * i] = f.x; v[2 * i + 1] = f.y;
  }
}
__device__ __forceinline__ uint4 pack8(const float* v) {
  uint4 r;
  r.x = pack_bf16(v[0], v[1]); r.y = pack_bf16(v[2], v[3]);
  r.z = pack_bf16(v[4], v[5]); r.w = pack_bf16(v[6], v[7]);
  return r;
}
__device__ __forceinline__ float bf16_round(float x) { return __bfloat162float(__float2bfloat16_rn(x)); }

// A warp owns RPW rows at a time and issues all their 16-byte loads (VPL per lane and row)
// before using any, so that enough bytes are in flight to cover the HBM latency.
template <int VPL, int RPW>
__global__ void __launch_bounds__(256) rms_rows_kernel(const __nv_bfloat16* __restrict__ x, const float* __restrict__ gain,
                                                       __nv_bfloat16* __restrict__ y, int64_t rows, int d, float eps) {
  griddep_wait();                 // launched as a programmatic dependent of the kernel ahead in the stream
  const int lane = threadIdx.x & 31;
  const int64_t warp_global = (int64_t(blockIdx.x) * blockDim.x + threadIdx.x) >> 5;
  const int64_t warps_total = (int64_t(gridDim.x) * blockDim.x) >> 5;
  const int nvec = d / 8;
  for (int64_t row0 = warp_global * RPW; row0 < rows; row0 += warps_total * RPW) {
    uint4 raw[RPW][VPL];
#pragma unroll
    for (int r = 0; r < RPW; ++r) {
      const int64_t row = row0 + r < rows ? row0 + r : rows - 1;
      const uint4* src = reinterpret_cast<const uint4*>(x + row * d);
#pragma unroll
      for (int u = 0; u < VPL; ++u) {
        const int vi = u * 32 + lane;
        raw[r][u] = vi < nvec ? src[vi] : make_uint4(0, 0, 0, 0);
      }
    }
#pragma unroll
    for (int r = 0; r < RPW; ++r) {
      float ss = 0.f;
#pragma unroll
      for (int u = 0; u < VPL; ++u) {
        float v[8];
        unpack8(raw[r][u], v);
#pragma unroll
        for (int i = 0; i < 8; ++i) ss = fmaf(v[i], v[i], ss);
      }
      ss = warp_sum(ss);
      const float tau = rsqrtf(ss / float(d) + eps);
      if (row0 + r < rows) {
        uint4* dst = reinterpret_cast<uint4*>(y + (row0 + r) * d);
#pragma unroll
        for (int u = 0; u < VPL; ++u) {
          const int vi = u * 32 + lane;
          if (vi < nvec) {
            float v[8];
            unpack8(raw[r][u], v);
            if (gain != nullptr) {
              const float4 g0 = *reinterpret_cast<const float4*>(gain + vi * 8);
              const float4 g1 = *reinterpret_cast<const float4*>(gain + vi * 8 + 4);
              const float g[8] = {g0.x, g0.y, g0.z, g0.w, g1.x, g1.y, g1.z, g1.w};
#pragma unroll
              for (int i = 0; i < 8; ++i) v[i] = (v[i] * tau) * g[i];
            } else {
#pragma unroll
              for (int i = 0; i < 8; ++i) v[i] = v[i] * tau;
            }
            dst[vi] = pack8(v);
          }
        }
      }
    }
  }
}

// gate, up: (rows, f) with row stride ld_in (both halves of one GEMM output qualify); out: row stride ld_out
__global__ void __launch_bounds__(256) alu_glu_kernel(const __nv_bfloat16* __restrict__ gate, const __nv_bfloat16* __restrict__ up,
                                                      __nv_bfloat16* __restrict__ out, int64_t rows, int f, int64_t ld_in,
                                                      int64_t ld_out, float beta) {
  griddep_wait();                 // launched as a programmatic dependent of the kernel ahead in the stream
  const size_t stride = size_t(gridDim.x) * blockDim.x;
  const int vpr = f / 8;
  const size_t nvec = size_t(rows) * vpr;
  for (size_t i = size_t(blockIdx.x) * blockDim.x + threadIdx.x; i < nvec; i += stride) {
    const int64_t row = int64_t(i / vpr);
    const int col = int(i % vpr) * 8;
    float g[8], u[8], o[8];
    unpack8(*reinterpret_cast<const uint4*>(gate + row * ld_in + col), g);
    unpack8(*reinterpret_cast<const uint4*>(up + row * ld_in + col), u);
#pragma unroll
    for (int k = 0; k < 8; ++k) {
      const float bz = beta * u[k];
      const float r = rsqrtf(fmaf(bz, bz, 1.0f));
      const float uu = bz * r;
      // for bz < 0 use 1 + u = r^2 / (1 - u) so that the negative tail survives
      const float one_plus_u = bz < 0.f ? __fdividef(r * r, 1.0f - uu) : 1.0f + uu;
      const float act = bf16_round(0.5f * u[k] * one_plus_u);
      o[k] = g[k] * act;
    }
    *reinterpret_cast<uint4*>(out + row * ld_out + col) = pack8(o);
  }
}

}  // namespace

int launch_rms_rows(const void* x, const float* gain, void* y, int64_t rows, int d, float eps, cudaStream_t stream) {
  if (rows == 0) return ALG_OK;
  const int vpl = (d / 8 + 31) / 32;
  constexpr int RPW = 4;                               // rows per warp step (<= 4 x 4 vectors per lane in flight)
  int64_t blocks = (rows + 8 * RPW - 1) / (8 * RPW);
  if (blocks > sm_count() * 6) blocks = sm_count() * 6;
  const __nv_bfloat16* xp = static_cast<const __nv_bfloat16*>(x);
  __nv_bfloat16* yp = static_cast<__nv_bfloat16*>(y);
  if ((reinterpret_cast<uintptr_t>(gain) & 15) != 0) {
    set_error("rms_norm: gain must be 16-byte aligned");
    return ALG_ERR_INVALID;
  }
  cudaError_t err = cudaSuccess;
  switch (vpl) {
    case 1: err = launch_dependent(rms_rows_kernel<1, RPW>, dim3(unsigned(blocks)), dim3(256), 0, stream, xp, gain, yp, rows, d, eps); break;
    case 2: err = launch_dependent(rms_rows_kernel<2, RPW>, dim3(unsigned(blocks)), dim3(256), 0, stream, xp, gain, yp, rows, d, eps); break;
    case 3: err = launch_dependent(rms_rows_kernel<3, RPW>, dim3(unsigned(blocks)), dim3(256), 0, stream, xp, gain, yp, rows, d, eps); break;
    case 4: err = launch_dependent(rms_rows_kernel<4, RPW>, dim3(unsigned(blocks)), dim3(256), 0, stream, xp, gain, yp, rows, d, eps); break;
    case 5: case 6: err = launch_dependent(rms_rows_kernel<6, 2>, dim3(unsigned(blocks)), dim3(256), 0, stream, xp, gain, yp, rows, d, eps); break;
    case 7: case 8: err = launch_dependent(rms_rows_kernel<8, 2>, dim3(unsigned(blocks)), dim3(256), 0, stream, xp, gain, yp, rows, d, eps); break;
    default:
      set_error("rms_norm: row width %d is above the supported 2048", d);
      return ALG_ERR_UNSUPPORTED;
  }
  ALG_CUDA_TRY(err);
  count_launch();
  return ALG_OK;
}

int launch_alu_glu(const void* gate, const void* up, void* out, int64_t rows, int f, int64_t ld_in, int64_t ld_out,
                   float beta, cudaStream_t stream) {
  if (rows == 0 || f == 0) return ALG_OK;
  const size_t nvec = size_t(rows) * (f / 8);
  size_t blocks = (nvec + 255) / 256;
  if (blocks > size_t(sm_count()) * 16) blocks = size_t(sm_count()) * 16;
  ALG_CUDA_TRY(launch_dependent(alu_glu_kernel, dim3(unsigned(blocks)), dim3(256), 0, stream, static_cast<const __nv_bfloat16*>(gate),
                                static_cast<const __nv_bfloat16*>(up), static_cast<__nv_bfloat16*>(out), rows, f, ld_in, ld_out, beta));
  count_launch();
  return ALG_OK;
}

// Sum of squares of every row: one warp per row, 16-byte loads.
__global__ void __launch_bounds__(256) row_sumsq_kernel(const __nv_bfloat16* __restrict__ x, int64_t rows, int d, int64_t ld,
                                                        float* __restrict__ ss_out) {
  griddep_wait();                 // launched as a programmatic dependent of the kernel ahead in the stream
  const int lane = threadIdx.x & 31;
  const int64_t warp_global = (int64_t(blockIdx.x) * blockDim.x + threadIdx.x) >> 5;
  const int64_t warps_total = (int64_t(gridDim.x) * blockDim.x) >> 5;
  for (int64_t row = warp_global; row < rows; row += warps_total) {
    const uint4* src = reinterpret_cast<const uint4*>(x + row * ld);
    float ss = 0.f;
    for (int vi = lane; vi < d / 8; vi += 32) {
      float v[8];
      unpack8(src[vi], v);
#pragma unroll
      for (int i = 0; i < 8; ++i) ss = fmaf(v[i], v[i], ss);
    }
    ss = warp_sum(ss);
    if (lane == 0) ss_out[row] = ss;
  }
}

int launch_row_sumsq(const void* x, int64_t rows, int d, int64_t ld, float* ss_out, cudaStream_t stream) {
  if (rows == 0) return ALG_OK;
  int64_t blocks = (rows + 7) / 8;
  if (blocks > int64_t(sm_count()) * 8) blocks = int64_t(sm_count()) * 8;
  ALG_CUDA_TRY(launch_dependent(row_sumsq_kernel, dim3(unsigned(blocks)), dim3(256), 0, stream, static_cast<const __nv_bfloat16*>(x), rows, d, ld, ss_out));
  count_launch();
  return ALG_OK;
}

}  // namespace alg

using namespace alg;

extern "C" int alg_rms_norm_fwd(const void* x, const float* gain, void* y, int64_t rows, int d, float eps, void* stream) {
  if (x == nullptr || y == nullptr || rows < 0 || d < 8 || d % 8 != 0) { set_error("rms_norm: bad argument"); return ALG_ERR_INVALID; }
  if (!(eps > 0.0f)) { set_error("rms_norm: epsilon must be positive"); return ALG_ERR_INVALID; }
  if ((reinterpret_cast<uintptr_t>(x) | reinterpret_cast<uintptr_t>(y)) & 15) { set_error("rms_norm: 16-byte alignment required"); return ALG_ERR_INVALID; }
  return launch_rms_rows(x, gain, y, rows, d, eps, static_cast<cudaStream_t>(stream));
}

extern "C" int alg_alu_glu_fwd(const void* gate, const void* up, void* out, int64_t rows, int f, int64_t ld_in,
                               int64_t ld_out, float beta, void* stream) {
  if (rows < 0 || f < 0 || (rows * f != 0 && (gate == nullptr || up == nullptr || out == nullptr))) { set_error("alu_glu: bad argument"); return ALG_ERR_INVALID; }
  if (f % 8 != 0 || ld_in % 8 != 0 || ld_out % 8 != 0 || ld_in < f || ld_out < f) { set_error("alu_glu: f and the row strides must be multiples of 8, strides >= f"); return ALG_ERR_INVALID; }
  if ((reinterpret_cast<uintptr_t>(gate) | reinterpret_cast<uintptr_t>(up) | reinterpret_cast<uintptr_t>(out)) & 15) {
    set_error("alu_glu: 16-byte alignment required");
    return ALG_ERR_INVALID;
  }
  return launch_alu_glu(gate, up, out, rows, f, ld_in, ld_out, beta, static_cast<cudaStream_t>(stream));
}
