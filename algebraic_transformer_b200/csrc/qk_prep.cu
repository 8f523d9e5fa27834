// QK RMS-normalisation, Cayley rotation and the range-guard maxima in one HBM-bound pass.
//
// One 16-byte vector per lane, D*sizeof(T)/16 lanes per row, so a warp streams whole
// rows with fully coalesced 128-bit loads and stores.  The rotate-half partner of an
// element lives in lane ^ (lanes_per_row/2) and is fetched with one shuffle.
//
// Semantics (reference paths): rms_norm src/algebraic/algebraic.py:76-83 (fp32 math, one
// rounding to the I/O dtype), apply_rotary src/algebraic/algebraic.py:172-179 (tables cast
// to the I/O dtype, arithmetic in that dtype), guard maxima src/algebraic/kernels/flash.py:
// 831-849 (row norms of the re-rounded scaled q, row norms of k, max |v|).
#include "common.cuh"
#include "launchers.h"

namespace alg {

template <typename T> struct Vec16;
template <> struct Vec16<float> {
  static constexpr int N = 4;
  static __device__ __forceinline__ void load(const float* p, float* v) {
    float4 r = *reinterpret_cast<const float4*>(p);
    v[0] = r.x; v[1] = r.y; v[2] = r.z; v[3] = r.w;
  }
  static __device__ __forceinline__ void store(float* p, const float* v) {
    *reinterpret_cast<float4*>(p) = make_float4(v[0], v[1], v[2], v[3]);
  }
  static __device__ __forceinline__ float round(float x) { return x; }
};
template <> struct Vec16<__nv_bfloat16> {
  static constexpr int N = 8;
  static __device__ __forceinline__ void load(const __nv_bfloat16* p, float* v) {
    uint4 r = *reinterpret_cast<const uint4*>(p);
    const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&r);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      float2 f = __bfloat1622float2(h[i]);
      v[2 * i] = f.x; v[2 * i + 1] = f.y;
    }
  }
  static __device__ __forceinline__ void store(__nv_bfloat16* p, const float* v) {
    uint4 r;
    uint32_t* w = reinterpret_cast<uint32_t*>(&r);
#pragma unroll
    for (int i = 0; i < 4; ++i) w[i] = pack_bf16(v[2 * i], v[2 * i + 1]);
    *reinterpret_cast<uint4*>(p) = r;
  }
  static __device__ __forceinline__ float round(float x) {
    return __bfloat162float(__float2bfloat16_rn(x));
  }
};

template <typename T, int D>
__global__ void __launch_bounds__(256) qk_prep_kernel(PrepParams p) {
  using V = Vec16<T>;
  constexpr int VEC = V::N;
  constexpr int LPR = D / VEC;         // lanes per row
  constexpr int RPW = 32 / LPR;        // rows per warp
  constexpr int HALF = D / 2;
  const int lane = threadIdx.x & 31;
  const int lir = lane % LPR;          // lane in row
  const int sub = lane / LPR;
  const int64_t rows = int64_t(p.B) * p.H * p.T;
  const int64_t warp_global = (int64_t(blockIdx.x) * blockDim.x + threadIdx.x) >> 5;
  const int64_t warps_total = (int64_t(gridDim.x) * blockDim.x) >> 5;

  float gain[VEC];
#pragma unroll
  for (int i = 0; i < VEC; ++i) gain[i] = (p.gain != nullptr) ? p.gain[lir * VEC + i] : 1.0f;

  float stat = 0.0f;
  for (int64_t r0 = warp_global * RPW; r0 < rows; r0 += warps_total * RPW) {
    const int64_t row = r0 + sub;
    const bool live = row < rows;
    const int64_t rr = live ? row : rows - 1;
    const int t = int(rr % p.T);
    const int64_t bh = rr / p.T;
    const int h = int(bh % p.H);
    const int64_t b = bh / p.H;
    const T* src = reinterpret_cast<const T*>(p.x) + b * p.xs.b + h * p.xs.h + t * p.xs.t + lir * VEC;
    float v[VEC];
    V::load(src, v);

    if (p.normalise) {
      float ss = 0.0f;
#pragma unroll
      for (int i = 0; i < VEC; ++i) ss = fmaf(v[i], v[i], ss);
#pragma unroll
      for (int o = LPR / 2; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
      const float tau = rsqrtf(ss * (1.0f / D) + p.eps);
#pragma unroll
      for (int i = 0; i < VEC; ++i) v[i] = V::round((v[i] * tau) * gain[i]);
    }
    if (p.cos != nullptr) {
      const bool first = lir < LPR / 2;
      const int j0 = (lir % (LPR / 2)) * VEC;
      const float* ct = p.cos + int64_t(t) * HALF + j0;
      const float* st = p.sin + int64_t(t) * HALF + j0;
#pragma unroll
      for (int i = 0; i < VEC; ++i) {
        const float other = __shfl_xor_sync(0xffffffffu, v[i], LPR / 2);
        const float c = V::round(ct[i]), s = V::round(st[i]);
        const float x1 = first ? v[i] : other;
        const float x2 = first ? other : v[i];
        // first half: x1 c - x2 s ; second half: x1 s + x2 c, each product rounded to T
        const float a = V::round(x1 * (first ? c : s));
        const float bb = V::round(x2 * (first ? s : c));
        v[i] = V::round(first ? a - bb : a + bb);
      }
    }
    if (p.y != nullptr && live) {
      T* dst = reinterpret_cast<T*>(p.y) + b * p.ys.b + h * p.ys.h + t * p.ys.t + lir * VEC;
      V::store(dst, v);
    }
    if (p.stat_mode == 1) {            // squared row norm of the re-rounded scaled row
      float ss = 0.0f;
#pragma unroll
      for (int i = 0; i < VEC; ++i) {
        const float s = V::round(v[i] * p.stat_scale);
        ss = fmaf(s, s, ss);
      }
#pragma unroll
      for (int o = LPR / 2; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
      if (live) stat = fmaxf(stat, ss);
    } else if (p.stat_mode == 2) {     // max |x|
      float m = 0.0f;
#pragma unroll
      for (int i = 0; i < VEC; ++i) m = fmaxf(m, fabsf(v[i]));
      if (live) stat = fmaxf(stat, m);
    }
  }
  if (p.stat_mode != 0) {
    stat = warp_max(stat);
    // NaN inputs must fail the guard: map NaN to +inf before the integer max.
    if (!(stat == stat)) stat = __int_as_float(0x7f800000);
    if (lane == 0) atomicMax(p.stat_out, __float_as_uint(stat));
  }
}

template <typename T, int D>
static int launch_t(const PrepParams& p, cudaStream_t stream) {
  constexpr int LPR = D * int(sizeof(T)) / 16;
  constexpr int RPW = 32 / LPR;
  const int64_t rows = int64_t(p.B) * p.H * p.T;
  if (rows == 0) return ALG_OK;
  const int64_t warps = (rows + RPW - 1) / RPW;
  int64_t blocks = (warps + 7) / 8;
  const int64_t cap = 148 * 16;        // a few waves of resident CTAs; grid-stride covers the rest
  if (blocks > cap) blocks = cap;
  qk_prep_kernel<T, D><<<dim3(unsigned(blocks)), 256, 0, stream>>>(p);
  ALG_CUDA_TRY(cudaGetLastError());
  count_launch();
  return ALG_OK;
}

int launch_prep(const PrepParams& p, int dtype, cudaStream_t stream) {
  if (p.D != 64 && p.D != 128) {
    set_error("QK prologue needs head_dim 64 or 128, got %d", p.D);
    return ALG_ERR_UNSUPPORTED;
  }
  if (dtype == ALG_BF16)
    return p.D == 64 ? launch_t<__nv_bfloat16, 64>(p, stream) : launch_t<__nv_bfloat16, 128>(p, stream);
  if (dtype == ALG_F32)
    return p.D == 64 ? launch_t<float, 64>(p, stream) : launch_t<float, 128>(p, stream);
  set_error("unknown dtype %d", dtype);
  return ALG_ERR_INVALID;
}

__global__ void cast_f32_bf16_kernel(const float* __restrict__ src, __nv_bfloat16* __restrict__ dst,
                                     size_t count) {
  const size_t stride = size_t(gridDim.x) * blockDim.x * 8;
  for (size_t i = (size_t(blockIdx.x) * blockDim.x + threadIdx.x) * 8; i < count; i += stride) {
    if (i + 8 <= count) {
      const float4 a = *reinterpret_cast<const float4*>(src + i);
      const float4 b = *reinterpret_cast<const float4*>(src + i + 4);
      uint4 r;
      r.x = pack_bf16(a.x, a.y); r.y = pack_bf16(a.z, a.w);
      r.z = pack_bf16(b.x, b.y); r.w = pack_bf16(b.z, b.w);
      *reinterpret_cast<uint4*>(dst + i) = r;
    } else {
      for (size_t j = i; j < count; ++j) dst[j] = __float2bfloat16_rn(src[j]);
    }
  }
}

int launch_cast(const float* src, void* dst, size_t count, cudaStream_t stream) {
  if (count == 0) return ALG_OK;
  size_t blocks = (count / 8 + 255) / 256;
  if (blocks > 148 * 16) blocks = 148 * 16;
  if (blocks == 0) blocks = 1;
  cast_f32_bf16_kernel<<<unsigned(blocks), 256, 0, stream>>>(src, reinterpret_cast<__nv_bfloat16*>(dst), count);
  ALG_CUDA_TRY(cudaGetLastError());
  count_launch();
  return ALG_OK;
}

}  // namespace alg
