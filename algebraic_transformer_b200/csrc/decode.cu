// Single-query asinh-power attention against a KV cache (Tq = 1, all keys visible).
//
// HBM-bound: every K and V row is read exactly once with 128-bit loads.  Keys are split
// over CTAs (grid = splits x heads x batch) so that all SMs stream; inside a CTA a group of
// D/8 lanes owns one key at a time and keeps an online (m, l, acc) state in the
// max-shifted form  w = (rho(x) rho(-m))^n  of src/algebraic/algebraic.py:186-204.
// States are merged with the exact rescale (rho(m_a) rho(-m))^n — first across the lane
// groups of a CTA, then across splits (and the sink) by decode_combine_kernel.
#include "common.cuh"
#include "launchers.h"

namespace alg {
namespace {

constexpr int NTHREADS = 256;

__device__ __forceinline__ void load8(const __nv_bfloat16* p, float* v) {
  uint4 r = *reinterpret_cast<const uint4*>(p);
  const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&r);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    float2 f = __bfloat1622float2(h[i]);
    v[2 * i] = f.x; v[2 * i + 1] = f.y;
  }
}

template <int D>
__global__ void __launch_bounds__(NTHREADS) decode_partial_kernel(const DecodeParams p) {
  constexpr int LPK = D / 8;                    // lanes per key
  constexpr int SLOTS = NTHREADS / LPK;         // keys in flight per CTA step
  constexpr int UNROLL = 4;
  __shared__ float s_acc[SLOTS][D];
  __shared__ float s_m[SLOTS], s_l[SLOTS];

  const int split = blockIdx.x, h = blockIdx.y, b = blockIdx.z;
  const int slot = threadIdx.x / LPK, lik = threadIdx.x % LPK;
  const int per = (p.Tk + p.splits - 1) / p.splits;
  const int k_begin = split * per, k_end = min(p.Tk, k_begin + per);

  const __nv_bfloat16* qp = reinterpret_cast<const __nv_bfloat16*>(p.q) + (int64_t(b) * p.H + h) * D + lik * 8;
  const __nv_bfloat16* kb = reinterpret_cast<const __nv_bfloat16*>(p.k) + b * p.ks.b + h * p.ks.h + lik * 8;
  const __nv_bfloat16* vb = reinterpret_cast<const __nv_bfloat16*>(p.v) + b * p.vs.b + h * p.vs.h + lik * 8;
  float q[8];
  load8(qp, q);
#pragma unroll
  for (int i = 0; i < 8; ++i) q[i] *= p.scale;

  float m = -1e30f, l = 0.f, acc[8];
#pragma unroll
  for (int i = 0; i < 8; ++i) acc[i] = 0.f;
  float shift = 0.f;                            // rho(-m), refreshed when m moves

  // Trip count is uniform over the CTA (the shuffles below use the full warp mask).
  for (int kb0 = k_begin; kb0 < k_end; kb0 += SLOTS * UNROLL) {
    const int k0 = kb0 + slot;
    float kv[UNROLL][8], vv[UNROLL][8];
#pragma unroll
    for (int u = 0; u < UNROLL; ++u) {
      const int key = k0 + u * SLOTS;
      if (key < k_end) {
        load8(kb + int64_t(key) * p.ks.t, kv[u]);
        load8(vb + int64_t(key) * p.vs.t, vv[u]);
      } else {
#pragma unroll
        for (int i = 0; i < 8; ++i) { kv[u][i] = 0.f; vv[u][i] = 0.f; }
      }
    }
#pragma unroll
    for (int u = 0; u < UNROLL; ++u) {
      const int key = k0 + u * SLOTS;
      float x = 0.f;
#pragma unroll
      for (int i = 0; i < 8; ++i) x = fmaf(q[i], kv[u][i], x);
#pragma unroll
      for (int o = LPK / 2; o > 0; o >>= 1) x += __shfl_xor_sync(0xffffffffu, x, o);
      if (key < k_end) {                        // uniform within the lane group
        if (x > m) {
          const float ns = rho_stable(-x);
          const float alpha = (m > -1e29f) ? pow2n_rt(rho_stable(m) * ns, p.log2n) : 0.f;
          l *= alpha;
#pragma unroll
          for (int i = 0; i < 8; ++i) acc[i] *= alpha;
          m = x;
          shift = ns;
        }
        const float w = pow2n_rt(rho_stable(x) * shift, p.log2n);
        l += w;
#pragma unroll
        for (int i = 0; i < 8; ++i) acc[i] = fmaf(w, vv[u][i], acc[i]);
      }
    }
  }
  if (lik == 0) { s_m[slot] = m; s_l[slot] = l; }
#pragma unroll
  for (int i = 0; i < 8; ++i) s_acc[slot][lik * 8 + i] = acc[i];
  __syncthreads();

  // merge the CTA's lane groups: thread j < D owns output column j
  if (threadIdx.x < D) {
    float mm = -1e30f;
    for (int s = 0; s < SLOTS; ++s) mm = fmaxf(mm, s_m[s]);
    float lt = 0.f, at = 0.f;
    if (mm > -1e29f) {
      const float ns = rho_stable(-mm);
      for (int s = 0; s < SLOTS; ++s) {
        if (s_m[s] <= -1e29f) continue;
        const float a = pow2n_rt(rho_stable(s_m[s]) * ns, p.log2n);
        lt = fmaf(a, s_l[s], lt);
        at = fmaf(a, s_acc[s][threadIdx.x], at);
      }
    }
    float* out = p.part + ((int64_t(b) * p.H + h) * p.splits + split) * (D + 2);
    out[threadIdx.x] = at;
    if (threadIdx.x == 0) { out[D] = mm; out[D + 1] = lt; }
  }
}

template <int D>
__global__ void __launch_bounds__(D) decode_combine_kernel(const DecodeParams p) {
  const int bh = blockIdx.x, h = bh % p.H;
  const float* part = p.part + int64_t(bh) * p.splits * (D + 2);
  const bool has_sink = p.sink != nullptr;
  const float bs = has_sink ? p.sink[h] * p.inv_c : -1e30f;
  float mm = bs;
  for (int s = 0; s < p.splits; ++s) mm = fmaxf(mm, part[s * (D + 2) + D]);
  const float ns = rho_stable(-mm);
  float lt = has_sink ? pow2n_rt(rho_stable(bs) * ns, p.log2n) : 0.f;
  float at = 0.f;
  for (int s = 0; s < p.splits; ++s) {
    const float ms = part[s * (D + 2) + D];
    if (ms <= -1e29f) continue;
    const float a = pow2n_rt(rho_stable(ms) * ns, p.log2n);
    lt = fmaf(a, part[s * (D + 2) + D + 1], lt);
    at = fmaf(a, part[s * (D + 2) + threadIdx.x], at);
  }
  reinterpret_cast<__nv_bfloat16*>(p.o)[int64_t(bh) * D + threadIdx.x] = __float2bfloat16_rn(at / lt);
}

}  // namespace

int decode_splits(int B, int H, int Tk) {
  const int bh = B * H > 0 ? B * H : 1;
  int s = (148 * 4 + bh - 1) / bh;
  const int cap = (Tk + 255) / 256;
  if (s > cap) s = cap;
  return s < 1 ? 1 : s;
}

int launch_decode(const DecodeParams& p, cudaStream_t stream) {
  if (p.B == 0 || p.H == 0) return ALG_OK;
  dim3 grid(p.splits, p.H, p.B);
  if (p.D == 64) {
    decode_partial_kernel<64><<<grid, NTHREADS, 0, stream>>>(p);
    decode_combine_kernel<64><<<p.B * p.H, 64, 0, stream>>>(p);
  } else if (p.D == 128) {
    decode_partial_kernel<128><<<grid, NTHREADS, 0, stream>>>(p);
    decode_combine_kernel<128><<<p.B * p.H, 128, 0, stream>>>(p);
  } else {
    set_error("decode needs head_dim 64 or 128, got %d", p.D);
    return ALG_ERR_UNSUPPORTED;
  }
  ALG_CUDA_TRY(cudaGetLastError());
  count_launch(2);
  return ALG_OK;
}

}  // namespace alg
