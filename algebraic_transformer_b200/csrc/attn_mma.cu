// Asinh-power attention forward on the legacy warp-level MMA path (mma.sync m16n8k16 bf16).
//
// This is the shape-general kernel: any Tq/Tk (tails masked), head_dim 64 or 128, bf16 or
// fp32 I/O, causal or not, with or without a sink, both accumulation strategies of the
// reference (src/algebraic/kernels/flash.py:227-259):
//   unshifted  p = rho_fast(x)^n,              l0 = rho(b')^n,  o = acc / l, stat = 1/l
//   shifted    p = (rho(x) rho(-m'))^n, alpha = (rho(m) rho(-m'))^n, running max m,
//              stat = rho(-m) l^(-1/n)
// chosen per launch, or on the device from the range-guard maxima.
//
// fp32 I/O keeps fp32-grade results on bf16 tensor cores by splitting every operand into
// hi + lo bf16 halves and issuing the three significant products (hi.hi, hi.lo, lo.hi);
// the dropped lo.lo term is below 2^-16 relative.
//
// One CTA = 64 query rows (4 warps x 16 rows), key tiles of 64, operands staged in padded
// shared memory and fed to the MMAs with ldmatrix.  The tcgen05 kernel (attn_sm100.cu) is
// the throughput path; this one defines the behaviour for everything it does not cover.
#include <math.h>

#include "common.cuh"
#include "launchers.h"

namespace alg {
namespace {

constexpr int BM = 64, BN = 64, NTHREADS = 128;

__device__ __forceinline__ void ldsm_x4(uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3, const void* p) {
  uint32_t a = static_cast<uint32_t>(__cvta_generic_to_shared(p));
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(a));
}
__device__ __forceinline__ void ldsm_x4_t(uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3, const void* p) {
  uint32_t a = static_cast<uint32_t>(__cvta_generic_to_shared(p));
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(a));
}
__device__ __forceinline__ void mma_bf16(float* c, const uint32_t* a, uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
               : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
               : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

// Stage `BM` rows x D of a (T, D) matrix into padded bf16 shared memory; rows >= T are zero.
template <typename T, int D, bool SPLIT>
__device__ __forceinline__ void stage_tile(const T* base, int64_t row_stride, int row0, int Tn,
                                           __nv_bfloat16* s_hi, __nv_bfloat16* s_lo) {
  constexpr int LD = D + 8;
  if constexpr (sizeof(T) == 2) {
    constexpr int VPR = D / 8;                       // 16-byte vectors per row
    for (int i = threadIdx.x; i < BM * VPR; i += NTHREADS) {
      const int r = i / VPR, cv = i % VPR;
      uint4 val = make_uint4(0, 0, 0, 0);
      if (row0 + r < Tn) val = *reinterpret_cast<const uint4*>(base + int64_t(row0 + r) * row_stride + cv * 8);
      *reinterpret_cast<uint4*>(s_hi + r * LD + cv * 8) = val;
    }
  } else {
    constexpr int VPR = D / 4;
    for (int i = threadIdx.x; i < BM * VPR; i += NTHREADS) {
      const int r = i / VPR, cv = i % VPR;
      float4 val = make_float4(0.f, 0.f, 0.f, 0.f);
      if (row0 + r < Tn) val = *reinterpret_cast<const float4*>(base + int64_t(row0 + r) * row_stride + cv * 4);
      const float f[4] = {val.x, val.y, val.z, val.w};
      float hi[4], lo[4];
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        hi[j] = __bfloat162float(__float2bfloat16_rn(f[j]));
        lo[j] = f[j] - hi[j];
      }
      *reinterpret_cast<uint2*>(s_hi + r * LD + cv * 4) = make_uint2(pack_bf16(hi[0], hi[1]), pack_bf16(hi[2], hi[3]));
      if constexpr (SPLIT)
        *reinterpret_cast<uint2*>(s_lo + r * LD + cv * 4) = make_uint2(pack_bf16(lo[0], lo[1]), pack_bf16(lo[2], lo[3]));
    }
  }
}

template <typename T, int D, bool SPLIT>
__global__ void __launch_bounds__(NTHREADS) attn_mma_kernel(const AttnParams p) {
  constexpr int LD = D + 8;
  constexpr int TILE = BM * LD;                      // elements per staged tile
  constexpr int NS = SPLIT ? 2 : 1;
  extern __shared__ __align__(16) unsigned char smem_raw[];
  __nv_bfloat16* sQ = reinterpret_cast<__nv_bfloat16*>(smem_raw);
  __nv_bfloat16* sK = sQ + NS * TILE;
  __nv_bfloat16* sV = sK + NS * TILE;
  __shared__ int s_shift;

  if (threadIdx.x < 32) {
    const bool sh = attn_use_shift(p, threadIdx.x);
    if (threadIdx.x == 0) s_shift = sh ? 1 : 0;
  }
  __syncthreads();
  const bool shift_mode = s_shift != 0;
  if ((p.run_if == 1 && shift_mode) || (p.run_if == 2 && !shift_mode)) return;

  // Persistent over work items (query tile, head, batch), long (late) query tiles first.  A
  // small grid keeps the launch cheap when the kernel only has to find out that the other
  // kernel family is doing the work (run_if).
  const int nqt = (p.Tq + BM - 1) / BM;
  const int total_items = nqt * p.H * p.B;
  for (int item = blockIdx.x; item < total_items; item += gridDim.x) {
  const int qt = nqt - 1 - item / (p.H * p.B);
  const int h = item % p.H, b = (item / p.H) % p.B;
  const int q0 = qt * BM;
  __syncthreads();                                        // the previous item's reads of sQ are done
  const int off = p.Tk - p.Tq;                            // causal: key j visible iff j <= i + off
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int g = lane >> 2, tq = lane & 3;

  if (item == 0 && threadIdx.x == 0 && p.stat_kind != nullptr)
    *p.stat_kind = shift_mode ? ALG_VARIANT_SHIFT : ALG_VARIANT_NOSHIFT;

  const T* qb = reinterpret_cast<const T*>(p.q) + b * p.qs.b + h * p.qs.h;
  const T* kb = reinterpret_cast<const T*>(p.k) + b * p.ks.b + h * p.ks.h;
  const T* vb = reinterpret_cast<const T*>(p.v) + b * p.vs.b + h * p.vs.h;

  stage_tile<T, D, SPLIT>(qb, p.qs.t, q0, p.Tq, sQ, sQ + TILE);

  const bool has_sink = p.sink != nullptr;
  const float bsink = has_sink ? p.sink[h] * p.inv_c : 0.0f;
  float m_run[2], l_run[2];
  float acc[D / 8][4];
#pragma unroll
  for (int i = 0; i < D / 8; ++i) { acc[i][0] = acc[i][1] = acc[i][2] = acc[i][3] = 0.f; }
  if (!shift_mode) {
    const float l0 = has_sink ? pow2n_rt(rho_stable(fminf(bsink, p.score_clamp)), p.log2n) : 0.0f;
    l_run[0] = l_run[1] = (tq == 0) ? l0 : 0.0f;         // partial sums live per lane; count l0 once
    m_run[0] = m_run[1] = 0.0f;
  } else {
    m_run[0] = m_run[1] = has_sink ? bsink : -1e30f;
    l_run[0] = l_run[1] = (has_sink && tq == 0) ? 1.0f : 0.0f;
  }

  int kt_last = (p.Tk + BN - 1) / BN - 1;
  if (p.causal) {
    const int last_key = min(p.Tk - 1, q0 + BM - 1 + off);
    kt_last = last_key < 0 ? -1 : min(kt_last, last_key / BN);
  }
  const int row_a = q0 + warp * 16 + g;                   // this lane's two query rows
  const int row_b = row_a + 8;

  for (int kt = 0; kt <= kt_last; ++kt) {
    const int k0 = kt * BN;
    __syncthreads();                                      // previous tile's reads are done (and sQ visible)
    stage_tile<T, D, SPLIT>(kb, p.ks.t, k0, p.Tk, sK, sK + TILE);
    stage_tile<T, D, SPLIT>(vb, p.vs.t, k0, p.Tk, sV, sV + TILE);
    __syncthreads();

    // ---- S = Q K^T (16 x 64 per warp) ----
    float s[BN / 8][4];
#pragma unroll
    for (int i = 0; i < BN / 8; ++i) { s[i][0] = s[i][1] = s[i][2] = s[i][3] = 0.f; }
#pragma unroll
    for (int ks = 0; ks < D / 16; ++ks) {
      uint32_t a_hi[4], a_lo[4];
      const int arow = warp * 16 + (lane & 15), acol = ks * 16 + (lane >> 4) * 8;
      ldsm_x4(a_hi[0], a_hi[1], a_hi[2], a_hi[3], sQ + arow * LD + acol);
      if constexpr (SPLIT) ldsm_x4(a_lo[0], a_lo[1], a_lo[2], a_lo[3], sQ + TILE + arow * LD + acol);
#pragma unroll
      for (int np = 0; np < BN / 16; ++np) {
        const int brow = np * 16 + (lane & 7) + (lane >> 4) * 8, bcol = ks * 16 + ((lane >> 3) & 1) * 8;
        uint32_t b0, b1, b2, b3;
        ldsm_x4(b0, b1, b2, b3, sK + brow * LD + bcol);
        mma_bf16(s[2 * np], a_hi, b0, b1);
        mma_bf16(s[2 * np + 1], a_hi, b2, b3);
        if constexpr (SPLIT) {
          mma_bf16(s[2 * np], a_lo, b0, b1);
          mma_bf16(s[2 * np + 1], a_lo, b2, b3);
          ldsm_x4(b0, b1, b2, b3, sK + TILE + brow * LD + bcol);
          mma_bf16(s[2 * np], a_hi, b0, b1);
          mma_bf16(s[2 * np + 1], a_hi, b2, b3);
        }
      }
    }

    // ---- weights ----
    const bool masked = (k0 + BN > p.Tk) || (p.causal && (k0 + BN - 1 > q0 + off));
    float alpha[2] = {1.f, 1.f};
    if (!shift_mode) {
      // rho^n as log2n passes over the fragment: every pass is a set of independent multiplications
      // (a loop per value would serialise on its own latency)
#pragma unroll
      for (int nt = 0; nt < BN / 8; ++nt)
#pragma unroll
        for (int e = 0; e < 4; ++e) s[nt][e] = rho_fast(fminf(s[nt][e] * p.scale, p.score_clamp));
      for (int it = 0; it < p.log2n; ++it) {
#pragma unroll
        for (int nt = 0; nt < BN / 8; ++nt)
#pragma unroll
          for (int e = 0; e < 4; ++e) s[nt][e] *= s[nt][e];
      }
#pragma unroll
      for (int nt = 0; nt < BN / 8; ++nt)
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const int col = k0 + nt * 8 + tq * 2 + (e & 1);
          const int row = (e < 2) ? row_a : row_b;
          float w = s[nt][e];
          if (masked) {
            const bool ok = col < p.Tk && (!p.causal || col <= row + off);
            w = ok ? w : 0.0f;
          }
          s[nt][e] = w;
          l_run[e >> 1] += w;
        }
    } else {
      float tmax[2] = {-1e30f, -1e30f};
#pragma unroll
      for (int nt = 0; nt < BN / 8; ++nt)
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const int col = k0 + nt * 8 + tq * 2 + (e & 1);
          const int row = (e < 2) ? row_a : row_b;
          const bool ok = !masked || (col < p.Tk && (!p.causal || col <= row + off));
          const float x = s[nt][e] * p.scale;
          s[nt][e] = ok ? x : -1e30f;
          tmax[e >> 1] = fmaxf(tmax[e >> 1], s[nt][e]);
        }
#pragma unroll
      for (int r = 0; r < 2; ++r) {
        tmax[r] = fmaxf(tmax[r], __shfl_xor_sync(0xffffffffu, tmax[r], 1));
        tmax[r] = fmaxf(tmax[r], __shfl_xor_sync(0xffffffffu, tmax[r], 2));
      }
      float shiftv[2];
#pragma unroll
      for (int r = 0; r < 2; ++r) {
        float m_prev = m_run[r];
        float m_new = fmaxf(m_prev, tmax[r]);
        if (!has_sink && kt == 0) { m_new = tmax[r]; m_prev = m_new; }   // first tile sets the maximum
        shiftv[r] = rho_stable(-m_new);
        alpha[r] = pow2n_rt(rho_stable(m_prev) * shiftv[r], p.log2n);
        m_run[r] = m_new;
        l_run[r] *= alpha[r];
      }
#pragma unroll
      for (int nt = 0; nt < BN / 8; ++nt)
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const bool ok = s[nt][e] > -1e29f;
          const float x = ok ? s[nt][e] : 0.0f;
          s[nt][e] = ok ? rho_stable(x) * shiftv[e >> 1] : 0.0f;   // a masked entry stays 0 under the power
        }
      for (int it = 0; it < p.log2n; ++it) {
#pragma unroll
        for (int nt = 0; nt < BN / 8; ++nt)
#pragma unroll
          for (int e = 0; e < 4; ++e) s[nt][e] *= s[nt][e];
      }
#pragma unroll
      for (int nt = 0; nt < BN / 8; ++nt)
#pragma unroll
        for (int e = 0; e < 4; ++e) l_run[e >> 1] += s[nt][e];
#pragma unroll
      for (int i = 0; i < D / 8; ++i) {
        acc[i][0] *= alpha[0]; acc[i][1] *= alpha[0];
        acc[i][2] *= alpha[1]; acc[i][3] *= alpha[1];
      }
    }

    // ---- O += P V ----
#pragma unroll
    for (int kk = 0; kk < BN / 16; ++kk) {
      uint32_t p_hi[4], p_lo[4];
      p_hi[0] = pack_bf16(s[2 * kk][0], s[2 * kk][1]);
      p_hi[1] = pack_bf16(s[2 * kk][2], s[2 * kk][3]);
      p_hi[2] = pack_bf16(s[2 * kk + 1][0], s[2 * kk + 1][1]);
      p_hi[3] = pack_bf16(s[2 * kk + 1][2], s[2 * kk + 1][3]);
      if constexpr (SPLIT) {
        auto lo2 = [](float a, float b2) {
          const float ra = a - __bfloat162float(__float2bfloat16_rn(a));
          const float rb = b2 - __bfloat162float(__float2bfloat16_rn(b2));
          return pack_bf16(ra, rb);
        };
        p_lo[0] = lo2(s[2 * kk][0], s[2 * kk][1]);
        p_lo[1] = lo2(s[2 * kk][2], s[2 * kk][3]);
        p_lo[2] = lo2(s[2 * kk + 1][0], s[2 * kk + 1][1]);
        p_lo[3] = lo2(s[2 * kk + 1][2], s[2 * kk + 1][3]);
      }
#pragma unroll
      for (int dp = 0; dp < D / 16; ++dp) {
        const int vrow = kk * 16 + (lane & 15), vcol = dp * 16 + (lane >> 4) * 8;
        uint32_t b0, b1, b2, b3;
        ldsm_x4_t(b0, b1, b2, b3, sV + vrow * LD + vcol);
        mma_bf16(acc[2 * dp], p_hi, b0, b1);
        mma_bf16(acc[2 * dp + 1], p_hi, b2, b3);
        if constexpr (SPLIT) {
          mma_bf16(acc[2 * dp], p_lo, b0, b1);
          mma_bf16(acc[2 * dp + 1], p_lo, b2, b3);
          ldsm_x4_t(b0, b1, b2, b3, sV + TILE + vrow * LD + vcol);
          mma_bf16(acc[2 * dp], p_hi, b0, b1);
          mma_bf16(acc[2 * dp + 1], p_hi, b2, b3);
        }
      }
    }
  }

  // ---- finalize ----
#pragma unroll
  for (int r = 0; r < 2; ++r) {
    l_run[r] += __shfl_xor_sync(0xffffffffu, l_run[r], 1);
    l_run[r] += __shfl_xor_sync(0xffffffffu, l_run[r], 2);
  }
  T* ob = reinterpret_cast<T*>(p.o) + b * p.os.b + h * p.os.h;
#pragma unroll
  for (int r = 0; r < 2; ++r) {
    const int row = r == 0 ? row_a : row_b;
    if (row >= p.Tq) continue;
    const float inv = 1.0f / l_run[r];
    T* orow = ob + int64_t(row) * p.os.t;
#pragma unroll
    for (int nt = 0; nt < D / 8; ++nt) {
      const float x0 = acc[nt][2 * r] * inv, x1 = acc[nt][2 * r + 1] * inv;
      const int col = nt * 8 + tq * 2;
      if constexpr (sizeof(T) == 2) *reinterpret_cast<uint32_t*>(orow + col) = pack_bf16(x0, x1);
      else *reinterpret_cast<float2*>(orow + col) = make_float2(x0, x1);
    }
    if (p.stat != nullptr && tq == 0) {
      const float st = shift_mode ? rho_stable(-m_run[r]) * inv_root_rt(l_run[r], p.log2n) : inv;
      p.stat[(int64_t(b) * p.H + h) * p.Tq + row] = st;
    }
  }
  }  // work items
}

template <typename T, int D, bool SPLIT>
int launch_one(const AttnParams& p, cudaStream_t stream) {
  constexpr int NS = SPLIT ? 2 : 1;
  constexpr size_t smem = size_t(3) * NS * BM * (D + 8) * sizeof(__nv_bfloat16);
  auto kern = attn_mma_kernel<T, D, SPLIT>;
  static PerDeviceOnce configured;
  int sms = 0;
  if (int rc = configured.run([&] { return cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, int(smem)); }, &sms)) return rc;
  const long long items = (long long)((p.Tq + BM - 1) / BM) * p.H * p.B;
  const int cap = sms * 4;                             // a few resident CTAs per SM; the loop covers the rest
  const unsigned grid = unsigned(items < cap ? items : cap);
  kern<<<grid, NTHREADS, smem, stream>>>(p);
  ALG_CUDA_TRY(cudaGetLastError());
  count_launch();
  return ALG_OK;
}

}  // namespace

int launch_attn_mma(const AttnParams& p, int dtype, cudaStream_t stream) {
  if (p.B == 0 || p.H == 0 || p.Tq == 0) return ALG_OK;
  if (p.D == 64) {
    return dtype == ALG_BF16 ? launch_one<__nv_bfloat16, 64, false>(p, stream)
                             : launch_one<float, 64, true>(p, stream);
  }
  if (p.D == 128) {
    return dtype == ALG_BF16 ? launch_one<__nv_bfloat16, 128, false>(p, stream)
                             : launch_one<float, 128, true>(p, stream);
  }
  set_error("attention needs head_dim 64 or 128, got %d", p.D);
  return ALG_ERR_UNSUPPORTED;
}

}  // namespace alg
