// Asinh-power attention backward (dQ, dK, dV, dsink) from the forward's saved per-row statistic,
// on warp-level MMAs (mma.sync m16n8k16 bf16).  Reference: the custom VJP of
// src/algebraic/kernels/flash.py:333-727 (algorithm: recompute the normalised weights of a tile
// from q, k and the statistic, never the (T, T) matrix).
//
// With x = q.k / (sqrt(D) c), w = rho(x)^n, l = sum_j w + w_sink, p = w / l, o = sum_j p v:
//   delta_i = dO_i . o_i                      dP_ij = dO_i . v_j
//   dx_ij   = n p_ij (dP_ij - delta_i) / sqrt(1 + x_ij^2)        (d log rho / dx = 1 / sqrt(1 + x^2))
//   dQ_i = sum_j dx_ij k_j / (sqrt(D) c)      dK_j = sum_i dx_ij q_i / (sqrt(D) c)
//   dV_j = sum_i p_ij dO_i                    dsink = -sum_i delta_i p_sink,i n / (c sqrt(1 + (b/c)^2))
// p is rebuilt from the statistic: p = rho_fast(x)^n * stat (stat = 1/l, unshifted forward) or
// p = (rho(x) * stat)^n (stat = rho(-m) l^(-1/n), shifted forward).
//
// Two kernels, both shaped like the forward kernel of attn_mma.cu so that only its two operand
// patterns occur (A.B^T from two row-major tiles; (weights from registers).B):
//   attn_bwd_dq_kernel   one CTA = 64 query rows; for every visible key tile: S = Q K^T,
//                        dP = dO V^T, dS, dQ += dS K.  Also writes delta and adds up dsink.
//   attn_bwd_dkv_kernel  one CTA = 64 keys; for every query tile that sees them: S^T = K Q^T,
//                        dP^T = V dO^T, dV += P^T dO, dK += dS^T Q.
// S is therefore evaluated twice; in exchange no atomics and no transposes are needed.  The
// tiles a CTA streams (K, V in the first kernel, Q, dO in the second) are double-buffered with
// cp.async, so the next tile's copy runs under the current tile's MMAs.
// bf16 tensors, fp32 accumulation.
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

// 64 rows x D of a (T, D) bf16 matrix into padded shared memory; rows >= Tn are zero.
template <int D>
__device__ __forceinline__ void stage_tile(const __nv_bfloat16* base, int64_t row_stride, int row0, int Tn,
                                           __nv_bfloat16* s) {
  constexpr int LD = D + 8, VPR = D / 8;
  for (int i = threadIdx.x; i < BM * VPR; i += NTHREADS) {
    const int r = i / VPR, cv = i % VPR;
    uint4 val = make_uint4(0, 0, 0, 0);
    if (row0 + r < Tn) val = *reinterpret_cast<const uint4*>(base + int64_t(row0 + r) * row_stride + cv * 8);
    *reinterpret_cast<uint4*>(s + r * LD + cv * 8) = val;
  }
}

// The same with cp.async (16-byte pieces, zero-filled past Tn): the copy of the next tile runs
// while the current one is multiplied.  Completed with cp_async_wait<N>() + __syncthreads().
template <int D>
__device__ __forceinline__ void stage_tile_async(const __nv_bfloat16* base, int64_t row_stride, int row0, int Tn,
                                                 __nv_bfloat16* s) {
  constexpr int LD = D + 8, VPR = D / 8;
  for (int i = threadIdx.x; i < BM * VPR; i += NTHREADS) {
    const int r = i / VPR, cv = i % VPR;
    const bool live = row0 + r < Tn;
    const __nv_bfloat16* src = base + int64_t(live ? row0 + r : 0) * row_stride + cv * 8;
    const uint32_t dst = static_cast<uint32_t>(__cvta_generic_to_shared(s + r * LD + cv * 8));
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(dst), "l"(src), "r"(live ? 16 : 0) : "memory");
  }
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N> __device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

// c (16 x 64 per warp) = A[warp's 16 rows] . B^T, both tiles row-major [row][D] in shared memory
template <int D>
__device__ __forceinline__ void gemm_abt(float (*c)[4], const __nv_bfloat16* sA, const __nv_bfloat16* sB, int warp, int lane) {
  constexpr int LD = D + 8;
#pragma unroll
  for (int i = 0; i < BN / 8; ++i) { c[i][0] = c[i][1] = c[i][2] = c[i][3] = 0.f; }
#pragma unroll
  for (int ks = 0; ks < D / 16; ++ks) {
    uint32_t a[4];
    const int arow = warp * 16 + (lane & 15), acol = ks * 16 + (lane >> 4) * 8;
    ldsm_x4(a[0], a[1], a[2], a[3], sA + arow * LD + acol);
#pragma unroll
    for (int np = 0; np < BN / 16; ++np) {
      const int brow = np * 16 + (lane & 7) + (lane >> 4) * 8, bcol = ks * 16 + ((lane >> 3) & 1) * 8;
      uint32_t b0, b1, b2, b3;
      ldsm_x4(b0, b1, b2, b3, sB + brow * LD + bcol);
      mma_bf16(c[2 * np], a, b0, b1);
      mma_bf16(c[2 * np + 1], a, b2, b3);
    }
  }
}

// acc (16 x D per warp) += W (16 x 64, fp32 accumulator layout in registers) . B, B row-major [64][D]
template <int D>
__device__ __forceinline__ void gemm_wb(float (*acc)[4], const float (*w)[4], const __nv_bfloat16* sB, int lane) {
  constexpr int LD = D + 8;
#pragma unroll
  for (int kk = 0; kk < BN / 16; ++kk) {
    uint32_t a[4];
    a[0] = pack_bf16(w[2 * kk][0], w[2 * kk][1]);
    a[1] = pack_bf16(w[2 * kk][2], w[2 * kk][3]);
    a[2] = pack_bf16(w[2 * kk + 1][0], w[2 * kk + 1][1]);
    a[3] = pack_bf16(w[2 * kk + 1][2], w[2 * kk + 1][3]);
#pragma unroll
    for (int dp = 0; dp < D / 16; ++dp) {
      const int brow = kk * 16 + (lane & 15), bcol = dp * 16 + (lane >> 4) * 8;
      uint32_t b0, b1, b2, b3;
      ldsm_x4_t(b0, b1, b2, b3, sB + brow * LD + bcol);
      mma_bf16(acc[2 * dp], a, b0, b1);
      mma_bf16(acc[2 * dp + 1], a, b2, b3);
    }
  }
}

// The normalised weight of a score is base^n (times the statistic on the unshifted path); the power
// is taken afterwards for a whole fragment at once (power_passes).  Returns the base and, in `slope`,
// n / (sqrt(1 + x^2) sqrt(D) c): weight * slope turns (dP - delta) into dS.
__device__ __forceinline__ float weight_base(float s_raw, float stat, bool shifted, const AttnBwdParams& p, float& slope) {
  const float x = s_raw * p.scale;
  const float rs = rsqrtf(fmaf(x, x, 1.0f));           // 1 / sqrt(1 + x^2)
  slope = p.n_scale * rs;
  return shifted ? rho_stable(x) * stat : rho_fast(x);
}
// w <- w^(2^log2n) for the 32 values of a fragment: log2n passes of independent multiplications (a
// loop per value would serialise on its own latency).
__device__ __forceinline__ void power_passes(float (*w)[4], int log2n) {
  for (int it = 0; it < log2n; ++it) {
#pragma unroll
    for (int nt = 0; nt < BN / 8; ++nt)
#pragma unroll
      for (int e = 0; e < 4; ++e) w[nt][e] *= w[nt][e];
  }
}

template <int D>
__device__ __forceinline__ void store_rows(const float (*acc)[4], __nv_bfloat16* base, int64_t row_stride, int row_a,
                                           int Tn, int tq) {
#pragma unroll
  for (int r = 0; r < 2; ++r) {
    const int row = row_a + 8 * r;
    if (row >= Tn) continue;
    __nv_bfloat16* orow = base + int64_t(row) * row_stride;
#pragma unroll
    for (int nt = 0; nt < D / 8; ++nt)
      *reinterpret_cast<uint32_t*>(orow + nt * 8 + tq * 2) = pack_bf16(acc[nt][2 * r], acc[nt][2 * r + 1]);
  }
}

template <int D>
__global__ void __launch_bounds__(NTHREADS) attn_bwd_dq_kernel(const AttnBwdParams p) {
  constexpr int LD = D + 8, TILE = BM * LD;
  extern __shared__ __align__(16) unsigned char smem_raw[];
  __nv_bfloat16* sQ = reinterpret_cast<__nv_bfloat16*>(smem_raw);
  __nv_bfloat16* sdO = sQ + TILE;
  __nv_bfloat16* sKV = sdO + TILE;                     // two stages of [K tile | V tile]
  __shared__ float s_delta[BM];
  __shared__ float s_sink[NTHREADS / 32];

  const int nqt = (p.Tq + BM - 1) / BM;
  const int qt = nqt - 1 - int(blockIdx.x), h = blockIdx.y, b = blockIdx.z;   // heavy (late) tiles first
  const int q0 = qt * BM, off = p.Tk - p.Tq;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, tq = lane & 3;
  const bool shifted = *p.stat_kind == ALG_VARIANT_SHIFT;

  const __nv_bfloat16* qb = p.q + b * p.qs.b + h * p.qs.h;
  const __nv_bfloat16* kb = p.k + b * p.ks.b + h * p.ks.h;
  const __nv_bfloat16* vb = p.v + b * p.vs.b + h * p.vs.h;
  const __nv_bfloat16* ob = p.o + b * p.os.b + h * p.os.h;
  const __nv_bfloat16* dob = p.d_o + b * p.os.b + h * p.os.h;
  const int64_t bh = int64_t(b) * p.H + h;

  stage_tile<D>(qb, p.qs.t, q0, p.Tq, sQ);
  stage_tile<D>(dob, p.os.t, q0, p.Tq, sdO);
  // delta_i = dO_i . o_i: two threads per row, half of the columns each
  {
    const int r = threadIdx.x >> 1, half = threadIdx.x & 1;
    float d = 0.f;
    if (q0 + r < p.Tq) {
      const __nv_bfloat16* orow = ob + int64_t(q0 + r) * p.os.t + half * (D / 2);
      const __nv_bfloat16* drow = dob + int64_t(q0 + r) * p.os.t + half * (D / 2);
#pragma unroll
      for (int cv = 0; cv < D / 16; ++cv) {
        const uint4 a = *reinterpret_cast<const uint4*>(orow + cv * 8), c = *reinterpret_cast<const uint4*>(drow + cv * 8);
        const __nv_bfloat162* a2 = reinterpret_cast<const __nv_bfloat162*>(&a);
        const __nv_bfloat162* c2 = reinterpret_cast<const __nv_bfloat162*>(&c);
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const float2 fa = __bfloat1622float2(a2[i]), fc = __bfloat1622float2(c2[i]);
          d = fmaf(fa.x, fc.x, d);
          d = fmaf(fa.y, fc.y, d);
        }
      }
    }
    d += __shfl_xor_sync(0xffffffffu, d, 1);
    if (half == 0) {
      s_delta[r] = d;
      if (q0 + r < p.Tq) p.delta[bh * p.Tq + q0 + r] = d;
    }
  }
  __syncthreads();

  const int row_a = q0 + warp * 16 + g, row_b = row_a + 8;
  const float stat_a = row_a < p.Tq ? p.stat[bh * p.Tq + row_a] : 0.f;
  const float stat_b = row_b < p.Tq ? p.stat[bh * p.Tq + row_b] : 0.f;
  const float delta_a = s_delta[warp * 16 + g], delta_b = s_delta[warp * 16 + g + 8];

  float acc[D / 8][4];
#pragma unroll
  for (int i = 0; i < D / 8; ++i) { acc[i][0] = acc[i][1] = acc[i][2] = acc[i][3] = 0.f; }

  int kt_last = (p.Tk + BN - 1) / BN - 1;
  if (p.causal) {
    const int last_key = min(p.Tk - 1, q0 + BM - 1 + off);
    kt_last = last_key < 0 ? -1 : min(kt_last, last_key / BN);
  }
  if (kt_last >= 0) {
    stage_tile_async<D>(kb, p.ks.t, 0, p.Tk, sKV);
    stage_tile_async<D>(vb, p.vs.t, 0, p.Tk, sKV + TILE);
  }
  cp_async_commit();
  for (int kt = 0; kt <= kt_last; ++kt) {
    const int k0 = kt * BN;
    const __nv_bfloat16* sK = sKV + (kt & 1) * 2 * TILE;
    const __nv_bfloat16* sV = sK + TILE;
    if (kt < kt_last) {                                   // next tile into the other stage (its readers finished
      __nv_bfloat16* nx = sKV + ((kt + 1) & 1) * 2 * TILE;   // at the barrier that ended the previous step)
      stage_tile_async<D>(kb, p.ks.t, k0 + BN, p.Tk, nx);
      stage_tile_async<D>(vb, p.vs.t, k0 + BN, p.Tk, nx + TILE);
    }
    cp_async_commit();
    cp_async_wait<1>();                                   // this step's tile has landed
    __syncthreads();
    float s[BN / 8][4], dp[BN / 8][4];
    gemm_abt<D>(s, sQ, sK, warp, lane);                   // S  = Q K^T
    gemm_abt<D>(dp, sdO, sV, warp, lane);                 // dP = dO V^T
    const bool masked = (k0 + BN > p.Tk) || (p.causal && (k0 + BN - 1 > q0 + off));
#pragma unroll
    for (int nt = 0; nt < BN / 8; ++nt)
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        float slope;
        s[nt][e] = weight_base(s[nt][e], (e < 2) ? stat_a : stat_b, shifted, p, slope);
        dp[nt][e] = slope * (dp[nt][e] - ((e < 2) ? delta_a : delta_b));
      }
    power_passes(s, p.log2n);
#pragma unroll
    for (int nt = 0; nt < BN / 8; ++nt)
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const int col = k0 + nt * 8 + tq * 2 + (e & 1);
        const int row = (e < 2) ? row_a : row_b;
        const float pw = shifted ? s[nt][e] : s[nt][e] * ((e < 2) ? stat_a : stat_b);
        float ds = pw * dp[nt][e];
        if (masked && !(col < p.Tk && (!p.causal || col <= row + off))) ds = 0.f;
        s[nt][e] = ds;
      }
    gemm_wb<D>(acc, s, sK, lane);                         // dQ += dS K
    __syncthreads();                                      // this stage may be refilled by the next step
  }
  store_rows<D>(acc, p.dq + b * p.qs.b + h * p.qs.h, p.qs.t, row_a, p.Tq, tq);

  // dsink: -sum_i delta_i p_sink,i * n / (c sqrt(1 + (b/c)^2))
  if (p.sink != nullptr && p.dsink != nullptr) {
    float part = 0.f;
    if (threadIdx.x < BM && q0 + int(threadIdx.x) < p.Tq) {
      const float bs = p.sink[h] * p.inv_c, st = p.stat[bh * p.Tq + q0 + threadIdx.x];
      const float ps = shifted ? pow2n_rt(rho_stable(bs) * st, p.log2n) : pow2n_rt(rho_stable(bs), p.log2n) * st;
      part = -s_delta[threadIdx.x] * ps * p.n_f * p.inv_c * rsqrtf(fmaf(bs, bs, 1.0f));
    }
    part = warp_sum(part);
    if (lane == 0) s_sink[warp] = part;
    __syncthreads();
    if (threadIdx.x == 0) atomicAdd(p.dsink + h, (s_sink[0] + s_sink[1]) + (s_sink[2] + s_sink[3]));
  }
}

template <int D>
__global__ void __launch_bounds__(NTHREADS) attn_bwd_dkv_kernel(const AttnBwdParams p) {
  constexpr int LD = D + 8, TILE = BM * LD;
  extern __shared__ __align__(16) unsigned char smem_raw[];
  __nv_bfloat16* sK = reinterpret_cast<__nv_bfloat16*>(smem_raw);
  __nv_bfloat16* sV = sK + TILE;
  __nv_bfloat16* sQO = sV + TILE;                      // two stages of [Q tile | dO tile]
  __shared__ float s_stat[2][BM], s_delta[2][BM];

  const int kt = blockIdx.x, h = blockIdx.y, b = blockIdx.z;                  // early key tiles are the heavy ones
  const int k0 = kt * BN, off = p.Tk - p.Tq;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, tq = lane & 3;
  const bool shifted = *p.stat_kind == ALG_VARIANT_SHIFT;

  const __nv_bfloat16* qb = p.q + b * p.qs.b + h * p.qs.h;
  const __nv_bfloat16* kb = p.k + b * p.ks.b + h * p.ks.h;
  const __nv_bfloat16* vb = p.v + b * p.vs.b + h * p.vs.h;
  const __nv_bfloat16* dob = p.d_o + b * p.os.b + h * p.os.h;
  const int64_t bh = int64_t(b) * p.H + h;

  stage_tile<D>(kb, p.ks.t, k0, p.Tk, sK);
  stage_tile<D>(vb, p.vs.t, k0, p.Tk, sV);

  float dk[D / 8][4], dv[D / 8][4];
#pragma unroll
  for (int i = 0; i < D / 8; ++i) {
    dk[i][0] = dk[i][1] = dk[i][2] = dk[i][3] = 0.f;
    dv[i][0] = dv[i][1] = dv[i][2] = dv[i][3] = 0.f;
  }
  const int key_a = k0 + warp * 16 + g, key_b = key_a + 8;   // this lane's two keys (rows of S^T)

  const int nqt = (p.Tq + BM - 1) / BM;
  int qt_first = 0;
  if (p.causal) {                                           // first query row that sees key k0: i >= k0 - off
    const int first_row = max(0, k0 - off);
    qt_first = first_row / BM;
  }
  auto stage_queries = [&](int qt, int stage) {           // Q, dO (asynchronously) and the rows' stat, delta
    const int q0 = qt * BM;
    __nv_bfloat16* dst = sQO + stage * 2 * TILE;
    stage_tile_async<D>(qb, p.qs.t, q0, p.Tq, dst);
    stage_tile_async<D>(dob, p.os.t, q0, p.Tq, dst + TILE);
    if (threadIdx.x < BM) {
      const bool live = q0 + int(threadIdx.x) < p.Tq;
      s_stat[stage][threadIdx.x] = live ? p.stat[bh * p.Tq + q0 + threadIdx.x] : 0.f;
      s_delta[stage][threadIdx.x] = live ? p.delta[bh * p.Tq + q0 + threadIdx.x] : 0.f;
    }
  };
  if (qt_first < nqt) stage_queries(qt_first, 0);
  cp_async_commit();
  for (int qt = qt_first; qt < nqt; ++qt) {
    const int q0 = qt * BM, stage = (qt - qt_first) & 1;
    const __nv_bfloat16* sQ = sQO + stage * 2 * TILE;
    const __nv_bfloat16* sdO = sQ + TILE;
    if (qt + 1 < nqt) stage_queries(qt + 1, stage ^ 1);     // its readers finished at the previous step's last barrier
    cp_async_commit();
    cp_async_wait<1>();
    __syncthreads();                                        // this step's tiles (and, first time, sK, sV) are visible
    float st[BN / 8][4], dpt[BN / 8][4];
    gemm_abt<D>(st, sK, sQ, warp, lane);                    // S^T  = K Q^T   (keys x queries)
    gemm_abt<D>(dpt, sV, sdO, warp, lane);                  // dP^T = V dO^T
    // the key tile straddles the diagonal or an edge of either sequence
    const bool masked = (q0 + BM > p.Tq) || (k0 + BN > p.Tk) || (p.causal && (k0 + BN - 1 > q0 + off));
#pragma unroll
    for (int nt = 0; nt < BN / 8; ++nt)
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const int qc = nt * 8 + tq * 2 + (e & 1);           // query inside the tile (column of S^T)
        float slope;
        st[nt][e] = weight_base(st[nt][e], s_stat[stage][qc], shifted, p, slope);
        dpt[nt][e] = slope * (dpt[nt][e] - s_delta[stage][qc]);
      }
    power_passes(st, p.log2n);
#pragma unroll
    for (int nt = 0; nt < BN / 8; ++nt)
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const int qc = nt * 8 + tq * 2 + (e & 1);
        const int qi = q0 + qc, kj = (e < 2) ? key_a : key_b;
        float pw = shifted ? st[nt][e] : st[nt][e] * s_stat[stage][qc];
        float ds = pw * dpt[nt][e];
        if (masked && !(qi < p.Tq && kj < p.Tk && (!p.causal || kj <= qi + off))) { pw = 0.f; ds = 0.f; }
        st[nt][e] = pw;
        dpt[nt][e] = ds;
      }
    gemm_wb<D>(dv, st, sdO, lane);                          // dV += P^T dO
    gemm_wb<D>(dk, dpt, sQ, lane);                          // dK += dS^T Q
    __syncthreads();                                        // this stage may be refilled by the next step
  }
  store_rows<D>(dk, p.dk + b * p.ks.b + h * p.ks.h, p.ks.t, key_a, p.Tk, tq);
  store_rows<D>(dv, p.dv + b * p.vs.b + h * p.vs.h, p.vs.t, key_a, p.Tk, tq);
}

template <int D>
int launch_d(const AttnBwdParams& p, cudaStream_t stream) {
  constexpr size_t smem = size_t(6) * BM * (D + 8) * sizeof(__nv_bfloat16);   // 2 resident tiles + 2 stages of 2
  static PerDeviceOnce configured;
  if (int rc = configured.run([&] {
        cudaError_t e = cudaFuncSetAttribute(attn_bwd_dq_kernel<D>, cudaFuncAttributeMaxDynamicSharedMemorySize, int(smem));
        return e != cudaSuccess ? e : cudaFuncSetAttribute(attn_bwd_dkv_kernel<D>, cudaFuncAttributeMaxDynamicSharedMemorySize, int(smem));
      })) return rc;
  const dim3 gq((p.Tq + BM - 1) / BM, p.H, p.B), gk((p.Tk + BN - 1) / BN, p.H, p.B);
  attn_bwd_dq_kernel<D><<<gq, NTHREADS, smem, stream>>>(p);
  ALG_CUDA_TRY(cudaGetLastError());
  attn_bwd_dkv_kernel<D><<<gk, NTHREADS, smem, stream>>>(p);
  ALG_CUDA_TRY(cudaGetLastError());
  count_launch(2);
  return ALG_OK;
}

}  // namespace

int launch_attn_bwd(const AttnBwdParams& p, cudaStream_t stream) {
  if (p.B == 0 || p.H == 0 || p.Tq == 0 || p.Tk == 0) return ALG_OK;
  if (!p.force_mma && attn_bwd_tcgen05_supports(p)) return launch_attn_bwd_tcgen05(p, stream);
  if (p.dsink != nullptr) ALG_CUDA_TRY(cudaMemsetAsync(p.dsink, 0, sizeof(float) * p.H, stream));
  if (p.D == 64) return launch_d<64>(p, stream);
  if (p.D == 128) return launch_d<128>(p, stream);
  set_error("attention backward needs head_dim 64 or 128, got %d", p.D);
  return ALG_ERR_UNSUPPORTED;
}

}  // namespace alg
