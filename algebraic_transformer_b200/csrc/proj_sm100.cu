// The two wide projections of a prefill block as tcgen05 GEMMs whose consumers run in the
// epilogue, on the accumulator tile while it is still in tensor memory:
//
//   QKV  y = x . W_qkv^T, then per head: round to bf16, RMS-normalise q and k over the head
//        (fp32, gain, one rounding), Cayley rotate-half in bf16 arithmetic, and the range
//        guard's maxima (largest |q_scaled|^2, |k|^2, |v|) — reference: the q/k/v lines of
//        src/algebraic/model.py:165-174 with algebraic.py:76-83 (rms_norm), :172-179
//        (apply_rotary) and kernels/flash.py:831-849 (guard).  The stand-alone kernels for
//        these steps (qk_prep.cu) never run; the un-normalised projections never reach HBM.
//   GLU  [gate | up] = x . W_gu^T, then out = gate * ALU(up) — src/algebraic/model.py:184-193
//        with algebraic.py's alu.  The weight rows are interleaved in blocks of 128 (gate
//        block j, up block j, ...) so that one 256-wide accumulator tile holds both operands of
//        128 output features; gate and up never reach HBM.
//
// The main loop is the persistent, warp-specialised GEMM of head_sm100.cu: warp 0 (one lane)
// feeds a 4-stage shared-memory ring with TMA (128x64 activation tiles, 256x64 weight tiles,
// 128-byte swizzle), warp 1 (one lane) issues tcgen05.mma 128x256x16 into one of two 256-column
// TMEM accumulators, warps 2..9 drain the finished accumulator (thread = row) while the other
// one fills.  Every wait is bounded; a wait that runs out sets ALG_DEV_TIMEOUT.
#include <cuda_bf16.h>

#include "common.cuh"
#include "launchers.h"
#include "sm100_ptx.cuh"

namespace alg {
namespace {

using namespace sm100;

constexpr int BM = 128, BN = 256, BK = 64, STAGES = 4, UMMA_K = 16;
constexpr int A_BYTES = BM * BK * 2, B_BYTES = BN * BK * 2, STAGE_BYTES = A_BYTES + B_BYTES;
constexpr int NTHREADS = 320, EPI_THREADS = 256;
constexpr uint32_t TMEM_COLS = 512;
constexpr uint32_t IDESC = make_idesc_bf16(BM, BN, 0, 0);

struct __align__(16) Control {
  uint64_t full[STAGES], empty[STAGES], tfull[2], tempty[2];
  uint32_t tmem_base;
  int abort_flag;
};
constexpr size_t SMEM_BYTES = size_t(STAGES) * STAGE_BYTES + sizeof(Control) + 1024;

enum { EPI_QKV = 0, EPI_GLU = 1 };

__device__ __forceinline__ float bf16r(float x) { return __bfloat162float(__float2bfloat16_rn(x)); }
__device__ __forceinline__ __nv_bfloat162 as_bf162(uint32_t u) { return *reinterpret_cast<__nv_bfloat162*>(&u); }
__device__ __forceinline__ uint32_t as_u32(__nv_bfloat162 h) { return *reinterpret_cast<uint32_t*>(&h); }

// ---- QKV epilogue: one head (D columns starting at TMEM column `tcol`) of one row ---------
// kind 0 = q, 1 = k (normalise, rotate, statistic), 2 = v (round, statistic).
template <int D>
__device__ __forceinline__ void qkv_head(const ProjParams& p, const float* s_gain, uint32_t taddr, int kind, int t,
                                         __nv_bfloat16* dst, bool store, float& best_q, float& best_k, float& best_v) {
  constexpr int HALF = D / 2;
  if (kind == 2) {
#pragma unroll 1
    for (int c = 0; c < D / 32; ++c) {
      uint32_t r[32];
      tmem_ld_32x32(taddr + c * 32, r);
      tmem_ld_wait();
      uint32_t pk[16];
      float m = 0.f;
#pragma unroll
      for (int i = 0; i < 16; ++i) {
        pk[i] = pack_bf16(__uint_as_float(r[2 * i]), __uint_as_float(r[2 * i + 1]));
        m = fmaxf(m, fmaxf(fabsf(__uint_as_float(pk[i] << 16)), fabsf(__uint_as_float(pk[i] & 0xffff0000u))));
      }
      if (store) {
        best_v = fmaxf(best_v, m);
#pragma unroll
        for (int i = 0; i < 4; ++i)
          *reinterpret_cast<uint4*>(dst + c * 32 + i * 8) = make_uint4(pk[4 * i], pk[4 * i + 1], pk[4 * i + 2], pk[4 * i + 3]);
      }
    }
    return;
  }
  // pass 1: mean square of the bf16-rounded projection (the GEMM's output dtype)
  float ss = 0.f;
#pragma unroll 1
  for (int c = 0; c < D / 32; ++c) {
    uint32_t r[32];
    tmem_ld_32x32(taddr + c * 32, r);
    tmem_ld_wait();
#pragma unroll
    for (int i = 0; i < 32; ++i) {
      const float v = bf16r(__uint_as_float(r[i]));
      ss = fmaf(v, v, ss);
    }
  }
  const float tau = rsqrtf(ss * (1.0f / D) + p.eps);
  const float* gain = s_gain + kind * 128;           // shared-memory copy: q gains, then k gains
  const float stat_scale = (kind == 0) ? p.q_scale : 1.0f;
  float stat = 0.f;
  // pass 2: 32 elements of the first half with their rotate-half partners of the second half
#pragma unroll 1
  for (int c = 0; c < HALF / 32; ++c) {
    uint32_t r1[32], r2[32];
    tmem_ld_32x32(taddr + c * 32, r1);
    tmem_ld_32x32(taddr + HALF + c * 32, r2);
    tmem_ld_wait();
    uint32_t o1[16], o2[16];
    const uint4* ct = reinterpret_cast<const uint4*>(p.cos + int64_t(t) * HALF + c * 32);
    const uint4* st = reinterpret_cast<const uint4*>(p.sin + int64_t(t) * HALF + c * 32);
#pragma unroll
    for (int q4 = 0; q4 < 4; ++q4) {
      const uint4 cv = ct[q4], sv = st[q4];
      const uint32_t cw[4] = {cv.x, cv.y, cv.z, cv.w}, sw[4] = {sv.x, sv.y, sv.z, sv.w};
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const int i = q4 * 8 + j * 2;              // element index inside the 32-chunk
        const float2 g1 = *reinterpret_cast<const float2*>(gain + c * 32 + i);
        const float2 g2 = *reinterpret_cast<const float2*>(gain + HALF + c * 32 + i);
        const float g1a = g1.x, g1b = g1.y, g2a = g2.x, g2b = g2.y;
        // x <- round((round(acc) * tau) * gain)
        const uint32_t x1 = pack_bf16((bf16r(__uint_as_float(r1[i])) * tau) * g1a, (bf16r(__uint_as_float(r1[i + 1])) * tau) * g1b);
        const uint32_t x2 = pack_bf16((bf16r(__uint_as_float(r2[i])) * tau) * g2a, (bf16r(__uint_as_float(r2[i + 1])) * tau) * g2b);
        const __nv_bfloat162 X1 = as_bf162(x1), X2 = as_bf162(x2), Cc = as_bf162(cw[j]), Ss = as_bf162(sw[j]);
        // bf16 arithmetic, every product and sum rounded: (x1 c - x2 s, x1 s + x2 c)
        const __nv_bfloat162 y1 = __hsub2(__hmul2(X1, Cc), __hmul2(X2, Ss));
        const __nv_bfloat162 y2 = __hadd2(__hmul2(X1, Ss), __hmul2(X2, Cc));
        o1[q4 * 4 + j] = as_u32(y1);
        o2[q4 * 4 + j] = as_u32(y2);
        const float2 f1 = __bfloat1622float2(y1), f2 = __bfloat1622float2(y2);
        const float a = bf16r(f1.x * stat_scale), b = bf16r(f1.y * stat_scale);
        const float cc = bf16r(f2.x * stat_scale), d = bf16r(f2.y * stat_scale);
        stat = fmaf(a, a, stat); stat = fmaf(b, b, stat); stat = fmaf(cc, cc, stat); stat = fmaf(d, d, stat);
      }
    }
    if (store) {
#pragma unroll
      for (int i = 0; i < 4; ++i) {
        *reinterpret_cast<uint4*>(dst + c * 32 + i * 8) = make_uint4(o1[4 * i], o1[4 * i + 1], o1[4 * i + 2], o1[4 * i + 3]);
        *reinterpret_cast<uint4*>(dst + HALF + c * 32 + i * 8) = make_uint4(o2[4 * i], o2[4 * i + 1], o2[4 * i + 2], o2[4 * i + 3]);
      }
    }
  }
  if (store) {
    if (kind == 0) best_q = fmaxf(best_q, stat); else best_k = fmaxf(best_k, stat);
  }
}

// ---- GLU epilogue: 64 output features of one row -------------------------------------------
__device__ __forceinline__ void glu_cols(const ProjParams& p, uint32_t t_gate, uint32_t t_up, __nv_bfloat16* dst, bool store) {
#pragma unroll 1
  for (int c = 0; c < 2; ++c) {
    uint32_t g[32], u[32];
    tmem_ld_32x32(t_gate + c * 32, g);
    tmem_ld_32x32(t_up + c * 32, u);
    tmem_ld_wait();
    uint32_t pk[16];
#pragma unroll
    for (int i = 0; i < 32; i += 2) {
      float o[2];
#pragma unroll
      for (int e = 0; e < 2; ++e) {
        const float gv = bf16r(__uint_as_float(g[i + e])), uv = bf16r(__uint_as_float(u[i + e]));
        const float bz = p.beta * uv;
        const float r = rsqrtf(fmaf(bz, bz, 1.0f));
        const float uu = bz * r;
        // for bz < 0 use 1 + u = r^2 / (1 - u) so that the negative tail survives
        const float one_plus_u = bz < 0.f ? __fdividef(r * r, 1.0f - uu) : 1.0f + uu;
        o[e] = gv * bf16r(0.5f * uv * one_plus_u);
      }
      pk[i >> 1] = pack_bf16(o[0], o[1]);
    }
    if (store) {
#pragma unroll
      for (int i = 0; i < 4; ++i)
        *reinterpret_cast<uint4*>(dst + c * 32 + i * 8) = make_uint4(pk[4 * i], pk[4 * i + 1], pk[4 * i + 2], pk[4 * i + 3]);
    }
  }
}

template <int EPI, int D>
__global__ void __launch_bounds__(NTHREADS, 1)
proj_tc_kernel(const __grid_constant__ CUtensorMap tm_x, const __grid_constant__ CUtensorMap tm_w, const ProjParams p) {
  extern __shared__ unsigned char smem_raw[];
  unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  Control* ctl = reinterpret_cast<Control*>(smem + size_t(STAGES) * STAGE_BYTES);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  __shared__ __align__(16) float s_gain[2 * 128];      // QKV epilogue: q gains [0,128), k gains [128,256)
  if (EPI == EPI_QKV && threadIdx.x < 2 * D) {
    const float* g = (threadIdx.x < D) ? p.q_gain : p.k_gain;
    s_gain[(threadIdx.x / D) * 128 + threadIdx.x % D] = (g != nullptr) ? g[threadIdx.x % D] : 1.0f;
  }

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) { mbar_init(&ctl->full[s], 1); mbar_init(&ctl->empty[s], 1); }
    for (int b = 0; b < 2; ++b) { mbar_init(&ctl->tfull[b], 1); mbar_init(&ctl->tempty[b], EPI_THREADS); }
    ctl->abort_flag = 0;
    fence_barrier_init();
  }
  if (warp == 1) {
    tmem_alloc(&ctl->tmem_base, TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = ctl->tmem_base;
  const BoundedWait bw{&ctl->abort_flag, 1000000000ull};
  const int tiles_n = (p.N + BN - 1) / BN;
  const int tiles = ((p.M + BM - 1) / BM) * tiles_n;
  const int kblocks = p.K / BK;

  if (warp == 0) {
    if (lane == 0) {
      tma_prefetch_desc(&tm_x);
      tma_prefetch_desc(&tm_w);
      uint32_t stage = 0, phase = 0;
      bool ok = true;
      for (int u = blockIdx.x; u < tiles && ok; u += gridDim.x) {
        const int m = u / tiles_n, n = u % tiles_n;
        for (int kb = 0; kb < kblocks; ++kb) {
          if (!bw.wait(&ctl->empty[stage], phase ^ 1u)) { ok = false; break; }
          unsigned char* dst = smem + size_t(stage) * STAGE_BYTES;
          mbar_arrive_expect_tx(&ctl->full[stage], STAGE_BYTES);
          tma_load_2d(dst, &tm_x, &ctl->full[stage], kb * BK, m * BM);
          tma_load_2d(dst + A_BYTES, &tm_w, &ctl->full[stage], kb * BK, n * BN);
          if (++stage == STAGES) { stage = 0; phase ^= 1u; }
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      uint32_t stage = 0, phase = 0, tile_count = 0;
      const uint32_t a_lo0 = sw128_desc_lo(smem_u32(smem), 16), b_lo0 = sw128_desc_lo(smem_u32(smem) + A_BYTES, 16);
      bool ok = true;
      for (int u = blockIdx.x; u < tiles && ok; u += gridDim.x, ++tile_count) {
        const uint32_t buf = tile_count & 1u, tphase = (tile_count >> 1) & 1u;
        if (!bw.wait(&ctl->tempty[buf], tphase ^ 1u)) { ok = false; break; }
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + buf * BN;
        for (int kb = 0; kb < kblocks; ++kb) {
          if (!bw.wait(&ctl->full[stage], phase)) { ok = false; break; }
          tc_fence_after();
          const uint32_t a_lo = a_lo0 + stage * (STAGE_BYTES >> 4), b_lo = b_lo0 + stage * (STAGE_BYTES >> 4);
#pragma unroll
          for (int k = 0; k < BK / UMMA_K; ++k)
            umma_f16_ss_parts(d_tmem, a_lo + k * (UMMA_K * 2 >> 4), SW128_DESC_HI, b_lo + k * (UMMA_K * 2 >> 4),
                              SW128_DESC_HI, IDESC, (kb | k) != 0 ? 1u : 0u);
          umma_commit(&ctl->empty[stage]);             // smem stage is free once these MMAs retire
          if (++stage == STAGES) { stage = 0; phase ^= 1u; }
        }
        if (ok) umma_commit(&ctl->tfull[buf]);          // accumulator tile complete
      }
    }
  } else {
    const int quarter = warp & 3;                        // TMEM lanes 32*quarter .. +31 belong to this warp
    const int half = (warp - 2) >> 2;
    const int row_in_tile = quarter * 32 + lane;
    const uint32_t lane_sel = uint32_t(quarter * 32) << 16;
    uint32_t tile_count = 0;
    float best_q = 0.f, best_k = 0.f, best_v = 0.f;
    bool ok = true;
    for (int u = blockIdx.x; u < tiles && ok; u += gridDim.x, ++tile_count) {
      const int m = u / tiles_n, n = u % tiles_n;
      const uint32_t buf = tile_count & 1u, tphase = (tile_count >> 1) & 1u;
      if (!bw.wait(&ctl->tfull[buf], tphase)) { ok = false; break; }
      tc_fence_after();
      const int row = m * BM + row_in_tile;
      const bool live = row < p.M;
      const uint32_t tbuf = tmem_base + lane_sel + buf * BN;
      if (EPI == EPI_QKV) {
        const int t = live ? row % p.T : 0;
        const int hd = p.H * D;
#pragma unroll 1
        for (int hh = 0; hh < 128 / D; ++hh) {
          const int lcol = half * 128 + hh * D;          // column inside the tile
          const int gcol = n * BN + lcol;                // output feature
          if (gcol >= p.N) break;
          qkv_head<D>(p, s_gain, tbuf + lcol, gcol / hd, t, p.out + int64_t(live ? row : 0) * p.ld_out + gcol, live, best_q, best_k,
                      best_v);
        }
      } else {
        const int fcol = n * 128 + half * 64;            // output feature of this thread's first column
        if (fcol < p.f)
          glu_cols(p, tbuf + half * 64, tbuf + 128 + half * 64, p.out + int64_t(live ? row : 0) * p.ld_out + fcol, live);
      }
      tc_fence_before();
      mbar_arrive(&ctl->tempty[buf]);                    // this thread is done reading the buffer
    }
    if (EPI == EPI_QKV && p.guard != nullptr) {          // one atomic per warp and statistic
      float m[3] = {warp_max(best_q), warp_max(best_k), warp_max(best_v)};
      unsigned* out[3] = {&p.guard->q2, &p.guard->k2, &p.guard->vmax};
#pragma unroll
      for (int i = 0; i < 3; ++i) {
        if (!(m[i] == m[i])) m[i] = __int_as_float(0x7f800000);   // NaN must fail the guard
        if (lane == 0 && m[i] != 0.f) atomicMax(out[i], __float_as_uint(m[i]));
      }
    }
  }

  tc_fence_before();
  __syncthreads();
  if (ctl->abort_flag != 0) {
    if (threadIdx.x == 0) {
      if (p.status != nullptr) atomicExch(p.status, ALG_DEV_TIMEOUT);
      const uint64_t t0 = global_timer_ns();           // let issued loads land before shared memory is released
      while (global_timer_ns() - t0 < 200000ull) { }
    }
    __syncthreads();
  }
  if (warp == 1) {
    __syncwarp();
    tc_fence_after();
    tmem_dealloc(tmem_base, TMEM_COLS);
  }
}

template <int EPI, int D>
int launch_variant(const CUtensorMap& tm_x, const CUtensorMap& tm_w, const ProjParams& p, int grid, cudaStream_t stream) {
  auto kern = proj_tc_kernel<EPI, D>;
  static bool configured = false;
  if (!configured) {
    ALG_CUDA_TRY(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, int(SMEM_BYTES)));
    configured = true;
  }
  kern<<<grid, NTHREADS, SMEM_BYTES, stream>>>(tm_x, tm_w, p);
  ALG_CUDA_TRY(cudaGetLastError());
  count_launch();
  return ALG_OK;
}

}  // namespace

int launch_proj(const ProjParams& p, const void* x, const void* w, int epi, cudaStream_t stream) {
  if (p.M == 0) return ALG_OK;
  CUtensorMap tm_x, tm_w;
  {
    const uint64_t dims[2] = {uint64_t(p.K), uint64_t(p.M)};
    const uint64_t strides[1] = {uint64_t(p.ld_x)};
    const uint32_t box[2] = {BK, BM};
    if (int rc = make_tmap_bf16(&tm_x, x, 2, dims, strides, box, true)) return rc;
  }
  {
    const uint64_t dims[2] = {uint64_t(p.K), uint64_t(p.N)};
    const uint64_t strides[1] = {uint64_t(p.K)};
    const uint32_t box[2] = {BK, BN};
    if (int rc = make_tmap_bf16(&tm_w, w, 2, dims, strides, box, true)) return rc;
  }
  int dev = 0, sms = 148;
  ALG_CUDA_TRY(cudaGetDevice(&dev));
  ALG_CUDA_TRY(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev));
  const int tiles = ((p.M + BM - 1) / BM) * ((p.N + BN - 1) / BN);
  const int grid = tiles < sms ? tiles : sms;
  if (epi == 1) return launch_variant<EPI_GLU, 64>(tm_x, tm_w, p, grid, stream);
  return p.D == 64 ? launch_variant<EPI_QKV, 64>(tm_x, tm_w, p, grid, stream)
                   : launch_variant<EPI_QKV, 128>(tm_x, tm_w, p, grid, stream);
}

}  // namespace alg
