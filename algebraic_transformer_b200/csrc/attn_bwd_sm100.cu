// Asinh-power attention backward on tcgen05 tensor cores (the throughput path of alg_attn_bwd).
//
// Same mathematics as attn_bwd_mma.cu (reference: the custom VJP of
// src/algebraic/kernels/flash.py:333-727): with x = q.k / (sqrt(D) c), p rebuilt from the saved
// statistic, delta_i = dO_i . o_i and dP = dO V^T,
//   dS = n p (dP - delta) / sqrt(1 + x^2) / (sqrt(D) c),  dQ = dS K,  dK = dS^T Q,  dV = P^T dO.
// bf16, causal, Tq == Tk a multiple of 128, head_dim 64 or 128; everything else stays on the
// mma.sync kernels.
//
// One kernel template, two modes, one CTA per 128-row tile of one (batch, head):
//   MODE 0 (dQ, dsink)  rows = queries.  Resident: Q, dO tiles.  Streamed: K_j, V_j for every key
//                       tile up to the diagonal.  S = Q K_j^T, dP = dO V_j^T, dQ += dS K_j.
//   MODE 1 (dK, dV)     rows = keys.  Resident: K, V tiles.  Streamed: Q_i, dO_i for every query
//                       tile from the diagonal on.  S^T = K Q_i^T, dP^T = V dO_i^T,
//                       dV += P^T dO_i, dK += dS^T Q_i.
// Roles: warp 0 (one lane) TMA producer, warp 1 (one lane) tcgen05.mma issuer, warps 2..9 the
// element-wise stage (thread = row, two column halves of 64).  Tensor memory: the two score
// tiles (128 columns each) and one or two D-column accumulators; the bf16 operands of the second
// products (P^T, dS) are written back over the columns their own thread has already read — half
// h keeps its 64 packed values in columns [64 h, 64 h + 32) — and fed to the tensor core from
// tensor memory (TS form) with the streamed tile as an MN-major B operand, so nothing is
// transposed or staged.  With both accumulators of MODE 1 all 512 columns are taken, so the two
// score tiles cannot be double-buffered; instead a step has two element-wise phases and the
// tensor core works on one region while the threads work on the other:
//   phase 1  reads S, forms p (MODE 1 writes P^T over S) and keeps n p / sqrt(1+x^2) in registers;
//            meanwhile: dK/dQ product of the previous step, then dP of this step;
//   phase 2  reads dP, writes dS = (kept factor) (dP - delta) over it;
//            meanwhile: dV product of this step (MODE 1), then S of the next step.
// Every mbarrier wait is bounded; a wait that runs out reports ALG_DEV_TIMEOUT.
#include "common.cuh"
#include "launchers.h"
#include "sm100_ptx.cuh"

namespace alg {
namespace {

using namespace sm100;

constexpr int BT = 128, NTHREADS = 320, EW_THREADS = 256;
constexpr int PANEL_BYTES = 128 * 128;
constexpr uint32_t TMEM_COLS = 512;
constexpr int MAX_STEPS = 4;

template <int D> struct Cfg {
  static constexpr int PANELS = D / 64;
  static constexpr int TILE_BYTES = PANELS * PANEL_BYTES;
  static constexpr int NS = (D == 128) ? 2 : 4;                 // ring depth in steps (two tiles per step)
  static constexpr int RES_OFF = 0;
  static constexpr int RING_OFF = 2 * TILE_BYTES;
  static constexpr int CTL_OFF = RING_OFF + NS * 2 * TILE_BYTES;
  static constexpr uint32_t S_COL = 0, DP_COL = 128, ACC0_COL = 256, ACC1_COL = 256 + D;
  static constexpr uint32_t S1_COL = 384;   // second score buffer, where the accumulators leave room for it
  static constexpr uint32_t IDESC_S = make_idesc_bf16(BT, BT, 0, 0);
  static constexpr uint32_t IDESC_TS = make_idesc_bf16(BT, D, 0, 1);
};

struct __align__(16) Control {
  uint64_t res_full, full[MAX_STEPS], empty[MAX_STEPS], s_full[2], dp_full, p_done[2], ds_done, acc_full;
  uint32_t tmem_base;
  int abort_flag;
  float sink_part[8];
};

template <int D> constexpr size_t smem_bytes() { return size_t(Cfg<D>::CTL_OFF) + sizeof(Control) + 1024; }

// Phase 1 on 32 scores of this thread's row: the weights p, packed to bf16 in pw_out, and the factor
// p / sqrt(1 + x^2) that phase 2 multiplies (dP - delta) by, in `slope`.  `stat` comes by
// row (MODE 0: one value) or by column (MODE 1: 32 values).  Pairs of values go through the packed
// fp32 instructions (mul.f32x2 / fma.f32x2).  The 2^log2n-th power runs as log2n passes over the 16
// pairs, so that every pass has independent multiplications whatever n is (a loop per element
// serialises on its own latency).
template <bool SHIFTED, bool BY_COLUMN>
__device__ __forceinline__ void weights_from_scores(const uint32_t* s, float2* slope, const AttnBwdParams& p,
                                                    float stat_row, const float2* stat_col, int log2n, bool diag, int row,
                                                    int col0, bool row_is_query, uint32_t* pw_out) {
  // Two factors that are constant over a row of the accumulator are left to the kernel's epilogue instead
  // of being multiplied into every score: n / (sqrt(D) c) always, and the row's statistic when it is a
  // plain factor of the weight (rows = queries, unshifted forward).  What is written to tensor memory is
  // then an unnormalised dS, as the forward's P is unnormalised.
  const float2 sc = make_float2(p.scale, p.scale), one = make_float2(1.f, 1.f);
  const float2 st_row = make_float2(stat_row, stat_row);
  float2 t[16];
#pragma unroll
  for (int i = 0; i < 16; ++i) {
    const float2 x = __fmul2_rn(make_float2(__uint_as_float(s[2 * i]), __uint_as_float(s[2 * i + 1])), sc);
    const float2 rad = __ffma2_rn(x, x, one);
    const float2 rs = make_float2(rsqrt_approx(rad.x), rsqrt_approx(rad.y));
    if (SHIFTED) {
      const float2 st = BY_COLUMN ? stat_col[i] : st_row;
      t[i] = make_float2(rho_stable(x.x) * st.x, rho_stable(x.y) * st.y);
    } else {
      t[i] = __ffma2_rn(rad, rs, x);
    }
    slope[i] = rs;
  }
  for (int it = 0; it < log2n; ++it) {
#pragma unroll
    for (int i = 0; i < 16; ++i) t[i] = __fmul2_rn(t[i], t[i]);
  }
  if (!SHIFTED && BY_COLUMN) {
#pragma unroll
    for (int i = 0; i < 16; ++i) t[i] = __fmul2_rn(t[i], stat_col[i]);
  }
  if (diag) {   // causal: key <= query.  Rows are queries in MODE 0 (mask col > row), keys in MODE 1 (mask col < row)
#pragma unroll
    for (int i = 0; i < 16; ++i) {
      const int c = col0 + 2 * i;
      if (row_is_query ? (c > row) : (c < row)) t[i].x = 0.f;
      if (row_is_query ? (c + 1 > row) : (c + 1 < row)) t[i].y = 0.f;
    }
  }
#pragma unroll
  for (int i = 0; i < 16; ++i) {
    slope[i] = __fmul2_rn(slope[i], t[i]);
    pw_out[i] = pack_bf16(t[i].x, t[i].y);
  }
}

template <int D, int MODE>
__global__ void __launch_bounds__(NTHREADS, 1)
attn_bwd_tc_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_k,
                   const __grid_constant__ CUtensorMap tm_v, const __grid_constant__ CUtensorMap tm_do,
                   const AttnBwdParams p) {
  using C = Cfg<D>;
  extern __shared__ unsigned char smem_raw[];
  unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  Control* ctl = reinterpret_cast<Control*>(smem + C::CTL_OFF);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    mbar_init(&ctl->res_full, 1);
    for (int i = 0; i < C::NS; ++i) { mbar_init(&ctl->full[i], 1); mbar_init(&ctl->empty[i], 1); }
    mbar_init(&ctl->s_full[0], 1);
    mbar_init(&ctl->s_full[1], 1);
    mbar_init(&ctl->dp_full, 1);
    mbar_init(&ctl->p_done[0], EW_THREADS);
    mbar_init(&ctl->p_done[1], EW_THREADS);
    mbar_init(&ctl->ds_done, EW_THREADS);
    mbar_init(&ctl->acc_full, 1);
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
  // Two score buffers where tensor memory has 128 columns to spare (one accumulator, or two of 64 columns):
  // S of step j + 1 is then computed while the threads are still reading S of step j.
  constexpr bool DB = (MODE == 0) || (D == 64);
  auto sbuf = [](int j) { return DB ? (j & 1) : 0; };
  auto sphase = [](int j) -> uint32_t { return DB ? ((j >> 1) & 1u) : (j & 1u); };
  auto s_col = [](int j) -> uint32_t { return (DB && (j & 1)) ? C::S1_COL : C::S_COL; };

  const int nt = p.Tq / BT;
  const int h = blockIdx.x, b = blockIdx.y;
  // heavy tiles first, over all heads: late query tiles see many keys, early key tiles are seen by many queries
  const int tile = (MODE == 0) ? nt - 1 - int(blockIdx.z) : int(blockIdx.z);
  const int row0 = tile * BT;
  const int first = (MODE == 0) ? 0 : tile;                  // streamed tiles first .. last, diagonal = `tile`
  const int last = (MODE == 0) ? tile : nt - 1;
  const int nsteps = last - first + 1;
  const bool shifted = *p.stat_kind == ALG_VARIANT_SHIFT;

  if (warp == 0) {
    if (lane == 0) {
      tma_prefetch_desc(&tm_q); tma_prefetch_desc(&tm_k); tma_prefetch_desc(&tm_v); tma_prefetch_desc(&tm_do);
      const CUtensorMap* res0 = (MODE == 0) ? &tm_q : &tm_k;   // A operand of the first score product
      const CUtensorMap* res1 = (MODE == 0) ? &tm_do : &tm_v;  // A operand of the second
      const CUtensorMap* str0 = (MODE == 0) ? &tm_k : &tm_q;   // their streamed B operands
      const CUtensorMap* str1 = (MODE == 0) ? &tm_v : &tm_do;
      mbar_arrive_expect_tx(&ctl->res_full, 2 * C::TILE_BYTES);
      for (int pn = 0; pn < C::PANELS; ++pn) {
        tma_load_4d(smem + C::RES_OFF + pn * PANEL_BYTES, res0, &ctl->res_full, pn * 64, row0, h, b);
        tma_load_4d(smem + C::RES_OFF + C::TILE_BYTES + pn * PANEL_BYTES, res1, &ctl->res_full, pn * 64, row0, h, b);
      }
      for (int j = 0; j < nsteps; ++j) {
        const int slot = j % C::NS;
        if (!bw.wait(&ctl->empty[slot], ((j / C::NS) & 1u) ^ 1u)) break;
        unsigned char* dst = smem + C::RING_OFF + slot * 2 * C::TILE_BYTES;
        mbar_arrive_expect_tx(&ctl->full[slot], 2 * C::TILE_BYTES);
        for (int pn = 0; pn < C::PANELS; ++pn) {
          tma_load_4d(dst + pn * PANEL_BYTES, str0, &ctl->full[slot], pn * 64, (first + j) * BT, h, b);
          tma_load_4d(dst + C::TILE_BYTES + pn * PANEL_BYTES, str1, &ctl->full[slot], pn * 64, (first + j) * BT, h, b);
        }
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      const uint32_t res_addr = smem_u32(smem + C::RES_OFF), ring_addr = smem_u32(smem + C::RING_OFF);
      const uint32_t a0_lo = sw128_desc_lo(res_addr, 16), a1_lo = sw128_desc_lo(res_addr + C::TILE_BYTES, 16);
      // S-like product: d = A . B^T, both K-major tiles of D columns
      auto issue_scores = [&](uint32_t d_tmem, uint32_t a_lo, uint32_t b_addr) {
        const uint32_t b_lo = sw128_desc_lo(b_addr, 16);
#pragma unroll
        for (int ks = 0; ks < D / 16; ++ks) {
          const uint32_t off = ((ks >> 2) * PANEL_BYTES + (ks & 3) * 32) >> 4;
          umma_f16_ss_parts(d_tmem, a_lo + off, SW128_DESC_HI, b_lo + off, SW128_DESC_HI, C::IDESC_S, ks != 0 ? 1u : 0u);
        }
      };
      // acc += W . B: W = packed bf16 in tensor memory (64 values per column half, see the header), B = a
      // streamed [row][D] tile read as an MN-major operand
      auto issue_product = [&](uint32_t d_tmem, uint32_t w_tmem, uint32_t b_addr, bool first_step) {
        const uint32_t b_lo = sw128_desc_lo(b_addr, PANEL_BYTES);
#pragma unroll
        for (int ks = 0; ks < BT / 16; ++ks) {
          const uint32_t a_col = (ks < 4) ? ks * 8 : 64 + (ks - 4) * 8;
          umma_f16_ts_parts(d_tmem, w_tmem + a_col, b_lo + ks * (2048 >> 4), SW128_DESC_HI, C::IDESC_TS,
                            (first_step && ks == 0) ? 0u : 1u);
        }
      };
      // S of step j goes to buffer sbuf(j); with two buffers (DB) it is issued one step earlier
      auto tile0 = [&](int j) { return ring_addr + (j % C::NS) * 2 * C::TILE_BYTES; };
      auto score_s = [&](int j) -> bool {               // waits for step j's tiles, then S (or S^T) of step j
        if (!bw.wait(&ctl->full[j % C::NS], (j / C::NS) & 1u)) return false;
        tc_fence_after();
        issue_scores(tmem_base + s_col(j), a0_lo, tile0(j));
        umma_commit(&ctl->s_full[sbuf(j)]);
        return true;
      };
      bool ok = bw.wait(&ctl->res_full, 0) && score_s(0);
      if (ok) {
        issue_scores(tmem_base + C::DP_COL, a1_lo, tile0(0) + C::TILE_BYTES);      // dP (or dP^T) of step 0
        umma_commit(&ctl->dp_full);
        if (DB && nsteps > 1) ok = score_s(1);
      }
      for (int j = 0; j < nsteps && ok; ++j) {
        const bool has_next = j + 1 < nsteps;
        const uint32_t t0 = tile0(j), t1 = t0 + C::TILE_BYTES;
        // phase 1 is over: S has been read (MODE 1: P^T stands in its place)
        if (!bw.wait(&ctl->p_done[sbuf(j)], sphase(j))) { ok = false; break; }
        tc_fence_after();
        if (MODE == 1) issue_product(tmem_base + C::ACC0_COL, tmem_base + s_col(j), t1, j == 0);   // dV += P^T dO_i
        if (!DB && has_next && !score_s(j + 1)) { ok = false; break; }   // after the dV product: may overwrite P^T
        // phase 2 is over: dS stands in place of dP
        if (!bw.wait(&ctl->ds_done, j & 1u)) { ok = false; break; }
        tc_fence_after();
        issue_product(tmem_base + (MODE == 0 ? C::ACC0_COL : C::ACC1_COL), tmem_base + C::DP_COL, t0, j == 0);  // dQ += dS K_j / dK += dS^T Q_i
        umma_commit(&ctl->empty[j % C::NS]);
        if (has_next) {
          issue_scores(tmem_base + C::DP_COL, a1_lo, tile0(j + 1) + C::TILE_BYTES);   // after that product: may overwrite dS
          umma_commit(&ctl->dp_full);
        }
        if (DB && j + 2 < nsteps && !score_s(j + 2)) { ok = false; break; }   // into the buffer phase 1 of step j has left
      }
      if (ok) umma_commit(&ctl->acc_full);
    }
  } else {
    const int quarter = warp & 3, half = (warp - 2) >> 2;
    const int r = quarter * 32 + lane;                        // row inside the tile
    const int row = row0 + r;
    const uint32_t lane_sel = uint32_t(quarter * 32) << 16;
    const int64_t bh = int64_t(b) * p.H + h;
    float stat_row = 0.f, delta_row = 0.f;
    if (MODE == 0) { stat_row = p.stat[bh * p.Tq + row]; delta_row = p.delta[bh * p.Tq + row]; }
    const uint32_t dp_t = tmem_base + lane_sel + C::DP_COL + half * 64;
    bool ok = true;
    for (int j = 0; j < nsteps && ok; ++j) {
      const int other0 = (first + j) * BT;                    // first row of the streamed tile
      const bool diag = (first + j) == tile;
      const float* col_stat = p.stat + bh * p.Tq + other0 + half * 64;     // MODE 1: of the streamed queries
      const float* col_delta = p.delta + bh * p.Tq + other0 + half * 64;
      float2 slope[2][16];
      // ---- phase 1: scores -> weights
      const uint32_t s_t = tmem_base + lane_sel + s_col(j) + half * 64;
      if (!bw.wait(&ctl->s_full[sbuf(j)], sphase(j))) { ok = false; break; }
      tc_fence_after();
#pragma unroll
      for (int c = 0; c < 2; ++c) {
        uint32_t s[32], pw[16];
        tmem_ld_32x32(s_t + c * 32, s);
        float2 stc[16];
        if (MODE == 1) {
#pragma unroll
          for (int i = 0; i < 8; ++i) {
            const float4 a = __ldg(reinterpret_cast<const float4*>(col_stat + c * 32) + i);
            stc[2 * i] = make_float2(a.x, a.y);
            stc[2 * i + 1] = make_float2(a.z, a.w);
          }
        }
        tmem_ld_wait();
        const int col0 = half * 64 + c * 32;                   // column inside the streamed tile
        if (shifted) weights_from_scores<true, MODE == 1>(s, slope[c], p, stat_row, stc, p.log2n, diag, r, col0, MODE == 0, pw);
        else weights_from_scores<false, MODE == 1>(s, slope[c], p, stat_row, stc, p.log2n, diag, r, col0, MODE == 0, pw);
        // packed output over columns this thread has read already: chunk c -> [64 half + 16 c, +16)
        if (MODE == 1) tmem_st_32x16(s_t + c * 16, pw);
      }
      if (MODE == 1) tmem_st_wait();
      tc_fence_before();
      mbar_arrive(&ctl->p_done[sbuf(j)]);
      // ---- phase 2: dP -> dS = slope (dP - delta)
      if (!bw.wait(&ctl->dp_full, j & 1u)) { ok = false; break; }
      tc_fence_after();
      {
        uint32_t dp0[32], dp1[32], ds[16];
        tmem_ld_32x32(dp_t, dp0);
        tmem_ld_32x32(dp_t + 32, dp1);
        const float2 minus_one = make_float2(-1.f, -1.f), dl_row = make_float2(delta_row, delta_row);
#pragma unroll
        for (int c = 0; c < 2; ++c) {
          float2 dlc[16];
          if (MODE == 1) {
#pragma unroll
            for (int i = 0; i < 8; ++i) {
              const float4 a = __ldg(reinterpret_cast<const float4*>(col_delta + c * 32) + i);
              dlc[2 * i] = make_float2(a.x, a.y);
              dlc[2 * i + 1] = make_float2(a.z, a.w);
            }
          }
          if (c == 0) tmem_ld_wait_for(dp0); else tmem_ld_wait_for(dp1);
          const uint32_t* dp = c == 0 ? dp0 : dp1;
#pragma unroll
          for (int i = 0; i < 16; ++i) {
            const float2 d = make_float2(__uint_as_float(dp[2 * i]), __uint_as_float(dp[2 * i + 1]));
            const float2 v = __fmul2_rn(slope[c][i], __ffma2_rn(MODE == 1 ? dlc[i] : dl_row, minus_one, d));
            ds[i] = pack_bf16(v.x, v.y);
          }
          tmem_st_32x16(dp_t + c * 16, ds);
        }
      }
      tmem_st_wait();
      tc_fence_before();
      mbar_arrive(&ctl->ds_done);
    }
    if (ok && bw.wait(&ctl->acc_full, 0)) {
      tc_fence_after();
      constexpr int CPT = D / 2;                               // accumulator columns per thread
      __nv_bfloat16* out0 = ((MODE == 0) ? p.dq + b * p.qs.b + h * p.qs.h + int64_t(row) * p.qs.t
                                         : p.dv + b * p.vs.b + h * p.vs.h + int64_t(row) * p.vs.t) + half * CPT;
      __nv_bfloat16* out1 = (MODE == 1) ? p.dk + b * p.ks.b + h * p.ks.h + int64_t(row) * p.ks.t + half * CPT : nullptr;
#pragma unroll 1
      for (int which = 0; which < (MODE == 0 ? 1 : 2); ++which) {
        const uint32_t acc_t = tmem_base + lane_sel + (which == 0 ? C::ACC0_COL : C::ACC1_COL) + half * CPT;
        __nv_bfloat16* dst = which == 0 ? out0 : out1;
        // the row factors phase 1 left out: n / (sqrt(D) c) on dQ and dK, and on dQ the row's statistic
        // where it is a plain factor of the weight (dV carries none)
        const float fac = (MODE == 0) ? (shifted ? p.n_scale : p.n_scale * stat_row) : (which == 1 ? p.n_scale : 1.0f);
#pragma unroll 1
        for (int c = 0; c < CPT / 32; ++c) {
          uint32_t a[32];
          tmem_ld_32x32(acc_t + c * 32, a);
          tmem_ld_wait();
#pragma unroll
          for (int i = 0; i < 32; ++i) a[i] = __float_as_uint(__uint_as_float(a[i]) * fac);
#pragma unroll
          for (int i = 0; i < 4; ++i)
            *reinterpret_cast<uint4*>(dst + c * 32 + i * 8) =
                make_uint4(pack_bf16(__uint_as_float(a[8 * i]), __uint_as_float(a[8 * i + 1])),
                           pack_bf16(__uint_as_float(a[8 * i + 2]), __uint_as_float(a[8 * i + 3])),
                           pack_bf16(__uint_as_float(a[8 * i + 4]), __uint_as_float(a[8 * i + 5])),
                           pack_bf16(__uint_as_float(a[8 * i + 6]), __uint_as_float(a[8 * i + 7])));
        }
      }
    }
    // dsink: -sum_i delta_i p_sink,i n / (c sqrt(1 + (b/c)^2)), one atomic per warp of the first column half
    if (MODE == 0 && p.sink != nullptr && p.dsink != nullptr && half == 0) {
      const float bs = p.sink[h] * p.inv_c;
      const float ps = shifted ? pow2n_rt(rho_stable(bs) * stat_row, p.log2n) : pow2n_rt(rho_stable(bs), p.log2n) * stat_row;
      float part = -delta_row * ps * p.n_f * p.inv_c * rsqrtf(fmaf(bs, bs, 1.0f));
      part = warp_sum(part);
      if (lane == 0) atomicAdd(p.dsink + h, part);
    }
  }

  tc_fence_before();
  __syncthreads();
  if (ctl->abort_flag != 0) {
    if (threadIdx.x == 0) {
      if (p.status != nullptr) atomicExch(p.status, ALG_DEV_TIMEOUT);
      const uint64_t t0 = global_timer_ns();                 // let issued loads land before shared memory is released
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

// delta_i = dO_i . o_i, one row per LPR lanes
template <int D>
__global__ void __launch_bounds__(256) attn_delta_kernel(const AttnBwdParams p) {
  constexpr int LPR = D / 8, RPW = 32 / LPR;
  const int lane = threadIdx.x & 31, lir = lane % LPR, sub = lane / LPR;
  const int64_t rows = int64_t(p.B) * p.H * p.Tq;
  const int64_t warp_global = (int64_t(blockIdx.x) * blockDim.x + threadIdx.x) >> 5;
  const int64_t warps_total = (int64_t(gridDim.x) * blockDim.x) >> 5;
  for (int64_t r0 = warp_global * RPW; r0 < rows; r0 += warps_total * RPW) {
    const int64_t row = min(r0 + sub, rows - 1);
    const int t = int(row % p.Tq);
    const int64_t bh = row / p.Tq;
    const int h = int(bh % p.H);
    const int64_t b = bh / p.H;
    const int64_t off = b * p.os.b + h * p.os.h + int64_t(t) * p.os.t + lir * 8;
    const uint4 a = *reinterpret_cast<const uint4*>(p.o + off), c = *reinterpret_cast<const uint4*>(p.d_o + off);
    const __nv_bfloat162* a2 = reinterpret_cast<const __nv_bfloat162*>(&a);
    const __nv_bfloat162* c2 = reinterpret_cast<const __nv_bfloat162*>(&c);
    float d = 0.f;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const float2 fa = __bfloat1622float2(a2[i]), fc = __bfloat1622float2(c2[i]);
      d = fmaf(fa.x, fc.x, d);
      d = fmaf(fa.y, fc.y, d);
    }
#pragma unroll
    for (int o = LPR / 2; o > 0; o >>= 1) d += __shfl_xor_sync(0xffffffffu, d, o);
    if (lir == 0 && r0 + sub < rows) p.delta[row] = d;
  }
}

int make_map(CUtensorMap* tm, const void* base, const Strides3& s, int B, int H, int T, int D) {
  const uint64_t dims[4] = {uint64_t(D), uint64_t(T), uint64_t(H), uint64_t(B)};
  const uint64_t strides[3] = {uint64_t(s.t), uint64_t(s.h), uint64_t(s.b)};
  const uint32_t box[4] = {64, 128, 1, 1};
  return make_tmap_bf16(tm, base, 4, dims, strides, box, true);
}

template <int D>
int launch_d(const AttnBwdParams& p, cudaStream_t stream) {
  CUtensorMap tq, tk, tv, tdo;
  if (int rc = make_map(&tq, p.q, p.qs, p.B, p.H, p.Tq, D)) return rc;
  if (int rc = make_map(&tk, p.k, p.ks, p.B, p.H, p.Tk, D)) return rc;
  if (int rc = make_map(&tv, p.v, p.vs, p.B, p.H, p.Tk, D)) return rc;
  if (int rc = make_map(&tdo, p.d_o, p.os, p.B, p.H, p.Tq, D)) return rc;
  static PerDeviceOnce configured;
  int sms = 0;
  if (int rc = configured.run([&] {
        cudaError_t e = cudaFuncSetAttribute(attn_bwd_tc_kernel<D, 0>, cudaFuncAttributeMaxDynamicSharedMemorySize, int(smem_bytes<D>()));
        return e != cudaSuccess ? e : cudaFuncSetAttribute(attn_bwd_tc_kernel<D, 1>, cudaFuncAttributeMaxDynamicSharedMemorySize, int(smem_bytes<D>()));
      }, &sms)) return rc;
  const int64_t rows = int64_t(p.B) * p.H * p.Tq;
  int64_t blocks = (rows / (32 / (D / 8)) + 7) / 8;
  if (blocks > sms * 8) blocks = sms * 8;
  attn_delta_kernel<D><<<unsigned(blocks), 256, 0, stream>>>(p);
  ALG_CUDA_TRY(cudaGetLastError());
  const dim3 grid(p.H, p.B, p.Tq / BT);
  attn_bwd_tc_kernel<D, 0><<<grid, NTHREADS, smem_bytes<D>(), stream>>>(tq, tk, tv, tdo, p);
  ALG_CUDA_TRY(cudaGetLastError());
  attn_bwd_tc_kernel<D, 1><<<grid, NTHREADS, smem_bytes<D>(), stream>>>(tq, tk, tv, tdo, p);
  ALG_CUDA_TRY(cudaGetLastError());
  count_launch(3);
  return ALG_OK;
}

}  // namespace

bool attn_bwd_tcgen05_supports(const AttnBwdParams& p) {
  const bool strides_fit = p.qs.t > 0 && p.ks.t > 0 && p.vs.t > 0 && p.os.t > 0 && p.qs.h >= 0 && p.qs.b >= 0 &&
                           p.ks.h >= 0 && p.ks.b >= 0 && p.vs.h >= 0 && p.vs.b >= 0 && p.os.h >= 0 && p.os.b >= 0;
  const bool rows_fit = p.B <= 65535 && p.Tq / BT <= 65535 && (reinterpret_cast<uintptr_t>(p.stat) & 15) == 0;
  return p.causal && p.Tq == p.Tk && p.Tq % BT == 0 && (p.D == 64 || p.D == 128) && strides_fit && rows_fit &&
         (p.B == 1 || (p.qs.b > 0 && p.os.b > 0)) && (p.H == 1 || (p.qs.h > 0 && p.os.h > 0));
}

int launch_attn_bwd_tcgen05(const AttnBwdParams& p, cudaStream_t stream) {
  if (p.dsink != nullptr) ALG_CUDA_TRY(cudaMemsetAsync(p.dsink, 0, sizeof(float) * p.H, stream));
  return p.D == 64 ? launch_d<64>(p, stream) : launch_d<128>(p, stream);
}

}  // namespace alg
