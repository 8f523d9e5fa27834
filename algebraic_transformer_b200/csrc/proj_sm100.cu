// The two wide projections of a prefill block as tcgen05 GEMMs whose consumers run in the
// epilogue, on the accumulator tile while it is still in tensor memory:
//
//   QKV  y = x . W_qkv^T, then per head: round to bf16, RMS-normalise q and k over the head
//        (fp32, gain, one rounding), Cayley rotate-half in bf16 arithmetic, and the range
//        guard's maxima (largest |q_scaled|^2, |k|^2, |v|) — reference: the q/k/v lines of
//        src/algebraic/model.py:165-174 with algebraic.py:76-83 (rms_norm), :172-179
//        (apply_rotary) and kernels/flash.py:831-849 (guard).  The stand-alone kernels for
//        these steps (qk_prep.cu) never run; the un-normalised projections never reach HBM.
//   DZ   z = h . E^T once more, then the Alg-CE head's logit gradient dz from the saved row
//        statistic (src/algebraic/kernels/fused_head.py:120-156), written as bf16 for the two
//        library GEMMs dh = dz . E and dE = dz^T . h that follow, as the reference does.
//   RESID out = resid + x . W^T (the block's out- and down-projection with its residual add,
//        src/algebraic/model.py:183, 193: the product rounded to bf16, then a bf16 add), and per
//        row the sum of squares of what was written, as one partial per 128 or 64 output columns:
//        the RMS normalisation that follows in the reference (model.py:141-143) is then carried
//        by the NEXT projection, which multiplies its accumulator rows by tau = rsqrt(mean + eps)
//        (`row_ss`) and has the norm's gain folded into its weight columns.  The normalised
//        activations never exist in memory and the norm is no launch of its own.
//   GLU  [gate | up] = x . W_gu^T, then out = gate * ALU(up) — src/algebraic/model.py:184-193
//        with algebraic.py's alu.  The weight rows are interleaved in blocks of 128 (gate
//        block j, up block j, ...) so that one 256-wide accumulator tile holds both operands of
//        128 output features; gate and up never reach HBM.
//
// The main loop is the persistent, warp-specialised GEMM of head_sm100.cu: warp 0 (one lane)
// feeds a 4-stage shared-memory ring with TMA (128x64 activation tiles, 256x64 weight tiles,
// 128-byte swizzle), warp 1 (one lane) issues tcgen05.mma 128x256x16 into one of two 256-column
// TMEM accumulators, warps 2..9 drain the finished accumulator (thread = row) while the other
// one fills.  The epilogues keep values as packed bf16 pairs wherever the reference's
// arithmetic is bf16 (one conversion or one HMUL2/HADD2 per two elements) and keep the next
// tensor-memory load in flight while the current chunk is worked on: with K of only 768..1536
// the accumulator turns over every few microseconds and the epilogue is what has to keep up.
// Every wait is bounded; a wait that runs out sets ALG_DEV_TIMEOUT.
#include <cuda_bf16.h>

#include "common.cuh"
#include "launchers.h"
#include "sm100_ptx.cuh"

namespace alg {
namespace {

using namespace sm100;

constexpr int BM = 128, BK = 64, STAGES = 4, UMMA_K = 16;
constexpr int BN_MAX = 256;                      // accumulator tile width: 256, or 128 for the residual GEMM on few rows
constexpr int A_BYTES = BM * BK * 2;
constexpr int STAGE_BYTES = A_BYTES + BN_MAX * BK * 2;   // ring slots are sized for the wide tile
constexpr int NTHREADS = 320, EPI_THREADS = 256;
constexpr uint32_t TMEM_COLS = 512;

struct __align__(16) Control {
  uint64_t full[STAGES], empty[STAGES], tfull[2], tempty[2];
  uint32_t tmem_base;
  int abort_flag;
};
// ring | control | one 4 KB output staging buffer per epilogue warp | slack to align the base
constexpr int WARP_STAGE_BYTES = 32 * 128;
constexpr size_t STAGE_OFF = size_t(STAGES) * STAGE_BYTES + 256;
constexpr size_t SMEM_BYTES = STAGE_OFF + 8 * WARP_STAGE_BYTES + 1024;
static_assert(sizeof(Control) <= 256, "control block outgrew its slot");
static_assert(SMEM_BYTES + 1024 <= 232448, "shared memory budget (dynamic + the static gain table)");

enum { EPI_QKV = 0, EPI_GLU = 1, EPI_DZ = 2, EPI_RESID = 3 };

__device__ __forceinline__ __nv_bfloat162 as_bf162(uint32_t u) { return *reinterpret_cast<__nv_bfloat162*>(&u); }
__device__ __forceinline__ uint32_t as_u32(__nv_bfloat162 h) { return *reinterpret_cast<uint32_t*>(&h); }
// the two bf16 of a packed pair as fp32 (exact)
__device__ __forceinline__ float pair_lo(uint32_t pk) { return __uint_as_float(pk << 16); }
__device__ __forceinline__ float pair_hi(uint32_t pk) { return __uint_as_float(pk & 0xffff0000u); }

// Where a warp's 32 rows of output go: its 4 KB staging buffer in shared memory, the global
// address of (its first row, column 0 of the tile's output) and how many of its rows exist.
struct WarpOut {
  unsigned char* stage;
  __nv_bfloat16* base;
  int64_t ld;
  int rows;
};

// 64 consecutive output elements (32 packed pairs) of this thread's row, starting at column
// `col` -> global memory by way of the staging buffer.  Thread-per-row stores would hit 32
// different 128-byte lines with 16 bytes each per instruction, and that request rate, not the
// math, bounded these kernels; staged, every store instruction writes four whole lines.  The
// 16-byte chunks are XOR-swizzled by row so that both the row-wise writes and the line-wise
// reads are free of bank conflicts.  Only this warp touches its buffer: __syncwarp suffices.
// `cols` = how many of the 64 columns exist (a multiple of 8; 64 everywhere but at a ragged edge).
__device__ __forceinline__ void store_rows64(const WarpOut& w, int lane, const uint32_t* v, int col, int cols = 64) {
#pragma unroll
  for (int c = 0; c < 8; ++c)
    *reinterpret_cast<uint4*>(w.stage + lane * 128 + ((c ^ (lane & 7)) << 4)) =
        make_uint4(v[4 * c], v[4 * c + 1], v[4 * c + 2], v[4 * c + 3]);
  __syncwarp();
  const int sub = lane >> 3, ch = lane & 7;
#pragma unroll
  for (int k = 0; k < 8; ++k) {
    const int r = 4 * k + sub;
    const uint4 val = *reinterpret_cast<const uint4*>(w.stage + r * 128 + ((ch ^ (r & 7)) << 4));
    if (r < w.rows && ch * 8 < cols) *reinterpret_cast<uint4*>(w.base + int64_t(r) * w.ld + col + ch * 8) = val;
  }
  __syncwarp();
}

// The reverse: 64 consecutive elements of this thread's row of a row-major bf16 matrix (`base` = the
// warp's first row, column 0) -> 32 packed pairs in registers, read as whole lines through the
// same staging buffer.  Rows beyond `rows` read as zero.
__device__ __forceinline__ void load_rows64(unsigned char* stage, const __nv_bfloat16* base, int64_t ld, int rows, int lane,
                                            uint32_t* v, int col) {
  const int sub = lane >> 3, ch = lane & 7;
#pragma unroll
  for (int k = 0; k < 8; ++k) {
    const int r = 4 * k + sub;
    uint4 val = make_uint4(0u, 0u, 0u, 0u);
    if (r < rows) val = *reinterpret_cast<const uint4*>(base + int64_t(r) * ld + col + ch * 8);
    *reinterpret_cast<uint4*>(stage + r * 128 + ((ch ^ (r & 7)) << 4)) = val;
  }
  __syncwarp();
#pragma unroll
  for (int c = 0; c < 8; ++c) {
    const uint4 val = *reinterpret_cast<const uint4*>(stage + lane * 128 + ((c ^ (lane & 7)) << 4));
    v[4 * c] = val.x; v[4 * c + 1] = val.y; v[4 * c + 2] = val.z; v[4 * c + 3] = val.w;
  }
  __syncwarp();
}

// ---- residual epilogue: 64 output columns of one row -------------------------------------------
// out = resid + round_bf16(acc), a bf16 add (src/algebraic/model.py:183, 193: `x + a @ w`, both bf16);
// returns the sum of squares of the 64 values written.
__device__ __forceinline__ float resid_cols(const ProjParams& p, uint32_t taddr, const WarpOut& wo, const __nv_bfloat16* rbase,
                                            int lane, int col) {
  uint32_t res[32], out[32];
  load_rows64(wo.stage, rbase, p.ld_resid, wo.rows, lane, res, col);
  float ss = 0.f;
#pragma unroll
  for (int c = 0; c < 2; ++c) {
    uint32_t r[32];
    tmem_ld_32x32(taddr + c * 32, r);
    tmem_ld_wait();
#pragma unroll
    for (int i = 0; i < 16; ++i) {
      const uint32_t prod = pack_bf16(__uint_as_float(r[2 * i]), __uint_as_float(r[2 * i + 1]));
      const uint32_t y = as_u32(__hadd2(as_bf162(res[c * 16 + i]), as_bf162(prod)));
      out[c * 16 + i] = y;
      ss = fmaf(pair_lo(y), pair_lo(y), ss);
      ss = fmaf(pair_hi(y), pair_hi(y), ss);
    }
  }
  store_rows64(wo, lane, out, col);
  return ss;
}

// tau of this row for a projection whose input is the un-normalised residual stream: the partial sums
// of squares the producing kernel left, added in slot order.
__device__ __forceinline__ float row_tau(const ProjParams& p, int row, bool live) {
  if (p.row_ss == nullptr) return 1.0f;
  float ss = 0.f;
  if (live)
    for (int s = 0; s < p.ss_slots; ++s) ss += p.row_ss[int64_t(s) * p.M + row];
  return rsqrtf(ss * (1.0f / float(p.K)) + p.row_eps);
}

// ---- head-backward epilogue: dz for 128 vocabulary columns of one row ------------------------
// The reference's custom VJP does not differentiate the primal value mean_i (1 - pt_i): it applies
// the gradient of the negative log-likelihood,
//   dz_ij = (g / N) (n / c) r_ij (p_ij - [j == t_i]),  p = w / l,  w = rho(x)^n,
//   x = min(z / c, clamp),  r = 1 / sqrt(1 + x^2)  (the clamp is straight-through: r of the clamped x)
// (src/algebraic/kernels/fused_head.py:120-145 and 236-243, src/algebraic/algebraic.py:309-316).
// `a_i` = g / N and 1/l_i come in as arguments; `tgt` is the target's column inside this shard
// (any value outside [0, V_local) when it lives elsewhere).
__device__ __forceinline__ void dz_cols(const ProjParams& p, uint32_t taddr, const WarpOut& wo, int lane, int col0,
                                        float a_i, float inv_l, int tgt) {
#pragma unroll 1
  for (int u = 0; u < 2; ++u) {                          // two units of 64 columns
    uint32_t pk[32];
#pragma unroll
    for (int c = 0; c < 2; ++c) {
      uint32_t r[32];
      tmem_ld_32x32(taddr + u * 64 + c * 32, r);
      tmem_ld_wait();
      const int cbase = col0 + u * 64 + c * 32;
      if (p.head_kind == ALG_HEAD_CE) {
        // softmax cross-entropy: dz = (g / N) (exp(z - lse) - y), `inv_l` carries the row's logsumexp
        // (src/algebraic/kernels/fused_head.py:134-135)
        constexpr float LOG2E = 1.4426950408889634f;
        const float off = -inv_l * LOG2E;
#pragma unroll
        for (int i = 0; i < 32; i += 2) {
          const float p0 = exp2_approx(fmaf(__uint_as_float(r[i]), LOG2E, off));
          const float p1 = exp2_approx(fmaf(__uint_as_float(r[i + 1]), LOG2E, off));
          pk[c * 16 + (i >> 1)] = pack_bf16(a_i * (p0 - ((cbase + i == tgt) ? 1.f : 0.f)),
                                            a_i * (p1 - ((cbase + i + 1 == tgt) ? 1.f : 0.f)));
        }
        continue;
      }
      // the n-th power as log2n passes over the 32 values: every pass is 32 independent
      // multiplications (a loop per value would serialise on its own latency)
      // (pairs of columns through the packed fp32 instructions)
      float2 w[16], sl[16];
      const float an = a_i * p.n_over_c;
      const float2 an2 = make_float2(an, an), ic2 = make_float2(p.inv_c, p.inv_c), one2 = make_float2(1.f, 1.f);
      const float2 il2 = make_float2(inv_l, inv_l);
#pragma unroll
      for (int i = 0; i < 16; ++i) {
        float2 x = __fmul2_rn(make_float2(__uint_as_float(r[2 * i]), __uint_as_float(r[2 * i + 1])), ic2);
        x.x = fminf(x.x, p.clamp);
        x.y = fminf(x.y, p.clamp);
        const float2 rad = __ffma2_rn(x, x, one2);
        const float2 rs = make_float2(rsqrt_approx(rad.x), rsqrt_approx(rad.y));
        w[i] = __ffma2_rn(rad, rs, x);                                          // rho_fast(x)
        sl[i] = __fmul2_rn(an2, rs);                                            // (g / N) (n / c) r_ij
      }
      for (int it = 0; it < p.log2n; ++it) {
#pragma unroll
        for (int i = 0; i < 16; ++i) w[i] = __fmul2_rn(w[i], w[i]);
      }
#pragma unroll
      for (int i = 0; i < 16; ++i) {
        const float2 negy = make_float2((cbase + 2 * i == tgt) ? -1.f : 0.f, (cbase + 2 * i + 1 == tgt) ? -1.f : 0.f);
        const float2 d = __fmul2_rn(sl[i], __ffma2_rn(w[i], il2, negy));
        pk[c * 16 + i] = pack_bf16(d.x, d.y);
      }
    }
    const int first = col0 + u * 64;
    if (first < p.N) store_rows64(wo, lane, pk, first, min(64, p.N - first));   // warp-uniform
  }
}

// ---- QKV epilogue: one head (D accumulator columns from `taddr`) of one row ----------------
// kind 0 = q, 1 = k (normalise, rotate, statistic), 2 = v (round, statistic).
// `tc`, `ts`: this row's cos / sin table entries as packed bf16 pairs (D/4 each), in registers.
template <int D>
__device__ __forceinline__ void qkv_head(const ProjParams& p, const float* s_gain, uint32_t taddr, int kind,
                                         const uint32_t* tc, const uint32_t* ts, const WarpOut& wo, int lane, int col,
                                         bool live, float tau_row, float& best_q, float& best_k, float& best_v) {
  constexpr int NP = D / 2, QP = D / 4;                // packed pairs per head / per half
  uint32_t pk[NP];                                     // the projection rounded to bf16 (the GEMM's output dtype)
  float2 ss2 = make_float2(0.f, 0.f);                  // packed fp32 throughout: the epilogue's instruction count, not the
  const float2 tau_row2 = make_float2(tau_row, tau_row);   // main loop, bounds this kernel
  __nv_bfloat162 vmax2 = as_bf162(0u);
  {
    // two chunks in flight for D = 64; for D = 128 the table already holds 64 registers, so one
    constexpr bool DOUBLE = (D == 64);
    uint32_t a[32], b[DOUBLE ? 32 : 1];
    tmem_ld_32x32(taddr, a);
#pragma unroll
    for (int c = 0; c < D / 32; ++c) {
      uint32_t* cur = (DOUBLE && (c & 1)) ? b : a;
      uint32_t* nxt = (DOUBLE && !(c & 1)) ? b : a;
      tmem_ld_wait_for(cur);
      if (DOUBLE && c + 1 < D / 32) tmem_ld_32x32(taddr + (c + 1) * 32, nxt);
#pragma unroll
      for (int i = 0; i < 16; ++i) {
        const float2 sc = __fmul2_rn(make_float2(__uint_as_float(cur[2 * i]), __uint_as_float(cur[2 * i + 1])), tau_row2);
        const uint32_t w = pack_bf16(sc.x, sc.y);
        pk[c * 16 + i] = w;
        if (kind == 2) {
          vmax2 = __hmax2(vmax2, __habs2(as_bf162(w)));
        } else {
          const float2 r2 = make_float2(pair_lo(w), pair_hi(w));
          ss2 = __ffma2_rn(r2, r2, ss2);
        }
      }
      if (!DOUBLE && c + 1 < D / 32) tmem_ld_32x32(taddr + (c + 1) * 32, a);
    }
  }
  if (kind == 2) {
    if (live) {
      const float2 m = __bfloat1622float2(vmax2);
      best_v = fmaxf(best_v, fmaxf(m.x, m.y));
    }
#pragma unroll
    for (int h64 = 0; h64 < D / 64; ++h64) store_rows64(wo, lane, pk + 32 * h64, col + 64 * h64);
    return;
  }
  const float tau = rsqrtf((ss2.x + ss2.y) * (1.0f / D) + p.eps);
  const float2 tau2 = make_float2(tau, tau);
  const float* gain = s_gain + kind * 128;             // shared-memory copy: q gains, then k gains
  const bool exact_scale = (kind == 1) || (p.q_scale_pow2 != 0);
  const float stat_scale = (kind == 0) ? p.q_scale : 1.0f;
  float2 stat2 = make_float2(0.f, 0.f);
  const float2 stat_scale2 = make_float2(stat_scale, stat_scale);
#pragma unroll
  for (int g2i = 0; g2i < QP / 2; ++g2i) {             // two pairs = four gains of each half per step
    const float4 ga = *reinterpret_cast<const float4*>(gain + 4 * g2i);
    const float4 gb = *reinterpret_cast<const float4*>(gain + D / 2 + 4 * g2i);
    const float g1v[4] = {ga.x, ga.y, ga.z, ga.w}, g2v[4] = {gb.x, gb.y, gb.z, gb.w};
#pragma unroll
    for (int jj = 0; jj < 2; ++jj) {
      const int j = g2i * 2 + jj;                      // pair j of the first half, partner pair j + QP
      // x <- round((x * tau) * gain)
      const float2 a1 = __fmul2_rn(__fmul2_rn(make_float2(pair_lo(pk[j]), pair_hi(pk[j])), tau2), make_float2(g1v[2 * jj], g1v[2 * jj + 1]));
      const float2 a2 = __fmul2_rn(__fmul2_rn(make_float2(pair_lo(pk[j + QP]), pair_hi(pk[j + QP])), tau2), make_float2(g2v[2 * jj], g2v[2 * jj + 1]));
      const uint32_t x1 = pack_bf16(a1.x, a1.y), x2 = pack_bf16(a2.x, a2.y);
      const __nv_bfloat162 X1 = as_bf162(x1), X2 = as_bf162(x2), Cc = as_bf162(tc[j]), Ss = as_bf162(ts[j]);
      // bf16 arithmetic, every product and sum rounded: (x1 c - x2 s, x1 s + x2 c)
      const uint32_t y1 = as_u32(__hsub2(__hmul2(X1, Cc), __hmul2(X2, Ss)));
      const uint32_t y2 = as_u32(__hadd2(__hmul2(X1, Ss), __hmul2(X2, Cc)));
      pk[j] = y1;
      pk[j + QP] = y2;
      uint32_t s1 = y1, s2 = y2;
      if (!exact_scale) {                              // the guard looks at the scaled, re-rounded q
        const float2 b1 = __fmul2_rn(make_float2(pair_lo(y1), pair_hi(y1)), stat_scale2);
        const float2 b2 = __fmul2_rn(make_float2(pair_lo(y2), pair_hi(y2)), stat_scale2);
        s1 = pack_bf16(b1.x, b1.y);
        s2 = pack_bf16(b2.x, b2.y);
      }
      const float2 q1 = make_float2(pair_lo(s1), pair_hi(s1)), q2 = make_float2(pair_lo(s2), pair_hi(s2));
      stat2 = __ffma2_rn(q1, q1, stat2);
      stat2 = __ffma2_rn(q2, q2, stat2);
    }
  }
  const float stat = stat2.x + stat2.y;
  if (live) {
    // a power-of-two scale commutes with every rounding above: apply it to the sum
    if (kind == 0) best_q = fmaxf(best_q, exact_scale ? stat * (stat_scale * stat_scale) : stat);
    else best_k = fmaxf(best_k, stat);
  }
#pragma unroll
  for (int h64 = 0; h64 < D / 64; ++h64) store_rows64(wo, lane, pk + 32 * h64, col + 64 * h64);
}

// ---- GLU epilogue ---------------------------------------------------------------------------
// gu[0..15] = 16 gate accumulators, gu[16..31] = the matching up accumulators -> 8 packed outputs
__device__ __forceinline__ void glu16(const uint32_t* gu, float beta, float tau_row, uint32_t* out) {
#pragma unroll
  for (int i = 0; i < 8; ++i) {
    const uint32_t gp = pack_bf16(__uint_as_float(gu[2 * i]) * tau_row, __uint_as_float(gu[2 * i + 1]) * tau_row);
    const uint32_t up = pack_bf16(__uint_as_float(gu[16 + 2 * i]) * tau_row, __uint_as_float(gu[16 + 2 * i + 1]) * tau_row);
    // both values of the pair through the packed fp32 instructions
    const float2 uv = make_float2(pair_lo(up), pair_hi(up));
    const float2 one = make_float2(1.f, 1.f);
    const float2 bz = __fmul2_rn(uv, make_float2(beta, beta));
    const float2 rad = __ffma2_rn(bz, bz, one);
    const float2 r = make_float2(rsqrt_approx(rad.x), rsqrt_approx(rad.y));
    const float2 uu = __fmul2_rn(bz, r);
    // for bz < 0 use 1 + u = r^2 / (1 - u) so that the negative tail survives
    const float2 den = __ffma2_rn(uu, make_float2(-1.f, -1.f), one);
    const float2 neg = __fmul2_rn(__fmul2_rn(r, r), make_float2(__fdividef(1.0f, den.x), __fdividef(1.0f, den.y)));
    const float2 pos = __fadd2_rn(uu, one);
    const float2 opu = make_float2(bz.x < 0.f ? neg.x : pos.x, bz.y < 0.f ? neg.y : pos.y);
    const float2 act = __fmul2_rn(__fmul2_rn(uv, make_float2(0.5f, 0.5f)), opu);
    // gate (bf16) times the bf16-rounded activation, rounded once: a bf16 multiply
    out[i] = as_u32(__hmul2(as_bf162(gp), as_bf162(pack_bf16(act.x, act.y))));
  }
}

// 64 output features of one row: gate columns from t_gate, up columns from t_up
__device__ __forceinline__ void glu_cols(const ProjParams& p, uint32_t t_gate, uint32_t t_up, const WarpOut& wo, int lane,
                                         int col, float tau_row) {
  uint32_t a[32], b[32], o[32];
  tmem_ld_32x16(t_gate, a);
  tmem_ld_32x16(t_up, a + 16);
#pragma unroll
  for (int c = 0; c < 4; ++c) {
    uint32_t* cur = (c & 1) ? b : a;
    uint32_t* nxt = (c & 1) ? a : b;
    tmem_ld_wait_for(cur);
    if (c + 1 < 4) {
      tmem_ld_32x16(t_gate + (c + 1) * 16, nxt);
      tmem_ld_32x16(t_up + (c + 1) * 16, nxt + 16);
    }
    glu16(cur, p.beta, tau_row, o + 8 * c);
  }
  store_rows64(wo, lane, o, col);
}

template <int EPI, int D, int BN>
__global__ void __launch_bounds__(NTHREADS, 1)
proj_tc_kernel(const __grid_constant__ CUtensorMap tm_x, const __grid_constant__ CUtensorMap tm_w, const ProjParams p) {
  extern __shared__ unsigned char smem_raw[];
  unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  Control* ctl = reinterpret_cast<Control*>(smem + size_t(STAGES) * STAGE_BYTES);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  constexpr uint32_t IDESC = make_idesc_bf16(BM, BN, 0, 0);
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
  // Launched as a programmatic dependent: everything above overlapped the tail of the kernel ahead in the
  // stream; from here on its results are complete.
  griddep_wait();
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
          mbar_arrive_expect_tx(&ctl->full[stage], A_BYTES + BN * BK * 2);
          tma_load_2d(dst, &tm_x, &ctl->full[stage], kb * BK, m * BM);
          tma_load_2d(dst + A_BYTES, &tm_w, &ctl->full[stage], kb * BK, n * BN);
          if (++stage == STAGES) { stage = 0; phase ^= 1u; }
        }
      }
    }
  } else if (warp == 1) {
    // The whole warp runs the loop and one elected lane issues: an issue then costs the thread about
    // 32 cycles instead of 48, which matters for the 128-wide tile, whose MMAs take only 64.
    uint32_t stage = 0, phase = 0, tile_count = 0;
    const uint32_t a_lo0 = sw128_desc_lo(smem_u32(smem), 16), b_lo0 = sw128_desc_lo(smem_u32(smem) + A_BYTES, 16);
    auto wait_all = [&](uint64_t* bar, uint32_t parity) { return __all_sync(0xffffffffu, bw.wait(bar, parity)) != 0; };
    bool ok = true;
    for (int u = blockIdx.x; u < tiles && ok; u += gridDim.x, ++tile_count) {
      const uint32_t buf = tile_count & 1u, tphase = (tile_count >> 1) & 1u;
      if (!wait_all(&ctl->tempty[buf], tphase ^ 1u)) { ok = false; break; }
      tc_fence_after();
      const uint32_t d_tmem = tmem_base + buf * BN;
      for (int kb = 0; kb < kblocks; ++kb) {
        if (!wait_all(&ctl->full[stage], phase)) { ok = false; break; }
        tc_fence_after();
        if (elect_one()) {
          const uint32_t a_lo = a_lo0 + stage * (STAGE_BYTES >> 4), b_lo = b_lo0 + stage * (STAGE_BYTES >> 4);
#pragma unroll
          for (int k = 0; k < BK / UMMA_K; ++k)
            umma_f16_ss_parts(d_tmem, a_lo + k * (UMMA_K * 2 >> 4), SW128_DESC_HI, b_lo + k * (UMMA_K * 2 >> 4),
                              SW128_DESC_HI, IDESC, (kb | k) != 0 ? 1u : 0u);
          umma_commit(&ctl->empty[stage]);             // smem stage is free once these MMAs retire
          if (kb == kblocks - 1) umma_commit(&ctl->tfull[buf]);   // accumulator tile complete
        }
        __syncwarp();
        if (++stage == STAGES) { stage = 0; phase ^= 1u; }
      }
    }
  } else {
    const int quarter = warp & 3;                        // TMEM lanes 32*quarter .. +31 belong to this warp
    const int half = (warp - 2) >> 2;
    const int row_in_tile = quarter * 32 + lane;
    const uint32_t lane_sel = uint32_t(quarter * 32) << 16;
    unsigned char* stage = smem + STAGE_OFF + (warp - 2) * WARP_STAGE_BYTES;
    uint32_t tile_count = 0;
    float best_q = 0.f, best_k = 0.f, best_v = 0.f;
    bool ok = true;
    for (int u = blockIdx.x; u < tiles && ok; u += gridDim.x, ++tile_count) {
      const int m = u / tiles_n, n = u % tiles_n;
      const uint32_t buf = tile_count & 1u, tphase = (tile_count >> 1) & 1u;
      const int row = m * BM + row_in_tile;
      const bool live = row < p.M;
      // QKV: this row's rotation table entries, the same for every q and k head of the tile,
      // fetched before the wait so that their latency hides behind the accumulator filling
      constexpr int TQ = (EPI == EPI_QKV) ? D / 4 : 1;
      uint32_t tc[TQ], ts[TQ];
      const int hd = p.H * D;
      if (EPI == EPI_QKV && (n * BN + half * 128) / hd < 2) {   // kinds only grow along a tile: q/k present
        const int t = live ? row % p.T : 0;
        const uint4* ct = reinterpret_cast<const uint4*>(p.cos + int64_t(t) * (D / 2));
        const uint4* st = reinterpret_cast<const uint4*>(p.sin + int64_t(t) * (D / 2));
#pragma unroll
        for (int i = 0; i < TQ / 4; ++i) {
          const uint4 cv = ct[i], sv = st[i];
          tc[4 * i] = cv.x; tc[4 * i + 1] = cv.y; tc[4 * i + 2] = cv.z; tc[4 * i + 3] = cv.w;
          ts[4 * i] = sv.x; ts[4 * i + 1] = sv.y; ts[4 * i + 2] = sv.z; ts[4 * i + 3] = sv.w;
        }
      }
      const float tau_row = (EPI == EPI_QKV || EPI == EPI_GLU) ? row_tau(p, row, live) : 1.0f;   // before the wait, like the table rows
      if (!bw.wait(&ctl->tfull[buf], tphase)) { ok = false; break; }
      tc_fence_after();
      const uint32_t tbuf = tmem_base + lane_sel + buf * BN;
      const int wrow = m * BM + quarter * 32;            // first row of this warp
      const WarpOut wo{stage, p.out + int64_t(wrow) * p.ld_out, p.ld_out, min(32, max(0, p.M - wrow))};
      if (EPI == EPI_QKV) {
#pragma unroll 1
        for (int hh = 0; hh < 128 / D; ++hh) {
          const int lcol = half * 128 + hh * D;          // column inside the tile
          const int gcol = n * BN + lcol;                // output feature
          if (gcol >= p.N) break;
          qkv_head<D>(p, s_gain, tbuf + lcol, gcol / hd, tc, ts, wo, lane, gcol, live, tau_row, best_q, best_k, best_v);
        }
      } else if (EPI == EPI_DZ) {
        // per-row constants of the head's backward: 1 / l_i and the common factor g / N
        float inv_l = 0.f, a_i = 0.f;
        int tgt = -1;
        if (live) {
          inv_l = p.head_kind == ALG_HEAD_CE ? p.l[row] : 1.0f / p.l[row];   // ce: the logsumexp itself
          a_i = p.gscale;
          tgt = p.targets[row] - p.vocab_offset;
        }
        dz_cols(p, tbuf + half * 128, wo, lane, n * BN + half * 128, a_i, inv_l, tgt);
      } else if (EPI == EPI_RESID) {
        // this thread's BN / 2 columns of its row, 64 at a time; one partial sum of squares per thread
        const __nv_bfloat16* rbase = p.resid + int64_t(wrow) * p.ld_resid;
        float ss = 0.f;
#pragma unroll 1
        for (int u64 = 0; u64 < BN / 128; ++u64) {
          const int lcol = half * (BN / 2) + u64 * 64;
          if (n * BN + lcol < p.N) ss += resid_cols(p, tbuf + lcol, wo, rbase, lane, n * BN + lcol);
        }
        if (p.ss_out != nullptr && live) p.ss_out[int64_t(n * 2 + half) * p.M + row] = ss;
      } else {
        const int fcol = n * 128 + half * 64;            // output feature of this thread's first column
        if (fcol < p.f)
          glu_cols(p, tbuf + half * 64, tbuf + 128 + half * 64, wo, lane, fcol, tau_row);
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

template <int EPI, int D, int BN = BN_MAX>
int launch_variant(const CUtensorMap& tm_x, const CUtensorMap& tm_w, const ProjParams& p, int grid, cudaStream_t stream) {
  auto kern = proj_tc_kernel<EPI, D, BN>;
  static PerDeviceOnce configured;
  if (int rc = configured.run([&] { return cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, int(SMEM_BYTES)); })) return rc;
  ALG_CUDA_TRY(launch_dependent(kern, dim3(grid), dim3(NTHREADS), SMEM_BYTES, stream, tm_x, tm_w, p));
  count_launch();
  return ALG_OK;
}

}  // namespace

// The residual GEMM's tile is 128 x 256 unless 128 x 128 tiles spread better over the SMs (few rows: a
// rank's share of a batch split over many GPUs).  Cost model: rounds of tiles per CTA times the time of
// one tile, a narrow tile taking a little more than half of a wide one.
int proj_resid_tile_width(int M, int N) {
  const int sms = sm_count(), mt = (M + BM - 1) / BM;
  const int wide = mt * ((N + 255) / 256), narrow = mt * ((N + 127) / 128);
  const double cost_wide = double((wide + sms - 1) / sms), cost_narrow = 0.55 * double((narrow + sms - 1) / sms);
  return cost_narrow < cost_wide ? 128 : 256;
}

int launch_proj(const ProjParams& p, const void* x, const void* w, int epi, cudaStream_t stream) {
  if (p.M == 0) return ALG_OK;
  CUtensorMap tm_x, tm_w;
  {
    const uint64_t dims[2] = {uint64_t(p.K), uint64_t(p.M)};
    const uint64_t strides[1] = {uint64_t(p.ld_x)};
    const uint32_t box[2] = {BK, BM};
    if (int rc = make_tmap_bf16(&tm_x, x, 2, dims, strides, box, true)) return rc;
  }
  const int bn = epi == 3 ? proj_resid_tile_width(p.M, p.N) : BN_MAX;
  {
    const uint64_t dims[2] = {uint64_t(p.K), uint64_t(p.N)};
    const uint64_t strides[1] = {uint64_t(p.K)};
    const uint32_t box[2] = {BK, uint32_t(bn)};
    if (int rc = make_tmap_bf16(&tm_w, w, 2, dims, strides, box, true)) return rc;
  }
  const int sms = sm_count();
  const int tiles = ((p.M + BM - 1) / BM) * ((p.N + bn - 1) / bn);
  const int grid = tiles < sms ? tiles : sms;
  if (epi == 3) return bn == 128 ? launch_variant<EPI_RESID, 64, 128>(tm_x, tm_w, p, grid, stream)
                                 : launch_variant<EPI_RESID, 64, 256>(tm_x, tm_w, p, grid, stream);
  if (epi == 1) return launch_variant<EPI_GLU, 64>(tm_x, tm_w, p, grid, stream);
  if (epi == 2) return launch_variant<EPI_DZ, 64>(tm_x, tm_w, p, grid, stream);
  return p.D == 64 ? launch_variant<EPI_QKV, 64>(tm_x, tm_w, p, grid, stream)
                   : launch_variant<EPI_QKV, 128>(tm_x, tm_w, p, grid, stream);
}

}  // namespace alg
