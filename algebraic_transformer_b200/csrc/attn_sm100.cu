// Asinh-power attention forward on tcgen05 tensor cores (the throughput path).
//
// Covers the unshifted accumulation of the reference (src/algebraic/kernels/flash.py:
// 227-234): p = rho_fast(x)^n, l = rho(b')^n + sum p, o = (sum p v) / l, stat = 1/l — the
// branch the range guard selects for QK-normalised inputs - and its max-shifted form.  bf16 I/O
// (fp32 at head_dim 64, see the F32 mode), causal, Tq == Tk of any length, head_dim 64 or 128.
// Because nothing is rescaled in the unshifted form, the output accumulator simply stays in
// tensor memory from the first key tile to the last.  A sequence that does not fill its last
// 256-row block needs no special case beyond masked stores: TMA fills rows past the end with
// zeros, keys past the end lie above the diagonal of every real row, and rows past the end
// compute finite values nobody stores.
//
// One CTA owns 256 consecutive query rows of one (batch, head): two 128-row tiles.
//   warp 0 (one lane)  TMA: both Q tiles once, then K_j / V_j tiles through a ring
//   warp 1             tcgen05.mma (the whole warp runs the loop, one elected lane issues):
//                      S_w = Q_w K_j^T (both operands in shared memory) and O_w += P_w V_j with P_w
//                      read from TENSOR MEMORY (the A operand) and V_j from shared memory as an
//                      MN-major B operand
//   warp 2             scales the Q tiles in shared memory by a power of two (see below)
//   warp 3             on request, takes the range guard's maxima of q, k, v beside the attention
//                      work, so that a guarded call needs no separate pass over its inputs
//   weight group 0     weights for query tile 0: tcgen05.ld S_0 (one thread = one row),
//                      x -> rho_fast(x)^n in packed fp32, row sum, bf16 P_0 written back
//                      with tcgen05.st over columns S_0 occupied
//   weight group 1     the same for query tile 1
// A weight group is 4 * SPLIT warps.  With SPLIT = 2 two warps share each 32-lane quarter of
// tensor memory and take 64 of the tile's 128 key columns each.
//
// The score scale.  x = s / (sqrt(D) c) with 1 / (sqrt(D) c) = 2^e m, 1 <= m < 2.  The factor
// 2^e goes onto Q in shared memory (an exact exponent shift of bf16 values), so tensor memory
// holds y = x / m, and with kappa = 1 / m^2
//     t' = y + sqrt(kappa + y^2) = rho(x) / m
// costs one multiplication less per score than scaling s first.  Every weight is then short of
// the reference's by the constant m^n, which cancels in o = sum(p v) / l; the sink's weight and
// the saved statistic carry the constant explicitly.
//
// Tensor-memory layout (512 columns): S_0, S_1 (128 each) + O_0, O_1 (head_dim each).  The bf16
// weights of S columns [32 g, 32 g + 32) are written over columns [32 g, 32 g + 16) of the same
// block, so a thread only ever overwrites scores it has already read and two warps working on
// different 32-column blocks never touch each other's columns.  P never touches shared memory,
// which leaves the tensor core's shared-memory operand path to Q, K and V alone.
//
// Hand-overs.  The tensor pipe executes one thread's MMAs in issue order, so issuing S_w(j+1)
// after P_w(j).V_j is what protects P_w(j) from being overwritten.  P_w V_j is issued in two
// halves of 64 keys: the weight warps signal after the first 64 keys of a tile, and the first
// half of the product runs while they evaluate the second.  Key tiles above the diagonal are
// never loaded; only the diagonal tile evaluates a mask, and it skips the 32-column blocks that
// lie wholly above the diagonal for its rows.
// The kernel is persistent: one CTA per SM walks a fixed list of work items (heaviest row
// blocks first, dealt out boustrophedon so the per-CTA sums stay level).  Barriers, tensor
// memory and the K/V ring live across items, so the loads of the next item's first tiles
// are in flight while the current item finishes.
// Every mbarrier wait is bounded (sm100_ptx.cuh); on a timeout the kernel reports
// ALG_DEV_TIMEOUT through the status word and returns.
#include "common.cuh"
#include "launchers.h"
#include "sm100_ptx.cuh"

#include <math.h>
#include <stdlib.h>

#include <algorithm>

namespace alg {
namespace {

using namespace sm100;

constexpr int BQ = 128, BKEY = 128;
constexpr int FIRST_WEIGHT_WARP = 4;            // warps 0..3: TMA, MMA, two Q scalers
template <int SPLIT> constexpr int nthreads() { return FIRST_WEIGHT_WARP * 32 + 2 * 4 * SPLIT * 32; }
constexpr int PANEL_BYTES = 128 * 128;          // 128 rows x 64 bf16, one swizzle-128B panel
constexpr uint32_t TMEM_COLS = 512;
constexpr int MAX_NKV = 10;

template <int D> struct Cfg {
  static constexpr int PANELS = D / 64;
  static constexpr int TILE_BYTES = PANELS * PANEL_BYTES;   // one Q / K / V tile
  static constexpr int NKV = (D == 128) ? 5 : 10;           // K/V ring depth (tiles)
  static constexpr int Q_OFF = 0;
  static constexpr int KV_OFF = 2 * TILE_BYTES;
  static constexpr int CTL_OFF = KV_OFF + NKV * TILE_BYTES;
  static constexpr uint32_t S_COL = 0;                      // S_w at S_COL + 128 w; P_w inside it
  static constexpr uint32_t O_COL = 256;                    // O_w at O_COL + D w
  static constexpr uint32_t IDESC_S = make_idesc_bf16(BQ, BKEY, 0, 0);
  static constexpr uint32_t IDESC_PV = make_idesc_bf16(BQ, D, 0, 1);   // V is [key][d]: MN-major B
  static constexpr uint32_t IDESC_PV64 = make_idesc_bf16(BQ, 64, 0, 1); // fp32 rows: 64 output columns from a hi|lo tile
};

struct __align__(16) Control {
  uint64_t q_full[2], q_ready[2], q_free[2], kv_full[MAX_NKV], kv_empty[MAX_NKV];
  uint64_t s_full[2], p_half[2], p_full[2], o_full[2], o_free[2];
  uint64_t s_read[2], pv_done[2];   // head_dim 64: scores read (S_w may be overwritten), second P.V product of a tile done
  uint64_t l_part[2], l_total[2];   // split weight groups: hand-over of the row sums between the column halves
  uint32_t tmem_base;
  int abort_flag;
  int shift_mode;
  float row_sum[2][BQ];       // [query tile][row]: half 1's partial row sum, then the row's total
};

// Tensor-memory column (relative to the S block) of the packed weights of S column `scol`.
__device__ __forceinline__ constexpr uint32_t p_col_of(uint32_t scol) { return 32u * (scol >> 5) + ((scol & 31u) >> 1); }

// W (16 or 32) scores y -> W weights (y + sqrt(kappa + y^2))^n, two at a time on the packed fp32
// pipe (fma.f32x2 / mul.f32x2); row-sum partials in `la`, `lb`; bf16 pairs in `packed`.
// With HILO, packed[W/2 ..] additionally receives the bf16 pairs of what the first rounding left
// over (w - bf16(w)), so that hi + lo carries 16 bits of each weight into the P.V products.
template <int LOG2N, bool DIAG, int W, bool HILO = false>
__device__ __forceinline__ void weigh(const uint32_t* s, float kappa, int col0, int r, float2& la, float2& lb,
                                      uint32_t* packed) {
  if (DIAG && col0 > (r | 31)) {                    // warp-uniform: the block lies above the diagonal for all 32 rows
#pragma unroll
    for (int i = 0; i < (HILO ? W : W / 2); ++i) packed[i] = 0u;
    return;
  }
  const float2 kp = make_float2(kappa, kappa);
#pragma unroll
  for (int i = 0; i < W; i += 4) {
    const float2 y0 = make_float2(__uint_as_float(s[i]), __uint_as_float(s[i + 1]));
    const float2 y1 = make_float2(__uint_as_float(s[i + 2]), __uint_as_float(s[i + 3]));
    const float2 rad0 = __ffma2_rn(y0, y0, kp), rad1 = __ffma2_rn(y1, y1, kp);
    const float2 rs0 = make_float2(rsqrt_approx(rad0.x), rsqrt_approx(rad0.y));
    const float2 rs1 = make_float2(rsqrt_approx(rad1.x), rsqrt_approx(rad1.y));
    float2 t0 = __ffma2_rn(rad0, rs0, y0), t1 = __ffma2_rn(rad1, rs1, y1);
#pragma unroll
    for (int k = 0; k < LOG2N; ++k) { t0 = __fmul2_rn(t0, t0); t1 = __fmul2_rn(t1, t1); }
    if (DIAG) {                                     // causal mask inside the diagonal tile
      t0.x = (col0 + i <= r) ? t0.x : 0.f;     t0.y = (col0 + i + 1 <= r) ? t0.y : 0.f;
      t1.x = (col0 + i + 2 <= r) ? t1.x : 0.f; t1.y = (col0 + i + 3 <= r) ? t1.y : 0.f;
    }
    la = __fadd2_rn(la, t0);
    lb = __fadd2_rn(lb, t1);
    const uint32_t h0 = pack_bf16(t0.x, t0.y), h1 = pack_bf16(t1.x, t1.y);
    packed[i >> 1] = h0;
    packed[(i >> 1) + 1] = h1;
    if (HILO) {
      packed[W / 2 + (i >> 1)] = pack_bf16(t0.x - __uint_as_float(h0 << 16), t0.y - __uint_as_float(h0 & 0xffff0000u));
      packed[W / 2 + (i >> 1) + 1] = pack_bf16(t1.x - __uint_as_float(h1 << 16), t1.y - __uint_as_float(h1 & 0xffff0000u));
    }
  }
}

// "The first 64 keys of this tile are weighed": stores complete, then one arrival per thread.
__device__ __forceinline__ void signal_weights(uint64_t* bar) {
  tmem_st_wait();
  tc_fence_before();
  mbar_arrive(bar);
}

// One 128-key score tile of this thread's row (one warp per tensor-memory quarter): S from
// tensor memory -> weights -> packed bf16 P back over the block the scores came from.  The load
// of the next 32 columns is in flight while the current 32 are evaluated.
template <int LOG2N, bool DIAG>
__device__ __forceinline__ void weigh_tile(uint32_t s_taddr, int r, float kappa, float2& la, float2& lb,
                                           uint64_t* p_half, uint64_t* p_full) {
  uint32_t a[32], b[32], packed[16];
  tmem_ld_32x32(s_taddr, a);
  tmem_ld_wait_for(a);
  tmem_ld_32x32(s_taddr + 32, b);
  weigh<LOG2N, DIAG, 32>(a, kappa, 0, r, la, lb, packed);
  tmem_st_32x16(s_taddr + p_col_of(0), packed);
  tmem_ld_wait_for(b);
  tmem_ld_32x32(s_taddr + 64, a);
  weigh<LOG2N, DIAG, 32>(b, kappa, 32, r, la, lb, packed);
  tmem_st_32x16(s_taddr + p_col_of(32), packed);
  signal_weights(p_half);
  tmem_ld_wait_for(a);
  tmem_ld_32x32(s_taddr + 96, b);
  weigh<LOG2N, DIAG, 32>(a, kappa, 64, r, la, lb, packed);
  tmem_st_32x16(s_taddr + p_col_of(64), packed);
  tmem_ld_wait_for(b);
  weigh<LOG2N, DIAG, 32>(b, kappa, 96, r, la, lb, packed);
  tmem_st_32x16(s_taddr + p_col_of(96), packed);
  signal_weights(p_full);
}

// fp32 rows: the weights go back as two bf16 halves, hi in the first 16 columns of each 32-column
// block of scores and lo in the other 16 (the whole block is overwritten, still after it was read).
template <int LOG2N, bool DIAG>
__device__ __forceinline__ void weigh_tile_hilo(uint32_t s_taddr, int r, float kappa, float2& la, float2& lb,
                                                uint64_t* p_half, uint64_t* p_full) {
  uint32_t a[32], b[32], packed[32];
  tmem_ld_32x32(s_taddr, a);
  tmem_ld_wait_for(a);
  tmem_ld_32x32(s_taddr + 32, b);
  weigh<LOG2N, DIAG, 32, true>(a, kappa, 0, r, la, lb, packed);
  tmem_st_32x32(s_taddr, packed);
  tmem_ld_wait_for(b);
  tmem_ld_32x32(s_taddr + 64, a);
  weigh<LOG2N, DIAG, 32, true>(b, kappa, 32, r, la, lb, packed);
  tmem_st_32x32(s_taddr + 32, packed);
  signal_weights(p_half);
  tmem_ld_wait_for(a);
  tmem_ld_32x32(s_taddr + 96, b);
  weigh<LOG2N, DIAG, 32, true>(a, kappa, 64, r, la, lb, packed);
  tmem_st_32x32(s_taddr + 64, packed);
  tmem_ld_wait_for(b);
  weigh<LOG2N, DIAG, 32, true>(b, kappa, 96, r, la, lb, packed);
  tmem_st_32x32(s_taddr + 96, packed);
  signal_weights(p_full);
}

// The same for a warp that shares its tensor-memory quarter with a second one (`half` 0 or 1): it
// owns S columns [32 half, 32 half + 32) of the tile's first 64 keys and the same block of the
// second 64.  Sixteen columns at a time: a thread has 96 registers here (requesting both blocks
// at once, for more independent chains in flight, spilled and measured 7 % slower).
template <int LOG2N, bool DIAG>
__device__ __forceinline__ void weigh_half_tile(uint32_t s_taddr, int half, int r, float kappa, float2& la, float2& lb,
                                                uint64_t* p_half, uint64_t* p_full) {
  uint32_t a[16], b[16], packed[8];
  const int c0 = 32 * half;
  const uint32_t base = s_taddr + c0;
  tmem_ld_32x16(base, a);
  tmem_ld_wait_for16(a);
  tmem_ld_32x16(base + 16, b);
  weigh<LOG2N, DIAG, 16>(a, kappa, c0, r, la, lb, packed);
  tmem_st_32x8(base, packed);                       // p_col_of(32 half) = 32 half
  tmem_ld_wait_for16(b);
  tmem_ld_32x16(base + 64, a);
  weigh<LOG2N, DIAG, 16>(b, kappa, c0 + 16, r, la, lb, packed);
  tmem_st_32x8(base + 8, packed);
  signal_weights(p_half);
  tmem_ld_wait_for16(a);
  tmem_ld_32x16(base + 80, b);
  weigh<LOG2N, DIAG, 16>(a, kappa, c0 + 64, r, la, lb, packed);
  tmem_st_32x8(base + 64, packed);
  tmem_ld_wait_for16(b);
  weigh<LOG2N, DIAG, 16>(b, kappa, c0 + 80, r, la, lb, packed);
  tmem_st_32x8(base + 72, packed);
  signal_weights(p_full);
}

// Head_dim 64 leaves tensor memory for the weights to have columns of their own (P_w beside S_w instead of
// inside it).  Then S_w can be overwritten by the next tile's scores as soon as this group has READ the
// current ones, which it says through `s_read` after its last load - a quarter of the tile's arithmetic
// before it is done - instead of after the second P.V product has consumed the weights; the wait for the
// next scores, a quarter of a group's time per tile before, all but disappears.  What still orders P_w:
// the first half is only rewritten after "scores there" (which the MMA warp commits behind the first P.V
// product of the previous tile), the second half after `pv_done` of the previous tile.
template <int LOG2N, bool DIAG>
__device__ __forceinline__ bool weigh_half_tile_early(uint32_t s_taddr, uint32_t p_taddr, int half, int r, float kappa, float2& la,
                                                      float2& lb, uint64_t* p_half, uint64_t* p_full, uint64_t* s_read,
                                                      uint64_t* pv_done, bool wait_pv, uint32_t pv_parity, const BoundedWait& bw,
                                                      uint64_t* release_v) {
  uint32_t a[16], b[16], packed[8];
  const int c0 = 32 * half;
  const uint32_t base = s_taddr + c0, pbase = p_taddr + 16 * half;     // weights of S column c sit in P column c / 2
  tmem_ld_32x16(base, a);
  tmem_ld_wait_for16(a);
  tmem_ld_32x16(base + 16, b);
  weigh<LOG2N, DIAG, 16>(a, kappa, c0, r, la, lb, packed);
  tmem_st_32x8(pbase, packed);
  tmem_ld_wait_for16(b);
  tmem_ld_32x16(base + 64, a);
  weigh<LOG2N, DIAG, 16>(b, kappa, c0 + 16, r, la, lb, packed);
  tmem_st_32x8(pbase + 8, packed);
  signal_weights(p_half);
  tmem_ld_wait_for16(a);
  tmem_ld_32x16(base + 80, b);
  weigh<LOG2N, DIAG, 16>(a, kappa, c0 + 64, r, la, lb, packed);
  tmem_ld_wait_for16(b);
  tc_fence_before();
  mbar_arrive(s_read);                              // every score of this tile is in registers
  if (wait_pv && !bw.wait(pv_done, pv_parity)) return false;
  tc_fence_after();
  if (release_v != nullptr) mbar_arrive(release_v); // the previous tile's V is no longer read either
  tmem_st_32x8(pbase + 32, packed);
  weigh<LOG2N, DIAG, 16>(b, kappa, c0 + 80, r, la, lb, packed);
  tmem_st_32x8(pbase + 40, packed);
  signal_weights(p_full);
  return true;
}

// ---- max-shifted form (src/algebraic/kernels/flash.py:235-259): p = (rho(x) rho(-m'))^n with the
// running row maximum m', so that no weight exceeds 1 whatever the inputs.  rho is taken in its
// cancellation-free form: T = |x| + sqrt(1 + x^2) >= 1, rho(x) = T for x >= 0 and 1/T below, which
// costs a reciprocal per score on top of the rsqrt (the MUFU then bounds this form: about twice
// the unshifted time per tile).  Scores are scaled explicitly here (Q is not pre-scaled).

// First pass over a tile: the row's largest score in kernel units (masked entries excluded).
template <bool DIAG>
__device__ __forceinline__ float tile_row_max(uint32_t s_taddr, int r, float scale) {
  uint32_t a[32], b[32];
  float m0 = -3.0e38f, m1 = -3.0e38f, m2 = -3.0e38f, m3 = -3.0e38f;
  auto scan = [&](const uint32_t* s, int col0) {
    if (DIAG && col0 > (r | 31)) return;
#pragma unroll
    for (int i = 0; i < 32; i += 4) {
      float x0 = __uint_as_float(s[i]) * scale, x1 = __uint_as_float(s[i + 1]) * scale;
      float x2 = __uint_as_float(s[i + 2]) * scale, x3 = __uint_as_float(s[i + 3]) * scale;
      if (DIAG) {
        x0 = (col0 + i <= r) ? x0 : -3.0e38f;     x1 = (col0 + i + 1 <= r) ? x1 : -3.0e38f;
        x2 = (col0 + i + 2 <= r) ? x2 : -3.0e38f; x3 = (col0 + i + 3 <= r) ? x3 : -3.0e38f;
      }
      m0 = fmaxf(m0, x0); m1 = fmaxf(m1, x1); m2 = fmaxf(m2, x2); m3 = fmaxf(m3, x3);
    }
  };
  tmem_ld_32x32(s_taddr, a);
  tmem_ld_wait_for(a);
  tmem_ld_32x32(s_taddr + 32, b);
  scan(a, 0);
  tmem_ld_wait_for(b);
  tmem_ld_32x32(s_taddr + 64, a);
  scan(b, 32);
  tmem_ld_wait_for(a);
  tmem_ld_32x32(s_taddr + 96, b);
  scan(a, 64);
  tmem_ld_wait_for(b);
  scan(b, 96);
  return fmaxf(fmaxf(m0, m1), fmaxf(m2, m3));
}

// 32 scores -> 32 shifted weights (rho(x) sigma)^n; NaN scores give NaN weights (as the reference's do).
template <int LOG2N, bool DIAG>
__device__ __forceinline__ void weigh_shifted(const uint32_t* s, float scale, float sigma, int col0, int r, float2& la,
                                              float2& lb, uint32_t* packed) {
  if (DIAG && col0 > (r | 31)) {
#pragma unroll
    for (int i = 0; i < 16; ++i) packed[i] = 0u;
    return;
  }
  const float2 sc = make_float2(scale, scale), one = make_float2(1.f, 1.f), sg = make_float2(sigma, sigma);
#pragma unroll
  for (int i = 0; i < 32; i += 4) {
    const float2 x0 = __fmul2_rn(make_float2(__uint_as_float(s[i]), __uint_as_float(s[i + 1])), sc);
    const float2 x1 = __fmul2_rn(make_float2(__uint_as_float(s[i + 2]), __uint_as_float(s[i + 3])), sc);
    const float2 rad0 = __ffma2_rn(x0, x0, one), rad1 = __ffma2_rn(x1, x1, one);
    const float2 rs0 = make_float2(rsqrt_approx(rad0.x), rsqrt_approx(rad0.y));
    const float2 rs1 = make_float2(rsqrt_approx(rad1.x), rsqrt_approx(rad1.y));
    // T = |x| + sqrt(1 + x^2); an infinite score has rad * rsqrt(rad) = inf * 0: take |x| there
    float2 T0 = __ffma2_rn(rad0, rs0, make_float2(fabsf(x0.x), fabsf(x0.y)));
    float2 T1 = __ffma2_rn(rad1, rs1, make_float2(fabsf(x1.x), fabsf(x1.y)));
    T0.x = (rad0.x < 3.0e38f) ? T0.x : fabsf(x0.x); T0.y = (rad0.y < 3.0e38f) ? T0.y : fabsf(x0.y);
    T1.x = (rad1.x < 3.0e38f) ? T1.x : fabsf(x1.x); T1.y = (rad1.y < 3.0e38f) ? T1.y : fabsf(x1.y);
    float2 t0 = make_float2(x0.x >= 0.f ? T0.x : __fdividef(1.0f, T0.x), x0.y >= 0.f ? T0.y : __fdividef(1.0f, T0.y));
    float2 t1 = make_float2(x1.x >= 0.f ? T1.x : __fdividef(1.0f, T1.x), x1.y >= 0.f ? T1.y : __fdividef(1.0f, T1.y));
    t0 = __fmul2_rn(t0, sg); t1 = __fmul2_rn(t1, sg);
#pragma unroll
    for (int k = 0; k < LOG2N; ++k) { t0 = __fmul2_rn(t0, t0); t1 = __fmul2_rn(t1, t1); }
    if (DIAG) {
      t0.x = (col0 + i <= r) ? t0.x : 0.f;     t0.y = (col0 + i + 1 <= r) ? t0.y : 0.f;
      t1.x = (col0 + i + 2 <= r) ? t1.x : 0.f; t1.y = (col0 + i + 3 <= r) ? t1.y : 0.f;
    }
    la = __fadd2_rn(la, t0);
    lb = __fadd2_rn(lb, t1);
    packed[i >> 1] = pack_bf16(t0.x, t0.y);
    packed[(i >> 1) + 1] = pack_bf16(t1.x, t1.y);
  }
}

// Second pass: the tile's shifted weights, written back as in weigh_tile.
template <int LOG2N, bool DIAG>
__device__ __forceinline__ void weigh_tile_shifted(uint32_t s_taddr, int r, float scale, float sigma, float2& la, float2& lb,
                                                   uint64_t* p_half, uint64_t* p_full) {
  uint32_t a[32], b[32], packed[16];
  tmem_ld_32x32(s_taddr, a);
  tmem_ld_wait_for(a);
  tmem_ld_32x32(s_taddr + 32, b);
  weigh_shifted<LOG2N, DIAG>(a, scale, sigma, 0, r, la, lb, packed);
  tmem_st_32x16(s_taddr + p_col_of(0), packed);
  tmem_ld_wait_for(b);
  tmem_ld_32x32(s_taddr + 64, a);
  weigh_shifted<LOG2N, DIAG>(b, scale, sigma, 32, r, la, lb, packed);
  tmem_st_32x16(s_taddr + p_col_of(32), packed);
  signal_weights(p_half);
  tmem_ld_wait_for(a);
  tmem_ld_32x32(s_taddr + 96, b);
  weigh_shifted<LOG2N, DIAG>(a, scale, sigma, 64, r, la, lb, packed);
  tmem_st_32x16(s_taddr + p_col_of(64), packed);
  tmem_ld_wait_for(b);
  weigh_shifted<LOG2N, DIAG>(b, scale, sigma, 96, r, la, lb, packed);
  tmem_st_32x16(s_taddr + p_col_of(96), packed);
  signal_weights(p_full);
}

// Position in the K/V ring: slot and the parity of how often the ring has wrapped.
template <int NKV> struct RingCursor {
  int slot = 0;
  uint32_t phase = 0;
  __device__ __forceinline__ void next() { if (++slot == NKV) { slot = 0; phase ^= 1u; } }
};

// Which work items a CTA takes, in which order.  Items are numbered heaviest first (last row block
// of every (batch, head), then the one before, ...).  Up to MAX_LISTED items the host deals them
// out greedily - every item, heaviest first, to the CTA with the least work so far - and passes the
// lists as a kernel argument: per-CTA sums then differ by about one key tile, where dealing the items
// out in rows, left to right and back, left 9 % between the lightest and the heaviest CTA at 512
// items over 148 CTAs.  Larger problems use the row-wise deal (many items per CTA level it out).
constexpr int MAX_LISTED = 1024, MAX_LIST_CTAS = 160;
struct ItemLists {
  uint16_t start[MAX_LIST_CTAS + 1];   // CTA c owns item[start[c] .. start[c + 1])
  uint16_t item[MAX_LISTED];
  int listed;                          // 0: row-wise deal
};

// The k-th work item of this CTA.  A listed entry is a 16-bit code: item number (10 bits), part (3 bits) and
// number of parts - 1 (3 bits).  A problem with fewer items than would keep every SM busy has its long items
// SPLIT ALONG THE KEYS into up to eight parts (unshifted form only: there the parts' accumulators and row sums
// simply add up); a part covers a contiguous range of key-tile steps for both query tiles, only the last
// part holds the diagonal tiles (and only it masks), only the first adds the sink, and every part writes
// its raw accumulator and row sums to its own slot of the workspace for attn_split_combine_kernel.
struct Item {
  int b, h, row0, n0, n1;
  int k0;                         // first key tile of this part
  int slot;                       // list position: the part's slot in the workspace
  bool diag, first, partial;
};
// KS = false is the kernel for lists without parts (every problem large enough to fill the GPU): the part
// arithmetic and the partial epilogue are compiled out, which the head_dim-64 kernel with its 96 registers
// per thread notices (5 % at the 125M layer shape).
template <bool KS>
__device__ __forceinline__ bool item_at(const AttnParams& p, const ItemLists& lists, int k, Item& it) {
  const int units = p.B * p.H, nblk = (p.Tq + 2 * BQ - 1) / (2 * BQ), G = int(gridDim.x);
  int idx, part = 0, parts = 1;
  it.slot = 0;
  if (lists.listed) {
    const int at = int(lists.start[blockIdx.x]) + k;
    if (at >= int(lists.start[blockIdx.x + 1])) return false;
    const int code = lists.item[at];
    if (KS) { idx = code & 1023; part = (code >> 10) & 7; parts = ((code >> 13) & 7) + 1; it.slot = at; }
    else idx = code;
  } else {
    // row k of the deal goes left to right for even k and right to left for odd k
    idx = k * G + ((k & 1) ? G - 1 - int(blockIdx.x) : int(blockIdx.x));
    if (idx >= units * nblk) return false;
  }
  const int blk = nblk - 1 - idx / units, bh = idx % units;
  it.b = bh / p.H; it.h = bh % p.H;
  it.row0 = blk * 2 * BQ;
  const int steps = 2 * blk + 2;                 // key tiles needed by query tile 1 (tile 0: one fewer)
  it.k0 = steps * part / parts;
  it.n1 = steps * (part + 1) / parts - it.k0;
  it.diag = part == parts - 1;
  it.n0 = it.diag ? it.n1 - 1 : it.n1;
  it.first = part == 0;
  it.partial = parts > 1;
  return true;
}

// The range guard's three maxima (src/algebraic/kernels/flash.py:834-849) taken by one otherwise idle
// warp while the CTA does its attention work: the largest squared row norm of q in score units, the
// largest squared row norm of k, the largest |v|, each over the rows this CTA looks at (the reader
// takes the largest over the CTAs' records).  A lane owns a row (all of its 16-byte loads in
// flight at once, no shuffles); the rows of the whole problem are dealt over all CTAs.  The
// reference takes the norm of q after re-rounding q / (sqrt(D) c) to the input dtype; here the
// unrounded norm is multiplied by (1 + 2^-8), an upper bound on what that rounding can add, so the
// guard can only err towards the shifted (always valid) form.  NaN anywhere fails the guard.
// Row r of a (B, H, T, D) tensor with strides `st`; 32-bit division where the row count allows (the 64-bit
// one costs more instructions than the row's arithmetic).
__device__ __forceinline__ const uint4* guard_row(const void* base, const Strides3& st, int H, int T, int64_t r, bool narrow) {
  int64_t b;
  int h, t;
  if (narrow) {
    const uint32_t bh = uint32_t(r) / uint32_t(T), bb = bh / uint32_t(H);
    t = int(uint32_t(r) - bh * uint32_t(T)); h = int(bh - bb * uint32_t(H)); b = bb;
  } else {
    const int64_t bh = r / T;
    t = int(r - bh * T); h = int(bh % H); b = bh / H;
  }
  return reinterpret_cast<const uint4*>(static_cast<const __nv_bfloat16*>(base) + b * st.b + h * st.h + int64_t(t) * st.t);
}

template <int D>
__device__ __forceinline__ void guard_statistics(const AttnParams& p, GuardWords* out, int lane) {
  constexpr int NV = D / 8;                       // 16-byte vectors per row
  const int64_t step = int64_t(gridDim.x) * 32;
  const bool narrow = int64_t(p.B) * p.H * max(p.Tq, p.Tk) < (int64_t(1) << 31);
  float best[2] = {0.f, 0.f};
  for (int which = 0; which < 2; ++which) {
    const __nv_bfloat16* base = reinterpret_cast<const __nv_bfloat16*>(which == 0 ? p.q : p.k);
    const Strides3& st = which == 0 ? p.qs : p.ks;
    const int T = which == 0 ? p.Tq : p.Tk;
    const int64_t rows = int64_t(p.B) * p.H * T;
    float m = 0.f;
    for (int64_t r = int64_t(blockIdx.x) * 32 + lane; r < rows; r += step) {
      const uint4* src = guard_row(base, st, p.H, T, r, narrow);
      uint4 raw[NV];
#pragma unroll
      for (int i = 0; i < NV; ++i) raw[i] = __ldg(src + i);
      float2 acc = make_float2(0.f, 0.f);
#pragma unroll
      for (int i = 0; i < NV; ++i) {
        const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&raw[i]);
#pragma unroll
        for (int e = 0; e < 4; ++e) { const float2 f = __bfloat1622float2(h[e]); acc = __ffma2_rn(f, f, acc); }
      }
      const float ss = acc.x + acc.y;
      m = (ss > m || ss != ss) ? ss : m;          // a NaN sticks
    }
    best[which] = m;
  }
  __nv_bfloat162 vm2 = __float2bfloat162_rn(0.f);
  {
    const __nv_bfloat16* base = reinterpret_cast<const __nv_bfloat16*>(p.v);
    const int64_t rows = int64_t(p.B) * p.H * p.Tk;
    for (int64_t r = int64_t(blockIdx.x) * 32 + lane; r < rows; r += step) {
      const uint4* src = guard_row(base, p.vs, p.H, p.Tk, r, narrow);
      uint4 raw[NV];
#pragma unroll
      for (int i = 0; i < NV; ++i) raw[i] = __ldg(src + i);
#pragma unroll
      for (int i = 0; i < NV; ++i) {
        const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&raw[i]);
#pragma unroll
        for (int e = 0; e < 4; ++e) vm2 = __hmax2_nan(vm2, __habs2(h[e]));
      }
    }
  }
  const float2 vm = __bfloat1622float2(vm2);
  float stat[3] = {best[0] * (p.scale * p.scale * 1.00390625f), best[1], (vm.x > vm.y || vm.x != vm.x) ? vm.x : vm.y};
#pragma unroll
  for (int i = 0; i < 3; ++i) {
    float x = stat[i];
    if (!(x == x)) x = __int_as_float(0x7f800000);  // NaN -> +inf, which orders above everything as an unsigned word
    stat[i] = warp_max(x);
  }
  // one record per CTA, plain stores: nothing to zero beforehand, nothing to contend for
  if (lane == 0) *reinterpret_cast<uint4*>(out + blockIdx.x) = make_uint4(__float_as_uint(stat[0]), __float_as_uint(stat[1]), __float_as_uint(stat[2]), 0u);
}

template <int D> constexpr size_t smem_bytes() { return size_t(Cfg<D>::CTL_OFF) + sizeof(Control) + 1024; }
static_assert(smem_bytes<128>() <= 232448 && smem_bytes<64>() <= 232448, "shared memory budget of one CTA");

// The constants of the score scale 1 / (sqrt(D) c) = 2^e m (see the head of the file).
struct ScaleSplit {
  float pow2;      // 2^e: applied to Q in shared memory
  float kappa;     // 1 / m^2
  float inv_mn;    // 1 / m^n: the factor every weight is short of the reference's
};

#ifdef ALG_ATTN_TIMING   // optional instrumentation build: cycle counters written into `stat`
#define ALG_T(acc, expr) [&] { const long long t_ = clock64(); const bool r_ = (expr); acc += clock64() - t_; return r_; }()
#else
#define ALG_T(acc, expr) (expr)
#endif

// F32 (with D = 128, SPLIT = 1, unshifted): head_dim-64 fp32 rows.  q, k, v arrive as bf16 tiles of
// 128 columns, the first 64 the bf16 rounding of the fp32 values (hi) and the other 64 what it left
// over (lo); every product is issued as hi.hi + hi.lo + lo.hi into the same accumulator, for the
// scores and - with the weights split the same way - for the output, which is written as fp32.
template <int D, int LOG2N, int SPLIT, bool SHIFT, bool F32 = false, bool KS = false>
__global__ void __launch_bounds__(nthreads<SPLIT>(), 1)
attn_tc_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_k,
               const __grid_constant__ CUtensorMap tm_v, const __grid_constant__ AttnParams p, const ScaleSplit sc,
               const __grid_constant__ ItemLists lists) {
  using C = Cfg<D>;
  static_assert(!F32 || (D == 128 && SPLIT == 1 && !SHIFT), "the fp32 mode: hi|lo tiles of head_dim 64, unshifted form");
  static_assert(!KS || (!SHIFT && !F32), "items are split along the keys in the unshifted bf16 form only");
  constexpr int DV = F32 ? 64 : D;                  // output columns
  // head_dim 64, unshifted, split weight groups: P_w has tensor-memory columns of its own and S_w is re-issued
  // early (see weigh_half_tile_early); the layout is then S 0..255, P 256..383, O 384..511
  constexpr bool EARLY = (D == 64 && SPLIT == 2 && !SHIFT && !F32);
  constexpr uint32_t O_COL = EARLY ? 384u : C::O_COL;
  constexpr uint32_t P_COL = 256u;                  // EARLY only: P_w at P_COL + 64 w
  extern __shared__ unsigned char smem_raw[];
  unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  Control* ctl = reinterpret_cast<Control*>(smem + C::CTL_OFF);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

  if (warp == 0) {
    griddep_wait();                               // launched as a programmatic dependent: q, k, v and (for a stand-by launch)
                                                  // the guard records come from kernels ahead in the stream
    const bool sh = attn_use_shift(p, lane);
    if (lane == 0) ctl->shift_mode = sh ? 1 : 0;
  }
  __syncthreads();
  // each form runs only when it is the one called for: under a guard the unshifted kernel leaves when the
  // guard failed and the shifted kernel leaves when it held
  if ((ctl->shift_mode != 0) != SHIFT) return;

  if (threadIdx.x == 0) {
    for (int w = 0; w < 2; ++w) { mbar_init(&ctl->q_full[w], 1); mbar_init(&ctl->q_ready[w], 1); mbar_init(&ctl->q_free[w], 1); }
    for (int i = 0; i < C::NKV; ++i) { mbar_init(&ctl->kv_full[i], 1); mbar_init(&ctl->kv_empty[i], 1); }
    for (int w = 0; w < 2; ++w) {
      mbar_init(&ctl->s_full[w], 1);
      mbar_init(&ctl->s_read[w], 128 * SPLIT);
      mbar_init(&ctl->pv_done[w], 1);
      mbar_init(&ctl->p_half[w], 128 * SPLIT);
      mbar_init(&ctl->p_full[w], 128 * SPLIT);
      mbar_init(&ctl->o_full[w], 1);
      mbar_init(&ctl->o_free[w], 128 * SPLIT);
      mbar_init(&ctl->l_part[w], 128);
      mbar_init(&ctl->l_total[w], 128);
    }
    ctl->abort_flag = 0;
   
    fence_barrier_init();
    if (blockIdx.x == 0 && p.stat_kind != nullptr) *p.stat_kind = SHIFT ? ALG_VARIANT_SHIFT : ALG_VARIANT_NOSHIFT;
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

  long long tm0 = 0, tm1 = 0, tm2 = 0;            // timing accumulators (instrumentation build only)
  (void)tm0; (void)tm1; (void)tm2;
  Item it;

  if (warp == 0) {
    if (lane == 0) {
      tma_prefetch_desc(&tm_q); tma_prefetch_desc(&tm_k); tma_prefetch_desc(&tm_v);
      bool ok = true;
      RingCursor<C::NKV> cur;                       // runs on over all items
      for (int k = 0; ok && item_at<KS>(p, lists, k, it); ++k) {
        auto load_kv = [&](int idx) {               // K_0, V_0, K_1, V_1, ... of this item
          const int buf = cur.slot;
          if (!bw.wait(&ctl->kv_empty[buf], cur.phase ^ 1u)) return false;
          mbar_arrive_expect_tx(&ctl->kv_full[buf], C::TILE_BYTES);
          const CUtensorMap* tm = (idx & 1) ? &tm_v : &tm_k;
          for (int pn = 0; pn < C::PANELS; ++pn)
            tma_load_4d(smem + C::KV_OFF + buf * C::TILE_BYTES + pn * PANEL_BYTES, tm, &ctl->kv_full[buf], pn * 64,
                        (it.k0 + (idx >> 1)) * BKEY, it.h, it.b);
          cur.next();
          return true;
        };
        auto load_q = [&](int w) {                  // after the previous item's last S_w has read the tile
          if (k > 0 && !bw.wait(&ctl->q_free[w], (k - 1) & 1u)) return false;
          mbar_arrive_expect_tx(&ctl->q_full[w], C::TILE_BYTES);
          for (int pn = 0; pn < C::PANELS; ++pn)
            tma_load_4d(smem + C::Q_OFF + w * C::TILE_BYTES + pn * PANEL_BYTES, &tm_q, &ctl->q_full[w], pn * 64,
                        it.row0 + w * BQ, it.h, it.b);
          return true;
        };
        // At the start nothing is resident, so what the first MMA needs goes first.  Later the
        // K/V tiles only need ring slots the previous item drains by itself, while each Q tile
        // has to wait for that item's last use of it.
        if (k == 0) ok = load_q(0) && load_kv(0) && load_q(1) && load_kv(1);
        else ok = load_kv(0) && load_q(0) && load_kv(1) && load_q(1);
        for (int idx = 2; idx < 2 * it.n1 && ok; ++idx) ok = load_kv(idx);
      }
    }
  } else if (warp == 1) {
    // The MMA warp.  Its own instruction time is the scarce resource: an issue costs the issuing
    // thread 30 to 50 cycles (the lower figure when the whole warp runs the loop and one elected
    // lane issues, as here) and a commit about 90, against 64 cycles of tensor-pipe time per
    // 128x128x16 product.  So it commits only what nobody else can signal (scores ready, output
    // ready); the K/V slots and the Q tiles are released by the weight warps, which learn of an
    // MMA's completion through those same two barriers.  Serving the two query tiles in turn also
    // keeps their weight groups half a step apart, so that one evaluates while the other's
    // products run.
    const uint32_t q_addr = smem_u32(smem + C::Q_OFF), kv_addr = smem_u32(smem + C::KV_OFF);
    using Cur = RingCursor<C::NKV>;
    Cur cur;                                        // the next K/V tile in ring order, over all items
    int t0 = 0, t1 = 0;                             // score tiles of query tile 0 / 1 in earlier items
    auto wait_all = [&](uint64_t* bar, uint32_t parity) { return __all_sync(0xffffffffu, bw.wait(bar, parity)) != 0; };
    auto kv_wait = [&](const Cur& c) { return wait_all(&ctl->kv_full[c.slot], c.phase); };
    // descriptor low halves: Q tiles and ring slot 0 as K (K-major, LBO 16) and as V (MN-major,
    // LBO = one panel); a slot adds slot * TILE_BYTES / 16, a K step adds a constant
    const uint32_t q_lo0 = sw128_desc_lo(q_addr, 16), k_lo0 = sw128_desc_lo(kv_addr, 16),
                   v_lo0 = sw128_desc_lo(kv_addr, PANEL_BYTES);
#ifdef ALG_ATTN_TIMING
    long long tm3 = 0;
#define ALG_TI0 const long long ti_ = clock64();
#define ALG_TI1 tm3 += clock64() - ti_;
#else
#define ALG_TI0
#define ALG_TI1
#endif
    auto issue_s = [&](int w, int slot) {           // S_w = Q_w K^T
      ALG_TI0
      const uint32_t qa = q_lo0 + w * (C::TILE_BYTES >> 4), ka = k_lo0 + slot * (C::TILE_BYTES >> 4);
      const uint32_t d_tmem = tmem_base + C::S_COL + w * 128;
      if constexpr (F32) {                         // q_hi.k_hi + q_hi.k_lo + q_lo.k_hi: panel 0 holds hi, panel 1 lo
        constexpr uint32_t LO = PANEL_BYTES >> 4;
#pragma unroll
        for (int g = 0; g < 3; ++g) {
          const uint32_t qo = (g == 2) ? LO : 0u, ko = (g == 1) ? LO : 0u;
#pragma unroll
          for (int ks = 0; ks < 4; ++ks)
            umma_f16_ss_parts(d_tmem, qa + qo + ((ks * 32) >> 4), SW128_DESC_HI, ka + ko + ((ks * 32) >> 4), SW128_DESC_HI, C::IDESC_S,
                              (g != 0 || ks != 0) ? 1u : 0u);
        }
      } else {
#pragma unroll
        for (int ks = 0; ks < D / 16; ++ks) {
          const uint32_t off = ((ks >> 2) * PANEL_BYTES + (ks & 3) * 32) >> 4;
          umma_f16_ss_parts(d_tmem, qa + off, SW128_DESC_HI, ka + off, SW128_DESC_HI, C::IDESC_S, ks != 0 ? 1u : 0u);
        }
      }
      ALG_TI1
    };
    // O_w += P_w V for the first (h64 = 0) or second 64 keys of the tile, P_w from tensor memory
    auto issue_pv = [&](int w, int slot, int h64, bool first) {
      ALG_TI0
      const uint32_t va = v_lo0 + slot * (C::TILE_BYTES >> 4);
      const uint32_t d_tmem = tmem_base + O_COL + w * D;
      const uint32_t p_tmem = EARLY ? tmem_base + P_COL + w * 64 : tmem_base + C::S_COL + w * 128;
      if constexpr (F32) {                         // p_hi.v_hi + p_lo.v_hi + p_hi.v_lo; p_lo sits 16 columns behind p_hi
        constexpr uint32_t LO = PANEL_BYTES >> 4;
#pragma unroll
        for (int g = 0; g < 3; ++g) {
          const uint32_t po = (g == 1) ? 16u : 0u, vo = (g == 2) ? LO : 0u;
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            const int ks = 4 * h64 + i;
            umma_f16_ts_parts(d_tmem, p_tmem + p_col_of(16 * ks) + po, va + vo + ks * (2048 >> 4), SW128_DESC_HI, C::IDESC_PV64,
                              (first && ks == 0 && g == 0) ? 0u : 1u);
          }
        }
      } else {
#pragma unroll
        for (int i = 0; i < 4; ++i) {               // 16 keys = 8 packed-bf16 columns of P per step
          const int ks = 4 * h64 + i;
          umma_f16_ts_parts(d_tmem, p_tmem + (EARLY ? uint32_t(8 * ks) : p_col_of(16 * ks)), va + ks * (2048 >> 4), SW128_DESC_HI,
                            C::IDESC_PV, (first && ks == 0) ? 0u : 1u);
        }
      }
      ALG_TI1
    };
#ifdef ALG_ATTN_TIMING
    const long long t_begin = clock64();
#endif
    bool ok = true;
    for (int k = 0; ok && item_at<KS>(p, lists, k, it); ++k) {
      const int n0 = it.n0, n1 = it.n1;
      if (!wait_all(&ctl->q_ready[0], k & 1u) || !kv_wait(cur)) { ok = false; break; }
      tc_fence_after();
      if (elect_one()) { issue_s(0, cur.slot); umma_commit(&ctl->s_full[0]); }
      __syncwarp();
      if (!wait_all(&ctl->q_ready[1], k & 1u)) { ok = false; break; }
      tc_fence_after();
      if (elect_one()) { issue_s(1, cur.slot); umma_commit(&ctl->s_full[1]); }
      __syncwarp();
      cur.next();
      for (int j = 0; j < n1 && ok; ++j) {
        const Cur vc = cur;                         // V_j
        cur.next();
        const Cur kc = cur;                         // K_{j+1}: only meaningful while j + 1 < n1
        if (j + 1 < n1) cur.next();
        // Both tiles of this step are waited for up front (they are normally long there), so
        // that nothing stands between "weights ready" and the issue of P.V and the next S.
        if (!ALG_T(tm0, kv_wait(vc)) || (j + 1 < n1 && !ALG_T(tm0, kv_wait(kc)))) { ok = false; break; }
        if constexpr (EARLY) {
          // per query tile: first P.V half, then the NEXT scores as soon as the current ones have been read,
          // then the second P.V half (announced by itself: the weight warps order their writes to P_w by it)
          bool fine = true;
#pragma unroll
          for (int w = 0; w < 2 && fine; ++w) {
            const int nw = w == 0 ? n0 : n1, tw = w == 0 ? t0 : t1;
            if (j >= nw) continue;
            if (!ALG_T(tm1, wait_all(&ctl->p_half[w], (tw + j) & 1u))) { fine = false; break; }
            if (j == 0 && k > 0 && !wait_all(&ctl->o_free[w], (k - 1) & 1u)) { fine = false; break; }
            tc_fence_after();
            if (elect_one()) issue_pv(w, vc.slot, 0, j == 0);
            __syncwarp();
            if (j + 1 < nw) {
              if (!ALG_T(tm2, wait_all(&ctl->s_read[w], (tw + j) & 1u))) { fine = false; break; }
              tc_fence_after();
              if (elect_one()) { issue_s(w, kc.slot); umma_commit(&ctl->s_full[w]); }
              __syncwarp();
            }
            if (!ALG_T(tm1, wait_all(&ctl->p_full[w], (tw + j) & 1u))) { fine = false; break; }
            tc_fence_after();
            if (elect_one()) {
              issue_pv(w, vc.slot, 1, false);
              umma_commit(&ctl->pv_done[w]);
              if (j + 1 == nw) umma_commit(&ctl->o_full[w]);
            }
            __syncwarp();
          }
          if (!fine) { ok = false; break; }
          continue;
        }
        if (j < n0) {
          if (!ALG_T(tm1, wait_all(&ctl->p_half[0], (t0 + j) & 1u))) { ok = false; break; }
          // the first product of an item overwrites O_0: the previous output must have been read
          if (j == 0 && k > 0 && !wait_all(&ctl->o_free[0], (k - 1) & 1u)) { ok = false; break; }
          tc_fence_after();
          if (elect_one()) issue_pv(0, vc.slot, 0, j == 0);
          __syncwarp();
          if (!ALG_T(tm1, wait_all(&ctl->p_full[0], (t0 + j) & 1u))) { ok = false; break; }
          tc_fence_after();
          if (elect_one()) {
            issue_pv(0, vc.slot, 1, false);
            if (j + 1 < n0) { issue_s(0, kc.slot); umma_commit(&ctl->s_full[0]); }   // after P_0.V: may overwrite P_0
            else umma_commit(&ctl->o_full[0]);
          }
          __syncwarp();
        }
        if (!ALG_T(tm2, wait_all(&ctl->p_half[1], (t1 + j) & 1u))) { ok = false; break; }
        if (j == 0 && k > 0 && !wait_all(&ctl->o_free[1], (k - 1) & 1u)) { ok = false; break; }
        tc_fence_after();
        if (elect_one()) issue_pv(1, vc.slot, 0, j == 0);
        __syncwarp();
        if (!ALG_T(tm2, wait_all(&ctl->p_full[1], (t1 + j) & 1u))) { ok = false; break; }
        tc_fence_after();
        if (elect_one()) {
          issue_pv(1, vc.slot, 1, false);
          if (j + 1 < n1) { issue_s(1, kc.slot); umma_commit(&ctl->s_full[1]); }
          else umma_commit(&ctl->o_full[1]);
        }
        __syncwarp();
      }
      t0 += n0; t1 += n1;
    }
#ifdef ALG_ATTN_TIMING
    if (blockIdx.x == 0 && lane == 0 && p.stat != nullptr) {
      float* dbg = p.stat + 16;
      dbg[0] = float(tm0); dbg[1] = float(tm1); dbg[2] = float(tm2); dbg[3] = float(clock64() - t_begin); dbg[4] = float(tm3);
    }
#endif
  } else if (warp == 2) {
    // Q scaler: once a Q tile has landed, multiply it by 2^e where it lies (element-wise, so
    // the swizzled layout does not matter), make the result visible to the tensor core's reads
    // and release the tile to the MMA warp.
    const __nv_bfloat162 f2 = __float2bfloat162_rn(sc.pow2);
    bool ok = true;
    for (int k = 0; ok && item_at<KS>(p, lists, k, it); ++k) {
      for (int w = 0; w < 2 && ok; ++w) {
        if (!bw.wait(&ctl->q_full[w], k & 1u)) { ok = false; break; }
        if (sc.pow2 != 1.0f) {
          uint4* tile = reinterpret_cast<uint4*>(smem + C::Q_OFF + w * C::TILE_BYTES);
#pragma unroll 4
          for (int i = lane; i < C::TILE_BYTES / 16; i += 32) {
            uint4 v = tile[i];
            __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&v);
            h[0] = __hmul2(h[0], f2); h[1] = __hmul2(h[1], f2); h[2] = __hmul2(h[2], f2); h[3] = __hmul2(h[3], f2);
            tile[i] = v;
          }
          fence_async_shared();
        }
        __syncwarp();
        if (lane == 0) mbar_arrive(&ctl->q_ready[w]);
      }
    }
  } else if (warp == 3) {
#ifdef ALG_ATTN_TIMING
    const long long tg0 = clock64();
#endif
    if (p.guard_out != nullptr) guard_statistics<D>(p, p.guard_out, lane);
#ifdef ALG_ATTN_TIMING
    if (lane == 0 && p.stat != nullptr) p.stat[40 + 2 * blockIdx.x] = float(clock64() - tg0);
#endif
  } else {
    const int ww = warp - FIRST_WEIGHT_WARP;
    const int w = ww / (4 * SPLIT);                 // query tile of this weight group
    const int half = (ww >> 2) & (SPLIT - 1);       // which 32-column blocks (split groups)
    const int quarter = warp & 3;                   // TMEM lanes 32*quarter.. are this warp's
    const int r = quarter * 32 + lane;              // row inside the query tile
    const uint32_t lane_sel = uint32_t(quarter * 32) << 16;
    const uint32_t s_taddr = tmem_base + lane_sel + C::S_COL + w * 128;
    bool ok = true;
    int tiles_before = 0;                           // score tiles of this group in earlier items
    // One thread per group passes on what the arrival of scores implies.  The tensor pipe runs the
    // MMA thread's instructions in order, so "S_w(j) is there" means every product issued before it
    // has finished reading its operands: for query tile 1 (served second in every step) that is all
    // of step j - 1, hence V_{j-1} and K_j can be overwritten; for either tile, the last scores of
    // an item mean its Q tile can be.  The releasing thread walks the K/V ring in load order.
    const bool releaser = (ww % (4 * SPLIT)) == 0 && lane == 0;
    RingCursor<C::NKV> rel;
    // EARLY: K and V slots are released at different moments, so each has its own position in the ring
    // (loads go K_0 V_0 K_1 V_1 ...: the K slots are every other one from 0, the V slots from 1)
    int kslot = 0, vslot = 1 % C::NKV;
    const uint32_t p_taddr = tmem_base + lane_sel + P_COL + w * 64;
#ifdef ALG_ATTN_TIMING
    const long long t_begin = clock64();
#endif
    for (int k = 0; ok && item_at<KS>(p, lists, k, it); ++k) {
      const int nk = (w == 0) ? it.n0 : it.n1;
      const int last_masked = (!KS || it.diag) ? nk - 1 : -1; // the tile that holds this query tile's diagonal (last part of an item only)
      float l = 0.f;                                // the sink's weight, fetched while the first scores are computed
      float m_run = -1.0e30f;                       // shifted form: running row maximum (kernel units) ...
      if (p.sink != nullptr && (!KS || it.first)) {
        if (SHIFT) { m_run = p.sink[it.h] * p.inv_c; l = 1.0f; }   // ... which starts at the sink, whose weight under its own shift is 1
        else l = pow2n<LOG2N>(rho_stable(p.sink[it.h] * p.inv_c)) * sc.inv_mn;
      }
      float2 la = make_float2(0.f, 0.f), lb = make_float2(0.f, 0.f);
      for (int j = 0; j < nk && ok; ++j) {
        if (!ALG_T(tm0, bw.wait(&ctl->s_full[w], (tiles_before + j) & 1u))) { ok = false; break; }
        tc_fence_after();
        if (releaser) {
          if (w == 1) {
            if (EARLY) {                                                         // K_j; V_{j-1} follows at pv_done
              mbar_arrive(&ctl->kv_empty[kslot]); kslot = (kslot + 2) % C::NKV;
            } else {
              if (j > 0) { mbar_arrive(&ctl->kv_empty[rel.slot]); rel.next(); }  // V_{j-1}
              mbar_arrive(&ctl->kv_empty[rel.slot]); rel.next();                 // K_j
            }
          }
          if (j == nk - 1) mbar_arrive(&ctl->q_free[w]);
        }
#ifdef ALG_ATTN_TIMING
        const long long tc0 = clock64();
#endif
        if (SHIFT) {
          // pass 1: the tile's row maximum; then the rescale factor of what has been accumulated so far
          const float tmax = (j == last_masked) ? tile_row_max<true>(s_taddr, r, p.scale) : tile_row_max<false>(s_taddr, r, p.scale);
          const float m_new = fmaxf(m_run, tmax);
          if (j == 0 && p.sink == nullptr) m_run = m_new;          // without a sink the first tile sets the maximum
          const float sigma = rho_stable(-m_new);
          const float alpha = pow2n<LOG2N>(rho_stable(m_run) * sigma);
          // O_w of the earlier tiles is at rest (S_w(j) complete means P_w(j-1).V complete): rescale it in
          // tensor memory where some row's maximum moved; an unchanged row multiplies by exactly 1
          const bool moved = j > 0 && alpha != 1.0f;
          if (__any_sync(0xffffffffu, moved)) {
            const float a_row = (j > 0) ? alpha : 1.0f;
#pragma unroll 1
            for (int chunk = 0; chunk < D / 32; ++chunk) {
              uint32_t o[32];
              const uint32_t o_taddr = tmem_base + lane_sel + C::O_COL + w * D + chunk * 32;
              tmem_ld_32x32(o_taddr, o);
              tmem_ld_wait_for(o);
#pragma unroll
              for (int i = 0; i < 32; ++i) o[i] = __float_as_uint(__uint_as_float(o[i]) * a_row);
              tmem_st_32x32(o_taddr, o);
            }
            tmem_st_wait();
          }
          l *= alpha;                                      // sink and earlier tiles, now relative to the new maximum
          m_run = m_new;
          if (j == last_masked) weigh_tile_shifted<LOG2N, true>(s_taddr, r, p.scale, sigma, la, lb, &ctl->p_half[w], &ctl->p_full[w]);
          else weigh_tile_shifted<LOG2N, false>(s_taddr, r, p.scale, sigma, la, lb, &ctl->p_half[w], &ctl->p_full[w]);
          l += (la.x + la.y) + (lb.x + lb.y);              // this tile's weights
          la = make_float2(0.f, 0.f); lb = make_float2(0.f, 0.f);
        } else if (EARLY) {
          const int tile = tiles_before + j;               // this group's tiles, counted over all items
          // V_{j-1} of this item goes back to the ring once its second P.V product is done (the item's last V
          // tile waits for "output ready" below)
          uint64_t* release_v = (releaser && w == 1 && j > 0) ? &ctl->kv_empty[vslot] : nullptr;
          if (release_v != nullptr) vslot = (vslot + 2) % C::NKV;
          if (j == last_masked) ok = weigh_half_tile_early<LOG2N, true>(s_taddr, p_taddr, half, r, sc.kappa, la, lb, &ctl->p_half[w], &ctl->p_full[w],
                                                                   &ctl->s_read[w], &ctl->pv_done[w], tile > 0, uint32_t(tile - 1) & 1u, bw, release_v);
          else ok = weigh_half_tile_early<LOG2N, false>(s_taddr, p_taddr, half, r, sc.kappa, la, lb, &ctl->p_half[w], &ctl->p_full[w],
                                                        &ctl->s_read[w], &ctl->pv_done[w], tile > 0, uint32_t(tile - 1) & 1u, bw, release_v);
        } else if (SPLIT == 2) {
          if (j == last_masked) weigh_half_tile<LOG2N, true>(s_taddr, half, r, sc.kappa, la, lb, &ctl->p_half[w], &ctl->p_full[w]);   // diagonal tile: masked
          else weigh_half_tile<LOG2N, false>(s_taddr, half, r, sc.kappa, la, lb, &ctl->p_half[w], &ctl->p_full[w]);
        } else if (F32) {
          if (j == last_masked) weigh_tile_hilo<LOG2N, true>(s_taddr, r, sc.kappa, la, lb, &ctl->p_half[w], &ctl->p_full[w]);
          else weigh_tile_hilo<LOG2N, false>(s_taddr, r, sc.kappa, la, lb, &ctl->p_half[w], &ctl->p_full[w]);
        } else {
          if (j == last_masked) weigh_tile<LOG2N, true>(s_taddr, r, sc.kappa, la, lb, &ctl->p_half[w], &ctl->p_full[w]);
          else weigh_tile<LOG2N, false>(s_taddr, r, sc.kappa, la, lb, &ctl->p_half[w], &ctl->p_full[w]);
        }
#ifdef ALG_ATTN_TIMING
        tm1 += clock64() - tc0;
#endif
      }
      tiles_before += nk;
      float part = (la.x + la.y) + (lb.x + lb.y);
      if (SPLIT == 2 && half == 1) {                // row sums of the two column halves meet in shared memory:
        ctl->row_sum[w][r] = part;                  // half 1 hands its partial to half 0 ...
        mbar_arrive(&ctl->l_part[w]);
      }
      if (!ok || !bw.wait(&ctl->o_full[w], k & 1u)) { ok = false; break; }
      if (releaser && w == 1) {                                                        // the item's last V tile
        if (EARLY) { mbar_arrive(&ctl->kv_empty[vslot]); vslot = (vslot + 2) % C::NKV; }
        else { mbar_arrive(&ctl->kv_empty[rel.slot]); rel.next(); }
      }
      if (SPLIT == 2) {
        if (half == 0) {                            // ... which returns the row's total through the same word
          if (!bw.wait(&ctl->l_part[w], k & 1u)) { ok = false; break; }
          part += ctl->row_sum[w][r];
          ctl->row_sum[w][r] = part;
          mbar_arrive(&ctl->l_total[w]);
        } else {
          if (!bw.wait(&ctl->l_total[w], k & 1u)) { ok = false; break; }
          part = ctl->row_sum[w][r];
        }
      }
      tc_fence_after();
      item_at<KS>(p, lists, k, it);                            // recomputed: nothing of it stays live over the tile loop
      l += part;                                    // shifted form: the last tile's sums (already at the final maximum)
      const float inv = 1.0f / l;
      const int row = it.row0 + w * BQ + r;
      const int64_t o_off = it.b * p.os.b + it.h * p.os.h + int64_t(row) * p.os.t;
      __nv_bfloat16* orow = reinterpret_cast<__nv_bfloat16*>(p.o) + o_off;
      constexpr int CHUNKS = DV / 32 / SPLIT;        // a split group divides the output columns as well
#pragma unroll 1
      for (int chunk = half * CHUNKS; chunk < (half + 1) * CHUNKS; ++chunk) {
        uint32_t o[32];
        tmem_ld_32x32(tmem_base + lane_sel + O_COL + w * D + chunk * 32, o);
        tmem_ld_wait_for(o);
        if (chunk == (half + 1) * CHUNKS - 1) {     // O_w is in registers: the next item may overwrite it
          tc_fence_before();
          mbar_arrive(&ctl->o_free[w]);
        }
        if (KS && it.partial) {                      // one part of a split item: the raw accumulator, for the combine kernel
          float* dst = p.split_ws + (int64_t(it.slot) * 2 * BQ + w * BQ + r) * (DV + 4) + chunk * 32;
#pragma unroll
          for (int c = 0; c < 8; ++c)
            *reinterpret_cast<uint4*>(dst + 4 * c) = make_uint4(o[4 * c], o[4 * c + 1], o[4 * c + 2], o[4 * c + 3]);
          continue;
        }
        if (row >= p.Tq) continue;                   // a row past the end of a sequence that does not fill its last tile
        if constexpr (F32) {
          float* frow = reinterpret_cast<float*>(p.o) + o_off + chunk * 32;
#pragma unroll
          for (int c = 0; c < 8; ++c)
            *reinterpret_cast<float4*>(frow + 4 * c) = make_float4(__uint_as_float(o[4 * c]) * inv, __uint_as_float(o[4 * c + 1]) * inv,
                                                                   __uint_as_float(o[4 * c + 2]) * inv, __uint_as_float(o[4 * c + 3]) * inv);
        } else {
#pragma unroll
          for (int c = 0; c < 4; ++c) {
            uint4 val;
            val.x = pack_bf16(__uint_as_float(o[8 * c + 0]) * inv, __uint_as_float(o[8 * c + 1]) * inv);
            val.y = pack_bf16(__uint_as_float(o[8 * c + 2]) * inv, __uint_as_float(o[8 * c + 3]) * inv);
            val.z = pack_bf16(__uint_as_float(o[8 * c + 4]) * inv, __uint_as_float(o[8 * c + 5]) * inv);
            val.w = pack_bf16(__uint_as_float(o[8 * c + 6]) * inv, __uint_as_float(o[8 * c + 7]) * inv);
            *reinterpret_cast<uint4*>(orow + chunk * 32 + c * 8) = val;
          }
        }
      }
      if (KS && it.partial) {                        // its row sums (the sink's weight included by the first part)
        if (half == 0) p.split_ws[(int64_t(it.slot) * 2 * BQ + w * BQ + r) * (DV + 4) + DV] = l;
        continue;
      }
#ifndef ALG_ATTN_TIMING
      // unshifted: 1 / l of the reference = 1 / (l' m^n); shifted: rho(-m) l^(-1/n)  (flash.py:271-284)
      if (p.stat != nullptr && half == 0 && row < p.Tq)
        p.stat[(int64_t(it.b) * p.H + it.h) * p.Tq + row] = SHIFT ? rho_stable(-m_run) * inv_root_rt(l, LOG2N) : inv * sc.inv_mn;
#endif
    }
#ifdef ALG_ATTN_TIMING
    if (w == 1 && r == 0 && half == 0 && p.stat != nullptr) p.stat[41 + 2 * blockIdx.x] = float(clock64() - t_begin);
    if (blockIdx.x == 0 && r == 0 && half == 0 && p.stat != nullptr) {
      float* dbg = p.stat + 8 * w;
      dbg[0] = float(tm0); dbg[1] = 0.f; dbg[2] = float(tm1); dbg[3] = float(clock64() - t_begin); dbg[4] = float(tiles_before);
    }
#endif
  }

  tc_fence_before();
  __syncthreads();
  if (ctl->abort_flag != 0) {
    if (threadIdx.x == 0) {
      if (p.status != nullptr) atomicExch(p.status, ALG_DEV_TIMEOUT);
      const uint64_t t0 = global_timer_ns();       // let issued loads land before shared memory is released
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

// Greedy deal (every entry, heaviest first, to the CTA with the least work so far) of the items, or of the
// parts of items when the problem is short: cost of row block blk = its 4 blk + 3 score tiles.  `split`: a
// problem whose heaviest item is well above a CTA's fair share of the work may have its long items cut along the
// keys (item_at says how a part reads its range), at most eight parts per item.  A part writes its fp32
// accumulator (132 KB at head_dim 128) and the combine kernel reads it back, as much traffic as four key-tile
// steps load: measured, parts of 4 to 8 steps made every short problem slower ((1,16,2048,128): 36 -> 82 us), so
// a part is at least MIN_PART_TILES score tiles (16 steps) long and sequences up to 2048 are never split.  The
// part size is chosen by trying a few and dealing each: the estimate is the heaviest CTA's tiles plus what the
// parts' traffic and the second kernel cost (in tiles; fitted to (1,2,8192,128): 113 -> 85 us with 160 parts of
// 32 tiles), and the unsplit deal stays when it is not beaten.  Returns the number of list entries that are parts.
constexpr int MIN_PART_TILES = 32, MAX_SPLIT_ENTRIES = 512;
struct DealEntry { int cost; uint16_t code; };

// the entries for parts of about `target` tiles (0: whole items); returns their number, or -1 if they do not fit
int deal_entries(DealEntry* entry, int units, int nblk, int target, int* parts_total) {
  const int items = units * nblk;
  int entries = 0;
  *parts_total = 0;
  for (int i = 0; i < items; ++i) {
    const int blk = nblk - 1 - i / units, cost = 4 * blk + 3, steps = 2 * blk + 2;
    int parts = 1;
    if (target > 0 && cost > target) {
      parts = (cost + target - 1) / target;
      if (parts > 8) parts = 8;
      if (parts > steps / 2) parts = steps / 2;
    }
    if (entries + parts > (target > 0 ? MAX_SPLIT_ENTRIES : MAX_LISTED)) return -1;
    for (int pt = 0; pt < parts; ++pt) {
      const int k0 = steps * pt / parts, k1 = steps * (pt + 1) / parts;
      entry[entries].cost = 2 * (k1 - k0) - (pt == parts - 1 ? 1 : 0);
      entry[entries].code = uint16_t(i | (pt << 10) | ((parts - 1) << 13));
      ++entries;
    }
    if (parts > 1) *parts_total += parts;
  }
  if (*parts_total > 0)                                  // parts are lighter than whole items of the same row block: restore the order
    std::stable_sort(entry, entry + entries, [](const DealEntry& a, const DealEntry& b) { return a.cost > b.cost; });
  return entries;
}

// deal `entries` over `grid` CTAs; returns the heaviest CTA's load
int deal_greedy(const DealEntry* entry, int entries, int grid, uint16_t* owner, int* count) {
  int load[MAX_LIST_CTAS] = {0};
  for (int c = 0; c < grid; ++c) count[c] = 0;
  int worst = 0;
  for (int i = 0; i < entries; ++i) {
    int best = 0;
    for (int c = 1; c < grid; ++c)
      if (load[c] < load[best]) best = c;
    owner[i] = uint16_t(best);
    load[best] += entry[i].cost;
    ++count[best];
    if (load[best] > worst) worst = load[best];
  }
  return worst;
}

int deal_items(ItemLists* out, int units, int nblk, int grid, bool split) {
  const int items = units * nblk;
  out->listed = 0;
  if (items > MAX_LISTED || grid > MAX_LIST_CTAS) return 0;
  static thread_local DealEntry entry[MAX_LISTED];
  static thread_local uint16_t owner[MAX_LISTED];
  int count[MAX_LIST_CTAS];
  long total = 0;
  for (int i = 0; i < items; ++i) total += 4 * (nblk - 1 - i / units) + 3;
  const int share = int((total + grid - 1) / grid), heaviest = 4 * (nblk - 1) + 3;
  int best_target = 0, parts_total = 0;
  if (split && 2 * heaviest > 3 * share) {
    int entries = deal_entries(entry, units, nblk, 0, &parts_total);
    int best_score = deal_greedy(entry, entries, grid, owner, count);
    for (int target = MIN_PART_TILES; target < heaviest; target += (target < 64 ? 8 : (target < 128 ? 16 : 64))) {
      entries = deal_entries(entry, units, nblk, target, &parts_total);
      if (entries < 0 || parts_total == 0) continue;
      const int score = deal_greedy(entry, entries, grid, owner, count) + parts_total / 10 + 6;
      if (score < best_score) { best_score = score; best_target = target; }
    }
  }
  const int entries = deal_entries(entry, units, nblk, best_target, &parts_total);
  deal_greedy(entry, entries, grid, owner, count);
  out->start[0] = 0;
  for (int c = 0; c < grid; ++c) out->start[c + 1] = uint16_t(out->start[c] + count[c]);
  int fill[MAX_LIST_CTAS];
  for (int c = 0; c < grid; ++c) fill[c] = out->start[c];
  for (int i = 0; i < entries; ++i) out->item[fill[owner[i]]++] = entry[i].code;
  out->listed = 1;
  return parts_total;
}

// The deal depends on four integers only: keep the last few (a launch path must stay cheap, and a call asks
// twice - once for the workspace size, with splitting, once at the launch, with or without).
struct Dealt { int units, nblk, grid, split, parts; ItemLists lists; };
const Dealt& dealt_for(int units, int nblk, int grid, bool split) {
  constexpr int KEPT = 16;
  static thread_local Dealt kept[KEPT];
  static thread_local int used = 0, next = 0;
  for (int i = 0; i < used; ++i)
    if (kept[i].units == units && kept[i].nblk == nblk && kept[i].grid == grid && kept[i].split == int(split)) return kept[i];
  Dealt& d = kept[next];
  next = (next + 1) % KEPT;
  if (used < KEPT) ++used;
  d.units = units; d.nblk = nblk; d.grid = grid; d.split = int(split);
  d.parts = deal_items(&d.lists, units, nblk, grid, split);
  return d;
}

// Adds up the parts of every split item: out = (sum of accumulators) / (sum of row sums), the statistic 1 / l.
// Grid (list entries, 8): the entry that is part 0 of a split item does the item's work, every other entry
// leaves at once; a CTA takes 32 of the item's 256 rows, a warp four of them, a lane DV / 32 columns of a row, and
// all of a warp's loads are issued before any is used (a thread per row walking its parts one load latency at a
// time made this kernel as long as the attention it finishes).
template <int DV>
__global__ void __launch_bounds__(256) attn_split_combine_kernel(const __grid_constant__ ItemLists lists, const AttnParams p, int entries,
                                                                 float inv_mn) {
  griddep_wait();                                        // a programmatic dependent of the attention kernel
  __shared__ int slots[8];
  const int code = lists.item[blockIdx.x];
  const int idx = code & 1023, parts = ((code >> 13) & 7) + 1;
  if (((code >> 10) & 7) != 0 || parts == 1) return;
  for (int i = threadIdx.x; i < entries; i += blockDim.x) {
    const int c = lists.item[i];
    if ((c & 1023) == idx && ((c >> 13) & 7) + 1 == parts) slots[(c >> 10) & 7] = i;
  }
  __syncthreads();
  constexpr int CPL = DV / 32;                           // columns per lane
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int units = p.B * p.H, nblk = (p.Tq + 2 * BQ - 1) / (2 * BQ);
  const int blk = nblk - 1 - idx / units, bh = idx % units, b = bh / p.H, h = bh % p.H;
  const int in_item0 = blockIdx.y * 32 + warp * 4;       // this warp's first row inside the item (query tile = row / 128)
  float acc[4][CPL], l[4];
#pragma unroll
  for (int rr = 0; rr < 4; ++rr) {
    l[rr] = 0.f;
#pragma unroll
    for (int c = 0; c < CPL; ++c) acc[rr][c] = 0.f;
  }
  for (int pt = 0; pt < parts; ++pt) {
    const float* base = p.split_ws + (int64_t(slots[pt]) * 2 * BQ + in_item0) * (DV + 4);
    float v[4][CPL], lv[4];
#pragma unroll
    for (int rr = 0; rr < 4; ++rr) {
      const float* row = base + rr * (DV + 4);
      if (CPL == 4) {
        const float4 x = __ldcg(reinterpret_cast<const float4*>(row + lane * 4));
        v[rr][0] = x.x; v[rr][1] = x.y; v[rr][CPL - 2] = x.z; v[rr][CPL - 1] = x.w;
      } else {
        const float2 x = __ldcg(reinterpret_cast<const float2*>(row + lane * 2));
        v[rr][0] = x.x; v[rr][1] = x.y;
      }
      lv[rr] = __ldcg(row + DV);
    }
#pragma unroll
    for (int rr = 0; rr < 4; ++rr) {
      l[rr] += lv[rr];
#pragma unroll
      for (int c = 0; c < CPL; ++c) acc[rr][c] += v[rr][c];
    }
  }
#pragma unroll
  for (int rr = 0; rr < 4; ++rr) {
    const int row = blk * 2 * BQ + in_item0 + rr;
    if (row >= p.Tq) continue;
    const float inv = 1.0f / l[rr];
    __nv_bfloat16* orow = reinterpret_cast<__nv_bfloat16*>(p.o) + b * p.os.b + h * p.os.h + int64_t(row) * p.os.t;
    if (CPL == 4)
      *reinterpret_cast<uint2*>(orow + lane * 4) = make_uint2(pack_bf16(acc[rr][0] * inv, acc[rr][1] * inv),
                                                              pack_bf16(acc[rr][CPL - 2] * inv, acc[rr][CPL - 1] * inv));
    else
      *reinterpret_cast<uint32_t*>(orow + lane * 2) = pack_bf16(acc[rr][0] * inv, acc[rr][1] * inv);
    if (p.stat != nullptr && lane == 0) p.stat[(int64_t(b) * p.H + h) * p.Tq + row] = inv * inv_mn;
  }
}

int make_qkv_map(CUtensorMap* tm, const void* base, const Strides3& s, int B, int H, int T, int D) {
  const uint64_t dims[4] = {uint64_t(D), uint64_t(T), uint64_t(H), uint64_t(B)};
  const uint64_t strides[3] = {uint64_t(s.t), uint64_t(s.h), uint64_t(s.b)};
  const uint32_t box[4] = {64, 128, 1, 1};
  return make_tmap_bf16(tm, base, 4, dims, strides, box, true);
}

template <int D, int LOG2N, int SPLIT, bool SHIFT, bool F32, bool KS>
int launch_kernel(const CUtensorMap& tq, const CUtensorMap& tk, const CUtensorMap& tv, const AttnParams& p, const ScaleSplit& sc,
                  const ItemLists& lists, int grid, cudaStream_t stream) {
  auto kern = attn_tc_kernel<D, LOG2N, SPLIT, SHIFT, F32, KS>;
  static PerDeviceOnce configured;
  if (int rc = configured.run([&] { return cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, int(smem_bytes<D>())); })) return rc;
  ALG_CUDA_TRY(launch_dependent(kern, dim3(grid), dim3(nthreads<SPLIT>()), smem_bytes<D>(), stream, tq, tk, tv, p, sc, lists));
  return ALG_OK;
}

template <int D, int LOG2N, int SPLIT, bool SHIFT, bool F32 = false>
int launch_dns(const AttnParams& p, cudaStream_t stream) {
  CUtensorMap tq, tk, tv;
  if (int rc = make_qkv_map(&tq, p.q, p.qs, p.B, p.H, p.Tq, D)) return rc;
  if (int rc = make_qkv_map(&tk, p.k, p.ks, p.B, p.H, p.Tk, D)) return rc;
  if (int rc = make_qkv_map(&tv, p.v, p.vs, p.B, p.H, p.Tk, D)) return rc;
  // 1 / (sqrt(D) c) = 2^e m with 1 <= m < 2
  ScaleSplit sc;
  {
    int ex = 0;
    const double f = frexp(double(p.scale), &ex);         // scale = f 2^ex, 0.5 <= f < 1
    const double m = 2.0 * f;
    sc.pow2 = float(ldexp(1.0, ex - 1));
    sc.kappa = float(1.0 / (m * m));
    sc.inv_mn = float(pow(m, -double(1 << LOG2N)));
    if (SHIFT) { sc.pow2 = 1.0f; sc.kappa = 1.0f; sc.inv_mn = 1.0f; }   // the shifted form scales its scores itself
  }
  const int grid = attn_tcgen05_grid(p);
  const int units = p.B * p.H, nblk = (p.Tq + 2 * BQ - 1) / (2 * BQ);
  // short problems: long items are cut along the keys when the caller's workspace has room for the parts' slots
  static const bool never_split = getenv("ALG_ATTN_NO_KEY_SPLIT") != nullptr;      // measurement aid
  const bool may_split = !SHIFT && !F32 && p.split_ws != nullptr && !never_split;
  const Dealt* dealt = &dealt_for(units, nblk, grid, may_split);
  if (dealt->parts > 0 && int(dealt->lists.start[grid]) > p.split_slots) dealt = &dealt_for(units, nblk, grid, false);
  if constexpr (!SHIFT && !F32) {
    if (dealt->parts > 0) {
      if (int rc = launch_kernel<D, LOG2N, SPLIT, SHIFT, F32, true>(tq, tk, tv, p, sc, dealt->lists, grid, stream)) return rc;
    } else if (int rc = launch_kernel<D, LOG2N, SPLIT, SHIFT, F32, false>(tq, tk, tv, p, sc, dealt->lists, grid, stream)) return rc;
  } else if (int rc = launch_kernel<D, LOG2N, SPLIT, SHIFT, F32, false>(tq, tk, tv, p, sc, dealt->lists, grid, stream)) return rc;
  if (dealt->parts > 0) {
    const int entries = int(dealt->lists.start[grid]);
    ALG_CUDA_TRY(launch_dependent(attn_split_combine_kernel<D>, dim3(entries, 8), dim3(256), 0, stream, dealt->lists, p, entries, sc.inv_mn));
    count_launch();
  }
  count_launch();
  return ALG_OK;
}

// How many warps weigh a score tile.  Four (one per tensor-memory quarter) are fastest at head_dim
// 128, where the tensor pipe has as much to do per tile as the weight warps; eight (two per
// quarter, half the key columns each) are 10 to 14 % faster at head_dim 64, where the weights
// dominate.  ALG_ATTN_SPLIT = 1 or 2 in the environment overrides the choice (measurement aid).
template <int D, int LOG2N>
int launch_dn(const AttnParams& p, cudaStream_t stream) {
  static const int forced = [] { const char* e = getenv("ALG_ATTN_SPLIT"); return e != nullptr ? atoi(e) : 0; }();
  if (p.tc_shift) return launch_dns<D, LOG2N, 1, true>(p, stream);     // one thread sees its whole row of a tile
  const int split = forced == 1 || forced == 2 ? forced : (D == 64 ? 2 : 1);
  return split == 1 ? launch_dns<D, LOG2N, 1, false>(p, stream) : launch_dns<D, LOG2N, 2, false>(p, stream);
}

template <int D>
int launch_d(const AttnParams& p, cudaStream_t stream) {
  switch (p.log2n) {
    case 3: return launch_dn<D, 3>(p, stream);
    case 4: return launch_dn<D, 4>(p, stream);
    case 5: return launch_dn<D, 5>(p, stream);
  }
  set_error("attention (tcgen05): n must be 8, 16 or 32");
  return ALG_ERR_UNSUPPORTED;
}

// ---- fp32 rows (head_dim 64): split into bf16 hi | lo tiles of 128 columns ---------------------
// x (B, H, T, 64) fp32 with strides -> y (B, H, T, 128) bf16 dense: y[.., j] = bf16(x[.., j]) and
// y[.., 64 + j] = bf16(x[.., j] - y[.., j]).  hi + lo carries 16 bits of the mantissa, and the three
// products hi.hi + hi.lo + lo.hi reproduce an fp32 product to about 2^-16 (src/algebraic/kernels/
// flash.py computes its fp32 path in fp32; the parity bar for fp32 I/O is rel-L2 1e-3).
struct SplitJob { const float* x; __nv_bfloat16* y; Strides3 xs; int T; };
struct SplitBatch { SplitJob t[3]; int B, H; };

__global__ void __launch_bounds__(256) split_f32_kernel(const SplitBatch batch) {
  griddep_wait();
  const SplitJob& job = batch.t[blockIdx.y];
  const int64_t vecs = int64_t(batch.B) * batch.H * job.T * 16;       // float4 pieces: 16 per row
  for (int64_t i = int64_t(blockIdx.x) * blockDim.x + threadIdx.x; i < vecs; i += int64_t(gridDim.x) * blockDim.x) {
    const int piece = int(i & 15);
    const int64_t row = i >> 4;
    const int t = int(row % job.T);
    const int64_t bh = row / job.T;
    const float4 v = *reinterpret_cast<const float4*>(job.x + (bh / batch.H) * job.xs.b + (bh % batch.H) * job.xs.h + int64_t(t) * job.xs.t + piece * 4);
    const uint32_t h0 = pack_bf16(v.x, v.y), h1 = pack_bf16(v.z, v.w);
    const uint32_t l0 = pack_bf16(v.x - __uint_as_float(h0 << 16), v.y - __uint_as_float(h0 & 0xffff0000u));
    const uint32_t l1 = pack_bf16(v.z - __uint_as_float(h1 << 16), v.w - __uint_as_float(h1 & 0xffff0000u));
    __nv_bfloat16* out = job.y + row * 128 + piece * 4;
    *reinterpret_cast<uint2*>(out) = make_uint2(h0, h1);
    *reinterpret_cast<uint2*>(out + 64) = make_uint2(l0, l1);
  }
}

}  // namespace

size_t attn_tcgen05_f32_split_bytes(int B, int H, int T) { return size_t(B) * H * T * 128 * sizeof(__nv_bfloat16); }

bool attn_tcgen05_f32_supports(const AttnParams& p, int dtype) {
  return dtype == ALG_F32 && p.causal && p.Tq == p.Tk && p.Tq >= 1 && p.D == 64 && p.log2n >= 3 && p.log2n <= 5;
}

// p describes the fp32 problem (q, k, v, o fp32 with their strides); `split` holds three buffers of
// attn_tcgen05_f32_split_bytes each.  Unshifted form only (under a guard the kernel leaves when the
// guard calls for the shift, like the bf16 one).
int launch_attn_tcgen05_f32(const AttnParams& p, void* split, cudaStream_t stream) {
  const size_t each = attn_tcgen05_f32_split_bytes(p.B, p.H, p.Tq);
  unsigned char* base = static_cast<unsigned char*>(split);
  SplitBatch batch{};
  batch.B = p.B; batch.H = p.H;
  batch.t[0] = {static_cast<const float*>(p.q), reinterpret_cast<__nv_bfloat16*>(base), p.qs, p.Tq};
  batch.t[1] = {static_cast<const float*>(p.k), reinterpret_cast<__nv_bfloat16*>(base + each), p.ks, p.Tk};
  batch.t[2] = {static_cast<const float*>(p.v), reinterpret_cast<__nv_bfloat16*>(base + 2 * each), p.vs, p.Tk};
  const int64_t vecs = int64_t(p.B) * p.H * p.Tq * 16;
  int64_t blocks = (vecs + 255) / 256;
  if (blocks > int64_t(sm_count()) * 8) blocks = int64_t(sm_count()) * 8;
  ALG_CUDA_TRY(launch_dependent(split_f32_kernel, dim3(unsigned(blocks), 3), dim3(256), 0, stream, batch));
  count_launch();
  AttnParams ps = p;
  ps.q = batch.t[0].y; ps.k = batch.t[1].y; ps.v = batch.t[2].y;
  const Strides3 dense = {int64_t(p.H) * p.Tq * 128, int64_t(p.Tq) * 128, 128};
  ps.qs = dense; ps.ks = dense; ps.vs = dense;
  ps.guard_out = nullptr;
  switch (p.log2n) {
    case 3: return launch_dns<128, 3, 1, false, true>(ps, stream);
    case 4: return launch_dns<128, 4, 1, false, true>(ps, stream);
    case 5: return launch_dns<128, 5, 1, false, true>(ps, stream);
  }
  set_error("attention (tcgen05): n must be 8, 16 or 32");
  return ALG_ERR_UNSUPPORTED;
}

bool attn_tcgen05_supports(const AttnParams& p, int dtype) {
  const bool strides_fit = p.qs.t > 0 && p.ks.t > 0 && p.vs.t > 0 && p.qs.h >= 0 && p.qs.b >= 0 &&
                           p.ks.h >= 0 && p.ks.b >= 0 && p.vs.h >= 0 && p.vs.b >= 0;
  return dtype == ALG_BF16 && p.causal && p.Tq == p.Tk && p.Tq >= 1 && (p.D == 64 || p.D == 128) &&
         p.log2n >= 3 && p.log2n <= 5 && strides_fit &&
         (p.B == 1 || p.qs.b > 0) && (p.H == 1 || p.qs.h > 0);
}

// One warp per SM streams 6 B H T D bytes at about 5 GB/s per SM while the kernel needs time in
// proportion to B H T^2 D: from T D = 3/4 Mi elements per head on, the statistics are ready well
// before the attention is (T >= 6144 at head_dim 128).
// One CTA per SM; a problem with fewer items than that still gets up to eight CTAs per item, because its long
// items may be split along the keys (a CTA whose list stays empty leaves at once).
int attn_tcgen05_grid(const AttnParams& p) {
  const int64_t items = int64_t(p.B) * p.H * ((p.Tq + 2 * BQ - 1) / (2 * BQ));
  const int sms = sm_count();
  return int(items * 8 < sms ? items * 8 : sms);
}

size_t attn_tcgen05_split_bytes(const AttnParams& p) {
  if (p.D != 64 && p.D != 128) return 0;
  const int units = p.B * p.H, nblk = (p.Tq + 2 * BQ - 1) / (2 * BQ), grid = attn_tcgen05_grid(p);
  const Dealt& d = dealt_for(units, nblk, grid, true);
  return d.parts > 0 ? size_t(d.lists.start[grid]) * 2 * BQ * (p.D + 4) * sizeof(float) : 0;
}

bool attn_tcgen05_takes_guard_statistics(const AttnParams& p) { return int64_t(p.Tq) * p.D >= 786432; }

int launch_attn_tcgen05(const AttnParams& p, cudaStream_t stream) {
  return p.D == 64 ? launch_d<64>(p, stream) : launch_d<128>(p, stream);
}

}  // namespace alg
