// QK RMS-normalisation, Cayley rotation and the range-guard maxima in one HBM-bound pass.
//
// One 16-byte vector per lane, D*sizeof(T)/16 lanes per row, so a warp streams whole
// rows with fully coalesced 128-bit loads and stores.  A warp owns a few positions (b, t)
// and walks over the heads, four heads per step with all four loads issued before any is
// used (memory-level parallelism), so the rotation table row of a position is loaded once
// and reused for every head.  The rotate-half partner of an element lives in lane ^
// (lanes_per_row/2) and is fetched with one shuffle.  Up to three tensors (q, k, v) are
// processed by one launch (blockIdx.y selects the tensor).
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
  using Raw = float4;
  static __device__ __forceinline__ Raw load(const float* p) { return *reinterpret_cast<const float4*>(p); }
  static __device__ __forceinline__ void unpack(const Raw& r, float* v) { v[0] = r.x; v[1] = r.y; v[2] = r.z; v[3] = r.w; }
  static __device__ __forceinline__ void store(float* p, const float* v) {
    *reinterpret_cast<float4*>(p) = make_float4(v[0], v[1], v[2], v[3]);
  }
  static __device__ __forceinline__ float round(float x) { return x; }
};
template <> struct Vec16<__nv_bfloat16> {
  static constexpr int N = 8;
  using Raw = uint4;
  static __device__ __forceinline__ Raw load(const __nv_bfloat16* p) { return *reinterpret_cast<const uint4*>(p); }
  static __device__ __forceinline__ void unpack(const Raw& r, float* v) {
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
  static __device__ __forceinline__ float round(float x) { return __bfloat162float(__float2bfloat16_rn(x)); }
};


// MODE 0: statistics only (guard maxima of ready-made q / k / v); 1: normalise (+ gain);
// 2: normalise + rotate.  Modes 1 and 2 can also accumulate a statistic in the same pass.
template <typename T, int D, int MODE>
__global__ void __launch_bounds__(256, MODE == 0 ? 4 : 3) qk_prep_kernel(const PrepBatch batch) {
  using V = Vec16<T>;
  constexpr int VEC = V::N;
  constexpr int LPR = D / VEC;         // lanes per row
  constexpr int RPW = 32 / LPR;        // positions per warp step
  constexpr int HALF = D / 2;
  // 16-byte loads kept in flight per lane.  Eight of them at three CTAs per SM put about 100 KB
  // per SM in flight, which is what 6.5 TB/s needs at the loaded memory latency (with four the
  // normalising pass stopped at 5.0 TB/s; with eight it reaches 5.4).
  constexpr int HEADS_PER_STEP = 8;
  const PrepParams& p = batch.t[blockIdx.y];
  const int lane = threadIdx.x & 31;
  const int lir = lane % LPR;          // lane in row
  const int sub = lane / LPR;
  const int64_t positions = int64_t(p.B) * p.T;
  const int64_t warp_global = (int64_t(blockIdx.x) * blockDim.x + threadIdx.x) >> 5;
  const int64_t warps_total = (int64_t(gridDim.x) * blockDim.x) >> 5;
  const bool first = lir < LPR / 2;
  const int j0 = (lir % (LPR / 2)) * VEC;

  float gain[VEC];
  if constexpr (MODE >= 1) {
#pragma unroll
    for (int i = 0; i < VEC; ++i) gain[i] = (p.gain != nullptr) ? p.gain[lir * VEC + i] : 1.0f;
  }

  float stat = 0.0f;
  for (int64_t g0 = warp_global * RPW; g0 < positions; g0 += warps_total * RPW) {
    const int64_t pos = g0 + sub;
    const bool live = pos < positions;
    const int64_t pp = live ? pos : positions - 1;
    const int t = int(pp % p.T);
    const int64_t b = pp / p.T;
    const T* src0 = reinterpret_cast<const T*>(p.x) + b * p.xs.b + int64_t(t) * p.xs.t + lir * VEC;
    T* dst0 = (MODE >= 1 && p.y != nullptr) ? reinterpret_cast<T*>(p.y) + b * p.ys.b + int64_t(t) * p.ys.t + lir * VEC : nullptr;

    float c[VEC], s[VEC];              // this position's table row, cast to T, signed for the half
    uint32_t c2[VEC / 2], s2[VEC / 2]; // the same as packed bf16 pairs (bf16 rows only)
    if constexpr (MODE == 2 && sizeof(T) == 2) {
#pragma unroll
      for (int i = 0; i < VEC; i += 4) {
        const float4 cv = *reinterpret_cast<const float4*>(p.cos + int64_t(t) * HALF + j0 + i);
        const float4 sv = *reinterpret_cast<const float4*>(p.sin + int64_t(t) * HALF + j0 + i);
        c2[i / 2] = pack_bf16(cv.x, cv.y); c2[i / 2 + 1] = pack_bf16(cv.z, cv.w);
        s2[i / 2] = pack_bf16(sv.x, sv.y); s2[i / 2 + 1] = pack_bf16(sv.z, sv.w);
      }
      if (first) {                       // the first half subtracts x2 s: flip both sign bits
#pragma unroll
        for (int i = 0; i < VEC / 2; ++i) s2[i] ^= 0x80008000u;
      }
    } else if constexpr (MODE == 2) {
#pragma unroll
      for (int i = 0; i < VEC; i += 4) {
        const float4 cv = *reinterpret_cast<const float4*>(p.cos + int64_t(t) * HALF + j0 + i);
        const float4 sv = *reinterpret_cast<const float4*>(p.sin + int64_t(t) * HALF + j0 + i);
        c[i] = V::round(cv.x); c[i + 1] = V::round(cv.y); c[i + 2] = V::round(cv.z); c[i + 3] = V::round(cv.w);
        s[i] = V::round(sv.x); s[i + 1] = V::round(sv.y); s[i + 2] = V::round(sv.z); s[i + 3] = V::round(sv.w);
      }
      if (first) {                       // the first half subtracts x2 s
#pragma unroll
        for (int i = 0; i < VEC; ++i) s[i] = -s[i];
      }
    }

    for (int h0 = 0; h0 < p.H; h0 += HEADS_PER_STEP) {
      typename V::Raw raw[HEADS_PER_STEP];
#pragma unroll
      for (int u = 0; u < HEADS_PER_STEP; ++u) {
        const int h = min(h0 + u, p.H - 1);
        raw[u] = V::load(src0 + int64_t(h) * p.xs.h);
      }
#pragma unroll
      for (int u = 0; u < HEADS_PER_STEP; ++u) {
        const int h = h0 + u;
        const bool on = live && h < p.H;         // uniform per lane group; shuffles below stay warp-wide
        float v[VEC];
        V::unpack(raw[u], v);
        if constexpr (MODE >= 1) {
          float2 ss2 = make_float2(0.0f, 0.0f);        // two elements per instruction on the packed fp32 pipe
#pragma unroll
          for (int i = 0; i < VEC; i += 2) { const float2 x2 = make_float2(v[i], v[i + 1]); ss2 = __ffma2_rn(x2, x2, ss2); }
          float ss = ss2.x + ss2.y;
#pragma unroll
          for (int o = LPR / 2; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
          const float tau = rsqrtf(ss * (1.0f / D) + p.eps);
          const float2 tau2 = make_float2(tau, tau);
          if constexpr (MODE == 2 && sizeof(T) == 2) {
            // bf16 rows.  The reference rotates in bf16 arithmetic (each product and the sum rounded
            // to bf16), which is what HMUL2 / HADD2 compute, two elements per instruction; a pair
            // also travels to its rotate-half partner lane as one 32-bit shuffle.
            uint32_t yp[VEC / 2];
#pragma unroll
            for (int i = 0; i < VEC / 2; ++i) {
              const float2 sc2 = __fmul2_rn(__fmul2_rn(make_float2(v[2 * i], v[2 * i + 1]), tau2), make_float2(gain[2 * i], gain[2 * i + 1]));
              const uint32_t own = pack_bf16(sc2.x, sc2.y);
              const uint32_t oth = __shfl_xor_sync(0xffffffffu, own, LPR / 2);
              // first half: x1 c - x2 s ; second half: x2 c + x1 s  ==  own * c + other * (-+ s)
              const __nv_bfloat162 y = __hadd2(__hmul2(*reinterpret_cast<const __nv_bfloat162*>(&own), *reinterpret_cast<const __nv_bfloat162*>(&c2[i])),
                                               __hmul2(*reinterpret_cast<const __nv_bfloat162*>(&oth), *reinterpret_cast<const __nv_bfloat162*>(&s2[i])));
              yp[i] = *reinterpret_cast<const uint32_t*>(&y);
            }
            if (dst0 != nullptr && on)
              *reinterpret_cast<uint4*>(dst0 + int64_t(h) * p.ys.h) = make_uint4(yp[0], yp[1], yp[2], yp[3]);
            if (p.stat_mode != 0) {          // the statistic below wants the written values
#pragma unroll
              for (int i = 0; i < VEC / 2; ++i) {
                v[2 * i] = __uint_as_float(yp[i] << 16);
                v[2 * i + 1] = __uint_as_float(yp[i] & 0xffff0000u);
              }
            }
          } else {
#pragma unroll
            for (int i = 0; i < VEC; i += 2) {
              const float2 sc2 = __fmul2_rn(__fmul2_rn(make_float2(v[i], v[i + 1]), tau2), make_float2(gain[i], gain[i + 1]));
              v[i] = V::round(sc2.x); v[i + 1] = V::round(sc2.y);
            }
          }
        }
        if constexpr (MODE == 2 && sizeof(T) != 2) {
#pragma unroll
          for (int i = 0; i < VEC; ++i) {
            // fp32 rows: own * c + other * (-+ s), s[] carrying the sign of this half
            const float o = __shfl_xor_sync(0xffffffffu, v[i], LPR / 2);
            v[i] = v[i] * c[i] + o * s[i];
          }
        }
        if (MODE >= 1 && !(MODE == 2 && sizeof(T) == 2) && dst0 != nullptr && on) V::store(dst0 + int64_t(h) * p.ys.h, v);
        if (p.stat_mode == 1) {          // squared row norm of the re-rounded scaled row
          float ss = 0.0f;
#pragma unroll
          for (int i = 0; i < VEC; ++i) {
            const float sc = V::round(v[i] * p.stat_scale);
            ss = fmaf(sc, sc, ss);
          }
#pragma unroll
          for (int o = LPR / 2; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
          if (on) stat = fmaxf(stat, ss);
        } else if (p.stat_mode == 2) {   // max |x|
          float m = 0.0f;
#pragma unroll
          for (int i = 0; i < VEC; ++i) m = fmaxf(m, fabsf(v[i]));
          if (on) stat = fmaxf(stat, m);
        }
      }
    }
  }
  if (p.stat_mode != 0) {                     // one atomic per block: warp max -> block max -> global
    __shared__ float s_stat[8];
    stat = warp_max(stat);
    // NaN inputs must fail the guard: map NaN to +inf before the integer max.
    if (!(stat == stat)) stat = __int_as_float(0x7f800000);
    if (lane == 0) s_stat[threadIdx.x >> 5] = stat;
    __syncthreads();
    if (threadIdx.x == 0) {
      float m = s_stat[0];
      for (int w = 1; w < int(blockDim.x >> 5); ++w) m = fmaxf(m, s_stat[w]);
      atomicMax(p.stat_out, __float_as_uint(m));
    }
  }
}

template <typename T, int D>
static int launch_t(const PrepBatch& batch, cudaStream_t stream) {
  // every tensor of a batch runs the same mode (the callers group them that way)
  const int mode = !batch.t[0].normalise ? 0 : (batch.t[0].cos != nullptr ? 2 : 1);
  for (int i = 1; i < batch.count; ++i) {
    const int m = !batch.t[i].normalise ? 0 : (batch.t[i].cos != nullptr ? 2 : 1);
    if (m != mode) { set_error("internal: mixed modes in one prep batch"); return ALG_ERR_INVALID; }
  }
  constexpr int LPR = D * int(sizeof(T)) / 16;
  constexpr int RPW = 32 / LPR;
  int64_t positions = 0;
  for (int i = 0; i < batch.count; ++i) {
    const int64_t n = int64_t(batch.t[i].B) * batch.t[i].T;
    if (n > positions) positions = n;
    if (batch.t[i].H == 0) return ALG_OK;
  }
  if (positions == 0) return ALG_OK;
  const int threads = 256;
  const int64_t warps = (positions + RPW - 1) / RPW;
  int64_t blocks = (warps + threads / 32 - 1) / (threads / 32);
  // resident CTAs only (the grid-stride loop covers the rest): 4 per SM for the
  // statistics-only mode, 3 for the others, per tensor of the launch (sharing one wave among
  // the tensors measured slightly slower)
  const int64_t cap = int64_t(sm_count()) * (mode == 0 ? 4 : 3);
  if (blocks > cap) blocks = cap;
  const dim3 grid(unsigned(blocks), unsigned(batch.count));
  if (mode == 0) qk_prep_kernel<T, D, 0><<<grid, threads, 0, stream>>>(batch);
  else if (mode == 1) qk_prep_kernel<T, D, 1><<<grid, 256, 0, stream>>>(batch);
  else qk_prep_kernel<T, D, 2><<<grid, 256, 0, stream>>>(batch);
  ALG_CUDA_TRY(cudaGetLastError());
  count_launch();
  return ALG_OK;
}

int launch_prep_batch(const PrepBatch& batch, int dtype, cudaStream_t stream) {
  if (batch.count < 1 || batch.count > 3) {
    set_error("internal: prep batch of %d tensors", batch.count);
    return ALG_ERR_INVALID;
  }
  const int D = batch.t[0].D;
  if (D != 64 && D != 128) {
    set_error("QK prologue needs head_dim 64 or 128, got %d", D);
    return ALG_ERR_UNSUPPORTED;
  }
  if (dtype == ALG_BF16)
    return D == 64 ? launch_t<__nv_bfloat16, 64>(batch, stream) : launch_t<__nv_bfloat16, 128>(batch, stream);
  if (dtype == ALG_F32) return D == 64 ? launch_t<float, 64>(batch, stream) : launch_t<float, 128>(batch, stream);
  set_error("unknown dtype %d", dtype);
  return ALG_ERR_INVALID;
}

int launch_prep(const PrepParams& p, int dtype, cudaStream_t stream) {
  PrepBatch batch{};
  batch.t[0] = p;
  batch.count = 1;
  return launch_prep_batch(batch, dtype, stream);
}

// ---- backward of the QK RMS-norm --------------------------------------------------------------
// y = x tau g with tau = rsqrt(mean(x^2) + eps).  With u = g dy (all in fp32, one rounding to the
// I/O dtype at the end):
//   dx      = tau (u - x tau^2 mean(u x))        the input gradient of src/algebraic/algebraic.py:76-83
//   dgain_j = sum over rows of dy_j x_j tau      src/algebraic/kernels/qk_norm.py:20-26
// The reference reduces the gain gradient in row blocks and sums the block partials afterwards
// (qk_norm.py:47-56); here every CTA writes one partial row and a second kernel adds the rows in
// block order, so the result does not depend on scheduling.  Same lane layout as the forward pass.
constexpr int RMS_BWD_BLOCKS = 1024;    // rows of scratch: an upper bound on the CTAs of one launch
int rms_bwd_max_blocks() { return RMS_BWD_BLOCKS; }

template <typename T, int D>
__global__ void __launch_bounds__(256, 3) qk_rms_bwd_kernel(const RmsBwdParams p) {
  using V = Vec16<T>;
  constexpr int VEC = V::N;
  constexpr int LPR = D / VEC;         // lanes per row
  constexpr int RPW = 32 / LPR;        // rows per warp step
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int lir = lane % LPR, sub = lane / LPR;
  const int64_t rows = int64_t(p.B) * p.H * p.T;
  const int64_t warp_global = (int64_t(blockIdx.x) * blockDim.x + threadIdx.x) >> 5;
  const int64_t warps_total = (int64_t(gridDim.x) * blockDim.x) >> 5;
  float g[VEC], dg[VEC];
#pragma unroll
  for (int i = 0; i < VEC; ++i) {
    g[i] = (p.gain != nullptr) ? p.gain[lir * VEC + i] : 1.0f;
    dg[i] = 0.f;
  }
  // Four row groups per step, all eight 16-byte loads issued before any is used (memory-level parallelism).
  // A step of a warp covers U * RPW CONSECUTIVE rows: where they all lie in one (batch, head) - the rule - the
  // row -> (batch, head, position) arithmetic is done once per step for the whole warp and a row's three
  // offsets are one multiply-add each.  (With one division chain per row group the kernel executed 196
  // warp instructions per row-group lane, nearly half of them addressing, and ran at 52 % issue
  // utilisation: instruction-bound as much as HBM-bound.)
  constexpr int U = 4;
  constexpr int STEP_ROWS = U * RPW;
  const bool narrow = rows < (int64_t(1) << 31);
  for (int64_t base = warp_global * STEP_ROWS; base < rows; base += warps_total * STEP_ROWS) {
    typename V::Raw rx[U], rd[U];
    int64_t off_dx[U];
    bool alive[U];
    // position of the step's first row (warp-uniform)
    int64_t bh0, b0;
    int t0, h0;
    if (narrow) {                      // 32-bit division where the row count allows
      const uint32_t q1 = uint32_t(base) / uint32_t(p.T), q2 = q1 / uint32_t(p.H);
      bh0 = q1; t0 = int(uint32_t(base) - q1 * uint32_t(p.T)); b0 = q2; h0 = int(q1 - q2 * uint32_t(p.H));
    } else {
      bh0 = base / p.T; t0 = int(base - bh0 * p.T); h0 = int(bh0 % p.H); b0 = bh0 / p.H;
    }
    const bool one_head = t0 + STEP_ROWS <= p.T;
    const int64_t x0 = b0 * p.xs.b + h0 * p.xs.h + int64_t(t0) * p.xs.t + lir * VEC;
    const int64_t g0 = b0 * p.gs.b + h0 * p.gs.h + int64_t(t0) * p.gs.t + lir * VEC;
    const int64_t d0 = b0 * p.ds.b + h0 * p.ds.h + int64_t(t0) * p.ds.t + lir * VEC;
#pragma unroll
    for (int u = 0; u < U; ++u) {
      const int in_step = u * RPW + sub;
      const int64_t row = base + in_step;
      alive[u] = row < rows;
      int64_t ox, og, od;
      if (one_head) {
        ox = x0 + int64_t(in_step) * p.xs.t;
        og = g0 + int64_t(in_step) * p.gs.t;
        od = d0 + int64_t(in_step) * p.ds.t;
      } else {                         // the step straddles a (batch, head) boundary or the end: per-row arithmetic
        const int64_t rr = alive[u] ? row : rows - 1;
        const int t = int(rr % p.T);
        const int64_t bh = rr / p.T;
        const int h = int(bh % p.H);
        const int64_t b = bh / p.H;
        ox = b * p.xs.b + h * p.xs.h + int64_t(t) * p.xs.t + lir * VEC;
        og = b * p.gs.b + h * p.gs.h + int64_t(t) * p.gs.t + lir * VEC;
        od = b * p.ds.b + h * p.ds.h + int64_t(t) * p.ds.t + lir * VEC;
      }
      rx[u] = V::load(reinterpret_cast<const T*>(p.x) + ox);
      rd[u] = V::load(reinterpret_cast<const T*>(p.dy) + og);
      off_dx[u] = od;
    }
#pragma unroll
    for (int u = 0; u < U; ++u) {
    const bool live = alive[u];
    float x[VEC], d[VEC];
    V::unpack(rx[u], x);
    V::unpack(rd[u], d);
    // two elements per instruction on the packed fp32 pipe: this kernel is bound by its instruction count
    // as much as by HBM (one thread per 16 bytes of each stream)
    float2 gd[VEC / 2];
    float2 ss2 = make_float2(0.f, 0.f), su2 = make_float2(0.f, 0.f);
#pragma unroll
    for (int i = 0; i < VEC / 2; ++i) {
      const float2 xi = make_float2(x[2 * i], x[2 * i + 1]);
      gd[i] = __fmul2_rn(make_float2(g[2 * i], g[2 * i + 1]), make_float2(d[2 * i], d[2 * i + 1]));
      ss2 = __ffma2_rn(xi, xi, ss2);
      su2 = __ffma2_rn(gd[i], xi, su2);
    }
    float ss = ss2.x + ss2.y, su = su2.x + su2.y;
#pragma unroll
    for (int o = LPR / 2; o > 0; o >>= 1) {
      ss += __shfl_xor_sync(0xffffffffu, ss, o);
      su += __shfl_xor_sync(0xffffffffu, su, o);
    }
    const float tau = rsqrtf(ss * (1.0f / D) + p.eps);
    const float coef = tau * tau * su * (1.0f / D);
    const float2 ncoef2 = make_float2(-coef, -coef), tau2 = make_float2(live ? tau : 0.f, live ? tau : 0.f);
    float out[VEC];
#pragma unroll
    for (int i = 0; i < VEC / 2; ++i) {
      const float2 xi = make_float2(x[2 * i], x[2 * i + 1]);
      const float2 o2 = __fmul2_rn(__ffma2_rn(xi, ncoef2, gd[i]), make_float2(tau, tau));     // tau (g dy - x coef)
      out[2 * i] = o2.x; out[2 * i + 1] = o2.y;
      float2 dg2 = make_float2(dg[2 * i], dg[2 * i + 1]);
      dg2 = __ffma2_rn(__fmul2_rn(make_float2(d[2 * i], d[2 * i + 1]), xi), tau2, dg2);       // a dead row adds d x 0
      dg[2 * i] = dg2.x; dg[2 * i + 1] = dg2.y;
    }
    if (live) V::store(reinterpret_cast<T*>(p.dx) + off_dx[u], out);
    }
  }
  if (p.dgain == nullptr) return;
  // the rows a warp handled side by side, then the warps of the CTA, in a fixed order
#pragma unroll
  for (int i = 0; i < VEC; ++i)
    for (int o = LPR; o < 32; o <<= 1) dg[i] += __shfl_xor_sync(0xffffffffu, dg[i], o);
  __shared__ float s_dg[8][D];
  if (sub == 0) {
#pragma unroll
    for (int i = 0; i < VEC; ++i) s_dg[warp][lir * VEC + i] = dg[i];
  }
  __syncthreads();
  if (threadIdx.x < D) {
    float s = 0.f;
    for (int w = 0; w < int(blockDim.x >> 5); ++w) s += s_dg[w][threadIdx.x];
    p.partials[int64_t(blockIdx.x) * D + threadIdx.x] = s;
  }
}

// Adds the CTAs' partial rows in a fixed order.  One CTA; column j is summed by DGAIN_GROUPS threads,
// each over every DGAIN_GROUPS-th row with eight independent loads in flight (a single thread per
// column walking all rows one memory latency at a time took as long as the main kernel), then the
// groups' sums are added in group order.
constexpr int DGAIN_GROUPS = 8;
template <int D>
__global__ void __launch_bounds__(D * DGAIN_GROUPS) qk_rms_dgain_kernel(const float* __restrict__ partials, int blocks,
                                                                       float* __restrict__ dgain) {
  __shared__ float s_sum[DGAIN_GROUPS][D];
  griddep_wait();                 // a programmatic dependent of the kernel that writes the partial rows
  const int j = threadIdx.x % D, grp = threadIdx.x / D;
  float acc[8];
#pragma unroll
  for (int u = 0; u < 8; ++u) acc[u] = 0.f;
  for (int b0 = grp; b0 < blocks; b0 += 8 * DGAIN_GROUPS) {
#pragma unroll
    for (int u = 0; u < 8; ++u) {
      const int b = b0 + u * DGAIN_GROUPS;
      if (b < blocks) acc[u] += partials[int64_t(b) * D + j];
    }
  }
  s_sum[grp][j] = ((acc[0] + acc[1]) + (acc[2] + acc[3])) + ((acc[4] + acc[5]) + (acc[6] + acc[7]));
  __syncthreads();
  if (grp == 0) {
    float s = 0.f;
#pragma unroll
    for (int g2 = 0; g2 < DGAIN_GROUPS; ++g2) s += s_sum[g2][j];
    dgain[j] = s;
  }
}

template <typename T, int D>
static int launch_rms_bwd_t(const RmsBwdParams& p, cudaStream_t stream) {
  constexpr int RPW = 32 / (D * int(sizeof(T)) / 16);
  const int64_t rows = int64_t(p.B) * p.H * p.T;
  if (rows == 0) {
    if (p.dgain != nullptr) ALG_CUDA_TRY(cudaMemsetAsync(p.dgain, 0, sizeof(float) * D, stream));
    return ALG_OK;
  }
  int64_t blocks = ((rows + RPW - 1) / RPW + 7) / 8;
  const int64_t wave = int64_t(sm_count()) * 3;         // one resident wave: three CTAs per SM
  if (blocks > wave) blocks = wave;
  if (blocks > RMS_BWD_BLOCKS) blocks = RMS_BWD_BLOCKS;
  qk_rms_bwd_kernel<T, D><<<unsigned(blocks), 256, 0, stream>>>(p);
  ALG_CUDA_TRY(cudaGetLastError());
  count_launch();
  if (p.dgain != nullptr) {
    ALG_CUDA_TRY(launch_dependent(qk_rms_dgain_kernel<D>, dim3(1), dim3(D * DGAIN_GROUPS), 0, stream, p.partials, int(blocks), p.dgain));
    count_launch();
  }
  return ALG_OK;
}

int launch_rms_bwd(const RmsBwdParams& p, int dtype, cudaStream_t stream) {
  if (p.D != 64 && p.D != 128) {
    set_error("QK RMS backward needs head_dim 64 or 128, got %d", p.D);
    return ALG_ERR_UNSUPPORTED;
  }
  if (dtype == ALG_BF16)
    return p.D == 64 ? launch_rms_bwd_t<__nv_bfloat16, 64>(p, stream) : launch_rms_bwd_t<__nv_bfloat16, 128>(p, stream);
  if (dtype == ALG_F32) return p.D == 64 ? launch_rms_bwd_t<float, 64>(p, stream) : launch_rms_bwd_t<float, 128>(p, stream);
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
  if (blocks > size_t(sm_count()) * 16) blocks = size_t(sm_count()) * 16;
  if (blocks == 0) blocks = 1;
  cast_f32_bf16_kernel<<<unsigned(blocks), 256, 0, stream>>>(src, reinterpret_cast<__nv_bfloat16*>(dst), count);
  ALG_CUDA_TRY(cudaGetLastError());
  count_launch();
  return ALG_OK;
}

}  // namespace alg
