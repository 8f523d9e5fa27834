// Asinh-power attention forward on tcgen05 tensor cores (the throughput path).
//
// Covers the unshifted accumulation of the reference (src/algebraic/kernels/flash.py:
// 227-234): p = rho_fast(x)^n, l = rho(b')^n + sum p, o = (sum p v) / l, stat = 1/l — the
// branch the range guard selects for QK-normalised inputs.  bf16 I/O, causal, Tq == Tk a
// multiple of 256, head_dim 64 or 128.  Because nothing is rescaled in this form, the
// output accumulator simply stays in tensor memory from the first key tile to the last.
//
// One CTA owns 256 consecutive query rows of one (batch, head): two 128-row tiles.
//   warp 0 (one lane)  TMA: both Q tiles once, then K_j / V_j tiles through a ring
//   warp 1 (one lane)  tcgen05.mma: S_w = Q_w K_j^T (both operands in shared memory) and
//                      O_w += P_w V_j with P_w read from TENSOR MEMORY (the A operand) and
//                      V_j from shared memory as an MN-major B operand
//   warps 2..5         weights for query tile 0: tcgen05.ld S_0 (one thread = one row),
//                      x -> rho_fast(x)^n in packed fp32, row sum, bf16 P_0 written back
//                      with tcgen05.st over the columns S_0 occupied
//   warps 6..9         the same for query tile 1
// The two tiles run out of phase, so the tensor pipe works for one while the other
// evaluates rho.  TMEM (512 columns): S_0, S_1 (128 each; P_w aliases the first 64 columns
// of S_w as packed bf16) + O_0, O_1 (head_dim each).  P never touches shared memory, which
// leaves the tensor core's shared-memory operand path to Q, K and V alone.  The tensor pipe
// executes one thread's MMAs in issue order, so issuing S_w(j+1) after P_w(j).V_j is what
// protects P_w(j) from being overwritten, and S_w(j+1) complete implies P_w(j).V_j complete.
// Key tiles above the diagonal are never loaded; only the diagonal tile evaluates a mask.
// Every mbarrier wait is bounded (sm100_ptx.cuh); on a timeout the kernel reports
// ALG_DEV_TIMEOUT through the status word and returns.
#include "common.cuh"
#include "launchers.h"
#include "sm100_ptx.cuh"

namespace alg {
namespace {

using namespace sm100;

constexpr int BQ = 128, BKEY = 128, NTHREADS = 320;
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
  static constexpr uint32_t S_COL = 0;                      // S_w at S_COL + 128 w; P_w = its first 64 columns
  static constexpr uint32_t O_COL = 256;                    // O_w at O_COL + D w
  static constexpr uint32_t IDESC_S = make_idesc_bf16(BQ, BKEY, 0, 0);
  static constexpr uint32_t IDESC_PV = make_idesc_bf16(BQ, D, 0, 1);   // V is [key][d]: MN-major B
};

struct __align__(16) Control {
  uint64_t q_full, kv_full[MAX_NKV], kv_empty[MAX_NKV], s_full[2], p_full[2], o_full[2];
  uint32_t tmem_base;
  int abort_flag;
  int shift_mode;
};

// 32 scores -> 32 weights rho_fast(s * scale)^n, two at a time on the packed fp32 pipe
// (fma.f32x2 / mul.f32x2); row-sum partials in `la`, `lb`; bf16 pairs in `packed`.
template <int LOG2N, bool DIAG>
__device__ __forceinline__ void weigh32(const uint32_t* s, float scale, int col0, int r, float2& la, float2& lb,
                                        uint32_t* packed) {
  const float2 sc = make_float2(scale, scale), one = make_float2(1.f, 1.f);
#pragma unroll
  for (int i = 0; i < 32; i += 4) {
    float2 x0 = __fmul2_rn(make_float2(__uint_as_float(s[i]), __uint_as_float(s[i + 1])), sc);
    float2 x1 = __fmul2_rn(make_float2(__uint_as_float(s[i + 2]), __uint_as_float(s[i + 3])), sc);
    const float2 rad0 = __ffma2_rn(x0, x0, one), rad1 = __ffma2_rn(x1, x1, one);
    const float2 rs0 = make_float2(rsqrt_approx(rad0.x), rsqrt_approx(rad0.y));
    const float2 rs1 = make_float2(rsqrt_approx(rad1.x), rsqrt_approx(rad1.y));
    float2 t0 = __ffma2_rn(rad0, rs0, x0), t1 = __ffma2_rn(rad1, rs1, x1);
#pragma unroll
    for (int k = 0; k < LOG2N; ++k) { t0 = __fmul2_rn(t0, t0); t1 = __fmul2_rn(t1, t1); }
    if (DIAG) {                                     // causal mask inside the diagonal tile
      t0.x = (col0 + i <= r) ? t0.x : 0.f;     t0.y = (col0 + i + 1 <= r) ? t0.y : 0.f;
      t1.x = (col0 + i + 2 <= r) ? t1.x : 0.f; t1.y = (col0 + i + 3 <= r) ? t1.y : 0.f;
    }
    la = __fadd2_rn(la, t0);
    lb = __fadd2_rn(lb, t1);
    packed[i >> 1] = pack_bf16(t0.x, t0.y);
    packed[(i >> 1) + 1] = pack_bf16(t1.x, t1.y);
  }
}

// One 128-key score tile of this thread's row: S from TMEM -> weights -> packed bf16 P back
// into TMEM over the same columns.  Columns 32c..32c+31 of S become columns 16c..16c+15 of
// P, always at or below what has already been read, and the load of the next 32 columns is
// in flight while the current 32 are evaluated.
template <int LOG2N, bool DIAG>
__device__ __forceinline__ void weigh_tile(uint32_t s_taddr, int r, float scale, float2& la, float2& lb) {
  uint32_t a[32], b[32], packed[16];
  tmem_ld_32x32(s_taddr, a);
  tmem_ld_wait_for(a);
  tmem_ld_32x32(s_taddr + 32, b);
  weigh32<LOG2N, DIAG>(a, scale, 0, r, la, lb, packed);
  tmem_st_32x16(s_taddr, packed);
  tmem_ld_wait_for(b);
  tmem_ld_32x32(s_taddr + 64, a);
  weigh32<LOG2N, DIAG>(b, scale, 32, r, la, lb, packed);
  tmem_st_32x16(s_taddr + 16, packed);
  tmem_ld_wait_for(a);
  tmem_ld_32x32(s_taddr + 96, b);
  weigh32<LOG2N, DIAG>(a, scale, 64, r, la, lb, packed);
  tmem_st_32x16(s_taddr + 32, packed);
  tmem_ld_wait_for(b);
  weigh32<LOG2N, DIAG>(b, scale, 96, r, la, lb, packed);
  tmem_st_32x16(s_taddr + 48, packed);
  tmem_st_wait();
}

template <int D> constexpr size_t smem_bytes() { return size_t(Cfg<D>::CTL_OFF) + sizeof(Control) + 1024; }

#ifdef ALG_ATTN_TIMING   // optional instrumentation build: cycle counters written into `stat`
#define ALG_T(acc, expr) [&] { const long long t_ = clock64(); const bool r_ = (expr); acc += clock64() - t_; return r_; }()
#else
#define ALG_T(acc, expr) (expr)
#endif

template <int D, int LOG2N>
__global__ void __launch_bounds__(NTHREADS, 1)
attn_tc_kernel(const __grid_constant__ CUtensorMap tm_q, const __grid_constant__ CUtensorMap tm_k,
               const __grid_constant__ CUtensorMap tm_v, const AttnParams p) {
  using C = Cfg<D>;
  extern __shared__ unsigned char smem_raw[];
  unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  Control* ctl = reinterpret_cast<Control*>(smem + C::CTL_OFF);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

  if (threadIdx.x == 0) ctl->shift_mode = attn_use_shift(p) ? 1 : 0;
  __syncthreads();
  if (ctl->shift_mode != 0) return;               // the guard failed: the stable kernel does this launch's work

  if (threadIdx.x == 0) {
    mbar_init(&ctl->q_full, 1);
    for (int i = 0; i < C::NKV; ++i) { mbar_init(&ctl->kv_full[i], 1); mbar_init(&ctl->kv_empty[i], 1); }
    for (int w = 0; w < 2; ++w) {
      mbar_init(&ctl->s_full[w], 1);
      mbar_init(&ctl->p_full[w], 128);
      mbar_init(&ctl->o_full[w], 1);
    }
    ctl->abort_flag = 0;
    fence_barrier_init();
    if (blockIdx.x == 0 && p.stat_kind != nullptr) *p.stat_kind = ALG_VARIANT_NOSHIFT;
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

  // work item: heavy (late) row blocks first
  const int units = p.B * p.H;
  const int nblk = p.Tq / (2 * BQ);
  const int blk = nblk - 1 - int(blockIdx.x) / units;
  const int bh = int(blockIdx.x) % units;
  const int b = bh / p.H, h = bh % p.H;
  const int row0 = blk * 2 * BQ;
  const int n0 = 2 * blk + 1, n1 = 2 * blk + 2;   // key tiles needed by query tile 0 / 1
  long long tm0 = 0, tm1 = 0, tm2 = 0;            // timing accumulators (instrumentation build only)
  (void)tm0; (void)tm1; (void)tm2;

  if (warp == 0) {
    if (lane == 0) {
      tma_prefetch_desc(&tm_q); tma_prefetch_desc(&tm_k); tma_prefetch_desc(&tm_v);
      mbar_arrive_expect_tx(&ctl->q_full, 2 * C::TILE_BYTES);
      for (int w = 0; w < 2; ++w)
        for (int pn = 0; pn < C::PANELS; ++pn)
          tma_load_4d(smem + C::Q_OFF + w * C::TILE_BYTES + pn * PANEL_BYTES, &tm_q, &ctl->q_full, pn * 64,
                      row0 + w * BQ, h, b);
      bool ok = true;
      for (int idx = 0; idx < 2 * n1 && ok; ++idx) {   // K_0, V_0, K_1, V_1, ...
        const int buf = idx % C::NKV;
        const uint32_t phase = (idx / C::NKV) & 1u;
        if (!bw.wait(&ctl->kv_empty[buf], phase ^ 1u)) { ok = false; break; }
        mbar_arrive_expect_tx(&ctl->kv_full[buf], C::TILE_BYTES);
        const CUtensorMap* tm = (idx & 1) ? &tm_v : &tm_k;
        for (int pn = 0; pn < C::PANELS; ++pn)
          tma_load_4d(smem + C::KV_OFF + buf * C::TILE_BYTES + pn * PANEL_BYTES, tm, &ctl->kv_full[buf], pn * 64,
                      (idx >> 1) * BKEY, h, b);
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      const uint32_t q_addr = smem_u32(smem + C::Q_OFF), kv_addr = smem_u32(smem + C::KV_OFF);
      auto kv_wait = [&](int idx) { return bw.wait(&ctl->kv_full[idx % C::NKV], (idx / C::NKV) & 1u); };
      auto issue_s = [&](int w, int idx) {            // S_w = Q_w K^T
        const uint32_t qa = q_addr + w * C::TILE_BYTES, ka = kv_addr + (idx % C::NKV) * C::TILE_BYTES;
#pragma unroll
        for (int ks = 0; ks < D / 16; ++ks) {
          const uint32_t off = (ks >> 2) * PANEL_BYTES + (ks & 3) * 32;
          umma_f16_ss(tmem_base + C::S_COL + w * 128, make_sw128_desc(qa + off, 16, 1024),
                      make_sw128_desc(ka + off, 16, 1024), C::IDESC_S, ks != 0 ? 1u : 0u);
        }
      };
      auto issue_pv = [&](int w, int idx, bool first) {   // O_w += P_w V, P_w from tensor memory
        const uint32_t va = kv_addr + (idx % C::NKV) * C::TILE_BYTES;
#pragma unroll
        for (int ks = 0; ks < BKEY / 16; ++ks)        // 16 keys = 8 packed-bf16 columns of P per step
          umma_f16_ts(tmem_base + C::O_COL + w * D, tmem_base + C::S_COL + w * 128 + ks * 8,
                      make_sw128_desc(va + ks * 2048, PANEL_BYTES, 1024), C::IDESC_PV, (first && ks == 0) ? 0u : 1u);
      };
#ifdef ALG_ATTN_TIMING
      const long long t_begin = clock64();
#endif
      bool ok = bw.wait(&ctl->q_full, 0) && kv_wait(0);
      if (ok) {
        tc_fence_after();
        issue_s(0, 0); umma_commit(&ctl->s_full[0]);
        issue_s(1, 0); umma_commit(&ctl->s_full[1]);
        umma_commit(&ctl->kv_empty[0]);
      }
      for (int j = 0; j < n1 && ok; ++j) {
        const int vidx = 2 * j + 1, kidx = 2 * j + 2;
        bool k_ready = false;
        if (!ALG_T(tm0, kv_wait(vidx))) { ok = false; break; }
        if (j < n0) {
          if (!ALG_T(tm1, bw.wait(&ctl->p_full[0], j & 1u))) { ok = false; break; }
          tc_fence_after();
          issue_pv(0, vidx, j == 0);
          if (j + 1 < n0) {
            if (!ALG_T(tm0, kv_wait(kidx))) { ok = false; break; }
            k_ready = true;
            tc_fence_after();
            issue_s(0, kidx);                       // after P_0.V: may overwrite P_0
            umma_commit(&ctl->s_full[0]);
          } else {
            umma_commit(&ctl->o_full[0]);
          }
        }
        if (!ALG_T(tm2, bw.wait(&ctl->p_full[1], j & 1u))) { ok = false; break; }
        tc_fence_after();
        issue_pv(1, vidx, j == 0);
        umma_commit(&ctl->kv_empty[vidx % C::NKV]);
        if (j + 1 < n1) {
          if (!k_ready && !ALG_T(tm0, kv_wait(kidx))) { ok = false; break; }
          tc_fence_after();
          issue_s(1, kidx);
          umma_commit(&ctl->s_full[1]);
          umma_commit(&ctl->kv_empty[kidx % C::NKV]);
        } else {
          umma_commit(&ctl->o_full[1]);
        }
      }
#ifdef ALG_ATTN_TIMING
      if (blockIdx.x == 0 && p.stat != nullptr) {
        float* dbg = p.stat + 16;
        dbg[0] = float(tm0); dbg[1] = float(tm1); dbg[2] = float(tm2); dbg[3] = float(clock64() - t_begin);
      }
#endif
    }
  } else {
    const int w = (warp - 2) >> 2;                  // query tile of this weight group
    const int quarter = warp & 3;                   // TMEM lanes 32*quarter.. are this warp's
    const int r = quarter * 32 + lane;              // row inside the query tile
    const int nk = (w == 0) ? n0 : n1;
    const uint32_t lane_sel = uint32_t(quarter * 32) << 16;
    float l = 0.f;
    if (p.sink != nullptr) l = pow2n<LOG2N>(rho_stable(p.sink[h] * p.inv_c));
    const uint32_t s_taddr = tmem_base + lane_sel + C::S_COL + w * 128;
    float2 la = make_float2(0.f, 0.f), lb = make_float2(0.f, 0.f);
    bool ok = true;
#ifdef ALG_ATTN_TIMING
    const long long t_begin = clock64();
#endif
    for (int j = 0; j < nk && ok; ++j) {
      if (!ALG_T(tm0, bw.wait(&ctl->s_full[w], j & 1u))) { ok = false; break; }
      tc_fence_after();
#ifdef ALG_ATTN_TIMING
      const long long tc0 = clock64();
#endif
      if (j == nk - 1) weigh_tile<LOG2N, true>(s_taddr, r, p.scale, la, lb);   // diagonal tile: masked
      else weigh_tile<LOG2N, false>(s_taddr, r, p.scale, la, lb);
      tc_fence_before();
      mbar_arrive(&ctl->p_full[w]);
#ifdef ALG_ATTN_TIMING
      tm1 += clock64() - tc0;
#endif
    }
#ifdef ALG_ATTN_TIMING
    if (blockIdx.x == 0 && r == 0 && p.stat != nullptr) {
      float* dbg = p.stat + 8 * w;
      dbg[0] = float(tm0); dbg[1] = 0.f; dbg[2] = float(tm1); dbg[3] = float(clock64() - t_begin); dbg[4] = float(nk);
    }
#endif
    l += (la.x + la.y) + (lb.x + lb.y);
    if (ok && bw.wait(&ctl->o_full[w], 0)) {
      tc_fence_after();
      const float inv = 1.0f / l;
      const int row = row0 + w * BQ + r;
      __nv_bfloat16* orow = reinterpret_cast<__nv_bfloat16*>(p.o) + b * p.os.b + h * p.os.h + int64_t(row) * p.os.t;
#pragma unroll 1
      for (int chunk = 0; chunk < D / 32; ++chunk) {
        uint32_t o[32];
        tmem_ld_32x32(tmem_base + lane_sel + C::O_COL + w * D + chunk * 32, o);
        tmem_ld_wait_for(o);
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
#ifndef ALG_ATTN_TIMING
      if (p.stat != nullptr) p.stat[(int64_t(b) * p.H + h) * p.Tq + row] = inv;
#endif
    }
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

int make_qkv_map(CUtensorMap* tm, const void* base, const Strides3& s, int B, int H, int T, int D) {
  const uint64_t dims[4] = {uint64_t(D), uint64_t(T), uint64_t(H), uint64_t(B)};
  const uint64_t strides[3] = {uint64_t(s.t), uint64_t(s.h), uint64_t(s.b)};
  const uint32_t box[4] = {64, 128, 1, 1};
  return make_tmap_bf16(tm, base, 4, dims, strides, box, true);
}

template <int D, int LOG2N>
int launch_dn(const AttnParams& p, cudaStream_t stream) {
  CUtensorMap tq, tk, tv;
  if (int rc = make_qkv_map(&tq, p.q, p.qs, p.B, p.H, p.Tq, D)) return rc;
  if (int rc = make_qkv_map(&tk, p.k, p.ks, p.B, p.H, p.Tk, D)) return rc;
  if (int rc = make_qkv_map(&tv, p.v, p.vs, p.B, p.H, p.Tk, D)) return rc;
  auto kern = attn_tc_kernel<D, LOG2N>;
  static bool configured = false;
  if (!configured) {
    ALG_CUDA_TRY(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, int(smem_bytes<D>())));
    configured = true;
  }
  const int grid = p.B * p.H * (p.Tq / (2 * BQ));
  kern<<<grid, NTHREADS, smem_bytes<D>(), stream>>>(tq, tk, tv, p);
  ALG_CUDA_TRY(cudaGetLastError());
  count_launch();
  return ALG_OK;
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

}  // namespace

bool attn_tcgen05_supports(const AttnParams& p, int dtype) {
  const bool strides_fit = p.qs.t > 0 && p.ks.t > 0 && p.vs.t > 0 && p.qs.h >= 0 && p.qs.b >= 0 &&
                           p.ks.h >= 0 && p.ks.b >= 0 && p.vs.h >= 0 && p.vs.b >= 0;
  return dtype == ALG_BF16 && p.causal && p.Tq == p.Tk && p.Tq % (2 * BQ) == 0 && (p.D == 64 || p.D == 128) &&
         p.log2n >= 3 && p.log2n <= 5 && p.variant != ALG_VARIANT_SHIFT && strides_fit &&
         (p.B == 1 || p.qs.b > 0) && (p.H == 1 || p.qs.h > 0);
}

int launch_attn_tcgen05(const AttnParams& p, cudaStream_t stream) {
  return p.D == 64 ? launch_d<64>(p, stream) : launch_d<128>(p, stream);
}

}  // namespace alg
