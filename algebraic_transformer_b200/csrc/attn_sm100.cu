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
// The kernel is persistent: one CTA per SM walks a fixed list of work items (heaviest row
// blocks first, dealt out boustrophedon so the per-CTA sums stay level).  Barriers, tensor
// memory and the K/V ring live across items, so the loads of the next item's first tiles
// are in flight while the current item finishes, and its first S is issued while the
// weight warps still write the current output.
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
  uint64_t q_full[2], q_free[2], kv_full[MAX_NKV], kv_empty[MAX_NKV], s_full[2], p_full[2], o_full[2], o_free[2];
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

// Position in the K/V ring: slot and the parity of how often the ring has wrapped.
template <int NKV> struct RingCursor {
  int slot = 0;
  uint32_t phase = 0;
  __device__ __forceinline__ void next() { if (++slot == NKV) { slot = 0; phase ^= 1u; } }
};

// The k-th work item of this CTA.  Items are numbered heaviest first (last row block of
// every (batch, head), then the one before, ...); row k of the deal goes left to right for
// even k and right to left for odd k.
struct Item { int b, h, row0, n0, n1; };
__device__ __forceinline__ bool item_at(const AttnParams& p, int k, Item& it) {
  const int units = p.B * p.H, nblk = p.Tq / (2 * BQ), G = int(gridDim.x);
  const int idx = k * G + ((k & 1) ? G - 1 - int(blockIdx.x) : int(blockIdx.x));
  if (idx >= units * nblk) return false;
  const int blk = nblk - 1 - idx / units, bh = idx % units;
  it.b = bh / p.H; it.h = bh % p.H;
  it.row0 = blk * 2 * BQ;
  it.n0 = 2 * blk + 1; it.n1 = 2 * blk + 2;      // key tiles needed by query tile 0 / 1
  return true;
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
    for (int w = 0; w < 2; ++w) { mbar_init(&ctl->q_full[w], 1); mbar_init(&ctl->q_free[w], 1); }
    for (int i = 0; i < C::NKV; ++i) { mbar_init(&ctl->kv_full[i], 1); mbar_init(&ctl->kv_empty[i], 1); }
    for (int w = 0; w < 2; ++w) {
      mbar_init(&ctl->s_full[w], 1);
      mbar_init(&ctl->p_full[w], 128);
      mbar_init(&ctl->o_full[w], 1);
      mbar_init(&ctl->o_free[w], 128);
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

  long long tm0 = 0, tm1 = 0, tm2 = 0;            // timing accumulators (instrumentation build only)
  (void)tm0; (void)tm1; (void)tm2;
  Item it;

  if (warp == 0) {
    if (lane == 0) {
      tma_prefetch_desc(&tm_q); tma_prefetch_desc(&tm_k); tma_prefetch_desc(&tm_v);
      bool ok = true;
      RingCursor<C::NKV> cur;                       // runs on over all items
      for (int k = 0; ok && item_at(p, k, it); ++k) {
        auto load_kv = [&](int idx) {               // K_0, V_0, K_1, V_1, ... of this item
          const int buf = cur.slot;
          if (!bw.wait(&ctl->kv_empty[buf], cur.phase ^ 1u)) return false;
          mbar_arrive_expect_tx(&ctl->kv_full[buf], C::TILE_BYTES);
          const CUtensorMap* tm = (idx & 1) ? &tm_v : &tm_k;
          for (int pn = 0; pn < C::PANELS; ++pn)
            tma_load_4d(smem + C::KV_OFF + buf * C::TILE_BYTES + pn * PANEL_BYTES, tm, &ctl->kv_full[buf], pn * 64,
                        (idx >> 1) * BKEY, it.h, it.b);
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
    if (lane == 0) {
      const uint32_t q_addr = smem_u32(smem + C::Q_OFF), kv_addr = smem_u32(smem + C::KV_OFF);
      using Cur = RingCursor<C::NKV>;
      Cur cur;                                      // the next K/V tile in ring order, over all items
      int t0 = 0, t1 = 0;                           // score tiles of query tile 0 / 1 in earlier items
      auto kv_wait = [&](const Cur& c) { return bw.wait(&ctl->kv_full[c.slot], c.phase); };
      // descriptor low halves: Q tiles and ring slot 0 as K (K-major, LBO 16) and as V (MN-major,
      // LBO = one panel); a slot adds slot * TILE_BYTES / 16, a K step adds a constant
      const uint32_t q_lo0 = sw128_desc_lo(q_addr, 16), k_lo0 = sw128_desc_lo(kv_addr, 16),
                     v_lo0 = sw128_desc_lo(kv_addr, PANEL_BYTES);
      auto issue_s = [&](int w, int slot) {           // S_w = Q_w K^T
        const uint32_t qa = q_lo0 + w * (C::TILE_BYTES >> 4), ka = k_lo0 + slot * (C::TILE_BYTES >> 4);
        const uint32_t d_tmem = tmem_base + C::S_COL + w * 128;
#pragma unroll
        for (int ks = 0; ks < D / 16; ++ks) {
          const uint32_t off = ((ks >> 2) * PANEL_BYTES + (ks & 3) * 32) >> 4;
          umma_f16_ss_parts(d_tmem, qa + off, SW128_DESC_HI, ka + off, SW128_DESC_HI, C::IDESC_S, ks != 0 ? 1u : 0u);
        }
      };
      auto issue_pv = [&](int w, int slot, bool first) {  // O_w += P_w V, P_w from tensor memory
        const uint32_t va = v_lo0 + slot * (C::TILE_BYTES >> 4);
        const uint32_t d_tmem = tmem_base + C::O_COL + w * D, p_tmem = tmem_base + C::S_COL + w * 128;
#pragma unroll
        for (int ks = 0; ks < BKEY / 16; ++ks)        // 16 keys = 8 packed-bf16 columns of P per step
          umma_f16_ts_parts(d_tmem, p_tmem + ks * 8, va + ks * (2048 >> 4), SW128_DESC_HI, C::IDESC_PV,
                            (first && ks == 0) ? 0u : 1u);
      };
#ifdef ALG_ATTN_TIMING
      const long long t_begin = clock64();
#endif
      bool ok = true;
      for (int k = 0; ok && item_at(p, k, it); ++k) {
        const int n0 = it.n0, n1 = it.n1;
        if (!bw.wait(&ctl->q_full[0], k & 1u) || !kv_wait(cur)) { ok = false; break; }
        tc_fence_after();
        issue_s(0, cur.slot); umma_commit(&ctl->s_full[0]);
        if (n0 == 1) umma_commit(&ctl->q_free[0]);
        if (!bw.wait(&ctl->q_full[1], k & 1u)) { ok = false; break; }
        tc_fence_after();
        issue_s(1, cur.slot); umma_commit(&ctl->s_full[1]);
        umma_commit(&ctl->kv_empty[cur.slot]);
        cur.next();
        for (int j = 0; j < n1 && ok; ++j) {
          const Cur vc = cur;                         // V_j
          cur.next();
          const Cur kc = cur;                         // K_{j+1}: only meaningful while j + 1 < n1
          if (j + 1 < n1) cur.next();
          // Both tiles of this step are waited for up front (they are normally long there), so
          // that nothing stands between "weights ready" and the issue of P.V and the next S.
          if (!ALG_T(tm0, kv_wait(vc)) || (j + 1 < n1 && !ALG_T(tm0, kv_wait(kc)))) { ok = false; break; }
          if (j < n0) {
            if (!ALG_T(tm1, bw.wait(&ctl->p_full[0], (t0 + j) & 1u))) { ok = false; break; }
            // the first product of an item overwrites O_0: the previous output must have been read
            if (j == 0 && k > 0 && !bw.wait(&ctl->o_free[0], (k - 1) & 1u)) { ok = false; break; }
            tc_fence_after();
            issue_pv(0, vc.slot, j == 0);
            if (j + 1 < n0) {
              issue_s(0, kc.slot);                     // after P_0.V: may overwrite P_0
              umma_commit(&ctl->s_full[0]);
              if (j + 2 == n0) umma_commit(&ctl->q_free[0]);   // the item's last read of Q tile 0
            } else {
              umma_commit(&ctl->o_full[0]);
            }
          }
          if (!ALG_T(tm2, bw.wait(&ctl->p_full[1], (t1 + j) & 1u))) { ok = false; break; }
          if (j == 0 && k > 0 && !bw.wait(&ctl->o_free[1], (k - 1) & 1u)) { ok = false; break; }
          tc_fence_after();
          issue_pv(1, vc.slot, j == 0);
          umma_commit(&ctl->kv_empty[vc.slot]);
          if (j + 1 < n1) {
            issue_s(1, kc.slot);
            umma_commit(&ctl->s_full[1]);
            umma_commit(&ctl->kv_empty[kc.slot]);
            if (j + 2 == n1) umma_commit(&ctl->q_free[1]);     // the item's last read of Q tile 1
          } else {
            umma_commit(&ctl->o_full[1]);
          }
        }
        t0 += n0; t1 += n1;
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
    const uint32_t lane_sel = uint32_t(quarter * 32) << 16;
    const uint32_t s_taddr = tmem_base + lane_sel + C::S_COL + w * 128;
    bool ok = true;
    int tiles_before = 0;                           // score tiles of this group in earlier items
#ifdef ALG_ATTN_TIMING
    const long long t_begin = clock64();
#endif
    for (int k = 0; ok && item_at(p, k, it); ++k) {
      const int nk = (w == 0) ? it.n0 : it.n1;
      float l = 0.f;                                // the sink's weight, fetched while the first scores are computed
      if (p.sink != nullptr) l = pow2n<LOG2N>(rho_stable(p.sink[it.h] * p.inv_c));
      float2 la = make_float2(0.f, 0.f), lb = make_float2(0.f, 0.f);
      for (int j = 0; j < nk && ok; ++j) {
        if (!ALG_T(tm0, bw.wait(&ctl->s_full[w], (tiles_before + j) & 1u))) { ok = false; break; }
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
      tiles_before += nk;
      if (!ok || !bw.wait(&ctl->o_full[w], k & 1u)) { ok = false; break; }
      tc_fence_after();
      item_at(p, k, it);                            // recomputed: nothing of it stays live over the tile loop
      l += (la.x + la.y) + (lb.x + lb.y);
      const float inv = 1.0f / l;
      const int row = it.row0 + w * BQ + r;
      __nv_bfloat16* orow = reinterpret_cast<__nv_bfloat16*>(p.o) + it.b * p.os.b + it.h * p.os.h + int64_t(row) * p.os.t;
#pragma unroll 1
      for (int chunk = 0; chunk < D / 32; ++chunk) {
        uint32_t o[32];
        tmem_ld_32x32(tmem_base + lane_sel + C::O_COL + w * D + chunk * 32, o);
        tmem_ld_wait_for(o);
        if (chunk == D / 32 - 1) {                  // O_w is in registers: the next item may overwrite it
          tc_fence_before();
          mbar_arrive(&ctl->o_free[w]);
        }
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
      if (p.stat != nullptr) p.stat[(int64_t(it.b) * p.H + it.h) * p.Tq + row] = inv;
#endif
    }
#ifdef ALG_ATTN_TIMING
    if (blockIdx.x == 0 && r == 0 && p.stat != nullptr) {
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
  int dev = 0, sms = 148;
  ALG_CUDA_TRY(cudaGetDevice(&dev));
  ALG_CUDA_TRY(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev));
  const int items = p.B * p.H * (p.Tq / (2 * BQ));
  const int grid = items < sms ? items : sms;
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
