// Single-query asinh-power attention against a KV cache (Tq = 1, all keys visible).
//
// HBM-bound: every K and V row is read from HBM exactly once.  Keys are split over CTAs
// (grid = splits x heads x batch); inside a CTA a producer warp streams 64-key K and V tiles
// into a 3-stage shared-memory ring with TMA (two CTAs per SM keep ~190 KB in flight), and
// eight consumer warps each take 8 keys of a tile.  A group of D/8 lanes owns one key: 8 FMAs
// per lane + a shuffle reduction give its score, w = (rho(x) rho(-m))^n is the max-shifted
// weight of src/algebraic/algebraic.py:186-204 with the WARP's running maximum m (rescale
// (rho(m_old) rho(-m_new))^n applied to the warp's accumulators when m moves), and every lane
// accumulates w * V for the 8 columns it holds.  No step of the key loop involves the whole
// CTA, so nothing but the ring's barriers paces it; the eight warp states are merged once at
// the end with the same exact rescale and written out as the split's (acc, m, l) state.  The split
// that finishes last for its (batch, head) merges the states, with the sink, and writes the output
// row: one launch.  "Last" is decided by an arrival word per (batch, head) that carries the call's
// number, so that nothing has to be zeroed between calls (a word left by another call counts as
// zero arrivals).  All mbarrier waits are bounded.
#include "common.cuh"
#include "launchers.h"
#include "sm100_ptx.cuh"

namespace alg {
namespace {

using namespace sm100;

constexpr int TILE = 64, STAGES = 3, CONSUMERS = 256, NTHREADS = CONSUMERS + 32;

struct __align__(16) DecodeCtl {
  uint64_t full[STAGES], empty[STAGES];
  int abort_flag;
  int tile_ok;
  int last_split;
  float x[2][TILE], w[2][TILE];
  float red[8];
};

template <int D> constexpr size_t decode_smem() { return size_t(STAGES) * 2 * TILE * D * 2 + sizeof(DecodeCtl) + 128; }

__device__ __forceinline__ void consumer_sync() { asm volatile("bar.sync 1, %0;" ::"n"(CONSUMERS) : "memory"); }

__device__ __forceinline__ void unpack8(const uint4& r, float* v) {
  const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&r);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    float2 f = __bfloat1622float2(h[i]);
    v[2 * i] = f.x; v[2 * i + 1] = f.y;
  }
}

constexpr int MAX_SPLITS = 1024;

// Merge the splits (and the sink) of one (batch, head); called by every thread of the CTA that
// arrived last, thread d < D owns output column d.  `scratch`: 2 * MAX_SPLITS floats of shared memory.
template <int D>
__device__ __forceinline__ void decode_combine(const DecodeParams& p, int b, int h, float* scratch) {
  float* s_f = scratch;                          // rescale factor per split
  float* s_l = scratch + MAX_SPLITS;
  float* s_red = scratch + 2 * MAX_SPLITS;       // D / 32 partial maxima
  const int bh = b * p.H + h;
  const float* part = p.part + int64_t(bh) * p.splits * (D + 2);
  const bool has_sink = p.sink != nullptr;
  const float bs = has_sink ? p.sink[h] * p.inv_c : -1e30f;
  const bool mine = threadIdx.x < D;
  float mm = bs;                                 // all loads below are independent of one another
  if (mine) {
    for (int s = threadIdx.x; s < p.splits; s += D) {
      const float ms = __ldcg(part + s * (D + 2) + D);      // written by other CTAs: read past L1
      s_f[s] = ms;
      s_l[s] = __ldcg(part + s * (D + 2) + D + 1);
      mm = fmaxf(mm, ms);
    }
    mm = warp_max(mm);
    if ((threadIdx.x & 31) == 0) s_red[threadIdx.x >> 5] = mm;
  }
  __syncthreads();
  mm = s_red[0];
#pragma unroll
  for (int i = 1; i < D / 32; ++i) mm = fmaxf(mm, s_red[i]);
  const float ns = rho_stable(-mm);
  if (mine) {
    for (int s = threadIdx.x; s < p.splits; s += D) {
      const float ms = s_f[s];
      s_f[s] = (ms > -1e29f) ? pow2n_rt(rho_stable(ms) * ns, p.log2n) : 0.f;
    }
  }
  __syncthreads();
  if (!mine) return;
  float lt = has_sink ? pow2n_rt(rho_stable(bs) * ns, p.log2n) : 0.f;
  float at = 0.f;
#pragma unroll 8
  for (int s = 0; s < p.splits; ++s) {
    lt = fmaf(s_f[s], s_l[s], lt);
    at = fmaf(s_f[s], __ldcg(part + s * (D + 2) + threadIdx.x), at);
  }
  reinterpret_cast<__nv_bfloat16*>(p.o)[int64_t(bh) * D + threadIdx.x] = __float2bfloat16_rn(at / lt);
}

template <int D>
__global__ void __launch_bounds__(NTHREADS, 2)
decode_partial_kernel(const __grid_constant__ CUtensorMap tm_k, const __grid_constant__ CUtensorMap tm_v,
                      const DecodeParams p) {
  constexpr int LPK = D / 8;                    // lanes per key
  constexpr int TILE_BYTES = TILE * D * 2;
  extern __shared__ unsigned char smem_raw[];
  unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 127) & ~uintptr_t(127));
  DecodeCtl* ctl = reinterpret_cast<DecodeCtl*>(smem + size_t(STAGES) * 2 * TILE_BYTES);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int split = blockIdx.x, h = blockIdx.y, b = blockIdx.z;
  const int k_begin = split * p.keys_per_split;           // tile aligned
  const int k_end = min(p.Tk, k_begin + p.keys_per_split);
  const int ntiles = k_end > k_begin ? (k_end - k_begin + TILE - 1) / TILE : 0;

  if (threadIdx.x == 0) {
    for (int s = 0; s < STAGES; ++s) { mbar_init(&ctl->full[s], 1); mbar_init(&ctl->empty[s], CONSUMERS / 32); }
    ctl->abort_flag = 0;
    ctl->tile_ok = 1;
    fence_barrier_init();
  }
  __syncthreads();
  griddep_wait();                               // launched as a programmatic dependent of the kernel ahead in the stream
  const BoundedWait bw{&ctl->abort_flag, 1000000000ull};

  if (warp == CONSUMERS / 32) {                 // producer warp
    if (lane == 0) {
      tma_prefetch_desc(&tm_k); tma_prefetch_desc(&tm_v);
      for (int t = 0; t < ntiles; ++t) {
        const int stage = t % STAGES;
        if (!bw.wait(&ctl->empty[stage], ((t / STAGES) & 1) ^ 1)) break;
        unsigned char* dst = smem + size_t(stage) * 2 * TILE_BYTES;
        mbar_arrive_expect_tx(&ctl->full[stage], 2 * TILE_BYTES);
        tma_load_4d(dst, &tm_k, &ctl->full[stage], 0, k_begin + t * TILE, h, b);
        tma_load_4d(dst + TILE_BYTES, &tm_v, &ctl->full[stage], 0, k_begin + t * TILE, h, b);
      }
    }
  } else {
    // Consumers.  Every warp takes 8 of the tile's 64 keys and carries a state of its own (running
    // maximum m, normaliser l, accumulator), so the key loop has no CTA-wide step at all: a
    // key's LPK lanes form its score with shuffles, every lane evaluates the key's weight
    // (rho(x) rho(-m))^n, and lane i of a key accumulates the 8 output columns it holds.  The
    // eight states are merged once, after the last tile, with the exact rescale.
    constexpr int KPW = TILE / (CONSUMERS / 32);            // keys per warp and tile
    constexpr int KPI = 32 / LPK;                           // keys per warp instruction
    const int lig = lane % LPK, sub = lane / LPK;
    float q[8];
    {
      const uint4 raw = *reinterpret_cast<const uint4*>(reinterpret_cast<const __nv_bfloat16*>(p.q) +
                                                        (int64_t(b) * p.H + h) * D + lig * 8);
      unpack8(raw, q);
#pragma unroll
      for (int i = 0; i < 8; ++i) q[i] *= p.scale;
    }
    float acc[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) acc[i] = 0.f;
    float m_ref = -1e30f, shift = 0.f, l_part = 0.f;
    bool ok = true;
    for (int t = 0; t < ntiles; ++t) {
      const int stage = t % STAGES;
      if (!bw.wait(&ctl->full[stage], (t / STAGES) & 1)) { ok = false; break; }
      const unsigned char* sk = smem + size_t(stage) * 2 * TILE_BYTES;
      const unsigned char* sv = sk + TILE_BYTES;
      const int key0 = k_begin + t * TILE;
      uint4 kraw[KPW / KPI], vraw[KPW / KPI];
#pragma unroll
      for (int ps = 0; ps < KPW / KPI; ++ps) {
        const int key = warp * KPW + ps * KPI + sub;
        kraw[ps] = *reinterpret_cast<const uint4*>(sk + key * (D * 2) + lig * 16);
        vraw[ps] = *reinterpret_cast<const uint4*>(sv + key * (D * 2) + lig * 16);
      }
      float x[KPW / KPI];
      float tmax = -1e30f;
#pragma unroll
      for (int ps = 0; ps < KPW / KPI; ++ps) {
        float kv[8];
        unpack8(kraw[ps], kv);
        float s = 0.f;
#pragma unroll
        for (int i = 0; i < 8; ++i) s = fmaf(q[i], kv[i], s);
#pragma unroll
        for (int o = LPK / 2; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
        x[ps] = (key0 + warp * KPW + ps * KPI + sub < k_end) ? s : -1e30f;
        tmax = fmaxf(tmax, x[ps]);
      }
#pragma unroll
      for (int o = LPK; o < 32; o <<= 1) tmax = fmaxf(tmax, __shfl_xor_sync(0xffffffffu, tmax, o));
      if (tmax > m_ref) {                                    // warp-uniform
        const float ns = rho_stable(-tmax);
        const float alpha = (m_ref > -1e29f) ? pow2n_rt(rho_stable(m_ref) * ns, p.log2n) : 0.f;
        l_part *= alpha;
#pragma unroll
        for (int i = 0; i < 8; ++i) acc[i] *= alpha;
        m_ref = tmax;
        shift = ns;
      }
#pragma unroll
      for (int ps = 0; ps < KPW / KPI; ++ps) {
        const float w = (x[ps] > -1e29f) ? pow2n_rt(rho_stable(x[ps]) * shift, p.log2n) : 0.f;
        l_part += w;
        float vv[8];
        unpack8(vraw[ps], vv);
#pragma unroll
        for (int i = 0; i < 8; ++i) acc[i] = fmaf(w, vv[i], acc[i]);
      }
      __syncwarp();
      if (lane == 0) mbar_arrive(&ctl->empty[stage]);      // this warp is done with the stage
    }
    // ---- this warp's state: add up its keys' lane groups, then merge the eight warps
#pragma unroll
    for (int o = LPK; o < 32; o <<= 1) {
      l_part += __shfl_xor_sync(0xffffffffu, l_part, o);
#pragma unroll
      for (int i = 0; i < 8; ++i) acc[i] += __shfl_xor_sync(0xffffffffu, acc[i], o);
    }
    consumer_sync();                                       // ring no longer read: reuse it as scratch
    float* s_acc = reinterpret_cast<float*>(smem);         // [warps][D]
    if (sub == 0) {
#pragma unroll
      for (int i = 0; i < 8; ++i) s_acc[warp * D + lig * 8 + i] = acc[i];
    }
    if (lane == 0) { ctl->w[0][warp] = m_ref; ctl->w[1][warp] = l_part; if (!ok) ctl->tile_ok = 0; }
    consumer_sync();
    float* out = p.part + ((int64_t(b) * p.H + h) * p.splits + split) * (D + 2);
    if (threadIdx.x < D) {
      const bool fine = ctl->tile_ok != 0;
      float mm = -1e30f;
#pragma unroll
      for (int wv = 0; wv < CONSUMERS / 32; ++wv) mm = fmaxf(mm, ctl->w[0][wv]);
      const float ns = rho_stable(-mm);
      float a = 0.f, l = 0.f;
#pragma unroll
      for (int wv = 0; wv < CONSUMERS / 32; ++wv) {
        const float mw = ctl->w[0][wv];
        const float f = (mw > -1e29f) ? pow2n_rt(rho_stable(mw) * ns, p.log2n) : 0.f;
        a = fmaf(f, s_acc[wv * D + threadIdx.x], a);
        l = fmaf(f, ctl->w[1][wv], l);
      }
      out[threadIdx.x] = fine ? a : 0.f;
      if (threadIdx.x == 0) {
        out[D] = fine ? mm : -1e30f;
        out[D + 1] = fine ? l : 0.f;
      }
      __threadfence();                                     // the state is visible before this split counts as arrived
    }
  }
  __syncthreads();
  // ---- arrival: the split that completes the count merges all states of its (batch, head)
  if (threadIdx.x == 0) {
    unsigned long long* word = p.arrivals + (int64_t(b) * p.H + h);
    unsigned long long seen = *reinterpret_cast<volatile unsigned long long*>(word), next;
    for (;;) {                                             // at most `splits` contenders, each retries a few times
      next = ((seen >> 16) == p.call) ? seen + 1 : ((p.call << 16) | 1ull);
      const unsigned long long prev = atomicCAS(word, seen, next);
      if (prev == seen) break;
      seen = prev;
    }
    ctl->last_split = int(next & 0xffffull) == p.splits ? 1 : 0;
    // the last one leaves the word at zero: a replay of this very launch (a captured graph carries the
    // same call number) starts counting afresh
    if (ctl->last_split) *reinterpret_cast<volatile unsigned long long*>(word) = 0ull;
    __threadfence();
  }
  __syncthreads();
  if (ctl->last_split) decode_combine<D>(p, b, h, reinterpret_cast<float*>(smem));
  __syncthreads();
  if (ctl->abort_flag != 0 && threadIdx.x == 0) {
    if (p.status != nullptr) atomicExch(p.status, ALG_DEV_TIMEOUT);
    const uint64_t t0 = global_timer_ns();                 // let issued loads land before the CTA retires
    while (global_timer_ns() - t0 < 200000ull) { }
  }
}

int make_kv_map(CUtensorMap* tm, const void* base, const Strides3& s, int B, int H, int T, int D) {
  const uint64_t dims[4] = {uint64_t(D), uint64_t(T), uint64_t(H), uint64_t(B)};
  const uint64_t strides[3] = {uint64_t(s.t), uint64_t(s.h), uint64_t(s.b)};
  const uint32_t box[4] = {uint32_t(D), TILE, 1, 1};
  return make_tmap_bf16(tm, base, 4, dims, strides, box, false);
}

template <int D>
int launch_d(const DecodeParams& p, cudaStream_t stream) {
  CUtensorMap tk, tv;
  if (int rc = make_kv_map(&tk, p.k, p.ks, p.B, p.H, p.Tk, D)) return rc;
  if (int rc = make_kv_map(&tv, p.v, p.vs, p.B, p.H, p.Tk, D)) return rc;
  auto kern = decode_partial_kernel<D>;
  static PerDeviceOnce configured;
  if (int rc = configured.run([&] { return cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, int(decode_smem<D>())); })) return rc;
  ALG_CUDA_TRY(launch_dependent(kern, dim3(p.splits, p.H, p.B), dim3(NTHREADS), decode_smem<D>(), stream, tk, tv, p));
  count_launch();
  return ALG_OK;
}

}  // namespace

// Splits are whole 64-key tiles.  The grid is ONE wave: at most two CTAs per SM (a
// second wave would pay the ring's start-up latency again: 62 -> 56 us on a 32768-key cache),
// never more splits than the merging CTA's table.
int decode_splits(int B, int H, int Tk) {
  const int bh = B * H > 0 ? B * H : 1;
  const int tiles = (Tk + TILE - 1) / TILE;
  int s = (sm_count() * 2) / bh;
  if (s > tiles) s = tiles;
  if (s > MAX_SPLITS) s = MAX_SPLITS;
  if (s < 1) s = 1;
  const int tiles_per_split = (tiles + s - 1) / s;
  return (tiles + tiles_per_split - 1) / tiles_per_split;
}

int decode_keys_per_split(int B, int H, int Tk) {
  const int tiles = (Tk + TILE - 1) / TILE;
  const int s = decode_splits(B, H, Tk);
  return ((tiles + s - 1) / s) * TILE;
}

int launch_decode(const DecodeParams& p, cudaStream_t stream) {
  if (p.B == 0 || p.H == 0) return ALG_OK;
  if (p.D == 64) return launch_d<64>(p, stream);
  if (p.D == 128) return launch_d<128>(p, stream);
  set_error("decode needs head_dim 64 or 128, got %d", p.D);
  return ALG_ERR_UNSUPPORTED;
}

}  // namespace alg
