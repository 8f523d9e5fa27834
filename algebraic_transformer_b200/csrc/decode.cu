// Single-query asinh-power attention against a KV cache (Tq = 1, all keys visible).
//
// HBM-bound: every K and V row is read from HBM exactly once.  Keys are split over CTAs
// (grid = splits x heads x batch); inside a CTA a producer warp streams 64-key K and V tiles
// into a 3-stage shared-memory ring with TMA (two CTAs per SM keep ~190 KB in flight), and
// eight consumer warps walk each tile in three short phases:
//   A  scores: a group of D/8 lanes owns one key, 8 FMAs per lane + a shuffle reduction
//   B  weights: one thread per key, w = (rho(x) rho(-m))^n in the max-shifted form of
//      src/algebraic/algebraic.py:186-204 with a CTA-wide running maximum m (rescale
//      (rho(m_old) rho(-m_new))^n applied to the accumulators when m moves)
//   C  values: the lane groups accumulate w * V for their keys
// so rho is evaluated once per key rather than once per lane.  Partial (acc, m, l) states
// of the splits are merged, with the sink, by decode_combine_kernel using the same exact
// rescale.  All mbarrier waits are bounded.
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

template <int D>
__global__ void __launch_bounds__(NTHREADS, 2)
decode_partial_kernel(const __grid_constant__ CUtensorMap tm_k, const __grid_constant__ CUtensorMap tm_v,
                      const DecodeParams p) {
  constexpr int LPK = D / 8;                    // lanes per key
  constexpr int GROUPS = CONSUMERS / LPK;       // keys handled per pass
  constexpr int PASSES = TILE / GROUPS;
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
    fence_barrier_init();
  }
  __syncthreads();
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
    const int group = threadIdx.x / LPK, lig = threadIdx.x % LPK;
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
    float m_ref = -1e30f, l_part = 0.f;
    bool ok = true;
    for (int t = 0; t < ntiles && ok; ++t) {
      const int stage = t % STAGES, buf = t & 1;
      // One thread performs the bounded wait and the verdict is shared through a barrier, so
      // that all consumer warps leave the loop together if a wait ever runs out (the named
      // barriers below must never be entered by only a part of them).
      if (threadIdx.x == 0) ctl->tile_ok = bw.wait(&ctl->full[stage], (t / STAGES) & 1) ? 1 : 0;
      consumer_sync();
      if (ctl->tile_ok == 0) { ok = false; break; }
      (void)mbar_try_wait(&ctl->full[stage], (t / STAGES) & 1);   // completed phase: acquire the tile for this thread
      const unsigned char* sk = smem + size_t(stage) * 2 * TILE_BYTES;
      const unsigned char* sv = sk + TILE_BYTES;
      const int key0 = k_begin + t * TILE;
      // ---- A: scores
#pragma unroll
      for (int ps = 0; ps < PASSES; ++ps) {
        const int key = ps * GROUPS + group;
        float kv[8];
        unpack8(*reinterpret_cast<const uint4*>(sk + key * (D * 2) + lig * 16), kv);
        float x = 0.f;
#pragma unroll
        for (int i = 0; i < 8; ++i) x = fmaf(q[i], kv[i], x);
#pragma unroll
        for (int o = LPK / 2; o > 0; o >>= 1) x += __shfl_xor_sync(0xffffffffu, x, o);
        if (lig == 0) ctl->x[buf][key] = (key0 + key < k_end) ? x : -1e30f;
      }
      consumer_sync();
      // ---- B: running maximum (every warp derives the same value) and one weight per key
      float tmax = warp_max(fmaxf(ctl->x[buf][lane], ctl->x[buf][lane + 32]));
      const float m_new = fmaxf(m_ref, tmax);
      const float shift = rho_stable(-m_new);
      if (m_new > m_ref) {
        const float alpha = (m_ref > -1e29f) ? pow2n_rt(rho_stable(m_ref) * shift, p.log2n) : 0.f;
        l_part *= alpha;
#pragma unroll
        for (int i = 0; i < 8; ++i) acc[i] *= alpha;
        m_ref = m_new;
      }
      if (threadIdx.x < TILE) {
        const float x = ctl->x[buf][threadIdx.x];
        const float w = (x > -1e29f) ? pow2n_rt(rho_stable(x) * shift, p.log2n) : 0.f;
        ctl->w[buf][threadIdx.x] = w;
        l_part += w;
      }
      consumer_sync();
      // ---- C: values
#pragma unroll
      for (int ps = 0; ps < PASSES; ++ps) {
        const int key = ps * GROUPS + group;
        const float w = ctl->w[buf][key];
        float vv[8];
        unpack8(*reinterpret_cast<const uint4*>(sv + key * (D * 2) + lig * 16), vv);
#pragma unroll
        for (int i = 0; i < 8; ++i) acc[i] = fmaf(w, vv[i], acc[i]);
      }
      __syncwarp();
      if (lane == 0) mbar_arrive(&ctl->empty[stage]);      // this warp is done with the stage
    }
    // ---- merge the lane groups (all share m_ref) and write the split's partial state
    consumer_sync();                                       // ring no longer read: reuse it as scratch
    float* s_acc = reinterpret_cast<float*>(smem);         // [GROUPS][D]
#pragma unroll
    for (int i = 0; i < 8; ++i) s_acc[group * D + lig * 8 + i] = acc[i];
    l_part = warp_sum(l_part);
    if (lane == 0) ctl->red[warp] = l_part;
    consumer_sync();
    float* out = p.part + ((int64_t(b) * p.H + h) * p.splits + split) * (D + 2);
    if (threadIdx.x < D) {
      float a = 0.f;
      for (int g = 0; g < GROUPS; ++g) a += s_acc[g * D + threadIdx.x];
      out[threadIdx.x] = ok ? a : 0.f;
    }
    if (threadIdx.x == 0) {
      float l = 0.f;
      for (int wv = 0; wv < CONSUMERS / 32; ++wv) l += ctl->red[wv];
      out[D] = ok ? m_ref : -1e30f;
      out[D + 1] = ok ? l : 0.f;
    }
  }
  __syncthreads();
  if (ctl->abort_flag != 0 && threadIdx.x == 0) {
    if (p.status != nullptr) atomicExch(p.status, ALG_DEV_TIMEOUT);
    const uint64_t t0 = global_timer_ns();                 // let issued loads land before the CTA retires
    while (global_timer_ns() - t0 < 200000ull) { }
  }
}

constexpr int MAX_SPLITS = 1024;

// Merge the splits (and the sink) of one (batch, head): thread d owns output column d.
template <int D>
__global__ void __launch_bounds__(D) decode_combine_kernel(const DecodeParams p) {
  __shared__ float s_f[MAX_SPLITS];             // rescale factor per split
  __shared__ float s_l[MAX_SPLITS];
  __shared__ float s_red[D / 32];
  const int bh = blockIdx.x, h = bh % p.H;
  const float* part = p.part + int64_t(bh) * p.splits * (D + 2);
  const bool has_sink = p.sink != nullptr;
  const float bs = has_sink ? p.sink[h] * p.inv_c : -1e30f;
  float mm = bs;                                 // all loads below are independent of one another
  for (int s = threadIdx.x; s < p.splits; s += D) {
    const float ms = part[s * (D + 2) + D];
    s_f[s] = ms;
    s_l[s] = part[s * (D + 2) + D + 1];
    mm = fmaxf(mm, ms);
  }
  mm = warp_max(mm);
  if ((threadIdx.x & 31) == 0) s_red[threadIdx.x >> 5] = mm;
  __syncthreads();
  mm = s_red[0];
#pragma unroll
  for (int i = 1; i < D / 32; ++i) mm = fmaxf(mm, s_red[i]);
  const float ns = rho_stable(-mm);
  for (int s = threadIdx.x; s < p.splits; s += D) {
    const float ms = s_f[s];
    s_f[s] = (ms > -1e29f) ? pow2n_rt(rho_stable(ms) * ns, p.log2n) : 0.f;
  }
  __syncthreads();
  float lt = has_sink ? pow2n_rt(rho_stable(bs) * ns, p.log2n) : 0.f;
  float at = 0.f;
#pragma unroll 4
  for (int s = 0; s < p.splits; ++s) {
    lt = fmaf(s_f[s], s_l[s], lt);
    at = fmaf(s_f[s], part[s * (D + 2) + threadIdx.x], at);
  }
  reinterpret_cast<__nv_bfloat16*>(p.o)[int64_t(bh) * D + threadIdx.x] = __float2bfloat16_rn(at / lt);
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
  static bool configured = false;
  if (!configured) {
    ALG_CUDA_TRY(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, int(decode_smem<D>())));
    configured = true;
  }
  kern<<<dim3(p.splits, p.H, p.B), NTHREADS, decode_smem<D>(), stream>>>(tk, tv, p);
  ALG_CUDA_TRY(cudaGetLastError());
  decode_combine_kernel<D><<<p.B * p.H, D, 0, stream>>>(p);
  ALG_CUDA_TRY(cudaGetLastError());
  count_launch(2);
  return ALG_OK;
}

}  // namespace

// Splits are whole 64-key tiles; enough CTAs for two per SM on 148 SMs, never more than the
// combine kernel's table.
int decode_splits(int B, int H, int Tk) {
  const int bh = B * H > 0 ? B * H : 1;
  const int tiles = (Tk + TILE - 1) / TILE;
  int s = (148 * 4 + bh - 1) / bh;
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
