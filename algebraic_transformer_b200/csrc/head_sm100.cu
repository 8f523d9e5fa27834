// Fused Alg-CE head forward on tcgen05 tensor cores: a persistent, warp-specialised GEMM
// z = h . E^T whose fp32 accumulator tiles live in tensor memory and are consumed there.
//
//   warp 0 (one lane)  TMA producer: 128x64 tiles of h and 256x64 tiles of E (bf16,
//                      128-byte swizzle) into a 4-stage shared-memory ring
//   warp 1 (one lane)  MMA issuer: tcgen05.mma 128x256x16, accumulating a 128x256 fp32 tile
//                      in one of two TMEM buffers (2 x 256 columns = all 512)
//   warps 2..9         epilogue: tcgen05.ld the finished tile (each warp its 32 lanes x 128
//                      columns), w = rho_fast(min(z/c, clamp))^n, row sums, target pick —
//                      while the MMA warp already fills the other TMEM buffer
//
// Logits never leave the SM.  A CTA walks "units" = (128-token block, run of vocabulary
// tiles); per unit each epilogue thread writes one partial (l, zt) for its row and column
// half, and head_reduce adds the partials in a fixed order (deterministic results).
// Semantics: src/algebraic/kernels/fused_head.py:72-117 of the reference.  Every wait is
// bounded; a wait that runs out sets ALG_DEV_TIMEOUT in the caller's status word.
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

struct Plan {
  int row_blocks, ntiles, tps, S, units;
};

Plan make_plan(int N, int V_local) {
  Plan pl;
  pl.row_blocks = (N + BM - 1) / BM;
  pl.ntiles = (V_local + BN - 1) / BN;
  const long long total = (long long)pl.row_blocks * pl.ntiles;
  long long tps = total / (sm_count() * 8);
  if (tps < 1) tps = 1;
  if (tps > 8) tps = 8;
  pl.tps = int(tps);
  pl.S = (pl.ntiles + pl.tps - 1) / pl.tps;
  pl.units = pl.row_blocks * pl.S;
  return pl;
}

// LOG2N = log2 of the power of the algebraic likelihood, or LOG2N_CE for the softmax cross-entropy
// kind: the same GEMM and partial layout, with an online logsumexp (running maximum m, sum of
// exp(z - m) rescaled when m grows; src/algebraic/kernels/fused_head.py:87-94) in place of rho^n.
constexpr int LOG2N_CE = -1;

template <int LOG2N>
__global__ void __launch_bounds__(NTHREADS, 1)
head_tc_kernel(const __grid_constant__ CUtensorMap tm_h, const __grid_constant__ CUtensorMap tm_e,
               const HeadParams p, const int S, const int tps, const int units, const int row_blocks) {
  extern __shared__ unsigned char smem_raw[];
  unsigned char* smem = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  Control* ctl = reinterpret_cast<Control*>(smem + size_t(STAGES) * STAGE_BYTES);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

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
  const int ntiles = (p.V_local + BN - 1) / BN;
  const int kblocks = p.d / BK;

  if (warp == 0) {
    if (lane == 0) {
      tma_prefetch_desc(&tm_h);
      tma_prefetch_desc(&tm_e);
      uint32_t it = 0;
      bool ok = true;
      for (int u = blockIdx.x; u < units && ok; u += gridDim.x) {
        const int m = u % row_blocks, s = u / row_blocks;
        const int t0 = s * tps, t1 = min(ntiles, t0 + tps);
        for (int t = t0; t < t1 && ok; ++t)
          for (int kb = 0; kb < kblocks; ++kb, ++it) {
            const uint32_t stage = it % STAGES, phase = (it / STAGES) & 1u;
            if (!bw.wait(&ctl->empty[stage], phase ^ 1u)) { ok = false; break; }
            unsigned char* dst = smem + size_t(stage) * STAGE_BYTES;
            mbar_arrive_expect_tx(&ctl->full[stage], STAGE_BYTES);
            tma_load_2d(dst, &tm_h, &ctl->full[stage], kb * BK, m * BM);
            tma_load_2d(dst + A_BYTES, &tm_e, &ctl->full[stage], kb * BK, t * BN);
          }
      }
    }
  } else if (warp == 1) {
    if (lane == 0) {
      uint32_t it = 0, tile_count = 0;
      // descriptor low halves of stage 0 (sm100_ptx.cuh: sw128_desc_lo); a stage adds STAGE_BYTES / 16,
      // a K step 2 — the issue loop then spends one add per operand and MMA
      const uint32_t a_lo0 = sw128_desc_lo(smem_u32(smem), 16), b_lo0 = sw128_desc_lo(smem_u32(smem) + A_BYTES, 16);
      bool ok = true;
      for (int u = blockIdx.x; u < units && ok; u += gridDim.x) {
        const int s = u / row_blocks;
        const int t0 = s * tps, t1 = min(ntiles, t0 + tps);
        for (int t = t0; t < t1 && ok; ++t, ++tile_count) {
          const uint32_t buf = tile_count & 1u, tphase = (tile_count >> 1) & 1u;
          if (!bw.wait(&ctl->tempty[buf], tphase ^ 1u)) { ok = false; break; }
          tc_fence_after();
          const uint32_t d_tmem = tmem_base + buf * BN;
          for (int kb = 0; kb < kblocks; ++kb, ++it) {
            const uint32_t stage = it % STAGES, phase = (it / STAGES) & 1u;
            if (!bw.wait(&ctl->full[stage], phase)) { ok = false; break; }
            tc_fence_after();
            const uint32_t a_lo = a_lo0 + stage * (STAGE_BYTES >> 4), b_lo = b_lo0 + stage * (STAGE_BYTES >> 4);
#pragma unroll
            for (int k = 0; k < BK / UMMA_K; ++k)
              umma_f16_ss_parts(d_tmem, a_lo + k * (UMMA_K * 2 >> 4), SW128_DESC_HI, b_lo + k * (UMMA_K * 2 >> 4),
                                SW128_DESC_HI, IDESC, (kb | k) != 0 ? 1u : 0u);
            umma_commit(&ctl->empty[stage]);           // smem stage is free once these MMAs retire
          }
          if (ok) umma_commit(&ctl->tfull[buf]);        // accumulator tile complete
        }
      }
    }
  } else {
    const int quarter = warp & 3;                        // TMEM lanes 32*quarter .. +31 belong to this warp
    const int half = (warp - 2) >> 2;                    // which 128 of the tile's 256 columns
    const int row_in_tile = quarter * 32 + lane;
    uint32_t tile_count = 0;
    bool ok = true;
    for (int u = blockIdx.x; u < units && ok; u += gridDim.x) {
      const int m = u % row_blocks, s = u / row_blocks;
      const int t0 = s * tps, t1 = min(ntiles, t0 + tps);
      const int row = m * BM + row_in_tile;
      const int tgt = (row < p.N) ? (p.targets[row] - p.vocab_offset) : -0x40000000;
      float l0 = 0.f, l1 = 0.f, l2 = 0.f, l3 = 0.f, zt = 0.f;
      float m_run = -1e30f;                                // ce kind: running maximum of this thread's logits
      for (int t = t0; t < t1 && ok; ++t, ++tile_count) {
        const uint32_t buf = tile_count & 1u, tphase = (tile_count >> 1) & 1u;
        if (!bw.wait(&ctl->tfull[buf], tphase)) { ok = false; break; }
        tc_fence_after();
        const int col_base = t * BN + half * 128;
#pragma unroll 1
        for (int chunk = 0; chunk < 4; ++chunk) {
          uint32_t r[32];
          tmem_ld_32x32(tmem_base + (uint32_t(quarter * 32) << 16) + buf * BN + half * 128 + chunk * 32, r);
          tmem_ld_wait();
          const int c0 = col_base + chunk * 32;
          const bool tail = c0 + 32 > p.V_local;
          const unsigned dt = unsigned(tgt - c0);
          if (dt < 32u) {
#pragma unroll
            for (int j = 0; j < 32; ++j) zt += (unsigned(j) == dt) ? __uint_as_float(r[j]) : 0.f;
          }
          if (LOG2N == LOG2N_CE) {
            if (c0 >= p.V_local) continue;                 // nothing but zero-filled columns (same for the whole warp)
            constexpr float LOG2E = 1.4426950408889634f;
            float cmax = -1e30f;
#pragma unroll
            for (int j = 0; j < 32; ++j) {
              if (tail && c0 + j >= p.V_local) r[j] = __float_as_uint(-1e30f);   // exp -> 0 below
              cmax = fmaxf(cmax, __uint_as_float(r[j]));
            }
            const float m_new = fmaxf(m_run, cmax);
            const float resc = exp2_approx((m_run - m_new) * LOG2E);   // 0 on the first chunk, where the sums are 0
            const float off = -m_new * LOG2E;
            l0 *= resc; l1 *= resc; l2 *= resc; l3 *= resc;
#pragma unroll
            for (int j = 0; j < 32; j += 4) {
              l0 += exp2_approx(fmaf(__uint_as_float(r[j]), LOG2E, off));
              l1 += exp2_approx(fmaf(__uint_as_float(r[j + 1]), LOG2E, off));
              l2 += exp2_approx(fmaf(__uint_as_float(r[j + 2]), LOG2E, off));
              l3 += exp2_approx(fmaf(__uint_as_float(r[j + 3]), LOG2E, off));
            }
            m_run = m_new;
            continue;
          }
          // pairs of columns through the packed fp32 instructions (mul.f32x2 / fma.f32x2 / add.f32x2)
          const float2 ic2 = make_float2(p.inv_c, p.inv_c), one2 = make_float2(1.f, 1.f);
#pragma unroll
          for (int j = 0; j < 32; j += 4) {
            float2 xa = __fmul2_rn(make_float2(__uint_as_float(r[j]), __uint_as_float(r[j + 1])), ic2);
            float2 xb = __fmul2_rn(make_float2(__uint_as_float(r[j + 2]), __uint_as_float(r[j + 3])), ic2);
            xa.x = fminf(xa.x, p.clamp); xa.y = fminf(xa.y, p.clamp);
            xb.x = fminf(xb.x, p.clamp); xb.y = fminf(xb.y, p.clamp);
            const float2 ra = __ffma2_rn(xa, xa, one2), rb = __ffma2_rn(xb, xb, one2);
            float2 wa = __ffma2_rn(ra, make_float2(rsqrt_approx(ra.x), rsqrt_approx(ra.y)), xa);   // rho_fast
            float2 wb = __ffma2_rn(rb, make_float2(rsqrt_approx(rb.x), rsqrt_approx(rb.y)), xb);
#pragma unroll
            for (int k = 0; k < LOG2N; ++k) { wa = __fmul2_rn(wa, wa); wb = __fmul2_rn(wb, wb); }
            if (tail) {                                    // zero-filled columns must not add rho(0)^n
              if (c0 + j >= p.V_local) wa.x = 0.f;
              if (c0 + j + 1 >= p.V_local) wa.y = 0.f;
              if (c0 + j + 2 >= p.V_local) wb.x = 0.f;
              if (c0 + j + 3 >= p.V_local) wb.y = 0.f;
            }
            const float2 la = __fadd2_rn(make_float2(l0, l1), wa), lb = __fadd2_rn(make_float2(l2, l3), wb);
            l0 = la.x; l1 = la.y; l2 = lb.x; l3 = lb.y;
          }
        }
        tc_fence_before();
        mbar_arrive(&ctl->tempty[buf]);                  // this thread is done reading the buffer
      }
      if (ok && row < p.N) {
        const int slot = s * 2 + half;
        p.l_part[int64_t(slot) * p.N + row] = (l0 + l1) + (l2 + l3);
        p.zt_part[int64_t(slot) * p.N + row] = zt;
        if (LOG2N == LOG2N_CE) p.m_part[int64_t(slot) * p.N + row] = m_run;   // (-1e30, 0) when the slot saw no column
      }
    }
  }

  tc_fence_before();
  __syncthreads();
  if (ctl->abort_flag != 0) {
    if (threadIdx.x == 0) {
      if (p.status != nullptr) atomicExch(p.status, ALG_DEV_TIMEOUT);
      // let loads that were already issued land before the CTA's shared memory is released
      const uint64_t t0 = global_timer_ns();
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

template <int LOG2N>
int launch_log2n(const CUtensorMap& tm_h, const CUtensorMap& tm_e, const HeadParams& p, const Plan& pl, int grid,
                 cudaStream_t stream) {
  auto kern = head_tc_kernel<LOG2N>;
  static PerDeviceOnce configured;
  if (int rc = configured.run([&] { return cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, int(SMEM_BYTES)); })) return rc;
  ALG_CUDA_TRY(launch_dependent(kern, dim3(grid), dim3(NTHREADS), SMEM_BYTES, stream, tm_h, tm_e, p, pl.S, pl.tps, pl.units, pl.row_blocks));
  count_launch();
  return ALG_OK;
}

}  // namespace

bool head_tcgen05_supports(const HeadParams& p) {
  return p.d >= BK && p.d % BK == 0 && (p.kind == ALG_HEAD_CE || (p.log2n >= 1 && p.log2n <= 5));
}

int head_tcgen05_splits(int N, int V_local) {
  if (N <= 0 || V_local <= 0) return 2;
  return 2 * make_plan(N, V_local).S;
}

int launch_head_tcgen05(const HeadParams& p, cudaStream_t stream) {
  const Plan pl = make_plan(p.N, p.V_local);
  CUtensorMap tm_h, tm_e;
  {
    const uint64_t dims[2] = {uint64_t(p.d), uint64_t(p.N)};
    const uint64_t strides[1] = {uint64_t(p.d)};
    const uint32_t box[2] = {BK, BM};
    if (int rc = make_tmap_bf16(&tm_h, p.h, 2, dims, strides, box, true)) return rc;
  }
  {
    const uint64_t dims[2] = {uint64_t(p.d), uint64_t(p.V_local)};
    const uint64_t strides[1] = {uint64_t(p.d)};
    const uint32_t box[2] = {BK, BN};
    if (int rc = make_tmap_bf16(&tm_e, p.e, 2, dims, strides, box, true)) return rc;
  }
  const int sms = sm_count();
  const int grid = pl.units < sms ? pl.units : sms;
  if (p.kind == ALG_HEAD_CE) return launch_log2n<LOG2N_CE>(tm_h, tm_e, p, pl, grid, stream);
  switch (p.log2n) {
    case 1: return launch_log2n<1>(tm_h, tm_e, p, pl, grid, stream);
    case 2: return launch_log2n<2>(tm_h, tm_e, p, pl, grid, stream);
    case 3: return launch_log2n<3>(tm_h, tm_e, p, pl, grid, stream);
    case 4: return launch_log2n<4>(tm_h, tm_e, p, pl, grid, stream);
    case 5: return launch_log2n<5>(tm_h, tm_e, p, pl, grid, stream);
  }
  set_error("head: n out of range");
  return ALG_ERR_INVALID;
}

}  // namespace alg
