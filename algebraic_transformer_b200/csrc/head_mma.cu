// Fused Alg-CE head forward on the legacy warp-level MMA path, plus the split reduction
// and the telemetry finalize shared with the tcgen05 kernel.
//
// z = h . E^T is produced tile by tile (128 tokens x 128 vocabulary columns, K streamed in
// 64-wide chunks through a two-stage cp.async pipeline) and consumed in registers:
// w = rho_fast(min(z/c, clamp))^n is added to the row normaliser, the target column's
// logit is picked by comparison, and the tile is dropped.  Nothing of size N x V exists
// in memory.  Semantics: src/algebraic/kernels/fused_head.py:72-117 of the reference
// (additive accumulation with an upper clamp, columns >= V masked so that rho(0)^n = 1
// never leaks into the normaliser).
//
// Grid = (token blocks, vocabulary splits): every CTA owns 128 tokens and a contiguous
// range of vocabulary tiles and writes one partial (l, zt) pair per token; head_reduce sums
// the splits in a fixed order, so results are run-to-run identical.
#include "common.cuh"
#include "launchers.h"

namespace alg {
namespace {

constexpr int BM = 128, BN = 128, BK = 64, NTHREADS = 256;
constexpr int STAGE_BYTES = (BM + BN) * BK * 2;          // one A chunk + one B chunk

__device__ __forceinline__ void cp_async16(void* dst, const void* src, bool valid) {
  uint32_t d = static_cast<uint32_t>(__cvta_generic_to_shared(dst));
  int sz = valid ? 16 : 0;                                // 0 => destination zero-filled
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(d), "l"(src), "r"(sz));
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;"); }
template <int N> __device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N)); }

__device__ __forceinline__ void ldsm_x4(uint32_t& r0, uint32_t& r1, uint32_t& r2, uint32_t& r3, const void* p) {
  uint32_t a = static_cast<uint32_t>(__cvta_generic_to_shared(p));
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3) : "r"(a));
}
__device__ __forceinline__ void mma_bf16(float* c, const uint32_t* a, uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
               : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
               : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

// 128-byte rows, 16-byte chunk index XOR-swizzled by row so ldmatrix is conflict free.
__device__ __forceinline__ const unsigned char* swz(const unsigned char* tile, int row, int col) {
  return tile + row * 128 + ((((col >> 3) ^ row) & 7) << 4);
}

__device__ __forceinline__ void load_stage(unsigned char* stage, const __nv_bfloat16* hrow0, int rows_h,
                                           const __nv_bfloat16* erow0, int rows_e, int d, int kc) {
  unsigned char* sa = stage;
  unsigned char* sb = stage + BM * BK * 2;
  for (int i = threadIdx.x; i < BM * 8; i += NTHREADS) {
    const int r = i >> 3, c = i & 7;
    const bool ok = r < rows_h;
    cp_async16(sa + r * 128 + (((c ^ r) & 7) << 4), hrow0 + int64_t(ok ? r : 0) * d + kc * BK + c * 8, ok);
  }
  for (int i = threadIdx.x; i < BN * 8; i += NTHREADS) {
    const int r = i >> 3, c = i & 7;
    const bool ok = r < rows_e;
    cp_async16(sb + r * 128 + (((c ^ r) & 7) << 4), erow0 + int64_t(ok ? r : 0) * d + kc * BK + c * 8, ok);
  }
}

__global__ void __launch_bounds__(NTHREADS) head_mma_kernel(const HeadParams p) {
  extern __shared__ __align__(128) unsigned char smem[];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int g = lane >> 2, tq = lane & 3;
  const int row0 = blockIdx.x * BM;
  const int split = blockIdx.y;
  const int ntiles = (p.V_local + BN - 1) / BN;
  const int tps = (ntiles + p.splits - 1) / p.splits;
  const int t_begin = split * tps, t_end = min(ntiles, t_begin + tps);
  const int kchunks = p.d / BK;
  const int rows_h = min(BM, p.N - row0);

  const __nv_bfloat16* hb = reinterpret_cast<const __nv_bfloat16*>(p.h) + int64_t(row0) * p.d;
  const __nv_bfloat16* eb = reinterpret_cast<const __nv_bfloat16*>(p.e);

  const int my_row[2] = {row0 + warp * 16 + g, row0 + warp * 16 + g + 8};
  int tgt[2];
#pragma unroll
  for (int r = 0; r < 2; ++r) tgt[r] = (my_row[r] < p.N ? p.targets[my_row[r]] : -1) - p.vocab_offset;
  float l_acc[2] = {0.f, 0.f}, zt_acc[2] = {0.f, 0.f};

  const int total = (t_end - t_begin) * kchunks;
  if (total > 0) {
    load_stage(smem, hb, rows_h, eb + int64_t(t_begin) * BN * p.d, min(BN, p.V_local - t_begin * BN), p.d, 0);
    cp_async_commit();
  }
  float acc[BN / 8][4];
  for (int it = 0; it < total; ++it) {
    const int tile = t_begin + it / kchunks, kc = it % kchunks;
    if (kc == 0) {
#pragma unroll
      for (int i = 0; i < BN / 8; ++i) { acc[i][0] = acc[i][1] = acc[i][2] = acc[i][3] = 0.f; }
    }
    if (it + 1 < total) {
      const int nt = t_begin + (it + 1) / kchunks, nk = (it + 1) % kchunks;
      load_stage(smem + ((it + 1) & 1) * STAGE_BYTES, hb, rows_h, eb + int64_t(nt) * BN * p.d,
                 min(BN, p.V_local - nt * BN), p.d, nk);
      cp_async_commit();
      cp_async_wait<1>();
    } else {
      cp_async_wait<0>();
    }
    __syncthreads();
    const unsigned char* sa = smem + (it & 1) * STAGE_BYTES;
    const unsigned char* sb = sa + BM * BK * 2;
#pragma unroll
    for (int ks = 0; ks < BK / 16; ++ks) {
      uint32_t a[4];
      ldsm_x4(a[0], a[1], a[2], a[3], swz(sa, warp * 16 + (lane & 15), ks * 16 + (lane >> 4) * 8));
#pragma unroll
      for (int np = 0; np < BN / 16; ++np) {
        uint32_t b0, b1, b2, b3;
        ldsm_x4(b0, b1, b2, b3, swz(sb, np * 16 + (lane & 7) + (lane >> 4) * 8, ks * 16 + ((lane >> 3) & 1) * 8));
        mma_bf16(acc[2 * np], a, b0, b1);
        mma_bf16(acc[2 * np + 1], a, b2, b3);
      }
    }
    __syncthreads();                                     // stage (it&1) may be overwritten next round
    if (kc == kchunks - 1) {
      const int v0 = tile * BN;
      const bool tail = v0 + BN > p.V_local;
      // rho^n as log2n passes over the fragment (independent multiplications in every pass)
      float wt[BN / 8][4];
#pragma unroll
      for (int nt = 0; nt < BN / 8; ++nt)
#pragma unroll
        for (int e = 0; e < 4; ++e) wt[nt][e] = rho_fast(fminf(acc[nt][e] * p.inv_c, p.clamp));
      for (int it = 0; it < p.log2n; ++it) {
#pragma unroll
        for (int nt = 0; nt < BN / 8; ++nt)
#pragma unroll
          for (int e = 0; e < 4; ++e) wt[nt][e] *= wt[nt][e];
      }
#pragma unroll
      for (int nt = 0; nt < BN / 8; ++nt)
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const int col = v0 + nt * 8 + tq * 2 + (e & 1);
          const float z = acc[nt][e];
          float w = wt[nt][e];
          if (tail && col >= p.V_local) w = 0.0f;
          l_acc[e >> 1] += w;
          if (col == tgt[e >> 1]) zt_acc[e >> 1] += z;
        }
    }
  }
#pragma unroll
  for (int r = 0; r < 2; ++r) {
    l_acc[r] += __shfl_xor_sync(0xffffffffu, l_acc[r], 1);
    l_acc[r] += __shfl_xor_sync(0xffffffffu, l_acc[r], 2);
    zt_acc[r] += __shfl_xor_sync(0xffffffffu, zt_acc[r], 1);
    zt_acc[r] += __shfl_xor_sync(0xffffffffu, zt_acc[r], 2);
    if (tq == 0 && my_row[r] < p.N) {
      p.l_part[int64_t(split) * p.N + my_row[r]] = l_acc[r];
      p.zt_part[int64_t(split) * p.N + my_row[r]] = zt_acc[r];
    }
  }
}

// Sums the split partials of a row.  With `m_part` (softmax cross-entropy) a partial is the pair
// (m, sum exp(z - m)) and the result written to l_out is the row's logsumexp m + log l
// (src/algebraic/kernels/fused_head.py:87-94, 113-114).
// A CTA takes 32 rows; thread (row, g) of its 32 x 8 threads adds every eighth split slot of its row (the loads of
// a warp are 32 consecutive rows of one slot), the eight partial sums of a row are then added in a fixed order.  One
// thread per row walking all slots one load latency at a time took 28 us at 2048 rows x 50 slots.
constexpr int RED_ROWS = 32, RED_GROUPS = 8;
__global__ void __launch_bounds__(RED_ROWS * RED_GROUPS)
head_reduce_kernel(const float* __restrict__ l_part, const float* __restrict__ zt_part, const float* __restrict__ m_part, int N,
                   int splits, float* __restrict__ l_out, float* __restrict__ zt_out) {
  griddep_wait();                 // launched as a programmatic dependent of the kernel ahead in the stream
  __shared__ float s_l[RED_GROUPS][RED_ROWS], s_z[RED_GROUPS][RED_ROWS], s_m[RED_GROUPS][RED_ROWS];
  const int rr = threadIdx.x % RED_ROWS, g = threadIdx.x / RED_ROWS;
  const int i = blockIdx.x * RED_ROWS + rr;
  const bool live = i < N;
  float l = 0.f, z = 0.f, m = -1e30f;
  if (live) {
    if (m_part == nullptr) {
#pragma unroll 4
      for (int s = g; s < splits; s += RED_GROUPS) {
        l += l_part[int64_t(s) * N + i];
        z += zt_part[int64_t(s) * N + i];
      }
    } else {
#pragma unroll 4
      for (int s = g; s < splits; s += RED_GROUPS) m = fmaxf(m, m_part[int64_t(s) * N + i]);
    }
  }
  if (m_part != nullptr) {          // softmax cross-entropy: the row's maximum first, then the rescaled sums
    s_m[g][rr] = m;
    __syncthreads();
#pragma unroll
    for (int k = 0; k < RED_GROUPS; ++k) m = fmaxf(m, s_m[k][rr]);
    if (live) {
#pragma unroll 4
      for (int s = g; s < splits; s += RED_GROUPS) {
        l += l_part[int64_t(s) * N + i] * expf(m_part[int64_t(s) * N + i] - m);
        z += zt_part[int64_t(s) * N + i];
      }
    }
  }
  s_l[g][rr] = l;
  s_z[g][rr] = z;
  __syncthreads();
  if (g != 0 || !live) return;
  l = 0.f; z = 0.f;
#pragma unroll
  for (int k = 0; k < RED_GROUPS; ++k) { l += s_l[k][rr]; z += s_z[k][rr]; }
  l_out[i] = (m_part == nullptr) ? l : m + logf(l);
  zt_out[i] = z;
}

constexpr int FIN_THREADS = 256;

// pt = (rho(min(zt/c, clamp)) l^(-1/n))^n, nll = -log(max(pt, 1e-30)), obj = mean(1 - pt).
// src/algebraic/kernels/fused_head.py:116,219-229; src/algebraic/train.py:239.  The mean is
// formed from per-block sums added in block order by the last block to finish.
__global__ void __launch_bounds__(FIN_THREADS) head_finalize_kernel(
    const float* __restrict__ l, const float* __restrict__ zt, int N, int log2n, float inv_c, float clamp,
    float* __restrict__ pt_out, float* __restrict__ nll_out, float* __restrict__ obj_out,
    float* __restrict__ block_sums, unsigned* __restrict__ ticket) {
  griddep_wait();                 // launched as a programmatic dependent of the kernel ahead in the stream
  __shared__ float red[FIN_THREADS / 32];
  __shared__ bool last;
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  float miss = 0.f;
  if (i < N && log2n < 0) {
    // softmax cross-entropy: l holds the logsumexp; nll = lse - zt, objective = mean nll
    // (src/algebraic/kernels/fused_head.py:221-223, src/algebraic/standard.py:41-47)
    const float nll = l[i] - zt[i];
    if (pt_out != nullptr) pt_out[i] = expf(-nll);
    if (nll_out != nullptr) nll_out[i] = nll;
    miss = nll;
  } else if (i < N) {
    const float x = fminf(zt[i] * inv_c, clamp);
    const float ptv = pow2n_rt(rho_stable(x) * inv_root_rt(l[i], log2n), log2n);
    if (pt_out != nullptr) pt_out[i] = ptv;
    if (nll_out != nullptr) nll_out[i] = -logf(fmaxf(ptv, 1e-30f));
    miss = 1.0f - ptv;
  }
  if (obj_out == nullptr) return;
  miss = warp_sum(miss);
  if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = miss;
  __syncthreads();
  if (threadIdx.x == 0) {
    float s = 0.f;
    for (int w = 0; w < FIN_THREADS / 32; ++w) s += red[w];
    block_sums[blockIdx.x] = s;
    __threadfence();
    last = (atomicAdd(ticket, 1u) == gridDim.x - 1);
  }
  __syncthreads();
  if (last && threadIdx.x == 0) {
    __threadfence();
    float s = 0.f;
    for (unsigned b = 0; b < gridDim.x; ++b) s += reinterpret_cast<volatile float*>(block_sums)[b];
    *obj_out = s / float(N);
    *ticket = 0u;                                        // leave the workspace reusable
  }
}

}  // namespace

int head_mma_splits(int N, int V_local) {
  const int row_blocks = (N + BM - 1) / BM;
  const int ntiles = (V_local + BN - 1) / BN;
  int s = (2 * sm_count() + row_blocks - 1) / (row_blocks > 0 ? row_blocks : 1);
  if (s > ntiles) s = ntiles;
  if (s > 64) s = 64;
  return s < 1 ? 1 : s;
}

int launch_head_mma(const HeadParams& p, cudaStream_t stream) {
  if (p.kind != ALG_HEAD_ALG_CE) {
    set_error("head (legacy MMA path): only the alg_ce kind; softmax cross-entropy needs d to be a multiple of 64");
    return ALG_ERR_UNSUPPORTED;
  }
  if (p.d % BK != 0) {
    set_error("head (legacy MMA path): d must be a multiple of %d, got %d", BK, p.d);
    return ALG_ERR_UNSUPPORTED;
  }
  static PerDeviceOnce configured;
  if (int rc = configured.run([&] { return cudaFuncSetAttribute(head_mma_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 2 * STAGE_BYTES); })) return rc;
  dim3 grid((p.N + BM - 1) / BM, p.splits);
  head_mma_kernel<<<grid, NTHREADS, 2 * STAGE_BYTES, stream>>>(p);
  ALG_CUDA_TRY(cudaGetLastError());
  count_launch();
  return ALG_OK;
}

int launch_head_reduce(const HeadParams& p, cudaStream_t stream) {
  ALG_CUDA_TRY(launch_dependent(head_reduce_kernel, dim3((p.N + RED_ROWS - 1) / RED_ROWS), dim3(RED_ROWS * RED_GROUPS), 0, stream, p.l_part, p.zt_part,
                                p.kind == ALG_HEAD_CE ? p.m_part : nullptr, p.N, p.splits, p.l_out, p.zt_out));
  count_launch();
  return ALG_OK;
}

int head_finalize_blocks(int N) { return (N + FIN_THREADS - 1) / FIN_THREADS; }

int launch_head_finalize(const float* l, const float* zt, int N, int log2n, float inv_c, float clamp,
                         float* pt, float* nll, float* obj, float* block_sums, unsigned* ticket,
                         cudaStream_t stream) {
  ALG_CUDA_TRY(launch_dependent(head_finalize_kernel, dim3(head_finalize_blocks(N)), dim3(FIN_THREADS), 0, stream, l, zt, N, log2n, inv_c,
                                clamp, pt, nll, obj, block_sums, ticket));
  count_launch();
  return ALG_OK;
}

}  // namespace alg
