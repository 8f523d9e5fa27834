// Vocabulary-sharded Alg-CE head: split reduction + cross-GPU exchange + telemetry in ONE kernel.
//
// After head_tc_kernel / head_mma_kernel every rank holds per-row partial (l, zt) slots for its
// vocabulary shard.  This kernel replaces head_reduce + ncclAllReduce + head_finalize:
//   1. each thread sums its row's slots and stores the rank's (l, zt) pair straight into the
//      exchange buffer of EVERY peer over NVLink (plain st.global to peer-mapped memory —
//      no TMA, no multicast), then the block publishes one flag per peer with release
//      semantics at system scope;
//   2. the block waits (bounded) for the same-numbered block of every rank, sums the world's
//      pairs in rank order (so all ranks get bit-identical totals) and evaluates
//      pt = (rho(min(zt/c, clamp)) l^(-1/n))^n, nll, and the objective mean(1 - pt).
// Blocks only ever wait for their own block index on the peers and the grid is at most 128
// blocks of 256 threads, so every block of a launch is resident and no block waits for one
// that cannot be scheduled.  Buffers are double-buffered by call parity and flags carry a
// monotonically increasing call number kept in device memory, which also makes the launch
// replayable from a CUDA graph.  Semantics: src/algebraic/kernels/fused_head.py:116,219-229
// of the reference (telemetry) applied to the shard sums described in include/alg_b200.h.
#include "common.cuh"
#include "launchers.h"
#include "sm100_ptx.cuh"

namespace alg {
namespace {

constexpr int XT = 256;                 // threads per block
constexpr int MAX_BLOCKS = 128;

__device__ __forceinline__ void st_release_sys(unsigned* p, unsigned v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ unsigned ld_acquire_sys(const unsigned* p) {
  unsigned v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}

__global__ void __launch_bounds__(XT) head_exchange_kernel(const ExchangeParams p) {
  __shared__ unsigned s_call;
  __shared__ int s_ok;
  __shared__ float s_red[XT / 32];
  __shared__ bool s_last;
  const int nb = gridDim.x;
  griddep_wait();                 // launched as a programmatic dependent of the head kernel ahead in the stream
  // call number: read by every block at its start; advanced by the last block to finish
  if (threadIdx.x == 0) s_call = *reinterpret_cast<volatile unsigned*>(p.call_counter) + 1u;
  __syncthreads();
  const unsigned call = s_call;
  // Planes are laid out by the region's CAPACITY, not by this call's N: consecutive calls may differ
  // in N, and the two parities must never overlap while a slow peer still reads the previous call's.
  const size_t plane = size_t(2) * p.N_capacity;                   // one rank's (l, zt) pair
  const size_t parity_off = size_t(call & 1u) * p.world * plane;

  // ---- 1. reduce my slots, push to every peer
  for (int i = blockIdx.x * XT + threadIdx.x; i < p.N; i += nb * XT) {
    float l = 0.f, z = 0.f;
    for (int s = 0; s < p.slots; ++s) {
      l += p.l_part[size_t(s) * p.N + i];
      z += p.zt_part[size_t(s) * p.N + i];
    }
    for (int r = 0; r < p.world; ++r) {
      float* dst = p.peer_data[(p.rank + r) % p.world] + parity_off + size_t(p.rank) * plane;
      dst[i] = l;
      dst[p.N + i] = z;
    }
  }
  __threadfence_system();
  __syncthreads();
  if (threadIdx.x < p.world)
    st_release_sys(p.peer_flags[threadIdx.x] + size_t(p.rank) * MAX_BLOCKS + blockIdx.x, call);

  // ---- 2. wait for block `blockIdx.x` of every rank (bounded), then finish locally
  if (threadIdx.x == 0) s_ok = 1;
  __syncthreads();
  if (threadIdx.x < p.world) {
    const unsigned* flag = p.peer_flags[p.rank] + size_t(threadIdx.x) * MAX_BLOCKS + blockIdx.x;
    const uint64_t t0 = sm100::global_timer_ns();
    while (int(ld_acquire_sys(flag) - call) < 0) {
      if (sm100::global_timer_ns() - t0 > p.budget_ns) { s_ok = 0; break; }
    }
  }
  __syncthreads();
  const bool ok = s_ok != 0;
  float miss = 0.f;
  const float* mine = p.peer_data[p.rank] + parity_off;
  for (int i = blockIdx.x * XT + threadIdx.x; i < p.N; i += nb * XT) {
    float l = 0.f, z = 0.f;
    for (int r = 0; r < p.world; ++r) {                            // rank order: same sum everywhere
      l += __ldcg(mine + size_t(r) * plane + i);
      z += __ldcg(mine + size_t(r) * plane + p.N + i);
    }
    const float x = fminf(z * p.inv_c, p.clamp);
    const float ptv = ok ? pow2n_rt(rho_stable(x) * inv_root_rt(l, p.log2n), p.log2n) : 0.f;
    if (p.l_out != nullptr) { p.l_out[i] = l; p.zt_out[i] = z; }
    if (p.pt != nullptr) p.pt[i] = ptv;
    if (p.nll != nullptr) p.nll[i] = -logf(fmaxf(ptv, 1e-30f));
    miss += 1.0f - ptv;
  }
  miss = warp_sum(miss);
  if ((threadIdx.x & 31) == 0) s_red[threadIdx.x >> 5] = miss;
  __syncthreads();
  if (threadIdx.x == 0) {
    float s = 0.f;
    for (int w = 0; w < XT / 32; ++w) s += s_red[w];
    p.block_sums[blockIdx.x] = s;
    if (!ok && p.status != nullptr) atomicExch(p.status, ALG_DEV_TIMEOUT);
    __threadfence();
    s_last = (atomicAdd(p.ticket, 1u) == unsigned(nb) - 1u);
  }
  __syncthreads();
  if (s_last && threadIdx.x == 0) {
    __threadfence();
    float s = 0.f;
    for (int b = 0; b < nb; ++b) s += reinterpret_cast<volatile float*>(p.block_sums)[b];
    if (p.obj != nullptr) *p.obj = s / float(p.N);
    *p.ticket = 0u;
    *reinterpret_cast<volatile unsigned*>(p.call_counter) = call;   // every block has read it by now
  }
}

}  // namespace

int head_exchange_blocks(int N) {
  int nb = (N + XT - 1) / XT;
  if (nb > MAX_BLOCKS) nb = MAX_BLOCKS;
  return nb < 1 ? 1 : nb;
}

int launch_head_exchange(const ExchangeParams& p, cudaStream_t stream) {
  ALG_CUDA_TRY(launch_dependent(head_exchange_kernel, dim3(head_exchange_blocks(p.N)), dim3(XT), 0, stream, p));
  count_launch();
  return ALG_OK;
}

}  // namespace alg

using namespace alg;

namespace {
constexpr size_t kStateBytes = 256, kSumsBytes = 512;
inline size_t align256x(size_t x) { return (x + 255) & ~size_t(255); }
inline size_t flags_bytes(int world) { return align256x(size_t(world) * 128 * sizeof(unsigned)); }
}  // namespace

extern "C" size_t alg_head_exchange_region_bytes(int world, int N_capacity) {
  if (world < 1 || world > ALG_MAX_RANKS || N_capacity < 1) return 0;
  return kStateBytes + kSumsBytes + flags_bytes(world) + size_t(2) * world * 2 * size_t(N_capacity) * sizeof(float);
}

extern "C" int alg_head_fwd_exchange(const alg_head_args* a, const alg_head_exchange_args* x, void* stream_) {
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  if (a == nullptr || x == nullptr) { set_error("head exchange: null argument"); return ALG_ERR_INVALID; }
  if (x->world < 1 || x->world > ALG_MAX_RANKS || x->rank < 0 || x->rank >= x->world) {
    set_error("head exchange: bad rank/world (%d/%d, at most %d ranks)", x->rank, x->world, ALG_MAX_RANKS);
    return ALG_ERR_INVALID;
  }
  if (a->N > x->N_capacity) {
    set_error("head exchange: N=%d exceeds the region's capacity of %d rows", a->N, x->N_capacity);
    return ALG_ERR_WORKSPACE;
  }
  for (int r = 0; r < x->world; ++r)
    if (x->peer_region[r] == nullptr || (reinterpret_cast<uintptr_t>(x->peer_region[r]) & 255)) {
      set_error("head exchange: region of rank %d is null or not 256-byte aligned", r);
      return ALG_ERR_INVALID;
    }
  unsigned char* mine = static_cast<unsigned char*>(x->peer_region[x->rank]);
  alg_head_args tmp = *a;                         // outputs are optional here; the checks want non-null
  if (tmp.l_out == nullptr) tmp.l_out = reinterpret_cast<float*>(mine + kStateBytes);
  if (tmp.zt_out == nullptr) tmp.zt_out = reinterpret_cast<float*>(mine + kStateBytes);
  HeadParams p{};
  bool fast = false;
  if (int rc = head_fill(&tmp, &p, &fast)) return rc;
  if (p.kind != ALG_HEAD_ALG_CE) { set_error("head exchange: only the alg_ce kind (ce shards combine by logsumexp)"); return ALG_ERR_UNSUPPORTED; }
  if (a->N == 0) return ALG_OK;
  const size_t need = size_t(2) * p.splits * size_t(a->N) * sizeof(float);
  if (a->workspace == nullptr || a->workspace_bytes < need || (reinterpret_cast<uintptr_t>(a->workspace) & 15)) {
    set_error("head exchange: workspace of %zu bytes required, got %zu", need, a->workspace_bytes);
    return ALG_ERR_WORKSPACE;
  }
  p.l_part = static_cast<float*>(a->workspace);
  p.zt_part = p.l_part + size_t(p.splits) * a->N;
  if (int rc = fast ? launch_head_tcgen05(p, stream) : launch_head_mma(p, stream)) return rc;

  ExchangeParams e{};
  e.l_part = p.l_part; e.zt_part = p.zt_part; e.slots = p.splits; e.N = a->N; e.N_capacity = x->N_capacity;
  e.log2n = p.log2n; e.inv_c = p.inv_c; e.clamp = p.clamp;
  e.rank = x->rank; e.world = x->world;
  for (int r = 0; r < x->world; ++r) {
    unsigned char* base = static_cast<unsigned char*>(x->peer_region[r]);
    e.peer_flags[r] = reinterpret_cast<unsigned*>(base + kStateBytes + kSumsBytes);
    e.peer_data[r] = reinterpret_cast<float*>(base + kStateBytes + kSumsBytes + flags_bytes(x->world));
  }
  e.call_counter = reinterpret_cast<unsigned*>(mine);
  e.ticket = reinterpret_cast<unsigned*>(mine + 16);
  e.block_sums = reinterpret_cast<float*>(mine + kStateBytes);
  e.l_out = a->l_out; e.zt_out = a->zt_out;
  e.pt = x->pt; e.nll = x->nll; e.obj = x->obj;
  e.status = a->status;
  e.budget_ns = x->wait_budget_ns ? x->wait_budget_ns : 1000000000ull;
  return launch_head_exchange(e, stream);
}
