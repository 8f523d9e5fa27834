// Host-side launch interfaces between the C-ABI layer (c_api.cu) and the kernel files.
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>

#include "common.cuh"

namespace alg {

// ---- qk_prep.cu ---------------------------------------------------------------------
struct PrepParams {
  const void* x;
  void* y;                 // nullptr: statistics only
  const float* gain;       // nullptr: unit gain
  const float* cos;        // nullptr: no rotation
  const float* sin;
  float eps;
  int normalise;           // 0: pass-through (used for guard statistics on ready-made q/k/v)
  int B, H, T, D;
  Strides3 xs, ys;
  int stat_mode;           // 0 none, 1 max squared row norm of round(x*stat_scale), 2 max |x|
  float stat_scale;
  unsigned* stat_out;
};
struct PrepBatch {         // up to three tensors (q, k, v) of one dtype / head_dim in one launch
  PrepParams t[3];
  int count;
};
// backward of the QK RMS-norm (qk_prep.cu): dx, and the gain gradient as per-CTA partial rows summed in order
struct RmsBwdParams {
  const void* x;
  const void* dy;
  const float* gain;       // (D) or nullptr (no gain: dgain is not produced)
  void* dx;
  float* dgain;            // (D) or nullptr
  float* partials;         // (rms_bwd_max_blocks(), D) scratch
  float eps;
  int B, H, T, D;
  Strides3 xs, gs, ds;     // of x, dy, dx
};
int rms_bwd_max_blocks();
int launch_rms_bwd(const RmsBwdParams& p, int dtype, cudaStream_t stream);
int launch_prep(const PrepParams& p, int dtype, cudaStream_t stream);
int launch_prep_batch(const PrepBatch& batch, int dtype, cudaStream_t stream);
int launch_cast(const float* src, void* dst, size_t count, cudaStream_t stream);

// ---- attention ----------------------------------------------------------------------
struct AttnParams {
  const void* q;
  const void* k;
  const void* v;
  void* o;
  float* stat;
  int* stat_kind;
  const float* sink;       // (H) logit units or nullptr
  int B, H, Tq, Tk, D;
  int log2n;
  float scale;             // 1 / (sqrt(D) c): score -> kernel units
  float inv_c;
  int causal;
  int variant;             // ALG_VARIANT_*
  Strides3 qs, ks, vs, os;
  const GuardWords* guard; // required when variant == GUARD
  int guard_slots;         // 0: `guard` is one record; n > 0: n records (one per CTA of the kernel that
                           // took the maxima), the guard's maxima being the largest of each word
  float guard_bound_sq;    // (bound/1.01)^2
  float guard_sink_bound;  // bound/1.01
  float guard_vmax;
  float score_clamp;       // unshifted path: x <- min(x, score_clamp); +inf when off
  int run_if;              // 0 always, 1 only when the guard holds, 2 only when it fails
  int* status;
  GuardWords* guard_out;   // tcgen05 kernel only: CTA i writes the maxima of the rows it looked at to guard_out[i]
  int tc_shift;            // tcgen05 kernel only: launch the max-shifted form (it runs when the shift is called for)
  float* split_ws;         // tcgen05 kernel only: slots for the parts of items split along the keys, or NULL (no splitting)
  int split_slots;         // how many such slots the buffer holds
};
int launch_attn_mma(const AttnParams& p, int dtype, cudaStream_t stream);
bool attn_tcgen05_supports(const AttnParams& p, int dtype);
// Long enough sequences leave one warp of the tcgen05 kernel time to take the guard's maxima itself.
bool attn_tcgen05_takes_guard_statistics(const AttnParams& p);
int attn_tcgen05_grid(const AttnParams& p);          // CTAs of that kernel = records it writes to guard_out
size_t attn_tcgen05_split_bytes(const AttnParams& p);  // workspace the key-split of a short problem would use (0: it would not split)
int launch_attn_tcgen05(const AttnParams& p, cudaStream_t stream);
// fp32 rows of head_dim 64 on the same kernel: q, k, v are first split into bf16 hi | lo tiles (three
// buffers of attn_tcgen05_f32_split_bytes each, at `split`); unshifted form, fp32 output
bool attn_tcgen05_f32_supports(const AttnParams& p, int dtype);
size_t attn_tcgen05_f32_split_bytes(int B, int H, int T);
int launch_attn_tcgen05_f32(const AttnParams& p, void* split, cudaStream_t stream);

// Shared by both attention kernels: does this launch use the max-shifted form?  Called by all 32
// lanes of one warp; every lane gets the answer.
__device__ __forceinline__ bool attn_use_shift(const AttnParams& p, int lane) {
  if (p.variant == ALG_VARIANT_NOSHIFT) return false;
  if (p.variant == ALG_VARIANT_SHIFT) return true;
  bool ok;
  if (p.guard_slots > 0) {                              // per-CTA records: the words order as unsigned integers
    unsigned q2 = 0, k2 = 0, vm = 0;
    for (int i = lane; i < p.guard_slots; i += 32) {
      const uint4 r = *reinterpret_cast<const uint4*>(p.guard + i);
      q2 = max(q2, r.x); k2 = max(k2, r.y); vm = max(vm, r.z);
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      q2 = max(q2, __shfl_xor_sync(0xffffffffu, q2, o));
      k2 = max(k2, __shfl_xor_sync(0xffffffffu, k2, o));
      vm = max(vm, __shfl_xor_sync(0xffffffffu, vm, o));
    }
    ok = (__uint_as_float(q2) * __uint_as_float(k2) <= p.guard_bound_sq) && (__uint_as_float(vm) <= p.guard_vmax);
  } else {
    ok = guard_in_range(p.guard, p.guard_bound_sq, p.guard_vmax);
  }
  if (p.sink != nullptr)
    for (int h = 0; h < p.H; ++h) ok = ok && (fabsf(p.sink[h] * p.inv_c) <= p.guard_sink_bound);
  return !ok;
}

// ---- attn_bwd_mma.cu: attention backward ---------------------------------------------------
struct AttnBwdParams {
  const __nv_bfloat16* q;
  const __nv_bfloat16* k;
  const __nv_bfloat16* v;
  const __nv_bfloat16* o;
  const __nv_bfloat16* d_o;  // strides of o
  const float* stat;         // (B, H, Tq) saved by the forward
  const int* stat_kind;      // device: ALG_VARIANT_NOSHIFT / ALG_VARIANT_SHIFT, as the forward wrote it
  const float* sink;         // (H) or nullptr
  __nv_bfloat16* dq;         // strides of q
  __nv_bfloat16* dk;         // strides of k
  __nv_bfloat16* dv;         // strides of v
  float* dsink;              // (H) or nullptr
  float* delta;              // (B, H, Tq) scratch: dO . o per row
  int B, H, Tq, Tk, D;
  int log2n;
  float scale, inv_c;        // 1 / (sqrt(D) c), 1 / c
  float n_scale, n_f;        // n * scale, n
  int causal;
  Strides3 qs, ks, vs, os;
  int* status;               // device word for ALG_DEV_TIMEOUT, or nullptr
  int force_mma;             // 1: stay on the mma.sync kernels whatever the shape
};
// Dispatcher (attn_bwd_mma.cu): tcgen05 kernels when the shape fits them, else mma.sync.
int launch_attn_bwd(const AttnBwdParams& p, cudaStream_t stream);
// attn_bwd_sm100.cu: causal, Tq == Tk a multiple of 128, head_dim 64 or 128
bool attn_bwd_tcgen05_supports(const AttnBwdParams& p);
int launch_attn_bwd_tcgen05(const AttnBwdParams& p, cudaStream_t stream);

// ---- proj_sm100.cu: projection GEMMs with fused epilogues -------------------------------
struct ProjParams {
  int M, K, N;             // activations (M, K), weights (N, K), both K-major bf16
  int64_t ld_x;
  __nv_bfloat16* out;
  int64_t ld_out;
  // QKV epilogue
  const float* q_gain;
  const float* k_gain;
  const __nv_bfloat16* cos;
  const __nv_bfloat16* sin;
  int H, D, T;
  float eps, q_scale;
  int q_scale_pow2;        // q_scale is an exact power of two (scaling then commutes with rounding)
  GuardWords* guard;
  // GLU epilogue
  int f;
  float beta;
  // head-backward (dz) epilogue
  const int* targets;      // (M) global vocabulary ids
  const float* l;          // (M) row normaliser of the forward, summed over all shards
  const float* zt;         // (M) target logit of the forward
  int vocab_offset, log2n;
  float inv_c, clamp, n_over_c, gscale;   // 1/c, logit clamp, n/c, upstream gradient / M
  int head_kind;                          // ALG_HEAD_ALG_CE, or ALG_HEAD_CE: `l` holds the rows' logsumexp
  int* status;
  // row scale of the QKV / GLU epilogues: tau = rsqrt(sum over slots of row_ss[slot][row] / K + row_eps)
  const float* row_ss;     // (ss_slots, M) partial sums of squares of the input rows, or nullptr (tau = 1)
  int ss_slots;
  float row_eps;
  // residual epilogue
  const __nv_bfloat16* resid;   // (M, N) added to the product
  int64_t ld_resid;
  float* ss_out;           // (2 * ceil(N / tile width), M) partial sums of squares of the rows written, or nullptr
};
int launch_proj(const ProjParams& p, const void* x, const void* w, int epi, cudaStream_t stream);   // epi 0 QKV, 1 GLU, 2 head dz, 3 residual
int proj_resid_tile_width(int M, int N);
// prefill_ops.cu
int launch_row_sumsq(const void* x, int64_t rows, int d, int64_t ld, float* ss_out, cudaStream_t stream);

// ---- decode -------------------------------------------------------------------------
struct DecodeParams {
  const void* q;
  const void* k;
  const void* v;
  void* o;
  const float* sink;
  int B, H, Tk, D;
  int log2n;
  float scale, inv_c;
  Strides3 ks, vs;
  int splits;
  int keys_per_split;      // multiple of the 64-key tile
  float* part;             // (B*H, splits, D + 2) fp32 partials: acc[D], m, l
  unsigned long long* arrivals;   // (B*H) words: call number << 16 | splits of that call that have written their partial
  unsigned long long call;        // this call's number (unique per process): stale words of other calls read as zero arrivals
  int* status;
};
int decode_splits(int B, int H, int Tk);
int decode_keys_per_split(int B, int H, int Tk);
int launch_decode(const DecodeParams& p, cudaStream_t stream);

// ---- Alg-CE head --------------------------------------------------------------------
struct HeadParams {
  const void* h;
  const void* e;
  const int32_t* targets;
  float* l_out;
  float* zt_out;
  int N, d, V_local, vocab_offset;
  int log2n;
  float inv_c, clamp;
  int splits;              // vocab splits per row block (partials reduced by head_reduce)
  float* l_part;           // (splits, N)
  float* zt_part;          // (splits, N)
  int* status;
  int kind;                // ALG_HEAD_ALG_CE, or ALG_HEAD_CE: softmax cross-entropy, l_out = logsumexp
  float* m_part;           // (splits, N) running maxima of the partial sums, ALG_HEAD_CE only
};
int head_mma_splits(int N, int V_local);
int launch_head_mma(const HeadParams& p, cudaStream_t stream);
bool head_tcgen05_supports(const HeadParams& p);
int head_tcgen05_splits(int N, int V_local);
int launch_head_tcgen05(const HeadParams& p, cudaStream_t stream);
int launch_head_reduce(const HeadParams& p, cudaStream_t stream);
int launch_head_finalize(const float* l, const float* zt, int N, int log2n, float inv_c, float clamp,
                         float* pt, float* nll, float* obj, float* block_sums, unsigned* ticket,
                         cudaStream_t stream);
int head_finalize_blocks(int N);
// ---- head_exchange.cu: split reduction + peer-memory exchange + telemetry in one kernel
struct ExchangeParams {
  const float* l_part;
  const float* zt_part;
  int slots, N;
  int N_capacity;                        // rows the exchange region was sized for (layout of its planes)
  int log2n;
  float inv_c, clamp;
  int rank, world;
  float* peer_data[ALG_MAX_RANKS];       // every rank's exchange data, mapped on this device
  unsigned* peer_flags[ALG_MAX_RANKS];   // every rank's flag table [world][128]
  unsigned* call_counter;                // local, persists across calls
  unsigned* ticket;
  float* block_sums;
  float* l_out;                          // optional: world totals
  float* zt_out;
  float* pt;
  float* nll;
  float* obj;
  int* status;
  unsigned long long budget_ns;
};
int head_exchange_blocks(int N);
int launch_head_exchange(const ExchangeParams& p, cudaStream_t stream);
// c_api.cu: argument checks + HeadParams derivation common to the head entry points
extern "C" int head_fill(const alg_head_args* a, HeadParams* p, bool* use_fast);

}  // namespace alg
