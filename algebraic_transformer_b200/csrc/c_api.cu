// The C ABI declared in include/alg_b200.h: argument validation, workspace carving and
// kernel selection.  Nothing here allocates device memory, creates streams or events, or
// synchronises: every call only enqueues work on the caller's stream.
#include <math.h>
#include <atomic>
#include <mutex>
#include <stdarg.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>

#include "common.cuh"
#include "launchers.h"

namespace alg {

static thread_local char g_err[512] = "";

void set_error(const char* fmt, ...) {
  va_list ap;
  va_start(ap, fmt);
  vsnprintf(g_err, sizeof(g_err), fmt, ap);
  va_end(ap);
}

int cuda_fail(cudaError_t e, const char* what) {
  set_error("CUDA error %d (%s) at %s", int(e), cudaGetErrorString(e), what);
  return ALG_ERR_CUDA;
}

int sm_count() {
  static std::atomic<int> cached[PerDeviceOnce::kMaxDevices];
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= PerDeviceOnce::kMaxDevices) {
    cudaGetLastError();
    return 148;
  }
  int n = cached[dev].load(std::memory_order_relaxed);
  if (n == 0) {
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) {
      cudaGetLastError();
      return 148;
    }
    cached[dev].store(n, std::memory_order_relaxed);
  }
  return n;
}

static std::atomic<unsigned long long> g_launches{0};
void count_launch(int n) { g_launches.fetch_add((unsigned long long)n, std::memory_order_relaxed); }

namespace {

const int64_t kDense[3] = {0, 0, 0};
constexpr size_t kGuardBytes = 8192;                    // 512 guard records of 16 bytes
inline float __int_as_float_host(uint32_t u) { float f; memcpy(&f, &u, 4); return f; }
inline size_t align256(size_t x) { return (x + 255) & ~size_t(255); }
inline size_t elem_size(int dtype) { return dtype == ALG_BF16 ? 2 : 4; }
inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; }

// value^(1/n), n a power of two, by repeated square roots (src/algebraic/kernels/flash.py:106-112)
double root_pow2(double value, int n) {
  while (n > 1) { value = sqrt(value); n /= 2; }
  return value;
}

bool strides_ok(const Strides3& s, int dtype) {
  const int64_t vec = 16 / int64_t(elem_size(dtype));
  return s.b % vec == 0 && s.h % vec == 0 && s.t % vec == 0 && s.t > 0;
}

int check_common(int D, int n, float c, int dtype) {
  if (dtype != ALG_BF16 && dtype != ALG_F32) { set_error("dtype must be ALG_BF16 or ALG_F32"); return ALG_ERR_INVALID; }
  if (D != 64 && D != 128) { set_error("head_dim must be 64 or 128, got %d", D); return ALG_ERR_UNSUPPORTED; }
  if (n < 2 || n > 32 || ilog2_exact(n) < 0) {
    set_error("asinh kernel needs n to be a power of two in [2, 32], got %d", n);
    return ALG_ERR_INVALID;
  }
  if (!(c > 0.0f) || !isfinite(c)) { set_error("asinh scale c must be positive and finite"); return ALG_ERR_INVALID; }
  return ALG_OK;
}

bool attn_has_prologue(const alg_attn_args* a) {
  return a->q_gain != nullptr || a->k_gain != nullptr || a->cos != nullptr || a->sin != nullptr;
}

}  // namespace
}  // namespace alg

using namespace alg;

extern "C" {

int alg_version(void) { return ALG_B200_VERSION; }
const char* alg_last_error(void) { return g_err; }
unsigned long long alg_kernel_launches(void) { return g_launches.load(std::memory_order_relaxed); }

int alg_qk_rms_fwd(const alg_qk_rms_args* a, void* stream) {
  if (a == nullptr || a->x == nullptr || a->y == nullptr) { set_error("qk_rms: null argument"); return ALG_ERR_INVALID; }
  if (a->dtype != ALG_BF16 && a->dtype != ALG_F32) { set_error("QK RMS kernel needs float32/BF16 input"); return ALG_ERR_INVALID; }
  if (a->D != 64 && a->D != 128) { set_error("QK RMS kernel needs D=64 or D=128, got %d", a->D); return ALG_ERR_UNSUPPORTED; }
  if (!(a->eps > 0.0f)) { set_error("QK RMS epsilon must be positive"); return ALG_ERR_INVALID; }
  if (a->B < 0 || a->H < 0 || a->T < 0) { set_error("qk_rms: negative extent"); return ALG_ERR_INVALID; }
  if ((a->cos == nullptr) != (a->sin == nullptr)) { set_error("qk_rms: cos and sin tables come as a pair"); return ALG_ERR_INVALID; }
  PrepParams p{};
  p.x = a->x; p.y = a->y; p.gain = a->gain; p.cos = a->cos; p.sin = a->sin; p.eps = a->eps;
  p.normalise = 1; p.B = a->B; p.H = a->H; p.T = a->T; p.D = a->D;
  p.xs = strides_or_dense(a->x_stride, a->H, a->T, a->D);
  p.ys = strides_or_dense(a->y_stride, a->H, a->T, a->D);
  if (!strides_ok(p.xs, a->dtype) || !strides_ok(p.ys, a->dtype) || !aligned16(a->x) || !aligned16(a->y)) {
    set_error("qk_rms: rows must start on 16-byte boundaries");
    return ALG_ERR_INVALID;
  }
  p.stat_mode = 0; p.stat_scale = 1.0f; p.stat_out = nullptr;
  return launch_prep(p, a->dtype, static_cast<cudaStream_t>(stream));
}

size_t alg_qk_rms_bwd_workspace_bytes(int D) {
  return (D == 64 || D == 128) ? size_t(rms_bwd_max_blocks()) * size_t(D) * sizeof(float) : 0;
}

int alg_qk_rms_bwd(const alg_qk_rms_bwd_args* a, void* stream) {
  if (a == nullptr || a->x == nullptr || a->dy == nullptr || a->dx == nullptr) { set_error("qk_rms backward: null argument"); return ALG_ERR_INVALID; }
  if (a->dtype != ALG_BF16 && a->dtype != ALG_F32) { set_error("QK RMS kernel needs float32/BF16 input"); return ALG_ERR_INVALID; }
  if (a->D != 64 && a->D != 128) { set_error("QK RMS kernel needs D=64 or D=128, got %d", a->D); return ALG_ERR_UNSUPPORTED; }
  if (!(a->eps > 0.0f)) { set_error("QK RMS epsilon must be positive"); return ALG_ERR_INVALID; }
  if (a->B < 0 || a->H < 0 || a->T < 0) { set_error("qk_rms backward: negative extent"); return ALG_ERR_INVALID; }
  if (a->dgain != nullptr && a->gain == nullptr) { set_error("qk_rms backward: dgain without gain"); return ALG_ERR_INVALID; }
  const size_t need = alg_qk_rms_bwd_workspace_bytes(a->D);
  if (a->dgain != nullptr && (a->workspace == nullptr || a->workspace_bytes < need || !aligned16(a->workspace))) {
    set_error("qk_rms backward: workspace of %zu bytes (16-byte aligned) required, got %zu", need, a->workspace_bytes);
    return ALG_ERR_WORKSPACE;
  }
  RmsBwdParams p{};
  p.x = a->x; p.dy = a->dy; p.gain = a->gain; p.dx = a->dx; p.dgain = a->dgain;
  p.partials = static_cast<float*>(a->workspace);
  p.eps = a->eps; p.B = a->B; p.H = a->H; p.T = a->T; p.D = a->D;
  p.xs = strides_or_dense(a->x_stride, a->H, a->T, a->D);
  p.gs = strides_or_dense(a->dy_stride, a->H, a->T, a->D);
  p.ds = strides_or_dense(a->dx_stride, a->H, a->T, a->D);
  if (!strides_ok(p.xs, a->dtype) || !strides_ok(p.gs, a->dtype) || !strides_ok(p.ds, a->dtype) || !aligned16(a->x) ||
      !aligned16(a->dy) || !aligned16(a->dx) || (a->gain != nullptr && !aligned16(a->gain))) {
    set_error("qk_rms backward: rows must start on 16-byte boundaries");
    return ALG_ERR_INVALID;
  }
  return launch_rms_bwd(p, a->dtype, static_cast<cudaStream_t>(stream));
}

static size_t attn_key_split_bytes(const alg_attn_args* a);

size_t alg_attn_workspace_bytes(const alg_attn_args* a) {
  if (a == nullptr) return 0;
  size_t bytes = kGuardBytes;                           // guard words: one record, or one per CTA of the tcgen05 kernel
  if (attn_has_prologue(a)) {
    const size_t es = elem_size(a->dtype);
    bytes += align256(size_t(a->B) * a->H * a->Tq * a->D * es);
    bytes += align256(size_t(a->B) * a->H * a->Tk * a->D * es);
  }
  // fp32 rows the tcgen05 kernel can take (head_dim 64, causal self-attention): room for
  // the bf16 hi | lo copies of q, k, v.  A call that brings less than this runs on the mma.sync kernel.
  if (a->dtype == ALG_F32 && a->D == 64 && a->causal && a->Tq == a->Tk && a->Tq > 0)
    bytes = align256(bytes) + 3 * align256(attn_tcgen05_f32_split_bytes(a->B, a->H, a->Tq));
  // bf16 problems too short to keep every SM busy: slots for the parts of items split along the keys.  A call
  // that brings less than this runs unsplit.
  bytes = align256(bytes) + attn_key_split_bytes(a);
  return bytes;
}

// Workspace the tcgen05 kernel's key split would use for this call (0: not that kernel, or nothing to split).
static size_t attn_key_split_bytes(const alg_attn_args* a) {
  if (a->dtype != ALG_BF16 || !a->causal || a->Tq != a->Tk || a->Tq < 1 || a->B < 1 || a->H < 1 || (a->D != 64 && a->D != 128) ||
      a->variant == ALG_VARIANT_SHIFT || a->impl == ALG_IMPL_MMA || a->score_clamp > 0.0f)
    return 0;
  AttnParams p{};
  p.B = a->B; p.H = a->H; p.Tq = a->Tq; p.Tk = a->Tk; p.D = a->D;
  return attn_tcgen05_split_bytes(p);
}

// The part of the attention workspace every call may need (guard records, prologue outputs): a call
// without the fp32 split buffers is still valid with this much.
static size_t attn_workspace_bytes_without_split(const alg_attn_args* a) {
  size_t bytes = kGuardBytes;
  if (attn_has_prologue(a)) {
    const size_t es = elem_size(a->dtype);
    bytes += align256(size_t(a->B) * a->H * a->Tq * a->D * es);
    bytes += align256(size_t(a->B) * a->H * a->Tk * a->D * es);
  }
  return bytes;
}

int alg_attn_fwd(const alg_attn_args* a, void* stream_) {
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  if (a == nullptr || a->q == nullptr || a->k == nullptr || a->v == nullptr || a->o == nullptr) {
    set_error("attention: null tensor argument");
    return ALG_ERR_INVALID;
  }
  if (int rc = check_common(a->D, a->n, a->c, a->dtype)) return rc;
  if (a->B < 0 || a->H < 0 || a->Tq < 0 || a->Tk < 1) { set_error("attention: bad extents"); return ALG_ERR_INVALID; }
  if (a->causal && a->Tk < a->Tq) { set_error("causal attention needs Tk >= Tq"); return ALG_ERR_INVALID; }
  if (a->variant < ALG_VARIANT_GUARD || a->variant > ALG_VARIANT_SHIFT) { set_error("unknown variant %d", a->variant); return ALG_ERR_INVALID; }
  if (a->impl < ALG_IMPL_AUTO || a->impl > ALG_IMPL_TCGEN05) { set_error("unknown impl %d", a->impl); return ALG_ERR_INVALID; }
  const bool prologue = attn_has_prologue(a);
  if (prologue && ((a->cos == nullptr) != (a->sin == nullptr))) { set_error("attention: cos and sin tables come as a pair"); return ALG_ERR_INVALID; }
  if (prologue && a->Tq != a->Tk) { set_error("attention: the fused QK prologue needs Tq == Tk"); return ALG_ERR_INVALID; }
  const bool guard_given = a->guard_words != nullptr && a->variant == ALG_VARIANT_GUARD;
  if (guard_given && prologue) { set_error("attention: guard_words describe ready-made q, k, v; not with the fused prologue"); return ALG_ERR_INVALID; }
  if (guard_given && !aligned16(a->guard_words)) { set_error("attention: guard_words must be 16-byte aligned"); return ALG_ERR_INVALID; }
  const size_t need = attn_workspace_bytes_without_split(a);
  const bool need_ws = prologue || (a->variant == ALG_VARIANT_GUARD && !guard_given);
  if (need_ws && (a->workspace == nullptr || a->workspace_bytes < need || !aligned16(a->workspace))) {
    set_error("attention: workspace of %zu bytes (16-byte aligned) required, got %zu", need, a->workspace_bytes);
    return ALG_ERR_WORKSPACE;
  }
  if (a->B == 0 || a->H == 0 || a->Tq == 0) return ALG_OK;

  AttnParams p{};
  p.q = a->q; p.k = a->k; p.v = a->v; p.o = a->o; p.stat = a->stat; p.stat_kind = a->stat_kind; p.sink = a->sink;
  p.B = a->B; p.H = a->H; p.Tq = a->Tq; p.Tk = a->Tk; p.D = a->D;
  p.log2n = ilog2_exact(a->n);
  p.scale = float(1.0 / (sqrt(double(a->D)) * double(a->c)));
  p.inv_c = 1.0f / a->c;
  p.causal = a->causal ? 1 : 0;
  p.variant = a->variant;
  p.qs = strides_or_dense(a->q_stride, a->H, a->Tq, a->D);
  p.ks = strides_or_dense(a->k_stride, a->H, a->Tk, a->D);
  p.vs = strides_or_dense(a->v_stride, a->H, a->Tk, a->D);
  p.os = strides_or_dense(a->o_stride, a->H, a->Tq, a->D);
  if (!strides_ok(p.qs, a->dtype) || !strides_ok(p.ks, a->dtype) || !strides_ok(p.vs, a->dtype) ||
      !strides_ok(p.os, a->dtype) || !aligned16(a->q) || !aligned16(a->k) || !aligned16(a->v) || !aligned16(a->o)) {
    set_error("attention: rows must start on 16-byte boundaries");
    return ALG_ERR_INVALID;
  }
  p.status = a->status;
  p.score_clamp = a->score_clamp > 0.0f ? a->score_clamp : __int_as_float_host(0x7f800000);

  unsigned char* ws = static_cast<unsigned char*>(a->workspace);
  // short bf16 problems: the slots for a split along the keys sit at the end of the workspace (a call that
  // brings less runs unsplit)
  {
    const size_t split_bytes = attn_key_split_bytes(a), all_bytes = alg_attn_workspace_bytes(a);
    if (split_bytes > 0 && ws != nullptr && aligned16(ws) && a->workspace_bytes >= all_bytes) {
      p.split_ws = reinterpret_cast<float*>(ws + all_bytes - split_bytes);
      p.split_slots = int(split_bytes / (size_t(2) * 128 * (a->D + 4) * sizeof(float)));
    }
  }
  GuardWords* guard = guard_given ? static_cast<GuardWords*>(const_cast<void*>(a->guard_words)) : reinterpret_cast<GuardWords*>(ws);
  const bool guarded = a->variant == ALG_VARIANT_GUARD;
  // Speculation: when the guard's maxima still have to be measured and the sequences are long, the
  // tcgen05 kernel runs at once, for the unshifted form, and one of its warps takes the maxima of
  // q, k, v beside the attention work; the stable kernel follows and does its work (overwriting o,
  // stat and stat_kind) only if the guard failed.  In-range inputs - the case the guard exists to
  // make fast - then cost no pass over q, k, v at all; out-of-range inputs pay for a discarded kernel.
  const bool speculate = guarded && !guard_given && !prologue && a->impl != ALG_IMPL_MMA && !(a->score_clamp > 0.0f) &&
                         attn_tcgen05_supports(p, a->dtype) && attn_tcgen05_takes_guard_statistics(p);
  if (guarded) {
    // src/algebraic/kernels/flash.py:744-748, 840-849
    const double t = root_pow2(1e37 / (double(a->Tk) + 1.0), a->n);
    const double clamp = 0.5 * (t - 1.0 / t);
    const double bound = fmin(16.0, clamp / 2);
    p.guard = guard;
    p.guard_bound_sq = float((bound / 1.01) * (bound / 1.01));
    p.guard_sink_bound = float(bound / 1.01);
    p.guard_vmax = float(fmin(1e8, 1e37 / ((double(a->Tk) + (a->sink ? 1 : 0)) * pow(2 * bound + 1, a->n))));
  }
  if (speculate) {
    AttnParams ps = p;
    ps.variant = ALG_VARIANT_NOSHIFT;
    ps.run_if = 0;
    ps.guard_out = guard;                               // one record per CTA: no memset, no atomics
    p.guard_slots = attn_tcgen05_grid(p);
    if (size_t(p.guard_slots) * sizeof(GuardWords) > kGuardBytes) { set_error("attention: more CTAs than guard records"); return ALG_ERR_UNSUPPORTED; }
    if (int rc = launch_attn_tcgen05(ps, stream)) return rc;
    p.run_if = 2;                                       // the max-shifted form runs only if the guard failed; its CTAs
    p.tc_shift = 1;                                     // move in as the first kernel's leave and wait there for its records
    return launch_attn_tcgen05(p, stream);
  }
  if (guarded && !guard_given) ALG_CUDA_TRY(cudaMemsetAsync(guard, 0, sizeof(GuardWords), stream));
  if (prologue || (guarded && !guard_given)) {
    const size_t es = elem_size(a->dtype);
    void* qn = ws + kGuardBytes;
    void* kn = ws + kGuardBytes + align256(size_t(a->B) * a->H * a->Tq * a->D * es);
    PrepBatch batch{};
    PrepParams pp{};
    pp.eps = a->eps; pp.B = a->B; pp.H = a->H; pp.D = a->D;
    pp.cos = prologue ? a->cos : nullptr; pp.sin = prologue ? a->sin : nullptr;
    pp.normalise = prologue ? 1 : 0;
    // q
    pp.x = a->q; pp.xs = p.qs; pp.T = a->Tq; pp.gain = a->q_gain;
    pp.y = prologue ? qn : nullptr; pp.ys = strides_or_dense(kDense, a->H, a->Tq, a->D);
    pp.stat_mode = guarded ? 1 : 0; pp.stat_scale = p.scale; pp.stat_out = &guard->q2;
    batch.t[batch.count++] = pp;
    // k
    pp.x = a->k; pp.xs = p.ks; pp.T = a->Tk; pp.gain = a->k_gain;
    pp.y = prologue ? kn : nullptr; pp.ys = strides_or_dense(kDense, a->H, a->Tk, a->D);
    pp.stat_scale = 1.0f; pp.stat_out = &guard->k2;
    batch.t[batch.count++] = pp;
    if (guarded) {                                      // v: max |v| only
      if (prologue) {                                   // q,k are normalised in their own launch
        if (int rc = launch_prep_batch(batch, a->dtype, stream)) return rc;
        batch.count = 0;
      }
      pp.x = a->v; pp.xs = p.vs; pp.y = nullptr; pp.gain = nullptr; pp.cos = nullptr; pp.sin = nullptr;
      pp.normalise = 0; pp.stat_mode = 2; pp.stat_out = &guard->vmax;
      batch.t[batch.count++] = pp;
    }
    if (int rc = launch_prep_batch(batch, a->dtype, stream)) return rc;  // statistics-only tensors share a launch
    if (prologue) {
      p.q = qn; p.k = kn;
      p.qs = strides_or_dense(kDense, a->H, a->Tq, a->D);
      p.ks = strides_or_dense(kDense, a->H, a->Tk, a->D);
    }
  }

  // fp32 rows of head_dim 64: the same tcgen05 kernel on bf16 hi | lo copies, when the caller's workspace has
  // room for them; the max-shifted form (explicit, or a failed guard) stays on the mma.sync kernel
  const size_t split_off = align256(need), split_each = align256(attn_tcgen05_f32_split_bytes(a->B, a->H, a->Tq));
  const bool f32_tc = attn_tcgen05_f32_supports(p, a->dtype) && a->variant != ALG_VARIANT_SHIFT && !(a->score_clamp > 0.0f) &&
                      a->impl != ALG_IMPL_MMA && ws != nullptr && aligned16(ws) && a->workspace_bytes >= split_off + 3 * split_each;
  if (f32_tc) {
    p.run_if = guarded ? 1 : 0;
    if (int rc = launch_attn_tcgen05_f32(p, ws + split_off, stream)) return rc;
    if (!guarded) return ALG_OK;
    p.run_if = 2;                                       // the max-shifted form runs only if the guard failed
    return launch_attn_mma(p, a->dtype, stream);
  }
  // the tcgen05 kernel has the unshifted form without a score clamp and the max-shifted form
  const bool shape_ok = attn_tcgen05_supports(p, a->dtype);
  const bool fast_ok = shape_ok && (a->variant == ALG_VARIANT_SHIFT || !(a->score_clamp > 0.0f));
  if (a->impl == ALG_IMPL_TCGEN05 && !fast_ok) {
    set_error("attention: the tcgen05 kernel covers causal Tq == Tk without a score clamp: bf16 with head_dim 64 or 128, fp32 "
              "with head_dim 64 in the unshifted form given the workspace alg_attn_workspace_bytes asks for");
    return ALG_ERR_UNSUPPORTED;
  }
  if (fast_ok && a->impl != ALG_IMPL_MMA) {
    if (a->variant == ALG_VARIANT_SHIFT) { p.tc_shift = 1; return launch_attn_tcgen05(p, stream); }
    p.run_if = guarded ? 1 : 0;
    if (int rc = launch_attn_tcgen05(p, stream)) return rc;
    if (!guarded) return ALG_OK;
    p.run_if = 2;                                       // the max-shifted form runs only if the guard failed
    p.tc_shift = 1;
    return launch_attn_tcgen05(p, stream);
  }
  p.run_if = 0;
  return launch_attn_mma(p, a->dtype, stream);
}

int alg_qkv_proj_fwd(const alg_qkv_proj_args* a, void* stream_) {
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  if (a == nullptr || a->x == nullptr || a->w == nullptr || a->qkv == nullptr || a->cos == nullptr || a->sin == nullptr) {
    set_error("qkv_proj: null argument");
    return ALG_ERR_INVALID;
  }
  if (a->M < 0 || a->H < 1 || a->T < 1 || (a->D != 64 && a->D != 128) || a->d < 64 || a->d % 64 != 0 || a->ld_x < a->d ||
      a->ld_x % 8 != 0 || !(a->eps > 0.0f) || !(a->attn_c > 0.0f)) {
    set_error("qkv_proj: head_dim 64 or 128, d a multiple of 64, row stride a multiple of 8 and >= d, eps and c positive");
    return ALG_ERR_INVALID;
  }
  if (!aligned16(a->x) || !aligned16(a->w) || !aligned16(a->qkv) || !aligned16(a->cos) || !aligned16(a->sin) ||
      (a->guard != nullptr && !aligned16(a->guard)) || (a->q_gain != nullptr && !aligned16(a->q_gain)) ||
      (a->k_gain != nullptr && !aligned16(a->k_gain))) {
    set_error("qkv_proj: 16-byte alignment required");
    return ALG_ERR_INVALID;
  }
  ProjParams p{};
  p.M = a->M; p.K = a->d; p.N = 3 * a->H * a->D; p.ld_x = a->ld_x;
  p.out = static_cast<__nv_bfloat16*>(a->qkv); p.ld_out = p.N;
  p.q_gain = a->q_gain; p.k_gain = a->k_gain;
  p.cos = static_cast<const __nv_bfloat16*>(a->cos); p.sin = static_cast<const __nv_bfloat16*>(a->sin);
  p.H = a->H; p.D = a->D; p.T = a->T; p.eps = a->eps;
  p.q_scale = float(1.0 / (sqrt(double(a->D)) * double(a->attn_c)));
  {
    int e = 0;
    p.q_scale_pow2 = (frexpf(p.q_scale, &e) == 0.5f && e > -60) ? 1 : 0;
  }
  p.guard = static_cast<GuardWords*>(a->guard);
  p.status = a->status;
  if (a->row_ss != nullptr && (a->ss_slots < 1 || !(a->row_eps > 0.0f) || !aligned16(a->row_ss))) {
    set_error("qkv_proj: row_ss needs ss_slots >= 1, a positive row_eps and 16-byte alignment");
    return ALG_ERR_INVALID;
  }
  p.row_ss = a->row_ss; p.ss_slots = a->ss_slots; p.row_eps = a->row_eps;
  if (a->M == 0) return ALG_OK;
  if (p.guard != nullptr && !a->guard_is_zero) ALG_CUDA_TRY(cudaMemsetAsync(p.guard, 0, sizeof(GuardWords), stream));
  return launch_proj(p, a->x, a->w, 0, stream);
}

int alg_glu_proj_fwd(const alg_glu_proj_args* a, void* stream_) {
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  if (a == nullptr || a->x == nullptr || a->w == nullptr || a->out == nullptr) { set_error("glu_proj: null argument"); return ALG_ERR_INVALID; }
  if (a->M < 0 || a->f < 128 || a->f % 128 != 0 || a->d < 64 || a->d % 64 != 0 || a->ld_x < a->d || a->ld_x % 8 != 0 ||
      a->ld_out < a->f || a->ld_out % 8 != 0) {
    set_error("glu_proj: f a multiple of 128, d a multiple of 64, row strides multiples of 8 and wide enough");
    return ALG_ERR_INVALID;
  }
  if (!aligned16(a->x) || !aligned16(a->w) || !aligned16(a->out)) { set_error("glu_proj: 16-byte alignment required"); return ALG_ERR_INVALID; }
  ProjParams p{};
  p.M = a->M; p.K = a->d; p.N = 2 * a->f; p.ld_x = a->ld_x;
  p.out = static_cast<__nv_bfloat16*>(a->out); p.ld_out = a->ld_out;
  p.f = a->f; p.beta = a->beta; p.D = 64;
  p.status = a->status;
  if (a->row_ss != nullptr && (a->ss_slots < 1 || !(a->row_eps > 0.0f) || !aligned16(a->row_ss))) {
    set_error("glu_proj: row_ss needs ss_slots >= 1, a positive row_eps and 16-byte alignment");
    return ALG_ERR_INVALID;
  }
  p.row_ss = a->row_ss; p.ss_slots = a->ss_slots; p.row_eps = a->row_eps;
  return launch_proj(p, a->x, a->w, 1, stream);
}

int alg_resid_proj_ss_slots(int M, int N) {
  if (M < 1 || N < 1) return 0;
  const int bn = proj_resid_tile_width(M, N);
  return 2 * ((N + bn - 1) / bn);
}

int alg_resid_proj_fwd(const alg_resid_proj_args* a, void* stream_) {
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  if (a == nullptr || a->x == nullptr || a->w == nullptr || a->resid == nullptr || a->out == nullptr) {
    set_error("resid_proj: null argument");
    return ALG_ERR_INVALID;
  }
  if (a->M < 0 || a->K < 64 || a->K % 64 != 0 || a->N < 64 || a->N % 64 != 0 || a->ld_x < a->K || a->ld_x % 8 != 0 ||
      a->ld_resid < a->N || a->ld_resid % 8 != 0 || a->ld_out < a->N || a->ld_out % 8 != 0) {
    set_error("resid_proj: K and N multiples of 64, row strides multiples of 8 and wide enough");
    return ALG_ERR_INVALID;
  }
  if (!aligned16(a->x) || !aligned16(a->w) || !aligned16(a->resid) || !aligned16(a->out) ||
      (a->ss_out != nullptr && !aligned16(a->ss_out))) {
    set_error("resid_proj: 16-byte alignment required");
    return ALG_ERR_INVALID;
  }
  if (a->M == 0) return ALG_OK;
  ProjParams p{};
  p.M = a->M; p.K = a->K; p.N = a->N; p.ld_x = a->ld_x;
  p.out = static_cast<__nv_bfloat16*>(a->out); p.ld_out = a->ld_out;
  p.resid = static_cast<const __nv_bfloat16*>(a->resid); p.ld_resid = a->ld_resid;
  p.ss_out = a->ss_out;
  p.D = 64;
  p.status = a->status;
  return launch_proj(p, a->x, a->w, 3, stream);
}

int alg_row_sumsq(const void* x, int64_t rows, int d, int64_t ld_x, float* ss_out, void* stream) {
  if (rows < 0 || d < 8 || d % 8 != 0 || ld_x < d || ld_x % 8 != 0 || (rows > 0 && (x == nullptr || ss_out == nullptr)) ||
      !aligned16(x)) {
    set_error("row_sumsq: d a multiple of 8, row stride a multiple of 8 and >= d, 16-byte aligned rows");
    return ALG_ERR_INVALID;
  }
  return launch_row_sumsq(x, rows, d, ld_x, ss_out, static_cast<cudaStream_t>(stream));
}

size_t alg_attn_bwd_workspace_bytes(const alg_attn_bwd_args* a) {
  if (a == nullptr || a->B < 0 || a->H < 0 || a->Tq < 0) return 0;
  return size_t(a->B) * a->H * a->Tq * sizeof(float);
}

int alg_attn_bwd(const alg_attn_bwd_args* a, void* stream_) {
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  if (a == nullptr || a->q == nullptr || a->k == nullptr || a->v == nullptr || a->o == nullptr || a->d_o == nullptr ||
      a->stat == nullptr || a->stat_kind == nullptr || a->dq == nullptr || a->dk == nullptr || a->dv == nullptr) {
    set_error("attention backward: null tensor argument");
    return ALG_ERR_INVALID;
  }
  if (int rc = check_common(a->D, a->n, a->c, ALG_BF16)) return rc;
  if (a->B < 0 || a->H < 0 || a->Tq < 0 || a->Tk < 1) { set_error("attention backward: bad extents"); return ALG_ERR_INVALID; }
  if (a->causal && a->Tk < a->Tq) { set_error("causal attention needs Tk >= Tq"); return ALG_ERR_INVALID; }
  if ((a->sink == nullptr) != (a->dsink == nullptr)) { set_error("attention backward: sink and dsink come as a pair"); return ALG_ERR_INVALID; }
  const size_t need = alg_attn_bwd_workspace_bytes(a);
  if (need > 0 && (a->workspace == nullptr || a->workspace_bytes < need || !aligned16(a->workspace))) {
    set_error("attention backward: workspace of %zu bytes (16-byte aligned) required, got %zu", need, a->workspace_bytes);
    return ALG_ERR_WORKSPACE;
  }
  AttnBwdParams p{};
  p.q = static_cast<const __nv_bfloat16*>(a->q); p.k = static_cast<const __nv_bfloat16*>(a->k);
  p.v = static_cast<const __nv_bfloat16*>(a->v); p.o = static_cast<const __nv_bfloat16*>(a->o);
  p.d_o = static_cast<const __nv_bfloat16*>(a->d_o);
  p.stat = a->stat; p.stat_kind = a->stat_kind; p.sink = a->sink;
  p.dq = static_cast<__nv_bfloat16*>(a->dq); p.dk = static_cast<__nv_bfloat16*>(a->dk); p.dv = static_cast<__nv_bfloat16*>(a->dv);
  p.dsink = a->dsink; p.delta = static_cast<float*>(a->workspace);
  p.B = a->B; p.H = a->H; p.Tq = a->Tq; p.Tk = a->Tk; p.D = a->D;
  p.log2n = ilog2_exact(a->n);
  p.scale = float(1.0 / (sqrt(double(a->D)) * double(a->c)));
  p.inv_c = 1.0f / a->c;
  p.n_f = float(a->n);
  p.n_scale = p.n_f * p.scale;
  p.causal = a->causal ? 1 : 0;
  p.status = a->status;
  p.force_mma = a->impl == 1 ? 1 : 0;
  if (a->impl != 0 && a->impl != 1) { set_error("attention backward: impl must be 0 or 1, got %d", a->impl); return ALG_ERR_INVALID; }
  p.qs = strides_or_dense(a->q_stride, a->H, a->Tq, a->D);
  p.ks = strides_or_dense(a->k_stride, a->H, a->Tk, a->D);
  p.vs = strides_or_dense(a->v_stride, a->H, a->Tk, a->D);
  p.os = strides_or_dense(a->o_stride, a->H, a->Tq, a->D);
  if (!strides_ok(p.qs, ALG_BF16) || !strides_ok(p.ks, ALG_BF16) || !strides_ok(p.vs, ALG_BF16) || !strides_ok(p.os, ALG_BF16) ||
      !aligned16(a->q) || !aligned16(a->k) || !aligned16(a->v) || !aligned16(a->o) || !aligned16(a->d_o) ||
      !aligned16(a->dq) || !aligned16(a->dk) || !aligned16(a->dv)) {
    set_error("attention backward: rows must start on 16-byte boundaries");
    return ALG_ERR_INVALID;
  }
  return launch_attn_bwd(p, stream);
}

int alg_head_bwd_dz(const alg_head_bwd_args* a, void* stream_) {
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  if (a == nullptr || a->h == nullptr || a->e == nullptr || a->targets == nullptr || a->l == nullptr || a->zt == nullptr ||
      a->dz == nullptr) {
    set_error("head backward: null argument");
    return ALG_ERR_INVALID;
  }
  if (a->N < 0 || a->V_local < 8 || a->V_local % 8 != 0 || a->d < 64 || a->d % 64 != 0 || a->vocab_offset < 0 ||
      a->vocab_offset + a->V_local > a->V_total) {
    set_error("head backward: V_local a multiple of 8 inside the vocabulary, d a multiple of 64");
    return ALG_ERR_INVALID;
  }
  if (a->kind != ALG_HEAD_ALG_CE && a->kind != ALG_HEAD_CE) { set_error("head backward: unknown kind %d", a->kind); return ALG_ERR_INVALID; }
  const bool ce = a->kind == ALG_HEAD_CE;
  if (!ce && (a->n < 2 || a->n > 32 || ilog2_exact(a->n) < 0 || !(a->c > 0.0f))) { set_error("head backward: n a power of two in [2, 32], c positive"); return ALG_ERR_INVALID; }
  if (!aligned16(a->h) || !aligned16(a->e) || !aligned16(a->dz)) { set_error("head backward: 16-byte alignment required"); return ALG_ERR_INVALID; }
  if (a->N == 0) return ALG_OK;
  ProjParams p{};
  p.M = a->N; p.K = a->d; p.N = a->V_local; p.ld_x = a->d;
  p.out = static_cast<__nv_bfloat16*>(a->dz); p.ld_out = a->V_local;
  p.targets = a->targets; p.l = a->l; p.zt = a->zt;
  p.vocab_offset = a->vocab_offset;
  p.head_kind = a->kind;
  if (!ce) {
    p.log2n = ilog2_exact(a->n);
    p.inv_c = 1.0f / a->c;
    p.clamp = float(0.25 * root_pow2(1e38 / double(a->V_total), a->n));       // fused_head.py:273
    p.n_over_c = float(a->n) / a->c;
  }
  p.gscale = a->upstream / float(a->N);                                        // ce: slope 1 (fused_head.py:240)
  p.D = 64;
  p.status = a->status;
  return launch_proj(p, a->h, a->e, 2, stream);
}

size_t alg_decode_workspace_bytes(const alg_decode_args* a) {
  if (a == nullptr) return 0;
  // the splits' partial states, then one arrival word per (batch, head)
  return align256(size_t(a->B) * a->H * decode_splits(a->B, a->H, a->Tk) * (a->D + 2) * sizeof(float)) + size_t(a->B) * a->H * 8;
}

int alg_attn_decode(const alg_decode_args* a, void* stream) {
  if (a == nullptr || a->q == nullptr || a->k == nullptr || a->v == nullptr || a->o == nullptr) {
    set_error("decode: null tensor argument");
    return ALG_ERR_INVALID;
  }
  if (int rc = check_common(a->D, a->n, a->c, ALG_BF16)) return rc;
  if (a->B < 0 || a->H < 0 || a->Tk < 1) { set_error("decode: bad extents"); return ALG_ERR_INVALID; }
  const size_t need = alg_decode_workspace_bytes(a);
  if (a->workspace == nullptr || a->workspace_bytes < need) {
    set_error("decode: workspace of %zu bytes required, got %zu", need, a->workspace_bytes);
    return ALG_ERR_WORKSPACE;
  }
  DecodeParams p{};
  p.q = a->q; p.k = a->k; p.v = a->v; p.o = a->o; p.sink = a->sink;
  p.B = a->B; p.H = a->H; p.Tk = a->Tk; p.D = a->D;
  p.log2n = ilog2_exact(a->n);
  p.scale = float(1.0 / (sqrt(double(a->D)) * double(a->c)));
  p.inv_c = 1.0f / a->c;
  p.ks = strides_or_dense(a->k_stride, a->H, a->Tk, a->D);
  p.vs = strides_or_dense(a->v_stride, a->H, a->Tk, a->D);
  if (!strides_ok(p.ks, ALG_BF16) || !strides_ok(p.vs, ALG_BF16) || !aligned16(a->q) || !aligned16(a->k) || !aligned16(a->v)) {
    set_error("decode: rows must start on 16-byte boundaries");
    return ALG_ERR_INVALID;
  }
  p.splits = decode_splits(a->B, a->H, a->Tk);
  p.keys_per_split = decode_keys_per_split(a->B, a->H, a->Tk);
  p.status = nullptr;
  p.part = static_cast<float*>(a->workspace);
  if (!aligned16(a->workspace)) { set_error("decode: workspace must be 16-byte aligned"); return ALG_ERR_INVALID; }
  p.arrivals = reinterpret_cast<unsigned long long*>(static_cast<unsigned char*>(a->workspace) +
                                                     align256(size_t(a->B) * a->H * p.splits * (a->D + 2) * sizeof(float)));
  static std::atomic<unsigned long long> calls{0};
  p.call = (calls.fetch_add(1) + 1) & ((1ull << 47) - 1);
  return launch_decode(p, static_cast<cudaStream_t>(stream));
}

// Validation and parameter derivation shared by every head entry point (not exported).
int head_fill(const alg_head_args* a, HeadParams* p, bool* use_fast) {
  if (a == nullptr || a->h == nullptr || a->e == nullptr || a->targets == nullptr || a->l_out == nullptr || a->zt_out == nullptr) {
    set_error("head: null argument");
    return ALG_ERR_INVALID;
  }
  if (a->kind != ALG_HEAD_ALG_CE && a->kind != ALG_HEAD_CE) { set_error("head: unknown kind %d", a->kind); return ALG_ERR_INVALID; }
  const bool ce = a->kind == ALG_HEAD_CE;
  if (!ce && (a->n < 2 || a->n > 32 || ilog2_exact(a->n) < 0)) { set_error("n must be a power of two"); return ALG_ERR_INVALID; }
  if (!ce && (!(a->c > 0.0f) || !isfinite(a->c))) { set_error("head scale c must be positive and finite"); return ALG_ERR_INVALID; }
  if (a->N < 0 || a->d < 8 || a->d % 8 != 0 || a->V_local < 1 || a->V_total < a->V_local || a->vocab_offset < 0 ||
      a->vocab_offset + a->V_local > a->V_total) {
    set_error("head: bad extents (N=%d d=%d V_local=%d offset=%d V_total=%d)", a->N, a->d, a->V_local, a->vocab_offset, a->V_total);
    return ALG_ERR_INVALID;
  }
  if (!aligned16(a->h) || !aligned16(a->e)) { set_error("head: h and e must be 16-byte aligned"); return ALG_ERR_INVALID; }
  if (a->impl < ALG_IMPL_AUTO || a->impl > ALG_IMPL_TCGEN05) { set_error("unknown impl %d", a->impl); return ALG_ERR_INVALID; }
  p->h = a->h; p->e = a->e; p->targets = a->targets; p->l_out = a->l_out; p->zt_out = a->zt_out;
  p->N = a->N; p->d = a->d; p->V_local = a->V_local; p->vocab_offset = a->vocab_offset;
  p->kind = a->kind;
  p->log2n = ce ? -1 : ilog2_exact(a->n);
  p->inv_c = ce ? 1.0f : 1.0f / a->c;
  p->clamp = ce ? 0.0f : float(0.25 * root_pow2(1e38 / double(a->V_total), a->n));   // fused_head.py:273
  p->status = a->status;
  const bool fast = head_tcgen05_supports(*p);
  if ((a->impl == ALG_IMPL_TCGEN05 || ce) && !fast) {
    set_error("head: the tcgen05 kernel (the only one with the ce kind) needs d to be a multiple of 64");
    return ALG_ERR_UNSUPPORTED;
  }
  if (ce && a->impl == ALG_IMPL_MMA) { set_error("head: the ce kind has no legacy-MMA kernel"); return ALG_ERR_UNSUPPORTED; }
  *use_fast = fast && a->impl != ALG_IMPL_MMA;
  p->splits = *use_fast ? head_tcgen05_splits(a->N, a->V_local) : head_mma_splits(a->N, a->V_local);
  return ALG_OK;
}

size_t alg_head_workspace_bytes(const alg_head_args* a) {
  if (a == nullptr) return 0;
  // large enough for either kernel family, so that `impl` can change between calls
  int s = head_mma_splits(a->N, a->V_local);
  const int s2 = head_tcgen05_splits(a->N, a->V_local);
  if (s2 > s) s = s2;
  return align256(size_t(3) * s * size_t(a->N > 0 ? a->N : 0) * sizeof(float));   // l, zt and (ce kind) m partials
}

int alg_head_fwd(const alg_head_args* a, void* stream_) {
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  HeadParams p{};
  bool fast = false;
  if (int rc = head_fill(a, &p, &fast)) return rc;
  if (a->N == 0) return ALG_OK;
  const size_t need = size_t(p.kind == ALG_HEAD_CE ? 3 : 2) * p.splits * size_t(a->N) * sizeof(float);
  if (a->workspace == nullptr || a->workspace_bytes < need || !aligned16(a->workspace)) {
    set_error("head: workspace of %zu bytes required, got %zu", alg_head_workspace_bytes(a), a->workspace_bytes);
    return ALG_ERR_WORKSPACE;
  }
  p.l_part = static_cast<float*>(a->workspace);
  p.zt_part = p.l_part + size_t(p.splits) * a->N;
  p.m_part = p.kind == ALG_HEAD_CE ? p.zt_part + size_t(p.splits) * a->N : nullptr;
  if (int rc = fast ? launch_head_tcgen05(p, stream) : launch_head_mma(p, stream)) return rc;
  return launch_head_reduce(p, stream);
}

size_t alg_head_finalize_workspace_bytes(int N) {
  return align256(size_t(head_finalize_blocks(N > 0 ? N : 0)) * sizeof(float) + 16);
}

int alg_head_finalize(const float* l, const float* zt, int N, int n, float c, int V_total,
                      float* pt, float* nll, float* obj, void* workspace, size_t workspace_bytes, void* stream_) {
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  if (l == nullptr || zt == nullptr || N < 0 || V_total < 1) { set_error("head_finalize: bad argument"); return ALG_ERR_INVALID; }
  if (n < 2 || n > 32 || ilog2_exact(n) < 0) { set_error("n must be a power of two"); return ALG_ERR_INVALID; }
  if (N == 0) return ALG_OK;
  float* sums = nullptr;
  unsigned* ticket = nullptr;
  if (obj != nullptr) {
    if (workspace == nullptr || workspace_bytes < alg_head_finalize_workspace_bytes(N)) {
      set_error("head_finalize: workspace of %zu bytes required", alg_head_finalize_workspace_bytes(N));
      return ALG_ERR_WORKSPACE;
    }
    ticket = static_cast<unsigned*>(workspace);
    sums = reinterpret_cast<float*>(static_cast<unsigned char*>(workspace) + 16);
    ALG_CUDA_TRY(cudaMemsetAsync(ticket, 0, sizeof(unsigned), stream));
  }
  const float clamp = float(0.25 * root_pow2(1e38 / double(V_total), n));
  return launch_head_finalize(l, zt, N, ilog2_exact(n), 1.0f / c, clamp, pt, nll, obj, sums, ticket, stream);
}

int alg_head_finalize_ce(const float* lse, const float* zt, int N, float* pt, float* nll, float* obj,
                         void* workspace, size_t workspace_bytes, void* stream_) {
  cudaStream_t stream = static_cast<cudaStream_t>(stream_);
  if (lse == nullptr || zt == nullptr || N < 0) { set_error("head_finalize_ce: bad argument"); return ALG_ERR_INVALID; }
  if (N == 0) return ALG_OK;
  float* sums = nullptr;
  unsigned* ticket = nullptr;
  if (obj != nullptr) {
    if (workspace == nullptr || workspace_bytes < alg_head_finalize_workspace_bytes(N)) {
      set_error("head_finalize_ce: workspace of %zu bytes required", alg_head_finalize_workspace_bytes(N));
      return ALG_ERR_WORKSPACE;
    }
    ticket = static_cast<unsigned*>(workspace);
    sums = reinterpret_cast<float*>(static_cast<unsigned char*>(workspace) + 16);
    ALG_CUDA_TRY(cudaMemsetAsync(ticket, 0, sizeof(unsigned), stream));
  }
  return launch_head_finalize(lse, zt, N, /*log2n=*/-1, 1.0f, 0.0f, pt, nll, obj, sums, ticket, stream);
}

int alg_cast_f32_to_bf16(const float* src, void* dst, size_t count, void* stream) {
  if (count != 0 && (src == nullptr || dst == nullptr)) { set_error("cast: null argument"); return ALG_ERR_INVALID; }
  if (!aligned16(src) || !aligned16(dst)) { set_error("cast: pointers must be 16-byte aligned"); return ALG_ERR_INVALID; }
  return launch_cast(src, dst, count, static_cast<cudaStream_t>(stream));
}

}  // extern "C"
