/*
 * alg_b200 — C ABI of the B200 (sm_100a) kernels for the Algebraic Transformer's
 * forward hot path: QK RMS-norm + Cayley rotation, asinh-power attention, the
 * fused Alg-CE head, and single-query decode.
 *
 * Conventions
 *   - every pointer is a DEVICE pointer unless the comment says "host";
 *   - the library allocates nothing: outputs, workspaces and the status word are
 *     the caller's; `alg_*_workspace_bytes` says how much scratch a call needs;
 *   - calls only enqueue work on `stream` (a cudaStream_t passed as void*), they
 *     never synchronise;
 *   - return value 0 = enqueued, < 0 = ALG_ERR_* raised BEFORE any launch, with a
 *     human-readable reason in alg_last_error() (thread-local);
 *   - device-side problems (a bounded wait that ran out) are reported through the
 *     caller's `status` word: it is left untouched on success and set to a non-zero
 *     ALG_DEV_* code otherwise; the kernel returns instead of trapping.
 *
 * Each entry point names the reference interface it stands in for, by the file's
 * path inside the reference project (tasmaikeni13/algebraic-transformer).
 */
#ifndef ALG_B200_H_
#define ALG_B200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define ALG_B200_VERSION 100

#if defined(__GNUC__)
#define ALG_API __attribute__((visibility("default")))
#else
#define ALG_API
#endif

enum {
  ALG_OK = 0,
  ALG_ERR_INVALID = -1,      /* bad shape / dtype / null pointer / alignment      */
  ALG_ERR_UNSUPPORTED = -2,  /* valid request this build has no kernel for        */
  ALG_ERR_CUDA = -3,         /* a CUDA runtime / driver call failed               */
  ALG_ERR_WORKSPACE = -4     /* workspace missing or smaller than required        */
};

enum { ALG_DEV_OK = 0, ALG_DEV_TIMEOUT = 1, ALG_DEV_BAD_STATE = 2 };

enum { ALG_BF16 = 0, ALG_F32 = 1 };

/* Accumulation strategy of the attention weights (src/algebraic/kernels/flash.py:732-760,
 * 834-856): GUARD evaluates the reference's run-time range guard on the device and takes
 * the unshifted fast path when it holds, the max-shifted stable path otherwise. */
enum { ALG_VARIANT_GUARD = 0, ALG_VARIANT_NOSHIFT = 1, ALG_VARIANT_SHIFT = 2 };

/* Which kernel family runs.  AUTO picks the tcgen05/TMEM kernel whenever the shape
 * qualifies and the legacy-MMA kernel otherwise; the other two force one family and
 * fail with ALG_ERR_UNSUPPORTED if it cannot run the request. */
enum { ALG_IMPL_AUTO = 0, ALG_IMPL_MMA = 1, ALG_IMPL_TCGEN05 = 2 };

/* The two kinds of the reference's fused head (src/algebraic/kernels/fused_head.py:260-275):
 * "alg_ce" (the algebraic likelihood) and "ce" (softmax cross-entropy, the control arm). */
enum { ALG_HEAD_ALG_CE = 0, ALG_HEAD_CE = 1 };

ALG_API int alg_version(void);
ALG_API const char* alg_last_error(void);
/* Number of kernels this library has launched in this process so far (diagnostics: lets a
 * caller verify that work ran on the GPU kernels here and count launches per step). */
ALG_API unsigned long long alg_kernel_launches(void);

/* ------------------------------------------------------------------------------------
 * QK RMS normalisation (+ optional Cayley rotation).
 * Replaces: qk_rms_norm(x, gain, eps)          src/algebraic/kernels/qk_norm.py:62-76
 *           rms_norm                            src/algebraic/algebraic.py:76-83
 *           apply_rotary (when cos/sin given)   src/algebraic/algebraic.py:172-179
 * x, y: (B, H, T, D) with D contiguous; `x_stride`/`y_stride` are the element strides of
 * (batch, head, row), so transposed views such as a (B, T, H*D) projection output can be
 * read in place; all 0 means densely packed.  gain: (D) fp32 or NULL (no gain).
 * cos, sin: (T, D/2) fp32 or both NULL.  y may alias x.  D in {64, 128}.
 * ---------------------------------------------------------------------------------- */
typedef struct {
  const void* x;
  void* y;
  const float* gain;
  const float* cos;
  const float* sin;
  float eps;
  int B, H, T, D;
  int dtype;               /* ALG_BF16 | ALG_F32 (input and output) */
  int64_t x_stride[3];     /* elements: batch, head, row; all 0 = contiguous (B,H,T,D) */
  int64_t y_stride[3];
} alg_qk_rms_args;

ALG_API int alg_qk_rms_fwd(const alg_qk_rms_args* args, void* stream);

/* Backward of the QK RMS normalisation (no rotation): dx and the learned-gain gradient.
 * Replaces: the custom VJP of qk_rms_norm      src/algebraic/kernels/qk_norm.py:29-56
 *           (_gain_kernel :20-26 reduces dy * x * tau over row blocks, the partials are summed
 *           afterwards; the input gradient is the autodiff gradient of rms_norm,
 *           src/algebraic/algebraic.py:76-83).
 * x, dy, dx: (B, H, T, D) of one dtype, D contiguous, strides as above (dx may alias dy).
 * gain: (D) fp32 or NULL; dgain: (D) fp32, or NULL when gain is NULL.  workspace:
 * alg_qk_rms_bwd_workspace_bytes(D) bytes (per-CTA partial rows of the gain gradient, added in
 * block order: the result does not depend on scheduling). */
typedef struct {
  const void* x;
  const void* dy;
  const float* gain;
  void* dx;
  float* dgain;
  float eps;
  int B, H, T, D;
  int dtype;               /* ALG_BF16 | ALG_F32 (x, dy and dx) */
  int64_t x_stride[3];
  int64_t dy_stride[3];
  int64_t dx_stride[3];
  void* workspace;
  size_t workspace_bytes;
} alg_qk_rms_bwd_args;
ALG_API size_t alg_qk_rms_bwd_workspace_bytes(int D);
ALG_API int alg_qk_rms_bwd(const alg_qk_rms_bwd_args* args, void* stream);

/* ------------------------------------------------------------------------------------
 * Asinh-power attention forward.
 * Replaces: flash_attention(q,k,v,sink_logit,kind="asinh",n,c,range_guard=...)
 *                                               src/algebraic/kernels/flash.py:763-857
 *           (call site model._attention,       src/algebraic/model.py:145-155)
 *           and, with q_gain/k_gain/cos/sin given, the QK-norm + rotation that precede
 *           it in model._block                  src/algebraic/model.py:170-174
 * q: (B,H,Tq,D), k,v: (B,H,Tk,D), o: (B,H,Tq,D) in `dtype`; D contiguous, other strides
 * free (all 0 = contiguous).  sink: (H) fp32 logit units, or NULL.  stat: (B,H,Tq) fp32
 * or NULL — the per-row statistic a backward pass consumes (flash.py:271-284): 1/l on
 * the unshifted path, rho(-m) l^(-1/n) on the shifted one.  stat_kind (1 int, device,
 * may be NULL) receives which of the two was written (ALG_VARIANT_NOSHIFT/SHIFT).
 * causal: key j visible to query i iff j <= i + (Tk - Tq).  n: power of two in [2, 32].
 * ---------------------------------------------------------------------------------- */
typedef struct {
  const void* q;
  const void* k;
  const void* v;
  void* o;
  float* stat;
  int* stat_kind;
  const float* sink;
  const float* q_gain;     /* fused prologue: all four of q_gain,k_gain,cos,sin or none */
  const float* k_gain;
  const float* cos;
  const float* sin;
  float eps;
  int B, H, Tq, Tk, D;
  int n;
  float c;
  int causal;
  int variant;             /* ALG_VARIANT_* */
  int dtype;               /* ALG_BF16 | ALG_F32 */
  int impl;                /* ALG_IMPL_* */
  float score_clamp;       /* > 0: unshifted weights use min(x, score_clamp), the reference's
                              explicit unguarded shift=False link (flash.py:744-748); <= 0: off */
  int64_t q_stride[3], k_stride[3], v_stride[3], o_stride[3];
  void* workspace;
  size_t workspace_bytes;
  int* status;             /* device int, may be NULL */
  const void* guard_words; /* NULL, or the 16 bytes alg_qkv_proj_fwd filled for these very q, k, v:
                              a guarded call then skips its own statistics pass (not together
                              with the fused prologue) */
} alg_attn_args;

/* A guarded call (variant = ALG_VARIANT_GUARD) without guard_words and without the fused prologue has to
 * take the guard's maxima of q, k, v itself.  On long sequences that the tcgen05 kernel covers
 * (Tq * D >= 786432) that kernel is launched at once for the unshifted form and takes the maxima
 * with one of its own warps, into per-CTA records in the workspace; the stable kernel follows and
 * redoes the work only if the guard failed, so until the call's work has completed o, stat and
 * stat_kind may hold the speculative result.  Otherwise a statistics pass runs first.  Either way
 * the call only enqueues kernels (and at most a 16-byte memset) on `stream`: it creates no stream or
 * event of its own and can be captured into a CUDA graph.
 * bf16 problems with few long items for the GPU's SMs (say two heads of 8192 positions) have those items split
 * along the keys; the parts' accumulators live in the workspace and a second kernel adds them up.
 * alg_attn_workspace_bytes includes that room, and a call that brings less runs unsplit.
 * fp32 rows of head_dim 64 (causal, Tq == Tk, unshifted form or guard, no score clamp) run on
 * the tcgen05 kernel too: q, k, v are copied into the workspace as bf16 hi | lo halves and every product is
 * formed as hi.hi + hi.lo + lo.hi; alg_attn_workspace_bytes includes the room for those copies, and a call that
 * brings less workspace than that runs on the mma.sync kernel instead (same results to the fp32 tolerance). */
ALG_API size_t alg_attn_workspace_bytes(const alg_attn_args* args);
ALG_API int alg_attn_fwd(const alg_attn_args* args, void* stream);

/* ------------------------------------------------------------------------------------
 * Attention backward: dq, dk, dv and dsink from the forward's inputs, output and saved
 * statistic.  Replaces the custom VJP of flash_attention, src/algebraic/kernels/flash.py:333-727
 * (_dq_kernel, _dkv_kernel, _fused_bwd_kernel, _sink_mass_and_slope): the normalised weights of a
 * tile are rebuilt from q, k and `stat`, the (T, T) matrix is never formed.
 * bf16 tensors; q, o, d_o, dq: (B,H,Tq,D), k, v, dk, dv: (B,H,Tk,D), D contiguous, strides as in
 * alg_attn_args (d_o uses o's strides, dq/dk/dv those of q/k/v).  stat: (B,H,Tq) fp32 and
 * stat_kind (1 device int) exactly as alg_attn_fwd wrote them.  sink, dsink: (H) fp32 or NULL
 * (dsink is zeroed, then accumulated).  workspace: B*H*Tq floats.
 * ---------------------------------------------------------------------------------- */
typedef struct {
  const void* q;
  const void* k;
  const void* v;
  const void* o;
  const void* d_o;
  const float* stat;
  const int* stat_kind;
  const float* sink;
  void* dq;
  void* dk;
  void* dv;
  float* dsink;
  int B, H, Tq, Tk, D;
  int n;
  float c;
  int causal;
  int64_t q_stride[3], k_stride[3], v_stride[3], o_stride[3];
  void* workspace;
  size_t workspace_bytes;
  int* status;             /* device int, may be NULL */
  int impl;                /* 0: tcgen05 kernels when causal, Tq == Tk, Tq % 128 == 0 (else mma.sync); 1: mma.sync */
} alg_attn_bwd_args;
ALG_API size_t alg_attn_bwd_workspace_bytes(const alg_attn_bwd_args* args);
ALG_API int alg_attn_bwd(const alg_attn_bwd_args* args, void* stream);

/* ------------------------------------------------------------------------------------
 * Single-query decode against a KV cache (Tq = 1, every key visible), split over keys.
 * No reference kernel exists (the reference re-runs the full forward per token,
 * src/algebraic/benchmarking.py:250-263); semantics are asinh_power_weights with an
 * all-true mask, src/algebraic/algebraic.py:186-204.  Uses the max-shifted form.
 * q: (B,H,1,D), k,v: (B,H,Tk,D) bf16, o: (B,H,1,D) bf16.
 * One launch: the CTA that finishes last for a (batch, head) merges the splits' states.  The workspace
 * (16-byte aligned) holds those states and one arrival word per (batch, head); it needs no
 * initialisation, but two calls in flight at the same time must not share one.
 * ---------------------------------------------------------------------------------- */
typedef struct {
  const void* q;
  const void* k;
  const void* v;
  void* o;
  const float* sink;
  int B, H, Tk, D;
  int n;
  float c;
  int64_t k_stride[3], v_stride[3];
  void* workspace;
  size_t workspace_bytes;
} alg_decode_args;

ALG_API size_t alg_decode_workspace_bytes(const alg_decode_args* args);
ALG_API int alg_attn_decode(const alg_decode_args* args, void* stream);

/* ------------------------------------------------------------------------------------
 * Fused Alg-CE head, forward, over one vocabulary shard.
 * Replaces: fused_head(h, embed, targets, kind="alg_ce", n, c)
 *                                               src/algebraic/kernels/fused_head.py:260-275
 *           (_fwd_kernel :72-117; call site model.head_loss, src/algebraic/model.py:211-231)
 * h: (N,d) bf16.  e: (V_local,d) bf16 — rows [vocab_offset, vocab_offset+V_local) of the
 * tied embedding, already cast.  targets: (N) int32 GLOBAL ids.  Outputs, fp32 (N):
 *   l_out  = sum over the shard's columns of rho_fast(min(z/c, clamp))^n
 *   zt_out = the target's logit if the target lies in this shard, else 0
 * with clamp = 0.25 (1e38 / V_total)^(1/n).  No (N x V) logits are written anywhere.
 * Summing l_out and zt_out over shards (one all-reduce) gives the full statistic.
 * kind = ALG_HEAD_CE (fused_head's kind="ce", _fwd_kernel :87-94, 113-114): n and c are ignored and
 *   l_out = logsumexp of the shard's logits (running maximum + rescaled sum, as the reference);
 * shards then combine by logsumexp, not by a sum.  This kind runs on the tcgen05 kernel only
 * (d a multiple of 64) and is not offered by alg_head_fwd_static / alg_head_fwd_exchange.
 * ---------------------------------------------------------------------------------- */
typedef struct {
  const void* h;
  const void* e;
  const int32_t* targets;
  float* l_out;
  float* zt_out;
  int N, d, V_local, vocab_offset, V_total;
  int n;
  float c;
  int impl;                /* ALG_IMPL_* */
  void* workspace;
  size_t workspace_bytes;
  int* status;
  int kind;                /* ALG_HEAD_ALG_CE (0) or ALG_HEAD_CE */
} alg_head_args;

ALG_API size_t alg_head_workspace_bytes(const alg_head_args* args);
ALG_API int alg_head_fwd(const alg_head_args* args, void* stream);

/* The same computation as alg_head_fwd for callers that cannot allocate device memory and
 * therefore cannot supply `workspace` — for example a custom-call handler under a runtime
 * that owns every device buffer and hands the handler only its operands and results, or a
 * long-running server whose memory plan is frozen after start-up.
 * This entry point has no counterpart in the reference.
 *   - `workspace`, `workspace_bytes` are ignored.  The split partials go to a fixed array
 *     of ALG_HEAD_STATIC_SCRATCH_BYTES compiled into the library; every GPU that loads the
 *     library keeps that much memory reserved until the process ends.
 *   - Limit: 8 * N * (partial slots) bytes must fit in the array — N = 8192 tokens with the
 *     full 50304-row vocabulary does; larger problems are refused with ALG_ERR_WORKSPACE
 *     and a message, and should use alg_head_fwd.
 *   - It calls no cudaMalloc / cudaFree and no allocating library routine.  The first call
 *     on each device looks up the array's device address (with that device current); make
 *     that first call outside any stream capture.
 *   - All calls on a device share the one array, and a call overwrites what the previous
 *     one left there (nothing in it has to be cleared).  Two calls whose kernels may
 *     overlap on the GPU — different streams, no ordering between them — race on it;
 *     serialise them, or give one of them alg_head_fwd with its own workspace.
 * Inputs, outputs and results are exactly those of alg_head_fwd. */
#define ALG_HEAD_STATIC_SCRATCH_BYTES (4u << 20)
ALG_API int alg_head_fwd_static(const alg_head_args* args, void* stream);

/* ------------------------------------------------------------------------------------
 * Vocabulary-sharded head with the cross-GPU exchange fused in: runs the shard's GEMM +
 * statistic kernel, then ONE kernel that sums the split partials, writes this rank's
 * per-row (l, zt) into every peer's exchange region over NVLink (plain peer stores; no
 * TMA, no multicast), waits with a bound for the peers' contributions, adds them in rank
 * order (bit-identical totals on every rank) and evaluates pt, nll and the objective.
 * It stands in for alg_head_fwd + an all-reduce + alg_head_finalize; the reference has no
 * multi-device head (its only collective is the trainer's gradient mean,
 * src/algebraic/train.py:245-246).
 *   peer_region[r]: address, valid on THIS device, of rank r's exchange region (own rank
 *     included) of alg_head_exchange_region_bytes(world, N_capacity) bytes, 256-byte
 *     aligned, peer-mapped (e.g. torch symmetric memory, cudaIpc, cuMemMap), zero-filled
 *     once by every rank before the first call, with a barrier after the fill.
 *   Every rank must call with the same N, n, c, V_total, in the same order; one rank per
 *     GPU.  `args->l_out` / `zt_out` may be NULL; when given they receive the world totals.
 *   A wait that runs out (a peer that never arrives) sets `args->status` to
 *     ALG_DEV_TIMEOUT after wait_budget_ns (0 = 1 s); outputs are then undefined.
 * ---------------------------------------------------------------------------------- */
#define ALG_MAX_RANKS 16
typedef struct {
  int rank, world;
  void* peer_region[ALG_MAX_RANKS];
  int N_capacity;
  float* pt;                /* (N) or NULL */
  float* nll;               /* (N) or NULL */
  float* obj;               /* 1 float or NULL */
  unsigned long long wait_budget_ns;
} alg_head_exchange_args;

ALG_API size_t alg_head_exchange_region_bytes(int world, int N_capacity);
ALG_API int alg_head_fwd_exchange(const alg_head_args* args, const alg_head_exchange_args* xargs, void* stream);

/* Telemetry from the (all-reduced) statistic.
 * Replaces: _telemetry + the _inv_root finalize  src/algebraic/kernels/fused_head.py:116,219-229
 *           NLL = -log(max(pt,1e-30))            src/algebraic/train.py:239
 * pt, nll: (N) fp32 (either may be NULL); obj: 1 fp32 = mean(1 - pt) (may be NULL).
 * workspace: alg_head_finalize_workspace_bytes(N) bytes. */
ALG_API size_t alg_head_finalize_workspace_bytes(int N);
ALG_API int alg_head_finalize(const float* l, const float* zt, int N, int n, float c, int V_total,
                      float* pt, float* nll, float* obj,
                      void* workspace, size_t workspace_bytes, void* stream);
/* The same for kind "ce" (_telemetry, fused_head.py:221-223; standard.cross_entropy,
 * src/algebraic/standard.py:41-47): lse = the (shard-combined) logsumexp that alg_head_fwd wrote to
 * l_out; nll = lse - zt, pt = exp(-nll), obj = mean(nll).  Same workspace. */
ALG_API int alg_head_finalize_ce(const float* lse, const float* zt, int N, float* pt, float* nll, float* obj,
                                 void* workspace, size_t workspace_bytes, void* stream);

/* ------------------------------------------------------------------------------------
 * Elementwise stages of the prefill body between the GEMMs (bf16 in / out, fp32 math).
 * Replaces: model._norm = rms_norm over d_model rows   src/algebraic/model.py:141-143,
 *                                                     src/algebraic/algebraic.py:76-83
 *           gate * alu(up, beta) of the ALU-GLU FFN   src/algebraic/model.py:184-193,
 *                                                     src/algebraic/algebraic.py:86-105
 * x, y: (rows, d) bf16 contiguous, d a multiple of 8 and <= 2048; gain: (d) fp32 or NULL.
 * gate, up: (rows, f) bf16 with row stride ld_in elements (the two halves of one fused
 * gate|up GEMM output qualify); out: (rows, f) with row stride ld_out; f and the strides
 * multiples of 8.
 * ---------------------------------------------------------------------------------- */
ALG_API int alg_rms_norm_fwd(const void* x, const float* gain, void* y, int64_t rows, int d, float eps, void* stream);
ALG_API int alg_alu_glu_fwd(const void* gate, const void* up, void* out, int64_t rows, int f, int64_t ld_in,
                            int64_t ld_out, float beta, void* stream);

/* ------------------------------------------------------------------------------------
 * The two wide projections of a prefill block, each one tcgen05 GEMM whose consumer runs in
 * the epilogue on the accumulator tile (bf16 in / out, fp32 accumulation).
 * alg_qkv_proj_fwd replaces, in model._block (src/algebraic/model.py:165-174): the three
 *   projections h @ w_q, h @ w_k, h @ w_v, the QK RMS-norm (model._qk_norm, algebraic.py:76-83)
 *   and apply_rotary (algebraic.py:172-179); it also takes the range guard's maxima
 *   (src/algebraic/kernels/flash.py:831-849) so that alg_attn_fwd(guard_words) need not.
 *   x: (M, d) bf16, row stride ld_x; row m is position m % T of its sequence.
 *   w: (3*H*D, d) bf16 contiguous, one row per output feature: q heads, k heads, v heads.
 *   qkv: (M, 3*H*D) bf16 contiguous out.  cos, sin: (T, D/2) bf16 (the reference casts its
 *   tables to the compute dtype).  q_gain, k_gain: (D) fp32 or NULL.  D = 64 or 128,
 *   d a multiple of 64.  guard: 16 device bytes (zeroed here, then maximised) or NULL.
 * alg_glu_proj_fwd replaces the FFN's gate = h2 @ w_g, up = h2 @ w_u and gate * alu(up, beta)
 *   (src/algebraic/model.py:184-193, algebraic.py:86-105).
 *   w: (2*f, d) bf16 contiguous with the rows interleaved in blocks of 128: gate features
 *   0..127, up features 0..127, gate 128..255, up 128..255, ...; f a multiple of 128.
 *   out: (M, f) bf16 with row stride ld_out.
 * ---------------------------------------------------------------------------------- */
typedef struct {
  const void* x;
  const void* w;
  void* qkv;
  const float* q_gain;
  const float* k_gain;
  const void* cos;
  const void* sin;
  float eps;
  int M, d, H, D, T;
  int64_t ld_x;
  float attn_c;            /* q is scaled by 1 / (sqrt(D) attn_c) for the guard's statistic */
  void* guard;
  int* status;             /* device int, may be NULL */
  /* Optional: x is the UN-normalised residual stream and the block's RMS norm (model.py:141-143, 164) is
   * carried by this call: every accumulator row is multiplied by tau = rsqrt(sum_s row_ss[s][row] / d +
   * row_eps) before anything else happens to it, and the caller has multiplied the norm's gain into the
   * columns of w.  row_ss: (ss_slots, M) fp32 as alg_resid_proj_fwd or alg_row_sumsq left them; NULL = off. */
  const float* row_ss;
  int ss_slots;
  float row_eps;
  int guard_is_zero;       /* nonzero: the caller has zeroed `guard` in this stream since it was last maximised, so
                              this call enqueues no memset (a caller with one record per layer zeroes them all at
                              the start of its step, and no memset then sits between two kernels of the step) */
} alg_qkv_proj_args;
ALG_API int alg_qkv_proj_fwd(const alg_qkv_proj_args* args, void* stream);

typedef struct {
  const void* x;
  const void* w;
  void* out;
  int M, d, f;
  int64_t ld_x, ld_out;
  float beta;
  int* status;             /* device int, may be NULL */
  const float* row_ss;     /* as in alg_qkv_proj_args (model.py:184: the norm in front of gate and up) */
  int ss_slots;
  float row_eps;
} alg_glu_proj_args;
ALG_API int alg_glu_proj_fwd(const alg_glu_proj_args* args, void* stream);

/* The block's out-projection and down-projection with their residual add:
 *   out = resid + x . w^T        Replaces: `x + a @ w_o`, `x + (gate * act) @ w_d`   src/algebraic/model.py:183, 193
 * (the product rounded to bf16, then a bf16 add, as the reference's bf16 expression does), and, when
 * ss_out is given, per row the sum of squares of what was written, as alg_resid_proj_ss_slots(M, N)
 * partials of M floats each — what the NEXT projection needs to apply the RMS norm that follows in
 * the reference (model.py:141-143) without a pass of its own (`row_ss` of alg_qkv_proj_fwd /
 * alg_glu_proj_fwd).  x: (M, K) bf16, row stride ld_x; w: (N, K) bf16 contiguous (one row per output
 * feature); resid, out: (M, N) bf16 with row strides ld_resid, ld_out (out may alias resid).
 * K a multiple of 64, N a multiple of 64, strides multiples of 8, pointers 16-byte aligned. */
typedef struct {
  const void* x;
  const void* w;
  const void* resid;
  void* out;
  float* ss_out;           /* (alg_resid_proj_ss_slots(M, N), M) fp32, or NULL */
  int M, K, N;
  int64_t ld_x, ld_resid, ld_out;
  int* status;             /* device int, may be NULL */
} alg_resid_proj_args;
ALG_API int alg_resid_proj_ss_slots(int M, int N);
ALG_API int alg_resid_proj_fwd(const alg_resid_proj_args* args, void* stream);

/* Sum of squares of every row of a (rows, d) bf16 matrix: ss_out[row], one slot, for the first
 * projection of a model (its input comes from the embedding's norm, not from a residual GEMM). */
ALG_API int alg_row_sumsq(const void* x, int64_t rows, int d, int64_t ld_x, float* ss_out, void* stream);

/* Backward of the Alg-CE head, first half: the logit gradient.  Replaces fused_head._bwd_kernel
 * (src/algebraic/kernels/fused_head.py:120-156), which also writes dz in bf16 and leaves
 * dh = dz . E and dE = dz^T . h to library matmuls (fused_head.py:194-216).
 * h: (N, d) bf16; e: (V_local, d) bf16; targets: (N) int32 global ids; l, zt: (N) fp32 — the
 * forward's statistic, l summed over all vocabulary shards (zt is accepted for symmetry with the
 * forward and not read); dz: (N, V_local) bf16 contiguous out, V_local a multiple of 8;
 * upstream = the cotangent of the objective.  As in the reference's custom VJP, the gradient is
 * that of the negative log-likelihood, not of the primal value mean(1 - pt):
 * dz = upstream / N * (n / c) * (p - onehot) / sqrt(1 + x^2), x = min(z / c, clamp), the clamp
 * straight-through (fused_head.py:236-243, src/algebraic/algebraic.py:232-262, 309-316). */
typedef struct {
  const void* h;
  const void* e;
  const int* targets;
  const float* l;
  const float* zt;
  void* dz;
  int N, d, V_local, vocab_offset, V_total;
  int n;
  float c;
  float upstream;
  int* status;             /* device int, may be NULL */
  int kind;                /* ALG_HEAD_ALG_CE (0), or ALG_HEAD_CE: l = the rows' logsumexp from alg_head_fwd,
                              dz = upstream / N * (exp(z - l) - onehot)  (fused_head.py:134-135); n, c ignored */
} alg_head_bwd_args;
ALG_API int alg_head_bwd_dz(const alg_head_bwd_args* args, void* stream);

/* Failure-detection self-test (no counterpart in the reference).  Launches a one-CTA kernel
 * whose threads wait, through the same bounded-wait helper every TMA/tcgen05 kernel here
 * uses, on a barrier that is never signalled.  After `budget_ns` (at most 1 s) the wait
 * gives up: `*status` (device int) becomes ALG_DEV_TIMEOUT, `*waited_ns` (device, may be
 * NULL) the time actually spent, and the kernel returns normally. */
ALG_API int alg_selftest_bounded_wait(int* status, unsigned long long budget_ns, unsigned long long* waited_ns,
                                      void* stream);

/* fp32 -> bf16 cast of the embedding shard (the reference casts E per call,
 * src/algebraic/kernels/fused_head.py:165; model.py:225). */
ALG_API int alg_cast_f32_to_bf16(const float* src, void* dst, size_t count, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* ALG_B200_H_ */
