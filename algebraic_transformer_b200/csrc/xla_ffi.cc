// XLA typed-FFI handlers over the C ABI of include/alg_b200.h: the layer a JAX program binds with
// jax.ffi.register_ffi_target / jax.ffi.ffi_call where the reference issues pl.pallas_call
// (src/algebraic/kernels/flash.py:292-326, fused_head.py:174-191, qk_norm.py:47-54).
//
// Pure argument marshalling: buffers and the stream come from XLA, scratch arrives as an extra
// result buffer sized by the Python side with alg_*_workspace_bytes, nothing is allocated or
// synchronised here, and a failed host-side check becomes ffi::Error::InvalidArgument carrying
// alg_last_error().  Built by algebraic_transformer_b200/build.py only when the jaxlib headers
// can be found (jax.ffi.include_dir()); the rest of the package does not depend on it.
//
//   AlgAttnFwd       q, k, v, sink -> o, stat, stat_kind, workspace        attrs n, c, variant, has_sink, causal
//   AlgQkRmsFwd      x, gain -> y                                           attrs eps
//   AlgQkRmsRotFwd   x, gain, cos, sin -> y                                 attrs eps
//   AlgHeadFwd       h, e, targets -> stats (2, N), workspace               attrs n, c, vocab_offset, vocab_total
//   AlgHeadFinalize  stats -> obj, pt, workspace                            attrs n, c, vocab_total
#include <cuda_runtime.h>

#include <cstdint>

#include "xla/ffi/api/ffi.h"

#include "../../include/alg_b200.h"

namespace ffi = xla::ffi;

namespace {

ffi::Error done(int rc) {
  return rc == ALG_OK ? ffi::Error::Success() : ffi::Error::InvalidArgument(alg_last_error());
}

int dtype_of(ffi::DataType t) { return t == ffi::DataType::BF16 ? ALG_BF16 : (t == ffi::DataType::F32 ? ALG_F32 : -1); }

ffi::Error AttnFwdImpl(cudaStream_t stream, ffi::AnyBuffer q, ffi::AnyBuffer k, ffi::AnyBuffer v,
                       ffi::Buffer<ffi::DataType::F32> sink, ffi::Result<ffi::AnyBuffer> o,
                       ffi::Result<ffi::Buffer<ffi::DataType::F32>> stat, ffi::Result<ffi::Buffer<ffi::DataType::S32>> stat_kind,
                       ffi::Result<ffi::AnyBuffer> workspace, int64_t n, float c, int64_t variant, int64_t has_sink,
                       int64_t causal) {
  const auto qd = q.dimensions(), kd = k.dimensions();          // (B, H, T, D)
  if (qd.size() != 4 || kd.size() != 4) return ffi::Error::InvalidArgument("attention: q, k, v must be (B, H, T, D)");
  alg_attn_args a = {};
  a.q = q.untyped_data(); a.k = k.untyped_data(); a.v = v.untyped_data(); a.o = o->untyped_data();
  a.stat = stat->typed_data(); a.stat_kind = stat_kind->typed_data();
  a.sink = has_sink ? sink.typed_data() : nullptr;
  a.B = int(qd[0]); a.H = int(qd[1]); a.Tq = int(qd[2]); a.Tk = int(kd[2]); a.D = int(qd[3]);
  a.n = int(n); a.c = c; a.causal = int(causal); a.variant = int(variant);
  a.dtype = dtype_of(q.element_type());
  a.workspace = workspace->untyped_data(); a.workspace_bytes = workspace->size_bytes();
  return done(alg_attn_fwd(&a, stream));
}

ffi::Error qk_rms(cudaStream_t stream, ffi::AnyBuffer x, ffi::Buffer<ffi::DataType::F32> gain, const float* cos,
                  const float* sin, ffi::Result<ffi::AnyBuffer> y, float eps) {
  const auto d = x.dimensions();
  if (d.size() != 4) return ffi::Error::InvalidArgument("qk_rms: x must be (B, H, T, D)");
  alg_qk_rms_args a = {};
  a.x = x.untyped_data(); a.y = y->untyped_data(); a.gain = gain.typed_data(); a.cos = cos; a.sin = sin;
  a.eps = eps; a.B = int(d[0]); a.H = int(d[1]); a.T = int(d[2]); a.D = int(d[3]);
  a.dtype = dtype_of(x.element_type());
  return done(alg_qk_rms_fwd(&a, stream));
}

ffi::Error QkRmsFwdImpl(cudaStream_t stream, ffi::AnyBuffer x, ffi::Buffer<ffi::DataType::F32> gain,
                        ffi::Result<ffi::AnyBuffer> y, float eps) {
  return qk_rms(stream, x, gain, nullptr, nullptr, y, eps);
}

ffi::Error QkRmsRotFwdImpl(cudaStream_t stream, ffi::AnyBuffer x, ffi::Buffer<ffi::DataType::F32> gain,
                           ffi::Buffer<ffi::DataType::F32> cos, ffi::Buffer<ffi::DataType::F32> sin,
                           ffi::Result<ffi::AnyBuffer> y, float eps) {
  return qk_rms(stream, x, gain, cos.typed_data(), sin.typed_data(), y, eps);
}

ffi::Error HeadFwdImpl(cudaStream_t stream, ffi::Buffer<ffi::DataType::BF16> h, ffi::Buffer<ffi::DataType::BF16> e,
                       ffi::Buffer<ffi::DataType::S32> targets, ffi::Result<ffi::Buffer<ffi::DataType::F32>> stats,
                       ffi::Result<ffi::AnyBuffer> workspace, int64_t n, float c, int64_t vocab_offset,
                       int64_t vocab_total) {
  const auto hd = h.dimensions(), ed = e.dimensions();          // (N, d), (V_local, d)
  if (hd.size() != 2 || ed.size() != 2 || hd[1] != ed[1]) return ffi::Error::InvalidArgument("head: h (N, d) and e (V, d)");
  alg_head_args a = {};
  a.h = h.untyped_data(); a.e = e.untyped_data(); a.targets = targets.typed_data();
  a.l_out = stats->typed_data(); a.zt_out = stats->typed_data() + hd[0];
  a.N = int(hd[0]); a.d = int(hd[1]); a.V_local = int(ed[0]); a.vocab_offset = int(vocab_offset);
  a.V_total = int(vocab_total > 0 ? vocab_total : ed[0]);
  a.n = int(n); a.c = c; a.impl = ALG_IMPL_AUTO; a.kind = ALG_HEAD_ALG_CE;
  a.workspace = workspace->untyped_data(); a.workspace_bytes = workspace->size_bytes();
  return done(alg_head_fwd(&a, stream));
}

ffi::Error HeadFinalizeImpl(cudaStream_t stream, ffi::Buffer<ffi::DataType::F32> stats,
                            ffi::Result<ffi::Buffer<ffi::DataType::F32>> obj, ffi::Result<ffi::Buffer<ffi::DataType::F32>> pt,
                            ffi::Result<ffi::AnyBuffer> workspace, int64_t n, float c, int64_t vocab_total) {
  const auto d = stats.dimensions();                            // (2, N)
  if (d.size() != 2 || d[0] != 2) return ffi::Error::InvalidArgument("head_finalize: stats must be (2, N)");
  const int N = int(d[1]);
  return done(alg_head_finalize(stats.typed_data(), stats.typed_data() + N, N, int(n), c, int(vocab_total),
                                pt->typed_data(), nullptr, obj->typed_data(), workspace->untyped_data(),
                                workspace->size_bytes(), stream));
}

}  // namespace

XLA_FFI_DEFINE_HANDLER_SYMBOL(AlgAttnFwd, AttnFwdImpl,
                              ffi::Ffi::Bind()
                                  .Ctx<ffi::PlatformStream<cudaStream_t>>()
                                  .Arg<ffi::AnyBuffer>().Arg<ffi::AnyBuffer>().Arg<ffi::AnyBuffer>()
                                  .Arg<ffi::Buffer<ffi::DataType::F32>>()
                                  .Ret<ffi::AnyBuffer>().Ret<ffi::Buffer<ffi::DataType::F32>>()
                                  .Ret<ffi::Buffer<ffi::DataType::S32>>().Ret<ffi::AnyBuffer>()
                                  .Attr<int64_t>("n").Attr<float>("c").Attr<int64_t>("variant")
                                  .Attr<int64_t>("has_sink").Attr<int64_t>("causal"));

XLA_FFI_DEFINE_HANDLER_SYMBOL(AlgQkRmsFwd, QkRmsFwdImpl,
                              ffi::Ffi::Bind()
                                  .Ctx<ffi::PlatformStream<cudaStream_t>>()
                                  .Arg<ffi::AnyBuffer>().Arg<ffi::Buffer<ffi::DataType::F32>>()
                                  .Ret<ffi::AnyBuffer>().Attr<float>("eps"));

XLA_FFI_DEFINE_HANDLER_SYMBOL(AlgQkRmsRotFwd, QkRmsRotFwdImpl,
                              ffi::Ffi::Bind()
                                  .Ctx<ffi::PlatformStream<cudaStream_t>>()
                                  .Arg<ffi::AnyBuffer>().Arg<ffi::Buffer<ffi::DataType::F32>>()
                                  .Arg<ffi::Buffer<ffi::DataType::F32>>().Arg<ffi::Buffer<ffi::DataType::F32>>()
                                  .Ret<ffi::AnyBuffer>().Attr<float>("eps"));

XLA_FFI_DEFINE_HANDLER_SYMBOL(AlgHeadFwd, HeadFwdImpl,
                              ffi::Ffi::Bind()
                                  .Ctx<ffi::PlatformStream<cudaStream_t>>()
                                  .Arg<ffi::Buffer<ffi::DataType::BF16>>().Arg<ffi::Buffer<ffi::DataType::BF16>>()
                                  .Arg<ffi::Buffer<ffi::DataType::S32>>()
                                  .Ret<ffi::Buffer<ffi::DataType::F32>>().Ret<ffi::AnyBuffer>()
                                  .Attr<int64_t>("n").Attr<float>("c").Attr<int64_t>("vocab_offset")
                                  .Attr<int64_t>("vocab_total"));

XLA_FFI_DEFINE_HANDLER_SYMBOL(AlgHeadFinalize, HeadFinalizeImpl,
                              ffi::Ffi::Bind()
                                  .Ctx<ffi::PlatformStream<cudaStream_t>>()
                                  .Arg<ffi::Buffer<ffi::DataType::F32>>()
                                  .Ret<ffi::Buffer<ffi::DataType::F32>>().Ret<ffi::Buffer<ffi::DataType::F32>>()
                                  .Ret<ffi::AnyBuffer>()
                                  .Attr<int64_t>("n").Attr<float>("c").Attr<int64_t>("vocab_total"));
