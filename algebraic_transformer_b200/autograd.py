"""`torch.autograd.Function` wrappers that tie each forward kernel to the backward half of the
reference's custom VJP, so that `.backward()` flows through the three fused operators the way
`jax.grad` flows through the reference's:

    attention(q, k, v, sink, ...)      src/algebraic/kernels/flash.py:333-857   (dq, dk, dv, dsink)
    head_loss(h, embed, targets, ...)  src/algebraic/kernels/fused_head.py:232-254 (dh, dembed)
    qk_norm(x, gain, eps)              src/algebraic/kernels/qk_norm.py:29-56   (dx, dgain)

Host code only: every tensor operation is one of the calls in `ops`.  bf16 activations, as the
backward kernels require; the head's gradient is the reference's (the gradient of the mean negative
log-likelihood for `alg_ce`, of the mean cross-entropy for `ce`), not the derivative of the
`alg_ce` primal value.
"""

from typing import Optional

import torch

from . import ops


class _Attention(torch.autograd.Function):
    @staticmethod
    def forward(ctx, q, k, v, sink, n, c, causal, range_guard):
        # Without the guard the reference's default would be the unshifted form with a score clamp, whose
        # backward zeroes the slope of clamped scores (flash.py:346, 357-360, 698-704); the backward
        # kernels here rebuild weights from unclamped scores.  So the unguarded differentiable call takes
        # the max-shifted form, which needs no clamp and is exact for any input.
        o, stat, kind = ops.flash_attention(q, k, v, sink, kind="asinh", n=n, c=c, causal=causal,
                                            range_guard=range_guard, shift=None if range_guard else True,
                                            return_stat=True)
        ctx.save_for_backward(q, k, v, o, stat, kind, sink if sink is not None else q.new_empty(0))
        ctx.has_sink, ctx.n, ctx.c, ctx.causal = sink is not None, n, c, causal
        return o

    @staticmethod
    def backward(ctx, d_o):
        q, k, v, o, stat, kind, sink = ctx.saved_tensors
        sink = sink if ctx.has_sink else None
        dq, dk, dv, dsink = ops.flash_attention_backward(q, k, v, o, d_o.to(o.dtype), stat, kind, sink, n=ctx.n,
                                                         c=ctx.c, causal=ctx.causal)
        return dq, dk, dv, dsink, None, None, None, None


def attention(q, k, v, sink_logit: Optional[torch.Tensor] = None, *, n: int = 16, c: float = 8.0,
              causal: bool = True, range_guard: bool = True):
    """Differentiable asinh-power attention on bf16 (B,H,T,D) tensors; `sink_logit` is a float32 (H,)
    tensor or None.  Forward: `ops.flash_attention`; backward: `ops.flash_attention_backward` fed with
    the statistic the forward saved.  `range_guard=False` runs the max-shifted form (never the
    clamped unshifted one, whose clamp the backward kernels do not model)."""
    if sink_logit is not None and (sink_logit.dtype != torch.float32 or sink_logit.shape != (q.shape[1],)):
        raise ValueError("sink_logit must be a float32 tensor of shape (H,)")
    return _Attention.apply(q, k, v, sink_logit, int(n), float(c), bool(causal), bool(range_guard))


class _HeadLoss(torch.autograd.Function):
    @staticmethod
    def forward(ctx, h, embed, targets, kind, n, c):
        e = ops.cast_embedding(embed)
        t = targets.reshape(-1).to(torch.int32).contiguous()
        stats = ops.head_statistic(h, e, t, n=n, c=c, kind=kind)
        obj, tel = ops.head_finalize(stats, n=n, c=c, vocab_total=e.shape[0], kind=kind)
        ctx.save_for_backward(h, e, t, stats)
        ctx.kind, ctx.n, ctx.c, ctx.embed_dtype = kind, n, c, embed.dtype
        ctx.mark_non_differentiable(tel)
        return obj, tel

    @staticmethod
    def backward(ctx, g_obj, _g_tel):
        h, e, t, stats = ctx.saved_tensors
        dh, de = ops.fused_head_backward(h, e, t, stats, n=ctx.n, c=ctx.c, kind=ctx.kind)
        # the kernels ran with a unit cotangent; the real one is a device scalar and scales both results
        return (dh.float() * g_obj).to(h.dtype), (de.float() * g_obj).to(ctx.embed_dtype), None, None, None, None


def head_loss(h, embed, targets, *, kind: str = "alg_ce", n: int = 8, c: float = 2.0):
    """Differentiable fused head on one device: `(objective, telemetry)` like `ops.fused_head` (per-token
    target probability for "alg_ce", per-token nll for "ce"; the telemetry carries no gradient), with
    `objective.backward()` producing the reference's gradients for `h` (N, d) bf16 and `embed` (V, d)."""
    if kind not in ("ce", "alg_ce"):
        raise ValueError(kind)
    if h.ndim != 2 or h.dtype != torch.bfloat16 or embed.ndim != 2 or embed.shape[1] != h.shape[1]:
        raise ValueError("h must be (N, d) bfloat16 and embed (V, d)")
    if embed.shape[0] % 8 or h.shape[1] % 64:
        raise ValueError("the backward kernel needs V to be a multiple of 8 and d a multiple of 64")
    return _HeadLoss.apply(h.contiguous(), embed, targets, kind, int(n), float(c))


class _QkNorm(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, gain, eps):
        ctx.save_for_backward(x, gain if gain is not None else x.new_empty(0))
        ctx.has_gain, ctx.eps = gain is not None, eps
        return ops.qk_rms_norm(x, gain, eps)

    @staticmethod
    def backward(ctx, dy):
        x, gain = ctx.saved_tensors
        dx, dgain = ops.qk_rms_norm_backward(x, gain if ctx.has_gain else None, dy.to(x.dtype), ctx.eps)
        return dx, dgain, None


def qk_norm(x, gain: Optional[torch.Tensor], eps: float = 1e-5):
    """Differentiable QK RMS-norm (no rotation) on (..., D) rows, D in {64, 128}."""
    return _QkNorm.apply(x, gain, float(eps))
