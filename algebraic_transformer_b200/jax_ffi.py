"""`jax.ffi` binding of the B200 kernels: the functions a JAX program calls where the reference
calls its Pallas kernels, with the reference's signatures.

    flash_attention(q, k, v, sink_logit=None, *, kind, n, c, block, ..., range_guard)   src/algebraic/kernels/flash.py:763-857
    fused_head(h, embed, targets, *, kind, n, c, block_n, block_v)                       src/algebraic/kernels/fused_head.py:260-275
    qk_rms_norm(x, gain, eps=1e-5, *, block=1024)                                        src/algebraic/kernels/qk_norm.py:62-76

Each wrapper validates its arguments as the reference does (same `ValueError`s, raised at trace time),
sizes the scratch buffer on the host with `alg_*_workspace_bytes`, and issues `jax.ffi.ffi_call` on a
target whose handler lives in `csrc/xla_ffi.cc` (library `lib/libalg_b200_xla.so`, built by
`python -m algebraic_transformer_b200.build` when the jaxlib headers are present).  The module imports
without JAX; `available()` says whether the binding can be used and the wrappers raise ImportError with
the reason when it cannot.  Forward only: the reference's custom VJPs stay with the caller.
"""

import ctypes
import math
import os

from . import _lib as L

PKG = os.path.dirname(os.path.abspath(__file__))
XLA_LIB_PATH = os.path.join(PKG, "lib", "libalg_b200_xla.so")

# ffi target name -> handler symbol exported by csrc/xla_ffi.cc
TARGETS = {
    "alg_attn_fwd": "AlgAttnFwd",
    "alg_qk_rms_fwd": "AlgQkRmsFwd",
    "alg_qk_rms_rot_fwd": "AlgQkRmsRotFwd",
    "alg_head_fwd": "AlgHeadFwd",
    "alg_head_finalize": "AlgHeadFinalize",
}

_state = {"registered": False, "why_not": None}


def _register():
    if _state["registered"] or _state["why_not"]:
        return
    try:
        import jax
        import jax.ffi  # noqa: F401
    except Exception as e:                                  # no JAX in this environment
        _state["why_not"] = f"jax is not importable ({e.__class__.__name__}: {e})"
        return
    if not os.path.exists(XLA_LIB_PATH):
        _state["why_not"] = (f"{XLA_LIB_PATH} is missing: run `python -m algebraic_transformer_b200.build` "
                             "in an environment where jax.ffi.include_dir() resolves")
        return
    L.load()                                                # libalg_b200.so first: the handlers link against it
    lib = ctypes.CDLL(XLA_LIB_PATH)
    for target, symbol in TARGETS.items():
        jax.ffi.register_ffi_target(target, jax.ffi.pycapsule(getattr(lib, symbol)), platform="CUDA")
    _state["registered"] = True


def available() -> bool:
    """True when JAX is importable and the handler library is built (registers the targets on first use)."""
    _register()
    return _state["registered"]


def _need():
    _register()
    if not _state["registered"]:
        raise ImportError("the jax.ffi binding of algebraic_transformer_b200 is unavailable: " + _state["why_not"])
    import jax
    import jax.numpy as jnp
    return jax, jnp


def qk_rms_norm(x, gain, eps: float = 1e-5, *, block: int = 1024, cos=None, sin=None):
    """RMS normalisation over the last axis with a learned gain (`algebraic.rms_norm` semantics:
    float32 arithmetic, one rounding to `x.dtype`); `cos`, `sin` (T, D/2) also apply the Cayley rotation."""
    if x.ndim != 4 or x.shape[-1] not in (64, 128):
        raise ValueError("QK RMS kernel needs (B, H, T, D) input with D=64 or D=128")
    if gain.shape != (x.shape[-1],):
        raise ValueError("QK RMS gain shape mismatch")
    if not (eps > 0):
        raise ValueError("QK RMS epsilon must be positive")
    if (cos is None) != (sin is None):
        raise ValueError("cos and sin tables come as a pair")
    jax, jnp = _need()
    if x.dtype not in (jnp.float32, jnp.bfloat16):
        raise ValueError("QK RMS kernel needs float32/BF16 input")
    out = jax.ShapeDtypeStruct(x.shape, x.dtype)
    g = gain.astype(jnp.float32)
    if cos is None:
        return jax.ffi.ffi_call("alg_qk_rms_fwd", out)(x, g, eps=float(eps))
    return jax.ffi.ffi_call("alg_qk_rms_rot_fwd", out)(x, g, cos.astype(jnp.float32), sin.astype(jnp.float32), eps=float(eps))


def flash_attention(q, k, v, sink_logit=None, *, kind: str = "softmax", n: int = 16, c: float = 16.0, block: int = 512,
                    block_q=None, block_k=None, shift=None, range_guard: bool = False, return_stat: bool = False):
    """Causal asinh-power attention on (B, H, T, D), the forward of the reference's `flash_attention`.
    `shift=None` with `range_guard=True` is the reference's guarded dispatch (decided on the device from
    the maxima of q, k, v); `shift=True` forces the max-shifted form, `shift=False` the unshifted one."""
    if kind != "asinh":
        raise NotImplementedError("only kind='asinh' is served by the B200 kernels")
    if q.shape != k.shape or q.shape != v.shape or q.ndim != 4:
        raise ValueError("q, k, v must have the same (B, H, T, D) shape")
    B, H, T, D = q.shape
    if n < 2 or n & (n - 1):
        raise ValueError("asinh kernel needs n to be a power of two")
    bq, bk = block_q or block, block_k or block
    if T % min(bq, T) or T % min(bk, T):
        raise ValueError("sequence length must be divisible by blocks")
    jax, jnp = _need()
    variant = L.ALG_VARIANT_GUARD if (range_guard and shift is None) else (L.ALG_VARIANT_SHIFT if shift in (None, True) else L.ALG_VARIANT_NOSHIFT)
    dtype = L.ALG_BF16 if q.dtype == jnp.bfloat16 else L.ALG_F32
    args = L.AttnArgs(B=B, H=H, Tq=T, Tk=T, D=D, n=int(n), c=float(c), causal=1, variant=variant, dtype=dtype)
    ws_bytes = int(L.load().alg_attn_workspace_bytes(args))
    sink = jnp.zeros((H,), jnp.float32) if sink_logit is None else jnp.reshape(sink_logit, (H,)).astype(jnp.float32)
    o, stat, stat_kind, _ = jax.ffi.ffi_call(
        "alg_attn_fwd",
        (jax.ShapeDtypeStruct(q.shape, q.dtype), jax.ShapeDtypeStruct((B, H, T), jnp.float32),
         jax.ShapeDtypeStruct((1,), jnp.int32), jax.ShapeDtypeStruct((max(ws_bytes, 256),), jnp.uint8)))(
        q, k, v, sink, n=int(n), c=float(c), variant=int(variant), has_sink=int(sink_logit is not None), causal=1)
    return (o, stat, stat_kind) if return_stat else o


def fused_head(h, embed, targets, *, kind: str = "ce", n: int = 16, c: float = 16.0, block_n: int = 128, block_v: int = 512,
               vocab_offset: int = 0, vocab_total: int = 0, axis_name=None):
    """`(objective, p_target)` of the Alg-CE head without forming the logits.  With `axis_name`, `embed` is
    this device's vocabulary shard (rows `vocab_offset ...`) of a `vocab_total`-row embedding and the per-row
    statistic is summed over that mapped axis (`jax.lax.psum`) between the two kernels."""
    if kind != "alg_ce":
        raise NotImplementedError("the jax.ffi binding serves kind='alg_ce'")
    if n < 2 or n & (n - 1):
        raise ValueError("n must be a power of two")
    N, d = h.shape
    if N % min(block_n, N):
        raise ValueError("tokens must be divisible by block_n")
    jax, jnp = _need()
    e = embed.astype(jnp.bfloat16)
    V = int(vocab_total) or e.shape[0]
    args = L.HeadArgs(N=N, d=d, V_local=e.shape[0], vocab_offset=int(vocab_offset), V_total=V, n=int(n), c=float(c))
    lib = L.load()
    ws = jax.ShapeDtypeStruct((int(lib.alg_head_workspace_bytes(args)),), jnp.uint8)
    stats, _ = jax.ffi.ffi_call("alg_head_fwd", (jax.ShapeDtypeStruct((2, N), jnp.float32), ws))(
        h.astype(jnp.bfloat16), e, targets.astype(jnp.int32), n=int(n), c=float(c), vocab_offset=int(vocab_offset),
        vocab_total=V)
    if axis_name is not None:
        stats = jax.lax.psum(stats, axis_name)
    ws2 = jax.ShapeDtypeStruct((int(lib.alg_head_finalize_workspace_bytes(N)),), jnp.uint8)
    obj, pt, _ = jax.ffi.ffi_call(
        "alg_head_finalize", (jax.ShapeDtypeStruct((1,), jnp.float32), jax.ShapeDtypeStruct((N,), jnp.float32), ws2))(
        stats, n=int(n), c=float(c), vocab_total=V)
    return obj[0], jax.lax.stop_gradient(pt)


def inverse_sqrt_dim(head_dim: int) -> float:
    """1 / sqrt(D): the kernels fold it (with 1 / c) into the fp32 score, so callers pass UNSCALED q."""
    return 1.0 / math.sqrt(head_dim)
