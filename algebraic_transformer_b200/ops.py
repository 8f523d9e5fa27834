"""Python entry points with the reference's call surface, driving the C ABI.

    flash_attention(q, k, v, sink_logit, kind="asinh", n, c, range_guard=...)   src/algebraic/kernels/flash.py:763-772
    fused_head(h, embed, targets, kind="alg_ce", n, c, block_n, block_v)        src/algebraic/kernels/fused_head.py:260
    qk_rms_norm(x, gain, eps, block=...)                                        src/algebraic/kernels/qk_norm.py:62
    position tables cayley_table_geometric(head_dim, seq_len, ...)              src/algebraic/algebraic.py:152-169

Tensors are CUDA `torch.Tensor`s; PyTorch is only the owner of device memory and
streams here.  Every op runs a hand-written sm_100a kernel from
`lib/libalg_b200.so`; there is no eager or CPU fallback, and argument errors are
raised as `ValueError` where the reference raises them.
"""

import functools
import math
from typing import Optional

import torch

from . import _lib as L

_DTYPES = {torch.bfloat16: L.ALG_BF16, torch.float32: L.ALG_F32}
_workspaces = {}


def _stream():
    return torch.cuda.current_stream().cuda_stream


def _ptr(t: Optional[torch.Tensor]):
    return None if t is None else t.data_ptr()


def _workspace(device, nbytes: int, tag: str) -> torch.Tensor:
    """A cached, grow-only scratch buffer per (device, tag): ops enqueue on one stream."""
    key = (device.index, tag)
    buf = _workspaces.get(key)
    if buf is None or buf.numel() < nbytes:
        buf = torch.empty(max(int(nbytes), 256), dtype=torch.uint8, device=device)
        _workspaces[key] = buf
    return buf


def _require_cuda(*tensors):
    for t in tensors:
        if t is not None and not t.is_cuda:
            raise ValueError("algebraic_transformer_b200 ops need CUDA tensors (there is no CPU path)")


def _on_tensor_device(fn):
    """Every op launches on the device that holds its tensors, on that device's current stream.
    All tensor arguments must sit on one device (ValueError otherwise): the C side builds TMA maps
    and launches on the current device, so a tensor from another GPU would be addressed from the
    wrong one.  When the tensors' device is not the current one, the call runs under
    `torch.cuda.device(...)`."""
    @functools.wraps(fn)
    def call(*args, **kwargs):
        dev = None
        for a in list(args) + list(kwargs.values()):
            if isinstance(a, torch.Tensor) and a.device.type == "cuda":
                if dev is None:
                    dev = a.device
                elif a.device != dev:
                    raise ValueError(f"{fn.__name__}: tensors on different devices ({dev} and {a.device})")
        if dev is None or dev.index == torch.cuda.current_device():
            return fn(*args, **kwargs)
        with torch.cuda.device(dev):
            return fn(*args, **kwargs)
    return call


def _strides3(t: torch.Tensor):
    if t.stride(-1) != 1:
        raise ValueError("the last (head_dim) axis must be contiguous")
    return L.I64x3(t.stride(0), t.stride(1), t.stride(2))


def _root(value: float, n: int) -> float:
    out = float(value)
    while n > 1:
        out = math.sqrt(out)
        n //= 2
    return out


# --------------------------------------------------------------------------- tables

def cayley_powers(w: torch.Tensor, seq_len: int):
    """(cos, sin) rows ((1+iw)^2/(1+w^2))^m for m < seq_len, fp32, built on the host by
    binary exponentiation with renormalised squarings (src/algebraic/algebraic.py:124-149).
    Computed once per (head_dim, seq_len); not a hot kernel."""
    w = w.to(torch.float32).cpu()
    w2 = w * w
    c = (1.0 - w2) / (1.0 + w2)
    s = (2.0 * w) / (1.0 + w2)
    pos = torch.arange(seq_len, dtype=torch.int32)
    out_c = torch.ones((seq_len, w.shape[0]), dtype=torch.float32)
    out_s = torch.zeros((seq_len, w.shape[0]), dtype=torch.float32)
    bit = 0
    while (1 << bit) < seq_len:
        take = ((pos >> bit) & 1).bool()[:, None]
        out_c, out_s = (torch.where(take, out_c * c - out_s * s, out_c),
                        torch.where(take, out_c * s + out_s * c, out_s))
        c, s = c * c - s * s, 2.0 * c * s
        inv = torch.rsqrt(c * c + s * s)
        c, s = c * inv, s * inv
        bit += 1
    inv = torch.rsqrt(out_c * out_c + out_s * out_s)
    return out_c * inv, out_s * inv


def cayley_table_geometric(head_dim: int, seq_len: int, base: float = 10000.0, w0: float = 0.5,
                           fraction: float = 1.0, device=None):
    """Geometric frequency grid w_k = w0 base^(-k/half); tables of shape (T, D/2)."""
    half = head_dim // 2
    levels = int(round(math.log2(half)))
    if 1 << levels != half:
        raise ValueError("geometric Cayley grid needs head_dim/2 to be a power of two")
    root = float(base)
    for _ in range(levels):
        root = math.sqrt(root)
    ratio = 1.0 / root
    active = int(round(fraction * half))
    w = torch.tensor([w0 * ratio ** i if i < active else 0.0 for i in range(half)], dtype=torch.float64)
    c, s = cayley_powers(w.to(torch.float32), seq_len)
    if device is not None:
        c, s = c.to(device), s.to(device)
    return c, s


# --------------------------------------------------------------------------- qk_rms

@_on_tensor_device
def qk_rms_norm(x: torch.Tensor, gain: Optional[torch.Tensor], eps: float = 1e-5, *, block: int = 1024,
                cos: Optional[torch.Tensor] = None, sin: Optional[torch.Tensor] = None,
                out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """RMS-normalise the rows of (B,H,T,D) with a learned gain; with `cos`/`sin` also apply
    the Cayley rotation in the same pass.  `block` is accepted for call compatibility (the
    CUDA kernel picks its own tiling) but validated as the reference does."""
    _require_cuda(x, gain, cos, sin)
    if x.ndim < 2 or x.shape[-1] not in (64, 128) or (gain is not None and gain.shape != (x.shape[-1],)):
        raise ValueError("QK RMS kernel needs D=64 or D=128 and a one-dimensional gain")
    if x.dtype not in _DTYPES or (gain is not None and gain.dtype != torch.float32):
        raise ValueError("QK RMS kernel needs float32/BF16 input and float32 gain")
    if block < 8 or block % 8:
        raise ValueError("QK RMS row count must be divisible by a block aligned to eight rows")
    if eps <= 0:
        raise ValueError("QK RMS epsilon must be positive")
    D = x.shape[-1]
    x4 = x.reshape(1, 1, -1, D) if x.ndim != 4 else x
    if (cos is None) != (sin is None):
        raise ValueError("cos and sin tables come as a pair")
    if cos is not None:
        if x.ndim != 4 or cos.shape[0] < x.shape[-2] or cos.shape[1] != D // 2:
            raise ValueError("rotation tables must have shape (>=T, D/2) and x must be (B,H,T,D)")
        cos, sin = cos.contiguous().float(), sin.contiguous().float()
    y = torch.empty(x4.shape, dtype=x.dtype, device=x.device) if out is None else out.view(x4.shape)
    a = L.QkRmsArgs(x=x4.data_ptr(), y=y.data_ptr(), gain=_ptr(gain), cos=_ptr(cos), sin=_ptr(sin),
                    eps=float(eps), B=x4.shape[0], H=x4.shape[1], T=x4.shape[2], D=D, dtype=_DTYPES[x.dtype],
                    x_stride=_strides3(x4), y_stride=_strides3(y))
    L.check(L.load().alg_qk_rms_fwd(a, _stream()))
    return y.view(x.shape)


@_on_tensor_device
def qk_rms_norm_backward(x: torch.Tensor, gain: Optional[torch.Tensor], dy: torch.Tensor, eps: float = 1e-5):
    """`(dx, dgain)` of `qk_rms_norm(x, gain, eps)` (no rotation) for the output gradient `dy`: what
    the reference's custom VJP returns (src/algebraic/kernels/qk_norm.py:29-56) — the autodiff input
    gradient of `rms_norm` and the gain gradient reduced over row blocks.  `dgain` is None without a
    gain.  Same shapes, dtypes and layouts as the forward; `dx` comes back in the layout of `x`."""
    _require_cuda(x, gain, dy)
    if x.ndim < 2 or x.shape[-1] not in (64, 128) or (gain is not None and gain.shape != (x.shape[-1],)):
        raise ValueError("QK RMS kernel needs D=64 or D=128 and a one-dimensional gain")
    if x.dtype not in _DTYPES or dy.dtype != x.dtype or (gain is not None and gain.dtype != torch.float32):
        raise ValueError("QK RMS kernel needs float32/BF16 input and float32 gain")
    if dy.shape != x.shape:
        raise ValueError("dy must have the shape of x")
    if eps <= 0:
        raise ValueError("QK RMS epsilon must be positive")
    D = x.shape[-1]
    x4 = x.reshape(1, 1, -1, D) if x.ndim != 4 else x
    dy4 = dy.reshape(1, 1, -1, D) if dy.ndim != 4 else dy
    dx = torch.empty_strided(x4.shape, x4.stride(), dtype=x.dtype, device=x.device)
    dgain = torch.empty(D, dtype=torch.float32, device=x.device) if gain is not None else None
    if x4.numel() == 0:
        return dx.view(x.shape), (dgain.zero_() if dgain is not None else None)
    lib = L.load()
    ws = _workspace(x.device, lib.alg_qk_rms_bwd_workspace_bytes(D), "qk_rms_bwd")
    a = L.QkRmsBwdArgs(x=x4.data_ptr(), dy=dy4.data_ptr(), gain=_ptr(gain), dx=dx.data_ptr(), dgain=_ptr(dgain),
                       eps=float(eps), B=x4.shape[0], H=x4.shape[1], T=x4.shape[2], D=D, dtype=_DTYPES[x.dtype],
                       x_stride=_strides3(x4), dy_stride=_strides3(dy4), dx_stride=_strides3(dx),
                       workspace=ws.data_ptr(), workspace_bytes=ws.numel())
    L.check(lib.alg_qk_rms_bwd(a, _stream()))
    return (dx if x.ndim == 4 else dx.view(x.shape)), dgain


@_on_tensor_device
def rms_norm(x: torch.Tensor, gain: Optional[torch.Tensor], eps: float = 1e-5, out=None) -> torch.Tensor:
    """RMS normalisation over the last axis of a contiguous bf16 tensor (the model's `_norm`,
    src/algebraic/model.py:141-143): fp32 math, one rounding to bf16."""
    _require_cuda(x, gain)
    if x.dtype != torch.bfloat16 or not x.is_contiguous():
        raise ValueError("rms_norm needs a contiguous bfloat16 tensor")
    d = x.shape[-1]
    y = torch.empty_like(x) if out is None else out
    g = None if gain is None else gain.contiguous().float()
    L.check(L.load().alg_rms_norm_fwd(x.data_ptr(), _ptr(g), y.data_ptr(), x.numel() // d, d, float(eps), _stream()))
    return y


@_on_tensor_device
def alu_glu(gate: torch.Tensor, up: torch.Tensor, beta: float = 0.5, out=None) -> torch.Tensor:
    """gate * alu(up, beta), the ALU-GLU gating of the feed-forward block
    (src/algebraic/model.py:184-193, src/algebraic/algebraic.py:86-105)."""
    _require_cuda(gate, up)
    if gate.dtype != torch.bfloat16 or up.dtype != torch.bfloat16 or gate.shape != up.shape or gate.ndim != 2:
        raise ValueError("alu_glu needs two (rows, f) bfloat16 tensors of one shape")
    if gate.stride(1) != 1 or up.stride(1) != 1 or gate.stride(0) != up.stride(0):
        raise ValueError("alu_glu needs unit inner stride and one row stride for gate and up")
    rows, f = gate.shape
    y = torch.empty((rows, f), dtype=torch.bfloat16, device=gate.device) if out is None else out
    L.check(L.load().alg_alu_glu_fwd(gate.data_ptr(), up.data_ptr(), y.data_ptr(), rows, f, gate.stride(0), y.stride(0),
                                     float(beta), _stream()))
    return y


@_on_tensor_device
def qkv_projection(x: torch.Tensor, w: torch.Tensor, n_heads: int, seq_len: int, cos: torch.Tensor,
                   sin: torch.Tensor, q_gain: Optional[torch.Tensor] = None, k_gain: Optional[torch.Tensor] = None,
                   eps: float = 1e-5, attn_c: float = 8.0, guard_words: Optional[torch.Tensor] = None,
                   out: Optional[torch.Tensor] = None, row_ss: Optional[torch.Tensor] = None,
                   guard_is_zero: bool = False) -> torch.Tensor:
    """The q, k, v projections of a block with the QK-norm, the Cayley rotation and the range
    guard's maxima fused into the GEMM (src/algebraic/model.py:165-174).

    x: (M, d) bf16 rows in (batch, position) order, position = row % seq_len.  w: (3*H*D, d) bf16,
    one row per output feature (q heads, k heads, v heads).  cos, sin: (>= seq_len, D/2) bf16.
    Returns (M, 3*H*D) bf16: q and k normalised and rotated, v as projected.  `guard_words`
    (4 int32, device) receives the maxima for `flash_attention(..., guard_words=...)`; it is zeroed
    here first unless `guard_is_zero` says the caller has done that on this stream already.
    `row_ss` (slots, M) float32: x is the un-normalised residual stream and the block's RMS norm is
    applied here as a row scale (the norm's gain folded into `w` by the caller); see `resid_projection`."""
    _require_cuda(x, w, cos, sin, q_gain, k_gain, guard_words, row_ss)
    _check_row_ss(row_ss, x.shape[0])
    if x.dtype != torch.bfloat16 or w.dtype != torch.bfloat16 or x.ndim != 2 or w.ndim != 2 or x.stride(1) != 1:
        raise ValueError("qkv_projection needs bf16 (M, d) activations and (3*H*D, d) weights")
    M, d = x.shape
    if w.shape[1] != d or w.shape[0] % (3 * n_heads) or not w.is_contiguous():
        raise ValueError("weights must be contiguous (3*H*D, d)")
    D = w.shape[0] // (3 * n_heads)
    if cos.dtype != torch.bfloat16 or sin.dtype != torch.bfloat16 or cos.shape != sin.shape or cos.shape[1] != D // 2 \
            or cos.shape[0] < seq_len or not cos.is_contiguous() or not sin.is_contiguous():
        raise ValueError("rotation tables must be contiguous bf16 (>= seq_len, D/2)")
    for t in (q_gain, k_gain):
        if t is not None and (t.dtype != torch.float32 or t.shape != (D,)):
            raise ValueError("q_gain / k_gain must be float32 of shape (D,)")
    if guard_words is not None and (guard_words.dtype != torch.int32 or guard_words.numel() < 4):
        raise ValueError("guard_words must hold 4 int32")
    y = torch.empty((M, w.shape[0]), dtype=torch.bfloat16, device=x.device) if out is None else out
    if not y.is_contiguous() or y.shape != (M, w.shape[0]):
        raise ValueError("out must be contiguous (M, 3*H*D)")
    a = L.QkvProjArgs(x=x.data_ptr(), w=w.data_ptr(), qkv=y.data_ptr(), q_gain=_ptr(q_gain), k_gain=_ptr(k_gain),
                      cos=cos.data_ptr(), sin=sin.data_ptr(), eps=float(eps), M=M, d=d, H=n_heads, D=D, T=int(seq_len),
                      ld_x=x.stride(0), attn_c=float(attn_c), guard=_ptr(guard_words), status=None,
                      row_ss=_ptr(row_ss), ss_slots=0 if row_ss is None else row_ss.shape[0], row_eps=float(eps),
                      guard_is_zero=int(bool(guard_is_zero)))
    L.check(L.load().alg_qkv_proj_fwd(a, _stream()))
    return y


def interleave_gate_up(w_gate: torch.Tensor, w_up: torch.Tensor) -> torch.Tensor:
    """(f, d) gate and up weights (one row per output feature) -> the (2f, d) row order
    `glu_projection` expects: blocks of 128 gate rows and the matching 128 up rows in turn."""
    f, d = w_gate.shape
    if w_up.shape != (f, d) or f % 128:
        raise ValueError("gate and up weights must both be (f, d) with f a multiple of 128")
    return torch.stack([w_gate.reshape(f // 128, 128, d), w_up.reshape(f // 128, 128, d)], dim=1).reshape(2 * f, d).contiguous()


@_on_tensor_device
def glu_projection(x: torch.Tensor, w: torch.Tensor, beta: float = 0.5, out: Optional[torch.Tensor] = None,
                   row_ss: Optional[torch.Tensor] = None, eps: float = 1e-5) -> torch.Tensor:
    """gate * alu(up, beta) with gate = x @ w_g and up = x @ w_u computed by the same kernel
    (src/algebraic/model.py:184-193); `w` comes from `interleave_gate_up`.  x: (M, d) bf16.
    `row_ss`, `eps`: as in `qkv_projection` (the norm in front of gate and up applied as a row scale)."""
    _require_cuda(x, w, row_ss)
    _check_row_ss(row_ss, x.shape[0])
    if x.dtype != torch.bfloat16 or w.dtype != torch.bfloat16 or x.ndim != 2 or w.ndim != 2 or x.stride(1) != 1:
        raise ValueError("glu_projection needs bf16 (M, d) activations and (2f, d) weights")
    M, d = x.shape
    if w.shape[1] != d or w.shape[0] % 256 or not w.is_contiguous():
        raise ValueError("weights must be contiguous (2f, d) with f a multiple of 128")
    f = w.shape[0] // 2
    y = torch.empty((M, f), dtype=torch.bfloat16, device=x.device) if out is None else out
    a = L.GluProjArgs(x=x.data_ptr(), w=w.data_ptr(), out=y.data_ptr(), M=M, d=d, f=f, ld_x=x.stride(0),
                      ld_out=y.stride(0), beta=float(beta), status=None, row_ss=_ptr(row_ss),
                      ss_slots=0 if row_ss is None else row_ss.shape[0], row_eps=float(eps))
    L.check(L.load().alg_glu_proj_fwd(a, _stream()))
    return y


def _check_row_ss(row_ss, M):
    if row_ss is not None and (row_ss.dtype != torch.float32 or row_ss.ndim != 2 or row_ss.shape[1] != M
                               or not row_ss.is_contiguous()):
        raise ValueError("row_ss must be contiguous float32 (slots, M)")


@_on_tensor_device
def resid_projection(x: torch.Tensor, w: torch.Tensor, resid: torch.Tensor, out: Optional[torch.Tensor] = None,
                     want_row_ss: bool = True):
    """`resid + x @ w.T` as one GEMM with the add in its epilogue (the block's `x + a @ w_o` and
    `x + (gate * act) @ w_d`, src/algebraic/model.py:183, 193), plus — `want_row_ss` — the per-row
    partial sums of squares of the result, (slots, M) float32, which let the NEXT projection apply the
    RMS norm that follows as a row scale (`qkv_projection(row_ss=...)`, `glu_projection(row_ss=...)`).
    x: (M, K) bf16; w: (N, K) bf16, one row per output feature; resid: (M, N) bf16; `out` may be `resid`.
    Returns `(out, row_ss or None)`."""
    _require_cuda(x, w, resid, out)
    if any(t.dtype != torch.bfloat16 or t.ndim != 2 or t.stride(1) != 1 for t in (x, w, resid)):
        raise ValueError("resid_projection needs bf16 matrices with contiguous rows")
    M, K = x.shape
    N = w.shape[0]
    if w.shape[1] != K or not w.is_contiguous() or resid.shape != (M, N) or K % 64 or N % 64:
        raise ValueError("shapes: x (M, K), w (N, K) contiguous, resid (M, N); K and N multiples of 64")
    y = torch.empty((M, N), dtype=torch.bfloat16, device=x.device) if out is None else out
    if y.shape != (M, N) or y.dtype != torch.bfloat16 or y.stride(1) != 1:
        raise ValueError("out must be bf16 (M, N) with contiguous rows")
    lib = L.load()
    ss = None
    if want_row_ss and M > 0:
        ss = torch.empty((lib.alg_resid_proj_ss_slots(M, N), M), dtype=torch.float32, device=x.device)
    a = L.ResidProjArgs(x=x.data_ptr(), w=w.data_ptr(), resid=resid.data_ptr(), out=y.data_ptr(), ss_out=_ptr(ss),
                        M=M, K=K, N=N, ld_x=x.stride(0), ld_resid=resid.stride(0), ld_out=y.stride(0), status=None)
    L.check(lib.alg_resid_proj_fwd(a, _stream()))
    return y, ss


@_on_tensor_device
def row_sumsq(x: torch.Tensor) -> torch.Tensor:
    """(1, M) float32 sums of squares of the rows of a bf16 (M, d) matrix: the `row_ss` of a projection
    whose input did not come out of `resid_projection` (the first block of a model)."""
    _require_cuda(x)
    if x.dtype != torch.bfloat16 or x.ndim != 2 or x.stride(1) != 1:
        raise ValueError("row_sumsq needs a bf16 matrix with contiguous rows")
    ss = torch.empty((1, x.shape[0]), dtype=torch.float32, device=x.device)
    L.check(L.load().alg_row_sumsq(x.data_ptr(), x.shape[0], x.shape[1], x.stride(0), ss.data_ptr(), _stream()))
    return ss


# ------------------------------------------------------------------------ attention

def flash_clamp(seq_len: int, n: int) -> float:
    """Upper score clamp of the unguarded unshifted link (src/algebraic/kernels/flash.py:744-748)."""
    t = _root(1e37 / (seq_len + 1), n)
    return 0.5 * (t - 1.0 / t)


@_on_tensor_device
def flash_attention(q, k, v, sink_logit=None, *, kind: str = "softmax", n: int = 16, c: float = 16.0,
                    block: int = 512, block_q: Optional[int] = None, block_k: Optional[int] = None,
                    shift: Optional[bool] = None, fast_rho: Optional[bool] = None,
                    inv_stat: Optional[bool] = None, compact_stat: bool = True, poly_rho: bool = False,
                    range_guard: bool = False, resident_bwd: Optional[bool] = None,
                    diagonal_bwd: Optional[bool] = None, diagonal_fwd: Optional[bool] = None,
                    head_resident: Optional[bool] = None,
                    q_gain=None, k_gain=None, cos=None, sin=None, eps: float = 1e-5,
                    causal: bool = True, return_stat: bool = False, impl: str = "auto", out=None,
                    bounded_scores: bool = False, guard_words: Optional[torch.Tensor] = None):
    """Causal asinh-power attention on (B,H,T,D); `sink_logit` broadcastable to (H,).

    Same keywords as the reference entry point.  TPU tiling/residency knobs (`block*`,
    `resident_bwd`, `diagonal_*`, `head_resident`, `compact_stat`, `fast_rho`) are validated
    where the reference validates them and otherwise have no effect on a GPU.  Extras:
    `q_gain/k_gain/cos/sin/eps` run the QK-norm + Cayley rotation of the layer in front of
    the attention inside the same call; `return_stat=True` also returns the per-row
    statistic and which kind it is; `impl` forces a kernel family ("auto", "mma",
    "tcgen05"); `guard_words` hands a guarded call the maxima `qkv_projection` took for these
    very q, k, v, so that it skips its own pass over them.  `kind="softmax"` (the reference's
    control arm) is not built."""
    _require_cuda(q, k, v)
    if kind == "softmax":
        raise NotImplementedError("only the algebraic (kind='asinh') arm is built for B200")
    if kind != "asinh":
        raise ValueError(f"unknown attention kernel: {kind}")
    if q.ndim != 4 or k.ndim != 4 or v.ndim != 4:
        raise ValueError("q, k, v must be (B, H, T, D)")
    B, H, T, D = q.shape
    Tk = k.shape[2]
    bq = min(block_q or block, T)
    bk = min(block_k or block, T)
    if T % bq or T % bk:
        raise ValueError(f"sequence length {T} must be divisible by blocks ({bq}, {bk})")
    if n < 2 or n & (n - 1):
        raise ValueError("asinh kernel needs n to be a power of two")
    if not math.isfinite(c) or c <= 0:
        raise ValueError("asinh scale c must be positive and finite")
    clamp = flash_clamp(T, n)
    if shift is None:
        shift = clamp < 20.0
    if inv_stat is None:
        inv_stat = not shift
    if inv_stat and shift:
        raise ValueError("inverse-denominator statistic requires shift=False")
    if poly_rho:
        raise ValueError("bounded radical approximation is not built; use the exact radical")
    if head_resident is True and not (T == 2048 and D == 64 and q.dtype == torch.bfloat16):
        raise ValueError("whole-head residency needs resident bfloat16 T=2048,D=64, "
                         "512-square public tiles, and compact statistics")
    if q.dtype not in _DTYPES or k.dtype != q.dtype or v.dtype != q.dtype:
        raise ValueError("q, k, v must share dtype float32 or bfloat16")
    if k.shape != (B, H, Tk, D) or v.shape != (B, H, Tk, D):
        raise ValueError("k and v must be (B, H, Tk, D) matching q")
    if range_guard and n <= 32:
        variant, score_clamp = L.ALG_VARIANT_GUARD, 0.0
    elif shift:
        variant, score_clamp = L.ALG_VARIANT_SHIFT, 0.0
    else:
        # `bounded_scores` is the reference's internal flag of the guard's in-range branch
        # (flash.py:850): the caller vouches for the score range, so no upper clamp is applied.
        variant, score_clamp = L.ALG_VARIANT_NOSHIFT, (0.0 if bounded_scores else clamp)

    sink = None
    if sink_logit is not None:
        s = torch.as_tensor(sink_logit, dtype=torch.float32, device=q.device).reshape(-1)
        sink = s.expand(H).contiguous() if s.numel() == 1 else s.contiguous()
        if sink.numel() != H:
            raise ValueError("sink_logit must broadcast to (H,)")
    for t in (q_gain, k_gain):
        if t is not None and (t.dtype != torch.float32 or t.shape != (D,)):
            raise ValueError("q_gain / k_gain must be float32 of shape (D,)")
    if cos is not None:
        cos, sin = cos.contiguous().float(), sin.contiguous().float()
    o = torch.empty((B, H, T, D), dtype=q.dtype, device=q.device) if out is None else out
    stat = torch.empty((B, H, T), dtype=torch.float32, device=q.device) if return_stat else None
    stat_kind = torch.zeros(1, dtype=torch.int32, device=q.device) if return_stat else None
    if q.numel() == 0:
        return (o, stat, stat_kind) if return_stat else o
    a = L.AttnArgs(q=q.data_ptr(), k=k.data_ptr(), v=v.data_ptr(), o=o.data_ptr(), stat=_ptr(stat),
                   stat_kind=_ptr(stat_kind), sink=_ptr(sink), q_gain=_ptr(q_gain), k_gain=_ptr(k_gain),
                   cos=_ptr(cos), sin=_ptr(sin), eps=float(eps), B=B, H=H, Tq=T, Tk=Tk, D=D, n=int(n),
                   c=float(c), causal=int(bool(causal)), variant=variant, dtype=_DTYPES[q.dtype],
                   impl=L.IMPL[impl], score_clamp=float(score_clamp), q_stride=_strides3(q),
                   k_stride=_strides3(k), v_stride=_strides3(v), o_stride=_strides3(o),
                   guard_words=_ptr(guard_words))
    lib = L.load()
    ws = _workspace(q.device, lib.alg_attn_workspace_bytes(a), "attn")
    a.workspace, a.workspace_bytes = ws.data_ptr(), ws.numel()
    L.check(lib.alg_attn_fwd(a, _stream()))
    if return_stat:
        return o, stat, stat_kind
    return o


@_on_tensor_device
def flash_attention_backward(q, k, v, o, d_o, stat, stat_kind, sink_logit=None, *, n: int = 16, c: float = 8.0,
                             causal: bool = True, impl: str = "auto"):
    """Gradients of `flash_attention(kind="asinh", return_stat=True)`: `(dq, dk, dv, dsink)` from the
    forward's inputs, its output `o`, the incoming gradient `d_o` and the saved `(stat, stat_kind)`
    (the custom VJP of the reference, src/algebraic/kernels/flash.py:333-727).  bf16 tensors,
    (B,H,T,D) with D contiguous; `dsink` is None without a sink.  `impl`: "auto" runs the tcgen05
    kernels when the call is causal self-attention over a multiple of 128 positions and the mma.sync
    kernels otherwise; "mma" always runs the latter."""
    if impl not in ("auto", "mma"):
        raise ValueError('impl must be "auto" or "mma"')
    _require_cuda(q, k, v, o, d_o, stat, stat_kind)
    if q.ndim != 4 or k.ndim != 4 or v.shape != k.shape or o.shape != q.shape or d_o.shape != q.shape:
        raise ValueError("q, o, d_o must be (B, H, Tq, D) and k, v (B, H, Tk, D)")
    if any(t.dtype != torch.bfloat16 for t in (q, k, v, o, d_o)):
        raise ValueError("the backward kernels take bfloat16 tensors")
    B, H, T, D = q.shape
    Tk = k.shape[2]
    if stat.shape != (B, H, T) or stat.dtype != torch.float32 or not stat.is_contiguous():
        raise ValueError("stat must be the contiguous float32 (B, H, Tq) statistic of the forward")
    if n < 2 or n & (n - 1):
        raise ValueError("asinh kernel needs n to be a power of two")
    if d_o.stride() != o.stride():
        d_o = torch.empty_strided(o.shape, o.stride(), dtype=o.dtype, device=o.device).copy_(d_o)
    sink = None
    if sink_logit is not None:
        s = torch.as_tensor(sink_logit, dtype=torch.float32, device=q.device).reshape(-1)
        sink = s.expand(H).contiguous() if s.numel() == 1 else s.contiguous()
    dq, dk, dv = (torch.empty_strided(t.shape, t.stride(), dtype=t.dtype, device=t.device) for t in (q, k, v))
    dsink = torch.empty(H, dtype=torch.float32, device=q.device) if sink is not None else None
    if q.numel() == 0:
        return dq, dk, dv, dsink
    a = L.AttnBwdArgs(q=q.data_ptr(), k=k.data_ptr(), v=v.data_ptr(), o=o.data_ptr(), d_o=d_o.data_ptr(),
                      stat=stat.data_ptr(), stat_kind=stat_kind.data_ptr(), sink=_ptr(sink), dq=dq.data_ptr(),
                      dk=dk.data_ptr(), dv=dv.data_ptr(), dsink=_ptr(dsink), B=B, H=H, Tq=T, Tk=Tk, D=D, n=int(n),
                      c=float(c), causal=int(bool(causal)), q_stride=_strides3(q), k_stride=_strides3(k),
                      v_stride=_strides3(v), o_stride=_strides3(o), status=None, impl=int(impl == "mma"))
    lib = L.load()
    ws = _workspace(q.device, lib.alg_attn_bwd_workspace_bytes(a), "attn_bwd")
    a.workspace, a.workspace_bytes = ws.data_ptr(), ws.numel()
    L.check(lib.alg_attn_bwd(a, _stream()))
    return dq, dk, dv, dsink


def _attention_unshifted_unclamped(q, k, v, sink_logit=None, *, n=16, c=8.0, impl="auto", out=None):
    """The attention kernel the range guard selects when it holds, launched directly with no
    guard pre-pass (benchmarks use it to time that kernel alone)."""
    return flash_attention(q, k, v, sink_logit, kind="asinh", n=n, c=c, shift=False, bounded_scores=True,
                           impl=impl, out=out)


@_on_tensor_device
def decode_attention(q, k, v, sink_logit=None, *, n: int = 16, c: float = 8.0, out=None):
    """One query per (batch, head) against a (B,H,Tk,D) bf16 KV cache, every key visible.
    The reference has no decode kernel; semantics follow its dense weights with an all-true
    mask (src/algebraic/algebraic.py:186-204)."""
    _require_cuda(q, k, v)
    B, H, Tq, D = q.shape
    if Tq != 1:
        raise ValueError("decode_attention takes exactly one query row per head")
    if q.dtype != torch.bfloat16 or k.dtype != torch.bfloat16 or v.dtype != torch.bfloat16:
        raise ValueError("decode_attention needs bfloat16 q, k, v")
    if n < 2 or n & (n - 1):
        raise ValueError("asinh kernel needs n to be a power of two")
    Tk = k.shape[2]
    sink = None
    if sink_logit is not None:
        s = torch.as_tensor(sink_logit, dtype=torch.float32, device=q.device).reshape(-1)
        sink = s.expand(H).contiguous() if s.numel() == 1 else s.contiguous()
    q = q.contiguous()
    o = torch.empty((B, H, 1, D), dtype=q.dtype, device=q.device) if out is None else out
    a = L.DecodeArgs(q=q.data_ptr(), k=k.data_ptr(), v=v.data_ptr(), o=o.data_ptr(), sink=_ptr(sink),
                     B=B, H=H, Tk=Tk, D=D, n=int(n), c=float(c), k_stride=_strides3(k), v_stride=_strides3(v))
    lib = L.load()
    ws = _workspace(q.device, lib.alg_decode_workspace_bytes(a), "decode")
    a.workspace, a.workspace_bytes = ws.data_ptr(), ws.numel()
    L.check(lib.alg_attn_decode(a, _stream()))
    return o


# ----------------------------------------------------------------------------- head

@_on_tensor_device
def cast_embedding(embed: torch.Tensor) -> torch.Tensor:
    """fp32 (V,d) -> bf16 with the library's cast kernel (the reference casts per call)."""
    _require_cuda(embed)
    if embed.dtype == torch.bfloat16:
        return embed.contiguous()
    e32 = embed.contiguous().float()
    out = torch.empty(e32.shape, dtype=torch.bfloat16, device=embed.device)
    L.check(L.load().alg_cast_f32_to_bf16(e32.data_ptr(), out.data_ptr(), e32.numel(), _stream()))
    return out


@_on_tensor_device
def head_statistic(h, e_bf16, targets, *, n: int = 16, c: float = 16.0, vocab_offset: int = 0,
                   vocab_total: Optional[int] = None, impl: str = "auto", out=None, kind: str = "alg_ce"):
    """Per-row (l, zt) of one vocabulary shard as a (2, N) fp32 tensor: row 0 the partial
    normaliser, row 1 the target logit (0 where the target is not in the shard).  With
    `kind="ce"` row 0 is the logsumexp of the shard's logits instead (n and c are unused)."""
    N, d = h.shape
    V_local = e_bf16.shape[0]
    stats = torch.empty((2, N), dtype=torch.float32, device=h.device) if out is None else out
    if V_local == 0:                                   # a rank that owns no vocabulary tile
        stats.zero_()
        if kind == "ce":
            stats[0].fill_(-1e30)                      # the logsumexp of nothing
        return stats
    a = L.HeadArgs(h=h.data_ptr(), e=e_bf16.data_ptr(), targets=targets.data_ptr(), l_out=stats[0].data_ptr(),
                   zt_out=stats[1].data_ptr(), N=N, d=d, V_local=V_local, vocab_offset=int(vocab_offset),
                   V_total=int(vocab_total or V_local), n=int(n), c=float(c), impl=L.IMPL[impl],
                   kind=L.HEAD_CE if kind == "ce" else L.HEAD_ALG_CE)
    lib = L.load()
    ws = _workspace(h.device, lib.alg_head_workspace_bytes(a), "head")
    a.workspace, a.workspace_bytes = ws.data_ptr(), ws.numel()
    L.check(lib.alg_head_fwd(a, _stream()))
    return stats


@_on_tensor_device
def head_statistic_no_alloc(h, e_bf16, targets, out, *, n: int, c: float, vocab_offset: int = 0,
                            vocab_total: Optional[int] = None, impl: str = "auto"):
    """`head_statistic` through `alg_head_fwd_static`: the same (2, N) statistic, written
    into the caller's `out`, with the kernel's scratch taken from the array built into the
    library instead of a workspace allocated here.  Meant for callers that may not allocate
    device memory at call time; problems whose partials exceed the built-in array raise
    ValueError.  Calls on one device share that array, so do not let two of them overlap."""
    N, d = h.shape
    a = L.HeadArgs(h=h.data_ptr(), e=e_bf16.data_ptr(), targets=targets.data_ptr(), l_out=out[0].data_ptr(),
                   zt_out=out[1].data_ptr(), N=N, d=d, V_local=e_bf16.shape[0], vocab_offset=int(vocab_offset),
                   V_total=int(vocab_total or e_bf16.shape[0]), n=int(n), c=float(c), impl=L.IMPL[impl])
    L.check(L.load().alg_head_fwd_static(a, _stream()))
    return out


@_on_tensor_device
def head_finalize(stats, *, n: int = 16, c: float = 16.0, vocab_total: int = 0, want_nll: bool = False,
                  kind: str = "alg_ce"):
    """(objective, p_target[, nll]) from the (all-reduced) (2, N) statistic.  `kind="ce"`: row 0
    is the logsumexp; returns (mean nll, nll) like the reference's "ce" arm (`want_nll=True`
    appends the nll once more, so that both kinds unpack alike)."""
    N = stats.shape[1]
    dev = stats.device
    pt = torch.empty(N, dtype=torch.float32, device=dev)
    nll = torch.empty(N, dtype=torch.float32, device=dev) if (want_nll or kind == "ce") else None
    obj = torch.empty((), dtype=torch.float32, device=dev)
    lib = L.load()
    ws = _workspace(dev, lib.alg_head_finalize_workspace_bytes(N), "head_fin")
    if kind == "ce":
        L.check(lib.alg_head_finalize_ce(stats[0].data_ptr(), stats[1].data_ptr(), N, pt.data_ptr(), nll.data_ptr(),
                                         obj.data_ptr(), ws.data_ptr(), ws.numel(), _stream()))
        return (obj, nll, nll) if want_nll else (obj, nll)
    L.check(lib.alg_head_finalize(stats[0].data_ptr(), stats[1].data_ptr(), N, int(n), float(c), int(vocab_total),
                                  pt.data_ptr(), _ptr(nll), obj.data_ptr(), ws.data_ptr(), ws.numel(), _stream()))
    return (obj, pt, nll) if want_nll else (obj, pt)


@_on_tensor_device
def fused_head(h, embed, targets, *, kind: str = "ce", n: int = 16, c: float = 16.0, block_n: int = 128,
               block_v: int = 512, vocab_offset: int = 0, vocab_total: Optional[int] = None,
               group=None, want_nll: bool = False, impl: str = "auto", exchange=None):
    """Fused tied-embedding projection and Alg-CE likelihood: returns `(objective,
    p_target)` like the reference (`want_nll=True` appends the per-token NLL).

    `embed` is this rank's vocabulary shard: rows [vocab_offset, vocab_offset + V_local) of a
    `vocab_total`-row embedding (defaults: the whole thing).  With a `torch.distributed`
    `group`, the per-row partials (normaliser, target logit) of all shards are summed with one
    all-reduce before the telemetry is formed.  `kind="ce"` (the reference's softmax control arm)
    returns `(mean nll, nll)`; its shards combine by logsumexp (a MAX and a SUM all-reduce), and
    it is not offered through `exchange`."""
    _require_cuda(h, embed, targets)
    if kind not in ("ce", "alg_ce"):
        raise ValueError(kind)
    if kind == "alg_ce" and n & (n - 1):
        raise ValueError("n must be a power of two")
    if kind == "ce" and exchange is not None:
        raise NotImplementedError("the one-kernel exchange is built for kind='alg_ce' only")
    if h.ndim != 2 or embed.ndim != 2 or h.shape[1] != embed.shape[1]:
        raise ValueError("h must be (N, d) and embed (V, d)")
    N = h.shape[0]
    bn = min(block_n, N)
    if N % bn:
        raise ValueError(f"token count {N} must be divisible by block {bn}")
    if h.dtype != torch.bfloat16:
        raise ValueError("fused_head needs bfloat16 hidden states")
    h = h.contiguous()
    e = cast_embedding(embed)
    t = targets.reshape(N).to(torch.int32).contiguous()
    V_total = int(vocab_total or embed.shape[0])
    if exchange is not None:
        # fused path: GEMM + statistic kernel, then one kernel that reduces the splits, exchanges
        # the per-row partials with the peers over NVLink and forms the telemetry
        return _fused_head_exchange(h, e, t, exchange, n=n, c=c, vocab_offset=vocab_offset, vocab_total=V_total,
                                    want_nll=want_nll, impl=impl)
    stats = head_statistic(h, e, t, n=n, c=c, vocab_offset=vocab_offset, vocab_total=V_total, impl=impl, kind=kind)
    if group is not None:
        import torch.distributed as dist
        if kind == "ce":
            combine_ce_statistics(stats, group)
        else:
            dist.all_reduce(stats, op=dist.ReduceOp.SUM, group=group)
    return head_finalize(stats, n=n, c=c, vocab_total=V_total, want_nll=want_nll, kind=kind)


def combine_ce_statistics(stats, group):
    """In place: the (2, N) statistics of the "ce" kind over the vocabulary shards of `group` —
    row 0 (per-shard logsumexp) by logsumexp (one MAX all-reduce for the common shift, then the
    shifted exponentials ride the SUM all-reduce of row 1), row 1 (target logit) by a sum."""
    import torch.distributed as dist
    top = stats[0].clone()
    dist.all_reduce(top, op=dist.ReduceOp.MAX, group=group)
    stats[0] = torch.exp(stats[0] - top)
    dist.all_reduce(stats, op=dist.ReduceOp.SUM, group=group)
    stats[0] = top + torch.log(stats[0])
    return stats


@_on_tensor_device
def fused_head_backward(h, e_bf16, targets, stats, *, n: int = 8, c: float = 2.0, vocab_offset: int = 0,
                        vocab_total: Optional[int] = None, upstream: float = 1.0, kind: str = "alg_ce"):
    """What the reference's custom VJP of the Alg-CE head returns for the hidden states and this
    shard's embedding rows, `(dh, de)` (src/algebraic/kernels/fused_head.py:120-156, 194-216,
    236-243): the gradient of the mean negative log-likelihood, `dz = upstream/N * (n/c) * (p - y) /
    sqrt(1 + x^2)` with the clamp straight-through — not the derivative of the primal value
    `mean(1 - pt)`, which the reference uses as a monotone stand-in only (algebraic.py:232-262).
    `stats` is the forward's `(2, N)` statistic (`head_statistic`, summed over all shards).  The
    logit gradient is rebuilt tile by tile from `stats` by one kernel and written as bf16; the two
    products `dz . E` and `dz^T . h` are library GEMMs, as in the reference.  With several shards
    the caller sums `dh` over them.  `kind="ce"`: `stats` is the "ce" statistic (row 0 the
    logsumexp over all shards) and `dz = upstream/N * (softmax - y)` (fused_head.py:134-135)."""
    if kind not in ("ce", "alg_ce"):
        raise ValueError(kind)
    _require_cuda(h, e_bf16, targets, stats)
    if h.dtype != torch.bfloat16 or e_bf16.dtype != torch.bfloat16 or h.ndim != 2 or e_bf16.ndim != 2:
        raise ValueError("fused_head_backward needs bf16 (N, d) hidden states and (V, d) embedding rows")
    N, d = h.shape
    V_local = e_bf16.shape[0]
    if e_bf16.shape[1] != d or V_local % 8 or not h.is_contiguous() or not e_bf16.is_contiguous():
        raise ValueError("contiguous operands, embedding (V_local, d) with V_local a multiple of 8")
    if stats.shape != (2, N) or stats.dtype != torch.float32 or not stats.is_contiguous():
        raise ValueError("stats must be the contiguous float32 (2, N) statistic of the forward")
    V_total = V_local if vocab_total is None else int(vocab_total)
    t = targets.to(torch.int32).contiguous()
    dz = torch.empty((N, V_local), dtype=torch.bfloat16, device=h.device)
    a = L.HeadBwdArgs(h=h.data_ptr(), e=e_bf16.data_ptr(), targets=t.data_ptr(), l=stats[0].data_ptr(),
                      zt=stats[1].data_ptr(), dz=dz.data_ptr(), N=N, d=d, V_local=V_local, vocab_offset=int(vocab_offset),
                      V_total=V_total, n=int(n), c=float(c), upstream=float(upstream), status=None,
                      kind=L.HEAD_CE if kind == "ce" else L.HEAD_ALG_CE)
    L.check(L.load().alg_head_bwd_dz(a, _stream()))
    return torch.mm(dz, e_bf16), torch.mm(dz.t(), h)


@_on_tensor_device
def _fused_head_exchange(h, e_bf16, targets, exchange, *, n, c, vocab_offset, vocab_total, want_nll, impl):
    """`alg_head_fwd_exchange`: see include/alg_b200.h.  `exchange` is a dist.HeadExchange."""
    N, d = h.shape
    dev = h.device
    pt = torch.empty(N, dtype=torch.float32, device=dev)
    nll = torch.empty(N, dtype=torch.float32, device=dev) if want_nll else None
    obj = torch.empty((), dtype=torch.float32, device=dev)
    a = L.HeadArgs(h=h.data_ptr(), e=e_bf16.data_ptr(), targets=targets.data_ptr(), l_out=None, zt_out=None, N=N, d=d,
                   V_local=e_bf16.shape[0], vocab_offset=int(vocab_offset), V_total=int(vocab_total), n=int(n),
                   c=float(c), impl=L.IMPL[impl])
    lib = L.load()
    ws = _workspace(dev, lib.alg_head_workspace_bytes(a), "head")
    a.workspace, a.workspace_bytes = ws.data_ptr(), ws.numel()
    x = L.HeadExchangeArgs(rank=exchange.rank, world=exchange.world, N_capacity=exchange.n_capacity,
                           pt=pt.data_ptr(), nll=_ptr(nll), obj=obj.data_ptr(), wait_budget_ns=0)
    for r, p in enumerate(exchange.ptrs):
        x.peer_region[r] = p
    L.check(lib.alg_head_fwd_exchange(a, x, _stream()))
    return (obj, pt, nll) if want_nll else (obj, pt)
