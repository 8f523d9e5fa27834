"""CPU restatement of the Algebraic Transformer's forward hot path.

THIS FILE IS TEST INFRASTRUCTURE.  It is the checker the CUDA kernels are
compared against, and the timed CPU baseline of the benchmark; nothing in the
product package imports it and there is no CPU fallback in the product.

It restates, in PyTorch-on-CPU tensor ops (fp32 by default, fp64 on request),
the dense definitions of the reference (paths within the reference project):

  rho, int_pow ...................... src/algebraic/algebraic.py:31-51
  rms_norm (QK-norm forward) ........ src/algebraic/algebraic.py:76-83
  alu ............................... src/algebraic/algebraic.py:86-105
  cayley_powers / table ............. src/algebraic/algebraic.py:124-169
  apply_rotary ...................... src/algebraic/algebraic.py:172-179
  asinh_power_weights / attention ... src/algebraic/algebraic.py:186-216
  algebraic_probs / likelihood ...... src/algebraic/algebraic.py:223-245
  likelihood_clamp / lean ........... src/algebraic/algebraic.py:277-301
  flash dispatch (clamp, guard) ..... src/algebraic/kernels/flash.py:732-760, 823-856
  kernel-side rho / root statistic .. src/algebraic/kernels/flash.py:76-113
  fused head statistic + telemetry .. src/algebraic/kernels/fused_head.py:98-117, 219-229, 273
  NLL from target probability ....... src/algebraic/train.py:239

Pinning: `tests/test_oracle_golden.py` checks every function here against
`tests/golden/reference_vectors.npz`, whose values were produced by the
reference's own source files executed over a NumPy stand-in for `jax.numpy`
(JAX itself cannot be installed offline), and against the formula identities of
the reference's `tests/test_components.py` (rho = exp(asinh), weights =
softmax(n asinh(s/c)), Cayley = cos/sin(m 2 atan w), lean = exact).
"""

import math
from typing import Optional, Tuple

import torch

F32 = torch.float32


def _acc(x: torch.Tensor) -> torch.Tensor:
    """At least fp32 (bf16/fp16 -> fp32, fp64 stays).  algebraic.py:25-28."""
    return x if x.dtype in (torch.float32, torch.float64) else x.to(F32)


def rsqrt(x):
    return torch.rsqrt(x)


# --------------------------------------------------------------------------- rho

def rho(x: torch.Tensor) -> torch.Tensor:
    """x + sqrt(1+x^2), cancellation-free for x < 0.  algebraic.py:31-35."""
    rad = 1.0 + x * x
    t = x.abs() + rad * rsqrt(rad)
    return torch.where(x >= 0, t, 1.0 / t)


def rho_fast(x: torch.Tensor) -> torch.Tensor:
    """x + rad*rsqrt(rad): the kernels' summation form.  flash.py:84-88."""
    rad = 1.0 + x * x
    return x + rad * rsqrt(rad)


def int_pow(x, n: int):
    """x**n by binary exponentiation.  algebraic.py:38-51."""
    n = int(n)
    if n < 1:
        raise ValueError("n must be a positive integer")
    result, base = None, x
    while n:
        if n & 1:
            result = base if result is None else result * base
        n >>= 1
        if n:
            base = base * base
    return result


def root_pow2(value: float, n: int) -> float:
    """value**(1/n), n a power of two, by repeated sqrt.  flash.py:106-112."""
    out = float(value)
    while n > 1:
        out = math.sqrt(out)
        n //= 2
    return out


def inv_root(l: torch.Tensor, n: int) -> torch.Tensor:
    """l**(-1/n) via rsqrt then square roots.  flash.py:95-104, fused_head.py:57-63."""
    y = rsqrt(l)
    k = n // 2
    while k > 1:
        y = y * rsqrt(y)
        k //= 2
    return y


def kernel_sink_logit(omega: float, n: int, c: float) -> float:
    """Sink logit b with rho(b/c)^n = omega.  algebraic.py:54-69."""
    if omega <= 0:
        raise ValueError("omega must be positive")
    k = int(round(math.log2(n)))
    if 1 << k != n:
        raise ValueError("n must be a power of two")
    t = root_pow2(omega, n)
    return c * 0.5 * (t - 1.0 / t)


# ------------------------------------------------------------------ norm, ALU

def rms_norm(x: torch.Tensor, gain: Optional[torch.Tensor], eps: float = 1e-5) -> torch.Tensor:
    """y = x * rsqrt(mean(x^2) + eps) * gain, math in >= fp32.  algebraic.py:76-83."""
    xf = _acc(x)
    tau = rsqrt((xf * xf).mean(dim=-1, keepdim=True) + eps)
    y = xf * tau
    if gain is not None:
        y = y * gain.to(y.dtype)
    return y.to(x.dtype)


def alu(x: torch.Tensor, beta: float = 1.0) -> torch.Tensor:
    """x/2 (1 + bx/sqrt(1+b^2x^2)) with the negative tail kept.  algebraic.py:86-105."""
    z = _acc(x)
    bz = beta * z
    r = rsqrt(1.0 + bz * bz)
    u = bz * r
    one_plus_u = torch.where(bz < 0, (r * r) / (1.0 - u), 1.0 + u)
    return (0.5 * z * one_plus_u).to(x.dtype)


# ------------------------------------------------------------- Cayley rotation

def cayley_powers(w: torch.Tensor, seq_len: int) -> Tuple[torch.Tensor, torch.Tensor]:
    """Rows ((1+iw)^2/(1+w^2))^m, m < seq_len, by binary exponentiation with
    renormalised squarings.  algebraic.py:124-149."""
    w = w.to(F32)
    w2 = w * w
    c = (1.0 - w2) / (1.0 + w2)
    s = (2.0 * w) / (1.0 + w2)
    positions = torch.arange(seq_len, dtype=torch.int32)
    out_c = torch.ones((seq_len, w.shape[0]), dtype=F32)
    out_s = torch.zeros((seq_len, w.shape[0]), dtype=F32)
    bit = 0
    while (1 << bit) < seq_len:
        take = ((positions >> bit) & 1).bool()[:, None]
        new_c = out_c * c - out_s * s
        new_s = out_c * s + out_s * c
        out_c = torch.where(take, new_c, out_c)
        out_s = torch.where(take, new_s, out_s)
        c, s = c * c - s * s, 2.0 * c * s
        inv = rsqrt(c * c + s * s)
        c, s = c * inv, s * inv
        bit += 1
    inv = rsqrt(out_c * out_c + out_s * out_s)
    return out_c * inv, out_s * inv


def cayley_table_geometric(head_dim: int, seq_len: int, base: float = 10000.0,
                           w0: float = 0.5, fraction: float = 1.0):
    """Geometric grid w_k = w0 base^(-k/half); tables (T, D/2).  algebraic.py:152-169."""
    half = head_dim // 2
    levels = int(round(math.log2(half)))
    if 1 << levels != half:
        raise ValueError("geometric Cayley grid needs head_dim/2 to be a power of two")
    root = float(base)
    for _ in range(levels):
        root = math.sqrt(root)
    ratio = 1.0 / root
    active = int(round(fraction * half))
    w = [w0 * ratio ** i if i < active else 0.0 for i in range(half)]
    return cayley_powers(torch.tensor(w, dtype=torch.float64).to(F32), seq_len)


def apply_rotary(x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor) -> torch.Tensor:
    """Rotate-half by (T, D/2) tables, in x.dtype.  algebraic.py:172-179."""
    half = x.shape[-1] // 2
    t = x.shape[-2]
    c = cos[:t].to(x.dtype)[None, None]
    s = sin[:t].to(x.dtype)[None, None]
    x1, x2 = x[..., :half], x[..., half:]
    return torch.cat([x1 * c - x2 * s, x1 * s + x2 * c], dim=-1)


# ------------------------------------------------------------------- attention

def asinh_power_weights(scores, mask, n: int, c: float, sink_logit):
    """Normalised rho(s/c)^n weights, max shifted, optional sink.  algebraic.py:186-204."""
    x = scores / c
    neg = torch.full((), -1e30, dtype=x.dtype)
    m = torch.where(mask, x, neg).amax(dim=-1, keepdim=True)
    if sink_logit is not None:
        xb = sink_logit / c
        m = torch.maximum(m, xb.to(m.dtype))
    shift = rho(-m)
    w = torch.where(mask, int_pow(rho(x) * shift, n), torch.zeros((), dtype=x.dtype))
    denom = w.sum(dim=-1, keepdim=True)
    if sink_logit is not None:
        denom = denom + int_pow(rho(xb.to(m.dtype)) * shift, n)
    return w / denom


def _sink4(sink_logit, H, dtype):
    if sink_logit is None:
        return None
    s = torch.as_tensor(sink_logit, dtype=dtype).reshape(-1)
    return s.expand(H).reshape(1, H, 1, 1) if s.numel() in (1, H) else s.reshape(1, H, 1, 1)


def asinh_attention(q, k, v, *, n: int, c: float, sink_logit=None, causal: bool = True,
                    acc_dtype=None, row_block: int = 0):
    """Dense (causal) asinh-power attention on (B,H,Tq,D) x (B,H,Tk,D).
    algebraic.py:207-216.  Scores accumulate in fp32 (`acc_dtype=torch.float64`
    gives the fp64 cross-check); the weights are cast to v.dtype before P.V as in
    the reference; output in q.dtype.  `row_block > 0` evaluates that many query
    rows at a time so that (T,T) never has to fit in memory; results are
    identical because rows are independent.  `causal=False` with Tq != Tk is the
    decode case (all keys visible), which the reference expresses through
    `asinh_power_weights` with an all-true mask."""
    B, H, Tq, D = q.shape
    Tk = k.shape[-2]
    acc = acc_dtype or (torch.float64 if q.dtype == torch.float64 else F32)
    sink = _sink4(sink_logit, H, acc)
    kf, vf = k.to(acc), v.to(acc)
    out = torch.empty((B, H, Tq, D), dtype=q.dtype)
    step = row_block if row_block > 0 else Tq
    for r0 in range(0, Tq, step):
        r1 = min(Tq, r0 + step)
        kmax = min(Tk, r1 + (Tk - Tq)) if causal else Tk
        s = torch.matmul(q[:, :, r0:r1].to(acc), kf[:, :, :kmax].transpose(-1, -2))
        s = s * (1.0 / math.sqrt(D))
        if causal:
            # query i sits at absolute position i + (Tk - Tq): square problems are the
            # reference's tril mask, Tq < Tk is "the last Tq rows of the square problem"
            rows = torch.arange(r0, r1)[:, None] + (Tk - Tq)
            cols = torch.arange(kmax)[None, :]
            mask = (cols <= rows)[None, None]
        else:
            mask = torch.ones((1, 1, r1 - r0, kmax), dtype=torch.bool)
        p = asinh_power_weights(s, mask, n, c, sink)
        p = p.to(v.dtype).to(acc)
        out[:, :, r0:r1] = torch.matmul(p, vf[:, :, :kmax]).to(q.dtype)
    return out


def flash_clamp(seq_len: int, n: int) -> float:
    """Score clamp of the unshifted variant: rho(clamp) = t, (T+1) t^n = 1e37.
    flash.py:744-748."""
    t = root_pow2(1e37 / (seq_len + 1), n)
    return 0.5 * (t - 1.0 / t)


def flash_default_shift(seq_len: int, n: int) -> bool:
    """Default accumulation strategy when `shift=None`.  flash.py:749-750."""
    return flash_clamp(seq_len, n) < 20.0


def range_guard_in_range(q, k, v, sink_logit, *, n: int, c: float) -> bool:
    """The reference's run-time guard choosing the unshifted fast path.
    flash.py:831-849: with q pre-scaled by 1/(sqrt(D) c) and re-rounded to
    q.dtype, in range iff max|q_s|^2 max|k|^2 <= (bound/1.01)^2, |sink/c| <=
    bound/1.01 and max|v| <= vmax."""
    B, H, T, D = q.shape
    clamp = flash_clamp(T, n)
    bound = min(16.0, clamp / 2)
    scale = 1.0 / (math.sqrt(D) * c)
    qs = (q.to(F32) * scale).to(q.dtype).to(F32)
    q2 = (qs ** 2).sum(-1).max()
    k2 = (k.to(F32) ** 2).sum(-1).max()
    ok = bool(q2 * k2 <= (bound / 1.01) ** 2)
    has_sink = sink_logit is not None
    if has_sink:
        ok = ok and bool((torch.as_tensor(sink_logit, dtype=F32) / c).abs().max() <= bound / 1.01)
    vmax = min(1e8, 1e37 / ((T + int(has_sink)) * (2 * bound + 1) ** n))
    return ok and bool(v.to(F32).abs().max() <= vmax)


def attention_row_stat(q, k, *, n: int, c: float, sink_logit=None, shifted: bool):
    """Per-row statistic the forward kernels save for a backward pass
    (flash.py:271-284): unshifted 1/l with l = rho(b')^n + sum_j rho_fast(x_ij)^n;
    shifted rho(-m) l^(-1/n) with the max-shifted l.  With fewer query rows than keys the
    queries are the last rows of the square problem, as in `asinh_attention`."""
    B, H, T, D = q.shape
    Tk = k.shape[-2]
    x = torch.matmul(q.to(F32), k.to(F32).transpose(-1, -2)) * (1.0 / (math.sqrt(D) * c))
    mask = (torch.arange(Tk)[None, :] <= torch.arange(T)[:, None] + (Tk - T))[None, None]
    sink = _sink4(sink_logit, H, F32)
    if not shifted:
        w = torch.where(mask, int_pow(rho_fast(x), n), torch.zeros(()))
        l = w.sum(-1)
        if sink is not None:
            l = l + int_pow(rho(sink / c), n).reshape(1, H, 1)
        return 1.0 / l
    m = torch.where(mask, x, torch.full((), -1e30)).amax(-1, keepdim=True)
    if sink is not None:
        m = torch.maximum(m, sink / c)
    shift = rho(-m)
    w = torch.where(mask, int_pow(rho(x) * shift, n), torch.zeros(()))
    l = w.sum(-1, keepdim=True)
    if sink is not None:
        l = l + int_pow(rho(sink / c) * shift, n)
    return (shift * inv_root(l, n))[..., 0]


# ---------------------------------------------------------------- Alg-CE head

def algebraic_probs(z, n: int, c: float):
    """p_j ~ rho(z_j/c)^n, max shifted.  algebraic.py:223-228."""
    x = z / c
    m = x.amax(dim=-1, keepdim=True)
    w = int_pow(rho(x) * rho(-m), n)
    return w / w.sum(dim=-1, keepdim=True)


def algebraic_likelihood(logits, targets, n: int, c: float):
    """(mean(1 - p_t), p_t) with the exact max-shifted form.  algebraic.py:231-245."""
    p = algebraic_probs(_acc(logits), n, c)
    pt = p.gather(-1, targets.long()[:, None])[:, 0]
    return (1.0 - pt).mean(), pt


def likelihood_clamp(vocab: int, n: int) -> float:
    """0.25 (1e38/V)^(1/n) by repeated sqrt.  algebraic.py:277-283, fused_head.py:273."""
    out = 1e38 / vocab
    k = n
    while k > 1:
        out = math.sqrt(out)
        k //= 2
    return 0.25 * out


def lean_weights(z, n: int, c: float, clamp: float):
    """w = (x + rad*rsqrt(rad))^n, x = min(z/c, clamp).  algebraic.py:286-291."""
    x = torch.clamp(z / c, max=clamp)
    rad = 1.0 + x * x
    return int_pow(x + rad * rsqrt(rad), n)


def algebraic_likelihood_lean(logits, targets, n: int, c: float):
    """Unshifted additive form used by the model's dense head.  algebraic.py:294-301."""
    z = _acc(logits)
    w = lean_weights(z, n, c, likelihood_clamp(z.shape[-1], n))
    wt = w.gather(-1, targets.long()[:, None])[:, 0]
    pt = wt / w.sum(dim=-1)
    return (1.0 - pt).mean(), pt


def algebraic_likelihood_lean_vjp(logits, targets, n: int, c: float, g: float = 1.0):
    """The logit cotangent the reference's custom VJP returns for the Alg-CE head
    (algebraic.py:309-316, same rule in algebraic.py:255-262 and kernels/fused_head.py:120-145,
    236-243): `g (n/c)/N * r * (p - y)` with `r = rsqrt(1 + x^2)` of the CLAMPED x (straight-through
    clamp).  This is the gradient of the mean negative log-likelihood, not of the primal value
    mean(1 - pt) that `algebraic_likelihood_lean` returns, so autograd through that function does
    NOT reproduce it."""
    z = _acc(logits)
    x = torch.clamp(z / c, max=likelihood_clamp(z.shape[-1], n))
    rad = 1.0 + x * x
    r = rsqrt(rad)
    w = int_pow(x + rad * r, n)
    p = w / w.sum(dim=-1, keepdim=True)
    y = torch.zeros_like(p)
    y.scatter_(-1, targets.long()[:, None], 1.0)
    return (g * (n / c) / z.shape[0]) * r * (p - y)


def head_vjp_dense(h, embed, targets, n: int = 8, c: float = 2.0, g: float = 1.0):
    """(dh, dE) of the model's Alg-CE head under the reference's custom VJP: the logit cotangent
    above pushed through z = h . E^T (fused_head.py:194-216: dh = dz . E, dE = dz^T . h)."""
    e = embed.to(h.dtype).to(F32)
    dz = algebraic_likelihood_lean_vjp(head_logits(h, embed), targets, n, c, g)
    return dz @ e, dz.t() @ h.to(F32)


def cross_entropy(logits, targets):
    """The "ce" head: (mean cross-entropy, per-token nll), nll = logsumexp(z) - z_target in fp32.
    src/algebraic/standard.py:41-47; the fused kernel's telemetry is the same quantity
    (kernels/fused_head.py:113-114, 221-223)."""
    z = logits.to(F32) if logits.dtype != torch.float64 else logits
    lse = torch.logsumexp(z, dim=-1)
    zt = z.gather(-1, targets.long()[:, None])[:, 0]
    nll = lse - zt
    return nll.mean(), nll


def head_logits(h, embed):
    """z = h . bf16(E)^T with fp32 accumulation.  model.py:225."""
    e = embed.to(h.dtype)
    return torch.matmul(h.to(F32), e.to(F32).t())


def head_loss_dense(h, embed, targets, n: int = 8, c: float = 2.0):
    """The model's dense Alg-CE head: (objective, p_target).  model.py:211-231."""
    return algebraic_likelihood_lean(head_logits(h, embed), targets, n, c)


def fused_head_stats(h, embed, targets, n: int, c: float, *, row_block: int = 1024,
                     vocab_lo: int = 0, vocab_hi: Optional[int] = None,
                     vocab_total: Optional[int] = None):
    """The fused kernel's per-row outputs (fused_head.py:72-117): the normaliser
    l_i = sum_j rho_fast(min(z_ij/c, clamp))^n over the vocab range
    [vocab_lo, vocab_hi) and the target logit zt_i (zero when the target lies
    outside the range).  The clamp always uses the FULL vocabulary size, as a
    vocab-sharded caller must."""
    N = h.shape[0]
    V = embed.shape[0]
    vocab_hi = V if vocab_hi is None else vocab_hi
    clamp = likelihood_clamp(vocab_total or V, n)
    e = embed[vocab_lo:vocab_hi].to(h.dtype).to(F32)
    l = torch.empty(N, dtype=F32)
    zt = torch.zeros(N, dtype=F32)
    tl = targets.long()
    for r0 in range(0, N, row_block):
        r1 = min(N, r0 + row_block)
        z = torch.matmul(h[r0:r1].to(F32), e.t())
        l[r0:r1] = lean_weights(z, n, c, clamp).sum(-1)
        t = tl[r0:r1]
        own = (t >= vocab_lo) & (t < vocab_hi)
        zloc = z.gather(-1, (t - vocab_lo).clamp(0, e.shape[0] - 1)[:, None])[:, 0]
        zt[r0:r1] = torch.where(own, zloc, torch.zeros(()))
    return l, zt


def fused_head_telemetry(l, zt, n: int, c: float, clamp: float):
    """p_t = (rho(min(zt/c, clamp)) l^(-1/n))^n and mean(1 - p_t).
    fused_head.py:116, 219-229."""
    x = torch.clamp(zt / c, max=clamp)
    pt = int_pow(rho(x) * inv_root(l, n), n)
    return pt, (1.0 - pt).mean()


def nll_from_pt(pt):
    """-log(max(p_t, 1e-30)).  train.py:239."""
    return -torch.log(torch.clamp(pt, min=1e-30))


def fused_head(h, embed, targets, *, n: int = 8, c: float = 2.0, row_block: int = 1024):
    """(objective, p_target) through the fused kernel's statistic.  fused_head.py:260-275."""
    l, zt = fused_head_stats(h, embed, targets, n, c, row_block=row_block)
    pt, obj = fused_head_telemetry(l, zt, n, c, likelihood_clamp(embed.shape[0], n))
    return obj, pt


# -------------------------------------------------------------- fp64 cross-oracles

def attention_fp64_transcendental(q, k, v, *, n: int, c: float, sink_logit=None, causal=True):
    """softmax(n asinh(s/c)) with an optional sink column, in fp64 — the
    independent formula the reference's tests pin the weights to
    (tests/test_components.py:27-40)."""
    B, H, Tq, D = q.shape
    Tk = k.shape[-2]
    s = torch.matmul(q.double(), k.double().transpose(-1, -2)) / math.sqrt(D)
    logits = n * torch.asinh(s / c)
    if causal:
        mask = torch.tril(torch.ones((Tq, Tk), dtype=torch.bool))
        logits = logits.masked_fill(~mask, float("-inf"))
    if sink_logit is not None:
        b = _sink4(sink_logit, H, torch.float64)
        col = (n * torch.asinh(b / c)).expand(B, H, Tq, 1)
        logits = torch.cat([logits, col], dim=-1)
    p = torch.softmax(logits, dim=-1)[..., :Tk]
    return torch.matmul(p, v.double())


def head_logprob_fp64(z, targets, n: int, c: float):
    """log p_t = n asinh(z_t/c) - logsumexp_j n asinh(z_j/c)  (evaluation.py:13-23)."""
    a = n * torch.asinh(z.double() / c)
    return a.gather(-1, targets.long()[:, None])[:, 0] - torch.logsumexp(a, dim=-1)
