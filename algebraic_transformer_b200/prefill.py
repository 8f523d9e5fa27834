"""Prefill (forward-only) of the algebraic Transformer, hosted in PyTorch around the kernels.

Mirrors the reference's model forward for the `algebraic` preset
(src/algebraic/model.py:162-231, src/algebraic/config.py:8-42): embedding gather ->
RMS(embed_gain) -> L x [RMS -> QKV GEMMs -> QK-norm + Cayley rotation + asinh attention
(one library call) -> out-projection + residual -> RMS -> gate/up GEMMs -> gate * ALU(up)
-> down GEMM + residual] -> final RMS -> fused Alg-CE head over all positions.
GEMMs are plain library GEMMs (cuBLAS through torch); every other stage is a kernel of
this package.  Projections are consumed in place as strided (B,H,T,D) views and the
attention output is written straight into (B,T,H*D) layout, so no transposes are copied.

Multi-GPU (one process per GPU): the batch is split over ranks (weights replicated, no
communication in the body), the final hidden states are all-gathered, and the head runs
vocabulary-sharded with one all-reduce of the per-row statistic.
"""

from dataclasses import dataclass
from typing import Optional

import torch

from . import ops
from .dist import vocab_shard

SIZES = {   # src/algebraic/config.py:8-14
    "proxy": dict(d_model=384, n_layers=8, n_heads=6, d_ff=1024),
    "125m": dict(d_model=768, n_layers=12, n_heads=12, d_ff=2048),
    "350m": dict(d_model=1024, n_layers=24, n_heads=16, d_ff=2688),
    "1b": dict(d_model=1536, n_layers=32, n_heads=24, d_ff=4224),
}


@dataclass(frozen=True)
class PrefillConfig:
    """The `algebraic` preset's constants (src/algebraic/config.py:32-35, model.py:24-63)."""
    vocab_size: int = 32768
    d_model: int = 384
    n_layers: int = 8
    n_heads: int = 6
    d_ff: int = 1024
    eps: float = 1e-5
    alu_beta: float = 0.5
    rope_base: float = 10000.0
    attn_n: int = 16
    attn_c: float = 8.0
    head_n: int = 8
    head_c: float = 2.0
    init_std: float = 0.02

    @property
    def head_dim(self) -> int:
        return self.d_model // self.n_heads

    @staticmethod
    def preset(size: str, **overrides) -> "PrefillConfig":
        return PrefillConfig(**{**SIZES[size], **overrides})

    def flops_per_token(self, seq_len: int) -> float:
        """Forward FLOPs per token: GEMMs + causal attention + head (2 N d V)."""
        d, f, L, V = self.d_model, self.d_ff, self.n_layers, self.vocab_size
        return 2.0 * (L * (4 * d * d + 3 * d * f) + V * d) + L * 4.0 * seq_len * d / 2.0


def init_params(cfg: PrefillConfig, seed: int = 0, device="cpu"):
    """Random-init parameters with the reference's shapes and scales
    (src/algebraic/model.py:84-117): N(0, init_std) matrices, unit gains, zero sinks.
    Kept in fp32 on `device`; `cast_params` makes the bf16 working copy."""
    g = torch.Generator().manual_seed(seed)
    L, d, f, V, H, D = cfg.n_layers, cfg.d_model, cfg.d_ff, cfg.vocab_size, cfg.n_heads, cfg.head_dim

    def normal(*shape):
        return (torch.randn(shape, generator=g) * cfg.init_std).to(device)

    return {
        "embed": normal(V, d), "embed_gain": torch.ones(d, device=device), "final_gain": torch.ones(d, device=device),
        "w_q": normal(L, d, d), "w_k": normal(L, d, d), "w_v": normal(L, d, d), "w_o": normal(L, d, d),
        "w_g": normal(L, d, f), "w_u": normal(L, d, f), "w_d": normal(L, f, d),
        "ln1": torch.ones(L, d, device=device), "ln2": torch.ones(L, d, device=device),
        "q_gain": torch.ones(L, D, device=device), "k_gain": torch.ones(L, D, device=device),
        "sink": torch.zeros(L, H, device=device),
    }


def cast_params(params, device, fused_proj: bool = False, fused_norm: bool = False):
    """bf16 copies of the matrices (the reference casts at use, model.py:167), fp32 gains.
    `fused_proj` lays the q|k|v and gate|up weights out for `ops.qkv_projection` /
    `ops.glu_projection` instead of for a plain GEMM.  `fused_norm` (with `fused_proj`) also lays
    w_o and w_d out for `ops.resid_projection` and multiplies the block norms' gains into the
    input columns of the q|k|v and gate|up weights (in fp32, before the one rounding to bf16): the
    norms themselves then run as row scales inside those projections."""
    out = {}
    src = {k: v.to(device) for k, v in params.items()}
    if fused_norm:
        src = dict(src)
        for name in ("w_q", "w_k", "w_v"):
            src[name] = src[name].float() * src["ln1"].float()[:, :, None]      # (L, d_in, d_out) * gain over d_in
        for name in ("w_g", "w_u"):
            src[name] = src[name].float() * src["ln2"].float()[:, :, None]
    for k, v in src.items():
        out[k] = v.bfloat16().contiguous() if k.startswith("w_") or k == "embed" else v.float().contiguous()
    # q, k, v projections share their input: one GEMM with the concatenated weight
    if fused_proj:
        # one row per output feature (K-major), gate/up rows interleaved in blocks of 128
        out["w_qkv_t"] = torch.cat([out["w_q"], out["w_k"], out["w_v"]], dim=2).transpose(1, 2).contiguous()
        out["w_gu_t"] = torch.stack([ops.interleave_gate_up(g.t(), u.t()) for g, u in zip(out["w_g"], out["w_u"])])
        if fused_norm:
            # one row per output feature; the library-GEMM path reads the same storage through `.t()`
            out["w_o_t"] = out["w_o"].transpose(1, 2).contiguous()
            out["w_d_t"] = out["w_d"].transpose(1, 2).contiguous()
            del out["w_o"], out["w_d"]
    else:
        out["w_qkv"] = torch.cat([out["w_q"], out["w_k"], out["w_v"]], dim=2).contiguous()
        out["w_gu"] = torch.cat([out["w_g"], out["w_u"]], dim=2).contiguous()
    for k in ("w_q", "w_k", "w_v", "w_g", "w_u"):        # only the fused copies are used
        del out[k]
    return out


class Prefill:
    """Forward pass of one rank: `hidden(tokens)` and `loss(tokens, targets)`."""

    def __init__(self, cfg: PrefillConfig, params, device, seq_len: int, impl: str = "auto", exchange=None,
                 fused_proj: Optional[bool] = None, fused_norm: Optional[bool] = None):
        self.cfg, self.device, self.impl = cfg, torch.device(device), impl
        self.exchange = exchange        # dist.HeadExchange: fuse the head's cross-GPU sum into its last kernel
        # The projections with their consumers fused in (ops.qkv_projection / glu_projection)
        # cover the production shapes; anything else takes library GEMMs + separate kernels.
        can_fuse = cfg.head_dim in (64, 128) and cfg.d_model % 64 == 0 and cfg.d_ff % 128 == 0 and impl != "mma"
        if fused_proj and not can_fuse:
            raise ValueError("fused projections need head_dim 64/128, d_model % 64 == 0, d_ff % 128 == 0")
        self.fused_proj = can_fuse if fused_proj is None else bool(fused_proj)
        # `fused_norm`: the block norms as row scales inside the projections and the residual adds inside
        # the out- and down-projection (five GEMM launches per block, no stand-alone norm).  Measured
        # against stand-alone norms + library GEMMs with the residual in their epilogue: 3-4 % faster
        # per step up to 4096 tokens per call (a rank's share of a batch split over several GPUs), 2-5 %
        # slower at 16384, where the library's two-CTA 256 x 256 tiles win.  None = choose per call by the
        # token count; the weights are laid out once for both (norm gains folded into the q|k|v and
        # gate|up weights either way: above 4096 tokens the library takes the residual GEMMs, a pass that
        # only reads x leaves the row statistic, and the norms still ride in the two wide projections).
        if fused_norm and not self.fused_proj:
            raise ValueError("fused_norm needs the fused projections")
        self.fused_norm = fused_norm if (fused_norm is None or not self.fused_proj) else bool(fused_norm)
        if not self.fused_proj:
            self.fused_norm = False
        self.norm_in_weights = self.fused_proj and self.fused_norm is not False
        self.p = cast_params(params, self.device, self.fused_proj, self.norm_in_weights)
        self.cos, self.sin = ops.cayley_table_geometric(cfg.head_dim, seq_len, cfg.rope_base, device=self.device)
        self.cos_lp, self.sin_lp = self.cos.bfloat16().contiguous(), self.sin.bfloat16().contiguous()
        # one record of the range guard's maxima per layer: all zeroed by one fill at the start of a step,
        # so that no memset sits between two kernels of the step
        self.guard_words = torch.zeros((cfg.n_layers, 4), dtype=torch.int32, device=self.device)

    def hidden(self, tokens: torch.Tensor) -> torch.Tensor:
        """Final normalised hidden states (B, T, d) in bf16 (model.forward_hidden, model.py:196-208)."""
        cfg, p = self.cfg, self.p
        B, T = tokens.shape
        d, H, D, f = cfg.d_model, cfg.n_heads, cfg.head_dim, cfg.d_ff
        x = ops.rms_norm(p["embed"][tokens].contiguous(), p["embed_gain"], cfg.eps).view(B * T, d)
        attn_out = torch.empty((B, T, H, D), dtype=torch.bfloat16, device=self.device)
        use_fused_norm = (B * T <= 4096) if self.fused_norm is None else self.fused_norm
        if self.fused_proj:
            self.guard_words.zero_()
        if use_fused_norm:
            # x stays the un-normalised residual stream; `ss` carries the row statistic of the next norm
            ss = ops.row_sumsq(x)
            for layer in range(cfg.n_layers):
                qkv = ops.qkv_projection(x, p["w_qkv_t"][layer], H, T, self.cos_lp, self.sin_lp, p["q_gain"][layer],
                                         p["k_gain"][layer], cfg.eps, cfg.attn_c, self.guard_words[layer],
                                         row_ss=ss, guard_is_zero=True).view(B, T, 3, H, D)
                q, k, v = (qkv[:, :, i].transpose(1, 2) for i in range(3))      # (B,H,T,D) views
                ops.flash_attention(q, k, v, p["sink"][layer], kind="asinh", n=cfg.attn_n, c=cfg.attn_c, block=T,
                                    range_guard=True, impl=self.impl, guard_words=self.guard_words[layer],
                                    out=attn_out.transpose(1, 2))
                x, ss = ops.resid_projection(attn_out.view(B * T, d), p["w_o_t"][layer], x, out=x)
                ff = ops.glu_projection(x, p["w_gu_t"][layer], cfg.alu_beta, row_ss=ss, eps=cfg.eps)
                x, ss = ops.resid_projection(ff, p["w_d_t"][layer], x, out=x)
            return ops.rms_norm(x, p["final_gain"], cfg.eps).view(B, T, d)
        # with the gains folded into the weights the stand-alone norms run without one
        ln1 = (lambda l: None) if self.norm_in_weights else (lambda l: p["ln1"][l])
        ln2 = (lambda l: None) if self.norm_in_weights else (lambda l: p["ln2"][l])
        w_o = (lambda l: p["w_o_t"][l].t()) if self.norm_in_weights else (lambda l: p["w_o"][l])
        w_d = (lambda l: p["w_d_t"][l].t()) if self.norm_in_weights else (lambda l: p["w_d"][l])
        for layer in range(cfg.n_layers):
            if self.norm_in_weights:
                # library residual GEMMs, but the block norms still ride in the two wide projections: a pass
                # that only reads x for its row statistic replaces one that reads x and writes norm(x)
                qkv = ops.qkv_projection(x, p["w_qkv_t"][layer], H, T, self.cos_lp, self.sin_lp, p["q_gain"][layer],
                                         p["k_gain"][layer], cfg.eps, cfg.attn_c, self.guard_words[layer],
                                         row_ss=ops.row_sumsq(x), guard_is_zero=True).view(B, T, 3, H, D)
                q, k, v = (qkv[:, :, i].transpose(1, 2) for i in range(3))      # (B,H,T,D) views
                ops.flash_attention(q, k, v, p["sink"][layer], kind="asinh", n=cfg.attn_n, c=cfg.attn_c, block=T,
                                    range_guard=True, impl=self.impl, guard_words=self.guard_words[layer],
                                    out=attn_out.transpose(1, 2))
                x = torch.addmm(x, attn_out.view(B * T, d), w_o(layer))
                ff = ops.glu_projection(x, p["w_gu_t"][layer], cfg.alu_beta, row_ss=ops.row_sumsq(x), eps=cfg.eps)
                x = torch.addmm(x, ff, w_d(layer))
                continue
            h = ops.rms_norm(x, ln1(layer), cfg.eps)
            if self.fused_proj:
                qkv = ops.qkv_projection(h, p["w_qkv_t"][layer], H, T, self.cos_lp, self.sin_lp, p["q_gain"][layer],
                                         p["k_gain"][layer], cfg.eps, cfg.attn_c, self.guard_words[layer],
                                         guard_is_zero=True).view(B, T, 3, H, D)
                q, k, v = (qkv[:, :, i].transpose(1, 2) for i in range(3))      # (B,H,T,D) views
                ops.flash_attention(q, k, v, p["sink"][layer], kind="asinh", n=cfg.attn_n, c=cfg.attn_c, block=T,
                                    range_guard=True, impl=self.impl, guard_words=self.guard_words[layer],
                                    out=attn_out.transpose(1, 2))
                x = torch.addmm(x, attn_out.view(B * T, d), w_o(layer))
                h2 = ops.rms_norm(x, ln2(layer), cfg.eps)
                x = torch.addmm(x, ops.glu_projection(h2, p["w_gu_t"][layer], cfg.alu_beta), w_d(layer))
                continue
            qkv = torch.mm(h, p["w_qkv"][layer]).view(B, T, 3, H, D)
            q, k, v = (qkv[:, :, i].transpose(1, 2) for i in range(3))          # (B,H,T,D) views
            ops.flash_attention(q, k, v, p["sink"][layer], kind="asinh", n=cfg.attn_n, c=cfg.attn_c, block=T,
                                range_guard=True, q_gain=p["q_gain"][layer], k_gain=p["k_gain"][layer],
                                cos=self.cos, sin=self.sin, eps=cfg.eps, impl=self.impl,
                                out=attn_out.transpose(1, 2))
            x = torch.addmm(x, attn_out.view(B * T, d), p["w_o"][layer])
            h2 = ops.rms_norm(x, p["ln2"][layer], cfg.eps)
            gu = torch.mm(h2, p["w_gu"][layer])                                  # gate | up in one GEMM
            x = torch.addmm(x, ops.alu_glu(gu[:, :f], gu[:, f:], cfg.alu_beta), p["w_d"][layer])
        return ops.rms_norm(x, p["final_gain"], cfg.eps).view(B, T, d)

    def graphed_loss(self, tokens: torch.Tensor, targets: torch.Tensor, group=None, rank: int = 0, world: int = 1):
        """Capture one `loss` step in a CUDA graph and return `(replay, outputs, how)`.
        `replay()` re-runs the captured launches on the inputs' storage (copy new token ids
        into `tokens` / `targets` in place before calling it); `outputs` are the tensors the
        step writes.  The whole step is ~170 short launches, so at small per-GPU batches the
        host cannot enqueue them as fast as the GPU retires them; a graph removes that limit.
        If the collectives cannot be captured, only the body is captured and the head with
        its two collectives runs eagerly after each replay (`how` says which)."""
        side = torch.cuda.Stream(device=self.device)
        side.wait_stream(torch.cuda.current_stream(self.device))
        with torch.cuda.stream(side):                     # warm-up: attributes, workspaces, NCCL
            for _ in range(2):
                self.loss(tokens, targets, group=group, rank=rank, world=world)
        torch.cuda.current_stream(self.device).wait_stream(side)
        torch.cuda.synchronize(self.device)
        try:
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph):
                outputs = self.loss(tokens, targets, group=group, rank=rank, world=world)
            return graph.replay, outputs, "whole step captured"
        except Exception:                                  # fall back: body only
            torch.cuda.synchronize(self.device)
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph):
                hid = self.hidden(tokens)
            box = {}

            def replay():
                graph.replay()
                box["out"] = self._head(hid.reshape(-1, self.cfg.d_model), targets, group, rank, world, False)
                return box["out"]
            return replay, box, "body captured, head and collectives eager"

    def loss(self, tokens: torch.Tensor, targets: torch.Tensor, group=None, rank: int = 0, world: int = 1,
             want_nll: bool = False):
        """(objective, p_target[, nll]) over all positions (model.head_loss, model.py:211-231).
        With `group`, `tokens` is this rank's batch slice: the hidden states of all ranks are
        all-gathered and the head runs over this rank's vocabulary shard."""
        hid = self.hidden(tokens).reshape(-1, self.cfg.d_model)
        return self._head(hid, targets, group, rank, world, want_nll)

    def _head(self, hid, targets, group, rank, world, want_nll):
        cfg = self.cfg
        tgt = targets.reshape(-1).to(torch.int32)
        if group is None or world == 1:
            return ops.fused_head(hid, self.p["embed"], tgt, kind="alg_ce", n=cfg.head_n, c=cfg.head_c,
                                  block_n=hid.shape[0], want_nll=want_nll, impl=self.impl)
        import torch.distributed as dist
        full = torch.empty((world * hid.shape[0], cfg.d_model), dtype=hid.dtype, device=hid.device)
        dist.all_gather_into_tensor(full, hid.contiguous(), group=group)
        all_t = torch.empty(world * tgt.shape[0], dtype=torch.int32, device=hid.device)
        dist.all_gather_into_tensor(all_t, tgt.contiguous(), group=group)
        lo, cnt = vocab_shard(cfg.vocab_size, rank, world)
        return ops.fused_head(full, self.p["embed"][lo:lo + cnt], all_t, kind="alg_ce", n=cfg.head_n, c=cfg.head_c,
                              block_n=full.shape[0], vocab_offset=lo, vocab_total=cfg.vocab_size,
                              group=None if self.exchange is not None else group, exchange=self.exchange,
                              want_nll=want_nll, impl=self.impl)
