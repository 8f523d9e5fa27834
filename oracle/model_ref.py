"""CPU restatement of the reference model's forward pass (algebraic preset).

TEST INFRASTRUCTURE, like the rest of oracle/.  Follows src/algebraic/model.py:141-231
of the reference for `norm="rms", ffn="alu_glu", pos="cayley_geo", qk_norm=True,
attn="asinh", sink="learned", head="alg_ce"` with `attn_impl="dense"`, `head_impl="dense"`:
activations in bf16, every matmul with bf16 operands and fp32 accumulation rounded to bf16
(what `h @ w.astype(bf16)` gives in XLA), norms and ALU in fp32 rounded once.
"""

import torch

from . import algebraic_ref as R


def _mm(a, w):
    """The activations' dtype x the weight cast to it -> fp32 accumulate -> that dtype
    (model.py:167-169, 183, 186-187, 193)."""
    return (a.float() @ w.to(a.dtype).float()).to(a.dtype)


def forward_hidden(params, tokens, cfg, dtype=torch.bfloat16):
    """model.forward_hidden (model.py:196-208) + model._block (model.py:162-193).
    `dtype` is the reference's `cfg.dtype` (bfloat16 in every preset)."""
    B, T = tokens.shape
    d, H = cfg.d_model, cfg.n_heads
    D = d // H
    cos, sin = R.cayley_table_geometric(D, T, cfg.rope_base)
    x = params["embed"][tokens].to(dtype)
    x = R.rms_norm(x, params["embed_gain"], cfg.eps)
    for l in range(cfg.n_layers):
        h = R.rms_norm(x, params["ln1"][l], cfg.eps)
        q = _mm(h, params["w_q"][l]).reshape(B, T, H, D).transpose(1, 2)
        k = _mm(h, params["w_k"][l]).reshape(B, T, H, D).transpose(1, 2)
        v = _mm(h, params["w_v"][l]).reshape(B, T, H, D).transpose(1, 2)
        q = R.apply_rotary(R.rms_norm(q, params["q_gain"][l], cfg.eps), cos, sin)
        k = R.apply_rotary(R.rms_norm(k, params["k_gain"][l], cfg.eps), cos, sin)
        a = R.asinh_attention(q, k, v, n=cfg.attn_n, c=cfg.attn_c, sink_logit=params["sink"][l])
        a = a.transpose(1, 2).reshape(B, T, d)
        x = (x.float() + _mm(a, params["w_o"][l]).float()).to(dtype)
        h2 = R.rms_norm(x, params["ln2"][l], cfg.eps)
        gate = _mm(h2, params["w_g"][l])
        up = _mm(h2, params["w_u"][l])
        act = R.alu(up, cfg.alu_beta)
        x = (x.float() + _mm((gate.float() * act.float()).to(dtype), params["w_d"][l]).float()).to(dtype)
    return R.rms_norm(x, params["final_gain"], cfg.eps)


def head_loss(params, hidden, targets, cfg):
    """model.head_loss, dense branch (model.py:225-230)."""
    h = hidden.reshape(-1, cfg.d_model)
    return R.head_loss_dense(h, params["embed"], targets.reshape(-1), cfg.head_n, cfg.head_c)
