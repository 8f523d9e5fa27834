"""Prefill body (PyTorch-hosted GEMMs + this package's kernels) against the CPU restatement
of the reference model, and the elementwise kernels against the oracle."""

import os

import numpy as np
import pytest
import torch

import algebraic_transformer_b200 as A
from algebraic_transformer_b200 import prefill as P
from oracle import algebraic_ref as R
from oracle import model_ref as M

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def rel_l2(a, b):
    a, b = a.detach().double().cpu(), b.detach().double().cpu()
    return float((a - b).norm() / b.norm().clamp_min(1e-30))


@pytest.mark.parametrize("d", [384, 768, 1024, 1536])
def test_rms_norm_rows(d):
    g = torch.Generator().manual_seed(d)
    x = (torch.randn((300, d), generator=g) * 2).bfloat16()
    x[7] = 0
    gain = 0.5 + torch.rand(d, generator=g)
    want = R.rms_norm(x, gain, 1e-5)
    got = A.ops.rms_norm(x.to(DEV), gain.to(DEV), 1e-5).cpu()
    np.testing.assert_allclose(got.float(), want.float(), rtol=0.01, atol=0.01)
    assert rel_l2(got, want) < 3e-3 and torch.all(got[7] == 0)


def test_alu_glu():
    g = torch.Generator().manual_seed(3)
    gate = torch.randn((257, 2048), generator=g).bfloat16()
    up = (torch.randn((257, 2048), generator=g) * 8).bfloat16()
    want = (gate.float() * R.alu(up, 0.5).float()).bfloat16()
    got = A.ops.alu_glu(gate.to(DEV), up.to(DEV), 0.5).cpu()
    assert rel_l2(got, want) < 3e-3
    # the negative tail of the ALU survives (cancellation-free branch)
    tail = torch.full((8,), -200.0).bfloat16()
    out = A.ops.alu_glu(torch.ones(1, 8).bfloat16().to(DEV), tail.to(DEV)[None], 0.5).cpu().float()[0]
    np.testing.assert_allclose(out, R.alu(tail, 0.5).float(), rtol=0.02)
    assert (out < 0).all()
    # both halves of one fused gate|up GEMM output, read in place through the row stride
    gu = torch.cat([gate, up], dim=1).to(DEV)
    got2 = A.ops.alu_glu(gu[:, :2048], gu[:, 2048:], 0.5).cpu()
    assert torch.equal(got2, got)


def _mm(a, w):                                           # bf16 x bf16 -> fp32 accumulate -> bf16
    return (a.float() @ w.float()).bfloat16()


@pytest.mark.parametrize("H,D,B,T", [(6, 64, 2, 256), (2, 128, 1, 200), (12, 64, 1, 128)])
def test_qkv_projection_fused_epilogue(H, D, B, T):
    """Projection + QK-norm + rotation + guard maxima in one kernel (model.py:165-174) against the
    same steps of the oracle; d = H*D gives a ragged last weight tile for H=6 and a row count
    that is not a multiple of the tile for T=200."""
    d = H * D
    g = torch.Generator().manual_seed(7 + H)
    x = torch.randn((B * T, d), generator=g).bfloat16()
    wq, wk, wv = ((torch.randn((d, d), generator=g) * 0.05).bfloat16() for _ in range(3))
    qg, kg = (0.75 + 0.5 * torch.rand(D, generator=g) for _ in range(2))
    cos, sin = R.cayley_table_geometric(D, T)
    heads = lambda y: y.reshape(B, T, H, D).transpose(1, 2)
    want_q = R.apply_rotary(R.rms_norm(heads(_mm(x, wq)), qg, 1e-5), cos, sin)
    want_k = R.apply_rotary(R.rms_norm(heads(_mm(x, wk)), kg, 1e-5), cos, sin)
    want_v = heads(_mm(x, wv))
    w = torch.cat([wq, wk, wv], dim=1).t().contiguous()                  # (3d, d): one row per feature
    words = torch.zeros(4, dtype=torch.int32, device=DEV)
    got = A.qkv_projection(x.to(DEV), w.to(DEV), H, T, cos.bfloat16().to(DEV), sin.bfloat16().to(DEV),
                           qg.to(DEV), kg.to(DEV), 1e-5, 8.0, words).view(B, T, 3, H, D)
    q, k, v = (got[:, :, i].transpose(1, 2).cpu() for i in range(3))
    assert rel_l2(q, want_q) < 6e-3 and rel_l2(k, want_k) < 6e-3 and rel_l2(v, want_v) < 4e-3
    # the guard maxima of exactly what was written
    stats = words.cpu().view(torch.float32)
    qs = (q.float() * (1.0 / (D ** 0.5 * 8.0))).bfloat16().float()
    np.testing.assert_allclose(float(stats[0]), float((qs * qs).sum(-1).max()), rtol=1e-4)
    np.testing.assert_allclose(float(stats[1]), float((k.float() ** 2).sum(-1).max()), rtol=1e-4)
    assert float(stats[2]) == float(v.float().abs().max())
    # and the attention that consumes them agrees with the one that takes its own maxima
    qd, kd, vd = (got[:, :, i].transpose(1, 2) for i in range(3))
    if T % 8 == 0:
        a1 = A.flash_attention(qd, kd, vd, None, kind="asinh", n=16, c=8.0, block=T, range_guard=True, guard_words=words)
        a2 = A.flash_attention(qd, kd, vd, None, kind="asinh", n=16, c=8.0, block=T, range_guard=True)
        assert torch.equal(a1, a2)


@pytest.mark.parametrize("M,d,f", [(300, 384, 256), (1024, 256, 1024)])
def test_glu_projection_fused_epilogue(M, d, f):
    """gate/up projections + gate * alu(up) in one kernel (model.py:184-193)."""
    g = torch.Generator().manual_seed(f)
    x = torch.randn((M, d), generator=g).bfloat16()
    wg = (torch.randn((d, f), generator=g) * 0.05).bfloat16()
    wu = (torch.randn((d, f), generator=g) * 0.4).bfloat16()
    want = (_mm(x, wg).float() * R.alu(_mm(x, wu), 0.5).float()).bfloat16()
    w = A.interleave_gate_up(wg.t().contiguous(), wu.t().contiguous())
    got = A.glu_projection(x.to(DEV), w.to(DEV), 0.5).cpu()
    assert got.shape == (M, f)
    assert rel_l2(got, want) < 6e-3


@pytest.mark.parametrize("M,K,N", [(300, 256, 768), (4096, 2048, 768), (1000, 2688, 1024), (130, 64, 64)])
def test_residual_projection_and_row_statistic(M, K, N):
    """`resid + x @ w.T` with the reference's rounding (product to bf16, then a bf16 add; model.py:183,
    193) on both tile widths, in place, and the row sums of squares it leaves for the next norm."""
    g = torch.Generator().manual_seed(M + N)
    x = torch.randn((M, K), generator=g).bfloat16()
    w = (torch.randn((N, K), generator=g) * 0.05).bfloat16()
    resid = torch.randn((M, N), generator=g).bfloat16()
    prod = (x.float() @ w.float().t()).bfloat16()
    want = (resid.float() + prod.float()).bfloat16()
    rd = resid.to(DEV)
    got, ss = A.resid_projection(x.to(DEV), w.to(DEV), rd, out=rd)           # in place
    assert got.data_ptr() == rd.data_ptr() and ss.shape[1] == M
    assert rel_l2(got, want) < 4e-3                                              # fp32 summation order only
    want_ss = got.float().pow(2).sum(-1).cpu()
    np.testing.assert_allclose(ss.sum(0).cpu(), want_ss, rtol=1e-5)
    np.testing.assert_allclose(A.row_sumsq(got)[0].cpu(), want_ss, rtol=1e-5)


def test_projections_apply_the_block_norm_as_a_row_scale():
    """qkv_projection / glu_projection fed the un-normalised stream plus its row statistic, with the
    norm's gain folded into the weights, against normalising first (model.py:164-169, 184-187)."""
    M, d, H, D, T, f = 512, 256, 2, 64, 256, 512
    g = torch.Generator().manual_seed(77)
    x = (torch.randn((M, d), generator=g) * 3).bfloat16()
    gain = 0.5 + torch.rand(d, generator=g)
    wq = torch.randn((3 * H * D, d), generator=g) * 0.05
    wg, wu = torch.randn((f, d), generator=g) * 0.05, torch.randn((f, d), generator=g) * 0.2
    cos, sin = A.cayley_table_geometric(D, T, device=DEV)
    cos, sin = cos.bfloat16().contiguous(), sin.bfloat16().contiguous()
    ones = torch.ones(D, device=DEV)
    h = A.ops.rms_norm(x.to(DEV), gain.to(DEV), 1e-5)
    ss = A.row_sumsq(x.to(DEV))
    want = A.qkv_projection(h, wq.bfloat16().to(DEV), H, T, cos, sin, ones, ones, 1e-5, 8.0)
    got = A.qkv_projection(x.to(DEV), (wq * gain).bfloat16().to(DEV), H, T, cos, sin, ones, ones, 1e-5, 8.0, row_ss=ss)
    assert rel_l2(got, want) < 8e-3                                              # rounding points differ, nothing else
    w_plain = A.interleave_gate_up(wg.bfloat16(), wu.bfloat16()).to(DEV)
    w_fold = A.interleave_gate_up((wg * gain).bfloat16(), (wu * gain).bfloat16()).to(DEV)
    want = A.glu_projection(h, w_plain, 0.5)
    got = A.glu_projection(x.to(DEV), w_fold, 0.5, row_ss=ss, eps=1e-5)
    assert rel_l2(got, want) < 1.5e-2


@pytest.mark.parametrize("fused", [True, "auto", "proj_only", False])
@pytest.mark.parametrize("head_dim,T", [(64, 256), (128, 512)])
def test_tiny_prefill_matches_reference_model(head_dim, T, fused):
    cfg = P.PrefillConfig(vocab_size=1000, d_model=2 * head_dim, n_layers=2, n_heads=2, d_ff=256)
    params = P.init_params(cfg, seed=0)
    g = torch.Generator().manual_seed(1)
    for k in ("q_gain", "k_gain", "ln1", "ln2"):         # exercise non-trivial gains and sinks
        params[k] = 0.75 + 0.5 * torch.rand(params[k].shape, generator=g)
    params["sink"] = torch.randn(params["sink"].shape, generator=g) * 0.3
    tokens = torch.randint(0, cfg.vocab_size, (2, T), generator=g)
    want_h = M.forward_hidden(params, tokens, cfg)
    obj_w, pt_w = M.head_loss(params, want_h, tokens, cfg)
    # True: norms and residual adds inside the GEMMs; "auto": chosen per call (these sizes take the fused path);
    # "proj_only": stand-alone norms and library residual GEMMs around the fused projections; False: nothing fused
    fused_norm = {True: True, "auto": None, "proj_only": False, False: False}[fused]
    model = P.Prefill(cfg, params, DEV, seq_len=T, fused_proj=bool(fused), fused_norm=fused_norm)
    assert model.fused_norm is fused_norm
    got_h = model.hidden(tokens.to(DEV))
    assert rel_l2(got_h, want_h) < 2e-2                  # two layers of bf16 activations
    obj, pt, nll = model.loss(tokens.to(DEV), tokens.to(DEV), want_nll=True)
    assert rel_l2(nll, R.nll_from_pt(pt_w)) < 1e-2
    np.testing.assert_allclose(float(obj), float(obj_w), rtol=5e-3)


@pytest.mark.parametrize("size,vocab,T", [("125m", 50304, 1024), ("350m", 32000, 2048)])
def test_prefill_at_the_benchmark_shapes(size, vocab, T):
    """Benchmark configurations 3 and 4 at their real widths and depths (125M: 12 layers, d 768,
    12 heads of 64, vocabulary 50304; 350M: 24 layers, d 1024, 16 heads of 64, vocabulary 32000), one
    sequence each so that the CPU model finishes in seconds: per-token NLL within rel-L2 1e-2 of
    oracle/model_ref.py (itself pinned to the reference's model.py)."""
    cfg = P.PrefillConfig.preset(size, vocab_size=vocab)
    params = P.init_params(cfg, seed=0)
    g = torch.Generator().manual_seed(3)
    tokens = torch.randint(0, vocab, (1, T), generator=g)
    torch.set_num_threads(max(1, (os.cpu_count() or 1)))
    want_h = M.forward_hidden(params, tokens, cfg)
    obj_w, pt_w = M.head_loss(params, want_h, tokens, cfg)
    model = P.Prefill(cfg, params, DEV, seq_len=T)
    got_h = model.hidden(tokens.to(DEV))
    obj, pt, nll = model.loss(tokens.to(DEV), tokens.to(DEV), want_nll=True)
    e_h, e_nll = rel_l2(got_h, want_h), rel_l2(nll, R.nll_from_pt(pt_w))
    print(f"{size}: hidden rel-L2 {e_h:.2e}, NLL rel-L2 {e_nll:.2e}")
    assert e_nll < 1e-2, (e_h, e_nll)
    assert e_h < 6e-2, e_h                               # bf16 activations through every layer, summation order differs
    np.testing.assert_allclose(float(obj), float(obj_w), rtol=5e-3)
