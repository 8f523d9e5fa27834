"""Prefill body (PyTorch-hosted GEMMs + this package's kernels) against the CPU restatement
of the reference model, and the elementwise kernels against the oracle."""

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


@pytest.mark.parametrize("head_dim,T", [(64, 256), (128, 512)])
def test_tiny_prefill_matches_reference_model(head_dim, T):
    cfg = P.PrefillConfig(vocab_size=1000, d_model=2 * head_dim, n_layers=2, n_heads=2, d_ff=256)
    params = P.init_params(cfg, seed=0)
    g = torch.Generator().manual_seed(1)
    for k in ("q_gain", "k_gain"):                       # exercise non-trivial gains and sinks
        params[k] = 0.75 + 0.5 * torch.rand(params[k].shape, generator=g)
    params["sink"] = torch.randn(params["sink"].shape, generator=g) * 0.3
    tokens = torch.randint(0, cfg.vocab_size, (2, T), generator=g)
    want_h = M.forward_hidden(params, tokens, cfg)
    obj_w, pt_w = M.head_loss(params, want_h, tokens, cfg)
    model = P.Prefill(cfg, params, DEV, seq_len=T)
    got_h = model.hidden(tokens.to(DEV))
    assert rel_l2(got_h, want_h) < 2e-2                  # two layers of bf16 activations
    obj, pt, nll = model.loss(tokens.to(DEV), tokens.to(DEV), want_nll=True)
    assert rel_l2(nll, R.nll_from_pt(pt_w)) < 1e-2
    np.testing.assert_allclose(float(obj), float(obj_w), rtol=5e-3)
