"""The CPU oracle against vectors produced by the reference's own source files
(tests/golden/make_golden.py) — this is what pins the oracle."""

import math

import numpy as np
import pytest
import torch

from oracle import algebraic_ref as R


def T(a):
    return torch.from_numpy(np.asarray(a))


def close(a, b, rtol, atol=0.0):
    np.testing.assert_allclose(np.asarray(a), np.asarray(b), rtol=rtol, atol=atol)


def test_rho_int_pow_alu(golden):
    g = golden
    close(R.rho(T(g["rho_x64"])), g["rho_y64"], 1e-14)
    close(R.rho(T(g["rho_x32"])), g["rho_y32"], 3e-7)
    for n in (8, 16, 32):
        close(R.int_pow(R.rho(T(g["rho_x64"]) / 10.0), n), g[f"ipow{n}_y64"], 1e-13)
    for beta in (1.0, 0.5):
        x = T(g[f"alu_b{beta}_x64"])
        close(R.alu(x, beta), g[f"alu_b{beta}_y64"], 1e-13, 1e-300)
        close(R.alu(x.float(), beta), g[f"alu_b{beta}_y32"], 1e-6, 1e-30)
    close(R.kernel_sink_logit(2.0, 16, 8.0), g["sink_logit_omega2_n16_c8"], 1e-15)


def test_rms_norm(golden):
    g = golden
    x, gain = T(g["rms_x"]), T(g["rms_gain"])
    close(R.rms_norm(x, gain, 1e-5), g["rms_y_eps1e-5"], 2e-6, 2e-6)
    close(R.rms_norm(x, gain, 1e-3), g["rms_y_eps1e-3"], 2e-6, 2e-6)
    close(R.rms_norm(x, None, 1e-5), g["rms_y_nogain"], 2e-6, 2e-6)
    close(R.rms_norm(T(g["rms128_x"]), torch.ones(128), 1e-5), g["rms128_y"], 2e-6, 2e-6)
    assert torch.all(R.rms_norm(x, gain)[0, 0, 0] == 0)       # the all-zero row stays zero


def test_cayley_and_rotary(golden):
    g = golden
    for D, Tn in ((64, 300), (128, 257)):
        c, s = R.cayley_table_geometric(D, Tn)
        close(c, g[f"cayley_cos_D{D}_T{Tn}"], 0, 2e-6)
        close(s, g[f"cayley_sin_D{D}_T{Tn}"], 0, 2e-6)
    c, s = R.cayley_table_geometric(64, 300)
    close(R.apply_rotary(T(g["rot_x"]), c, s), g["rot_y"], 1e-5, 1e-5)


@pytest.mark.parametrize("n,c", [(8, 1.0), (16, 16.0), (32, 4.0)])
def test_weights(golden, n, c):
    g = golden
    s = T(g["w_scores"])
    mask = torch.tril(torch.ones(7, 7, dtype=torch.bool))[None, None]
    b = torch.full((1, 3, 1, 1), 0.7, dtype=torch.float64)
    close(R.asinh_power_weights(s, mask, n, c, b), g[f"w_n{n}_c{c}_sink"], 1e-12, 1e-300)
    close(R.asinh_power_weights(s, mask, n, c, None), g[f"w_n{n}_c{c}_nosink"], 1e-12, 1e-300)
    big = R.asinh_power_weights(s * 1e6, mask, n, c, None)
    close(big, g[f"w_n{n}_c{c}_big"], 1e-11, 1e-300)
    assert torch.isfinite(big).all()


def test_attention(golden):
    g = golden
    q, k, v, sink = (T(g[x]) for x in ("att_q", "att_k", "att_v", "att_sink"))
    cases = {"att_o_n16_c16_sink": (16, 16.0, sink), "att_o_n16_c8_sink": (16, 8.0, sink),
             "att_o_n16_c8_nosink": (16, 8.0, None), "att_o_n8_c1_sink": (8, 1.0, sink),
             "att_o_n32_c8_nosink": (32, 8.0, None)}
    for key, (n, c, s) in cases.items():
        o = R.asinh_attention(q, k, v, n=n, c=c, sink_logit=s)
        close(o, g[key], 2e-5, 1e-5)
        ob = R.asinh_attention(q, k, v, n=n, c=c, sink_logit=s, row_block=32)
        close(ob, g[key], 2e-5, 1e-5)
    qt, vt = T(g["tail_q"]), T(g["tail_v"])
    for sign in (1.0, -1.0):
        for ws in (0, 1):
            sk = torch.zeros(1) if ws else None
            o = R.asinh_attention(qt, qt * sign, vt, n=16, c=8.0, sink_logit=sk)
            assert torch.isfinite(o).all()
            close(o, g[f"tail_o_sign{sign}_sink{ws}"], 2e-5, 1e-5)


@pytest.mark.parametrize("D", [64, 128])
def test_layer_front_end(golden, D):
    g = golden
    q0, k0, v0 = (T(g[f"layer_D{D}_{x}"]) for x in "qkv")
    Tn = q0.shape[-2]
    cs, sn = R.cayley_table_geometric(D, Tn)
    gain = torch.ones(D)
    qn = R.apply_rotary(R.rms_norm(q0, gain), cs, sn)
    kn = R.apply_rotary(R.rms_norm(k0, gain), cs, sn)
    close(qn, g[f"layer_D{D}_qn"], 1e-5, 1e-5)
    close(kn, g[f"layer_D{D}_kn"], 1e-5, 1e-5)
    o = R.asinh_attention(qn, kn, v0, n=16, c=8.0, sink_logit=T(g[f"layer_D{D}_sink"]))
    close(o, g[f"layer_D{D}_o"], 2e-5, 1e-5)


@pytest.mark.parametrize("n,c", [(16, 16.0), (8, 2.0)])
def test_likelihoods(golden, n, c):
    g = golden
    z, t = T(g["lik_z"]), T(g["lik_t"])
    o, p = R.algebraic_likelihood(z, t, n, c)
    close(p, g[f"lik_exact_n{n}_pt"], 1e-12); close(o, g[f"lik_exact_n{n}_obj"], 1e-12)
    o, p = R.algebraic_likelihood_lean(z, t, n, c)
    close(p, g[f"lik_lean_n{n}_pt"], 1e-12); close(o, g[f"lik_lean_n{n}_obj"], 1e-12)
    o, p = R.algebraic_likelihood_lean(z.float(), t, n, c)
    close(p, g[f"lik_lean32_n{n}_pt"], 2e-5); close(o, g[f"lik_lean32_n{n}_obj"], 2e-6)
    close(R.algebraic_probs(z, n, c), g[f"probs_n{n}"], 1e-12, 1e-300)


@pytest.mark.parametrize("n,c", [(16, 16.0), (8, 2.0)])
def test_likelihood_vjp_rule(golden, n, c):
    """The logit cotangent of the reference's custom VJPs (algebraic.py:255-262, 309-316), evaluated by
    the reference's own backward functions, against the oracle's restatement; the exact and the lean
    rule agree while the clamp is idle; and the rule is the gradient of the mean negative
    log-likelihood, which autograd through the primal value mean(1 - pt) is not."""
    g = golden
    z, t = T(g["lik_z"]), T(g["lik_t"])
    got = R.algebraic_likelihood_lean_vjp(z, t, n, c, 0.75)
    close(got, g[f"lik_lean_n{n}_vjp"], 1e-11, 1e-15)
    close(got, g[f"lik_exact_n{n}_vjp"], 1e-9, 1e-13)
    zz = z.clone().requires_grad_(True)
    p = R.algebraic_probs(zz, n, c)
    nll = -torch.log(p.gather(-1, t.long()[:, None])[:, 0]).mean()
    nll.backward()
    close(got, 0.75 * zz.grad, 1e-9, 1e-13)
    zp = z.clone().requires_grad_(True)
    R.algebraic_likelihood_lean(zp, t, n, c)[0].backward()
    assert float((0.75 * zp.grad - got).abs().max()) > 1e-3 * float(got.abs().max())


@pytest.mark.parametrize("tag,zkey", [("", "lik_z"), ("_huge", "ce_zhuge")])
def test_cross_entropy_head(golden, tag, zkey):
    """The "ce" kind: the reference's dense definition (standard.py:41-47) and the fused kernel's
    telemetry from (logsumexp, target logit) (fused_head.py:221-223) against the oracle."""
    g = golden
    z, t = T(g[zkey]).float(), T(g["lik_t"])
    obj, nll = R.cross_entropy(z, t)
    close(nll, g[f"ce{tag}_nll"], 2e-6, 2e-6); close(obj, g[f"ce{tag}_obj"], 2e-6)
    close(nll, g[f"ce{tag}_tel_nll"], 2e-6, 2e-6); close(obj, g[f"ce{tag}_tel_obj"], 2e-6)


def test_likelihood_vjp_rule_clamp_is_straight_through(golden):
    g = golden
    z, t = T(g["lik_zclamp"]), T(g["lik_t"])
    got = R.algebraic_likelihood_lean_vjp(z, t, 8, 2.0, 1.0)
    close(got, g["lik_lean_n8_vjp_clamped"], 1e-11, 1e-15)
    assert float(got[2, 11]) > 0.0            # the clamped entry still receives (p - y) r n / (c N)


def test_dispatch_constants(golden):
    g = golden
    for n in (8, 16):
        for V, a, b in zip(g["clamp_vocabs"], g[f"lik_clamp_n{n}"], g[f"head_clamp_n{n}"]):
            assert R.likelihood_clamp(int(V), n) == a
            close(R.likelihood_clamp(int(V), n), b, 1e-15)
    for n in (8, 16, 32):
        for Tn, cl, sh in zip(g["variant_seqs"], g[f"variant_clamp_n{n}"], g[f"variant_shift_n{n}"]):
            assert R.flash_clamp(int(Tn), n) == cl
            assert R.flash_default_shift(int(Tn), n) == bool(sh)


def test_kernel_side_forms(golden):
    g = golden
    x = T(g["krho_x"])
    close(R.rho_fast(x), g["krho_fast"], 1e-6, 1e-7)
    close(R.rho(x), g["krho_exact"], 1e-6)
    l = T(g["invroot_l"])
    close(R.inv_root(l, 16), g["invroot_n16"], 1e-6)
    close(R.inv_root(l, 8), g["invroot_n8"], 1e-6)
    clamp8 = np.float32(R.likelihood_clamp(50304, 8))
    pt, obj = R.fused_head_telemetry(T(g["tel_l"]), T(g["tel_zt"]), 8, 2.0, float(clamp8))
    close(pt, g["tel_pt"], 2e-5, 1e-30)
    close(obj, g["tel_obj"], 1e-6)


@pytest.mark.parametrize("tag,dtype,tol_hidden,tol_nll", [("f32", torch.float32, 2e-5, 2e-5), ("bf16", torch.bfloat16, 1e-2, 1e-2)])
def test_model_forward_matches_reference_model(golden, tag, dtype, tol_hidden, tol_nll):
    """oracle/model_ref.py against the reference's own model.forward_hidden + head_loss
    (src/algebraic/model.py:162-231, executed by tests/golden/make_golden.py) on a two-layer
    algebraic configuration with random gains and sinks: in float32, where only summation order
    differs, and in bfloat16, where every rounding point has to sit where the reference's does."""
    from algebraic_transformer_b200.prefill import PrefillConfig
    from oracle import model_ref as MR
    g = golden
    cfg = PrefillConfig(vocab_size=384, d_model=128, n_layers=2, n_heads=2, d_ff=256)
    params = {"embed": T(g["model_embed"]), "embed_gain": T(g["model_embed_gain"]), "final_gain": T(g["model_final_gain"])}
    for name in ("w_q", "w_k", "w_v", "w_o", "w_g", "w_u", "w_d", "ln1", "ln2", "q_gain", "k_gain", "sink"):
        params[name] = T(g[f"model_layers_{name}"])
    tokens, targets = T(g["model_tokens"]), T(g["model_targets"])
    hidden = MR.forward_hidden(params, tokens, cfg, dtype=dtype)
    assert hidden.dtype == dtype
    want = T(g[f"model_{tag}_hidden"])
    rel = float((hidden.float() - want).norm() / want.norm())
    assert rel <= tol_hidden, rel
    obj, pt = MR.head_loss(params, hidden, targets, cfg)
    want_nll = -torch.log(T(g[f"model_{tag}_pt"]).clamp_min(1e-30))
    nll = -torch.log(pt.float().clamp_min(1e-30))
    rel_nll = float((nll - want_nll).norm() / want_nll.norm())
    assert rel_nll <= tol_nll, rel_nll
    close(obj, g[f"model_{tag}_obj"], 1e-4 if tag == "f32" else 2e-2)
