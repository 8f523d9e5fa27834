"""Generate `reference_vectors.npz`: inputs and outputs of the reference's own
dense definitions, evaluated by the reference's unmodified source files.

The reference is JAX code and JAX is not installable here, so its modules are
imported on top of a NumPy-backed stand-in for the handful of `jax.numpy` /
`jax.lax` calls they make (`_jax_numpy_shim.py`).  Every number stored is
computed by the reference's code (src/algebraic/algebraic.py,
src/algebraic/kernels/flash.py host helpers, src/algebraic/kernels/fused_head.py
host helpers); inputs come from `numpy.random.default_rng(seed)`.

Usage (build container only; the reference checkout is not needed by tests):

    python tests/golden/make_golden.py --reference /path/to/reference

The tests read only the committed `.npz`.
"""

import argparse
import math
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", required=True, help="path of the reference checkout")
    ap.add_argument("--out", default=os.path.join(HERE, "reference_vectors.npz"))
    args = ap.parse_args()

    sys.path.insert(0, HERE)
    import _jax_numpy_shim
    _jax_numpy_shim.install()
    sys.path.insert(0, os.path.join(args.reference, "src"))
    from algebraic import algebraic as A
    from algebraic.kernels import flash as FK
    from algebraic.kernels import fused_head as FH
    from algebraic import standard as S
    import jax                                            # the stand-in installed above

    def jax_logsumexp(a):
        return jax.nn.logsumexp(a, axis=-1)

    f32, f64 = np.float32, np.float64
    out = {}

    # --- rho / int_pow / alu (algebraic.py:31-51, 86-105) -----------------------
    x64 = np.linspace(-50, 50, 1001, dtype=f64)
    x32 = np.linspace(-12, 12, 769).astype(f32)
    out["rho_x64"], out["rho_y64"] = x64, A.rho(x64)
    out["rho_x32"], out["rho_y32"] = x32, A.rho(x32)
    for n in (8, 16, 32):
        out[f"ipow{n}_y64"] = A.int_pow(A.rho(x64 / 10.0), n)
    xa = np.linspace(-40, 40, 801, dtype=f64)
    for beta in (1.0, 0.5):
        out[f"alu_b{beta}_x64"] = xa
        out[f"alu_b{beta}_y64"] = A.alu(xa, beta)
        out[f"alu_b{beta}_y32"] = A.alu(xa.astype(f32), beta)
    out["sink_logit_omega2_n16_c8"] = np.array(A.kernel_sink_logit(2.0, 16, 8.0))

    # --- rms_norm (algebraic.py:76-83) ------------------------------------------
    rng = np.random.default_rng(181)
    x = (3 * rng.standard_normal((2, 3, 8, 64))).astype(f32)
    x[0, 0, 0] = 0
    gain = (0.25 + 4 * rng.random(64)).astype(f32)
    out["rms_x"], out["rms_gain"] = x, gain
    out["rms_y_eps1e-5"] = A.rms_norm(x, gain, 1e-5)
    out["rms_y_eps1e-3"] = A.rms_norm(x, gain, 1e-3)
    out["rms_y_nogain"] = A.rms_norm(x, None, 1e-5)
    x128 = rng.standard_normal((1, 2, 8, 128)).astype(f32)
    out["rms128_x"] = x128
    out["rms128_y"] = A.rms_norm(x128, np.ones(128, f32), 1e-5)

    # --- Cayley tables + rotary (algebraic.py:124-179) --------------------------
    for D, T in ((64, 300), (128, 257)):
        c, s = A.cayley_table_geometric(D, T)
        out[f"cayley_cos_D{D}_T{T}"], out[f"cayley_sin_D{D}_T{T}"] = c, s
    c, s = A.cayley_table_geometric(64, 300)
    xr = rng.standard_normal((1, 1, 300, 64)).astype(f32)
    out["rot_x"], out["rot_y"] = xr, A.apply_rotary(xr, c, s)

    # --- normalised weights (algebraic.py:186-204) ------------------------------
    rng = np.random.default_rng(0)
    s64 = rng.standard_normal((2, 3, 7, 7)) * 5
    mask = np.tril(np.ones((7, 7), bool))[None, None]
    b = np.full((1, 3, 1, 1), 0.7, f64)
    out["w_scores"] = s64
    for n, c_ in ((8, 1.0), (16, 16.0), (32, 4.0)):
        out[f"w_n{n}_c{c_}_sink"] = A.asinh_power_weights(s64, mask, n, c_, b)
        out[f"w_n{n}_c{c_}_nosink"] = A.asinh_power_weights(s64, mask, n, c_, None)
        out[f"w_n{n}_c{c_}_big"] = A.asinh_power_weights(s64 * 1e6, mask, n, c_, None)

    # --- dense attention (algebraic.py:207-216) ---------------------------------
    rng = np.random.default_rng(1)
    q = (rng.standard_normal((1, 3, 80, 64)) * 1.5).astype(f32)
    k = (rng.standard_normal((1, 3, 80, 64)) * 1.5).astype(f32)
    v = rng.standard_normal((1, 3, 80, 64)).astype(f32)
    sink = (rng.standard_normal(3) * 0.5).astype(f32)[None, :, None, None]
    out["att_q"], out["att_k"], out["att_v"], out["att_sink"] = q, k, v, sink
    out["att_o_n16_c16_sink"] = A.asinh_attention(q, k, v, n=16, c=16.0, sink_logit=sink)
    out["att_o_n16_c8_sink"] = A.asinh_attention(q, k, v, n=16, c=8.0, sink_logit=sink)
    out["att_o_n16_c8_nosink"] = A.asinh_attention(q, k, v, n=16, c=8.0, sink_logit=None)
    out["att_o_n8_c1_sink"] = A.asinh_attention(q, k, v, n=8, c=1.0, sink_logit=sink)
    out["att_o_n32_c8_nosink"] = A.asinh_attention(q, k, v, n=32, c=8.0, sink_logit=None)
    # constant +/- tails: weight overflow and whole-row underflow without the shift
    qt = np.full((1, 1, 64, 64), math.sqrt(1000.0), f32)
    vt = rng.standard_normal((1, 1, 64, 64)).astype(f32)
    out["tail_q"], out["tail_v"] = qt, vt
    for sign in (1.0, -1.0):
        for with_sink in (False, True):
            sk = np.zeros((1, 1, 1, 1), f32) if with_sink else None
            out[f"tail_o_sign{sign}_sink{int(with_sink)}"] = A.asinh_attention(
                qt, qt * f32(sign), vt, n=16, c=8.0, sink_logit=sk)
    # whole layer front end: QK-norm (unit gain) -> Cayley rotation -> attention
    rng = np.random.default_rng(2)
    for D, T in ((64, 128), (128, 64)):
        shp = (1, 2, T, D)
        q0, k0, v0 = (rng.standard_normal(shp).astype(f32) for _ in range(3))
        g = np.ones(D, f32)
        cs, sn = A.cayley_table_geometric(D, T)
        qn = A.apply_rotary(A.rms_norm(q0, g, 1e-5), cs, sn)
        kn = A.apply_rotary(A.rms_norm(k0, g, 1e-5), cs, sn)
        sk = (rng.standard_normal(2) * 0.02).astype(f32)[None, :, None, None]
        out[f"layer_D{D}_q"], out[f"layer_D{D}_k"], out[f"layer_D{D}_v"] = q0, k0, v0
        out[f"layer_D{D}_sink"] = sk
        out[f"layer_D{D}_qn"], out[f"layer_D{D}_kn"] = qn, kn
        out[f"layer_D{D}_o"] = A.asinh_attention(qn, kn, v0, n=16, c=8.0, sink_logit=sk)

    # --- likelihood heads (algebraic.py:223-245, 277-301) -----------------------
    rng = np.random.default_rng(3)
    z = rng.standard_normal((7, 300)) * 6
    t = np.array([0, 5, 299, 17, 17, 100, 3])
    out["lik_z"], out["lik_t"] = z, t
    for n, c_ in ((16, 16.0), (8, 2.0)):
        o1, p1 = A.algebraic_likelihood(z, t, n, c_)
        o2, p2 = A.algebraic_likelihood_lean(z, t, n, c_)
        o3, p3 = A.algebraic_likelihood_lean(z.astype(f32), t, n, c_)
        out[f"lik_exact_n{n}_obj"], out[f"lik_exact_n{n}_pt"] = np.array(o1), p1
        out[f"lik_lean_n{n}_obj"], out[f"lik_lean_n{n}_pt"] = np.array(o2), p2
        out[f"lik_lean32_n{n}_obj"], out[f"lik_lean32_n{n}_pt"] = np.array(o3), p3
        out[f"probs_n{n}"] = A.algebraic_probs(z, n, c_)
        # the custom VJPs' backward rules, called directly (algebraic.py:255-262, 309-316): the logit
        # cotangent for an objective cotangent of 0.75
        out[f"lik_exact_n{n}_vjp"] = A._alg_lik_bwd(n, c_, (A.algebraic_probs(z, n, c_), z, t), (0.75, None))[0]
        out[f"lik_lean_n{n}_vjp"] = A._lean_bwd(n, c_, (z, t), (0.75, None))[0]
    # a row whose largest logit sits above the clamp: the lean rule is straight-through there
    zc = z.copy()
    zc[2, 11] = 2.0 * 8 * A.likelihood_clamp(300, 8)
    out["lik_zclamp"] = zc
    out["lik_lean_n8_vjp_clamped"] = A._lean_bwd(8, 2.0, (zc, t), (1.0, None))[0]
    # the "ce" head (standard.py:41-47) and the fused kernel's telemetry for it (fused_head.py:221-223),
    # on the same logits and on a copy with one huge logit per row sign (the shift must absorb it)
    zh = z.copy()
    zh[1, 4], zh[3, 200] = 3.0e4, -3.0e4
    out["ce_zhuge"] = zh
    for tag, zz in (("", z), ("_huge", zh)):
        o_ce, nll_ce = S.cross_entropy(zz.astype(f32), t)
        out[f"ce{tag}_obj"], out[f"ce{tag}_nll"] = np.array(o_ce), nll_ce
        lse = jax_logsumexp(zz.astype(f32))
        zt_ = np.take_along_axis(zz.astype(f32), t[:, None], axis=-1)[:, 0]
        tel, tobj = FH._telemetry(lse, zt_, "ce", 16, 16.0, 0.0)
        out[f"ce{tag}_tel_nll"], out[f"ce{tag}_tel_obj"] = tel, np.array(tobj)
    vocabs = np.array([50304, 32768, 32000, 4096, 97])
    out["clamp_vocabs"] = vocabs
    for n in (8, 16):
        out[f"lik_clamp_n{n}"] = np.array([A.likelihood_clamp(int(V), n) for V in vocabs])
        # fused_head.py:273 computes the same bound with its own helper
        out[f"head_clamp_n{n}"] = np.array([0.25 * FH._root(1e38 / int(V), n) for V in vocabs])

    # --- flash dispatch constants (flash.py:732-760) ----------------------------
    seqs = np.array([256, 512, 1024, 2048, 8192, 16384, 32768])
    out["variant_seqs"] = seqs
    for n in (8, 16, 32):
        vs = [FK.make_variant("asinh", n, 8.0, int(T)) for T in seqs]
        out[f"variant_clamp_n{n}"] = np.array([v_.clamp for v_ in vs])
        out[f"variant_shift_n{n}"] = np.array([v_.shift for v_ in vs])
    # kernel-side rho forms and root statistic (flash.py:76-113)
    xs = np.linspace(-8, 8, 513).astype(f32)
    out["krho_x"] = xs
    out["krho_fast"] = FK._rho(xs, True)[0]
    out["krho_exact"] = FK._rho(xs, False)[0]
    l = np.geomspace(1e-3, 1e12, 61).astype(f32)
    out["invroot_l"] = l
    out["invroot_n16"] = FK._inv_root(l, 16)
    out["invroot_n8"] = FH._inv_root(l, 8)
    # fused head telemetry from (sigma, zt) (fused_head.py:219-229)
    zt = np.linspace(-30, 30, 61).astype(f32)
    lrow = np.geomspace(5e4, 5e9, 61).astype(f32)
    clamp8 = f32(0.25 * FH._root(1e38 / 50304, 8))
    pt, obj = FH._telemetry(FH._inv_root(lrow, 8), zt, "alg_ce", 8, 2.0, clamp8)
    out["tel_zt"], out["tel_l"], out["tel_pt"], out["tel_obj"] = zt, lrow, pt, np.array(obj)

    # --- the model's forward pass (model.py:162-231): two tiny algebraic configurations, one in
    #     float32 (pins the structure to 1e-5) and one in bfloat16 (pins the rounding points) ---
    from algebraic import config as CFG
    from algebraic import model as M
    for tag, dtype in (("f32", "float32"), ("bf16", "bfloat16")):
        cfg = CFG.algebraic("proxy", vocab_size=384, d_model=128, n_layers=2, n_heads=2, d_ff=256, seq_len=48,
                            dtype=dtype, attn_impl="dense", head_impl="dense")
        params = M.init_params(cfg, jax.random.PRNGKey(7))
        rng = np.random.default_rng(70)
        params["embed"] = (params["embed"] * 5).astype(f32)      # logits of order one, so that pt is not flat
        for name in ("embed_gain", "final_gain"):                 # non-trivial gains and sinks: a swapped or
            params[name] = (params[name] + 0.2 * rng.standard_normal(params[name].shape)).astype(f32)
        for name in ("ln1", "ln2", "q_gain", "k_gain", "sink"):   # dropped one must show
            leaf = params["layers"][name]
            params["layers"][name] = (leaf + 0.2 * rng.standard_normal(leaf.shape)).astype(f32)
        for name in ("w_q", "w_k", "w_v", "w_o", "w_g", "w_u", "w_d"):
            params["layers"][name] = (params["layers"][name] * 3).astype(f32)
        tokens = rng.integers(0, cfg.vocab_size, (2, cfg.seq_len))
        targets = rng.integers(0, cfg.vocab_size, (2, cfg.seq_len))
        targets[0] = tokens[0]                                    # likely targets in one sequence, unlikely in the other
        tables = M.position_tables(cfg)
        hidden = M.forward_hidden(params, tokens, cfg, tables)
        obj, pt = M.head_loss(params, hidden, targets, cfg)
        if tag == "f32":
            out["model_tokens"], out["model_targets"] = tokens.astype(np.int64), targets.astype(np.int64)
            out["model_embed"] = np.asarray(params["embed"])
            out["model_embed_gain"], out["model_final_gain"] = np.asarray(params["embed_gain"]), np.asarray(params["final_gain"])
            for name, leaf in params["layers"].items():
                out[f"model_layers_{name}"] = np.asarray(leaf)
        assert str(np.asarray(hidden).dtype) == dtype, hidden.dtype
        out[f"model_{tag}_hidden"] = np.asarray(hidden).astype(f32)
        out[f"model_{tag}_obj"], out[f"model_{tag}_pt"] = np.asarray(obj, f32), np.asarray(pt, f32)

    np.savez_compressed(args.out, **{k_: np.asarray(v_) for k_, v_ in out.items()})
    print(f"wrote {args.out}: {len(out)} arrays, {os.path.getsize(args.out)} bytes")


if __name__ == "__main__":
    main()
