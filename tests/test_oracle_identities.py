"""Formula identities the reference's own CPU tests pin (tests/test_components.py
of the reference), re-run against the oracle with NumPy transcendental functions
as the independent side."""

import numpy as np
import pytest
import torch

from oracle import algebraic_ref as R


def test_rho_identities():                                   # test_components.py:18-24
    x = torch.linspace(-50, 50, 1001, dtype=torch.float64)
    y = torch.linspace(-3, 7, 1001, dtype=torch.float64)
    np.testing.assert_allclose(R.rho(x), np.exp(np.arcsinh(x.numpy())), rtol=1e-12)
    np.testing.assert_allclose(R.rho(x) * R.rho(-x), 1.0, rtol=1e-12)
    oplus = x * torch.sqrt(1 + y * y) + y * torch.sqrt(1 + x * x)
    np.testing.assert_allclose(R.rho(x) * R.rho(y), R.rho(oplus), rtol=1e-10)


@pytest.mark.parametrize("n,c", [(8, 1.0), (16, 16.0), (32, 4.0)])
def test_weights_equal_softmax_of_compressed_logits(n, c):   # test_components.py:27-40
    g = torch.Generator().manual_seed(0)
    s = torch.randn((2, 3, 7, 7), generator=g, dtype=torch.float64) * 5
    mask = torch.tril(torch.ones(7, 7, dtype=torch.bool))[None, None]
    b = torch.full((1, 3, 1, 1), 0.7, dtype=torch.float64)
    w = R.asinh_power_weights(s, mask, n, c, b)
    logits = torch.where(mask, n * torch.asinh(s / c), torch.tensor(float("-inf"), dtype=torch.float64))
    full = torch.cat([logits, (n * torch.asinh(b / c)).expand(2, 3, 7, 1)], -1)
    ref = torch.softmax(full, -1)[..., :-1]
    np.testing.assert_allclose(w, ref, rtol=1e-10, atol=1e-14)
    big = R.asinh_power_weights(s * 1e6, mask, n, c, None)
    assert torch.isfinite(big).all() and np.allclose(big.sum(-1), 1.0)


def test_cayley_tables_are_exact_rotations():                # test_components.py:59-68
    c, s = R.cayley_table_geometric(64, 300)
    angles = 2 * np.arctan(0.5 * 1e4 ** (-np.arange(32) / 32))
    m = np.arange(300)[:, None]
    np.testing.assert_allclose(c, np.cos(m * angles), atol=2e-5)
    np.testing.assert_allclose(s, np.sin(m * angles), atol=2e-5)
    np.testing.assert_allclose(c * c + s * s, 1.0, atol=1e-6)


def test_alu():                                              # test_components.py:71-78
    x = torch.linspace(-40, 40, 2001, dtype=torch.float64)
    for beta in (1.0, 0.5):
        ref = 0.5 * x * (1 + beta * x / torch.sqrt(1 + (beta * x) ** 2))
        np.testing.assert_allclose(R.alu(x, beta), ref, rtol=1e-9, atol=1e-15)


@pytest.mark.parametrize("n,c", [(16, 16.0), (8, 2.0)])
def test_lean_equals_exact_and_true_logprob(n, c):           # test_components.py:43-56, 99-109
    g = torch.Generator().manual_seed(3)
    z = torch.randn((7, 300), generator=g, dtype=torch.float64) * 6
    t = torch.tensor([0, 5, 299, 17, 17, 100, 3])
    _, p1 = R.algebraic_likelihood_lean(z, t, n, c)
    _, p2 = R.algebraic_likelihood(z, t, n, c)
    np.testing.assert_allclose(p1, p2, rtol=1e-9)
    np.testing.assert_allclose(np.log(p2), R.head_logprob_fp64(z, t, n, c), rtol=1e-9)


def test_attention_matches_fp64_formula_and_is_causal():     # test_e2e_acceptance.py:563-594
    g = torch.Generator().manual_seed(5)
    q, k, v = (torch.randn((1, 2, 48, 64), generator=g) for _ in range(3))
    sink = torch.tensor([0.3, -0.2])
    o = R.asinh_attention(q, k, v, n=16, c=8.0, sink_logit=sink)
    ref = R.attention_fp64_transcendental(q, k, v, n=16, c=8.0, sink_logit=sink)
    assert (o.double() - ref).norm() / ref.norm() < 2e-6
    k2, v2 = k.clone(), v.clone()
    k2[:, :, 30:] += 5.0
    v2[:, :, 30:] -= 3.0
    o2 = R.asinh_attention(q, k2, v2, n=16, c=8.0, sink_logit=sink)
    assert torch.equal(o[:, :, :30], o2[:, :, :30])          # the future never leaks


def test_fused_statistic_equals_dense_head():
    """The fused kernel's (l, zt) route gives the dense head's p_t; vocab shards add up."""
    g = torch.Generator().manual_seed(7)
    N, d, V = 64, 96, 1000
    h = torch.randn((N, d), generator=g).bfloat16()
    E = torch.randn((V, d), generator=g) * 0.1
    t = torch.randint(0, V, (N,), generator=g)
    obj_d, pt_d = R.head_loss_dense(h, E, t, 8, 2.0)
    obj_f, pt_f = R.fused_head(h, E, t, n=8, c=2.0)
    np.testing.assert_allclose(pt_f, pt_d, rtol=2e-5)
    np.testing.assert_allclose(obj_f, obj_d, rtol=1e-5)
    parts = [R.fused_head_stats(h, E, t, 8, 2.0, vocab_lo=a, vocab_hi=b, vocab_total=V)
             for a, b in ((0, 384), (384, 640), (640, 1000))]
    l = sum(p[0] for p in parts)
    zt = sum(p[1] for p in parts)
    l0, zt0 = R.fused_head_stats(h, E, t, 8, 2.0)
    np.testing.assert_allclose(l, l0, rtol=1e-5)
    np.testing.assert_allclose(zt, zt0, rtol=1e-6, atol=1e-6)
    lp = R.head_logprob_fp64(R.head_logits(h, E), t, 8, 2.0)
    np.testing.assert_allclose(-R.nll_from_pt(pt_f), lp, rtol=1e-4, atol=1e-5)


def test_range_guard_and_stat():
    g = torch.Generator().manual_seed(9)
    q, k, v = (torch.randn((1, 2, 64, 64), generator=g) for _ in range(3))
    qn, kn = R.rms_norm(q, torch.ones(64)), R.rms_norm(k, torch.ones(64))
    assert R.range_guard_in_range(qn, kn, v, torch.zeros(2), n=16, c=8.0)
    big = torch.full((1, 1, 64, 64), 1000.0 ** 0.5)
    assert not R.range_guard_in_range(big, big, v[:, :1], None, n=16, c=8.0)
    assert not R.range_guard_in_range(qn, kn, v * 1e9, None, n=16, c=8.0)
    s0 = R.attention_row_stat(qn, kn, n=16, c=8.0, sink_logit=torch.zeros(2), shifted=False)
    s1 = R.attention_row_stat(qn, kn, n=16, c=8.0, sink_logit=torch.zeros(2), shifted=True)
    # both statistics encode the same denominator: (shifted stat)^n == 1/l
    np.testing.assert_allclose(R.int_pow(s1, 16), s0, rtol=2e-4)
