"""`.backward()` through the three fused operators (algebraic_transformer_b200.autograd) against
autograd through the CPU oracle — and, for the algebraic head, against the oracle's restatement of
the reference's custom VJP, which is what the reference's `jax.grad` returns."""

import pytest
import torch

from algebraic_transformer_b200 import autograd as G
from oracle import algebraic_ref as R

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def rel_l2(a, b):
    a, b = a.detach().double().cpu(), b.detach().double().cpu()
    return float((a - b).norm() / b.norm().clamp_min(1e-30))


def randn(shape, seed, dtype=torch.float32, scale=1.0):
    g = torch.Generator().manual_seed(seed)
    return (torch.randn(shape, generator=g) * scale).to(dtype)


def test_layer_front_end_backward():
    """QK-norm -> attention, a weighted sum of the output as the loss: gradients reach q, k, v, both
    gains and the sink through two chained operators."""
    B, H, T, D = 1, 2, 256, 64
    q, k, v = (randn((B, H, T, D), 601 + i, torch.bfloat16) for i in range(3))
    gq, gk = 0.5 + torch.rand(D, generator=torch.Generator().manual_seed(611)), torch.ones(D)
    sink = randn((H,), 612) * 0.3
    w = randn((B, H, T, D), 613, torch.bfloat16)

    leaves = [t.float().clone().requires_grad_(True) for t in (q, k, v, gq, gk, sink)]
    qf, kf, vf, gqf, gkf, sf = leaves
    # (the kernels round the normalised q, k to bf16 between the two operators; the oracle chain does not,
    # which the tolerance below absorbs)
    qn = R.rms_norm(qf, gqf, 1e-5)
    kn = R.rms_norm(kf, gkf, 1e-5)
    out = R.asinh_attention(qn, kn, vf, n=16, c=8.0, sink_logit=sf)
    (out * w.float()).sum().backward()

    dl = [t.to(DEV).clone().requires_grad_(True) for t in (q, k, v, gq, gk, sink)]
    qd, kd, vd, gqd, gkd, sd = dl
    o = G.attention(G.qk_norm(qd, gqd), G.qk_norm(kd, gkd), vd, sd, n=16, c=8.0)
    (o.float() * w.to(DEV).float()).sum().backward()
    for got, want, name in zip(dl, leaves, "q k v q_gain k_gain sink".split()):
        assert got.grad is not None, name
        assert rel_l2(got.grad, want.grad) < 3e-2, (name, rel_l2(got.grad, want.grad))


@pytest.mark.parametrize("kind", ["alg_ce", "ce"])
def test_head_loss_backward(kind):
    N, d, V = 256, 128, 1000
    h = randn((N, d), 621, torch.bfloat16)
    E = randn((V, d), 622) * 0.3
    t = torch.randint(0, V, (N,), generator=torch.Generator().manual_seed(623))
    if kind == "alg_ce":
        want_dh, want_de = R.head_vjp_dense(h, E.bfloat16(), t, 8, 2.0, g=3.0)
        want_obj = R.head_loss_dense(h, E.bfloat16(), t, 8, 2.0)[0]
    else:
        hf, ef = h.float().requires_grad_(True), E.bfloat16().float().requires_grad_(True)
        want_obj = R.cross_entropy(hf @ ef.t(), t)[0]
        (3.0 * want_obj).backward()
        want_dh, want_de, want_obj = hf.grad, ef.grad, want_obj.detach()
    hd = h.to(DEV).requires_grad_(True)
    Ed = E.to(DEV).requires_grad_(True)
    obj, tel = G.head_loss(hd, Ed, t.to(DEV), kind=kind, n=8, c=2.0)
    assert not tel.requires_grad
    (3.0 * obj).backward()
    assert abs(float(obj.detach()) - float(want_obj)) < 2e-3 * max(1.0, abs(float(want_obj)))
    assert hd.grad.dtype == torch.bfloat16 and Ed.grad.dtype == torch.float32
    assert rel_l2(hd.grad, want_dh) < 2e-2 and rel_l2(Ed.grad, want_de) < 2e-2
