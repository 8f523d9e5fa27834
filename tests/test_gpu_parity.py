"""GPU parity: the CUDA kernels, called through the C ABI (via the ctypes-backed Python
surface), against the CPU oracle on identical seeded inputs.  Cases and tolerances follow
the reference's own kernel tests (tests/test_flash_kernel_tpu.py, test_fused_head_tpu.py,
test_qk_norm_tpu.py) plus the acceptance bar: rel-L2 <= 1e-3 for fp32 I/O, <= 1e-2 for
bf16 I/O, for attention outputs and the per-token NLL."""

import math

import numpy as np
import pytest
import torch

import algebraic_transformer_b200 as A
from algebraic_transformer_b200 import _lib as L
from oracle import algebraic_ref as R

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
IMPLS = ["mma", "auto"]


def rel_l2(a, b):
    a, b = a.detach().double().cpu(), b.detach().double().cpu()
    return float((a - b).norm() / b.norm().clamp_min(1e-30))


def randn(shape, seed, dtype=torch.float32, scale=1.0):
    g = torch.Generator().manual_seed(seed)
    return (torch.randn(shape, generator=g) * scale).to(dtype)


def dev(*ts):
    return [None if t is None else t.to(DEV) for t in ts]


# ------------------------------------------------------------------------------ qk_rms

@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("eps", [1e-5, 1e-3])
@pytest.mark.parametrize("D", [64, 128])
def test_qk_rms_matches_oracle(dtype, eps, D):              # test_qk_norm_tpu.py:21-43
    x = randn((2, 3, 512, D), 181, dtype, 3.0)
    x[0, 0, 0] = 0
    g = torch.Generator().manual_seed(182)
    gain = 0.25 + 4 * torch.rand(D, generator=g)
    want = R.rms_norm(x, gain, eps)
    got = A.qk_rms_norm(*dev(x, gain), eps).cpu()
    tol = 2e-6 if dtype == torch.float32 else 0.01
    np.testing.assert_allclose(got.float(), want.float(), atol=tol, rtol=tol)
    assert torch.all(got[0, 0, 0] == 0)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("D", [64, 128])
def test_qk_rms_with_rotation_and_strided_view(dtype, D):
    B, H, T = 2, 3, 200
    proj = randn((B, T, H * D), 7, dtype)                    # a projection output, (B,T,H*D)
    x = proj.view(B, T, H, D).transpose(1, 2)                # (B,H,T,D) view, not contiguous
    gain = torch.ones(D)
    cos, sin = R.cayley_table_geometric(D, T)
    want = R.apply_rotary(R.rms_norm(x, gain), cos, sin)
    xd = proj.to(DEV).view(B, T, H, D).transpose(1, 2)
    got = A.qk_rms_norm(xd, gain.to(DEV), cos=cos.to(DEV), sin=sin.to(DEV)).cpu()
    assert rel_l2(got, want) < (2e-6 if dtype == torch.float32 else 6e-3)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("D", [64, 128])
def test_qk_rms_backward_matches_oracle_autograd(dtype, D):
    """dx and dgain of the QK RMS-norm (custom VJP of qk_norm.py:29-56: autodiff input gradient, gain
    gradient reduced over row blocks) against autograd through the oracle's rms_norm; a strided view
    of a projection output, a zero row, and the call without a gain."""
    B, H, T = 2, 3, 300
    proj = randn((B, T, H * D), 281, dtype, 2.0)
    proj[0, 7] = 0
    x = proj.view(B, T, H, D).transpose(1, 2)                # (B,H,T,D) view, not contiguous
    dy = randn((B, H, T, D), 282, dtype)
    g = torch.Generator().manual_seed(283)
    gain = 0.25 + 2 * torch.rand(D, generator=g)
    xf, gf = x.float().clone().requires_grad_(True), gain.clone().requires_grad_(True)
    R.rms_norm(xf, gf, 1e-5).backward(dy.float())
    xd = proj.to(DEV).view(B, T, H, D).transpose(1, 2)
    dx, dgain = A.ops.qk_rms_norm_backward(xd, gain.to(DEV), dy.to(DEV), 1e-5)
    assert dx.stride() == xd.stride()
    tol = 2e-5 if dtype == torch.float32 else 1e-2
    assert rel_l2(dx, xf.grad) < tol and rel_l2(dgain, gf.grad) < tol
    assert torch.isfinite(dx).all()
    x2 = x.float().clone().requires_grad_(True)
    R.rms_norm(x2, None, 1e-5).backward(dy.float())
    dx2, none = A.ops.qk_rms_norm_backward(xd, None, dy.to(DEV), 1e-5)
    assert none is None and rel_l2(dx2, x2.grad) < tol
    # the same call twice gives the same bits (partials are added in block order)
    dx3, dgain3 = A.ops.qk_rms_norm_backward(xd, gain.to(DEV), dy.to(DEV), 1e-5)
    assert torch.equal(dgain, dgain3) and torch.equal(dx, dx3)


def test_qk_rms_golden(golden):
    x, gain = torch.from_numpy(golden["rms_x"]), torch.from_numpy(golden["rms_gain"])
    got = A.qk_rms_norm(*dev(x, gain), 1e-5).cpu()
    np.testing.assert_allclose(got, golden["rms_y_eps1e-5"], rtol=2e-6, atol=2e-6)
    xr = torch.from_numpy(golden["rot_x"])
    cos, sin = A.cayley_table_geometric(64, 300, device=DEV)
    rot = A.qk_rms_norm(xr.to(DEV), None, cos=cos, sin=sin).cpu()
    want = R.apply_rotary(R.rms_norm(xr, None), *R.cayley_table_geometric(64, 300))
    np.testing.assert_allclose(rot, want, rtol=1e-5, atol=1e-5)


# --------------------------------------------------------------------------- attention

def run_attn(q, k, v, sink, **kw):
    qd, kd, vd, sd = dev(q, k, v, sink)
    return A.flash_attention(qd, kd, vd, sd, kind="asinh", **kw).cpu()


CASES = [(16, 16.0, True, True), (16, 16.0, True, False), (16, 16.0, False, False),
         (8, 1.0, True, True), (32, 8.0, False, True)]


@pytest.mark.parametrize("n,c,with_sink,shift", CASES)
@pytest.mark.parametrize("impl", IMPLS)
def test_flash_matches_dense_fp32(n, c, with_sink, shift, impl):   # test_flash_kernel_tpu.py:36-70
    B, H, T, D = 2, 3, 512, 64
    q, k, v = randn((B, H, T, D), 1, scale=1.5), randn((B, H, T, D), 2, scale=1.5), randn((B, H, T, D), 3)
    sink = randn((H,), 4, scale=0.5) if with_sink else None
    want = R.asinh_attention(q, k, v, n=n, c=c, sink_logit=sink)
    got = run_attn(q, k, v, sink, n=n, c=c, block=128, shift=shift, impl=impl)
    np.testing.assert_allclose(got, want, atol=2e-3, rtol=2e-3)
    assert rel_l2(got, want) < 1e-3


@pytest.mark.parametrize("mode", ["noshift", "guarded"])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("D", [64, 128])
@pytest.mark.parametrize("impl", IMPLS)
def test_model_attention_statistics(mode, dtype, D, impl):          # test_flash_kernel_tpu.py:73-101
    shape = (1, 2, 512, D)
    q, k, v = (randn(shape, 13 + i, dtype) for i in range(3))
    sink = randn((2,), 17)
    want = R.asinh_attention(q, k, v, n=16, c=8.0, sink_logit=sink)
    qd, kd, vd, sd = dev(q, k, v, sink)
    got, stat, kind = A.flash_attention(qd, kd, vd, sd, kind="asinh", n=16, c=8.0, shift=False,
                                        range_guard=mode == "guarded", return_stat=True, impl=impl)
    np.testing.assert_allclose(got.cpu().float(), want.float(), atol=0.012, rtol=0.012)
    assert rel_l2(got, want) < (1e-3 if dtype == torch.float32 else 1e-2)
    assert int(kind) == 1                                           # unshifted statistic 1/l
    want_stat = R.attention_row_stat(q, k, n=16, c=8.0, sink_logit=sink, shifted=False)
    assert rel_l2(stat, want_stat) < 2e-3


@pytest.mark.parametrize("sign", [-1.0, 1.0])
@pytest.mark.parametrize("with_sink", [False, True])
@pytest.mark.parametrize("magnitude", [1000.0, 1e7])
@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_guarded_attention_tail(sign, with_sink, magnitude, dtype):  # test_flash_kernel_tpu.py:104-123
    shape = (1, 1, 256, 64)
    q = torch.full(shape, math.sqrt(magnitude)).to(dtype)
    k = q * sign
    v = randn(shape, 29, dtype)
    sink = torch.zeros(1) if with_sink else None
    want = R.asinh_attention(q, k, v, n=16, c=8.0, sink_logit=sink)
    qd, kd, vd, sd = dev(q, k, v, sink)
    got, stat, kind = A.flash_attention(qd, kd, vd, sd, kind="asinh", n=16, c=8.0, block=128,
                                        range_guard=True, return_stat=True)
    assert int(kind) == 2                                           # the guard failed: shifted path
    assert torch.isfinite(got).all() and torch.isfinite(stat).all()
    tol = 2e-3 if dtype == torch.float32 else 0.012
    np.testing.assert_allclose(got.cpu().float(), want.float(), atol=tol, rtol=tol)
    want_stat = R.attention_row_stat(q, k, n=16, c=8.0, sink_logit=sink, shifted=True)
    assert rel_l2(stat, want_stat) < 5e-3


def test_guarded_call_replays_from_a_cuda_graph():
    """A stand-alone guarded call only enqueues kernels and a 16-byte memset on the caller's stream, so
    it can be captured into a CUDA graph; replays on fresh inputs — in range, then out of range —
    give the eager results."""
    shape = (1, 2, 512, 64)
    q, k, v = (randn(shape, 871 + i, torch.bfloat16) for i in range(3))
    qd, kd, vd = dev(q, k, v)
    sink = torch.zeros(2, device=DEV)
    out = torch.empty_like(qd)
    A.flash_attention(qd, kd, vd, sink, kind="asinh", n=16, c=8.0, range_guard=True, out=out)   # eager, warms up
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        A.flash_attention(qd, kd, vd, sink, kind="asinh", n=16, c=8.0, range_guard=True, out=out)
    out.zero_()
    graph.replay()
    torch.cuda.synchronize()
    want = R.asinh_attention(q, k, v, n=16, c=8.0, sink_logit=torch.zeros(2))
    assert rel_l2(out, want) < 1e-2
    big = (q.float() * 40).bfloat16()                      # the same graph, inputs that fail the guard
    qd.copy_(big.to(DEV))
    graph.replay()
    torch.cuda.synchronize()
    want2 = R.asinh_attention(big, k, v, n=16, c=8.0, sink_logit=torch.zeros(2))
    assert torch.isfinite(out).all() and rel_l2(out, want2) < 1e-2


@pytest.mark.parametrize("which", ["q", "k", "v"])
@pytest.mark.parametrize("row", [3, 700, 1023])
@pytest.mark.parametrize("D", [64, 128])
def test_guard_sees_one_bad_row_anywhere(which, row, D):
    """A single out-of-range row of q, k or v anywhere in the tensors must send the whole call
    down the shifted path (the guard's maxima cover every row of every head)."""
    shape = (1, 3, 1024, D)
    q, k, v = (randn(shape, 881 + i, torch.bfloat16) for i in range(3))
    if which == "v":
        v[0, 1, row, 5] = 1e9                      # above the guard's bound on |v| (1e8)
    else:
        (q if which == "q" else k)[0, 2, row] = 300.0
    want = R.asinh_attention(q, k, v, n=16, c=8.0)
    qd, kd, vd = dev(q, k, v)
    got, stat, kind = A.flash_attention(qd, kd, vd, None, kind="asinh", n=16, c=8.0, range_guard=True,
                                        return_stat=True)
    assert int(kind) == 2
    assert torch.isfinite(got).all() and torch.isfinite(stat).all()
    assert rel_l2(got, want) < 1e-2
    # and the same tensors without the bad row stay on the unshifted path
    q2, k2, v2 = (randn(shape, 881 + i, torch.bfloat16) for i in range(3))
    _, _, kind2 = A.flash_attention(*dev(q2, k2, v2), None, kind="asinh", n=16, c=8.0, range_guard=True,
                                    return_stat=True)
    assert int(kind2) == 1


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("seq", [512, 2048])
@pytest.mark.parametrize("impl", IMPLS)
def test_nearly_constant_negative_scores_without_sink(dtype, seq, impl):   # test_flash_kernel_tpu.py:181-233
    shape = (1, 2, seq, 64)
    q, k, v = (randn(shape, 439 + i) for i in range(3))
    q = (1 + 0.05 * q).to(dtype)
    k = (-1 + 0.05 * k).to(dtype)
    v = v.to(dtype)
    want = R.asinh_attention(q, k, v, n=16, c=8.0)
    got = run_attn(q, k, v, None, n=16, c=8.0, range_guard=True, impl=impl)
    tol = 0.002 if dtype == torch.float32 else 0.015
    np.testing.assert_allclose(got.float(), want.float(), atol=tol, rtol=tol)


@pytest.mark.parametrize("mode", ["sink", "no_sink", "negative", "gain_two", "positive_tail", "negative_tail"])
def test_model_shape_bf16_2048(mode):                                # test_flash_kernel_tpu.py:258-334
    shape = (1, 2, 2048, 64)
    q, k, v = (randn(shape, 563 + i, torch.bfloat16) for i in range(3))
    sink = torch.tensor([-0.35, 0.125])
    if mode in ("no_sink", "negative"):
        sink = None
    if mode == "negative":
        q = (1 + 0.05 * q.float()).bfloat16()
        k = (-1 + 0.05 * k.float()).bfloat16()
    if mode == "gain_two":
        q, k = 2 * R.rms_norm(q, None), 2 * R.rms_norm(k, None)
    if mode.endswith("tail"):
        q = torch.full(shape, math.sqrt(1000.0)).bfloat16()
        k = q if mode == "positive_tail" else -q
    want = R.asinh_attention(q, k, v, n=16, c=8.0, sink_logit=sink)
    got = run_attn(q, k, v, sink, n=16, c=8.0, range_guard=True)
    np.testing.assert_allclose(got.float(), want.float(), atol=0.015, rtol=0.015)
    assert rel_l2(got, want) < 1e-2


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("D", [64, 128])
@pytest.mark.parametrize("impl", IMPLS)
def test_fused_qk_prologue_layer(dtype, D, impl):
    """QK-norm + Cayley rotation + attention in one call == the three reference steps."""
    B, H, T = 2, 3, 384
    q, k, v = (randn((B, H, T, D), 40 + i, dtype) for i in range(3))
    g = torch.Generator().manual_seed(44)
    qg, kg = 0.5 + torch.rand(D, generator=g), 0.5 + torch.rand(D, generator=g)
    sink = randn((H,), 45, scale=0.02)
    cos, sin = R.cayley_table_geometric(D, T)
    qn = R.apply_rotary(R.rms_norm(q, qg), cos, sin)
    kn = R.apply_rotary(R.rms_norm(k, kg), cos, sin)
    want = R.asinh_attention(qn, kn, v, n=16, c=8.0, sink_logit=sink)
    qd, kd, vd, sd, qgd, kgd, cd, sn = dev(q, k, v, sink, qg, kg, cos, sin)
    got = A.flash_attention(qd, kd, vd, sd, kind="asinh", n=16, c=8.0, block=128, range_guard=True,
                            q_gain=qgd, k_gain=kgd, cos=cd, sin=sn, impl=impl)
    assert rel_l2(got, want) < (1e-3 if dtype == torch.float32 else 1e-2)


def test_config1_single_layer_fp32():
    """benchmark configuration 1: (4,12,1024,64) fp32 causal, unit gains, Cayley over 0..1023,
    n=16, c=8, sink ~ N(0, 0.02)."""
    B, H, T, D = 4, 12, 1024, 64
    q, k, v = (randn((B, H, T, D), i) for i in range(3))
    sink = randn((H,), 1, scale=0.02)
    gain = torch.ones(D)
    cos, sin = R.cayley_table_geometric(D, T)
    qn = R.apply_rotary(R.rms_norm(q, gain), cos, sin)
    kn = R.apply_rotary(R.rms_norm(k, gain), cos, sin)
    want = R.asinh_attention(qn, kn, v, n=16, c=8.0, sink_logit=sink, row_block=256)
    qd, kd, vd, sd, gd, cd, sn = dev(q, k, v, sink, gain, cos, sin)
    got = A.flash_attention(qd, kd, vd, sd, kind="asinh", n=16, c=8.0, range_guard=True,
                            q_gain=gd, k_gain=gd, cos=cd, sin=sn)
    assert got.shape == (B, H, T, D)
    assert rel_l2(got, want) < 1e-3


@pytest.mark.parametrize("impl", IMPLS)
def test_config5_long_context_sampled(impl):
    """benchmark configuration 5 at T=8192: (1,16,8192,128) bf16.  The oracle checks two heads in
    full (row-blocked); run-to-run determinism is checked on everything."""
    B, H, T, D = 1, 16, 8192, 128
    g = torch.Generator().manual_seed(0)
    q, k, v = (torch.randn((B, H, T, D), generator=g).bfloat16() for _ in range(3))
    qd, kd, vd = dev(q, k, v)
    got = A.flash_attention(qd, kd, vd, torch.zeros(H, device=DEV), kind="asinh", n=16, c=8.0,
                            range_guard=True, impl=impl)
    again = A.flash_attention(qd, kd, vd, torch.zeros(H, device=DEV), kind="asinh", n=16, c=8.0,
                              range_guard=True, impl=impl)
    assert torch.equal(got, again)
    for h in (0, 11):
        want = R.asinh_attention(q[:, h:h + 1], k[:, h:h + 1], v[:, h:h + 1], n=16, c=8.0,
                                 sink_logit=torch.zeros(1), row_block=1024)
        assert rel_l2(got[:, h:h + 1], want) < 1e-2


@pytest.mark.parametrize("D,T", [(64, 512), (128, 1024), (128, 2304)])
@pytest.mark.parametrize("n,c", [(16, 8.0), (8, 1.0), (32, 8.0)])
@pytest.mark.parametrize("case", ["normal", "sink", "big", "all_negative", "late_maximum"])
def test_shifted_form_on_tcgen05(D, T, n, c, case):
    """The max-shifted accumulation (flash.py:235-259) on the tcgen05 kernel, forced with shift=True and
    impl="tcgen05": ordinary scores with and without a sink, scores of the order of 1e3 (far outside the
    guard), rows whose scores are all far below zero (no sink: the first tile sets the maximum), and rows
    whose maximum arrives in a late key tile, so that the output accumulated in tensor memory has to be
    rescaled.  Output and the saved statistic rho(-m) l^(-1/n) against the oracle."""
    B, H = 1, 2
    q, k, v = (randn((B, H, T, D), 950 + i, torch.bfloat16) for i in range(3))
    sink = None
    if case == "sink":
        sink = randn((H,), 955, scale=0.5)
    elif case == "big":
        q = (q.float() * 30).bfloat16()
        k = (k.float() * 30).bfloat16()
    elif case == "all_negative":
        q = (1 + 0.05 * q.float()).bfloat16() * 6
        k = ((-1 + 0.05 * k.float()) * 6).bfloat16()
    elif case == "late_maximum":
        k[:, :, T - 200] = (q[:, :, T - 100].float() * 4).bfloat16()     # one key that most late rows score highest on
        k[:, :, 700 % T] = (q[:, :, T - 50].float() * 2).bfloat16()
    want = R.asinh_attention(q, k, v, n=n, c=c, sink_logit=sink)
    qd, kd, vd, sd = dev(q, k, v, sink)
    got, stat, kind = A.flash_attention(qd, kd, vd, sd, kind="asinh", n=n, c=c, block=256, shift=True, impl="tcgen05",
                                        return_stat=True)
    assert int(kind) == 2
    assert torch.isfinite(got).all() and torch.isfinite(stat).all()
    assert rel_l2(got, want) < 1e-2
    want_stat = R.attention_row_stat(q, k, n=n, c=c, sink_logit=sink, shifted=True)
    assert rel_l2(stat, want_stat) < 5e-3
    again = A.flash_attention(qd, kd, vd, sd, kind="asinh", n=n, c=c, block=256, shift=True, impl="tcgen05")
    assert torch.equal(got, again)


@pytest.mark.parametrize("T", [256, 1024, 1280])
@pytest.mark.parametrize("n,c", [(16, 8.0), (8, 1.0), (32, 8.0)])
@pytest.mark.parametrize("case", ["plain", "sink", "guard_holds", "guard_fails", "strided"])
def test_fp32_rows_on_tcgen05(T, n, c, case):
    """fp32 q, k, v of head_dim 64 on the tcgen05 kernel (impl="tcgen05" is an error where that kernel does
    not apply): rows split into bf16 hi | lo halves, every product as hi.hi + hi.lo + lo.hi.  The fp32 bar of
    1e-3 (plain bf16 operands miss it) against the oracle, for the unshifted form with and without a sink,
    under the guard when it holds (unshifted statistic) and when it fails (the max-shifted mma.sync kernel
    takes over: statistic of the shifted kind), and on strided (B, T, H, D) views."""
    B, H, D = 2, 3, 64
    q, k, v = (randn((B, H, T, D), 970 + i) for i in range(3))
    sink = randn((H,), 975, scale=0.5) if case in ("sink", "guard_holds") else None
    # bounded_scores is the reference's internal flag of the guard's in-range branch: the unshifted
    # kernel without a guard pass and without the score clamp of the public unguarded link
    kw = dict(shift=False, bounded_scores=True)
    if case in ("guard_holds", "guard_fails"):
        kw = dict(range_guard=True)
    if case == "guard_fails":
        q = q * 40
        k = k * 40
    want = R.asinh_attention(q, k, v, n=n, c=c, sink_logit=sink)
    if case == "strided":
        qd, kd, vd = (t.transpose(1, 2).contiguous().to(DEV).transpose(1, 2) for t in (q, k, v))
        sd = None
    else:
        qd, kd, vd, sd = dev(q, k, v, sink)
    got, stat, kind = A.flash_attention(qd, kd, vd, sd, kind="asinh", n=n, c=c, block=256, impl="tcgen05", return_stat=True, **kw)
    assert got.dtype == torch.float32 and torch.isfinite(got).all()
    assert rel_l2(got, want) < 1e-3
    shifted = case == "guard_fails"
    assert int(kind) == (2 if shifted else 1)
    want_stat = R.attention_row_stat(q, k, n=n, c=c, sink_logit=sink, shifted=shifted)
    assert rel_l2(stat, want_stat) < 1e-3
    # the mma.sync kernel on the same inputs: two independent paths to the same fp32 result
    other = A.flash_attention(qd, kd, vd, sd, kind="asinh", n=n, c=c, block=256, impl="mma", **kw)
    assert rel_l2(got, other) < 1e-3
    again = A.flash_attention(qd, kd, vd, sd, kind="asinh", n=n, c=c, block=256, impl="tcgen05", **kw)
    assert torch.equal(got, again)


@pytest.mark.parametrize("T", [1, 100, 128, 257, 384, 1000, 1500])
@pytest.mark.parametrize("D,dtype", [(64, torch.bfloat16), (128, torch.bfloat16), (64, torch.float32)])
@pytest.mark.parametrize("mode", ["guarded", "shift"])
def test_any_sequence_length_on_tcgen05(T, D, dtype, mode):
    """Causal self-attention over lengths that do not fill the last 256-row block (impl="tcgen05" is an error
    where that kernel does not apply): rows and keys past the end are TMA zero fill, masked by causality and
    never stored.  Output and statistic against the oracle; the memory just behind the output stays untouched."""
    if dtype == torch.float32 and mode == "shift":
        pytest.skip("fp32 rows run the max-shifted form on the mma.sync kernel")
    B, H = 2, 3
    q, k, v = (randn((B, H, T, D), 990 + i, dtype) for i in range(3))
    sink = randn((H,), 995, scale=0.5)
    want = R.asinh_attention(q, k, v, n=16, c=8.0, sink_logit=sink)
    qd, kd, vd, sd = dev(q, k, v, sink)
    # the output is a view into a larger buffer pre-filled with a sentinel: a store past row T would show
    buf = torch.full((B, H, T + 8, D), 7.0, dtype=dtype, device=DEV)
    out = buf[:, :, :T]
    kw = dict(range_guard=True) if mode == "guarded" else dict(shift=True)
    got, stat, kind = A.flash_attention(qd, kd, vd, sd, kind="asinh", n=16, c=8.0, block=T, impl="tcgen05", return_stat=True,
                                        out=out, **kw)
    assert int(kind) == (1 if mode == "guarded" else 2)
    assert torch.isfinite(got).all() and torch.isfinite(stat).all()
    assert rel_l2(got, want) < (1e-3 if dtype == torch.float32 else 1e-2)
    assert bool((buf[:, :, T:] == 7.0).all())
    want_stat = R.attention_row_stat(q, k, n=16, c=8.0, sink_logit=sink, shifted=mode == "shift")
    assert rel_l2(stat, want_stat) < 5e-3


@pytest.mark.parametrize("B,H,T,D,splits", [(1, 2, 2048, 128, False), (1, 1, 4096, 64, True), (1, 3, 3900, 128, True),
                                             (2, 2, 4096, 64, True), (1, 2, 8192, 128, True)])
@pytest.mark.parametrize("with_sink", [False, True])
def test_short_problems_split_along_the_keys(B, H, T, D, splits, with_sink):
    """Few long items for 148 SMs: the long items are cut along the keys into parts of at least 16 key-tile steps whose
    raw accumulators and row sums a second kernel adds up (the sink's weight counted once); sequences up to 2048 are
    never split.  Output and statistic against the oracle (sampled rows at 8192), bit-equal repeats, and bit-equal to
    the guarded call on the same inputs."""
    q, k, v = (randn((B, H, T, D), 930 + i, torch.bfloat16) for i in range(3))
    sink = randn((H,), 935, scale=0.5) if with_sink else None
    qd, kd, vd, sd = dev(q, k, v, sink)
    lib = L.load()
    before = lib.alg_kernel_launches()
    got, stat, kind = A.flash_attention(qd, kd, vd, sd, kind="asinh", n=16, c=8.0, block=T, shift=False, bounded_scores=True,
                                        impl="tcgen05", return_stat=True)
    assert lib.alg_kernel_launches() - before == (2 if splits else 1)   # the attention kernel and, if it split, the combine kernel
    assert int(kind) == 1
    rows = slice(None) if T <= 4096 else slice(T - 300, T)
    if T <= 4096:
        want = R.asinh_attention(q, k, v, n=16, c=8.0, sink_logit=sink)
        want_stat = R.attention_row_stat(q, k, n=16, c=8.0, sink_logit=sink, shifted=False)
    else:                                                    # the last 300 rows of the square problem
        want = R.asinh_attention(q[:, :, T - 300:], k, v, n=16, c=8.0, sink_logit=sink)
        want_stat = R.attention_row_stat(q[:, :, T - 300:], k, n=16, c=8.0, sink_logit=sink, shifted=False)
    assert torch.isfinite(got).all() and torch.isfinite(stat).all()
    assert rel_l2(got[:, :, rows], want) < 1e-2
    assert rel_l2(stat[:, :, rows], want_stat) < 5e-3
    again = A.flash_attention(qd, kd, vd, sd, kind="asinh", n=16, c=8.0, block=T, shift=False, bounded_scores=True, impl="tcgen05")
    assert torch.equal(got, again)
    # the guarded call on the same inputs (statistics inside the kernel or a pass in front, stand-by launch behind)
    guarded = A.flash_attention(qd, kd, vd, sd, kind="asinh", n=16, c=8.0, block=T, range_guard=True, impl="tcgen05")
    assert torch.equal(got, guarded)


@pytest.mark.parametrize("T", [16384, 32768])
def test_config5_longer_sequences_sampled(T):
    """benchmark configuration 5 at T = 16384 and 32768: (1,16,T,128) bf16 through the guarded public
    call.  The dense (T,T) oracle does not fit, so it is evaluated on a deterministic sample of 256-row
    blocks (the first, one in mid-sequence, the last: rows r0:r1 of the square problem are the causal
    problem of q[r0:r1] against the first r1 keys) of two heads; all heads are checked for run-to-run
    bit equality, which also exercises the kernel's ring and phase arithmetic at 64 to 128 key tiles
    per item."""
    B, H, D = 1, 16, 128
    g = torch.Generator().manual_seed(0)
    q, k, v = (torch.randn((B, H, T, D), generator=g).bfloat16() for _ in range(3))
    qd, kd, vd = dev(q, k, v)
    sink = torch.zeros(H, device=DEV)
    got, stat, kind = A.flash_attention(qd, kd, vd, sink, kind="asinh", n=16, c=8.0, range_guard=True, return_stat=True)
    again = A.flash_attention(qd, kd, vd, sink, kind="asinh", n=16, c=8.0, range_guard=True)
    assert int(kind) == 1 and torch.equal(got, again)
    assert torch.isfinite(got).all() and torch.isfinite(stat).all()
    for h in (3, 15):
        for r0 in (0, (T // 2 // 256) * 256 + 256, T - 256):
            r1 = r0 + 256
            want = R.asinh_attention(q[:, h:h + 1, r0:r1], k[:, h:h + 1, :r1], v[:, h:h + 1, :r1], n=16, c=8.0,
                                     sink_logit=torch.zeros(1))
            assert rel_l2(got[:, h:h + 1, r0:r1], want) < 1e-2, (h, r0)
            want_stat = R.attention_row_stat(q[:, h:h + 1, r0:r1], k[:, h:h + 1, :r1], n=16, c=8.0,
                                             sink_logit=torch.zeros(1), shifted=False)
            assert rel_l2(stat[:, h:h + 1, r0:r1], want_stat) < 2e-3, (h, r0)


@pytest.mark.parametrize("which", ["none", "q", "k", "v", "v_nan"])
def test_guard_inside_the_attention_kernel(which):
    """From T * head_dim = 3/4 Mi on, a guarded stand-alone call takes the guard's maxima of q, k, v
    with one warp of the attention kernel itself instead of a pass of its own.  In range the result is
    the unshifted kernel's; one out-of-range row anywhere (here in the last head, far from row 0) must
    still send the whole call down the shifted path."""
    B, H, T, D = 1, 2, 6144, 128
    q, k, v = (randn((B, H, T, D), 901 + i, torch.bfloat16) for i in range(3))
    if which == "q":
        q[0, 1, 5000] = 300.0
    elif which == "k":
        k[0, 1, 4097] = 300.0
    elif which == "v":
        v[0, 1, 6143, 77] = 1e9
    elif which == "v_nan":
        v[0, 0, 3000, 1] = float("nan")
    qd, kd, vd = dev(q, k, v)
    got, stat, kind = A.flash_attention(qd, kd, vd, None, kind="asinh", n=16, c=8.0, range_guard=True, return_stat=True)
    assert int(kind) == (1 if which == "none" else 2)
    if which == "v_nan":
        return                                         # the output carries the NaN either way
    assert torch.isfinite(got).all() and torch.isfinite(stat).all()
    for h, r0 in ((0, 0), (1, 4864), (1, T - 256)):
        r1 = r0 + 256
        want = R.asinh_attention(q[:, h:h + 1, r0:r1], k[:, h:h + 1, :r1], v[:, h:h + 1, :r1], n=16, c=8.0)
        assert rel_l2(got[:, h:h + 1, r0:r1], want) < 1e-2, (h, r0)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_ragged_lengths_cross_and_noncausal(dtype):
    """Shapes off the tile grid, Tq != Tk (bottom-right aligned causal), and no mask."""
    q, k, v = randn((1, 2, 77, 64), 1, dtype), randn((1, 2, 200, 64), 2, dtype), randn((1, 2, 200, 64), 3, dtype)
    sink = torch.tensor([0.2, -0.1])
    tol = 1e-3 if dtype == torch.float32 else 1e-2
    qd, kd, vd, sd = dev(q, k, v, sink)
    got = A.flash_attention(qd, kd, vd, sd, kind="asinh", n=16, c=8.0, block=77, causal=False, range_guard=True)
    want = R.asinh_attention(q, k, v, n=16, c=8.0, sink_logit=sink, causal=False)
    assert rel_l2(got, want) < tol
    # causal with Tk > Tq == the last Tq rows of the square problem
    qq = randn((1, 2, 200, 64), 5, dtype)
    full = R.asinh_attention(qq, k, v, n=16, c=8.0, sink_logit=sink)
    qd2 = qq[:, :, 123:].contiguous().to(DEV)
    got2 = A.flash_attention(qd2, kd, vd, sd, kind="asinh", n=16, c=8.0, block=77, range_guard=True)
    assert rel_l2(got2, full[:, :, 123:]) < tol
    # empty batch is a no-op
    e = torch.empty((0, 2, 64, 64), dtype=dtype, device=DEV)
    assert A.flash_attention(e, e, e, kind="asinh", n=16, c=8.0).shape == (0, 2, 64, 64)


def test_attention_golden_vectors(golden):
    g = golden
    q, k, v, sink = (torch.from_numpy(g[x]) for x in ("att_q", "att_k", "att_v", "att_sink"))
    cases = {"att_o_n16_c16_sink": (16, 16.0, sink), "att_o_n16_c8_sink": (16, 8.0, sink),
             "att_o_n16_c8_nosink": (16, 8.0, None), "att_o_n8_c1_sink": (8, 1.0, sink),
             "att_o_n32_c8_nosink": (32, 8.0, None)}
    for key, (n, c, s) in cases.items():
        s1 = None if s is None else s.reshape(-1)
        got = run_attn(q, k, v, s1, n=n, c=c, block=80, range_guard=True)
        assert rel_l2(got, torch.from_numpy(g[key])) < 1e-3, key
    for D in (64, 128):
        q0, k0, v0 = (torch.from_numpy(g[f"layer_D{D}_{x}"]) for x in "qkv")
        T = q0.shape[2]
        cos, sin = A.cayley_table_geometric(D, T, device=DEV)
        ones = torch.ones(D, device=DEV)
        got = A.flash_attention(*dev(q0, k0, v0), torch.from_numpy(g[f"layer_D{D}_sink"]).reshape(-1).to(DEV),
                                kind="asinh", n=16, c=8.0, block=T, range_guard=True, q_gain=ones, k_gain=ones,
                                cos=cos, sin=sin)
        assert rel_l2(got, torch.from_numpy(g[f"layer_D{D}_o"])) < 1e-3
    qt, vt = torch.from_numpy(g["tail_q"]), torch.from_numpy(g["tail_v"])
    for sign in (1.0, -1.0):
        for ws in (0, 1):
            sk = torch.zeros(1) if ws else None
            got = run_attn(qt, qt * sign, vt, sk, n=16, c=8.0, block=64, range_guard=True)
            np.testing.assert_allclose(got, g[f"tail_o_sign{sign}_sink{ws}"], atol=2e-3, rtol=2e-3)


def test_causality_on_device():                                      # test_e2e_acceptance.py:563-594
    q, k, v = (randn((1, 2, 256, 64), 5 + i, torch.bfloat16) for i in range(3))
    k2, v2 = k.clone(), v.clone()
    k2[:, :, 130:] += 5.0
    v2[:, :, 130:] -= 3.0
    a = run_attn(q, k, v, None, n=16, c=8.0, range_guard=True)
    b = run_attn(q, k2, v2, None, n=16, c=8.0, range_guard=True)
    assert torch.equal(a[:, :, :130], b[:, :, :130])


@pytest.mark.parametrize("D,Tk", [(128, 32768), (64, 1000)])
def test_decode_single_query(D, Tk):
    """Config 5's decode: one query against a Tk-token KV cache, all keys visible."""
    B, H = 1, 16
    q, k, v = randn((B, H, 1, D), 1, torch.bfloat16), randn((B, H, Tk, D), 2, torch.bfloat16), \
        randn((B, H, Tk, D), 3, torch.bfloat16)
    sink = randn((H,), 4, scale=0.5)
    want = R.asinh_attention(q, k, v, n=16, c=8.0, sink_logit=sink, causal=False)
    got = A.decode_attention(*dev(q, k, v, sink), n=16, c=8.0).cpu()
    assert rel_l2(got, want) < 1e-2
    got2 = A.decode_attention(*dev(q, k, v), None, n=16, c=8.0).cpu()
    want2 = R.asinh_attention(q, k, v, n=16, c=8.0, causal=False)
    assert rel_l2(got2, want2) < 1e-2


@pytest.mark.parametrize("B,H,D,Tk", [(2, 4, 128, 4096), (1, 3, 64, 700), (3, 16, 64, 64)])
def test_decode_is_one_launch_and_repeats(B, H, D, Tk):
    """The split that arrives last merges its (batch, head): the arrival words live in the workspace, are never
    zeroed by the host, and must come out right on the first call (whatever the workspace held), on repeated
    calls, and when one captured launch is replayed (same call number every time)."""
    q, k, v = randn((B, H, 1, D), 11, torch.bfloat16), randn((B, H, Tk, D), 12, torch.bfloat16), \
        randn((B, H, Tk, D), 13, torch.bfloat16)
    sink = randn((H,), 14, scale=0.5)
    want = R.asinh_attention(q, k, v, n=16, c=8.0, sink_logit=sink, causal=False)
    qd, kd, vd, sd = dev(q, k, v, sink)
    lib = L.load()
    before = lib.alg_kernel_launches()
    first = A.decode_attention(qd, kd, vd, sd, n=16, c=8.0)
    assert lib.alg_kernel_launches() - before == 1
    assert rel_l2(first, want) < 1e-2
    for _ in range(3):
        assert torch.equal(A.decode_attention(qd, kd, vd, sd, n=16, c=8.0), first)
    out = torch.empty_like(first)
    A.decode_attention(qd, kd, vd, sd, n=16, c=8.0, out=out)          # warm: workspace exists before capture
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        A.decode_attention(qd, kd, vd, sd, n=16, c=8.0, out=out)
    for _ in range(3):
        out.zero_()
        graph.replay()
        torch.cuda.synchronize()
        assert torch.equal(out, first)


# -------------------------------------------------------------------------------- head

def head_inputs(N, d, V, escale, seed=0):
    g = torch.Generator().manual_seed(seed)
    h = torch.randn((N, d), generator=g).bfloat16()
    E = torch.randn((V, d), generator=g) * escale
    t = torch.randint(0, V, (N,), generator=g)
    return h, E, t


def check_head(h, E, t, n, c, impl, nll_tol=1e-2, **kw):
    obj_w, pt_w = R.algebraic_likelihood(R.head_logits(h, E), t, n, c)     # the exact form, as the TPU tests use
    obj, pt, nll = A.fused_head(*dev(h, E, t), kind="alg_ce", n=n, c=c, want_nll=True, impl=impl, **kw)
    np.testing.assert_allclose(float(obj), float(obj_w), rtol=2e-3, atol=2e-4)
    np.testing.assert_allclose(pt.cpu(), pt_w, rtol=2e-2, atol=2e-7)
    assert rel_l2(nll, R.nll_from_pt(pt_w)) < nll_tol
    return pt


@pytest.mark.parametrize("n,c", [(16, 16.0), (8, 2.0)])
@pytest.mark.parametrize("V", [32768, 4096])
@pytest.mark.parametrize("impl", IMPLS)
def test_fused_head_matches_dense(n, c, V, impl):                    # test_fused_head_tpu.py:14-43
    h, E, t = head_inputs(1024, 256, V, 0.15)
    check_head(h, E, t, n, c, impl, block_n=256, block_v=1024)


@pytest.mark.parametrize("width", [1024, 1536])
@pytest.mark.parametrize("impl", IMPLS)
def test_production_head_widths(width, impl):                        # test_fused_head_tpu.py:46-70
    h, E, t = head_inputs(256, width, 32768, 0.02, seed=42)
    check_head(h, E, t, 8, 2.0, impl)


@pytest.mark.parametrize("impl", IMPLS)
def test_head_ragged_vocab_rows_and_clamp(impl):
    """V off the 128 grid (padded columns must not leak rho(0)^n = 1), N off the row tile,
    and logits large enough for the clamp to bind."""
    h, E, t = head_inputs(200, 128, 50257 // 8, 0.15, seed=3)
    t[:5] = torch.tensor([0, 1, 6281, 6280, 127])
    check_head(h, E, t, 8, 2.0, impl, block_n=200)
    # logits beyond clamp * c = 7265: the clamped additive form is the semantics here, so
    # the comparison is against the oracle's restatement of the fused kernel
    h2, E2, t2 = head_inputs(128, 64, 1000, 1200.0, seed=4)
    assert float(R.head_logits(h2, E2).max()) > 2 * R.likelihood_clamp(1000, 8)
    obj_w, pt_w = R.fused_head(h2, E2, t2, n=8, c=2.0)
    obj, pt = A.fused_head(*dev(h2, E2, t2), kind="alg_ce", n=8, c=2.0, impl=impl)
    assert torch.isfinite(pt).all()
    np.testing.assert_allclose(pt.cpu(), pt_w, rtol=2e-2, atol=1e-6)
    np.testing.assert_allclose(float(obj), float(obj_w), rtol=2e-3)


@pytest.mark.parametrize("impl", IMPLS)
def test_config2_full_head(impl):
    """benchmark configuration 2: hidden (8192,768) bf16 ~ N(0,1), E (50304,768) ~ N(0,0.02),
    targets uniform in [0, 50257); NLL rel-L2 <= 1e-2."""
    g = torch.Generator().manual_seed(0)
    h = torch.randn((8192, 768), generator=g).bfloat16()
    E = torch.randn((50304, 768), generator=g) * 0.02
    t = torch.randint(0, 50257, (8192,), generator=g)
    obj_w, pt_w = R.fused_head(h, E, t, n=8, c=2.0, row_block=1024)
    obj, pt, nll = A.fused_head(*dev(h, E, t), kind="alg_ce", n=8, c=2.0, want_nll=True, impl=impl)
    assert rel_l2(nll, R.nll_from_pt(pt_w)) < 1e-2
    np.testing.assert_allclose(float(obj), float(obj_w), rtol=2e-3)
    obj2, pt2 = A.fused_head(*dev(h, E, t), kind="alg_ce", n=8, c=2.0, impl=impl)
    assert torch.equal(pt, pt2)                                       # run-to-run identical


@pytest.mark.parametrize("world", [2, 8])
@pytest.mark.parametrize("impl", IMPLS)
def test_head_vocab_shards_sum_to_whole(world, impl):
    """Linearity over vocabulary shards: partials of the 128-column-tile shards add up to
    the unsharded statistic (what the all-reduce computes), uneven 49/50-tile split included."""
    h, E, t = head_inputs(512, 256, 50304 // 4, 0.1, seed=9)
    V = E.shape[0]
    hd, td = h.to(DEV), t.to(torch.int32).to(DEV)
    eb = A.cast_embedding(E.to(DEV))
    whole = A.head_statistic(hd, eb, td, n=8, c=2.0, impl=impl).clone()
    total = torch.zeros_like(whole)
    for r in range(world):
        lo, cnt = A.vocab_shard(V, r, world)
        total += A.head_statistic(hd, eb[lo:lo + cnt], td, n=8, c=2.0, vocab_offset=lo, vocab_total=V, impl=impl)
    assert rel_l2(total[0], whole[0]) < 1e-5
    np.testing.assert_allclose(total[1].cpu(), whole[1].cpu(), rtol=1e-5, atol=1e-5)
    obj, pt = A.head_finalize(total, n=8, c=2.0, vocab_total=V)
    _, pt_w = R.fused_head(h, E, t, n=8, c=2.0)
    np.testing.assert_allclose(pt.cpu(), pt_w, rtol=2e-2, atol=2e-7)


def test_embedding_cast_kernel():
    E = randn((1000, 72), 1, scale=0.02)
    got = A.cast_embedding(E.to(DEV)).cpu()
    assert torch.equal(got, E.bfloat16())


# ------------------------------------------------------------------------ attention backward

def _oracle_grads(q, k, v, sink, d_o, causal=True):
    """Autograd through the CPU oracle (fp32 math on the bf16-rounded inputs)."""
    qf, kf, vf = (t.float().requires_grad_(True) for t in (q, k, v))
    sf = None if sink is None else sink.clone().float().requires_grad_(True)
    out = R.asinh_attention(qf, kf, vf, n=16, c=8.0, sink_logit=sf, causal=causal)
    out.backward(d_o.float())
    return qf.grad, kf.grad, vf.grad, None if sf is None else sf.grad


@pytest.mark.parametrize("shape,with_sink,causal", [((2, 3, 256, 64), True, True), ((1, 2, 512, 128), True, True),
                                                   ((1, 2, 200, 64), False, True), ((1, 2, 192, 64), True, False),
                                                   ((1, 2, 1152, 128), True, True), ((1, 1, 1152, 64), True, True)])
@pytest.mark.parametrize("impl", ["auto", "mma"])
def test_attention_backward_matches_oracle_autograd(shape, with_sink, causal, impl):
    """dq, dk, dv, dsink from the saved statistic (custom VJP of flash.py:333-727) against autograd
    through the CPU oracle; ragged length 200 exercises the masked tails, 192 the non-causal form,
    1152 = 9 tiles of 128 wraps the tcgen05 kernels' tile ring several times.  "auto" takes the
    tcgen05 kernels on the causal multiples of 128 and the mma.sync kernels elsewhere."""
    q, k, v, d_o = (randn(shape, 900 + i, torch.bfloat16) for i in range(4))
    sink = randn((shape[1],), 905) * 0.5 if with_sink else None
    qd, kd, vd, dod, sd = dev(q, k, v, d_o, sink)
    o, stat, kind = A.flash_attention(qd, kd, vd, sd, kind="asinh", n=16, c=8.0, block=shape[2], range_guard=True,
                                      causal=causal, return_stat=True)
    dq, dk, dv, ds = A.ops.flash_attention_backward(qd, kd, vd, o, dod, stat, kind, sd, n=16, c=8.0, causal=causal,
                                                    impl=impl)
    wq, wk, wv, ws = _oracle_grads(q, k, v, sink, d_o, causal)
    assert rel_l2(dq, wq) < 2e-2 and rel_l2(dk, wk) < 2e-2 and rel_l2(dv, wv) < 2e-2
    if with_sink:
        assert rel_l2(ds, ws) < 2e-2


@pytest.mark.parametrize("V", [32768, 4096, 6280])
def test_fused_head_ce_kind_matches_dense(V):                        # test_fused_head_tpu.py:14-43, kind "ce"
    """The softmax cross-entropy kind: objective, per-token nll and both gradients against the dense
    definition (standard.py:41-47) with the reference test's tolerances; 6280 is off the 256-column
    tile grid (zero-filled columns must not add exp(0)); then a logit of 3e4 (the running maximum
    must absorb it) and the statistic combined over two vocabulary shards by logsumexp."""
    N, d = 1024, 256
    h, E, t = head_inputs(N, d, V, 0.15)
    hf, ef = h.float().requires_grad_(True), E.bfloat16().float().requires_grad_(True)
    want_obj, want_nll = R.cross_entropy(hf @ ef.t(), t)
    want_obj.backward()
    want_obj = want_obj.detach()
    hd, Ed, td = dev(h, E, t)
    obj, nll = A.fused_head(hd, Ed, td, kind="ce", block_n=256, block_v=1024)
    np.testing.assert_allclose(float(obj), float(want_obj), rtol=2e-3, atol=2e-4)
    np.testing.assert_allclose(nll.cpu(), want_nll.detach(), rtol=2e-2, atol=2e-4)
    eb = A.ops.cast_embedding(Ed)
    stats = A.head_statistic(hd, eb, td.int(), kind="ce")
    dh, de = A.ops.fused_head_backward(hd, eb, td, stats, kind="ce")
    for got, want in ((dh, hf.grad), (de, ef.grad)):
        a, b = got.float().cpu().numpy(), want.numpy()
        scale = np.abs(b).max() + 1e-12
        np.testing.assert_allclose(a / scale, b / scale, atol=2e-2)
        assert (a * b).sum() / np.sqrt((a * a).sum() * (b * b).sum()) > 0.999
    # two shards: per-shard logsumexp, combined by logsumexp; target logits add
    lo = (V // 2) // 8 * 8 + 8
    s0 = A.head_statistic(hd, eb[:lo].contiguous(), td.int(), kind="ce", vocab_offset=0, vocab_total=V)
    s1 = A.head_statistic(hd, eb[lo:].contiguous(), td.int(), kind="ce", vocab_offset=lo, vocab_total=V)
    both = torch.stack([torch.logsumexp(torch.stack([s0[0], s1[0]]), dim=0), s0[1] + s1[1]])
    obj2, nll2 = A.ops.head_finalize(both, kind="ce")
    np.testing.assert_allclose(nll2.cpu(), want_nll.detach(), rtol=2e-2, atol=2e-4)
    np.testing.assert_allclose(float(obj2), float(want_obj), rtol=2e-3, atol=2e-4)
    # one very large logit: h row 3 and E row 9 aligned
    h2, E2 = h.clone(), E.clone()
    h2[3], E2[9] = 12.0, 10.0                                         # z[3, 9] = 256 * 120 = 30720
    w_obj, w_nll = R.cross_entropy(R.head_logits(h2, E2), t)
    obj3, nll3 = A.fused_head(*dev(h2, E2, t), kind="ce", block_n=256)
    assert torch.isfinite(nll3).all()
    np.testing.assert_allclose(nll3.cpu(), w_nll, rtol=2e-2, atol=2e-3)
    np.testing.assert_allclose(float(obj3), float(w_obj), rtol=2e-3)


def test_head_backward_matches_reference_vjp():
    """dh and dE of the Alg-CE head as the reference's custom VJP defines them (fused_head.py:120-156,
    194-216, 236-243: the gradient of the mean negative log-likelihood, clamp straight-through)
    against the oracle's restatement of that rule, which is pinned to the reference's own backward
    functions; ragged N and V; a non-unit cotangent; then the same through two vocabulary shards."""
    N, d, V = 300, 128, 1000
    h = randn((N, d), 971).bfloat16()
    E = (randn((V, d), 972) * 0.3).bfloat16()
    g = torch.Generator().manual_seed(973)
    t = torch.randint(0, V, (N,), generator=g)
    want_dh, want_de = R.head_vjp_dense(h, E, t, 8, 2.0)

    class _Grad:                                          # keeps the assertions below readable
        def __init__(self, v):
            self.grad = v
    hf, ef = _Grad(want_dh), _Grad(want_de)
    hd, Ed, td = dev(h, E, t)
    stats = A.head_statistic(hd, Ed, td.int(), n=8, c=2.0)
    dh, de = A.ops.fused_head_backward(hd, Ed, td, stats, n=8, c=2.0)
    assert rel_l2(dh, hf.grad) < 2e-2 and rel_l2(de, ef.grad) < 2e-2
    dh2, de2 = A.ops.fused_head_backward(hd, Ed, td, stats, n=8, c=2.0, upstream=0.5)
    assert rel_l2(dh2, 0.5 * hf.grad) < 2e-2 and rel_l2(de2, 0.5 * ef.grad) < 2e-2
    # a logit far above the clamp (z / c = 57600 against a clamp of 5928): the rule is straight-through,
    # so that entry still contributes r (p - y) n / (c N) to its row of dh and to its row of dE
    hc, Ec, tc = h.clone(), E.clone(), t.clone()
    hc[5], Ec[7] = 30.0, 30.0
    tc[5] = 11
    wc_dh, wc_de = R.head_vjp_dense(hc, Ec, tc, 8, 2.0)
    hcd, Ecd, tcd = dev(hc, Ec, tc)
    sc = A.head_statistic(hcd, Ecd, tcd.int(), n=8, c=2.0)
    dhc, dec = A.ops.fused_head_backward(hcd, Ecd, tcd, sc, n=8, c=2.0)
    assert rel_l2(dhc, wc_dh) < 2e-2 and rel_l2(dec, wc_de) < 2e-2
    assert rel_l2(dhc[5], wc_dh[5]) < 3e-2 and rel_l2(dec[7], wc_de[7]) < 3e-2
    # two shards: the statistic is summed over them, each shard returns its rows of dE and a part of dh
    lo = 504
    s0 = A.head_statistic(hd, Ed[:lo].contiguous(), td.int(), n=8, c=2.0, vocab_offset=0, vocab_total=V)
    s1 = A.head_statistic(hd, Ed[lo:].contiguous(), td.int(), n=8, c=2.0, vocab_offset=lo, vocab_total=V)
    both = s0 + s1
    dh0, de0 = A.ops.fused_head_backward(hd, Ed[:lo].contiguous(), td, both, n=8, c=2.0, vocab_offset=0, vocab_total=V)
    dh1, de1 = A.ops.fused_head_backward(hd, Ed[lo:].contiguous(), td, both, n=8, c=2.0, vocab_offset=lo, vocab_total=V)
    assert rel_l2(dh0.float() + dh1.float(), hf.grad) < 2e-2
    assert rel_l2(torch.cat([de0, de1]), ef.grad) < 2e-2


@pytest.mark.parametrize("impl", ["auto", "mma"])
def test_attention_backward_on_views_of_a_fused_projection(impl):
    """q, k, v as the (B,H,T,D) views of one (B,T,3,H,D) projection output, d_o a view of a
    (B,T,H,D) tensor: strides reach the kernels (tensor maps for the tcgen05 path) unchanged, and the
    gradients come back in the layout of their inputs."""
    B, H, T, D = 2, 2, 384, 64
    qkv = randn((B, T, 3, H, D), 990, torch.bfloat16)
    q, k, v = (qkv[:, :, i].transpose(1, 2) for i in range(3))
    d_o = randn((B, T, H, D), 991, torch.bfloat16).transpose(1, 2)
    sink = randn((H,), 992) * 0.5
    qkvd = qkv.to(DEV)
    qd, kd, vd = (qkvd[:, :, i].transpose(1, 2) for i in range(3))
    dod, sd = d_o.to(DEV), sink.to(DEV)
    assert not qd.is_contiguous()
    o, stat, kind = A.flash_attention(qd, kd, vd, sd, kind="asinh", n=16, c=8.0, range_guard=True, return_stat=True)
    dq, dk, dv, ds = A.ops.flash_attention_backward(qd, kd, vd, o, dod, stat, kind, sd, n=16, c=8.0, impl=impl)
    assert dq.stride() == qd.stride() and dv.stride() == vd.stride()
    wq, wk, wv, ws = _oracle_grads(q.contiguous(), k.contiguous(), v.contiguous(), sink, d_o.contiguous())
    assert rel_l2(dq, wq) < 2e-2 and rel_l2(dk, wk) < 2e-2 and rel_l2(dv, wv) < 2e-2 and rel_l2(ds, ws) < 2e-2


@pytest.mark.parametrize("impl", ["auto", "mma"])
def test_attention_backward_after_shifted_forward(impl):
    """Out-of-range inputs: the forward takes the max-shifted path and saves rho(-m) l^(-1/n); the
    backward must rebuild the same weights from that statistic."""
    shape = (1, 2, 256, 64)
    q, k, v, d_o = (randn(shape, 950 + i, torch.bfloat16) for i in range(4))
    q = (q.float() * 6).bfloat16()
    k = (k.float() * 6).bfloat16()
    qd, kd, vd, dod = dev(q, k, v, d_o)
    o, stat, kind = A.flash_attention(qd, kd, vd, None, kind="asinh", n=16, c=8.0, block=256, range_guard=True,
                                      return_stat=True)
    assert int(kind) == 2
    dq, dk, dv, _ = A.ops.flash_attention_backward(qd, kd, vd, o, dod, stat, kind, None, n=16, c=8.0, impl=impl)
    wq, wk, wv, _ = _oracle_grads(q, k, v, None, d_o)
    assert rel_l2(dq, wq) < 3e-2 and rel_l2(dk, wk) < 3e-2 and rel_l2(dv, wv) < 3e-2
