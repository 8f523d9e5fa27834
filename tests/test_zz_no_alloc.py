"""alg_head_fwd_static — the head entry point for callers that cannot allocate.

Some users of the library are not allowed to obtain device memory at call time: a
custom-call handler under a runtime that owns all buffers, or a server with a frozen
memory plan.  They cannot give alg_head_fwd its workspace, so alg_head_fwd_static keeps
the scratch in an array compiled into the library.  This test drives both entry points
through the C ABI on the same inputs and expects the same per-row statistic — twice in a
row with different inputs, because the second call finds the first call's partials still
sitting in the shared array and must not be affected by them.  The expected values come from
the CPU oracle (`fused_head_stats`), so the two entry points are not merely checked against
each other.

Collected last on purpose (file name), so a run that stops at the first failure has already
covered every other test; it also passes when run alone in a fresh process.
"""

import ctypes as C

import numpy as np
import pytest
import torch

from algebraic_transformer_b200 import _lib as L
from oracle import algebraic_ref as R

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
STATIC_BYTES = 4 << 20          # ALG_HEAD_STATIC_SCRATCH_BYTES in include/alg_b200.h


def _inputs(N, d, V, seed):
    g = torch.Generator().manual_seed(seed)
    h = torch.randn((N, d), generator=g).bfloat16().to(DEV)
    e = (torch.randn((V, d), generator=g) * 0.05).bfloat16().to(DEV)
    t = torch.randint(0, V, (N,), generator=g).to(torch.int32).to(DEV)
    return h, e, t


def _args(h, e, t, out, impl):
    return L.HeadArgs(h=h.data_ptr(), e=e.data_ptr(), targets=t.data_ptr(), l_out=out[0].data_ptr(),
                      zt_out=out[1].data_ptr(), N=h.shape[0], d=h.shape[1], V_local=e.shape[0], vocab_offset=0,
                      V_total=e.shape[0], n=8, c=2.0, impl=L.IMPL[impl])


@pytest.mark.parametrize("impl", ["auto", "mma"])
def test_static_scratch_head_matches_workspace_head_twice(impl):
    lib = L.load()
    stream = torch.cuda.current_stream().cuda_stream
    # two different problems back to back: the second one is smaller, so stale partials of
    # the first remain in the array beyond what the second call writes
    for N, d, V, seed in ((1024, 256, 20000, 1), (384, 128, 5000, 2)):
        h, e, t = _inputs(N, d, V, seed)
        want = torch.full((2, N), float("nan"), device=DEV)
        got = torch.full((2, N), float("nan"), device=DEV)
        a = _args(h, e, t, want, impl)
        ws = torch.empty(lib.alg_head_workspace_bytes(a), dtype=torch.uint8, device=DEV)
        a.workspace, a.workspace_bytes = ws.data_ptr(), ws.numel()
        assert lib.alg_head_fwd(a, stream) == L.ALG_OK, lib.alg_last_error()
        b = _args(h, e, t, got, impl)                   # no workspace at all
        assert lib.alg_head_fwd_static(b, stream) == L.ALG_OK, lib.alg_last_error()
        torch.cuda.synchronize()
        assert torch.isfinite(got).all()
        np.testing.assert_allclose(got.cpu(), want.cpu(), rtol=1e-6, atol=0)
        # both against the oracle: row normaliser l and target logit zt of the fused kernel
        l_ref, zt_ref = R.fused_head_stats(h.cpu(), e.cpu(), t.cpu(), 8, 2.0)
        for name, res in (("alg_head_fwd_static", got), ("alg_head_fwd", want)):
            l, zt = res[0].cpu().double(), res[1].cpu().double()
            assert float((l - l_ref.double()).norm() / l_ref.double().norm()) < 1e-3, name
            np.testing.assert_allclose(zt, zt_ref.double(), rtol=2e-3, atol=2e-3, err_msg=name)


def test_static_scratch_head_rejects_oversized_problem():
    lib = L.load()
    # validation happens on the host before any launch, so dummy non-null addresses suffice
    a = L.HeadArgs(h=256, e=256, targets=256, l_out=256, zt_out=256, N=1 << 20, d=768, V_local=50304,
                   vocab_offset=0, V_total=50304, n=8, c=2.0, impl=L.ALG_IMPL_AUTO)
    assert 8 * a.N > STATIC_BYTES
    assert lib.alg_head_fwd_static(a, None) == L.ALG_ERR_WORKSPACE
    msg = lib.alg_last_error().decode()
    assert "alg_head_fwd" in msg and "scratch" in msg
    with pytest.raises(ValueError):
        L.check(L.ALG_ERR_WORKSPACE)
