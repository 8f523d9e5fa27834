"""Failure detection without a GPU fault: a device-side wait that can never be satisfied
runs out after its budget, the kernel reports ALG_DEV_TIMEOUT through the status word and
returns, and the context stays usable for the next launch."""

import pytest
import torch

import algebraic_transformer_b200 as A
from algebraic_transformer_b200 import _lib as L

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def test_bounded_wait_times_out_and_reports_status():
    lib = L.load()
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    waited = torch.zeros(1, dtype=torch.int64, device=DEV)
    budget_ns = 5_000_000                                  # 5 ms
    stream = torch.cuda.current_stream().cuda_stream
    assert lib.alg_selftest_bounded_wait(status.data_ptr(), budget_ns, waited.data_ptr(), stream) == L.ALG_OK
    torch.cuda.synchronize()                               # returns: the kernel did not hang
    assert int(status) == 1                                # ALG_DEV_TIMEOUT
    assert budget_ns <= int(waited) < 100 * budget_ns
    # the context is intact: a real kernel runs right after and gives the right answer
    x = torch.randn(4, 2, 16, 64, device=DEV)
    y = A.qk_rms_norm(x, torch.ones(64, device=DEV))
    want = x * torch.rsqrt((x * x).mean(-1, keepdim=True) + 1e-5)
    assert torch.allclose(y, want, rtol=1e-5, atol=1e-6)
    # bad arguments are refused on the host
    assert lib.alg_selftest_bounded_wait(None, budget_ns, None, stream) == L.ALG_ERR_INVALID
    assert lib.alg_selftest_bounded_wait(status.data_ptr(), 5_000_000_000, None, stream) == L.ALG_ERR_INVALID
