"""CPU checks of the drop-in boundary: the library loads, exports every symbol the
header declares, rejects bad arguments before any launch, and the host-side logic
(partitioning, argument validation of the Python surface, position tables) is right."""

import ctypes as C
import os
import re

import numpy as np
import pytest
import torch

import algebraic_transformer_b200 as A
from algebraic_transformer_b200 import _lib as L
from oracle import algebraic_ref as R

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_library_exports_every_declared_symbol():
    header = open(os.path.join(ROOT, "include", "alg_b200.h")).read()
    declared = set(re.findall(r"ALG_API\s+[\w\s\*]+?\b(alg_\w+)\s*\(", header))
    assert declared, "no declarations parsed"
    assert declared == set(L.SYMBOLS), (declared ^ set(L.SYMBOLS))
    lib = L.load()
    raw = C.CDLL(L.LIB_PATH)
    for name in declared:
        assert getattr(raw, name) is not None
    assert lib.alg_version() == 100


def test_invalid_arguments_fail_before_launch():
    lib = L.load()
    a = L.AttnArgs()                                   # all null
    assert lib.alg_attn_fwd(a, None) == L.ALG_ERR_INVALID
    assert b"null" in lib.alg_last_error()
    a = L.AttnArgs(q=16, k=16, v=16, o=16, B=1, H=1, Tq=8, Tk=8, D=48, n=16, c=8.0)
    assert lib.alg_attn_fwd(a, None) == L.ALG_ERR_UNSUPPORTED
    a.D, a.n = 64, 12
    assert lib.alg_attn_fwd(a, None) == L.ALG_ERR_INVALID
    assert b"power of two" in lib.alg_last_error()
    a.n, a.variant = 16, L.ALG_VARIANT_GUARD             # guard needs a workspace
    assert lib.alg_attn_fwd(a, None) == L.ALG_ERR_WORKSPACE
    h = L.HeadArgs(h=16, e=16, targets=16, l_out=16, zt_out=16, N=128, d=64, V_local=10, vocab_offset=5,
                   V_total=12, n=8, c=2.0)
    assert lib.alg_head_fwd(h, None) == L.ALG_ERR_INVALID   # shard exceeds the vocabulary
    h = L.HeadArgs(h=16, e=16, targets=16, l_out=16, zt_out=16, N=128, d=64, V_local=8, V_total=8, n=8, c=2.0, kind=7)
    assert lib.alg_head_fwd(h, None) == L.ALG_ERR_INVALID and b"kind" in lib.alg_last_error()
    h.kind, h.n, h.c, h.d = L.HEAD_CE, 0, 0.0, 72            # the ce kind ignores n and c, but has no kernel for d % 64 != 0
    assert lib.alg_head_fwd(h, None) == L.ALG_ERR_UNSUPPORTED
    h.d, h.impl = 64, L.IMPL["mma"]
    assert lib.alg_head_fwd(h, None) == L.ALG_ERR_UNSUPPORTED
    h.impl = L.IMPL["auto"]
    assert lib.alg_head_fwd_static(h, None) == L.ALG_ERR_UNSUPPORTED
    assert lib.alg_head_finalize_ce(None, None, 4, None, None, None, None, 0, None) == L.ALG_ERR_INVALID
    q = L.QkRmsArgs(x=16, y=16, eps=0.0, B=1, H=1, T=1, D=64)
    assert lib.alg_qk_rms_fwd(q, None) == L.ALG_ERR_INVALID
    assert lib.alg_qk_rms_bwd(L.QkRmsBwdArgs(), None) == L.ALG_ERR_INVALID
    qb = L.QkRmsBwdArgs(x=16, dy=16, dx=16, dgain=16, eps=1e-5, B=1, H=1, T=8, D=64, dtype=L.ALG_BF16)
    assert lib.alg_qk_rms_bwd(qb, None) == L.ALG_ERR_INVALID and b"dgain without gain" in lib.alg_last_error()
    qb.gain = 16
    assert lib.alg_qk_rms_bwd(qb, None) == L.ALG_ERR_WORKSPACE
    qb.D = 96
    assert lib.alg_qk_rms_bwd(qb, None) == L.ALG_ERR_UNSUPPORTED
    assert lib.alg_qk_rms_bwd_workspace_bytes(128) == 1024 * 128 * 4 and lib.alg_qk_rms_bwd_workspace_bytes(96) == 0
    # guard words handed over by the QKV projection describe ready-made q, k, v: not with the prologue
    a = L.AttnArgs(q=16, k=16, v=16, o=16, B=1, H=1, Tq=256, Tk=256, D=64, n=16, c=8.0, variant=L.ALG_VARIANT_GUARD,
                   guard_words=16, q_gain=16, k_gain=16, cos=16, sin=16, eps=1e-5)
    assert lib.alg_attn_fwd(a, None) == L.ALG_ERR_INVALID
    assert b"guard_words" in lib.alg_last_error()
    # the fused projections
    assert lib.alg_qkv_proj_fwd(L.QkvProjArgs(), None) == L.ALG_ERR_INVALID
    pj = L.QkvProjArgs(x=16, w=16, qkv=16, cos=16, sin=16, eps=1e-5, M=128, d=768, H=12, D=48, T=128, ld_x=768,
                       attn_c=8.0)
    assert lib.alg_qkv_proj_fwd(pj, None) == L.ALG_ERR_INVALID     # head_dim must be 64 or 128
    pj.D, pj.d, pj.ld_x = 64, 700, 700
    assert lib.alg_qkv_proj_fwd(pj, None) == L.ALG_ERR_INVALID     # d must be a multiple of 64
    pj.d, pj.ld_x, pj.x = 768, 768, 8
    assert lib.alg_qkv_proj_fwd(pj, None) == L.ALG_ERR_INVALID     # 16-byte alignment
    assert b"alignment" in lib.alg_last_error()
    gl = L.GluProjArgs(x=16, w=16, out=16, M=128, d=768, f=100, ld_x=768, ld_out=100, beta=0.5)
    assert lib.alg_glu_proj_fwd(gl, None) == L.ALG_ERR_INVALID     # f must be a multiple of 128
    gl.f, gl.ld_out = 256, 128
    assert lib.alg_glu_proj_fwd(gl, None) == L.ALG_ERR_INVALID     # output rows narrower than f
    # head backward
    assert lib.alg_head_bwd_dz(L.HeadBwdArgs(), None) == L.ALG_ERR_INVALID
    hb = L.HeadBwdArgs(h=16, e=16, targets=16, l=16, zt=16, dz=16, N=128, d=768, V_local=1001, vocab_offset=0,
                       V_total=1001, n=8, c=2.0, upstream=1.0)
    assert lib.alg_head_bwd_dz(hb, None) == L.ALG_ERR_INVALID        # V_local must be a multiple of 8
    hb.V_local, hb.V_total, hb.n = 1000, 1000, 12
    assert lib.alg_head_bwd_dz(hb, None) == L.ALG_ERR_INVALID        # n must be a power of two
    hb.n, hb.kind = 8, 5
    assert lib.alg_head_bwd_dz(hb, None) == L.ALG_ERR_INVALID and b"kind" in lib.alg_last_error()
    # attention backward
    assert lib.alg_attn_bwd(L.AttnBwdArgs(), None) == L.ALG_ERR_INVALID
    bw = L.AttnBwdArgs(q=16, k=16, v=16, o=16, d_o=16, stat=16, stat_kind=16, dq=16, dk=16, dv=16, B=1, H=2, Tq=64,
                       Tk=64, D=64, n=16, c=8.0, causal=1)
    assert lib.alg_attn_bwd_workspace_bytes(bw) == 1 * 2 * 64 * 4
    assert lib.alg_attn_bwd(bw, None) == L.ALG_ERR_WORKSPACE         # delta scratch missing
    bw.sink = 16                                                     # sink without dsink
    assert lib.alg_attn_bwd(bw, None) == L.ALG_ERR_INVALID
    assert b"pair" in lib.alg_last_error()
    with pytest.raises(ValueError):
        L.check(L.ALG_ERR_INVALID)


def test_workspace_sizes():
    lib = L.load()
    a = L.AttnArgs(B=2, H=3, Tq=512, Tk=512, D=64, dtype=L.ALG_BF16)
    assert lib.alg_attn_workspace_bytes(a) == 8192
    a.cos = 16
    assert lib.alg_attn_workspace_bytes(a) == 8192 + 2 * (2 * 3 * 512 * 64 * 2)
    # fp32 rows the tcgen05 kernel can take (head_dim 64, causal, Tq == Tk): room for the
    # bf16 hi | lo copies of q, k, v on top; other fp32 shapes ask for no more than bf16 ones
    f = L.AttnArgs(B=2, H=3, Tq=512, Tk=512, D=64, dtype=L.ALG_F32, causal=1)
    assert lib.alg_attn_workspace_bytes(f) == 8192 + 3 * (2 * 3 * 512 * 128 * 2)
    f.causal = 0
    assert lib.alg_attn_workspace_bytes(f) == 8192
    f.causal, f.Tq, f.Tk = 1, 384, 512
    assert lib.alg_attn_workspace_bytes(f) == 8192
    f.Tq, f.Tk = 300, 300                                   # any length: rows, not tiles, are copied
    assert lib.alg_attn_workspace_bytes(f) == 8192 + 3 * ((2 * 3 * 300 * 128 * 2 + 255) // 256 * 256)
    h = L.HeadArgs(N=8192, d=768, V_local=50304)
    assert lib.alg_head_workspace_bytes(h) >= 2 * 8192 * 4
    assert lib.alg_head_finalize_workspace_bytes(8192) >= 32 * 4 + 16


def test_python_surface_validation_matches_reference_errors():
    x = torch.zeros(1, 1, 512, 64)
    with pytest.raises(ValueError, match="CUDA"):
        A.flash_attention(x, x, x, kind="asinh")
    # the remaining checks run before any device work, on meta-like CUDA-less tensors
    class FakeCuda(torch.Tensor):
        @property
        def is_cuda(self):
            return True
    xf = x.as_subclass(FakeCuda)

    # tensors of one call must share a device; checked before anything touches CUDA
    def on(index):
        class Placed(FakeCuda):
            @property
            def device(self):
                return torch.device("cuda", index)
        return x.as_subclass(Placed)
    with pytest.raises(ValueError, match="different devices"):
        A.flash_attention(on(0), on(1), on(0), kind="asinh")
    with pytest.raises(ValueError, match="different devices"):
        A.qk_rms_norm(on(1), on(0))
    with pytest.raises(ValueError, match="divisible by blocks"):
        A.flash_attention(xf[:, :, :500], xf[:, :, :500], xf[:, :, :500], kind="asinh", block=128)
    with pytest.raises(ValueError, match="power of two"):
        A.flash_attention(xf, xf, xf, kind="asinh", n=12)
    with pytest.raises(ValueError, match="positive and finite"):
        A.flash_attention(xf, xf, xf, kind="asinh", c=0.0)
    with pytest.raises(ValueError, match="unknown attention kernel"):
        A.flash_attention(xf, xf, xf, kind="linear")
    with pytest.raises(ValueError, match="inverse-denominator"):
        A.flash_attention(xf, xf, xf, kind="asinh", shift=True, inv_stat=True)
    with pytest.raises(ValueError, match="whole-head residency"):
        A.flash_attention(xf, xf, xf, kind="asinh", c=8.0, head_resident=True)
    with pytest.raises(NotImplementedError):
        A.flash_attention(xf, xf, xf)                  # softmax control arm: not built
    h = torch.zeros(100, 64, dtype=torch.bfloat16).as_subclass(FakeCuda)
    e = torch.zeros(300, 64).as_subclass(FakeCuda)
    t = torch.zeros(100, dtype=torch.int64).as_subclass(FakeCuda)
    with pytest.raises(ValueError, match="power of two"):
        A.fused_head(h, e, t, kind="alg_ce", n=12)
    with pytest.raises(ValueError, match="must be divisible by block"):
        A.fused_head(torch.zeros(200, 64, dtype=torch.bfloat16).as_subclass(FakeCuda), e, t, kind="alg_ce",
                     n=8, block_n=128)
    with pytest.raises(ValueError):
        A.fused_head(h, e, t, kind="mse")
    g = torch.ones(64).as_subclass(FakeCuda)
    with pytest.raises(ValueError, match="epsilon"):
        A.qk_rms_norm(xf, g, 0.0)
    with pytest.raises(ValueError, match="D=64"):
        A.qk_rms_norm(torch.zeros(4, 48).as_subclass(FakeCuda), torch.ones(48).as_subclass(FakeCuda))
    with pytest.raises(ValueError, match="eight rows"):
        A.qk_rms_norm(xf, g, block=4)


def test_host_tables_match_oracle(golden):
    for D, T in ((64, 300), (128, 257)):
        c, s = A.cayley_table_geometric(D, T)
        np.testing.assert_allclose(c, golden[f"cayley_cos_D{D}_T{T}"], atol=2e-6)
        np.testing.assert_allclose(s, golden[f"cayley_sin_D{D}_T{T}"], atol=2e-6)
    c, s = A.cayley_table_geometric(64, 1024)
    c2, s2 = R.cayley_table_geometric(64, 1024)
    assert torch.equal(c, c2) and torch.equal(s, s2)
    with pytest.raises(ValueError):
        A.cayley_table_geometric(96, 8)
    assert A.flash_clamp(1024, 16) == R.flash_clamp(1024, 16)


def test_partitioning_rules():
    for V, world in ((50304, 8), (50304, 4), (32000, 8), (50257, 8), (1000, 3), (100, 8)):
        spans = [A.vocab_shard(V, r, world) for r in range(world)]
        assert spans[0][0] == 0 and sum(n for _, n in spans) == V
        for (lo, n), (lo2, _) in zip(spans, spans[1:]):
            assert lo + n == lo2 and (lo % 128 == 0 or n == 0)
        tiles = [-(-n // 128) for _, n in spans]
        assert max(tiles) - min(tiles) <= 1
    assert [A.vocab_shard(50304, r, 8)[1] // 128 for r in range(8)].count(50) == 1   # 393 = 7*49 + 50
    for units, world in ((16, 8), (48, 8), (16, 3), (5, 8)):
        spans = [A.unit_shard(units, r, world) for r in range(world)]
        assert sum(n for _, n in spans) == units
        assert all(a[0] + a[1] == b[0] for a, b in zip(spans, spans[1:]))
