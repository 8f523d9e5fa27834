"""Host-side checks of the jax.ffi layer: the Python module imports and degrades cleanly without JAX,
and every handler it would register is defined in the XLA-FFI translation unit and calls only
functions the C header declares."""

import os
import re

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
TU = os.path.join(ROOT, "algebraic_transformer_b200", "csrc", "xla_ffi.cc")
HEADER = os.path.join(ROOT, "include", "alg_b200.h")


def test_module_imports_without_jax_and_says_why():
    from algebraic_transformer_b200 import jax_ffi
    try:
        import jax  # noqa: F401
        has_jax = True
    except Exception:
        has_jax = False
    if has_jax and jax_ffi.available():
        pytest.skip("JAX and the handler library are present: nothing to degrade")
    assert jax_ffi.available() is False
    with pytest.raises(ImportError, match="unavailable"):
        jax_ffi._need()


def test_argument_errors_come_before_any_use_of_jax():
    from algebraic_transformer_b200 import jax_ffi

    class Shape:
        def __init__(self, *shape):
            self.shape, self.ndim = tuple(shape), len(shape)

    x = Shape(1, 2, 512, 64)
    with pytest.raises(NotImplementedError):
        jax_ffi.flash_attention(x, x, x, kind="softmax")
    with pytest.raises(ValueError, match="power of two"):
        jax_ffi.flash_attention(x, x, x, kind="asinh", n=12)
    with pytest.raises(ValueError, match="divisible by blocks"):
        jax_ffi.flash_attention(Shape(1, 2, 500, 64), Shape(1, 2, 500, 64), Shape(1, 2, 500, 64), kind="asinh", block=128)
    with pytest.raises(ValueError, match="D=64 or D=128"):
        jax_ffi.qk_rms_norm(Shape(1, 2, 8, 96), Shape(96))
    with pytest.raises(ValueError, match="gain shape"):
        jax_ffi.qk_rms_norm(Shape(1, 2, 8, 64), Shape(32))
    with pytest.raises(ValueError, match="divisible by block_n"):
        jax_ffi.fused_head(Shape(100, 64), Shape(512, 64), Shape(100), kind="alg_ce", n=8, block_n=64)


def test_every_registered_handler_is_defined_and_uses_declared_entry_points():
    from algebraic_transformer_b200 import jax_ffi
    tu = open(TU).read()
    header = open(HEADER).read()
    defined = set(re.findall(r"XLA_FFI_DEFINE_HANDLER_SYMBOL\(\s*(\w+)", tu))
    assert set(jax_ffi.TARGETS.values()) == defined
    called = set(re.findall(r"\b(alg_[a-z0-9_]+)\s*\(", tu))
    declared = set(re.findall(r"ALG_API\s+[\w\s\*]+?\b(alg_[a-z0-9_]+)\s*\(", header))
    assert called and called <= declared, called - declared
    # the attributes each Python wrapper passes are the ones its handler binds
    for target, attrs in (("AlgAttnFwd", {"n", "c", "variant", "has_sink", "causal"}), ("AlgQkRmsFwd", {"eps"}),
                          ("AlgHeadFwd", {"n", "c", "vocab_offset", "vocab_total"}),
                          ("AlgHeadFinalize", {"n", "c", "vocab_total"})):
        block = tu[tu.index(f"XLA_FFI_DEFINE_HANDLER_SYMBOL({target},"):]
        block = block[:block.index(");") + 2]
        assert set(re.findall(r'Attr<[\w:]+>\("(\w+)"\)', block)) == attrs, target
