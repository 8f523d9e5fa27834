"""A NumPy-backed stand-in for the small slice of the `jax` API that the
reference's dense math modules use, so that the reference's OWN source files
can be executed in an environment without JAX.

Only `make_golden.py` uses this.  It is generation-time tooling: no test, no
product path and no benchmark imports it.  It substitutes the array backend
(NumPy, IEEE fp32/fp64 on the host) and nothing else: every formula that ends
up in the golden files is evaluated by the reference's unmodified code.

Covered API: `jax.numpy` array functions used by `src/algebraic/algebraic.py`,
`src/algebraic/kernels/flash.py` (host-side helpers only) and
`src/algebraic/kernels/fused_head.py` (host-side helpers only); `jax.lax.rsqrt`,
`jax.lax.stop_gradient`; `jax.custom_vjp` as a primal pass-through.  For
`src/algebraic/model.py` (the forward pass only): `jax.lax.scan` as a Python loop over the
leading axis, `jax.checkpoint` as the identity, `jax.random.PRNGKey/split/normal` on
NumPy generators, bfloat16 through `ml_dtypes`, and an ndarray subclass (`XlaArray`) whose
`@` multiplies with float32 accumulation and rounds to the operands' dtype as XLA does.
"""

import sys
import types

import numpy as np


def _einsum(subscripts, *operands, preferred_element_type=None, **kw):
    if preferred_element_type is not None:
        operands = [np.asarray(o).astype(preferred_element_type) for o in operands]
    return np.einsum(subscripts, *operands, **kw)


def _matmul(a, b, preferred_element_type=None):
    if preferred_element_type is not None:
        a = np.asarray(a).astype(preferred_element_type)
        b = np.asarray(b).astype(preferred_element_type)
    return np.matmul(a, b)


class _CustomVjp:
    """`jax.custom_vjp` reduced to its primal function."""

    def __init__(self, fn, nondiff_argnums=()):
        self.fn = fn
        self.__doc__ = getattr(fn, "__doc__", None)
        self.__name__ = getattr(fn, "__name__", "custom_vjp")

    def defvjp(self, fwd, bwd):
        return None

    def __call__(self, *a, **k):
        return self.fn(*a, **k)


def _xla_matmul(a, b):
    a, b = np.asarray(a), np.asarray(b)
    out = np.promote_types(a.dtype, b.dtype)
    acc = np.float64 if out == np.float64 else np.float32
    return np.matmul(a.astype(acc), b.astype(acc)).astype(out).view(XlaArray)


class XlaArray(np.ndarray):
    """ndarray whose `@` follows XLA's dot: accumulate in float32, round to the promoted
    operand dtype (NumPy would return float32 for two bfloat16 operands)."""

    def __matmul__(self, other):
        return _xla_matmul(self, other)

    def __rmatmul__(self, other):
        return _xla_matmul(other, self)


def _scan(body, carry, xs):
    """`lax.scan` over the leading axis of every leaf of the dict `xs`; outputs are dropped
    (model.py's body returns None for them)."""
    length = len(next(iter(xs.values())))
    for i in range(length):
        carry, _ = body(carry, {k: v[i] for k, v in xs.items()})
    return carry, None


def _rsqrt(x):
    x = np.asarray(x)
    one = np.ones((), dtype=x.dtype)
    return (one / np.sqrt(x)).astype(x.dtype)


def install():
    """Insert shim modules into ``sys.modules`` under the jax names."""
    jax = types.ModuleType("jax")
    jnp = types.ModuleType("jax.numpy")
    lax = types.ModuleType("jax.lax")
    experimental = types.ModuleType("jax.experimental")
    pallas = types.ModuleType("jax.experimental.pallas")
    pltpu = types.ModuleType("jax.experimental.pallas.tpu")

    for name in ("float32", "float64", "int32", "bool_", "abs", "where", "mean", "max",
                 "sum", "tril", "ones", "zeros", "arange", "take_along_axis", "minimum",
                 "maximum", "concatenate", "full_like", "full", "sqrt", "promote_types",
                 "expand_dims", "broadcast_to", "reshape", "transpose", "dtype", "pad",
                 "logical_and", "logical_not", "tile", "linspace", "isfinite"):
        setattr(jnp, name, getattr(np, name))
    jnp.asarray = lambda x, dtype=None: np.asarray(x, dtype=dtype)
    jnp.array = lambda x, dtype=None: np.array(x, dtype=dtype)
    jnp.einsum = _einsum
    jnp.matmul = _matmul
    jnp.ndarray = np.ndarray

    lax.rsqrt = _rsqrt
    lax.stop_gradient = lambda x: x

    # what src/algebraic/standard.py calls (the "ce" head and its neighbours)
    for name in ("exp", "log", "cos", "sin"):
        setattr(jnp, name, getattr(np, name))
    nn = types.ModuleType("jax.nn")

    def _logsumexp(a, axis=None):
        a = np.asarray(a)
        top = np.max(a, axis=axis, keepdims=True)
        out = np.log(np.sum(np.exp(a - top), axis=axis, keepdims=True)) + top
        return np.squeeze(out, axis=axis).astype(a.dtype)

    nn.logsumexp = _logsumexp
    nn.sigmoid = lambda x: (1.0 / (1.0 + np.exp(-np.asarray(x)))).astype(np.asarray(x).dtype)
    nn.softmax = lambda x, axis=-1: np.exp(np.asarray(x) - np.expand_dims(_logsumexp(x, axis=axis), axis))
    jax.nn = nn
    sys.modules["jax.nn"] = nn

    # what src/algebraic/model.py needs on top (forward pass only)
    import ml_dtypes                                      # registers the NumPy dtype "bfloat16"
    jnp.bfloat16 = ml_dtypes.bfloat16
    lax.scan = _scan
    jax.checkpoint = lambda fn, **kw: fn
    random = types.ModuleType("jax.random")
    random.PRNGKey = lambda seed: int(seed)
    random.split = lambda key, num=2: [int(key) * 1000003 + i + 1 for i in range(num)]
    random.normal = lambda key, shape, dtype=np.float32: (
        np.random.default_rng(int(key)).standard_normal(shape).astype(dtype).view(XlaArray))
    jax.random = random
    jax.tree_util = types.ModuleType("jax.tree_util")
    sys.modules["jax.random"] = random
    sys.modules["jax.tree_util"] = jax.tree_util

    jax.Array = np.ndarray
    jax.custom_vjp = _CustomVjp
    jax.numpy = jnp
    jax.lax = lax
    jax.experimental = experimental
    experimental.pallas = pallas
    pallas.tpu = pltpu

    sys.modules.update({
        "jax": jax, "jax.numpy": jnp, "jax.lax": lax, "jax.experimental": experimental,
        "jax.experimental.pallas": pallas, "jax.experimental.pallas.tpu": pltpu,
    })
    return jax
