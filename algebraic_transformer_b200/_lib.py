"""ctypes binding of `lib/libalg_b200.so` (the C ABI of include/alg_b200.h).

There is no fallback: if the shared object is missing, importing the ops fails
with an instruction to build it.
"""

import ctypes as C
import os

PKG = os.path.dirname(os.path.abspath(__file__))
# ALG_B200_LIB selects another build of the same ABI (e.g. an instrumented one).
LIB_PATH = os.environ.get("ALG_B200_LIB") or os.path.join(PKG, "lib", "libalg_b200.so")

ALG_OK = 0
ALG_ERR_INVALID, ALG_ERR_UNSUPPORTED, ALG_ERR_CUDA, ALG_ERR_WORKSPACE = -1, -2, -3, -4
ALG_BF16, ALG_F32 = 0, 1
ALG_VARIANT_GUARD, ALG_VARIANT_NOSHIFT, ALG_VARIANT_SHIFT = 0, 1, 2
ALG_IMPL_AUTO, ALG_IMPL_MMA, ALG_IMPL_TCGEN05 = 0, 1, 2
IMPL = {"auto": ALG_IMPL_AUTO, "mma": ALG_IMPL_MMA, "tcgen05": ALG_IMPL_TCGEN05}

I64x3 = C.c_int64 * 3


class QkRmsArgs(C.Structure):
    _fields_ = [("x", C.c_void_p), ("y", C.c_void_p), ("gain", C.c_void_p), ("cos", C.c_void_p),
                ("sin", C.c_void_p), ("eps", C.c_float), ("B", C.c_int), ("H", C.c_int), ("T", C.c_int),
                ("D", C.c_int), ("dtype", C.c_int), ("x_stride", I64x3), ("y_stride", I64x3)]


class QkRmsBwdArgs(C.Structure):
    _fields_ = [("x", C.c_void_p), ("dy", C.c_void_p), ("gain", C.c_void_p), ("dx", C.c_void_p),
                ("dgain", C.c_void_p), ("eps", C.c_float), ("B", C.c_int), ("H", C.c_int), ("T", C.c_int),
                ("D", C.c_int), ("dtype", C.c_int), ("x_stride", I64x3), ("dy_stride", I64x3), ("dx_stride", I64x3),
                ("workspace", C.c_void_p), ("workspace_bytes", C.c_size_t)]


class AttnArgs(C.Structure):
    _fields_ = [("q", C.c_void_p), ("k", C.c_void_p), ("v", C.c_void_p), ("o", C.c_void_p),
                ("stat", C.c_void_p), ("stat_kind", C.c_void_p), ("sink", C.c_void_p),
                ("q_gain", C.c_void_p), ("k_gain", C.c_void_p), ("cos", C.c_void_p), ("sin", C.c_void_p),
                ("eps", C.c_float), ("B", C.c_int), ("H", C.c_int), ("Tq", C.c_int), ("Tk", C.c_int),
                ("D", C.c_int), ("n", C.c_int), ("c", C.c_float), ("causal", C.c_int), ("variant", C.c_int),
                ("dtype", C.c_int), ("impl", C.c_int), ("score_clamp", C.c_float),
                ("q_stride", I64x3), ("k_stride", I64x3), ("v_stride", I64x3), ("o_stride", I64x3),
                ("workspace", C.c_void_p), ("workspace_bytes", C.c_size_t), ("status", C.c_void_p),
                ("guard_words", C.c_void_p)]


class AttnBwdArgs(C.Structure):
    _fields_ = [("q", C.c_void_p), ("k", C.c_void_p), ("v", C.c_void_p), ("o", C.c_void_p), ("d_o", C.c_void_p),
                ("stat", C.c_void_p), ("stat_kind", C.c_void_p), ("sink", C.c_void_p), ("dq", C.c_void_p),
                ("dk", C.c_void_p), ("dv", C.c_void_p), ("dsink", C.c_void_p), ("B", C.c_int), ("H", C.c_int),
                ("Tq", C.c_int), ("Tk", C.c_int), ("D", C.c_int), ("n", C.c_int), ("c", C.c_float), ("causal", C.c_int),
                ("q_stride", I64x3), ("k_stride", I64x3), ("v_stride", I64x3), ("o_stride", I64x3),
                ("workspace", C.c_void_p), ("workspace_bytes", C.c_size_t), ("status", C.c_void_p),
                ("impl", C.c_int)]


class HeadBwdArgs(C.Structure):
    _fields_ = [("h", C.c_void_p), ("e", C.c_void_p), ("targets", C.c_void_p), ("l", C.c_void_p), ("zt", C.c_void_p),
                ("dz", C.c_void_p), ("N", C.c_int), ("d", C.c_int), ("V_local", C.c_int), ("vocab_offset", C.c_int),
                ("V_total", C.c_int), ("n", C.c_int), ("c", C.c_float), ("upstream", C.c_float), ("status", C.c_void_p),
                ("kind", C.c_int)]


class QkvProjArgs(C.Structure):
    _fields_ = [("x", C.c_void_p), ("w", C.c_void_p), ("qkv", C.c_void_p), ("q_gain", C.c_void_p),
                ("k_gain", C.c_void_p), ("cos", C.c_void_p), ("sin", C.c_void_p), ("eps", C.c_float),
                ("M", C.c_int), ("d", C.c_int), ("H", C.c_int), ("D", C.c_int), ("T", C.c_int),
                ("ld_x", C.c_int64), ("attn_c", C.c_float), ("guard", C.c_void_p), ("status", C.c_void_p),
                ("row_ss", C.c_void_p), ("ss_slots", C.c_int), ("row_eps", C.c_float), ("guard_is_zero", C.c_int)]


class GluProjArgs(C.Structure):
    _fields_ = [("x", C.c_void_p), ("w", C.c_void_p), ("out", C.c_void_p), ("M", C.c_int), ("d", C.c_int),
                ("f", C.c_int), ("ld_x", C.c_int64), ("ld_out", C.c_int64), ("beta", C.c_float),
                ("status", C.c_void_p), ("row_ss", C.c_void_p), ("ss_slots", C.c_int), ("row_eps", C.c_float)]


class ResidProjArgs(C.Structure):
    _fields_ = [("x", C.c_void_p), ("w", C.c_void_p), ("resid", C.c_void_p), ("out", C.c_void_p),
                ("ss_out", C.c_void_p), ("M", C.c_int), ("K", C.c_int), ("N", C.c_int), ("ld_x", C.c_int64),
                ("ld_resid", C.c_int64), ("ld_out", C.c_int64), ("status", C.c_void_p)]


class DecodeArgs(C.Structure):
    _fields_ = [("q", C.c_void_p), ("k", C.c_void_p), ("v", C.c_void_p), ("o", C.c_void_p),
                ("sink", C.c_void_p), ("B", C.c_int), ("H", C.c_int), ("Tk", C.c_int), ("D", C.c_int),
                ("n", C.c_int), ("c", C.c_float), ("k_stride", I64x3), ("v_stride", I64x3),
                ("workspace", C.c_void_p), ("workspace_bytes", C.c_size_t)]


class HeadArgs(C.Structure):
    _fields_ = [("h", C.c_void_p), ("e", C.c_void_p), ("targets", C.c_void_p), ("l_out", C.c_void_p),
                ("zt_out", C.c_void_p), ("N", C.c_int), ("d", C.c_int), ("V_local", C.c_int),
                ("vocab_offset", C.c_int), ("V_total", C.c_int), ("n", C.c_int), ("c", C.c_float),
                ("impl", C.c_int), ("workspace", C.c_void_p), ("workspace_bytes", C.c_size_t),
                ("status", C.c_void_p), ("kind", C.c_int)]


HEAD_ALG_CE, HEAD_CE = 0, 1


ALG_MAX_RANKS = 16


class HeadExchangeArgs(C.Structure):
    _fields_ = [("rank", C.c_int), ("world", C.c_int), ("peer_region", C.c_void_p * ALG_MAX_RANKS),
                ("N_capacity", C.c_int), ("pt", C.c_void_p), ("nll", C.c_void_p), ("obj", C.c_void_p),
                ("wait_budget_ns", C.c_ulonglong)]


# every symbol include/alg_b200.h declares: name -> (restype, argtypes)
SYMBOLS = {
    "alg_version": (C.c_int, []),
    "alg_last_error": (C.c_char_p, []),
    "alg_kernel_launches": (C.c_ulonglong, []),
    "alg_qk_rms_fwd": (C.c_int, [C.POINTER(QkRmsArgs), C.c_void_p]),
    "alg_qk_rms_bwd_workspace_bytes": (C.c_size_t, [C.c_int]),
    "alg_qk_rms_bwd": (C.c_int, [C.POINTER(QkRmsBwdArgs), C.c_void_p]),
    "alg_attn_workspace_bytes": (C.c_size_t, [C.POINTER(AttnArgs)]),
    "alg_attn_fwd": (C.c_int, [C.POINTER(AttnArgs), C.c_void_p]),
    "alg_attn_bwd_workspace_bytes": (C.c_size_t, [C.POINTER(AttnBwdArgs)]),
    "alg_attn_bwd": (C.c_int, [C.POINTER(AttnBwdArgs), C.c_void_p]),
    "alg_head_bwd_dz": (C.c_int, [C.POINTER(HeadBwdArgs), C.c_void_p]),
    "alg_decode_workspace_bytes": (C.c_size_t, [C.POINTER(DecodeArgs)]),
    "alg_attn_decode": (C.c_int, [C.POINTER(DecodeArgs), C.c_void_p]),
    "alg_head_workspace_bytes": (C.c_size_t, [C.POINTER(HeadArgs)]),
    "alg_head_fwd": (C.c_int, [C.POINTER(HeadArgs), C.c_void_p]),
    "alg_head_fwd_static": (C.c_int, [C.POINTER(HeadArgs), C.c_void_p]),
    "alg_head_exchange_region_bytes": (C.c_size_t, [C.c_int, C.c_int]),
    "alg_head_fwd_exchange": (C.c_int, [C.POINTER(HeadArgs), C.POINTER(HeadExchangeArgs), C.c_void_p]),
    "alg_head_finalize_workspace_bytes": (C.c_size_t, [C.c_int]),
    "alg_head_finalize": (C.c_int, [C.c_void_p, C.c_void_p, C.c_int, C.c_int, C.c_float, C.c_int,
                                    C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p, C.c_size_t, C.c_void_p]),
    "alg_head_finalize_ce": (C.c_int, [C.c_void_p, C.c_void_p, C.c_int, C.c_void_p, C.c_void_p, C.c_void_p,
                                       C.c_void_p, C.c_size_t, C.c_void_p]),
    "alg_cast_f32_to_bf16": (C.c_int, [C.c_void_p, C.c_void_p, C.c_size_t, C.c_void_p]),
    "alg_qkv_proj_fwd": (C.c_int, [C.POINTER(QkvProjArgs), C.c_void_p]),
    "alg_glu_proj_fwd": (C.c_int, [C.POINTER(GluProjArgs), C.c_void_p]),
    "alg_resid_proj_fwd": (C.c_int, [C.POINTER(ResidProjArgs), C.c_void_p]),
    "alg_resid_proj_ss_slots": (C.c_int, [C.c_int, C.c_int]),
    "alg_row_sumsq": (C.c_int, [C.c_void_p, C.c_int64, C.c_int, C.c_int64, C.c_void_p, C.c_void_p]),
    "alg_selftest_bounded_wait": (C.c_int, [C.c_void_p, C.c_ulonglong, C.c_void_p, C.c_void_p]),
    "alg_rms_norm_fwd":(C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_int64, C.c_int, C.c_float, C.c_void_p]),
    "alg_alu_glu_fwd": (C.c_int, [C.c_void_p, C.c_void_p, C.c_void_p, C.c_int64, C.c_int, C.c_int64, C.c_int64, C.c_float,
                                  C.c_void_p]),
}

_lib = None


def load():
    """Load the shared object once; raise if it has not been built."""
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(LIB_PATH):
        raise RuntimeError(
            f"{LIB_PATH} is missing: build it with `python -m algebraic_transformer_b200.build` "
            "(nvcc, sm_100a). This package has no CPU or PyTorch fallback.")
    lib = C.CDLL(LIB_PATH)
    for name, (res, args) in SYMBOLS.items():
        fn = getattr(lib, name)          # AttributeError if the library lacks a declared symbol
        fn.restype = res
        fn.argtypes = args
    _lib = lib
    return lib


def check(rc):
    """Map an ALG_ERR_* return code to the exception the reference's API raises."""
    if rc == ALG_OK:
        return
    msg = load().alg_last_error().decode()
    if rc in (ALG_ERR_INVALID, ALG_ERR_UNSUPPORTED, ALG_ERR_WORKSPACE):
        raise ValueError(msg)
    raise RuntimeError(msg)
