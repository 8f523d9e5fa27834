"""B200 (sm_100a) kernels for the Algebraic Transformer's hot path — the forward kernels and the
backward halves of their custom VJPs — behind the reference's Python call surface.  See `ops` for
the entry points and `include/alg_b200.h` for the C ABI underneath."""

from .ops import (cast_embedding, cayley_powers, cayley_table_geometric, decode_attention,  # noqa: F401
                  flash_attention, flash_attention_backward, flash_clamp, fused_head, fused_head_backward,
                  glu_projection, head_finalize, head_statistic, interleave_gate_up, qk_rms_norm,
                  qk_rms_norm_backward, qkv_projection, resid_projection, row_sumsq)
from .dist import unit_shard, vocab_shard  # noqa: F401

__all__ = ["flash_attention", "fused_head", "qk_rms_norm", "decode_attention", "cayley_table_geometric",
           "cayley_powers", "cast_embedding", "head_statistic", "head_finalize", "flash_clamp",
           "vocab_shard", "unit_shard", "qkv_projection", "glu_projection", "interleave_gate_up",
           "flash_attention_backward", "fused_head_backward", "qk_rms_norm_backward", "resid_projection",
           "row_sumsq"]
