"""Names of the upstream FlashAttention package, served by the sm_100a kernels.

The reference ships a top-level `flash_attn` package for this (flash_attn/__init__.py:4-22: the
FlashAttention-2 names plus the FlashAttention-1 `*_unpadded_*` aliases, `bert_padding`, and
`layers.rotary`).  Here the same modules live under `flash_attn_triton_b200.compat` so that
importing them never shadows an installed upstream `flash_attn` wheel; code written against the
reference switches with

    import flash_attn_triton_b200.compat as flash_attn
    from flash_attn_triton_b200.compat.bert_padding import unpad_input, pad_input
    from flash_attn_triton_b200.compat.layers.rotary import RotaryEmbedding, apply_rotary_emb
"""
from ..flash_attn_interface import (  # noqa: F401
    FlashAttention,
    flash_attn_func,
    flash_attn_kvpacked_func,
    flash_attn_qkvpacked_func,
    flash_attn_varlen_func,
    flash_attn_varlen_kvpacked_func,
    flash_attn_varlen_qkvpacked_func,
    flash_attn_with_kvcache,
)

# FlashAttention 1.x names (flash_attn/__init__.py:17-22)
flash_attn_unpadded_func = flash_attn_varlen_func
flash_attn_unpadded_qkvpacked_func = flash_attn_varlen_qkvpacked_func
flash_attn_unpadded_kvpacked_func = flash_attn_varlen_kvpacked_func
