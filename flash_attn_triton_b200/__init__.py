"""B200 (sm_100a) attention kernels behind the `flash_attn_triton` public API.

Same eleven names as the reference's flash_attn_triton/__init__.py:6-18, plus
`attention_int8` (which the reference keeps in triton_kernel/attention_kernel_int8.py).
"""
from .flash_attn_interface import (  # noqa: F401
    FlashAttention,
    FlashCrossAttention,
    FlashSelfAttention,
    attention_int8,
    flash_attn_func,
    flash_attn_func_cross,
    flash_attn_kvpacked_func,
    flash_attn_qkvpacked_func,
    flash_attn_varlen_func,
    flash_attn_varlen_kvpacked_func,
    flash_attn_varlen_qkvpacked_func,
    flash_attn_with_kvcache,
    set_validation,
)

__version__ = "0.1.0"
