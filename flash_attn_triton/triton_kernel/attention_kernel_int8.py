"""`from flash_attn_triton.triton_kernel.attention_kernel_int8 import attention_int8` is how
the reference's tests reach the INT8 entry point; keep that import path working."""
from flash_attn_triton_b200.flash_attn_interface import attention_int8  # noqa: F401
