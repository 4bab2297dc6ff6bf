"""`from flash_attn_triton.triton_kernel.attention_kernel import attention, attention_varlen`:
the import path of the reference's operator layer, resolved to the B200 implementation."""
from flash_attn_triton_b200.attention_kernel import attention, attention_varlen  # noqa: F401
