"""Drop-in alias: `import flash_attn_triton` resolves to the B200 implementation, so code
written against the reference package runs unchanged."""
from flash_attn_triton_b200 import *  # noqa: F401,F403
from flash_attn_triton_b200 import (  # noqa: F401
    FlashAttention, FlashCrossAttention, FlashSelfAttention, attention_int8, flash_attn_func,
    flash_attn_func_cross, flash_attn_kvpacked_func, flash_attn_qkvpacked_func,
    flash_attn_varlen_func, flash_attn_varlen_kvpacked_func, flash_attn_varlen_qkvpacked_func,
    flash_attn_with_kvcache)
