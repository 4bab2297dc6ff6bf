"""Host-side argument checking of the public wrappers (no GPU): same ValueErrors, in the
same order, as the reference's wrappers raise before they reach a kernel."""
import pytest
import torch

import flash_attn_triton_b200 as fa


def t(*shape, dtype=torch.float16):
    return torch.zeros(*shape, dtype=dtype)


def test_flash_attn_func_errors():
    q = t(1, 8, 2, 64)
    with pytest.raises(ValueError, match="FP16"):
        fa.flash_attn_func(q.double(), q.double(), q.double())
    with pytest.raises(ValueError, match="softcap"):
        fa.flash_attn_func(q, q, q, softcap=-1)
    with pytest.raises(ValueError, match="dropout_p"):
        fa.flash_attn_func(q, q, q, dropout_p=1.0)
    with pytest.raises(ValueError, match="CUDA"):
        fa.flash_attn_func(q, q, q)
    with pytest.raises(ValueError, match="CUDA"):
        fa.flash_attn_func_cross(q, q, q)
    with pytest.raises(ValueError, match="matching"):
        fa.flash_attn_func_cross(q, q.float(), q)


def test_packed_shape_errors():
    with pytest.raises(ValueError):
        fa.flash_attn_qkvpacked_func(t(1, 8, 2, 2, 64))
    with pytest.raises(ValueError):
        fa.flash_attn_kvpacked_func(t(1, 8, 2, 64), t(1, 8, 3, 2, 64))


def test_kvcache_errors():
    q, c = t(2, 1, 4, 64), t(2, 16, 2, 64)
    with pytest.raises(ValueError, match="together"):
        fa.flash_attn_with_kvcache(q, c, c, rotary_cos=t(4, 8))
    with pytest.raises(ValueError, match="rank-4"):
        fa.flash_attn_with_kvcache(q[0], c, c)
    with pytest.raises(ValueError, match="same shape"):
        fa.flash_attn_with_kvcache(q, c, c[:, :8])
    with pytest.raises(ValueError, match="CUDA"):
        fa.flash_attn_with_kvcache(q, c, c)


def test_varlen_errors():
    q = t(8, 2, 64)
    cu = torch.tensor([0, 8], dtype=torch.int32)
    with pytest.raises(ValueError, match="rank-3"):
        fa.flash_attn_varlen_func(q[None], q, q, cu, cu, 8, 8)
    with pytest.raises(ValueError, match="one-dimensional"):
        fa.flash_attn_varlen_func(q, q, q, cu[None], cu[None], 8, 8)
    with pytest.raises(ValueError, match="same batch size"):
        fa.flash_attn_varlen_func(q, q, q, cu, torch.tensor([0, 4, 8], dtype=torch.int32), 8, 8)
    with pytest.raises(ValueError, match="CUDA"):
        fa.flash_attn_varlen_func(q, q, q, cu, cu, 8, 8)


def test_int8_errors():
    with pytest.raises(ValueError, match="CUDA"):
        fa.attention_int8(t(1, 1, 64, 64), t(1, 1, 64, 64), t(1, 1, 64, 64))


def test_missing_library_fails_loudly(monkeypatch):
    from flash_attn_triton_b200 import _native as N
    monkeypatch.setattr(N, "_lib", None)
    monkeypatch.setattr(N, "LIB_PATH", "/nonexistent/libfa_b200.so")
    with pytest.raises(RuntimeError, match="no CPU fallback"):
        N.lib()
