"""apply_rotary: launcher of the rotary-embedding kernel (fa_rotary in the C ABI).

Same contract as the reference's flash_attn/ops/triton/rotary.py:133-234 (the module keeps the
reference's path, although nothing here is Triton): x (batch, seqlen, nheads, headdim) or packed
(total, nheads, headdim) with cu_seqlens; cos/sin (seqlen_ro, rotary_dim / 2) in x's dtype;
an int or (batch,) tensor of position offsets; rotate-half or interleaved pairs; in place or not;
the conjugate form is the backward.  Arithmetic in fp32 with one rounding per element, table rows
past seqlen_ro read as cos = 1, sin = 0, like the kernel it replaces (:11-130).
"""
from __future__ import annotations

import ctypes as C
from typing import Optional, Union

import torch

from .... import _native as N

_DT = {torch.float16: N.FA_F16, torch.bfloat16: N.FA_BF16, torch.float32: N.FA_F32}


def apply_rotary(x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor,
                 seqlen_offsets: Union[int, torch.Tensor] = 0, cu_seqlens: Optional[torch.Tensor] = None,
                 max_seqlen: Optional[int] = None, interleaved=False, inplace=False, conjugate=False) -> torch.Tensor:
    is_varlen = cu_seqlens is not None
    if not is_varlen:
        batch, seqlen, nheads, headdim = x.shape
    else:
        assert max_seqlen is not None, "If cu_seqlens is passed in, then max_seqlen must be passed"
        _, nheads, headdim = x.shape
        batch = cu_seqlens.shape[0] - 1
        seqlen = max_seqlen
    seqlen_ro, rotary_dim = cos.shape
    assert sin.shape == cos.shape
    rotary_dim *= 2
    assert rotary_dim <= headdim, "rotary_dim must be <= headdim"
    assert headdim <= 256, "Only support headdim <= 256"
    assert seqlen_ro >= seqlen, "seqlen_ro must be >= seqlen"
    assert cos.dtype == sin.dtype, f"cos and sin must have the same dtype, got {cos.dtype} and {sin.dtype}"
    assert x.dtype == cos.dtype, f"Input and cos/sin must have the same dtype, got {x.dtype} and {cos.dtype}"
    if x.dtype not in _DT or not x.is_cuda:
        raise ValueError("apply_rotary needs a CUDA tensor of float16, bfloat16 or float32")
    cos, sin = cos.contiguous(), sin.contiguous()
    offsets = None
    if isinstance(seqlen_offsets, torch.Tensor):
        if seqlen_offsets.shape != (batch,):
            raise ValueError("seqlen_offsets must have one value per batch item")
        if seqlen_offsets.dtype not in (torch.int32, torch.int64):
            raise ValueError("seqlen_offsets must use int32 or int64")
        if seqlen_offsets.device != x.device:
            raise ValueError("seqlen_offsets must be on the same device as x")
        if torch.any(seqlen_offsets < 0) or torch.any(seqlen_offsets + seqlen > seqlen_ro):
            raise ValueError("seqlen_offsets must keep every rotary position within the table")
        offsets = seqlen_offsets.to(torch.int32).contiguous()
    elif seqlen_offsets < 0 or seqlen_offsets + seqlen > seqlen_ro:
        raise ValueError("seqlen_offsets must keep every rotary position within the table")
    if x.stride(-1) != 1:
        if inplace:
            raise ValueError("in-place rotary needs a unit head-dim stride")
        x = x.contiguous()
    output = x if inplace else torch.empty_like(x)
    if output.stride(-1) != 1:
        output = torch.empty(x.shape, dtype=x.dtype, device=x.device)
    a = N.RotaryArgs()
    a.dtype = _DT[x.dtype]
    a.device = x.device.index if x.device.index is not None else torch.cuda.current_device()
    a.batch, a.seqlen, a.heads, a.head_dim = batch, seqlen, nheads, headdim
    a.x, a.out = x.data_ptr(), output.data_ptr()
    dims = (None, 0, 1) if is_varlen else (0, 1, 2)
    a.x_stride, a.out_stride = N.strides3(x, dims), N.strides3(output, dims)
    a.cos, a.sin = cos.data_ptr(), sin.data_ptr()
    a.rotary_dim, a.rotary_seqlen = rotary_dim, seqlen_ro
    a.interleaved, a.conjugate = int(bool(interleaved)), int(bool(conjugate))
    cu = None
    if offsets is not None:
        a.seqlen_offsets = offsets.data_ptr()
    else:
        a.seqlen_offset = int(seqlen_offsets)
    if is_varlen:
        cu = cu_seqlens.to(device=x.device, dtype=torch.int32).contiguous()
        a.cu_seqlens = cu.data_ptr()
    with torch.cuda.device(x.device):
        N.check(N.lib().fa_rotary(C.byref(a), N.stream_ptr(x.device)), "fa_rotary")
    return output
