"""Rotary position embedding: functional forms with autograd and the RotaryEmbedding module.

Same names and contracts as the reference's flash_attn/layers/rotary.py (rotate_half :11-17,
apply_rotary_emb_torch :20-32, apply_rotary_emb :94-128, apply_rotary_emb_qkv_ :210-233,
apply_rotary_emb_kv_ :276-296, RotaryEmbedding :299-481), over the CUDA kernel behind
compat.ops.triton.rotary.apply_rotary.  The backward of a rotation is the rotation by the
conjugate angle, applied to the incoming gradient.
"""
from __future__ import annotations

from typing import Optional, Tuple, Union

import torch

from ..ops.triton.rotary import apply_rotary


def rotate_half(x, interleaved=False):
    if not interleaved:
        x1, x2 = x.chunk(2, dim=-1)
        return torch.cat((-x2, x1), dim=-1)
    x1, x2 = x[..., ::2], x[..., 1::2]
    return torch.stack((-x2, x1), dim=-1).flatten(-2)


def apply_rotary_emb_torch(x, cos, sin, interleaved=False):
    """Eager restatement: x (batch, seqlen, nheads, headdim), cos/sin (seqlen, rotary_dim / 2)
    or (batch, seqlen, rotary_dim / 2)."""
    ro_dim = cos.shape[-1] * 2
    assert ro_dim <= x.shape[-1]
    rep = (lambda t: t.repeat_interleave(2, dim=-1)) if interleaved else (lambda t: torch.cat((t, t), dim=-1))
    cos, sin = rep(cos).unsqueeze(-2), rep(sin).unsqueeze(-2)
    return torch.cat([x[..., :ro_dim] * cos + rotate_half(x[..., :ro_dim], interleaved) * sin, x[..., ro_dim:]],
                     dim=-1)


def _save_offsets(ctx, tensors, seqlen_offsets):
    if isinstance(seqlen_offsets, int):
        ctx.save_for_backward(*tensors)
        ctx.seqlen_offsets = seqlen_offsets
    else:
        ctx.save_for_backward(*tensors, seqlen_offsets)
        ctx.seqlen_offsets = None


def _load_offsets(ctx):
    saved = ctx.saved_tensors
    if ctx.seqlen_offsets is None:
        return saved[:-1], saved[-1]
    return saved, ctx.seqlen_offsets


class ApplyRotaryEmb(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, cos, sin, interleaved=False, inplace=False, seqlen_offsets: Union[int, torch.Tensor] = 0,
                cu_seqlens: Optional[torch.Tensor] = None, max_seqlen: Optional[int] = None):
        out = apply_rotary(x, cos, sin, seqlen_offsets=seqlen_offsets, cu_seqlens=cu_seqlens,
                           max_seqlen=max_seqlen, interleaved=interleaved, inplace=inplace)
        ctx.has_cu = cu_seqlens is not None
        _save_offsets(ctx, (cos, sin) + ((cu_seqlens,) if ctx.has_cu else ()), seqlen_offsets)
        ctx.interleaved, ctx.inplace, ctx.max_seqlen = interleaved, inplace, max_seqlen
        if inplace:
            ctx.mark_dirty(x)
            return x
        return out

    @staticmethod
    def backward(ctx, do):
        tensors, seqlen_offsets = _load_offsets(ctx)
        cos, sin = tensors[0], tensors[1]
        cu_seqlens = tensors[2] if ctx.has_cu else None
        do = do.contiguous()
        dx = apply_rotary(do, cos, sin, seqlen_offsets=seqlen_offsets, cu_seqlens=cu_seqlens,
                          max_seqlen=ctx.max_seqlen, interleaved=ctx.interleaved, inplace=ctx.inplace,
                          conjugate=True)
        return dx, None, None, None, None, None, None, None


def apply_rotary_emb(x, cos, sin, interleaved=False, inplace=False, seqlen_offsets: Union[int, torch.Tensor] = 0,
                     cu_seqlens: Optional[torch.Tensor] = None, max_seqlen: Optional[int] = None):
    """x (batch, seqlen, nheads, headdim), or (total, nheads, headdim) with cu_seqlens;
    cos/sin (seqlen_rotary, rotary_dim / 2).  Rotates the first rotary_dim columns."""
    return ApplyRotaryEmb.apply(x, cos, sin, interleaved, inplace, seqlen_offsets, cu_seqlens, max_seqlen)


apply_rotary_emb_func = apply_rotary_emb


def _rotate_qk_(qkv, cos, sin, cos_k, sin_k, interleaved, seqlen_offsets, conjugate):
    """q and k slices of a (batch, seqlen, 3, nheads, headdim) tensor rotated in place: one launch
    over the (2 * nheads) combined heads when q and k share the tables and the tensor is
    contiguous, else one per slice."""
    batch, seqlen, three, nheads, headdim = qkv.shape
    assert three == 3
    if cos_k is None and sin_k is None and qkv.is_contiguous():
        qk = qkv[:, :, :2].reshape(batch, seqlen, -1, headdim)   # a view: the slices are adjacent
        apply_rotary(qk, cos, sin, seqlen_offsets=seqlen_offsets, interleaved=interleaved, inplace=True,
                     conjugate=conjugate)
    else:
        apply_rotary(qkv[:, :, 0], cos, sin, seqlen_offsets, interleaved=interleaved, inplace=True,
                     conjugate=conjugate)
        apply_rotary(qkv[:, :, 1], cos if cos_k is None else cos_k, sin if sin_k is None else sin_k,
                     seqlen_offsets, interleaved=interleaved, inplace=True, conjugate=conjugate)


class ApplyRotaryEmbQKV_(torch.autograd.Function):
    @staticmethod
    def forward(ctx, qkv, cos, sin, cos_k=None, sin_k=None, interleaved=False,
                seqlen_offsets: Union[int, torch.Tensor] = 0):
        _rotate_qk_(qkv, cos, sin, cos_k, sin_k, interleaved, seqlen_offsets, conjugate=False)
        ctx.has_k = cos_k is not None
        _save_offsets(ctx, (cos, sin) + ((cos_k, sin_k) if ctx.has_k else ()), seqlen_offsets)
        ctx.interleaved = interleaved
        ctx.mark_dirty(qkv)
        return qkv

    @staticmethod
    def backward(ctx, dqkv):
        tensors, seqlen_offsets = _load_offsets(ctx)
        cos, sin = tensors[0], tensors[1]
        cos_k, sin_k = (tensors[2], tensors[3]) if ctx.has_k else (None, None)
        dqkv = dqkv.contiguous()
        _rotate_qk_(dqkv, cos, sin, cos_k, sin_k, ctx.interleaved, seqlen_offsets, conjugate=True)
        return dqkv, None, None, None, None, None, None


def apply_rotary_emb_qkv_(qkv, cos, sin, cos_k=None, sin_k=None, interleaved=False,
                          seqlen_offsets: Union[int, torch.Tensor] = 0):
    """qkv (batch, seqlen, 3, nheads, headdim): q and k rotated IN PLACE (k with cos_k/sin_k when given)."""
    return ApplyRotaryEmbQKV_.apply(qkv, cos, sin, cos_k, sin_k, interleaved, seqlen_offsets)


class ApplyRotaryEmbKV_(torch.autograd.Function):
    @staticmethod
    def forward(ctx, kv, cos, sin, interleaved=False, seqlen_offsets: Union[int, torch.Tensor] = 0):
        assert kv.shape[2] == 2
        apply_rotary(kv[:, :, 0], cos, sin, seqlen_offsets=seqlen_offsets, interleaved=interleaved, inplace=True)
        _save_offsets(ctx, (cos, sin), seqlen_offsets)
        ctx.interleaved = interleaved
        ctx.mark_dirty(kv)
        return kv

    @staticmethod
    def backward(ctx, dkv):
        (cos, sin), seqlen_offsets = _load_offsets(ctx)
        dkv = dkv.contiguous()
        apply_rotary(dkv[:, :, 0], cos, sin, seqlen_offsets=seqlen_offsets, interleaved=ctx.interleaved,
                     inplace=True, conjugate=True)
        return dkv, None, None, None, None


def apply_rotary_emb_kv_(kv, cos, sin, interleaved=False, seqlen_offsets: Union[int, torch.Tensor] = 0):
    """kv (batch, seqlen, 2, nheads, headdim): k rotated IN PLACE."""
    return ApplyRotaryEmbKV_.apply(kv, cos, sin, interleaved, seqlen_offsets)


class RotaryEmbedding(torch.nn.Module):
    """Rotary embedding with cached cos/sin tables (RoFormer; optional XPos scaling through
    `scale_base`).  forward() rotates qkv -- or q and kv -- IN PLACE.  Table construction follows
    the reference (flash_attn/layers/rotary.py:362-411): positions and inverse frequencies in
    fp32 unless pos_idx_in_fp32 is off, tables cast to the activations' dtype."""

    def __init__(self, dim: int, base=10000.0, interleaved=False, scale_base=None, pos_idx_in_fp32=True,
                 device=None):
        super().__init__()
        self.dim = dim
        self.base = float(base)
        self.pos_idx_in_fp32 = pos_idx_in_fp32
        self.register_buffer("inv_freq", self._compute_inv_freq(device), persistent=False)
        self.interleaved = interleaved
        self.scale_base = scale_base
        scale = ((torch.arange(0, dim, 2, device=device, dtype=torch.float32) + 0.4 * dim) / (1.4 * dim)
                 if scale_base is not None else None)
        self.register_buffer("scale", scale, persistent=False)
        self._seq_len_cached = 0
        self._cos_cached = self._sin_cached = self._cos_k_cached = self._sin_k_cached = None

    def _compute_inv_freq(self, device=None):
        return 1.0 / (self.base ** (torch.arange(0, self.dim, 2, device=device, dtype=torch.float32) / self.dim))

    def _update_cos_sin_cache(self, seqlen, device=None, dtype=None):
        stale = (seqlen > self._seq_len_cached or self._cos_cached is None or self._cos_cached.device != device
                 or self._cos_cached.dtype != dtype or (self.training and self._cos_cached.is_inference()))
        if not stale:
            return
        self._seq_len_cached = seqlen
        if self.pos_idx_in_fp32:
            t = torch.arange(seqlen, device=device, dtype=torch.float32)
            inv_freq = self.inv_freq if self.inv_freq.dtype == torch.float32 else self._compute_inv_freq(device=device)
        else:
            t = torch.arange(seqlen, device=device, dtype=self.inv_freq.dtype)
            inv_freq = self.inv_freq
        freqs = torch.outer(t, inv_freq)
        if self.scale is None:
            self._cos_cached, self._sin_cached = torch.cos(freqs).to(dtype), torch.sin(freqs).to(dtype)
            return
        power = (torch.arange(seqlen, dtype=self.scale.dtype, device=self.scale.device) - seqlen // 2) / self.scale_base
        scale = self.scale.to(device=power.device) ** power.unsqueeze(-1)
        self._cos_cached, self._sin_cached = (torch.cos(freqs) * scale).to(dtype), (torch.sin(freqs) * scale).to(dtype)
        self._cos_k_cached, self._sin_k_cached = (torch.cos(freqs) / scale).to(dtype), (torch.sin(freqs) / scale).to(dtype)

    def forward(self, qkv: torch.Tensor, kv: Optional[torch.Tensor] = None,
                seqlen_offset: Union[int, torch.Tensor] = 0, max_seqlen: Optional[int] = None
                ) -> Union[torch.Tensor, Tuple[torch.Tensor, torch.Tensor]]:
        """qkv (batch, seqlen, 3, nheads, headdim), or q (batch, seqlen, nheads, headdim) with
        kv (batch, seqlen, 2, nheads, headdim).  seqlen_offset: int or (batch,) tensor (then pass
        max_seqlen so that the tables cover every position)."""
        seqlen = qkv.shape[1]
        if max_seqlen is not None:
            self._update_cos_sin_cache(max_seqlen, device=qkv.device, dtype=qkv.dtype)
        elif isinstance(seqlen_offset, int):
            self._update_cos_sin_cache(seqlen + seqlen_offset, device=qkv.device, dtype=qkv.dtype)
        xpos = self.scale is not None
        if kv is None:
            return apply_rotary_emb_qkv_(qkv, self._cos_cached, self._sin_cached,
                                         self._cos_k_cached if xpos else None, self._sin_k_cached if xpos else None,
                                         interleaved=self.interleaved, seqlen_offsets=seqlen_offset)
        q = apply_rotary_emb_func(qkv, self._cos_cached, self._sin_cached, interleaved=self.interleaved,
                                  inplace=True, seqlen_offsets=seqlen_offset)
        kv = apply_rotary_emb_kv_(kv, self._cos_k_cached if xpos else self._cos_cached,
                                  self._sin_k_cached if xpos else self._sin_cached,
                                  interleaved=self.interleaved, seqlen_offsets=seqlen_offset)
        return q, kv
