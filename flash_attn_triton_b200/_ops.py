"""Operator layer: torch.autograd.Function wrappers that fill the C-ABI argument blocks.

Takes the place of the reference's `_attention`, `_attention_varlen` and
`_attention_int8` autograd functions (flash_attn_triton/triton_kernel/attention_kernel.py:1158-1198,
:1281-1361; attention_kernel_int8.py:220-267).  Differences that matter to callers: tensors
stay in their (batch, seq, heads, dim) layout (strides are passed down, nothing is
transposed or padded), GQA is native in forward and backward, and the backward is
deterministic.
"""
from __future__ import annotations

import ctypes as C

import torch

from . import _native as N


def _prep(t):
    return t if N.kernel_ready(t) else t.contiguous()


def _alibi_ptr(alibi):
    return None if alibi is None else alibi.data_ptr()


class Features:
    """The options beyond the score pipeline that the argument block carries: an additive fp32
    bias (batch, heads, rows, cols; broadcast dimensions have stride 0), dropout with the
    reference's random stream, and the per-sequence length overrides of a packed batch."""

    __slots__ = ("bias", "dropout_p", "seed", "row_stride", "seqused_q", "seqused_k")

    def __init__(self, bias=None, dropout_p=0.0, seed=0, row_stride=0, seqused_q=None, seqused_k=None):
        self.bias, self.dropout_p, self.seed, self.row_stride = bias, float(dropout_p), int(seed), int(row_stride)
        self.seqused_q, self.seqused_k = seqused_q, seqused_k

    def tensors(self):
        return [t for t in (self.bias, self.seqused_q, self.seqused_k) if t is not None]

    def fill(self, a):
        if self.bias is not None:
            a.attn_bias = self.bias.data_ptr()
            a.bias_stride = (C.c_int64 * 4)(*self.bias.stride())
        if self.dropout_p > 0.0:
            a.dropout_p, a.dropout_seed, a.dropout_row_stride = self.dropout_p, self.seed, self.row_stride
        a.seqused_q, a.seqused_k = N.ptr(self.seqused_q), N.ptr(self.seqused_k)


_NO_FEATURES = Features()


def _fill_common(a, q, k, v, o, dims_q, dims_k, *, batch, sq, sk, hq, hkv, d, scale, causal, wl,
                 wr, softcap, alibi, q_pos_offset, impl, cu_q=None, cu_k=None, feat=None):
    a.dtype = N.dtype_code(q.dtype)
    a.device = q.device.index if q.device.index is not None else torch.cuda.current_device()
    a.impl = impl
    a.batch, a.seqlen_q, a.seqlen_k = batch, sq, sk
    a.heads_q, a.heads_kv, a.head_dim = hq, hkv, d
    a.q, a.k, a.v, a.o = N.ptr(q), N.ptr(k), N.ptr(v), N.ptr(o)
    a.q_stride = N.strides3(q, dims_q)
    a.k_stride = N.strides3(k, dims_k)
    a.v_stride = N.strides3(v, dims_k)
    a.o_stride = N.strides3(o, dims_q)
    a.cu_seqlens_q = N.ptr(cu_q)
    a.cu_seqlens_k = N.ptr(cu_k)
    if cu_q is not None:
        a.total_q, a.total_k = q.shape[0], k.shape[0]
    a.softmax_scale = float(scale)
    a.softcap = float(softcap)
    a.alibi_slopes = _alibi_ptr(alibi)
    a.causal = int(bool(causal))
    a.window_left, a.window_right = int(wl), int(wr)
    a.q_pos_offset = int(q_pos_offset)
    (feat or _NO_FEATURES).fill(a)


# dimension indices of (batch, row, head) in each layout
_BSHD = (0, 1, 2)      # (batch, seq, heads, dim)
_BHSD = (0, 2, 1)      # (batch, heads, seq, dim)
_THD = (None, 0, 1)    # packed (tokens, heads, dim)


def dense_forward(q, k, v, scale, causal, wl, wr, softcap, alibi, q_pos_offset, impl, layout,
                  want_lse, feat=None):
    dims = _BSHD if layout == "bshd" else _BHSD
    B = q.shape[0]
    Sq, Hq = q.shape[dims[1]], q.shape[dims[2]]
    Sk, Hkv = k.shape[dims[1]], k.shape[dims[2]]
    D = q.shape[-1]
    q, k, v = _prep(q), _prep(k), _prep(v)
    o = torch.empty(q.shape, dtype=q.dtype, device=q.device)
    lse = torch.empty((B, Hq, Sq), dtype=torch.float32, device=q.device) if want_lse else None
    a = N.AttnArgs()
    _fill_common(a, q, k, v, o, dims, dims, batch=B, sq=Sq, sk=Sk, hq=Hq, hkv=Hkv, d=D,
                 scale=scale, causal=causal, wl=wl, wr=wr, softcap=softcap, alibi=alibi,
                 q_pos_offset=q_pos_offset, impl=impl, feat=feat)
    if lse is not None:
        a.lse2 = lse.data_ptr()
        a.lse_stride = N._I64x3(Hq * Sq, 1, Sq)
    with torch.cuda.device(q.device):
        N.check(N.lib().fa_fwd(C.byref(a), N.stream_ptr(q.device)), "fa_fwd")
    return o, lse, (q, k, v)


def dense_probs(q, k, v, lse, scale, causal, wl, wr, softcap, alibi, q_pos_offset, layout, feat=None):
    """(probabilities fp32 (B, Hq, Sq, Sk), natural-log LSE (B, Hq, Sq)) of a dense call whose
    forward produced the base-2 `lse`: the return_attn_probs surface
    (flash_attn_interface.py:139-143 of the reference), from the fa_attn_probs kernel."""
    dims = _BSHD if layout == "bshd" else _BHSD
    B = q.shape[0]
    Sq, Hq = q.shape[dims[1]], q.shape[dims[2]]
    Sk, Hkv = k.shape[dims[1]], k.shape[dims[2]]
    probs = torch.zeros((B, Hq, Sq, Sk), dtype=torch.float32, device=q.device)
    lse_nat = torch.full((B, Hq, Sq), float("-inf"), dtype=torch.float32, device=q.device)
    a = N.AttnArgs()
    _fill_common(a, q, k, v, q, dims, dims, batch=B, sq=Sq, sk=Sk, hq=Hq, hkv=Hkv, d=q.shape[-1], scale=scale,
                 causal=causal, wl=wl, wr=wr, softcap=softcap, alibi=alibi, q_pos_offset=q_pos_offset,
                 impl=N.IMPL_AUTO, feat=feat)
    a.lse2 = lse.data_ptr()
    a.lse_stride = N._I64x3(Hq * Sq, 1, Sq)
    ps = (C.c_int64 * 4)(*probs.stride())
    with torch.cuda.device(q.device):
        N.check(N.lib().fa_attn_probs(C.byref(a), probs.data_ptr(), C.byref(ps), lse_nat.data_ptr(), Sq,
                                      N.stream_ptr(q.device)), "fa_attn_probs")
    return probs, lse_nat


def dense_backward(q, k, v, o, lse, dout, scale, causal, wl, wr, softcap, alibi, q_pos_offset,
                   impl, layout, feat=None):
    dims = _BSHD if layout == "bshd" else _BHSD
    B = q.shape[0]
    Sq, Hq = q.shape[dims[1]], q.shape[dims[2]]
    Sk, Hkv = k.shape[dims[1]], k.shape[dims[2]]
    D = q.shape[-1]
    dout = _prep(dout)
    dq = torch.empty(q.shape, dtype=q.dtype, device=q.device)
    dk = torch.empty(k.shape, dtype=k.dtype, device=k.device)
    dv = torch.empty(v.shape, dtype=v.dtype, device=v.device)
    delta = torch.empty_like(lse)
    a = N.AttnArgs()
    _fill_common(a, q, k, v, o, dims, dims, batch=B, sq=Sq, sk=Sk, hq=Hq, hkv=Hkv, d=D,
                 scale=scale, causal=causal, wl=wl, wr=wr, softcap=softcap, alibi=alibi,
                 q_pos_offset=q_pos_offset, impl=impl, feat=feat)
    a.lse2 = lse.data_ptr()
    a.lse_stride = N._I64x3(Hq * Sq, 1, Sq)
    a.dout, a.do_stride = dout.data_ptr(), N.strides3(dout, dims)
    a.delta = delta.data_ptr()
    a.dq, a.dk, a.dv = dq.data_ptr(), dk.data_ptr(), dv.data_ptr()
    a.dq_stride, a.dk_stride, a.dv_stride = (N.strides3(dq, dims), N.strides3(dk, dims),
                                             N.strides3(dv, dims))
    st = N.stream_ptr(q.device)
    with torch.cuda.device(q.device):
        L = N.lib()
        N.check(L.fa_bwd_preprocess(C.byref(a), st), "fa_bwd_preprocess")
        N.check(L.fa_bwd_dq(C.byref(a), st), "fa_bwd_dq")
        N.check(L.fa_bwd_dkdv(C.byref(a), st), "fa_bwd_dkdv")
    return dq, dk, dv


class DenseAttention(torch.autograd.Function):
    """q (B,Sq,Hq,D), k/v (B,Sk,Hkv,D) ["bshd"] or head-major ["bhsd"]; returns o like q."""

    @staticmethod
    def forward(ctx, q, k, v, scale, causal, wl, wr, softcap, alibi, q_pos_offset, impl, layout, feat=None,
                want_lse=False):
        need = any(t.requires_grad for t in (q, k, v))
        o, lse, (q, k, v) = dense_forward(q, k, v, scale, causal, wl, wr, softcap, alibi,
                                          q_pos_offset, impl, layout, want_lse=need or want_lse, feat=feat)
        if need:
            ctx.save_for_backward(q, k, v, o, lse, alibi if alibi is not None else q.new_empty(0))
            ctx.cfg = (scale, causal, wl, wr, softcap, alibi is not None, q_pos_offset, impl, layout)
            ctx.feat = feat
        if want_lse:
            ctx.mark_non_differentiable(lse)
            return o, lse
        return o

    @staticmethod
    def backward(ctx, dout, *unused):
        q, k, v, o, lse, alibi = ctx.saved_tensors
        scale, causal, wl, wr, softcap, has_alibi, off, impl, layout = ctx.cfg
        dq, dk, dv = dense_backward(q, k, v, o, lse, dout, scale, causal, wl, wr, softcap,
                                    alibi if has_alibi else None, off, impl, layout, feat=ctx.feat)
        return (dq, dk, dv) + (None,) * 11


def varlen_forward(q, k, v, cu_q, cu_k, max_q, max_k, scale, causal, wl, wr, softcap, alibi, impl,
                   want_lse, feat=None):
    Tq, Hq, D = q.shape
    Hkv = k.shape[1]
    batch = cu_q.numel() - 1
    q, k, v = _prep(q), _prep(k), _prep(v)
    o = torch.empty(q.shape, dtype=q.dtype, device=q.device)
    # base-2 LSE laid out (heads, tokens): consecutive rows of a head are contiguous
    lse = torch.empty((Hq, Tq), dtype=torch.float32, device=q.device) if want_lse else None
    a = N.AttnArgs()
    _fill_common(a, q, k, v, o, _THD, _THD, batch=batch, sq=max_q, sk=max_k, hq=Hq, hkv=Hkv, d=D,
                 scale=scale, causal=causal, wl=wl, wr=wr, softcap=softcap, alibi=alibi,
                 q_pos_offset=0, impl=impl, cu_q=cu_q, cu_k=cu_k, feat=feat)
    if lse is not None:
        a.lse2 = lse.data_ptr()
        a.lse_stride = N._I64x3(0, 1, Tq)
    with torch.cuda.device(q.device):
        N.check(N.lib().fa_varlen_fwd(C.byref(a), N.stream_ptr(q.device)), "fa_varlen_fwd")
    return o, lse, (q, k, v)


def varlen_probs(q, k, v, lse, cu_q, cu_k, max_q, max_k, scale, causal, wl, wr, softcap, alibi, feat=None):
    """(probabilities fp32 (batch, Hq, max_q, max_k) zero-padded, natural-log LSE (batch, Hq, max_q)
    padded with -inf) of a packed call: flash_attn_interface.py:642-659 of the reference."""
    Tq, Hq, D = q.shape
    batch = cu_q.numel() - 1
    probs = torch.zeros((batch, Hq, max_q, max_k), dtype=torch.float32, device=q.device)
    lse_nat = torch.full((batch, Hq, max_q), float("-inf"), dtype=torch.float32, device=q.device)
    a = N.AttnArgs()
    _fill_common(a, q, k, v, q, _THD, _THD, batch=batch, sq=max_q, sk=max_k, hq=Hq, hkv=k.shape[1], d=D,
                 scale=scale, causal=causal, wl=wl, wr=wr, softcap=softcap, alibi=alibi, q_pos_offset=0,
                 impl=N.IMPL_AUTO, cu_q=cu_q, cu_k=cu_k, feat=feat)
    a.lse2 = lse.data_ptr()
    a.lse_stride = N._I64x3(0, 1, Tq)
    ps = (C.c_int64 * 4)(*probs.stride())
    with torch.cuda.device(q.device):
        N.check(N.lib().fa_attn_probs(C.byref(a), probs.data_ptr(), C.byref(ps), lse_nat.data_ptr(), max_q,
                                      N.stream_ptr(q.device)), "fa_attn_probs")
    return probs, lse_nat


def varlen_backward(q, k, v, o, lse, dout, cu_q, cu_k, max_q, max_k, scale, causal, wl, wr,
                    softcap, alibi, impl, feat=None):
    Tq, Hq, D = q.shape
    Hkv = k.shape[1]
    batch = cu_q.numel() - 1
    dout = _prep(dout)
    # rows past cu_seqlens[-1] or past a sequence's used length never get a writer: start from zero
    # when the packed tensors are not fully covered
    partial = feat is not None and (feat.seqused_q is not None or feat.seqused_k is not None)
    alloc = torch.zeros if partial else torch.empty
    dq = alloc(q.shape, dtype=q.dtype, device=q.device)
    dk = alloc(k.shape, dtype=k.dtype, device=k.device)
    dv = alloc(v.shape, dtype=v.dtype, device=v.device)
    delta = torch.empty_like(lse)
    a = N.AttnArgs()
    _fill_common(a, q, k, v, o, _THD, _THD, batch=batch, sq=max_q, sk=max_k, hq=Hq, hkv=Hkv, d=D,
                 scale=scale, causal=causal, wl=wl, wr=wr, softcap=softcap, alibi=alibi,
                 q_pos_offset=0, impl=impl, cu_q=cu_q, cu_k=cu_k, feat=feat)
    a.lse2 = lse.data_ptr()
    a.lse_stride = N._I64x3(0, 1, Tq)
    a.dout, a.do_stride = dout.data_ptr(), N.strides3(dout, _THD)
    a.delta = delta.data_ptr()
    a.dq, a.dk, a.dv = dq.data_ptr(), dk.data_ptr(), dv.data_ptr()
    a.dq_stride, a.dk_stride, a.dv_stride = (N.strides3(dq, _THD), N.strides3(dk, _THD),
                                             N.strides3(dv, _THD))
    st = N.stream_ptr(q.device)
    with torch.cuda.device(q.device):
        L = N.lib()
        N.check(L.fa_bwd_preprocess(C.byref(a), st), "fa_bwd_preprocess")
        N.check(L.fa_varlen_bwd_dq(C.byref(a), st), "fa_varlen_bwd_dq")
        N.check(L.fa_varlen_bwd_dkdv(C.byref(a), st), "fa_varlen_bwd_dkdv")
    return dq, dk, dv


class VarlenAttention(torch.autograd.Function):
    """Packed q (Tq,Hq,D), k/v (Tk,Hkv,D) with int32 cu_seqlens on the device."""

    @staticmethod
    def forward(ctx, q, k, v, cu_q, cu_k, max_q, max_k, scale, causal, wl, wr, softcap, alibi, impl, feat=None,
                want_lse=False):
        need = any(t.requires_grad for t in (q, k, v))
        o, lse, (q, k, v) = varlen_forward(q, k, v, cu_q, cu_k, max_q, max_k, scale, causal, wl,
                                           wr, softcap, alibi, impl, want_lse=need or want_lse, feat=feat)
        if need:
            ctx.save_for_backward(q, k, v, o, lse, cu_q, cu_k,
                                  alibi if alibi is not None else q.new_empty(0))
            ctx.cfg = (max_q, max_k, scale, causal, wl, wr, softcap, alibi is not None, impl)
            ctx.feat = feat
        if want_lse:
            ctx.mark_non_differentiable(lse)
            return o, lse
        return o

    @staticmethod
    def backward(ctx, dout, *unused):
        q, k, v, o, lse, cu_q, cu_k, alibi = ctx.saved_tensors
        max_q, max_k, scale, causal, wl, wr, softcap, has_alibi, impl = ctx.cfg
        dq, dk, dv = varlen_backward(q, k, v, o, lse, dout, cu_q, cu_k, max_q, max_k, scale,
                                     causal, wl, wr, softcap, alibi if has_alibi else None, impl, feat=ctx.feat)
        return (dq, dk, dv) + (None,) * 13


# ----------------------------------------------------------------------------------------
# INT8
# ----------------------------------------------------------------------------------------
def quantize_k_int8(k):
    """k fp16 (..., S, D) contiguous -> (k8 int8 same shape, s_k fp32 (..., S))."""
    if k.dtype != torch.float16 or not k.is_cuda:
        raise ValueError("quantize_k_int8 needs a CUDA fp16 tensor")
    k = k.contiguous()
    D = k.shape[-1]
    rows = k.numel() // D
    k8 = torch.empty(k.shape, dtype=torch.int8, device=k.device)
    s_k = torch.empty(k.shape[:-1], dtype=torch.float32, device=k.device)
    dev = k.device.index if k.device.index is not None else torch.cuda.current_device()
    with torch.cuda.device(k.device):
        N.check(N.lib().fa_quantize_k_int8(k.data_ptr(), k8.data_ptr(), s_k.data_ptr(), rows, D,
                                           dev, N.stream_ptr(k.device)), "fa_quantize_k_int8")
    return k8, s_k


def int8_forward(q, k, v, causal, scale, impl=N.IMPL_AUTO, k_valid=0, q_pos_offset=0):
    B, H, S, D = q.shape
    k8, s_k = quantize_k_int8(k)
    o = torch.empty_like(q)
    lse = torch.empty((B, H, S), dtype=torch.float32, device=q.device)
    a = N.Int8Args()
    a.device = q.device.index if q.device.index is not None else torch.cuda.current_device()
    a.impl = impl
    a.batch, a.heads, a.seqlen, a.head_dim = B, H, S, D
    a.q, a.k8, a.s_k, a.v, a.o, a.lse2 = (q.data_ptr(), k8.data_ptr(), s_k.data_ptr(),
                                           v.data_ptr(), o.data_ptr(), lse.data_ptr())
    a.softmax_scale = float(scale)
    a.causal = int(bool(causal))
    a.seqlen_k_valid, a.q_pos_offset = int(k_valid), int(q_pos_offset)
    if D == 128 and impl != N.IMPL_MMA:
        q8 = torch.empty(q.shape, dtype=torch.int8, device=q.device)
        s_q = torch.empty(q.shape[:-1], dtype=torch.float32, device=q.device)
        a.q8_scratch, a.sq_scratch = q8.data_ptr(), s_q.data_ptr()
    with torch.cuda.device(q.device):
        N.check(N.lib().fa_fwd_int8(C.byref(a), N.stream_ptr(q.device)), "fa_fwd_int8")
    return o, lse, k8, s_k


class Int8Attention(torch.autograd.Function):
    """INT8-QK^T forward, fp16 backward (attention_kernel_int8.py:220-267).  [B,H,S,D]."""

    @staticmethod
    def forward(ctx, q, k, v, causal, scale, impl, k_valid=0, q_pos_offset=0):
        o, lse, _, _ = int8_forward(q, k, v, causal, scale, impl, k_valid, q_pos_offset)
        ctx.save_for_backward(q, k, v, o, lse)
        ctx.cfg = (causal, scale, k_valid, q_pos_offset)
        return o

    @staticmethod
    def backward(ctx, dout):
        q, k, v, o, lse = ctx.saved_tensors
        causal, scale, k_valid, off = ctx.cfg
        S = k.shape[2]
        if k_valid and k_valid < S:
            # padded call: the keys past k_valid take no part; their gradients are zero
            dq, dk_s, dv_s = dense_backward(q, k[:, :, :k_valid], v[:, :, :k_valid], o, lse, dout, scale,
                                            causal, -1, -1, 0.0, None, off, N.IMPL_AUTO, "bhsd")
            dk, dv = torch.zeros_like(k), torch.zeros_like(v)
            dk[:, :, :k_valid] = dk_s
            dv[:, :, :k_valid] = dv_s
        else:
            dq, dk, dv = dense_backward(q, k, v, o, lse, dout, scale, causal, -1, -1, 0.0, None, off,
                                        N.IMPL_AUTO, "bhsd")
        return dq, dk, dv, None, None, None, None, None


# ----------------------------------------------------------------------------------------
# KV-cache decode
# ----------------------------------------------------------------------------------------
_workspaces = {}


def _workspace(device, nbytes):
    """Grow-only scratch for split-KV partials, one per (device, stream)."""
    key = (device, torch.cuda.current_stream(device).cuda_stream)
    buf = _workspaces.get(key)
    if buf is None or buf.numel() < nbytes:
        buf = torch.empty(max(nbytes, 1 << 20), dtype=torch.uint8, device=device)
        _workspaces[key] = buf
    return buf


def kvcache_decode(q, k_cache, v_cache, k_new, v_new, cos, sin, cache_seqlens, cache_batch_idx,
                   cache_leftpad, block_table, scale, causal, wl, wr, rotary_interleaved, alibi,
                   num_splits=0):
    B, Sq, Hq, D = q.shape
    Hkv = k_cache.shape[2]
    q = _prep(q)
    o = torch.empty((B, Sq, Hq, D), dtype=q.dtype, device=q.device)
    a = N.DecodeArgs()
    a.dtype = N.dtype_code(q.dtype)
    a.device = q.device.index if q.device.index is not None else torch.cuda.current_device()
    a.batch, a.seqlen_q, a.heads_q, a.heads_kv, a.head_dim = B, Sq, Hq, Hkv, D
    a.q, a.o = q.data_ptr(), o.data_ptr()
    a.q_stride, a.o_stride = N.strides3(q, _BSHD), N.strides3(o, _BSHD)
    a.k_cache, a.v_cache = k_cache.data_ptr(), v_cache.data_ptr()
    a.kc_stride, a.vc_stride = N.strides3(k_cache, _BSHD), N.strides3(v_cache, _BSHD)
    a.page_size, a.num_pages = k_cache.shape[1], k_cache.shape[0]
    if block_table is not None:
        a.block_table = block_table.data_ptr()
        a.block_table_stride = block_table.stride(0)
    a.cache_batch_idx = N.ptr(cache_batch_idx)
    a.cache_seqlens = cache_seqlens.data_ptr()
    a.cache_leftpad = N.ptr(cache_leftpad)
    if k_new is not None:
        k_new, v_new = _prep(k_new), _prep(v_new)
        a.k_new, a.v_new = k_new.data_ptr(), v_new.data_ptr()
        a.kn_stride, a.vn_stride = N.strides3(k_new, _BSHD), N.strides3(v_new, _BSHD)
        a.seqlen_new = k_new.shape[1]
    if cos is not None:
        a.rotary_cos, a.rotary_sin = cos.data_ptr(), sin.data_ptr()
        a.rotary_dim = cos.shape[-1] * 2
        a.rotary_seqlen = cos.shape[0]
        a.rotary_interleaved = int(bool(rotary_interleaved))
    a.softmax_scale = float(scale)
    a.alibi_slopes = _alibi_ptr(alibi)
    a.causal = int(bool(causal))
    a.window_left, a.window_right = int(wl), int(wr)
    a.num_splits = int(num_splits)
    L = N.lib()
    need = L.fa_decode_workspace_bytes(C.byref(a))
    ws = None
    if need:
        ws = _workspace(q.device, need)
        a.workspace, a.workspace_bytes = ws.data_ptr(), ws.numel()
    with torch.cuda.device(q.device):
        N.check(L.fa_decode_paged(C.byref(a), N.stream_ptr(q.device)), "fa_decode_paged")
    return o


def kvcache_decode_static(q, out, k_cache, v_cache, cache_seqlens, block_table=None, k_new=None,
                          v_new=None, cos=None, sin=None, rotary_interleaved=True, scale=None,
                          causal=False, num_splits=0):
    """fa_decode_paged_static through ctypes: same decode, but the split-KV partials go to the
    16 MiB array built into the library, so neither this function nor the C entry point
    allocates anything -- `out` and every other tensor come from the caller.  For callers that
    must not touch an allocator at call time (a frozen serving pool, a callback inside another
    runtime).  q/out (B,Sq,Hq,D), caches (pages,page,Hkv,D), cache_seqlens int32 (B,),
    block_table int32 (B,max_pages) or None, all already on the device and kernel-ready."""
    B, Sq, Hq, D = q.shape
    a = N.DecodeArgs()
    a.dtype = N.dtype_code(q.dtype)
    a.device = q.device.index if q.device.index is not None else torch.cuda.current_device()
    a.batch, a.seqlen_q, a.heads_q, a.heads_kv, a.head_dim = B, Sq, Hq, k_cache.shape[2], D
    a.q, a.o = q.data_ptr(), out.data_ptr()
    a.q_stride, a.o_stride = N.strides3(q, _BSHD), N.strides3(out, _BSHD)
    a.k_cache, a.v_cache = k_cache.data_ptr(), v_cache.data_ptr()
    a.kc_stride, a.vc_stride = N.strides3(k_cache, _BSHD), N.strides3(v_cache, _BSHD)
    a.page_size, a.num_pages = k_cache.shape[1], k_cache.shape[0]
    if block_table is not None:
        a.block_table, a.block_table_stride = block_table.data_ptr(), block_table.stride(0)
    a.cache_seqlens = cache_seqlens.data_ptr()
    if k_new is not None:
        a.k_new, a.v_new = k_new.data_ptr(), v_new.data_ptr()
        a.kn_stride, a.vn_stride = N.strides3(k_new, _BSHD), N.strides3(v_new, _BSHD)
        a.seqlen_new = k_new.shape[1]
    if cos is not None:
        a.rotary_cos, a.rotary_sin = cos.data_ptr(), sin.data_ptr()
        a.rotary_dim, a.rotary_seqlen = cos.shape[-1] * 2, cos.shape[0]
        a.rotary_interleaved = int(bool(rotary_interleaved))
    a.softmax_scale = float(scale if scale is not None else D ** -0.5)
    a.causal = int(bool(causal))
    a.window_left = a.window_right = -1
    a.num_splits = int(num_splits)
    with torch.cuda.device(q.device):
        N.check(N.lib().fa_decode_paged_static(C.byref(a), N.stream_ptr(q.device)),
                "fa_decode_paged_static")
    return out
