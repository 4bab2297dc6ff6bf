"""Public API: the same functions, argument names, defaults and ValueErrors as the
reference's flash_attn_triton/flash_attn_interface.py, on top of the sm_100a kernels.

What is different underneath (results are the same within fp16 tolerance):
* tensors are handed to the kernels in place -- no pad-to-64, no head-major transposes,
  no repeat_interleave for GQA (reference: flash_attn_interface.py:168-212, :300-317);
* `flash_attn_with_kvcache` really appends to the cache, in place, and runs as one launch
  chain (no host synchronisation once the value checks are off, see set_validation; the reference
  loops over the batch in Python, :501-525, and its append at :487-492 writes into a temporary);
* bf16 is accepted as well as fp16;
* `use_native_gqa` and `deterministic` are accepted and change nothing: GQA is always native
  and the backward always has a single writer per element.
* `return_attn_probs`, `attn_bias`, `dropout_p`, `seqused_q/k` and paged packed K/V run on the
  kernels too (the reference materialises them in torch, :15-49, :139-148, :533-581, :642-659):
  the probabilities come from a kernel of their own, the bias and the dropout mask (the
  reference's Philox stream, attention_kernel.py:345-358) are applied inside the mma.sync
  kernels, the length overrides are read by every kernel, pages are gathered by a row mover;
* fp32 tensors are computed with fp16 operands and fp32 accumulation (the precision of the
  TF32 products the reference's fp32 path uses) and returned as fp32; values beyond the fp16
  range are not supported there.
"""
from __future__ import annotations

import math
import os
import random

import torch

from . import _native as N
from . import _ops

_VALIDATE = os.environ.get("FA_B200_VALIDATE", "1") != "0"


def set_validation(enabled: bool) -> None:
    """Turn the value checks that need a device->host sync (page indices in range, lengths
    fit the cache, cu_seqlens monotone ...) on or off.  Shape/dtype checks always run."""
    global _VALIDATE
    _VALIDATE = bool(enabled)


_KERNEL_DTYPES = (torch.float16, torch.bfloat16)
_ALL_DTYPES = (torch.float16, torch.bfloat16, torch.float32)


def _as_kernel_dtype(*tensors):
    """fp32 tensors are computed at fp16 operand precision (see the module docstring)."""
    if tensors[0].dtype == torch.float32:
        return tuple(t.to(torch.float16) for t in tensors)
    return tensors


def _dense_features(q, k, dropout_p, attn_bias):
    """Bias and dropout settings of a dense call, or None when neither is used."""
    if attn_bias is None and not dropout_p:
        return None
    bias = None
    if attn_bias is not None:
        if attn_bias.requires_grad:
            raise ValueError("attn_bias gradients are not produced; pass a tensor that does not require grad")
        B, Sq, Hq = q.shape[0], q.shape[1], q.shape[2]
        bias = attn_bias.detach().to(device=q.device, dtype=torch.float32)
        try:
            bias = bias.expand(B, Hq, Sq, k.shape[1])          # broadcast dimensions get stride 0
        except RuntimeError:
            raise ValueError("attn_bias must be broadcastable to (batch, nheads, seqlen_q, seqlen_k)")
    seed = row_stride = 0
    if dropout_p:
        # one seed per call (attention_kernel.py:1238-1239); the counter of element (row, col) uses the
        # sequence length the reference pads to: the next multiple of 64 of the longer side (:168-184, :300-307)
        seed = random.randrange(2 ** 31 - 1)
        row_stride = (max(q.shape[1], k.shape[1]) + 63) // 64 * 64
    return _ops.Features(bias=bias, dropout_p=dropout_p, seed=seed, row_stride=row_stride)


def _dense_call(q, k, v, dropout_p, softmax_scale, causal, window_size, softcap, alibi_slopes, attn_bias,
                return_attn_probs, q_pos_offset):
    out_dtype = q.dtype
    q, k, v = _as_kernel_dtype(q, k, v)
    if softmax_scale is None:
        softmax_scale = 1.0 / math.sqrt(q.shape[-1])
    feat = _dense_features(q, k, dropout_p, attn_bias)
    args = (softmax_scale, causal, window_size[0], window_size[1], softcap, alibi_slopes, int(q_pos_offset))
    if not return_attn_probs:
        return _ops.DenseAttention.apply(q, k, v, *args, N.IMPL_AUTO, "bshd", feat).to(out_dtype)
    out, lse2 = _ops.DenseAttention.apply(q, k, v, *args, N.IMPL_AUTO, "bshd", feat, True)
    probs, lse = _ops.dense_probs(q.detach(), k.detach(), v.detach(), lse2, *args, "bshd", feat)
    return out.to(out_dtype), lse, probs


def _raise_first(checks):
    """checks: [(0-d bool tensor on the device, message)] in order of precedence.  One reduction and
    ONE device->host read decide whether any of them is set; only then are they looked at one by one."""
    if not checks:
        return
    if bool(torch.stack([c for c, _ in checks]).any()):
        for c, msg in checks:
            if bool(c):
                raise ValueError(msg)


def _normalise_alibi(alibi_slopes, batch, heads, device):
    """(nheads,) or (batch, nheads) -> contiguous fp32 (batch, nheads); None stays None."""
    if alibi_slopes is None:
        return None
    alibi_slopes = torch.as_tensor(alibi_slopes, device=device, dtype=torch.float32)
    if alibi_slopes.ndim == 1:
        if alibi_slopes.shape[0] != heads:
            raise ValueError("alibi_slopes must have one value per query head")
        alibi_slopes = alibi_slopes.unsqueeze(0).expand(batch, -1)
    elif alibi_slopes.shape != (batch, heads):
        raise ValueError("alibi_slopes must have shape (nheads,) or (batch, nheads)")
    return alibi_slopes.contiguous()


def _check_head_dim(d):
    if d not in (16, 32, 64, 128, 256):
        raise ValueError("head dimension must be one of 16, 32, 64, 128, or 256")


def flash_attn_func(q, k, v, dropout_p=0.0, softmax_scale=None, causal=False,
                    window_size=(-1, -1), softcap=0.0, alibi_slopes=None,
                    deterministic=False, return_attn_probs=False, use_native_gqa=False,
                    attn_bias=None):
    """Attention over (batch, seqlen, nheads, headdim) tensors; k/v may have fewer heads
    (GQA/MQA) and a different sequence length (upper-left aligned masks).
    Same contract as the reference's flash_attn_func (flash_attn_interface.py:68-246)."""
    if q.dtype not in _ALL_DTYPES:
        raise ValueError("This implementation supports FP16, BF16 and FP32 tensors")
    if softcap < 0.0:
        raise ValueError("softcap must be non-negative")
    if dropout_p < 0.0 or dropout_p >= 1.0:
        raise ValueError("dropout_p must be in the range [0, 1)")
    if not (q.is_cuda and k.is_cuda and v.is_cuda):
        raise ValueError("All attention tensors must be CUDA tensors")
    if q.ndim != 4 or k.ndim != 4 or v.ndim != 4:
        raise ValueError("q, k, and v must have shape (batch, seqlen, heads, headdim)")
    if q.dtype != k.dtype or q.dtype != v.dtype:
        raise ValueError("q, k, and v must have the same dtype")
    if q.device != k.device or q.device != v.device:
        raise ValueError("q, k, and v must be on the same CUDA device")
    batch_size, seq_len_q, n_heads_q, head_dim = q.shape
    key_batch_size, seq_len_k, n_heads_k, key_head_dim = k.shape
    value_batch_size, value_seq_len, value_heads, value_head_dim = v.shape
    if key_batch_size != batch_size or value_batch_size != batch_size:
        raise ValueError("q, k, and v must have the same batch size")
    if value_seq_len != seq_len_k:
        raise ValueError("k and v must have the same sequence length")
    if key_head_dim != head_dim or value_head_dim != head_dim:
        raise ValueError("q, k, and v must have the same head dimension")
    if value_heads != n_heads_k:
        raise ValueError("k and v must have the same number of heads")
    if n_heads_k == 0 or n_heads_q % n_heads_k != 0:
        raise ValueError(
            f"Number of heads in Q ({n_heads_q}) must be divisible by number of heads in K/V ({n_heads_k})"
        )
    alibi_slopes = _normalise_alibi(alibi_slopes, batch_size, n_heads_q, q.device)

    _check_head_dim(head_dim)
    return _dense_call(q, k, v, dropout_p, softmax_scale, causal, window_size, softcap, alibi_slopes,
                       attn_bias, return_attn_probs, 0)


def flash_attn_func_cross(q, k, v, dropout_p=0.0, softmax_scale=None, causal=False,
                          use_native_gqa=False, softcap=0.0, alibi_slopes=None,
                          window_size=(-1, -1), deterministic=False,
                          return_attn_probs=False, attn_bias=None, _causal_offset=0):
    """Cross-attention for unequal query and KV lengths (flash_attn_interface.py:249-330).
    Query row i sits at position i + _causal_offset (0 = upper-left alignment)."""
    if q.dtype not in _ALL_DTYPES or k.dtype != q.dtype or v.dtype != q.dtype:
        raise ValueError("flash_attn_func_cross supports matching FP16, BF16 or FP32 tensors")
    if not (q.is_cuda and k.is_cuda and v.is_cuda):
        raise ValueError("All attention tensors must be CUDA tensors")
    if q.ndim != 4 or k.ndim != 4 or v.ndim != 4:
        raise ValueError("q, k, and v must have shape (batch, seqlen, heads, headdim)")
    if q.device != k.device or q.device != v.device:
        raise ValueError("q, k, and v must be on the same CUDA device")
    if k.shape[0] != q.shape[0] or v.shape[:2] != k.shape[:2]:
        raise ValueError("q, k, and v have incompatible batch or sequence dimensions")
    if q.shape[-1] != k.shape[-1] or k.shape[-1] != v.shape[-1]:
        raise ValueError("q, k, and v must have the same head dimension")
    _check_head_dim(q.shape[-1])
    if k.shape[2] == 0 or q.shape[2] % k.shape[2] != 0 or v.shape[2] != k.shape[2]:
        raise ValueError("The number of query heads must be divisible by KV heads")
    if dropout_p < 0.0 or dropout_p >= 1.0:
        raise ValueError("dropout_p must be in the range [0, 1)")
    if softcap < 0.0:
        raise ValueError("softcap must be non-negative")
    alibi_slopes = _normalise_alibi(alibi_slopes, q.shape[0], q.shape[2], q.device)
    return _dense_call(q, k, v, dropout_p, softmax_scale, causal, window_size, softcap, alibi_slopes,
                       attn_bias, return_attn_probs, _causal_offset)


def flash_attn_qkvpacked_func(qkv, dropout_p=0.0, softmax_scale=None, causal=False,
                              window_size=(-1, -1), softcap=0.0, alibi_slopes=None,
                              deterministic=False, return_attn_probs=False, use_native_gqa=False,
                              attn_bias=None):
    """qkv: (batch, seqlen, 3, nheads, headdim).  The three slices are read in place through
    their strides (flash_attn_interface.py:337-371 copies them)."""
    if qkv.ndim != 5 or qkv.shape[2] != 3:
        raise ValueError("qkv must have shape (batch, seqlen, 3, nheads, headdim)")
    q, k, v = qkv.unbind(dim=2)
    return flash_attn_func(q, k, v, dropout_p, softmax_scale, causal, window_size, softcap,
                           alibi_slopes, deterministic, return_attn_probs, use_native_gqa, attn_bias)


def flash_attn_kvpacked_func(q, kv, dropout_p=0.0, softmax_scale=None, causal=False,
                             window_size=(-1, -1), softcap=0.0, alibi_slopes=None,
                             deterministic=False, return_attn_probs=False, use_native_gqa=False,
                             attn_bias=None):
    """q: (batch, seqlen_q, nheads, headdim); kv: (batch, seqlen_k, 2, nheads_k, headdim)
    (flash_attn_interface.py:374-406)."""
    if kv.ndim != 5 or kv.shape[2] != 2:
        raise ValueError("kv must have shape (batch, seqlen, 2, nheads_k, headdim)")
    k, v = kv.unbind(dim=2)
    return flash_attn_func(q, k, v, dropout_p, softmax_scale, causal, window_size, softcap,
                           alibi_slopes, deterministic, return_attn_probs, use_native_gqa, attn_bias)


def _as_i32(x, device):
    return torch.as_tensor(x, device=device).to(torch.int32).flatten().contiguous()


def flash_attn_with_kvcache(q, k_cache, v_cache, k=None, v=None, rotary_cos=None, rotary_sin=None,
                            cache_seqlens=None, cache_batch_idx=None, cache_leftpad=None,
                            block_table=None, softmax_scale=None, causal=False,
                            window_size=(-1, -1), rotary_interleaved=True, alibi_slopes=None,
                            num_splits=0):
    """Attention against a KV cache, optionally appending new k/v first (in place) with
    rotary embedding applied to the new keys and to q.

    Contract of the reference's flash_attn_with_kvcache (flash_attn_interface.py:409-525):
    q (batch, seqlen_q, nheads, d); cache (batch_cache, capacity, nheads_k, d) or paged
    (num_pages, page_size, nheads_k, d) with block_table (batch, max_pages);
    cache_seqlens = tokens already in the cache before this call.  The query rows are the
    last seqlen_q positions of the sequence after the append; causal, window and ALiBi are
    measured from there (also without `causal`: the reference only shifts the causal mask,
    flash_attn_interface.py:523).  `num_splits` (0 = automatic) is an extra tuning knob.

    With value checks on (the default) the call reads ONE flag back from the device (page indices
    in range, lengths fit the cache and the rotary tables, reduced on the device);
    `set_validation(False)` or FA_B200_VALIDATE=0 turns them off and the call then never
    synchronises."""
    paged = block_table is not None
    checks = []          # value checks, evaluated together just before the launch (one host read)
    if (rotary_cos is None) != (rotary_sin is None):
        raise ValueError("rotary_cos and rotary_sin must be supplied together")
    if q.ndim != 4 or k_cache.ndim != 4 or v_cache.ndim != 4:
        raise ValueError("q and KV caches must be rank-4 tensors")
    if k_cache.shape != v_cache.shape:
        raise ValueError("k_cache and v_cache must have the same shape")
    if not (q.is_cuda and k_cache.is_cuda and v_cache.is_cuda):
        raise ValueError("All attention tensors must be CUDA tensors")
    B = q.shape[0]
    dev = q.device
    if paged:
        if block_table.ndim != 2 or block_table.shape[0] != B:
            raise ValueError("block_table must have shape (batch, max_num_pages)")
        if block_table.dtype not in (torch.int32, torch.int64):
            raise ValueError("block_table must contain integer page indices")
        if cache_leftpad is not None:
            raise ValueError("cache_leftpad cannot be combined with paged KV caches")
        if cache_batch_idx is not None:
            raise ValueError("cache_batch_idx cannot be combined with paged KV caches")
        page_size = k_cache.shape[1]
        cache_capacity = block_table.shape[1] * page_size
        block_table = block_table.to(device=dev, dtype=torch.int32).contiguous()
        if _VALIDATE:
            checks.append((torch.any((block_table < 0) | (block_table >= k_cache.shape[0])),
                           "block_table contains an invalid physical page index"))
    else:
        cache_capacity = k_cache.shape[1]
    if q.shape[-1] != k_cache.shape[-1]:
        raise ValueError("q and KV cache dimensions are incompatible")
    if q.device != k_cache.device or q.device != v_cache.device:
        raise ValueError("q and KV caches must be on the same device")
    if q.dtype != k_cache.dtype or q.dtype != v_cache.dtype:
        raise ValueError("q and KV caches must have the same dtype")
    if q.dtype not in _KERNEL_DTYPES:
        raise ValueError("flash_attn_with_kvcache supports FP16 and BF16 tensors")
    _check_head_dim(q.shape[-1])
    if k_cache.shape[2] == 0 or q.shape[2] % k_cache.shape[2] != 0:
        raise ValueError("The number of query heads must be divisible by KV heads")
    if k_cache.stride(-1) != 1 or v_cache.stride(-1) != 1 or not (
            N.kernel_ready(k_cache) and N.kernel_ready(v_cache)):
        raise ValueError("KV caches must have a unit head-dim stride and 16-byte aligned rows")
    rows = None
    if cache_batch_idx is not None:
        rows = _as_i32(cache_batch_idx, dev)
        if rows.numel() != B:
            raise ValueError("cache_batch_idx must contain valid cache-row indices")
        if _VALIDATE:
            checks.append((torch.any((rows < 0) | (rows >= k_cache.shape[0])),
                           "cache_batch_idx must contain valid cache-row indices"))
    elif not paged and k_cache.shape[0] < B:
        raise ValueError("cache_batch_idx must contain valid cache-row indices")
    pads = None
    if cache_leftpad is not None:
        pads = _as_i32(cache_leftpad, dev)
        if pads.numel() != B:
            raise ValueError("cache_leftpad must contain one non-negative value per query batch")
        if _VALIDATE:
            checks.append((torch.any(pads < 0), "cache_leftpad must contain one non-negative value per query batch"))
    n_new = 0
    if k is not None or v is not None:
        if k is None or v is None or k.shape != v.shape:
            raise ValueError("k and v must be supplied together with matching shapes")
        if k.ndim != 4 or k.shape[0] != B or k.shape[2:] != k_cache.shape[2:]:
            raise ValueError("new k/v tensors are incompatible with the cache")
        if k.dtype != q.dtype or v.dtype != q.dtype:
            raise ValueError("q and KV caches must have the same dtype")
        n_new = k.shape[1]
        if cache_seqlens is None:
            cache_seqlens = torch.zeros(B, dtype=torch.int32, device=dev)
        lengths = _as_i32(cache_seqlens, dev)
        if lengths.numel() != B:
            raise ValueError("new KV tensors do not fit in the cache")
        if _VALIDATE:
            total = lengths.long() + n_new + (pads.long() if pads is not None else 0)
            checks.append((torch.any((lengths < 0) | (total > cache_capacity)), "new KV tensors do not fit in the cache"))
        if n_new == 0:
            k = v = None
    else:
        if cache_seqlens is None:
            lengths = torch.full((B,), cache_capacity, dtype=torch.int32, device=dev)
        else:
            lengths = _as_i32(cache_seqlens, dev)
        if lengths.numel() != B:
            raise ValueError("cache_seqlens must contain valid lengths for every batch item")
        if _VALIDATE:
            total = lengths.long() + (pads.long() if pads is not None else 0)
            checks.append((torch.any((lengths < 0) | (total > cache_capacity)),
                           "cache_seqlens must contain valid lengths for every batch item"))
    cos = sin = None
    if rotary_cos is not None:
        if rotary_cos.shape != rotary_sin.shape or rotary_cos.ndim != 2:
            raise ValueError("rotary_cos and rotary_sin must be (seqlen_ro, rotary_dim / 2)")
        if rotary_cos.shape[-1] * 2 > q.shape[-1]:
            raise ValueError("rotary tables exceed the head dimension")
        if _VALIDATE:
            # every rotated position (new keys and query rows) must have a table row
            last = lengths.long() + n_new + (pads.long() if pads is not None else 0)
            checks.append((torch.any(last > rotary_cos.shape[0]),
                           "rotary tables are shorter than the longest sequence after the append"))
        cos = rotary_cos.to(device=dev, dtype=q.dtype).contiguous()
        sin = rotary_sin.to(device=dev, dtype=q.dtype).contiguous()
    alibi = _normalise_alibi(alibi_slopes, B, q.shape[2], dev)
    _raise_first(checks)
    if B == 0 or q.shape[1] == 0:
        return q.new_empty(q.shape)
    if softmax_scale is None:
        softmax_scale = 1.0 / math.sqrt(q.shape[-1])
    return _ops.kvcache_decode(q, k_cache, v_cache, k, v, cos, sin, lengths, rows, pads,
                               block_table, softmax_scale, causal, window_size[0], window_size[1],
                               rotary_interleaved, alibi, num_splits)


def flash_attn_varlen_func(q, k, v, cu_seqlens_q, cu_seqlens_k, max_seqlen_q, max_seqlen_k,
                           dropout_p=0.0, softmax_scale=None, causal=False, window_size=(-1, -1),
                           softcap=0.0, alibi_slopes=None, deterministic=False,
                           return_attn_probs=False, block_table=None, seqused_q=None,
                           seqused_k=None, **kwargs):
    """Attention over packed variable-length sequences (flash_attn_interface.py:527-690):
    q (total_q, nheads, d), k/v (total_k, nheads_k, d), int32 cu_seqlens on the device.
    Each sequence is masked with upper-left alignment."""
    batch_size = cu_seqlens_q.numel() - 1
    paged = block_table is not None
    if paged:
        k, v = _gather_pages(k, v, block_table, cu_seqlens_k, max_seqlen_k)
    used_q = used_k = None
    if seqused_q is not None:
        used_q = torch.as_tensor(seqused_q, device=q.device).to(torch.int32).flatten().contiguous()
        if used_q.numel() != batch_size:
            raise ValueError("seqused_q must contain one value per sequence")
    if seqused_k is not None:
        used_k = torch.as_tensor(seqused_k, device=q.device).to(torch.int32).flatten().contiguous()
        if used_k.numel() != batch_size:
            raise ValueError("seqused_k must contain one value per sequence")
    if _VALIDATE and (used_q is not None or used_k is not None):
        checks = []
        if used_q is not None:
            lq = (cu_seqlens_q[1:] - cu_seqlens_q[:-1]).to(q.device)
            checks.append((torch.any((used_q < 0) | (used_q > lq)), "seqused_q exceeds the packed query sequence"))
        if used_k is not None:
            lk = (cu_seqlens_k[1:] - cu_seqlens_k[:-1]).to(q.device)
            checks.append((torch.any((used_k < 0) | (used_k > lk)), "seqused_k exceeds the packed KV sequence"))
        _raise_first(checks)
    if q.ndim != 3 or k.ndim != 3 or v.ndim != 3 or k.shape != v.shape:
        raise ValueError("packed q, k, and v must be rank-3 tensors with matching KV shapes")
    if cu_seqlens_q.ndim != 1 or cu_seqlens_k.ndim != 1:
        raise ValueError("cu_seqlens arrays must be one-dimensional")
    if cu_seqlens_q.numel() != cu_seqlens_k.numel():
        raise ValueError("cu_seqlens_q and cu_seqlens_k must describe the same batch size")
    if cu_seqlens_q.numel() < 2:
        raise ValueError("cu_seqlens arrays must describe at least one sequence")
    if q.dtype not in _ALL_DTYPES or k.dtype != q.dtype or v.dtype != q.dtype:
        raise ValueError("flash_attn_varlen_func supports matching FP16, BF16 or FP32 tensors")
    if not (q.is_cuda and k.is_cuda and v.is_cuda):
        raise ValueError("All attention tensors must be CUDA tensors")
    if q.device != k.device or q.device != v.device:
        raise ValueError("q, k, and v must be on the same CUDA device")
    if q.shape[-1] != k.shape[-1] or k.shape[-1] != v.shape[-1]:
        raise ValueError("q, k, and v must have the same head dimension")
    _check_head_dim(q.shape[-1])
    if k.shape[1] == 0 or q.shape[1] % k.shape[1] != 0:
        raise ValueError("The number of query heads must be divisible by KV heads")
    if dropout_p < 0.0 or dropout_p >= 1.0:
        raise ValueError("dropout_p must be in the range [0, 1)")
    if softcap < 0.0:
        raise ValueError("softcap must be non-negative")
    if cu_seqlens_q.device != q.device or cu_seqlens_k.device != q.device:
        raise ValueError("cu_seqlens arrays must be on the same CUDA device as q, k, and v")
    if max_seqlen_q < 0 or max_seqlen_k < 0:
        raise ValueError("max sequence lengths must be non-negative")
    cu_seqlens_q = cu_seqlens_q.to(dtype=torch.int32).contiguous()
    cu_seqlens_k = cu_seqlens_k.to(dtype=torch.int32).contiguous()
    if _VALIDATE:
        # one device->host transfer for every value check the reference makes (:588-626)
        both = torch.cat((cu_seqlens_q, cu_seqlens_k)).tolist()
        cq, ck = both[:batch_size + 1], both[batch_size + 1:]
        if cq[0] != 0 or ck[0] != 0:
            raise ValueError("cu_seqlens arrays must start at zero and contain a batch boundary")
        if any(b < a for a, b in zip(cq, cq[1:])) or any(b < a for a, b in zip(ck, ck[1:])):
            raise ValueError("cu_seqlens arrays must be monotonically non-decreasing")
        # gathered pages are sized by batch * max_seqlen_k, an upper bound of cu_seqlens_k[-1]
        if cq[-1] != q.shape[0] or (ck[-1] > k.shape[0] if paged else ck[-1] != k.shape[0]):
            raise ValueError("cu_seqlens arrays must cover the packed q and KV tensors")
        if max_seqlen_q < max(b - a for a, b in zip(cq, cq[1:])) or \
                max_seqlen_k < max(b - a for a, b in zip(ck, ck[1:])):
            raise ValueError("max sequence lengths must cover every packed sequence")
    if max_seqlen_q == 0 or max_seqlen_k == 0:
        return q.new_zeros((q.shape[0], q.shape[1], q.shape[2]))
    alibi = _normalise_alibi(alibi_slopes, batch_size, q.shape[1], q.device)
    out_dtype = q.dtype
    q, k, v = _as_kernel_dtype(q, k, v)
    if softmax_scale is None:
        softmax_scale = 1.0 / math.sqrt(q.shape[-1])
    if dropout_p and deterministic and not return_attn_probs:
        # The reference's deterministic path runs every sequence through its dense kernel
        # (:660-681): one seed draw and dense dropout counters per sequence.  The kernels here
        # are deterministic either way, so only this combination needs the same walk to
        # reproduce the reference's masks.
        if used_q is not None or used_k is not None:
            q, cu_seqlens_q = (_compact_rows(q, cu_seqlens_q, used_q), _cu_of(used_q)) if used_q is not None \
                else (q, cu_seqlens_q)
            if used_k is not None:
                k, v = _compact_rows(k, cu_seqlens_k, used_k), _compact_rows(v, cu_seqlens_k, used_k)
                cu_seqlens_k = _cu_of(used_k)
        both = torch.cat((cu_seqlens_q, cu_seqlens_k)).tolist()
        cq, ck = both[:batch_size + 1], both[batch_size + 1:]
        outs = []
        for i in range(batch_size):
            qp, kp, vp = q[cq[i]:cq[i + 1]], k[ck[i]:ck[i + 1]], v[ck[i]:ck[i + 1]]
            if qp.shape[0] == 0:
                outs.append(qp.new_empty((0, q.shape[1], q.shape[2])))
            elif kp.shape[0] == 0:
                outs.append(qp.new_zeros((qp.shape[0], q.shape[1], q.shape[2])))
            else:
                outs.append(_dense_call(qp.unsqueeze(0), kp.unsqueeze(0), vp.unsqueeze(0), dropout_p, softmax_scale,
                                        causal, window_size, softcap,
                                        None if alibi is None else alibi[i:i + 1], None, False, 0).squeeze(0))
        return torch.cat(outs, dim=0).to(out_dtype)
    if dropout_p and used_q is not None:
        # The reference packs the used query rows before it launches (:552-566), so its dropout
        # counters run over the packed rows.  Do the same here, for this combination only.
        q = _compact_rows(q, cu_seqlens_q, used_q)
        cu_seqlens_q = _cu_of(used_q)
        used_q = None
        compacted = True
    else:
        compacted = False
    feat = None
    if dropout_p or used_q is not None or used_k is not None:
        # dropout counters follow the reference: (first packed row of the sequence + row) * max_seqlen_k + col
        # (attention_kernel.py:91-93)
        feat = _ops.Features(dropout_p=dropout_p, seed=random.randrange(2 ** 31 - 1) if dropout_p else 0,
                             row_stride=int(max_seqlen_k), seqused_q=used_q, seqused_k=used_k)
    args = (cu_seqlens_q, cu_seqlens_k, int(max_seqlen_q), int(max_seqlen_k), softmax_scale, causal,
            window_size[0], window_size[1], softcap, alibi)
    if return_attn_probs:
        out, lse2 = _ops.VarlenAttention.apply(q, k, v, *args, N.IMPL_AUTO, feat, True)
        probs, lse = _ops.varlen_probs(q.detach(), k.detach(), v.detach(), lse2, *args, feat)
    else:
        out = _ops.VarlenAttention.apply(q, k, v, *args, N.IMPL_AUTO, feat)
    if used_q is not None and not compacted:
        # the reference returns only the used rows, packed (flash_attn_interface.py:552-566); the one
        # host read of the lengths sizes that result
        out = _compact_rows(out, cu_seqlens_q, used_q)
    out = out.to(out_dtype)
    return (out, lse, probs) if return_attn_probs else out


def _cu_of(lengths):
    return torch.cat([lengths.new_zeros(1), torch.cumsum(lengths, 0, dtype=torch.int32)])


def _compact_rows(x, cu_seqlens, used):
    """Rows [cu[b], cu[b] + used[b]) of every sequence b, concatenated (differentiable gather)."""
    from .compat.bert_padding import index_first_axis
    used64 = used.to(torch.int64)
    total = int(used64.sum().item())
    starts_out = torch.cumsum(used64, 0) - used64
    seq = torch.repeat_interleave(torch.arange(used.numel(), device=x.device), used64, output_size=total)
    idx = cu_seqlens[:-1].to(torch.int64)[seq] + (torch.arange(total, device=x.device) - starts_out[seq])
    if total == 0:
        return x[:0]
    return index_first_axis(x, idx)


def _gather_pages(k, v, block_table, cu_seqlens_k, max_seqlen_k):
    """Paged K/V (pages, page_size, heads, dim) + block_table (batch, max_pages) -> packed
    (rows, heads, dim) tensors laid out by cu_seqlens_k, with a row mover on the device and no
    host read (flash_attn_interface.py:533-550 loops over the batch in Python).  The packed
    tensors get batch * max_seqlen_k rows, an upper bound of cu_seqlens_k[-1]; rows past it are
    zero and never read."""
    from .compat.bert_padding import index_first_axis
    if k.ndim != 4 or v.ndim != 4 or k.shape != v.shape:
        raise ValueError("paged varlen k and v must have shape (pages, page_size, heads, dim)")
    batch = cu_seqlens_k.numel() - 1
    if block_table.ndim != 2 or block_table.shape[0] != batch:
        raise ValueError("block_table must have shape (batch, max_num_pages)")
    if max_seqlen_k < 0:
        raise ValueError("max sequence lengths must be non-negative")
    page_size = k.shape[1]
    dev = k.device
    if _VALIDATE and bool(torch.any(block_table < 0) | torch.any(block_table >= k.shape[0])):
        raise ValueError("block_table contains an invalid physical page index")
    cu = cu_seqlens_k.to(device=dev, dtype=torch.int64)
    rows = batch * int(max_seqlen_k)
    t = torch.arange(rows, device=dev)
    seq = torch.searchsorted(cu[1:].contiguous(), t, right=True).clamp_(max=batch - 1)
    pos = t - cu[seq]
    page = block_table.to(device=dev, dtype=torch.int64)[seq, (pos // page_size).clamp_(0, block_table.shape[1] - 1)]
    idx = torch.where(t < cu[-1], page * page_size + pos % page_size, torch.full_like(t, -1))
    flat = lambda x: x.reshape(-1, x.shape[2], x.shape[3])
    return index_first_axis(flat(k), idx), index_first_axis(flat(v), idx)


def flash_attn_varlen_kvpacked_func(q, kv, cu_seqlens_q, cu_seqlens_k, max_seqlen_q,
                                    max_seqlen_k, dropout_p=0.0, softmax_scale=None,
                                    causal=False, **kwargs):
    """kv: (total_k, 2, nheads_k, d) (flash_attn_interface.py:692-699)."""
    k, v = kv.unbind(dim=1)
    return flash_attn_varlen_func(q, k, v, cu_seqlens_q, cu_seqlens_k, max_seqlen_q, max_seqlen_k,
                                  dropout_p=dropout_p, softmax_scale=softmax_scale, causal=causal,
                                  **kwargs)


def flash_attn_varlen_qkvpacked_func(qkv, cu_seqlens, max_seqlen, dropout_p=0.0,
                                     softmax_scale=None, causal=False, **kwargs):
    """qkv: (total, 3, nheads, d) (flash_attn_interface.py:702-708)."""
    q, k, v = qkv.unbind(dim=1)
    return flash_attn_varlen_func(q, k, v, cu_seqlens, cu_seqlens, max_seqlen, max_seqlen,
                                  dropout_p=dropout_p, softmax_scale=softmax_scale, causal=causal,
                                  **kwargs)


def attention_int8(q, k, v, causal=False, sm_scale=None, seq_len_k=None, seq_len_q=None):
    """INT8-QK^T attention on contiguous fp16 [B, H, S, D] tensors; fp16 backward.
    Same contract as the reference's attention_int8 (attention_kernel_int8.py:270-299) minus
    its Turing-only gate: this one runs on sm_100.  S must be a multiple of 64; a caller with
    another length pads q, k, v and passes the true lengths as seq_len_k / seq_len_q."""
    head_dim = q.shape[-1]
    if not q.is_cuda:
        raise ValueError("The INT8 kernel requires CUDA tensors")
    if q.dtype != torch.float16 or k.dtype != torch.float16 or v.dtype != torch.float16:
        raise ValueError("The INT8 kernel requires FP16 tensors")
    if head_dim < 32 or head_dim & (head_dim - 1):
        raise ValueError("The INT8 kernel requires a power-of-two head dim of at least 32")
    if q.shape[2] % 64:
        raise ValueError("The INT8 kernel requires sequence lengths divisible by 64")
    if not (q.is_contiguous() and k.is_contiguous() and v.is_contiguous()):
        raise ValueError("The INT8 kernel requires contiguous inputs")
    if q.shape[2] != k.shape[2] or k.shape[2] != v.shape[2]:
        raise ValueError("The INT8 kernel requires equal sequence lengths")
    if q.shape != k.shape or q.shape != v.shape:
        raise ValueError("The INT8 kernel requires q, k and v of the same shape")
    if sm_scale is None:
        sm_scale = 1.0 / math.sqrt(q.shape[-1])
    S = q.shape[2]
    seq_len_k = S if seq_len_k is None else int(seq_len_k)
    seq_len_q = S if seq_len_q is None else int(seq_len_q)
    if not 0 < seq_len_k <= S or not 0 < seq_len_q <= S:
        raise ValueError("seq_len_k and seq_len_q must lie in (0, padded sequence length]")
    # Padded calls (attention_kernel_int8.py:108-118, :245): keys at or past seq_len_k are masked and
    # the causal diagonal is shifted by seq_len_k - seq_len_q, in the forward and in the backward.
    return _ops.Int8Attention.apply(q, k, v, causal, sm_scale, N.IMPL_AUTO,
                                    seq_len_k if seq_len_k < S else 0, seq_len_k - seq_len_q)


class FlashSelfAttention(torch.nn.Module):
    """Self-attention over packed qkv (flash_attn_interface.py:711-736)."""

    def __init__(self, causal=False, softmax_scale=None, attention_dropout=0.0,
                 window_size=(-1, -1), alibi_slopes=None, deterministic=False):
        super().__init__()
        self.causal = causal
        self.softmax_scale = softmax_scale
        self.drop = torch.nn.Dropout(attention_dropout)
        self.window_size = window_size
        self.alibi_slopes = alibi_slopes
        self.deterministic = deterministic

    def forward(self, qkv, causal=None, cu_seqlens=None, max_seqlen=None):
        dropout_p = self.drop.p if self.training else 0.0
        causal = self.causal if causal is None else causal
        if cu_seqlens is None:
            return flash_attn_qkvpacked_func(qkv, dropout_p, self.softmax_scale, causal,
                                             self.window_size, 0.0, self.alibi_slopes,
                                             self.deterministic)
        return flash_attn_varlen_qkvpacked_func(qkv, cu_seqlens, max_seqlen, dropout_p,
                                                self.softmax_scale, causal,
                                                window_size=self.window_size,
                                                alibi_slopes=self.alibi_slopes,
                                                deterministic=self.deterministic)


class FlashCrossAttention(torch.nn.Module):
    """Cross-attention over q and packed kv (flash_attn_interface.py:739-770)."""

    def __init__(self, causal=False, softmax_scale=None, attention_dropout=0.0,
                 window_size=(-1, -1), alibi_slopes=None, deterministic=False):
        super().__init__()
        self.causal = causal
        self.softmax_scale = softmax_scale
        self.drop = torch.nn.Dropout(attention_dropout)
        self.window_size = window_size
        self.alibi_slopes = alibi_slopes
        self.deterministic = deterministic

    def forward(self, q, kv, causal=None, cu_seqlens=None, max_seqlen=None, cu_seqlens_k=None,
                max_seqlen_k=None):
        dropout_p = self.drop.p if self.training else 0.0
        causal = self.causal if causal is None else causal
        if cu_seqlens is None:
            k, v = kv.unbind(dim=2)
            return flash_attn_func_cross(q, k, v, dropout_p, self.softmax_scale, causal,
                                         use_native_gqa=not self.training, softcap=0.0,
                                         alibi_slopes=self.alibi_slopes,
                                         window_size=self.window_size,
                                         deterministic=self.deterministic)
        k, v = kv.unbind(dim=1)
        return flash_attn_varlen_func(q, k, v, cu_seqlens, cu_seqlens_k, max_seqlen, max_seqlen_k,
                                      dropout_p, self.softmax_scale, causal,
                                      window_size=self.window_size, alibi_slopes=self.alibi_slopes,
                                      deterministic=self.deterministic)


class FlashAttention(torch.nn.Module):
    """Module form of flash_attn_func (flash_attn_interface.py:773-804)."""

    def __init__(self, attention_dropout=0.0, softmax_scale=None):
        super().__init__()
        self.dropout_p = attention_dropout
        self.softmax_scale = softmax_scale

    def forward(self, q, k, v, causal=False, attn_bias=None):
        return flash_attn_func(q, k, v, dropout_p=self.dropout_p if self.training else 0.0,
                               softmax_scale=self.softmax_scale, causal=causal, attn_bias=attn_bias)
