"""The reference's operator layer, `flash_attn_triton/triton_kernel/attention_kernel.py`: the two
functions its public wrappers call, with the same names, argument order, defaults and errors, on
the sm_100a kernels.

* `attention` (attention_kernel.py:1201-1259): head-major (batch, heads, seqlen, head_dim) tensors
  of equal, 64-aligned sequence length; `seq_len_k` masks the padded keys, `seq_len_q` shifts the
  query positions by `seq_len_k - seq_len_q` (what the cross wrapper passes for its causal offset,
  flash_attn_interface.py:321-322); `dropout_seed` fixes the Philox seed.
* `attention_varlen` (attention_kernel.py:1364-1380): packed (tokens, heads, head_dim) tensors.

Differences: nothing is padded or copied (the masks are applied by the kernels, the tensors are
read through their strides), bf16 is accepted, and the 64-alignment of the reference's tiling is
not needed by the kernels but is still enforced so that a caller sees the reference's errors.
"""
from __future__ import annotations

import math
import random

import torch

from . import _native as N
from . import _ops


def attention(q, k, v, causal=False, sm_scale=None, dropout_p=0.0, dropout_seed=None,
              seq_len_k=None, seq_len_q=None, kv_heads=None, softcap=0.0, alibi_slopes=None,
              window_left=-1, window_right=-1, use_alibi=None):
    if sm_scale is None:
        sm_scale = 1.0 / math.sqrt(q.shape[-1])
    if q.shape[2] != k.shape[2] or k.shape[2] != v.shape[2]:
        raise ValueError("The low-level attention kernel requires equal sequence lengths")
    if q.shape[2] % 64 != 0:
        raise ValueError("The low-level attention kernel requires sequence lengths divisible by 64")
    if kv_heads is None:
        kv_heads = k.shape[1]
    if q.shape[1] % kv_heads != 0:
        raise ValueError("The number of query heads must be divisible by KV heads")
    if k.shape[1] != kv_heads or v.shape[1] != kv_heads:
        raise ValueError("k and v must carry kv_heads heads")
    if alibi_slopes is None or use_alibi is False:
        alibi = None
    else:
        alibi = torch.as_tensor(alibi_slopes, device=q.device, dtype=torch.float32).contiguous()
        if alibi.ndim == 1:
            alibi = alibi.unsqueeze(0).expand(q.shape[0], -1).contiguous()
    if dropout_seed is None:
        dropout_seed = random.randrange(2 ** 31 - 1)
    n_ctx = q.shape[2]
    seq_len_k = n_ctx if seq_len_k is None else int(seq_len_k)
    seq_len_q = n_ctx if seq_len_q is None else int(seq_len_q)
    if not 0 < seq_len_k <= n_ctx:
        raise ValueError("seq_len_k must lie in (0, seqlen]")
    # keys past seq_len_k are padding: a view of the first seq_len_k rows is all the kernels read
    kk, vv = k[:, :, :seq_len_k], v[:, :, :seq_len_k]
    feat = None
    if dropout_p:
        # counters of the reference: row * N_CTX + col over the PADDED length (attention_kernel.py:345-358)
        feat = _ops.Features(dropout_p=dropout_p, seed=int(dropout_seed), row_stride=n_ctx)
    return _ops.DenseAttention.apply(q, kk, vv, sm_scale, bool(causal), int(window_left), int(window_right),
                                     float(softcap), alibi, seq_len_k - seq_len_q, N.IMPL_AUTO, "bhsd", feat)


def attention_varlen(q, k, v, cu_seqlens_q, cu_seqlens_k, max_seqlen_q, max_seqlen_k, causal=False,
                     sm_scale=None, dropout_p=0.0, dropout_seed=None, softcap=0.0, alibi_slopes=None,
                     window_left=-1, window_right=-1, use_alibi=None):
    if sm_scale is None:
        sm_scale = 1.0 / math.sqrt(q.shape[-1])
    if dropout_seed is None:
        dropout_seed = random.randrange(2 ** 31 - 1)
    batch = cu_seqlens_q.numel() - 1
    if alibi_slopes is None or use_alibi is False:
        alibi = None
    else:
        alibi = torch.as_tensor(alibi_slopes, device=q.device, dtype=torch.float32)
        if alibi.ndim == 1:
            alibi = alibi.unsqueeze(0).expand(batch, -1)
        alibi = alibi.contiguous()
    feat = None
    if dropout_p:
        feat = _ops.Features(dropout_p=dropout_p, seed=int(dropout_seed), row_stride=int(max_seqlen_k))
    cu_q = cu_seqlens_q.to(dtype=torch.int32).contiguous()
    cu_k = cu_seqlens_k.to(dtype=torch.int32).contiguous()
    return _ops.VarlenAttention.apply(q, k, v, cu_q, cu_k, int(max_seqlen_q), int(max_seqlen_k), sm_scale,
                                      bool(causal), int(window_left), int(window_right), float(softcap), alibi,
                                      N.IMPL_AUTO, feat)
