"""CPU restatement of the reference attention arithmetic (luyanaa/flash-attn-triton).

TEST INFRASTRUCTURE ONLY.  This module is the checker for the CUDA kernels: only the
test-suite, the smoke check and the benchmark's CPU-baseline leg may import it.  The
product package never does; it fails loudly when its CUDA library is missing.

Everything here is plain fp32 torch on the CPU (dense matrices, no tiling), written
from the reference's own eager restatement and kernels:

* score pipeline and mask alignment .......... flash_attn_triton/flash_attn_interface.py:15-49
* rotary embedding ........................... flash_attn_triton/flash_attn_interface.py:52-66
* KV-cache append + attend (intended form) ... flash_attn_triton/flash_attn_interface.py:409-525
* packed variable-length batches ............. flash_attn_triton/triton_kernel/attention_kernel.py:27-104
* base-2 LSE saved for the backward .......... flash_attn_triton/triton_kernel/attention_kernel.py:522-533
* per-token INT8 K quantiser ................. flash_attn_triton/triton_kernel/attention_kernel_int8.py:27-30,58-79
* INT8 QK^T forward .......................... flash_attn_triton/triton_kernel/attention_kernel_int8.py:82-141,167-217
* rotary-embedding kernel (helper package) ... flash_attn/ops/triton/rotary.py:11-130
* un-padding / re-padding (helper package) ... flash_attn/bert_padding.py:98-213

Parity pin: tests/golden/*.npz hold outputs of the unmodified reference kernels run
under Triton's CPU interpreter (tests/golden/make_golden.py, make_golden_compat.py); tests/test_oracle_golden.py
checks every function below against them.
"""
from __future__ import annotations

import math

import numpy as np
import torch

LOG2E = 1.4426950408889634


# ----------------------------------------------------------------------------------------
# score pipeline (flash_attn_interface.py:15-49)
# ----------------------------------------------------------------------------------------
def keep_mask(q_len, k_len, causal, window, q_pos_offset=0):
    """Boolean (q_len, k_len) mask.  Query i sits at position i + q_pos_offset, key j at j;
    causal keeps j <= pos, the window keeps pos-left <= j <= pos+right
    (flash_attn_interface.py:27-35: upper-left alignment when the offset is 0)."""
    q_pos = torch.arange(q_len)[:, None] + q_pos_offset
    k_pos = torch.arange(k_len)[None, :]
    keep = torch.ones(q_len, k_len, dtype=torch.bool)
    if causal:
        keep &= q_pos >= k_pos
    if window[0] >= 0:
        keep &= k_pos >= q_pos - window[0]
    if window[1] >= 0:
        keep &= k_pos <= q_pos + window[1]
    return keep


def scores_ref(q, k, softmax_scale=None, causal=False, window=(-1, -1), softcap=0.0,
               alibi_slopes=None, attn_bias=None, q_pos_offset=0):
    """Masked fp32 scores (B, Hq, Sq, Sk) in the natural-log domain.

    Order of operations is the reference's contract (flash_attn_interface.py:26-43):
    scale -> minus slope*|i-j| -> plus bias -> softcap*tanh(s/softcap) -> -inf mask.
    q: (B, Sq, Hq, D), k: (B, Sk, Hkv, D)."""
    q = q.float()
    k = k.float()
    B, Sq, Hq, D = q.shape
    Sk, Hkv = k.shape[1], k.shape[2]
    if Hq != Hkv:
        k = k.repeat_interleave(Hq // Hkv, dim=2)
    scale = 1.0 / math.sqrt(D) if softmax_scale is None else softmax_scale
    s = torch.einsum("bqhd,bkhd->bhqk", q, k) * scale
    if alibi_slopes is not None:
        slopes = torch.as_tensor(alibi_slopes, dtype=torch.float32)
        slopes = slopes if slopes.ndim == 2 else slopes[None, :]
        q_pos = torch.arange(Sq)[:, None] + q_pos_offset
        k_pos = torch.arange(Sk)[None, :]
        s = s - slopes[:, :, None, None] * (q_pos - k_pos).abs()
    if attn_bias is not None:
        s = s + attn_bias.float()
    if softcap > 0:
        s = softcap * torch.tanh(s / softcap)
    keep = keep_mask(Sq, Sk, causal, window, q_pos_offset)
    return s.masked_fill(~keep[None, None], float("-inf"))


def attention_ref(q, k, v, softmax_scale=None, causal=False, window=(-1, -1), softcap=0.0,
                  alibi_slopes=None, attn_bias=None, q_pos_offset=0, p_dtype=None):
    """Dense attention.  Returns (out fp32 (B,Sq,Hq,D), lse natural-log (B,Hq,Sq)).

    Rows with no visible key give out = 0 and lse = -inf
    (flash_attn_interface.py:43-45; attention_kernel.py:522-533).
    p_dtype: when given, probabilities are rounded to that dtype before P@V, as the
    kernels do (attention_kernel.py:366)."""
    s = scores_ref(q, k, softmax_scale, causal, window, softcap, alibi_slopes, attn_bias,
                   q_pos_offset)
    probs = torch.nan_to_num(torch.softmax(s, dim=-1))
    lse = torch.logsumexp(s, dim=-1)
    vv = v.float()
    if q.shape[2] != v.shape[2]:
        vv = vv.repeat_interleave(q.shape[2] // v.shape[2], dim=2)
    if p_dtype is not None:
        probs = probs.to(p_dtype).float()
    out = torch.einsum("bhqk,bkhd->bqhd", probs, vv)
    return out, lse


# ----------------------------------------------------------------------------------------
# dropout with the reference's random stream (attention_kernel.py:345-358, :91-93, :641-652, :749-762)
# ----------------------------------------------------------------------------------------
def philox_uniform(seed, offsets):
    """tl.rand(seed, offset) restated: Philox4x32-10 with key = the 64-bit seed and counter
    (offset, 0, 0, 0); the first output word, read as a signed int, folded to non-negative
    (x < 0 -> -x - 1) and scaled by 2^-31.  offsets: integer array (wraps to 32 bits)."""
    c0 = np.asarray(offsets).astype(np.uint64) & np.uint64(0xFFFFFFFF)
    c1 = np.zeros_like(c0)
    c2 = np.zeros_like(c0)
    c3 = np.zeros_like(c0)
    k0 = np.uint64(int(seed) & 0xFFFFFFFF)
    k1 = np.uint64((int(seed) >> 32) & 0xFFFFFFFF)
    A, B_, M = np.uint64(0xD2511F53), np.uint64(0xCD9E8D57), np.uint64(0xFFFFFFFF)
    for _ in range(10):
        pa, pb = A * c0, B_ * c2                      # 32 x 32 -> 64 bit products
        c0, c2, c1, c3 = (pb >> np.uint64(32)) ^ c1 ^ k0, (pa >> np.uint64(32)) ^ c3 ^ k1, pb & M, pa & M
        k0 = (k0 + np.uint64(0x9E3779B9)) & M
        k1 = (k1 + np.uint64(0xBB67AE85)) & M
    x = c0.astype(np.uint32).view(np.int32).astype(np.int64)
    x = np.where(x < 0, -x - 1, x)
    return (x.astype(np.float32) * np.float32(4.6566127342e-10)).astype(np.float32)


def dropout_keep_ref(q_len, k_len, p, seed, row_stride, row0=0):
    """Keep mask (q_len, k_len): element (i, j) is kept when the uniform drawn at counter
    (row0 + i) * row_stride + j exceeds p.  Dense calls use row0 = 0 and row_stride = the longer
    sequence length rounded up to 64 (the length the reference pads to); packed calls use
    row0 = cu_seqlens_q[b] and row_stride = max_seqlen_k."""
    off = (np.arange(q_len, dtype=np.int64)[:, None] + row0) * row_stride + np.arange(k_len, dtype=np.int64)[None, :]
    return torch.from_numpy(philox_uniform(seed, off) > np.float32(p))


def attention_dropout_ref(q, k, v, dout=None, dropout_p=0.0, seed=0, row_stride=None, row0=0, **kw):
    """Dense attention with dropout, forward and (when dout is given) the gradients AS THE
    REFERENCE'S KERNELS COMPUTE THEM: P is normalised before the mask is applied, kept entries are
    scaled by 1/(1-p), and the backward multiplies (dP - delta) by the dropped-and-rescaled P
    (attention_kernel.py:652-664, :760-762) -- not the exact derivative, whose delta term uses
    the undropped P.  Returns (out, lse, probs_after_dropout[, dq, dk, dv]); layouts as attention_ref."""
    B, Sq, Hq, D = q.shape
    Sk, Hkv = k.shape[1], k.shape[2]
    scale = 1.0 / math.sqrt(D) if kw.get("softmax_scale") is None else kw["softmax_scale"]
    softcap = kw.get("softcap", 0.0)
    s = scores_ref(q, k, kw.get("softmax_scale"), kw.get("causal", False), kw.get("window", (-1, -1)), softcap,
                   kw.get("alibi_slopes"), kw.get("attn_bias"), kw.get("q_pos_offset", 0))
    probs = torch.nan_to_num(torch.softmax(s, dim=-1))
    lse = torch.logsumexp(s, dim=-1)
    if dropout_p > 0:
        if row_stride is None:
            row_stride = (max(Sq, Sk) + 63) // 64 * 64
        keep = dropout_keep_ref(Sq, Sk, dropout_p, seed, row_stride, row0)
        pd = torch.where(keep[None, None], probs / (1.0 - dropout_p), torch.zeros(()))
    else:
        pd = probs
    g = Hq // Hkv
    kf = k.float().repeat_interleave(g, dim=2)
    vf = v.float().repeat_interleave(g, dim=2)
    out = torch.einsum("bhqk,bkhd->bqhd", pd, vf)
    if dout is None:
        return out, lse, pd
    dof = dout.float()
    dv_full = torch.einsum("bhqk,bqhd->bkhd", pd, dof)
    dp = torch.einsum("bqhd,bkhd->bhqk", dof, vf)
    delta = (out * dof).sum(-1).transpose(1, 2)                      # (B, H, Sq)
    ds = pd * (dp - delta[..., None])
    if softcap > 0:
        # d(softcap * tanh(u / softcap)) / du = 1 - tanh^2, with the capped score s = softcap * tanh(.)
        ds = ds * (1.0 - (torch.nan_to_num(s, neginf=0.0) / softcap) ** 2)
    dq = torch.einsum("bhqk,bkhd->bqhd", ds, kf) * scale
    dk_full = torch.einsum("bhqk,bqhd->bkhd", ds, q.float()) * scale
    fold = lambda t: t.reshape(B, Sk, Hkv, g, D).sum(3)
    return out, lse, pd, dq, fold(dk_full), fold(dv_full)


def attention_grads_ref(q, k, v, dout, **kw):
    """(out, lse, dq, dk, dv) in fp32 by autograd through attention_ref.  GQA gradients of
    a KV head are the sum over its query heads (attention_kernel.py:188-272)."""
    q32 = q.detach().float().requires_grad_()
    k32 = k.detach().float().requires_grad_()
    v32 = v.detach().float().requires_grad_()
    out, lse = attention_ref(q32, k32, v32, **kw)
    dq, dk, dv = torch.autograd.grad((out * dout.float()).sum(), (q32, k32, v32))
    return out.detach(), lse.detach(), dq, dk, dv


def lse2_from_natural(lse):
    """Natural-log LSE -> the base-2 LSE the kernels save (attention_kernel.py:524)."""
    return lse * LOG2E


# ----------------------------------------------------------------------------------------
# packed variable-length batches (attention_kernel.py:27-104; interface.py:527-690)
# ----------------------------------------------------------------------------------------
def varlen_attention_ref(q, k, v, cu_q, cu_k, softmax_scale=None, causal=False,
                         window=(-1, -1), softcap=0.0, alibi_slopes=None):
    """q (Tq,Hq,D), k/v (Tk,Hkv,D); cu_* int (batch+1,).  Returns (out (Tq,Hq,D) fp32,
    lse natural (Tq,Hq)).  Each sequence is attended on its own with upper-left
    alignment (attention_kernel.py:47-48)."""
    cu_q = [int(x) for x in cu_q]
    cu_k = [int(x) for x in cu_k]
    batch = len(cu_q) - 1
    out = torch.zeros(q.shape, dtype=torch.float32)
    lse = torch.full((q.shape[0], q.shape[1]), float("-inf"))
    slopes = None
    if alibi_slopes is not None:
        slopes = torch.as_tensor(alibi_slopes, dtype=torch.float32)
        if slopes.ndim == 1:
            slopes = slopes[None, :].expand(batch, -1)
    for b in range(batch):
        qs, qe, ks, ke = cu_q[b], cu_q[b + 1], cu_k[b], cu_k[b + 1]
        if qe == qs:
            continue
        if ke == ks:
            continue
        o, l = attention_ref(q[qs:qe][None], k[ks:ke][None], v[ks:ke][None], softmax_scale,
                             causal, window, softcap,
                             None if slopes is None else slopes[b:b + 1])
        out[qs:qe] = o[0]
        lse[qs:qe] = l[0].transpose(0, 1)
    return out, lse


def varlen_attention_grads_ref(q, k, v, dout, cu_q, cu_k, **kw):
    q32 = q.detach().float().requires_grad_()
    k32 = k.detach().float().requires_grad_()
    v32 = v.detach().float().requires_grad_()
    out, lse = varlen_attention_ref(q32, k32, v32, cu_q, cu_k, **kw)
    dq, dk, dv = torch.autograd.grad((out * dout.float()).sum(), (q32, k32, v32),
                                     allow_unused=True)
    z = lambda g, t: torch.zeros_like(t) if g is None else g
    return out.detach(), lse.detach(), z(dq, q32), z(dk, k32), z(dv, v32)


def varlen_attention_dropout_ref(q, k, v, cu_q, cu_k, max_seqlen_k, dout=None, dropout_p=0.0, seed=0,
                                 alibi_slopes=None, **kw):
    """Packed attention with dropout: every sequence through attention_dropout_ref with the
    packed kernels' counters, (cu_q[b] + row) * max_seqlen_k + col (attention_kernel.py:91-93).
    Returns (out (Tq,Hq,D), lse (Tq,Hq), probs list per sequence (Hq,q_len,k_len)[, dq, dk, dv])."""
    cu_q = [int(x) for x in cu_q]
    cu_k = [int(x) for x in cu_k]
    batch = len(cu_q) - 1
    out = torch.zeros(q.shape, dtype=torch.float32)
    lse = torch.full((q.shape[0], q.shape[1]), float("-inf"))
    dq = torch.zeros(q.shape, dtype=torch.float32)
    dk = torch.zeros(k.shape, dtype=torch.float32)
    dv = torch.zeros(v.shape, dtype=torch.float32)
    probs = []
    slopes = None
    if alibi_slopes is not None:
        slopes = torch.as_tensor(alibi_slopes, dtype=torch.float32)
        if slopes.ndim == 1:
            slopes = slopes[None, :].expand(batch, -1)
    for b in range(batch):
        qs, qe, ks, ke = cu_q[b], cu_q[b + 1], cu_k[b], cu_k[b + 1]
        if qe == qs or ke == ks:
            probs.append(torch.zeros((q.shape[1], qe - qs, ke - ks)))
            continue
        r = attention_dropout_ref(q[qs:qe][None], k[ks:ke][None], v[ks:ke][None],
                                  None if dout is None else dout[qs:qe][None], dropout_p=dropout_p, seed=seed,
                                  row_stride=max_seqlen_k, row0=qs,
                                  alibi_slopes=None if slopes is None else slopes[b:b + 1], **kw)
        out[qs:qe] = r[0][0]
        lse[qs:qe] = r[1][0].transpose(0, 1)
        probs.append(r[2][0])
        if dout is not None:
            dq[qs:qe], dk[ks:ke], dv[ks:ke] = r[3][0], r[4][0], r[5][0]
    return (out, lse, probs) if dout is None else (out, lse, probs, dq, dk, dv)


def seqused_view(cu, used):
    """Index list of the rows a packed call with seqused lengths reads: rows
    [cu[b], cu[b] + used[b]) of every sequence, and the cu_seqlens of that packing
    (flash_attn_interface.py:552-581)."""
    cu = [int(x) for x in cu]
    used = [int(x) for x in used]
    idx = [cu[b] + i for b in range(len(used)) for i in range(used[b])]
    new_cu = [0]
    for u in used:
        new_cu.append(new_cu[-1] + u)
    return torch.tensor(idx, dtype=torch.long), new_cu


def unpage_ref(pages, block_table, cu_k):
    """Packed (Tk, H, D) rows of a paged tensor (pages, page_size, H, D): sequence b's tokens are
    the first cu_k[b+1]-cu_k[b] slots of its pages, in block_table order
    (flash_attn_interface.py:533-550)."""
    page = pages.shape[1]
    cu_k = [int(x) for x in cu_k]
    parts = []
    for b in range(len(cu_k) - 1):
        n = cu_k[b + 1] - cu_k[b]
        ids = block_table[b, :(n + page - 1) // page].long()
        parts.append(pages[ids].reshape(-1, pages.shape[2], pages.shape[3])[:n])
    return torch.cat(parts, dim=0)


# ----------------------------------------------------------------------------------------
# rotary + KV cache (flash_attn_interface.py:52-66, 409-525)
# ----------------------------------------------------------------------------------------
def apply_rotary_ref(x, cos, sin, positions, interleaved):
    """x (S,H,D) in its own dtype; cos/sin (seqlen_ro, rotary_dim/2); positions (S,) ints.
    The arithmetic is carried out in x's dtype, like the reference
    (flash_attn_interface.py:57-66)."""
    rotary_dim = cos.shape[-1] * 2
    c = cos[positions].to(x.dtype)[:, None, :]
    s = sin[positions].to(x.dtype)[:, None, :]
    part = x[..., :rotary_dim]
    if interleaved:
        even, odd = part[..., 0::2], part[..., 1::2]
        rot = torch.stack((even * c - odd * s, even * s + odd * c), dim=-1).flatten(-2)
    else:
        h = rotary_dim // 2
        a, b = part[..., :h], part[..., h:]
        rot = torch.cat((a * c - b * s, a * s + b * c), dim=-1)
    return torch.cat((rot, x[..., rotary_dim:]), dim=-1)


def kvcache_ref(q, k_cache, v_cache, k_new=None, v_new=None, cos=None, sin=None,
                cache_seqlens=None, cache_batch_idx=None, cache_leftpad=None,
                block_table=None, softmax_scale=None, causal=False, window=(-1, -1),
                rotary_interleaved=True, alibi_slopes=None, reference_alignment=False):
    """Append-then-attend against a contiguous or paged cache.

    This is the behaviour the reference's code is written to have
    (flash_attn_interface.py:468-525): rotate the new keys at positions
    len+leftpad+i, write new k/v into the cache at those slots, rotate q at
    len_after-Sq+leftpad+i and attend over the first len_after cached tokens.  (In the
    reference the two `cache[idx, idx].copy_` lines at :487-492 write into a temporary,
    so its cache stays stale; tests pin the reference by doing the append themselves.)
    Query rows are bottom-right aligned for the causal mask (offset len_after-Sq, :523);
    for window/ALiBi this oracle uses the same offset.  `reference_alignment=True` restates the
    reference instead: without `causal` it measures window and ALiBi from query position 0
    (flash_attn_interface.py:523 passes `_causal_offset=0`), which the library deliberately does
    not do.
    Returns (out fp32 (B,Sq,Hq,D), k_cache_after, v_cache_after)."""
    kc = k_cache.clone()
    vc = v_cache.clone()
    B, Sq = q.shape[0], q.shape[1]
    paged = block_table is not None
    page = kc.shape[1]
    lens = (torch.as_tensor(cache_seqlens).long().flatten() if cache_seqlens is not None else
            torch.full((B,), (block_table.shape[1] * page) if paged else kc.shape[1]).long())
    if cache_seqlens is None and k_new is not None:
        lens = torch.zeros(B, dtype=torch.long)
    pads = (torch.as_tensor(cache_leftpad).long().flatten() if cache_leftpad is not None
            else torch.zeros(B, dtype=torch.long))
    rows = (torch.as_tensor(cache_batch_idx).long().flatten() if cache_batch_idx is not None
            else torch.arange(B))
    outs = []
    for b in range(B):
        L, pad, row = int(lens[b]), int(pads[b]), int(rows[b])
        if k_new is not None:
            Sn = k_new.shape[1]
            kn = k_new[b]
            if cos is not None:
                kn = apply_rotary_ref(kn, cos, sin, torch.arange(Sn) + L + pad, rotary_interleaved)
            for i in range(Sn):
                pos = L + pad + i
                if paged:
                    pg = int(block_table[b, pos // page])
                    kc[pg, pos % page] = kn[i]
                    vc[pg, pos % page] = v_new[b, i]
                else:
                    kc[row, pos] = kn[i]
                    vc[row, pos] = v_new[b, i]
            L += Sn
        if paged:
            npages = (pad + L + page - 1) // page
            ids = block_table[b, :npages].long()
            kb = kc[ids].reshape(-1, kc.shape[2], kc.shape[3])[pad:pad + L]
            vb = vc[ids].reshape(-1, vc.shape[2], vc.shape[3])[pad:pad + L]
        else:
            kb = kc[row, pad:pad + L]
            vb = vc[row, pad:pad + L]
        qb = q[b]
        if cos is not None:
            qb = apply_rotary_ref(qb, cos, sin, torch.arange(Sq) + L - Sq + pad, rotary_interleaved)
        sl = None
        if alibi_slopes is not None:
            sl = torch.as_tensor(alibi_slopes, dtype=torch.float32)
            sl = sl[b:b + 1] if sl.ndim == 2 else sl[None]
        o, _ = attention_ref(qb[None], kb[None], vb[None], softmax_scale, causal, window, 0.0,
                             sl, q_pos_offset=0 if (reference_alignment and not causal) else L - Sq)
        outs.append(o)
    return torch.cat(outs, dim=0), kc, vc


# ----------------------------------------------------------------------------------------
# INT8 path (attention_kernel_int8.py)
# ----------------------------------------------------------------------------------------
def round_i8_np(x):
    """floor(x+0.5) for x>=0, ceil(x-0.5) otherwise, in IEEE fp32
    (attention_kernel_int8.py:27-30).  Not the same as rint or roundf at x=0.49999997."""
    x = np.asarray(x, dtype=np.float32)
    half = np.float32(0.5)
    r = np.where(x >= 0, np.floor(x + half), np.ceil(x - half))
    return r.astype(np.int8)


def quantize_k_rows_ref(k):
    """Per-key-token INT8 codes and fp32 scales (attention_kernel_int8.py:58-79).

    k: fp16 array/tensor (..., S, D).  amax in fp16 (exact), s = fp32(max(amax,1))/127,
    inv = 1/s, x = fp32(k)*inv, code = round_i8(x).  Every step is a single IEEE fp32
    operation, so numpy reproduces the kernel bit for bit."""
    kn = k.detach().cpu().numpy() if isinstance(k, torch.Tensor) else np.asarray(k)
    assert kn.dtype == np.float16
    amax = np.abs(kn).max(axis=-1).astype(np.float32)
    s = (np.maximum(amax, np.float32(1.0)) / np.float32(127.0)).astype(np.float32)
    inv = (np.float32(1.0) / s).astype(np.float32)
    x = (kn.astype(np.float32) * inv[..., None]).astype(np.float32)
    return round_i8_np(x), s


def quantize_q_rows_ref(q):
    """Per-query-row codes, division form q/s (attention_kernel_int8.py:33-39, :100)."""
    qn = q.detach().cpu().numpy() if isinstance(q, torch.Tensor) else np.asarray(q)
    amax = np.abs(qn).max(axis=-1).astype(np.float32)
    s = (np.maximum(amax, np.float32(1.0)) / np.float32(127.0)).astype(np.float32)
    x = (qn.astype(np.float32) / s[..., None]).astype(np.float32)
    return round_i8_np(x), s


def _int8_keep(S, causal, seq_len_k, seq_len_q):
    """Mask of a padded INT8 call (attention_kernel_int8.py:108-118): keys at or past seq_len_k
    are dropped, query row i sits at position i + seq_len_k - seq_len_q for the causal test."""
    seq_len_k = S if seq_len_k is None else seq_len_k
    seq_len_q = S if seq_len_q is None else seq_len_q
    keep = keep_mask(S, S, causal, (-1, -1), q_pos_offset=seq_len_k - seq_len_q)
    return keep & (torch.arange(S) < seq_len_k)[None, :]


def attention_int8_ref(q, k, v, causal=False, sm_scale=None, seq_len_k=None, seq_len_q=None):
    """INT8-QK^T forward in the reference's arithmetic.  q,k,v: fp16 (B,H,S,D).

    scores(log2) = float(int32 q8.k8) * (s_q*s_k) * (sm_scale*1.44269504)
    (attention_kernel_int8.py:106-107, :200); masked entries get -1.0e6 added, not -inf
    (:113); probabilities are rounded to fp16 before P@V (:135-137).
    Returns (out fp32 (B,H,S,D), lse base-2 (B,H,S), k8 int8, s_k fp32)."""
    B, H, S, D = q.shape
    if sm_scale is None:
        sm_scale = 1.0 / math.sqrt(D)
    k8, s_k = quantize_k_rows_ref(k)
    q8, s_q = quantize_q_rows_ref(q)
    acc = torch.einsum("bhqd,bhkd->bhqk", torch.from_numpy(q8.astype(np.float32)),
                       torch.from_numpy(k8.astype(np.float32)))  # exact: |sum| < 2^24
    qk = acc * (torch.from_numpy(s_q)[..., :, None] * torch.from_numpy(s_k)[..., None, :])
    qk = qk * np.float32(sm_scale * 1.44269504)
    keep = _int8_keep(S, causal, seq_len_k, seq_len_q)
    qk = qk + torch.where(keep, 0.0, -1.0e6)[None, None]
    m = qk.max(dim=-1, keepdim=True).values
    p = torch.exp2(qk - m)
    l = p.sum(dim=-1, keepdim=True)
    out = torch.einsum("bhqk,bhkd->bhqd", p.half().float(), v.float()) / l
    lse2 = (m + torch.log2(l)).squeeze(-1)
    return out, lse2, k8, s_k


def attention_int8_grads_ref(q, k, v, dout, causal=False, sm_scale=None, seq_len_k=None, seq_len_q=None):
    """Gradients the INT8 path returns: the fp16 dense backward run on the ORIGINAL fp16
    q,k,v with the base-2 LSE and the output saved by the INT8 forward
    (attention_kernel_int8.py:256-267 -> attention_kernel.py:1104-1155).  So
    P = exp2(q.k*scale*log2e - lse2_int8) is not exactly normalised, and
    delta = rowsum(o_int8 * dout).  q,k,v,dout: (B,H,S,D).  Returns fp32 (dq, dk, dv)."""
    B, H, S, D = q.shape
    if sm_scale is None:
        sm_scale = 1.0 / math.sqrt(D)
    out, lse2, _, _ = attention_int8_ref(q, k, v, causal, sm_scale, seq_len_k, seq_len_q)
    o16 = out.half().float()
    qf, kf, vf, dof = q.float(), k.float(), v.float(), dout.float()
    s2 = torch.einsum("bhqd,bhkd->bhqk", qf, kf) * (sm_scale * LOG2E)
    p = torch.exp2(s2 - lse2[..., None])
    p = p * _int8_keep(S, causal, seq_len_k, seq_len_q)[None, None]
    delta = (o16 * dof).sum(-1, keepdim=True)
    dp = torch.einsum("bhqd,bhkd->bhqk", dof, vf)
    ds = p * (dp - delta)
    dv = torch.einsum("bhqk,bhqd->bhkd", p, dof)
    dq = torch.einsum("bhqk,bhkd->bhqd", ds, kf) * sm_scale
    dk = torch.einsum("bhqk,bhqd->bhkd", ds, qf) * sm_scale
    return dq, dk, dv


# ---------------------------------------------------------------------------------------
# helper package: rotary embedding kernel and un-padding (flash_attn/ in the reference)
# ---------------------------------------------------------------------------------------
def rotary_emb_ref(x, cos, sin, seqlen_offsets=0, cu_seqlens=None, max_seqlen=None, interleaved=False,
                   conjugate=False):
    """Rotary embedding as the reference's kernel computes it
    (flash_attn/ops/triton/rotary.py:11-130): fp32 arithmetic on the first rotary_dim columns,
    o0 = x0 cos - x1 sin, o1 = x0 sin + x1 cos with pairs (i, i + rotary_dim/2) or, interleaved,
    (2i, 2i+1); sin negated for the conjugate (backward) form; table rows past the end read
    cos = 1, sin = 0; one rounding to x's dtype.  x (B,S,H,D), or packed (T,H,D) with cu_seqlens."""
    xf = x.float()
    out = xf.clone()
    half = cos.shape[1]
    rot = 2 * half
    cf, sf = cos.float(), sin.float()
    if conjugate:
        sf = -sf

    def one(seq, offset):                              # seq (S,H,D) view of `out`, rotated in place
        pos = torch.arange(seq.shape[0]) + int(offset)
        ok = (pos >= 0) & (pos < cf.shape[0])
        c = torch.where(ok[:, None], cf[pos.clamp(0, cf.shape[0] - 1)], torch.ones(1))[:, None, :]
        s = torch.where(ok[:, None], sf[pos.clamp(0, cf.shape[0] - 1)], torch.zeros(1))[:, None, :]
        if interleaved:
            x0, x1 = seq[..., 0:rot:2].clone(), seq[..., 1:rot:2].clone()
            seq[..., 0:rot:2] = x0 * c - x1 * s
            seq[..., 1:rot:2] = x0 * s + x1 * c
        else:
            x0, x1 = seq[..., :half].clone(), seq[..., half:rot].clone()
            seq[..., :half] = x0 * c - x1 * s
            seq[..., half:rot] = x0 * s + x1 * c

    if cu_seqlens is None:
        for b in range(x.shape[0]):
            off = seqlen_offsets[b] if isinstance(seqlen_offsets, torch.Tensor) else seqlen_offsets
            one(out[b], off)
    else:
        cu = [int(c) for c in cu_seqlens]
        for b in range(len(cu) - 1):
            off = seqlen_offsets[b] if isinstance(seqlen_offsets, torch.Tensor) else seqlen_offsets
            one(out[cu[b]:cu[b + 1]], off)
    return out.to(x.dtype)


def unpad_ref(hidden_states, attention_mask):
    """(tokens, indices, cu_seqlens int32, max_seqlen) of the valid positions of a padded batch
    (flash_attn/bert_padding.py:98-122), with plain indexing."""
    lens = attention_mask.sum(dim=-1).to(torch.int32)
    idx = torch.nonzero(attention_mask.flatten()).flatten()
    cu = torch.cat([torch.zeros(1, dtype=torch.int32), torch.cumsum(lens, 0).to(torch.int32)])
    flat = hidden_states.reshape((-1,) + tuple(hidden_states.shape[2:]))
    return flat[idx], idx, cu, int(lens.max())


def pad_ref(tokens, indices, batch, seqlen):
    """Zero-padded (batch, seqlen, ...) tensor with `tokens` at `indices`
    (flash_attn/bert_padding.py:197-213)."""
    out = torch.zeros((batch * seqlen,) + tuple(tokens.shape[1:]), dtype=tokens.dtype)
    out[indices] = tokens
    return out.reshape((batch, seqlen) + tuple(tokens.shape[1:]))
