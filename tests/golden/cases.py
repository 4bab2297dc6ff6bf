"""Seeded inputs for the golden-vector cases.

Inputs are regenerated from numpy's PCG64 stream (stable across platforms), so the
fixtures only store the reference's outputs plus a checksum of the inputs.
"""
from __future__ import annotations

import hashlib

import numpy as np
import torch


def randn16(rng, *shape):
    return torch.from_numpy(rng.standard_normal(shape, dtype=np.float32).astype(np.float16))


def checksum(*tensors):
    h = hashlib.sha256()
    for t in tensors:
        h.update(np.ascontiguousarray(t.detach().cpu().numpy()).tobytes())
    return h.hexdigest()[:16]


def dense_case(seed, B, Sq, Sk, Hq, Hkv, D):
    """q (B,Sq,Hq,D), k,v (B,Sk,Hkv,D), dout like q; fp16 N(0,1)."""
    rng = np.random.default_rng(seed)
    q = randn16(rng, B, Sq, Hq, D)
    k = randn16(rng, B, Sk, Hkv, D)
    v = randn16(rng, B, Sk, Hkv, D)
    do = randn16(rng, B, Sq, Hq, D)
    return q, k, v, do


def varlen_case(seed, q_lens, k_lens, Hq, Hkv, D):
    rng = np.random.default_rng(seed)
    Tq, Tk = sum(q_lens), sum(k_lens)
    q = randn16(rng, Tq, Hq, D)
    k = randn16(rng, Tk, Hkv, D)
    v = randn16(rng, Tk, Hkv, D)
    do = randn16(rng, Tq, Hq, D)
    cu_q = torch.tensor(np.concatenate([[0], np.cumsum(q_lens)]), dtype=torch.int32)
    cu_k = torch.tensor(np.concatenate([[0], np.cumsum(k_lens)]), dtype=torch.int32)
    return q, k, v, do, cu_q, cu_k


def k_with_outliers(seed, *shape):
    """fp16 N(0,1) with 1 % of entries scaled x8."""
    rng = np.random.default_rng(seed)
    k = rng.standard_normal(shape, dtype=np.float32)
    mask = rng.random(shape) < 0.01
    k = np.where(mask, k * 8.0, k).astype(np.float16)
    return torch.from_numpy(k)


def int8_case(seed, B, H, S, D):
    rng = np.random.default_rng(seed)
    q = randn16(rng, B, H, S, D)
    v = randn16(rng, B, H, S, D)
    k = k_with_outliers(seed + 1, B, H, S, D)
    return q, k, v


def rotary_tables(seqlen, rotary_dim, base=10000.0, dtype=torch.float16):
    inv = 1.0 / (base ** (torch.arange(0, rotary_dim, 2, dtype=torch.float32) / rotary_dim))
    ang = torch.arange(seqlen, dtype=torch.float32)[:, None] * inv[None, :]
    return torch.cos(ang).to(dtype), torch.sin(ang).to(dtype)


def paged_case(seed, B, Hq, Hkv, D, page, n_pages, lens, max_pages):
    """Paged cache + one new token per sequence; block_table rows are disjoint slices of
    one permutation, unused tail entries repeat a valid index."""
    rng = np.random.default_rng(seed)
    kc = randn16(rng, n_pages, page, Hkv, D)
    vc = randn16(rng, n_pages, page, Hkv, D)
    q = randn16(rng, B, 1, Hq, D)
    kn = randn16(rng, B, 1, Hkv, D)
    vn = randn16(rng, B, 1, Hkv, D)
    perm = rng.permutation(n_pages)
    bt = np.zeros((B, max_pages), dtype=np.int32)
    at = 0
    for b, L in enumerate(lens):
        need = (L + 1 + page - 1) // page
        assert need <= max_pages and at + need <= n_pages
        bt[b, :need] = perm[at:at + need]
        bt[b, need:] = perm[at]
        at += need
    return q, kc, vc, kn, vn, torch.from_numpy(bt), torch.tensor(lens, dtype=torch.int32)


# ----------------------------------------------------------------------------------------
# helper package (rotary embedding, un-padding)
# ----------------------------------------------------------------------------------------
ROTARY_CASES = {
    # name: generator arguments
    "half": dict(seed=50, B=2, S=9, H=3, D=32, rot=32, S_ro=16),
    "half_partial": dict(seed=51, B=2, S=9, H=3, D=64, rot=32, S_ro=16),
    "interleaved": dict(seed=52, B=2, S=10, H=2, D=32, rot=16, S_ro=24, interleaved=True),
    "offset_int": dict(seed=53, B=1, S=7, H=2, D=32, rot=32, S_ro=16, offset=5),
    "offset_tensor": dict(seed=54, B=3, S=6, H=2, D=32, rot=32, S_ro=20, offsets=[0, 7, 14]),
    "conjugate": dict(seed=55, B=2, S=8, H=2, D=32, rot=32, S_ro=8, conjugate=True, interleaved=True),
    "varlen": dict(seed=56, B=3, S=0, H=2, D=32, rot=32, S_ro=16, lens=[5, 1, 9]),
}


def rotary_case(seed, B, S, H, D, rot, S_ro, interleaved=False, conjugate=False, offset=0, offsets=None,
                lens=None):
    """x (B,S,H,D) -- or packed (sum(lens),H,D) -- fp16 N(0,1); cos/sin (S_ro, rot/2) fp16 from
    base-10000 frequencies.  Returns (x, cos, sin, kwargs of apply_rotary)."""
    rng = np.random.default_rng(seed)
    inv = 1.0 / (10000.0 ** (np.arange(0, rot, 2, dtype=np.float32) / rot))
    ang = np.arange(S_ro, dtype=np.float32)[:, None] * inv[None, :]
    cos = torch.from_numpy(np.cos(ang).astype(np.float16))
    sin = torch.from_numpy(np.sin(ang).astype(np.float16))
    kw = dict(interleaved=interleaved, conjugate=conjugate)
    if lens is not None:
        x = randn16(rng, sum(lens), H, D)
        kw.update(cu_seqlens=torch.tensor(np.concatenate([[0], np.cumsum(lens)]), dtype=torch.int32),
                  max_seqlen=max(lens))
    else:
        x = randn16(rng, B, S, H, D)
    if offsets is not None:
        kw["seqlen_offsets"] = torch.tensor(offsets, dtype=torch.int32)
    elif offset:
        kw["seqlen_offsets"] = offset
    return x, cos, sin, kw


def padding_case(seed, B, S, H, D):
    """hidden states (B,S,H,D) fp16, a (B,S) 0/1 mask with ragged valid prefixes, and the
    (B,S) lengths-in-row table of the concatenated-samples variant."""
    rng = np.random.default_rng(seed)
    hs = randn16(rng, B, S, H, D)
    valid = rng.integers(1, S + 1, size=B)
    mask = torch.from_numpy((np.arange(S)[None, :] < valid[:, None]).astype(np.int32))
    lens_in_row = np.zeros((B, S), dtype=np.int32)
    for b in range(B):
        left, i = int(valid[b]), 0
        while left > 0:
            n = int(rng.integers(1, left + 1))
            lens_in_row[b, i] = n
            left -= n
            i += 1
    return hs, mask, torch.from_numpy(lens_in_row)
