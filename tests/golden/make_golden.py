"""Generate tests/golden/*.npz from the UNMODIFIED reference run on the CPU.

Run from the repository root in a container that has the reference checked out:

    python tests/golden/make_golden.py /path/to/reference [case ...]     (or FA_REF_PATH=...)

The reference's Triton kernels are executed by Triton's interpreter (see
oracle/ref_loader.py for the three harness shims).  Inputs come from tests/golden/cases.py;
only outputs and an input checksum are stored.
"""
from __future__ import annotations

import os
import sys
import types

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, ROOT)
sys.path.insert(0, HERE)

from oracle.ref_loader import load_reference  # noqa: E402

_REF_PATH = sys.argv[1] if len(sys.argv) > 1 else os.environ.get("FA_REF_PATH")
if not _REF_PATH:
    sys.exit("pass the reference checkout as argv[1] or in FA_REF_PATH")
REF = load_reference(_REF_PATH)

import numpy as np  # noqa: E402
import torch  # noqa: E402

import cases  # noqa: E402


def save(name, **arrays):
    out = {}
    for k, v in arrays.items():
        if isinstance(v, torch.Tensor):
            v = v.detach().cpu().numpy()
        out[k] = v
    np.savez_compressed(os.path.join(HERE, name + ".npz"), **out)
    print("wrote", name, {k: getattr(v, "shape", v) for k, v in out.items()})


class _Ctx:
    def save_for_backward(self, *t):
        self.saved = t


def dense_lowlevel():
    """Config 1 of the benchmark spec: B2 H4 S128 D64 through the reference's operator
    layer (attention_kernel.py:1057-1155): out, base-2 LSE, dq, dk, dv."""
    AK = REF.AK
    for causal in (False, True):
        q, k, v, do = cases.dense_case(0, 2, 128, 128, 4, 4, 64)
        qh, kh, vh, doh = (t.transpose(1, 2).contiguous() for t in (q, k, v, do))
        kw = dict(causal=causal, sm_scale=0.125, dropout_p=0.0, dropout_seed=0, seq_len_k=128,
                  seq_len_q=128, kv_heads=4, softcap=0.0,
                  alibi_slopes=qh.new_empty((1,), dtype=torch.float32), window_left=-1,
                  window_right=-1, use_alibi=False)
        out, M = AK._launch_dense_forward(qh, kh, vh, kw["causal"], kw["sm_scale"], 0.0, 0, 128,
                                          128, 4, 0.0, kw["alibi_slopes"], -1, -1, False,
                                          store_lse=True)
        dq, dk, dv = AK._dense_backward(qh, kh, vh, out, M, doh, sm_scale=0.125, head_dim=64,
                                        causal=causal, seq_len_k=128, seq_len_q=128, kv_heads=4)
        save(f"dense_c1_causal{int(causal)}", checksum=cases.checksum(q, k, v, do),
             out=out.transpose(1, 2), lse2=M, dq=dq.transpose(1, 2), dk=dk.transpose(1, 2),
             dv=dv.transpose(1, 2))


def dense_public():
    """Small shapes of the reference's own tests (tests/test_compare_implementations.py:85-212)
    plus the surfaces they leave unpinned, through the public wrappers."""
    IF = REF.IF
    specs = {
        # name: (B,Sq,Sk,Hq,Hkv,D, kwargs)
        "eq17_causal0": (2, 17, 17, 2, 2, 16, dict(causal=False, softmax_scale=0.125)),
        "eq17_causal1": (2, 17, 17, 2, 2, 16, dict(causal=True, softmax_scale=0.125)),
        "win32_causal0": (1, 17, 17, 2, 2, 16, dict(causal=False, window_size=(3, 2))),
        "win32_causal1": (1, 17, 17, 2, 2, 16, dict(causal=True, window_size=(3, 2))),
        "cross7x13_causal0": (2, 7, 13, 2, 2, 16, dict(causal=False)),
        "cross7x13_causal1": (2, 7, 13, 2, 2, 16, dict(causal=True)),
        "cross13x7_causal1": (2, 13, 7, 2, 2, 16, dict(causal=True)),
        "alibi": (2, 17, 17, 2, 2, 16, dict(causal=False, alibi_slopes=[[0.05, 0.11], [0.02, 0.2]])),
        "softcap": (2, 70, 70, 2, 2, 32, dict(causal=True, softcap=5.0)),
        "gqa": (2, 70, 70, 4, 2, 64, dict(causal=True)),
        "all": (1, 150, 150, 4, 2, 64, dict(causal=True, window_size=(40, 0), softcap=8.0,
                                             alibi_slopes=[0.5, 0.25, 0.125, 0.0625])),
    }
    blob = {}
    for i, (name, (B, Sq, Sk, Hq, Hkv, D, kw)) in enumerate(specs.items()):
        q, k, v, do = cases.dense_case(100 + i, B, Sq, Sk, Hq, Hkv, D)
        qg, kg, vg = (t.clone().requires_grad_() for t in (q, k, v))
        kw2 = dict(kw)
        if "alibi_slopes" in kw2:
            kw2["alibi_slopes"] = torch.tensor(kw2["alibi_slopes"], dtype=torch.float32)
        out = IF.flash_attn_func(qg, kg, vg, **kw2)
        dq, dk, dv = torch.autograd.grad((out.float() * do.float()).sum(), (qg, kg, vg))
        blob[name + ".checksum"] = np.array(cases.checksum(q, k, v, do))
        for n, t in (("out", out), ("dq", dq), ("dk", dk), ("dv", dv)):
            blob[f"{name}.{n}"] = t.detach().numpy()
        print(name, "done")
    blob["_specs"] = np.array(repr(specs))
    np.savez_compressed(os.path.join(HERE, "dense_public.npz"), **blob)


def varlen():
    """Packed batch with every score feature on, GQA 4/2
    (attention_kernel.py:27-272, :1281-1361): out, base-2 LSE (T,H), grads."""
    AK = REF.AK
    q_lens, k_lens = [37, 64, 130], [37, 64, 130]
    q, k, v, do, cu_q, cu_k = cases.varlen_case(7, q_lens, k_lens, 4, 2, 64)
    slopes = torch.tensor([2.0 ** (-8 * (i + 1) / 4) for i in range(4)], dtype=torch.float32)
    al = slopes[None].expand(3, -1).contiguous()
    qg, kg, vg = (t.clone().requires_grad_() for t in (q, k, v))
    ctx = _Ctx()
    out = AK._attention_varlen.forward(ctx, qg.detach(), kg.detach(), vg.detach(), cu_q, cu_k, 130,
                                       130, True, 0.125, 0.0, 0, 30.0, al, 48, 0, True)
    lse2 = ctx.saved[4]
    out2 = AK.attention_varlen(qg, kg, vg, cu_q, cu_k, 130, 130, causal=True, sm_scale=0.125,
                               softcap=30.0, alibi_slopes=al, window_left=48, window_right=0,
                               use_alibi=True)
    dq, dk, dv = torch.autograd.grad((out2.float() * do.float()).sum(), (qg, kg, vg))
    assert torch.equal(out, out2.detach())
    save("varlen_all", checksum=cases.checksum(q, k, v, do), out=out, lse2=lse2, dq=dq, dk=dk,
         dv=dv, q_lens=np.array(q_lens), k_lens=np.array(k_lens), slopes=slopes)

    # rectangular causal varlen of the reference's own test (:140-159), forward only
    q, k, v, do, cu_q, cu_k = cases.varlen_case(8, [3, 5], [4, 6], 2, 2, 16)
    out = REF.IF.flash_attn_varlen_func(q, k, v, cu_q, cu_k, 5, 6, causal=True)
    save("varlen_rect", checksum=cases.checksum(q, k, v, do), out=out)


def int8():
    """K quantiser codes/scales (bit-exact target) and the INT8-QK^T forward
    (attention_kernel_int8.py:58-79, :167-253)."""
    AK8 = REF.AK8
    import triton
    k = cases.k_with_outliers(21, 4, 192, 128)
    k8 = torch.empty((4, 192, 128), dtype=torch.int8)
    sk = torch.empty((4, 192), dtype=torch.float32)
    AK8._quantize_k_rows[(triton.cdiv(192, 64), 4)](k, k8, sk, 192, HEAD_DIM=128, BLOCK_R=64,
                                                    num_warps=4)
    save("int8_kquant", checksum=cases.checksum(k), k8=k8, s_k=sk)
    for causal in (False, True):
        q, k, v = cases.int8_case(30, 1, 2, 256, 128)
        ctx = _Ctx()
        out = AK8._attention_int8.forward(ctx, q, k, v, causal, 1.0 / 128 ** 0.5, 256, 256)
        save(f"int8_fwd_causal{int(causal)}", checksum=cases.checksum(q, k, v), out=out,
             lse2=ctx.saved[4])
        # forward + backward at the shape of the reference's own INT8 test (:222-235)
        q, k, v = cases.int8_case(31, 2, 2, 128, 64)
        do = cases.randn16(np.random.default_rng(32), 2, 2, 128, 64)
        qg, kg, vg = (t.clone().requires_grad_() for t in (q, k, v))
        out = AK8._attention_int8.apply(qg, kg, vg, causal, 0.125, 128, 128)
        dq, dk, dv = torch.autograd.grad((out.float() * do.float()).sum(), (qg, kg, vg))
        save(f"int8_bwd_causal{int(causal)}", checksum=cases.checksum(q, k, v, do), out=out,
             dq=dq, dk=dk, dv=dv)
        # padded call: 150 valid tokens inside 192 rows, seq_len_k = seq_len_q = 150 (:108-118, :245)
        q, k, v = cases.int8_case(33, 1, 2, 192, 64)
        do = cases.randn16(np.random.default_rng(34), 1, 2, 192, 64)
        qg, kg, vg = (t.clone().requires_grad_() for t in (q, k, v))
        out = AK8._attention_int8.apply(qg, kg, vg, causal, 0.125, 150, 150)
        dq, dk, dv = torch.autograd.grad((out.float() * do.float()).sum(), (qg, kg, vg))
        save(f"int8_padded_causal{int(causal)}", checksum=cases.checksum(q, k, v, do), out=out,
             dq=dq, dk=dk, dv=dv)


def kvcache():
    """Paged decode, GQA 8/2, page 64, non-interleaved rotary.  The reference never
    writes its cache (flash_attn_interface.py:487-492 copy into a temporary) and its
    causal path ignores the query offset, so the reference is pinned like this: the
    harness rotates the new key with the reference's own _apply_rotary, writes new k/v
    into a clone of the cache at slot `len`, then calls the reference with k=None,
    cache_seqlens=len+1, causal=False and the rotary tables (which rotate q at `len`)."""
    IF = REF.IF
    lens = [70, 5, 191]
    q, kc, vc, kn, vn, bt, cl = cases.paged_case(40, 3, 8, 2, 64, 64, 12, lens, 4)
    cos, sin = cases.rotary_tables(256, 64)
    kc2, vc2 = kc.clone(), vc.clone()
    for b, L in enumerate(lens):
        kr = IF._apply_rotary(kn[b:b + 1], cos, sin, torch.tensor([L]), False)[0]
        pg = int(bt[b, L // 64])
        kc2[pg, L % 64] = kr[0]
        vc2[pg, L % 64] = vn[b, 0]
    out = IF.flash_attn_with_kvcache(q, kc2, vc2, rotary_cos=cos, rotary_sin=sin,
                                     cache_seqlens=cl + 1, block_table=bt, causal=False,
                                     rotary_interleaved=False)
    # The same call without `causal` but with a right window and ALiBi: the reference measures both
    # from query position 0 here (:523), the library from the end of the sequence.  Stored so that
    # the difference is pinned, not to be matched.
    sl = torch.tensor([0.5, 0.25, 0.125, 0.0625, 0.03, 0.02, 0.01, 0.005])
    out_nc = IF.flash_attn_with_kvcache(q, kc2, vc2, rotary_cos=cos, rotary_sin=sin, cache_seqlens=cl + 1,
                                        block_table=bt, causal=False, rotary_interleaved=False,
                                        window_size=(-1, 40), alibi_slopes=sl)
    save("kvcache_noncausal_window", out=out_nc, slopes=sl)
    touched = torch.tensor([[int(bt[b, L // 64]), L % 64] for b, L in enumerate(lens)])
    save("kvcache_paged", checksum=cases.checksum(q, kc, vc, kn, vn, bt), out=out,
         touched=touched, k_rows=torch.stack([kc2[p, o] for p, o in touched.tolist()]),
         v_rows=torch.stack([vc2[p, o] for p, o in touched.tolist()]), lens=np.array(lens))


def dropout():
    """Dropout through the public wrappers with Python's `random` seeded, which fixes the seed the
    reference draws (attention_kernel.py:1238-1239, :1371-1372): equal-length dense (padded to 64),
    the cross path (both sides padded to the longer one) and the packed kernels."""
    import random
    IF, AK = REF.IF, REF.AK
    blob = {}
    specs = {
        "eq100_causal": (2, 100, 100, 2, 2, 64, dict(causal=True, softmax_scale=0.125, dropout_p=0.25)),
        "cross70x100_gqa": (1, 70, 100, 4, 2, 32, dict(causal=False, dropout_p=0.1)),
        "cross100x70_cap": (1, 100, 70, 2, 2, 32, dict(causal=True, dropout_p=0.3, softcap=6.0)),
    }
    for i, (name, (B, Sq, Sk, Hq, Hkv, D, kw)) in enumerate(specs.items()):
        q, k, v, do = cases.dense_case(300 + i, B, Sq, Sk, Hq, Hkv, D)
        qg, kg, vg = (t.clone().requires_grad_() for t in (q, k, v))
        random.seed(4242 + i)
        out = IF.flash_attn_func(qg, kg, vg, **kw)
        dq, dk, dv = torch.autograd.grad((out.float() * do.float()).sum(), (qg, kg, vg))
        random.seed(4242 + i)
        blob[name + ".seed"] = np.array(random.randrange(2 ** 31 - 1))
        blob[name + ".checksum"] = np.array(cases.checksum(q, k, v, do))
        for n, t in (("out", out), ("dq", dq), ("dk", dk), ("dv", dv)):
            blob[f"{name}.{n}"] = t.detach().numpy()
        print(name, "done")
    blob["_specs"] = np.array(repr(specs))
    q_lens, k_lens = [37, 64, 130], [50, 64, 101]
    q, k, v, do, cu_q, cu_k = cases.varlen_case(9, q_lens, k_lens, 4, 2, 64)
    qg, kg, vg = (t.clone().requires_grad_() for t in (q, k, v))
    random.seed(99)
    out = IF.flash_attn_varlen_func(qg, kg, vg, cu_q, cu_k, 130, 101, dropout_p=0.2, causal=True)
    dq, dk, dv = torch.autograd.grad((out.float() * do.float()).sum(), (qg, kg, vg))
    random.seed(99)
    blob["varlen.seed"] = np.array(random.randrange(2 ** 31 - 1))
    blob["varlen.checksum"] = np.array(cases.checksum(q, k, v, do))
    blob["varlen.q_lens"], blob["varlen.k_lens"] = np.array(q_lens), np.array(k_lens)
    for n, t in (("out", out), ("dq", dq), ("dk", dk), ("dv", dv)):
        blob[f"varlen.{n}"] = t.detach().numpy()
    # the deterministic packed path: one dense call, and one seed draw, per sequence (:660-681)
    qg, kg, vg = (t.clone().requires_grad_() for t in (q, k, v))
    random.seed(77)
    out = IF.flash_attn_varlen_func(qg, kg, vg, cu_q, cu_k, 130, 101, dropout_p=0.2, causal=True, deterministic=True)
    dq, dk, dv = torch.autograd.grad((out.float() * do.float()).sum(), (qg, kg, vg))
    random.seed(77)
    blob["varlen_det.seeds"] = np.array([random.randrange(2 ** 31 - 1) for _ in q_lens])
    for n, t in (("out", out), ("dq", dq), ("dk", dk), ("dv", dv)):
        blob[f"varlen_det.{n}"] = t.detach().numpy()
    np.savez_compressed(os.path.join(HERE, "dropout.npz"), **blob)
    print("wrote dropout")


if __name__ == "__main__":
    torch.manual_seed(0)
    only = sys.argv[2:]
    for fn in (dense_lowlevel, dense_public, varlen, int8, kvcache, dropout):
        if not only or fn.__name__ in only:
            fn()
