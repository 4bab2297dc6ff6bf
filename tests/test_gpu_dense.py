"""Dense forward/backward parity: CUDA kernels (through the C ABI) against the golden
vectors of the reference and against the fp32 CPU oracle.

Tolerances (max-abs): 2e-3 forward, 1e-2 gradients for fp16 -- the bars stated for this
path; bf16 (not supported by the reference) gets its own rounding-limited bars in util.py.
"""
import ast

import numpy as np
import pytest
import torch

import cases
import util
from oracle import attention_oracle as orc
from util import DEV, LN2, maxdiff

pytestmark = pytest.mark.gpu


def fa():
    import flash_attn_triton_b200 as m
    return m


@pytest.mark.parametrize("causal", [0, 1])
def test_golden_config1(golden, causal):
    """B2 H4 S128 D64: out, base-2 LSE and all gradients vs the reference's own output."""
    from flash_attn_triton_b200 import _native as N, _ops
    g = golden(f"dense_c1_causal{causal}")
    q, k, v, do = cases.dense_case(0, 2, 128, 128, 4, 4, 64)
    assert cases.checksum(q, k, v, do) == str(g["checksum"])
    qd, kd, vd, dod = (t.to(DEV) for t in (q, k, v, do))
    o, lse, _ = _ops.dense_forward(qd, kd, vd, 0.125, bool(causal), -1, -1, 0.0, None, 0,
                                   N.IMPL_AUTO, "bshd", True)
    dq, dk, dv = _ops.dense_backward(qd, kd, vd, o, lse, dod, 0.125, bool(causal), -1, -1, 0.0,
                                     None, 0, N.IMPL_AUTO, "bshd")
    assert maxdiff(o, g["out"]) <= util.FWD_TOL
    assert maxdiff(lse, g["lse2"]) <= util.FWD_TOL
    for name, t in (("dq", dq), ("dk", dk), ("dv", dv)):
        assert maxdiff(t, g[name]) <= util.GRAD_TOL, name
    # and against the exact oracle
    ro, rl, rdq, rdk, rdv = orc.attention_grads_ref(q, k, v, do, softmax_scale=0.125,
                                                    causal=bool(causal))
    assert maxdiff(o, ro) <= util.FWD_TOL
    assert maxdiff(lse * LN2, rl) <= util.FWD_TOL
    for t, r in ((dq, rdq), (dk, rdk), (dv, rdv)):
        assert maxdiff(t, r) <= util.GRAD_TOL


def test_golden_public_cases(golden):
    """The shapes of the reference's own test file and the surfaces it leaves unpinned
    (window, cross, ALiBi, softcap, GQA, everything at once), forward and backward."""
    g = golden("dense_public")
    specs = ast.literal_eval(str(g["_specs"]))
    for i, (name, (B, Sq, Sk, Hq, Hkv, D, kw)) in enumerate(specs.items()):
        q, k, v, do = cases.dense_case(100 + i, B, Sq, Sk, Hq, Hkv, D)
        kw = dict(kw)
        if "alibi_slopes" in kw:
            kw["alibi_slopes"] = torch.tensor(kw["alibi_slopes"], dtype=torch.float32, device=DEV)
        out, dq, dk, dv = util.run_dense(fa().flash_attn_func, q, k, v, do, **kw)
        assert maxdiff(out, g[name + ".out"]) <= util.FWD_TOL, name
        for n, t in (("dq", dq), ("dk", dk), ("dv", dv)):
            assert maxdiff(t, g[f"{name}.{n}"]) <= util.GRAD_TOL, (name, n)


SHAPES = [
    # B, Sq, Sk, Hq, Hkv, D
    (1, 1, 1, 1, 1, 16),
    (2, 17, 17, 2, 2, 16),
    (2, 64, 64, 2, 1, 32),
    (1, 100, 100, 4, 2, 64),
    (2, 129, 129, 4, 4, 128),
    (1, 300, 300, 2, 1, 128),
    (1, 200, 200, 2, 2, 256),
    (2, 7, 13, 2, 2, 64),
    (2, 13, 7, 2, 2, 64),
    (1, 257, 63, 8, 2, 128),
    (1, 65, 400, 4, 1, 128),
]
FEATURES = [
    dict(),
    dict(causal=True),
    dict(window_size=(5, 3)),
    dict(causal=True, window_size=(20, -1)),
    dict(softcap=4.0),
    dict(alibi="heads"),
    dict(causal=True, softcap=15.0, alibi="batch", window_size=(33, 0), softmax_scale=0.3),
]


@pytest.mark.parametrize("shape", SHAPES, ids=lambda s: "x".join(map(str, s)))
@pytest.mark.parametrize("feat", range(len(FEATURES)))
def test_dense_vs_oracle(shape, feat):
    B, Sq, Sk, Hq, Hkv, D = shape
    kw = dict(FEATURES[feat])
    q, k, v, do = cases.dense_case(1000 + feat, B, Sq, Sk, Hq, Hkv, D)
    alibi = kw.pop("alibi", None)
    okw = dict(softmax_scale=kw.get("softmax_scale"), causal=kw.get("causal", False),
               window=kw.get("window_size", (-1, -1)), softcap=kw.get("softcap", 0.0))
    if alibi == "heads":
        sl = torch.tensor([2.0 ** (-(i + 1)) for i in range(Hq)])
    elif alibi == "batch":
        sl = torch.rand(B, Hq, generator=torch.Generator().manual_seed(5)) * 0.5
    else:
        sl = None
    if sl is not None:
        kw["alibi_slopes"] = sl.to(DEV)
        okw["alibi_slopes"] = sl
    out, dq, dk, dv = util.run_dense(fa().flash_attn_func, q, k, v, do, **kw)
    ro, _, rdq, rdk, rdv = orc.attention_grads_ref(q, k, v, do, **okw)
    assert maxdiff(out, ro) <= util.FWD_TOL
    assert maxdiff(dq, rdq) <= util.GRAD_TOL
    assert maxdiff(dk, rdk) <= util.GRAD_TOL
    assert maxdiff(dv, rdv) <= util.GRAD_TOL


@pytest.mark.parametrize("D", [64, 128])
def test_bf16(D):
    q, k, v, do = cases.dense_case(7, 2, 150, 150, 4, 2, D)
    qb, kb, vb, dob = (t.bfloat16() for t in (q, k, v, do))
    out, dq, dk, dv = util.run_dense(fa().flash_attn_func, qb, kb, vb, dob, causal=True)
    ro, _, rdq, rdk, rdv = orc.attention_grads_ref(qb, kb, vb, dob, causal=True)
    ft, gt = util.tols(torch.bfloat16)
    assert maxdiff(out, ro) <= ft
    for t, r in ((dq, rdq), (dk, rdk), (dv, rdv)):
        assert maxdiff(t, r) <= gt


def test_cross_offset_and_empty_rows():
    """flash_attn_func_cross with _causal_offset (bottom-right style alignment) and a
    window that leaves some rows without any visible key: those rows are 0, not NaN."""
    q, k, v, do = cases.dense_case(11, 1, 40, 100, 2, 2, 64)
    out, dq, dk, dv = util.run_dense(fa().flash_attn_func_cross, q, k, v, do, causal=True,
                                     _causal_offset=60)
    ro, _, rdq, rdk, rdv = orc.attention_grads_ref(q, k, v, do, causal=True, q_pos_offset=60)
    assert maxdiff(out, ro) <= util.FWD_TOL and maxdiff(dk, rdk) <= util.GRAD_TOL
    # Sq > Sk with a right-only window: rows past Sk+2 see nothing
    q, k, v, do = cases.dense_case(12, 1, 90, 30, 2, 2, 64)
    out, dq, dk, dv = util.run_dense(fa().flash_attn_func, q, k, v, do, window_size=(2, 0))
    ro, rl, rdq, rdk, rdv = orc.attention_grads_ref(q, k, v, do, window=(2, 0))
    assert torch.isinf(rl).any()
    assert torch.isfinite(out).all() and torch.isfinite(dq).all()
    assert maxdiff(out, ro) <= util.FWD_TOL
    for t, r in ((dq, rdq), (dk, rdk), (dv, rdv)):
        assert maxdiff(t, r) <= util.GRAD_TOL


def test_packed_and_strided_inputs():
    """qkv-packed and kv-packed layouts are read in place through strides
    (reference: tests/test_compare_implementations.py:181-201)."""
    q, k, v, do = cases.dense_case(13, 2, 128, 128, 2, 2, 16)
    qkv = torch.stack((q, k, v), dim=2).to(DEV)
    out = fa().flash_attn_qkvpacked_func(qkv, causal=True)
    ro, _ = orc.attention_ref(q, k, v, causal=True)
    assert maxdiff(out, ro) <= util.FWD_TOL
    qs, ks, vs = qkv.unbind(dim=2)
    assert not qs.is_contiguous()
    assert maxdiff(fa().flash_attn_func(qs, ks, vs), orc.attention_ref(q, k, v)[0]) <= util.FWD_TOL
    kv = torch.stack((k, v), dim=2).to(DEV)
    out = fa().flash_attn_kvpacked_func(q.to(DEV), kv)
    assert maxdiff(out, orc.attention_ref(q, k, v)[0]) <= util.FWD_TOL
    # gradient flows back into the packed tensor
    qkv.requires_grad_()
    fa().flash_attn_qkvpacked_func(qkv, causal=True).float().mul(do.to(DEV).float()).sum().backward()
    _, _, rdq, rdk, rdv = orc.attention_grads_ref(q, k, v, do, causal=True)
    assert maxdiff(qkv.grad[:, :, 0], rdq) <= util.GRAD_TOL
    assert maxdiff(qkv.grad[:, :, 1], rdk) <= util.GRAD_TOL
    assert maxdiff(qkv.grad[:, :, 2], rdv) <= util.GRAD_TOL


def test_bias_probs_dropout_fp32_smallest():
    """attn_bias / return_attn_probs / dropout / fp32 at the sizes of the reference's own checks
    (tests/test_compare_implementations.py:161-178); tests/test_gpu_features.py goes further."""
    q, k, v, do = cases.dense_case(14, 2, 7, 13, 2, 2, 16)
    bias = (torch.randn(2, 2, 7, 13, generator=torch.Generator().manual_seed(11)) * 0.1).half()
    out = fa().flash_attn_func_cross(q.to(DEV), k.to(DEV), v.to(DEV), attn_bias=bias.to(DEV))
    ro, _ = orc.attention_ref(q, k, v, attn_bias=bias)
    assert maxdiff(out, ro) <= util.FWD_TOL
    out, lse, probs = fa().flash_attn_func(q.to(DEV), k.to(DEV), v.to(DEV), causal=True,
                                           return_attn_probs=True)
    ro, rl = orc.attention_ref(q, k, v, causal=True)
    assert maxdiff(out, ro) <= util.FWD_TOL and maxdiff(lse, rl) <= util.FWD_TOL
    assert probs.shape == (2, 2, 7, 13)
    z = torch.zeros(1, 1, 1, 16, device=DEV, dtype=torch.float16)
    o = fa().flash_attn_func(z, z, torch.ones_like(z), dropout_p=0.5)
    assert torch.all(torch.isclose(o, torch.full_like(o, 2.0), atol=1e-3) | (o.abs() < 1e-3))
    o32 = fa().flash_attn_func(q.float().to(DEV), k.float().to(DEV), v.float().to(DEV))
    assert o32.dtype == torch.float32 and maxdiff(o32, orc.attention_ref(q, k, v)[0]) <= util.FWD_TOL


def test_modules():
    m = fa()
    q, k, v, do = cases.dense_case(15, 2, 33, 33, 2, 2, 32)
    out = m.FlashAttention()(q.to(DEV), k.to(DEV), v.to(DEV), causal=True)
    assert maxdiff(out, orc.attention_ref(q, k, v, causal=True)[0]) <= util.FWD_TOL
    qkv = torch.stack((q, k, v), dim=2).to(DEV)
    out = m.FlashSelfAttention(causal=True).eval()(qkv)
    assert maxdiff(out, orc.attention_ref(q, k, v, causal=True)[0]) <= util.FWD_TOL
    kv = torch.stack((k, v), dim=2).to(DEV)
    out = m.FlashCrossAttention().eval()(q.to(DEV), kv)
    assert maxdiff(out, orc.attention_ref(q, k, v)[0]) <= util.FWD_TOL


def test_reference_import_paths():
    """Code written against the reference package imports unchanged."""
    from flash_attn_triton import flash_attn_func, flash_attn_varlen_func  # noqa: F401
    from flash_attn_triton.triton_kernel.attention_kernel_int8 import attention_int8  # noqa: F401


def test_value_errors_on_gpu():
    m = fa()
    q = torch.zeros(1, 8, 2, 64, device=DEV, dtype=torch.float16)
    with pytest.raises(ValueError):
        m.flash_attn_func(q, q[:, :, :1].repeat(1, 1, 3, 1), q[:, :, :1].repeat(1, 1, 3, 1))
    with pytest.raises(ValueError):
        m.flash_attn_func(q, q, q, softcap=-1.0)
    with pytest.raises(ValueError):
        m.flash_attn_func(q[..., :24], q[..., :24], q[..., :24])  # head_dim 24


def test_full_size_properties():
    """Config 2 size (B16 H16 S4096 D128 causal): properties that need no oracle at this
    size, plus the oracle on one (batch, head) slice."""
    m = fa()
    torch.manual_seed(0)
    B, S, H, D = 16, 4096, 16, 128
    q = torch.randn(B, S, H, D, device=DEV, dtype=torch.float16)
    k = torch.randn(B, S, H, D, device=DEV, dtype=torch.float16)
    v = torch.randn(B, S, H, D, device=DEV, dtype=torch.float16)
    out = m.flash_attn_func(q, k, v, causal=True)
    # row 0 attends to key 0 only
    assert torch.equal(out[:, 0], v[:, 0])
    # softmax rows sum to one: V = 1 gives O = 1
    ones = m.flash_attn_func(q, k, torch.ones_like(v), causal=True)
    assert (ones.float() - 1).abs().max().item() <= 2e-3
    # linear in V
    out2 = m.flash_attn_func(q, k, (2 * v), causal=True)
    assert (out2.float() - 2 * out.float()).abs().max().item() <= 4e-3
    # one slice against the oracle (fp32, CPU)
    b, h = 3, 5
    ro, _, rdq, rdk, rdv = orc.attention_grads_ref(q[b:b + 1, :, h:h + 1].cpu(), k[b:b + 1, :, h:h + 1].cpu(),
                                                   v[b:b + 1, :, h:h + 1].cpu(),
                                                   torch.ones(1, S, 1, D), causal=True)
    assert maxdiff(out[b:b + 1, :, h:h + 1], ro) <= util.FWD_TOL
    qg, kg, vg = (t.clone().requires_grad_() for t in (q, k, v))
    o = m.flash_attn_func(qg, kg, vg, causal=True)
    mask = torch.zeros_like(o)
    mask[b, :, h] = 1
    o.backward(mask)
    assert maxdiff(qg.grad[b:b + 1, :, h:h + 1], rdq) <= util.GRAD_TOL
    assert maxdiff(kg.grad[b:b + 1, :, h:h + 1], rdk) <= util.GRAD_TOL
    assert maxdiff(vg.grad[b:b + 1, :, h:h + 1], rdv) <= util.GRAD_TOL
    # the other slices received a zero upstream gradient
    assert qg.grad[0].abs().max().item() == 0.0


def test_lowlevel_attention_entry_points(golden):
    """`attention` / `attention_varlen`, the operator layer under the public wrappers
    (attention_kernel.py:1201-1259, :1364-1380 of the reference): head-major tensors, explicit
    dropout seed, key-length mask and causal offset through seq_len_k / seq_len_q."""
    from flash_attn_triton.triton_kernel.attention_kernel import attention, attention_varlen
    g = golden("dense_c1_causal1")
    q, k, v, do = cases.dense_case(0, 2, 128, 128, 4, 4, 64)
    qh, kh, vh = (t.transpose(1, 2).contiguous().to(DEV).requires_grad_() for t in (q, k, v))
    out = attention(qh, kh, vh, True, 0.125)
    dq, dk, dv = torch.autograd.grad((out.float() * do.transpose(1, 2).to(DEV).float()).sum(), (qh, kh, vh))
    assert maxdiff(out.transpose(1, 2), g["out"]) <= util.FWD_TOL
    for n, t in (("dq", dq), ("dk", dk), ("dv", dv)):
        assert maxdiff(t.transpose(1, 2), g[n]) <= util.GRAD_TOL, n
    # explicit seed: the mask is the oracle's Philox stream with counters row * S + col
    q, k, v, do = cases.dense_case(16, 1, 192, 192, 2, 2, 64)
    qh, kh, vh = (t.transpose(1, 2).contiguous().to(DEV) for t in (q, k, v))
    out = attention(qh, kh, vh, False, None, 0.3, 4711)
    ro = orc.attention_dropout_ref(q, k, v, dropout_p=0.3, seed=4711, row_stride=192)[0]
    assert maxdiff(out.transpose(1, 2), ro) <= util.FWD_TOL / 0.7
    # a padded call: 150 valid keys, queries shifted so that row i sits at position i + 30
    out = attention(qh, kh, vh, True, None, 0.0, None, 150, 120)
    ro, _ = orc.attention_ref(q, k[:, :150], v[:, :150], causal=True, q_pos_offset=30)
    assert maxdiff(out.transpose(1, 2), ro) <= util.FWD_TOL
    with pytest.raises(ValueError, match="equal sequence lengths"):
        attention(qh, kh[:, :, :128], vh[:, :, :128])
    with pytest.raises(ValueError, match="divisible by 64"):
        attention(qh[:, :, :100], kh[:, :, :100], vh[:, :, :100])
    # packed
    ql = [37, 64, 130]
    q, k, v, do, cu_q, cu_k = cases.varlen_case(17, ql, ql, 4, 2, 64)
    out = attention_varlen(q.to(DEV), k.to(DEV), v.to(DEV), cu_q.to(DEV), cu_k.to(DEV), 130, 130, True, None, 0.25, 99)
    ro = orc.varlen_attention_dropout_ref(q, k, v, cu_q, cu_k, 130, dropout_p=0.25, seed=99, causal=True)[0]
    assert maxdiff(out, ro) <= util.FWD_TOL / 0.75
