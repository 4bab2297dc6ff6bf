"""Packed variable-length attention parity (forward and backward)."""
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


def run_varlen(q, k, v, do, cu_q, cu_k, max_q, max_k, **kw):
    qd, kd, vd = (t.to(DEV).requires_grad_() for t in (q, k, v))
    out = fa().flash_attn_varlen_func(qd, kd, vd, cu_q.to(DEV), cu_k.to(DEV), max_q, max_k, **kw)
    dq, dk, dv = torch.autograd.grad((out.float() * do.to(DEV).float()).sum(), (qd, kd, vd))
    return out.detach().cpu(), dq.cpu(), dk.cpu(), dv.cpu()


def test_golden_varlen_all(golden):
    """3 sequences, GQA 4/2, causal + window + ALiBi + softcap: reference output, base-2
    LSE and gradients."""
    from flash_attn_triton_b200 import _native as N, _ops
    g = golden("varlen_all")
    ql, kl = g["q_lens"].tolist(), g["k_lens"].tolist()
    q, k, v, do, cu_q, cu_k = cases.varlen_case(7, ql, kl, 4, 2, 64)
    assert cases.checksum(q, k, v, do) == str(g["checksum"])
    sl = torch.from_numpy(g["slopes"])
    out, dq, dk, dv = run_varlen(q, k, v, do, cu_q, cu_k, 130, 130, softmax_scale=0.125,
                                 causal=True, window_size=(48, 0), softcap=30.0,
                                 alibi_slopes=sl.to(DEV))
    assert maxdiff(out, g["out"]) <= util.FWD_TOL
    for n, t in (("dq", dq), ("dk", dk), ("dv", dv)):
        assert maxdiff(t, g[n]) <= util.GRAD_TOL, n
    al = sl[None].expand(3, -1).contiguous().to(DEV)
    _, lse, _ = _ops.varlen_forward(q.to(DEV), k.to(DEV), v.to(DEV), cu_q.to(DEV), cu_k.to(DEV),
                                    130, 130, 0.125, True, 48, 0, 30.0, al, N.IMPL_AUTO, True)
    assert maxdiff(lse.transpose(0, 1), g["lse2"]) <= util.FWD_TOL


def test_golden_varlen_rect(golden):
    g = golden("varlen_rect")
    q, k, v, do, cu_q, cu_k = cases.varlen_case(8, [3, 5], [4, 6], 2, 2, 16)
    out = fa().flash_attn_varlen_func(q.to(DEV), k.to(DEV), v.to(DEV), cu_q.to(DEV), cu_k.to(DEV),
                                      5, 6, causal=True)
    assert maxdiff(out, g["out"]) <= util.FWD_TOL


CASES = [
    # q_lens, k_lens, Hq, Hkv, D, kwargs
    ([5, 70, 1, 130], [5, 70, 1, 130], 4, 4, 64, dict(causal=True)),
    ([64, 0, 33], [64, 0, 33], 2, 1, 128, dict(causal=True)),
    ([10, 20, 30], [40, 5, 64], 4, 2, 32, dict()),
    ([10, 20], [0, 7], 2, 2, 64, dict(causal=True)),
    ([200, 129], [200, 129], 8, 2, 128, dict(causal=True, window_size=(50, 0), softcap=30.0,
                                              alibi="heads")),
    ([17, 260], [17, 260], 2, 2, 256, dict(window_size=(7, 9))),
    ([33], [33], 2, 2, 16, dict(causal=True)),
]


@pytest.mark.parametrize("case", range(len(CASES)))
def test_varlen_vs_oracle(case):
    ql, kl, Hq, Hkv, D, kw = CASES[case]
    kw = dict(kw)
    q, k, v, do, cu_q, cu_k = cases.varlen_case(50 + case, ql, kl, Hq, Hkv, D)
    okw = dict(causal=kw.get("causal", False), window=kw.get("window_size", (-1, -1)),
               softcap=kw.get("softcap", 0.0))
    if kw.pop("alibi", None):
        sl = torch.tensor([2.0 ** (-8 * (i + 1) / Hq) for i in range(Hq)])
        kw["alibi_slopes"] = sl.to(DEV)
        okw["alibi_slopes"] = sl
    out, dq, dk, dv = run_varlen(q, k, v, do, cu_q, cu_k, max(ql), max(kl), **kw)
    ro, _, rdq, rdk, rdv = orc.varlen_attention_grads_ref(q, k, v, do, cu_q, cu_k, **okw)
    assert maxdiff(out, ro) <= util.FWD_TOL
    assert maxdiff(dq, rdq) <= util.GRAD_TOL
    assert maxdiff(dk, rdk) <= util.GRAD_TOL
    assert maxdiff(dv, rdv) <= util.GRAD_TOL


def test_packed_variants_and_options():
    m = fa()
    ql = [12, 40]
    q, k, v, do, cu, _ = cases.varlen_case(70, ql, ql, 2, 2, 64)
    ro, _ = orc.varlen_attention_ref(q, k, v, cu, cu, causal=True)
    qkv = torch.stack((q, k, v), dim=1).to(DEV)
    assert maxdiff(m.flash_attn_varlen_qkvpacked_func(qkv, cu.to(DEV), 40, causal=True), ro) <= util.FWD_TOL
    kv = torch.stack((k, v), dim=1).to(DEV)
    assert maxdiff(m.flash_attn_varlen_kvpacked_func(q.to(DEV), kv, cu.to(DEV), cu.to(DEV), 40, 40,
                                                     causal=True), ro) <= util.FWD_TOL
    # deterministic=True is the same computation
    o2 = m.flash_attn_varlen_func(q.to(DEV), k.to(DEV), v.to(DEV), cu.to(DEV), cu.to(DEV), 40, 40,
                                  causal=True, deterministic=True)
    assert maxdiff(o2, ro) <= util.FWD_TOL
    # return_attn_probs: natural-log lse padded with -inf
    o3, lse, probs = m.flash_attn_varlen_func(q.to(DEV), k.to(DEV), v.to(DEV), cu.to(DEV),
                                              cu.to(DEV), 40, 40, causal=True, return_attn_probs=True)
    assert maxdiff(o3, ro) <= util.FWD_TOL and lse.shape == (2, 2, 40) and torch.isinf(lse[0, :, 12:]).all()
    # seqused_k trims each sequence's keys
    o4 = m.flash_attn_varlen_func(q.to(DEV), k.to(DEV), v.to(DEV), cu.to(DEV), cu.to(DEV), 40, 40,
                                  seqused_k=[6, 20])
    kk = torch.cat([k[0:6], k[12:32]])
    vv = torch.cat([v[0:6], v[12:32]])
    r4, _ = orc.varlen_attention_ref(q, kk, vv, cu, torch.tensor([0, 6, 26]))
    assert maxdiff(o4, r4) <= util.FWD_TOL
    # paged k/v
    page = 16
    pool_k = torch.zeros(8, page, 2, 64, dtype=torch.float16)
    pool_v = torch.zeros(8, page, 2, 64, dtype=torch.float16)
    table = torch.tensor([[5, 0, 0], [2, 7, 1]], dtype=torch.int32)
    for b, (s, e) in enumerate(((0, 12), (12, 52))):
        for t in range(s, e):
            pg = table[b, (t - s) // page]
            pool_k[pg, (t - s) % page] = k[t]
            pool_v[pg, (t - s) % page] = v[t]
    o5 = m.flash_attn_varlen_func(q.to(DEV), pool_k.to(DEV), pool_v.to(DEV), cu.to(DEV), cu.to(DEV),
                                  40, 40, causal=True, block_table=table.to(DEV))
    assert maxdiff(o5, ro) <= util.FWD_TOL
    # value errors
    with pytest.raises(ValueError):
        m.flash_attn_varlen_func(q.to(DEV), k.to(DEV), v.to(DEV), cu.to(DEV), cu.to(DEV), 10, 40)
    bad = torch.tensor([0, 30, 20], dtype=torch.int32, device=DEV)
    with pytest.raises(ValueError):
        m.flash_attn_varlen_func(q.to(DEV), k.to(DEV), v.to(DEV), bad, bad, 40, 40)
    z = m.flash_attn_varlen_func(q[:0].to(DEV), k[:0].to(DEV), v[:0].to(DEV),
                                 torch.zeros(3, dtype=torch.int32, device=DEV),
                                 torch.zeros(3, dtype=torch.int32, device=DEV), 0, 0)
    assert z.shape == (0, 2, 64)


def test_config3_shape_reduced_and_full():
    """32 sequences, H32 D128, causal + window 1024 + ALiBi + softcap 30.  The oracle checks
    two whole sequences of a reduced-head run; the full-size run is checked through
    properties (finite, rows of V=1 give 1, agreement of the shared sequences)."""
    m = fa()
    rng = np.random.default_rng(3)
    lens = (64 * rng.integers(4, 65, size=32)).tolist()
    H, D = 32, 128
    T = sum(lens)
    g = torch.Generator(device=DEV).manual_seed(3)
    q = torch.randn(T, H, D, device=DEV, dtype=torch.float16, generator=g)
    k = torch.randn(T, H, D, device=DEV, dtype=torch.float16, generator=g)
    v = torch.randn(T, H, D, device=DEV, dtype=torch.float16, generator=g)
    cu = torch.tensor(np.concatenate([[0], np.cumsum(lens)]), dtype=torch.int32, device=DEV)
    sl = torch.tensor([2.0 ** (-8 * (i + 1) / H) for i in range(H)], device=DEV)
    kw = dict(causal=True, window_size=(1024, 0), alibi_slopes=sl, softcap=30.0)
    do = torch.randn(T, H, D, device=DEV, dtype=torch.float16, generator=g)
    qg, kg, vg = (t.detach().requires_grad_() for t in (q, k, v))
    out = m.flash_attn_varlen_func(qg, kg, vg, cu, cu, max(lens), max(lens), **kw)
    dq, dk, dv = torch.autograd.grad(out, (qg, kg, vg), do)
    out = out.detach()
    assert torch.isfinite(out).all() and all(torch.isfinite(t).all() for t in (dq, dk, dv))
    ones = m.flash_attn_varlen_func(q, k, torch.ones_like(v), cu, cu, max(lens), max(lens), **kw)
    assert (ones.float() - 1).abs().max().item() <= 2e-3
    # shortest, longest, first and last sequence against the oracle, 2 heads: output and gradients
    # (every head has its own K/V here, so a head's slice of the gradients is self-contained)
    for b in sorted({int(np.argmin(lens)), int(np.argmax(lens)), 0, len(lens) - 1}):
        s, e = int(cu[b]), int(cu[b + 1])
        hs = [0, H - 1]
        ro, _, rdq, rdk, rdv = orc.attention_grads_ref(
            q[s:e, hs].cpu()[None], k[s:e, hs].cpu()[None], v[s:e, hs].cpu()[None], do[s:e, hs].cpu()[None],
            causal=True, window=(1024, 0), softcap=30.0, alibi_slopes=sl[hs].cpu())
        assert maxdiff(out[s:e, hs], ro[0]) <= util.FWD_TOL, b
        for n, a, r in (("dq", dq, rdq), ("dk", dk, rdk), ("dv", dv, rdv)):
            assert maxdiff(a[s:e, hs], r[0]) <= util.GRAD_TOL, (b, n)
