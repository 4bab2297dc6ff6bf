"""The surfaces the reference serves from torch code and this library serves from kernels:
dropout (same Philox stream), attn_bias, return_attn_probs, seqused_q/k, paged packed K/V and
fp32 tensors.  Goldens come from the unmodified reference where it is deterministic (dropout with
Python's `random` seeded); the rest is checked against the CPU oracle."""
import ast
import random

import numpy as np
import pytest
import torch

import cases
import util
from oracle import attention_oracle as orc
from util import DEV, maxdiff

pytestmark = pytest.mark.gpu


def fa():
    import flash_attn_triton_b200 as m
    return m


def grads(out, do, leaves):
    return [g.cpu() for g in torch.autograd.grad((out.float() * do.to(DEV).float()).sum(), leaves)]


# ------------------------------------------------------------------------------------------------
# dropout
# ------------------------------------------------------------------------------------------------
def test_dropout_golden_dense(golden):
    """Same seed draw (random.randrange after random.seed), same counters, same backward formula as
    the reference: outputs and gradients match its own run."""
    g = golden("dropout")
    specs = ast.literal_eval(str(g["_specs"]))
    for i, (name, (B, Sq, Sk, Hq, Hkv, D, kw)) in enumerate(specs.items()):
        q, k, v, do = cases.dense_case(300 + i, B, Sq, Sk, Hq, Hkv, D)
        assert cases.checksum(q, k, v, do) == str(g[name + ".checksum"]), name
        qd, kd, vd = (t.to(DEV).requires_grad_() for t in (q, k, v))
        random.seed(4242 + i)
        out = fa().flash_attn_func(qd, kd, vd, **kw)
        dq, dk, dv = grads(out, do, (qd, kd, vd))
        amp = 1.0 / (1.0 - kw["dropout_p"])        # kept entries, and their rounding errors, are scaled by this
        assert maxdiff(out, g[name + ".out"]) <= util.FWD_TOL * amp, name
        for n, t in (("dq", dq), ("dk", dk), ("dv", dv)):
            assert maxdiff(t, g[f"{name}.{n}"]) <= util.GRAD_TOL * amp, (name, n)


def test_dropout_golden_varlen(golden):
    g = golden("dropout")
    ql, kl = g["varlen.q_lens"].tolist(), g["varlen.k_lens"].tolist()
    q, k, v, do, cu_q, cu_k = cases.varlen_case(9, ql, kl, 4, 2, 64)
    assert cases.checksum(q, k, v, do) == str(g["varlen.checksum"])
    qd, kd, vd = (t.to(DEV).requires_grad_() for t in (q, k, v))
    random.seed(99)
    out = fa().flash_attn_varlen_func(qd, kd, vd, cu_q.to(DEV), cu_k.to(DEV), 130, 101, dropout_p=0.2, causal=True)
    dq, dk, dv = grads(out, do, (qd, kd, vd))
    assert maxdiff(out, g["varlen.out"]) <= util.FWD_TOL / 0.8
    for n, t in (("dq", dq), ("dk", dk), ("dv", dv)):
        assert maxdiff(t, g["varlen." + n]) <= util.GRAD_TOL / 0.8, n


def test_dropout_golden_varlen_deterministic(golden):
    """deterministic=True walks the sequences like the reference does (one seed draw and dense
    dropout counters per sequence), so its masks are reproduced too."""
    g = golden("dropout")
    ql, kl = g["varlen.q_lens"].tolist(), g["varlen.k_lens"].tolist()
    q, k, v, do, cu_q, cu_k = cases.varlen_case(9, ql, kl, 4, 2, 64)
    qd, kd, vd = (t.to(DEV).requires_grad_() for t in (q, k, v))
    random.seed(77)
    out = fa().flash_attn_varlen_func(qd, kd, vd, cu_q.to(DEV), cu_k.to(DEV), 130, 101, dropout_p=0.2, causal=True,
                                      deterministic=True)
    dq, dk, dv = grads(out, do, (qd, kd, vd))
    assert maxdiff(out, g["varlen_det.out"]) <= util.FWD_TOL / 0.8
    for n, t in (("dq", dq), ("dk", dk), ("dv", dv)):
        assert maxdiff(t, g["varlen_det." + n]) <= util.GRAD_TOL / 0.8, n


@pytest.mark.parametrize("shape", [(2, 200, 200, 4, 2, 128), (1, 333, 150, 2, 2, 64), (1, 64, 64, 2, 1, 16),
                                   (1, 150, 150, 2, 2, 256)])
@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
def test_dropout_vs_oracle(shape, dtype):
    B, Sq, Sk, Hq, Hkv, D = shape
    q, k, v, do = (t.to(dtype) for t in cases.dense_case(310, B, Sq, Sk, Hq, Hkv, D))
    kw = dict(causal=True, window=(90, 40), softcap=12.0)
    qd, kd, vd = (t.to(DEV).requires_grad_() for t in (q, k, v))
    random.seed(7)
    seed = random.randrange(2 ** 31 - 1)
    random.seed(7)
    out, lse, probs = fa().flash_attn_func(qd, kd, vd, dropout_p=0.35, causal=True, window_size=(90, 40),
                                           softcap=12.0, return_attn_probs=True)
    dq, dk, dv = grads(out, do, (qd, kd, vd))
    ro, rl, rp, rdq, rdk, rdv = orc.attention_dropout_ref(q, k, v, do, dropout_p=0.35, seed=seed, **kw)
    f, gt = util.tols(dtype)
    amp = 1.0 / 0.65
    assert maxdiff(out, ro) <= f * amp
    assert maxdiff(probs, rp) <= 2e-3 * amp
    # the mask itself: exactly the same entries are dropped
    assert torch.equal(probs.cpu() == 0, rp == 0)
    fin = torch.isfinite(rl)
    assert maxdiff(lse.cpu()[fin], rl[fin]) <= f and torch.equal(torch.isfinite(lse.cpu()), fin)
    for n, a, b in (("dq", dq, rdq), ("dk", dk, rdk), ("dv", dv, rdv)):
        assert maxdiff(a, b) <= gt * amp, n


def test_dropout_statistics_and_determinism():
    """Property checks at a size the oracle does not reach: the drop rate, different masks for
    different seeds, the same mask for the same seed, no dropout when p = 0."""
    B, S, H, D = 1, 1024, 2, 64
    q, k, v, _ = cases.dense_case(311, B, S, S, H, H, D)
    qd, kd, vd = (t.to(DEV) for t in (q, k, v))
    random.seed(1)
    _, _, p1 = fa().flash_attn_func(qd, kd, vd, dropout_p=0.2, return_attn_probs=True)
    random.seed(1)
    o1b, _, p1b = fa().flash_attn_func(qd, kd, vd, dropout_p=0.2, return_attn_probs=True)
    random.seed(2)
    _, _, p2 = fa().flash_attn_func(qd, kd, vd, dropout_p=0.2, return_attn_probs=True)
    assert torch.equal(p1, p1b)
    rate = (p1 == 0).float().mean().item()
    assert abs(rate - 0.2) < 0.005
    assert (p1 == 0).ne(p2 == 0).float().mean().item() > 0.25        # independent masks differ in 2p(1-p) = 32 %
    # all heads and batches share the mask (the reference's counters do not include them)
    assert torch.equal(p1[0, 0] == 0, p1[0, 1] == 0)
    random.seed(1)
    o1 = fa().flash_attn_func(qd, kd, vd, dropout_p=0.2)
    assert torch.equal(o1, o1b)
    o0 = fa().flash_attn_func(qd, kd, vd, dropout_p=0.0)
    ro, _ = orc.attention_ref(q, k, v)
    assert maxdiff(o0, ro) <= util.FWD_TOL


def test_dropout_varlen_vs_oracle():
    ql, kl = [70, 5, 191, 64], [70, 9, 130, 64]
    q, k, v, do, cu_q, cu_k = cases.varlen_case(312, ql, kl, 4, 2, 128)
    qd, kd, vd = (t.to(DEV).requires_grad_() for t in (q, k, v))
    sl = torch.tensor([0.5, 0.25, 0.125, 0.0625])
    random.seed(11)
    seed = random.randrange(2 ** 31 - 1)
    random.seed(11)
    out, lse, probs = fa().flash_attn_varlen_func(qd, kd, vd, cu_q.to(DEV), cu_k.to(DEV), 200, 140, dropout_p=0.15,
                                                  causal=True, alibi_slopes=sl.to(DEV), return_attn_probs=True)
    dq, dk, dv = grads(out, do, (qd, kd, vd))
    ro, rl, rp, rdq, rdk, rdv = orc.varlen_attention_dropout_ref(q, k, v, cu_q, cu_k, 140, do, dropout_p=0.15,
                                                                seed=seed, causal=True, alibi_slopes=sl)
    amp = 1 / 0.85
    assert maxdiff(out, ro) <= util.FWD_TOL * amp
    assert probs.shape == (4, 4, 200, 140) and lse.shape == (4, 4, 200)
    for b in range(4):
        assert maxdiff(probs[b, :, :ql[b], :kl[b]], rp[b]) <= 2e-3 * amp
        assert probs[b, :, ql[b]:].abs().max().item() == 0 and probs[b, :, :, kl[b]:].abs().max().item() == 0
        want = rl[int(cu_q[b]):int(cu_q[b + 1])].transpose(0, 1)
        assert maxdiff(lse[b, :, :ql[b]], want) <= util.FWD_TOL
        assert torch.isinf(lse[b, :, ql[b]:]).all()
    for n, a, b in (("dq", dq, rdq), ("dk", dk, rdk), ("dv", dv, rdv)):
        assert maxdiff(a, b) <= util.GRAD_TOL * amp, n


# ------------------------------------------------------------------------------------------------
# attn_bias and return_attn_probs
# ------------------------------------------------------------------------------------------------
@pytest.mark.parametrize("bias_shape", ["full", "head", "row", "col"])
@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
def test_attn_bias(bias_shape, dtype):
    B, Sq, Sk, Hq, Hkv, D = 2, 150, 210, 4, 2, 64
    q, k, v, do = (t.to(dtype) for t in cases.dense_case(320, B, Sq, Sk, Hq, Hkv, D))
    shp = dict(full=(B, Hq, Sq, Sk), head=(1, Hq, 1, 1), row=(B, 1, Sq, 1), col=(1, 1, 1, Sk))[bias_shape]
    bias = torch.from_numpy(np.random.default_rng(321).standard_normal(shp).astype(np.float32)) * 2
    if bias_shape == "col":
        bias[..., 100:130] = float("-inf")           # a padding mask expressed as a bias
    qd, kd, vd = (t.to(DEV).requires_grad_() for t in (q, k, v))
    out = fa().flash_attn_func(qd, kd, vd, causal=(bias_shape != "col"), attn_bias=bias.to(DEV), softcap=20.0)
    dq, dk, dv = grads(out, do, (qd, kd, vd))
    ro, _, rdq, rdk, rdv = orc.attention_grads_ref(q, k, v, do, causal=(bias_shape != "col"), attn_bias=bias,
                                                   softcap=20.0)
    f, gt = util.tols(dtype)
    assert maxdiff(out, ro) <= f
    for n, a, b in (("dq", dq, rdq), ("dk", dk, rdk), ("dv", dv, rdv)):
        assert maxdiff(a, b) <= gt, n


def test_attn_bias_errors():
    q, k, v, _ = cases.dense_case(322, 1, 8, 8, 2, 2, 16)
    qd, kd, vd = (t.to(DEV) for t in (q, k, v))
    with pytest.raises(ValueError, match="broadcastable"):
        fa().flash_attn_func(qd, kd, vd, attn_bias=torch.zeros(3, 2, 8, 8, device=DEV))
    with pytest.raises(ValueError, match="require grad"):
        fa().flash_attn_func(qd, kd, vd, attn_bias=torch.zeros(1, 2, 8, 8, device=DEV, requires_grad=True))


@pytest.mark.parametrize("shape,kw", [
    ((2, 70, 70, 4, 2, 64), dict(causal=True)),
    ((1, 33, 129, 2, 2, 128), dict(window_size=(20, 10), softcap=9.0)),
    ((2, 129, 33, 2, 1, 32), dict(causal=True, alibi=True)),
    ((1, 300, 300, 2, 2, 256), dict(causal=True)),
    ((1, 17, 17, 2, 2, 16), dict()),
])
def test_return_attn_probs_dense(shape, kw):
    """(out, lse, probs) like the reference's dense return_attn_probs call
    (flash_attn_interface.py:15-49): natural-log LSE, fp32 probabilities, rows without a visible
    key all zero with lse = -inf; gradients still flow through `out`."""
    B, Sq, Sk, Hq, Hkv, D = shape
    q, k, v, do = cases.dense_case(330, B, Sq, Sk, Hq, Hkv, D)
    kw = dict(kw)
    okw = dict(causal=kw.get("causal", False), window=kw.get("window_size", (-1, -1)), softcap=kw.get("softcap", 0.0))
    if kw.pop("alibi", None):
        sl = torch.tensor([0.3, 0.07][:Hq])
        kw["alibi_slopes"], okw["alibi_slopes"] = sl.to(DEV), sl
    qd, kd, vd = (t.to(DEV).requires_grad_() for t in (q, k, v))
    out, lse, probs = fa().flash_attn_func(qd, kd, vd, return_attn_probs=True, **kw)
    assert probs.dtype == torch.float32 and probs.shape == (B, Hq, Sq, Sk) and lse.shape == (B, Hq, Sq)
    dq, dk, dv = grads(out, do, (qd, kd, vd))
    ro, rl, rdq, rdk, rdv = orc.attention_grads_ref(q, k, v, do, **okw)
    rp = torch.nan_to_num(torch.softmax(orc.scores_ref(q, k, None, okw["causal"], okw["window"], okw["softcap"],
                                                       okw.get("alibi_slopes")), dim=-1))
    assert maxdiff(out, ro) <= util.FWD_TOL
    assert maxdiff(probs, rp) <= 2e-3
    fin = torch.isfinite(rl)
    assert torch.equal(torch.isfinite(lse.cpu()), fin) and maxdiff(lse.cpu()[fin], rl[fin]) <= util.FWD_TOL
    for n, a, b in (("dq", dq, rdq), ("dk", dk, rdk), ("dv", dv, rdv)):
        assert maxdiff(a, b) <= util.GRAD_TOL, n


def test_return_attn_probs_cross_offset():
    q, k, v, _ = cases.dense_case(331, 1, 5, 40, 2, 2, 64)
    out, lse, probs = fa().flash_attn_func_cross(q.to(DEV), k.to(DEV), v.to(DEV), causal=True, return_attn_probs=True,
                                                 _causal_offset=35)
    ro, rl = orc.attention_ref(q, k, v, causal=True, q_pos_offset=35)
    assert maxdiff(out, ro) <= util.FWD_TOL and maxdiff(lse, rl) <= util.FWD_TOL
    assert probs[0, 0, 0, 36:].abs().max().item() == 0 and abs(probs[0, 0, 0].sum().item() - 1) < 1e-3


# ------------------------------------------------------------------------------------------------
# seqused_q / seqused_k, paged packed K/V
# ------------------------------------------------------------------------------------------------
@pytest.mark.parametrize("which", ["q", "k", "both"])
@pytest.mark.parametrize("causal", [False, True])
def test_seqused(which, causal):
    """seqused lengths are read by the kernels; results equal the reference's semantics of packing
    the used rows first (flash_attn_interface.py:552-581).  With seqused_q only the used query rows
    come back, packed."""
    ql, kl = [70, 33, 130, 8], [90, 33, 200, 8]
    uq, uk = [64, 0, 130, 3], [50, 33, 0, 8]
    q, k, v, do, cu_q, cu_k = cases.varlen_case(340, ql, kl, 4, 2, 64)
    kw = {}
    q2, k2, v2, cq2, ck2 = q, k, v, cu_q.tolist(), cu_k.tolist()
    iq = torch.arange(q.shape[0])
    ik = torch.arange(k.shape[0])
    if which in ("q", "both"):
        kw["seqused_q"] = torch.tensor(uq, device=DEV)
        iq, cq2 = orc.seqused_view(cu_q, uq)
        q2 = q[iq]
    if which in ("k", "both"):
        kw["seqused_k"] = uk                           # a plain list is accepted too
        ik, ck2 = orc.seqused_view(cu_k, uk)
        k2, v2 = k[ik], v[ik]
    do2 = do[iq]
    qd, kd, vd = (t.to(DEV).requires_grad_() for t in (q, k, v))
    out = fa().flash_attn_varlen_func(qd, kd, vd, cu_q.to(DEV), cu_k.to(DEV), 130, 200, causal=causal, **kw)
    assert out.shape[0] == q2.shape[0]
    dq, dk, dv = grads(out, do2, (qd, kd, vd))
    ro, _, rdq, rdk, rdv = orc.varlen_attention_grads_ref(q2, k2, v2, do2, cq2, ck2, causal=causal)
    assert maxdiff(out, ro) <= util.FWD_TOL
    full = lambda g, idx, like: torch.zeros(like.shape).index_copy_(0, idx, g)
    assert maxdiff(dq, full(rdq, iq, q)) <= util.GRAD_TOL
    assert maxdiff(dk, full(rdk, ik, k)) <= util.GRAD_TOL
    assert maxdiff(dv, full(rdv, ik, v)) <= util.GRAD_TOL


def test_seqused_errors():
    q, k, v, do, cu_q, cu_k = cases.varlen_case(341, [5, 6], [5, 6], 2, 2, 16)
    a = (q.to(DEV), k.to(DEV), v.to(DEV), cu_q.to(DEV), cu_k.to(DEV), 6, 6)
    with pytest.raises(ValueError, match="one value per sequence"):
        fa().flash_attn_varlen_func(*a, seqused_q=[1])
    with pytest.raises(ValueError, match="seqused_q exceeds"):
        fa().flash_attn_varlen_func(*a, seqused_q=[6, 6])
    with pytest.raises(ValueError, match="seqused_k exceeds"):
        fa().flash_attn_varlen_func(*a, seqused_k=[5, -1])


def test_seqused_q_with_dropout():
    """The one combination that is packed on the host first, so that the dropout counters run over
    the packed rows as the reference's do."""
    ql, kl, uq = [70, 33], [70, 33], [10, 33]
    q, k, v, do, cu_q, cu_k = cases.varlen_case(342, ql, kl, 2, 2, 64)
    iq, cq2 = orc.seqused_view(cu_q, uq)
    random.seed(5)
    seed = random.randrange(2 ** 31 - 1)
    random.seed(5)
    out = fa().flash_attn_varlen_func(q.to(DEV), k.to(DEV), v.to(DEV), cu_q.to(DEV), cu_k.to(DEV), 70, 70,
                                      dropout_p=0.3, seqused_q=uq)
    ro, _, _ = orc.varlen_attention_dropout_ref(q[iq], k, v, cq2, cu_k, 70, dropout_p=0.3, seed=seed)
    assert maxdiff(out, ro) <= util.FWD_TOL / 0.7


@pytest.mark.parametrize("page_size", [16, 64])
def test_paged_varlen(page_size):
    """k/v as (pages, page_size, heads, dim) + block_table: gathered on the device, results and
    gradients as if the caller had packed them (flash_attn_interface.py:533-550)."""
    ql, kl = [40, 100, 7], [75, 130, 16]
    H, Hkv, D = 4, 2, 64
    rng = np.random.default_rng(350)
    q = cases.randn16(rng, sum(ql), H, D)
    do = cases.randn16(rng, sum(ql), H, D)
    n_pages = 40
    kp = cases.randn16(rng, n_pages, page_size, Hkv, D)
    vp = cases.randn16(rng, n_pages, page_size, Hkv, D)
    max_pages = (max(kl) + page_size - 1) // page_size
    perm = rng.permutation(n_pages)[:3 * max_pages].reshape(3, max_pages)
    bt = torch.from_numpy(perm.astype(np.int32))
    cu_q = torch.tensor([0] + np.cumsum(ql).tolist(), dtype=torch.int32)
    cu_k = torch.tensor([0] + np.cumsum(kl).tolist(), dtype=torch.int32)
    qd, kd, vd = (t.to(DEV).requires_grad_() for t in (q, kp, vp))
    out = fa().flash_attn_varlen_func(qd, kd, vd, cu_q.to(DEV), cu_k.to(DEV), 100, 130, causal=True,
                                      block_table=bt.to(DEV))
    dq, dk, dv = grads(out, do, (qd, kd, vd))
    k2, v2 = orc.unpage_ref(kp, bt, cu_k), orc.unpage_ref(vp, bt, cu_k)
    ro, _, rdq, rdk, rdv = orc.varlen_attention_grads_ref(q, k2, v2, do, cu_q, cu_k, causal=True)
    assert maxdiff(out, ro) <= util.FWD_TOL and maxdiff(dq, rdq) <= util.GRAD_TOL
    # gradients land in the pages the tokens came from, every other slot is zero
    want_k, want_v = torch.zeros(kp.shape), torch.zeros(vp.shape)
    for b in range(3):
        for i in range(kl[b]):
            pg = int(bt[b, i // page_size])
            want_k[pg, i % page_size] = rdk[int(cu_k[b]) + i]
            want_v[pg, i % page_size] = rdv[int(cu_k[b]) + i]
    assert maxdiff(dk, want_k) <= util.GRAD_TOL and maxdiff(dv, want_v) <= util.GRAD_TOL
    with pytest.raises(ValueError, match="invalid physical page"):
        bad = bt.clone()
        bad[0, 0] = n_pages
        fa().flash_attn_varlen_func(qd, kd, vd, cu_q.to(DEV), cu_k.to(DEV), 100, 130, block_table=bad.to(DEV))
    with pytest.raises(ValueError, match="block_table must have shape"):
        fa().flash_attn_varlen_func(qd, kd, vd, cu_q.to(DEV), cu_k.to(DEV), 100, 130, block_table=bt[:2].to(DEV))


def test_return_attn_probs_varlen():
    ql, kl = [37, 64, 5], [50, 64, 0]
    q, k, v, do, cu_q, cu_k = cases.varlen_case(360, ql, kl, 4, 2, 64)
    out, lse, probs = fa().flash_attn_varlen_func(q.to(DEV), k.to(DEV), v.to(DEV), cu_q.to(DEV), cu_k.to(DEV), 64, 64,
                                                  causal=True, window_size=(30, 0), return_attn_probs=True)
    ro, rl, rp = orc.varlen_attention_dropout_ref(q, k, v, cu_q, cu_k, 64, causal=True, window=(30, 0))
    assert maxdiff(out, ro) <= util.FWD_TOL
    for b in range(3):
        assert maxdiff(probs[b, :, :ql[b], :kl[b]], rp[b]) <= 2e-3
        if kl[b]:
            assert maxdiff(lse[b, :, :ql[b]], rl[int(cu_q[b]):int(cu_q[b + 1])].transpose(0, 1)) <= util.FWD_TOL
        else:
            assert torch.isinf(lse[b]).all()


# ------------------------------------------------------------------------------------------------
# fp32 tensors
# ------------------------------------------------------------------------------------------------
def test_fp32_inputs():
    """fp32 q/k/v are accepted (flash_attn_interface.py:97 of the reference), computed with fp16
    operands and fp32 accumulation, and returned as fp32 with fp32 gradients."""
    q, k, v, do = (t.float() for t in cases.dense_case(370, 2, 100, 100, 4, 2, 64))
    qd, kd, vd = (t.to(DEV).requires_grad_() for t in (q, k, v))
    out = fa().flash_attn_func(qd, kd, vd, causal=True)
    assert out.dtype == torch.float32
    dq, dk, dv = grads(out, do, (qd, kd, vd))
    assert dq.dtype == torch.float32
    ro, _, rdq, rdk, rdv = orc.attention_grads_ref(q, k, v, do, causal=True)
    assert maxdiff(out, ro) <= util.FWD_TOL
    for n, a, b in (("dq", dq, rdq), ("dk", dk, rdk), ("dv", dv, rdv)):
        assert maxdiff(a, b) <= util.GRAD_TOL, n
    ql = [30, 70]
    q, k, v, do, cu_q, cu_k = cases.varlen_case(371, ql, ql, 2, 2, 32)
    out = fa().flash_attn_varlen_func(q.float().to(DEV), k.float().to(DEV), v.float().to(DEV), cu_q.to(DEV),
                                      cu_k.to(DEV), 70, 70, causal=True)
    ro, _ = orc.varlen_attention_ref(q, k, v, cu_q, cu_k, causal=True)
    assert out.dtype == torch.float32 and maxdiff(out, ro) <= util.FWD_TOL
