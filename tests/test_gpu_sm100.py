"""The tcgen05/TMEM/TMA kernels, forced on (FA_IMPL_TCGEN05) at sizes below the automatic
switch-over too, against the fp32 oracle and against the independent mma.sync kernels."""
import numpy as np
import pytest
import torch

import cases
import util
from oracle import attention_oracle as orc
from util import DEV, LN2, maxdiff

pytestmark = pytest.mark.gpu

SHAPES = [
    # B, Sq, Sk, Hq, Hkv, D
    (1, 128, 128, 1, 1, 128),
    (2, 512, 512, 2, 1, 128),
    (1, 300, 300, 2, 2, 128),
    (2, 1000, 777, 4, 2, 128),
    (1, 384, 384, 2, 2, 64),
    (2, 100, 900, 2, 1, 64),
    (1, 640, 640, 8, 2, 128),
]
FEATS = [
    dict(causal=False), dict(causal=True), dict(causal=True, wl=100, wr=0), dict(causal=False, wl=50, wr=70),
    dict(causal=True, softcap=10.0), dict(causal=True, alibi=True),
    dict(causal=True, wl=200, wr=0, softcap=30.0, alibi=True),
    # keys on both sides of the diagonal: ALiBi needs |distance|
    dict(causal=False, alibi=True), dict(causal=False, wl=300, wr=100, softcap=20.0, alibi=True),
]


def _run(impl, q, k, v, do, scale, kw, alibi):
    from flash_attn_triton_b200 import _ops
    args = (scale, kw.get("causal", False), kw.get("wl", -1), kw.get("wr", -1), kw.get("softcap", 0.0), alibi, 0)
    o, lse, _ = _ops.dense_forward(q, k, v, *args, impl, "bshd", True)
    dq, dk, dv = _ops.dense_backward(q, k, v, o, lse, do, *args, impl, "bshd")
    return o, lse, dq, dk, dv


@pytest.mark.parametrize("shape", SHAPES, ids=lambda s: "x".join(map(str, s)))
@pytest.mark.parametrize("feat", range(len(FEATS)))
def test_tcgen05_forward_backward(shape, feat):
    from flash_attn_triton_b200 import _native as N
    B, Sq, Sk, Hq, Hkv, D = shape
    kw = FEATS[feat]
    q, k, v, do = cases.dense_case(2000 + feat, B, Sq, Sk, Hq, Hkv, D)
    sl = torch.tensor([[2.0 ** (-(i + 1)) for i in range(Hq)]] * B) if kw.get("alibi") else None
    scale = 0.1 if feat >= 2 else 1.0 / np.sqrt(D)
    out = _run(N.IMPL_TCGEN05, *(t.to(DEV) for t in (q, k, v, do)), scale, kw, None if sl is None else sl.to(DEV))
    assert N.lib().fa_device_wait_status(0) == 0
    ro, rl, rdq, rdk, rdv = orc.attention_grads_ref(
        q, k, v, do, softmax_scale=scale, causal=kw.get("causal", False),
        window=(kw.get("wl", -1), kw.get("wr", -1)), softcap=kw.get("softcap", 0.0), alibi_slopes=sl)
    assert maxdiff(out[0], ro) <= util.FWD_TOL
    assert maxdiff(out[1] * LN2, rl) <= util.FWD_TOL
    for t, r in zip(out[2:], (rdq, rdk, rdv)):
        assert maxdiff(t, r) <= util.GRAD_TOL


def test_tcgen05_varlen_and_bf16():
    from flash_attn_triton_b200 import _native as N, _ops
    ql = [200, 129, 640, 64]
    q, k, v, do, cu, _ = cases.varlen_case(77, ql, ql, 8, 2, 128)
    sl = torch.tensor([[2.0 ** (-8 * (i + 1) / 8) for i in range(8)]] * 4)
    args = (max(ql), max(ql), 0.09, True, 150, 0, 30.0, sl.to(DEV))
    qd, kd, vd, dod, cud = (t.to(DEV) for t in (q, k, v, do, cu))
    o, lse, _ = _ops.varlen_forward(qd, kd, vd, cud, cud, *args, N.IMPL_TCGEN05, True)
    dq, dk, dv = _ops.varlen_backward(qd, kd, vd, o, lse, dod, cud, cud, *args, N.IMPL_TCGEN05)
    assert N.lib().fa_device_wait_status(0) == 0
    ro, _, rdq, rdk, rdv = orc.varlen_attention_grads_ref(q, k, v, do, cu, cu, softmax_scale=0.09, causal=True,
                                                          window=(150, 0), softcap=30.0, alibi_slopes=sl[0])
    assert maxdiff(o, ro) <= util.FWD_TOL
    for t, r in zip((dq, dk, dv), (rdq, rdk, rdv)):
        assert maxdiff(t, r) <= util.GRAD_TOL
    # bf16
    q, k, v, do = (t.bfloat16() for t in cases.dense_case(78, 2, 400, 400, 4, 2, 128))
    out = _run(N.IMPL_TCGEN05, *(t.to(DEV) for t in (q, k, v, do)), 0.088, dict(causal=True), None)
    ro, _, rdq, rdk, rdv = orc.attention_grads_ref(q, k, v, do, softmax_scale=0.088, causal=True)
    assert maxdiff(out[0], ro) <= util.BF16_FWD_TOL
    for t, r in zip(out[2:], (rdq, rdk, rdv)):
        assert maxdiff(t, r) <= util.BF16_GRAD_TOL


def test_tcgen05_agrees_with_mma_at_full_size():
    """B16 H16 S4096 D128 causal: two independent implementations of every kernel."""
    from flash_attn_triton_b200 import _native as N
    torch.manual_seed(1)
    q, k, v, do = (torch.randn(16, 4096, 16, 128, device=DEV, dtype=torch.float16) for _ in range(4))
    a = _run(N.IMPL_TCGEN05, q, k, v, do, 128 ** -0.5, dict(causal=True), None)
    assert N.lib().fa_device_wait_status(0) == 0
    b = _run(N.IMPL_MMA, q, k, v, do, 128 ** -0.5, dict(causal=True), None)
    assert (a[0].float() - b[0].float()).abs().max().item() <= util.FWD_TOL
    assert maxdiff(a[1], b[1]) <= util.FWD_TOL
    for x, y in zip(a[2:], b[2:]):
        assert (x.float() - y.float()).abs().max().item() <= util.GRAD_TOL


def test_tcgen05_forward_query_tile_without_keys():
    """A 256-row CTA whose second query tile sees no key at all (window far left of the rows):
    that tile's output must be exactly zero and its LSE -inf, whatever the output buffer held
    before -- the zeros are staged over the tile's Q slot and must not race with the Q load."""
    from flash_attn_triton_b200 import _native as N, _ops
    B, Sq, Sk, Hq, Hkv, D = 2, 1000, 777, 4, 2, 128
    q, k, v, _ = cases.dense_case(2003, B, Sq, Sk, Hq, Hkv, D)
    qd, kd, vd = (t.to(DEV) for t in (q, k, v))
    args = (0.1, False, 50, 70, 0.0, None, 0)
    for _ in range(4):
        junk = torch.full((B, Sq, Hq, D), 7.0, dtype=torch.float16, device=DEV)
        del junk  # the caching allocator hands this block to the forward's output
        o, lse, _ = _ops.dense_forward(qd, kd, vd, *args, N.IMPL_TCGEN05, "bshd", True)
        assert N.lib().fa_device_wait_status(0) == 0
        empty_rows = slice(Sk + 50, Sq)  # query positions whose window [q-50, q+70] lies past the last key
        assert torch.count_nonzero(o[:, empty_rows]).item() == 0
        assert torch.isinf(lse[:, :, empty_rows]).all() and (lse[:, :, empty_rows] < 0).all()


@pytest.mark.parametrize("shape", SHAPES, ids=lambda s: "x".join(map(str, s)))
@pytest.mark.parametrize("feat", [0, 1, 3, 6])
def test_persistent_forward_on_small_shapes(shape, feat, monkeypatch):
    """The persistent forward kernel normally takes calls from 2048 keys up; here it is forced on
    for the small shapes (ragged tiles, streams without tiles, items of one step) and must agree
    with the oracle and, bit for bit, with the one-CTA-per-item kernel."""
    from flash_attn_triton_b200 import _native as N, _ops
    B, Sq, Sk, Hq, Hkv, D = shape
    kw = FEATS[feat]
    q, k, v, do = cases.dense_case(2100 + feat, B, Sq, Sk, Hq, Hkv, D)
    sl = torch.tensor([[2.0 ** (-(i + 1)) for i in range(Hq)]] * B) if kw.get("alibi") else None
    scale = 0.1 if feat >= 2 else 1.0 / np.sqrt(D)
    args = (scale, kw.get("causal", False), kw.get("wl", -1), kw.get("wr", -1), kw.get("softcap", 0.0),
            None if sl is None else sl.to(DEV), 0)
    qd, kd, vd = (t.to(DEV) for t in (q, k, v))
    monkeypatch.setenv("FA_B200_FWD_POLY", "0")       # both kernels with every exponential on the MUFU
    monkeypatch.setenv("FA_B200_FWD_PERSISTENT_FROM", "0")
    o0, l0, _ = _ops.dense_forward(qd, kd, vd, *args, N.IMPL_TCGEN05, "bshd", True)
    monkeypatch.setenv("FA_B200_FWD_PERSISTENT_FROM", "1")
    o1, l1, _ = _ops.dense_forward(qd, kd, vd, *args, N.IMPL_TCGEN05, "bshd", True)
    o2, l2, _ = _ops.dense_forward(qd, kd, vd, *args, N.IMPL_TCGEN05, "bshd", True)
    assert N.lib().fa_device_wait_status(0) == 0
    assert torch.equal(o1, o2) and torch.equal(l1, l2)
    assert torch.equal(o0, o1) and torch.equal(l0, l1)
    ro, rl = orc.attention_ref(q, k, v, softmax_scale=scale, causal=kw.get("causal", False),
                               window=(kw.get("wl", -1), kw.get("wr", -1)), softcap=kw.get("softcap", 0.0),
                               alibi_slopes=sl)
    assert maxdiff(o1, ro) <= util.FWD_TOL and maxdiff(l1 * LN2, rl) <= util.FWD_TOL


@pytest.mark.parametrize("shape", SHAPES, ids=lambda s: "x".join(map(str, s)))
@pytest.mark.parametrize("feat", [0, 1, 3])
def test_persistent_forward_with_fma_pipe_exponentials(shape, feat, monkeypatch):
    """The variant of the persistent forward that the host picks for long items (a quarter of the
    exponentials of unmasked tiles as a polynomial on the FMA pipe, scores re-read from tensor
    memory), forced on for the small shapes: the oracle's bars hold and two runs agree bit for bit."""
    from flash_attn_triton_b200 import _native as N, _ops
    B, Sq, Sk, Hq, Hkv, D = shape
    kw = FEATS[feat]
    q, k, v, do = cases.dense_case(2300 + feat, B, Sq, Sk, Hq, Hkv, D)
    scale = 0.1 if feat >= 2 else 1.0 / np.sqrt(D)
    args = (scale, kw.get("causal", False), kw.get("wl", -1), kw.get("wr", -1), 0.0, None, 0)
    qd, kd, vd, dod = (t.to(DEV) for t in (q, k, v, do))
    monkeypatch.setenv("FA_B200_FWD_PERSISTENT_FROM", "1")
    monkeypatch.setenv("FA_B200_FWD_POLY", "1")
    o1, l1, _ = _ops.dense_forward(qd, kd, vd, *args, N.IMPL_TCGEN05, "bshd", True)
    o2, l2, _ = _ops.dense_forward(qd, kd, vd, *args, N.IMPL_TCGEN05, "bshd", True)
    dq, dk, dv = _ops.dense_backward(qd, kd, vd, o1, l1, dod, *args, N.IMPL_TCGEN05, "bshd")
    assert N.lib().fa_device_wait_status(0) == 0
    assert torch.equal(o1, o2) and torch.equal(l1, l2)
    ro, rl, rdq, rdk, rdv = orc.attention_grads_ref(q, k, v, do, softmax_scale=scale, causal=kw.get("causal", False),
                                                    window=(kw.get("wl", -1), kw.get("wr", -1)))
    assert maxdiff(o1, ro) <= util.FWD_TOL and maxdiff(l1 * LN2, rl) <= util.FWD_TOL
    # the backward takes this forward's LSE
    for t, r in zip((dq, dk, dv), (rdq, rdk, rdv)):
        assert maxdiff(t, r) <= util.GRAD_TOL


def test_persistent_forward_packed(monkeypatch):
    from flash_attn_triton_b200 import _native as N, _ops
    lens = [100, 60, 300, 513, 1]
    q, k, v, do, cu_q, cu_k = cases.varlen_case(2200, lens, lens, 4, 2, 128)
    args = (cu_q.to(DEV), cu_k.to(DEV), 513, 513, 128 ** -0.5, True, 200, 0, 0.0, None)
    monkeypatch.setenv("FA_B200_FWD_PERSISTENT_FROM", "0")
    o0, l0, _ = _ops.varlen_forward(q.to(DEV), k.to(DEV), v.to(DEV), *args, N.IMPL_TCGEN05, True)
    monkeypatch.setenv("FA_B200_FWD_PERSISTENT_FROM", "1")
    o1, l1, _ = _ops.varlen_forward(q.to(DEV), k.to(DEV), v.to(DEV), *args, N.IMPL_TCGEN05, True)
    assert N.lib().fa_device_wait_status(0) == 0
    assert torch.equal(o0, o1) and torch.equal(l0, l1)
    ro, _ = orc.varlen_attention_ref(q, k, v, cu_q, cu_k, causal=True, window=(200, 0))
    assert maxdiff(o1, ro) <= util.FWD_TOL


@pytest.mark.parametrize("shape,kw", [
    ((1, 16384, 16384, 2, 1, 128), dict(causal=True)),              # 128 key tiles per work item
    ((1, 16384, 16384, 1, 1, 64), dict(causal=True, wl=3000)),      # a window that ends inside tiles
    ((1, 700, 20000, 2, 2, 128), dict()),                           # short queries over a long context
], ids=["causal16k", "window16k", "cross20k"])
def test_long_sequences_vs_oracle(shape, kw):
    """Sequences far beyond the benchmark's 4096: the ring positions, barrier parities and the work
    queue of the persistent kernels wrap many times inside one item; every output and gradient
    against the fp32 oracle."""
    from flash_attn_triton_b200 import _native as N
    B, Sq, Sk, Hq, Hkv, D = shape
    q, k, v, do = cases.dense_case(4242, B, Sq, Sk, Hq, Hkv, D)
    scale = 1.0 / np.sqrt(D)
    out = _run(N.IMPL_TCGEN05, *(t.to(DEV) for t in (q, k, v, do)), scale, kw, None)
    assert N.lib().fa_device_wait_status(0) == 0
    ro, rl, rdq, rdk, rdv = orc.attention_grads_ref(q, k, v, do, softmax_scale=scale, causal=kw.get("causal", False),
                                                    window=(kw.get("wl", -1), kw.get("wr", -1)))
    assert maxdiff(out[0], ro) <= util.FWD_TOL
    assert maxdiff(out[1] * LN2, rl) <= util.FWD_TOL
    for t, r in zip(out[2:], (rdq, rdk, rdv)):
        assert maxdiff(t, r) <= util.GRAD_TOL


@pytest.mark.parametrize("shape", [(2, 512, 512, 2, 1, 128), (1, 640, 640, 8, 2, 128), (1, 384, 384, 2, 2, 64),
                                   (2, 1000, 777, 4, 2, 128)], ids=lambda s: "x".join(map(str, s)))
@pytest.mark.parametrize("causal", [False, True])
def test_both_dkdv_kernels_on_dense_shapes(shape, causal, monkeypatch):
    """Plain dense problems go to the one-CTA-per-key-block dK/dV kernel; the persistent kernel (packed
    batches, feature variants) is forced onto the same shapes here: both meet the oracle's bar and
    each is bit-identical from run to run."""
    from flash_attn_triton_b200 import _native as N, _ops
    B, Sq, Sk, Hq, Hkv, D = shape
    q, k, v, do = cases.dense_case(2500, B, Sq, Sk, Hq, Hkv, D)
    scale = 1.0 / np.sqrt(D)
    args = (scale, causal, -1, -1, 0.0, None, 0)
    qd, kd, vd, dod = (t.to(DEV) for t in (q, k, v, do))
    o, lse, _ = _ops.dense_forward(qd, kd, vd, *args, N.IMPL_TCGEN05, "bshd", True)
    _, _, _, rdk, rdv = orc.attention_grads_ref(q, k, v, do, softmax_scale=scale, causal=causal)
    for below in ("0", "1e9"):
        monkeypatch.setenv("FA_B200_DKDV_CTA_BELOW", below)
        _, dk1, dv1 = _ops.dense_backward(qd, kd, vd, o, lse, dod, *args, N.IMPL_TCGEN05, "bshd")
        _, dk2, dv2 = _ops.dense_backward(qd, kd, vd, o, lse, dod, *args, N.IMPL_TCGEN05, "bshd")
        assert N.lib().fa_device_wait_status(0) == 0
        assert torch.equal(dk1, dk2) and torch.equal(dv1, dv2)
        assert maxdiff(dk1, rdk) <= util.GRAD_TOL and maxdiff(dv1, rdv) <= util.GRAD_TOL
