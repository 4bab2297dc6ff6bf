"""INT8 path parity: bit-exact K codes/scales, INT8-QK^T forward, fp16 backward."""
import numpy as np
import pytest
import torch

import cases
import util
from oracle import attention_oracle as orc
from util import DEV, maxdiff

pytestmark = pytest.mark.gpu
INT8_GRAD_TOL = 5e-2  # the reference's own bar for this path (tests/test_compare_implementations.py:27)


def test_golden_k_quantiser_bit_exact(golden):
    from flash_attn_triton_b200 import _ops
    g = golden("int8_kquant")
    k = cases.k_with_outliers(21, 4, 192, 128)
    assert cases.checksum(k) == str(g["checksum"])
    k8, s_k = _ops.quantize_k_int8(k.to(DEV))
    assert np.array_equal(k8.cpu().numpy(), g["k8"])
    assert np.array_equal(s_k.cpu().numpy().view(np.uint32), g["s_k"].view(np.uint32))


@pytest.mark.parametrize("D", [32, 64, 128, 256])
def test_k_quantiser_bit_exact_vs_oracle(D):
    from flash_attn_triton_b200 import _ops
    k = cases.k_with_outliers(500 + D, 3, 5, 333, D)
    # rounding ties and the amax<1 clamp
    k[0, 0, 0] = 0.0
    k[0, 0, 1, :] = 0.25
    k[0, 0, 2, 0] = 127.0
    k[0, 0, 2, 1:] = torch.linspace(-60, 60, D - 1).half() + 0.5
    k8, s_k = _ops.quantize_k_int8(k.to(DEV))
    r8, rs = orc.quantize_k_rows_ref(k)
    assert np.array_equal(k8.cpu().numpy(), r8)
    assert np.array_equal(s_k.cpu().numpy().view(np.uint32), rs.view(np.uint32))


@pytest.mark.parametrize("causal", [0, 1])
def test_golden_int8_forward(golden, causal):
    from flash_attn_triton_b200 import _ops
    g = golden(f"int8_fwd_causal{causal}")
    q, k, v = cases.int8_case(30, 1, 2, 256, 128)
    assert cases.checksum(q, k, v) == str(g["checksum"])
    o, lse, _, _ = _ops.int8_forward(q.to(DEV), k.to(DEV), v.to(DEV), bool(causal), 1.0 / 128 ** 0.5)
    assert maxdiff(o, g["out"]) <= util.FWD_TOL
    assert maxdiff(lse, g["lse2"]) <= util.FWD_TOL


@pytest.mark.parametrize("shape", [(2, 2, 128, 64), (1, 3, 320, 128), (1, 1, 64, 32), (1, 2, 192, 256)])
@pytest.mark.parametrize("causal", [False, True])
def test_int8_forward_backward_vs_oracle(shape, causal):
    import flash_attn_triton_b200 as fa
    B, H, S, D = shape
    q, k, v = cases.int8_case(600 + S, B, H, S, D)
    do = torch.from_numpy(np.random.default_rng(S).standard_normal((B, H, S, D), dtype=np.float32)).half()
    qd, kd, vd = (t.to(DEV).requires_grad_() for t in (q, k, v))
    out = fa.attention_int8(qd, kd, vd, causal=causal, sm_scale=0.125)
    ro, _, _, _ = orc.attention_int8_ref(q, k, v, causal=causal, sm_scale=0.125)
    assert maxdiff(out, ro) <= util.FWD_TOL
    dq, dk, dv = torch.autograd.grad((out.float() * do.to(DEV).float()).sum(), (qd, kd, vd))
    # backward = fp16 dense backward with the INT8 forward's LSE and output
    # (attention_kernel_int8.py:256-267), restated by attention_int8_grads_ref
    rdq, rdk, rdv = orc.attention_int8_grads_ref(q, k, v, do, causal=causal, sm_scale=0.125)
    # K carries x8 outliers, so dq reaches magnitudes of 20-30 where one fp16 rounding step
    # of the stored gradient is already 1.6e-2: allow that step on top of the 1e-2 bar
    for t, r in ((dq, rdq), (dk, rdk), (dv, rdv)):
        assert util.excess(t, r) <= util.GRAD_TOL


@pytest.mark.parametrize("causal", [0, 1])
def test_golden_int8_backward(golden, causal):
    """Shape of the reference's own INT8 test: gradients of the reference, and (without K
    outliers) its 5e-2 bar against the fp32 attention gradients."""
    import flash_attn_triton_b200 as fa
    g = golden(f"int8_bwd_causal{causal}")
    q, k, v = cases.int8_case(31, 2, 2, 128, 64)
    do = cases.randn16(np.random.default_rng(32), 2, 2, 128, 64)
    qd, kd, vd = (t.to(DEV).requires_grad_() for t in (q, k, v))
    out = fa.attention_int8(qd, kd, vd, causal=bool(causal), sm_scale=0.125)
    dq, dk, dv = torch.autograd.grad((out.float() * do.to(DEV).float()).sum(), (qd, kd, vd))
    assert maxdiff(out, g["out"]) <= util.FWD_TOL
    for n, t in (("dq", dq), ("dk", dk), ("dv", dv)):
        assert maxdiff(t, g[n]) <= util.GRAD_TOL, n
    rng = np.random.default_rng(9)
    q, k, v, do = (cases.randn16(rng, 2, 2, 128, 64) for _ in range(4))
    qd, kd, vd = (t.to(DEV).requires_grad_() for t in (q, k, v))
    out = fa.attention_int8(qd, kd, vd, causal=bool(causal), sm_scale=0.125)
    grads = torch.autograd.grad((out.float() * do.to(DEV).float()).sum(), (qd, kd, vd))
    tr = lambda t: t.transpose(1, 2)
    ro, _, rdq, rdk, rdv = orc.attention_grads_ref(tr(q), tr(k), tr(v), tr(do), softmax_scale=0.125,
                                                   causal=bool(causal))
    assert maxdiff(tr(out), ro) <= INT8_GRAD_TOL
    for t, r in zip(grads, (rdq, rdk, rdv)):
        assert util.excess(tr(t), r, rel=2e-2) <= INT8_GRAD_TOL  # atol and rtol of the reference's test


@pytest.mark.parametrize("causal", [0, 1])
def test_golden_int8_padded(golden, causal):
    """A padded call: 150 valid tokens in 192 rows, seq_len_k = seq_len_q = 150
    (attention_kernel_int8.py:108-118, :245), against the reference's outputs and gradients."""
    import flash_attn_triton_b200 as fa
    g = golden(f"int8_padded_causal{causal}")
    q, k, v = cases.int8_case(33, 1, 2, 192, 64)
    do = cases.randn16(np.random.default_rng(34), 1, 2, 192, 64)
    qd, kd, vd = (t.to(DEV).requires_grad_() for t in (q, k, v))
    out = fa.attention_int8(qd, kd, vd, causal=bool(causal), sm_scale=0.125, seq_len_k=150, seq_len_q=150)
    dq, dk, dv = torch.autograd.grad((out.float() * do.to(DEV).float()).sum(), (qd, kd, vd))
    assert maxdiff(out, g["out"]) <= util.FWD_TOL
    # the reference's dq of the padded query rows is not meaningful under a causal mask (it skips
    # the key-length mask there); everything a caller keeps is compared
    assert maxdiff(dq[:, :, :150], g["dq"][:, :, :150]) <= util.GRAD_TOL
    assert maxdiff(dk, g["dk"]) <= util.GRAD_TOL and maxdiff(dv, g["dv"]) <= util.GRAD_TOL
    assert not dk[:, :, 150:].any() and not dv[:, :, 150:].any()
    # D = 128 takes the tcgen05 kernel: same call against the oracle, with a causal offset too
    q, k, v = cases.int8_case(35, 1, 2, 320, 128)
    for lk, lq in ((300, 300), (257, 200)):
        o = fa.attention_int8(q.to(DEV), k.to(DEV), v.to(DEV), causal=bool(causal), seq_len_k=lk, seq_len_q=lq)
        ro, _, _, _ = orc.attention_int8_ref(q, k, v, causal=bool(causal), seq_len_k=lk, seq_len_q=lq)
        assert maxdiff(o, ro) <= util.FWD_TOL, (lk, lq)
    with pytest.raises(ValueError):
        fa.attention_int8(q.to(DEV), k.to(DEV), v.to(DEV), seq_len_k=321)


def test_int8_value_errors():
    import flash_attn_triton_b200 as fa
    q = torch.zeros(1, 1, 64, 64, device=DEV, dtype=torch.float16)
    with pytest.raises(ValueError):
        fa.attention_int8(q[..., :16], q[..., :16], q[..., :16])
    with pytest.raises(ValueError):
        fa.attention_int8(q[:, :, :50], q[:, :, :50], q[:, :, :50])
    with pytest.raises(ValueError):
        fa.attention_int8(q.transpose(1, 2), q.transpose(1, 2), q.transpose(1, 2).contiguous())
    with pytest.raises(ValueError):
        fa.attention_int8(q.cpu(), q.cpu(), q.cpu())


def test_config5_shape():
    """B8 H32 S8192 D128 with 1 % x8 K outliers: codes/scales bit-exact on four (batch, head)
    slices (numpy oracle), forward finite and checked on the same four against the int8-math oracle."""
    from flash_attn_triton_b200 import _ops
    import flash_attn_triton_b200 as fa
    B, H, S, D = 8, 32, 8192, 128
    g = torch.Generator(device=DEV).manual_seed(5)
    q = torch.randn(B, H, S, D, device=DEV, dtype=torch.float16, generator=g)
    v = torch.randn(B, H, S, D, device=DEV, dtype=torch.float16, generator=g)
    k = torch.randn(B, H, S, D, device=DEV, dtype=torch.float16, generator=g)
    k = torch.where(torch.rand(B, H, S, D, device=DEV, generator=g) < 0.01, k * 8, k)
    k8, s_k = _ops.quantize_k_int8(k)
    slices = [(0, 0), (1, 2), (4, 17), (7, 31)]            # first, last and two in between
    for b, h in slices:
        r8, rs = orc.quantize_k_rows_ref(k[b, h].cpu())
        assert np.array_equal(k8[b, h].cpu().numpy(), r8) and np.array_equal(s_k[b, h].cpu().numpy(), rs), (b, h)
    # dequantised codes reproduce k to half a step everywhere (size-independent property)
    err = (k8.float() * s_k[..., None] - k.float()).abs()
    assert (err <= 0.5001 * s_k[..., None]).all()
    for causal in (False, True):
        out = fa.attention_int8(q, k, v, causal=causal)
        assert torch.isfinite(out).all()
        for b, h in slices:
            sl = (slice(b, b + 1), slice(h, h + 1))
            ro, _, _, _ = orc.attention_int8_ref(q[sl].cpu(), k[sl].cpu(), v[sl].cpu(), causal=causal)
            assert maxdiff(out[sl], ro) <= util.FWD_TOL, (b, h, causal)
