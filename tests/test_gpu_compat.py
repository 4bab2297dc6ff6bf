"""The helper package (compat): rotary-embedding kernel and row movers behind un-padding,
against the golden vectors the unmodified reference produced and against the CPU oracle."""
import numpy as np
import pytest
import torch

import cases
from oracle import attention_oracle as orc
from util import DEV

pytestmark = pytest.mark.gpu

ROT_TOL = 1e-6     # after allowing one fp16 rounding step of the reference value (excess below)


def excess16(a, b):
    a, b = a.float().cpu(), torch.as_tensor(b).float()
    return ((a - b).abs() - 2.0 ** -10 * b.abs()).max().item()


def _dev_kw(kw):
    return {k: (v.to(DEV) if isinstance(v, torch.Tensor) else v) for k, v in kw.items()}


@pytest.mark.parametrize("name", list(cases.ROTARY_CASES))
def test_rotary_kernel_vs_reference_golden(golden, name):
    from flash_attn_triton_b200.compat.ops.triton.rotary import apply_rotary
    g = golden("compat_rotary")
    x, cos, sin, kw = cases.rotary_case(**cases.ROTARY_CASES[name])
    y = apply_rotary(x.to(DEV), cos.to(DEV), sin.to(DEV), **_dev_kw(kw))
    assert excess16(y, g[name]) <= ROT_TOL
    assert excess16(y, orc.rotary_emb_ref(x, cos, sin, **kw)) <= ROT_TOL
    # in place gives the same bits
    xi = x.to(DEV).clone()
    y2 = apply_rotary(xi, cos.to(DEV), sin.to(DEV), inplace=True, **_dev_kw(kw))
    assert y2.data_ptr() == xi.data_ptr() and torch.equal(y2, y)


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16, torch.float32])
def test_rotary_sizes_dtypes_and_strides(dtype):
    from flash_attn_triton_b200.compat.ops.triton.rotary import apply_rotary
    rng = np.random.default_rng(9)
    B, S, H, D, rot = 3, 333, 5, 128, 96
    x = torch.from_numpy(rng.standard_normal((B, S, 3, H, D), dtype=np.float32)).to(dtype)
    ang = torch.arange(400, dtype=torch.float32)[:, None] * (1.0 / 10000 ** (torch.arange(0, rot, 2) / rot))[None]
    cos, sin = torch.cos(ang).to(dtype), torch.sin(ang).to(dtype)
    off = torch.tensor([0, 13, 67], dtype=torch.int64)
    xs = x.to(DEV)[:, :, 1]                               # a strided slice of a packed qkv tensor
    y = apply_rotary(xs, cos.to(DEV), sin.to(DEV), seqlen_offsets=off.to(DEV), interleaved=True)
    ref = orc.rotary_emb_ref(x[:, :, 1], cos, sin, seqlen_offsets=off, interleaved=True)
    tol = {torch.float16: 2.0 ** -10, torch.bfloat16: 2.0 ** -7, torch.float32: 1e-6}[dtype]
    assert ((y.float().cpu() - ref.float()).abs() - tol * ref.float().abs()).max().item() <= 1e-5
    assert torch.equal(y[..., rot:].cpu(), x[:, :, 1][..., rot:])   # columns past rotary_dim are copied


def test_rotary_autograd_and_module():
    from flash_attn_triton_b200.compat.layers import rotary as R
    rng = np.random.default_rng(3)
    B, S, H, D = 2, 37, 4, 64
    qkv = torch.from_numpy(rng.standard_normal((B, S, 3, H, D), dtype=np.float32)).half()
    g = torch.from_numpy(rng.standard_normal((B, S, 3, H, D), dtype=np.float32)).half()
    mod = R.RotaryEmbedding(D, interleaved=False, device=DEV)
    x = qkv.to(DEV).requires_grad_()
    out = mod(x.clone(), seqlen_offset=3)                  # forward() rotates its argument in place
    (out.float() * g.to(DEV).float()).sum().backward()
    cos, sin = mod._cos_cached.cpu(), mod._sin_cached.cpu()
    # reference: the eager restatement on fp32 copies
    xr = qkv.float().requires_grad_()
    pos = slice(3, 3 + S)
    q_r = R.apply_rotary_emb_torch(xr[:, :, 0], cos[pos].float(), sin[pos].float())
    k_r = R.apply_rotary_emb_torch(xr[:, :, 1], cos[pos].float(), sin[pos].float())
    ref = torch.stack([q_r, k_r, xr[:, :, 2]], dim=2)
    (ref * g.float()).sum().backward()
    assert excess16(out, ref.detach()) <= 1e-3            # tables are fp16 in the module, fp32 here
    assert (x.grad.float().cpu() - xr.grad).abs().max().item() <= 4e-3
    # functional form, q with kv, XPos scaling, tensor offsets
    mod2 = R.RotaryEmbedding(D, interleaved=True, scale_base=512, device=DEV)
    q = qkv[:, :, 0].contiguous().to(DEV)
    kv = qkv[:, :, 1:].contiguous().to(DEV)
    offs = torch.tensor([2, 9], dtype=torch.int32, device=DEV)
    q2, kv2 = mod2(q.clone(), kv.clone(), seqlen_offset=offs, max_seqlen=64)
    want_q = orc.rotary_emb_ref(qkv[:, :, 0], mod2._cos_cached.cpu(), mod2._sin_cached.cpu(),
                                seqlen_offsets=offs.cpu(), interleaved=True)
    want_k = orc.rotary_emb_ref(qkv[:, :, 1], mod2._cos_k_cached.cpu(), mod2._sin_k_cached.cpu(),
                                seqlen_offsets=offs.cpu(), interleaved=True)
    assert excess16(q2, want_q) <= ROT_TOL and excess16(kv2[:, :, 0], want_k) <= ROT_TOL
    assert torch.equal(kv2[:, :, 1].cpu(), qkv[:, :, 2])


def test_padding_vs_reference_golden(golden):
    from flash_attn_triton_b200.compat import bert_padding as BP
    g = golden("compat_padding")
    hs, mask, lens_in_row = cases.padding_case(7, 3, 12, 2, 16)
    u, idx, cu, mx = BP.unpad_input(hs.to(DEV), mask.to(DEV))
    assert torch.equal(u.cpu(), torch.from_numpy(g["unpadded"]))
    assert torch.equal(idx.cpu(), torch.from_numpy(g["indices"])) and torch.equal(cu.cpu(), torch.from_numpy(g["cu_seqlens"]))
    assert mx == int(g["max_seqlen"])
    assert torch.equal(BP.pad_input(u, idx, 3, 12).cpu(), torch.from_numpy(g["repadded"]))
    u2, idx2, cu2, mx2 = BP.unpad_input_for_concatenated_sequences(hs.to(DEV), lens_in_row.to(DEV))
    assert torch.equal(u2.cpu(), torch.from_numpy(g["unpadded_concat"]))
    assert torch.equal(cu2.cpu(), torch.from_numpy(g["cu_seqlens_concat"])) and mx2 == int(g["max_seqlen_concat"])
    # gradient of the gather: the reference's scatter into zeros
    hs_g = hs.float().to(DEV).requires_grad_()
    w = (torch.arange(u.numel(), dtype=torch.float32) / u.numel()).reshape(u.shape).to(DEV)
    (BP.index_first_axis(hs_g.reshape(-1, 2, 16), idx) * w).sum().backward()
    assert torch.equal(hs_g.grad.cpu(), torch.from_numpy(g["grad_gather"]))


def test_padding_large_roundtrip_and_residual():
    from flash_attn_triton_b200.compat import bert_padding as BP
    rng = np.random.default_rng(11)
    B, S, Hd = 16, 1000, 1024
    hs = torch.from_numpy(rng.standard_normal((B, S, Hd), dtype=np.float32)).to(torch.bfloat16).to(DEV)
    lens = rng.integers(1, S + 1, size=B)
    mask = torch.from_numpy((np.arange(S)[None, :] < lens[:, None])).to(DEV)
    u, idx, cu, mx = BP.unpad_input(hs, mask)
    ru, ridx, rcu, rmx = orc.unpad_ref(hs.cpu(), mask.cpu())
    assert torch.equal(u.cpu(), ru) and torch.equal(idx.cpu(), ridx) and torch.equal(cu.cpu(), rcu) and mx == rmx
    back = BP.pad_input(u, idx, B, S)
    assert torch.equal(back.cpu(), orc.pad_ref(ru, ridx, B, S))
    assert torch.equal(back[mask], hs[mask]) and not back[~mask].any()
    # residual form: gradient = grad_residual + scatter(grad_output)
    x = hs.reshape(-1, Hd).float().requires_grad_()
    out, res = BP.index_first_axis_residual(x, idx)
    go = torch.ones_like(out) * 0.5
    gr = torch.full_like(res, 0.25)
    torch.autograd.backward([out, res], [go, gr])
    want = torch.full((B * S, Hd), 0.25)
    want[ridx] += 0.5
    assert torch.equal(x.grad.cpu(), want)
