"""Helpers shared by the GPU parity tests."""
import numpy as np
import torch

FWD_TOL = 2e-3   # max-abs, fp16 forward vs the fp32 oracle
GRAD_TOL = 1e-2  # max-abs, gradients vs the fp32 oracle
# bf16 carries 8 mantissa bits instead of 11: outputs of O(1) magnitude round to 2^-8
BF16_FWD_TOL = 2e-2
BF16_GRAD_TOL = 6e-2
LN2 = 0.6931471805599453
DEV = "cuda"


def maxdiff(a, b):
    a = torch.as_tensor(np.asarray(a) if not isinstance(a, torch.Tensor) else a).float().cpu()
    b = torch.as_tensor(np.asarray(b) if not isinstance(b, torch.Tensor) else b).float().cpu()
    assert a.shape == b.shape, (a.shape, b.shape)
    if a.numel() == 0:
        return 0.0
    d = (a - b).abs()
    d = torch.where(torch.isinf(a) & torch.isinf(b) & (a == b), torch.zeros_like(d), d)
    return d.max().item()


def tols(dtype):
    return (FWD_TOL, GRAD_TOL) if dtype == torch.float16 else (BF16_FWD_TOL, BF16_GRAD_TOL)


def run_dense(fn, q, k, v, do, **kw):
    """Run a public dense entry point on the GPU with gradients; returns cpu tensors."""
    qd, kd, vd = (t.to(DEV).requires_grad_() for t in (q, k, v))
    out = fn(qd, kd, vd, **kw)
    dq, dk, dv = torch.autograd.grad((out.float() * do.to(DEV).float()).sum(), (qd, kd, vd))
    return out.detach().cpu(), dq.cpu(), dk.cpu(), dv.cpu()


def excess(a, b, rel=2.0 ** -10):
    """max(|a-b| - rel*|b|): the max-abs error left after allowing one fp16 rounding step
    of the reference value (values of magnitude 16-32 have an fp16 spacing of 2^-6)."""
    a = torch.as_tensor(a).float().cpu()
    b = torch.as_tensor(b).float().cpu()
    return ((a - b).abs() - rel * b.abs()).max().item()
