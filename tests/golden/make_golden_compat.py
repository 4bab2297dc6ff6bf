"""Generate tests/golden/compat_*.npz from the UNMODIFIED reference's helper package.

    FA_REF_PATH=/path/to/reference python tests/golden/make_golden_compat.py

The reference's rotary kernel (flash_attn/ops/triton/rotary.py) runs in Triton's CPU
interpreter; its padding helpers (flash_attn/bert_padding.py) are plain torch.  Inputs are
regenerated from seeds by tests/golden/cases.py; only outputs and an input checksum are stored.
"""
from __future__ import annotations

import importlib.util
import os
import sys

os.environ["TRITON_INTERPRET"] = "1"
HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, HERE)

import numpy as np  # noqa: E402
import torch  # noqa: E402

import cases  # noqa: E402

REF = sys.argv[1] if len(sys.argv) > 1 else os.environ.get("FA_REF_PATH")
if not REF:
    sys.exit("pass the reference checkout as argv[1] or FA_REF_PATH")


def load(name, rel):
    spec = importlib.util.spec_from_file_location(name, os.path.join(REF, rel))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


class _NoDevice:
    def __init__(self, *a):
        pass

    def __enter__(self):
        return self

    def __exit__(self, *a):
        return False


torch.cuda.device = _NoDevice          # the launcher wraps its launch in torch.cuda.device(None) on CPU tensors
rot = load("ref_rotary", "flash_attn/ops/triton/rotary.py")
pad = load("ref_bert_padding", "flash_attn/bert_padding.py")


def save(name, **arrays):
    out = {k: (v.detach().cpu().numpy() if isinstance(v, torch.Tensor) else v) for k, v in arrays.items()}
    np.savez_compressed(os.path.join(HERE, name + ".npz"), **out)
    print("wrote", name, {k: getattr(v, "shape", v) for k, v in out.items()})


def rotary():
    out = {}
    for name, spec in cases.ROTARY_CASES.items():
        x, cos, sin, kw = cases.rotary_case(**spec)
        y = rot.apply_rotary(x.clone(), cos, sin, **kw)
        out[name] = y
        out[name + "_checksum"] = np.frombuffer(cases.checksum(x, cos, sin).encode(), dtype=np.uint8)
    save("compat_rotary", **out)


def padding():
    hs, mask, lens_in_row = cases.padding_case(7, 3, 12, 2, 16)
    u, idx, cu, mx = pad.unpad_input(hs, mask)
    back = pad.pad_input(u, idx, 3, 12)
    u2, idx2, cu2, mx2 = pad.unpad_input_for_concatenated_sequences(hs, lens_in_row)
    # gradients of the gather / scatter pair, through the reference's autograd functions
    hs_g = hs.clone().float().requires_grad_()
    w = torch.arange(u.numel(), dtype=torch.float32).reshape(u.shape) / u.numel()
    (pad.index_first_axis(hs_g.reshape(-1, 2, 16), idx) * w).sum().backward()
    save("compat_padding", checksum=np.frombuffer(cases.checksum(hs, mask, lens_in_row).encode(), dtype=np.uint8),
         unpadded=u, indices=idx, cu_seqlens=cu, max_seqlen=np.int64(mx), repadded=back,
         unpadded_concat=u2, indices_concat=idx2, cu_seqlens_concat=cu2, max_seqlen_concat=np.int64(mx2),
         grad_gather=hs_g.grad)


if __name__ == "__main__":
    rotary()
    padding()
