"""Load the unmodified reference (luyanaa/flash-attn-triton) on a CPU-only machine.

TEST INFRASTRUCTURE ONLY: used by tests/golden/make_golden.py to produce the golden
vectors.  The reference sources are read from where they lie; nothing is copied.

The reference is pure Python + Triton and refuses CPU tensors, so three harness-side
shims are applied, none of which touches its arithmetic:

1. TRITON_INTERPRET=1 is set before Triton is imported (kernels run in the NumPy
   interpreter).
2. The two autotuned kernels get a single pinned config (the autotuner would otherwise
   try to benchmark without a GPU driver): attention_kernel.py:419-423, :809-812.
3. The `is_cuda` guards of the public wrappers (flash_attn_interface.py:102-103,
   :256-257, :597-598) are neutralised in the in-memory copy of that one module, and
   torch.cuda.get_device_capability is stubbed (attention_kernel.py:1264, :1272).

The package is imported under the alias `fa_ref` so the name `flash_attn_triton` stays
free.
"""
from __future__ import annotations

import importlib.util
import os
import sys
import types


def load_reference(path: str):
    os.environ["TRITON_INTERPRET"] = "1"
    import torch
    import triton

    pkg_dir = os.path.join(path, "flash_attn_triton")
    if not os.path.isdir(pkg_dir):
        raise FileNotFoundError(f"reference not found at {path}")
    torch.cuda.get_device_capability = lambda *a, **k: (8, 0)

    if "fa_ref" not in sys.modules:
        # parent package object without running its __init__ (which imports the guarded wrappers)
        pkg = types.ModuleType("fa_ref")
        pkg.__path__ = [pkg_dir]
        sys.modules["fa_ref"] = pkg
        sub = types.ModuleType("fa_ref.triton_kernel")
        sub.__path__ = [os.path.join(pkg_dir, "triton_kernel")]
        sys.modules["fa_ref.triton_kernel"] = sub
        for name in ("attention_kernel", "attention_kernel_int8"):
            full = f"fa_ref.triton_kernel.{name}"
            spec = importlib.util.spec_from_file_location(
                full, os.path.join(pkg_dir, "triton_kernel", name + ".py"))
            mod = importlib.util.module_from_spec(spec)
            sys.modules[full] = mod
            spec.loader.exec_module(mod)
            setattr(sub, name, mod)
        ak = sys.modules["fa_ref.triton_kernel.attention_kernel"]
        ak._attn_fwd.configs = [triton.Config({"BLOCK_M": 64, "BLOCK_N": 16},
                                              num_stages=2, num_warps=4)]
        ak._attn_bwd.configs = ak._attn_bwd.configs[:1]

        src_path = os.path.join(pkg_dir, "flash_attn_interface.py")
        with open(src_path) as f:
            src = f.read()
        guard = "if not (q.is_cuda and k.is_cuda and v.is_cuda):"
        assert src.count(guard) == 3, "reference layout changed"
        src = src.replace(guard, "if False:")
        iface = types.ModuleType("fa_ref.flash_attn_interface")
        iface.__package__ = "fa_ref"
        iface.__file__ = src_path
        sys.modules["fa_ref.flash_attn_interface"] = iface
        exec(compile(src, src_path, "exec"), iface.__dict__)
        pkg.flash_attn_interface = iface

    ns = types.SimpleNamespace()
    ns.AK = sys.modules["fa_ref.triton_kernel.attention_kernel"]
    ns.AK8 = sys.modules["fa_ref.triton_kernel.attention_kernel_int8"]
    ns.IF = sys.modules["fa_ref.flash_attn_interface"]
    return ns
