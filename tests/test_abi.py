"""The C-ABI library: builds, loads without a GPU, exports every symbol the header declares
and agrees with the Python binding on the argument-block layouts.  No compute calls."""
import ctypes
import os
import re

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module")
def built():
    from flash_attn_triton_b200.build import build
    return build()


def header_functions():
    src = open(os.path.join(ROOT, "include", "fa_b200.h")).read()
    src = re.sub(r"/\*.*?\*/", "", src, flags=re.S)
    return sorted(set(re.findall(r"\b(fa_[a-z0-9_]+)\s*\(", src)))


def test_header_symbols_exported(built):
    lib = ctypes.CDLL(built)
    names = header_functions()
    assert len(names) >= 14
    for n in names:
        assert hasattr(lib, n), f"{n} declared in include/fa_b200.h but not exported"


def test_binding_covers_header(built):
    from flash_attn_triton_b200 import _native as N
    assert sorted(N.EXPORTS) == header_functions()
    lib = N.lib()  # also checks struct sizes against fa_sizeof_args
    assert lib.fa_version().startswith(b"fa_b200")
    assert lib.fa_sizeof_args(0) == ctypes.sizeof(N.AttnArgs)
    assert lib.fa_sizeof_args(1) == ctypes.sizeof(N.DecodeArgs)
    assert lib.fa_sizeof_args(2) == ctypes.sizeof(N.Int8Args)


def test_argument_errors_without_gpu(built):
    """Validation runs before any CUDA call, so bad arguments are reported on a CPU box."""
    from flash_attn_triton_b200 import _native as N
    lib = N.lib()
    a = N.AttnArgs()
    a.heads_q, a.heads_kv, a.head_dim = 4, 3, 64
    assert lib.fa_fwd(ctypes.byref(a), None) == -1
    assert b"multiple" in lib.fa_last_error()
    a.heads_kv, a.head_dim = 2, 24
    assert lib.fa_fwd(ctypes.byref(a), None) == -1
    assert b"head dimension" in lib.fa_last_error()
    a.head_dim = 64
    assert lib.fa_varlen_fwd(ctypes.byref(a), None) == -1  # packed entry needs cu_seqlens
    d = N.DecodeArgs()
    d.heads_q, d.heads_kv, d.head_dim, d.batch, d.seqlen_q = 8, 2, 128, 1, 1
    assert lib.fa_decode_paged(ctypes.byref(d), None) == -1
    assert lib.fa_quantize_k_int8(None, None, None, 4, 16, 0, None) == -1


def test_no_oracle_in_product():
    """The package must not import, read or call the oracle or any CPU fallback."""
    pkg = os.path.join(ROOT, "flash_attn_triton_b200")
    for dirpath, _, files in os.walk(pkg):
        if "build" in os.path.relpath(dirpath, pkg).split(os.sep):
            continue
        for f in files:
            if f.endswith((".py", ".cu", ".cuh")):
                text = open(os.path.join(dirpath, f)).read()
                assert "oracle" not in text.replace("no CPU fallback", ""), f
