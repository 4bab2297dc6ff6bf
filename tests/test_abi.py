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


def test_decode_argument_errors_without_gpu(built):
    """Alignment, stride and table checks of the decode entry points are made on the host."""
    from flash_attn_triton_b200 import _native as N
    lib = N.lib()

    def base():
        d = N.DecodeArgs()
        d.heads_q, d.heads_kv, d.head_dim, d.batch, d.seqlen_q = 8, 2, 128, 1, 1
        d.q = d.o = d.k_cache = d.v_cache = d.cache_seqlens = 4096   # never dereferenced: validation only
        d.page_size = 64
        for f in ("q_stride", "o_stride", "kc_stride", "vc_stride"):
            setattr(d, f, N._I64x3(1024, 1024, 128))
        return d

    def err(d, word):
        assert lib.fa_decode_paged(ctypes.byref(d), None) == -1
        assert word.encode() in lib.fa_last_error(), lib.fa_last_error()
        assert lib.fa_decode_paged_static(ctypes.byref(d), None) == -1

    d = base(); d.o = 4096 + 8
    err(d, "16-byte aligned")
    d = base(); d.o_stride = N._I64x3(1024, 1020, 128)
    err(d, "multiples of 8")
    d = base(); d.workspace = 4096 + 4
    err(d, "workspace")
    d = base(); d.num_splits = -1
    err(d, "num_splits")
    d = base(); d.block_table = 4096; d.block_table_stride = 0
    err(d, "block_table_stride")
    d = base(); d.rotary_cos = d.rotary_sin = 4096; d.rotary_dim = 64; d.rotary_seqlen = 0
    err(d, "rotary_seqlen")
    d = base(); d.k_new = d.v_new = 4096 + 2; d.seqlen_new = 1
    d.kn_stride = d.vn_stride = N._I64x3(1024, 1024, 128)
    err(d, "new k/v")


def test_wait_status_refusal_without_gpu(built):
    """Once the host mirror of the wait-status word is set, the tcgen05 launchers refuse with
    FA_ERR_DEVICE_WAIT before touching the GPU; clearing the mirror lifts the refusal."""
    from flash_attn_triton_b200 import _native as N
    lib = N.lib()
    a = N.AttnArgs()
    a.impl = N.IMPL_TCGEN05
    a.batch, a.seqlen_q, a.seqlen_k, a.heads_q, a.heads_kv, a.head_dim = 1, 512, 512, 2, 2, 128
    a.q = a.k = a.v = a.o = a.dout = a.lse2 = a.delta = a.dq = a.dk = a.dv = 4096
    for f in ("q_stride", "k_stride", "v_stride", "o_stride", "do_stride", "dq_stride", "dk_stride", "dv_stride"):
        setattr(a, f, N._I64x3(512 * 256, 256, 128))
    a.softmax_scale = 0.1
    a.window_left = a.window_right = -1
    a.device = 0
    assert lib.fa_debug_set_wait_status(0, 31) == 0
    try:
        for fn in (lib.fa_fwd, lib.fa_bwd_dq, lib.fa_bwd_dkdv):
            r = fn(ctypes.byref(a), None)
            assert r == -5, r                      # refused before any CUDA call
            assert b"fa_device_wait_clear" in lib.fa_last_error()
            with pytest.raises(N.DeviceWaitError):
                N.check(r, "probe")
    finally:
        assert lib.fa_debug_set_wait_status(0, 0) == 0
