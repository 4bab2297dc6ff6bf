"""fa_decode_paged_static: the decode entry point for callers that cannot allocate.

Some users of this library run where device allocation is off the table at call time: an
inference server that sized its pools at start-up and froze them, or code invoked from
another runtime's callback where cudaMalloc is forbidden (or would stall every stream).
For them the split-KV scratch lives in a fixed 16 MiB array inside the library instead of a
caller-provided workspace.  This file checks, through the C ABI, that the entry point gives
the same answer as fa_decode_paged on two calls in a row (the array is shared and keeps the
previous call's contents), and that it refuses problems that do not fit.

It is collected last on purpose: if it fails, `pytest -x` has already run everything else.
"""
import ctypes as C

import numpy as np
import pytest
import torch

import cases
import util
from util import DEV, maxdiff

pytestmark = pytest.mark.gpu


def _case(seed, lens, page=64, maxp=40, pool=200, Hq=8, Hkv=2, D=128):
    q, kc, vc, kn, vn, bt, cl = cases.paged_case(seed, len(lens), Hq, Hkv, D, page, pool, lens, maxp)
    cos, sin = cases.rotary_tables(maxp * page + 1, D)
    return [t.to(DEV) for t in (q, kc, vc, kn, vn, bt, cl, cos, sin)]


def test_static_scratch_matches_workspace_entry_point_twice():
    import flash_attn_triton_b200 as fa
    from flash_attn_triton_b200 import _native as N, _ops
    assert N.lib().fa_decode_static_scratch_bytes() == 16 << 20
    # two different problems back to back: the second call sees the first one's leftovers
    for call, (seed, lens, splits) in enumerate(((900, [2500, 70, 1300, 640], 6),
                                                 (901, [31, 2000, 999], 4))):
        q, kc, vc, kn, vn, bt, cl, cos, sin = _case(seed, lens)
        kc_ref, vc_ref = kc.clone(), vc.clone()
        want = fa.flash_attn_with_kvcache(q, kc_ref, vc_ref, kn, vn, cos, sin, cache_seqlens=cl,
                                          block_table=bt, rotary_interleaved=False, num_splits=splits)
        out = torch.empty_like(q)
        _ops.kvcache_decode_static(q, out, kc, vc, cl, block_table=bt, k_new=kn, v_new=vn, cos=cos,
                                   sin=sin, rotary_interleaved=False, num_splits=splits)
        assert maxdiff(out, want) <= util.FWD_TOL, call
        assert torch.equal(out, want), call  # same kernels, same split: bit-identical
        assert torch.equal(kc, kc_ref) and torch.equal(vc, vc_ref)
    # and against the CPU oracle once
    from oracle import attention_oracle as orc
    q, kc, vc, kn, vn, bt, cl, cos, sin = _case(902, [700, 65])
    ro, _, _ = orc.kvcache_ref(q.cpu(), kc.cpu(), vc.cpu(), kn.cpu(), vn.cpu(), cos.cpu(), sin.cpu(),
                               cache_seqlens=cl.cpu(), block_table=bt.cpu(), rotary_interleaved=False)
    out = torch.empty_like(q)
    _ops.kvcache_decode_static(q, out, kc, vc, cl, block_table=bt, k_new=kn, v_new=vn, cos=cos, sin=sin,
                               rotary_interleaved=False, num_splits=5)
    assert maxdiff(out, ro) <= util.FWD_TOL


def test_static_scratch_rejects_oversized_problem():
    from flash_attn_triton_b200 import _native as N, _ops
    # 64 sequences x 32 heads x 129 floats x 40 splits > 16 MiB
    B, Hq, Hkv, D, page = 64, 32, 8, 128, 64
    q = torch.zeros(B, 1, Hq, D, device=DEV, dtype=torch.float16)
    kc = torch.zeros(64, page, Hkv, D, device=DEV, dtype=torch.float16)
    bt = torch.zeros(B, 640, dtype=torch.int32, device=DEV)
    cl = torch.ones(B, dtype=torch.int32, device=DEV)
    with pytest.raises(RuntimeError, match="built-in array"):
        _ops.kvcache_decode_static(q, torch.empty_like(q), kc, kc.clone(), cl, block_table=bt,
                                   num_splits=40)
