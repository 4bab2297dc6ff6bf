"""Checks that stand in for a memory checker and a race detector (neither is available for these
kernels): run-twice bit equality (one writer per element, no atomics), guard bands around every
output (nothing outside the tensor is touched, nothing inside is left unwritten), the oracle on
slices spread over the whole benchmark-size problem, and the time-out path of the bounded waits."""
import ctypes as C
import os
import subprocess
import sys

import numpy as np
import pytest
import torch

import cases
import util
from oracle import attention_oracle as orc
from util import DEV, maxdiff

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
SENTINEL = 0x7BCD  # fp16 bit pattern written into guard bands and outputs before a call (a NaN-free, odd value)


def _guarded(shape, dtype=torch.float16, guard=4096):
    """A tensor of `shape` carved out of a larger buffer whose bytes are all the sentinel."""
    per = torch.empty((), dtype=dtype).element_size() // 2      # sentinel words per element
    n = int(np.prod(shape)) * per
    buf = torch.full((guard + n + guard,), SENTINEL, dtype=torch.int16, device=DEV)
    return buf, buf[guard:guard + n].view(dtype).view(shape)


def _guards_intact(buf, numel, guard=4096):
    """`buf` as returned by _guarded for a tensor of `numel` elements of 2 bytes (pass twice the
    count for 4-byte elements)."""
    return bool((buf[:guard] == SENTINEL).all() and (buf[guard + numel:] == SENTINEL).all())


def _attn_args(N, _ops, q, k, v, o, lse, do, dq, dk, dv, delta, dims, *, scale, causal, wl=-1, wr=-1, cu=None,
               max_len=None, impl=None, alibi=None, softcap=0.0):
    a = N.AttnArgs()
    if cu is None:
        B, S, H, D = q.shape
        _ops._fill_common(a, q, k, v, o, dims, dims, batch=B, sq=S, sk=k.shape[1], hq=H, hkv=k.shape[2], d=D,
                          scale=scale, causal=causal, wl=wl, wr=wr, softcap=softcap, alibi=alibi, q_pos_offset=0,
                          impl=impl)
        a.lse_stride = N._I64x3(H * S, 1, S)
    else:
        T, H, D = q.shape
        _ops._fill_common(a, q, k, v, o, dims, dims, batch=cu.numel() - 1, sq=max_len, sk=max_len, hq=H,
                          hkv=k.shape[1], d=D, scale=scale, causal=causal, wl=wl, wr=wr, softcap=softcap,
                          alibi=alibi, q_pos_offset=0, impl=impl, cu_q=cu, cu_k=cu)
        a.lse_stride = N._I64x3(0, 1, T)
    a.lse2 = lse.data_ptr()
    a.dout, a.do_stride, a.delta = do.data_ptr(), N.strides3(do, dims), delta.data_ptr()
    a.dq, a.dk, a.dv = dq.data_ptr(), dk.data_ptr(), dv.data_ptr()
    a.dq_stride, a.dk_stride, a.dv_stride = N.strides3(dq, dims), N.strides3(dk, dims), N.strides3(dv, dims)
    return a


DENSE = [
    # B, S, H, Hkv, D, causal, window      (S not a multiple of the 128-row tiles: clipped TMA stores)
    (2, 1000, 4, 2, 128, True, (-1, -1)),
    (1, 3300, 2, 2, 128, False, (-1, -1)),   # 26 query tiles per key block: the persistent dK/dV kernel
    (2, 777, 4, 4, 64, True, (300, 0)),
    (1, 4096, 16, 16, 128, True, (-1, -1)),
]


@pytest.mark.parametrize("case", DENSE, ids=lambda c: "x".join(map(str, c[:5])))
def test_dense_guard_bands_and_run_twice(case):
    """fwd, preprocess, dQ, dK/dV through the C ABI into guarded, sentinel-filled buffers, twice."""
    from flash_attn_triton_b200 import _native as N, _ops
    B, S, H, Hkv, D, causal, (wl, wr) = case
    rng = np.random.default_rng(S)
    mk = lambda h: torch.from_numpy(rng.standard_normal((B, S, h, D), dtype=np.float32)).half().to(DEV)
    q, k, v, do = mk(H), mk(Hkv), mk(Hkv), mk(H)
    L, st = N.lib(), N.stream_ptr(torch.device(DEV))
    runs = []
    for _ in range(2):
        bo, o = _guarded((B, S, H, D))
        bq, dq = _guarded((B, S, H, D))
        bk, dk = _guarded((B, S, Hkv, D))
        bv, dv = _guarded((B, S, Hkv, D))
        bl, lse = _guarded((B, H, S), torch.float32)
        bd, delta = _guarded((B, H, S), torch.float32)
        a = _attn_args(N, _ops, q, k, v, o, lse, do, dq, dk, dv, delta, _ops._BSHD, scale=D ** -0.5, causal=causal,
                       wl=wl, wr=wr, impl=N.IMPL_TCGEN05)
        for fn in (L.fa_fwd, L.fa_bwd_preprocess, L.fa_bwd_dq, L.fa_bwd_dkdv):
            N.check(fn(C.byref(a), st), "call")
        assert L.fa_device_wait_status(0) == 0
        for buf, t in ((bo, o), (bq, dq), (bk, dk), (bv, dv)):
            assert _guards_intact(buf, t.numel()), "wrote outside the tensor"
            assert not (t.view(torch.int16) == SENTINEL).all(dim=-1).any(), "left a row unwritten"
        assert _guards_intact(bl, lse.numel() * 2) and _guards_intact(bd, delta.numel() * 2)
        runs.append([t.clone() for t in (o, lse, dq, dk, dv)])
    for x, y in zip(*runs):
        assert torch.equal(x.view(torch.int16) if x.dtype == torch.float16 else x.view(torch.int32),
                           y.view(torch.int16) if y.dtype == torch.float16 else y.view(torch.int32)), "two runs differ"
    # and the values: one (batch, head) slice against the oracle
    b, h = B - 1, H - 1
    hk = h // (H // Hkv)
    sl = lambda t, hh: t[b:b + 1, :, hh:hh + 1].cpu()
    ro, _, rdq, _, _ = orc.attention_grads_ref(sl(q, h), sl(k, hk), sl(v, hk), sl(do, h), causal=causal, window=(wl, wr))
    assert maxdiff(sl(runs[0][0], h), ro) <= util.FWD_TOL and maxdiff(sl(runs[0][2], h), rdq) <= util.GRAD_TOL


def test_packed_guard_rows_and_run_twice():
    """Packed batch whose sequences end inside tiles, in buffers that carry 130 more rows than
    cu_seqlens covers: tail stores must not spill into the next sequence's rows (checked through
    the values) nor into the rows no sequence owns (which must keep the sentinel)."""
    from flash_attn_triton_b200 import _native as N, _ops
    lens, extra, H, Hkv, D = [200, 129, 640, 64, 1], 130, 8, 2, 128
    used = sum(lens)
    rows = used + extra
    rng = np.random.default_rng(5)
    cu = torch.tensor(np.concatenate([[0], np.cumsum(lens)]), dtype=torch.int32, device=DEV)
    mk = lambda h: torch.from_numpy(rng.standard_normal((rows, h, D), dtype=np.float32)).half().to(DEV)
    q, k, v, do = mk(H), mk(Hkv), mk(Hkv), mk(H)
    sl = torch.tensor([[2.0 ** (-(i + 1)) for i in range(H)]] * len(lens), device=DEV)
    L, st = N.lib(), N.stream_ptr(torch.device(DEV))
    runs = []
    for _ in range(2):
        bo, o = _guarded((rows, H, D))
        bq, dq = _guarded((rows, H, D))
        bk, dk = _guarded((rows, Hkv, D))
        bv, dv = _guarded((rows, Hkv, D))
        lse = torch.empty((H, rows), dtype=torch.float32, device=DEV)
        delta = torch.empty_like(lse)
        a = _attn_args(N, _ops, q, k, v, o, lse, do, dq, dk, dv, delta, _ops._THD, scale=0.09, causal=True, wl=150,
                       wr=0, cu=cu, max_len=max(lens), impl=N.IMPL_TCGEN05, alibi=sl, softcap=30.0)
        for fn in (L.fa_varlen_fwd, L.fa_bwd_preprocess, L.fa_varlen_bwd_dq, L.fa_varlen_bwd_dkdv):
            N.check(fn(C.byref(a), st), "call")
        assert L.fa_device_wait_status(0) == 0
        for buf, t in ((bo, o), (bq, dq), (bk, dk), (bv, dv)):
            assert _guards_intact(buf, t.numel())
            assert (t[used:].view(torch.int16) == SENTINEL).all(), "rows past the last sequence were written"
            assert not (t[:used].view(torch.int16) == SENTINEL).all(dim=-1).any(), "left a row unwritten"
        runs.append([t[:used].clone() for t in (o, dq, dk, dv)])
    for x, y in zip(*runs):
        assert torch.equal(x.view(torch.int16), y.view(torch.int16))
    c = lambda t: t[:used].cpu()
    ro, _, rdq, rdk, rdv = orc.varlen_attention_grads_ref(c(q), c(k), c(v), c(do), cu.cpu(), cu.cpu(),
                                                          softmax_scale=0.09, causal=True, window=(150, 0),
                                                          softcap=30.0, alibi_slopes=sl[0].cpu())
    assert maxdiff(runs[0][0], ro) <= util.FWD_TOL
    for t, r in zip(runs[0][1:], (rdq, rdk, rdv)):
        assert maxdiff(t, r) <= util.GRAD_TOL


def test_decode_and_quantiser_run_twice():
    import flash_attn_triton_b200 as fa
    from flash_attn_triton_b200 import _ops
    lens = [2500, 70, 1300, 640]
    q, kc, vc, kn, vn, bt, cl = (t.to(DEV) for t in cases.paged_case(910, len(lens), 8, 2, 128, 64, 200, lens, 40))
    cos, sin = (t.to(DEV) for t in cases.rotary_tables(40 * 64 + 1, 128))
    outs = []
    for _ in range(2):
        kc2, vc2 = kc.clone(), vc.clone()
        outs.append((fa.flash_attn_with_kvcache(q, kc2, vc2, kn, vn, cos, sin, cache_seqlens=cl, block_table=bt,
                                                rotary_interleaved=False), kc2, vc2))
    for x, y in zip(*outs):
        assert torch.equal(x, y)
    k = cases.k_with_outliers(21, 64, 1024, 128).to(DEV)
    (a8, asc), (b8, bsc) = _ops.quantize_k_int8(k), _ops.quantize_k_int8(k)
    assert torch.equal(a8, b8) and torch.equal(asc, bsc)


def test_benchmark_size_oracle_on_sixteen_slices():
    """B16 H16 S4096 D128 causal: forward, dQ, dK, dV of 16 (batch, head) slices spread over the
    whole problem (first and last included) against the fp32 oracle."""
    from flash_attn_triton_b200 import _native as N, _ops
    torch.manual_seed(2)
    B, S, H, D = 16, 4096, 16, 128
    q, k, v, do = (torch.randn(B, S, H, D, device=DEV, dtype=torch.float16) for _ in range(4))
    o, lse, _ = _ops.dense_forward(q, k, v, D ** -0.5, True, -1, -1, 0.0, None, 0, N.IMPL_AUTO, "bshd", True)
    dq, dk, dv = _ops.dense_backward(q, k, v, o, lse, do, D ** -0.5, True, -1, -1, 0.0, None, 0, N.IMPL_AUTO, "bshd")
    assert N.lib().fa_device_wait_status(0) == 0
    slices = [(0, 0), (15, 15)] + [(i + 1, (7 * i + 3) % 16) for i in range(14)]
    assert len(set(slices)) == 16
    for b, h in slices:
        s = lambda t: t[b:b + 1, :, h:h + 1].cpu()
        ro, rl, rdq, rdk, rdv = orc.attention_grads_ref(s(q), s(k), s(v), s(do), causal=True)
        assert maxdiff(s(o), ro) <= util.FWD_TOL, (b, h)
        assert maxdiff(lse[b:b + 1, h:h + 1].cpu() * util.LN2, rl) <= util.FWD_TOL, (b, h)
        for t, r in ((dq, rdq), (dk, rdk), (dv, rdv)):
            assert maxdiff(s(t), r) <= util.GRAD_TOL, (b, h)


_PROBE = r"""
import ctypes as C, sys, torch
sys.path.insert(0, %r)
from flash_attn_triton_b200 import _native as N, _ops
L = N.lib()
assert L.fa_device_wait_status(0) == 0
q = torch.randn(1, 512, 2, 128, device="cuda", dtype=torch.float16)
_ops.dense_forward(q, q, q, 0.1, True, -1, -1, 0.0, None, 0, N.IMPL_TCGEN05, "bshd", True)    # works
assert L.fa_wait_probe(0, 200000, None) == 0          # ~0.1 ms on a barrier nothing arrives at
code = L.fa_device_wait_status(0)
assert code == 99, code
try:
    _ops.dense_forward(q, q, q, 0.1, True, -1, -1, 0.0, None, 0, N.IMPL_TCGEN05, "bshd", True)
    raise SystemExit("launch was not refused")
except N.DeviceWaitError:
    pass
o_mma, _, _ = _ops.dense_forward(q, q, q, 0.1, True, -1, -1, 0.0, None, 0, N.IMPL_MMA, "bshd", True)   # other kernels unaffected
assert L.fa_device_wait_clear(0) == 0 and L.fa_device_wait_status(0) == 0
o, _, _ = _ops.dense_forward(q, q, q, 0.1, True, -1, -1, 0.0, None, 0, N.IMPL_TCGEN05, "bshd", True)
assert (o.float() - o_mma.float()).abs().max().item() <= 2e-3
print("probe ok")
"""


def test_bounded_wait_times_out_and_is_reported():
    """A wait that nothing satisfies gives up, raises the status word and its host mirror, the
    tcgen05 entry points refuse to launch until the word is cleared.  Runs in a process of its own
    (the word is per process)."""
    r = subprocess.run([sys.executable, "-c", _PROBE % ROOT], capture_output=True, text=True, timeout=600)
    assert r.returncode == 0 and "probe ok" in r.stdout, r.stdout + r.stderr


@pytest.mark.parametrize("causal", [False, True])
def test_packed_forward_ignores_non_finite_rows_of_the_next_sequence(causal):
    """The last key tile of a packed sequence also stages rows of the next sequence; their
    probabilities are 0, and 0 * inf must not reach the output (tcgen05 and mma.sync forward)."""
    from flash_attn_triton_b200 import _native as N, _ops
    lens = [100, 60, 300]
    q, k, v, do, cu_q, cu_k = cases.varlen_case(77, lens, lens, 4, 2, 128)
    k2, v2 = k.clone(), v.clone()
    k2[100:160] = float("nan")                 # the whole second sequence is poisoned
    v2[100:160] = float("inf")
    ref, _ = orc.varlen_attention_ref(q, k, v, cu_q, cu_k, causal=causal)
    for impl in (N.IMPL_TCGEN05, N.IMPL_MMA):
        o, _, _ = _ops.varlen_forward(q.to(DEV), k2.to(DEV), v2.to(DEV), cu_q.to(DEV), cu_k.to(DEV), 300, 300,
                                      128 ** -0.5, causal, -1, -1, 0.0, None, impl, False)
        o = o.float().cpu()
        assert torch.isfinite(o[:100]).all() and torch.isfinite(o[160:]).all(), impl
        assert (o[:100] - ref[:100]).abs().max().item() <= 2e-3 and (o[160:] - ref[160:]).abs().max().item() <= 2e-3


@pytest.mark.parametrize("lens", [[100, 60, 300], [200, 60, 300], [3300, 60, 200]])
@pytest.mark.parametrize("causal", [False, True])
def test_packed_backward_ignores_non_finite_rows_of_the_next_sequence(lens, causal):
    """Tail tiles of a packed sequence stage Q, K, V and dO rows of the next sequence.  dS = P (dP -
    delta) is 0 * inf there, and dS K, dS^T Q and P^T dO contract over those rows: nothing of a
    poisoned neighbour may reach the gradients of the other sequences (tcgen05 and mma.sync)."""
    from flash_attn_triton_b200 import _native as N, _ops
    q, k, v, do, cu_q, cu_k = cases.varlen_case(78, lens, lens, 2, 1, 128)
    a, b = lens[0], lens[0] + lens[1]
    bad = [t.clone() for t in (q, k, v, do)]
    bad[0][a:b] = float("nan")
    bad[1][a:b] = float("inf")
    bad[2][a:b] = float("nan")
    bad[3][a:b] = float("-inf")
    _, _, rdq, rdk, rdv = orc.varlen_attention_grads_ref(q, k, v, do, cu_q, cu_k, causal=causal)
    for impl in (N.IMPL_TCGEN05, N.IMPL_MMA):
        qd, kd, vd, dod = (t.to(DEV) for t in bad)
        args = (cu_q.to(DEV), cu_k.to(DEV), max(lens), max(lens), 128 ** -0.5, causal, -1, -1, 0.0, None, impl)
        o, lse, _ = _ops.varlen_forward(qd, kd, vd, *args, True)
        dq, dk, dv = _ops.varlen_backward(qd, kd, vd, o, lse, dod, *args)
        assert N.lib().fa_device_wait_status(0) == 0
        for g, r in zip((dq, dk, dv), (rdq, rdk, rdv)):
            g = g.float().cpu()
            assert torch.isfinite(g[:a]).all() and torch.isfinite(g[b:]).all(), impl
            assert (g[:a] - r[:a]).abs().max().item() <= util.GRAD_TOL, impl
            assert (g[b:] - r[b:]).abs().max().item() <= util.GRAD_TOL, impl
