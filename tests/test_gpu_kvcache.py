"""KV-cache decode parity: in-place append, fused rotary, paged gather, split-KV."""
import numpy as np
import pytest
import torch

import cases
import util
from oracle import attention_oracle as orc
from util import DEV, maxdiff

pytestmark = pytest.mark.gpu


def fa():
    import flash_attn_triton_b200 as m
    return m


def dev(t):
    return None if t is None else t.to(DEV)


def test_golden_paged(golden):
    """Reference output (with the append done by the harness, see make_golden.py) and the
    cache rows the append must produce, bit for bit."""
    g = golden("kvcache_paged")
    lens = g["lens"].tolist()
    q, kc, vc, kn, vn, bt, cl = cases.paged_case(40, 3, 8, 2, 64, 64, 12, lens, 4)
    cos, sin = cases.rotary_tables(256, 64)
    kcd, vcd = kc.to(DEV), vc.to(DEV)
    for splits in (0, 1, 3):
        kcd.copy_(kc); vcd.copy_(vc)
        out = fa().flash_attn_with_kvcache(dev(q), kcd, vcd, dev(kn), dev(vn), dev(cos), dev(sin),
                                           cache_seqlens=dev(cl), block_table=dev(bt),
                                           rotary_interleaved=False, num_splits=splits)
        assert maxdiff(out, g["out"]) <= util.FWD_TOL
        for i, (p, o) in enumerate(g["touched"].tolist()):
            assert torch.equal(kcd[p, o].cpu(), torch.from_numpy(g["k_rows"][i]))
            assert torch.equal(vcd[p, o].cpu(), torch.from_numpy(g["v_rows"][i]))
        mask = torch.ones(kc.shape[:2], dtype=torch.bool)
        for p, o in g["touched"].tolist():
            mask[p, o] = False
        assert torch.equal(kcd.cpu()[mask], kc[mask]) and torch.equal(vcd.cpu()[mask], vc[mask])


def _contig_case(seed, B, Bc, cap, Hq, Hkv, D, Sq, Sn, dtype=torch.float16):
    rng = np.random.default_rng(seed)
    mk = lambda *s: torch.from_numpy(rng.standard_normal(s, dtype=np.float32)).to(dtype)
    return mk(B, Sq, Hq, D), mk(Bc, cap, Hkv, D), mk(Bc, cap, Hkv, D), (mk(B, Sn, Hkv, D) if Sn else None), \
        (mk(B, Sn, Hkv, D) if Sn else None)


def test_noncausal_window_alibi_is_bottom_right(golden):
    """Without `causal`, window and ALiBi of a decode call are still measured from the end of the
    sequence here.  The reference measures them from query position 0 in that case
    (flash_attn_interface.py:523); its output is pinned in the golden so that the difference is a
    known one (the CPU suite checks the oracle's restatement of the reference against it)."""
    g = golden("kvcache_noncausal_window")
    lens = golden("kvcache_paged")["lens"].tolist()
    q, kc, vc, kn, vn, bt, cl = cases.paged_case(40, 3, 8, 2, 64, 64, 12, lens, 4)
    cos, sin = cases.rotary_tables(256, 64)
    sl = torch.from_numpy(g["slopes"])
    out = fa().flash_attn_with_kvcache(dev(q), dev(kc), dev(vc), dev(kn), dev(vn), dev(cos), dev(sin),
                                       cache_seqlens=dev(cl), block_table=dev(bt), rotary_interleaved=False,
                                       causal=False, window_size=(-1, 40), alibi_slopes=dev(sl))
    ro, _, _ = orc.kvcache_ref(q, kc, vc, kn, vn, cos, sin, cache_seqlens=cl, block_table=bt, causal=False,
                               window=(-1, 40), alibi_slopes=sl, rotary_interleaved=False)
    assert maxdiff(out, ro) <= util.FWD_TOL
    assert maxdiff(out, g["out"]) > 0.05


CONTIG = [
    # B, Bc, cap, Hq, Hkv, D, Sq, Sn, lens, kwargs
    (2, 2, 128, 4, 4, 64, 1, 1, [0, 100], dict()),
    (3, 5, 300, 8, 2, 128, 1, 1, [299, 17, 64], dict(rotary=64, interleaved=True, batch_idx=[4, 0, 2])),
    (2, 2, 200, 4, 1, 128, 1, 0, [200, 3], dict(window=(20, -1))),
    (2, 2, 256, 8, 2, 64, 3, 3, [50, 200], dict(causal=True, rotary=32, interleaved=False)),
    (2, 2, 256, 16, 2, 64, 2, 2, [10, 100], dict(causal=True, alibi=True)),
    (2, 2, 160, 4, 2, 32, 1, 1, [30, 90], dict(leftpad=[5, 0], rotary=32, interleaved=True)),
    (1, 1, 96, 2, 2, 256, 1, 1, [40], dict()),
    (2, 2, 64, 2, 2, 16, 5, 0, [64, 9], dict(causal=True)),
    (2, 2, 2100, 32, 8, 128, 1, 1, [2099, 1500], dict(splits=5, rotary=128, interleaved=False)),
]


@pytest.mark.parametrize("case", range(len(CONTIG)))
def test_contiguous_cache_vs_oracle(case):
    B, Bc, cap, Hq, Hkv, D, Sq, Sn, lens, kw = CONTIG[case]
    q, kc, vc, kn, vn = _contig_case(200 + case, B, Bc, cap, Hq, Hkv, D, Sq, Sn)
    cl = torch.tensor(lens, dtype=torch.int32)
    cos = sin = None
    if "rotary" in kw:
        cos, sin = cases.rotary_tables(cap + 8, kw["rotary"])
    idx = torch.tensor(kw["batch_idx"], dtype=torch.int32) if "batch_idx" in kw else None
    pad = torch.tensor(kw["leftpad"], dtype=torch.int32) if "leftpad" in kw else None
    sl = torch.tensor([0.5 ** (i + 1) for i in range(Hq)]) if kw.get("alibi") else None
    common = dict(causal=kw.get("causal", False), rotary_interleaved=kw.get("interleaved", True))
    ro, rkc, rvc = orc.kvcache_ref(q, kc, vc, kn, vn, cos, sin, cache_seqlens=cl, cache_batch_idx=idx,
                                   cache_leftpad=pad, window=kw.get("window", (-1, -1)),
                                   alibi_slopes=sl, **common)
    kcd, vcd = kc.to(DEV), vc.to(DEV)
    out = fa().flash_attn_with_kvcache(dev(q), kcd, vcd, dev(kn), dev(vn), dev(cos), dev(sin),
                                       cache_seqlens=dev(cl), cache_batch_idx=dev(idx),
                                       cache_leftpad=dev(pad), window_size=kw.get("window", (-1, -1)),
                                       alibi_slopes=dev(sl), num_splits=kw.get("splits", 0), **common)
    assert maxdiff(out, ro) <= util.FWD_TOL
    assert torch.equal(kcd.cpu(), rkc) and torch.equal(vcd.cpu(), rvc)


@pytest.mark.parametrize("page,dtype", [(16, torch.float16), (48, torch.float16), (256, torch.bfloat16)])
def test_paged_vs_oracle(page, dtype):
    B, Hq, Hkv, D = 4, 8, 2, 128
    lens = [1, page * 3 - 1, page * 2, 5 * page + 7]
    maxp = 7
    q, kc, vc, kn, vn, bt, cl = cases.paged_case(300 + page, B, Hq, Hkv, D, page, 32, lens, maxp)
    q, kc, vc, kn, vn = (t.to(dtype) for t in (q, kc, vc, kn, vn))
    cos, sin = cases.rotary_tables(maxp * page + 1, 64, dtype=dtype)
    ro, rkc, rvc = orc.kvcache_ref(q, kc, vc, kn, vn, cos, sin, cache_seqlens=cl, block_table=bt,
                                   rotary_interleaved=True, causal=True)
    kcd, vcd = kc.to(DEV), vc.to(DEV)
    out = fa().flash_attn_with_kvcache(dev(q), kcd, vcd, dev(kn), dev(vn), dev(cos), dev(sin),
                                       cache_seqlens=dev(cl), block_table=dev(bt.long()),
                                       rotary_interleaved=True, causal=True)
    tol = util.FWD_TOL if dtype == torch.float16 else util.BF16_FWD_TOL
    assert maxdiff(out, ro) <= tol
    assert torch.equal(kcd.cpu(), rkc) and torch.equal(vcd.cpu(), rvc)


def test_no_seqlens_and_errors():
    m = fa()
    q, kc, vc, _, _ = _contig_case(400, 2, 2, 64, 4, 2, 64, 1, 0)
    out = m.flash_attn_with_kvcache(dev(q), dev(kc), dev(vc))
    ro, _, _ = orc.kvcache_ref(q, kc, vc)
    assert maxdiff(out, ro) <= util.FWD_TOL
    with pytest.raises(ValueError):
        m.flash_attn_with_kvcache(dev(q), dev(kc), dev(vc), rotary_cos=torch.zeros(4, 8, device=DEV))
    with pytest.raises(ValueError):
        m.flash_attn_with_kvcache(dev(q), dev(kc), dev(vc), cache_seqlens=torch.tensor([65, 0], device=DEV))
    with pytest.raises(ValueError):
        m.flash_attn_with_kvcache(dev(q), dev(kc), dev(vc), block_table=torch.tensor([[0], [9]], device=DEV))
    with pytest.raises(ValueError):
        m.flash_attn_with_kvcache(dev(q), dev(kc), dev(vc), k=dev(q[:, :, :2]), v=None)


def test_config4_shape():
    """batch 64, Hq32/Hkv8, D128, page 256, 4096-page pool, lengths U[1024,32768], one new
    token with non-interleaved rotary.  Output checked on four sequences against the
    oracle; the appended rows are checked for every sequence; nothing else may change."""
    m = fa()
    B, Hq, Hkv, D, page, pool = 64, 32, 8, 128, 256, 4096
    for seed in range(100):
        rng = np.random.default_rng(seed)
        lens = rng.integers(1024, 32769, size=B)
        if int(np.sum((lens + 1 + page - 1) // page)) <= pool:
            break
    maxp = 129
    g = torch.Generator(device=DEV).manual_seed(seed)
    kc = torch.randn(pool, page, Hkv, D, device=DEV, dtype=torch.float16, generator=g)
    vc = torch.randn(pool, page, Hkv, D, device=DEV, dtype=torch.float16, generator=g)
    q = torch.randn(B, 1, Hq, D, device=DEV, dtype=torch.float16, generator=g)
    kn = torch.randn(B, 1, Hkv, D, device=DEV, dtype=torch.float16, generator=g)
    vn = torch.randn(B, 1, Hkv, D, device=DEV, dtype=torch.float16, generator=g)
    perm = rng.permutation(pool)
    bt = np.zeros((B, maxp), dtype=np.int32)
    at = 0
    for b, L in enumerate(lens):
        need = (L + 1 + page - 1) // page
        bt[b, :need] = perm[at:at + need]
        bt[b, need:] = perm[at]
        at += need
    bt = torch.from_numpy(bt)
    cl = torch.tensor(lens, dtype=torch.int32)
    cos, sin = cases.rotary_tables(32769 + 8, 128)
    kc0, vc0 = kc.clone(), vc.clone()
    out = m.flash_attn_with_kvcache(q, kc, vc, kn, vn, cos.to(DEV), sin.to(DEV), cache_seqlens=cl.to(DEV),
                                    block_table=bt.to(DEV), rotary_interleaved=False)
    assert torch.isfinite(out).all()
    touched = torch.zeros(pool, page, dtype=torch.bool)
    for b, L in enumerate(lens.tolist()):
        pg, row = int(bt[b, L // page]), L % page
        touched[pg, row] = True
        kr = orc.apply_rotary_ref(kn[b].cpu(), cos, sin, torch.tensor([L]), False)
        assert torch.equal(kc[pg, row].cpu(), kr[0]) and torch.equal(vc[pg, row].cpu(), vn[b, 0].cpu())
    t = touched.to(DEV)
    assert torch.equal(kc[~t], kc0[~t]) and torch.equal(vc[~t], vc0[~t])
    for b in (0, int(np.argmin(lens)), int(np.argmax(lens)), B - 1):
        L = int(lens[b])
        ids = bt[b, :(L + 1 + page - 1) // page].long()
        kb = kc[ids.to(DEV)].reshape(-1, Hkv, D)[:L + 1].cpu()
        vb = vc[ids.to(DEV)].reshape(-1, Hkv, D)[:L + 1].cpu()
        qb = orc.apply_rotary_ref(q[b].cpu(), cos, sin, torch.tensor([L]), False)
        ro, _ = orc.attention_ref(qb[None], kb[None], vb[None])
        assert maxdiff(out[b:b + 1], ro) <= util.FWD_TOL
