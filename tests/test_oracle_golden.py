"""The CPU oracle against the golden vectors produced by the unmodified reference
(tests/golden/make_golden.py).  No GPU needed.

Tolerances: the reference computes in fp16 with fp32 accumulation and its own measured
error against fp32 SDPA is ~1e-3 (outputs) / ~2e-3 (gradients) at these sizes, so the
oracle (exact fp32) must agree with it within 2e-3 / 1e-2, the bars the GPU kernels are
held to.  Quantised K codes and scales are bit-exact.
"""
import ast

import numpy as np
import pytest
import torch

import cases
from oracle import attention_oracle as orc

FWD_TOL = 2e-3
GRAD_TOL = 1e-2
LN2 = 0.6931471805599453


def maxdiff(a, b):
    a = torch.as_tensor(np.asarray(a)).float()
    b = torch.as_tensor(np.asarray(b)).float()
    return (a - b).abs().max().item()


@pytest.mark.parametrize("causal", [0, 1])
def test_dense_c1(golden, causal):
    g = golden(f"dense_c1_causal{causal}")
    q, k, v, do = cases.dense_case(0, 2, 128, 128, 4, 4, 64)
    assert cases.checksum(q, k, v, do) == str(g["checksum"])
    out, lse, dq, dk, dv = orc.attention_grads_ref(q, k, v, do, softmax_scale=0.125,
                                                   causal=bool(causal))
    assert maxdiff(out, g["out"]) <= FWD_TOL
    assert maxdiff(lse, g["lse2"] * LN2) <= FWD_TOL
    for name, t in (("dq", dq), ("dk", dk), ("dv", dv)):
        assert maxdiff(t, g[name]) <= GRAD_TOL, name


def test_dense_public(golden):
    g = golden("dense_public")
    specs = ast.literal_eval(str(g["_specs"]))
    for i, (name, (B, Sq, Sk, Hq, Hkv, D, kw)) in enumerate(specs.items()):
        q, k, v, do = cases.dense_case(100 + i, B, Sq, Sk, Hq, Hkv, D)
        assert cases.checksum(q, k, v, do) == str(g[name + ".checksum"]), name
        out, lse, dq, dk, dv = orc.attention_grads_ref(
            q, k, v, do, softmax_scale=kw.get("softmax_scale"), causal=kw.get("causal", False),
            window=kw.get("window_size", (-1, -1)), softcap=kw.get("softcap", 0.0),
            alibi_slopes=kw.get("alibi_slopes"))
        assert maxdiff(out, g[name + ".out"]) <= FWD_TOL, name
        for n, t in (("dq", dq), ("dk", dk), ("dv", dv)):
            assert maxdiff(t, g[f"{name}.{n}"]) <= GRAD_TOL, (name, n)


def test_varlen_all(golden):
    g = golden("varlen_all")
    ql, kl = g["q_lens"].tolist(), g["k_lens"].tolist()
    q, k, v, do, cu_q, cu_k = cases.varlen_case(7, ql, kl, 4, 2, 64)
    assert cases.checksum(q, k, v, do) == str(g["checksum"])
    out, lse, dq, dk, dv = orc.varlen_attention_grads_ref(
        q, k, v, do, cu_q, cu_k, softmax_scale=0.125, causal=True, window=(48, 0),
        softcap=30.0, alibi_slopes=torch.from_numpy(g["slopes"]))
    assert maxdiff(out, g["out"]) <= FWD_TOL
    assert maxdiff(lse, g["lse2"] * LN2) <= FWD_TOL
    for name, t in (("dq", dq), ("dk", dk), ("dv", dv)):
        assert maxdiff(t, g[name]) <= GRAD_TOL, name


def test_varlen_rect(golden):
    g = golden("varlen_rect")
    q, k, v, do, cu_q, cu_k = cases.varlen_case(8, [3, 5], [4, 6], 2, 2, 16)
    out, _ = orc.varlen_attention_ref(q, k, v, cu_q, cu_k, causal=True)
    assert maxdiff(out, g["out"]) <= FWD_TOL


def test_k_quantiser_bit_exact(golden):
    g = golden("int8_kquant")
    k = cases.k_with_outliers(21, 4, 192, 128)
    assert cases.checksum(k) == str(g["checksum"])
    k8, s_k = orc.quantize_k_rows_ref(k)
    assert np.array_equal(k8, g["k8"])
    assert np.array_equal(s_k.view(np.uint32), g["s_k"].view(np.uint32))


def test_round_i8_is_not_rint():
    x = np.array([0.49999997, 0.5, 1.5, 2.5, -0.5, -1.5, -0.49999997], dtype=np.float32)
    assert orc.round_i8_np(x).tolist() == [1, 1, 2, 3, -1, -2, -1]


@pytest.mark.parametrize("causal", [0, 1])
def test_int8_forward(golden, causal):
    g = golden(f"int8_fwd_causal{causal}")
    q, k, v = cases.int8_case(30, 1, 2, 256, 128)
    assert cases.checksum(q, k, v) == str(g["checksum"])
    out, lse2, _, _ = orc.attention_int8_ref(q, k, v, causal=bool(causal))
    assert maxdiff(out, g["out"]) <= FWD_TOL
    assert maxdiff(lse2, g["lse2"]) <= FWD_TOL


@pytest.mark.parametrize("causal", [0, 1])
def test_int8_backward(golden, causal):
    g = golden(f"int8_bwd_causal{causal}")
    q, k, v = cases.int8_case(31, 2, 2, 128, 64)
    do = cases.randn16(np.random.default_rng(32), 2, 2, 128, 64)
    assert cases.checksum(q, k, v, do) == str(g["checksum"])
    out, _, _, _ = orc.attention_int8_ref(q, k, v, causal=bool(causal), sm_scale=0.125)
    assert maxdiff(out, g["out"]) <= FWD_TOL
    dq, dk, dv = orc.attention_int8_grads_ref(q, k, v, do, causal=bool(causal), sm_scale=0.125)
    for name, t in (("dq", dq), ("dk", dk), ("dv", dv)):
        assert maxdiff(t, g[name]) <= GRAD_TOL, name


def test_kvcache_paged(golden):
    g = golden("kvcache_paged")
    lens = g["lens"].tolist()
    q, kc, vc, kn, vn, bt, cl = cases.paged_case(40, 3, 8, 2, 64, 64, 12, lens, 4)
    assert cases.checksum(q, kc, vc, kn, vn, bt) == str(g["checksum"])
    cos, sin = cases.rotary_tables(256, 64)
    out, kc2, vc2 = orc.kvcache_ref(q, kc, vc, kn, vn, cos, sin, cache_seqlens=cl,
                                    block_table=bt, causal=False, rotary_interleaved=False)
    assert maxdiff(out, g["out"]) <= FWD_TOL
    for i, (p, o) in enumerate(g["touched"].tolist()):
        assert torch.equal(kc2[p, o], torch.from_numpy(g["k_rows"][i]))
        assert torch.equal(vc2[p, o], torch.from_numpy(g["v_rows"][i]))
    # nothing else in the cache moved
    mask = torch.ones(kc.shape[:2], dtype=torch.bool)
    for p, o in g["touched"].tolist():
        mask[p, o] = False
    assert torch.equal(kc2[mask], kc[mask]) and torch.equal(vc2[mask], vc[mask])
    # causal=True is the same thing for one query row
    out_c, _, _ = orc.kvcache_ref(q, kc, vc, kn, vn, cos, sin, cache_seqlens=cl,
                                  block_table=bt, causal=True, rotary_interleaved=False)
    assert maxdiff(out_c, out) == 0.0


def test_compat_rotary(golden):
    """rotary_emb_ref against the reference's rotary kernel (run under the Triton interpreter):
    both compute in fp32 and round once, so they agree to the last bit or one fp16 step."""
    g = golden("compat_rotary")
    for name, spec in cases.ROTARY_CASES.items():
        x, cos, sin, kw = cases.rotary_case(**spec)
        assert cases.checksum(x, cos, sin) == bytes(g[name + "_checksum"]).decode()
        y = orc.rotary_emb_ref(x, cos, sin, **kw)
        ref = torch.from_numpy(g[name])
        assert ((y.float() - ref.float()).abs() - 2.0 ** -10 * ref.float().abs()).max().item() <= 1e-6, name


def test_compat_padding(golden):
    g = golden("compat_padding")
    hs, mask, lens_in_row = cases.padding_case(7, 3, 12, 2, 16)
    assert cases.checksum(hs, mask, lens_in_row) == bytes(g["checksum"]).decode()
    u, idx, cu, mx = orc.unpad_ref(hs, mask)
    assert torch.equal(u, torch.from_numpy(g["unpadded"])) and torch.equal(idx, torch.from_numpy(g["indices"]))
    assert torch.equal(cu, torch.from_numpy(g["cu_seqlens"])) and mx == int(g["max_seqlen"])
    assert torch.equal(orc.pad_ref(u, idx, 3, 12), torch.from_numpy(g["repadded"]))


@pytest.mark.parametrize("causal", [0, 1])
def test_int8_padded(golden, causal):
    """A padded call (150 valid tokens in 192 rows, seq_len_k = seq_len_q = 150): keys past the
    valid length take no part, in the forward and in the gradients."""
    g = golden(f"int8_padded_causal{causal}")
    q, k, v = cases.int8_case(33, 1, 2, 192, 64)
    do = cases.randn16(np.random.default_rng(34), 1, 2, 192, 64)
    assert cases.checksum(q, k, v, do) == str(g["checksum"])
    out, _, _, _ = orc.attention_int8_ref(q, k, v, causal=bool(causal), sm_scale=0.125, seq_len_k=150, seq_len_q=150)
    assert maxdiff(out, g["out"]) <= FWD_TOL
    dq, dk, dv = orc.attention_int8_grads_ref(q, k, v, do, causal=bool(causal), sm_scale=0.125,
                                              seq_len_k=150, seq_len_q=150)
    # dq of the padded query rows (>= seq_len_q) is left out: under a causal mask the reference's
    # backward does not apply the key-length mask to them and returns values of magnitude 45 there;
    # they are padding the caller discards.  dk and dv agree everywhere.
    assert maxdiff(dq[:, :, :150], g["dq"][:, :, :150]) <= GRAD_TOL
    for name, t in (("dk", dk), ("dv", dv)):
        assert maxdiff(t, g[name]) <= GRAD_TOL, name


def test_philox_known_answers():
    """The first Philox4x32-10 word for a few (seed, counter) pairs, as Triton's tl.rand produced
    them under its interpreter."""
    u = orc.philox_uniform(0, np.array([5, 982, 1959]))
    assert u.tolist() == [0.9006523489952087, 0.7447494268417358, 0.2224503457546234]
    u = orc.philox_uniform(1234, np.array([5, 982, 1959]))
    assert u.tolist() == [0.4206197261810303, 0.9028539061546326, 0.7525394558906555]


def test_dropout_dense(golden):
    """The reference's dropout, forward and backward, restated: same Philox counters, same
    dS = P_dropped * (dP - delta) backward."""
    g = golden("dropout")
    specs = ast.literal_eval(str(g["_specs"]))
    for i, (name, (B, Sq, Sk, Hq, Hkv, D, kw)) in enumerate(specs.items()):
        q, k, v, do = cases.dense_case(300 + i, B, Sq, Sk, Hq, Hkv, D)
        assert cases.checksum(q, k, v, do) == str(g[name + ".checksum"]), name
        out, lse, pd, dq, dk, dv = orc.attention_dropout_ref(
            q, k, v, do, dropout_p=kw["dropout_p"], seed=int(g[name + ".seed"]),
            softmax_scale=kw.get("softmax_scale"), causal=kw.get("causal", False), softcap=kw.get("softcap", 0.0))
        # kept probabilities are scaled by 1/(1-p), and fp16 rounding errors with them
        amp = 1.0 / (1.0 - kw["dropout_p"])
        assert maxdiff(out, g[name + ".out"]) <= FWD_TOL * amp, name
        for n, t in (("dq", dq), ("dk", dk), ("dv", dv)):
            assert maxdiff(t, g[f"{name}.{n}"]) <= GRAD_TOL * amp, (name, n)


def test_dropout_varlen(golden):
    g = golden("dropout")
    ql, kl = g["varlen.q_lens"].tolist(), g["varlen.k_lens"].tolist()
    q, k, v, do, cu_q, cu_k = cases.varlen_case(9, ql, kl, 4, 2, 64)
    assert cases.checksum(q, k, v, do) == str(g["varlen.checksum"])
    out, lse, pd, dq, dk, dv = orc.varlen_attention_dropout_ref(
        q, k, v, cu_q, cu_k, 101, do, dropout_p=0.2, seed=int(g["varlen.seed"]), causal=True)
    assert maxdiff(out, g["varlen.out"]) <= FWD_TOL / 0.8
    for n, t in (("dq", dq), ("dk", dk), ("dv", dv)):
        assert maxdiff(t, g["varlen." + n]) <= GRAD_TOL / 0.8, n


def test_dropout_varlen_deterministic(golden):
    """deterministic=True: every sequence through the dense path with a seed of its own."""
    g = golden("dropout")
    ql, kl = g["varlen.q_lens"].tolist(), g["varlen.k_lens"].tolist()
    q, k, v, do, cu_q, cu_k = cases.varlen_case(9, ql, kl, 4, 2, 64)
    seeds = g["varlen_det.seeds"].tolist()
    for b in range(len(ql)):
        qs, qe, ks, ke = int(cu_q[b]), int(cu_q[b + 1]), int(cu_k[b]), int(cu_k[b + 1])
        out, _, _, dq, dk, dv = orc.attention_dropout_ref(q[qs:qe][None], k[ks:ke][None], v[ks:ke][None],
                                                         do[qs:qe][None], dropout_p=0.2, seed=seeds[b], causal=True)
        assert maxdiff(out[0], g["varlen_det.out"][qs:qe]) <= FWD_TOL / 0.8, b
        assert maxdiff(dq[0], g["varlen_det.dq"][qs:qe]) <= GRAD_TOL / 0.8, b
        assert maxdiff(dk[0], g["varlen_det.dk"][ks:ke]) <= GRAD_TOL / 0.8, b
        assert maxdiff(dv[0], g["varlen_det.dv"][ks:ke]) <= GRAD_TOL / 0.8, b


def test_kvcache_noncausal_window_reference_alignment(golden):
    """Without `causal` the reference measures window and ALiBi of a decode call from query
    position 0 (flash_attn_interface.py:523); the oracle restates that behind a flag.  The library
    measures them from the end of the sequence (tests/test_gpu_kvcache.py), a documented difference."""
    g = golden("kvcache_noncausal_window")
    lens = golden("kvcache_paged")["lens"].tolist()
    q, kc, vc, kn, vn, bt, cl = cases.paged_case(40, 3, 8, 2, 64, 64, 12, lens, 4)
    cos, sin = cases.rotary_tables(256, 64)
    sl = torch.from_numpy(g["slopes"])
    out, _, _ = orc.kvcache_ref(q, kc, vc, kn, vn, cos, sin, cache_seqlens=cl, block_table=bt, causal=False,
                                window=(-1, 40), alibi_slopes=sl, rotary_interleaved=False, reference_alignment=True)
    assert maxdiff(out, g["out"]) <= FWD_TOL
    ours, _, _ = orc.kvcache_ref(q, kc, vc, kn, vn, cos, sin, cache_seqlens=cl, block_table=bt, causal=False,
                                 window=(-1, 40), alibi_slopes=sl, rotary_interleaved=False)
    assert maxdiff(ours, g["out"]) > 0.05          # the two conventions really differ on this case
