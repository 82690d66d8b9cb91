"""CPU checks of the oracle: against the golden outputs of the reference's own PyTorch module, against
the defining identities of the path, and on the edge cases the domain has."""
import glob
import math
import os

import numpy as np
import pytest
import torch

from oracle.attn_oracle import (
    attn_fwd_oracle,
    paged_kv_append_oracle,
    make_paged_inputs,
    make_prefill_inputs,
    paged_decode_oracle,
    robustness_check,
)

GOLDEN = sorted(glob.glob(os.path.join(os.path.dirname(__file__), "golden", "case_*.npz")))


def _bf16(bits: np.ndarray) -> torch.Tensor:
    return torch.from_numpy(bits.view(np.int16).copy()).view(torch.bfloat16)


def test_golden_files_present():
    assert len(GOLDEN) >= 5


@pytest.mark.parametrize("path", GOLDEN, ids=[os.path.basename(p) for p in GOLDEN])
def test_oracle_matches_reference_module(path):
    z = np.load(path)
    b, n, h, hkv, d, causal, _seed = [int(x) for x in z["shape"]]
    q, k, v = _bf16(z["q"]), _bf16(z["k"]), _bf16(z["v"])
    assert q.shape == (b, n, h, d) and k.shape == (b, n, hkv, d)
    kv_lens = torch.from_numpy(z["kv_lens"]) if "kv_lens" in z.files else None
    o, lse = attn_fwd_oracle(q, k, v, causal=bool(causal), kv_lens=kv_lens)
    o_ref = torch.from_numpy(z["o_ref_fp32"])
    # The reference module run on fp32 copies computes the same math; the only difference left is the
    # oracle's final rounding of O to bf16 (half an ulp: 2^-9 relative).
    err = (o.float() - o_ref).abs()
    assert float((err - o_ref.abs() * 2.0 ** -8).max()) <= 1e-5
    # L against the definition applied to the reference's score expression (fp64)
    l_ref = torch.from_numpy(z["lse_def_fp64"]).float()  # [B,H,N]
    assert lse.shape == (b, h, 1, n)
    assert float((lse[:, :, 0, :] - l_ref).abs().max()) <= 2e-5
    if "o_ref_native_bf16" in z.files:
        # stock bf16 behaviour of the reference (bf16 softmax): agrees within the build tolerance
        o_nat = _bf16(z["o_ref_native_bf16"]).reshape(b, n, h, d)
        assert float((o.float() - o_nat.float()).abs().max()) <= 2e-2


LPIN = sorted(glob.glob(os.path.join(os.path.dirname(__file__), "golden", "lpin_*.npz")))


@pytest.mark.parametrize("path", LPIN, ids=[os.path.basename(p) for p in LPIN])
def test_lse_is_what_the_reference_backward_harness_consumes(path):
    """L is pinned by the reference code that uses it: the backward harness's simple_flash_backward
    (kernels/attn/gqa_backwards/test_python.py:100-137) recomputes P = exp(S - L); the fixture holds what that
    function, taken from the harness source and run on the oracle's L, returned. (i) the L stored there is the L the
    oracle computes now; (ii) rows of the function's P sum to one; (iii) its gradients are the reference module's
    autograd gradients. A wrong base of the logarithm, a missing scale or a transposed layout fails (ii) and (iii)."""
    z = np.load(path)
    case = np.load(path.replace("lpin_", "case_"))
    b, n, h, hkv, d, causal, _seed = [int(x) for x in case["shape"]]
    assert not causal  # the harness function applies no mask
    q, k, v = _bf16(case["q"]), _bf16(case["k"]), _bf16(case["v"])
    _o, lse = attn_fwd_oracle(q, k, v, causal=False)
    assert z["lse_fed"].shape == (b, h, n)
    assert float((lse[:, :, 0, :] - torch.from_numpy(z["lse_fed"])).abs().max()) <= 1e-6
    assert float(np.abs(z["p_rowsum"] - 1.0).max()) <= 1e-6
    for name in ("dq", "dk", "dv"):
        ref = case[name + "_ref_fp32"]
        assert float(np.abs(z[name] - ref).max()) <= 2e-5 * float(np.abs(ref).max())


CROSS = sorted(glob.glob(os.path.join(os.path.dirname(__file__), "golden", "cross_*.npz")))


def load_cross(path):
    """A cross_*.npz fixture (tests/golden/make_golden.py, cross_main): tensors and the case's parameters."""
    z = np.load(path)
    b, sq, sk, h, hkv, d, causal, _seed = [int(x) for x in z["shape"]]
    q = _bf16(z["q"]).reshape(b, sq, h, d)
    k = _bf16(z["k"]).reshape(b, sk, hkv, d)
    v = _bf16(z["v"]).reshape(b, sk, hkv, d)
    d_o = _bf16(z["d_o"]).reshape(b, sq, h, d)
    kv_lens = torch.from_numpy(z["kv_lens"]) if "kv_lens" in z.files else None
    return z, q, k, v, d_o, kv_lens, bool(causal), torch.from_numpy(z["row_valid"])


def test_cross_fixtures_present():
    assert len(CROSS) >= 4


@pytest.mark.parametrize("path", CROSS, ids=[os.path.basename(p) for p in CROSS])
def test_oracle_matches_reference_module_with_unequal_lengths_and_causal_padding(path):
    """Sq != Sk, and causal together with key padding, against the reference's CrossAttention (base.py:104-116: the
    causal mask is aligned to the last query and the last kept key). Rows the mask leaves without any key are O = 0,
    L = -inf here and are excluded from the comparison (the reference's -10000 fill spreads them over masked keys)."""
    z, q, k, v, _d_o, kv_lens, causal, valid = load_cross(path)
    o, lse = attn_fwd_oracle(q, k, v, causal=causal, kv_lens=kv_lens)
    o_ref = torch.from_numpy(z["o_ref_fp32"])
    err = (o.float() - o_ref).abs() - o_ref.abs() * 2.0 ** -8
    assert float(err[valid].max()) <= 1e-5
    l_ref = torch.from_numpy(z["lse_def_fp64"]).float()                  # [B,H,Sq]
    vh = valid.unsqueeze(1).expand_as(l_ref)
    assert float((lse[:, :, 0, :] - l_ref)[vh].abs().max()) <= 2e-5
    if not bool(valid.all()):
        assert float(o[~valid].float().abs().max()) == 0.0
        assert bool(torch.isinf(lse[:, :, 0, :][~vh]).all()) and bool((lse[:, :, 0, :][~vh] < 0).all())


def test_generators_reproduce_golden_inputs():
    z = np.load([p for p in GOLDEN if "c1_" in p][0])
    b, n, h, hkv, d, _c, seed = [int(x) for x in z["shape"]]
    q, k, v = make_prefill_inputs(b, n, h, hkv, d, seed)
    assert torch.equal(q, _bf16(z["q"]).reshape(q.shape))
    assert torch.equal(k, _bf16(z["k"]).reshape(k.shape))
    assert torch.equal(v, _bf16(z["v"]).reshape(v.shape))


def test_lse_identity_and_rows_sum_to_one():
    q, k, v = make_prefill_inputs(1, 128, 4, 2, 64, seed=5)
    o, lse = attn_fwd_oracle(q, k, v, causal=True)
    scale = 1.0 / math.sqrt(64)
    kk = k.float().repeat_interleave(2, dim=2)
    vv = v.float().repeat_interleave(2, dim=2)
    s = torch.einsum("bthd,bshd->bhts", q.float(), kk) * scale
    s = s.masked_fill(torch.triu(torch.ones(128, 128, dtype=torch.bool), 1), float("-inf"))
    p = torch.exp(s - lse[:, :, 0, :, None])  # O = sum_j exp(s_j - L) v_j
    assert float((p.sum(-1) - 1).abs().max()) < 1e-5
    o2 = torch.einsum("bhts,bshd->bthd", p, vv)
    assert float((o2 - o.float()).abs().max()) < 2e-2


def test_first_causal_row_sees_one_key():
    q, k, v = make_prefill_inputs(1, 128, 2, 1, 64, seed=6)
    o, lse = attn_fwd_oracle(q, k, v, causal=True)
    assert torch.equal(o[0, 0, 0], v[0, 0, 0])
    s00 = float((q[0, 0, 0].float() * k[0, 0, 0].float()).sum()) / 8.0
    assert abs(float(lse[0, 0, 0, 0]) - s00) < 1e-5


def test_extreme_logits_stay_finite():
    q, k, v = make_prefill_inputs(1, 128, 2, 2, 64, seed=7)
    q = (q.float() * 30).to(torch.bfloat16)  # logits of several hundred
    o, lse = attn_fwd_oracle(q, k, v)
    assert torch.isfinite(o.float()).all() and torch.isfinite(lse).all()
    # all-equal logits: softmax is uniform, O is the mean of V
    qz = torch.zeros_like(q)
    o, lse = attn_fwd_oracle(qz, k, v)
    assert float((o[0, 5, 0].float() - v[0, :, 0].float().mean(0)).abs().max()) < 1e-2
    assert abs(float(lse[0, 0, 0, 0]) - math.log(128)) < 1e-5


def test_gqa_equals_mha_with_repeated_kv():
    q, k, v = make_prefill_inputs(1, 128, 4, 2, 64, seed=8)
    o1, l1 = attn_fwd_oracle(q, k, v)
    o2, l2 = attn_fwd_oracle(q, k.repeat_interleave(2, dim=2), v.repeat_interleave(2, dim=2))
    assert torch.equal(o1, o2) and torch.equal(l1, l2)


def test_paged_oracle_equals_contiguous_attention_last_row():
    qd, kp, vp, table, ctx = make_paged_inputs(3, 8, 2, 64, 16, 64, 5, 200, seed=9)
    o, lse = paged_decode_oracle(qd, kp, vp, table, ctx)
    assert o.shape == (3, 1, 8, 64) and lse.shape == (3, 8, 1, 1)
    for s in range(3):
        c = int(ctx[s])
        npg = (c + 15) // 16
        ks = kp[table[s, :npg].long()].reshape(-1, 2, 64)[:c]
        vs = vp[table[s, :npg].long()].reshape(-1, 2, 64)[:c]
        # contiguous causal attention whose last query row is the decode query
        qfull = torch.zeros((1, c, 8, 64), dtype=torch.bfloat16)
        qfull[0, -1] = qd[s, 0]
        o_c, l_c = attn_fwd_oracle(qfull, ks[None], vs[None], causal=True)
        assert torch.equal(o_c[0, -1], o[s, 0])
        assert float((l_c[0, :, 0, -1] - lse[s, :, 0, 0]).abs().max()) < 1e-5


def test_paged_inputs_are_well_formed():
    q, kp, vp, table, ctx = make_paged_inputs(8, 8, 2, 64, 16, 400, 1, 700, seed=3)
    used = []
    for s in range(8):
        npg = (int(ctx[s]) + 15) // 16
        used += table[s, :npg].tolist()
    assert len(set(used)) == len(used), "page ids must be distinct across sequences"
    assert min(used) >= 0 and max(used) < 400
    assert int(ctx.min()) >= 1 and int(ctx.max()) <= 700


def test_robustness_check_counts_like_the_reference_harness():
    ref = torch.ones(10)
    pred = ref.clone()
    pred[0] += 0.2  # beyond 0.001 + 0.05*1
    pred[1] += 0.01  # within
    max_abs, err, numel, _l2, cos = robustness_check(ref, pred)
    assert err == 1 and numel == 10 and abs(max_abs - 0.2) < 1e-6 and cos > 0.99


def test_paged_append_equals_contiguous_slice_assignment():
    """The reference updates a contiguous cache with kv_cache[b, off:off+T] = kv (mha.py:16-42); gathering the
    paged cache through the block table after the paged append must give the same contiguous result."""
    q, kp, vp, table, ctx = make_paged_inputs(3, 4, 2, 64, 16, 80, 30, 200, seed=11)
    t = 5
    gen = torch.Generator().manual_seed(1)
    k_new = torch.randn((3, t, 2, 64), generator=gen).to(torch.bfloat16)
    v_new = torch.randn((3, t, 2, 64), generator=gen).to(torch.bfloat16)
    start = (ctx - t).to(torch.int32)
    kp2, vp2 = paged_kv_append_oracle(k_new, v_new, kp, vp, table, start)
    for s in range(3):
        c = int(ctx[s])
        npg = (c + 15) // 16
        ids = table[s, :npg].long()
        before = kp[ids].reshape(-1, 2, 64)[:c].clone()
        before[c - t:c] = k_new[s]  # the reference's slice assignment on the contiguous view
        after = kp2[ids].reshape(-1, 2, 64)[:c]
        assert torch.equal(before.view(torch.int16), after.view(torch.int16))
    # pages of other sequences are untouched
    used = set()
    for s in range(3):
        used |= set(table[s, :(int(ctx[s]) + 15) // 16].tolist())
    rest = [i for i in range(80) if i not in used]
    assert torch.equal(kp2[rest].view(torch.int16), kp[rest].view(torch.int16))
