"""CPU checks of the backward oracle: against gradients that autograd produced through the reference's own
PyTorch module (golden fixtures), against autograd through this build's forward oracle math, and against
identities the gradients of attention satisfy at any size."""
import glob
import math
import os

import numpy as np
import pytest
import torch

from oracle.attn_oracle import attn_bwd_oracle, attn_fwd_oracle, make_prefill_inputs

GOLDEN = [p for p in sorted(glob.glob(os.path.join(os.path.dirname(__file__), "golden", "case_*.npz")))
          if "dq_ref_fp32" in np.load(p).files]


def _bf16(bits: np.ndarray) -> torch.Tensor:
    return torch.from_numpy(bits.view(np.int16).copy()).view(torch.bfloat16)


def test_golden_gradient_cases_present():
    assert len(GOLDEN) >= 5


@pytest.mark.parametrize("path", GOLDEN, ids=[os.path.basename(p) for p in GOLDEN])
def test_oracle_matches_reference_module_gradients(path):
    z = np.load(path)
    b, n, h, hkv, d, causal, _seed = [int(x) for x in z["shape"]]
    q, k, v, d_o = _bf16(z["q"]), _bf16(z["k"]), _bf16(z["v"]), _bf16(z["d_o"])
    assert d_o.shape == (b, n, h, d)
    kv_lens = torch.from_numpy(z["kv_lens"]) if "kv_lens" in z.files else None  # the reference's key_padding_mask
    dq, dk, dv, _delta = attn_bwd_oracle(q, k, v, d_o, causal=bool(causal), kv_lens=kv_lens)
    for name, got in (("dq", dq), ("dk", dk), ("dv", dv)):
        ref = torch.from_numpy(z[name + "_ref_fp32"])
        assert got.shape == ref.shape
        # both sides are fp32 evaluations of the same formulas in a different operation order
        assert float((got - ref).abs().max()) <= 2e-5 * max(1.0, float(ref.abs().max())), name


CROSS = sorted(glob.glob(os.path.join(os.path.dirname(__file__), "golden", "cross_*.npz")))


@pytest.mark.parametrize("path", CROSS, ids=[os.path.basename(p) for p in CROSS])
def test_oracle_matches_reference_gradients_with_unequal_lengths_and_causal_padding(path):
    """Sq != Sk and causal + key padding: gradients autograd produced through the reference's CrossAttention
    (base.py:104-116 mask alignment). The fixtures' upstream gradient is zero on rows that see no key, so those rows
    contribute nothing on either side; their dq is zero here (the reference's is not: it differentiates its uniform
    attention over masked keys) and is excluded."""
    from test_oracle import load_cross

    z, q, k, v, d_o, kv_lens, causal, valid = load_cross(path)
    dq, dk, dv, _delta = attn_bwd_oracle(q, k, v, d_o, causal=causal, kv_lens=kv_lens)
    for name, got in (("dq", dq), ("dk", dk), ("dv", dv)):
        ref = torch.from_numpy(z[name + "_ref_fp32"])
        assert got.shape == ref.shape
        diff = (got - ref).abs()
        if name == "dq":
            diff = diff[valid]
        assert float(diff.max()) <= 2e-5 * float(ref.abs().max()), name
    if not bool(valid.all()):
        assert float(dq[~valid].abs().max()) == 0.0


def test_oracle_matches_autograd_in_fp64():
    q, k, v = make_prefill_inputs(2, 128, 6, 2, 64, seed=31)
    d_o = torch.randn((2, 128, 6, 64), generator=torch.Generator().manual_seed(32)).to(torch.bfloat16)
    for causal in (False, True):
        qf, kf, vf = (t.double().requires_grad_(True) for t in (q, k, v))
        kk = kf.repeat_interleave(3, dim=2)
        vv = vf.repeat_interleave(3, dim=2)
        s = torch.einsum("bthd,bshd->bhts", qf, kk) / math.sqrt(64)
        if causal:
            s = s.masked_fill(torch.triu(torch.ones(128, 128, dtype=torch.bool), 1), float("-inf"))
        o = torch.einsum("bhts,bshd->bthd", torch.softmax(s, dim=-1), vv)
        o.backward(d_o.double())
        dq, dk, dv, delta = attn_bwd_oracle(q, k, v, d_o, causal=causal, dtype=torch.float64)
        assert float((dq - qf.grad).abs().max()) < 1e-12
        assert float((dk - kf.grad).abs().max()) < 1e-12
        assert float((dv - vf.grad).abs().max()) < 1e-12
        ref_delta = (o.detach() * d_o.double()).sum(-1).permute(0, 2, 1).unsqueeze(2)
        assert float((delta - ref_delta).abs().max()) < 1e-12


def test_gradient_identities():
    """Identities that hold for any size and are used as full-size checks on the GPU:
    (1) the output does not change under q -> a q, k -> k / a, hence <q, dq> == <k, dk> per (batch, kv head);
    (2) softmax rows sum to one, hence sum_s dv[s] == sum_t sum_heads d_o[t] per (batch, kv head);
    (3) the gradients are linear in d_o."""
    q, k, v = make_prefill_inputs(1, 256, 4, 2, 64, seed=33)
    gen = torch.Generator().manual_seed(34)
    d1 = torch.randn((1, 256, 4, 64), generator=gen).to(torch.bfloat16)
    d2 = torch.randn((1, 256, 4, 64), generator=gen).to(torch.bfloat16)
    for causal in (False, True):
        dq, dk, dv, _ = attn_bwd_oracle(q, k, v, d1, causal=causal, dtype=torch.float64)
        for kh in range(2):
            lhs = (q[0, :, 2 * kh:2 * kh + 2].double() * dq[0, :, 2 * kh:2 * kh + 2]).sum()
            rhs = (k[0, :, kh].double() * dk[0, :, kh]).sum()
            assert abs(float(lhs - rhs)) < 1e-9 * max(1.0, abs(float(lhs)))
            assert float((dv[0, :, kh].sum(0) - d1[0, :, 2 * kh:2 * kh + 2].double().sum((0, 1))).abs().max()) < 1e-9
        dq2, dk2, dv2, _ = attn_bwd_oracle(q, k, v, d2, causal=causal, dtype=torch.float64)
        dqs, dks, dvs, _ = attn_bwd_oracle(q, k, v, 0.5 * d1.double() + d2.double(), causal=causal, dtype=torch.float64)
        assert float((dqs - (0.5 * dq + dq2)).abs().max()) < 1e-10
        assert float((dks - (0.5 * dk + dk2)).abs().max()) < 1e-10
        assert float((dvs - (0.5 * dv + dv2)).abs().max()) < 1e-10


def test_first_causal_key_collects_everything_from_row_zero():
    """Query 0 of a causal problem sees only key 0: P[0,0] = 1, so dv[0] contains d_o[0] in full and its
    score gradient vanishes (dq[0] == 0)."""
    q, k, v = make_prefill_inputs(1, 128, 1, 1, 64, seed=35)
    d_o = torch.zeros((1, 128, 1, 64), dtype=torch.bfloat16)
    d_o[0, 0, 0] = 1.0
    dq, dk, dv, _ = attn_bwd_oracle(q, k, v, d_o, causal=True)
    assert float(dq.abs().max()) < 1e-6 and float(dk.abs().max()) < 1e-6
    assert torch.allclose(dv[0, 0, 0], torch.ones(64)) and float(dv[0, 1:].abs().max()) == 0.0


def test_delta_uses_forward_output():
    q, k, v = make_prefill_inputs(1, 128, 2, 1, 64, seed=36)
    d_o = torch.randn((1, 128, 2, 64), generator=torch.Generator().manual_seed(37)).to(torch.bfloat16)
    o, _ = attn_fwd_oracle(q, k, v, causal=False)
    _, _, _, delta = attn_bwd_oracle(q, k, v, d_o, causal=False)
    ref = (o.float() * d_o.float()).sum(-1).permute(0, 2, 1).unsqueeze(2)
    assert float((delta - ref).abs().max()) < 2e-2  # o is rounded to bf16 on one side only
