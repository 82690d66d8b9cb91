"""Paged KV-cache append: byte movement, so the GPU result must equal the CPU oracle bit for bit."""
import pytest
import torch

import hipkittens_b200 as hk
from hipkittens_b200 import _native
from hipkittens_b200.synthetic import make_paged_inputs
from oracle.attn_oracle import paged_decode_oracle, paged_kv_append_oracle

pytestmark = pytest.mark.gpu


def _bits(t):
    return t.contiguous().view(torch.int16)


@pytest.mark.parametrize("s,t,hkv,d,lo,hi,seed", [
    (4, 1, 8, 128, 1, 500, 0),     # one decode step: one token per sequence
    (3, 40, 2, 128, 1, 300, 1),    # a prefill chunk crossing page boundaries
    (2, 16, 4, 64, 16, 16, 2),     # starts exactly on a page boundary, D = 64
    (5, 7, 1, 128, 1, 90, 3),
])
def test_append_is_bit_exact(s, t, hkv, d, lo, hi, seed):
    dev = torch.device("cuda:0")
    h = hkv
    _q, kp, vp, bt, ctx = make_paged_inputs(s, h, hkv, d, 16, 400, lo + t, hi + t, seed)
    start = (ctx - t).to(torch.int32)  # the last t positions of every context are (re)written
    gen = torch.Generator().manual_seed(100 + seed)
    k_new = torch.randn((s, t, hkv, d), generator=gen).to(torch.bfloat16)
    v_new = torch.randn((s, t, hkv, d), generator=gen).to(torch.bfloat16)
    kp_ref, vp_ref = paged_kv_append_oracle(k_new, v_new, kp, vp, bt, start)
    kp_d, vp_d = kp.to(dev), vp.to(dev)
    hk.paged_kv_append(k_new.to(dev), v_new.to(dev), kp_d, vp_d, bt.to(dev), start.to(dev))
    assert _native.device_status(0) == 0
    assert torch.equal(_bits(kp_d.cpu()), _bits(kp_ref)) and torch.equal(_bits(vp_d.cpu()), _bits(vp_ref))


def test_append_then_decode_matches_oracle_on_updated_cache():
    dev = torch.device("cuda:0")
    q, kp, vp, bt, ctx = make_paged_inputs(3, 16, 2, 128, 16, 300, 40, 900, seed=5)
    gen = torch.Generator().manual_seed(7)
    k_new = torch.randn((3, 1, 2, 128), generator=gen).to(torch.bfloat16)
    v_new = torch.randn((3, 1, 2, 128), generator=gen).to(torch.bfloat16)
    start = (ctx - 1).to(torch.int32)
    kp_d, vp_d = kp.to(dev), vp.to(dev)
    hk.paged_kv_append(k_new.to(dev), v_new.to(dev), kp_d, vp_d, bt.to(dev), start.to(dev))
    o, l = hk.paged_decode(q.to(dev), kp_d, vp_d, bt.to(dev), ctx.to(dev))
    assert _native.device_status(0) == 0
    kp_ref, vp_ref = paged_kv_append_oracle(k_new, v_new, kp, vp, bt, start)
    o_ref, l_ref = paged_decode_oracle(q, kp_ref, vp_ref, bt, ctx)
    assert float((o.float().cpu() - o_ref.float()).abs().max()) <= 2e-2
    assert float((l.cpu() - l_ref).abs().max()) <= 1e-3


def test_bad_positions_and_ids_are_skipped_and_reported():
    dev = torch.device("cuda:0")
    _q, kp, vp, bt, ctx = make_paged_inputs(2, 4, 4, 128, 16, 50, 20, 60, seed=6)
    k_new = torch.ones((2, 1, 4, 128), dtype=torch.bfloat16)
    v_new = torch.ones((2, 1, 4, 128), dtype=torch.bfloat16)
    kp_d, vp_d = kp.to(dev), vp.to(dev)
    # position beyond the block table
    start = torch.tensor([int(ctx[0]) - 1, bt.shape[1] * 16], dtype=torch.int32)
    hk.paged_kv_append(k_new.to(dev), v_new.to(dev), kp_d, vp_d, bt.to(dev), start.to(dev))
    assert _native.device_status(0) == _native.HK_EBADPAGE
    kp_ref, vp_ref = paged_kv_append_oracle(k_new, v_new, kp, vp, bt, start)
    assert torch.equal(_bits(kp_d.cpu()), _bits(kp_ref))
    # page id outside the pool
    bad = bt.clone()
    bad[0, (int(ctx[0]) - 1) // 16] = 50
    start = (ctx - 1).to(torch.int32)
    kp_d2 = kp.to(dev)
    hk.paged_kv_append(k_new.to(dev), v_new.to(dev), kp_d2, vp_d, bad.to(dev), start.to(dev))
    assert _native.device_status(0) == _native.HK_EBADPAGE
    kp_ref2, _ = paged_kv_append_oracle(k_new, v_new, kp, vp, bad, start)
    assert torch.equal(_bits(kp_d2.cpu()), _bits(kp_ref2))
