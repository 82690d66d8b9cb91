"""GPU parity of the chunked prefill against the paged KV cache (hk_attn_fwd_paged): T query rows per sequence against
that sequence's cached context, K and V gathered page by page through the block table. No counterpart exists in the
reference; the math is the forward's on the gathered K / V with the causal mask aligned to the end of the context
(training/llama/llama/models/attentions/base.py:104-116), so the oracle is attn_fwd_oracle on the gathered tensors.
Tolerances are the build's: max-abs 2e-2 on O, 1e-3 on L."""
import pytest
import torch

import hipkittens_b200 as hk
from hipkittens_b200 import _native
from hipkittens_b200.synthetic import make_paged_inputs
from oracle.attn_oracle import attn_fwd_oracle

pytestmark = pytest.mark.gpu
TOL_O, TOL_L = 2e-2, 1e-3


def gather(kp, vp, bt, max_len):
    """Contiguous [S, max_len, H_KV, D] K and V read through the block table (pages beyond a row's table are page 0)."""
    s_n = bt.shape[0]
    n_pg = (max_len + 15) // 16
    ids = bt[:, :n_pg].long().clamp(0, kp.shape[0] - 1)
    k = kp[ids].reshape(s_n, n_pg * 16, kp.shape[2], kp.shape[3])[:, :max_len].contiguous()
    v = vp[ids].reshape(s_n, n_pg * 16, vp.shape[2], vp.shape[3])[:, :max_len].contiguous()
    return k, v


CASES = [
    # S, T, H, H_KV, D, pool, ctx_lo, ctx_hi, causal, seed
    (3, 128, 8, 2, 128, 400, 128, 1500, True, 0),    # one query block, contexts of 1 to 12 tiles
    (2, 200, 4, 4, 64, 300, 200, 900, True, 1),      # T not a multiple of the tile, D = 64, MHA
    (4, 1, 16, 2, 128, 300, 1, 700, True, 2),        # a single token: the decode problem through the prefill kernel
    (2, 300, 6, 2, 128, 300, 300, 1000, True, 3),    # three query blocks, odd group size
    (2, 64, 8, 1, 64, 200, 64, 1100, False, 4),      # non-causal: every query sees the whole context
    (2, 256, 4, 2, 128, 200, 40, 256, True, 5),      # contexts shorter than the chunk: rows that see no key
]


@pytest.mark.parametrize("s_n,t_n,h,hkv,d,pool,lo,hi,causal,seed", CASES)
def test_parity_and_bit_identity_with_the_contiguous_entry(s_n, t_n, h, hkv, d, pool, lo, hi, causal, seed):
    dev = torch.device("cuda:0")
    _q1, kp, vp, bt, cl = make_paged_inputs(s_n, h, hkv, d, 16, pool, lo, hi, seed)
    q = torch.randn((s_n, t_n, h, d), generator=torch.Generator().manual_seed(100 + seed)).to(torch.bfloat16)
    o = torch.full((s_n, t_n, h, d), float("nan"), dtype=torch.bfloat16, device=dev)
    l = torch.full((s_n, h, 1, t_n), float("nan"), dtype=torch.float32, device=dev)
    hk.attn_fwd_paged(q.to(dev), kp.to(dev), vp.to(dev), bt.to(dev), cl.to(dev), causal=causal, out=o, lse=l)
    assert _native.device_status(0) == 0
    k, v = gather(kp, vp, bt, int(cl.max()))
    o_ref, l_ref = attn_fwd_oracle(q, k, v, causal, kv_lens=cl)
    assert not torch.isnan(o.float()).any() and not torch.isnan(l).any()
    assert float((o.float().cpu() - o_ref.float()).abs().max()) <= TOL_O
    finite = torch.isfinite(l_ref)
    assert torch.equal(torch.isfinite(l.cpu()), finite)
    assert float((l.cpu() - l_ref)[finite].abs().max()) <= TOL_L
    # the same kernel on the gathered tensors gives the same bits (the gather pads to the table's capacity the way the
    # paged entry sees it)
    cap = bt.shape[1] * 16
    kc, vc = gather(kp, vp, bt, cap)
    o2, l2 = hk.attn_fwd(q.to(dev), kc.to(dev), vc.to(dev), causal=causal, kv_lens=cl.to(dev))
    assert torch.equal(o, o2) and torch.equal(l, l2)


def test_single_token_equals_the_decode_kernel():
    """T = 1, causal: the paged decode problem. The two kernels share nothing but the math."""
    dev = torch.device("cuda:0")
    q, kp, vp, bt, cl = make_paged_inputs(5, 16, 2, 128, 16, 600, 1, 1800, seed=7)
    qd, kpd, vpd, btd, cld = (t.to(dev) for t in (q, kp, vp, bt, cl))
    o_p, l_p = hk.attn_fwd_paged(qd, kpd, vpd, btd, cld, causal=True)
    o_d, l_d = hk.paged_decode(qd, kpd, vpd, btd, cld)
    assert _native.device_status(0) == 0
    assert float((o_p.float() - o_d.float()).abs().max()) <= 1e-2
    assert float((l_p[:, :, 0, 0] - l_d[:, :, 0, 0]).abs().max()) <= 1e-4


def test_append_then_prefill_chunk_equals_rows_of_a_full_causal_forward():
    """The serving sequence: append a chunk's K / V to the cache, then attend. The chunk's rows equal the last T rows
    of a causal forward over the whole sequence."""
    dev = torch.device("cuda:0")
    n, t_n, h, hkv, d = 700, 180, 8, 2, 128
    gen = torch.Generator().manual_seed(11)
    q = torch.randn((1, n, h, d), generator=gen).to(torch.bfloat16).to(dev)
    k = torch.randn((1, n, hkv, d), generator=gen).to(torch.bfloat16).to(dev)
    v = torch.randn((1, n, hkv, d), generator=gen).to(torch.bfloat16).to(dev)
    o_full, l_full = hk.attn_fwd(q, k, v, causal=True)
    max_pages = (n + 15) // 16
    pool = max_pages + 5
    bt = torch.randperm(pool, generator=gen)[:max_pages].to(torch.int32).view(1, max_pages).to(dev)
    kp = torch.zeros((pool, 16, hkv, d), dtype=torch.bfloat16, device=dev)
    vp = torch.zeros_like(kp)
    zero = torch.zeros(1, dtype=torch.int32, device=dev)
    hk.paged_kv_append(k[:, : n - t_n].contiguous(), v[:, : n - t_n].contiguous(), kp, vp, bt, zero)      # the prefix
    hk.paged_kv_append(k[:, n - t_n:].contiguous(), v[:, n - t_n:].contiguous(), kp, vp, bt, zero + (n - t_n))  # the chunk
    o_c, l_c = hk.attn_fwd_paged(q[:, n - t_n:].contiguous(), kp, vp, bt, torch.full((1,), n, dtype=torch.int32, device=dev))
    assert _native.device_status(0) == 0
    assert float((o_c.float() - o_full[:, n - t_n:].float()).abs().max()) <= 8e-3
    assert float((l_c - l_full[:, :, :, n - t_n:]).abs().max()) <= 1e-4


def test_bad_page_id_is_reported_not_dereferenced():
    dev = torch.device("cuda:0")
    q1, kp, vp, bt, cl = make_paged_inputs(2, 8, 2, 128, 16, 200, 300, 600, seed=9)
    q = torch.randn((2, 64, 8, 128), generator=torch.Generator().manual_seed(9)).to(torch.bfloat16)
    bad = bt.clone()
    bad[1, 3] = kp.shape[0] + 7
    hk.attn_fwd_paged(q.to(dev), kp.to(dev), vp.to(dev), bad.to(dev), cl.to(dev))
    assert _native.device_status(0) == _native.HK_EBADPAGE
    o, l = hk.attn_fwd_paged(q.to(dev), kp.to(dev), vp.to(dev), bt.to(dev), cl.to(dev))
    assert _native.device_status(0) == 0 and torch.isfinite(o.float()).all()
