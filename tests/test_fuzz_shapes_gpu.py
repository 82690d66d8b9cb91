"""Seeded random shapes through the forward and the backward on the GPU against the oracle: odd head counts, group sizes,
lengths that are and are not multiples of the tile, both head dimensions, causal or not, with and without key lengths.
The persistent kernels deal work items to CTAs in rounds, so shapes with few, many and uneven numbers of items all
exercise different paths of the item schedule and of the ring and barrier bookkeeping."""
import random

import pytest
import torch

import hipkittens_b200 as hk
from hipkittens_b200 import _native
from hipkittens_b200.synthetic import make_prefill_inputs
from oracle.attn_oracle import attn_bwd_oracle, attn_fwd_oracle

pytestmark = pytest.mark.gpu


def _cases(n_cases=28, seed=2024):
    rng = random.Random(seed)
    out = []
    for i in range(n_cases):
        d = rng.choice([64, 128])
        hkv = rng.choice([1, 2, 3, 4])
        g = rng.choice([1, 2, 3, 4, 8])
        b = rng.randint(1, 4)
        n = rng.choice([rng.randint(1, 1100), 128 * rng.randint(1, 9)])
        causal = rng.random() < 0.5
        lens = None
        if not causal and rng.random() < 0.4:
            lens = [rng.randint(1, n) for _ in range(b)]
        out.append((i, b, n, hkv * g, hkv, d, causal, lens))
    return out


@pytest.mark.parametrize("i,b,n,h,hkv,d,causal,lens", _cases(), ids=lambda v: str(v) if not isinstance(v, list) else "lens")
def test_random_shape(i, b, n, h, hkv, d, causal, lens):
    dev = torch.device("cuda:0")
    q, k, v = make_prefill_inputs(b, n, h, hkv, d, seed=500 + i)
    d_o = make_prefill_inputs(b, n, h, hkv, d, seed=900 + i)[0]
    kv_lens = torch.tensor(lens, dtype=torch.int32) if lens is not None else None
    kv_dev = kv_lens.to(dev) if kv_lens is not None else None
    qd, kd, vd, dod = (t.to(dev) for t in (q, k, v, d_o))
    o, lse = hk.attn_fwd(qd, kd, vd, causal=causal, kv_lens=kv_dev)
    delta = hk.attn_bwd_prep(o, dod)
    dq, dk, dv = hk.attn_bwd(qd, kd, vd, dod, lse, delta, causal=causal, kv_lens=kv_dev)
    assert _native.device_status(0) == 0
    o_ref, l_ref = attn_fwd_oracle(q, k, v, causal, kv_lens=kv_lens)
    assert float((o.float().cpu() - o_ref.float()).abs().max()) <= 2e-2
    assert float((lse.cpu() - l_ref).abs().max()) <= 1e-3
    rq, rk, rv, _ = attn_bwd_oracle(q, k, v, d_o, causal=causal, kv_lens=kv_lens)
    for name, got, ref in (("dq", dq, rq), ("dk", dk, rk), ("dv", dv, rv)):
        diff = (got.float().cpu() - ref).abs()
        assert not torch.isnan(diff).any(), name
        tol = max(2e-2, 1e-2 * float(ref.abs().max())) + 1e-2 * ref.abs()
        assert bool((diff <= tol).all()), f"{name}: max|diff| = {float(diff.max())}"


def _cross_cases(n_cases=24, seed=4048):
    """Random query and key lengths, with and without key lengths, causal or not: offsets kv_len - Nq of either sign and
    not a multiple of the tile, query blocks and rows that see no key, key blocks nobody sees."""
    rng = random.Random(seed)
    out = []
    for i in range(n_cases):
        d = rng.choice([64, 128])
        hkv = rng.choice([1, 2, 3])
        g = rng.choice([1, 2, 3, 4])
        b = rng.randint(1, 3)
        nq = rng.choice([rng.randint(1, 700), 128 * rng.randint(1, 5)])
        nk = rng.choice([rng.randint(1, 900), 128 * rng.randint(1, 7)])
        causal = rng.random() < 0.65
        lens = [rng.randint(1, nk) for _ in range(b)] if rng.random() < 0.5 else None
        out.append((i, b, nq, nk, hkv * g, hkv, d, causal, lens))
    return out


@pytest.mark.parametrize("i,b,nq,nk,h,hkv,d,causal,lens", _cross_cases(),
                         ids=lambda v: str(v) if not isinstance(v, list) else "lens")
def test_random_unequal_lengths(i, b, nq, nk, h, hkv, d, causal, lens):
    dev = torch.device("cuda:0")
    gen = torch.Generator().manual_seed(7000 + i)
    q = torch.randn((b, nq, h, d), generator=gen).to(torch.bfloat16)
    k = torch.randn((b, nk, hkv, d), generator=gen).to(torch.bfloat16)
    v = torch.randn((b, nk, hkv, d), generator=gen).to(torch.bfloat16)
    d_o = torch.randn((b, nq, h, d), generator=gen).to(torch.bfloat16)
    kv_lens = torch.tensor(lens, dtype=torch.int32) if lens is not None else None
    kv_dev = kv_lens.to(dev) if kv_lens is not None else None
    qd, kd, vd, dod = (t.to(dev) for t in (q, k, v, d_o))
    o = torch.full(q.shape, float("nan"), dtype=torch.bfloat16, device=dev)
    lse = torch.full((b, h, 1, nq), float("nan"), dtype=torch.float32, device=dev)
    hk.attn_fwd(qd, kd, vd, causal=causal, kv_lens=kv_dev, out=o, lse=lse)
    delta = hk.attn_bwd_prep(o, dod)
    dq = torch.full(q.shape, float("nan"), dtype=torch.bfloat16, device=dev)
    dk = torch.full(k.shape, float("nan"), dtype=torch.bfloat16, device=dev)
    dv = torch.full(v.shape, float("nan"), dtype=torch.bfloat16, device=dev)
    hk.attn_bwd(qd, kd, vd, dod, lse, delta, causal=causal, kv_lens=kv_dev, dq=dq, dk=dk, dv=dv)
    assert _native.device_status(0) == 0
    o_ref, l_ref = attn_fwd_oracle(q, k, v, causal, kv_lens=kv_lens)
    assert not torch.isnan(o.float()).any() and not torch.isnan(lse).any()
    assert float((o.float().cpu() - o_ref.float()).abs().max()) <= 2e-2
    finite = torch.isfinite(l_ref)
    assert torch.equal(torch.isfinite(lse.cpu()), finite)
    if bool(finite.any()):
        assert float((lse.cpu() - l_ref)[finite].abs().max()) <= 1e-3
    rq, rk, rv, _ = attn_bwd_oracle(q, k, v, d_o, causal=causal, kv_lens=kv_lens)
    for name, got, ref in (("dq", dq, rq), ("dk", dk, rk), ("dv", dv, rv)):
        diff = (got.float().cpu() - ref).abs()
        assert not torch.isnan(diff).any(), name
        tol = max(2e-2, 1e-2 * float(ref.abs().max())) + 1e-2 * ref.abs()
        assert bool((diff <= tol).all()), f"{name}: max|diff| = {float(diff.max())}"
