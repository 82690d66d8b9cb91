"""Many seeded random shapes through the forward and the backward, checked on the GPU against an fp32 restatement of
the reference's math path (training/llama/llama/models/attentions/base.py:95-131: scores, key-padding mask, causal
mask aligned to the last query and the last kept key, softmax, P V) written with torch on the device and differentiated
by autograd. The CPU oracle is the checker of record and takes seconds per case; this restatement is first pinned to
it on a few shapes and then used for volume: query and key lengths that are and are not multiples of the tile and
differ from each other, group sizes 1 to 8, both head dimensions, causal or not, per-batch key lengths, rows and whole
query blocks without a visible key. Work lists of a few items up to several rounds of the persistent kernels come out
of these shapes, and causal key-block counts odd and even (the causal dK/dV kernel deals key blocks in pairs)."""
import random

import pytest
import torch

import hipkittens_b200 as hk
from hipkittens_b200 import _native
from oracle.attn_oracle import attn_bwd_oracle, attn_fwd_oracle

pytestmark = pytest.mark.gpu


def device_restatement(q, k, v, d_o, causal, lens):
    q32, k32, v32 = (t.float().detach().requires_grad_(True) for t in (q, k, v))
    b, nq, h, d = q.shape
    nk, hkv = k.shape[1], k.shape[2]
    g = h // hkv
    kk, vv = k32.repeat_interleave(g, dim=2), v32.repeat_interleave(g, dim=2)
    s = torch.einsum("bqhd,bkhd->bhqk", q32, kk) / d ** 0.5
    kvl = torch.tensor(lens if lens is not None else [nk] * b, device=q.device)[:, None, None, None]
    kidx = torch.arange(nk, device=q.device)[None, None, None, :]
    mask = kidx >= kvl
    if causal:
        qidx = torch.arange(nq, device=q.device)[None, None, :, None]
        mask = mask | (kidx > qidx + (kvl - nq))
    s = s.masked_fill(mask, float("-inf"))
    l = torch.logsumexp(s, dim=-1)
    seen = torch.isfinite(l)
    p = torch.exp(s - torch.where(seen, l, torch.zeros_like(l))[..., None])
    p = torch.where(seen[..., None], p, torch.zeros_like(p))  # a row without keys: O = 0, zero gradients
    o = torch.einsum("bhqk,bkhd->bqhd", p, vv)
    o.backward(d_o.float())
    return o.detach(), l.detach(), q32.grad, k32.grad, v32.grad


def run_case(seed, b, nq, nk, h, hkv, d, causal, lens):
    gen = torch.Generator(device="cuda").manual_seed(seed)
    q = torch.randn((b, nq, h, d), generator=gen, device="cuda").bfloat16()
    k = torch.randn((b, nk, hkv, d), generator=gen, device="cuda").bfloat16()
    v = torch.randn((b, nk, hkv, d), generator=gen, device="cuda").bfloat16()
    d_o = torch.randn((b, nq, h, d), generator=gen, device="cuda").bfloat16()
    kvd = torch.tensor(lens, dtype=torch.int32, device="cuda") if lens is not None else None
    o = torch.full_like(q, float("nan"))
    lse = torch.full((b, h, 1, nq), float("nan"), dtype=torch.float32, device="cuda")
    hk.attn_fwd(q, k, v, causal=causal, kv_lens=kvd, out=o, lse=lse)
    delta = hk.attn_bwd_prep(o, d_o)
    dq, dk, dv = (torch.full_like(t, float("nan")) for t in (q, k, v))
    hk.attn_bwd(q, k, v, d_o, lse, delta, causal=causal, kv_lens=kvd, dq=dq, dk=dk, dv=dv)
    assert _native.device_status(0) == 0
    return (q, k, v, d_o), (o, lse, dq, dk, dv)


def check(case, got, ref):
    o, lse, dq, dk, dv = got
    ro, rl, rq, rk, rv = ref
    assert not torch.isnan(o.float()).any(), case
    assert float((o.float() - ro).abs().max()) <= 2e-2, case
    seen = torch.isfinite(rl)
    assert torch.equal(torch.isfinite(lse[:, :, 0]), seen), case
    if bool(seen.any()):
        assert float((lse[:, :, 0][seen] - rl[seen]).abs().max()) <= 1e-3, case
    for name, a, r in (("dq", dq, rq), ("dk", dk, rk), ("dv", dv, rv)):
        diff = (a.float() - r).abs()
        assert not torch.isnan(diff).any(), (name, case)
        tol = max(2e-2, 1e-2 * float(r.abs().max())) + 1e-2 * r.abs()
        assert bool((diff <= tol).all()), (name, float(diff.max()), case)


def test_device_restatement_agrees_with_the_oracle():
    for seed, (b, nq, nk, h, hkv, d, causal, lens) in enumerate([(2, 200, 200, 4, 2, 64, True, None),
                                                                 (1, 130, 300, 6, 2, 128, True, [170]),
                                                                 (2, 256, 256, 2, 2, 128, False, [256, 100])]):
        (q, k, v, d_o), _ = run_case(50 + seed, b, nq, nk, h, hkv, d, causal, lens)
        ro, rl, rq, rk, rv = device_restatement(q, k, v, d_o, causal, lens)
        kvl = torch.tensor(lens, dtype=torch.int32) if lens is not None else None
        oo, ol = attn_fwd_oracle(q.cpu(), k.cpu(), v.cpu(), causal, kv_lens=kvl)
        oq, ok_, ov, _ = attn_bwd_oracle(q.cpu(), k.cpu(), v.cpu(), d_o.cpu(), causal=causal, kv_lens=kvl)
        assert float((ro.cpu() - oo.float()).abs().max()) <= 1e-2  # the oracle rounds O to bf16 (half an ulp below 4)
        seen = torch.isfinite(ol[:, :, 0])
        assert float((rl.cpu()[seen] - ol[:, :, 0][seen]).abs().max()) <= 1e-4
        for a, r in ((rq, oq), (rk, ok_), (rv, ov)):
            assert float((a.cpu() - r).abs().max()) <= 2e-2 * max(1.0, float(r.abs().max()))


@pytest.mark.parametrize("seed", [11, 12, 13])
def test_random_shapes_against_device_restatement(seed):
    rng = random.Random(seed)
    for i in range(60):
        d = rng.choice([64, 128])
        hkv = rng.choice([1, 2, 3, 4])
        g = rng.choice([1, 2, 3, 4, 8])
        b = rng.randint(1, 4)
        nq = rng.choice([rng.randint(1, 900), 128 * rng.randint(1, 12)])
        nk = nq if rng.random() < 0.5 else rng.choice([rng.randint(1, 1200), 128 * rng.randint(1, 12)])
        causal = rng.random() < 0.6
        lens = [rng.randint(1, nk) for _ in range(b)] if rng.random() < 0.4 else None
        case = dict(seed=seed, i=i, b=b, nq=nq, nk=nk, h=hkv * g, hkv=hkv, d=d, causal=causal, lens=lens)
        inputs, got = run_case(1000 * seed + i, b, nq, nk, hkv * g, hkv, d, causal, lens)
        check(case, got, device_restatement(*inputs, causal, lens))
