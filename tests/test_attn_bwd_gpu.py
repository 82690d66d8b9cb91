"""GPU parity of the attention backward (delta prep, dK/dV kernel, dQ kernel, dQ shuffle) against the CPU
oracle and against gradients of the reference's own PyTorch module, through the C ABI, the reference's
Python entry points and the autograd function.

Tolerance (written here, floating point): every gradient element within max(2e-2, 1e-2 * max|ref|) + 1e-2 * |ref|
of the fp32 oracle (outputs are bf16: half an ulp is 2^-9 relative; P and dS are rounded to bf16 before the last
products, and a dK or dV element sums thousands of such terms, so its absolute error scales with the size of the
tensor, not of the element), and a relative L2 error of at most 5e-3 per tensor."""
import glob
import os

import numpy as np
import pytest
import torch

import hipkittens_b200 as hk
from hipkittens_b200 import _native
from hipkittens_b200.synthetic import make_prefill_inputs
from oracle.attn_oracle import attn_bwd_oracle

pytestmark = pytest.mark.gpu
ATOL, RTOL, L2TOL = 2e-2, 1e-2, 5e-3
GOLDEN = [p for p in sorted(glob.glob(os.path.join(os.path.dirname(__file__), "golden", "case_*.npz")))
          if "dq_ref_fp32" in np.load(p).files]


@pytest.fixture(scope="module")
def dev():
    assert torch.cuda.is_available(), "these tests need a B200"
    return torch.device("cuda:0")


def make_do(shape, seed):
    return torch.randn(shape, generator=torch.Generator().manual_seed(seed)).to(torch.bfloat16)


def run_bwd(q, k, v, d_o, causal, dev, scale=None, dq_layout=hk.HK_DQ_BNHD, kv_lens=None):
    """Forward + prep + backward on the GPU; gradient buffers are poisoned with NaN first."""
    qd, kd, vd, dod = (t.to(dev) for t in (q, k, v, d_o))
    o, lse = hk.attn_fwd(qd, kd, vd, causal=causal, softmax_scale=scale, kv_lens=kv_lens)
    delta = hk.attn_bwd_prep(o, dod)
    b, n, h, d = q.shape
    dq_shape = (b, n, h, d) if dq_layout == hk.HK_DQ_BNHD else (b, h, n, d)
    dq = torch.full(dq_shape, float("nan"), dtype=torch.bfloat16, device=dev)
    dk = torch.full(k.shape, float("nan"), dtype=torch.bfloat16, device=dev)
    dv = torch.full(v.shape, float("nan"), dtype=torch.bfloat16, device=dev)
    hk.attn_bwd(qd, kd, vd, dod, lse, delta, causal=causal, softmax_scale=scale, dq=dq, dk=dk, dv=dv,
                dq_layout=dq_layout, kv_lens=kv_lens)
    assert _native.device_status(0) == 0
    return dq.cpu(), dk.cpu(), dv.cpu(), delta.cpu(), o.cpu()


def assert_grad_parity(got, ref, name):
    got = got.float()
    assert not torch.isnan(got).any(), f"{name} has unwritten elements"
    diff = (got - ref).abs()
    bad = diff > (max(ATOL, RTOL * float(ref.abs().max())) + RTOL * ref.abs())
    assert not bool(bad.any()), f"{name}: {int(bad.sum())} elements out of tolerance, max|diff| = {float(diff.max())}"
    if float(ref.abs().max()) > 1e-3:  # a single key gives P = 1 and dq = dk = 0 up to rounding: no relative figure then
        l2 = float(diff.pow(2).sum().sqrt() / ref.pow(2).sum().sqrt())
        assert l2 <= L2TOL, f"{name}: relative L2 error {l2}"


def _gpu_fp32_unit_grads(q, k, v, d_o, causal):
    """fp32 autograd restatement on the GPU of one (batch, kv-head) unit: q, d_o [N,G,D], k, v [N,D]. A checker for
    full-size shapes (the CPU oracle on a whole tensor would take minutes); it shares nothing with the kernels or
    with the oracle's hand-written derivative."""
    import math

    n = q.shape[0]
    qf, kf, vf = (t.float().requires_grad_(True) for t in (q, k, v))
    s = torch.einsum("tgd,sd->gts", qf, kf) / math.sqrt(q.shape[-1])
    if causal:
        s = s.masked_fill(torch.triu(torch.ones(n, n, dtype=torch.bool, device=q.device), 1), float("-inf"))
    o = torch.einsum("gts,sd->tgd", torch.softmax(s, -1), vf)
    o.backward(d_o.float())
    return qf.grad, kf.grad, vf.grad


def _assert_every_unit_matches_fp32(q, k, v, d_o, dq, dk, dv, causal):
    """Every (batch, kv-head) unit of a full-size backward against the fp32 restatement above, with the build's
    gradient tolerance per unit."""
    b, n, h, d = q.shape
    hkv = k.shape[2]
    g = h // hkv
    for bi in range(b):
        for kh in range(hkv):
            hs = slice(kh * g, (kh + 1) * g)
            rq, rk, rv = _gpu_fp32_unit_grads(q[bi, :, hs], k[bi, :, kh], v[bi, :, kh], d_o[bi, :, hs], causal)
            assert_grad_parity(dq[bi, :, hs], rq, f"dq unit ({bi},{kh})")
            assert_grad_parity(dk[bi, :, kh], rk, f"dk unit ({bi},{kh})")
            assert_grad_parity(dv[bi, :, kh], rv, f"dv unit ({bi},{kh})")
            del rq, rk, rv


SHAPES = [
    # B, N, H, H_KV, D, causal
    (1, 256, 8, 2, 64, False),     # BASELINE config 1
    (1, 128, 1, 1, 128, False),    # one tile, one iteration per kernel
    (1, 128, 1, 1, 128, True),     # a single diagonal tile
    (2, 384, 4, 2, 128, True),     # odd block count, GQA
    (1, 512, 2, 2, 128, True),     # MHA causal
    (1, 384, 3, 3, 64, False),     # odd head count
    (2, 256, 8, 8, 64, True),      # MHA, D = 64, causal
    (1, 1024, 16, 2, 128, False),  # group of 8
    (3, 256, 12, 4, 64, False),    # group of 3
    (1, 1152, 4, 1, 128, True),    # group of 4, nine blocks: the K ring wraps several times in one item
    # sequence lengths that are not a multiple of the 128-row tile (the reference cannot run these)
    (2, 200, 4, 2, 128, False),
    (1, 333, 8, 2, 64, True),
    (2, 129, 2, 2, 128, True),
    (1, 1000, 8, 1, 128, False),
    (1, 1, 2, 1, 64, False),       # a single token
    (1, 77, 3, 3, 64, True),
    (1, 515, 2, 1, 128, True),     # N % 4 != 0: statistics rows are not 16-byte aligned
]


@pytest.mark.parametrize("b,n,h,hkv,d,causal", SHAPES)
def test_parity_against_oracle(dev, b, n, h, hkv, d, causal):
    q, k, v = make_prefill_inputs(b, n, h, hkv, d, seed=b * 1000 + n + h)
    d_o = make_do((b, n, h, d), seed=7 * n + h)
    dq, dk, dv, delta, _o = run_bwd(q, k, v, d_o, causal, dev)
    rq, rk, rv, rdelta = attn_bwd_oracle(q, k, v, d_o, causal=causal)
    # delta uses the bf16-rounded O of the forward kernel (half an ulp of O per term)
    assert bool(((delta - rdelta).abs() <= ATOL + RTOL * rdelta.abs()).all())
    assert_grad_parity(dq, rq, "dq")
    assert_grad_parity(dk, rk, "dk")
    assert_grad_parity(dv, rv, "dv")


@pytest.mark.parametrize("path", GOLDEN, ids=[os.path.basename(p) for p in GOLDEN])
def test_parity_against_reference_module_gradients(dev, path):
    """Directly against the committed autograd gradients of the reference's CrossAttention (fp32 run)."""
    z = np.load(path)
    b, n, h, hkv, d, causal, _ = [int(x) for x in z["shape"]]
    bits = lambda a: torch.from_numpy(a.view(np.int16).copy()).view(torch.bfloat16)  # noqa: E731
    q, k, v, d_o = bits(z["q"]), bits(z["k"]), bits(z["v"]), bits(z["d_o"])
    kv_lens = torch.from_numpy(z["kv_lens"]).to(dev) if "kv_lens" in z.files else None
    dq, dk, dv, _delta, _o = run_bwd(q, k, v, d_o, bool(causal), dev, kv_lens=kv_lens)
    assert_grad_parity(dq, torch.from_numpy(z["dq_ref_fp32"]), "dq")
    assert_grad_parity(dk, torch.from_numpy(z["dk_ref_fp32"]), "dk")
    assert_grad_parity(dv, torch.from_numpy(z["dv_ref_fp32"]), "dv")


def test_delta_prep_is_exact_rowsum(dev):
    """delta = rowsum(O * dO) in fp32 of the bf16 values, for both head dimensions."""
    for d in (64, 128):
        gen = torch.Generator().manual_seed(40 + d)
        o = torch.randn((2, 200, 6, d), generator=gen).to(torch.bfloat16)
        d_o = torch.randn((2, 200, 6, d), generator=gen).to(torch.bfloat16)
        delta = hk.attn_bwd_prep(o.to(dev), d_o.to(dev)).cpu()
        ref = (o.double() * d_o.double()).sum(-1).permute(0, 2, 1).unsqueeze(2)
        assert delta.shape == (2, 6, 1, 200)
        assert float((delta.double() - ref).abs().max()) <= 1e-5 * float(ref.abs().max())


def test_runs_are_bit_identical_and_layouts_agree(dev):
    """No atomics anywhere: two runs give the same bits. The pre-shuffle [B,H,N,D] layout followed by the
    shuffle kernel gives the same dQ as writing [B,N,H,D] directly."""
    q, k, v = make_prefill_inputs(2, 512, 8, 2, 128, seed=41)
    d_o = make_do((2, 512, 8, 128), seed=42)
    a = run_bwd(q, k, v, d_o, True, dev)
    b = run_bwd(q, k, v, d_o, True, dev)
    for x, y in zip(a[:3], b[:3]):
        assert torch.equal(x, y)
    dq_bhnd = run_bwd(q, k, v, d_o, True, dev, dq_layout=hk.HK_DQ_BHND)[0]
    assert dq_bhnd.shape == (2, 8, 512, 128)
    assert torch.equal(dq_bhnd.permute(0, 2, 1, 3), a[0])
    assert torch.equal(hk.dq_shuffle(dq_bhnd.to(dev)).cpu(), a[0])


def test_through_reference_entry_points(dev):
    """The reference's three calls, in its order and with its argument lists
    (training/llama/llama/models/attentions/hipkittens.py:96-112, kernels/attn/gqa_backwards/test_python.py:242-263)."""
    q, k, v = make_prefill_inputs(2, 256, 8, 2, 128, seed=43)
    d_o = make_do((2, 256, 8, 128), seed=44)
    for causal in (False, True):
        Q, K, V, dO = (t.to(dev) for t in (q, k, v, d_o))
        O = torch.zeros(2, 256, 8, 128, dtype=torch.bfloat16, device=dev)
        L = torch.zeros(2, 8, 1, 256, dtype=torch.float32, device=dev)
        hk.load_tk_kernel_fwd(causal).dispatch_fwd(Q, K, V, O, L)
        tk_kernel_bkwd = hk.load_tk_kernel_bkwd(causal)
        tk_kernel_bkwd_prep = hk.load_tk_kernel_bkwd_prep(causal)
        assert tk_kernel_bkwd.default_causal == causal
        dQ_in = torch.zeros((2, 8, 256, 128), dtype=torch.bfloat16, device=dev)
        dQ = torch.empty((2, 256, 8, 128), dtype=torch.bfloat16, device=dev)
        dK = torch.empty((2, 256, 2, 128), dtype=torch.bfloat16, device=dev)
        dV = torch.empty((2, 256, 2, 128), dtype=torch.bfloat16, device=dev)
        delta = torch.empty((2, 8, 1, 256), dtype=torch.float32, device=dev)
        tk_kernel_bkwd_prep.dispatch_prep(O, dO, delta)
        tk_kernel_bkwd.dispatch_bwd_combined(Q, K, V, dO, dQ_in, dK, dV, L, delta)
        tk_kernel_bkwd_prep.dispatch_dq_shuffle(dQ_in, dQ)
        rq, rk, rv, _ = attn_bwd_oracle(q, k, v, d_o, causal=causal)
        assert_grad_parity(dQ.cpu(), rq, "dq")
        assert_grad_parity(dK.cpu(), rk, "dk")
        assert_grad_parity(dV.cpu(), rv, "dv")
        # the reference's argument checks, with its messages (include/pyutils/pyutils.cuh:22,25,33)
        with pytest.raises(RuntimeError, match="Tensor must be on CUDA device"):
            tk_kernel_bkwd_prep.dispatch_prep(O.cpu(), dO, delta)
        with pytest.raises(RuntimeError, match="Tensor must be contiguous"):
            tk_kernel_bkwd.dispatch_bwd_combined(Q, K, V, dO, dQ_in.transpose(1, 2), dK, dV, L, delta)
        with pytest.raises(RuntimeError, match="Expected a torch.Tensor"):
            tk_kernel_bkwd_prep.dispatch_dq_shuffle(None, dQ)
        with pytest.raises(RuntimeError, match="pre-shuffle"):
            tk_kernel_bkwd.dispatch_bwd_combined(Q, K, V, dO, dQ, dK, dV, L, delta)


def test_autograd_function_backward(dev):
    """loss.backward() through the modules the training code uses (hipkittens.py:122-202)."""
    from hipkittens_b200.attention import HipCrossAttention, HipSelfAttention

    q, k, v = make_prefill_inputs(1, 256, 8, 2, 64, seed=45)
    d_o = make_do((1, 256, 8, 64), seed=46)
    qd = q.to(dev).requires_grad_(True)
    kvd = torch.stack([k, v], dim=2).to(dev).requires_grad_(True)
    out = HipCrossAttention(causal=True)(qd, kvd)
    out.backward(d_o.to(dev))
    rq, rk, rv, _ = attn_bwd_oracle(q, k, v, d_o, causal=True)
    assert qd.grad.dtype == torch.bfloat16 and kvd.grad.shape == kvd.shape
    assert_grad_parity(qd.grad.cpu(), rq, "dq")
    assert_grad_parity(kvd.grad[:, :, 0].cpu(), rk, "dk")
    assert_grad_parity(kvd.grad[:, :, 1].cpu(), rv, "dv")
    # self-attention on a packed projection: the forward reads strided views, the backward makes them contiguous
    q, k, v = make_prefill_inputs(2, 128, 4, 4, 128, seed=47)
    d_o = make_do((2, 128, 4, 128), seed=48)
    qkv = torch.stack([q, k, v], dim=2).to(dev).requires_grad_(True)
    HipSelfAttention(causal=False)(qkv).backward(d_o.to(dev))
    rq, rk, rv, _ = attn_bwd_oracle(q, k, v, d_o, causal=False)
    assert_grad_parity(qkv.grad[:, :, 0].cpu(), rq, "dq")
    assert_grad_parity(qkv.grad[:, :, 1].cpu(), rk, "dk")
    assert_grad_parity(qkv.grad[:, :, 2].cpu(), rv, "dv")


def test_modules_with_key_padding_mask(dev):
    """A right-padded key_padding_mask through the module, forward and backward, against the oracle (the reference's
    PyTorch modules implement the mask, base.py:97-103; its kernel-backed modules ignore it)."""
    from hipkittens_b200.attention import HipCrossAttention
    from oracle.attn_oracle import attn_fwd_oracle

    q, k, v = make_prefill_inputs(3, 256, 4, 2, 64, seed=58)
    d_o = make_do((3, 256, 4, 64), seed=59)
    lens = torch.tensor([256, 100, 129], dtype=torch.int32)
    mask = (torch.arange(256).view(1, 256) < lens.view(3, 1)).to(dev)
    qd = q.to(dev).requires_grad_(True)
    kvd = torch.stack([k, v], dim=2).to(dev).requires_grad_(True)
    out = HipCrossAttention(causal=False)(qd, kvd, key_padding_mask=mask)
    o_ref, _ = attn_fwd_oracle(q, k, v, False, kv_lens=lens)
    assert float((out.detach().float().cpu() - o_ref.float()).abs().max()) <= 2e-2
    out.backward(d_o.to(dev))
    rq, rk, rv, _ = attn_bwd_oracle(q, k, v, d_o, causal=False, kv_lens=lens)
    assert_grad_parity(qd.grad.cpu(), rq, "dq")
    assert_grad_parity(kvd.grad[:, :, 0].cpu(), rk, "dk")
    assert_grad_parity(kvd.grad[:, :, 1].cpu(), rv, "dv")
    holes = mask.clone()
    holes[1, 3] = False
    with pytest.raises(ValueError):
        HipCrossAttention(causal=False)(qd, kvd, key_padding_mask=holes)


def test_custom_softmax_scale(dev):
    q, k, v = make_prefill_inputs(1, 256, 2, 1, 128, seed=49)
    d_o = make_do((1, 256, 2, 128), seed=50)
    dq, dk, dv, _, _ = run_bwd(q, k, v, d_o, False, dev, scale=0.05)
    rq, rk, rv, _ = attn_bwd_oracle(q, k, v, d_o, causal=False, softmax_scale=0.05)
    assert_grad_parity(dq, rq, "dq")
    assert_grad_parity(dk, rk, "dk")
    assert_grad_parity(dv, rv, "dv")


def test_bad_arguments(dev):
    lib = hk.capi()
    assert lib.hk_attn_bwd(None, 64, 64, 64, 64, 64, 64, 64, 64, 1, 128, 2, 1, 128, 0, 0.0, 0, 0, None) == _native.HK_EINVAL
    assert lib.hk_attn_bwd(64, 64, 64, 64, 64, 64, 64, 64, 64, 1, 128, 2, 1, 128, 0, 0.0, 7, 0, None) == _native.HK_EINVAL
    assert lib.hk_attn_dq_shuffle(64, 64, 1, 128, 2, 128, 0, None) == _native.HK_EINVAL  # aliasing buffers
    q, k, v = make_prefill_inputs(1, 128, 2, 1, 128, seed=51)
    with pytest.raises(RuntimeError):
        hk.attn_bwd(q.to(dev), k.to(dev), v.to(dev), q.to(dev), torch.zeros(1, 2, 1, 64, device=dev),
                    torch.zeros(1, 2, 1, 128, device=dev))  # L of the wrong length


def test_key_padding_lengths(dev):
    """Per-batch key lengths (the reference's key_padding_mask): a length inside the first block, one on a block
    boundary, the full length, and one inside a later block; key blocks wholly beyond a length are skipped by both
    kernels and their dK / dV rows come back as exact zeros, whatever the padded keys contain."""
    q, k, v = make_prefill_inputs(4, 512, 8, 2, 128, seed=56)
    d_o = make_do((4, 512, 8, 128), seed=57)
    lens = torch.tensor([512, 5, 256, 300], dtype=torch.int32)
    dq, dk, dv, _, _ = run_bwd(q, k, v, d_o, False, dev, kv_lens=lens.to(dev))
    rq, rk, rv, _ = attn_bwd_oracle(q, k, v, d_o, causal=False, kv_lens=lens)
    assert_grad_parity(dq, rq, "dq")
    assert_grad_parity(dk, rk, "dk")
    assert_grad_parity(dv, rv, "dv")
    k2, v2 = k.clone(), v.clone()
    for b in range(4):
        assert float(dk[b, int(lens[b]):].abs().max() if int(lens[b]) < 512 else 0) == 0.0
        assert float(dv[b, int(lens[b]):].abs().max() if int(lens[b]) < 512 else 0) == 0.0
        k2[b, int(lens[b]):] = 1e4
        v2[b, int(lens[b]):] = -3e4  # finite: a padded key inside a loaded tile still meets p = 0 in the products
    dq2, dk2, dv2, _, _ = run_bwd(q, k2, v2, d_o, False, dev, kv_lens=lens.to(dev))
    assert torch.equal(dq, dq2) and torch.equal(dk, dk2) and torch.equal(dv, dv2)


CROSS = sorted(glob.glob(os.path.join(os.path.dirname(__file__), "golden", "cross_*.npz")))


@pytest.mark.parametrize("path", CROSS, ids=[os.path.basename(p) for p in CROSS])
def test_unequal_lengths_and_causal_padding_against_reference_gradients(dev, path):
    """hk_attn_bwd_cross against gradients autograd produced through the reference's CrossAttention with Sq != Sk
    and with causal + key_padding_mask (base.py:104-116). The fixtures' dO is zero on rows that see no key; dq of
    those rows is zero here and excluded from the comparison with the reference."""
    from test_oracle import load_cross

    z, q, k, v, d_o, kv_lens, causal, valid = load_cross(path)
    dq, dk, dv, _, _ = run_bwd(q, k, v, d_o, causal, dev, kv_lens=kv_lens.to(dev) if kv_lens is not None else None)
    rq = torch.from_numpy(z["dq_ref_fp32"]) * valid.view(*valid.shape, 1, 1)
    assert_grad_parity(dq, rq, "dq")
    assert_grad_parity(dk, torch.from_numpy(z["dk_ref_fp32"]), "dk")
    assert_grad_parity(dv, torch.from_numpy(z["dv_ref_fp32"]), "dv")
    if not bool(valid.all()):
        assert float(dq[~valid].float().abs().max()) == 0.0


CROSS_SHAPES = [
    # B, Nq, Nk, H, H_KV, D, causal, kv_lens
    (2, 128, 1024, 8, 2, 128, True, None),
    (1, 100, 1000, 4, 4, 64, True, None),
    (2, 300, 700, 6, 2, 128, True, [700, 301]),
    (3, 256, 256, 4, 2, 64, True, [256, 129, 1]),
    (1, 520, 130, 2, 1, 128, True, None),
    (2, 1, 777, 8, 1, 128, True, [777, 5]),
    (2, 200, 456, 4, 2, 64, False, [456, 77]),
    (1, 640, 384, 3, 3, 128, False, None),
    (1, 384, 640, 3, 3, 64, True, None),
]


@pytest.mark.parametrize("b,nq,nk,h,hkv,d,causal,lens", CROSS_SHAPES)
def test_unequal_lengths_parity(dev, b, nq, nk, h, hkv, d, causal, lens):
    gen = torch.Generator().manual_seed(4321 + nq + nk)
    q = torch.randn((b, nq, h, d), generator=gen).to(torch.bfloat16)
    k = torch.randn((b, nk, hkv, d), generator=gen).to(torch.bfloat16)
    v = torch.randn((b, nk, hkv, d), generator=gen).to(torch.bfloat16)
    d_o = torch.randn((b, nq, h, d), generator=gen).to(torch.bfloat16)
    kv_lens = torch.tensor(lens, dtype=torch.int32) if lens is not None else None
    dq, dk, dv, _, _ = run_bwd(q, k, v, d_o, causal, dev, kv_lens=kv_lens.to(dev) if kv_lens is not None else None)
    rq, rk, rv, _ = attn_bwd_oracle(q, k, v, d_o, causal=causal, kv_lens=kv_lens)
    assert_grad_parity(dq, rq, "dq")
    assert_grad_parity(dk, rk, "dk")
    assert_grad_parity(dv, rv, "dv")


def test_module_backward_with_causal_key_padding_and_longer_kv(dev):
    """HipCrossAttention(causal=True)(q, kv, key_padding_mask=...) with Sq < Sk through loss.backward(): the call
    inference and padded training make (mha.py:164-168, base.py:104-116)."""
    from hipkittens_b200.attention import HipCrossAttention

    b, sq, sk, h, hkv, d = 2, 96, 320, 4, 2, 128
    gen = torch.Generator().manual_seed(99)
    q = torch.randn((b, sq, h, d), generator=gen).to(torch.bfloat16)
    kv = torch.randn((b, sk, 2, hkv, d), generator=gen).to(torch.bfloat16)
    d_o = torch.randn((b, sq, h, d), generator=gen).to(torch.bfloat16)
    lens = torch.tensor([320, 150], dtype=torch.int32)
    mask = torch.arange(sk).view(1, sk) < lens.view(b, 1)
    qd = q.to(dev).requires_grad_(True)
    kvd = kv.to(dev).requires_grad_(True)
    out = HipCrossAttention(causal=True)(qd, kvd, key_padding_mask=mask.to(dev))
    out.backward(d_o.to(dev))
    o_ref, _ = attn_fwd_oracle_for_bwd(q, kv[:, :, 0], kv[:, :, 1], True, lens)
    assert float((out.detach().float().cpu() - o_ref.float()).abs().max()) <= 2e-2
    rq, rk, rv, _ = attn_bwd_oracle(q, kv[:, :, 0], kv[:, :, 1], d_o, causal=True, kv_lens=lens)
    assert_grad_parity(qd.grad.cpu(), rq, "dq")
    assert_grad_parity(kvd.grad[:, :, 0].cpu(), rk, "dk")
    assert_grad_parity(kvd.grad[:, :, 1].cpu(), rv, "dv")


def attn_fwd_oracle_for_bwd(q, k, v, causal, lens):
    from oracle.attn_oracle import attn_fwd_oracle

    return attn_fwd_oracle(q, k, v, causal, kv_lens=lens)


def test_padded_rows_do_not_leak(dev):
    """N = 200: the second tile has 72 real rows. Poisoning memory around the tensors must not change anything, and
    gradient buffers larger than needed must stay untouched beyond row N."""
    q, k, v = make_prefill_inputs(1, 200, 4, 2, 128, seed=54)
    d_o = make_do((1, 200, 4, 128), seed=55)
    dq, dk, dv, _, _ = run_bwd(q, k, v, d_o, True, dev)
    rq, rk, rv, _ = attn_bwd_oracle(q, k, v, d_o, causal=True)
    assert_grad_parity(dq, rq, "dq")
    assert_grad_parity(dk, rk, "dk")
    assert_grad_parity(dv, rv, "dv")


def test_full_size_identities_config2(dev):
    """BASELINE config 2 (B16 N2048 H64 H_KV8 D128), too large for the oracle as a whole: size-independent
    identities over every (batch, kv head) unit, every unit against an fp32 autograd restatement on the GPU, plus
    oracle parity on one unit.
      <q, dq> == <k, dk> per unit (the output is invariant under q -> a q, k -> k / a);
      sum_s dv[s] == sum over the group's heads and rows of dO (softmax rows sum to one)."""
    b, n, h, hkv, d = 16, 2048, 64, 8, 128
    g = h // hkv
    gen = torch.Generator(device=dev).manual_seed(53)
    q = torch.randn((b, n, h, d), generator=gen, device=dev).to(torch.bfloat16)
    k = torch.randn((b, n, hkv, d), generator=gen, device=dev).to(torch.bfloat16)
    v = torch.randn((b, n, hkv, d), generator=gen, device=dev).to(torch.bfloat16)
    d_o = torch.randn((b, n, h, d), generator=gen, device=dev).to(torch.bfloat16)
    o, lse = hk.attn_fwd(q, k, v, causal=False)
    delta = hk.attn_bwd_prep(o, d_o)
    dq, dk, dv = hk.attn_bwd(q, k, v, d_o, lse, delta, causal=False)
    assert _native.device_status(0) == 0
    assert not torch.isnan(dq.float()).any() and not torch.isnan(dk.float()).any() and not torch.isnan(dv.float()).any()
    qdq = (q.float() * dq.float()).view(b, n, hkv, g * d).sum((1, 3))            # [B, H_KV]
    kdk = (k.float() * dk.float()).sum((1, 3))
    scale_ref = (q.float() * dq.float()).abs().view(b, n, hkv, g * d).sum((1, 3))
    assert float(((qdq - kdk).abs() / scale_ref).max()) <= 1e-3
    dv_sum = dv.float().sum(1)                                                   # [B, H_KV, D]
    do_sum = d_o.float().view(b, n, hkv, g, d).sum((1, 3))
    assert float((dv_sum - do_sum).abs().max()) <= 2e-2 * float(do_sum.abs().max())
    # every unit against the fp32 autograd restatement evaluated on the GPU
    _assert_every_unit_matches_fp32(q, k, v, d_o, dq, dk, dv, causal=False)
    # one unit against the oracle
    bi, kh = 5, 3
    hs = slice(kh * g, (kh + 1) * g)
    rq, rk, rv, _ = attn_bwd_oracle(q[bi:bi + 1, :, hs].cpu(), k[bi:bi + 1, :, kh:kh + 1].cpu(),
                                    v[bi:bi + 1, :, kh:kh + 1].cpu(), d_o[bi:bi + 1, :, hs].cpu(), causal=False)
    # gradients at this size are small (~1e-2): compare with a tolerance scaled to the tensor
    for name, got, ref in (("dq", dq[bi:bi + 1, :, hs], rq), ("dk", dk[bi:bi + 1, :, kh:kh + 1], rk),
                           ("dv", dv[bi:bi + 1, :, kh:kh + 1], rv)):
        diff = (got.float().cpu() - ref).abs()
        assert float(diff.max()) <= 2e-2 * float(ref.abs().max()) + 1e-2 * float(ref.abs().max()), name
        assert float(diff.pow(2).sum().sqrt() / ref.pow(2).sum().sqrt()) <= L2TOL, name


def test_full_size_identities_config3_causal(dev):
    """BASELINE config 3 shape (B4 N8192 H64 H_KV8 D128, causal): the same two size-independent identities over every
    (batch, kv head) unit, plus the first rows of one unit against the oracle restricted to the keys they can see."""
    b, n, h, hkv, d = 4, 8192, 64, 8, 128
    g = h // hkv
    gen = torch.Generator(device=dev).manual_seed(61)
    q = torch.randn((b, n, h, d), generator=gen, device=dev).to(torch.bfloat16)
    k = torch.randn((b, n, hkv, d), generator=gen, device=dev).to(torch.bfloat16)
    v = torch.randn((b, n, hkv, d), generator=gen, device=dev).to(torch.bfloat16)
    d_o = torch.randn((b, n, h, d), generator=gen, device=dev).to(torch.bfloat16)
    o, lse = hk.attn_fwd(q, k, v, causal=True)
    delta = hk.attn_bwd_prep(o, d_o)
    dq, dk, dv = hk.attn_bwd(q, k, v, d_o, lse, delta, causal=True)
    assert _native.device_status(0) == 0
    for t in (dq, dk, dv):
        assert not torch.isnan(t.float()).any()
    qdq = (q.float() * dq.float()).view(b, n, hkv, g * d).sum((1, 3))
    kdk = (k.float() * dk.float()).sum((1, 3))
    scale_ref = (q.float() * dq.float()).abs().view(b, n, hkv, g * d).sum((1, 3))
    assert float(((qdq - kdk).abs() / scale_ref).max()) <= 1e-3
    dv_sum = dv.float().sum(1)
    do_sum = d_o.float().view(b, n, hkv, g, d).sum((1, 3))
    assert float((dv_sum - do_sum).abs().max()) <= 2e-2 * float(do_sum.abs().max())
    # every unit against the fp32 autograd restatement evaluated on the GPU
    _assert_every_unit_matches_fp32(q, k, v, d_o, dq, dk, dv, causal=True)
    # causality makes the first 256 query rows independent of everything behind them: dq of those rows equals the dq of
    # the 256-token problem (dk and dv of the first keys also collect from later queries, so only dq is compared)
    bi, kh, m = 2, 5, 256
    hs = slice(kh * g, (kh + 1) * g)
    rq, _, _, _ = attn_bwd_oracle(q[bi:bi + 1, :m, hs].cpu(), k[bi:bi + 1, :m, kh:kh + 1].cpu(),
                                  v[bi:bi + 1, :m, kh:kh + 1].cpu(), d_o[bi:bi + 1, :m, hs].cpu(), causal=True)
    assert_grad_parity(dq[bi:bi + 1, :m, hs].cpu(), rq, "dq (first 256 rows)")
