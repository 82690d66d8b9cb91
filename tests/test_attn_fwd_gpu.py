"""GPU parity of the attention forward against the CPU oracle, through the C ABI and the reference's Python
entry points. Tolerances are the build's: max-abs 2e-2 on O, 1e-3 on L."""
import glob
import math
import os

import numpy as np
import pytest
import torch

import hipkittens_b200 as hk
from hipkittens_b200 import _native
from hipkittens_b200.synthetic import make_prefill_inputs
from oracle.attn_oracle import attn_fwd_oracle, robustness_check

pytestmark = pytest.mark.gpu
TOL_O, TOL_L = 2e-2, 1e-3
GOLDEN = sorted(glob.glob(os.path.join(os.path.dirname(__file__), "golden", "case_*.npz")))


@pytest.fixture(scope="module")
def dev():
    assert torch.cuda.is_available(), "these tests need a B200"
    return torch.device("cuda:0")


def run_fwd(q, k, v, causal, dev, scale=None, kv_lens=None):
    """Poison the outputs with NaN first so rows the kernel failed to write are caught."""
    b, n, h, d = q.shape
    o = torch.full((b, n, h, d), float("nan"), dtype=torch.bfloat16, device=dev)
    l = torch.full((b, h, 1, n), float("nan"), dtype=torch.float32, device=dev)
    hk.attn_fwd(q.to(dev), k.to(dev), v.to(dev), causal=causal, softmax_scale=scale, out=o, lse=l, kv_lens=kv_lens)
    assert _native.device_status(0) == 0
    return o.cpu(), l.cpu()


def assert_parity(o, l, o_ref, l_ref):
    assert not torch.isnan(o.float()).any() and not torch.isnan(l).any()
    eo = float((o.float() - o_ref.float()).abs().max())
    el = float((l - l_ref).abs().max())
    assert eo <= TOL_O, f"max|dO| = {eo}"
    assert el <= TOL_L, f"max|dL| = {el}"


SMALL = [
    # B, N, H, H_KV, D, causal
    (1, 256, 8, 2, 64, False),     # BASELINE config 1
    (1, 128, 2, 1, 128, False),    # one tile per slot
    (1, 128, 1, 1, 128, True),     # a single tile: second slot unused
    (2, 384, 4, 2, 128, True),     # head-paired slots, odd q-block count
    (1, 512, 2, 2, 128, True),     # MHA causal: q-block pairs of unequal length
    (1, 384, 3, 3, 64, False),     # odd group size and odd q-block count
    (2, 256, 8, 8, 64, True),      # MHA, D=64, causal
    (1, 1024, 16, 2, 128, False),  # group of 8
    (3, 256, 12, 4, 64, False),    # group of 3 (q-block pairing under GQA)
    # sequence lengths that are not a multiple of the 128-row tile (the reference cannot run these)
    (2, 200, 4, 2, 128, False),
    (1, 333, 8, 2, 64, True),
    (2, 129, 2, 2, 128, True),
    (1, 1000, 8, 1, 128, False),
    (1, 1, 2, 1, 64, False),       # a single token
    (1, 77, 3, 3, 64, True),
]


@pytest.mark.parametrize("b,n,h,hkv,d,causal", SMALL)
def test_parity_small(dev, b, n, h, hkv, d, causal):
    q, k, v = make_prefill_inputs(b, n, h, hkv, d, seed=b * 1000 + n + h)
    o, l = run_fwd(q, k, v, causal, dev)
    o_ref, l_ref = attn_fwd_oracle(q, k, v, causal)
    assert_parity(o, l, o_ref, l_ref)
    # the reference harness's own statistic: no element beyond 0.001 + 0.05|ref| ... for L; O within a few
    _max_abs, err, numel, _l2, cos = robustness_check(l_ref, l)
    assert err == 0 and cos > 0.99999


@pytest.mark.parametrize("path", GOLDEN, ids=[os.path.basename(p) for p in GOLDEN])
def test_parity_against_reference_module_outputs(dev, path):
    """Directly against the committed outputs of the reference's PyTorch module (fp32 run)."""
    z = np.load(path)
    b, n, h, hkv, d, causal, _ = [int(x) for x in z["shape"]]
    bits = lambda a: torch.from_numpy(a.view(np.int16).copy()).view(torch.bfloat16)  # noqa: E731
    q, k, v = bits(z["q"]), bits(z["k"]), bits(z["v"])
    kv_lens = torch.from_numpy(z["kv_lens"]).to(dev) if "kv_lens" in z.files else None
    o, l = run_fwd(q, k, v, bool(causal), dev, kv_lens=kv_lens)
    assert float((o.float() - torch.from_numpy(z["o_ref_fp32"])).abs().max()) <= TOL_O
    assert float((l[:, :, 0, :] - torch.from_numpy(z["lse_def_fp64"]).float()).abs().max()) <= TOL_L


LPIN = sorted(glob.glob(os.path.join(os.path.dirname(__file__), "golden", "lpin_*.npz")))


@pytest.mark.parametrize("path", LPIN, ids=[os.path.basename(p) for p in LPIN])
def test_lse_against_the_l_the_reference_backward_consumed(dev, path):
    """The fixture's L was accepted by the reference's own simple_flash_backward (rows of its exp(S - L) sum to one
    and its gradients equal the module's; tests/test_oracle.py). The kernel's L must be that L within 1e-3, and the
    same check the fixture passed is repeated on the kernel's L itself: rows of exp(scale q k^T - L) sum to one."""
    z = np.load(path)
    case = np.load(path.replace("lpin_", "case_"))
    b, n, h, hkv, d, _causal, _seed = [int(x) for x in case["shape"]]
    bf = lambda a: torch.from_numpy(a.view(np.int16).copy()).view(torch.bfloat16)  # noqa: E731
    q, k, v = bf(case["q"]).reshape(b, n, h, d), bf(case["k"]).reshape(b, n, hkv, d), bf(case["v"]).reshape(b, n, hkv, d)
    _o, l = run_fwd(q, k, v, False, dev)
    assert float((l[:, :, 0, :] - torch.from_numpy(z["lse_fed"])).abs().max()) <= TOL_L
    kk = k.double().repeat_interleave(h // hkv, dim=2)
    s = torch.einsum("bthd,bshd->bhts", q.double(), kk) / math.sqrt(d)
    rowsum = torch.exp(s - l[:, :, 0, :].double().unsqueeze(-1)).sum(-1)
    assert float((rowsum - 1).abs().max()) <= TOL_L


def test_through_reference_entry_points(dev):
    """tk_kernel.dispatch_micro and tk_kernel_fwd.dispatch_fwd, called as the reference's harness and
    training code call them (kernels/attn/gqa/test_python.py:97-102, hipkittens.py:43-51)."""
    q, k, v = make_prefill_inputs(2, 256, 8, 2, 128, seed=11)
    qd, kd, vd = (t.to(dev).requires_grad_(True) for t in (q, k, v))
    for causal in (False, True):
        o_ref, l_ref = attn_fwd_oracle(q, k, v, causal)
        tk = hk.load_tk_kernel(causal)
        out = torch.zeros(2, 256, 8, 128, dtype=torch.bfloat16, device=dev, requires_grad=True)
        lse = torch.zeros(2, 8, 1, 256, dtype=torch.float32, device=dev, requires_grad=True)
        tk.dispatch_micro(qd, kd, vd, out, lse)
        torch.cuda.synchronize()
        assert_parity(out.detach().cpu(), lse.detach().cpu(), o_ref, l_ref)
        fwd = hk.load_tk_kernel_fwd(causal)
        O = torch.empty(2, 256, 8, 128, dtype=torch.bfloat16, device=dev)
        L = torch.empty(2, 8, 1, 256, dtype=torch.float32, device=dev)
        fwd.dispatch_fwd(qd, kd, vd, O, L)  # blocking, like the reference's
        assert_parity(O.cpu(), L.cpu(), o_ref, l_ref)


def test_autograd_function_forward(dev):
    from hipkittens_b200.attention import HipCrossAttention, HipSelfAttention

    q, k, v = make_prefill_inputs(1, 256, 4, 4, 64, seed=12)
    qkv = torch.stack([q, k, v], dim=2).to(dev)
    out = HipSelfAttention(causal=True)(qkv)
    o_ref, _ = attn_fwd_oracle(q, k, v, True)
    assert out.dtype == torch.bfloat16 and float((out.float().cpu() - o_ref.float()).abs().max()) <= TOL_O
    q, k, v = make_prefill_inputs(1, 256, 8, 2, 64, seed=13)
    out = HipCrossAttention(causal=False)(q.to(dev), torch.stack([k, v], dim=2).to(dev))
    o_ref, _ = attn_fwd_oracle(q, k, v, False)
    assert float((out.float().cpu() - o_ref.float()).abs().max()) <= TOL_O


def test_strided_views_of_a_packed_projection(dev):
    """q, k, v as views of [B,N,3,H,D] / [B,N,2,H_KV,D] (what mha.py:213-243 produces) give the same bits as
    contiguous copies, without any copy being made."""
    from hipkittens_b200.attention import HipCrossAttention, HipSelfAttention

    gen = torch.Generator().manual_seed(21)
    qkv = torch.randn((2, 384, 3, 4, 128), generator=gen).to(torch.bfloat16).to(dev)
    q, k, v = qkv.unbind(dim=2)
    assert not q.is_contiguous()
    o_s, l_s = hk.attn_fwd(q, k, v, causal=True)
    o_c, l_c = hk.attn_fwd(q.contiguous(), k.contiguous(), v.contiguous(), causal=True)
    assert _native.device_status(0) == 0
    assert torch.equal(o_s, o_c) and torch.equal(l_s, l_c)
    o_ref, l_ref = attn_fwd_oracle(q.cpu(), k.cpu(), v.cpu(), True)
    assert_parity(o_s.cpu(), l_s.cpu(), o_ref, l_ref)
    out = HipSelfAttention(causal=True)(qkv)
    assert torch.equal(out, o_c)
    # GQA: q from its own projection, k/v views of a packed [B,N,2,H_KV,D]
    qg = torch.randn((2, 256, 8, 64), generator=gen).to(torch.bfloat16).to(dev)
    kv = torch.randn((2, 256, 2, 2, 64), generator=gen).to(torch.bfloat16).to(dev)
    out = HipCrossAttention(causal=False)(qg, kv)
    o_ref, _ = attn_fwd_oracle(qg.cpu(), kv[:, :, 0].cpu(), kv[:, :, 1].cpu(), False)
    assert float((out.float().cpu() - o_ref.float()).abs().max()) <= TOL_O


def test_key_padding_lengths(dev):
    """Per-batch key lengths (the reference's key_padding_mask), including a length inside the first tile, one on a
    tile boundary and the full length; whole KV tiles beyond a length are skipped by the kernel."""
    q, k, v = make_prefill_inputs(4, 512, 8, 2, 128, seed=22)
    lens = torch.tensor([512, 5, 256, 300], dtype=torch.int32)
    o, l = run_fwd(q, k, v, False, dev, kv_lens=lens.to(dev))
    o_ref, l_ref = attn_fwd_oracle(q, k, v, False, kv_lens=lens)
    assert_parity(o, l, o_ref, l_ref)
    # poisoning the padded keys must not change anything
    k2, v2 = k.clone(), v.clone()
    for b in range(4):
        k2[b, int(lens[b]):] = 1e4
        v2[b, int(lens[b]):] = -3e4  # finite: a padded key inside a loaded tile still meets p = 0 in the product
    o2, l2 = run_fwd(q, k2, v2, False, dev, kv_lens=lens.to(dev))
    assert torch.equal(o, o2) and torch.equal(l, l2)


CROSS = sorted(glob.glob(os.path.join(os.path.dirname(__file__), "golden", "cross_*.npz")))


@pytest.mark.parametrize("path", CROSS, ids=[os.path.basename(p) for p in CROSS])
def test_unequal_lengths_and_causal_padding_against_reference_module(dev, path):
    """hk_attn_fwd_cross against outputs of the reference's CrossAttention(causal=...)(q, kv, key_padding_mask=...)
    with Sq != Sk (base.py:104-116 aligns the causal mask to the last query and the last kept key). Rows that see no
    key are O = 0, L = -inf here and are not compared with the reference (its -10000 fill is an artefact)."""
    from test_oracle import load_cross

    z, q, k, v, _d_o, kv_lens, causal, valid = load_cross(path)
    o, l = run_fwd(q, k, v, causal, dev, kv_lens=kv_lens.to(dev) if kv_lens is not None else None)
    assert not torch.isnan(o.float()).any() and not torch.isnan(l).any()
    o_ref = torch.from_numpy(z["o_ref_fp32"])
    assert float((o.float() - o_ref)[valid].abs().max()) <= TOL_O
    l_ref = torch.from_numpy(z["lse_def_fp64"]).float()
    vh = valid.unsqueeze(1).expand_as(l_ref)
    assert float((l[:, :, 0, :] - l_ref)[vh].abs().max()) <= TOL_L
    if not bool(valid.all()):
        assert float(o[~valid].float().abs().max()) == 0.0
        assert bool((l[:, :, 0, :][~vh] == float("-inf")).all())


CROSS_SHAPES = [
    # B, Nq, Nk, H, H_KV, D, causal, kv_lens
    (2, 128, 1024, 8, 2, 128, True, None),          # a 128-token chunk against a longer cache, offset 896
    (1, 100, 1000, 4, 4, 64, True, None),           # neither a multiple of the tile: the diagonal crosses two tiles
    (2, 300, 700, 6, 2, 128, True, [700, 301]),     # causal + padding, offsets 400 and 1
    (3, 256, 256, 4, 2, 64, True, [256, 129, 1]),   # self-attention shape, kept keys < queries: rows without keys
    (1, 520, 130, 2, 1, 128, True, None),           # more queries than keys: whole query blocks see nothing
    (2, 1, 777, 8, 1, 128, True, [777, 5]),         # a single query token against a cache (decode through the prefill kernel)
    (2, 200, 456, 4, 2, 64, False, [456, 77]),      # non-causal cross attention with padding
    (1, 640, 384, 3, 3, 128, False, None),          # odd head count (q-block pairing), Nk < Nq
    (1, 384, 640, 3, 3, 64, True, None),            # q-block pairs whose two blocks have different tile counts
]


@pytest.mark.parametrize("b,nq,nk,h,hkv,d,causal,lens", CROSS_SHAPES)
def test_unequal_lengths_parity(dev, b, nq, nk, h, hkv, d, causal, lens):
    gen = torch.Generator().manual_seed(1234 + nq + nk)
    q = torch.randn((b, nq, h, d), generator=gen).to(torch.bfloat16)
    k = torch.randn((b, nk, hkv, d), generator=gen).to(torch.bfloat16)
    v = torch.randn((b, nk, hkv, d), generator=gen).to(torch.bfloat16)
    kv_lens = torch.tensor(lens, dtype=torch.int32) if lens is not None else None
    o, l = run_fwd(q, k, v, causal, dev, kv_lens=kv_lens.to(dev) if kv_lens is not None else None)
    o_ref, l_ref = attn_fwd_oracle(q, k, v, causal, kv_lens=kv_lens)
    assert not torch.isnan(o.float()).any() and not torch.isnan(l).any()
    assert float((o.float() - o_ref.float()).abs().max()) <= TOL_O
    finite = torch.isfinite(l_ref)
    assert torch.equal(torch.isfinite(l), finite)            # rows without keys: L = -inf on both sides
    assert float((l - l_ref)[finite].abs().max()) <= TOL_L
    assert float(o[~finite[:, :, 0, :].transpose(1, 2)].float().abs().max() if not bool(finite.all()) else 0.0) == 0.0


def test_chunk_against_cache_equals_rows_of_the_full_causal_forward(dev):
    """Size-independent property of the bottom-right aligned mask: the last T query rows of a causal self-attention
    over N tokens are exactly a T-row chunk attending causally to all N keys (chunked prefill)."""
    q, k, v = make_prefill_inputs(2, 1024, 8, 2, 128, seed=77)
    o_full, l_full = run_fwd(q, k, v, True, dev)
    for t in (128, 200, 1):
        o_c, l_c = run_fwd(q[:, -t:].contiguous(), k, v, True, dev)
        assert torch.equal(o_c, o_full[:, -t:]) or float((o_c.float() - o_full[:, -t:].float()).abs().max()) <= 8e-3
        assert float((l_c - l_full[:, :, :, -t:]).abs().max()) <= 1e-4


def test_long_sequence_n16384(dev):
    """The longest length of the reference's sweeps (analysis/attn/fwd/benchmark/mi355x_benchmark.sh:18)."""
    q, k, v = make_prefill_inputs(1, 16384, 8, 1, 128, seed=23)
    o, l = run_fwd(q, k, v, True, dev)
    rows = slice(16384 - 256, 16384)
    o_ref, l_ref = _band_oracle(q, k, v, True, rows)
    assert float((o[0, rows].float() - o_ref[0].float()).abs().max()) <= TOL_O
    assert float((l[0, :, 0, rows] - l_ref[0, :, 0]).abs().max()) <= TOL_L
    rows = slice(0, 128)
    o_ref, l_ref = _band_oracle(q, k, v, True, rows)
    assert float((o[0, rows].float() - o_ref[0].float()).abs().max()) <= TOL_O


def test_custom_softmax_scale(dev):
    q, k, v = make_prefill_inputs(1, 256, 2, 1, 128, seed=14)
    o, l = run_fwd(q, k, v, False, dev, scale=0.05)
    o_ref, l_ref = attn_fwd_oracle(q, k, v, False, softmax_scale=0.05)
    assert_parity(o, l, o_ref, l_ref)


def test_adversarial_numerics(dev):
    q, k, v = make_prefill_inputs(1, 512, 2, 1, 128, seed=15)
    # (a) one huge logit per row late in the sequence: the running max jumps, forcing the rescale path
    k2 = k.clone()
    k2[0, 400] = (q[0, 100, 0].float() * 4).to(torch.bfloat16)
    o, l = run_fwd(q, k2, v, False, dev)
    assert_parity(o, l, *attn_fwd_oracle(q, k2, v, False))
    # (b) logits that keep growing tile after tile (max rises by more than the lazy threshold each tile)
    kg = (k.float() * torch.linspace(0.2, 6.0, 512).view(1, 512, 1, 1)).to(torch.bfloat16)
    o, l = run_fwd(q, kg, v, False, dev)
    assert_parity(o, l, *attn_fwd_oracle(q, kg, v, False))
    # (c) all-equal logits: uniform softmax, L = ln N
    qz = torch.zeros_like(q)
    o, l = run_fwd(qz, k, v, False, dev)
    assert float((l - math.log(512)).abs().max()) <= 1e-5
    assert_parity(o, l, *attn_fwd_oracle(qz, k, v, False))
    # (d) causal first row sees exactly one key: O = V[0], L = its logit
    o, l = run_fwd(q, k, v, True, dev)
    assert torch.equal(o[0, 0, 0], v[0, 0, 0])
    assert_parity(o, l, *attn_fwd_oracle(q, k, v, True))
    # (e) large-magnitude logits (|s| of several hundred) stay finite
    qb = (q.float() * 30).to(torch.bfloat16)
    o, l = run_fwd(qb, k, v, False, dev)
    assert torch.isfinite(o.float()).all() and torch.isfinite(l).all()
    o_ref, l_ref = attn_fwd_oracle(qb, k, v, False)
    assert float((o.float() - o_ref.float()).abs().max()) <= TOL_O
    assert float(((l - l_ref).abs() / l_ref.abs().clamp_min(1)).max()) <= 1e-5
    # (f) logits that jump by hundreds of powers of two after the first tiles: the kernel takes its exponentials
    # against the maximum it already has and must notice the overflow and redo the tile exactly; the jump sits in a
    # full tile, in the partial last tile, and (causal) in a diagonal tile, for both head dimensions
    for n, causal, jump_at, hd in ((512, False, 300, 128), (450, False, 400, 128), (640, True, 520, 128),
                                   (512, False, 300, 64), (450, False, 400, 64), (640, True, 520, 64)):
        qf, kf, vf = make_prefill_inputs(2, n, 4, 2, hd, seed=17 + n)
        kj = kf.clone()
        kj[:, jump_at:] = (kf[:, jump_at:].float() * 60).to(torch.bfloat16)
        qj = (qf.float() * 4).to(torch.bfloat16)
        o, l = run_fwd(qj, kj, vf, causal, dev)
        o_ref, l_ref = attn_fwd_oracle(qj, kj, vf, causal)
        assert torch.isfinite(o.float()).all() and torch.isfinite(l).all()
        assert float((o.float() - o_ref.float()).abs().max()) <= TOL_O
        if hd == 128:
            assert float(((l - l_ref).abs() / l_ref.abs().clamp_min(1)).max()) <= 1e-5
        else:
            # a quarter of the D = 64 exponentials come from a polynomial with a relative error of 1e-4, which is the
            # absolute error of L when one such term dominates a row
            assert float((l - l_ref).abs().max()) <= 2.5e-4
    # (g) logits that FALL by hundreds of powers of two after the first tile: later tiles underflow to zero, as they
    # should (their true weight is below fp32 resolution)
    kd = kf.clone()
    kd[:, :128] = (kf[:, :128].float() * 60).to(torch.bfloat16)
    o, l = run_fwd(qj, kd, vf, False, dev)
    o_ref, l_ref = attn_fwd_oracle(qj, kd, vf, False)
    assert float((o.float() - o_ref.float()).abs().max()) <= TOL_O
    assert float((l - l_ref).abs().max()) <= 2.5e-4  # D = 64 here (the last shape of the loop above)


def test_bitwise_deterministic_and_gqa_equals_mha(dev):
    q, k, v = make_prefill_inputs(2, 512, 8, 2, 128, seed=16)
    o1, l1 = run_fwd(q, k, v, True, dev)
    o2, l2 = run_fwd(q, k, v, True, dev)
    assert torch.equal(o1, o2) and torch.equal(l1, l2)
    o3, l3 = run_fwd(q, k.repeat_interleave(4, dim=2), v.repeat_interleave(4, dim=2), True, dev)
    assert torch.equal(o1, o3) and torch.equal(l1, l3)


def _gpu_fp32_unit(q, k, v, causal):
    """fp32 restatement on the GPU for one (batch, kv-head) unit of a full-size shape (the CPU oracle on
    the whole tensor would take minutes); used only next to CPU-oracle spot checks."""
    n = q.shape[0]
    s = torch.einsum("tgd,sd->gts", q.float(), k.float()) / math.sqrt(q.shape[-1])
    if causal:
        s = s.masked_fill(torch.triu(torch.ones(n, n, dtype=torch.bool, device=q.device), 1), float("-inf"))
    lse = torch.logsumexp(s, -1)
    return torch.einsum("gts,sd->tgd", torch.exp(s - lse[..., None]), v.float()).to(torch.bfloat16), lse


FULL = [
    (16, 2048, 64, 8, 128, False),  # BASELINE config 2
    (4, 8192, 64, 8, 128, True),    # config 3
    (16, 4096, 16, 16, 64, False),  # config 4
]


@pytest.mark.parametrize("b,n,h,hkv,d,causal", FULL)
def test_full_size_configs(dev, b, n, h, hkv, d, causal):
    g = h // hkv
    q, k, v = make_prefill_inputs(b, n, h, hkv, d, seed=0)
    qd, kd, vd = q.to(dev), k.to(dev), v.to(dev)
    o = torch.full_like(qd, float("nan"))
    l = torch.full((b, h, 1, n), float("nan"), dtype=torch.float32, device=dev)
    hk.attn_fwd(qd, kd, vd, causal=causal, out=o, lse=l)
    assert _native.device_status(0) == 0
    assert not torch.isnan(o.float()).any() and not torch.isnan(l).any()
    # (1) CPU oracle on the first and last (batch, kv-head) unit, a row band of the queries for long N
    for bi, kh in ((0, 0), (b - 1, hkv - 1)):
        rows = slice(0, n) if n <= 2048 else slice(n - 512, n)
        qs = q[bi:bi + 1, :, kh * g:(kh + 1) * g]
        o_ref, l_ref = _band_oracle(qs, k[bi:bi + 1, :, kh:kh + 1], v[bi:bi + 1, :, kh:kh + 1], causal, rows)
        eo = float((o[bi, rows, kh * g:(kh + 1) * g].float().cpu() - o_ref[0].float()).abs().max())
        el = float((l[bi, kh * g:(kh + 1) * g, 0, rows].cpu() - l_ref[0, :, 0]).abs().max())
        assert eo <= TOL_O and el <= TOL_L, (bi, kh, eo, el)
    # (2) every unit against the fp32 restatement evaluated on the GPU
    worst_o = worst_l = 0.0
    for bi in range(b):
        for kh in range(hkv):
            o_ref, l_ref = _gpu_fp32_unit(qd[bi, :, kh * g:(kh + 1) * g], kd[bi, :, kh], vd[bi, :, kh], causal)
            worst_o = max(worst_o, float((o[bi, :, kh * g:(kh + 1) * g].float() - o_ref.float()).abs().max()))
            worst_l = max(worst_l, float((l[bi, kh * g:(kh + 1) * g, 0] - l_ref).abs().max()))
            del o_ref, l_ref
    assert worst_o <= TOL_O and worst_l <= TOL_L, (worst_o, worst_l)
    # (3) size-independent properties: scaling V by 2 doubles O exactly and leaves L unchanged
    o2 = torch.empty_like(o)
    l2 = torch.empty_like(l)
    hk.attn_fwd(qd, kd, (vd.float() * 2).to(torch.bfloat16), causal=causal, out=o2, lse=l2)
    assert torch.equal(o2.float(), o.float() * 2) and torch.equal(l2, l)


def _band_oracle(q, k, v, causal, rows):
    """CPU oracle for a band of query rows of one unit (keeps the score matrix small for N = 8192)."""
    n = q.shape[1]
    qb = q[:, rows]
    nb = qb.shape[1]
    g = q.shape[2]
    scale = 1.0 / math.sqrt(q.shape[-1])
    s = torch.einsum("tgd,sd->gts", qb[0].float(), k[0, :, 0].float() * scale)
    if causal:
        row = torch.arange(rows.start, rows.stop).view(nb, 1)
        col = torch.arange(n).view(1, n)
        s = s.masked_fill((col > row).unsqueeze(0), float("-inf"))
    lse = torch.logsumexp(s, -1)
    o = torch.einsum("gts,sd->tgd", torch.exp(s - lse[..., None]), v[0, :, 0].float())
    return o.to(torch.bfloat16)[None], lse[None, :, None, :].reshape(1, g, 1, nb)


def test_causal_prefix_property(dev):
    """Causal attention on the first half of a sequence equals the first half of causal attention on the
    whole sequence, bit for bit (same tiles, same order of accumulation)."""
    q, k, v = make_prefill_inputs(1, 2048, 8, 2, 128, seed=17)
    o_full, l_full = run_fwd(q, k, v, True, dev)
    o_half, l_half = run_fwd(q[:, :1024].contiguous(), k[:, :1024].contiguous(), v[:, :1024].contiguous(), True, dev)
    assert torch.equal(o_full[:, :1024], o_half) and torch.equal(l_full[..., :1024], l_half)


def test_bounded_wait_reports_timeout_and_context_survives(dev):
    lib = hk.capi()
    assert lib.hk_selftest_bounded_wait(0, 2000) == _native.HK_ETIMEOUT
    assert lib.hk_last_device_status(0) == 0  # cleared on read
    q, k, v = make_prefill_inputs(1, 128, 2, 1, 64, seed=18)
    o, l = run_fwd(q, k, v, False, dev)
    assert_parity(o, l, *attn_fwd_oracle(q, k, v, False))


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two visible GPUs")
def test_callers_current_device_is_left_alone():
    """A call on another GPU's tensors must not change the calling thread's current device (the reference
    launcher never touches it): torch's current device and stream stay what they were."""
    torch.cuda.set_device(0)
    try:
        other = torch.device("cuda:1")
        q, k, v = (t.to(other) for t in make_prefill_inputs(1, 256, 4, 2, 128, seed=3))
        o, l = hk.attn_fwd(q, k, v, causal=True)
        assert torch.cuda.current_device() == 0
        assert _native.device_status(1) == 0
        assert torch.cuda.current_device() == 0
        o_ref, l_ref = attn_fwd_oracle(q.cpu(), k.cpu(), v.cpu(), True)
        assert float((o.float().cpu() - o_ref.float()).abs().max()) <= TOL_O
        # the runtime's own view, not just torch's cached one: a fresh allocation lands on device 0
        assert torch.ones(4, device="cuda").device.index == 0
    finally:
        torch.cuda.set_device(0)
