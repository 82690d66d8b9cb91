"""Rotary embedding: the oracle against the fixture produced by the reference harness's own functions (CPU), and the
CUDA kernel against the oracle, bit for bit (GPU). All arithmetic is bf16 with one rounding per operation, so the
bar is exact equality."""
import os

import numpy as np
import pytest
import torch

import hipkittens_b200 as hk
from hipkittens_b200 import _native
from oracle.attn_oracle import rotary_cos_sin, rotary_oracle

FIXTURE = os.path.join(os.path.dirname(__file__), "golden", "rotary_b2_h3_n160_d128.npz")


def _bf16(bits: np.ndarray) -> torch.Tensor:
    return torch.from_numpy(bits.view(np.int16).copy()).view(torch.bfloat16)


def test_oracle_matches_reference_harness_functions():
    z = np.load(FIXTURE)
    b, h, n, d, ro = [int(v) for v in z["shape"]]
    x, cos, sin, ref = _bf16(z["x"]), _bf16(z["cos"]), _bf16(z["sin"]), _bf16(z["o_ref"])
    assert x.shape == (b, h, n, d) and cos.shape == (n, ro // 2)
    assert torch.equal(rotary_oracle(x, cos, sin).view(torch.int16), ref.view(torch.int16))
    c2, s2 = rotary_cos_sin(n, ro)
    assert torch.equal(c2.view(torch.int16), cos.view(torch.int16)) and torch.equal(s2.view(torch.int16), sin.view(torch.int16))


def test_oracle_properties():
    gen = torch.Generator().manual_seed(1)
    x = torch.randn((1, 2, 64, 64), generator=gen).to(torch.bfloat16)
    cos, sin = rotary_cos_sin(64, 32)          # partial rotary: the last 32 dimensions pass through
    o = rotary_oracle(x, cos, sin)
    assert torch.equal(o[..., 32:], x[..., 32:])
    assert torch.equal(o[:, :, 0], x[:, :, 0])  # position 0: cos = 1, sin = 0
    # rotation preserves the norm of each (x_i, x_{i+R/2}) pair up to bf16 rounding
    n_in = x[..., :16].float() ** 2 + x[..., 16:32].float() ** 2
    n_out = o[..., :16].float() ** 2 + o[..., 16:32].float() ** 2
    assert float((n_in - n_out).abs().max()) <= 0.05 * float(n_in.max())


def test_capi_rejects_bad_arguments_before_cuda(native_built):
    lib = hk.capi()
    assert lib.hk_rotary(None, 64, 64, 64, 1, 1, 16, 128, 128, 0, None) == _native.HK_EINVAL
    assert lib.hk_rotary(64, 64, 64, 72, 1, 1, 16, 128, 128, 0, None) == _native.HK_EINVAL      # misaligned cos
    assert lib.hk_rotary(64, 64, 64, 64, 1, 1, 16, 128, 136, 0, None) == _native.HK_EUNSUPPORTED  # R > D
    assert lib.hk_rotary(64, 64, 64, 64, 1, 1, 16, 100, 64, 0, None) == _native.HK_EUNSUPPORTED   # D % 8
    assert lib.hk_rotary(64, 64, 64, 64, 1, 0, 16, 128, 128, 0, None) == _native.HK_EINVAL
    mod = hk.load_tk_kernel_rotary()
    assert mod.__name__.endswith("kernels.rotary.tk_kernel") and hasattr(mod, "dispatch_rotary")
    with pytest.raises(RuntimeError, match="Expected a torch.Tensor"):
        mod.dispatch_rotary(None, None, None, None)
    with pytest.raises(RuntimeError, match="Tensor must be on CUDA device"):
        mod.dispatch_rotary(*(torch.zeros(1, 1, 16, 128, dtype=torch.bfloat16),) * 2,
                            *(torch.zeros(16, 64, dtype=torch.bfloat16),) * 2)


@pytest.mark.gpu
@pytest.mark.parametrize("b,h,n,d,ro", [(2, 3, 160, 128, 128), (1, 2, 77, 64, 64), (2, 4, 256, 128, 64),
                                        (1, 1, 1, 128, 128), (16, 16, 2048, 128, 128)])
def test_kernel_is_bit_exact(b, h, n, d, ro):
    dev = torch.device("cuda:0")
    gen = torch.Generator().manual_seed(b * 100 + n)
    x = torch.randn((b, h, n, d), generator=gen).to(torch.bfloat16)
    cos, sin = rotary_cos_sin(n, ro)
    ref = rotary_oracle(x, cos, sin)
    out = hk.rotary(x.to(dev), cos.to(dev), sin.to(dev))
    assert _native.device_status(0) == 0
    assert torch.equal(out.cpu().view(torch.int16), ref.view(torch.int16))
    # the reference's entry point, argument order (x, o, sin, cos), and in place
    mod = hk.load_tk_kernel_rotary()
    xd = x.to(dev)
    o2 = torch.full_like(xd, float("nan"))
    mod.dispatch_rotary(xd, o2, sin.to(dev), cos.to(dev))
    torch.cuda.synchronize()
    assert torch.equal(o2.cpu().view(torch.int16), ref.view(torch.int16))
    hk.rotary(xd, cos.to(dev), sin.to(dev), out=xd)
    assert torch.equal(xd.cpu().view(torch.int16), ref.view(torch.int16))


@pytest.mark.gpu
def test_kernel_against_reference_harness_fixture():
    z = np.load(FIXTURE)
    dev = torch.device("cuda:0")
    x, cos, sin, ref = _bf16(z["x"]), _bf16(z["cos"]), _bf16(z["sin"]), _bf16(z["o_ref"])
    out = hk.rotary(x.to(dev), cos.to(dev), sin.to(dev))
    assert torch.equal(out.cpu().view(torch.int16), ref.view(torch.int16))


@pytest.mark.gpu
def test_opposite_angle_undoes_the_rotation():
    """The backward of the pre-pass is the rotation by the opposite angle (-sin): applying both gives x back up to bf16
    rounding of the two passes (cos^2 + sin^2 = 1 only to bf16 precision)."""
    dev = torch.device("cuda:0")
    x = torch.randn((2, 4, 256, 128), generator=torch.Generator().manual_seed(9)).to(torch.bfloat16).to(dev)
    cos, sin = rotary_cos_sin(256, 128)
    cos, sin = cos.to(dev), sin.to(dev)
    y = hk.rotary(x, cos, sin)
    back = hk.rotary(y, cos, (-sin.float()).to(torch.bfloat16))
    assert float((back.float() - x.float()).abs().max()) <= 0.06 * float(x.float().abs().max())
    # and it is the transpose: <rot(x), g> == <x, rot^T(g)>
    g = torch.randn(x.shape, generator=torch.Generator().manual_seed(10)).to(torch.bfloat16).to(dev)
    lhs = float((y.float() * g.float()).sum())
    rhs = float((x.float() * hk.rotary(g, cos, (-sin.float()).to(torch.bfloat16)).float()).sum())
    assert abs(lhs - rhs) <= 2e-3 * float((x.float().abs() * g.float().abs()).sum())


@pytest.mark.gpu
@pytest.mark.parametrize("b,n,h,d,ro,pos0", [(2, 160, 3, 128, 128, 0), (1, 77, 2, 64, 32, 5), (3, 1, 8, 128, 128, 300)])
def test_attention_layout_kernel_is_bit_exact(b, n, h, d, ro, pos0):
    """hk_rotary_bnhd on x [B,N,H,D] equals the oracle applied to the transposed tensor with the table rows
    pos0 .. pos0 + N - 1 (a chunk that continues a cached prefix), bit for bit, also in place."""
    dev = torch.device("cuda:0")
    x = torch.randn((b, n, h, d), generator=torch.Generator().manual_seed(n + h)).to(torch.bfloat16)
    cos, sin = rotary_cos_sin(n + pos0 + 3, ro)
    ref = rotary_oracle(x.transpose(1, 2).contiguous(), cos[pos0:pos0 + n], sin[pos0:pos0 + n]).transpose(1, 2).contiguous()
    out = hk.rotary_bnhd(x.to(dev), cos.to(dev), sin.to(dev), pos_offset=pos0)
    assert _native.device_status(0) == 0
    assert torch.equal(out.cpu().view(torch.int16), ref.view(torch.int16))
    xd = x.to(dev)
    hk.rotary_bnhd(xd, cos.to(dev), sin.to(dev), out=xd, pos_offset=pos0)
    assert torch.equal(xd.cpu().view(torch.int16), ref.view(torch.int16))


@pytest.mark.gpu
@pytest.mark.parametrize("s_n,t_n,hkv,d,ro", [(3, 40, 2, 128, 128), (2, 1, 8, 128, 64), (4, 130, 1, 64, 64)])
def test_append_with_fused_rotary_equals_rotary_then_append(s_n, t_n, hkv, d, ro):
    """hk_paged_kv_append_rotary leaves in the pages exactly what the reference's order leaves (rotate k, then update
    the cache, mha.py:217-220 then 16-42): checked against the rotary oracle followed by the append oracle, and
    against the two separate kernels, bit for bit. V is copied untouched; pages not named by the call keep their
    contents."""
    from oracle.attn_oracle import paged_kv_append_oracle

    dev = torch.device("cuda:0")
    gen = torch.Generator().manual_seed(s_n * 10 + t_n)
    k_new = torch.randn((s_n, t_n, hkv, d), generator=gen).to(torch.bfloat16)
    v_new = torch.randn((s_n, t_n, hkv, d), generator=gen).to(torch.bfloat16)
    start = torch.randint(0, 50, (s_n,), generator=gen, dtype=torch.int32)
    max_pages = (50 + t_n + 15) // 16
    pool = s_n * max_pages + 3
    bt = torch.randperm(pool, generator=gen)[: s_n * max_pages].to(torch.int32).view(s_n, max_pages)
    kp0 = torch.randn((pool, 16, hkv, d), generator=gen).to(torch.bfloat16)
    vp0 = torch.randn((pool, 16, hkv, d), generator=gen).to(torch.bfloat16)
    cos, sin = rotary_cos_sin(50 + t_n + 1, ro)
    # oracle: rotate each sequence's new keys at its own positions, then append
    k_rot = torch.empty_like(k_new)
    for s in range(s_n):
        p0 = int(start[s])
        k_rot[s] = rotary_oracle(k_new[s].transpose(0, 1).unsqueeze(0).contiguous(), cos[p0:p0 + t_n],
                                 sin[p0:p0 + t_n])[0].transpose(0, 1)
    kp_ref, vp_ref = paged_kv_append_oracle(k_rot, v_new, kp0, vp0, bt, start)
    kp, vp = kp0.to(dev), vp0.to(dev)
    hk.paged_kv_append_rotary(k_new.to(dev), v_new.to(dev), kp, vp, bt.to(dev), start.to(dev), cos.to(dev), sin.to(dev))
    assert _native.device_status(0) == 0
    assert torch.equal(kp.cpu().view(torch.int16), kp_ref.view(torch.int16))
    assert torch.equal(vp.cpu().view(torch.int16), vp_ref.view(torch.int16))
    # a position beyond the cos / sin table is skipped and reported, like one beyond the block table
    hk.paged_kv_append_rotary(k_new.to(dev), v_new.to(dev), kp, vp, bt.to(dev), start.to(dev), cos[:10].to(dev).contiguous(),
                              sin[:10].to(dev).contiguous())
    assert _native.device_status(0) == _native.HK_EBADPAGE


@pytest.mark.gpu
def test_rotary_append_decode_chain_against_oracles():
    """The serving step end to end: rotate the new token's q and k, append k and v to the paged cache (fused), decode.
    Equals rotary_oracle followed by the append and decode oracles within the decode tolerances."""
    from hipkittens_b200.synthetic import make_paged_inputs
    from oracle.attn_oracle import paged_decode_oracle, paged_kv_append_oracle

    dev = torch.device("cuda:0")
    s_n, h, hkv, d = 3, 8, 2, 128
    q, kp, vp, bt, cl = make_paged_inputs(s_n, h, hkv, d, 16, 300, 100, 900, seed=41)
    gen = torch.Generator().manual_seed(42)
    k_new = torch.randn((s_n, 1, hkv, d), generator=gen).to(torch.bfloat16)
    v_new = torch.randn((s_n, 1, hkv, d), generator=gen).to(torch.bfloat16)
    start = (cl - 1).to(torch.int32)               # the new token takes the last position of each context
    cos, sin = rotary_cos_sin(1024, d)
    # oracle chain
    q_rot = torch.stack([rotary_oracle(q[s].transpose(0, 1).unsqueeze(0).contiguous(), cos[int(start[s]):int(start[s]) + 1],
                                       sin[int(start[s]):int(start[s]) + 1])[0].transpose(0, 1) for s in range(s_n)])
    k_rot = torch.stack([rotary_oracle(k_new[s].transpose(0, 1).unsqueeze(0).contiguous(), cos[int(start[s]):int(start[s]) + 1],
                                       sin[int(start[s]):int(start[s]) + 1])[0].transpose(0, 1) for s in range(s_n)])
    kp_ref, vp_ref = paged_kv_append_oracle(k_rot, v_new, kp, vp, bt, start)
    o_ref, l_ref = paged_decode_oracle(q_rot, kp_ref, vp_ref, bt, cl)
    # device chain: q rotated per sequence at its own position, k fused into the append
    kpd, vpd, btd, cld = kp.to(dev), vp.to(dev), bt.to(dev), cl.to(dev)
    qd = torch.cat([hk.rotary_bnhd(q[s:s + 1].to(dev), cos.to(dev), sin.to(dev), pos_offset=int(start[s])) for s in range(s_n)])
    hk.paged_kv_append_rotary(k_new.to(dev), v_new.to(dev), kpd, vpd, btd, start.to(dev), cos.to(dev), sin.to(dev))
    o, l = hk.paged_decode(qd, kpd, vpd, btd, cld)
    assert _native.device_status(0) == 0
    assert torch.equal(qd.cpu().view(torch.int16), q_rot.view(torch.int16))
    assert float((o.float().cpu() - o_ref.float()).abs().max()) <= 2e-2
    assert float((l.cpu() - l_ref).abs().max()) <= 1e-3
