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
