"""The C-ABI library: loads, exports every symbol the header declares, and validates arguments before it
touches CUDA (so these checks run without a GPU)."""
import ctypes
import os
import re

import pytest
import torch

import hipkittens_b200 as hk
from hipkittens_b200 import _native

HEADER = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "include", "hk_attn.h")


def declared_symbols():
    text = open(HEADER).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    text = re.sub(r"#ifdef HK_TRACE.*?#endif", "", text, flags=re.S)  # declarations of tuning builds only
    return sorted(set(re.findall(r"\b(hk_[a-z0-9_]+)\s*\(", text)))


def test_header_symbols_are_exported(native_built):
    lib = ctypes.CDLL(hk.lib_path())
    names = declared_symbols()
    assert len(names) >= 8
    for name in names:
        assert hasattr(lib, name), f"{name} is declared in hk_attn.h but not exported"
    assert set(names) == set(_native.EXPORTED_SYMBOLS)


def test_strerror_texts(native_built):
    lib = hk.capi()
    assert lib.hk_strerror(0) == b"ok"
    for code in (-1, -2, -3, -4, -5, -6, -7):
        assert lib.hk_strerror(code) not in (b"", b"ok", b"unknown error code")
    assert lib.hk_strerror(-99) == b"unknown error code"


def test_item_decode_division_selftest(native_built):
    """The kernels decode a work-item index with multiply-and-shift divisions by launch constants; the library checks
    that arithmetic against integer division on the host (no GPU involved)."""
    assert hk.capi().hk_selftest_fastdiv() == 0


def _fwd(lib, q=64, k=64, v=64, o=64, l=64, B=1, N=128, H=2, HKV=1, D=128, causal=0):
    return lib.hk_attn_fwd(q, k, v, o, l, B, N, H, HKV, D, causal, 0.0, 0, None)


def test_fwd_rejects_bad_arguments_before_cuda(native_built):
    lib = hk.capi()
    assert _fwd(lib, q=None) == _native.HK_EINVAL
    assert _fwd(lib, l=None) == _native.HK_EINVAL
    assert _fwd(lib, q=72) == _native.HK_EINVAL  # not 16-byte aligned
    assert _fwd(lib, N=0) == _native.HK_EINVAL
    assert _fwd(lib, H=3, HKV=2) == _native.HK_EINVAL
    assert _fwd(lib, B=0) == _native.HK_EINVAL
    assert _fwd(lib, D=96) == _native.HK_EUNSUPPORTED
    assert _fwd(lib, D=256) == _native.HK_EUNSUPPORTED


def test_strided_fwd_rejects_bad_strides_before_cuda(native_built):
    lib = hk.capi()
    arr = lambda *v: (ctypes.c_longlong * 3)(*v)  # noqa: E731

    def call(qs, ks=None, vs=None):
        ks = ks or arr(128 * 1 * 128, 128, 128)
        vs = vs or ks
        return lib.hk_attn_fwd_strided(64, 64, 64, 64, 64, 1, 128, 2, 1, 128, qs, ks, vs, 0, 0.0, 0, None)

    assert call(arr(128 * 2 * 128, 2 * 128 + 4, 128)) == _native.HK_EINVAL  # not a multiple of 8 elements
    assert call(arr(128 * 2 * 128, 0, 128)) == _native.HK_EINVAL
    assert call(arr(128 * 2 * 128, 2 * 128, -128)) == _native.HK_EINVAL
    assert call(None) == _native.HK_EINVAL


def test_decode_rejects_bad_arguments_before_cuda(native_built):
    lib = hk.capi()

    def call(q=64, S=2, H=8, HKV=1, D=128, page=16, max_pages=4, pool=8, ws=256, ws_bytes=1 << 20):
        return lib.hk_attn_paged_decode(q, 64, 64, 64, 64, 64, 64, S, H, HKV, D, page, max_pages, pool, 0.0, ws,
                                        ws_bytes, 0, None)

    assert call(q=None) == _native.HK_EINVAL
    assert call(D=64) == _native.HK_EUNSUPPORTED
    assert call(page=32) == _native.HK_EUNSUPPORTED
    assert call(H=9, HKV=1) == _native.HK_EUNSUPPORTED  # group size 9: more heads than rows of the MMA tile
    assert call(H=8, HKV=3) == _native.HK_EINVAL
    assert call(ws=None) == _native.HK_EWORKSPACE
    assert call(ws_bytes=16) == _native.HK_EWORKSPACE
    assert call(ws=264) == _native.HK_EWORKSPACE  # not 256-byte aligned


def test_workspace_size_formula(native_built):
    # one chunk = 32 pages; partial O fp32 [S][H][splits][128] + (m, l) pairs, each part rounded to 256 B
    assert hk.paged_decode_workspace_bytes(64, 64, 128, 512) == 64 * 64 * 16 * 128 * 4 + 64 * 64 * 16 * 2 * 4
    assert hk.paged_decode_workspace_bytes(1, 1, 128, 1) == 512 + 256
    assert hk.paged_decode_workspace_bytes(1, 1, 64, 1) == 0  # unsupported head dim


@pytest.mark.skipif(torch.cuda.is_available(), reason="checks the no-GPU failure mode")
def test_fails_loudly_without_a_gpu(native_built):
    lib = hk.capi()
    rc = _fwd(lib)
    assert rc == _native.HK_ECUDA
    assert lib.hk_last_cuda_error() != b""
    with pytest.raises(RuntimeError):
        hk.attn_fwd(torch.zeros(1, 128, 2, 128, dtype=torch.bfloat16), torch.zeros(1, 128, 1, 128, dtype=torch.bfloat16),
                    torch.zeros(1, 128, 1, 128, dtype=torch.bfloat16))


def test_bwd_rejects_bad_arguments_before_cuda(native_built):
    lib = hk.capi()

    def bwd(q=64, lse=64, dq=64, B=1, N=128, H=2, HKV=1, D=128, layout=0):
        return lib.hk_attn_bwd(q, 64, 64, 64, lse, 64, dq, 64, 64, B, N, H, HKV, D, 0, 0.0, layout, 0, None)

    assert bwd(q=None) == _native.HK_EINVAL
    assert bwd(lse=None) == _native.HK_EINVAL
    assert bwd(dq=72) == _native.HK_EINVAL      # not 16-byte aligned
    assert bwd(lse=66) == _native.HK_EINVAL     # fp32 arrays need 4-byte alignment
    assert bwd(H=3, HKV=2) == _native.HK_EINVAL
    assert bwd(layout=2) == _native.HK_EINVAL
    assert bwd(D=96) == _native.HK_EUNSUPPORTED
    assert bwd(N=0) == _native.HK_EINVAL
    assert lib.hk_attn_bwd_prep(None, 64, 64, 1, 128, 2, 128, 0, None) == _native.HK_EINVAL
    assert lib.hk_attn_bwd_prep(64, 64, 64, 1, 128, 2, 96, 0, None) == _native.HK_EUNSUPPORTED
    assert lib.hk_attn_bwd_prep(64, 64, 64, 1, 0, 2, 128, 0, None) == _native.HK_EINVAL
    assert lib.hk_attn_dq_shuffle(64, 64, 1, 128, 2, 128, 0, None) == _native.HK_EINVAL  # aliasing buffers
    assert lib.hk_attn_dq_shuffle(64, 128, 1, 128, 2, 100, 0, None) == _native.HK_EINVAL  # D not a multiple of 8
