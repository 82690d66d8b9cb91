"""ctypes binding of ``libhk_attn.so`` plus torch-tensor front ends.

torch is used for device memory and streams only; all arithmetic happens in the CUDA library.
"""
from __future__ import annotations

import ctypes
import importlib.util
import math
import os
import sys
import sysconfig
from typing import Optional, Tuple

import torch

_PKG = os.path.dirname(os.path.abspath(__file__))
_LIB = os.path.join(_PKG, "lib", "libhk_attn.so")

HK_OK, HK_EINVAL, HK_EUNSUPPORTED, HK_ECUDA, HK_ETIMEOUT, HK_EWORKSPACE, HK_EBADPAGE, HK_EBADLEN = 0, -1, -2, -3, -4, -5, -6, -7

# Every symbol declared in include/hk_attn.h.
EXPORTED_SYMBOLS = (
    "hk_attn_fwd",
    "hk_attn_fwd_strided",
    "hk_attn_fwd_varlen",
    "hk_attn_fwd_cross",
    "hk_attn_fwd_paged",
    "hk_attn_bwd_prep",
    "hk_attn_bwd",
    "hk_attn_bwd_varlen",
    "hk_attn_bwd_cross",
    "hk_attn_dq_shuffle",
    "hk_rotary",
    "hk_rotary_bnhd",
    "hk_paged_kv_append_rotary",
    "hk_attn_paged_decode_workspace_bytes",
    "hk_attn_paged_decode",
    "hk_attn_paged_decode_static",
    "hk_paged_kv_append",
    "hk_last_device_status",
    "hk_selftest_bounded_wait",
    "hk_selftest_fastdiv",
    "hk_kernel_launch_count",
    "hk_strerror",
    "hk_last_cuda_error",
)


class HkError(RuntimeError):
    """A libhk_attn call returned a negative HK_E* code."""

    def __init__(self, code: int, what: str, detail: str = ""):
        self.code = code
        msg = f"{what}: error {code}"
        if detail:
            msg += f" ({detail})"
        super().__init__(msg)


def lib_path() -> str:
    return _LIB


_capi = None


def capi() -> ctypes.CDLL:
    """The loaded C-ABI library with argument types declared. Raises if it has not been built."""
    global _capi
    if _capi is not None:
        return _capi
    if not os.path.exists(_LIB):
        raise ImportError(
            f"{_LIB} is missing: build it with `python -m hipkittens_b200._build` (needs nvcc); "
            "there is no fallback implementation"
        )
    lib = ctypes.CDLL(_LIB)
    vp, ci, cf = ctypes.c_void_p, ctypes.c_int, ctypes.c_float
    lib.hk_attn_fwd.argtypes = [vp, vp, vp, vp, vp, ci, ci, ci, ci, ci, ci, cf, ci, vp]
    lib.hk_attn_fwd.restype = ci
    ll3 = ctypes.POINTER(ctypes.c_longlong)
    lib.hk_attn_fwd_strided.argtypes = [vp, vp, vp, vp, vp, ci, ci, ci, ci, ci, ll3, ll3, ll3, ci, cf, ci, vp]
    lib.hk_attn_fwd_strided.restype = ci
    lib.hk_attn_fwd_varlen.argtypes = [vp, vp, vp, vp, vp, ci, ci, ci, ci, ci, ll3, ll3, ll3, vp, ci, cf, ci, vp]
    lib.hk_attn_fwd_varlen.restype = ci
    lib.hk_attn_fwd_cross.argtypes = [vp, vp, vp, vp, vp, ci, ci, ci, ci, ci, ci, ll3, ll3, ll3, vp, ci, cf, ci, vp]
    lib.hk_attn_fwd_cross.restype = ci
    lib.hk_attn_fwd_paged.argtypes = [vp, vp, vp, vp, vp, vp, vp, ci, ci, ci, ci, ci, ci, ci, ci, ci, cf, ci, vp]
    lib.hk_attn_fwd_paged.restype = ci
    lib.hk_attn_bwd_prep.argtypes = [vp, vp, vp, ci, ci, ci, ci, ci, vp]
    lib.hk_attn_bwd_prep.restype = ci
    lib.hk_attn_bwd.argtypes = [vp, vp, vp, vp, vp, vp, vp, vp, vp, ci, ci, ci, ci, ci, ci, cf, ci, ci, vp]
    lib.hk_attn_bwd.restype = ci
    lib.hk_attn_bwd_varlen.argtypes = [vp, vp, vp, vp, vp, vp, vp, vp, vp, ci, ci, ci, ci, ci, vp, ci, cf, ci, ci, vp]
    lib.hk_attn_bwd_varlen.restype = ci
    lib.hk_attn_bwd_cross.argtypes = [vp, vp, vp, vp, vp, vp, vp, vp, vp, ci, ci, ci, ci, ci, ci, vp, ci, cf, ci, ci, vp]
    lib.hk_attn_bwd_cross.restype = ci
    lib.hk_attn_dq_shuffle.argtypes = [vp, vp, ci, ci, ci, ci, ci, vp]
    lib.hk_attn_dq_shuffle.restype = ci
    lib.hk_rotary.argtypes = [vp, vp, vp, vp, ci, ci, ci, ci, ci, ci, vp]
    lib.hk_rotary.restype = ci
    lib.hk_rotary_bnhd.argtypes = [vp, vp, vp, vp, ci, ci, ci, ci, ci, ci, ci, vp]
    lib.hk_rotary_bnhd.restype = ci
    lib.hk_paged_kv_append_rotary.argtypes = [vp, vp, vp, vp, vp, vp, vp, vp, ci, ci, ci, ci, ci, ci, ci, ci, ci, ci, vp]
    lib.hk_paged_kv_append_rotary.restype = ci
    lib.hk_attn_paged_decode_workspace_bytes.argtypes = [ci, ci, ci, ci, ci]
    lib.hk_attn_paged_decode_workspace_bytes.restype = ctypes.c_size_t
    lib.hk_attn_paged_decode.argtypes = [vp, vp, vp, vp, vp, vp, vp, ci, ci, ci, ci, ci, ci, ci, cf, vp,
                                         ctypes.c_size_t, ci, vp]
    lib.hk_attn_paged_decode.restype = ci
    lib.hk_attn_paged_decode_static.argtypes = [vp, vp, vp, vp, vp, vp, vp, ci, ci, ci, ci, ci, ci, ci, cf, ci, vp,
                                                ctypes.POINTER(ci)]
    lib.hk_attn_paged_decode_static.restype = ci
    lib.hk_paged_kv_append.argtypes = [vp, vp, vp, vp, vp, vp, ci, ci, ci, ci, ci, ci, ci, ci, vp]
    lib.hk_paged_kv_append.restype = ci
    lib.hk_last_device_status.argtypes = [ci]
    lib.hk_last_device_status.restype = ci
    lib.hk_selftest_bounded_wait.argtypes = [ci, ctypes.c_uint]
    lib.hk_selftest_bounded_wait.restype = ci
    lib.hk_selftest_fastdiv.argtypes = []
    lib.hk_selftest_fastdiv.restype = ci
    lib.hk_kernel_launch_count.argtypes = []
    lib.hk_kernel_launch_count.restype = ctypes.c_ulonglong
    lib.hk_strerror.argtypes = [ci]
    lib.hk_strerror.restype = ctypes.c_char_p
    lib.hk_last_cuda_error.argtypes = []
    lib.hk_last_cuda_error.restype = ctypes.c_char_p
    _capi = lib
    return lib


def _check(rc: int, what: str) -> None:
    if rc != HK_OK:
        lib = capi()
        detail = lib.hk_strerror(rc).decode()
        extra = lib.hk_last_cuda_error().decode()
        if extra and rc in (HK_ECUDA, HK_EUNSUPPORTED):
            detail += "; " + extra
        raise HkError(rc, what, detail)


def kernel_launch_count() -> int:
    return int(capi().hk_kernel_launch_count())


def _require_cuda_bf16(name: str, t: torch.Tensor, ndim: int) -> None:
    if not isinstance(t, torch.Tensor):
        raise RuntimeError("Expected a torch.Tensor")
    if not t.is_contiguous():
        raise RuntimeError("Tensor must be contiguous")
    if t.device.type != "cuda":
        raise RuntimeError("Tensor must be on CUDA device")
    if t.dim() != ndim:
        raise RuntimeError(f"{name} must have {ndim} dimensions, got {t.dim()}")


def _require_same_device(ref: torch.Tensor, **tensors) -> None:
    """Every pointer handed to the library must be device memory on the device the call names; a CPU tensor's
    pointer would be dereferenced by a kernel."""
    for name, t in tensors.items():
        if t is None:
            continue
        if not isinstance(t, torch.Tensor) or t.device != ref.device:
            raise RuntimeError(f"{name} must be a tensor on {ref.device} (got "
                               f"{t.device if isinstance(t, torch.Tensor) else type(t).__name__})")


def attn_fwd(
    q: torch.Tensor,
    k: torch.Tensor,
    v: torch.Tensor,
    causal: bool = False,
    softmax_scale: Optional[float] = None,
    out: Optional[torch.Tensor] = None,
    lse: Optional[torch.Tensor] = None,
    stream: Optional[torch.cuda.Stream] = None,
    kv_lens: Optional[torch.Tensor] = None,
) -> Tuple[torch.Tensor, torch.Tensor]:
    """O = softmax(scale q k^T) v and L = logsumexp(scale q k^T) on the GPU.

    q [B,N,H,D] bf16, k/v [B,Nk,H_KV,D] bf16 CUDA tensors (Nk may differ from N), contiguous or strided views with
    a contiguous last dimension (e.g. slices of a packed qkv projection; no copy is made); returns O [B,N,H,D] bf16
    and L [B,H,1,N] fp32 (the layouts of kernels/attn/gqa/test_python.py:97-98). Asynchronous on `stream`
    (default: torch's current stream). `kv_lens` (int32 [B]) restricts batch element b to its first kv_lens[b]
    keys, the reference's key_padding_mask (base.py:97-103). With `causal`, query row r sees keys up to
    r + (kv_len_b - N): the mask is aligned to the last query and the last kept key as in base.py:104-116; a row
    that sees no key gets O = 0 and L = -inf.
    """
    strided = not (q.is_contiguous() and k.is_contiguous() and v.is_contiguous())
    for name, t in (("q", q), ("k", k), ("v", v)):
        if strided:
            if not isinstance(t, torch.Tensor) or t.device.type != "cuda" or t.dim() != 4:
                raise RuntimeError(f"{name} must be a 4-D CUDA tensor")
            if t.stride(3) != 1 or any(st <= 0 or st % 8 for st in t.stride()[:3]):
                raise RuntimeError(f"{name}: the last dimension must be contiguous and the other strides positive "
                                   "multiples of 8 elements")
        else:
            _require_cuda_bf16(name, t, 4)
        if t.dtype != torch.bfloat16:
            raise RuntimeError(f"{name} must be torch.bfloat16")
    b, n, h, d = q.shape
    hkv = k.shape[2]
    nk = k.shape[1]
    if k.shape != v.shape or k.shape[0] != b or k.shape[3] != d:
        raise RuntimeError("k/v must be [B, Nk, H_KV, D] matching q's batch and head dimension")
    if out is None:
        out = torch.empty((b, n, h, d), dtype=torch.bfloat16, device=q.device)
    if lse is None:
        lse = torch.empty((b, h, 1, n), dtype=torch.float32, device=q.device)
    if out.shape != q.shape or out.dtype != torch.bfloat16 or not out.is_contiguous():
        raise RuntimeError("out must be a contiguous bf16 tensor of q's shape")
    if lse.shape != (b, h, 1, n) or lse.dtype != torch.float32 or not lse.is_contiguous():
        raise RuntimeError("lse must be a contiguous fp32 tensor [B, H, 1, N]")
    _require_same_device(q, k=k, v=v, out=out, lse=lse)
    s = stream if stream is not None else torch.cuda.current_stream(q.device)
    if kv_lens is not None or nk != n:
        if kv_lens is not None and (kv_lens.dtype != torch.int32 or kv_lens.shape != (b,) or kv_lens.device != q.device):
            raise RuntimeError("kv_lens must be an int32 tensor [B] on q's device")
        arr = lambda t: (ctypes.c_longlong * 3)(*t.stride()[:3])  # noqa: E731
        rc = capi().hk_attn_fwd_cross(q.data_ptr(), k.data_ptr(), v.data_ptr(), out.data_ptr(), lse.data_ptr(),
                                      b, n, nk, h, hkv, d, arr(q), arr(k), arr(v),
                                      kv_lens.data_ptr() if kv_lens is not None else None,
                                      int(bool(causal)), float(softmax_scale or 0.0), q.device.index, s.cuda_stream)
    elif strided:
        arr = lambda t: (ctypes.c_longlong * 3)(*t.stride()[:3])  # noqa: E731
        rc = capi().hk_attn_fwd_strided(q.data_ptr(), k.data_ptr(), v.data_ptr(), out.data_ptr(), lse.data_ptr(),
                                        b, n, h, hkv, d, arr(q), arr(k), arr(v), int(bool(causal)),
                                        float(softmax_scale or 0.0), q.device.index, s.cuda_stream)
    else:
        rc = capi().hk_attn_fwd(q.data_ptr(), k.data_ptr(), v.data_ptr(), out.data_ptr(), lse.data_ptr(),
                                b, n, h, hkv, d, int(bool(causal)), float(softmax_scale or 0.0),
                                q.device.index, s.cuda_stream)
    _check(rc, "hk_attn_fwd")
    return out, lse


HK_DQ_BNHD, HK_DQ_BHND = 0, 1


def attn_bwd_prep(o: torch.Tensor, d_o: torch.Tensor, delta: Optional[torch.Tensor] = None,
                  stream: Optional[torch.cuda.Stream] = None) -> torch.Tensor:
    """delta [B,H,1,N] fp32 = rowsum(O * dO) for O, dO [B,N,H,D] bf16 (the reference's ``dispatch_prep``,
    kernels/attn/gqa_backwards/attn_bkwd_prep.cpp:164-195)."""
    for name, t in (("o", o), ("d_o", d_o)):
        _require_cuda_bf16(name, t, 4)
        if t.dtype != torch.bfloat16:
            raise RuntimeError(f"{name} must be torch.bfloat16")
    if o.shape != d_o.shape:
        raise RuntimeError("o and d_o must have the same shape")
    b, n, h, d = o.shape
    if delta is None:
        delta = torch.empty((b, h, 1, n), dtype=torch.float32, device=o.device)
    if delta.shape != (b, h, 1, n) or delta.dtype != torch.float32 or not delta.is_contiguous():
        raise RuntimeError("delta must be a contiguous fp32 tensor [B, H, 1, N]")
    _require_same_device(o, d_o=d_o, delta=delta)
    s = stream if stream is not None else torch.cuda.current_stream(o.device)
    _check(capi().hk_attn_bwd_prep(o.data_ptr(), d_o.data_ptr(), delta.data_ptr(), b, n, h, d, o.device.index,
                                   s.cuda_stream), "hk_attn_bwd_prep")
    return delta


def attn_bwd(
    q: torch.Tensor,
    k: torch.Tensor,
    v: torch.Tensor,
    d_o: torch.Tensor,
    lse: torch.Tensor,
    delta: torch.Tensor,
    causal: bool = False,
    softmax_scale: Optional[float] = None,
    dq: Optional[torch.Tensor] = None,
    dk: Optional[torch.Tensor] = None,
    dv: Optional[torch.Tensor] = None,
    dq_layout: int = HK_DQ_BNHD,
    stream: Optional[torch.cuda.Stream] = None,
    kv_lens: Optional[torch.Tensor] = None,
) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    """dQ, dK, dV of the attention forward (the reference's ``dispatch_bwd_combined``,
    kernels/attn/gqa_backwards/attn_bkwd_non_causal.cpp:37-49). q, d_o [B,N,H,D], k, v [B,Nk,H_KV,D] bf16 (Nk may
    differ from N); lse, delta [B,H,1,N] fp32. dQ comes back as [B,N,H,D], or [B,H,N,D] with
    ``dq_layout=HK_DQ_BHND`` (the reference's pre-shuffle layout). Any N, Nk >= 1. `kv_lens` (int32 [B]) and `causal`
    mean what they mean in ``attn_fwd``: dK and dV rows of keys nobody sees come back as zeros."""
    for name, t in (("q", q), ("k", k), ("v", v), ("d_o", d_o)):
        _require_cuda_bf16(name, t, 4)
        if t.dtype != torch.bfloat16:
            raise RuntimeError(f"{name} must be torch.bfloat16")
    b, n, h, d = q.shape
    hkv = k.shape[2]
    nk = k.shape[1]
    if k.shape != v.shape or k.shape[0] != b or k.shape[3] != d or d_o.shape != q.shape:
        raise RuntimeError("k/v must be [B, Nk, H_KV, D] and d_o [B, N, H, D] matching q")
    for name, t in (("lse", lse), ("delta", delta)):
        if t.shape != (b, h, 1, n) or t.dtype != torch.float32 or not t.is_contiguous() or t.device != q.device:
            raise RuntimeError(f"{name} must be a contiguous fp32 tensor [B, H, 1, N] on q's device")
    dq_shape = (b, n, h, d) if dq_layout == HK_DQ_BNHD else (b, h, n, d)
    if dq is None:
        dq = torch.empty(dq_shape, dtype=torch.bfloat16, device=q.device)
    if dk is None:
        dk = torch.empty_like(k)
    if dv is None:
        dv = torch.empty_like(v)
    for name, t, shp in (("dq", dq, dq_shape), ("dk", dk, tuple(k.shape)), ("dv", dv, tuple(v.shape))):
        if tuple(t.shape) != tuple(shp) or t.dtype != torch.bfloat16 or not t.is_contiguous():
            raise RuntimeError(f"{name} must be a contiguous bf16 tensor of shape {tuple(shp)}")
    _require_same_device(q, k=k, v=v, d_o=d_o, dq=dq, dk=dk, dv=dv)
    s = stream if stream is not None else torch.cuda.current_stream(q.device)
    if kv_lens is not None and (kv_lens.dtype != torch.int32 or kv_lens.shape != (b,) or kv_lens.device != q.device):
        raise RuntimeError("kv_lens must be an int32 tensor [B] on q's device")
    rc = capi().hk_attn_bwd_cross(q.data_ptr(), k.data_ptr(), v.data_ptr(), d_o.data_ptr(), lse.data_ptr(),
                                  delta.data_ptr(), dq.data_ptr(), dk.data_ptr(), dv.data_ptr(), b, n, nk, h, hkv, d,
                                  kv_lens.data_ptr() if kv_lens is not None else None,
                                   int(bool(causal)), float(softmax_scale or 0.0), int(dq_layout), q.device.index,
                                   s.cuda_stream)
    _check(rc, "hk_attn_bwd")
    return dq, dk, dv


def dq_shuffle(dq_bhnd: torch.Tensor, dq_bnhd: Optional[torch.Tensor] = None,
               stream: Optional[torch.cuda.Stream] = None) -> torch.Tensor:
    """[B,H,N,D] -> [B,N,H,D] (the reference's ``dispatch_dq_shuffle``, attn_bkwd_prep.cpp:199-223)."""
    _require_cuda_bf16("dq_bhnd", dq_bhnd, 4)
    b, h, n, d = dq_bhnd.shape
    if dq_bnhd is None:
        dq_bnhd = torch.empty((b, n, h, d), dtype=dq_bhnd.dtype, device=dq_bhnd.device)
    if dq_bnhd.shape != (b, n, h, d) or dq_bnhd.dtype != dq_bhnd.dtype or not dq_bnhd.is_contiguous():
        raise RuntimeError("dq_bnhd must be a contiguous tensor [B, N, H, D] of the source's dtype")
    if dq_bhnd.dtype != torch.bfloat16:
        raise RuntimeError("dq_bhnd must be torch.bfloat16")
    _require_same_device(dq_bhnd, dq_bnhd=dq_bnhd)
    s = stream if stream is not None else torch.cuda.current_stream(dq_bhnd.device)
    _check(capi().hk_attn_dq_shuffle(dq_bhnd.data_ptr(), dq_bnhd.data_ptr(), b, n, h, d, dq_bhnd.device.index,
                                     s.cuda_stream), "hk_attn_dq_shuffle")
    return dq_bnhd


def rotary(x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor, out: Optional[torch.Tensor] = None,
           stream: Optional[torch.cuda.Stream] = None) -> torch.Tensor:
    """Rotary embedding of x [B,H,N,D] bf16 with cos, sin [N, R/2] bf16 (R <= D, the rest passes through): the
    reference's ``tk_kernel.dispatch_rotary`` (kernels/rotary/kernel.cpp:44-98). `out` may be `x` itself."""
    for name, t in (("x", x), ("cos", cos), ("sin", sin)):
        if not isinstance(t, torch.Tensor):
            raise RuntimeError("Expected a torch.Tensor")
        if not t.is_contiguous():
            raise RuntimeError("Tensor must be contiguous")
        if t.device.type != "cuda":
            raise RuntimeError("Tensor must be on CUDA device")
        if t.dtype != torch.bfloat16:
            raise RuntimeError(f"{name} must be torch.bfloat16")
    if x.dim() != 4 or cos.dim() != 2 or cos.shape != sin.shape or cos.shape[0] != x.shape[2]:
        raise RuntimeError("x must be [B,H,N,D] and cos/sin [N, R/2]")
    b, h, n, d = x.shape
    if out is None:
        out = torch.empty_like(x)
    if out.shape != x.shape or out.dtype != x.dtype or not out.is_contiguous():
        raise RuntimeError("out must be a contiguous bf16 tensor of x's shape")
    _require_same_device(x, cos=cos, sin=sin, out=out)
    s = stream if stream is not None else torch.cuda.current_stream(x.device)
    _check(capi().hk_rotary(x.data_ptr(), out.data_ptr(), sin.data_ptr(), cos.data_ptr(), b, h, n, d,
                            2 * cos.shape[1], x.device.index, s.cuda_stream), "hk_rotary")
    return out


def rotary_bnhd(x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor, out: Optional[torch.Tensor] = None,
                pos_offset: int = 0, stream: Optional[torch.cuda.Stream] = None) -> torch.Tensor:
    """Rotary embedding of x [B,N,H,D] bf16 (the attention entries' layout) with cos, sin [>= N + pos_offset, R/2]
    bf16; row n of the sequence uses table row n + pos_offset. `out` may be `x` itself."""
    for name, t in (("x", x), ("cos", cos), ("sin", sin)):
        if not isinstance(t, torch.Tensor) or not t.is_contiguous() or t.device.type != "cuda" or t.dtype != torch.bfloat16:
            raise RuntimeError(f"{name} must be a contiguous bf16 CUDA tensor")
    if x.dim() != 4 or cos.dim() != 2 or cos.shape != sin.shape or cos.shape[0] < x.shape[1] + pos_offset or pos_offset < 0:
        raise RuntimeError("x must be [B,N,H,D] and cos/sin [>= N + pos_offset, R/2]")
    b, n, h, d = x.shape
    if out is None:
        out = torch.empty_like(x)
    if out.shape != x.shape or out.dtype != x.dtype or not out.is_contiguous():
        raise RuntimeError("out must be a contiguous bf16 tensor of x's shape")
    _require_same_device(x, cos=cos, sin=sin, out=out)
    s = stream if stream is not None else torch.cuda.current_stream(x.device)
    _check(capi().hk_rotary_bnhd(x.data_ptr(), out.data_ptr(), sin.data_ptr(), cos.data_ptr(), b, n, h, d,
                                 2 * cos.shape[1], int(pos_offset), x.device.index, s.cuda_stream), "hk_rotary_bnhd")
    return out


def paged_decode_workspace_bytes(s: int, h: int, d: int, max_pages: int, page_size: int = 16) -> int:
    return int(capi().hk_attn_paged_decode_workspace_bytes(s, h, d, max_pages, page_size))


def paged_decode(
    q: torch.Tensor,
    k_pages: torch.Tensor,
    v_pages: torch.Tensor,
    block_table: torch.Tensor,
    ctx_lens: torch.Tensor,
    softmax_scale: Optional[float] = None,
    out: Optional[torch.Tensor] = None,
    lse: Optional[torch.Tensor] = None,
    workspace: Optional[torch.Tensor] = None,
    stream: Optional[torch.cuda.Stream] = None,
) -> Tuple[torch.Tensor, torch.Tensor]:
    """Paged-KV decode: q [S,1,H,D] bf16, pages [P,16,H_KV,D] bf16, block_table [S,max_pages] int32,
    ctx_lens [S] int32 -> O [S,1,H,D] bf16, L [S,H,1,1] fp32. `workspace` is a uint8 CUDA tensor of at
    least ``paged_decode_workspace_bytes(...)`` bytes (allocated here when omitted)."""
    for name, t in (("q", q), ("k_pages", k_pages), ("v_pages", v_pages)):
        _require_cuda_bf16(name, t, 4)
        if t.dtype != torch.bfloat16:
            raise RuntimeError(f"{name} must be torch.bfloat16")
    if block_table.dtype != torch.int32 or ctx_lens.dtype != torch.int32:
        raise RuntimeError("block_table and ctx_lens must be torch.int32")
    if not (block_table.is_contiguous() and ctx_lens.is_contiguous()):
        raise RuntimeError("Tensor must be contiguous")
    s_n, one, h, d = q.shape
    p_n, page, hkv, d2 = k_pages.shape
    if one != 1 or d2 != d or v_pages.shape != k_pages.shape:
        raise RuntimeError("q must be [S,1,H,D] and k_pages/v_pages [P,page,H_KV,D]")
    if block_table.dim() != 2 or block_table.shape[0] != s_n or ctx_lens.shape != (s_n,):
        raise RuntimeError("block_table must be [S, max_pages] and ctx_lens [S]")
    max_pages = block_table.shape[1]
    if out is None:
        out = torch.empty_like(q)
    if lse is None:
        lse = torch.empty((s_n, h, 1, 1), dtype=torch.float32, device=q.device)
    need = paged_decode_workspace_bytes(s_n, h, d, max_pages, page)
    if need == 0:
        raise HkError(HK_EUNSUPPORTED, "hk_attn_paged_decode",
                      "shape outside the decode kernels' limits (D = 128, 16-token pages, S <= 65535, "
                      "max_pages <= 8192)")
    if workspace is None:
        workspace = torch.empty(max(need, 256), dtype=torch.uint8, device=q.device)
    _require_same_device(q, k_pages=k_pages, v_pages=v_pages, block_table=block_table, ctx_lens=ctx_lens, out=out,
                         lse=lse, workspace=workspace)
    st = stream if stream is not None else torch.cuda.current_stream(q.device)
    rc = capi().hk_attn_paged_decode(q.data_ptr(), k_pages.data_ptr(), v_pages.data_ptr(),
                                     block_table.data_ptr(), ctx_lens.data_ptr(), out.data_ptr(), lse.data_ptr(),
                                     s_n, h, hkv, d, page, max_pages, p_n, float(softmax_scale or 0.0),
                                     workspace.data_ptr(), workspace.numel(), q.device.index, st.cuda_stream)
    _check(rc, "hk_attn_paged_decode")
    return out, lse


def attn_fwd_paged(
    q: torch.Tensor,
    k_pages: torch.Tensor,
    v_pages: torch.Tensor,
    block_table: torch.Tensor,
    ctx_lens: torch.Tensor,
    causal: bool = True,
    softmax_scale: Optional[float] = None,
    out: Optional[torch.Tensor] = None,
    lse: Optional[torch.Tensor] = None,
    stream: Optional[torch.cuda.Stream] = None,
) -> Tuple[torch.Tensor, torch.Tensor]:
    """Chunked prefill against the paged KV cache: q [S,T,H,D] bf16 (the last T tokens of each context when `causal`),
    pages [P,16,H_KV,D] bf16, block_table [S,max_pages] int32, ctx_lens [S] int32 -> O [S,T,H,D] bf16,
    L [S,H,1,T] fp32. The chunk's keys must already be in the cache (`paged_kv_append` first)."""
    for name, t in (("q", q), ("k_pages", k_pages), ("v_pages", v_pages)):
        _require_cuda_bf16(name, t, 4)
        if t.dtype != torch.bfloat16:
            raise RuntimeError(f"{name} must be torch.bfloat16")
    if block_table.dtype != torch.int32 or ctx_lens.dtype != torch.int32:
        raise RuntimeError("block_table and ctx_lens must be torch.int32")
    if not (block_table.is_contiguous() and ctx_lens.is_contiguous()):
        raise RuntimeError("Tensor must be contiguous")
    s_n, t_n, h, d = q.shape
    p_n, page, hkv, d2 = k_pages.shape
    if d2 != d or v_pages.shape != k_pages.shape:
        raise RuntimeError("q must be [S,T,H,D] and k_pages/v_pages [P,page,H_KV,D]")
    if block_table.dim() != 2 or block_table.shape[0] != s_n or ctx_lens.shape != (s_n,):
        raise RuntimeError("block_table must be [S, max_pages] and ctx_lens [S]")
    if out is None:
        out = torch.empty_like(q)
    if lse is None:
        lse = torch.empty((s_n, h, 1, t_n), dtype=torch.float32, device=q.device)
    if out.shape != q.shape or out.dtype != torch.bfloat16 or not out.is_contiguous():
        raise RuntimeError("out must be a contiguous bf16 tensor of q's shape")
    if lse.shape != (s_n, h, 1, t_n) or lse.dtype != torch.float32 or not lse.is_contiguous():
        raise RuntimeError("lse must be a contiguous fp32 tensor [S, H, 1, T]")
    _require_same_device(q, k_pages=k_pages, v_pages=v_pages, block_table=block_table, ctx_lens=ctx_lens, out=out,
                         lse=lse)
    st = stream if stream is not None else torch.cuda.current_stream(q.device)
    rc = capi().hk_attn_fwd_paged(q.data_ptr(), k_pages.data_ptr(), v_pages.data_ptr(), block_table.data_ptr(),
                                  ctx_lens.data_ptr(), out.data_ptr(), lse.data_ptr(), s_n, t_n, h, hkv, d, page,
                                  block_table.shape[1], p_n, int(bool(causal)), float(softmax_scale or 0.0),
                                  q.device.index, st.cuda_stream)
    _check(rc, "hk_attn_fwd_paged")
    return out, lse


def paged_kv_append(
    k_new: torch.Tensor,
    v_new: torch.Tensor,
    k_pages: torch.Tensor,
    v_pages: torch.Tensor,
    block_table: torch.Tensor,
    start_pos: torch.Tensor,
    stream: Optional[torch.cuda.Stream] = None,
) -> None:
    """Write k_new/v_new [S,T,H_KV,D] into the page pools at positions start_pos[s] .. start_pos[s]+T-1 of each
    sequence (the paged form of the reference's `_update_kv_cache`, training/llama/llama/models/mha.py:16-42)."""
    for name, t in (("k_new", k_new), ("v_new", v_new), ("k_pages", k_pages), ("v_pages", v_pages)):
        _require_cuda_bf16(name, t, 4)
        if t.dtype != torch.bfloat16:
            raise RuntimeError(f"{name} must be torch.bfloat16")
    if block_table.dtype != torch.int32 or start_pos.dtype != torch.int32:
        raise RuntimeError("block_table and start_pos must be torch.int32")
    if not (block_table.is_contiguous() and start_pos.is_contiguous()):
        raise RuntimeError("Tensor must be contiguous")
    s_n, t_n, hkv, d = k_new.shape
    p_n, page, hkv2, d2 = k_pages.shape
    if v_new.shape != k_new.shape or v_pages.shape != k_pages.shape or (hkv2, d2) != (hkv, d):
        raise RuntimeError("k_new/v_new must be [S,T,H_KV,D] and k_pages/v_pages [P,page,H_KV,D]")
    if block_table.dim() != 2 or block_table.shape[0] != s_n or start_pos.shape != (s_n,):
        raise RuntimeError("block_table must be [S, max_pages] and start_pos [S]")
    _require_same_device(k_new, v_new=v_new, k_pages=k_pages, v_pages=v_pages, block_table=block_table,
                         start_pos=start_pos)
    st = stream if stream is not None else torch.cuda.current_stream(k_new.device)
    rc = capi().hk_paged_kv_append(k_new.data_ptr(), v_new.data_ptr(), k_pages.data_ptr(), v_pages.data_ptr(),
                                   block_table.data_ptr(), start_pos.data_ptr(), s_n, t_n, hkv, d, page,
                                   block_table.shape[1], p_n, k_new.device.index, st.cuda_stream)
    _check(rc, "hk_paged_kv_append")


def paged_kv_append_rotary(
    k_new: torch.Tensor,
    v_new: torch.Tensor,
    k_pages: torch.Tensor,
    v_pages: torch.Tensor,
    block_table: torch.Tensor,
    start_pos: torch.Tensor,
    cos: torch.Tensor,
    sin: torch.Tensor,
    stream: Optional[torch.cuda.Stream] = None,
) -> None:
    """`paged_kv_append` with the rotary embedding of K applied on the way: token t of sequence s is rotated with row
    start_pos[s] + t of cos / sin [rows, R/2] bf16 (V is copied). The pages end up bit-identical to `rotary_bnhd`
    followed by `paged_kv_append` (the reference's order, mha.py:217-220 then 16-42)."""
    for name, t in (("k_new", k_new), ("v_new", v_new), ("k_pages", k_pages), ("v_pages", v_pages)):
        _require_cuda_bf16(name, t, 4)
        if t.dtype != torch.bfloat16:
            raise RuntimeError(f"{name} must be torch.bfloat16")
    for name, t in (("cos", cos), ("sin", sin)):
        if not t.is_contiguous() or t.dtype != torch.bfloat16 or t.dim() != 2:
            raise RuntimeError(f"{name} must be a contiguous bf16 tensor [rows, R/2]")
    if cos.shape != sin.shape:
        raise RuntimeError("cos and sin must have the same shape")
    if block_table.dtype != torch.int32 or start_pos.dtype != torch.int32:
        raise RuntimeError("block_table and start_pos must be torch.int32")
    if not (block_table.is_contiguous() and start_pos.is_contiguous()):
        raise RuntimeError("Tensor must be contiguous")
    s_n, t_n, hkv, d = k_new.shape
    p_n, page, hkv2, d2 = k_pages.shape
    if v_new.shape != k_new.shape or v_pages.shape != k_pages.shape or (hkv2, d2) != (hkv, d):
        raise RuntimeError("k_new/v_new must be [S,T,H_KV,D] and k_pages/v_pages [P,page,H_KV,D]")
    if block_table.dim() != 2 or block_table.shape[0] != s_n or start_pos.shape != (s_n,):
        raise RuntimeError("block_table must be [S, max_pages] and start_pos [S]")
    _require_same_device(k_new, v_new=v_new, k_pages=k_pages, v_pages=v_pages, block_table=block_table,
                         start_pos=start_pos, cos=cos, sin=sin)
    st = stream if stream is not None else torch.cuda.current_stream(k_new.device)
    rc = capi().hk_paged_kv_append_rotary(k_new.data_ptr(), v_new.data_ptr(), k_pages.data_ptr(), v_pages.data_ptr(),
                                          block_table.data_ptr(), start_pos.data_ptr(), sin.data_ptr(), cos.data_ptr(),
                                          s_n, t_n, hkv, d, 2 * cos.shape[1], cos.shape[0], page, block_table.shape[1],
                                          p_n, k_new.device.index, st.cuda_stream)
    _check(rc, "hk_paged_kv_append_rotary")


def device_status(device: int = 0) -> int:
    """Synchronise `device` and return the kernels' status word as an HK_* code (0 = OK)."""
    return int(capi().hk_last_device_status(device))


def _load_ext(subdir: str, module: str):
    path = os.path.join(_PKG, subdir, module + sysconfig.get_config_var("EXT_SUFFIX"))
    if not os.path.exists(path):
        raise ImportError(f"{path} is missing: build it with `python -m hipkittens_b200._build`")
    # The dotted name keeps the two same-named builds (causal / non-causal) apart inside one process;
    # from its own directory each is still importable as plain `tk_kernel`, as in the reference.
    full = "hipkittens_b200." + subdir.replace("/", ".") + "." + module
    if full in sys.modules:
        return sys.modules[full]
    spec = importlib.util.spec_from_file_location(full, path)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    sys.modules[full] = mod
    return mod


def load_tk_kernel(causal: bool = False):
    """The ``tk_kernel`` module of kernels/attn/gqa (or gqa_causal): ``dispatch_micro(q,k,v,out,lse)``."""
    return _load_ext("kernels/attn/gqa_causal" if causal else "kernels/attn/gqa", "tk_kernel")


def load_tk_kernel_fwd(causal: bool = True):
    """The ``tk_kernel_fwd`` module of the training call site: blocking ``dispatch_fwd(q,k,v,O,L)``."""
    return _load_ext("kernels/attn/gqa_causal_backwards" if causal else "kernels/attn/gqa_backwards",
                     "tk_kernel_fwd")


def load_tk_kernel_bkwd(causal: bool = True):
    """The ``tk_kernel_bkwd`` module of kernels/attn/gqa_backwards (or gqa_causal_backwards):
    blocking ``dispatch_bwd_combined(Q, K, V, dO, dQ_in, dK, dV, L, delta)``."""
    return _load_ext("kernels/attn/gqa_causal_backwards" if causal else "kernels/attn/gqa_backwards",
                     "tk_kernel_bkwd")


def load_tk_kernel_bkwd_prep(causal: bool = True):
    """The ``tk_kernel_bkwd_prep`` module: blocking ``dispatch_prep(O, dO, delta)`` and
    ``dispatch_dq_shuffle(dQ_in, dQ)``. (Both builds are identical; `causal` only picks the directory.)"""
    return _load_ext("kernels/attn/gqa_causal_backwards" if causal else "kernels/attn/gqa_backwards",
                     "tk_kernel_bkwd_prep")


def load_tk_kernel_rotary():
    """The ``tk_kernel`` module of kernels/rotary: ``dispatch_rotary(x, o, sin, cos)``."""
    return _load_ext("kernels/rotary", "tk_kernel")
