"""Host-side mirror of the reference's attention call site (forward and backward).

``HipAttnFunction`` / ``HipSelfAttention`` / ``HipCrossAttention`` follow
``training/llama/llama/models/attentions/hipkittens.py:17-61,122-202``: inputs and outputs are BNHD,
q/k/v are cast to bf16 and made contiguous, O [B,N,H,D] bf16 and L [B,H,1,N] fp32 are allocated by the
caller side and filled by the blocking ``tk_kernel_fwd.dispatch_fwd(q, k, v, O, L)``; O is returned in the
input dtype and (q, k, v, O, L) are saved for the backward pass, which runs the reference's three calls
(hipkittens.py:64-119): ``dispatch_prep(O, dO, delta)``, ``dispatch_bwd_combined(q, k, v, dO, dQ_in, dK, dV,
L, delta)`` and ``dispatch_dq_shuffle(dQ_in, dQ)``.

Differences: dQ_in is not zero-filled (nothing is accumulated into it); a right-padded ``key_padding_mask``
(True = keep, as in ``base.py:88-103``) is honoured through per-batch key lengths, also together with ``causal``
and with more keys than queries (``base.py:104-116``), where the reference's modules accept the argument and ignore
it (hipkittens.py:147-162); and causality and the softmax scale are honoured here (they are baked into the reference's compiled module, and its modules
ignore the ``causal`` and ``softmax_scale`` they are constructed with, hipkittens.py:147-162).
"""
from __future__ import annotations

import torch
import torch.nn as nn
from torch.autograd import Function

from ._native import (
    attn_bwd,
    attn_bwd_prep,
    attn_fwd,
    device_status,
    load_tk_kernel_bkwd,
    load_tk_kernel_bkwd_prep,
    load_tk_kernel_fwd,
)

_fwd_modules = {}
_bkwd_modules = {}


def _tk_kernel_bkwd(causal: bool):
    if causal not in _bkwd_modules:
        _bkwd_modules[causal] = (load_tk_kernel_bkwd(causal), load_tk_kernel_bkwd_prep(causal))
    return _bkwd_modules[causal]


def _tk_kernel_fwd(causal: bool):
    if causal not in _fwd_modules:
        _fwd_modules[causal] = load_tk_kernel_fwd(causal)
    return _fwd_modules[causal]


def _tma_viewable(t: torch.Tensor) -> bool:
    """bf16, last dimension contiguous, other strides positive multiples of 8 elements (16 bytes)."""
    return (t.dtype == torch.bfloat16 and t.dim() == 4 and t.stride(3) == 1
            and all(st > 0 and st % 8 == 0 for st in t.stride()[:3]))


class HipAttnFunction(Function):
    @staticmethod
    def forward(ctx, q_bnhd: torch.Tensor, k_bnhd: torch.Tensor, v_bnhd: torch.Tensor, causal: bool = True,
                softmax_scale=None, kv_lens=None):
        B, N, H, D = q_bnhd.shape
        HKV, NK = k_bnhd.shape[2], k_bnhd.shape[1]
        dev = q_bnhd.device
        out_dtype = q_bnhd.dtype
        assert k_bnhd.shape == (B, NK, HKV, D), f"K shape mismatch: expected ({B}, {NK}, {HKV}, {D}), got {k_bnhd.shape}"
        assert v_bnhd.shape == (B, NK, HKV, D), f"V shape mismatch: expected ({B}, {NK}, {HKV}, {D}), got {v_bnhd.shape}"
        assert q_bnhd.is_cuda and k_bnhd.is_cuda and v_bnhd.is_cuda, "All tensors must be on CUDA device"
        assert q_bnhd.device == k_bnhd.device == v_bnhd.device, "All tensors must be on same device"
        assert H % HKV == 0, f"H ({H}) must be divisible by HKV ({HKV}) for GQA"

        O = torch.empty((B, N, H, D), dtype=torch.bfloat16, device=dev)
        L = torch.empty((B, H, 1, N), dtype=torch.float32, device=dev)
        ctx.general = kv_lens is not None or NK != N  # cases the reference's compiled modules have no entry for
        if ctx.general or (all(_tma_viewable(t) for t in (q_bnhd, k_bnhd, v_bnhd)) and not all(
                t.is_contiguous() for t in (q_bnhd, k_bnhd, v_bnhd))):
            # bf16 views of a packed projection (what qkv.unbind(2) gives): the kernel reads them through
            # strided TMA descriptors, so the reference's three .contiguous() copies (hipkittens.py:37-39) go
            # (key lengths go the same way: the reference's dispatch_fwd has no argument for them)
            if all(_tma_viewable(t) for t in (q_bnhd, k_bnhd, v_bnhd)):
                q, k, v = q_bnhd, k_bnhd, v_bnhd
            else:
                q, k, v = (t.to(torch.bfloat16).contiguous() for t in (q_bnhd, k_bnhd, v_bnhd))
            attn_fwd(q, k, v, causal=bool(causal), softmax_scale=softmax_scale, out=O, lse=L, kv_lens=kv_lens)
            status = device_status(dev.index)  # blocks on the device like dispatch_fwd does
            if status != 0:
                raise RuntimeError(f"attention forward failed on the device (status {status})")
        else:
            q = q_bnhd.to(torch.bfloat16).contiguous()
            k = k_bnhd.to(torch.bfloat16).contiguous()
            v = v_bnhd.to(torch.bfloat16).contiguous()
            _tk_kernel_fwd(bool(causal)).dispatch_fwd(q, k, v, O, L, softmax_scale=softmax_scale)

        ctx.save_for_backward(q, k, v, O, L)
        ctx.causal = bool(causal)
        ctx.softmax_scale = softmax_scale
        ctx.kv_lens = kv_lens
        return O.to(out_dtype)

    @staticmethod
    def backward(ctx, dO_bnhd: torch.Tensor):
        q, k, v, O, L = ctx.saved_tensors
        B, N, H, D = O.shape
        HKV = k.shape[2]
        dev = dO_bnhd.device
        assert dO_bnhd.shape == (B, N, H, D), f"dO shape mismatch: expected ({B}, {N}, {H}, {D}), got {dO_bnhd.shape}"
        assert dO_bnhd.is_cuda and dO_bnhd.device == O.device, "dO must be on correct CUDA device"

        # the strided forward path saves views; the backward kernels read contiguous tensors
        q, k, v = q.contiguous(), k.contiguous(), v.contiguous()
        dO = dO_bnhd.to(torch.bfloat16).contiguous()

        dQ_in = torch.empty((B, H, N, D), dtype=torch.bfloat16, device=dev)  # BHND (pre-shuffle)
        dQ = torch.empty((B, N, H, D), dtype=torch.bfloat16, device=dev)
        dK = torch.empty(k.shape, dtype=torch.bfloat16, device=dev)
        dV = torch.empty(v.shape, dtype=torch.bfloat16, device=dev)
        delta = torch.empty((B, H, 1, N), dtype=torch.float32, device=dev)

        if ctx.general:
            # padded batch, or more keys than queries: the C ABI's general entry (no counterpart among the reference's
            # three calls); dQ is written in its final layout, so no shuffle pass
            attn_bwd_prep(O, dO, delta)
            attn_bwd(q, k, v, dO, L, delta, causal=ctx.causal, softmax_scale=ctx.softmax_scale, dq=dQ, dk=dK, dv=dV,
                     kv_lens=ctx.kv_lens)
            status = device_status(dev.index)
            if status != 0:
                raise RuntimeError(f"attention backward failed on the device (status {status})")
            return dQ.to(dO_bnhd.dtype), dK.to(dO_bnhd.dtype), dV.to(dO_bnhd.dtype), None, None, None

        tk_kernel_bkwd, tk_kernel_bkwd_prep = _tk_kernel_bkwd(ctx.causal)
        tk_kernel_bkwd_prep.dispatch_prep(O, dO, delta)
        tk_kernel_bkwd.dispatch_bwd_combined(q, k, v, dO, dQ_in, dK, dV, L, delta, causal=ctx.causal,
                                             softmax_scale=ctx.softmax_scale)
        tk_kernel_bkwd_prep.dispatch_dq_shuffle(dQ_in, dQ)

        return dQ.to(dO_bnhd.dtype), dK.to(dO_bnhd.dtype), dV.to(dO_bnhd.dtype), None, None, None


def _lens_from_key_padding_mask(mask: torch.Tensor, seqlen: int):
    """(B, S) bool, True = keep (base.py:88-89) -> int32 key lengths, for masks that keep a prefix of each row
    (right padding, what padded batches have). Anything else cannot be expressed as lengths and is refused."""
    if mask.dim() != 2 or mask.shape[1] != seqlen or mask.dtype != torch.bool:
        raise ValueError("key_padding_mask must be a bool tensor (batch, seqlen), True = keep")
    lens = mask.sum(dim=1).to(torch.int32)
    prefix = torch.arange(seqlen, device=mask.device).unsqueeze(0) < lens.unsqueeze(1)
    if not bool((mask == prefix).all()) or bool((lens < 1).any()):
        raise ValueError("only right-padded key_padding_mask (a kept prefix of at least one key per row) is supported")
    return lens.contiguous()


class HipSelfAttention(nn.Module):
    """qkv [B, S, 3, H, D] -> [B, S, H, D] (hipkittens.py:122-162). Same constructor as the reference;
    `causal` and `softmax_scale` take effect here, dropout is not applied (the reference builds an
    nn.Dropout but never calls it, hipkittens.py:141,158-161)."""

    def __init__(self, causal=False, softmax_scale=None, attention_dropout=0.0, deterministic=False):
        super().__init__()
        self.causal = causal
        self.softmax_scale = softmax_scale
        self.drop = nn.Dropout(attention_dropout)
        self.deterministic = deterministic

    def forward(self, qkv, causal=None, key_padding_mask=None):
        assert qkv.dtype in [torch.float16, torch.bfloat16]
        assert qkv.is_cuda
        causal = self.causal if causal is None else causal
        kv_lens = None
        if key_padding_mask is not None:
            kv_lens = _lens_from_key_padding_mask(key_padding_mask, qkv.shape[1])
        q, k, v = qkv.unbind(dim=2)
        out_bnhd = HipAttnFunction.apply(q, k, v, causal, self.softmax_scale, kv_lens)
        return out_bnhd.to(q.dtype).contiguous()


class HipCrossAttention(nn.Module):
    """q [B, Sq, H, D], kv [B, Sk, 2, H_KV, D] -> [B, Sq, H, D] (hipkittens.py:165-202). Sq may differ from Sk and
    `causal` may be combined with a right-padded `key_padding_mask`, with the reference math path's alignment of the
    causal mask to the last query and the last kept key (base.py:104-116)."""

    def __init__(self, causal=False, softmax_scale=None, attention_dropout=0.0, deterministic=False):
        super().__init__()
        self.causal = causal
        self.softmax_scale = softmax_scale
        self.drop = nn.Dropout(attention_dropout)
        self.deterministic = deterministic

    def forward(self, q, kv, causal=None, key_padding_mask=None):
        batch_size = q.shape[0]
        causal = self.causal if causal is None else causal
        assert kv.shape[0] == batch_size and kv.shape[4] == q.shape[3]
        kv_lens = None
        if key_padding_mask is not None:
            kv_lens = _lens_from_key_padding_mask(key_padding_mask, kv.shape[1])
        k, v = kv.unbind(dim=2)
        out_bnhd = HipAttnFunction.apply(q, k, v, causal, self.softmax_scale, kv_lens)
        return out_bnhd.to(q.dtype).contiguous()
