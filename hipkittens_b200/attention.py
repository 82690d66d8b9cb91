"""Host-side mirror of the reference's attention call site for the forward path.

``HipAttnFunction`` / ``HipSelfAttention`` / ``HipCrossAttention`` follow
``training/llama/llama/models/attentions/hipkittens.py:17-61,122-202``: inputs and outputs are BNHD,
q/k/v are cast to bf16 and made contiguous, O [B,N,H,D] bf16 and L [B,H,1,N] fp32 are allocated by the
caller side and filled by the blocking ``tk_kernel_fwd.dispatch_fwd(q, k, v, O, L)``; O is returned in the
input dtype and (q, k, v, O, L) are saved for a backward pass.

Differences: the backward kernels are not part of this build, so ``backward`` raises; and causality and
the softmax scale are honoured here (they are baked into the reference's compiled module, and its modules
ignore the ``causal`` and ``softmax_scale`` they are constructed with, hipkittens.py:147-162).
"""
from __future__ import annotations

import torch
import torch.nn as nn
from torch.autograd import Function

from ._native import attn_fwd, device_status, load_tk_kernel_fwd

_fwd_modules = {}


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
                softmax_scale=None):
        B, N, H, D = q_bnhd.shape
        HKV = k_bnhd.shape[2]
        dev = q_bnhd.device
        out_dtype = q_bnhd.dtype
        assert k_bnhd.shape == (B, N, HKV, D), f"K shape mismatch: expected ({B}, {N}, {HKV}, {D}), got {k_bnhd.shape}"
        assert v_bnhd.shape == (B, N, HKV, D), f"V shape mismatch: expected ({B}, {N}, {HKV}, {D}), got {v_bnhd.shape}"
        assert q_bnhd.is_cuda and k_bnhd.is_cuda and v_bnhd.is_cuda, "All tensors must be on CUDA device"
        assert q_bnhd.device == k_bnhd.device == v_bnhd.device, "All tensors must be on same device"
        assert H % HKV == 0, f"H ({H}) must be divisible by HKV ({HKV}) for GQA"

        O = torch.empty((B, N, H, D), dtype=torch.bfloat16, device=dev)
        L = torch.empty((B, H, 1, N), dtype=torch.float32, device=dev)
        if all(_tma_viewable(t) for t in (q_bnhd, k_bnhd, v_bnhd)) and not all(
                t.is_contiguous() for t in (q_bnhd, k_bnhd, v_bnhd)):
            # bf16 views of a packed projection (what qkv.unbind(2) gives): the kernel reads them through
            # strided TMA descriptors, so the reference's three .contiguous() copies (hipkittens.py:37-39) go
            q, k, v = q_bnhd, k_bnhd, v_bnhd
            attn_fwd(q, k, v, causal=bool(causal), softmax_scale=softmax_scale, out=O, lse=L)
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
        return O.to(out_dtype)

    @staticmethod
    def backward(ctx, dO_bnhd: torch.Tensor):
        raise NotImplementedError(
            "attention backward (dispatch_prep / dispatch_bwd_combined / dispatch_dq_shuffle) is outside this "
            "build; q, k, v, O and L are saved on ctx for it"
        )


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
        if key_padding_mask is not None:
            raise ValueError("key_padding_mask is not supported by the kernels")
        causal = self.causal if causal is None else causal
        q, k, v = qkv.unbind(dim=2)
        out_bnhd = HipAttnFunction.apply(q, k, v, causal, self.softmax_scale)
        return out_bnhd.to(q.dtype).contiguous()


class HipCrossAttention(nn.Module):
    """q [B, S, H, D], kv [B, S, 2, H_KV, D] -> [B, S, H, D] (hipkittens.py:165-202)."""

    def __init__(self, causal=False, softmax_scale=None, attention_dropout=0.0, deterministic=False):
        super().__init__()
        self.causal = causal
        self.softmax_scale = softmax_scale
        self.drop = nn.Dropout(attention_dropout)
        self.deterministic = deterministic

    def forward(self, q, kv, causal=None, key_padding_mask=None):
        if key_padding_mask is not None:
            raise ValueError("key_padding_mask is not supported by the kernels")
        batch_size = q.shape[0]
        causal = self.causal if causal is None else causal
        assert kv.shape[0] == batch_size and kv.shape[4] == q.shape[3]
        k, v = kv.unbind(dim=2)
        out_bnhd = HipAttnFunction.apply(q, k, v, causal, self.softmax_scale)
        return out_bnhd.to(q.dtype).contiguous()
