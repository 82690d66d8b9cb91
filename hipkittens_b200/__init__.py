"""hipkittens_b200: B200-native bf16 GQA flash-attention forward and paged-KV decode.

Everything here runs on hand-written sm_100a CUDA kernels behind a C ABI (``include/hk_attn.h``,
``lib/libhk_attn.so``). There is no CPU or PyTorch fallback: if the native library is missing or no
sm_100 device is present, calls raise.

Public surface
--------------
* ``attn_fwd(q, k, v, causal=False, ...) -> (O, L)``, ``attn_bwd_prep`` / ``attn_bwd`` / ``dq_shuffle`` (the
  backward pass), ``paged_decode(...) -> (O, L)`` and ``paged_kv_append(...)``: torch-tensor front ends over
  the C ABI (ctypes).
* ``load_tk_kernel(causal)`` / ``load_tk_kernel_fwd(causal)`` / ``load_tk_kernel_bkwd(causal)`` /
  ``load_tk_kernel_bkwd_prep(causal)``: the reference's extension modules (``tk_kernel.dispatch_micro``,
  ``tk_kernel_fwd.dispatch_fwd``, ``tk_kernel_bkwd.dispatch_bwd_combined``, ``tk_kernel_bkwd_prep.dispatch_prep``
  and ``.dispatch_dq_shuffle``) built for B200.
* ``HipAttnFunction`` in :mod:`hipkittens_b200.attention`: the reference's autograd-function forward.
"""
from ._native import (  # noqa: F401
    HK_DQ_BHND,
    HK_DQ_BNHD,
    HkError,
    attn_bwd,
    attn_bwd_prep,
    attn_fwd,
    capi,
    dq_shuffle,
    kernel_launch_count,
    lib_path,
    load_tk_kernel,
    load_tk_kernel_bkwd,
    load_tk_kernel_bkwd_prep,
    load_tk_kernel_fwd,
    load_tk_kernel_rotary,
    paged_decode,
    paged_decode_workspace_bytes,
    attn_fwd_paged,
    paged_kv_append,
    paged_kv_append_rotary,
    rotary,
    rotary_bnhd,
)

__all__ = [
    "HK_DQ_BHND",
    "HK_DQ_BNHD",
    "HkError",
    "attn_bwd",
    "attn_bwd_prep",
    "attn_fwd",
    "capi",
    "dq_shuffle",
    "kernel_launch_count",
    "lib_path",
    "load_tk_kernel",
    "load_tk_kernel_bkwd",
    "load_tk_kernel_bkwd_prep",
    "load_tk_kernel_fwd",
    "load_tk_kernel_rotary",
    "paged_decode",
    "attn_fwd_paged",
    "paged_kv_append",
    "paged_kv_append_rotary",
    "paged_decode_workspace_bytes",
    "rotary",
    "rotary_bnhd",
]
