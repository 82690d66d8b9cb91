"""CPU oracle for the bf16 GQA attention forward and the paged-KV decode variant.

TEST INFRASTRUCTURE ONLY. Nothing in the product package imports this module; it is used by the
tests, by the smoke check and by the CPU-baseline leg of the benchmark as the checker / baseline.

What it restates
----------------
The reference's PyTorch math path, ``training/llama/llama/models/attentions/base.py:78-120``
(``CrossAttention.forward``): GQA by repeating each KV head over its group (``:92-93``),
``scores = einsum("bthd,bshd->bhts", q, k * scale)`` (``:96``), causal mask ``col > row + Sk - Sq``
(``:104-116``), softmax over keys (``:117``), ``einsum("bhts,bshd->bthd", attention, v)`` (``:119``).

Deliberate deltas (they define the parity target of this build):
  1. the softmax and both contractions run in fp32 on the bf16 inputs (the reference softmaxes in
     ``v.dtype``, i.e. bf16 for bf16 inputs);
  2. masked logits are ``-inf`` instead of ``-10000`` (identical after exp in fp32);
  3. it also returns ``L = logsumexp(scale * q k^T)`` (natural log) per (batch, head, row), laid out
     ``[B, H, 1, N]`` as the kernels do: ``kernels/attn/gqa/kernel.cpp:569-573`` computes
     ``max * ln2 + ln(sum)`` in the log2 domain and stores it at ``L[b, h, 0, row]``;
  4. O is rounded to bf16 once at the end, as the kernels do (``kernels/attn/gqa/kernel.cpp:565-567``).

Parity pin
----------
O is pinned against outputs of the reference module itself, run in this build's container on fp32
copies of bf16-valued inputs (then delta 1 vanishes and the reference computes exactly this math);
see ``tests/golden/make_golden.py`` and ``tests/test_oracle.py``. The reference has no CPU path that
emits L and no recorded kernel outputs, so L is pinned only to its definition above, and parity
against the reference's HIP kernels themselves is unpinned (they cannot run here).

The paged decode variant has no counterpart in the reference; its oracle gathers each sequence's
pages through the block table and applies the same math to one query row.

Backward
--------
``attn_bwd_oracle`` is the derivative of that same math path written out by hand (what autograd computes
for ``base.py:96-119``; the reference states the same formulas in ``simple_flash_backward``,
``kernels/attn/gqa_backwards/test_python.py:100-137``): with P the softmax, dP = dO V^T,
delta = rowsum(dO * O) and dS = P * (dP - delta): dV = P^T dO, dK = scale * dS^T Q, dQ = scale * dS K, each
summed over the heads of a group for dK and dV. It is pinned against gradients that autograd produced
through the reference's own ``CrossAttention`` module (``tests/golden/make_golden.py``).
"""
from __future__ import annotations

import math
from typing import Optional, Tuple

import torch

from hipkittens_b200.synthetic import make_paged_inputs, make_prefill_inputs  # noqa: F401  (re-exported for tests)

__all__ = [
    "attn_fwd_oracle",
    "attn_bwd_oracle",
    "rotary_oracle",
    "rotary_cos_sin",
    "paged_decode_oracle",
    "paged_kv_append_oracle",
    "make_prefill_inputs",
    "make_paged_inputs",
    "robustness_check",
]


def _unit(q_g: torch.Tensor, k_g: torch.Tensor, v_g: torch.Tensor, scale: float, causal: bool):
    """One (batch, kv-head) unit. q_g [N, G, D] fp32, k_g/v_g [S, D] fp32 -> O [N, G, D] fp32, L [G, N]."""
    n, _, _ = q_g.shape
    s = k_g.shape[0]
    # base.py:96  scores = einsum(q, k * scale)
    scores = torch.einsum("tgd,sd->gts", q_g, k_g * scale)
    if causal:
        # base.py:104-116  col > row + Sk - Sq is masked
        row = torch.arange(n).view(n, 1)
        col = torch.arange(s).view(1, s)
        scores = scores.masked_fill((col > row + (s - n)).unsqueeze(0), float("-inf"))
    lse = torch.logsumexp(scores, dim=-1)  # [G, N]
    # base.py:117,119  softmax then contraction with v. A row that sees no key (causal with fewer kept keys than
    # queries) has lse = -inf and is defined as O = 0; the reference's -10000 fill would spread it over masked keys.
    attn = torch.exp(scores - lse.masked_fill(torch.isinf(lse), 0.0).unsqueeze(-1))
    out = torch.einsum("gts,sd->tgd", attn, v_g)
    return out, lse


def attn_fwd_oracle(
    q: torch.Tensor,
    k: torch.Tensor,
    v: torch.Tensor,
    causal: bool = False,
    softmax_scale: Optional[float] = None,
    kv_lens: Optional[torch.Tensor] = None,
) -> Tuple[torch.Tensor, torch.Tensor]:
    """q [B,N,H,D], k/v [B,S,H_KV,D] (any float dtype; values are used as given, math in fp32).

    ``kv_lens`` [B] restricts batch element b to its first kv_lens[b] keys: the reference's
    ``key_padding_mask`` (``base.py:97-103``, True = keep), with masked logits at -inf instead of -10000.
    With ``causal`` the mask is ``col > row + sk - Sq`` with sk the number of kept keys (``base.py:104-116``),
    whether or not S equals N.

    Returns O [B,N,H,D] bf16 and L [B,H,1,N] fp32. Work is chunked per (batch, kv-head) so that the
    largest benchmark shapes fit in host memory.
    """
    b, n, h, d = q.shape
    hkv = k.shape[2]
    assert h % hkv == 0 and k.shape == v.shape and k.shape[0] == b and k.shape[3] == d
    g = h // hkv
    scale = softmax_scale if softmax_scale else 1.0 / math.sqrt(d)
    out = torch.empty((b, n, h, d), dtype=torch.bfloat16)
    lse = torch.empty((b, h, 1, n), dtype=torch.float32)
    for bi in range(b):
        for kh in range(hkv):
            qg = q[bi, :, kh * g:(kh + 1) * g, :].float()
            klen = k.shape[1] if kv_lens is None else int(kv_lens[bi])
            o_u, l_u = _unit(qg, k[bi, :klen, kh, :].float(), v[bi, :klen, kh, :].float(), scale, causal)
            out[bi, :, kh * g:(kh + 1) * g, :] = o_u.to(torch.bfloat16)
            lse[bi, kh * g:(kh + 1) * g, 0, :] = l_u
    return out, lse


def attn_bwd_oracle(
    q: torch.Tensor,
    k: torch.Tensor,
    v: torch.Tensor,
    d_o: torch.Tensor,
    causal: bool = False,
    softmax_scale: Optional[float] = None,
    dtype: torch.dtype = torch.float32,
    kv_lens: Optional[torch.Tensor] = None,
) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor, torch.Tensor]:
    """Gradients of O = softmax(scale q k^T) v with respect to q, k, v for the upstream gradient d_o.

    q, d_o [B,N,H,D], k, v [B,Nk,H_KV,D] (values used as given, math in `dtype`). Returns dq [B,N,H,D],
    dk, dv [B,Nk,H_KV,D] and delta [B,H,1,N] = rowsum(d_o * O), all in `dtype` (no bf16 rounding: the
    tolerance of the comparison covers the kernels' bf16 outputs). O here is the unrounded attention
    output; the kernels compute delta from the bf16-rounded O of the forward pass
    (kernels/attn/gqa_backwards/attn_bkwd_prep.cpp:176-185). ``kv_lens`` [B] masks keys at or beyond a batch
    element's length (the reference's ``key_padding_mask``, ``base.py:97-103``); their dk and dv are zero.
    """
    b, n, h, d = q.shape
    hkv = k.shape[2]
    nk = k.shape[1]
    assert h % hkv == 0 and k.shape == v.shape and d_o.shape == q.shape
    g = h // hkv
    scale = softmax_scale if softmax_scale else 1.0 / math.sqrt(d)
    dq = torch.empty((b, n, h, d), dtype=dtype)
    dk = torch.empty((b, nk, hkv, d), dtype=dtype)
    dv = torch.empty((b, nk, hkv, d), dtype=dtype)
    delta = torch.empty((b, h, 1, n), dtype=dtype)
    row = torch.arange(n).view(n, 1)
    col = torch.arange(nk).view(1, nk)
    for bi in range(b):
        klen = nk if kv_lens is None else int(kv_lens[bi])
        for kh in range(hkv):
            qg = q[bi, :, kh * g:(kh + 1) * g, :].to(dtype)      # [N, G, D]
            dog = d_o[bi, :, kh * g:(kh + 1) * g, :].to(dtype)
            ku = k[bi, :, kh, :].to(dtype)                       # [Nk, D]
            vu = v[bi, :, kh, :].to(dtype)
            scores = torch.einsum("tgd,sd->gts", qg, ku * scale)
            if causal:
                # base.py:104-116: col > row + sk - Sq is masked, sk = kept keys
                scores = scores.masked_fill((col > row + (klen - n)).unsqueeze(0), float("-inf"))
            if kv_lens is not None:
                scores = scores.masked_fill((col >= klen).unsqueeze(0), float("-inf"))
            # a row that sees no key is defined as O = 0 (see attn_fwd_oracle): all its probabilities are zero
            lse = torch.logsumexp(scores, dim=-1, keepdim=True)
            p = torch.exp(scores - lse.masked_fill(torch.isinf(lse), 0.0))  # [G, N, Nk]
            o = torch.einsum("gts,sd->tgd", p, vu)
            dl = (dog * o).sum(-1)                               # [N, G]
            dp = torch.einsum("tgd,sd->gts", dog, vu)
            ds = p * (dp - dl.t().unsqueeze(-1))
            dv[bi, :, kh, :] = torch.einsum("gts,tgd->sd", p, dog)
            dk[bi, :, kh, :] = torch.einsum("gts,tgd->sd", ds, qg) * scale
            dq[bi, :, kh * g:(kh + 1) * g, :] = torch.einsum("gts,sd->tgd", ds, ku) * scale
            delta[bi, kh * g:(kh + 1) * g, 0, :] = dl.t()
    return dq, dk, dv, delta


def paged_decode_oracle(
    q: torch.Tensor,
    k_pages: torch.Tensor,
    v_pages: torch.Tensor,
    block_table: torch.Tensor,
    ctx_lens: torch.Tensor,
    softmax_scale: Optional[float] = None,
) -> Tuple[torch.Tensor, torch.Tensor]:
    """q [S,1,H,D]; k_pages/v_pages [P,page,H_KV,D]; block_table [S,max_pages] int32; ctx_lens [S] int32.

    Token j of sequence s lives at ``pages[block_table[s, j // page], j % page]``. The single query row
    sees all ``ctx_lens[s]`` keys. Returns O [S,1,H,D] bf16 and L [S,H,1,1] fp32.
    """
    s_n, one, h, d = q.shape
    assert one == 1
    page = k_pages.shape[1]
    hkv = k_pages.shape[2]
    g = h // hkv
    scale = softmax_scale if softmax_scale else 1.0 / math.sqrt(d)
    out = torch.empty((s_n, 1, h, d), dtype=torch.bfloat16)
    lse = torch.empty((s_n, h, 1, 1), dtype=torch.float32)
    for si in range(s_n):
        ctx = int(ctx_lens[si])
        npg = (ctx + page - 1) // page
        ids = block_table[si, :npg].long()
        ks = k_pages[ids].reshape(npg * page, hkv, d)[:ctx].float()
        vs = v_pages[ids].reshape(npg * page, hkv, d)[:ctx].float()
        for kh in range(hkv):
            qg = q[si, :, kh * g:(kh + 1) * g, :].float()  # [1, G, D]
            o_u, l_u = _unit(qg, ks[:, kh, :], vs[:, kh, :], scale, causal=False)
            out[si, :, kh * g:(kh + 1) * g, :] = o_u.to(torch.bfloat16)
            lse[si, kh * g:(kh + 1) * g, 0, :] = l_u
    return out, lse


def robustness_check(ref: torch.Tensor, pred: torch.Tensor):
    """The reference harness's error statistics (``kernels/attn/gqa/test_python.py:46-57``).

    Returns (max_abs, error_count, numel, rel_l2, cosine) where an element counts as an error when
    ``|diff| > 0.001 + 0.05 * |ref|``.
    """
    ref = ref.float()
    pred = pred.float()
    diff = (ref - pred).abs()
    denom = ref.abs().clamp_min(1e-6)
    err = int((diff > (0.001 + 0.05 * denom)).sum())
    l2 = float(diff.pow(2).sum().sqrt() / ref.pow(2).sum().sqrt())
    cos = float(torch.nn.functional.cosine_similarity(ref.flatten(), pred.flatten(), dim=0))
    return float(diff.max()), err, ref.numel(), l2, cos


def paged_kv_append_oracle(k_new, v_new, k_pages, v_pages, block_table, start_pos):
    """Paged form of the reference's cache update ``kv_cache[b, offset:offset+T] = kv``
    (``training/llama/llama/models/mha.py:16-42``): token t of sequence s goes to position
    ``start_pos[s] + t``, i.e. row ``pos % page`` of page ``block_table[s, pos // page]``.
    Returns updated copies of the pools; positions outside the table or ids outside the pool are skipped."""
    kp, vp = k_pages.clone(), v_pages.clone()
    page = kp.shape[1]
    s_n, t_n = k_new.shape[:2]
    for s in range(s_n):
        for t in range(t_n):
            pos = int(start_pos[s]) + t
            if pos < 0 or pos // page >= block_table.shape[1]:
                continue
            pid = int(block_table[s, pos // page])
            if pid < 0 or pid >= kp.shape[0]:
                continue
            kp[pid, pos % page] = k_new[s, t]
            vp[pid, pos % page] = v_new[s, t]
    return kp, vp


def rotary_cos_sin(n: int, rotary_dim: int, base: float = 10000.0):
    """cos, sin [N, rotary_dim / 2] bf16 as the reference harness builds them, in bf16 throughout
    (``kernels/rotary/test_python.py:36-45``: positions, inverse frequencies and their outer product are bf16)."""
    dt = torch.bfloat16
    t = torch.arange(n, dtype=dt)
    inv_freq = 1.0 / (base ** (torch.arange(0, rotary_dim, 2, dtype=dt) / rotary_dim))
    freqs = torch.outer(t, inv_freq).to(dtype=dt)
    return torch.cos(freqs).to(dtype=dt), torch.sin(freqs).to(dtype=dt)


def rotary_oracle(x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor) -> torch.Tensor:
    """Rotary embedding of x [B,H,N,D] bf16 with cos, sin [N, R/2] bf16, restating ``get_output`` of the reference
    harness (``kernels/rotary/test_python.py:48-58``) on bf16 tensors: x * cos + rotate_half(x) * sin over the first R
    dimensions, every product and the sum rounded to bf16 (what the kernel's __hmul2 / __hsub2 / __hadd2 do,
    ``kernels/rotary/kernel.cpp:62-71``); the remaining dimensions pass through. Bit-exact target."""
    assert x.dtype == torch.bfloat16 and cos.dtype == torch.bfloat16 and sin.dtype == torch.bfloat16
    ro_dim = cos.shape[-1] * 2
    assert ro_dim <= x.shape[-1] and cos.shape[0] == x.shape[2]
    x_ro, x_end = x[..., :ro_dim], x[..., ro_dim:]
    x1, x2 = x_ro.chunk(2, dim=-1)
    rotated = torch.cat((-x2, x1), dim=-1)
    c = torch.cat((cos, cos), dim=-1).view(1, 1, cos.shape[0], ro_dim)
    s_ = torch.cat((sin, sin), dim=-1).view(1, 1, sin.shape[0], ro_dim)
    return torch.cat([x_ro * c + rotated * s_, x_end], dim=-1)
