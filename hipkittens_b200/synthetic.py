"""Seeded synthetic inputs with the shapes and value distributions of the benchmark configurations.

The reference's harness draws q, k, v with ``torch.randn`` in bf16 (kernels/attn/gqa/test_python.py:30-32);
these generators do the same from an explicit seed, on the CPU, so that a CPU checker and the GPU see
identical bits. The paged-KV problem (no counterpart in the reference) draws context lengths uniformly,
and gives every sequence a slice of one seeded permutation of page ids so that ids are distinct.
"""
from __future__ import annotations

from typing import Optional

import torch


def make_prefill_inputs(b: int, n: int, h: int, hkv: int, d: int, seed: int = 0):
    """bf16 i.i.d. N(0,1) q, k, v drawn on the CPU in that order from one seed.

    This is the reference harness's distribution (``kernels/attn/gqa/test_python.py:30-32``); drawing on
    the CPU lets the oracle and the GPU see identical bits.
    """
    gen = torch.Generator().manual_seed(seed)
    q = torch.randn((b, n, h, d), generator=gen, dtype=torch.float32).to(torch.bfloat16)
    k = torch.randn((b, n, hkv, d), generator=gen, dtype=torch.float32).to(torch.bfloat16)
    v = torch.randn((b, n, hkv, d), generator=gen, dtype=torch.float32).to(torch.bfloat16)
    return q, k, v


def make_paged_inputs(
    n_seq: int,
    h: int,
    hkv: int,
    d: int,
    page: int,
    num_pages: int,
    ctx_lo: int,
    ctx_hi: int,
    seed: int = 0,
    pool_on: Optional[str] = None,
):
    """Synthetic paged-KV decode problem.

    Context lengths are uniform integers in [ctx_lo, ctx_hi]; every sequence's block table is a slice
    of one seeded permutation of page ids, so ids are distinct across the whole batch. The K/V pools
    are bf16 N(0,1). ``pool_on`` may name a device on which to draw the (large) pools directly.
    """
    gen = torch.Generator().manual_seed(seed)
    ctx = torch.randint(ctx_lo, ctx_hi + 1, (n_seq,), generator=gen, dtype=torch.int32)
    npg = (ctx + page - 1) // page
    total = int(npg.sum())
    assert total <= num_pages, "page pool too small for the drawn context lengths"
    perm = torch.randperm(num_pages, generator=gen, dtype=torch.int64)[:total].to(torch.int32)
    max_pages = int(npg.max())
    table = torch.zeros((n_seq, max_pages), dtype=torch.int32)
    off = 0
    for s in range(n_seq):
        c = int(npg[s])
        table[s, :c] = perm[off:off + c]
        off += c
    q = torch.randn((n_seq, 1, h, d), generator=gen, dtype=torch.float32).to(torch.bfloat16)
    if pool_on is None:
        kp = torch.randn((num_pages, page, hkv, d), generator=gen, dtype=torch.float32).to(torch.bfloat16)
        vp = torch.randn((num_pages, page, hkv, d), generator=gen, dtype=torch.float32).to(torch.bfloat16)
    else:
        dgen = torch.Generator(device=pool_on).manual_seed(seed + 1)
        kp = torch.randn((num_pages, page, hkv, d), generator=dgen, dtype=torch.bfloat16, device=pool_on)
        vp = torch.randn((num_pages, page, hkv, d), generator=dgen, dtype=torch.bfloat16, device=pool_on)
    return q, kp, vp, table, ctx
