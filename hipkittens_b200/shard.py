"""Partitioning of the attention workload over the GPUs of one box.

Attention for different (batch, kv-head) pairs shares nothing, so the B * H_KV units are dealt out
contiguously to ranks and every rank runs the single-GPU kernel on its own slice; no collective is
needed on the data path. The reference has no multi-device attention code (its only multi-device
mechanism is Lightning DDP around the training loop, training/llama/train/training.py:166-176).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import List, Tuple


@dataclass(frozen=True)
class UnitSlice:
    """A run of kv heads [kvh_lo, kvh_hi) of one batch element."""

    batch: int
    kvh_lo: int
    kvh_hi: int


def unit_range(n_units: int, world: int, rank: int) -> Tuple[int, int]:
    """Contiguous, balanced split of n_units into `world` parts; the first (n_units % world) ranks get one more."""
    if world <= 0 or not (0 <= rank < world):
        raise ValueError("rank must be in [0, world)")
    base, extra = divmod(n_units, world)
    lo = rank * base + min(rank, extra)
    return lo, lo + base + (1 if rank < extra else 0)


def partition_units(b: int, h_kv: int, world: int, rank: int) -> List[UnitSlice]:
    """Slices of (batch, kv-head range) owned by `rank`. Units are ordered batch-major, so ranks take whole
    batch elements when B >= world and split kv heads inside a batch element otherwise."""
    lo, hi = unit_range(b * h_kv, world, rank)
    out: List[UnitSlice] = []
    u = lo
    while u < hi:
        bi, kh = divmod(u, h_kv)
        run = min(hi - u, h_kv - kh)
        out.append(UnitSlice(bi, kh, kh + run))
        u += run
    return out


def shard_tensors(q, k, v, h_kv: int, slices: List[UnitSlice]):
    """Materialise this rank's shard as contiguous [n, N, H', D] tensors, one entry per group of slices that
    have the same number of kv heads (the kernel entry wants dense [B,N,H,D] / [B,N,H_KV,D] tensors).

    Returns a list of (q_s, k_s, v_s, slices_in_group). q heads follow their kv heads: kv head j owns query
    heads [j*G, (j+1)*G).
    """
    import torch

    g = q.shape[2] // h_kv
    groups = {}
    for s in slices:
        groups.setdefault(s.kvh_hi - s.kvh_lo, []).append(s)
    out = []
    for _width, members in sorted(groups.items()):
        qs = torch.stack([q[s.batch, :, s.kvh_lo * g:s.kvh_hi * g] for s in members]).contiguous()
        ks = torch.stack([k[s.batch, :, s.kvh_lo:s.kvh_hi] for s in members]).contiguous()
        vs = torch.stack([v[s.batch, :, s.kvh_lo:s.kvh_hi] for s in members]).contiguous()
        out.append((qs, ks, vs, members))
    return out


def scatter_outputs(o_full, l_full, o_s, l_s, members: List[UnitSlice], h_kv: int) -> None:
    """Write a shard's O [n,N,H',D] and L [n,H',1,N] back into full-size O [B,N,H,D] and L [B,H,1,N]."""
    g = o_full.shape[2] // h_kv
    for i, s in enumerate(members):
        o_full[s.batch, :, s.kvh_lo * g:s.kvh_hi * g] = o_s[i]
        l_full[s.batch, s.kvh_lo * g:s.kvh_hi * g] = l_s[i]


def shard_like_q(t, h_kv: int, members: List[UnitSlice]):
    """This rank's part of another [B,N,H,D] tensor that follows q's heads (dO, O), for one group returned by
    `shard_tensors`."""
    import torch

    g = t.shape[2] // h_kv
    return torch.stack([t[s.batch, :, s.kvh_lo * g:s.kvh_hi * g] for s in members]).contiguous()


def shard_stats(t, h_kv: int, members: List[UnitSlice]):
    """This rank's part of a per-row statistic [B,H,1,N] (L, delta) for one group returned by `shard_tensors`."""
    import torch

    g = t.shape[1] // h_kv
    return torch.stack([t[s.batch, s.kvh_lo * g:s.kvh_hi * g] for s in members]).contiguous()


def scatter_grads(dq_full, dk_full, dv_full, dq_s, dk_s, dv_s, members: List[UnitSlice], h_kv: int) -> None:
    """Write a shard's dQ [n,N,H',D], dK and dV [n,N,H_KV',D] back into the full-size gradient tensors. The backward
    shards exactly like the forward: dK and dV of a kv head only need the query heads of its own group."""
    g = dq_full.shape[2] // h_kv
    for i, s in enumerate(members):
        dq_full[s.batch, :, s.kvh_lo * g:s.kvh_hi * g] = dq_s[i]
        dk_full[s.batch, :, s.kvh_lo:s.kvh_hi] = dk_s[i]
        dv_full[s.batch, :, s.kvh_lo:s.kvh_hi] = dv_s[i]
