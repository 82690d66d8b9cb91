"""The multi-GPU path shards independent (batch, kv-head) units and needs no collective on the data path.
Its host logic is exercised here with two gloo ranks on the CPU, each computing its shard with the oracle
in place of the kernel and rank 0 checking the reassembled result."""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from hipkittens_b200.shard import partition_units, scatter_outputs, shard_tensors, unit_range
from hipkittens_b200.synthetic import make_prefill_inputs
from oracle.attn_oracle import attn_fwd_oracle


def test_unit_range_covers_everything_once():
    for n_units in (1, 7, 32, 128, 512):
        for world in (1, 2, 3, 4, 8):
            seen = []
            for r in range(world):
                lo, hi = unit_range(n_units, world, r)
                seen += list(range(lo, hi))
                assert hi - lo in (n_units // world, n_units // world + 1)
            assert seen == list(range(n_units))


def test_partition_prefers_whole_batches_then_splits_heads():
    # config 2 on 8 GPUs: 16 batches x 8 kv heads -> 2 whole batch elements per rank
    s = partition_units(16, 8, 8, 3)
    assert [(x.batch, x.kvh_lo, x.kvh_hi) for x in s] == [(6, 0, 8), (7, 0, 8)]
    # config 3 on 8 GPUs: 4 batches x 8 kv heads -> half a batch element per rank
    s = partition_units(4, 8, 8, 5)
    assert [(x.batch, x.kvh_lo, x.kvh_hi) for x in s] == [(2, 4, 8)]
    # uneven: 3 batches x 2 heads over 4 ranks
    all_units = []
    for r in range(4):
        for x in partition_units(3, 2, 4, r):
            all_units += [(x.batch, kh) for kh in range(x.kvh_lo, x.kvh_hi)]
    assert all_units == [(b, kh) for b in range(3) for kh in range(2)]


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, b, n, h, hkv, d, causal, ret):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    torch.set_num_threads(2)
    q, k, v = make_prefill_inputs(b, n, h, hkv, d, seed=0)
    o_full = torch.zeros((b, n, h, d), dtype=torch.float32)
    l_full = torch.zeros((b, h, 1, n), dtype=torch.float32)
    for qs, ks, vs, members in shard_tensors(q, k, v, hkv, partition_units(b, hkv, world, rank)):
        assert qs.is_contiguous() and ks.is_contiguous()
        o_s, l_s = attn_fwd_oracle(qs, ks, vs, causal)  # stands in for the kernel on this rank
        scatter_outputs(o_full, l_full, o_s.float(), l_s, members, hkv)
    # verification-only gather (shards are disjoint, so a sum reassembles them); not part of the data path
    dist.all_reduce(o_full)
    dist.all_reduce(l_full)
    if rank == 0:
        o_ref, l_ref = attn_fwd_oracle(q, k, v, causal)
        ret["o"] = float((o_full - o_ref.float()).abs().max())
        ret["l"] = float((l_full - l_ref).abs().max())
    dist.barrier()
    dist.destroy_process_group()


@pytest.mark.parametrize("b,hkv", [(4, 2), (1, 4), (3, 2)])
def test_two_rank_sharded_forward_matches_unsharded(b, hkv):
    mgr = mp.Manager()
    ret = mgr.dict()
    mp.spawn(_worker, args=(2, _free_port(), b, 128, 2 * hkv, hkv, 64, True, ret), nprocs=2, join=True)
    # the oracle on a shard and on the whole tensor runs the same arithmetic per unit, but torch's CPU contractions may
    # split their reductions differently from call to call, and a last-bit difference in fp32 can flip the rounding of
    # an O element to bf16: allow one bf16 ulp of |O| < 2, and 1e-4 on L, ten times the largest difference seen (a
    # unit placed wrongly would be off by the size of O and L themselves)
    assert ret["o"] <= 1e-2 and ret["l"] <= 1e-4


def _bwd_worker(rank, world, port, b, n, h, hkv, d, causal, ret):
    from hipkittens_b200.shard import scatter_grads, shard_like_q
    from oracle.attn_oracle import attn_bwd_oracle

    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    torch.set_num_threads(2)
    q, k, v = make_prefill_inputs(b, n, h, hkv, d, seed=0)
    d_o = make_prefill_inputs(b, n, h, hkv, d, seed=1)[0]
    dq_full, dk_full, dv_full = torch.zeros(q.shape), torch.zeros(k.shape), torch.zeros(v.shape)
    for qs, ks, vs, members in shard_tensors(q, k, v, hkv, partition_units(b, hkv, world, rank)):
        dos = shard_like_q(d_o, hkv, members)
        dq_s, dk_s, dv_s, _ = attn_bwd_oracle(qs, ks, vs, dos, causal)  # stands in for the kernels on this rank
        scatter_grads(dq_full, dk_full, dv_full, dq_s, dk_s, dv_s, members, hkv)
    for t in (dq_full, dk_full, dv_full):
        dist.all_reduce(t)  # verification only: shards are disjoint
    if rank == 0:
        rq, rk, rv, _ = attn_bwd_oracle(q, k, v, d_o, causal)
        ret["err"] = max(float((dq_full - rq).abs().max()), float((dk_full - rk).abs().max()),
                         float((dv_full - rv).abs().max()))
    dist.barrier()
    dist.destroy_process_group()


@pytest.mark.parametrize("b,hkv", [(4, 2), (1, 4)])
def test_two_rank_sharded_backward_matches_unsharded(b, hkv):
    """dK and dV of a kv head need only the query heads of its own group, so the backward shards over the same
    (batch, kv-head) units as the forward, again without a collective on the data path."""
    mgr = mp.Manager()
    ret = mgr.dict()
    mp.spawn(_bwd_worker, args=(2, _free_port(), b, 128, 2 * hkv, hkv, 64, True, ret), nprocs=2, join=True)
    assert ret["err"] <= 1e-4  # see the forward test: same arithmetic per unit, last bits may differ


def test_both_bench_arms_print_the_same_config_object():
    """bench.py's GPU arm and its reference arm take `config` from one function, so the two JSON lines describe the
    same workload key for key; what describes the run (per-GPU batch, sharding) lives beside it, not in it."""
    import importlib.util
    import inspect
    import os

    path = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "bench.py")
    spec = importlib.util.spec_from_file_location("bench_module", path)
    bench = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(bench)
    cfg = bench.workload_config(bench.DEFAULT_WORKLOAD)
    assert cfg == {"workload": "gqa_fwd_b16_n2048_h64_kv8_d128", "B": 16, "N": 2048, "H": 64, "H_KV": 8, "D": 128,
                   "causal": False, "cache": "inputs_exceed_l2"}
    assert '"config": workload_config(args.workload)' in inspect.getsource(bench.main)
    assert "workload_config(args.workload)" in inspect.getsource(bench.run_reference_arm)
    for name in bench.OTHER_WORKLOADS:
        assert bench.workload_config(name)["workload"] == name
    # the split of config 2 the N-GPU run makes: whole batch elements per rank, equal shares at 2, 4 and 8 ranks
    for world in (2, 4, 8):
        shares = [sum(s.kvh_hi - s.kvh_lo for s in partition_units(16, 8, world, r)) for r in range(world)]
        assert shares == [128 // world] * world
