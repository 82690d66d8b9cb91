"""GPU parity of the paged-KV decode against the CPU oracle (max-abs 2e-2 on O, 1e-3 on L)."""
import pytest
import torch

import hipkittens_b200 as hk
from hipkittens_b200 import _native
from hipkittens_b200.synthetic import make_paged_inputs, make_prefill_inputs
from oracle.attn_oracle import paged_decode_oracle

pytestmark = pytest.mark.gpu
TOL_O, TOL_L = 2e-2, 1e-3


@pytest.fixture(scope="module")
def dev():
    assert torch.cuda.is_available(), "these tests need a B200"
    return torch.device("cuda:0")


def run_decode(q, kp, vp, bt, cl, dev, use_shim=False):
    s, _, h, d = q.shape
    o = torch.full((s, 1, h, d), float("nan"), dtype=torch.bfloat16, device=dev)
    l = torch.full((s, h, 1, 1), float("nan"), dtype=torch.float32, device=dev)
    ws = torch.empty(hk.paged_decode_workspace_bytes(s, h, d, bt.shape[1]), dtype=torch.uint8, device=dev)
    args = (q.to(dev), kp.to(dev), vp.to(dev), bt.to(dev), cl.to(dev))
    if use_shim:
        hk.load_tk_kernel(False).dispatch_paged_decode(*args, o, l, ws)
    else:
        hk.paged_decode(*args, out=o, lse=l, workspace=ws)
    assert _native.device_status(0) == 0
    return o.cpu(), l.cpu()


CASES = [
    # S, H, H_KV, pool pages, ctx_lo, ctx_hi, seed
    (4, 8, 1, 200, 1, 600, 0),        # group 8; contexts from one token up, one and two chunks
    (3, 16, 2, 300, 500, 1500, 1),    # around the 512-token chunk boundary
    (2, 4, 4, 300, 17, 2000, 2),      # MHA (group 1)
    (2, 2, 1, 300, 1030, 1100, 3),    # group 2, three chunks with a short tail
    (5, 4, 1, 64, 1, 16, 4),          # everything inside the first page
    (2, 64, 8, 1200, 8000, 8192, 5),  # the configuration's head counts at maximum context
    (10, 16, 8, 5300, 6000, 8192, 6),  # enough CTAs for the launcher to pick 1024-token chunks
    # group sizes that are not powers of two (28 / 4 = 7, 40 / 8 = 5, 12 / 2 = 6, 3 / 1 = 3 query heads per kv head)
    (3, 28, 4, 600, 50, 2100, 7),
    (2, 40, 8, 700, 900, 3000, 8),
    (4, 12, 2, 300, 1, 700, 9),
    (2, 3, 1, 200, 200, 1300, 10),
]


@pytest.mark.parametrize("s,h,hkv,pool,lo,hi,seed", CASES)
@pytest.mark.parametrize("use_shim", [False, True])
def test_parity(dev, s, h, hkv, pool, lo, hi, seed, use_shim):
    q, kp, vp, bt, cl = make_paged_inputs(s, h, hkv, 128, 16, pool, lo, hi, seed)
    o, l = run_decode(q, kp, vp, bt, cl, dev, use_shim)
    o_ref, l_ref = paged_decode_oracle(q, kp, vp, bt, cl)
    assert not torch.isnan(o.float()).any() and not torch.isnan(l).any()
    assert float((o.float() - o_ref.float()).abs().max()) <= TOL_O
    assert float((l - l_ref).abs().max()) <= TOL_L


def test_exact_chunk_and_page_boundaries(dev):
    q, kp, vp, bt, _ = make_paged_inputs(6, 8, 2, 128, 16, 800, 1100, 1100, seed=6)
    cl = torch.tensor([16, 512, 513, 1024, 1025, 15], dtype=torch.int32)
    o, l = run_decode(q, kp, vp, bt, cl, dev)
    o_ref, l_ref = paged_decode_oracle(q, kp, vp, bt, cl)
    assert float((o.float() - o_ref.float()).abs().max()) <= TOL_O
    assert float((l - l_ref).abs().max()) <= TOL_L


def test_decode_equals_last_row_of_causal_prefill(dev):
    """Ties the two kernels together: gather one sequence's pages into a contiguous K/V, run the causal
    forward on it with the decode query as the last row, compare that row with the decode result."""
    q, kp, vp, bt, cl = make_paged_inputs(1, 8, 2, 128, 16, 200, 1024, 1024, seed=7)
    o, l = run_decode(q, kp, vp, bt, cl, dev)
    n = 1024
    ids = bt[0, : n // 16].long()
    ks = kp[ids].reshape(1, n, 2, 128).contiguous()
    vs = vp[ids].reshape(1, n, 2, 128).contiguous()
    qfull, _, _ = make_prefill_inputs(1, n, 8, 2, 128, seed=8)
    qfull[0, -1] = q[0, 0]
    o_p, l_p = hk.attn_fwd(qfull.to(dev), ks.to(dev), vs.to(dev), causal=True)
    assert float((o_p[0, -1].float().cpu() - o[0, 0].float()).abs().max()) <= 1e-2
    assert float((l_p[0, :, 0, -1].cpu() - l[0, :, 0, 0]).abs().max()) <= 1e-4


def test_out_of_range_page_id_is_reported_not_dereferenced(dev):
    q, kp, vp, bt, cl = make_paged_inputs(2, 8, 1, 128, 16, 100, 100, 200, seed=9)
    bad = bt.clone()
    bad[1, 0] = 100  # == num_pages
    s, _, h, d = q.shape
    ws = torch.empty(hk.paged_decode_workspace_bytes(s, h, d, bt.shape[1]), dtype=torch.uint8, device=dev)
    hk.paged_decode(q.to(dev), kp.to(dev), vp.to(dev), bad.to(dev), cl.to(dev), workspace=ws)
    assert _native.device_status(0) == _native.HK_EBADPAGE
    bad[1, 0] = -3
    hk.paged_decode(q.to(dev), kp.to(dev), vp.to(dev), bad.to(dev), cl.to(dev), workspace=ws)
    assert _native.device_status(0) == _native.HK_EBADPAGE
    # the context is intact and a clean call still works
    o, l = run_decode(q, kp, vp, bt, cl, dev)
    o_ref, l_ref = paged_decode_oracle(q, kp, vp, bt, cl)
    assert float((o.float() - o_ref.float()).abs().max()) <= TOL_O


def test_context_length_beyond_the_block_table_is_clamped_and_reported(dev):
    """ctx_lens is device data the host never reads: a length above max_pages * 16 must not make the kernels walk
    past the block-table row. It is clamped to the row's capacity, reported as HK_EBADLEN, and the result equals the
    result for the clamped length."""
    q, kp, vp, bt, cl = make_paged_inputs(3, 8, 2, 128, 16, 400, 900, 1500, seed=31)
    cap = bt.shape[1] * 16
    cl_full = cl.clone()
    cl_full[-1] = cap                       # the last sequence's row is the end of the block-table buffer
    o_ref, l_ref = run_decode(q, kp, vp, bt, cl_full, dev)
    for excess in (1, 5000, 2 ** 30):
        cl_bad = cl_full.clone()
        cl_bad[-1] = cap + excess
        s, _, h, d = q.shape
        ws = torch.empty(hk.paged_decode_workspace_bytes(s, h, d, bt.shape[1]), dtype=torch.uint8, device=dev)
        o, l = hk.paged_decode(q.to(dev), kp.to(dev), vp.to(dev), bt.to(dev), cl_bad.to(dev), workspace=ws)
        assert _native.device_status(0) == _native.HK_EBADLEN
        assert torch.equal(o.cpu(), o_ref) and torch.equal(l.cpu(), l_ref)
    # the status word is cleared on read and a clean call is clean again
    run_decode(q, kp, vp, bt, cl_full, dev)


def test_unsupported_shapes_are_refused_before_any_launch(dev):
    assert hk.paged_decode_workspace_bytes(2, 8, 128, 8192) > 0
    assert hk.paged_decode_workspace_bytes(2, 8, 128, 8193) == 0     # more than 256 chunks of 32 pages
    assert hk.paged_decode_workspace_bytes(70000, 8, 128, 64) == 0   # sequences are a grid dimension
    q, kp, vp, bt, cl = make_paged_inputs(1, 8, 1, 128, 16, 40, 100, 200, seed=32)
    wide = torch.zeros((1, 8200), dtype=torch.int32, device=dev)
    before = hk.kernel_launch_count()
    rc = hk.capi().hk_attn_paged_decode(q.to(dev).data_ptr(), kp.to(dev).data_ptr(), vp.to(dev).data_ptr(),
                                        wide.data_ptr(), cl.to(dev).data_ptr(), q.to(dev).data_ptr(),
                                        torch.empty(8, device=dev).data_ptr(), 1, 8, 1, 128, 16, 8200, 40, 0.0,
                                        torch.empty(1 << 20, dtype=torch.uint8, device=dev).data_ptr(), 1 << 20, 0, None)
    assert rc == _native.HK_EUNSUPPORTED and hk.kernel_launch_count() == before
    assert b"max_pages_per_seq" in hk.capi().hk_last_cuda_error()


def test_host_tensors_are_rejected_by_the_front_end(dev):
    q, kp, vp, bt, cl = make_paged_inputs(1, 8, 1, 128, 16, 40, 100, 200, seed=33)
    with pytest.raises(RuntimeError, match="block_table must be a tensor on cuda"):
        hk.paged_decode(q.to(dev), kp.to(dev), vp.to(dev), bt, cl.to(dev))   # bt left on the host
    with pytest.raises(RuntimeError, match="ctx_lens must be a tensor on cuda"):
        hk.paged_decode(q.to(dev), kp.to(dev), vp.to(dev), bt.to(dev), cl)


def test_full_size_configuration(dev):
    """BASELINE config 5: 64 sequences, ctx ~ U{512..8192}, H=64, H_KV=8, D=128, 40 000-page pool."""
    q, kp, vp, bt, cl = make_paged_inputs(64, 64, 8, 128, 16, 40000, 512, 8192, seed=0, pool_on="cuda:0")
    qd, btd, cld = q.to(dev), bt.to(dev), cl.to(dev)
    o, l = hk.paged_decode(qd, kp, vp, btd, cld)
    assert _native.device_status(0) == 0
    o2, l2 = hk.paged_decode(qd, kp, vp, btd, cld)
    assert torch.equal(o, o2) and torch.equal(l, l2)  # deterministic
    # oracle on a spread of sequences (shortest, longest, first, last); the pools come back to the host once
    order = torch.argsort(cl)
    idx = sorted({int(order[0]), int(order[-1]), 0, 63, int(order[32])})
    kp_h, vp_h = kp.cpu(), vp.cpu()
    o_ref, l_ref = paged_decode_oracle(q[idx], kp_h, vp_h, bt[idx], cl[idx])
    assert float((o[idx].float().cpu() - o_ref.float()).abs().max()) <= TOL_O
    assert float((l[idx].cpu() - l_ref).abs().max()) <= TOL_L
    # size-independent property: doubling V doubles O exactly and leaves L unchanged
    o3, l3 = hk.paged_decode(qd, kp, (vp.float() * 2).to(torch.bfloat16), btd, cld)
    assert torch.equal(o3.float(), o.float() * 2) and torch.equal(l3, l)


def test_decode_replays_from_a_cuda_graph(dev):
    """A serving loop captures the decode step once and replays it: the split and combine launches of
    hk_attn_paged_decode (workspace owned by the caller) go onto the capturing stream, and a replay after the inputs
    changed in place gives the same bits as an eager call."""
    q, kp, vp, bt, cl = make_paged_inputs(3, 16, 2, 128, 16, 400, 100, 1500, seed=12)
    q, kp, vp, bt, cl = (t.to(dev) for t in (q, kp, vp, bt, cl))
    ws = torch.empty(hk.paged_decode_workspace_bytes(3, 16, 128, bt.shape[1]), dtype=torch.uint8, device=dev)
    o = torch.empty_like(q)
    l = torch.empty((3, 16, 1, 1), dtype=torch.float32, device=dev)
    side = torch.cuda.Stream()
    with torch.cuda.stream(side):
        hk.paged_decode(q, kp, vp, bt, cl, out=o, lse=l, workspace=ws, stream=side)  # warm-up outside the capture
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph, stream=side):
        hk.paged_decode(q, kp, vp, bt, cl, out=o, lse=l, workspace=ws, stream=side)
    q.copy_(torch.randn(q.shape, generator=torch.Generator().manual_seed(13)).to(torch.bfloat16))  # a new query token
    graph.replay()
    torch.cuda.synchronize()
    o_replay, l_replay = o.clone(), l.clone()
    o_eager, l_eager = hk.paged_decode(q, kp, vp, bt, cl)
    assert _native.device_status(0) == 0
    assert torch.equal(o_replay, o_eager) and torch.equal(l_replay, l_eager)
    o_ref, l_ref = paged_decode_oracle(q.cpu(), kp.cpu(), vp.cpu(), bt.cpu(), cl.cpu())
    assert float((o_replay.float().cpu() - o_ref.float()).abs().max()) <= 2e-2
