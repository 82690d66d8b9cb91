"""Shared body of the backward timing and accuracy harnesses (kernels/attn/gqa_backwards/test_python.py and
kernels/attn/gqa_causal_backwards/test_python.py call into this file).

Protocol of the reference's kernels/attn/gqa_backwards/test_python.py: tk_kernel_fwd.dispatch_fwd produces O and L once
(test_python.py:227), then every timed iteration runs the three backward calls between two CUDA events
(test_python.py:268-303): tk_kernel_bkwd_prep.dispatch_prep(O, dO, delta), tk_kernel_bkwd.dispatch_bwd_combined(Q, K, V,
dO, dQ_in, dK, dV, L, delta) and tk_kernel_bkwd_prep.dispatch_dq_shuffle(dQ_in, dQ). TFLOPS = 2.5 * 4*B*N^2*H*D / (2 if
causal) / mean time (test_python.py:45-48). The comparison target is autograd through torch's
scaled_dot_product_attention (the reference compares with AITER, an AMD-only package), reported with the reference's
robustness statistics (test_python.py:56-68).
"""
import os

import torch

from harness_fwd import parse, robustness_check  # noqa: F401


def run_backward(tk_kernel_fwd, tk_kernel_bkwd, tk_kernel_bkwd_prep, c):
    B, D, H, HKV, N, causal = c["B"], c["D"], c["H"], c["H_KV"], c["N"], bool(c["causal"])
    warmup, iters = int(os.environ.get("HK_WARMUP", 20)), int(os.environ.get("HK_ITERS", 50))
    torch.manual_seed(0)
    dev = "cuda"
    mk = lambda h: torch.randn(B, N, h, D, dtype=torch.bfloat16, device=dev)  # noqa: E731
    Q, K, V, dO = mk(H), mk(HKV), mk(HKV), mk(H)
    O = torch.zeros(B, N, H, D, dtype=torch.bfloat16, device=dev)
    L = torch.zeros(B, H, 1, N, dtype=torch.float32, device=dev)
    tk_kernel_fwd.dispatch_fwd(Q, K, V, O, L, causal=causal)

    def step():
        dQ_in = torch.zeros(B, H, N, D, dtype=torch.bfloat16, device=dev)
        dQ = torch.zeros(B, N, H, D, dtype=torch.bfloat16, device=dev)
        dK = torch.zeros(B, N, HKV, D, dtype=torch.bfloat16, device=dev)
        dV = torch.zeros(B, N, HKV, D, dtype=torch.bfloat16, device=dev)
        delta = torch.zeros(B, H, 1, N, dtype=torch.float32, device=dev)
        torch.cuda.synchronize()
        start.record()
        tk_kernel_bkwd_prep.dispatch_prep(O, dO, delta)
        tk_kernel_bkwd.dispatch_bwd_combined(Q, K, V, dO, dQ_in, dK, dV, L, delta, causal=causal)
        tk_kernel_bkwd_prep.dispatch_dq_shuffle(dQ_in, dQ)
        end.record()
        torch.cuda.synchronize()
        return start.elapsed_time(end), dQ, dK, dV

    start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    for _ in range(warmup):
        step()
    times = []
    for _ in range(iters):
        ms, dQ, dK, dV = step()
        times.append(ms)
    ms = sum(times) / len(times)
    flop = 2.5 * 4 * B * N * N * H * D / (2 if causal else 1)
    print(f"Average execution time: {ms:.4f} ms")
    print(f"Performance: {flop / ms / 1e9:.2f} TFLOPS for {B=} {H=} {HKV=} {N=} {D=} {causal=} attention backward.")

    # accuracy against autograd through torch SDPA (fp32 math on the bf16 inputs), one batch element at a time
    q1, k1, v1 = (t[:1].float().requires_grad_(True) for t in (Q, K, V))
    g = H // HKV
    o_ref = torch.nn.functional.scaled_dot_product_attention(
        q1.transpose(1, 2), k1.transpose(1, 2).repeat_interleave(g, dim=1), v1.transpose(1, 2).repeat_interleave(g, dim=1),
        is_causal=causal).transpose(1, 2)
    o_ref.backward(dO[:1].float())
    for name, ours, ref in (("dQ", dQ[:1], q1.grad), ("dK", dK[:1], k1.grad), ("dV", dV[:1], v1.grad)):
        mx, errs, total, l2, cos = robustness_check(ref, ours)
        print(f"{name}: max_abs={mx:.6f}, errors={errs}/{total} ({100 * errs / total:.4f}%), rel_l2={l2:.6f}, cos={cos:.6f}")

