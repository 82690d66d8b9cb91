"""Shared body of the forward timing and accuracy harnesses (kernels/attn/gqa/test_python.py and
kernels/attn/gqa_causal/test_python.py keep the reference's two command lines and call into this file).

Protocol of the reference's harness: fresh torch.randn inputs per call, CUDA events around each call, TFLOPS =
4*B*N^2*H*D / (2 if causal) / mean time (kernels/attn/gqa/test_python.py:35-38,106-123). The comparison target is
torch's scaled_dot_product_attention on the same inputs (the reference compares with AITER, an AMD-only package),
reported with the reference's robustness statistics (test_python.py:46-57).
"""
import os

import torch


def parse(argv, arg_order, defaults):
    cfg = dict(defaults)
    for name, val in zip(arg_order, argv[1:]):
        cfg[name] = int(val)
    return cfg


def robustness_check(ref, pred):
    ref, pred = ref.float(), pred.float()
    diff = (ref - pred).abs()
    errors = int((diff > 0.001 + 0.05 * ref.abs().clamp_min(1e-6)).sum())
    l2 = float(diff.pow(2).sum().sqrt() / ref.pow(2).sum().sqrt())
    cos = float(torch.nn.functional.cosine_similarity(ref.flatten(), pred.flatten(), dim=0))
    return float(diff.max()), errors, ref.numel(), l2, cos


def run_forward(tk_kernel, c):
    B, D, H, HKV, N, causal = c["B"], c["D"], c["H"], c["H_KV"], c["N"], bool(c["causal"])
    warmup, iters = int(os.environ.get("HK_WARMUP", 50)), int(os.environ.get("HK_ITERS", 100))
    torch.manual_seed(0)
    flop = 4 * B * N * N * H * D // (2 if causal else 1)
    mk = lambda h: torch.randn(B, N, h, D, dtype=torch.bfloat16, device="cuda", requires_grad=True)  # noqa: E731
    out = torch.zeros(B, N, H, D, dtype=torch.bfloat16, device="cuda")
    lse = torch.zeros(B, H, 1, N, dtype=torch.float32, device="cuda")
    for _ in range(warmup):
        tk_kernel.dispatch_micro(mk(H), mk(HKV), mk(HKV), out, lse, causal=causal)
    start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    times = []
    for _ in range(iters):
        q, k, v = mk(H), mk(HKV), mk(HKV)
        torch.cuda.synchronize()
        start.record()
        tk_kernel.dispatch_micro(q, k, v, out, lse, causal=causal)
        end.record()
        torch.cuda.synchronize()
        times.append(start.elapsed_time(end))
    ms = sum(times) / len(times)
    print(f"Average execution time: {ms:.4f} ms")
    print(f"Performance: {flop / ms / 1e9:.2f} TFLOPS for {B=} {H=} {HKV=} {N=} {D=} {causal=} attention.")
    with torch.no_grad():
        g = H // HKV
        ref = torch.nn.functional.scaled_dot_product_attention(
            q.transpose(1, 2), k.repeat_interleave(g, 2).transpose(1, 2), v.repeat_interleave(g, 2).transpose(1, 2),
            is_causal=causal).transpose(1, 2)
    mx, err, tot, l2, cos = robustness_check(ref, out)
    print(f"O vs torch SDPA: max_abs={mx:.6f} rel_l2={l2:.4f} cos={cos:.6f} errors={err}/{tot}")
    print("status:", tk_kernel.device_status(q.device.index))

