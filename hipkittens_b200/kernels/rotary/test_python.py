"""Timing and accuracy harness for tk_kernel.dispatch_rotary on B200.

Same shapes and protocol as the reference's kernels/rotary/test_python.py: x [B=16, H=16, N=2048, D=128] bf16, cos and sin
[N, D/2] built in bf16 (test_python.py:36-45), the PyTorch expression x * cos + rotate_half(x) * sin as the comparison
target (test_python.py:48-58), CUDA events around each call. The result is expected to be bit-identical: both sides
round every product and the sum to bf16.
"""
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
import tk_kernel  # noqa: E402

B, H, N, D = 16, 16, 2048, 128


def get_cos_sin(n, dim, base=10000.0, dtype=torch.bfloat16, device="cuda"):
    t = torch.arange(n, device=device, dtype=dtype)
    inv_freq = 1.0 / (base ** (torch.arange(0, dim, 2, device=device, dtype=dtype) / dim))
    freqs = torch.outer(t, inv_freq).to(dtype=dtype)
    return torch.cos(freqs).to(dtype=dtype), torch.sin(freqs).to(dtype=dtype)


def reference(x, cos, sin):
    x1, x2 = x.chunk(2, dim=-1)
    rotated = torch.cat((-x2, x1), dim=-1)
    c = torch.cat((cos, cos), dim=-1)[None, None]
    s = torch.cat((sin, sin), dim=-1)[None, None]
    return x * c + rotated * s


def main():
    warmup, iters = int(os.environ.get("HK_WARMUP", 50)), int(os.environ.get("HK_ITERS", 100))
    torch.manual_seed(42)
    x = torch.randn((B, H, N, D), dtype=torch.bfloat16, device="cuda")
    cos, sin = get_cos_sin(N, D)
    o = torch.zeros_like(x)
    for _ in range(warmup):
        tk_kernel.dispatch_rotary(x, o, sin, cos)
    start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    times = []
    for _ in range(iters):
        torch.cuda.synchronize()
        start.record()
        tk_kernel.dispatch_rotary(x, o, sin, cos)
        end.record()
        torch.cuda.synchronize()
        times.append(start.elapsed_time(end))
    ms = sum(times) / len(times)
    print(f"Average execution time: {ms * 1e3:.1f} us, {2 * x.numel() * 2 / ms / 1e6:.0f} GB/s read + written")
    ref = reference(x, cos, sin)
    same = torch.equal(o.view(torch.int16), ref.view(torch.int16))
    print(f"bit-identical to the bf16 PyTorch expression: {same}; max |diff| = {float((o.float() - ref.float()).abs().max())}")


if __name__ == "__main__":
    main()
