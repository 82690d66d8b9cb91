"""Timing and accuracy harness for the backward modules on B200.

Same command line as the reference's kernels/attn/gqa_causal_backwards/test_python.py (B D H H_KV N causal); the protocol and
the statistics are in ../harness_bwd.py, shared with the harness of the sibling directory.
"""
import os
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, HERE)
sys.path.insert(0, os.path.dirname(HERE))
import harness_bwd  # noqa: E402
import tk_kernel_bkwd  # noqa: E402
import tk_kernel_bkwd_prep  # noqa: E402
import tk_kernel_fwd  # noqa: E402

ARG_ORDER = ("B", "D", "H", "H_KV", "N", "causal")
DEFAULTS = {"B": 16, "D": 128, "H": 64, "H_KV": 8, "N": 2048, "causal": int(tk_kernel_bkwd.default_causal)}


def parse(argv):
    return harness_bwd.parse(argv, ARG_ORDER, DEFAULTS)


if __name__ == "__main__":
    harness_bwd.run_backward(tk_kernel_fwd, tk_kernel_bkwd, tk_kernel_bkwd_prep, parse(sys.argv))
