"""Timing and accuracy harness for tk_kernel.dispatch_micro on B200.

Same command line as the reference's kernels/attn/gqa/test_python.py (B D H H_KV N causal); the protocol and the
statistics are in ../harness_fwd.py, shared with the harness of the sibling directory.
"""
import os
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, HERE)
sys.path.insert(0, os.path.dirname(HERE))
import harness_fwd  # noqa: E402
import tk_kernel  # noqa: E402

ARG_ORDER = ('B', 'D', 'H', 'H_KV', 'N', 'causal')
DEFAULTS = {"B": 16, "D": 128, "H": 64, "H_KV": 8, "N": 2048, "causal": int(tk_kernel.default_causal)}


def parse(argv):
    return harness_fwd.parse(argv, ARG_ORDER, DEFAULTS)


if __name__ == "__main__":
    harness_fwd.run_forward(tk_kernel, parse(sys.argv))
