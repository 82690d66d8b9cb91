"""The pybind11 modules keep the reference's calling surface and its argument checks
(include/pyutils/pyutils.cuh:14-47): same module and function names, same RuntimeError messages."""
import pytest
import torch

import hipkittens_b200 as hk


class _Dev:
    def __init__(self, type_="cuda", index=0):
        self.type = type_
        self.index = index


class Tensor:  # duck-typed stand-in: the shim only looks at the class name and a few attributes
    def __init__(self, shape, dtype="torch.bfloat16", contiguous=True, device="cuda", ptr=4096):
        self.shape = tuple(shape)
        self.dtype = dtype
        self._c = contiguous
        self.device = _Dev(device)
        self._ptr = ptr

    def is_contiguous(self):
        return self._c

    def data_ptr(self):
        return self._ptr


def _five(B=1, N=128, H=2, HKV=1, D=128):
    return [Tensor((B, N, H, D)), Tensor((B, N, HKV, D)), Tensor((B, N, HKV, D)), Tensor((B, N, H, D)),
            Tensor((B, H, 1, N), dtype="torch.float32")]


@pytest.fixture(scope="module")
def mods(native_built):
    return {
        "micro": hk.load_tk_kernel(False),
        "micro_causal": hk.load_tk_kernel(True),
        "fwd": hk.load_tk_kernel_fwd(False),
        "fwd_causal": hk.load_tk_kernel_fwd(True),
    }


def test_module_and_entry_names(mods):
    assert mods["micro"].__name__.endswith(".gqa.tk_kernel") and hasattr(mods["micro"], "dispatch_micro")
    assert mods["micro_causal"].__name__.endswith(".gqa_causal.tk_kernel")
    assert mods["fwd"].__name__.endswith(".tk_kernel_fwd") and hasattr(mods["fwd"], "dispatch_fwd")
    assert mods["micro"].default_causal is False and mods["micro_causal"].default_causal is True
    assert mods["fwd"].default_causal is False and mods["fwd_causal"].default_causal is True


def test_plain_import_from_the_kernel_directory(native_built):
    """`import tk_kernel` with the kernel directory on sys.path, as kernels/attn/gqa/test_python.py:2 does."""
    import os
    import subprocess
    import sys

    d = os.path.join(os.path.dirname(hk.__file__), "kernels", "attn", "gqa_causal")
    code = "import tk_kernel; assert tk_kernel.__name__ == 'tk_kernel' and tk_kernel.default_causal; print('ok')"
    out = subprocess.run([sys.executable, "-c", code], cwd=d, capture_output=True, text=True,
                         env={**os.environ, "PYTHONPATH": d})
    assert out.returncode == 0 and "ok" in out.stdout, out.stderr


def test_reference_error_messages(mods):
    f = mods["micro"].dispatch_micro
    args = _five()
    with pytest.raises(RuntimeError, match="Expected a torch.Tensor"):
        f(1.0, *args[1:])
    with pytest.raises(RuntimeError, match="Tensor must be contiguous"):
        f(Tensor((1, 128, 2, 128), contiguous=False), *args[1:])
    with pytest.raises(RuntimeError, match="Tensor must be on CUDA device"):
        f(Tensor((1, 128, 2, 128), device="cpu"), *args[1:])
    with pytest.raises(RuntimeError, match="Expected Tensor.ndim <= 4"):
        f(Tensor((1, 1, 128, 2, 128)), *args[1:])


def test_real_cpu_tensors_are_rejected_like_the_reference(mods):
    q = torch.zeros(1, 128, 2, 128, dtype=torch.bfloat16)
    kv = torch.zeros(1, 128, 1, 128, dtype=torch.bfloat16)
    lse = torch.zeros(1, 2, 1, 128)
    with pytest.raises(RuntimeError, match="Tensor must be on CUDA device"):
        mods["fwd"].dispatch_fwd(q, kv, kv, torch.zeros_like(q), lse)
    with pytest.raises(RuntimeError, match="Tensor must be contiguous"):
        mods["fwd"].dispatch_fwd(q.transpose(1, 2), kv, kv, torch.zeros_like(q), lse)
    # requires_grad leaves are accepted as far as the binding is concerned (test_python.py:30-32)
    q2 = q.clone().requires_grad_(True)
    with pytest.raises(RuntimeError, match="Tensor must be on CUDA device"):
        mods["micro"].dispatch_micro(q2, kv, kv, torch.zeros_like(q), lse)


def test_added_shape_and_dtype_checks(mods):
    f = mods["micro"].dispatch_micro
    a = _five()
    a[0] = Tensor((1, 128, 2, 128), dtype="torch.float16")
    with pytest.raises(RuntimeError, match="bfloat16"):
        f(*a)
    a = _five()
    a[4] = Tensor((1, 2, 1, 128), dtype="torch.float16")
    with pytest.raises(RuntimeError, match="float32"):
        f(*a)
    a = _five()
    a[4] = Tensor((1, 2, 128), dtype="torch.float32")  # [B,H,N] instead of [B,H,1,N]
    with pytest.raises(RuntimeError, match=r"\[B, H, 1, N\]"):
        f(*a)
    a = _five()
    a[2] = Tensor((1, 128, 2, 128))
    with pytest.raises(RuntimeError, match="k and v shapes differ"):
        f(*a)
    a = _five()
    a[3] = Tensor((1, 128, 4, 128))
    with pytest.raises(RuntimeError, match="out must have q's shape"):
        f(*a)


def test_c_abi_errors_surface_as_runtime_errors(mods):
    f = mods["micro"].dispatch_micro
    with pytest.raises(RuntimeError, match="invalid argument"):
        f(*_five(H=3, HKV=2))  # H not a multiple of H_KV
    with pytest.raises(RuntimeError, match="unsupported"):
        f(*_five(D=32))


@pytest.mark.skipif(torch.cuda.is_available(), reason="checks the no-GPU failure mode")
def test_no_silent_fallback_without_gpu(mods):
    with pytest.raises(RuntimeError, match="CUDA call failed"):
        mods["micro"].dispatch_micro(*_five())


def test_harness_keeps_both_reference_argument_orders(native_built):
    """kernels/attn/gqa/test_python.py takes B D H H_KV N causal, gqa_causal/test_python.py B N H H_KV causal D
    (test_python.py:22-27 in each directory); the harnesses shipped beside the modules keep both."""
    import importlib.util
    import os
    import sys

    base = os.path.join(os.path.dirname(hk.__file__), "kernels", "attn")
    got = {}
    for d in ("gqa", "gqa_causal"):
        path = os.path.join(base, d, "test_python.py")
        sys_path = list(sys.path)
        mods = {k: v for k, v in sys.modules.items() if k == "tk_kernel"}
        try:
            sys.modules.pop("tk_kernel", None)
            spec = importlib.util.spec_from_file_location(f"harness_{d}", path)
            mod = importlib.util.module_from_spec(spec)
            spec.loader.exec_module(mod)
            got[d] = mod.parse(["x", "2", "64", "8", "4", "256", "1"]) if d == "gqa" else mod.parse(
                ["x", "2", "256", "8", "4", "1", "64"])
            assert os.path.exists(os.path.join(base, d, "Makefile"))
        finally:
            sys.path[:] = sys_path
            sys.modules.pop("tk_kernel", None)
            sys.modules.update(mods)
    assert got["gqa"] == got["gqa_causal"] == {"B": 2, "D": 64, "H": 8, "H_KV": 4, "N": 256, "causal": 1}


# ---------------------------------------------------------------------------------------------- backward modules
@pytest.fixture(scope="module")
def bkwd_mods(native_built):
    return {c: (hk.load_tk_kernel_bkwd(c), hk.load_tk_kernel_bkwd_prep(c)) for c in (False, True)}


def _bwd_nine(B=1, N=128, H=2, HKV=1, D=128):
    q, kv, stat = (B, N, H, D), (B, N, HKV, D), (B, H, 1, N)
    return [Tensor(q), Tensor(kv), Tensor(kv), Tensor(q), Tensor((B, H, N, D)), Tensor(kv), Tensor(kv),
            Tensor(stat, dtype="torch.float32"), Tensor(stat, dtype="torch.float32")]


def test_backward_module_and_entry_names(bkwd_mods):
    """tk_kernel_bkwd.dispatch_bwd_combined, tk_kernel_bkwd_prep.dispatch_prep / dispatch_dq_shuffle
    (kernels/attn/gqa_backwards/attn_bkwd_non_causal.cpp:3171-3185, attn_bkwd_prep.cpp:227-240)."""
    for causal, (bk, prep) in bkwd_mods.items():
        assert bk.__name__.endswith(".tk_kernel_bkwd") and hasattr(bk, "dispatch_bwd_combined")
        assert prep.__name__.endswith(".tk_kernel_bkwd_prep")
        assert hasattr(prep, "dispatch_prep") and hasattr(prep, "dispatch_dq_shuffle")
        assert bk.default_causal is causal
        assert ("gqa_causal_backwards" in bk.__name__) == causal


def test_backward_argument_checks(bkwd_mods):
    bk, prep = bkwd_mods[False]
    args = _bwd_nine()
    with pytest.raises(RuntimeError, match="Expected a torch.Tensor"):
        bk.dispatch_bwd_combined(None, *args[1:])
    with pytest.raises(RuntimeError, match="Tensor must be on CUDA device"):
        bk.dispatch_bwd_combined(Tensor((1, 128, 2, 128), device="cpu"), *args[1:])
    bad = _bwd_nine()
    bad[4] = Tensor((1, 128, 2, 128))  # dQ_in given in the post-shuffle layout
    with pytest.raises(RuntimeError, match="pre-shuffle"):
        bk.dispatch_bwd_combined(*bad)
    bad = _bwd_nine()
    bad[7] = Tensor((1, 2, 1, 128))  # L as bf16
    with pytest.raises(RuntimeError, match="torch.float32"):
        bk.dispatch_bwd_combined(*bad)
    bad = _bwd_nine()
    bad[5] = Tensor((1, 128, 2, 128))  # dK with Q's head count
    with pytest.raises(RuntimeError, match="dK/dV"):
        bk.dispatch_bwd_combined(*bad)
    with pytest.raises(RuntimeError, match="delta must be"):
        prep.dispatch_prep(Tensor((1, 128, 2, 128)), Tensor((1, 128, 2, 128)),
                           Tensor((1, 2, 128, 1), dtype="torch.float32"))
    with pytest.raises(RuntimeError, match="Tensor must be contiguous"):
        prep.dispatch_dq_shuffle(Tensor((1, 2, 128, 128), contiguous=False), Tensor((1, 128, 2, 128)))
    with pytest.raises(RuntimeError, match=r"dQ_in must be \[B, H, N, D\]"):
        prep.dispatch_dq_shuffle(Tensor((1, 2, 128, 128)), Tensor((1, 2, 128, 128)))


def test_backward_has_no_silent_fallback_without_gpu(bkwd_mods):
    if torch.cuda.is_available():
        pytest.skip("a GPU is present")
    bk, prep = bkwd_mods[True]
    with pytest.raises(RuntimeError, match="CUDA call failed|unsupported"):
        bk.dispatch_bwd_combined(*_bwd_nine())
    with pytest.raises(RuntimeError, match="CUDA call failed|unsupported"):
        prep.dispatch_prep(Tensor((1, 128, 2, 128)), Tensor((1, 128, 2, 128)), Tensor((1, 2, 1, 128), dtype="torch.float32"))
