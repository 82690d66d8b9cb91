"""In-tree build of the native pieces: ``lib/libhk_attn.so`` (CUDA kernels + C ABI, nvcc, sm_100a only)
and the pybind11 modules that keep the reference's Python entry points.

The reference builds one ``tk_kernel`` extension per kernel directory with ``make`` and hipcc
(``kernels/attn/gqa/Makefile:32-69``); here the same module names are produced, from one shim source,
into directories that mirror the reference's:

    kernels/attn/gqa/tk_kernel                     dispatch_micro, non-causal default
    kernels/attn/gqa_causal/tk_kernel              dispatch_micro, causal default
    kernels/attn/gqa_backwards/tk_kernel_fwd       dispatch_fwd (blocking), non-causal default
    kernels/attn/gqa_causal_backwards/tk_kernel_fwd  dispatch_fwd (blocking), causal default
    kernels/attn/gqa{,_causal}_backwards/tk_kernel_bkwd       dispatch_bwd_combined
    kernels/attn/gqa{,_causal}_backwards/tk_kernel_bkwd_prep  dispatch_prep, dispatch_dq_shuffle
    kernels/rotary/tk_kernel                       dispatch_rotary

Run as ``python -m hipkittens_b200._build``. nvcc cross-compiles without a GPU.
"""
from __future__ import annotations

import os
import subprocess
import sys
import sysconfig

PKG = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(PKG, "csrc")
LIB_DIR = os.path.join(PKG, "lib")
LIB_PATH = os.path.join(LIB_DIR, "libhk_attn.so")
INCLUDE = os.path.join(os.path.dirname(PKG), "include")

NVCC_FLAGS = [
    "-gencode", "arch=compute_100a,code=sm_100a",
    "-O3", "-std=c++17", "-lineinfo",
    "-Xcompiler", "-fPIC", "-shared",
]

# (directory under the package, module name, entry name, default causal, sync after launch)
SHIMS = [
    ("kernels/attn/gqa", "tk_kernel", "dispatch_micro", 0, 0),
    ("kernels/attn/gqa_causal", "tk_kernel", "dispatch_micro", 1, 0),
    ("kernels/attn/gqa_backwards", "tk_kernel_fwd", "dispatch_fwd", 0, 1),
    ("kernels/attn/gqa_causal_backwards", "tk_kernel_fwd", "dispatch_fwd", 1, 1),
]


# (directory under the package, module name, HK_BKWD_PREP, default causal): the reference's two backward modules
# (kernels/attn/gqa_backwards/Makefile: tk_kernel_bkwd, tk_kernel_bkwd_prep)
BKWD_SHIMS = [
    ("kernels/attn/gqa_backwards", "tk_kernel_bkwd", 0, 0),
    ("kernels/attn/gqa_backwards", "tk_kernel_bkwd_prep", 1, 0),
    ("kernels/attn/gqa_causal_backwards", "tk_kernel_bkwd", 0, 1),
    ("kernels/attn/gqa_causal_backwards", "tk_kernel_bkwd_prep", 1, 1),
]


def _newer(target: str, sources) -> bool:
    if not os.path.exists(target):
        return False
    t = os.path.getmtime(target)
    return all(os.path.getmtime(s) <= t for s in sources)


def _run(cmd) -> None:
    proc = subprocess.run(cmd, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    if proc.returncode != 0:
        raise RuntimeError("build command failed:\n  " + " ".join(cmd) + "\n" + proc.stdout)


def nvcc_path() -> str:
    cand = os.path.join(os.environ.get("CUDA_HOME", "/usr/local/cuda"), "bin", "nvcc")
    return cand if os.path.exists(cand) else "nvcc"


def build_lib(force: bool = False) -> str:
    srcs = [os.path.join(CSRC, f) for f in os.listdir(CSRC) if f.endswith((".cu", ".cuh"))]
    srcs.append(os.path.join(INCLUDE, "hk_attn.h"))
    if not force and _newer(LIB_PATH, srcs):
        return LIB_PATH
    os.makedirs(LIB_DIR, exist_ok=True)
    _run([nvcc_path(), *NVCC_FLAGS, "-o", LIB_PATH, os.path.join(CSRC, "hk_attn_api.cu")])
    return LIB_PATH


def shim_path(subdir: str, module: str) -> str:
    return os.path.join(PKG, subdir, module + sysconfig.get_config_var("EXT_SUFFIX"))


def build_shims(force: bool = False):
    import pybind11

    src = os.path.join(CSRC, "tk_kernel_shim.cpp")
    common = os.path.join(CSRC, "shim_common.h")
    out = []
    for subdir, module, entry, causal, sync in SHIMS:
        target = shim_path(subdir, module)
        out.append(target)
        if not force and _newer(target, [src, common, os.path.join(INCLUDE, "hk_attn.h"), LIB_PATH]):
            continue
        os.makedirs(os.path.dirname(target), exist_ok=True)
        rel = os.path.relpath(LIB_DIR, os.path.dirname(target))
        _run([
            "g++", "-O2", "-std=c++17", "-shared", "-fPIC", "-fvisibility=hidden",
            f"-DHK_MODULE_NAME={module}", f'-DHK_ENTRY_NAME="{entry}"',
            f"-DHK_DEFAULT_CAUSAL={causal}", f"-DHK_SYNC_AFTER={sync}",
            "-I", pybind11.get_include(), "-I", sysconfig.get_paths()["include"],
            src, "-o", target,
            "-L", LIB_DIR, "-lhk_attn", f"-Wl,-rpath,$ORIGIN/{rel}",
        ])
    bsrc = os.path.join(CSRC, "tk_kernel_bkwd_shim.cpp")
    for subdir, module, prep, causal in BKWD_SHIMS:
        target = shim_path(subdir, module)
        out.append(target)
        if not force and _newer(target, [bsrc, common, os.path.join(INCLUDE, "hk_attn.h"), LIB_PATH]):
            continue
        os.makedirs(os.path.dirname(target), exist_ok=True)
        rel = os.path.relpath(LIB_DIR, os.path.dirname(target))
        _run([
            "g++", "-O2", "-std=c++17", "-shared", "-fPIC", "-fvisibility=hidden",
            f"-DHK_BKWD_PREP={prep}", f"-DHK_DEFAULT_CAUSAL={causal}",
            "-I", pybind11.get_include(), "-I", sysconfig.get_paths()["include"],
            bsrc, "-o", target,
            "-L", LIB_DIR, "-lhk_attn", f"-Wl,-rpath,$ORIGIN/{rel}",
        ])
    rsrc = os.path.join(CSRC, "tk_kernel_rotary_shim.cpp")
    target = shim_path("kernels/rotary", "tk_kernel")
    out.append(target)
    if force or not _newer(target, [rsrc, common, os.path.join(INCLUDE, "hk_attn.h"), LIB_PATH]):
        os.makedirs(os.path.dirname(target), exist_ok=True)
        rel = os.path.relpath(LIB_DIR, os.path.dirname(target))
        _run([
            "g++", "-O2", "-std=c++17", "-shared", "-fPIC", "-fvisibility=hidden",
            "-I", pybind11.get_include(), "-I", sysconfig.get_paths()["include"],
            rsrc, "-o", target,
            "-L", LIB_DIR, "-lhk_attn", f"-Wl,-rpath,$ORIGIN/{rel}",
        ])
    return out


def build_all(force: bool = False):
    lib = build_lib(force)
    shims = build_shims(force)
    return [lib, *shims]


if __name__ == "__main__":
    for path in build_all(force="--force" in sys.argv):
        print(path)
