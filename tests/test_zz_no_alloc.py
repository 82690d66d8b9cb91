"""hk_attn_paged_decode_static: the paged decode for callers that cannot allocate device memory (a serving
engine that gave all of HBM to its own allocator; a decode loop that must never hit cudaMalloc's device-wide
synchronisation). Its scratch is a fixed array inside the library, so the things to check are that it computes
exactly what hk_attn_paged_decode computes, that a second call is not disturbed by what the first one left in
the shared array, that problems beyond the array's size are refused, and that the device's free memory is the
same before and after warm calls.

Collected last on purpose (file name): if it fails under -x every other test has already run.
"""
import ctypes
import os
import subprocess
import sys

import pytest
import torch

import hipkittens_b200 as hk
from hipkittens_b200 import _native
from hipkittens_b200.synthetic import make_paged_inputs

pytestmark = pytest.mark.gpu


def _call_static(lib, q, kp, vp, bt, cl, o, l, want_status=True):
    s, _, h, d = q.shape
    status = ctypes.c_int(-99)
    rc = lib.hk_attn_paged_decode_static(
        q.data_ptr(), kp.data_ptr(), vp.data_ptr(), bt.data_ptr(), cl.data_ptr(), o.data_ptr(), l.data_ptr(),
        s, h, kp.shape[2], d, kp.shape[1], bt.shape[1], kp.shape[0], 0.0, q.device.index,
        torch.cuda.current_stream(q.device).cuda_stream, ctypes.byref(status) if want_status else None)
    return rc, status.value


def _problem(dev, s, h, hkv, pool, lo, hi, seed):
    q, kp, vp, bt, cl = make_paged_inputs(s, h, hkv, 128, 16, pool, lo, hi, seed)
    return [t.to(dev) for t in (q, kp, vp, bt, cl)]


def test_static_scratch_variant_matches_workspace_variant_twice():
    dev = torch.device("cuda:0")
    lib = hk.capi()
    # call 1: multi-chunk sequences (partials go through the built-in array); call 2: a different, smaller
    # problem whose slots overlap the ones call 1 left behind
    for (s, h, hkv, pool, lo, hi, seed) in [(6, 16, 2, 900, 600, 2000, 21), (3, 8, 1, 400, 1, 1500, 22)]:
        q, kp, vp, bt, cl = _problem(dev, s, h, hkv, pool, lo, hi, seed)
        o_ref, l_ref = hk.paged_decode(q, kp, vp, bt, cl)  # existing entry point, caller-provided workspace
        assert _native.device_status(0) == 0
        o = torch.full_like(o_ref, float("nan"))
        l = torch.full_like(l_ref, float("nan"))
        rc, status = _call_static(lib, q, kp, vp, bt, cl, o, l)
        assert rc == 0 and status == 0
        # same kernels, same inputs: the build's tolerances (2e-2 on O, 1e-3 on L) are met with zero error
        assert float((o.float() - o_ref.float()).abs().max()) <= 2e-2
        assert float((l - l_ref).abs().max()) <= 1e-3
        assert torch.equal(o, o_ref) and torch.equal(l, l_ref)


def test_asynchronous_form_and_status_reporting():
    dev = torch.device("cuda:0")
    lib = hk.capi()
    q, kp, vp, bt, cl = _problem(dev, 2, 8, 1, 300, 700, 1200, 23)
    o_ref, l_ref = hk.paged_decode(q, kp, vp, bt, cl)
    o = torch.empty_like(o_ref)
    l = torch.empty_like(l_ref)
    rc, _ = _call_static(lib, q, kp, vp, bt, cl, o, l, want_status=False)  # no status_out: returns at once
    assert rc == 0
    torch.cuda.synchronize()
    assert torch.equal(o, o_ref) and torch.equal(l, l_ref)
    # an out-of-range page id is reported through status_out and not dereferenced ...
    bad = bt.clone()
    bad[0, 1] = kp.shape[0] + 5
    rc, status = _call_static(lib, q, kp, vp, bad, cl, o, l)
    assert rc == 0 and status == _native.HK_EBADPAGE
    # ... and the next call starts from a cleared status word
    rc, status = _call_static(lib, q, kp, vp, bt, cl, o, l)
    assert rc == 0 and status == 0 and torch.equal(o, o_ref)


def test_problems_beyond_the_built_in_array_are_refused():
    dev = torch.device("cuda:0")
    lib = hk.capi()
    q, kp, vp, bt, cl = _problem(dev, 2, 8, 1, 300, 100, 200, 24)
    o = torch.empty_like(q)
    l = torch.empty((2, 8, 1, 1), dtype=torch.float32, device=dev)
    limit = 8 << 20
    assert hk.paged_decode_workspace_bytes(16, 64, 128, 480) <= limit < hk.paged_decode_workspace_bytes(16, 64, 128, 512)
    status = ctypes.c_int(-99)
    # S=64, H=64, 8192-token sequences need 34 MB of partials: refused before any launch
    rc = lib.hk_attn_paged_decode_static(q.data_ptr(), kp.data_ptr(), vp.data_ptr(), bt.data_ptr(), cl.data_ptr(),
                                         o.data_ptr(), l.data_ptr(), 64, 64, 8, 128, 16, 512, 40000, 0.0, 0, None,
                                         ctypes.byref(status))
    assert rc == _native.HK_EWORKSPACE and status.value == -99
    assert b"built-in array" in lib.hk_last_cuda_error()


def test_warm_calls_leave_the_free_device_memory_unchanged():
    """The property in the entry point's name: once the first call on the device has happened, later calls take
    nothing from the device's memory. The driver's own count of free bytes is read before and after the second and
    third call (torch's caching allocator is not involved: the call gets raw pointers)."""
    dev = torch.device("cuda:0")
    lib = hk.capi()
    q, kp, vp, bt, cl = _problem(dev, 6, 16, 2, 900, 600, 2000, 25)
    o = torch.empty_like(q)
    l = torch.empty((6, 16, 1, 1), dtype=torch.float32, device=dev)
    rc, status = _call_static(lib, q, kp, vp, bt, cl, o, l)   # first call: one-time set-up may happen here
    assert rc == 0 and status == 0
    torch.cuda.synchronize()
    free_before = torch.cuda.mem_get_info(dev)[0]
    for _ in range(2):
        rc, status = _call_static(lib, q, kp, vp, bt, cl, o, l)
        assert rc == 0 and status == 0
        torch.cuda.synchronize()
        assert torch.cuda.mem_get_info(dev)[0] == free_before


def test_static_entry_as_the_first_library_call_of_a_process():
    """In a fresh process the static entry is the first hk_* call on the device, so its own set-up (address
    look-up of the built-in array, kernel attributes) is what runs, not the ordinary entry's. The child also checks
    that the caller's current device is what it was."""
    code = r"""
import ctypes, sys, torch
sys.path.insert(0, %r)
import hipkittens_b200 as hk
from hipkittens_b200.synthetic import make_paged_inputs
dev = torch.device("cuda:0")
q, kp, vp, bt, cl = [t.to(dev) for t in make_paged_inputs(3, 8, 1, 128, 16, 400, 1, 1500, 22)]
o = torch.empty_like(q); l = torch.empty((3, 8, 1, 1), dtype=torch.float32, device=dev)
lib = hk.capi()
assert lib.hk_kernel_launch_count() == 0
status = ctypes.c_int(-99)
rc = lib.hk_attn_paged_decode_static(q.data_ptr(), kp.data_ptr(), vp.data_ptr(), bt.data_ptr(), cl.data_ptr(),
        o.data_ptr(), l.data_ptr(), 3, 8, 1, 128, 16, bt.shape[1], kp.shape[0], 0.0, 0,
        torch.cuda.current_stream(dev).cuda_stream, ctypes.byref(status))
assert rc == 0 and status.value == 0, (rc, status.value, lib.hk_last_cuda_error())
o_ref, l_ref = hk.paged_decode(q, kp, vp, bt, cl)
torch.cuda.synchronize()
assert torch.equal(o, o_ref) and torch.equal(l, l_ref)
print("ok")
""" % os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    out = subprocess.run([sys.executable, "-c", code], capture_output=True, text=True, timeout=300)
    assert out.returncode == 0 and out.stdout.strip().endswith("ok"), out.stdout + out.stderr
