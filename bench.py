#!/usr/bin/env python
"""Benchmark of the bf16 GQA attention forward (and backward, and paged decode) on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload NAME] [--impl ours|reference]

A step is one pass of the hot path over one batch of synthetic input (one kernel launch for the
forward; split + combine launches for decode; delta prep + dK/dV + dQ launches for the backward). The default workload is the reference README's default
shape: B=16, N=2048, H=64, H_KV=8, D=128, non-causal (kernels/attn/gqa/test_python.py:22-27).
TFLOPS = 4*B*N^2*H*D / (2 if causal) / time, the reference's convention (test_python.py:35-38).

With N > 1 (torchrun, one rank per GPU) the one workload's (batch, kv-head) units are dealt to the ranks with
hipkittens_b200.shard.partition_units (strong scaling; the units are independent, there is no collective on the
data path) and `value` is the workload's FLOP divided by the slowest rank's time. Outside the timed region the ranks
then check their shards on the GPU (`shard_parity`: NCCL gather of O and L against one single-GPU launch) and time the
replica arrangement as well (`replicas`: every rank the whole workload on its own inputs). `--scaling weak` makes
the replica arrangement the headline instead.

The default single-GPU run also times the other configurations for K steps each (`other_workloads`: causal N = 8192,
D = 64 MHA, paged decode, the backward) and runs the headline workload back to back for two seconds
(`sustained`), after the headline numbers have been taken.

One JSON line is printed by rank 0.
"""
from __future__ import annotations

import argparse
import json
import math
import os
import statistics
import sys
import threading
import time

import torch

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

WORKLOADS = {
    # name: (kind, B, N, H, H_KV, D, causal)
    "gqa_fwd_b16_n2048_h64_kv8_d128": ("fwd", 16, 2048, 64, 8, 128, False),
    "gqa_causal_fwd_b4_n8192_h64_kv8_d128": ("fwd", 4, 8192, 64, 8, 128, True),
    "mha_fwd_b16_n4096_h16_d64": ("fwd", 16, 4096, 16, 16, 64, False),
    "paged_decode_s64_ctx512_8192_h64_kv8_d128": ("decode", 64, 0, 64, 8, 128, False),
    # backward pass (delta prep + dK/dV kernel + dQ kernel), flops = 2.5 x forward (kernels/attn/gqa_backwards/test_python.py:45-48)
    "gqa_bwd_b16_n2048_h64_kv8_d128": ("bwd", 16, 2048, 64, 8, 128, False),
    "gqa_causal_bwd_b4_n8192_h64_kv8_d128": ("bwd", 4, 8192, 64, 8, 128, True),
    "mha_bwd_b16_n4096_h16_d64": ("bwd", 16, 4096, 16, 16, 64, False),
    # the two byte-moving neighbours of the path: rotary pre-pass (the reference harness's shape, kernels/rotary/test_python.py:10-13)
    # and the KV-cache append of one prefill chunk (16 sequences x 2048 new tokens)
    "rotary_b16_h16_n2048_d128": ("rotary", 16, 2048, 16, 16, 128, False),
    "paged_kv_append_s16_t2048_kv8_d128": ("append", 16, 2048, 64, 8, 128, False),
    # reduced copies of the above for ncu captures (same kernels and tile shapes, inputs still beyond L2)
    "profile_gqa_fwd_b4_n2048_h64_kv8_d128": ("fwd", 4, 2048, 64, 8, 128, False),
    "profile_gqa_causal_fwd_b2_n8192_h64_kv8_d128": ("fwd", 2, 8192, 64, 8, 128, True),
    "profile_mha_fwd_b8_n4096_h16_d64": ("fwd", 8, 4096, 16, 16, 64, False),
    "profile_paged_decode_s14_ctx512_8192_h64_kv8_d128": ("decode", 14, 0, 64, 8, 128, False),
    "profile_gqa_bwd_b4_n2048_h64_kv8_d128": ("bwd", 4, 2048, 64, 8, 128, False),
    "profile_gqa_causal_bwd_b1_n8192_h64_kv8_d128": ("bwd", 1, 8192, 64, 8, 128, True),
}
DECODE_POOL_PAGES = {"paged_decode_s64_ctx512_8192_h64_kv8_d128": 40000,
                     "profile_paged_decode_s14_ctx512_8192_h64_kv8_d128": 8000}
DEFAULT_WORKLOAD = "gqa_fwd_b16_n2048_h64_kv8_d128"

# dram__bytes_read.sum + dram__bytes_write.sum per launch of the dominant kernel, from the ncu captures
# summarised under profiles/ (None = not captured for that workload).
NCU_TRAFFIC_BYTES = {
    # 4 x the B=4 capture (264.7 MB per launch; traffic grows with the (batch, kv-head) units)
    "gqa_fwd_b16_n2048_h64_kv8_d128": 4 * 264.7e6,
    # 2 x the B=2 / B=8 captures (profiles/attn_fwd_kernel_causal_d128_and_mha_d64.md)
    "gqa_causal_fwd_b4_n8192_h64_kv8_d128": 2 * (337.2e6 + 237.8e6),
    "mha_fwd_b16_n4096_h16_d64": 2 * (201.4e6 + 50.0e6),
    # backward, 4 x the B=4 capture of the two main kernels (profiles/attn_bwd_kernels_gqa_bwd_d128.md) + the prep kernel
    "gqa_bwd_b16_n2048_h64_kv8_d128": 4 * (363.0e6 + 416.4e6) + 1.082e9,
    # rate x duration of the section capture (profiles/rotary_kernel_and_paged_kv_append_kernel.md)
    "rotary_b16_h16_n2048_d128": 216.6e6,
    "paged_kv_append_s16_t2048_kv8_d128": 222.6e6,
    # 14-sequence capture (280.26 MB for sum ctx 66 608) scaled by sum ctx to 275 479; split + combine
    "paged_decode_s64_ctx512_8192_h64_kv8_d128": (273.46e6 + 4.73e6 + 2.47e6) * 275479 / 66608,
}

FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0}


def load_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    try:
        with open(path) as f:
            d = json.load(f)
        return {k: float(d[k]) for k in FALLBACK_PEAKS}, "measured"
    except Exception:
        return dict(FALLBACK_PEAKS), "fallback"


def fwd_flops(b, n, h, d, causal):
    return 4 * b * n * n * h * d // (2 if causal else 1)


def bwd_flops(b, n, h, d, causal):
    """The reference's convention: 2.5 x the forward count (five products instead of two)."""
    return 5 * fwd_flops(b, n, h, d, causal) // 2


# ------------------------------------------------------------------------------------------ clocks
class ClockSampler:
    """Samples SM clock and throttle reasons through NVML (read-only) while the GPU is under load."""

    REASONS = {
        0x4: "sw_power_cap",
        0x8: "hw_slowdown",
        0x20: "sw_thermal_slowdown",
        0x40: "hw_thermal_slowdown",
        0x80: "hw_power_brake_slowdown",
    }

    def __init__(self, device_index: int, period_s: float = 0.004):
        self.period = period_s
        self.samples = []
        self.tag = None   # name of the timed region in progress (None outside timed regions)
        self._stop = threading.Event()
        self._thread = None
        self.sm_max = None
        self.handle = None
        try:
            import pynvml

            self.nv = pynvml
            pynvml.nvmlInit()
            uuid = str(torch.cuda.get_device_properties(device_index).uuid)
            if not uuid.startswith("GPU-"):
                uuid = "GPU-" + uuid
            try:
                self.handle = pynvml.nvmlDeviceGetHandleByUUID(uuid.encode())
            except Exception:
                self.handle = pynvml.nvmlDeviceGetHandleByIndex(device_index)
            self.sm_max = int(pynvml.nvmlDeviceGetMaxClockInfo(self.handle, pynvml.NVML_CLOCK_SM))
        except Exception:
            self.handle = None

    def _loop(self):
        nv = self.nv
        while not self._stop.is_set():
            try:
                mhz = int(nv.nvmlDeviceGetClockInfo(self.handle, nv.NVML_CLOCK_SM))
                try:
                    mask = int(nv.nvmlDeviceGetCurrentClocksEventReasons(self.handle))
                except Exception:
                    mask = int(nv.nvmlDeviceGetCurrentClocksThrottleReasons(self.handle))
                self.samples.append((self.tag, mhz, mask))
            except Exception:
                pass
            self._stop.wait(self.period)

    def start(self):
        if self.handle is not None:
            self._thread = threading.Thread(target=self._loop, daemon=True)
            self._thread.start()

    def stop(self):
        self._stop.set()
        if self._thread is not None:
            self._thread.join(timeout=2)

    def summary(self, tag="timed"):
        """Median SM clock and the union of throttle reasons over the samples taken while region `tag` was timed
        (over all samples when that region was too short to be sampled three times)."""
        if self.handle is None or not self.samples:
            return {"sm_mhz": None, "sm_max_mhz": self.sm_max, "reasons": [], "samples": 0}
        timed = [s for s in self.samples if s[0] == tag]
        use = timed if len(timed) >= 3 else self.samples
        mask = 0
        for s in use:
            mask |= s[2]
        reasons = [name for bit, name in self.REASONS.items() if mask & bit]
        return {
            "sm_mhz": statistics.median(s[1] for s in use),
            "sm_max_mhz": self.sm_max,
            "reasons": reasons,
            "samples": len(use),
            "window": "timed" if use is timed else "whole run",
        }


# ------------------------------------------------------------------------------------------ CPU arm
def cpu_prefill_sample(b, n, h, hkv, d, causal, budget_s: float, max_units: int):
    """Times the oracle on (batch, kv-head) units of the workload's shape until `budget_s` is spent.
    Returns (flops_done, seconds, units_done)."""
    from hipkittens_b200.synthetic import make_prefill_inputs
    from oracle.attn_oracle import attn_fwd_oracle

    g = h // hkv
    q, k, v = make_prefill_inputs(1, n, g, 1, d, seed=123)
    attn_fwd_oracle(q[:, :128], k[:, :128], v[:, :128], causal)  # warm the thread pool
    done, t0 = 0, time.perf_counter()
    while done < max_units:
        attn_fwd_oracle(q, k, v, causal)
        done += 1
        if time.perf_counter() - t0 >= budget_s:
            break
    dt = time.perf_counter() - t0
    return done * fwd_flops(1, n, g, d, causal), dt, done


def cpu_bwd_sample(b, n, h, hkv, d, causal, budget_s: float, max_units: int):
    """Times the backward oracle on (batch, kv-head) units of the workload's shape until `budget_s` is spent."""
    from hipkittens_b200.synthetic import make_prefill_inputs
    from oracle.attn_oracle import attn_bwd_oracle

    g = h // hkv
    q, k, v = make_prefill_inputs(1, n, g, 1, d, seed=123)
    d_o = make_prefill_inputs(1, n, g, 1, d, seed=124)[0]
    attn_bwd_oracle(q[:, :128], k[:, :128], v[:, :128], d_o[:, :128], causal)  # warm the thread pool
    done, t0 = 0, time.perf_counter()
    while done < max_units:
        attn_bwd_oracle(q, k, v, d_o, causal)
        done += 1
        if time.perf_counter() - t0 >= budget_s:
            break
    dt = time.perf_counter() - t0
    return done * bwd_flops(1, n, g, d, causal), dt, done


def cpu_decode_sample(budget_s: float):
    from hipkittens_b200.synthetic import make_paged_inputs
    from oracle.attn_oracle import paged_decode_oracle

    q, kp, vp, bt, cl = make_paged_inputs(8, 64, 8, 128, 16, 4200, 512, 8192, seed=0)
    done, t0 = 0, time.perf_counter()
    toks = 0
    while True:
        paged_decode_oracle(q, kp, vp, bt, cl)
        done += 1
        toks += 8
        if time.perf_counter() - t0 >= budget_s:
            break
    return toks, int(cl.sum()) * done, time.perf_counter() - t0, done


# ------------------------------------------------------------------------------------------ workloads on the device
L2_BYTES = 126e6


def workload_config(name: str) -> dict:
    """The `config` object of a workload: printed identically by the GPU arm and by the reference arm."""
    kind, b, n, h, hkv, d, causal = WORKLOADS[name]
    if kind == "decode":
        return {"workload": name, "S": b, "H": h, "H_KV": hkv, "D": d, "page": 16,
                "pool_pages": DECODE_POOL_PAGES[name], "ctx": "U{512..8192}", "cache": "inputs_exceed_l2"}
    in_bytes = 2 * b * n * d * (h + 2 * hkv) * (2 if kind == "bwd" else 1)
    return {"workload": name, "B": b, "N": n, "H": h, "H_KV": hkv, "D": d, "causal": causal,
            "cache": "inputs_exceed_l2" if in_bytes > L2_BYTES else "inputs_fit_l2"}


class PrefillRun:
    """One rank's share of a forward or backward workload, resident in HBM.

    `slices` (from hipkittens_b200.shard.partition_units) selects this rank's (batch, kv-head) units of the one
    seeded workload; None = the whole workload. When the share's inputs would fit in L2, several differently
    seeded input sets are kept and the steps rotate through them, so that no step finds its inputs cached by the
    previous one."""

    def __init__(self, hk, dev, stream, kind, b, n, h, hkv, d, causal, seed, slices=None):
        from hipkittens_b200.shard import shard_tensors
        from hipkittens_b200.synthetic import make_prefill_inputs

        self.hk, self.kind, self.causal, self.stream, self.n, self.d = hk, kind, causal, stream, n, d
        self.sets = []
        self.members = []
        n_sets = 1
        while True:
            qf, kf, vf = make_prefill_inputs(b, n, h, hkv, d, seed=seed + 7919 * len(self.sets))
            if slices is None:
                parts = [(qf, kf, vf, None)]
            else:
                parts = shard_tensors(qf, kf, vf, hkv, slices)
            shards = [(qs.to(dev), ks.to(dev), vs.to(dev)) for qs, ks, vs, _m in parts]
            if not self.sets:
                self.members = [m for _q, _k, _v, m in parts]
                self.in_bytes = sum(t.numel() * 2 for sh in shards for t in sh) * (2 if kind == "bwd" else 1)
                if self.in_bytes <= L2_BYTES:
                    n_sets = int(L2_BYTES // max(self.in_bytes, 1)) + 2
            outs = [(torch.empty_like(qs), torch.empty((qs.shape[0], qs.shape[2], 1, n), dtype=torch.float32,
                                                       device=dev)) for qs, _k, _v in shards]
            bwd_in = None
            if kind == "bwd":
                # the backward's inputs: dO (seeded), and O and L from one forward pass outside the timed region
                gen = torch.Generator(device=dev).manual_seed(1000 + seed + len(self.sets))
                bwd_in = []
                for (qs, ks, vs), (o, l) in zip(shards, outs):
                    hk.attn_fwd(qs, ks, vs, causal=causal, out=o, lse=l, stream=stream)
                    d_o = torch.randn(qs.shape, generator=gen, device=dev).to(torch.bfloat16)
                    bwd_in.append((d_o, torch.empty_like(l), torch.empty_like(qs), torch.empty_like(ks),
                                   torch.empty_like(vs)))
            self.sets.append((shards, outs, bwd_in))
            del qf, kf, vf
            if len(self.sets) >= n_sets:
                break
        flops_of = fwd_flops if kind == "fwd" else bwd_flops
        self.flops = sum(flops_of(qs.shape[0], n, qs.shape[2], d, causal) for qs, _k, _v in self.sets[0][0])
        self.launches_per_step = len(self.sets[0][0]) * (1 if kind == "fwd" else 3)
        self.cache = ("inputs_exceed_l2" if len(self.sets) == 1 else
                      f"inputs_exceed_l2 (steps rotate through {len(self.sets)} input sets of {self.in_bytes / 1e6:.0f} MB)")

    def step(self, i: int = 0):
        hk, stream, causal = self.hk, self.stream, self.causal
        shards, outs, bwd_in = self.sets[i % len(self.sets)]
        if self.kind == "fwd":
            for (qs, ks, vs), (o, l) in zip(shards, outs):
                hk.attn_fwd(qs, ks, vs, causal=causal, out=o, lse=l, stream=stream)
        else:
            for (qs, ks, vs), (o, l), (d_o, delta, dq, dk, dv) in zip(shards, outs, bwd_in):
                hk.attn_bwd_prep(o, d_o, delta, stream=stream)
                hk.attn_bwd(qs, ks, vs, d_o, l, delta, causal=causal, dq=dq, dk=dk, dv=dv, stream=stream)


class DecodeRun:
    def __init__(self, hk, dev, stream, name, b, h, hkv, d, seed):
        from hipkittens_b200.synthetic import make_paged_inputs

        q, kp, vp, bt, cl = make_paged_inputs(b, h, hkv, d, 16, DECODE_POOL_PAGES[name], 512, 8192, seed=seed,
                                               pool_on=str(dev))
        self.hk, self.stream = hk, stream
        self.q, self.bt, self.cl, self.kp, self.vp = q.to(dev), bt.to(dev), cl.to(dev), kp, vp
        self.ws = torch.empty(hk.paged_decode_workspace_bytes(b, h, d, bt.shape[1]), dtype=torch.uint8, device=dev)
        self.o = torch.empty_like(self.q)
        self.l = torch.empty((b, h, 1, 1), dtype=torch.float32, device=dev)
        self.sum_ctx = int(cl.sum())
        self.tokens = float(b)                          # tokens generated per step
        self.kv_bytes = 2 * self.sum_ctx * hkv * d * 2  # K and V of the live context, once
        self.launches_per_step = 2
        self.cache = "inputs_exceed_l2"

    def step(self, i: int = 0):
        self.hk.paged_decode(self.q, self.kp, self.vp, self.bt, self.cl, out=self.o, lse=self.l, workspace=self.ws,
                             stream=self.stream)


def time_steps(run, steps, warmup, stream, barrier, sampler=None, tag=None):
    """W untimed steps, then K steps between two events on the launching stream, a barrier and a device
    synchronisation on both sides. Returns the milliseconds between the events."""
    for i in range(warmup):
        run.step(i)
    barrier()
    e0 = torch.cuda.Event(enable_timing=True)
    e1 = torch.cuda.Event(enable_timing=True)
    if sampler is not None:
        sampler.tag = tag
    e0.record(stream)
    for i in range(steps):
        run.step(i)
    e1.record(stream)
    barrier()
    if sampler is not None:
        sampler.tag = None
    return e0.elapsed_time(e1)


def prefill_roofline(name, kind, ach_tflops, peaks, peaks_src, flops_per_launch):
    r = {"bound": "tensor", "achieved": ach_tflops, "peak": peaks["bf16_tflops"], "unit": "TFLOP/s",
         "frac": ach_tflops / peaks["bf16_tflops"], "peak_sustained": peaks["bf16_tflops_sustained"],
         "frac_of_sustained": ach_tflops / peaks["bf16_tflops_sustained"],
         "peak_kind": f"of {peaks_src} (burst cuBLAS bf16)", "traffic": NCU_TRAFFIC_BYTES.get(name),
         "flops_per_launch": flops_per_launch}
    if kind == "bwd":
        r["note"] = ("a step is three launches (delta prep, dK/dV kernel, dQ kernel) timed together; flops are the "
                     "reference's 2.5 x forward count, the recomputation of S and dP in the second kernel is not counted")
    return r


def decode_roofline(name, ach_gbs, peaks, peaks_src, kv_bytes):
    return {"bound": "hbm", "achieved": ach_gbs, "peak": peaks["hbm_gbs"], "unit": "GB/s",
            "frac": ach_gbs / peaks["hbm_gbs"], "peak_kind": f"of {peaks_src} (copy)",
            "traffic": NCU_TRAFFIC_BYTES.get(name), "bytes_per_launch": kv_bytes}


METRIC = {
    "fwd": "bf16 GQA attn-fwd TFLOPS (4*B*N^2*H*D, /2 causal)",
    "bwd": "bf16 GQA attn-bwd TFLOPS (2.5 * 4*B*N^2*H*D, /2 causal; delta prep + dK/dV + dQ kernels)",
    "decode": "paged-KV GQA decode tokens/s",
}
# The other configurations of the benchmark, timed after the headline workload in the default single-GPU run.
OTHER_WORKLOADS = ["gqa_causal_fwd_b4_n8192_h64_kv8_d128", "mha_fwd_b16_n4096_h16_d64",
                   "paged_decode_s64_ctx512_8192_h64_kv8_d128", "gqa_bwd_b16_n2048_h64_kv8_d128",
                   "gqa_causal_bwd_b4_n8192_h64_kv8_d128"]


def run_other_workloads(hk, _native, dev, stream, local_rank, sampler, barrier, peaks, peaks_src, steps, warmup):
    """One entry per remaining configuration: same timing rules as the headline (W warm-up steps, K timed steps
    between events on the launching stream, clocks sampled during the timed steps)."""
    out = []
    for name in OTHER_WORKLOADS:
        kind, b, n, h, hkv, d, causal = WORKLOADS[name]
        if kind == "decode":
            run = DecodeRun(hk, dev, stream, name, b, h, hkv, d, seed=0)
        else:
            run = PrefillRun(hk, dev, stream, kind, b, n, h, hkv, d, causal, seed=0)
        l0 = hk.kernel_launch_count()
        ms = time_steps(run, steps, warmup, stream, barrier, sampler, tag=name) / steps
        launches = hk.kernel_launch_count() - l0 - warmup * run.launches_per_step
        if _native.device_status(local_rank) != 0:
            raise SystemExit(f"device status non-zero after {name}")
        entry = {"workload": name, "metric": METRIC[kind], "steps": steps, "warmup": warmup, "ms_per_step": ms,
                 "gpu_launches": int(launches), "config": dict(workload_config(name), cache=run.cache)}
        if kind == "decode":
            entry.update({"value": run.tokens / (ms * 1e-3), "unit": "tokens/s",
                          "roofline": decode_roofline(name, run.kv_bytes / (ms * 1e-3) / 1e9, peaks, peaks_src,
                                                      run.kv_bytes)})
            entry["roofline"]["sum_ctx"] = run.sum_ctx
        else:
            tf = run.flops / (ms * 1e-3) / 1e12
            entry.update({"value": tf, "unit": "TFLOP/s",
                          "roofline": prefill_roofline(name, kind, tf, peaks, peaks_src, run.flops)})
        entry["clocks"] = sampler.summary(name)
        out.append(entry)
        del run
        torch.cuda.empty_cache()
    return out


def run_sustained(hk, run, stream, barrier, sampler, seconds, ms_per_step_hint, flops):
    """The headline workload back to back for at least `seconds`: the figure a long job sees once the part sits at
    its power limit, beside the burst figure of the K-step run. Clocks are sampled, never set."""
    steps = max(50, int(math.ceil(seconds * 1e3 / max(ms_per_step_hint, 1e-3) * 1.25)))
    ms = time_steps(run, steps, 0, stream, barrier, sampler, tag="sustained")
    c = sampler.summary("sustained")
    return {"steps": steps, "seconds": ms * 1e-3, "ms_per_step": ms / steps, "value": flops * steps / (ms * 1e-3) / 1e12,
            "unit": "TFLOP/s", "sm_mhz_median": c["sm_mhz"], "sm_max_mhz": c["sm_max_mhz"], "reasons": c["reasons"],
            "samples": c["samples"]}


def fp32_attention_on_device(q, k, v, causal):
    """fp32 restatement of the math for ONE (batch, kv-head) unit, evaluated with torch on the GPU; a checker for
    the shard parity report, not part of any timed region. q [N,G,D], k, v [N,D] -> O [N,G,D] fp32, L [G,N]."""
    n, g, d = q.shape
    s = torch.einsum("ngd,md->gnm", q.float(), k.float()) / math.sqrt(d)
    if causal:
        s = s.masked_fill(torch.ones(n, n, dtype=torch.bool, device=q.device).triu(1), float("-inf"))
    lse = torch.logsumexp(s, dim=-1)
    o = torch.einsum("gnm,md->ngd", torch.softmax(s, dim=-1), v.float())
    return o, lse


def shard_parity_report(hk, dist, run, dev, stream, rank, world, b, n, h, hkv, d, causal):
    """Outside every timed region: (1) every rank checks one unit of its own O / L shard against the fp32
    restatement on its GPU; (2) the O and L shards of all ranks are gathered with NCCL (all_gather_into_tensor when
    the shards have one shape, else one broadcast per rank) and rank 0 compares the reassembled tensors with one
    single-GPU launch on the whole workload from the same seed. Returns the dict rank 0 prints."""
    from hipkittens_b200.shard import partition_units, scatter_outputs
    from hipkittens_b200.synthetic import make_prefill_inputs

    g = h // hkv
    shards, outs, _ = run.sets[0]
    for (qs, ks, vs), (o, l) in zip(shards, outs):
        hk.attn_fwd(qs, ks, vs, causal=causal, out=o, lse=l, stream=stream)
    torch.cuda.synchronize()
    (qs, ks, vs), (o, l) = shards[0], outs[0]
    o_ref, l_ref = fp32_attention_on_device(qs[0, :, :g], ks[0, :, 0], vs[0, :, 0], causal)
    unit_err = torch.tensor([float((o[0, :, :g].float() - o_ref).abs().max()),
                             float((l[0, :g, 0] - l_ref).abs().max())], dtype=torch.float64, device=dev)
    dist.all_reduce(unit_err, op=dist.ReduceOp.MAX)

    o_full = torch.zeros((b, n, h, d), dtype=torch.bfloat16, device=dev)
    l_full = torch.zeros((b, h, 1, n), dtype=torch.float32, device=dev)
    shapes = []
    for r in range(world):
        groups = {}
        for sl in partition_units(b, hkv, world, r):
            groups.setdefault(sl.kvh_hi - sl.kvh_lo, []).append(sl)
        shapes.append([(width, members) for width, members in sorted(groups.items())])
    same = all(len(sh) == 1 and len(sh[0][1]) == len(shapes[0][0][1]) and sh[0][0] == shapes[0][0][0] for sh in shapes)
    if same:
        og = torch.empty((world,) + tuple(outs[0][0].shape), dtype=torch.bfloat16, device=dev)
        lg = torch.empty((world,) + tuple(outs[0][1].shape), dtype=torch.float32, device=dev)
        dist.all_gather_into_tensor(og, outs[0][0].contiguous())
        dist.all_gather_into_tensor(lg, outs[0][1].contiguous())
        for r in range(world):
            scatter_outputs(o_full, l_full, og[r], lg[r], shapes[r][0][1], hkv)
        how = "all_gather_into_tensor"
    else:
        for r in range(world):
            for gi, (width, members) in enumerate(shapes[r]):
                if r == rank:
                    ob, lb = outs[gi][0].contiguous(), outs[gi][1].contiguous()
                else:
                    ob = torch.empty((len(members), n, width * g, d), dtype=torch.bfloat16, device=dev)
                    lb = torch.empty((len(members), width * g, 1, n), dtype=torch.float32, device=dev)
                dist.broadcast(ob, src=r)
                dist.broadcast(lb, src=r)
                scatter_outputs(o_full, l_full, ob, lb, members, hkv)
        how = "broadcast per rank (shards of unequal shape)"
    report = None
    if rank == 0:
        qf, kf, vf = make_prefill_inputs(b, n, h, hkv, d, seed=0)
        o1, l1 = hk.attn_fwd(qf.to(dev), kf.to(dev), vf.to(dev), causal=causal, stream=stream)
        torch.cuda.synchronize()
        report = {"max_abs_o": float((o_full.float() - o1.float()).abs().max()),
                  "max_abs_l": float((l_full - l1).abs().max()),
                  "unit_vs_fp32_max_abs_o": float(unit_err[0]), "unit_vs_fp32_max_abs_l": float(unit_err[1]),
                  "gather": how,
                  "what": "O and L shards of all ranks gathered over NCCL and compared on rank 0 with one single-GPU "
                          "launch on the whole workload (same seed); plus, on every rank, one (batch, kv-head) unit "
                          "against an fp32 restatement on the GPU (max over ranks)"}
    return report


# ------------------------------------------------------------------------------------------ main
def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--workload", default=DEFAULT_WORKLOAD, choices=sorted(WORKLOADS))
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--scaling", default=None, choices=["weak", "strong"],
                    help="default: strong (one workload split over the ranks) with more than one rank")
    ap.add_argument("--cpu-budget-s", type=float, default=12.0)
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--no-others", action="store_true", help="skip the other configurations and the sustained run")
    ap.add_argument("--sustained-s", type=float, default=2.0)
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3)

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    kind, b, n, h, hkv, d, causal = WORKLOADS[args.workload]
    if args.scaling is None:
        args.scaling = "strong" if (world > 1 and kind in ("fwd", "bwd")) else "weak"
    if kind == "decode":
        args.scaling = "weak"   # sequences are drawn per rank; the decode workload is not split
    peaks, peaks_src = load_peaks()

    if kind in ("rotary", "append"):
        return run_stream_workload(args, rank, world, local_rank, kind, b, n, h, hkv, d, peaks, peaks_src)
    if args.impl == "reference":
        return run_reference_arm(args, rank, world, kind, b, n, h, hkv, d, causal)

    import hipkittens_b200 as hk
    from hipkittens_b200 import _native
    from hipkittens_b200.shard import partition_units

    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the product has no CPU path")
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    dist = None
    if world > 1:
        import torch.distributed as dist

        dist.init_process_group("nccl", device_id=dev)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    stream = torch.cuda.current_stream(dev)
    sampler = ClockSampler(local_rank)

    # ---------------- inputs resident in HBM
    strong = args.scaling == "strong" and world > 1
    if kind in ("fwd", "bwd"):
        if strong:
            run = PrefillRun(hk, dev, stream, kind, b, n, h, hkv, d, causal, seed=0,
                             slices=partition_units(b, hkv, world, rank))
        else:
            run = PrefillRun(hk, dev, stream, kind, b, n, h, hkv, d, causal, seed=rank)
        my_units = float(run.flops)
        flops_per_launch = run.flops / max(len(run.sets[0][0]), 1)
    else:
        run = DecodeRun(hk, dev, stream, args.workload, b, h, hkv, d, seed=rank)
        my_units = run.tokens
    headline_cache = run.cache

    # ---------------- device-resident timing of the headline workload
    sampler.start()
    launches0 = hk.kernel_launch_count()
    ms_total = time_steps(run, args.steps, args.warmup, stream, barrier, sampler, tag="timed")
    launches = hk.kernel_launch_count() - launches0 - args.warmup * run.launches_per_step
    status = _native.device_status(local_rank)
    if status != 0:
        raise SystemExit(f"device status {status} after the timed region")

    # ---------------- end-to-end through the reference-facing module, host buffers
    e2e = None
    if not args.no_e2e:
        shards0, outs0, bwd0 = run.sets[0] if kind != "decode" else (None, None, None)
        e2e = measure_e2e(hk, kind, args, dev, stream, causal, b, n, h, hkv, d, shards0,
                          (run.q, run.kp, run.vp, run.bt, run.cl, run.ws) if kind == "decode" else None, barrier,
                          (outs0, bwd0) if kind == "bwd" else None)

    # ---------------- reduce over ranks: slowest rank's time, summed work
    ms = torch.tensor([ms_total, e2e["ms_total"] if e2e else 0.0], dtype=torch.float64, device=dev)
    units = torch.tensor([my_units], dtype=torch.float64, device=dev)
    if world > 1:
        dist.all_reduce(ms, op=dist.ReduceOp.MAX)
        dist.all_reduce(units, op=dist.ReduceOp.SUM)
    ms_total_max, e2e_ms_max = float(ms[0]), float(ms[1])
    total_units = float(units[0])
    ms_per_step = ms_total_max / args.steps

    # ---------------- N > 1: shard parity on the GPUs, and the replica (weak-scaling) figure beside the split one
    shard_parity = replicas = None
    if strong and kind == "fwd":
        shard_parity = shard_parity_report(hk, dist, run, dev, stream, rank, world, b, n, h, hkv, d, causal)
    if strong:
        del run
        torch.cuda.empty_cache()
        rep = PrefillRun(hk, dev, stream, kind, b, n, h, hkv, d, causal, seed=rank)
        rep_ms = torch.tensor([time_steps(rep, args.steps, args.warmup, stream, barrier)], dtype=torch.float64,
                              device=dev)
        dist.all_reduce(rep_ms, op=dist.ReduceOp.MAX)
        replicas = {"scaling": "weak", "ms_per_step": float(rep_ms[0]) / args.steps,
                    "value": rep.flops * world / (float(rep_ms[0]) / args.steps * 1e-3) / 1e12, "unit": "TFLOP/s",
                    "what": "every rank runs the whole workload on its own seeded inputs (independent replicas)"}
        run = rep

    # ---------------- N = 1: the other configurations and the sustained figure, after the headline numbers
    others = sustained = None
    if world == 1 and not args.no_others and args.workload == DEFAULT_WORKLOAD:
        sustained_run = run
        others = run_other_workloads(hk, _native, dev, stream, local_rank, sampler, barrier, peaks, peaks_src,
                                     args.steps, args.warmup)
        sustained = run_sustained(hk, sustained_run, stream, barrier, sampler, args.sustained_s,
                                  ms_total / args.steps, run.flops)
        if _native.device_status(local_rank) != 0:
            raise SystemExit("device status non-zero after the sustained run")
    sampler.stop()

    if rank == 0:
        clocks = sampler.summary("timed")
        line = {
            "n_gpus": world, "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms_per_step,
            "higher_is_better": True, "scaling": args.scaling, "vs_baseline": None, "data": "synthetic",
            "gpu_launches": int(launches), "clocks": clocks, "peaks_source": peaks_src,
            "metric": METRIC[kind], "dtype": "bf16", "config": workload_config(args.workload),
        }
        if kind in ("fwd", "bwd"):
            tflops = total_units / (ms_per_step * 1e-3) / 1e12
            ach = my_units / (ms_total / args.steps * 1e-3) / 1e12
            line.update({
                "value": tflops, "unit": "TFLOP/s",
                "partition": {"scaling": args.scaling,
                              "units_total": b * hkv * (world if not strong else 1),
                              "units_per_gpu": (b * hkv / world) if strong else b * hkv,
                              "per_gpu_batch": (b / world) if strong else b,
                              "cache": headline_cache,
                              "sharding": "independent (batch, kv-head) units dealt contiguously to ranks, no collective "
                                          "on the data path"},
                "roofline": prefill_roofline(args.workload, kind, ach, peaks, peaks_src, flops_per_launch),
            })
            if strong and line["roofline"]["traffic"] is not None:
                # the capture is of the whole workload on one GPU; a rank's launch moves its share of the units
                line["roofline"]["traffic"] = line["roofline"]["traffic"] / world
            if e2e:
                line["e2e"] = {"value": total_units / (e2e_ms_max / e2e["steps"] * 1e-3) / 1e12, "unit": "TFLOP/s",
                               "h2d_bytes_per_step": e2e["h2d"], "d2h_bytes_per_step": e2e["d2h"],
                               "steps": e2e["steps"], "path": e2e["path"]}
        else:
            tok_s = total_units / (ms_per_step * 1e-3)
            ach = run.kv_bytes / (ms_total / args.steps * 1e-3) / 1e9
            line.update({"value": tok_s, "unit": "tokens/s",
                         "roofline": decode_roofline(args.workload, ach, peaks, peaks_src, run.kv_bytes)})
            line["roofline"]["sum_ctx"] = run.sum_ctx
            if e2e:
                line["e2e"] = {"value": total_units / (e2e_ms_max / e2e["steps"] * 1e-3), "unit": "tokens/s",
                               "h2d_bytes_per_step": e2e["h2d"], "d2h_bytes_per_step": e2e["d2h"],
                               "steps": e2e["steps"], "path": e2e["path"]}
        if shard_parity is not None:
            line["shard_parity"] = shard_parity
        if replicas is not None:
            line["replicas"] = replicas
        if others is not None:
            line["other_workloads"] = others
        if sustained is not None:
            line["sustained"] = sustained
        if world == 1 and not args.no_cpu_baseline:
            line["cpu_baseline"] = cpu_baseline(kind, b, n, h, hkv, d, causal, args.cpu_budget_s)
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()
    return 0


def run_stream_workload(args, rank, world, local_rank, kind, b, n, h, hkv, d, peaks, peaks_src) -> int:
    """The HBM-bound byte movers next to the attention path: rotary pre-pass and paged KV-cache append. Single GPU
    (under torchrun every rank runs its own copy; rank 0 reports its own figure times the number of ranks)."""
    from oracle.attn_oracle import rotary_cos_sin

    cores = os.cpu_count() or 1
    if kind == "rotary":
        gen = torch.Generator().manual_seed(rank)
        x_h = torch.randn((b, h, n, d), generator=gen).to(torch.bfloat16)
        cos_h, sin_h = rotary_cos_sin(n, d)
        alg_bytes = 2 * x_h.numel() * 2
    else:
        gen = torch.Generator().manual_seed(rank)
        s_n, t_n = b, n
        k_h = torch.randn((s_n, t_n, hkv, d), generator=gen).to(torch.bfloat16)
        v_h = torch.randn((s_n, t_n, hkv, d), generator=gen).to(torch.bfloat16)
        pages_per_seq = t_n // 16
        pool = s_n * pages_per_seq
        bt_h = torch.randperm(pool, generator=gen).to(torch.int32).view(s_n, pages_per_seq)
        sp_h = torch.zeros(s_n, dtype=torch.int32)
        alg_bytes = 2 * 2 * k_h.numel() * 2
    if args.impl == "reference":
        if rank != 0:
            return 0
        torch.set_num_threads(cores)
        from oracle.attn_oracle import paged_kv_append_oracle, rotary_oracle
        t0 = time.perf_counter()
        reps = 0
        while time.perf_counter() - t0 < 10.0:
            if kind == "rotary":
                rotary_oracle(x_h[:2], cos_h, sin_h)
                frac = 2 / b
            else:
                kp = torch.zeros((16 * 8, 16, hkv, d), dtype=torch.bfloat16)
                paged_kv_append_oracle(k_h[:1, :128], v_h[:1, :128], kp, kp.clone(), torch.arange(8, dtype=torch.int32).view(1, 8),
                                       sp_h[:1])
                frac = 128 / (b * n)
            reps += 1
        dt = time.perf_counter() - t0
        value = alg_bytes * frac * reps / dt / 1e9
        line = {"impl": "reference", "metric": f"{kind} GB/s (bytes read + written)", "value": value, "unit": "GB/s",
                "n_gpus": world, "steps": args.steps, "warmup": args.warmup, "ms_per_step": dt / reps * 1e3,
                "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
                "config": {"workload": args.workload},
                "cpu_baseline": {"value": value, "unit": "GB/s", "cores": cores, "kind": "port",
                                 "sample": f"{reps} passes over {frac:.4f} of the workload in {dt:.1f} s, oracle"},
                "e2e": {"value": value, "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}, "gpu_launches": 0}
        print(json.dumps(line), flush=True)
        return 0

    import hipkittens_b200 as hk
    from hipkittens_b200 import _native

    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the product has no CPU path")
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    stream = torch.cuda.current_stream(dev)
    sampler = ClockSampler(local_rank)
    if kind == "rotary":
        x, cos, sin = x_h.to(dev), cos_h.to(dev), sin_h.to(dev)
        out = torch.empty_like(x)
        tk = hk.load_tk_kernel_rotary()

        def step():
            hk.rotary(x, cos, sin, out=out, stream=stream)

        host_in, dev_in = [x_h.pin_memory()], [x]
        host_out, dev_out = [torch.empty(x_h.shape, dtype=x_h.dtype).pin_memory()], [out]

        def api_step():
            tk.dispatch_rotary(x, out, sin, cos, stream=stream.cuda_stream)

        path = "pinned host x -> H2D -> tk_kernel.dispatch_rotary -> D2H o"
    else:
        k_new, v_new, bt, sp = k_h.to(dev), v_h.to(dev), bt_h.to(dev), sp_h.to(dev)
        kp = torch.zeros((pool, 16, hkv, d), dtype=torch.bfloat16, device=dev)
        vp = torch.zeros_like(kp)

        def step():
            hk.paged_kv_append(k_new, v_new, kp, vp, bt, sp, stream=stream)

        host_in, dev_in = [k_h.pin_memory(), v_h.pin_memory()], [k_new, v_new]
        host_out, dev_out = [], []
        api_step = step
        path = "pinned host k_new, v_new -> H2D -> hipkittens_b200.paged_kv_append (the cache stays on the device)"
    sampler.start()
    for _ in range(args.warmup):
        step()
    torch.cuda.synchronize()
    l0 = hk.kernel_launch_count()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    sampler.tag = "timed"
    e0.record(stream)
    for _ in range(args.steps):
        step()
    e1.record(stream)
    torch.cuda.synchronize()
    sampler.tag = None
    launches = hk.kernel_launch_count() - l0
    ms = e0.elapsed_time(e1) / args.steps
    if _native.device_status(local_rank) != 0:
        raise SystemExit("device status non-zero after the timed region")
    e2e = None
    if not args.no_e2e:
        def e2e_step():
            for src, dst in zip(host_in, dev_in):
                dst.copy_(src, non_blocking=True)
            api_step()
            for src, dst in zip(dev_out, host_out):
                dst.copy_(src, non_blocking=True)
        for _ in range(2):
            e2e_step()
        torch.cuda.synchronize()
        steps = max(1, min(args.steps, 10))
        e0.record(stream)
        for _ in range(steps):
            e2e_step()
        e1.record(stream)
        torch.cuda.synchronize()
        e2e = {"value": alg_bytes * world / (e0.elapsed_time(e1) / steps * 1e-3) / 1e9, "unit": "GB/s",
               "h2d_bytes_per_step": sum(t.numel() * t.element_size() for t in host_in),
               "d2h_bytes_per_step": sum(t.numel() * t.element_size() for t in host_out), "steps": steps, "path": path}
    sampler.stop()
    if rank == 0:
        ach = alg_bytes / (ms * 1e-3) / 1e9
        line = {"n_gpus": world, "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": True,
                "scaling": "weak", "vs_baseline": None, "data": "synthetic", "gpu_launches": int(launches),
                "clocks": sampler.summary(), "peaks_source": peaks_src,
                "metric": f"{kind} GB/s (bytes read + written)", "value": ach * world, "unit": "GB/s", "dtype": "bf16",
                "config": {"workload": args.workload, "B_or_S": b, "N_or_T": n, "H": h, "H_KV": hkv, "D": d,
                           "cache": "inputs_exceed_l2" if alg_bytes > 126e6 else "inputs_fit_l2"},
                "roofline": {"bound": "hbm", "achieved": ach, "peak": peaks["hbm_gbs"], "unit": "GB/s",
                             "frac": ach / peaks["hbm_gbs"], "peak_kind": f"of {peaks_src} (copy)",
                             "traffic": NCU_TRAFFIC_BYTES.get(args.workload), "bytes_per_launch": alg_bytes}}
        if e2e:
            line["e2e"] = e2e
        print(json.dumps(line), flush=True)
    return 0


def measure_e2e(hk, kind, args, dev, stream, causal, b, n, h, hkv, d, shards, dec, barrier, bwd=None):
    """Same step, but inputs start in pinned host memory and results end in pinned host memory, through
    the reference's Python entry (tk_kernel.dispatch_micro / dispatch_paged_decode)."""
    steps = max(1, min(args.steps, 10))
    tk = hk.load_tk_kernel(causal)
    if kind == "fwd":
        host_in = [[t.cpu().pin_memory() for t in sh] for sh in shards]
        dev_in = shards
        dev_out = [(torch.empty_like(sh[0]), torch.empty((sh[0].shape[0], sh[0].shape[2], 1, n), dtype=torch.float32,
                                                          device=dev)) for sh in shards]
        host_out = [(torch.empty(o.shape, dtype=o.dtype).pin_memory(), torch.empty(l.shape, dtype=l.dtype).pin_memory())
                    for o, l in dev_out]
        h2d = sum(t.numel() * t.element_size() for hs in host_in for t in hs)
        d2h = sum(t.numel() * t.element_size() for ho in host_out for t in ho)

        # The (batch, kv-head) units are independent, so a step is cut into batch chunks that flow through three
        # streams: chunk c+1 is copied in while chunk c is computed and chunk c-1 is copied out (PCIe is full duplex).
        s_in, s_cmp, s_out = torch.cuda.Stream(dev), torch.cuda.Stream(dev), torch.cuda.Stream(dev)

        def step():
            start = torch.cuda.Event()
            start.record(stream)
            for st in (s_in, s_cmp, s_out):
                st.wait_event(start)
            for hs, ds, do, ho in zip(host_in, dev_in, dev_out, host_out):
                nb = ds[0].shape[0]
                n_chunks = min(nb, 8)
                bounds = [nb * c // n_chunks for c in range(n_chunks + 1)]
                for lo, hi in zip(bounds[:-1], bounds[1:]):
                    with torch.cuda.stream(s_in):
                        for src, dst in zip(hs, ds):
                            dst[lo:hi].copy_(src[lo:hi], non_blocking=True)
                        ready = torch.cuda.Event()
                        ready.record(s_in)
                    s_cmp.wait_event(ready)
                    tk.dispatch_micro(ds[0][lo:hi], ds[1][lo:hi], ds[2][lo:hi], do[0][lo:hi], do[1][lo:hi], causal=causal,
                                      stream=s_cmp.cuda_stream)
                    done = torch.cuda.Event()
                    done.record(s_cmp)
                    s_out.wait_event(done)
                    with torch.cuda.stream(s_out):
                        ho[0][lo:hi].copy_(do[0][lo:hi], non_blocking=True)
                        ho[1][lo:hi].copy_(do[1][lo:hi], non_blocking=True)
            for st in (s_in, s_cmp, s_out):
                stream.wait_stream(st)

        path = ("pinned host -> H2D -> tk_kernel.dispatch_micro -> D2H (O and L), in up to 8 batch chunks pipelined over "
                "three streams")
    elif kind == "bwd":
        # one training-step backward (hipkittens.py:96-112): q, k, v, O, L (saved by the forward) and dO arrive from
        # pinned host memory, delta prep and the backward run, dQ, dK, dV go back to pinned host memory
        outs, bwd_in = bwd
        sets = []
        for (qs, ks, vs), (o, l), (d_o, delta, dq, dk, dv) in zip(shards, outs, bwd_in):
            dev_in = [qs, ks, vs, o, l, d_o]
            hin = [t.cpu().pin_memory() for t in dev_in]
            hout = [torch.empty(t.shape, dtype=t.dtype).pin_memory() for t in (dq, dk, dv)]
            sets.append((hin, dev_in, delta, (dq, dk, dv), hout))
        h2d = sum(t.numel() * t.element_size() for st in sets for t in st[0])
        d2h = sum(t.numel() * t.element_size() for st in sets for t in st[4])

        # batch chunks pipelined over three streams, as in the forward; the C ABI's asynchronous entries are used
        # (the reference's three dispatchers block on the device after every call, which would serialise the chunks)
        s_in, s_cmp, s_out = torch.cuda.Stream(dev), torch.cuda.Stream(dev), torch.cuda.Stream(dev)

        def step():
            start = torch.cuda.Event()
            start.record(stream)
            for st in (s_in, s_cmp, s_out):
                st.wait_event(start)
            for hin, dev_in, delta, (dq, dk, dv), hout in sets:
                qs, ks, vs, o, l, d_o = dev_in
                nb = qs.shape[0]
                n_chunks = min(nb, 8)
                bounds = [nb * c // n_chunks for c in range(n_chunks + 1)]
                for lo, hi in zip(bounds[:-1], bounds[1:]):
                    with torch.cuda.stream(s_in):
                        for src, dst in zip(hin, dev_in):
                            dst[lo:hi].copy_(src[lo:hi], non_blocking=True)
                        ready = torch.cuda.Event()
                        ready.record(s_in)
                    s_cmp.wait_event(ready)
                    hk.attn_bwd_prep(o[lo:hi], d_o[lo:hi], delta[lo:hi], stream=s_cmp)
                    hk.attn_bwd(qs[lo:hi], ks[lo:hi], vs[lo:hi], d_o[lo:hi], l[lo:hi], delta[lo:hi], causal=causal,
                                dq=dq[lo:hi], dk=dk[lo:hi], dv=dv[lo:hi], stream=s_cmp)
                    done = torch.cuda.Event()
                    done.record(s_cmp)
                    s_out.wait_event(done)
                    with torch.cuda.stream(s_out):
                        for src, dst in zip((dq, dk, dv), hout):
                            dst[lo:hi].copy_(src[lo:hi], non_blocking=True)
            for st in (s_in, s_cmp, s_out):
                stream.wait_stream(st)

        path = ("pinned host (q, k, v, O, L, dO) -> H2D -> hk_attn_bwd_prep, hk_attn_bwd (dQ written as [B,N,H,D]) -> D2H "
                "(dQ, dK, dV), in up to 8 batch chunks pipelined over three streams")
    else:
        q, kp, vp, bt, cl, ws = dec
        # decode step inputs: the new query token, block table and lengths; the KV pool is state that
        # lives on the device between steps, as in a serving loop
        host_in = [t.cpu().pin_memory() for t in (q, bt, cl)]
        dev_in = [q, bt, cl]
        o = torch.empty_like(q)
        l = torch.empty((b, h, 1, 1), dtype=torch.float32, device=dev)
        host_out = [torch.empty(o.shape, dtype=o.dtype).pin_memory(), torch.empty(l.shape, dtype=l.dtype).pin_memory()]
        h2d = sum(t.numel() * t.element_size() for t in host_in)
        d2h = sum(t.numel() * t.element_size() for t in host_out)

        def step():
            for src, dst in zip(host_in, dev_in):
                dst.copy_(src, non_blocking=True)
            tk.dispatch_paged_decode(q, kp, vp, bt, cl, o, l, ws, stream=stream.cuda_stream)
            host_out[0].copy_(o, non_blocking=True)
            host_out[1].copy_(l, non_blocking=True)

        path = "pinned host (q, block table, lengths) -> H2D -> tk_kernel.dispatch_paged_decode -> D2H (O and L)"
    for _ in range(2):
        step()
    barrier()
    e0 = torch.cuda.Event(enable_timing=True)
    e1 = torch.cuda.Event(enable_timing=True)
    e0.record(stream)
    for _ in range(steps):
        step()
    e1.record(stream)
    barrier()
    return {"ms_total": e0.elapsed_time(e1), "steps": steps, "h2d": h2d, "d2h": d2h, "path": path}


def cpu_baseline(kind, b, n, h, hkv, d, causal, budget_s):
    cores = os.cpu_count() or 1
    torch.set_num_threads(cores)
    if kind in ("fwd", "bwd"):
        sample_fn = cpu_prefill_sample if kind == "fwd" else cpu_bwd_sample
        flops, dt, units = sample_fn(b, n, h, hkv, d, causal, budget_s, max_units=b * hkv)
        return {"value": flops / dt / 1e12, "unit": "TFLOP/s", "cores": cores, "kind": "port",
                "sample": f"{units} of {b * hkv} (batch, kv-head) units of the workload shape, {dt:.1f} s, "
                          "oracle (fp32 PyTorch restatement of the reference math path"
                          + (")" if kind == "fwd" else " and of its derivative)")}
    toks, _ctx, dt, reps = cpu_decode_sample(budget_s)
    return {"value": toks / dt, "unit": "tokens/s", "cores": cores, "kind": "port",
            "sample": f"{reps} passes over 8 sequences with ctx ~ U{{512..8192}}, {dt:.1f} s, paged oracle"}


def run_reference_arm(args, rank, world, kind, b, n, h, hkv, d, causal) -> int:
    """The reference's CPU implementation of the path (the oracle port: the reference's HIP kernels cannot be
    built or run here) on the host cores. Rank 0 only."""
    if rank != 0:
        return 0
    cores = os.cpu_count() or 1
    torch.set_num_threads(cores)
    total_steps = args.warmup + args.steps
    per_step_budget = max(0.2, min(3.0, 150.0 / total_steps))
    times, work = [], []
    for i in range(total_steps):
        if kind in ("fwd", "bwd"):
            sample_fn = cpu_prefill_sample if kind == "fwd" else cpu_bwd_sample
            flops, dt, units = sample_fn(b, n, h, hkv, d, causal, per_step_budget, max_units=b * hkv)
            if i >= args.warmup:
                times.append(dt)
                work.append(flops)
        else:
            toks, _ctx, dt, _reps = cpu_decode_sample(per_step_budget)
            if i >= args.warmup:
                times.append(dt)
                work.append(toks)
    total_t, total_w = sum(times), sum(work)
    if kind in ("fwd", "bwd"):
        value, unit = total_w / total_t / 1e12, "TFLOP/s"
        metric = ("bf16 GQA attn-fwd TFLOPS (4*B*N^2*H*D, /2 causal)" if kind == "fwd" else
                  "bf16 GQA attn-bwd TFLOPS (2.5 * 4*B*N^2*H*D, /2 causal; delta prep + dK/dV + dQ kernels)")
        sample = (f"each step: as many (batch, kv-head) units of the workload shape as fit in {per_step_budget:.1f} s "
                  f"(of {b * hkv} per full pass)")
    else:
        value, unit = total_w / total_t, "tokens/s"
        metric = "paged-KV GQA decode tokens/s"
        sample = f"each step: passes over 8 sequences with ctx ~ U{{512..8192}} for {per_step_budget:.1f} s"
    line = {
        "impl": "reference", "metric": metric, "value": value, "unit": unit, "n_gpus": world, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": total_t / max(len(times), 1) * 1e3, "higher_is_better": True,
        "scaling": args.scaling, "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": workload_config(args.workload),
        "cpu_baseline": {"value": value, "unit": unit, "cores": cores, "kind": "port", "sample": sample},
        "e2e": {"value": value, "unit": unit, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)
    return 0


if __name__ == "__main__":
    sys.exit(main())
