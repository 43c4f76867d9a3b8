#!/usr/bin/env python
"""Benchmark of the fused-attention path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--workload NAME] [--impl reference]

One JSON line is printed (by rank 0).  A *step* is one pass of the hot path
over one batch of synthetic input:

  prefill_c2 (default)  fp16 non-causal prefill, B8 H32 Lq=Lk=2048 D128, scale
                        1/sqrt(128), N(0,1)*0.5 inputs, seed 1.  With N GPUs every
                        rank runs its own B8 H32 batch (the heads are independent
                        problems: batch x heads sharding, no collective) -> weak
                        scaling, value = aggregate TFLOP/s.
  prefill_c5            bf16 B16 H64 L8192 D128, batch x heads split over the ranks
                        (strong scaling).
  decode_c3             flash decoding B32 H32 Lk8192 D128, chunks of 512, seed 2;
                        value = GB/s of K+V bytes read.  With N GPUs: one batch per
                        rank (weak).
  decode_c4             long-context decode B4 H32 Lk131072 D128, KV sharded by
                        sequence over the ranks, one NCCL all-gather feeds the
                        combine (strong scaling).

`value` is measured with inputs resident in HBM, CUDA events on the launching
stream, max over ranks: W warm-up steps, then timed regions of exactly K steps
each, bracketed by a barrier and a device synchronisation on both sides.  The
region is repeated (a short idle gap in between, so that every region starts
from the same burst state a kernel timed alone sees) until about a quarter of
a second has been spent under load; `value` and `ms_per_step` are the median
region, `region_ms_per_step` lists them all, and `clocks` holds the NVML
samples that fell inside the regions.  `e2e` is the same metric through the
public Python operator with inputs copied from pinned host memory and the
result copied back inside the timed region.  `roofline` describes the dominant
kernel against the measured peaks in MEASURED_PEAKS.json; `cpu_baseline` times
the oracle (the reference's torch expression, fp32) on the host cores on a
bounded sample.

Besides the headline workload the default line carries, at every N:
  decode      decode_c3, one batch per rank
  decode_fp8  decode_c3 over an e4m3 K/V cache (written on the device by the
              library's conversion kernel); GB/s count the 8-bit bytes
  decode_c4   long-context decode with the KV length sharded over the N ranks
              (N = 1: the whole sequence on one GPU), both transports, with a
              parity object: every rank evaluates the fp32 expression on its own
              KV shard for two (batch, head) rows, the partial rows are gathered
              and merged by the oracle's combine, and the kernel's O / LSE are
              held against that
  prefill_c5  bf16 B16 H64 L8192, batch x heads split over the N ranks
  causal      prefill_c2 with the causal mask (FLOPs of unmasked pairs only)

`--impl reference` times that CPU expression alone, as the reference arm.
"""

from __future__ import annotations

import argparse
import json
import math
import os
import sys
import threading
import time
from pathlib import Path

import torch

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

WORKLOADS = {
    "prefill_c2": dict(kind="prefill", dtype="fp16", B=8, H=32, L=2048, D=128, seed=1, sigma=0.5,
                       scaling="weak"),
    "prefill_c5": dict(kind="prefill", dtype="bf16", B=16, H=64, L=8192, D=128, seed=4, sigma=0.5,
                       scaling="strong"),
    "decode_c3": dict(kind="decode", dtype="fp16", B=32, H=32, L=8192, D=128, seed=2, sigma=1.0,
                      scaling="weak"),
    "decode_c4": dict(kind="decode", dtype="fp16", B=4, H=32, L=131072, D=128, seed=3, sigma=1.0,
                      scaling="strong"),
}
# Grouped-query decoding (beyond the reference's configs): 32 query heads on 8 KV heads.
WORKLOADS["decode_gqa"] = dict(WORKLOADS["decode_c3"], B=64, Hkv=8)
# Smaller cases of the same kernels for `ncu --set full` captures: inputs still
# exceed the 126 MB L2, but only a few hundred MB are held on the device.
WORKLOADS["prefill_profile"] = dict(WORKLOADS["prefill_c2"], B=4)
WORKLOADS["decode_profile"] = dict(WORKLOADS["decode_c3"], B=4)
# the short-decode config over an 8-bit (e4m3) K/V cache: half the bytes per key
WORKLOADS["decode_c3_fp8"] = dict(WORKLOADS["decode_c3"], kv="e4m3")
WORKLOADS["decode_fp8_profile"] = dict(WORKLOADS["decode_c3_fp8"], B=8)
WORKLOADS["decode_gqa_profile"] = dict(WORKLOADS["decode_gqa"], B=16)
# A 1-GiB case of the sharded decode step (split, merge, exchange and combine in one launch) for captures.
WORKLOADS["decode_c4_profile"] = dict(WORKLOADS["decode_c4"], L=16384)
# One rank's share of decode_c4 when the KV length is sharded over 8 GPUs.
WORKLOADS["decode_c4_shard8"] = dict(WORKLOADS["decode_c4"], L=131072 // 8, scaling="weak")
# fused_two_gemms, D = (A B^T) C^T: the reference's own test case and one GEMM-sized case.
# the backward pass of the C2 shapes on its own line (and the smaller case an ncu capture takes)
WORKLOADS["backward_c2"] = dict(WORKLOADS["prefill_c2"], kind="backward")
WORKLOADS["backward_profile"] = dict(WORKLOADS["backward_c2"], B=4)
# not a benchmark of the path: SM clocks per tcgen05.mma for the operand forms the kernels use
WORKLOADS["mma_rate"] = dict(kind="mma_rate", dtype="fp16", scaling="weak")
WORKLOADS["two_gemms_ref"] = dict(kind="two_gemms", dtype="fp16", M=256, N=128, K=64, P=64, scaling="weak")
WORKLOADS["two_gemms"] = dict(kind="two_gemms", dtype="fp16", M=262144, N=8192, K=128, P=128, scaling="weak")
FALLBACK_PEAKS = dict(hbm_gbs=6650.0, bf16_tflops=1590.0)   # earlier measurement on this pool

# DRAM traffic (dram__bytes_read.sum + dram__bytes_write.sum) of the dominant kernel
# comes from the ncu captures summarised under profiles/: NCU_TRAFFIC.json (beside
# profiles/) holds, per kernel and captured case, the bytes of one launch, the (batch, head)
# problems that launch processed, and a hash of the kernel's source files at the
# time of the capture.  Traffic grows in proportion to the problems processed, so a
# launch is scaled by that; when the kernel source has changed since the capture the
# figure is withheld (null) rather than carried over.
KERNEL_SOURCES = {
    "attn_fwd_pair_kernel": ("attn_fwd_pair_sm100.cuh", "sm100_ptx.cuh"),
    "decode_split_kernel": ("decode_sm100.cuh", "sm100_ptx.cuh"),
}


def kernel_source_hash(kernel):
    import hashlib

    h = hashlib.sha256()
    for name in KERNEL_SOURCES[kernel]:
        h.update((ROOT / "tilefusion_b200" / "csrc" / name).read_bytes())
    return h.hexdigest()[:16]


def ncu_traffic(w, units_in_launch):
    """(bytes per launch or None, note).  `units_in_launch`: (batch, head) problems
    for one-head-per-KV-head workloads, (batch, KV head) groups for grouped-query."""
    table = ROOT / "NCU_TRAFFIC.json"
    if not table.exists():
        return None, "no capture recorded"
    kernel = "attn_fwd_pair_kernel" if (w["kind"] == "prefill" or "Hkv" in w) else "decode_split_kernel"
    case = f"{w['kind']}{'_gqa' if 'Hkv' in w else ''}{'_' + w['kv'] if 'kv' in w else ''}_L{w['L']}_D{w['D']}"
    entry = json.loads(table.read_text()).get(kernel, {}).get(case)
    if entry is None:
        return None, f"no capture of {kernel} for {case}"
    if entry["source_hash"] != kernel_source_hash(kernel):
        return None, f"{kernel} changed since its capture ({entry['capture']}); not carried over"
    per_unit = (entry["dram_bytes_read"] + entry["dram_bytes_write"]) / entry["units"]
    return per_unit * units_in_launch, f"{entry['capture']}, scaled by problems per launch"


def peaks():
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        d = json.loads(p.read_text())
        return dict(hbm_gbs=float(d["hbm_gbs"]), bf16_tflops=float(d["bf16_tflops"]),
                    bf16_tflops_sustained=float(d.get("bf16_tflops_sustained", 0.0)), source="measured")
    return dict(FALLBACK_PEAKS, bf16_tflops_sustained=0.0, source="fallback")


def torch_dtype(name):
    return {"fp16": torch.float16, "bf16": torch.bfloat16}[name]


def prefill_flops(b, h, lq, lk, d, causal=False):
    pairs = lq * lk if not causal else sum(min(lk, r + 1) for r in range(lq))
    return 4.0 * b * h * pairs * d


def decode_bytes(b, h, lk, d, elem_bytes=2):
    return 2.0 * b * h * lk * d * elem_bytes


# ------------------------------------------------------------------ clocks ---
class ClockSampler:
    """Samples SM clock and throttle reasons through NVML while work is queued."""

    REASONS = {
        0x8: "hw_slowdown", 0x40: "hw_thermal_slowdown", 0x20: "sw_thermal_slowdown",
        0x4: "sw_power_cap", 0x80: "hw_power_brake_slowdown",
    }

    def __init__(self, device_index: int):
        self.samples, self.reasons, self.max_mhz, self.timed = [], set(), None, []
        self._stop = threading.Event()
        self._thread = None
        try:
            import pynvml

            pynvml.nvmlInit()
            vis = os.environ.get("CUDA_VISIBLE_DEVICES")
            phys = int(vis.split(",")[device_index]) if vis and vis.split(",")[0].isdigit() else device_index
            self._nv = pynvml
            self._h = pynvml.nvmlDeviceGetHandleByIndex(phys)
            self.max_mhz = pynvml.nvmlDeviceGetMaxClockInfo(self._h, pynvml.NVML_CLOCK_SM)
        except Exception:
            self._nv = None

    def _sample(self):
        try:
            mhz = self._nv.nvmlDeviceGetClockInfo(self._h, self._nv.NVML_CLOCK_SM)
            mask = self._nv.nvmlDeviceGetCurrentClocksEventReasons(self._h)
            self.timed.append((time.perf_counter(), mhz, mask))
        except Exception:
            pass

    def _run(self):
        while not self._stop.is_set():
            self._sample()
            time.sleep(0.001)

    def keep_within(self, windows):
        """Keeps the samples taken inside the (start, end) host-time windows."""
        for t, mhz, mask in self.timed:
            if any(a <= t <= b for a, b in windows):
                self.samples.append(mhz)
                for bit, name in self.REASONS.items():
                    if mask & bit:
                        self.reasons.add(name)

    def __enter__(self):
        if self._nv is not None:
            self._thread = threading.Thread(target=self._run, daemon=True)
            self._thread.start()
        return self

    def __exit__(self, *exc):
        self._stop.set()
        if self._thread is not None:
            self._thread.join()

    def summary(self):
        if not self.samples:
            return {"sm_mhz": None, "sm_max_mhz": self.max_mhz, "reasons": sorted(self.reasons), "samples": 0}
        s = sorted(self.samples)
        return {"sm_mhz": s[len(s) // 2], "sm_max_mhz": self.max_mhz, "reasons": sorted(self.reasons),
                "samples": len(s), "sm_mhz_min": s[0], "sm_mhz_all": self.samples,
                "sampled": "NVML, 1 ms period, samples inside the timed regions only"}


# ------------------------------------------------------------------- inputs --
def make_inputs(w, device, b=None, l=None):
    """Seeded synthetic Q, K, V on `device` (fp32 draw -> 16-bit), order Q, K, V."""
    dt = torch_dtype(w["dtype"])
    b = w["B"] if b is None else b
    l = w["L"] if l is None else l
    g = torch.Generator(device=device).manual_seed(w["seed"])
    lq = l if w["kind"] == "prefill" else 1
    q = (torch.randn(b, w["H"], lq, w["D"], generator=g, device=device) * w["sigma"]).to(dt)
    hkv = w.get("Hkv", w["H"])
    k = torch.empty(b, hkv, l, w["D"], dtype=dt, device=device)
    v = torch.empty_like(k)
    for t in (k, v):            # per-batch draws keep the fp32 staging buffer small
        for i in range(b):
            t[i] = (torch.randn(hkv, l, w["D"], generator=g, device=device) * w["sigma"]).to(dt)
    return q, k, v


# -------------------------------------------------------------- CPU oracle ---
_CPU_INPUTS = {}


def cpu_inputs(w, n_heads):
    """Seeded CPU inputs for `n_heads` (batch, head) problems (generated once, reused)."""
    key = (w["kind"], w["L"], w["D"], w["dtype"], w["seed"], n_heads)
    if key not in _CPU_INPUTS:
        dt = torch_dtype(w["dtype"])
        g = torch.Generator().manual_seed(w["seed"])
        lq = w["L"] if w["kind"] == "prefill" else 1
        _CPU_INPUTS.clear()
        _CPU_INPUTS[key] = tuple(
            (torch.randn(n_heads, rows, w["D"], generator=g) * w["sigma"]).to(dt) for rows in (lq, w["L"], w["L"]))
    return _CPU_INPUTS[key]


def cpu_heads_cap(w):
    """Largest sample (in (batch, head) problems) whose K and V stay below 256 MiB each."""
    return max(1, (256 << 20) // (w["L"] * w["D"] * 2))


def cpu_attention_sample(w, n_heads, threads):
    """Times the fp32 torch expression on `n_heads` (b,h) problems of workload w."""
    from oracle import attention_oracle as orc

    torch.set_num_threads(threads)
    q, k, v = cpu_inputs(w, n_heads)
    scale = 1.0 / math.sqrt(w["D"])
    t0 = time.perf_counter()
    for i in range(n_heads):
        orc.attention_fp32(q[i], k[i], v[i], scale, False)
    return time.perf_counter() - t0


def unit_per_head(w):
    if w["kind"] == "prefill":
        return prefill_flops(1, 1, w["L"], w["L"], w["D"]) / 1e12      # TFLOP
    # GB of K+V per query head; query heads of a group share one KV head
    return decode_bytes(1, 1, w["L"], w["D"]) * w.get("Hkv", w["H"]) / w["H"] / 1e9


def cpu_baseline(w, budget_s=12.0):
    threads = os.cpu_count() or 1
    t1 = cpu_attention_sample(w, 1, threads)        # also warms the thread pool
    t1 = cpu_attention_sample(w, 1, threads)
    total = w["B"] * w["H"]
    n = int(max(1, min(total, cpu_heads_cap(w), budget_s / max(t1, 1e-6))))
    passes, t = 0, 0.0
    while t < budget_s and passes < 4096:      # whole passes until about budget_s of CPU work
        t += cpu_attention_sample(w, n, threads)
        passes += 1
    unit = "TFLOP/s" if w["kind"] == "prefill" else "GB/s"
    return {"value": unit_per_head(w) * n * passes / t, "unit": unit, "cores": threads, "kind": "port",
            "sample": f"{passes} pass(es) over {n} of {total} (batch, head) problems of the workload, "
                      f"oracle fp32 torch expression, {t:.1f} s"}


def run_reference_arm(args, w, name):
    """The reference's CPU expression for this path, timed alone (rank 0 only)."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    threads = os.cpu_count() or 1
    t1 = cpu_attention_sample(w, 1, threads)
    t1 = cpu_attention_sample(w, 1, threads)
    total = w["B"] * w["H"]
    steps, warm = args.steps, max(args.warmup, 1)
    n = int(max(1, min(total, cpu_heads_cap(w), 120.0 / max(t1 * (steps + warm), 1e-6))))
    for _ in range(warm):
        cpu_attention_sample(w, n, threads)
    t0 = time.perf_counter()
    for _ in range(steps):
        cpu_attention_sample(w, n, threads)
    dt = time.perf_counter() - t0
    unit = "TFLOP/s" if w["kind"] == "prefill" else "GB/s"
    value = unit_per_head(w) * n * steps / dt
    sample = f"each step = {n} of {total} (batch, head) problems, oracle fp32 torch expression"
    line = {
        "impl": "reference", "metric": metric_name(w), "value": value, "unit": unit, "n_gpus": args.gpus,
        "steps": steps, "warmup": warm, "ms_per_step": dt / steps * 1e3, "higher_is_better": True,
        "scaling": w["scaling"], "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": workload_config(w, name, args.gpus),
        "cpu_baseline": {"value": value, "unit": unit, "cores": threads, "kind": "port", "sample": sample},
        "e2e": {"value": value, "unit": unit, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    print(json.dumps(line), flush=True)


def metric_name(w):
    return {"prefill": "prefill_tflops", "decode": "decode_hbm_gbs", "two_gemms": "fused_two_gemms_tflops",
            "backward": "backward_tflops"}[w["kind"]]


def workload_config(w, name, n_gpus, causal=False):
    if w["kind"] == "two_gemms":
        return {"workload": name, "m": w["M"], "n": w["N"], "k": w["K"], "p": w["P"],
                "l2": ("A and D larger than L2 (64 MB each); no flush between steps" if w["M"] * w["K"] * 2 >= 64 << 20
                       else "plumbing case: everything is L2-resident, launch-latency bound"),
                "timing": "median of repeated regions of exactly `steps` steps, idle gap between regions"}
    return {"workload": name + ("+causal" if causal else ""), "batch_per_step": w["B"] * (n_gpus if w["scaling"] == "weak" else 1),
            "heads": w["H"], "len_q": w["L"] if w["kind"] in ("prefill", "backward") else 1, "len_kv": w["L"],
            "head_dim": w["D"], "causal": bool(causal), "softmax_scale": "1/sqrt(D)",
            "sharding": ("batch x heads, no collective" if w["kind"] in ("prefill", "backward") or w["scaling"] == "weak"
                         else "KV length; (O, m, l) rows exchanged by peer stores inside the decode kernel, "
                              "or by one NCCL all-gather"),
            "l2": "inputs larger than L2 (126 MB); no flush between steps",
            "timing": "median of repeated regions of exactly `steps` steps, idle gap between regions"}


# ------------------------------------------------------------- GPU timing ----
TARGET_LOADED_S = 0.25     # time under load over which clock samples are collected
MAX_REPEATS = 25
IDLE_GAP_S = 0.02


def time_steps(fn, steps, warmup, device, world, max_repeats=None):
    """W warm-up steps, then regions of exactly `steps` steps, each bracketed by
    barrier + synchronize on both sides and timed with CUDA events on the current
    stream, max over ranks.  Returns (median seconds per region, info)."""
    import torch.distributed as dist

    def fence():
        torch.cuda.synchronize(device)
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize(device)

    max_repeats = MAX_REPEATS if max_repeats is None else max_repeats
    for _ in range(warmup):
        fn()
    sampler = ClockSampler(device.index if device.index is not None else 0)
    regions, windows = [], []
    with sampler:
        repeats = 1
        r = 0
        while r < repeats:
            fence()
            start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            t0 = time.perf_counter()
            start.record()
            for _ in range(steps):
                fn()
            end.record()
            end.synchronize()
            t1 = time.perf_counter()
            fence()
            secs = start.elapsed_time(end) / 1e3
            if world > 1:
                t = torch.tensor([secs], dtype=torch.float64, device=device)
                dist.all_reduce(t, op=dist.ReduceOp.MAX)
                secs = t.item()
            regions.append(secs)
            windows.append((t0, t1))
            if r == 0:      # every rank derives the same count from the max-over-ranks time
                repeats = int(max(1, min(max_repeats, math.ceil(TARGET_LOADED_S / max(secs, 1e-6)))))
            r += 1
            if r < repeats:
                time.sleep(IDLE_GAP_S)
    sampler.keep_within(windows)
    ordered = sorted(regions)
    median = ordered[len(ordered) // 2]
    info = {"clocks": sampler.summary(), "repeats": len(regions),
            "region_ms_per_step": [round(x / steps * 1e3, 5) for x in regions]}
    return median, info


def attn_desc_for(q, k, v, o, dtype_name, scale, causal):
    from tilefusion_b200 import _cabi

    d = _cabi.TfAttnDesc()
    d.dtype = _cabi.TF_F16 if dtype_name == "fp16" else _cabi.TF_BF16
    d.batch, d.heads, d.len_q, d.head_dim = q.shape
    d.len_kv, d.head_dim_v = k.size(2), v.size(3)
    d.softmax_scale = scale
    d.causal = int(causal)
    d.q_stride_b, d.q_stride_h, d.q_stride_l = q.stride(0), q.stride(1), q.stride(2)
    d.k_stride_b, d.k_stride_h, d.k_stride_l, d.k_stride_d = k.stride()
    d.v_stride_b, d.v_stride_h, d.v_stride_l, d.v_stride_d = v.stride()
    d.o_stride_b, d.o_stride_h, d.o_stride_l = o.stride(0), o.stride(1), o.stride(2)
    return d


def gpu_attention_fp32(q, k, v, scale, causal):
    """softmax(q k^T * scale [+ mask]) v and LSE in fp32 with torch on the device,
    for one (batch, head): q [Lq, D], k/v [Lk, D].  Used for parity only."""
    s = (q.float() @ k.float().t()) * scale
    if causal:
        lq, lk = s.shape
        s = s.masked_fill(torch.arange(lk, device=s.device)[None, :] > torch.arange(lq, device=s.device)[:, None],
                          float("-inf"))
    lse = torch.logsumexp(s, dim=-1)
    return torch.exp(s - lse[:, None]) @ v.float(), lse


def prefill_roofline(w, local_flops, per_launch_s, units, loaded_s, reasons, causal=False):
    pk = peaks()
    # A kernel timed alone in a short region is held against the burst cuBLAS figure;
    # when the timed region is long enough to run into the power cap (seconds-long
    # loops, sw_power_cap active) the sustained figure is the like-for-like peak.
    sustained = ("sw_power_cap" in reasons or loaded_s > 0.5) and pk.get("bf16_tflops_sustained", 0) > 0
    peak_tf = pk["bf16_tflops_sustained"] if sustained else pk["bf16_tflops"]
    ach = local_flops / per_launch_s / 1e12
    traffic, note = (None, "not captured with the causal mask") if causal else ncu_traffic(w, units)
    return {"bound": "tensor", "achieved": ach, "peak": peak_tf, "unit": "TFLOP/s", "frac": ach / peak_tf,
            "traffic": traffic, "traffic_source": note, "kernel": "attn_fwd_pair_kernel",
            "algorithmic_bytes": 4.0 * units * w["L"] * w["D"] * 2,
            "peak_source": pk["source"] + (" (sustained cuBLAS bf16, power-capped loop)" if sustained
                                           else " (burst cuBLAS bf16)"),
            "frac_of_burst": ach / pk["bf16_tflops"],
            "frac_of_sustained": (ach / pk["bf16_tflops_sustained"]) if pk.get("bf16_tflops_sustained") else None,
            "frac_of_nominal_2250": ach / 2250.0}


def run_prefill(args, w, name, device, rank, world, causal=False, steps=None, warmup=None, with_e2e=True):
    import ctypes as C

    from tilefusion_b200 import _cabi
    import tilefusion_b200 as tilefusion

    steps = args.steps if steps is None else steps
    warmup = args.warmup if warmup is None else warmup
    lib = _cabi.lib()
    scale = 1.0 / math.sqrt(w["D"])
    stream = torch.cuda.current_stream(device).cuda_stream
    if w["scaling"] == "weak":
        # every rank runs its own batch of the same shape
        b_local, h_local = w["B"], w["H"]
        total_units = prefill_flops(w["B"] * world, w["H"], w["L"], w["L"], w["D"], causal)
        q, k, v = make_inputs(dict(w, seed=w["seed"] + 1000 * rank), device)
        o = torch.empty_like(q)
        d = attn_desc_for(q, k, v, o, w["dtype"], scale, causal)
        qp, kp, vp, op = q.data_ptr(), k.data_ptr(), v.data_ptr(), o.data_ptr()

        def step():
            rc = lib.tf_attn_fwd(qp, kp, vp, op, None, C.byref(d), stream)
            if rc != 0:
                _cabi.check(rc)
        local_heads = b_local * h_local
    else:
        # strong scaling: the flattened (batch x heads) axis is split by tf_prefill_sharded; a
        # rank holds only its slice, laid out where the full [B, H, L, D] tensor would have it
        from tilefusion_b200.shard import head_slice

        h0, h1 = head_slice(w["B"] * w["H"], rank, world)
        local_heads = h1 - h0
        total_units = prefill_flops(w["B"], w["H"], w["L"], w["L"], w["D"], causal)
        q, k, v = make_inputs(dict(w, H=1, seed=w["seed"] + 1000 * rank), device, b=local_heads)
        o = torch.empty_like(q)
        full = torch.empty(0, dtype=q.dtype, device="meta").new_empty((w["B"], w["H"], w["L"], w["D"]))
        d = attn_desc_for(full, full, full, full, w["dtype"], scale, causal)
        head_bytes = w["L"] * w["D"] * q.element_size()
        bases = [t.data_ptr() - h0 * head_bytes for t in (q, k, v, o)]

        def step():
            rc = lib.tf_prefill_sharded(rank, world, bases[0], bases[1], bases[2], bases[3], None, C.byref(d),
                                        stream, None, None)
            if rc != 0:
                _cabi.check(rc)

    secs, info = time_steps(step, steps, warmup, device, world)
    value = total_units * steps / secs / 1e12
    per_launch_s = secs / steps
    local_flops = prefill_flops(1, local_heads, w["L"], w["L"], w["D"], causal)
    roof = prefill_roofline(w, local_flops, per_launch_s, local_heads, secs * info["repeats"],
                            info["clocks"]["reasons"], causal)
    res = dict(value=value, unit="TFLOP/s", secs=secs, info=info, roofline=roof, launches=steps)
    if args.profile:
        return res

    # parity of the timed output: one (batch, head) against the fp32 expression evaluated on the
    # device, and (where a head is small enough for the host) against the oracle on the CPU
    from oracle import attention_oracle as orc

    ref, _ = gpu_attention_fp32(q[0, 0], k[0, 0], v[0, 0], scale, causal)
    dt = torch_dtype(w["dtype"])
    parity = {"max_abs": (o[0, 0].float() - ref).abs().max().item(), "rel_l2": orc.rel_l2(o[0, 0].cpu(), ref.cpu()),
              "rel_l2_bound": orc.rel_l2_bound(ref.cpu(), dt), "rel_l2_rounding_floor": orc.rounding_floor(ref.cpu(), dt),
              "checked": "one (batch, head) of the timed output vs softmax(QK^T s)V in fp32 (torch, on the device)"}
    if w["L"] <= 4096:
        ref_cpu, _ = orc.attention_fp32(q[0, 0].cpu(), k[0, 0].cpu(), v[0, 0].cpu(), scale, causal)
        parity["oracle_max_abs"] = orc.max_abs(o[0, 0].cpu(), ref_cpu)
        parity["oracle_rel_l2"] = orc.rel_l2(o[0, 0].cpu(), ref_cpu)
        parity["checked"] += " and vs the CPU oracle"
    res["parity"] = parity
    if not with_e2e:
        return res

    # end to end through the public operator, host buffers in and out
    e2e_steps = max(1, min(steps, 20))
    hq, hk, hv = (t.cpu().pin_memory() for t in (q, k, v))
    ho = torch.empty(o.shape, dtype=o.dtype).pin_memory()
    pipe = tilefusion.HostPipeline(
        lambda dq, dk, dv: tilefusion.ops.flash_attention(dq, dk.transpose(-1, -2), dv, 0, 0, 0, 0, scale, causal),
        device)

    def e2e_steps_timed(n):
        # pinned host Q, K, V in, O back into pinned host memory; copies of neighbouring
        # steps overlap with the kernel (tilefusion_b200.HostPipeline)
        torch.cuda.synchronize(device)
        t0 = time.perf_counter()
        for _ in range(n):
            pipe.submit((hq, hk, hv), ho)
        pipe.flush()
        return time.perf_counter() - t0

    e2e_steps_timed(3)
    e2e_secs = e2e_steps_timed(e2e_steps)
    if world > 1:
        import torch.distributed as dist

        t = torch.tensor([e2e_secs], dtype=torch.float64, device=device)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        e2e_secs = t.item()
    res["e2e"] = {"value": total_units * e2e_steps / e2e_secs / 1e12, "unit": "TFLOP/s",
                  "h2d_bytes_per_step": 3 * q.numel() * q.element_size(),
                  "d2h_bytes_per_step": o.numel() * o.element_size(), "steps": e2e_steps,
                  "timing": "host wall clock around submit..flush (three streams), max over ranks"}
    return res


def run_backward(args, w, device, rank, world, steps, warmup):
    """Backward of the prefill workload `w` (dQ, dK, dV through tf_attn_bwd: three launches per
    step); FLOPs counted as 2.5 x the forward (five tile products against two)."""
    import ctypes as C

    from tilefusion_b200 import _cabi

    lib = _cabi.lib()
    scale = 1.0 / math.sqrt(w["D"])
    stream = torch.cuda.current_stream(device).cuda_stream
    q, k, v = make_inputs(dict(w, kind="prefill", seed=w["seed"] + 1000 * rank), device)
    g = torch.Generator(device=device).manual_seed(w["seed"] + 77 + 1000 * rank)
    d_o = (torch.randn(q.shape, generator=g, device=device) * w["sigma"]).to(q.dtype)
    o = torch.empty_like(q)
    lse = torch.empty(w["B"], w["H"], w["L"], dtype=torch.float32, device=device)
    d = attn_desc_for(q, k, v, o, w["dtype"], scale, False)
    _cabi.check(lib.tf_attn_fwd(q.data_ptr(), k.data_ptr(), v.data_ptr(), o.data_ptr(), lse.data_ptr(), C.byref(d), stream))
    dq, dk, dv = torch.empty_like(q), torch.empty_like(k), torch.empty_like(v)
    ws = torch.empty(lib.tf_attn_bwd_workspace_bytes(C.byref(d)) // 4, dtype=torch.float32, device=device)
    ptrs = [t.data_ptr() for t in (q, k, v, o, d_o, lse, dq, dk, dv, ws)]

    def step():
        rc = lib.tf_attn_bwd(*ptrs[:9], C.byref(d), ptrs[9], ws.numel() * 4, stream)
        if rc != 0:
            _cabi.check(rc)

    secs, info = time_steps(step, steps, warmup, device, world)
    flops = 2.5 * prefill_flops(w["B"] * world, w["H"], w["L"], w["L"], w["D"])
    pk = peaks()
    ach = flops / world * steps / secs / 1e12
    res = dict(value=flops * steps / secs / 1e12, unit="TFLOP/s", secs=secs, info=info, launches=3 * steps,
               roofline={"bound": "tensor", "achieved": ach, "peak": pk["bf16_tflops"], "unit": "TFLOP/s",
                         "frac": ach / pk["bf16_tflops"], "traffic": None, "traffic_source": "not captured",
                         "kernel": "attn_bwd_kernel (dK/dV and dQ) + attn_bwd_delta_kernel",
                         "flops_counted": "10*B*H*Lq*Lk*D (2.5 x forward); the kernels execute 14 (S and dP are "
                                          "recomputed by the dQ kernel)",
                         "peak_source": pk["source"] + " (burst cuBLAS bf16)"})
    if args.profile:
        return res
    # parity of one head: gradient of the fp32 expression by torch.autograd on the device
    qh, kh, vh = (t[0, 0].float().detach().requires_grad_(True) for t in (q, k, v))
    ref, _ = gpu_attention_fp32(qh, kh, vh, scale, False)
    ref.backward(d_o[0, 0].float())
    from oracle import attention_oracle as orc

    res["parity"] = {name: orc.rel_l2(got[0, 0].cpu(), want.grad.cpu())
                     for name, got, want in (("dq_rel_l2", dq, qh), ("dk_rel_l2", dk, kh), ("dv_rel_l2", dv, vh))}
    res["parity"]["checked"] = "one (batch, head): gradients of softmax(QK^T s)V in fp32 by torch.autograd on the device"
    return res


def sharded_parity(q, k_local, v_local, o, lse, scale, device, world):
    """Parity of a KV-sharded decode step without ever holding the whole sequence in
    one place: every rank evaluates the fp32 expression on its own shard for two
    (batch, head) rows with torch on the device, giving one (O, m, l) partial row
    each; the rows of all ranks are gathered (NCCL) and merged by the oracle's
    combine on the host; the kernel's O / LSE of those rows are compared with it."""
    import torch.distributed as dist

    from oracle import attention_oracle as orc

    b_n, h_n = q.size(0), q.size(1)
    picks = [(0, 0), (b_n - 1, h_n - 1)]
    dim = q.size(3)
    rows = torch.zeros(len(picks), dim + 2, dtype=torch.float32, device=device)
    for i, (b, h) in enumerate(picks):
        hk = h * k_local.size(1) // h_n
        if k_local.size(2) == 0:
            rows[i, dim] = float("-inf")
            continue
        sc = (k_local[b, hk].float() @ q[b, h, 0].float()) * (scale * orc.LOG2E)
        m = sc.max()
        p = torch.exp2(sc - m)
        rows[i, :dim] = p @ v_local[b, hk].float()
        rows[i, dim], rows[i, dim + 1] = m, p.sum()
    if world > 1:
        gathered = torch.empty(world, len(picks), dim + 2, dtype=torch.float32, device=device)
        dist.all_gather_into_tensor(gathered, rows)
    else:
        gathered = rows[None]
    g = gathered.cpu().permute(1, 0, 2)                       # [rows, ranks, D + 2]
    ref_o, ref_lse, _ = orc.decode_combine(g[..., :dim], g[..., dim:])
    got_o = torch.stack([o[b, h, 0] for b, h in picks]).float().cpu()
    got_lse = torch.stack([lse[b, h, 0] for b, h in picks]).cpu()
    return {"max_abs": (got_o - ref_o).abs().max().item(), "rel_l2": orc.rel_l2(got_o, ref_o),
            "lse_abs": (got_lse - ref_lse).abs().max().item(),
            "checked": "two (batch, head) rows: per-rank fp32 partials on each rank's own KV shard (torch, on the "
                       "device), gathered and merged by the oracle's combine, vs the kernel's O / LSE on rank 0"}


def decode_roofline(w, local_units, secs, steps, units_in_launch, sharded):
    pk = peaks()
    ach = local_units * steps / secs / 1e9
    traffic, note = (None, "not captured for the sharded step") if sharded else ncu_traffic(w, units_in_launch)
    return {"bound": "hbm", "achieved": ach, "peak": pk["hbm_gbs"], "unit": "GB/s", "frac": ach / pk["hbm_gbs"],
            "traffic": traffic, "traffic_source": note, "algorithmic_bytes": local_units,
            "kernel": ("attn_fwd_pair_kernel in split-KV mode (+ combine)" if "Hkv" in w
                       else "decode_split_kernel" + (" (split, merge, exchange and combine in one launch)" if sharded
                                                     else " (+ combine)")),
            "peak_source": pk["source"] + " (torch copy, read+write)", "frac_of_nominal_8000": ach / 8000.0}


def run_decode_sharded(args, w, name, device, rank, world, steps, warmup):
    """decode_c4: the KV length split over the ranks (world 1: one GPU holds it all),
    through tf_decode_sharded, once per transport."""
    from tilefusion_b200.shard import ShardedDecoder, kv_slice

    scale = 1.0 / math.sqrt(w["D"])
    k0, k1 = kv_slice(w["L"], rank, world)
    q = make_inputs(dict(w, L=128), device)[0]                 # replicated Q (same seed on every rank)
    _, k, v = make_inputs(dict(w, seed=w["seed"] + 1000 * rank), device, l=k1 - k0)
    out = torch.empty(w["B"], w["H"], 1, w["D"], dtype=q.dtype, device=device)
    lse = torch.empty(w["B"], w["H"], 1, dtype=torch.float32, device=device)
    total_units = decode_bytes(w["B"], w["H"], w["L"], w["D"])
    local_units = decode_bytes(w["B"], w["H"], k1 - k0, w["D"])
    wanted = [args.transport] if getattr(args, "transport", None) else ["p2p", "nccl"]
    results = {}
    for transport in wanted:
        dec = ShardedDecoder(w["B"], w["H"], w["D"], q.dtype, device, transport=transport)

        def step():
            dec(q, k, v, scale, out=out, lse=lse)

        secs, info = time_steps(step, steps, warmup, device, world)
        r = dict(value=total_units * steps / secs / 1e9, unit="GB/s", secs=secs, info=info,
                 roofline=decode_roofline(w, local_units, secs, steps, w["B"] * w["H"], True),
                 transport=dec.transport, transport_note=dec.transport_note,
                 launches=(1 if dec.transport == "p2p" else 3) * steps)
        if not args.profile:
            r["parity"] = sharded_parity(q, k, v, out, lse, scale, device, world)
        torch.cuda.synchronize(device)
        if world > 1:
            import torch.distributed as dist

            dist.barrier()          # no rank frees its gather buffer while a peer may still store into it
        dec.close()
        results[transport] = r
    return results


def run_decode(args, w, name, device, rank, world, steps=None, warmup=None):
    import ctypes as C

    from tilefusion_b200 import _cabi

    steps = args.steps if steps is None else steps
    warmup = args.warmup if warmup is None else warmup
    if w["scaling"] == "strong":
        results = run_decode_sharded(args, w, name, device, rank, world, steps, warmup)
        first = next(iter(results.values()))
        res = dict(first)
        res["by_transport"] = results
        return res
    lib = _cabi.lib()
    scale = 1.0 / math.sqrt(w["D"])
    stream = torch.cuda.current_stream(device).cuda_stream
    q, k, v = make_inputs(dict(w, seed=w["seed"] + 1000 * rank), device)
    o = torch.empty_like(q)
    lse = torch.empty(w["B"], w["H"], 1, dtype=torch.float32, device=device)
    d = _cabi.TfDecodeDesc()
    kv_bytes = 2
    if "kv" in w:
        # 8-bit cache: the 16-bit draws are quantised on the device (factor 1: the values fit the format)
        import tilefusion_b200 as tilefusion

        fp8_dtype = {"e4m3": torch.float8_e4m3fn, "e5m2": torch.float8_e5m2}[w["kv"]]
        k = tilefusion.ops.fp8_quantize(k, fp8_dtype)
        v = tilefusion.ops.fp8_quantize(v, fp8_dtype)
        d.kv_dtype = {"e4m3": _cabi.TF_FP8_E4M3, "e5m2": _cabi.TF_FP8_E5M2}[w["kv"]]
        kv_bytes = 1
        torch.cuda.empty_cache()
    d.dtype = _cabi.TF_F16 if w["dtype"] == "fp16" else _cabi.TF_BF16
    d.batch, d.heads, d.len_kv, d.head_dim = w["B"], w["H"], w["L"], w["D"]
    kv_chunk = 512 if "kv" not in w else 0       # 0: the registry's choice (1024 keys for an 8-bit cache)
    d.kv_chunk, d.num_splits, d.softmax_scale = kv_chunk, 0, scale
    d.q_stride_b, d.q_stride_h = q.stride(0), q.stride(1)
    d.k_stride_b, d.k_stride_h = k.stride(0), k.stride(1)
    d.v_stride_b, d.v_stride_h = v.stride(0), v.stride(1)
    d.o_stride_b, d.o_stride_h = o.stride(0), o.stride(1)
    hkv = w.get("Hkv", w["H"])
    d.heads_kv = hkv
    plan = _cabi.TfDecodePlan()
    _cabi.check(lib.tf_decode_plan(C.byref(d), C.byref(plan)))
    ws = torch.empty(plan.workspace_bytes // 4, dtype=torch.float32, device=device)
    ptrs = (q.data_ptr(), k.data_ptr(), v.data_ptr(), o.data_ptr(), lse.data_ptr(), ws.data_ptr())

    def step():
        rc = lib.tf_decode(ptrs[0], ptrs[1], ptrs[2], ptrs[3], ptrs[4], ptrs[5], ws.numel() * 4,
                           C.byref(d), stream)
        if rc != 0:
            _cabi.check(rc)

    total_units = decode_bytes(w["B"] * world, hkv, w["L"], w["D"], kv_bytes)
    local_units = decode_bytes(w["B"], hkv, w["L"], w["D"], kv_bytes)
    secs, info = time_steps(step, steps, warmup, device, world)
    res = dict(value=total_units * steps / secs / 1e9, unit="GB/s", secs=secs, info=info,
               roofline=decode_roofline(w, local_units, secs, steps, w["B"] * hkv, False), launches=2 * steps)
    if args.profile:
        return res
    from oracle import attention_oracle as orc

    grp = w["H"] // hkv
    ref, lse_ref = orc.decode_fp32(q[:1, :2].cpu(), k[:1, :1].cpu().expand(-1, 2, -1, -1) if grp > 1 else k[:1, :2].cpu(),
                                   v[:1, :1].cpu().expand(-1, 2, -1, -1) if grp > 1 else v[:1, :2].cpu(), scale)
    res["parity"] = {"max_abs": orc.max_abs(o[:1, :2].cpu(), ref), "rel_l2": orc.rel_l2(o[:1, :2].cpu(), ref),
                     "lse_abs": orc.max_abs(lse[:1, :2].cpu(), lse_ref),
                     "checked": "two (batch, head) rows of the timed output vs the fp32 oracle"}
    # end to end: pinned host K/V/Q in, O and LSE out, through the public operator
    import tilefusion_b200 as tilefusion

    e2e_steps = max(1, min(steps, 5))
    hq, hk, hv = (t.cpu().pin_memory() for t in (q, k, v))
    ho = torch.empty(o.shape, dtype=o.dtype).pin_memory()

    def e2e_step():
        out, _ = tilefusion.ops.flash_decoding(hq.to(device, non_blocking=True), hk.to(device, non_blocking=True),
                                               hv.to(device, non_blocking=True), kv_chunk, 0, scale)
        ho.copy_(out, non_blocking=True)

    e2e_secs, _ = time_steps(e2e_step, e2e_steps, 2, device, world, max_repeats=1)
    res["e2e"] = {"value": total_units * e2e_steps / e2e_secs / 1e9, "unit": "GB/s",
                  "h2d_bytes_per_step": q.numel() * 2 + 2 * k.numel() * kv_bytes,
                  "d2h_bytes_per_step": o.numel() * 2, "steps": e2e_steps}
    return res


def run_two_gemms(args, w, device, rank, world):
    """fused_two_gemms through tf_fused_two_gemms: A [M,K], B [N,K], C [P,N] -> D [M,P]."""
    from tilefusion_b200 import _cabi

    lib = _cabi.lib()
    dt = torch_dtype(w["dtype"])
    g = torch.Generator(device=device).manual_seed(5 + rank)
    a = (torch.randn(w["M"], w["K"], generator=g, device=device)).to(dt)
    b = (torch.randn(w["N"], w["K"], generator=g, device=device) * 0.125).to(dt)
    c = (torch.randn(w["P"], w["N"], generator=g, device=device) * 0.125).to(dt)
    d = torch.empty(w["M"], w["P"], dtype=dt, device=device)
    stream = torch.cuda.current_stream(device).cuda_stream
    code = _cabi.TF_F16 if w["dtype"] == "fp16" else _cabi.TF_BF16
    argv = (a.data_ptr(), b.data_ptr(), c.data_ptr(), d.data_ptr(), w["M"], w["N"], w["K"], w["P"], code,
            a.stride(0), b.stride(0), c.stride(0), d.stride(0), stream)

    def step():
        rc = lib.tf_fused_two_gemms(*argv)
        if rc != 0:
            _cabi.check(rc)

    secs, info = time_steps(step, args.steps, args.warmup, device, world)
    flops = 2.0 * w["M"] * w["N"] * (w["K"] + w["P"])
    pk = peaks()
    ach = flops * args.steps / secs / 1e12
    from oracle import attention_oracle as orc

    rows = slice(0, min(w["M"], 256))
    ref = ((a[rows].float() @ b.float().t()).to(dt).float() @ c.float().t()).cpu()
    res = dict(value=ach * world, unit="TFLOP/s", secs=secs, info=info, launches=args.steps,
               roofline={"bound": "tensor", "achieved": ach, "peak": pk["bf16_tflops"], "unit": "TFLOP/s",
                         "frac": ach / pk["bf16_tflops"], "traffic": None, "traffic_source": "not captured",
                         "kernel": "attn_fwd_kernel<T, D, true> (one CTA per 128 rows of A: M/128 CTAs)",
                         "peak_source": pk["source"] + " (burst cuBLAS bf16)"},
               parity={"rel_l2": orc.rel_l2(d[rows].cpu(), ref), "max_abs": orc.max_abs(d[rows].cpu(), ref),
                       "checked": "first 256 rows vs (A B^T rounded to 16 bits) C^T in fp32 (torch, on the device)"})
    return res


def run_mma_rate():
    """Prints one JSON line: SM clocks per M128 K16 tcgen05.mma (fp16 operands, fp32 accumulators), 256
    issued back to back by one thread on one SM, for the operand forms the kernels use, and for the
    two-CTA form (M256 over a pair of SMs) the kernels do not use."""
    import ctypes as C

    from tilefusion_b200 import _cabi

    lib = _cabi.lib()
    rows = []
    for n in (64, 128, 256):
        for a_tmem in (0, 1):
            for b_mn in (0, 1):
                for desc32, uniform in ((0, 0), (1, 0), (1, 1)):
                    best = None
                    for _ in range(3):
                        issue, done = C.c_int64(0), C.c_int64(0)
                        _cabi.check(lib.tf_probe_mma_clocks(a_tmem, n, b_mn, desc32, uniform, 256, C.byref(issue), C.byref(done)))
                        if best is None or done.value < best[1]:
                            best = (issue.value, done.value)
                    rows.append({"n": n, "a": "tmem" if a_tmem else "smem", "b": "mn-major" if b_mn else "k-major",
                                 "descriptors": "32-bit halves" if desc32 else "64-bit, built per MMA",
                                 "issuer": "elected lane of a whole warp" if uniform else "lane 0 in a branch",
                                 "issue_clk_per_mma": best[0] / 256, "complete_clk_per_mma": best[1] / 256,
                                 "nominal_clk_per_mma": 128 * n * 16 * 2 / 8192})
    # the two-CTA form: M256 over two SMs, the same arithmetic per SM as the M128 rows above
    for n in (64, 128, 256):
        for a_tmem in (0, 1):
            for b_mn in (0, 1):
                best = None
                for _ in range(3):
                    issue, done = C.c_int64(0), C.c_int64(0)
                    _cabi.check(lib.tf_probe_mma_pair_clocks(a_tmem, n, b_mn, 256, C.byref(issue), C.byref(done)))
                    if best is None or done.value < best[1]:
                        best = (issue.value, done.value)
                rows.append({"n": n, "form": "cta_group::2, M256 over two SMs", "a": "tmem" if a_tmem else "smem",
                             "b": "mn-major" if b_mn else "k-major", "descriptors": "32-bit halves",
                             "issuer": "elected lane of a whole warp", "issue_clk_per_mma": best[0] / 256,
                             "complete_clk_per_mma": best[1] / 256, "nominal_clk_per_mma": 128 * n * 16 * 2 / 8192})
    print(json.dumps({"metric": "mma_clocks", "unit": "SM clocks per tcgen05.mma (M128 K16)", "n_mma": 256,
                      "nominal": "8192 dense fp16 FLOP per clock and SM", "rows": rows}), flush=True)


def secondary_object(wname, res, steps, world):
    """Compact form of a secondary workload's result for the default line."""
    obj = {"workload": wname, "value": res["value"], "unit": res["unit"], "value_per_gpu": res["value"] / world,
           "steps": steps, "ms_per_step": res["secs"] / steps * 1e3, "repeats": res["info"]["repeats"],
           "roofline": res["roofline"], "clocks": {k: v for k, v in res["info"]["clocks"].items() if k != "sm_mhz_all"},
           "gpu_launches": res["launches"]}
    for key in ("e2e", "parity", "transport", "transport_note"):
        if key in res and res[key] not in (None, ""):
            obj[key] = res[key]
    return obj


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="tilefusion_b200", choices=["tilefusion_b200", "reference"])
    ap.add_argument("--workload", default="prefill_c2", choices=sorted(WORKLOADS))
    ap.add_argument("--causal", action="store_true",
                    help="prefill workloads: mask key index > query index (FLOPs counted over unmasked pairs)")
    ap.add_argument("--transport", default=None, choices=["p2p", "nccl"],
                    help="KV-sharded decode: only this transport (default: both, peer-memory exchange first)")
    ap.add_argument("--no-secondary", action="store_true",
                    help="skip the decode / decode_c4 / prefill_c5 / causal objects and the CPU baseline")
    ap.add_argument("--profile", action="store_true",
                    help="device-timed steps only (no end-to-end pass, parity check, secondary objects or CPU "
                         "baseline): the command to put under ncu")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3)
    if args.profile:
        args.no_secondary = True
        global MAX_REPEATS
        MAX_REPEATS = 1          # one timed region: a capture should see few launches
    w = WORKLOADS[args.workload]

    if args.impl == "reference":
        run_reference_arm(args, w, args.workload)
        return

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the attention path has no CPU fallback")
    device = torch.device("cuda", local_rank)
    torch.cuda.set_device(device)
    if world > 1:
        import torch.distributed as dist

        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=device)

    if w["kind"] == "mma_rate":
        if rank == 0:
            run_mma_rate()
        return
    if w["kind"] == "prefill":
        res = run_prefill(args, w, args.workload, device, rank, world, causal=args.causal)
    elif w["kind"] == "two_gemms":
        res = run_two_gemms(args, w, device, rank, world)
    elif w["kind"] == "backward":
        res = run_backward(args, w, device, rank, world, args.steps, args.warmup)
    else:
        res = run_decode(args, w, args.workload, device, rank, world)

    line = {
        "metric": metric_name(w), "value": res["value"], "unit": res["unit"], "n_gpus": world,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": res["secs"] / args.steps * 1e3,
        "higher_is_better": True, "scaling": w["scaling"], "vs_baseline": None,
        "dtype": "f16" if w["dtype"] == "fp16" else "bf16", "data": "synthetic",
        "config": workload_config(w, args.workload, world, args.causal and w["kind"] == "prefill"),
        "value_per_gpu": res["value"] / world,
        "clocks": res["info"]["clocks"], "repeats": res["info"]["repeats"],
        "region_ms_per_step": res["info"]["region_ms_per_step"], "gpu_launches": res["launches"],
        "roofline": res["roofline"],
    }
    for key in ("e2e", "parity"):
        if key in res:
            line[key] = res[key]
    if "transport" in res:
        line["config"]["transport"] = res["transport"]
    if "by_transport" in res:
        line["by_transport"] = {t: secondary_object(args.workload, r, args.steps, world)
                                for t, r in res["by_transport"].items()}

    if not args.no_secondary and args.workload == "prefill_c2" and not args.causal:
        # the rest of the metric, every object at every N
        sec_steps = max(10, min(args.steps, 50))
        dres = run_decode(args, WORKLOADS["decode_c3"], "decode_c3", device, rank, world, steps=sec_steps, warmup=3)
        line["decode"] = secondary_object("decode_c3", dres, sec_steps, world)
        del dres
        torch.cuda.empty_cache()
        d8 = run_decode(args, WORKLOADS["decode_c3_fp8"], "decode_c3_fp8", device, rank, world, steps=sec_steps, warmup=3)
        line["decode_fp8"] = secondary_object("decode_c3_fp8", d8, sec_steps, world)
        line["decode_fp8"]["kv_cache"] = "e4m3, one byte per element; GB/s counts the 8-bit bytes"
        line["decode_fp8"]["speedup_vs_16bit_cache"] = line["decode"]["ms_per_step"] / line["decode_fp8"]["ms_per_step"]
        del d8
        torch.cuda.empty_cache()
        c4 = run_decode(args, WORKLOADS["decode_c4"], "decode_c4", device, rank, world, steps=sec_steps, warmup=3)
        line["decode_c4"] = secondary_object("decode_c4", c4, sec_steps, world)
        line["decode_c4"]["by_transport"] = {t: secondary_object("decode_c4", r, sec_steps, world)
                                             for t, r in c4["by_transport"].items()}
        torch.cuda.empty_cache()
        c5_steps = max(3, min(args.steps, 6 * world))
        c5 = run_prefill(args, WORKLOADS["prefill_c5"], "prefill_c5", device, rank, world, steps=c5_steps, warmup=3,
                         with_e2e=False)
        line["prefill_c5"] = secondary_object("prefill_c5", c5, c5_steps, world)
        torch.cuda.empty_cache()
        cz = run_prefill(args, w, "prefill_c2", device, rank, world, causal=True, with_e2e=False)
        line["causal"] = secondary_object("prefill_c2+causal", cz, args.steps, world)
        line["causal"]["flops_counted"] = "unmasked (query, key) pairs only"
        torch.cuda.empty_cache()
        bw = run_backward(args, w, device, rank, world, max(5, min(args.steps, 20)), 3)
        line["backward"] = secondary_object("prefill_c2 backward", bw, max(5, min(args.steps, 20)), world)

    if rank == 0 and world == 1 and not args.no_secondary and w["kind"] in ("prefill", "decode"):
        line["cpu_baseline"] = cpu_baseline(w)
    if world > 1:
        import torch.distributed as dist

        dist.barrier()
        dist.destroy_process_group()
    if rank == 0:
        print(json.dumps(line), flush=True)


if __name__ == "__main__":
    main()
