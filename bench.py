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
stream, max over ranks.  `e2e` is the same metric through the public Python
operator with inputs copied from pinned host memory and the result copied back
inside the timed region.  `roofline` describes the dominant kernel against the
measured peaks in MEASURED_PEAKS.json; `cpu_baseline` times the oracle (the
reference's torch expression, fp32) on the host cores on a bounded sample.

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
WORKLOADS["decode_gqa_profile"] = dict(WORKLOADS["decode_gqa"], B=16)
# One rank's share of decode_c4 when the KV length is sharded over 8 GPUs.
WORKLOADS["decode_c4_shard8"] = dict(WORKLOADS["decode_c4"], L=131072 // 8, scaling="weak")
FALLBACK_PEAKS = dict(hbm_gbs=6650.0, bf16_tflops=1590.0)   # earlier measurement on this pool

# DRAM traffic (dram__bytes_read.sum + dram__bytes_write.sum) of the dominant
# kernel from the ncu captures summarised under profiles/, per (batch, head)
# problem of the captured case; traffic grows in proportion to batch x heads,
# so a launch is scaled by the problems it processes.
NCU_TRAFFIC_PER_HEAD = {
    # attn_fwd_pair_kernel, B4 H32 L2048 D128 fp16: 203.0 MB read + 46.9 MB written over 128 heads
    ("prefill", 2048, 128): (203.0e6 + 46.9e6) / 128,
    # decode_split_kernel, B4 H32 Lk8192 D128 fp16: 536.9 MB read + 3.8 MB written over 128 heads
    ("decode", 8192, 128): (536.9e6 + 3.8e6) / 128,
}
# attn_fwd_pair_kernel in split-KV mode, B16 Hq32 Hkv8 Lk8192 D128 fp16: 537.2 MB read + 5.9 MB
# written over 128 (batch, KV head) groups
NCU_TRAFFIC_PER_KV_HEAD_GQA = {("decode", 8192, 128): (537.2e6 + 5.9e6) / 128}


def ncu_traffic(w, heads_in_launch):
    if "Hkv" in w:      # grouped-query decode: traffic scales with the KV heads
        per_head = NCU_TRAFFIC_PER_KV_HEAD_GQA.get((w["kind"], w["L"], w["D"]))
        heads_in_launch = heads_in_launch // w["H"] * w["Hkv"]
    else:
        per_head = NCU_TRAFFIC_PER_HEAD.get((w["kind"], w["L"], w["D"]))
    return None if per_head is None else per_head * heads_in_launch


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


def decode_bytes(b, h, lk, d):
    return 2.0 * b * h * lk * d * 2


# ------------------------------------------------------------------ clocks ---
class ClockSampler:
    """Samples SM clock and throttle reasons through NVML while work is queued."""

    REASONS = {
        0x8: "hw_slowdown", 0x40: "hw_thermal_slowdown", 0x20: "sw_thermal_slowdown",
        0x4: "sw_power_cap", 0x80: "hw_power_brake_slowdown",
    }

    def __init__(self, device_index: int):
        self.samples, self.reasons, self.max_mhz = [], set(), None
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
            self.samples.append(self._nv.nvmlDeviceGetClockInfo(self._h, self._nv.NVML_CLOCK_SM))
            mask = self._nv.nvmlDeviceGetCurrentClocksEventReasons(self._h)
            for bit, name in self.REASONS.items():
                if mask & bit:
                    self.reasons.add(name)
        except Exception:
            pass

    def _run(self):
        while not self._stop.is_set():
            self._sample()
            time.sleep(0.005)

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
                "samples": len(s)}


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
    return "prefill_tflops" if w["kind"] == "prefill" else "decode_hbm_gbs"


def workload_config(w, name, n_gpus, causal=False):
    return {"workload": name + ("+causal" if causal else ""), "batch_per_step": w["B"] * (n_gpus if w["scaling"] == "weak" else 1),
            "heads": w["H"], "len_q": w["L"] if w["kind"] == "prefill" else 1, "len_kv": w["L"],
            "head_dim": w["D"], "causal": bool(causal), "softmax_scale": "1/sqrt(D)",
            "sharding": ("batch x heads, no collective" if w["kind"] == "prefill" or w["scaling"] == "weak"
                         else "KV length + NCCL all-gather of (m,l,O) rows"),
            "l2": "inputs larger than L2 (126 MB); no flush between steps"}


# ------------------------------------------------------------- GPU timing ----
def time_steps(fn, steps, warmup, device, world, sampler_holder=None):
    """W warm-up steps, then K steps bracketed by barrier+synchronize; CUDA events on
    the current stream; returns max-over-ranks seconds."""
    import torch.distributed as dist

    for _ in range(warmup):
        fn()
    torch.cuda.synchronize(device)
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize(device)
    start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    sampler = ClockSampler(device.index if device.index is not None else 0)
    with sampler:
        start.record()
        for _ in range(steps):
            fn()
        end.record()
        end.synchronize()
    torch.cuda.synchronize(device)
    if world > 1:
        dist.barrier()
    secs = start.elapsed_time(end) / 1e3
    if world > 1:
        t = torch.tensor([secs], dtype=torch.float64, device=device)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        secs = t.item()
    if sampler_holder is not None:
        sampler_holder.append(sampler.summary())
    return secs


def run_prefill(args, w, name, device, rank, world):
    import ctypes as C

    from tilefusion_b200 import _cabi
    import tilefusion_b200 as tilefusion

    lib = _cabi.lib()
    # local batch: weak scaling keeps B per rank; strong scaling splits batch x heads
    causal = bool(getattr(args, "causal", False))
    if w["scaling"] == "weak":
        b_local, h_local = w["B"], w["H"]
        total_units = prefill_flops(w["B"] * world, w["H"], w["L"], w["L"], w["D"], causal)
    else:
        from tilefusion_b200.shard import head_slice

        h0, h1 = head_slice(w["B"] * w["H"], rank, world)
        b_local, h_local = (h1 - h0), 1         # flattened heads as the batch axis
        total_units = prefill_flops(w["B"], w["H"], w["L"], w["L"], w["D"], causal)
    wl = dict(w, H=h_local, seed=w["seed"] + 1000 * rank)
    q, k, v = make_inputs(wl, device, b=b_local)
    o = torch.empty_like(q)
    scale = 1.0 / math.sqrt(w["D"])
    d = _cabi.TfAttnDesc()
    d.dtype = _cabi.TF_F16 if w["dtype"] == "fp16" else _cabi.TF_BF16
    d.batch, d.heads, d.len_q, d.len_kv, d.head_dim, d.head_dim_v = b_local, h_local, w["L"], w["L"], w["D"], w["D"]
    d.softmax_scale = scale
    d.causal = int(causal)
    d.q_stride_b, d.q_stride_h, d.q_stride_l = q.stride(0), q.stride(1), q.stride(2)
    d.k_stride_b, d.k_stride_h, d.k_stride_l, d.k_stride_d = k.stride()
    d.v_stride_b, d.v_stride_h, d.v_stride_l, d.v_stride_d = v.stride()
    d.o_stride_b, d.o_stride_h, d.o_stride_l = o.stride(0), o.stride(1), o.stride(2)
    stream = torch.cuda.current_stream(device).cuda_stream
    qp, kp, vp, op = q.data_ptr(), k.data_ptr(), v.data_ptr(), o.data_ptr()

    def step():
        rc = lib.tf_attn_fwd(qp, kp, vp, op, None, C.byref(d), stream)
        if rc != 0:
            _cabi.check(rc)

    clocks = []
    secs = time_steps(step, args.steps, args.warmup, device, world, clocks)
    value = total_units * args.steps / secs / 1e12
    per_launch_s = secs / args.steps
    local_flops = prefill_flops(b_local, h_local, w["L"], w["L"], w["D"], causal)

    pk = peaks()
    # A kernel timed alone in a short region is held against the burst cuBLAS figure;
    # when the timed region is long enough to run into the power cap (seconds-long
    # loops, sw_power_cap active) the sustained figure is the like-for-like peak.
    sustained = ("sw_power_cap" in clocks[0]["reasons"] or secs > 0.5) and pk.get("bf16_tflops_sustained", 0) > 0
    peak_tf = pk["bf16_tflops_sustained"] if sustained else pk["bf16_tflops"]
    roof = {"bound": "tensor", "achieved": local_flops / per_launch_s / 1e12, "peak": peak_tf,
            "unit": "TFLOP/s", "frac": local_flops / per_launch_s / 1e12 / peak_tf,
            "traffic": ncu_traffic(w, b_local * h_local), "kernel": "attn_fwd_pair_kernel",
            "algorithmic_bytes": 4.0 * b_local * h_local * w["L"] * w["D"] * 2,
            "peak_source": pk["source"] + (" (sustained cuBLAS bf16, power-capped loop)" if sustained
                                           else " (burst cuBLAS bf16)"),
            "frac_of_burst": local_flops / per_launch_s / 1e12 / pk["bf16_tflops"],
            "frac_of_nominal_2250": local_flops / per_launch_s / 1e12 / 2250.0}
    if args.profile:
        return dict(value=value, unit="TFLOP/s", secs=secs, clocks=clocks[0], roofline=roof,
                    launches=args.steps)

    # parity spot check on one (b, h) against the oracle
    from oracle import attention_oracle as orc

    ref, _ = orc.attention_fp32(q[0, 0].cpu(), k[0, 0].cpu(), v[0, 0].cpu(), scale, causal)
    parity = {"max_abs": orc.max_abs(o[0, 0].cpu(), ref), "rel_l2": orc.rel_l2(o[0, 0].cpu(), ref),
              "checked": "one (batch, head) of the timed output vs the fp32 oracle"}

    # end to end through the public operator, host buffers in and out
    e2e_steps = max(1, min(args.steps, 20))
    hq, hk, hv = (t.cpu().pin_memory() for t in (q, k, v))
    ho = torch.empty(o.shape, dtype=o.dtype).pin_memory()

    pipe = tilefusion.HostPipeline(
        lambda dq, dk, dv: tilefusion.ops.flash_attention(dq, dk.transpose(-1, -2), dv, 0, 0, 0, 0, scale, causal),
        device)

    def e2e_step():
        # pinned host Q, K, V in, O back into pinned host memory; copies of neighbouring
        # steps overlap with the kernel (tilefusion_b200.HostPipeline)
        pipe.submit((hq, hk, hv), ho)

    def e2e_steps_timed(n):
        torch.cuda.synchronize(device)
        t0 = time.perf_counter()
        for _ in range(n):
            e2e_step()
        pipe.flush()
        return time.perf_counter() - t0

    e2e_steps_timed(3)
    e2e_secs = e2e_steps_timed(e2e_steps)
    if world > 1:
        import torch.distributed as dist

        t = torch.tensor([e2e_secs], dtype=torch.float64, device=device)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        e2e_secs = t.item()
    e2e = {"value": total_units * e2e_steps / e2e_secs / 1e12, "unit": "TFLOP/s",
           "h2d_bytes_per_step": 3 * q.numel() * q.element_size(),
           "d2h_bytes_per_step": o.numel() * o.element_size(), "steps": e2e_steps,
           "timing": "host wall clock around submit..flush (three streams), max over ranks"}
    return dict(value=value, unit="TFLOP/s", secs=secs, clocks=clocks[0], parity=parity, e2e=e2e,
                roofline=roof, launches=args.steps)


def run_decode(args, w, name, device, rank, world, steps=None, warmup=None):
    import ctypes as C

    from tilefusion_b200 import _cabi

    steps = args.steps if steps is None else steps
    warmup = args.warmup if warmup is None else warmup
    lib = _cabi.lib()
    scale = 1.0 / math.sqrt(w["D"])
    stream = torch.cuda.current_stream(device).cuda_stream
    sharded = w["scaling"] == "strong" and world > 1
    if sharded:
        from tilefusion_b200.shard import ShardedDecoder, kv_slice

        k0, k1 = kv_slice(w["L"], rank, world)
        wq = dict(w)
        q = make_inputs(dict(wq, L=128), device)[0]                # replicated Q (same seed on every rank)
        _, k, v = make_inputs(dict(w, seed=w["seed"] + 1000 * rank), device, l=k1 - k0)
        dec = ShardedDecoder(w["B"], w["H"], w["D"], q.dtype, device, transport=getattr(args, "transport", None))

        def step():
            dec(q, k, v, scale)

        total_units = decode_bytes(w["B"], w["H"], w["L"], w["D"])
        local_units = decode_bytes(w["B"], w["H"], k1 - k0, w["D"])
        launches_per_step = 3      # split, merge (+ peer scatter), combine; the nccl transport adds one collective
    else:
        q, k, v = make_inputs(dict(w, seed=w["seed"] + 1000 * rank), device)
        o = torch.empty_like(q)
        lse = torch.empty(w["B"], w["H"], 1, dtype=torch.float32, device=device)
        d = _cabi.TfDecodeDesc()
        d.dtype = _cabi.TF_F16 if w["dtype"] == "fp16" else _cabi.TF_BF16
        d.batch, d.heads, d.len_kv, d.head_dim = w["B"], w["H"], w["L"], w["D"]
        d.kv_chunk, d.num_splits, d.softmax_scale = 512, 0, scale
        d.q_stride_b, d.q_stride_h = q.stride(0), q.stride(1)
        d.k_stride_b, d.k_stride_h = k.stride(0), k.stride(1)
        d.v_stride_b, d.v_stride_h = v.stride(0), v.stride(1)
        d.o_stride_b, d.o_stride_h = o.stride(0), o.stride(1)
        d.heads_kv = w.get("Hkv", w["H"])
        plan = _cabi.TfDecodePlan()
        _cabi.check(lib.tf_decode_plan(C.byref(d), C.byref(plan)))
        ws = torch.empty(plan.workspace_bytes // 4, dtype=torch.float32, device=device)
        ptrs = (q.data_ptr(), k.data_ptr(), v.data_ptr(), o.data_ptr(), lse.data_ptr(), ws.data_ptr())

        def step():
            rc = lib.tf_decode(ptrs[0], ptrs[1], ptrs[2], ptrs[3], ptrs[4], ptrs[5], ws.numel() * 4,
                               C.byref(d), stream)
            if rc != 0:
                _cabi.check(rc)

        mult = world if w["scaling"] == "weak" else 1
        hkv = w.get("Hkv", w["H"])
        total_units = decode_bytes(w["B"] * mult, hkv, w["L"], w["D"])
        local_units = decode_bytes(w["B"], hkv, w["L"], w["D"])
        d.heads_kv = hkv
        launches_per_step = 2

    clocks = []
    secs = time_steps(step, steps, warmup, device, world, clocks)
    value = total_units * steps / secs / 1e9
    pk = peaks()
    ach = local_units * steps / secs / 1e9
    roof = {"bound": "hbm", "achieved": ach, "peak": pk["hbm_gbs"], "unit": "GB/s",
            "frac": ach / pk["hbm_gbs"], "traffic": ncu_traffic(w, w["B"] * w["H"]) if not sharded else None,
            "algorithmic_bytes": local_units, "kernel": ("attn_fwd_pair_kernel in split-KV mode (+ combine)" if "Hkv" in w
                                                   else "decode_split_kernel (+ combine)"),
            "peak_source": pk["source"] + " (torch copy, read+write)", "frac_of_nominal_8000": ach / 8000.0}
    res = dict(value=value, unit="GB/s", secs=secs, clocks=clocks[0], roofline=roof,
               launches=launches_per_step * steps)
    if sharded:
        res["transport"] = dec.transport

    if not sharded and not args.profile:
        from oracle import attention_oracle as orc

        grp = w["H"] // w.get("Hkv", w["H"])
        ref, lse_ref = orc.decode_fp32(q[:1, :2].cpu(), k[:1, :1].cpu().expand(-1, 2, -1, -1) if grp > 1 else k[:1, :2].cpu(),
                                       v[:1, :1].cpu().expand(-1, 2, -1, -1) if grp > 1 else v[:1, :2].cpu(), scale)
        res["parity"] = {"max_abs": orc.max_abs(o[:1, :2].cpu(), ref),
                         "lse_abs": orc.max_abs(lse[:1, :2].cpu(), lse_ref),
                         "checked": "two (batch, head) rows of the timed output vs the fp32 oracle"}
        # end to end: pinned host K/V/Q in, O and LSE out, through the public operator
        import tilefusion_b200 as tilefusion

        e2e_steps = max(1, min(steps, 5))
        hq, hk, hv = (t.cpu().pin_memory() for t in (q, k, v))
        ho = torch.empty(o.shape, dtype=o.dtype).pin_memory()

        def e2e_step():
            out, _ = tilefusion.ops.flash_decoding(hq.to(device, non_blocking=True), hk.to(device, non_blocking=True),
                                                   hv.to(device, non_blocking=True), 512, 0, scale)
            ho.copy_(out, non_blocking=True)

        e2e_secs = time_steps(e2e_step, e2e_steps, 3, device, world)
        res["e2e"] = {"value": total_units * e2e_steps / e2e_secs / 1e9, "unit": "GB/s",
                      "h2d_bytes_per_step": (q.numel() + 2 * k.numel()) * 2,
                      "d2h_bytes_per_step": o.numel() * 2, "steps": e2e_steps}
    return res


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
                    help="KV-sharded decode: fused peer-memory gather (default) or NCCL all-gather")
    ap.add_argument("--no-secondary", action="store_true", help="skip the decode line and CPU baseline")
    ap.add_argument("--profile", action="store_true",
                    help="device-timed steps only (no end-to-end pass, parity check, decode line or CPU "
                         "baseline): the command to put under ncu")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3)
    if args.profile:
        args.no_secondary = True
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

    runner = run_prefill if w["kind"] == "prefill" else run_decode
    res = runner(args, w, args.workload, device, rank, world)

    line = {
        "metric": metric_name(w), "value": res["value"], "unit": res["unit"], "n_gpus": world,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": res["secs"] / args.steps * 1e3,
        "higher_is_better": True, "scaling": w["scaling"], "vs_baseline": None,
        "dtype": "f16" if w["dtype"] == "fp16" else "bf16", "data": "synthetic",
        "config": workload_config(w, args.workload, world, args.causal and w["kind"] == "prefill"),
        "value_per_gpu": res["value"] / world,
        "clocks": res["clocks"], "gpu_launches": res["launches"],
        "roofline": res["roofline"],
    }
    if "e2e" in res:
        line["e2e"] = res["e2e"]
    if "parity" in res:
        line["parity"] = res["parity"]
    if "transport" in res:
        line["config"]["transport"] = res["transport"]

    if not args.no_secondary and w["kind"] == "prefill":
        # the other half of the metric: decode GB/s (config 3 on one GPU per rank;
        # config 4 sharded over the ranks when there is more than one)
        dname = "decode_c3" if world == 1 else "decode_c4"
        dres = run_decode(args, WORKLOADS[dname], dname, device, rank, world,
                          steps=max(10, min(args.steps, 50)), warmup=3)
        line["decode"] = {"workload": dname, "value": dres["value"], "unit": "GB/s",
                          "value_per_gpu": dres["value"] / world,
                          "ms_per_step": dres["secs"] / max(10, min(args.steps, 50)) * 1e3,
                          "roofline": dres["roofline"], "clocks": dres["clocks"]}
        for key in ("e2e", "parity", "transport"):
            if key in dres:
                line["decode"][key] = dres[key]

    if rank == 0 and world == 1 and not args.no_secondary:
        line["cpu_baseline"] = cpu_baseline(w)
    if world > 1:
        import torch.distributed as dist

        dist.barrier()
        dist.destroy_process_group()
    if rank == 0:
        print(json.dumps(line), flush=True)


if __name__ == "__main__":
    main()
