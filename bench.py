#!/usr/bin/env python
"""Benchmark of the ring-attention hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

A "step" is one complete causal prefill pass (all cp_size ring steps) over one synthetic batch
of the workload BASELINE.json's metric is quoted on:

    causal ring-overlap prefill, zig-zag layout, fp16, batch 1, seq 32768, 8 heads,
    head_dim 64, MHA, Q/K/V ~ N(0,1); cp_size = number of GPUs (total work fixed: strong scaling)

Metric: causal-adjusted attention TFLOP/s, FLOPs = 4 * B * H * S^2 * D / 2 (the reference's own
model, apps/bench_attention/bench_attention.cu:46-51). `value` is the whole-job figure (all
GPUs together, inputs resident in HBM); `e2e` is the same pass through the host-buffer entry
point (host->device copies of Q/K/V and device->host copy of the output inside the timed
region). At N=1 the line also carries the split-K decode measurement (tokens/s, HBM GB/s) for
the decode workload (batch 4, 32 query / 8 KV heads, head_dim 128, 262144 cached tokens, fp16)
and a CPU baseline: the reference's own cpu_attention (compiled unchanged into oracle/_ref)
timed on this box's host cores on a bounded sample of the same workload.

`--impl reference` times that CPU reference alone, on all host threads, on a bounded sample per
step, and prints the same line with "impl": "reference".

For N > 1 launch with torchrun (one rank per GPU):
    python -m torch.distributed.run --nnodes=1 --nproc-per-node N --master-addr 127.0.0.1 \
        --master-port P bench.py --gpus N --steps K --warmup W
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

WORKLOAD = dict(batch=1, heads=8, kv_heads=8, seq=32768, head_dim=64, dtype="fp16", causal=True,
                layout="zigzag", n_splits=2)
DECODE = dict(batch=4, heads=32, kv_heads=8, head_dim=128, prompt=262144, dtype="fp16")
METRIC = "causal-adjusted attention TFLOP/s (prefill, whole job)"


def causal_flops(B, H, S, D):
    return 4.0 * B * H * float(S) * float(S) * D * 0.5


def measured_peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        with open(p) as f:
            d = json.load(f)
        return dict(tflops=d.get("bf16_tflops"), tflops_sustained=d.get("bf16_tflops_sustained"),
                    hbm_gbs=d.get("hbm_gbs"), source="measured")
    return dict(tflops=1590.0, tflops_sustained=1400.0, hbm_gbs=6650.0, source="fallback")


class ClockSampler:
    """Samples SM clock and throttle reasons with nvidia-smi while the timed region runs."""

    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
         "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index):
        self.index = index
        self.proc = None
        self.lines = []

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits",
                                          "-lms", "100", "-i", str(self.index)],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except Exception:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def stop(self):
        if not self.proc:
            return dict(sm_mhz=None, sm_max_mhz=None, reasons=["nvidia-smi unavailable"])
        self.proc.terminate()  # the exact process started above
        try:
            self.proc.wait(timeout=5)
        except Exception:
            pass
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for ln in self.lines:
            f = [x.strip() for x in ln.split(",")]
            if len(f) < 9:
                continue
            try:
                sm.append(float(f[1]))
                mx.append(float(f[2]))
            except ValueError:
                continue
            for name, val in zip(names, f[5:9]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        return dict(sm_mhz=statistics.median(sm) if sm else None, sm_max_mhz=max(mx) if mx else None,
                    samples=len(sm), reasons=sorted(reasons))


# ------------------------------------------------------------------ CPU reference arm ----

def cpu_reference_sample(threads):
    """One bounded sample of the prefill workload on the reference's cpu_attention: `threads`
    heads of causal attention at S = 8192, head_dim 64, N(0,1) inputs, one head per thread.
    Returns (seconds, causal-adjusted FLOPs, description, kind)."""
    import numpy as np

    import oracle
    S, D = 8192, WORKLOAD["head_dim"]
    H = max(1, threads)
    rng = np.random.default_rng(42)
    q = rng.standard_normal((1, H, S, D), dtype=np.float32)
    k = rng.standard_normal((1, H, S, D), dtype=np.float32)
    v = rng.standard_normal((1, H, S, D), dtype=np.float32)
    kind = "reference" if oracle.ref() is not None else "port"
    t0 = time.perf_counter()
    if kind == "reference":
        oracle.cpu_attention(q, k, v, True, impl="ref", threads=threads)
    else:
        oracle.cpu_attention(q[:, :1], k[:, :1], v[:, :1], True)
        H = 1
    dt = time.perf_counter() - t0
    desc = (f"{H} heads x causal S={S} D={D} fp32 N(0,1) (of the S=32768 workload), one head per thread, "
            f"{'unchanged reference cpu_attention (oracle/_ref)' if kind == 'reference' else 'C port of cpu_attention'}")
    return dt, causal_flops(1, H, S, D), desc, kind


def host_threads():
    try:
        return max(1, len(os.sched_getaffinity(0)))
    except Exception:
        return os.cpu_count() or 1


def run_reference_arm(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return 0
    threads = min(host_threads(), 64)
    for _ in range(min(args.warmup, 1)):
        cpu_reference_sample(threads)
    times, flops, desc, kind = [], 0.0, "", "reference"
    steps = max(1, args.steps)
    for _ in range(steps):
        dt, flops, desc, kind = cpu_reference_sample(threads)
        times.append(dt)
    ms = 1e3 * sum(times) / len(times)
    val = flops / (ms * 1e-3) / 1e12
    line = {
        "impl": "reference", "metric": METRIC, "value": val, "unit": "TFLOP/s", "n_gpus": args.gpus,
        "steps": steps, "warmup": min(args.warmup, 1), "ms_per_step": ms, "higher_is_better": True,
        "scaling": "strong", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": {"workload": "causal zig-zag ring-overlap prefill fp16 B1 S32768 H8 D64 (config 2)",
                   **WORKLOAD, "reference_sample": desc},
        "cpu_baseline": {"value": val, "unit": "TFLOP/s", "cores": threads, "kind": kind, "sample": desc},
        "e2e": {"value": val, "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)
    return 0


# ------------------------------------------------------------------------- GPU arm ----

def run_gpu_arm(args):
    import torch
    import torch.distributed as dist

    from ring_attention_b200 import api
    from ring_attention_b200._lib import SegMap

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if world != args.gpus:
        if world == 1 and args.gpus > 1:
            raise SystemExit("--gpus N > 1 needs torchrun (one rank per GPU); see the module docstring")
        args.gpus = world
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    P = world
    w = WORKLOAD
    B, H, S, D = w["batch"], w["heads"], w["seq"], w["head_dim"]
    part = api.RingPartition(P, rank, S, api.RingPartition.ZIGZAG, w["n_splits"])
    rows = part.local_positions()
    sloc = len(rows)

    # Synthetic N(0,1) inputs, one seeded generator for the global tensors; each rank keeps its rows.
    g = torch.Generator(device="cpu").manual_seed(42)
    host = [torch.randn((B, H, S, D), generator=g).to(torch.float16)[:, :, rows].contiguous().pin_memory()
            for _ in range(3)]
    dq, dk, dv = (t.to(dev, non_blocking=True) for t in host)
    out = torch.empty((B, H, sloc, D), dtype=torch.float32, device=dev)
    host_out = torch.empty((B, H, sloc, D), dtype=torch.float32).pin_memory()
    ring = api.Ring(rank, P)
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)  # > 126 MB L2
    stream = torch.cuda.current_stream()

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def one_pass():
        ring.prefill(dq, dk, dv, seq=S, causal=True, layout=1, n_splits=w["n_splits"], out=out)

    qmap1 = kmap1 = None
    if P == 1:
        qmap1, kmap1, _ = part.step_maps(0)

    def one_pass_host():
        if P == 1:
            # the host-buffer entry point of the C ABI: upload, step, download, synchronise
            api.check(api.lib().ra_prefill_host(
                api.RA_F16, host[0].data_ptr(), host[1].data_ptr(), host[2].data_ptr(), host_out.data_ptr(),
                None, api.AttentionShape(B, H, S, S, D).c(), qmap1, kmap1, 1, api.RA_STEP_CAUSAL, 0))
        else:
            dq.copy_(host[0], non_blocking=True)
            dk.copy_(host[1], non_blocking=True)
            dv.copy_(host[2], non_blocking=True)
            one_pass()
            host_out.copy_(out, non_blocking=True)
            torch.cuda.current_stream().synchronize()

    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()  # nvidia-smi needs a moment to start: begin before the warm-up
    for _ in range(max(args.warmup, 3)):
        flush.fill_(1)
        one_pass()
    barrier()
    assert api.device_status()[0] == 0, "a device-side wait ran out during warm-up"
    K = max(1, args.steps)
    ev = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(K)]
    barrier()
    for i in range(K):
        flush.fill_(i & 1)  # evict L2 between timed iterations (not timed)
        if world > 1:
            dist.barrier()
        ev[i][0].record(stream)
        one_pass()
        ev[i][1].record(stream)
    barrier()
    ms_steps = [a.elapsed_time(b) for a, b in ev]
    ms = sum(ms_steps) / K

    # end to end: host buffers in, host result out, copies inside the timed region
    for _ in range(2):
        one_pass_host()
    barrier()
    t0 = time.perf_counter()
    for _ in range(K):
        one_pass_host()
    barrier()
    ms_e2e = 1e3 * (time.perf_counter() - t0) / K
    clocks = sampler.stop() if rank == 0 else None
    status = api.device_status()

    if world > 1:
        t = torch.tensor([ms, ms_e2e], device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms, ms_e2e = float(t[0]), float(t[1])

    flops = causal_flops(B, H, S, D)
    peaks = measured_peaks()
    line = None
    if rank == 0:
        value = flops / (ms * 1e-3) / 1e12
        per_gpu = value / P
        h2d = sum(t.numel() * t.element_size() for t in host)
        d2h = host_out.numel() * host_out.element_size()
        line = {
            "metric": METRIC, "value": value, "unit": "TFLOP/s", "n_gpus": P, "steps": K,
            "warmup": max(args.warmup, 3), "ms_per_step": ms, "higher_is_better": True, "scaling": "strong",
            "vs_baseline": None, "dtype": "fp16", "data": "synthetic",
            "config": {"workload": "causal zig-zag ring-overlap prefill fp16 B1 S32768 H8 D64 (config 2)", **w,
                       "cp_size": P, "per_gpu_tflops": per_gpu, "l2": "256 MB flush between timed iterations",
                       "timing": "CUDA events per pass on the launching stream, mean of K, max over ranks"},
            "e2e": {"value": flops / (ms_e2e * 1e-3) / 1e12, "unit": "TFLOP/s", "ms_per_step": ms_e2e,
                    "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
                    "api": "ra_prefill_host" if P == 1 else "pinned H2D + ra_ring_prefill + D2H per rank"},
            "gpu_launches": K * P,  # one step kernel per ring step per pass on each rank
            "clocks": clocks,
            "roofline": {"bound": "tensor", "achieved": per_gpu, "peak": peaks["tflops"], "unit": "TFLOP/s",
                         "frac": per_gpu / peaks["tflops"], "traffic": None,
                         "peak_source": f"{peaks['source']} bf16 GEMM burst",
                         "kernel": "step_tc_kernel<64> (one launch per ring step)"},
            "device_status": status,
        }
    if P == 1 and rank == 0:
        if not args.no_decode:
            line["decode"] = bench_decode(api, torch, dev, args, peaks)
        if not args.no_cpu:
            threads = min(host_threads(), 64)
            dt, fl, desc, kind = cpu_reference_sample(threads)
            line["cpu_baseline"] = {"value": fl / dt / 1e12, "unit": "TFLOP/s", "cores": threads, "kind": kind,
                                    "sample": desc, "seconds": dt}
    if rank == 0:
        print(json.dumps(line), flush=True)
    ring.close()
    if world > 1:
        dist.destroy_process_group()
    return 0


def bench_decode(api, torch, dev, args, peaks):
    """Split-K decode against the decode workload's cache on one GPU: tokens/s and HBM GB/s."""
    d = DECODE
    B, H, kvH, D, L = d["batch"], d["heads"], d["kv_heads"], d["head_dim"], d["prompt"]
    g = torch.Generator(device=dev).manual_seed(7)
    k = torch.randn((B, kvH, L, D), generator=g, device=dev, dtype=torch.float16)
    v = torch.randn((B, kvH, L, D), generator=g, device=dev, dtype=torch.float16)
    q = torch.randn((B, H, 1, D), generator=g, device=dev, dtype=torch.float16)
    shape = api.AttentionShape(B, H, 1, L, D, kvH)
    out = torch.empty((B, H, 1, D), device=dev)
    m = torch.empty((B, H, 1), device=dev)
    l = torch.empty((B, H, 1), device=dev)
    stream = torch.cuda.current_stream()

    def step():
        api.launch_attention_init(out, m, l, shape)
        api.launch_attention_decode_step(q, k, v, out, m, l, shape, 0, 0, False)
        api.launch_attention_finalize(out, l, shape)

    for _ in range(3):
        step()
    torch.cuda.synchronize()
    n = max(args.steps, 10)
    ev = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(n)]
    for i in range(n):  # the 4.3 GB cache is far larger than L2: no flush needed
        ev[i][0].record(stream)
        step()
        ev[i][1].record(stream)
    torch.cuda.synchronize()
    ms = sum(a.elapsed_time(b) for a, b in ev) / n
    kv_bytes = 2.0 * B * kvH * L * D * 2
    gbs = kv_bytes / (ms * 1e-3) / 1e9
    return {"workload": "decode B4 H32 kvH8 D128 fp16, 262144 cached tokens, cp_size 1 (config 4)",
            "ms_per_step": ms, "tokens_per_s": B / (ms * 1e-3), "hbm_gbs": gbs,
            "roofline": {"bound": "hbm", "achieved": gbs, "peak": peaks["hbm_gbs"], "unit": "GB/s",
                         "frac": gbs / peaks["hbm_gbs"], "traffic": None,
                         "peak_source": f"{peaks['source']} copy bandwidth",
                         "algorithmic_bytes": kv_bytes},
            "gpu_launches_per_step": 4}


def run_profile_case(args):
    """A small, self-ending case for `ncu`: few launches, at most ~1 GB on the device.
    prefill: the benchmark's own shape (100 MB of Q/K/V, larger than L2 together with the 67 MB
    output), 1 warm-up + 2 launches of the step kernel. decode: the decode workload at a
    quarter of the cached length (65536 tokens, 1 GB of K/V), 1 warm-up + 2 steps."""
    import torch

    from ring_attention_b200 import api
    from ring_attention_b200._lib import SegMap
    torch.cuda.set_device(0)
    dev = torch.device("cuda", 0)
    g = torch.Generator(device=dev).manual_seed(42)
    if args.profile == "prefill":
        w = WORKLOAD
        B, H, S, D = w["batch"], w["heads"], w["seq"], w["head_dim"]
        q, k, v = (torch.randn((B, H, S, D), generator=g, device=dev, dtype=torch.float16) for _ in range(3))
        out = torch.empty((B, H, S, D), device=dev)
        m = torch.empty((B, H, S), device=dev)
        l = torch.empty_like(m)
        part = api.RingPartition(1, 0, S, api.RingPartition.ZIGZAG, w["n_splits"])
        qmap, kmap, stride = part.step_maps(0)
        for _ in range(3):
            api.attention_step_ex(q, k, v, out, m, l, api.AttentionShape(B, H, S, S, D), qmap, kmap, stride,
                                  causal=True, fresh=True, finalize=True)
    else:
        d = DECODE
        B, H, kvH, D, L = d["batch"], d["heads"], d["kv_heads"], d["head_dim"], d["prompt"] // 4
        k = torch.randn((B, kvH, L, D), generator=g, device=dev, dtype=torch.float16)
        v = torch.randn((B, kvH, L, D), generator=g, device=dev, dtype=torch.float16)
        q = torch.randn((B, H, 1, D), generator=g, device=dev, dtype=torch.float16)
        shape = api.AttentionShape(B, H, 1, L, D, kvH)
        out = torch.empty((B, H, 1, D), device=dev)
        m = torch.empty((B, H, 1), device=dev)
        l = torch.empty_like(m)
        for _ in range(3):
            api.launch_attention_init(out, m, l, shape)
            api.launch_attention_decode_step(q, k, v, out, m, l, shape, 0, 0, False)
            api.launch_attention_finalize(out, l, shape)
    torch.cuda.synchronize()
    assert api.device_status()[0] == 0
    print(json.dumps({"profile_case": args.profile, "ok": True}))
    return 0


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--profile", default=None, choices=["prefill", "decode"],
                    help="run a small self-ending case for ncu instead of the benchmark")
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--no-decode", action="store_true")
    ap.add_argument("--no-cpu", action="store_true")
    args = ap.parse_args()
    if args.profile:
        return run_profile_case(args)
    if args.impl == "reference":
        return run_reference_arm(args)
    return run_gpu_arm(args)


if __name__ == "__main__":
    sys.exit(main())
