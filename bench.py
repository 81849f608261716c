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
points of the C ABI (ra_prefill_host at N = 1, ra_ring_prefill_host at N > 1: host->device copies
of Q/K/V and device->host copy of the output inside the timed region). `checked_rows`: output rows
of every rank against the CPU oracle at full size, untimed, at every N. The line also carries
the split-K decode measurement (tokens/s, HBM GB/s) for the decode workload (batch 4, 32 query /
8 KV heads, head_dim 128, 262144 cached tokens, fp16; sharded over the ranks at N > 1, with one
output row per batch element checked against the oracle), the other prefill workloads of the
metric as secondary objects (`config5`: 131072 tokens per GPU, zig-zag-n 2, four documents, the
1 M-token workload at N = 8; `config3`: GQA striped), and at N = 1 a CPU baseline: the
reference's own cpu_attention (compiled unchanged into oracle/_ref) timed on this box's host
cores on a bounded sample of the same workload.

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
# The benchmark line is config 2 (the workload the metric is quoted on). The other prefill
# workloads of the same metric can be run with --workload for the scaling tables; they keep the
# same JSON contract and say which workload they are in config.workload.
WORKLOADS = {
    "config2": dict(WORKLOAD, name="causal zig-zag ring-overlap prefill fp16 B1 S32768 H8 D64 (config 2)",
                    scale=1.0, doc_len=0, seq_per_gpu=None),
    "config3": dict(batch=2, heads=32, kv_heads=8, seq=131072, head_dim=128, dtype="fp16", causal=True,
                    layout="striped", n_splits=2, scale=0.5, doc_len=0, seq_per_gpu=None,
                    name="causal GQA striped ring-overlap prefill fp16 B2 S131072 H32/kvH8 D128 (config 3)"),
    # 1 M tokens on 8 GPUs, 512 K on 4: 131072 tokens per GPU, four equal documents
    "config5": dict(batch=1, heads=16, kv_heads=16, seq=None, head_dim=128, dtype="fp16", causal=True,
                    layout="zigzag", n_splits=4, scale=1.0, doc_len="seq/4", seq_per_gpu=131072,
                    name="long-context causal prefill fp16 B1 H16 D128, zig-zag-n=2, 4 documents, "
                         "131072 tokens per GPU (config 5: 1048576 tokens on 8 GPUs)"),
}
LAYOUTS = {"contiguous": 0, "zigzag": 1, "striped": 2}
DECODE = dict(batch=4, heads=32, kv_heads=8, head_dim=128, prompt=262144, dtype="fp16")
METRIC = "causal-adjusted attention TFLOP/s (prefill, whole job)"
# DRAM bytes (read + write) of one step-kernel launch on the benchmark shape at N = 1, from one ncu
# capture of that launch (179.5 MB read + 35.6 MB written; algorithmic: 100.7 MB of Q/K/V in, 68.2 MB
# of out / m / l). A property of the workload: the run that prints it does not re-measure it.
TRAFFIC_CONFIG2_N1 = 215.0e6


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
                                          "-lms", "10", "-i", str(self.index)],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
            t0 = time.perf_counter()  # the first sample takes nvidia-smi a moment: wait for it
            while not self.lines and time.perf_counter() - t0 < 5.0:
                time.sleep(0.01)
        except Exception:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.lines.append((time.perf_counter(), line.strip()))

    def now(self):
        return time.perf_counter()

    def window(self, t0, t1):
        """Clocks and throttle reasons of the samples taken between two perf_counter stamps
        (all samples when the window caught none: a timed region shorter than the sampling period)."""
        if not self.proc:
            return dict(sm_mhz=None, sm_max_mhz=None, reasons=["nvidia-smi unavailable"])
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        lines = list(self.lines)
        timed = [ln for t, ln in lines if t0 <= t <= t1]
        for ln in (timed if timed else [ln for _, ln in lines]):
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
                    samples=len(sm), in_window=bool(timed), reasons=sorted(reasons))

    def stop(self):
        if not self.proc:
            return
        self.proc.terminate()  # the exact process started above
        try:
            self.proc.wait(timeout=5)
        except Exception:
            pass


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

class Case:
    """One prefill workload materialised on this rank: shards, partition, output buffer."""

    def __init__(self, api, torch, name, P, rank, dev, want_host):
        w = dict(WORKLOADS[name])
        if w["seq"] is None:
            w["seq"] = w["seq_per_gpu"] * P
        self.key, self.w, self.P, self.rank = name, w, P, rank
        B, H, kvH, S, D = w["batch"], w["heads"], w["kv_heads"], w["seq"], w["head_dim"]
        self.layout = LAYOUTS[w["layout"]]
        self.doc_len = S // 4 if w["doc_len"] == "seq/4" else int(w["doc_len"])
        w["doc_len"] = self.doc_len
        self.part = api.RingPartition(P, rank, S, self.layout, w["n_splits"])
        self.rows = self.part.local_positions()
        sloc = len(self.rows)
        self.host = None
        if name == "config2":
            # Synthetic N(0,1) inputs, one seeded generator for the global tensors; each rank keeps its rows.
            g = torch.Generator(device="cpu").manual_seed(42)
            host = [torch.randn((B, H, S, D), generator=g).to(torch.float16)[:, :, self.rows].contiguous()
                    for _ in range(3)]
            self.host = [t.pin_memory() for t in host] if want_host else None
            self.dq, self.dk, self.dv = (t.to(dev) for t in host)
        else:
            # The larger workloads generate each rank's shard on its GPU (same distribution, seed + rank),
            # one (batch, head) slice at a time: materialising the global tensors on the host would take
            # tens of GB, and a whole fp32 shard on the device several more.
            g = torch.Generator(device=dev).manual_seed(42 + rank)

            def gen(heads):
                t = torch.empty((B, heads, sloc, D), dtype=torch.float16, device=dev)
                for b in range(B):
                    for h in range(heads):
                        t[b, h] = (torch.randn((sloc, D), generator=g, device=dev) * w["scale"]).to(torch.float16)
                return t
            self.dq, self.dk, self.dv = gen(H), gen(kvH), gen(kvH)
        self.out = torch.empty((B, H, sloc, D), dtype=torch.float32, device=dev)
        # causal-adjusted FLOPs; with documents the mask is block-diagonal causal (per document)
        self.flops = (causal_flops(B, H, S, D) if not self.doc_len
                      else (S // self.doc_len) * causal_flops(B, H, self.doc_len, D))

    def release(self):
        self.dq = self.dk = self.dv = self.out = self.host = None


def time_case(api, torch, dist, case, ring, schedule, K, W, world, dev, flush, sampler):
    """W warm-up passes, then K passes timed with CUDA events on the launching stream (L2 flushed
    between them, ranks aligned by a stream-ordered all-reduce that does not block the host),
    bracketed by barrier + synchronize; then one pass with the driver's own event timings."""
    w, S = case.w, case.w["seq"]
    stream = torch.cuda.current_stream()
    token = torch.zeros(1, device=dev)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def one_pass(timed=False):
        return ring.prefill(case.dq, case.dk, case.dv, seq=S, causal=True, layout=case.layout,
                            n_splits=w["n_splits"], doc_len=case.doc_len, out=case.out, schedule=schedule,
                            timed=timed)

    for _ in range(W):
        flush.fill_(1)
        one_pass()
    barrier()
    assert api.device_status()[0] == 0, "a device-side wait ran out during warm-up"
    ev = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(K)]
    barrier()
    t_begin = sampler.now()
    for i in range(K):
        flush.fill_(i & 1)  # evict L2 between timed iterations (not timed)
        if world > 1:
            dist.all_reduce(token)  # aligns the ranks on the device; the host runs ahead
        ev[i][0].record(stream)
        one_pass()
        ev[i][1].record(stream)
    barrier()
    t_end = sampler.now()
    ms = sum(a.elapsed_time(b) for a, b in ev) / K
    # one more pass with the driver's own event timings (the reference's RingResult fields):
    # compute = sum of the step kernels, comm = sum of the transfers on the side stream,
    # wait = pass time the compute stream spent not computing (transfers that were not hidden)
    # (three such passes, ranks aligned on the device before each as in the timed loop; the
    # median by pass time is reported, so that one rank entering late does not read as exposed
    # communication)
    passes = []
    for i in range(3):
        flush.fill_(i & 1)
        if world > 1:
            dist.all_reduce(token)
        _, rt = one_pass(timed=True)
        passes.append((rt.total_ms, rt.comp_ms, rt.comm_ms, rt.wait_ms))
    passes.sort()
    times = [ms, *passes[1]]
    if world > 1:
        t = torch.tensor(times, device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        times = [float(x) for x in t]
    clocks = sampler.window(t_begin, t_end)
    return times, clocks


def case_report(case, times, clocks, peaks, plan, checked):
    """The figures of one workload (used for the secondary objects of the line)."""
    ms = times[0]
    value = case.flops / (ms * 1e-3) / 1e12
    per_gpu = value / case.P
    return {"workload": case.w["name"], "seq": case.w["seq"], "cp_size": case.P, "ms_per_step": ms,
            "value": value, "unit": "TFLOP/s", "per_gpu_tflops": per_gpu,
            "frac_burst": per_gpu / peaks["tflops"], "frac_sustained": per_gpu / peaks["tflops_sustained"],
            "ring": {"total_ms": times[1], "comp_ms": times[2], "comm_ms": times[3], "wait_ms": times[4],
                     "exposed_comm_frac": times[4] / max(times[1], 1e-9), "schedule": plan[0],
                     "key_parts": plan[1], "kernel_launches_per_pass": plan[2]},
            "checked_rows": checked, "clocks": clocks}


def run_gpu_arm(args):
    import torch
    import torch.distributed as dist

    from ring_attention_b200 import api

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
    peaks = measured_peaks()
    ring = api.Ring(rank, P)
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)  # > 126 MB L2
    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()  # nvidia-smi needs a moment to start: begin before the warm-up
    K, W = max(1, args.steps), max(args.warmup, 3)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def plan_of(case):
        w = case.w
        return ring.plan(batch=w["batch"], heads=w["heads"], kv_heads=w["kv_heads"], seq=w["seq"],
                         head_dim=w["head_dim"], causal=True, layout=case.layout, n_splits=w["n_splits"],
                         doc_len=case.doc_len, schedule=args.schedule)

    # ---- the benchmark line: the workload the metric is quoted on (or --workload) ----
    case = Case(api, torch, args.workload, P, rank, dev, want_host=True)
    w = case.w
    B, H, kvH, S, D = w["batch"], w["heads"], w["kv_heads"], w["seq"], w["head_dim"]
    times, clocks = time_case(api, torch, dist, case, ring, args.schedule, K, W, world, dev, flush, sampler)
    ms = times[0]
    plan = plan_of(case)

    # end to end: this rank's shards in pinned host memory in, host result out, through the
    # host-buffer entry points of the C ABI (copies inside the timed region)
    host = case.host if case.host is not None else [t.cpu().pin_memory() for t in (case.dq, case.dk, case.dv)]
    host_out = torch.empty(tuple(case.out.shape), dtype=torch.float32).pin_memory()
    if P == 1:
        qmap1, kmap1, stride1 = case.part.step_maps(0)

        def one_pass_host():
            api.check(api.lib().ra_prefill_host(
                api.RA_F16, host[0].data_ptr(), host[1].data_ptr(), host[2].data_ptr(), host_out.data_ptr(),
                None, api.AttentionShape(B, H, S, S, D, kvH).c(), qmap1, kmap1, stride1, api.RA_STEP_CAUSAL,
                case.doc_len))
    else:
        def one_pass_host():
            ring.prefill_host(host[0], host[1], host[2], host_out, seq=S, causal=True, layout=case.layout,
                              n_splits=w["n_splits"], doc_len=case.doc_len, schedule=args.schedule)
    for _ in range(2):
        one_pass_host()
    barrier()
    t0 = time.perf_counter()
    for _ in range(K):
        one_pass_host()
    barrier()
    ms_e2e = 1e3 * (time.perf_counter() - t0) / K
    e2e_err = float((host_out.to(dev) - case.out).abs().max())  # the two paths computed the same thing
    status = api.device_status()
    if world > 1:
        t = torch.tensor([ms_e2e, e2e_err], device=dev, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms_e2e, e2e_err = float(t[0]), float(t[1])
    checked = check_rows(api, torch, dist, w, rank, P, case.rows, case.dq, case.dk, case.dv, case.out, dev)

    line = None
    if rank == 0:
        value = case.flops / (ms * 1e-3) / 1e12
        per_gpu = value / P
        h2d = sum(t.numel() * t.element_size() for t in host)
        d2h = host_out.numel() * host_out.element_size()
        line = {
            "metric": METRIC, "value": value, "unit": "TFLOP/s", "n_gpus": P, "steps": K,
            "warmup": W, "ms_per_step": ms, "higher_is_better": True, "scaling": "strong",
            "vs_baseline": None, "dtype": "fp16", "data": "synthetic",
            "config": {"workload": w["name"], **{k: v for k, v in w.items() if k not in ("name", "seq_per_gpu")},
                       "cp_size": P, "per_gpu_tflops": per_gpu, "l2": "256 MB flush between timed iterations",
                       "timing": "CUDA events per pass on the launching stream, mean of K, max over ranks"},
            "e2e": {"value": case.flops / (ms_e2e * 1e-3) / 1e12, "unit": "TFLOP/s", "ms_per_step": ms_e2e,
                    "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
                    "api": "ra_prefill_host" if P == 1 else "ra_ring_prefill_host",
                    "max_abs_diff_vs_device_path": e2e_err},
            # kernels of this library per pass on each rank (step kernels and the merge of partial states)
            "gpu_launches": K * P * plan[2],
            "clocks": clocks,
            "roofline": {"bound": "tensor", "achieved": per_gpu, "peak": peaks["tflops"], "unit": "TFLOP/s",
                         "frac": per_gpu / peaks["tflops"],
                         "traffic": TRAFFIC_CONFIG2_N1 if (P == 1 and args.workload == "config2") else None,
                         "traffic_unit": "bytes per launch (dram read + write; one ncu capture of this launch, "
                                         "a constant of the workload, not re-measured by this run)",
                         "peak_source": f"{peaks['source']} bf16 GEMM burst",
                         "kernel": f"step_tc_kernel<{D}>"},
            "device_status": status,
            "ring": {"total_ms": times[1], "comp_ms": times[2], "comm_ms": times[3], "wait_ms": times[4],
                     "exposed_comm_frac": times[4] / max(times[1], 1e-9),
                     "schedule": plan[0] if P > 1 else None, "key_parts": plan[1],
                     "kernel_launches_per_pass": plan[2],
                     "note": "one pass, max over ranks; wait = pass time not covered by step kernels"},
            "checked_rows": checked,
        }
    del host, host_out
    case.release()

    # ---- decode (config 4) ----
    if args.workload == "config2" and not args.no_decode:
        dec = (bench_ring_decode(api, torch, dist, dev, args, peaks, ring, rank, P) if P > 1
               else bench_decode(api, torch, dev, args, peaks))
        if rank == 0:
            line["decode"] = dec

    # ---- the other prefill workloads of the metric, as secondary objects of the same line ----
    if args.workload == "config2" and not args.no_extra:
        for name in ("config5", "config3"):
            torch.cuda.empty_cache()
            extra = Case(api, torch, name, P, rank, dev, want_host=False)
            k2 = max(2, min(K, 5))
            t2, c2 = time_case(api, torch, dist, extra, ring, args.schedule, k2, 2, world, dev, flush, sampler)
            chk = check_rows(api, torch, dist, extra.w, rank, P, extra.rows, extra.dq, extra.dk, extra.dv,
                             extra.out, dev)
            rep = case_report(extra, t2, c2, peaks, plan_of(extra), chk)
            rep["steps"], rep["warmup"] = k2, 2
            if rank == 0:
                line[name] = rep
            extra.release()
            del extra

    if P == 1 and rank == 0 and args.workload == "config2" and not args.no_cpu:
        threads = min(host_threads(), 64)
        dt, fl, desc, kind = cpu_reference_sample(threads)
        line["cpu_baseline"] = {"value": fl / dt / 1e12, "unit": "TFLOP/s", "cores": threads, "kind": kind,
                                "sample": desc, "seconds": dt}
    if rank == 0:
        sampler.stop()
        print(json.dumps(line), flush=True)
    ring.close()
    if world > 1:
        dist.destroy_process_group()
    return 0


def check_rows(api, torch, dist, w, rank, P, rows, dq, dk, dv, out, dev):
    """Parity at full size: a few output rows of head 0 on every rank against the CPU oracle
    (one causal row over the keys of its own document). K/V of head 0 are gathered from all
    ranks for this; nothing here is timed."""
    import numpy as np

    import oracle
    S, D, doc = w["seq"], w["head_dim"], w["doc_len"]
    kh, vh, pos = dk[0, 0].contiguous(), dv[0, 0].contiguous(), rows.to(dev)
    if P > 1:
        ks = [torch.empty_like(kh) for _ in range(P)]
        vs = [torch.empty_like(vh) for _ in range(P)]
        ps = [torch.empty_like(pos) for _ in range(P)]
        dist.all_gather(ks, kh)
        dist.all_gather(vs, vh)
        dist.all_gather(ps, pos)
        kh, vh, pos = torch.cat(ks), torch.cat(vs), torch.cat(ps)
    order = torch.argsort(pos)
    kg = kh[order].float().cpu().numpy()  # keys of head 0 in global order
    vg = vh[order].float().cpu().numpy()
    worst, n = 0.0, 0
    local = [0, 1, len(rows) // 4 - 1, len(rows) // 4, len(rows) // 2 + 5, len(rows) - 1]
    for li in local:
        p = int(rows[li])
        lo = (p // doc) * doc if doc else 0
        want, _ = oracle.attention_row(dq[0, 0, li].float().cpu().numpy(), kg[lo:p + 1], vg[lo:p + 1])
        got = out[0, 0, li].cpu().numpy()
        err = np.abs(got - want)
        assert np.all(err <= 1e-3 + 1e-3 * np.abs(want)), f"rank {rank} row {p}: max err {err.max()}"
        worst, n = max(worst, float(err.max())), n + 1
    t = torch.tensor([worst], device=dev)
    if P > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return {"rows_per_rank": n, "max_abs_err": float(t[0]), "tolerance": "atol=rtol=1e-3 vs CPU oracle"}


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
                         "frac": gbs / peaks["hbm_gbs"],
                         # ncu on a quarter of this cache (1.0738 GB read + 5.1 MB written per launch),
                         # scaled by 4: traffic is proportional to the cached length
                         # (profiles/decode_mma_kernel_config4_decode.md)
                         "traffic": 4 * (1.0738e9 + 5.1e6),
                         "traffic_unit": "bytes per launch (dram read + write, ncu, scaled x4)",
                         "peak_source": f"{peaks['source']} copy bandwidth",
                         "algorithmic_bytes": kv_bytes},
            "gpu_launches_per_step": 4}


def run_profile_case(args):
    """A small, self-ending case for `ncu`: few launches, at most ~1 GB on the device.
    prefill: the benchmark's own shape (100 MB of Q/K/V, larger than L2 together with the 67 MB
    output), 1 warm-up + 2 launches of the step kernel. decode: the decode workload at a
    quarter of the cached length (65536 tokens, 1 GB of K/V), 1 warm-up + 2 steps.
    prefill-d128 / prefill-d256 / prefill-d256-pair: the step kernel's other head_dims (and its
    cluster-pair form) on B1 H8 S16384 causal (0.4 GB on the device). prefill-gqa /
    prefill-gqa-heads-fastest: B2 H32/kvH8 S32768 D128 causal in either block order."""
    import torch

    from ring_attention_b200 import api
    from ring_attention_b200._lib import SegMap
    torch.cuda.set_device(0)
    dev = torch.device("cuda", 0)
    g = torch.Generator(device=dev).manual_seed(42)
    if args.profile == "prefill-docs":
        # one query head per KV head, four documents: config 5's shard on one GPU (2.7 GB)
        B, H, S, D, doc = 1, 16, 131072, 128, 32768
        q, k, v = (torch.randn((B, H, S, D), generator=g, device=dev, dtype=torch.float16) for _ in range(3))
        out = torch.empty((B, H, S, D), device=dev)
        m = torch.empty((B, H, S), device=dev)
        l = torch.empty_like(m)
        one = SegMap.make([0], S)
        for _ in range(3):
            api.attention_step_ex(q, k, v, out, m, l, api.AttentionShape(B, H, S, S, D), one, one, 1,
                                  causal=True, fresh=True, finalize=True, doc_len=doc)
    elif args.profile.startswith("prefill-gqa"):
        # grouped KV heads, 512 query blocks per KV head: the shape class of config 3 at a quarter
        # of its length (2 GB on the device), in the kernel's default block order for it (all
        # query blocks of the heads of one KV head first) or with (batch, head) fastest
        B, H, kvH, S, D = 2, 32, 8, 32768, 128
        q = torch.randn((B, H, S, D), generator=g, device=dev, dtype=torch.float16)
        k, v = (torch.randn((B, kvH, S, D), generator=g, device=dev, dtype=torch.float16) for _ in range(2))
        out = torch.empty((B, H, S, D), device=dev)
        m = torch.empty((B, H, S), device=dev)
        l = torch.empty_like(m)
        one = SegMap.make([0], S)
        if args.profile.endswith("heads-fastest"):
            api.lib().ra_debug_set_block_order(0)
        for _ in range(3):
            api.attention_step_ex(q, k, v, out, m, l, api.AttentionShape(B, H, S, S, D, kvH), one, one, 1,
                                  causal=True, fresh=True, finalize=True)
        api.lib().ra_debug_set_block_order(-1)
    elif args.profile.startswith("prefill-d"):
        D = 128 if "128" in args.profile else 256
        B, H, S = 1, 8, 16384
        q, k, v = (torch.randn((B, H, S, D), generator=g, device=dev, dtype=torch.float16) for _ in range(3))
        out = torch.empty((B, H, S, D), device=dev)
        m = torch.empty((B, H, S), device=dev)
        l = torch.empty_like(m)
        one = SegMap.make([0], S)
        for _ in range(3):
            api.attention_step_ex(q, k, v, out, m, l, api.AttentionShape(B, H, S, S, D), one, one, 1,
                                  causal=True, fresh=True, finalize=True,
                                  cta_pair=args.profile.endswith("pair"))
    elif args.profile == "prefill":
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


def bench_ring_decode(api, torch, dist, dev, args, peaks, ring, rank, P):
    """The decode workload with the cache sharded over P ranks (262144 / P cached tokens each):
    every step appends on the round-robin owner, folds the local shard, all-gathers the
    partials and merges (ra_ring_decode_step). tokens/s counts the batch rows per step."""
    d = DECODE
    B, H, kvH, D, L = d["batch"], d["heads"], d["kv_heads"], d["head_dim"], d["prompt"]
    per = L // P
    n = max(args.steps, 10)
    g = torch.Generator(device=dev).manual_seed(7 + rank)
    cache = api.DeviceKVCache(B, kvH, per + n + 8, D, torch.float16)
    k0 = torch.randn((B, kvH, per, D), generator=g, device=dev, dtype=torch.float16)
    v0 = torch.randn((B, kvH, per, D), generator=g, device=dev, dtype=torch.float16)
    cache.copy_prefill(k0, v0, per)
    del k0, v0
    gq = torch.Generator(device=dev).manual_seed(99)  # the query is replicated: same seed on every rank
    q = torch.randn((B, H, 1, D), generator=gq, device=dev, dtype=torch.float16)
    kn = torch.randn((B, kvH, 1, D), generator=g, device=dev, dtype=torch.float16)
    vn = torch.randn((B, kvH, 1, D), generator=g, device=dev, dtype=torch.float16)
    out = torch.empty((B, H, 1, D), device=dev)
    lens = [per] * P
    stream = torch.cuda.current_stream()
    t = 0
    for _ in range(3):
        lens[t % P] += 1
        ring.decode_step(q, kn, vn, t % P, cache, lens, out)
        t += 1
    torch.cuda.synchronize()
    dist.barrier()
    ev = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(n)]
    for i in range(n):
        lens[t % P] += 1
        ev[i][0].record(stream)
        ring.decode_step(q, kn, vn, t % P, cache, lens, out)
        ev[i][1].record(stream)
        t += 1
    torch.cuda.synchronize()
    # one more step with the driver's own event timings: fold of the local shard / all-gather of the
    # partials / whole step (the reference's RingResult fields, src/ring_decode.cu:206-224)
    lens[t % P] += 1
    rt = ring.decode_step(q, kn, vn, t % P, cache, lens, out, timed=True)
    t += 1
    tt = torch.tensor([sum(a.elapsed_time(b) for a, b in ev) / n, rt.comp_ms, rt.comm_ms, rt.total_ms],
                      device=dev, dtype=torch.float64)
    dist.all_reduce(tt, op=dist.ReduceOp.MAX)
    ms, comp_ms, comm_ms, total_ms = (float(x) for x in tt)
    checked = check_decode_rows(torch, dist, dev, cache, lens, q, out, rank, P)
    kv_bytes = 2.0 * B * kvH * L * D * 2
    gbs = kv_bytes / (ms * 1e-3) / 1e9
    return {"workload": f"decode B4 H32 kvH8 D128 fp16, 262144 cached tokens sharded over {P} ranks (config 4)",
            "ms_per_step": ms, "tokens_per_s": B / (ms * 1e-3), "hbm_gbs": gbs, "hbm_gbs_per_gpu": gbs / P,
            "step": {"comp_ms": comp_ms, "comm_ms": comm_ms, "total_ms": total_ms,
                     "note": "one step, max over ranks: split-K fold of the local shard, all-gather of the "
                             "partials, whole step including the merge"},
            "checked_rows": checked,
            "roofline": {"bound": "hbm", "achieved": gbs / P, "peak": peaks["hbm_gbs"], "unit": "GB/s",
                         "frac": gbs / P / peaks["hbm_gbs"], "traffic": None,
                         "peak_source": f"{peaks['source']} copy bandwidth",
                         "note": "per GPU, whole step including the all-gather of partials and the merge"}}


def check_decode_rows(torch, dist, dev, cache, lens, q, out, rank, P):
    """Parity of the sharded decode at full size: the output row of query head 0 of every batch
    element against the CPU oracle over the cache rows of KV head 0 gathered from all ranks
    (decode is unmasked: every cached row is visible). Untimed."""
    import numpy as np

    import oracle
    kview, vview = cache.k_view(), cache.v_view()
    n_max = max(lens)
    worst = 0.0
    B = q.shape[0]
    for b in range(B):
        kh = torch.zeros((n_max, q.shape[3]), dtype=kview.dtype, device=dev)
        vh = torch.zeros_like(kh)
        kh[:lens[rank]] = kview[b, 0, :lens[rank]]
        vh[:lens[rank]] = vview[b, 0, :lens[rank]]
        ks = [torch.empty_like(kh) for _ in range(P)]
        vs = [torch.empty_like(vh) for _ in range(P)]
        dist.all_gather(ks, kh)
        dist.all_gather(vs, vh)
        kg = torch.cat([ks[r][:lens[r]] for r in range(P)]).float().cpu().numpy()
        vg = torch.cat([vs[r][:lens[r]] for r in range(P)]).float().cpu().numpy()
        want, _ = oracle.attention_row(q[b, 0, 0].float().cpu().numpy(), kg, vg)
        got = out[b, 0, 0].cpu().numpy()
        err = np.abs(got - want)
        assert np.all(err <= 1e-3 + 1e-3 * np.abs(want)), f"decode rank {rank} batch {b}: max err {err.max()}"
        worst = max(worst, float(err.max()))
    t = torch.tensor([worst], device=dev)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return {"rows_per_rank": B, "max_abs_err": float(t[0]), "tolerance": "atol=rtol=1e-3 vs CPU oracle"}


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--profile", default=None, choices=["prefill", "decode", "prefill-d128", "prefill-d256", "prefill-d256-pair", "prefill-gqa",
                             "prefill-gqa-heads-fastest", "prefill-docs"],
                    help="run a small self-ending case for ncu instead of the benchmark")
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="config2", choices=sorted(WORKLOADS),
                    help="prefill workload; config2 is the benchmark line, the others are for the tables")
    ap.add_argument("--schedule", default="auto", choices=["auto", "ring", "gather"],
                    help="how K/V shards travel at N>1: hop-by-hop ring, one all-gather, or by shard size")
    ap.add_argument("--no-decode", action="store_true")
    ap.add_argument("--no-extra", action="store_true",
                    help="skip the secondary workloads (config 5 and config 3 objects of the line)")
    ap.add_argument("--no-cpu", action="store_true")
    args = ap.parse_args()
    if args.profile:
        return run_profile_case(args)
    if args.impl == "reference":
        return run_reference_arm(args)
    return run_gpu_arm(args)


if __name__ == "__main__":
    sys.exit(main())
