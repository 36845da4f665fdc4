#!/usr/bin/env python
"""Benchmark of the non-GEMM operator path: fused-op HBM GB/s on the Wan2.1-1.3B DiT-block chain.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

N > 1 is launched with torch.distributed.run, one rank per GPU (NCCL); the driver of this
repository's round runs `python -m torch.distributed.run --nnodes=1 --nproc-per-node N ...`.

A step = one pass of the chain over one batch: both classifier-free-guidance branches of one
DiT block (2 x 11 fused launches, 32760 tokens x 1536, FFN 8960; synthetic data).  The path
partitions by token rows and needs no collective, so ranks work on independent batches
(weak scaling) and `value` is the bytes all ranks moved divided by the slowest rank's time.
`strong` additionally reports the same single batch split by tokens over the N ranks.

One JSON line on stdout (rank 0):
  value      algorithmic GB/s with inputs resident in HBM, CUDA-event time, max over ranks
  e2e        the same metric through the host-buffer entry points of the C ABI (pinned host
             inputs uploaded, results downloaded, inside the timed region)
  roofline   the dominant kernel (table-driven GELU-tanh) against the measured HBM copy peak
  cpu_baseline  the CPU oracle's chain on a bounded row sample, all host cores (N=1 only)
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
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

METRIC = "fused-op HBM GB/s (Wan2.1-1.3B DiT-block non-GEMM chain)"
UNIT = "GB/s"
WORKLOAD = {
    "workload": "wan2.1-1.3b dit block non-gemm chain, batch 2 (cfg)", "tokens": 32760, "dim": 1536, "heads": 12,
    "head_dim": 128, "ffn": 8960, "hidden_dtype": "bf16", "launches_per_step": 11,
    "batching": "both CFG branches as one [2, 32760, 1536] batch, one modulation vector set per branch",
    "l2": "every launch streams 0.2-1.2 GB of distinct tensors (> 126 MB L2), no flush needed",
}
# DRAM bytes (read + write) of one launch of the dominant kernel, unary_lut_kernel<2> on
# [2, 32760, 8960] bf16: twice the figure the ncu capture of one [32760, 8960] branch gives
# (profiles/gelu_tanh_lut_wan21.md); the kernel streams, so its traffic grows with the element count
DOMINANT_TRAFFIC_BYTES = 2 * 1_125_900_000
NOMINAL_HBM_GBS = 8000.0


def measured_hbm_peak():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    try:
        with open(path) as fh:
            return float(json.load(fh)["hbm_gbs"]), "measured"
    except Exception:
        return 6650.0, "fallback"


class ClockSampler:
    """nvidia-smi samples of SM clock / throttle reasons while the timed region runs."""
    FIELDS = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index, self.proc, self.lines = index, None, []

    def start(self):
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", str(self.index), f"--query-gpu={self.FIELDS}",
                                          "--format=csv,noheader,nounits", "-lms", "20"],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            threading.Thread(target=self._pump, daemon=True).start()
        except OSError:
            self.proc = None

    def _pump(self):
        for line in self.proc.stdout:
            self.lines.append((time.monotonic(), line.strip()))

    def stop(self, begin=None, end=None):
        """Summary of the samples taken between `begin` and `end` (time.monotonic() values of the
        timed region); all samples if the window caught none."""
        if not self.proc:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.05)
        self.proc.terminate()
        inside = [l for t, l in self.lines if begin is not None and begin <= t <= end + 0.03]
        window = "timed region" if inside else "whole run"
        sm, smax, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for line in (inside or [l for _, l in self.lines]):
            parts = [p.strip() for p in line.split(",")]
            if len(parts) < 6:
                continue
            try:
                sm.append(float(parts[0])); smax.append(float(parts[1]))
            except ValueError:
                continue
            for name, flag in zip(names, parts[2:6]):
                if flag.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(smax) if smax else None,
                "samples": len(sm), "window": window, "reasons": sorted(reasons)}


def cpu_arm(steps: int, warmup: int):
    """Times the CPU arm on a bounded sample of the step's 65520 token rows (the chain is
    row-independent).  Preferred: the reference's OWN host path (oracle/_ref/libvrhino_ref_host.so,
    its F32 host backend driven through its helper seams, rows spread over all host threads);
    otherwise the CPU oracle's restatement with OpenMP.  Returns (GB/s, seconds/step, description)."""
    from oracle import ref
    threads = os.cpu_count() or 1
    if ref.available_host():
        tokens = 1024
        host = ref.RefHost()
        for _ in range(max(warmup, 0)):
            host.wan_chain_seconds(tokens=tokens, threads=threads, steps=1)
        sec, nbytes = host.wan_chain_seconds(tokens=tokens, threads=threads, steps=max(steps, 1))
        return nbytes / sec / 1e9, sec, {
            "cores": threads, "kind": "reference",
            "sample": f"{tokens} of 65520 token rows per step; the reference's host backend (F32, family_test::Backend) "
                      f"through its own modulate/attention_norm/rope/residual helpers, {threads} threads"}
    from oracle import cpu_chain
    tokens = 2048
    sec, nbytes, threads = cpu_chain.time_chain(tokens, steps=max(steps, 1), warmup=max(warmup, 1))
    return nbytes / sec / 1e9, sec, {
        "cores": threads, "kind": "port",
        "sample": f"{tokens} of 65520 token rows per step; unfused operator chain of the CPU oracle, {threads} OpenMP threads"}


def run_reference(args, rank, world):
    """The reference arm: the reference's CPU implementation of the path on the host cores."""
    if rank != 0:
        return
    value, sec, info = cpu_arm(min(args.steps, 20), min(args.warmup, 2))
    line = {
        "impl": "reference", "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": args.gpus, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": sec * 1e3, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "f32" if info["kind"] == "reference" else "bf16", "data": "synthetic", "config": WORKLOAD,
        "cpu_baseline": {"value": value, "unit": UNIT, **info},
        "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=400)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--e2e-steps", type=int, default=2)
    ap.add_argument("--no-cpu-baseline", action="store_true")
    args = ap.parse_args()
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if args.impl == "reference":
        run_reference(args, rank, world)
        return
    args.warmup = max(args.warmup, 3)

    import torch
    import torch.distributed as dist
    from vrhino_b200 import _lib, ops, workloads

    torch.cuda.set_device(local)
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    lib = _lib.load()
    be = ops.B200Backend(device=f"cuda:{local}")

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def max_over_ranks(ms: float) -> float:
        if world == 1:
            return ms
        t = torch.tensor([ms], device="cuda", dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    # ---- resident arm: both CFG branches of one block -------------------------------------------
    branches = [workloads.WanBlock(be, seed=1000 * rank, batch=2)]
    launches = [l for blk in branches for l in blk.launches()]
    step_bytes = sum(l.bytes for l in launches)
    dominant = [l for l in launches if l.name.startswith("H ")]
    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
    for _ in range(args.warmup):
        for l in launches:
            l.fn()
    barrier()
    launches_before = lib.vrb_launch_count()
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    dom_events = []
    barrier()
    wall_begin = time.monotonic()
    start.record()
    for _ in range(args.steps):
        for l in launches:
            if l in dominant:
                a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                a.record(); l.fn(); b.record()
                dom_events.append((a, b))
            else:
                l.fn()
    stop.record()
    barrier()
    wall_end = time.monotonic()
    total_ms = max_over_ranks(start.elapsed_time(stop))
    gpu_launches = lib.vrb_launch_count() - launches_before
    clocks = sampler.stop(wall_begin, wall_end) if rank == 0 else None
    ms_per_step = total_ms / args.steps
    value = world * step_bytes / (ms_per_step * 1e-3) / 1e9
    dom_ms = statistics.mean(a.elapsed_time(b) for a, b in dom_events)
    dom_bytes = dominant[0].bytes
    peak, peak_kind = measured_hbm_peak()
    achieved = dom_bytes / (dom_ms * 1e-3) / 1e9

    # ---- the same step replayed from a CUDA graph (no host launch latency between kernels) ------
    graph_obj = None
    try:
        side = torch.cuda.Stream()
        g = torch.cuda.CUDAGraph()
        with torch.cuda.stream(side):
            with torch.cuda.graph(g, stream=side):
                for l in launches:
                    l.fn()
        barrier()
        g0, g1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        for _ in range(3):
            g.replay()
        barrier()
        g0.record()
        for _ in range(args.steps):
            g.replay()
        g1.record()
        barrier()
        graph_ms = max_over_ranks(g0.elapsed_time(g1)) / args.steps
        graph_obj = {"ms_per_step": graph_ms, "value": world * step_bytes / (graph_ms * 1e-3) / 1e9, "unit": UNIT,
                     "kernels_per_replay": len(launches)}
        del g
    except Exception as exc:  # graph capture is an extra measurement, never the headline
        graph_obj = {"error": str(exc)[:200]}

    # ---- the same block with each residual update merged into the LayerNorm that follows it ----
    # (9 launches; the merged launches read residual + branch and write stream + normalised output,
    # 4 passes where the two launches they replace make 5, so this form moves fewer bytes: it is
    # reported in microseconds per block, and in GB/s of the bytes it actually has to move)
    fused_obj = None
    try:
        fused = [l for blk in branches for l in blk.launches(fuse_residual_norm=True)]
        for _ in range(args.warmup):
            for l in fused:
                l.fn()
        barrier()
        f0, f1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        f0.record()
        for _ in range(args.steps):
            for l in fused:
                l.fn()
        f1.record()
        barrier()
        fused_ms = max_over_ranks(f0.elapsed_time(f1)) / args.steps
        fused_bytes = sum(l.bytes for l in fused)
        fused_obj = {"ms_per_step": fused_ms, "us_per_dit_block": fused_ms * 1e3, "launches_per_step": len(fused),
                     "bytes_per_step": fused_bytes, "value": world * fused_bytes / (fused_ms * 1e-3) / 1e9, "unit": UNIT}
        del fused
    except Exception as exc:  # an extra measurement, never the headline
        fused_obj = {"error": str(exc)[:200]}

    # ---- strong scaling: one batch split by tokens over the ranks ------------------------------
    strong = None
    if world > 1:
        tokens = 32760 // world
        shard = [workloads.WanBlock(be, tokens=tokens, grid=(1, 1, tokens), seed=7, batch=2)]
        sl = [l for blk in shard for l in blk.launches()]
        for _ in range(args.warmup):
            for l in sl:
                l.fn()
        barrier()
        s0, s1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s0.record()
        for _ in range(args.steps):
            for l in sl:
                l.fn()
        s1.record()
        barrier()
        strong_ms = max_over_ranks(s0.elapsed_time(s1)) / args.steps
        strong = {"us_per_dit_block": strong_ms * 1e3, "tokens_per_rank": tokens,
                  "value": world * sum(l.bytes for l in sl) / (strong_ms * 1e-3) / 1e9, "unit": UNIT}
        try:   # small per-rank kernels are launch-bound: the same sharded step from a CUDA graph
            side = torch.cuda.Stream()
            g = torch.cuda.CUDAGraph()
            with torch.cuda.stream(side):
                with torch.cuda.graph(g, stream=side):
                    for l in sl:
                        l.fn()
            for _ in range(3):
                g.replay()
            barrier()
            g0, g1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            g0.record()
            for _ in range(args.steps):
                g.replay()
            g1.record()
            barrier()
            strong["us_per_dit_block_cuda_graph"] = max_over_ranks(g0.elapsed_time(g1)) / args.steps * 1e3
            del g
        except Exception as exc:
            strong["cuda_graph_error"] = str(exc)[:200]
        del shard, sl
        torch.cuda.empty_cache()
    del branches, launches
    torch.cuda.empty_cache()
    branches = [workloads.WanBlock(be, seed=1000 * rank)]
    # ---- end-to-end arm: host buffers through the C ABI ------------------------------------------
    e2e = workloads.WanBlockHost(branches[0])
    e2e.step()   # first call sizes the staging buffers
    barrier()
    t0 = time.perf_counter()
    for _ in range(args.e2e_steps):
        e2e.step()
    torch.cuda.synchronize()
    e2e_ms = max_over_ranks((time.perf_counter() - t0) * 1e3) / args.e2e_steps
    # one branch per e2e step: half the bytes of a resident step
    e2e_value = world * e2e.bytes_per_step / (e2e_ms * 1e-3) / 1e9
    e2e_obj = {"value": e2e_value, "unit": UNIT, "h2d_bytes_per_step": e2e.h2d_bytes, "d2h_bytes_per_step": e2e.d2h_bytes,
               "ms_per_step": e2e_ms, "note": "one CFG branch (11 launches) per e2e step, pinned host buffers, 3-stream pipeline"}
    lib.vrb_host_release()

    cpu = None
    if rank == 0 and world == 1 and not args.no_cpu_baseline:
        v, _, info = cpu_arm(steps=3, warmup=1)
        cpu = {"value": v, "unit": UNIT, **info}

    if rank == 0:
        line = {
            "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16",
            "data": "synthetic", "config": WORKLOAD,
            "us_per_dit_block": ms_per_step * 1e3,
            "pct_of_nominal_8tbs": 100.0 * value / world / NOMINAL_HBM_GBS,
            "pct_of_measured_copy_peak": 100.0 * value / world / peak,
            "roofline": {"bound": "hbm", "kernel": "unary_lut_kernel<gelu_tanh> on [2, 32760, 8960] bf16", "achieved": achieved,
                         "peak": peak, "peak_kind": peak_kind, "unit": "GB/s", "frac": achieved / peak,
                         "traffic": DOMINANT_TRAFFIC_BYTES, "algorithmic_bytes": dom_bytes, "ms_per_launch": dom_ms},
            "e2e": e2e_obj, "gpu_launches": int(gpu_launches), "clocks": clocks,
        }
        if graph_obj:
            line["cuda_graph_replay"] = graph_obj
        if fused_obj:
            line["residual_norm_merged"] = fused_obj
        if strong:
            line["strong"] = strong
        if cpu:
            line["cpu_baseline"] = cpu
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
