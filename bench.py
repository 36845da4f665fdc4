#!/usr/bin/env python
"""Benchmark of the non-GEMM operator path: fused-op HBM GB/s on the Wan2.1-1.3B DiT-block chain.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--no-extras]

N > 1 is launched with torch.distributed.run, one rank per GPU (NCCL).

A step = one pass of the chain over ONE batch: both classifier-free-guidance branches of one DiT
block (9 fused launches over [2, 32760, 1536], FFN 8960; synthetic, seeded data).  The path
partitions by token rows and needs no collective: with N ranks the SAME batch is split into N
contiguous token ranges, one per rank ("scaling": "strong"), and `value` is the batch's algorithmic
bytes divided by the slowest rank's time.  Outside the timed region every rank also runs the whole
batch and checks that its shard's outputs are the whole batch's outputs on its rows, bit for bit.

One JSON line on stdout (rank 0):
  value      algorithmic GB/s with inputs resident in HBM, CUDA-event time, max over ranks
  e2e        the same step through the host-buffer entry points of the C ABI (pinned host inputs
             uploaded, results downloaded, inside the timed region)
  roofline   the dominant kernel (table-driven GELU-tanh) against the measured HBM copy peak; its launch duration comes
             from event pairs around that launch in a second pass of the same K steps
  cpu_baseline  the reference's host path on a bounded row sample, all host cores (N=1 only)
  spread     min / median / max over further K-step repetitions of the same timed region
  configs    (N=1) the other headline configurations: Wan2.2 step, Mochi block, VAE GroupNorm+SiLU
  reference_cuda  (N=1) the reference's own CUDA kernels on the same chain, for comparison
  sharded    (N>1) the Mochi block split by tokens, the H-sharded GroupNorm with its NCCL moments
             all-reduce (compute only / + NCCL gather / + peer stores), the sampler all-gather
  replicas   (N>1) every rank running the whole batch on its own (the weak-scaling figure)
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
    "head_dim": 128, "ffn": 8960, "hidden_dtype": "bf16", "launches_per_step": 9,
    "launches": "LN+modulate, RMS+RoPE(q,k as one launch), gated residual, LN affine, RMS(cross q, text k as one launch), "
                "residual add, LN+modulate, GELU-tanh, gated residual",
    "batching": "both CFG branches as one [2, 32760, 1536] batch, one modulation vector set per branch",
    "sharding": "N ranks: the same batch split into N contiguous token ranges, no collective on the data path",
    "l2": "every launch streams 0.2-1.2 GB of distinct tensors (> 126 MB L2) at N=1; no flush needed",
}
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
        timed regions); all samples if the window caught none."""
        if not self.proc:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.05)
        self.proc.terminate()
        inside = [l for t, l in self.lines if begin is not None and begin <= t <= end + 0.03]
        window = "timed region + its repetitions" if inside else "whole run"
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


def reference_cuda_arm():
    """The reference's own CUDA kernels (its cuda_backend.cu compiled for sm_100a into oracle/_ref) timed
    on the same chains, each configuration in a process of its own.  A comparison figure only."""
    from oracle import ref
    if not ref.available_cuda():
        return {"unavailable": "oracle/_ref/libvrhino_ref_cuda.so is not built"}
    out = {}
    for config in ("wan21", "wan22_sampler", "vae_gn", "mochi", "vae_layout"):
        try:
            proc = subprocess.run([sys.executable, "-m", "oracle.ref_timing", "--config", config], cwd=ROOT,
                                  capture_output=True, text=True, timeout=420)
            lines = [l for l in proc.stdout.splitlines() if l.startswith("{")]
            out[config] = json.loads(lines[-1]) if lines else {"error": (proc.stderr or proc.stdout)[-300:]}
        except Exception as exc:
            out[config] = {"error": str(exc)[:200]}
    return out


def run_reference(args, rank, world):
    """The reference arm: the reference's CPU implementation of the path on the host cores."""
    if rank != 0:
        return
    value, sec, info = cpu_arm(min(args.steps, 20), min(args.warmup, 2))
    line = {
        "impl": "reference", "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": args.gpus, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": sec * 1e3, "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
        "dtype": "f32" if info["kind"] == "reference" else "bf16", "data": "synthetic", "config": WORKLOAD,
        "cpu_baseline": {"value": value, "unit": UNIT, **info},
        "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=200)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--e2e-steps", type=int, default=2)
    ap.add_argument("--repeats", type=int, default=5, help="further K-step repetitions reported as `spread`")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-extras", action="store_true", help="headline, e2e and roofline only")
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
    from vrhino_b200 import _lib, bench_extras, ops, workloads

    torch.cuda.set_device(local)
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    lib = _lib.load()
    numa = bench_extras.bind_to_gpu_numa_node(local) if world > 1 else None      # before any pinned buffer is touched
    be = ops.B200Backend(device=f"cuda:{local}")
    peak, peak_kind = measured_hbm_peak()

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

    def timed(fns, steps, per_launch=None):
        """K steps of `fns` bracketed by barrier + synchronize, CUDA events on the launching stream;
        returns ms per step, max over ranks.  per_launch: {index: []} collects event pairs of those launches."""
        barrier()
        start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        start.record()
        for _ in range(steps):
            for i, fn in enumerate(fns):
                if per_launch is not None and i in per_launch:
                    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                    a.record(); fn(); b.record()
                    per_launch[i].append((a, b))
                else:
                    fn()
        stop.record()
        barrier()
        return max_over_ranks(start.elapsed_time(stop)) / steps

    # ---- the batch: identical on every rank (same seed); rank r works on its token rows ----------
    whole = workloads.WanBlock(be, seed=0, batch=2)
    work = whole if world == 1 else whole.token_shard(rank, world)
    step_bytes = sum(l.bytes for l in whole.launches(pair_qk=True))          # the whole batch, whatever N
    python_launches = work.launches(pair_qk=True)
    for l in python_launches:
        l.fn()                                                   # allocates the outputs
    torch.cuda.synchronize()
    launches = workloads.compile_launches(python_launches)       # recorded C-ABI calls: no Python per operator
    fns = [l.fn for l in launches]
    dominant_index = next(i for i, l in enumerate(launches) if l.name.startswith("H "))

    shard_check = None
    if world > 1:
        shard_check = bench_extras.check_shard_against_whole(whole, work, dist)

    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
        deadline = time.monotonic() + 1.0          # its start-up (process spawn, NVML init) stays outside the timed region
        while not sampler.lines and time.monotonic() < deadline:
            time.sleep(0.01)
    for _ in range(args.warmup):
        for fn in fns:
            fn()
    launches_before = lib.vrb_launch_count()
    wall_begin = time.monotonic()
    ms_per_step = timed(fns, args.steps)
    gpu_launches = lib.vrb_launch_count() - launches_before
    # the dominant kernel's launch duration: the same K steps once more with an event pair around that launch (kept out
    # of the headline pass: an event record between two launches takes away their overlap and costs host time per step)
    dom_events = {dominant_index: []}
    timed(fns, args.steps, dom_events)
    repeats = [timed(fns, args.steps) for _ in range(max(args.repeats, 0))]
    wall_end = time.monotonic()
    clocks = sampler.stop(wall_begin, wall_end) if rank == 0 else None
    value = step_bytes / (ms_per_step * 1e-3) / 1e9
    dom_ms = statistics.mean(a.elapsed_time(b) for a, b in dom_events[dominant_index])
    dom_launch = launches[dominant_index]
    dom_elements = work.ffn_hidden.numel()
    achieved = dom_launch.bytes / (dom_ms * 1e-3) / 1e9
    spread = None
    if repeats:
        spread = {"ms_per_step_min": min(repeats), "ms_per_step_median": statistics.median(repeats), "ms_per_step_max": max(repeats),
                  "repetitions": len(repeats), "steps_each": args.steps}

    # ---- the same step replayed from a CUDA graph ---------------------------------------------------
    graph_obj = None
    try:
        side = torch.cuda.Stream()
        g = torch.cuda.CUDAGraph()
        with torch.cuda.stream(side):
            with torch.cuda.graph(g, stream=side):
                for l in python_launches:
                    l.fn()
        for _ in range(3):
            g.replay()
        graph_ms = timed([g.replay], args.steps)
        graph_obj = {"ms_per_step": graph_ms, "us_per_dit_block": graph_ms * 1e3, "value": step_bytes / (graph_ms * 1e-3) / 1e9,
                     "unit": UNIT, "kernels_per_replay": len(launches)}
        del g
    except Exception as exc:  # an extra measurement, never the headline
        graph_obj = {"error": str(exc)[:200]}

    # ---- plain launches (no programmatic dependent launch), for comparison -------------------------
    plain_obj = None
    try:
        previous = lib.vrb_set_launch_overlap(0)
        for fn in fns:
            fn()
        plain_ms = timed(fns, args.steps)
        lib.vrb_set_launch_overlap(previous)
        plain_obj = {"ms_per_step": plain_ms, "value": step_bytes / (plain_ms * 1e-3) / 1e9, "unit": UNIT}
    except Exception as exc:
        plain_obj = {"error": str(exc)[:200]}

    extras = {}
    if not args.no_extras:
        extras = bench_extras.run(be, whole, work, world, rank, dist, timed, barrier, max_over_ranks, peak, args)

    # ---- end-to-end arm: the same step from host buffers through the C ABI ---------------------------
    for blk in (whole, work):
        blk.out.clear()
    del launches, fns, python_launches
    torch.cuda.empty_cache()
    e2e = workloads.WanBlockHost(work)
    del whole
    torch.cuda.empty_cache()
    e2e.step()   # first call sizes the staging buffers
    barrier()
    t0 = time.perf_counter()
    for _ in range(args.e2e_steps):
        e2e.step()
    torch.cuda.synchronize()
    e2e_ms = max_over_ranks((time.perf_counter() - t0) * 1e3) / args.e2e_steps

    def total_over_ranks(n: int) -> int:
        if world == 1:
            return n
        t = torch.tensor([n], device="cuda", dtype=torch.int64)
        dist.all_reduce(t)
        return int(t.item())

    e2e_obj = {"value": step_bytes / (e2e_ms * 1e-3) / 1e9, "unit": UNIT,
               "h2d_bytes_per_step": total_over_ranks(e2e.h2d_bytes), "d2h_bytes_per_step": total_over_ranks(e2e.d2h_bytes),
               "ms_per_step": e2e_ms,
               "note": "the same step's operators (both CFG branches, 22 host-buffer calls; each rank its token rows), pinned host buffers, "
                       "3-stream upload/kernel/download pipeline per call"}
    if numa is not None:
        e2e_obj["numa"] = numa     # rank 0's GPU node and how many CPUs the rank was bound to
    lib.vrb_host_release()

    cpu = None
    if rank == 0 and world == 1 and not args.no_cpu_baseline:
        v, _, info = cpu_arm(steps=3, warmup=1)
        cpu = {"value": v, "unit": UNIT, **info}
    if rank == 0 and world == 1 and not args.no_extras:
        del e2e
        torch.cuda.empty_cache()
        extras["reference_cuda"] = reference_cuda_arm()

    if rank == 0:
        line = {
            "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "bf16",
            "data": "synthetic", "config": WORKLOAD,
            "us_per_dit_block": ms_per_step * 1e3,
            "pct_of_nominal_8tbs": 100.0 * value / world / NOMINAL_HBM_GBS,
            "pct_of_measured_copy_peak": 100.0 * value / world / peak,
            "roofline": {"bound": "hbm", "kernel": f"unary_lut_kernel<gelu_tanh> on {list(work.ffn_hidden.shape)} bf16", "achieved": achieved,
                         "peak": peak, "peak_kind": peak_kind, "unit": "GB/s", "frac": achieved / peak,
                         "traffic": int(workloads.WanBlock.GELU_DRAM_BYTES_PER_ELEMENT * dom_elements),
                         "algorithmic_bytes": dom_launch.bytes, "ms_per_launch": dom_ms},
            "e2e": e2e_obj, "gpu_launches": int(gpu_launches), "clocks": clocks,
            "launch_path": "C-ABI calls recorded once and replayed (no Python per operator), programmatic dependent launch on",
        }
        for key, obj in (("spread", spread), ("cuda_graph_replay", graph_obj), ("plain_launches", plain_obj),
                         ("shard_check", shard_check), ("cpu_baseline", cpu)):
            if obj:
                line[key] = obj
        line.update(extras)
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
