"""Measurements bench.py reports beside its headline: the other headline configurations on one
GPU, and the multi-GPU forms (token shards, the H-sharded GroupNorm with its statistics
all-reduce and output gather, the sampler's latent all-gather) on N GPUs.  Every figure is a
CUDA-event time on the launching stream, max over ranks; nothing here is inside the headline's
timed region.  Each section is guarded: a failure becomes {"error": ...} in that section only.
"""
from __future__ import annotations

import torch

from . import ops, sharded, workloads

BF16, F32 = torch.bfloat16, torch.float32


def _bits(t):
    return t.contiguous().view(torch.int16 if t.dtype == BF16 else torch.int32)


def check_shard_against_whole(whole, shard, dist):
    """Runs the whole batch on this rank and compares the shard's outputs with the whole batch's
    outputs on the shard's rows, element for element; then checks across ranks that every rank's
    whole-batch outputs are the same tensors (checksums), so the N shards together ARE the N=1
    result.  Returns a dict for the bench line; all ranks call it."""
    for l in whole.launches(pair_qk=True):
        l.fn()
    torch.cuda.synchronize()
    (r0, r1), (t0, t1) = shard.token_rows, shard.text_rows
    mismatched = 0
    sums = []
    for key in sorted(whole.out):
        full = whole.out[key]
        want = full[:, t0:t1] if key == "Ek" else full[:, r0:r1]
        mismatched += int((_bits(want) != _bits(shard.out[key])).sum())
        sums.append(_bits(full).to(torch.int64).sum())
    local = torch.stack(sums + [torch.tensor(mismatched, device=sums[0].device, dtype=torch.int64)])
    gathered = [torch.empty_like(local) for _ in range(dist.get_world_size())]
    dist.all_gather(gathered, local)
    table = torch.stack(gathered).cpu()
    whole.out.clear()
    torch.cuda.empty_cache()
    return {"outputs_compared": len(sums), "mismatched_elements": int(table[:, -1].sum()),
            "whole_batch_checksums_agree_across_ranks": bool((table[:, :-1] == table[0, :-1]).all()),
            "how": "every rank: whole batch vs its token shard, bit for bit; checksums of the whole-batch outputs all-gathered"}


def _launch_table(launches, steps, warmup, peak):
    total, per = workloads.time_launches(launches, steps=steps, warmup=warmup)
    rows = [{"launch": l.name, "us": per[l.name] * 1e3, "gbs": l.bytes / per[l.name] / 1e6, "algorithmic_mb": l.bytes / 1e6,
             "frac_of_measured_peak": l.bytes / per[l.name] / 1e6 / peak} for l in launches]
    nbytes = sum(l.bytes for l in launches)
    return {"us": total * 1e3, "gbs": nbytes / total / 1e6, "algorithmic_mb": nbytes / 1e6,
            "frac_of_measured_peak": nbytes / total / 1e6 / peak, "launches": rows,
            "timing": "whole list back to back; each launch back to back with itself (tensors under 126 MB stay in L2 then)"}


def single_gpu_configs(be, peak, steps=10, warmup=2):
    """Headline configurations 3, 4 and 5 at full size on one GPU, and the VAE / layout kernels: per-launch device times."""
    out = {}
    builders = {
        "wan22_step (config 3: D=5120 block chain, FP8 dequant 5120x13824, CFG + Euler on the F32 latent)":
            lambda: workloads.Wan22Step(be, tokens=32760).launches(pair_qk=True),
        "mochi_block (config 4: 44520 tokens x 3072, SwiGLU 8192)": lambda: workloads.MochiBlock(be, tokens=44520).launches(),
        "mochi_block, fewest launches (q+k as one launch, residual update + next pre-norm + tanh(gate) as one)":
            lambda: workloads.MochiBlock(be, tokens=44520).launches(merge_tail=True),
        "ltx_block (LTX-Video block chain, both CFG branches: [2, 6144, 2048], 32 heads x 64, FFN 8192, per-batch RoPE tables [2, 6144, 2048])":
            lambda: workloads.LtxBlock(be).launches(),
        "vae_group_norm_silu (config 5: [1,256,28,240,424] bf16, 32 groups)": lambda: workloads.VaeGroupNorm(be).launches(),
        "ltx_vae_pixel_norm ([1,128,16,256,384] bf16: pixel_norm, + modulate + SiLU -> F32 / bf16)":
            lambda: workloads.LtxVaeNorm(be, shape=(1, 128, 16, 256, 384)).launches(),
        "wan_vae_rms_channel ([1,192,4,240,416] bf16, + SiLU)": lambda: workloads.WanVaeRmsChannel(be).launches(),
        "layout_operators ([1,128,8,256,384] feature map, [1,1536,32760] patch embedding, bf16)": lambda: workloads.LayoutOps(be).launches(),
    }
    for name, build in builders.items():
        try:
            launches = build()
            out[name] = _launch_table(launches, steps, warmup, peak)
            del launches
        except Exception as exc:
            out[name] = {"error": str(exc)[:200]}
        torch.cuda.empty_cache()
    return out


def _time_steps(step, steps, warmup, barrier, max_over_ranks):
    for _ in range(warmup):
        step()
    barrier()
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a.record()
    for _ in range(steps):
        step()
    b.record()
    barrier()
    return max_over_ranks(a.elapsed_time(b)) / steps


def sharded_forms(be, world, rank, dist, barrier, max_over_ranks, peak, steps=10, warmup=3):
    """The multi-GPU forms on `world` ranks.  Aggregate GB/s = whole-problem algorithmic bytes / slowest rank."""
    out = {}
    # ---- config 4: the Mochi visual stream split by tokens, no collective ----
    try:
        tokens = 44520
        t0, t1 = sharded.token_range(tokens, rank, world)
        blk = workloads.MochiBlock(be, tokens=t1 - t0, seed=100 + rank)
        entry = {"tokens_per_rank": t1 - t0, "collectives": "none (row-independent operators)"}
        for label, merge in (("five_launches", False), ("three_launches", True)):
            launches = blk.launches(merge_tail=True) if merge else blk.launches()
            for l in launches:
                l.fn()
            compiled = workloads.compile_launches(launches)
            ms = _time_steps(lambda: [l.fn() for l in compiled], steps, warmup, barrier, max_over_ranks)
            whole_bytes = sum(l.bytes for l in launches) * tokens / (t1 - t0)
            entry[label] = {"us": ms * 1e3, "aggregate_gbs": whole_bytes / ms / 1e6}
            del launches, compiled
        out["mochi_block_token_sharded"] = entry
        del blk
    except Exception as exc:
        out["mochi_block_token_sharded"] = {"error": str(exc)[:200]}
    torch.cuda.empty_cache()

    # ---- config 5: GroupNorm(32) + SiLU on [1,256,28,240,424] bf16 split along H ----
    try:
        frames, height, width, channels = 28, 240, 424, 256
        h0, h1 = sharded.h_range(height, rank, world)
        g = torch.Generator(device="cuda").manual_seed(200 + rank)
        x = (torch.randn((1, channels, frames, h1 - h0, width), device="cuda", generator=g) * 2.0).to(BF16)
        gamma, beta = torch.ones(channels, device="cuda"), torch.zeros(channels, device="cuda")
        pieces = sharded.KernelMoments(be)
        full_bytes = channels * frames * height * width * 6
        entry = {"h_rows_per_rank": h1 - h0, "statistics": "NCCL all-reduce of [32, 3] doubles (+ broadcast of 32 shift values)"}
        compute = _time_steps(lambda: sharded.sharded_group_norm(pieces, x, 32, gamma, beta, 1e-6, True), steps, warmup, barrier, max_over_ranks)
        entry["compute_and_moments_allreduce_us"] = compute * 1e3
        entry["compute_aggregate_gbs"] = full_bytes / compute / 1e6
        gather = _time_steps(lambda: sharded.sharded_group_norm(pieces, x, 32, gamma, beta, 1e-6, True, None, 3), steps, warmup, barrier, max_over_ranks)
        entry["with_nccl_all_gather_and_placement_us"] = gather * 1e3
        try:
            peer = sharded.PeerOutput((1, channels, frames, height, width), BF16, torch.device("cuda", torch.cuda.current_device()))
            fused = _time_steps(lambda: sharded.sharded_group_norm(pieces, x, 32, gamma, beta, 1e-6, True, None, None, peer, h0),
                                steps, warmup, barrier, max_over_ranks)
            entry["with_peer_stores_us"] = fused * 1e3
            ingress = channels * frames * (height - (h1 - h0)) * width * 2
            entry["nvlink_ingress_bytes_per_gpu"] = ingress
            entry["peer_store_fraction_of_770gbs_link"] = (ingress / 770e9) / (fused * 1e-3) if ingress else None
            entry["limiter"] = "NVLink ingress: every GPU receives the other ranks' slices of the full output"
            del peer
        except Exception as exc:
            entry["with_peer_stores_error"] = str(exc)[:200]
        out["group_norm_silu_h_sharded"] = entry
        del x, pieces
    except Exception as exc:
        out["group_norm_silu_h_sharded"] = {"error": str(exc)[:200]}
    torch.cuda.empty_cache()

    # ---- sampler: cfg_combine + euler_update on flat ranges, then the latent all-gather ----
    try:
        g = torch.Generator(device="cuda").manual_seed(300)
        latent, uncond, cond = (torch.randn((1, 16, 21, 60, 104), device="cuda", generator=g) for _ in range(3))
        be32 = ops.B200Backend(execution_dtype=F32, device=str(be.device))
        pol = ops.Policy.fp32()
        ms = _time_steps(lambda: sharded.sharded_cfg_euler(be32, ops, pol, latent, uncond, cond, 5.0, 0.02), steps, warmup, barrier, max_over_ranks)
        whole = ops.fused_cfg_euler(be32, pol, latent, uncond, cond, 5.0, 0.02, True)
        got = sharded.sharded_cfg_euler(be32, ops, pol, latent, uncond, cond, 5.0, 0.02)
        out["cfg_euler_flat_sharded"] = {"us": ms * 1e3, "collectives": "NCCL all-gather of the F32 latent (8.4 MB)",
                                         "equals_single_gpu_result": bool(torch.equal(whole.view(torch.int32), got.view(torch.int32)))}
    except Exception as exc:
        out["cfg_euler_flat_sharded"] = {"error": str(exc)[:200]}
    torch.cuda.empty_cache()
    return out


def bind_to_gpu_numa_node(device_index: int):
    """Keep this rank's threads (and so the first touch of its pinned staging buffers) on the NUMA node its GPU hangs
    off: with one rank per GPU the host side of `e2e` is otherwise placed wherever the launcher started the process.
    Reads sysfs only; returns what it found and did ({"node": -1} = the platform reports no node, nothing bound)."""
    import os
    found = {"node": -1, "cpus_bound": 0}
    try:
        bus = torch.cuda.get_device_properties(device_index)
        address = f"{bus.pci_domain_id:04x}:{bus.pci_bus_id:02x}:{bus.pci_device_id:02x}.0"
        with open(f"/sys/bus/pci/devices/{address}/numa_node") as fh:
            node = int(fh.read().strip())
        found["node"] = node
        if node < 0:
            return found
        with open(f"/sys/devices/system/node/node{node}/cpulist") as fh:
            cpus = set()
            for part in fh.read().strip().split(","):
                lo, _, hi = part.partition("-")
                cpus.update(range(int(lo), int(hi or lo) + 1))
        allowed = cpus & os.sched_getaffinity(0)
        if allowed:
            os.sched_setaffinity(0, allowed)
            found["cpus_bound"] = len(allowed)
    except (OSError, ValueError, AttributeError):
        pass
    return found


def pcie_probe(world, barrier, max_over_ranks, nbytes=256 << 20, steps=4):
    """Host<->device copy rates with every rank copying at once (pinned buffers): what bounds `e2e`."""
    host_a, host_b = torch.empty(nbytes, dtype=torch.uint8).pin_memory(), torch.empty(nbytes, dtype=torch.uint8).pin_memory()
    dev_a, dev_b = torch.empty(nbytes, dtype=torch.uint8, device="cuda"), torch.empty(nbytes, dtype=torch.uint8, device="cuda")
    up, down = torch.cuda.Stream(), torch.cuda.Stream()

    def h2d():
        dev_a.copy_(host_a, non_blocking=True)

    def d2h():
        host_b.copy_(dev_b, non_blocking=True)

    def both():
        with torch.cuda.stream(up):
            dev_a.copy_(host_a, non_blocking=True)
        with torch.cuda.stream(down):
            host_b.copy_(dev_b, non_blocking=True)

    out = {}
    for name, fn, factor in (("h2d", h2d, 1), ("d2h", d2h, 1)):
        ms = _time_steps(fn, steps, 1, barrier, max_over_ranks)
        out[f"{name}_gbs_per_rank"] = factor * nbytes / ms / 1e6
    import time
    barrier()
    t0 = time.perf_counter()
    for _ in range(steps):
        both()
    torch.cuda.synchronize()
    ms = max_over_ranks((time.perf_counter() - t0) * 1e3) / steps
    out["both_directions_gbs_per_rank_each_way"] = nbytes / ms / 1e6
    out["ranks_copying_at_once"] = world
    return out


def run(be, whole, work, world, rank, dist, timed, barrier, max_over_ranks, peak, args):
    """All extras for this rank count; returns the keys to merge into the bench line."""
    out = {}
    # the residual updates merged into the LayerNorm that follows (9 launches): fewer bytes to move
    try:
        merged = work.launches(fuse_residual_norm=True, pair_qk=True)
        for l in merged:
            l.fn()
        compiled = workloads.compile_launches(merged)
        ms = timed([l.fn for l in compiled], args.steps)
        nbytes = sum(l.bytes for l in whole.launches(fuse_residual_norm=True, pair_qk=True))
        out["residual_norm_merged"] = {"ms_per_step": ms, "us_per_dit_block": ms * 1e3, "launches_per_step": len(merged),
                                       "bytes_per_step": nbytes, "value": nbytes / (ms * 1e-3) / 1e9, "unit": "GB/s"}
        del merged, compiled
    except Exception as exc:
        out["residual_norm_merged"] = {"error": str(exc)[:200]}
    if world > 1:
        # every rank running the whole batch on its own data path: N independent replicas
        try:
            fns = [l.fn for l in workloads.compile_launches(_ran(whole.launches(pair_qk=True)))]
            ms = timed(fns, max(args.steps // 4, 5))
            nbytes = sum(l.bytes for l in whole.launches(pair_qk=True))
            out["replicas"] = {"ms_per_step": ms, "value": world * nbytes / (ms * 1e-3) / 1e9, "unit": "GB/s",
                               "note": "weak scaling: every rank runs the whole batch, no communication"}
            whole.out.clear()
        except Exception as exc:
            out["replicas"] = {"error": str(exc)[:200]}
        torch.cuda.empty_cache()
        out["sharded"] = sharded_forms(be, world, rank, dist, barrier, max_over_ranks, peak)
    else:
        out["configs"] = single_gpu_configs(be, peak)
    try:
        out["pcie"] = pcie_probe(world, barrier, max_over_ranks)
    except Exception as exc:
        out["pcie"] = {"error": str(exc)[:200]}
    return out


def _ran(launches):
    for l in launches:
        l.fn()
    torch.cuda.synchronize()
    return launches
