"""Multi-GPU forms of the path: one process per GPU, torch.distributed (NCCL) for the plumbing.

What shards how:

* every DiT operator is independent per token row -> contiguous token ranges per rank, no
  collective (``token_range``);
* the sampler update is flat elementwise -> flat ranges per rank, then ONE all-gather of the
  latent (``sharded_cfg_euler``);
* GroupNorm over a feature map split along H: per-rank shifted moments -> ONE all-reduce of
  [units, 3] doubles -> finalize -> local normalise (+SiLU) -> optional gather of the output,
  whose H-slices are strided in the full NC(T)HW tensor (``sharded_group_norm``).

The shift that makes the one-pass variance safe must be the same on every rank: rank 0's first
element of each unit is broadcast (units floats) before the moments pass.

``MomentsBackend`` abstracts the three GroupNorm pieces so the choreography (what is reduced,
in which order, with which shapes) is testable on CPU ranks with gloo, where the test supplies
CPU stand-ins for the three kernels; on GPUs the pieces are the C-ABI entry points.
"""
from __future__ import annotations

import ctypes

import torch
import torch.distributed as dist


def token_range(tokens: int, rank: int, world: int):
    """Contiguous rows [start, stop) of rank `rank`; sizes differ by at most one row."""
    base, extra = divmod(tokens, world)
    start = rank * base + min(rank, extra)
    return start, start + base + (1 if rank < extra else 0)


def h_range(height: int, rank: int, world: int):
    return token_range(height, rank, world)


class KernelMoments:
    """GroupNorm pieces on the GPU through the C ABI."""

    def __init__(self, be):
        from . import _lib
        self.be, self._lib = be, _lib
        self._ws = None

    def _workspace(self, batch, groups):
        need = self._lib.load().vrb_group_norm_workspace_bytes(batch, groups)
        if self._ws is None or self._ws.numel() < need:
            self._ws = torch.empty(need, dtype=torch.uint8, device=self.be.device)
        return self._ws, need

    @staticmethod
    def _code(t):
        return 2 if t.dtype == torch.bfloat16 else 0

    def first_elements(self, x, groups):
        batch, channels = x.shape[0], x.shape[1]
        per = channels // groups
        return x.reshape(batch, groups, per, -1)[:, :, 0, 0].reshape(-1).float().contiguous()

    def moments(self, x, groups, shift):
        P = ctypes.c_void_p
        batch, channels = x.shape[0], x.shape[1]
        spatial = x.numel() // (batch * channels)
        out = torch.empty(batch * groups * 3, dtype=torch.float64, device=x.device)
        ws, need = self._workspace(batch, groups)
        self._lib.call("vrb_group_norm_moments", P(x.data_ptr()), self._code(x), batch, channels, spatial, groups,
                       P(shift.data_ptr()), P(out.data_ptr()), P(ws.data_ptr()), need,
                       ctypes.c_void_p(torch.cuda.current_stream().cuda_stream))
        return out

    def finalize(self, moments, shift, eps):
        P = ctypes.c_void_p
        units = shift.numel()
        mean = torch.empty(units, dtype=torch.float32, device=shift.device)
        inv = torch.empty_like(mean)
        self._lib.call("vrb_group_norm_finalize", P(moments.data_ptr()), P(shift.data_ptr()), units, ctypes.c_float(eps),
                       P(mean.data_ptr()), P(inv.data_ptr()), ctypes.c_void_p(torch.cuda.current_stream().cuda_stream))
        return mean, inv

    def apply(self, x, groups, weight, bias, mean, inv, silu):
        P = ctypes.c_void_p
        batch, channels = x.shape[0], x.shape[1]
        spatial = x.numel() // (batch * channels)
        out = torch.empty_like(x)
        wp = None if weight is None else P(weight.data_ptr())
        bp = None if bias is None else P(bias.data_ptr())
        self._lib.call("vrb_group_norm_apply", P(x.data_ptr()), self._code(x), wp, 0 if weight is None else self._code(weight),
                       bp, 0 if bias is None else self._code(bias), P(out.data_ptr()), batch, channels, spatial, groups,
                       P(mean.data_ptr()), P(inv.data_ptr()), int(silu),
                       ctypes.c_void_p(torch.cuda.current_stream().cuda_stream))
        return out


    def apply_scatter(self, x, groups, weight, bias, mean, inv, silu, destinations, rows_full, row0):
        """Normalise this rank's H-slice x [N, C, T, h_local, W] and store it into every tensor of
        `destinations` (data pointers of full [N, C, T, rows_full, W] tensors: this GPU's own and the
        peer-mapped ones) at rows [row0, row0 + h_local)."""
        P = ctypes.c_void_p
        n, c, t, h, w = x.shape
        ptrs = (ctypes.c_void_p * len(destinations))(*destinations)
        wp = None if weight is None else P(weight.data_ptr())
        bp = None if bias is None else P(bias.data_ptr())
        self._lib.call("vrb_group_norm_apply_scatter", P(x.data_ptr()), self._code(x), wp, 0 if weight is None else self._code(weight),
                       bp, 0 if bias is None else self._code(bias), ptrs, len(destinations), n, c, t, h * w, rows_full * w, row0 * w,
                       groups, P(mean.data_ptr()), P(inv.data_ptr()), int(silu),
                       ctypes.c_void_p(torch.cuda.current_stream().cuda_stream))


class PeerOutput:
    """The full output tensor of every rank, mapped into every rank (torch symmetric memory):
    the normalise kernel of each rank stores its H-slice straight into all of them, so no
    all-gather and no placement copy follow.  Two orderings, both on the current stream:
    `acquire()` before the stores -- every rank has finished whatever it was doing with the previous
    contents of its tensor (work it enqueued before its own acquire), so peers may overwrite it --
    and `ready()` after them -- every rank's stores have landed before anyone reads the result."""

    def __init__(self, shape, dtype, device, group=None):
        import torch.distributed._symmetric_memory as symm
        self.group = group if group is not None else dist.group.WORLD
        self.tensor = symm.empty(*shape, dtype=dtype, device=device)
        self.handle = symm.rendezvous(self.tensor, self.group)
        self.pointers = [int(p) for p in self.handle.buffer_ptrs]
        self._flag = torch.zeros(1, device=device)

    def acquire(self):
        dist.all_reduce(self._flag, group=self.group)   # every rank's earlier reads precede its contribution

    def ready(self):
        dist.all_reduce(self._flag, group=self.group)   # every rank's kernel precedes its contribution


def sharded_group_norm(pieces, x_local, groups, weight, bias, eps, silu=True, group=None, gather_dim=None, peer_out=None,
                       row0=0):
    """GroupNorm(+SiLU) of a tensor whose spatial extent is split over the ranks of `group`.

    x_local: this rank's slice [N, C, ...] (contiguous).  Returns the normalised slice, or, with
    gather_dim set (the axis the tensor was split along, e.g. 3 for H of [N,C,T,H,W]), the full
    tensor assembled from all ranks' slices.
    Collectives: broadcast of [units] floats, all-reduce(sum) of [units*3] doubles, and the
    optional all-gather of the output.
    """
    world = dist.get_world_size(group) if dist.is_initialized() else 1
    shift = pieces.first_elements(x_local, groups)
    if world > 1:
        dist.broadcast(shift, src=dist.get_global_rank(group, 0) if group is not None else 0, group=group)
    moments = pieces.moments(x_local, groups, shift)
    if world > 1:
        dist.all_reduce(moments, op=dist.ReduceOp.SUM, group=group)
    mean, inv = pieces.finalize(moments, shift, eps)
    if peer_out is not None:
        # the "gather" happens in the normalise kernel's stores (peer memory over NVLink).  The
        # statistics all-reduce above already is the "acquire": no rank gets past it before every rank
        # has reached it, i.e. has finished the reads of the previous result it enqueued earlier.
        if world == 1:
            peer_out.acquire()
        pieces.apply_scatter(x_local, groups, weight, bias, mean, inv, silu, peer_out.pointers, peer_out.tensor.shape[3], row0)
        peer_out.ready()
        return peer_out.tensor
    out = pieces.apply(x_local, groups, weight, bias, mean, inv, silu)
    if gather_dim is None or world == 1:
        return out
    return gather_slices(out, gather_dim, group)


def gather_slices(local, dim, group=None):
    """All-gather equal-sized slices and place them along `dim` of the full tensor.  The slices
    are contiguous per rank but strided in the result, so the gather lands in a staging buffer
    [world, *local.shape] and one strided copy places it."""
    world = dist.get_world_size(group)
    staging = torch.empty((world,) + tuple(local.shape), dtype=local.dtype, device=local.device)
    dist.all_gather_into_tensor(staging.view(-1), local.contiguous().view(-1), group=group)
    shape = list(local.shape)
    full_shape = shape[:dim] + [world * shape[dim]] + shape[dim + 1:]
    full = torch.empty(full_shape, dtype=local.dtype, device=local.device)
    view = full.view(shape[:dim] + [world, shape[dim]] + shape[dim + 1:])
    view.copy_(staging.movedim(0, dim))
    return full


def sharded_cfg_euler(be, ops, policy, sample, unconditional, conditional, scale, delta, group=None):
    """cfg_combine + euler_update on this rank's flat range of the latent, then the latent
    all-gather.  Inputs are the FULL tensors (replicated); returns the full updated latent."""
    world = dist.get_world_size(group) if dist.is_initialized() else 1
    rank = dist.get_rank(group) if dist.is_initialized() else 0
    n = sample.numel()
    if world == 1 or n % (world * 8):
        return ops.fused_cfg_euler(be, policy, sample, unconditional, conditional, scale, delta, True)
    per = n // world
    sl = slice(rank * per, (rank + 1) * per)
    flat = lambda t: t.reshape(-1)[sl]
    local = ops.fused_cfg_euler(be, policy, flat(sample), flat(unconditional), flat(conditional), scale, delta, True)
    full = torch.empty(n, dtype=sample.dtype, device=sample.device)
    dist.all_gather_into_tensor(full, local, group=group)
    return full.reshape(sample.shape)


def _main():
    """torchrun ... -m vrhino_b200.sharded [--frames T] [--steps K]

    GroupNorm(32) + SiLU on [1, 256, T, 240, 424] bf16 split along H over the ranks: device time of
    the local work + the statistics all-reduce ("compute"), and of the same followed by the
    all-gather of the output ("compute+gather"); max over ranks, CUDA events."""
    import argparse
    import os
    ap = argparse.ArgumentParser()
    ap.add_argument("--frames", type=int, default=28)
    ap.add_argument("--steps", type=int, default=10)
    a = ap.parse_args()
    world, rank, local = int(os.environ.get("WORLD_SIZE", "1")), int(os.environ.get("RANK", "0")), int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    from . import ops
    be = ops.B200Backend(device=f"cuda:{local}")
    pieces = KernelMoments(be)
    h0, h1 = h_range(240, rank, world)
    g = torch.Generator(device="cuda").manual_seed(rank)
    x = (torch.randn((1, 256, a.frames, h1 - h0, 424), device="cuda", generator=g) * 2.0).to(torch.bfloat16)
    gamma, beta = torch.ones(256, device="cuda"), torch.zeros(256, device="cuda")

    peer = PeerOutput((1, 256, a.frames, 240, 424), torch.bfloat16, torch.device("cuda", local)) if world > 1 else None

    def timed(gather):
        def step():
            if gather == "peer":
                return sharded_group_norm(pieces, x, 32, gamma, beta, 1e-6, True, None, None, peer, h0)
            return sharded_group_norm(pieces, x, 32, gamma, beta, 1e-6, True, None, 3 if gather and world > 1 else None)
        for _ in range(3):
            step()
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(a.steps):
            step()
        e1.record()
        torch.cuda.synchronize()
        t = torch.tensor([e0.elapsed_time(e1) / a.steps], device="cuda", dtype=torch.float64)
        if world > 1:
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    compute, both = timed(False), timed(True)
    fused = timed("peer") if world > 1 else compute
    if rank == 0:
        full_bytes = 256 * a.frames * 240 * 424 * 6
        print(f"n_gpus {world}  H rows per rank {h1 - h0}  compute {compute * 1e3:.1f} us ({full_bytes / compute / 1e6:.0f} GB/s aggregate)"
              f"  compute + NCCL all-gather + placement {both * 1e3:.1f} us  compute with peer stores {fused * 1e3:.1f} us")
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    _main()
