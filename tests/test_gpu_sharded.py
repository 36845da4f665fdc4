"""Two NCCL ranks on two GPUs (skipped on a single-GPU box): the sharded GroupNorm+SiLU (with the
output gathered by NCCL, and by the normalise kernel's own peer stores) and the sharded sampler
update give the single-GPU result; token-sharded row kernels give the same rows."""
import os
import socket
import sys

import numpy as np
import pytest

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _rank(rank, world, port, tmp):
    import torch
    import torch.distributed as dist
    sys.path.insert(0, ROOT)
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    from vrhino_b200 import ops, sharded, synth
    be = ops.B200Backend(device=f"cuda:{rank}")
    shape, groups, eps = (1, 32, 4, 16, 24), 8, 1e-6
    x = torch.from_numpy(synth.normal(shape, 0.5, 2.0, seed=5)).to(torch.bfloat16).cuda()
    w = torch.from_numpy(synth.normal((32,), 1.0, 0.1, seed=1)).cuda()
    b = torch.from_numpy(synth.normal((32,), 0.0, 0.1, seed=2)).cuda()
    h0, h1 = sharded.h_range(shape[3], rank, world)
    full = sharded.sharded_group_norm(sharded.KernelMoments(be), x[:, :, :, h0:h1, :].contiguous(), groups, w, b, eps, True, None, 3)
    whole = ops.fused_group_norm_silu(be, x, groups, w, b, eps)
    # the same with the gather done by the normalise kernel's stores into every rank's (peer-mapped) output
    peer = sharded.PeerOutput(shape, torch.bfloat16, torch.device("cuda", rank))
    via_peer = sharded.sharded_group_norm(sharded.KernelMoments(be), x[:, :, :, h0:h1, :].contiguous(), groups, w, b, eps, True,
                                          None, None, peer, h0)
    torch.cuda.synchronize()
    assert torch.equal(via_peer.view(torch.int16), full.view(torch.int16)), "peer-store gather differs from the NCCL gather"
    torch.save({"full": full.cpu(), "whole": whole.cpu()}, os.path.join(tmp, f"gn_{rank}.pt"))
    pol = ops.Policy.fp32()
    n = 16 * 21 * 60 * 104
    lat, u, c = (torch.from_numpy(synth.normal((n,), seed=s)).cuda() for s in (1, 2, 3))
    got = sharded.sharded_cfg_euler(be, ops, pol, lat, u, c, 5.0, 0.02)
    want = ops.fused_cfg_euler(be, pol, lat, u, c, 5.0, 0.02, True)
    assert torch.equal(got, want)
    t0, t1 = sharded.token_range(600, rank, world)
    xs = torch.from_numpy(synth.normal((1, 600, 1536), seed=9)).to(torch.bfloat16).cuda()
    sh = torch.from_numpy(synth.normal((1, 1, 1536), std=0.1, seed=10)).cuda()
    sc = torch.from_numpy(synth.normal((1, 1, 1536), std=0.1, seed=11)).cuda()
    part = ops.fused_layer_norm_modulate(be, xs[:, t0:t1].contiguous(), None, None, 1e-6, sh, sc)
    all_rows = ops.fused_layer_norm_modulate(be, xs, None, None, 1e-6, sh, sc)
    assert torch.equal(part.view(torch.int16), all_rows[:, t0:t1].contiguous().view(torch.int16))
    torch.cuda.synchronize()
    dist.destroy_process_group()


def _native_rank(rank, world, port, tmp, leave):
    """The C++ host layer (libvrb_sharded.so) over its own NCCL communicator: the three gather modes of the
    H-sharded GroupNorm + SiLU and the sampler's all-gather against the Python layer / the whole tensor.
    leave: rank 1 destroys its communicator and exits BETWEEN steps (nothing of its own in flight); rank 0
    enqueues the next step and its bounded wait must give up, abort the communicator and say so."""
    import ctypes
    import torch
    import torch.distributed as dist
    sys.path.insert(0, ROOT)
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    dist.init_process_group("gloo", rank=rank, world_size=world)      # only carries the unique id and barriers
    from vrhino_b200 import _lib, ops, sharded, synth
    lib = _lib.load_sharded()
    P = ctypes.c_void_p
    ident = [None]
    if rank == 0:
        buf = ctypes.create_string_buffer(128)
        assert lib.vrbs_unique_id(buf) == 0, lib.vrbs_last_error()
        ident[0] = buf.raw
    dist.broadcast_object_list(ident, src=0)
    comm = ctypes.c_void_p()
    assert lib.vrbs_create(ctypes.byref(comm), rank, world, ident[0], 2000) == 0, lib.vrbs_last_error()
    be = ops.B200Backend(device=f"cuda:{rank}")
    shape, groups, eps = (1, 32, 4, 16, 24), 8, 1e-6
    x = torch.from_numpy(synth.normal(shape, 0.5, 2.0, seed=5)).to(torch.bfloat16).cuda()
    w = torch.from_numpy(synth.normal((32,), 1.0, 0.1, seed=1)).cuda()
    b = torch.from_numpy(synth.normal((32,), 0.0, 0.1, seed=2)).cuda()
    h0, h1 = sharded.h_range(shape[3], rank, world)
    local = x[:, :, :, h0:h1, :].contiguous()
    stream = P(torch.cuda.current_stream().cuda_stream)

    def group_norm(gather, out, destinations=None):
        need = lib.vrbs_group_norm_workspace_bytes(comm, 1, groups, gather, local.numel() * 2)
        ws = torch.empty(need, dtype=torch.uint8, device="cuda")
        rc = lib.vrbs_group_norm(comm, P(local.data_ptr()), 2, P(w.data_ptr()), 0, P(b.data_ptr()), 0,
                                 None if out is None else P(out.data_ptr()), 1, 32, 4, h1 - h0, 16, h0, 24, groups, ctypes.c_float(eps), 1,
                                 gather, destinations, P(ws.data_ptr()), need, stream)
        assert rc == 0, lib.vrbs_last_error()
        assert lib.vrbs_wait(comm, stream) == 0, lib.vrbs_last_error()
        return ws

    whole = ops.fused_group_norm_silu(be, x, groups, w, b, eps)
    sliced, gathered = torch.empty_like(local), torch.empty_like(x)
    group_norm(0, sliced)
    group_norm(1, gathered)
    assert torch.equal(sliced.view(torch.int16), gathered[:, :, :, h0:h1].contiguous().view(torch.int16))
    d = (gathered.float() - whole.float()).abs().max().item()
    assert d <= 0.02, d                     # the same tensor up to the last bit of a few statistics
    lat, u, c = (torch.from_numpy(synth.normal((16 * 21 * 60 * 104,), seed=s)).cuda() for s in (1, 2, 3))
    got = torch.empty_like(lat)
    assert lib.vrbs_cfg_euler(comm, P(lat.data_ptr()), P(u.data_ptr()), P(c.data_ptr()), P(got.data_ptr()), 0, lat.numel(),
                              ctypes.c_float(5.0), ctypes.c_float(0.02), 1, 0, 0, stream) == 0, lib.vrbs_last_error()
    assert lib.vrbs_wait(comm, stream) == 0, lib.vrbs_last_error()
    be32 = ops.B200Backend(execution_dtype=torch.float32, device=f"cuda:{rank}")   # F32 execution: delta is passed as it is
    assert torch.equal(got, ops.fused_cfg_euler(be32, ops.Policy.fp32(), lat, u, c, 5.0, 0.02, True))
    torch.save({"gathered": gathered.cpu()}, os.path.join(tmp, f"native_{rank}.pt"))
    torch.cuda.synchronize()
    dist.barrier()                           # the step is over on every rank
    if leave and rank == 1:
        lib.vrbs_destroy(comm)
        return                               # leaves between steps
    if leave:
        need = lib.vrbs_group_norm_workspace_bytes(comm, 1, groups, 0, local.numel() * 2)
        ws = torch.empty(need, dtype=torch.uint8, device="cuda")
        rc = lib.vrbs_group_norm(comm, P(local.data_ptr()), 2, P(w.data_ptr()), 0, P(b.data_ptr()), 0, P(sliced.data_ptr()), 1, 32, 4,
                                 h1 - h0, 16, h0, 24, groups, ctypes.c_float(eps), 1, 0, None, P(ws.data_ptr()), need, stream)
        status = lib.vrbs_wait(comm, stream) if rc == 0 else rc
        assert status in (-6, -5), (status, lib.vrbs_last_error())    # timed out (or NCCL saw the peer go): aborted
        assert lib.vrbs_aborted(comm) == 1
        assert lib.vrbs_wait(comm, stream) == -7
        torch.save({"status": status}, os.path.join(tmp, "left.pt"))
    lib.vrbs_destroy(comm)


@pytest.mark.parametrize("leave", [False, True], ids=["steady", "a_rank_leaves_between_steps"])
def test_two_rank_native_host_layer(tmp_path, leave):
    import torch
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    import torch.multiprocessing as mp
    port = _port()
    ctx = mp.get_context("spawn")
    procs = [ctx.Process(target=_native_rank, args=(r, 2, port, str(tmp_path), leave)) for r in range(2)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(300)
    assert [p.exitcode for p in procs] == [0, 0]
    a, b = torch.load(tmp_path / "native_0.pt"), torch.load(tmp_path / "native_1.pt")
    assert torch.equal(a["gathered"].view(torch.int16), b["gathered"].view(torch.int16))
    if leave:
        assert torch.load(tmp_path / "left.pt")["status"] in (-6, -5)


def test_two_rank_group_norm_sampler_and_token_shards(orc, tmp_path):
    import torch
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    import torch.multiprocessing as mp
    port = _port()
    ctx = mp.get_context("spawn")
    procs = [ctx.Process(target=_rank, args=(r, 2, port, str(tmp_path))) for r in range(2)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(300)
    assert [p.exitcode for p in procs] == [0, 0]
    a, b = torch.load(tmp_path / "gn_0.pt"), torch.load(tmp_path / "gn_1.pt")
    assert torch.equal(a["full"].view(torch.int16), b["full"].view(torch.int16))
    d = orc.bf16_ulp_distance(a["full"].view(torch.int16).numpy().view(np.uint16), a["whole"].view(torch.int16).numpy().view(np.uint16))
    assert d.max() <= 1 and (d > 0).mean() < 1e-3
