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
