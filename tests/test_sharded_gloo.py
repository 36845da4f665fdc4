"""The N > 1 choreography on CPU: two gloo ranks, the CPU oracle standing in for the kernels.

Checked: token / H ranges tile the axis; the sharded GroupNorm (broadcast of the shift, one
all-reduce of [units, 3] doubles, local apply, strided gather along H) equals the whole-tensor
oracle result; the sharded sampler update all-gathers to the whole-tensor result; a rank that
fails before the collective makes its peer's collective time out with an error instead of hanging.
"""
import os
import socket
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)


def free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def test_ranges_tile_the_axis():
    from vrhino_b200.sharded import token_range
    for tokens in (32760, 44520, 7, 256):
        for world in (1, 2, 4, 8):
            spans = [token_range(tokens, r, world) for r in range(world)]
            assert spans[0][0] == 0 and spans[-1][1] == tokens
            assert all(a[1] == b[0] for a, b in zip(spans, spans[1:]))
            sizes = [b - a for a, b in spans]
            assert max(sizes) - min(sizes) <= 1
    assert token_range(32760, 3, 8) == (3 * 4095, 4 * 4095)      # 32760 and 44520 divide evenly by 8
    assert token_range(44520, 7, 8) == (7 * 5565, 44520)


class OraclePieces:
    """CPU stand-ins for the three GroupNorm kernels, with their exact contracts."""

    def __init__(self, orc):
        self.orc = orc

    def first_elements(self, x, groups):
        import torch
        b, c = x.shape[0], x.shape[1]
        return x.reshape(b, groups, c // groups, -1)[:, :, 0, 0].reshape(-1).float().contiguous()

    def moments(self, x, groups, shift):
        import torch
        b, c = x.shape[0], x.shape[1]
        d = x.float().reshape(b * groups, -1) - shift.reshape(-1, 1)          # F32 subtraction, as the kernel
        d = d.double()
        n = torch.full((b * groups,), d.shape[1], dtype=torch.float64)
        return torch.stack([n, d.sum(1), (d * d).sum(1)], dim=1).reshape(-1).contiguous()

    def finalize(self, moments, shift, eps):
        import torch
        m = moments.reshape(-1, 3)
        m1 = m[:, 1] / m[:, 0]
        var = torch.clamp(m[:, 2] / m[:, 0] - m1 * m1, min=0.0)
        mean = (shift.double() + m1).float()
        inv = 1.0 / torch.sqrt(var.float() + np.float32(eps))
        return mean, inv

    def apply(self, x, groups, weight, bias, mean, inv, silu):
        import torch
        b, c = x.shape[0], x.shape[1]
        per = c // groups
        xf = x.float().reshape(b, groups, per, -1)
        y = (xf - mean.reshape(b, groups, 1, 1)) * inv.reshape(b, groups, 1, 1)
        w = weight.to(x.dtype).float().reshape(1, groups, per, 1)
        bb = bias.to(x.dtype).float().reshape(1, groups, per, 1)
        y = (y * w + bb).reshape(x.shape).to(x.dtype)
        if silu:
            yf = y.float()
            y = (yf / (1.0 + torch.exp(-yf))).to(x.dtype)
        return y


def _rank_main(rank, world, port, mode, tmp):
    import torch
    import torch.distributed as dist
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    from datetime import timedelta
    dist.init_process_group("gloo", rank=rank, world_size=world, timeout=timedelta(seconds=20))
    from oracle import oracle as orc
    from vrhino_b200 import sharded, synth
    try:
        if mode == "group_norm":
            shape, groups, eps = (1, 16, 3, 8, 12), 4, 1e-6
            x = torch.from_numpy(synth.normal(shape, 0.5, 2.0, seed=5)).to(torch.bfloat16)
            w = torch.from_numpy(synth.normal((16,), 1.0, 0.1, seed=1))
            b = torch.from_numpy(synth.normal((16,), 0.0, 0.1, seed=2))
            h0, h1 = sharded.h_range(shape[3], rank, world)
            local = x[:, :, :, h0:h1, :].contiguous()
            full = sharded.sharded_group_norm(OraclePieces(orc), local, groups, w, b, eps, silu=True, gather_dim=3)
            assert tuple(full.shape) == shape
            np.save(os.path.join(tmp, f"gn_{rank}.npy"), full.view(torch.int16).numpy())
        elif mode == "sampler":
            class FakeOps:
                @staticmethod
                def fused_cfg_euler(be, policy, x, u, c, scale, delta, subtract):
                    g = u + (c + u * -1.0) * scale
                    return x + g * (-delta)
            n = 16 * 3 * 10 * 16
            x, u, c = (torch.from_numpy(synth.normal((n,), seed=s)) for s in (1, 2, 3))
            whole = FakeOps.fused_cfg_euler(None, None, x, u, c, 5.0, 0.02, True)
            got = sharded.sharded_cfg_euler(None, FakeOps, None, x, u, c, 5.0, 0.02)
            assert torch.equal(got, whole)
        elif mode == "peer_failure":
            if rank == 1:
                raise RuntimeError("injected failure before the collective")
            t = torch.zeros(4, dtype=torch.float64)
            try:
                dist.all_reduce(t)
                open(os.path.join(tmp, "no_error"), "w").close()
            except Exception:
                open(os.path.join(tmp, "peer_error_seen"), "w").close()
    finally:
        if mode != "peer_failure":
            dist.destroy_process_group()


def _spawn(mode, tmp, expect_failure=False):
    import torch.multiprocessing as mp
    port = free_port()
    ctx = mp.get_context("spawn")
    procs = [ctx.Process(target=_rank_main, args=(r, 2, port, mode, str(tmp))) for r in range(2)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(120)
    codes = [p.exitcode for p in procs]
    for p in procs:
        if p.is_alive():
            p.kill()
    if not expect_failure:
        assert codes == [0, 0], codes
    return codes


def test_sharded_group_norm_two_ranks(orc, tmp_path):
    from vrhino_b200 import synth
    _spawn("group_norm", tmp_path)
    shape, groups, eps = (1, 16, 3, 8, 12), 4, 1e-6
    x = orc.tensor(synth.normal(shape, 0.5, 2.0, seed=5), "bf16")
    w, b = orc.tensor(synth.normal((16,), 1.0, 0.1, seed=1)), orc.tensor(synth.normal((16,), 0.0, 0.1, seed=2))
    want = orc.group_norm_silu(orc.OracleBackend(), x, groups, w, b, eps)
    got0 = np.load(tmp_path / "gn_0.npy").view(np.uint16)
    got1 = np.load(tmp_path / "gn_1.npy").view(np.uint16)
    assert np.array_equal(got0, got1), "ranks disagree on the gathered tensor"
    d = orc.bf16_ulp_distance(got0, want.data)
    assert d.max() <= 2, int(d.max())


def test_sharded_sampler_two_ranks(tmp_path):
    _spawn("sampler", tmp_path)


def test_peer_failure_surfaces_as_an_error(tmp_path):
    """A rank that dies before the collective (host-side failure, no GPU involved): the survivor's
    collective ends with an error within the process-group timeout instead of hanging."""
    codes = _spawn("peer_failure", tmp_path, expect_failure=True)
    assert codes[1] != 0
    assert (tmp_path / "peer_error_seen").exists() and not (tmp_path / "no_error").exists()
