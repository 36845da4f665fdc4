"""Overlapped launches (programmatic dependent launch) change when a kernel may start, never what it
computes: the Wan block chain gives the same bits with overlap on and off, launched eagerly through
the Python layer, replayed from recorded C-ABI calls, and replayed from a CUDA graph; and token
shards of the block concatenate to the whole block's outputs."""
import pytest

pytestmark = pytest.mark.gpu


def _outputs(blk):
    import torch
    torch.cuda.synchronize()
    return {k: v.clone() for k, v in blk.out.items()}


def _same(a, b, what):
    import torch
    assert a.keys() == b.keys()
    for k in a:
        view = torch.int16 if a[k].dtype == torch.bfloat16 else torch.int32
        assert torch.equal(a[k].view(view), b[k].view(view)), f"{what}: output {k} differs"


def test_overlap_on_off_graph_and_recorded_calls_agree(gpu):
    import torch
    from vrhino_b200 import _lib, workloads
    be, ops = gpu
    lib = _lib.load()
    blk = workloads.WanBlock(be, tokens=4096, grid=(4, 32, 32), ffn=8960, text_tokens=64, seed=21, batch=2)
    previous = lib.vrb_set_launch_overlap(0)
    try:
        for l in blk.launches():
            l.fn()
        plain = _outputs(blk)
        assert lib.vrb_set_launch_overlap(1) == 0
        for v in blk.out.values():
            v.zero_()
        for _ in range(3):          # back to back, so that launches really overlap their predecessors
            for l in blk.launches():
                l.fn()
        _same(plain, _outputs(blk), "overlapped eager")
        compiled = workloads.compile_launches(blk.launches())
        for v in blk.out.values():
            v.zero_()
        for _ in range(3):
            for l in compiled:
                l.fn()
        _same(plain, _outputs(blk), "recorded C-ABI calls")
        side = torch.cuda.Stream()
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.stream(side):
            with torch.cuda.graph(graph, stream=side):
                for l in blk.launches():
                    l.fn()
        for v in blk.out.values():
            v.zero_()
        for _ in range(3):
            graph.replay()
        _same(plain, _outputs(blk), "CUDA graph of overlapped launches")
    finally:
        lib.vrb_set_launch_overlap(previous)


@pytest.mark.parametrize("world", [2, 8])
def test_token_shards_concatenate_to_the_whole_block(gpu, world):
    """What bench.py's multi-GPU arm does, on one GPU: every rank's shard of the same seeded block."""
    import torch
    from vrhino_b200 import workloads
    be, ops = gpu
    blk = workloads.WanBlock(be, tokens=1040, grid=(2, 20, 26), ffn=1024, text_tokens=64, seed=22, batch=2)
    for l in blk.launches():
        l.fn()
    whole = _outputs(blk)
    for rank in range(world):
        shard = blk.token_shard(rank, world)
        for l in shard.launches():
            l.fn()
        torch.cuda.synchronize()
        (r0, r1), (t0, t1) = shard.token_rows, shard.text_rows
        for k, v in shard.out.items():
            want = whole[k][:, t0:t1] if k == "Ek" else whole[k][:, r0:r1]
            view = torch.int16 if v.dtype == torch.bfloat16 else torch.int32
            assert torch.equal(v.view(view), want.contiguous().view(view)), (rank, k)


def test_pair_launch_equals_two_launches(gpu):
    """q and k (and the cross-attention q and text-token k, whose row counts differ) normalised and
    rotated by one launch: the same bits as one launch each; so is the whole chain with pairs."""
    import torch
    from vrhino_b200 import workloads
    be, ops = gpu
    blk = workloads.WanBlock(be, tokens=2080, grid=(2, 26, 40), ffn=1024, text_tokens=77, seed=23, batch=2)
    for l in blk.launches():
        l.fn()
    separate = _outputs(blk)
    for v in blk.out.values():
        v.zero_()
    names = [l.name for l in blk.launches(pair_qk=True)]
    assert len(names) == 9 and "B rms_rope q+k" in names and "E rms cross q+k" in names
    for l in blk.launches(pair_qk=True):
        l.fn()
    _same(separate, _outputs(blk), "pair launches")
    # per-head norm with per-head tables (the Mochi form), F32 output
    g = torch.Generator(device="cuda").manual_seed(5)
    q, k = (torch.randn((1, 300, 24 * 128), device="cuda", generator=g).to(torch.bfloat16) for _ in range(2))
    wq, wk = (torch.randn(128, device="cuda", generator=g) * 0.1 + 1 for _ in range(2))
    phase = torch.rand((1, 300, 24, 128), device="cuda", generator=g) * 6.28
    cos, sin = torch.cos(phase), torch.sin(phase)
    for out_dtype in (torch.bfloat16, torch.float32):
        a = ops.fused_rms_norm_rope(be, q, wq, 1e-5, cos, sin, heads=24, per_head_norm=True, out_dtype=out_dtype)
        b = ops.fused_rms_norm_rope(be, k, wk, 1e-5, cos, sin, heads=24, per_head_norm=True, out_dtype=out_dtype)
        pa, pb = ops.fused_rms_norm_rope_pair(be, q, wq, k, wk, 1e-5, cos, sin, heads=24, per_head_norm=True, out_dtype=out_dtype)
        view = torch.int16 if out_dtype == torch.bfloat16 else torch.int32
        assert torch.equal(a.view(view), pa.view(view)) and torch.equal(b.view(view), pb.view(view)), out_dtype
    # one row against many rows: the reference would pick different summation formulas, so the entry
    # point falls back to two launches -- still the same results
    one = q[:, :1].contiguous()
    a = ops.fused_rms_norm_rope(be, one, wq.repeat(24), 1e-6, None, None)
    pa, pb = ops.fused_rms_norm_rope_pair(be, one, wq.repeat(24), k, wk.repeat(24), 1e-6, None, None)
    assert torch.equal(a.view(torch.int16), pa.view(torch.int16))
    assert torch.equal(ops.fused_rms_norm_rope(be, k, wk.repeat(24), 1e-6, None, None).view(torch.int16), pb.view(torch.int16))
