"""GPU parity of GroupNorm (+SiLU) against the oracle, which restates the reference's anchored
two-pass F32 statistics (direct and multi-partial paths).  The kernel here uses a shifted
one-pass double accumulation; both are accurate to F32 rounding of the mean / variance, so
outputs are compared at <= 2 bf16 ulp / 1e-5 relative (+ 1e-6 absolute for the beta add)."""
import numpy as np
import pytest

from conftest import assert_close, from_torch, to_torch

pytestmark = pytest.mark.gpu

CASES = [
    # (shape, groups, eps)                                  which reference path
    ((1, 2, 2), 2, 1e-5),                                  # primitive_tests.cpp:539
    ((2, 4, 1, 2), 4, 1e-5),                               # primitive_tests.cpp:539
    ((2, 32, 5, 7), 8, 1e-6),                              # direct, scalar kernel (odd spatial)
    ((1, 64, 4, 16, 16), 32, 1e-6),                        # direct, 5-D statistics
    ((3, 64, 24, 40), 32, 1e-5),                           # direct, Mochi per-frame form
    ((1, 32, 3, 120, 128), 4, 1e-6),                       # count = 368640 > 2^18: multi-partial path
    ((1, 32, 9, 120, 128), 8, 1e-6),                       # 4.4 M elements: bf16 + SiLU takes the table kernel
    ((5, 64, 1, 120, 112), 32, 1e-6),                      # same, per-frame form with a ragged last tile
]


@pytest.mark.parametrize("dtype", ["f32", "bf16"])
@pytest.mark.parametrize("shape,groups,eps", CASES)
@pytest.mark.parametrize("affine", [True, False])
def test_group_norm(orc, gpu, dtype, shape, groups, eps, affine):
    be, ops = gpu
    from vrhino_b200 import synth
    obe = orc.OracleBackend()
    x = orc.tensor(synth.normal(shape, 0.3, 2.0, seed=len(shape)), dtype)
    w = orc.tensor(synth.normal((shape[1],), 1.0, 0.1, seed=1)) if affine else None
    b = orc.tensor(synth.normal((shape[1],), 0.0, 0.1, seed=2)) if affine else None
    want, mean, inv = obe.group_norm(x, groups, w, b, eps, return_moments=True)
    tw, tb = (to_torch(w), to_torch(b)) if affine else (None, None)
    got = be.group_norm(to_torch(x), groups, tw, tb, eps)
    assert_close(orc, got, want, rel=1e-5, atol=2e-6, what="group_norm")
    want_s = obe.activation(want, orc.SILU)
    got_s = ops.fused_group_norm_silu(be, to_torch(x), groups, tw, tb, eps)
    assert_close(orc, got_s, want_s, rel=1e-5, atol=2e-6, what="group_norm+silu")


def test_group_norm_against_double_precision(orc, gpu):
    """Independent check (neither the oracle nor the kernel): float64 centred statistics, at the
    reference's F32 gate 2e-5 + 2e-5|r|, on data with a large common offset."""
    be, ops = gpu
    from vrhino_b200 import synth
    shape, groups, eps = (2, 16, 6, 32, 32), 4, 1e-6
    x = synth.normal(shape, 40.0, 2.0, seed=3)
    got, _ = from_torch(be.group_norm(to_torch(orc.tensor(x)), groups, None, None, eps))
    xd = x.astype(np.float64).reshape(2, groups, -1)
    ref = ((xd - xd.mean(axis=2, keepdims=True)) / np.sqrt(xd.var(axis=2, keepdims=True) + eps)).reshape(shape)
    assert (np.abs(got - ref) <= 2e-5 + 2e-5 * np.abs(ref)).all()


def test_group_norm_repeat_is_bit_exact(gpu):
    import torch
    be, ops = gpu
    x = torch.randn(1, 32, 3, 120, 128, device="cuda", dtype=torch.bfloat16)
    a, b = be.group_norm(x, 4, None, None, 1e-6), be.group_norm(x, 4, None, None, 1e-6)
    assert torch.equal(a.view(torch.int16), b.view(torch.int16))


def test_group_norm_rejections(gpu):
    import ctypes
    import torch
    be, ops = gpu
    with pytest.raises(ops.VrbError, match="group norm shape/groups mismatch"):
        be.group_norm(torch.zeros(1, 6, 4, device="cuda"), 4, None, None, 1e-5)
    from vrhino_b200 import _lib
    x = torch.zeros(1, 8, 16, device="cuda")
    rc = _lib.load().vrb_group_norm(ctypes.c_void_p(x.data_ptr()), 0, None, 0, None, 0, ctypes.c_void_p(x.data_ptr()),
                                    1, 8, 16, 4, ctypes.c_float(1e-5), 0, None, 0, None)
    assert rc == -4 and b"workspace" in _lib.load().vrb_last_error()


def test_group_norm_split_statistics_match_whole(orc, gpu):
    """The multi-GPU pieces on one GPU: moments of H-slices added, finalised and applied per
    slice give the same result as the whole-tensor call (bit for bit on the statistics path up
    to the double additions; outputs compared at the usual tolerance)."""
    import ctypes
    import torch
    be, ops = gpu
    from vrhino_b200 import _lib, synth
    lib = _lib.load()
    C, T, H, W, groups, eps, parts = 16, 3, 16, 24, 4, 1e-6, 4
    x = orc.tensor(synth.normal((1, C, T, H, W), 0.5, 2.0, seed=5), "bf16")
    w, b = orc.tensor(synth.normal((C,), 1.0, 0.1, seed=1)), orc.tensor(synth.normal((C,), 0.0, 0.1, seed=2))
    tx, tw, tb = to_torch(x), to_torch(w), to_torch(b)
    whole = ops.fused_group_norm_silu(be, tx, groups, tw, tb, eps)
    units = groups
    shift = torch.zeros(units, device="cuda")
    total = torch.zeros(units * 3, dtype=torch.float64, device="cuda")
    need = lib.vrb_group_norm_workspace_bytes(1, groups)
    ws = torch.empty(need, dtype=torch.uint8, device="cuda")
    slices = [tx[:, :, :, r * H // parts:(r + 1) * H // parts, :].contiguous() for r in range(parts)]
    P = ctypes.c_void_p
    for sl in slices:
        m = torch.empty(units * 3, dtype=torch.float64, device="cuda")
        _lib.call("vrb_group_norm_moments", P(sl.data_ptr()), 2, 1, C, sl.numel() // C, groups, P(shift.data_ptr()),
                  P(m.data_ptr()), P(ws.data_ptr()), need, None)
        total += m                      # stands in for the all-reduce
    mean, inv = torch.empty(units, device="cuda"), torch.empty(units, device="cuda")
    _lib.call("vrb_group_norm_finalize", P(total.data_ptr()), P(shift.data_ptr()), units, ctypes.c_float(eps),
              P(mean.data_ptr()), P(inv.data_ptr()), None)
    outs = []
    for sl in slices:
        o = torch.empty_like(sl)
        _lib.call("vrb_group_norm_apply", P(sl.data_ptr()), 2, P(tw.data_ptr()), 0, P(tb.data_ptr()), 0, P(o.data_ptr()),
                  1, C, sl.numel() // C, groups, P(mean.data_ptr()), P(inv.data_ptr()), 1, None)
        outs.append(o)
    joined = torch.cat(outs, dim=3)
    want = orc.group_norm_silu(orc.OracleBackend(), x, groups, w, b, eps)
    assert_close(orc, joined, want, rel=1e-5, atol=2e-6, what="sliced group_norm+silu")
    d = orc.bf16_ulp_distance(from_torch(joined)[0], from_torch(whole)[0])
    assert d.max() <= 1 and (d > 0).mean() < 1e-3



@pytest.mark.parametrize("dtype", ["f32", "bf16"])
@pytest.mark.parametrize("shape,groups", [((2, 32, 3, 8, 16), 8), ((1, 64, 5, 24, 40), 32), ((1, 32, 9, 120, 128), 8)])
@pytest.mark.parametrize("silu", [False, True])
def test_group_norm_frames_equals_permute_norm_permute(orc, gpu, dtype, shape, groups, silu):
    """frame_group_norm (native/src/architectures/mochi.cpp:365-371): permute [B,C,T,H,W] ->
    [B*T,C,H,W], group_norm(32, 1e-5), permute back.  The kernel reads and writes [B,C,T,H,W]
    directly; the oracle does the three steps."""
    be, ops = gpu
    from vrhino_b200 import synth
    B, C, T, H, W = shape
    obe = orc.OracleBackend()
    raw = synth.normal(shape, 0.3, 2.0, seed=T)
    x = orc.tensor(raw, dtype)
    w = orc.tensor(synth.normal((C,), 1.0, 0.1, seed=1))
    b = orc.tensor(synth.normal((C,), 0.0, 0.1, seed=2))
    frames = orc.T(np.ascontiguousarray(x.data.transpose(0, 2, 1, 3, 4)).reshape(B * T, C, H, W), dtype)
    normed = obe.group_norm(frames, groups, w, b, 1e-5)
    if silu:
        normed = obe.activation(normed, orc.SILU)
    want = orc.T(np.ascontiguousarray(normed.data.reshape(B, T, C, H, W).transpose(0, 2, 1, 3, 4)), dtype)
    got = be.group_norm_frames(to_torch(x), groups, to_torch(w), to_torch(b), 1e-5, fuse_silu=silu)
    if silu and dtype == "bf16":
        # SiLU amplifies a one-ulp difference of a very negative y: compare through the unfused pair
        y = be.group_norm_frames(to_torch(x), groups, to_torch(w), to_torch(b), 1e-5)
        import torch
        assert torch.equal(got.view(torch.int16), be.activation(y, 0).view(torch.int16))
        return
    assert_close(orc, got, want, rel=1e-5, atol=2e-6, what="group_norm_frames")


@pytest.mark.parametrize("dtype,silu", [("bf16", True), ("bf16", False), ("f32", True)])
def test_group_norm_apply_scatter_places_the_slice(gpu, dtype, silu):
    """The normalise pass that stores an H-slice into several full-size tensors (the all-gather of
    an H-sharded feature map done by the kernel's stores): on one GPU, two destination buffers
    stand in for this rank's and a peer's tensor.  Rows [row0, row0 + h_local) of every plane must
    equal the plain apply pass on the slice, everything else must stay untouched."""
    import torch
    from vrhino_b200 import sharded
    be, ops = gpu
    td = torch.bfloat16 if dtype == "bf16" else torch.float32
    n, c, t, h_full, w, groups, row0, h_local = 1, 64, 3, 20, 424, 8, 5, 10
    if silu and dtype == "bf16":
        t = 36                                          # 64 * 36 * 10 * 424 = 9.8 M elements: the table kernel
    g = torch.Generator(device="cuda").manual_seed(1)
    x = (torch.randn((n, c, t, h_local, w), device="cuda", generator=g) * 2).to(td)
    gamma = torch.randn(c, device="cuda", generator=g) * 0.1 + 1
    beta = torch.randn(c, device="cuda", generator=g) * 0.1
    pieces = sharded.KernelMoments(be)
    shift = pieces.first_elements(x, groups)
    mean, inv = pieces.finalize(pieces.moments(x, groups, shift), shift, 1e-6)
    want = pieces.apply(x, groups, gamma, beta, mean, inv, silu)
    dests = [torch.full((n, c, t, h_full, w), 7.0, device="cuda", dtype=td) for _ in range(2)]
    pieces.apply_scatter(x, groups, gamma, beta, mean, inv, silu, [d.data_ptr() for d in dests], h_full, row0)
    torch.cuda.synchronize()
    for d in dests:
        assert torch.equal(d[:, :, :, row0:row0 + h_local], want)
        assert bool((d[:, :, :, :row0] == 7.0).all()) and bool((d[:, :, :, row0 + h_local:] == 7.0).all())
