"""pixel_norm over the channel axis and its merged form with modulate + SiLU: every path of the
launcher (shared-memory tiles of 8 / 4 / 2 / 1 chunks, ragged last tile, the strided fallback for odd
extents, the row kernel for inner == 1) against the oracle -- bit for bit up to the modulation, and
within F32 tolerance after expf."""
import numpy as np
import pytest

from conftest import assert_bits_equal, assert_close, to_torch

pytestmark = pytest.mark.gpu

SHAPES = [
    (2, 128, 3, 8, 16),     # tiles of 8 chunks
    (1, 64, 1, 5, 8),       # inner 40: one ragged tile (5 chunks of bf16, 10 of f32)
    (1, 1024, 2, 4, 12),    # 1024 channels: narrower tiles
    (1, 2048, 1, 2, 16),    # 2 chunks per row
    (1, 4000, 1, 1, 16),    # one CTA per SM
    (1, 20, 2, 3, 5),       # odd inner: strided fallback
    (3, 7, 1, 1, 24),       # channels not a multiple of the 8 lanes
    (6, 300),               # inner == 1: row kernel
    (2, 9, 1),              # inner == 1, fewer channels than threads
]


@pytest.mark.parametrize("shape", SHAPES)
@pytest.mark.parametrize("dt", ["bf16", "f32"])
def test_pixel_norm_bit_exact(orc, gpu, shape, dt):
    be, ops = gpu
    from vrhino_b200 import synth
    x = orc.tensor(synth.normal(shape, 0.2, 1.5, seed=len(shape) + shape[1]), dt)
    want = orc.OracleBackend().pixel_norm(x, 1, 1e-8)
    assert_bits_equal(be.pixel_norm(to_torch(x), 1, 1e-8), want, "pixel_norm")


@pytest.mark.parametrize("l2", [False, True], ids=["pixel_norm", "l2_normalize"])
def test_quotient_guards_at_extreme_exponents(orc, gpu, l2):
    """The tile kernels divide bf16 columns through a per-position reciprocal; outside its proven range (denominators
    beyond [2^-30, 2^30], results below 2^-28, zeros of either sign, denormals, inf, NaN) they must fall back to the
    division and still give the reference's bits.  Every position of this tensor is one such case."""
    be, ops = gpu
    from vrhino_b200 import synth
    shape = (1, 64, 1, 4, 16)                         # 64 positions, tile path
    x = synth.normal(shape, 0.0, 1.0, seed=77).reshape(64, 64)        # [channel, position]
    scale = lambda position, factor: x.__setitem__((slice(None), position), x[:, position] * np.float32(factor))
    scale(1, 2.0 ** -40); scale(2, 2.0 ** 40); scale(3, 2.0 ** -100); scale(4, 2.0 ** 100); scale(5, 2.0 ** -120)
    scale(6, 2.0 ** 62); scale(7, 2.0 ** -29); scale(8, 2.0 ** 29.5)
    x[:, 9] = 0.0; x[::2, 9] = -0.0                    # all zeros, both signs
    x[:, 10] = 0.0; x[5, 10] = 3.0; x[6, 10] = -0.0    # zeros beside one value
    x[:, 11] *= np.float32(2.0 ** -130)                # bf16 denormals
    x[3, 12] = np.inf
    x[3, 13] = np.nan
    x[3, 14] = np.float32(2.0 ** 90); x[4, 14] = np.float32(2.0 ** -90)   # huge and tiny in one position
    x[3, 15] = np.float32(2.0 ** 20); x[4:, 15] *= np.float32(2.0 ** -20)  # quotients near the 2^-28 floor
    x[3, 16] = np.float32(2.0 ** 25); x[4:, 16] *= np.float32(2.0 ** -10)
    x[:, 17] = np.float32(3.3895314e38)                # the largest bf16: the sum of squares overflows
    t = orc.tensor(x.reshape(shape), "bf16")
    obe = orc.OracleBackend()
    with np.errstate(all="ignore"):
        want = obe.l2_normalize(t, 1, 1e-10) if l2 else obe.pixel_norm(t, 1, 1e-8)
    got = be.l2_normalize(to_torch(t), 1, 1e-10) if l2 else be.pixel_norm(to_torch(t), 1, 1e-8)
    g = got.view(__import__("torch").int16).cpu().numpy().view(np.uint16).reshape(64, 64)
    w = want.data.reshape(64, 64)
    nan = lambda b: (b & 0x7FFF) > 0x7F80
    same = (g == w) | (nan(g) & nan(w))
    if l2:      # the sums are added in a different order there: compare the cases, not the last bit
        d = orc.bf16_ulp_distance(g, w)
        same |= d <= 2
    assert same.all(), f"positions {sorted(set(np.argwhere(~same)[:, 1].tolist()))} differ"


@pytest.mark.parametrize("shape", [(2, 128, 3, 8, 16), (1, 64, 1, 5, 8), (1, 1024, 2, 4, 12), (1, 512, 1, 7, 24), (3, 96, 2, 6, 40), (1, 4000, 1, 1, 16)])
@pytest.mark.parametrize("dt", ["bf16", "f32"])
def test_tensor_map_tiles_equal_per_thread_copies(orc, gpu, cuda_lib, shape, dt):
    """The tile kernels (pixel_norm, l2_normalize, the axis RMSNorm) load through tensor maps (cp.async.bulk.tensor + mbarrier) where slab and tile sizes allow, else
    through per-thread 16-byte copies: the same bits either way, on full and ragged tiles, one and several slabs of
    channels, and no bounded wait may have run out."""
    import ctypes
    import torch
    be, ops = gpu
    from vrhino_b200 import synth
    x = to_torch(orc.tensor(synth.normal(shape, 0.2, 1.5, seed=shape[1] + 1), dt))
    vec = (shape[0], shape[1], 1, 1, 1)
    shift, scale = to_torch(orc.tensor(synth.normal(vec, 0, 0.2, seed=1))), to_torch(orc.tensor(synth.normal(vec, 0, 0.2, seed=2)))
    gamma = to_torch(orc.tensor(synth.normal((shape[1],), 1.0, 0.1, seed=3)))

    def run():
        return [be.pixel_norm(x, 1, 1e-8), be.l2_normalize(x, 1, 1e-10), ops.fused_pixel_norm_modulate(be, x, shift, scale, 1e-8),
                ops.fused_pixel_norm_modulate(be, x, shift, scale, 1e-8, out_dtype=torch.bfloat16),
                ops.fused_pixel_norm_modulate(be, x, shift, scale, 1e-8, silu=False),
                be.rms_norm(x, gamma, 1e-12, 1), ops.fused_rms_channel_silu(be, x, gamma, 1e-12)]

    previous = cuda_lib.vrb_set_tensor_map_tiles(1)
    try:
        with_maps = run()
        cuda_lib.vrb_set_tensor_map_tiles(0)
        without = run()
    finally:
        cuda_lib.vrb_set_tensor_map_tiles(previous)
    bits = lambda t: t.view(torch.int16 if t.dtype == torch.bfloat16 else torch.int32)
    for a, b in zip(with_maps, without):
        assert torch.equal(bits(a), bits(b))
    failures = ctypes.c_int(-1)
    assert cuda_lib.vrb_async_wait_failures(ctypes.byref(failures)) == 0 and failures.value == 0


def test_rms_channel_silu_over_every_bf16_argument(gpu):
    """The axis RMSNorm's fused SiLU takes a bf16 argument: with x = 1 everywhere the normalised value is exactly 1 and
    the argument of channel c is weight[c], so a weight vector running through all 65536 bf16 codes drives every
    argument through the kernel; the result must be SiLU of that bf16 value as vrb_activation gives it."""
    import torch
    be, ops = gpu
    channels = 2048
    x = torch.ones(1, channels, 1, 1, 8, device="cuda", dtype=torch.bfloat16)
    for start in range(0, 1 << 16, channels):
        codes = torch.arange(start, start + channels, device="cuda", dtype=torch.int32)
        w = codes.to(torch.int16).view(torch.bfloat16)
        got = ops.fused_rms_channel_silu(be, x, w.float(), 1e-12)
        want = be.activation(w, ops.SILU)
        g, e = got.view(channels, 8).view(torch.int16), want.view(torch.int16)
        nan = lambda t: (t & 0x7FFF) > 0x7F80
        same = (g[:, 0] == e) | (nan(g[:, 0]) & nan(e))
        assert bool(same.all()) and bool((g == g[:, :1]).all()), f"codes {codes[~same][:8].tolist()} differ"


def test_bf16_store_silu_over_every_f32_argument(gpu):
    """pixel_norm -> modulate -> SiLU with a bf16 result evaluates SiLU through approximate special functions wherever
    the bf16 rounding provably cannot differ, else exactly.  All 2^32 F32 arguments go through the kernel here: with
    x = 0 and scale = 0 the SiLU argument of channel c is shift[c] bit for bit, and the result must be the bf16
    rounding of the exact expression (vrb_activation on F32, then vrb_cast)."""
    import torch
    be, ops = gpu
    outer, channels, inner, per_call = 32768, 2048, 8, 1 << 26
    x = torch.zeros(outer, channels, 1, 1, inner, device="cuda", dtype=torch.bfloat16)
    scale = torch.zeros(outer, channels, 1, 1, 1, device="cuda")
    index = torch.arange(per_call, device="cuda", dtype=torch.int64)
    out = torch.empty_like(x)
    mismatches, examples = 0, []
    for call in range((1 << 32) // per_call):
        bits = index + call * per_call
        bits = torch.where(bits >= (1 << 31), bits - (1 << 32), bits).to(torch.int32)
        v = bits.view(torch.float32)
        got = ops.fused_pixel_norm_modulate(be, x, v.view(outer, channels, 1, 1, 1), scale, 1e-8, out_dtype=torch.bfloat16, out=out)
        # the kernel's argument is 0 * 1 + shift: -0 arrives as +0 (every other argument unchanged)
        want = be.cast(be.activation(v + 0.0, ops.SILU), torch.bfloat16).view(outer, channels)
        g = got.view(outer, channels, inner).view(torch.int16)
        w = want.view(torch.int16)
        wrong = (g[:, :, 0] != w) | (g[:, :, inner - 1] != w)
        count = int(wrong.sum())
        if count:
            mismatches += count
            at = wrong.view(-1).nonzero().view(-1)[:4]
            examples += [(hex(int(bits[i]) & 0xFFFFFFFF), hex(int(g[:, :, 0].reshape(-1)[i]) & 0xFFFF), hex(int(w.reshape(-1)[i]) & 0xFFFF))
                         for i in at.tolist()]
    assert mismatches == 0, f"{mismatches} arguments round to another bf16 value, e.g. (argument, got, want) {examples[:8]}"


@pytest.mark.parametrize("shape", [s for s in SHAPES if len(s) == 5])
@pytest.mark.parametrize("dt", ["bf16", "f32"])
def test_pixel_norm_modulate_silu(orc, gpu, shape, dt):
    import torch
    be, ops = gpu
    from vrhino_b200 import synth
    obe, pol = orc.OracleBackend(), orc.Policy()
    vec = (shape[0], shape[1], 1, 1, 1)
    x = orc.tensor(synth.normal(shape, 0.2, 1.5, seed=shape[1]), dt)
    shift, scale = orc.tensor(synth.normal(vec, 0, 0.2, seed=1)), orc.tensor(synth.normal(vec, 0, 0.2, seed=2))
    mod = orc.modulate(obe, pol, obe.pixel_norm(x, 1, 1e-8), shift, scale)
    got = ops.fused_pixel_norm_modulate(be, to_torch(x), to_torch(shift), to_torch(scale), 1e-8, silu=False)
    assert_bits_equal(got, mod, "pixel_norm + modulate")
    act = obe.activation(mod, orc.SILU)
    got = ops.fused_pixel_norm_modulate(be, to_torch(x), to_torch(shift), to_torch(scale), 1e-8)
    assert_close(orc, got, act, rel=1e-5, atol=2e-6, what="pixel_norm + modulate + silu")
    # the merged form equals this library's own operator chain bit for bit, in both output dtypes
    chain = be.activation(ops.modulate(be, ops.Policy(), be.pixel_norm(to_torch(x), 1, 1e-8), to_torch(shift), to_torch(scale)), ops.SILU)
    assert torch.equal(got.view(torch.int32), chain.view(torch.int32))
    got16 = ops.fused_pixel_norm_modulate(be, to_torch(x), to_torch(shift), to_torch(scale), 1e-8, out_dtype=torch.bfloat16)
    assert torch.equal(got16.view(torch.int16), be.cast(chain, torch.bfloat16).view(torch.int16))


def test_pixel_norm_other_axes_and_errors(orc, gpu):
    import torch
    be, ops = gpu
    from vrhino_b200 import synth
    x = orc.tensor(synth.normal((4, 6, 40), seed=3), "f32")
    obe = orc.OracleBackend()
    assert_bits_equal(be.pixel_norm(to_torch(x), -1, 1e-8), obe.pixel_norm(x, -1, 1e-8), "last axis")
    assert_bits_equal(be.pixel_norm(to_torch(x), 0, 1e-6), obe.pixel_norm(x, 0, 1e-6), "first axis")
    with pytest.raises(ops.VrbError):
        be.pixel_norm(to_torch(x), 3, 1e-8)
    with pytest.raises(ops.VrbError):
        ops.fused_pixel_norm_modulate(be, to_torch(x), torch.zeros(4, 5, 1, device="cuda"), torch.zeros(4, 5, 1, device="cuda"))


@pytest.mark.parametrize("shape", SHAPES + [(1, 512, 38, 38), (2, 256, 19, 24)])      # + the detector's feature maps
@pytest.mark.parametrize("dt", ["bf16", "f32"])
def test_l2_normalize(orc, gpu, shape, dt):
    """CudaBackend::l2_normalize: x / (sqrt(sum of squares over the channels) + eps).  The kernels add the
    squares in the tile kernels' order, the reference (and the oracle) in its 256-thread tree: <= 2 bf16 ulp /
    1e-5 relative, and within this library inner == 1 and inner > 1 must agree with a permuted call."""
    be, ops = gpu
    from vrhino_b200 import synth
    x = orc.tensor(synth.normal(shape, 0.2, 1.5, seed=shape[1]), dt)
    want = orc.OracleBackend().l2_normalize(x, 1, 1e-10)
    got = be.l2_normalize(to_torch(x), 1, 1e-10)
    assert_close(orc, got, want, max_ulp=2, rel=1e-5, what=f"l2_normalize {shape} {dt}")
    with pytest.raises(ops.VrbError, match="l2 normalize contract violation"):
        be.l2_normalize(to_torch(x), len(shape), 1e-10)
    with pytest.raises(ops.VrbError, match="l2 normalize contract violation"):
        be.l2_normalize(to_torch(x), 1, -1.0)
