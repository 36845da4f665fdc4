"""Layout operators of the C ABI (vrb_permute / vrb_slice / vrb_concat / vrb_pad / vrb_sinusoidal_embedding) against
the oracle: copies bit for bit over every kernel path (16-byte, 4-byte and element units; compile-time and
run-time ranks; transposition tiles with ragged edges; 64-bit indexing), the reference's argument rules and
error texts (cuda_backend.cu:3936-3970, :4190-4196, :4875-4883), and the embedding within the host-libm bound."""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu


def _dev(torch, a, dt):
    if dt == "bf16":
        from vrhino_b200 import synth
        return torch.from_numpy(synth.to_bf16_bits(a).view(np.int16).copy()).view(torch.bfloat16).cuda()
    return torch.from_numpy(np.ascontiguousarray(a, dtype=np.float32)).cuda()


def _bits(torch, t):
    t = t.detach().cpu().contiguous()
    return t.view(torch.int16).numpy().view(np.uint16) if t.dtype == torch.bfloat16 else t.numpy().view(np.uint32)


def _orc_bits(t):
    return t.data if t.dtype == "bf16" else t.data.view(np.uint32)


def _pair(orc, torch, shape, dt, seed):
    from vrhino_b200 import synth
    a = synth.normal(shape, seed=seed)
    return _dev(torch, a, dt), orc.tensor(a, dt)


PERMUTES = [
    ((2, 6, 3, 4, 16), (0, 2, 1, 3, 4)),          # inner axes kept: 16-byte units
    ((3, 5, 7), (1, 0, 2)),                       # inner axis kept, odd extent: element units
    ((1, 1536, 333), (0, 2, 1)),                  # patch embedding: tiles, ragged in one direction
    ((2, 70, 130), (0, 2, 1)),                    # tiles ragged in both
    ((1, 24, 2, 5, 7), (0, 2, 3, 4, 1)),          # channels last
    ((1, 2, 5, 7, 24), (0, 4, 1, 2, 3)),          # and back
    ((1, 2, 3, 4, 1, 2, 2, 16), (0, 7, 1, 4, 2, 5, 3, 6)),   # Wan unpatchify, rank 8
    ((2, 3, 4, 5, 6), (4, 3, 2, 1, 0)),           # full reversal: short tile sides, element walk
    ((4, 9), (0, 1)),                             # identity
    ((7,), (0,)),
    ((2, 1, 40, 1, 24), (3, 2, 0, 1, 4)),         # extent-1 axes moved around
]


@pytest.mark.parametrize("dt", ["bf16", "f32"])
@pytest.mark.parametrize("shape,dims", PERMUTES, ids=[f"{s}->{d}".replace(" ", "") for s, d in PERMUTES])
def test_permute(orc, gpu, shape, dims, dt):
    import torch
    be, _ = gpu
    x, ox = _pair(orc, torch, shape, dt, 3)
    got = be.permute(x, dims)
    want = orc.OracleBackend().permute(ox, dims)
    assert tuple(got.shape) == want.shape
    assert np.array_equal(_bits(torch, got), _orc_bits(want))


SLICES = [
    ((1, 20, 64), 2, 0, 32), ((1, 20, 64), 2, 32, 64), ((1, 20, 64), 2, 3, 10), ((2, 9, 24), 1, 2, 7), ((2, 9, 24), 0, 1, 2),
    ((2, 9, 24), -1, -5, 100), ((2, 9, 24), 1, -100, 3), ((2, 9, 24), 1, 4, 4), ((2, 9, 24), 2, 30, 40), ((5, 6, 12), 2, 4, 12),
    ((3, 4, 5, 6, 7, 2, 3, 4), 4, 2, 6), ((64,), 0, 8, 24),
    ((4, 300), 1, 3, 250), ((2, 3, 1000), 2, 1, 999), ((5, 129), 1, 0, 65),      # long rows at odd offsets: the row form
]


@pytest.mark.parametrize("dt", ["bf16", "f32"])
@pytest.mark.parametrize("shape,dim,start,stop", SLICES, ids=[f"{s}[{d}:{a}:{b}]".replace(" ", "") for s, d, a, b in SLICES])
def test_slice(orc, gpu, shape, dim, start, stop, dt):
    import torch
    be, _ = gpu
    x, ox = _pair(orc, torch, shape, dt, 4)
    got = be.slice(x, dim, start, stop)
    want = orc.OracleBackend().slice(ox, dim, start, stop)
    assert tuple(got.shape) == want.shape
    assert np.array_equal(_bits(torch, got), _orc_bits(want))


@pytest.mark.parametrize("dt", ["bf16", "f32"])
def test_row_copies_at_every_pair_of_phases(orc, gpu, dt):
    """Long rows whose two sides start at every combination of offsets inside a 16-byte chunk (the row length moves
    the output side from row to row, the slice's start moves the source side), as a slice and under a pad."""
    import torch
    be, _ = gpu
    obe = orc.OracleBackend()
    x, ox = _pair(orc, torch, (9, 211), dt, 41)
    for start in range(9):
        for length in (64, 65, 71, 78, 200):
            got, want = be.slice(x, 1, start, start + length), obe.slice(ox, 1, start, start + length)
            assert np.array_equal(_bits(torch, got), _orc_bits(want)), (start, length)
    for width in (66, 67, 69, 72):
        y, oy = _pair(orc, torch, (5, 3, width), dt, 42 + width)
        for left, right in ((1, 1), (2, 0), (0, 3), (5, 8)):
            for replicate in (False, True):
                got, want = be.pad(y, [left, right], -0.5, replicate), obe.pad(oy, [left, right], -0.5, replicate)
                assert np.array_equal(_bits(torch, got), _orc_bits(want)), (width, left, right, replicate)


@pytest.mark.parametrize("dt", ["bf16", "f32"])
def test_inner_runs_of_whole_2_kb_blocks(orc, gpu, dt):
    """Padded walks whose innermost axis is a contiguous run of a multiple of 2 KB on both sides take the block form (a
    warp per 2 KB block): pads of outer axes in both modes -- and, on the unit walk, permutes that keep the inner axes,
    slices and concats of outer axes -- with row counts around and beyond one pass of the grid."""
    import torch
    be, _ = gpu
    obe = orc.OracleBackend()
    inner = 1024 if dt == "bf16" else 512                       # 2 KB
    for shape in ((2, 5, 3, inner), (3, 7, 2 * inner), (1, 37, 11, 3 * inner)):
        x, ox = _pair(orc, torch, shape, dt, 51)
        rank = len(shape)
        for padding, replicate in (((0, 0) * (rank - 2) + (2, 1), True), ((0, 0) * (rank - 2) + (2, 1), False),
                                   ((0, 0) * (rank - 2) + (0, 3, 1, 0), False), ((0, 0) * (rank - 2) + (1, 1, 1, 1), True)):
            got, want = be.pad(x, list(padding), 0.25, replicate), obe.pad(ox, list(padding), 0.25, replicate)
            assert np.array_equal(_bits(torch, got), _orc_bits(want)), (shape, padding, replicate)
        dims = (1, 0) + tuple(range(2, rank))
        assert np.array_equal(_bits(torch, be.permute(x, dims)), _orc_bits(obe.permute(ox, dims))), shape
        assert np.array_equal(_bits(torch, be.slice(x, 1, 1, shape[1] - 1)), _orc_bits(obe.slice(ox, 1, 1, shape[1] - 1))), shape
        assert np.array_equal(_bits(torch, be.concat([x, x, x], 1)), _orc_bits(obe.concat([ox, ox, ox], 1))), shape
    # more blocks than one pass of the grid takes: [40, 257, 4 KB] -> 20560 blocks
    x, ox = _pair(orc, torch, (40, 257, 2 * inner), dt, 52)
    assert np.array_equal(_bits(torch, be.pad(x, [0, 0, 1, 2], 0.0, True)), _orc_bits(obe.pad(ox, [0, 0, 1, 2], 0.0, True)))
    assert np.array_equal(_bits(torch, be.permute(x, (1, 0, 2))), _orc_bits(obe.permute(ox, (1, 0, 2))))


@pytest.mark.parametrize("dt", ["bf16", "f32"])
def test_split_and_concat(orc, gpu, dt):
    import torch
    be, _ = gpu
    obe = orc.OracleBackend()
    x, ox = _pair(orc, torch, (2, 10, 48), dt, 5)
    for dim, sections in ((2, (16, 32)), (-1, (5, 43)), (1, (3, 3, 4)), (0, (1, 1))):
        parts, want = be.split(x, list(sections), dim), obe.split(ox, list(sections), dim)
        for g, w in zip(parts, want):
            assert np.array_equal(_bits(torch, g), _orc_bits(w))
        back = be.concat(parts, dim)
        assert torch.equal(back.view(torch.int16 if dt == "bf16" else torch.int32), x.view(torch.int16 if dt == "bf16" else torch.int32))
        assert np.array_equal(_bits(torch, back), _orc_bits(obe.concat(want, dim)))
    a, oa = _pair(orc, torch, (3, 4, 1, 5), dt, 6)
    b, ob = _pair(orc, torch, (3, 4, 3, 5), dt, 7)
    assert np.array_equal(_bits(torch, be.concat([a, b, a], 2)), _orc_bits(obe.concat([oa, ob, oa], 2)))
    from vrhino_b200._lib import VrbError
    with pytest.raises(VrbError, match="concat shape mismatch"):
        be.concat([a, x[:, :4].contiguous().reshape(2, 4, 1, 48)], 2)
    with pytest.raises(VrbError, match="concat requires inputs"):
        be.concat([], 0)
    with pytest.raises(VrbError, match="split sections mismatch"):
        be.split(x, [1, 2], 1)


PADS = [
    ((1, 8, 3, 6, 16), (0, 0, 0, 0, 2, 2), 0.0, True),       # LTX causal padding: 16-byte units, rank 3 after merging
    ((1, 8, 3, 6, 16), (0, 0, 0, 0, 1, 0), 0.5, False),
    ((1, 4, 2, 5, 7), (1, 1, 1, 1), 0.0, False),             # spatial: element units
    ((1, 4, 2, 5, 7), (1, 2, 0, 1, 2, 0), -1.3, False),
    ((1, 4, 2, 5, 7), (1, 2, 0, 1, 2, 0), 0.0, True),
    ((2, 3, 2, 5, 7), (1, 0, 1, 0, 1, 0, 1, 0, 1, 0), 2.0, False),   # every axis: run-time rank
    ((1, 2), (1, 2), 0.0, True),
    ((6, 40), (0, 8), 1.0, False),                           # inner axis by a multiple of the unit
    ((2, 3, 70), (3, 2), -2.5, False),                       # long padded rows: the row form
    ((2, 3, 70), (3, 2, 1, 1), 0.0, True),
    ((1, 2, 3, 130), (1, 0, 0, 0, 2, 1), 0.25, False),
    ((3, 5, 4), (40, 40), 0.75, False),                      # a source row shorter than one 16-byte chunk inside a long output row
    ((3, 5, 4), (40, 40), 0.0, True),
    ((2, 7, 90), (9, 17), 0.0, True),                        # replicated pads wider than a chunk
    ((40, 33, 67), (1, 1, 1, 1), 0.0, False),                # more rows than one warp's group
    ((2, 3, 5), (0, 0), 0.0, False),                         # nothing to do
    ((2, 3, 5), (), 0.0, False),
]


@pytest.mark.parametrize("dt", ["bf16", "f32"])
@pytest.mark.parametrize("shape,padding,value,replicate", PADS, ids=[f"{s}+{p}{'r' if r else 'c'}".replace(" ", "") for s, p, v, r in PADS])
def test_pad(orc, gpu, shape, padding, value, replicate, dt):
    import torch
    be, _ = gpu
    x, ox = _pair(orc, torch, shape, dt, 8)
    got = be.pad(x, list(padding), value, replicate)
    want = orc.OracleBackend().pad(ox, list(padding), value, replicate)
    assert tuple(got.shape) == want.shape
    assert np.array_equal(_bits(torch, got), _orc_bits(want))


@pytest.mark.parametrize("dt", ["bf16", "f32"])
@pytest.mark.parametrize("shape,temporal,pad_h,pad_w", [((1, 8, 3, 6, 16), 1, 1, 1), ((2, 3, 2, 5, 7), 2, 1, 2), ((1, 4, 1, 4, 8), 1, 0, 0),
                                                        ((1, 4, 5, 4, 8), 0, 1, 1), ((1, 2, 3, 9, 24), 1, 1, 0)])
def test_edge_time_pad_equals_the_two_pads(orc, gpu, shape, temporal, pad_h, pad_w, dt):
    """vrb_pad_axes: replicate along T and zeros around H, W in one pass == the reference's two pads in their order."""
    import torch
    be, ops = gpu
    x, ox = _pair(orc, torch, shape, dt, 9)
    obe = orc.OracleBackend()
    want = obe.pad(obe.pad(ox, [0, 0, 0, 0, temporal, temporal], 0.0, True), [pad_w, pad_w, pad_h, pad_h], 0.0, False)
    got = ops.fused_edge_time_pad(be, x, temporal, pad_h, pad_w)
    assert tuple(got.shape) == want.shape
    assert np.array_equal(_bits(torch, got), _orc_bits(want))
    two = be.pad(be.pad(x, [0, 0, 0, 0, temporal, temporal], 0.0, True), [pad_w, pad_w, pad_h, pad_h], 0.0, False)
    assert np.array_equal(_bits(torch, got), _bits(torch, two))


NEAREST = [
    ((3, 4, 6, 16), (2.0, 2.0)),            # doubled width and height: 16 bytes in, 2 x 32 bytes out
    ((3, 4, 6, 16), (1.0, 2.0)),            # doubled width only
    ((2, 3, 5, 8), (2.0, 2.0)),
    ((1, 2, 3, 5), (2.0, 2.0)),             # odd width: a warp per row
    ((1, 2, 3, 5, 7), (2.0, 2.0, 2.0)),     # three resized axes
    ((1, 2, 3, 5, 7), (1.0, 2.0, 2.0)),
    ((1, 2, 3, 5, 7), (1.5, 0.5)),          # fractional factors, shrinking
    ((1, 1, 24), (0.5,)), ((1, 1, 24), (3.0,)), ((2, 3, 40), (2.0,)),
    ((1, 2, 3, 5), (2.5, 1.4)),
]


@pytest.mark.parametrize("dt", ["bf16", "f32"])
@pytest.mark.parametrize("shape,factors", NEAREST, ids=[f"{s}x{f}".replace(" ", "") for s, f in NEAREST])
def test_interpolate_nearest(orc, gpu, shape, factors, dt):
    import torch
    be, _ = gpu
    x, ox = _pair(orc, torch, shape, dt, 10)
    got = be.interpolate_nearest(x, list(factors))
    want = orc.OracleBackend().interpolate_nearest(ox, list(factors))
    assert tuple(got.shape) == want.shape
    assert np.array_equal(_bits(torch, got), _orc_bits(want))


def test_interpolate_nearest_at_size_and_rules(gpu):
    """The Wan VAE's 2x spatial upsampling of [frames, C, H, W] (wan.cpp:266-268) against torch's nearest resize, in
    both dtypes; the reference's argument rules."""
    import torch
    from vrhino_b200._lib import VrbError
    be, _ = gpu
    x = torch.randn(6, 96, 120, 208, device="cuda")
    for t in (x, x.to(torch.bfloat16)):
        got = be.interpolate_nearest(t, [2.0, 2.0])
        want = torch.nn.functional.interpolate(t, scale_factor=2.0, mode="nearest")
        assert torch.equal(got, want)
        assert torch.equal(be.interpolate_nearest(t, [1.0, 2.0]), torch.nn.functional.interpolate(t, scale_factor=(1.0, 2.0), mode="nearest"))
    with pytest.raises(VrbError, match="interpolate factor rank mismatch"):
        be.interpolate_nearest(x, [2.0, 2.0, 2.0])
    with pytest.raises(VrbError, match="Invalid interpolation factor"):
        be.interpolate_nearest(x, [0.0, 2.0])


@pytest.mark.parametrize("dt", ["bf16", "f32"])
@pytest.mark.parametrize("shape,dim,keep", [((2, 37, 64), 1, True), ((2, 37, 64), -1, False), ((2, 37, 64), 0, False), ((3, 5, 7), 1, False),
                                            ((3, 5, 7), 2, True), ((1, 256, 1536), 1, True), ((4, 1, 9), 1, False), ((2, 6), 1, False)])
def test_reduce_sum(orc, gpu, shape, dim, keep, dt):
    """F32 accumulation in index order, like the reference's one-thread-per-output loop: the same bits."""
    import torch
    be, _ = gpu
    x, ox = _pair(orc, torch, shape, dt, 11)
    got = be.reduce_sum(x, dim, keep)
    want = orc.OracleBackend().reduce_sum(ox, dim, keep)
    assert tuple(got.shape) == want.shape
    assert np.array_equal(_bits(torch, got), _orc_bits(want))


@pytest.mark.parametrize("dt", ["bf16", "f32"])
@pytest.mark.parametrize("shape,axis", [((3, 5, 77), -1), ((3, 5, 77), 1), ((3, 5, 77), 0), ((2, 19, 6, 4), 1), ((4, 1100), 1), ((6, 1), 1),
                                        ((2, 32), -1), ((1, 33), -1), ((600, 512), 1)])
def test_softmax(orc, gpu, shape, axis, dt):
    """Maximum, denominator in index order, quotient: the oracle differs from the device only by its host expf."""
    import torch
    be, _ = gpu
    from vrhino_b200 import synth
    scores = (synth.normal(shape, seed=12) * 3.0).astype(np.float32)
    x, ox = _dev(torch, scores, dt), orc.tensor(scores, dt)
    got = be.softmax(x, axis)
    want = orc.OracleBackend().softmax(ox, axis)
    assert tuple(got.shape) == want.shape
    if dt == "bf16":
        assert int(orc.bf16_ulp_distance(_bits(torch, got), _orc_bits(want)).max()) <= 1
    else:
        assert np.allclose(got.cpu().numpy(), want.f32(), rtol=2e-6, atol=1e-9)
    total = got.float().sum(dim=axis)
    assert torch.allclose(total, torch.ones_like(total), atol=2e-2 if dt == "bf16" else 1e-5)
    # the primitive tests' known answers (primitive_tests.cpp:523-524)
    kat = be.softmax(torch.tensor([[80.0, 81.0], [-80.0, -79.0]], device="cuda"), -1).cpu().numpy().reshape(-1)
    assert np.allclose(kat, [0.26894143, 0.7310586, 0.26894143, 0.7310586], atol=2e-5)


@pytest.mark.parametrize("dt", ["bf16", "f32"])
def test_indexed_gather(orc, gpu, dt):
    import torch
    from vrhino_b200._lib import VrbError
    from vrhino_b200 import ops as vops
    be = vops.B200Backend(execution_dtype=torch.bfloat16 if dt == "bf16" else torch.float32)
    obe = orc.OracleBackend(execution_dtype=dt)
    rng = np.random.default_rng(3)
    for shape, index_shape, itype in (((50, 64), (2, 5), np.int64), ((50, 64), (7,), np.int32), ((9, 7), (3,), np.int64),
                                      ((1000, 4096), (2, 512), np.int64), ((33, 6), (4, 4), np.int32), ((5, 8), (0,), np.int64)):
        table, otable = _pair(orc, torch, shape, dt, 13)
        indices = rng.integers(0, shape[0], size=index_shape).astype(itype)
        got, want = be.indexed_gather(table, indices), obe.indexed_gather(otable, indices)
        assert tuple(got.shape) == want.shape == tuple(index_shape) + (shape[1],)
        assert np.array_equal(_bits(torch, got), _orc_bits(want))
        assert np.array_equal(_bits(torch, be.indexed_gather(table, torch.from_numpy(indices).cuda())), _orc_bits(want))   # indices on the device
    table, otable = _pair(orc, torch, (3, 11, 24), dt, 14)                    # a table per batch entry
    for index_shape in ((3, 4), (3, 2, 5)):
        indices = rng.integers(0, 11, size=index_shape).astype(np.int64)
        got, want = be.indexed_gather(table, indices), obe.indexed_gather(otable, indices)
        assert np.array_equal(_bits(torch, got), _orc_bits(want))
    # a table of the other dtype is converted to the execution dtype first (copy_to_device, cuda_backend.cu:4032)
    other = "f32" if dt == "bf16" else "bf16"
    table, otable = _pair(orc, torch, (12, 16), other, 15)
    indices = np.array([11, 0, 5], dtype=np.int64)
    assert np.array_equal(_bits(torch, be.indexed_gather(table, indices)), _orc_bits(obe.indexed_gather(otable, indices)))
    with pytest.raises(VrbError, match="index out of range"):
        be.indexed_gather(table, np.array([12], dtype=np.int64))
    with pytest.raises(VrbError, match="index out of range"):
        be.indexed_gather(table, np.array([-1], dtype=np.int32))
    with pytest.raises(VrbError, match="rank 2 or 3"):
        be.indexed_gather(table.reshape(-1), indices)
    with pytest.raises(VrbError, match="int64/int32"):
        be.indexed_gather(table, np.array([1.0], dtype=np.float32))
    with pytest.raises(VrbError, match="batch dimension mismatch"):
        be.indexed_gather(table.reshape(2, 6, 16), np.zeros((3, 2), dtype=np.int64))


@pytest.mark.parametrize("dt", ["bf16", "f32"])
def test_rng_normal(orc, gpu, dt):
    """The reference's Philox stream: its known answers (primitive_tests.cpp:549), the oracle's restatement (host
    log / sin: a few F32 ulp), the offset bookkeeping, and the moments of a latent-sized draw."""
    import torch
    from vrhino_b200._lib import VrbError
    from vrhino_b200 import ops as vops
    be, _ = gpu
    tdt = torch.bfloat16 if dt == "bf16" else torch.float32
    state = vops.RngState(5701, 0)
    got = be.rng_normal(state, (8,), tdt)
    want = [-1.1955757141, .5111286044, -1.0140079260, -.4857170284, -.2519632876, -1.9857326746, 1.1355758905, .4264008999]
    assert state.offset == 4
    assert np.allclose(got.float().cpu().numpy(), want, atol=1e-6 if dt == "f32" else 8e-3)
    for seed, offset, shape in ((5701, 4, (2, 256)), (2 ** 63 + 11, 4000, (1, 16, 21, 60, 104)), (0, 0, (3,))):
        mine, theirs = vops.RngState(seed, offset), vops.RngState(seed, offset)
        got = be.rng_normal(mine, shape, tdt)
        want = orc.OracleBackend().rng_normal(theirs, shape, dt)
        assert mine.offset == theirs.offset == offset + 4 and tuple(got.shape) == want.shape
        diff = np.abs(got.float().cpu().numpy().astype(np.float64) - want.f32().astype(np.float64))
        bound = 2e-5 + (2.0 ** -7 * np.abs(want.f32().astype(np.float64)) if dt == "bf16" else 0.0)   # + one bf16 ulp of the value
        assert (diff <= bound).all(), diff.max()
    latent = be.rng_normal(vops.RngState(7, 0), (1, 16, 21, 60, 104), tdt).float()
    assert abs(float(latent.mean())) < 5e-3 and abs(float(latent.std()) - 1.0) < 5e-3
    again = be.rng_normal(vops.RngState(7, 0), (1, 16, 21, 60, 104), tdt).float()
    assert torch.equal(latent, again)
    assert not torch.equal(latent, be.rng_normal(vops.RngState(7, 4), (1, 16, 21, 60, 104), tdt).float())
    with pytest.raises(VrbError, match="Unsupported RNG algorithm"):
        be.rng_normal(vops.RngState(1, 0, "mt19937"), (4,), tdt)
    with pytest.raises(VrbError, match="dtype unsupported"):
        be.rng_normal(vops.RngState(1, 0), (4,), torch.float16)


def test_argument_rules(orc, gpu):
    import torch
    from vrhino_b200._lib import VrbError
    be, _ = gpu
    x = torch.zeros(2, 3, 4, device="cuda")
    with pytest.raises(VrbError, match="permute rank mismatch"):
        be.permute(x, (0, 1))
    with pytest.raises(VrbError, match="Invalid permutation"):
        be.permute(x, (0, 1, 1))
    with pytest.raises(VrbError, match="slice dimension invalid"):
        be.slice(x, 3, 0, 1)
    with pytest.raises(VrbError, match="Invalid pad vector"):
        be.pad(x, [1, 1, 1])
    with pytest.raises(VrbError, match="Negative padding unsupported"):
        be.pad(x, [0, -1])
    with pytest.raises(VrbError, match="reduce dimension invalid"):
        be.reduce_sum(x, 3)
    with pytest.raises(VrbError, match="sinusoidal embedding contract violation"):
        be.sinusoidal_embedding(x, 8, True, 0.0, False)
    assert be.slice(x, 1, 2, 1).shape == (2, 0, 4)       # an empty range launches nothing


def test_raw_entry_point_checks(gpu, cuda_lib):
    """The C entry points refuse what the wrappers would not pass on."""
    import ctypes
    import torch
    x = torch.zeros(4, 4, device="cuda")
    out = torch.zeros(4, 4, device="cuda")
    P, I = ctypes.c_void_p, ctypes.c_int64
    shape = (I * 2)(4, 4)
    bad = (I * 2)(0, 0)
    assert cuda_lib.vrb_permute(P(x.data_ptr()), P(out.data_ptr()), 0, 2, shape, bad, None) != 0
    assert b"Invalid permutation" in cuda_lib.vrb_last_error()
    assert cuda_lib.vrb_permute(P(x.data_ptr()), P(out.data_ptr()), 0, 9, shape, bad, None) != 0
    neg = (I * 2)(0, -1)
    zero = (I * 2)(0, 0)
    assert cuda_lib.vrb_pad(P(x.data_ptr()), P(out.data_ptr()), 0, 2, shape, neg, zero, ctypes.c_float(0), 0, None) != 0
    assert b"Negative padding unsupported" in cuda_lib.vrb_last_error()
    ptrs = (ctypes.c_void_p * 1)(x.data_ptr())
    ext = (I * 1)(3)
    assert cuda_lib.vrb_concat(ptrs, ext, 1, P(out.data_ptr()), 0, 2, shape, 0, None) != 0
    assert b"concat shape mismatch" in cuda_lib.vrb_last_error()
    U = ctypes.c_uint64
    assert cuda_lib.vrb_softmax(P(x.data_ptr()), P(out.data_ptr()), 5, I(4), I(4), I(1), None) != 0          # a dtype that is not a float type
    assert cuda_lib.vrb_softmax(None, P(out.data_ptr()), 0, I(4), I(4), I(1), None) != 0
    assert cuda_lib.vrb_softmax(None, None, 0, I(0), I(4), I(1), None) == 0                                  # nothing to do
    indices = torch.zeros(2, dtype=torch.int64, device="cuda")
    assert cuda_lib.vrb_indexed_gather(P(x.data_ptr()), P(indices.data_ptr()), 0, P(out.data_ptr()), 0, I(0), I(4), I(4), I(2), None) != 0
    assert b"int64/int32" in cuda_lib.vrb_last_error()
    assert cuda_lib.vrb_indexed_gather(P(x.data_ptr()), None, 3, P(out.data_ptr()), 0, I(0), I(4), I(4), I(2), None) != 0
    # an index out of range (the wrappers refuse it earlier) leaves its row unwritten instead of reading outside the table
    indices[1] = 7
    out.fill_(-1.0)
    table = torch.arange(16, dtype=torch.float32, device="cuda").reshape(4, 4) + 1.0
    assert cuda_lib.vrb_indexed_gather(P(table.data_ptr()), P(indices.data_ptr()), 3, P(out.data_ptr()), 0, I(0), I(4), I(4), I(2), None) == 0
    torch.cuda.synchronize()
    assert torch.equal(out[0], table[0]) and bool((out[1:] == -1.0).all())
    assert cuda_lib.vrb_rng_normal(P(out.data_ptr()), 5, I(16), U(1), U(0), None) != 0
    assert b"rng_normal dtype unsupported" in cuda_lib.vrb_last_error()
    assert cuda_lib.vrb_rng_normal(None, 0, I(16), U(1), U(0), None) != 0
    assert cuda_lib.vrb_rng_normal(None, 0, I(0), U(1), U(0), None) == 0


@pytest.mark.parametrize("dt", ["bf16", "f32"])
def test_sinusoidal_embedding(orc, gpu, dt):
    import torch
    be, _ = gpu
    positions = np.array([0.0, 1.0, 0.5, 999.0, 37.25, -2.0, 1000.0, 250.0], dtype=np.float32)
    x, ox = _dev(torch, positions, dt), orc.tensor(positions, dt)
    obe = orc.OracleBackend()
    for width, flip, downscale, f64 in ((256, True, 0.0, False), (7, False, 1.0, False), (320, True, 0.0, True), (6, True, 0.0, False)):
        got = be.sinusoidal_embedding(x, width, flip, downscale, f64).float().cpu().numpy()
        want = obe.sinusoidal_embedding(ox, width, flip, downscale, f64).f32()
        bound = (2e-5 + 2.0 ** -21 * np.abs(ox.f32().astype(np.float64)))[:, None] + (2.0 ** -7 * np.abs(want) if dt == "bf16" else 0.0)
        assert (np.abs(got.astype(np.float64) - want) <= bound).all()
        if width % 2:
            assert (got[:, -1] == 0).all()


def test_large_tensors_use_every_unit_and_wide_indices(orc, gpu):
    """Full-size shapes: the Wan patch embedding transposition, a frames-first permute of a VAE feature map, LTX's causal
    padding, SwiGLU's halves, and one tensor beyond 2^31 elements (64-bit index kernel) -- against torch's own copies."""
    import torch
    be, _ = gpu
    bits = lambda t: t.view(torch.int16)
    x = torch.randn(1, 1536, 32760, device="cuda").to(torch.bfloat16)
    assert torch.equal(bits(be.permute(x, (0, 2, 1))), bits(x.permute(0, 2, 1).contiguous()))
    x = torch.randn(1, 128, 9, 64, 96, device="cuda").to(torch.bfloat16)
    assert torch.equal(bits(be.permute(x, (0, 2, 1, 3, 4))), bits(x.permute(0, 2, 1, 3, 4).contiguous()))
    assert torch.equal(bits(be.permute(x, (0, 2, 3, 4, 1))), bits(x.permute(0, 2, 3, 4, 1).contiguous()))
    padded = be.pad(x, [0, 0, 0, 0, 2, 2], 0.0, True)
    want = torch.cat([x[:, :, :1].expand(-1, -1, 2, -1, -1), x, x[:, :, -1:].expand(-1, -1, 2, -1, -1)], 2)
    assert torch.equal(bits(padded), bits(want.contiguous()))
    spatial = be.pad(x, [1, 1, 1, 1], 0.0, False)
    assert torch.equal(bits(spatial), bits(torch.nn.functional.pad(x, (1, 1, 1, 1))))
    del padded, want, spatial
    proj = torch.randn(1, 8192, 16384, device="cuda").to(torch.bfloat16)
    a, g = be.split(proj, [8192, 8192], -1)
    assert torch.equal(bits(a), bits(proj[..., :8192].contiguous())) and torch.equal(bits(g), bits(proj[..., 8192:].contiguous()))
    del proj, a, g
    big = torch.empty(5, 2 ** 29 + 8, device="cuda", dtype=torch.bfloat16)           # 2.5 Gi + 40 elements, 5 GiB
    big.view(torch.int16).random_()
    part = be.slice(big, 1, 3, big.shape[1] - 1)                                      # odd offset: 2-byte units, > 2^31 of them
    assert torch.equal(bits(part), bits(big[:, 3:-1].contiguous()))
