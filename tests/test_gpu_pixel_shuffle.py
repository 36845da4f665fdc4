"""pixel_shuffle_nd and the one-pass LTX depth_to_space block: index work and one add, so every
comparison is bit for bit -- against the oracle (numpy index map of the reference's kernel) and
against this library's own operator-by-operator chain; row (vector) and element-wise paths."""
import numpy as np
import pytest

from conftest import assert_bits_equal, to_torch

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("shape,factors", [
    ((1, 32, 3, 6, 16), (2, 2, 2)),    # row path, interleaving pairs of rows
    ((2, 12, 2, 3, 8), (1, 2, 2)),     # Mochi-style spatial only
    ((1, 12, 2, 5, 24), (3, 2, 1)),    # fw = 1: row copies
    ((2, 8, 2, 3, 5), (2, 2, 2)),      # odd width: element-wise path
    ((1, 27, 2, 4, 8), (3, 3, 3)),     # fw = 3: element-wise path
])
@pytest.mark.parametrize("dt", ["bf16", "f32"])
def test_pixel_shuffle_bit_exact(orc, gpu, shape, factors, dt):
    be, ops = gpu
    # integer-valued payload: the position of every element is visible in its value
    x = orc.tensor((np.arange(np.prod(shape)) % 251).astype(np.float32).reshape(shape), dt)
    want = orc.OracleBackend().pixel_shuffle_nd(x, factors)
    assert_bits_equal(be.pixel_shuffle_nd(to_torch(x), factors), want, "pixel_shuffle")


@pytest.mark.parametrize("shape", [(1, 32, 3, 6, 16), (2, 8, 2, 3, 8), (2, 8, 2, 3, 5), (1, 64, 1, 4, 32)])
@pytest.mark.parametrize("dt", ["bf16", "f32"])
def test_depth_to_space_residual(orc, gpu, shape, dt):
    import torch
    be, ops = gpu
    from vrhino_b200 import synth
    b, c, t, h, w = shape
    x = orc.tensor(synth.normal(shape, seed=c), dt)
    y = orc.tensor(synth.normal((b, 4 * c, t, h, w), seed=c + 1), dt)
    obe = orc.OracleBackend()
    got = ops.fused_depth_to_space_residual(be, to_torch(y), to_torch(x))
    if t > 1:
        assert_bits_equal(got, orc.depth_to_space_residual(obe, y, x), "depth_to_space")
        residual = torch.cat([be.pixel_shuffle_nd(to_torch(x), (2, 2, 2))] * 4, dim=1)[:, :, 1:].contiguous()
        chain = be.add(be.pixel_shuffle_nd(to_torch(y), (2, 2, 2))[:, :, 1:].contiguous(), residual)
        view = torch.int16 if dt == "bf16" else torch.int32
        assert torch.equal(got.view(view), chain.view(view))
    assert tuple(got.shape) == (b, c // 2, 2 * t - 1, 2 * h, 2 * w)


def test_errors(gpu):
    import torch
    be, ops = gpu
    x = torch.zeros((1, 12, 2, 4, 8), device="cuda")
    with pytest.raises(ops.VrbError):
        be.pixel_shuffle_nd(x, (2, 2, 2))          # 12 channels, product 8
    with pytest.raises(ops.VrbError):
        be.pixel_shuffle_nd(x[0], (1, 2, 2))
    with pytest.raises(ops.VrbError):
        ops.fused_depth_to_space_residual(be, torch.zeros((1, 40, 2, 4, 8), device="cuda"), x)
