"""The bf16 linear's epilogue (fused_bf16_linear_output_kernel of the reference) alone and merged
with the operator that reads its result: activation, gated residual / residual add, SwiGLU.

Bit-exact checks only: the epilogue is one F32 add and one rounding; the merged forms must equal
the epilogue kernel followed by the consumer kernel bit for bit (which the golden-vector tests in
turn pin to the reference's kernels), on vector, scalar (odd width / misaligned) and table paths.
"""
import numpy as np
import pytest

from conftest import assert_bits_equal, to_torch

pytestmark = pytest.mark.gpu


def _bits(t):
    import torch
    return t.contiguous().view(torch.int16 if t.dtype == torch.bfloat16 else torch.int32)


def _operands(rows, width, seed, bias=True, specials=False):
    import torch
    g = torch.Generator(device="cuda").manual_seed(seed)
    acc = torch.randn((rows, width), device="cuda", generator=g) * 3.0
    if specials:
        flat = acc.view(-1)
        vals = [0.0, -0.0, float("inf"), float("-inf"), float("nan"), 3.3895314e38, -3.3895314e38, 1e-40, -1e-40, 65280.0]
        flat[:len(vals)] = torch.tensor(vals, device="cuda")
    b = (torch.randn((width,), device="cuda", generator=g) * 0.5).bfloat16() if bias else None
    return acc, b


@pytest.mark.parametrize("rows,width", [(7, 1536), (3, 24), (5, 257), (64, 8960), (33, 100)])
@pytest.mark.parametrize("bias", [True, False])
def test_linear_output_matches_oracle_bit_for_bit(orc, gpu, rows, width, bias):
    import torch
    be, ops = gpu
    acc, b = _operands(rows, width, rows * width, bias, specials=True)
    got = ops.linear_output(be, acc, b)
    want = orc.linear_output(orc.T(acc.cpu().numpy(), "f32"),
                             None if b is None else orc.T(b.cpu().view(torch.int16).numpy().view(np.uint16), "bf16"))
    assert_bits_equal(got, want, "linear_output")


@pytest.mark.parametrize("rows,width", [(9, 1536), (5, 257), (600, 8960), (2048, 3072)])   # the last two take the table path
@pytest.mark.parametrize("kind", [0, 1, 2, 3, 4])
@pytest.mark.parametrize("bias", [True, False])
def test_activation_form_equals_epilogue_then_activation(gpu, rows, width, kind, bias):
    import torch
    be, ops = gpu
    acc, b = _operands(rows, width, 7 + kind, bias, specials=True)
    fused = ops.linear_output_activation(be, acc, b, kind)
    chain = be.activation(ops.linear_output(be, acc, b), kind)
    assert torch.equal(_bits(fused), _bits(chain))


@pytest.mark.parametrize("batch,tokens,width", [(1, 9, 1536), (2, 7, 1536), (3, 5, 264), (1, 5, 257), (2, 1100, 3072)])
@pytest.mark.parametrize("state", ["bf16", "f32"])
@pytest.mark.parametrize("res_dt", ["bf16", "f32"])
@pytest.mark.parametrize("gated", [True, False])
def test_gated_residual_form_equals_epilogue_then_gated_residual(gpu, batch, tokens, width, state, res_dt, gated):
    import torch
    be, ops = gpu
    dt = {"bf16": torch.bfloat16, "f32": torch.float32}
    acc, b = _operands(batch * tokens, width, 11, True)
    acc = acc.view(batch, tokens, width)
    g = torch.Generator(device="cuda").manual_seed(5)
    res = torch.randn((batch, tokens, width), device="cuda", generator=g).to(dt[res_dt])
    gate = torch.randn((batch, 1, width), device="cuda", generator=g) * 0.3 if gated else None
    pol = ops.Policy(residual=dt[state])
    fused = ops.linear_output_gated_residual(be, pol, res, acc, b, gate)
    chain = ops.fused_gated_residual(be, pol, res, ops.linear_output(be, acc, b), gate)
    assert fused.dtype == dt[state]
    assert torch.equal(_bits(fused), _bits(chain))


@pytest.mark.parametrize("rows,hidden", [(9, 768), (5, 100), (3, 129), (700, 8192)])   # the last takes the table path
@pytest.mark.parametrize("bias", [True, False])
def test_swiglu_form_equals_epilogue_then_swiglu(gpu, rows, hidden, bias):
    import torch
    be, ops = gpu
    acc, b = _operands(rows, 2 * hidden, 13, bias, specials=True)
    fused = ops.linear_output_swiglu(be, acc, b)
    chain = ops.fused_swiglu(be, ops.linear_output(be, acc, b))
    assert torch.equal(_bits(fused), _bits(chain))


def test_misaligned_operands_take_the_scalar_path(gpu):
    import torch
    be, ops = gpu
    acc, b = _operands(6, 1536 + 8, 3, True)
    view = acc[:, 4:1540]                      # rows start 16 bytes into each line: dense copy below is aligned
    want = be.activation(ops.linear_output(be, view.contiguous(), b[:1536].contiguous()), 2)
    flat = torch.empty(6 * 1536 + 1, device="cuda")
    shifted = flat[1:].view(6, 1536)           # 4-byte aligned only
    shifted.copy_(view)
    got = ops.linear_output_activation(be, shifted, b[:1536].contiguous(), 2)
    assert torch.equal(_bits(got), _bits(want))


def test_errors(gpu):
    import torch
    be, ops = gpu
    acc, b = _operands(4, 64, 1, True)
    with pytest.raises(ops.VrbError):
        ops.linear_output(be, acc.bfloat16(), b)
    with pytest.raises(ops.VrbError):
        ops.linear_output(be, acc, b[:32].contiguous())
    with pytest.raises(ops.VrbError):
        ops.linear_output_activation(be, acc, b, 9)
    with pytest.raises(ops.VrbError):
        ops.linear_output_swiglu(be, acc[:, :63].contiguous(), None)
