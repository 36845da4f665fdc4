"""GPU parity of the elementwise / broadcast kernels against the CPU oracle, through the C ABI.

Tolerances: integer-like and single-IEEE-operation results are compared bit for bit; results
that go through expf / tanhf / erff are compared at <= 2 bf16 ulp (bf16) or 1e-5 relative
(f32), because the CUDA and the C math libraries are each specified to 1-2 ulp.  Where
1 + tanhf / 1 + erff cancels (negative tail of GELU) two conforming libraries agree only
absolutely, so an absolute bound of 4 * 2^-24 * |x| is allowed there and stated in the test.
"""
import numpy as np
import pytest

from conftest import assert_bits_equal, assert_close, to_torch

pytestmark = pytest.mark.gpu

DTYPES = ["f32", "bf16"]


def indexing_input(orc, shape, dtype, seed):
    """Inputs of native/tests/cuda_binary_indexing_tests.cu:50-61 (incl. +-0, +-inf, NaN)."""
    count = int(np.prod(shape)) if len(shape) else 1
    i = np.arange(count, dtype=np.int64)
    v = (((i * 17 + seed) % 255 - 127).astype(np.float32) / np.float32(128.0))
    special = np.array([0.0, -0.0, np.inf, -np.inf, np.nan], dtype=np.float32)
    for k in range(min(count, 5)):
        v[k] = special[(k + seed) % 5]
    return orc.tensor(v.reshape(shape), dtype)


BINARY_CASES = [
    ("full", (1, 32760, 1536), (1, 32760, 1536)),
    ("suffix", (1, 32760, 1536), (1, 1, 1536)),
    ("scalar_first", (), (3, 257)),
    ("scalar_last", (3, 257), (1, 1)),
    ("suffix_first", (7,), (3, 5, 7)),
    ("suffix_matrix", (3, 7), (2, 3, 7)),
    ("internal_singleton", (3, 1, 7), (1, 5, 1)),
    ("rank8", (1, 1, 1, 1, 1, 1, 257, 3), (257, 3)),
]


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("label,a_shape,b_shape", BINARY_CASES)
def test_binary_indexing_bit_exact(orc, gpu, dtype, label, a_shape, b_shape):
    """The 64 byte-exact cases of cuda_binary_indexing_tests.cu:111-118, Wan adaLN shape included."""
    be, ops = gpu
    obe = orc.OracleBackend(execution_dtype=dtype)
    a, b = indexing_input(orc, a_shape, dtype, 1), indexing_input(orc, b_shape, dtype, 3)
    ta, tb = to_torch(a), to_torch(b)
    for kind, name in enumerate(["add", "mul", "div", "maximum"]):
        want = obe._binary(kind, a, b)
        got = getattr(be, name)(ta, tb)
        assert_bits_equal(got, want, f"{label}/{dtype}/{name}")


@pytest.mark.parametrize("dtype", ["bf16", "f32"])
@pytest.mark.parametrize("a_shape,b_shape", [
    ((2, 16, 3, 4, 8), (2, 16, 1, 1, 1)),     # channel vector over [B, C, T, H, W]: two merged axes
    ((1, 16, 1, 1, 1), (2, 16, 3, 4, 8)),     # the same with the operands swapped
    ((2, 5, 64), (2, 1, 64)),                 # per-batch row vector: three merged axes
    ((4, 6, 8), (4, 1, 1)),                   # one value per row
    ((3, 5, 7, 16), (1, 5, 1, 16)),           # four merged axes: general indexing
    ((2, 3, 24), (2, 3, 1)),                  # innermost run 24
    ((2, 16, 3, 4, 8), (1, 1, 3, 1, 1)),      # vector along a middle axis
    ((2, 1, 40), (1, 7, 1)),                  # both operands broadcast
])
def test_binary_inner_axis_broadcasts_bit_exact(orc, gpu, dtype, a_shape, b_shape):
    """Broadcasts along inner axes (VAE per-channel statistics, per-batch modulation rows): the
    merged-axes vector path and the general path must agree with the oracle bit for bit."""
    be, ops = gpu
    obe = orc.OracleBackend(execution_dtype=dtype)
    a, b = indexing_input(orc, a_shape, dtype, 1), indexing_input(orc, b_shape, dtype, 3)
    ta, tb = to_torch(a), to_torch(b)
    for kind, name in enumerate(["add", "mul", "div", "maximum"]):
        assert_bits_equal(getattr(be, name)(ta, tb), obe._binary(kind, a, b), f"{a_shape}x{b_shape}/{dtype}/{name}")


def test_binary_rejections(gpu):
    be, ops = gpu
    import torch
    with pytest.raises(ops.VrbError, match="CUDA primitive rank exceeds 8"):
        be.add(torch.zeros((1,) * 9, device="cuda", dtype=torch.bfloat16), torch.zeros((), device="cuda", dtype=torch.bfloat16))
    with pytest.raises(ops.VrbError, match="Incompatible broadcast shapes"):
        be.mul(torch.zeros(2, 3, device="cuda"), torch.zeros(2, 4, device="cuda"))


def test_binary_operand_dtype_rule(orc, gpu):
    """add(bf16, f32) computes in bf16, add(f32, bf16) in f32 (cuda_backend.cu:3875-3880)."""
    be, ops = gpu
    obe = orc.OracleBackend()
    from vrhino_b200 import synth
    a = orc.tensor(synth.normal((5, 64), seed=1), "bf16")
    b = orc.tensor(synth.normal((5, 64), seed=2), "f32")
    for x, y in ((a, b), (b, a)):
        want = obe.add(x, y)
        got = be.add(to_torch(x), to_torch(y))
        assert_bits_equal(got, want, f"add({x.dtype},{y.dtype})")


@pytest.mark.parametrize("n", [4, 1000, 8 * 1031])
def test_cast_bit_exact(orc, gpu, n):
    be, ops = gpu
    import torch
    from vrhino_b200 import synth
    obe = orc.OracleBackend()
    x = orc.tensor(np.concatenate([synth.normal((n - 4,), std=3.0, seed=n), np.array([np.inf, -np.inf, np.nan, -0.0], dtype=np.float32)]))
    want = obe.cast(x, "bf16")
    got = be.cast(to_torch(x), torch.bfloat16)
    assert_bits_equal(got, want, "f32->bf16")
    assert_bits_equal(be.cast(got, torch.float32), obe.cast(want, "f32"), "bf16->f32")
    assert be.cast(got, torch.bfloat16) is got  # same handle on a no-op cast
    kat = be.cast(be.cast(torch.tensor([1.1, -2.3, 0, 8], device="cuda"), torch.bfloat16), torch.float32)
    assert kat.tolist() == [1.1015625, -2.296875, 0.0, 8.0]
    u8 = torch.arange(0, 256, dtype=torch.uint8, device="cuda")
    assert torch.equal(be.cast(u8, torch.float32).cpu(), torch.arange(0, 256, dtype=torch.float32))


ACT_NAMES = {0: "silu", 1: "gelu", 2: "gelu_tanh", 3: "tanh", 4: "relu"}


@pytest.mark.parametrize("kind", [0, 1, 2, 3, 4])
def test_activation_exhaustive_bf16(orc, gpu, kind):
    """Every finite bf16 input (and the infinities): the whole function table of the kernel."""
    be, ops = gpu
    bits = np.arange(65536, dtype=np.uint32).astype(np.uint16)
    finite_or_inf = (bits & 0x7FFF) <= 0x7F80
    bits = bits[finite_or_inf]
    x = orc.T(bits, "bf16")
    want = orc.OracleBackend().activation(x, kind)
    got = be.activation(to_torch(x), kind)
    xf = np.abs(x.f32())
    from conftest import from_torch
    data, _ = from_torch(got)
    d = orc.bf16_ulp_distance(data, want.data)
    diff = np.abs(orc.bf16_bits_to_f32(data).astype(np.float64) - want.f32().astype(np.float64))
    with np.errstate(invalid="ignore"):
        allowed = (d <= 2) | (diff <= 4 * 2.0 ** -24 * xf) | (np.isnan(orc.bf16_bits_to_f32(data)) & np.isnan(want.f32()))
    assert allowed.all(), (ACT_NAMES[kind], int((~allowed).sum()), x.f32()[~allowed][:5])
    assert (d == 0).mean() > 0.99, f"{ACT_NAMES[kind]}: only {(d == 0).mean():.4f} of the table is bit-identical"


def test_table_path_equals_direct_path(gpu):
    """bf16 tensors of 4M elements and more run through the 128 KB function table in shared
    memory (prebuilt once per operator and parameters, then reused): every bf16 code must come
    out exactly as from the direct kernel, on the first launch (which builds the table) and on
    the second (which reuses it); same for clamp bounds and for SwiGLU's SiLU table."""
    import torch
    be, ops = gpu
    codes = torch.arange(65536, dtype=torch.int32, device="cuda").to(torch.int16).view(torch.bfloat16)
    big = codes.repeat(80)
    for label, fn in [("silu", lambda t: be.activation(t, 0)), ("gelu_tanh", lambda t: be.activation(t, 2)),
                      ("clamp", lambda t: be.clamp(t, -0.5, 0.75)), ("clamp2", lambda t: be.clamp(t, -1.0, 2.0)),
                      ("exp", be.exp), ("sqrt", be.sqrt)]:
        direct = fn(codes).view(torch.int16)
        for attempt in range(2):
            got = fn(big).view(torch.int16).reshape(80, 65536)
            assert torch.equal(got, direct.expand(80, 65536)), (label, attempt)
    from vrhino_b200 import synth
    proj = torch.from_numpy(synth.normal((1, 640, 2 * 8192), seed=3)).cuda().to(torch.bfloat16)
    whole = ops.fused_swiglu(be, proj)
    parts = torch.cat([ops.fused_swiglu(be, proj[:, r:r + 64].contiguous()) for r in range(0, 640, 64)], dim=1)
    assert torch.equal(whole.view(torch.int16), parts.view(torch.int16))


_TABLE_STATES_SCRIPT = r"""
import ctypes, sys, torch
sys.path.insert(0, sys.argv[1])
from vrhino_b200 import _lib
lib = _lib.load()
P = ctypes.c_void_p
codes = torch.arange(65536, dtype=torch.int32, device="cuda").to(torch.int16).view(torch.bfloat16)
big = codes.repeat(80)
outs = [torch.empty_like(big) for _ in range(4)]
direct = torch.empty_like(codes)
def act(x, out, stream):
    assert lib.vrb_activation(2, P(x.data_ptr()), P(out.data_ptr()), 2, x.numel(), P(stream)) == 0, lib.vrb_last_error()
side = torch.cuda.Stream()
graph = torch.cuda.CUDAGraph()
# 1. the FIRST use of the library is captured: no table exists, none may be built inside a capture
with torch.cuda.graph(graph, stream=side):
    act(big, outs[0], side.cuda_stream)
graph.replay(); torch.cuda.synchronize()
first = outs[0].clone()
outs[0].zero_()
assert lib.vrb_prepare_tables(P(side.cuda_stream)) == 0
act(big, outs[1], side.cuda_stream)            # 2. same stream as the build: ordered behind it
act(big, outs[2], torch.cuda.current_stream().cuda_stream)   # 3. another stream: flag set or not, same bits
torch.cuda.synchronize()
act(big, outs[3], torch.cuda.current_stream().cuda_stream)   # 4. table certainly published
graph.replay()                                 # 5. the captured kernel now finds the table
act(codes, direct, torch.cuda.current_stream().cuda_stream)  # small tensor: the direct kernel
torch.cuda.synchronize()
want = direct.view(torch.int16).expand(80, 65536)
for k, t in enumerate([first] + outs):
    assert torch.equal(t.view(torch.int16).reshape(80, 65536), want), k
with torch.cuda.graph(torch.cuda.CUDAGraph(), stream=side):
    assert lib.vrb_prepare_tables(P(side.cuda_stream)) == -1
assert lib.vrb_device_allocation_count() == 0
print("ok")
"""


def test_function_table_states_in_a_fresh_process():
    """The table kernels decide on the device whether the resident table may be read: captured
    before any table was built (evaluates its own), right behind the build on the same stream,
    on another stream, after publication, and the first graph replayed again.  All five give the
    direct kernel's bits; the library allocates nothing; vrb_prepare_tables refuses a capturing
    stream."""
    import os
    import subprocess
    import sys
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    proc = subprocess.run([sys.executable, "-c", _TABLE_STATES_SCRIPT, root], capture_output=True, text=True, timeout=600)
    assert proc.returncode == 0 and proc.stdout.strip().endswith("ok"), proc.stderr[-3000:]


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("kind", [0, 2, 3])
@pytest.mark.parametrize("n", [37, 8 * 4096 + 8])
def test_activation_random(orc, gpu, dtype, kind, n):
    be, ops = gpu
    from vrhino_b200 import synth
    x = orc.tensor(synth.normal((n,), std=2.0, seed=kind + n), dtype)
    want = orc.OracleBackend().activation(x, kind)
    got = be.activation(to_torch(x), kind)
    assert_close(orc, got, want, max_ulp=2, rel=1e-5, atol=float(4 * 2.0 ** -24 * np.abs(x.f32()).max()), what=ACT_NAMES[kind])


def test_clamp_exp_sqrt(orc, gpu):
    be, ops = gpu
    from vrhino_b200 import synth
    obe = orc.OracleBackend()
    for dtype in DTYPES:
        x = orc.tensor(synth.normal((3, 1000), std=2.0, seed=5), dtype)
        tx = to_torch(x)
        assert_bits_equal(be.clamp(tx, -0.5, 0.75), obe.clamp(x, -0.5, 0.75), "clamp")
        assert_close(orc, be.exp(tx), obe.exp(x), what="exp")
        pos = orc.tensor(np.abs(x.f32()), dtype)
        assert_bits_equal(be.sqrt(to_torch(pos)), obe.sqrt(pos), "sqrt")  # sqrtf is correctly rounded on both sides
    with pytest.raises(ops.VrbError, match="Invalid clamp bounds"):
        be.clamp(tx, 1.0, 0.0)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("rows,hidden", [(5, 24), (3, 7), (33, 8192)])
def test_swiglu(orc, gpu, dtype, rows, hidden):
    be, ops = gpu
    from vrhino_b200 import synth
    proj = orc.tensor(synth.normal((1, rows, 2 * hidden), seed=rows), dtype)
    want = orc.swiglu_hidden(orc.OracleBackend(), proj)
    got = ops.fused_swiglu(be, to_torch(proj))
    assert_close(orc, got, want, what="swiglu")


@pytest.mark.parametrize("res_dt,br_dt,state", [("bf16", "bf16", "bf16"), ("f32", "bf16", "f32"), ("bf16", "bf16", "f32"), ("f32", "f32", "f32")])
@pytest.mark.parametrize("rows,width,batch", [(6, 64, 1), (6, 64, 2), (5, 7, 1)])
@pytest.mark.parametrize("gated", [True, False])
def test_gated_residual_bit_exact(orc, gpu, res_dt, br_dt, state, rows, width, batch, gated):
    """gated_residual / residual_add are chains of single IEEE operations: bit for bit."""
    import torch
    be, ops = gpu
    from vrhino_b200 import synth
    obe = orc.OracleBackend()
    res = orc.tensor(synth.normal((batch, rows, width), seed=1), res_dt)
    br = orc.tensor(synth.normal((batch, rows, width), seed=2), br_dt)
    gate = orc.tensor(synth.normal((batch, 1, width), std=0.1, seed=3), "f32")
    opol = orc.Policy(residual=state)
    pol = ops.Policy(residual=torch.float32 if state == "f32" else torch.bfloat16)
    want = orc.gated_residual(obe, opol, res, br, gate) if gated else orc.residual_add(obe, opol, res, br)
    got = ops.fused_gated_residual(be, pol, to_torch(res), to_torch(br), to_torch(gate) if gated else None)
    assert_bits_equal(got, want, "fused gated_residual")
    chain = ops.gated_residual(be, pol, to_torch(res), to_torch(br), to_torch(gate)) if gated else \
        ops.residual_add(be, pol, to_torch(res), to_torch(br))
    assert_bits_equal(chain, want, "per-op chain")


@pytest.mark.parametrize("batch,rows,width", [(3, 13000, 1024), (1, 32760, 1536), (2, 6200, 5120)])
def test_gated_residual_staged_gate_path(orc, gpu, batch, rows, width):
    """Large all-bf16 launches keep the gate vectors in shared memory and carry column / vector along instead of
    dividing them out of the index.  Same bits as the general kernel (the same tensors in launches too small for the
    staged path) and as the oracle on the first and last rows of every batch entry."""
    import torch
    be, ops = gpu
    from vrhino_b200 import synth
    g = torch.Generator(device="cuda").manual_seed(batch * 7 + width)
    res = torch.randn(batch, rows, width, device="cuda", generator=g).to(torch.bfloat16)
    br = torch.randn(batch, rows, width, device="cuda", generator=g).to(torch.bfloat16)
    gate = torch.randn(batch, 1, width, device="cuda", generator=g) * 0.3
    pol = ops.Policy(residual=torch.bfloat16)
    got = ops.fused_gated_residual(be, pol, res, br, gate)
    pieces = []
    for b in range(batch):
        for r0 in range(0, rows, 2048):          # 2048 rows: well below the staged path's threshold
            pieces.append(ops.fused_gated_residual(be, pol, res[b:b + 1, r0:r0 + 2048].contiguous(), br[b:b + 1, r0:r0 + 2048].contiguous(),
                                                   gate[b:b + 1]))
    want = torch.cat(pieces, 1).view(batch, rows, width)
    assert torch.equal(got.view(torch.int16), want.view(torch.int16))
    obe, opol = orc.OracleBackend(), orc.Policy(residual="bf16")
    bits = lambda t: orc.T(t.contiguous().view(torch.int16).cpu().numpy().view(np.uint16), "bf16")
    for b in range(batch):
        for sl in (slice(0, 3), slice(rows - 3, rows)):
            ref = orc.gated_residual(obe, opol, bits(res[b:b + 1, sl]), bits(br[b:b + 1, sl]), orc.tensor(gate[b:b + 1].cpu().numpy(), "f32"))
            assert np.array_equal(got[b:b + 1, sl].contiguous().view(torch.int16).cpu().numpy().view(np.uint16), ref.data)


@pytest.mark.parametrize("x_dt", DTYPES)
@pytest.mark.parametrize("f_dt", DTYPES)
@pytest.mark.parametrize("shape,f_shape", [((1, 3, 2, 6), (1, 3, 1, 6)), ((1, 3, 2, 64), (1, 3, 1, 64)), ((1, 3, 2, 128), (1, 3, 1, 128)),
                                           ((2, 5, 4, 128), (1, 5, 4, 128)), ((2, 5, 256), (2, 5, 256)), ((2, 3, 4, 16), (2, 1, 1, 16))])
def test_rope_bit_exact(orc, gpu, x_dt, f_dt, shape, f_shape):
    """rope_nd is three IEEE operations per element with fixed rounding: bit for bit, on the
    dtype matrix of precision_operation_contract_tests.cpp:41-83 plus per-head, per-batch and
    inner-broadcast tables."""
    be, ops = gpu
    from vrhino_b200 import synth
    x = orc.tensor(synth.normal(shape, seed=11), x_dt)
    phase = synth.uniform_range(f_shape, -3.1, 3.1, seed=12)
    co, si = orc.tensor(np.cos(phase), f_dt), orc.tensor(np.sin(phase), f_dt)
    want = orc.OracleBackend().rope_nd(x, co, si)
    got = be.rope_nd(to_torch(x), to_torch(co), to_torch(si))
    assert_bits_equal(got, want, "rope")


def test_rope_no_contraction_kat(gpu):
    """precision_operation_contract_tests.cpp:26-37"""
    import torch
    be, ops = gpu
    u = 2.0 ** -23
    x = torch.tensor([1.0 + u, 1.0], device="cuda").reshape(1, 1, 1, 2)
    c = torch.tensor([1.0 - u, 0.0], device="cuda").reshape(1, 1, 1, 2)
    s = torch.tensor([1.0, 0.0], device="cuda").reshape(1, 1, 1, 2)
    assert be.rope_nd(x, c, s).reshape(-1)[0].item() == 0.0
    with pytest.raises(ops.VrbError, match="RoPE width must be even"):
        be.rope_nd(torch.zeros(1, 2, 1, 3, device="cuda"), torch.zeros(1, 2, 1, 3, device="cuda"), torch.zeros(1, 2, 1, 3, device="cuda"))


@pytest.mark.parametrize("out_dt", DTYPES)
@pytest.mark.parametrize("kind,rows,inner,group", [("fp8_e4m3fn", 6, 8, 4), ("fp8_e4m3fn", 16, 256, 256), ("fp8_e4m3fn", 5, 96, 32),
                                                   ("fp8_e4m3fn", 3, 40, 8), ("int8", 16, 256, 64), ("int8", 3, 10, 5), ("int4", 4, 16, 8),
                                                   ("int4", 6, 1024, 1024), ("int4", 5, 1088, 64), ("int4", 3, 96, 32)])
def test_dequantize_bit_exact(orc, gpu, out_dt, kind, rows, inner, group):
    import torch
    be, ops = gpu
    from vrhino_b200 import synth
    count = rows * inner
    if kind == "fp8_e4m3fn":
        packed = np.arange(count, dtype=np.int64).astype(np.uint8) if count >= 256 else synth.fp8_codes((count,), seed=3)
    elif kind == "int8":
        packed = (np.arange(count) * 37 % 256).astype(np.uint8)
    else:
        packed = (np.arange((count + 1) // 2) * 53 % 256).astype(np.uint8)
    groups = (inner + group - 1) // group
    scales = synth.uniform_range((rows, groups), 1e-3, 1e-2, seed=4)
    t = orc.T(packed, "u8", host=True, quant={"type": kind, "group_size": group, "scales": scales, "shape": (rows, inner)})
    want = orc.OracleBackend().copy_to_device(t, out_dt)
    code = {"fp8_e4m3fn": 0, "int8": 1, "int4": 2}[kind]
    got = be.dequantize(torch.from_numpy(packed), torch.from_numpy(scales), group, kind=code,
                        dtype=torch.float32 if out_dt == "f32" else torch.bfloat16, shape=(rows, inner))
    assert_bits_equal(got, want, f"dequant {kind}")


def test_dequantize_all_fp8_codes(orc, gpu):
    """All 256 codes, scale 1: the decode table itself, incl. 0x7f/0xff -> +-480 and -0."""
    import torch
    be, ops = gpu
    packed = np.arange(256, dtype=np.uint8)
    got = be.dequantize(torch.from_numpy(packed), torch.ones(1, 1), 256, dtype=torch.float32, shape=(1, 256)).cpu().numpy().reshape(-1)
    want = np.array([orc.lib().orc_decode_fp8(int(c)) for c in packed], dtype=np.float32)
    assert np.array_equal(got.view(np.uint32), want.view(np.uint32))


def test_dequantize_scale_extremes(orc, gpu):
    """Every code against scales that stress the branch-free decode (which multiplies the code
    lifted by 2^-120 with the scale lifted by 2^120): zero and negative zero, a denormal, the
    largest scale the lifted form takes, scales beyond it (other path), huge and negative ones.
    Expected: the F32 product decode(code) * scale rounded once, then to the output dtype."""
    import torch
    be, ops = gpu
    scales = np.array([0.0, -0.0, 1e-40, 2.0 ** -126, 1e-3, 127.99, 128.0, 300.0, 1e30, -3.5, 2.0 ** 100, -1e-42],
                      dtype=np.float32)
    rows = scales.size
    packed = np.tile(np.arange(256, dtype=np.uint8), (rows, 1))
    decoded = np.array([orc.lib().orc_decode_fp8(int(c)) for c in range(256)], dtype=np.float32)
    with np.errstate(over="ignore", under="ignore"):
        want = decoded[None, :] * scales[:, None]            # one IEEE F32 multiply per element
    got = be.dequantize(torch.from_numpy(packed), torch.from_numpy(scales.reshape(rows, 1)), 256, dtype=torch.float32).cpu().numpy()
    assert np.array_equal(got.view(np.uint32), want.view(np.uint32)), np.argwhere(got.view(np.uint32) != want.view(np.uint32))[:5]
    got16 = be.dequantize(torch.from_numpy(packed), torch.from_numpy(scales.reshape(rows, 1)), 256, dtype=torch.bfloat16)
    want16 = torch.from_numpy(want).to(torch.bfloat16)
    assert torch.equal(got16.cpu().view(torch.int16), want16.view(torch.int16))
    # per-group scales on the same path
    gs = np.linspace(1e-3, 1e-2, rows * 16, dtype=np.float32).reshape(rows, 16)
    got = be.dequantize(torch.from_numpy(packed), torch.from_numpy(gs), 16, dtype=torch.float32).cpu().numpy()
    want = decoded[None, :] * np.repeat(gs, 16, axis=1)
    assert np.array_equal(got.view(np.uint32), want.view(np.uint32))


SAMPLER_POLICIES = ["fp32", "bf16_legacy", "bf16_roles", "bf16_guidance_only"]


def _policies(orc, ops, name):
    import torch
    if name == "fp32":
        return orc.Policy.fp32(), ops.Policy.fp32(), "f32", orc.F32, torch.float32
    o, p = orc.Policy.unqualified_default("bf16"), ops.Policy.unqualified_default(torch.bfloat16)
    if name == "bf16_roles":
        roles = {"GuidanceCoefficient", "SolverCoefficient", "Sigma"}
        o, p = o.with_scalar_roles(roles), p.with_scalar_roles(roles)
    if name == "bf16_guidance_only":
        o, p = o.with_scalar_roles({"GuidanceCoefficient"}), p.with_scalar_roles({"GuidanceCoefficient"})
    return o, p, "bf16", orc.BF16, torch.bfloat16


@pytest.mark.parametrize("policy", SAMPLER_POLICIES)
@pytest.mark.parametrize("n", [12, 2 * 16 * 21 * 13])
def test_sampler_updates_bit_exact(orc, gpu, policy, n):
    """cfg_combine / euler_update / flow_to_x0 and the fused cfg+euler: chains of single IEEE
    operations, so bit for bit under every scalar contract (semantic_scalar_tests.cpp:20-28)."""
    _, ops = gpu
    opol, pol, dt, oexec, texec = _policies(orc, ops, policy)
    be = ops.B200Backend(execution_dtype=texec)
    obe = orc.OracleBackend(execution_dtype=oexec)
    from vrhino_b200 import synth
    x, u, c = (orc.tensor(synth.normal((n,), seed=s), dt) for s in (1, 2, 3))
    tx, tu, tc = to_torch(x), to_torch(u), to_torch(c)
    scale, delta, sigma = 5.0, 0.02, 0.877877295
    want_g = orc.cfg_combine(obe, opol, u, c, scale)
    assert_bits_equal(ops.fused_cfg_combine(be, pol, tu, tc, scale), want_g, "fused cfg")
    assert_bits_equal(ops.cfg_combine(be, pol, tu, tc, scale), want_g, "chain cfg")
    want_e = orc.euler_update(obe, opol, x, u, orc.scalar_f32(delta), True)
    assert_bits_equal(ops.fused_euler_update(be, pol, tx, tu, delta, True), want_e, "fused euler")
    assert_bits_equal(ops.euler_update(be, pol, tx, tu, delta, True), want_e, "chain euler")
    want_f = orc.flow_to_x0(obe, opol, x, u, sigma)
    assert_bits_equal(ops.fused_flow_to_x0(be, pol, tx, tu, sigma), want_f, "fused flow_to_x0")
    want_ge = orc.euler_update(obe, opol, x, want_g, orc.scalar_f32(delta), True)
    out, guided = ops.fused_cfg_euler(be, pol, tx, tu, tc, scale, delta, True, want_guided=True)
    assert_bits_equal(guided, want_g, "fused cfg+euler guided")
    assert_bits_equal(out, want_ge, "fused cfg+euler")


def test_null_and_empty_arguments_are_rejected(gpu):
    import ctypes
    be, ops = gpu
    from vrhino_b200 import _lib
    lib = _lib.load()
    assert lib.vrb_activation(0, None, None, 0, 16, None) == -1
    assert b"null tensor" in lib.vrb_last_error()
    import torch
    x = torch.zeros(8, device="cuda")
    assert lib.vrb_activation(0, ctypes.c_void_p(x.data_ptr()), ctypes.c_void_p(x.data_ptr()), 0, 0, None) == -1
    assert lib.vrb_activation(9, ctypes.c_void_p(x.data_ptr()), ctypes.c_void_p(x.data_ptr()), 0, 8, None) == -1
    assert lib.vrb_activation(0, ctypes.c_void_p(x.data_ptr()), ctypes.c_void_p(x.data_ptr()), 5, 8, None) == -2



@pytest.mark.parametrize("dt", ["bf16", "f32"])
@pytest.mark.parametrize("roles", [False, True])
@pytest.mark.parametrize("terms", [1, 2, 3, 4])
@pytest.mark.parametrize("shape", [(16, 3, 10, 13), (1, 16, 4, 8, 16)])
def test_linear_combine_one_pass(orc, gpu, dt, roles, terms, shape):
    """linear_combine (and its two-term uses v_to_x0 / affine_first_order) in one launch: bit for bit
    against the oracle's operator chain and against this library's own chain, under the legacy and
    the declared-role scalar contracts."""
    import torch
    be, ops = gpu
    from vrhino_b200 import synth
    coefs = [0.877877295, -0.4786229, 1.5, -0.0625][:terms]
    vals = [orc.tensor(synth.normal(shape, seed=20 + t), dt) for t in range(terms)]
    obe = orc.OracleBackend(execution_dtype=dt)
    opol = orc.Policy.fp32() if dt == "f32" else orc.Policy()
    pol = ops.Policy.fp32() if dt == "f32" else ops.Policy()
    if roles:
        opol = opol.with_scalar_roles({orc.GUIDANCE})
        pol = pol.with_scalar_roles({ops.GUIDANCE})
    want = orc.linear_combine(obe, opol, vals, coefs)
    tv = [to_torch(v) for v in vals]
    be2 = ops.B200Backend(execution_dtype=torch.float32 if dt == "f32" else torch.bfloat16)
    got = ops.fused_linear_combine(be2, pol, tv, coefs)
    assert_bits_equal(got, want, "linear_combine")
    chain = ops.linear_combine(be2, pol, tv, coefs)
    view = torch.int16 if dt == "bf16" else torch.int32
    assert torch.equal(got.view(view), chain.view(view))
