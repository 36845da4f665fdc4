"""GPU parity of LayerNorm / RMSNorm and their fused chains against the CPU oracle.

LayerNorm statistics are accumulated in double exactly as the reference does, so for bf16
inputs mean and variance are bit-identical and only rsqrtf (CUDA) vs 1/sqrtf (C) can differ,
by 1-2 F32 ulp: outputs are compared at <= 2 bf16 ulp / 1e-5 relative.  RMSNorm statistics
are F32 sums whose order depends on the launch geometry; same tolerance.
"""
import numpy as np
import pytest

from conftest import assert_bits_equal, assert_close, from_torch, to_torch

pytestmark = pytest.mark.gpu

DTYPES = ["f32", "bf16"]
# tail, sub-warp, warp, production and wide rows; 17 / 257 / 6 exercise the scalar kernel
WIDTHS = [6, 17, 64, 128, 257, 1536, 2048, 3072, 5120, 8192]


def _torch_dtype(tag):
    import torch
    return torch.float32 if tag == "f32" else torch.bfloat16


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("width", WIDTHS)
@pytest.mark.parametrize("affine", [False, True])
def test_layer_norm(orc, gpu, dtype, width, affine):
    be, ops = gpu
    from vrhino_b200 import synth
    rows = 5
    x = orc.tensor(synth.normal((1, rows, width), seed=width), dtype)
    w = orc.tensor(synth.normal((width,), 1.0, 0.1, seed=1), "f32") if affine else None
    b = orc.tensor(synth.normal((width,), 0.0, 0.1, seed=2), "f32") if affine else None
    want = orc.OracleBackend().layer_norm(x, w, b, 1e-6)
    got = be.layer_norm(to_torch(x), to_torch(w) if affine else None, to_torch(b) if affine else None, 1e-6)
    # outputs near zero come from x - mean cancelling: absolute 2e-6 (the reference's own F32 gate
    # is 2e-5 + 2e-5|r|, native/tests/neural_graph_layernorm_tests.cpp:161)
    frac = assert_close(orc, got, want, rel=1e-5, atol=2e-6, what=f"layer_norm w={width}")
    if dtype == "bf16":
        assert frac < 0.02, "more than 2% of the bf16 outputs are not bit-identical to the oracle"


def test_layer_norm_repeat_is_bit_exact(gpu):
    """primitive_tests.cpp:130-144 (exact_repeat)."""
    import torch
    be, ops = gpu
    x = torch.randn(64, 1536, device="cuda", dtype=torch.bfloat16)
    a, b = be.layer_norm(x, None, None, 1e-6), be.layer_norm(x, None, None, 1e-6)
    assert torch.equal(a.view(torch.int16), b.view(torch.int16))
    a, b = be.rms_norm(x, None, 1e-6), be.rms_norm(x, None, 1e-6)
    assert torch.equal(a.view(torch.int16), b.view(torch.int16))


def test_layer_norm_known_reference_limitation_is_reproduced(orc, gpu):
    """Rows of 1000 / nextafter(1000): the reference kernel's E[x^2] - float(mean)^2 goes
    negative and it returns NaN (its release notes list this as its one failing public test,
    native/tests/neural_graph_layernorm_tests.cpp:230-260).  Same formula here, same NaNs; the
    centred and constant patterns stay finite and match."""
    be, ops = gpu
    low = np.float32(1000.0)
    high = np.nextafter(low, np.float32(np.inf))
    for width in (16, 1536, 5120):
        lane = np.arange(width) % 4
        for values in (np.where(lane == 0, low, high), np.array([-0.25, 0.25, 0.5, -0.5], dtype=np.float32)[lane], np.full(width, low)):
            x = orc.tensor(values.astype(np.float32).reshape(1, width))
            want = orc.OracleBackend(execution_dtype="f32").layer_norm(x, None, None, 1e-6)
            got, _ = from_torch(be.layer_norm(to_torch(x), None, None, 1e-6))
            assert np.array_equal(np.isnan(got), np.isnan(want.data))
            finite = ~np.isnan(want.data)
            assert np.allclose(got[finite], want.data[finite], rtol=1e-5, atol=1e-7)


@pytest.mark.parametrize("in_dt,out_dt,weighted", [("f32", "f32", True), ("f32", "f32", False), ("bf16", "bf16", True),
                                                  ("bf16", "bf16", False), ("bf16", "f32", True)])
@pytest.mark.parametrize("width", WIDTHS)
def test_rms_norm(orc, gpu, in_dt, out_dt, weighted, width):
    be, ops = gpu
    from vrhino_b200 import synth
    rows = 600 if width <= 2048 else 16   # >= 512 rows selects the reference's one-warp schedule
    x = orc.tensor(synth.normal((rows, width), seed=width + 1), in_dt)
    w = orc.tensor(synth.normal((width,), 1.0, 0.1, seed=3), "f32") if weighted else None
    want = orc.OracleBackend().rms_norm(x, w, 1e-6, -1, None if out_dt == in_dt else out_dt)
    got = be.rms_norm(to_torch(x), to_torch(w) if weighted else None, 1e-6, -1, None if out_dt == in_dt else _torch_dtype(out_dt))
    # bf16 -> F32 output: the normalised value is rounded to bf16 before the weight multiply
    flips = dict(flip_atol=2.0 ** -8 * 8.0, flip_frac=2e-3) if (in_dt, out_dt) == ("bf16", "f32") else {}
    assert_close(orc, got, want, rel=1e-5, what=f"rms_norm w={width}", **flips)


def test_rms_norm_rejections(gpu):
    import torch
    be, ops = gpu
    x = torch.zeros(4, 64, device="cuda", dtype=torch.bfloat16)
    with pytest.raises(ops.VrbError, match="BF16-to-FP32 rms_norm requires affine weight"):
        be.rms_norm(x, None, 1e-6, -1, torch.float32)
    with pytest.raises(ops.VrbError, match="rms_norm output dtype unsupported"):
        be.rms_norm(x.float(), None, 1e-6, -1, torch.bfloat16)
    with pytest.raises(ops.VrbError, match="rms norm weight mismatch"):
        be.rms_norm(x, torch.ones(63, device="cuda"), 1e-6)
    with pytest.raises(ops.VrbError, match="rms_norm axis invalid"):
        be.rms_norm(x, None, 1e-6, 5)


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("shape,axis", [((2, 5, 3), 1), ((2, 7, 4, 5), 1), ((2, 3, 9, 5), 2), ((1, 17, 2, 3, 5), 1), ((1, 96, 2, 8, 16), 1),
                                        ((2, 384, 1, 5, 8), 1), ((1, 1024, 1, 3, 16), 1), ((1, 3000, 1, 1, 16), 1), ((3, 13, 1, 1, 24), 1)])
def test_rms_norm_axis(orc, gpu, dtype, shape, axis):
    """primitive_tests.cpp:406-424 shapes plus Wan-VAE-like [1, C, T, H, W] tensors that take the
    shared-memory tile path (full and ragged tiles, 8 / 4 / 2 / 1 chunks per channel row)."""
    be, ops = gpu
    from vrhino_b200 import synth
    x = orc.tensor(synth.normal(shape, seed=9), dtype)
    w = orc.tensor(synth.normal((shape[axis],), 1.0, 0.1, seed=4), "f32")
    want = orc.OracleBackend().rms_norm(x, w, 1e-6, axis)
    got = be.rms_norm(to_torch(x), to_torch(w), 1e-6, axis)
    assert_close(orc, got, want, rel=1e-5, what="rms axis")
    if axis == 1:
        want_s = orc.rms_channel_silu(orc.OracleBackend(), x, w, 1e-12)
        got_s = ops.fused_rms_channel_silu(be, to_torch(x), to_torch(w), 1e-12)
        assert_close(orc, got_s, want_s, rel=1e-5, what="rms channel + silu")
        # bit-identical to the two operators run one after the other (the fused form reads SiLU of common
        # magnitudes from a table built with the same expression)
        import torch
        chain = be.activation(be.rms_norm(to_torch(x), to_torch(w), 1e-12, 1), ops.SILU)
        view = torch.int16 if dtype == "bf16" else torch.int32
        assert torch.equal(got_s.view(view), chain.view(view))


# ------------------------------------------------------------------------------ fused chains --
@pytest.mark.parametrize("x_dt", DTYPES)
@pytest.mark.parametrize("out_dt", DTYPES)
@pytest.mark.parametrize("width,batch,per_token", [(1536, 1, False), (1536, 2, False), (1536, 3, False), (1536, 4, False), (1536, 5, False),
                                                    (64, 2, True), (17, 1, False), (5120, 1, False), (5120, 2, False)])
def test_layer_norm_modulate(orc, gpu, x_dt, out_dt, width, batch, per_token):
    """Config-1 chain: layer_norm(no affine) -> modulate -> consumer cast, vs the same chain of
    per-operator kernels and vs the oracle."""
    be, ops = gpu
    from vrhino_b200 import synth
    tokens = 7
    obe, opol = orc.OracleBackend(), orc.Policy()
    x = orc.tensor(synth.normal((batch, tokens, width), seed=width), x_dt)
    mshape = (batch, tokens if per_token else 1, width)
    shift = orc.tensor(synth.normal(mshape, std=0.1, seed=1), "f32")
    scale = orc.tensor(synth.normal(mshape, std=0.1, seed=2), "f32")
    want = obe.cast(orc.modulate(obe, opol, obe.layer_norm(x, None, None, 1e-6), shift, scale), out_dt)
    tx, tsh, tsc = to_torch(x), to_torch(shift), to_torch(scale)
    got = ops.fused_layer_norm_modulate(be, tx, None, None, 1e-6, tsh, tsc, _torch_dtype(out_dt))
    flips = dict(flip_atol=2.0 ** -8 * 8.0, flip_frac=2e-3) if (x_dt, out_dt) == ("bf16", "f32") else {}
    assert_close(orc, got, want, rel=1e-5, atol=2e-6, what="fused ln+modulate", **flips)
    chain = be.cast(ops.modulate(be, ops.Policy(), be.layer_norm(tx, None, None, 1e-6), tsh, tsc), _torch_dtype(out_dt))
    import torch
    assert torch.equal(chain.view(torch.int16 if out_dt == "bf16" else torch.int32),
                       got.view(torch.int16 if out_dt == "bf16" else torch.int32)), "fused != per-op chain"


def test_layer_norm_affine_modulate(orc, gpu):
    """norm with gamma/beta followed by modulation (CogVideoX, native/src/architectures/cogvideox.cpp:35-60)."""
    be, ops = gpu
    from vrhino_b200 import synth
    obe = orc.OracleBackend()
    x = orc.tensor(synth.normal((2, 9, 1920), seed=5), "bf16")
    w, b = orc.tensor(synth.normal((1920,), 1.0, 0.1, seed=6)), orc.tensor(synth.normal((1920,), 0.0, 0.1, seed=7))
    shift, scale = orc.tensor(synth.normal((2, 1, 1920), std=0.1, seed=8)), orc.tensor(synth.normal((2, 1, 1920), std=0.1, seed=9))
    want = obe.cast(orc.modulate(obe, orc.Policy(), obe.layer_norm(x, w, b, 1e-5), shift, scale), "bf16")
    got = ops.fused_layer_norm_modulate(be, to_torch(x), to_torch(w), to_torch(b), 1e-5, to_torch(shift), to_torch(scale))
    assert_close(orc, got, want, what="ln affine + modulate")


@pytest.mark.parametrize("x_dt", DTYPES)
@pytest.mark.parametrize("width,batch,per_token", [(2048, 2, False), (2048, 2, True), (24, 1, False)])
def test_rms_norm_modulate(orc, gpu, x_dt, width, batch, per_token):
    """LTX: rms_norm(no weight, 1e-6) -> modulate, per-batch and per-token vectors."""
    be, ops = gpu
    from vrhino_b200 import synth
    tokens = 5
    obe = orc.OracleBackend()
    x = orc.tensor(synth.normal((batch, tokens, width), seed=3), x_dt)
    mshape = (batch, tokens if per_token else 1, width)
    shift, scale = orc.tensor(synth.normal(mshape, std=0.1, seed=1)), orc.tensor(synth.normal(mshape, std=0.1, seed=2))
    want = obe.cast(orc.modulate(obe, orc.Policy(), obe.rms_norm(x, None, 1e-6), shift, scale), "bf16")
    got = ops.fused_rms_norm_modulate(be, to_torch(x), 1e-6, to_torch(shift), to_torch(scale))
    assert_close(orc, got, want, what="rms + modulate")


@pytest.mark.parametrize("x_dt", DTYPES)
@pytest.mark.parametrize("width,batch", [(3072, 1), (1536, 2), (40, 1)])
def test_rms_norm_scale_mochi(orc, gpu, x_dt, width, batch):
    be, ops = gpu
    from vrhino_b200 import synth
    obe = orc.OracleBackend()
    x = orc.tensor(synth.normal((batch, 6, width), seed=4), x_dt)
    scale = orc.tensor(synth.normal((batch, width), std=0.1, seed=5), "f32")
    want = orc.mochi_norm_scale(obe, x, scale)
    got = ops.fused_rms_norm_scale(be, to_torch(x), to_torch(scale), 1e-6)
    assert_close(orc, got, want, rel=1e-5, what="mochi rms*(1+scale)")


@pytest.mark.parametrize("out_dt", DTYPES)
@pytest.mark.parametrize("mode", ["wan", "wan_no_rope", "mochi_per_head_tables", "hunyuan_shared_tables", "ltx_per_batch_tables"])
def test_rms_norm_rope(orc, gpu, out_dt, mode):
    """attention_norm -> split_heads -> operation_rope -> attention operand cast.  (LTX: the norm over the full
    width, then tables [B, S, width] of its own for every batch entry, ltx_self_attention_graph.cpp:30-44.)"""
    be, ops = gpu
    from vrhino_b200 import synth
    obe, opol = orc.OracleBackend(), orc.Policy()
    heads, d = (12, 128) if mode.startswith("wan") else (24, 128) if mode.startswith("mochi") else (4, 64)
    tokens, width = 2 * 3 * 4, heads * d
    batch = 2 if mode.startswith("ltx") else 1
    x = orc.tensor(synth.normal((batch, tokens, width), seed=7), "bf16")
    per_head = not (mode.startswith("wan") or mode.startswith("ltx"))
    wn = d if per_head else width
    w = orc.tensor(synth.normal((wn,), 1.0, 0.1, seed=8), "f32")
    if mode == "wan" or mode == "hunyuan_shared_tables":
        if mode == "wan":
            c, s = synth.wan_rope_tables(2, 3, 4, d)
        else:
            ph = synth.uniform_range((1, tokens, 1, d), -3, 3, seed=9)
            c, s = np.cos(ph), np.sin(ph)
    elif mode == "mochi_per_head_tables" or mode == "ltx_per_batch_tables":
        ph = synth.uniform_range((batch, tokens, heads, d), -3, 3, seed=9)
        c, s = np.cos(ph), np.sin(ph)
    else:
        c = s = None
    eps = 1e-6 if mode.startswith("wan") else 1e-5
    if per_head:
        normed = orc.attention_norm(obe, opol, x.reshape((batch, tokens, heads, d)), w, eps)
    else:
        normed = orc.attention_norm(obe, opol, x, w, eps).reshape((batch, tokens, heads, d))
    if c is not None:
        co, si = orc.tensor(c), orc.tensor(s)
        normed = orc.operation_rope(obe, opol, normed, co, si)
    want = obe.cast(normed, out_dt).reshape((batch, tokens, width))
    got = ops.fused_rms_norm_rope(be, to_torch(x), to_torch(w), eps, to_torch(co) if c is not None else None,
                                  to_torch(si) if c is not None else None, heads=heads, per_head_norm=per_head,
                                  out_dtype=_torch_dtype(out_dt))
    assert_close(orc, got, want, rel=1e-5, atol=1e-6, flip_atol=2.0 ** -8 * 8.0, flip_frac=2e-3, what=f"rms+rope {mode}")


@pytest.mark.parametrize("state", DTYPES)
@pytest.mark.parametrize("width,batch", [(3072, 1), (1536, 2), (24, 1)])
def test_rms_norm_gated_residual_mochi(orc, gpu, state, width, batch):
    import torch
    be, ops = gpu
    from vrhino_b200 import synth
    obe = orc.OracleBackend()
    opol = orc.Policy(residual=state)
    pol = ops.Policy(residual=_torch_dtype(state))
    res = orc.tensor(synth.normal((batch, 5, width), seed=1), state)
    branch = orc.tensor(synth.normal((batch, 5, width), seed=2), "bf16")
    gate = orc.tensor(synth.normal((batch, width), std=0.5, seed=3), "f32")
    want = orc.normalized_gated_residual(obe, opol, res, branch, gate)
    bounded = be.activation(to_torch(gate), ops.TANH)
    got = ops.fused_rms_norm_gated_residual(be, pol, to_torch(res), to_torch(branch), bounded, 1e-6)
    assert_close(orc, got, want, rel=1e-5, atol=1e-6, what="mochi normalized gated residual")


@pytest.mark.parametrize("state", DTYPES)
@pytest.mark.parametrize("width,batch,tokens", [(3072, 1, 37), (3072, 2, 9), (1536, 2, 300), (264, 1, 11), (24, 3, 5)])
def test_mochi_residual_update_merged_with_the_next_pre_norm(orc, gpu, state, width, batch, tokens):
    """mochi.cpp:204-211 then :228-231: x' = x + rms_norm(branch) * tanh(gate);  y = rms_norm(x') * (1 + scale).
    The one-kernel form (bf16 stream) gives the bits of this library's three launches (tanh, residual update,
    pre-norm), and both agree with the oracle's operator chain; an F32 stream takes the separate launches."""
    import torch
    be, ops = gpu
    from vrhino_b200 import synth
    obe = orc.OracleBackend()
    opol = orc.Policy(residual=state)
    pol = ops.Policy(residual=_torch_dtype(state))
    res = orc.tensor(synth.normal((batch, tokens, width), seed=1), state)
    branch = orc.tensor(synth.normal((batch, tokens, width), seed=2), "bf16")
    gate = orc.tensor(synth.normal((batch, width), std=0.5, seed=3), "f32")
    scale = orc.tensor(synth.normal((batch, 1, width), std=0.1, seed=4), "f32")
    want_state = orc.normalized_gated_residual(obe, opol, res, branch, gate)
    want_out = orc.mochi_norm_scale(obe, want_state, scale)
    got_state, got_out = ops.fused_rms_norm_gated_residual_norm_scale(be, pol, to_torch(res), to_torch(branch), to_torch(gate),
                                                                      to_torch(scale))
    bounded = be.activation(to_torch(gate), ops.TANH)
    sep_state = ops.fused_rms_norm_gated_residual(be, pol, to_torch(res), to_torch(branch), bounded, 1e-6)
    sep_out = ops.fused_rms_norm_scale(be, sep_state, to_torch(scale), 1e-6)
    view = torch.int16 if state == "bf16" else torch.int32
    assert torch.equal(got_state.view(view), sep_state.view(view)), "merged stream differs from the separate launches"
    assert torch.equal(got_out.view(view), sep_out.view(view)), "merged pre-norm differs from the separate launches"
    assert_close(orc, got_state, want_state, rel=1e-5, atol=1e-6, what=f"mochi merged: stream {state} {width}")
    assert_close(orc, got_out, want_out, rel=1e-5, atol=1e-6, flip_atol=2.0 ** -8 * 8.0, flip_frac=2e-3,
                 what=f"mochi merged: pre-norm {state} {width}")


@pytest.mark.parametrize("width,batch,tokens", [(1536, 1, 21), (1536, 2, 9), (5120, 1, 5), (3072, 2, 6), (2048, 1, 7), (128, 1, 40),
                                                (264, 1, 11), (24, 3, 5)])
@pytest.mark.parametrize("gated", [True, False])
@pytest.mark.parametrize("mode", ["affine", "modulate", "plain"])
@pytest.mark.parametrize("state", ["bf16", "f32"])
def test_gated_residual_layer_norm_one_pass(orc, gpu, width, batch, tokens, gated, mode, state):
    """Residual update + the LayerNorm that follows it (one kernel for a bf16 stream, the two
    operators otherwise): the updated stream must be bit-identical to gated_residual / residual_add,
    the normalised output bit-identical to running the norm kernel on that stream, and both match
    the oracle's unfused chain."""
    import torch
    be, ops = gpu
    from vrhino_b200 import synth
    obe = orc.OracleBackend()
    opol = orc.Policy.unqualified_default("bf16") if state == "bf16" else orc.Policy.fp32()
    pol = ops.Policy.unqualified_default(torch.bfloat16) if state == "bf16" else ops.Policy.fp32()
    shape = (batch, tokens, width)
    res = orc.tensor(synth.normal(shape, seed=width + 1), state)
    branch = orc.tensor(synth.normal(shape, seed=width + 2), "bf16")
    gate = orc.tensor(synth.normal((batch, 1, width), std=0.3, seed=3)) if gated else None
    w = orc.tensor(synth.normal((width,), 1.0, 0.1, seed=4)) if mode == "affine" else None
    b = orc.tensor(synth.normal((width,), 0.0, 0.1, seed=5)) if mode == "affine" else None
    shift = orc.tensor(synth.normal((batch, 1, width), std=0.1, seed=6)) if mode == "modulate" else None
    scale = orc.tensor(synth.normal((batch, 1, width), std=0.1, seed=7)) if mode == "modulate" else None
    T = lambda t: None if t is None else to_torch(t)
    got_state, got_norm = ops.fused_gated_residual_layer_norm(be, pol, T(res), T(branch), T(gate), T(w), T(b), 1e-6, T(shift), T(scale))
    # against this library's separate kernels: identical bits
    sep_state = ops.fused_gated_residual(be, pol, T(res), T(branch), T(gate))
    if mode == "modulate":
        sep_norm = ops.fused_layer_norm_modulate(be, sep_state, None, None, 1e-6, T(shift), T(scale))
    else:
        sep_norm = ops.fused_layer_norm_cast(be, sep_state, T(w), T(b), 1e-6)
    bits = lambda t: t.view(torch.int16 if t.dtype == torch.bfloat16 else torch.int32)
    assert torch.equal(bits(got_state), bits(sep_state)), "updated stream differs from gated_residual"
    assert torch.equal(bits(got_norm), bits(sep_norm)), "normalised output differs from the norm kernel on the same stream"
    # against the oracle's chain
    want_state = orc.gated_residual(obe, opol, res, branch, gate) if gated else orc.residual_add(obe, opol, res, branch)
    assert_bits_equal(got_state, want_state, "state")
    normed = obe.layer_norm(want_state, w, b, 1e-6)
    want = obe.cast(orc.modulate(obe, opol, normed, shift, scale), "bf16") if mode == "modulate" else obe.cast(normed, "bf16")
    flips = dict(flip_atol=2.0 ** -8 * 8.0, flip_frac=2e-3)
    assert_close(orc, got_norm, want, rel=1e-5, atol=2e-6, what="norm after residual update", **flips)



@pytest.mark.parametrize("width,batch,tokens", [(2048, 2, 9), (2048, 1, 5), (1536, 3, 4), (264, 1, 7), (24, 2, 5)])
@pytest.mark.parametrize("gated", [True, False])
@pytest.mark.parametrize("state", ["bf16", "f32"])
def test_gated_residual_rms_norm_modulate_one_pass(orc, gpu, width, batch, tokens, gated, state):
    """The LTX form (residual update + RMSNorm without weight + modulate): bit-identical to this
    library's two launches, the updated stream bit-exact and the output within tolerance of the
    oracle's unfused chain."""
    import torch
    be, ops = gpu
    from vrhino_b200 import synth
    obe = orc.OracleBackend()
    opol = orc.Policy.unqualified_default("bf16") if state == "bf16" else orc.Policy.fp32()
    pol = ops.Policy.unqualified_default(torch.bfloat16) if state == "bf16" else ops.Policy.fp32()
    shape = (batch, tokens, width)
    res = orc.tensor(synth.normal(shape, seed=width + 1), state)
    branch = orc.tensor(synth.normal(shape, seed=width + 2), "bf16")
    gate = orc.tensor(synth.normal((batch, 1, width), std=0.3, seed=3)) if gated else None
    shift = orc.tensor(synth.normal((batch, 1, width), std=0.1, seed=6))
    scale = orc.tensor(synth.normal((batch, 1, width), std=0.1, seed=7))
    T = lambda t: None if t is None else to_torch(t)
    got_state, got_norm = ops.fused_gated_residual_rms_norm_modulate(be, pol, T(res), T(branch), T(gate), 1e-6, T(shift), T(scale))
    sep_state = ops.fused_gated_residual(be, pol, T(res), T(branch), T(gate))
    sep_norm = ops.fused_rms_norm_modulate(be, sep_state, 1e-6, T(shift), T(scale))
    bits = lambda t: t.view(torch.int16 if t.dtype == torch.bfloat16 else torch.int32)
    assert torch.equal(bits(got_state), bits(sep_state))
    assert torch.equal(bits(got_norm), bits(sep_norm))
    want_state = orc.gated_residual(obe, opol, res, branch, gate) if gated else orc.residual_add(obe, opol, res, branch)
    assert_bits_equal(got_state, want_state, "state")
    want = obe.cast(orc.modulate(obe, opol, obe.rms_norm(want_state, None, 1e-6), shift, scale), "bf16")
    assert_close(orc, got_norm, want, rel=1e-5, atol=2e-6, what="rms norm after residual update", flip_atol=2.0 ** -8 * 8.0, flip_frac=2e-3)
