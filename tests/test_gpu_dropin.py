"""The C++ host layer as a drop-in: vrhino_b200::B200Backend (vrhino_b200/host) wrapped around the
reference's own CudaBackend, built by `make -C oracle dropin` against the reference's headers.

The SAME call sequences that produced the golden vectors on the reference's CUDA backend
(tests/golden/cases.py: run_reference, i.e. the reference's unmodified helper code -- modulate,
attention_norm, operation_rope, gated_residual, SamplingPrimitives ...) are run with the replaced
backend behind the `Backend&`, and compared with those golden vectors under the tolerances of
test_golden.py.  Then the fused call-site forms, and the error / session behaviour.

Skipped where the drop-in library has not been built (it needs the reference's headers).
"""
import os
import sys

import numpy as np
import pytest

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.join(HERE, "golden"))

import cases  # noqa: E402
from test_golden import compare, golden  # noqa: E402,F401  (fixture)

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def dropin():
    from oracle import ref
    if not ref.available_dropin():
        pytest.skip("oracle/_ref/libvrhino_dropin_cuda.so has not been built (make -C oracle dropin)")
    import torch
    if not torch.cuda.is_available():
        pytest.skip("needs a GPU")
    rd = ref.RefDropin()
    assert rd.name().startswith("b200+")
    yield rd
    rd.lib.refc_shutdown()


@pytest.mark.parametrize("case", cases.CASES, ids=[c["name"] for c in cases.CASES])
def test_reference_call_sites_on_the_replaced_backend(orc, golden, dropin, case):
    want = golden[case["name"]]
    got = cases.run_reference(dropin, case)
    assert set(got) == set(want)
    for name in want:
        compare(orc, case, name, got[name], want[name], strict_tables=True, who="library (C++ drop-in backend)")


def _upload(rd, case):
    from oracle import ref
    code = {"f32": ref.F32, "bf16": ref.BF16}
    return {k: rd.upload(cases.to_bits(a, dt), code[dt]) for k, (a, dt) in cases._inputs(case).items() if dt != "u8"}


def _grab(rd, case, handle, shape):
    from oracle import ref
    payload, dt = rd.download(handle, shape)
    return cases._sub(case, payload), {ref.F32: "f32", ref.BF16: "bf16"}[dt]


@pytest.mark.parametrize("case", [c for c in cases.CASES if c["kind"] in
                                  ("ln_modulate", "rms_rope", "gated_residual", "mochi", "group_norm", "sampler", "linear_output",
                                   "pixel_norm", "depth_to_space")],
                         ids=lambda c: c["name"])
def test_fused_call_site_forms(orc, golden, dropin, case):
    """One kernel per chain through vrhino_b200::layer_norm_modulate / rms_norm_rope / ... ."""
    from oracle import ref
    rd, want, k = dropin, golden[case["name"]], case["kind"]
    h = _upload(rd, case)
    pol = ref.POLICY_BF16
    try:
        if k == "ln_modulate":
            got = rd.fused_layer_norm_modulate(pol, h["x"], 0, 0, cases.EPS, h["shift"], h["scale"])
            compare(orc, case, "cast", _grab(rd, case, got, case["shape"]), want["cast"])
        elif k == "rms_rope":
            S, H, d = case["tokens"], case["heads"], case["head_dim"]
            got = rd.fused_rms_norm_rope(pol, h["x"], h["w"], 1e-5 if case["per_head"] else cases.EPS, h["cos"], h["sin"], H,
                                         per_head=case["per_head"])
            compare(orc, case, "cast", _grab(rd, case, got, (1, S, H, d)), want["cast"])
            got = rd.fused_rms_norm_rope(pol, h["x"], h["w"], 1e-5 if case["per_head"] else cases.EPS, 0, 0, H,
                                         per_head=case["per_head"])
            compare(orc, case, "norm_cast", _grab(rd, case, got, (1, S, H, d)), want["norm_cast"])
            # q and k of one attention in one launch: each half is what the single launch gives
            eps = 1e-5 if case["per_head"] else cases.EPS
            other = rd.upload(cases.to_bits(np.random.default_rng(5).normal(1.0, 0.1, cases._inputs(case)["w"][0].shape)
                                            .astype(np.float32), "f32"), ref.F32)
            first, second = rd.fused_rms_norm_rope_pair(pol, h["x"], h["w"], h["x"], other, eps, h["cos"], h["sin"], H,
                                                        per_head=case["per_head"])
            compare(orc, case, "cast", _grab(rd, case, first, (1, S, H, d)), want["cast"])
            alone = rd.fused_rms_norm_rope(pol, h["x"], other, eps, h["cos"], h["sin"], H, per_head=case["per_head"])
            assert np.array_equal(rd.download(second, (1, S, H, d))[0], rd.download(alone, (1, S, H, d))[0])
        elif k == "gated_residual":
            p = ref.POLICY_BF16 if case["state"] == "bf16" else ref.POLICY_FP32
            compare(orc, case, "gated", _grab(rd, case, rd.fused_gated_residual(p, h["res"], h["branch"], h["gate"]), case["shape"]),
                    want["gated"])
            compare(orc, case, "added", _grab(rd, case, rd.fused_gated_residual(p, h["res"], h["branch"], 0), case["shape"]),
                    want["added"])
            # the update together with the LayerNorm that reads the updated stream next: the stream
            # against the golden vector, the normalised tensor bit for bit against the replaced
            # backend's own layer_norm -> modulate -> cast on that stream
            width = case["shape"][-1]
            vec = lambda seed, mean, std: rd.upload(cases.to_bits(np.random.default_rng(seed).normal(mean, std, (1, 1, width))
                                                                  .astype(np.float32), "f32"), ref.F32)
            w, b, shift, scale = vec(1, 1.0, 0.1), vec(2, 0.0, 0.1), vec(3, 0.0, 0.1), vec(4, 0.0, 0.1)
            for gate, key in ((h["gate"], "gated"), (0, "added")):
                for affine, modulated in ((True, False), (False, True), (False, False)):
                    state, normed = rd.fused_gated_residual_layer_norm(p, h["res"], h["branch"], gate, w if affine else 0,
                                                                       b if affine else 0, cases.EPS, shift if modulated else 0,
                                                                       scale if modulated else 0)
                    compare(orc, case, key, _grab(rd, case, state, case["shape"]), want[key])
                    chain = rd.layer_norm(state, w if affine else 0, b if affine else 0, cases.EPS)
                    if modulated:
                        chain = rd.modulate(p, chain, shift, scale)
                    chain = rd.cast(chain, ref.BF16)
                    got_bits, got_dt = rd.download(normed, case["shape"])
                    want_bits, want_dt = rd.download(chain, case["shape"])
                    assert got_dt == want_dt == ref.BF16
                    if case["state"] == "bf16" and not modulated:
                        assert np.array_equal(got_bits, want_bits)
                    else:   # the one-kernel modulate rounds once where the chain rounds per operator
                        compare(orc, case, "normed", (cases._sub(case, got_bits), "bf16"), (cases._sub(case, want_bits), "bf16"))
        elif k == "depth_to_space":
            b, c, t, h_, w = case["shape"]
            got = rd.fused_depth_to_space_residual(h["y"], h["x"])
            compare(orc, case, "depth_to_space", _grab(rd, case, got, (b, c // 2, 2 * t - 1, 2 * h_, 2 * w)), want["depth_to_space"])
        elif k == "pixel_norm":
            got = rd.fused_pixel_norm_modulate_silu(pol, h["x"], h["shift"], h["scale"], 1e-8)
            compare(orc, case, "silu", _grab(rd, case, got, case["shape"]), want["silu"], strict_tables=True)
            got = rd.fused_pixel_norm_modulate_silu(pol, h["x"], h["shift"], h["scale"], 1e-8, ref.BF16)
            compare(orc, case, "cast", _grab(rd, case, got, case["shape"]), want["cast"], strict_tables=True)
        elif k == "linear_output":
            # the device runtime's GEMM (exact accumulators in this case) + the merged epilogue kernels,
            # bit for bit against the reference's linear -> consumer chain
            M, N = case["m"], case["n"]
            p = ref.POLICY_BF16 if case["state"] == "bf16" else ref.POLICY_FP32
            for kind, name in ((2, "gelu_tanh"), (0, "silu")):
                got = rd.fused_linear_activation(h["x"], h["w"], h["bias"], kind)
                compare(orc, case, name, _grab(rd, case, got, (1, M, N)), want[name], strict_tables=True)
            compare(orc, case, "gated", _grab(rd, case, rd.fused_linear_gated_residual(p, h["res"], h["x"], h["w"], h["bias"], h["gate"]),
                                              (1, M, N)), want["gated"])
            compare(orc, case, "added", _grab(rd, case, rd.fused_linear_gated_residual(p, h["res"], h["x"], h["w"], h["bias"], 0),
                                              (1, M, N)), want["added"])
            compare(orc, case, "swiglu", _grab(rd, case, rd.fused_linear_swiglu(h["x"], h["w"], h["bias"]), (1, M, N // 2)),
                    want["swiglu"], strict_tables=True)
        elif k == "mochi":
            B, S, D = case["shape"]
            compare(orc, case, "swiglu", _grab(rd, case, rd.fused_swiglu(h["proj"]), (B, S, case["hidden"])), want["swiglu"])
            # the layer boundary in one kernel: the updated stream against the golden vector, the next
            # layer's pre-norm against the replaced backend's own rms_norm -> (1 + scale) chain on that stream
            p = ref.POLICY_BF16 if case["state"] == "bf16" else ref.POLICY_FP32
            state, normed = rd.fused_mochi_residual_norm(p, h["x"], h["branch"], h["gate"], h["scale"], cases.EPS)
            compare(orc, case, "norm_gated", _grab(rd, case, state, (B, S, D)), want["norm_gated"])
            one = rd.host_f32(np.array(1.0, dtype=np.float32))
            chain = rd.binary(1, rd.rms_norm(state, 0, cases.EPS), rd.binary(0, one, rd.reshape(h["scale"], (B, 1, D))))
            got_bits, got_dt = rd.download(normed, (B, S, D))
            want_bits, want_dt = rd.download(chain, (B, S, D))
            assert got_dt == want_dt
            compare(orc, case, "norm_scale", (cases._sub(case, got_bits), "bf16" if got_dt == ref.BF16 else "f32"),
                    (cases._sub(case, want_bits), "bf16" if want_dt == ref.BF16 else "f32"))
        elif k == "group_norm":
            got = rd.fused_group_norm_silu(h["x"], case["groups"], h["w"], h["b"], case["eps"])
            compare(orc, case, "silu", _grab(rd, case, got, case["shape"]), want["silu"])
        elif k == "sampler":
            rd.lib.refc_init(ref.F32 if case["policy"] == "fp32" else ref.BF16)
            roles = case["policy"] == "bf16_roles"
            delta = 0.02
            if case["policy"] == "bf16":     # no solver role: the coefficient tensor is rounded to the execution dtype
                delta = float(orc.bf16_bits_to_f32(cases.to_bits(np.array([0.02], dtype=np.float32), "bf16"))[0])
            got = rd.fused_cfg_euler(h["x"], h["u"], h["c"], 5.0, delta, True, roles, roles)
            rd.lib.refc_init(ref.BF16)
            compare(orc, case, "euler", _grab(rd, case, got, case["shape"]), want["euler"])
    finally:
        rd.clear()


def test_edge_time_pad_call_site(orc, dropin):
    """vrhino_b200::edge_time_pad on the replaced backend (one pass) against the reference's CUDA backend running
    LTX's two pads (ltx.cpp:210-214), bit for bit."""
    from oracle import ref
    from vrhino_b200 import synth
    if not ref.available_cuda():
        pytest.skip("reference CUDA library not built")
    shape = (1, 8, 3, 6, 16)
    bits = cases.to_bits(synth.normal(shape, seed=41), "bf16")
    rc = ref.RefCuda()
    want = rc.pad(rc.pad(rc.upload(bits, ref.BF16), [0, 0, 0, 0, 1, 1], 0.0, True), [1, 1, 1, 1], 0.0, False)
    want_bits, _ = rc.download(want, (1, 8, 5, 8, 18))
    rc.clear()
    got = dropin.fused_edge_time_pad(dropin.upload(bits, ref.BF16), 1, 1, 1)
    got_bits, dt = dropin.download(got, (1, 8, 5, 8, 18))
    dropin.clear()
    assert dt == ref.BF16 and np.array_equal(got_bits, want_bits)


@pytest.mark.parametrize("hidden", ["bf16", "f32"])
def test_graph_fusion_pass(orc, dropin, hidden):
    """The non-GEMM part of the Wan self-attention graph (the reference's node sequence, q / k / the
    attention projection supplied as inputs) evaluated three ways: the reference's evaluator on
    the reference's CUDA backend; the reference's evaluator on the replaced backend (node by
    node); vrhino_b200::evaluate_fused, which must find 1 LayerNorm-modulate, 2 RMSNorm-RoPE and
    1 gated-residual chain and launch nothing for the nodes inside them."""
    from oracle import ref
    from vrhino_b200 import synth
    if not ref.available_cuda():
        pytest.skip("reference CUDA library not built")
    S, W, H, d = 600, 1536, 12, 128
    hd = ref.BF16 if hidden == "bf16" else ref.F32
    n = lambda shape, st, mean=0.0, std=1.0: synth.normal(shape, mean, std, seed=77, stream=st)
    cos, sin = synth.wan_rope_tables(2, 15, 20, head_dim=d)
    host = {
        "hidden": (n((1, S, W), 0), hidden), "modulation": (n((1, 6, W), 1, 0, 0.1), "f32"),
        "cos": (cos.reshape(1, S, 1, d), "f32"), "sin": (sin.reshape(1, S, 1, d), "f32"),
        "q": (n((1, S, W), 2), "bf16"), "k": (n((1, S, W), 3), "bf16"), "proj": (n((1, S, W), 4), "bf16"),
        "table": (n((1, 6, W), 5, 0, 0.1), "f32"), "norm_q": (n((W,), 6, 1.0, 0.1), "f32"), "norm_k": (n((W,), 7, 1.0, 0.1), "f32"),
    }
    order = ["hidden", "modulation", "cos", "sin", "q", "k", "proj", "table", "norm_q", "norm_k"]
    code = {"f32": ref.F32, "bf16": ref.BF16}
    shapes = [(1, S, W), (1, S, H, d), (1, S, H, d), (1, S, W)]

    def run(backend, fused):
        handles = [backend.upload(cases.to_bits(host[k][0], host[k][1]), code[host[k][1]]) for k in order]
        outs, stats = backend.wan_chain_graph(S, W, H, hd, 1e-6, handles, fused=fused)
        got = [backend.download(o, shape) for o, shape in zip(outs, shapes)]
        backend.clear()
        return got, stats

    rc = ref.RefCuda()
    want, _ = run(rc, False)
    node_by_node, _ = run(dropin, False)
    fused, stats = run(dropin, True)
    assert stats[:3] == [1, 2, 1], stats
    assert stats[4] >= 9, stats            # LN, (cast), mul, add, 1+scale; 2 x (rms, reshape, rope); casts, mul
    undrained, _ = run(dropin, 2)          # no per-graph device synchronisation: same stream order, same bits
    for (g, _), (w, _) in zip(undrained, fused):
        assert np.array_equal(g, w)
    for got in (node_by_node, fused):
        for (g, gdt), (w, wdt), name in zip(got, want, ("attention input", "q operand", "k operand", "residual")):
            assert gdt == wdt and g.shape == w.shape, name
            if name == "residual":         # exact casts, one F32 multiply, one F32 add
                assert np.array_equal(g.view(np.uint32), w.view(np.uint32)), name
                continue
            dist = orc.bf16_ulp_distance(g, w)
            bad = dist > 2
            if bad.any():                   # RoPE cancellation: see test_golden.compare
                diff = np.abs(orc.bf16_bits_to_f32(g).astype(np.float64) - orc.bf16_bits_to_f32(w).astype(np.float64))
                assert name != "attention input" and bad.mean() <= 2e-3 and (diff[bad] <= 2.0 ** -8 * 8.0).all(), (name, int(bad.sum()))


@pytest.mark.parametrize("dt", ["bf16", "f32"])
def test_frame_group_norm_without_permutes(orc, dropin, dt):
    """Mochi's frame_group_norm: the reference permutes [B,C,T,H,W] to frames, normalises and permutes
    back on its CUDA backend; vrhino_b200::frame_group_norm reads and writes the tensor as it lies."""
    from oracle import ref
    from vrhino_b200 import synth
    if not ref.available_cuda():
        pytest.skip("reference CUDA library not built")
    shape, groups = (1, 64, 5, 24, 40), 32
    code = {"f32": ref.F32, "bf16": ref.BF16}[dt]
    x = cases.to_bits(synth.normal(shape, 0.3, 2.0, seed=3), dt)
    w, b = synth.normal((64,), 1.0, 0.1, seed=1), synth.normal((64,), 0.0, 0.1, seed=2)

    def run(backend):
        hx, hw, hb = backend.upload(x, code), backend.upload(w, ref.F32), backend.upload(b, ref.F32)
        out, _ = backend.download(backend.frame_group_norm(hx, groups, hw, hb, 1e-5, silu=False), shape)
        backend.clear()
        return out

    want, got = run(ref.RefCuda()), run(dropin)
    if dt == "bf16":
        d = orc.bf16_ulp_distance(got, want)
        diff = np.abs(orc.bf16_bits_to_f32(got).astype(np.float64) - orc.bf16_bits_to_f32(want).astype(np.float64))
        assert ((d <= 2) | (diff <= 2e-6)).all(), int(d.max())
    else:
        diff = np.abs(got.astype(np.float64) - want.astype(np.float64))
        assert (diff <= 2e-6 + 1e-5 * np.abs(want)).all(), float(diff.max())


def test_production_wan_graph_with_fusion(orc, dropin):
    """The reference's production Wan self-attention graph itself
    (native/src/architectures/wan_self_attention_graph.h), GEMMs and attention included, on a small
    configuration (256 wide, 2 heads, 128 tokens): the reference's evaluator on its CUDA backend
    against evaluate_fused on the replaced backend.  GEMM and attention run in the reference's own
    code on both sides; the fused chains may flip single bf16 roundings of their operands, so the
    F32 residual is compared statistically (mean |d| <= 2e-3, max |d| <= 5e-2 on O(1) values)."""
    from oracle import ref
    from vrhino_b200 import synth
    if not ref.available_cuda():
        pytest.skip("reference CUDA library not built")
    S, W, H = 128, 256, 2
    d = W // H
    n = lambda shape, st, mean=0.0, std=1.0: synth.normal(shape, mean, std, seed=91, stream=st)
    cos, sin = synth.wan_rope_tables(2, 8, 8, head_dim=d)
    lin = 1.0 / np.sqrt(W)
    host = [
        (n((1, S, W), 0), "bf16"), (n((1, 6, W), 1, 0, 0.1), "f32"), (cos.reshape(1, S, 1, d), "f32"), (sin.reshape(1, S, 1, d), "f32"),
        (n((1, 6, W), 2, 0, 0.1), "f32"),
        (n((W, W), 3, 0, lin), "bf16"), (n((W,), 4, 0, 0.02), "bf16"), (n((W, W), 5, 0, lin), "bf16"), (n((W,), 6, 0, 0.02), "bf16"),
        (n((W, W), 7, 0, lin), "bf16"), (n((W,), 8, 0, 0.02), "bf16"),
        (n((W,), 9, 1.0, 0.1), "f32"), (n((W,), 10, 1.0, 0.1), "f32"),
        (n((W, W), 11, 0, lin), "bf16"), (n((W,), 12, 0, 0.02), "bf16"),
    ]
    code = {"f32": ref.F32, "bf16": ref.BF16}

    def run(backend, fused):
        handles = [backend.upload(cases.to_bits(a, dt), code[dt]) for a, dt in host]
        outs, stats = backend.wan_self_attention_graph(S, W, H, handles, fused=fused)
        residual, _ = backend.download(outs[0], (1, S, W))
        combined, _ = backend.download(outs[1], (1, 6, W))
        backend.clear()
        return residual, combined, stats

    rc = ref.RefCuda()
    want, want_combined, _ = run(rc, False)
    got, got_combined, stats = run(dropin, True)
    assert stats[:3] == [1, 2, 1], stats
    assert np.array_equal(got_combined.view(np.uint32), want_combined.view(np.uint32))
    assert np.isfinite(want).all() and np.abs(want).max() > 0.5
    diff = np.abs(got.astype(np.float64) - want.astype(np.float64))
    assert diff.mean() <= 2e-3 and diff.max() <= 5e-2, (float(diff.mean()), float(diff.max()))


@pytest.mark.parametrize("hidden", ["f32", "bf16"])
def test_production_ltx_graph_with_fusion(orc, dropin, hidden):
    """The reference's production LTX self-attention graph (width 2048, 32 heads; RMSNorm-modulate,
    q/k RMSNorm + RoPE with whole-row bf16 tables, gated residual; GEMMs and attention in the
    reference's code) for 2 x 96 tokens: reference evaluator on its CUDA backend against
    evaluate_fused on the replaced backend.  Statistical bound as for the Wan graph."""
    from oracle import ref
    from vrhino_b200 import synth
    if not ref.available_cuda():
        pytest.skip("reference CUDA library not built")
    B, S, W = 2, 96, 2048
    n = lambda shape, st, mean=0.0, std=1.0: synth.normal(shape, mean, std, seed=55, stream=st)
    phase = synth.uniform_range((B, S, W // 2), -3.0, 3.0, seed=55, stream=20)
    cos, sin = np.repeat(np.cos(phase), 2, axis=-1).astype(np.float32), np.repeat(np.sin(phase), 2, axis=-1).astype(np.float32)
    lin = 1.0 / np.sqrt(W)
    host = [
        (n((B, S, W), 0), hidden), (n((B, 1, 6 * W), 1, 0, 0.1), "f32"), (cos, "bf16"), (sin, "bf16"),
        (n((6, W), 2, 0, 0.1), "bf16"),
        (n((W, W), 3, 0, lin), "bf16"), (n((W,), 4, 0, 0.02), "bf16"), (n((W, W), 5, 0, lin), "bf16"), (n((W,), 6, 0, 0.02), "bf16"),
        (n((W, W), 7, 0, lin), "bf16"), (n((W,), 8, 0, 0.02), "bf16"),
        (n((W,), 9, 1.0, 0.1), "bf16"), (n((W,), 10, 1.0, 0.1), "bf16"),
        (n((W, W), 11, 0, lin), "bf16"), (n((W,), 12, 0, 0.02), "bf16"),
    ]
    code = {"f32": ref.F32, "bf16": ref.BF16}

    def run(backend, fused):
        handles = [backend.upload(cases.to_bits(a, dt), code[dt]) for a, dt in host]
        out, stats = backend.ltx_self_attention_graph(B, S, hidden == "bf16", handles, fused=fused)
        residual, _ = backend.download(out, (B, S, W))
        backend.clear()
        return residual, stats

    want, _ = run(ref.RefCuda(), False)
    got, stats = run(dropin, True)
    assert stats[:3] == [1, 2, 1], stats
    assert np.isfinite(want).all() and np.abs(want).max() > 0.5
    diff = np.abs(got.astype(np.float64) - want.astype(np.float64))
    assert diff.mean() <= 2e-3 and diff.max() <= 5e-2, (float(diff.mean()), float(diff.max()))


def test_errors_and_session_semantics(dropin):
    """Same texts as the reference's wrappers; a rejected argument in an unguarded operator
    (layer_norm) leaves the session usable, one in a guarded operator (clamp) retires it, after
    which every call fails with the reference's terminal-session message."""
    from oracle import ref
    rd = dropin
    try:
        x = rd.upload(np.zeros((2, 8), dtype=np.float32), ref.F32)
        w = rd.upload(np.ones((7,), dtype=np.float32), ref.F32)
        with pytest.raises(RuntimeError, match="layer norm weight mismatch"):
            rd.layer_norm(x, w, 0, 1e-5)
        assert not rd.session_terminal()
        a, _ = rd.download(rd.layer_norm(x, 0, 0, 1e-5), (2, 8))
        assert np.isfinite(a).all()
        with pytest.raises(RuntimeError, match="Invalid clamp bounds"):
            rd.clamp(x, 1.0, 0.0)
        assert rd.session_terminal()
        with pytest.raises(RuntimeError, match="Resource session is terminal"):
            rd.activation(x, 0)
    finally:
        rd.lib.refc_shutdown()          # a fresh backend for whoever uses the library next
        rd.lib.refc_init(ref.BF16)


def test_merged_linear_forms_on_a_dense_gemm(orc, dropin):
    """A dense K=512 GEMM: the merged forms take the device runtime's F32 accumulation, the stock chain
    takes whichever plan the reference's linear picks for a bf16 result, so accumulators may differ in
    their last bits: <= 2 bf16 ulp (activation, SwiGLU) and the gated residual within one bf16 ulp of
    the branch."""
    from oracle import ref
    rd = dropin
    rng = np.random.default_rng(3)
    M, N, K = 256, 1536, 512
    up = lambda a, dt=ref.BF16: rd.upload(cases.to_bits(a.astype(np.float32), "bf16" if dt == ref.BF16 else "f32"), dt)
    x, w = up(rng.normal(0, 1, (1, M, K))), up(rng.normal(0, K ** -0.5, (N, K)))
    bias, res, gate = up(rng.normal(0, 0.5, (N,))), up(rng.normal(0, 1, (1, M, N))), up(rng.normal(0, 0.3, (1, 1, N)), ref.F32)
    case = {"name": "dense_gemm", "kind": "dense_linear"}
    try:
        lin = rd.linear(x, w, bias)
        pairs = [
            ("gelu_tanh", rd.fused_linear_activation(x, w, bias, 2), rd.activation(lin, 2), (1, M, N)),
            ("gated", rd.fused_linear_gated_residual(ref.POLICY_BF16, res, x, w, bias, gate),
             rd.gated_residual(ref.POLICY_BF16, res, lin, gate), (1, M, N)),
            ("swiglu", rd.fused_linear_swiglu(x, w, bias),
             rd.binary(1, rd.slice(lin, 2, 0, N // 2), rd.activation(rd.slice(lin, 2, N // 2, N), 0)), (1, M, N // 2)),
        ]
        for name, got, want, shape in pairs:
            g, gdt = rd.download(got, shape)
            w_, wdt = rd.download(want, shape)
            assert gdt == wdt == ref.BF16
            d = orc.bf16_ulp_distance(g, w_)
            assert (d <= 2).mean() >= 0.998, f"{name}: {(d > 2).sum()} of {d.size} beyond 2 ulp"
            diff = np.abs(orc.bf16_bits_to_f32(g).astype(np.float64) - orc.bf16_bits_to_f32(w_).astype(np.float64))
            assert diff.max() <= 2.0 ** -8 * 8.0, f"{name}: max difference {diff.max()}"
    finally:
        rd.clear()


def test_replaced_operators_appear_in_profile_stats_under_the_reference_names(dropin):
    """The reference's operators record themselves in profile_stats() (cuda_backend.cu:3011-3064, e.g.
    "norm.layer|rows=..|width=..|dtype=.." :4073-4076).  The replaced operators keep those names, and
    the backend adds the bytes each one moved."""
    from oracle import ref
    rd = dropin
    rng = np.random.default_rng(5)
    x = rd.upload(cases.to_bits(rng.standard_normal((1, 40, 1536)).astype(np.float32), "bf16"), ref.BF16)
    w = rd.upload(rng.standard_normal(1536).astype(np.float32), ref.F32)
    rd.profile(True)
    try:
        made = [rd.layer_norm(x, None, None, 1e-6), rd.rms_norm(x, w, 1e-6), rd.activation(x, 2), rd.binary(0, x, x),
                rd.cast(x, ref.F32), rd.clamp(x, -1.0, 1.0), rd.permute(x, (0, 2, 1)), rd.slice(x, 2, 0, 768), rd.concat([x, x], 1),
                rd.pad(x, [0, 0, 1, 1], 0.0, True),
                rd.fused_layer_norm_modulate(ref.POLICY_BF16, x, None, None, 1e-6,
                                             rd.upload(rng.standard_normal((1, 1, 1536)).astype(np.float32), ref.F32),
                                             rd.upload(rng.standard_normal((1, 1, 1536)).astype(np.float32), ref.F32))]
        report = rd.profile_report()
    finally:
        rd.profile(False)
    nbytes = 40 * 1536 * 2
    expected = {
        "norm.layer|rows=40|width=1536|dtype=bfloat16": 2 * nbytes,
        "norm.rms|rows=40|width=1536|axis=2|dtype=bfloat16": 2 * nbytes,
        "activation|elements=61440|kind=2|dtype=bfloat16": 2 * nbytes,
        "elementwise.add": 3 * nbytes,
        "cast": 3 * nbytes,
        "clamp": 2 * nbytes,
        "permute": 2 * nbytes, "slice": nbytes, "concat": 4 * nbytes, "pad": 2 * nbytes,
        "fused.norm.layer+modulate": 2 * nbytes,
    }
    for name, moved in expected.items():
        assert name in report, (name, sorted(report))
        calls, ms, recorded = report[name]
        assert calls >= 1 and ms > 0.0 and recorded >= moved, (name, report[name])
    for h in made:
        rd.free(h)


def test_dequantised_weight_is_decoded_once(dropin):
    """linear() on a quantised weight uploads and decodes it on every call in the reference
    (cuda_backend.cu:3276-3295); the replaced backend keeps the decoded weight, within a byte budget,
    until release_cached_device_memory()."""
    from oracle import ref
    rd = dropin
    rng = np.random.default_rng(6)
    rows, inner = 64, 256
    packed = rng.integers(0, 254, size=(rows, inner)).astype(np.uint8)
    scales = rng.uniform(1e-3, 1e-2, size=(rows, 1)).astype(np.float32)
    once = rd.dequantize(0, packed, scales, rows, inner, inner, ref.BF16)
    want, _ = rd.download(once, (rows, inner))
    _, before = rd.dequantize_repeated(0, packed, scales, rows, inner, inner, ref.BF16, repeats=0)
    h, after = rd.dequantize_repeated(0, packed, scales, rows, inner, inner, ref.BF16, repeats=3)
    got, _ = rd.download(h, (rows, inner))
    assert np.array_equal(got, want)
    assert after["misses"] - before["misses"] == 1 and after["hits"] - before["hits"] == 2
    assert after["resident_bytes"] >= rows * inner * 2
    assert rd.release_cached() == 0
    # a budget smaller than the weight: decoded per call, nothing kept
    h2, small = rd.dequantize_repeated(0, packed, scales, rows, inner, inner, ref.BF16, repeats=2, budget=1024)
    assert small["hits"] == after["hits"] and small["misses"] - after["misses"] == 2 and small["resident_bytes"] == 0
    got2, _ = rd.download(h2, (rows, inner))
    assert np.array_equal(got2, want)
    rd.dequantize_repeated(0, packed, scales, rows, inner, inner, ref.BF16, repeats=0, budget=48 << 30)


def test_l2_normalize_reference_kernel_oracle_and_drop_in_agree(orc, dropin):
    """No golden vector exists for l2_normalize, so the three are compared live: the reference's own kernel
    (its CUDA backend compiled for sm_100a), the CPU oracle that restates it (bit for bit on F32: same
    summation order), and the replaced backend (other summation order: <= 2 bf16 ulp / 1e-5)."""
    from oracle import ref
    if not ref.available_cuda():
        pytest.skip("oracle/_ref/libvrhino_ref_cuda.so has not been built")
    rc = ref.RefCuda()
    rng = np.random.default_rng(8)
    try:
        for shape, dt in (((1, 512, 6, 10), "f32"), ((2, 256, 5, 8), "bf16"), ((3, 40), "f32")):
            x = (rng.standard_normal(shape) * 1.5 + 0.2).astype(np.float32)
            bits = cases.to_bits(x, dt)
            code = {"f32": ref.F32, "bf16": ref.BF16}[dt]
            reference, _ = rc.download(rc.l2_normalize(rc.upload(bits, code), 1, 1e-10), shape)
            mine, _ = dropin.download(dropin.l2_normalize(dropin.upload(bits, code), 1, 1e-10), shape)
            want = orc.OracleBackend().l2_normalize(orc.T(bits, dt), 1, 1e-10)
            if dt == "f32":
                assert np.array_equal(want.data.view(np.uint32), reference.view(np.uint32)), "oracle vs the reference's kernel"
                assert np.allclose(mine, reference, rtol=1e-5, atol=1e-8)
            else:
                assert orc.bf16_ulp_distance(want.data, reference).max() <= 1
                assert orc.bf16_ulp_distance(mine, reference).max() <= 2
    finally:
        rc.lib.refc_shutdown()
