"""The CPU oracle against the REFERENCE's own host path (native/tests/family_lowering_test_backend.h
driven through the reference's helper seams), compiled from the reference's sources by
`make -C oracle ref_host` into oracle/_ref/libvrhino_ref_host.so.

The host backend is F32 only.  Chains of single IEEE operations (modulate, gated_residual,
residual_add, RoPE, cfg_combine, euler_update) must agree bit for bit; LayerNorm / RMSNorm use
different-but-equivalent formulas on the two sides (two-pass variance and a division by sqrt on the
host, E[x^2]-mean^2 and rsqrtf in the CUDA kernel the oracle restates), so they are compared at the
reference's own F32 gate 2e-5 + 2e-5|r| (docs/protocol/numerical-boundary-contract.md:10-12)."""
import os
import subprocess

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module")
def host(orc):
    from oracle import ref
    if not ref.available_host() and os.path.isdir(ref.reference_tree()):
        subprocess.run(["make", "-C", os.path.join(ROOT, "oracle"), "-j4", "ref_host"], check=True, capture_output=True)
    if not ref.available_host():
        pytest.skip("oracle/_ref/libvrhino_ref_host.so is not built and the reference tree is not mounted")
    return ref.RefHost()


@pytest.fixture(scope="module")
def be(orc):
    return orc.OracleBackend(execution_dtype=orc.F32)


def gate(a, r):
    assert (np.abs(a - r) <= 2e-5 + 2e-5 * np.abs(r)).all(), float(np.abs(a - r).max())


def data(shape, seed, mean=0.0, std=1.0):
    from vrhino_b200 import synth
    return synth.normal(shape, mean, std, seed=seed)


@pytest.mark.parametrize("width", [17, 128, 1536])
def test_layer_norm_and_rms_norm(orc, be, host, width):
    x, w, b = data((5, width), 1), data((width,), 2, 1.0, 0.1), data((width,), 3, 0.0, 0.1)
    gate(be.layer_norm(orc.tensor(x), None, None, 1e-6).data, host.layer_norm(x, None, None, 1e-6))
    gate(be.layer_norm(orc.tensor(x), orc.tensor(w), orc.tensor(b), 1e-5).data, host.layer_norm(x, w, b, 1e-5))
    gate(be.rms_norm(orc.tensor(x), orc.tensor(w), 1e-6).data, host.rms_norm(x, w, 1e-6))
    gate(be.rms_norm(orc.tensor(x), None, 1e-6).data, host.rms_norm(x, None, 1e-6))


def test_activations(orc, be, host):
    x = data((4096,), 4, 0.0, 2.0)
    for kind in (orc.SILU, orc.GELU_TANH):
        gate(be.activation(orc.tensor(x), kind).data, host.activation(x, kind))


def test_rope_bit_exact(orc, be, host):
    x = data((1, 6, 3, 128), 5)
    ph = np.linspace(-3, 3, 6 * 128, dtype=np.float32).reshape(1, 6, 1, 128)
    c, s = np.cos(ph).astype(np.float32), np.sin(ph).astype(np.float32)
    got = be.rope_nd(orc.tensor(x), orc.tensor(c), orc.tensor(s)).data
    assert np.array_equal(got, host.rope(x, c, s))


def test_modulate_and_residuals_bit_exact(orc, be, host):
    policy = orc.Policy.fp32()
    x, sh, sc = data((1, 7, 96), 6), data((1, 1, 96), 7, 0.0, 0.1), data((1, 1, 96), 8, 0.0, 0.1)
    assert np.array_equal(orc.modulate(be, policy, orc.tensor(x), orc.tensor(sh), orc.tensor(sc)).data, host.modulate(x, sh, sc))
    br, g = data((1, 7, 96), 9), data((1, 1, 96), 10, 0.0, 0.3)
    assert np.array_equal(orc.gated_residual(be, policy, orc.tensor(x), orc.tensor(br), orc.tensor(g)).data,
                          host.gated_residual(x, br, g))
    assert np.array_equal(orc.residual_add(be, policy, orc.tensor(x), orc.tensor(br)).data, host.gated_residual(x, br, None))


def test_cfg_and_euler_bit_exact(orc, be, host):
    policy = orc.Policy.fp32()
    x, u, c = data((999,), 11), data((999,), 12), data((999,), 13)
    guided, out = host.cfg_euler(x, u, c, 5.0, 0.02)
    g = orc.cfg_combine(be, policy, orc.tensor(u), orc.tensor(c), 5.0)
    assert np.array_equal(g.data, guided)
    assert np.array_equal(orc.euler_update(be, policy, orc.tensor(x), g, orc.scalar_f32(0.02), True).data, out)


def test_layout_operators_bit_exact(orc, be, host):
    """permute / slice / the one pad the host backend implements: pure copies, bit for bit; the sinusoidal embedding
    (the host backend's phase is always double) against the oracle's double path at the F32 gate."""
    x = data((2, 3, 4, 5), 11)
    for axes in ((0, 2, 1, 3), (3, 2, 1, 0), (1, 0, 3, 2), (0, 1, 2, 3)):
        assert np.array_equal(be.permute(orc.tensor(x), axes).data, host.permute(x, axes))
    for axis, start, stop in ((3, 1, 4), (1, 0, 2), (0, 1, 2), (2, 3, 4)):
        assert np.array_equal(be.slice(orc.tensor(x), axis, start, stop).data, host.slice(x, axis, start, stop))
    rows = data((3, 8), 12)
    assert np.array_equal(be.pad(orc.tensor(rows[None]), [0, 0, 0, 2], -0.5).data[0], host.pad_rows(rows, 2, -0.5))
    positions = np.array([0.0, 1.0, 0.5, 999.0, 37.25, -2.0], dtype=np.float32)
    for width, flip, shift in ((256, True, 0.0), (64, False, 1.0), (6, True, 0.0)):
        gate(be.sinusoidal_embedding(orc.tensor(positions), width, flip, shift, True).data, host.sinusoidal_embedding(positions, width, flip, shift))


def test_reference_chain_runs_threaded(host):
    sec, nbytes = host.wan_chain_seconds(tokens=64, threads=2, steps=1, ffn=256)
    assert sec > 0 and nbytes > 0
