"""Times the REFERENCE's own CUDA kernels (cuda_backend.cu compiled for sm_100a into
``oracle/_ref/libvrhino_ref_cuda.so``) on the headline operator chains, through the reference's own
helper seams (layer_norm -> modulate, attention_norm -> operation_rope, gated_residual, activation,
group_norm -> activation, quantised copy_to_device, cfg_combine -> euler_update).

TEST / BASELINE INFRASTRUCTURE ONLY: this is the "GPU number to beat", reported beside the
library's own; nothing in the product path uses it.  Run as a process of its own

    python -m oracle.ref_timing [--config wan21|wan22|wan22_sampler|vae_gn|mochi|vae_layout] [--tokens N] [--repeat R]

and it prints one JSON object.  Each seam is bracketed by a device synchronisation and timed with the
host clock (the seams take 0.1-3 ms, far above launch latency); where the reference's profiler is
available its summed device time is reported as well.
"""
from __future__ import annotations

import argparse
import json
import sys
import time

import numpy as np

from . import ref

GELU_TANH, SILU = 2, 0


def _bf16_bits(a: np.ndarray) -> np.ndarray:
    """float32 -> bf16 bit patterns, round to nearest even (finite inputs)."""
    u = np.ascontiguousarray(a, dtype=np.float32).view(np.uint32)
    return ((u + np.uint32(0x7FFF) + ((u >> np.uint32(16)) & np.uint32(1))) >> np.uint32(16)).astype(np.uint16)


class Pool:
    """Seeded N(0,1) values for tensors of any size: a 4 Mi-element random block repeated.  The kernels
    timed here are data-independent, so only the distribution matters, not the period."""

    def __init__(self, seed):
        self.rng = np.random.default_rng(seed)
        self.block = self.rng.standard_normal(1 << 22, dtype=np.float32)

    def standard_normal(self, shape, dtype=np.float32):
        shape = (shape,) if isinstance(shape, int) else tuple(shape)
        n = int(np.prod(shape))
        start = int(self.rng.integers(0, self.block.size))
        return np.resize(np.roll(self.block, -start), n).reshape(shape)

    def uniform(self, lo, hi, size):
        return self.rng.uniform(lo, hi, size=size)

    def integers(self, *a, **k):
        return self.rng.integers(*a, **k)


class Timer:
    def __init__(self, rc: ref.RefCuda, repeat: int):
        self.rc, self.repeat, self.rows = rc, repeat, []

    def seam(self, name, algorithmic_bytes, fn):
        """fn() runs the seam and returns the handles it created (freed here)."""
        rc = self.rc
        for h in fn():
            rc.free(h)
        rc.synchronize()
        best = None
        for _ in range(self.repeat):
            rc.synchronize()
            t0 = time.perf_counter()
            handles = fn()
            rc.synchronize()
            dt = time.perf_counter() - t0
            for h in handles:
                rc.free(h)
            best = dt if best is None else min(best, dt)
        self.rows.append({"seam": name, "us": best * 1e6, "algorithmic_mb": algorithmic_bytes / 1e6,
                          "gbs_of_algorithmic_bytes": algorithmic_bytes / best / 1e9})

    def result(self, **extra):
        return {"seams": self.rows, "us": sum(r["us"] for r in self.rows),
                "algorithmic_mb": sum(r["algorithmic_mb"] for r in self.rows), **extra}


def wan_chain(rc, tokens, dim, heads, ffn, repeat, text=512, seed=0):
    """One CFG branch of the Wan block chain, bf16 hidden state, through the reference's seams."""
    rng = Pool(seed)
    P = ref.POLICY_BF16
    S, D, d = tokens, dim, dim // heads
    up = lambda shape, std=1.0, mean=0.0: rc.upload(_bf16_bits(rng.standard_normal(shape, dtype=np.float32) * std + mean), ref.BF16)
    upf = lambda shape, std=1.0, mean=0.0: rc.upload((rng.standard_normal(shape, dtype=np.float32) * std + mean).astype(np.float32), ref.F32)
    x, q, k, proj, cq, cross, fo = (up((1, S, D)) for _ in range(7))
    ck = up((1, text, D))
    fh = up((1, S, ffn))
    mod = [upf((1, 1, D), 0.1) for _ in range(6)]
    wq, wk, wcq, wck, g3 = (upf((D,), 0.1, 1.0) for _ in range(5))
    b3 = upf((D,), 0.1)
    phase = rng.uniform(-3, 3, size=(1, S, 1, d)).astype(np.float32)
    cos, sin = rc.upload(np.cos(phase), ref.F32), rc.upload(np.sin(phase), ref.F32)
    t = Timer(rc, repeat)
    act, vec, table = S * D, D * 4, S * d * 4 * 2

    def ln_mod(shift, scale):
        a = rc.layer_norm(x, None, None, 1e-6)
        b = rc.modulate(P, a, shift, scale)
        c = rc.cast(b, ref.BF16)
        return [a, b, c]

    def norm_rope(src, w):
        a = rc.attention_norm(P, src, w, 1e-6)
        b = rc.reshape(a, (1, S, heads, d))
        c = rc.operation_rope(P, b, cos, sin)
        e = rc.cast(c, ref.BF16)
        return [a, b, c, e]

    def norm_only(src, w):
        a = rc.attention_norm(P, src, w, 1e-6)
        return [a, rc.cast(a, ref.BF16)]

    t.seam("A ln_modulate", act * 4 + 2 * vec, lambda: ln_mod(mod[0], mod[1]))
    t.seam("B rms_rope q", act * 4 + vec + table // 2, lambda: norm_rope(q, wq))
    t.seam("B rms_rope k", act * 4 + vec + table // 2, lambda: norm_rope(k, wk))
    t.seam("C gated_residual", act * 6 + vec, lambda: [rc.gated_residual(P, x, proj, mod[2])])
    t.seam("D ln_affine", act * 4 + 2 * vec, lambda: [rc.layer_norm(x, g3, b3, 1e-6)])
    t.seam("E rms cross q", act * 4 + vec, lambda: norm_only(cq, wcq))
    t.seam("E rms cross k", text * D * 4 + vec, lambda: norm_only(ck, wck))
    t.seam("F residual_add", act * 6, lambda: [rc.residual_add(P, x, cross)])
    t.seam("G ln_modulate", act * 4 + 2 * vec, lambda: ln_mod(mod[3], mod[4]))
    t.seam("H gelu_tanh", S * ffn * 4, lambda: [rc.activation(fh, GELU_TANH)])
    t.seam("I gated_residual", act * 6 + vec, lambda: [rc.gated_residual(P, x, fo, mod[5])])
    return t.result(tokens=S, dim=D, ffn=ffn, branches=1,
                    note="one CFG branch (the reference's graphs take batch 1); a block runs it twice")


def sampler_and_dequant(rc, repeat, seed=1):
    rng = np.random.default_rng(seed)
    P = ref.POLICY_FP32
    shape = (1, 16, 21, 60, 104)
    x, u, c = (rc.upload(rng.standard_normal(shape, dtype=np.float32), ref.F32) for _ in range(3))
    n = int(np.prod(shape))
    t = Timer(rc, repeat)

    def cfg_euler():
        g = rc.cfg_combine(P, u, c, 5.0)
        return [g, rc.euler_update(P, x, g, 0.02, True)]

    t.seam("cfg_combine + euler_update (F32 latent)", n * 16, cfg_euler)
    rows, inner = 5120, 13824
    codes = rng.integers(0, 254, size=(rows, inner), dtype=np.int16)
    packed = (codes + (codes >= 127)).astype(np.uint8)
    scales = rng.uniform(1e-3, 1e-2, size=(rows, 1)).astype(np.float32)
    rc.lib.refc_profile(1)
    calls = (ref._c.c_int64 * 1)()
    before = rc.lib.refc_profile_total_ms(calls)
    handle = rc.dequantize(0, packed, scales, rows, inner, inner, ref.BF16)
    rc.synchronize()
    after = rc.lib.refc_profile_total_ms(calls)
    rc.lib.refc_profile(0)
    rc.free(handle)
    out = t.result()
    if before >= 0 and after > before:
        out["fp8_dequant_5120x13824_device_us_from_reference_profiler"] = (after - before) * 1e3
        out["fp8_dequant_note"] = "quantised copy_to_device: the profiler's device time covers the upload of the codes and dequantize_kernel"
    return out


def vae_group_norm(rc, repeat, frames=28, seed=2):
    rng = Pool(seed)
    shape = (1, 256, frames, 240, 424)
    n = int(np.prod(shape))
    bits = np.empty(shape, dtype=np.uint16)
    for c0 in range(0, 256, 32):                       # in slabs: bounds the host scratch
        bits[:, c0:c0 + 32] = _bf16_bits(rng.standard_normal((1, 32) + shape[2:], dtype=np.float32) * 2.0)
    x = rc.upload(bits, ref.BF16)
    del bits
    gamma = rc.upload((1 + 0.1 * rng.standard_normal(256)).astype(np.float32), ref.F32)
    beta = rc.upload((0.1 * rng.standard_normal(256)).astype(np.float32), ref.F32)
    t = Timer(rc, repeat)

    def gn_silu():
        a = rc.group_norm(x, 32, gamma, beta, 1e-6)
        return [a, rc.activation(a, SILU)]

    t.seam("group_norm + silu", n * 6, gn_silu)
    return t.result(shape=list(shape))


def mochi(rc, tokens, repeat, seed=3):
    """SwiGLU through split + silu + mul, and the per-head q norm + RoPE, at the Mochi sizes."""
    rng = Pool(seed)
    P = ref.POLICY_BF16
    S, H, d, hidden = tokens, 24, 128, 8192
    t = Timer(rc, repeat)
    proj = rc.upload(_bf16_bits(rng.standard_normal((1, S, 2 * hidden), dtype=np.float32)), ref.BF16)

    def swiglu():
        a = rc.slice(proj, 2, 0, hidden)
        g = rc.slice(proj, 2, hidden, 2 * hidden)
        s = rc.activation(g, SILU)
        return [a, g, s, rc.binary(1, a, s)]

    t.seam("swiglu (slice, slice, silu, mul)", S * hidden * 6, swiglu)
    rc.free(proj)
    q = rc.upload(_bf16_bits(rng.standard_normal((1, S, H, d), dtype=np.float32)), ref.BF16)
    w = rc.upload((1 + 0.1 * rng.standard_normal(d)).astype(np.float32), ref.F32)
    phase = rng.uniform(-3, 3, size=(1, S, H, d)).astype(np.float32)
    cos, sin = rc.upload(np.cos(phase), ref.F32), rc.upload(np.sin(phase), ref.F32)

    def head_norm_rope():
        a = rc.attention_norm(P, q, w, 1e-5)
        b = rc.operation_rope(P, a, cos, sin)
        return [a, b, rc.cast(b, ref.BF16)]

    t.seam("per-head rms_rope q", S * H * d * (4 + 8), head_norm_rope)
    return t.result(tokens=S)


def vae_layout(rc, repeat, frames=8, seed=4):
    """LTX / Wan VAE kernels outside the headline chains: pixel_norm -> modulate -> silu (ltx.cpp:221-227), the two pads in
    front of an LTX convolution (ltx.cpp:205-215), rms_channel + silu of the Wan VAE, and the Wan patch embedding's
    transposition (wan.cpp:159), on the shapes `workloads --config 10 / 12 / 13` use."""
    rng = Pool(seed)
    P = ref.POLICY_BF16
    t = Timer(rc, repeat)
    shape = (1, 128, frames, 256, 384)
    n = int(np.prod(shape))
    x = rc.upload(_bf16_bits(rng.standard_normal(shape, dtype=np.float32) * 1.5 + 0.2), ref.BF16)
    shift = rc.upload((0.2 * rng.standard_normal((1, 128, 1, 1, 1))).astype(np.float32), ref.F32)
    scale = rc.upload((0.2 * rng.standard_normal((1, 128, 1, 1, 1))).astype(np.float32), ref.F32)

    def norm_chain():
        a = rc.pixel_norm(x, 1, 1e-8)
        b = rc.modulate(P, a, shift, scale)
        return [a, b, rc.activation(b, SILU)]

    def pads():
        a = rc.pad(x, [0, 0, 0, 0, 1, 1], 0.0, True)
        return [a, rc.pad(a, [1, 1, 1, 1], 0.0, False)]

    t.seam("pixel_norm", n * 4, lambda: [rc.pixel_norm(x, 1, 1e-8)])
    t.seam("pixel_norm -> modulate -> silu (F32 result)", n * 6, norm_chain)
    t.seam("pad T replicate, then pad H, W zero", n * 2 + n * 2 * (frames + 2) * 258 * 386 // (frames * 256 * 384), pads)
    t.seam("permute frames first (0,2,1,3,4)", n * 4, lambda: [rc.permute(x, (0, 2, 1, 3, 4))])
    rc.free(x)
    wan = (1, 192, 4, 240, 416)
    m = int(np.prod(wan))
    y = rc.upload(_bf16_bits(rng.standard_normal(wan, dtype=np.float32)), ref.BF16)
    gamma = rc.upload((1 + 0.1 * rng.standard_normal(192)).astype(np.float32), ref.F32)

    def rms_silu():
        a = rc.rms_norm(y, gamma, 1e-12, axis=1)
        return [a, rc.activation(a, SILU)]

    t.seam("rms_channel", m * 4, lambda: [rc.rms_norm(y, gamma, 1e-12, axis=1)])
    t.seam("rms_channel -> silu", m * 4, rms_silu)
    rc.free(y)
    patches = rc.upload(_bf16_bits(rng.standard_normal((1, 1536, 32760), dtype=np.float32)), ref.BF16)
    t.seam("permute [1,1536,32760] -> [1,32760,1536]", 1536 * 32760 * 4, lambda: [rc.permute(patches, (0, 2, 1))])
    return t.result(shape=list(shape))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--config", default="wan21", choices=["wan21", "wan22", "wan22_sampler", "vae_gn", "mochi", "vae_layout"])
    ap.add_argument("--tokens", type=int, default=None)
    ap.add_argument("--frames", type=int, default=28)
    ap.add_argument("--repeat", type=int, default=3)
    a = ap.parse_args()
    if not ref.available_cuda():
        print(json.dumps({"unavailable": "oracle/_ref/libvrhino_ref_cuda.so has not been built"}))
        return
    rc = ref.RefCuda(ref.BF16)
    if a.config == "wan21":
        out = wan_chain(rc, a.tokens or 32760, 1536, 12, 8960, a.repeat)
    elif a.config == "wan22":
        out = wan_chain(rc, a.tokens or 32760, 5120, 40, 13824, a.repeat)
    elif a.config == "wan22_sampler":
        out = sampler_and_dequant(rc, a.repeat)
    elif a.config == "vae_gn":
        out = vae_group_norm(rc, a.repeat, frames=a.frames)
    elif a.config == "vae_layout":
        out = vae_layout(rc, a.repeat)
    else:
        out = mochi(rc, a.tokens or 44520, a.repeat)
    out["config"] = a.config
    out["kernels"] = "the reference's cuda_backend.cu, compiled for sm_100a, unmodified"
    print(json.dumps(out))
    sys.stdout.flush()
    rc.clear()
    rc.lib.refc_shutdown()      # the backend owns worker state that must go before the interpreter does


if __name__ == "__main__":
    main()
