"""Seeded synthetic inputs shared by the tests, the smoke check and the benchmark.

Counter-based generator so any element can be produced independently and C++ or Python
callers agree bit for bit:

    u64 state(i)  = splitmix64(seed * 0x9E3779B97F4A7C15 + stream * 0xD1B54A32D192ED03 + i)
    uniform(i)    = (state(i) >> 11) * 2^-53                         in [0, 1)
    normal(i)     = sqrt(-2 ln(1 - uniform(2i))) * cos(2 pi uniform(2i+1))   (Box-Muller, f64)

Values are produced in float64, narrowed to float32, then (for bf16 tensors) rounded to
nearest-even bf16.  ``stream`` distinguishes tensors of one configuration.
"""
from __future__ import annotations

import numpy as np

_M64 = np.uint64(0xFFFFFFFFFFFFFFFF)


def splitmix64(x: np.ndarray) -> np.ndarray:
    with np.errstate(over="ignore"):
        z = (x + np.uint64(0x9E3779B97F4A7C15)) & _M64
        z = ((z ^ (z >> np.uint64(30))) * np.uint64(0xBF58476D1CE4E5B9)) & _M64
        z = ((z ^ (z >> np.uint64(27))) * np.uint64(0x94D049BB133111EB)) & _M64
        return z ^ (z >> np.uint64(31))


def _base(seed: int, stream: int) -> np.uint64:
    return np.uint64((seed * 0x9E3779B97F4A7C15 + stream * 0xD1B54A32D192ED03) & 0xFFFFFFFFFFFFFFFF)


def uniform(n: int, seed: int = 0, stream: int = 0, offset: int = 0) -> np.ndarray:
    with np.errstate(over="ignore"):
        idx = np.arange(offset, offset + n, dtype=np.uint64) + _base(seed, stream)
    return (splitmix64(idx) >> np.uint64(11)).astype(np.float64) * (2.0 ** -53)


def normal(shape, mean: float = 0.0, std: float = 1.0, seed: int = 0, stream: int = 0) -> np.ndarray:
    n = int(np.prod(shape))
    u = uniform(2 * n, seed, stream)
    r = np.sqrt(-2.0 * np.log1p(-u[0::2]))
    z = r * np.cos(2.0 * np.pi * u[1::2])
    return (mean + std * z).astype(np.float32).reshape(shape)


def uniform_range(shape, lo: float, hi: float, seed: int = 0, stream: int = 0) -> np.ndarray:
    n = int(np.prod(shape))
    return (lo + (hi - lo) * uniform(n, seed, stream)).astype(np.float32).reshape(shape)


def fp8_codes(shape, seed: int = 0, stream: int = 0) -> np.ndarray:
    """Uniform over the 254 finite e4m3fn codes (0x7f and 0xff excluded)."""
    n = int(np.prod(shape))
    k = np.floor(uniform(n, seed, stream) * 254.0).astype(np.int64)  # 0..253
    codes = np.where(k < 127, k, k + 1)                               # skip 0x7f; 253+1 = 0xfe
    return codes.astype(np.uint8).reshape(shape)


def to_bf16_bits(a: np.ndarray) -> np.ndarray:
    bits = np.ascontiguousarray(a, dtype=np.float32).view(np.uint32).astype(np.uint64)
    nan = (bits & 0x7FFFFFFF) > 0x7F800000
    out = ((bits + 0x7FFF + ((bits >> 16) & 1)) >> 16).astype(np.uint16)
    out[nan] = 0x7FFF
    return out.reshape(a.shape)


def wan_rope_tables(frames: int, height: int, width: int, head_dim: int = 128, theta: float = 1e4):
    """cos / sin tables [1, S, 1, head_dim] F32 with the semantics of standard_rope
    (native/src/architectures/common.cpp:160-186 of the reference): axis split
    (d - 4*(d//6), 2*(d//6), 2*(d//6)), f64 frequencies, each value duplicated for its pair."""
    sixth = head_dim // 6
    axis_dims = [head_dim - 4 * sixth, 2 * sixth, 2 * sixth]
    t, h, w = np.meshgrid(np.arange(frames), np.arange(height), np.arange(width), indexing="ij")
    coords = [t.reshape(-1).astype(np.float64), h.reshape(-1).astype(np.float64), w.reshape(-1).astype(np.float64)]
    cos_parts, sin_parts = [], []
    for axis, dim in enumerate(axis_dims):
        pair = np.arange(dim // 2, dtype=np.float64)
        inverse = 1.0 / np.power(theta, 2.0 * pair / dim)
        phase = coords[axis][:, None].astype(np.float32).astype(np.float64) * inverse[None, :]
        c = np.cos(phase).astype(np.float32)
        s = np.sin(phase).astype(np.float32)
        cos_parts.append(np.repeat(c, 2, axis=1))
        sin_parts.append(np.repeat(s, 2, axis=1))
    cos = np.concatenate(cos_parts, axis=1).reshape(1, -1, 1, head_dim)
    sin = np.concatenate(sin_parts, axis=1).reshape(1, -1, 1, head_dim)
    return np.ascontiguousarray(cos), np.ascontiguousarray(sin)
