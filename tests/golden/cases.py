"""Parity cases shared by the golden-vector generator and the tests.

Every case is a chain of the hot path on seeded synthetic inputs.  Three runners evaluate it:
``run_reference`` on the reference's own CUDA backend (oracle/_ref/libvrhino_ref_cuda.so, only where
that library exists), ``run_oracle`` on the CPU oracle, ``run_library`` on this repository's CUDA
library through its host-side mirror.  Each returns {output name: (numpy payload, dtype tag)} with
bf16 payloads as uint16 bits.
"""
from __future__ import annotations

import ctypes

import numpy as np

from vrhino_b200 import synth

EPS = 1e-6


def _inputs(case):
    """name -> (float32 array, dtype tag) for a case; all values come from the seeded generator."""
    k, s = case["kind"], case.get("seed", 0)
    n = lambda shape, st, mean=0.0, std=1.0: synth.normal(shape, mean, std, seed=s, stream=st)
    if k in ("ln_modulate", "rms_modulate", "ln_affine"):
        B, S, D = case["shape"]
        return {"x": (n((B, S, D), 0), case["x_dt"]), "shift": (n((B, 1, D), 1, 0, 0.1), "f32"), "scale": (n((B, 1, D), 2, 0, 0.1), "f32"),
                "w": (n((D,), 3, 1.0, 0.1), "f32"), "b": (n((D,), 4, 0.0, 0.1), "f32")}
    if k == "rms_rope":
        S, H, d = case["tokens"], case["heads"], case["head_dim"]
        grid = case["grid"]
        cos, sin = synth.wan_rope_tables(*grid, head_dim=d)
        wn = d if case["per_head"] else H * d
        return {"x": (n((1, S, H * d), 0), "bf16"), "w": (n((wn,), 1, 1.0, 0.1), "f32"), "cos": (cos, "f32"), "sin": (sin, "f32")}
    if k == "gated_residual":
        B, S, D = case["shape"]
        return {"res": (n((B, S, D), 0), case["state"]), "branch": (n((B, S, D), 1), "bf16"), "gate": (n((B, 1, D), 2, 0, 0.3), "f32")}
    if k == "mochi":
        B, S, D = case["shape"]
        return {"x": (n((B, S, D), 0), case["state"]), "branch": (n((B, S, D), 1), "bf16"), "scale": (n((B, D), 2, 0, 0.1), "f32"),
                "gate": (n((B, D), 3, 0, 0.5), "f32"), "proj": (n((B, S, 2 * case["hidden"]), 4), "bf16")}
    if k == "activation_table":
        bits = np.arange(65536, dtype=np.uint32).astype(np.uint16)
        bits = bits[(bits & 0x7FFF) <= 0x7F80]
        return {"x": ((bits.astype(np.uint32) << 16).view(np.float32), "bf16")}
    if k == "activation_f32":
        return {"x": (n((4096,), 0, 0, 2.5), "f32")}
    if k == "sampler":
        shape = case["shape"]
        return {"x": (n(shape, 0), case["dt"]), "u": (n(shape, 1), case["dt"]), "c": (n(shape, 2), case["dt"])}
    if k == "group_norm":
        shape = case["shape"]
        return {"x": (n(shape, 0, 0.3, 2.0), case["dt"]), "w": (n((shape[1],), 1, 1.0, 0.1), "f32"), "b": (n((shape[1],), 2, 0.0, 0.1), "f32")}
    if k == "dequant":
        rows, inner = case["rows"], case["inner"]
        codes = np.arange(rows * inner, dtype=np.int64).astype(np.uint8) if case.get("all_codes") else synth.fp8_codes((rows * inner,), seed=s)
        groups = (inner + case["group"] - 1) // case["group"]
        return {"packed": (codes.reshape(rows, inner), "u8"), "scales": (synth.uniform_range((rows, groups), 1e-3, 1e-2, seed=s, stream=1), "f32")}
    if k == "binary":
        return {"a": (n(case["a"], 0), case["dt"]), "b": (n(case["b"], 1), case["dt"])}
    if k == "pixel_norm":
        shape = case["shape"]
        vec = (shape[0], shape[1]) + (1,) * (len(shape) - 2)
        return {"x": (n(shape, 0, 0.2, 1.5), case["dt"]), "shift": (n(vec, 1, 0, 0.2), "f32"), "scale": (n(vec, 2, 0, 0.2), "f32")}
    if k == "depth_to_space":
        b, c, t, h, w = case["shape"]
        return {"x": (n((b, c, t, h, w), 0), case["dt"]), "y": (n((b, 4 * c, t, h, w), 1), case["dt"])}
    if k == "layout":
        made = {}
        for index, (name, shape) in enumerate(case["inputs"].items()):
            made[name] = (np.asarray(shape, dtype=np.float32) if name == "positions" else n(shape, index), case["dt"])
        return made
    if k == "linear_output":
        # A GEMM whose F32 accumulators are exact whatever the summation order: only column 0 of x
        # is non-zero, so accumulation[m, n] = x[m, 0] * w[n, 0], the exact product of two bf16 values.
        M, N, K = case["m"], case["n"], case["k"]
        x = np.zeros((1, M, K), dtype=np.float32)
        x[0, :, 0] = n((M,), 0)
        return {"x": (x, "bf16"), "w": (n((N, K), 1, 0.0, 2.0), "bf16"), "bias": (n((N,), 2, 0.0, 0.5), "bf16"),
                "res": (n((1, M, N), 3), case["state"]), "gate": (n((1, 1, N), 4, 0, 0.3), "f32")}
    raise KeyError(k)


def linear_accumulation(case):
    """The F32 accumulation buffer of a linear_output case (exact, see _inputs)."""
    ins = _inputs(case)
    widen = lambda a: (to_bits(a, "bf16").astype(np.uint32) << 16).view(np.float32)
    x, w = widen(ins["x"][0])[0, :, 0], widen(ins["w"][0])[:, 0]
    return np.ascontiguousarray(np.outer(x, w).astype(np.float32)[None])


CASES = [
    {"name": "config1_ln_modulate_bf16", "kind": "ln_modulate", "shape": (1, 64, 1536), "x_dt": "bf16", "subsample": 7},
    {"name": "ln_modulate_f32_hidden", "kind": "ln_modulate", "shape": (1, 32, 1536), "x_dt": "f32", "seed": 1, "subsample": 5},
    {"name": "ln_modulate_5120_batch2", "kind": "ln_modulate", "shape": (2, 9, 5120), "x_dt": "bf16", "seed": 2, "subsample": 3},
    {"name": "ln_affine_bf16", "kind": "ln_affine", "shape": (1, 48, 1536), "x_dt": "bf16", "seed": 3, "subsample": 5},
    {"name": "ln_affine_f32_odd_width", "kind": "ln_affine", "shape": (1, 5, 257), "x_dt": "f32", "seed": 4},
    {"name": "rms_modulate_ltx", "kind": "rms_modulate", "shape": (2, 16, 2048), "x_dt": "bf16", "seed": 5, "subsample": 7},
    {"name": "wan_q_norm_rope", "kind": "rms_rope", "tokens": 600, "grid": (2, 15, 20), "heads": 12, "head_dim": 128, "per_head": False, "seed": 6, "subsample": 13},
    {"name": "per_head_norm_rope", "kind": "rms_rope", "tokens": 48, "grid": (2, 4, 6), "heads": 24, "head_dim": 128, "per_head": True, "seed": 7, "subsample": 11},
    {"name": "gated_residual_bf16", "kind": "gated_residual", "shape": (1, 40, 1536), "state": "bf16", "seed": 8, "subsample": 3},
    {"name": "gated_residual_f32", "kind": "gated_residual", "shape": (2, 12, 1536), "state": "f32", "seed": 9, "subsample": 3},
    {"name": "mochi_bf16", "kind": "mochi", "shape": (1, 600, 3072), "state": "bf16", "hidden": 512, "seed": 10, "subsample": 29},
    {"name": "mochi_f32_residual", "kind": "mochi", "shape": (1, 24, 3072), "state": "f32", "hidden": 512, "seed": 11, "subsample": 5},
    {"name": "activation_tables_bf16", "kind": "activation_table"},
    {"name": "activation_f32", "kind": "activation_f32", "seed": 12},
    {"name": "sampler_f32", "kind": "sampler", "shape": (16, 3, 10, 13), "dt": "f32", "policy": "fp32", "seed": 13},
    {"name": "sampler_bf16_legacy", "kind": "sampler", "shape": (16, 3, 10, 13), "dt": "bf16", "policy": "bf16", "seed": 14},
    {"name": "sampler_bf16_roles", "kind": "sampler", "shape": (16, 3, 10, 13), "dt": "bf16", "policy": "bf16_roles", "seed": 15},
    {"name": "group_norm_direct_bf16", "kind": "group_norm", "shape": (2, 32, 4, 12, 16), "groups": 8, "dt": "bf16", "eps": 1e-6, "seed": 16, "subsample": 3},
    {"name": "group_norm_partial_bf16", "kind": "group_norm", "shape": (1, 32, 3, 120, 128), "groups": 4, "dt": "bf16", "eps": 1e-6, "seed": 17,
     "subsample": 97},
    {"name": "group_norm_direct_f32", "kind": "group_norm", "shape": (3, 64, 24, 40), "groups": 32, "dt": "f32", "eps": 1e-5, "seed": 18, "subsample": 7},
    {"name": "dequant_fp8_all_codes", "kind": "dequant", "rows": 8, "inner": 256, "group": 256, "all_codes": True, "seed": 19},
    {"name": "dequant_fp8_groups", "kind": "dequant", "rows": 16, "inner": 96, "group": 32, "seed": 20},
    {"name": "binary_internal_broadcast", "kind": "binary", "a": (3, 1, 7), "b": (1, 5, 1), "dt": "bf16", "seed": 21},
    {"name": "pixel_norm_ltx_bf16", "kind": "pixel_norm", "shape": (2, 128, 3, 8, 16), "dt": "bf16", "seed": 24, "subsample": 7},
    {"name": "pixel_norm_wide_bf16", "kind": "pixel_norm", "shape": (1, 1024, 2, 4, 12), "dt": "bf16", "seed": 25, "subsample": 5},
    {"name": "pixel_norm_f32_odd", "kind": "pixel_norm", "shape": (1, 20, 2, 3, 5), "dt": "f32", "seed": 26},
    {"name": "pixel_norm_f32_tiles", "kind": "pixel_norm", "shape": (2, 96, 2, 6, 10), "dt": "f32", "seed": 27, "subsample": 3},
    {"name": "pixel_norm_rows_f32", "kind": "pixel_norm", "shape": (6, 300), "dt": "f32", "seed": 28},
    {"name": "depth_to_space_bf16", "kind": "depth_to_space", "shape": (1, 32, 3, 6, 16), "dt": "bf16", "seed": 29, "subsample": 5},
    {"name": "depth_to_space_f32_odd", "kind": "depth_to_space", "shape": (2, 8, 2, 3, 5), "dt": "f32", "seed": 30},
    {"name": "layout_permute_bf16", "kind": "layout", "dt": "bf16", "seed": 31,
     "inputs": {"frames": (2, 6, 3, 4, 16), "matrix": (1, 96, 200), "map": (1, 24, 2, 5, 7), "patches": (1, 2, 3, 4, 1, 2, 2, 16)},
     "steps": [("frames_first", "permute", ["frames"], (0, 2, 1, 3, 4)), ("transposed", "permute", ["matrix"], (0, 2, 1)),
               ("channels_last", "permute", ["map"], (0, 2, 3, 4, 1)), ("channels_first", "permute", ["channels_last"], (0, 4, 1, 2, 3)),
               ("unpatchified", "permute", ["patches"], (0, 7, 1, 4, 2, 5, 3, 6)), ("reversed", "permute", ["map"], (4, 3, 2, 1, 0))]},
    {"name": "layout_permute_f32", "kind": "layout", "dt": "f32", "seed": 32,
     "inputs": {"matrix": (2, 40, 72), "heads": (1, 20, 3, 4, 8), "patches": (1, 2, 3, 4, 1, 2, 2, 16)},
     "steps": [("transposed", "permute", ["matrix"], (0, 2, 1)), ("qkv", "permute", ["heads"], (2, 0, 3, 1, 4)),
               ("unpatchified", "permute", ["patches"], (0, 7, 1, 4, 2, 5, 3, 6)), ("swapped", "permute", ["matrix"], (1, 0, 2))]},
    {"name": "layout_slice_concat_bf16", "kind": "layout", "dt": "bf16", "seed": 33,
     "inputs": {"proj": (1, 20, 64), "x": (2, 9, 24), "a": (2, 3, 8), "b": (2, 5, 8), "c": (2, 3, 5), "d": (2, 3, 3)},
     "steps": [("first_half", "slice", ["proj"], (2, 0, 32)), ("second_half", "slice", ["proj"], (2, 32, 64)),
               ("odd_inner", "slice", ["proj"], (2, 3, 10)), ("middle", "slice", ["x"], (1, 2, 7)), ("outer", "slice", ["x"], (0, 1, 2)),
               ("from_the_end", "slice", ["x"], (-1, -5, 100)), ("clamped_start", "slice", ["x"], (1, -100, 3)),
               ("joined_rows", "concat", ["a", "b"], 1), ("joined_inner", "concat", ["c", "d", "c"], -1),
               ("joined_outer", "concat", ["a", "a", "a"], 0), ("halves_back", "concat", ["first_half", "second_half"], 2)]},
    {"name": "layout_slice_concat_f32", "kind": "layout", "dt": "f32", "seed": 34,
     "inputs": {"x": (3, 7, 10), "a": (1, 4, 6), "b": (2, 4, 6)},
     "steps": [("inner", "slice", ["x"], (2, 1, 9)), ("aligned", "slice", ["x"], (2, 4, 8)), ("rows", "slice", ["x"], (1, 3, 4)),
               ("joined", "concat", ["a", "b"], 0), ("joined_inner", "concat", ["a", "a"], 2)]},
    {"name": "layout_pad_bf16", "kind": "layout", "dt": "bf16", "seed": 35,
     "inputs": {"video": (1, 8, 3, 6, 16), "map": (1, 4, 2, 5, 7), "row": (1, 2)},
     "steps": [("causal", "pad", ["video"], ((0, 0, 0, 0, 2, 2), 0.0, True)), ("spatial_zero", "pad", ["map"], ((1, 1, 1, 1), 0.0, False)),
               ("all_axes_value", "pad", ["map"], ((1, 2, 0, 1, 2, 0), -1.3, False)), ("all_axes_edge", "pad", ["map"], ((1, 2, 0, 1, 2, 0), 0.0, True)),
               ("row_edge", "pad", ["row"], ((1, 2), 0.0, True)), ("after_only", "pad", ["map"], ((0, 1, 0, 1), 0.0, False)),
               ("outer_constant", "pad", ["video"], ((0, 0, 0, 0, 1, 0, 2, 1), 0.75, False))]},
    {"name": "layout_pad_f32", "kind": "layout", "dt": "f32", "seed": 36,
     "inputs": {"video": (1, 3, 2, 4, 8), "map": (2, 3, 5)},
     "steps": [("causal", "pad", ["video"], ((0, 0, 0, 0, 1, 1), 0.0, True)), ("spatial_value", "pad", ["map"], ((2, 1, 1, 2), 0.1, False)),
               ("spatial_edge", "pad", ["map"], ((2, 1, 1, 2), 0.0, True)), ("nothing", "pad", ["map"], ((0, 0), 0.0, False))]},
    {"name": "layout_nearest_bf16", "kind": "layout", "dt": "bf16", "seed": 39,
     "inputs": {"frames": (3, 4, 6, 16), "video": (1, 2, 3, 5, 7), "row": (1, 1, 24)},
     "steps": [("wan_upsample", "nearest", ["frames"], (2.0, 2.0)), ("width_only", "nearest", ["frames"], (1.0, 2.0)),
               ("all_three", "nearest", ["video"], (2.0, 2.0, 2.0)), ("spatial_of_video", "nearest", ["video"], (1.0, 2.0, 2.0)),
               ("fractional", "nearest", ["video"], (1.5, 0.5)), ("shrink", "nearest", ["row"], (0.5,)), ("triple", "nearest", ["row"], (3.0,))]},
    {"name": "layout_nearest_f32", "kind": "layout", "dt": "f32", "seed": 40,
     "inputs": {"frames": (2, 3, 5, 8), "odd": (1, 2, 3, 5)},
     "steps": [("wan_upsample", "nearest", ["frames"], (2.0, 2.0)), ("odd_doubled", "nearest", ["odd"], (2.0, 2.0)),
               ("fractional", "nearest", ["odd"], (2.5, 1.4))]},
    {"name": "layout_reduce_sum_bf16", "kind": "layout", "dt": "bf16", "seed": 41,
     "inputs": {"text": (2, 37, 64), "odd": (3, 5, 7)},
     "steps": [("pooled", "reduce", ["text"], (1, True)), ("last_axis", "reduce", ["text"], (-1, False)), ("first_axis", "reduce", ["text"], (0, False)),
               ("odd_middle", "reduce", ["odd"], (1, False)), ("odd_last", "reduce", ["odd"], (2, True))]},
    {"name": "layout_reduce_sum_f32", "kind": "layout", "dt": "f32", "seed": 42,
     "inputs": {"text": (2, 37, 64), "odd": (3, 5, 7)},
     "steps": [("pooled", "reduce", ["text"], (1, True)), ("last_axis", "reduce", ["text"], (-1, False)), ("odd_middle", "reduce", ["odd"], (1, False))]},
    {"name": "layout_rng_normal_f32", "kind": "layout", "dt": "f32", "seed": 46, "inputs": {},
     "steps": [("known_answers", "rng", [], (5701, 0, (8,))), ("latent", "rng", [], (1234567890123, 0, (1, 16, 3, 8, 12))),
               ("second_call", "rng", [], (5701, 4, (2, 256))), ("later_call", "rng", [], (99, 4000, (5, 7)))]},
    {"name": "layout_rng_normal_bf16", "kind": "layout", "dt": "bf16", "seed": 47, "inputs": {},
     "steps": [("known_answers", "rng", [], (5701, 0, (8,))), ("latent", "rng", [], (2 ** 63 + 11, 8, (1, 16, 3, 8, 12)))]},
    {"name": "layout_softmax_bf16", "kind": "layout", "dt": "bf16", "seed": 43,
     "inputs": {"scores": (3, 5, 77), "map": (2, 19, 6, 4), "wide": (2, 1100)},
     "steps": [("last_axis", "softmax", ["scores"], (-1,)), ("classes", "softmax", ["map"], (1,)), ("first_axis", "softmax", ["scores"], (0,)),
               ("long_rows", "softmax", ["wide"], (1,))]},
    {"name": "layout_softmax_f32", "kind": "layout", "dt": "f32", "seed": 44,
     "inputs": {"scores": (3, 5, 77), "map": (2, 19, 6, 4)},
     "steps": [("last_axis", "softmax", ["scores"], (-1,)), ("classes", "softmax", ["map"], (1,)), ("middle", "softmax", ["scores"], (1,))]},
    {"name": "layout_gather_bf16", "kind": "layout", "dt": "bf16", "seed": 45,
     "inputs": {"embedding": (50, 64), "odd": (9, 7), "batched": (2, 11, 24)},
     "steps": [("tokens", "gather", ["embedding"], ([[3, 0, 49, 7, 7], [1, 48, 2, 0, 31]], "i64")),
               ("tokens_i32", "gather", ["embedding"], ([5, 4, 3, 2, 1, 0], "i32")),
               ("odd_width", "gather", ["odd"], ([8, 0, 3], "i64")),
               ("per_batch", "gather", ["batched"], ([[10, 0, 5], [1, 1, 9]], "i64")),
               ("per_batch_2d", "gather", ["batched"], ([[[0, 1], [2, 3]], [[10, 9], [8, 7]]], "i32"))]},
    {"name": "layout_sinusoidal_f32", "kind": "layout", "dt": "f32", "seed": 37,
     "inputs": {"positions": (0.0, 1.0, 0.5, 999.0, 37.25, -2.0, 1000.0, 250.0)},
     "steps": [("timestep_256", "sinusoidal", ["positions"], (256, True, 0.0, False)), ("odd_width", "sinusoidal", ["positions"], (7, False, 1.0, False)),
               ("double_320", "sinusoidal", ["positions"], (320, True, 0.0, True)), ("double_downscale", "sinusoidal", ["positions"], (64, False, 1.0, True))]},
    {"name": "layout_sinusoidal_bf16", "kind": "layout", "dt": "bf16", "seed": 38,
     "inputs": {"positions": (0.0, 1.0, 0.5, 999.0, 37.25, -2.0)},
     "steps": [("timestep_256", "sinusoidal", ["positions"], (256, True, 0.0, False)), ("double_64", "sinusoidal", ["positions"], (64, False, 0.0, True))]},
    {"name": "linear_output_bf16_state", "kind": "linear_output", "m": 72, "n": 1536, "k": 16, "state": "bf16", "seed": 22, "subsample": 3},
    {"name": "linear_output_f32_state", "kind": "linear_output", "m": 40, "n": 3072, "k": 32, "state": "f32", "seed": 23, "subsample": 5},
]


class RngState:
    """struct RngState (native/include/vrhino/backend.h:17-21) for the back ends that take one."""

    def __init__(self, seed, offset):
        self.seed, self.offset, self.algorithm_id = seed, offset, "pytorch_compat.v1"


def run_layout(case, values, api, grab, rng=None):
    """The steps of a layout case -- (output name, operator, operand names, arguments) -- on any of the three
    back ends; `api` supplies permute / slice / concat / pad / sinusoidal_embedding for that back end's tensors,
    `rng(seed, offset, shape)` one rng_normal call on a fresh state in the case's dtype."""
    for name, op, operands, args in case["steps"]:
        x = [values[o] for o in operands]
        if op == "rng":
            values[name] = rng(args[0], args[1], tuple(args[2]))
        elif op == "permute":
            values[name] = api.permute(x[0], list(args))
        elif op == "slice":
            values[name] = api.slice(x[0], *args)
        elif op == "concat":
            values[name] = api.concat(x, args)
        elif op == "pad":
            values[name] = api.pad(x[0], list(args[0]), args[1], args[2])
        elif op == "reduce":
            values[name] = api.reduce_sum(x[0], *args)
        elif op == "nearest":
            values[name] = api.interpolate_nearest(x[0], list(args))
        elif op == "sinusoidal":
            values[name] = api.sinusoidal_embedding(x[0], *args)
        elif op == "softmax":
            values[name] = api.softmax(x[0], args[0])
        elif op == "gather":
            values[name] = api.indexed_gather(x[0], np.asarray(args[0], dtype=np.int64 if args[1] == "i64" else np.int32))
        else:
            raise KeyError(op)
        grab(name, values[name])


def to_bits(a, dt):
    if dt == "bf16":
        return synth.to_bf16_bits(np.asarray(a, dtype=np.float32))
    if dt == "u8":
        return np.ascontiguousarray(a, dtype=np.uint8)
    return np.ascontiguousarray(a, dtype=np.float32)


def _sub(case, payload):
    step = case.get("subsample")
    return payload.reshape(-1)[::step].copy() if step else payload


# ------------------------------------------------------------------------------ reference CUDA --
def run_reference(rc, case):
    from oracle import ref
    code = {"f32": ref.F32, "bf16": ref.BF16, "u8": ref.U8}
    ins = _inputs(case)
    h = {k: rc.upload(to_bits(a, dt), code[dt]) for k, (a, dt) in ins.items() if dt != "u8"}
    k = case["kind"]
    pol = ref.POLICY_BF16
    out = {}

    def grab(name, handle, shape):
        payload, dt = rc.download(handle, shape)
        out[name] = (_sub(case, payload), {ref.F32: "f32", ref.BF16: "bf16"}[dt])

    if k in ("ln_modulate", "rms_modulate", "ln_affine"):
        shape = case["shape"]
        if k == "ln_affine":
            normed = rc.layer_norm(h["x"], h["w"], h["b"], EPS)
            grab("norm", normed, shape)
            grab("cast", rc.cast(normed, ref.BF16), shape)
        else:
            normed = rc.layer_norm(h["x"], 0, 0, EPS) if k == "ln_modulate" else rc.rms_norm(h["x"], 0, EPS)
            grab("norm", normed, shape)
            mod = rc.modulate(pol, normed, h["shift"], h["scale"])
            grab("modulate", mod, shape)
            grab("cast", rc.cast(mod, ref.BF16), shape)
    elif k == "rms_rope":
        S, H, d = case["tokens"], case["heads"], case["head_dim"]
        if case["per_head"]:
            normed = rc.attention_norm(pol, rc.reshape(h["x"], (1, S, H, d)), h["w"], 1e-5)
        else:
            normed = rc.reshape(rc.attention_norm(pol, h["x"], h["w"], EPS), (1, S, H, d))
        grab("norm", normed, (1, S, H, d))
        roped = rc.operation_rope(pol, normed, h["cos"], h["sin"])
        grab("rope", roped, (1, S, H, d))
        grab("cast", rc.cast(roped, ref.BF16), (1, S, H, d))
        grab("norm_cast", rc.cast(normed, ref.BF16), (1, S, H, d))
    elif k == "gated_residual":
        p = ref.POLICY_BF16 if case["state"] == "bf16" else ref.POLICY_FP32
        grab("gated", rc.gated_residual(p, h["res"], h["branch"], h["gate"]), case["shape"])
        grab("added", rc.residual_add(p, h["res"], h["branch"]), case["shape"])
    elif k == "mochi":
        B, S, D = case["shape"]
        p = ref.POLICY_BF16 if case["state"] == "bf16" else ref.POLICY_FP32
        one = rc.host_f32(np.array(1.0, dtype=np.float32))
        scaled = rc.binary(1, rc.rms_norm(h["x"], 0, EPS), rc.binary(0, one, rc.reshape(h["scale"], (B, 1, D))))
        grab("norm_scale", scaled, (B, S, D))
        normalized = rc.rms_norm(h["branch"], 0, EPS)
        bounded = rc.reshape(rc.activation(h["gate"], 3), (B, 1, D))
        grab("norm_gated", rc.gated_residual(p, h["x"], normalized, bounded), (B, S, D))
        hid = case["hidden"]
        a, g = rc.slice(h["proj"], 2, 0, hid), rc.slice(h["proj"], 2, hid, 2 * hid)
        grab("swiglu", rc.binary(1, a, rc.activation(g, 0)), (B, S, hid))
    elif k in ("activation_table", "activation_f32"):
        n = ins["x"][0].size
        for kind, name in ((0, "silu"), (1, "gelu"), (2, "gelu_tanh"), (3, "tanh"), (4, "relu")):
            grab(name, rc.activation(h["x"], kind), (n,))
        grab("exp", rc.exp(h["x"]), (n,))
        grab("clamp", rc.clamp(h["x"], -0.5, 0.75), (n,))
    elif k == "sampler":
        p = {"fp32": ref.POLICY_FP32, "bf16": ref.POLICY_BF16, "bf16_roles": ref.POLICY_BF16_ROLES}[case["policy"]]
        rc.lib.refc_init(ref.F32 if case["policy"] == "fp32" else ref.BF16)
        g = rc.cfg_combine(p, h["u"], h["c"], 5.0)
        grab("cfg", g, case["shape"])
        grab("euler", rc.euler_update(p, h["x"], g, 0.02, True), case["shape"])
        grab("flow_x0", rc.flow_to_x0(p, h["x"], h["u"], 0.877877295), case["shape"])
        rc.lib.refc_init(ref.BF16)
    elif k == "group_norm":
        gn = rc.group_norm(h["x"], case["groups"], h["w"], h["b"], case["eps"])
        grab("group_norm", gn, case["shape"])
        grab("silu", rc.activation(gn, 0), case["shape"])
    elif k == "dequant":
        packed, scales = ins["packed"][0], ins["scales"][0]
        for dt, name in ((ref.BF16, "bf16"), (ref.F32, "f32")):
            grab(name, rc.dequantize(0, packed, scales, case["rows"], case["inner"], case["group"], dt), (case["rows"], case["inner"]))
    elif k == "binary":
        shape = np.broadcast_shapes(case["a"], case["b"])
        for kind, name in enumerate(("add", "mul", "div", "max")):
            grab(name, rc.binary(kind, h["a"], h["b"]), shape)
    elif k == "pixel_norm":
        shape = case["shape"]
        normed = rc.pixel_norm(h["x"], 1, 1e-8)
        grab("pnorm", normed, shape)
        mod = rc.modulate(pol, normed, h["shift"], h["scale"])
        grab("pmod", mod, shape)
        act = rc.activation(mod, 0)
        grab("silu", act, shape)
        grab("cast", rc.cast(act, ref.BF16), shape)
    elif k == "layout":
        class Api:
            permute = staticmethod(rc.permute); slice = staticmethod(rc.slice); concat = staticmethod(rc.concat)
            pad = staticmethod(rc.pad); sinusoidal_embedding = staticmethod(rc.sinusoidal_embedding)
            interpolate_nearest = staticmethod(rc.interpolate_nearest); reduce_sum = staticmethod(rc.reduce_sum)
            softmax = staticmethod(rc.softmax); indexed_gather = staticmethod(rc.indexed_gather)
        run_layout(case, dict(h), Api, lambda name, handle: grab(name, handle, (int(rc.lib.refc_numel(ctypes.c_int64(handle))),)),
                   rng=lambda seed, offset, shape: rc.rng_normal(seed, offset, shape, code[case["dt"]]))
    elif k == "depth_to_space":
        b, c, t, h_, w = case["shape"]
        full = (b, c // 2, 2 * t, 2 * h_, 2 * w)
        shuffled = rc.pixel_shuffle(h["y"], (2, 2, 2))
        grab("shuffle", shuffled, full)
        grab("shuffle_122", rc.pixel_shuffle(h["y"], (1, 2, 2)), (b, c, t, 2 * h_, 2 * w))
        grab("shuffle_211", rc.pixel_shuffle(h["x"], (2, 1, 1)), (b, c // 2, 2 * t, h_, w))
        residual = rc.slice(rc.repeat(rc.pixel_shuffle(h["x"], (2, 2, 2)), 4, 1), 2, 1, 2 * t)
        grab("depth_to_space", rc.binary(0, rc.slice(shuffled, 2, 1, 2 * t), residual), (b, c // 2, 2 * t - 1, 2 * h_, 2 * w))
    elif k == "linear_output":
        M, N = case["m"], case["n"]
        p = ref.POLICY_BF16 if case["state"] == "bf16" else ref.POLICY_FP32
        lin = rc.linear(h["x"], h["w"], h["bias"])
        grab("linear", lin, (1, M, N))
        grab("linear_nobias", rc.linear(h["x"], h["w"], 0), (1, M, N))
        grab("gelu_tanh", rc.activation(lin, 2), (1, M, N))
        grab("silu", rc.activation(lin, 0), (1, M, N))
        grab("gated", rc.gated_residual(p, h["res"], lin, h["gate"]), (1, M, N))
        grab("added", rc.residual_add(p, h["res"], lin), (1, M, N))
        a, g = rc.slice(lin, 2, 0, N // 2), rc.slice(lin, 2, N // 2, N)
        grab("swiglu", rc.binary(1, a, rc.activation(g, 0)), (1, M, N // 2))
    rc.clear()
    return out


# ------------------------------------------------------------------------------------ CPU oracle --
def run_oracle(orc, case):
    ins = {k: (orc.T(to_bits(a, dt), dt) if dt != "u8" else a) for k, (a, dt) in _inputs(case).items()}
    be = orc.OracleBackend(execution_dtype=orc.BF16)
    pol = orc.Policy()
    k = case["kind"]
    out = {}

    def grab(name, t):
        out[name] = (_sub(case, t.data), t.dtype)

    if k in ("ln_modulate", "rms_modulate", "ln_affine"):
        if k == "ln_affine":
            normed = be.layer_norm(ins["x"], ins["w"], ins["b"], EPS)
            grab("norm", normed); grab("cast", be.cast(normed, "bf16"))
        else:
            normed = be.layer_norm(ins["x"], None, None, EPS) if k == "ln_modulate" else be.rms_norm(ins["x"], None, EPS)
            grab("norm", normed)
            mod = orc.modulate(be, pol, normed, ins["shift"], ins["scale"])
            grab("modulate", mod); grab("cast", be.cast(mod, "bf16"))
    elif k == "rms_rope":
        S, H, d = case["tokens"], case["heads"], case["head_dim"]
        if case["per_head"]:
            normed = orc.attention_norm(be, pol, ins["x"].reshape((1, S, H, d)), ins["w"], 1e-5)
        else:
            normed = orc.attention_norm(be, pol, ins["x"], ins["w"], EPS).reshape((1, S, H, d))
        grab("norm", normed)
        roped = orc.operation_rope(be, pol, normed, ins["cos"], ins["sin"])
        grab("rope", roped); grab("cast", be.cast(roped, "bf16")); grab("norm_cast", be.cast(normed, "bf16"))
    elif k == "gated_residual":
        p = orc.Policy(residual=case["state"])
        grab("gated", orc.gated_residual(be, p, ins["res"], ins["branch"], ins["gate"]))
        grab("added", orc.residual_add(be, p, ins["res"], ins["branch"]))
    elif k == "mochi":
        p = orc.Policy(residual=case["state"])
        grab("norm_scale", orc.mochi_norm_scale(be, ins["x"], ins["scale"]))
        grab("norm_gated", orc.normalized_gated_residual(be, p, ins["x"], ins["branch"], ins["gate"]))
        grab("swiglu", orc.swiglu_hidden(be, ins["proj"]))
    elif k in ("activation_table", "activation_f32"):
        for kind, name in ((0, "silu"), (1, "gelu"), (2, "gelu_tanh"), (3, "tanh"), (4, "relu")):
            grab(name, be.activation(ins["x"], kind))
        grab("exp", be.exp(ins["x"])); grab("clamp", be.clamp(ins["x"], -0.5, 0.75))
    elif k == "sampler":
        be = orc.OracleBackend(execution_dtype=orc.F32 if case["policy"] == "fp32" else orc.BF16)
        p = {"fp32": orc.Policy.fp32(), "bf16": orc.Policy(), "bf16_roles": orc.Policy().with_scalar_roles({orc.GUIDANCE, orc.SOLVER, orc.SIGMA})}[case["policy"]]
        g = orc.cfg_combine(be, p, ins["u"], ins["c"], 5.0)
        grab("cfg", g); grab("euler", orc.euler_update(be, p, ins["x"], g, orc.scalar_f32(0.02), True))
        grab("flow_x0", orc.flow_to_x0(be, p, ins["x"], ins["u"], 0.877877295))
    elif k == "group_norm":
        gn = be.group_norm(ins["x"], case["groups"], ins["w"], ins["b"], case["eps"])
        grab("group_norm", gn); grab("silu", be.activation(gn, orc.SILU))
    elif k == "dequant":
        t = orc.T(ins["packed"], orc.U8, host=True, quant={"type": "fp8_e4m3fn", "group_size": case["group"],
                                                           "scales": ins["scales"].data, "shape": (case["rows"], case["inner"])})
        grab("bf16", be.copy_to_device(t, "bf16")); grab("f32", be.copy_to_device(t, "f32"))
    elif k == "binary":
        for kind, name in enumerate(("add", "mul", "div", "max")):
            grab(name, be._binary(kind, ins["a"], ins["b"]))
    elif k == "pixel_norm":
        normed = be.pixel_norm(ins["x"], 1, 1e-8)
        mod = orc.modulate(be, pol, normed, ins["shift"], ins["scale"])
        act = be.activation(mod, 0)
        grab("pnorm", normed); grab("pmod", mod); grab("silu", act); grab("cast", be.cast(act, "bf16"))
    elif k == "layout":
        run_layout(case, dict(ins), be, lambda name, t: grab(name, t.reshape((-1,))),
                   rng=lambda seed, offset, shape: be.rng_normal(RngState(seed, offset), shape, case["dt"]))
    elif k == "depth_to_space":
        grab("shuffle", be.pixel_shuffle_nd(ins["y"], (2, 2, 2)))
        grab("shuffle_122", be.pixel_shuffle_nd(ins["y"], (1, 2, 2)))
        grab("shuffle_211", be.pixel_shuffle_nd(ins["x"], (2, 1, 1)))
        grab("depth_to_space", orc.depth_to_space_residual(be, ins["y"], ins["x"]))
    elif k == "linear_output":
        p = orc.Policy(residual=case["state"])
        acc = orc.T(linear_accumulation(case), "f32")
        lin = orc.linear_output(acc, ins["bias"])
        grab("linear", lin); grab("linear_nobias", orc.linear_output(acc, None))
        grab("gelu_tanh", be.activation(lin, 2)); grab("silu", be.activation(lin, 0))
        grab("gated", orc.gated_residual(be, p, ins["res"], lin, ins["gate"]))
        grab("added", orc.residual_add(be, p, ins["res"], lin))
        grab("swiglu", orc.swiglu_hidden(be, lin))
    return out


# ------------------------------------------------------------------------- this library (CUDA) --
def run_library(be, ops, case, fused=True):
    """fused=True evaluates each chain with the one-pass entry points; False with the same chain of
    per-operator kernels the reference uses.  Intermediates only exist in the unfused form."""
    import torch
    tdt = {"f32": torch.float32, "bf16": torch.bfloat16}

    def dev(a, dt):
        if dt == "bf16":
            return torch.from_numpy(to_bits(a, dt).view(np.int16).copy()).view(torch.bfloat16).cuda()
        return torch.from_numpy(np.ascontiguousarray(a)).cuda()

    ins = {k: dev(a, dt) for k, (a, dt) in _inputs(case).items()}
    out = {}

    def grab(name, t):
        t = t.detach().cpu().contiguous()
        payload = t.view(torch.int16).numpy().view(np.uint16) if t.dtype == torch.bfloat16 else t.numpy()
        out[name] = (_sub(case, payload), "bf16" if t.dtype == torch.bfloat16 else "f32")

    pol = ops.Policy()
    k = case["kind"]
    if k in ("ln_modulate", "rms_modulate", "ln_affine"):
        if k == "ln_affine":
            if fused:
                grab("cast", ops.fused_layer_norm_cast(be, ins["x"], ins["w"], ins["b"], EPS))
            else:
                normed = be.layer_norm(ins["x"], ins["w"], ins["b"], EPS)
                grab("norm", normed); grab("cast", be.cast(normed, torch.bfloat16))
        elif fused:
            f = ops.fused_layer_norm_modulate if k == "ln_modulate" else None
            if k == "ln_modulate":
                grab("cast", f(be, ins["x"], None, None, EPS, ins["shift"], ins["scale"]))
                grab("modulate", f(be, ins["x"], None, None, EPS, ins["shift"], ins["scale"], torch.float32))
            else:
                grab("cast", ops.fused_rms_norm_modulate(be, ins["x"], EPS, ins["shift"], ins["scale"]))
                grab("modulate", ops.fused_rms_norm_modulate(be, ins["x"], EPS, ins["shift"], ins["scale"], torch.float32))
        else:
            normed = be.layer_norm(ins["x"], None, None, EPS) if k == "ln_modulate" else be.rms_norm(ins["x"], None, EPS)
            grab("norm", normed)
            mod = ops.modulate(be, pol, normed, ins["shift"], ins["scale"])
            grab("modulate", mod); grab("cast", be.cast(mod, torch.bfloat16))
    elif k == "rms_rope":
        S, H, d = case["tokens"], case["heads"], case["head_dim"]
        eps = 1e-5 if case["per_head"] else EPS
        if fused:
            args = dict(heads=H, per_head_norm=case["per_head"])
            grab("cast", ops.fused_rms_norm_rope(be, ins["x"], ins["w"], eps, ins["cos"], ins["sin"], **args).reshape(1, S, H, d))
            grab("rope", ops.fused_rms_norm_rope(be, ins["x"], ins["w"], eps, ins["cos"], ins["sin"], out_dtype=torch.float32, **args).reshape(1, S, H, d))
            grab("norm_cast", ops.fused_rms_norm_rope(be, ins["x"], ins["w"], eps, None, None, **args).reshape(1, S, H, d))
        else:
            if case["per_head"]:
                normed = ops.attention_norm(be, pol, ins["x"].reshape(1, S, H, d), ins["w"], eps)
            else:
                normed = ops.attention_norm(be, pol, ins["x"], ins["w"], eps).reshape(1, S, H, d)
            grab("norm", normed)
            roped = ops.operation_rope(be, pol, normed, ins["cos"], ins["sin"])
            grab("rope", roped); grab("cast", be.cast(roped, torch.bfloat16)); grab("norm_cast", be.cast(normed, torch.bfloat16))
    elif k == "gated_residual":
        p = ops.Policy(residual=tdt[case["state"]])
        if fused:
            grab("gated", ops.fused_gated_residual(be, p, ins["res"], ins["branch"], ins["gate"]))
            grab("added", ops.fused_gated_residual(be, p, ins["res"], ins["branch"], None))
        else:
            grab("gated", ops.gated_residual(be, p, ins["res"], ins["branch"], ins["gate"]))
            grab("added", ops.residual_add(be, p, ins["res"], ins["branch"]))
    elif k == "mochi":
        B, S, D = case["shape"]
        p = ops.Policy(residual=tdt[case["state"]])
        bounded = be.activation(ins["gate"], ops.TANH)
        if fused:
            grab("norm_scale", ops.fused_rms_norm_scale(be, ins["x"], ins["scale"], EPS))
            grab("norm_gated", ops.fused_rms_norm_gated_residual(be, p, ins["x"], ins["branch"], bounded, EPS))
            grab("swiglu", ops.fused_swiglu(be, ins["proj"]))
        else:
            grab("norm_scale", be.mul(be.rms_norm(ins["x"], None, EPS), be.add(ops.scalar_f32(1.0), ins["scale"].reshape(B, 1, D))))
            grab("norm_gated", ops.gated_residual(be, p, ins["x"], be.rms_norm(ins["branch"], None, EPS), bounded.reshape(B, 1, D)))
            hid = case["hidden"]
            a, g = ins["proj"][..., :hid].contiguous(), ins["proj"][..., hid:].contiguous()
            grab("swiglu", be.mul(a, be.activation(g, ops.SILU)))
    elif k in ("activation_table", "activation_f32"):
        for kind, name in ((0, "silu"), (1, "gelu"), (2, "gelu_tanh"), (3, "tanh"), (4, "relu")):
            grab(name, be.activation(ins["x"], kind))
        grab("exp", be.exp(ins["x"])); grab("clamp", be.clamp(ins["x"], -0.5, 0.75))
    elif k == "sampler":
        be = ops.B200Backend(execution_dtype=torch.float32 if case["policy"] == "fp32" else torch.bfloat16)
        p = {"fp32": ops.Policy.fp32(), "bf16": ops.Policy(), "bf16_roles": ops.Policy().with_scalar_roles({ops.GUIDANCE, ops.SOLVER, ops.SIGMA})}[case["policy"]]
        if fused:
            g = ops.fused_cfg_combine(be, p, ins["u"], ins["c"], 5.0)
            grab("cfg", g); grab("euler", ops.fused_cfg_euler(be, p, ins["x"], ins["u"], ins["c"], 5.0, 0.02, True))
            grab("flow_x0", ops.fused_flow_to_x0(be, p, ins["x"], ins["u"], 0.877877295))
        else:
            g = ops.cfg_combine(be, p, ins["u"], ins["c"], 5.0)
            grab("cfg", g); grab("euler", ops.euler_update(be, p, ins["x"], g, 0.02, True))
            grab("flow_x0", ops.flow_to_x0(be, p, ins["x"], ins["u"], 0.877877295))
    elif k == "group_norm":
        if fused:
            grab("silu", ops.fused_group_norm_silu(be, ins["x"], case["groups"], ins["w"], ins["b"], case["eps"]))
        gn = be.group_norm(ins["x"], case["groups"], ins["w"], ins["b"], case["eps"])
        grab("group_norm", gn)
        if not fused:
            grab("silu", be.activation(gn, ops.SILU))
    elif k == "dequant":
        grab("bf16", be.dequantize(ins["packed"], ins["scales"], case["group"], dtype=torch.bfloat16))
        grab("f32", be.dequantize(ins["packed"], ins["scales"], case["group"], dtype=torch.float32))
    elif k == "binary":
        for name in ("add", "mul", "div", "maximum"):
            grab("max" if name == "maximum" else name, getattr(be, name)(ins["a"], ins["b"]))
    elif k == "pixel_norm":
        grab("pnorm", be.pixel_norm(ins["x"], 1, 1e-8))
        if fused:
            grab("pmod", ops.fused_pixel_norm_modulate(be, ins["x"], ins["shift"], ins["scale"], 1e-8, silu=False))
            grab("silu", ops.fused_pixel_norm_modulate(be, ins["x"], ins["shift"], ins["scale"], 1e-8))
            grab("cast", ops.fused_pixel_norm_modulate(be, ins["x"], ins["shift"], ins["scale"], 1e-8, out_dtype=torch.bfloat16))
        else:
            mod = ops.modulate(be, pol, be.pixel_norm(ins["x"], 1, 1e-8), ins["shift"], ins["scale"])
            act = be.activation(mod, ops.SILU)
            grab("pmod", mod); grab("silu", act); grab("cast", be.cast(act, torch.bfloat16))
    elif k == "layout":
        run_layout(case, dict(ins), be, lambda name, t: grab(name, t.reshape(-1)),
                   rng=lambda seed, offset, shape: be.rng_normal(RngState(seed, offset), shape, tdt[case["dt"]]))
    elif k == "depth_to_space":
        shuffled = be.pixel_shuffle_nd(ins["y"], (2, 2, 2))
        grab("shuffle", shuffled)
        grab("shuffle_122", be.pixel_shuffle_nd(ins["y"], (1, 2, 2)))
        grab("shuffle_211", be.pixel_shuffle_nd(ins["x"], (2, 1, 1)))
        if fused:
            grab("depth_to_space", ops.fused_depth_to_space_residual(be, ins["y"], ins["x"]))
        else:
            residual = torch.cat([be.pixel_shuffle_nd(ins["x"], (2, 2, 2))] * 4, dim=1)[:, :, 1:].contiguous()
            grab("depth_to_space", be.add(shuffled[:, :, 1:].contiguous(), residual))
    elif k == "linear_output":
        p = ops.Policy(residual=tdt[case["state"]])
        acc = torch.from_numpy(linear_accumulation(case)).cuda()
        lin = ops.linear_output(be, acc, ins["bias"])
        grab("linear", lin); grab("linear_nobias", ops.linear_output(be, acc, None))
        if fused:
            grab("gelu_tanh", ops.linear_output_activation(be, acc, ins["bias"], ops.GELU_TANH))
            grab("silu", ops.linear_output_activation(be, acc, ins["bias"], ops.SILU))
            grab("gated", ops.linear_output_gated_residual(be, p, ins["res"], acc, ins["bias"], ins["gate"]))
            grab("added", ops.linear_output_gated_residual(be, p, ins["res"], acc, ins["bias"], None))
            grab("swiglu", ops.linear_output_swiglu(be, acc, ins["bias"]))
        else:
            grab("gelu_tanh", be.activation(lin, ops.GELU_TANH)); grab("silu", be.activation(lin, ops.SILU))
            grab("gated", ops.fused_gated_residual(be, p, ins["res"], lin, ins["gate"]))
            grab("added", ops.fused_gated_residual(be, p, ins["res"], lin, None))
            grab("swiglu", ops.fused_swiglu(be, lin))
    return out
