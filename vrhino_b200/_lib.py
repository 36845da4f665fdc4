"""ctypes binding of ``libvrb.so`` (the C ABI declared in ``include/vrb.h``).

There is no fallback: if the shared library is missing or a call fails, an exception is
raised.  ``VrbError`` mirrors ``vrhino::Error`` (native/include/vrhino/error.h:8-13 of the
reference) -- the text is what ``vrb_last_error()`` reports.
"""
from __future__ import annotations

import ctypes
import os

_PKG = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_PKG, "libvrb.so")

F32, BF16, U8 = 0, 2, 5
SILU, GELU, GELU_TANH, TANH, RELU = 0, 1, 2, 3, 4
ADD, MUL, DIV, MAX = 0, 1, 2, 3
Q_FP8, Q_INT8, Q_INT4 = 0, 1, 2


class VrbError(RuntimeError):
    """Raised when an entry point returns a negative status."""


_c = ctypes
_vp, _i, _i64, _f, _sz, _d = _c.c_void_p, _c.c_int, _c.c_int64, _c.c_float, _c.c_size_t, _c.c_double
_pi64 = _c.POINTER(_c.c_int64)

# name -> argtypes; every entry returns int unless listed in _RESTYPES
SIGNATURES = {
    "vrb_abi_version": [],
    "vrb_last_error": [],
    "vrb_launch_count": [],
    "vrb_device_allocation_count": [],
    "vrb_prepare_tables": [_vp],
    "vrb_set_launch_overlap": [_i],
    "vrb_binary": [_i, _vp, _pi64, _i, _vp, _pi64, _i, _vp, _i, _vp],
    "vrb_cast": [_vp, _i, _vp, _i, _i64, _vp],
    "vrb_activation": [_i, _vp, _vp, _i, _i64, _vp],
    "vrb_clamp": [_vp, _vp, _i, _i64, _f, _f, _vp],
    "vrb_exp": [_vp, _vp, _i, _i64, _vp],
    "vrb_sqrt": [_vp, _vp, _i, _i64, _vp],
    "vrb_layer_norm": [_vp, _i, _vp, _i, _vp, _i, _vp, _i64, _i64, _f, _vp],
    "vrb_rms_norm": [_vp, _i, _vp, _i, _vp, _i, _i64, _i64, _f, _vp],
    "vrb_rms_norm_axis": [_vp, _i, _vp, _i, _vp, _i64, _i64, _i64, _f, _i, _vp],
    "vrb_rope": [_vp, _i, _pi64, _i, _vp, _vp, _i, _pi64, _i, _vp, _vp],
    "vrb_dequantize": [_i, _vp, _vp, _vp, _i, _i64, _i64, _i64, _vp],
    "vrb_group_norm_workspace_bytes": [_i64, _i],
    "vrb_group_norm": [_vp, _i, _vp, _i, _vp, _i, _vp, _i64, _i64, _i64, _i, _f, _i, _vp, _sz, _vp],
    "vrb_group_norm_frames_workspace_bytes": [_i64, _i64, _i],
    "vrb_group_norm_frames": [_vp, _i, _vp, _i, _vp, _i, _vp, _i64, _i64, _i64, _i64, _i, _f, _i, _vp, _sz, _vp],
    "vrb_group_norm_fixed_scratch": [_vp, _i, _vp, _i, _vp, _i, _vp, _i64, _i64, _i64, _i, _f, _i, _vp],
    "vrb_group_norm_moments": [_vp, _i, _i64, _i64, _i64, _i, _vp, _vp, _vp, _sz, _vp],
    "vrb_group_norm_finalize": [_vp, _vp, _i64, _f, _vp, _vp, _vp],
    "vrb_group_norm_apply": [_vp, _i, _vp, _i, _vp, _i, _vp, _i64, _i64, _i64, _i, _vp, _vp, _i, _vp],
    "vrb_group_norm_apply_scatter": [_vp, _i, _vp, _i, _vp, _i, _vp, _i, _i64, _i64, _i64, _i64, _i64, _i64, _i, _vp, _vp, _i, _vp],
    "vrb_layer_norm_modulate": [_vp, _i, _vp, _i, _vp, _i, _vp, _vp, _i, _i64, _i64, _vp, _i, _i64, _i64, _f, _vp],
    "vrb_gated_residual_rms_norm_modulate": [_vp, _i, _vp, _i, _vp, _i, _i64, _i64, _vp, _i, _vp, _vp, _i, _i64, _i64,
                                             _vp, _i, _i64, _i64, _f, _vp],
    "vrb_gated_residual_layer_norm_modulate": [_vp, _i, _vp, _i, _vp, _i, _i64, _i64, _vp, _i, _vp, _i, _vp, _i, _vp, _vp, _i, _i64, _i64,
                                               _vp, _i, _i64, _i64, _f, _vp],
    "vrb_layer_norm_cast": [_vp, _i, _vp, _i, _vp, _i, _vp, _i, _i64, _i64, _f, _vp],
    "vrb_rms_norm_modulate": [_vp, _i, _vp, _vp, _i, _i64, _i64, _vp, _i, _i64, _i64, _f, _vp],
    "vrb_rms_norm_scale": [_vp, _i, _vp, _i, _i64, _i64, _vp, _i64, _i64, _f, _vp],
    "vrb_rms_norm_rope": [_vp, _i, _vp, _i, _vp, _vp, _i64, _i64, _i64, _vp, _i, _i64, _i64, _i64, _f, _vp],
    "vrb_rms_norm_rope_tables": [_vp, _i, _vp, _i, _vp, _vp, _i, _i64, _i64, _i64, _vp, _i, _i64, _i64, _i64, _f, _vp],
    "vrb_rms_norm_rope_pair": [_vp, _vp, _vp, _i64, _vp, _vp, _vp, _i64, _i, _i, _vp, _vp, _i, _i64, _i64, _i64, _i, _i64, _i64, _f, _vp],
    "vrb_gated_residual": [_vp, _i, _vp, _i, _vp, _i, _i64, _i64, _vp, _i, _i64, _i64, _vp],
    "vrb_rms_norm_gated_residual": [_vp, _i, _vp, _i, _vp, _i, _i64, _i64, _vp, _i, _i64, _i64, _f, _vp],
    "vrb_rms_norm_gated_residual_rms_norm_scale": [_vp, _i, _vp, _i, _f, _vp, _i, _i, _i64, _i64, _vp, _i, _vp, _i, _i64, _i64,
                                                   _vp, _i64, _i64, _f, _vp],
    "vrb_swiglu": [_vp, _vp, _i, _i64, _i64, _vp],
    "vrb_linear_combine": [_vp, _vp, _i, _vp, _i, _i64, _i, _vp],
    "vrb_pixel_shuffle": [_vp, _vp, _i, _i64, _i64, _i64, _i64, _i64, _i, _i, _i, _vp],
    "vrb_depth_to_space_residual": [_vp, _vp, _vp, _i, _i64, _i64, _i64, _i64, _i64, _vp],
    "vrb_l2_normalize": [_vp, _vp, _i, _i64, _i64, _i64, _f, _vp],
    "vrb_set_tensor_map_tiles": [_i],
    "vrb_async_wait_failures": [_vp],
    "vrb_permute": [_vp, _vp, _i, _i, _vp, _vp, _vp],
    "vrb_slice": [_vp, _vp, _i, _i, _vp, _i, _i64, _i64, _vp],
    "vrb_concat": [_vp, _vp, _i, _vp, _i, _i, _vp, _i, _vp],
    "vrb_pad": [_vp, _vp, _i, _i, _vp, _vp, _vp, _f, _i, _vp],
    "vrb_pad_axes": [_vp, _vp, _i, _i, _vp, _vp, _vp, _f, _vp, _vp],
    "vrb_interpolate_nearest": [_vp, _vp, _i, _i, _vp, _vp, _vp],
    "vrb_reduce_sum": [_vp, _vp, _i, _i64, _i64, _i64, _vp],
    "vrb_softmax": [_vp, _vp, _i, _i64, _i64, _i64, _vp],
    "vrb_rng_normal": [_vp, _i, _i64, _c.c_uint64, _c.c_uint64, _vp],
    "vrb_indexed_gather": [_vp, _vp, _i, _vp, _i, _i64, _i64, _i64, _i64, _vp],
    "vrb_sinusoidal_embedding": [_vp, _vp, _i, _i64, _i64, _i, _d, _i, _vp],
    "vrb_pixel_norm": [_vp, _i, _vp, _vp, _i, _i, _vp, _i, _i64, _i64, _i64, _f, _vp],
    "vrb_linear_output": [_vp, _vp, _vp, _i64, _i64, _vp],
    "vrb_linear_output_activation": [_vp, _vp, _i, _vp, _i64, _i64, _vp],
    "vrb_linear_output_gated_residual": [_vp, _vp, _vp, _i, _vp, _i, _i64, _i64, _vp, _i, _i64, _i64, _vp],
    "vrb_linear_output_swiglu": [_vp, _vp, _vp, _i64, _i64, _vp],
    "vrb_cfg_combine": [_vp, _vp, _vp, _i, _i64, _f, _i, _vp],
    "vrb_euler_update": [_vp, _vp, _vp, _i, _i64, _f, _i, _i, _vp],
    "vrb_flow_to_x0": [_vp, _vp, _vp, _i, _i64, _f, _i, _vp],
    "vrb_cfg_euler": [_vp, _vp, _vp, _vp, _vp, _i, _i64, _f, _f, _i, _i, _i, _vp],
    "vrb_host_layer_norm_modulate": [_vp, _i, _vp, _i, _vp, _i, _vp, _vp, _i, _vp, _i, _i64, _i64, _f],
    "vrb_host_rms_norm_rope": [_vp, _i, _vp, _i, _vp, _vp, _i64, _vp, _i, _i64, _i64, _i64, _f],
    "vrb_host_gated_residual": [_vp, _i, _vp, _i, _vp, _i, _vp, _i, _i64, _i64],
    "vrb_host_activation": [_i, _vp, _vp, _i, _i64, _i64],
    "vrb_host_release": [],
}
_RESTYPES = {
    "vrb_last_error": _c.c_char_p,
    "vrb_launch_count": _c.c_uint64,
    "vrb_device_allocation_count": _c.c_uint64,
    "vrb_group_norm_workspace_bytes": _c.c_size_t,
    "vrb_group_norm_frames_workspace_bytes": _c.c_size_t,
    "vrb_host_release": None,
}

# the multi-GPU host layer (include/vrb_sharded.h)
SHARDED_LIB_PATH = os.path.join(_PKG, "libvrb_sharded.so")
_pp = _c.POINTER(_c.c_void_p)
SHARDED_SIGNATURES = {
    "vrbs_last_error": [],
    "vrbs_unique_id": [_vp],
    "vrbs_create": [_pp, _i, _i, _vp, _i],
    "vrbs_destroy": [_vp],
    "vrbs_rank": [_vp],
    "vrbs_world": [_vp],
    "vrbs_aborted": [_vp],
    "vrbs_group_norm_workspace_bytes": [_vp, _i64, _i, _i, _sz],
    "vrbs_group_norm": [_vp, _vp, _i, _vp, _i, _vp, _i, _vp, _i64, _i64, _i64, _i64, _i64, _i64, _i64, _i, _f, _i, _i, _vp, _vp, _sz, _vp],
    "vrbs_cfg_euler": [_vp, _vp, _vp, _vp, _vp, _i, _i64, _f, _f, _i, _i, _i, _vp],
    "vrbs_wait": [_vp, _vp],
    "vrbs_watchdog_selftest": [_i, _c.POINTER(_c.c_int64)],
}
_SHARDED_RESTYPES = {"vrbs_last_error": _c.c_char_p, "vrbs_group_norm_workspace_bytes": _c.c_size_t}

_lib = None
_sharded = None


def load_sharded() -> ctypes.CDLL:
    """Load libvrb_sharded.so (C++ over NCCL and libvrb.so).  Raises if it was not built."""
    global _sharded
    if _sharded is None:
        # A process has ONE libnccl.so.2.  torch brings its own (newer than the system's this library is
        # linked against) and fails to import if another one was loaded first, so torch goes first here.
        import torch  # noqa: F401
        load()
        if not os.path.exists(SHARDED_LIB_PATH):
            raise VrbError(f"{SHARDED_LIB_PATH} is missing: build it with `python -m vrhino_b200.build`")
        lib = ctypes.CDLL(SHARDED_LIB_PATH)
        for name, argtypes in SHARDED_SIGNATURES.items():
            fn = getattr(lib, name)
            fn.argtypes = argtypes
            fn.restype = _SHARDED_RESTYPES.get(name, _c.c_int)
        _sharded = lib
    return _sharded


def load() -> ctypes.CDLL:
    """Load libvrb.so, declaring every signature.  Raises if the library was not built."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise VrbError(f"{LIB_PATH} is missing: build it with `python -m vrhino_b200.build` "
                           "(nvcc, sm_100a); there is no CPU or PyTorch fallback")
        lib = ctypes.CDLL(LIB_PATH)
        for name, argtypes in SIGNATURES.items():
            fn = getattr(lib, name)
            fn.argtypes = argtypes
            fn.restype = _RESTYPES.get(name, _c.c_int)
        _lib = lib
    return _lib


def check(status: int) -> None:
    if status != 0:
        text = load().vrb_last_error().decode("utf-8", "replace")
        raise VrbError(text or f"vrb status {status}")


def call(name: str, *args) -> None:
    """Invoke an int-returning entry point and raise VrbError on a negative status."""
    check(getattr(load(), name)(*args))
