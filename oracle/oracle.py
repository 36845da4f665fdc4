"""ctypes front-end of the CPU oracle plus the reference's helper chains restated on top of it.

TEST INFRASTRUCTURE ONLY.  Only the tests, the smoke check and the benchmark's CPU-baseline
leg import this module; the product package never does.

Two layers:

* ``OracleBackend`` mirrors the per-operator surface of the reference's ``vrhino::Backend``
  (native/include/vrhino/backend.h:74-207) for the non-GEMM operators, including the
  operand-dtype rules of the CUDA host wrappers (native/src/backend/cuda/cuda_backend.cu:
  binary :3871-3902, layer_norm :4057-4089, rms_norm :4091-4177, rope_nd :4198-4213,
  group_norm :4919-5008, copy_to_device quantized branch :3214-3296).
* free functions restate the helper chains that call it:
  native/src/architectures/common.cpp (modulate :51-61, attention_norm :62-68,
  operation_rope :69-76, residual_add :134-138, gated_residual :139-144),
  native/src/architectures/mochi.cpp (swiglu :195-202, normalized_gated_residual :204-211),
  native/src/sampling/sampling.cpp (cfg_combine :181-183, euler_update :185-193,
  flow_to_x0 :200-202) with native/src/precision/precision.cpp precision_scalar_binary
  :196-223.

Tensors are numpy arrays tagged with the reference dtype; bf16 lives in uint16 arrays.
"""
from __future__ import annotations

import ctypes
import os
import subprocess
from dataclasses import dataclass, field

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB_PATH = os.path.join(_HERE, "libvrb_oracle.so")
_SRC_PATH = os.path.join(_HERE, "vrb_oracle.c")

F32, BF16, U8 = "f32", "bf16", "u8"
_CODE = {F32: 0, BF16: 2, U8: 5}
_NP = {F32: np.float32, BF16: np.uint16, U8: np.uint8}

SILU, GELU, GELU_TANH, TANH, RELU = 0, 1, 2, 3, 4


def build(force: bool = False) -> str:
    """Compile the C restatement next to its source (gcc, -ffp-contract=off, OpenMP)."""
    if (not force and os.path.exists(_LIB_PATH)
            and os.path.getmtime(_LIB_PATH) >= os.path.getmtime(_SRC_PATH)):
        return _LIB_PATH
    cmd = ["gcc", "-O2", "-ffp-contract=off", "-fopenmp", "-shared", "-fPIC",
           "-o", _LIB_PATH, _SRC_PATH, "-lm"]
    subprocess.run(cmd, check=True)
    return _LIB_PATH


_lib = None


def lib():
    global _lib
    if _lib is None:
        if not os.path.exists(_LIB_PATH):
            build()
        _lib = ctypes.CDLL(_LIB_PATH)
        _lib.orc_bf16_to_f32.restype = ctypes.c_float
        _lib.orc_bf16_to_f32.argtypes = [ctypes.c_uint16]
        _lib.orc_f32_to_bf16.restype = ctypes.c_uint16
        _lib.orc_f32_to_bf16.argtypes = [ctypes.c_float]
        _lib.orc_decode_fp8.restype = ctypes.c_float
        _lib.orc_decode_fp8.argtypes = [ctypes.c_uint8]
        _lib.orc_rms_lanes.restype = ctypes.c_int
        _lib.orc_rms_lanes.argtypes = [ctypes.c_int64, ctypes.c_int64]
        _lib.orc_group_norm_partials.restype = ctypes.c_int
        _lib.orc_group_norm_partials.argtypes = [ctypes.c_int64, ctypes.c_int64, ctypes.c_int]
    return _lib


def _p(a):
    return None if a is None else ctypes.c_void_p(a.ctypes.data)


def _shape_arg(shape):
    return (ctypes.c_int64 * max(len(shape), 1))(*shape)


# ---------------------------------------------------------------- dtype helpers (numpy) --
def f32_to_bf16_bits(a: np.ndarray) -> np.ndarray:
    """RNE narrowing, NaN -> 0x7fff (same as the device conversion)."""
    bits = np.ascontiguousarray(a, dtype=np.float32).view(np.uint32).astype(np.uint64)
    nan = (bits & 0x7FFFFFFF) > 0x7F800000
    rounded = ((bits + 0x7FFF + ((bits >> 16) & 1)) >> 16).astype(np.uint16)
    rounded[nan] = 0x7FFF
    return rounded.reshape(a.shape)


def bf16_bits_to_f32(a: np.ndarray) -> np.ndarray:
    return (np.ascontiguousarray(a, dtype=np.uint16).astype(np.uint32) << 16).view(np.float32).reshape(a.shape)


@dataclass
class T:
    """Oracle tensor: contiguous numpy payload + reference dtype tag.

    ``host`` marks values the reference keeps in host memory (scalars made by scalar_f32,
    un-uploaded weights); the CUDA wrappers pick operand dtypes differently for those.
    """
    data: np.ndarray
    dtype: str
    host: bool = False
    quant: dict | None = None

    def __post_init__(self):
        self.data = np.ascontiguousarray(self.data, dtype=_NP[self.dtype])

    @property
    def shape(self):
        return tuple(self.data.shape)

    @property
    def numel(self):
        return int(self.data.size)

    def f32(self) -> np.ndarray:
        """Exact widening to float32 for comparisons."""
        if self.dtype == BF16:
            return bf16_bits_to_f32(self.data)
        return self.data.astype(np.float32)

    def reshape(self, shape):
        return T(self.data.reshape(shape), self.dtype, self.host)


def tensor(values, dtype=F32, host=False) -> T:
    """Build an oracle tensor from float values, rounding to bf16 when asked."""
    a = np.asarray(values, dtype=np.float32)
    if dtype == BF16:
        return T(f32_to_bf16_bits(a), BF16, host)
    return T(a, F32, host)


def scalar_f32(value: float) -> T:
    """native/src/tensor_util.cpp:20 -- a rank-0 host F32 tensor."""
    return T(np.array(value, dtype=np.float32), F32, host=True)


# ------------------------------------------------------------------------- the backend --
class OracleBackend:
    """Per-operator CPU oracle with the CUDA backend's dtype rules."""

    def __init__(self, execution_dtype: str = BF16, sm_count: int = 148,
                 layer_norm_affine_fma: bool = True):
        self.execution_dtype = execution_dtype
        self.sm_count = sm_count
        self.layer_norm_affine_fma = layer_norm_affine_fma

    # dtype an op computes in: the tensor's own if it is a device F32/BF16 tensor
    def _dtype_of(self, t: T) -> str:
        if not t.host and t.dtype in (F32, BF16):
            return t.dtype
        return self.execution_dtype

    def copy_to_device(self, t: T, dtype: str) -> T:
        if t.quant is not None:
            return self._dequantize(t, dtype)
        if not t.host and t.dtype == dtype:
            return t
        return self._convert(t, dtype)

    def cast(self, t: T, dtype: str) -> T:
        return self.copy_to_device(t, dtype)

    def _convert(self, t: T, dtype: str) -> T:
        out = np.empty(t.shape, dtype=_NP[dtype])
        if t.dtype == U8:
            lib().orc_cast_u8(_p(t.data), _p(out), _CODE[dtype], ctypes.c_int64(t.numel))
        else:
            lib().orc_cast(_p(t.data), _CODE[t.dtype], _p(out), _CODE[dtype], ctypes.c_int64(t.numel))
        return T(out, dtype)

    def _dequantize(self, t: T, dtype: str) -> T:
        q = t.quant
        kind = {"fp8_e4m3fn": 0, "int8": 1, "int4": 2}[q["type"]]
        shape = q.get("shape", t.shape)
        numel = int(np.prod(shape))
        inner = numel // shape[0]
        group_size = int(q["group_size"])
        groups = (inner + group_size - 1) // group_size
        scales = np.ascontiguousarray(q["scales"], dtype=np.float32)
        out = np.empty(shape, dtype=_NP[dtype])
        lib().orc_dequant(kind, _p(t.data), _p(scales), _p(out), _CODE[dtype],
                          ctypes.c_int64(numel), ctypes.c_int64(inner), ctypes.c_int64(groups),
                          ctypes.c_int64(group_size))
        return T(out, dtype)

    def _binary(self, kind: int, a_raw: T, b_raw: T) -> T:
        if not a_raw.host and a_raw.dtype in (F32, BF16):
            dtype = a_raw.dtype
        elif not b_raw.host and b_raw.dtype in (F32, BF16):
            dtype = b_raw.dtype
        else:
            dtype = self.execution_dtype
        a, b = self.copy_to_device(a_raw, dtype), self.copy_to_device(b_raw, dtype)
        shape = np.broadcast_shapes(a.shape, b.shape)
        out = np.empty(shape, dtype=_NP[dtype])
        rank = lib().orc_binary(kind, _p(a.data), len(a.shape), _shape_arg(a.shape),
                                _p(b.data), len(b.shape), _shape_arg(b.shape),
                                _p(out), _CODE[dtype], None)
        if rank < 0:
            raise ValueError("Incompatible broadcast shapes")
        return T(out, dtype)

    def add(self, a, b): return self._binary(0, a, b)
    def mul(self, a, b): return self._binary(1, a, b)
    def div(self, a, b): return self._binary(2, a, b)
    def maximum(self, a, b): return self._binary(3, a, b)

    def reshape(self, x: T, shape) -> T:
        return self.copy_to_device(x, self._dtype_of(x)).reshape(shape)

    def slice(self, raw: T, dim: int, start: int, stop: int) -> T:
        """CudaBackend::slice (native/src/backend/cuda/cuda_backend.cu:3960-3970): negative dim / start / stop count
        from the end, start is clamped into [0, extent], stop into [start, extent]."""
        x = self.copy_to_device(raw, self._dtype_of(raw))
        if dim < 0:
            dim += len(x.shape)
        if not 0 <= dim < len(x.shape):
            raise ValueError("slice dimension invalid")
        size = x.shape[dim]
        start = start + size if start < 0 else start
        stop = stop + size if stop < 0 else stop
        start = min(max(start, 0), size)
        stop = min(max(stop, start), size)
        index = [slice(None)] * len(x.shape)
        index[dim] = slice(start, stop)
        return T(x.data[tuple(index)], x.dtype)

    def permute(self, raw: T, dims) -> T:
        """CudaBackend::permute (:3936-3947, permute_kernel :767-780): output axis d is input axis dims[d]."""
        if len(dims) != len(raw.shape):
            raise ValueError("permute rank mismatch")
        if sorted(int(d) for d in dims) != list(range(len(raw.shape))):
            raise ValueError("Invalid permutation")
        x = self.copy_to_device(raw, self._dtype_of(raw))
        return T(np.transpose(x.data, [int(d) for d in dims]), x.dtype)

    def concat(self, tensors, dim: int) -> T:
        """CudaBackend::concat (:3949-3958): dtype of the first input if it is a device F32 / BF16 tensor."""
        if not tensors:
            raise ValueError("concat requires inputs")
        rank = len(tensors[0].shape)
        if dim < 0:
            dim += rank
        if not 0 <= dim < rank:
            raise ValueError("concat dimension invalid")
        for t in tensors:
            if len(t.shape) != rank:
                raise ValueError("concat rank mismatch")
            if any(t.shape[d] != tensors[0].shape[d] for d in range(rank) if d != dim):
                raise ValueError("concat shape mismatch")
        dtype = self._dtype_of(tensors[0])
        return T(np.concatenate([self.copy_to_device(t, dtype).data for t in tensors], axis=dim), dtype)

    def pad(self, raw: T, padding, value: float = 0.0, replicate: bool = False) -> T:
        """CudaBackend::pad (:4875-4883, pad_kernel :1771-1788): `padding` holds (before, after) pairs from the
        innermost axis outwards; constant mode stores `value` rounded to the dtype, replicate clamps the
        source coordinate per axis."""
        rank = len(raw.shape)
        if len(padding) % 2 or len(padding) > 2 * rank:
            raise ValueError("Invalid pad vector")
        if any(p < 0 for p in padding):
            raise ValueError("Negative padding unsupported")
        x = self.copy_to_device(raw, self._dtype_of(raw))
        widths = [(0, 0)] * rank
        for pair in range(len(padding) // 2):
            widths[rank - 1 - pair] = (int(padding[2 * pair]), int(padding[2 * pair + 1]))
        if replicate:
            return T(np.pad(x.data, widths, mode="edge"), x.dtype)
        fill = tensor(np.array(value, dtype=np.float32), x.dtype).data.reshape(())
        return T(np.pad(x.data, widths, mode="constant", constant_values=fill), x.dtype)

    def interpolate_nearest(self, raw: T, factors) -> T:
        """CudaBackend::interpolate_nearest (:5010-5016, interpolate_kernel :2033-2045): the trailing len(factors) axes
        grow to floor(extent * factor); every output coordinate c reads input coordinate c * in // out."""
        if len(factors) > len(raw.shape) - 2:
            raise ValueError("interpolate factor rank mismatch")
        if any(f <= 0 for f in factors):
            raise ValueError("Invalid interpolation factor")
        x = self.copy_to_device(raw, self._dtype_of(raw))
        data = x.data
        start = len(x.shape) - len(factors)
        for i, f in enumerate(factors):
            axis = start + i
            size = x.shape[axis]
            grown = int(np.floor(size * float(f)))
            index = (np.arange(grown, dtype=np.int64) * size) // max(grown, 1)
            data = np.take(data, index, axis=axis)
        return T(data, x.dtype)

    def reduce_sum(self, raw: T, dim: int, keepdim: bool = False) -> T:
        """CudaBackend::reduce_sum (:4885-4892, reduce_sum_kernel :1790-1806): F32 accumulation in increasing index
        order along `dim`, stored in the operand dtype."""
        if dim < 0:
            dim += len(raw.shape)
        if not 0 <= dim < len(raw.shape):
            raise ValueError("reduce dimension invalid")
        x = self.copy_to_device(raw, self._dtype_of(raw))
        values = np.moveaxis(x.f32(), dim, 0)
        total = np.zeros(values.shape[1:], dtype=np.float32)
        for r in range(values.shape[0]):
            total = (total + values[r]).astype(np.float32)
        if keepdim:
            total = np.expand_dims(total, dim)
        return tensor(total, x.dtype)

    def rng_normal(self, state, shape, dtype: str) -> T:
        """CudaBackend::rng_normal (:5120-5126, rng_normal_kernel :2225-2231): element i is the first normal of
        cuRAND's Philox4x32-10 stream (seed, subsequence i, offset).  Restated from the published algorithm
        (Salmon et al., "Parallel random numbers: as easy as 1, 2, 3", 2011: ten rounds of two 32 x 32 -> 64
        multiplications with the constants below, the key bumped by the Weyl constants between rounds) with cuRAND's
        layout -- key = the seed's halves, counter = (offset / 4 low, offset / 4 high, subsequence low, subsequence
        high) -- and its Box-Muller step on the first two outputs x, y: u = x * 2^-32 + 2^-33,
        v = y * (2 pi * 2^-32) + pi * 2^-32, value = sqrt(-2 ln u) * sin v.  Pinned by the reference's own known answers
        (primitive_tests.cpp:549: seed 5701, offset 0, eight values to 1e-6); log / sin here are the host's.
        `state` is any object with seed, offset and algorithm_id; its offset grows by 4."""
        if state.algorithm_id != "pytorch_compat.v1":
            raise ValueError("Unsupported RNG algorithm")
        if dtype not in (F32, BF16):
            raise ValueError("rng_normal dtype unsupported")
        if state.offset % 4:
            raise ValueError("rng_normal: this restatement covers offsets that are multiples of 4 (all the reference produces)")
        count = int(np.prod(shape, dtype=np.int64)) if len(shape) else 1
        mask = np.uint64(0xFFFFFFFF)
        index = np.arange(count, dtype=np.uint64)
        block = np.uint64(state.offset // 4)
        c = [np.full(count, block & mask, dtype=np.uint64), np.full(count, block >> np.uint64(32), dtype=np.uint64),
             index & mask, index >> np.uint64(32)]
        k0, k1 = int(state.seed) & 0xFFFFFFFF, (int(state.seed) >> 32) & 0xFFFFFFFF
        for _ in range(10):
            p0, p1 = np.uint64(0xD2511F53) * c[0], np.uint64(0xCD9E8D57) * c[2]
            c = [((p1 >> np.uint64(32)) ^ c[1] ^ np.uint64(k0)) & mask, p1 & mask,
                 ((p0 >> np.uint64(32)) ^ c[3] ^ np.uint64(k1)) & mask, p0 & mask]
            k0, k1 = (k0 + 0x9E3779B9) & 0xFFFFFFFF, (k1 + 0xBB67AE85) & 0xFFFFFFFF
        x, y = c[0].astype(np.float32), c[1].astype(np.float32)
        u = x * np.float32(2.0 ** -32) + np.float32(2.0 ** -33)
        v = y * np.float32(2.0 ** -32 * 6.283185307179586) + np.float32(2.0 ** -33 * 6.283185307179586)
        values = (np.sqrt(np.float32(-2.0) * np.log(u)).astype(np.float32) * np.sin(v).astype(np.float32)).astype(np.float32)
        state.offset += 4
        return tensor(values.reshape(tuple(shape)), dtype)

    def softmax(self, raw: T, axis: int) -> T:
        """CudaBackend::softmax (:4893-4917, softmax_axis_kernel :1808-1829): maximum over the axis, then the sum of
        expf(x - max) accumulated in F32 in increasing index order, then expf(x - max) / sum, stored in x's dtype.
        (expf here is the host's; its last bit can differ from the device function.)"""
        if axis < 0:
            axis += len(raw.shape)
        if not 0 <= axis < len(raw.shape):
            raise ValueError("softmax axis invalid")
        x = self.copy_to_device(raw, self._dtype_of(raw))
        values = np.moveaxis(x.f32(), axis, 0)
        maximum = np.full(values.shape[1:], -np.inf, dtype=np.float32)
        for r in range(values.shape[0]):
            maximum = np.fmax(maximum, values[r])
        shifted = np.exp((values - maximum).astype(np.float32)).astype(np.float32)
        denominator = np.zeros(values.shape[1:], dtype=np.float32)
        for r in range(values.shape[0]):
            denominator = (denominator + shifted[r]).astype(np.float32)
        return tensor(np.moveaxis((shifted / denominator).astype(np.float32), 0, axis), x.dtype)

    def indexed_gather(self, table_raw: T, indices) -> T:
        """CudaBackend::indexed_gather (:3981-4055, indexed_gather_kernel :1754-1768): rows of table [rows, width] (or
        of table[b] when the table is [batch, rows, width] and indices [batch, ...]) picked by integer indices;
        the result has the indices' shape plus the width, in the execution dtype."""
        indices = np.asarray(indices)
        if len(table_raw.shape) not in (2, 3):
            raise ValueError("indexed_gather table must have rank 2 or 3")
        if indices.ndim < 1 or indices.dtype not in (np.int64, np.int32):
            raise ValueError("indexed_gather indices must be rank >=1 int64/int32")
        batched = len(table_raw.shape) == 3
        if batched and indices.shape[0] != table_raw.shape[0]:
            raise ValueError("indexed_gather batch dimension mismatch")
        rows = table_raw.shape[-2]
        if indices.size and (indices.min() < 0 or indices.max() >= rows):
            raise ValueError("indexed_gather index out of range")
        table = self.copy_to_device(table_raw, self.execution_dtype).f32()
        if batched:
            picked = np.stack([table[b][indices[b]] for b in range(indices.shape[0])]) if indices.shape[0] else \
                np.zeros(indices.shape + (table.shape[-1],), dtype=np.float32)
        else:
            picked = table[indices]
        return tensor(picked, self.execution_dtype)

    def sinusoidal_embedding(self, raw: T, width: int, flip: bool, downscale: float, frequency_f64: bool) -> T:
        """CudaBackend::sinusoidal_embedding (:4190-4196, sinusoidal_kernel :1178-1198).  The single-precision path
        rounds after every operation like the kernel; exp / sin / cos come from the host's libm, whose last bit
        can differ from the device functions (the comparison with the reference's device output allows for it)."""
        if len(raw.shape) != 1 or width <= 0:
            raise ValueError("sinusoidal embedding contract violation")
        x = self.copy_to_device(raw, self._dtype_of(raw))
        positions = x.f32()
        half = width // 2
        out = np.zeros((x.numel, width), dtype=np.float32)
        f32 = np.float32
        for column in range(2 * half):
            logical = (column + half) % (2 * half) if flip else column
            frequency = logical % half
            if frequency_f64:
                exponent = -np.log(np.float64(10000.0)) * frequency / (half - np.float64(downscale))
                phase = positions.astype(np.float64) * np.exp(exponent)
                out[:, column] = (np.sin(phase) if logical < half else np.cos(phase)).astype(np.float32)
            else:
                exponent = f32(f32(-np.log(f32(10000.0))) * f32(frequency)) / f32(f32(half) - f32(downscale))
                phase = positions * np.exp(f32(exponent)).astype(np.float32)
                out[:, column] = (np.sin(phase) if logical < half else np.cos(phase)).astype(np.float32)
        return tensor(out, x.dtype)

    def split(self, x: T, sections, dim: int):
        out, offset = [], 0
        if dim < 0:
            dim += len(x.shape)
        for s in sections:
            out.append(self.slice(x, dim, offset, offset + s))
            offset += s
        return out

    def layer_norm(self, raw: T, weight: T | None, bias: T | None, eps: float) -> T:
        dtype = self._dtype_of(raw)
        x = self.copy_to_device(raw, dtype)
        w = self.copy_to_device(weight, dtype) if weight is not None else None
        b = self.copy_to_device(bias, dtype) if bias is not None else None
        width = x.shape[-1]
        rows = x.numel // width
        out = np.empty(x.shape, dtype=_NP[dtype])
        lib().orc_layer_norm(_p(x.data), _p(w.data) if w else None, _p(b.data) if b else None,
                             _p(out), _CODE[dtype], ctypes.c_int64(rows), ctypes.c_int64(width),
                             ctypes.c_float(eps), int(self.layer_norm_affine_fma))
        return T(out, dtype)

    def rms_norm(self, raw: T, weight: T | None, eps: float, axis: int = -1,
                 output: str | None = None, rows_for_schedule: int = 0) -> T:
        """``output=None`` stands for the reference's default DType::F16 = "same as input"."""
        rank = len(raw.shape)
        if axis < 0:
            axis += rank
        dtype = self._dtype_of(raw)
        out_dtype = dtype if output is None else output
        if not (out_dtype == dtype or (dtype == BF16 and out_dtype == F32)):
            raise ValueError("rms_norm output dtype unsupported")
        x = self.copy_to_device(raw, dtype)
        w = self.copy_to_device(weight, out_dtype) if weight is not None else None
        out = np.empty(x.shape, dtype=_NP[out_dtype])
        if axis == rank - 1:
            if dtype == BF16 and out_dtype == F32 and w is None:
                raise ValueError("BF16-to-FP32 rms_norm requires affine weight")
            width = x.shape[-1]
            rows = x.numel // width
            lib().orc_rms_norm(_p(x.data), _CODE[dtype], _p(w.data) if w else None, _p(out),
                               _CODE[out_dtype], ctypes.c_int64(rows), ctypes.c_int64(width),
                               ctypes.c_float(eps), ctypes.c_int64(rows_for_schedule))
        else:
            if out_dtype != dtype:
                raise ValueError("mixed-dtype rms_norm currently requires final axis")
            width = x.shape[axis]
            inner = int(np.prod(x.shape[axis + 1:]))
            outer = x.numel // (width * inner)
            lib().orc_rms_norm_axis(_p(x.data), _p(w.data) if w else None, _p(out), _CODE[dtype],
                                    ctypes.c_int64(outer), ctypes.c_int64(width),
                                    ctypes.c_int64(inner), ctypes.c_float(eps))
        return T(out, out_dtype)

    def pixel_norm(self, raw: T, dim: int = 1, eps: float = 1e-8) -> T:
        """CudaBackend::pixel_norm (native/src/backend/cuda/cuda_backend.cu:5048-5086): x / sqrt(mean(x^2)
        over `dim` + eps) in x's dtype, with the kernels' F32 summation schedules."""
        dtype = self._dtype_of(raw)
        x = self.copy_to_device(raw, dtype)
        dim = dim + len(x.shape) if dim < 0 else dim
        channels = x.shape[dim]
        inner = int(np.prod(x.shape[dim + 1:]))
        outer = x.numel // (channels * inner)
        out = np.empty(x.shape, dtype=_NP[dtype])
        lib().orc_pixel_norm(_p(x.data), _p(out), _CODE[dtype], ctypes.c_int64(outer), ctypes.c_int64(channels),
                             ctypes.c_int64(inner), ctypes.c_float(eps))
        return T(out, dtype)

    def l2_normalize(self, raw: T, dim: int, eps: float) -> T:
        """CudaBackend::l2_normalize (native/src/backend/cuda/cuda_backend.cu:5088-5110): x / (sqrt(sum(x^2)
        over `dim`) + eps) in x's dtype, the kernel's 256-partial summation schedule (:1142-1176)."""
        dtype = self._dtype_of(raw)
        x = self.copy_to_device(raw, dtype)
        dim = dim + len(x.shape) if dim < 0 else dim
        if not (0 <= dim < len(x.shape)) or eps < 0:
            raise ValueError("l2 normalize contract violation")
        channels = x.shape[dim]
        inner = int(np.prod(x.shape[dim + 1:]))
        outer = x.numel // (channels * inner)
        out = np.empty(x.shape, dtype=_NP[dtype])
        lib().orc_l2_normalize(_p(x.data), _p(out), _CODE[dtype], ctypes.c_int64(outer), ctypes.c_int64(channels),
                               ctypes.c_int64(inner), ctypes.c_float(eps))
        return T(out, dtype)

    def pixel_shuffle_nd(self, raw: T, factors) -> T:
        """CudaBackend::pixel_shuffle_nd (native/src/backend/cuda/cuda_backend.cu:5112-5118) with the index map of
        pixel_shuffle_kernel (:2170-2186): packed channel ((c*ft+pt)*fh+ph)*fw+pw."""
        dtype = self._dtype_of(raw)
        x = self.copy_to_device(raw, dtype)
        ft, fh, fw = (int(f) for f in factors)
        b, cp, t, h, w = x.shape
        c = cp // (ft * fh * fw)
        v = x.data.reshape(b, c, ft, fh, fw, t, h, w).transpose(0, 1, 5, 2, 6, 3, 7, 4)   # b c t pt h ph w pw
        return T(np.ascontiguousarray(v).reshape(b, c, t * ft, h * fh, w * fw), dtype)

    def activation(self, raw: T, kind: int) -> T:
        dtype = self._dtype_of(raw)
        x = self.copy_to_device(raw, dtype)
        out = np.empty(x.shape, dtype=_NP[dtype])
        lib().orc_activation(kind, _p(x.data), _p(out), _CODE[dtype], ctypes.c_int64(x.numel))
        return T(out, dtype)

    def _unary(self, fn, raw: T, *extra) -> T:
        dtype = self._dtype_of(raw)
        x = self.copy_to_device(raw, dtype)
        out = np.empty(x.shape, dtype=_NP[dtype])
        fn(_p(x.data), _p(out), _CODE[dtype], ctypes.c_int64(x.numel), *extra)
        return T(out, dtype)

    def clamp(self, x, lo, hi):
        return self._unary(lib().orc_clamp, x, ctypes.c_float(lo), ctypes.c_float(hi))

    def exp(self, x): return self._unary(lib().orc_exp, x)
    def sqrt(self, x): return self._unary(lib().orc_sqrt, x)

    def rope_nd(self, raw: T, cos_raw: T, sin_raw: T) -> T:
        dtype = self._dtype_of(raw)
        f_dtype = cos_raw.dtype if (not cos_raw.host and cos_raw.dtype in (F32, BF16)) else dtype
        x = self.copy_to_device(raw, dtype)
        c, s = self.copy_to_device(cos_raw, f_dtype), self.copy_to_device(sin_raw, f_dtype)
        if c.shape != s.shape:
            raise ValueError("RoPE frequency mismatch")
        np.broadcast_shapes(x.shape, c.shape)
        out = np.empty(x.shape, dtype=_NP[dtype])
        rc = lib().orc_rope(_p(x.data), _CODE[dtype], len(x.shape), _shape_arg(x.shape),
                            _p(c.data), _p(s.data), _CODE[f_dtype], len(c.shape), _shape_arg(c.shape),
                            _p(out))
        if rc != 0:
            raise ValueError("RoPE width must be even")
        return T(out, dtype)

    def group_norm(self, raw: T, groups: int, weight: T | None, bias: T | None, eps: float,
                   return_moments: bool = False):
        if len(raw.shape) < 3 or groups <= 0 or raw.shape[1] % groups:
            raise ValueError("group norm shape/groups mismatch")
        dtype = self._dtype_of(raw)
        x = self.copy_to_device(raw, dtype)
        w = self.copy_to_device(weight, dtype) if weight is not None else None
        b = self.copy_to_device(bias, dtype) if bias is not None else None
        batch, channels = x.shape[0], x.shape[1]
        spatial = x.numel // (batch * channels)
        out = np.empty(x.shape, dtype=_NP[dtype])
        mean = np.empty(batch * groups, dtype=np.float32)
        inverse = np.empty(batch * groups, dtype=np.float32)
        lib().orc_group_norm(_p(x.data), _p(w.data) if w else None, _p(b.data) if b else None,
                             _p(out), _CODE[dtype], ctypes.c_int64(batch), ctypes.c_int64(channels),
                             ctypes.c_int64(spatial), int(groups), ctypes.c_float(eps),
                             int(self.sm_count), _p(mean), _p(inverse))
        if return_moments:
            return T(out, dtype), mean, inverse
        return T(out, dtype)


# ---------------------------------------------------------------- precision policy view --
@dataclass
class Policy:
    """The part of native/src/precision/precision.cpp the hot path consults.

    ``residual`` = persistent_state_dtype(ResidualState); ``requested`` = requested_dtype();
    ``scalar_roles`` = roles a v2 policy declares (has_scalar_role).  Modulation and RoPE
    contracts are F32 under every policy (operation_contract :311-327) and attention-norm
    output is F32 (:292-297).
    """
    requested: str = BF16
    residual: str = BF16
    scalar_roles: frozenset = field(default_factory=frozenset)

    @staticmethod
    def unqualified_default(dtype: str = BF16) -> "Policy":
        return Policy(requested=dtype, residual=dtype)

    @staticmethod
    def production_bf16() -> "Policy":
        """bf16-operation-contract-v1: residual stream in F32, heavy operands bf16."""
        return Policy(requested=BF16, residual=F32)

    @staticmethod
    def fp32() -> "Policy":
        return Policy(requested=F32, residual=F32)

    def with_scalar_roles(self, roles) -> "Policy":
        return Policy(self.requested, self.residual, frozenset(roles))


GUIDANCE, SOLVER, SIGMA = "GuidanceCoefficient", "SolverCoefficient", "Sigma"


def precision_scalar_binary(be: OracleBackend, policy: Policy, role: str, op: str, value: T, scalar: T) -> T:
    """precision.cpp:196-223 (Add / Multiply / Divide with a semantic scalar)."""
    apply = {"add": be.add, "mul": be.mul, "div": be.div}[op]
    if role not in policy.scalar_roles:
        return apply(value, scalar)
    compute = F32  # scalar_contract: every non-data role computes in F32
    output = value.dtype
    result = apply(be.copy_to_device(value, compute), be.copy_to_device(scalar, compute))
    return result if result.dtype == output else be.cast(result, output)


# ------------------------------------------------------------------ helper-chain restatements --
def modulate(be, policy, x, shift, scale):
    t = be.add(be.mul(be.cast(x, F32), be.add(scalar_f32(1.0), be.cast(scale, F32))), be.cast(shift, F32))
    return be.cast(t, F32)


def attention_norm(be, policy, x, weight, eps, axis=-1, rows_for_schedule=0):
    return be.rms_norm(x, weight, eps, axis, F32, rows_for_schedule=rows_for_schedule)


def operation_rope(be, policy, x, cosine, sine):
    return be.rope_nd(be.cast(x, F32), cosine, sine)


def residual_add(be, policy, residual, branch):
    d = policy.residual
    return be.add(be.cast(residual, d), be.cast(branch, d))


def gated_residual(be, policy, residual, branch, gate):
    d = policy.residual
    return be.add(be.cast(residual, d), be.mul(be.cast(branch, d), be.cast(gate, d)))


def linear_output(accumulation: T, bias: T | None) -> T:
    """fused_bf16_linear_output_kernel (native/src/backend/cuda/cuda_backend.cu:754-764), the epilogue of
    CudaBackend::linear for bf16 compute and bf16 output (:3831, :3846): one F32 add of the
    accumulation and the bf16 bias (broadcast over rows), one RNE rounding to bf16."""
    assert accumulation.dtype == F32 and (bias is None or bias.dtype == BF16)
    acc = np.ascontiguousarray(accumulation.data, dtype=np.float32)
    if bias is not None:
        acc = (acc + bf16_bits_to_f32(bias.data).reshape(-1).astype(np.float32)).astype(np.float32)
    return T(f32_to_bf16_bits(acc), BF16)


def swiglu_hidden(be, projected):
    half = projected.shape[-1] // 2
    parts = be.split(projected, [half, half], -1)
    return be.mul(parts[0], be.activation(parts[1], SILU))


def normalized_gated_residual(be, policy, residual, branch, gate):
    normalized = be.rms_norm(branch, None, 1e-6)
    bounded = be.activation(gate, TANH)
    return gated_residual(be, policy, residual, normalized,
                          be.reshape(bounded, (residual.shape[0], 1, residual.shape[-1])))


def mochi_norm_scale(be, x, scale):
    """mochi.cpp:230-231: rms_norm(x, no weight, 1e-6) * (1 + scale[B,1,D])."""
    return be.mul(be.rms_norm(x, None, 1e-6),
                  be.add(scalar_f32(1.0), be.reshape(scale, (x.shape[0], 1, x.shape[-1]))))


def multiply_coefficient(be, policy, value, coefficient, role=SOLVER):
    return precision_scalar_binary(be, policy, role, "mul", value, scalar_f32(coefficient))


def linear_combine(be, policy, values, coefficients, role=GUIDANCE):
    """SamplingPrimitives::linear_combine (native/src/sampling/sampling.cpp:173-179)."""
    result = multiply_coefficient(be, policy, values[0], coefficients[0], role)
    for v, c in zip(values[1:], coefficients[1:]):
        result = be.add(result, multiply_coefficient(be, policy, v, c, role))
    return result


def cfg_combine(be, policy, unconditional, conditional, scale):
    neg = multiply_coefficient(be, policy, unconditional, -1.0, GUIDANCE)
    diff = be.add(conditional, neg)
    return be.add(unconditional, multiply_coefficient(be, policy, diff, scale, GUIDANCE))


def euler_update(be, policy, sample, prediction, delta, subtract_prediction):
    sign = -1.0 if subtract_prediction else 1.0
    if SOLVER in policy.scalar_roles:
        coefficient = multiply_coefficient(be, policy, delta, sign)
        return be.add(sample, precision_scalar_binary(be, policy, SOLVER, "mul", prediction, coefficient))
    return be.add(sample, be.mul(prediction, be.mul(delta, scalar_f32(sign))))


def flow_to_x0(be, policy, sample, model_output, sigma):
    return be.add(sample, multiply_coefficient(be, policy, model_output, -sigma, SIGMA))


def group_norm_silu(be, x, groups, weight, bias, eps):
    """autoencoder_kl.cpp:40-41 / mochi.cpp:373-377: GroupNorm, then a separate SiLU kernel."""
    return be.activation(be.group_norm(x, groups, weight, bias, eps), SILU)


def pixel_norm_modulate_silu(be, policy, x, shift, scale, eps=1e-8):
    """LTX decoder_residual (native/src/architectures/ltx.cpp:221-227): silu(modulate(pixel_norm(x), shift,
    scale)) with shift / scale [B, C, 1, 1, 1]; the result is F32 (modulate's contract output)."""
    return be.activation(modulate(be, policy, be.pixel_norm(x, 1, eps), shift, scale), SILU)


def depth_to_space_residual(be, projected, x):
    """LTX depth_to_space (native/src/architectures/ltx.cpp:250-259) after its convolution `projected`:
    pixel_shuffle of the input repeated four times along the channels, both shuffles without their
    first frame, one add."""
    residual = be.pixel_shuffle_nd(x, (2, 2, 2))
    residual = T(np.concatenate([residual.data] * 4, axis=1), residual.dtype)
    residual = be.slice(residual, 2, 1, residual.shape[2])
    y = be.pixel_shuffle_nd(projected, (2, 2, 2))
    return be.add(be.slice(y, 2, 1, y.shape[2]), residual)


def rms_channel_silu(be, x, gamma, eps=1e-12):
    """components/executor.cpp:90-98 as used by the Wan VAE: rms over axis 1, then SiLU."""
    return be.activation(be.rms_norm(x, gamma, eps, 1), SILU)


# ------------------------------------------------------------------------- comparisons --
def bf16_ulp_distance(a_bits: np.ndarray, b_bits: np.ndarray) -> np.ndarray:
    """Distance on the bf16 grid; +0 and -0 coincide; NaN must match NaN, inf must match inf."""
    def key(bits):
        bits = bits.astype(np.int32)
        mag = bits & 0x7FFF
        return np.where(bits & 0x8000, -mag, mag)
    a_bits = np.asarray(a_bits, dtype=np.uint16)
    b_bits = np.asarray(b_bits, dtype=np.uint16)
    d = np.abs(key(a_bits) - key(b_bits)).astype(np.int64)
    a_nan = (a_bits & 0x7FFF) > 0x7F80
    b_nan = (b_bits & 0x7FFF) > 0x7F80
    d[a_nan & b_nan] = 0
    d[a_nan ^ b_nan] = 1 << 20
    a_inf = (a_bits & 0x7FFF) == 0x7F80
    b_inf = (b_bits & 0x7FFF) == 0x7F80
    d[(a_inf ^ b_inf)] = 1 << 20
    return d
