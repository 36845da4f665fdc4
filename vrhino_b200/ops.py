"""Host-side mirror of the reference's operator interface for the non-GEMM path, on top of the
C ABI in ``libvrb.so``.  torch is used for device memory and streams only.

* ``B200Backend`` has the per-operator methods of ``vrhino::Backend``
  (native/include/vrhino/backend.h:74-207 of the reference) that lie on the path, with the
  same names, argument meaning, operand-dtype rules and error texts as the CUDA backend
  (native/src/backend/cuda/cuda_backend.cu).
* module functions ``modulate`` ... ``flow_to_x0`` have the signatures of the helper seams
  (native/include/vrhino/architecture.h:63-86, native/include/vrhino/sampling.h:171-203) and
  run the same chain of per-operator kernels.
* ``fused_*`` functions are the one-pass forms of those chains; each states which chain it
  replaces.  They return exactly what the chain returns.

Every call goes to the CUDA library; nothing here computes on the CPU or through torch ops.
"""
from __future__ import annotations

import ctypes
from dataclasses import dataclass, field

import torch

from . import _lib
from ._lib import VrbError, call

F32, BF16 = torch.float32, torch.bfloat16
_CODE = {torch.float32: _lib.F32, torch.bfloat16: _lib.BF16, torch.uint8: _lib.U8}
SILU, GELU, GELU_TANH, TANH, RELU = 0, 1, 2, 3, 4


def _ptr(t):
    if t is None:
        return None
    if not t.is_cuda:
        raise VrbError("Tensor must be device-resident")
    return ctypes.c_void_p(t.data_ptr())


def _code(t_or_dtype):
    dt = t_or_dtype.dtype if isinstance(t_or_dtype, torch.Tensor) else t_or_dtype
    try:
        return _CODE[dt]
    except KeyError:
        raise VrbError(f"Unsupported dtype {dt}") from None


def _stream():
    return ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)


def _shape(t):
    n = max(t.dim(), 1)
    return (ctypes.c_int64 * n)(*t.shape), t.dim()


def _dense(t):
    if not t.is_contiguous():
        raise VrbError("Tensor must be contiguous")
    return t


def _result(out, shape, dtype, device):
    """The output tensor of an operator: a fresh one, or the caller's reusable buffer after a
    shape / dtype / device / density check."""
    if out is None:
        return torch.empty(tuple(shape), dtype=dtype, device=device)
    if tuple(out.shape) != tuple(shape) or out.dtype != dtype or out.device != device or not out.is_contiguous():
        raise VrbError("output buffer does not match the result's shape, dtype or device")
    return out


@dataclass
class RngState:
    """struct RngState, native/include/vrhino/backend.h:17-21."""
    seed: int = 0
    offset: int = 0
    algorithm_id: str = "pytorch_compat.v1"


class HostScalar:
    """A rank-0 host F32 value (scalar_f32 of native/src/tensor_util.cpp:20)."""

    def __init__(self, value: float):
        self.value = float(value)


def scalar_f32(value: float) -> HostScalar:
    return HostScalar(value)


class B200Backend:
    """Per-operator surface; every method launches one kernel of libvrb.so."""

    def __init__(self, execution_dtype=BF16, device="cuda:0"):
        _lib.load()
        if not torch.cuda.is_available():
            raise VrbError("B200Backend requires a CUDA device; there is no CPU path")
        self.device = torch.device(device)
        self.execution_dtype = execution_dtype
        self._gn_workspace = None

    def name(self):
        return "b200"

    # ---- dtype rule shared by the CUDA host wrappers ----
    def _dtype_of(self, t):
        if isinstance(t, torch.Tensor) and t.is_cuda and t.dtype in (F32, BF16):
            return t.dtype
        return self.execution_dtype

    def copy_to_device(self, t, dtype):
        if isinstance(t, HostScalar):
            return torch.tensor(t.value, dtype=torch.float32).to(self.device).to(dtype) if dtype == F32 else \
                self.cast(torch.tensor(t.value, dtype=torch.float32, device=self.device), dtype)
        if not t.is_cuda:
            t = t.to(self.device)
        return t if t.dtype == dtype else self.cast(t, dtype)

    def cast(self, x, dtype):
        if isinstance(x, HostScalar):
            return self.copy_to_device(x, dtype)
        if not x.is_cuda:
            x = x.to(self.device)
        if x.dtype == dtype:
            return x  # same handle, as the reference (cuda_backend.cu:3200)
        x = _dense(x)
        out = torch.empty(x.shape, dtype=dtype, device=x.device)
        if x.numel():
            call("vrb_cast", _ptr(x), _code(x), _ptr(out), _code(dtype), x.numel(), _stream())
        return out

    def _binary(self, kind, a_raw, b_raw):
        if isinstance(a_raw, torch.Tensor) and a_raw.is_cuda and a_raw.dtype in (F32, BF16):
            dtype = a_raw.dtype
        elif isinstance(b_raw, torch.Tensor) and b_raw.is_cuda and b_raw.dtype in (F32, BF16):
            dtype = b_raw.dtype
        else:
            dtype = self.execution_dtype
        a, b = _dense(self.copy_to_device(a_raw, dtype)), _dense(self.copy_to_device(b_raw, dtype))
        try:
            shape = torch.broadcast_shapes(a.shape, b.shape)
        except RuntimeError:
            raise VrbError("Incompatible broadcast shapes") from None
        out = torch.empty(shape, dtype=dtype, device=self.device)
        (ashape, arank), (bshape, brank) = _shape(a), _shape(b)
        call("vrb_binary", kind, _ptr(a), ashape, arank, _ptr(b), bshape, brank, _ptr(out), _code(dtype), _stream())
        return out

    def add(self, a, b): return self._binary(_lib.ADD, a, b)
    def mul(self, a, b): return self._binary(_lib.MUL, a, b)
    def div(self, a, b): return self._binary(_lib.DIV, a, b)
    def maximum(self, a, b): return self._binary(_lib.MAX, a, b)

    def reshape(self, x, shape):
        return self.copy_to_device(x, self._dtype_of(x)).reshape(shape)

    def _param(self, t):
        """Optional affine parameter: uploaded if it still lives on the host."""
        return None if t is None else _dense(t if t.is_cuda else t.to(self.device))

    def layer_norm(self, raw, weight, bias, eps, out=None):
        weight, bias = self._param(weight), self._param(bias)
        dtype = self._dtype_of(raw)
        x = _dense(self.copy_to_device(raw, dtype))
        width = x.shape[-1]
        for name, t in (("weight", weight), ("bias", bias)):
            if t is not None and t.numel() != width:
                raise VrbError(f"layer norm {name} mismatch")
        out = _result(out, x.shape, x.dtype, x.device)
        call("vrb_layer_norm", _ptr(x), _code(x), _ptr(weight), _code(weight) if weight is not None else 0,
             _ptr(bias), _code(bias) if bias is not None else 0, _ptr(out), x.numel() // width, width,
             ctypes.c_float(eps), _stream())
        return out

    def rms_norm(self, raw, weight, eps, axis=-1, output=None):
        """``output=None`` is the reference default (DType::F16 meaning "same as the input")."""
        weight = self._param(weight)
        rank = raw.dim()
        if axis < 0:
            axis += rank
        if not 0 <= axis < rank:
            raise VrbError("rms_norm axis invalid")
        dtype = self._dtype_of(raw)
        out_dtype = dtype if output is None else output
        x = _dense(self.copy_to_device(raw, dtype))
        if weight is not None and weight.numel() != x.shape[axis]:
            raise VrbError("rms norm weight mismatch")
        out = torch.empty(x.shape, dtype=out_dtype, device=x.device)
        wcode = _code(weight) if weight is not None else 0
        if axis == rank - 1:
            width = x.shape[-1]
            call("vrb_rms_norm", _ptr(x), _code(x), _ptr(weight), wcode, _ptr(out), _code(out_dtype),
                 x.numel() // width, width, ctypes.c_float(eps), _stream())
        else:
            if out_dtype != dtype:
                raise VrbError("mixed-dtype rms_norm currently requires final axis")
            width = x.shape[axis]
            inner = 1
            for d in x.shape[axis + 1:]:
                inner *= d
            call("vrb_rms_norm_axis", _ptr(x), _code(x), _ptr(weight), wcode, _ptr(out),
                 x.numel() // (width * inner), width, inner, ctypes.c_float(eps), 0, _stream())
        return out

    def pixel_norm(self, raw, dim=1, eps=1e-8, out=None):
        """CudaBackend::pixel_norm (native/src/backend/cuda/cuda_backend.cu:5048-5086)."""
        rank = raw.dim()
        if dim < 0:
            dim += rank
        if not 0 <= dim < rank:
            raise VrbError("pixel norm dim invalid")
        dtype = self._dtype_of(raw)
        x = _dense(self.copy_to_device(raw, dtype))
        channels, inner = x.shape[dim], 1
        for d in x.shape[dim + 1:]:
            inner *= d
        out = _result(out, x.shape, dtype, x.device)
        call("vrb_pixel_norm", _ptr(x), _code(x), None, None, 0, 0, _ptr(out), _code(dtype),
             x.numel() // (channels * inner), channels, inner, ctypes.c_float(eps), _stream())
        return out

    def l2_normalize(self, x, dim, eps, out=None):
        """CudaBackend::l2_normalize (cuda_backend.cu:5088-5110): x / (sqrt(sum(x^2) over `dim`) + eps)."""
        if dim < 0:
            dim += x.dim()
        if not (0 <= dim < x.dim()) or eps < 0:
            raise VrbError("l2 normalize contract violation")
        dtype = self._dtype_of(x)
        x = _dense(self.copy_to_device(x, dtype))
        channels = x.shape[dim]
        inner = 1
        for d in x.shape[dim + 1:]:
            inner *= d
        out = _result(out, x.shape, dtype, x.device)
        call("vrb_l2_normalize", _ptr(x), _ptr(out), _code(dtype), x.numel() // (channels * inner), channels, inner,
             ctypes.c_float(eps), _stream())
        return out

    # ---- layout operators (cuda_backend.cu:3936-3970, :4190-4196, :4875-4883) ----
    @staticmethod
    def _extents(values):
        return (ctypes.c_int64 * max(len(values), 1))(*[int(v) for v in values])

    def permute(self, raw, dims, out=None):
        """CudaBackend::permute: out[c] = x[c permuted back]; "Invalid permutation" unless dims permutes the axes."""
        if len(dims) != raw.dim():
            raise VrbError("permute rank mismatch")
        dtype = self._dtype_of(raw)
        x = _dense(self.copy_to_device(raw, dtype))
        if sorted(int(d) for d in dims) != list(range(x.dim())):
            raise VrbError("Invalid permutation")
        out = _result(out, tuple(x.shape[int(d)] for d in dims), dtype, x.device)
        call("vrb_permute", _ptr(x), _ptr(out), _code(dtype), x.dim(), self._extents(x.shape), self._extents(dims), _stream())
        return out

    def slice(self, raw, dim, start, stop, out=None):
        """CudaBackend::slice: negative dim / start / stop count from the end, then start is clamped into
        [0, extent] and stop into [start, extent]."""
        if dim < 0:
            dim += raw.dim()
        if not 0 <= dim < raw.dim():
            raise VrbError("slice dimension invalid")
        size = raw.shape[dim]
        start = start + size if start < 0 else start
        stop = stop + size if stop < 0 else stop
        start = min(max(start, 0), size)
        stop = min(max(stop, start), size)
        dtype = self._dtype_of(raw)
        x = _dense(self.copy_to_device(raw, dtype))
        shape = list(x.shape)
        shape[dim] = stop - start
        out = _result(out, tuple(shape), dtype, x.device)
        call("vrb_slice", _ptr(x), _ptr(out), _code(dtype), x.dim(), self._extents(x.shape), dim, start, stop, _stream())
        return out

    def split(self, x, sections, dim):
        """CudaBackend::split (cuda_backend.cu:3972-3976): consecutive slices."""
        if dim < 0:
            dim += x.dim()
        if sum(sections) != x.shape[dim]:
            raise VrbError("split sections mismatch")
        parts, offset = [], 0
        for section in sections:
            parts.append(self.slice(x, dim, offset, offset + section))
            offset += section
        return parts

    def concat(self, tensors, dim, out=None):
        """CudaBackend::concat: the dtype is the first input's (a device F32 / BF16 tensor) else the execution dtype."""
        if not tensors:
            raise VrbError("concat requires inputs")
        rank = tensors[0].dim()
        if dim < 0:
            dim += rank
        if not 0 <= dim < rank:
            raise VrbError("concat dimension invalid")
        shape = list(tensors[0].shape)
        shape[dim] = 0
        for t in tensors:
            if t.dim() != rank:
                raise VrbError("concat rank mismatch")
            if any(t.shape[d] != tensors[0].shape[d] for d in range(rank) if d != dim):
                raise VrbError("concat shape mismatch")
            shape[dim] += t.shape[dim]
        dtype = self._dtype_of(tensors[0])
        parts = [_dense(self.copy_to_device(t, dtype)) for t in tensors]
        out = _result(out, tuple(shape), dtype, parts[0].device)
        pointers = (ctypes.c_void_p * len(parts))(*[_ptr(t).value for t in parts])
        call("vrb_concat", pointers, self._extents([t.shape[dim] for t in parts]), len(parts), _ptr(out), _code(dtype), rank,
             self._extents(shape), dim, _stream())
        return out

    def pad(self, raw, padding, value=0.0, replicate=False, out=None):
        """CudaBackend::pad: `padding` is (before, after) pairs from the innermost axis outwards."""
        if len(padding) % 2 or len(padding) > 2 * raw.dim():
            raise VrbError("Invalid pad vector")
        if any(p < 0 for p in padding):
            raise VrbError("Negative padding unsupported")
        dtype = self._dtype_of(raw)
        x = _dense(self.copy_to_device(raw, dtype))
        before, after = [0] * x.dim(), [0] * x.dim()
        for pair in range(len(padding) // 2):
            before[x.dim() - 1 - pair], after[x.dim() - 1 - pair] = int(padding[2 * pair]), int(padding[2 * pair + 1])
        out = _result(out, tuple(s + b + a for s, b, a in zip(x.shape, before, after)), dtype, x.device)
        call("vrb_pad", _ptr(x), _ptr(out), _code(dtype), x.dim(), self._extents(x.shape), self._extents(before), self._extents(after),
             ctypes.c_float(value), int(bool(replicate)), _stream())
        return out

    def pad_axes(self, raw, before, after, value, replicate_axes, out=None):
        """vrb_pad_axes: per-axis before / after extents and per-axis mode (True replicates, False fills with value)."""
        dtype = self._dtype_of(raw)
        x = _dense(self.copy_to_device(raw, dtype))
        if not (len(before) == len(after) == len(replicate_axes) == x.dim()):
            raise VrbError("Invalid pad vector")
        if any(p < 0 for p in list(before) + list(after)):
            raise VrbError("Negative padding unsupported")
        out = _result(out, tuple(s + b + a for s, b, a in zip(x.shape, before, after)), dtype, x.device)
        modes = (ctypes.c_int * x.dim())(*[int(bool(m)) for m in replicate_axes])
        call("vrb_pad_axes", _ptr(x), _ptr(out), _code(dtype), x.dim(), self._extents(x.shape), self._extents(before),
             self._extents(after), ctypes.c_float(value), modes, _stream())
        return out

    def interpolate_nearest(self, raw, factors, out=None):
        """CudaBackend::interpolate_nearest (cuda_backend.cu:5010-5016): the trailing len(factors) axes grow to
        floor(extent * factor); out[c] = x[floor(c * in / out)] along every axis."""
        import math
        if len(factors) > raw.dim() - 2:
            raise VrbError("interpolate factor rank mismatch")
        if any(f <= 0 for f in factors):
            raise VrbError("Invalid interpolation factor")
        dtype = self._dtype_of(raw)
        x = _dense(self.copy_to_device(raw, dtype))
        shape = list(x.shape)
        start = x.dim() - len(factors)
        for i, f in enumerate(factors):
            shape[start + i] = int(math.floor(shape[start + i] * float(f)))
        out = _result(out, tuple(shape), dtype, x.device)
        call("vrb_interpolate_nearest", _ptr(x), _ptr(out), _code(dtype), x.dim(), self._extents(x.shape), self._extents(shape), _stream())
        return out

    def reduce_sum(self, raw, dim, keepdim=False, out=None):
        """CudaBackend::reduce_sum (cuda_backend.cu:4885-4892): the sum over `dim`, accumulated in F32 in index order."""
        if dim < 0:
            dim += raw.dim()
        if not 0 <= dim < raw.dim():
            raise VrbError("reduce dimension invalid")
        dtype = self._dtype_of(raw)
        x = _dense(self.copy_to_device(raw, dtype))
        outer, inner = 1, 1
        for d in x.shape[:dim]:
            outer *= d
        for d in x.shape[dim + 1:]:
            inner *= d
        shape = list(x.shape)
        if keepdim:
            shape[dim] = 1
        else:
            del shape[dim]
        out = _result(out, tuple(shape), dtype, x.device)
        call("vrb_reduce_sum", _ptr(x), _ptr(out), _code(dtype), outer, x.shape[dim], inner, _stream())
        return out

    def rng_normal(self, state, shape, dtype, out=None):
        """CudaBackend::rng_normal (cuda_backend.cu:5120-5126): element i = the first normal of the Philox4x32-10 stream
        (state.seed, subsequence i, state.offset); the state's offset grows by 4."""
        if state.algorithm_id != "pytorch_compat.v1":
            raise VrbError("Unsupported RNG algorithm")
        if dtype not in (F32, BF16):
            raise VrbError("rng_normal dtype unsupported")
        out = _result(out, tuple(shape), dtype, self.device)
        call("vrb_rng_normal", _ptr(out), _code(dtype), out.numel(), int(state.seed) & (2 ** 64 - 1), int(state.offset) & (2 ** 64 - 1),
             _stream())
        state.offset += 4
        return out

    def softmax(self, raw, axis, out=None):
        """CudaBackend::softmax (cuda_backend.cu:4893-4917): over `axis`, the denominator accumulated in F32 in index order."""
        if axis < 0:
            axis += raw.dim()
        if not 0 <= axis < raw.dim():
            raise VrbError("softmax axis invalid")
        dtype = self._dtype_of(raw)
        x = _dense(self.copy_to_device(raw, dtype))
        outer, inner = 1, 1
        for d in x.shape[:axis]:
            outer *= d
        for d in x.shape[axis + 1:]:
            inner *= d
        out = _result(out, tuple(x.shape), dtype, x.device)
        call("vrb_softmax", _ptr(x), _ptr(out), _code(dtype), outer, x.shape[axis], inner, _stream())
        return out

    def indexed_gather(self, table_raw, indices_raw, out=None):
        """CudaBackend::indexed_gather (cuda_backend.cu:3981-4055): table [rows, width] or [batch, rows, width], integer
        indices [...] (their first axis the batch when the table has one) -> [..., width] in the execution dtype.  The
        indices are checked on the host first, as the reference does."""
        import numpy as np
        if table_raw.dim() not in (2, 3):
            raise VrbError("indexed_gather table must have rank 2 or 3")
        indices = torch.as_tensor(np.asarray(indices_raw)) if not isinstance(indices_raw, torch.Tensor) else indices_raw
        if indices.dim() < 1 or indices.dtype not in (torch.int64, torch.int32):
            raise VrbError("indexed_gather indices must be rank >=1 int64/int32")
        batched = table_raw.dim() == 3
        if batched and indices.shape[0] != table_raw.shape[0]:
            raise VrbError("indexed_gather batch dimension mismatch")
        rows, width = table_raw.shape[-2], table_raw.shape[-1]
        host = indices.cpu()
        if host.numel() and (int(host.min()) < 0 or int(host.max()) >= rows):
            raise VrbError("indexed_gather index out of range")
        dtype = self.execution_dtype
        table = _dense(self.copy_to_device(table_raw, dtype))
        device_indices = _dense(indices.to(table.device))
        out = _result(out, tuple(indices.shape) + (width,), dtype, table.device)
        per_batch = indices.numel() // indices.shape[0] if batched else indices.numel()
        call("vrb_indexed_gather", _ptr(table), _ptr(device_indices), 3 if indices.dtype == torch.int64 else 4, _ptr(out), _code(dtype),
             table.shape[0] if batched else 0, rows, width, per_batch, _stream())
        return out

    def sinusoidal_embedding(self, raw, width, flip, downscale, frequency_f64, out=None):
        """CudaBackend::sinusoidal_embedding: positions [n] -> [n, width]."""
        if raw.dim() != 1 or width <= 0:
            raise VrbError("sinusoidal embedding contract violation")
        dtype = self._dtype_of(raw)
        x = _dense(self.copy_to_device(raw, dtype))
        out = _result(out, (x.numel(), width), dtype, x.device)
        call("vrb_sinusoidal_embedding", _ptr(x), _ptr(out), _code(dtype), x.numel(), width, int(bool(flip)),
             ctypes.c_double(downscale), int(bool(frequency_f64)), _stream())
        return out

    def pixel_shuffle_nd(self, raw, factors, out=None):
        """CudaBackend::pixel_shuffle_nd (native/src/backend/cuda/cuda_backend.cu:5112-5118)."""
        if raw.dim() != 5 or len(factors) != 3:
            raise VrbError("pixel_shuffle_nd requires 5D and 3 factors")
        ft, fh, fw = (int(f) for f in factors)
        product = ft * fh * fw
        if raw.shape[1] % product:
            raise VrbError("pixel shuffle channel mismatch")
        dtype = self._dtype_of(raw)
        x = _dense(self.copy_to_device(raw, dtype))
        b, c, t, h, w = x.shape
        out = _result(out, (b, c // product, t * ft, h * fh, w * fw), dtype, x.device)
        call("vrb_pixel_shuffle", _ptr(x), _ptr(out), _code(dtype), b, c // product, t, h, w, ft, fh, fw, _stream())
        return out

    def activation(self, raw, kind, out=None):
        dtype = self._dtype_of(raw)
        x = _dense(self.copy_to_device(raw, dtype))
        out = _result(out, x.shape, x.dtype, x.device)
        call("vrb_activation", int(kind), _ptr(x), _ptr(out), _code(x), x.numel(), _stream())
        return out

    def clamp(self, raw, minimum, maximum):
        x = _dense(self.copy_to_device(raw, self._dtype_of(raw)))
        out = torch.empty_like(x)
        call("vrb_clamp", _ptr(x), _ptr(out), _code(x), x.numel(), ctypes.c_float(minimum), ctypes.c_float(maximum), _stream())
        return out

    def exp(self, raw):
        x = _dense(self.copy_to_device(raw, self._dtype_of(raw)))
        out = torch.empty_like(x)
        call("vrb_exp", _ptr(x), _ptr(out), _code(x), x.numel(), _stream())
        return out

    def sqrt(self, raw):
        x = _dense(self.copy_to_device(raw, self._dtype_of(raw)))
        out = torch.empty_like(x)
        call("vrb_sqrt", _ptr(x), _ptr(out), _code(x), x.numel(), _stream())
        return out

    def rope_nd(self, raw, cos_raw, sin_raw):
        dtype = self._dtype_of(raw)
        f_dtype = cos_raw.dtype if (cos_raw.is_cuda and cos_raw.dtype in (F32, BF16)) else dtype
        x = _dense(self.copy_to_device(raw, dtype))
        c, s = _dense(self.copy_to_device(cos_raw, f_dtype)), _dense(self.copy_to_device(sin_raw, f_dtype))
        if c.shape != s.shape:
            raise VrbError("RoPE frequency mismatch")
        out = torch.empty_like(x)
        (xs, xr), (fs, fr) = _shape(x), _shape(c)
        call("vrb_rope", _ptr(x), _code(x), xs, xr, _ptr(c), _ptr(s), _code(c), fs, fr, _ptr(out), _stream())
        return out

    def dequantize(self, packed, scales, group_size, kind=_lib.Q_FP8, dtype=BF16, shape=None, out=None):
        """copy_to_device of a quantized weight (cuda_backend.cu:3214-3296)."""
        packed = _dense(packed.to(self.device))
        scales = _dense(scales.to(self.device, torch.float32))
        shape = tuple(shape or packed.shape)
        rows = shape[0]
        inner = 1
        for d in shape[1:]:
            inner *= d
        out = _result(out, shape, dtype, packed.device)
        call("vrb_dequantize", kind, _ptr(packed), _ptr(scales), _ptr(out), _code(dtype), rows, inner, group_size, _stream())
        return out

    def _workspace(self, batch, groups):
        need = _lib.load().vrb_group_norm_workspace_bytes(batch, groups)
        if self._gn_workspace is None or self._gn_workspace.numel() < need:
            self._gn_workspace = torch.empty(need, dtype=torch.uint8, device=self.device)
        return self._gn_workspace, need

    def group_norm(self, raw, groups, weight, bias, eps, fuse_silu=False, out=None):
        if raw.dim() < 3 or groups <= 0 or raw.shape[1] % groups:
            raise VrbError("group norm shape/groups mismatch")
        weight, bias = self._param(weight), self._param(bias)
        dtype = self._dtype_of(raw)
        x = _dense(self.copy_to_device(raw, dtype))
        batch, channels = x.shape[0], x.shape[1]
        spatial = x.numel() // (batch * channels)
        out = _result(out, x.shape, x.dtype, x.device)
        ws, need = self._workspace(batch, groups)
        call("vrb_group_norm", _ptr(x), _code(x), _ptr(weight), _code(weight) if weight is not None else 0,
             _ptr(bias), _code(bias) if bias is not None else 0, _ptr(out), batch, channels, spatial, groups,
             ctypes.c_float(eps), int(fuse_silu), _ptr(ws), need, _stream())
        return out


    def group_norm_frames(self, raw, groups, weight, bias, eps, fuse_silu=False, out=None):
        """Per-frame GroupNorm of [B, C, T, H, W] without the two permutes of frame_group_norm
        (native/src/architectures/mochi.cpp:365-371): statistics per (batch entry, frame, group)."""
        if raw.dim() != 5 or groups <= 0 or raw.shape[1] % groups:
            raise VrbError("group norm shape/groups mismatch")
        weight, bias = self._param(weight), self._param(bias)
        dtype = self._dtype_of(raw)
        x = _dense(self.copy_to_device(raw, dtype))
        batch, channels, frames = x.shape[0], x.shape[1], x.shape[2]
        spatial = x.shape[3] * x.shape[4]
        out = _result(out, x.shape, x.dtype, x.device)
        need = _lib.load().vrb_group_norm_frames_workspace_bytes(batch, frames, groups)
        if self._gn_workspace is None or self._gn_workspace.numel() < need:
            self._gn_workspace = torch.empty(need, dtype=torch.uint8, device=self.device)
        call("vrb_group_norm_frames", _ptr(x), _code(x), _ptr(weight), _code(weight) if weight is not None else 0,
             _ptr(bias), _code(bias) if bias is not None else 0, _ptr(out), batch, channels, frames, spatial, groups,
             ctypes.c_float(eps), int(fuse_silu), _ptr(self._gn_workspace), need, _stream())
        return out


# ------------------------------------------------------------------ precision policy view --
GUIDANCE, SOLVER, SIGMA = "GuidanceCoefficient", "SolverCoefficient", "Sigma"


@dataclass
class Policy:
    """The decisions of native/src/precision/precision.cpp the path depends on: residual-state
    dtype, requested dtype, and which scalar roles a v2 policy declares.  Modulation and RoPE
    contracts are F32 under every policy (precision.cpp:311-327)."""
    requested: torch.dtype = BF16
    residual: torch.dtype = BF16
    scalar_roles: frozenset = field(default_factory=frozenset)

    @staticmethod
    def unqualified_default(dtype=BF16):
        return Policy(dtype, dtype)

    @staticmethod
    def production_bf16():
        return Policy(BF16, F32)

    @staticmethod
    def fp32():
        return Policy(F32, F32)

    def with_scalar_roles(self, roles):
        return Policy(self.requested, self.residual, frozenset(roles))


# ------------------------------------------------ helper seams: same chains as the reference --
def modulate(be, policy, x, shift, scale):
    """native/src/architectures/common.cpp:51-61"""
    t = be.add(be.mul(be.cast(x, F32), be.add(scalar_f32(1.0), be.cast(scale, F32))), be.cast(shift, F32))
    return be.cast(t, F32)


def attention_norm(be, policy, x, weight, eps, axis=-1):
    """common.cpp:62-68"""
    return be.rms_norm(x, weight, eps, axis, F32)


def operation_rope(be, policy, x, cosine, sine):
    """common.cpp:69-76"""
    return be.rope_nd(be.cast(x, F32), cosine, sine)


def residual_add(be, policy, residual, branch):
    """common.cpp:134-138"""
    d = policy.residual
    return be.add(be.cast(residual, d), be.cast(branch, d))


def gated_residual(be, policy, residual, branch, gate):
    """common.cpp:139-144"""
    d = policy.residual
    return be.add(be.cast(residual, d), be.mul(be.cast(branch, d), be.cast(gate, d)))


def precision_scalar_binary(be, policy, role, value, coefficient: float):
    """native/src/precision/precision.cpp:196-223, Multiply with a host F32 scalar."""
    if role not in policy.scalar_roles:
        return be.mul(value, scalar_f32(coefficient))
    result = be.mul(be.copy_to_device(value, F32), be.copy_to_device(scalar_f32(coefficient), F32))
    return result if result.dtype == value.dtype else be.cast(result, value.dtype)


def cfg_combine(be, policy, unconditional, conditional, scale):
    """native/src/sampling/sampling.cpp:181-183"""
    neg = precision_scalar_binary(be, policy, GUIDANCE, unconditional, -1.0)
    diff = be.add(conditional, neg)
    return be.add(unconditional, precision_scalar_binary(be, policy, GUIDANCE, diff, scale))


def _euler_delta(be, policy, delta: float) -> float:
    """Magnitude the one-element coefficient tensor of euler_update holds (sampling.cpp:185-193):
    with a declared solver role, or F32 execution, delta itself; otherwise the product of two
    host scalars runs in the BF16 execution dtype and rounds delta to BF16."""
    if SOLVER in policy.scalar_roles or be.execution_dtype == F32:
        return float(delta)
    return float(torch.tensor(delta, dtype=torch.float32).to(torch.bfloat16).float())


def euler_update(be, policy, sample, prediction, delta: float, subtract_prediction: bool):
    k = _euler_delta(be, policy, delta) * (-1.0 if subtract_prediction else 1.0)
    return be.add(sample, precision_scalar_binary(be, policy, SOLVER, prediction, k))


def flow_to_x0(be, policy, sample, model_output, sigma: float):
    """sampling.cpp:200-202"""
    return be.add(sample, precision_scalar_binary(be, policy, SIGMA, model_output, -sigma))


# ------------------------------------------------------------------------- fused one-pass forms --
def _vec_layout(rows, x_shape, vec):
    """rows_per_vector / vector count for a [B,1,D]- or [B,S,D]-shaped (or flat [D]) vector."""
    width = x_shape[-1]
    n = vec.numel() // width
    if n * width != vec.numel():
        raise VrbError("Incompatible broadcast shapes")
    if n == 1:
        return rows, 1
    if n == rows:
        return 1, rows
    batch = x_shape[0]
    if n == batch and rows % batch == 0:
        return rows // batch, batch
    raise VrbError("Incompatible broadcast shapes")


def fused_layer_norm_modulate(be, x, weight, bias, eps, shift, scale, out_dtype=BF16, out=None):
    """cast(modulate(layer_norm(x, weight, bias, eps), shift, scale), out_dtype) in one pass."""
    x = _dense(x)
    width = x.shape[-1]
    rows = x.numel() // width
    rpv, nvec = _vec_layout(rows, x.shape, scale)
    if shift is not None and (shift.dtype != scale.dtype or shift.numel() != scale.numel()):
        raise VrbError("modulate: shift and scale must share dtype and shape")
    out = _result(out, x.shape, out_dtype, x.device)
    call("vrb_layer_norm_modulate", _ptr(x), _code(x), _ptr(weight), _code(weight) if weight is not None else 0,
         _ptr(bias), _code(bias) if bias is not None else 0, _ptr(_dense(scale)), _ptr(shift), _code(scale),
         rpv, nvec, _ptr(out), _code(out_dtype), rows, width, ctypes.c_float(eps), _stream())
    return out


def fused_layer_norm_cast(be, x, weight, bias, eps, out_dtype=BF16, out=None):
    """cast(layer_norm(x, weight, bias, eps), out_dtype) in one pass."""
    x = _dense(x)
    width = x.shape[-1]
    out = _result(out, x.shape, out_dtype, x.device)
    call("vrb_layer_norm_cast", _ptr(x), _code(x), _ptr(weight), _code(weight) if weight is not None else 0,
         _ptr(bias), _code(bias) if bias is not None else 0, _ptr(out), _code(out_dtype), x.numel() // width, width,
         ctypes.c_float(eps), _stream())
    return out


def fused_rms_norm_modulate(be, x, eps, shift, scale, out_dtype=BF16, out=None):
    """cast(modulate(rms_norm(x, None, eps), shift, scale), out_dtype) -- the LTX block."""
    x = _dense(x)
    width = x.shape[-1]
    rows = x.numel() // width
    rpv, nvec = _vec_layout(rows, x.shape, scale)
    out = _result(out, x.shape, out_dtype, x.device)
    call("vrb_rms_norm_modulate", _ptr(x), _code(x), _ptr(_dense(scale)), _ptr(shift), _code(scale), rpv, nvec,
         _ptr(out), _code(out_dtype), rows, width, ctypes.c_float(eps), _stream())
    return out


def fused_rms_norm_scale(be, x, scale, eps=1e-6, out=None):
    """mul(rms_norm(x, None, eps), add(1, scale[B,1,D])) -- native/src/architectures/mochi.cpp:230-231."""
    x = _dense(x)
    width = x.shape[-1]
    rows = x.numel() // width
    rpv, nvec = _vec_layout(rows, x.shape, scale)
    out = _result(out, x.shape, x.dtype, x.device)
    call("vrb_rms_norm_scale", _ptr(x), _code(x), _ptr(_dense(scale)), _code(scale), rpv, nvec, _ptr(out),
         rows, width, ctypes.c_float(eps), _stream())
    return out


def fused_rms_norm_rope(be, x, weight, eps, cosine, sine, heads=1, per_head_norm=False, out_dtype=BF16, out=None):
    """cast(operation_rope(split_heads(attention_norm(x, weight, eps)), cos, sin), out_dtype).

    x is [B, S, D].  per_head_norm=False: normalise over D, then split into `heads` (Wan,
    native/src/architectures/wan.cpp:38-52); True: split first, normalise each head (Mochi,
    mochi.cpp:182-187).  cosine/sine: F32 [1|B, S, 1, d] (shared by the heads) or [1|B, S, H, d],
    or None for norm + cast only.
    """
    x = _dense(x)
    width = x.shape[-1]
    rows = x.numel() // width
    head_width = width // heads
    norm_width = head_width if per_head_norm else width
    out = _result(out, x.shape, out_dtype, x.device)
    if cosine is None:
        f_rows, f_width, rpf, cp, sp = 0, 8, 1, None, None
    else:
        if cosine.dtype != F32 or cosine.shape != sine.shape:
            raise VrbError("RoPE frequency mismatch")
        cosine, sine = _dense(cosine), _dense(sine)
        f_width = cosine.shape[-1] * cosine.shape[-2] if cosine.dim() >= 2 else cosine.shape[-1]
        if cosine.shape[-1] != head_width or f_width not in (head_width, width):
            raise VrbError("Incompatible broadcast shapes")
        f_rows = cosine.numel() // f_width
        if f_rows not in (rows, rows // x.shape[0]):
            raise VrbError("Incompatible broadcast shapes")
        rpf, cp, sp = 1, _ptr(cosine), _ptr(sine)
    call("vrb_rms_norm_rope", _ptr(x), _code(x), _ptr(weight), _code(weight), cp, sp, f_rows, f_width, rpf,
         _ptr(out), _code(out_dtype), rows, width, norm_width, ctypes.c_float(eps), _stream())
    return out


def fused_rms_norm_rope_pair(be, x_a, weight_a, x_b, weight_b, eps, cosine, sine, heads=1, per_head_norm=False,
                             out_dtype=BF16, out=None):
    """fused_rms_norm_rope on two tensors in ONE launch: the q and k projections of an attention
    block (wan.cpp:38-52), or -- cosine None -- the cross-attention q and its text-token k, whose row
    counts differ.  Same width, dtype and tables for both; each has its own norm weight.  Returns
    (out_a, out_b), bit-identical to two fused_rms_norm_rope calls."""
    x_a, x_b = _dense(x_a), _dense(x_b)
    width = x_a.shape[-1]
    if x_b.shape[-1] != width or x_a.dtype != x_b.dtype or weight_a.dtype != weight_b.dtype:
        raise VrbError("Incompatible broadcast shapes")
    rows_a, rows_b = x_a.numel() // width, x_b.numel() // width
    head_width = width // heads
    norm_width = head_width if per_head_norm else width
    out_a, out_b = out if out is not None else (None, None)
    out_a = _result(out_a, x_a.shape, out_dtype, x_a.device)
    out_b = _result(out_b, x_b.shape, out_dtype, x_b.device)
    if cosine is None:
        f_rows, f_width, cp, sp = 0, 8, None, None
    else:
        if cosine.dtype != F32 or cosine.shape != sine.shape:
            raise VrbError("RoPE frequency mismatch")
        cosine, sine = _dense(cosine), _dense(sine)
        f_width = cosine.shape[-1] * cosine.shape[-2] if cosine.dim() >= 2 else cosine.shape[-1]
        if cosine.shape[-1] != head_width or f_width not in (head_width, width):
            raise VrbError("Incompatible broadcast shapes")
        f_rows = cosine.numel() // f_width
        for x, rows in ((x_a, rows_a), (x_b, rows_b)):
            if f_rows not in (rows, rows // x.shape[0]):
                raise VrbError("Incompatible broadcast shapes")
        cp, sp = _ptr(cosine), _ptr(sine)
    call("vrb_rms_norm_rope_pair", _ptr(x_a), _ptr(weight_a), _ptr(out_a), rows_a, _ptr(x_b), _ptr(weight_b), _ptr(out_b), rows_b,
         _code(x_a), _code(weight_a), cp, sp, _lib.F32, f_rows, f_width, 1, _code(out_dtype), width, norm_width,
         ctypes.c_float(eps), _stream())
    return out_a, out_b


def fused_gated_residual(be, policy, residual, branch, gate, out=None):
    """gated_residual(...) / residual_add(...) (gate None) of common.cpp:134-144 in one pass."""
    residual, branch = _dense(residual), _dense(branch)
    width = residual.shape[-1]
    rows = residual.numel() // width
    rpv, nvec = (1, 1) if gate is None else _vec_layout(rows, residual.shape, gate)
    out = _result(out, residual.shape, policy.residual, residual.device)
    call("vrb_gated_residual", _ptr(residual), _code(residual), _ptr(branch), _code(branch),
         _ptr(gate), _code(gate) if gate is not None else 0, rpv, nvec, _ptr(out), _code(policy.residual),
         rows, width, _stream())
    return out


def fused_gated_residual_layer_norm(be, policy, residual, branch, gate, weight, bias, eps, shift=None, scale=None,
                                    out_dtype=BF16, state_out=None, out=None):
    """The residual update and the LayerNorm the block applies to the updated stream next
    (native/src/architectures/wan.cpp:95-110), one pass when the stream is bf16:
        state = gated_residual(residual, branch, gate)            (residual_add when gate is None)
        normed = cast(modulate(layer_norm(state, weight, bias, eps), shift, scale), out_dtype)
                 (no modulation when scale is None)
    Returns (state, normed)."""
    residual, branch = _dense(residual), _dense(branch)
    width = residual.shape[-1]
    rows = residual.numel() // width
    grpv, gvec = (1, 1) if gate is None else _vec_layout(rows, residual.shape, gate)
    mrpv, mvec = (1, 1) if scale is None else _vec_layout(rows, residual.shape, scale)
    if scale is not None and shift is not None and (shift.dtype != scale.dtype or shift.numel() != scale.numel()):
        raise VrbError("modulate: shift and scale must share dtype and shape")
    state = _result(state_out, residual.shape, policy.residual, residual.device)
    normed = _result(out, residual.shape, out_dtype, residual.device)
    call("vrb_gated_residual_layer_norm_modulate", _ptr(residual), _code(residual), _ptr(branch), _code(branch),
         _ptr(gate), _code(gate) if gate is not None else 0, grpv, gvec, _ptr(state), _code(policy.residual),
         _ptr(weight), _code(weight) if weight is not None else 0, _ptr(bias), _code(bias) if bias is not None else 0,
         _ptr(_dense(scale)) if scale is not None else None, _ptr(shift), _code(scale) if scale is not None else 0, mrpv, mvec,
         _ptr(normed), _code(out_dtype), rows, width, ctypes.c_float(eps), _stream())
    return state, normed


def fused_gated_residual_rms_norm_modulate(be, policy, residual, branch, gate, eps, shift, scale, out_dtype=BF16,
                                           state_out=None, out=None):
    """The LTX block's residual update and its next RMSNorm (no weight) -> modulate
    (native/src/architectures/ltx.cpp:100-151), one pass when the branch is bf16 and the stream keeps its dtype.
    Returns (state, normed)."""
    residual, branch = _dense(residual), _dense(branch)
    width = residual.shape[-1]
    rows = residual.numel() // width
    grpv, gvec = (1, 1) if gate is None else _vec_layout(rows, residual.shape, gate)
    mrpv, mvec = _vec_layout(rows, residual.shape, scale)
    if shift is not None and (shift.dtype != scale.dtype or shift.numel() != scale.numel()):
        raise VrbError("modulate: shift and scale must share dtype and shape")
    state = _result(state_out, residual.shape, policy.residual, residual.device)
    normed = _result(out, residual.shape, out_dtype, residual.device)
    call("vrb_gated_residual_rms_norm_modulate", _ptr(residual), _code(residual), _ptr(branch), _code(branch),
         _ptr(gate), _code(gate) if gate is not None else 0, grpv, gvec, _ptr(state), _code(policy.residual),
         _ptr(_dense(scale)), _ptr(shift), _code(scale), mrpv, mvec, _ptr(normed), _code(out_dtype), rows, width,
         ctypes.c_float(eps), _stream())
    return state, normed


def fused_rms_norm_gated_residual(be, policy, residual, branch, bounded_gate, eps=1e-6, out=None):
    """gated_residual(residual, rms_norm(branch, None, eps), bounded_gate) -- mochi.cpp:204-211
    after the tanh on the [B, D] gate."""
    residual, branch = _dense(residual), _dense(branch)
    width = residual.shape[-1]
    rows = residual.numel() // width
    rpv, nvec = _vec_layout(rows, residual.shape, bounded_gate)
    out = _result(out, residual.shape, policy.residual, residual.device)
    call("vrb_rms_norm_gated_residual", _ptr(residual), _code(residual), _ptr(branch), _code(branch),
         _ptr(_dense(bounded_gate)), _code(bounded_gate), rpv, nvec, _ptr(out), _code(policy.residual),
         rows, width, ctypes.c_float(eps), _stream())
    return out


def fused_rms_norm_gated_residual_norm_scale(be, policy, residual, branch, gate, scale, branch_eps=1e-6, eps=1e-6, gate_tanh=True,
                                             state_out=None, out=None):
    """The Mochi block's residual update and the next layer's pre-norm in one pass (mochi.cpp:204-211, :228-231):
        state = gated_residual(residual, rms_norm(branch, None, branch_eps), tanh(gate) if gate_tanh else gate)
        out   = mul(rms_norm(state, None, eps), add(1, scale))
    Returns (state, out).  Other contracts than an all-bf16 stream run tanh, the residual update and the
    norm as separate launches."""
    residual, branch = _dense(residual), _dense(branch)
    width = residual.shape[-1]
    rows = residual.numel() // width
    grpv, gvec = _vec_layout(rows, residual.shape, gate)
    rpv, nvec = _vec_layout(rows, residual.shape, scale)
    state = _result(state_out, residual.shape, policy.residual, residual.device)
    one_pass = residual.dtype == BF16 and branch.dtype == BF16 and policy.residual == BF16
    if gate_tanh and not one_pass:
        gate, gate_tanh = be.activation(gate, TANH), False
    out = _result(out, residual.shape, policy.residual, residual.device)
    call("vrb_rms_norm_gated_residual_rms_norm_scale", _ptr(residual), _code(residual), _ptr(branch), _code(branch),
         ctypes.c_float(branch_eps), _ptr(_dense(gate)), _code(gate), int(bool(gate_tanh)), grpv, gvec, _ptr(state),
         _code(policy.residual), _ptr(_dense(scale)), _code(scale), rpv, nvec, _ptr(out), rows, width, ctypes.c_float(eps), _stream())
    return state, out


def fused_swiglu(be, projected, out=None):
    """mul(parts[0], silu(parts[1])) with parts = split(projected, 2, -1) -- mochi.cpp:195-202."""
    projected = _dense(projected)
    hidden = projected.shape[-1] // 2
    rows = projected.numel() // (2 * hidden)
    out = _result(out, projected.shape[:-1] + (hidden,), projected.dtype, projected.device)
    call("vrb_swiglu", _ptr(projected), _ptr(out), _code(projected), rows, hidden, _stream())
    return out


def fused_pixel_norm_modulate(be, x, shift, scale, eps=1e-8, silu=True, out_dtype=F32, out=None):
    """[silu](modulate(pixel_norm(x, 1, eps), shift, scale)) for x [B, C, ...] and shift / scale
    [B, C, 1, ...] -- the head of LTX's decoder_residual (native/src/architectures/ltx.cpp:221-227) in one
    pass.  out_dtype F32 is modulate's contract output; BF16 also folds the consumer's operand cast."""
    x = _dense(x)
    channels, inner = x.shape[1], 1
    for d in x.shape[2:]:
        inner *= d
    if shift.dtype != scale.dtype or shift.numel() != x.shape[0] * channels or scale.numel() != shift.numel():
        raise VrbError("Incompatible broadcast shapes")
    out = _result(out, x.shape, out_dtype, x.device)
    call("vrb_pixel_norm", _ptr(x), _code(x), _ptr(_dense(scale)), _ptr(_dense(shift)), _code(scale), int(bool(silu)),
         _ptr(out), _code(out_dtype), x.shape[0], channels, inner, ctypes.c_float(eps), _stream())
    return out


def fused_edge_time_pad(be, x, temporal, pad_h, pad_w, out=None):
    """The two pads in front of every LTX convolution (edge_time_conv, native/src/architectures/ltx.cpp:205-215) in one
    pass: replicate `temporal` frames at both ends of T, then zeros around H and W, on x [B, C, T, H, W]."""
    return be.pad_axes(x, [0, 0, temporal, pad_h, pad_w], [0, 0, temporal, pad_h, pad_w], 0.0, [False, False, True, False, False], out=out)


def fused_depth_to_space_residual(be, projected, x, out=None):
    """LTX depth_to_space (native/src/architectures/ltx.cpp:250-259) after its convolution: projected
    [B, 4C, T, H, W] is the convolution output, x [B, C, T, H, W] the block input; returns
    pixel_shuffle(projected)[:, :, 1:] + repeat4(pixel_shuffle(x))[:, :, 1:] as [B, C/2, 2T-1, 2H, 2W]."""
    projected, x = _dense(projected), _dense(x)
    b, c, t, h, w = x.shape
    if projected.dtype != x.dtype or tuple(projected.shape) != (b, 4 * c, t, h, w):
        raise VrbError("Incompatible broadcast shapes")
    out = _result(out, (b, c // 2, 2 * t - 1, 2 * h, 2 * w), x.dtype, x.device)
    call("vrb_depth_to_space_residual", _ptr(projected), _ptr(x), _ptr(out), _code(x), b, c, t, h, w, _stream())
    return out


def _linear_operands(accumulation, bias):
    accumulation = _dense(accumulation)
    if accumulation.dtype != F32:
        raise VrbError("linear_output: the accumulation must be F32")
    if bias is not None:
        bias = _dense(bias)
        if bias.dtype != BF16 or bias.numel() != accumulation.shape[-1]:
            raise VrbError("linear bias mismatch")
    width = accumulation.shape[-1]
    return accumulation, bias, accumulation.numel() // width, width


def linear_output(be, accumulation, bias, out=None):
    """The epilogue of the reference's bf16 linear (fused_bf16_linear_output_kernel,
    native/src/backend/cuda/cuda_backend.cu:754-764): bf16(accumulation + float(bias))."""
    accumulation, bias, rows, width = _linear_operands(accumulation, bias)
    out = _result(out, accumulation.shape, BF16, accumulation.device)
    call("vrb_linear_output", _ptr(accumulation), _ptr(bias), _ptr(out), rows, width, _stream())
    return out


def linear_output_activation(be, accumulation, bias, kind, out=None):
    """activation(linear_output(accumulation, bias), kind) without writing the linear output
    (wan.cpp:109-112)."""
    accumulation, bias, rows, width = _linear_operands(accumulation, bias)
    out = _result(out, accumulation.shape, BF16, accumulation.device)
    call("vrb_linear_output_activation", _ptr(accumulation), _ptr(bias), int(kind), _ptr(out), rows, width, _stream())
    return out


def linear_output_gated_residual(be, policy, residual, accumulation, bias, gate, out=None):
    """gated_residual(residual, linear_output(accumulation, bias), gate) (residual_add when gate is
    None) without writing the linear output (wan.cpp:99-103, 114-116)."""
    accumulation, bias, rows, width = _linear_operands(accumulation, bias)
    residual = _dense(residual)
    if tuple(residual.shape) != tuple(accumulation.shape):
        raise VrbError("Incompatible broadcast shapes")
    rpv, nvec = (1, 1) if gate is None else _vec_layout(rows, residual.shape, gate)
    out = _result(out, residual.shape, policy.residual, residual.device)
    call("vrb_linear_output_gated_residual", _ptr(accumulation), _ptr(bias), _ptr(residual), _code(residual),
         _ptr(_dense(gate)) if gate is not None else None, _code(gate) if gate is not None else 0, rpv, nvec, _ptr(out),
         _code(policy.residual), rows, width, _stream())
    return out


def linear_output_swiglu(be, accumulation, bias, out=None):
    """fused_swiglu(linear_output(accumulation, bias)) without writing the linear output
    (mochi.cpp:195-202)."""
    accumulation, bias, rows, width = _linear_operands(accumulation, bias)
    if width % 2:
        raise VrbError("split sections mismatch")
    out = _result(out, accumulation.shape[:-1] + (width // 2,), BF16, accumulation.device)
    call("vrb_linear_output_swiglu", _ptr(accumulation), _ptr(bias), _ptr(out), rows, width // 2, _stream())
    return out


def fused_cfg_combine(be, policy, unconditional, conditional, scale, out=None):
    out = _result(out, unconditional.shape, unconditional.dtype, unconditional.device)
    call("vrb_cfg_combine", _ptr(_dense(unconditional)), _ptr(_dense(conditional)), _ptr(out), _code(out),
         out.numel(), ctypes.c_float(scale), int(GUIDANCE in policy.scalar_roles), _stream())
    return out


def fused_euler_update(be, policy, sample, prediction, delta, subtract_prediction, out=None):
    out = _result(out, sample.shape, sample.dtype, sample.device)
    k = _euler_delta(be, policy, delta)
    call("vrb_euler_update", _ptr(_dense(sample)), _ptr(_dense(prediction)), _ptr(out), _code(out), out.numel(),
         ctypes.c_float(k), int(subtract_prediction), int(SOLVER in policy.scalar_roles), _stream())
    return out


def linear_combine(be, policy, values, coefficients, role=GUIDANCE):
    """SamplingPrimitives::linear_combine (native/src/sampling/sampling.cpp:173-179) operator by operator."""
    result = precision_scalar_binary(be, policy, role, values[0], coefficients[0])
    for v, c in zip(values[1:], coefficients[1:]):
        result = be.add(result, precision_scalar_binary(be, policy, role, v, c))
    return result


def fused_linear_combine(be, policy, values, coefficients, role=GUIDANCE, out=None):
    """linear_combine / v_to_x0 / affine_first_order (sampling.cpp:173-179, 204-214, 229-239) in one pass,
    1..4 terms of one shape and dtype."""
    if not values or len(values) != len(coefficients) or len(values) > 4:
        raise VrbError("linear combine arity mismatch")
    first = _dense(values[0])
    for v in values:
        if v.dtype != first.dtype or tuple(v.shape) != tuple(first.shape):
            raise VrbError("Incompatible broadcast shapes")
    out = _result(out, first.shape, first.dtype, first.device)
    pointers = (ctypes.c_void_p * len(values))(*[_dense(v).data_ptr() for v in values])
    coefs = (ctypes.c_float * len(values))(*[float(c) for c in coefficients])
    call("vrb_linear_combine", ctypes.cast(pointers, ctypes.c_void_p), ctypes.cast(coefs, ctypes.c_void_p), len(values),
         _ptr(out), _code(out), out.numel(), int(role in policy.scalar_roles), _stream())
    return out


def fused_flow_to_x0(be, policy, sample, model_output, sigma):
    out = torch.empty_like(sample)
    call("vrb_flow_to_x0", _ptr(_dense(sample)), _ptr(_dense(model_output)), _ptr(out), _code(out), out.numel(),
         ctypes.c_float(sigma), int(SIGMA in policy.scalar_roles), _stream())
    return out


def fused_cfg_euler(be, policy, sample, unconditional, conditional, scale, delta, subtract_prediction=True,
                    want_guided=False, out=None):
    """euler_update(sample, cfg_combine(u, c, scale), delta, subtract) in one pass."""
    out = _result(out, sample.shape, sample.dtype, sample.device)
    guided = torch.empty_like(sample) if want_guided else None
    k = _euler_delta(be, policy, delta)
    call("vrb_cfg_euler", _ptr(_dense(sample)), _ptr(_dense(unconditional)), _ptr(_dense(conditional)), _ptr(guided),
         _ptr(out), _code(out), out.numel(), ctypes.c_float(scale), ctypes.c_float(k), int(subtract_prediction),
         int(GUIDANCE in policy.scalar_roles), int(SOLVER in policy.scalar_roles), _stream())
    return (out, guided) if want_guided else out


def fused_group_norm_silu(be, x, groups, weight, bias, eps, out=None):
    """activation(group_norm(x, ...), Silu) -- native/src/components/autoencoder_kl.cpp:40-41."""
    return be.group_norm(x, groups, weight, bias, eps, fuse_silu=True, out=out)


def fused_rms_channel_silu(be, x, gamma, eps=1e-12):
    """silu(rms_norm(x, gamma, eps, axis=1)) -- native/src/components/executor.cpp:90-98 as the Wan VAE uses it."""
    x = _dense(x)
    axis = x.shape[1]
    inner = x.numel() // (x.shape[0] * axis)
    out = torch.empty_like(x)
    call("vrb_rms_norm_axis", _ptr(x), _code(x), _ptr(gamma), _code(gamma), _ptr(out), x.shape[0], axis, inner,
         ctypes.c_float(eps), 1, _stream())
    return out
