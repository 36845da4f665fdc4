"""ctypes front-ends of the two libraries built from the REFERENCE's own sources by
``oracle/Makefile`` (``make -C oracle ref``): ``_ref/libvrhino_ref_host.so`` (the reference's
F32 host test backend + helper seams) and ``_ref/libvrhino_ref_cuda.so`` (the reference's CUDA
backend compiled for sm_100a).

TEST / BASELINE INFRASTRUCTURE ONLY: used to validate the oracle, to generate the golden
vectors under ``tests/golden/`` and to time baselines.  ``available_*()`` say whether the
libraries exist; nothing here reads the reference tree at run time.
"""
from __future__ import annotations

import ctypes
import os

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
HOST_LIB = os.path.join(_HERE, "_ref", "libvrhino_ref_host.so")
CUDA_LIB = os.path.join(_HERE, "_ref", "libvrhino_ref_cuda.so")
DROPIN_LIB = os.path.join(_HERE, "_ref", "libvrhino_dropin_cuda.so")
_c = ctypes
_fp = _c.POINTER(_c.c_float)
F32, BF16, U8 = 0, 2, 5
POLICY_BF16, POLICY_FP32, POLICY_BF16_ROLES, POLICY_BF16_GUIDANCE = 0, 1, 2, 3


def reference_tree() -> str:
    """The reference checkout's native/ directory: $VRHINO_REF, else a `reference` checkout beside this
    repository.  Only the build recipes read it (oracle/Makefile); nothing does at run time."""
    return os.environ.get("VRHINO_REF") or os.path.join(os.path.dirname(os.path.dirname(_HERE)), "reference", "native")


def available_host() -> bool:
    return os.path.exists(HOST_LIB)


def available_cuda() -> bool:
    return os.path.exists(CUDA_LIB)


def available_dropin() -> bool:
    return os.path.exists(DROPIN_LIB)


def _f(a):
    return np.ascontiguousarray(a, dtype=np.float32)


def _ptr(a):
    return None if a is None else a.ctypes.data_as(_fp)


class RefHost:
    """The reference's host path (F32, family_test::Backend)."""

    def __init__(self):
        self.lib = ctypes.CDLL(HOST_LIB)
        self.lib.refh_last_error.restype = _c.c_char_p
        self.lib.refh_wan_chain_seconds.restype = _c.c_double

    def _check(self, rc):
        if rc != 0:
            raise RuntimeError(self.lib.refh_last_error().decode())

    def layer_norm(self, x, w, b, eps):
        x = _f(x); out = np.empty_like(x)
        w = None if w is None else _f(w); b = None if b is None else _f(b)
        self._check(self.lib.refh_layer_norm(_ptr(x), _ptr(w), _ptr(b), _ptr(out), _c.c_int64(x.size // x.shape[-1]),
                                             _c.c_int64(x.shape[-1]), _c.c_float(eps)))
        return out

    def rms_norm(self, x, w, eps):
        x = _f(x); out = np.empty_like(x); w = None if w is None else _f(w)
        self._check(self.lib.refh_rms_norm(_ptr(x), _ptr(w), _ptr(out), _c.c_int64(x.size // x.shape[-1]),
                                           _c.c_int64(x.shape[-1]), _c.c_float(eps)))
        return out

    def activation(self, x, kind):
        x = _f(x); out = np.empty_like(x)
        self._check(self.lib.refh_activation(_ptr(x), _ptr(out), _c.c_int64(x.size), int(kind)))
        return out

    def rope(self, x, c, s):
        x, c, s = _f(x), _f(c), _f(s); out = np.empty_like(x)
        _, tokens, heads, width = x.shape
        self._check(self.lib.refh_rope(_ptr(x), _ptr(c), _ptr(s), _ptr(out), _c.c_int64(tokens), _c.c_int64(heads), _c.c_int64(width)))
        return out

    def modulate(self, x, shift, scale):
        x, shift, scale = _f(x), _f(shift), _f(scale); out = np.empty_like(x)
        self._check(self.lib.refh_modulate(_ptr(x), _ptr(shift), _ptr(scale), _ptr(out), _c.c_int64(x.size // x.shape[-1]),
                                           _c.c_int64(x.shape[-1])))
        return out

    def gated_residual(self, res, branch, gate):
        res, branch = _f(res), _f(branch); out = np.empty_like(res)
        gate = None if gate is None else _f(gate)
        self._check(self.lib.refh_gated_residual(_ptr(res), _ptr(branch), _ptr(gate), _ptr(out),
                                                 _c.c_int64(res.size // res.shape[-1]), _c.c_int64(res.shape[-1])))
        return out

    @staticmethod
    def _i64(values):
        return (_c.c_int64 * max(len(values), 1))(*[int(v) for v in values])

    def permute(self, x, axes):
        x = _f(x); out = np.empty([x.shape[a] for a in axes], dtype=np.float32)
        self._check(self.lib.refh_permute(_ptr(x), x.ndim, self._i64(x.shape), self._i64(axes), _ptr(out)))
        return out

    def slice(self, x, axis, start, stop):
        """The host backend takes the range as it is (no negative indices, no clamping)."""
        x = _f(x); shape = list(x.shape); shape[axis] = stop - start
        out = np.empty(shape, dtype=np.float32)
        self._check(self.lib.refh_slice(_ptr(x), x.ndim, self._i64(x.shape), _c.c_int64(axis), _c.c_int64(start), _c.c_int64(stop), _ptr(out)))
        return out

    def sinusoidal_embedding(self, positions, width, flip, shift):
        """The host backend always computes the phase in double; it has no zero column for an odd width."""
        positions = _f(positions); out = np.zeros((positions.size, width), dtype=np.float32)
        self._check(self.lib.refh_sinusoidal(_ptr(positions), _c.c_int64(positions.size), _c.c_int64(width), int(bool(flip)),
                                             _c.c_double(shift), _ptr(out)))
        return out

    def pad_rows(self, x, after, value):
        x = _f(x); out = np.empty((x.shape[0] + after, x.shape[1]), dtype=np.float32)
        self._check(self.lib.refh_pad_rows(_ptr(x), _c.c_int64(x.shape[0]), _c.c_int64(x.shape[1]), _c.c_int64(after), _c.c_float(value),
                                           _ptr(out)))
        return out

    def cfg_euler(self, x, u, c, scale, delta):
        x, u, c = _f(x), _f(u), _f(c)
        guided, out = np.empty_like(x), np.empty_like(x)
        self._check(self.lib.refh_cfg_euler(_ptr(x), _ptr(u), _ptr(c), _ptr(guided), _ptr(out), _c.c_int64(x.size),
                                            _c.c_float(scale), _c.c_float(delta)))
        return guided, out

    def fusion_plan(self, which, contract, diagnostics=False, tokens=64):
        """Chains vrhino_b200::plan_fusion finds in the reference's production graphs.  which: "wan" |
        "ltx"; contract: "f32" | "bf16_f32_hidden" | "bf16".  Returns a dict of counts."""
        out = (_c.c_int * 6)()
        rc = self.lib.refh_fusion_plan({"wan": 0, "ltx": 1}[which], {"f32": 0, "bf16_f32_hidden": 1, "bf16": 2}[contract],
                                       int(diagnostics), _c.c_int64(tokens), out)
        if rc != 0:
            raise RuntimeError(self.lib.refh_last_error().decode())
        keys = ("layer_norm_modulate", "rms_norm_modulate", "rms_norm_rope", "gated_residual", "nodes_total", "nodes_absorbed")
        return dict(zip(keys, out))

    CODES = ("UnsupportedSchema", "UnsupportedPrimitive", "InvalidOperation", "LimitExceeded", "InvalidShape", "InvalidDType",
             "InvalidValue", "InvalidDependency", "InvalidInputBinding", "InvalidParameterBinding", "InvalidContext",
             "BackendFailure", "InvalidNodeOutput", "CompletionFailure", "InvalidOutput")
    PHASES = ("Admit", "Bind", "Run", "Drain", "Capture")

    def fused_faults(self, scenario, tokens=4, n=0):
        """vrhino_b200::evaluate_fused under a failure injected on the host (see refh_fused_faults in
        ref_host.cpp).  Returns a dict: threw, code, phase, node, value, primitive, syncs,
        secondary_completion, calls, outputs, text."""
        report = (_c.c_int64 * 10)()
        if self.lib.refh_fused_faults(int(scenario), _c.c_int64(tokens), int(n), report) != 0:
            raise RuntimeError(self.lib.refh_last_error().decode())
        r = list(report)
        loc = lambda v: None if v < 0 else v
        return {"threw": bool(r[0]), "code": self.CODES[r[1]] if r[0] else None, "phase": self.PHASES[r[2]] if r[0] else None,
                "node": loc(r[3]), "value": loc(r[4]), "primitive": loc(r[5]), "syncs": r[6], "secondary_completion": bool(r[7]),
                "calls": r[8], "outputs": r[9], "text": self.lib.refh_last_error().decode() if r[0] else ""}

    def wan_chain_seconds(self, tokens, threads, steps, dim=1536, heads=12, ffn=8960, text=512, seed=0):
        """Seconds per step of the Wan block chain on `tokens` rows, and its algorithmic bytes
        (same accounting as the GPU arm, bf16-hidden contract, so the GB/s are comparable)."""
        rng = np.random.default_rng(seed)
        text = min(text, tokens)
        t = lambda *shape: rng.standard_normal(shape, dtype=np.float32)
        x, q, k, proj, cq, cr, fo = (t(tokens, dim) for _ in range(7))
        ck, fh, mod = t(text, dim), t(tokens, ffn), t(6, dim) * 0.1
        ws = [1 + 0.1 * t(dim) for _ in range(5)]
        beta = 0.1 * t(dim)
        ph = rng.uniform(-3, 3, size=(tokens, dim // heads)).astype(np.float32)
        co, si = np.cos(ph), np.sin(ph)
        sec = self.lib.refh_wan_chain_seconds(
            _ptr(x), _ptr(q), _ptr(k), _ptr(proj), _ptr(cq), _ptr(ck), _ptr(cr), _ptr(fo), _ptr(fh), _ptr(mod),
            _ptr(ws[0]), _ptr(ws[1]), _ptr(ws[2]), _ptr(ws[3]), _ptr(ws[4]), _ptr(beta), _ptr(co), _ptr(si),
            _c.c_int64(tokens), _c.c_int64(text), _c.c_int64(dim), _c.c_int64(heads), _c.c_int64(ffn), int(threads), int(steps))
        if sec < 0:
            raise RuntimeError(self.lib.refh_last_error().decode())
        act, vec, table = tokens * dim, dim * 4, tokens * (dim // heads) * 4
        nbytes = (3 * (act * 4 + 2 * vec) + 2 * (act * 4 + vec + table) + 3 * (act * 6) + 2 * vec + (act * 4 + vec)
                  + (text * dim * 4 + vec) + tokens * ffn * 4)
        return sec, nbytes


class RefCuda:
    """The reference's CUDA backend; tensors are handles kept on the device between calls."""

    LIB = CUDA_LIB

    def __init__(self, execution_dtype=BF16):
        lib = ctypes.CDLL(self.LIB)
        lib.refc_last_error.restype = _c.c_char_p
        lib.refc_backend_name.restype = _c.c_char_p
        for name in ("refc_upload", "refc_host_f32", "refc_numel", "refc_binary", "refc_cast", "refc_reshape", "refc_slice",
                     "refc_layer_norm", "refc_rms_norm", "refc_activation", "refc_rope", "refc_group_norm", "refc_clamp",
                     "refc_exp", "refc_sqrt", "refc_dequantize", "refc_modulate", "refc_attention_norm", "refc_operation_rope",
                     "refc_residual_add", "refc_gated_residual", "refc_cfg_combine", "refc_euler_update", "refc_flow_to_x0",
                     "refc_frame_group_norm", "refc_linear", "refc_pixel_norm", "refc_pixel_shuffle", "refc_repeat",
                     "refc_l2_normalize", "refc_permute", "refc_concat", "refc_pad", "refc_sinusoidal", "refc_interpolate_nearest", "refc_reduce_sum",
                     "refc_softmax", "refc_indexed_gather", "refc_rng_normal"):
            getattr(lib, name).restype = _c.c_int64
        lib.refc_profile_total_ms.restype = _c.c_double
        self.lib = lib
        if lib.refc_init(int(execution_dtype)) != 0:
            raise RuntimeError(lib.refc_last_error().decode())

    def _h(self, h):
        if h < 0:
            raise RuntimeError(self.lib.refc_last_error().decode())
        return h

    @staticmethod
    def _shape(shape):
        return (_c.c_int64 * max(len(shape), 1))(*shape), len(shape)

    def upload(self, array: np.ndarray, dtype: int):
        """array: float32 payload for F32, uint16 bits for BF16, uint8 for U8."""
        a = np.ascontiguousarray(array)
        s, r = self._shape(a.shape)
        return self._h(self.lib.refc_upload(_c.c_void_p(a.ctypes.data), int(dtype), r, s))

    def host_f32(self, array):
        a = _f(array)
        s, r = self._shape(a.shape)
        return self._h(self.lib.refc_host_f32(_ptr(a), r, s))

    def download(self, h, shape):
        dt = self.lib.refc_dtype(_c.c_int64(h))
        np_dt = {F32: np.float32, BF16: np.uint16, U8: np.uint8}[dt]
        out = np.empty(shape, dtype=np_dt)
        if self.lib.refc_download(_c.c_int64(h), _c.c_void_p(out.ctypes.data), _c.c_int64(out.nbytes)) != 0:
            raise RuntimeError(self.lib.refc_last_error().decode())
        return out, dt

    def free(self, h): self.lib.refc_free(_c.c_int64(h))
    def clear(self): self.lib.refc_clear()
    def synchronize(self): self.lib.refc_synchronize()

    def _i(self, h): return _c.c_int64(h or 0)

    def binary(self, kind, a, b): return self._h(self.lib.refc_binary(int(kind), self._i(a), self._i(b)))
    def cast(self, x, dtype): return self._h(self.lib.refc_cast(self._i(x), int(dtype)))
    def reshape(self, x, shape):
        s, r = self._shape(shape)
        return self._h(self.lib.refc_reshape(self._i(x), r, s))
    def slice(self, x, dim, start, stop): return self._h(self.lib.refc_slice(self._i(x), _c.c_int64(dim), _c.c_int64(start), _c.c_int64(stop)))
    def layer_norm(self, x, w, b, eps): return self._h(self.lib.refc_layer_norm(self._i(x), self._i(w), self._i(b), _c.c_float(eps)))
    def rms_norm(self, x, w, eps, axis=-1, out_dtype=-1):
        return self._h(self.lib.refc_rms_norm(self._i(x), self._i(w), _c.c_float(eps), _c.c_int64(axis), int(out_dtype)))
    def linear(self, x, w, bias): return self._h(self.lib.refc_linear(self._i(x), self._i(w), self._i(bias)))
    def pixel_norm(self, x, dim, eps): return self._h(self.lib.refc_pixel_norm(self._i(x), _c.c_int64(dim), _c.c_float(eps)))
    def l2_normalize(self, x, dim, eps): return self._h(self.lib.refc_l2_normalize(self._i(x), _c.c_int64(dim), _c.c_float(eps)))
    def pixel_shuffle(self, x, factors):
        return self._h(self.lib.refc_pixel_shuffle(self._i(x), *(_c.c_int64(int(f)) for f in factors)))
    def permute(self, x, dims):
        d, r = self._shape(tuple(int(v) for v in dims))
        return self._h(self.lib.refc_permute(self._i(x), r, d))
    def concat(self, handles, dim):
        h = (_c.c_int64 * len(handles))(*[int(v) for v in handles])
        return self._h(self.lib.refc_concat(h, len(handles), _c.c_int64(dim)))
    def pad(self, x, padding, value=0.0, replicate=False):
        p = (_c.c_int64 * max(len(padding), 1))(*[int(v) for v in padding])
        return self._h(self.lib.refc_pad(self._i(x), len(padding), p, _c.c_float(value), int(bool(replicate))))
    def reduce_sum(self, x, dim, keepdim=False):
        return self._h(self.lib.refc_reduce_sum(self._i(x), _c.c_int64(dim), int(bool(keepdim))))
    def rng_normal(self, seed, offset, shape, dtype):
        s, r = self._shape(tuple(int(v) for v in shape))
        return self._h(self.lib.refc_rng_normal(_c.c_uint64(seed), _c.c_uint64(offset), r, s, int(dtype)))
    def softmax(self, x, axis): return self._h(self.lib.refc_softmax(self._i(x), _c.c_int64(axis)))
    def indexed_gather(self, table, indices):
        import numpy as np
        indices = np.ascontiguousarray(indices)
        shape, rank = self._shape(tuple(int(v) for v in indices.shape))
        return self._h(self.lib.refc_indexed_gather(self._i(table), 64 if indices.dtype == np.int64 else 32, rank, shape,
                                                    indices.ctypes.data_as(_c.c_void_p)))
    def interpolate_nearest(self, x, factors):
        f = (_c.c_double * max(len(factors), 1))(*[float(v) for v in factors])
        return self._h(self.lib.refc_interpolate_nearest(self._i(x), len(factors), f))
    def sinusoidal_embedding(self, positions, width, flip, downscale, frequency_f64):
        return self._h(self.lib.refc_sinusoidal(self._i(positions), _c.c_int64(width), int(bool(flip)), _c.c_double(downscale),
                                                int(bool(frequency_f64))))
    def repeat(self, x, copies, dim): return self._h(self.lib.refc_repeat(self._i(x), int(copies), _c.c_int64(dim)))
    def activation(self, x, kind): return self._h(self.lib.refc_activation(self._i(x), int(kind)))
    def rope(self, x, c, s): return self._h(self.lib.refc_rope(self._i(x), self._i(c), self._i(s)))
    def group_norm(self, x, groups, w, b, eps): return self._h(self.lib.refc_group_norm(self._i(x), int(groups), self._i(w), self._i(b), _c.c_float(eps)))
    def clamp(self, x, lo, hi): return self._h(self.lib.refc_clamp(self._i(x), _c.c_float(lo), _c.c_float(hi)))
    def exp(self, x): return self._h(self.lib.refc_exp(self._i(x)))
    def sqrt(self, x): return self._h(self.lib.refc_sqrt(self._i(x)))
    def dequantize(self, kind, packed, scales, rows, inner, group_size, out_dtype):
        p = np.ascontiguousarray(packed, dtype=np.uint8); s = _f(scales)
        return self._h(self.lib.refc_dequantize(int(kind), _c.c_void_p(p.ctypes.data), _c.c_int64(p.nbytes), _ptr(s),
                                                _c.c_int64(rows), _c.c_int64(inner), _c.c_int64(group_size), int(out_dtype)))
    def modulate(self, policy, x, shift, scale): return self._h(self.lib.refc_modulate(int(policy), self._i(x), self._i(shift), self._i(scale)))
    def attention_norm(self, policy, x, w, eps, axis=-1):
        return self._h(self.lib.refc_attention_norm(int(policy), self._i(x), self._i(w), _c.c_float(eps), _c.c_int64(axis)))
    def operation_rope(self, policy, x, c, s): return self._h(self.lib.refc_operation_rope(int(policy), self._i(x), self._i(c), self._i(s)))
    def residual_add(self, policy, r, b): return self._h(self.lib.refc_residual_add(int(policy), self._i(r), self._i(b)))
    def gated_residual(self, policy, r, b, g): return self._h(self.lib.refc_gated_residual(int(policy), self._i(r), self._i(b), self._i(g)))
    def cfg_combine(self, policy, u, c, scale): return self._h(self.lib.refc_cfg_combine(int(policy), self._i(u), self._i(c), _c.c_float(scale)))
    def euler_update(self, policy, x, pred, delta, subtract=True):
        return self._h(self.lib.refc_euler_update(int(policy), self._i(x), self._i(pred), _c.c_float(delta), int(subtract)))
    def flow_to_x0(self, policy, x, out, sigma): return self._h(self.lib.refc_flow_to_x0(int(policy), self._i(x), self._i(out), _c.c_float(sigma)))

    def frame_group_norm(self, x, groups, w, b, eps, silu=False):
        return self._h(self.lib.refc_frame_group_norm(self._i(x), int(groups), self._i(w), self._i(b), _c.c_float(eps), int(silu)))

    def wan_self_attention_graph(self, tokens, width, heads, handles, fused=False):
        """The reference's production Wan self-attention graph (GEMMs and attention included).
        handles: hidden, modulation, cos, sin + the 11 canonical parameters.  Returns
        ([first residual, combined modulation], stats)."""
        h = (_c.c_int64 * 15)(*handles)
        out = (_c.c_int64 * 2)()
        stats = (_c.c_int * 5)()
        rc = self.lib.refc_wan_self_attention_graph(_c.c_int64(tokens), _c.c_int64(width), _c.c_int64(heads), h, int(fused), out, stats)
        if rc != 0:
            raise RuntimeError(self.lib.refc_last_error().decode())
        return list(out), list(stats)

    def ltx_self_attention_graph(self, batch, tokens, hidden_bf16, handles, fused=False):
        """The reference's production LTX self-attention graph (BF16 execution).  handles: hidden,
        modulation, cos, sin + 11 parameters.  Returns (first residual handle, stats)."""
        h = (_c.c_int64 * 15)(*handles)
        out = (_c.c_int64 * 1)()
        stats = (_c.c_int * 5)()
        rc = self.lib.refc_ltx_self_attention_graph(_c.c_int64(batch), _c.c_int64(tokens), int(hidden_bf16), h, int(fused), out, stats)
        if rc != 0:
            raise RuntimeError(self.lib.refc_last_error().decode())
        return out[0], list(stats)

    def wan_chain_graph(self, tokens, width, heads, hidden_dtype, eps, handles, fused=False):
        """Evaluates the non-GEMM part of the Wan self-attention graph (built node for node in
        ref_cuda.cpp) through neural_graph::evaluate, or -- drop-in build, fused=True -- through
        vrhino_b200::evaluate_fused (fused=2: without its per-graph synchronisation).  handles: hidden, modulation, cos, sin, q, k, projection,
        table, norm_q, norm_k.  Returns ([attention input, q operand, k operand, residual], stats)."""
        h = (_c.c_int64 * 10)(*handles)
        out = (_c.c_int64 * 4)()
        stats = (_c.c_int * 5)()
        rc = self.lib.refc_wan_chain_graph(_c.c_int64(tokens), _c.c_int64(width), _c.c_int64(heads), int(hidden_dtype),
                                           _c.c_float(eps), h, int(fused), out, stats)
        if rc != 0:
            raise RuntimeError(self.lib.refc_last_error().decode())
        return list(out), list(stats)


class RefDropin(RefCuda):
    """The same call surface over vrhino_b200::B200Backend (this repository's C++ host layer and
    kernels) wrapped around the reference's CudaBackend: the reference's unmodified helper code
    runs on the replaced operators.  The fused_* methods reach the one-kernel forms."""
    LIB = DROPIN_LIB

    def __init__(self, execution_dtype=BF16):
        super().__init__(execution_dtype)
        for name in ("refd_layer_norm_modulate", "refd_rms_norm_rope", "refd_gated_residual", "refd_swiglu",
                     "refd_group_norm_silu", "refd_cfg_euler", "refd_gated_residual_layer_norm",
                     "refd_linear_activation", "refd_linear_gated_residual", "refd_linear_swiglu",
                     "refd_pixel_norm_modulate_silu", "refd_depth_to_space_residual", "refd_profile_report",
                     "refd_dequantize_repeated", "refd_release_cached", "refd_rms_norm_rope_pair", "refd_mochi_residual_norm", "refd_edge_time_pad"):
            getattr(self.lib, name).restype = _c.c_int64

    def profile(self, enabled): self.lib.refc_profile(int(enabled))
    def profile_report(self):
        """{name: (calls, device ms, bytes moved)} of the wrapped backend's profile_stats()."""
        buf = _c.create_string_buffer(1 << 20)
        self._h(self.lib.refd_profile_report(buf, _c.c_int64(len(buf))))
        out = {}
        for line in buf.value.decode().splitlines():
            name, calls, ms, nbytes = line.split("\t")
            out[name] = (int(calls), float(ms), int(nbytes))
        return out
    def dequantize_repeated(self, kind, packed, scales, rows, inner, group_size, out_dtype, repeats, budget=-1):
        """(handle of the last result, {hits, misses, resident_bytes})"""
        p = np.ascontiguousarray(packed, dtype=np.uint8); s = _f(scales)
        stats = (_c.c_int64 * 3)()
        h = self._h(self.lib.refd_dequantize_repeated(int(kind), _c.c_void_p(p.ctypes.data), _c.c_int64(p.nbytes), _ptr(s),
                                                      _c.c_int64(rows), _c.c_int64(inner), _c.c_int64(group_size), int(out_dtype),
                                                      int(repeats), _c.c_int64(budget), stats))
        return h, {"hits": stats[0], "misses": stats[1], "resident_bytes": stats[2]}
    def release_cached(self): return self._h(self.lib.refd_release_cached())

    def name(self): return self.lib.refc_backend_name().decode()
    def session_terminal(self): return bool(self.lib.refd_session_terminal())
    def fused_layer_norm_modulate(self, policy, x, w, b, eps, shift, scale, out_dtype=BF16):
        return self._h(self.lib.refd_layer_norm_modulate(int(policy), self._i(x), self._i(w), self._i(b), _c.c_float(eps),
                                                         self._i(shift), self._i(scale), int(out_dtype)))
    def fused_rms_norm_rope(self, policy, x, w, eps, c, s, heads, per_head=False, out_dtype=BF16):
        return self._h(self.lib.refd_rms_norm_rope(int(policy), self._i(x), self._i(w), _c.c_float(eps), self._i(c), self._i(s),
                                                   int(heads), int(per_head), int(out_dtype)))
    def fused_rms_norm_rope_pair(self, policy, q, wq, k, wk, eps, c, s, heads, per_head=False, out_dtype=BF16):
        second = _c.c_int64(0)
        first = self._h(self.lib.refd_rms_norm_rope_pair(int(policy), self._i(q), self._i(wq), self._i(k), self._i(wk), _c.c_float(eps),
                                                         self._i(c), self._i(s), int(heads), int(per_head), int(out_dtype),
                                                         _c.byref(second)))
        return first, second.value
    def fused_mochi_residual_norm(self, policy, r, b, g, scale, eps=1e-6):
        """(updated stream handle, next pre-norm handle)"""
        normed = _c.c_int64(0)
        state = self._h(self.lib.refd_mochi_residual_norm(int(policy), self._i(r), self._i(b), self._i(g), self._i(scale),
                                                          _c.c_float(eps), _c.byref(normed)))
        return state, normed.value
    def fused_gated_residual(self, policy, r, b, g): return self._h(self.lib.refd_gated_residual(int(policy), self._i(r), self._i(b), self._i(g)))
    def fused_gated_residual_layer_norm(self, policy, r, b, g, w, bias, eps, shift, scale, out_dtype=BF16):
        """(state handle, normalised handle)"""
        state = _c.c_int64(0)
        normed = self._h(self.lib.refd_gated_residual_layer_norm(int(policy), self._i(r), self._i(b), self._i(g), self._i(w),
                                                                 self._i(bias), _c.c_float(eps), self._i(shift), self._i(scale),
                                                                 int(out_dtype), _c.byref(state)))
        return state.value, normed
    def fused_linear_activation(self, x, w, bias, kind):
        return self._h(self.lib.refd_linear_activation(self._i(x), self._i(w), self._i(bias), int(kind)))
    def fused_linear_gated_residual(self, policy, r, x, w, bias, g):
        return self._h(self.lib.refd_linear_gated_residual(int(policy), self._i(r), self._i(x), self._i(w), self._i(bias), self._i(g)))
    def fused_linear_swiglu(self, x, w, bias):
        return self._h(self.lib.refd_linear_swiglu(self._i(x), self._i(w), self._i(bias)))
    def fused_pixel_norm_modulate_silu(self, policy, x, shift, scale, eps=1e-8, out_dtype=F32):
        return self._h(self.lib.refd_pixel_norm_modulate_silu(int(policy), self._i(x), self._i(shift), self._i(scale),
                                                              _c.c_float(eps), int(out_dtype)))
    def fused_edge_time_pad(self, x, temporal, pad_h, pad_w):
        return self._h(self.lib.refd_edge_time_pad(self._i(x), _c.c_int64(temporal), _c.c_int64(pad_h), _c.c_int64(pad_w)))
    def fused_depth_to_space_residual(self, projected, x):
        return self._h(self.lib.refd_depth_to_space_residual(self._i(projected), self._i(x)))
    def fused_swiglu(self, x): return self._h(self.lib.refd_swiglu(self._i(x)))
    def fused_group_norm_silu(self, x, groups, w, b, eps):
        return self._h(self.lib.refd_group_norm_silu(self._i(x), int(groups), self._i(w), self._i(b), _c.c_float(eps)))
    def fused_cfg_euler(self, x, u, c, guidance, delta, subtract=True, guidance_role=False, solver_role=False):
        return self._h(self.lib.refd_cfg_euler(self._i(x), self._i(u), self._i(c), _c.c_float(guidance), _c.c_float(delta),
                                               int(subtract), int(guidance_role), int(solver_role)))
