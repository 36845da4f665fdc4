// Elementwise and broadcast kernels: binary arithmetic, casts, activations, SwiGLU, gated
// residual, RoPE, weight dequantisation and the sampler's guidance / Euler updates.
//
// All of them are pure HBM streams, so the shape is the same everywhere: a persistent grid
// (a multiple of the SM count), every thread moving 16 bytes per access with several
// independent accesses in flight, streaming cache hints on tensors that are touched once,
// read-only cached loads on the small broadcast operands.  Arithmetic restates the
// reference kernels of native/src/backend/cuda/cuda_backend.cu expression for expression.
#include "vrb_common.cuh"

namespace vrb {
namespace {

constexpr int kThreads = 256;
constexpr int kPerSm = 8;  // 8 x 256 threads = a full SM

inline bool vec8_ok(int64_t count, std::initializer_list<const void*> ptrs) {
    if (count % 8) return false;
    for (const void* p : ptrs) if (p && !aligned16(p)) return false;
    return true;
}

// ------------------------------------------------------------------------------- unary --
enum UnaryOp { kActSilu = 0, kActGelu, kActGeluTanh, kActTanh, kActRelu, kClamp, kExp, kSqrt, kCast };

template <int OP>
__device__ __forceinline__ float unary_value(float x, float p0, float p1) {
    if constexpr (OP <= kActRelu) return activation_value(OP, x);
    else if constexpr (OP == kClamp) return fminf(p1, fmaxf(p0, x));   // :2188
    else if constexpr (OP == kExp) return expf(x);                     // :2195
    else if constexpr (OP == kSqrt) return sqrtf(x);                   // :2202
    else return x;                                                     // cast
}

template <int OP>
__global__ void __launch_bounds__(kThreads) unary_vec_kernel(const void* x, int in_dt, void* out, int out_dt,
                                                            int64_t chunks, float p0, float p1) {
    constexpr int U = 4;  // independent 16-byte loads in flight per thread
    const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
    for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < chunks; i += stride * U) {
        float v[U][8];
#pragma unroll
        for (int u = 0; u < U; ++u)
            if (i + u * stride < chunks) load8<true>(x, in_dt, (i + u * stride) * 8, v[u]);
#pragma unroll
        for (int u = 0; u < U; ++u) {
            if (i + u * stride >= chunks) break;
#pragma unroll
            for (int e = 0; e < 8; ++e) v[u][e] = unary_value<OP>(v[u][e], p0, p1);
            store8(out, out_dt, (i + u * stride) * 8, v[u]);
        }
    }
}
template <int OP>
__global__ void __launch_bounds__(kThreads) unary_scalar_kernel(const void* x, int in_dt, void* out, int out_dt,
                                                               int64_t count, float p0, float p1) {
    const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
    for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < count; i += stride)
        store1(out, out_dt, i, unary_value<OP>(load1(x, in_dt, i), p0, p1));
}
__global__ void __launch_bounds__(kThreads) cast_u8_kernel(const uint8_t* x, void* out, int out_dt, int64_t count) {
    const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
    for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < count; i += stride)
        store1(out, out_dt, i, static_cast<float>(x[i]));
}

template <int OP>
int launch_unary(const void* x, int in_dt, void* out, int out_dt, int64_t count, float p0, float p1,
                 cudaStream_t stream, const char* what) {
    VRB_REQUIRE(x && out, VRB_ERR_INVALID, "%s: null tensor", what);
    VRB_REQUIRE(count > 0, VRB_ERR_INVALID, "%s: element count must be positive", what);
    VRB_REQUIRE(is_float_dtype(in_dt) && is_float_dtype(out_dt), VRB_ERR_UNSUPPORTED, "%s: dtype must be F32 or BF16", what);
    if (OP != kCast && in_dt == out_dt && unary_lut_applicable(in_dt, count, x, out))
        return launch_unary_lut(OP, x, out, count, p0, p1, stream);
    if (vec8_ok(count, {x, out})) {
        const int64_t chunks = count / 8;
        unary_vec_kernel<OP><<<grid_for((chunks + kThreads - 1) / kThreads, kPerSm), kThreads, 0, stream>>>(
            x, in_dt, out, out_dt, chunks, p0, p1);
    } else {
        unary_scalar_kernel<OP><<<grid_for((count + kThreads - 1) / kThreads, kPerSm), kThreads, 0, stream>>>(
            x, in_dt, out, out_dt, count, p0, p1);
    }
    return after_launch(what);
}

// ------------------------------------------------------------------------------ binary --
struct Meta { int rank; int64_t shape[8]; int64_t strides[8]; };

template <int KIND>
__device__ __forceinline__ float binary_value(float a, float b) {
    if constexpr (KIND == VRB_ADD) return __fadd_rn(a, b);
    else if constexpr (KIND == VRB_MUL) return __fmul_rn(a, b);
    else if constexpr (KIND == VRB_DIV) return __fdiv_rn(a, b);
    else return fmaxf(a, b);
}

// Operand classes after shape analysis: the whole tensor, one scalar, or a dense trailing
// block that repeats every `period` elements (the adaLN [S,D] op [1,1,D] case).
template <int KIND>
__global__ void __launch_bounds__(kThreads) binary_flat_vec_kernel(const void* a, const void* b, void* out, int dt,
                                                                   int64_t chunks, int64_t a_period, int64_t b_period,
                                                                   int64_t count) {
    const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
    for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < chunks; i += stride) {
        const int64_t e0 = i * 8;
        float av[8], bv[8];
        if (a_period == count) load8<true>(a, dt, e0, av);
        else if (a_period == 1) { const float s = load1(a, dt, 0);
#pragma unroll
            for (int e = 0; e < 8; ++e) av[e] = s; }
        else load8<false>(a, dt, e0 % a_period, av);
        if (b_period == count) load8<true>(b, dt, e0, bv);
        else if (b_period == 1) { const float s = load1(b, dt, 0);
#pragma unroll
            for (int e = 0; e < 8; ++e) bv[e] = s; }
        else load8<false>(b, dt, e0 % b_period, bv);
#pragma unroll
        for (int e = 0; e < 8; ++e) av[e] = binary_value<KIND>(av[e], bv[e]);
        store8(out, dt, e0, av);
    }
}

__device__ __forceinline__ int64_t broadcast_offset(int64_t linear, const Meta& o, const Meta& in) {
    int64_t offset = 0;
    const int shift = o.rank - in.rank;
    for (int d = o.rank - 1; d >= 0; --d) {
        const int64_t c = linear % o.shape[d];
        linear /= o.shape[d];
        const int id = d - shift;
        if (id >= 0 && in.shape[id] != 1) offset += c * in.strides[id];
    }
    return offset;
}
template <int KIND>
__global__ void __launch_bounds__(kThreads) binary_general_kernel(const void* a, const void* b, void* out, int dt,
                                                                  int64_t count, Meta om, Meta am, Meta bm) {
    const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
    for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < count; i += stride)
        store1(out, dt, i, binary_value<KIND>(load1(a, dt, broadcast_offset(i, om, am)),
                                              load1(b, dt, broadcast_offset(i, om, bm))));
}

Meta make_meta(const int64_t* shape, int rank) {
    Meta m{};
    m.rank = rank;
    int64_t s = 1;
    for (int d = rank - 1; d >= 0; --d) { m.shape[d] = shape[d]; m.strides[d] = s; s *= shape[d]; }
    return m;
}
// Elements after which a trailing-dense operand repeats; 0 when the operand broadcasts along
// an inner axis and needs general indexing.
int64_t flat_period(const Meta& out, const Meta& in) {
    int64_t elements = 1;
    for (int d = 0; d < in.rank; ++d) elements *= in.shape[d];
    if (elements <= 0) return 0;
    int64_t remaining = elements;
    const int shift = out.rank - in.rank;
    for (int d = out.rank - 1; remaining > 1 && d >= 0; --d) {
        const int id = d - shift;
        if (id < 0 || in.shape[id] != out.shape[d]) return 0;
        remaining /= out.shape[d];
    }
    return remaining == 1 ? elements : 0;
}

// Broadcast along inner axes (a [B, C, T, H, W] tensor with a [B, C, 1, 1, 1] vector, [B, S, D] with
// [B, 1, D], ...): the output's axes are merged wherever both operands stay dense or both stay
// broadcast, and if at most three merged axes remain and the innermost run is a multiple of 8
// elements, each operand is either read in 16-byte chunks along it or is one value per run.
struct Collapsed {
    int dims;            // 1..3, innermost last
    int64_t shape[3];
    int64_t a_stride[3], b_stride[3];   // in elements; 0 = broadcast
};
bool collapse(const Meta& om, const Meta& am, const Meta& bm, Collapsed& c) {
    int64_t shape[8], as[8], bs[8];
    int n = 0;
    for (int d = 0; d < om.rank; ++d) {
        if (om.shape[d] == 1) continue;
        const int ad = d - (om.rank - am.rank), bd = d - (om.rank - bm.rank);
        const int64_t sa = (ad >= 0 && am.shape[ad] != 1) ? am.strides[ad] : 0;
        const int64_t sb = (bd >= 0 && bm.shape[bd] != 1) ? bm.strides[bd] : 0;
        if (n > 0) {
            // merge into the previous (outer) axis when it continues densely, or stays broadcast, in both operands
            const bool a_ok = (as[n - 1] == sa * om.shape[d]) && (sa != 0 || as[n - 1] == 0);
            const bool b_ok = (bs[n - 1] == sb * om.shape[d]) && (sb != 0 || bs[n - 1] == 0);
            if (a_ok && b_ok) { shape[n - 1] *= om.shape[d]; as[n - 1] = sa; bs[n - 1] = sb; continue; }
        }
        shape[n] = om.shape[d]; as[n] = sa; bs[n] = sb; ++n;
    }
    if (n == 0 || n > 3) return false;
    c.dims = 3;
    for (int k = 0; k < 3; ++k) {
        const int src = n - 3 + k;
        c.shape[k] = src >= 0 ? shape[src] : 1;
        c.a_stride[k] = src >= 0 ? as[src] : 0;
        c.b_stride[k] = src >= 0 ? bs[src] : 0;
    }
    if (c.shape[2] % 8 != 0) return false;
    for (int k = 0; k < 3; ++k) {
        if (k < 2 && (c.a_stride[k] % 8 != 0 || c.b_stride[k] % 8 != 0) ) {
            // an outer stride that is not a multiple of 8 elements is fine for an operand that is one
            // value per run (its chunk loads are scalar), not for one read in chunks
            if ((c.a_stride[k] % 8 != 0 && c.a_stride[2] != 0) || (c.b_stride[k] % 8 != 0 && c.b_stride[2] != 0)) return false;
        }
    }
    return (c.a_stride[2] == 0 || c.a_stride[2] == 1) && (c.b_stride[2] == 0 || c.b_stride[2] == 1);
}

template <int KIND, typename I>
__global__ void __launch_bounds__(kThreads) binary_collapsed_vec_kernel(const void* __restrict__ a, const void* __restrict__ b,
                                                                        void* __restrict__ out, int dt, Collapsed c) {
    const I n1 = static_cast<I>(c.shape[1]), n2 = static_cast<I>(c.shape[2] / 8);
    const I total = static_cast<I>(c.shape[0]) * n1 * n2;
    const I stride = static_cast<I>(gridDim.x) * blockDim.x;
    for (I i = static_cast<I>(blockIdx.x) * blockDim.x + threadIdx.x; i < total; i += stride) {
        const I r = i / n2, i2 = i - r * n2;
        const I i0 = r / n1, i1 = r - i0 * n1;
        const int64_t ao = static_cast<int64_t>(i0) * c.a_stride[0] + static_cast<int64_t>(i1) * c.a_stride[1];
        const int64_t bo = static_cast<int64_t>(i0) * c.b_stride[0] + static_cast<int64_t>(i1) * c.b_stride[1];
        float av[8], bv[8];
        if (c.a_stride[2]) load8<true>(a, dt, ao + static_cast<int64_t>(i2) * 8, av);
        else { const float v = load1(a, dt, ao);
#pragma unroll
            for (int e = 0; e < 8; ++e) av[e] = v; }
        if (c.b_stride[2]) load8<true>(b, dt, bo + static_cast<int64_t>(i2) * 8, bv);
        else { const float v = load1(b, dt, bo);
#pragma unroll
            for (int e = 0; e < 8; ++e) bv[e] = v; }
#pragma unroll
        for (int e = 0; e < 8; ++e) av[e] = binary_value<KIND>(av[e], bv[e]);
        store8(out, dt, static_cast<int64_t>(i) * 8, av);
    }
}

template <int KIND>
int launch_binary(const void* a, const Meta& am, const void* b, const Meta& bm, void* out, const Meta& om,
                  int64_t count, int dt, cudaStream_t stream) {
    const int64_t ap = flat_period(om, am), bp = flat_period(om, bm);
    const bool periods_ok = ap && bp && (ap == count || ap == 1 || ap % 8 == 0) && (bp == count || bp == 1 || bp % 8 == 0);
    if (periods_ok && vec8_ok(count, {a, b, out})) {
        const int64_t chunks = count / 8;
        binary_flat_vec_kernel<KIND><<<grid_for((chunks + kThreads - 1) / kThreads, kPerSm), kThreads, 0, stream>>>(
            a, b, out, dt, chunks, ap, bp, count);
    } else if (Collapsed c; vec8_ok(count, {a, b, out}) && collapse(om, am, bm, c)) {
        const int64_t chunks = count / 8;
        const int grid = grid_for((chunks + kThreads - 1) / kThreads, kPerSm);
        if (chunks + static_cast<int64_t>(grid) * kThreads < (int64_t{1} << 32))
            binary_collapsed_vec_kernel<KIND, unsigned><<<grid, kThreads, 0, stream>>>(a, b, out, dt, c);
        else
            binary_collapsed_vec_kernel<KIND, int64_t><<<grid, kThreads, 0, stream>>>(a, b, out, dt, c);
    } else {
        binary_general_kernel<KIND><<<grid_for((count + kThreads - 1) / kThreads, kPerSm), kThreads, 0, stream>>>(
            a, b, out, dt, count, om, am, bm);
    }
    return after_launch("binary");
}

// ------------------------------------------------------------------------------ SwiGLU --
// mochi.cpp:195-202: silu(b) is stored (rounded to the tensor dtype) before a * silu(b).
__global__ void __launch_bounds__(kThreads) swiglu_kernel(const void* proj, void* out, int dt, int64_t rows,
                                                         int64_t hidden_chunks) {
    const int64_t total = rows * hidden_chunks;
    const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
    for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < total; i += stride) {
        const int64_t row = i / hidden_chunks, chunk = i - row * hidden_chunks;
        const int64_t in0 = (row * 2 * hidden_chunks + chunk) * 8;
        float a[8], g[8];
        load8<true>(proj, dt, in0, a);
        load8<true>(proj, dt, in0 + hidden_chunks * 8, g);
#pragma unroll
        for (int e = 0; e < 8; ++e) a[e] = __fmul_rn(a[e], round_to(dt, activation_value(VRB_SILU, g[e])));
        store8(out, dt, i * 8, a);
    }
}
__global__ void __launch_bounds__(kThreads) swiglu_scalar_kernel(const void* proj, void* out, int dt, int64_t rows,
                                                                int64_t hidden) {
    const int64_t total = rows * hidden;
    const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
    for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < total; i += stride) {
        const int64_t row = i / hidden, c = i - row * hidden;
        const float a = load1(proj, dt, row * 2 * hidden + c), g = load1(proj, dt, row * 2 * hidden + hidden + c);
        store1(out, dt, i, __fmul_rn(a, round_to(dt, activation_value(VRB_SILU, g))));
    }
}

// ----------------------------------------------------------------------- gated residual --
// common.cpp:134-144 with T = state dtype: T(res) + round_T(T(branch) * T(gate)).
__global__ void __launch_bounds__(kThreads) gated_residual_kernel(
        const void* res, int res_dt, const void* branch, int br_dt, const void* gate, int gate_dt,
        void* out, int state_dt, int64_t rows, int64_t width_chunks, int64_t rows_per_vector, int64_t vectors) {
    constexpr int U = 2;
    const int64_t total = rows * width_chunks;
    const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
    for (int64_t i0 = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i0 < total; i0 += stride * U) {
        float r[U][8], b[U][8], g[U][8];
#pragma unroll
        for (int u = 0; u < U; ++u) {
            const int64_t i = i0 + u * stride;
            if (i >= total) break;
            load8<true>(res, res_dt, i * 8, r[u]);
            load8<true>(branch, br_dt, i * 8, b[u]);
            if (gate) {
                const int64_t row = i / width_chunks, chunk = i - row * width_chunks;
                const int64_t vec = vectors > 1 ? (row / rows_per_vector) % vectors : 0;
                load8<false>(gate, gate_dt, (vec * width_chunks + chunk) * 8, g[u]);
            }
        }
#pragma unroll
        for (int u = 0; u < U; ++u) {
            const int64_t i = i0 + u * stride;
            if (i >= total) break;
#pragma unroll
            for (int e = 0; e < 8; ++e) {
                float br = round_to(state_dt, b[u][e]);
                if (gate) br = round_to(state_dt, __fmul_rn(br, round_to(state_dt, g[u][e])));
                r[u][e] = __fadd_rn(round_to(state_dt, r[u][e]), br);
            }
            store8(out, state_dt, i * 8, r[u]);
        }
    }
}
// Same arithmetic with the three tensor dtypes fixed at compile time and 32-bit indexing (the
// common case: fewer than 2^31 chunks).  All-bf16 takes two packed bf16 instructions per pair of
// elements: the product of two bf16 values is exact in F32, so mul.rn.bf16x2 rounds once exactly
// like the reference's F32 multiply + bf16 store; likewise add.rn.bf16x2 (an exact bf16 sum needs
// at most 24 bits whenever it is not absorbed by the larger operand).
template <bool BF16>
__device__ __forceinline__ void load8_typed(const void* base, int64_t e, float (&v)[8]) {
    load8<true>(base, BF16 ? VRB_BF16 : VRB_F32, e, v);
}
template <bool RES_BF16, bool BR_BF16, bool STATE_BF16>
__global__ void __launch_bounds__(kThreads) gated_residual_typed_kernel(
        const void* __restrict__ res, const void* __restrict__ branch, const void* __restrict__ gate, int gate_dt,
        void* __restrict__ out, unsigned total, unsigned width_chunks, unsigned rows_per_vector, unsigned vectors) {
    constexpr int U = 2;
    const unsigned stride = gridDim.x * blockDim.x;
    pdl_launch_dependents();
    pdl_wait();
    // the chunk's column and gate vector are carried from step to step instead of being divided out of
    // the index (column = i % width_chunks, vector = (i / period) % vectors, period = rows_per_vector * width_chunks)
    const unsigned first = blockIdx.x * blockDim.x + threadIdx.x;
    const unsigned long long period = static_cast<unsigned long long>(rows_per_vector) * width_chunks;
    unsigned column = 0, vector = 0, column_step = 0, vector_step = 0;
    unsigned long long within = 0, within_step = 0;
    if (gate) {
        column = first % width_chunks; within = first % period; vector = static_cast<unsigned>((first / period) % vectors);
        column_step = stride % width_chunks; within_step = stride % period; vector_step = static_cast<unsigned>((stride / period) % vectors);
    }
    for (unsigned i0 = first; i0 < total; i0 += stride * U) {
        if constexpr (RES_BF16 && BR_BF16 && STATE_BF16) {
            uint4 r[U], b[U];
            float g[U][8];
#pragma unroll
            for (int u = 0; u < U; ++u) {
                const unsigned i = i0 + u * stride;
                if (i < total) {
                    r[u] = __ldcs(static_cast<const uint4*>(res) + i);
                    b[u] = __ldcs(static_cast<const uint4*>(branch) + i);
                    if (gate) load8<false>(gate, gate_dt, (static_cast<int64_t>(vector) * width_chunks + column) * 8, g[u]);
                }
                if (gate) {
                    column += column_step;
                    if (column >= width_chunks) column -= width_chunks;
                    within += within_step;
                    vector += vector_step;
                    if (within >= period) { within -= period; ++vector; }
                    if (vector >= vectors) vector -= vectors;
                }
            }
#pragma unroll
            for (int u = 0; u < U; ++u) {
                const unsigned i = i0 + u * stride;
                if (i >= total) break;
                const uint32_t rw[4] = {r[u].x, r[u].y, r[u].z, r[u].w};
                const uint32_t bw[4] = {b[u].x, b[u].y, b[u].z, b[u].w};
                uint32_t ow[4];
#pragma unroll
                for (int k = 0; k < 4; ++k) {
                    __nv_bfloat162 br = *reinterpret_cast<const __nv_bfloat162*>(&bw[k]);
                    if (gate) br = __hmul2_rn(br, __floats2bfloat162_rn(g[u][2 * k], g[u][2 * k + 1]));
                    const __nv_bfloat162 sum = __hadd2_rn(*reinterpret_cast<const __nv_bfloat162*>(&rw[k]), br);
                    ow[k] = *reinterpret_cast<const uint32_t*>(&sum);
                }
                __stcs(static_cast<uint4*>(out) + i, make_uint4(ow[0], ow[1], ow[2], ow[3]));
            }
        } else {
            float r[U][8], b[U][8], g[U][8];
#pragma unroll
            for (int u = 0; u < U; ++u) {
                const unsigned i = i0 + u * stride;
                if (i >= total) break;
                load8_typed<RES_BF16>(res, static_cast<int64_t>(i) * 8, r[u]);
                load8_typed<BR_BF16>(branch, static_cast<int64_t>(i) * 8, b[u]);
                if (gate) {
                    load8<false>(gate, gate_dt, (static_cast<int64_t>(vector) * width_chunks + column) * 8, g[u]);
                    column += column_step;
                    if (column >= width_chunks) column -= width_chunks;
                    within += within_step;
                    vector += vector_step;
                    if (within >= period) { within -= period; ++vector; }
                    if (vector >= vectors) vector -= vectors;
                }
            }
#pragma unroll
            for (int u = 0; u < U; ++u) {
                const unsigned i = i0 + u * stride;
                if (i >= total) break;
                if constexpr (STATE_BF16) {
                    if constexpr (!RES_BF16) round8_bf16_inplace(r[u]);
                    if constexpr (!BR_BF16) round8_bf16_inplace(b[u]);
                }
                if (gate) {
                    if constexpr (STATE_BF16) round8_bf16_inplace(g[u]);
#pragma unroll
                    for (int e = 0; e < 8; ++e) b[u][e] = __fmul_rn(b[u][e], g[u][e]);
                    if constexpr (STATE_BF16) round8_bf16_inplace(b[u]);
                }
#pragma unroll
                for (int e = 0; e < 8; ++e) r[u][e] = __fadd_rn(r[u][e], b[u][e]);
                store8(out, STATE_BF16 ? VRB_BF16 : VRB_F32, static_cast<int64_t>(i) * 8, r[u]);
            }
        }
    }
}

// All-bf16 tensors with a gate, large launches: the gate vectors are rounded to bf16 once per CTA into shared memory
// (the reference rounds the gate to the state dtype before the multiply, so this is the same value), and the chunk's
// column and vector are carried along instead of being divided out of the index: one 16-byte shared-memory load per
// chunk where the general kernel has three 32-bit divisions, two 16-byte gate loads and four conversions.
// gate_bf16 holds vectors * width_chunks chunks of 8 bf16.
__global__ void __launch_bounds__(kThreads) gated_residual_staged_kernel(
        const uint4* __restrict__ res, const uint4* __restrict__ branch, const void* __restrict__ gate, int gate_dt,
        uint4* __restrict__ out, unsigned total, unsigned width_chunks, unsigned rows_per_vector, unsigned vectors) {
    extern __shared__ __align__(16) uint4 gate_bf16[];
    constexpr int U = 2;
    pdl_launch_dependents();
    pdl_wait();
    for (unsigned c = threadIdx.x; c < vectors * width_chunks; c += kThreads) {
        float g[8];
        load8<false>(gate, gate_dt, static_cast<int64_t>(c) * 8, g);
        gate_bf16[c] = make_uint4(pack_bf16x2(g[0], g[1]), pack_bf16x2(g[2], g[3]), pack_bf16x2(g[4], g[5]), pack_bf16x2(g[6], g[7]));
    }
    __syncthreads();
    const unsigned stride = gridDim.x * kThreads;
    // chunk i lies in column i % width_chunks of vector (i / period) % vectors, period = rows_per_vector * width_chunks
    // (a 64-bit product: with one vector the period only has to exceed every index)
    const unsigned long long period = static_cast<unsigned long long>(rows_per_vector) * width_chunks;
    const unsigned first = blockIdx.x * kThreads + threadIdx.x;
    unsigned column = first % width_chunks;
    unsigned long long within = first % period;
    unsigned vector = static_cast<unsigned>((first / period) % vectors);
    const unsigned column_step = stride % width_chunks;
    const unsigned long long within_step = stride % period;
    const unsigned vector_step = static_cast<unsigned>((stride / period) % vectors);
    auto advance = [&] {
        column += column_step;
        if (column >= width_chunks) column -= width_chunks;
        within += within_step;
        vector += vector_step;
        if (within >= period) { within -= period; ++vector; }
        if (vector >= vectors) vector -= vectors;
    };
    for (unsigned i0 = first; i0 < total; i0 += stride * U) {
        uint4 r[U], b[U], g[U];
#pragma unroll
        for (int u = 0; u < U; ++u) {
            const unsigned i = i0 + u * stride;
            if (i < total) {
                r[u] = __ldcs(res + i);
                b[u] = __ldcs(branch + i);
                g[u] = gate_bf16[vector * width_chunks + column];
            }
            advance();
        }
#pragma unroll
        for (int u = 0; u < U; ++u) {
            const unsigned i = i0 + u * stride;
            if (i >= total) break;
            const uint32_t rw[4] = {r[u].x, r[u].y, r[u].z, r[u].w}, bw[4] = {b[u].x, b[u].y, b[u].z, b[u].w};
            const uint32_t gw[4] = {g[u].x, g[u].y, g[u].z, g[u].w};
            uint32_t ow[4];
#pragma unroll
            for (int k = 0; k < 4; ++k) {
                const __nv_bfloat162 br = __hmul2_rn(*reinterpret_cast<const __nv_bfloat162*>(&bw[k]), *reinterpret_cast<const __nv_bfloat162*>(&gw[k]));
                const __nv_bfloat162 sum = __hadd2_rn(*reinterpret_cast<const __nv_bfloat162*>(&rw[k]), br);
                ow[k] = *reinterpret_cast<const uint32_t*>(&sum);
            }
            __stcs(out + i, make_uint4(ow[0], ow[1], ow[2], ow[3]));
        }
    }
}

__global__ void __launch_bounds__(kThreads) gated_residual_scalar_kernel(
        const void* res, int res_dt, const void* branch, int br_dt, const void* gate, int gate_dt,
        void* out, int state_dt, int64_t rows, int64_t width, int64_t rows_per_vector, int64_t vectors) {
    const int64_t total = rows * width;
    const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
    for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < total; i += stride) {
        float br = round_to(state_dt, load1(branch, br_dt, i));
        if (gate) {
            const int64_t row = i / width, c = i - row * width;
            const int64_t vec = (row / rows_per_vector) % vectors;
            br = round_to(state_dt, __fmul_rn(br, round_to(state_dt, load1(gate, gate_dt, vec * width + c))));
        }
        store1(out, state_dt, i, __fadd_rn(round_to(state_dt, load1(res, res_dt, i)), br));
    }
}

// -------------------------------------------------------------------------------- RoPE --
// rope_kernel :1200-1215 (standalone form).  Tables may broadcast along any axis.
__global__ void __launch_bounds__(kThreads) rope_general_kernel(const void* x, int x_dt, const void* cosine, const void* sine,
                                                               int f_dt, void* out, int64_t count, Meta xm, Meta fm) {
    const int64_t width = xm.shape[xm.rank - 1];
    const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
    for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < count; i += stride) {
        const int64_t col = i % width;
        const float paired = load1(x, x_dt, i - col + (col ^ 1));
        const float rotated = (i & 1) ? paired : -paired;
        const int64_t f = broadcast_offset(i, xm, fm);
        store1(out, x_dt, i, __fadd_rn(__fmul_rn(load1(x, x_dt, i), load1(cosine, f_dt, f)),
                                       __fmul_rn(rotated, load1(sine, f_dt, f))));
    }
}
// Two table layouts cover the pipelines.  heads == 0: the table equals x's trailing axes and
// repeats every `period` elements.  heads > 0: one table row of `width` per token shared by
// that token's `heads` rows of x ([.., T, 1, W] against [.., T, H, W]); f_tokens table rows.
__global__ void __launch_bounds__(kThreads) rope_vec_kernel(const void* x, int x_dt, const void* cosine, const void* sine,
                                                           int f_dt, void* out, int64_t chunks, int64_t width,
                                                           int64_t heads, int64_t f_tokens, int64_t period) {
    const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
    for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < chunks; i += stride) {
        float v[8], co[8], si[8], r[8];
        const int64_t e0 = i * 8;
        load8<true>(x, x_dt, e0, v);
        int64_t f;
        if (heads > 0) f = ((e0 / (heads * width)) % f_tokens) * width + e0 % width;
        else f = e0 % period;
        load8<false>(cosine, f_dt, f, co);
        load8<false>(sine, f_dt, f, si);
#pragma unroll
        for (int e = 0; e < 8; ++e) {
            const float rotated = (e & 1) ? v[e ^ 1] : -v[e ^ 1];
            r[e] = __fadd_rn(__fmul_rn(v[e], co[e]), __fmul_rn(rotated, si[e]));
        }
        store8(out, x_dt, i * 8, r);
    }
}

// ------------------------------------------------------------------------ dequantisation --
// decode_fp8_e4m3fn :630-638 as bit manipulation: value = sign * (e ? (8+m) * 2^(e-10) : m * 2^-9).
// Both forms are exact in F32, so this equals ldexpf() on every one of the 256 codes
// (0x7f / 0xff give +-480, no NaN case, as in the reference).
__device__ __forceinline__ float decode_fp8(uint32_t raw) {
    const uint32_t e = (raw >> 3) & 0xfu, m = raw & 0x7u;
    const float mag = e ? __uint_as_float(((e + 120u) << 23) | (m << 20))   // (1 + m/8) * 2^(e-7)
                        : static_cast<float>(m) * 0.001953125f;             // m * 2^-9
    return (raw & 0x80u) ? -mag : mag;
}
template <int KIND>
__device__ __forceinline__ float quant_value(const uint8_t* packed, int64_t index) {
    if constexpr (KIND == VRB_Q_FP8_E4M3FN) return decode_fp8(packed[index]);
    else if constexpr (KIND == VRB_Q_INT8) return static_cast<float>(static_cast<int8_t>(packed[index]));
    else {
        const uint8_t byte = packed[index / 2];
        const uint32_t nibble = (index & 1) ? (byte >> 4) : (byte & 0xfu);
        return static_cast<float>(nibble >= 8 ? static_cast<int>(nibble) - 16 : static_cast<int>(nibble));
    }
}
// General form (:641-658): any group size, any alignment.
template <int KIND>
__global__ void __launch_bounds__(kThreads) dequant_scalar_kernel(const uint8_t* packed, const float* scales, void* out,
                                                                 int out_dt, int64_t count, int64_t inner, int64_t groups,
                                                                 int64_t group_size) {
    const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
    for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < count; i += stride) {
        const int64_t outer = i / inner, group = (i % inner) / group_size;
        store1(out, out_dt, i, __fmul_rn(quant_value<KIND>(packed, i), scales[outer * groups + group]));
    }
}
// Byte-per-element kinds with inner % 16 == 0 and group_size % 16 == 0.  Every row is cut into
// equal tiles of at most kThreads * U 16-code chunks, so the row (and with per-channel scales
// the scale itself) is found once per tile instead of by two 64-bit divisions per chunk.
//
// FP8 decode without a branch: the seven magnitude bits eeee mmm placed at bits 26..20 of an
// F32 word read as (1 + m/8) * 2^(e-127) for e != 0 and as the F32 denormal m/8 * 2^-126 for
// e == 0, i.e. exactly the e4m3 value times 2^-120 in both cases (0x7f / 0xff give 480 * 2^-120,
// no NaN case, as decode_fp8_e4m3fn :630-638).  Multiplying by scale * 2^120 (exact while
// |scale| < 2^7, checked per tile) therefore rounds the same real product the reference rounds;
// the code's sign bit is XOR-ed into the scale.  Five integer/FP instructions per code.
__device__ __forceinline__ float fp8_times(uint32_t word, int k, uint32_t scale_bits) {   // scale_bits = bits of scale * 2^120
    const uint32_t mag = (k == 3 ? word >> 4 : word << (20 - 8 * k)) & 0x07f00000u;
    const uint32_t sign = (k == 3 ? word : word << (24 - 8 * k)) & 0x80000000u;
    return __fmul_rn(__uint_as_float(mag), __uint_as_float(scale_bits ^ sign));
}
// Flat persistent form: thread t takes 16-byte code chunks t, t + stride, ... of the whole [rows, inner] matrix
// (U loads in flight), finds each chunk's row with one 32-bit division, and writes the chunk's 16 results
// with ONE 32-byte store (bf16).  Every thread has the same amount of work whatever the row length.
template <int KIND, bool OUT_BF16, bool ROW_SCALE>
__global__ void __launch_bounds__(kThreads, 4) dequant_tile_kernel(const uint4* __restrict__ packed, const float* __restrict__ scales,
                                                                  void* __restrict__ out, unsigned total_chunks, unsigned inner_chunks,
                                                                  unsigned groups, unsigned group_chunks) {
    constexpr int U = 4;
    const unsigned stride = gridDim.x * kThreads;
    for (unsigned i0 = blockIdx.x * kThreads + threadIdx.x; i0 < total_chunks; i0 += stride * U) {
        uint4 raw[U];
        float scale[U];
#pragma unroll
        for (int u = 0; u < U; ++u) {
            const unsigned i = i0 + u * stride;
            if (i < total_chunks) {
                raw[u] = __ldcs(packed + i);
                const unsigned row = i / inner_chunks;
                scale[u] = __ldg(scales + (ROW_SCALE ? row : row * groups + (i - row * inner_chunks) / group_chunks));
            }
        }
#pragma unroll
        for (int u = 0; u < U; ++u) {
            const unsigned i = i0 + u * stride;
            if (i >= total_chunks) break;
            const uint32_t words[4] = {raw[u].x, raw[u].y, raw[u].z, raw[u].w};
            float v[16];
            const float lifted = scale[u] * 0x1p120f;
            if (KIND == VRB_Q_FP8_E4M3FN && fabsf(scale[u]) < 128.0f) {
                const uint32_t sb = __float_as_uint(lifted);
#pragma unroll
                for (int w = 0; w < 4; ++w)
#pragma unroll
                    for (int k = 0; k < 4; ++k) v[w * 4 + k] = fp8_times(words[w], k, sb);
            } else {
#pragma unroll
                for (int w = 0; w < 4; ++w)
#pragma unroll
                    for (int k = 0; k < 4; ++k) {
                        const uint32_t code = (words[w] >> (8 * k)) & 0xffu;
                        const float q = KIND == VRB_Q_FP8_E4M3FN ? decode_fp8(code)
                                                                 : static_cast<float>(static_cast<int8_t>(code));
                        v[w * 4 + k] = __fmul_rn(q, scale[u]);
                    }
            }
            const int64_t e0 = static_cast<int64_t>(i) * 16;
            if constexpr (OUT_BF16) {
                store16_bf16(out, e0, v);
            } else {
                float lo[8], hi[8];
#pragma unroll
                for (int e = 0; e < 8; ++e) { lo[e] = v[e]; hi[e] = v[8 + e]; }
                store8(out, VRB_F32, e0, lo);
                store8(out, VRB_F32, e0 + 8, hi);
            }
        }
    }
}
// INT4 (two's complement nibbles, low nibble first, :641-658 with Kind 2): 32 codes per 16-byte
// load, same row tiles.  inner % 32 == 0 and group_size % 32 == 0.
template <bool OUT_BF16, bool ROW_SCALE>
__global__ void __launch_bounds__(kThreads, 4) dequant_int4_tile_kernel(const uint4* __restrict__ packed, const float* __restrict__ scales,
                                                                       void* __restrict__ out, int64_t rows, int64_t inner_chunks,
                                                                       int64_t groups, int group_chunks, int64_t tiles_per_row,
                                                                       int64_t tile_chunks) {
    const int64_t tiles = rows * tiles_per_row;
    for (int64_t t = blockIdx.x; t < tiles; t += gridDim.x) {
        const int64_t row = t / tiles_per_row;
        const int64_t tile_begin = (t - row * tiles_per_row) * tile_chunks;
        const int64_t tile_end = tile_begin + tile_chunks < inner_chunks ? tile_begin + tile_chunks : inner_chunks;
        for (int64_t c = tile_begin + threadIdx.x; c < tile_end; c += kThreads) {
            const uint4 raw = __ldcs(packed + row * inner_chunks + c);
            const float scale = __ldg(scales + (ROW_SCALE ? row : row * groups + static_cast<int>(c) / group_chunks));
            const uint32_t words[4] = {raw.x, raw.y, raw.z, raw.w};
            const int64_t e0 = (row * inner_chunks + c) * 32;
#pragma unroll
            for (int w = 0; w < 4; ++w) {
                float v[8];
#pragma unroll
                for (int k = 0; k < 8; ++k) {
                    const int q = static_cast<int>(words[w] << (28 - 4 * k)) >> 28;   // sign-extended nibble k
                    v[k] = __fmul_rn(static_cast<float>(q), scale);
                }
                store8(out, OUT_BF16 ? VRB_BF16 : VRB_F32, e0 + w * 8, v);
            }
        }
    }
}
void launch_dequant_int4_tiles(const uint8_t* packed, const float* scales, void* out, int out_dtype, int64_t rows, int64_t inner,
                               int64_t groups, int64_t group_size, cudaStream_t s) {
    const int64_t inner_chunks = inner / 32;
    const int64_t tiles_per_row = (inner_chunks + kThreads * 2 - 1) / (kThreads * 2);
    const int64_t tile_chunks = ((inner_chunks + tiles_per_row - 1) / tiles_per_row + 7) & ~int64_t{7};
    const int grid = grid_for(rows * tiles_per_row, 8);
    const uint4* p = reinterpret_cast<const uint4*>(packed);
    const int gc = static_cast<int>(group_size / 32);
#define VRB_DQ4(BF, ROW) dequant_int4_tile_kernel<BF, ROW><<<grid, kThreads, 0, s>>>( \
        p, scales, out, rows, inner_chunks, groups, gc, tiles_per_row, tile_chunks)
    if (out_dtype == VRB_BF16) { if (groups == 1) VRB_DQ4(true, true); else VRB_DQ4(true, false); }
    else { if (groups == 1) VRB_DQ4(false, true); else VRB_DQ4(false, false); }
#undef VRB_DQ4
}

template <int KIND>
void launch_dequant_tiles(const uint8_t* packed, const float* scales, void* out, int out_dtype, int64_t rows, int64_t inner,
                          int64_t groups, int64_t group_size, cudaStream_t s) {
    const int64_t inner_chunks = inner / 16, total = rows * inner_chunks;   // the caller checked total < 2^32
    const int grid = grid_for((total + kThreads - 1) / kThreads, 8);
    const uint4* p = reinterpret_cast<const uint4*>(packed);
    const unsigned gc = static_cast<unsigned>(group_size / 16);
#define VRB_DQ(BF, ROW) dequant_tile_kernel<KIND, BF, ROW><<<grid, kThreads, 0, s>>>( \
        p, scales, out, static_cast<unsigned>(total), static_cast<unsigned>(inner_chunks), static_cast<unsigned>(groups), gc)
    if (out_dtype == VRB_BF16) { if (groups == 1) VRB_DQ(true, true); else VRB_DQ(true, false); }
    else { if (groups == 1) VRB_DQ(false, true); else VRB_DQ(false, false); }
#undef VRB_DQ
}

// -------------------------------------------------------------------- sampler arithmetic --
// precision_scalar_binary (precision.cpp:196-223): value (x) coefficient.
//   declared role: F32 product, result rounded to the storage dtype
//   legacy:        coefficient rounded to the storage dtype first, product rounded
__device__ __forceinline__ float coef_mul(int dt, int role, float v, float coef) {
    return round_to(dt, __fmul_rn(v, role ? coef : round_to(dt, coef)));
}
struct SamplerParams {
    const void* sample; const void* uncond; const void* cond; void* guided; void* out;
    int dt, mode;            // mode 0 cfg, 1 euler, 2 cfg+euler, 3 flow_to_x0
    int role, axpy_role;     // declared scalar role of the guidance / of the solver-or-sigma coefficient
    float scale, coefficient; // coefficient: value of the one-element Euler / sigma multiplier tensor
};
// cfg:   g = u + ((c + u*(-1)) * s)                                  sampling.cpp:181-183
// euler: x' = x + p * k, k = delta * (+-1) computed on a 1-element tensor  sampling.cpp:185-193
__device__ __forceinline__ float cfg_value(int dt, int role, float u, float c, float s) {
    const float n = coef_mul(dt, role, u, -1.0f);
    const float d = round_to(dt, __fadd_rn(c, n));
    const float e = coef_mul(dt, role, d, s);
    return round_to(dt, __fadd_rn(u, e));
}
__device__ __forceinline__ float axpy_value(int dt, int role, float x, float p, float k) {
    return round_to(dt, __fadd_rn(x, coef_mul(dt, role, p, k)));
}
template <bool VEC>
__global__ void __launch_bounds__(kThreads) sampler_kernel(SamplerParams q, int64_t n) {
    const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
    for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < n; i += stride) {
        constexpr int W = VEC ? 8 : 1;
        float x[8], u[8], c[8], g[8], y[8];
        if constexpr (VEC) {
            if (q.sample) load8<true>(q.sample, q.dt, i * 8, x);
            if (q.uncond) load8<true>(q.uncond, q.dt, i * 8, u);
            if (q.cond) load8<true>(q.cond, q.dt, i * 8, c);
        } else {
            if (q.sample) x[0] = load1(q.sample, q.dt, i);
            if (q.uncond) u[0] = load1(q.uncond, q.dt, i);
            if (q.cond) c[0] = load1(q.cond, q.dt, i);
        }
#pragma unroll
        for (int e = 0; e < W; ++e) {
            if (q.mode == 0) y[e] = cfg_value(q.dt, q.role, u[e], c[e], q.scale);
            else if (q.mode == 1 || q.mode == 3) y[e] = axpy_value(q.dt, q.axpy_role, x[e], u[e], q.coefficient);
            else { g[e] = cfg_value(q.dt, q.role, u[e], c[e], q.scale); y[e] = axpy_value(q.dt, q.axpy_role, x[e], g[e], q.coefficient); }
        }
        if constexpr (VEC) {
            if (q.mode == 2 && q.guided) store8(q.guided, q.dt, i * 8, g);
            store8(q.out, q.dt, i * 8, y);
        } else {
            if (q.mode == 2 && q.guided) store1(q.guided, q.dt, i, g[0]);
            store1(q.out, q.dt, i, y[0]);
        }
    }
}
int launch_sampler(SamplerParams q, int64_t count, cudaStream_t stream, const char* what) {
    VRB_REQUIRE(q.out && count > 0, VRB_ERR_INVALID, "%s: null output or empty tensor", what);
    VRB_REQUIRE(is_float_dtype(q.dt), VRB_ERR_UNSUPPORTED, "%s: dtype must be F32 or BF16", what);
    if (vec8_ok(count, {q.sample, q.uncond, q.cond, q.guided, q.out})) {
        const int64_t chunks = count / 8;
        sampler_kernel<true><<<grid_for((chunks + kThreads - 1) / kThreads, kPerSm), kThreads, 0, stream>>>(q, chunks);
    } else {
        sampler_kernel<false><<<grid_for((count + kThreads - 1) / kThreads, kPerSm), kThreads, 0, stream>>>(q, count);
    }
    return after_launch(what);
}
// linear_combine (sampling.cpp:173-179): ((v0*c0 + v1*c1) + v2*c2) + ..., every product through
// precision_scalar_binary, every sum one add in the storage dtype.  Also v_to_x0 (:204-214) and
// affine_first_order (:229-239), which are two-term combinations.
constexpr int kMaxTerms = 4;
struct CombineParams {
    const void* value[kMaxTerms];
    float coefficient[kMaxTerms];
    void* out;
    int terms, dt, role;
};
template <bool VEC>
__global__ void __launch_bounds__(kThreads) linear_combine_kernel(CombineParams q, int64_t n) {
    constexpr int W = VEC ? 8 : 1;
    const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
    for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < n; i += stride) {
        float v[kMaxTerms][8];
#pragma unroll
        for (int t = 0; t < kMaxTerms; ++t) {
            if (t >= q.terms) break;
            if constexpr (VEC) load8<true>(q.value[t], q.dt, i * 8, v[t]);
            else v[t][0] = load1(q.value[t], q.dt, i);
        }
        float y[8];
#pragma unroll
        for (int e = 0; e < W; ++e) {
            y[e] = coef_mul(q.dt, q.role, v[0][e], q.coefficient[0]);
#pragma unroll
            for (int t = 1; t < kMaxTerms; ++t) {
                if (t >= q.terms) break;
                y[e] = round_to(q.dt, __fadd_rn(y[e], coef_mul(q.dt, q.role, v[t][e], q.coefficient[t])));
            }
        }
        if constexpr (VEC) store8(q.out, q.dt, i * 8, y);
        else store1(q.out, q.dt, i, y[0]);
    }
}

// The Euler coefficient: k = delta (x) (+-1) is itself a product on a one-element F32 tensor
// (exact), so k = +-delta in F32 for both scalar contracts.
inline float euler_coefficient(float delta, int subtract) { return subtract ? -delta : delta; }

}  // namespace
}  // namespace vrb

using namespace vrb;

extern "C" int vrb_linear_combine(const void* const* values, const float* coefficients, int terms, void* out, int dtype,
                                  int64_t count, int scalar_role, vrb_stream stream) {
    VRB_REQUIRE(values && coefficients && out, VRB_ERR_INVALID, "linear_combine: null argument");
    VRB_REQUIRE(terms >= 1 && terms <= kMaxTerms, VRB_ERR_INVALID, "linear combine arity mismatch");
    VRB_REQUIRE(count > 0, VRB_ERR_INVALID, "linear_combine: empty tensor");
    VRB_REQUIRE(is_float_dtype(dtype), VRB_ERR_UNSUPPORTED, "linear_combine: dtype must be F32 or BF16");
    CombineParams q{};
    bool vec = vec8_ok(count, {out});
    for (int t = 0; t < terms; ++t) {
        VRB_REQUIRE(values[t], VRB_ERR_INVALID, "linear_combine: null tensor");
        q.value[t] = values[t];
        q.coefficient[t] = coefficients[t];
        vec = vec && aligned16(values[t]);
    }
    q.out = out; q.terms = terms; q.dt = dtype; q.role = scalar_role ? 1 : 0;
    cudaStream_t s = as_stream(stream);
    if (vec) {
        const int64_t chunks = count / 8;
        linear_combine_kernel<true><<<grid_for((chunks + kThreads - 1) / kThreads, kPerSm), kThreads, 0, s>>>(q, chunks);
    } else {
        linear_combine_kernel<false><<<grid_for((count + kThreads - 1) / kThreads, kPerSm), kThreads, 0, s>>>(q, count);
    }
    return after_launch("linear_combine");
}

extern "C" int vrb_cast(const void* src, int src_dtype, void* dst, int dst_dtype, int64_t count, vrb_stream stream) {
    if (src_dtype == VRB_U8) {
        VRB_REQUIRE(src && dst && count > 0, VRB_ERR_INVALID, "cast: null tensor or empty");
        VRB_REQUIRE(is_float_dtype(dst_dtype), VRB_ERR_UNSUPPORTED, "Unsupported CUDA dtype conversion");
        cast_u8_kernel<<<grid_for((count + kThreads - 1) / kThreads, kPerSm), kThreads, 0, as_stream(stream)>>>(
            static_cast<const uint8_t*>(src), dst, dst_dtype, count);
        return after_launch("cast");
    }
    return launch_unary<kCast>(src, src_dtype, dst, dst_dtype, count, 0.f, 0.f, as_stream(stream), "cast");
}

extern "C" int vrb_activation(int kind, const void* x, void* out, int dtype, int64_t count, vrb_stream stream) {
    cudaStream_t s = as_stream(stream);
    switch (kind) {
        case VRB_SILU: return launch_unary<kActSilu>(x, dtype, out, dtype, count, 0.f, 0.f, s, "activation");
        case VRB_GELU: return launch_unary<kActGelu>(x, dtype, out, dtype, count, 0.f, 0.f, s, "activation");
        case VRB_GELU_TANH: return launch_unary<kActGeluTanh>(x, dtype, out, dtype, count, 0.f, 0.f, s, "activation");
        case VRB_TANH: return launch_unary<kActTanh>(x, dtype, out, dtype, count, 0.f, 0.f, s, "activation");
        case VRB_RELU: return launch_unary<kActRelu>(x, dtype, out, dtype, count, 0.f, 0.f, s, "activation");
        default: set_error("activation: unknown kind %d", kind); return VRB_ERR_INVALID;
    }
}
extern "C" int vrb_clamp(const void* x, void* out, int dtype, int64_t count, float minimum, float maximum, vrb_stream stream) {
    VRB_REQUIRE(minimum <= maximum, VRB_ERR_INVALID, "Invalid clamp bounds");
    return launch_unary<kClamp>(x, dtype, out, dtype, count, minimum, maximum, as_stream(stream), "clamp");
}
extern "C" int vrb_exp(const void* x, void* out, int dtype, int64_t count, vrb_stream stream) {
    return launch_unary<kExp>(x, dtype, out, dtype, count, 0.f, 0.f, as_stream(stream), "exp");
}
extern "C" int vrb_sqrt(const void* x, void* out, int dtype, int64_t count, vrb_stream stream) {
    return launch_unary<kSqrt>(x, dtype, out, dtype, count, 0.f, 0.f, as_stream(stream), "sqrt");
}

extern "C" int vrb_binary(int kind, const void* a, const int64_t* a_shape, int a_rank,
                          const void* b, const int64_t* b_shape, int b_rank,
                          void* out, int dtype, vrb_stream stream) {
    VRB_REQUIRE(a && b && out, VRB_ERR_INVALID, "binary: null tensor");
    VRB_REQUIRE(a_rank >= 0 && b_rank >= 0 && a_rank <= 8 && b_rank <= 8, VRB_ERR_INVALID, "CUDA primitive rank exceeds 8");
    VRB_REQUIRE((a_rank == 0 || a_shape) && (b_rank == 0 || b_shape), VRB_ERR_INVALID, "binary: null shape");
    VRB_REQUIRE(is_float_dtype(dtype), VRB_ERR_UNSUPPORTED, "binary: dtype must be F32 or BF16");
    const int rank = a_rank > b_rank ? a_rank : b_rank;
    int64_t oshape[8];
    int64_t count = 1;
    for (int i = 0; i < rank; ++i) {
        const int ai = i - (rank - a_rank), bi = i - (rank - b_rank);
        const int64_t av = ai < 0 ? 1 : a_shape[ai], bv = bi < 0 ? 1 : b_shape[bi];
        VRB_REQUIRE(av > 0 && bv > 0, VRB_ERR_INVALID, "binary: extents must be positive");
        VRB_REQUIRE(av == bv || av == 1 || bv == 1, VRB_ERR_INVALID, "Incompatible broadcast shapes");
        oshape[i] = av > bv ? av : bv;
        count *= oshape[i];
    }
    const Meta om = make_meta(oshape, rank), am = make_meta(a_shape, a_rank), bm = make_meta(b_shape, b_rank);
    cudaStream_t s = as_stream(stream);
    switch (kind) {
        case VRB_ADD: return launch_binary<VRB_ADD>(a, am, b, bm, out, om, count, dtype, s);
        case VRB_MUL: return launch_binary<VRB_MUL>(a, am, b, bm, out, om, count, dtype, s);
        case VRB_DIV: return launch_binary<VRB_DIV>(a, am, b, bm, out, om, count, dtype, s);
        case VRB_MAX: return launch_binary<VRB_MAX>(a, am, b, bm, out, om, count, dtype, s);
        default: set_error("binary: unknown kind %d", kind); return VRB_ERR_INVALID;
    }
}

extern "C" int vrb_swiglu(const void* projected, void* out, int dtype, int64_t rows, int64_t hidden, vrb_stream stream) {
    VRB_REQUIRE(projected && out, VRB_ERR_INVALID, "swiglu: null tensor");
    VRB_REQUIRE(rows > 0 && hidden > 0, VRB_ERR_INVALID, "swiglu: extents must be positive");
    VRB_REQUIRE(is_float_dtype(dtype), VRB_ERR_UNSUPPORTED, "swiglu: dtype must be F32 or BF16");
    if (dtype == VRB_BF16 && hidden % 8 == 0 && aligned16(projected) && aligned16(out) && rows * hidden >= kLutMinElements)
        return launch_swiglu_lut(projected, out, rows, hidden, as_stream(stream));
    if (hidden % 8 == 0 && aligned16(projected) && aligned16(out)) {
        const int64_t work = rows * (hidden / 8);
        swiglu_kernel<<<grid_for((work + kThreads - 1) / kThreads, kPerSm), kThreads, 0, as_stream(stream)>>>(
            projected, out, dtype, rows, hidden / 8);
    } else {
        const int64_t work = rows * hidden;
        swiglu_scalar_kernel<<<grid_for((work + kThreads - 1) / kThreads, kPerSm), kThreads, 0, as_stream(stream)>>>(
            projected, out, dtype, rows, hidden);
    }
    return after_launch("swiglu");
}

extern "C" int vrb_gated_residual(const void* residual, int residual_dtype, const void* branch, int branch_dtype,
                                  const void* gate, int gate_dtype, int64_t rows_per_vector, int64_t gate_vectors,
                                  void* out, int state_dtype, int64_t rows, int64_t width, vrb_stream stream) {
    VRB_REQUIRE(residual && branch && out, VRB_ERR_INVALID, "gated_residual: null tensor");
    VRB_REQUIRE(rows > 0 && width > 0, VRB_ERR_INVALID, "gated_residual: extents must be positive");
    VRB_REQUIRE(!gate || (rows_per_vector > 0 && gate_vectors > 0), VRB_ERR_INVALID,
                "gated_residual: rows_per_vector and vector count must be positive");
    VRB_REQUIRE(is_float_dtype(residual_dtype) && is_float_dtype(branch_dtype) && is_float_dtype(state_dtype) &&
                (!gate || is_float_dtype(gate_dtype)), VRB_ERR_UNSUPPORTED, "gated_residual: dtypes must be F32 or BF16");
    const bool vec_ok = width % 8 == 0 && aligned16(residual) && aligned16(branch) && aligned16(out) && (!gate || aligned16(gate));
    const int64_t chunks = vec_ok ? rows * (width / 8) : 0;
    if (vec_ok && chunks < (int64_t{1} << 31) && rows_per_vector < (int64_t{1} << 31) && gate_vectors < (int64_t{1} << 31)) {
        const int grid = grid_for((chunks + kThreads - 1) / kThreads, kPerSm);
        const unsigned total = static_cast<unsigned>(chunks), wc = static_cast<unsigned>(width / 8);
        const unsigned rpv = static_cast<unsigned>(gate ? rows_per_vector : 1), nv = static_cast<unsigned>(gate ? gate_vectors : 1);
        cudaStream_t s = as_stream(stream);
        const int key = (residual_dtype == VRB_BF16 ? 4 : 0) | (branch_dtype == VRB_BF16 ? 2 : 0) | (state_dtype == VRB_BF16 ? 1 : 0);
        // staged gate: worth its per-CTA prologue from 16 chunks per thread; the vectors must fit 48 KB of shared memory
        const int64_t gate_bytes = static_cast<int64_t>(nv) * wc * 16;
        if (key == 7 && gate && gate_bytes <= 48 * 1024 && chunks >= static_cast<int64_t>(grid) * kThreads * 16 &&
            static_cast<int64_t>(total) + static_cast<int64_t>(grid) * kThreads * 2 < (int64_t{1} << 32)) {
            launch_overlapped(gated_residual_staged_kernel, dim3(grid), dim3(kThreads), static_cast<size_t>(gate_bytes), s,
                              static_cast<const uint4*>(residual), static_cast<const uint4*>(branch), gate, gate_dtype,
                              static_cast<uint4*>(out), total, wc, rpv, nv);
            return after_launch("gated_residual");
        }
#define VRB_GR(R, B, S) launch_overlapped(gated_residual_typed_kernel<R, B, S>, dim3(grid), dim3(kThreads), 0, s, residual, branch, gate, gate_dtype, out, total, wc, rpv, nv)
        switch (key) {
            case 0: VRB_GR(false, false, false); break;
            case 1: VRB_GR(false, false, true); break;
            case 2: VRB_GR(false, true, false); break;
            case 3: VRB_GR(false, true, true); break;
            case 4: VRB_GR(true, false, false); break;
            case 5: VRB_GR(true, false, true); break;
            case 6: VRB_GR(true, true, false); break;
            default: VRB_GR(true, true, true); break;
        }
#undef VRB_GR
    } else if (vec_ok) {
        const int64_t work = rows * (width / 8);
        gated_residual_kernel<<<grid_for((work + kThreads - 1) / kThreads, kPerSm), kThreads, 0, as_stream(stream)>>>(
            residual, residual_dtype, branch, branch_dtype, gate, gate_dtype, out, state_dtype, rows, width / 8,
            rows_per_vector, gate_vectors);
    } else {
        const int64_t work = rows * width;
        gated_residual_scalar_kernel<<<grid_for((work + kThreads - 1) / kThreads, kPerSm), kThreads, 0, as_stream(stream)>>>(
            residual, residual_dtype, branch, branch_dtype, gate, gate_dtype, out, state_dtype, rows, width,
            rows_per_vector, gate_vectors);
    }
    return after_launch("gated_residual");
}

extern "C" int vrb_rope(const void* x, int x_dtype, const int64_t* x_shape, int x_rank,
                        const void* cosine, const void* sine, int f_dtype, const int64_t* f_shape, int f_rank,
                        void* out, vrb_stream stream) {
    VRB_REQUIRE(x && cosine && sine && out && x_shape && f_shape, VRB_ERR_INVALID, "rope: null tensor");
    VRB_REQUIRE(x_rank >= 1 && x_rank <= 8 && f_rank >= 0 && f_rank <= x_rank, VRB_ERR_INVALID, "CUDA primitive rank exceeds 8");
    VRB_REQUIRE(is_float_dtype(x_dtype) && is_float_dtype(f_dtype), VRB_ERR_UNSUPPORTED, "rope: dtypes must be F32 or BF16");
    VRB_REQUIRE(x_shape[x_rank - 1] % 2 == 0, VRB_ERR_INVALID, "RoPE width must be even");
    int64_t count = 1;
    for (int d = 0; d < x_rank; ++d) { VRB_REQUIRE(x_shape[d] > 0, VRB_ERR_INVALID, "rope: extents must be positive"); count *= x_shape[d]; }
    for (int d = 0; d < f_rank; ++d) {
        const int64_t xv = x_shape[d + (x_rank - f_rank)];
        VRB_REQUIRE(f_shape[d] == xv || f_shape[d] == 1, VRB_ERR_INVALID, "Incompatible broadcast shapes");
    }
    const Meta xm = make_meta(x_shape, x_rank), fm = make_meta(f_shape, f_rank);
    const int64_t width = x_shape[x_rank - 1];
    // Fast layouts (after dropping the table's leading broadcast axes): the table equals x's
    // trailing axes, or it is [T.., 1, W] against x's [T.., H, W].
    bool fast = width % 8 == 0 && aligned16(x) && aligned16(out) && aligned16(cosine) && aligned16(sine) &&
                f_rank >= 1 && f_shape[f_rank - 1] == width;
    int64_t heads = 0, f_tokens = 1, period = 1;
    if (fast) {
        const int shift = x_rank - f_rank;
        int first = 0;
        while (first < f_rank - 1 && f_shape[first] == 1) ++first;
        bool same = true;
        for (int k = first; k < f_rank; ++k) { same = same && f_shape[k] == x_shape[k + shift]; period *= f_shape[k]; }
        if (!same) {
            const int h = f_rank - 2;
            bool shared = h >= first && f_shape[h] == 1;
            for (int k = first; shared && k < h; ++k) { shared = f_shape[k] == x_shape[k + shift]; f_tokens *= f_shape[k]; }
            if (shared) heads = x_shape[h + shift];
            else fast = false;
        }
    }
    cudaStream_t s = as_stream(stream);
    if (fast) {
        const int64_t chunks = count / 8;
        rope_vec_kernel<<<grid_for((chunks + kThreads - 1) / kThreads, kPerSm), kThreads, 0, s>>>(
            x, x_dtype, cosine, sine, f_dtype, out, chunks, width, heads, f_tokens, period);
    } else {
        rope_general_kernel<<<grid_for((count + kThreads - 1) / kThreads, kPerSm), kThreads, 0, s>>>(
            x, x_dtype, cosine, sine, f_dtype, out, count, xm, fm);
    }
    return after_launch("rope");
}

extern "C" int vrb_dequantize(int kind, const void* packed, const float* scales, void* out, int out_dtype,
                              int64_t rows, int64_t inner, int64_t group_size, vrb_stream stream) {
    VRB_REQUIRE(packed && scales && out, VRB_ERR_INVALID, "dequantize: null tensor");
    VRB_REQUIRE(rows > 0 && inner > 0 && group_size > 0, VRB_ERR_INVALID, "Unsupported quantized tensor layout/policy");
    VRB_REQUIRE(is_float_dtype(out_dtype), VRB_ERR_UNSUPPORTED, "Quantized tensors require CPU storage and float compute output");
    VRB_REQUIRE(kind >= 0 && kind <= 2, VRB_ERR_UNSUPPORTED, "Unsupported quantized tensor packing");
    const int64_t count = rows * inner, groups = (inner + group_size - 1) / group_size;
    const uint8_t* p = static_cast<const uint8_t*>(packed);
    cudaStream_t s = as_stream(stream);
    const bool vec = kind != VRB_Q_INT4 && inner % 16 == 0 && group_size % 16 == 0 && rows * (inner / 16) < 0xffffffffLL &&
                     groups * rows < 0xffffffffLL && aligned16(packed) && aligned16(out);
    const bool vec4 = kind == VRB_Q_INT4 && inner % 32 == 0 && group_size % 32 == 0 && inner / 32 < 0x7fffffff &&
                      aligned16(packed) && aligned16(out);
    if (vec4) {
        launch_dequant_int4_tiles(p, scales, out, out_dtype, rows, inner, groups, group_size, s);
    } else if (vec) {
        if (kind == VRB_Q_FP8_E4M3FN) launch_dequant_tiles<VRB_Q_FP8_E4M3FN>(p, scales, out, out_dtype, rows, inner, groups, group_size, s);
        else launch_dequant_tiles<VRB_Q_INT8>(p, scales, out, out_dtype, rows, inner, groups, group_size, s);
    } else {
        const int grid = grid_for((count + kThreads - 1) / kThreads, kPerSm);
        if (kind == VRB_Q_FP8_E4M3FN) dequant_scalar_kernel<VRB_Q_FP8_E4M3FN><<<grid, kThreads, 0, s>>>(p, scales, out, out_dtype, count, inner, groups, group_size);
        else if (kind == VRB_Q_INT8) dequant_scalar_kernel<VRB_Q_INT8><<<grid, kThreads, 0, s>>>(p, scales, out, out_dtype, count, inner, groups, group_size);
        else dequant_scalar_kernel<VRB_Q_INT4><<<grid, kThreads, 0, s>>>(p, scales, out, out_dtype, count, inner, groups, group_size);
    }
    return after_launch("dequantize");
}

extern "C" int vrb_cfg_combine(const void* unconditional, const void* conditional, void* out, int dtype,
                               int64_t count, float scale, int scalar_role, vrb_stream stream) {
    VRB_REQUIRE(unconditional && conditional, VRB_ERR_INVALID, "cfg_combine: null tensor");
    SamplerParams q{}; q.uncond = unconditional; q.cond = conditional; q.out = out; q.dt = dtype;
    q.role = scalar_role; q.mode = 0; q.scale = scale;
    return launch_sampler(q, count, as_stream(stream), "cfg_combine");
}
extern "C" int vrb_euler_update(const void* sample, const void* prediction, void* out, int dtype,
                                int64_t count, float delta, int subtract_prediction, int scalar_role, vrb_stream stream) {
    VRB_REQUIRE(sample && prediction, VRB_ERR_INVALID, "euler_update: null tensor");
    SamplerParams q{}; q.sample = sample; q.uncond = prediction; q.out = out; q.dt = dtype;
    q.axpy_role = scalar_role; q.mode = 1; q.coefficient = euler_coefficient(delta, subtract_prediction);
    return launch_sampler(q, count, as_stream(stream), "euler_update");
}
extern "C" int vrb_flow_to_x0(const void* sample, const void* model_output, void* out, int dtype,
                              int64_t count, float sigma, int scalar_role, vrb_stream stream) {
    VRB_REQUIRE(sample && model_output, VRB_ERR_INVALID, "flow_to_x0: null tensor");
    SamplerParams q{}; q.sample = sample; q.uncond = model_output; q.out = out; q.dt = dtype;
    q.axpy_role = scalar_role; q.mode = 3; q.coefficient = -sigma;
    return launch_sampler(q, count, as_stream(stream), "flow_to_x0");
}
extern "C" int vrb_cfg_euler(const void* sample, const void* unconditional, const void* conditional,
                             void* guided, void* out, int dtype, int64_t count, float scale, float delta,
                             int subtract_prediction, int guidance_role, int solver_role, vrb_stream stream) {
    VRB_REQUIRE(sample && unconditional && conditional, VRB_ERR_INVALID, "cfg_euler: null tensor");
    SamplerParams q{}; q.sample = sample; q.uncond = unconditional; q.cond = conditional; q.guided = guided; q.out = out;
    q.dt = dtype; q.role = guidance_role; q.axpy_role = solver_role; q.mode = 2; q.scale = scale;
    q.coefficient = euler_coefficient(delta, subtract_prediction);
    return launch_sampler(q, count, as_stream(stream), "cfg_euler");
}
