// The epilogue of the reference's bf16 linear and the operator that consumes its result.
//
// CudaBackend::linear (native/src/backend/cuda/cuda_backend.cu:3661-3866) runs the GEMM into an
// F32 accumulation buffer and then fused_bf16_linear_output_kernel (:754-764; call sites :3831
// and :3846): out = bf16(accumulation + float(bf16 bias)), one F32 add and one RNE rounding.  In
// the DiT blocks that bf16 tensor is read back at once by an activation (wan.cpp:109-112), a gated
// residual (wan.cpp:114-116), or SwiGLU (mochi.cpp:195-202).  The kernels here read the F32
// accumulation once and write the consumer's result: the rounded linear output never goes to
// memory, and every intermediate rounding of the separate kernels is kept, so results are
// bit-identical to epilogue kernel + consumer kernel.
//
//   follow none        : 4 B read + 2 B written per element (the reference's kernel)
//   activation         : 4 + 2 instead of (4 + 2) + (2 + 2)
//   gated residual     : 4 + residual + state instead of (4 + 2) + (2 + residual + state)
//   SwiGLU             : 8 + 2 per output element instead of (8 + 4) + (4 + 4 + ...) of split/silu/mul
//
// Large activation / SwiGLU launches read the activation from the 65536-entry function table of
// vrb_lut.cu (the value fed to the activation is a bf16 value); smaller ones evaluate it.
#include "vrb_common.cuh"

namespace vrb {
namespace {

constexpr int kThreads = 256;
constexpr int kPerSm = 8;

enum Follow { kFollowNone = 0, kFollowActivation = 1, kFollowGated = 2, kFollowSwiglu = 3 };

struct LinearOutputParams {
    const float* accumulation;
    const uint16_t* bias;      // bf16 [width] or nullptr
    void* out;
    int64_t rows, width;       // of the accumulation
    int kind;                  // activation kind
    const void* residual;      // gated residual
    const void* gate;
    int residual_dt, gate_dt, state_dt;
    int64_t rows_per_vector, vectors;
};

// bf16(accumulation + bias) for 8 consecutive columns, as F32 values on the bf16 grid
__device__ __forceinline__ void linear_value8(const LinearOutputParams& p, int64_t row, int64_t column, float (&v)[8]) {
    load8<true>(p.accumulation, VRB_F32, row * p.width + column, v);
    if (p.bias != nullptr) {
        float b[8];
        load8<false>(p.bias, VRB_BF16, column, b);
#pragma unroll
        for (int e = 0; e < 8; ++e) v[e] = __fadd_rn(v[e], b[e]);
    }
    round8_bf16_inplace(v);
}

// Vector kernel: width % 8 == 0 (SwiGLU: hidden % 8 == 0), 16-byte aligned operands.
template <int FOLLOW>
__global__ void __launch_bounds__(kThreads) linear_output_kernel(const LinearOutputParams p) {
    constexpr int U = 2;
    const int64_t out_width = FOLLOW == kFollowSwiglu ? p.width / 2 : p.width;
    const int64_t width_chunks = out_width / 8;
    const int64_t total = p.rows * width_chunks;
    const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
    for (int64_t i0 = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i0 < total; i0 += stride * U) {
        float v[U][8], w[U][8], g[U][8];
        int64_t row[U], column[U];
#pragma unroll
        for (int u = 0; u < U; ++u) {
            const int64_t i = i0 + u * stride;
            if (i >= total) break;
            row[u] = i / width_chunks;
            column[u] = (i - row[u] * width_chunks) * 8;
            linear_value8(p, row[u], column[u], v[u]);
            if constexpr (FOLLOW == kFollowSwiglu) linear_value8(p, row[u], out_width + column[u], w[u]);
            if constexpr (FOLLOW == kFollowGated) {
                load8<true>(p.residual, p.residual_dt, i * 8, w[u]);
                if (p.gate != nullptr) {
                    const int64_t vec = p.vectors > 1 ? (row[u] / p.rows_per_vector) % p.vectors : 0;
                    load8<false>(p.gate, p.gate_dt, vec * out_width + column[u], g[u]);
                }
            }
        }
#pragma unroll
        for (int u = 0; u < U; ++u) {
            const int64_t i = i0 + u * stride;
            if (i >= total) break;
            if constexpr (FOLLOW == kFollowNone) {
                store8(p.out, VRB_BF16, i * 8, v[u]);
            } else if constexpr (FOLLOW == kFollowActivation) {
#pragma unroll
                for (int e = 0; e < 8; ++e) v[u][e] = activation_value(p.kind, v[u][e]);
                store8(p.out, VRB_BF16, i * 8, v[u]);
            } else if constexpr (FOLLOW == kFollowSwiglu) {
                // value half * bf16(silu(gate half)), mochi.cpp:195-202
#pragma unroll
                for (int e = 0; e < 8; ++e) v[u][e] = __fmul_rn(v[u][e], round_to_bf16(activation_value(VRB_SILU, w[u][e])));
                store8(p.out, VRB_BF16, i * 8, v[u]);
            } else {
                // common.cpp:134-144 with T = state dtype; the branch is the bf16 linear output
                const bool narrow = p.state_dt == VRB_BF16;
                if (narrow) round8_bf16_inplace(w[u]);
                if (p.gate != nullptr) {
                    if (narrow) round8_bf16_inplace(g[u]);
#pragma unroll
                    for (int e = 0; e < 8; ++e) v[u][e] = __fmul_rn(v[u][e], g[u][e]);
                    if (narrow) round8_bf16_inplace(v[u]);
                }
#pragma unroll
                for (int e = 0; e < 8; ++e) w[u][e] = __fadd_rn(w[u][e], v[u][e]);
                store8(p.out, p.state_dt, i * 8, w[u]);
            }
        }
    }
}

// The gated-residual form with the tensor dtypes fixed at compile time and 32-bit indexing (fewer
// than 2^31 chunks): same arithmetic as the kernel above.
template <bool RES_BF16, bool STATE_BF16>
__global__ void __launch_bounds__(kThreads) linear_output_gated_typed_kernel(
        const float4* __restrict__ accumulation, const uint4* __restrict__ bias, const void* __restrict__ residual,
        const void* __restrict__ gate, int gate_dt, void* __restrict__ out, unsigned total, unsigned width_chunks,
        unsigned rows_per_vector, unsigned vectors) {
        // work items per thread and iteration, measured: with a bf16 stream one item (four to five 16-byte loads
    // in flight already) beats two by 15 %; with an F32 stream two items beat one by 7 %
    constexpr int U = (RES_BF16 && STATE_BF16) ? 1 : 2;
    const unsigned stride = gridDim.x * blockDim.x;
    const bool has_bias = bias != nullptr, has_gate = gate != nullptr;
    for (unsigned i0 = blockIdx.x * blockDim.x + threadIdx.x; i0 < total; i0 += stride * U) {
        float4 a[U][2];
        uint4 b[U];
        float r[U][8], g[U][8];
#pragma unroll
        for (int u = 0; u < U; ++u) {
            const unsigned i = i0 + u * stride;
            if (i >= total) break;
            a[u][0] = __ldcs(accumulation + 2 * static_cast<int64_t>(i));
            a[u][1] = __ldcs(accumulation + 2 * static_cast<int64_t>(i) + 1);
            load8<true>(residual, RES_BF16 ? VRB_BF16 : VRB_F32, static_cast<int64_t>(i) * 8, r[u]);
            const unsigned row = i / width_chunks, chunk = i - row * width_chunks;
            if (has_bias) b[u] = __ldg(bias + chunk);
            if (has_gate) {
                const unsigned vec = vectors > 1 ? (row / rows_per_vector) % vectors : 0;
                load8<false>(gate, gate_dt, (static_cast<int64_t>(vec) * width_chunks + chunk) * 8, g[u]);
            }
        }
#pragma unroll
        for (int u = 0; u < U; ++u) {
            const unsigned i = i0 + u * stride;
            if (i >= total) break;
            float v[8] = {a[u][0].x, a[u][0].y, a[u][0].z, a[u][0].w, a[u][1].x, a[u][1].y, a[u][1].z, a[u][1].w};
            if (has_bias) {
                const uint32_t bw[4] = {b[u].x, b[u].y, b[u].z, b[u].w};
#pragma unroll
                for (int k = 0; k < 4; ++k) {
                    v[2 * k] = __fadd_rn(v[2 * k], __uint_as_float(bw[k] << 16));
                    v[2 * k + 1] = __fadd_rn(v[2 * k + 1], __uint_as_float(bw[k] & 0xffff0000u));
                }
            }
            round8_bf16_inplace(v);                           // the linear output
            if constexpr (STATE_BF16) {
                if constexpr (!RES_BF16) round8_bf16_inplace(r[u]);
                if (has_gate) {
                    round8_bf16_inplace(g[u]);
#pragma unroll
                    for (int e = 0; e < 8; ++e) v[e] = __fmul_rn(v[e], g[u][e]);
                    round8_bf16_inplace(v);
                }
            } else if (has_gate) {
#pragma unroll
                for (int e = 0; e < 8; ++e) v[e] = __fmul_rn(v[e], g[u][e]);
            }
#pragma unroll
            for (int e = 0; e < 8; ++e) r[u][e] = __fadd_rn(r[u][e], v[e]);
            store8(out, STATE_BF16 ? VRB_BF16 : VRB_F32, static_cast<int64_t>(i) * 8, r[u]);
        }
    }
}

// Any width / alignment.
template <int FOLLOW>
__global__ void __launch_bounds__(kThreads) linear_output_scalar_kernel(const LinearOutputParams p) {
    const int64_t out_width = FOLLOW == kFollowSwiglu ? p.width / 2 : p.width;
    const int64_t total = p.rows * out_width;
    const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
    auto value = [&](int64_t row, int64_t column) {
        float a = p.accumulation[row * p.width + column];
        if (p.bias != nullptr) a = __fadd_rn(a, bf16_bits_to_float(p.bias[column]));
        return round_to_bf16(a);
    };
    for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < total; i += stride) {
        const int64_t row = i / out_width, column = i - row * out_width;
        float v = value(row, column);
        if constexpr (FOLLOW == kFollowNone) {
            store1(p.out, VRB_BF16, i, v);
        } else if constexpr (FOLLOW == kFollowActivation) {
            store1(p.out, VRB_BF16, i, activation_value(p.kind, v));
        } else if constexpr (FOLLOW == kFollowSwiglu) {
            store1(p.out, VRB_BF16, i, __fmul_rn(v, round_to_bf16(activation_value(VRB_SILU, value(row, out_width + column)))));
        } else {
            if (p.gate != nullptr) {
                const int64_t vec = (row / p.rows_per_vector) % p.vectors;
                v = round_to(p.state_dt, __fmul_rn(v, round_to(p.state_dt, load1(p.gate, p.gate_dt, vec * out_width + column))));
            }
            store1(p.out, p.state_dt, i, __fadd_rn(round_to(p.state_dt, load1(p.residual, p.residual_dt, i)), v));
        }
    }
}

template <int FOLLOW>
int launch(const LinearOutputParams& p, bool vector_ok, cudaStream_t stream, const char* what) {
    const int64_t out_width = FOLLOW == kFollowSwiglu ? p.width / 2 : p.width;
    if (vector_ok) {
        const int64_t work = p.rows * (out_width / 8);
        linear_output_kernel<FOLLOW><<<grid_for((work + kThreads - 1) / kThreads, kPerSm), kThreads, 0, stream>>>(p);
    } else {
        const int64_t work = p.rows * out_width;
        linear_output_scalar_kernel<FOLLOW><<<grid_for((work + kThreads - 1) / kThreads, kPerSm), kThreads, 0, stream>>>(p);
    }
    return after_launch(what);
}

int check_common(const void* accumulation, const void* out, int64_t rows, int64_t width, const char* what) {
    VRB_REQUIRE(accumulation && out, VRB_ERR_INVALID, "%s: null tensor", what);
    VRB_REQUIRE(rows > 0 && width > 0, VRB_ERR_INVALID, "%s: extents must be positive", what);
    VRB_REQUIRE((reinterpret_cast<uintptr_t>(accumulation) & 3u) == 0, VRB_ERR_INVALID, "%s: misaligned accumulation", what);
    return VRB_OK;
}

}  // namespace
}  // namespace vrb

using namespace vrb;

extern "C" int vrb_linear_output(const float* accumulation, const void* bias, void* out, int64_t rows, int64_t width,
                                 vrb_stream stream) {
    if (int rc = check_common(accumulation, out, rows, width, "linear_output")) return rc;
    LinearOutputParams p{};
    p.accumulation = accumulation; p.bias = static_cast<const uint16_t*>(bias); p.out = out; p.rows = rows; p.width = width;
    const bool vector_ok = width % 8 == 0 && aligned16(accumulation) && aligned16(out) && (!bias || aligned16(bias));
    return launch<kFollowNone>(p, vector_ok, as_stream(stream), "linear_output");
}

extern "C" int vrb_linear_output_activation(const float* accumulation, const void* bias, int kind, void* out, int64_t rows,
                                            int64_t width, vrb_stream stream) {
    if (int rc = check_common(accumulation, out, rows, width, "linear_output_activation")) return rc;
    VRB_REQUIRE(kind >= VRB_SILU && kind <= VRB_RELU, VRB_ERR_INVALID, "linear_output_activation: unknown activation kind %d", kind);
    const bool vector_ok = width % 8 == 0 && aligned16(accumulation) && aligned16(out) && (!bias || aligned16(bias));
    if (vector_ok && rows * width >= kLutMinElements && rows * (width / 8) < (int64_t{1} << 32))
        return launch_linear_output_lut(kind, accumulation, bias, out, rows, width, as_stream(stream));
    LinearOutputParams p{};
    p.accumulation = accumulation; p.bias = static_cast<const uint16_t*>(bias); p.out = out; p.rows = rows; p.width = width;
    p.kind = kind;
    return launch<kFollowActivation>(p, vector_ok, as_stream(stream), "linear_output_activation");
}

extern "C" int vrb_linear_output_gated_residual(const float* accumulation, const void* bias, const void* residual,
                                                int residual_dtype, const void* gate, int gate_dtype,
                                                int64_t rows_per_vector, int64_t gate_vectors, void* out, int state_dtype,
                                                int64_t rows, int64_t width, vrb_stream stream) {
    if (int rc = check_common(accumulation, out, rows, width, "linear_output_gated_residual")) return rc;
    VRB_REQUIRE(residual, VRB_ERR_INVALID, "linear_output_gated_residual: null tensor");
    VRB_REQUIRE(!gate || (rows_per_vector > 0 && gate_vectors > 0), VRB_ERR_INVALID,
                "linear_output_gated_residual: rows_per_vector and vector count must be positive");
    VRB_REQUIRE(is_float_dtype(residual_dtype) && is_float_dtype(state_dtype) && (!gate || is_float_dtype(gate_dtype)),
                VRB_ERR_UNSUPPORTED, "linear_output_gated_residual: dtypes must be F32 or BF16");
    LinearOutputParams p{};
    p.accumulation = accumulation; p.bias = static_cast<const uint16_t*>(bias); p.out = out; p.rows = rows; p.width = width;
    p.residual = residual; p.gate = gate; p.residual_dt = residual_dtype; p.gate_dt = gate_dtype; p.state_dt = state_dtype;
    p.rows_per_vector = gate ? rows_per_vector : 1; p.vectors = gate ? gate_vectors : 1;
    const bool vector_ok = width % 8 == 0 && aligned16(accumulation) && aligned16(out) && (!bias || aligned16(bias)) &&
                           aligned16(residual) && (!gate || aligned16(gate));
    const int64_t chunks = vector_ok ? rows * (width / 8) : 0;
    if (vector_ok && chunks < (int64_t{1} << 31) && p.rows_per_vector < (int64_t{1} << 31) && p.vectors < (int64_t{1} << 31)) {
        const int grid = grid_for((chunks + kThreads - 1) / kThreads, kPerSm);
        cudaStream_t s = as_stream(stream);
#define VRB_LG(R, S) linear_output_gated_typed_kernel<R, S><<<grid, kThreads, 0, s>>>(                                  \
        reinterpret_cast<const float4*>(accumulation), static_cast<const uint4*>(bias), residual, gate, gate_dtype, out, \
        static_cast<unsigned>(chunks), static_cast<unsigned>(width / 8), static_cast<unsigned>(p.rows_per_vector),       \
        static_cast<unsigned>(p.vectors))
        if (residual_dtype == VRB_BF16) { if (state_dtype == VRB_BF16) VRB_LG(true, true); else VRB_LG(true, false); }
        else { if (state_dtype == VRB_BF16) VRB_LG(false, true); else VRB_LG(false, false); }
#undef VRB_LG
        return after_launch("linear_output_gated_residual");
    }
    return launch<kFollowGated>(p, vector_ok, as_stream(stream), "linear_output_gated_residual");
}

extern "C" int vrb_linear_output_swiglu(const float* accumulation, const void* bias, void* out, int64_t rows, int64_t hidden,
                                        vrb_stream stream) {
    if (int rc = check_common(accumulation, out, rows, hidden, "linear_output_swiglu")) return rc;
    const bool vector_ok = hidden % 8 == 0 && aligned16(accumulation) && aligned16(out) && (!bias || aligned16(bias));
    if (vector_ok && rows * hidden >= kLutMinElements && rows * (hidden / 8) < (int64_t{1} << 32))
        return launch_linear_output_swiglu_lut(accumulation, bias, out, rows, hidden, as_stream(stream));
    LinearOutputParams p{};
    p.accumulation = accumulation; p.bias = static_cast<const uint16_t*>(bias); p.out = out; p.rows = rows; p.width = 2 * hidden;
    return launch<kFollowSwiglu>(p, vector_ok, as_stream(stream), "linear_output_swiglu");
}
