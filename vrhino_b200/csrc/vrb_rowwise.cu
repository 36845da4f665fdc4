// Row-wise normalisation kernels (LayerNorm / RMSNorm) fused with the operator that the
// reference's pipelines apply next: adaLN modulation, the Mochi (1+scale) product, RoPE, or
// a gated residual.  One kernel family, one pass over HBM: a row is loaded once with 128-bit
// loads, kept in registers while its statistics are reduced (warp shuffles, plus one shared-
// memory exchange when a row spans several warps), then normalised, post-processed and
// stored.  Every rounding the reference's chain of separate kernels performs between its
// steps is reproduced in registers.
//
// Reference semantics restated here (native/src/backend/cuda/cuda_backend.cu):
//   layer_norm_parallel_kernel :910-943  double sum / sum of squares, mean = float(S/W),
//       inv = rsqrtf(float(Q/W - double(mean)*mean) + eps), (x-mean)*inv [*w] [+b]
//   rms_norm_contiguous_f32_kernel :853-907  F32 sum of squares, mean = S*(1/W),
//       inv = rsqrtf(mean+eps), x*inv, round to bf16 if the input is bf16, *w
//   rms_norm_parallel_kernel :963-991 (and :1013-1040)  same with a double sum and
//       inv = rsqrtf(float(Q/W) + eps); chosen by rms_contiguous_reduction_lanes :838-850
//   rope_kernel :1200-1215, modulate / gated_residual: native/src/architectures/common.cpp
#include "vrb_common.cuh"

namespace vrb {
namespace {

enum Norm { kNormLayer = 1, kNormRmsF32 = 2, kNormRmsF64 = 3 };
enum Post { kPostNone = 0, kPostModulate = 1, kPostScaleX = 2, kPostRope = 3, kPostGatedResidual = 4 };

struct RowParams {
    const void* x; void* out;
    const void* weight; const void* bias;
    const void* scale; const void* shift;
    const void* cosine; const void* sine;
    const void* residual; const void* gate;
    int64_t rows, width;       // storage rows
    int64_t norm_width;        // normalised extent, divides width
    int64_t rows_per_vector, vectors;            // scale / shift / gate row selection
    int64_t f_rows, f_width, rows_per_f_row;     // cos / sin table selection
    float eps;
    int x_dt, out_dt, w_dt, b_dt, mod_dt, f_dt, res_dt, gate_dt, state_dt;
    int norm, norm_out_dt, post, affine_fma;
    int tpr;                   // threads cooperating on one normalised row (power of two)
};

constexpr int kRowThreads = 256;

// The reference's choice between the F32-accumulating and the double-accumulating RMS
// kernels depends on the row width and the row count (launch-geometry rule of
// rms_contiguous_reduction_lanes).  Returns true when the F32 kernel would run.
bool rms_uses_f32_accumulation(int64_t width, int64_t rows) {
    if (width <= 0 || rows <= 0) return false;
    if (width > 128 && (width & 3)) return false;
    const int64_t inputs = width > 128 ? width >> 2 : width;
    int64_t in_pow = 1, row_pow = 1;
    while (in_pow < 512 && in_pow * 2 <= inputs) in_pow <<= 1;
    while (row_pow < 512 && row_pow * 2 <= rows) row_pow <<= 1;
    int64_t lanes = in_pow < 32 ? in_pow : 32;
    const int64_t groups = row_pow < 512 / lanes ? row_pow : 512 / lanes;
    lanes = in_pow < 512 / groups ? in_pow : 512 / groups;
    const int64_t per_lane = (width + lanes - 1) / lanes;
    const int64_t limit = groups * 16 < 256 ? groups * 16 : 256;
    return per_lane < limit;
}

// ---- per-element pipeline shared by the vector and the scalar kernels --------------------

// Normalised value as the unfused norm operator would have stored it (dtype norm_out_dt).
__device__ __forceinline__ float normalise(const RowParams& p, float x, float mean, float inv,
                                           float w, float b) {
    float v;
    if (p.norm == kNormLayer) {
        v = __fmul_rn(__fsub_rn(x, mean), inv);
        if (p.weight && p.bias && p.affine_fma) v = __fmaf_rn(v, w, b);
        else {
            if (p.weight) v = __fmul_rn(v, w);
            if (p.bias) v = __fadd_rn(v, b);
        }
    } else {
        v = __fmul_rn(x, inv);
        if (p.x_dt == VRB_BF16) v = round_to_bf16(v);
        if (p.weight) v = __fmul_rn(v, w);
    }
    return round_to(p.norm_out_dt, v);
}

// LayerNorm converts weight and bias to x's dtype; RMSNorm converts the weight to the norm's
// output dtype (host wrappers :4069-4070, :4115).
__device__ __forceinline__ float affine_operand(const RowParams& p, float raw) {
    return round_to(p.norm == kNormLayer ? p.x_dt : p.norm_out_dt, raw);
}

__device__ __forceinline__ float post_modulate(float v, float scale, float shift, bool has_shift) {
    // common.cpp:51-61: three separately rounded F32 kernels
    const float t = __fmul_rn(v, __fadd_rn(1.0f, scale));
    return has_shift ? __fadd_rn(t, shift) : t;
}
__device__ __forceinline__ float post_scale_x(int dt, float v, float scale) {
    // mochi.cpp:230-231: (1+scale) is an F32 tensor, converted to x's dtype by the binary
    // operand rule, product rounded to x's dtype
    const float s = round_to(dt, __fadd_rn(1.0f, scale));
    return round_to(dt, __fmul_rn(v, s));
}
__device__ __forceinline__ float post_gated(int dt, float residual, float v, float gate, bool has_gate) {
    // common.cpp:134-144 in state dtype dt
    float branch = round_to(dt, v);
    if (has_gate) branch = round_to(dt, __fmul_rn(branch, round_to(dt, gate)));
    return round_to(dt, __fadd_rn(round_to(dt, residual), branch));
}

// ---- vector kernel: width % 8 == 0, 16-byte aligned operands -----------------------------
template <int NCH>
__global__ void __launch_bounds__(kRowThreads) row_kernel(const RowParams p) {
    __shared__ double s_red[2][2][kRowThreads / 32];
    const int tpr = p.tpr;
    const int lane_in_row = threadIdx.x & (tpr - 1);
    const int row_in_cta = threadIdx.x / tpr;
    const int rows_per_cta = blockDim.x / tpr;
    const int nchunks = static_cast<int>(p.norm_width >> 3);
    const int64_t sub = p.width / p.norm_width;
    const int64_t nrows = p.rows * sub;
    const int warps_per_row = tpr >> 5;
    int parity = 0;

    for (int64_t base = static_cast<int64_t>(blockIdx.x) * rows_per_cta; base < nrows;
         base += static_cast<int64_t>(gridDim.x) * rows_per_cta) {
        const int64_t nrow = base + row_in_cta;
        const bool valid = nrow < nrows;
        const int64_t row_offset = nrow * p.norm_width;

        float v[NCH][8];
#pragma unroll
        for (int i = 0; i < NCH; ++i) {
            const int chunk = lane_in_row + i * tpr;
            if (valid && chunk < nchunks) load8<true>(p.x, p.x_dt, row_offset + chunk * 8, v[i]);
            else {
#pragma unroll
                for (int e = 0; e < 8; ++e) v[i][e] = 0.0f;
            }
        }

        // ---- statistics ----
        double acc0 = 0.0, acc1 = 0.0;
        if (p.norm == kNormLayer) {
#pragma unroll
            for (int i = 0; i < NCH; ++i)
#pragma unroll
                for (int e = 0; e < 8; ++e) {
                    const double d = static_cast<double>(v[i][e]);
                    acc0 += d;
                    acc1 = fma(d, d, acc1);
                }
        } else if (p.norm == kNormRmsF64) {
#pragma unroll
            for (int i = 0; i < NCH; ++i)
#pragma unroll
                for (int e = 0; e < 8; ++e) {
                    const double d = static_cast<double>(v[i][e]);
                    acc1 = fma(d, d, acc1);
                }
        } else {
            float s = 0.0f;
#pragma unroll
            for (int i = 0; i < NCH; ++i)
#pragma unroll
                for (int e = 0; e < 8; ++e) s = __fadd_rn(s, __fmul_rn(v[i][e], v[i][e]));
            acc1 = static_cast<double>(s);  // carried as a double container; summed in F32 below
        }
        const bool f32_sum = p.norm == kNormRmsF32;
        const int span = tpr < 32 ? tpr : 32;
        for (int offset = span >> 1; offset > 0; offset >>= 1) {
            if (f32_sum) {
                const float mine = static_cast<float>(acc1);
                acc1 = static_cast<double>(__fadd_rn(mine, __shfl_xor_sync(0xffffffffu, mine, offset)));
            } else {
                acc0 += __shfl_xor_sync(0xffffffffu, acc0, offset);
                acc1 += __shfl_xor_sync(0xffffffffu, acc1, offset);
            }
        }
        if (warps_per_row > 1) {
            const int warp = threadIdx.x >> 5;
            if ((threadIdx.x & 31) == 0) { s_red[parity][0][warp] = acc0; s_red[parity][1][warp] = acc1; }
            __syncthreads();
            const int first = row_in_cta * warps_per_row;
            acc0 = 0.0; acc1 = 0.0;
            if (f32_sum) {
                float s = 0.0f;
                for (int w = 0; w < warps_per_row; ++w)
                    s = __fadd_rn(s, static_cast<float>(s_red[parity][1][first + w]));
                acc1 = static_cast<double>(s);
            } else {
                for (int w = 0; w < warps_per_row; ++w) {
                    acc0 += s_red[parity][0][first + w];
                    acc1 += s_red[parity][1][first + w];
                }
            }
            parity ^= 1;
        }
        float mean = 0.0f, inv;
        const double w_d = static_cast<double>(p.norm_width);
        if (p.norm == kNormLayer) {
            mean = static_cast<float>(acc0 / w_d);
            inv = rsqrtf(static_cast<float>(acc1 / w_d - static_cast<double>(mean) * mean) + p.eps);
        } else if (p.norm == kNormRmsF64) {
            inv = rsqrtf(static_cast<float>(acc1 / w_d) + p.eps);
        } else {
            const float m = __fmul_rn(static_cast<float>(acc1), __fdiv_rn(1.0f, static_cast<float>(p.norm_width)));
            inv = rsqrtf(__fadd_rn(m, p.eps));
        }
        if (!valid) continue;  // no barrier follows in this iteration

        // ---- normalise, post-process, store ----
        const int64_t srow = nrow / sub;                              // storage row
        const int64_t col0 = (nrow - srow * sub) * p.norm_width;      // first storage column
        const int64_t vec = p.vectors > 0 ? (srow / p.rows_per_vector) % p.vectors : 0;
        const int64_t frow = p.f_rows > 0 ? (srow / p.rows_per_f_row) % p.f_rows : 0;
#pragma unroll
        for (int i = 0; i < NCH; ++i) {
            const int chunk = lane_in_row + i * tpr;
            if (chunk >= nchunks) continue;
            const int c = chunk * 8;
            float w[8], b[8], y[8];
            if (p.weight) load8<false>(p.weight, p.w_dt, c, w);
            if (p.bias) load8<false>(p.bias, p.b_dt, c, b);
#pragma unroll
            for (int e = 0; e < 8; ++e)
                y[e] = normalise(p, v[i][e], mean, inv,
                                 p.weight ? affine_operand(p, w[e]) : 1.0f,
                                 p.bias ? affine_operand(p, b[e]) : 0.0f);
            if (p.post == kPostModulate) {
                float sc[8], sh[8];
                load8<false>(p.scale, p.mod_dt, vec * p.width + col0 + c, sc);
                if (p.shift) load8<false>(p.shift, p.mod_dt, vec * p.width + col0 + c, sh);
#pragma unroll
                for (int e = 0; e < 8; ++e) y[e] = post_modulate(y[e], sc[e], p.shift ? sh[e] : 0.0f, p.shift != nullptr);
            } else if (p.post == kPostScaleX) {
                float sc[8];
                load8<false>(p.scale, p.mod_dt, vec * p.width + col0 + c, sc);
#pragma unroll
                for (int e = 0; e < 8; ++e) y[e] = post_scale_x(p.norm_out_dt, y[e], sc[e]);
            } else if (p.post == kPostRope) {
                float co[8], si[8], r[8];
                const int64_t f = frow * p.f_width + (col0 + c) % p.f_width;
                load8<false>(p.cosine, p.f_dt, f, co);
                load8<false>(p.sine, p.f_dt, f, si);
#pragma unroll
                for (int e = 0; e < 8; ++e) {
                    const float rotated = (e & 1) ? y[e ^ 1] : -y[e ^ 1];
                    r[e] = __fadd_rn(__fmul_rn(y[e], co[e]), __fmul_rn(rotated, si[e]));
                }
#pragma unroll
                for (int e = 0; e < 8; ++e) y[e] = r[e];
            } else if (p.post == kPostGatedResidual) {
                float res[8], g[8];
                load8<true>(p.residual, p.res_dt, row_offset + c, res);
                if (p.gate) load8<false>(p.gate, p.gate_dt, vec * p.width + col0 + c, g);
#pragma unroll
                for (int e = 0; e < 8; ++e)
                    y[e] = post_gated(p.state_dt, res[e], y[e], p.gate ? g[e] : 0.0f, p.gate != nullptr);
            }
            store8(p.out, p.out_dt, row_offset + c, y);
        }
    }
}

// ---- scalar kernel: any width / alignment; one CTA per normalised row ---------------------
__device__ __forceinline__ double block_sum(double value, double* ws) {
    for (int offset = 16; offset > 0; offset >>= 1) value += __shfl_xor_sync(0xffffffffu, value, offset);
    __syncthreads();
    if ((threadIdx.x & 31) == 0) ws[threadIdx.x >> 5] = value;
    __syncthreads();
    double total = 0.0;
    for (int w = 0; w < (blockDim.x >> 5); ++w) total += ws[w];
    return total;
}
__device__ __forceinline__ float block_sum_f32(float value, float* ws) {
    for (int offset = 16; offset > 0; offset >>= 1)
        value = __fadd_rn(value, __shfl_xor_sync(0xffffffffu, value, offset));
    __syncthreads();
    if ((threadIdx.x & 31) == 0) ws[threadIdx.x >> 5] = value;
    __syncthreads();
    float total = 0.0f;
    for (int w = 0; w < (blockDim.x >> 5); ++w) total = __fadd_rn(total, ws[w]);
    return total;
}

__global__ void __launch_bounds__(kRowThreads) row_kernel_scalar(const RowParams p) {
    __shared__ double ws_d[8];
    __shared__ float ws_f[8];
    const int64_t sub = p.width / p.norm_width;
    const int64_t nrows = p.rows * sub;
    for (int64_t nrow = blockIdx.x; nrow < nrows; nrow += gridDim.x) {
        const int64_t row_offset = nrow * p.norm_width;
        double a0 = 0.0, a1 = 0.0;
        float s = 0.0f;
        for (int64_t c = threadIdx.x; c < p.norm_width; c += blockDim.x) {
            const float x = load1(p.x, p.x_dt, row_offset + c);
            if (p.norm == kNormRmsF32) s = __fadd_rn(s, __fmul_rn(x, x));
            else { a0 += x; a1 = fma(static_cast<double>(x), static_cast<double>(x), a1); }
        }
        float mean = 0.0f, inv;
        const double w_d = static_cast<double>(p.norm_width);
        if (p.norm == kNormLayer) {
            const double t0 = block_sum(a0, ws_d), t1 = block_sum(a1, ws_d);
            mean = static_cast<float>(t0 / w_d);
            inv = rsqrtf(static_cast<float>(t1 / w_d - static_cast<double>(mean) * mean) + p.eps);
        } else if (p.norm == kNormRmsF64) {
            inv = rsqrtf(static_cast<float>(block_sum(a1, ws_d) / w_d) + p.eps);
        } else {
            const float m = __fmul_rn(block_sum_f32(s, ws_f), __fdiv_rn(1.0f, static_cast<float>(p.norm_width)));
            inv = rsqrtf(__fadd_rn(m, p.eps));
        }
        const int64_t srow = nrow / sub;
        const int64_t col0 = (nrow - srow * sub) * p.norm_width;
        const int64_t vec = p.vectors > 0 ? (srow / p.rows_per_vector) % p.vectors : 0;
        const int64_t frow = p.f_rows > 0 ? (srow / p.rows_per_f_row) % p.f_rows : 0;
        auto value_at = [&](int64_t c) {
            return normalise(p, load1(p.x, p.x_dt, row_offset + c), mean, inv,
                             p.weight ? affine_operand(p, load1(p.weight, p.w_dt, c)) : 1.0f,
                             p.bias ? affine_operand(p, load1(p.bias, p.b_dt, c)) : 0.0f);
        };
        for (int64_t c = threadIdx.x; c < p.norm_width; c += blockDim.x) {
            float y = value_at(c);
            const int64_t m = vec * p.width + col0 + c;
            if (p.post == kPostModulate)
                y = post_modulate(y, load1(p.scale, p.mod_dt, m), p.shift ? load1(p.shift, p.mod_dt, m) : 0.0f,
                                  p.shift != nullptr);
            else if (p.post == kPostScaleX)
                y = post_scale_x(p.norm_out_dt, y, load1(p.scale, p.mod_dt, m));
            else if (p.post == kPostRope) {
                const float partner = value_at(c ^ 1);
                const float rotated = (c & 1) ? partner : -partner;
                const int64_t f = frow * p.f_width + (col0 + c) % p.f_width;
                y = __fadd_rn(__fmul_rn(y, load1(p.cosine, p.f_dt, f)), __fmul_rn(rotated, load1(p.sine, p.f_dt, f)));
            } else if (p.post == kPostGatedResidual)
                y = post_gated(p.state_dt, load1(p.residual, p.res_dt, row_offset + c), y,
                               p.gate ? load1(p.gate, p.gate_dt, m) : 0.0f, p.gate != nullptr);
            store1(p.out, p.out_dt, row_offset + c, y);
        }
    }
}

// ---- launch ------------------------------------------------------------------------------
constexpr int kMaxChunks = 8;

// Grid = every CTA the device can hold at once (occupancy of this instantiation x SM count),
// capped by the amount of work; CTAs stride over the rows.
template <int NCH>
void launch_row_kernel(const RowParams& p, int64_t ctas, cudaStream_t stream) {
    static int per_sm = 0;
    if (per_sm == 0) {
        int n = 0;
        if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&n, row_kernel<NCH>, kRowThreads, 0) != cudaSuccess || n < 1) n = 1;
        per_sm = n;
    }
    row_kernel<NCH><<<grid_for(ctas, per_sm), kRowThreads, 0, stream>>>(p);
}

int launch_rows(RowParams p, cudaStream_t stream, const char* what) {
    VRB_REQUIRE(p.x && p.out, VRB_ERR_INVALID, "%s: null tensor", what);
    VRB_REQUIRE(p.rows > 0 && p.width > 0 && p.norm_width > 0 && p.width % p.norm_width == 0,
                VRB_ERR_INVALID, "%s: rows/width must be positive and norm_width must divide width", what);
    VRB_REQUIRE(is_float_dtype(p.x_dt) && is_float_dtype(p.out_dt), VRB_ERR_UNSUPPORTED,
                "%s: tensors must be F32 or BF16", what);
    const int64_t nrows = p.rows * (p.width / p.norm_width);
    bool vector_ok = (p.norm_width % 8 == 0) && aligned16(p.x) && aligned16(p.out) &&
                     (!p.weight || aligned16(p.weight)) && (!p.bias || aligned16(p.bias)) &&
                     (!p.scale || aligned16(p.scale)) && (!p.shift || aligned16(p.shift)) &&
                     (!p.cosine || (aligned16(p.cosine) && aligned16(p.sine) && p.f_width % 8 == 0)) &&
                     (!p.residual || aligned16(p.residual)) && (!p.gate || aligned16(p.gate));
    const int64_t chunks = p.norm_width / 8;
    if (vector_ok && chunks > static_cast<int64_t>(kMaxChunks) * kRowThreads) vector_ok = false;
    if (!vector_ok) {
        p.tpr = kRowThreads;
        row_kernel_scalar<<<grid_for(nrows, 8), kRowThreads, 0, stream>>>(p);
        return after_launch(what);
    }
    // Threads per row: the smallest power of two (8..256) that leaves at most 4 chunks of 8
    // elements per thread; wider rows take more chunks per thread, up to kMaxChunks.
    int tpr = 8;
    while (tpr < kRowThreads && static_cast<int64_t>(tpr) * 4 < chunks) tpr <<= 1;
    const int nch = static_cast<int>((chunks + tpr - 1) / tpr);
    p.tpr = tpr;
    const int rows_per_cta = kRowThreads / tpr;
    const int64_t ctas = (nrows + rows_per_cta - 1) / rows_per_cta;
    switch (nch) {
        case 1: launch_row_kernel<1>(p, ctas, stream); break;
        case 2: launch_row_kernel<2>(p, ctas, stream); break;
        case 3: launch_row_kernel<3>(p, ctas, stream); break;
        case 4: launch_row_kernel<4>(p, ctas, stream); break;
        case 5: launch_row_kernel<5>(p, ctas, stream); break;
        case 6: launch_row_kernel<6>(p, ctas, stream); break;
        case 7: launch_row_kernel<7>(p, ctas, stream); break;
        default: launch_row_kernel<8>(p, ctas, stream); break;
    }
    return after_launch(what);
}

RowParams blank() {
    RowParams p{};
    p.x_dt = p.out_dt = p.w_dt = p.b_dt = p.mod_dt = p.f_dt = p.res_dt = p.gate_dt = p.state_dt = VRB_F32;
    p.norm_out_dt = VRB_F32;
    p.rows_per_vector = 1; p.vectors = 0; p.f_rows = 0; p.f_width = 8; p.rows_per_f_row = 1;
    p.affine_fma = 1;
    return p;
}

int check_vectors(const char* what, int64_t rows_per_vector, int64_t vectors) {
    VRB_REQUIRE(rows_per_vector > 0 && vectors > 0, VRB_ERR_INVALID,
                "%s: rows_per_vector and vector count must be positive", what);
    return VRB_OK;
}

}  // namespace
}  // namespace vrb

using namespace vrb;

extern "C" int vrb_layer_norm(const void* x, int dtype, const void* weight, int weight_dtype,
                              const void* bias, int bias_dtype, void* out,
                              int64_t rows, int64_t width, float eps, vrb_stream stream) {
    RowParams p = blank();
    p.x = x; p.out = out; p.x_dt = p.out_dt = p.norm_out_dt = dtype;
    p.weight = weight; p.w_dt = weight_dtype; p.bias = bias; p.b_dt = bias_dtype;
    VRB_REQUIRE((!weight || is_float_dtype(weight_dtype)) && (!bias || is_float_dtype(bias_dtype)),
                VRB_ERR_UNSUPPORTED, "layer_norm: weight/bias must be F32 or BF16");
    p.rows = rows; p.width = p.norm_width = width; p.eps = eps; p.norm = kNormLayer;
    return launch_rows(p, as_stream(stream), "layer_norm");
}

extern "C" int vrb_rms_norm(const void* x, int x_dtype, const void* weight, int weight_dtype,
                            void* out, int out_dtype, int64_t rows, int64_t width, float eps,
                            vrb_stream stream) {
    VRB_REQUIRE(out_dtype == x_dtype || (x_dtype == VRB_BF16 && out_dtype == VRB_F32),
                VRB_ERR_UNSUPPORTED, "rms_norm output dtype unsupported");
    VRB_REQUIRE(!(x_dtype == VRB_BF16 && out_dtype == VRB_F32 && !weight), VRB_ERR_UNSUPPORTED,
                "BF16-to-FP32 rms_norm requires affine weight");
    RowParams p = blank();
    p.x = x; p.out = out; p.x_dt = x_dtype; p.out_dt = p.norm_out_dt = out_dtype;
    p.weight = weight; p.w_dt = weight_dtype;
    p.rows = rows; p.width = p.norm_width = width; p.eps = eps;
    p.norm = rms_uses_f32_accumulation(width, rows) ? kNormRmsF32 : kNormRmsF64;
    return launch_rows(p, as_stream(stream), "rms_norm");
}

extern "C" int vrb_layer_norm_modulate(const void* x, int x_dtype, const void* weight, int weight_dtype,
                                       const void* bias, int bias_dtype,
                                       const void* scale, const void* shift, int mod_dtype,
                                       int64_t rows_per_vector, int64_t mod_vectors,
                                       void* out, int out_dtype, int64_t rows, int64_t width, float eps,
                                       vrb_stream stream) {
    VRB_REQUIRE(scale != nullptr, VRB_ERR_INVALID, "layer_norm_modulate: scale is null");
    if (int rc = check_vectors("layer_norm_modulate", rows_per_vector, mod_vectors)) return rc;
    RowParams p = blank();
    p.x = x; p.out = out; p.x_dt = p.norm_out_dt = x_dtype; p.out_dt = out_dtype;
    p.weight = weight; p.w_dt = weight_dtype; p.bias = bias; p.b_dt = bias_dtype;
    p.scale = scale; p.shift = shift; p.mod_dt = mod_dtype;
    p.rows_per_vector = rows_per_vector; p.vectors = mod_vectors;
    p.rows = rows; p.width = p.norm_width = width; p.eps = eps;
    p.norm = kNormLayer; p.post = kPostModulate;
    return launch_rows(p, as_stream(stream), "layer_norm_modulate");
}

extern "C" int vrb_rms_norm_modulate(const void* x, int x_dtype, const void* scale, const void* shift,
                                     int mod_dtype, int64_t rows_per_vector, int64_t mod_vectors,
                                     void* out, int out_dtype, int64_t rows, int64_t width, float eps,
                                     vrb_stream stream) {
    VRB_REQUIRE(scale != nullptr, VRB_ERR_INVALID, "rms_norm_modulate: scale is null");
    if (int rc = check_vectors("rms_norm_modulate", rows_per_vector, mod_vectors)) return rc;
    RowParams p = blank();
    p.x = x; p.out = out; p.x_dt = p.norm_out_dt = x_dtype; p.out_dt = out_dtype;
    p.scale = scale; p.shift = shift; p.mod_dt = mod_dtype;
    p.rows_per_vector = rows_per_vector; p.vectors = mod_vectors;
    p.rows = rows; p.width = p.norm_width = width; p.eps = eps;
    p.norm = rms_uses_f32_accumulation(width, rows) ? kNormRmsF32 : kNormRmsF64;
    p.post = kPostModulate;
    return launch_rows(p, as_stream(stream), "rms_norm_modulate");
}

extern "C" int vrb_rms_norm_scale(const void* x, int dtype, const void* scale, int scale_dtype,
                                  int64_t rows_per_vector, int64_t mod_vectors,
                                  void* out, int64_t rows, int64_t width, float eps, vrb_stream stream) {
    VRB_REQUIRE(scale != nullptr, VRB_ERR_INVALID, "rms_norm_scale: scale is null");
    if (int rc = check_vectors("rms_norm_scale", rows_per_vector, mod_vectors)) return rc;
    RowParams p = blank();
    p.x = x; p.out = out; p.x_dt = p.norm_out_dt = p.out_dt = dtype;
    p.scale = scale; p.mod_dt = scale_dtype;
    p.rows_per_vector = rows_per_vector; p.vectors = mod_vectors;
    p.rows = rows; p.width = p.norm_width = width; p.eps = eps;
    p.norm = rms_uses_f32_accumulation(width, rows) ? kNormRmsF32 : kNormRmsF64;
    p.post = kPostScaleX;
    return launch_rows(p, as_stream(stream), "rms_norm_scale");
}

extern "C" int vrb_rms_norm_rope(const void* x, int x_dtype, const void* weight, int weight_dtype,
                                 const void* cosine, const void* sine, int64_t f_rows, int64_t f_width,
                                 int64_t rows_per_f_row, void* out, int out_dtype,
                                 int64_t rows, int64_t width, int64_t norm_width, float eps,
                                 vrb_stream stream) {
    VRB_REQUIRE(weight != nullptr, VRB_ERR_UNSUPPORTED, "BF16-to-FP32 rms_norm requires affine weight");
    VRB_REQUIRE((cosine == nullptr) == (sine == nullptr), VRB_ERR_INVALID, "RoPE frequency mismatch");
    VRB_REQUIRE(norm_width > 0 && width % norm_width == 0, VRB_ERR_INVALID,
                "rms_norm_rope: norm_width must divide width");
    RowParams p = blank();
    p.x = x; p.out = out; p.x_dt = x_dtype; p.out_dt = out_dtype;
    p.norm_out_dt = VRB_F32;  // attention_norm widens to F32 (precision.cpp:292-297)
    p.weight = weight; p.w_dt = weight_dtype;
    p.rows = rows; p.width = width; p.norm_width = norm_width; p.eps = eps;
    p.norm = rms_uses_f32_accumulation(norm_width, rows * (width / norm_width)) ? kNormRmsF32 : kNormRmsF64;
    if (cosine) {
        VRB_REQUIRE(f_rows > 0 && f_width > 0 && rows_per_f_row > 0 && width % f_width == 0 && (norm_width % 2) == 0,
                    VRB_ERR_INVALID, "rms_norm_rope: table extents must be positive, f_width must divide width, width even");
        p.cosine = cosine; p.sine = sine; p.f_dt = VRB_F32;
        p.f_rows = f_rows; p.f_width = f_width; p.rows_per_f_row = rows_per_f_row;
        p.post = kPostRope;
    }
    return launch_rows(p, as_stream(stream), "rms_norm_rope");
}

extern "C" int vrb_rms_norm_gated_residual(const void* residual, int residual_dtype,
                                           const void* branch, int branch_dtype,
                                           const void* gate, int gate_dtype,
                                           int64_t rows_per_vector, int64_t gate_vectors,
                                           void* out, int state_dtype, int64_t rows, int64_t width,
                                           float eps, vrb_stream stream) {
    VRB_REQUIRE(residual != nullptr, VRB_ERR_INVALID, "rms_norm_gated_residual: residual is null");
    if (gate) { if (int rc = check_vectors("rms_norm_gated_residual", rows_per_vector, gate_vectors)) return rc; }
    RowParams p = blank();
    p.x = branch; p.out = out; p.x_dt = p.norm_out_dt = branch_dtype; p.out_dt = p.state_dt = state_dtype;
    p.residual = residual; p.res_dt = residual_dtype; p.gate = gate; p.gate_dt = gate_dtype;
    p.rows_per_vector = rows_per_vector; p.vectors = gate ? gate_vectors : 0;
    p.rows = rows; p.width = p.norm_width = width; p.eps = eps;
    p.norm = rms_uses_f32_accumulation(width, rows) ? kNormRmsF32 : kNormRmsF64;
    p.post = kPostGatedResidual;
    return launch_rows(p, as_stream(stream), "rms_norm_gated_residual");
}

extern "C" int vrb_layer_norm_cast(const void* x, int x_dtype, const void* weight, int weight_dtype,
                                   const void* bias, int bias_dtype, void* out, int out_dtype,
                                   int64_t rows, int64_t width, float eps, vrb_stream stream) {
    RowParams p = blank();
    p.x = x; p.out = out; p.x_dt = p.norm_out_dt = x_dtype; p.out_dt = out_dtype;
    p.weight = weight; p.w_dt = weight_dtype; p.bias = bias; p.b_dt = bias_dtype;
    VRB_REQUIRE((!weight || is_float_dtype(weight_dtype)) && (!bias || is_float_dtype(bias_dtype)),
                VRB_ERR_UNSUPPORTED, "layer_norm_cast: weight/bias must be F32 or BF16");
    p.rows = rows; p.width = p.norm_width = width; p.eps = eps; p.norm = kNormLayer;
    return launch_rows(p, as_stream(stream), "layer_norm_cast");
}
