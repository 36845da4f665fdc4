// Entry points of the row-wise normalisation family, the dispatch onto the templated vector
// kernels (vrb_rowwise.cuh, instantiated in vrb_rowwise_ln.cu / _rms_a.cu / _rms_b.cu) and the
// scalar kernel that covers any width or alignment.
#include "vrb_rowwise.cuh"

namespace vrb {
namespace rowwise {
namespace {

// The reference's choice between the F32-accumulating and the double-accumulating RMS
// kernels depends on the row width and the row count (launch-geometry rule of
// rms_contiguous_reduction_lanes, cuda_backend.cu:838-850).  True when the F32 kernel runs.
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

template <int NORM>
__global__ void __launch_bounds__(kRowThreads) row_kernel_scalar(const RowParams p) {
    __shared__ double ws_d[8];
    __shared__ float ws_f[8];
    const int64_t sub = p.width / p.norm_width;
    const int64_t nrows = p.rows * sub;
    const bool has_w = p.weight != nullptr, has_b = p.bias != nullptr;
    const bool x_bf16 = p.x_dt == VRB_BF16;
    const int affine_dt = NORM == kNormLayer ? p.x_dt : p.norm_out_dt;
    const bool f32_sum = NORM == kNormRms && !p.rms_f64;
    for (int64_t nrow = blockIdx.x; nrow < nrows; nrow += gridDim.x) {
        const int64_t row_offset = nrow * p.norm_width;
        double a0 = 0.0, a1 = 0.0;
        float s = 0.0f;
        for (int64_t c = threadIdx.x; c < p.norm_width; c += blockDim.x) {
            const float x = load1(p.x, p.x_dt, row_offset + c);
            if (f32_sum) s = __fadd_rn(s, __fmul_rn(x, x));
            else { a0 += x; a1 = fma(static_cast<double>(x), static_cast<double>(x), a1); }
        }
        float mean = 0.0f, inv;
        const double w_d = static_cast<double>(p.norm_width);
        if constexpr (NORM == kNormLayer) {
            const double t0 = block_sum(a0, ws_d), t1 = block_sum(a1, ws_d);
            mean = static_cast<float>(t0 / w_d);
            inv = rsqrtf(static_cast<float>(t1 / w_d - static_cast<double>(mean) * mean) + p.eps);
        } else if (!f32_sum) {
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
            return normalise<NORM>(p, load1(p.x, p.x_dt, row_offset + c), mean, inv,
                                   has_w ? round_to(affine_dt, load1(p.weight, p.w_dt, c)) : 1.0f,
                                   has_b ? round_to(affine_dt, load1(p.bias, p.b_dt, c)) : 0.0f, has_w, has_b, x_bf16);
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

// ---- dispatch ----------------------------------------------------------------------------
constexpr int kMaxChunks = 8;
// launch_rows() result when a fused residual update was asked for but the vector kernel cannot
// take it (alignment, width, too many gate vectors): the caller then runs the two operators.
constexpr int kPreNotFused = 1;
// ... and when a two-problem launch was asked for but needs the scalar kernel: the caller launches twice.
constexpr int kPairNotFused = 2;

// Which dtype classes exist for a (norm, post) pair; anything else takes the scalar kernel.
template <int NORM, int POST>
bool launch_by_dtype(const RowParams& p, int geometry, int64_t ctas, size_t smem, cudaStream_t s) {
    constexpr bool rope = POST == kPostRope || POST == kPostRopeShared;
    const bool x_bf16 = p.x_dt == VRB_BF16, n_bf16 = p.norm_out_dt == VRB_BF16;
    if (p.pre_branch != nullptr) {   // fused residual update: bf16 stream, LayerNorm, no / staged / plain modulate
        if constexpr (NORM == kNormLayer && (POST == kPostNone || POST == kPostModulate || POST == kPostModulateStaged)) {
            if (x_bf16 && n_bf16) { launch_row_variant<NORM, POST, kBf16Bf16Pre>(p, geometry, ctas, smem, s); return true; }
            if (!x_bf16 && !n_bf16) { launch_row_variant<NORM, POST, kF32Pre>(p, geometry, ctas, smem, s); return true; }
        }
        if constexpr (NORM == kNormRms && (POST == kPostModulate || POST == kPostModulateStaged)) {   // the LTX block's form
            if (x_bf16 && n_bf16) { launch_row_variant<NORM, POST, kBf16Bf16Pre>(p, geometry, ctas, smem, s); return true; }
            if (!x_bf16 && !n_bf16) { launch_row_variant<NORM, POST, kF32Pre>(p, geometry, ctas, smem, s); return true; }
        }
        if constexpr (NORM == kNormRms && POST == kPostScaleX) {   // the Mochi block's form
            if (x_bf16 && n_bf16) { launch_row_variant<NORM, POST, kBf16Bf16Pre>(p, geometry, ctas, smem, s); return true; }
        }
        return false;
    }
    if (!x_bf16 && !n_bf16) { launch_row_variant<NORM, POST, kF32F32>(p, geometry, ctas, smem, s); return true; }
    if constexpr (!rope) {
        if (x_bf16 && n_bf16) { launch_row_variant<NORM, POST, kBf16Bf16>(p, geometry, ctas, smem, s); return true; }
    }
    if constexpr (NORM == kNormRms && (POST == kPostNone || rope)) {
        if (x_bf16 && !n_bf16) { launch_row_variant<NORM, POST, kBf16F32>(p, geometry, ctas, smem, s); return true; }
    }
    return false;
}

// second_rows > 0: (p.x_b, p.out_b, p.weight_b) is a second problem of second_rows storage rows that
// runs in the same launch; the caller has checked that both problems take the same kernel.
int launch_rows(RowParams p, cudaStream_t stream, const char* what, int64_t second_rows = 0) {
    VRB_REQUIRE(p.x && p.out, VRB_ERR_INVALID, "%s: null tensor", what);
    VRB_REQUIRE(p.rows > 0 && p.width > 0 && p.norm_width > 0 && p.width % p.norm_width == 0,
                VRB_ERR_INVALID, "%s: rows/width must be positive and norm_width must divide width", what);
    VRB_REQUIRE(is_float_dtype(p.x_dt) && is_float_dtype(p.out_dt), VRB_ERR_UNSUPPORTED,
                "%s: tensors must be F32 or BF16", what);
    const int64_t sub = p.width / p.norm_width;
    const int64_t nrows = p.rows * sub;
    bool vector_ok = (p.norm_width % 8 == 0) && aligned16(p.x) && aligned16(p.out) &&
                     (!p.weight || aligned16(p.weight)) && (!p.bias || aligned16(p.bias)) &&
                     (!p.scale || aligned16(p.scale)) && (!p.shift || aligned16(p.shift)) &&
                     (!p.cosine || (aligned16(p.cosine) && aligned16(p.sine) && p.f_width % 8 == 0)) &&
                     (!p.residual || aligned16(p.residual)) && (!p.gate || aligned16(p.gate));
    if (second_rows > 0) {
        VRB_REQUIRE(p.x_b && p.out_b, VRB_ERR_INVALID, "%s: null tensor", what);
        vector_ok = vector_ok && aligned16(p.x_b) && aligned16(p.out_b) && (!p.weight_b || aligned16(p.weight_b)) &&
                    second_rows * sub < (1LL << 31);
        if (!vector_ok) return kPairNotFused;
    }
    const int64_t chunks = p.norm_width / 8;
    if (chunks > static_cast<int64_t>(kMaxChunks) * kRowThreads) vector_ok = false;
    // The vector kernel indexes rows and table rows in 32 bits.
    if (nrows >= (1LL << 31) || p.rows_per_vector >= (1LL << 31) || p.vectors >= (1LL << 31) ||
        p.f_rows >= (1LL << 31) || p.rows_per_f_row >= (1LL << 31) || p.width >= (1LL << 31))
        vector_ok = false;
    auto scalar_path = [&]() {
        p.tpr = kRowThreads;
        const int grid = grid_for(nrows, 8);
        if (p.norm == kNormLayer) row_kernel_scalar<kNormLayer><<<grid, kRowThreads, 0, stream>>>(p);
        else row_kernel_scalar<kNormRms><<<grid, kRowThreads, 0, stream>>>(p);
        return after_launch(what);
    };
    if (p.pre_branch != nullptr &&
        (!vector_ok || !aligned16(p.pre_branch) || !aligned16(p.state_out) || (p.pre_gate && p.pre_vectors > 4) || sub != 1))
        return kPreNotFused;
    if (!vector_ok) return scalar_path();
    // Threads per row: a row of up to 32*6 chunks stays inside one warp (no barrier); narrower
    // rows take a fraction of a warp with 1-2 chunks per thread; wider rows take 2-8 warps.
    int tpr;
    if (chunks <= 32 * 6) {
        tpr = 8;
        while (tpr < 32 && static_cast<int64_t>(tpr) * 2 < chunks) tpr <<= 1;
    } else {
        tpr = 64;
        while (tpr < kRowThreads && static_cast<int64_t>(tpr) * 6 < chunks) tpr <<= 1;
    }
    int nch = static_cast<int>((chunks + tpr - 1) / tpr);
    if (nch == 7) nch = 8;
    int geometry = nch <= 6 ? nch - 1 : 6;
    switch (p.norm_width) {   // production widths have exact instantiations
        case 1536: geometry = kExact1536; tpr = 32; break;
        case 3072: geometry = kExact3072; tpr = 64; break;
        case 5120: geometry = kExact5120; tpr = 128; break;
        case 2048: geometry = kExact2048; tpr = 64; break;
        case 128: geometry = kExact128; tpr = 8; break;
        case 64: geometry = kExact64; tpr = 8; break;
        default: break;
    }
    p.tpr = tpr;
    p.nrows32 = static_cast<unsigned>(nrows);
    p.sub32 = static_cast<unsigned>(sub);
    p.inv_width = 1.0 / static_cast<double>(p.norm_width);
    const int rows_per_cta = kRowThreads / tpr;
    int64_t ctas = (nrows + rows_per_cta - 1) / rows_per_cta;
    if (second_rows > 0) {
        p.nrows_b = static_cast<unsigned>(second_rows * sub);
        ctas += (second_rows * sub + rows_per_cta - 1) / rows_per_cta;
    }
    size_t smem = 0;
    int post = p.post;
    const size_t region = static_cast<size_t>(geometry <= 6 ? nch : (chunks / tpr)) * tpr * 8 * sizeof(float);
    // Up to four modulation vectors (one per batch entry): stage 1+scale and shift per CTA instead
    // of re-reading them for every row.  The budget leaves room for two resident CTAs per SM
    // (sizes above 48 KB are opted into by the launcher).
    // The fused residual update with a modulating epilogue runs three CTAs per SM: smaller budget,
    // its gate vectors included.
    const bool pre = p.pre_branch != nullptr;
    // gate vectors: bf16 pairs for a bf16 stream, F32 for an F32 stream
    const size_t gate_bytes = pre && p.pre_gate ? static_cast<size_t>(p.pre_vectors) * (p.x_dt == VRB_BF16 ? region / 2 : region) : 0;
    if (gate_bytes > 48 * 1024) return kPreNotFused;
    const size_t budget = (pre && post != kPostNone ? 72 * 1024 : 100 * 1024) - gate_bytes;
    if (post == kPostModulate && p.vectors >= 1 && p.vectors <= 4 && sub == 1 &&
        static_cast<size_t>(p.vectors) * 2 * region <= budget) {
        post = kPostModulateStaged;
        smem += static_cast<size_t>(p.vectors) * 2 * region;
    }
    // LayerNorm weight and bias both present: stage them per CTA, already converted to x's dtype.
    // (Staging the RMSNorm weight the same way was measured and does not pay: its 16-byte loads
    // hit L1 and cost the same as the shared-memory reads.)
    if (p.norm == kNormLayer && p.weight && p.bias && smem + 2 * region <= budget) {
        p.affine_staged = 1;
        smem += 2 * region;
    }
    // Fused residual update: the gate vectors, bf16 pairs, behind everything else.
    if (pre) smem += gate_bytes;
    // RoPE table shared by the heads: the columns a thread needs are the same for all its chunks.
    if (post == kPostRope && p.norm_width % p.f_width == 0 && (static_cast<int64_t>(tpr) * 8) % p.f_width == 0)
        post = kPostRopeShared;
    bool launched;
    if (p.norm == kNormLayer) {
        if (post == kPostModulateStaged) launched = launch_by_dtype<kNormLayer, kPostModulateStaged>(p, geometry, ctas, smem, stream);
        else if (post == kPostModulate) launched = launch_by_dtype<kNormLayer, kPostModulate>(p, geometry, ctas, smem, stream);
        else launched = launch_by_dtype<kNormLayer, kPostNone>(p, geometry, ctas, smem, stream);
    } else {
        switch (post) {
            case kPostModulateStaged: launched = launch_by_dtype<kNormRms, kPostModulateStaged>(p, geometry, ctas, smem, stream); break;
            case kPostModulate: launched = launch_by_dtype<kNormRms, kPostModulate>(p, geometry, ctas, smem, stream); break;
            case kPostScaleX: launched = launch_by_dtype<kNormRms, kPostScaleX>(p, geometry, ctas, smem, stream); break;
            case kPostRopeShared: launched = launch_by_dtype<kNormRms, kPostRopeShared>(p, geometry, ctas, smem, stream); break;
            case kPostRope: launched = launch_by_dtype<kNormRms, kPostRope>(p, geometry, ctas, smem, stream); break;
            case kPostGatedResidual: launched = launch_by_dtype<kNormRms, kPostGatedResidual>(p, geometry, ctas, smem, stream); break;
            default: launched = launch_by_dtype<kNormRms, kPostNone>(p, geometry, ctas, smem, stream); break;
        }
    }
    if (!launched) return p.pre_branch != nullptr ? kPreNotFused : second_rows > 0 ? kPairNotFused : scalar_path();
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

void set_rms(RowParams& p, int64_t norm_rows) {
    p.norm = kNormRms;
    p.rms_f64 = rms_uses_f32_accumulation(p.norm_width, norm_rows) ? 0 : 1;
}

int check_vectors(const char* what, int64_t rows_per_vector, int64_t vectors) {
    VRB_REQUIRE(rows_per_vector > 0 && vectors > 0, VRB_ERR_INVALID,
                "%s: rows_per_vector and vector count must be positive", what);
    return VRB_OK;
}

}  // namespace
}  // namespace rowwise
}  // namespace vrb

using namespace vrb;
using namespace vrb::rowwise;

extern "C" int vrb_layer_norm(const void* x, int dtype, const void* weight, int weight_dtype,
                              const void* bias, int bias_dtype, void* out,
                              int64_t rows, int64_t width, float eps, vrb_stream stream) {
    return vrb_layer_norm_cast(x, dtype, weight, weight_dtype, bias, bias_dtype, out, dtype, rows, width, eps, stream);
}

extern "C" int vrb_layer_norm_cast(const void* x, int x_dtype, const void* weight, int weight_dtype,
                                   const void* bias, int bias_dtype, void* out, int out_dtype,
                                   int64_t rows, int64_t width, float eps, vrb_stream stream) {
    RowParams p = blank();
    p.x = x; p.out = out; p.x_dt = p.norm_out_dt = x_dtype; p.out_dt = out_dtype;
    p.weight = weight; p.w_dt = weight_dtype; p.bias = bias; p.b_dt = bias_dtype;
    VRB_REQUIRE((!weight || is_float_dtype(weight_dtype)) && (!bias || is_float_dtype(bias_dtype)),
                VRB_ERR_UNSUPPORTED, "layer_norm: weight/bias must be F32 or BF16");
    p.rows = rows; p.width = p.norm_width = width; p.eps = eps; p.norm = kNormLayer;
    return launch_rows(p, as_stream(stream), "layer_norm");
}

extern "C" int vrb_gated_residual_layer_norm_modulate(
        const void* residual, int residual_dtype, const void* branch, int branch_dtype,
        const void* gate, int gate_dtype, int64_t gate_rows_per_vector, int64_t gate_vectors,
        void* state_out, int state_dtype,
        const void* weight, int weight_dtype, const void* bias, int bias_dtype,
        const void* scale, const void* shift, int mod_dtype, int64_t rows_per_vector, int64_t mod_vectors,
        void* out, int out_dtype, int64_t rows, int64_t width, float eps, vrb_stream stream) {
    VRB_REQUIRE(residual && branch && state_out && out, VRB_ERR_INVALID, "gated_residual_layer_norm: null tensor");
    VRB_REQUIRE((!weight || is_float_dtype(weight_dtype)) && (!bias || is_float_dtype(bias_dtype)),
                VRB_ERR_UNSUPPORTED, "layer_norm: weight/bias must be F32 or BF16");
    if (gate) { if (int rc = check_vectors("gated_residual_layer_norm", gate_rows_per_vector, gate_vectors)) return rc; }
    if (scale) { if (int rc = check_vectors("gated_residual_layer_norm", rows_per_vector, mod_vectors)) return rc; }
    // one pass for a bf16 stream, and for the production contract (F32 stream, bf16 branch)
    if (branch_dtype == VRB_BF16 && residual_dtype == state_dtype) {
        RowParams p = blank();
        p.x = residual; p.x_dt = p.norm_out_dt = residual_dtype; p.out = out; p.out_dt = out_dtype;
        p.pre_branch = branch; p.pre_gate = gate; p.pre_gate_dt = gate_dtype; p.state_out = state_out;
        p.pre_rows_per_vector = gate ? gate_rows_per_vector : 1; p.pre_vectors = gate ? gate_vectors : 0;
        p.weight = weight; p.w_dt = weight_dtype; p.bias = bias; p.b_dt = bias_dtype;
        p.rows = rows; p.width = p.norm_width = width; p.eps = eps; p.norm = kNormLayer;
        if (scale) {
            p.scale = scale; p.shift = shift; p.mod_dt = mod_dtype;
            p.rows_per_vector = rows_per_vector; p.vectors = mod_vectors; p.post = kPostModulate;
        }
        const int rc = launch_rows(p, as_stream(stream), "gated_residual_layer_norm");
        if (rc != kPreNotFused) return rc;
    }
    // any other dtype contract or geometry: the two operators, one after the other
    if (int rc = vrb_gated_residual(residual, residual_dtype, branch, branch_dtype, gate, gate_dtype, gate_rows_per_vector,
                                    gate_vectors, state_out, state_dtype, rows, width, stream))
        return rc;
    if (scale)
        return vrb_layer_norm_modulate(state_out, state_dtype, weight, weight_dtype, bias, bias_dtype, scale, shift, mod_dtype,
                                       rows_per_vector, mod_vectors, out, out_dtype, rows, width, eps, stream);
    return vrb_layer_norm_cast(state_out, state_dtype, weight, weight_dtype, bias, bias_dtype, out, out_dtype, rows, width, eps,
                               stream);
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
    set_rms(p, rows);
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
    set_rms(p, rows);
    p.post = kPostModulate;
    return launch_rows(p, as_stream(stream), "rms_norm_modulate");
}

extern "C" int vrb_gated_residual_rms_norm_modulate(
        const void* residual, int residual_dtype, const void* branch, int branch_dtype,
        const void* gate, int gate_dtype, int64_t gate_rows_per_vector, int64_t gate_vectors,
        void* state_out, int state_dtype,
        const void* scale, const void* shift, int mod_dtype, int64_t rows_per_vector, int64_t mod_vectors,
        void* out, int out_dtype, int64_t rows, int64_t width, float eps, vrb_stream stream) {
    VRB_REQUIRE(residual && branch && state_out && out, VRB_ERR_INVALID, "gated_residual_rms_norm: null tensor");
    VRB_REQUIRE(scale != nullptr, VRB_ERR_INVALID, "gated_residual_rms_norm: scale is null");
    if (gate) { if (int rc = check_vectors("gated_residual_rms_norm", gate_rows_per_vector, gate_vectors)) return rc; }
    if (int rc = check_vectors("gated_residual_rms_norm", rows_per_vector, mod_vectors)) return rc;
    if (branch_dtype == VRB_BF16 && residual_dtype == state_dtype) {
        RowParams p = blank();
        p.x = residual; p.x_dt = p.norm_out_dt = residual_dtype; p.out = out; p.out_dt = out_dtype;
        p.pre_branch = branch; p.pre_gate = gate; p.pre_gate_dt = gate_dtype; p.state_out = state_out;
        p.pre_rows_per_vector = gate ? gate_rows_per_vector : 1; p.pre_vectors = gate ? gate_vectors : 0;
        p.scale = scale; p.shift = shift; p.mod_dt = mod_dtype;
        p.rows_per_vector = rows_per_vector; p.vectors = mod_vectors;
        p.rows = rows; p.width = p.norm_width = width; p.eps = eps;
        set_rms(p, rows);
        p.post = kPostModulate;
        const int rc = launch_rows(p, as_stream(stream), "gated_residual_rms_norm");
        if (rc != kPreNotFused) return rc;
    }
    if (int rc = vrb_gated_residual(residual, residual_dtype, branch, branch_dtype, gate, gate_dtype, gate_rows_per_vector,
                                    gate_vectors, state_out, state_dtype, rows, width, stream))
        return rc;
    return vrb_rms_norm_modulate(state_out, state_dtype, scale, shift, mod_dtype, rows_per_vector, mod_vectors, out, out_dtype,
                                 rows, width, eps, stream);
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
    set_rms(p, rows);
    p.post = kPostScaleX;
    return launch_rows(p, as_stream(stream), "rms_norm_scale");
}

extern "C" int vrb_rms_norm_rope(const void* x, int x_dtype, const void* weight, int weight_dtype,
                                 const void* cosine, const void* sine, int64_t f_rows, int64_t f_width,
                                 int64_t rows_per_f_row, void* out, int out_dtype,
                                 int64_t rows, int64_t width, int64_t norm_width, float eps,
                                 vrb_stream stream) {
    return vrb_rms_norm_rope_tables(x, x_dtype, weight, weight_dtype, cosine, sine, VRB_F32, f_rows, f_width, rows_per_f_row,
                                    out, out_dtype, rows, width, norm_width, eps, stream);
}

extern "C" int vrb_rms_norm_rope_tables(const void* x, int x_dtype, const void* weight, int weight_dtype,
                                        const void* cosine, const void* sine, int table_dtype, int64_t f_rows,
                                        int64_t f_width, int64_t rows_per_f_row, void* out, int out_dtype,
                                        int64_t rows, int64_t width, int64_t norm_width, float eps, vrb_stream stream) {
    VRB_REQUIRE(is_float_dtype(table_dtype), VRB_ERR_UNSUPPORTED, "rms_norm_rope: tables must be F32 or BF16");
    VRB_REQUIRE(weight != nullptr, VRB_ERR_UNSUPPORTED, "BF16-to-FP32 rms_norm requires affine weight");
    VRB_REQUIRE((cosine == nullptr) == (sine == nullptr), VRB_ERR_INVALID, "RoPE frequency mismatch");
    VRB_REQUIRE(norm_width > 0 && width % norm_width == 0, VRB_ERR_INVALID,
                "rms_norm_rope: norm_width must divide width");
    RowParams p = blank();
    p.x = x; p.out = out; p.x_dt = x_dtype; p.out_dt = out_dtype;
    p.norm_out_dt = VRB_F32;  // attention_norm widens to F32 (precision.cpp:292-297)
    p.weight = weight; p.w_dt = weight_dtype;
    p.rows = rows; p.width = width; p.norm_width = norm_width; p.eps = eps;
    set_rms(p, rows * (width / norm_width));
    if (cosine) {
        VRB_REQUIRE(f_rows > 0 && f_width > 0 && rows_per_f_row > 0 && width % f_width == 0 && (norm_width % 2) == 0,
                    VRB_ERR_INVALID, "rms_norm_rope: table extents must be positive, f_width must divide width, width even");
        p.cosine = cosine; p.sine = sine; p.f_dt = table_dtype;
        p.f_rows = f_rows; p.f_width = f_width; p.rows_per_f_row = rows_per_f_row;
        p.post = kPostRope;
    }
    return launch_rows(p, as_stream(stream), "rms_norm_rope");
}

extern "C" int vrb_rms_norm_gated_residual_rms_norm_scale(
        const void* residual, int residual_dtype, const void* branch, int branch_dtype, float branch_eps,
        const void* gate, int gate_dtype, int gate_tanh, int64_t gate_rows_per_vector, int64_t gate_vectors,
        void* state_out, int state_dtype, const void* scale, int scale_dtype, int64_t rows_per_vector, int64_t scale_vectors,
        void* out, int64_t rows, int64_t width, float eps, vrb_stream stream) {
    VRB_REQUIRE(residual && branch && state_out && out && scale, VRB_ERR_INVALID, "rms_norm_gated_residual_rms_norm_scale: null tensor");
    if (gate) { if (int rc = check_vectors("rms_norm_gated_residual_rms_norm_scale", gate_rows_per_vector, gate_vectors)) return rc; }
    if (int rc = check_vectors("rms_norm_gated_residual_rms_norm_scale", rows_per_vector, scale_vectors)) return rc;
    VRB_REQUIRE(is_float_dtype(residual_dtype) && is_float_dtype(branch_dtype) && is_float_dtype(state_dtype) &&
                    is_float_dtype(scale_dtype) && (!gate || is_float_dtype(gate_dtype)),
                VRB_ERR_UNSUPPORTED, "rms_norm_gated_residual_rms_norm_scale: dtypes must be F32 or BF16");
    // one pass for a bf16 stream (residual, branch, updated stream and normalised output all bf16)
    if (residual_dtype == VRB_BF16 && branch_dtype == VRB_BF16 && state_dtype == VRB_BF16) {
        RowParams p = blank();
        p.x = residual; p.x_dt = p.norm_out_dt = p.out_dt = VRB_BF16; p.out = out;
        p.pre_branch = branch; p.pre_gate = gate; p.pre_gate_dt = gate_dtype; p.state_out = state_out;
        p.pre_rows_per_vector = gate ? gate_rows_per_vector : 1; p.pre_vectors = gate ? gate_vectors : 0;
        p.pre_norm = 1; p.pre_eps = branch_eps; p.pre_gate_tanh = gate && gate_tanh ? 1 : 0;
        p.scale = scale; p.mod_dt = scale_dtype; p.rows_per_vector = rows_per_vector; p.vectors = scale_vectors;
        p.post = kPostScaleX;
        p.rows = rows; p.width = p.norm_width = width; p.eps = eps;
        set_rms(p, rows);
        const int rc = launch_rows(p, as_stream(stream), "rms_norm_gated_residual_rms_norm_scale");
        if (rc != kPreNotFused) return rc;
    }
    // otherwise the two operators; tanh(gate) would need a temporary, which an entry point does not allocate
    VRB_REQUIRE(!(gate && gate_tanh), VRB_ERR_UNSUPPORTED,
                "rms_norm_gated_residual_rms_norm_scale: for this dtype contract or geometry apply tanh to the gate first "
                "(vrb_activation) and pass gate_tanh = 0");
    if (int rc = vrb_rms_norm_gated_residual(residual, residual_dtype, branch, branch_dtype, gate, gate_dtype, gate_rows_per_vector,
                                             gate_vectors, state_out, state_dtype, rows, width, branch_eps, stream))
        return rc;
    return vrb_rms_norm_scale(state_out, state_dtype, scale, scale_dtype, rows_per_vector, scale_vectors, out, rows, width, eps, stream);
}

extern "C" int vrb_rms_norm_rope_pair(const void* x_a, const void* weight_a, void* out_a, int64_t rows_a,
                                      const void* x_b, const void* weight_b, void* out_b, int64_t rows_b,
                                      int x_dtype, int weight_dtype, const void* cosine, const void* sine, int table_dtype,
                                      int64_t f_rows, int64_t f_width, int64_t rows_per_f_row, int out_dtype,
                                      int64_t width, int64_t norm_width, float eps, vrb_stream stream) {
    VRB_REQUIRE(x_a && x_b && out_a && out_b && weight_a && weight_b, VRB_ERR_INVALID, "rms_norm_rope_pair: null tensor");
    VRB_REQUIRE(rows_a > 0 && rows_b > 0, VRB_ERR_INVALID, "rms_norm_rope_pair: extents must be positive");
    VRB_REQUIRE(norm_width > 0 && width % norm_width == 0, VRB_ERR_INVALID, "rms_norm_rope: norm_width must divide width");
    const int64_t sub = width / norm_width;
    // One launch only if both problems take the same kernel: the reference picks its summation formula
    // from the row count (rms_contiguous_reduction_lanes, :838-850).
    if (rms_uses_f32_accumulation(norm_width, rows_a * sub) == rms_uses_f32_accumulation(norm_width, rows_b * sub)) {
        VRB_REQUIRE(is_float_dtype(table_dtype), VRB_ERR_UNSUPPORTED, "rms_norm_rope: tables must be F32 or BF16");
        VRB_REQUIRE((cosine == nullptr) == (sine == nullptr), VRB_ERR_INVALID, "RoPE frequency mismatch");
        RowParams p = blank();
        p.x = x_a; p.out = out_a; p.weight = weight_a;
        p.x_b = x_b; p.out_b = out_b; p.weight_b = weight_b;
        p.x_dt = x_dtype; p.out_dt = out_dtype; p.norm_out_dt = VRB_F32; p.w_dt = weight_dtype;
        p.rows = rows_a; p.width = width; p.norm_width = norm_width; p.eps = eps;
        set_rms(p, rows_a * sub);
        if (cosine) {
            VRB_REQUIRE(f_rows > 0 && f_width > 0 && rows_per_f_row > 0 && width % f_width == 0 && (norm_width % 2) == 0,
                        VRB_ERR_INVALID, "rms_norm_rope: table extents must be positive, f_width must divide width, width even");
            p.cosine = cosine; p.sine = sine; p.f_dt = table_dtype;
            p.f_rows = f_rows; p.f_width = f_width; p.rows_per_f_row = rows_per_f_row;
            p.post = kPostRope;
        }
        const int rc = launch_rows(p, as_stream(stream), "rms_norm_rope_pair", rows_b);
        if (rc != kPairNotFused) return rc;
    }
    if (int rc = vrb_rms_norm_rope_tables(x_a, x_dtype, weight_a, weight_dtype, cosine, sine, table_dtype, f_rows, f_width,
                                          rows_per_f_row, out_a, out_dtype, rows_a, width, norm_width, eps, stream))
        return rc;
    return vrb_rms_norm_rope_tables(x_b, x_dtype, weight_b, weight_dtype, cosine, sine, table_dtype, f_rows, f_width,
                                    rows_per_f_row, out_b, out_dtype, rows_b, width, norm_width, eps, stream);
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
    set_rms(p, rows);
    p.post = kPostGatedResidual;
    return launch_rows(p, as_stream(stream), "rms_norm_gated_residual");
}
