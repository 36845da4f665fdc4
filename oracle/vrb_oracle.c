/*
 * vrb_oracle.c -- CPU restatement of the arithmetic of the reference's non-GEMM CUDA
 * operators.  TEST INFRASTRUCTURE ONLY: this file is the checker the parity tests, the
 * smoke test and the benchmark's cpu_baseline leg compare the CUDA library against.
 * Nothing in the product library links, loads or calls it.
 *
 * Every function restates one reference kernel (paths are inside the reference project,
 * native/src/backend/cuda/cuda_backend.cu unless another file is named) with the same
 * order of floating-point operations, the same intermediate roundings and the same
 * partial-sum schedule the kernel's launch geometry produces.  Device-only math functions
 * are replaced by their C counterparts: rsqrtf(x) -> 1.0f/sqrtf(x), expf/tanhf/erff ->
 * libm.  Those agree with the CUDA library to within its documented 1-2 ulp, which is why
 * floating-point parity is stated as a tolerance and not bit-for-bit.
 *
 * Parity pins: the known-answer values and inline reference formulas of the reference's own
 * tests (native/tests/primitive_tests.cpp, precision_operation_contract_tests.cpp,
 * semantic_scalar_tests.cpp, phase9_quant_tests.cpp) are replayed against this file by
 * tests/test_oracle_pins.py, and the reference's own host backend
 * (native/tests/family_lowering_test_backend.h) compiled from its sources is compared with
 * it by tests/test_oracle_vs_ref_host.py when that build is present.
 *
 * Build: gcc -O2 -ffp-contract=off -fopenmp -shared -fPIC vrb_oracle.c -lm
 * (-ffp-contract=off: every contraction the oracle wants is written as fmaf()).
 *
 * dtype codes follow the reference's DType enum (native/include/vrhino/tensor.h:13):
 * 0 = F32, 2 = BF16, 5 = U8.
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#define ORC_F32 0
#define ORC_BF16 2
#define ORC_MAX_DIMS 8

/* ---- scalar conversions (tensor.h: bf16 is the upper half of an f32; stores are RNE,
 * cuda_backend.cu:546-549) ---- */
static inline float bf16_to_f32(uint16_t v) {
    uint32_t bits = (uint32_t)v << 16;
    float f;
    memcpy(&f, &bits, 4);
    return f;
}
static inline uint16_t f32_to_bf16(float f) {
    uint32_t bits;
    memcpy(&bits, &f, 4);
    if ((bits & 0x7fffffffu) > 0x7f800000u) return 0x7fff; /* __float2bfloat16 NaN result */
    bits += 0x7fffu + ((bits >> 16) & 1u);
    return (uint16_t)(bits >> 16);
}
static inline float round_bf16(float f) { return bf16_to_f32(f32_to_bf16(f)); }

static inline float ld(const void* p, int dt, int64_t i) {
    return dt == ORC_BF16 ? bf16_to_f32(((const uint16_t*)p)[i]) : ((const float*)p)[i];
}
static inline void st(void* p, int dt, int64_t i, float v) {
    if (dt == ORC_BF16) ((uint16_t*)p)[i] = f32_to_bf16(v);
    else ((float*)p)[i] = v;
}
static inline float rsqrt_ref(float v) { return 1.0f / sqrtf(v); }
/* fmaxf as the device evaluates it (PTX max.f32): a NaN operand yields the other operand and
 * -0 orders below +0; C's fmaxf leaves the sign of max(-0,+0) unspecified. */
static inline float max_ref(float a, float b) {
    if (isnan(a)) return b;
    if (isnan(b)) return a;
    if (a == 0.0f && b == 0.0f) return (signbit(a) && signbit(b)) ? -0.0f : 0.0f;
    return a > b ? a : b;
}

uint16_t orc_f32_to_bf16(float f) { return f32_to_bf16(f); }
float orc_bf16_to_f32(uint16_t v) { return bf16_to_f32(v); }

/* ---- cast (cuda_backend.cu:597-628): widening is exact, narrowing is RNE ---- */
void orc_cast(const void* src, int sdt, void* dst, int ddt, int64_t n) {
#pragma omp parallel for schedule(static)
    for (int64_t i = 0; i < n; ++i) st(dst, ddt, i, ld(src, sdt, i));
}
/* numeric_to_float / numeric_to_bf16 (cuda_backend.cu:617-628) for u8 / bool sources */
void orc_cast_u8(const uint8_t* src, void* dst, int ddt, int64_t n) {
    for (int64_t i = 0; i < n; ++i) st(dst, ddt, i, (float)src[i]);
}

/* ---- binary with full broadcast (binary_kernel :560, broadcast_offset :534-544) ----
 * kind: 0 add, 1 mul, 2 div, 3 max.  Both operands are already in dtype dt (the host
 * wrapper :3871-3880 converts them first).  out_shape is the broadcast shape. */
static int64_t bcast_offset(int64_t linear, int out_rank, const int64_t* out_shape,
                            int in_rank, const int64_t* in_shape, const int64_t* in_strides) {
    int64_t offset = 0;
    const int shift = out_rank - in_rank;
    for (int d = out_rank - 1; d >= 0; --d) {
        const int64_t c = linear % out_shape[d];
        linear /= out_shape[d];
        const int id = d - shift;
        if (id >= 0 && in_shape[id] != 1) offset += c * in_strides[id];
    }
    return offset;
}
static void strides_of(int rank, const int64_t* shape, int64_t* strides) {
    int64_t s = 1;
    for (int d = rank - 1; d >= 0; --d) { strides[d] = s; s *= shape[d]; }
}
int orc_binary(int kind, const void* a, int a_rank, const int64_t* a_shape,
               const void* b, int b_rank, const int64_t* b_shape,
               void* out, int dt, int64_t* out_shape_ret) {
    const int rank = a_rank > b_rank ? a_rank : b_rank;
    if (rank > ORC_MAX_DIMS) return -1;
    int64_t out_shape[ORC_MAX_DIMS], as[ORC_MAX_DIMS], bs[ORC_MAX_DIMS];
    int64_t count = 1;
    for (int i = 0; i < rank; ++i) {
        const int ai = i - (rank - a_rank), bi = i - (rank - b_rank);
        const int64_t av = ai < 0 ? 1 : a_shape[ai], bv = bi < 0 ? 1 : b_shape[bi];
        if (!(av == bv || av == 1 || bv == 1)) return -2; /* "Incompatible broadcast shapes" */
        out_shape[i] = av > bv ? av : bv;
        count *= out_shape[i];
        if (out_shape_ret) out_shape_ret[i] = out_shape[i];
    }
    strides_of(a_rank, a_shape, as);
    strides_of(b_rank, b_shape, bs);
#pragma omp parallel for schedule(static)
    for (int64_t i = 0; i < count; ++i) {
        const float av = ld(a, dt, bcast_offset(i, rank, out_shape, a_rank, a_shape, as));
        const float bv = ld(b, dt, bcast_offset(i, rank, out_shape, b_rank, b_shape, bs));
        float r;
        if (kind == 0) r = av + bv;
        else if (kind == 1) r = av * bv;
        else if (kind == 2) r = av / bv;
        else r = max_ref(av, bv);
        st(out, dt, i, r);
    }
    return rank;
}

/* ---- unary elementwise (activation_kernel :1098-1109; clamp/exp/sqrt :2188-2206) ----
 * kind 0 SiLU, 1 GELU(erf), 2 GELU(tanh), 3 tanh, 4 ReLU  (enum Activation, backend.h:14)
 * nvcc's default -fmad=true contracts the cubic of GELU-tanh: x + (0.044715f*x*x)*x is one
 * fused multiply-add; written as fmaf here. */
static inline float act_value(int kind, float x) {
    if (kind == 0) return x / (1.0f + expf(-x));
    if (kind == 1) return 0.5f * x * (1.0f + erff(x * 0.7071067811865475f));
    if (kind == 2) {
        const float inner = fmaf(0.044715f * x * x, x, x);
        return 0.5f * x * (1.0f + tanhf(0.7978845608028654f * inner));
    }
    if (kind == 3) return tanhf(x);
    return max_ref(x, 0.0f);
}
void orc_activation(int kind, const void* x, void* out, int dt, int64_t n) {
#pragma omp parallel for schedule(static)
    for (int64_t i = 0; i < n; ++i) st(out, dt, i, act_value(kind, ld(x, dt, i)));
}
void orc_clamp(const void* x, void* out, int dt, int64_t n, float lo, float hi) {
    for (int64_t i = 0; i < n; ++i) st(out, dt, i, -max_ref(-hi, -max_ref(lo, ld(x, dt, i))));
}
void orc_exp(const void* x, void* out, int dt, int64_t n) {
    for (int64_t i = 0; i < n; ++i) st(out, dt, i, expf(ld(x, dt, i)));
}
void orc_sqrt(const void* x, void* out, int dt, int64_t n) {
    for (int64_t i = 0; i < n; ++i) st(out, dt, i, sqrtf(ld(x, dt, i)));
}

/* ---- LayerNorm (layer_norm_parallel_kernel :910-943) ----
 * 256 threads per row, thread t accumulates columns t, t+256, ... in double, pairwise
 * shared-memory tree (stride 128..1).  weight/bias are already in x's dtype (:4069-4070).
 * affine_fma: whether "v *= w; v += b" is evaluated as one fused multiply-add. */
void orc_layer_norm(const void* x, const void* w, const void* b, void* out, int dt,
                    int64_t rows, int64_t width, float eps, int affine_fma) {
#pragma omp parallel for schedule(static)
    for (int64_t row = 0; row < rows; ++row) {
        double sum_ws[256], sq_ws[256];
        for (int t = 0; t < 256; ++t) {
            double s = 0.0, q = 0.0;
            for (int64_t c = t; c < width; c += 256) {
                const float v = ld(x, dt, row * width + c);
                s += v;
                q += (double)v * v;
            }
            sum_ws[t] = s; sq_ws[t] = q;
        }
        for (int stride = 128; stride > 0; stride /= 2)
            for (int t = 0; t < stride; ++t) { sum_ws[t] += sum_ws[t + stride]; sq_ws[t] += sq_ws[t + stride]; }
        const float mean = (float)(sum_ws[0] / (double)width);
        const float inverse = rsqrt_ref((float)(sq_ws[0] / (double)width - (double)mean * mean) + eps);
        for (int64_t c = 0; c < width; ++c) {
            float v = (ld(x, dt, row * width + c) - mean) * inverse;
            if (w && b && affine_fma) v = fmaf(v, ld(w, dt, c), ld(b, dt, c));
            else {
                if (w) v *= ld(w, dt, c);
                if (b) v += ld(b, dt, c);
            }
            st(out, dt, row * width + c, v);
        }
    }
}

/* ---- RMSNorm over the last axis ----
 * rms_contiguous_reduction_lanes (:838-850) picks the launch width; 0 selects the
 * double-accumulating fallback kernels (:963-991, :1013-1040). */
int orc_rms_lanes(int64_t width, int64_t rows) {
    if (width <= 0 || rows <= 0 || (width > 128 && width % 4 != 0)) return 0;
    const int64_t inputs = width > 128 ? width / 4 : width;
    int input_power = 1, row_power = 1;
    while (input_power < 512 && (int64_t)input_power * 2 <= inputs) input_power *= 2;
    while (row_power < 512 && (int64_t)row_power * 2 <= rows) row_power *= 2;
    int lanes = input_power < 32 ? input_power : 32;
    const int row_groups = row_power < 512 / lanes ? row_power : 512 / lanes;
    lanes = input_power < 512 / row_groups ? input_power : 512 / row_groups;
    const int64_t values_per_lane = width / lanes + (width % lanes != 0);
    const int limit = row_groups * 16 < 256 ? row_groups * 16 : 256;
    if (values_per_lane >= limit) return 0;
    return lanes;
}

/* in_dt: dtype of x; out_dt: dtype of the output AND of the weight (the wrapper :4115
 * converts the weight to the output dtype).  rows_for_schedule lets a caller that splits a
 * tensor into row blocks keep the lane count the whole tensor would get. */
void orc_rms_norm(const void* x, int in_dt, const void* w, void* out, int out_dt,
                  int64_t rows, int64_t width, float eps, int64_t rows_for_schedule) {
    const int lanes = orc_rms_lanes(width, rows_for_schedule > 0 ? rows_for_schedule : rows);
#pragma omp parallel for schedule(static)
    for (int64_t row = 0; row < rows; ++row) {
        float inverse;
        if (lanes != 0) {
            /* rms_norm_contiguous_f32_kernel :853-907, explicit round-to-nearest F32 */
            float partials[512];
            for (int lane = 0; lane < lanes; ++lane) {
                float sums[4] = {0.0f, 0.0f, 0.0f, 0.0f};
                if (width > 128) {
                    for (int64_t c = (int64_t)lane * 4; c < width; c += (int64_t)lanes * 4)
                        for (int k = 0; k < 4; ++k) {
                            const float v = ld(x, in_dt, row * width + c + k);
                            sums[k] = sums[k] + v * v;
                        }
                } else {
                    for (int64_t c = lane; c < width; c += (int64_t)lanes * 4)
                        for (int k = 0; k < 4; ++k) {
                            const int64_t idx = c + (int64_t)k * lanes;
                            if (idx < width) {
                                const float v = ld(x, in_dt, row * width + idx);
                                sums[k] = sums[k] + v * v;
                            }
                        }
                }
                partials[lane] = ((sums[0] + sums[1]) + sums[2]) + sums[3];
            }
            for (int offset = lanes / 2; offset >= 32; offset /= 2)
                for (int lane = 0; lane < offset; ++lane) partials[lane] += partials[lane + offset];
            /* shfl_down with offsets 1,2,4,... over the first min(lanes,32) lanes */
            const int warp = lanes < 32 ? lanes : 32;
            float total[32];
            for (int lane = 0; lane < warp; ++lane) total[lane] = partials[lane];
            for (int offset = 1; offset < warp; offset *= 2) {
                float next[32];
                for (int lane = 0; lane < warp; ++lane)
                    next[lane] = total[lane] + (lane + offset < warp ? total[lane + offset] : total[lane]);
                memcpy(total, next, sizeof(float) * (size_t)warp);
            }
            const float mean = total[0] * (1.0f / (float)width);
            inverse = rsqrt_ref(mean + eps);
        } else {
            double ws[256];
            for (int t = 0; t < 256; ++t) {
                double q = 0.0;
                for (int64_t c = t; c < width; c += 256) {
                    const float v = ld(x, in_dt, row * width + c);
                    q += (double)v * v;
                }
                ws[t] = q;
            }
            for (int stride = 128; stride > 0; stride /= 2)
                for (int t = 0; t < stride; ++t) ws[t] += ws[t + stride];
            inverse = rsqrt_ref((float)(ws[0] / (double)width) + eps);
        }
        for (int64_t c = 0; c < width; ++c) {
            float v = ld(x, in_dt, row * width + c) * inverse;
            if (in_dt == ORC_BF16) v = round_bf16(v);
            if (w) v = v * ld(w, out_dt, c);
            st(out, out_dt, row * width + c, v);
        }
    }
}

/* ---- RMSNorm over an inner axis (rms_norm_axis_parallel_kernel :1045-1095) ----
 * 8 reduction lanes per inner position: lane a takes coordinates a, a+8, ...; lanes are
 * combined in lane order; double accumulation. */
void orc_rms_norm_axis(const void* x, const void* w, void* out, int dt,
                       int64_t outer, int64_t axis, int64_t inner, float eps) {
#pragma omp parallel for schedule(static)
    for (int64_t o = 0; o < outer; ++o)
        for (int64_t i = 0; i < inner; ++i) {
            const int64_t base = o * axis * inner + i;
            double lane_sum[8];
            for (int a = 0; a < 8; ++a) {
                double q = 0.0;
                for (int64_t c = a; c < axis; c += 8) {
                    const float v = ld(x, dt, base + c * inner);
                    q += (double)v * v;
                }
                lane_sum[a] = q;
            }
            double total = 0.0;
            for (int a = 0; a < 8; ++a) total += lane_sum[a];
            const float inverse = rsqrt_ref((float)(total / (double)axis) + eps);
            for (int64_t c = 0; c < axis; ++c) {
                float v = ld(x, dt, base + c * inner) * inverse;
                if (dt == ORC_BF16) v = round_bf16(v);
                if (w) v *= ld(w, dt, c);
                st(out, dt, base + c * inner, v);
            }
        }
}

/* ---- pixel_norm (CudaBackend::pixel_norm :5048-5086) over axis 1 of x [outer, channels, inner] ----
 * inner > 1: pixel_norm_strided_axis_kernel :2131-2165 -- 8 channel lanes per position, lane a
 * accumulates channels a, a+8, ... with `square += value * value` (one FFMA after nvcc's
 * contraction), then the shared-memory tree with strides 4, 2, 1.
 * inner == 1: pixel_norm_contiguous_axis_kernel :2097-2126 -- 256 thread partials (thread t takes
 * channels t, t+256, ...), then group_norm_block_sum's tree (:1884-1893, strides 128 ... 1).
 * denominator = sqrtf(total / channels + eps); out = x / denominator, rounded to x's dtype. */
void orc_pixel_norm(const void* x, void* out, int dt, int64_t outer, int64_t channels, int64_t inner, float eps) {
#pragma omp parallel for schedule(static)
    for (int64_t o = 0; o < outer; ++o)
        for (int64_t i = 0; i < inner; ++i) {
            const int64_t base = o * channels * inner + i;
            float total;
            if (inner > 1) {
                float lane[8];
                for (int a = 0; a < 8; ++a) {
                    float q = 0.0f;
                    for (int64_t c = a; c < channels; c += 8) {
                        const float v = ld(x, dt, base + c * inner);
                        q = fmaf(v, v, q);
                    }
                    lane[a] = q;
                }
                for (int stride = 4; stride > 0; stride /= 2)
                    for (int a = 0; a < stride; ++a) lane[a] += lane[a + stride];
                total = lane[0];
            } else {
                float part[256];
                for (int t = 0; t < 256; ++t) {
                    float q = 0.0f;
                    for (int64_t c = t; c < channels; c += 256) {
                        const float v = ld(x, dt, base + c);
                        q = fmaf(v, v, q);
                    }
                    part[t] = q;
                }
                for (int stride = 128; stride > 0; stride /= 2)
                    for (int t = 0; t < stride; ++t) part[t] += part[t + stride];
                total = part[0];
            }
            const float denominator = sqrtf(total / (float)channels + eps);
            for (int64_t c = 0; c < channels; ++c)
                st(out, dt, base + c * inner, ld(x, dt, base + c * inner) / denominator);
        }
}

/* ---- l2_normalize (CudaBackend::l2_normalize :5088-5110, l2_normalize_kernel :1142-1176) ----
 * x [outer, channels, inner], one 256-thread block per (outer, inner) position: thread t adds the squares of
 * channels t, t+256, ... with one FMA each, the block tree (strides 128 ... 1) adds the partials;
 * denominator = sqrtf(total) + eps; out = x / denominator, rounded to x's dtype. */
void orc_l2_normalize(const void* x, void* out, int dt, int64_t outer, int64_t channels, int64_t inner, float eps) {
#pragma omp parallel for schedule(static)
    for (int64_t o = 0; o < outer; ++o)
        for (int64_t i = 0; i < inner; ++i) {
            const int64_t base = o * channels * inner + i;
            float part[256];
            for (int t = 0; t < 256; ++t) {
                float q = 0.0f;
                for (int64_t c = t; c < channels; c += 256) {
                    const float v = ld(x, dt, base + c * inner);
                    q = fmaf(v, v, q);
                }
                part[t] = q;
            }
            for (int stride = 128; stride > 0; stride /= 2)
                for (int t = 0; t < stride; ++t) part[t] += part[t + stride];
            const float denominator = sqrtf(part[0]) + eps;
            for (int64_t c = 0; c < channels; ++c)
                st(out, dt, base + c * inner, ld(x, dt, base + c * inner) / denominator);
        }
}

/* ---- RoPE (rope_kernel :1200-1215): adjacent pairs, two separately rounded products ---- */
int orc_rope(const void* x, int x_dt, int x_rank, const int64_t* x_shape,
             const void* cosine, const void* sine, int f_dt, int f_rank, const int64_t* f_shape,
             void* out) {
    if (x_rank > ORC_MAX_DIMS || f_rank > x_rank) return -1;
    int64_t fs[ORC_MAX_DIMS];
    strides_of(f_rank, f_shape, fs);
    int64_t count = 1;
    for (int d = 0; d < x_rank; ++d) count *= x_shape[d];
    const int64_t width = x_shape[x_rank - 1];
    if (width % 2) return -2; /* "RoPE width must be even" :4200 */
#pragma omp parallel for schedule(static)
    for (int64_t i = 0; i < count; ++i) {
        const int64_t pair = (i % width) ^ 1;
        const int64_t paired_index = i - i % width + pair;
        const float paired = ld(x, x_dt, paired_index);
        const float rotated = (i & 1) ? paired : -paired;
        const int64_t f = bcast_offset(i, x_rank, x_shape, f_rank, f_shape, fs);
        const float first = ld(x, x_dt, i) * ld(cosine, f_dt, f);
        const float second = rotated * ld(sine, f_dt, f);
        st(out, x_dt, i, first + second);
    }
    return 0;
}

/* ---- weight dequantisation (decode_fp8_e4m3fn :630-638, dequantize_kernel :641-658) ----
 * kind 0 FP8-e4m3fn (no NaN case: 0x7f / 0xff decode to +-480), 1 INT8, 2 INT4 low nibble
 * first. */
float orc_decode_fp8(uint8_t raw) {
    const int sign = raw >> 7, exponent = (raw >> 3) & 0xf, mantissa = raw & 0x7;
    float value;
    if (exponent == 0) value = ldexpf((float)mantissa, -9);
    else value = ldexpf(1.0f + (float)mantissa / 8.0f, exponent - 7);
    return sign ? -value : value;
}
void orc_dequant(int kind, const uint8_t* packed, const float* scales, void* out, int out_dt,
                 int64_t count, int64_t inner, int64_t groups, int64_t group_size) {
#pragma omp parallel for schedule(static)
    for (int64_t i = 0; i < count; ++i) {
        float q;
        if (kind == 0) q = orc_decode_fp8(packed[i]);
        else if (kind == 1) q = (float)(int8_t)packed[i];
        else {
            const uint8_t byte = packed[i / 2];
            const uint8_t nibble = (i & 1) ? (uint8_t)(byte >> 4) : (uint8_t)(byte & 0xf);
            q = (float)(nibble >= 8 ? (int)nibble - 16 : (int)nibble);
        }
        const int64_t outer = i / inner, group = (i % inner) / group_size;
        st(out, out_dt, i, q * scales[outer * groups + group]);
    }
}

/* ---- GroupNorm (:1884-2030, host :4919-5008) ----
 * Unit = (batch, group); anchor = first element; pass 1 mean of (x - anchor), pass 2 centred
 * sum of squares, all F32; 256-thread strided partial sums, pairwise tree; large units are
 * split into `partials` blocks whose totals a 256-thread tree adds.  nvcc contracts
 * "square += delta*delta" and "normalized*scale + shift" to fused multiply-adds.
 * weight/bias are already in x's dtype.  sm_count enters the partial count (:4951-4961). */
static float block_tree_sum(float* ws /* 256 entries */) {
    for (int stride = 128; stride > 0; stride /= 2)
        for (int t = 0; t < stride; ++t) ws[t] += ws[t + stride];
    return ws[0];
}
int orc_group_norm_partials(int64_t units, int64_t count, int sm_count) {
    if (count <= (1LL << 18)) return 0;
    const int work = (int)((count + (1LL << 20) - 1) / (1LL << 20));
    const int occupancy = (int)((2LL * sm_count + units - 1) / units);
    int64_t useful64 = (count + 255) / 256;
    const int useful = (int)(useful64 < 32 ? useful64 : 32);
    int m = 2;
    if (work > m) m = work;
    if (occupancy > m) m = occupancy;
    if (m < 2) m = 2;
    if (m > 32) m = 32;
    return useful < m ? useful : m;
}
void orc_group_norm(const void* x, const void* w, const void* b, void* out, int dt,
                    int64_t batch, int64_t channels, int64_t spatial, int groups, float eps,
                    int sm_count, float* mean_out, float* inverse_out) {
    const int64_t units = batch * groups;
    const int64_t channels_per = channels / groups;
    const int64_t count = channels_per * spatial;
    const int partials = orc_group_norm_partials(units, count, sm_count);
#pragma omp parallel for schedule(dynamic, 1)
    for (int64_t unit = 0; unit < units; ++unit) {
        const int64_t base = unit * count;
        const int group = (int)(unit % groups);
        const float anchor = ld(x, dt, base);
        float ws[256], mean, inverse;
        if (partials == 0) {
            for (int t = 0; t < 256; ++t) {
                float s = 0.0f;
                for (int64_t i = t; i < count; i += 256) s += ld(x, dt, base + i) - anchor;
                ws[t] = s;
            }
            mean = anchor + block_tree_sum(ws) / (float)count;
            for (int t = 0; t < 256; ++t) {
                float q = 0.0f;
                for (int64_t i = t; i < count; i += 256) {
                    const float d = ld(x, dt, base + i) - mean;
                    q = fmaf(d, d, q);
                }
                ws[t] = q;
            }
            inverse = rsqrt_ref(block_tree_sum(ws) / (float)count + eps);
        } else {
            float part[32];
            for (int p = 0; p < partials; ++p) {
                for (int t = 0; t < 256; ++t) {
                    float s = 0.0f;
                    for (int64_t i = (int64_t)p * 256 + t; i < count; i += (int64_t)partials * 256)
                        s += ld(x, dt, base + i) - anchor;
                    ws[t] = s;
                }
                part[p] = block_tree_sum(ws);
            }
            for (int t = 0; t < 256; ++t) ws[t] = t < partials ? part[t] : 0.0f;
            mean = anchor + block_tree_sum(ws) / (float)count;
            for (int p = 0; p < partials; ++p) {
                for (int t = 0; t < 256; ++t) {
                    float q = 0.0f;
                    for (int64_t i = (int64_t)p * 256 + t; i < count; i += (int64_t)partials * 256) {
                        const float d = ld(x, dt, base + i) - mean;
                        q = fmaf(d, d, q);
                    }
                    ws[t] = q;
                }
                part[p] = block_tree_sum(ws);
            }
            for (int t = 0; t < 256; ++t) ws[t] = t < partials ? part[t] : 0.0f;
            inverse = rsqrt_ref(block_tree_sum(ws) / (float)count + eps);
        }
        if (mean_out) mean_out[unit] = mean;
        if (inverse_out) inverse_out[unit] = inverse;
        for (int64_t c = 0; c < channels_per; ++c) {
            const int64_t ac = (int64_t)group * channels_per + c;
            const float scale = w ? ld(w, dt, ac) : 1.0f;
            const float shift = b ? ld(b, dt, ac) : 0.0f;
            const int64_t cb = base + c * spatial;
            for (int64_t p = 0; p < spatial; ++p) {
                const float normalized = (ld(x, dt, cb + p) - mean) * inverse;
                st(out, dt, cb + p, fmaf(normalized, scale, shift));
            }
        }
    }
}
