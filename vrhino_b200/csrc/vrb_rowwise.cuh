// Row-wise normalisation kernel family (LayerNorm / RMSNorm) fused with the operator the
// reference's pipelines apply next: adaLN modulation, the Mochi (1+scale) product, RoPE, or a
// gated residual.  One pass over HBM: a row is loaded once with 128-bit loads, kept PACKED in
// registers while its statistics are reduced, then normalised, post-processed and stored.
// Every rounding the reference's chain of separate kernels performs between its steps is
// reproduced in registers.
//
// Work split: `tpr` threads (8..256, power of two) cooperate on one normalised row, each
// holding NCH chunks of 8 elements.  Rows narrower than a warp pack several rows into one
// warp; a row of at most 32*6 chunks stays inside one warp and needs no barrier at all; wider
// rows exchange one partial per warp through shared memory under a NAMED barrier that only the
// warps of that row wait on, so the rows of a CTA never wait for each other.
//
// At 6.5 TB/s an SM has about 22 issue slots per bf16 element it streams, so the per-element
// instruction count is what decides whether these kernels reach the HBM roofline.  Hence:
// dtype classes are template parameters (no per-element dtype tests), bf16 roundings are done
// two at a time (cvt.rn.bf16x2.f32), and the statistics are accumulated per thread in F32
// (at most 64 terms, pairwise inside a chunk) and only then widened to double for the
// cross-thread reduction and the final mean / variance formula.
//
// Latency: the exact geometries (production widths) prefetch the next row into a second packed
// register set while the current one is reduced; everything a row needs besides x -- its RoPE
// table row, its residual row -- is requested BEFORE the statistics so that it arrives during the
// reduction instead of stalling the epilogue; vectors shared by all rows (1+scale | shift, LayerNorm
// weight | bias) are staged once per CTA in shared memory in a bank-conflict-free layout.
//
// Reference semantics restated (native/src/backend/cuda/cuda_backend.cu):
//   layer_norm_parallel_kernel :910-943  sum / sum of squares (double in the reference),
//       mean = float(S/W), inv = rsqrtf(float(Q/W - double(mean)*mean) + eps),
//       (x-mean)*inv [*w] [+b]
//   rms_norm_contiguous_f32_kernel :853-907  F32 sum of squares, mean = S*(1/W),
//       inv = rsqrtf(mean+eps), x*inv, round to bf16 if the input is bf16, *w
//   rms_norm_parallel_kernel :963-991 (and :1013-1040)  same with a double sum and
//       inv = rsqrtf(float(Q/W) + eps); chosen by rms_contiguous_reduction_lanes :838-850
//   rope_kernel :1200-1215; modulate / gated_residual: native/src/architectures/common.cpp
#pragma once

#include "vrb_common.cuh"

namespace vrb {
namespace rowwise {

enum Norm { kNormLayer = 1, kNormRms = 2 };
enum Post {
    kPostNone = 0, kPostModulate = 1, kPostScaleX = 2, kPostRope = 3, kPostGatedResidual = 4,
    kPostModulateStaged = 5,   // modulate with one vector for all rows, staged in shared memory
    kPostRopeShared = 6,       // RoPE whose table columns do not depend on the thread's chunk index
};
// dtype class of (x, output of the unfused norm operator)
// kBf16Bf16Pre: like kBf16Bf16, but the row the norm sees is first COMPUTED as the bf16 gated
// residual  state = residual + branch * gate  (common.cpp:134-144 in a bf16 residual stream) and
// stored to state_out -- the residual update and the norm that follows it in one pass.
enum DtClass { kF32F32 = 0, kBf16Bf16 = 1, kBf16F32 = 2, kBf16Bf16Pre = 3, kF32Pre = 4 };
// kF32Pre: like kBf16Bf16Pre with an F32 residual stream (the production contract): x F32, branch bf16,
// gate in F32, the updated stream stored F32, then the kF32F32 norm.

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
    int rms_f64;               // RMS: the reference's double-accumulating fallback formula
    int tpr;                   // threads per normalised row
    unsigned nrows32, sub32;   // normalised rows, normalised rows per storage row
    double inv_width;          // 1 / norm_width
    int affine_staged;         // LayerNorm weight / bias pre-rounded into shared memory
    // kBf16Bf16Pre: x is the residual stream, pre_branch the branch, pre_gate an optional gate
    // ([pre_vectors, width], staged bf16-rounded), state_out receives the updated stream
    const void* pre_branch; const void* pre_gate; void* state_out;
    int pre_gate_dt;
    int64_t pre_rows_per_vector, pre_vectors;
    // kBf16Bf16Pre, Mochi's form (mochi.cpp:204-211): the branch is RMS-normalised (no weight, pre_eps) before
    // it is gated and added, and the gate is tanh(pre_gate)
    int pre_norm, pre_gate_tanh;
    float pre_eps;
    // Two problems in one launch (q and k of an attention block: same geometry, dtypes, tables and
    // epilogue, their own tensors, weights and row counts): CTAs [0, blocks_a) work on (x, out, weight,
    // nrows32), the others on (x_b, out_b, weight_b, nrows_b).  blocks_a == 0: a single problem.
    const void* x_b; void* out_b; const void* weight_b;
    unsigned nrows_b, blocks_a;
};

constexpr int kRowThreads = 256;

#ifdef __CUDACC__

template <bool X_BF16> struct Packed;
template <> struct Packed<true> { uint4 r; };
template <> struct Packed<false> { float4 a, b; };

template <bool X_BF16>
__device__ __forceinline__ Packed<X_BF16> load_packed(const void* base, int64_t e) {
    Packed<X_BF16> c;
    if constexpr (X_BF16) c.r = __ldcs(reinterpret_cast<const uint4*>(static_cast<const uint16_t*>(base) + e));
    else {
        const float4* p = reinterpret_cast<const float4*>(static_cast<const float*>(base) + e);
        c.a = __ldcs(p); c.b = __ldcs(p + 1);
    }
    return c;
}
template <bool X_BF16>
__device__ __forceinline__ Packed<X_BF16> zero_packed() {
    Packed<X_BF16> c;
    if constexpr (X_BF16) c.r = make_uint4(0, 0, 0, 0);
    else { c.a = make_float4(0, 0, 0, 0); c.b = c.a; }
    return c;
}
template <bool X_BF16>
__device__ __forceinline__ void unpack(const Packed<X_BF16>& c, float (&v)[8]) {
    if constexpr (X_BF16) {
        v[0] = __uint_as_float(c.r.x << 16); v[1] = __uint_as_float(c.r.x & 0xffff0000u);
        v[2] = __uint_as_float(c.r.y << 16); v[3] = __uint_as_float(c.r.y & 0xffff0000u);
        v[4] = __uint_as_float(c.r.z << 16); v[5] = __uint_as_float(c.r.z & 0xffff0000u);
        v[6] = __uint_as_float(c.r.w << 16); v[7] = __uint_as_float(c.r.w & 0xffff0000u);
    } else {
        v[0] = c.a.x; v[1] = c.a.y; v[2] = c.a.z; v[3] = c.a.w;
        v[4] = c.b.x; v[5] = c.b.y; v[6] = c.b.z; v[7] = c.b.w;
    }
}

// Round eight values to bf16 precision, two per conversion instruction.
__device__ __forceinline__ void round8_bf16(float (&v)[8]) {
#pragma unroll
    for (int e = 0; e < 8; e += 2) {
        const uint32_t h = pack_bf16x2(v[e], v[e + 1]);
        v[e] = __uint_as_float(h << 16);
        v[e + 1] = __uint_as_float(h & 0xffff0000u);
    }
}
template <bool BF16>
__device__ __forceinline__ void round8(float (&v)[8]) {
    if constexpr (BF16) round8_bf16(v);
}
__device__ __forceinline__ void round8_rt(int dt, float (&v)[8]) {
    if (dt == VRB_BF16) round8_bf16(v);
}

// ---- scalar forms of the per-element pipeline (used by the any-width kernel) --------------
template <int NORM>
__device__ __forceinline__ float normalise(const RowParams& p, float x, float mean, float inv,
                                           float w, float b, bool has_w, bool has_b, bool x_bf16) {
    float v;
    if constexpr (NORM == kNormLayer) {
        v = __fmul_rn(__fsub_rn(x, mean), inv);
        if (has_w && has_b && p.affine_fma) v = __fmaf_rn(v, w, b);
        else {
            if (has_w) v = __fmul_rn(v, w);
            if (has_b) v = __fadd_rn(v, b);
        }
    } else {
        v = __fmul_rn(x, inv);
        if (x_bf16) v = round_to_bf16(v);
        if (has_w) v = __fmul_rn(v, w);
    }
    return round_to(p.norm_out_dt, v);
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

__device__ __forceinline__ void named_barrier(int id, int threads) {
    asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(threads) : "memory");
}

// Staging of per-CTA vectors: `groups` float4 groups, up to four loads in flight per thread before
// the first store, so a CTA pays the L2 / DRAM latency once instead of once per loop iteration (the
// staging is a fixed cost of every launch; it is what a short launch on a token shard feels most).
template <typename Load, typename Store>
__device__ __forceinline__ void stage_groups(int groups, Load load, Store store) {
    for (int g0 = threadIdx.x; g0 < groups; g0 += 4 * kRowThreads) {
        float4 v[4];
#pragma unroll
        for (int k = 0; k < 4; ++k) {
            const int g = g0 + k * kRowThreads;
            if (g < groups) v[k] = load(g);
        }
#pragma unroll
        for (int k = 0; k < 4; ++k) {
            const int g = g0 + k * kRowThreads;
            if (g < groups) store(g, v[k]);
        }
    }
}
__device__ __forceinline__ bool f32_vector_ok(const void* p, int dt) {
    return dt == VRB_F32 && (reinterpret_cast<uintptr_t>(p) & 15u) == 0;
}

// ---- vector kernel: norm_width % 8 == 0, 16-byte aligned operands ------------------------
// CTAs per SM the register allocator must leave room for: the packed row takes 4 (bf16) or 8
// (f32) registers per chunk; the rest of the budget is working state.
__host__ __device__ constexpr int packed_regs(int nch, bool x_bf16) { return nch * (x_bf16 ? 4 : 8); }
// The exact geometries prefetch the next row into a second register set while the current one
// is being processed, if two packed rows fit in 48 registers.
__host__ __device__ constexpr bool prefetches(int nch, bool x_bf16, bool full) { return full && 2 * packed_regs(nch, x_bf16) <= 48; }
// The fused residual update (dtype class kBf16Bf16Pre) loads two raw rows (residual stream and
// branch) per normalised row.  With no epilogue operands (plain or affine LayerNorm) it keeps the
// next pair in flight in a second register set; with a modulating epilogue the extra registers
// spill, and one more resident CTA without the prefetch measured faster.
__host__ __device__ constexpr bool pre_prefetches(int nch, bool full, int post) {
    return prefetches(nch, true, full) && post == kPostNone;
}
__host__ __device__ constexpr int min_ctas_per_sm(int nch, bool x_bf16, bool full, bool pre = false, int post = kPostNone) {
    if (pre && x_bf16 && full && prefetches(nch, true, full) && !pre_prefetches(nch, full, post)) return 3;
    const int sets = (prefetches(nch, x_bf16, full) ? 2 : 1) + (pre ? 1 : 0);
    const int row_regs = packed_regs(nch, x_bf16) * sets;
    return row_regs <= 16 ? 4 : row_regs <= 32 ? 3 : 2;
}

// Geometry: TPR == 0 reads the threads-per-row from the parameters and guards every chunk;
// TPR > 0 with FULL means the row is exactly NCH * TPR chunks wide, so chunk offsets are
// compile-time constants and no chunk needs a bounds test (the production widths).
template <int NCH, int TPR, bool FULL, int NORM, int POST, int DT>
__global__ void __launch_bounds__(kRowThreads, min_ctas_per_sm(NCH, DT != kF32F32 && DT != kF32Pre, FULL,
                                                              DT == kBf16Bf16Pre || DT == kF32Pre, POST))
row_kernel(const RowParams p) {
    constexpr bool X_BF16 = DT != kF32F32 && DT != kF32Pre;
    constexpr bool PRE = DT == kBf16Bf16Pre || DT == kF32Pre;
    constexpr bool PRE_F32 = DT == kF32Pre;
    constexpr bool PF = PRE ? (X_BF16 && pre_prefetches(NCH, FULL, POST)) : prefetches(NCH, X_BF16, FULL);
    constexpr bool N_BF16 = DT == kBf16Bf16 || DT == kBf16Bf16Pre;   // the unfused norm operator would store bf16
    constexpr bool kStaged = POST == kPostModulateStaged;
    constexpr bool kModulate = POST == kPostModulate || kStaged;
    constexpr bool kRope = POST == kPostRope || POST == kPostRopeShared;
    __shared__ double s_red[2][kRowThreads / 32][2];
    extern __shared__ __align__(16) float s_vec[];   // staged modulate: [1+scale | shift], each NCH*tpr*8 floats
    const int tpr = TPR ? TPR : p.tpr;
    const int lane_in_row = threadIdx.x & (tpr - 1);
    const int row_in_cta = threadIdx.x / tpr;
    const int rows_per_cta = kRowThreads / tpr;
    const int nchunks = FULL ? NCH * TPR : static_cast<int>(p.norm_width >> 3);
    const int width = nchunks * 8;
    const int warps_per_row = tpr >> 5;
    // this CTA's problem: the only one, or one of a pair
    unsigned block = blockIdx.x, blocks = gridDim.x, nrows = p.nrows32;
    const void* x_base = p.x;
    void* out_base = p.out;
    const void* weight_base = p.weight;
    if (p.blocks_a != 0) {
        if (block >= p.blocks_a) {
            block -= p.blocks_a; blocks -= p.blocks_a;
            nrows = p.nrows_b; x_base = p.x_b; out_base = p.out_b; weight_base = p.weight_b;
        } else {
            blocks = p.blocks_a;
        }
    }
    const bool has_w = weight_base != nullptr, has_b = p.bias != nullptr;
    const bool has_shift = p.shift != nullptr;
    const bool f32_formula = NORM == kNormRms && !p.rms_f64;
    int parity = 0;

    // nothing below this line may run before the previous kernel of the stream has completed: the
    // vectors staged next are caller memory like the rows themselves
    pdl_launch_dependents();
    pdl_wait();

    // LayerNorm weight / bias, already converted to x's dtype, staged once per CTA (same
    // conflict-free layout as the modulation vectors, placed before them)
    const int pad = NCH * tpr * 8;
    float* const s_mod = s_vec + (p.affine_staged ? 2 * pad : 0);
    // float4 group g of a staged vector (elements 4g .. 4g+3 of the row) -> float4 slot in shared memory
    auto group_slot = [&](int g) {
        const int chunk = g >> 1, i = chunk / tpr, l = chunk - i * tpr;
        return (i * 2 + (g & 1)) * tpr + l;
    };
    if (NORM == kNormLayer && p.affine_staged) {
        const bool fast_w = !has_w || f32_vector_ok(p.weight, p.w_dt), fast_b = !has_b || f32_vector_ok(p.bias, p.b_dt);
        if (fast_w && fast_b && (width & 3) == 0) {
            const bool to_bf16 = p.x_dt == VRB_BF16;
            auto rounded = [&](float4 v) {
                if (to_bf16) { v.x = round_to_bf16(v.x); v.y = round_to_bf16(v.y); v.z = round_to_bf16(v.z); v.w = round_to_bf16(v.w); }
                return v;
            };
            stage_groups(width >> 2,
                         [&](int g) { return has_w ? __ldg(static_cast<const float4*>(p.weight) + g) : make_float4(1.f, 1.f, 1.f, 1.f); },
                         [&](int g, float4 v) { reinterpret_cast<float4*>(s_vec)[group_slot(g)] = rounded(v); });
            stage_groups(width >> 2,
                         [&](int g) { return has_b ? __ldg(static_cast<const float4*>(p.bias) + g) : make_float4(0.f, 0.f, 0.f, 0.f); },
                         [&](int g, float4 v) { reinterpret_cast<float4*>(s_vec + pad)[group_slot(g)] = rounded(v); });
        } else {
            for (int c = threadIdx.x; c < width; c += kRowThreads) {
                const int chunk = c >> 3, e = c & 7, i = chunk / tpr, l = chunk - i * tpr;
                const int pos = (((i * 2 + (e >> 2)) * tpr + l) << 2) + (e & 3);
                s_vec[pos] = has_w ? round_to(p.x_dt, load1(p.weight, p.w_dt, c)) : 1.0f;
                s_vec[pad + pos] = has_b ? round_to(p.x_dt, load1(p.bias, p.b_dt, c)) : 0.0f;
            }
        }
        if constexpr (!kStaged) __syncthreads();
    }
    if constexpr (kStaged) {
        // a few modulation vectors (one per batch entry): keep 1+scale and shift in shared memory,
        // vector v at s_mod + v * 2 * pad
        // layout: for chunk (l + i*tpr) the two float4 halves sit at float4 index (2i + half)*tpr + l,
        // so the lanes of a warp read consecutive 16-byte words (no bank conflicts)
        const int staged_vectors = static_cast<int>(p.vectors);
        if (f32_vector_ok(p.scale, p.mod_dt) && (!has_shift || f32_vector_ok(p.shift, p.mod_dt)) && p.width == width) {
            // vector v's groups follow vector v-1's (the vectors are contiguous rows of `width` elements)
            const int per_vector = width >> 2;
            auto slot = [&](int g) {
                const int v = g / per_vector;
                return v * (2 * pad / 4) + group_slot(g - v * per_vector);
            };
            stage_groups(per_vector * staged_vectors,
                         [&](int g) { return __ldg(static_cast<const float4*>(p.scale) + g); },
                         [&](int g, float4 v) {
                             reinterpret_cast<float4*>(s_mod)[slot(g)] =
                                 make_float4(__fadd_rn(1.0f, v.x), __fadd_rn(1.0f, v.y), __fadd_rn(1.0f, v.z), __fadd_rn(1.0f, v.w));
                         });
            stage_groups(per_vector * staged_vectors,
                         [&](int g) { return has_shift ? __ldg(static_cast<const float4*>(p.shift) + g) : make_float4(0.f, 0.f, 0.f, 0.f); },
                         [&](int g, float4 v) { reinterpret_cast<float4*>(s_mod + pad)[slot(g)] = v; });
        } else {
            for (int cv = threadIdx.x; cv < width * staged_vectors; cv += kRowThreads) {
                const int v = cv / width, c = cv - v * width;
                const int chunk = c >> 3, e = c & 7, i = chunk / tpr, l = chunk - i * tpr;
                const int pos = v * 2 * pad + (((i * 2 + (e >> 2)) * tpr + l) << 2) + (e & 3);
                s_mod[pos] = __fadd_rn(1.0f, load1(p.scale, p.mod_dt, static_cast<int64_t>(v) * p.width + c));
                s_mod[pad + pos] = has_shift ? load1(p.shift, p.mod_dt, static_cast<int64_t>(v) * p.width + c) : 0.0f;
            }
        }
        __syncthreads();
    }
    // kBf16Bf16Pre: the gate vectors, rounded to bf16 and packed in pairs, one 16-byte word per chunk
    // at word index i * tpr + l (conflict-free); vector v at s_gate + v * (pad / 2)
    uint32_t* const s_gate = reinterpret_cast<uint32_t*>(s_mod + (kStaged ? static_cast<int>(p.vectors) * 2 * pad : 0));
    const bool has_pre_gate = PRE && p.pre_gate != nullptr;
    if constexpr (PRE) {
        if (has_pre_gate && PRE_F32) {
            // F32 stream: the gate stays F32, in the modulation vectors' layout, vector v at s_gate + v * pad
            float* const gate_f32 = reinterpret_cast<float*>(s_gate);
            const int gate_vectors = static_cast<int>(p.pre_vectors);
            for (int cv = threadIdx.x; cv < width * gate_vectors; cv += kRowThreads) {
                const int v = cv / width, c = cv - v * width;
                const int chunk = c >> 3, e = c & 7, i = chunk / tpr, l = chunk - i * tpr;
                gate_f32[v * pad + (((i * 2 + (e >> 2)) * tpr + l) << 2) + (e & 3)] =
                    load1(p.pre_gate, p.pre_gate_dt, static_cast<int64_t>(v) * p.width + c);
            }
            __syncthreads();
        } else if (has_pre_gate) {
            const int gate_vectors = static_cast<int>(p.pre_vectors);
            for (int cv = threadIdx.x; cv < (width / 2) * gate_vectors; cv += kRowThreads) {
                const int v = cv / (width / 2), pair = cv - v * (width / 2);
                const int c = pair * 2, chunk = c >> 3, i = chunk / tpr, l = chunk - i * tpr;
                const int64_t at = static_cast<int64_t>(v) * p.width + c;
                float g0 = load1(p.pre_gate, p.pre_gate_dt, at), g1 = load1(p.pre_gate, p.pre_gate_dt, at + 1);
                if (p.pre_gate_tanh) {   // activation(gate, Tanh) in the gate's dtype, then the cast to the stream's
                    g0 = round_to(p.pre_gate_dt, tanhf(g0));
                    g1 = round_to(p.pre_gate_dt, tanhf(g1));
                }
                s_gate[v * (pad / 2) + ((i * tpr + l) << 2) + ((c & 7) >> 1)] = pack_bf16x2(g0, g1);
            }
            __syncthreads();
        }
    }
    // elements of this thread that exist (a partial last chunk never happens: width % 8 == 0)
    int own = 0;
#pragma unroll
    for (int i = 0; i < NCH; ++i) own += (FULL || lane_in_row + i * tpr < nchunks) ? 8 : 0;

    const unsigned row_step = blocks * rows_per_cta;
    auto load_row = [&](unsigned first_row, Packed<X_BF16> (&dst)[NCH]) {
        const unsigned r = first_row + row_in_cta;
        const bool ok = r < nrows;
        const int64_t off = static_cast<int64_t>(r) * width;
#pragma unroll
        for (int i = 0; i < NCH; ++i) {
            const int chunk = lane_in_row + i * tpr;
            dst[i] = (ok && (FULL || chunk < nchunks)) ? load_packed<X_BF16>(x_base, off + chunk * 8) : zero_packed<X_BF16>();
        }
    };
    // kBf16Bf16Pre: the raw residual-stream row and branch row of a normalised row
    auto load_raw = [&](unsigned first_row, Packed<true> (&res)[NCH], Packed<true> (&br)[NCH]) {
        const unsigned r = first_row + row_in_cta;
        const bool ok = r < nrows;
        const int64_t off = static_cast<int64_t>(r) * width;
#pragma unroll
        for (int i = 0; i < NCH; ++i) {
            const int chunk = lane_in_row + i * tpr;
            const bool here = ok && (FULL || chunk < nchunks);
            if constexpr (!PRE_F32) res[i] = here ? load_packed<true>(x_base, off + chunk * 8) : zero_packed<true>();
            br[i] = here ? load_packed<true>(p.pre_branch, off + chunk * 8) : zero_packed<true>();
        }
    };
    // RMS statistics of one row from this thread's sum of squares: warp shuffles, one partial per warp
    // through shared memory for rows wider than a warp, then the reference's formula (:853-907 / :963-991).
    auto rms_inverse = [&](float squares, float eps) -> float {
        const int span = tpr < 32 ? tpr : 32;
        double wide = static_cast<double>(squares);
        for (int offset = span >> 1; offset > 0; offset >>= 1) {
            if (f32_formula) squares = __fadd_rn(squares, __shfl_xor_sync(0xffffffffu, squares, offset));
            else wide += __shfl_xor_sync(0xffffffffu, wide, offset);
        }
        if (warps_per_row > 1) {
            if ((threadIdx.x & 31) == 0) s_red[parity][threadIdx.x >> 5][1] = f32_formula ? static_cast<double>(squares) : wide;
            named_barrier(1 + row_in_cta, tpr);
            const int first = row_in_cta * warps_per_row;
            squares = 0.0f; wide = 0.0;
            for (int w = 0; w < warps_per_row; ++w) {
                if (f32_formula) squares = __fadd_rn(squares, static_cast<float>(s_red[parity][first + w][1]));
                else wide += s_red[parity][first + w][1];
            }
            parity ^= 1;
        }
        if (f32_formula) return rsqrtf(__fadd_rn(__fmul_rn(squares, __fdiv_rn(1.0f, static_cast<float>(width))), eps));
        return rsqrtf(static_cast<float>(wide * p.inv_width) + eps);
    };
    Packed<X_BF16> xr[NCH];
    Packed<true> raw_res[(PRE && !PRE_F32) ? NCH : 1], raw_br[PRE ? NCH : 1];   // PRE: the row being combined next
    if constexpr (PRE) {
        if constexpr (PF) load_raw(block * rows_per_cta, raw_res, raw_br);
    } else if constexpr (PF) {
        load_row(block * rows_per_cta, xr);
    }

    for (unsigned base = block * rows_per_cta; base < nrows; base += row_step) {
        const unsigned nrow = base + row_in_cta;
        const bool valid = nrow < nrows;
        const int64_t row_offset = static_cast<int64_t>(nrow) * width;

        Packed<X_BF16> xn[(PF && !PRE) ? NCH : 1];
        if constexpr (PRE_F32) {
            // F32 stream: state = residual + F32(branch) * gate, product and sum each rounded once in F32
            // (common.cpp:134-144 with T = F32), stored F32 and normalised from the registers
            load_row(base, xr);
            (void)raw_res;
#pragma unroll
            for (int i = 0; i < NCH; ++i) {
                const int chunk = lane_in_row + i * tpr;
                const bool here = valid && (FULL || chunk < nchunks);
                raw_br[i] = here ? load_packed<true>(p.pre_branch, row_offset + chunk * 8) : zero_packed<true>();
            }
            unsigned gate_base = 0;
            if (has_pre_gate && p.pre_vectors > 1)
                gate_base = ((nrow / static_cast<unsigned>(p.pre_rows_per_vector)) % static_cast<unsigned>(p.pre_vectors)) *
                            static_cast<unsigned>(pad);
            const float* const gate_f32 = reinterpret_cast<const float*>(s_gate) + gate_base;
#pragma unroll
            for (int i = 0; i < NCH; ++i) {
                const int chunk = lane_in_row + i * tpr;
                if (!FULL && chunk >= nchunks) continue;
                const uint32_t bw[4] = {raw_br[i].r.x, raw_br[i].r.y, raw_br[i].r.z, raw_br[i].r.w};
                float b[8];
#pragma unroll
                for (int k = 0; k < 4; ++k) { b[2 * k] = __uint_as_float(bw[k] << 16); b[2 * k + 1] = __uint_as_float(bw[k] & 0xffff0000u); }
                if (has_pre_gate) {
                    const float4 g0 = *reinterpret_cast<const float4*>(gate_f32 + (((i * 2) * tpr + lane_in_row) << 2));
                    const float4 g1 = *reinterpret_cast<const float4*>(gate_f32 + (((i * 2 + 1) * tpr + lane_in_row) << 2));
                    b[0] = __fmul_rn(b[0], g0.x); b[1] = __fmul_rn(b[1], g0.y); b[2] = __fmul_rn(b[2], g0.z); b[3] = __fmul_rn(b[3], g0.w);
                    b[4] = __fmul_rn(b[4], g1.x); b[5] = __fmul_rn(b[5], g1.y); b[6] = __fmul_rn(b[6], g1.z); b[7] = __fmul_rn(b[7], g1.w);
                }
                xr[i].a = make_float4(__fadd_rn(xr[i].a.x, b[0]), __fadd_rn(xr[i].a.y, b[1]), __fadd_rn(xr[i].a.z, b[2]), __fadd_rn(xr[i].a.w, b[3]));
                xr[i].b = make_float4(__fadd_rn(xr[i].b.x, b[4]), __fadd_rn(xr[i].b.y, b[5]), __fadd_rn(xr[i].b.z, b[6]), __fadd_rn(xr[i].b.w, b[7]));
                if (valid) {
                    store32(static_cast<float*>(p.state_out) + row_offset + chunk * 8,
                            make_uint4(__float_as_uint(xr[i].a.x), __float_as_uint(xr[i].a.y), __float_as_uint(xr[i].a.z), __float_as_uint(xr[i].a.w)),
                            make_uint4(__float_as_uint(xr[i].b.x), __float_as_uint(xr[i].b.y), __float_as_uint(xr[i].b.z), __float_as_uint(xr[i].b.w)));
                }
            }
        } else if constexpr (PRE) {
            if constexpr (!PF) load_raw(base, raw_res, raw_br);
            // state = residual + branch * gate in packed bf16 (two roundings, as the reference's
            // F32 multiply and add each followed by the bf16 store), written back as the new stream
            unsigned gate_base = 0;
            if (has_pre_gate && p.pre_vectors > 1)
                gate_base = ((nrow / static_cast<unsigned>(p.pre_rows_per_vector)) % static_cast<unsigned>(p.pre_vectors)) *
                            static_cast<unsigned>(pad / 2);
            // Mochi: the branch enters as rms_norm(branch, no weight, pre_eps), rounded to bf16 like the
            // operator's own store (absent chunks were loaded as zeros)
            float branch_inverse = 1.0f;
            if (p.pre_norm) {
                unsigned long long squares = 0ull;
#pragma unroll
                for (int i = 0; i < NCH; ++i) {
                    float v[8];
                    unpack<true>(raw_br[i], v);
                    const unsigned long long p0 = pack_f32x2(v[0], v[1]), p1 = pack_f32x2(v[2], v[3]);
                    const unsigned long long p2 = pack_f32x2(v[4], v[5]), p3 = pack_f32x2(v[6], v[7]);
                    squares = add_f32x2(squares, add_f32x2(fma_f32x2(p1, p1, mul_f32x2(p0, p0)), fma_f32x2(p3, p3, mul_f32x2(p2, p2))));
                }
                float lo, hi;
                unpack_f32x2(squares, lo, hi);
                branch_inverse = rms_inverse(lo + hi, p.pre_eps);
            }
#pragma unroll
            for (int i = 0; i < NCH; ++i) {
                const int chunk = lane_in_row + i * tpr;
                if (!FULL && chunk >= nchunks) { xr[i] = zero_packed<X_BF16>(); continue; }   // statistics see zeros there
                const uint32_t rw[4] = {raw_res[i].r.x, raw_res[i].r.y, raw_res[i].r.z, raw_res[i].r.w};
                uint32_t bw[4] = {raw_br[i].r.x, raw_br[i].r.y, raw_br[i].r.z, raw_br[i].r.w};
                if (p.pre_norm) {
#pragma unroll
                    for (int k = 0; k < 4; ++k)
                        bw[k] = pack_bf16x2(__fmul_rn(__uint_as_float(bw[k] << 16), branch_inverse),
                                            __fmul_rn(__uint_as_float(bw[k] & 0xffff0000u), branch_inverse));
                }
                uint4 gw = make_uint4(0, 0, 0, 0);
                if (has_pre_gate) gw = *reinterpret_cast<const uint4*>(s_gate + gate_base + ((i * tpr + lane_in_row) << 2));
                const uint32_t gws[4] = {gw.x, gw.y, gw.z, gw.w};
                uint32_t ow[4];
#pragma unroll
                for (int k = 0; k < 4; ++k) {
                    __nv_bfloat162 br2 = *reinterpret_cast<const __nv_bfloat162*>(&bw[k]);
                    if (has_pre_gate) br2 = __hmul2_rn(br2, *reinterpret_cast<const __nv_bfloat162*>(&gws[k]));
                    const __nv_bfloat162 sum = __hadd2_rn(*reinterpret_cast<const __nv_bfloat162*>(&rw[k]), br2);
                    ow[k] = *reinterpret_cast<const uint32_t*>(&sum);
                }
                xr[i].r = make_uint4(ow[0], ow[1], ow[2], ow[3]);
                if (valid) __stcs(reinterpret_cast<uint4*>(static_cast<uint16_t*>(p.state_out) + row_offset + chunk * 8), xr[i].r);
            }
            if constexpr (PF) load_raw(base + row_step, raw_res, raw_br);   // next row, in flight during this one
        } else if constexpr (PF) {
            load_row(base + row_step, xn);   // next row, in flight during this one
        } else {
            load_row(base, xr);
        }

        // ---- per-row operand offsets (32-bit arithmetic) ----
        unsigned srow = nrow, col0 = 0;
        if (p.sub32 > 1) { srow = nrow / p.sub32; col0 = (nrow - srow * p.sub32) * static_cast<unsigned>(width); }
        int64_t vec_offset = col0;
        int staged_base = 0;   // staged modulate: float offset of this row's vector pair in s_mod
        if constexpr (kStaged) {
            if (p.vectors > 1)
                staged_base = static_cast<int>((srow / static_cast<unsigned>(p.rows_per_vector)) % static_cast<unsigned>(p.vectors)) * 2 * pad;
        }
        if constexpr (POST == kPostModulate || POST == kPostScaleX || POST == kPostGatedResidual) {
            if (p.vectors > 1) {
                const unsigned vec = (srow / static_cast<unsigned>(p.rows_per_vector)) % static_cast<unsigned>(p.vectors);
                vec_offset += static_cast<int64_t>(vec) * p.width;
            }
        }
        int64_t f_offset = 0;
        const unsigned f_width = static_cast<unsigned>(p.f_width);
        float co[8], si[8];
        if constexpr (kRope) {
            unsigned frow = srow;
            if (p.rows_per_f_row != 1) frow = srow / static_cast<unsigned>(p.rows_per_f_row);
            if (frow >= static_cast<unsigned>(p.f_rows)) frow %= static_cast<unsigned>(p.f_rows);
            f_offset = static_cast<int64_t>(frow) * p.f_width;
            if constexpr (POST == kPostRopeShared) {
                // every chunk of this thread reads the same table columns: load them once, and
                // now, so that they arrive while the statistics are reduced
                if (valid) {
                    const unsigned fc = (static_cast<unsigned>(lane_in_row) * 8u) % f_width;
                    load8<false>(p.cosine, p.f_dt, f_offset + fc, co);
                    load8<false>(p.sine, p.f_dt, f_offset + fc, si);
                }
            }
        }

        // Gated residual with a bf16 residual: its row is requested now, so the loads are in
        // flight during the statistics instead of stalling the epilogue chunk by chunk.
        constexpr bool kEarlyResidual = POST == kPostGatedResidual && FULL && X_BF16 &&
                                        min_ctas_per_sm(NCH, X_BF16, FULL) == 2;   // only where 128 registers are available
        Packed<true> early_res[kEarlyResidual ? NCH : 1];
        const bool early = kEarlyResidual && p.res_dt == VRB_BF16;
        if constexpr (kEarlyResidual) {
            if (early && valid) {
#pragma unroll
                for (int i = 0; i < NCH; ++i) {
                    const int chunk = lane_in_row + i * tpr;
                    if (FULL || chunk < nchunks) early_res[i] = load_packed<true>(p.residual, row_offset + chunk * 8);
                }
            }
        }

        // ---- statistics: per-thread F32 partials (pairwise inside a chunk) ----
        // LayerNorm sums x - K and (x - K)^2 with K = the thread's first element, so the
        // partials stay small and accurate however large the row's common offset is; the exact
        // sums are rebuilt in double: S = s1 + n K, Q = s2 + 2 K s1 + n K^2.
        // Two elements per instruction: the partial sums are kept as (even, odd) pairs and folded once
        // at the end.
        float s1 = 0.0f, s2 = 0.0f, pivot = 0.0f;
        unsigned long long s1_pair = 0ull, s2_pair = 0ull;   // +0.0f in both halves
#pragma unroll
        for (int i = 0; i < NCH; ++i) {
            float v[8];
            unpack<X_BF16>(xr[i], v);
            if constexpr (NORM == kNormLayer) {
                if (i == 0) pivot = v[0];
                if (FULL || lane_in_row + i * tpr < nchunks) {
                    sub8_scalar(v, pivot);
                    const unsigned long long p0 = pack_f32x2(v[0], v[1]), p1 = pack_f32x2(v[2], v[3]);
                    const unsigned long long p2 = pack_f32x2(v[4], v[5]), p3 = pack_f32x2(v[6], v[7]);
                    s1_pair = add_f32x2(s1_pair, add_f32x2(add_f32x2(p0, p1), add_f32x2(p2, p3)));
                } else {
#pragma unroll
                    for (int e = 0; e < 8; ++e) v[e] = 0.0f;
                }
            }
            const unsigned long long p0 = pack_f32x2(v[0], v[1]), p1 = pack_f32x2(v[2], v[3]);
            const unsigned long long p2 = pack_f32x2(v[4], v[5]), p3 = pack_f32x2(v[6], v[7]);
            unsigned long long qa = mul_f32x2(p0, p0), qb = mul_f32x2(p2, p2);
            qa = fma_f32x2(p1, p1, qa);
            qb = fma_f32x2(p3, p3, qb);
            s2_pair = add_f32x2(s2_pair, add_f32x2(qa, qb));
        }
        {
            float lo, hi;
            unpack_f32x2(s1_pair, lo, hi); s1 = lo + hi;
            unpack_f32x2(s2_pair, lo, hi); s2 = lo + hi;
        }
        const int span = tpr < 32 ? tpr : 32;
        double acc0 = 0.0, acc1 = 0.0;
        if (f32_formula) {
            for (int offset = span >> 1; offset > 0; offset >>= 1)
                s2 = __fadd_rn(s2, __shfl_xor_sync(0xffffffffu, s2, offset));
        } else {
            if constexpr (NORM == kNormLayer) {
                const double k = static_cast<double>(pivot), n = static_cast<double>(own), d1 = static_cast<double>(s1);
                acc0 = d1 + n * k;
                acc1 = static_cast<double>(s2) + (2.0 * k) * d1 + (n * k) * k;
            } else {
                acc1 = static_cast<double>(s2);
            }
            for (int offset = span >> 1; offset > 0; offset >>= 1) {
                if constexpr (NORM == kNormLayer) acc0 += __shfl_xor_sync(0xffffffffu, acc0, offset);
                acc1 += __shfl_xor_sync(0xffffffffu, acc1, offset);
            }
        }
        if (warps_per_row > 1) {
            const int warp = threadIdx.x >> 5;
            if ((threadIdx.x & 31) == 0) {
                s_red[parity][warp][0] = acc0;
                s_red[parity][warp][1] = f32_formula ? static_cast<double>(s2) : acc1;
            }
            named_barrier(1 + row_in_cta, tpr);
            const int first = row_in_cta * warps_per_row;
            acc0 = 0.0; acc1 = 0.0; s2 = 0.0f;
            for (int w = 0; w < warps_per_row; ++w) {
                acc0 += s_red[parity][first + w][0];
                if (f32_formula) s2 = __fadd_rn(s2, static_cast<float>(s_red[parity][first + w][1]));
                else acc1 += s_red[parity][first + w][1];
            }
            parity ^= 1;
        }
        float mean = 0.0f, inv;
        if constexpr (NORM == kNormLayer) {
            // S/W and Q/W as products with 1/W: equal to the quotients to within one ulp of a double,
            // i.e. the same float except with probability 2^-29
            mean = static_cast<float>(acc0 * p.inv_width);
            inv = rsqrtf(static_cast<float>(acc1 * p.inv_width - static_cast<double>(mean) * mean) + p.eps);
        } else if (f32_formula) {
            const float m = __fmul_rn(s2, __fdiv_rn(1.0f, static_cast<float>(width)));
            inv = rsqrtf(__fadd_rn(m, p.eps));
        } else {
            inv = rsqrtf(static_cast<float>(acc1 * p.inv_width) + p.eps);
        }
        if (valid) {
        // ---- normalise, post-process, store ----
#pragma unroll
        for (int i = 0; i < NCH; ++i) {
            const int chunk = lane_in_row + i * tpr;
            if (!FULL && chunk >= nchunks) continue;
            const int c = chunk * 8;
            float y[8];
            unpack<X_BF16>(xr[i], y);
            if constexpr (NORM == kNormLayer) {
                sub8_scalar(y, mean);
                mul8_scalar(y, inv);
                if (has_w || has_b) {
                    // weight / bias are converted to x's dtype first (:4069-4070)
                    float w[8], b[8];
                    if (p.affine_staged) {
                        const float4* wa = reinterpret_cast<const float4*>(s_vec) + (i * 2 * tpr + lane_in_row);
                        const float4* ba = reinterpret_cast<const float4*>(s_vec + pad) + (i * 2 * tpr + lane_in_row);
                        const float4 w0 = wa[0], w1 = wa[tpr], b0 = ba[0], b1 = ba[tpr];
                        w[0] = w0.x; w[1] = w0.y; w[2] = w0.z; w[3] = w0.w; w[4] = w1.x; w[5] = w1.y; w[6] = w1.z; w[7] = w1.w;
                        b[0] = b0.x; b[1] = b0.y; b[2] = b0.z; b[3] = b0.w; b[4] = b1.x; b[5] = b1.y; b[6] = b1.z; b[7] = b1.w;
                    } else {
                        if (has_w) { load8<false>(weight_base, p.w_dt, c, w); round8<X_BF16>(w); }
                        if (has_b) { load8<false>(p.bias, p.b_dt, c, b); round8<X_BF16>(b); }
                    }
                    if (has_w && has_b && p.affine_fma) {
                        fma8(y, w, b);
                    } else {
                        if (has_w) mul8(y, w);
                        if (has_b) add8(y, b);
                    }
                }
            } else {
                mul8_scalar(y, inv);
                round8<X_BF16>(y);   // the normalised value is stored in the input dtype first (:900-902)
                if (has_w) {
                    // the weight is converted to the norm's output dtype (:4115)
                    float w[8];
                    load8<false>(weight_base, p.w_dt, c, w);
                    round8<N_BF16>(w);
                    mul8(y, w);
                }
            }
            round8<N_BF16>(y);       // what the unfused norm operator stores

            if constexpr (kModulate) {
                // common.cpp:51-61: 1+scale, product, +shift are three separately rounded F32 steps
                float t1[8], sh[8];
                if constexpr (kStaged) {
                    const float4* a = reinterpret_cast<const float4*>(s_mod + staged_base) + (i * 2 * tpr + lane_in_row);
                    const float4* b = reinterpret_cast<const float4*>(s_mod + staged_base + pad) + (i * 2 * tpr + lane_in_row);
                    const float4 a0 = a[0], a1 = a[tpr], b0 = b[0], b1 = b[tpr];
                    t1[0] = a0.x; t1[1] = a0.y; t1[2] = a0.z; t1[3] = a0.w; t1[4] = a1.x; t1[5] = a1.y; t1[6] = a1.z; t1[7] = a1.w;
                    sh[0] = b0.x; sh[1] = b0.y; sh[2] = b0.z; sh[3] = b0.w; sh[4] = b1.x; sh[5] = b1.y; sh[6] = b1.z; sh[7] = b1.w;
                } else {
                    load8<false>(p.scale, p.mod_dt, vec_offset + c, t1);
                    add8_scalar(t1, 1.0f);
                    if (has_shift) load8<false>(p.shift, p.mod_dt, vec_offset + c, sh);
                }
                mul8(y, t1);
                if (has_shift) add8(y, sh);
            } else if constexpr (POST == kPostScaleX) {
                float sc[8];
                load8<false>(p.scale, p.mod_dt, vec_offset + c, sc);
                add8_scalar(sc, 1.0f);
                round8<N_BF16>(sc);
                mul8(y, sc);
                round8<N_BF16>(y);
            } else if constexpr (kRope) {
                float r[8];
                if constexpr (POST == kPostRope) {
                    const unsigned fc = (col0 + static_cast<unsigned>(c)) % f_width;
                    load8<false>(p.cosine, p.f_dt, f_offset + fc, co);
                    load8<false>(p.sine, p.f_dt, f_offset + fc, si);
                }
                // pair (e, e+1): out = (y_e, y_e+1) * (cos_e, cos_e+1) + (-y_e+1, y_e) * (sin_e, sin_e+1), each
                // product and the sum rounded separately (rope_kernel uses __fmul_rn / __fadd_rn)
#pragma unroll
                for (int e = 0; e < 8; e += 2) {
                    const unsigned long long direct = mul_f32x2(pack_f32x2(y[e], y[e + 1]), pack_f32x2(co[e], co[e + 1]));
                    const unsigned long long turned = mul_f32x2(pack_f32x2(-y[e + 1], y[e]), pack_f32x2(si[e], si[e + 1]));
                    unpack_f32x2(add_f32x2(direct, turned), r[e], r[e + 1]);
                }
#pragma unroll
                for (int e = 0; e < 8; ++e) y[e] = r[e];
            } else if constexpr (POST == kPostGatedResidual) {
                float res[8], g[8];
                if (early) unpack<true>(early_res[i], res);
                else load8<true>(p.residual, p.res_dt, row_offset + c, res);
                const bool has_gate = p.gate != nullptr;
                const int sd = p.state_dt;
                round8_rt(sd, res);
                round8_rt(sd, y);
                if (has_gate) {
                    load8<false>(p.gate, p.gate_dt, vec_offset + c, g);
                    round8_rt(sd, g);
                    mul8(y, g);
                    round8_rt(sd, y);
                }
                add8(y, res);
            }
            store8(out_base, p.out_dt, row_offset + c, y);
        }
        }  // valid
        if constexpr (PF && !PRE) {
#pragma unroll
            for (int i = 0; i < NCH; ++i) xr[i] = xn[i];
        }
    }
}

#endif  // __CUDACC__

// Row geometries with their own instantiation: the generic ones (threads per row read at run
// time, every chunk guarded) for 1..8 chunks per thread, and the exact ones for the
// production widths.
enum Geometry {
    kGenericFirst = 0,   // + index into {1,2,3,4,5,6,8} chunks per thread
    kExact1536 = 7,      // 6 chunks x 32 threads   (Wan2.1-1.3B, Mochi text stream)
    kExact3072 = 8,      // 6 chunks x 64 threads   (Mochi visual stream)
    kExact5120 = 9,      // 5 chunks x 128 threads  (Wan2.2-A14B)
    kExact2048 = 10,     // 4 chunks x 64 threads   (LTX)
    kExact128 = 11,      // 2 chunks x 8 threads    (per-head q/k norm)
    kExact64 = 12,       // 1 chunk x 8 threads     (per-head q/k norm over 64: CogVideoX)
};

// Launches the row_kernel instantiation for `geometry`; one definition per (NORM, POST, DT)
// lives in its own translation unit so the family compiles in parallel.
template <int NORM, int POST, int DT>
void launch_row_variant(const RowParams& p, int geometry, int64_t ctas, size_t smem, cudaStream_t stream);

}  // namespace rowwise
}  // namespace vrb
