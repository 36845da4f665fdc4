// pixel_norm over the channel axis of x [outer, channels, inner] (CudaBackend::pixel_norm,
// native/src/backend/cuda/cuda_backend.cu:5048-5086), optionally followed by modulate with one
// (1 + scale, shift) pair per (outer, channel) and SiLU -- the head of LTX's decoder_residual
// (native/src/architectures/ltx.cpp:221-227: pixel_norm -> modulate -> silu), which the reference runs
// as 7 kernels with F32 intermediates of the full tensor.
//
// Arithmetic follows the reference's kernels operation by operation:
//   inner > 1  (pixel_norm_strided_axis_kernel :2131-2165): per position 8 channel lanes, lane a sums
//              channels a, a+8, ... with one FFMA each (`square += value * value` after contraction),
//              lanes combined by the tree with strides 4, 2, 1;
//   inner == 1 (pixel_norm_contiguous_axis_kernel :2097-2126): 256 thread partials + the tree of
//              group_norm_block_sum (:1884-1893);
//   denominator = sqrtf(total / channels + eps);  y = x / denominator rounded to x's dtype;
//   modulate (common.cpp:51-61): F32(y) * (1 + F32(scale)) + F32(shift), each operation rounded;
//   SiLU on that F32 value (activation_kernel :1098-1109).
//
// Tile kernel: a CTA stages [channels x P positions] of the input in shared memory with 16-byte
// asynchronous copies (the whole tile is in flight at once and costs no registers), reduces it from
// there, and writes the finished elements: the tensor is read from HBM once, where statistics pass +
// normalise pass of the reference read it twice.  Two tile buffers: the next tile's copies are in
// flight while the current tile is reduced and written.  P is chosen so that three CTAs fit on an SM.
#include "vrb_common.cuh"
#include "vrb_tma.cuh"

#include <mutex>
#include <vector>

namespace vrb {
namespace {

constexpr int kThreads = 256;
constexpr int kLanes = 8;

struct PixelNormParams {
    const void* x;
    void* out;
    const void* scale;   // [outer, channels] or nullptr
    const void* shift;   // [outer, channels] or nullptr (with scale: added; alone: not accepted)
    int x_dt, out_dt, mod_dt;
    int64_t outer, channels, inner;
    float eps;
    int silu;
    int l2;              // l2_normalize: denominator = sqrtf(sum) + eps instead of sqrtf(sum / channels + eps)
};

// The denominator of one position from the sum of its channels' squares: pixel_norm (:2121, :2160) or
// l2_normalize (l2_normalize_kernel :1170).
__device__ __forceinline__ float denominator_of(const PixelNormParams& p, float total, float channel_count) {
    if (p.l2) return __fadd_rn(__fsqrt_rn(total), p.eps);
    return __fsqrt_rn(__fadd_rn(__fdiv_rn(total, channel_count), p.eps));
}

// One normalised element to the stored result; `one_plus_scale` / `shift` are ignored without modulation.
__device__ __forceinline__ float finish(const PixelNormParams& p, float x, float denominator, bool modulated,
                                        float one_plus_scale, float shift) {
    float v = round_to(p.x_dt, __fdiv_rn(x, denominator));
    if (modulated) v = __fadd_rn(__fmul_rn(v, one_plus_scale), shift);
    if (p.silu) v = activation_value(VRB_SILU, v);
    return v;
}

__device__ __forceinline__ float tree8(const float (&s)[kLanes]) {
    // strides 4, 2, 1 of the reference's shared-memory reduction
    const float a0 = __fadd_rn(s[0], s[4]), a1 = __fadd_rn(s[1], s[5]), a2 = __fadd_rn(s[2], s[6]), a3 = __fadd_rn(s[3], s[7]);
    return __fadd_rn(__fadd_rn(a0, a2), __fadd_rn(a1, a3));
}

__device__ __forceinline__ void async_copy16(void* shared_dst, const void* global_src) {
    const unsigned dst = static_cast<unsigned>(__cvta_generic_to_shared(shared_dst));
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(global_src) : "memory");
}
__device__ __forceinline__ void async_copy_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
// waits until at most `pending` of this thread's committed groups are still in flight
template <int pending>
__device__ __forceinline__ void async_copy_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(pending) : "memory"); }

// Epilogue variants of the tile kernel, fixed at compile time.
enum Mode { kNormOnly = 0, kModulate = 1, kModulateSilu = 2 };

// x / d for a bf16-representable x without a division per element.  With r = RN(1 / d):
//   q = RN(x * r);  e = x - d * q (one FMA, exact);  q' = RN(q + e * r)
// equals RN(x / d) for EVERY pair (bf16 significand of x, F32 significand of d) -- all 2^7 x 2^23
// pairs are enumerated by tests/test_reciprocal_division.py -- and scaling x or d by a power of two
// changes nothing as long as x, d, r, q and e stay normal.  reciprocal_or_zero() therefore hands out r
// only for d in [2^-30, 2^30] and 0 otherwise (also for an infinite or NaN d), and a result below
// 2^-28 in magnitude, or NaN, -- a zero (its sign), a tiny x, or r == 0 -- is redone with the division.
constexpr float kReciprocalLow = 9.313225746154785e-10f, kReciprocalHigh = 1073741824.0f;   // 2^-30, 2^30
constexpr float kQuotientFloor = 3.725290298461914e-09f;                                     // 2^-28
__device__ __forceinline__ float reciprocal_or_zero(float d) {
    return d >= kReciprocalLow && d <= kReciprocalHigh ? __frcp_rn(d) : 0.0f;
}

// SiLU of an F32 value whose result is STORED AS bf16.  v / (1 + expf(-v)) costs two range-reduced special
// functions and an IEEE division per element.  The approximate form (ex2.approx, rcp.approx and three F32
// operations) is within a few F32 ulp of it for |v| <= 8, so both round to the same bf16 unless the
// approximation's low 16 bits lie within kSiluGuardUlps of the rounding boundary 0x8000; those elements (1 in
// 3000), larger arguments and NaN are redone with the exact expression.  The F32 value differs from the exact one,
// its bf16 rounding does not: tests/test_gpu_pixel_norm.py drives all 2^32 arguments through the kernel against
// the exact expression.  (The flush-to-zero forms are exact here: 1 + t is in [1, 2^24] and a denormal argument
// gives t = 1 either way.)
constexpr int kSiluGuardUlps = 10;
// whether the low 16 bits of an F32 value lie within kSiluGuardUlps of 0x8000, where its bf16 rounding turns
__device__ __forceinline__ bool near_bf16_boundary(float value) {
    return ((__float_as_uint(value) - (0x8000u - kSiluGuardUlps)) & 0xffffu) <= 2u * kSiluGuardUlps;
}
__device__ __forceinline__ float silu_approximate(float v, bool& redo) {
    float t, inverse;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(t) : "f"(__fmul_rn(v, -1.4426950408889634f)));
    asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(inverse) : "f"(__fadd_rn(1.0f, t)));
    const float fast = __fmul_rn(v, inverse);
    redo = redo || !(fabsf(v) <= 8.0f) || near_bf16_boundary(fast);
    return fast;
}

// The same for two values at once, the multiplications and the addition as packed F32 operations (they round like
// the scalar ones).  Returns whether either result has to be redone (silu_redo() says which).
__device__ __forceinline__ bool silu_approximate_pair(float v0, float v1, float& s0, float& s1) {
    const unsigned long long v2 = pack_f32x2(v0, v1);
    float t0, t1, i0, i1;
    unpack_f32x2(mul_f32x2(v2, pack_f32x2(-1.4426950408889634f, -1.4426950408889634f)), t0, t1);
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(t0) : "f"(t0));
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(t1) : "f"(t1));
    unpack_f32x2(add_f32x2(pack_f32x2(t0, t1), pack_f32x2(1.0f, 1.0f)), t0, t1);
    asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(i0) : "f"(t0));
    asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(i1) : "f"(t1));
    unpack_f32x2(mul_f32x2(v2, pack_f32x2(i0, i1)), s0, s1);
    return !(fabsf(v0) <= 8.0f) || !(fabsf(v1) <= 8.0f) || near_bf16_boundary(s0) || near_bf16_boundary(s1);
}
// Whether an approximate result has to be redone, judged from the result alone (the argument is no longer at hand):
// an argument outside [-8, 8] or NaN shows as a result above 7.9, in (-0.01, 0], or NaN.  A superset of
// silu_approximate's own conditions; where it flags a valid result the exact expression gives the same bits.
__device__ __forceinline__ bool silu_redo(float approximate) {
    return !(approximate <= 7.9f) || !(approximate <= -0.01f || approximate > 0.0f) || near_bf16_boundary(approximate);
}

// One normalised element to the stored value, everything known at compile time.  EXACT: the reference's operations
// one by one.  Otherwise the short forms above where the template arguments allow them, with `redo` set when the
// element has to be evaluated again with EXACT (the caller does that once per 16-byte chunk, so the common path has
// one branch per chunk).
// The steps after the quotient: rounding to x's dtype, modulate, SiLU.
template <bool X_BF16, int MODE, bool OUT_BF16, bool EXACT>
__device__ __forceinline__ float finish_quotient(float v, float one_plus_scale, float shift, bool& redo) {
    if constexpr (X_BF16 && MODE != kNormOnly) v = round_to_bf16(v);   // kNormOnly: the bf16 store rounds
    if constexpr (MODE != kNormOnly) v = __fadd_rn(__fmul_rn(v, one_plus_scale), shift);
    if constexpr (MODE == kModulateSilu) {
        if constexpr (OUT_BF16 && !EXACT) v = silu_approximate(v, redo);
        else v = activation_value(VRB_SILU, v);
    }
    return v;
}
template <bool X_BF16, int MODE, bool OUT_BF16, bool EXACT>
__device__ __forceinline__ float finish_tile(float x, float denominator, float reciprocal, float one_plus_scale, float shift,
                                             bool& redo) {
    float v;
    if constexpr (X_BF16 && !EXACT) {
        const float q = __fmul_rn(x, reciprocal);
        v = __fmaf_rn(__fmaf_rn(-denominator, q, x), reciprocal, q);
        redo = redo || !(fabsf(v) >= kQuotientFloor);
    } else {
        v = __fdiv_rn(x, denominator);
    }
    return finish_quotient<X_BF16, MODE, OUT_BF16, EXACT>(v, one_plus_scale, shift, redo);
}
// whether the short forms exist for a variant (else the first evaluation is already the exact one)
template <bool X_BF16, int MODE, bool OUT_BF16>
constexpr bool kHasShortForm = X_BF16 || (MODE == kModulateSilu && OUT_BF16);

// set by a tile kernel whose bounded wait for a tensor-map copy ran out (vrb_async_wait_failures() reads it)
__device__ int g_async_wait_gave_up = 0;

// Tile kernel: inner % EPC == 0, 16-byte aligned tensors, fewer than 2^31 tiles and chunks per channel row; `cols` (a
// power of two, at most 8) 16-byte chunks per channel.  kNormOnly stores x's dtype; the modulated forms store F32 or
// (OUT_BF16) bf16.  The block size is a multiple of cols, so a thread's chunks all lie in one chunk column k and
// its channel advances by kThreads / cols per step: addresses are advanced, not recomputed.
// TMA: the tile is loaded by tensor-map copies (one per slab of `slab` channels, issued by thread 0, completion counted
// on an mbarrier per buffer) instead of one cp.async per chunk and thread; needs tile and slab sizes that are multiples
// of 128 bytes.  The shared-memory layout of the tile is the same either way.
template <bool X_BF16, int MODE, bool OUT_BF16, bool TMA>
__global__ void __launch_bounds__(kThreads) pixel_norm_tile_kernel(const PixelNormParams p, int cols, int cols_log2,
                                                                   const __grid_constant__ CUtensorMap map, int slab) {
    constexpr int EPC = X_BF16 ? 8 : 4;   // elements per 16-byte chunk
    constexpr int OUT_CHUNK = (MODE == kNormOnly ? X_BF16 : OUT_BF16) ? EPC * 2 : EPC * 4;   // bytes written per chunk
    extern __shared__ __align__(128) uint4 tiles_buffer[];   // two tiles of [channels][cols], then the reduction scratch
    const int channels = static_cast<int>(p.channels);
    const int positions = cols * EPC;
    const int tile_chunks = channels * cols;
    float* const partial = reinterpret_cast<float*>(tiles_buffer + 2 * static_cast<size_t>(tile_chunks));   // [kLanes][positions]
    float* const denominator = partial + kLanes * positions;                                              // [positions]
    float* const reciprocal = denominator + positions;                                                    // [positions], bf16 input only
    uint64_t* const barriers = reinterpret_cast<uint64_t*>(reciprocal + positions);                       // [2], TMA only
    float2* const modulation = reinterpret_cast<float2*>(barriers + 2);                                   // [channels] (1 + scale, shift)
    const uint32_t inner_chunks = static_cast<uint32_t>(p.inner / EPC);
    const uint32_t tiles_per_outer = (inner_chunks + cols - 1) >> cols_log2;
    const uint32_t tiles = static_cast<uint32_t>(p.outer) * tiles_per_outer;
    const float channel_count = static_cast<float>(p.channels);
    const int k = threadIdx.x & (cols - 1), c0 = threadIdx.x >> cols_log2, c_step = kThreads >> cols_log2;
    const int64_t row_step = static_cast<int64_t>(c_step) * inner_chunks;   // chunks between a thread's consecutive channels
    if constexpr (TMA) {
        if (threadIdx.x == 0) {
            mbarrier_init(&barriers[0], 1);
            mbarrier_init(&barriers[1], 1);
            mbarrier_init_fence();
        }
        __syncthreads();
    }
    unsigned phases = 0;   // bit b: parity of the phase buffer b's barrier completes next

    // asynchronous copy of tile t into buffer b (cp.async: one committed group per tile and thread)
    auto request = [&](uint32_t t, int b) {
        if constexpr (TMA) {
            if (t < tiles && threadIdx.x == 0) {
                const uint32_t o = t / tiles_per_outer;
                const uint32_t chunk0 = (t - o * tiles_per_outer) << cols_log2;
                uint4* const dst = tiles_buffer + static_cast<size_t>(b) * tile_chunks;
                async_proxy_fence();   // the buffer was read through the generic proxy until the barrier before this call
                mbarrier_expect_bytes(&barriers[b], static_cast<unsigned>(tile_chunks) * 16u);
                // columns beyond the row's end are filled with zeros by the copy (and count as transferred bytes)
                for (int c = 0; c < channels; c += slab)
                    tma_load_3d(dst + static_cast<size_t>(c) * cols, &map, static_cast<int>(chunk0 * EPC), c, static_cast<int>(o), &barriers[b]);
            }
            return;
        }
        if (t < tiles) {
            const uint32_t o = t / tiles_per_outer;
            const uint32_t chunk0 = (t - o * tiles_per_outer) << cols_log2;
            const bool inside = chunk0 + k < inner_chunks;
            const uint4* src = static_cast<const uint4*>(p.x) + (static_cast<int64_t>(o) * channels + c0) * inner_chunks + chunk0 + k;
            uint4* dst = tiles_buffer + static_cast<size_t>(b) * tile_chunks + threadIdx.x;
            if (inside) {
                for (int idx = threadIdx.x; idx < tile_chunks; idx += kThreads, src += row_step, dst += kThreads) async_copy16(dst, src);
            } else {
                for (int idx = threadIdx.x; idx < tile_chunks; idx += kThreads, dst += kThreads) *dst = make_uint4(0, 0, 0, 0);
            }
        }
        async_copy_commit();
    };

    int buffer = 0;
    uint32_t modulation_of = 0xffffffffu;   // the batch entry whose vectors the table holds
    request(blockIdx.x, 0);
    for (uint32_t t = blockIdx.x; t < tiles; t += gridDim.x, buffer ^= 1) {
        const uint32_t o = t / tiles_per_outer;
        const uint32_t chunk0 = (t - o * tiles_per_outer) << cols_log2;
        const uint4* const tile = tiles_buffer + static_cast<size_t>(buffer) * tile_chunks;
        request(t + gridDim.x, buffer ^ 1);   // the next tile arrives while this one is reduced and written
        if constexpr (TMA) {
            const bool arrived = mbarrier_wait_bounded(&barriers[buffer], (phases >> buffer) & 1u, &g_async_wait_gave_up);
            phases ^= 1u << buffer;
            if (!__syncthreads_and(arrived)) {
                // a wait ran out somewhere in the CTA: every thread leaves, after one more bounded wait for the copy
                // that may still be in flight into the other buffer
                if (t + gridDim.x < tiles) mbarrier_wait_bounded(&barriers[buffer ^ 1], (phases >> (buffer ^ 1)) & 1u, &g_async_wait_gave_up);
                break;
            }
        } else {
            async_copy_wait<1>();
            __syncthreads();
        }
        // (lane, position) partial sums in the reference's order; a thread takes the positions of one
        // 32-bit shared-memory word (two bf16 positions, one F32 position); words is a power of two
        constexpr int PPW = X_BF16 ? 2 : 1;
        const int words_log2 = cols_log2 + 2, words = 1 << words_log2;
        const uint32_t* const tile_words = reinterpret_cast<const uint32_t*>(tile);
        for (int item = threadIdx.x; item < words * kLanes; item += kThreads) {
            const int lane = item >> words_log2, word = item & (words - 1);
            float q0 = 0.0f, q1 = 0.0f;
            const uint32_t* e = tile_words + lane * words + word;
            const int step = kLanes * words;
            int c = lane;
#pragma unroll 4
            for (; c < channels; c += kLanes, e += step) {
                const uint32_t w = *e;
                if constexpr (X_BF16) {
                    const float lo = __uint_as_float(w << 16), hi = __uint_as_float(w & 0xffff0000u);
                    q0 = __fmaf_rn(lo, lo, q0);
                    q1 = __fmaf_rn(hi, hi, q1);
                } else {
                    const float v = __uint_as_float(w);
                    q0 = __fmaf_rn(v, v, q0);
                }
            }
            if constexpr (X_BF16) *reinterpret_cast<float2*>(partial + lane * positions + word * 2) = make_float2(q0, q1);
            else partial[lane * positions + word] = q0;
        }
        __syncthreads();
        if (threadIdx.x < positions) {
            float s[kLanes];
#pragma unroll
            for (int a = 0; a < kLanes; ++a) s[a] = partial[a * positions + threadIdx.x];
            const float d = denominator_of(p, tree8(s), channel_count);
            denominator[threadIdx.x] = d;
            if constexpr (X_BF16) reciprocal[threadIdx.x] = reciprocal_or_zero(d);
        }
        if constexpr (MODE != kNormOnly) {
            // this batch entry's (1 + scale, shift) per channel, once per tile instead of once per chunk
            if (o != modulation_of) {
                for (int c = threadIdx.x; c < channels; c += kThreads) {
                    const int64_t vector = static_cast<int64_t>(o) * channels + c;
                    modulation[c] = make_float2(__fadd_rn(1.0f, load1(p.scale, p.mod_dt, vector)), load1(p.shift, p.mod_dt, vector));
                }
                modulation_of = o;
            }
        }
        __syncthreads();
        if (chunk0 + k < inner_chunks) {
            // this thread's positions: denominators and reciprocals once per tile
            float d[EPC], r[EPC];
            {
                const float4* d4 = reinterpret_cast<const float4*>(denominator + k * EPC);
                const float4* r4 = reinterpret_cast<const float4*>(reciprocal + k * EPC);
                const float4 da = d4[0];
                d[0] = da.x; d[1] = da.y; d[2] = da.z; d[3] = da.w;
                if constexpr (X_BF16) {
                    const float4 db = d4[1], ra = r4[0], rb = r4[1];
                    d[4] = db.x; d[5] = db.y; d[6] = db.z; d[7] = db.w;
                    r[0] = ra.x; r[1] = ra.y; r[2] = ra.z; r[3] = ra.w; r[4] = rb.x; r[5] = rb.y; r[6] = rb.z; r[7] = rb.w;
                } else {
#pragma unroll
                    for (int j = 0; j < EPC; ++j) r[j] = 0.0f;
                }
            }
            const int64_t first = (static_cast<int64_t>(o) * channels + c0) * inner_chunks + chunk0 + k;   // in chunks
            char* out = static_cast<char*>(p.out) + first * OUT_CHUNK;
            const int64_t out_step = row_step * OUT_CHUNK;
            float minus_d[EPC];
#pragma unroll
            for (int j = 0; j < EPC; ++j) minus_d[j] = -d[j];
            const float2* vectors = modulation + c0;
            const uint4* chunk = tile + threadIdx.x;
            for (int idx = threadIdx.x; idx < tile_chunks; idx += kThreads, chunk += kThreads, out += out_step, vectors += c_step) {
                float ops = 1.0f, sh = 0.0f;
                if constexpr (MODE != kNormOnly) {
                    const float2 pair = *vectors;
                    ops = pair.x;
                    sh = pair.y;
                }
                const uint4 raw = *chunk;
                float in[EPC], v[EPC];
                if constexpr (X_BF16) {
                    const uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
                    for (int j = 0; j < 4; ++j) {
                        in[2 * j] = __uint_as_float(w[j] << 16);
                        in[2 * j + 1] = __uint_as_float(w[j] & 0xffff0000u);
                    }
                } else {
                    in[0] = __uint_as_float(raw.x); in[1] = __uint_as_float(raw.y); in[2] = __uint_as_float(raw.z); in[3] = __uint_as_float(raw.w);
                }
                if constexpr (X_BF16) {
                    // The short forms, two elements at a time (packed F32 operations round like the scalar ones).  `any`
                    // collects, for the whole chunk, whether some element must be evaluated again with the exact forms;
                    // which ones is found out afterwards, from values still in registers, only in the chunks that need it.
                    bool any = false;
                    const unsigned long long ops2 = pack_f32x2(ops, ops);
#pragma unroll
                    for (int j = 0; j < EPC; j += 2) {
                        const unsigned long long x2 = pack_f32x2(in[j], in[j + 1]), r2 = pack_f32x2(r[j], r[j + 1]);
                        const unsigned long long q2 = mul_f32x2(x2, r2);
                        const unsigned long long c2 = fma_f32x2(fma_f32x2(pack_f32x2(minus_d[j], minus_d[j + 1]), q2, x2), r2, q2);
                        float c0, c1;
                        unpack_f32x2(c2, c0, c1);
                        any = any || !(fabsf(c0) >= kQuotientFloor) || !(fabsf(c1) >= kQuotientFloor);
                        if constexpr (MODE != kNormOnly) {
                            // rounding to bf16 as a pair (one conversion); modulate: a multiplication and an addition,
                            // each rounded
                            const __nv_bfloat162 y2 = __floats2bfloat162_rn(c0, c1);
                            const uint32_t yw = *reinterpret_cast<const uint32_t*>(&y2);
                            // (the product packed, the sums scalar: with the addition packed as well, 28 % of the results were
                            // one ulp off -- the rate of a fused multiply-add -- although both instructions carry .rn)
                            unpack_f32x2(mul_f32x2(pack_f32x2(__uint_as_float(yw << 16), __uint_as_float(yw & 0xffff0000u)), ops2), c0, c1);
                            c0 = __fadd_rn(c0, sh);
                            c1 = __fadd_rn(c1, sh);
                            if constexpr (MODE == kModulateSilu) {
                                if constexpr (OUT_BF16) {
                                    float s0, s1;
                                    any = silu_approximate_pair(c0, c1, s0, s1) || any;
                                    c0 = s0;
                                    c1 = s1;
                                } else {
                                    c0 = activation_value(VRB_SILU, c0);
                                    c1 = activation_value(VRB_SILU, c1);
                                }
                            }
                        }
                        v[j] = c0;
                        v[j + 1] = c1;
                    }
                    if (any) {
                        // rare (one chunk in a few hundred).  An element is evaluated again with the reference's operations
                        // one by one if its reciprocal was withheld, its quotient may lie below the floor (|x| < 2^-27 d is a
                        // superset of |x / d| < 2^-28), or -- approximate SiLU -- its result says the argument may have been
                        // outside [-8, 8] (SiLU > 7.9, or in (-0.01, 0]) or lies near the rounding boundary; a few elements
                        // too many are harmless, the exact form gives the same bits where both are valid.
                        bool unused = false;
#pragma unroll
                        for (int j = 0; j < EPC; ++j) {
                            bool again = r[j] == 0.0f || !(fabsf(in[j]) >= __fmul_rn(d[j], 2.0f * kQuotientFloor));
                            if constexpr (MODE == kModulateSilu && OUT_BF16)
                                again = again || silu_redo(v[j]);
                            if (again) v[j] = finish_tile<X_BF16, MODE, OUT_BF16, true>(in[j], d[j], r[j], ops, sh, unused);
                        }
                    }
                } else {
                    unsigned redo = 0;   // bit j: element j has to be evaluated with the exact forms
#pragma unroll
                    for (int j = 0; j < EPC; ++j) {
                        bool again = false;
                        v[j] = finish_tile<X_BF16, MODE, OUT_BF16, false>(in[j], d[j], r[j], ops, sh, again);
                        redo |= (again ? 1u : 0u) << j;
                    }
                    if constexpr (kHasShortForm<X_BF16, MODE, OUT_BF16>) {
                        if (redo != 0) {   // rare: only the flagged elements, with the reference's operations one by one
                            bool unused = false;
#pragma unroll
                            for (int j = 0; j < EPC; ++j)
                                if ((redo >> j) & 1u) v[j] = finish_tile<X_BF16, MODE, OUT_BF16, true>(in[j], d[j], r[j], ops, sh, unused);
                        }
                    }
                }
                if constexpr (X_BF16) {
                    if constexpr (MODE == kNormOnly || OUT_BF16) {
                        __stcs(reinterpret_cast<uint4*>(out), make_uint4(pack_bf16x2(v[0], v[1]), pack_bf16x2(v[2], v[3]),
                                                                         pack_bf16x2(v[4], v[5]), pack_bf16x2(v[6], v[7])));
                    } else {
                        store32(out, make_uint4(__float_as_uint(v[0]), __float_as_uint(v[1]), __float_as_uint(v[2]), __float_as_uint(v[3])),
                                make_uint4(__float_as_uint(v[4]), __float_as_uint(v[5]), __float_as_uint(v[6]), __float_as_uint(v[7])));
                    }
                } else {
                    if constexpr (MODE != kNormOnly && OUT_BF16) {
                        __stcs(reinterpret_cast<uint2*>(out), make_uint2(pack_bf16x2(v[0], v[1]), pack_bf16x2(v[2], v[3])));
                    } else {
                        __stcs(reinterpret_cast<float4*>(out), make_float4(v[0], v[1], v[2], v[3]));
                    }
                }
            }
        }
        __syncthreads();   // this buffer is the target of the next iteration's copies
    }
    async_copy_wait<0>();
}

// Any inner extent / alignment / channel count, inner > 1: one thread per position, two passes over
// global memory with the same lane schedule.
__global__ void __launch_bounds__(kThreads) pixel_norm_strided_kernel(const PixelNormParams p) {
    const int64_t units = p.outer * p.inner;
    const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
    const bool modulated = p.scale != nullptr;
    for (int64_t u = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; u < units; u += stride) {
        const int64_t o = u / p.inner, i = u - o * p.inner;
        const int64_t base = o * p.channels * p.inner + i;
        float s[kLanes];
#pragma unroll
        for (int a = 0; a < kLanes; ++a) s[a] = 0.0f;
        for (int64_t c0 = 0; c0 < p.channels; c0 += kLanes) {
#pragma unroll
            for (int a = 0; a < kLanes; ++a) {
                if (c0 + a < p.channels) {
                    const float v = load1(p.x, p.x_dt, base + (c0 + a) * p.inner);
                    s[a] = __fmaf_rn(v, v, s[a]);
                }
            }
        }
        const float denominator = denominator_of(p, tree8(s), static_cast<float>(p.channels));
        for (int64_t c = 0; c < p.channels; ++c) {
            float ops = 1.0f, sh = 0.0f;
            if (modulated) {
                ops = __fadd_rn(1.0f, load1(p.scale, p.mod_dt, o * p.channels + c));
                sh = load1(p.shift, p.mod_dt, o * p.channels + c);
            }
            store1(p.out, p.out_dt, base + c * p.inner,
                   finish(p, load1(p.x, p.x_dt, base + c * p.inner), denominator, modulated, ops, sh));
        }
    }
}

// inner == 1: one CTA per row, the contiguous-axis kernel's summation schedule.
__global__ void __launch_bounds__(kThreads) pixel_norm_rows_kernel(const PixelNormParams p) {
    __shared__ float workspace[kThreads];
    const bool modulated = p.scale != nullptr;
    for (int64_t row = blockIdx.x; row < p.outer; row += gridDim.x) {
        const int64_t base = row * p.channels;
        float q = 0.0f;
        for (int64_t c = threadIdx.x; c < p.channels; c += kThreads) {
            const float v = load1(p.x, p.x_dt, base + c);
            q = __fmaf_rn(v, v, q);
        }
        workspace[threadIdx.x] = q;
        __syncthreads();
        for (int stride = kThreads / 2; stride > 0; stride /= 2) {
            if (threadIdx.x < stride) workspace[threadIdx.x] = __fadd_rn(workspace[threadIdx.x], workspace[threadIdx.x + stride]);
            __syncthreads();
        }
        const float denominator = denominator_of(p, workspace[0], static_cast<float>(p.channels));
        __syncthreads();   // workspace is rewritten by the next row
        for (int64_t c = threadIdx.x; c < p.channels; c += kThreads) {
            float ops = 1.0f, sh = 0.0f;
            if (modulated) {
                ops = __fadd_rn(1.0f, load1(p.scale, p.mod_dt, base + c));
                sh = load1(p.shift, p.mod_dt, base + c);
            }
            store1(p.out, p.out_dt, base + c, finish(p, load1(p.x, p.x_dt, base + c), denominator, modulated, ops, sh));
        }
    }
}

// Resident CTAs per SM of a tile kernel for a dynamic shared-memory size; remembered per (kernel,
// device, size), guarded for concurrent callers.  The kernel is opted into the largest tile the
// launcher ever asks for the first time it is seen on a device (the attribute is a limit that a
// later, smaller request must not lower).
constexpr size_t kMaxTileBytes = 208 * 1024;
template <typename K>
int tile_ctas_per_sm(K kernel, size_t smem) {
    struct Entry { const void* kernel; int device; size_t smem; int per_sm; };
    static std::mutex mutex;
    static std::vector<Entry> known;
    int device = 0;
    if (cudaGetDevice(&device) != cudaSuccess) return 0;
    const void* const key = reinterpret_cast<const void*>(kernel);
    std::lock_guard<std::mutex> lock(mutex);
    bool opted = false;
    for (const Entry& e : known) {
        if (e.kernel != key || e.device != device) continue;
        if (e.smem == smem) return e.per_sm;
        opted = true;
    }
    int n = 0;
    if ((!opted && cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                        static_cast<int>(kMaxTileBytes)) != cudaSuccess) ||
        cudaOccupancyMaxActiveBlocksPerMultiprocessor(&n, kernel, kThreads, smem) != cudaSuccess) {
        cudaGetLastError();
        n = 0;
    }
    if (known.size() < 1024) known.push_back({key, device, smem, n});
    return n;
}

// ---- RMSNorm over the channel axis with the same tile scheme ------------------------------------
// CudaBackend::rms_norm over an inner axis (rms_norm_axis_parallel_kernel,
// native/src/backend/cuda/cuda_backend.cu:1045-1095; the Wan VAE's rms_channel, components/executor.cpp:90-93):
// per position 8 reduction lanes, lane a takes channels a, a+8, ... in double, lanes combined in
// lane order; inverse = rsqrtf(float(total / channels) + eps); y = x * inverse rounded to x's
// dtype, times the weight (converted to x's dtype), rounded; optionally SiLU of that value.
struct RmsAxisParams {
    const void* x;
    void* out;
    const void* weight;   // [channels] or nullptr
    int w_dt;
    int64_t outer, channels, inner;
    float eps;
};

template <bool X_BF16, bool SILU, bool TMA>
__global__ void __launch_bounds__(kThreads) rms_axis_tile_kernel(const RmsAxisParams p, int cols, int cols_log2,
                                                                 const __grid_constant__ CUtensorMap map, int slab) {
    constexpr int EPC = X_BF16 ? 8 : 4;
    constexpr int X_DT = X_BF16 ? VRB_BF16 : VRB_F32;
    extern __shared__ __align__(128) uint4 tiles_buffer[];   // two tiles of [channels][cols], then the reduction scratch
    const int channels = static_cast<int>(p.channels);
    const int positions = cols * EPC;
    const int tile_chunks = channels * cols;
    double* const partial = reinterpret_cast<double*>(tiles_buffer + 2 * static_cast<size_t>(tile_chunks));   // [kLanes][positions]
    float* const inverse = reinterpret_cast<float*>(partial + kLanes * positions);                          // [positions]
    // two mbarriers (TMA only) behind the scratch, 8-byte aligned: positions is a multiple of 4
    uint64_t* const barriers = reinterpret_cast<uint64_t*>(inverse + positions);
    // the weight per channel, rounded to x's dtype (a bf16 weight twice in one word, for the packed product)
    uint32_t* const weights = reinterpret_cast<uint32_t*>(barriers + 2);
    if (p.weight != nullptr) {
        for (int c = threadIdx.x; c < channels; c += kThreads) {
            const float w = round_to(X_DT, load1(p.weight, p.w_dt, c));
            weights[c] = X_BF16 ? (__float_as_uint(w) >> 16) * 0x10001u : __float_as_uint(w);
        }
    }
    __syncthreads();
    if constexpr (TMA) {
        if (threadIdx.x == 0) {
            mbarrier_init(&barriers[0], 1);
            mbarrier_init(&barriers[1], 1);
            mbarrier_init_fence();
        }
        __syncthreads();
    }
    unsigned phases = 0;
    // fewer than 2^31 tiles and chunks per channel row (the launcher checks); a thread's chunks all lie in chunk
    // column k and its channel advances by kThreads / cols per step, so addresses are advanced, not recomputed
    const uint32_t inner_chunks = static_cast<uint32_t>(p.inner / EPC);
    const uint32_t tiles_per_outer = (inner_chunks + cols - 1) >> cols_log2;
    const uint32_t tiles = static_cast<uint32_t>(p.outer) * tiles_per_outer;
    const int k = threadIdx.x & (cols - 1), c0 = threadIdx.x >> cols_log2, c_step = kThreads >> cols_log2;
    const int64_t row_step = static_cast<int64_t>(c_step) * inner_chunks;

    auto request = [&](uint32_t t, int b) {
        if constexpr (TMA) {
            if (t < tiles && threadIdx.x == 0) {
                const uint32_t o = t / tiles_per_outer;
                const uint32_t chunk0 = (t - o * tiles_per_outer) << cols_log2;
                uint4* const dst = tiles_buffer + static_cast<size_t>(b) * tile_chunks;
                async_proxy_fence();
                mbarrier_expect_bytes(&barriers[b], static_cast<unsigned>(tile_chunks) * 16u);
                for (int c = 0; c < channels; c += slab)
                    tma_load_3d(dst + static_cast<size_t>(c) * cols, &map, static_cast<int>(chunk0 * EPC), c, static_cast<int>(o), &barriers[b]);
            }
            return;
        }
        if (t < tiles) {
            const uint32_t o = t / tiles_per_outer;
            const uint32_t chunk0 = (t - o * tiles_per_outer) << cols_log2;
            const uint4* src = static_cast<const uint4*>(p.x) + (static_cast<int64_t>(o) * channels + c0) * inner_chunks + chunk0 + k;
            uint4* dst = tiles_buffer + static_cast<size_t>(b) * tile_chunks + threadIdx.x;
            if (chunk0 + k < inner_chunks) {
                for (int idx = threadIdx.x; idx < tile_chunks; idx += kThreads, src += row_step, dst += kThreads) async_copy16(dst, src);
            } else {
                for (int idx = threadIdx.x; idx < tile_chunks; idx += kThreads, dst += kThreads) *dst = make_uint4(0, 0, 0, 0);
            }
        }
        async_copy_commit();
    };

    int buffer = 0;
    request(blockIdx.x, 0);
    for (uint32_t t = blockIdx.x; t < tiles; t += gridDim.x, buffer ^= 1) {
        const uint32_t o = t / tiles_per_outer;
        const uint32_t chunk0 = (t - o * tiles_per_outer) << cols_log2;
        const uint4* const tile = tiles_buffer + static_cast<size_t>(buffer) * tile_chunks;
        request(t + gridDim.x, buffer ^ 1);
        if constexpr (TMA) {
            const bool arrived = mbarrier_wait_bounded(&barriers[buffer], (phases >> buffer) & 1u, &g_async_wait_gave_up);
            phases ^= 1u << buffer;
            if (!__syncthreads_and(arrived)) {
                if (t + gridDim.x < tiles) mbarrier_wait_bounded(&barriers[buffer ^ 1], (phases >> (buffer ^ 1)) & 1u, &g_async_wait_gave_up);
                break;
            }
        } else {
            async_copy_wait<1>();
            __syncthreads();
        }
        constexpr int PPW = X_BF16 ? 2 : 1;
        const int words_log2 = cols_log2 + 2, words = 1 << words_log2;
        const uint32_t* const tile_words = reinterpret_cast<const uint32_t*>(tile);
        for (int item = threadIdx.x; item < words * kLanes; item += kThreads) {
            const int lane = item >> words_log2, word = item & (words - 1);
            double q0 = 0.0, q1 = 0.0;
            const uint32_t* e = tile_words + lane * words + word;
            const int step = kLanes * words;
#pragma unroll 4
            for (int c = lane; c < channels; c += kLanes, e += step) {
                const uint32_t w = *e;
                if constexpr (X_BF16) {
                    const double lo = static_cast<double>(__uint_as_float(w << 16)), hi = static_cast<double>(__uint_as_float(w & 0xffff0000u));
                    q0 = fma(lo, lo, q0);
                    q1 = fma(hi, hi, q1);
                } else {
                    const double v = static_cast<double>(__uint_as_float(w));
                    q0 = fma(v, v, q0);
                }
            }
            partial[lane * positions + word * PPW] = q0;
            if constexpr (X_BF16) partial[lane * positions + word * PPW + 1] = q1;
        }
        __syncthreads();
        if (threadIdx.x < positions) {
            double total = 0.0;
#pragma unroll
            for (int a = 0; a < kLanes; ++a) total += partial[a * positions + threadIdx.x];
            inverse[threadIdx.x] = rsqrtf(__fadd_rn(static_cast<float>(total / static_cast<double>(p.channels)), p.eps));
        }
        __syncthreads();
        if (chunk0 + k < inner_chunks) {
        // this thread's positions: inverses once per tile
        const float4* i4 = reinterpret_cast<const float4*>(inverse + k * EPC);
        const float4 ia = i4[0];
        float4 ib = ia;
        if constexpr (X_BF16) ib = i4[1];
        const bool weighted = p.weight != nullptr;
        uint4* out = static_cast<uint4*>(p.out) + (static_cast<int64_t>(o) * channels + c0) * inner_chunks + chunk0 + k;
        const uint4* chunk_at = tile + threadIdx.x;
        const uint32_t* weight_at = weights + c0;
        for (int idx = threadIdx.x; idx < tile_chunks; idx += kThreads, chunk_at += kThreads, out += row_step, weight_at += c_step) {
            const uint32_t weight_word = weighted ? *weight_at : 0u;
            const float w = weighted ? (X_BF16 ? __uint_as_float(weight_word << 16) : __uint_as_float(weight_word)) : 1.0f;
            const uint4 raw = *chunk_at;
            auto finish_one = [&](float v, float inv) {
                float y = __fmul_rn(v, inv);
                if constexpr (X_BF16) y = round_to_bf16(y);
                if (weighted) { y = __fmul_rn(y, w); if constexpr (X_BF16) y = round_to_bf16(y); }
                if constexpr (SILU) y = activation_value(VRB_SILU, y);
                return y;
            };
            if constexpr (X_BF16) {
                // two elements at a time: F32 products rounded to bf16 as a pair (one conversion), the weight applied as a
                // bf16 x bf16 product rounded once (exact product, same rounding as the F32 multiply + store of the
                // reference), SiLU per element on the bf16 bits
                const float inv[8] = {ia.x, ia.y, ia.z, ia.w, ib.x, ib.y, ib.z, ib.w};
                const uint32_t wd[4] = {raw.x, raw.y, raw.z, raw.w};
                const __nv_bfloat162 w2 = *reinterpret_cast<const __nv_bfloat162*>(&weight_word);
                uint32_t ow[4];
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    float a, b;
                    unpack_f32x2(mul_f32x2(pack_f32x2(__uint_as_float(wd[j] << 16), __uint_as_float(wd[j] & 0xffff0000u)),
                                           pack_f32x2(inv[2 * j], inv[2 * j + 1])), a, b);
                    __nv_bfloat162 y2 = __floats2bfloat162_rn(a, b);
                    if (weighted) y2 = __hmul2_rn(y2, w2);
                    uint32_t word = *reinterpret_cast<const uint32_t*>(&y2);
                    if constexpr (SILU) {
                        // the approximate form wherever its bf16 rounding provably equals the exact expression's
                        // (silu_approximate above; all 65536 bf16 arguments are checked by tests/test_gpu_pixel_norm.py),
                        // else the exact expression
                        const float lo = __uint_as_float(word << 16), hi = __uint_as_float(word & 0xffff0000u);
                        float s_lo, s_hi;
                        if (silu_approximate_pair(lo, hi, s_lo, s_hi)) {
                            if (!(fabsf(lo) <= 8.0f) || near_bf16_boundary(s_lo)) s_lo = activation_value(VRB_SILU, lo);
                            if (!(fabsf(hi) <= 8.0f) || near_bf16_boundary(s_hi)) s_hi = activation_value(VRB_SILU, hi);
                        }
                        word = pack_bf16x2(s_lo, s_hi);
                    }
                    ow[j] = word;
                }
                __stcs(out, make_uint4(ow[0], ow[1], ow[2], ow[3]));
            } else {
                __stcs(reinterpret_cast<float4*>(out),
                       make_float4(finish_one(__uint_as_float(raw.x), ia.x), finish_one(__uint_as_float(raw.y), ia.y),
                                   finish_one(__uint_as_float(raw.z), ia.z), finish_one(__uint_as_float(raw.w), ia.w)));
            }
        }
        }
        __syncthreads();
    }
    async_copy_wait<0>();
}

}  // namespace

// Launches the tile form of the axis RMSNorm when the layout allows it; false = caller's fallback.
bool launch_rms_axis_tiles(const void* x, int dtype, const void* weight, int weight_dtype, void* out, int64_t outer,
                           int64_t channels, int64_t inner, float eps, int fuse_silu, cudaStream_t stream) {
    const int epc = dtype == VRB_BF16 ? 8 : 4;
    if (inner % epc != 0 || !aligned16(x) || !aligned16(out) || channels >= (int64_t{1} << 20)) return false;
    const int64_t inner_chunks = inner / epc;
    if (outer * inner_chunks >= (int64_t{1} << 31)) return false;   // the tile kernel counts tiles and chunks in 32 bits
    RmsAxisParams p{x, out, weight, weight_dtype, outer, channels, inner, eps};
    for (int budget_ctas : {3, 1}) {
        for (int cols = 8, log2 = 3; cols >= 1; cols >>= 1, --log2) {
            if (cols > 1 && cols / 2 >= inner_chunks) continue;
            // two tile buffers, the partial sums and inverses, the weight per channel
            const size_t smem = 2 * static_cast<size_t>(channels) * cols * 16 + static_cast<size_t>(cols) * epc * (kLanes * 8 + 4) +
                                (weight ? static_cast<size_t>(channels) * 4 : 0);
            if (smem > (budget_ctas == 3 ? 72 * 1024 : 200 * 1024) || smem > kMaxTileBytes) continue;
            const int64_t tiles = outer * ((inner_chunks + cols - 1) / cols);
            bool launched = true;
            CUtensorMap map{};
            int slab = 0;
            if (g_tma_tiles.load(std::memory_order_relaxed) != 0 && (channels * cols) % 8 == 0) {
                for (int candidate = static_cast<int>(channels < 256 ? channels : 256); candidate >= 8 && slab == 0; --candidate)
                    if (channels % candidate == 0 && (static_cast<int64_t>(candidate) * cols) % 8 == 0) slab = candidate;
                if (slab != 0 && !encode_tile_map(&map, x, dtype, outer, channels, inner, cols * epc, slab)) slab = 0;
            }
            const size_t smem_all = smem + 16;   // + the two mbarriers
#define VRB_RA(XB, S)                                                                                                    \
    {                                                                                                                    \
        if (slab != 0) {                                                                                                 \
            const int per_sm = tile_ctas_per_sm(rms_axis_tile_kernel<XB, S, true>, smem_all);                            \
            if (per_sm < 1) launched = false;                                                                            \
            else rms_axis_tile_kernel<XB, S, true><<<grid_for(tiles, per_sm), kThreads, smem_all, stream>>>(p, cols, log2, map, slab);  \
        } else {                                                                                                         \
            const int per_sm = tile_ctas_per_sm(rms_axis_tile_kernel<XB, S, false>, smem_all);                           \
            if (per_sm < 1) launched = false;                                                                            \
            else rms_axis_tile_kernel<XB, S, false><<<grid_for(tiles, per_sm), kThreads, smem_all, stream>>>(p, cols, log2, map, slab); \
        }                                                                                                                \
    }
            if (dtype == VRB_BF16) { if (fuse_silu) VRB_RA(true, true) else VRB_RA(true, false) }
            else { if (fuse_silu) VRB_RA(false, true) else VRB_RA(false, false) }
#undef VRB_RA
            if (launched) return true;
        }
    }
    return false;
}

}  // namespace vrb

using namespace vrb;

namespace {
int pixel_norm_family(const void* x, int dtype, const void* scale, const void* shift, int mod_dtype, int fuse_silu, void* out,
                      int out_dtype, int64_t outer, int64_t channels, int64_t inner, float eps, int l2, vrb_stream stream);
}

extern "C" int vrb_async_wait_failures(int* failures) {
    VRB_REQUIRE(failures, VRB_ERR_INVALID, "async_wait_failures: null result");
    const cudaError_t e = cudaMemcpyFromSymbol(failures, g_async_wait_gave_up, sizeof(int));
    if (e != cudaSuccess) {
        set_error("CUDA error: %s (async_wait_failures)", cudaGetErrorString(e));
        return VRB_ERR_CUDA;
    }
    return VRB_OK;
}

extern "C" int vrb_pixel_norm(const void* x, int dtype, const void* scale, const void* shift, int mod_dtype, int fuse_silu,
                              void* out, int out_dtype, int64_t outer, int64_t channels, int64_t inner, float eps,
                              vrb_stream stream) {
    return pixel_norm_family(x, dtype, scale, shift, mod_dtype, fuse_silu, out, out_dtype, outer, channels, inner, eps, 0, stream);
}

extern "C" int vrb_l2_normalize(const void* x, void* out, int dtype, int64_t outer, int64_t channels, int64_t inner, float eps,
                                vrb_stream stream) {
    VRB_REQUIRE(eps >= 0.0f, VRB_ERR_INVALID, "l2 normalize contract violation");
    return pixel_norm_family(x, dtype, nullptr, nullptr, 0, 0, out, dtype, outer, channels, inner, eps, 1, stream);
}

namespace {
int pixel_norm_family(const void* x, int dtype, const void* scale, const void* shift, int mod_dtype, int fuse_silu, void* out,
                      int out_dtype, int64_t outer, int64_t channels, int64_t inner, float eps, int l2, vrb_stream stream) {
    VRB_REQUIRE(x && out, VRB_ERR_INVALID, "pixel_norm: null tensor");
    VRB_REQUIRE(outer > 0 && channels > 0 && inner > 0, VRB_ERR_INVALID, "pixel_norm: extents must be positive");
    VRB_REQUIRE(is_float_dtype(dtype) && is_float_dtype(out_dtype), VRB_ERR_UNSUPPORTED, "pixel_norm: tensors must be F32 or BF16");
    VRB_REQUIRE((scale == nullptr) == (shift == nullptr), VRB_ERR_INVALID, "pixel_norm: scale and shift come together");
    VRB_REQUIRE(!scale || is_float_dtype(mod_dtype), VRB_ERR_UNSUPPORTED, "pixel_norm: modulation vectors must be F32 or BF16");
    VRB_REQUIRE(scale || out_dtype == dtype, VRB_ERR_UNSUPPORTED, "pixel_norm: without modulation the result has x's dtype");
    PixelNormParams p{};
    p.x = x; p.out = out; p.scale = scale; p.shift = shift; p.x_dt = dtype; p.out_dt = out_dtype; p.mod_dt = mod_dtype;
    p.outer = outer; p.channels = channels; p.inner = inner; p.eps = eps; p.silu = fuse_silu ? 1 : 0; p.l2 = l2;
    cudaStream_t s = as_stream(stream);
    if (inner == 1) {
        pixel_norm_rows_kernel<<<grid_for(outer, 8), kThreads, 0, s>>>(p);
        return after_launch("pixel_norm");
    }
    const int epc = dtype == VRB_BF16 ? 8 : 4;
    if (inner % epc == 0 && aligned16(x) && aligned16(out) && channels < (int64_t{1} << 20) &&
        outer * (inner / epc) < (int64_t{1} << 31)) {      // the tile kernel counts tiles and chunks in 32 bits
        const int64_t inner_chunks = inner / epc;
        // widest tile (16-byte chunks per channel row) that leaves room for three CTAs per SM, else
        // for one; never wider than the row
        for (int budget_ctas : {3, 1}) {
            for (int cols = 8, log2 = 3; cols >= 1; cols >>= 1, --log2) {
                if (cols > 1 && cols / 2 >= inner_chunks) continue;
                const int mode = !scale ? kNormOnly : fuse_silu ? kModulateSilu : kModulate;
                // two tile buffers, the partial sums / denominators / reciprocals, and (1 + scale, shift) per channel
                const size_t smem = 2 * static_cast<size_t>(channels) * cols * 16 + static_cast<size_t>(kLanes + 2) * cols * epc * 4 +
                                    (mode != kNormOnly ? static_cast<size_t>(channels) * 8 : 0);
                if (smem > (budget_ctas == 3 ? 72 * 1024 : 200 * 1024) || smem > kMaxTileBytes) continue;
                const int variant = (dtype == VRB_BF16 ? 8 : 0) | (mode << 1) | (out_dtype == VRB_BF16 ? 1 : 0);
                const int64_t tiles = outer * ((inner_chunks + cols - 1) / cols);
                bool launched = true;
                // tensor-map loads: slabs of at most 256 channels whose bytes, like the tile's, are multiples of 128
                CUtensorMap map{};
                int slab = 0;
                if (g_tma_tiles.load(std::memory_order_relaxed) != 0 && (channels * cols) % 8 == 0) {
                    for (int candidate = static_cast<int>(channels < 256 ? channels : 256); candidate >= 8 && slab == 0; --candidate)
                        if (channels % candidate == 0 && (static_cast<int64_t>(candidate) * cols) % 8 == 0) slab = candidate;
                    if (slab != 0 && !encode_tile_map(&map, x, dtype, outer, channels, inner, cols * epc, slab)) slab = 0;
                }
                const size_t smem_all = smem + 16;   // + the two mbarriers
#define VRB_PN(XB, M, OB)                                                                                             \
    {                                                                                                                 \
        if (slab != 0) {                                                                                              \
            const int per_sm = tile_ctas_per_sm(pixel_norm_tile_kernel<XB, M, OB, true>, smem_all);                   \
            if (per_sm < 1) { launched = false; break; }                                                              \
            pixel_norm_tile_kernel<XB, M, OB, true><<<grid_for(tiles, per_sm), kThreads, smem_all, s>>>(p, cols, log2, map, slab); \
        } else {                                                                                                      \
            const int per_sm = tile_ctas_per_sm(pixel_norm_tile_kernel<XB, M, OB, false>, smem_all);                  \
            if (per_sm < 1) { launched = false; break; }                                                              \
            pixel_norm_tile_kernel<XB, M, OB, false><<<grid_for(tiles, per_sm), kThreads, smem_all, s>>>(p, cols, log2, map, slab); \
        }                                                                                                             \
    }                                                                                                                 \
    break
                switch (variant) {
                    case 0: case 1: VRB_PN(false, kNormOnly, false);
                    case 2: VRB_PN(false, kModulate, false);
                    case 3: VRB_PN(false, kModulate, true);
                    case 4: VRB_PN(false, kModulateSilu, false);
                    case 5: VRB_PN(false, kModulateSilu, true);
                    case 8: case 9: VRB_PN(true, kNormOnly, true);
                    case 10: VRB_PN(true, kModulate, false);
                    case 11: VRB_PN(true, kModulate, true);
                    case 12: VRB_PN(true, kModulateSilu, false);
                    default: VRB_PN(true, kModulateSilu, true);
                }
#undef VRB_PN
                if (!launched) continue;
                return after_launch("pixel_norm");
            }
        }
    }
    const int64_t units = outer * inner;
    pixel_norm_strided_kernel<<<grid_for((units + kThreads - 1) / kThreads, 8), kThreads, 0, s>>>(p);
    return after_launch("pixel_norm");
}
}  // namespace
