// Reductions over one axis that keep the reference's order of additions: reduce_sum and softmax.
//
// reduce_sum over one axis (CudaBackend::reduce_sum, native/src/backend/cuda/cuda_backend.cu:4885-4892,
// reduce_sum_kernel :1790-1806): x [outer, reduced, inner] -> out [outer, inner],
//   out[o, i] = store(sum over r, in increasing r, of F32(x[o, r, i])), the sum held in F32.
// The order of the additions is the reference's (one thread per output element, r ascending), so the result is the
// same bits.  Mochi pools its text tokens with it (native/src/architectures/mochi.cpp:141-142).  With inner a
// multiple of 8 (bf16) / 4 (F32) a thread carries 8 / 4 adjacent columns through 16-byte loads -- each column still
// summed in its own order.
#include "vrb_common.cuh"

namespace vrb {
namespace {

constexpr int kThreads = 256;
constexpr int kPerSm = 8;

template <bool BF16>
__global__ void __launch_bounds__(kThreads) reduce_sum_vector_kernel(const uint4* __restrict__ x, void* __restrict__ out, int64_t outer,
                                                                     int64_t reduced, int64_t inner_chunks) {
    constexpr int EPC = BF16 ? 8 : 4;
    const int64_t total = outer * inner_chunks, step = static_cast<int64_t>(gridDim.x) * kThreads;
    for (int64_t item = static_cast<int64_t>(blockIdx.x) * kThreads + threadIdx.x; item < total; item += step) {
        const int64_t o = item / inner_chunks, chunk = item - o * inner_chunks;
        const uint4* p = x + o * reduced * inner_chunks + chunk;
        float sum[EPC];
#pragma unroll
        for (int e = 0; e < EPC; ++e) sum[e] = 0.0f;
        for (int64_t r = 0; r < reduced; ++r, p += inner_chunks) {
            const uint4 v = __ldg(p);
            if constexpr (BF16) {
                const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
                for (int k = 0; k < 4; ++k) {
                    sum[2 * k] = __fadd_rn(sum[2 * k], __uint_as_float(w[k] << 16));
                    sum[2 * k + 1] = __fadd_rn(sum[2 * k + 1], __uint_as_float(w[k] & 0xffff0000u));
                }
            } else {
                sum[0] = __fadd_rn(sum[0], __uint_as_float(v.x)); sum[1] = __fadd_rn(sum[1], __uint_as_float(v.y));
                sum[2] = __fadd_rn(sum[2], __uint_as_float(v.z)); sum[3] = __fadd_rn(sum[3], __uint_as_float(v.w));
            }
        }
        if constexpr (BF16) {
            static_cast<uint4*>(out)[item] = make_uint4(pack_bf16x2(sum[0], sum[1]), pack_bf16x2(sum[2], sum[3]), pack_bf16x2(sum[4], sum[5]),
                                                        pack_bf16x2(sum[6], sum[7]));
        } else {
            static_cast<float4*>(out)[item] = make_float4(sum[0], sum[1], sum[2], sum[3]);
        }
    }
}

__global__ void __launch_bounds__(kThreads) reduce_sum_scalar_kernel(const void* __restrict__ x, void* __restrict__ out, int dtype,
                                                                     int64_t outer, int64_t reduced, int64_t inner) {
    const int64_t total = outer * inner, step = static_cast<int64_t>(gridDim.x) * kThreads;
    for (int64_t item = static_cast<int64_t>(blockIdx.x) * kThreads + threadIdx.x; item < total; item += step) {
        const int64_t o = item / inner, i = item - o * inner;
        const int64_t base = o * reduced * inner + i;
        float sum = 0.0f;
        for (int64_t r = 0; r < reduced; ++r) sum = __fadd_rn(sum, load1(x, dtype, base + r * inner));
        store1(out, dtype, item, sum);
    }
}

// ---- softmax over one axis ---------------------------------------------------------------------------
// CudaBackend::softmax (:4893-4917, softmax_axis_kernel :1808-1829), x [outer, axis, inner]: per (o, i) the maximum
// (fmaxf from -inf), the denominator = sum over the axis, IN INDEX ORDER, of expf(x - max) held in F32, and
// out = store(expf(x - max) / denominator).  The reference runs one thread per (o, i); the order of its additions
// is kept here, so the results are the same bits.
//
// inner == 1 (rows contiguous): a warp per row.  The maximum is a shuffle reduction (order does not matter); for
// the denominator the lanes evaluate 32 exponentials side by side and every lane then adds them in index order
// (one shuffle + one add per element: the sum's dependency chain is the reference's, only the exponentials are
// parallel).
__global__ void __launch_bounds__(kThreads) softmax_rows_kernel(const void* __restrict__ x, void* __restrict__ out, int dtype, int64_t rows,
                                                                int64_t axis) {
    const int lane = threadIdx.x % 32;
    const int64_t warps = static_cast<int64_t>(gridDim.x) * (kThreads / 32);
    for (int64_t row = static_cast<int64_t>(blockIdx.x) * (kThreads / 32) + threadIdx.x / 32; row < rows; row += warps) {
        const int64_t base = row * axis;
        float maximum = -INFINITY;
        for (int64_t j = lane; j < axis; j += 32) maximum = fmaxf(maximum, load1(x, dtype, base + j));
#pragma unroll
        for (int offset = 16; offset > 0; offset >>= 1) maximum = fmaxf(maximum, __shfl_xor_sync(0xffffffffu, maximum, offset));
        float denominator = 0.0f;
        for (int64_t first = 0; first < axis; first += 32) {
            const int count = axis - first < 32 ? static_cast<int>(axis - first) : 32;
            float mine = 0.0f;
            if (lane < count) mine = expf(__fsub_rn(load1(x, dtype, base + first + lane), maximum));
            for (int l = 0; l < count; ++l) denominator = __fadd_rn(denominator, __shfl_sync(0xffffffffu, mine, l));
        }
        for (int64_t j = lane; j < axis; j += 32)
            store1(out, dtype, base + j, __fdiv_rn(expf(__fsub_rn(load1(x, dtype, base + j), maximum)), denominator));
    }
}

// inner > 1: a thread per (o, i), adjacent threads on adjacent i (coalesced along inner), the axis walked in order.
__global__ void __launch_bounds__(kThreads) softmax_columns_kernel(const void* __restrict__ x, void* __restrict__ out, int dtype,
                                                                   int64_t outer, int64_t axis, int64_t inner) {
    const int64_t total = outer * inner, step = static_cast<int64_t>(gridDim.x) * kThreads;
    for (int64_t item = static_cast<int64_t>(blockIdx.x) * kThreads + threadIdx.x; item < total; item += step) {
        const int64_t o = item / inner, i = item - o * inner;
        const int64_t base = o * axis * inner + i;
        float maximum = -INFINITY;
        for (int64_t r = 0; r < axis; ++r) maximum = fmaxf(maximum, load1(x, dtype, base + r * inner));
        float denominator = 0.0f;
        for (int64_t r = 0; r < axis; ++r) denominator = __fadd_rn(denominator, expf(__fsub_rn(load1(x, dtype, base + r * inner), maximum)));
        for (int64_t r = 0; r < axis; ++r)
            store1(out, dtype, base + r * inner, __fdiv_rn(expf(__fsub_rn(load1(x, dtype, base + r * inner), maximum)), denominator));
    }
}

}  // namespace
}  // namespace vrb

using namespace vrb;

extern "C" int vrb_softmax(const void* x, void* out, int dtype, int64_t outer, int64_t axis, int64_t inner, vrb_stream stream) {
    VRB_REQUIRE(is_float_dtype(dtype), VRB_ERR_UNSUPPORTED, "softmax: dtype must be F32 or BF16");
    VRB_REQUIRE(outer >= 0 && axis >= 0 && inner >= 0, VRB_ERR_INVALID, "softmax axis invalid");
    if (outer * axis * inner == 0) return VRB_OK;
    VRB_REQUIRE(x && out, VRB_ERR_INVALID, "softmax: null tensor");
    cudaStream_t s = as_stream(stream);
    if (inner == 1) {
        const int grid = grid_for((outer + kThreads / 32 - 1) / (kThreads / 32), kPerSm);
        softmax_rows_kernel<<<grid, kThreads, 0, s>>>(x, out, dtype, outer, axis);
    } else {
        const int64_t total = outer * inner;
        softmax_columns_kernel<<<grid_for((total + kThreads - 1) / kThreads, kPerSm), kThreads, 0, s>>>(x, out, dtype, outer, axis, inner);
    }
    return after_launch("softmax");
}

extern "C" int vrb_reduce_sum(const void* x, void* out, int dtype, int64_t outer, int64_t reduced, int64_t inner, vrb_stream stream) {
    VRB_REQUIRE(is_float_dtype(dtype), VRB_ERR_UNSUPPORTED, "reduce_sum: dtype must be F32 or BF16");
    VRB_REQUIRE(outer >= 0 && reduced >= 0 && inner >= 0, VRB_ERR_INVALID, "reduce dimension invalid");
    if (outer * inner == 0) return VRB_OK;
    VRB_REQUIRE(out && (x || reduced == 0), VRB_ERR_INVALID, "reduce_sum: null tensor");
    cudaStream_t s = as_stream(stream);
    const int epc = dtype == VRB_BF16 ? 8 : 4;
    if (inner % epc == 0 && aligned16(x) && aligned16(out)) {
        const int64_t inner_chunks = inner / epc, total = outer * inner_chunks;
        const int grid = grid_for((total + kThreads - 1) / kThreads, kPerSm);
        if (dtype == VRB_BF16)
            reduce_sum_vector_kernel<true><<<grid, kThreads, 0, s>>>(static_cast<const uint4*>(x), out, outer, reduced, inner_chunks);
        else
            reduce_sum_vector_kernel<false><<<grid, kThreads, 0, s>>>(static_cast<const uint4*>(x), out, outer, reduced, inner_chunks);
    } else {
        const int64_t total = outer * inner;
        reduce_sum_scalar_kernel<<<grid_for((total + kThreads - 1) / kThreads, kPerSm), kThreads, 0, s>>>(x, out, dtype, outer, reduced, inner);
    }
    return after_launch("reduce_sum");
}
