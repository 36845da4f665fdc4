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
// normalise pass of the reference read it twice.  P is chosen so that three CTAs fit on an SM.
#include "vrb_common.cuh"

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
};

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
__device__ __forceinline__ void async_copy_wait() { asm volatile("cp.async.wait_all;" ::: "memory"); }

// Tile kernel: inner % EPC == 0, 16-byte aligned tensors; `cols` (a power of two) 16-byte chunks per channel.
template <bool X_BF16>
__global__ void __launch_bounds__(kThreads) pixel_norm_tile_kernel(const PixelNormParams p, int cols, int cols_log2) {
    constexpr int EPC = X_BF16 ? 8 : 4;   // elements per 16-byte chunk
    extern __shared__ __align__(16) uint4 tile[];   // [channels][cols]
    const int channels = static_cast<int>(p.channels);
    const int positions = cols * EPC;
    float* const partial = reinterpret_cast<float*>(tile + static_cast<size_t>(channels) * cols);   // [kLanes][positions]
    float* const denominator = partial + kLanes * positions;                                        // [positions]
    const int64_t inner_chunks = p.inner / EPC;
    const int64_t tiles_per_outer = (inner_chunks + cols - 1) / cols;
    const int64_t tiles = p.outer * tiles_per_outer;
    const int tile_chunks = channels * cols;
    const bool modulated = p.scale != nullptr;
    const float channel_count = static_cast<float>(p.channels);
    const uint4* const x = static_cast<const uint4*>(p.x);

    for (int64_t t = blockIdx.x; t < tiles; t += gridDim.x) {
        const int64_t o = t / tiles_per_outer;
        const int64_t chunk0 = (t - o * tiles_per_outer) * cols;
        const int valid = static_cast<int>(inner_chunks - chunk0 < cols ? inner_chunks - chunk0 : cols);
        const uint4* const src = x + o * p.channels * inner_chunks + chunk0;
        for (int idx = threadIdx.x; idx < tile_chunks; idx += kThreads) {
            const int c = idx >> cols_log2, k = idx & (cols - 1);
            if (k < valid) async_copy16(tile + idx, src + static_cast<int64_t>(c) * inner_chunks + k);
            else tile[idx] = make_uint4(0, 0, 0, 0);
        }
        async_copy_wait();
        __syncthreads();
        // (position, lane) partial sums in the reference's order
        for (int pair = threadIdx.x; pair < positions * kLanes; pair += kThreads) {
            const int lane = pair / positions, pos = pair - lane * positions;
            float q = 0.0f;
            if constexpr (X_BF16) {
                const uint16_t* e = reinterpret_cast<const uint16_t*>(tile) + pos;
                for (int c = lane; c < channels; c += kLanes) {
                    const float v = bf16_bits_to_float(e[c * positions]);
                    q = __fmaf_rn(v, v, q);
                }
            } else {
                const float* e = reinterpret_cast<const float*>(tile) + pos;
                for (int c = lane; c < channels; c += kLanes) {
                    const float v = e[c * positions];
                    q = __fmaf_rn(v, v, q);
                }
            }
            partial[pair] = q;
        }
        __syncthreads();
        if (threadIdx.x < positions) {
            float s[kLanes];
#pragma unroll
            for (int a = 0; a < kLanes; ++a) s[a] = partial[a * positions + threadIdx.x];
            denominator[threadIdx.x] = __fsqrt_rn(__fadd_rn(__fdiv_rn(tree8(s), channel_count), p.eps));
        }
        __syncthreads();
        for (int idx = threadIdx.x; idx < tile_chunks; idx += kThreads) {
            const int c = idx >> cols_log2, k = idx & (cols - 1);
            if (k >= valid) continue;
            float ops = 1.0f, sh = 0.0f;
            if (modulated) {
                const int64_t at = o * p.channels + c;
                ops = __fadd_rn(1.0f, load1(p.scale, p.mod_dt, at));
                sh = load1(p.shift, p.mod_dt, at);
            }
            const uint4 raw = tile[idx];
            const int64_t element = ((o * p.channels + c) * inner_chunks + chunk0 + k) * EPC;
            const float* d = denominator + k * EPC;
            if constexpr (X_BF16) {
                const uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
                float v[8];
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    v[2 * j] = finish(p, __uint_as_float(w[j] << 16), d[2 * j], modulated, ops, sh);
                    v[2 * j + 1] = finish(p, __uint_as_float(w[j] & 0xffff0000u), d[2 * j + 1], modulated, ops, sh);
                }
                store8(p.out, p.out_dt, element, v);
            } else {
                const float in[4] = {__uint_as_float(raw.x), __uint_as_float(raw.y), __uint_as_float(raw.z), __uint_as_float(raw.w)};
                float v[4];
#pragma unroll
                for (int j = 0; j < 4; ++j) v[j] = finish(p, in[j], d[j], modulated, ops, sh);
                if (p.out_dt == VRB_BF16) {
                    __stcs(reinterpret_cast<uint2*>(static_cast<uint16_t*>(p.out) + element),
                           make_uint2(pack_bf16x2(v[0], v[1]), pack_bf16x2(v[2], v[3])));
                } else {
                    __stcs(reinterpret_cast<float4*>(static_cast<float*>(p.out) + element), make_float4(v[0], v[1], v[2], v[3]));
                }
            }
        }
        __syncthreads();   // the tile is overwritten by the next iteration's copies
    }
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
        const float denominator = __fsqrt_rn(__fadd_rn(__fdiv_rn(tree8(s), static_cast<float>(p.channels)), p.eps));
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
        const float denominator = __fsqrt_rn(__fadd_rn(__fdiv_rn(workspace[0], static_cast<float>(p.channels)), p.eps));
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

// Resident CTAs per SM of a tile kernel for a dynamic shared-memory size (opted into above 48 KB);
// remembered per (device, size), guarded for concurrent callers.
template <typename K>
int tile_ctas_per_sm(K kernel, size_t smem) {
    struct Entry { int device; size_t smem; int per_sm; };
    static std::mutex mutex;
    static std::vector<Entry> known;
    int device = 0;
    if (cudaGetDevice(&device) != cudaSuccess) return 0;
    std::lock_guard<std::mutex> lock(mutex);
    for (const Entry& e : known)
        if (e.device == device && e.smem == smem) return e.per_sm;
    int n = 0;
    if ((smem > 40 * 1024 &&
         cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem)) != cudaSuccess) ||
        cudaOccupancyMaxActiveBlocksPerMultiprocessor(&n, kernel, kThreads, smem) != cudaSuccess) {
        cudaGetLastError();
        n = 0;
    }
    if (known.size() < 256) known.push_back({device, smem, n});
    return n;
}

}  // namespace
}  // namespace vrb

using namespace vrb;

extern "C" int vrb_pixel_norm(const void* x, int dtype, const void* scale, const void* shift, int mod_dtype, int fuse_silu,
                              void* out, int out_dtype, int64_t outer, int64_t channels, int64_t inner, float eps,
                              vrb_stream stream) {
    VRB_REQUIRE(x && out, VRB_ERR_INVALID, "pixel_norm: null tensor");
    VRB_REQUIRE(outer > 0 && channels > 0 && inner > 0, VRB_ERR_INVALID, "pixel_norm: extents must be positive");
    VRB_REQUIRE(is_float_dtype(dtype) && is_float_dtype(out_dtype), VRB_ERR_UNSUPPORTED, "pixel_norm: tensors must be F32 or BF16");
    VRB_REQUIRE((scale == nullptr) == (shift == nullptr), VRB_ERR_INVALID, "pixel_norm: scale and shift come together");
    VRB_REQUIRE(!scale || is_float_dtype(mod_dtype), VRB_ERR_UNSUPPORTED, "pixel_norm: modulation vectors must be F32 or BF16");
    VRB_REQUIRE(scale || out_dtype == dtype, VRB_ERR_UNSUPPORTED, "pixel_norm: without modulation the result has x's dtype");
    PixelNormParams p{};
    p.x = x; p.out = out; p.scale = scale; p.shift = shift; p.x_dt = dtype; p.out_dt = out_dtype; p.mod_dt = mod_dtype;
    p.outer = outer; p.channels = channels; p.inner = inner; p.eps = eps; p.silu = fuse_silu ? 1 : 0;
    cudaStream_t s = as_stream(stream);
    if (inner == 1) {
        pixel_norm_rows_kernel<<<grid_for(outer, 8), kThreads, 0, s>>>(p);
        return after_launch("pixel_norm");
    }
    const int epc = dtype == VRB_BF16 ? 8 : 4;
    if (inner % epc == 0 && aligned16(x) && aligned16(out) && channels < (int64_t{1} << 20)) {
        const int64_t inner_chunks = inner / epc;
        // widest tile (16-byte chunks per channel row) that leaves room for three CTAs per SM, else
        // for one; never wider than the row
        for (int budget_ctas : {3, 1}) {
            for (int cols = 8, log2 = 3; cols >= 1; cols >>= 1, --log2) {
                if (cols > 1 && cols / 2 >= inner_chunks) continue;
                const size_t smem = static_cast<size_t>(channels) * cols * 16 + static_cast<size_t>(kLanes + 1) * cols * epc * 4;
                if (smem > (budget_ctas == 3 ? 72 * 1024 : 200 * 1024)) continue;
                const int per_sm = dtype == VRB_BF16 ? tile_ctas_per_sm(pixel_norm_tile_kernel<true>, smem)
                                                    : tile_ctas_per_sm(pixel_norm_tile_kernel<false>, smem);
                if (per_sm < 1) continue;
                const int64_t tiles = outer * ((inner_chunks + cols - 1) / cols);
                const int grid = grid_for(tiles, per_sm);
                if (dtype == VRB_BF16) pixel_norm_tile_kernel<true><<<grid, kThreads, smem, s>>>(p, cols, log2);
                else pixel_norm_tile_kernel<false><<<grid, kThreads, smem, s>>>(p, cols, log2);
                return after_launch("pixel_norm");
            }
        }
    }
    const int64_t units = outer * inner;
    pixel_norm_strided_kernel<<<grid_for((units + kThreads - 1) / kThreads, 8), kThreads, 0, s>>>(p);
    return after_launch("pixel_norm");
}
