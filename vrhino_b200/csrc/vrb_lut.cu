// Table-driven unary kernels for bf16 tensors.
//
// A unary operator on a bf16 tensor is a function of a 16-bit input, so its complete function
// table has 65536 bf16 entries = 128 KB, which fits the shared memory of one SM.  For large
// tensors that beats evaluating the expression per element: GELU-tanh through tanhf costs
// about 30 instructions per element, more than the ~22 issue slots per element an SM has at
// full HBM rate, while a table lookup costs about 3.  Every CTA (one per SM, 1024 threads)
// first fills its table by evaluating the SAME expression the direct kernel evaluates
// (activation_value(), i.e. the reference's activation_kernel expressions,
// native/src/backend/cuda/cuda_backend.cu:1098-1109) on every possible input, then streams the
// tensor through it.  The result is therefore bit-identical to the direct kernel by
// construction.  The fill costs about 10 us per launch, so callers use it only above a size
// threshold.
#include "vrb_common.cuh"

namespace vrb {
namespace {

constexpr int kLutThreads = 1024;
constexpr int kTableEntries = 65536;
constexpr int kTableBytes = kTableEntries * 2;

template <int OP>
__device__ __forceinline__ float lut_value(float x, float p0, float p1) {
    if constexpr (OP <= VRB_RELU) return activation_value(OP, x);
    else if constexpr (OP == 5) return fminf(p1, fmaxf(p0, x));
    else if constexpr (OP == 6) return expf(x);
    else return sqrtf(x);
}

template <int OP>
__device__ __forceinline__ void fill_table(uint16_t* table, float p0, float p1) {
    for (int i = threadIdx.x; i < kTableEntries; i += kLutThreads)
        table[i] = static_cast<uint16_t>(float_to_bf16_bits(lut_value<OP>(bf16_bits_to_float(static_cast<uint32_t>(i)), p0, p1)));
    __syncthreads();
}

__device__ __forceinline__ uint32_t lookup2(const uint16_t* table, uint32_t word) {
    return static_cast<uint32_t>(table[word & 0xffffu]) | (static_cast<uint32_t>(table[word >> 16]) << 16);
}

template <int OP>
__global__ void __launch_bounds__(kLutThreads, 1) unary_lut_kernel(const uint4* __restrict__ x, uint4* __restrict__ out,
                                                                  int64_t chunks, float p0, float p1) {
    extern __shared__ __align__(16) uint16_t table[];
    fill_table<OP>(table, p0, p1);
    constexpr int U = 4;
    const int64_t stride = static_cast<int64_t>(gridDim.x) * kLutThreads;
    for (int64_t i = static_cast<int64_t>(blockIdx.x) * kLutThreads + threadIdx.x; i < chunks; i += stride * U) {
        uint4 r[U];
#pragma unroll
        for (int u = 0; u < U; ++u)
            if (i + u * stride < chunks) r[u] = __ldcs(x + i + u * stride);
#pragma unroll
        for (int u = 0; u < U; ++u) {
            if (i + u * stride >= chunks) break;
            uint4 o;
            o.x = lookup2(table, r[u].x); o.y = lookup2(table, r[u].y);
            o.z = lookup2(table, r[u].z); o.w = lookup2(table, r[u].w);
            __stcs(out + i + u * stride, o);
        }
    }
}

// SwiGLU (native/src/architectures/mochi.cpp:195-202) on bf16: silu(gate) comes from the table
// already rounded to bf16, the product a * silu(gate) is one bf16 multiply (the exact product
// of two bf16 values rounded once, which is what the reference's F32 multiply followed by the
// bf16 store produces).
__global__ void __launch_bounds__(kLutThreads, 1) swiglu_lut_kernel(const uint4* __restrict__ proj, uint4* __restrict__ out,
                                                                   int64_t rows, int64_t hidden_chunks) {
    extern __shared__ __align__(16) uint16_t table[];
    fill_table<VRB_SILU>(table, 0.f, 0.f);
    constexpr int U = 2;
    const int64_t total = rows * hidden_chunks;
    const int64_t stride = static_cast<int64_t>(gridDim.x) * kLutThreads;
    for (int64_t i0 = static_cast<int64_t>(blockIdx.x) * kLutThreads + threadIdx.x; i0 < total; i0 += stride * U) {
        uint4 a[U], g[U];
#pragma unroll
        for (int u = 0; u < U; ++u) {
            const int64_t i = i0 + u * stride;
            if (i >= total) break;
            const int64_t row = i / hidden_chunks, chunk = i - row * hidden_chunks;
            const int64_t in0 = row * 2 * hidden_chunks + chunk;
            a[u] = __ldcs(proj + in0);
            g[u] = __ldcs(proj + in0 + hidden_chunks);
        }
#pragma unroll
        for (int u = 0; u < U; ++u) {
            const int64_t i = i0 + u * stride;
            if (i >= total) break;
            const uint32_t aw[4] = {a[u].x, a[u].y, a[u].z, a[u].w};
            const uint32_t gw[4] = {g[u].x, g[u].y, g[u].z, g[u].w};
            uint32_t ow[4];
#pragma unroll
            for (int k = 0; k < 4; ++k) {
                const uint32_t s = lookup2(table, gw[k]);
                const __nv_bfloat162 prod = __hmul2_rn(*reinterpret_cast<const __nv_bfloat162*>(&aw[k]),
                                                    *reinterpret_cast<const __nv_bfloat162*>(&s));
                ow[k] = *reinterpret_cast<const uint32_t*>(&prod);
            }
            __stcs(out + i, make_uint4(ow[0], ow[1], ow[2], ow[3]));
        }
    }
}

// The 128 KB table needs the opt-in shared-memory limit; set once per kernel and device.
template <typename K>
int reserve_table(K kernel, bool* done) {
    int device = 0;
    if (cudaGetDevice(&device) != cudaSuccess || device < 0 || device >= 64) device = 0;
    if (!done[device]) {
        if (cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, kTableBytes) != cudaSuccess) {
            set_error("CUDA error: cannot reserve %d bytes of shared memory for the function table", kTableBytes);
            return VRB_ERR_CUDA;
        }
        done[device] = true;
    }
    return VRB_OK;
}

template <int OP>
int launch_lut(const void* x, void* out, int64_t count, float p0, float p1, cudaStream_t stream) {
    static bool done[64] = {false};   // one flag set per OP instantiation
    if (int rc = reserve_table(unary_lut_kernel<OP>, done)) return rc;
    const int64_t chunks = count / 8;
    unary_lut_kernel<OP><<<sm_count(), kLutThreads, kTableBytes, stream>>>(
        static_cast<const uint4*>(x), static_cast<uint4*>(out), chunks, p0, p1);
    return after_launch("unary (table)");
}

}  // namespace

bool unary_lut_applicable(int dtype, int64_t count, const void* x, const void* out) {
    return dtype == VRB_BF16 && count >= kLutMinElements && count % 8 == 0 && aligned16(x) && aligned16(out);
}

int launch_unary_lut(int op, const void* x, void* out, int64_t count, float p0, float p1, cudaStream_t stream) {
    switch (op) {
        case 0: return launch_lut<0>(x, out, count, p0, p1, stream);
        case 1: return launch_lut<1>(x, out, count, p0, p1, stream);
        case 2: return launch_lut<2>(x, out, count, p0, p1, stream);
        case 3: return launch_lut<3>(x, out, count, p0, p1, stream);
        case 4: return launch_lut<4>(x, out, count, p0, p1, stream);
        case 5: return launch_lut<5>(x, out, count, p0, p1, stream);
        case 6: return launch_lut<6>(x, out, count, p0, p1, stream);
        default: return launch_lut<7>(x, out, count, p0, p1, stream);
    }
}

int launch_swiglu_lut(const void* proj, void* out, int64_t rows, int64_t hidden, cudaStream_t stream) {
    static bool done[64] = {false};
    if (int rc = reserve_table(swiglu_lut_kernel, done)) return rc;
    swiglu_lut_kernel<<<sm_count(), kLutThreads, kTableBytes, stream>>>(
        static_cast<const uint4*>(proj), static_cast<uint4*>(out), rows, hidden / 8);
    return after_launch("swiglu (table)");
}

}  // namespace vrb
