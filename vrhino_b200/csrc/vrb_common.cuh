// Shared device helpers and launch plumbing for the sm_100a operator kernels.
#pragma once

#include <cuda_bf16.h>
#include <cuda_runtime.h>

#include <atomic>
#include <cstdarg>
#include <cstdint>
#include <cstdio>

#include "vrb.h"

namespace vrb {

// ------------------------------------------------------------------ host-side plumbing --
void set_error(const char* format, ...);
extern std::atomic<uint64_t> g_launches;
extern std::atomic<uint64_t> g_device_allocations;   // cudaMalloc calls made by the library (host-buffer entry points only)

// SM count of the current device, cached per device index.
int sm_count();

inline cudaStream_t as_stream(vrb_stream s) { return static_cast<cudaStream_t>(s); }
inline bool is_float_dtype(int dt) { return dt == VRB_F32 || dt == VRB_BF16; }
inline size_t dtype_bytes(int dt) { return dt == VRB_F32 ? 4 : dt == VRB_BF16 ? 2 : 1; }
inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

#define VRB_REQUIRE(cond, code, ...)      \
    do {                                  \
        if (!(cond)) {                    \
            ::vrb::set_error(__VA_ARGS__); \
            return (code);                \
        }                                 \
    } while (0)

// Call after a kernel launch: counts it and turns a launch error into a status.
inline int after_launch(const char* what) {
    g_launches.fetch_add(1, std::memory_order_relaxed);
    const cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) {
        set_error("CUDA error: %s (%s)", cudaGetErrorString(e), what);
        return VRB_ERR_CUDA;
    }
    return VRB_OK;
}

// ---- overlapped launches (programmatic dependent launch) ------------------------------------
// With overlap enabled (the default; vrb_set_launch_overlap) the hot kernels are launched with the
// programmatic-stream-serialization attribute: the GPU may start scheduling their CTAs while the
// previous kernel of the stream drains, which hides the launch gap between short kernels.  Such a
// kernel calls pdl_wait() -- which returns once the previous kernel has completed and its writes
// are visible -- before it touches ANY memory the caller passed in (inputs, outputs, vectors,
// tables); only work on the library's own immutable data may precede it.  Every thread calls it
// unconditionally, so "this kernel has finished" always implies "its predecessors have finished".
// Without the attribute pdl_wait() returns at once.
extern std::atomic<int> g_launch_overlap;

template <typename... KArgs, typename... Args>
inline void launch_overlapped(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t stream, Args&&... args) {
    cudaLaunchConfig_t config = {};
    config.gridDim = grid;
    config.blockDim = block;
    config.dynamicSmemBytes = smem;
    config.stream = stream;
    cudaLaunchAttribute attribute[1];
    if (g_launch_overlap.load(std::memory_order_relaxed) != 0) {
        attribute[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attribute[0].val.programmaticStreamSerializationAllowed = 1;
        config.attrs = attribute;
        config.numAttrs = 1;
        if (cudaLaunchKernelEx(&config, kernel, static_cast<KArgs>(args)...) == cudaSuccess) return;
        // a driver / stream that refuses the attribute: plain launches from here on
        cudaGetLastError();
        g_launch_overlap.store(0, std::memory_order_relaxed);
        config.attrs = nullptr;
        config.numAttrs = 0;
    }
    cudaLaunchKernelEx(&config, kernel, static_cast<KArgs>(args)...);   // an error stays for after_launch()
}

// Persistent-style grid: enough CTAs to fill every SM `per_sm` times, never more than `work`.
inline int grid_for(int64_t work_items, int per_sm) {
    const int64_t cap = static_cast<int64_t>(sm_count()) * per_sm;
    const int64_t g = work_items < cap ? work_items : cap;
    return static_cast<int>(g < 1 ? 1 : g);
}

// Table-driven bf16 unary / SwiGLU kernels (vrb_lut.cu).  op: 0-4 activation kinds, 5 clamp,
// 6 exp, 7 sqrt.  Worth the 128 KB table copy per SM only for large tensors.
constexpr int64_t kLutMinElements = int64_t{4} << 20;
bool unary_lut_applicable(int dtype, int64_t count, const void* x, const void* out);
int launch_unary_lut(int op, const void* x, void* out, int64_t count, float p0, float p1, cudaStream_t stream);
int launch_swiglu_lut(const void* proj, void* out, int64_t rows, int64_t hidden, cudaStream_t stream);
// Linear epilogue + activation / SwiGLU through the table: width (hidden) % 8 == 0, 16-byte aligned
// operands, fewer than 2^32 chunks of 8 output elements.
int launch_linear_output_lut(int kind, const float* accumulation, const void* bias, void* out, int64_t rows, int64_t width,
                             cudaStream_t stream);
int launch_linear_output_swiglu_lut(const float* accumulation, const void* bias, void* out, int64_t rows, int64_t hidden,
                                    cudaStream_t stream);
// Where the GroupNorm normalise pass writes.  count == 0: `out`, laid out like x.  count > 0: the
// same values go to every dst[k] (this GPU's and peer-mapped full-size tensors), plane p of x
// landing at element p * plane_stride + plane_offset -- the all-gather of an H-sharded feature map
// done by the kernel's own stores.
// Axis RMSNorm through shared-memory tiles (vrb_pixel_norm.cu); false when the layout needs the
// caller's two-pass kernel (inner extent not a multiple of a 16-byte chunk, misaligned tensors).
bool launch_rms_axis_tiles(const void* x, int dtype, const void* weight, int weight_dtype, void* out, int64_t outer,
                           int64_t channels, int64_t inner, float eps, int fuse_silu, cudaStream_t stream);

struct GnScatter {
    void* dst[8];
    int count;
    int64_t plane_stride, plane_offset;
};
// GroupNorm normalise pass on bf16 followed by SiLU through the table: x is [planes, spatial]
// with spatial % 8 == 0; plane p = (batch entry, channel, frame) (frames == 1 for the contiguous
// form) belongs to statistics unit ((batch entry) * stat_frames + (stat_frames > 1 ? frame : 0)) *
// groups + channel / channels_per.
int launch_group_norm_apply_silu_lut(const void* x, const void* weight, int w_dt, const void* bias, int b_dt, void* out,
                                     int64_t planes, int64_t channels, int channels_per, int groups, int64_t frames,
                                     int64_t stat_frames, int64_t spatial, const float* mean, const float* inverse,
                                     const GnScatter& scatter, cudaStream_t stream);

// ------------------------------------------------------------------------ device side --
#ifdef __CUDACC__

// See launch_overlapped(): let the next kernel of the stream start being scheduled / wait for the
// previous kernel of the stream to have completed.
__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }

__device__ __forceinline__ float bf16_bits_to_float(uint32_t bits16) {
    return __uint_as_float(bits16 << 16);
}
// RNE narrowing, identical to __float2bfloat16 (NaN -> 0x7fff).
__device__ __forceinline__ uint32_t float_to_bf16_bits(float v) {
    return static_cast<uint32_t>(__bfloat16_as_ushort(__float2bfloat16_rn(v)));
}
__device__ __forceinline__ float round_to_bf16(float v) {
    return __bfloat162float(__float2bfloat16_rn(v));
}
// Value a tensor of dtype `dt` would hold after storing v.
__device__ __forceinline__ float round_to(int dt, float v) {
    return dt == VRB_BF16 ? round_to_bf16(v) : v;
}

// 128-bit streaming load of 8 consecutive elements starting at element index `e`
// (e % 8 == 0, base 16-byte aligned).  bf16: one 16-byte load; f32: two.
template <bool kStreaming>
__device__ __forceinline__ void load8(const void* base, int dt, int64_t e, float (&v)[8]) {
    if (dt == VRB_BF16) {
        const uint4* p = reinterpret_cast<const uint4*>(static_cast<const uint16_t*>(base) + e);
        const uint4 r = kStreaming ? __ldcs(p) : __ldg(p);
        v[0] = __uint_as_float(r.x << 16); v[1] = __uint_as_float(r.x & 0xffff0000u);
        v[2] = __uint_as_float(r.y << 16); v[3] = __uint_as_float(r.y & 0xffff0000u);
        v[4] = __uint_as_float(r.z << 16); v[5] = __uint_as_float(r.z & 0xffff0000u);
        v[6] = __uint_as_float(r.w << 16); v[7] = __uint_as_float(r.w & 0xffff0000u);
    } else {
        const float4* p = reinterpret_cast<const float4*>(static_cast<const float*>(base) + e);
        const float4 a = kStreaming ? __ldcs(p) : __ldg(p);
        const float4 b = kStreaming ? __ldcs(p + 1) : __ldg(p + 1);
        v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w;
        v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
    }
}

__device__ __forceinline__ uint32_t pack_bf16x2(float lo, float hi) {
    const __nv_bfloat162 h = __floats2bfloat162_rn(lo, hi);  // .x = lo (low half), RNE each
    return *reinterpret_cast<const uint32_t*>(&h);
}

// Round eight F32 values to bf16 precision in place, two per conversion instruction.
__device__ __forceinline__ void round8_bf16_inplace(float (&v)[8]) {
#pragma unroll
    for (int e = 0; e < 8; e += 2) {
        const uint32_t h = pack_bf16x2(v[e], v[e + 1]);
        v[e] = __uint_as_float(h << 16);
        v[e + 1] = __uint_as_float(h & 0xffff0000u);
    }
}

// 32 consecutive bytes in ONE store instruction (sm_100 has 256-bit global accesses).  A thread that
// writes 32 adjacent bytes as two 16-byte stores makes every store instruction of its warp touch each
// 32-byte sector half: measured on B200 a 1-read : 2-write stream reaches 4.6 TB/s that way and 5.6 TB/s
// with 32-byte stores (write-only: 5.9 TB/s either way).  `p` must be 32-byte aligned; store32() checks
// and falls back to two 16-byte stores.
__device__ __forceinline__ void store32_aligned(void* p, const uint4& a, const uint4& b) {
    asm volatile("st.global.cs.v8.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8};" ::"l"(p), "r"(a.x), "r"(a.y), "r"(a.z), "r"(a.w),
                 "r"(b.x), "r"(b.y), "r"(b.z), "r"(b.w)
                 : "memory");
}
__device__ __forceinline__ void store32(void* p, const uint4& a, const uint4& b) {
    if ((reinterpret_cast<uintptr_t>(p) & 31u) == 0) {
        store32_aligned(p, a, b);
    } else {
        __stcs(static_cast<uint4*>(p), a);
        __stcs(static_cast<uint4*>(p) + 1, b);
    }
}

// Streaming store of 8 consecutive elements (RNE narrowing for bf16).
__device__ __forceinline__ void store8(void* base, int dt, int64_t e, const float (&v)[8]) {
    if (dt == VRB_BF16) {
        uint4 r;
        r.x = pack_bf16x2(v[0], v[1]); r.y = pack_bf16x2(v[2], v[3]);
        r.z = pack_bf16x2(v[4], v[5]); r.w = pack_bf16x2(v[6], v[7]);
        __stcs(reinterpret_cast<uint4*>(static_cast<uint16_t*>(base) + e), r);
    } else {
        store32(static_cast<float*>(base) + e,
                make_uint4(__float_as_uint(v[0]), __float_as_uint(v[1]), __float_as_uint(v[2]), __float_as_uint(v[3])),
                make_uint4(__float_as_uint(v[4]), __float_as_uint(v[5]), __float_as_uint(v[6]), __float_as_uint(v[7])));
    }
}
// Streaming store of 16 consecutive bf16 elements (32 bytes) from F32 values.
__device__ __forceinline__ void store16_bf16(void* base, int64_t e, const float (&v)[16]) {
    store32(static_cast<uint16_t*>(base) + e,
            make_uint4(pack_bf16x2(v[0], v[1]), pack_bf16x2(v[2], v[3]), pack_bf16x2(v[4], v[5]), pack_bf16x2(v[6], v[7])),
            make_uint4(pack_bf16x2(v[8], v[9]), pack_bf16x2(v[10], v[11]), pack_bf16x2(v[12], v[13]), pack_bf16x2(v[14], v[15])));
}

__device__ __forceinline__ float load1(const void* base, int dt, int64_t e) {
    return dt == VRB_BF16 ? bf16_bits_to_float(static_cast<const uint16_t*>(base)[e])
                          : static_cast<const float*>(base)[e];
}
__device__ __forceinline__ void store1(void* base, int dt, int64_t e, float v) {
    if (dt == VRB_BF16) static_cast<__nv_bfloat16*>(base)[e] = __float2bfloat16_rn(v);
    else static_cast<float*>(base)[e] = v;
}

// ---- packed F32 arithmetic (two IEEE round-to-nearest operations per instruction) ------------
// sm_100 has add / sub / mul / fma on pairs of F32 values held in a 64-bit register; each half is
// rounded exactly like the scalar _rn operation, so results are bit-identical to per-element
// __fadd_rn / __fmul_rn / __fmaf_rn (no contraction either: these are explicit instructions).  The row
// kernels are bound by issue slots, and these halve the arithmetic's share of them.
__device__ __forceinline__ unsigned long long pack_f32x2(float lo, float hi) {
    unsigned long long r;
    asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(lo), "f"(hi));
    return r;
}
__device__ __forceinline__ void unpack_f32x2(unsigned long long v, float& lo, float& hi) {
    asm("mov.b64 {%0, %1}, %2;" : "=f"(lo), "=f"(hi) : "l"(v));
}
__device__ __forceinline__ unsigned long long add_f32x2(unsigned long long a, unsigned long long b) {
    unsigned long long r;
    asm("add.rn.f32x2 %0, %1, %2;" : "=l"(r) : "l"(a), "l"(b));
    return r;
}
__device__ __forceinline__ unsigned long long sub_f32x2(unsigned long long a, unsigned long long b) {
    unsigned long long r;
    asm("sub.rn.f32x2 %0, %1, %2;" : "=l"(r) : "l"(a), "l"(b));
    return r;
}
__device__ __forceinline__ unsigned long long mul_f32x2(unsigned long long a, unsigned long long b) {
    unsigned long long r;
    asm("mul.rn.f32x2 %0, %1, %2;" : "=l"(r) : "l"(a), "l"(b));
    return r;
}
__device__ __forceinline__ unsigned long long fma_f32x2(unsigned long long a, unsigned long long b, unsigned long long c) {
    unsigned long long r;
    asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(r) : "l"(a), "l"(b), "l"(c));
    return r;
}
// Eight-element forms over float[8] register arrays: pairs (0,1) (2,3) (4,5) (6,7).
#define VRB_PAIRWISE8(EXPR)                                              \
    _Pragma("unroll") for (int e = 0; e < 8; e += 2) {                   \
        const unsigned long long r_ = (EXPR);                            \
        unpack_f32x2(r_, y[e], y[e + 1]);                                \
    }
__device__ __forceinline__ void sub8_scalar(float (&y)[8], float s) {
    const unsigned long long ss = pack_f32x2(s, s);
    VRB_PAIRWISE8(sub_f32x2(pack_f32x2(y[e], y[e + 1]), ss))
}
__device__ __forceinline__ void mul8_scalar(float (&y)[8], float s) {
    const unsigned long long ss = pack_f32x2(s, s);
    VRB_PAIRWISE8(mul_f32x2(pack_f32x2(y[e], y[e + 1]), ss))
}
__device__ __forceinline__ void add8_scalar(float (&y)[8], float s) {
    const unsigned long long ss = pack_f32x2(s, s);
    VRB_PAIRWISE8(add_f32x2(pack_f32x2(y[e], y[e + 1]), ss))
}
__device__ __forceinline__ void mul8(float (&y)[8], const float (&b)[8]) {
    VRB_PAIRWISE8(mul_f32x2(pack_f32x2(y[e], y[e + 1]), pack_f32x2(b[e], b[e + 1])))
}
__device__ __forceinline__ void add8(float (&y)[8], const float (&b)[8]) {
    VRB_PAIRWISE8(add_f32x2(pack_f32x2(y[e], y[e + 1]), pack_f32x2(b[e], b[e + 1])))
}
__device__ __forceinline__ void fma8(float (&y)[8], const float (&b)[8], const float (&c)[8]) {   // y = y * b + c
    VRB_PAIRWISE8(fma_f32x2(pack_f32x2(y[e], y[e + 1]), pack_f32x2(b[e], b[e + 1]), pack_f32x2(c[e], c[e + 1])))
}
#undef VRB_PAIRWISE8

// The reference's activation_kernel expressions (cuda_backend.cu:1098-1109), written so the
// compiler sees the same operations in the same order.
__device__ __forceinline__ float activation_value(int kind, float x) {
    if (kind == VRB_SILU) return x / (1.0f + expf(-x));
    if (kind == VRB_GELU) return 0.5f * x * (1.0f + erff(x * 0.7071067811865475f));
    if (kind == VRB_GELU_TANH)
        return 0.5f * x * (1.0f + tanhf(0.7978845608028654f * (x + 0.044715f * x * x * x)));
    if (kind == VRB_TANH) return tanhf(x);
    return fmaxf(x, 0.0f);
}

#endif  // __CUDACC__

}  // namespace vrb
