// Table-driven unary kernels for bf16 tensors.
//
// A unary operator on a bf16 tensor is a function of a 16-bit input, so its complete function
// table has 65536 bf16 entries = 128 KB, which fits the shared memory of one SM.  For large
// tensors that beats evaluating the expression per element: GELU-tanh through tanhf costs
// about 30 instructions per element, more than the ~22 issue slots per element an SM has at
// full HBM rate, while a table lookup costs about 3.  The table is built by evaluating the SAME
// expression the direct kernel evaluates (activation_value(), i.e. the reference's
// activation_kernel expressions, native/src/backend/cuda/cuda_backend.cu:1098-1109) on every
// possible input, so the result is bit-identical to the direct kernel by construction.
//
// Building the table costs about 10 us of an SM's time, so the tables of the parameter-free
// operators (five activation kinds, exp, sqrt) live in a file-scope __device__ array (7 x 128 KB
// that every GPU loading the library holds until exit): nothing is allocated.  The first table
// launch per (device, operator) is preceded by a small build kernel on the same stream; when its
// last CTA has stored its entries it publishes a device-side flag.  Every table kernel reads that
// flag: set -> it copies the 128 KB from L2 into its shared memory (about 1 us, issued behind the
// first tensor loads); not set (another stream's build still running, a graph captured before any
// build, clamp with its caller-chosen bounds) -> it evaluates the table itself.  Either way the
// entries are the same bits, and no host-side synchronisation, event or allocation is involved.
#include "vrb_common.cuh"

#include <atomic>

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
__device__ __forceinline__ uint16_t table_entry(int i, float p0, float p1) {
    return static_cast<uint16_t>(float_to_bf16_bits(lut_value<OP>(bf16_bits_to_float(static_cast<uint32_t>(i)), p0, p1)));
}

// Resident tables of the parameter-free operators: slot = operator code (0-4 activation kinds),
// 5 = exp, 6 = sqrt.  g_table_done[slot] counts the build kernel's finished CTAs;
// g_table_published[slot] becomes 1 once all of them have stored their entries.
constexpr int kResidentTables = 7;
constexpr int kBuildCtas = kTableEntries / kLutThreads;
__device__ __align__(256) uint16_t g_resident_tables[kResidentTables][kTableEntries];
__device__ unsigned g_table_done[kResidentTables];
__device__ unsigned g_table_published[kResidentTables];

__host__ __device__ constexpr int resident_slot(int op) { return op <= 4 ? op : op == 6 ? 5 : op == 7 ? 6 : -1; }

// Shared table from the resident copy when `slot` has been published, evaluated here otherwise.
template <int OP>
__device__ __forceinline__ void fill_table(uint16_t* table, int slot, float p0, float p1) {
    __shared__ unsigned published;
    if (threadIdx.x == 0) {
        unsigned flag = 0;
        if (slot >= 0) asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(flag) : "l"(&g_table_published[slot]) : "memory");
        published = flag;
    }
    __syncthreads();
    if (published != 0) {
        const uint4* ready = reinterpret_cast<const uint4*>(g_resident_tables[slot]);
        uint4* dst = reinterpret_cast<uint4*>(table);
#pragma unroll
        for (int i = 0; i < kTableBytes / 16 / kLutThreads; ++i)
            dst[threadIdx.x + i * kLutThreads] = __ldcg(ready + threadIdx.x + i * kLutThreads);
    } else {
        for (int i = threadIdx.x; i < kTableEntries; i += kLutThreads) table[i] = table_entry<OP>(i, p0, p1);
    }
    __syncthreads();
}

// kBuildCtas CTAs of kLutThreads threads; the CTA that finishes last publishes the slot.
template <int OP>
__global__ void __launch_bounds__(kLutThreads) build_table_kernel(int slot) {
    const int i = blockIdx.x * kLutThreads + threadIdx.x;
    g_resident_tables[slot][i] = table_entry<OP>(i, 0.f, 0.f);
    __threadfence();
    __syncthreads();
    if (threadIdx.x == 0) {
        const unsigned finished = atomicAdd(&g_table_done[slot], 1u) + 1u;
        if (finished % kBuildCtas == 0) {   // a repeated build rewrites the same bits: still complete
            __threadfence();
            asm volatile("st.release.gpu.global.u32 [%0], %1;" :: "l"(&g_table_published[slot]), "r"(1u) : "memory");
        }
    }
}

__device__ __forceinline__ uint32_t lookup2(const uint16_t* table, uint32_t word) {
    return static_cast<uint32_t>(table[word & 0xffffu]) | (static_cast<uint32_t>(table[word >> 16]) << 16);
}

template <int OP>
__global__ void __launch_bounds__(kLutThreads, 1) unary_lut_kernel(const uint4* __restrict__ x, uint4* __restrict__ out,
                                                                  int64_t chunks, int slot,
                                                                  float p0, float p1, int overlapped) {
    extern __shared__ __align__(16) uint16_t table[];
    constexpr int U = 3;   // 16-byte loads in flight per thread; 3 measured 8 % faster than 2 or 4 (5 and more: slower)
    const int64_t stride = static_cast<int64_t>(gridDim.x) * kLutThreads;
    const int64_t first = static_cast<int64_t>(blockIdx.x) * kLutThreads + threadIdx.x;
    uint4 r[U];
    pdl_launch_dependents();
    // Overlapped launch: the table (library data) is filled while the previous kernel drains, the
    // tensor is touched only after it has completed.  Plain launch: the first tensor loads go out
    // before the table copy so HBM is busy while the table arrives.
    if (overlapped) fill_table<OP>(table, slot, p0, p1);
    pdl_wait();
#pragma unroll
    for (int u = 0; u < U; ++u)
        if (first + u * stride < chunks) r[u] = __ldcs(x + first + u * stride);
    if (!overlapped) fill_table<OP>(table, slot, p0, p1);
    for (int64_t i = first; i < chunks; i += stride * U) {
        if (i != first) {
#pragma unroll
            for (int u = 0; u < U; ++u)
                if (i + u * stride < chunks) r[u] = __ldcs(x + i + u * stride);
        }
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
                                                                   int64_t rows, int64_t hidden_chunks,
                                                                   int slot) {
    extern __shared__ __align__(16) uint16_t table[];
    pdl_launch_dependents();
    fill_table<VRB_SILU>(table, slot, 0.f, 0.f);   // library data: may overlap the previous kernel's tail
    pdl_wait();
    constexpr int U = 2;   // 3 measured slower here
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

// The bf16 linear epilogue (fused_bf16_linear_output_kernel, native/src/backend/cuda/cuda_backend.cu:
// 754-764) followed by an activation: y = bf16(accumulation + float(bias)) is a bf16 value, so
// activation(y) is read from the table.  8 accumulators -> 4 packed bf16 pairs:
__device__ __forceinline__ uint4 biased_pack(const float4& lo, const float4& hi, const uint4& bias, bool has_bias) {
    float v[8] = {lo.x, lo.y, lo.z, lo.w, hi.x, hi.y, hi.z, hi.w};
    if (has_bias) {
        const uint32_t bw[4] = {bias.x, bias.y, bias.z, bias.w};
#pragma unroll
        for (int k = 0; k < 4; ++k) {
            v[2 * k] = __fadd_rn(v[2 * k], __uint_as_float(bw[k] << 16));
            v[2 * k + 1] = __fadd_rn(v[2 * k + 1], __uint_as_float(bw[k] & 0xffff0000u));
        }
    }
    return make_uint4(pack_bf16x2(v[0], v[1]), pack_bf16x2(v[2], v[3]), pack_bf16x2(v[4], v[5]), pack_bf16x2(v[6], v[7]));
}

template <int OP>
__global__ void __launch_bounds__(kLutThreads, 1) linear_output_lut_kernel(const float4* __restrict__ accumulation,
                                                                          const uint4* __restrict__ bias,
                                                                          uint4* __restrict__ out, int64_t chunks,
                                                                          unsigned width_chunks,
                                                                          int slot, int overlapped) {
    extern __shared__ __align__(16) uint16_t table[];
        constexpr int U = 2;   // registers: U x (8 accumulators + 4 bias); 3 measured slower
    const int64_t stride = static_cast<int64_t>(gridDim.x) * kLutThreads;
    const int64_t first = static_cast<int64_t>(blockIdx.x) * kLutThreads + threadIdx.x;
    const bool has_bias = bias != nullptr;
    float4 a[U][2];
    uint4 b[U];
    auto request = [&](int64_t i) {
#pragma unroll
        for (int u = 0; u < U; ++u) {
            const int64_t c = i + u * stride;
            if (c >= chunks) break;
            a[u][0] = __ldcs(accumulation + 2 * c);
            a[u][1] = __ldcs(accumulation + 2 * c + 1);
            if (has_bias) b[u] = __ldg(bias + static_cast<unsigned>(c) % width_chunks);   // chunks < 2^32
        }
    };
    pdl_launch_dependents();
    if (overlapped) fill_table<OP>(table, slot, 0.f, 0.f);   // see unary_lut_kernel
    pdl_wait();
    request(first);   // plain launch: before the table copy, so HBM is busy while the table arrives
    if (!overlapped) fill_table<OP>(table, slot, 0.f, 0.f);
    for (int64_t i = first; i < chunks; i += stride * U) {
        if (i != first) request(i);
#pragma unroll
        for (int u = 0; u < U; ++u) {
            if (i + u * stride >= chunks) break;
            const uint4 y = biased_pack(a[u][0], a[u][1], b[u], has_bias);
            __stcs(out + i + u * stride,
                   make_uint4(lookup2(table, y.x), lookup2(table, y.y), lookup2(table, y.z), lookup2(table, y.w)));
        }
    }
}

// ... followed by SwiGLU (mochi.cpp:195-202): accumulation is [rows, 2 * hidden]; the value half and
// the gate half are each rounded to bf16 as the linear output would be, silu(gate) comes from the
// table, the product is one bf16 multiply.
__global__ void __launch_bounds__(kLutThreads, 1) linear_output_swiglu_lut_kernel(const float4* __restrict__ accumulation,
                                                                                 const uint4* __restrict__ bias,
                                                                                 uint4* __restrict__ out, int64_t chunks,
                                                                                 unsigned hidden_chunks,
                                                                                 int slot, int overlapped) {
    extern __shared__ __align__(16) uint16_t table[];
    const int64_t stride = static_cast<int64_t>(gridDim.x) * kLutThreads;
    const int64_t first = static_cast<int64_t>(blockIdx.x) * kLutThreads + threadIdx.x;
    const bool has_bias = bias != nullptr;
    float4 a[2], g[2];
    uint4 ba, bg;
    auto request = [&](int64_t c) {
        if (c >= chunks) return;
        const unsigned row = static_cast<unsigned>(c) / hidden_chunks, chunk = static_cast<unsigned>(c) - row * hidden_chunks;
        const float4* src = accumulation + (static_cast<int64_t>(row) * 2 * hidden_chunks + chunk) * 2;
        a[0] = __ldcs(src); a[1] = __ldcs(src + 1);
        g[0] = __ldcs(src + 2 * hidden_chunks); g[1] = __ldcs(src + 2 * hidden_chunks + 1);
        if (has_bias) { ba = __ldg(bias + chunk); bg = __ldg(bias + hidden_chunks + chunk); }
    };
    pdl_launch_dependents();
    if (overlapped) fill_table<VRB_SILU>(table, slot, 0.f, 0.f);   // see unary_lut_kernel
    pdl_wait();
    request(first);
    if (!overlapped) fill_table<VRB_SILU>(table, slot, 0.f, 0.f);
    for (int64_t i = first; i < chunks; i += stride) {
        if (i != first) request(i);
        const uint4 value = biased_pack(a[0], a[1], ba, has_bias), gate = biased_pack(g[0], g[1], bg, has_bias);
        const uint32_t vw[4] = {value.x, value.y, value.z, value.w}, gw[4] = {gate.x, gate.y, gate.z, gate.w};
        uint32_t ow[4];
#pragma unroll
        for (int k = 0; k < 4; ++k) {
            const uint32_t s = lookup2(table, gw[k]);
            const __nv_bfloat162 prod = __hmul2_rn(*reinterpret_cast<const __nv_bfloat162*>(&vw[k]),
                                                *reinterpret_cast<const __nv_bfloat162*>(&s));
            ow[k] = *reinterpret_cast<const uint32_t*>(&prod);
        }
        __stcs(out + i, make_uint4(ow[0], ow[1], ow[2], ow[3]));
    }
}

// GroupNorm normalise pass + SiLU on bf16 (CudaBackend::group_norm :4919-5008 followed by
// activation(Silu), native/src/components/autoencoder_kl.cpp:40-41): y = bf16((x - mean) * inv *
// gamma + beta) with the reference's rounding order, then silu(y) read from the table, since y is
// a bf16 value.  Every plane is cut into equal tiles of at most kLutThreads * U chunks, so the
// four constants are fetched once per tile and no tile is much emptier than the others.
__global__ void __launch_bounds__(kLutThreads, 1) gn_apply_silu_lut_kernel(
    const uint4* __restrict__ x, uint4* __restrict__ out, const void* __restrict__ weight, int w_dt,
    const void* __restrict__ bias, int b_dt, const float* __restrict__ mean, const float* __restrict__ inverse,
    int64_t planes, int64_t channels, int channels_per, int groups, int64_t frames, int64_t stat_frames, int64_t plane_chunks,
    int64_t tiles_per_plane, int64_t tile_chunks, GnScatter scatter, int slot) {
    extern __shared__ __align__(16) uint16_t table[];
    fill_table<VRB_SILU>(table, slot, 0.f, 0.f);
    constexpr int U = 4;   // 3 and 2 measured slower (760 / 840 us against 730 us on [1,256,28,240,424])
    // the launcher guarantees planes * tiles_per_plane < 2^31: 32-bit index arithmetic
    const unsigned tiles = static_cast<unsigned>(planes * tiles_per_plane), tpp = static_cast<unsigned>(tiles_per_plane);
    const unsigned nframes = static_cast<unsigned>(frames), nchannels = static_cast<unsigned>(channels);
    for (unsigned t = blockIdx.x; t < tiles; t += gridDim.x) {
        const unsigned plane = t / tpp;
        const int64_t tile_begin = static_cast<int64_t>(t - plane * tpp) * tile_chunks;
        const int64_t tile_end = tile_begin + tile_chunks < plane_chunks ? tile_begin + tile_chunks : plane_chunks;
        const int64_t c0 = tile_begin + threadIdx.x;
        unsigned frame = 0, bc = plane;
        if (nframes > 1) { bc = plane / nframes; frame = plane - bc * nframes; }
        const unsigned batch_entry = bc / nchannels, channel = bc - batch_entry * nchannels;
        const unsigned unit = (stat_frames > 1 ? batch_entry * nframes + frame : batch_entry) * static_cast<unsigned>(groups) +
                              channel / static_cast<unsigned>(channels_per);
        const float m = __ldg(mean + unit), inv = __ldg(inverse + unit);
        const float gamma = weight ? round_to(VRB_BF16, load1(weight, w_dt, channel)) : 1.0f;
        const float beta = bias ? round_to(VRB_BF16, load1(bias, b_dt, channel)) : 0.0f;
        const uint4* px = x + static_cast<int64_t>(plane) * plane_chunks;
        uint4* po = out + static_cast<int64_t>(plane) * plane_chunks;
        uint4 r[U];
#pragma unroll
        for (int u = 0; u < U; ++u)
            if (c0 + u * kLutThreads < tile_end) r[u] = __ldcs(px + c0 + u * kLutThreads);
#pragma unroll
        for (int u = 0; u < U; ++u) {
            if (c0 + u * kLutThreads >= tile_end) break;
            const uint32_t w[4] = {r[u].x, r[u].y, r[u].z, r[u].w};
            uint32_t o[4];
#pragma unroll
            for (int k = 0; k < 4; ++k) {
                const float lo = __uint_as_float(w[k] << 16), hi = __uint_as_float(w[k] & 0xffff0000u);
                const float ylo = __fmaf_rn(__fmul_rn(__fsub_rn(lo, m), inv), gamma, beta);
                const float yhi = __fmaf_rn(__fmul_rn(__fsub_rn(hi, m), inv), gamma, beta);
                o[k] = lookup2(table, pack_bf16x2(ylo, yhi));
            }
            const uint4 packed = make_uint4(o[0], o[1], o[2], o[3]);
            if (scatter.count == 0) {
                __stcs(po + c0 + u * kLutThreads, packed);
            } else {
                const int64_t at = (static_cast<int64_t>(plane) * scatter.plane_stride + scatter.plane_offset) / 8 + c0 + u * kLutThreads;
                for (int k = 0; k < scatter.count; ++k) __stcs(static_cast<uint4*>(scatter.dst[k]) + at, packed);
            }
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

// Host side of the resident tables: which (device, slot) build kernels have been launched.  The
// state only avoids launching a build twice; whether a table may be READ is decided on the device
// by the published flag, so a stale entry here (after cudaDeviceReset) costs speed, not results.
constexpr int kMaxDevices = 64;
std::atomic<int> g_build_launched[kMaxDevices][kResidentTables];

template <int OP>
void launch_build(int slot, cudaStream_t stream) {
    build_table_kernel<OP><<<kBuildCtas, kLutThreads, 0, stream>>>(slot);
    if (cudaGetLastError() == cudaSuccess) g_launches.fetch_add(1, std::memory_order_relaxed);
}

// Slot of OP's resident table (-1: none, the kernel evaluates its own), making sure its build
// kernel has been launched on this device -- on `stream`, ahead of the caller's kernel, unless
// that stream is being captured (a captured build would be rebuilt by every replay).
template <int OP>
int ready_table(cudaStream_t stream) {
    constexpr int slot = resident_slot(OP);
    if constexpr (slot >= 0) {
        int device = 0;
        if (cudaGetDevice(&device) != cudaSuccess || device < 0 || device >= kMaxDevices) return slot;
        std::atomic<int>& launched = g_build_launched[device][slot];
        if (launched.load(std::memory_order_acquire) != 0) return slot;
        cudaStreamCaptureStatus capturing = cudaStreamCaptureStatusNone;
        if (cudaStreamIsCapturing(stream, &capturing) != cudaSuccess || capturing != cudaStreamCaptureStatusNone) {
            cudaGetLastError();
            return slot;
        }
        if (launched.exchange(1, std::memory_order_acq_rel) == 0) launch_build<OP>(slot, stream);
    }
    return slot;
}

inline int overlapped_now() { return g_launch_overlap.load(std::memory_order_relaxed); }

template <int OP>
int launch_lut(const void* x, void* out, int64_t count, float p0, float p1, cudaStream_t stream) {
    static bool done[64] = {false};   // one flag set per OP instantiation
    if (int rc = reserve_table(unary_lut_kernel<OP>, done)) return rc;
    const int64_t chunks = count / 8;
    const int64_t per_cta = (chunks + kLutThreads - 1) / kLutThreads;
    const int grid = static_cast<int>(per_cta < sm_count() ? per_cta : sm_count());
    const int slot = ready_table<OP>(stream);
    launch_overlapped(unary_lut_kernel<OP>, dim3(grid), dim3(kLutThreads), kTableBytes, stream,
                      static_cast<const uint4*>(x), static_cast<uint4*>(out), chunks, slot, p0, p1, overlapped_now());
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

template <int OP>
int launch_linear_lut(const float* accumulation, const void* bias, void* out, int64_t rows, int64_t width, cudaStream_t stream) {
    static bool done[64] = {false};
    if (int rc = reserve_table(linear_output_lut_kernel<OP>, done)) return rc;
    const int64_t chunks = rows * (width / 8);
    const int64_t per_cta = (chunks + kLutThreads - 1) / kLutThreads;
    const int grid = static_cast<int>(per_cta < sm_count() ? per_cta : sm_count());
    const int slot = ready_table<OP>(stream);
    launch_overlapped(linear_output_lut_kernel<OP>, dim3(grid), dim3(kLutThreads), kTableBytes, stream,
                      reinterpret_cast<const float4*>(accumulation), static_cast<const uint4*>(bias), static_cast<uint4*>(out), chunks,
                      static_cast<unsigned>(width / 8), slot, overlapped_now());
    return after_launch("linear_output_activation (table)");
}

int launch_linear_output_lut(int kind, const float* accumulation, const void* bias, void* out, int64_t rows, int64_t width,
                             cudaStream_t stream) {
    switch (kind) {
        case 0: return launch_linear_lut<0>(accumulation, bias, out, rows, width, stream);
        case 1: return launch_linear_lut<1>(accumulation, bias, out, rows, width, stream);
        case 2: return launch_linear_lut<2>(accumulation, bias, out, rows, width, stream);
        case 3: return launch_linear_lut<3>(accumulation, bias, out, rows, width, stream);
        default: return launch_linear_lut<4>(accumulation, bias, out, rows, width, stream);
    }
}

int launch_linear_output_swiglu_lut(const float* accumulation, const void* bias, void* out, int64_t rows, int64_t hidden,
                                    cudaStream_t stream) {
    static bool done[64] = {false};
    if (int rc = reserve_table(linear_output_swiglu_lut_kernel, done)) return rc;
    const int64_t chunks = rows * (hidden / 8);
    const int64_t per_cta = (chunks + kLutThreads - 1) / kLutThreads;
    const int grid = static_cast<int>(per_cta < sm_count() ? per_cta : sm_count());
    const int slot = ready_table<VRB_SILU>(stream);
    launch_overlapped(linear_output_swiglu_lut_kernel, dim3(grid), dim3(kLutThreads), kTableBytes, stream,
                      reinterpret_cast<const float4*>(accumulation), static_cast<const uint4*>(bias), static_cast<uint4*>(out), chunks,
                      static_cast<unsigned>(hidden / 8), slot, overlapped_now());
    return after_launch("linear_output_swiglu (table)");
}

int launch_swiglu_lut(const void* proj, void* out, int64_t rows, int64_t hidden, cudaStream_t stream) {
    static bool done[64] = {false};
    if (int rc = reserve_table(swiglu_lut_kernel, done)) return rc;
    const int slot = ready_table<VRB_SILU>(stream);
    launch_overlapped(swiglu_lut_kernel, dim3(sm_count()), dim3(kLutThreads), kTableBytes, stream,
                      static_cast<const uint4*>(proj), static_cast<uint4*>(out), rows, hidden / 8, slot);
    return after_launch("swiglu (table)");
}

int launch_group_norm_apply_silu_lut(const void* x, const void* weight, int w_dt, const void* bias, int b_dt, void* out,
                                     int64_t planes, int64_t channels, int channels_per, int groups, int64_t frames,
                                     int64_t stat_frames, int64_t spatial, const float* mean, const float* inverse,
                                     const GnScatter& scatter, cudaStream_t stream) {
    static bool done[64] = {false};
    if (int rc = reserve_table(gn_apply_silu_lut_kernel, done)) return rc;
    const int64_t plane_chunks = spatial / 8;
    const int64_t tiles_per_plane = (plane_chunks + kLutThreads * 4 - 1) / (kLutThreads * 4);
    const int64_t tile_chunks = ((plane_chunks + tiles_per_plane - 1) / tiles_per_plane + 7) & ~int64_t{7};   // tiles start on 128-byte lines
    const int64_t tiles = planes * tiles_per_plane;
    const int grid = static_cast<int>(tiles < sm_count() ? tiles : sm_count());
    gn_apply_silu_lut_kernel<<<grid, kLutThreads, kTableBytes, stream>>>(
        static_cast<const uint4*>(x), static_cast<uint4*>(out), weight, w_dt, bias, b_dt, mean, inverse, planes, channels,
        channels_per, groups, frames, stat_frames, plane_chunks, tiles_per_plane, tile_chunks, scatter,
        ready_table<VRB_SILU>(stream));
    return after_launch("group_norm apply (table)");
}

}  // namespace vrb

// Builds every resident table of the current device on `stream` (seven small kernels).  Optional:
// the operator entry points do this on first use; a caller that captures its first launches into a
// CUDA graph calls it once per device before the capture so the captured kernels find the tables.
extern "C" int vrb_prepare_tables(vrb_stream stream) {
    using namespace vrb;
    cudaStream_t s = as_stream(stream);
    cudaStreamCaptureStatus capturing = cudaStreamCaptureStatusNone;
    if (cudaStreamIsCapturing(s, &capturing) != cudaSuccess || capturing != cudaStreamCaptureStatusNone) {
        cudaGetLastError();
        set_error("prepare_tables: the stream is being captured; call it before the capture begins");
        return VRB_ERR_INVALID;
    }
    ready_table<0>(s); ready_table<1>(s); ready_table<2>(s); ready_table<3>(s); ready_table<4>(s);
    ready_table<6>(s); ready_table<7>(s);
    const cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) {
        set_error("CUDA error: %s (function-table build)", cudaGetErrorString(e));
        return VRB_ERR_CUDA;
    }
    return VRB_OK;
}
