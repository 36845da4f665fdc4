// pixel_shuffle_nd (CudaBackend::pixel_shuffle_nd, native/src/backend/cuda/cuda_backend.cu:5112-5118,
// pixel_shuffle_kernel :2170-2186) and LTX's depth_to_space block built on it
// (native/src/architectures/ltx.cpp:250-259).  Pure index work plus one add: bit-exact.
//
// pixel_shuffle: x [B, C*ft*fh*fw, T, H, W] -> out [B, C, T*ft, H*fh, W*fw] with
//   out[b, c, t*ft+pt, h*fh+ph, w*fw+pw] = x[b, ((c*ft+pt)*fh+ph)*fw+pw, t, h, w].
// For a fixed (b, c, output frame, output row) the output row interleaves fw contiguous input
// rows, so a thread loads 16 bytes from each of them and stores fw * 16 contiguous bytes
// (fw = 1 or 2); other factors take the element-wise kernel.
//
// depth_to_space (LTX decoder up-block), with y = the block's convolution output [B, 4C, T, H, W]
// and x = the block's input [B, C, T, H, W]:
//   residual = slice(concat(4 x pixel_shuffle(x, {2,2,2}), dim 1), dim 2, 1, 2T)
//   out      = slice(pixel_shuffle(y, {2,2,2}), dim 2, 1, 2T) + residual            [B, C/2, 2T-1, 2H, 2W]
// The reference materialises six intermediates (two shuffles, the four-fold concat, two slices) before
// the add; here each output element gathers its two sources directly and the four output channels
// that share a residual element are produced together: y and x are read once, the result is written once.
#include "vrb_common.cuh"

namespace vrb {
namespace {

constexpr int kThreads = 256;
constexpr int kPerSm = 8;

struct ShuffleGeom {
    int64_t batch, channels, frames, height, width;   // of the OUTPUT's channel count and the INPUT's T, H, W
    int ft, fh, fw;
    int skip_frames;      // leading output frames dropped (depth_to_space: 1)
    int residual_period;  // depth_to_space: channels of pixel_shuffle(x) (the four-fold concat repeats them)
};

// Element-wise form: any factors.
template <typename T, bool RESIDUAL>
__global__ void __launch_bounds__(kThreads) shuffle_scalar_kernel(const T* __restrict__ y, const T* __restrict__ x,
                                                                  T* __restrict__ out, ShuffleGeom g) {
    const int64_t out_frames = g.frames * g.ft - g.skip_frames, out_h = g.height * g.fh, out_w = g.width * g.fw;
    const int64_t total = g.batch * g.channels * out_frames * out_h * out_w;
    const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
    const int64_t plane = g.frames * g.height * g.width;
    const int product = g.ft * g.fh * g.fw;
    for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < total; i += stride) {
        int64_t r = i;
        const int64_t ow = r % out_w; r /= out_w;
        const int64_t oh = r % out_h; r /= out_h;
        const int64_t ot = r % out_frames + g.skip_frames; r /= out_frames;
        const int64_t c = r % g.channels, b = r / g.channels;
        const int64_t iw = ow / g.fw, pw = ow % g.fw, ih = oh / g.fh, ph = oh % g.fh, it = ot / g.ft, pt = ot % g.ft;
        const int64_t sub = (pt * g.fh + ph) * g.fw + pw;
        const int64_t at = (it * g.height + ih) * g.width + iw;
        const T* src = y + ((b * g.channels + c) * product + sub) * plane + at;
        if constexpr (RESIDUAL) {
            const int64_t cr = c % g.residual_period;
            const T* res = x + ((b * g.residual_period + cr) * product + sub) * plane + at;
            if constexpr (sizeof(T) == 2) {
                const float sum = __fadd_rn(bf16_bits_to_float(*reinterpret_cast<const uint16_t*>(src)),
                                            bf16_bits_to_float(*reinterpret_cast<const uint16_t*>(res)));
                reinterpret_cast<uint16_t*>(out)[i] = static_cast<uint16_t>(float_to_bf16_bits(sum));
            } else {
                reinterpret_cast<float*>(out)[i] = __fadd_rn(*reinterpret_cast<const float*>(src), *reinterpret_cast<const float*>(res));
            }
        } else {
            out[i] = *src;
        }
    }
}

__device__ __forceinline__ uint4 add_chunks(const uint4& a, const uint4& b, bool bf16) {
    if (bf16) {
        const uint32_t aw[4] = {a.x, a.y, a.z, a.w}, bw[4] = {b.x, b.y, b.z, b.w};
        uint32_t o[4];
#pragma unroll
        for (int k = 0; k < 4; ++k) {
            // F32 add of two bf16 values followed by the bf16 store == one bf16 add (the exact sum is rounded once)
            const __nv_bfloat162 s = __hadd2_rn(*reinterpret_cast<const __nv_bfloat162*>(&aw[k]),
                                                *reinterpret_cast<const __nv_bfloat162*>(&bw[k]));
            o[k] = *reinterpret_cast<const uint32_t*>(&s);
        }
        return make_uint4(o[0], o[1], o[2], o[3]);
    }
    return make_uint4(__float_as_uint(__fadd_rn(__uint_as_float(a.x), __uint_as_float(b.x))),
                      __float_as_uint(__fadd_rn(__uint_as_float(a.y), __uint_as_float(b.y))),
                      __float_as_uint(__fadd_rn(__uint_as_float(a.z), __uint_as_float(b.z))),
                      __float_as_uint(__fadd_rn(__uint_as_float(a.w), __uint_as_float(b.w))));
}

// Interleave two 16-byte chunks element by element (ELEM = 2 or 4 bytes): even elements from a, odd from b.
template <int ELEM>
__device__ __forceinline__ void interleave(const uint4& a, const uint4& b, uint4& lo, uint4& hi) {
    if constexpr (ELEM == 4) {
        lo = make_uint4(a.x, b.x, a.y, b.y);
        hi = make_uint4(a.z, b.z, a.w, b.w);
    } else {
        auto mix = [](uint32_t p, uint32_t q, uint32_t& first, uint32_t& second) {
            first = __byte_perm(p, q, 0x5410);    // p.lo16 | q.lo16 << 16
            second = __byte_perm(p, q, 0x7632);   // p.hi16 | q.hi16 << 16
        };
        mix(a.x, b.x, lo.x, lo.y); mix(a.y, b.y, lo.z, lo.w);
        mix(a.z, b.z, hi.x, hi.y); mix(a.w, b.w, hi.z, hi.w);
    }
}

// Row form: fw = 1 or 2, the input width a multiple of the elements in 16 bytes, 16-byte aligned
// tensors.  One work item = one 16-byte chunk position of an input row group -> FW * 16 output bytes.
// I: index type of the work-item decode (unsigned when everything fits 32 bits: the divisions
// are the bulk of the instructions).
template <int ELEM, int FW, bool RESIDUAL, typename I>
__global__ void __launch_bounds__(kThreads) shuffle_rows_kernel(const uint4* __restrict__ y, const uint4* __restrict__ x,
                                                                uint4* __restrict__ out, ShuffleGeom g) {
    constexpr int EPC = 16 / ELEM;
    const I row_chunks = static_cast<I>(g.width / EPC);                    // per input row
    const I out_frames = static_cast<I>(g.frames * g.ft - g.skip_frames), out_h = static_cast<I>(g.height * g.fh);
    const I channels = static_cast<I>(g.channels), fh = static_cast<I>(g.fh), ft = static_cast<I>(g.ft);
    const I total = static_cast<I>(g.batch * g.channels) * out_frames * out_h * row_chunks;
    const I stride = static_cast<I>(gridDim.x) * blockDim.x;
    const int64_t plane_chunks = g.frames * g.height * (g.width / EPC);    // one input channel
    const int product = g.ft * g.fh * g.fw;
    constexpr int U = 2;   // work items per thread and iteration: all their loads are issued before any is used
    for (I i0 = static_cast<I>(blockIdx.x) * blockDim.x + threadIdx.x; i0 < total; i0 += stride * U) {
        uint4 v[U][FW], w[U][FW];
#pragma unroll
        for (int u = 0; u < U; ++u) {
            const I i = i0 + static_cast<I>(u) * stride;
            if (i >= total || i < i0) break;
            const I row = i / row_chunks, k = i - row * row_chunks;
            I r = row;
            const I oh = r % out_h; r /= out_h;
            const I ot = r % out_frames + static_cast<I>(g.skip_frames); r /= out_frames;
            const I c = r % channels, b = r / channels;
            const I ih = oh / fh, ph = oh - ih * fh, it = ot / ft, pt = ot - it * ft;
            const int64_t sub = static_cast<int64_t>(pt * fh + ph) * FW;          // + pw
            const int64_t at = (static_cast<int64_t>(it) * g.height + ih) * row_chunks + k;
            const uint4* src = y + ((static_cast<int64_t>(b) * g.channels + c) * product + sub) * plane_chunks + at;
#pragma unroll
            for (int pw = 0; pw < FW; ++pw) v[u][pw] = __ldcs(src + pw * plane_chunks);
            if constexpr (RESIDUAL) {
                const I cr = c % static_cast<I>(g.residual_period);
                const uint4* res = x + ((static_cast<int64_t>(b) * g.residual_period + cr) * product + sub) * plane_chunks + at;
#pragma unroll
                for (int pw = 0; pw < FW; ++pw) w[u][pw] = __ldg(res + pw * plane_chunks);
            }
        }
#pragma unroll
        for (int u = 0; u < U; ++u) {
            const I i = i0 + static_cast<I>(u) * stride;
            if (i >= total || i < i0) break;
            if constexpr (RESIDUAL) {
#pragma unroll
                for (int pw = 0; pw < FW; ++pw) v[u][pw] = add_chunks(v[u][pw], w[u][pw], ELEM == 2);
            }
            uint4* dst = out + static_cast<int64_t>(i) * FW;
            if constexpr (FW == 1) {
                __stcs(dst, v[u][0]);
            } else {
                uint4 lo, hi;
                interleave<ELEM>(v[u][0], v[u][1], lo, hi);
                store32(dst, lo, hi);
            }
        }
    }
}

// depth_to_space on rows: factors (2, 2, 2), first output frame dropped.  One work item = one 16-byte
// chunk position of the residual's row pair, serving the FOUR output channels that share it (the
// four-fold concat): the block input is read once, not once per copy.
template <int ELEM, typename I>
__global__ void __launch_bounds__(kThreads) depth_to_space_rows_kernel(const uint4* __restrict__ y, const uint4* __restrict__ x,
                                                                       uint4* __restrict__ out, ShuffleGeom g) {
    constexpr int EPC = 16 / ELEM, REPS = 4;
    const I row_chunks = static_cast<I>(g.width / EPC);
    const I out_frames = static_cast<I>(g.frames * 2 - 1), out_h = static_cast<I>(g.height * 2);
    const I period = static_cast<I>(g.residual_period);
    const I total = static_cast<I>(g.batch) * period * out_frames * out_h * row_chunks;
    const I stride = static_cast<I>(gridDim.x) * blockDim.x;
    const int64_t plane_chunks = g.frames * g.height * (g.width / EPC);                    // one input channel
    const int64_t out_channel_chunks = static_cast<int64_t>(out_frames) * out_h * row_chunks * 2;
    for (I i = static_cast<I>(blockIdx.x) * blockDim.x + threadIdx.x; i < total; i += stride) {
        const I row = i / row_chunks, k = i - row * row_chunks;
        I r = row;
        const I oh = r % out_h; r /= out_h;
        const I frame = r % out_frames; r /= out_frames;
        const I cr = r % period, b = r / period;
        const I ot = frame + 1, ih = oh >> 1, ph = oh & 1, it = ot >> 1, pt = ot & 1;
        const int64_t sub = static_cast<int64_t>(pt * 2 + ph) * 2;                         // + pw
        const int64_t at = (static_cast<int64_t>(it) * g.height + ih) * row_chunks + k;
        const uint4* res = x + ((static_cast<int64_t>(b) * period + cr) * 8 + sub) * plane_chunks + at;
        const uint4 w0 = __ldcs(res), w1 = __ldcs(res + plane_chunks);
        uint4 v[REPS][2];
#pragma unroll
        for (int rep = 0; rep < REPS; ++rep) {
            const int64_t c = static_cast<int64_t>(rep) * period + cr;
            const uint4* src = y + ((static_cast<int64_t>(b) * g.channels + c) * 8 + sub) * plane_chunks + at;
            v[rep][0] = __ldcs(src);
            v[rep][1] = __ldcs(src + plane_chunks);
        }
#pragma unroll
        for (int rep = 0; rep < REPS; ++rep) {
            const int64_t c = static_cast<int64_t>(rep) * period + cr;
            uint4 lo, hi;
            interleave<ELEM>(add_chunks(v[rep][0], w0, ELEM == 2), add_chunks(v[rep][1], w1, ELEM == 2), lo, hi);
            uint4* dst = out + (static_cast<int64_t>(b) * g.channels + c) * out_channel_chunks +
                         ((static_cast<int64_t>(frame) * out_h + oh) * row_chunks + k) * 2;
            store32(dst, lo, hi);
        }
    }
}

int run(const void* y, const void* x, void* out, int dtype, const ShuffleGeom& g, bool residual, cudaStream_t s,
        const char* what) {
    const int elem = dtype == VRB_BF16 ? 2 : 4;
    const int epc = 16 / elem;
    const int64_t out_frames = g.frames * g.ft - g.skip_frames;
    const int64_t total = g.batch * g.channels * out_frames * g.height * g.fh * g.width * g.fw;
    const bool rows_ok = (g.fw == 1 || g.fw == 2) && g.width % epc == 0 && aligned16(y) && aligned16(out) && (!residual || aligned16(x));
    if (rows_ok && residual) {
        const int64_t items = total / (epc * g.fw) / 4;   // four output channels per work item
        const int grid = grid_for((items + kThreads - 1) / kThreads, kPerSm);
        const bool narrow = items + static_cast<int64_t>(grid) * kThreads < (int64_t{1} << 32);   // i += stride cannot wrap
        const uint4 *yy = static_cast<const uint4*>(y), *xx = static_cast<const uint4*>(x);
        uint4* oo = static_cast<uint4*>(out);
        if (elem == 2) {
            if (narrow) depth_to_space_rows_kernel<2, unsigned><<<grid, kThreads, 0, s>>>(yy, xx, oo, g);
            else depth_to_space_rows_kernel<2, int64_t><<<grid, kThreads, 0, s>>>(yy, xx, oo, g);
        } else {
            if (narrow) depth_to_space_rows_kernel<4, unsigned><<<grid, kThreads, 0, s>>>(yy, xx, oo, g);
            else depth_to_space_rows_kernel<4, int64_t><<<grid, kThreads, 0, s>>>(yy, xx, oo, g);
        }
    } else if (rows_ok) {
        const int64_t items = total / (epc * g.fw);
        const int grid = grid_for((items + kThreads - 1) / kThreads, kPerSm);
        const bool narrow = items + 2 * static_cast<int64_t>(grid) * kThreads < (int64_t{1} << 32);   // i0 += 2 * stride cannot wrap
#define VRB_SH(E, F, R)                                                                                               \
    do {                                                                                                              \
        if (narrow) shuffle_rows_kernel<E, F, R, unsigned><<<grid, kThreads, 0, s>>>(                                  \
            static_cast<const uint4*>(y), static_cast<const uint4*>(x), static_cast<uint4*>(out), g);                  \
        else shuffle_rows_kernel<E, F, R, int64_t><<<grid, kThreads, 0, s>>>(                                          \
            static_cast<const uint4*>(y), static_cast<const uint4*>(x), static_cast<uint4*>(out), g);                  \
    } while (0)
        if (elem == 2) {
            if (g.fw == 2) { if (residual) VRB_SH(2, 2, true); else VRB_SH(2, 2, false); }
            else { if (residual) VRB_SH(2, 1, true); else VRB_SH(2, 1, false); }
        } else {
            if (g.fw == 2) { if (residual) VRB_SH(4, 2, true); else VRB_SH(4, 2, false); }
            else { if (residual) VRB_SH(4, 1, true); else VRB_SH(4, 1, false); }
        }
#undef VRB_SH
    } else {
        const int grid = grid_for((total + kThreads - 1) / kThreads, kPerSm);
        if (elem == 2) {
            if (residual) shuffle_scalar_kernel<uint16_t, true><<<grid, kThreads, 0, s>>>(static_cast<const uint16_t*>(y), static_cast<const uint16_t*>(x), static_cast<uint16_t*>(out), g);
            else shuffle_scalar_kernel<uint16_t, false><<<grid, kThreads, 0, s>>>(static_cast<const uint16_t*>(y), nullptr, static_cast<uint16_t*>(out), g);
        } else {
            if (residual) shuffle_scalar_kernel<float, true><<<grid, kThreads, 0, s>>>(static_cast<const float*>(y), static_cast<const float*>(x), static_cast<float*>(out), g);
            else shuffle_scalar_kernel<float, false><<<grid, kThreads, 0, s>>>(static_cast<const float*>(y), nullptr, static_cast<float*>(out), g);
        }
    }
    return after_launch(what);
}

}  // namespace
}  // namespace vrb

using namespace vrb;

extern "C" int vrb_pixel_shuffle(const void* x, void* out, int dtype, int64_t batch, int64_t channels, int64_t frames,
                                 int64_t height, int64_t width, int factor_t, int factor_h, int factor_w, vrb_stream stream) {
    VRB_REQUIRE(x && out, VRB_ERR_INVALID, "pixel_shuffle: null tensor");
    VRB_REQUIRE(batch > 0 && channels > 0 && frames > 0 && height > 0 && width > 0 && factor_t > 0 && factor_h > 0 && factor_w > 0,
                VRB_ERR_INVALID, "pixel_shuffle: extents and factors must be positive");
    VRB_REQUIRE(is_float_dtype(dtype), VRB_ERR_UNSUPPORTED, "pixel_shuffle: dtype must be F32 or BF16");
    ShuffleGeom g{batch, channels, frames, height, width, factor_t, factor_h, factor_w, 0, 1};
    return run(x, nullptr, out, dtype, g, false, as_stream(stream), "pixel_shuffle");
}

extern "C" int vrb_depth_to_space_residual(const void* projected, const void* input, void* out, int dtype, int64_t batch,
                                           int64_t input_channels, int64_t frames, int64_t height, int64_t width,
                                           vrb_stream stream) {
    VRB_REQUIRE(projected && input && out, VRB_ERR_INVALID, "depth_to_space_residual: null tensor");
    VRB_REQUIRE(batch > 0 && input_channels > 0 && frames > 0 && height > 0 && width > 0, VRB_ERR_INVALID,
                "depth_to_space_residual: extents must be positive");
    VRB_REQUIRE(input_channels % 8 == 0, VRB_ERR_INVALID, "pixel shuffle channel mismatch");
    VRB_REQUIRE(is_float_dtype(dtype), VRB_ERR_UNSUPPORTED, "depth_to_space_residual: dtype must be F32 or BF16");
    ShuffleGeom g{batch, input_channels / 2, frames, height, width, 2, 2, 2, 1, static_cast<int>(input_channels / 8)};
    return run(projected, input, out, dtype, g, true, as_stream(stream), "depth_to_space_residual");
}
