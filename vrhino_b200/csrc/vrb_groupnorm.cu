// GroupNorm (+SiLU) and channel-axis RMSNorm (+SiLU) for the VAE feature maps.
//
// GroupNorm reference: native/src/backend/cuda/cuda_backend.cu:1884-2030 (kernels) and
// :4919-5008 (host).  The reference reads x three times (shifted mean, centred variance,
// normalise) plus a separate SiLU kernel.  Here x is read twice and written once:
//   1. gn_partial_kernel   every CTA reduces one slice of one (batch, group) unit to the
//                          shifted sums S1 = sum(x - a), S2 = sum((x - a)^2) with
//                          a = the unit's first element (the reference's anchor); F32 inside a
//                          128-bit vector, double across vectors
//   2. gn_finalize_kernel  adds the slices of a unit in slice order (deterministic),
//                          mean = a + S1/n, var = S2/n - (S1/n)^2, inv = rsqrtf(var + eps)
//   3. gn_apply_kernel     y = fma((x - mean) * inv, gamma, beta) rounded to x's dtype, then
//                          optionally SiLU of that rounded value, rounded again
// The shifted one-pass variance in double agrees with the reference's centred two-pass F32
// variance to F32 rounding.  The three pieces are also exported separately so a tensor that is
// split along its spatial axis over several GPUs can add the per-slice sums between 1 and 2.
//
// Axis RMSNorm reference: rms_norm_axis_parallel_kernel :1045-1095.
#include <mutex>

#include "vrb_common.cuh"

namespace vrb {
namespace {

constexpr int kThreads = 256;
constexpr int kMaxSplits = 64;

// frames == 1: x is [batch, channels, spatial] and a unit (batch entry, group) is one contiguous
// run of channels_per * spatial elements.  frames > 1: x is [batch, channels, frames, spatial] and a
// unit is (batch entry, frame, group): channels_per separate runs of `spatial` elements, which is
// what the reference reaches by permuting to [batch*frames, channels, spatial] first
// (frame_group_norm, native/src/architectures/mochi.cpp:365-371).
struct GnGeom {
    int64_t batch, channels, spatial, count, units, frames;
    int64_t stat_frames;   // == frames; 1 when planes are split by frame but the statistics span all frames
    int groups, channels_per;
};
// First element of run `j` (channel j of the group) of unit `unit`.
__device__ __forceinline__ int64_t run_base(const GnGeom& g, int64_t unit, int j) {
    if (g.frames == 1) return unit * g.count + static_cast<int64_t>(j) * g.spatial;
    const int64_t group = unit % g.groups, bt = unit / g.groups, t = bt % g.frames, b = bt / g.frames;
    return (((b * g.channels + group * g.channels_per + j) * g.frames) + t) * g.spatial;
}

// Slices per unit: enough CTAs to fill the machine several times over, at least 16 K elements
// per slice so the per-CTA reduction stays negligible.
int choose_splits(int64_t units, int64_t count) {
    const int64_t want = (static_cast<int64_t>(sm_count()) * 8 + units - 1) / units;
    int64_t by_size = count / 16384;
    if (by_size < 1) by_size = 1;
    int64_t s = want < by_size ? want : by_size;
    if (s > kMaxSplits) s = kMaxSplits;
    if (s < 1) s = 1;
    return static_cast<int>(s);
}

__device__ __forceinline__ void block_reduce2(double& a, double& b, double (*ws)[8]) {
    for (int offset = 16; offset > 0; offset >>= 1) {
        a += __shfl_xor_sync(0xffffffffu, a, offset);
        b += __shfl_xor_sync(0xffffffffu, b, offset);
    }
    if ((threadIdx.x & 31) == 0) { ws[0][threadIdx.x >> 5] = a; ws[1][threadIdx.x >> 5] = b; }
    __syncthreads();
    a = 0.0; b = 0.0;
    for (int w = 0; w < kThreads / 32; ++w) { a += ws[0][w]; b += ws[1][w]; }
}

// partial[(unit * splits + split) * 2 + {0,1}] = {S1, S2} over the slice; element-wise form for
// units whose size or alignment rules out 16-byte loads.
__global__ void __launch_bounds__(kThreads) gn_partial_kernel(const void* x, int dt, const float* shift,
                                                             double* partial, int64_t count, int splits) {
    __shared__ double ws[2][8];
    const int64_t unit = blockIdx.x / splits;
    const int split = blockIdx.x % splits;
    const int64_t base = unit * count;
    const float a = shift ? shift[unit] : load1(x, dt, base);
    double s1 = 0.0, s2 = 0.0;
    const int64_t begin = count * split / splits, end = count * (split + 1) / splits;
    for (int64_t i = begin + threadIdx.x; i < end; i += kThreads) {
        const double d = static_cast<double>(__fsub_rn(load1(x, dt, base + i), a));
        s1 += d;
        s2 = fma(d, d, s2);
    }
    block_reduce2(s1, s2, ws);
    if (threadIdx.x == 0) {
        partial[(unit * splits + split) * 2] = s1;
        partial[(unit * splits + split) * 2 + 1] = s2;
    }
}

// The vector form of the moments pass, software-pipelined: the 16-byte loads of the next
// iteration are issued before the current registers are consumed, so every warp always has U
// loads in flight; x stays packed in registers until it is used.  BF16: U = 4 chunks of 8
// elements per thread and iteration; F32: U = 2 chunks (two 16-byte loads each).
template <bool X_BF16>
struct Packed8 {
    uint4 lo, hi;   // BF16 uses lo only
};
template <bool X_BF16>
__device__ __forceinline__ Packed8<X_BF16> load_packed8(const void* x, int64_t element) {
    Packed8<X_BF16> r;
    if constexpr (X_BF16) {
        r.lo = __ldcs(reinterpret_cast<const uint4*>(static_cast<const uint16_t*>(x) + element));
    } else {
        const uint4* p = reinterpret_cast<const uint4*>(static_cast<const float*>(x) + element);
        r.lo = __ldcs(p);
        r.hi = __ldcs(p + 1);
    }
    return r;
}
template <bool X_BF16>
__device__ __forceinline__ void accumulate_packed8(const Packed8<X_BF16>& r, float a, double& s1, double& s2) {
    float v[8];
    if constexpr (X_BF16) {
        v[0] = __uint_as_float(r.lo.x << 16); v[1] = __uint_as_float(r.lo.x & 0xffff0000u);
        v[2] = __uint_as_float(r.lo.y << 16); v[3] = __uint_as_float(r.lo.y & 0xffff0000u);
        v[4] = __uint_as_float(r.lo.z << 16); v[5] = __uint_as_float(r.lo.z & 0xffff0000u);
        v[6] = __uint_as_float(r.lo.w << 16); v[7] = __uint_as_float(r.lo.w & 0xffff0000u);
    } else {
        v[0] = __uint_as_float(r.lo.x); v[1] = __uint_as_float(r.lo.y); v[2] = __uint_as_float(r.lo.z); v[3] = __uint_as_float(r.lo.w);
        v[4] = __uint_as_float(r.hi.x); v[5] = __uint_as_float(r.hi.y); v[6] = __uint_as_float(r.hi.z); v[7] = __uint_as_float(r.hi.w);
    }
    // two independent 4-long chains per sum instead of one 8-long chain
    float t1a = 0.0f, t1b = 0.0f, t2a = 0.0f, t2b = 0.0f;
#pragma unroll
    for (int e = 0; e < 4; ++e) {
        const float da = __fsub_rn(v[e], a), db = __fsub_rn(v[e + 4], a);
        t1a = __fadd_rn(t1a, da); t1b = __fadd_rn(t1b, db);
        t2a = __fmaf_rn(da, da, t2a); t2b = __fmaf_rn(db, db, t2b);
    }
    s1 += static_cast<double>(__fadd_rn(t1a, t1b));
    s2 += static_cast<double>(__fadd_rn(t2a, t2b));
}

// frames == 1: the unit's `count` elements are cut into `splits` slices.  frames > 1: the unit's
// channels_per runs are cut into splits / channels_per slices each, run-major, so the partials of
// a unit are again combined in element order.
template <bool X_BF16>
__global__ void __launch_bounds__(kThreads, 4) gn_partial_vec_kernel(const void* __restrict__ x, const float* __restrict__ shift,
                                                                    double* __restrict__ partial, GnGeom g, int splits) {
    __shared__ double ws[2][8];
    constexpr int U = X_BF16 ? 4 : 2;
    const int64_t unit = blockIdx.x / splits;
    const int split = blockIdx.x % splits;
    const float a = shift ? shift[unit] : load1(x, X_BF16 ? VRB_BF16 : VRB_F32, run_base(g, unit, 0));
    int64_t base, begin, end;
    if (g.frames == 1) {
        const int64_t chunks = g.count >> 3;
        base = unit * g.count;
        begin = chunks * split / splits;
        end = chunks * (split + 1) / splits;
    } else {
        const int per_run = splits / g.channels_per, j = split / per_run, part = split - j * per_run;
        const int64_t chunks = g.spatial >> 3;
        base = run_base(g, unit, j);
        begin = chunks * part / per_run;
        end = chunks * (part + 1) / per_run;
    }
    double s1 = 0.0, s2 = 0.0;
    Packed8<X_BF16> cur[U], nxt[U];
    int64_t c0 = begin + threadIdx.x;
#pragma unroll
    for (int u = 0; u < U; ++u)
        if (c0 + u * kThreads < end) cur[u] = load_packed8<X_BF16>(x, base + (c0 + u * kThreads) * 8);
    while (c0 < end) {
        const int64_t c1 = c0 + kThreads * U;
#pragma unroll
        for (int u = 0; u < U; ++u)
            if (c1 + u * kThreads < end) nxt[u] = load_packed8<X_BF16>(x, base + (c1 + u * kThreads) * 8);
#pragma unroll
        for (int u = 0; u < U; ++u)
            if (c0 + u * kThreads < end) accumulate_packed8<X_BF16>(cur[u], a, s1, s2);
#pragma unroll
        for (int u = 0; u < U; ++u) cur[u] = nxt[u];
        c0 = c1;
    }
    block_reduce2(s1, s2, ws);
    if (threadIdx.x == 0) {
        partial[(unit * splits + split) * 2] = s1;
        partial[(unit * splits + split) * 2 + 1] = s2;
    }
}

// moments[unit*3 + {0,1,2}] = {n, S1, S2}: slices added in slice order.
__global__ void gn_collect_kernel(const double* partial, double* moments, int64_t units, int splits, int64_t count) {
    const int64_t unit = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
    if (unit >= units) return;
    double s1 = 0.0, s2 = 0.0;
    for (int s = 0; s < splits; ++s) { s1 += partial[(unit * splits + s) * 2]; s2 += partial[(unit * splits + s) * 2 + 1]; }
    moments[unit * 3] = static_cast<double>(count);
    moments[unit * 3 + 1] = s1;
    moments[unit * 3 + 2] = s2;
}

__global__ void gn_finalize_kernel(const double* moments, const float* shift, const void* x, int dt, GnGeom g,
                                   int64_t units, float eps, float* mean, float* inverse) {
    const int64_t unit = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x;
    if (unit >= units) return;
    const double a = shift ? static_cast<double>(shift[unit]) : static_cast<double>(load1(x, dt, run_base(g, unit, 0)));
    const double n = moments[unit * 3], m1 = moments[unit * 3 + 1] / n;
    double var = moments[unit * 3 + 2] / n - m1 * m1;
    if (var < 0.0) var = 0.0;
    mean[unit] = static_cast<float>(a + m1);
    inverse[unit] = rsqrtf(__fadd_rn(static_cast<float>(var), eps));
}

// Slice sums -> mean / inverse in one launch for the whole-operator path: one warp per unit, lane
// l adds slices l and l + 32 (at most 64 slices), then a fixed shuffle tree; lane 0 applies the
// formulas of gn_finalize_kernel.  The order of additions depends only on the slice count.
__global__ void __launch_bounds__(128) gn_collect_finalize_kernel(const double* __restrict__ partial, const void* x, int dt,
                                                                  GnGeom g, int splits, float eps, float* mean, float* inverse) {
    const int64_t unit = (static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x) >> 5;
    const int lane = threadIdx.x & 31;
    if (unit >= g.units) return;
    double s1 = 0.0, s2 = 0.0;
    for (int s = lane; s < splits; s += 32) {
        s1 += partial[(unit * splits + s) * 2];
        s2 += partial[(unit * splits + s) * 2 + 1];
    }
    for (int offset = 16; offset > 0; offset >>= 1) {
        s1 += __shfl_xor_sync(0xffffffffu, s1, offset);
        s2 += __shfl_xor_sync(0xffffffffu, s2, offset);
    }
    if (lane == 0) {
        const double a = static_cast<double>(load1(x, dt, run_base(g, unit, 0)));
        const double n = static_cast<double>(g.count), m1 = s1 / n;
        double var = s2 / n - m1 * m1;
        if (var < 0.0) var = 0.0;
        mean[unit] = static_cast<float>(a + m1);
        inverse[unit] = rsqrtf(__fadd_rn(static_cast<float>(var), eps));
    }
}

__device__ __forceinline__ float gn_value(float x, float mean, float inv, float gamma, float beta, int dt, int silu) {
    float y = round_to(dt, __fmaf_rn(__fmul_rn(__fsub_rn(x, mean), inv), gamma, beta));
    if (silu) y = activation_value(VRB_SILU, y);
    return y;
}

// Per-plane constants of the normalise pass.  gamma / beta are converted to x's dtype first (:4929).
struct PlaneTerms {
    float mean, inv, gamma, beta;
};
__device__ __forceinline__ PlaneTerms plane_terms(int64_t plane, const GnGeom& g, int dt, const void* weight, int w_dt,
                                                  const void* bias, int b_dt, const float* mean, const float* inverse) {
    // plane = (batch entry, channel, frame); frames == 1 for the contiguous form
    int64_t frame = 0, bc = plane;
    if (g.frames > 1) { bc = plane / g.frames; frame = plane - bc * g.frames; }
    const int64_t channel = bc % g.channels;
    const int64_t unit = (g.stat_frames > 1 ? (bc / g.channels) * g.frames + frame : bc / g.channels) * g.groups +
                         channel / g.channels_per;
    PlaneTerms t;
    t.mean = __ldg(mean + unit);
    t.inv = __ldg(inverse + unit);
    t.gamma = weight ? round_to(dt, load1(weight, w_dt, channel)) : 1.0f;
    t.beta = bias ? round_to(dt, load1(bias, b_dt, channel)) : 0.0f;
    return t;
}

// Normalise pass, vector form.  Every plane (one channel of one batch entry) is cut into
// tiles_per_plane equal tiles of at most kThreads * U chunks, so mean / inverse / gamma / beta are
// looked up once per tile, the inner loop has no index arithmetic beyond an add, and no tile is
// much emptier than the others.
template <bool X_BF16, bool SILU>
__global__ void __launch_bounds__(kThreads, 4) gn_apply_vec_kernel(const void* __restrict__ x, const void* weight, int w_dt,
                                                                  const void* bias, int b_dt, void* __restrict__ out, GnGeom g,
                                                                  const float* mean, const float* inverse,
                                                                  int64_t tiles_per_plane, int64_t tile_chunks, GnScatter scatter) {
    constexpr int U = 4;
    constexpr int dt = X_BF16 ? VRB_BF16 : VRB_F32;
    const int64_t plane_chunks = g.spatial >> 3;
    const int64_t tiles = g.batch * g.channels * g.frames * tiles_per_plane;
    for (int64_t t = blockIdx.x; t < tiles; t += gridDim.x) {
        const int64_t plane = t / tiles_per_plane;
        const int64_t tile_begin = (t - plane * tiles_per_plane) * tile_chunks;
        const int64_t tile_end = tile_begin + tile_chunks < plane_chunks ? tile_begin + tile_chunks : plane_chunks;
        const int64_t c0 = tile_begin + threadIdx.x;
        const PlaneTerms k = plane_terms(plane, g, dt, weight, w_dt, bias, b_dt, mean, inverse);
        const int64_t e_plane = plane * g.spatial;
        float v[U][8];
#pragma unroll
        for (int u = 0; u < U; ++u)
            if (c0 + u * kThreads < tile_end) load8<true>(x, dt, e_plane + (c0 + u * kThreads) * 8, v[u]);
#pragma unroll
        for (int u = 0; u < U; ++u) {
            if (c0 + u * kThreads >= tile_end) break;
#pragma unroll
            for (int e = 0; e < 8; ++e) v[u][e] = gn_value(v[u][e], k.mean, k.inv, k.gamma, k.beta, dt, SILU ? 1 : 0);
            if (scatter.count == 0) {
                store8(out, dt, e_plane + (c0 + u * kThreads) * 8, v[u]);
            } else {
                const int64_t at = plane * scatter.plane_stride + scatter.plane_offset + (c0 + u * kThreads) * 8;
                for (int d = 0; d < scatter.count; ++d) store8(scatter.dst[d], dt, at, v[u]);
            }
        }
    }
}

__global__ void __launch_bounds__(kThreads) gn_apply_kernel(const void* x, int dt, const void* weight, int w_dt,
                                                           const void* bias, int b_dt, void* out, GnGeom g,
                                                           const float* mean, const float* inverse, int silu) {
    const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
    const int64_t total = g.units * g.count;
    for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < total; i += stride) {
        const PlaneTerms k = plane_terms(i / g.spatial, g, dt, weight, w_dt, bias, b_dt, mean, inverse);   // plane-major order
        store1(out, dt, i, gn_value(load1(x, dt, i), k.mean, k.inv, k.gamma, k.beta, dt, silu));
    }
}

int make_geom(GnGeom& g, int64_t batch, int64_t channels, int64_t spatial, int groups, const char* what, int64_t frames = 1) {
    VRB_REQUIRE(batch > 0 && channels > 0 && spatial > 0 && groups > 0 && channels % groups == 0 && frames > 0, VRB_ERR_INVALID,
                "%s: group norm shape/groups mismatch", what);
    g.batch = batch; g.channels = channels; g.spatial = spatial; g.groups = groups; g.frames = frames; g.stat_frames = frames;
    g.channels_per = static_cast<int>(channels / groups);
    g.count = g.channels_per * spatial;
    g.units = batch * frames * groups;
    VRB_REQUIRE(g.units * kMaxSplits <= 0x7fffffffLL, VRB_ERR_INVALID,
                "%s: group norm launch extent exceeds CUDA grid capacity", what);
    return VRB_OK;
}

size_t workspace_layout(int64_t units, size_t* moments_off, size_t* mean_off) {
    size_t partial_bytes = static_cast<size_t>(units) * kMaxSplits * 2 * sizeof(double);
    size_t moments_bytes = static_cast<size_t>(units) * 3 * sizeof(double);
    size_t stats_bytes = static_cast<size_t>(units) * 2 * sizeof(float);
    auto up = [](size_t v) { return (v + 255) & ~static_cast<size_t>(255); };
    if (moments_off) *moments_off = up(partial_bytes);
    if (mean_off) *mean_off = up(partial_bytes) + up(moments_bytes);
    return up(partial_bytes) + up(moments_bytes) + up(stats_bytes);
}

int run_moments(const void* x, int dt, const GnGeom& g, const float* shift, double* partial, double* moments,
                cudaStream_t s, int* splits_out = nullptr) {
    int splits = choose_splits(g.units, g.count);
    const bool vec = (g.frames == 1 ? g.count : g.spatial) % 8 == 0 && aligned16(x);
    if (g.frames > 1) {
        // per-frame form: whole runs per slice, vector kernel only
        VRB_REQUIRE(vec && g.channels_per <= kMaxSplits, VRB_ERR_UNSUPPORTED,
                    "group_norm_frames: needs spatial %% 8 == 0, 16-byte aligned x and at most %d channels per group", kMaxSplits);
        int per_run = splits / g.channels_per;
        if (per_run < 1) per_run = 1;
        splits = per_run * g.channels_per;
    }
    const int grid = static_cast<int>(g.units * splits);
    if (vec && dt == VRB_BF16) gn_partial_vec_kernel<true><<<grid, kThreads, 0, s>>>(x, shift, partial, g, splits);
    else if (vec) gn_partial_vec_kernel<false><<<grid, kThreads, 0, s>>>(x, shift, partial, g, splits);
    else gn_partial_kernel<<<grid, kThreads, 0, s>>>(x, dt, shift, partial, g.count, splits);
    if (int rc = after_launch("group_norm moments")) return rc;
    if (splits_out) { *splits_out = splits; return VRB_OK; }   // the caller combines the slices itself
    gn_collect_kernel<<<static_cast<int>((g.units + 127) / 128), 128, 0, s>>>(partial, moments, g.units, splits, g.count);
    return after_launch("group_norm collect");
}

int run_apply(const void* x, int dt, const void* weight, int w_dt, const void* bias, int b_dt, void* out,
              const GnGeom& g, const float* mean, const float* inverse, int silu, cudaStream_t s,
              const GnScatter& scatter = GnScatter{}) {
    const bool vec = g.spatial % 8 == 0 && aligned16(x) && aligned16(out);
    const int64_t total = g.units * g.count;
    if (vec) {
        if (dt == VRB_BF16 && silu && total >= kLutMinElements && total / 8 < (int64_t{1} << 31))   // SiLU of a bf16 value: table lookup
            return launch_group_norm_apply_silu_lut(x, weight, w_dt, bias, b_dt, out, g.batch * g.channels * g.frames, g.channels,
                                                    g.channels_per, g.groups, g.frames, g.stat_frames, g.spatial, mean, inverse,
                                                    scatter, s);
        const int64_t plane_chunks = g.spatial / 8;
        const int64_t tiles_per_plane = (plane_chunks + kThreads * 4 - 1) / (kThreads * 4);
        const int64_t tile_chunks = ((plane_chunks + tiles_per_plane - 1) / tiles_per_plane + 7) & ~int64_t{7};   // tiles start on 128-byte lines
        const int grid = grid_for(g.batch * g.channels * g.frames * tiles_per_plane, 4);
#define VRB_GN_APPLY(BF, SI) gn_apply_vec_kernel<BF, SI><<<grid, kThreads, 0, s>>>( \
            x, weight, w_dt, bias, b_dt, out, g, mean, inverse, tiles_per_plane, tile_chunks, scatter)
        if (dt == VRB_BF16) { if (silu) VRB_GN_APPLY(true, true); else VRB_GN_APPLY(true, false); }
        else { if (silu) VRB_GN_APPLY(false, true); else VRB_GN_APPLY(false, false); }
#undef VRB_GN_APPLY
    } else {
        VRB_REQUIRE(scatter.count == 0, VRB_ERR_UNSUPPORTED,
                    "group_norm_apply_scatter: needs a local plane size that is a multiple of 8 and 16-byte aligned tensors");
        gn_apply_kernel<<<grid_for((total + kThreads - 1) / kThreads, 8), kThreads, 0, s>>>(
            x, dt, weight, w_dt, bias, b_dt, out, g, mean, inverse, silu);
    }
    return after_launch("group_norm apply");
}

// ---- RMSNorm over an inner axis: x [outer, axis, inner] ------------------------------------
// Pass 1 accumulates sum of squares over the axis in double per inner position, pass 2
// normalises; a thread owns 8 consecutive inner positions (VEC) or one.
template <bool VEC>
__global__ void __launch_bounds__(kThreads) rms_axis_kernel(const void* x, int dt, const void* weight, int w_dt,
                                                           void* out, int64_t outer, int64_t axis, int64_t inner,
                                                           float eps, int silu) {
    constexpr int W = VEC ? 8 : 1;
    const int64_t inner_items = VEC ? inner >> 3 : inner;
    const int64_t items = outer * inner_items;
    const int64_t stride = static_cast<int64_t>(gridDim.x) * blockDim.x;
    for (int64_t i = static_cast<int64_t>(blockIdx.x) * blockDim.x + threadIdx.x; i < items; i += stride) {
        const int64_t o = i / inner_items, p = (i - o * inner_items) * W;
        const int64_t base = o * axis * inner + p;
        double sq[W];
#pragma unroll
        for (int e = 0; e < W; ++e) sq[e] = 0.0;
        for (int64_t c = 0; c < axis; ++c) {
            float v[8];
            if constexpr (VEC) load8<false>(x, dt, base + c * inner, v);
            else v[0] = load1(x, dt, base + c * inner);
#pragma unroll
            for (int e = 0; e < W; ++e) sq[e] = fma(static_cast<double>(v[e]), static_cast<double>(v[e]), sq[e]);
        }
        float inv[W];
#pragma unroll
        for (int e = 0; e < W; ++e) inv[e] = rsqrtf(__fadd_rn(static_cast<float>(sq[e] / static_cast<double>(axis)), eps));
        for (int64_t c = 0; c < axis; ++c) {
            float v[8];
            if constexpr (VEC) load8<false>(x, dt, base + c * inner, v);
            else v[0] = load1(x, dt, base + c * inner);
            const float w = weight ? round_to(dt, load1(weight, w_dt, c)) : 1.0f;
#pragma unroll
            for (int e = 0; e < W; ++e) {
                float y = __fmul_rn(v[e], inv[e]);
                if (dt == VRB_BF16) y = round_to_bf16(y);
                if (weight) y = __fmul_rn(y, w);
                y = round_to(dt, y);
                if (silu) y = activation_value(VRB_SILU, y);
                v[e] = y;
            }
            if constexpr (VEC) store8(out, dt, base + c * inner, v);
            else store1(out, dt, base + c * inner, v[0]);
        }
    }
}

}  // namespace
}  // namespace vrb

using namespace vrb;

extern "C" size_t vrb_group_norm_workspace_bytes(int64_t batch, int groups) {
    if (batch <= 0 || groups <= 0) return 0;
    return workspace_layout(batch * groups, nullptr, nullptr);
}

namespace {
int group_norm_whole(const GnGeom& g, const void* x, int dtype, const void* weight, int weight_dtype,
                     const void* bias, int bias_dtype, void* out, float eps, int fuse_silu, void* workspace,
                     size_t workspace_bytes, vrb_stream stream) {
    size_t moments_off, mean_off;
    const size_t need = workspace_layout(g.units, &moments_off, &mean_off);
    VRB_REQUIRE(workspace && workspace_bytes >= need && (reinterpret_cast<uintptr_t>(workspace) & 255u) == 0,
                VRB_ERR_WORKSPACE, "group_norm: workspace needs %zu bytes, 256-byte aligned", need);
    char* ws = static_cast<char*>(workspace);
    double* partial = reinterpret_cast<double*>(ws);
    double* moments = reinterpret_cast<double*>(ws + moments_off);
    float* mean = reinterpret_cast<float*>(ws + mean_off);
    float* inverse = mean + g.units;
    cudaStream_t s = as_stream(stream);
    int splits = 0;
    if (int rc = run_moments(x, dtype, g, nullptr, partial, moments, s, &splits)) return rc;
    gn_collect_finalize_kernel<<<static_cast<int>((g.units * 32 + 127) / 128), 128, 0, s>>>(partial, x, dtype, g, splits, eps,
                                                                                         mean, inverse);
    if (int rc = after_launch("group_norm finalize")) return rc;
    return run_apply(x, dtype, weight, weight_dtype, bias, bias_dtype, out, g, mean, inverse, fuse_silu, s);
}
}  // namespace

extern "C" int vrb_group_norm(const void* x, int dtype, const void* weight, int weight_dtype,
                              const void* bias, int bias_dtype, void* out,
                              int64_t batch, int64_t channels, int64_t spatial, int groups, float eps,
                              int fuse_silu, void* workspace, size_t workspace_bytes, vrb_stream stream) {
    VRB_REQUIRE(x && out, VRB_ERR_INVALID, "group_norm: null tensor");
    VRB_REQUIRE(is_float_dtype(dtype), VRB_ERR_UNSUPPORTED, "group_norm: dtype must be F32 or BF16");
    GnGeom g;
    if (int rc = make_geom(g, batch, channels, spatial, groups, "group_norm")) return rc;
    return group_norm_whole(g, x, dtype, weight, weight_dtype, bias, bias_dtype, out, eps, fuse_silu, workspace,
                            workspace_bytes, stream);
}

extern "C" size_t vrb_group_norm_frames_workspace_bytes(int64_t batch, int64_t frames, int groups) {
    if (batch <= 0 || frames <= 0 || groups <= 0) return 0;
    return workspace_layout(batch * frames * groups, nullptr, nullptr);
}

extern "C" int vrb_group_norm_frames(const void* x, int dtype, const void* weight, int weight_dtype,
                                     const void* bias, int bias_dtype, void* out,
                                     int64_t batch, int64_t channels, int64_t frames, int64_t spatial, int groups,
                                     float eps, int fuse_silu, void* workspace, size_t workspace_bytes, vrb_stream stream) {
    VRB_REQUIRE(x && out, VRB_ERR_INVALID, "group_norm_frames: null tensor");
    VRB_REQUIRE(is_float_dtype(dtype), VRB_ERR_UNSUPPORTED, "group_norm_frames: dtype must be F32 or BF16");
    GnGeom g;
    if (int rc = make_geom(g, batch, channels, spatial, groups, "group_norm_frames", frames)) return rc;
    VRB_REQUIRE(aligned16(out), VRB_ERR_UNSUPPORTED, "group_norm_frames: out must be 16-byte aligned");
    return group_norm_whole(g, x, dtype, weight, weight_dtype, bias, bias_dtype, out, eps, fuse_silu, workspace,
                            workspace_bytes, stream);
}

// ---- GroupNorm with built-in scratch ----------------------------------------------------------
// vrb_group_norm wants a caller-provided scratch buffer.  Some callers have no way to get one:
// a backend whose whole device budget has been handed to a planner-owned pool (nothing may be
// allocated while a step runs, and every byte is accounted for), or a host thread that must
// never enter cudaMalloc because that call synchronises the device.  For them the library
// carries a fixed scratch area of its own.  It is a plain global array in device memory, so
// every GPU that loads the library gives up kFixedScratchBytes (about 1 MiB) until the process
// exits, and it bounds the problem size: at most kFixedScratchUnits (batch x groups) units.
namespace {
constexpr int64_t kFixedScratchUnits = 1024;
constexpr size_t fixed_up(size_t v) { return (v + 255) & ~static_cast<size_t>(255); }
constexpr size_t kFixedScratchBytes =
    fixed_up(static_cast<size_t>(kFixedScratchUnits) * vrb::kMaxSplits * 2 * sizeof(double)) +
    fixed_up(static_cast<size_t>(kFixedScratchUnits) * 3 * sizeof(double)) +
    fixed_up(static_cast<size_t>(kFixedScratchUnits) * 2 * sizeof(float));

static __device__ __align__(256) unsigned char g_fixed_scratch[kFixedScratchBytes];

// In host code `g_fixed_scratch` is only a handle for the symbol, not an address a kernel can
// use; the device address has to be asked for, per device, with that device current.  It is kept
// per device index and is not asked for again, so it does not survive cudaDeviceReset.
std::mutex g_fixed_mutex;
void* g_fixed_address[64] = {nullptr};

int fixed_scratch_address(void** address) {
    int device = 0;
    const cudaError_t e0 = cudaGetDevice(&device);
    if (e0 != cudaSuccess || device < 0 || device >= 64) {
        vrb::set_error("group_norm_fixed_scratch: cannot identify the current device (%s)", cudaGetErrorString(e0));
        return VRB_ERR_CUDA;
    }
    std::lock_guard<std::mutex> lock(g_fixed_mutex);
    if (!g_fixed_address[device]) {
        void* p = nullptr;
        const cudaError_t e = cudaGetSymbolAddress(&p, g_fixed_scratch);
        if (e != cudaSuccess || !p) {
            vrb::set_error("CUDA error: %s (address of the built-in GroupNorm scratch)", cudaGetErrorString(e));
            return VRB_ERR_CUDA;
        }
        g_fixed_address[device] = p;
    }
    *address = g_fixed_address[device];
    return VRB_OK;
}
}  // namespace

static_assert(kFixedScratchUnits == VRB_GROUP_NORM_FIXED_SCRATCH_MAX_UNITS, "header and kernel file disagree on the limit");

extern "C" int vrb_group_norm_fixed_scratch(const void* x, int dtype, const void* weight, int weight_dtype,
                                            const void* bias, int bias_dtype, void* out,
                                            int64_t batch, int64_t channels, int64_t spatial, int groups, float eps,
                                            int fuse_silu, vrb_stream stream) {
    VRB_REQUIRE(batch > 0 && groups > 0, VRB_ERR_INVALID, "group_norm_fixed_scratch: group norm shape/groups mismatch");
    const int64_t units = batch * groups;
    VRB_REQUIRE(units <= kFixedScratchUnits, VRB_ERR_WORKSPACE,
                "group_norm_fixed_scratch: %lld (batch x groups) units exceed the built-in scratch, which holds %lld; "
                "use vrb_group_norm with a caller-provided workspace",
                static_cast<long long>(units), static_cast<long long>(kFixedScratchUnits));
    void* scratch = nullptr;
    if (int rc = fixed_scratch_address(&scratch)) return rc;
    // Nothing in the scratch has to start at zero: every slot this call reads (per-slice sums,
    // per-unit moments, mean / inverse) is written earlier in the same call, so whatever the
    // previous call left behind is simply overwritten.
    return vrb_group_norm(x, dtype, weight, weight_dtype, bias, bias_dtype, out, batch, channels, spatial, groups, eps,
                          fuse_silu, scratch, kFixedScratchBytes, stream);
}

extern "C" int vrb_group_norm_moments(const void* x, int dtype, int64_t batch, int64_t channels,
                                      int64_t spatial_local, int groups, const float* shift,
                                      double* moments, void* workspace, size_t workspace_bytes, vrb_stream stream) {
    VRB_REQUIRE(x && moments && shift, VRB_ERR_INVALID, "group_norm_moments: null tensor");
    VRB_REQUIRE(is_float_dtype(dtype), VRB_ERR_UNSUPPORTED, "group_norm_moments: dtype must be F32 or BF16");
    GnGeom g;
    if (int rc = make_geom(g, batch, channels, spatial_local, groups, "group_norm_moments")) return rc;
    // A spatial slice of a unit is not contiguous: channel c of the unit starts at
    // (unit*channels_per + c) * spatial_local, and those planes are adjacent, so the unit's
    // slice IS one contiguous run of channels_per * spatial_local elements.
    const size_t need = workspace_layout(g.units, nullptr, nullptr);
    VRB_REQUIRE(workspace && workspace_bytes >= need && (reinterpret_cast<uintptr_t>(workspace) & 255u) == 0,
                VRB_ERR_WORKSPACE, "group_norm_moments: workspace needs %zu bytes, 256-byte aligned", need);
    return run_moments(x, dtype, g, shift, static_cast<double*>(workspace), moments, as_stream(stream));
}

extern "C" int vrb_group_norm_finalize(const double* moments, const float* shift, int64_t units, float eps,
                                       float* mean, float* inverse, vrb_stream stream) {
    VRB_REQUIRE(moments && shift && mean && inverse && units > 0, VRB_ERR_INVALID, "group_norm_finalize: null tensor");
    gn_finalize_kernel<<<static_cast<int>((units + 127) / 128), 128, 0, as_stream(stream)>>>(
        moments, shift, nullptr, VRB_F32, GnGeom{}, units, eps, mean, inverse);
    return after_launch("group_norm finalize");
}

extern "C" int vrb_group_norm_apply(const void* x, int dtype, const void* weight, int weight_dtype,
                                    const void* bias, int bias_dtype, void* out,
                                    int64_t batch, int64_t channels, int64_t spatial_local, int groups,
                                    const float* mean, const float* inverse, int fuse_silu, vrb_stream stream) {
    VRB_REQUIRE(x && out && mean && inverse, VRB_ERR_INVALID, "group_norm_apply: null tensor");
    VRB_REQUIRE(is_float_dtype(dtype), VRB_ERR_UNSUPPORTED, "group_norm_apply: dtype must be F32 or BF16");
    GnGeom g;
    if (int rc = make_geom(g, batch, channels, spatial_local, groups, "group_norm_apply")) return rc;
    return run_apply(x, dtype, weight, weight_dtype, bias, bias_dtype, out, g, mean, inverse, fuse_silu, as_stream(stream));
}

extern "C" int vrb_group_norm_apply_scatter(const void* x, int dtype, const void* weight, int weight_dtype,
                                            const void* bias, int bias_dtype, void* const* destinations, int destination_count,
                                            int64_t batch, int64_t channels, int64_t frames, int64_t spatial_local,
                                            int64_t spatial_full, int64_t spatial_offset, int groups,
                                            const float* mean, const float* inverse, int fuse_silu, vrb_stream stream) {
    VRB_REQUIRE(x && destinations && mean && inverse, VRB_ERR_INVALID, "group_norm_apply_scatter: null tensor");
    VRB_REQUIRE(destination_count >= 1 && destination_count <= 8, VRB_ERR_INVALID,
                "group_norm_apply_scatter: 1 to 8 destinations");
    VRB_REQUIRE(is_float_dtype(dtype), VRB_ERR_UNSUPPORTED, "group_norm_apply_scatter: dtype must be F32 or BF16");
    VRB_REQUIRE(spatial_offset >= 0 && spatial_local > 0 && spatial_offset + spatial_local <= spatial_full &&
                    spatial_offset % 8 == 0 && spatial_full % 8 == 0,
                VRB_ERR_INVALID, "group_norm_apply_scatter: the slice must lie inside the full plane on an 8-element boundary");
    GnGeom g;
    if (int rc = make_geom(g, batch, channels, spatial_local, groups, "group_norm_apply_scatter", frames)) return rc;
    g.stat_frames = 1;   // mean / inverse are per (batch entry, group): the frames only split the planes
    GnScatter scatter{};
    scatter.count = destination_count;
    scatter.plane_stride = spatial_full;
    scatter.plane_offset = spatial_offset;
    for (int k = 0; k < destination_count; ++k) {
        VRB_REQUIRE(destinations[k] != nullptr && aligned16(destinations[k]), VRB_ERR_INVALID,
                    "group_norm_apply_scatter: destinations must be non-null and 16-byte aligned");
        scatter.dst[k] = destinations[k];
    }
    return run_apply(x, dtype, weight, weight_dtype, bias, bias_dtype, scatter.dst[0], g, mean, inverse, fuse_silu,
                     as_stream(stream), scatter);
}

extern "C" int vrb_rms_norm_axis(const void* x, int dtype, const void* weight, int weight_dtype, void* out,
                                 int64_t outer, int64_t axis, int64_t inner, float eps, int fuse_silu,
                                 vrb_stream stream) {
    VRB_REQUIRE(x && out, VRB_ERR_INVALID, "rms_norm_axis: null tensor");
    VRB_REQUIRE(outer > 0 && axis > 0 && inner > 0, VRB_ERR_INVALID, "rms_norm axis invalid");
    VRB_REQUIRE(is_float_dtype(dtype), VRB_ERR_UNSUPPORTED, "rms_norm_axis: dtype must be F32 or BF16");
    cudaStream_t s = as_stream(stream);
    if (inner > 1 && launch_rms_axis_tiles(x, dtype, weight, weight_dtype, out, outer, axis, inner, eps, fuse_silu, s))
        return after_launch("rms_norm_axis");
    if (inner % 8 == 0 && aligned16(x) && aligned16(out)) {
        const int64_t items = outer * (inner / 8);
        rms_axis_kernel<true><<<grid_for((items + kThreads - 1) / kThreads, 8), kThreads, 0, s>>>(
            x, dtype, weight, weight_dtype, out, outer, axis, inner, eps, fuse_silu);
    } else {
        const int64_t items = outer * inner;
        rms_axis_kernel<false><<<grid_for((items + kThreads - 1) / kThreads, 8), kThreads, 0, s>>>(
            x, dtype, weight, weight_dtype, out, outer, axis, inner, eps, fuse_silu);
    }
    return after_launch("rms_norm_axis");
}
