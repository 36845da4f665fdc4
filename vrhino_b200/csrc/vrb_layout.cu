// Layout operators: permute, slice, concat, pad and the sinusoidal position embedding
// (CudaBackend::permute / concat / slice, native/src/backend/cuda/cuda_backend.cu:3936-3970, kernels
// :767-813; CudaBackend::pad :4875-4883, pad_kernel :1771-1788; CudaBackend::sinusoidal_embedding
// :4190-4196, sinusoidal_kernel :1178-1198).  Index work only (plus one F32 -> bf16 rounding of the
// pad value): bit-exact.
//
// The four copies are one operation: walk an iteration space and move out[Σ c·out_stride] =
// in[Σ c'·in_stride], where c' = c (permute, slice, concat) or c − before clamped into / tested
// against the source extent (pad).  The host side removes extent-1 dimensions, merges neighbours
// that are contiguous on both sides, and picks the widest unit (16, 4 or 2 bytes) that every
// stride, offset and base address is a multiple of, so a slice along any but the last axis, a
// concat, a permute that keeps the innermost axis, and a pad of outer axes move 16 bytes per
// thread and step.  A permute that moves the innermost axis goes through shared-memory tiles over
// (the input's innermost axis, the output's innermost axis), both sides coalesced; when either of
// those axes is short it is walked element by element with coalesced stores.
#include "vrb_common.cuh"

#include <algorithm>
#include <type_traits>

namespace vrb {
namespace {

constexpr int kThreads = 256;
constexpr int kPerSm = 8;
constexpr int kMaxDims = 8;
constexpr int kUnroll = 4;

struct Walk {
    int rank;
    int64_t extent[kMaxDims];      // iteration space, outermost first; the last extent counts units
    int64_t in_stride[kMaxDims];   // in units
    int64_t out_stride[kMaxDims];  // in units
    int64_t in_extent[kMaxDims];   // pad: extent of the source along the dimension
    int64_t before[kMaxDims];      // pad: leading pad along the dimension
    int64_t total;                 // units to move
};

template <typename Unit>
__device__ __forceinline__ Unit unit_of(const uint4& fill) {
    if constexpr (sizeof(Unit) == 16) return fill;
    else if constexpr (sizeof(Unit) == 4) return fill.x;
    else return static_cast<Unit>(fill.x & 0xffffu);
}

// RANK > 0: the number of dimensions is a compile-time constant; RANK == 0: any rank up to kMaxDims.
template <typename Unit, int RANK, bool PAD, typename Index>
__global__ void __launch_bounds__(kThreads) walk_kernel(const Unit* __restrict__ in, Unit* __restrict__ out, const Walk w,
                                                        const uint4 fill, const int replicate) {
    pdl_launch_dependents();
    pdl_wait();
    const Index total = static_cast<Index>(w.total);
    const Index stride = static_cast<Index>(gridDim.x) * kThreads;
    const int rank = RANK > 0 ? RANK : w.rank;
    for (Index base = static_cast<Index>(blockIdx.x) * kThreads + threadIdx.x; base < total; base += stride * kUnroll) {
        Unit value[kUnroll];
        int64_t target[kUnroll];
#pragma unroll
        for (int k = 0; k < kUnroll; ++k) {
            const Index index = base + static_cast<Index>(k) * stride;
            target[k] = -1;
            if (index < total) {
                Index remaining = index;
                int64_t source = 0, destination = 0;
                bool valid = true;
#pragma unroll
                for (int d = (RANK > 0 ? RANK : kMaxDims) - 1; d >= 0; --d) {
                    if (RANK == 0 && d >= rank) continue;
                    const Index extent = static_cast<Index>(w.extent[d]);
                    Index coordinate;
                    if (d == 0) {
                        coordinate = remaining;
                    } else {
                        const Index quotient = remaining / extent;
                        coordinate = remaining - quotient * extent;
                        remaining = quotient;
                    }
                    destination += static_cast<int64_t>(coordinate) * w.out_stride[d];
                    int64_t from = static_cast<int64_t>(coordinate);
                    if constexpr (PAD) {
                        from -= w.before[d];
                        if (from < 0 || from >= w.in_extent[d]) {
                            valid = valid && replicate != 0;
                            from = from < 0 ? 0 : w.in_extent[d] - 1;
                        }
                    }
                    source += from * w.in_stride[d];
                }
                target[k] = destination;
                value[k] = valid ? in[source] : unit_of<Unit>(fill);
            }
        }
#pragma unroll
        for (int k = 0; k < kUnroll; ++k)
            if (target[k] >= 0) out[target[k]] = value[k];
    }
}

// ---- tiled transposition -------------------------------------------------------------------------------
struct Transpose {
    int batch_rank;                       // dimensions other than the two of the tile
    int64_t batch_extent[kMaxDims], batch_in_stride[kMaxDims], batch_out_stride[kMaxDims];
    int64_t extent_a, extent_b;           // a: contiguous in the input; b: contiguous in the output
    int64_t in_stride_b, out_stride_a;    // elements
    int64_t tiles_a, tiles_b, tiles;      // tiles = batch * tiles_a * tiles_b
};

template <typename E, int TILE>
__global__ void __launch_bounds__(kThreads) transpose_kernel(const E* __restrict__ in, E* __restrict__ out, const Transpose g) {
    constexpr int kRows = kThreads / TILE;                     // tile rows one pass of the block covers
    constexpr int kPadding = sizeof(E) == 2 ? 2 : 1;           // odd number of 32-bit words per row
    __shared__ E tile[TILE][TILE + kPadding];
    pdl_launch_dependents();
    pdl_wait();
    const int tx = threadIdx.x % TILE, ty = threadIdx.x / TILE;
    for (int64_t t = blockIdx.x; t < g.tiles; t += gridDim.x) {
        int64_t remaining = t;
        const int64_t tile_b = remaining % g.tiles_b; remaining /= g.tiles_b;
        const int64_t tile_a = remaining % g.tiles_a; remaining /= g.tiles_a;
        int64_t in_base = 0, out_base = 0;
        for (int d = g.batch_rank - 1; d >= 0; --d) {
            const int64_t coordinate = remaining % g.batch_extent[d];
            remaining /= g.batch_extent[d];
            in_base += coordinate * g.batch_in_stride[d];
            out_base += coordinate * g.batch_out_stride[d];
        }
        const int64_t a0 = tile_a * TILE, b0 = tile_b * TILE;
        in_base += a0 + b0 * g.in_stride_b;
        out_base += a0 * g.out_stride_a + b0;
        const bool a_read = a0 + tx < g.extent_a, b_write = b0 + tx < g.extent_b;
#pragma unroll
        for (int j = ty; j < TILE; j += kRows)
            if (a_read && b0 + j < g.extent_b) tile[j][tx] = in[in_base + j * g.in_stride_b + tx];
        __syncthreads();
#pragma unroll
        for (int j = ty; j < TILE; j += kRows)
            if (b_write && a0 + j < g.extent_a) out[out_base + j * g.out_stride_a + tx] = tile[tx][j];
        __syncthreads();
    }
}

// ---- host side ----------------------------------------------------------------------------------------
struct Plan {
    int rank = 0;
    int64_t extent[kMaxDims]{}, in_stride[kMaxDims]{}, out_stride[kMaxDims]{}, in_extent[kMaxDims]{}, before[kMaxDims]{};
    int64_t in_offset = 0, out_offset = 0;   // elements
    bool padded = false;
    bool is_padded(int d) const { return before[d] != 0 || in_extent[d] != extent[d]; }
};

void contiguous_strides(int rank, const int64_t* shape, int64_t* strides) {
    int64_t running = 1;
    for (int d = rank - 1; d >= 0; --d) { strides[d] = running; running *= shape[d]; }
}

// Drops extent-1 dimensions and merges neighbours that are contiguous on both sides.
Plan simplified(const Plan& p) {
    Plan q;
    q.in_offset = p.in_offset; q.out_offset = p.out_offset; q.padded = false;
    for (int d = 0; d < p.rank; ++d) {
        if (p.extent[d] == 1 && !p.is_padded(d)) continue;
        const int last = q.rank - 1;
        if (q.rank > 0 && !p.is_padded(d) && !q.is_padded(last) && q.in_stride[last] == p.in_stride[d] * p.extent[d] &&
            q.out_stride[last] == p.out_stride[d] * p.extent[d]) {
            q.extent[last] *= p.extent[d]; q.in_extent[last] = q.extent[last];
            q.in_stride[last] = p.in_stride[d]; q.out_stride[last] = p.out_stride[d];
            continue;
        }
        q.extent[q.rank] = p.extent[d]; q.in_extent[q.rank] = p.in_extent[d]; q.before[q.rank] = p.before[d];
        q.in_stride[q.rank] = p.in_stride[d]; q.out_stride[q.rank] = p.out_stride[d];
        ++q.rank;
    }
    if (q.rank == 0) { q.rank = 1; q.extent[0] = q.in_extent[0] = 1; q.in_stride[0] = q.out_stride[0] = 1; }
    for (int d = 0; d < q.rank; ++d) q.padded = q.padded || q.is_padded(d);
    return q;
}

template <typename Unit, int RANK, bool PAD>
void launch_walk(const void* in, void* out, const Walk& w, const uint4& fill, int replicate, cudaStream_t stream) {
    const int64_t per_block = static_cast<int64_t>(kThreads) * kUnroll;
    const int grid = grid_for((w.total + per_block - 1) / per_block, kPerSm);
    const bool wide = w.total + static_cast<int64_t>(grid) * per_block >= (int64_t{1} << 31);
    if (wide)
        launch_overlapped(walk_kernel<Unit, 0, PAD, int64_t>, dim3(grid), dim3(kThreads), 0, stream, static_cast<const Unit*>(in),
                          static_cast<Unit*>(out), w, fill, replicate);
    else
        launch_overlapped(walk_kernel<Unit, RANK, PAD, uint32_t>, dim3(grid), dim3(kThreads), 0, stream, static_cast<const Unit*>(in),
                          static_cast<Unit*>(out), w, fill, replicate);
}

template <typename Unit>
void launch_walk_unit(const void* in, void* out, const Walk& w, bool padded, const uint4& fill, int replicate, cudaStream_t stream) {
    if (padded) {
        switch (w.rank) {
            case 3: launch_walk<Unit, 3, true>(in, out, w, fill, replicate, stream); return;
            case 4: launch_walk<Unit, 4, true>(in, out, w, fill, replicate, stream); return;
            default: launch_walk<Unit, 0, true>(in, out, w, fill, replicate, stream); return;
        }
    }
    switch (w.rank) {
        case 1: launch_walk<Unit, 1, false>(in, out, w, fill, replicate, stream); return;
        case 2: launch_walk<Unit, 2, false>(in, out, w, fill, replicate, stream); return;
        case 3: launch_walk<Unit, 3, false>(in, out, w, fill, replicate, stream); return;
        case 4: launch_walk<Unit, 4, false>(in, out, w, fill, replicate, stream); return;
        default: launch_walk<Unit, 0, false>(in, out, w, fill, replicate, stream); return;
    }
}

bool multiple_of(int64_t value, int64_t unit) { return value % unit == 0; }

// Runs a simplified plan: the walk in the widest unit that fits, or transposition tiles.
int run_plan(const void* in, void* out, int dtype, const Plan& raw, float pad_value, int replicate, cudaStream_t stream,
             const char* what) {
    const Plan p = simplified(raw);
    const int64_t element = static_cast<int64_t>(dtype_bytes(dtype));
    int64_t count = 1;
    for (int d = 0; d < p.rank; ++d) count *= p.extent[d];
    if (count == 0) return VRB_OK;
    const char* source = static_cast<const char*>(in) + p.in_offset * element;
    char* destination = static_cast<char*>(out) + p.out_offset * element;
    const int last = p.rank - 1;
    const bool inner_run = p.in_stride[last] == 1 && p.out_stride[last] == 1 && !p.is_padded(last);

    if (!inner_run && !p.padded && p.out_stride[last] == 1) {
        // the input's contiguous dimension sits elsewhere: transposition tiles when both tile sides are long enough
        int a = -1;
        for (int d = 0; d < last; ++d)
            if (p.in_stride[d] == 1) a = d;
        if (a >= 0 && p.extent[a] >= 16 && p.extent[last] >= 16) {
            Transpose g{};
            for (int d = 0; d < last; ++d) {
                if (d == a) continue;
                g.batch_extent[g.batch_rank] = p.extent[d]; g.batch_in_stride[g.batch_rank] = p.in_stride[d];
                g.batch_out_stride[g.batch_rank] = p.out_stride[d]; ++g.batch_rank;
            }
            g.extent_a = p.extent[a]; g.extent_b = p.extent[last];
            g.in_stride_b = p.in_stride[last]; g.out_stride_a = p.out_stride[a];
            const int tile = element == 2 ? 64 : 32;
            g.tiles_a = (g.extent_a + tile - 1) / tile; g.tiles_b = (g.extent_b + tile - 1) / tile;
            g.tiles = g.tiles_a * g.tiles_b;
            for (int d = 0; d < g.batch_rank; ++d) g.tiles *= g.batch_extent[d];
            const int grid = grid_for(g.tiles, kPerSm);
            if (element == 2)
                launch_overlapped(transpose_kernel<uint16_t, 64>, dim3(grid), dim3(kThreads), 0, stream,
                                  reinterpret_cast<const uint16_t*>(source), reinterpret_cast<uint16_t*>(destination), g);
            else
                launch_overlapped(transpose_kernel<uint32_t, 32>, dim3(grid), dim3(kThreads), 0, stream,
                                  reinterpret_cast<const uint32_t*>(source), reinterpret_cast<uint32_t*>(destination), g);
            return after_launch(what);
        }
    }

    int64_t unit = element;
    if (inner_run) {
        for (int64_t candidate : {int64_t{16}, int64_t{4}}) {
            if (candidate <= element) break;
            bool fits = multiple_of(p.extent[last] * element, candidate) &&
                        multiple_of(reinterpret_cast<intptr_t>(source), candidate) &&
                        multiple_of(reinterpret_cast<intptr_t>(destination), candidate);
            for (int d = 0; d < last && fits; ++d)
                fits = multiple_of(p.in_stride[d] * element, candidate) && multiple_of(p.out_stride[d] * element, candidate);
            if (fits) { unit = candidate; break; }
        }
    }
    const int64_t per_unit = unit / element;
    Walk w{};
    w.rank = p.rank;
    w.total = count / per_unit;
    for (int d = 0; d < p.rank; ++d) {
        const bool inner = d == last;
        w.extent[d] = inner ? p.extent[d] / per_unit : p.extent[d];
        w.in_extent[d] = inner && per_unit > 1 ? w.extent[d] : p.in_extent[d];
        w.before[d] = p.before[d];
        w.in_stride[d] = inner && per_unit > 1 ? 1 : p.in_stride[d] / per_unit;
        w.out_stride[d] = inner && per_unit > 1 ? 1 : p.out_stride[d] / per_unit;
    }
    uint32_t pattern;
    if (dtype == VRB_BF16) {
        const uint32_t bits = static_cast<uint32_t>(__bfloat16_as_ushort(__float2bfloat16_rn(pad_value)));
        pattern = bits | (bits << 16);
    } else {
        static_assert(sizeof(float) == 4, "F32");
        memcpy(&pattern, &pad_value, 4);
    }
    const uint4 fill = make_uint4(pattern, pattern, pattern, pattern);
    if (unit == 16) launch_walk_unit<uint4>(source, destination, w, p.padded, fill, replicate, stream);
    else if (unit == 4) launch_walk_unit<uint32_t>(source, destination, w, p.padded, fill, replicate, stream);
    else launch_walk_unit<uint16_t>(source, destination, w, p.padded, fill, replicate, stream);
    return after_launch(what);
}

bool valid_shape(int rank, const int64_t* shape) {
    if (rank < 0 || rank > kMaxDims || (rank > 0 && !shape)) return false;
    for (int d = 0; d < rank; ++d)
        if (shape[d] < 0) return false;
    return true;
}

// ---- sinusoidal embedding ------------------------------------------------------------------------------
template <typename T>
__device__ __forceinline__ float load_position(const T* p, int64_t i) {
    if constexpr (sizeof(T) == 2) return bf16_bits_to_float(reinterpret_cast<const uint16_t*>(p)[i]);
    else return reinterpret_cast<const float*>(p)[i];
}
template <typename T>
__device__ __forceinline__ void store_embedding(T* p, int64_t i, float v) {
    if constexpr (sizeof(T) == 2) reinterpret_cast<uint16_t*>(p)[i] = static_cast<uint16_t>(float_to_bf16_bits(v));
    else reinterpret_cast<float*>(p)[i] = v;
}

// out[row, column]: the first `half` logical columns hold sin, the next `half` cos (flip swaps the two
// halves), frequency f = logical % half with exponent −ln(10000)·f / (half − downscale); an odd last
// column is zero.  The float path is evaluated with the same single-precision operations, in the same
// order, as the kernel it replaces; the double path likewise in double.
template <typename T>
__global__ void __launch_bounds__(kThreads) sinusoidal_kernel(const T* __restrict__ positions, T* __restrict__ out, int64_t count,
                                                              int width, int flip, double downscale, int use_double) {
    pdl_launch_dependents();
    pdl_wait();
    const int half = width / 2;
    const int64_t total = count * width, stride = static_cast<int64_t>(gridDim.x) * kThreads;
    for (int64_t index = static_cast<int64_t>(blockIdx.x) * kThreads + threadIdx.x; index < total; index += stride) {
        const int column = static_cast<int>(index % width);
        const int64_t row = index / width;
        if (column >= 2 * half) { store_embedding(out, index, 0.0f); continue; }
        const int logical = flip ? (column + half) % (2 * half) : column;
        const int frequency = logical % half;
        const float position = load_position(positions, row);
        if (use_double) {
            const double exponent = -log(10000.0) * frequency / (half - downscale);
            const double phase = static_cast<double>(position) * exp(exponent);
            store_embedding(out, index, static_cast<float>(logical < half ? sin(phase) : cos(phase)));
        } else {
            const float exponent = __fdiv_rn(__fmul_rn(-logf(10000.0f), static_cast<float>(frequency)),
                                             __fsub_rn(static_cast<float>(half), static_cast<float>(downscale)));
            const float phase = __fmul_rn(position, expf(exponent));
            store_embedding(out, index, logical < half ? sinf(phase) : cosf(phase));
        }
    }
}

}  // namespace
}  // namespace vrb

using namespace vrb;

extern "C" int vrb_permute(const void* x, void* out, int dtype, int rank, const int64_t* shape, const int64_t* dims,
                           vrb_stream stream) {
    VRB_REQUIRE(x && out, VRB_ERR_INVALID, "permute: null tensor");
    VRB_REQUIRE(is_float_dtype(dtype), VRB_ERR_UNSUPPORTED, "permute: dtype must be F32 or BF16");
    VRB_REQUIRE(valid_shape(rank, shape) && (rank == 0 || dims), VRB_ERR_INVALID, "permute rank mismatch");
    bool seen[kMaxDims] = {};
    int64_t strides[kMaxDims];
    contiguous_strides(rank, shape, strides);
    Plan p;
    p.rank = rank;
    for (int d = 0; d < rank; ++d) {
        VRB_REQUIRE(dims[d] >= 0 && dims[d] < rank && !seen[dims[d]], VRB_ERR_INVALID, "Invalid permutation");
        seen[dims[d]] = true;
        p.extent[d] = p.in_extent[d] = shape[dims[d]];
        p.in_stride[d] = strides[dims[d]];
    }
    contiguous_strides(rank, p.extent, p.out_stride);
    return run_plan(x, out, dtype, p, 0.0f, 0, as_stream(stream), "permute");
}

extern "C" int vrb_slice(const void* x, void* out, int dtype, int rank, const int64_t* shape, int dim, int64_t start, int64_t stop,
                         vrb_stream stream) {
    VRB_REQUIRE(x && out, VRB_ERR_INVALID, "slice: null tensor");
    VRB_REQUIRE(is_float_dtype(dtype), VRB_ERR_UNSUPPORTED, "slice: dtype must be F32 or BF16");
    VRB_REQUIRE(valid_shape(rank, shape) && rank > 0, VRB_ERR_INVALID, "slice: invalid shape");
    if (dim < 0) dim += rank;
    VRB_REQUIRE(dim >= 0 && dim < rank, VRB_ERR_INVALID, "slice dimension invalid");
    const int64_t size = shape[dim];
    if (start < 0) start += size;
    if (stop < 0) stop += size;
    start = std::min(std::max<int64_t>(start, 0), size);
    stop = std::min(std::max(stop, start), size);
    Plan p;
    p.rank = rank;
    contiguous_strides(rank, shape, p.in_stride);
    for (int d = 0; d < rank; ++d) p.extent[d] = p.in_extent[d] = d == dim ? stop - start : shape[d];
    contiguous_strides(rank, p.extent, p.out_stride);
    p.in_offset = start * p.in_stride[dim];
    return run_plan(x, out, dtype, p, 0.0f, 0, as_stream(stream), "slice");
}

extern "C" int vrb_concat(const void* const* inputs, const int64_t* extents, int count, void* out, int dtype, int rank,
                          const int64_t* shape, int dim, vrb_stream stream) {
    VRB_REQUIRE(count > 0 && inputs && extents, VRB_ERR_INVALID, "concat requires inputs");
    VRB_REQUIRE(out, VRB_ERR_INVALID, "concat: null output");
    VRB_REQUIRE(is_float_dtype(dtype), VRB_ERR_UNSUPPORTED, "concat: dtype must be F32 or BF16");
    VRB_REQUIRE(valid_shape(rank, shape) && rank > 0, VRB_ERR_INVALID, "concat: invalid shape");
    if (dim < 0) dim += rank;
    VRB_REQUIRE(dim >= 0 && dim < rank, VRB_ERR_INVALID, "concat dimension invalid");
    int64_t sum = 0;
    for (int k = 0; k < count; ++k) {
        VRB_REQUIRE(inputs[k] && extents[k] >= 0, VRB_ERR_INVALID, "concat: null input or negative extent");
        sum += extents[k];
    }
    VRB_REQUIRE(sum == shape[dim], VRB_ERR_INVALID, "concat shape mismatch");
    int64_t out_strides[kMaxDims];
    contiguous_strides(rank, shape, out_strides);
    int64_t offset = 0;
    for (int k = 0; k < count; ++k) {
        Plan p;
        p.rank = rank;
        for (int d = 0; d < rank; ++d) {
            p.extent[d] = p.in_extent[d] = d == dim ? extents[k] : shape[d];
            p.out_stride[d] = out_strides[d];
        }
        contiguous_strides(rank, p.extent, p.in_stride);
        p.out_offset = offset * out_strides[dim];
        const int status = run_plan(inputs[k], out, dtype, p, 0.0f, 0, as_stream(stream), "concat");
        if (status != VRB_OK) return status;
        offset += extents[k];
    }
    return VRB_OK;
}

extern "C" int vrb_pad(const void* x, void* out, int dtype, int rank, const int64_t* shape, const int64_t* before,
                       const int64_t* after, float value, int replicate, vrb_stream stream) {
    VRB_REQUIRE(x && out, VRB_ERR_INVALID, "pad: null tensor");
    VRB_REQUIRE(is_float_dtype(dtype), VRB_ERR_UNSUPPORTED, "pad: dtype must be F32 or BF16");
    VRB_REQUIRE(valid_shape(rank, shape) && rank > 0 && before && after, VRB_ERR_INVALID, "Invalid pad vector");
    Plan p;
    p.rank = rank;
    contiguous_strides(rank, shape, p.in_stride);
    int64_t source_count = 1;
    for (int d = 0; d < rank; ++d) {
        VRB_REQUIRE(before[d] >= 0 && after[d] >= 0, VRB_ERR_INVALID, "Negative padding unsupported");
        p.in_extent[d] = shape[d];
        p.before[d] = before[d];
        p.extent[d] = shape[d] + before[d] + after[d];
        source_count *= shape[d];
    }
    // an empty source has nothing to replicate from: the clamp of the kernel this replaces would read
    // element -1; refuse it instead
    VRB_REQUIRE(source_count > 0 || !replicate, VRB_ERR_INVALID, "pad: replicate padding of an empty tensor");
    if (source_count == 0) {
        // constant padding of an empty tensor: every output element is the pad value
        for (int d = 0; d < rank; ++d) { p.in_extent[d] = 1; p.before[d] = p.extent[d]; p.in_stride[d] = 0; }
    }
    contiguous_strides(rank, p.extent, p.out_stride);
    return run_plan(x, out, dtype, p, value, replicate, as_stream(stream), "pad");
}

extern "C" int vrb_sinusoidal_embedding(const void* positions, void* out, int dtype, int64_t count, int64_t width, int flip,
                                        double downscale, int frequency_f64, vrb_stream stream) {
    VRB_REQUIRE(positions && out, VRB_ERR_INVALID, "sinusoidal_embedding: null tensor");
    VRB_REQUIRE(is_float_dtype(dtype), VRB_ERR_UNSUPPORTED, "sinusoidal_embedding: dtype must be F32 or BF16");
    VRB_REQUIRE(count >= 0 && width > 0 && width < (int64_t{1} << 30), VRB_ERR_INVALID, "sinusoidal embedding contract violation");
    if (count == 0) return VRB_OK;
    const int64_t total = count * width;
    const int grid = grid_for((total + kThreads - 1) / kThreads, kPerSm);
    if (dtype == VRB_BF16)
        launch_overlapped(sinusoidal_kernel<uint16_t>, dim3(grid), dim3(kThreads), 0, as_stream(stream),
                          static_cast<const uint16_t*>(positions), static_cast<uint16_t*>(out), count, static_cast<int>(width), flip,
                          downscale, frequency_f64);
    else
        launch_overlapped(sinusoidal_kernel<float>, dim3(grid), dim3(kThreads), 0, as_stream(stream),
                          static_cast<const float*>(positions), static_cast<float*>(out), count, static_cast<int>(width), flip, downscale,
                          frequency_f64);
    return after_launch("sinusoidal_embedding");
}
