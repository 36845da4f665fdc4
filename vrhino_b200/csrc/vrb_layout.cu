// Layout operators: permute, slice, concat, pad, nearest-neighbour resize and the sinusoidal position embedding
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
// those axes is short it is walked element by element with coalesced stores.  Element-unit walks with
// long innermost rows (a pad of the innermost axes, a slice at an odd offset) go by rows: whole 16-byte
// chunks at any phase of either side, a warp per group of rows.
#include "vrb_common.cuh"

#include <algorithm>
#include <type_traits>

namespace vrb {
namespace {

constexpr int kThreads = 256;
constexpr int kPerSm = 8;
constexpr int kBlockUnits = 128;   // walk_blocks_kernel: 16-byte units a warp moves per step
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
    int64_t step[kMaxDims];        // the distance between a thread's consecutive units (grid size x block size), as
                                   // coordinates: digits in the mixed radix of the extents (step[0] may exceed extent[0])
};

template <typename Unit>
__device__ __forceinline__ Unit unit_of(const uint4& fill) {
    if constexpr (sizeof(Unit) == 16) return fill;
    else if constexpr (sizeof(Unit) == 4) return fill.x;
    else return static_cast<Unit>(fill.x & 0xffffu);
}

// RANK > 0: the number of dimensions is a compile-time constant; RANK == 0: any rank up to kMaxDims.
// replicate: bit d set = positions outside the source along dimension d take the nearest source element,
// clear = they (and the whole element) take the fill value.
template <typename Unit, int RANK, bool PAD, typename Index>
__global__ void __launch_bounds__(kThreads) walk_kernel(const Unit* __restrict__ in, Unit* __restrict__ out, const Walk w,
                                                        const uint4 fill, const int replicate) {
    pdl_launch_dependents();
    pdl_wait();
    const Index total = static_cast<Index>(w.total);
    const Index stride = static_cast<Index>(gridDim.x) * kThreads;
    const int rank = RANK > 0 ? RANK : w.rank;
    if constexpr (RANK > 0) {
        // Compile-time rank: the coordinates of the thread's first unit are found by division once; from one unit to
        // the thread's next they advance by the launch's step, digit by digit with carries -- no division in the loop.
        using Offset = typename std::conditional<sizeof(Index) == 4, int32_t, int64_t>::type;
        Index coordinate[RANK];
        {
            Index remaining = static_cast<Index>(blockIdx.x) * kThreads + threadIdx.x;
#pragma unroll
            for (int d = RANK - 1; d > 0; --d) {
                const Index extent = static_cast<Index>(w.extent[d]);
                const Index quotient = remaining / extent;
                coordinate[d] = remaining - quotient * extent;
                remaining = quotient;
            }
            coordinate[0] = remaining;
        }
        for (Index base = static_cast<Index>(blockIdx.x) * kThreads + threadIdx.x; base < total; base += stride * kUnroll) {
            Unit value[kUnroll];
            Offset target[kUnroll];
#pragma unroll
            for (int k = 0; k < kUnroll; ++k) {
                target[k] = -1;
                if (base + static_cast<Index>(k) * stride < total) {
                    Offset source = 0, destination = 0;
                    bool valid = true;
#pragma unroll
                    for (int d = 0; d < RANK; ++d) {
                        destination += static_cast<Offset>(coordinate[d]) * static_cast<Offset>(w.out_stride[d]);
                        Offset from = static_cast<Offset>(coordinate[d]);
                        if constexpr (PAD) {
                            from -= static_cast<Offset>(w.before[d]);
                            if (from < 0 || from >= static_cast<Offset>(w.in_extent[d])) {
                                valid = valid && ((replicate >> d) & 1) != 0;
                                from = from < 0 ? 0 : static_cast<Offset>(w.in_extent[d]) - 1;
                            }
                        }
                        source += from * static_cast<Offset>(w.in_stride[d]);
                    }
                    target[k] = destination;
                    value[k] = valid ? in[source] : unit_of<Unit>(fill);
                }
                // on to the thread's next unit (past the end the coordinates are no longer used)
                Index carry = 0;
#pragma unroll
                for (int d = RANK - 1; d > 0; --d) {
                    const Index extent = static_cast<Index>(w.extent[d]);
                    Index next = coordinate[d] + static_cast<Index>(w.step[d]) + carry;
                    carry = next >= extent ? 1 : 0;
                    if (carry) next -= extent;
                    coordinate[d] = next;
                }
                coordinate[0] += static_cast<Index>(w.step[0]) + carry;
            }
#pragma unroll
            for (int k = 0; k < kUnroll; ++k)
                if (target[k] >= 0) out[target[k]] = value[k];
        }
        return;
    }
    for (Index base = static_cast<Index>(blockIdx.x) * kThreads + threadIdx.x; base < total; base += stride * kUnroll) {
        Unit value[kUnroll];
        int64_t target[kUnroll];
#pragma unroll
        for (int k = 0; k < kUnroll; ++k) {
            const Index index = base + static_cast<Index>(k) * stride;
            target[k] = -1;
            if (index < total) {
                // Index == uint32_t: every offset on either side fits 31 bits (the launcher checks), so the address
                // arithmetic is 32-bit as well
                using Offset = typename std::conditional<sizeof(Index) == 4, int32_t, int64_t>::type;
                Index remaining = index;
                Offset source = 0, destination = 0;
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
                    destination += static_cast<Offset>(coordinate) * static_cast<Offset>(w.out_stride[d]);
                    Offset from = static_cast<Offset>(coordinate);
                    if constexpr (PAD) {
                        from -= static_cast<Offset>(w.before[d]);
                        if (from < 0 || from >= static_cast<Offset>(w.in_extent[d])) {
                            valid = valid && ((replicate >> d) & 1) != 0;
                            from = from < 0 ? 0 : static_cast<Offset>(w.in_extent[d]) - 1;
                        }
                    }
                    source += from * static_cast<Offset>(w.in_stride[d]);
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

// 16-byte units whose innermost axis is a contiguous, unpadded run of a multiple of 128 units on both sides: the run
// is cut into blocks of 128 units (2 KB), the walk's innermost axis counts blocks, and a WARP takes a block at a time --
// its coordinates decoded once per warp (by division for the first block, then advanced by the launch's step with
// carries), its 128 units moved by the lanes as four fully coalesced 512-byte accesses.  One decode, with the pad's
// range tests per axis, per 2 KB instead of one per 16 bytes: the form of a pad along outer axes (LTX's causal padding
// of T).
template <int RANK, bool PAD, typename Index>
__global__ void __launch_bounds__(kThreads) walk_blocks_kernel(const uint4* __restrict__ in, uint4* __restrict__ out, const Walk w,
                                                               const uint4 fill, const int replicate) {
    pdl_launch_dependents();
    pdl_wait();
    using Offset = typename std::conditional<sizeof(Index) == 4, int32_t, int64_t>::type;
    constexpr int kPerLane = kBlockUnits / 32;
    const Index total = static_cast<Index>(w.total);
    const Index warps = static_cast<Index>(gridDim.x) * (kThreads / 32);
    const int lane = threadIdx.x % 32;
    Index block = static_cast<Index>(blockIdx.x) * (kThreads / 32) + threadIdx.x / 32;
    Index coordinate[RANK];
    {
        Index remaining = block;
#pragma unroll
        for (int d = RANK - 1; d > 0; --d) {
            const Index extent = static_cast<Index>(w.extent[d]);
            const Index quotient = remaining / extent;
            coordinate[d] = remaining - quotient * extent;
            remaining = quotient;
        }
        coordinate[0] = remaining;
    }
    for (; block < total; block += warps) {
        Offset source = 0, destination = 0;
        bool valid = true;
#pragma unroll
        for (int d = 0; d < RANK; ++d) {
            destination += static_cast<Offset>(coordinate[d]) * static_cast<Offset>(w.out_stride[d]);
            Offset from = static_cast<Offset>(coordinate[d]);
            if constexpr (PAD) {
                from -= static_cast<Offset>(w.before[d]);
                if (from < 0 || from >= static_cast<Offset>(w.in_extent[d])) {
                    valid = valid && ((replicate >> d) & 1) != 0;
                    from = from < 0 ? 0 : static_cast<Offset>(w.in_extent[d]) - 1;
                }
            }
            source += from * static_cast<Offset>(w.in_stride[d]);
        }
        uint4 value[kPerLane];
        if (valid) {
            const uint4* const from = in + source + lane;
#pragma unroll
            for (int j = 0; j < kPerLane; ++j) value[j] = from[32 * j];
        } else {
#pragma unroll
            for (int j = 0; j < kPerLane; ++j) value[j] = fill;
        }
        uint4* const to = out + destination + lane;
#pragma unroll
        for (int j = 0; j < kPerLane; ++j) to[32 * j] = value[j];
        Index carry = 0;
#pragma unroll
        for (int d = RANK - 1; d > 0; --d) {
            const Index extent = static_cast<Index>(w.extent[d]);
            Index next = coordinate[d] + static_cast<Index>(w.step[d]) + carry;
            carry = next >= extent ? 1 : 0;
            if (carry) next -= extent;
            coordinate[d] = next;
        }
        coordinate[0] += static_cast<Index>(w.step[0]) + carry;
    }
}

// Element units with long innermost rows (both innermost strides 1), whatever the alignment of either side: the form
// for a pad of the innermost axes and for a slice at an odd offset.  A warp takes `group` adjacent rows of the
// iteration space at a time, in three passes.  (1) Its first `group` lanes decompose one row index each (the
// divisions of all the rows run side by side).  (2) The lanes share out the aligned 16-byte chunks that lie inside
// the copied part of those output rows, each lane fetching its row's addresses from the lane that found them: a
// chunk is cut out of the two aligned 16-byte source blocks that hold it (words selected and shifted by the
// difference of the two sides' 16-byte phases; the second block is a cache hit, its neighbour's first) and stored
// whole, two chunks per lane in flight, their loads issued before the first store.  (3) What is left of every row
// (the pads, and the copied elements before the first and after the last whole chunk) goes one element per lane,
// the lanes shared out over all the rows' leftovers.  A row without a source is filled by the whole warp.  Loads of
// whole blocks touch only aligned 16-byte blocks that hold at least one byte of the source row.
template <typename E, bool PAD>
__global__ void __launch_bounds__(kThreads) walk_rows_kernel(const E* __restrict__ in, E* __restrict__ out, const Walk w,
                                                             const uint4 fill, const int replicate, const uint32_t rows,
                                                             const uint32_t group) {
    constexpr int kPerChunk = 16 / static_cast<int>(sizeof(E));
    constexpr int kInFlight = 2;
    pdl_launch_dependents();
    pdl_wait();
    const int last = w.rank - 1;
    const uint32_t lane = threadIdx.x % 32;
    const uint32_t warps = gridDim.x * (kThreads / 32);
    const int out_bytes = static_cast<int>(w.extent[last]) * static_cast<int>(sizeof(E));
    const int before_bytes = PAD ? static_cast<int>(w.before[last]) * static_cast<int>(sizeof(E)) : 0;
    const int in_bytes = PAD ? static_cast<int>(w.in_extent[last]) * static_cast<int>(sizeof(E)) : out_bytes;
    const bool replicate_last = PAD && ((replicate >> last) & 1) != 0;
    const E fill_value = unit_of<E>(fill);
    // where row `row` starts on either side, and whether it has a source at all
    auto locate = [&](const uint32_t row, const E*& src, E*& dst) {
        uint32_t remaining = row;
        int64_t source = 0, destination = 0;
        bool row_valid = true;
        for (int d = last - 1; d >= 0; --d) {
            uint32_t coordinate = remaining;
            if (d > 0) {
                const uint32_t extent = static_cast<uint32_t>(w.extent[d]);
                const uint32_t quotient = remaining / extent;
                coordinate = remaining - quotient * extent;
                remaining = quotient;
            }
            destination += static_cast<int64_t>(coordinate) * w.out_stride[d];
            int64_t from = coordinate;
            if constexpr (PAD) {
                from -= w.before[d];
                if (from < 0 || from >= w.in_extent[d]) {
                    row_valid = row_valid && ((replicate >> d) & 1) != 0;
                    from = from < 0 ? 0 : w.in_extent[d] - 1;
                }
            }
            source += from * w.in_stride[d];
        }
        src = in + source;
        dst = out + destination;
        return row_valid;
    };
    constexpr int kSize = static_cast<int>(sizeof(E));
    // whole chunks inside a row's copied part: at most body_slots, at least least_full (the part may start up to 14
    // bytes past a chunk boundary); everything else of a row is at most `leftovers` elements
    const uint32_t body_slots = static_cast<uint32_t>(in_bytes) / 16;
    const int least_full = in_bytes >= 30 ? (in_bytes - 14) / 16 : 0;
    const uint32_t leftovers = static_cast<uint32_t>(out_bytes / kSize - kPerChunk * least_full);
    const uint64_t stride = static_cast<uint64_t>(warps) * group;
    for (uint64_t first = static_cast<uint64_t>(blockIdx.x * (kThreads / 32) + threadIdx.x / 32) * group; first < rows; first += stride) {
        const uint32_t count = rows - first < group ? static_cast<uint32_t>(rows - first) : group;
        const E* my_src = in;
        E* my_dst = out;
        bool my_valid = false;
        if (lane < count) my_valid = locate(static_cast<uint32_t>(first) + lane, my_src, my_dst);
        const unsigned long long my_from = reinterpret_cast<unsigned long long>(my_src);
        // (the copied part's first byte on the output side; bit 0 is free in a 2-byte aligned address: the row has a source)
        const unsigned long long my_to = (reinterpret_cast<unsigned long long>(my_dst) + before_bytes) | (my_valid ? 1ull : 0ull);
        // what the chunk pass needs of a row, worked out once by the lane that located it: where the first whole
        // chunk starts on either side, and how many there are (none for a row without a source)
        const int my_head = static_cast<int>((16 - (my_to & 14)) & 15);
        const int my_full = my_valid && in_bytes >= my_head + 16 ? (in_bytes - my_head) >> 4 : 0;
        const unsigned long long my_chunks_from = my_from + my_head, my_chunks_to = (my_to & ~1ull) + my_head;

        if (body_slots != 0) {
            const uint32_t items = count * body_slots;
            const uint32_t step_rows = 32 / body_slots, step_slots = 32 % body_slots;
            uint32_t row = lane / body_slots, slot = lane % body_slots;
            for (uint32_t base = 0; base < items; base += 32 * kInFlight) {
                uint4 a[kInFlight], b[kInFlight];
                uint4* target[kInFlight];
                int phase[kInFlight];
#pragma unroll
                for (int u = 0; u < kInFlight; ++u) {
                    const bool active = base + 32 * u + lane < items;
                    const uint32_t owner = active ? row : 0;
                    const unsigned long long from = __shfl_sync(0xffffffffu, my_chunks_from, owner);
                    const unsigned long long to = __shfl_sync(0xffffffffu, my_chunks_to, owner);
                    const int full = __shfl_sync(0xffffffffu, my_full, owner);
                    a[u] = b[u] = make_uint4(0, 0, 0, 0);
                    phase[u] = 0;
                    target[u] = nullptr;
                    if (active && static_cast<int>(slot) < full) {
                        const unsigned int at = 16u * slot;
                        target[u] = reinterpret_cast<uint4*>(to + at);
                        const unsigned long long source = from + at;
                        phase[u] = static_cast<int>(source & 15);
                        const uint4* const blocks = reinterpret_cast<const uint4*>(source - phase[u]);
                        a[u] = __ldg(blocks);
                        if (phase[u] != 0) b[u] = __ldg(blocks + 1);
                    }
                    row += step_rows;
                    slot += step_slots;
                    if (slot >= body_slots) { slot -= body_slots; ++row; }
                }
#pragma unroll
                for (int u = 0; u < kInFlight; ++u) {
                    if (target[u] == nullptr) continue;
                    // words [phase / 4, phase / 4 + 4] of the two blocks, then half a word further when the phase is odd in 2-byte elements
                    uint32_t v0 = a[u].x, v1 = a[u].y, v2 = a[u].z, v3 = a[u].w, v4 = b[u].x, v5 = b[u].y, v6 = b[u].z, v7 = b[u].w;
                    if (phase[u] & 8) { v0 = v2; v1 = v3; v2 = v4; v3 = v5; v4 = v6; v5 = v7; }
                    if (phase[u] & 4) { v0 = v1; v1 = v2; v2 = v3; v3 = v4; v4 = v5; }
                    const int shift = (phase[u] & 2) * 8;
                    *target[u] = make_uint4(__funnelshift_r(v0, v1, shift), __funnelshift_r(v1, v2, shift), __funnelshift_r(v2, v3, shift),
                                            __funnelshift_r(v3, v4, shift));
                }
            }
        }

        if (leftovers != 0) {
            const uint32_t items = count * leftovers;
            const uint32_t step_rows = 32 / leftovers, step_slots = 32 % leftovers;
            uint32_t row = lane / leftovers, slot = lane % leftovers;
            for (uint32_t base = 0; base < items; base += 32) {
                const bool active = base + lane < items;
                const uint32_t owner = active ? row : 0;
                const unsigned long long from = __shfl_sync(0xffffffffu, my_from, owner);
                const unsigned long long to = __shfl_sync(0xffffffffu, my_to, owner);
                if (active && (to & 1) != 0) {
                    const int head = static_cast<int>((16 - (to & 14)) & 15);
                    const int full = in_bytes >= head + 16 ? (in_bytes - head) >> 4 : 0;
                    // leftover bytes of this row: [0, lead) and [lead + 16 * full, out_bytes)
                    const int lead = before_bytes + (full != 0 ? head : in_bytes);
                    int at = static_cast<int>(slot) * kSize;
                    if (at >= lead) at += 16 * full;
                    if (at < out_bytes) {
                        int source = at - before_bytes;
                        const bool inside = source >= 0 && source < in_bytes;
                        if (!inside) source = source < 0 ? 0 : in_bytes - kSize;
                        E value = fill_value;
                        if (inside || replicate_last) value = *reinterpret_cast<const E*>(from + source);
                        *reinterpret_cast<E*>((to & ~1ull) - before_bytes + at) = value;
                    }
                }
                row += step_rows;
                slot += step_slots;
                if (slot >= leftovers) { slot -= leftovers; ++row; }
            }
        }

        if constexpr (PAD) {
            unsigned without_source = __ballot_sync(0xffffffffu, lane < count && !my_valid);
            while (without_source != 0) {
                const int owner = __ffs(without_source) - 1;
                without_source &= without_source - 1;
                E* const dst = reinterpret_cast<E*>(__shfl_sync(0xffffffffu, reinterpret_cast<unsigned long long>(my_dst), owner));
                for (int j = lane; j < out_bytes / kSize; j += 32) dst[j] = fill_value;
            }
        }
    }
}

// Element units with a contiguous, 16-byte aligned output: a thread produces 16 adjacent output bytes (8 bf16 / 4 F32
// elements).  The first element's index is decomposed once; its neighbours differ in the innermost coordinate only,
// until a row ends (then the next index is decomposed again).  One 16-byte store per chunk instead of one
// decomposition, one load and one 2- or 4-byte store per element: the padded innermost axes of a spatial pad, a slice
// at an odd offset, a permute whose innermost axes are short.
template <typename E, bool PAD, typename Index>
__global__ void __launch_bounds__(kThreads) walk_chunks_kernel(const E* __restrict__ in, E* __restrict__ out, const Walk w,
                                                               const uint4 fill, const int replicate) {
    constexpr int K = 16 / sizeof(E);
    pdl_launch_dependents();
    pdl_wait();
    const int last = w.rank - 1;
    const Index extent_last = static_cast<Index>(w.extent[last]);
    const int64_t stride_last = w.in_stride[last];
    const int64_t before_last = PAD ? w.before[last] : 0, in_extent_last = PAD ? w.in_extent[last] : w.extent[last];
    const bool replicate_last = ((replicate >> last) & 1) != 0;
    const E fill_value = unit_of<E>(fill);
    const int64_t chunks = (w.total + K - 1) / K;
    const int64_t step = static_cast<int64_t>(gridDim.x) * kThreads;
    for (int64_t chunk = static_cast<int64_t>(blockIdx.x) * kThreads + threadIdx.x; chunk < chunks; chunk += step) {
        const int64_t first = chunk * K;
        Index inner = 0;
        int64_t outer_source = 0;
        bool outer_valid = true;
        // coordinates of element `index`: the innermost one in `inner`, the others folded into the source offset
        auto locate = [&](int64_t at) {
            const Index index = static_cast<Index>(at);
            Index remaining = index / extent_last;
            inner = index - remaining * extent_last;
            outer_source = 0;
            outer_valid = true;
            for (int d = last - 1; d >= 0; --d) {
                int64_t from = static_cast<int64_t>(remaining);
                if (d > 0) {
                    const Index extent = static_cast<Index>(w.extent[d]);
                    const Index quotient = remaining / extent;
                    from = static_cast<int64_t>(remaining - quotient * extent);
                    remaining = quotient;
                }
                if constexpr (PAD) {
                    from -= w.before[d];
                    if (from < 0 || from >= w.in_extent[d]) {
                        outer_valid = outer_valid && ((replicate >> d) & 1) != 0;
                        from = from < 0 ? 0 : w.in_extent[d] - 1;
                    }
                }
                outer_source += from * w.in_stride[d];
            }
        };
        locate(first);
        if (stride_last == 1 && outer_valid && first + K <= w.total && static_cast<int64_t>(inner) >= before_last) {
            // a run of K adjacent source elements inside one source row: aligned 32-bit loads, shifted by half a word
            // when the run starts at an odd 2-byte element (that form also reads the element after the run, so the run
            // must end before its row does)
            const E* const run = in + outer_source + (static_cast<int64_t>(inner) - before_last);
            const uintptr_t address = reinterpret_cast<uintptr_t>(run);
            const int odd = sizeof(E) == 2 && (address & 2) != 0 ? 1 : 0;
            if (static_cast<int64_t>(inner) + K + odd <= before_last + in_extent_last) {
                uint4 packed;
                if constexpr (sizeof(E) == 4) {
                    packed = make_uint4(run[0], run[1], run[2], run[3]);
                } else {
                    const uint32_t* const words = reinterpret_cast<const uint32_t*>(address & ~uintptr_t{3});
                    const uint32_t w0 = words[0], w1 = words[1], w2 = words[2], w3 = words[3];
                    if (!odd) {
                        packed = make_uint4(w0, w1, w2, w3);
                    } else {
                        const uint32_t w4 = words[4];
                        packed = make_uint4(__funnelshift_r(w0, w1, 16), __funnelshift_r(w1, w2, 16), __funnelshift_r(w2, w3, 16),
                                            __funnelshift_r(w3, w4, 16));
                    }
                }
                reinterpret_cast<uint4*>(out)[chunk] = packed;
                continue;
            }
        }
        E value[K];
#pragma unroll
        for (int k = 0; k < K; ++k) {
            value[k] = fill_value;
            if (first + k < w.total) {
                int64_t from = static_cast<int64_t>(inner) - before_last;
                bool valid = outer_valid;
                if constexpr (PAD) {
                    if (from < 0 || from >= in_extent_last) {
                        valid = valid && replicate_last;
                        from = from < 0 ? 0 : in_extent_last - 1;
                    }
                }
                if (valid) value[k] = in[outer_source + from * stride_last];
                if (++inner == extent_last && k + 1 < K) locate(first + k + 1);
            }
        }
        if (first + K <= w.total) {
            uint4 packed;
            if constexpr (sizeof(E) == 2) {
                packed = make_uint4(value[0] | (static_cast<uint32_t>(value[1]) << 16), value[2] | (static_cast<uint32_t>(value[3]) << 16),
                                    value[4] | (static_cast<uint32_t>(value[5]) << 16), value[6] | (static_cast<uint32_t>(value[7]) << 16));
            } else {
                packed = make_uint4(value[0], value[1], value[2], value[3]);
            }
            reinterpret_cast<uint4*>(out)[chunk] = packed;
        } else {
            for (int k = 0; first + k < w.total; ++k) out[first + k] = value[k];
        }
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
        // fewer than 2^31 tiles (the launcher checks): 32-bit divisions
        uint32_t remaining = static_cast<uint32_t>(t);
        const uint32_t tiles_b = static_cast<uint32_t>(g.tiles_b), tiles_a = static_cast<uint32_t>(g.tiles_a);
        uint32_t quotient = remaining / tiles_b;
        const int64_t tile_b = remaining - quotient * tiles_b;
        remaining = quotient;
        quotient = remaining / tiles_a;
        const int64_t tile_a = remaining - quotient * tiles_a;
        remaining = quotient;
        int64_t in_base = 0, out_base = 0;
        for (int d = g.batch_rank - 1; d >= 0; --d) {
            const uint32_t extent = static_cast<uint32_t>(g.batch_extent[d]);
            quotient = remaining / extent;
            const int64_t coordinate = remaining - quotient * extent;
            remaining = quotient;
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

// Even extents, strides and offsets: the tile is moved as pairs of elements (W = 32 bits for two bf16, 64 bits for two
// F32).  A thread loads the pairs (a, a+1) of rows b and b+1, transposes the 2 x 2 block in registers and stores the
// pairs (b, b+1) of rows a and a+1 into the tile, rows of even and odd a in separate halves so that the stores of a
// warp fall into different banks; the tile is then written out row by row, two pairs per thread.  Half the memory
// instructions of the element-wise tile, and every global access is a full 32-byte sector.
template <typename W>
__device__ __forceinline__ void transpose_2x2(W row0, W row1, W& even, W& odd) {
    if constexpr (sizeof(W) == 4) {
        even = __byte_perm(row0, row1, 0x5410);   // x(b, a), x(b + 1, a)
        odd = __byte_perm(row0, row1, 0x7632);    // x(b, a + 1), x(b + 1, a + 1)
    } else {
        even = (row0 & 0xffffffffull) | (row1 << 32);
        odd = (row0 >> 32) | (row1 & 0xffffffff00000000ull);
    }
}
// A_PAIRS: pairs of the input-contiguous axis per tile (32: 64 x 64 element tiles; 64: 128 x 64, i.e. twice as many
// contiguous bytes per input row visit).
template <typename W, int A_PAIRS>
__global__ void __launch_bounds__(kThreads) transpose_pairs_kernel(const W* __restrict__ in, W* __restrict__ out, const Transpose g) {
    constexpr int TILE_A = 2 * A_PAIRS, TILE_B = 64, B_PAIRS = TILE_B / 2, PITCH = B_PAIRS + 1;   // tile rows: a; columns: pairs of b
    constexpr int kHeld = (B_PAIRS / 8) * (A_PAIRS / 32) * 2;   // words of an interior tile a thread loads
    constexpr bool kAhead = true;                               // (64-bit words in 128-row tiles, twice the registers, were no faster: F32 uses 64-row tiles)
    __shared__ W tile[TILE_A * PITCH];
    pdl_launch_dependents();
    pdl_wait();
    const int lane = threadIdx.x % 32, warp = threadIdx.x / 32;
    struct TileAt {
        int64_t in_base, out_base, a0, b0;
        bool interior;
    };
    auto locate = [&](int64_t t) {
        // fewer than 2^31 tiles (the launcher checks): 32-bit divisions
        uint32_t remaining = static_cast<uint32_t>(t);
        const uint32_t tiles_b = static_cast<uint32_t>(g.tiles_b), tiles_a = static_cast<uint32_t>(g.tiles_a);
        uint32_t quotient = remaining / tiles_b;
        const int64_t tile_b = remaining - quotient * tiles_b;
        remaining = quotient;
        quotient = remaining / tiles_a;
        const int64_t tile_a = remaining - quotient * tiles_a;
        remaining = quotient;
        TileAt at{0, 0, tile_a * TILE_A, tile_b * TILE_B, false};
        for (int d = g.batch_rank - 1; d >= 0; --d) {
            const uint32_t extent = static_cast<uint32_t>(g.batch_extent[d]);
            quotient = remaining / extent;
            const int64_t coordinate = remaining - quotient * extent;
            remaining = quotient;
            at.in_base += coordinate * g.batch_in_stride[d];
            at.out_base += coordinate * g.batch_out_stride[d];
        }
        at.in_base += at.a0 + at.b0 * g.in_stride_b;          // elements; even
        at.out_base += at.a0 * g.out_stride_a + at.b0;
        at.interior = at.a0 + TILE_A <= g.extent_a && at.b0 + TILE_B <= g.extent_b;
        return at;
    };
    // An interior tile's words are fetched into registers one tile ahead (32-bit words, and 64-bit words in the
    // 64-row tiles): the loads of the next tile are in flight while this one is written out.  lane (+ 32) = pair of a, warp + 8 i = pair of b; no bounds tests, the row
    // pointers advanced instead of recomputed.
    W held[kHeld];
    auto fetch = [&](const TileAt& at) {
        const int64_t row_step = g.in_stride_b >> 1;                                   // one row of b, in pairs
        const W* rows = in + ((at.in_base + static_cast<int64_t>(2 * warp) * g.in_stride_b) >> 1) + lane;
        int n = 0;
#pragma unroll
        for (int i = 0; i < B_PAIRS / 8; ++i, rows += 16 * row_step) {
#pragma unroll
            for (int h = 0; h < A_PAIRS / 32; ++h) {
                held[n++] = rows[32 * h];
                held[n++] = rows[32 * h + row_step];
            }
        }
    };
    if (static_cast<int64_t>(blockIdx.x) >= g.tiles) return;
    TileAt here = locate(blockIdx.x);
    if (kAhead && here.interior) fetch(here);
    for (int64_t t = blockIdx.x; t < g.tiles; t += gridDim.x) {
        const int64_t in_base = here.in_base, out_base = here.out_base, a0 = here.a0, b0 = here.b0;
        const bool interior = here.interior;
        if (interior) {
            if constexpr (!kAhead) fetch(here);
            W* even_at = tile + lane * PITCH + warp;
            int n = 0;
#pragma unroll
            for (int i = 0; i < B_PAIRS / 8; ++i, even_at += 8) {
#pragma unroll
                for (int h = 0; h < A_PAIRS / 32; ++h, n += 2) {
                    W even, odd;
                    transpose_2x2<W>(held[n], held[n + 1], even, odd);
                    even_at[32 * h * PITCH] = even;
                    even_at[(A_PAIRS + 32 * h) * PITCH] = odd;
                }
            }
        } else {
#pragma unroll
            for (int i = 0; i < B_PAIRS / 8; ++i) {
                const int pair_b = warp + 8 * i;
                if (b0 + 2 * pair_b < g.extent_b) {
#pragma unroll
                    for (int h = 0; h < A_PAIRS / 32; ++h) {
                        const int pair_a = lane + 32 * h;
                        if (a0 + 2 * pair_a < g.extent_a) {
                            const int64_t at = in_base + static_cast<int64_t>(2 * pair_b) * g.in_stride_b + 2 * pair_a;
                            W even, odd;
                            transpose_2x2<W>(in[at >> 1], in[(at + g.in_stride_b) >> 1], even, odd);
                            tile[pair_a * PITCH + pair_b] = even;
                            tile[(A_PAIRS + pair_a) * PITCH + pair_b] = odd;
                        }
                    }
                }
            }
        }
        __syncthreads();
        // the next tile: located now, and, if it is an interior one, requested before this one is written out
        TileAt next = here;
        if (t + gridDim.x < g.tiles) {
            next = locate(t + gridDim.x);
            if (kAhead && next.interior) fetch(next);
        }
        // store: 16 threads cover the 32 pairs of one output row, two pairs each; the two half-warps take adjacent
        // tile rows (an odd pitch apart: no bank conflict)
        const int word = 2 * (threadIdx.x % 16);
        if (interior && (((out_base >> 1) | (g.out_stride_a >> 1)) & 1) == 0) {
            // every row start is aligned to two pairs: one vector store per thread and row, no tests
            const int row0 = threadIdx.x / 16;
#pragma unroll
            for (int i = 0; i < TILE_A / 16; ++i) {
                const int tile_row = row0 + 16 * i;
                const int a = tile_row < A_PAIRS ? 2 * tile_row : 2 * (tile_row - A_PAIRS) + 1;
                const W w0 = tile[tile_row * PITCH + word], w1 = tile[tile_row * PITCH + word + 1];
                W* const to = out + ((out_base + static_cast<int64_t>(a) * g.out_stride_a) >> 1) + word;
                if constexpr (sizeof(W) == 4) *reinterpret_cast<uint2*>(to) = make_uint2(w0, w1);
                else *reinterpret_cast<ulonglong2*>(to) = make_ulonglong2(w0, w1);
            }
        } else {
        const bool first_inside = b0 + 2 * word < g.extent_b, second_inside = b0 + 2 * word + 2 < g.extent_b;
#pragma unroll
        for (int i = 0; i < TILE_A / 16; ++i) {
            const int tile_row = threadIdx.x / 16 + 16 * i;
            const int a = tile_row < A_PAIRS ? 2 * tile_row : 2 * (tile_row - A_PAIRS) + 1;
            if (first_inside && a0 + a < g.extent_a) {
                const W w0 = tile[tile_row * PITCH + word], w1 = tile[tile_row * PITCH + word + 1];
                const int64_t at = (out_base + static_cast<int64_t>(a) * g.out_stride_a) / 2 + word;
                if (second_inside && (at & 1) == 0) {   // the base is aligned to two pairs (the launcher checks)
                    if constexpr (sizeof(W) == 4) *reinterpret_cast<uint2*>(out + at) = make_uint2(w0, w1);
                    else *reinterpret_cast<ulonglong2*>(out + at) = make_ulonglong2(w0, w1);
                } else {
                    out[at] = w0;
                    if (second_inside) out[at + 1] = w1;
                }
            }
        }
        }
        __syncthreads();
        here = next;
    }
}

// ---- host side ----------------------------------------------------------------------------------------
struct Plan {
    int rank = 0;
    int64_t extent[kMaxDims]{}, in_stride[kMaxDims]{}, out_stride[kMaxDims]{}, in_extent[kMaxDims]{}, before[kMaxDims]{};
    bool replicate[kMaxDims]{};              // pad: how positions outside the source along the dimension are filled
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
        q.replicate[q.rank] = p.replicate[d];
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
    int64_t reach_in = 0, reach_out = 0;   // largest offsets on either side, in units
    for (int d = 0; d < w.rank; ++d) {
        reach_in += ((PAD ? w.in_extent[d] : w.extent[d]) - 1) * w.in_stride[d];
        reach_out += (w.extent[d] - 1) * w.out_stride[d];
    }
    const int64_t limit = int64_t{1} << 31;
    const bool wide = w.total + static_cast<int64_t>(grid) * per_block >= limit || reach_in >= limit || reach_out >= limit;
    // the step between a thread's units, in coordinates
    Walk stepped = w;
    int64_t remaining = static_cast<int64_t>(grid) * kThreads;
    for (int d = w.rank - 1; d > 0; --d) {
        stepped.step[d] = remaining % w.extent[d];
        remaining /= w.extent[d];
    }
    stepped.step[0] = remaining;
    if (wide)
        launch_overlapped(walk_kernel<Unit, 0, PAD, int64_t>, dim3(grid), dim3(kThreads), 0, stream, static_cast<const Unit*>(in),
                          static_cast<Unit*>(out), stepped, fill, replicate);
    else
        launch_overlapped(walk_kernel<Unit, RANK, PAD, uint32_t>, dim3(grid), dim3(kThreads), 0, stream, static_cast<const Unit*>(in),
                          static_cast<Unit*>(out), stepped, fill, replicate);
}

// The block form of a 16-byte walk (walk_blocks_kernel) where it applies; false = the unit walk.
template <int RANK, bool PAD>
bool launch_walk_blocks(const void* in, void* out, const Walk& w, const uint4& fill, int replicate, cudaStream_t stream) {
    const int last = w.rank - 1;
    if (w.rank != RANK || w.in_stride[last] != 1 || w.out_stride[last] != 1 || w.extent[last] % kBlockUnits != 0 ||
        (PAD && (w.before[last] != 0 || w.in_extent[last] != w.extent[last])))
        return false;
    int64_t reach_in = 0, reach_out = 0;
    for (int d = 0; d < w.rank; ++d) {
        reach_in += ((PAD ? w.in_extent[d] : w.extent[d]) - 1) * w.in_stride[d];
        reach_out += (w.extent[d] - 1) * w.out_stride[d];
    }
    const int64_t limit = int64_t{1} << 31;
    if (w.total >= limit || reach_in >= limit || reach_out >= limit) return false;
    Walk blocks = w;
    blocks.extent[last] = w.extent[last] / kBlockUnits;
    blocks.in_extent[last] = blocks.extent[last];
    blocks.in_stride[last] = blocks.out_stride[last] = kBlockUnits;
    blocks.total = w.total / kBlockUnits;
    const int warps_per_cta = kThreads / 32;
    const int grid = grid_for((blocks.total + warps_per_cta - 1) / warps_per_cta, kPerSm);
    int64_t remaining = static_cast<int64_t>(grid) * warps_per_cta;
    for (int d = w.rank - 1; d > 0; --d) {
        blocks.step[d] = remaining % blocks.extent[d];
        remaining /= blocks.extent[d];
    }
    blocks.step[0] = remaining;
    launch_overlapped(walk_blocks_kernel<RANK, PAD, uint32_t>, dim3(grid), dim3(kThreads), 0, stream, static_cast<const uint4*>(in),
                      static_cast<uint4*>(out), blocks, fill, replicate);
    return true;
}

template <typename Unit>
void launch_walk_unit(const void* in, void* out, const Walk& w, bool padded, const uint4& fill, int replicate, cudaStream_t stream) {
    if constexpr (sizeof(Unit) == 16) {
        // (padded walks only: without the pad's tests per axis the unit walk is as fast or faster -- frames-first permute
        // 67 against 70 us, slice 44 against 46 us)
        if (padded && (launch_walk_blocks<3, true>(in, out, w, fill, replicate, stream) || launch_walk_blocks<4, true>(in, out, w, fill, replicate, stream)))
            return;
    }
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
int run_plan(const void* in, void* out, int dtype, const Plan& raw, float pad_value, cudaStream_t stream, const char* what) {
    const Plan p = simplified(raw);
    int replicate = 0;
    for (int d = 0; d < p.rank; ++d) replicate |= p.replicate[d] ? 1 << d : 0;
    const int64_t element = static_cast<int64_t>(dtype_bytes(dtype));
    int64_t count = 1;
    for (int d = 0; d < p.rank; ++d) count *= p.extent[d];
    if (count == 0) return VRB_OK;
    VRB_REQUIRE(in && out, VRB_ERR_INVALID, "%s: null tensor", what);
    const char* source = static_cast<const char*>(in) + p.in_offset * element;
    char* destination = static_cast<char*>(out) + p.out_offset * element;
    const int last = p.rank - 1;
    const bool inner_run = p.in_stride[last] == 1 && p.out_stride[last] == 1 && !p.is_padded(last);

    if (!inner_run && !p.padded && p.out_stride[last] == 1) {
        // the input's contiguous dimension sits elsewhere: transposition tiles when both tile sides are long enough
        int a = -1;
        for (int d = 0; d < last; ++d)
            if (p.in_stride[d] == 1) a = d;
        if (a >= 0 && p.extent[a] >= 16 && p.extent[last] >= 16 && count / 256 < (int64_t{1} << 31)) {
            Transpose g{};
            for (int d = 0; d < last; ++d) {
                if (d == a) continue;
                g.batch_extent[g.batch_rank] = p.extent[d]; g.batch_in_stride[g.batch_rank] = p.in_stride[d];
                g.batch_out_stride[g.batch_rank] = p.out_stride[d]; ++g.batch_rank;
            }
            g.extent_a = p.extent[a]; g.extent_b = p.extent[last];
            g.in_stride_b = p.in_stride[last]; g.out_stride_a = p.out_stride[a];
            bool pairs = g.extent_a % 2 == 0 && g.extent_b % 2 == 0 && g.in_stride_b % 2 == 0 && g.out_stride_a % 2 == 0 &&
                         reinterpret_cast<uintptr_t>(source) % (2 * element) == 0 && reinterpret_cast<uintptr_t>(destination) % (4 * element) == 0;
            for (int d = 0; d < g.batch_rank && pairs; ++d) pairs = g.batch_in_stride[d] % 2 == 0 && g.batch_out_stride[d] % 2 == 0;
            const int wide_a = pairs && g.extent_a >= 128 && element == 2 ? 1 : 0;   // bf16: 128 x 64 tiles, 256 contiguous bytes per input row visit (F32 has them with 64 rows)
            const int tile = pairs || element == 2 ? 64 : 32;
            g.tiles_a = (g.extent_a + (tile << wide_a) - 1) / (tile << wide_a); g.tiles_b = (g.extent_b + tile - 1) / tile;
            g.tiles = g.tiles_a * g.tiles_b;
            for (int d = 0; d < g.batch_rank; ++d) g.tiles *= g.batch_extent[d];
            const int grid = grid_for(g.tiles, kPerSm);
            if (pairs && element == 2 && wide_a)
                launch_overlapped(transpose_pairs_kernel<uint32_t, 64>, dim3(grid), dim3(kThreads), 0, stream,
                                  reinterpret_cast<const uint32_t*>(source), reinterpret_cast<uint32_t*>(destination), g);
            else if (pairs && element == 2)
                launch_overlapped(transpose_pairs_kernel<uint32_t, 32>, dim3(grid), dim3(kThreads), 0, stream,
                                  reinterpret_cast<const uint32_t*>(source), reinterpret_cast<uint32_t*>(destination), g);
            else if (pairs)
                launch_overlapped(transpose_pairs_kernel<unsigned long long, 32>, dim3(grid), dim3(kThreads), 0, stream,
                                  reinterpret_cast<const unsigned long long*>(source), reinterpret_cast<unsigned long long*>(destination), g);
            else if (element == 2)
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
    // (a 4-byte aligned source: the chunk kernel's word loads may start one 2-byte element before a run, never before the tensor)
    bool contiguous_output = aligned16(destination) && count >= 64 && reinterpret_cast<uintptr_t>(source) % 4 == 0;
    {
        int64_t running = 1;
        for (int d = last; d >= 0 && contiguous_output; --d) {
            contiguous_output = p.out_stride[d] == running;
            running *= p.extent[d];
        }
    }
    if (unit == element && p.in_stride[last] == 1 && p.out_stride[last] == 1 && p.extent[last] >= 64 && p.extent[last] < (int64_t{1} << 28) &&
        count / p.extent[last] < (int64_t{1} << 31)) {
        const uint32_t rows = static_cast<uint32_t>(count / p.extent[last]);
        // rows a warp decomposes side by side: about 512 chunks' worth (measured on the VAE's pads: 8 rows of 768 bytes,
        // 4 of 1536; fewer pay the decomposition more often, more leave the warps out of step), and never so many that
        // a resident warp (five CTAs per SM) has fewer than four groups to take
        const int64_t row_chunks = std::max<int64_t>(1, p.in_extent[last] * element / 16);
        uint32_t group = 32;
        while (group > 1 && (group * row_chunks > 512 || static_cast<int64_t>(rows) / group < int64_t{4} * sm_count() * 5 * (kThreads / 32)))
            group /= 2;
        const int64_t groups = (static_cast<int64_t>(rows) + group - 1) / group;
        const int grid = grid_for((groups + kThreads / 32 - 1) / (kThreads / 32), kPerSm);
#define VRB_ROWS(E, PAD)                                                                                                      \
    launch_overlapped(walk_rows_kernel<E, PAD>, dim3(grid), dim3(kThreads), 0, stream, reinterpret_cast<const E*>(source), \
                      reinterpret_cast<E*>(destination), w, fill, replicate, rows, group)
        if (element == 2) { if (p.padded) VRB_ROWS(uint16_t, true); else VRB_ROWS(uint16_t, false); }
        else { if (p.padded) VRB_ROWS(uint32_t, true); else VRB_ROWS(uint32_t, false); }
#undef VRB_ROWS
        return after_launch(what);
    }
    if (unit == element && contiguous_output) {
        const int64_t chunks = (count * element + 15) / 16;
        const int grid = grid_for((chunks + kThreads - 1) / kThreads, kPerSm);
        const bool wide = count + 16 >= (int64_t{1} << 32);
#define VRB_CHUNKS(E, PAD, INDEX)                                                                                          \
    launch_overlapped(walk_chunks_kernel<E, PAD, INDEX>, dim3(grid), dim3(kThreads), 0, stream, reinterpret_cast<const E*>(source), \
                      reinterpret_cast<E*>(destination), w, fill, replicate)
        if (element == 2) {
            if (wide) { if (p.padded) VRB_CHUNKS(uint16_t, true, int64_t); else VRB_CHUNKS(uint16_t, false, int64_t); }
            else if (p.padded) VRB_CHUNKS(uint16_t, true, uint32_t);
            else VRB_CHUNKS(uint16_t, false, uint32_t);
        } else {
            if (wide) { if (p.padded) VRB_CHUNKS(uint32_t, true, int64_t); else VRB_CHUNKS(uint32_t, false, int64_t); }
            else if (p.padded) VRB_CHUNKS(uint32_t, true, uint32_t);
            else VRB_CHUNKS(uint32_t, false, uint32_t);
        }
#undef VRB_CHUNKS
        return after_launch(what);
    }
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

// ---- nearest-neighbour resize --------------------------------------------------------------------------
// CudaBackend::interpolate_nearest (native/src/backend/cuda/cuda_backend.cu:5010-5016, interpolate_kernel :2033-2045):
// out[c_0 .. c_{r-1}] = x[floor(c_d * in_d / out_d) for every d].  Leading axes of equal extent are planes.
struct Resize {
    int64_t planes;                 // product of the leading axes the resize leaves alone
    int rank;                       // resized axes (at most 3), outermost first
    int64_t in_extent[3], out_extent[3];
};

// General factors: a warp per output row (the row index decomposed and mapped once), lanes over the row's elements.
template <typename E>
__global__ void __launch_bounds__(kThreads) resize_rows_kernel(const E* __restrict__ in, E* __restrict__ out, const Resize g,
                                                               const uint32_t rows) {
    pdl_launch_dependents();
    pdl_wait();
    const int lane = threadIdx.x % 32;
    const uint32_t warps = gridDim.x * (kThreads / 32);
    const int last = g.rank - 1;
    const uint32_t in_w = static_cast<uint32_t>(g.in_extent[last]), out_w = static_cast<uint32_t>(g.out_extent[last]);
    for (uint32_t row = blockIdx.x * (kThreads / 32) + threadIdx.x / 32; row < rows; row += warps) {
        uint32_t remaining = row;
        int64_t source = 0, stride = in_w;
        for (int d = last - 1; d >= 0; --d) {
            const uint32_t extent = static_cast<uint32_t>(g.out_extent[d]);
            const uint32_t quotient = remaining / extent;
            const uint32_t coordinate = remaining - quotient * extent;
            remaining = quotient;
            source += (static_cast<int64_t>(coordinate) * g.in_extent[d] / g.out_extent[d]) * stride;
            stride *= g.in_extent[d];
        }
        source += static_cast<int64_t>(remaining) * stride;   // the plane
        const E* const src = in + source;
        E* const dst = out + static_cast<int64_t>(row) * out_w;
        for (uint32_t j = lane; j < out_w; j += 32)
            dst[j] = src[static_cast<uint32_t>(static_cast<uint64_t>(j) * in_w / out_w)];
    }
}

// Exactly twice the width (and once or twice the height): a thread reads 16 bytes of an input row and writes them
// doubled -- 32 adjacent bytes -- into one output row (TWO_ROWS: into the two output rows that copy this input row).
template <typename E, bool TWO_ROWS>
__global__ void __launch_bounds__(kThreads) resize_double_kernel(const uint4* __restrict__ in, char* __restrict__ out,
                                                                 const uint32_t chunks_per_row, const uint32_t total_chunks) {
    pdl_launch_dependents();
    pdl_wait();
    const uint32_t step = gridDim.x * kThreads;
    for (uint32_t i = blockIdx.x * kThreads + threadIdx.x; i < total_chunks; i += step) {
        const uint4 v = __ldcs(in + i);
        uint4 lo, hi;
        if constexpr (sizeof(E) == 2) {
            lo = make_uint4(__byte_perm(v.x, v.x, 0x1010), __byte_perm(v.x, v.x, 0x3232), __byte_perm(v.y, v.y, 0x1010), __byte_perm(v.y, v.y, 0x3232));
            hi = make_uint4(__byte_perm(v.z, v.z, 0x1010), __byte_perm(v.z, v.z, 0x3232), __byte_perm(v.w, v.w, 0x1010), __byte_perm(v.w, v.w, 0x3232));
        } else {
            lo = make_uint4(v.x, v.x, v.y, v.y);
            hi = make_uint4(v.z, v.z, v.w, v.w);
        }
        const uint32_t row = i / chunks_per_row, chunk = i - row * chunks_per_row;
        const int64_t row_bytes = static_cast<int64_t>(chunks_per_row) * 32;
        char* const to = out + (TWO_ROWS ? 2 : 1) * static_cast<int64_t>(row) * row_bytes + static_cast<int64_t>(chunk) * 32;
        store32_aligned(to, lo, hi);
        if constexpr (TWO_ROWS) store32_aligned(to + row_bytes, lo, hi);
    }
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

// ---- indexed gather -------------------------------------------------------------------------------------
// CudaBackend::indexed_gather (:3981-4055, indexed_gather_kernel :1754-1768): out[b, n, :] = table[b, indices[b, n], :]
// (one table for all indices when it is not batched).  A warp per gathered row, the row moved in the widest unit its
// width and the two base addresses allow.  The caller has validated the indices, as the reference does on the host;
// a row whose index is out of range all the same is left unwritten rather than read from outside the table.
template <typename Unit, typename Index>
__global__ void __launch_bounds__(kThreads) gather_rows_kernel(const Unit* __restrict__ table, const Index* __restrict__ indices,
                                                               Unit* __restrict__ out, const int64_t gathered, const int64_t per_batch,
                                                               const int64_t rows, const int64_t units) {
    pdl_launch_dependents();
    pdl_wait();
    const int lane = threadIdx.x % 32;
    const int64_t warps = static_cast<int64_t>(gridDim.x) * (kThreads / 32);
    for (int64_t n = static_cast<int64_t>(blockIdx.x) * (kThreads / 32) + threadIdx.x / 32; n < gathered; n += warps) {
        const int64_t row = static_cast<int64_t>(indices[n]);
        if (row < 0 || row >= rows) continue;
        const int64_t batch = per_batch > 0 ? n / per_batch : 0;
        const Unit* const from = table + (batch * rows + row) * units;
        Unit* const to = out + n * units;
        int64_t u = lane;
        for (; u + 96 < units; u += 128) {
            const Unit a = from[u], b = from[u + 32], c = from[u + 64], d = from[u + 96];
            to[u] = a; to[u + 32] = b; to[u + 64] = c; to[u + 96] = d;
        }
        for (; u < units; u += 32) to[u] = from[u];
    }
}

template <typename Unit>
void launch_gather(const void* table, const void* indices, int index_dtype, void* out, int64_t gathered, int64_t per_batch, int64_t rows,
                   int64_t units, cudaStream_t stream) {
    const int grid = grid_for((gathered + kThreads / 32 - 1) / (kThreads / 32), kPerSm);
    if (index_dtype == VRB_I64)
        launch_overlapped(gather_rows_kernel<Unit, int64_t>, dim3(grid), dim3(kThreads), 0, stream, static_cast<const Unit*>(table),
                          static_cast<const int64_t*>(indices), static_cast<Unit*>(out), gathered, per_batch, rows, units);
    else
        launch_overlapped(gather_rows_kernel<Unit, int32_t>, dim3(grid), dim3(kThreads), 0, stream, static_cast<const Unit*>(table),
                          static_cast<const int32_t*>(indices), static_cast<Unit*>(out), gathered, per_batch, rows, units);
}

}  // namespace
}  // namespace vrb

using namespace vrb;

extern "C" int vrb_permute(const void* x, void* out, int dtype, int rank, const int64_t* shape, const int64_t* dims,
                           vrb_stream stream) {
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
    return run_plan(x, out, dtype, p, 0.0f, as_stream(stream), "permute");
}

extern "C" int vrb_slice(const void* x, void* out, int dtype, int rank, const int64_t* shape, int dim, int64_t start, int64_t stop,
                         vrb_stream stream) {
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
    return run_plan(x, out, dtype, p, 0.0f, as_stream(stream), "slice");
}

extern "C" int vrb_concat(const void* const* inputs, const int64_t* extents, int count, void* out, int dtype, int rank,
                          const int64_t* shape, int dim, vrb_stream stream) {
    VRB_REQUIRE(count > 0 && inputs && extents, VRB_ERR_INVALID, "concat requires inputs");
    VRB_REQUIRE(is_float_dtype(dtype), VRB_ERR_UNSUPPORTED, "concat: dtype must be F32 or BF16");
    VRB_REQUIRE(valid_shape(rank, shape) && rank > 0, VRB_ERR_INVALID, "concat: invalid shape");
    if (dim < 0) dim += rank;
    VRB_REQUIRE(dim >= 0 && dim < rank, VRB_ERR_INVALID, "concat dimension invalid");
    int64_t sum = 0;
    for (int k = 0; k < count; ++k) {
        VRB_REQUIRE(extents[k] >= 0, VRB_ERR_INVALID, "concat: negative extent");
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
        const int status = run_plan(inputs[k], out, dtype, p, 0.0f, as_stream(stream), "concat");
        if (status != VRB_OK) return status;
        offset += extents[k];
    }
    return VRB_OK;
}

namespace {
int pad_any(const void* x, void* out, int dtype, int rank, const int64_t* shape, const int64_t* before, const int64_t* after,
            float value, const int* replicate_axes, int replicate_all, cudaStream_t stream) {
    VRB_REQUIRE(is_float_dtype(dtype), VRB_ERR_UNSUPPORTED, "pad: dtype must be F32 or BF16");
    VRB_REQUIRE(valid_shape(rank, shape) && rank > 0 && before && after, VRB_ERR_INVALID, "Invalid pad vector");
    Plan p;
    p.rank = rank;
    contiguous_strides(rank, shape, p.in_stride);
    int64_t source_count = 1;
    bool any_replicate = false;
    for (int d = 0; d < rank; ++d) {
        VRB_REQUIRE(before[d] >= 0 && after[d] >= 0, VRB_ERR_INVALID, "Negative padding unsupported");
        p.in_extent[d] = shape[d];
        p.before[d] = before[d];
        p.extent[d] = shape[d] + before[d] + after[d];
        p.replicate[d] = replicate_axes ? replicate_axes[d] != 0 : replicate_all != 0;
        any_replicate = any_replicate || (p.replicate[d] && p.extent[d] != shape[d]);
        source_count *= shape[d];
    }
    // an empty source has nothing to replicate from (the clamp of the kernel this replaces would read element -1)
    VRB_REQUIRE(source_count > 0 || !any_replicate, VRB_ERR_INVALID, "pad: replicate padding of an empty tensor");
    if (source_count == 0) {
        // constant padding of an empty tensor: every output element is the pad value
        for (int d = 0; d < rank; ++d) { p.in_extent[d] = 1; p.before[d] = p.extent[d]; p.in_stride[d] = 0; p.replicate[d] = false; }
    }
    contiguous_strides(rank, p.extent, p.out_stride);
    return run_plan(x, out, dtype, p, value, stream, "pad");
}
}  // namespace

extern "C" int vrb_pad(const void* x, void* out, int dtype, int rank, const int64_t* shape, const int64_t* before,
                       const int64_t* after, float value, int replicate, vrb_stream stream) {
    return pad_any(x, out, dtype, rank, shape, before, after, value, nullptr, replicate, as_stream(stream));
}

extern "C" int vrb_pad_axes(const void* x, void* out, int dtype, int rank, const int64_t* shape, const int64_t* before,
                            const int64_t* after, float value, const int* replicate_axes, vrb_stream stream) {
    VRB_REQUIRE(replicate_axes, VRB_ERR_INVALID, "pad: null mode array");
    return pad_any(x, out, dtype, rank, shape, before, after, value, replicate_axes, 0, as_stream(stream));
}

extern "C" int vrb_interpolate_nearest(const void* x, void* out, int dtype, int rank, const int64_t* in_shape, const int64_t* out_shape,
                                       vrb_stream stream) {
    VRB_REQUIRE(is_float_dtype(dtype), VRB_ERR_UNSUPPORTED, "interpolate_nearest: dtype must be F32 or BF16");
    VRB_REQUIRE(valid_shape(rank, in_shape) && valid_shape(rank, out_shape) && rank > 0, VRB_ERR_INVALID, "interpolate_nearest: invalid shape");
    int64_t count = 1, source_count = 1;
    for (int d = 0; d < rank; ++d) { count *= out_shape[d]; source_count *= in_shape[d]; }
    if (count == 0) return VRB_OK;
    VRB_REQUIRE(source_count > 0, VRB_ERR_INVALID, "Invalid interpolation factor");
    VRB_REQUIRE(x && out, VRB_ERR_INVALID, "interpolate_nearest: null tensor");
    Resize g{};
    g.planes = 1;
    int first = 0;
    while (first < rank - 1 && in_shape[first] == out_shape[first]) g.planes *= in_shape[first++];
    VRB_REQUIRE(rank - first <= 3, VRB_ERR_UNSUPPORTED, "interpolate_nearest: at most three resized axes");
    g.rank = rank - first;
    for (int d = first; d < rank; ++d) { g.in_extent[d - first] = in_shape[d]; g.out_extent[d - first] = out_shape[d]; }
    const int64_t element = static_cast<int64_t>(dtype_bytes(dtype));
    const int last = g.rank - 1;
    cudaStream_t s = as_stream(stream);
    const int64_t in_w = g.in_extent[last], out_w = g.out_extent[last];
    // twice the width, once or twice the height, nothing else resized
    bool doubled = out_w == 2 * in_w && (in_w * element) % 16 == 0 && aligned16(x) && (reinterpret_cast<uintptr_t>(out) & 31u) == 0 &&
                   source_count * element / 16 < (int64_t{1} << 32);
    bool two_rows = false;
    if (doubled && g.rank >= 2) {
        two_rows = g.out_extent[last - 1] == 2 * g.in_extent[last - 1];
        doubled = two_rows || g.out_extent[last - 1] == g.in_extent[last - 1];
        for (int d = 0; d < last - 1 && doubled; ++d) doubled = g.out_extent[d] == g.in_extent[d];
    }
    if (doubled) {
        const uint32_t chunks_per_row = static_cast<uint32_t>(in_w * element / 16);
        const uint32_t total = static_cast<uint32_t>(source_count * element / 16);
        const int grid = grid_for((static_cast<int64_t>(total) + kThreads - 1) / kThreads, kPerSm);
#define VRB_DOUBLE(E, TWO) launch_overlapped(resize_double_kernel<E, TWO>, dim3(grid), dim3(kThreads), 0, s, static_cast<const uint4*>(x), static_cast<char*>(out), chunks_per_row, total)
        if (element == 2) { if (two_rows) VRB_DOUBLE(uint16_t, true); else VRB_DOUBLE(uint16_t, false); }
        else { if (two_rows) VRB_DOUBLE(uint32_t, true); else VRB_DOUBLE(uint32_t, false); }
#undef VRB_DOUBLE
        return after_launch("interpolate_nearest");
    }
    VRB_REQUIRE(out_w < (int64_t{1} << 31) && in_w < (int64_t{1} << 31) && count / out_w < (int64_t{1} << 31), VRB_ERR_UNSUPPORTED,
                "interpolate_nearest: extents beyond the 32-bit row arithmetic");
    const uint32_t rows = static_cast<uint32_t>(count / out_w);
    const int grid = grid_for((static_cast<int64_t>(rows) + kThreads / 32 - 1) / (kThreads / 32), kPerSm);
    if (element == 2)
        launch_overlapped(resize_rows_kernel<uint16_t>, dim3(grid), dim3(kThreads), 0, s, static_cast<const uint16_t*>(x), static_cast<uint16_t*>(out), g, rows);
    else
        launch_overlapped(resize_rows_kernel<uint32_t>, dim3(grid), dim3(kThreads), 0, s, static_cast<const uint32_t*>(x), static_cast<uint32_t*>(out), g, rows);
    return after_launch("interpolate_nearest");
}

extern "C" int vrb_sinusoidal_embedding(const void* positions, void* out, int dtype, int64_t count, int64_t width, int flip,
                                        double downscale, int frequency_f64, vrb_stream stream) {
    VRB_REQUIRE(is_float_dtype(dtype), VRB_ERR_UNSUPPORTED, "sinusoidal_embedding: dtype must be F32 or BF16");
    VRB_REQUIRE(count >= 0 && width > 0 && width < (int64_t{1} << 30), VRB_ERR_INVALID, "sinusoidal embedding contract violation");
    if (count == 0) return VRB_OK;
    VRB_REQUIRE(positions && out, VRB_ERR_INVALID, "sinusoidal_embedding: null tensor");
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


extern "C" int vrb_indexed_gather(const void* table, const void* indices, int index_dtype, void* out, int dtype, int64_t batches,
                                  int64_t rows, int64_t width, int64_t indices_per_batch, vrb_stream stream) {
    VRB_REQUIRE(is_float_dtype(dtype), VRB_ERR_UNSUPPORTED, "indexed_gather: dtype must be F32 or BF16");
    VRB_REQUIRE(index_dtype == VRB_I64 || index_dtype == VRB_I32, VRB_ERR_INVALID, "indexed_gather indices must be rank >=1 int64/int32");
    VRB_REQUIRE(batches >= 0 && rows >= 0 && width >= 0 && indices_per_batch >= 0, VRB_ERR_INVALID, "indexed_gather: invalid shape");
    // batches == 0: one table for every index (indices_per_batch is then the whole count)
    const int64_t gathered = (batches > 0 ? batches : 1) * indices_per_batch;
    if (gathered * width == 0) return VRB_OK;
    VRB_REQUIRE(rows > 0, VRB_ERR_INVALID, "indexed_gather index out of range");
    VRB_REQUIRE(table && indices && out, VRB_ERR_INVALID, "indexed_gather: null tensor");
    const int64_t row_bytes = width * static_cast<int64_t>(dtype_bytes(dtype));
    const int64_t per_batch = batches > 0 ? indices_per_batch : 0;
    cudaStream_t s = as_stream(stream);
    if (row_bytes % 16 == 0 && aligned16(table) && aligned16(out))
        launch_gather<uint4>(table, indices, index_dtype, out, gathered, per_batch, rows, row_bytes / 16, s);
    else if (row_bytes % 4 == 0 && reinterpret_cast<uintptr_t>(table) % 4 == 0 && reinterpret_cast<uintptr_t>(out) % 4 == 0)
        launch_gather<uint32_t>(table, indices, index_dtype, out, gathered, per_batch, rows, row_bytes / 4, s);
    else
        launch_gather<uint16_t>(table, indices, index_dtype, out, gathered, per_batch, rows, row_bytes / 2, s);
    return after_launch("indexed_gather");
}
