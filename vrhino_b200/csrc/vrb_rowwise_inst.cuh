// Instantiation helper for the row kernel family: each translation unit that includes this
// header defines launch_row_variant<> for a few (NORM, POST, dtype class) combinations.
#pragma once

#include "vrb_rowwise.cuh"

#include <mutex>

namespace vrb {
namespace rowwise {

// Grid = every CTA the device can hold at once (occupancy of this instantiation x SM count),
// capped by the amount of work; CTAs stride over the rows.
template <int NCH, int TPR, bool FULL, int NORM, int POST, int DT>
void launch_one(const RowParams& p, int64_t ctas, size_t smem, cudaStream_t stream) {
    // per device: resident CTAs per SM of this instantiation for the last shared-memory size seen,
    // and the largest dynamic shared-memory size opted into (dynamic plus static above 48 KB needs the opt-in);
    // guarded so that callers on several host threads may launch concurrently
    constexpr int kDevices = 32;
    static std::mutex mutex;
    static int cached_per_sm[kDevices] = {};
    static size_t cached_smem[kDevices] = {};
    static size_t opted_smem[kDevices] = {};
    int device = 0;
    if (cudaGetDevice(&device) != cudaSuccess || device < 0 || device >= kDevices) device = kDevices - 1;
    int per_sm;
    {
        std::lock_guard<std::mutex> lock(mutex);
        if (smem > 40 * 1024 && smem > opted_smem[device]) {
            if (cudaFuncSetAttribute(row_kernel<NCH, TPR, FULL, NORM, POST, DT>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                     static_cast<int>(smem)) == cudaSuccess)
                opted_smem[device] = smem;
            cached_per_sm[device] = 0;
        }
        if (cached_per_sm[device] == 0 || cached_smem[device] != smem) {
            int n = 0;
            if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&n, row_kernel<NCH, TPR, FULL, NORM, POST, DT>, kRowThreads, smem) !=
                    cudaSuccess || n < 1)
                n = 1;
            cached_per_sm[device] = n;
            cached_smem[device] = smem;
        }
        per_sm = cached_per_sm[device];
    }
    const int grid = grid_for(ctas, per_sm);
    if (p.nrows_b != 0) {
        // two problems: CTAs in proportion to the rows, at least one each
        RowParams pair = p;
        const double share = static_cast<double>(p.nrows32) / (static_cast<double>(p.nrows32) + static_cast<double>(p.nrows_b));
        int first = static_cast<int>(share * grid + 0.5);
        first = first < 1 ? 1 : first;
        const int total = grid < 2 ? 2 : grid;
        if (first > total - 1) first = total - 1;
        pair.blocks_a = static_cast<unsigned>(first);
        launch_overlapped(row_kernel<NCH, TPR, FULL, NORM, POST, DT>, dim3(total), dim3(kRowThreads), smem, stream, pair);
        return;
    }
    launch_overlapped(row_kernel<NCH, TPR, FULL, NORM, POST, DT>, dim3(grid), dim3(kRowThreads), smem, stream, p);
}

#define VRB_DEFINE_ROW_VARIANT(NORM, POST, DT)                                                                       \
    template <>                                                                                                      \
    void launch_row_variant<NORM, POST, DT>(const RowParams& p, int geometry, int64_t ctas, size_t smem,             \
                                            cudaStream_t s) {                                                        \
        switch (geometry) {                                                                                          \
            case 0: launch_one<1, 0, false, NORM, POST, DT>(p, ctas, smem, s); break;                                \
            case 1: launch_one<2, 0, false, NORM, POST, DT>(p, ctas, smem, s); break;                                \
            case 2: launch_one<3, 0, false, NORM, POST, DT>(p, ctas, smem, s); break;                                \
            case 3: launch_one<4, 0, false, NORM, POST, DT>(p, ctas, smem, s); break;                                \
            case 4: launch_one<5, 0, false, NORM, POST, DT>(p, ctas, smem, s); break;                                \
            case 5: launch_one<6, 0, false, NORM, POST, DT>(p, ctas, smem, s); break;                                \
            case 6: launch_one<8, 0, false, NORM, POST, DT>(p, ctas, smem, s); break;                                \
            case kExact1536: launch_one<6, 32, true, NORM, POST, DT>(p, ctas, smem, s); break;                       \
            case kExact3072: launch_one<6, 64, true, NORM, POST, DT>(p, ctas, smem, s); break;                       \
            case kExact5120: launch_one<5, 128, true, NORM, POST, DT>(p, ctas, smem, s); break;                      \
            case kExact2048: launch_one<4, 64, true, NORM, POST, DT>(p, ctas, smem, s); break;                       \
            case kExact64: launch_one<1, 8, true, NORM, POST, DT>(p, ctas, smem, s); break;                          \
            default: launch_one<2, 8, true, NORM, POST, DT>(p, ctas, smem, s); break;                                \
        }                                                                                                            \
    }

}  // namespace rowwise
}  // namespace vrb
