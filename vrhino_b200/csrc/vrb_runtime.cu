// Library runtime: error text, launch counter, device attribute cache.

#include "vrb_common.cuh"
#include "vrb_tma.cuh"

namespace vrb {

std::atomic<int> g_tma_tiles{1};

bool encode_tile_map(CUtensorMap* map, const void* base, int dtype, int64_t outer, int64_t channels, int64_t inner,
                     int box_inner, int box_channels) {
    using Encode = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
    static Encode encode = [] {
        void* entry = nullptr;
        cudaDriverEntryPointQueryResult status;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &entry, cudaEnableDefault, &status) != cudaSuccess ||
            status != cudaDriverEntryPointSuccess) {
            cudaGetLastError();
            entry = nullptr;
        }
        return reinterpret_cast<Encode>(entry);
    }();
    if (!encode || !is_float_dtype(dtype) || box_inner < 1 || box_inner > 256 || box_channels < 1 || box_channels > 256) return false;
    const cuuint64_t element = dtype_bytes(dtype);
    const cuuint64_t dims[3] = {static_cast<cuuint64_t>(inner), static_cast<cuuint64_t>(channels), static_cast<cuuint64_t>(outer)};
    const cuuint64_t strides[2] = {static_cast<cuuint64_t>(inner) * element, static_cast<cuuint64_t>(channels) * inner * element};
    const cuuint32_t box[3] = {static_cast<cuuint32_t>(box_inner), static_cast<cuuint32_t>(box_channels), 1};
    const cuuint32_t steps[3] = {1, 1, 1};
    if (strides[0] % 16 != 0 || strides[1] % 16 != 0 || (box_inner * element) % 16 != 0 || !aligned16(base)) return false;
    return encode(map, dtype == VRB_BF16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 3, const_cast<void*>(base), dims,
                  strides, box, steps, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                  CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

std::atomic<uint64_t> g_launches{0};
std::atomic<uint64_t> g_device_allocations{0};
std::atomic<int> g_launch_overlap{1};

namespace {
thread_local char t_error[512] = "";
}

void set_error(const char* format, ...) {
    va_list args;
    va_start(args, format);
    vsnprintf(t_error, sizeof(t_error), format, args);
    va_end(args);
}

int sm_count() {
    static int cached[64] = {0};
    int device = 0;
    if (cudaGetDevice(&device) != cudaSuccess || device < 0 || device >= 64) return 148;
    if (cached[device] == 0) {
        int n = 0;
        if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, device) != cudaSuccess || n <= 0) n = 148;
        cached[device] = n;
    }
    return cached[device];
}

}  // namespace vrb

using namespace vrb;

extern "C" int vrb_abi_version(void) { return VRB_ABI_VERSION; }
extern "C" const char* vrb_last_error(void) { return t_error; }
extern "C" uint64_t vrb_launch_count(void) { return g_launches.load(std::memory_order_relaxed); }
extern "C" uint64_t vrb_device_allocation_count(void) { return g_device_allocations.load(std::memory_order_relaxed); }
extern "C" int vrb_set_tensor_map_tiles(int enabled) { return g_tma_tiles.exchange(enabled != 0 ? 1 : 0, std::memory_order_relaxed); }
extern "C" int vrb_set_launch_overlap(int enabled) { return g_launch_overlap.exchange(enabled != 0 ? 1 : 0, std::memory_order_relaxed); }
