// Library runtime: error text, launch counter, device attribute cache.

#include "vrb_common.cuh"

namespace vrb {

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
extern "C" int vrb_set_launch_overlap(int enabled) { return g_launch_overlap.exchange(enabled != 0 ? 1 : 0, std::memory_order_relaxed); }
