// Tensor-map (TMA) tile loads for the shared-memory tile kernels: one elected thread issues
// cp.async.bulk.tensor copies of a [channels x positions] tile of a [outer, channels, inner] tensor and the CTA waits
// on an mbarrier, instead of every thread issuing one 16-byte cp.async per chunk.  The maps cover this GPU's own
// memory; each copy has one destination, the issuing CTA.
#pragma once

#include <cuda.h>

#include "vrb_common.cuh"

namespace vrb {

// Encodes a rank-3 tiled map over x [outer, channels, inner] (innermost first: inner, channels, outer) with a box of
// box_inner x box_channels x 1 elements, no swizzle, zero fill outside the tensor.  false: the driver entry point is
// missing or refused the geometry (the caller then takes its cp.async path).
bool encode_tile_map(CUtensorMap* map, const void* base, int dtype, int64_t outer, int64_t channels, int64_t inner,
                     int box_inner, int box_channels);
// 1 (default): tile kernels load through tensor maps where the geometry allows; 0: always cp.async.
extern std::atomic<int> g_tma_tiles;

#ifdef __CUDACC__
__device__ __forceinline__ unsigned shared_address(const void* p) { return static_cast<unsigned>(__cvta_generic_to_shared(p)); }

__device__ __forceinline__ void mbarrier_init(uint64_t* barrier, unsigned arrivals) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(shared_address(barrier)), "r"(arrivals) : "memory");
}
// makes the initialised barriers visible to the async proxy
__device__ __forceinline__ void mbarrier_init_fence() { asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory"); }
// orders this thread's earlier generic-proxy accesses to shared memory before later async-proxy (TMA) writes
__device__ __forceinline__ void async_proxy_fence() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }
__device__ __forceinline__ void mbarrier_expect_bytes(uint64_t* barrier, unsigned bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(shared_address(barrier)), "r"(bytes) : "memory");
}
// x: innermost coordinate in elements; its byte offset must be a multiple of 16
__device__ __forceinline__ void tma_load_3d(void* shared_dst, const CUtensorMap* map, int x, int y, int z, uint64_t* barrier) {
    asm volatile(
        "cp.async.bulk.tensor.3d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4}], [%5];" ::"r"(
            shared_address(shared_dst)),
        "l"(reinterpret_cast<uint64_t>(map)), "r"(x), "r"(y), "r"(z), "r"(shared_address(barrier))
        : "memory");
}
// Waits for the phase with the given parity, at most kAsyncWaitTries polls (each poll suspends for a bounded,
// hardware-chosen time); false = gave up, and *gave_up (a flag in device memory the host can read) is set.
constexpr unsigned kAsyncWaitTries = 1u << 22;
__device__ __forceinline__ bool mbarrier_wait_bounded(uint64_t* barrier, unsigned parity, int* gave_up) {
    const unsigned address = shared_address(barrier);
    for (unsigned tries = 0; tries < kAsyncWaitTries; ++tries) {
        unsigned done;
        asm volatile(
            "{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}"
            : "=r"(done)
            : "r"(address), "r"(parity)
            : "memory");
        if (done) return true;
    }
    *gave_up = 1;
    return false;
}
#endif

}  // namespace vrb
