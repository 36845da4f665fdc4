// rng_normal: standard-normal noise from the reference's counter-based generator.
// CudaBackend::rng_normal (native/src/backend/cuda/cuda_backend.cu:5120-5126, rng_normal_kernel :2225-2231):
// element i is the first of the four normals of cuRAND's Philox4x32-10 stream (seed, subsequence i, offset) --
// curand_init(seed, i, offset) followed by curand_normal4().x --, generated in F32 and, for a bf16 result, rounded
// to nearest even (the reference's separate cast).  The same cuRAND device functions are called here, compiled with
// the same contraction rules, so the values are the reference's bit for bit; the cast is folded into the store.
// The caller advances the offset by 4 per call, as the reference does.
#include <curand_kernel.h>

#include "vrb_common.cuh"

namespace vrb {
namespace {

constexpr int kThreads = 256;

template <bool OUT_BF16>
__global__ void __launch_bounds__(kThreads) rng_normal_kernel(void* __restrict__ out, const int64_t count, const unsigned long long seed,
                                                              const unsigned long long offset) {
    const int64_t stride = static_cast<int64_t>(gridDim.x) * kThreads;
    for (int64_t index = static_cast<int64_t>(blockIdx.x) * kThreads + threadIdx.x; index < count; index += stride) {
        curandStatePhilox4_32_10_t state;
        curand_init(seed, static_cast<unsigned long long>(index), offset, &state);
        const float value = curand_normal4(&state).x;
        if constexpr (OUT_BF16) static_cast<__nv_bfloat16*>(out)[index] = __float2bfloat16_rn(value);
        else static_cast<float*>(out)[index] = value;
    }
}

}  // namespace
}  // namespace vrb

using namespace vrb;

extern "C" int vrb_rng_normal(void* out, int dtype, int64_t count, uint64_t seed, uint64_t offset, vrb_stream stream) {
    VRB_REQUIRE(is_float_dtype(dtype), VRB_ERR_UNSUPPORTED, "rng_normal dtype unsupported");
    VRB_REQUIRE(count >= 0, VRB_ERR_INVALID, "rng_normal: invalid shape");
    if (count == 0) return VRB_OK;
    VRB_REQUIRE(out, VRB_ERR_INVALID, "rng_normal: null tensor");
    const int grid = grid_for((count + kThreads - 1) / kThreads, 8);
    cudaStream_t s = as_stream(stream);
    if (dtype == VRB_BF16) rng_normal_kernel<true><<<grid, kThreads, 0, s>>>(out, count, seed, offset);
    else rng_normal_kernel<false><<<grid, kThreads, 0, s>>>(out, count, seed, offset);
    return after_launch("rng_normal");
}
