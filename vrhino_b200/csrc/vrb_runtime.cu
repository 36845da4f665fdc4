// Library runtime: error text, launch counter, device attribute cache, and the host-buffer
// entry points that stream rows through pinned staging and device buffers.
#include <mutex>
#include <vector>

#include "vrb_common.cuh"

namespace vrb {

std::atomic<uint64_t> g_launches{0};

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

// ------------------------------------------------------------------ host-buffer streaming --
// A fused row operator applied to tensors that live in host memory is bound by the PCIe copies,
// so the rows are cut into blocks and pushed through `kSlots` staging slots: while block i
// runs its kernel, block i+1 is uploading and block i-1 is downloading.  Each slot owns a
// stream, a pinned input buffer, a pinned output buffer and the two device buffers.
namespace {

constexpr int kSlots = 3;

struct Slot {
    cudaStream_t stream = nullptr;
    void* host_in = nullptr; void* host_out = nullptr;
    void* dev_in = nullptr; void* dev_out = nullptr;
    size_t in_bytes = 0, out_bytes = 0;
};

struct HostPipe {
    std::mutex mutex;
    Slot slots[kSlots];
    void* dev_vectors = nullptr;
    size_t vector_bytes = 0;
    int device = -1;
};
HostPipe g_pipe;

int cuda_fail(cudaError_t e, const char* what) {
    set_error("CUDA error: %s (%s)", cudaGetErrorString(e), what);
    return VRB_ERR_CUDA;
}
#define VRB_CUDA(call, what) do { cudaError_t e_ = (call); if (e_ != cudaSuccess) return cuda_fail(e_, what); } while (0)

void free_slot(Slot& s) {
    if (s.host_in) cudaFreeHost(s.host_in);
    if (s.host_out) cudaFreeHost(s.host_out);
    if (s.dev_in) cudaFree(s.dev_in);
    if (s.dev_out) cudaFree(s.dev_out);
    if (s.stream) cudaStreamDestroy(s.stream);
    s = Slot{};
}

int ensure_slot(Slot& s, size_t in_bytes, size_t out_bytes) {
    if (!s.stream) VRB_CUDA(cudaStreamCreateWithFlags(&s.stream, cudaStreamNonBlocking), "stream create");
    if (s.in_bytes < in_bytes) {
        if (s.host_in) cudaFreeHost(s.host_in);
        if (s.dev_in) cudaFree(s.dev_in);
        s.host_in = s.dev_in = nullptr; s.in_bytes = 0;
        VRB_CUDA(cudaMallocHost(&s.host_in, in_bytes), "pinned staging");
        VRB_CUDA(cudaMalloc(&s.dev_in, in_bytes), "device staging");
        s.in_bytes = in_bytes;
    }
    if (s.out_bytes < out_bytes) {
        if (s.host_out) cudaFreeHost(s.host_out);
        if (s.dev_out) cudaFree(s.dev_out);
        s.host_out = s.dev_out = nullptr; s.out_bytes = 0;
        VRB_CUDA(cudaMallocHost(&s.host_out, out_bytes), "pinned staging");
        VRB_CUDA(cudaMalloc(&s.dev_out, out_bytes), "device staging");
        s.out_bytes = out_bytes;
    }
    return VRB_OK;
}

}  // namespace
}  // namespace vrb

using namespace vrb;

extern "C" int vrb_abi_version(void) { return VRB_ABI_VERSION; }
extern "C" const char* vrb_last_error(void) { return t_error; }
extern "C" uint64_t vrb_launch_count(void) { return g_launches.load(std::memory_order_relaxed); }

extern "C" int vrb_host_layer_norm_modulate(const void* x, int x_dtype, const void* scale, const void* shift,
                                            int mod_dtype, void* out, int out_dtype,
                                            int64_t rows, int64_t width, float eps, int host_is_pinned) {
    VRB_REQUIRE(x && out && scale, VRB_ERR_INVALID, "host_layer_norm_modulate: null tensor");
    VRB_REQUIRE(rows > 0 && width > 0, VRB_ERR_INVALID, "host_layer_norm_modulate: extents must be positive");
    VRB_REQUIRE(is_float_dtype(x_dtype) && is_float_dtype(out_dtype) && is_float_dtype(mod_dtype), VRB_ERR_UNSUPPORTED,
                "host_layer_norm_modulate: dtypes must be F32 or BF16");
    std::lock_guard<std::mutex> lock(g_pipe.mutex);
    const size_t in_row = static_cast<size_t>(width) * dtype_bytes(x_dtype);
    const size_t out_row = static_cast<size_t>(width) * dtype_bytes(out_dtype);
    // Blocks of about 8 MiB of input: large enough for full PCIe rate, small enough to overlap.
    int64_t block_rows = static_cast<int64_t>((8u << 20) / in_row);
    if (block_rows < 1) block_rows = 1;
    if (block_rows > rows) block_rows = rows;
    const size_t vec_bytes = static_cast<size_t>(width) * dtype_bytes(mod_dtype);
    if (g_pipe.vector_bytes < 2 * vec_bytes) {
        if (g_pipe.dev_vectors) cudaFree(g_pipe.dev_vectors);
        g_pipe.dev_vectors = nullptr; g_pipe.vector_bytes = 0;
        VRB_CUDA(cudaMalloc(&g_pipe.dev_vectors, 2 * vec_bytes), "device vectors");
        g_pipe.vector_bytes = 2 * vec_bytes;
    }
    for (auto& s : g_pipe.slots)
        if (int rc = ensure_slot(s, block_rows * in_row, block_rows * out_row)) return rc;
    char* dev_scale = static_cast<char*>(g_pipe.dev_vectors);
    char* dev_shift = shift ? dev_scale + vec_bytes : nullptr;
    cudaStream_t s0 = g_pipe.slots[0].stream;
    VRB_CUDA(cudaMemcpyAsync(dev_scale, scale, vec_bytes, cudaMemcpyHostToDevice, s0), "upload scale");
    if (shift) VRB_CUDA(cudaMemcpyAsync(dev_shift, shift, vec_bytes, cudaMemcpyHostToDevice, s0), "upload shift");
    VRB_CUDA(cudaStreamSynchronize(s0), "upload vectors");

    const int64_t blocks = (rows + block_rows - 1) / block_rows;
    for (int64_t b = 0; b < blocks; ++b) {
        Slot& s = g_pipe.slots[b % kSlots];
        const int64_t r0 = b * block_rows, n = (r0 + block_rows <= rows) ? block_rows : rows - r0;
        const char* src = static_cast<const char*>(x) + r0 * in_row;
        char* dst = static_cast<char*>(out) + r0 * out_row;
        // The slot's previous download must have landed before its buffers are reused.
        VRB_CUDA(cudaStreamSynchronize(s.stream), "slot drain");
        if (b >= kSlots && !host_is_pinned) {
            const int64_t pb = b - kSlots, pr0 = pb * block_rows;
            memcpy(static_cast<char*>(out) + pr0 * out_row, s.host_out, static_cast<size_t>(block_rows) * out_row);
        }
        if (host_is_pinned) {
            VRB_CUDA(cudaMemcpyAsync(s.dev_in, src, n * in_row, cudaMemcpyHostToDevice, s.stream), "upload rows");
        } else {
            memcpy(s.host_in, src, n * in_row);
            VRB_CUDA(cudaMemcpyAsync(s.dev_in, s.host_in, n * in_row, cudaMemcpyHostToDevice, s.stream), "upload rows");
        }
        if (int rc = vrb_layer_norm_modulate(s.dev_in, x_dtype, nullptr, VRB_F32, nullptr, VRB_F32, dev_scale, dev_shift,
                                             mod_dtype, n, 1, s.dev_out, out_dtype, n, width, eps, s.stream))
            return rc;
        VRB_CUDA(cudaMemcpyAsync(host_is_pinned ? static_cast<void*>(dst) : s.host_out, s.dev_out, n * out_row,
                                 cudaMemcpyDeviceToHost, s.stream), "download rows");
    }
    // Drain: the last min(blocks, kSlots) blocks are still in their slots.
    for (int64_t b = (blocks > kSlots ? blocks - kSlots : 0); b < blocks; ++b) {
        Slot& s = g_pipe.slots[b % kSlots];
        VRB_CUDA(cudaStreamSynchronize(s.stream), "slot drain");
        if (!host_is_pinned) {
            const int64_t r0 = b * block_rows, n = (r0 + block_rows <= rows) ? block_rows : rows - r0;
            memcpy(static_cast<char*>(out) + r0 * out_row, s.host_out, n * out_row);
        }
    }
    return VRB_OK;
}

extern "C" void vrb_host_release(void) {
    std::lock_guard<std::mutex> lock(g_pipe.mutex);
    for (auto& s : g_pipe.slots) free_slot(s);
    if (g_pipe.dev_vectors) cudaFree(g_pipe.dev_vectors);
    g_pipe.dev_vectors = nullptr;
    g_pipe.vector_bytes = 0;
}
