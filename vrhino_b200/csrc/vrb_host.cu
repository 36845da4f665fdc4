// Host-buffer entry points: fused chains applied to tensors that live in HOST memory.
//
// The reference's operators accept host tensors and upload them on demand (copy_to_device,
// native/src/backend/cuda/cuda_backend.cu:3195) and results are fetched with copy_to_host.
// For a bandwidth-bound operator that round trip is all PCIe time, so it is pipelined: the rows
// are cut into blocks of a few MiB that pass through kSlots staging buffers.  One stream carries
// every upload, one every kernel, one every download, and events hand a block from one to the
// next (uploaded -> computed -> downloaded, the last one freeing the slot for the upload three
// blocks later): each copy engine always has its next copy queued behind the current one, so
// both PCIe directions stay busy.  (With a stream per slot -- upload, kernel and download of a
// block in one stream -- every upload sat behind the previous download of its stream; this order
// measured 2-5 % more upload bandwidth per call.)
// Operands that are shared by all rows (modulation vectors, norm weights) are uploaded once.
//
// Device staging buffers and streams are owned by the library, one set per device (the device that is
// current when a call is made), grown on demand and freed by vrb_host_release(); these are the only
// entry points of the library that allocate (vrb_device_allocation_count() counts them).  When
// anything fails mid-pipeline the streams are drained before the call returns, so no copy to or
// from the caller's host buffers is still in flight when the caller sees the error.  Copies
// are asynchronous only if the host buffers are page-locked; with pageable memory the calls
// still work but CUDA stages the copies itself and little overlaps.
#include <mutex>
#include <vector>

#include "vrb_common.cuh"

namespace vrb {
namespace {

constexpr int kSlots = 3;                          // 4 and 6 slots measured no faster
constexpr size_t kBlockBytes = size_t{16} << 20;   // per-row-stream bytes per full block, about (4 and 8 MiB: 4-12 % slower; 32 MiB: the same)

struct Arena {
    void* base = nullptr;
    size_t bytes = 0;
};

constexpr int kStreams = 3;   // upload, compute, download
struct HostPipe {
    std::mutex mutex;
    cudaStream_t streams[kStreams] = {};
    cudaEvent_t uploaded[kSlots] = {}, computed[kSlots] = {}, downloaded[kSlots] = {};
    Arena slots[kSlots];
    Arena shared;
};
constexpr int kMaxDevices = 64;
HostPipe g_pipes[kMaxDevices];

int cuda_fail(cudaError_t e, const char* what) {
    set_error("CUDA error: %s (%s)", cudaGetErrorString(e), what);
    return VRB_ERR_CUDA;
}
#define VRB_CUDA(call, what) do { cudaError_t e_ = (call); if (e_ != cudaSuccess) return cuda_fail(e_, what); } while (0)

int ensure(Arena& a, size_t bytes) {
    if (a.bytes >= bytes) return VRB_OK;
    if (a.base) { VRB_CUDA(cudaDeviceSynchronize(), "drain before regrow"); cudaFree(a.base); a.base = nullptr; a.bytes = 0; }
    VRB_CUDA(cudaMalloc(&a.base, bytes), "device staging");
    g_device_allocations.fetch_add(1, std::memory_order_relaxed);
    a.bytes = bytes;
    return VRB_OK;
}

size_t align256(size_t v) { return (v + 255) & ~size_t{255}; }

// One tensor of a pipelined call: row_bytes > 0 means it is cut by rows (host_rows of them,
// possibly fewer than the call's rows when one host row serves `rows_per_host_row` rows);
// row_bytes == 0 means a shared operand of total_bytes uploaded once.
struct Operand {
    const void* host_in = nullptr;   // input (upload) ...
    void* host_out = nullptr;        // ... or output (download)
    size_t row_bytes = 0;
    size_t total_bytes = 0;
};

// launch(block_rows, dev_ptrs[], stream): dev_ptrs are in operand order.
template <typename Launch>
int enqueue_pipeline(HostPipe& pipe, std::vector<Operand>& ops, int64_t rows, Launch launch) {
    for (auto& s : pipe.streams)
        if (!s) VRB_CUDA(cudaStreamCreateWithFlags(&s, cudaStreamNonBlocking), "stream create");
    for (cudaEvent_t* events : {pipe.uploaded, pipe.computed, pipe.downloaded})
        for (int k = 0; k < kSlots; ++k)
            if (!events[k]) VRB_CUDA(cudaEventCreateWithFlags(&events[k], cudaEventDisableTiming), "event create");
    cudaStream_t up = pipe.streams[0], compute = pipe.streams[1], down = pipe.streams[2];

    size_t widest = 1, shared_bytes = 0;
    for (const auto& o : ops) {
        if (o.row_bytes) widest = o.row_bytes > widest ? o.row_bytes : widest;
        else shared_bytes += align256(o.total_bytes);
    }
    int64_t block_rows = static_cast<int64_t>(kBlockBytes / widest);
    if (block_rows < 1) block_rows = 1;
    if (block_rows > rows) block_rows = rows;
    size_t slot_bytes = 0;
    for (const auto& o : ops) if (o.row_bytes) slot_bytes += align256(o.row_bytes * static_cast<size_t>(block_rows));
    for (auto& a : pipe.slots) if (int rc = ensure(a, slot_bytes)) return rc;
    if (int rc = ensure(pipe.shared, shared_bytes ? shared_bytes : 256)) return rc;

    // shared operands: once, at the head of the upload stream (every block's kernel waits for an upload behind them)
    std::vector<void*> dev(ops.size(), nullptr);
    size_t off = 0;
    for (size_t k = 0; k < ops.size(); ++k) {
        if (ops[k].row_bytes || !ops[k].host_in) continue;
        dev[k] = static_cast<char*>(pipe.shared.base) + off;
        off += align256(ops[k].total_bytes);
        VRB_CUDA(cudaMemcpyAsync(dev[k], ops[k].host_in, ops[k].total_bytes, cudaMemcpyHostToDevice, up), "upload shared operand");
    }

    // Block sizes ramp up at the start and down at the end (1/8, 1/4, 1/2 of a full block): the call
    // returns only when everything is back on the host, so the first upload and the last download
    // overlap nothing, and they should be short.
    std::vector<int64_t> sizes;
    {
        int64_t head[3], tail[3], left = rows;
        int heads = 0, tails = 0;
        for (int shift = 3; shift >= 1 && left > 2 * block_rows; --shift) {
            const int64_t n = block_rows >> shift;
            if (n < 1) continue;
            head[heads++] = n; tail[tails++] = n;
            left -= 2 * n;
        }
        for (int i = 0; i < heads; ++i) sizes.push_back(head[i]);
        for (; left > 0; left -= block_rows) sizes.push_back(left < block_rows ? left : block_rows);
        for (int i = tails - 1; i >= 0; --i) sizes.push_back(tail[i]);
    }
    int64_t r0 = 0;
    for (size_t b = 0; b < sizes.size(); r0 += sizes[b], ++b) {
        const int slot = static_cast<int>(b % kSlots);
        const int64_t n = sizes[b];
        // the slot is free once the block that used it last has been downloaded
        if (b >= static_cast<size_t>(kSlots)) VRB_CUDA(cudaStreamWaitEvent(up, pipe.downloaded[slot], 0), "event wait");
        size_t so = 0;
        for (size_t k = 0; k < ops.size(); ++k) {
            if (!ops[k].row_bytes) continue;
            dev[k] = static_cast<char*>(pipe.slots[slot].base) + so;
            so += align256(ops[k].row_bytes * static_cast<size_t>(block_rows));
            if (ops[k].host_in)
                VRB_CUDA(cudaMemcpyAsync(dev[k], static_cast<const char*>(ops[k].host_in) + static_cast<size_t>(r0) * ops[k].row_bytes,
                                         static_cast<size_t>(n) * ops[k].row_bytes, cudaMemcpyHostToDevice, up), "upload rows");
        }
        VRB_CUDA(cudaEventRecord(pipe.uploaded[slot], up), "event record");
        VRB_CUDA(cudaStreamWaitEvent(compute, pipe.uploaded[slot], 0), "event wait");
        if (int rc = launch(n, dev.data(), compute)) return rc;
        VRB_CUDA(cudaEventRecord(pipe.computed[slot], compute), "event record");
        VRB_CUDA(cudaStreamWaitEvent(down, pipe.computed[slot], 0), "event wait");
        for (size_t k = 0; k < ops.size(); ++k)
            if (ops[k].row_bytes && ops[k].host_out)
                VRB_CUDA(cudaMemcpyAsync(static_cast<char*>(ops[k].host_out) + static_cast<size_t>(r0) * ops[k].row_bytes, dev[k],
                                         static_cast<size_t>(n) * ops[k].row_bytes, cudaMemcpyDeviceToHost, down), "download rows");
        VRB_CUDA(cudaEventRecord(pipe.downloaded[slot], down), "event record");
    }
    return VRB_OK;
}

template <typename Launch>
int run_pipeline(std::vector<Operand>& ops, int64_t rows, Launch launch) {
    int device = 0;
    VRB_CUDA(cudaGetDevice(&device), "current device");
    VRB_REQUIRE(device >= 0 && device < kMaxDevices, VRB_ERR_UNSUPPORTED, "host pipeline: device index %d out of range", device);
    HostPipe& pipe = g_pipes[device];
    std::lock_guard<std::mutex> lock(pipe.mutex);
    const int rc = enqueue_pipeline(pipe, ops, rows, launch);
    // Drain on success and on failure alike: the caller's host buffers are its own again on return.
    cudaError_t drained = cudaSuccess;
    for (auto& s : pipe.streams) {
        if (!s) continue;
        const cudaError_t e = cudaStreamSynchronize(s);
        if (e != cudaSuccess && drained == cudaSuccess) drained = e;
    }
    if (rc != VRB_OK) return rc;   // the first failure's text stays
    if (drained != cudaSuccess) return cuda_fail(drained, "pipeline drain");
    return VRB_OK;
}

Operand rows_in(const void* host, size_t row_bytes) { Operand o; o.host_in = host; o.row_bytes = row_bytes; return o; }
Operand rows_out(void* host, size_t row_bytes) { Operand o; o.host_out = host; o.row_bytes = row_bytes; return o; }
Operand shared_in(const void* host, size_t bytes) { Operand o; o.host_in = host; o.total_bytes = bytes; return o; }

}  // namespace
}  // namespace vrb

using namespace vrb;

extern "C" int vrb_host_layer_norm_modulate(const void* x, int x_dtype, const void* weight, int weight_dtype,
                                            const void* bias, int bias_dtype, const void* scale, const void* shift,
                                            int mod_dtype, void* out, int out_dtype,
                                            int64_t rows, int64_t width, float eps) {
    VRB_REQUIRE(x && out, VRB_ERR_INVALID, "host_layer_norm_modulate: null tensor");
    VRB_REQUIRE(rows > 0 && width > 0, VRB_ERR_INVALID, "host_layer_norm_modulate: extents must be positive");
    VRB_REQUIRE(is_float_dtype(x_dtype) && is_float_dtype(out_dtype), VRB_ERR_UNSUPPORTED, "host_layer_norm_modulate: dtypes must be F32 or BF16");
    const size_t w = static_cast<size_t>(width);
    std::vector<Operand> ops = {rows_in(x, w * dtype_bytes(x_dtype)), rows_out(out, w * dtype_bytes(out_dtype)),
                                shared_in(weight, w * dtype_bytes(weight_dtype)), shared_in(bias, w * dtype_bytes(bias_dtype)),
                                shared_in(scale, w * dtype_bytes(mod_dtype)), shared_in(shift, w * dtype_bytes(mod_dtype))};
    return run_pipeline(ops, rows, [&](int64_t n, void** d, cudaStream_t st) {
        if (scale)
            return vrb_layer_norm_modulate(d[0], x_dtype, d[2], weight_dtype, d[3], bias_dtype, d[4], d[5], mod_dtype, n, 1,
                                           d[1], out_dtype, n, width, eps, st);
        return vrb_layer_norm_cast(d[0], x_dtype, d[2], weight_dtype, d[3], bias_dtype, d[1], out_dtype, n, width, eps, st);
    });
}

extern "C" int vrb_host_rms_norm_rope(const void* x, int x_dtype, const void* weight, int weight_dtype,
                                      const void* cosine, const void* sine, int64_t f_width,
                                      void* out, int out_dtype, int64_t rows, int64_t width, int64_t norm_width, float eps) {
    VRB_REQUIRE(x && out && weight, VRB_ERR_INVALID, "host_rms_norm_rope: null tensor");
    VRB_REQUIRE(rows > 0 && width > 0 && norm_width > 0, VRB_ERR_INVALID, "host_rms_norm_rope: extents must be positive");
    VRB_REQUIRE((cosine == nullptr) == (sine == nullptr), VRB_ERR_INVALID, "RoPE frequency mismatch");
    VRB_REQUIRE(is_float_dtype(x_dtype) && is_float_dtype(out_dtype), VRB_ERR_UNSUPPORTED, "host_rms_norm_rope: dtypes must be F32 or BF16");
    const size_t w = static_cast<size_t>(width);
    const size_t fw = cosine ? static_cast<size_t>(f_width) * 4 : 0;   // one F32 table row per token
    std::vector<Operand> ops = {rows_in(x, w * dtype_bytes(x_dtype)), rows_out(out, w * dtype_bytes(out_dtype)),
                                shared_in(weight, static_cast<size_t>(norm_width) * dtype_bytes(weight_dtype))};
    if (cosine) { ops.push_back(rows_in(cosine, fw)); ops.push_back(rows_in(sine, fw)); }
    return run_pipeline(ops, rows, [&](int64_t n, void** d, cudaStream_t st) {
        return vrb_rms_norm_rope(d[0], x_dtype, d[2], weight_dtype, cosine ? d[3] : nullptr, cosine ? d[4] : nullptr,
                                 n, f_width, 1, d[1], out_dtype, n, width, norm_width, eps, st);
    });
}

extern "C" int vrb_host_gated_residual(const void* residual, int residual_dtype, const void* branch, int branch_dtype,
                                       const void* gate, int gate_dtype, void* out, int state_dtype,
                                       int64_t rows, int64_t width) {
    VRB_REQUIRE(residual && branch && out, VRB_ERR_INVALID, "host_gated_residual: null tensor");
    VRB_REQUIRE(rows > 0 && width > 0, VRB_ERR_INVALID, "host_gated_residual: extents must be positive");
    VRB_REQUIRE(is_float_dtype(residual_dtype) && is_float_dtype(branch_dtype) && is_float_dtype(state_dtype),
                VRB_ERR_UNSUPPORTED, "host_gated_residual: dtypes must be F32 or BF16");
    const size_t w = static_cast<size_t>(width);
    std::vector<Operand> ops = {rows_in(residual, w * dtype_bytes(residual_dtype)), rows_in(branch, w * dtype_bytes(branch_dtype)),
                                rows_out(out, w * dtype_bytes(state_dtype)), shared_in(gate, w * dtype_bytes(gate_dtype))};
    return run_pipeline(ops, rows, [&](int64_t n, void** d, cudaStream_t st) {
        return vrb_gated_residual(d[0], residual_dtype, d[1], branch_dtype, gate ? d[3] : nullptr, gate_dtype, n, 1, d[2],
                                  state_dtype, n, width, st);
    });
}

extern "C" int vrb_host_activation(int kind, const void* x, void* out, int dtype, int64_t rows, int64_t width) {
    VRB_REQUIRE(x && out, VRB_ERR_INVALID, "host_activation: null tensor");
    VRB_REQUIRE(rows > 0 && width > 0, VRB_ERR_INVALID, "host_activation: extents must be positive");
    VRB_REQUIRE(is_float_dtype(dtype), VRB_ERR_UNSUPPORTED, "host_activation: dtype must be F32 or BF16");
    const size_t rb = static_cast<size_t>(width) * dtype_bytes(dtype);
    std::vector<Operand> ops = {rows_in(x, rb), rows_out(out, rb)};
    return run_pipeline(ops, rows, [&](int64_t n, void** d, cudaStream_t st) {
        return vrb_activation(kind, d[0], d[1], dtype, n * width, st);
    });
}

// Frees the current device's staging buffers and streams.
extern "C" void vrb_host_release(void) {
    int device = 0;
    if (cudaGetDevice(&device) != cudaSuccess || device < 0 || device >= kMaxDevices) return;
    HostPipe& pipe = g_pipes[device];
    std::lock_guard<std::mutex> lock(pipe.mutex);
    cudaDeviceSynchronize();
    for (auto& a : pipe.slots) { if (a.base) cudaFree(a.base); a = Arena{}; }
    if (pipe.shared.base) cudaFree(pipe.shared.base);
    pipe.shared = Arena{};
    for (auto& s : pipe.streams) { if (s) cudaStreamDestroy(s); s = nullptr; }
    for (cudaEvent_t* events : {pipe.uploaded, pipe.computed, pipe.downloaded})
        for (int k = 0; k < kSlots; ++k)
            if (events[k]) { cudaEventDestroy(events[k]); events[k] = nullptr; }
}
