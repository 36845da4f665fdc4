// Multi-GPU host layer (include/vrb_sharded.h): one process per GPU, an NCCL communicator owned
// here, the operator kernels of libvrb.so in between.  C++ like the rest of the host side; Python
// (vrhino_b200/sharded.py) drives the same choreography over torch.distributed for the tests and the
// benchmark, this file is what a C++ pipeline links.
//
// Structure: `Transport` is the three collectives the path needs (NCCL in production, an in-process
// stand-in whose peer never answers for the watchdog's host-side test); `Communicator` adds the
// bounded wait -- poll the stream's completion event and NCCL's asynchronous error state, abort the
// communicator when the deadline passes -- and the two sharded operators.
#include "vrb_sharded.h"

#include <cuda_runtime.h>
#include <nccl.h>

#include <atomic>
#include <chrono>
#include <cstdarg>
#include <cstdio>
#include <cstring>
#include <functional>
#include <memory>
#include <string>
#include <thread>

namespace {

thread_local char t_error[512] = "";
void set_error(const char* format, ...) {
    va_list args;
    va_start(args, format);
    vsnprintf(t_error, sizeof(t_error), format, args);
    va_end(args);
}

#define VRBS_REQUIRE(cond, code, ...) \
    do {                              \
        if (!(cond)) {                \
            set_error(__VA_ARGS__);   \
            return (code);            \
        }                             \
    } while (0)

cudaStream_t as_stream(vrb_stream s) { return static_cast<cudaStream_t>(s); }
size_t up256(size_t v) { return (v + 255) & ~static_cast<size_t>(255); }
size_t element_bytes(int dtype) { return dtype == VRB_F32 ? 4 : 2; }

// ---- collectives ------------------------------------------------------------------------------
class Transport {
public:
    virtual ~Transport() = default;
    virtual int all_reduce_sum_f64(double* buffer, size_t count, cudaStream_t stream) = 0;
    virtual int broadcast_f32(float* buffer, size_t count, int root, cudaStream_t stream) = 0;
    virtual int all_gather(const void* send, void* receive, size_t bytes_per_rank, cudaStream_t stream) = 0;
    // nullptr while healthy, else a description of the asynchronous failure
    virtual const char* async_error() = 0;
    // tears the communicator down without waiting for the peers; in-flight collectives end with an error
    virtual void abort() = 0;
};

class NcclTransport final : public Transport {
public:
    static int create(std::unique_ptr<Transport>& out, int rank, int world, const void* id128) {
        ncclUniqueId id;
        static_assert(sizeof(id) == VRBS_UNIQUE_ID_BYTES, "NCCL unique id size");
        std::memcpy(&id, id128, sizeof(id));
        ncclComm_t comm = nullptr;
        const ncclResult_t rc = ncclCommInitRank(&comm, world, id, rank);
        VRBS_REQUIRE(rc == ncclSuccess, VRBS_ERR_NCCL, "NCCL error: %s (ncclCommInitRank)", ncclGetErrorString(rc));
        out.reset(new NcclTransport(comm));
        return VRBS_OK;
    }
    ~NcclTransport() override {
        if (comm_ != nullptr) ncclCommDestroy(comm_);
    }
    int all_reduce_sum_f64(double* buffer, size_t count, cudaStream_t stream) override {
        return check(ncclAllReduce(buffer, buffer, count, ncclDouble, ncclSum, comm_, stream), "ncclAllReduce");
    }
    int broadcast_f32(float* buffer, size_t count, int root, cudaStream_t stream) override {
        return check(ncclBroadcast(buffer, buffer, count, ncclFloat, root, comm_, stream), "ncclBroadcast");
    }
    int all_gather(const void* send, void* receive, size_t bytes_per_rank, cudaStream_t stream) override {
        return check(ncclAllGather(send, receive, bytes_per_rank, ncclInt8, comm_, stream), "ncclAllGather");
    }
    const char* async_error() override {
        if (comm_ == nullptr) return "communicator aborted";
        ncclResult_t state = ncclSuccess;
        if (ncclCommGetAsyncError(comm_, &state) != ncclSuccess) return "ncclCommGetAsyncError failed";
        return state == ncclSuccess || state == ncclInProgress ? nullptr : ncclGetErrorString(state);
    }
    void abort() override {
        if (comm_ != nullptr) ncclCommAbort(comm_);
        comm_ = nullptr;
    }

private:
    explicit NcclTransport(ncclComm_t comm) : comm_(comm) {}
    int check(ncclResult_t rc, const char* what) {
        VRBS_REQUIRE(rc == ncclSuccess, VRBS_ERR_NCCL, "NCCL error: %s (%s)", ncclGetErrorString(rc), what);
        return VRBS_OK;
    }
    ncclComm_t comm_;
};

// A rank whose peer never joins: collectives "enqueue" and never complete.  Host-side test of the watchdog.
class SilentPeerTransport final : public Transport {
public:
    int all_reduce_sum_f64(double*, size_t, cudaStream_t) override { return VRBS_OK; }
    int broadcast_f32(float*, size_t, int, cudaStream_t) override { return VRBS_OK; }
    int all_gather(const void*, void*, size_t, cudaStream_t) override { return VRBS_OK; }
    const char* async_error() override { return nullptr; }
    void abort() override { ++aborts; }
    int aborts = 0;
};

}  // namespace

// ---- communicator -------------------------------------------------------------------------------
struct vrbs_comm {
    std::unique_ptr<Transport> transport;
    int rank = 0, world = 1, timeout_ms = 30000;
    bool aborted = false;
    cudaEvent_t done = nullptr;

    ~vrbs_comm() {
        if (done != nullptr) cudaEventDestroy(done);
    }

    int refuse_if_aborted(const char* what) const {
        VRBS_REQUIRE(!aborted, VRBS_ERR_ABORTED, "%s: the communicator was aborted; create a new one", what);
        return VRBS_OK;
    }

    // Polls `pending` (true while work is outstanding; sets *failed on an execution error) until it clears,
    // NCCL reports an asynchronous error, or the deadline passes; the last two abort the communicator.
    int bounded_wait(const std::function<bool(bool* failed)>& pending) {
        const auto deadline = std::chrono::steady_clock::now() + std::chrono::milliseconds(timeout_ms);
        for (;;) {
            bool failed = false;
            if (!pending(&failed)) {
                VRBS_REQUIRE(!failed, VRBS_ERR_CUDA, "CUDA error while waiting for the stream");
                return VRBS_OK;
            }
            if (const char* text = transport->async_error()) {
                set_error("NCCL asynchronous error: %s; communicator aborted", text);
                transport->abort();
                aborted = true;
                return VRBS_ERR_NCCL;
            }
            if (std::chrono::steady_clock::now() >= deadline) {
                set_error("rank %d of %d waited %d ms for its stream (a peer that left?); communicator aborted", rank, world, timeout_ms);
                transport->abort();
                aborted = true;
                return VRBS_ERR_TIMEOUT;
            }
            std::this_thread::sleep_for(std::chrono::microseconds(200));
        }
    }
};

namespace {

int kernel_status(int rc) {
    if (rc == VRB_OK) return VRBS_OK;
    set_error("%s", vrb_last_error());
    return VRBS_ERR_KERNEL;
}
int cuda_status(cudaError_t e, const char* what) {
    VRBS_REQUIRE(e == cudaSuccess, VRBS_ERR_CUDA, "CUDA error: %s (%s)", cudaGetErrorString(e), what);
    return VRBS_OK;
}

// Layout of the statistics part of the workspace.
struct StatsLayout {
    size_t first_raw, shift, moments, mean, inverse, partials, partial_bytes, staging;
    static StatsLayout make(int64_t batch, int groups) {
        StatsLayout l{};
        const size_t units = static_cast<size_t>(batch) * static_cast<size_t>(groups);
        size_t at = 0;
        l.first_raw = at; at += up256(units * 4);
        l.shift = at; at += up256(units * 4);
        l.moments = at; at += up256(units * 3 * 8);
        l.mean = at; at += up256(units * 4);
        l.inverse = at; at += up256(units * 4);
        l.partials = at;
        l.partial_bytes = vrb_group_norm_workspace_bytes(batch, groups);
        at += up256(l.partial_bytes);
        l.staging = at;
        return l;
    }
};

}  // namespace

extern "C" const char* vrbs_last_error(void) { return t_error; }

extern "C" int vrbs_unique_id(void* id128) {
    VRBS_REQUIRE(id128 != nullptr, VRBS_ERR_INVALID, "unique_id: null buffer");
    ncclUniqueId id;
    const ncclResult_t rc = ncclGetUniqueId(&id);
    VRBS_REQUIRE(rc == ncclSuccess, VRBS_ERR_NCCL, "NCCL error: %s (ncclGetUniqueId)", ncclGetErrorString(rc));
    std::memcpy(id128, &id, sizeof(id));
    return VRBS_OK;
}

extern "C" int vrbs_create(vrbs_comm** comm, int rank, int world, const void* id128, int timeout_ms) {
    VRBS_REQUIRE(comm != nullptr && id128 != nullptr && world >= 1 && rank >= 0 && rank < world, VRBS_ERR_INVALID,
                 "create: rank %d of world %d", rank, world);
    std::unique_ptr<vrbs_comm> made(new vrbs_comm);
    made->rank = rank;
    made->world = world;
    if (timeout_ms > 0) made->timeout_ms = timeout_ms;
    if (int rc = NcclTransport::create(made->transport, rank, world, id128)) return rc;
    if (int rc = cuda_status(cudaEventCreateWithFlags(&made->done, cudaEventDisableTiming), "event create")) return rc;
    *comm = made.release();
    return VRBS_OK;
}

extern "C" int vrbs_destroy(vrbs_comm* comm) {
    delete comm;
    return VRBS_OK;
}
extern "C" int vrbs_rank(const vrbs_comm* comm) { return comm ? comm->rank : -1; }
extern "C" int vrbs_world(const vrbs_comm* comm) { return comm ? comm->world : -1; }
extern "C" int vrbs_aborted(const vrbs_comm* comm) { return comm && comm->aborted ? 1 : 0; }

extern "C" size_t vrbs_group_norm_workspace_bytes(const vrbs_comm* comm, int64_t batch, int groups, int gather, size_t local_bytes) {
    if (comm == nullptr || batch <= 0 || groups <= 0) return 0;
    const StatsLayout l = StatsLayout::make(batch, groups);
    return l.staging + (gather == VRBS_GATHER_NCCL ? up256(static_cast<size_t>(comm->world) * local_bytes) : 0);
}

extern "C" int vrbs_group_norm(vrbs_comm* comm, const void* x_local, int dtype, const void* weight, int weight_dtype,
                               const void* bias, int bias_dtype, void* out, int64_t batch, int64_t channels, int64_t frames,
                               int64_t rows_local, int64_t rows_full, int64_t row0, int64_t width, int groups, float eps,
                               int fuse_silu, int gather, void* const* destinations, void* workspace, size_t workspace_bytes,
                               vrb_stream stream) {
    VRBS_REQUIRE(comm != nullptr, VRBS_ERR_INVALID, "group_norm: null communicator");
    if (int rc = comm->refuse_if_aborted("group_norm")) return rc;
    VRBS_REQUIRE(x_local && workspace && (reinterpret_cast<uintptr_t>(workspace) & 255u) == 0, VRBS_ERR_INVALID,
                 "group_norm: null tensor or workspace not 256-byte aligned");
    VRBS_REQUIRE(dtype == VRB_F32 || dtype == VRB_BF16, VRBS_ERR_INVALID, "group_norm: dtype must be F32 or BF16");
    VRBS_REQUIRE(batch > 0 && channels > 0 && frames > 0 && rows_local > 0 && width > 0 && groups > 0 && channels % groups == 0 &&
                     row0 >= 0 && row0 + rows_local <= rows_full,
                 VRBS_ERR_INVALID, "group_norm: shape / groups / row range mismatch");
    VRBS_REQUIRE(gather == VRBS_GATHER_NONE || gather == VRBS_GATHER_NCCL || gather == VRBS_GATHER_PEER, VRBS_ERR_INVALID,
                 "group_norm: unknown gather mode %d", gather);
    const size_t es = element_bytes(dtype);
    const int64_t spatial_local = frames * rows_local * width;
    const size_t local_bytes = static_cast<size_t>(batch * channels * spatial_local) * es;
    VRBS_REQUIRE(workspace_bytes >= vrbs_group_norm_workspace_bytes(comm, batch, groups, gather, local_bytes), VRBS_ERR_INVALID,
                 "group_norm: workspace needs %zu bytes", vrbs_group_norm_workspace_bytes(comm, batch, groups, gather, local_bytes));
    if (gather == VRBS_GATHER_NCCL)
        VRBS_REQUIRE(out && rows_full == static_cast<int64_t>(comm->world) * rows_local && row0 == comm->rank * rows_local,
                     VRBS_ERR_INVALID, "group_norm: the NCCL gather needs equal row slices in rank order");
    if (gather == VRBS_GATHER_PEER) VRBS_REQUIRE(destinations != nullptr, VRBS_ERR_INVALID, "group_norm: peer gather without destinations");
    if (gather == VRBS_GATHER_NONE) VRBS_REQUIRE(out != nullptr, VRBS_ERR_INVALID, "group_norm: null output");

    cudaStream_t s = as_stream(stream);
    char* const ws = static_cast<char*>(workspace);
    const StatsLayout l = StatsLayout::make(batch, groups);
    const int64_t units = batch * groups;
    float* const shift = reinterpret_cast<float*>(ws + l.shift);
    double* const moments = reinterpret_cast<double*>(ws + l.moments);
    float* const mean = reinterpret_cast<float*>(ws + l.mean);
    float* const inverse = reinterpret_cast<float*>(ws + l.inverse);

    // 1. the common shift: rank 0's first element of every unit, as F32, broadcast
    const size_t unit_pitch = static_cast<size_t>(channels / groups) * static_cast<size_t>(spatial_local) * es;
    if (int rc = cuda_status(cudaMemcpy2DAsync(ws + l.first_raw, es, x_local, unit_pitch, es, static_cast<size_t>(units),
                                               cudaMemcpyDeviceToDevice, s), "gather first elements"))
        return rc;
    if (int rc = kernel_status(vrb_cast(ws + l.first_raw, dtype, shift, VRB_F32, units, stream))) return rc;
    if (comm->world > 1)
        if (int rc = comm->transport->broadcast_f32(shift, static_cast<size_t>(units), 0, s)) return rc;
    // 2. shifted moments of the local slice, summed over the ranks
    if (int rc = kernel_status(vrb_group_norm_moments(x_local, dtype, batch, channels, spatial_local, groups, shift, moments,
                                                      ws + l.partials, l.partial_bytes, stream)))
        return rc;
    if (comm->world > 1)
        if (int rc = comm->transport->all_reduce_sum_f64(moments, static_cast<size_t>(units) * 3, s)) return rc;
    // 3. the same mean / inverse deviation on every rank, then the local normalise pass
    if (int rc = kernel_status(vrb_group_norm_finalize(moments, shift, units, eps, mean, inverse, stream))) return rc;
    if (gather == VRBS_GATHER_PEER) {
        return kernel_status(vrb_group_norm_apply_scatter(x_local, dtype, weight, weight_dtype, bias, bias_dtype, destinations,
                                                          comm->world, batch, channels, frames, rows_local * width,
                                                          rows_full * width, row0 * width, groups, mean, inverse, fuse_silu, stream));
    }
    void* const local_out = gather == VRBS_GATHER_NCCL ? ws + l.staging + static_cast<size_t>(comm->rank) * local_bytes : out;
    if (int rc = kernel_status(vrb_group_norm_apply(x_local, dtype, weight, weight_dtype, bias, bias_dtype, local_out, batch, channels,
                                                    spatial_local, groups, mean, inverse, fuse_silu, stream)))
        return rc;
    if (gather == VRBS_GATHER_NONE) return VRBS_OK;
    // 4. NCCL gather of the slices (in place in the staging area), then one strided placement per rank
    if (int rc = comm->transport->all_gather(local_out, ws + l.staging, local_bytes, s)) return rc;
    const size_t slab = static_cast<size_t>(rows_local * width) * es, full_slab = static_cast<size_t>(rows_full * width) * es;
    for (int r = 0; r < comm->world; ++r) {
        if (int rc = cuda_status(cudaMemcpy2DAsync(static_cast<char*>(out) + static_cast<size_t>(r) * slab, full_slab,
                                                   ws + l.staging + static_cast<size_t>(r) * local_bytes, slab, slab,
                                                   static_cast<size_t>(batch * channels * frames), cudaMemcpyDeviceToDevice, s),
                                 "placement of a gathered slice"))
            return rc;
    }
    return VRBS_OK;
}

extern "C" int vrbs_cfg_euler(vrbs_comm* comm, const void* sample, const void* unconditional, const void* conditional, void* out,
                              int dtype, int64_t count, float scale, float delta, int subtract_prediction, int guidance_role,
                              int solver_role, vrb_stream stream) {
    VRBS_REQUIRE(comm != nullptr, VRBS_ERR_INVALID, "cfg_euler: null communicator");
    if (int rc = comm->refuse_if_aborted("cfg_euler")) return rc;
    VRBS_REQUIRE(sample && unconditional && conditional && out && count > 0, VRBS_ERR_INVALID, "cfg_euler: null tensor");
    VRBS_REQUIRE(dtype == VRB_F32 || dtype == VRB_BF16, VRBS_ERR_INVALID, "cfg_euler: dtype must be F32 or BF16");
    VRBS_REQUIRE(count % (8 * static_cast<int64_t>(comm->world)) == 0, VRBS_ERR_INVALID,
                 "cfg_euler: element count must be a multiple of 8 x world size");
    const int64_t per = count / comm->world;
    const size_t es = element_bytes(dtype), offset = static_cast<size_t>(comm->rank) * static_cast<size_t>(per) * es;
    auto at = [&](const void* base) { return static_cast<const char*>(base) + offset; };
    char* const mine = static_cast<char*>(out) + offset;
    if (int rc = kernel_status(vrb_cfg_euler(at(sample), at(unconditional), at(conditional), nullptr, mine, dtype, per, scale, delta,
                                             subtract_prediction, guidance_role, solver_role, stream)))
        return rc;
    if (comm->world == 1) return VRBS_OK;
    return comm->transport->all_gather(mine, out, static_cast<size_t>(per) * es, as_stream(stream));   // in place
}

extern "C" int vrbs_wait(vrbs_comm* comm, vrb_stream stream) {
    VRBS_REQUIRE(comm != nullptr, VRBS_ERR_INVALID, "wait: null communicator");
    if (int rc = comm->refuse_if_aborted("wait")) return rc;
    if (int rc = cuda_status(cudaEventRecord(comm->done, as_stream(stream)), "event record")) return rc;
    return comm->bounded_wait([&](bool* failed) {
        const cudaError_t e = cudaEventQuery(comm->done);
        if (e == cudaErrorNotReady) return true;
        *failed = e != cudaSuccess;
        return false;
    });
}

extern "C" int vrbs_watchdog_selftest(int timeout_ms, int64_t* report4) {
    VRBS_REQUIRE(report4 != nullptr && timeout_ms > 0, VRBS_ERR_INVALID, "watchdog_selftest: bad arguments");
    vrbs_comm comm;
    auto* silent = new SilentPeerTransport;
    comm.transport.reset(silent);
    comm.rank = 0;
    comm.world = 2;
    comm.timeout_ms = timeout_ms;
    const auto begin = std::chrono::steady_clock::now();
    report4[0] = comm.bounded_wait([](bool*) { return true; });   // the peer never joins: the work never completes
    report4[1] = std::chrono::duration_cast<std::chrono::milliseconds>(std::chrono::steady_clock::now() - begin).count();
    report4[2] = silent->aborts;
    report4[3] = vrbs_cfg_euler(&comm, &comm, &comm, &comm, &comm, VRB_F32, 16, 1.f, 1.f, 1, 0, 0, nullptr);   // refused before any use
    return VRBS_OK;
}
