// C wrapper around the REFERENCE's own CUDA backend, compiled from the reference's sources
// where they lie (see oracle/Makefile).  TEST INFRASTRUCTURE ONLY: it exists to produce golden
// vectors from, and to time, the reference's real kernels on the same GPU.  This file contains
// no reference code; it only calls the reference's public interfaces:
//   vrhino::CudaBackend            native/include/vrhino/backend/cuda_backend.h
//   helper seams                   native/include/vrhino/architecture.h:63-86
//   vrhino::SamplingPrimitives     native/include/vrhino/sampling.h:171-203
//   vrhino::PrecisionPolicy        native/include/vrhino/precision.h:95-140
// Tensors are kept in a handle table so chains stay on the device between calls.
//
// Compiled a second time with -DVRB_DROPIN (libvrhino_dropin_cuda.so) the SAME calls drive
// vrhino_b200::B200Backend wrapped around the reference's CudaBackend: the reference's unmodified
// helper code (modulate, gated_residual, SamplingPrimitives ...) then runs on this repository's
// kernels, which is the drop-in claim under test; the refd_* entry points reach the fused forms.
#include <cstdint>
#include <cstring>
#include <map>
#include <memory>
#include <string>
#include <vector>

#include "vrhino/architecture.h"
#include "vrhino/backend/cuda_backend.h"
#include "vrhino/error.h"
#include "vrhino/precision.h"
#include "vrhino/sampling.h"
#include "vrhino/tensor_util.h"
#include "runtime/neural_graph.h"
#include "architectures/wan_self_attention_graph.h"
#include "architectures/ltx_self_attention_graph.h"
#ifdef VRB_DROPIN
#include "b200_backend.h"
#include "graph_fusion.h"
#endif

using namespace vrhino;

namespace {
#ifdef VRB_DROPIN
std::unique_ptr<vrhino_b200::B200Backend> g_backend;
#else
std::unique_ptr<CudaBackend> g_backend;
#endif
std::map<int64_t, Tensor> g_tensors;
int64_t g_next = 1;
std::string g_error;

int64_t keep(Tensor t) { g_tensors[g_next] = std::move(t); return g_next++; }
const Tensor& at(int64_t h) {
    auto it = g_tensors.find(h);
    require(it != g_tensors.end(), "unknown tensor handle");
    return it->second;
}
const Tensor* opt(int64_t h) { return h ? &at(h) : nullptr; }

PrecisionPolicy policy_of(int id) {
    // 0: unqualified_default(BF16) (residual bf16)   1: fp32() (residual F32)
    // 2: 0 + guidance/solver/sigma scalar roles      3: 0 + guidance role only
    PrecisionPolicy base = id == 1 ? PrecisionPolicy::fp32() : PrecisionPolicy::unqualified_default(DType::BF16);
    if (id == 2)
        return base.with_scalar_roles({PrecisionScalarRole::GuidanceCoefficient, PrecisionScalarRole::SolverCoefficient,
                                       PrecisionScalarRole::Sigma});
    if (id == 3) return base.with_scalar_roles({PrecisionScalarRole::GuidanceCoefficient});
    return base;
}

template <typename F>
int64_t guarded(F&& f) {
    try {
        require(g_backend != nullptr, "refc_init was not called");
        return f();
    } catch (const std::exception& e) {
        g_error = e.what();
        return -1;
    }
}
}  // namespace

extern "C" {

const char* refc_last_error() { return g_error.c_str(); }

int refc_init(int execution_dtype) {
    try {
#ifdef VRB_DROPIN
        if (!g_backend) g_backend = std::make_unique<vrhino_b200::B200Backend>(std::make_unique<CudaBackend>());
#else
        if (!g_backend) g_backend = std::make_unique<CudaBackend>();
#endif
        g_backend->set_execution_dtype(static_cast<DType>(execution_dtype));
        return 0;
    } catch (const std::exception& e) { g_error = e.what(); return -1; }
}
void refc_shutdown() { g_tensors.clear(); g_backend.reset(); }
void refc_free(int64_t h) { g_tensors.erase(h); }
void refc_clear() { g_tensors.clear(); }
void refc_synchronize() { if (g_backend) g_backend->synchronize(); }

// host payload (dtype of the payload = dtype) -> device tensor of the same dtype
int64_t refc_upload(const void* host, int dtype, int rank, const int64_t* shape) {
    return guarded([&] {
        std::vector<int64_t> s(shape, shape + rank);
        Tensor h = Tensor::host(s, static_cast<DType>(dtype));
        std::memcpy(h.data(), host, h.bytes());
        return keep(g_backend->copy_to_device(h, static_cast<DType>(dtype)));
    });
}
// host F32 payload kept on the HOST side (the reference's weights / scalars start there)
int64_t refc_host_f32(const float* host, int rank, const int64_t* shape) {
    return guarded([&] {
        std::vector<int64_t> s(shape, shape + rank);
        Tensor h = Tensor::host(s, DType::F32);
        std::memcpy(h.data(), host, h.bytes());
        return keep(h);
    });
}
int refc_dtype(int64_t h) { return static_cast<int>(guarded([&] { return static_cast<int64_t>(at(h).dtype()); })); }
int64_t refc_numel(int64_t h) { return guarded([&] { return at(h).numel(); }); }
int refc_download(int64_t h, void* host, int64_t bytes) {
    return static_cast<int>(guarded([&] {
        Tensor t = g_backend->copy_to_host(at(h));
        require(static_cast<int64_t>(t.bytes()) == bytes, "download size mismatch");
        std::memcpy(host, t.data(), t.bytes());
        return int64_t{0};
    }));
}

int64_t refc_binary(int kind, int64_t a, int64_t b) {
    return guarded([&] {
        switch (kind) {
            case 0: return keep(g_backend->add(at(a), at(b)));
            case 1: return keep(g_backend->mul(at(a), at(b)));
            case 2: return keep(g_backend->div(at(a), at(b)));
            default: return keep(g_backend->maximum(at(a), at(b)));
        }
    });
}
int64_t refc_cast(int64_t x, int dtype) { return guarded([&] { return keep(g_backend->cast(at(x), static_cast<DType>(dtype))); }); }
int64_t refc_reshape(int64_t x, int rank, const int64_t* shape) {
    return guarded([&] { return keep(g_backend->reshape(at(x), std::vector<int64_t>(shape, shape + rank))); });
}
int64_t refc_slice(int64_t x, int64_t dim, int64_t start, int64_t stop) {
    return guarded([&] { return keep(g_backend->slice(at(x), dim, start, stop)); });
}
int64_t refc_permute(int64_t x, int rank, const int64_t* dims) {
    return guarded([&] { return keep(g_backend->permute(at(x), std::vector<int64_t>(dims, dims + rank))); });
}
int64_t refc_concat(const int64_t* handles, int count, int64_t dim) {
    return guarded([&] {
        std::vector<Tensor> parts;
        for (int k = 0; k < count; ++k) parts.push_back(at(handles[k]));
        return keep(g_backend->concat(parts, dim));
    });
}
// padding: the reference's vector of (before, after) pairs from the innermost axis outwards
int64_t refc_pad(int64_t x, int entries, const int64_t* padding, float value, int replicate) {
    return guarded([&] {
        return keep(g_backend->pad(at(x), std::vector<int64_t>(padding, padding + entries), value,
                                   replicate ? vrhino::PadMode::Replicate : vrhino::PadMode::Constant));
    });
}
int64_t refc_interpolate_nearest(int64_t x, int count, const double* factors) {
    return guarded([&] { return keep(g_backend->interpolate_nearest(at(x), std::vector<double>(factors, factors + count))); });
}
int64_t refc_reduce_sum(int64_t x, int64_t dim, int keepdim) {
    return guarded([&] { return keep(g_backend->reduce_sum(at(x), dim, keepdim != 0)); });
}
// one call of rng_normal on a fresh RngState{seed, offset}
int64_t refc_rng_normal(uint64_t seed, uint64_t offset, int rank, const int64_t* shape, int dtype) {
    return guarded([&] {
        RngState state{seed, offset, "pytorch_compat.v1"};
        Tensor made = g_backend->rng_normal(state, std::vector<int64_t>(shape, shape + rank), static_cast<DType>(dtype));
        require(state.offset == offset + 4, "RNG offset mismatch");
        return keep(made);
    });
}
int64_t refc_softmax(int64_t x, int64_t axis) { return guarded([&] { return keep(g_backend->softmax(at(x), axis)); }); }
// indices: host values of `index_bits` (64 or 32) bits each, shape [rank]; handed over as a host tensor, as the callers do
int64_t refc_indexed_gather(int64_t table, int index_bits, int rank, const int64_t* shape, const void* indices) {
    return guarded([&] {
        Tensor h = Tensor::host(std::vector<int64_t>(shape, shape + rank), index_bits == 64 ? DType::I64 : DType::I32);
        std::memcpy(h.data(), indices, h.bytes());
        return keep(g_backend->indexed_gather(at(table), h));
    });
}
int64_t refc_sinusoidal(int64_t positions, int64_t width, int flip, double downscale, int frequency_f64) {
    return guarded([&] { return keep(g_backend->sinusoidal_embedding(at(positions), width, flip != 0, downscale, frequency_f64 != 0)); });
}
int64_t refc_layer_norm(int64_t x, int64_t w, int64_t b, float eps) {
    return guarded([&] { return keep(g_backend->layer_norm(at(x), opt(w), opt(b), eps)); });
}
// out_dtype < 0: the reference's default (same as the input)
int64_t refc_rms_norm(int64_t x, int64_t w, float eps, int64_t axis, int out_dtype) {
    return guarded([&] {
        return keep(g_backend->rms_norm(at(x), opt(w), eps, axis, out_dtype < 0 ? DType::F16 : static_cast<DType>(out_dtype)));
    });
}
// CudaBackend::linear with its defaults (execution dtype compute and output): bf16 GEMM, F32
// accumulation, fused_bf16_linear_output_kernel
int64_t refc_linear(int64_t x, int64_t w, int64_t bias) {
    return guarded([&] { return keep(g_backend->linear(at(x), at(w), opt(bias))); });
}
int64_t refc_pixel_norm(int64_t x, int64_t dim, float eps) {
    return guarded([&] { return keep(g_backend->pixel_norm(at(x), dim, eps)); });
}
int64_t refc_l2_normalize(int64_t x, int64_t dim, float eps) {
    return guarded([&] { return keep(g_backend->l2_normalize(at(x), dim, eps)); });
}
int64_t refc_pixel_shuffle(int64_t x, int64_t ft, int64_t fh, int64_t fw) {
    return guarded([&] { return keep(g_backend->pixel_shuffle_nd(at(x), {ft, fh, fw})); });
}
// concat of `copies` references to the same tensor along `dim`
int64_t refc_repeat(int64_t x, int copies, int64_t dim) {
    return guarded([&] { return keep(g_backend->concat(std::vector<Tensor>(static_cast<size_t>(copies), at(x)), dim)); });
}
int64_t refc_activation(int64_t x, int kind) {
    return guarded([&] { return keep(g_backend->activation(at(x), static_cast<Activation>(kind))); });
}
int64_t refc_rope(int64_t x, int64_t c, int64_t s) { return guarded([&] { return keep(g_backend->rope_nd(at(x), at(c), at(s))); }); }
int64_t refc_group_norm(int64_t x, int groups, int64_t w, int64_t b, float eps) {
    return guarded([&] { return keep(g_backend->group_norm(at(x), groups, opt(w), opt(b), eps)); });
}
int64_t refc_clamp(int64_t x, float lo, float hi) { return guarded([&] { return keep(g_backend->clamp(at(x), lo, hi)); }); }
int64_t refc_exp(int64_t x) { return guarded([&] { return keep(g_backend->exp(at(x))); }); }
int64_t refc_sqrt(int64_t x) { return guarded([&] { return keep(g_backend->sqrt(at(x))); }); }

// quantized weight: packed bytes + F32 scales on the host -> dequantised device tensor
int64_t refc_dequantize(int type, const uint8_t* packed, int64_t packed_bytes, const float* scales, int64_t rows,
                        int64_t inner, int64_t group_size, int out_dtype) {
    return guarded([&] {
        auto payload = std::make_shared<std::vector<uint8_t>>(packed, packed + packed_bytes);
        Tensor weight = Tensor::borrowed(payload->data(), payload->size(), {rows, inner}, DType::U8);
        auto info = std::make_shared<QuantizationInfo>();
        info->type = type == 0 ? QuantType::FP8E4M3FN : type == 1 ? QuantType::INT8Symmetric : QuantType::INT4Symmetric;
        info->logical_dtype = DType::BF16; info->compute_dtype = DType::BF16; info->accumulation_dtype = DType::F32;
        info->group_size = group_size; info->axis = 1; info->symmetric = true;
        info->granularity = group_size == inner ? "per_channel" : "per_group";
        info->zero_point_mode = "none";
        info->packing_layout = type == 0 ? "byte_e4m3fn" : type == 1 ? "byte_twos_complement" : "nibble_low_first_twos_complement";
        const int64_t groups = (inner + group_size - 1) / group_size;
        info->scales = host_f32({rows, groups}, std::vector<float>(scales, scales + rows * groups));
        weight.set_quantization(info);
        Tensor out = g_backend->copy_to_device(weight, static_cast<DType>(out_dtype));
        g_backend->synchronize();   // payload must outlive the upload
        return keep(out);
    });
}

// ---- helper seams -------------------------------------------------------------------------
int64_t refc_modulate(int policy, int64_t x, int64_t shift, int64_t scale) {
    return guarded([&] { return keep(modulate(*g_backend, policy_of(policy), at(x), at(shift), at(scale))); });
}
int64_t refc_attention_norm(int policy, int64_t x, int64_t w, float eps, int64_t axis) {
    return guarded([&] { return keep(attention_norm(*g_backend, policy_of(policy), at(x), opt(w), eps, axis)); });
}
int64_t refc_operation_rope(int policy, int64_t x, int64_t c, int64_t s) {
    return guarded([&] { return keep(operation_rope(*g_backend, policy_of(policy), at(x), at(c), at(s))); });
}
int64_t refc_residual_add(int policy, int64_t r, int64_t b) {
    return guarded([&] { return keep(residual_add(*g_backend, policy_of(policy), at(r), at(b))); });
}
int64_t refc_gated_residual(int policy, int64_t r, int64_t b, int64_t g) {
    return guarded([&] { return keep(gated_residual(*g_backend, policy_of(policy), at(r), at(b), at(g))); });
}
int64_t refc_cfg_combine(int policy, int64_t u, int64_t c, float scale) {
    return guarded([&] { SamplingPrimitives p(*g_backend, policy_of(policy)); return keep(p.cfg_combine(at(u), at(c), scale)); });
}
int64_t refc_euler_update(int policy, int64_t x, int64_t pred, float delta, int subtract) {
    return guarded([&] {
        SamplingPrimitives p(*g_backend, policy_of(policy));
        return keep(p.euler_update(at(x), at(pred), scalar_f32(delta), subtract != 0));
    });
}
int64_t refc_flow_to_x0(int policy, int64_t x, int64_t out, float sigma) {
    return guarded([&] { SamplingPrimitives p(*g_backend, policy_of(policy)); return keep(p.flow_to_x0(at(x), at(out), sigma)); });
}

#ifdef VRB_DROPIN
// ---- fused forms of the drop-in backend (call-site view of vrhino_b200/host/b200_backend.h) ---
const char* refc_backend_name() { static std::string n; n = g_backend ? g_backend->name() : ""; return n.c_str(); }
int64_t refd_layer_norm_modulate(int policy, int64_t x, int64_t w, int64_t b, float eps, int64_t shift, int64_t scale, int out_dtype) {
    return guarded([&] {
        return keep(vrhino_b200::layer_norm_modulate(*g_backend, policy_of(policy), at(x), opt(w), opt(b), eps, at(shift), at(scale),
                                                     static_cast<DType>(out_dtype)));
    });
}
int64_t refd_rms_norm_rope(int policy, int64_t x, int64_t w, float eps, int64_t c, int64_t s, int heads, int per_head, int out_dtype) {
    return guarded([&] {
        return keep(vrhino_b200::rms_norm_rope(*g_backend, policy_of(policy), at(x), opt(w), eps, opt(c), opt(s), heads, per_head != 0,
                                               static_cast<DType>(out_dtype)));
    });
}
// {q operand, k operand} of one pair launch; returns the first handle, *second receives the other
int64_t refd_rms_norm_rope_pair(int policy, int64_t q, int64_t wq, int64_t k, int64_t wk, float eps, int64_t c, int64_t s, int heads,
                                int per_head, int out_dtype, int64_t* second) {
    return guarded([&] {
        auto both = vrhino_b200::rms_norm_rope_pair(*g_backend, policy_of(policy), at(q), at(wq), at(k), at(wk), eps, opt(c), opt(s),
                                                    heads, per_head != 0, static_cast<DType>(out_dtype));
        *second = keep(both.second);
        return keep(both.first);
    });
}
// Mochi's layer boundary: returns the updated stream's handle, *normed receives the next layer's pre-norm
int64_t refd_mochi_residual_norm(int policy, int64_t r, int64_t b, int64_t g, int64_t scale, float eps, int64_t* normed) {
    return guarded([&] {
        auto both = vrhino_b200::normalized_gated_residual_norm_scale(*g_backend, policy_of(policy), at(r), at(b), at(g), at(scale), eps);
        *normed = keep(both.second);
        return keep(both.first);
    });
}
int64_t refd_gated_residual(int policy, int64_t r, int64_t b, int64_t g) {
    return guarded([&] { return keep(vrhino_b200::fused_gated_residual(*g_backend, policy_of(policy), at(r), at(b), opt(g))); });
}
// Returns the normalised tensor's handle; *state_handle receives the updated residual stream's.
int64_t refd_gated_residual_layer_norm(int policy, int64_t r, int64_t b, int64_t g, int64_t w, int64_t bias, float eps,
                                       int64_t shift, int64_t scale, int out_dtype, int64_t* state_handle) {
    return guarded([&] {
        auto both = vrhino_b200::fused_gated_residual_layer_norm(*g_backend, policy_of(policy), at(r), at(b), opt(g), opt(w),
                                                                 opt(bias), eps, opt(shift), opt(scale),
                                                                 static_cast<DType>(out_dtype));
        *state_handle = keep(both.first);
        return keep(both.second);
    });
}
int64_t refd_linear_activation(int64_t x, int64_t w, int64_t bias, int kind) {
    return guarded([&] {
        return keep(vrhino_b200::linear_activation(*g_backend, at(x), at(w), opt(bias), static_cast<Activation>(kind)));
    });
}
int64_t refd_linear_gated_residual(int policy, int64_t r, int64_t x, int64_t w, int64_t bias, int64_t g) {
    return guarded([&] {
        return keep(vrhino_b200::linear_gated_residual(*g_backend, policy_of(policy), at(r), at(x), at(w), opt(bias), opt(g)));
    });
}
int64_t refd_linear_swiglu(int64_t x, int64_t w, int64_t bias) {
    return guarded([&] { return keep(vrhino_b200::linear_swiglu(*g_backend, at(x), at(w), opt(bias))); });
}
int64_t refd_pixel_norm_modulate_silu(int policy, int64_t x, int64_t shift, int64_t scale, float eps, int out_dtype) {
    return guarded([&] {
        return keep(vrhino_b200::pixel_norm_modulate_silu(*g_backend, policy_of(policy), at(x), at(shift), at(scale), eps,
                                                          static_cast<DType>(out_dtype)));
    });
}
int64_t refd_edge_time_pad(int64_t x, int64_t temporal, int64_t pad_h, int64_t pad_w) {
    return guarded([&] { return keep(vrhino_b200::edge_time_pad(*g_backend, at(x), temporal, pad_h, pad_w)); });
}
int64_t refd_depth_to_space_residual(int64_t projected, int64_t input) {
    return guarded([&] { return keep(vrhino_b200::depth_to_space_residual(*g_backend, at(projected), at(input))); });
}
int64_t refd_swiglu(int64_t x) { return guarded([&] { return keep(vrhino_b200::swiglu(*g_backend, at(x))); }); }
int64_t refd_group_norm_silu(int64_t x, int groups, int64_t w, int64_t b, float eps) {
    return guarded([&] { return keep(vrhino_b200::group_norm_silu(*g_backend, at(x), groups, opt(w), opt(b), eps)); });
}
int64_t refd_cfg_euler(int64_t x, int64_t u, int64_t c, float guidance, float delta, int subtract, int guidance_role, int solver_role) {
    return guarded([&] {
        return keep(g_backend->cfg_euler(at(x), at(u), at(c), guidance, delta, subtract != 0, guidance_role != 0, solver_role != 0));
    });
}
// profile_stats() of the wrapped backend as text, one "name\tcalls\tdevice ms\tbytes" line per entry
// (bytes from B200Backend::profile_bytes(), 0 for entries the device runtime recorded itself).
int64_t refd_profile_report(char* buffer, int64_t capacity) {
    return guarded([&] {
        std::string text;
        const auto& bytes = g_backend->profile_bytes();
        for (const auto& [name, stat] : g_backend->profile_stats()) {
            const auto found = bytes.find(name);
            text += name + "\t" + std::to_string(stat.calls) + "\t" + std::to_string(stat.device_milliseconds) + "\t" +
                    std::to_string(found == bytes.end() ? 0 : found->second) + "\n";
        }
        require(static_cast<int64_t>(text.size()) < capacity, "profile report buffer too small");
        std::memcpy(buffer, text.c_str(), text.size() + 1);
        return static_cast<int64_t>(text.size());
    });
}
// ONE quantised host weight uploaded `repeats` times (what linear() does with a quantised weight on
// every call, cuda_backend.cu:3276-3295); stats = {cache hits, misses, resident bytes} of the
// dequantised-weight cache afterwards.  budget < 0 keeps the current budget.
int64_t refd_dequantize_repeated(int type, const uint8_t* packed, int64_t packed_bytes, const float* scales, int64_t rows,
                                 int64_t inner, int64_t group_size, int out_dtype, int repeats, int64_t budget, int64_t* stats) {
    return guarded([&] {
        if (budget >= 0) g_backend->set_dequantized_cache_budget(static_cast<size_t>(budget));
        static std::vector<std::shared_ptr<std::vector<uint8_t>>> payloads;   // host weights outlive their cache entries
        auto payload = std::make_shared<std::vector<uint8_t>>(packed, packed + packed_bytes);
        payloads.push_back(payload);
        Tensor weight = Tensor::borrowed(payload->data(), payload->size(), {rows, inner}, DType::U8);
        auto info = std::make_shared<QuantizationInfo>();
        info->type = type == 0 ? QuantType::FP8E4M3FN : type == 1 ? QuantType::INT8Symmetric : QuantType::INT4Symmetric;
        info->logical_dtype = DType::BF16; info->compute_dtype = DType::BF16; info->accumulation_dtype = DType::F32;
        info->group_size = group_size; info->axis = 1; info->symmetric = true;
        info->granularity = group_size == inner ? "per_channel" : "per_group";
        info->zero_point_mode = "none";
        info->packing_layout = type == 0 ? "byte_e4m3fn" : type == 1 ? "byte_twos_complement" : "nibble_low_first_twos_complement";
        const int64_t groups = (inner + group_size - 1) / group_size;
        info->scales = host_f32({rows, groups}, std::vector<float>(scales, scales + rows * groups));
        weight.set_quantization(info);
        Tensor out;
        for (int i = 0; i < repeats; ++i) out = g_backend->copy_to_device(weight, static_cast<DType>(out_dtype));
        g_backend->synchronize();
        stats[0] = static_cast<int64_t>(g_backend->dequantized_cache_hits());
        stats[1] = static_cast<int64_t>(g_backend->dequantized_cache_misses());
        stats[2] = static_cast<int64_t>(g_backend->dequantized_cache_resident_bytes());
        return keep(out);
    });
}
int64_t refd_release_cached() {
    return guarded([&] {
        g_backend->release_cached_device_memory();
        return static_cast<int64_t>(g_backend->dequantized_cache_resident_bytes());
    });
}
// An operator failure must leave the session terminal, like the reference's (memory.h:225-236).
int refd_session_terminal() { return g_backend && g_backend->resource_session_terminal() ? 1 : 0; }
#else
const char* refc_backend_name() { static std::string n; n = g_backend ? g_backend->name() : ""; return n.c_str(); }
#endif

// frame_group_norm of native/src/architectures/mochi.cpp:365-371 (+ SiLU): the reference's permute ->
// group_norm -> permute on its backend, or, in the drop-in build, vrhino_b200::frame_group_norm
// (one pass over the unpermuted tensor).
int64_t refc_frame_group_norm(int64_t x, int groups, int64_t w, int64_t b, float eps, int silu) {
    return guarded([&] {
#ifdef VRB_DROPIN
        return keep(vrhino_b200::frame_group_norm(*g_backend, at(x), groups, opt(w), opt(b), eps, silu != 0));
#else
        const Tensor& input = at(x);
        const int64_t n = input.dim(0), c = input.dim(1), t = input.dim(2), h = input.dim(3), wd = input.dim(4);
        Tensor frames = g_backend->reshape(g_backend->permute(input, {0, 2, 1, 3, 4}), {n * t, c, h, wd});
        frames = g_backend->group_norm(frames, groups, opt(w), opt(b), eps);
        Tensor out = g_backend->permute(g_backend->reshape(frames, {n, t, c, h, wd}), {0, 2, 1, 3, 4});
        return keep(silu ? g_backend->activation(out, Activation::Silu) : out);
#endif
    });
}

// ---- executable graphs (native/src/runtime/neural_graph.h) ------------------------------------
// The non-GEMM part of the Wan self-attention graph (native/src/architectures/
// wan_self_attention_graph.h:46-70), node for node, with the GEMM / attention results (q, k and
// the attention projection) supplied as inputs: modulation table + input -> slices; LayerNorm ->
// [Cast] -> Mul(1 + scale) -> Add(shift) -> Cast; RmsNorm -> Reshape -> Rope -> Cast for q and k;
// Cast -> Mul(gate) -> Add(residual).  Outputs: attention input, q, k operands, first residual.
namespace {
neural_graph::Graph wan_chain_graph(int64_t s, int64_t width, int64_t heads_count, DType execution, DType hidden_dtype, float eps) {
    namespace ng = neural_graph;
    const int64_t b = 1, head_width = width / heads_count;
    const std::vector<int64_t> hidden{b, s, width}, part{b, 1, width}, heads{b, s, heads_count, head_width};
    ng::Description d;
    d.schema = ng::schema_v1;
    d.execution_dtype = execution;
    // 0 hidden, 1 modulation, 2 cos, 3 sin, 4 q, 5 k, 6 projection | 7 table, 8 norm_q, 9 norm_k | 10 one
    d.values = {{hidden, hidden_dtype}, {{b, 6, width}}, {{1, s, 1, head_width}}, {{1, s, 1, head_width}},
                {hidden, execution}, {hidden, execution}, {hidden, execution},
                {{1, 6, width}}, {{width}}, {{width}}, {{1}}};
    d.inputs = {0, 1, 2, 3, 4, 5, 6};
    d.parameters = {7, 8, 9};
    d.constants = {{10, 1.0f}};
    auto node = [&](ng::Primitive op, const std::vector<int64_t>& shape, DType dtype = DType::F32) {
        auto id = static_cast<ng::ValueId>(d.values.size());
        d.values.push_back({shape, dtype});
        d.nodes.push_back({id, std::move(op)});
        return id;
    };
    auto cast = [&](ng::ValueId x, DType dtype) { return d.values[x].dtype == dtype ? x : node(ng::Cast{x, dtype}, d.values[x].shape, dtype); };
    auto combined = node(ng::Add{7, 1}, {b, 6, width});
    auto shift = node(ng::Slice{combined, 1, 0, 1}, part);
    auto scale = node(ng::Slice{combined, 1, 1, 2}, part);
    auto gate = node(ng::Slice{combined, 1, 2, 3}, part);
    auto norm = node(ng::LayerNorm{0, {}, {}, eps}, hidden, hidden_dtype);
    auto scale_one = node(ng::Add{10, scale}, part);
    auto scaled = node(ng::Mul{cast(norm, DType::F32), scale_one}, hidden);
    auto self_input = node(ng::Add{scaled, shift}, hidden);
    auto operand = cast(self_input, execution);
    auto q_norm = node(ng::RmsNorm{4, 8, 2, eps}, hidden);
    auto k_norm = node(ng::RmsNorm{5, 9, 2, eps}, hidden);
    auto q_heads = node(ng::Reshape{q_norm, heads}, heads);
    auto k_heads = node(ng::Reshape{k_norm, heads}, heads);
    auto q_rope = node(ng::Rope{q_heads, 2, 3}, heads);
    auto k_rope = node(ng::Rope{k_heads, 2, 3}, heads);
    auto q_operand = cast(q_rope, execution), k_operand = cast(k_rope, execution);
    auto gated = node(ng::Mul{cast(6, DType::F32), gate}, hidden);
    auto residual = node(ng::Add{cast(0, DType::F32), gated}, hidden);
    d.outputs = {operand, q_operand, k_operand, residual};
    return ng::admit(d);
}
}  // namespace

// handles: hidden, modulation, cos, sin, q, k, projection, table, norm_q, norm_k (10); out: 4 handles.
// fused != 0 (drop-in build only) runs vrhino_b200::evaluate_fused (fused == 2: without the per-graph
// device synchronisation); stats (may be null) receives
// {layer_norm_modulate, rms_norm_rope, gated_residual, nodes_total, nodes_absorbed}.
int refc_wan_chain_graph(int64_t s, int64_t width, int64_t heads, int hidden_dtype, float eps, const int64_t* handles,
                         int fused, int64_t* out, int* stats) {
    return static_cast<int>(guarded([&] {
        const auto graph = wan_chain_graph(s, width, heads, g_backend->execution_dtype(), static_cast<DType>(hidden_dtype), eps);
        std::vector<Tensor> inputs, parameters;
        for (int i = 0; i < 7; ++i) inputs.push_back(at(handles[i]));
        for (int i = 7; i < 10; ++i) parameters.push_back(at(handles[i]));
        std::vector<Tensor> results;
        if (fused) {
#ifdef VRB_DROPIN
            vrhino_b200::FusionStats fs;
            results = vrhino_b200::evaluate_fused(*g_backend, graph, inputs, parameters, &fs, fused != 2);
            if (stats) { stats[0] = fs.layer_norm_modulate; stats[1] = fs.rms_norm_rope; stats[2] = fs.gated_residual;
                         stats[3] = fs.nodes_total; stats[4] = fs.nodes_absorbed; }
#else
            throw Error("the fused evaluator exists only in the drop-in build");
#endif
        } else {
            results = neural_graph::evaluate(*g_backend, graph, inputs, parameters);
        }
        for (size_t i = 0; i < results.size(); ++i) out[i] = keep(results[i]);
        return int64_t{0};
    }));
}

// The reference's production Wan self-attention graph itself (wan_self_attention_graph.h:22-72),
// GEMMs and attention included.  handles: hidden, modulation, cos, sin, then the 11 parameters in
// the header's canonical order, already on the device in the dtypes the graph declares.
// out: {first residual, combined modulation}.
int refc_wan_self_attention_graph(int64_t s, int64_t width, int64_t heads, const int64_t* handles, int fused, int64_t* out,
                                  int* stats) {
    return static_cast<int>(guarded([&] {
        wan_family::Config config;
        config.dim = width; config.heads = heads;
        const Tensor& hidden = at(handles[0]);
        const auto graph = wan_internal::self_attention_graph(1, s, g_backend->execution_dtype(), hidden.dtype(), false, config);
        std::vector<Tensor> inputs, parameters;
        for (int i = 0; i < 4; ++i) inputs.push_back(at(handles[i]));
        for (int i = 4; i < 15; ++i) parameters.push_back(at(handles[i]));
        std::vector<Tensor> results;
        if (fused) {
#ifdef VRB_DROPIN
            vrhino_b200::FusionStats fs;
            results = vrhino_b200::evaluate_fused(*g_backend, graph, inputs, parameters, &fs);
            if (stats) { stats[0] = fs.layer_norm_modulate; stats[1] = fs.rms_norm_rope; stats[2] = fs.gated_residual;
                         stats[3] = fs.nodes_total; stats[4] = fs.nodes_absorbed; }
#else
            throw Error("the fused evaluator exists only in the drop-in build");
#endif
        } else {
            results = neural_graph::evaluate(*g_backend, graph, inputs, parameters);
        }
        for (size_t i = 0; i < results.size(); ++i) out[i] = keep(results[i]);
        return int64_t{0};
    }));
}

// The reference's production LTX self-attention graph (ltx_self_attention_graph.cpp:10-82; width
// 2048, 32 heads), GEMMs and attention included.  handles: hidden, modulation, cos, sin, then the 11
// parameters in the header's order, on the device in the dtypes the BF16 contracts declare.
int refc_ltx_self_attention_graph(int64_t b, int64_t s, int hidden_bf16, const int64_t* handles, int fused, int64_t* out,
                                  int* stats) {
    return static_cast<int>(guarded([&] {
        const auto contract = hidden_bf16 ? ltx_internal::SelfAttentionContract::BF16Hidden
                                          : ltx_internal::SelfAttentionContract::BF16F32Hidden;
        const auto graph = ltx_internal::self_attention_graph(b, s, 1, false, false, contract);
        std::vector<Tensor> inputs, parameters;
        for (int i = 0; i < 4; ++i) inputs.push_back(at(handles[i]));
        for (int i = 4; i < 15; ++i) parameters.push_back(at(handles[i]));
        std::vector<Tensor> results;
        if (fused) {
#ifdef VRB_DROPIN
            vrhino_b200::FusionStats fs;
            results = vrhino_b200::evaluate_fused(*g_backend, graph, inputs, parameters, &fs);
            if (stats) { stats[0] = fs.rms_norm_modulate; stats[1] = fs.rms_norm_rope; stats[2] = fs.gated_residual;
                         stats[3] = fs.nodes_total; stats[4] = fs.nodes_absorbed; }
#else
            throw Error("the fused evaluator exists only in the drop-in build");
#endif
        } else {
            results = neural_graph::evaluate(*g_backend, graph, inputs, parameters);
        }
        out[0] = keep(results[0]);
        return int64_t{0};
    }));
}

// ---- timing through the reference's own profiler ---------------------------------------------
void refc_profile(int enabled) { if (g_backend) g_backend->enable_profiling(enabled != 0); }
// Cumulative device milliseconds and call count over every profile entry recorded since
// profiling was switched on (the reference keeps its aggregates; callers take differences).
double refc_profile_total_ms(int64_t* calls) {
    double total = 0.0;
    int64_t n = 0;
    try {
        for (const auto& [name, stat] : g_backend->profile_stats()) {
            if (name.rfind("reference.", 0) == 0) continue;
            total += stat.device_milliseconds;
            n += static_cast<int64_t>(stat.calls);
        }
    } catch (const std::exception& e) { g_error = e.what(); return -1.0; }
    if (calls) *calls = n;
    return total;
}

}  // extern "C"
