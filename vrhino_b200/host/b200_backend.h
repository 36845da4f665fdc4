// C++ host layer of the B200 operator path: a vrhino::Backend whose elementwise, reduction and
// broadcast operators run on the sm_100a kernels of libvrb.so (include/vrb.h), plus the fused
// forms of the helper seams.  It compiles against the reference's public headers
// (native/include/vrhino) and is meant to be built inside the reference's tree, next to
// native/src/backend/cuda/cuda_backend.cu.
//
// Everything that is not on this path -- allocation and the temporary pool, host<->device
// transfers and fences, GEMM, attention, convolutions, the memory runtime, the profiler itself -- is
// forwarded to the device runtime backend given at construction (normally the reference's own
// CudaBackend), so call sites that hold a `Backend&` (native/include/vrhino/architecture.h:33-42)
// need no change: construct B200Backend(std::make_unique<CudaBackend>()) where they used to
// construct CudaBackend.
//
// Replaced virtuals (same signatures, defaults, dtype rules and error texts as
// native/src/backend/cuda/cuda_backend.cu): add, mul, div, maximum (:3871-3902), cast (:3978),
// layer_norm (:4057), rms_norm (:4091), activation (:4179), rope_nd (:4198), group_norm (:4919),
// clamp (:5128), exp, sqrt (:5134-5173), pixel_norm (:5048), l2_normalize (:5088), pixel_shuffle_nd (:5112),
// permute / concat / split / slice (:3936-3976), sinusoidal_embedding (:4190), pad (:4875)
// and the quantised branch of copy_to_device (:3214-3296).
// Kernels run on the legacy default stream, which the runtime's pool reuse relies on
// (cuda_backend.cu:55-59).
#pragma once

#include <map>
#include <memory>
#include <utility>
#include <string>
#include <vector>

#include "vrhino/backend.h"
#include "vrhino/precision.h"

namespace vrhino_b200 {

class B200Backend final : public vrhino::Backend {
public:
    using Tensor = vrhino::Tensor;
    using DType = vrhino::DType;

    explicit B200Backend(std::unique_ptr<vrhino::Backend> device_runtime);
    ~B200Backend() override;
    vrhino::Backend& device_runtime() { return *rt_; }

    // ---- operators on this path -------------------------------------------------------------
    Tensor add(const Tensor& a, const Tensor& b) override;
    Tensor mul(const Tensor& a, const Tensor& b) override;
    Tensor div(const Tensor& a, const Tensor& b) override;
    Tensor maximum(const Tensor& a, const Tensor& b) override;
    Tensor cast(const Tensor& x, DType dtype) override;
    Tensor layer_norm(const Tensor& x, const Tensor* weight, const Tensor* bias, float eps) override;
    Tensor rms_norm(const Tensor& x, const Tensor* weight, float eps, int64_t axis = -1,
                    DType output = DType::F16) override;
    Tensor activation(const Tensor& x, vrhino::Activation kind) override;
    Tensor rope_nd(const Tensor& x, const Tensor& cosine, const Tensor& sine) override;
    Tensor group_norm(const Tensor& x, int groups, const Tensor* weight, const Tensor* bias, float eps) override;
    Tensor clamp(const Tensor& x, float minimum, float maximum) override;
    Tensor exp(const Tensor& x) override;
    Tensor sqrt(const Tensor& x) override;
    Tensor copy_to_device(const Tensor& input, DType dtype) override;
    Tensor pixel_norm(const Tensor& x, int64_t dim, float eps) override;
    Tensor pixel_shuffle_nd(const Tensor& x, const std::vector<int64_t>& factors) override;
    Tensor l2_normalize(const Tensor& x, int64_t dim, float eps) override;
    // layout operators (:3936-3976, :4190-4196, :4875-4883)
    Tensor permute(const Tensor& x, const std::vector<int64_t>& dims) override;
    Tensor concat(const std::vector<Tensor>& tensors, int64_t dim) override;
    std::vector<Tensor> split(const Tensor& x, const std::vector<int64_t>& sections, int64_t dim) override;
    Tensor slice(const Tensor& x, int64_t dim, int64_t start, int64_t stop) override;
    Tensor sinusoidal_embedding(const Tensor& positions, int64_t width, bool flip, double downscale_shift,
                                bool require_f64_semantics) override;
    Tensor pad(const Tensor& x, const std::vector<int64_t>& padding, float value = 0.0f,
               vrhino::PadMode mode = vrhino::PadMode::Constant) override;
    Tensor interpolate_nearest(const Tensor& x, const std::vector<double>& factors) override;   // :5010-5016
    Tensor reduce_sum(const Tensor& x, int64_t dim, bool keepdim = false) override;              // :4885-4892
    Tensor softmax(const Tensor& x, int64_t axis) override;                                      // :4893-4917
    Tensor rng_normal(vrhino::RngState& state, const std::vector<int64_t>& shape, DType dtype) override; // :5120-5126
    Tensor indexed_gather(const Tensor& table, const Tensor& indices) override;                  // :3981-4055
    // per-axis extents and modes in one pass (replicate axes first, then the constant axes)
    Tensor pad_axes(const Tensor& x, const std::vector<int64_t>& before, const std::vector<int64_t>& after, float value,
                    const std::vector<bool>& replicate);

    // ---- fused forms (one kernel each); see the free functions below for the call-site view --
    Tensor layer_norm_modulate(const Tensor& x, const Tensor* weight, const Tensor* bias, float eps,
                               const Tensor& shift, const Tensor& scale, DType output);
    // cast(modulate(rms_norm(x, no weight, eps), shift, scale), output) -- the LTX block
    Tensor rms_norm_modulate(const Tensor& x, float eps, const Tensor& shift, const Tensor& scale, DType output);
    Tensor rms_norm_rope(const Tensor& x, const Tensor* weight, float eps, const Tensor* cosine,
                         const Tensor* sine, int heads, bool per_head_norm, DType output);
    // rms_norm_rope on two tensors (q and k) in one launch: same width, dtype and tables, own weights and
    // row counts; {out_a, out_b}.  cosine / sine may be null (norm + cast only: cross-attention q and text k).
    std::pair<Tensor, Tensor> rms_norm_rope_pair(const Tensor& x_a, const Tensor& weight_a, const Tensor& x_b, const Tensor& weight_b,
                                                 float eps, const Tensor* cosine, const Tensor* sine, int heads, bool per_head_norm,
                                                 DType output);
    Tensor gated_residual(const Tensor& residual, const Tensor& branch, const Tensor* gate, DType state);
    // Mochi (mochi.cpp:204-211, :228-231): {state, normed} with state = residual + rms_norm(branch, none, branch_eps) *
    // tanh(gate) in `state` dtype and normed = rms_norm(state, none, eps) * (1 + scale) in the stream's dtype; one
    // kernel for a BF16 stream, tanh + the two operators otherwise
    std::pair<Tensor, Tensor> normalized_gated_residual_norm_scale(const Tensor& residual, const Tensor& branch, const Tensor& gate,
                                                                   const Tensor& scale, DType state, float branch_eps, float eps);
    // {state, normed}: state = gated_residual / residual_add (gate == nullptr) in `state` dtype,
    // normed = cast(layer_norm(state, weight, bias, eps) [modulated by shift, scale], output);
    // one kernel when the residual stream, the branch and both results are BF16
    std::pair<Tensor, Tensor> gated_residual_layer_norm(const Tensor& residual, const Tensor& branch, const Tensor* gate,
                                                        DType state, const Tensor* weight, const Tensor* bias, float eps,
                                                        const Tensor* shift, const Tensor* scale, DType output);
    // ---- linear + the operator that reads its result: the GEMM is the device runtime's, asked for
    // its F32 accumulation (linear(x, w, no bias, BF16 compute, F32 output)); the bf16 epilogue
    // (cuda_backend.cu:754-764) and the consumer run as ONE kernel, so the rounded linear output is
    // never written.  BF16 execution and unquantised weights only; otherwise the operators compose.
    Tensor linear_activation(const Tensor& x, const Tensor& weight, const Tensor* bias, vrhino::Activation kind);
    Tensor linear_gated_residual(const Tensor& residual, const Tensor& x, const Tensor& weight, const Tensor* bias,
                                 const Tensor* gate, DType state);
    Tensor linear_swiglu(const Tensor& x, const Tensor& weight, const Tensor* bias);
    // [silu](modulate(pixel_norm(x, 1, eps), shift, scale)) cast to `output`; shift / scale [B, C, 1, ...]
    Tensor pixel_norm_modulate(const Tensor& x, const Tensor& shift, const Tensor& scale, float eps, bool silu, DType output);
    // slice(pixel_shuffle(projected, {2,2,2}), 2, 1, 2T) + slice(concat(4 x pixel_shuffle(input, {2,2,2}), 1), 2, 1, 2T)
    Tensor depth_to_space_residual(const Tensor& projected, const Tensor& input);
    Tensor swiglu(const Tensor& projected);
    Tensor group_norm_silu(const Tensor& x, int groups, const Tensor* weight, const Tensor* bias, float eps);
    // x [B, C, T, H, W]: statistics per (batch entry, frame, group), no permutes
    Tensor group_norm_frames(const Tensor& x, int groups, const Tensor* weight, const Tensor* bias, float eps, bool silu);
    // SamplingPrimitives::linear_combine (sampling.cpp:173-179; also v_to_x0, affine_first_order) in one
    // kernel, 1..4 terms; declared_role: the policy declares the coefficient's scalar role
    Tensor linear_combine(const std::vector<Tensor>& values, const std::vector<float>& coefficients, bool declared_role);
    Tensor cfg_euler(const Tensor& sample, const Tensor& unconditional, const Tensor& conditional,
                     float guidance, float delta, bool subtract_prediction, bool guidance_role, bool solver_role);

    // ---- forwarded to the device runtime -----------------------------------------------------
    std::string name() const override { return "b200+" + rt_->name(); }
    int device_count() const override { return rt_->device_count(); }
    vrhino::DeviceCapability device_capability(int device = 0) const override { return rt_->device_capability(device); }
    vrhino::BackendMemoryCapabilities memory_capabilities() const override { return rt_->memory_capabilities(); }
    bool supports(DType dtype) const override { return rt_->supports(dtype); }
    void set_execution_dtype(DType dtype) override { rt_->set_execution_dtype(dtype); }
    DType execution_dtype() const override { return rt_->execution_dtype(); }
    Tensor allocate_host(const std::vector<int64_t>& s, DType d) override { return rt_->allocate_host(s, d); }
    Tensor allocate_device(const std::vector<int64_t>& s, DType d) override { return rt_->allocate_device(s, d); }
    vrhino::TransferFence copy(const Tensor& s, Tensor& d, CopyMode m = CopyMode::Synchronous) override { return rt_->copy(s, d, m); }
    vrhino::TransferFence create_fence(int device = 0) override { return rt_->create_fence(device); }
    void record_fence(vrhino::TransferFence f) override { rt_->record_fence(f); }
    void wait_fence(vrhino::TransferFence f) override { rt_->wait_fence(f); }
    bool query_fence(vrhino::TransferFence f) override { return rt_->query_fence(f); }
    void destroy_fence(vrhino::TransferFence f) override { rt_->destroy_fence(f); }
    Tensor copy_to_host(const Tensor& input) override { return rt_->copy_to_host(input); }
    void synchronize() override { rt_->synchronize(); }
    void release_cached_device_memory() override;   // also drops the dequantised-weight cache below
    size_t peak_device_bytes() const override { return rt_->peak_device_bytes(); }
    size_t weight_upload_bytes() const override { return rt_->weight_upload_bytes(); }
    double weight_upload_seconds() const override { return rt_->weight_upload_seconds(); }
    // Profiling: the replaced operators record themselves in the device runtime's profiler through
    // its region interface under the names the reference's own operators use
    // (cuda_backend.cu:3011-3064: "norm.layer|rows=..|width=..|dtype=..", "norm.rms|..", "activation|..",
    // "rope|..", "elementwise.add", "cast", "norm.group", "norm.pixel", "pixel_shuffle", "clamp", "exp",
    // "sqrt", "quantized_dequant"), so profile_stats() shows them beside the forwarded ones; the fused
    // forms appear as "fused.<name>".  profile_bytes() adds what the reference does not record: the
    // algorithmic bytes (inputs read once + output written once) each profiled name has moved.
    void enable_profiling(bool e) override { rt_->enable_profiling(e); }
    bool profiling_enabled() const override { return rt_->profiling_enabled(); }
    std::map<std::string, vrhino::ProfileStat> profile_stats() override { return rt_->profile_stats(); }
    const std::map<std::string, uint64_t>& profile_bytes() const { return profile_bytes_; }
    void profile_region_begin(const std::string& n) override { rt_->profile_region_begin(n); }
    void profile_region_end() override { rt_->profile_region_end(); }
    uint64_t weight_cache_hits() const override { return rt_->weight_cache_hits(); }
    uint64_t weight_cache_misses() const override { return rt_->weight_cache_misses(); }
    size_t weight_cache_resident_bytes() const override { return rt_->weight_cache_resident_bytes(); }
    size_t weight_cache_capacity_bytes() const override { return rt_->weight_cache_capacity_bytes(); }
    void enable_weight_cache(bool e) override { weight_cache_enabled_ = e; if (!e) drop_dequantized_cache(); rt_->enable_weight_cache(e); }
    // Dequantised weights are kept on the device, keyed by the host payload like the reference's
    // packed-byte cache (cuda_backend.cu:3236-3275), so a quantised weight is decoded once instead of
    // once per linear() call (:3276-3295).  Least-recently-used entries go when the budget is exceeded;
    // a weight larger than the budget is decoded per call as before.  Default budget: 48 GiB.
    void set_dequantized_cache_budget(size_t bytes);
    size_t dequantized_cache_resident_bytes() const { return dequant_resident_; }
    uint64_t dequantized_cache_hits() const { return dequant_hits_; }
    uint64_t dequantized_cache_misses() const { return dequant_misses_; }
    void enable_true_quant_compute(bool e) override { rt_->enable_true_quant_compute(e); }
    bool true_quant_compute_enabled() const override { return rt_->true_quant_compute_enabled(); }
    vrhino::QuantComputeStats quant_compute_stats() const override { return rt_->quant_compute_stats(); }
    void reset_quant_compute_stats() override { rt_->reset_quant_compute_stats(); }
    void configure_memory_runtime(const vrhino::MemoryBudget& b, const vrhino::MemoryRuntimeOptions& o) override { rt_->configure_memory_runtime(b, o); }
    bool memory_runtime_enabled() const override { return rt_->memory_runtime_enabled(); }
    void set_vrm_mapped_bytes(size_t b) override { rt_->set_vrm_mapped_bytes(b); }
    void begin_memory_trace() override { rt_->begin_memory_trace(); }
    std::vector<vrhino::MemoryAccess> end_memory_trace() override { return rt_->end_memory_trace(); }
    void set_memory_trace(std::vector<vrhino::MemoryAccess> t) override { rt_->set_memory_trace(std::move(t)); }
    vrhino::MemoryRuntimeStats memory_runtime_stats() const override { return rt_->memory_runtime_stats(); }

    Tensor linear(const Tensor& x, const Tensor& w, const Tensor* b = nullptr, DType c = DType::F16, DType o = DType::F16) override { return rt_->linear(x, w, b, c, o); }
    Tensor batched_matmul(const Tensor& a, const Tensor& b) override { return rt_->batched_matmul(a, b); }
    Tensor reshape(const Tensor& x, const std::vector<int64_t>& s) override { return rt_->reshape(x, s); }
    Tensor attention(const Tensor& q, const Tensor& k, const Tensor& v, const Tensor* mask = nullptr, bool causal = false,
                     float scale = 0.0f, const Tensor* bias = nullptr, vrhino::AttentionObservation* obs = nullptr) override {
        return rt_->attention(q, k, v, mask, causal, scale, bias, obs);
    }
    Tensor conv3d(const Tensor& x, const Tensor& w, const Tensor* b, const std::vector<int>& s, const std::vector<int>& p,
                  const std::vector<int>& d = {1, 1, 1}, int g = 1) override { return rt_->conv3d(x, w, b, s, p, d, g); }
    Tensor conv2d(const Tensor& x, const Tensor& w, const Tensor* b, const std::vector<int>& s, const std::vector<int>& p,
                  const std::vector<int>& d = {1, 1}, int g = 1) override { return rt_->conv2d(x, w, b, s, p, d, g); }
    Tensor conv_transpose2d(const Tensor& x, const Tensor& w, const Tensor* b, const std::vector<int>& s, const std::vector<int>& p,
                            const std::vector<int>& op = {0, 0}, const std::vector<int>& d = {1, 1}, int g = 1) override {
        return rt_->conv_transpose2d(x, w, b, s, p, op, d, g);
    }
    Tensor max_pool2d(const Tensor& x, const std::vector<int>& k, const std::vector<int>& s, const std::vector<int>& p = {0, 0}) override { return rt_->max_pool2d(x, k, s, p); }
    Tensor interpolate_bilinear_2d(const Tensor& x, int64_t h, int64_t w, bool a) override { return rt_->interpolate_bilinear_2d(x, h, w, a); }

private:
    DType operand_dtype(const Tensor& t) const;
    Tensor binary(int kind, const Tensor& a, const Tensor& b);
    Tensor unary(int which, const Tensor& x, int kind, float p0, float p1);
    Tensor parameter(const Tensor& t);
    Tensor dequantize(const Tensor& input, DType dtype);
    Tensor group_norm_impl(const Tensor& x, int groups, const Tensor* weight, const Tensor* bias, float eps, bool silu);
    void* workspace(size_t bytes);
    void begin_operator() const;
    template <typename F> Tensor guarded(F&& body);
    template <typename F> Tensor unguarded(F&& body);

    class ProfileRegion;
    friend class ProfileRegion;
    void drop_dequantized_cache();

    std::unique_ptr<vrhino::Backend> rt_;
    Tensor workspace_;
    std::map<std::string, uint64_t> profile_bytes_;
    struct DequantizedEntry { Tensor value; size_t bytes = 0; uint64_t last_use = 0; };
    std::map<std::pair<const void*, int>, DequantizedEntry> dequant_cache_;
    size_t dequant_resident_ = 0, dequant_budget_ = size_t{48} << 30;
    uint64_t dequant_clock_ = 0, dequant_hits_ = 0, dequant_misses_ = 0;
    bool weight_cache_enabled_ = true;
};

// ---- call-site view ---------------------------------------------------------------------------
// Same arguments as the seams of native/include/vrhino/architecture.h:63-86 they merge.  With a
// B200Backend behind `backend` each is ONE kernel; with any other backend they compose the
// reference's own seams, so a call site can be switched unconditionally.

// cast(modulate(layer_norm(x, weight, bias, eps), shift, scale), output)   (wan.cpp:85-92)
vrhino::Tensor layer_norm_modulate(vrhino::Backend& backend, const vrhino::PrecisionPolicy& policy,
                                   const vrhino::Tensor& x, const vrhino::Tensor* weight, const vrhino::Tensor* bias,
                                   float eps, const vrhino::Tensor& shift, const vrhino::Tensor& scale,
                                   vrhino::DType output = vrhino::DType::BF16);
// cast(operation_rope(split_heads(attention_norm(x, weight, eps)), cos, sin), output) for x [B,S,D]
// (wan.cpp:38-52); per_head_norm: heads are split before the norm (mochi.cpp:182-187).  cosine /
// sine may be null (norm + cast only).  The result keeps x's [B,S,D] shape.
vrhino::Tensor rms_norm_rope(vrhino::Backend& backend, const vrhino::PrecisionPolicy& policy,
                             const vrhino::Tensor& x, const vrhino::Tensor* weight, float eps,
                             const vrhino::Tensor* cosine, const vrhino::Tensor* sine, int heads,
                             bool per_head_norm = false, vrhino::DType output = vrhino::DType::BF16);
// the same for q and k together (wan.cpp:38-52 normalises and rotates one after the other): {q operand, k operand}
std::pair<vrhino::Tensor, vrhino::Tensor> rms_norm_rope_pair(vrhino::Backend& backend, const vrhino::PrecisionPolicy& policy,
                                                             const vrhino::Tensor& q, const vrhino::Tensor& weight_q,
                                                             const vrhino::Tensor& k, const vrhino::Tensor& weight_k, float eps,
                                                             const vrhino::Tensor* cosine, const vrhino::Tensor* sine, int heads,
                                                             bool per_head_norm = false,
                                                             vrhino::DType output = vrhino::DType::BF16);
// Mochi's layer boundary (mochi.cpp:204-211 then :228-231): {x', y} with x' = x + rms_norm(branch) * tanh(gate) and
// y = rms_norm(x') * (1 + scale); gate and scale are [B, D]
std::pair<vrhino::Tensor, vrhino::Tensor> normalized_gated_residual_norm_scale(
    vrhino::Backend& backend, const vrhino::PrecisionPolicy& policy, const vrhino::Tensor& residual,
    const vrhino::Tensor& branch, const vrhino::Tensor& gate, const vrhino::Tensor& scale, float eps = 1e-6f);
// gated_residual / residual_add (gate == nullptr) of common.cpp:134-144.
vrhino::Tensor fused_gated_residual(vrhino::Backend& backend, const vrhino::PrecisionPolicy& policy,
                                    const vrhino::Tensor& residual, const vrhino::Tensor& branch,
                                    const vrhino::Tensor* gate);
// The residual update and the LayerNorm of the updated stream that follows it in the Wan block
// (wan.cpp:95-98: first residual -> norm3; wan.cpp:103-107: residual_add -> layer_norm -> modulate):
// returns {state, cast(normed, output)}; shift / scale null = no modulation.
std::pair<vrhino::Tensor, vrhino::Tensor> fused_gated_residual_layer_norm(
    vrhino::Backend& backend, const vrhino::PrecisionPolicy& policy, const vrhino::Tensor& residual,
    const vrhino::Tensor& branch, const vrhino::Tensor* gate, const vrhino::Tensor* weight, const vrhino::Tensor* bias,
    float eps, const vrhino::Tensor* shift, const vrhino::Tensor* scale, vrhino::DType output = vrhino::DType::BF16);
// activation(linear(x, weight, bias), kind)   (wan.cpp:109-112)
vrhino::Tensor linear_activation(vrhino::Backend& backend, const vrhino::Tensor& x, const vrhino::Tensor& weight,
                                 const vrhino::Tensor* bias, vrhino::Activation kind);
// gated_residual / residual_add (gate == nullptr) of residual and linear(x, weight, bias)   (wan.cpp:113-116)
vrhino::Tensor linear_gated_residual(vrhino::Backend& backend, const vrhino::PrecisionPolicy& policy,
                                     const vrhino::Tensor& residual, const vrhino::Tensor& x,
                                     const vrhino::Tensor& weight, const vrhino::Tensor* bias, const vrhino::Tensor* gate);
// the SwiGLU of linear(x, weight, bias): split -> silu -> mul   (mochi.cpp:197-200)
vrhino::Tensor linear_swiglu(vrhino::Backend& backend, const vrhino::Tensor& x, const vrhino::Tensor& weight,
                             const vrhino::Tensor* bias);
// executor.silu(modulate(backend, policy, executor.pixel_norm(x), shift, scale))   (ltx.cpp:221-227), with the
// cast to the consumer's operand dtype when output is BF16 (F32 = modulate's contract output)
vrhino::Tensor pixel_norm_modulate_silu(vrhino::Backend& backend, const vrhino::PrecisionPolicy& policy,
                                        const vrhino::Tensor& x, const vrhino::Tensor& shift, const vrhino::Tensor& scale,
                                        float eps = 1e-8f, vrhino::DType output = vrhino::DType::F32);
// LTX depth_to_space (ltx.cpp:250-259) after its convolution `projected` = edge_time_conv(input): the two
// pixel_shuffles, the four-fold concat, the two slices and the add as one kernel
vrhino::Tensor depth_to_space_residual(vrhino::Backend& backend, const vrhino::Tensor& projected, const vrhino::Tensor& input);
// pad(pad(x, {0,0,0,0,temporal,temporal}, 0, Replicate), {pad_w,pad_w,pad_h,pad_h}, 0) on x [B, C, T, H, W]: the two
// pads in front of every LTX convolution (edge_time_conv, ltx.cpp:205-215) as one pass
vrhino::Tensor edge_time_pad(vrhino::Backend& backend, const vrhino::Tensor& x, int64_t temporal, int64_t pad_h, int64_t pad_w);
// mul(parts[0], silu(parts[1])), parts = split(projected, {H, H}, -1)   (mochi.cpp:195-202)
vrhino::Tensor swiglu(vrhino::Backend& backend, const vrhino::Tensor& projected);
// activation(group_norm(x, groups, weight, bias, eps), Silu)   (autoencoder_kl.cpp:31-41)
vrhino::Tensor group_norm_silu(vrhino::Backend& backend, const vrhino::Tensor& x, int groups,
                               const vrhino::Tensor* weight, const vrhino::Tensor* bias, float eps);

// frame_group_norm (native/src/architectures/mochi.cpp:365-371), optionally with the SiLU its callers
// apply next (:375-377): permute to [B*T, C, H, W] -> group_norm -> permute back, or one pass
// over the unpermuted tensor with a B200Backend.
vrhino::Tensor frame_group_norm(vrhino::Backend& backend, const vrhino::Tensor& x, int groups,
                                const vrhino::Tensor* weight, const vrhino::Tensor* bias, float eps, bool silu = false);

}  // namespace vrhino_b200
