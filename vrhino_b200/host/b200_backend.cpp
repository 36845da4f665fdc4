// B200Backend: the reference's Backend interface over the C ABI of libvrb.so.
// The host wrappers below keep the conventions of the reference's own wrappers
// (native/src/backend/cuda/cuda_backend.cu): the operand-dtype rule (a device F32/BF16 tensor
// keeps its dtype, anything else takes the execution dtype), upload-on-demand of host operands,
// `cast` / `copy_to_device` to the same dtype returning the SAME handle (:3200), results in
// freshly allocated device tensors, vrhino::Error on every failure, and a session that turns
// terminal once an operator has thrown (native/include/vrhino/memory.h:225-236).
#include "b200_backend.h"

#include <algorithm>
#include <cmath>
#include <limits>

#include "vrb.h"
#include "vrhino/architecture.h"
#include "vrhino/error.h"
#include "vrhino/tensor_util.h"

namespace vrhino_b200 {

using vrhino::DeviceId;
using vrhino::DType;
using vrhino::Error;
using vrhino::require;
using vrhino::Tensor;

namespace {

constexpr vrb_stream kLegacyStream = nullptr;

bool is_float(DType d) { return d == DType::F32 || d == DType::BF16; }
bool device_float(const Tensor& t) { return t.device() == DeviceId::accelerator() && is_float(t.dtype()); }
int code(DType d) { return static_cast<int>(d); }   // VRB_F32 / VRB_BF16 / VRB_U8 equal the DType values

void check(int status) {
    if (status == VRB_OK) return;
    const char* text = vrb_last_error();
    throw Error(text && *text ? text : "vrb status " + std::to_string(status));
}

// Right-aligned broadcast of two shapes (cuda_backend.cu:508-523).
std::vector<int64_t> broadcast_shape(const std::vector<int64_t>& a, const std::vector<int64_t>& b) {
    const size_t rank = std::max(a.size(), b.size());
    std::vector<int64_t> out(rank, 1);
    for (size_t i = 0; i < rank; ++i) {
        const int64_t x = i < rank - a.size() ? 1 : a[i - (rank - a.size())];
        const int64_t y = i < rank - b.size() ? 1 : b[i - (rank - b.size())];
        require(x == y || x == 1 || y == 1, "Incompatible broadcast shapes");
        out[i] = std::max(x, y);
    }
    return out;
}

// rows_per_vector / vector count of a modulation-like operand against x = [.., width]:
// one vector for all rows, one per batch entry, or one per row.
void vector_layout(const Tensor& x, const Tensor& vec, int64_t& rows_per_vector, int64_t& vectors) {
    const int64_t width = x.dim(-1), rows = x.numel() / width;
    require(vec.numel() % width == 0, "Incompatible broadcast shapes");
    const int64_t n = vec.numel() / width;
    if (n == 1) { rows_per_vector = rows; vectors = 1; return; }
    if (n == rows) { rows_per_vector = 1; vectors = rows; return; }
    require(x.ndim() >= 2 && n == x.dim(0) && rows % n == 0, "Incompatible broadcast shapes");
    rows_per_vector = rows / n;
    vectors = n;
}

}  // namespace

// One profiled operator: a region in the device runtime's profiler (events on the legacy stream the
// kernels run on) under the reference's name for that operator, plus the bytes it moves.  The name is
// only built when profiling is on.  Closing never throws: a failing profiler must not mask the
// operator's own outcome.
class B200Backend::ProfileRegion {
public:
    template <typename Name>
    ProfileRegion(B200Backend& backend, Name&& name, uint64_t bytes) : backend_(backend) {
        if (!backend_.rt_->profiling_enabled()) return;
        const std::string text = name();
        backend_.rt_->profile_region_begin(text);
        backend_.profile_bytes_[text] += bytes;
        open_ = true;
    }
    ~ProfileRegion() {
        if (!open_) return;
        try { backend_.rt_->profile_region_end(); } catch (...) {}
    }
    ProfileRegion(const ProfileRegion&) = delete;
    ProfileRegion& operator=(const ProfileRegion&) = delete;
private:
    B200Backend& backend_;
    bool open_ = false;
};

namespace {
std::string sized(const char* head, int64_t rows, int64_t width, DType dtype) {
    return std::string(head) + "|rows=" + std::to_string(rows) + "|width=" + std::to_string(width) + "|dtype=" + vrhino::dtype_name(dtype);
}
uint64_t bytes_of(const Tensor& t) { return t.defined() ? static_cast<uint64_t>(t.bytes()) : 0; }
}  // namespace

B200Backend::B200Backend(std::unique_ptr<vrhino::Backend> device_runtime) : rt_(std::move(device_runtime)) {
    require(rt_ != nullptr, "B200Backend needs a device runtime backend");
    require(vrb_abi_version() == VRB_ABI_VERSION, "libvrb.so ABI version mismatch");
}
B200Backend::~B200Backend() = default;

// The reference wraps add/mul/div/maximum, cast, copy_to_device, group_norm, clamp, exp and sqrt in
// a CudaFailureGuard (cuda_backend.cu:2601-2615, :3064): an exception escaping them leaves the
// session terminal.  layer_norm, rms_norm, activation and rope_nd carry no guard, so a rejected
// argument there leaves the session usable.  Both kinds refuse to start on a terminal session,
// this object's or the device runtime's.
template <typename F>
Tensor B200Backend::guarded(F&& body) {
    begin_operator();
    try {
        return body();
    } catch (...) {
        retire_resource_session();
        rt_->retire_resource_session();
        throw;
    }
}
template <typename F>
Tensor B200Backend::unguarded(F&& body) {
    begin_operator();
    return body();
}
void B200Backend::begin_operator() const {
    require_active_session();
    rt_->require_active_session();
}

DType B200Backend::operand_dtype(const Tensor& t) const { return device_float(t) ? t.dtype() : execution_dtype(); }

// Optional affine parameter on the device in a float dtype the kernels convert themselves.
Tensor B200Backend::parameter(const Tensor& t) {
    if (device_float(t)) return t;
    return copy_to_device(t, is_float(t.dtype()) ? t.dtype() : execution_dtype());
}

Tensor B200Backend::copy_to_device(const Tensor& input, DType dtype) {
    begin_operator();
    require(input.defined(), "Cannot upload undefined tensor");
    if (input.device() == DeviceId::accelerator() && input.dtype() == dtype) return input;
    if (input.is_quantized()) return dequantize(input, dtype);
    if (input.device() == DeviceId::accelerator() && is_float(dtype) &&
        (is_float(input.dtype()) || input.dtype() == DType::U8))
        return cast(input, dtype);
    return rt_->copy_to_device(input, dtype);   // host uploads (with the runtime's small-value and weight caches)
}

// Quantised weights (cuda_backend.cu:3214-3296): packed bytes and F32 scales go up as they are,
// then one kernel decodes, scales and rounds.  The preconditions and their texts are the reference's.
Tensor B200Backend::dequantize(const Tensor& input, DType dtype) {
    return guarded([&] {
        require(input.device() == DeviceId::host() && is_float(dtype),
                "Quantized tensors require CPU storage and float compute output");
        const vrhino::QuantizationInfo& q = input.quantization();
        require(q.axis == 1 && q.group_size > 0 && q.block_size == 0 && q.symmetric &&
                    (q.granularity == "per_group" || q.granularity == "per_channel") && q.zero_point_mode == "none" &&
                    q.dequantization == vrhino::DequantizationSemantics::ScaleThenCast,
                "Unsupported quantized tensor layout/policy");
        int kind = -1;
        if (q.type == vrhino::QuantType::FP8E4M3FN && q.packing_layout == "byte_e4m3fn") kind = VRB_Q_FP8_E4M3FN;
        else if (q.type == vrhino::QuantType::INT8Symmetric && q.packing_layout == "byte_twos_complement") kind = VRB_Q_INT8;
        else if (q.type == vrhino::QuantType::INT4Symmetric && q.packing_layout == "nibble_low_first_twos_complement") kind = VRB_Q_INT4;
        require(kind >= 0, "Unsupported quantized tensor packing");
        const auto key = std::make_pair(static_cast<const void*>(input.data()), code(dtype));
        if (weight_cache_enabled_) {
            const auto found = dequant_cache_.find(key);
            if (found != dequant_cache_.end() && found->second.value.shape() == input.shape()) {
                ++dequant_hits_;
                found->second.last_use = ++dequant_clock_;
                return found->second.value;
            }
        }
        ++dequant_misses_;
        Tensor host_bytes = Tensor::borrowed(input.data(), input.bytes(), {static_cast<int64_t>(input.bytes())}, DType::U8);
        Tensor packed = rt_->allocate_device(host_bytes.shape(), DType::U8);
        Tensor scales = rt_->allocate_device(q.scales.shape(), DType::F32);
        rt_->copy(host_bytes, packed);
        rt_->copy(q.scales, scales);
        Tensor output = rt_->allocate_device(input.shape(), dtype);
        const int64_t rows = input.dim(0), inner = input.numel() / rows;
        {
            ProfileRegion region(*this, [] { return std::string("quantized_dequant"); },
                                 bytes_of(packed) + bytes_of(scales) + bytes_of(output));
            check(vrb_dequantize(kind, packed.data(), scales.data_as<float>(), output.data(), code(dtype), rows, inner,
                                 q.group_size, kLegacyStream));
        }
        const size_t resident = output.bytes();
        if (weight_cache_enabled_ && resident <= dequant_budget_) {
            while (dequant_resident_ + resident > dequant_budget_ && !dequant_cache_.empty()) {
                auto oldest = dequant_cache_.begin();
                for (auto it = dequant_cache_.begin(); it != dequant_cache_.end(); ++it)
                    if (it->second.last_use < oldest->second.last_use) oldest = it;
                dequant_resident_ -= oldest->second.bytes;
                dequant_cache_.erase(oldest);
            }
            dequant_cache_[key] = DequantizedEntry{output, resident, ++dequant_clock_};
            dequant_resident_ += resident;
        }
        return output;
    });
}

void B200Backend::drop_dequantized_cache() {
    dequant_cache_.clear();
    dequant_resident_ = 0;
}
void B200Backend::set_dequantized_cache_budget(size_t bytes) {
    dequant_budget_ = bytes;
    if (dequant_resident_ > bytes) drop_dequantized_cache();
}
void B200Backend::release_cached_device_memory() {
    require_active_session();
    drop_dequantized_cache();
    rt_->release_cached_device_memory();
}

Tensor B200Backend::cast(const Tensor& x, DType dtype) {
    begin_operator();
    if (x.device() != DeviceId::accelerator()) return copy_to_device(x, dtype);
    if (x.dtype() == dtype) return x;
    if (!is_float(dtype) || !(is_float(x.dtype()) || x.dtype() == DType::U8)) return rt_->cast(x, dtype);
    return guarded([&] {
        Tensor out = rt_->allocate_device(x.shape(), dtype);
        ProfileRegion region(*this, [] { return std::string("cast"); }, bytes_of(x) + bytes_of(out));
        if (x.numel() > 0) check(vrb_cast(x.data(), code(x.dtype()), out.data(), code(dtype), x.numel(), kLegacyStream));
        return out;
    });
}

Tensor B200Backend::binary(int kind, const Tensor& a_raw, const Tensor& b_raw) {
    return guarded([&] {
        const DType dtype = device_float(a_raw) ? a_raw.dtype() : device_float(b_raw) ? b_raw.dtype() : execution_dtype();
        Tensor a = copy_to_device(a_raw, dtype), b = copy_to_device(b_raw, dtype);
        Tensor out = rt_->allocate_device(broadcast_shape(a.shape(), b.shape()), dtype);
        const int64_t one = 1;
        static const char* const names[] = {"elementwise.add", "elementwise.mul", "elementwise.div", "elementwise.maximum"};
        ProfileRegion region(*this, [&] { return std::string(names[kind]); }, bytes_of(a) + bytes_of(b) + bytes_of(out));
        check(vrb_binary(kind, a.data(), a.ndim() ? a.shape().data() : &one, static_cast<int>(a.ndim()),
                         b.data(), b.ndim() ? b.shape().data() : &one, static_cast<int>(b.ndim()),
                         out.data(), code(dtype), kLegacyStream));
        return out;
    });
}
Tensor B200Backend::add(const Tensor& a, const Tensor& b) { return binary(VRB_ADD, a, b); }
Tensor B200Backend::mul(const Tensor& a, const Tensor& b) { return binary(VRB_MUL, a, b); }
Tensor B200Backend::div(const Tensor& a, const Tensor& b) { return binary(VRB_DIV, a, b); }
Tensor B200Backend::maximum(const Tensor& a, const Tensor& b) { return binary(VRB_MAX, a, b); }

Tensor B200Backend::layer_norm(const Tensor& raw, const Tensor* weight_raw, const Tensor* bias_raw, float eps) {
    return unguarded([&] {
        const DType dtype = operand_dtype(raw);
        Tensor x = copy_to_device(raw, dtype), weight, bias;
        const int64_t width = x.dim(-1);
        if (weight_raw) { weight = parameter(*weight_raw); require(weight.numel() == width, "layer norm weight mismatch"); }
        if (bias_raw) { bias = parameter(*bias_raw); require(bias.numel() == width, "layer norm bias mismatch"); }
        Tensor out = rt_->allocate_device(x.shape(), dtype);
        ProfileRegion region(*this, [&] { return sized("norm.layer", x.numel() / width, width, dtype); }, bytes_of(x) + bytes_of(out));
        check(vrb_layer_norm(x.data(), code(dtype), weight_raw ? weight.data() : nullptr, weight_raw ? code(weight.dtype()) : 0,
                             bias_raw ? bias.data() : nullptr, bias_raw ? code(bias.dtype()) : 0, out.data(),
                             x.numel() / width, width, eps, kLegacyStream));
        return out;
    });
}

Tensor B200Backend::rms_norm(const Tensor& raw, const Tensor* weight_raw, float eps, int64_t axis, DType requested) {
    return unguarded([&] {
        if (axis < 0) axis += raw.ndim();
        require(axis >= 0 && axis < raw.ndim(), "rms_norm axis invalid");
        const DType dtype = operand_dtype(raw);
        const DType out_dtype = requested == DType::F16 ? dtype : requested;   // F16 = "same as the input" (:4105)
        require(out_dtype == dtype || (dtype == DType::BF16 && out_dtype == DType::F32), "rms_norm output dtype unsupported");
        Tensor x = copy_to_device(raw, dtype), weight;
        if (weight_raw) { weight = parameter(*weight_raw); require(weight.numel() == x.dim(axis), "rms norm weight mismatch"); }
        const void* w = weight_raw ? weight.data() : nullptr;
        const int wcode = weight_raw ? code(weight.dtype()) : 0;
        Tensor out = rt_->allocate_device(x.shape(), out_dtype);
        ProfileRegion region(*this, [&] {
            const int64_t w = x.dim(axis);
            return std::string("norm.rms|rows=") + std::to_string(x.numel() / w) + "|width=" + std::to_string(w) + "|axis=" +
                   std::to_string(axis) + "|dtype=" + vrhino::dtype_name(dtype);
        }, bytes_of(x) + bytes_of(out));
        if (axis == x.ndim() - 1) {
            if (dtype == DType::BF16 && out_dtype == DType::F32)
                require(weight_raw != nullptr, "BF16-to-FP32 rms_norm requires affine weight");
            const int64_t width = x.dim(-1);
            check(vrb_rms_norm(x.data(), code(dtype), w, wcode, out.data(), code(out_dtype), x.numel() / width, width, eps,
                               kLegacyStream));
        } else {
            require(out_dtype == dtype, "mixed-dtype rms_norm currently requires final axis");
            const int64_t width = x.dim(axis);
            int64_t inner = 1;
            for (int64_t i = axis + 1; i < x.ndim(); ++i) inner *= x.dim(i);
            check(vrb_rms_norm_axis(x.data(), code(dtype), w, wcode, out.data(), x.numel() / (width * inner), width, inner,
                                    eps, 0, kLegacyStream));
        }
        return out;
    });
}

// which: 0 activation(kind), 1 clamp(p0, p1), 2 exp, 3 sqrt
Tensor B200Backend::unary(int which, const Tensor& raw, int kind, float p0, float p1) {
    auto body = [&] {
        if (which == 1) require(p0 <= p1, "Invalid clamp bounds");
        const DType dtype = operand_dtype(raw);
        Tensor x = copy_to_device(raw, dtype), out = rt_->allocate_device(x.shape(), dtype);
        const int64_t n = x.numel();
        ProfileRegion region(*this, [&] {
            if (which == 0)
                return std::string("activation|elements=") + std::to_string(n) + "|kind=" + std::to_string(kind) + "|dtype=" +
                       vrhino::dtype_name(dtype);
            return std::string(which == 1 ? "clamp" : which == 2 ? "exp" : "sqrt");
        }, bytes_of(x) + bytes_of(out));
        switch (which) {
            case 0: check(vrb_activation(kind, x.data(), out.data(), code(dtype), n, kLegacyStream)); break;
            case 1: check(vrb_clamp(x.data(), out.data(), code(dtype), n, p0, p1, kLegacyStream)); break;
            case 2: check(vrb_exp(x.data(), out.data(), code(dtype), n, kLegacyStream)); break;
            default: check(vrb_sqrt(x.data(), out.data(), code(dtype), n, kLegacyStream)); break;
        }
        return out;
    };
    return which == 0 ? unguarded(body) : guarded(body);
}
Tensor B200Backend::activation(const Tensor& x, vrhino::Activation kind) { return unary(0, x, static_cast<int>(kind), 0.f, 0.f); }
Tensor B200Backend::clamp(const Tensor& x, float minimum, float maximum) { return unary(1, x, 0, minimum, maximum); }
Tensor B200Backend::exp(const Tensor& x) { return unary(2, x, 0, 0.f, 0.f); }
Tensor B200Backend::sqrt(const Tensor& x) { return unary(3, x, 0, 0.f, 0.f); }

Tensor B200Backend::rope_nd(const Tensor& raw, const Tensor& cos_raw, const Tensor& sin_raw) {
    return unguarded([&] {
        require(raw.dim(-1) % 2 == 0, "RoPE width must be even");
        const DType dtype = operand_dtype(raw);
        const DType f_dtype = device_float(cos_raw) ? cos_raw.dtype() : dtype;
        Tensor x = copy_to_device(raw, dtype), c = copy_to_device(cos_raw, f_dtype), s = copy_to_device(sin_raw, f_dtype);
        require(c.shape() == s.shape(), "RoPE frequency mismatch");
        broadcast_shape(x.shape(), c.shape());
        Tensor out = rt_->allocate_device(x.shape(), dtype);
        ProfileRegion region(*this, [&] {
            return std::string("rope|elements=") + std::to_string(x.numel()) + "|width=" + std::to_string(x.dim(-1)) + "|dtype=" +
                   vrhino::dtype_name(dtype);
        }, bytes_of(x) + bytes_of(c) + bytes_of(s) + bytes_of(out));
        check(vrb_rope(x.data(), code(dtype), x.shape().data(), static_cast<int>(x.ndim()), c.data(), s.data(), code(f_dtype),
                       c.shape().data(), static_cast<int>(c.ndim()), out.data(), kLegacyStream));
        return out;
    });
}

void* B200Backend::workspace(size_t bytes) {
    if (!workspace_.defined() || workspace_.bytes() < bytes)
        workspace_ = rt_->allocate_device({static_cast<int64_t>(bytes)}, DType::U8);
    return workspace_.data();
}

Tensor B200Backend::group_norm_impl(const Tensor& raw, int groups, const Tensor* weight_raw, const Tensor* bias_raw,
                                    float eps, bool silu) {
    return guarded([&] {
        require(raw.ndim() >= 3 && groups > 0 && raw.dim(1) % groups == 0, "group norm shape/groups mismatch");
        const DType dtype = operand_dtype(raw);
        Tensor x = copy_to_device(raw, dtype), weight, bias;
        if (weight_raw) weight = parameter(*weight_raw);
        if (bias_raw) bias = parameter(*bias_raw);
        const int64_t batch = x.dim(0), channels = x.dim(1), spatial = x.numel() / (batch * channels);
        require(batch * groups <= std::numeric_limits<int>::max(), "group norm launch extent exceeds CUDA grid capacity");
        const size_t need = vrb_group_norm_workspace_bytes(batch, groups);
        Tensor out = rt_->allocate_device(x.shape(), dtype);
        ProfileRegion region(*this, [&] { return std::string(silu ? "fused.norm.group+silu" : "norm.group"); },
                             2 * bytes_of(x) + bytes_of(out));   // statistics pass + normalise pass
        check(vrb_group_norm(x.data(), code(dtype), weight_raw ? weight.data() : nullptr, weight_raw ? code(weight.dtype()) : 0,
                             bias_raw ? bias.data() : nullptr, bias_raw ? code(bias.dtype()) : 0, out.data(), batch, channels,
                             spatial, groups, eps, silu ? 1 : 0, workspace(need), need, kLegacyStream));
        return out;
    });
}
Tensor B200Backend::group_norm(const Tensor& x, int groups, const Tensor* w, const Tensor* b, float eps) {
    return group_norm_impl(x, groups, w, b, eps, false);
}
Tensor B200Backend::group_norm_silu(const Tensor& x, int groups, const Tensor* w, const Tensor* b, float eps) {
    return group_norm_impl(x, groups, w, b, eps, true);
}

Tensor B200Backend::group_norm_frames(const Tensor& raw, int groups, const Tensor* weight_raw, const Tensor* bias_raw,
                                      float eps, bool silu) {
    return guarded([&] {
        require(raw.ndim() == 5 && groups > 0 && raw.dim(1) % groups == 0, "group norm shape/groups mismatch");
        const DType dtype = operand_dtype(raw);
        Tensor x = copy_to_device(raw, dtype), weight, bias;
        if (weight_raw) weight = parameter(*weight_raw);
        if (bias_raw) bias = parameter(*bias_raw);
        const int64_t batch = x.dim(0), channels = x.dim(1), frames = x.dim(2), spatial = x.dim(3) * x.dim(4);
        const size_t need = vrb_group_norm_frames_workspace_bytes(batch, frames, groups);
        Tensor out = rt_->allocate_device(x.shape(), dtype);
        ProfileRegion region(*this, [&] { return std::string(silu ? "fused.norm.group_frames+silu" : "fused.norm.group_frames"); },
                             2 * bytes_of(x) + bytes_of(out));
        check(vrb_group_norm_frames(x.data(), code(dtype), weight_raw ? weight.data() : nullptr,
                                    weight_raw ? code(weight.dtype()) : 0, bias_raw ? bias.data() : nullptr,
                                    bias_raw ? code(bias.dtype()) : 0, out.data(), batch, channels, frames, spatial, groups,
                                    eps, silu ? 1 : 0, workspace(need), need, kLegacyStream));
        return out;
    });
}

Tensor B200Backend::pixel_norm(const Tensor& raw, int64_t dim, float eps) {
    return guarded([&] {   // VRHINO_PROFILE("norm.pixel") carries the failure guard (cuda_backend.cu:3064, :5050)
        if (dim < 0) dim += static_cast<int64_t>(raw.ndim());
        require(dim >= 0 && dim < static_cast<int64_t>(raw.ndim()), "pixel norm dim invalid");
        const DType dtype = operand_dtype(raw);
        Tensor x = copy_to_device(raw, dtype);
        const int64_t channels = x.dim(dim);
        int64_t inner = 1;
        for (int64_t d = dim + 1; d < static_cast<int64_t>(x.ndim()); ++d) inner *= x.dim(d);
        Tensor out = rt_->allocate_device(x.shape(), dtype);
        ProfileRegion region(*this, [] { return std::string("norm.pixel"); }, bytes_of(x) + bytes_of(out));
        check(vrb_pixel_norm(x.data(), code(dtype), nullptr, nullptr, 0, 0, out.data(), code(dtype),
                             x.numel() / (channels * inner), channels, inner, eps, kLegacyStream));
        return out;
    });
}

Tensor B200Backend::l2_normalize(const Tensor& raw, int64_t dim, float eps) {
    return guarded([&] {   // VRHINO_PROFILE("norm.l2") carries the failure guard (cuda_backend.cu:3064, :5090)
        if (dim < 0) dim += static_cast<int64_t>(raw.ndim());
        require(dim >= 0 && dim < static_cast<int64_t>(raw.ndim()) && eps >= 0.0f, "l2 normalize contract violation");
        const DType dtype = operand_dtype(raw);
        Tensor x = copy_to_device(raw, dtype);
        const int64_t channels = x.dim(dim);
        int64_t inner = 1;
        for (int64_t d = dim + 1; d < static_cast<int64_t>(x.ndim()); ++d) inner *= x.dim(d);
        require(x.numel() / channels <= std::numeric_limits<int>::max(), "l2 normalize launch extent exceeds CUDA grid capacity");
        Tensor out = rt_->allocate_device(x.shape(), dtype);
        ProfileRegion region(*this, [] { return std::string("norm.l2"); }, bytes_of(x) + bytes_of(out));
        check(vrb_l2_normalize(x.data(), out.data(), code(dtype), x.numel() / (channels * inner), channels, inner, eps, kLegacyStream));
        return out;
    });
}

// ---- layout operators ----------------------------------------------------------------------------------
Tensor B200Backend::permute(const Tensor& raw, const std::vector<int64_t>& dims) {
    return guarded([&] {   // VRHINO_PROFILE("permute") carries the failure guard (cuda_backend.cu:3938)
        require(static_cast<int64_t>(dims.size()) == static_cast<int64_t>(raw.ndim()), "permute rank mismatch");
        const DType dtype = operand_dtype(raw);
        Tensor x = copy_to_device(raw, dtype);
        std::vector<int64_t> shape(dims.size());
        std::vector<bool> seen(dims.size());
        for (size_t d = 0; d < dims.size(); ++d) {
            require(dims[d] >= 0 && dims[d] < static_cast<int64_t>(x.ndim()) && !seen[dims[d]], "Invalid permutation");
            seen[dims[d]] = true;
            shape[d] = x.shape()[dims[d]];
        }
        Tensor out = rt_->allocate_device(shape, dtype);
        ProfileRegion region(*this, [] { return std::string("permute"); }, bytes_of(x) + bytes_of(out));
        check(vrb_permute(x.data(), out.data(), code(dtype), static_cast<int>(dims.size()), x.shape().data(), dims.data(), kLegacyStream));
        return out;
    });
}

Tensor B200Backend::concat(const std::vector<Tensor>& inputs, int64_t dim) {
    return guarded([&] {   // VRHINO_PROFILE("concat") (cuda_backend.cu:3951)
        require(!inputs.empty(), "concat requires inputs");
        const int rank = static_cast<int>(inputs[0].ndim());
        if (dim < 0) dim += rank;
        require(dim >= 0 && dim < rank, "concat dimension invalid");
        std::vector<int64_t> shape = inputs[0].shape();
        shape[dim] = 0;
        for (const Tensor& input : inputs) {
            require(static_cast<int>(input.ndim()) == rank, "concat rank mismatch");
            for (int d = 0; d < rank; ++d)
                if (d != dim) require(input.shape()[d] == inputs[0].shape()[d], "concat shape mismatch");
            shape[dim] += input.shape()[dim];
        }
        const DType dtype = operand_dtype(inputs[0]);
        Tensor out = rt_->allocate_device(shape, dtype);
        std::vector<Tensor> parts;          // converted inputs stay alive until the launches are enqueued
        std::vector<const void*> pointers;
        std::vector<int64_t> extents;
        for (const Tensor& raw : inputs) {
            parts.push_back(copy_to_device(raw, dtype));
            pointers.push_back(parts.back().data());
            extents.push_back(raw.shape()[dim]);
        }
        ProfileRegion region(*this, [] { return std::string("concat"); }, 2 * bytes_of(out));
        check(vrb_concat(pointers.data(), extents.data(), static_cast<int>(parts.size()), out.data(), code(dtype), rank, shape.data(),
                         static_cast<int>(dim), kLegacyStream));
        return out;
    });
}

Tensor B200Backend::slice(const Tensor& raw, int64_t dim, int64_t start, int64_t stop) {
    return guarded([&] {   // VRHINO_PROFILE("slice") (cuda_backend.cu:3962)
        if (dim < 0) dim += static_cast<int64_t>(raw.ndim());
        require(dim >= 0 && dim < static_cast<int64_t>(raw.ndim()), "slice dimension invalid");
        const int64_t size = raw.shape()[dim];
        if (start < 0) start += size;
        if (stop < 0) stop += size;
        start = std::clamp<int64_t>(start, 0, size);
        stop = std::clamp<int64_t>(stop, start, size);
        std::vector<int64_t> shape = raw.shape();
        shape[dim] = stop - start;
        const DType dtype = operand_dtype(raw);
        Tensor x = copy_to_device(raw, dtype);
        Tensor out = rt_->allocate_device(shape, dtype);
        ProfileRegion region(*this, [] { return std::string("slice"); }, 2 * bytes_of(out));
        check(vrb_slice(x.data(), out.data(), code(dtype), static_cast<int>(x.ndim()), x.shape().data(), static_cast<int>(dim), start, stop,
                        kLegacyStream));
        return out;
    });
}

std::vector<Tensor> B200Backend::split(const Tensor& x, const std::vector<int64_t>& sections, int64_t dim) {
    // cuda_backend.cu:3972-3976: consecutive slices
    if (dim < 0) dim += static_cast<int64_t>(x.ndim());
    require(dim >= 0 && dim < static_cast<int64_t>(x.ndim()), "slice dimension invalid");
    int64_t total = 0;
    for (int64_t section : sections) total += section;
    require(total == x.shape()[dim], "split sections mismatch");
    std::vector<Tensor> result;
    int64_t offset = 0;
    for (int64_t section : sections) {
        result.push_back(slice(x, dim, offset, offset + section));
        offset += section;
    }
    return result;
}

Tensor B200Backend::sinusoidal_embedding(const Tensor& raw, int64_t width, bool flip, double downscale, bool frequency_f64) {
    return guarded([&] {   // VRHINO_PROFILE("sinusoidal_embedding") (cuda_backend.cu:4192)
        require(raw.ndim() == 1 && width > 0, "sinusoidal embedding contract violation");
        const DType dtype = operand_dtype(raw);
        Tensor positions = copy_to_device(raw, dtype);
        Tensor out = rt_->allocate_device({raw.numel(), width}, dtype);
        ProfileRegion region(*this, [] { return std::string("sinusoidal_embedding"); }, bytes_of(positions) + bytes_of(out));
        check(vrb_sinusoidal_embedding(positions.data(), out.data(), code(dtype), raw.numel(), width, flip ? 1 : 0, downscale,
                                       frequency_f64 ? 1 : 0, kLegacyStream));
        return out;
    });
}

Tensor B200Backend::pad(const Tensor& raw, const std::vector<int64_t>& padding, float value, vrhino::PadMode mode) {
    return guarded([&] {   // VRHINO_PROFILE("pad") (cuda_backend.cu:4877)
        require(padding.size() % 2 == 0 && padding.size() <= static_cast<size_t>(2 * raw.ndim()), "Invalid pad vector");
        const DType dtype = operand_dtype(raw);
        Tensor x = copy_to_device(raw, dtype);
        const int rank = static_cast<int>(x.ndim());
        std::vector<int64_t> shape = x.shape(), before(rank, 0), after(rank, 0);
        for (size_t pair = 0; pair < padding.size() / 2; ++pair) {
            const int d = rank - 1 - static_cast<int>(pair);
            require(padding[2 * pair] >= 0 && padding[2 * pair + 1] >= 0, "Negative padding unsupported");
            before[d] = padding[2 * pair];
            after[d] = padding[2 * pair + 1];
            shape[d] += before[d] + after[d];
        }
        Tensor out = rt_->allocate_device(shape, dtype);
        ProfileRegion region(*this, [] { return std::string("pad"); }, bytes_of(x) + bytes_of(out));
        check(vrb_pad(x.data(), out.data(), code(dtype), rank, x.shape().data(), before.data(), after.data(), value,
                      mode == vrhino::PadMode::Replicate ? 1 : 0, kLegacyStream));
        return out;
    });
}

Tensor B200Backend::interpolate_nearest(const Tensor& raw, const std::vector<double>& factors) {
    return guarded([&] {   // VRHINO_PROFILE("interpolate_nearest") (cuda_backend.cu:5012)
        require(factors.size() <= static_cast<size_t>(raw.ndim() - 2), "interpolate factor rank mismatch");
        const DType dtype = operand_dtype(raw);
        Tensor x = copy_to_device(raw, dtype);
        std::vector<int64_t> shape = x.shape();
        const size_t start = static_cast<size_t>(raw.ndim()) - factors.size();
        for (size_t index = 0; index < factors.size(); ++index) {
            require(factors[index] > 0, "Invalid interpolation factor");
            shape[start + index] = static_cast<int64_t>(std::floor(shape[start + index] * factors[index]));
        }
        Tensor out = rt_->allocate_device(shape, dtype);
        ProfileRegion region(*this, [] { return std::string("interpolate_nearest"); }, bytes_of(x) + bytes_of(out));
        check(vrb_interpolate_nearest(x.data(), out.data(), code(dtype), static_cast<int>(x.ndim()), x.shape().data(), shape.data(),
                                      kLegacyStream));
        return out;
    });
}

Tensor B200Backend::reduce_sum(const Tensor& raw, int64_t dim, bool keepdim) {
    return guarded([&] {   // VRHINO_PROFILE("reduce_sum") (cuda_backend.cu:4887)
        if (dim < 0) dim += static_cast<int64_t>(raw.ndim());
        require(dim >= 0 && dim < static_cast<int64_t>(raw.ndim()), "reduce dimension invalid");
        const DType dtype = operand_dtype(raw);
        Tensor x = copy_to_device(raw, dtype);
        std::vector<int64_t> shape = x.shape();
        int64_t outer = 1, inner = 1;
        for (int64_t d = 0; d < dim; ++d) outer *= shape[d];
        for (int64_t d = dim + 1; d < static_cast<int64_t>(shape.size()); ++d) inner *= shape[d];
        const int64_t reduced = shape[dim];
        if (keepdim) shape[dim] = 1;
        else shape.erase(shape.begin() + dim);
        Tensor out = rt_->allocate_device(shape, dtype);
        ProfileRegion region(*this, [] { return std::string("reduce_sum"); }, bytes_of(x) + bytes_of(out));
        check(vrb_reduce_sum(x.data(), out.data(), code(dtype), outer, reduced, inner, kLegacyStream));
        return out;
    });
}

Tensor B200Backend::rng_normal(vrhino::RngState& state, const std::vector<int64_t>& shape, DType dtype) {
    return guarded([&] {   // VRHINO_PROFILE("rng_normal") (cuda_backend.cu:5122)
        require(state.algorithm_id == "pytorch_compat.v1", "Unsupported RNG algorithm");
        require(dtype == DType::F32 || dtype == DType::BF16, "rng_normal dtype unsupported");
        Tensor out = rt_->allocate_device(shape, dtype);
        ProfileRegion region(*this, [] { return std::string("rng_normal"); }, bytes_of(out));
        check(vrb_rng_normal(out.data(), code(dtype), out.numel(), state.seed, state.offset, kLegacyStream));
        state.offset += 4;
        return out;
    });
}

Tensor B200Backend::softmax(const Tensor& raw, int64_t axis) {
    return guarded([&] {   // VRHINO_PROFILE("softmax") (cuda_backend.cu:4895)
        if (axis < 0) axis += static_cast<int64_t>(raw.ndim());
        require(axis >= 0 && axis < static_cast<int64_t>(raw.ndim()), "softmax axis invalid");
        const DType dtype = operand_dtype(raw);
        Tensor x = copy_to_device(raw, dtype);
        int64_t outer = 1, inner = 1;
        for (int64_t d = 0; d < axis; ++d) outer *= x.dim(d);
        for (int64_t d = axis + 1; d < static_cast<int64_t>(x.ndim()); ++d) inner *= x.dim(d);
        Tensor out = rt_->allocate_device(x.shape(), dtype);
        ProfileRegion region(*this, [] { return std::string("softmax"); }, bytes_of(x) + bytes_of(out));
        check(vrb_softmax(x.data(), out.data(), code(dtype), outer, x.dim(axis), inner, kLegacyStream));
        return out;
    });
}

Tensor B200Backend::indexed_gather(const Tensor& table_raw, const Tensor& indices_raw) {
    return guarded([&] {   // VRHINO_PROFILE("indexed_gather") (cuda_backend.cu:3983)
        require(table_raw.ndim() == 2 || table_raw.ndim() == 3, "indexed_gather table must have rank 2 or 3");
        require(indices_raw.ndim() >= 1 && (indices_raw.dtype() == DType::I64 || indices_raw.dtype() == DType::I32),
                "indexed_gather indices must be rank >=1 int64/int32");
        const bool batched = table_raw.ndim() == 3;
        if (batched) require(indices_raw.dim(0) == table_raw.dim(0), "indexed_gather batch dimension mismatch");
        // quantised tables and dense host tables (of which the reference uploads the selected rows only) keep the runtime's path
        if (table_raw.is_quantized() || table_raw.device().is_host()) return rt_->indexed_gather(table_raw, indices_raw);
        const int64_t rows = table_raw.dim(batched ? 1 : 0), width = table_raw.dim(-1);
        const Tensor host_indices = indices_raw.device().is_host() ? indices_raw : copy_to_host(indices_raw);
        for (int64_t k = 0; k < host_indices.numel(); ++k) {
            const int64_t value = host_indices.dtype() == DType::I64 ? host_indices.data_as<int64_t>()[k]
                                                                      : static_cast<int64_t>(host_indices.data_as<int32_t>()[k]);
            require(value >= 0 && value < rows, "indexed_gather index out of range");
        }
        const DType dtype = execution_dtype();
        Tensor table = copy_to_device(table_raw, dtype);
        Tensor indices = copy_to_device(indices_raw, indices_raw.dtype());
        std::vector<int64_t> shape = indices_raw.shape();
        shape.push_back(width);
        Tensor out = rt_->allocate_device(shape, dtype);
        const int64_t per_batch = batched ? (indices_raw.dim(0) ? indices_raw.numel() / indices_raw.dim(0) : 0) : indices_raw.numel();
        ProfileRegion region(*this, [] { return std::string("indexed_gather"); }, 2 * bytes_of(out));
        check(vrb_indexed_gather(table.data(), indices.data(), indices_raw.dtype() == DType::I64 ? VRB_I64 : VRB_I32, out.data(), code(dtype),
                                 batched ? table.dim(0) : 0, rows, width, per_batch, kLegacyStream));
        return out;
    });
}

Tensor B200Backend::pad_axes(const Tensor& raw, const std::vector<int64_t>& before, const std::vector<int64_t>& after, float value,
                             const std::vector<bool>& replicate) {
    return guarded([&] {
        const size_t rank = static_cast<size_t>(raw.ndim());
        require(before.size() == rank && after.size() == rank && replicate.size() == rank, "Invalid pad vector");
        const DType dtype = operand_dtype(raw);
        Tensor x = copy_to_device(raw, dtype);
        std::vector<int64_t> shape = x.shape();
        std::vector<int> modes(rank);
        for (size_t d = 0; d < rank; ++d) {
            require(before[d] >= 0 && after[d] >= 0, "Negative padding unsupported");
            shape[d] += before[d] + after[d];
            modes[d] = replicate[d] ? 1 : 0;
        }
        Tensor out = rt_->allocate_device(shape, dtype);
        ProfileRegion region(*this, [] { return std::string("fused.pad"); }, bytes_of(x) + bytes_of(out));
        check(vrb_pad_axes(x.data(), out.data(), code(dtype), static_cast<int>(rank), x.shape().data(), before.data(), after.data(), value,
                           modes.data(), kLegacyStream));
        return out;
    });
}

Tensor B200Backend::pixel_shuffle_nd(const Tensor& raw, const std::vector<int64_t>& factors) {
    return guarded([&] {   // VRHINO_PROFILE("pixel_shuffle") carries the failure guard (cuda_backend.cu:5114)
        require(raw.ndim() == 5 && factors.size() == 3, "pixel_shuffle_nd requires 5D and 3 factors");
        const int64_t product = factors[0] * factors[1] * factors[2];
        require(product > 0 && raw.dim(1) % product == 0, "pixel shuffle channel mismatch");
        const DType dtype = operand_dtype(raw);
        Tensor x = copy_to_device(raw, dtype);
        Tensor out = rt_->allocate_device({x.dim(0), x.dim(1) / product, x.dim(2) * factors[0], x.dim(3) * factors[1],
                                           x.dim(4) * factors[2]}, dtype);
        ProfileRegion region(*this, [] { return std::string("pixel_shuffle"); }, bytes_of(x) + bytes_of(out));
        check(vrb_pixel_shuffle(x.data(), out.data(), code(dtype), x.dim(0), x.dim(1) / product, x.dim(2), x.dim(3), x.dim(4),
                                static_cast<int>(factors[0]), static_cast<int>(factors[1]), static_cast<int>(factors[2]),
                                kLegacyStream));
        return out;
    });
}

// ---- fused forms --------------------------------------------------------------------------------

Tensor B200Backend::depth_to_space_residual(const Tensor& projected_raw, const Tensor& input_raw) {
    return guarded([&] {
        require(input_raw.ndim() == 5 && projected_raw.ndim() == 5, "pixel_shuffle_nd requires 5D and 3 factors");
        const DType dtype = operand_dtype(projected_raw);
        Tensor projected = copy_to_device(projected_raw, dtype), input = copy_to_device(input_raw, dtype);
        require(input.dim(1) % 8 == 0 && projected.dim(1) == 4 * input.dim(1), "pixel shuffle channel mismatch");
        require(projected.dim(0) == input.dim(0) && projected.dim(2) == input.dim(2) && projected.dim(3) == input.dim(3) &&
                    projected.dim(4) == input.dim(4), "Incompatible broadcast shapes");
        Tensor out = rt_->allocate_device({input.dim(0), input.dim(1) / 2, 2 * input.dim(2) - 1, 2 * input.dim(3),
                                           2 * input.dim(4)}, dtype);
        ProfileRegion region(*this, [] { return std::string("fused.depth_to_space_residual"); }, bytes_of(projected) + bytes_of(input) + bytes_of(out));
        check(vrb_depth_to_space_residual(projected.data(), input.data(), out.data(), code(dtype), input.dim(0), input.dim(1),
                                          input.dim(2), input.dim(3), input.dim(4), kLegacyStream));
        return out;
    });
}

Tensor B200Backend::pixel_norm_modulate(const Tensor& raw, const Tensor& shift_raw, const Tensor& scale_raw, float eps,
                                        bool silu, DType output) {
    return guarded([&] {
        require(raw.ndim() >= 2, "pixel norm dim invalid");
        const DType dtype = operand_dtype(raw);
        Tensor x = copy_to_device(raw, dtype);
        const int64_t batch = x.dim(0), channels = x.dim(1), inner = x.numel() / (batch * channels);
        Tensor scale = parameter(scale_raw), shift = copy_to_device(shift_raw, scale.dtype());
        require(scale.numel() == batch * channels && shift.numel() == scale.numel(), "Incompatible broadcast shapes");
        Tensor out = rt_->allocate_device(x.shape(), output);
        ProfileRegion region(*this, [] { return std::string("fused.norm.pixel+modulate"); }, bytes_of(x) + bytes_of(out));
        check(vrb_pixel_norm(x.data(), code(dtype), scale.data(), shift.data(), code(scale.dtype()), silu ? 1 : 0, out.data(),
                             code(output), batch, channels, inner, eps, kLegacyStream));
        return out;
    });
}

Tensor B200Backend::layer_norm_modulate(const Tensor& raw, const Tensor* weight_raw, const Tensor* bias_raw, float eps,
                                        const Tensor& shift_raw, const Tensor& scale_raw, DType output) {
    return guarded([&] {
        const DType dtype = operand_dtype(raw);
        Tensor x = copy_to_device(raw, dtype), weight, bias;
        const int64_t width = x.dim(-1), rows = x.numel() / width;
        if (weight_raw) { weight = parameter(*weight_raw); require(weight.numel() == width, "layer norm weight mismatch"); }
        if (bias_raw) { bias = parameter(*bias_raw); require(bias.numel() == width, "layer norm bias mismatch"); }
        Tensor scale = parameter(scale_raw), shift = copy_to_device(shift_raw, scale.dtype());
        require(shift.numel() == scale.numel(), "modulate: shift and scale must share dtype and shape");
        int64_t rows_per_vector = 0, vectors = 0;
        vector_layout(x, scale, rows_per_vector, vectors);
        Tensor out = rt_->allocate_device(x.shape(), output);
        ProfileRegion region(*this, [] { return std::string("fused.norm.layer+modulate"); }, bytes_of(x) + bytes_of(out));
        check(vrb_layer_norm_modulate(x.data(), code(dtype), weight_raw ? weight.data() : nullptr,
                                      weight_raw ? code(weight.dtype()) : 0, bias_raw ? bias.data() : nullptr,
                                      bias_raw ? code(bias.dtype()) : 0, scale.data(), shift.data(), code(scale.dtype()),
                                      rows_per_vector, vectors, out.data(), code(output), rows, width, eps, kLegacyStream));
        return out;
    });
}

Tensor B200Backend::rms_norm_modulate(const Tensor& raw, float eps, const Tensor& shift_raw, const Tensor& scale_raw, DType output) {
    return guarded([&] {
        const DType dtype = operand_dtype(raw);
        Tensor x = copy_to_device(raw, dtype);
        const int64_t width = x.dim(-1), rows = x.numel() / width;
        Tensor scale = parameter(scale_raw), shift = copy_to_device(shift_raw, scale.dtype());
        require(shift.numel() == scale.numel(), "modulate: shift and scale must share dtype and shape");
        int64_t rows_per_vector = 0, vectors = 0;
        vector_layout(x, scale, rows_per_vector, vectors);
        Tensor out = rt_->allocate_device(x.shape(), output);
        ProfileRegion region(*this, [] { return std::string("fused.norm.rms+modulate"); }, bytes_of(x) + bytes_of(out));
        check(vrb_rms_norm_modulate(x.data(), code(dtype), scale.data(), shift.data(), code(scale.dtype()), rows_per_vector,
                                    vectors, out.data(), code(output), rows, width, eps, kLegacyStream));
        return out;
    });
}

Tensor B200Backend::rms_norm_rope(const Tensor& raw, const Tensor* weight_raw, float eps, const Tensor* cos_raw,
                                  const Tensor* sin_raw, int heads, bool per_head_norm, DType output) {
    return guarded([&] {
        require(raw.ndim() == 3 && heads > 0 && raw.dim(2) % heads == 0, "split_heads shape mismatch");
        const DType dtype = operand_dtype(raw);
        Tensor x = copy_to_device(raw, dtype), weight, c, s;
        const int64_t width = x.dim(2), rows = x.numel() / width, head_width = width / heads;
        const int64_t norm_width = per_head_norm ? head_width : width;
        if (weight_raw) { weight = parameter(*weight_raw); require(weight.numel() == norm_width, "rms norm weight mismatch"); }
        int64_t f_rows = 0, f_width = 8;
        DType table_dtype = DType::F32;
        if (cos_raw) {
            require(sin_raw != nullptr, "RoPE frequency mismatch");
            // tables keep their device dtype (F32 or BF16), as rope_nd does (cuda_backend.cu:4201-4203)
            table_dtype = device_float(*cos_raw) ? cos_raw->dtype() : DType::F32;
            c = copy_to_device(*cos_raw, table_dtype);
            s = copy_to_device(*sin_raw, table_dtype);
            require(c.shape() == s.shape(), "RoPE frequency mismatch");
            require(c.ndim() >= 2, "Incompatible broadcast shapes");
            // [.., S, H|1, d] tables, or [.., S, D] tables spanning the whole row (LTX)
            f_width = c.dim(-1) == width ? width : c.dim(-1) * c.dim(-2);
            require((c.dim(-1) == head_width || c.dim(-1) == width) && (f_width == head_width || f_width == width),
                    "Incompatible broadcast shapes");
            f_rows = c.numel() / f_width;
            require(f_rows == rows || f_rows == rows / x.dim(0), "Incompatible broadcast shapes");
        }
        Tensor out = rt_->allocate_device(x.shape(), output);
        ProfileRegion region(*this, [] { return std::string("fused.norm.rms+rope"); }, bytes_of(x) + bytes_of(out));
        check(vrb_rms_norm_rope_tables(x.data(), code(dtype), weight_raw ? weight.data() : nullptr,
                                       weight_raw ? code(weight.dtype()) : 0, cos_raw ? c.data() : nullptr,
                                       cos_raw ? s.data() : nullptr, code(table_dtype), f_rows, f_width, 1, out.data(),
                                       code(output), rows, width, norm_width, eps, kLegacyStream));
        return out;
    });
}

std::pair<Tensor, Tensor> B200Backend::rms_norm_rope_pair(const Tensor& a_raw, const Tensor& weight_a_raw, const Tensor& b_raw,
                                                          const Tensor& weight_b_raw, float eps, const Tensor* cos_raw,
                                                          const Tensor* sin_raw, int heads, bool per_head_norm, DType output) {
    std::pair<Tensor, Tensor> result;
    guarded([&] {
        require(a_raw.ndim() == 3 && b_raw.ndim() == 3 && heads > 0 && a_raw.dim(2) % heads == 0 && a_raw.dim(2) == b_raw.dim(2),
                "split_heads shape mismatch");
        const DType dtype = operand_dtype(a_raw);
        require(operand_dtype(b_raw) == dtype, "Incompatible broadcast shapes");
        Tensor a = copy_to_device(a_raw, dtype), b = copy_to_device(b_raw, dtype), c, s;
        const int64_t width = a.dim(2), rows_a = a.numel() / width, rows_b = b.numel() / width, head_width = width / heads;
        const int64_t norm_width = per_head_norm ? head_width : width;
        Tensor weight_a = parameter(weight_a_raw), weight_b = copy_to_device(weight_b_raw, weight_a.dtype());
        require(weight_a.numel() == norm_width && weight_b.numel() == norm_width, "rms norm weight mismatch");
        int64_t f_rows = 0, f_width = 8;
        DType table_dtype = DType::F32;
        if (cos_raw) {
            require(sin_raw != nullptr, "RoPE frequency mismatch");
            table_dtype = device_float(*cos_raw) ? cos_raw->dtype() : DType::F32;
            c = copy_to_device(*cos_raw, table_dtype);
            s = copy_to_device(*sin_raw, table_dtype);
            require(c.shape() == s.shape() && c.ndim() >= 2, "RoPE frequency mismatch");
            f_width = c.dim(-1) == width ? width : c.dim(-1) * c.dim(-2);
            require((c.dim(-1) == head_width || c.dim(-1) == width) && (f_width == head_width || f_width == width),
                    "Incompatible broadcast shapes");
            f_rows = c.numel() / f_width;
            require((f_rows == rows_a || f_rows == rows_a / a.dim(0)) && (f_rows == rows_b || f_rows == rows_b / b.dim(0)),
                    "Incompatible broadcast shapes");
        }
        result.first = rt_->allocate_device(a.shape(), output);
        result.second = rt_->allocate_device(b.shape(), output);
        ProfileRegion region(*this, [] { return std::string("fused.norm.rms+rope.pair"); },
                             bytes_of(a) + bytes_of(b) + bytes_of(result.first) + bytes_of(result.second));
        check(vrb_rms_norm_rope_pair(a.data(), weight_a.data(), result.first.data(), rows_a, b.data(), weight_b.data(),
                                     result.second.data(), rows_b, code(dtype), code(weight_a.dtype()), cos_raw ? c.data() : nullptr,
                                     cos_raw ? s.data() : nullptr, code(table_dtype), f_rows, f_width, 1, code(output), width,
                                     norm_width, eps, kLegacyStream));
        return result.first;
    });
    return result;
}

std::pair<Tensor, Tensor> B200Backend::normalized_gated_residual_norm_scale(const Tensor& residual_raw, const Tensor& branch_raw,
                                                                            const Tensor& gate_raw, const Tensor& scale_raw,
                                                                            DType state, float branch_eps, float eps) {
    std::pair<Tensor, Tensor> result;
    guarded([&] {
        Tensor residual = copy_to_device(residual_raw, operand_dtype(residual_raw));
        Tensor branch = copy_to_device(branch_raw, operand_dtype(branch_raw));
        require(residual.shape() == branch.shape(), "Incompatible broadcast shapes");
        Tensor gate = parameter(gate_raw), scale = parameter(scale_raw);
        const int64_t width = residual.dim(-1), rows = residual.numel() / width;
        int64_t gate_rows = 1, gate_vectors = 1, scale_rows = 1, scale_vectors = 1;
        vector_layout(residual, gate, gate_rows, gate_vectors);
        vector_layout(residual, scale, scale_rows, scale_vectors);
        const bool one_pass = residual.dtype() == DType::BF16 && branch.dtype() == DType::BF16 && state == DType::BF16;
        if (!one_pass) gate = activation(gate, vrhino::Activation::Tanh);   // a temporary of [B, D]
        result.first = rt_->allocate_device(residual.shape(), state);
        result.second = rt_->allocate_device(residual.shape(), state);
        ProfileRegion region(*this, [] { return std::string("fused.mochi.residual+norm"); },
                             bytes_of(residual) + bytes_of(branch) + bytes_of(result.first) + bytes_of(result.second));
        check(vrb_rms_norm_gated_residual_rms_norm_scale(residual.data(), code(residual.dtype()), branch.data(), code(branch.dtype()),
                                                         branch_eps, gate.data(), code(gate.dtype()), one_pass ? 1 : 0, gate_rows,
                                                         gate_vectors, result.first.data(), code(state), scale.data(),
                                                         code(scale.dtype()), scale_rows, scale_vectors, result.second.data(), rows,
                                                         width, eps, kLegacyStream));
        return result.first;
    });
    return result;
}

Tensor B200Backend::gated_residual(const Tensor& residual_raw, const Tensor& branch_raw, const Tensor* gate_raw, DType state) {
    return guarded([&] {
        Tensor residual = copy_to_device(residual_raw, operand_dtype(residual_raw));
        Tensor branch = copy_to_device(branch_raw, operand_dtype(branch_raw)), gate;
        require(residual.shape() == branch.shape(), "Incompatible broadcast shapes");
        const int64_t width = residual.dim(-1), rows = residual.numel() / width;
        int64_t rows_per_vector = 1, vectors = 1;
        if (gate_raw) { gate = parameter(*gate_raw); vector_layout(residual, gate, rows_per_vector, vectors); }
        Tensor out = rt_->allocate_device(residual.shape(), state);
        ProfileRegion region(*this, [] { return std::string("fused.gated_residual"); }, bytes_of(residual) + bytes_of(branch) + bytes_of(out));
        check(vrb_gated_residual(residual.data(), code(residual.dtype()), branch.data(), code(branch.dtype()),
                                 gate_raw ? gate.data() : nullptr, gate_raw ? code(gate.dtype()) : 0, rows_per_vector,
                                 vectors, out.data(), code(state), rows, width, kLegacyStream));
        return out;
    });
}

std::pair<Tensor, Tensor> B200Backend::gated_residual_layer_norm(const Tensor& residual_raw, const Tensor& branch_raw,
                                                                 const Tensor* gate_raw, DType state, const Tensor* weight_raw,
                                                                 const Tensor* bias_raw, float eps, const Tensor* shift_raw,
                                                                 const Tensor* scale_raw, DType output) {
    std::pair<Tensor, Tensor> result;
    guarded([&] {
        Tensor residual = copy_to_device(residual_raw, operand_dtype(residual_raw));
        Tensor branch = copy_to_device(branch_raw, operand_dtype(branch_raw)), gate, weight, bias, scale, shift;
        require(residual.shape() == branch.shape(), "Incompatible broadcast shapes");
        require((shift_raw == nullptr) == (scale_raw == nullptr), "modulate: shift and scale must share dtype and shape");
        const int64_t width = residual.dim(-1), rows = residual.numel() / width;
        int64_t gate_rows_per_vector = 1, gate_vectors = 1, rows_per_vector = 1, vectors = 1;
        if (gate_raw) { gate = parameter(*gate_raw); vector_layout(residual, gate, gate_rows_per_vector, gate_vectors); }
        if (weight_raw) { weight = parameter(*weight_raw); require(weight.numel() == width, "layer norm weight mismatch"); }
        if (bias_raw) { bias = parameter(*bias_raw); require(bias.numel() == width, "layer norm bias mismatch"); }
        if (scale_raw) {
            scale = parameter(*scale_raw);
            shift = copy_to_device(*shift_raw, scale.dtype());
            require(shift.numel() == scale.numel(), "modulate: shift and scale must share dtype and shape");
            vector_layout(residual, scale, rows_per_vector, vectors);
        }
        result.first = rt_->allocate_device(residual.shape(), state);
        result.second = rt_->allocate_device(residual.shape(), output);
        ProfileRegion region(*this, [] { return std::string("fused.gated_residual+norm.layer"); }, bytes_of(residual) + bytes_of(branch) + bytes_of(result.first) + bytes_of(result.second));
        check(vrb_gated_residual_layer_norm_modulate(
            residual.data(), code(residual.dtype()), branch.data(), code(branch.dtype()), gate_raw ? gate.data() : nullptr,
            gate_raw ? code(gate.dtype()) : 0, gate_rows_per_vector, gate_vectors, result.first.data(), code(state),
            weight_raw ? weight.data() : nullptr, weight_raw ? code(weight.dtype()) : 0, bias_raw ? bias.data() : nullptr,
            bias_raw ? code(bias.dtype()) : 0, scale_raw ? scale.data() : nullptr, scale_raw ? shift.data() : nullptr,
            scale_raw ? code(scale.dtype()) : 0, rows_per_vector, vectors, result.second.data(), code(output), rows, width,
            eps, kLegacyStream));
        return result.second;
    });
    return result;
}

namespace {
// The merged epilogue applies where the reference's linear would run fused_bf16_linear_output_kernel:
// bf16 compute and bf16 output, weights not quantised (cuda_backend.cu:3678-3790 take another route).
bool merged_linear_applies(const B200Backend& backend, const Tensor& weight) {
    return backend.execution_dtype() == DType::BF16 && !weight.is_quantized();
}
}  // namespace

Tensor B200Backend::linear_activation(const Tensor& x, const Tensor& weight, const Tensor* bias_raw, vrhino::Activation kind) {
    if (!merged_linear_applies(*this, weight)) return activation(linear(x, weight, bias_raw), kind);
    return guarded([&] {
        Tensor accumulation = rt_->linear(x, weight, nullptr, DType::BF16, DType::F32);
        const int64_t width = accumulation.dim(-1), rows = accumulation.numel() / width;
        Tensor bias;
        if (bias_raw) { bias = copy_to_device(*bias_raw, DType::BF16); require(bias.numel() == width, "linear bias mismatch"); }
        Tensor out = rt_->allocate_device(accumulation.shape(), DType::BF16);
        ProfileRegion region(*this, [] { return std::string("fused.linear_output+activation"); }, bytes_of(accumulation) + bytes_of(out));
        check(vrb_linear_output_activation(accumulation.data_as<float>(), bias_raw ? bias.data() : nullptr, static_cast<int>(kind),
                                           out.data(), rows, width, kLegacyStream));
        return out;
    });
}

Tensor B200Backend::linear_gated_residual(const Tensor& residual_raw, const Tensor& x, const Tensor& weight,
                                          const Tensor* bias_raw, const Tensor* gate_raw, DType state) {
    if (!merged_linear_applies(*this, weight)) return gated_residual(residual_raw, linear(x, weight, bias_raw), gate_raw, state);
    return guarded([&] {
        Tensor accumulation = rt_->linear(x, weight, nullptr, DType::BF16, DType::F32);
        Tensor residual = copy_to_device(residual_raw, operand_dtype(residual_raw)), bias, gate;
        require(residual.shape() == accumulation.shape(), "Incompatible broadcast shapes");
        const int64_t width = accumulation.dim(-1), rows = accumulation.numel() / width;
        if (bias_raw) { bias = copy_to_device(*bias_raw, DType::BF16); require(bias.numel() == width, "linear bias mismatch"); }
        int64_t rows_per_vector = 1, vectors = 1;
        if (gate_raw) { gate = parameter(*gate_raw); vector_layout(residual, gate, rows_per_vector, vectors); }
        Tensor out = rt_->allocate_device(residual.shape(), state);
        ProfileRegion region(*this, [] { return std::string("fused.linear_output+gated_residual"); }, bytes_of(accumulation) + bytes_of(residual) + bytes_of(out));
        check(vrb_linear_output_gated_residual(accumulation.data_as<float>(), bias_raw ? bias.data() : nullptr, residual.data(),
                                               code(residual.dtype()), gate_raw ? gate.data() : nullptr,
                                               gate_raw ? code(gate.dtype()) : 0, rows_per_vector, vectors, out.data(),
                                               code(state), rows, width, kLegacyStream));
        return out;
    });
}

Tensor B200Backend::linear_swiglu(const Tensor& x, const Tensor& weight, const Tensor* bias_raw) {
    if (!merged_linear_applies(*this, weight)) return swiglu(linear(x, weight, bias_raw));
    return guarded([&] {
        Tensor accumulation = rt_->linear(x, weight, nullptr, DType::BF16, DType::F32);
        const int64_t width = accumulation.dim(-1), rows = accumulation.numel() / width;
        require(width % 2 == 0, "split sections mismatch");
        Tensor bias;
        if (bias_raw) { bias = copy_to_device(*bias_raw, DType::BF16); require(bias.numel() == width, "linear bias mismatch"); }
        std::vector<int64_t> shape = accumulation.shape();
        shape.back() = width / 2;
        Tensor out = rt_->allocate_device(shape, DType::BF16);
        ProfileRegion region(*this, [] { return std::string("fused.linear_output+swiglu"); }, bytes_of(accumulation) + bytes_of(out));
        check(vrb_linear_output_swiglu(accumulation.data_as<float>(), bias_raw ? bias.data() : nullptr, out.data(), rows,
                                       width / 2, kLegacyStream));
        return out;
    });
}

Tensor B200Backend::swiglu(const Tensor& raw) {
    return guarded([&] {
        const DType dtype = operand_dtype(raw);
        Tensor projected = copy_to_device(raw, dtype);
        require(projected.dim(-1) % 2 == 0, "split sections mismatch");
        const int64_t hidden = projected.dim(-1) / 2, rows = projected.numel() / (2 * hidden);
        std::vector<int64_t> shape = projected.shape();
        shape.back() = hidden;
        Tensor out = rt_->allocate_device(shape, dtype);
        ProfileRegion region(*this, [] { return std::string("fused.swiglu"); }, bytes_of(projected) + bytes_of(out));
        check(vrb_swiglu(projected.data(), out.data(), code(dtype), rows, hidden, kLegacyStream));
        return out;
    });
}

Tensor B200Backend::linear_combine(const std::vector<Tensor>& values, const std::vector<float>& coefficients,
                                   bool declared_role) {
    return guarded([&] {
        require(!values.empty() && values.size() == coefficients.size() && values.size() <= 4, "linear combine arity mismatch");
        const DType dtype = operand_dtype(values[0]);
        std::vector<Tensor> device;
        std::vector<const void*> pointers;
        for (const Tensor& v : values) {
            device.push_back(copy_to_device(v, dtype));
            require(device.back().shape() == device.front().shape(), "Incompatible broadcast shapes");
            pointers.push_back(device.back().data());
        }
        Tensor out = rt_->allocate_device(device.front().shape(), dtype);
        ProfileRegion region(*this, [] { return std::string("fused.sampler.linear_combine"); }, bytes_of(out) * (values.size() + 1));
        check(vrb_linear_combine(pointers.data(), coefficients.data(), static_cast<int>(values.size()), out.data(), code(dtype),
                                 out.numel(), declared_role ? 1 : 0, kLegacyStream));
        return out;
    });
}

Tensor B200Backend::cfg_euler(const Tensor& sample_raw, const Tensor& u_raw, const Tensor& c_raw, float guidance,
                              float delta, bool subtract_prediction, bool guidance_role, bool solver_role) {
    return guarded([&] {
        const DType dtype = operand_dtype(sample_raw);
        Tensor sample = copy_to_device(sample_raw, dtype), u = copy_to_device(u_raw, dtype), c = copy_to_device(c_raw, dtype);
        require(sample.shape() == u.shape() && u.shape() == c.shape(), "Incompatible broadcast shapes");
        Tensor out = rt_->allocate_device(sample.shape(), dtype);
        ProfileRegion region(*this, [] { return std::string("fused.sampler.cfg+euler"); }, bytes_of(out) * 4);
        check(vrb_cfg_euler(sample.data(), u.data(), c.data(), nullptr, out.data(), code(dtype), sample.numel(), guidance,
                            delta, subtract_prediction ? 1 : 0, guidance_role ? 1 : 0, solver_role ? 1 : 0, kLegacyStream));
        return out;
    });
}

// ---- call-site view -----------------------------------------------------------------------------

Tensor layer_norm_modulate(vrhino::Backend& backend, const vrhino::PrecisionPolicy& policy, const Tensor& x,
                           const Tensor* weight, const Tensor* bias, float eps, const Tensor& shift, const Tensor& scale,
                           DType output) {
    if (auto* b200 = dynamic_cast<B200Backend*>(&backend))
        return b200->layer_norm_modulate(x, weight, bias, eps, shift, scale, output);
    return backend.cast(vrhino::modulate(backend, policy, backend.layer_norm(x, weight, bias, eps), shift, scale), output);
}

Tensor rms_norm_rope(vrhino::Backend& backend, const vrhino::PrecisionPolicy& policy, const Tensor& x, const Tensor* weight,
                     float eps, const Tensor* cosine, const Tensor* sine, int heads, bool per_head_norm, DType output) {
    if (auto* b200 = dynamic_cast<B200Backend*>(&backend))
        return b200->rms_norm_rope(x, weight, eps, cosine, sine, heads, per_head_norm, output);
    Tensor t = per_head_norm ? vrhino::attention_norm(backend, policy, vrhino::split_heads(backend, x, heads), weight, eps)
                             : vrhino::split_heads(backend, vrhino::attention_norm(backend, policy, x, weight, eps), heads);
    if (cosine) t = vrhino::operation_rope(backend, policy, t, *cosine, *sine);
    return backend.cast(vrhino::merge_heads(backend, t), output);
}

std::pair<Tensor, Tensor> rms_norm_rope_pair(vrhino::Backend& backend, const vrhino::PrecisionPolicy& policy, const Tensor& q,
                                             const Tensor& weight_q, const Tensor& k, const Tensor& weight_k, float eps,
                                             const Tensor* cosine, const Tensor* sine, int heads, bool per_head_norm, DType output) {
    if (auto* b200 = dynamic_cast<B200Backend*>(&backend))
        return b200->rms_norm_rope_pair(q, weight_q, k, weight_k, eps, cosine, sine, heads, per_head_norm, output);
    return {rms_norm_rope(backend, policy, q, &weight_q, eps, cosine, sine, heads, per_head_norm, output),
            rms_norm_rope(backend, policy, k, &weight_k, eps, cosine, sine, heads, per_head_norm, output)};
}

std::pair<Tensor, Tensor> normalized_gated_residual_norm_scale(vrhino::Backend& backend, const vrhino::PrecisionPolicy& policy,
                                                               const Tensor& residual, const Tensor& branch, const Tensor& gate,
                                                               const Tensor& scale, float eps) {
    if (auto* b200 = dynamic_cast<B200Backend*>(&backend))
        return b200->normalized_gated_residual_norm_scale(residual, branch, gate, scale,
                                                          policy.persistent_state_dtype(vrhino::PrecisionSemantic::ResidualState),
                                                          eps, eps);
    // the block's own operator sequence (mochi.cpp:204-211, :228-231)
    const std::vector<int64_t> row{residual.dim(0), 1, residual.dim(-1)};
    Tensor bounded = backend.reshape(backend.activation(gate, vrhino::Activation::Tanh), row);
    Tensor state = vrhino::gated_residual(backend, policy, residual, backend.rms_norm(branch, nullptr, eps), bounded);
    Tensor factor = backend.add(vrhino::scalar_f32(1.0f), backend.reshape(scale, row));
    return {state, backend.mul(backend.rms_norm(state, nullptr, eps), factor)};
}

Tensor fused_gated_residual(vrhino::Backend& backend, const vrhino::PrecisionPolicy& policy, const Tensor& residual,
                            const Tensor& branch, const Tensor* gate) {
    if (auto* b200 = dynamic_cast<B200Backend*>(&backend))
        return b200->gated_residual(residual, branch, gate, policy.persistent_state_dtype(vrhino::PrecisionSemantic::ResidualState));
    return gate ? vrhino::gated_residual(backend, policy, residual, branch, *gate)
                : vrhino::residual_add(backend, policy, residual, branch);
}

std::pair<Tensor, Tensor> fused_gated_residual_layer_norm(vrhino::Backend& backend, const vrhino::PrecisionPolicy& policy,
                                                          const Tensor& residual, const Tensor& branch, const Tensor* gate,
                                                          const Tensor* weight, const Tensor* bias, float eps,
                                                          const Tensor* shift, const Tensor* scale, DType output) {
    if (auto* b200 = dynamic_cast<B200Backend*>(&backend))
        return b200->gated_residual_layer_norm(residual, branch, gate,
                                               policy.persistent_state_dtype(vrhino::PrecisionSemantic::ResidualState), weight,
                                               bias, eps, shift, scale, output);
    Tensor state = gate ? vrhino::gated_residual(backend, policy, residual, branch, *gate)
                        : vrhino::residual_add(backend, policy, residual, branch);
    Tensor normed = backend.layer_norm(state, weight, bias, eps);
    if (scale) normed = vrhino::modulate(backend, policy, normed, *shift, *scale);
    return {state, backend.cast(normed, output)};
}

Tensor linear_activation(vrhino::Backend& backend, const Tensor& x, const Tensor& weight, const Tensor* bias,
                         vrhino::Activation kind) {
    if (auto* b200 = dynamic_cast<B200Backend*>(&backend)) return b200->linear_activation(x, weight, bias, kind);
    return backend.activation(backend.linear(x, weight, bias), kind);
}

Tensor linear_gated_residual(vrhino::Backend& backend, const vrhino::PrecisionPolicy& policy, const Tensor& residual,
                             const Tensor& x, const Tensor& weight, const Tensor* bias, const Tensor* gate) {
    if (auto* b200 = dynamic_cast<B200Backend*>(&backend))
        return b200->linear_gated_residual(residual, x, weight, bias, gate,
                                           policy.persistent_state_dtype(vrhino::PrecisionSemantic::ResidualState));
    Tensor branch = backend.linear(x, weight, bias);
    return gate ? vrhino::gated_residual(backend, policy, residual, branch, *gate)
                : vrhino::residual_add(backend, policy, residual, branch);
}

Tensor linear_swiglu(vrhino::Backend& backend, const Tensor& x, const Tensor& weight, const Tensor* bias) {
    if (auto* b200 = dynamic_cast<B200Backend*>(&backend)) return b200->linear_swiglu(x, weight, bias);
    return swiglu(backend, backend.linear(x, weight, bias));
}

Tensor pixel_norm_modulate_silu(vrhino::Backend& backend, const vrhino::PrecisionPolicy& policy, const Tensor& x,
                                const Tensor& shift, const Tensor& scale, float eps, DType output) {
    if (auto* b200 = dynamic_cast<B200Backend*>(&backend)) return b200->pixel_norm_modulate(x, shift, scale, eps, true, output);
    Tensor y = backend.activation(vrhino::modulate(backend, policy, backend.pixel_norm(x, 1, eps), shift, scale),
                                  vrhino::Activation::Silu);
    return y.dtype() == output ? y : backend.cast(y, output);
}

Tensor edge_time_pad(vrhino::Backend& backend, const Tensor& x, int64_t temporal, int64_t pad_h, int64_t pad_w) {
    if (auto* b200 = dynamic_cast<B200Backend*>(&backend); b200 && x.ndim() == 5 && (temporal > 0 || pad_h > 0 || pad_w > 0))
        return b200->pad_axes(x, {0, 0, temporal, pad_h, pad_w}, {0, 0, temporal, pad_h, pad_w}, 0.0f, {false, false, true, false, false});
    Tensor padded = x;   // the reference's two calls (ltx.cpp:210-214)
    if (temporal) padded = backend.pad(padded, {0, 0, 0, 0, temporal, temporal}, 0.0f, vrhino::PadMode::Replicate);
    if (pad_h > 0 || pad_w > 0) padded = backend.pad(padded, {pad_w, pad_w, pad_h, pad_h}, 0.0f);
    return padded;
}

Tensor depth_to_space_residual(vrhino::Backend& backend, const Tensor& projected, const Tensor& input) {
    if (auto* b200 = dynamic_cast<B200Backend*>(&backend)) return b200->depth_to_space_residual(projected, input);
    Tensor residual = backend.pixel_shuffle_nd(input, {2, 2, 2});
    residual = backend.concat({residual, residual, residual, residual}, 1);
    residual = backend.slice(residual, 2, 1, residual.dim(2));
    Tensor x = backend.pixel_shuffle_nd(projected, {2, 2, 2});
    return backend.add(backend.slice(x, 2, 1, x.dim(2)), residual);
}

Tensor swiglu(vrhino::Backend& backend, const Tensor& projected) {
    if (auto* b200 = dynamic_cast<B200Backend*>(&backend)) return b200->swiglu(projected);
    const int64_t hidden = projected.dim(-1) / 2;
    std::vector<Tensor> parts = backend.split(projected, {hidden, hidden}, -1);
    return backend.mul(parts[0], backend.activation(parts[1], vrhino::Activation::Silu));
}

Tensor group_norm_silu(vrhino::Backend& backend, const Tensor& x, int groups, const Tensor* weight, const Tensor* bias, float eps) {
    if (auto* b200 = dynamic_cast<B200Backend*>(&backend)) return b200->group_norm_silu(x, groups, weight, bias, eps);
    return backend.activation(backend.group_norm(x, groups, weight, bias, eps), vrhino::Activation::Silu);
}

Tensor frame_group_norm(vrhino::Backend& backend, const Tensor& x, int groups, const Tensor* weight, const Tensor* bias,
                        float eps, bool silu) {
    if (auto* b200 = dynamic_cast<B200Backend*>(&backend)) return b200->group_norm_frames(x, groups, weight, bias, eps, silu);
    const int64_t b = x.dim(0), c = x.dim(1), t = x.dim(2), h = x.dim(3), w = x.dim(4);
    Tensor frames = backend.reshape(backend.permute(x, {0, 2, 1, 3, 4}), {b * t, c, h, w});
    frames = backend.group_norm(frames, groups, weight, bias, eps);
    Tensor out = backend.permute(backend.reshape(frames, {b, t, c, h, w}), {0, 2, 1, 3, 4});
    return silu ? backend.activation(out, vrhino::Activation::Silu) : out;
}

}  // namespace vrhino_b200
