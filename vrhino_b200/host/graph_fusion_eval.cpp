// Evaluation half of the graph fusion pass (see graph_fusion.h): walks an admitted Graph, running
// the chains graph_fusion_plan.cpp found through FusedOperators and every other node through the
// plain vrhino::Backend interface.  Needs no CUDA: the B200Backend adapter lives in graph_fusion.cpp.
#include "graph_fusion.h"

#include <cstring>
#include <type_traits>
#include <variant>

#include "vrhino/backend.h"
#include "vrhino/error.h"

namespace vrhino_b200 {

namespace ng = vrhino::neural_graph;
using vrhino::DType;
using vrhino::Tensor;

namespace {

// One node that is not part of a fused chain -> the backend call the reference evaluator makes for
// it (neural_graph_evaluator.cpp:28-71).
Tensor run_plain_node(vrhino::Backend& be, const std::vector<Tensor>& v, DType result_dtype, const ng::Node& node) {
    auto optional = [&](const std::optional<ng::ValueId>& id) { return id ? &v[*id] : nullptr; };
    return std::visit([&](const auto& op) -> Tensor {
        using Op = std::decay_t<decltype(op)>;
        if constexpr (std::is_same_v<Op, ng::Add>) return be.add(v[op.a], v[op.b]);
        else if constexpr (std::is_same_v<Op, ng::Mul>) return be.mul(v[op.a], v[op.b]);
        else if constexpr (std::is_same_v<Op, ng::Cast>) return be.cast(v[op.x], op.destination);
        else if constexpr (std::is_same_v<Op, ng::Reshape>) return be.reshape(v[op.x], op.shape);
        else if constexpr (std::is_same_v<Op, ng::Permute>) return be.permute(v[op.x], op.axes);
        else if constexpr (std::is_same_v<Op, ng::Slice>) return be.slice(v[op.x], op.axis, op.start, op.stop);
        else if constexpr (std::is_same_v<Op, ng::Activate>) return be.activation(v[op.x], op.kind);
        else if constexpr (std::is_same_v<Op, ng::Gather>) return be.indexed_gather(v[op.table], v[op.indices]);
        else if constexpr (std::is_same_v<Op, ng::Rope>) return be.rope_nd(v[op.x], v[op.cosine], v[op.sine]);
        else if constexpr (std::is_same_v<Op, ng::LayerNorm>)
            return be.layer_norm(v[op.x], optional(op.weight), optional(op.bias), op.epsilon);
        else if constexpr (std::is_same_v<Op, ng::RmsNorm>)
            return be.rms_norm(v[op.x], optional(op.weight), op.epsilon, op.axis, result_dtype);
        else if constexpr (std::is_same_v<Op, ng::Linear>)
            return be.linear(v[op.x], v[op.weight], optional(op.bias), op.compute_dtype, result_dtype);
        else if constexpr (std::is_same_v<Op, ng::Attention>)
            return be.attention(v[op.q], v[op.k], v[op.v], nullptr, false, op.scale, nullptr, nullptr);
        else if constexpr (std::is_same_v<Op, ng::Concat>) {
            std::vector<Tensor> parts;
            parts.reserve(op.tensors.size());
            for (ng::ValueId id : op.tensors) parts.push_back(v[id]);
            return be.concat(parts, op.axis);
        } else {
            throw ng::GraphError(ng::Code::UnsupportedPrimitive, ng::Phase::Run, "Unsupported primitive");
        }
    }, node.op);
}

// Where the evaluation stands, for the error report.
struct Progress {
    ng::Phase phase = ng::Phase::Bind;
    ng::Location node, value, primitive;
    bool work_enqueued = false;   // a call that may have submitted device work has been made
    bool drained = false;         // the one drain (normal or after a failure) has been attempted
    [[noreturn]] void fail(ng::Code code, const char* detail) const {
        throw ng::GraphError(code, phase, detail, node, value, primitive);
    }
};

bool has_spec(const Tensor& t, const ng::TensorSpec& spec) {
    return t.defined() && !t.is_quantized() && t.dtype() == spec.dtype && t.shape() == spec.shape && t.data() != nullptr;
}

}  // namespace

std::vector<Tensor> evaluate_fused(FusedOperators& ops, const ng::Graph& graph, const std::vector<Tensor>& inputs,
                                   const std::vector<Tensor>& parameters, FusionStats* stats, bool drain) {
    vrhino::Backend& backend = ops.backend();
    const ng::Description& d = graph.description();
    Progress at;
    std::vector<Tensor> values, uploaded_sources;   // host owners of uploads stay alive through a failure drain
    Tensor result;                                  // so does a result that failed its metadata check

    // After a failure: give enqueued work one chance to finish, keep a second failure beside the first.
    auto drain_after_failure = [&](ng::GraphError& error) {
        if (!at.work_enqueued || at.drained) return;
        at.drained = true;
        try {
            backend.synchronize();
        } catch (const std::exception& e) {
            error.secondary_completion = std::string(e.what()).substr(0, ng::max_detail);
        } catch (...) {
            error.secondary_completion = "Non-standard completion failure";
        }
    };

    try {
        if (inputs.size() != d.inputs.size()) at.fail(ng::Code::InvalidInputBinding, "Input slot count mismatch");
        if (parameters.size() != d.parameters.size()) at.fail(ng::Code::InvalidParameterBinding, "Parameter slot count mismatch");
        if (backend.execution_dtype() != d.execution_dtype) at.fail(ng::Code::InvalidContext, "Backend execution dtype must match graph");
        if (d.execution_dtype == DType::BF16 && !backend.supports(DType::BF16)) at.fail(ng::Code::InvalidContext, "Backend does not support BF16");
        const FusionPlan plan = plan_fusion(d);
        values.resize(d.values.size());

        // Every binding is checked before anything is uploaded.
        auto bind = [&](const std::vector<ng::ValueId>& slots, const std::vector<Tensor>& handles, ng::Code code) {
            for (size_t i = 0; i < slots.size(); ++i) {
                at.value = slots[i];
                if (!has_spec(handles[i], d.values[slots[i]])) at.fail(code, "Invalid bound tensor metadata");
                values[slots[i]] = handles[i];
            }
        };
        bind(d.inputs, inputs, ng::Code::InvalidInputBinding);
        bind(d.parameters, parameters, ng::Code::InvalidParameterBinding);
        for (const auto& c : d.constants) {
            at.value = c.value;
            const DType dtype = d.values[c.value].dtype;
            Tensor scalar = Tensor::host({1}, dtype);
            if (dtype == DType::F32) {
                scalar.data_as<float>()[0] = c.scalar;
            } else {   // the evaluator truncates the F32 constant to its upper 16 bits (:120-123)
                uint32_t bits;
                std::memcpy(&bits, &c.scalar, sizeof(bits));
                scalar.data_as<uint16_t>()[0] = static_cast<uint16_t>(bits >> 16);
            }
            values[c.value] = std::move(scalar);
        }
        // host operands go up front when there is a device to go to (a host-only backend keeps them)
        const bool has_device = backend.device_count() > 0;
        for (size_t id = 0; has_device && id < values.size(); ++id) {
            const ng::TensorSpec& spec = d.values[id];
            if (!values[id].defined() || values[id].device() != vrhino::DeviceId::host() ||
                (spec.dtype != DType::F32 && spec.dtype != DType::BF16))
                continue;
            at.value = id;
            at.work_enqueued = true;
            result = backend.copy_to_device(values[id], spec.dtype);
            if (!has_spec(result, spec) || result.device() != vrhino::DeviceId::accelerator())
                at.fail(ng::Code::InvalidContext, "Invalid dtype-preserving binding placement");
            uploaded_sources.push_back(values[id]);
            values[id] = std::move(result);
        }

        at.phase = ng::Phase::Run;
        for (size_t i = 0; i < d.nodes.size(); ++i) {
            const ng::Node& n = d.nodes[i];
            const ng::TensorSpec& spec = d.values[n.result];
            const FusedGroup& g = plan.anchored[i];
            if (g.kind == FusedKind::None && plan.absorbed[i]) continue;   // its value exists only inside a fused kernel
            at.node = i;
            at.value = n.result;
            at.primitive = n.op.index();
            at.work_enqueued = true;   // a call that throws may already have launched something
            auto optional = [&](const std::optional<ng::ValueId>& id) { return id ? &values[*id] : nullptr; };
            switch (g.kind) {
                case FusedKind::LayerNormModulate:
                    result = ops.layer_norm_modulate(values[g.x], optional(g.weight), optional(g.bias), g.epsilon, values[g.shift],
                                                     values[g.scale], spec.dtype);
                    break;
                case FusedKind::RmsNormModulate:
                    result = ops.rms_norm_modulate(values[g.x], g.epsilon, values[g.shift], values[g.scale], spec.dtype);
                    break;
                case FusedKind::RmsNormRope:
                    result = backend.reshape(ops.rms_norm_rope(values[g.x], optional(g.weight), g.epsilon, &values[g.cosine],
                                                               &values[g.sine], g.heads, spec.dtype),
                                             spec.shape);
                    break;
                case FusedKind::GatedResidual:
                    result = ops.gated_residual(values[g.residual], values[g.branch], &values[g.gate], spec.dtype);
                    break;
                default:
                    result = run_plain_node(backend, values, spec.dtype, n);
            }
            if (!has_spec(result, spec)) at.fail(ng::Code::InvalidNodeOutput, "Backend returned invalid tensor metadata");
            values[n.result] = std::move(result);
        }

        at.node.reset();
        at.value.reset();
        at.primitive.reset();
        if (drain) {
            at.phase = ng::Phase::Drain;
            at.drained = true;
            backend.synchronize();
        }
        at.phase = ng::Phase::Capture;
        std::vector<Tensor> outputs;
        outputs.reserve(d.outputs.size());
        for (ng::ValueId id : d.outputs) {
            at.value = id;
            if (!has_spec(values[id], d.values[id])) at.fail(ng::Code::InvalidOutput, "Invalid output at capture");
            outputs.push_back(values[id]);
        }
        if (stats) *stats = plan.stats;
        return outputs;
    } catch (ng::GraphError& error) {
        drain_after_failure(error);
        throw;
    } catch (const std::exception& e) {
        ng::GraphError error(at.phase == ng::Phase::Drain ? ng::Code::CompletionFailure : ng::Code::BackendFailure, at.phase,
                             e.what(), at.node, at.value, at.primitive);
        drain_after_failure(error);
        throw error;
    } catch (...) {
        ng::GraphError error(at.phase == ng::Phase::Drain ? ng::Code::CompletionFailure : ng::Code::BackendFailure, at.phase,
                             "Non-standard Backend failure", at.node, at.value, at.primitive);
        drain_after_failure(error);
        throw error;
    }
}

}  // namespace vrhino_b200
