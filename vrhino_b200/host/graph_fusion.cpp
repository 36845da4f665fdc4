// Evaluation half of the graph fusion pass (see graph_fusion.h): runs the plan of
// graph_fusion_plan.cpp on a B200Backend.
#include "graph_fusion.h"

#include <variant>

#include "b200_backend.h"
#include "vrhino/error.h"

namespace vrhino_b200 {

namespace ng = vrhino::neural_graph;
using vrhino::DType;
using vrhino::require;
using vrhino::Tensor;

namespace {

// The reference evaluator's node dispatch (neural_graph_evaluator.cpp:28-71), unchanged.
struct Dispatch {
    vrhino::Backend& backend;
    const std::vector<Tensor>& values;
    DType output_dtype;
    Tensor operator()(std::monostate) const {
        throw ng::GraphError(ng::Code::UnsupportedPrimitive, ng::Phase::Run, "Unsupported primitive");
    }
    Tensor operator()(const ng::Add& op) const { return backend.add(values[op.a], values[op.b]); }
    Tensor operator()(const ng::Mul& op) const { return backend.mul(values[op.a], values[op.b]); }
    Tensor operator()(const ng::Reshape& op) const { return backend.reshape(values[op.x], op.shape); }
    Tensor operator()(const ng::Linear& op) const {
        return backend.linear(values[op.x], values[op.weight], op.bias ? &values[*op.bias] : nullptr, op.compute_dtype,
                              output_dtype);
    }
    Tensor operator()(const ng::RmsNorm& op) const {
        return backend.rms_norm(values[op.x], op.weight ? &values[*op.weight] : nullptr, op.epsilon, op.axis, output_dtype);
    }
    Tensor operator()(const ng::LayerNorm& op) const {
        return backend.layer_norm(values[op.x], op.weight ? &values[*op.weight] : nullptr,
                                  op.bias ? &values[*op.bias] : nullptr, op.epsilon);
    }
    Tensor operator()(const ng::Cast& op) const { return backend.cast(values[op.x], op.destination); }
    Tensor operator()(const ng::Activate& op) const { return backend.activation(values[op.x], op.kind); }
    Tensor operator()(const ng::Permute& op) const { return backend.permute(values[op.x], op.axes); }
    Tensor operator()(const ng::Slice& op) const { return backend.slice(values[op.x], op.axis, op.start, op.stop); }
    Tensor operator()(const ng::Concat& op) const {
        std::vector<Tensor> tensors;
        for (ng::ValueId id : op.tensors) tensors.push_back(values[id]);
        return backend.concat(tensors, op.axis);
    }
    Tensor operator()(const ng::Gather& op) const { return backend.indexed_gather(values[op.table], values[op.indices]); }
    Tensor operator()(const ng::Rope& op) const { return backend.rope_nd(values[op.x], values[op.cosine], values[op.sine]); }
    Tensor operator()(const ng::Attention& op) const {
        return backend.attention(values[op.q], values[op.k], values[op.v], nullptr, false, op.scale, nullptr, nullptr);
    }
};

}  // namespace

std::vector<Tensor> evaluate_fused(B200Backend& backend, const ng::Graph& graph, const std::vector<Tensor>& inputs,
                                   const std::vector<Tensor>& parameters, FusionStats* stats, bool drain) {
    const ng::Description& d = graph.description();
    require(inputs.size() == d.inputs.size(), "Input slot count mismatch");
    require(parameters.size() == d.parameters.size(), "Parameter slot count mismatch");
    require(backend.execution_dtype() == d.execution_dtype, "Backend execution dtype must match graph");
    const FusionPlan plan = plan_fusion(d);

    std::vector<Tensor> values(d.values.size());
    auto bind = [&](const std::vector<ng::ValueId>& slots, const std::vector<Tensor>& handles) {
        for (size_t i = 0; i < slots.size(); ++i) {
            const ng::TensorSpec& spec = d.values[slots[i]];
            require(handles[i].defined() && handles[i].dtype() == spec.dtype && handles[i].shape() == spec.shape,
                    "Invalid bound tensor metadata");
            values[slots[i]] = handles[i].device() == vrhino::DeviceId::host() &&
                                       (spec.dtype == DType::F32 || spec.dtype == DType::BF16)
                                   ? backend.copy_to_device(handles[i], spec.dtype)
                                   : handles[i];
        }
    };
    bind(d.inputs, inputs);
    bind(d.parameters, parameters);
    for (const auto& c : d.constants) {
        Tensor t = Tensor::host({1}, DType::F32);
        t.data_as<float>()[0] = c.scalar;
        values[c.value] = backend.copy_to_device(t, d.values[c.value].dtype);
    }

    for (size_t i = 0; i < d.nodes.size(); ++i) {
        const ng::Node& n = d.nodes[i];
        const ng::TensorSpec& spec = d.values[n.result];
        const FusedGroup& g = plan.anchored[i];
        Tensor result;
        switch (g.kind) {
            case FusedKind::LayerNormModulate:
                result = backend.layer_norm_modulate(values[g.x], g.weight ? &values[*g.weight] : nullptr,
                                                     g.bias ? &values[*g.bias] : nullptr, g.epsilon, values[g.shift],
                                                     values[g.scale], spec.dtype);
                break;
            case FusedKind::RmsNormModulate:
                result = backend.rms_norm_modulate(values[g.x], g.epsilon, values[g.shift], values[g.scale], spec.dtype);
                break;
            case FusedKind::RmsNormRope:
                result = backend.reshape(backend.rms_norm_rope(values[g.x], &values[*g.weight], g.epsilon, &values[g.cosine],
                                                               &values[g.sine], g.heads, false, spec.dtype),
                                         spec.shape);
                break;
            case FusedKind::GatedResidual:
                result = backend.gated_residual(values[g.residual], values[g.branch], &values[g.gate], spec.dtype);
                break;
            default:
                if (plan.absorbed[i]) continue;          // its value exists only inside a fused kernel
                result = std::visit(Dispatch{backend, values, spec.dtype}, n.op);
        }
        require(result.defined() && result.dtype() == spec.dtype && result.shape() == spec.shape,
                "Backend returned invalid tensor metadata");
        values[n.result] = std::move(result);
    }
    if (drain) backend.synchronize();
    std::vector<Tensor> outputs;
    outputs.reserve(d.outputs.size());
    for (ng::ValueId id : d.outputs) {
        require(values[id].defined(), "Invalid output at capture");
        outputs.push_back(values[id]);
    }
    if (stats) *stats = plan.stats;
    return outputs;
}

}  // namespace vrhino_b200
