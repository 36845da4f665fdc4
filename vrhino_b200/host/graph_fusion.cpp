// See graph_fusion.h.  The pass only reads the admitted Description; matching is structural
// (producer / consumer relations and dtypes), never by value names.
#include "graph_fusion.h"

#include <optional>
#include <variant>

#include "vrhino/error.h"

namespace vrhino_b200 {

namespace ng = vrhino::neural_graph;
using vrhino::DType;
using vrhino::require;
using vrhino::Tensor;

namespace {

enum class Kind { None, LayerNormModulate, RmsNormRope, GatedResidual };

struct Group {
    Kind kind = Kind::None;
    ng::ValueId x = 0, shift = 0, scale = 0, cosine = 0, sine = 0, residual = 0, branch = 0, gate = 0;
    std::optional<ng::ValueId> weight, bias;
    float epsilon = 0.0f;
    int heads = 1;
};

struct Plan {
    std::vector<Group> anchored;   // per node: the chain that ends (and runs) at this node
    std::vector<char> absorbed;    // per node: part of a chain, launches nothing itself
};

std::vector<ng::ValueId> operands(const ng::Primitive& op) {
    struct Visitor {
        std::vector<ng::ValueId> operator()(std::monostate) const { return {}; }
        std::vector<ng::ValueId> operator()(const ng::Add& o) const { return {o.a, o.b}; }
        std::vector<ng::ValueId> operator()(const ng::Mul& o) const { return {o.a, o.b}; }
        std::vector<ng::ValueId> operator()(const ng::Reshape& o) const { return {o.x}; }
        std::vector<ng::ValueId> operator()(const ng::Linear& o) const {
            std::vector<ng::ValueId> v{o.x, o.weight};
            if (o.bias) v.push_back(*o.bias);
            return v;
        }
        std::vector<ng::ValueId> operator()(const ng::RmsNorm& o) const {
            std::vector<ng::ValueId> v{o.x};
            if (o.weight) v.push_back(*o.weight);
            return v;
        }
        std::vector<ng::ValueId> operator()(const ng::Activate& o) const { return {o.x}; }
        std::vector<ng::ValueId> operator()(const ng::Permute& o) const { return {o.x}; }
        std::vector<ng::ValueId> operator()(const ng::Slice& o) const { return {o.x}; }
        std::vector<ng::ValueId> operator()(const ng::Concat& o) const { return o.tensors; }
        std::vector<ng::ValueId> operator()(const ng::Gather& o) const { return {o.table, o.indices}; }
        std::vector<ng::ValueId> operator()(const ng::Rope& o) const { return {o.x, o.cosine, o.sine}; }
        std::vector<ng::ValueId> operator()(const ng::Attention& o) const { return {o.q, o.k, o.v}; }
        std::vector<ng::ValueId> operator()(const ng::Cast& o) const { return {o.x}; }
        std::vector<ng::ValueId> operator()(const ng::LayerNorm& o) const {
            std::vector<ng::ValueId> v{o.x};
            if (o.weight) v.push_back(*o.weight);
            if (o.bias) v.push_back(*o.bias);
            return v;
        }
    };
    return std::visit(Visitor{}, op);
}

class Matcher {
public:
    explicit Matcher(const ng::Description& d)
        : d_(d), producer_(d.values.size(), -1), uses_(d.values.size(), 0), consumer_(d.values.size(), -1),
          exported_(d.values.size(), 0) {
        for (size_t i = 0; i < d.nodes.size(); ++i) {
            producer_[d.nodes[i].result] = static_cast<int>(i);
            for (ng::ValueId v : operands(d.nodes[i].op)) { ++uses_[v]; consumer_[v] = static_cast<int>(i); }
        }
        for (ng::ValueId v : d.outputs) exported_[v] = 1;
    }

    Plan plan() {
        Plan p;
        p.anchored.assign(d_.nodes.size(), Group{});
        p.absorbed.assign(d_.nodes.size(), 0);
        for (size_t i = 0; i < d_.nodes.size(); ++i) {
            if (p.absorbed[i] || p.anchored[i].kind != Kind::None) continue;
            if (const auto* add = std::get_if<ng::Add>(&d_.nodes[i].op)) {
                if (!modulate(p, static_cast<int>(i), *add)) gated(p, static_cast<int>(i), *add);
            } else if (const auto* cast = std::get_if<ng::Cast>(&d_.nodes[i].op)) {
                rope(p, static_cast<int>(i), *cast);
            }
        }
        return p;
    }

private:
    template <class T>
    const T* made_by(ng::ValueId v) const {
        return producer_[v] >= 0 ? std::get_if<T>(&d_.nodes[producer_[v]].op) : nullptr;
    }
    // interior value of a chain: one consumer, not exported
    bool interior(ng::ValueId v) const { return uses_[v] == 1 && !exported_[v]; }
    bool is_one(ng::ValueId v) const {
        for (const auto& c : d_.constants)
            if (c.value == v) return c.scalar == 1.0f && d_.values[v].dtype == DType::F32;
        return false;
    }
    // strips an interior Cast to F32 in front of `v`; returns the cast's node or -1
    int widening_cast(ng::ValueId v, ng::ValueId& source) const {
        source = v;
        const auto* c = made_by<ng::Cast>(v);
        if (c && c->destination == DType::F32 && interior(v)) { source = c->x; return producer_[v]; }
        return -1;
    }

    // Add(Mul([Cast] LayerNorm(x), Add(1, scale)), shift) [-> Cast execution]
    bool modulate(Plan& p, int node, const ng::Add& add) {
        const auto* mul = made_by<ng::Mul>(add.a);
        if (!mul || !interior(add.a)) return false;
        const auto* one_plus = made_by<ng::Add>(mul->b);
        if (!one_plus || !is_one(one_plus->a)) return false;
        ng::ValueId normed;
        const int cast_node = widening_cast(mul->a, normed);
        const auto* norm = made_by<ng::LayerNorm>(normed);
        if (!norm || !interior(normed)) return false;
        if (d_.values[add.b].dtype != d_.values[one_plus->b].dtype) return false;
        Group g;
        g.kind = Kind::LayerNormModulate;
        g.x = norm->x; g.weight = norm->weight; g.bias = norm->bias; g.epsilon = norm->epsilon;
        g.shift = add.b; g.scale = one_plus->b;
        int anchor = node;
        const ng::ValueId sum = d_.nodes[node].result;
        if (interior(sum) && std::get_if<ng::Cast>(&d_.nodes[consumer_[sum]].op)) {   // the GEMM operand cast
            p.absorbed[node] = 1;
            anchor = consumer_[sum];
        }
        p.absorbed[producer_[normed]] = 1;
        if (cast_node >= 0) p.absorbed[cast_node] = 1;
        p.absorbed[producer_[add.a]] = 1;
        if (interior(mul->b)) p.absorbed[producer_[mul->b]] = 1;
        p.anchored[anchor] = g;
        return true;
    }

    // Cast(Rope(Reshape(RmsNorm(x, w, last axis), [B,S,H,d]), cos, sin), execution)
    bool rope(Plan& p, int node, const ng::Cast& cast) {
        if (cast.destination != d_.execution_dtype || cast.destination == DType::F32) return false;
        const auto* rp = made_by<ng::Rope>(cast.x);
        if (!rp || !interior(cast.x)) return false;
        const auto* rs = made_by<ng::Reshape>(rp->x);
        if (!rs || !interior(rp->x) || rs->shape.size() != 4) return false;
        const auto* rms = made_by<ng::RmsNorm>(rs->x);
        if (!rms || !interior(rs->x) || !rms->weight) return false;
        const auto& xs = d_.values[rms->x].shape;
        if (xs.size() != 3 || (rms->axis != 2 && rms->axis != -1)) return false;
        if (d_.values[rs->x].dtype != DType::F32) return false;       // attention_norm widens to F32
        if (rs->shape[0] != xs[0] || rs->shape[1] != xs[1] || rs->shape[2] * rs->shape[3] != xs[2]) return false;
        Group g;
        g.kind = Kind::RmsNormRope;
        g.x = rms->x; g.weight = rms->weight; g.epsilon = rms->epsilon;
        g.cosine = rp->cosine; g.sine = rp->sine; g.heads = static_cast<int>(rs->shape[2]);
        p.absorbed[producer_[rs->x]] = 1;
        p.absorbed[producer_[rp->x]] = 1;
        p.absorbed[producer_[cast.x]] = 1;
        p.anchored[node] = g;
        return true;
    }

    // Add([Cast] residual, Mul([Cast] branch, gate))
    bool gated(Plan& p, int node, const ng::Add& add) {
        const auto* mul = made_by<ng::Mul>(add.b);
        if (!mul || !interior(add.b)) return false;
        const DType state = d_.values[d_.nodes[node].result].dtype;
        if (d_.values[add.a].dtype != state || d_.values[add.b].dtype != state) return false;
        ng::ValueId residual, branch;
        const int residual_cast = widening_cast(add.a, residual);
        const int branch_cast = widening_cast(mul->a, branch);
        if (d_.values[residual].shape != d_.values[branch].shape) return false;
        const auto& gs = d_.values[mul->b].shape;
        const auto& rs = d_.values[residual].shape;
        if (gs.size() != rs.size() || rs.size() < 2 || gs.back() != rs.back()) return false;
        for (size_t k = 1; k + 1 < gs.size(); ++k)
            if (gs[k] != 1) return false;                              // one gate vector per batch entry
        if (gs[0] != 1 && gs[0] != rs[0]) return false;
        Group g;
        g.kind = Kind::GatedResidual;
        g.residual = residual; g.branch = branch; g.gate = mul->b;
        if (residual_cast >= 0) p.absorbed[residual_cast] = 1;
        if (branch_cast >= 0) p.absorbed[branch_cast] = 1;
        p.absorbed[producer_[add.b]] = 1;
        p.anchored[node] = g;
        return true;
    }

    const ng::Description& d_;
    std::vector<int> producer_, uses_, consumer_;
    std::vector<char> exported_;
};

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
                                   const std::vector<Tensor>& parameters, FusionStats* stats) {
    const ng::Description& d = graph.description();
    require(inputs.size() == d.inputs.size(), "Input slot count mismatch");
    require(parameters.size() == d.parameters.size(), "Parameter slot count mismatch");
    require(backend.execution_dtype() == d.execution_dtype, "Backend execution dtype must match graph");
    const Plan plan = Matcher(d).plan();

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

    FusionStats local;
    local.nodes_total = static_cast<int>(d.nodes.size());
    for (size_t i = 0; i < d.nodes.size(); ++i) {
        const ng::Node& n = d.nodes[i];
        const ng::TensorSpec& spec = d.values[n.result];
        const Group& g = plan.anchored[i];
        Tensor result;
        if (g.kind == Kind::LayerNormModulate) {
            result = backend.layer_norm_modulate(values[g.x], g.weight ? &values[*g.weight] : nullptr,
                                                 g.bias ? &values[*g.bias] : nullptr, g.epsilon, values[g.shift],
                                                 values[g.scale], spec.dtype);
            ++local.layer_norm_modulate;
        } else if (g.kind == Kind::RmsNormRope) {
            Tensor flat = backend.rms_norm_rope(values[g.x], &values[*g.weight], g.epsilon, &values[g.cosine],
                                                &values[g.sine], g.heads, false, spec.dtype);
            result = backend.reshape(flat, spec.shape);
            ++local.rms_norm_rope;
        } else if (g.kind == Kind::GatedResidual) {
            result = backend.gated_residual(values[g.residual], values[g.branch], &values[g.gate], spec.dtype);
            ++local.gated_residual;
        } else if (plan.absorbed[i]) {
            ++local.nodes_absorbed;
            continue;                                   // its value exists only inside a fused kernel
        } else {
            result = std::visit(Dispatch{backend, values, spec.dtype}, n.op);
        }
        require(result.defined() && result.dtype() == spec.dtype && result.shape() == spec.shape,
                "Backend returned invalid tensor metadata");
        values[n.result] = std::move(result);
    }
    backend.synchronize();
    std::vector<Tensor> outputs;
    outputs.reserve(d.outputs.size());
    for (ng::ValueId id : d.outputs) {
        require(values[id].defined(), "Invalid output at capture");
        outputs.push_back(values[id]);
    }
    if (stats) *stats = local;
    return outputs;
}

}  // namespace vrhino_b200
