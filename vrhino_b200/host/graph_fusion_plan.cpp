// Analysis half of the graph fusion pass (see graph_fusion.h): structural matching on the
// admitted Description only -- producer / consumer relations and dtypes, never value names.
// Nothing here touches a backend, so it builds and runs without CUDA.
#include "graph_fusion.h"

#include <variant>

namespace vrhino_b200 {

namespace ng = vrhino::neural_graph;
using vrhino::DType;

namespace {

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

    FusionPlan plan() {
        FusionPlan p;
        p.anchored.assign(d_.nodes.size(), FusedGroup{});
        p.absorbed.assign(d_.nodes.size(), 0);
        for (size_t i = 0; i < d_.nodes.size(); ++i) {
            if (p.absorbed[i] || p.anchored[i].kind != FusedKind::None) continue;
            const int node = static_cast<int>(i);
            if (const auto* add = std::get_if<ng::Add>(&d_.nodes[i].op)) {
                if (!modulate(p, node, *add)) gated(p, node, *add);
            } else if (const auto* cast = std::get_if<ng::Cast>(&d_.nodes[i].op)) {
                rope_heads(p, node, *cast);
            } else if (const auto* rp = std::get_if<ng::Rope>(&d_.nodes[i].op)) {
                rope_rows(p, node, *rp);
            }
        }
        p.stats.nodes_total = static_cast<int>(d_.nodes.size());
        for (size_t i = 0; i < d_.nodes.size(); ++i) {
            p.stats.nodes_absorbed += p.absorbed[i] ? 1 : 0;
            switch (p.anchored[i].kind) {
                case FusedKind::LayerNormModulate: ++p.stats.layer_norm_modulate; break;
                case FusedKind::RmsNormModulate: ++p.stats.rms_norm_modulate; break;
                case FusedKind::RmsNormRope: ++p.stats.rms_norm_rope; break;
                case FusedKind::GatedResidual: ++p.stats.gated_residual; break;
                default: break;
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
    bool is_float(ng::ValueId v) const { return d_.values[v].dtype == DType::F32 || d_.values[v].dtype == DType::BF16; }
    bool last_axis(int64_t axis, ng::ValueId v) const {
        const int64_t rank = static_cast<int64_t>(d_.values[v].shape.size());
        return axis == rank - 1 || axis == -1;
    }
    // strips an interior Cast to F32 in front of `v` (an exact widening the kernels do themselves);
    // returns the cast's node or -1
    int widening_cast(ng::ValueId v, ng::ValueId& source) const {
        source = v;
        const auto* c = made_by<ng::Cast>(v);
        if (c && c->destination == DType::F32 && interior(v) && is_float(c->x)) { source = c->x; return producer_[v]; }
        return -1;
    }

    // Add(Mul([Cast] Norm(x), Add(1, [Cast] scale)), [Cast] shift) [-> Cast execution]
    // Norm = LayerNorm, or RmsNorm over the last axis without a weight
    bool modulate(FusionPlan& p, int node, const ng::Add& add) {
        const auto* mul = made_by<ng::Mul>(add.a);
        if (!mul || !interior(add.a)) return false;
        const auto* one_plus = made_by<ng::Add>(mul->b);
        if (!one_plus || !is_one(one_plus->a)) return false;
        ng::ValueId normed, scale, shift;
        const int norm_cast = widening_cast(mul->a, normed);
        if (!interior(normed)) return false;
        FusedGroup g;
        if (const auto* ln = made_by<ng::LayerNorm>(normed)) {
            g.kind = FusedKind::LayerNormModulate;
            g.x = ln->x; g.weight = ln->weight; g.bias = ln->bias; g.epsilon = ln->epsilon;
        } else if (const auto* rms = made_by<ng::RmsNorm>(normed)) {
            if (rms->weight || !last_axis(rms->axis, rms->x)) return false;
            g.kind = FusedKind::RmsNormModulate;
            g.x = rms->x; g.epsilon = rms->epsilon;
        } else {
            return false;
        }
        const int scale_cast = widening_cast(one_plus->b, scale);
        const int shift_cast = widening_cast(add.b, shift);
        if (d_.values[scale].dtype != d_.values[shift].dtype || d_.values[scale].shape != d_.values[shift].shape) return false;
        if (d_.values[d_.nodes[node].result].dtype != DType::F32) return false;   // the modulation arithmetic is F32
        g.shift = shift; g.scale = scale;
        int anchor = node;
        const ng::ValueId sum = d_.nodes[node].result;
        if (interior(sum) && std::get_if<ng::Cast>(&d_.nodes[consumer_[sum]].op)) {   // the GEMM operand cast
            p.absorbed[node] = 1;
            anchor = consumer_[sum];
        }
        p.absorbed[producer_[normed]] = 1;
        if (norm_cast >= 0) p.absorbed[norm_cast] = 1;
        p.absorbed[producer_[add.a]] = 1;
        if (interior(mul->b)) {          // 1 + scale feeds only this chain: it (and its operand cast) disappear
            p.absorbed[producer_[mul->b]] = 1;
            if (scale_cast >= 0) p.absorbed[scale_cast] = 1;
        }
        if (shift_cast >= 0) p.absorbed[shift_cast] = 1;
        p.anchored[anchor] = g;
        return true;
    }

    bool rms_for_rope(ng::ValueId v, const ng::RmsNorm*& rms) const {
        rms = made_by<ng::RmsNorm>(v);
        if (!rms || !interior(v) || !rms->weight) return false;
        if (d_.values[rms->x].shape.size() != 3 || !last_axis(rms->axis, rms->x)) return false;
        return d_.values[v].dtype == DType::F32;                      // attention_norm widens to F32
    }

    // Cast(Rope(Reshape(RmsNorm(x, w, last axis), [B,S,H,d]), cos, sin), execution)          (Wan)
    bool rope_heads(FusionPlan& p, int node, const ng::Cast& cast) {
        if (cast.destination != d_.execution_dtype || cast.destination == DType::F32) return false;
        const auto* rp = made_by<ng::Rope>(cast.x);
        if (!rp || !interior(cast.x)) return false;
        const auto* rs = made_by<ng::Reshape>(rp->x);
        if (!rs || !interior(rp->x) || rs->shape.size() != 4) return false;
        const ng::RmsNorm* rms = nullptr;
        if (!rms_for_rope(rs->x, rms)) return false;
        const auto& xs = d_.values[rms->x].shape;
        if (rs->shape[0] != xs[0] || rs->shape[1] != xs[1] || rs->shape[2] * rs->shape[3] != xs[2]) return false;
        FusedGroup g;
        g.kind = FusedKind::RmsNormRope;
        g.x = rms->x; g.weight = rms->weight; g.epsilon = rms->epsilon;
        g.cosine = rp->cosine; g.sine = rp->sine; g.heads = static_cast<int>(rs->shape[2]);
        p.absorbed[producer_[rs->x]] = 1;
        p.absorbed[producer_[rp->x]] = 1;
        p.absorbed[producer_[cast.x]] = 1;
        p.anchored[node] = g;
        return true;
    }

    // Rope(RmsNorm(x, w, last axis), cos, sin) with tables spanning whole rows ([B|1, S, D])   (LTX)
    bool rope_rows(FusionPlan& p, int node, const ng::Rope& rp) {
        const ng::RmsNorm* rms = nullptr;
        if (!rms_for_rope(rp.x, rms)) return false;
        const auto& xs = d_.values[rms->x].shape;
        const auto& ts = d_.values[rp.cosine].shape;
        if (ts != d_.values[rp.sine].shape || ts.size() != 3 || ts[2] != xs[2] || ts[1] != xs[1] || (ts[0] != xs[0] && ts[0] != 1))
            return false;
        if (!is_float(rp.cosine) || d_.values[d_.nodes[node].result].dtype != DType::F32) return false;
        FusedGroup g;
        g.kind = FusedKind::RmsNormRope;
        g.x = rms->x; g.weight = rms->weight; g.epsilon = rms->epsilon;
        g.cosine = rp.cosine; g.sine = rp.sine; g.heads = 1;
        p.absorbed[producer_[rp.x]] = 1;
        p.anchored[node] = g;
        return true;
    }

    // Add([Cast] residual, Mul([Cast] branch, [Cast] gate))
    bool gated(FusionPlan& p, int node, const ng::Add& add) {
        const auto* mul = made_by<ng::Mul>(add.b);
        if (!mul || !interior(add.b)) return false;
        const DType state = d_.values[d_.nodes[node].result].dtype;
        if (d_.values[add.a].dtype != state || d_.values[add.b].dtype != state) return false;
        ng::ValueId residual, branch, gate;
        const int residual_cast = widening_cast(add.a, residual);
        const int branch_cast = widening_cast(mul->a, branch);
        const int gate_cast = widening_cast(mul->b, gate);
        if (d_.values[residual].shape != d_.values[branch].shape || !is_float(residual) || !is_float(branch) || !is_float(gate))
            return false;
        const auto& gs = d_.values[gate].shape;
        const auto& rs = d_.values[residual].shape;
        if (gs.size() != rs.size() || rs.size() < 2 || gs.back() != rs.back()) return false;
        int64_t gate_rows = 1, rows = 1;
        for (size_t k = 0; k + 1 < gs.size(); ++k) { gate_rows *= gs[k]; rows *= rs[k]; }
        // one gate vector for everything, one per batch entry, or one per row
        const bool per_batch = gate_rows == gs[0] && (gs[0] == 1 || gs[0] == rs[0]);
        if (!per_batch && gate_rows != rows) return false;
        FusedGroup g;
        g.kind = FusedKind::GatedResidual;
        g.residual = residual; g.branch = branch; g.gate = gate;
        if (residual_cast >= 0) p.absorbed[residual_cast] = 1;
        if (branch_cast >= 0) p.absorbed[branch_cast] = 1;
        if (gate_cast >= 0) p.absorbed[gate_cast] = 1;
        p.absorbed[producer_[add.b]] = 1;
        p.anchored[node] = g;
        return true;
    }

    const ng::Description& d_;
    std::vector<int> producer_, uses_, consumer_;
    std::vector<char> exported_;
};

}  // namespace

FusionPlan plan_fusion(const ng::Description& description) { return Matcher(description).plan(); }

}  // namespace vrhino_b200
