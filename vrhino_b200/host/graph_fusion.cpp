// B200Backend behind the fusion pass's evaluator (graph_fusion_eval.cpp): the four chains map onto
// the backend's one-kernel forms.
#include "graph_fusion.h"

#include "b200_backend.h"

namespace vrhino_b200 {

using vrhino::DType;
using vrhino::Tensor;

namespace {

class B200Fused final : public FusedOperators {
public:
    explicit B200Fused(B200Backend& backend) : backend_(backend) {}
    vrhino::Backend& backend() override { return backend_; }
    Tensor layer_norm_modulate(const Tensor& x, const Tensor* weight, const Tensor* bias, float eps, const Tensor& shift,
                               const Tensor& scale, DType output) override {
        return backend_.layer_norm_modulate(x, weight, bias, eps, shift, scale, output);
    }
    Tensor rms_norm_modulate(const Tensor& x, float eps, const Tensor& shift, const Tensor& scale, DType output) override {
        return backend_.rms_norm_modulate(x, eps, shift, scale, output);
    }
    Tensor rms_norm_rope(const Tensor& x, const Tensor* weight, float eps, const Tensor* cosine, const Tensor* sine, int heads,
                         DType output) override {
        return backend_.rms_norm_rope(x, weight, eps, cosine, sine, heads, false, output);
    }
    Tensor gated_residual(const Tensor& residual, const Tensor& branch, const Tensor* gate, DType state) override {
        return backend_.gated_residual(residual, branch, gate, state);
    }
private:
    B200Backend& backend_;
};

}  // namespace

std::vector<Tensor> evaluate_fused(B200Backend& backend, const vrhino::neural_graph::Graph& graph,
                                   const std::vector<Tensor>& inputs, const std::vector<Tensor>& parameters,
                                   FusionStats* stats, bool drain) {
    B200Fused operators(backend);
    return evaluate_fused(operators, graph, inputs, parameters, stats, drain);
}

}  // namespace vrhino_b200
