// Fusion pass over the reference's executable graph (native/src/runtime/neural_graph.h): the
// Wan / LTX production graphs spell the non-GEMM chains out node by node
// (native/src/architectures/wan_self_attention_graph.h:46-70,
//  native/src/architectures/ltx_self_attention_graph.cpp:30-44).  evaluate_fused() walks the same
// admitted Graph as neural_graph::evaluate (native/src/runtime/neural_graph_evaluator.cpp:72-178),
// recognises three chains and runs each as ONE kernel of the B200 backend; every other node is
// dispatched exactly as the reference's evaluator dispatches it.  No architecture file changes.
//
//   LayerNorm | RmsNorm(no weight) -> [Cast F32] -> Mul(., Add(1, [Cast] scale)) -> Add(., [Cast] shift)
//       -> [Cast execution]                    => B200Backend::layer_norm_modulate / rms_norm_modulate
//   RmsNorm(last axis, weight) -> Reshape[B,S,H,d] -> Rope -> Cast execution       (Wan)
//   RmsNorm(last axis, weight) -> Rope with whole-row tables                        (LTX)
//                                              => B200Backend::rms_norm_rope
//   Add([Cast F32] residual, Mul([Cast F32] branch, [Cast F32] gate))
//                                              => B200Backend::gated_residual
//
// A chain is fused only when its interior values have no other consumer and are not graph
// outputs (so a diagnostics graph, which exports them, runs node by node).
#pragma once

#include <vector>

#include <optional>

#include "runtime/neural_graph.h"

namespace vrhino_b200 {

class B200Backend;

struct FusionStats {
    int layer_norm_modulate = 0, rms_norm_modulate = 0, rms_norm_rope = 0, gated_residual = 0;
    int nodes_total = 0, nodes_absorbed = 0;   // absorbed: nodes that no longer launch anything
};

// The result of the analysis, per node of the Description (no backend involved: this part also
// builds and runs without CUDA).
enum class FusedKind { None, LayerNormModulate, RmsNormModulate, RmsNormRope, GatedResidual };
struct FusedGroup {
    FusedKind kind = FusedKind::None;
    vrhino::neural_graph::ValueId x = 0, shift = 0, scale = 0, cosine = 0, sine = 0, residual = 0, branch = 0, gate = 0;
    std::optional<vrhino::neural_graph::ValueId> weight, bias;
    float epsilon = 0.0f;
    int heads = 1;
};
struct FusionPlan {
    std::vector<FusedGroup> anchored;   // per node: the chain that ends (and runs) at this node
    std::vector<char> absorbed;         // per node: inside a chain, launches nothing itself
    FusionStats stats;                  // counts of the chains found
};
FusionPlan plan_fusion(const vrhino::neural_graph::Description& description);

// What evaluate_fused needs from a backend beyond vrhino::Backend: the four one-kernel chains.
// B200Backend provides them; a test can provide stand-ins (fault injection on the host, no GPU).
class FusedOperators {
public:
    virtual ~FusedOperators() = default;
    virtual vrhino::Backend& backend() = 0;
    virtual vrhino::Tensor layer_norm_modulate(const vrhino::Tensor& x, const vrhino::Tensor* weight, const vrhino::Tensor* bias,
                                               float eps, const vrhino::Tensor& shift, const vrhino::Tensor& scale,
                                               vrhino::DType output) = 0;
    virtual vrhino::Tensor rms_norm_modulate(const vrhino::Tensor& x, float eps, const vrhino::Tensor& shift,
                                             const vrhino::Tensor& scale, vrhino::DType output) = 0;
    virtual vrhino::Tensor rms_norm_rope(const vrhino::Tensor& x, const vrhino::Tensor* weight, float eps,
                                         const vrhino::Tensor* cosine, const vrhino::Tensor* sine, int heads,
                                         vrhino::DType output) = 0;
    virtual vrhino::Tensor gated_residual(const vrhino::Tensor& residual, const vrhino::Tensor& branch,
                                          const vrhino::Tensor* gate, vrhino::DType state) = 0;
};

// Same contract as neural_graph::evaluate: inputs / parameters bound in slot order, host
// tensors uploaded on demand, outputs in d.outputs order after a synchronize().  Failures are
// reported the way the reference evaluator reports them (neural_graph_evaluator.cpp:84-93, :162-175):
// always a neural_graph::GraphError carrying code, phase (Bind / Run / Drain / Capture) and the node,
// value and primitive being worked on; a backend exception becomes BackendFailure (CompletionFailure
// while draining); and after a failure that may have left work enqueued the device is drained exactly
// once, a failure of that drain being kept in secondary_completion instead of replacing the error.
// drain = false leaves out that per-graph device synchronisation
// (native/src/runtime/neural_graph_evaluator.cpp:151): every operator of the backend is enqueued on
// the same stream, so a caller that keeps enqueueing (the next block's graph) needs no host
// wait between graphs; a device fault then surfaces at the caller's next synchronising call
// instead of as this graph's completion failure.
std::vector<vrhino::Tensor> evaluate_fused(FusedOperators& operators, const vrhino::neural_graph::Graph& graph,
                                           const std::vector<vrhino::Tensor>& inputs,
                                           const std::vector<vrhino::Tensor>& parameters,
                                           FusionStats* stats = nullptr, bool drain = true);
std::vector<vrhino::Tensor> evaluate_fused(B200Backend& backend, const vrhino::neural_graph::Graph& graph,
                                           const std::vector<vrhino::Tensor>& inputs,
                                           const std::vector<vrhino::Tensor>& parameters,
                                           FusionStats* stats = nullptr, bool drain = true);

}  // namespace vrhino_b200
