// Fusion pass over the reference's executable graph (native/src/runtime/neural_graph.h): the
// Wan / LTX production graphs spell the non-GEMM chains out node by node
// (native/src/architectures/wan_self_attention_graph.h:46-70,
//  native/src/architectures/ltx_self_attention_graph.cpp:30-44).  evaluate_fused() walks the same
// admitted Graph as neural_graph::evaluate (native/src/runtime/neural_graph_evaluator.cpp:72-178),
// recognises three chains and runs each as ONE kernel of the B200 backend; every other node is
// dispatched exactly as the reference's evaluator dispatches it.  No architecture file changes.
//
//   LayerNorm -> [Cast F32] -> Mul(., Add(1, scale)) -> Add(., shift) -> [Cast execution]
//                                                              => B200Backend::layer_norm_modulate
//   RmsNorm(last axis, weight) -> Reshape[B,S,H,d] -> Rope -> Cast execution
//                                                              => B200Backend::rms_norm_rope
//   Add([Cast F32] residual, Mul([Cast F32] branch, gate))     => B200Backend::gated_residual
//
// A chain is fused only when its interior values have no other consumer and are not graph
// outputs (so a diagnostics graph, which exports them, runs node by node).
#pragma once

#include <vector>

#include "b200_backend.h"
#include "runtime/neural_graph.h"

namespace vrhino_b200 {

struct FusionStats {
    int layer_norm_modulate = 0, rms_norm_rope = 0, gated_residual = 0;
    int nodes_total = 0, nodes_absorbed = 0;   // absorbed: nodes that no longer launch anything
};

// Same contract as neural_graph::evaluate: inputs / parameters bound in slot order, host
// tensors uploaded on demand, outputs in d.outputs order after a synchronize().
std::vector<vrhino::Tensor> evaluate_fused(B200Backend& backend, const vrhino::neural_graph::Graph& graph,
                                           const std::vector<vrhino::Tensor>& inputs,
                                           const std::vector<vrhino::Tensor>& parameters,
                                           FusionStats* stats = nullptr);

}  // namespace vrhino_b200
