// LayerNorm instantiations whose F32 input row is first computed as the gated residual of an F32
// residual stream and a bf16 branch (the production dtype contract): plain / affine, and adaLN modulate.
#include "vrb_rowwise_inst.cuh"

namespace vrb {
namespace rowwise {
VRB_DEFINE_ROW_VARIANT(kNormLayer, kPostNone, kF32Pre)
VRB_DEFINE_ROW_VARIANT(kNormLayer, kPostModulate, kF32Pre)
VRB_DEFINE_ROW_VARIANT(kNormLayer, kPostModulateStaged, kF32Pre)
}  // namespace rowwise
}  // namespace vrb
