// LayerNorm instantiations whose input row is first computed as the bf16 gated residual
// (residual update + the norm that follows it in one pass): plain / affine, and adaLN modulate.
#include "vrb_rowwise_inst.cuh"

namespace vrb {
namespace rowwise {
VRB_DEFINE_ROW_VARIANT(kNormLayer, kPostNone, kBf16Bf16Pre)
VRB_DEFINE_ROW_VARIANT(kNormLayer, kPostModulate, kBf16Bf16Pre)
VRB_DEFINE_ROW_VARIANT(kNormLayer, kPostModulateStaged, kBf16Bf16Pre)
}  // namespace rowwise
}  // namespace vrb
