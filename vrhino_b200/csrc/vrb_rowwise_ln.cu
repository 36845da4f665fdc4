// LayerNorm instantiations of the row kernel family (plain / cast, and fused adaLN modulate).
#include "vrb_rowwise_inst.cuh"

namespace vrb {
namespace rowwise {
VRB_DEFINE_ROW_VARIANT(kNormLayer, kPostNone, kF32F32)
VRB_DEFINE_ROW_VARIANT(kNormLayer, kPostNone, kBf16Bf16)
VRB_DEFINE_ROW_VARIANT(kNormLayer, kPostModulate, kF32F32)
VRB_DEFINE_ROW_VARIANT(kNormLayer, kPostModulate, kBf16Bf16)
}  // namespace rowwise
}  // namespace vrb
