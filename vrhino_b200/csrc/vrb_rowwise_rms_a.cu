// RMSNorm instantiations of the row kernel family: plain / cast, adaLN modulate, (1+scale).
#include "vrb_rowwise_inst.cuh"

namespace vrb {
namespace rowwise {
VRB_DEFINE_ROW_VARIANT(kNormRms, kPostNone, kF32F32)
VRB_DEFINE_ROW_VARIANT(kNormRms, kPostNone, kBf16Bf16)
VRB_DEFINE_ROW_VARIANT(kNormRms, kPostNone, kBf16F32)
VRB_DEFINE_ROW_VARIANT(kNormRms, kPostModulate, kF32F32)
VRB_DEFINE_ROW_VARIANT(kNormRms, kPostModulate, kBf16Bf16)
VRB_DEFINE_ROW_VARIANT(kNormRms, kPostScaleX, kF32F32)
VRB_DEFINE_ROW_VARIANT(kNormRms, kPostScaleX, kBf16Bf16)
}  // namespace rowwise
}  // namespace vrb
