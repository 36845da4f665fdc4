// RMSNorm instantiations of the row kernel family: fused RoPE and fused gated residual.
#include "vrb_rowwise_inst.cuh"

namespace vrb {
namespace rowwise {
VRB_DEFINE_ROW_VARIANT(kNormRms, kPostRope, kF32F32)
VRB_DEFINE_ROW_VARIANT(kNormRms, kPostRope, kBf16F32)
VRB_DEFINE_ROW_VARIANT(kNormRms, kPostGatedResidual, kF32F32)
VRB_DEFINE_ROW_VARIANT(kNormRms, kPostGatedResidual, kBf16Bf16)
}  // namespace rowwise
}  // namespace vrb
