// RMSNorm + modulate instantiations whose input row is first computed as the gated residual of the
// residual stream (bf16, or F32 with a bf16 branch): the LTX block's residual update followed by its
// next RMSNorm -> modulate, in one pass.
#include "vrb_rowwise_inst.cuh"

namespace vrb {
namespace rowwise {
VRB_DEFINE_ROW_VARIANT(kNormRms, kPostModulate, kBf16Bf16Pre)
VRB_DEFINE_ROW_VARIANT(kNormRms, kPostModulateStaged, kBf16Bf16Pre)
VRB_DEFINE_ROW_VARIANT(kNormRms, kPostModulate, kF32Pre)
VRB_DEFINE_ROW_VARIANT(kNormRms, kPostModulateStaged, kF32Pre)
// Mochi: residual + rms_norm(branch) * tanh(gate), then rms_norm(.) * (1 + scale) of the updated stream
VRB_DEFINE_ROW_VARIANT(kNormRms, kPostScaleX, kBf16Bf16Pre)
}  // namespace rowwise
}  // namespace vrb
