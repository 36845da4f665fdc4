// LayerNorm + adaLN modulate with the modulation vector staged in shared memory.
#include "vrb_rowwise_inst.cuh"

namespace vrb {
namespace rowwise {
VRB_DEFINE_ROW_VARIANT(kNormLayer, kPostModulateStaged, kF32F32)
VRB_DEFINE_ROW_VARIANT(kNormLayer, kPostModulateStaged, kBf16Bf16)
VRB_DEFINE_ROW_VARIANT(kNormRms, kPostModulateStaged, kF32F32)
VRB_DEFINE_ROW_VARIANT(kNormRms, kPostModulateStaged, kBf16Bf16)
}  // namespace rowwise
}  // namespace vrb
