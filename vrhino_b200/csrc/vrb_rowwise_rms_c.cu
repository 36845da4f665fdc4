// RMSNorm + RoPE with a table shared by the heads (one table row per token).
#include "vrb_rowwise_inst.cuh"

namespace vrb {
namespace rowwise {
VRB_DEFINE_ROW_VARIANT(kNormRms, kPostRopeShared, kF32F32)
VRB_DEFINE_ROW_VARIANT(kNormRms, kPostRopeShared, kBf16F32)
}  // namespace rowwise
}  // namespace vrb
