#include "common.cuh"
#include "gemm.cuh"

namespace vx {
bool gemm_available() { return false; }
int gemm_linear(const LinearArgs&, int, float) { return VELOX_ERR_UNSUPPORTED; }
}  // namespace vx
