// Tensor-core (tcgen05) prefill GEMM entry points used by the dispatcher.
#pragma once

#include "kernels.cuh"

namespace vx {

// Whether the tcgen05 GEMM path is usable in this process (driver entry point for tensor maps
// resolved, device is sm_100).
bool gemm_available();

// y[m, rows] = x . W^T through the tensor cores with activations rounded as `act` declares
// (VELOX_ACT_NVFP4 with `divisor`, VELOX_ACT_FP8_ROW, or VELOX_ACT_BF16). Handles the fused
// SwiGLU form. Returns VELOX_ERR_UNSUPPORTED for shapes it does not take.
int gemm_linear(const LinearArgs& a, int act, float divisor);

// Synchronises the device and returns the tensor-core kernels' status word: 0, or the code of the
// first bounded wait that gave up.
int gemm_status_sync();

}  // namespace vx
