// Tensor-core (tcgen05) prefill GEMM entry points used by the dispatcher.
#pragma once

#include <cuda.h>  // CUtensorMap

#include "kernels.cuh"

namespace vx {

// Whether the tcgen05 GEMM path is usable in this process (driver entry point for tensor maps
// resolved, device is sm_100).
bool gemm_available();

// y[m, rows] = x . W^T through the tensor cores with activations rounded as `act` declares
// (VELOX_ACT_NVFP4 with `divisor`, VELOX_ACT_FP8_ROW, or VELOX_ACT_BF16). Handles the fused
// SwiGLU form. Returns VELOX_ERR_UNSUPPORTED for shapes it does not take.
int gemm_linear(const LinearArgs& a, int act, float divisor);

// Up to three NVFP4 views of one width that read the same pre-quantised activations (a.q_codes /
// a.q_atoms), as one launch. `sync` (may be NULL): tensor-parallel flags to wait for.
int gemm_linears_q4(const LinearArgs* parts, int n, float divisor, const velox_sm100_tp_sync* sync);

// 2-D tensor map over a row-major byte matrix [rows, row_bytes]: boxes of 128 bytes x box_rows rows,
// 128-byte swizzle.
int gemm_make_map_u8(CUtensorMap* map, const void* ptr, long long rows, long long row_bytes, int box_rows);

int gemm_make_rs_maps(void* maps_dev, const unsigned long long* ptrs, int n, int rows_per_owner, long long cols);

// Decode linear (m <= 16) on the tensor cores: NVFP4 views with activations quantised to NVFP4 with
// `divisor` (or taken from a.q_codes / a.q_atoms), or FP8-row views with FP8-row activations (`act`
// says which). VELOX_ERR_UNSUPPORTED for other shapes.
int gemv_tc(const LinearArgs& a, int act, float divisor);
// The same for up to three views of one width that share the activations, in one launch.
int gemv_nvfp4_tc_parts(const LinearArgs* parts, int n, float divisor);

// Synchronises the device and returns the tensor-core kernels' status word: 0, or the code of the
// first bounded wait that gave up.
int gemm_status_sync();
// Clears it (and the words that elect a launch's last CTA), after a synchronise by the caller.
int gemm_status_reset();

}  // namespace vx
