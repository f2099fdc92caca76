// Shared helpers of the sm_100a quantized-linear kernels: stored-format geometry, exact scalar
// decoders, the bf16 rounding the twins use, launch-stream selection and grow-only scratch.
#pragma once

#include <cstdlib>

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_fp4.h>
#include <cuda_fp8.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/velox_sm100.h"

#define VX_WARP 32

namespace vx {

// ---- stored-format geometry (crates/velox-core/src/format.rs:147-177, 345-354) ---------------

__host__ __device__ __forceinline__ long long align256(long long x) {
    return (x + 255) / 256 * 256;
}

__host__ __device__ __forceinline__ long long payload_bytes(int fmt, long long n, long long k) {
    switch (fmt) {
        case VELOX_FMT_FP8_ROW_BF16: return align256(n * k) + 2 * n;
        case VELOX_FMT_NVFP4: return align256(n * k / 2) + n * k / 16 + 4;
        case VELOX_FMT_GGML_Q4_K: return n * (k / 256) * 144;
        default: return 0;
    }
}

// Byte offset of the scale of (row, 16-wide group g) inside the NVFP4 scale plane.
__host__ __device__ __forceinline__ long long nvfp4_scale_offset(long long row, long long g,
                                                                 long long k) {
    const long long k_tiles = k / 64;
    const long long row_tile = row / 128, row_inner = row % 128;
    return (row_tile * k_tiles + g / 4) * 512 + (row_inner % 32) * 16 + (row_inner / 32) * 4 +
           (g % 4);
}

// ---- early start of the next kernel in the stream (programmatic dependent launch) ----
// Returns once every kernel this launch depends on has completed and its writes are visible; at
// once if the launch was not allowed to start early.
__device__ __forceinline__ void grid_dependency_wait() {
    asm volatile("griddepcontrol.wait;" ::: "memory");
}
// Lets a dependent launch that allows it start once all CTAs of this grid have said so or exited.
__device__ __forceinline__ void grid_launch_dependents() {
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
}

constexpr int VX_MAX_PEERS = 8;   // ranks of a tensor-parallel group one kernel can store to

// f32 -> E4M3 byte and two f32 -> one byte of E2M1 codes (the first in the low nibble): the
// hardware's round-to-nearest-even, saturating conversions.
__device__ __forceinline__ uint32_t f32_to_e4m3(float v) {
    return (uint32_t)__nv_cvt_float_to_fp8(v, __NV_SATFINITE, __NV_E4M3);
}
__device__ __forceinline__ uint32_t f32x2_to_e2m1x2(float lo, float hi) {
    return (uint32_t)__nv_cvt_float2_to_fp4x2(make_float2(lo, hi), __NV_E2M1, cudaRoundNearest);
}

// ---- exact scalar decoders --------------------------------------------------------------------

// E4M3FN byte -> f32 (format.rs:320-332). The byte's low 7 bits, placed as a binary16 pattern
// shifted left by 7, are the same number scaled by 2^-8 (normals and subnormals alike), so one
// exact half->float conversion and an exact multiply give the value. 0x7f/0xff (NaN) map to 480.
__device__ __forceinline__ float e4m3_to_f32(uint32_t b) {
    const unsigned short h = (unsigned short)(((b & 0x80u) << 8) | ((b & 0x7fu) << 7));
    return __half2float(__ushort_as_half(h)) * 256.0f;
}

// E2M1 nibble -> f32 (format.rs:335-343).
__device__ __forceinline__ float e2m1_to_f32(uint32_t c) {
    // magnitudes 0, .5, 1, 1.5, 2, 3, 4, 6 doubled, packed one per nibble
    const uint32_t twice = (0xC8643210u >> ((c & 7u) * 4u)) & 0xfu;
    const float v = (float)twice * 0.5f;
    return (c & 8u) ? -v : v;
}

__device__ __forceinline__ float bf16_bits_to_f32(uint32_t bits) {
    return __uint_as_float(bits << 16);
}

// f32 -> bf16 bits, round to nearest even, NaN kept quiet (velox_common.cuh:74-82).
__host__ __device__ __forceinline__ unsigned short bf16_bits(float f) {
#ifdef __CUDA_ARCH__
    unsigned int u = __float_as_uint(f);
#else
    unsigned int u;
    memcpy(&u, &f, 4);
#endif
    if ((u & 0x7fffffffu) > 0x7f800000u) return (unsigned short)((u >> 16) | 0x40u);
    u += 0x7fffu + ((u >> 16) & 1u);
    return (unsigned short)(u >> 16);
}

__device__ __forceinline__ float round_bf16(float f) {
    return __uint_as_float(((unsigned int)bf16_bits(f)) << 16);
}

__device__ __forceinline__ float f16_bits_to_f32(uint32_t bits) {
    return __half2float(__ushort_as_half((unsigned short)bits));
}

// Q4_K 6-bit scale and min j of a block's 12 scale bytes (ggml.rs:159-169).
__device__ __forceinline__ void q4k_scale_min(int j, const uint8_t* q, uint32_t& sc, uint32_t& mn) {
    if (j < 4) {
        sc = q[j] & 63u;
        mn = q[j + 4] & 63u;
    } else {
        sc = (q[j + 4] & 0xfu) | ((uint32_t)(q[j - 4] >> 6) << 4);
        mn = (q[j + 4] >> 4) | ((uint32_t)(q[j] >> 6) << 4);
    }
}

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = VX_WARP / 2; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}

__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
    for (int o = VX_WARP / 2; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}

// ---- host side ---------------------------------------------------------------------------------

// Launch stream of the calling thread.
cudaStream_t stream();
void set_stream(cudaStream_t s);

// Launch configuration of the small kernels between the linears (norms, activation quantisers):
// early start allowed, so the blocks become resident while the kernel ahead drains and wait for it
// (grid_dependency_wait) before their first access. VELOX_SM100_NO_EARLY_START=1 turns it off.
struct EarlyLaunch {
    cudaLaunchConfig_t cfg{};
    cudaLaunchAttribute attr[1];
    EarlyLaunch(unsigned blocks, unsigned threads) {
        static const bool early = getenv("VELOX_SM100_NO_EARLY_START") == nullptr;
        cfg.gridDim = dim3(blocks);
        cfg.blockDim = dim3(threads);
        cfg.stream = stream();
        attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[0].val.programmaticStreamSerializationAllowed = 1;
        cfg.attrs = attr;
        cfg.numAttrs = early ? 1 : 0;
    }
};

// Grow-only device scratch, one pool per purpose and device. Never freed: captured CUDA graphs
// may reference it (velox_common.cuh:49-70).
enum ScratchSlot { SCRATCH_ACT_CODES = 0, SCRATCH_ACT_SCALES, SCRATCH_WEIGHT_BF16, SCRATCH_X_BF16,
                   SCRATCH_Y_F32, SCRATCH_SLOTS };
void* scratch(ScratchSlot slot, size_t bytes);

// Counts kernel launches (for the benchmark's launch report) and returns the launch's status.
void note_launch();
static inline int launch_status() {
    note_launch();
    return (int)cudaGetLastError();
}

// Optional CUDA-event timing of the main kernels, the counterpart of the reference's
// VELOX_GPU_TIMING (crates/velox-cuda/src/timing.rs:1-97): when enabled, an event pair brackets
// the kernel on its launch stream; totals per class are read back after a synchronise.
enum TimedClass { TIMED_GEMV = 0, TIMED_GEMM_FP4, TIMED_GEMM_FP8, TIMED_GEMM_BF16, TIMED_ACT_QUANT,
                  TIMED_DEQUANT, TIMED_NORM, TIMED_CLASSES };
struct TimedRegion {
    int slot;
    explicit TimedRegion(int cls);
    ~TimedRegion();
};

// check::weight + check::linear on the extents a C caller can state (check.rs:100-131).
int check_view(const velox_sm100_view* v);

}  // namespace vx
