// Total fallback for the linear family: any k, any m, any row view. One warp per output row and
// chunk of eight tokens; lanes stride over k decoding one weight at a time to its exact f32 value
// (the arithmetic of format::decode_rows, crates/velox-core/src/format.rs:426-490) and accumulate
// in f32. Used for shapes the streaming GEMV and the tensor-core GEMM do not take (k not a
// multiple of 64, unaligned activations); correctness first, speed second.
// Reference counterpart: linear_kernel, crates/velox-cuda/kernels/portable_model.cu:333-345.
#include "common.cuh"
#include "kernels.cuh"

namespace vx {

__device__ __forceinline__ float weight_at(int fmt, const uint8_t* __restrict__ w, long long n,
                                           long long k, long long r, long long c) {
    if (fmt == VELOX_FMT_NVFP4) {
        const long long scale_plane = align256(n * k / 2);
        const uint32_t byte = w[(r * k + c) / 2];
        const uint32_t code = (c & 1) ? (byte >> 4) : (byte & 0xfu);
        const float scale = e4m3_to_f32(w[scale_plane + nvfp4_scale_offset(r, c / 16, k)]);
        const float divisor = *reinterpret_cast<const float*>(w + scale_plane + n * k / 16);
        return __fdiv_rn(__fmul_rn(e2m1_to_f32(code), scale), divisor);
    }
    if (fmt == VELOX_FMT_FP8_ROW_BF16) {
        const float scale = bf16_bits_to_f32(
            (uint32_t)w[align256(n * k) + 2 * r] | ((uint32_t)w[align256(n * k) + 2 * r + 1] << 8));
        return __fmul_rn(e4m3_to_f32(w[r * k + c]), scale);
    }
    // Q4_K
    const uint8_t* blk = w + (r * (k / 256) + c / 256) * 144;
    const int in = (int)(c % 256);
    const int sub = in / 32, l = in % 32;
    const float d = f16_bits_to_f32((uint32_t)blk[0] | ((uint32_t)blk[1] << 8));
    const float dmin = f16_bits_to_f32((uint32_t)blk[2] | ((uint32_t)blk[3] << 8));
    uint32_t sc, mn;
    q4k_scale_min(sub, blk + 4, sc, mn);
    const uint32_t byte = blk[16 + 32 * (sub / 2) + l];
    const uint32_t q = (sub & 1) ? (byte >> 4) : (byte & 0xfu);
    return __fsub_rn(__fmul_rn(__fmul_rn(d, (float)sc), (float)q), __fmul_rn(dmin, (float)mn));
}

constexpr int GEN_TOK = 8;

__global__ void __launch_bounds__(256) linear_generic_kernel(const LinearArgs a) {
    const int lane = threadIdx.x % VX_WARP;
    const long long i = (long long)blockIdx.x * (blockDim.x / VX_WARP) + threadIdx.x / VX_WARP;
    if (i >= a.w.rows) return;
    const int t0 = blockIdx.y * GEN_TOK;
    const long long k = a.w.k;
    const long long r = a.w.row_begin + i, ru = a.up.row_begin + i;
    float acc[GEN_TOK], acc2[GEN_TOK];
#pragma unroll
    for (int t = 0; t < GEN_TOK; t++) acc[t] = acc2[t] = 0.0f;
    for (long long c = lane; c < k; c += VX_WARP) {
        const float wv = weight_at(a.w.format, a.w.w, a.w.n, k, r, c);
        const float uv = a.swiglu ? weight_at(a.up.format, a.up.w, a.up.n, k, ru, c) : 0.0f;
#pragma unroll
        for (int t = 0; t < GEN_TOK; t++) {
            if (t0 + t < a.m) {
                float xv;
                if (a.xb)
                    xv = bf16_bits_to_f32(a.xb[(long long)(t0 + t) * k + c]);
                else
                    xv = a.round_x ? round_bf16(a.x[(long long)(t0 + t) * k + c])
                                   : a.x[(long long)(t0 + t) * k + c];
                acc[t] = fmaf(wv, xv, acc[t]);
                acc2[t] = fmaf(uv, xv, acc2[t]);
            }
        }
    }
#pragma unroll
    for (int t = 0; t < GEN_TOK; t++) {
        acc[t] = warp_sum(acc[t]);
        if (a.swiglu) acc2[t] = warp_sum(acc2[t]);
    }
    if (lane == 0) {
#pragma unroll
        for (int t = 0; t < GEN_TOK; t++) {
            if (t0 + t >= a.m) continue;
            float v = acc[t];
            if (a.swiglu) v = v / (1.0f + expf(-v)) * acc2[t];
            const long long o = (long long)(t0 + t) * a.ld + a.col + i;
            if (a.y) a.y[o] = v;
            if (a.yb) a.yb[o] = bf16_bits(v);
        }
    }
}

int linear_generic(const LinearArgs& a) {
    const int warps = 8;
    dim3 grid((unsigned)((a.w.rows + warps - 1) / warps), (unsigned)((a.m + GEN_TOK - 1) / GEN_TOK));
    if (grid.y > 65535) return VELOX_ERR_UNSUPPORTED;
    linear_generic_kernel<<<grid, warps * VX_WARP, 0, stream()>>>(a);
    return launch_status();
}

}  // namespace vx
