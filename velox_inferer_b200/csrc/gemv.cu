// Decode / speculative-verify GEMV (m <= 16): y[m, rows] = x[m, k] . W^T on stored NVFP4,
// FP8-E4M3-per-row and GGML Q4_K rows. HBM-bound: every weight byte is read once with 128-bit
// loads, unpacked in registers, multiplied against bf16 activations held in shared memory and
// reduced with warp shuffles. Activations are rounded to bf16 (ActQuant::Bf16); accumulation is
// f32. The fused form writes silu(gate . x) * (up . x) without an intermediate buffer.
//
// Work split: a lane owns one 64-wide k tile per step (32 B of NVFP4 codes, 64 B of FP8 codes, or
// one 64-value Q4_K chunk) of each of the warp's four rows. For NVFP4 the four rows of a warp are
// {c, c+32, c+64, c+96} of one 128-row tile, so their block scales are the 16 adjacent bytes of
// one swizzled scale atom (crates/velox-core/src/format.rs:345-354).
//
// Reference counterpart: linear_gemv_vec_kernel / linear_gemv_ggml_kernel,
// crates/velox-cuda/kernels/portable_model.cu:1448-1716.
#include <cstdlib>

#include <cuda_fp4.h>
#include <cuda_fp8.h>

#include "common.cuh"
#include "kernels.cuh"

namespace vx {

constexpr int GEMV_WARPS = 4;
constexpr int GEMV_R = 4;

struct GemvParams {
    const uint8_t* w;
    long long n, k, row_begin;
    int rows;
    const uint8_t* w2;  // up view of the fused SwiGLU form
    long long n2, row_begin2;
    const float* x;
    const uint16_t* xb;
    int t0;        // first token of this pass
    int mt_valid;  // tokens in this pass (<= MT)
    float* y;
    uint16_t* yb;
    long long ld, col;
};

// Eight bf16 (one 16-byte chunk) -> f32.
__device__ __forceinline__ void bf16x8_to_f32(const uint4& v, float (&f)[8]) {
    const uint32_t u[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
    for (int i = 0; i < 4; i++) {
        f[2 * i] = __uint_as_float(u[i] << 16);
        f[2 * i + 1] = __uint_as_float(u[i] & 0xffff0000u);
    }
}

// Eight E2M1 codes of one word (low nibble = lower k) -> f32.
__device__ __forceinline__ void e2m1x8_to_f32(uint32_t word, float (&f)[8]) {
#pragma unroll
    for (int b = 0; b < 4; b++) {
        const __half2_raw h =
            __nv_cvt_fp4x2_to_halfraw2((__nv_fp4x2_storage_t)((word >> (8 * b)) & 0xffu), __NV_E2M1);
        const float2 v = __half22float2(*reinterpret_cast<const __half2*>(&h));
        f[2 * b] = v.x;
        f[2 * b + 1] = v.y;
    }
}

// Four E4M3 codes of one word -> f32.
__device__ __forceinline__ void e4m3x4_to_f32(uint32_t word, float (&f)[4]) {
#pragma unroll
    for (int b = 0; b < 2; b++) {
        const __half2_raw h = __nv_cvt_fp8x2_to_halfraw2(
            (__nv_fp8x2_storage_t)((word >> (16 * b)) & 0xffffu), __NV_E4M3);
        const float2 v = __half22float2(*reinterpret_cast<const __half2*>(&h));
        f[2 * b] = v.x;
        f[2 * b + 1] = v.y;
    }
}

__device__ __forceinline__ uint4 ldg16(const uint8_t* p) {
    return __ldg(reinterpret_cast<const uint4*>(p));
}

// ---- per-format accumulation: acc[j][t] += sum_k W[row_j][k] * x[t][k] over this lane's tiles ----

template <int MT>
__device__ __forceinline__ void accum_nvfp4(const uint8_t* __restrict__ w, long long n, long long k,
                                            const long long (&prow)[GEMV_R],
                                            const bool (&valid)[GEMV_R], const uint4* xs,
                                            int tiles, int lane, float (&acc)[GEMV_R][MT]) {
    const long long scale_plane = align256(n * k / 2);
    for (int T = lane; T < tiles; T += VX_WARP) {
        uint32_t codes[GEMV_R][8];
        uint32_t sc[GEMV_R];
#pragma unroll
        for (int j = 0; j < GEMV_R; j++) {
            uint4 a = make_uint4(0, 0, 0, 0), b = a;
            sc[j] = 0;
            if (valid[j]) {
                const uint8_t* p = w + (prow[j] * k) / 2 + (long long)T * 32;
                a = ldg16(p);
                b = ldg16(p + 16);
                sc[j] = __ldg(reinterpret_cast<const uint32_t*>(
                    w + scale_plane + nvfp4_scale_offset(prow[j], 4LL * T, k)));
            }
            codes[j][0] = a.x; codes[j][1] = a.y; codes[j][2] = a.z; codes[j][3] = a.w;
            codes[j][4] = b.x; codes[j][5] = b.y; codes[j][6] = b.z; codes[j][7] = b.w;
        }
#pragma unroll
        for (int g = 0; g < 4; g++) {
            float part[GEMV_R][MT];
#pragma unroll
            for (int j = 0; j < GEMV_R; j++)
#pragma unroll
                for (int t = 0; t < MT; t++) part[j][t] = 0.0f;
#pragma unroll
            for (int h = 0; h < 2; h++) {
                const int c = 2 * g + h;
                float xv[MT][8];
#pragma unroll
                for (int t = 0; t < MT; t++)
                    bf16x8_to_f32(xs[((long long)t * tiles + T) * 8 + (c ^ (T & 7))], xv[t]);
#pragma unroll
                for (int j = 0; j < GEMV_R; j++) {
                    float wv[8];
                    e2m1x8_to_f32(codes[j][c], wv);
#pragma unroll
                    for (int t = 0; t < MT; t++)
#pragma unroll
                        for (int e = 0; e < 8; e++) part[j][t] = fmaf(wv[e], xv[t][e], part[j][t]);
                }
            }
#pragma unroll
            for (int j = 0; j < GEMV_R; j++) {
                const float s = e4m3_to_f32((sc[j] >> (8 * g)) & 0xffu);
#pragma unroll
                for (int t = 0; t < MT; t++) acc[j][t] = fmaf(s, part[j][t], acc[j][t]);
            }
        }
    }
}

template <int MT>
__device__ __forceinline__ void accum_fp8(const uint8_t* __restrict__ w, long long k,
                                          const long long (&prow)[GEMV_R],
                                          const bool (&valid)[GEMV_R], const uint4* xs, int tiles,
                                          int lane, float (&acc)[GEMV_R][MT]) {
    for (int T = lane; T < tiles; T += VX_WARP) {
        uint4 codes[GEMV_R][4];
#pragma unroll
        for (int j = 0; j < GEMV_R; j++) {
#pragma unroll
            for (int q = 0; q < 4; q++) codes[j][q] = make_uint4(0, 0, 0, 0);
            if (valid[j]) {
                const uint8_t* p = w + prow[j] * k + (long long)T * 64;
#pragma unroll
                for (int q = 0; q < 4; q++) codes[j][q] = ldg16(p + 16 * q);
            }
        }
#pragma unroll
        for (int c = 0; c < 8; c++) {
            float xv[MT][8];
#pragma unroll
            for (int t = 0; t < MT; t++)
                bf16x8_to_f32(xs[((long long)t * tiles + T) * 8 + (c ^ (T & 7))], xv[t]);
#pragma unroll
            for (int j = 0; j < GEMV_R; j++) {
                const uint4 q = codes[j][c >> 1];
                const uint32_t w0 = (c & 1) ? q.z : q.x, w1 = (c & 1) ? q.w : q.y;
                float wv[8];
                float lo[4], hi[4];
                e4m3x4_to_f32(w0, lo);
                e4m3x4_to_f32(w1, hi);
#pragma unroll
                for (int e = 0; e < 4; e++) { wv[e] = lo[e]; wv[4 + e] = hi[e]; }
#pragma unroll
                for (int t = 0; t < MT; t++)
#pragma unroll
                    for (int e = 0; e < 8; e++) acc[j][t] = fmaf(wv[e], xv[t][e], acc[j][t]);
            }
        }
    }
}

// Q4_K: tile T = chunk (T % 4) of block (T / 4): values 64c..64c+31 are the low nibbles of
// qs[32c..32c+32), values 64c+32..64c+63 the high nibbles (ggml.rs:196-210).
template <int MT>
__device__ __forceinline__ void accum_q4k(const uint8_t* __restrict__ w, long long k,
                                          const long long (&prow)[GEMV_R],
                                          const bool (&valid)[GEMV_R], const uint4* xs, int tiles,
                                          int lane, float (&acc)[GEMV_R][MT]) {
    const long long row_bytes = k / 256 * 144;
    for (int T = lane; T < tiles; T += VX_WARP) {
        const int blk = T >> 2, c = T & 3;
        uint4 qs[GEMV_R][2];
        float d1[GEMV_R], m1[GEMV_R], d2[GEMV_R], m2[GEMV_R];
#pragma unroll
        for (int j = 0; j < GEMV_R; j++) {
            qs[j][0] = qs[j][1] = make_uint4(0, 0, 0, 0);
            d1[j] = m1[j] = d2[j] = m2[j] = 0.0f;
            if (valid[j]) {
                const uint8_t* b = w + prow[j] * row_bytes + (long long)blk * 144;
                const uint4 head = ldg16(b);
                qs[j][0] = ldg16(b + 16 + 32 * c);
                qs[j][1] = ldg16(b + 32 + 32 * c);
                const float d = f16_bits_to_f32(head.x & 0xffffu);
                const float dmin = f16_bits_to_f32(head.x >> 16);
                uint8_t s12[12];
                const uint32_t hw[3] = {head.y, head.z, head.w};
#pragma unroll
                for (int i = 0; i < 12; i++) s12[i] = (uint8_t)(hw[i >> 2] >> (8 * (i & 3)));
                uint32_t sc, mn;
                q4k_scale_min(2 * c, s12, sc, mn);
                d1[j] = d * (float)sc;
                m1[j] = dmin * (float)mn;
                q4k_scale_min(2 * c + 1, s12, sc, mn);
                d2[j] = d * (float)sc;
                m2[j] = dmin * (float)mn;
            }
        }
#pragma unroll
        for (int half = 0; half < 2; half++) {
            float qx[GEMV_R][MT], sx[MT];
#pragma unroll
            for (int t = 0; t < MT; t++) sx[t] = 0.0f;
#pragma unroll
            for (int j = 0; j < GEMV_R; j++)
#pragma unroll
                for (int t = 0; t < MT; t++) qx[j][t] = 0.0f;
#pragma unroll
            for (int cc = 0; cc < 4; cc++) {  // 8 values each
                float xv[MT][8];
#pragma unroll
                for (int t = 0; t < MT; t++) {
                    bf16x8_to_f32(xs[((long long)t * tiles + T) * 8 + ((4 * half + cc) ^ (T & 7))], xv[t]);
#pragma unroll
                    for (int e = 0; e < 8; e++) sx[t] += xv[t][e];
                }
#pragma unroll
                for (int j = 0; j < GEMV_R; j++) {
                    const uint4 q = qs[j][cc >> 1];
                    const uint32_t w0 = (cc & 1) ? q.z : q.x, w1 = (cc & 1) ? q.w : q.y;
                    // The four nibbles of a word at once, each moved to the top of a mantissa: one
                    // byte permute then makes the float 1 + q / 16 (bits 0x3F800000 | q << 19) with no
                    // conversion and no subtraction. The sum below is therefore sum(x) + sum(q x) / 16;
                    // the known sum(x) is taken off together with the block minimum.
                    const uint32_t n0 = ((half ? (w0 >> 1) : (w0 << 3)) & 0x78787878u) | 0x80808080u;
                    const uint32_t n1 = ((half ? (w1 >> 1) : (w1 << 3)) & 0x78787878u) | 0x80808080u;
#pragma unroll
                    for (int e = 0; e < 8; e++) {
                        const float qv = __uint_as_float(
                            __byte_perm(e < 4 ? n0 : n1, 0x3F000000u, 0x7044u | ((uint32_t)(e & 3) << 8)));
#pragma unroll
                        for (int t = 0; t < MT; t++) qx[j][t] = fmaf(qv, xv[t][e], qx[j][t]);
                    }
                }
            }
#pragma unroll
            for (int j = 0; j < GEMV_R; j++) {
                // d sc sum(q x) - dmin mn sum(x), with sum(q x) = 16 (qx - sum(x))
                const float ds = 16.0f * (half ? d2[j] : d1[j]);
                const float ms = ds + (half ? m2[j] : m1[j]);
#pragma unroll
                for (int t = 0; t < MT; t++) acc[j][t] += ds * qx[j][t] - ms * sx[t];
            }
        }
    }
}

template <int FMT, int MT, bool SWIGLU>
__global__ void __launch_bounds__(GEMV_WARPS* VX_WARP)
gemv_kernel(const GemvParams p) {
    extern __shared__ uint4 xs[];
    const int tiles = (int)(p.k / 64);
    const int warp = threadIdx.x / VX_WARP, lane = threadIdx.x % VX_WARP;
    const long long unit = (long long)blockIdx.x * GEMV_WARPS + warp;
    long long prow[GEMV_R], urow[GEMV_R];
    bool valid[GEMV_R];
#pragma unroll
    for (int j = 0; j < GEMV_R; j++) {
        if (FMT == VELOX_FMT_NVFP4) {
            const long long tile128 = p.row_begin / 128 + unit / 32;
            prow[j] = tile128 * 128 + unit % 32 + 32 * j;
        } else {
            prow[j] = p.row_begin + unit * GEMV_R + j;
        }
        valid[j] = prow[j] >= p.row_begin && prow[j] < p.row_begin + p.rows;
        urow[j] = p.row_begin2 + (prow[j] - p.row_begin);
    }

    // Stage this pass's tokens as bf16, chunk c of tile T at slot c ^ (T & 7) (conflict-free
    // 128-bit reads when consecutive lanes read the same chunk of consecutive tiles).
    for (int idx = threadIdx.x; idx < MT * tiles * 8; idx += blockDim.x) {
        const int t = idx / (tiles * 8);
        const int rem = idx - t * tiles * 8;
        const int T = rem >> 3, c = rem & 7;
        uint4 v = make_uint4(0, 0, 0, 0);
        if (t < p.mt_valid) {
            const long long off = (long long)(p.t0 + t) * p.k + (long long)T * 64 + c * 8;
            if (p.xb) {
                v = *reinterpret_cast<const uint4*>(p.xb + off);
            } else {
                const float4 a = *reinterpret_cast<const float4*>(p.x + off);
                const float4 b = *reinterpret_cast<const float4*>(p.x + off + 4);
                v.x = (uint32_t)bf16_bits(a.x) | ((uint32_t)bf16_bits(a.y) << 16);
                v.y = (uint32_t)bf16_bits(a.z) | ((uint32_t)bf16_bits(a.w) << 16);
                v.z = (uint32_t)bf16_bits(b.x) | ((uint32_t)bf16_bits(b.y) << 16);
                v.w = (uint32_t)bf16_bits(b.z) | ((uint32_t)bf16_bits(b.w) << 16);
            }
        }
        xs[((long long)t * tiles + T) * 8 + (c ^ (T & 7))] = v;
    }
    __syncthreads();

    float acc[GEMV_R][MT], acc2[GEMV_R][MT];
#pragma unroll
    for (int j = 0; j < GEMV_R; j++)
#pragma unroll
        for (int t = 0; t < MT; t++) acc[j][t] = acc2[j][t] = 0.0f;

    if (FMT == VELOX_FMT_NVFP4) {
        accum_nvfp4<MT>(p.w, p.n, p.k, prow, valid, xs, tiles, lane, acc);
        if (SWIGLU) accum_nvfp4<MT>(p.w2, p.n2, p.k, urow, valid, xs, tiles, lane, acc2);
    } else if (FMT == VELOX_FMT_FP8_ROW_BF16) {
        accum_fp8<MT>(p.w, p.k, prow, valid, xs, tiles, lane, acc);
        if (SWIGLU) accum_fp8<MT>(p.w2, p.k, urow, valid, xs, tiles, lane, acc2);
    } else {
        accum_q4k<MT>(p.w, p.k, prow, valid, xs, tiles, lane, acc);
        if (SWIGLU) accum_q4k<MT>(p.w2, p.k, urow, valid, xs, tiles, lane, acc2);
    }

#pragma unroll
    for (int j = 0; j < GEMV_R; j++)
#pragma unroll
        for (int t = 0; t < MT; t++) {
            acc[j][t] = warp_sum(acc[j][t]);
            if (SWIGLU) acc2[j][t] = warp_sum(acc2[j][t]);
        }

    if (lane == 0) {
#pragma unroll
        for (int j = 0; j < GEMV_R; j++) {
            if (!valid[j]) continue;
            float s1 = 1.0f, s2 = 1.0f;
            bool divide = false;
            if (FMT == VELOX_FMT_NVFP4) {
                divide = true;
                s1 = *reinterpret_cast<const float*>(p.w + align256(p.n * p.k / 2) + p.n * p.k / 16);
                if (SWIGLU)
                    s2 = *reinterpret_cast<const float*>(p.w2 + align256(p.n2 * p.k / 2) + p.n2 * p.k / 16);
            } else if (FMT == VELOX_FMT_FP8_ROW_BF16) {
                s1 = bf16_bits_to_f32(*reinterpret_cast<const unsigned short*>(
                    p.w + align256(p.n * p.k) + 2 * prow[j]));
                if (SWIGLU)
                    s2 = bf16_bits_to_f32(*reinterpret_cast<const unsigned short*>(
                        p.w2 + align256(p.n2 * p.k) + 2 * urow[j]));
            }
#pragma unroll
            for (int t = 0; t < MT; t++) {
                if (t >= p.mt_valid) continue;
                float v = divide ? acc[j][t] / s1 : acc[j][t] * s1;
                if (SWIGLU) {
                    const float u = divide ? acc2[j][t] / s2 : acc2[j][t] * s2;
                    v = v / (1.0f + expf(-v)) * u;
                }
                const long long o = (long long)(p.t0 + t) * p.ld + p.col + (prow[j] - p.row_begin);
                if (p.y) p.y[o] = v;
                if (p.yb) p.yb[o] = bf16_bits(v);
            }
        }
    }
}

template <int FMT, int MT, bool SWIGLU>
static int launch_gemv(const GemvParams& p, long long units) {
    const size_t smem = (size_t)MT * (size_t)(p.k / 64) * 8 * sizeof(uint4);
    if (smem > 200 * 1024) return VELOX_ERR_UNSUPPORTED;
    auto kern = gemv_kernel<FMT, MT, SWIGLU>;
    if (smem > 48 * 1024) {
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return (int)e;
    }
    const long long blocks = (units + GEMV_WARPS - 1) / GEMV_WARPS;
    TimedRegion timed(TIMED_GEMV);
    kern<<<(unsigned)blocks, GEMV_WARPS * VX_WARP, smem, stream()>>>(p);
    return launch_status();
}

template <int FMT, bool SWIGLU>
static int gemv_fmt(const LinearArgs& a) {
    GemvParams p;
    p.w = a.w.w; p.n = a.w.n; p.k = a.w.k; p.row_begin = a.w.row_begin; p.rows = a.w.rows;
    p.w2 = a.up.w; p.n2 = a.up.n; p.row_begin2 = a.up.row_begin;
    p.x = a.x; p.xb = a.xb; p.y = a.y; p.yb = a.yb; p.ld = a.ld; p.col = a.col;
    long long units;
    if (FMT == VELOX_FMT_NVFP4) {
        const long long first = p.row_begin / 128, last = (p.row_begin + p.rows - 1) / 128;
        units = (last - first + 1) * 32;
    } else {
        units = (p.rows + GEMV_R - 1) / GEMV_R;
    }
    for (int t0 = 0; t0 < a.m;) {
        const int left = a.m - t0;
        p.t0 = t0;
        int rc;
        if (left >= 4 || left == 3) {
            p.mt_valid = left >= 4 ? 4 : 3;
            rc = launch_gemv<FMT, 4, SWIGLU>(p, units);
        } else if (left == 2) {
            p.mt_valid = 2;
            rc = launch_gemv<FMT, 2, SWIGLU>(p, units);
        } else {
            p.mt_valid = 1;
            rc = launch_gemv<FMT, 1, SWIGLU>(p, units);
        }
        if (rc != 0) return rc;
        t0 += p.mt_valid;
    }
    return 0;
}

int gemv(const LinearArgs& a) {
    if (a.w.k % 64 != 0 || a.m < 1 || a.m > 16) return VELOX_ERR_UNSUPPORTED;
    if (a.x && (reinterpret_cast<uintptr_t>(a.x) & 15)) return VELOX_ERR_UNSUPPORTED;
    if (a.xb && (reinterpret_cast<uintptr_t>(a.xb) & 15)) return VELOX_ERR_UNSUPPORTED;
    switch (a.w.format) {
        case VELOX_FMT_NVFP4: {
            int rc = gemv_nvfp4_tma(a);
            if (rc != VELOX_ERR_UNSUPPORTED) return rc;
            rc = gemv_nvfp4_mma(a);
            if (rc != VELOX_ERR_UNSUPPORTED) return rc;
        }
            return a.swiglu ? gemv_fmt<VELOX_FMT_NVFP4, true>(a) : gemv_fmt<VELOX_FMT_NVFP4, false>(a);
        case VELOX_FMT_FP8_ROW_BF16: {
            const int rc = gemv_fp8_mma(a);
            if (rc != VELOX_ERR_UNSUPPORTED) return rc;
        }
            return a.swiglu ? gemv_fmt<VELOX_FMT_FP8_ROW_BF16, true>(a)
                            : gemv_fmt<VELOX_FMT_FP8_ROW_BF16, false>(a);
        case VELOX_FMT_GGML_Q4_K: {
            const int rc = gemv_q4k_mma(a);
            if (rc != VELOX_ERR_UNSUPPORTED) return rc;
        }
            return a.swiglu ? gemv_fmt<VELOX_FMT_GGML_Q4_K, true>(a)
                            : gemv_fmt<VELOX_FMT_GGML_Q4_K, false>(a);
        default:
            return VELOX_ERR_UNSUPPORTED;
    }
}

}  // namespace vx
