// NVFP4 decode GEMV (m <= 16) with the inner products on the tensor cores.
//
// The SIMT form spends its issue slots converting every weight to f32 and multiplying it; on B200
// that, not HBM, bounds it. Here a lane only unpacks: E2M1 codes become f16 pairs with the
// hardware converter, are multiplied by their E4M3 block scale (exact in f16: six significant
// bits), and go straight into mma.sync.m16n8k16 as the A operand; the activations are the B
// operand (tokens along n), the accumulator is f32.
//
// Work split. A CTA owns 32 weight rows of one 128-row scale tile: chunk rows {c0..c0+7} in each
// of the four 32-row bands, so that per 64-wide k tile the scales it needs are 128 contiguous
// bytes of the stored atom (crates/velox-core/src/format.rs:345-354). Its warps split K; each warp
// step covers 128 k: lane (g, t) of the mma fragment layout loads 16 bytes (32 codes) of chunk
// row c0+g in every band at k offset 32 t, and one 16-byte atom row with all its scales. The two
// m16 row tiles of a warp are bands {0, 1} and {2, 3}. K order inside an mma is a permutation
// (lane t supplies codes 4j..4j+3 of its 32 for mma j), matched by the order the activations are
// read from shared memory. Partial sums of the K-splitting warps are added in shared memory.
//
// Activations: bf16 (ActQuant::Bf16) converted to f16 after a per-token power-of-two scaling that
// puts max|x| in [2^14, 2^15), so nothing overflows; values more than 2^28 below the token's
// maximum lose low bits in f16's subnormal range, an error far below f32 accumulation rounding.
//
// Reference counterpart: linear_gemv_vec_kernel, crates/velox-cuda/kernels/portable_model.cu:1448-1626.
#include <cuda_fp4.h>
#include <cuda_fp8.h>

#include "common.cuh"
#include "kernels.cuh"

namespace vx {

constexpr int MG_WARPS = 4;      // K-splitting warps per CTA
constexpr int MG_ROWS = 32;      // rows per CTA: 8 chunk rows x 4 bands
constexpr int MG_XPAD = 32;      // f16 elements of padding per token row (64 B: conflict-free reads)

struct MmaGemvParams {
    const uint8_t* w[2];        // [1] = up view for the fused SwiGLU form
    long long n[2], row_begin[2];
    long long k;
    int rows;
    const float* x;
    const uint16_t* xb;
    int m;
    float* y;
    uint16_t* yb;
    long long ld, col;
    long long units;            // 32-row units the grid strides over
};

__device__ __forceinline__ void mma_f16(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, "
        "{%0, %1, %2, %3};"
        : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

// Two E2M1 codes of byte `sel` of `word` -> f16x2, times the f16x2 scale.
__device__ __forceinline__ uint32_t unpack2(uint32_t word, int sel, __half2 scale) {
    const __half2_raw h =
        __nv_cvt_fp4x2_to_halfraw2((__nv_fp4x2_storage_t)((word >> (8 * sel)) & 0xffu), __NV_E2M1);
    const __half2 v = __hmul2(*reinterpret_cast<const __half2*>(&h), scale);
    return *reinterpret_cast<const uint32_t*>(&v);
}

template <int NT, bool SWIGLU>
__global__ void __launch_bounds__(MG_WARPS* VX_WARP, 3)
gemv_nvfp4_mma_kernel(const MmaGemvParams p) {
    extern __shared__ __align__(16) uint8_t smem[];
    const int warp = threadIdx.x / VX_WARP, lane = threadIdx.x % VX_WARP;
    const int g = lane >> 2, t = lane & 3;
    const long long k = p.k;
    const int xpitch = (int)k + MG_XPAD;              // f16 elements per token row
    __half* xs = reinterpret_cast<__half*>(smem);    // [m][xpitch], chunk-permuted per 128 k
    float* tok_scale = reinterpret_cast<float*>(smem + (size_t)p.m * xpitch * 2);   // [m] 2^-e
    float* red = tok_scale + NT * 8;                 // [MG_WARPS][SWIGLU ? 2 : 1][32 rows][NT*8]

    // ---- stage the activations once per CTA: per token max -> power-of-two scale -> f16 ----
    // Only the m real tokens get a row; fragment slots of absent tokens are fed zeros. A warp owns
    // whole tokens, so no block-wide step separates the two passes of a token.
    for (int tk = warp; tk < p.m; tk += MG_WARPS) {
        float amax = 0.0f;
        const int chunks = (int)(k / 8);
        for (int c8 = lane; c8 < chunks; c8 += VX_WARP) {
            float f[8];
            if (p.xb) {
                const uint4 v = __ldg(reinterpret_cast<const uint4*>(p.xb + (long long)tk * k + 8LL * c8));
                const uint32_t u[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
                for (int i = 0; i < 4; i++) {
                    f[2 * i] = __uint_as_float(u[i] << 16);
                    f[2 * i + 1] = __uint_as_float(u[i] & 0xffff0000u);
                }
            } else {
#pragma unroll
                for (int i = 0; i < 8; i++) f[i] = round_bf16(p.x[(long long)tk * k + 8LL * c8 + i]);
            }
#pragma unroll
            for (int i = 0; i < 8; i++) amax = fmaxf(amax, fabsf(f[i]));
        }
        amax = warp_max(amax);
        // 2^e with max|x| * 2^e in [2^14, 2^15) (give or take a rounding of log2): exact scaling
        int e = 0;
        if (amax > 0.0f && amax < 3.0e38f) e = 14 - (int)floorf(log2f(amax));
        e = max(-60, min(60, e));
        const float up = exp2f((float)e);
        if (lane == 0) tok_scale[tk] = exp2f((float)-e);
        for (int c8 = lane; c8 < chunks; c8 += VX_WARP) {
            float f[8];
            if (p.xb) {
                const uint4 v = __ldg(reinterpret_cast<const uint4*>(p.xb + (long long)tk * k + 8LL * c8));
                const uint32_t u[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
                for (int i = 0; i < 4; i++) {
                    f[2 * i] = __uint_as_float(u[i] << 16);
                    f[2 * i + 1] = __uint_as_float(u[i] & 0xffff0000u);
                }
            } else {
#pragma unroll
                for (int i = 0; i < 8; i++) f[i] = round_bf16(p.x[(long long)tk * k + 8LL * c8 + i]);
            }
            // k = 8 c8: inside each 128-k step the 16-byte chunk (t, i) is stored at slot i * 4 + t
            const int step = c8 >> 4, in8 = c8 & 15, tt = in8 >> 2, i4 = in8 & 3;
            uint4 o;
            __half2 h;
            h = __floats2half2_rn(f[0] * up, f[1] * up); o.x = *reinterpret_cast<uint32_t*>(&h);
            h = __floats2half2_rn(f[2] * up, f[3] * up); o.y = *reinterpret_cast<uint32_t*>(&h);
            h = __floats2half2_rn(f[4] * up, f[5] * up); o.z = *reinterpret_cast<uint32_t*>(&h);
            h = __floats2half2_rn(f[6] * up, f[7] * up); o.w = *reinterpret_cast<uint32_t*>(&h);
            *reinterpret_cast<uint4*>(xs + (size_t)tk * xpitch + step * 128 + (i4 * 4 + tt) * 8) = o;
        }
    }
    __syncthreads();

    // ---- 32-row units of this CTA (persistent: unit = blockIdx.x, + gridDim.x, ...) ----
    for (long long unit = blockIdx.x; unit < p.units; unit += gridDim.x) {
    const long long tile128 = p.row_begin[0] / 128 + unit / 4;
    const int c0 = (int)(unit % 4) * 8;
    const int steps_total = (int)(k / 128);
    const int s_begin = (int)((long long)warp * steps_total / MG_WARPS);
    const int s_end = (int)((long long)(warp + 1) * steps_total / MG_WARPS);
    const int k_tiles = (int)(k / 64);

    float acc[SWIGLU ? 2 : 1][2][NT][4];
#pragma unroll
    for (int v = 0; v < (SWIGLU ? 2 : 1); v++)
#pragma unroll
        for (int rt = 0; rt < 2; rt++)
#pragma unroll
            for (int nt = 0; nt < NT; nt++)
#pragma unroll
                for (int q = 0; q < 4; q++) acc[v][rt][nt][q] = 0.0f;

#pragma unroll
    for (int v = 0; v < (SWIGLU ? 2 : 1); v++) {
        const uint8_t* w = p.w[v];
        const long long n = p.n[v];
        const long long scale_plane = align256(n * k / 2);
        // band rows of this lane's chunk row, in the view's parent coordinates
        long long prow[4];
        bool valid[4];
#pragma unroll
        for (int b = 0; b < 4; b++) {
            const long long r0 = tile128 * 128 + c0 + g + 32 * b;   // gate / plain coordinates
            valid[b] = r0 >= p.row_begin[0] && r0 < p.row_begin[0] + p.rows;
            prow[b] = v == 0 ? r0 : p.row_begin[1] + (r0 - p.row_begin[0]);
        }
        // Loads run one step ahead of the arithmetic so a warp always has a step in flight.
        auto load_step = [&](int s, uint4 (&codes)[4], uint32_t (&sc2)[4]) {
#pragma unroll
            for (int b = 0; b < 4; b++) {
                codes[b] = make_uint4(0, 0, 0, 0);
                sc2[b] = 0;
                if (valid[b] && s < s_end) {
                    codes[b] = __ldg(reinterpret_cast<const uint4*>(w + (prow[b] * k) / 2 + s * 64 + t * 16));
                    // scales: groups 2t, 2t+1 of this step's eight, adjacent bytes of the atom row
                    const long long off = scale_plane + nvfp4_scale_offset(prow[b], 8LL * s + 2 * t, k);
                    sc2[b] = __ldg(reinterpret_cast<const unsigned short*>(w + off));
                }
            }
        };
        uint4 codes[4], codes_n[4];
        uint32_t sc2[4], sc2_n[4];
        load_step(s_begin, codes, sc2);
        for (int s = s_begin; s < s_end; s++) {
            load_step(s + 1, codes_n, sc2_n);
            // activations of this step for token g of each n tile: 4 x 16 bytes
            uint4 xv[NT][4];
#pragma unroll
            for (int nt = 0; nt < NT; nt++)
#pragma unroll
                for (int i = 0; i < 4; i++)
                    xv[nt][i] = (nt * 8 + g < p.m)
                                    ? *reinterpret_cast<const uint4*>(xs + (size_t)(nt * 8 + g) * xpitch + s * 128 + (i * 4 + t) * 8)
                                    : make_uint4(0, 0, 0, 0);
#pragma unroll
            for (int rt = 0; rt < 2; rt++) {
                const int b_lo = 2 * rt, b_hi = 2 * rt + 1;
                const __half2_raw slo = __nv_cvt_fp8x2_to_halfraw2((__nv_fp8x2_storage_t)sc2[b_lo], __NV_E4M3);
                const __half2_raw shi = __nv_cvt_fp8x2_to_halfraw2((__nv_fp8x2_storage_t)sc2[b_hi], __NV_E4M3);
                const __half2 slo2 = *reinterpret_cast<const __half2*>(&slo);
                const __half2 shi2 = *reinterpret_cast<const __half2*>(&shi);
                const uint32_t wl[4] = {codes[b_lo].x, codes[b_lo].y, codes[b_lo].z, codes[b_lo].w};
                const uint32_t wh[4] = {codes[b_hi].x, codes[b_hi].y, codes[b_hi].z, codes[b_hi].w};
#pragma unroll
                for (int j = 0; j < 8; j++) {
                    // codes 4j..4j+3 of the lane's 32: word j/2, bytes 2(j%2) and 2(j%2)+1; group j/4
                    const __half2 sl = (j < 4) ? __low2half2(slo2) : __high2half2(slo2);
                    const __half2 sh = (j < 4) ? __low2half2(shi2) : __high2half2(shi2);
                    uint32_t a[4];
                    a[0] = unpack2(wl[j >> 1], 2 * (j & 1), sl);
                    a[1] = unpack2(wh[j >> 1], 2 * (j & 1), sh);
                    a[2] = unpack2(wl[j >> 1], 2 * (j & 1) + 1, sl);
                    a[3] = unpack2(wh[j >> 1], 2 * (j & 1) + 1, sh);
#pragma unroll
                    for (int nt = 0; nt < NT; nt++) {
                        // x values 4j..4j+3 of the lane's 32: 16-byte chunk j/2, half (j%2)
                        const uint4 c = xv[nt][j >> 1];
                        const uint32_t b0 = (j & 1) ? c.z : c.x, b1 = (j & 1) ? c.w : c.y;
                        mma_f16(acc[v][rt][nt], a, b0, b1);
                    }
                }
            }
#pragma unroll
            for (int b = 0; b < 4; b++) {
                codes[b] = codes_n[b];
                sc2[b] = sc2_n[b];
            }
        }
    }

    // ---- add the K-splitting warps' partial sums, then write ----
    constexpr int V = SWIGLU ? 2 : 1;
    // lane (g, t) holds, per (v, rt, nt): rows band 2rt (d0, d1) and band 2rt+1 (d2, d3), tokens nt*8 + 2t, +1
#pragma unroll
    for (int v = 0; v < V; v++)
#pragma unroll
        for (int rt = 0; rt < 2; rt++)
#pragma unroll
            for (int nt = 0; nt < NT; nt++)
#pragma unroll
                for (int q = 0; q < 4; q++) {
                    const int band = 2 * rt + (q >> 1);
                    const int row = band * 8 + g;                       // 0..31 within the CTA
                    const int tok = nt * 8 + 2 * t + (q & 1);
                    red[(((size_t)warp * V + v) * MG_ROWS + row) * (NT * 8) + tok] = acc[v][rt][nt][q];
                }
    __syncthreads();
    const float div0 = *reinterpret_cast<const float*>(p.w[0] + align256(p.n[0] * k / 2) + p.n[0] * k / 16);
    const float div1 = SWIGLU ? *reinterpret_cast<const float*>(p.w[1] + align256(p.n[1] * k / 2) + p.n[1] * k / 16) : 1.0f;
    for (int idx = threadIdx.x; idx < MG_ROWS * NT * 8; idx += blockDim.x) {
        const int row = idx / (NT * 8), tok = idx % (NT * 8);
        if (tok >= p.m) continue;
        const int band = row >> 3, gg = row & 7;
        const long long r0 = tile128 * 128 + c0 + gg + 32 * band;
        if (r0 < p.row_begin[0] || r0 >= p.row_begin[0] + p.rows) continue;
        float s0 = 0.0f, s1 = 0.0f;
#pragma unroll
        for (int wv = 0; wv < MG_WARPS; wv++) {
            s0 += red[(((size_t)wv * V + 0) * MG_ROWS + row) * (NT * 8) + tok];
            if (SWIGLU) s1 += red[(((size_t)wv * V + 1) * MG_ROWS + row) * (NT * 8) + tok];
        }
        float val = s0 * tok_scale[tok] / div0;
        if (SWIGLU) {
            const float u = s1 * tok_scale[tok] / div1;
            val = val / (1.0f + expf(-val)) * u;
        }
        const long long o = (long long)tok * p.ld + p.col + (r0 - p.row_begin[0]);
        if (p.y) p.y[o] = val;
        if (p.yb) p.yb[o] = bf16_bits(val);
    }
    __syncthreads();   // the partial-sum buffer is reused by the next unit
    }
}

template <int NT, bool SWIGLU>
static int launch_mma_gemv(const MmaGemvParams& p) {
    static int sms = 0;
    if (sms == 0) {
        int dev = 0;
        cudaGetDevice(&dev);
        cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
        if (sms <= 0) sms = 148;
    }
    const long long blocks = p.units < 3LL * sms ? p.units : 3LL * sms;
    const size_t smem = (size_t)p.m * (p.k + MG_XPAD) * 2 + (size_t)NT * 8 * 4 +
                        (size_t)MG_WARPS * (SWIGLU ? 2 : 1) * MG_ROWS * NT * 8 * 4;
    if (smem > 220 * 1024) return VELOX_ERR_UNSUPPORTED;
    auto kern = gemv_nvfp4_mma_kernel<NT, SWIGLU>;
    if (smem > 48 * 1024) {
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return (int)e;
    }
    TimedRegion timed(TIMED_GEMV);
    kern<<<(unsigned)blocks, MG_WARPS * VX_WARP, smem, stream()>>>(p);
    return launch_status();
}

// NVFP4, m <= 16, k a multiple of 128 with at least one 128-k step per warp; the SwiGLU form also
// needs gate and up at the same offset inside a 128-row tile.
int gemv_nvfp4_mma(const LinearArgs& a) {
    if (a.w.format != VELOX_FMT_NVFP4 || a.m < 1 || a.m > 16) return VELOX_ERR_UNSUPPORTED;
    if (a.w.k % 128 != 0 || a.w.k / 128 < MG_WARPS) return VELOX_ERR_UNSUPPORTED;
    if (a.swiglu && (a.w.row_begin - a.up.row_begin) % 128 != 0) return VELOX_ERR_UNSUPPORTED;
    MmaGemvParams p{};
    p.w[0] = a.w.w; p.n[0] = a.w.n; p.row_begin[0] = a.w.row_begin;
    p.w[1] = a.swiglu ? a.up.w : a.w.w; p.n[1] = a.swiglu ? a.up.n : a.w.n;
    p.row_begin[1] = a.swiglu ? a.up.row_begin : a.w.row_begin;
    p.k = a.w.k; p.rows = a.w.rows; p.x = a.x; p.xb = a.xb; p.m = a.m;
    p.y = a.y; p.yb = a.yb; p.ld = a.ld; p.col = a.col;
    p.units = ((a.w.row_begin + a.w.rows - 1) / 128 - a.w.row_begin / 128 + 1) * 4;
    if (a.xb && (reinterpret_cast<uintptr_t>(a.xb) & 15)) return VELOX_ERR_UNSUPPORTED;
    if (a.m <= 8) return a.swiglu ? launch_mma_gemv<1, true>(p) : launch_mma_gemv<1, false>(p);
    return a.swiglu ? launch_mma_gemv<2, true>(p) : launch_mma_gemv<2, false>(p);
}

}  // namespace vx
