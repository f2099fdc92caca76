// Decode (m <= 16) on FP8-E4M3-per-row weights with bf16 activations (ActQuant::Bf16, the rounding
// every policy admits, A16Only included) through the warp-level tensor-core MMA.
//
// An E4M3 byte s.eeee.mmm dropped into a bf16 as s.0000eeee.mmm0000 is the E4M3 value times 2^-120
// exactly, subnormals (eeee = 0) and zeros included: both formats are sign, biased exponent and a
// leading-one mantissa, only the biases differ (7 against 127). That is a shift and two masks per
// two weights instead of a conversion and a multiply per weight and per token on the general ALU,
// which is what holds the per-element kernel (gemv.cu) to a seventh of the memory rate as soon as
// there are several tokens. The activations are multiplied by 2^64 on the way in (exact in bf16 for
// any |x| < 2^63), so that products sit in the middle of the f32 range, and the epilogue takes the
// remaining 2^56 off together with the bf16 row scale (crates/velox-core/src/format.rs:147-160: row
// scales follow the code plane, padded to 256 bytes).
//
// mma.sync.m16n8k16 multiplies sixteen rows by eight tokens; the tokens are the B operand. A dot
// product does not care about the order along K, so the K slots of an MMA take whatever bytes a
// lane holds: lane (g, t) loads 16 consecutive bytes of rows g and g + 8 per 64-weight chunk, and
// the activations are fetched and paired in the matching order.
//
// Work split as in the Q4_K kernel: a block owns 16 MT rows, its warps (four or eight) each take
// a part of K, and the parts are added in warp order at the end (results do not depend
// on timing). The fused SwiGLU
// form runs the gate view and then the up view's rows through the same loop.
//
// Reference counterpart: linear_gemv_kernel on Fp8RowBf16,
// crates/velox-cuda/kernels/portable_model.cu:1448-1626.
#include <cuda_bf16.h>

#include "common.cuh"
#include "kernels.cuh"

namespace vx {

struct Fp8Params {
    const uint8_t* w;
    long long n, k, row_begin;
    int rows;
    const uint8_t* w2;    // fused SwiGLU form: the up view's parent (w: the gate view's), same k and row count
    long long n2, row_begin2;
    const uint16_t* xb;   // [m, k] bf16
    int m;
    float* y;
    uint16_t* yb;
    long long ld, col;
};

__device__ __forceinline__ void mma_bf16_k16(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                             uint32_t b0, uint32_t b1) {
    asm(
        "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, "
        "{%0, %1, %2, %3};"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// Four E4M3 bytes b0..b3 of a word -> two words of bf16 pairs: odd = (b1, b3), even = (b0, b2), each
// the byte's value times 2^-120.
__device__ __forceinline__ void e4m3x4_to_bf16(uint32_t w, uint32_t& even, uint32_t& odd) {
    odd = ((w >> 4) & 0x07F007F0u) | (w & 0x80008000u);
    const uint32_t v = w << 8;
    even = ((v >> 4) & 0x07F007F0u) | (v & 0x80008000u);
}

template <int MT, int NB, int WARPS, bool SWIGLU>
__global__ void __launch_bounds__(WARPS * 32) gemv_fp8_mma_kernel(const Fp8Params p) {
    constexpr int ROWS = 16 * MT;
    __shared__ float red[WARPS - 1][MT * NB * 4][32];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;
    const int chunks = (int)(p.k / 64);
    const int c0 = warp * chunks / WARPS, c1 = (warp + 1) * chunks / WARPS;
    const long long r_first = p.row_begin + (long long)blockIdx.x * ROWS;
    const long long r_last = p.row_begin + p.rows - 1;

    float acc[MT][NB][4], gate[MT][NB][4];
    // token rows of this lane's B fragments (a token past m reads token 0; its columns are never stored)
    const uint16_t* xrow[NB];
#pragma unroll
    for (int nb = 0; nb < NB; nb++) xrow[nb] = p.xb + (nb * 8 + g < p.m ? (long long)(nb * 8 + g) * p.k : 0) + 16 * t;
    const __nv_bfloat162 up64 = __floats2bfloat162_rn(18446744073709551616.0f, 18446744073709551616.0f);   // 2^64

#pragma unroll 1
    for (int pass = 0; pass < (SWIGLU ? 2 : 1); pass++) {
        const uint8_t* wbase = pass == 0 ? p.w : p.w2;
        const long long shift = pass == 0 ? 0 : p.row_begin2 - p.row_begin;
        const uint8_t* rp[MT][2];
#pragma unroll
        for (int mt = 0; mt < MT; mt++)
#pragma unroll
            for (int h = 0; h < 2; h++) {
                const long long r = r_first + 16 * mt + 8 * h + g;
                rp[mt][h] = wbase + ((r < r_last ? r : r_last) + shift) * p.k + 16 * t;
            }
#pragma unroll
        for (int mt = 0; mt < MT; mt++)
#pragma unroll
            for (int nb = 0; nb < NB; nb++)
#pragma unroll
                for (int i = 0; i < 4; i++) acc[mt][nb][i] = 0.0f;

        auto load_w = [&](int c, uint4 (&q)[MT][2]) {
#pragma unroll
            for (int mt = 0; mt < MT; mt++)
#pragma unroll
                for (int h = 0; h < 2; h++) q[mt][h] = __ldcs(reinterpret_cast<const uint4*>(rp[mt][h] + (long long)c * 64));
        };
        auto load_x = [&](int c, uint4 (&b)[NB][2]) {
#pragma unroll
            for (int nb = 0; nb < NB; nb++) {
                b[nb][0] = __ldg(reinterpret_cast<const uint4*>(xrow[nb] + (long long)c * 64));
                b[nb][1] = __ldg(reinterpret_cast<const uint4*>(xrow[nb] + (long long)c * 64 + 8));
            }
        };
        uint4 q[MT][2], bx[NB][2];
        if (c0 < c1) {
            load_w(c0, q);
            load_x(c0, bx);
        }
        for (int c = c0; c < c1; c++) {
            // the next chunk's bytes are requested before this chunk is worked on (the last pass
            // repeats its own chunk: no branch)
            uint4 qn[MT][2], bn[NB][2];
            const int cn = c + 1 < c1 ? c + 1 : c;
            load_w(cn, qn);
            load_x(cn, bn);
            // B fragments: the lane's 16 activations x0..x15 times 2^64, paired like the weights:
            // MMA j (j = 0..3) works on x[4j..4j+3], slots (2t, 2t+1) <- (x[4j], x[4j+2]), slots
            // (2t+8, 2t+9) <- (x[4j+1], x[4j+3]).
            uint32_t be[NB][4], bo[NB][4];
#pragma unroll
            for (int nb = 0; nb < NB; nb++) {
                const uint32_t xs[8] = {bx[nb][0].x, bx[nb][0].y, bx[nb][0].z, bx[nb][0].w,
                                        bx[nb][1].x, bx[nb][1].y, bx[nb][1].z, bx[nb][1].w};
                uint32_t sc[8];
#pragma unroll
                for (int i = 0; i < 8; i++) {
                    __nv_bfloat162 v = *reinterpret_cast<const __nv_bfloat162*>(&xs[i]);
                    v = __hmul2(v, up64);
                    sc[i] = *reinterpret_cast<const uint32_t*>(&v);
                }
#pragma unroll
                for (int j = 0; j < 4; j++) {
                    be[nb][j] = __byte_perm(sc[2 * j], sc[2 * j + 1], 0x5410u);   // (x[4j], x[4j+2])
                    bo[nb][j] = __byte_perm(sc[2 * j], sc[2 * j + 1], 0x7632u);   // (x[4j+1], x[4j+3])
                }
            }
#pragma unroll
            for (int mt = 0; mt < MT; mt++) {
                const uint32_t wa[4] = {q[mt][0].x, q[mt][0].y, q[mt][0].z, q[mt][0].w};   // row g
                const uint32_t wb[4] = {q[mt][1].x, q[mt][1].y, q[mt][1].z, q[mt][1].w};   // row g + 8
#pragma unroll
                for (int j = 0; j < 4; j++) {
                    uint32_t a0, a2, a1, a3;
                    e4m3x4_to_bf16(wa[j], a0, a2);
                    e4m3x4_to_bf16(wb[j], a1, a3);
#pragma unroll
                    for (int nb = 0; nb < NB; nb++) mma_bf16_k16(acc[mt][nb], a0, a1, a2, a3, be[nb][j], bo[nb][j]);
                }
            }
#pragma unroll
            for (int mt = 0; mt < MT; mt++)
#pragma unroll
                for (int h = 0; h < 2; h++) q[mt][h] = qn[mt][h];
#pragma unroll
            for (int nb = 0; nb < NB; nb++) {
                bx[nb][0] = bn[nb][0];
                bx[nb][1] = bn[nb][1];
            }
        }
        if (SWIGLU && pass == 0) {
#pragma unroll
            for (int mt = 0; mt < MT; mt++)
#pragma unroll
                for (int nb = 0; nb < NB; nb++)
#pragma unroll
                    for (int i = 0; i < 4; i++) gate[mt][nb][i] = acc[mt][nb][i];
        }
    }

    // add the K parts in warp order (the gate sums first, through the same buffer)
    if (WARPS > 1) {
        if (SWIGLU) {
            if (warp > 0) {
#pragma unroll
                for (int mt = 0; mt < MT; mt++)
#pragma unroll
                    for (int nb = 0; nb < NB; nb++)
#pragma unroll
                        for (int i = 0; i < 4; i++) red[warp - 1][(mt * NB + nb) * 4 + i][lane] = gate[mt][nb][i];
            }
            __syncthreads();
            if (warp == 0) {
#pragma unroll
                for (int w = 0; w < WARPS - 1; w++)
#pragma unroll
                    for (int mt = 0; mt < MT; mt++)
#pragma unroll
                        for (int nb = 0; nb < NB; nb++)
#pragma unroll
                            for (int i = 0; i < 4; i++) gate[mt][nb][i] += red[w][(mt * NB + nb) * 4 + i][lane];
            }
            __syncthreads();
        }
        if (warp > 0) {
#pragma unroll
            for (int mt = 0; mt < MT; mt++)
#pragma unroll
                for (int nb = 0; nb < NB; nb++)
#pragma unroll
                    for (int i = 0; i < 4; i++) red[warp - 1][(mt * NB + nb) * 4 + i][lane] = acc[mt][nb][i];
        }
        __syncthreads();
        if (warp != 0) return;
#pragma unroll
        for (int w = 0; w < WARPS - 1; w++)
#pragma unroll
            for (int mt = 0; mt < MT; mt++)
#pragma unroll
                for (int nb = 0; nb < NB; nb++)
#pragma unroll
                    for (int i = 0; i < 4; i++) acc[mt][nb][i] += red[w][(mt * NB + nb) * 4 + i][lane];
    }

    // lane (g, t) holds rows g and g + 8 of each tile for tokens 2t and 2t + 1 of each token tile
    const long long scales1 = align256(p.n * p.k), scales2 = SWIGLU ? align256(p.n2 * p.k) : 0;
#pragma unroll
    for (int mt = 0; mt < MT; mt++)
#pragma unroll
        for (int h = 0; h < 2; h++) {
            const long long r = r_first + 16 * mt + 8 * h + g;
            if (r > r_last) continue;
            const float s1 = bf16_bits_to_f32(*reinterpret_cast<const uint16_t*>(p.w + scales1 + 2 * r));
            float s2 = 0.0f;
            if (SWIGLU)
                s2 = bf16_bits_to_f32(*reinterpret_cast<const uint16_t*>(p.w2 + scales2 + 2 * (r + p.row_begin2 - p.row_begin)));
#pragma unroll
            for (int nb = 0; nb < NB; nb++)
#pragma unroll
                for (int i = 0; i < 2; i++) {
                    const int tok = nb * 8 + 2 * t + i;
                    if (tok >= p.m) continue;
                    // 2^-120 from the weights, 2^64 from the activations: 2^56 comes off exactly, then one rounding
                    float v = acc[mt][nb][2 * h + i] * 72057594037927936.0f;
                    if (SWIGLU) {
                        const float gv = gate[mt][nb][2 * h + i] * 72057594037927936.0f * s1;
                        v = gv / (1.0f + expf(-gv)) * (v * s2);
                    } else {
                        v *= s1;
                    }
                    const long long o = (long long)tok * p.ld + p.col + (r - p.row_begin);
                    if (p.y) p.y[o] = v;
                    if (p.yb) p.yb[o] = bf16_bits(v);
                }
        }
}

template <int MT, int NB, int WARPS>
static int launch_fp8(const Fp8Params& p, bool swiglu) {
    const unsigned blocks = (unsigned)((p.rows + 16 * MT - 1) / (16 * MT));
    if (swiglu) gemv_fp8_mma_kernel<MT, NB, WARPS, true><<<blocks, WARPS * 32, 0, stream()>>>(p);
    else gemv_fp8_mma_kernel<MT, NB, WARPS, false><<<blocks, WARPS * 32, 0, stream()>>>(p);
    return launch_status();
}

int gemv_fp8_mma(const LinearArgs& a) {
    if (a.w.format != VELOX_FMT_FP8_ROW_BF16 || a.w.k % 64 != 0 || a.m < 1 || a.m > 16 || a.w.rows < 1 ||
        (reinterpret_cast<uintptr_t>(a.w.w) & 15) || a.w.k % 16 != 0)
        return VELOX_ERR_UNSUPPORTED;
    const long long k = a.w.k;
    const uint16_t* xb = a.xb;
    if (!xb) {
        uint16_t* tmp = static_cast<uint16_t*>(scratch(SCRATCH_X_BF16, (size_t)a.m * k * sizeof(uint16_t)));
        if (!tmp) return (int)cudaErrorMemoryAllocation;
        const int rc = bf16_twin(a.x, tmp, (long long)a.m * k);
        if (rc != 0) return rc;
        xb = tmp;
    }
    if (reinterpret_cast<uintptr_t>(xb) & 15) return VELOX_ERR_UNSUPPORTED;

    Fp8Params p;
    p.w = a.w.w;
    p.n = a.w.n;
    p.k = k;
    p.row_begin = a.w.row_begin;
    p.rows = (int)a.w.rows;
    p.w2 = nullptr;
    p.n2 = 0;
    p.row_begin2 = 0;
    if (a.swiglu) {
        if (a.up.format != VELOX_FMT_FP8_ROW_BF16 || a.up.k != k || a.up.rows != a.w.rows ||
            (reinterpret_cast<uintptr_t>(a.up.w) & 15))
            return VELOX_ERR_UNSUPPORTED;
        p.w2 = a.up.w;
        p.n2 = a.up.n;
        p.row_begin2 = a.up.row_begin;
    }
    p.xb = xb;
    p.m = a.m;
    p.y = a.y;
    p.yb = a.yb;
    p.ld = a.ld;
    p.col = a.col;

    TimedRegion timed(TIMED_GEMV);
    static int sms = 0;
    if (sms == 0) {
        int dev = 0;
        cudaGetDevice(&dev);
        cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
        if (sms <= 0) sms = 148;
    }
    // Many rows: two row tiles per block halve what a block reads of the activations per weight byte.
    // Few row tiles with a long K (a down projection): eight K parts per block, so that the machine
    // has warps to hide latency with. More K parts than that were slower wherever tried (sixteen
    // on [5120, 25600]: 40 us against 37; eight instead of four on [14336, 4096]: 16.7 against 15.3).
    const long long tiles = (a.w.rows + 15) / 16;
    const bool two = a.m > 8;
    if (tiles >= 16LL * sms) return two ? launch_fp8<2, 2, 4>(p, a.swiglu) : launch_fp8<2, 1, 4>(p, a.swiglu);
    if (tiles * 4 < 12LL * sms && k >= 8 * 64 * 8) return two ? launch_fp8<1, 2, 8>(p, a.swiglu) : launch_fp8<1, 1, 8>(p, a.swiglu);
    return two ? launch_fp8<1, 2, 4>(p, a.swiglu) : launch_fp8<1, 1, 4>(p, a.swiglu);
}

}  // namespace vx
