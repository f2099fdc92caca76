// Decode (m <= 16) on GGML Q4_K rows through the warp-level tensor-core MMA.
//
// A Q4_K weight is d * sc * q - dmin * mn with a 4-bit q and 6-bit sc, mn shared by 32 weights
// (crates/velox-core/src/ggml.rs:159-210). Unpacking q to a float and multiplying it costs a general
// ALU two to three instructions per weight and per token, which bounds the SIMT kernel well below the
// memory rate as soon as there is more than one token. Here q goes to bf16 with one byte permute
// per two weights (0x4180 | q << 3 is the bf16 number 16 + q, exactly; an offset of 128 would be a
// plain byte insert but costs accuracy, because the offset's share of the sum cancels only in the
// epilogue) and mma.sync.m16n8k16 multiplies sixteen rows by eight tokens at once, the tokens as
// the B operand in bf16 (ActQuant::Bf16, which every policy admits). Per 32-weight group the MMA
// result c = sum((16 + q) x) is folded into the running sums as d sc c - (16 d sc + dmin mn) sum(x);
// sum(x) per group and token comes from an MMA whose A operand is all ones, which delivers it in
// the accumulator layout at once. The fused SwiGLU form runs the gate view and then the up view
// through the same loop and forms silu(gate) * up from the two complete sums.
//
// Work split: a block owns 16 or 32 rows (one or two MMA row tiles); its warps (two, four or eight)
// each take a part of K and the parts are added in warp order at the end, so results do not depend
// on timing. Within a warp, lane (g, t) loads 8 bytes of each of its rows per 64-weight chunk: the
// dot product does not care about the order along K, so the K slots of the MMA are assigned to
// whatever bytes a lane holds and the activations are fetched in the matching order (one 16-byte
// load of eight consecutive bf16 per group and token tile, from L1, one step ahead). Asking for
// the weight bytes with L2 prefetches at block start made the kernel 10 to 20 % slower and is not
// done.
//
// Reference counterpart: linear_gemv_ggml_kernel, crates/velox-cuda/kernels/portable_model.cu:1628-1716.
#include <cstdlib>
#include <type_traits>

#include "common.cuh"
#include "kernels.cuh"

namespace vx {


struct Q4kParams {
    const uint8_t* w;
    long long k, row_begin;
    int rows;
    const uint8_t* w2;    // fused SwiGLU form: the up view (w is the gate view), same k and row count
    long long row_begin2;
    const uint16_t* xb;   // [m, k] bf16
    int m;
    float* y;
    uint16_t* yb;
    long long ld, col;
};

// d = a b (+ c): the first MMA of a group starts from zero constants, the second adds in place.
__device__ __forceinline__ void mma_bf16_16816_first(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                                     uint32_t b0, uint32_t b1) {
    asm(
        "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, "
        "{%10, %10, %10, %10};"
        : "=f"(d[0]), "=f"(d[1]), "=f"(d[2]), "=f"(d[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1), "f"(0.0f));
}

__device__ __forceinline__ void mma_bf16_16816(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                               uint32_t b0, uint32_t b1) {
    asm(
        "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, "
        "{%0, %1, %2, %3};"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

// What a lane keeps of one row's block header: d, dmin and the eight 6-bit (scale, min) pairs as
// four words of bytes.
struct Q4kHead {
    float d, dmin, nd23, ndmin23;   // the last two: -d 2^23, -dmin 2^23
    uint32_t sc03, sc47, mn03, mn47;
};

__device__ __forceinline__ Q4kHead q4k_head(const uint4& h) {
    Q4kHead r;
    r.d = f16_bits_to_f32(h.x & 0xffffu);
    r.dmin = f16_bits_to_f32(h.x >> 16);
    r.nd23 = -r.d * 8388608.0f;
    r.ndmin23 = -r.dmin * 8388608.0f;
    // ggml.rs:159-169, four bytes at a time
    r.sc03 = h.y & 0x3f3f3f3fu;
    r.mn03 = h.z & 0x3f3f3f3fu;
    r.sc47 = (h.w & 0x0f0f0f0fu) | ((h.y >> 2) & 0x30303030u);
    r.mn47 = ((h.w >> 4) & 0x0f0f0f0fu) | ((h.z >> 2) & 0x30303030u);
    return r;
}

// d sc and 16 d sc + dmin mn of group S (a compile-time index): byte -> float by placing it in the
// mantissa of 2^23, the 2^23 taken off inside the multiply-add.
template <int S>
__device__ __forceinline__ void q4k_group_factors(const Q4kHead& h, float& ds, float& off) {
    const uint32_t scw = S < 4 ? h.sc03 : h.sc47, mnw = S < 4 ? h.mn03 : h.mn47;
    const float scf = __uint_as_float(__byte_perm(scw, 0x4B000000u, 0x7440u | (uint32_t)(S & 3)));
    const float mnf = __uint_as_float(__byte_perm(mnw, 0x4B000000u, 0x7440u | (uint32_t)(S & 3)));
    ds = fmaf(h.d, scf, h.nd23);
    off = fmaf(16.0f, ds, fmaf(h.dmin, mnf, h.ndmin23));
}

template <int MT, int NB, int QM_WARPS, bool PIPE, bool SWIGLU = false>
__global__ void __launch_bounds__(QM_WARPS * 32, QM_WARPS == 8 ? (NB == 1 ? 3 : 2) : !PIPE ? 7 : QM_WARPS == 2 ? 7 : NB == 1 ? 4 : 2) gemv_q4k_mma_kernel(const Q4kParams p) {
    constexpr int QM_ROWS = 16 * MT;   // weight rows per block: MT row tiles of the MMA; QM_WARPS: K parts, one per warp
    __shared__ float red[QM_WARPS - 1][MT * NB * 4][32];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, g = lane >> 2, t = lane & 3;
    const long long row_bytes = p.k / 256 * 144;
    const int bt = (int)(p.k / 256);
    const int kb0 = warp * bt / QM_WARPS, kb1 = (warp + 1) * bt / QM_WARPS;
    const long long r_first = p.row_begin + (long long)blockIdx.x * QM_ROWS;
    const long long r_last = p.row_begin + p.rows - 1;

    float acc[MT][NB][4], gate[MT][NB][4];   // (gate: the first pass of the fused SwiGLU form)
    const uint8_t* rp[MT][2];

    // token rows of this lane's B fragments
    const uint16_t* xrow[NB];
#pragma unroll
    for (int nb = 0; nb < NB; nb++) xrow[nb] = p.xb + (nb * 8 + g < p.m ? (long long)(nb * 8 + g) * p.k : 0) + 8 * t;

    // The next block's bytes are requested before the current block is worked on.
    auto load_blk = [&](int blk, uint4 (&hd)[MT][2], uint2 (&q)[MT][2][4]) {
#pragma unroll
        for (int mt = 0; mt < MT; mt++)
#pragma unroll
            for (int h = 0; h < 2; h++) {
                const uint8_t* b = rp[mt][h] + (long long)blk * 144;
                hd[mt][h] = __ldcs(reinterpret_cast<const uint4*>(b));
#pragma unroll
                for (int c = 0; c < 4; c++) q[mt][h][c] = __ldcs(reinterpret_cast<const uint2*>(b + 16 + 32 * c + 8 * t));
            }
    };
    // B fragments of the step being worked on: eight consecutive bf16 of this lane's token per token
    // tile. A token past m reads token 0; its accumulator columns are never stored.
    auto load_b = [&](long long k0, uint4 (&b)[NB]) {
#pragma unroll
        for (int nb = 0; nb < NB; nb++) b[nb] = __ldg(reinterpret_cast<const uint4*>(xrow[nb] + k0));
    };
    // Plain form: one pass over the view. Fused SwiGLU: the gate view, then the up view's rows at the
    // same offsets; silu(gate) * up is formed after both sums are complete.
#pragma unroll 1
    for (int pass = 0; pass < (SWIGLU ? 2 : 1); pass++) {
    const uint8_t* wbase = pass == 0 ? p.w : p.w2;
    const long long shift = pass == 0 ? 0 : p.row_begin2 - p.row_begin;
    // the lane's rows: tile mt, half h -> row r_first + 16 mt + 8 h + g (a row past the view reads the last one)
#pragma unroll
    for (int mt = 0; mt < MT; mt++)
#pragma unroll
        for (int h = 0; h < 2; h++) {
            const long long r = r_first + 16 * mt + 8 * h + g;
            rp[mt][h] = wbase + ((r < r_last ? r : r_last) + shift) * row_bytes;
        }
#pragma unroll
    for (int mt = 0; mt < MT; mt++)
#pragma unroll
        for (int nb = 0; nb < NB; nb++)
#pragma unroll
            for (int i = 0; i < 4; i++) acc[mt][nb][i] = 0.0f;
    uint4 bx[NB];
    uint4 raw_head[MT][2];
    uint2 qs[MT][2][4];
    if (kb0 < kb1) {
        if (PIPE) load_blk(kb0, raw_head, qs);
        load_b((long long)kb0 * 256, bx);
    }
    for (int blk = kb0; blk < kb1; blk++) {
        uint4 next_head[MT][2];
        uint2 next_qs[MT][2][4];
        if (PIPE)
            load_blk(blk + 1 < kb1 ? blk + 1 : blk, next_head, next_qs);   // (the last pass repeats its own block: no branch)
        else
            load_blk(blk, raw_head, qs);
        Q4kHead head[MT][2];
#pragma unroll
        for (int mt = 0; mt < MT; mt++)
#pragma unroll
            for (int h = 0; h < 2; h++) head[mt][h] = q4k_head(raw_head[mt][h]);

        // One step per 32-weight group: group S = 2c + half is the low (half = 0) or high nibbles of
        // the 32 bytes of chunk c. The next step's activations are requested before this step's work.
        auto step = [&](auto ss) {
            constexpr int S = decltype(ss)::value, c = S / 2, half = S % 2;
            uint4 nx[NB];
            load_b(S < 7 ? (long long)blk * 256 + (S + 1) * 32 : (long long)(blk + 1 < kb1 ? blk + 1 : blk) * 256, nx);
            float2 sx[NB];   // sum of the group's x for tokens 2t and 2t + 1: an MMA with ones as its A operand
#pragma unroll
            for (int nb = 0; nb < NB; nb++) {
                float ones[4];
                mma_bf16_16816_first(ones, 0x3F803F80u, 0x3F803F80u, 0x3F803F80u, 0x3F803F80u, bx[nb].x, bx[nb].y);
                mma_bf16_16816(ones, 0x3F803F80u, 0x3F803F80u, 0x3F803F80u, 0x3F803F80u, bx[nb].z, bx[nb].w);
                sx[nb] = make_float2(ones[0], ones[1]);
            }
#pragma unroll
            for (int mt = 0; mt < MT; mt++) {
                const uint2 qa = qs[mt][0][c], qb = qs[mt][1][c];
                // each nibble to the top of a bf16 mantissa: the byte 0x80 | q << 3 under the byte 0x41 is
                // the bf16 number 16 + q
                const uint32_t a_lo = ((half ? (qa.x >> 1) : (qa.x << 3)) & 0x78787878u) | 0x80808080u;   // values 8t .. 8t+3 of row g
                const uint32_t a_hi = ((half ? (qa.y >> 1) : (qa.y << 3)) & 0x78787878u) | 0x80808080u;   // values 8t+4 .. 8t+7
                const uint32_t b_lo = ((half ? (qb.x >> 1) : (qb.x << 3)) & 0x78787878u) | 0x80808080u;   // the same of row g + 8
                const uint32_t b_hi = ((half ? (qb.y >> 1) : (qb.y << 3)) & 0x78787878u) | 0x80808080u;
                // K slots (2t, 2t+1) and (2t+8, 2t+9) of the first MMA take values 8t .. 8t+3, those of
                // the second take 8t+4 .. 8t+7
                const uint32_t a0 = __byte_perm(a_lo, 0x41414141u, 0x4140u), a2 = __byte_perm(a_lo, 0x41414141u, 0x4342u);
                const uint32_t a1 = __byte_perm(b_lo, 0x41414141u, 0x4140u), a3 = __byte_perm(b_lo, 0x41414141u, 0x4342u);
                const uint32_t e0 = __byte_perm(a_hi, 0x41414141u, 0x4140u), e2 = __byte_perm(a_hi, 0x41414141u, 0x4342u);
                const uint32_t e1 = __byte_perm(b_hi, 0x41414141u, 0x4140u), e3 = __byte_perm(b_hi, 0x41414141u, 0x4342u);
                float ds_a, off_a, ds_b, off_b;
                q4k_group_factors<S>(head[mt][0], ds_a, off_a);
                q4k_group_factors<S>(head[mt][1], ds_b, off_b);
#pragma unroll
                for (int nb = 0; nb < NB; nb++) {
                    float cfr[4];
                    mma_bf16_16816_first(cfr, a0, a1, a2, a3, bx[nb].x, bx[nb].y);
                    mma_bf16_16816(cfr, e0, e1, e2, e3, bx[nb].z, bx[nb].w);
                    acc[mt][nb][0] = fmaf(-off_a, sx[nb].x, fmaf(ds_a, cfr[0], acc[mt][nb][0]));
                    acc[mt][nb][1] = fmaf(-off_a, sx[nb].y, fmaf(ds_a, cfr[1], acc[mt][nb][1]));
                    acc[mt][nb][2] = fmaf(-off_b, sx[nb].x, fmaf(ds_b, cfr[2], acc[mt][nb][2]));
                    acc[mt][nb][3] = fmaf(-off_b, sx[nb].y, fmaf(ds_b, cfr[3], acc[mt][nb][3]));
                }
            }
#pragma unroll
            for (int nb = 0; nb < NB; nb++) bx[nb] = nx[nb];
        };
        step(std::integral_constant<int, 0>{});
        step(std::integral_constant<int, 1>{});
        step(std::integral_constant<int, 2>{});
        step(std::integral_constant<int, 3>{});
        step(std::integral_constant<int, 4>{});
        step(std::integral_constant<int, 5>{});
        step(std::integral_constant<int, 6>{});
        step(std::integral_constant<int, 7>{});
        if (!PIPE) continue;
#pragma unroll
        for (int mt = 0; mt < MT; mt++)
#pragma unroll
            for (int h = 0; h < 2; h++) {
                raw_head[mt][h] = next_head[mt][h];
#pragma unroll
                for (int c = 0; c < 4; c++) qs[mt][h][c] = next_qs[mt][h][c];
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
    }   // pass

    // add the K parts in warp order (the gate sums first, through the same buffer)
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
            for (int w = 0; w < QM_WARPS - 1; w++)
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
    for (int w = 0; w < QM_WARPS - 1; w++)
#pragma unroll
        for (int mt = 0; mt < MT; mt++)
#pragma unroll
            for (int nb = 0; nb < NB; nb++)
#pragma unroll
                for (int i = 0; i < 4; i++) acc[mt][nb][i] += red[w][(mt * NB + nb) * 4 + i][lane];

    // lane (g, t) holds rows g and g + 8 of each tile for tokens 2t and 2t + 1 of each token tile
#pragma unroll
    for (int mt = 0; mt < MT; mt++)
#pragma unroll
        for (int h = 0; h < 2; h++) {
            const long long r = r_first + 16 * mt + 8 * h + g;
            if (r > r_last) continue;
#pragma unroll
            for (int nb = 0; nb < NB; nb++)
#pragma unroll
                for (int i = 0; i < 2; i++) {
                    const int tok = nb * 8 + 2 * t + i;
                    if (tok >= p.m) continue;
                    float v = acc[mt][nb][2 * h + i];
                    if (SWIGLU) {
                        const float gv = gate[mt][nb][2 * h + i];
                        v = gv / (1.0f + expf(-gv)) * v;
                    }
                    const long long o = (long long)tok * p.ld + p.col + (r - p.row_begin);
                    if (p.y) p.y[o] = v;
                    if (p.yb) p.yb[o] = bf16_bits(v);
                }
        }
}

int gemv_q4k_mma(const LinearArgs& a) {
    if (a.w.format != VELOX_FMT_GGML_Q4_K || a.w.k % 256 != 0 || a.m < 1 || a.m > 16 ||
        a.w.rows < 1 || (reinterpret_cast<uintptr_t>(a.w.w) & 15))
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

    Q4kParams p;
    p.w = a.w.w;
    p.k = k;
    p.row_begin = a.w.row_begin;
    p.rows = (int)a.w.rows;
    p.w2 = nullptr;
    p.row_begin2 = 0;
    if (a.swiglu) {
        if (a.up.format != VELOX_FMT_GGML_Q4_K || a.up.k != k || a.up.rows != a.w.rows ||
            (reinterpret_cast<uintptr_t>(a.up.w) & 15))
            return VELOX_ERR_UNSUPPORTED;
        p.w2 = a.up.w;
        p.row_begin2 = a.up.row_begin;
    }
    p.xb = xb;
    p.m = a.m;
    p.y = a.y;
    p.yb = a.yb;
    p.ld = a.ld;
    p.col = a.col;

    TimedRegion timed(TIMED_GEMV);
    // One row tile per block while that still leaves the machine short of warps (and the tokens fit L1),
    // two otherwise: the second tile halves what a block reads of the activations per weight byte.
    static int sms = 0;
    if (sms == 0) {
        int dev = 0;
        cudaGetDevice(&dev);
        cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
        if (sms <= 0) sms = 148;
    }
    const bool one = (a.w.rows + 31) / 32 < 6LL * sms && (size_t)a.m * k * sizeof(uint16_t) <= 160 * 1024;
    const unsigned blocks = (unsigned)((a.w.rows + (one ? 16 : 32) - 1) / (one ? 16 : 32));
    // Up to eight tokens: four K parts per block, loads at the top of each block of K (72 registers,
    // seven blocks per SM). More tokens: the next block's weight bytes are requested a block ahead,
    // which costs 24 registers per row tile, so two K parts per block keep every block resident.
    if (a.swiglu) {
        const unsigned gblocks = (unsigned)((a.w.rows + 15) / 16);
        if (a.m <= 8) gemv_q4k_mma_kernel<1, 1, 4, false, true><<<gblocks, 128, 0, stream()>>>(p);
        else gemv_q4k_mma_kernel<1, 2, 2, true, true><<<gblocks, 64, 0, stream()>>>(p);
        return launch_status();
    }
    // Few row tiles with a long K (a down projection): eight K parts per block, so that the machine
    // still has warps to hide latency with. (Eight parts on [14336, 4096] too, for more warps per
    // SM, were slower: 17.1 us against 15.9.)
    if (one && (long long)blocks * 4 < 12LL * sms && k >= 8 * 256) {
        if (a.m <= 8) gemv_q4k_mma_kernel<1, 1, 8, false><<<blocks, 256, 0, stream()>>>(p);
        else gemv_q4k_mma_kernel<1, 2, 8, false><<<blocks, 256, 0, stream()>>>(p);
        return launch_status();
    }
    if (a.m <= 8) {
        if (one) gemv_q4k_mma_kernel<1, 1, 4, false><<<blocks, 128, 0, stream()>>>(p);
        else gemv_q4k_mma_kernel<2, 1, 4, true><<<blocks, 128, 0, stream()>>>(p);
    } else {
        if (one) gemv_q4k_mma_kernel<1, 2, 2, true><<<blocks, 64, 0, stream()>>>(p);
        else gemv_q4k_mma_kernel<2, 2, 4, true><<<blocks, 128, 0, stream()>>>(p);
    }
    return launch_status();
}

}  // namespace vx
