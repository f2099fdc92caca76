// NVFP4 decode GEMV (m <= 16): weights streamed by TMA into a shared-memory ring, inner products on
// the tensor cores (mma.sync, f16 operands, f32 accumulate).
//
// Why this shape. The byte stream is what matters: 0.5625 B per weight, every byte once. Register
// loads leave too few bytes in flight; here one producer thread keeps a ring of 10 KB stages full
// with two bulk copies each (an 8 KB tensor-map box of codes and 2 KB of scale atoms; measured on
// B200, copies of 8-16 KB stream HBM at the copy-kernel rate, 1 KB copies do not), and four consumer
// warps only unpack: E2M1 pairs -> f16 with the hardware converter, times the E4M3 block scale
// (exact in f16), straight into the A operand of mma.sync.m16n8k16. The activations are the B
// operand (tokens along n).
//
// A persistent CTA walks 64-row units: two 32-row bands of a 128-row scale tile. A stage holds
// 256 k of the unit: 128 B x 64 rows of codes (128-byte swizzle) and the tile's four 512-byte scale
// atoms for those k (crates/velox-core/src/format.rs:345-354). Consumer warp w owns chunk rows
// 8w..8w+7 of both bands (one m16 row tile) for the whole K, so no partial sums cross warps. mma
// row slot g reads chunk row rho(g) = (g >> 1) | ((g & 1) << 2), which makes the swizzled 128-bit
// shared-memory reads conflict free. K order inside an mma is a permutation matched by the order
// the activations are stored.
//
// Activations: bf16 (ActQuant::Bf16) converted to f16 after an exact per-token power-of-two
// scaling that puts max|x| in [2^14, 2^15); values more than 2^28 below the token's maximum lose low
// bits in f16's subnormal range, far below f32 accumulation rounding.
//
// All mbarrier waits are bounded; a wait that gives up records a code in the status word.
//
// Reference counterpart: linear_gemv_vec_kernel, crates/velox-cuda/kernels/portable_model.cu:1448-1626.
#include <cstdlib>
#include <mutex>

#include <cuda.h>
#include <cuda_fp4.h>
#include <cuda_fp8.h>

#include "common.cuh"
#include "kernels.cuh"

namespace vx {

constexpr int TG_CONSUMERS = 4;
constexpr int TG_THREADS = (TG_CONSUMERS + 1) * VX_WARP;
constexpr int TG_STAGES = 4;
constexpr int TG_CODE_BOX = 8192;                      // 128 B x 64 rows
constexpr int TG_STAGE_BYTES = TG_CODE_BOX + 2048;     // + four 512-byte scale atoms
constexpr int TG_XPAD = 32;

struct TmaGemvParams {
    long long k;
    long long row_begin[2];
    int rows;
    long long k_tiles;
    const uint8_t* scale_plane[2];
    const float* wdiv[2];
    const float* x;
    const uint16_t* xb;
    int m;
    float* y;
    uint16_t* yb;
    long long ld, col;
    long long units;
    int splits;            // K splits per 64-row unit (work items = units * splits)
    float* partial;        // [items][V][64 rows][NT*8] partial sums when splits > 1
    int* tickets;          // [units] arrival counters, zero between launches
    int* status;
};

__device__ int g_gemv_status = 0;

namespace tg {

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ bool try_wait(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.b32 %0, 1, 0, p;\n\t}"
        : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
    return ok != 0;
}

__device__ __forceinline__ bool wait(uint32_t bar, uint32_t parity) {
    if (try_wait(bar, parity)) return true;
    unsigned long long t0;
    asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t0));
    for (uint32_t spins = 1;; spins++) {
        if (try_wait(bar, parity)) return true;
        if ((spins & 255u) == 0) {
            unsigned long long t1;
            asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t1));
            if (t1 - t0 > 2000000000ull) return false;
        }
    }
}

__device__ __forceinline__ void mma_f16(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, "
        "{%0, %1, %2, %3};"
        : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

__device__ __forceinline__ uint32_t unpack2(uint32_t word, int sel, __half2 scale) {
    const __half2_raw h =
        __nv_cvt_fp4x2_to_halfraw2((__nv_fp4x2_storage_t)((word >> (8 * sel)) & 0xffu), __NV_E2M1);
    const __half2 v = __hmul2(*reinterpret_cast<const __half2*>(&h), scale);
    return *reinterpret_cast<const uint32_t*>(&v);
}

// Eight E2M1 codes of a word -> four f16x2 (byte b holds codes 2b, 2b+1; lower code in the low half).
__device__ __forceinline__ void cvt_e2m1x8(uint32_t word, uint32_t (&h)[4]) {
    asm("{\n\t.reg .b8 b0, b1, b2, b3;\n\t"
        "mov.b32 {b0, b1, b2, b3}, %4;\n\t"
        "cvt.rn.f16x2.e2m1x2 %0, b0;\n\t"
        "cvt.rn.f16x2.e2m1x2 %1, b1;\n\t"
        "cvt.rn.f16x2.e2m1x2 %2, b2;\n\t"
        "cvt.rn.f16x2.e2m1x2 %3, b3;\n\t}"
        : "=r"(h[0]), "=r"(h[1]), "=r"(h[2]), "=r"(h[3])
        : "r"(word));
}

__device__ __forceinline__ uint32_t hmul2u(uint32_t a, __half2 s) {
    const __half2 v = __hmul2(*reinterpret_cast<const __half2*>(&a), s);
    return *reinterpret_cast<const uint32_t*>(&v);
}

__device__ __forceinline__ uint4 lds16(uint32_t addr) {
    uint4 v;
    asm volatile("ld.shared.v4.b32 {%0, %1, %2, %3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(addr));
    return v;
}

}  // namespace tg

template <int NT, bool SWIGLU>
__global__ void __launch_bounds__(TG_THREADS, 4)
gemv_nvfp4_tma_kernel(const __grid_constant__ CUtensorMap map_codes0, const __grid_constant__ CUtensorMap map_codes1,
                      const TmaGemvParams p) {
    using namespace tg;
    extern __shared__ uint8_t smem_raw[];
    const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    uint8_t* gen_base = smem_raw + (base - smem_u32(smem_raw));
    const int warp = threadIdx.x / VX_WARP, lane = threadIdx.x % VX_WARP;
    const long long k = p.k;
    const int xpitch = (int)k + TG_XPAD;
    // layout: [ring][barriers 128 B][x rows f16][token scales][partial sums]
    const uint32_t bars = base + TG_STAGES * TG_STAGE_BYTES;
    __half* xs = reinterpret_cast<__half*>(gen_base + TG_STAGES * TG_STAGE_BYTES + 128);
    float* tok_scale = reinterpret_cast<float*>(reinterpret_cast<uint8_t*>(xs) + (size_t)p.m * xpitch * 2);
    int* ticket_flag = reinterpret_cast<int*>(tok_scale + NT * 8 + TG_CONSUMERS);
    auto full_bar = [&](int s) { return bars + 8u * s; };
    auto empty_bar = [&](int s) { return bars + 8u * (TG_STAGES + s); };

    if (threadIdx.x == 0) {
        for (int s = 0; s < TG_STAGES; s++) {
            asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(full_bar(s)));
            asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(empty_bar(s)), "r"(TG_CONSUMERS));
        }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();

    const int stages_per_pass = (int)((k + 255) / 256);
    constexpr int V = SWIGLU ? 2 : 1;

    if (warp == TG_CONSUMERS) {
        // ---------------- producer ----------------
        if (lane == 0) {
            int stage = 0;
            uint32_t phase = 0;
            bool ok = true;
            for (long long item = blockIdx.x; item < p.units * p.splits && ok; item += gridDim.x) {
                const long long unit = item / p.splits;
                const int split = (int)(item % p.splits);
                const int ks_begin = (int)((long long)split * stages_per_pass / p.splits);
                const int ks_end = (int)((long long)(split + 1) * stages_per_pass / p.splits);
                for (int v = 0; v < V && ok; v++) {
                    const CUtensorMap* mc = v ? &map_codes1 : &map_codes0;
                    const long long tile128 = p.row_begin[v] / 128 + unit / 2;
                    const int row0 = (int)(tile128 * 128 + (unit % 2) * 64);
                    for (int ks = ks_begin; ks < ks_end; ks++) {
                        if (!wait(empty_bar(stage), phase ^ 1u)) {
                            atomicExch(p.status, 11);
                            ok = false;
                            break;
                        }
                        const uint32_t dst = base + stage * TG_STAGE_BYTES;
                        const int atoms = (int)min(4LL, p.k_tiles - 4LL * ks);
                        asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(full_bar(stage)),
                                     "r"((uint32_t)(TG_CODE_BOX + atoms * 512)) : "memory");
                        asm volatile(
                            "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
                            ::"r"(dst), "l"(mc), "r"(full_bar(stage)), "r"(ks * 128), "r"(row0) : "memory");
                        asm volatile(
                            "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                            ::"r"(dst + TG_CODE_BOX), "l"(p.scale_plane[v] + (tile128 * p.k_tiles + 4LL * ks) * 512),
                              "r"((uint32_t)(atoms * 512)), "r"(full_bar(stage)) : "memory");
                        if (++stage == TG_STAGES) {
                            stage = 0;
                            phase ^= 1u;
                        }
                    }
                }
            }
            if (!ok) __nanosleep(200000);
        }
    } else {
        // ---------------- consumers ----------------
        const int g = lane >> 2, t = lane & 3;
        const int rho = (g >> 1) | ((g & 1) << 2);   // chunk row read by mma row slot g

        // Stage the activations once per CTA while the producer fills the ring. All consumer threads
        // work on one token at a time, eight independent 16-byte loads each per batch, so a pass
        // costs about one memory round trip per batch; rows up to 8192 wide stay in registers
        // between the max pass and the convert pass.
        {
            const int tid = threadIdx.x;                       // 0 .. 127 (consumers only)
            const int chunks = (int)(k / 8);
            const int batches = (chunks + TG_CONSUMERS * VX_WARP * 8 - 1) / (TG_CONSUMERS * VX_WARP * 8);
            float* red_max = tok_scale + NT * 8;               // [TG_CONSUMERS]
            auto load_chunk = [&](int tk, int c8) -> uint4 {
                uint4 v = make_uint4(0, 0, 0, 0);
                if (c8 < chunks) {
                    if (p.xb) {
                        v = __ldg(reinterpret_cast<const uint4*>(p.xb + (long long)tk * k + 8LL * c8));
                    } else {
                        const float4 f0 = __ldg(reinterpret_cast<const float4*>(p.x + (long long)tk * k + 8LL * c8));
                        const float4 f1 = __ldg(reinterpret_cast<const float4*>(p.x + (long long)tk * k + 8LL * c8 + 4));
                        v.x = (uint32_t)bf16_bits(f0.x) | ((uint32_t)bf16_bits(f0.y) << 16);
                        v.y = (uint32_t)bf16_bits(f0.z) | ((uint32_t)bf16_bits(f0.w) << 16);
                        v.z = (uint32_t)bf16_bits(f1.x) | ((uint32_t)bf16_bits(f1.y) << 16);
                        v.w = (uint32_t)bf16_bits(f1.z) | ((uint32_t)bf16_bits(f1.w) << 16);
                    }
                }
                return v;
            };
            auto chunk_max = [&](const uint4& v, float m) {
                const uint32_t u[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
                for (int i = 0; i < 4; i++) {
                    m = fmaxf(m, fabsf(__uint_as_float(u[i] << 16)));
                    m = fmaxf(m, fabsf(__uint_as_float(u[i] & 0xffff0000u)));
                }
                return m;
            };
            auto store_chunk = [&](int tk, int c8, const uint4& v, float up) {
                if (c8 >= chunks) return;
                const uint32_t u[4] = {v.x, v.y, v.z, v.w};
                uint32_t o[4];
#pragma unroll
                for (int i = 0; i < 4; i++) {
                    const __half2 h = __floats2half2_rn(__uint_as_float(u[i] << 16) * up,
                                                        __uint_as_float(u[i] & 0xffff0000u) * up);
                    o[i] = *reinterpret_cast<const uint32_t*>(&h);
                }
                // k = 8 c8: inside each 128-k step the 16-byte chunk (t, i) is stored at slot i * 4 + t
                const int step = c8 >> 4, in8 = c8 & 15, tt = in8 >> 2, i4 = in8 & 3;
                *reinterpret_cast<uint4*>(xs + (size_t)tk * xpitch + step * 128 + (i4 * 4 + tt) * 8) =
                    make_uint4(o[0], o[1], o[2], o[3]);
            };
            for (int tk = 0; tk < p.m; tk++) {
                uint4 keep[8];
                float amax = 0.0f;
                for (int bt = 0; bt < batches; bt++) {
                    uint4 v[8];
#pragma unroll
                    for (int i = 0; i < 8; i++) v[i] = load_chunk(tk, (bt * 8 + i) * TG_CONSUMERS * VX_WARP + tid);
#pragma unroll
                    for (int i = 0; i < 8; i++) {
                        amax = chunk_max(v[i], amax);
                        keep[i] = v[i];
                    }
                }
                amax = warp_max(amax);
                if (lane == 0) red_max[warp] = amax;
                asm volatile("bar.sync 1, %0;" ::"r"(TG_CONSUMERS * VX_WARP) : "memory");
                amax = red_max[0];
#pragma unroll
                for (int i = 1; i < TG_CONSUMERS; i++) amax = fmaxf(amax, red_max[i]);
                asm volatile("bar.sync 1, %0;" ::"r"(TG_CONSUMERS * VX_WARP) : "memory");
                // 2^e with max|x| * 2^e in [2^14, 2^15) (give or take a rounding of log2): exact scaling
                int e = 0;
                if (amax > 0.0f && amax < 3.0e38f) e = 14 - (int)floorf(log2f(amax));
                e = max(-60, min(60, e));
                const float up = exp2f((float)e);
                if (tid == 0) tok_scale[tk] = exp2f((float)-e);
                if (batches == 1) {
#pragma unroll
                    for (int i = 0; i < 8; i++) store_chunk(tk, i * TG_CONSUMERS * VX_WARP + tid, keep[i], up);
                } else {
                    for (int bt = 0; bt < batches; bt++) {
                        uint4 v[8];
#pragma unroll
                        for (int i = 0; i < 8; i++) v[i] = load_chunk(tk, (bt * 8 + i) * TG_CONSUMERS * VX_WARP + tid);
#pragma unroll
                        for (int i = 0; i < 8; i++) store_chunk(tk, (bt * 8 + i) * TG_CONSUMERS * VX_WARP + tid, v[i], up);
                    }
                }
            }
        }
        asm volatile("bar.sync 1, %0;" ::"r"(TG_CONSUMERS * VX_WARP) : "memory");

        int stage = 0;
        uint32_t phase = 0;
        bool ok = true;
        const float div0 = *p.wdiv[0];
        const float div1 = SWIGLU ? *p.wdiv[1] : 1.0f;
        for (long long item = blockIdx.x; item < p.units * p.splits && ok; item += gridDim.x) {
            const long long unit = item / p.splits;
            const int split = (int)(item % p.splits);
            const int ks_begin = (int)((long long)split * stages_per_pass / p.splits);
            const int ks_end = (int)((long long)(split + 1) * stages_per_pass / p.splits);
            const int band0 = (int)(unit % 2) * 2;    // the unit's two bands of the 128-row tile
            float acc[V][NT][2][4];
#pragma unroll
            for (int v = 0; v < V; v++)
#pragma unroll
                for (int nt = 0; nt < NT; nt++)
#pragma unroll
                    for (int q = 0; q < 4; q++) acc[v][nt][0][q] = acc[v][nt][1][q] = 0.0f;
#pragma unroll
            for (int v = 0; v < V; v++) {
                for (int ks = ks_begin; ks < ks_end && ok; ks++) {
                    if (!wait(full_bar(stage), phase)) {
                        if (lane == 0) atomicExch(p.status, 12);
                        ok = false;
                        break;
                    }
                    const uint32_t sbase = base + stage * TG_STAGE_BYTES;
#pragma unroll
                    for (int sp = 0; sp < 2; sp++) {
                        const long long k0 = (long long)ks * 256 + sp * 128;   // this step
                        if (k0 >= k) continue;
                        const int piece = sp * 4 + t;
                        // rows of the box: band (0 = lo, 1 = hi) * 32 + chunk row 8 warp + rho
                        uint4 codes[2];
#pragma unroll
                        for (int b = 0; b < 2; b++)
                            codes[b] = lds16(sbase + (uint32_t)(b * 32 + warp * 8 + rho) * 128u + (uint32_t)((piece ^ rho) << 4));
                        // atom of k tile 2 sp + t/2 of the stage, chunk row 8 warp + rho: 4 bands x 4 groups
                        const uint4 sc = lds16(sbase + TG_CODE_BOX + (uint32_t)(2 * sp + (t >> 1)) * 512u + (uint32_t)(warp * 8 + rho) * 16u);
                        const uint32_t scw[4] = {sc.x, sc.y, sc.z, sc.w};
                        const int step = (int)(k0 >> 7);
                        uint4 xv[NT][4];
#pragma unroll
                        for (int nt = 0; nt < NT; nt++)
#pragma unroll
                            for (int i = 0; i < 4; i++)
                                xv[nt][i] = (nt * 8 + g < p.m)
                                                ? *reinterpret_cast<const uint4*>(xs + (size_t)(nt * 8 + g) * xpitch + step * 128 + (i * 4 + t) * 8)
                                                : make_uint4(0, 0, 0, 0);
                        // the lane's two groups: bytes 2*(t%2), 2*(t%2)+1 of the band's four
                        const uint32_t s_lo = (scw[band0] >> (16 * (t & 1))) & 0xffffu;
                        const uint32_t s_hi = (scw[band0 + 1] >> (16 * (t & 1))) & 0xffffu;
                        const __half2_raw slo = __nv_cvt_fp8x2_to_halfraw2((__nv_fp8x2_storage_t)s_lo, __NV_E4M3);
                        const __half2_raw shi = __nv_cvt_fp8x2_to_halfraw2((__nv_fp8x2_storage_t)s_hi, __NV_E4M3);
                        const __half2 slo2 = *reinterpret_cast<const __half2*>(&slo);
                        const __half2 shi2 = *reinterpret_cast<const __half2*>(&shi);
                        const uint32_t wl[4] = {codes[0].x, codes[0].y, codes[0].z, codes[0].w};
                        const uint32_t wh[4] = {codes[1].x, codes[1].y, codes[1].z, codes[1].w};
                        const __half2 sl0 = __low2half2(slo2), sl1 = __high2half2(slo2);
                        const __half2 sh0 = __low2half2(shi2), sh1 = __high2half2(shi2);
#pragma unroll
                        for (int wi = 0; wi < 4; wi++) {
                            // word wi = codes 8wi..8wi+7 of the lane's 32: mmas 2wi and 2wi+1; group wi/2
                            uint32_t hl[4], hh[4];
                            cvt_e2m1x8(wl[wi], hl);
                            cvt_e2m1x8(wh[wi], hh);
                            const __half2 sl = wi < 2 ? sl0 : sl1, sh = wi < 2 ? sh0 : sh1;
#pragma unroll
                            for (int q = 0; q < 4; q++) {
                                hl[q] = hmul2u(hl[q], sl);
                                hh[q] = hmul2u(hh[q], sh);
                            }
#pragma unroll
                            for (int jj = 0; jj < 2; jj++) {
                                const int j = 2 * wi + jj;
                                const uint32_t a[4] = {hl[2 * jj], hh[2 * jj], hl[2 * jj + 1], hh[2 * jj + 1]};
#pragma unroll
                                for (int nt = 0; nt < NT; nt++) {
                                    const uint4 c = xv[nt][j >> 1];
                                    const uint32_t b0 = (j & 1) ? c.z : c.x, b1 = (j & 1) ? c.w : c.y;
                                    // two accumulator chains per tile halve the dependent mma latency
                                    mma_f16(acc[v][nt][jj], a, b0, b1);
                                }
                            }
                        }
                    }
                    // the stage goes back to the TMA producer (async proxy): order this warp's
                    // generic-proxy reads of it ahead of that proxy before the arrive
                    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
                    __syncwarp();
                    if (lane == 0) asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(empty_bar(stage)) : "memory");
                    if (++stage == TG_STAGES) {
                        stage = 0;
                        phase ^= 1u;
                    }
                }
            }

            // lane (g, t): d0, d1 = chunk row rho of the lo band, tokens 2t, 2t+1; d2, d3 = the hi band
            const long long tile128 = p.row_begin[0] / 128 + unit / 2;
            bool finish = true;
            if (p.splits > 1) {
                // K-split: park this item's partial sums; the CTA that arrives last adds the splits
                // in index order (so the result does not depend on arrival order) and finishes.
                float* mine = p.partial + (size_t)item * (V * 64 * NT * 8);
#pragma unroll
                for (int v = 0; v < V; v++)
#pragma unroll
                    for (int nt = 0; nt < NT; nt++)
#pragma unroll
                        for (int q = 0; q < 4; q++)
                            mine[((v * 64 + (q >> 1) * 32 + warp * 8 + rho) * NT + nt) * 8 + 2 * t + (q & 1)] =
                                acc[v][nt][0][q] + acc[v][nt][1][q];
                __threadfence();
                asm volatile("bar.sync 1, %0;" ::"r"(TG_CONSUMERS * VX_WARP) : "memory");
                if (threadIdx.x == 0) {
                    const int prev = atomicAdd(p.tickets + unit, 1);
                    const int last = prev == p.splits - 1;
                    if (last) p.tickets[unit] = 0;     // self-cleaning for the next launch
                    *ticket_flag = last;
                }
                asm volatile("bar.sync 1, %0;" ::"r"(TG_CONSUMERS * VX_WARP) : "memory");
                finish = *ticket_flag != 0;
                if (finish) {
                    __threadfence();
                    const float* first = p.partial + (size_t)(unit * p.splits) * (V * 64 * NT * 8);
#pragma unroll
                    for (int v = 0; v < V; v++)
#pragma unroll
                        for (int nt = 0; nt < NT; nt++)
#pragma unroll
                            for (int q = 0; q < 4; q++) {
                                const int idx = ((v * 64 + (q >> 1) * 32 + warp * 8 + rho) * NT + nt) * 8 + 2 * t + (q & 1);
                                float sum = 0.0f;
                                for (int sp = 0; sp < p.splits; sp++)
                                    sum += __ldcg(first + (size_t)sp * (V * 64 * NT * 8) + idx);
                                acc[v][nt][0][q] = sum;
                                acc[v][nt][1][q] = 0.0f;
                            }
                }
                asm volatile("bar.sync 1, %0;" ::"r"(TG_CONSUMERS * VX_WARP) : "memory");
            }
            if (finish) {
#pragma unroll
            for (int nt = 0; nt < NT; nt++)
#pragma unroll
                for (int q = 0; q < 4; q++) {
                    const int tok = nt * 8 + 2 * t + (q & 1);
                    const long long r0 = tile128 * 128 + (band0 + (q >> 1)) * 32 + warp * 8 + rho;
                    if (tok >= p.m || r0 < p.row_begin[0] || r0 >= p.row_begin[0] + p.rows) continue;
                    float val = (acc[0][nt][0][q] + acc[0][nt][1][q]) * tok_scale[tok] / div0;
                    if (SWIGLU) {
                        const float u = (acc[V - 1][nt][0][q] + acc[V - 1][nt][1][q]) * tok_scale[tok] / div1;
                        val = val / (1.0f + expf(-val)) * u;
                    }
                    const long long o = (long long)tok * p.ld + p.col + (r0 - p.row_begin[0]);
                    if (p.y) p.y[o] = val;
                    if (p.yb) p.yb[o] = bf16_bits(val);
                }
            }
        }
    }
    __syncthreads();
}

// ---- host side ------------------------------------------------------------------------------------------

typedef CUresult (*EncodeTiledFn2)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                   const cuuint64_t*, const cuuint32_t*, const cuuint32_t*,
                                   CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion,
                                   CUtensorMapFloatOOBfill);

static EncodeTiledFn2 gemv_encode_fn() {
    static EncodeTiledFn2 fn = []() -> EncodeTiledFn2 {
        void* f = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &f, cudaEnableDefault, &q) != cudaSuccess ||
            q != cudaDriverEntryPointSuccess) {
            cudaGetLastError();
            return nullptr;
        }
        return reinterpret_cast<EncodeTiledFn2>(f);
    }();
    return fn;
}

// Codes of a parent [n, k] as a [n, k/2]-byte matrix, box 128 B x 64 rows, 128-byte swizzle.
static int make_gemv_map(const velox_sm100_view& v, CUtensorMap* codes) {
    const long long kb = v.k / 2;
    const cuuint64_t dims[2] = {(cuuint64_t)kb, (cuuint64_t)v.n};
    const cuuint64_t strides[1] = {(cuuint64_t)kb};
    const cuuint32_t box[2] = {128, 64};
    const cuuint32_t es[2] = {1, 1};
    if (gemv_encode_fn()(codes, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<uint8_t*>(v.w), dims, strides, box, es,
                         CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                         CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
        return VELOX_ERR_UNSUPPORTED;
    return 0;
}

template <int NT, bool SWIGLU>
static int launch_tma_gemv(const CUtensorMap (&maps)[2], const TmaGemvParams& p) {
    static int sms = 0;
    if (sms == 0) {
        int dev = 0;
        cudaGetDevice(&dev);
        cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
        if (sms <= 0) sms = 148;
    }
    const size_t smem = 1024 + (size_t)TG_STAGES * TG_STAGE_BYTES + 128 + (size_t)p.m * (p.k + TG_XPAD) * 2 +
                        (size_t)NT * 8 * 4 + TG_CONSUMERS * 4 + 16;
    if (smem > 220 * 1024) return VELOX_ERR_UNSUPPORTED;
    const int per_sm = smem <= 56 * 1024 ? 4 : smem <= 74 * 1024 ? 3 : smem <= 112 * 1024 ? 2 : 1;
    const long long items = p.units * p.splits;
    const long long blocks = items < (long long)per_sm * sms ? items : (long long)per_sm * sms;
    auto kern = gemv_nvfp4_tma_kernel<NT, SWIGLU>;
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return (int)e;
    TimedRegion timed(TIMED_GEMV);
    kern<<<(unsigned)blocks, TG_THREADS, smem, stream()>>>(maps[0], maps[1], p);
    return launch_status();
}

static std::mutex g_gemv_mu;
static int* gemv_status_ptr() {
    static int* ptrs[64] = {};
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return nullptr;
    std::lock_guard<std::mutex> lock(g_gemv_mu);
    if (!ptrs[dev]) cudaGetSymbolAddress(reinterpret_cast<void**>(&ptrs[dev]), g_gemv_status);
    return ptrs[dev];
}

// Arrival counters of the K-split fix-up: zeroed when (re)allocated, returned to zero by the kernel.
// One array per device, shared by every launch: launches on a device must be stream-ordered.
static int* g_gemv_ticket_ptrs[64] = {};
static size_t g_gemv_ticket_caps[64] = {};
static int* gemv_tickets(size_t count) {
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return nullptr;
    std::lock_guard<std::mutex> lock(g_gemv_mu);
    if (count > g_gemv_ticket_caps[dev]) {
        const size_t n = count < 4096 ? 4096 : count * 2;
        int* q = nullptr;
        if (cudaMalloc(&q, n * sizeof(int)) != cudaSuccess) {
            cudaGetLastError();
            return nullptr;
        }
        if (cudaMemsetAsync(q, 0, n * sizeof(int), stream()) != cudaSuccess) return nullptr;
        g_gemv_ticket_ptrs[dev] = q;   // the old block stays allocated: queued work may still use it
        g_gemv_ticket_caps[dev] = n;
    }
    return g_gemv_ticket_ptrs[dev];
}

// Clears the status word and the arrival counters (a launch that gave up leaves them non-zero).
// The caller has synchronised the device.
int gemv_status_reset() {
    const int zero = 0;
    cudaError_t e = cudaMemcpyToSymbol(g_gemv_status, &zero, sizeof(int));
    if (e != cudaSuccess) return (int)e;
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 0;
    std::lock_guard<std::mutex> lock(g_gemv_mu);
    if (g_gemv_ticket_ptrs[dev])
        e = cudaMemset(g_gemv_ticket_ptrs[dev], 0, g_gemv_ticket_caps[dev] * sizeof(int));
    return (int)e;
}

int gemv_status_sync() {
    int v = -1;
    if (cudaMemcpyFromSymbol(&v, g_gemv_status, sizeof(int)) != cudaSuccess) return -1;
    return v;
}

// NVFP4, m <= 16, k a multiple of 128; the SwiGLU form also needs gate and up at the same offset
// inside a 128-row tile.
int gemv_nvfp4_tma(const LinearArgs& a) {
    if (a.w.format != VELOX_FMT_NVFP4 || a.m < 1 || a.m > 16) return VELOX_ERR_UNSUPPORTED;
    if (a.w.k % 128 != 0 || !gemv_encode_fn()) return VELOX_ERR_UNSUPPORTED;
    if (a.swiglu && (a.w.row_begin - a.up.row_begin) % 128 != 0) return VELOX_ERR_UNSUPPORTED;
    if (a.xb && (reinterpret_cast<uintptr_t>(a.xb) & 15)) return VELOX_ERR_UNSUPPORTED;
    if (a.x && (reinterpret_cast<uintptr_t>(a.x) & 15)) return VELOX_ERR_UNSUPPORTED;
    if (reinterpret_cast<uintptr_t>(a.w.w) & 15) return VELOX_ERR_UNSUPPORTED;
    CUtensorMap maps[2];
    int rc = make_gemv_map(a.w, &maps[0]);
    if (rc != 0) return rc;
    rc = make_gemv_map(a.swiglu ? a.up : a.w, &maps[1]);
    if (rc != 0) return rc;
    TmaGemvParams p{};
    const velox_sm100_view& u = a.swiglu ? a.up : a.w;
    p.k = a.w.k;
    p.row_begin[0] = a.w.row_begin;
    p.row_begin[1] = u.row_begin;
    p.rows = a.w.rows;
    p.k_tiles = a.w.k / 64;
    p.scale_plane[0] = a.w.w + align256(a.w.n * a.w.k / 2);
    p.scale_plane[1] = u.w + align256(u.n * u.k / 2);
    p.wdiv[0] = reinterpret_cast<const float*>(a.w.w + align256(a.w.n * a.w.k / 2) + a.w.n * a.w.k / 16);
    p.wdiv[1] = reinterpret_cast<const float*>(u.w + align256(u.n * u.k / 2) + u.n * u.k / 16);
    p.x = a.x; p.xb = a.xb; p.m = a.m; p.y = a.y; p.yb = a.yb; p.ld = a.ld; p.col = a.col;
    p.units = ((a.w.row_begin + a.w.rows - 1) / 128 - a.w.row_begin / 128 + 1) * 2;
    // K splits: enough work items to give every SM about two, each split at least four stages long
    {
        const long long stages = (a.w.k + 255) / 256;
        long long want = (2LL * 148 + p.units - 1) / p.units;
        if (want > stages / 4) want = stages / 4;
        if (want < 1) want = 1;
        if (want > 16) want = 16;
        p.splits = (int)want;
        if (p.splits > 1) {
            const size_t per_item = (size_t)(a.swiglu ? 2 : 1) * 64 * (a.m <= 8 ? 8 : 16) * sizeof(float);
            p.partial = static_cast<float*>(scratch(SCRATCH_Y_F32, (size_t)p.units * p.splits * per_item));
            p.tickets = gemv_tickets((size_t)p.units);
            if (!p.partial || !p.tickets) return (int)cudaErrorMemoryAllocation;
        }
    }
    p.status = gemv_status_ptr();
    if (!p.status) return VELOX_ERR_UNSUPPORTED;
    if (a.m <= 8) return a.swiglu ? launch_tma_gemv<1, true>(maps, p) : launch_tma_gemv<1, false>(maps, p);
    return a.swiglu ? launch_tma_gemv<2, true>(maps, p) : launch_tma_gemv<2, false>(maps, p);
}

}  // namespace vx
