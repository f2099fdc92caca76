// Prefill GEMM on the 5th-generation tensor cores: y[m, rows] = x[m, k] . W^T for m > 16.
//
// One persistent CTA per SM walks output tiles of 128 tokens x 256 weight rows. Three roles:
//   warp 0      TMA producer: cp.async.bulk.tensor tiles of x and W (128-byte swizzled rows) and,
//               for NVFP4, whole 512-byte scale atoms, into a 4-stage shared-memory ring;
//   warp 1      MMA issuer: one elected thread issues tcgen05.mma with the accumulator in tensor
//               memory (128 lanes x 256 f32 columns); for NVFP4 it first copies the scale atoms
//               shared memory -> tensor memory (tcgen05.cp) and issues the block-scaled
//               kind::mxf4nvf4 form, for FP8 kind::f8f6f4, for bf16 kind::f16;
//   warps 2-5   epilogue: tcgen05.ld the accumulator, apply the per-tensor / per-row / per-token
//               factors, optionally silu(gate)*up, write f32 and/or bf16.
// Tokens are the MMA M operand and weight rows the N operand, so a lane of the epilogue owns one
// token and writes contiguous output columns. The stored NVFP4 layout is consumed as is: codes are
// K-major with the lower k in the low nibble, and the 128-row x 4-group scale tiles
// (crates/velox-core/src/format.rs:345-354) are exactly the 32-lane x 16-byte block the
// tcgen05.cp.32x128b.warpx4 copy expects, for weights (payload) and activations (quantiser
// output) alike. Row views are tiled on parent-row coordinates rounded down to a scale tile and
// masked in the epilogue.
//
// Every wait on an mbarrier is bounded: after about two seconds a role records a code in the
// status word, stops, and the CTA still frees its tensor memory and exits normally.
//
// No TMA load here uses cluster multicast; each CTA fetches its own tiles.
//
// Reference counterpart (SIMT f32): linear_tiled_kernel, crates/velox-cuda/kernels/portable_model.cu:349-398.
#include <cuda.h>  // CUtensorMap types; the encode entry point is resolved at run time

#include "common.cuh"
#include "gemm.cuh"

namespace vx {

enum GemmKind { KIND_MXF4 = 0, KIND_F8 = 1, KIND_BF16 = 2 };

constexpr int BM = 128;        // tokens per tile (MMA M)
constexpr int BN = 256;        // weight rows per tile (MMA N): two 128-row halves
constexpr int BK_BYTES = 128;  // bytes of K per row per stage: one swizzle row, four MMA k-steps
constexpr int STAGES = 4;
constexpr int A_BYTES = BM * BK_BYTES;
constexpr int B_HALF_BYTES = 128 * BK_BYTES;
constexpr int B_BYTES = 2 * B_HALF_BYTES;
constexpr int SFA_BYTES = 4 * 512;
constexpr int SFB_BYTES = 2 * 4 * 512;
constexpr int STAGE_BYTES = A_BYTES + B_BYTES + SFA_BYTES + SFB_BYTES;
constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + 1024 + 256;
constexpr int TMEM_COLS = 512;
constexpr int TMEM_SFA_COL = 256;  // 4 k-steps x 4 columns
constexpr int TMEM_SFB_COL = 272;  // 4 k-steps x 8 columns
constexpr int GEMM_THREADS = 192;

enum { ST_OK = 0, ST_TIMEOUT_EMPTY = 1, ST_TIMEOUT_FULL = 2, ST_TIMEOUT_ACC_EMPTY = 3,
       ST_TIMEOUT_ACC_FULL = 4 };

struct GemmParams {
    int m;
    int k_blocks;       // ceil(k_steps / 4)
    int k_steps;        // 32-byte MMA k-steps in a row
    int k_elems_per_block;  // tensor-map elements per 128-byte block (128 for byte maps, 64 bf16)
    int a_k_blocks;         // the activation operand wraps around after this many blocks
    int tiles_m, tiles_n;
    long long b_row0[2];       // first row (tensor-map coordinates) of n-tile 0, per half
    int b_tile_rows;           // rows advanced per n-tile
    long long b_rows_total[2]; // rows the half's tensor map / scale plane holds
    long long valid_begin[2], valid_end[2];  // rows of each half that belong to the view
    long long out_row0;        // row (half-0 coordinates) that maps to output column `col`
    const uint8_t* sfa;
    const uint8_t* sfb[2];
    int k_tiles64;
    float alpha;
    const float* wdiv[2];
    const float* tok_scale;
    const uint16_t* col_scale[2];  // bf16 per row, indexed by the half's row coordinate
    float* y;
    uint16_t* yb;
    long long ld, col;
    int* status;
};

__device__ int g_gemm_status = 0;

// ---- PTX wrappers ----------------------------------------------------------------------------------

__device__ __forceinline__ uint32_t smem_u32(const void* p) {
    return (uint32_t)__cvta_generic_to_shared(p);
}

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count));
}

__device__ __forceinline__ void mbar_arrive_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes)
                 : "memory");
}

__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}

__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.b32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(bar), "r"(parity)
        : "memory");
    return ok != 0;
}

__device__ __forceinline__ unsigned long long global_timer_ns() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
    return t;
}

// Bounded wait: false after ~2 s without the phase completing.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity) {
    if (mbar_try_wait(bar, parity)) return true;
    const unsigned long long t0 = global_timer_ns();
    for (uint32_t spins = 1;; spins++) {
        if (mbar_try_wait(bar, parity)) return true;
        if ((spins & 255u) == 0 && global_timer_ns() - t0 > 2000000000ull) return false;
    }
}

__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap* map, uint32_t bar,
                                            int x, int y) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
        ::"r"(dst), "l"(map), "r"(bar), "r"(x), "r"(y)
        : "memory");
}

__device__ __forceinline__ void bulk_load_1d(uint32_t dst, const void* src, uint32_t bytes,
                                             uint32_t bar) {
    asm volatile(
        "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
        ::"r"(dst), "l"(src), "r"(bytes), "r"(bar)
        : "memory");
}

__device__ __forceinline__ void tc_fence_before() {
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void tc_fence_after() {
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
}

__device__ __forceinline__ void tc_commit(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar)
                 : "memory");
}

// Shared-memory matrix descriptor, K-major. 128-byte swizzle: rows of 128 bytes, groups of eight
// rows 1024 bytes apart. No swizzle (scale atoms): 16-byte rows, groups of eight 128 bytes apart.
__device__ __forceinline__ uint64_t smem_desc_sw128(uint32_t addr) {
    return (uint64_t)((addr >> 4) & 0x3fffu) | ((uint64_t)1 << 16) | ((uint64_t)(1024 >> 4) << 32) |
           ((uint64_t)1 << 46) | ((uint64_t)2 << 61);
}
__device__ __forceinline__ uint64_t smem_desc_sf(uint32_t addr) {
    return (uint64_t)((addr >> 4) & 0x3fffu) | ((uint64_t)(128 >> 4) << 32) | ((uint64_t)1 << 46);
}

__device__ __forceinline__ void tc_cp_sf(uint32_t tmem_col_addr, uint64_t desc) {
    asm volatile("tcgen05.cp.cta_group::1.32x128b.warpx4 [%0], %1;" ::"r"(tmem_col_addr), "l"(desc)
                 : "memory");
}

template <int KIND>
__device__ __forceinline__ void tc_mma(uint32_t d, uint64_t a, uint64_t b, uint32_t idesc,
                                       uint32_t accumulate, uint32_t sfa, uint32_t sfb) {
    if (KIND == KIND_MXF4) {
        asm volatile(
            "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
            "tcgen05.mma.cta_group::1.kind::mxf4nvf4.block_scale.block16 [%0], %1, %2, %3, [%5], [%6], p;\n\t}"
            ::"r"(d), "l"(a), "l"(b), "r"(idesc), "r"(accumulate), "r"(sfa), "r"(sfb)
            : "memory");
    } else if (KIND == KIND_F8) {
        asm volatile(
            "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
            "tcgen05.mma.cta_group::1.kind::f8f6f4 [%0], %1, %2, %3, p;\n\t}"
            ::"r"(d), "l"(a), "l"(b), "r"(idesc), "r"(accumulate)
            : "memory");
    } else {
        asm volatile(
            "{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\t"
            "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
            ::"r"(d), "l"(a), "l"(b), "r"(idesc), "r"(accumulate)
            : "memory");
    }
}

// 32 lanes x 32 consecutive f32 columns of the accumulator.
__device__ __forceinline__ void tc_ld32(uint32_t taddr, uint32_t (&r)[32]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
        "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]),
          "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]),
          "=r"(r[14]), "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]),
          "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]),
          "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(taddr));
}
__device__ __forceinline__ void tc_wait_ld() {
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}

// Instruction descriptor: M = 128, N = 256, K-major operands, f32 accumulate.
template <int KIND>
__device__ __forceinline__ constexpr uint32_t instr_desc() {
    const uint32_t n = (uint32_t)(BN >> 3) << 17, m = (uint32_t)(BM >> 4) << 24;
    if (KIND == KIND_MXF4) return (1u << 7) | (1u << 10) | n | m;         // E2M1 x E2M1, UE4M3 scales
    if (KIND == KIND_F8) return (1u << 4) | n | m;                        // E4M3 x E4M3 -> f32
    return (1u << 4) | (1u << 7) | (1u << 10) | n | m;                    // BF16 x BF16 -> f32
}

// ---- kernel ------------------------------------------------------------------------------------------

template <int KIND, bool SWIGLU>
__global__ void __launch_bounds__(GEMM_THREADS, 1)
gemm_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b0,
            const __grid_constant__ CUtensorMap tmap_b1, const GemmParams p) {
    extern __shared__ uint8_t smem_raw[];
    const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    const uint32_t bars = base + STAGES * STAGE_BYTES;
    auto full_bar = [&](int s) { return bars + 8u * s; };
    auto empty_bar = [&](int s) { return bars + 8u * (STAGES + s); };
    const uint32_t acc_full = bars + 8u * (2 * STAGES);
    const uint32_t acc_empty = bars + 8u * (2 * STAGES + 1);
    const uint32_t tmem_slot = bars + 8u * (2 * STAGES + 2);
    uint32_t* tmem_slot_ptr = reinterpret_cast<uint32_t*>(smem_raw + (tmem_slot - smem_u32(smem_raw)));

    const int warp = threadIdx.x / 32, lane = threadIdx.x % 32;

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; s++) {
            mbar_init(full_bar(s), 1);
            mbar_init(empty_bar(s), 1);
        }
        mbar_init(acc_full, 1);
        mbar_init(acc_empty, 4);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("prefetch.tensormap [%0];" ::"l"(&tmap_a) : "memory");
        asm volatile("prefetch.tensormap [%0];" ::"l"(&tmap_b0) : "memory");
        asm volatile("prefetch.tensormap [%0];" ::"l"(&tmap_b1) : "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(tmem_slot),
                     "r"((uint32_t)TMEM_COLS)
                     : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = *tmem_slot_ptr;

    const int num_tiles = p.tiles_m * p.tiles_n;

    if (warp == 0) {
        // ---------------- TMA producer ----------------
        if (lane == 0) {
            int stage = 0;
            uint32_t phase = 0;
            bool ok = true;
            for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x) {
                const int mt = tile % p.tiles_m, nt = tile / p.tiles_m;
                const long long r0 = p.b_row0[0] + (long long)nt * p.b_tile_rows;
                const long long r1 = p.b_row0[1] + (long long)nt * p.b_tile_rows;
                for (int kb = 0; kb < p.k_blocks; kb++) {
                    if (!mbar_wait(empty_bar(stage), phase ^ 1u)) {
                        atomicExch(p.status, ST_TIMEOUT_EMPTY);
                        ok = false;
                        break;
                    }
                    const int steps = min(4, p.k_steps - 4 * kb);
                    const uint32_t sa = base + stage * STAGE_BYTES;
                    const uint32_t sb = sa + A_BYTES;
                    uint32_t tx = A_BYTES + B_BYTES;
                    const bool sf0 = KIND == KIND_MXF4 && r0 < p.b_rows_total[0];
                    const bool sf1 = KIND == KIND_MXF4 && r1 < p.b_rows_total[1];
                    if (KIND == KIND_MXF4) tx += (uint32_t)steps * 512u * (1u + (sf0 ? 1u : 0u) + (sf1 ? 1u : 0u));
                    mbar_arrive_expect_tx(full_bar(stage), tx);
                    tma_load_2d(sa, &tmap_a, full_bar(stage), (kb % p.a_k_blocks) * p.k_elems_per_block, mt * BM);
                    tma_load_2d(sb, &tmap_b0, full_bar(stage), kx, (int)r0);
                    tma_load_2d(sb + B_HALF_BYTES, &tmap_b1, full_bar(stage), kx, (int)r1);
                    if (KIND == KIND_MXF4) {
                        const uint32_t ssfa = sb + B_BYTES, ssfb = ssfa + SFA_BYTES;
                        const long long atom = 4LL * kb;
                        bulk_load_1d(ssfa, p.sfa + ((long long)mt * p.k_tiles64 + atom) * 512,
                                     (uint32_t)steps * 512u, full_bar(stage));
                        if (sf0)
                            bulk_load_1d(ssfb, p.sfb[0] + ((r0 / 128) * p.k_tiles64 + atom) * 512,
                                         (uint32_t)steps * 512u, full_bar(stage));
                        if (sf1)
                            bulk_load_1d(ssfb + 4 * 512, p.sfb[1] + ((r1 / 128) * p.k_tiles64 + atom) * 512,
                                         (uint32_t)steps * 512u, full_bar(stage));
                    }
                    if (++stage == STAGES) {
                        stage = 0;
                        phase ^= 1u;
                    }
                }
            }
            if (!ok) __nanosleep(200000);  // let copies already in flight land before the CTA exits
        }
    } else if (warp == 1) {
        // ---------------- MMA issuer ----------------
        if (lane == 0) {
            int stage = 0;
            uint32_t phase = 0, acc_phase = 0;
            bool ok = true;
            const uint32_t idesc = instr_desc<KIND>();
            for (int tile = blockIdx.x; tile < num_tiles && ok; tile += gridDim.x) {
                if (!mbar_wait(acc_empty, acc_phase ^ 1u)) {
                    atomicExch(p.status, ST_TIMEOUT_ACC_EMPTY);
                    break;
                }
                tc_fence_after();
                for (int kb = 0; kb < p.k_blocks; kb++) {
                    if (!mbar_wait(full_bar(stage), phase)) {
                        atomicExch(p.status, ST_TIMEOUT_FULL);
                        ok = false;
                        break;
                    }
                    tc_fence_after();
                    const int steps = min(4, p.k_steps - 4 * kb);
                    const uint32_t sa = base + stage * STAGE_BYTES;
                    const uint32_t sb = sa + A_BYTES;
                    if (KIND == KIND_MXF4) {
                        const uint32_t ssfa = sb + B_BYTES, ssfb = ssfa + SFA_BYTES;
                        for (int j = 0; j < steps; j++) {
                            tc_cp_sf(tmem + TMEM_SFA_COL + 4 * j, smem_desc_sf(ssfa + 512 * j));
                            tc_cp_sf(tmem + TMEM_SFB_COL + 8 * j, smem_desc_sf(ssfb + 512 * j));
                            tc_cp_sf(tmem + TMEM_SFB_COL + 8 * j + 4, smem_desc_sf(ssfb + 4 * 512 + 512 * j));
                        }
                    }
                    const uint64_t da = smem_desc_sw128(sa), db = smem_desc_sw128(sb);
                    for (int j = 0; j < steps; j++) {
                        // advancing 32 bytes along K inside the swizzle row: +2 in the address field
                        tc_mma<KIND>(tmem, da + 2u * j, db + 2u * j, idesc, (kb | j) != 0 ? 1u : 0u,
                                     tmem + TMEM_SFA_COL + 4 * j, tmem + TMEM_SFB_COL + 8 * j);
                    }
                    tc_commit(empty_bar(stage));
                    if (++stage == STAGES) {
                        stage = 0;
                        phase ^= 1u;
                    }
                }
                if (ok) tc_commit(acc_full);
                acc_phase ^= 1u;
            }
        }
    } else {
        // ---------------- epilogue ----------------
        const int quad = warp % 4;
        uint32_t acc_phase = 0;
        const float d0 = p.wdiv[0] ? *p.wdiv[0] : 1.0f;
        const float d1 = p.wdiv[1] ? *p.wdiv[1] : 1.0f;
        const float s_half[2] = {p.alpha / d0, p.alpha / d1};
        for (int tile = blockIdx.x; tile < num_tiles; tile += gridDim.x) {
            const int mt = tile % p.tiles_m, nt = tile / p.tiles_m;
            if (!mbar_wait(acc_full, acc_phase)) {
                if (lane == 0) atomicExch(p.status, ST_TIMEOUT_ACC_FULL);
                break;
            }
            tc_fence_after();
            const long long token = (long long)mt * BM + quad * 32 + lane;
            const bool tok_ok = token < p.m;
            const float ts = (p.tok_scale && tok_ok) ? p.tok_scale[token] : 1.0f;
            const uint32_t taddr = tmem + ((uint32_t)(quad * 32) << 16);
            const long long rbase[2] = {p.b_row0[0] + (long long)nt * p.b_tile_rows,
                                        p.b_row0[1] + (long long)nt * p.b_tile_rows};
            constexpr int CHUNKS = SWIGLU ? 4 : 8;
            for (int ch = 0; ch < CHUNKS; ch++) {
                uint32_t r[32], r2[32];
                tc_ld32(taddr + ch * 32, r);
                if (SWIGLU) tc_ld32(taddr + 128 + ch * 32, r2);
                tc_wait_ld();
                const int half = SWIGLU ? 0 : ch / 4;
                const long long row0 = rbase[half] + (ch % 4) * 32;   // first row of this chunk
                const long long urow0 = rbase[1] + ch * 32;           // SwiGLU: matching up rows
                float v[32];
#pragma unroll
                for (int c = 0; c < 32; c++) {
                    float g = __uint_as_float(r[c]) * s_half[half] * ts;
                    if (p.col_scale[half]) {
                        const long long rr = row0 + c;
                        g *= (rr < p.b_rows_total[half]) ? bf16_bits_to_f32(p.col_scale[half][rr]) : 0.0f;
                    }
                    if (SWIGLU) {
                        float u = __uint_as_float(r2[c]) * s_half[1] * ts;
                        if (p.col_scale[1]) {
                            const long long rr = urow0 + c;
                            u *= (rr < p.b_rows_total[1]) ? bf16_bits_to_f32(p.col_scale[1][rr]) : 0.0f;
                        }
                        g = g / (1.0f + expf(-g)) * u;
                    }
                    v[c] = g;
                }
                if (tok_ok) {
                    const long long o0 = token * p.ld + p.col + (row0 - p.out_row0);
                    const bool all = row0 >= p.valid_begin[half] && row0 + 32 <= p.valid_end[half];
                    if (all && p.yb && ((reinterpret_cast<uintptr_t>(p.yb + o0) & 15) == 0)) {
#pragma unroll
                        for (int q = 0; q < 4; q++) {
                            uint4 pk;
                            pk.x = (uint32_t)bf16_bits(v[8 * q]) | ((uint32_t)bf16_bits(v[8 * q + 1]) << 16);
                            pk.y = (uint32_t)bf16_bits(v[8 * q + 2]) | ((uint32_t)bf16_bits(v[8 * q + 3]) << 16);
                            pk.z = (uint32_t)bf16_bits(v[8 * q + 4]) | ((uint32_t)bf16_bits(v[8 * q + 5]) << 16);
                            pk.w = (uint32_t)bf16_bits(v[8 * q + 6]) | ((uint32_t)bf16_bits(v[8 * q + 7]) << 16);
                            *reinterpret_cast<uint4*>(p.yb + o0 + 8 * q) = pk;
                        }
                    } else if (p.yb) {
#pragma unroll
                        for (int c = 0; c < 32; c++)
                            if (row0 + c >= p.valid_begin[half] && row0 + c < p.valid_end[half])
                                p.yb[o0 + c] = bf16_bits(v[c]);
                    }
                    if (all && p.y && ((reinterpret_cast<uintptr_t>(p.y + o0) & 15) == 0)) {
#pragma unroll
                        for (int q = 0; q < 8; q++)
                            *reinterpret_cast<float4*>(p.y + o0 + 4 * q) =
                                make_float4(v[4 * q], v[4 * q + 1], v[4 * q + 2], v[4 * q + 3]);
                    } else if (p.y) {
#pragma unroll
                        for (int c = 0; c < 32; c++)
                            if (row0 + c >= p.valid_begin[half] && row0 + c < p.valid_end[half])
                                p.y[o0 + c] = v[c];
                    }
                }
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(acc_empty);
            acc_phase ^= 1u;
        }
    }

    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"((uint32_t)TMEM_COLS)
                     : "memory");
    }
}

// ---- host side -------------------------------------------------------------------------------------------

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*,
                                  CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion,
                                  CUtensorMapFloatOOBfill);

static EncodeTiledFn encode_fn() {
    static EncodeTiledFn fn = []() -> EncodeTiledFn {
        void* f = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &f, cudaEnableDefault, &q) != cudaSuccess ||
            q != cudaDriverEntryPointSuccess) {
            cudaGetLastError();
            return nullptr;
        }
        return reinterpret_cast<EncodeTiledFn>(f);
    }();
    return fn;
}

bool gemm_available() {
    static int ok = -1;
    if (ok < 0) {
        int dev = 0, major = 0;
        ok = 0;
        if (cudaGetDevice(&dev) == cudaSuccess &&
            cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, dev) == cudaSuccess &&
            major == 10 && encode_fn() != nullptr)
            ok = 1;
        cudaGetLastError();
    }
    return ok == 1;
}

// 2-D row-major tensor map [rows, row_elems], box = 128 bytes x 128 rows, 128-byte swizzle.
static int make_map(CUtensorMap* map, const void* ptr, bool bf16, long long rows, long long row_elems) {
    const cuuint64_t dims[2] = {(cuuint64_t)row_elems, (cuuint64_t)rows};
    const cuuint64_t strides[1] = {(cuuint64_t)row_elems * (bf16 ? 2 : 1)};
    const cuuint32_t box[2] = {bf16 ? 64u : 128u, 128u};
    const cuuint32_t estr[2] = {1, 1};
    CUresult r = encode_fn()(map, bf16 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16 : CU_TENSOR_MAP_DATA_TYPE_UINT8, 2,
                             const_cast<void*>(ptr), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                             CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                             CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r == CUDA_SUCCESS ? 0 : VELOX_ERR_UNSUPPORTED;
}

template <int KIND>
static int launch(bool swiglu, const CUtensorMap& a, const CUtensorMap& b0, const CUtensorMap& b1,
                  const GemmParams& p) {
    static int sms = 0;
    if (sms == 0) {
        int dev = 0;
        cudaGetDevice(&dev);
        cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
        if (sms <= 0) sms = 148;
    }
    const int tiles = p.tiles_m * p.tiles_n;
    const int grid = tiles < sms ? tiles : sms;
    cudaError_t e;
    if (swiglu) {
        auto kern = gemm_kernel<KIND, true>;
        e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES);
        if (e != cudaSuccess) return (int)e;
        kern<<<grid, GEMM_THREADS, SMEM_BYTES, stream()>>>(a, b0, b1, p);
    } else {
        auto kern = gemm_kernel<KIND, false>;
        e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES);
        if (e != cudaSuccess) return (int)e;
        kern<<<grid, GEMM_THREADS, SMEM_BYTES, stream()>>>(a, b0, b1, p);
    }
    return launch_status();
}

static int* status_ptr() {
    static int* ptr = nullptr;
    if (!ptr) cudaGetSymbolAddress(reinterpret_cast<void**>(&ptr), g_gemm_status);
    return ptr;
}

int gemm_status_sync() {
    int v = -1;
    if (cudaMemcpyFromSymbol(&v, g_gemm_status, sizeof(int)) != cudaSuccess) return -1;
    return v;
}

int gemm_linear(const LinearArgs& a, int act, float divisor) {
    if (!gemm_available()) return VELOX_ERR_UNSUPPORTED;
    const velox_sm100_view& w = a.w;
    const long long k = w.k;
    if (k % 64 != 0 || a.m < 1) return VELOX_ERR_UNSUPPORTED;
    const bool sw = a.swiglu != 0;
    const velox_sm100_view& w1 = sw ? a.up : a.w;

    GemmParams p{};
    p.m = a.m;
    p.tiles_m = (a.m + BM - 1) / BM;
    p.y = a.y;
    p.yb = a.yb;
    p.ld = a.ld;
    p.col = a.col;
    p.status = status_ptr();
    p.alpha = 1.0f;
    if (!p.status) return VELOX_ERR_UNSUPPORTED;

    CUtensorMap ma, mb0, mb1;
    int rc;

    if (act == VELOX_ACT_NVFP4) {
        if (w.format != VELOX_FMT_NVFP4) return VELOX_ERR_UNSUPPORTED;
        if (sw && (w.row_begin - w1.row_begin) % 128 != 0) return VELOX_ERR_UNSUPPORTED;
        const int mp = p.tiles_m * BM;
        uint8_t* codes = static_cast<uint8_t*>(scratch(SCRATCH_ACT_CODES, (size_t)a.m * k / 2));
        uint8_t* atoms = static_cast<uint8_t*>(scratch(SCRATCH_ACT_SCALES, (size_t)mp * k / 16));
        if (!codes || !atoms) return (int)cudaErrorMemoryAllocation;
        rc = quantize_act_nvfp4(a.x, a.xb, a.m, k, divisor, codes, atoms);
        if (rc != 0) return rc;
        p.k_steps = (int)(k / 64);
        p.k_elems_per_block = 128;
        p.k_tiles64 = (int)(k / 64);
        p.sfa = atoms;
        p.alpha = 1.0f / divisor;
        const velox_sm100_view* hv[2] = {&w, &w1};
        for (int h = 0; h < 2; h++) {
            const velox_sm100_view& v = *hv[h];
            const long long plane = align256(v.n * k / 2);
            p.sfb[h] = v.w + plane;
            p.wdiv[h] = reinterpret_cast<const float*>(v.w + plane + v.n * k / 16);
            p.b_rows_total[h] = v.n;
            p.valid_begin[h] = v.row_begin;
            p.valid_end[h] = v.row_begin + v.rows;
        }
        const long long base0 = w.row_begin / 128 * 128;
        if (sw) {
            p.b_row0[0] = base0;
            p.b_row0[1] = w1.row_begin - (w.row_begin - base0);
            p.b_tile_rows = 128;
            p.tiles_n = (int)((w.row_begin + w.rows - base0 + 127) / 128);
        } else {
            p.b_row0[0] = base0;
            p.b_row0[1] = base0 + 128;
            p.b_tile_rows = 256;
            p.tiles_n = (int)((w.row_begin + w.rows - base0 + 255) / 256);
        }
        p.out_row0 = w.row_begin;
        if ((rc = make_map(&ma, codes, false, a.m, k / 2)) != 0) return rc;
        if ((rc = make_map(&mb0, w.w, false, w.n, k / 2)) != 0) return rc;
        if ((rc = make_map(&mb1, w1.w, false, w1.n, k / 2)) != 0) return rc;
        p.k_blocks = (p.k_steps + 3) / 4;
        p.a_k_blocks = p.k_blocks;
        return launch<KIND_MXF4>(sw, ma, mb0, mb1, p);
    }

    if (act == VELOX_ACT_FP8_ROW) {
        if (w.format != VELOX_FMT_FP8_ROW_BF16 || k % 128 != 0) return VELOX_ERR_UNSUPPORTED;
        uint8_t* codes = static_cast<uint8_t*>(scratch(SCRATCH_ACT_CODES, (size_t)a.m * k));
        float* scales = static_cast<float*>(scratch(SCRATCH_ACT_SCALES, (size_t)a.m * sizeof(float)));
        if (!codes || !scales) return (int)cudaErrorMemoryAllocation;
        rc = quantize_act_fp8row(a.x, a.xb, a.m, k, codes, scales);
        if (rc != 0) return rc;
        p.k_steps = (int)(k / 32);
        p.k_elems_per_block = 128;
        p.tok_scale = scales;
        const velox_sm100_view* hv[2] = {&w, &w1};
        for (int h = 0; h < 2; h++) {
            const velox_sm100_view& v = *hv[h];
            p.col_scale[h] = reinterpret_cast<const uint16_t*>(v.w + align256(v.n * k));
            p.b_rows_total[h] = v.n;
            p.valid_begin[h] = v.row_begin;
            p.valid_end[h] = v.row_begin + v.rows;
        }
        p.b_row0[0] = w.row_begin;
        p.b_row0[1] = sw ? w1.row_begin : w.row_begin + 128;
        p.b_tile_rows = sw ? 128 : 256;
        p.tiles_n = (int)((w.rows + p.b_tile_rows - 1) / p.b_tile_rows);
        p.out_row0 = w.row_begin;
        if ((rc = make_map(&ma, codes, false, a.m, k)) != 0) return rc;
        if ((rc = make_map(&mb0, w.w, false, w.n, k)) != 0) return rc;
        if ((rc = make_map(&mb1, w1.w, false, w1.n, k)) != 0) return rc;
        p.k_blocks = (p.k_steps + 3) / 4;
        p.a_k_blocks = p.k_blocks;
        return launch<KIND_F8>(sw, ma, mb0, mb1, p);
    }

    if (act != VELOX_ACT_BF16) return VELOX_ERR_UNSUPPORTED;
    // bf16 activations x weights dequantised to bf16 in scratch (view rows only, row 0 = row_begin).
    // Q4_K values are not bf16 numbers: they go in as hi + lo, two bf16 terms side by side along K
    // ([rows, 2k]) multiplied by the same activations, which the producer re-reads for the second half.
    const bool split = w.format == VELOX_FMT_GGML_Q4_K;
    const long long kw = split ? 2 * k : k;
    const size_t wbytes = (size_t)w.rows * kw * 2;
    uint16_t* wq = static_cast<uint16_t*>(scratch(SCRATCH_WEIGHT_BF16, wbytes * (sw ? 2 : 1)));
    if (!wq) return (int)cudaErrorMemoryAllocation;
    if ((rc = dequant_rows_bf16(&w, wq, kw, split ? k : 0)) != 0) return rc;
    if (sw && (rc = dequant_rows_bf16(&w1, wq + (size_t)w.rows * kw, kw, split ? k : 0)) != 0) return rc;
    const uint16_t* xb = a.xb;
    if (!xb || (reinterpret_cast<uintptr_t>(xb) & 15)) {
        uint16_t* xs = static_cast<uint16_t*>(scratch(SCRATCH_X_BF16, (size_t)a.m * k * 2));
        if (!xs) return (int)cudaErrorMemoryAllocation;
        if (a.x) {
            if ((rc = bf16_twin(a.x, xs, (long long)a.m * k)) != 0) return rc;
        } else {
            cudaError_t e = cudaMemcpyAsync(xs, a.xb, (size_t)a.m * k * 2, cudaMemcpyDeviceToDevice, stream());
            if (e != cudaSuccess) return (int)e;
        }
        xb = xs;
    }
    p.k_steps = (int)(kw / 16);
    p.k_elems_per_block = 64;
    p.a_k_blocks = (int)((k / 16 + 3) / 4);
    const velox_sm100_view* hv[2] = {&w, &w1};
    for (int h = 0; h < 2; h++) {
        const velox_sm100_view& v = *hv[h];
        if (v.format == VELOX_FMT_NVFP4)
            p.wdiv[h] = reinterpret_cast<const float*>(v.w + align256(v.n * k / 2) + v.n * k / 16);
        if (v.format == VELOX_FMT_FP8_ROW_BF16)
            p.col_scale[h] = reinterpret_cast<const uint16_t*>(v.w + align256(v.n * k)) + v.row_begin;
        p.b_rows_total[h] = v.rows;
        p.valid_begin[h] = 0;
        p.valid_end[h] = v.rows;
    }
    p.b_row0[0] = 0;
    p.b_row0[1] = sw ? 0 : 128;
    p.b_tile_rows = sw ? 128 : 256;
    p.tiles_n = (int)((w.rows + p.b_tile_rows - 1) / p.b_tile_rows);
    p.out_row0 = 0;
    if ((rc = make_map(&ma, xb, true, a.m, k)) != 0) return rc;
    if ((rc = make_map(&mb0, wq, true, w.rows, kw)) != 0) return rc;
    if ((rc = make_map(&mb1, sw ? wq + (size_t)w.rows * kw : wq, true, w.rows, kw)) != 0) return rc;
    p.k_blocks = (p.k_steps + 3) / 4;
    return launch<KIND_BF16>(sw, ma, mb0, mb1, p);
}

}  // namespace vx
