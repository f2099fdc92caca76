// Prefill GEMM on the 5th-generation tensor cores: y[m, rows] = x[m, k] . W^T for m > 16.
//
// One persistent CTA per SM walks output tiles of 128 tokens x 256 weight rows. Roles:
//   warp 0      operand producer: cp.async.bulk.tensor tiles of x and W (128-byte swizzled rows)
//               into a 3-stage shared-memory ring;
//   warp 1      MMA issuer: one elected thread issues tcgen05.mma with the accumulator in tensor
//               memory (128 lanes x 256 f32 columns): block-scaled kind::mxf4nvf4 for NVFP4,
//               kind::f8f6f4 for FP8, kind::f16 for bf16;
//   warps 2-5   epilogue: tcgen05.ld the accumulator, apply the per-tensor / per-row / per-token
//               factors, optionally silu(gate)*up; bf16 tiles go through a swizzled staging
//               buffer and a tensor-map store, f32 (or ragged) output is written directly.
//               Tensor memory is handed back as soon as the last columns are in registers;
//   warp 6      (NVFP4) scale producer: bulk copies of whole 512-byte scale atoms into a 4-stage
//               ring of their own, so scales run ahead of the operands;
//   warps 8-11  (NVFP4) scale movers: shared memory -> registers -> tensor memory (tcgen05.st),
//               one warp per lane quadrant, into one of four column sets. Measured on B200, the
//               tcgen05.cp route (twelve 32x128b copies per k-block on the MMA pipe) serialised
//               with the MMAs and cost more than they did.
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
#include <cstdio>
#include <cstdlib>
#include <mutex>

#include <cuda.h>  // CUtensorMap types; the encode entry point is resolved at run time

#include "common.cuh"
#include "gemm.cuh"
#include "tcgen.cuh"
#include "tpsync.cuh"

namespace vx {


constexpr int BM = 128;        // tokens per tile (MMA M)
constexpr int BN = 256;        // weight rows per tile (MMA N): two 128-row halves
constexpr int BK_BYTES = 128;  // bytes of K per row per stage: one swizzle row, four MMA k-steps
constexpr int SF_STAGES = 4;   // scale ring in shared memory and scale column sets in tensor memory
constexpr int A_BYTES = BM * BK_BYTES;
constexpr int B_HALF_BYTES = 128 * BK_BYTES;
constexpr int SFA_BYTES = 4 * 512;
constexpr int SFB_BYTES = 2 * 4 * 512;
constexpr int SF_STAGE_BYTES = SFA_BYTES + SFB_BYTES;
constexpr int STAGING_BYTES = 2 * 16384;  // two swizzled boxes of 128 tokens x 64 bf16 columns, one per column half

// Shared-memory plan for a CTA working alone (CG = 1: it loads both 128-row halves of the W tile)
// or as one of a pair (CG = 2: it loads its own 128 tokens of x and one half of the W tile; the
// pair's MMA reads the other half from the partner's shared memory).
template <int CG>
struct Plan {
    static constexpr int B_BYTES = (CG == 2 ? 1 : 2) * B_HALF_BYTES;
    static constexpr int STAGE_BYTES = A_BYTES + B_BYTES;   // 32 KB in a pair, 48 KB alone
    static constexpr int STAGES = CG == 2 ? 5 : 3;          // operand ring
    static constexpr int OFF_STAGING = STAGES * STAGE_BYTES;
    static constexpr int OFF_SF = OFF_STAGING + STAGING_BYTES;
    static constexpr int OFF_BARS = OFF_SF + SF_STAGES * SF_STAGE_BYTES;
    static constexpr int SMEM_BYTES = OFF_BARS + 1024 + 512;
};
constexpr int TMEM_COLS = 512;
constexpr int TMEM_SF_COL = 256;  // scale sets follow the accumulator
constexpr int TMEM_SF_SET = 48;   // per set: 16 columns of x scales, 32 columns of W scales
constexpr int RAW_STAGES = 3;          // ring of stored-byte tiles (bf16 kind with conversion in the kernel) ...
constexpr int RAW_STAGE_BYTES = 8192;  // ... in the shared memory the scale ring has in the NVFP4 kind
constexpr int GEMM_THREADS = 512;
constexpr int EPI_WARP0 = 4;     // warps 4..11 drain the accumulator, two per lane quadrant
constexpr int MOVER_WARP0 = 12;  // warps 12..15 move scales into tensor memory

enum { ST_OK = 0, ST_TIMEOUT_EMPTY = 1, ST_TIMEOUT_FULL = 2, ST_TIMEOUT_ACC_EMPTY = 3,
       ST_TIMEOUT_ACC_FULL = 4, ST_TIMEOUT_SF = 5 };

constexpr int MAX_PARTS = 3;   // views one launch can serve (q, k, v of one input)

// What differs between the views of one launch. Index [2]: the two 128-row halves of a W tile
// (the same view twice for a plain linear, gate and up for the fused SwiGLU form).
struct PartParams {
    long long b_row0[2];       // first row (tensor-map coordinates) of n-tile 0, per half
    long long b_rows_total[2]; // rows the half's tensor map / scale plane holds
    long long valid_begin[2], valid_end[2];  // rows of each half that belong to the view
    long long out_row0;        // row (half-0 coordinates) that maps to output column `col`
    const uint8_t* sfb[2];
    const float* wdiv[2];
    const uint16_t* col_scale[2];  // bf16 per row, indexed by the half's row coordinate
    float* y;
    uint16_t* yb;
    long long ld, col;
    uint8_t* q_codes;   // optional: the output also (or only) as NVFP4 activations, codes [m, q_ld / 2] ...
    uint8_t* q_atoms;   // ... and scale atoms over ceil(m / 128) * 128 rows
    long long q_ld;     // columns of the quantised matrix (a multiple of 64)
    float q_divisor;
    int b_tile_rows;    // rows advanced per n-tile
    int tiles_n;
    int tma_store;      // bf16-only output that the part's output tensor map describes
    int tile_end;       // tiles of this and all earlier parts (work units are numbered part after part)
};

struct GemmParams {
    int m;
    int k_blocks;       // ceil(k_steps / 4)
    int k_steps;        // 32-byte MMA k-steps in a row
    int k_elems_per_block;  // tensor-map elements per 128-byte block (128 for byte maps, 64 bf16)
    int a_k_blocks;         // the activation operand wraps around after this many blocks
    int tiles_m;
    int nparts;
    int k_tiles64;
    const uint8_t* sfa;
    float alpha;
    const float* tok_scale;
    const CUtensorMap* out_maps;   // optional (tensor parallel): one output map per owning rank, in global memory;
    int rows_per_owner;            // token rows [o * rows_per_owner, (o + 1) * rows_per_owner) go to out_maps[o]
    int raw_fmt;    // bf16 kind, pairs only, 0 = off: the W maps describe stored bytes (1: FP8 rows) that four
                    // warps turn into bf16 operands in shared memory, instead of bf16 scratch
    int acc_chunk;  // bf16 and FP8 kinds, 0 = off: k-blocks summed in tensor memory before the epilogue takes the sum over
    int early;      // the launch may start before the kernel ahead of it has finished (see the producers)
    int* status;
    PartParams part[MAX_PARTS];
    TpSync sync;    // tensor parallel: flags to wait for before the first activation load, flags to raise at the end
};

// W operand maps (SwiGLU: [0] gate, [1] up; otherwise one per part) and bf16 output maps per part.
struct GemmMaps {
    CUtensorMap b[MAX_PARTS];
    CUtensorMap out[MAX_PARTS];
};

__device__ int g_gemm_status = 0;

// Instruction descriptor: M = 128 (256 across a pair), N = 256, K-major operands, f32 accumulate.
template <int KIND, int CG>
__device__ __forceinline__ constexpr uint32_t instr_desc() {
    const uint32_t n = (uint32_t)(BN >> 3) << 17, m = (uint32_t)((BM * CG) >> 4) << 24;
    if (KIND == KIND_MXF4) return (1u << 7) | (1u << 10) | n | m;         // E2M1 x E2M1, UE4M3 scales
    if (KIND == KIND_F8) return (1u << 4) | n | m;                        // E4M3 x E4M3 -> f32
    return (1u << 4) | (1u << 7) | (1u << 10) | n | m;                    // BF16 x BF16 -> f32
}

// ---- kernel ------------------------------------------------------------------------------------------

template <int KIND, bool SWIGLU, int CG>
__global__ void __launch_bounds__(GEMM_THREADS, 1)
gemm_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ GemmMaps maps,
            const __grid_constant__ GemmParams p) {
    using PL = Plan<CG>;
    constexpr int OP_STAGES = PL::STAGES;
    constexpr int OP_STAGE_BYTES = PL::STAGE_BYTES;
    extern __shared__ uint8_t smem_raw[];
    const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    const uint32_t staging = base + PL::OFF_STAGING;
    const uint32_t sf_ring = base + PL::OFF_SF;
    const uint32_t bars = base + PL::OFF_BARS;
    auto op_full = [&](int s) { return bars + 8u * s; };
    auto op_empty = [&](int s) { return bars + 8u * (OP_STAGES + s); };
    auto peer_full = [&](int s) { return bars + 8u * (2 * OP_STAGES + s); };   // pairs: partner's stage landed
    auto sf_full = [&](int s) { return bars + 8u * (3 * OP_STAGES + s); };
    auto sf_empty = [&](int s) { return bars + 8u * (3 * OP_STAGES + SF_STAGES + s); };
    auto tsf_full = [&](int s) { return bars + 8u * (3 * OP_STAGES + 2 * SF_STAGES + s); };
    auto tsf_empty = [&](int s) { return bars + 8u * (3 * OP_STAGES + 3 * SF_STAGES + s); };
    const uint32_t acc_full = bars + 8u * (3 * OP_STAGES + 4 * SF_STAGES);
    const uint32_t acc_empty = acc_full + 8u;
    const uint32_t tmem_slot = acc_full + 16u;
    // second accumulator (bf16 kind with chunked sums): buffer b's barriers and first column
    auto cfull = [&](uint32_t b) { return acc_full + 24u * b; };
    auto cempty = [&](uint32_t b) { return acc_empty + 24u * b; };
    const bool chunked = KIND != KIND_MXF4 && p.acc_chunk > 0;   // (the NVFP4 kind's scale sets take the second accumulator's columns)
    // stored-byte ring (bf16 kind, conversion in the kernel)
    auto raw_full = [&](int s) { return acc_full + 40u + 8u * s; };
    auto raw_empty = [&](int s) { return acc_full + 64u + 8u * s; };
    const bool raw = KIND == KIND_BF16 && CG == 2 && p.raw_fmt != 0;
    uint32_t* tmem_slot_ptr = reinterpret_cast<uint32_t*>(smem_raw + (tmem_slot - smem_u32(smem_raw)));

    const int warp = threadIdx.x / 32, lane = threadIdx.x % 32;
    // A kernel launched behind this one with early start allowed may begin as CTAs here retire.
    if (threadIdx.x == 0) grid_launch_dependents();
    // In a pair, CTA 0 issues the MMAs for both and owns the barriers the other CTA reports to.
    const uint32_t rank = CG == 2 ? cluster_ctarank() : 0u;
    auto arrive_lead = [&](uint32_t bar) {
        if (CG == 2)
            mbar_arrive_cluster(map_to_cta(bar, 0));
        else
            mbar_arrive(bar);
    };
    auto commit = [&](uint32_t bar) {
        if (CG == 2)
            tc_commit_pair(bar);
        else
            tc_commit(bar);
    };

    if (threadIdx.x == 0) {
        for (int s = 0; s < OP_STAGES; s++) {
            mbar_init(op_full(s), raw ? 3 : 1);   // the producer's arrive, plus two converting warps'
            mbar_init(op_empty(s), 1);
            mbar_init(peer_full(s), 1);
        }
        for (int s = 0; s < RAW_STAGES; s++) {
            mbar_init(raw_full(s), 1);
            mbar_init(raw_empty(s), 2);
        }
        for (int s = 0; s < SF_STAGES; s++) {
            mbar_init(sf_full(s), 1);
            mbar_init(sf_empty(s), 4);
            mbar_init(tsf_full(s), 4 * CG);
            mbar_init(tsf_empty(s), 1);
        }
        mbar_init(acc_full, 1);
        mbar_init(acc_empty, 8 * CG);
        mbar_init(cfull(1), 1);
        mbar_init(cempty(1), 8 * CG);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("prefetch.tensormap [%0];" ::"l"(&tmap_a) : "memory");
        asm volatile("prefetch.tensormap [%0];" ::"l"(&maps.b[0]) : "memory");
        if (SWIGLU) asm volatile("prefetch.tensormap [%0];" ::"l"(&maps.b[1]) : "memory");
        if (p.part[0].tma_store && !p.out_maps) asm volatile("prefetch.tensormap [%0];" ::"l"(&maps.out[0]) : "memory");
    }
    if (warp == 1) {
        // tensor memory: in a pair both CTAs' warp 1 take part and both get the same address
        if (CG == 2) {
            asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(tmem_slot),
                         "r"((uint32_t)TMEM_COLS)
                         : "memory");
            asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
        } else {
            asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(tmem_slot),
                         "r"((uint32_t)TMEM_COLS)
                         : "memory");
            asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
        }
    }
    tc_fence_before();
    __syncthreads();
    if (CG == 2) cluster_sync_all();   // the partner's barriers exist before anything arrives on them
    tc_fence_after();
    const uint32_t tmem = *tmem_slot_ptr;

    // Registers follow the work: the four warps that only issue copies and MMAs and the four that
    // move scales give most of theirs back, and the eight epilogue warps take them, so that a
    // warp can hold its whole part of the accumulator (128 values) at once and hands tensor memory
    // back after one round trip instead of four.
    // (each role executes the instruction at the head of its own branch: every warp of a group of
    // four the same one)
#define VX_REGS_ISSUE() asm volatile("setmaxnreg.dec.sync.aligned.u32 48;" ::: "memory")
#define VX_REGS_MOVER() asm volatile("setmaxnreg.dec.sync.aligned.u32 80;" ::: "memory")
#define VX_REGS_EPILOGUE() asm volatile("setmaxnreg.inc.sync.aligned.u32 192;" ::: "memory")

    // Work units: tiles of 128 x CG tokens by 256 weight rows, walked by CTA (pair) number.
    const int unit = CG == 2 ? (int)blockIdx.x / 2 : (int)blockIdx.x;
    const int units = (int)gridDim.x / CG;
    const int tiles_mu = (p.tiles_m + CG - 1) / CG;
    const int num_tiles = p.part[p.nparts - 1].tile_end;
    // Work unit -> (part, token tile, row tile). Token tiles vary fastest, so the CTAs working at
    // the same time share W tiles in L2.
    struct TileAt {
        int pi, mt, nt;
    };
    auto tile_at = [&](int tile) {
        TileAt t;
        t.pi = 0;
        int first = 0;
        if (!SWIGLU) {
            while (t.pi + 1 < p.nparts && tile >= p.part[t.pi].tile_end) {
                first = p.part[t.pi].tile_end;
                t.pi++;
            }
        }
        const int local = tile - first;
        t.mt = (local % tiles_mu) * CG + (int)rank;
        t.nt = local / tiles_mu;
        return t;
    };
    // Tensor parallel: the activations (and their scales) are complete once every rank's flag of
    // this launch's wait row has reached the step's epoch. Polled by one lane, after the launch
    // ahead in the stream has completed.
    auto peers_ready = [&](bool leader) {
        bool ok = true;
        if (p.sync.wait_phase >= 0) {
            if (leader) {
                ok = tp_wait_flags(p.sync);
                asm volatile("fence.proxy.async.global;" ::: "memory");
            }
            ok = __shfl_sync(0xffffffffu, ok ? 1 : 0, __ffs(__ballot_sync(0xffffffffu, leader)) - 1) != 0;
        }
        return ok;
    };

    if (warp == 0) {
        // ---------------- operand producer: this CTA's x tile and W rows per k-block ----------------
        // (whole warp in the loop, one elected lane issuing, as in the MMA warp below)
        VX_REGS_ISSUE();
        {
            int stage = 0, rstage = 0;
            uint32_t phase = 0, rphase = 0;
            bool ok = true;
            const bool leader = elect_one();
            // Weights that are read from their stored payload do not depend on the kernel ahead of
            // this one in the stream, the activations do: with early start allowed the first ring
            // pass requests its W boxes at once, then waits for that kernel and adds the x boxes.
            // (The bf16 path's W operand is scratch the kernel ahead wrote: it waits first.)
            int issued = 0, pend_x[OP_STAGES], pend_y[OP_STAGES];
            bool waited = !(p.early && KIND != KIND_BF16);
            if (waited) {
                grid_dependency_wait();
                ok = peers_ready(leader);
            }
            auto after_dependency = [&]() {
                grid_dependency_wait();
                ok = peers_ready(leader) && ok;
                if (leader)
                    for (int i = 0; i < issued; i++)
                        tma_load_2d(base + i * OP_STAGE_BYTES, &tmap_a, op_full(i), pend_x[i], pend_y[i]);
                waited = true;
            };
            for (int tile = unit; tile < num_tiles && ok; tile += units) {
                const TileAt t = tile_at(tile);
                const PartParams& pp = p.part[t.pi];
                const int mt = t.mt;
                const int r0 = (int)(pp.b_row0[0] + (long long)t.nt * pp.b_tile_rows);
                const int r1 = (int)(pp.b_row0[1] + (long long)t.nt * pp.b_tile_rows);
                const CUtensorMap* mb0 = SWIGLU ? &maps.b[0] : &maps.b[t.pi];
                const CUtensorMap* mb1 = SWIGLU ? &maps.b[1] : mb0;
                for (int kb = 0; kb < p.k_blocks && ok; kb++) {
                    if (!waited && issued == OP_STAGES) after_dependency();
                    if (!mbar_wait(op_empty(stage), phase ^ 1u, 20)) {
                        if (leader) atomicExch(p.status, ST_TIMEOUT_EMPTY);
                        ok = false;
                        break;
                    }
                    const uint32_t sa = base + stage * OP_STAGE_BYTES;
                    const uint32_t sb = sa + A_BYTES;
                    const int kx = kb * p.k_elems_per_block;
                    if (raw) {
                        // x as usual; this CTA's 128 W rows as stored bytes into the byte ring, from
                        // where four warps convert them into the stage
                        if (!mbar_wait(raw_empty(rstage), rphase ^ 1u, 20)) {
                            if (leader) atomicExch(p.status, ST_TIMEOUT_EMPTY);
                            ok = false;
                            break;
                        }
                        if (leader) {
                            mbar_arrive_expect_tx(op_full(stage), A_BYTES);
                            tma_load_2d(sa, &tmap_a, op_full(stage), (kb % p.a_k_blocks) * p.k_elems_per_block, mt * BM);
                            mbar_arrive_expect_tx(raw_full(rstage), RAW_STAGE_BYTES);
                            tma_load_2d(sf_ring + rstage * RAW_STAGE_BYTES, rank ? mb1 : mb0, raw_full(rstage), kb * 64,
                                        rank ? r1 : r0);
                        }
                        if (++rstage == RAW_STAGES) {
                            rstage = 0;
                            rphase ^= 1u;
                        }
                    } else if (leader) {
                        mbar_arrive_expect_tx(op_full(stage), A_BYTES + PL::B_BYTES);
                        if (waited)
                            tma_load_2d(sa, &tmap_a, op_full(stage), (kb % p.a_k_blocks) * p.k_elems_per_block,
                                        mt * BM);
                        if (CG == 2) {
                            // one half of the W tile; the MMA reads the other from the partner
                            if (rank)
                                tma_load_2d(sb, mb1, op_full(stage), kx, r1);
                            else
                                tma_load_2d(sb, mb0, op_full(stage), kx, r0);
                        } else {
                            tma_load_2d(sb, mb0, op_full(stage), kx, r0);
                            tma_load_2d(sb + B_HALF_BYTES, mb1, op_full(stage), kx, r1);
                        }
                    }
                    if (!waited) {
                        pend_x[issued] = (kb % p.a_k_blocks) * p.k_elems_per_block;
                        pend_y[issued] = mt * BM;
                        issued++;
                    }
                    if (++stage == OP_STAGES) {
                        stage = 0;
                        phase ^= 1u;
                    }
                }
            }
            if (!waited) after_dependency();
            if (!ok) __nanosleep(200000);  // let copies already in flight land before the CTA exits
        }
    } else if (warp == 1 && rank != 0) {
        // ---------------- pair, second CTA: tell the MMA issuer when this CTA's operands have landed ----------------
        VX_REGS_ISSUE();
        int stage = 0;
        uint32_t phase = 0;
        bool ok = true;
        const bool leader = elect_one();
        for (int tile = unit; tile < num_tiles && ok; tile += units) {
            for (int kb = 0; kb < p.k_blocks; kb++) {
                if (!mbar_wait(op_full(stage), phase)) {
                    if (leader) atomicExch(p.status, ST_TIMEOUT_FULL);
                    ok = false;
                    break;
                }
                if (leader) mbar_arrive_cluster(map_to_cta(peer_full(stage), 0));
                if (++stage == OP_STAGES) {
                    stage = 0;
                    phase ^= 1u;
                }
            }
        }
    } else if (warp == 1) {
        // ---------------- MMA issuer ----------------
        // The whole warp walks the loop and one elected lane issues: addresses, descriptors and
        // barrier operands are then warp-uniform values, which is what the asynchronous tensor
        // instructions take; a loop run by a single diverged lane pays a register move per operand.
        VX_REGS_ISSUE();
        {
            int stage = 0, sstage = 0;
            uint32_t phase = 0, sphase = 0, acc_phase = 0;
            bool ok = true;
            const uint32_t idesc = instr_desc<KIND, CG>();
            const bool leader = elect_one();
            // Chunked sums (bf16 kind): every acc_chunk k-blocks go to the other of two accumulators and
            // are handed to the epilogue, which adds the chunks with round-to-nearest adds. The tensor
            // core's own f32 accumulation truncates, and over a long K that bias reaches the fourth
            // digit of sums that cancel.
            uint32_t chunk_no = 0, buf = 0;
            for (int tile = unit; tile < num_tiles && ok; tile += units) {
                if (!chunked &&
                    !(CG == 2 ? mbar_wait_cluster(acc_empty, acc_phase ^ 1u) : mbar_wait(acc_empty, acc_phase ^ 1u))) {
                    if (leader) atomicExch(p.status, ST_TIMEOUT_ACC_EMPTY);
                    break;
                }
                for (int kb = 0; kb < p.k_blocks; kb++) {
                    const bool chunk_head = chunked && kb % p.acc_chunk == 0;
                    if (chunk_head) {
                        buf = chunk_no & 1u;
                        const uint32_t par = ((chunk_no >> 1) & 1u) ^ 1u;
                        if (!(CG == 2 ? mbar_wait_cluster(cempty(buf), par) : mbar_wait(cempty(buf), par))) {
                            if (leader) atomicExch(p.status, ST_TIMEOUT_ACC_EMPTY);
                            ok = false;
                            break;
                        }
                    }
                    if (!mbar_wait(op_full(stage), phase) ||
                        (CG == 2 && !mbar_wait_cluster(peer_full(stage), phase))) {
                        if (leader) atomicExch(p.status, ST_TIMEOUT_FULL);
                        ok = false;
                        break;
                    }
                    if (KIND == KIND_MXF4) {
                        if (!(CG == 2 ? mbar_wait_cluster(tsf_full(sstage), sphase) : mbar_wait(tsf_full(sstage), sphase))) {
                            if (leader) atomicExch(p.status, ST_TIMEOUT_SF);
                            ok = false;
                            break;
                        }
                    }
                    tc_fence_after();
                    const int steps = min(4, p.k_steps - 4 * kb);
                    const uint32_t sa = base + stage * OP_STAGE_BYTES;
                    const uint32_t sb = sa + A_BYTES;
                    const uint64_t da = smem_desc_sw128(sa), db = smem_desc_sw128(sb);
                    const uint32_t tsf = tmem + TMEM_SF_COL + sstage * TMEM_SF_SET;
                    const uint32_t tacc = tmem + (chunked ? buf * (uint32_t)BN : 0u);
                    const bool fresh = chunked ? chunk_head : kb == 0;   // the first MMA overwrites the accumulator
                    const bool chunk_tail = chunked && (kb % p.acc_chunk == p.acc_chunk - 1 || kb == p.k_blocks - 1);
                    if (leader) {
                        // advancing 32 bytes along K inside the swizzle row: +2 in the address field
                        if (steps == 4) {
                            tc_mma<KIND, CG>(tacc, da, db, idesc, fresh ? 0u : 1u, tsf, tsf + 16);
                            tc_mma<KIND, CG>(tacc, da + 2u, db + 2u, idesc, 1u, tsf + 4, tsf + 24);
                            tc_mma<KIND, CG>(tacc, da + 4u, db + 4u, idesc, 1u, tsf + 8, tsf + 32);
                            tc_mma<KIND, CG>(tacc, da + 6u, db + 6u, idesc, 1u, tsf + 12, tsf + 40);
                        } else {
                            for (int j = 0; j < steps; j++)
                                tc_mma<KIND, CG>(tacc, da + 2u * j, db + 2u * j, idesc, fresh && j == 0 ? 0u : 1u,
                                                 tsf + 4 * j, tsf + 16 + 8 * j);
                        }
                        commit(op_empty(stage));
                        if (KIND == KIND_MXF4) commit(tsf_empty(sstage));
                        if (chunk_tail) commit(cfull(buf));
                    }
                    if (chunk_tail) chunk_no++;
                    if (++stage == OP_STAGES) {
                        stage = 0;
                        phase ^= 1u;
                    }
                    if (KIND == KIND_MXF4) {
                        if (++sstage == SF_STAGES) {
                            sstage = 0;
                            sphase ^= 1u;
                        }
                    }
                }
                if (ok && leader && !chunked) commit(acc_full);
                acc_phase ^= 1u;
            }
        }
    } else if (warp >= EPI_WARP0 && warp < EPI_WARP0 + 8) {
        // ---------------- epilogue: eight warps, two per lane quadrant, each taking half the columns ----------------
        VX_REGS_EPILOGUE();
        const int quad = warp % 4;
        const int hsel = (warp - EPI_WARP0) / 4;
        uint32_t acc_phase = 0, epi_chunk = 0;
        const bool store_thread = (warp - EPI_WARP0) % 4 == 0 && lane == 0;   // one per column half
        const uint32_t my_box = staging + (uint32_t)hsel * 16384u;
        const int bar_id = 1 + hsel;                                          // the four warps of a half
        constexpr int CHUNKS = SWIGLU ? 4 : 8;   // 32-column output chunks in a tile
        constexpr int MINE = CHUNKS / 2;         // ... of which this warp takes half
        for (int tile = unit; tile < num_tiles; tile += units) {
            const TileAt t = tile_at(tile);
            const PartParams& pp = p.part[t.pi];
            const int mt = t.mt, nt = t.nt;
            // this part's factors (requested before the wait for the accumulator, which hides them)
            const float d0 = pp.wdiv[0] ? __ldg(pp.wdiv[0]) : 1.0f;
            const float d1 = pp.wdiv[1] ? __ldg(pp.wdiv[1]) : 1.0f;
            const uint16_t* cs0 = pp.col_scale[0];
            const uint16_t* cs1 = pp.col_scale[1];
            const long long cs_rows0 = pp.b_rows_total[0], cs_rows1 = pp.b_rows_total[1];
            const long long vb0 = pp.valid_begin[0], ve0 = pp.valid_end[0], vb1 = pp.valid_begin[1], ve1 = pp.valid_end[1];
            if (!chunked) {
                if (!mbar_wait(acc_full, acc_phase, 60)) {
                    if (lane == 0) atomicExch(p.status, ST_TIMEOUT_ACC_FULL);
                    break;
                }
                tc_fence_after();
            }
            const float s0 = p.alpha / d0, s1 = p.alpha / d1;
            const int row_in_tile = quad * 32 + lane;
            const long long token = (long long)mt * BM + row_in_tile;
            const bool tok_ok = token < p.m;
            const float ts = (p.tok_scale && tok_ok) ? p.tok_scale[token] : 1.0f;
            const uint32_t taddr = tmem + ((uint32_t)(quad * 32) << 16);
            const long long rbase[2] = {pp.b_row0[0] + (long long)nt * pp.b_tile_rows,
                                        pp.b_row0[1] + (long long)nt * pp.b_tile_rows};
            // Whole-tile bf16 output through shared memory and a tensor-map store: taken when the
            // tile does not start left of the output's first column.
            const bool staged = pp.tma_store && rbase[0] >= pp.out_row0;
            const bool any_token = (long long)mt * BM < p.m;   // false only for a pair's second CTA past the end
            // chunk ch of the accumulator (and its partner in the up half) -> 32 finished values
            auto compute = [&](const int ch, const uint32_t (&r)[32], const uint32_t (&r2)[32], float (&v)[32]) {
                const int half = SWIGLU ? 0 : ch / 4;
                const long long row0 = rbase[half] + (ch % 4) * 32;   // first row of this chunk
                const long long urow0 = rbase[1] + ch * 32;           // SwiGLU: matching up rows
                const float sg = (half ? s1 : s0) * ts;
                const float su = s1 * ts;
                const uint16_t* csg = half ? cs1 : cs0;
                const long long csg_rows = half ? cs_rows1 : cs_rows0;
                // The per-row (FP8) scales are applied in a loop of their own: testing for them per
                // element puts 32 branches into every chunk.
#pragma unroll
                for (int c = 0; c < 32; c++) v[c] = __uint_as_float(r[c]) * sg;
                if (csg) {
#pragma unroll
                    for (int c = 0; c < 32; c++) {
                        const long long rr = row0 + c < csg_rows ? row0 + c : csg_rows - 1;
                        const float f = bf16_bits_to_f32(csg[rr]);
                        v[c] *= row0 + c < csg_rows ? f : 0.0f;
                    }
                }
                if (SWIGLU) {
                    float u[32];
#pragma unroll
                    for (int c = 0; c < 32; c++) u[c] = __uint_as_float(r2[c]) * su;
                    if (cs1) {
#pragma unroll
                        for (int c = 0; c < 32; c++) {
                            const long long rr = urow0 + c < cs_rows1 ? urow0 + c : cs_rows1 - 1;
                            const float f = bf16_bits_to_f32(cs1[rr]);
                            u[c] *= urow0 + c < cs_rows1 ? f : 0.0f;
                        }
                    }
#pragma unroll
                    // fast reciprocal: the quotient's two units in the last place are far inside the 5e-4 bound
                    for (int c = 0; c < 32; c++) v[c] = __fdividef(v[c], 1.0f + __expf(-v[c])) * u[c];
                }
            };
            auto store_direct = [&](const int ch, const float (&v)[32]) {
                if (!tok_ok) return;
                const int half = SWIGLU ? 0 : ch / 4;
                const long long row0 = rbase[half] + (ch % 4) * 32;
                const long long o0 = token * pp.ld + pp.col + (row0 - pp.out_row0);
                const long long vb = half ? vb1 : vb0, ve = half ? ve1 : ve0;
                const bool all = row0 >= vb && row0 + 32 <= ve;
                if (all && pp.yb && ((reinterpret_cast<uintptr_t>(pp.yb + o0) & 15) == 0)) {
#pragma unroll
                    for (int q = 0; q < 4; q++) {
                        uint4 pk;
                        pk.x = pack_bf16(v[8 * q], v[8 * q + 1]);
                        pk.y = pack_bf16(v[8 * q + 2], v[8 * q + 3]);
                        pk.z = pack_bf16(v[8 * q + 4], v[8 * q + 5]);
                        pk.w = pack_bf16(v[8 * q + 6], v[8 * q + 7]);
                        *reinterpret_cast<uint4*>(pp.yb + o0 + 8 * q) = pk;
                    }
                } else if (pp.yb) {
#pragma unroll
                    for (int c = 0; c < 32; c++)
                        if (row0 + c >= vb && row0 + c < ve) pp.yb[o0 + c] = bf16_bits(v[c]);
                }
                if (all && pp.y && ((reinterpret_cast<uintptr_t>(pp.y + o0) & 15) == 0)) {
#pragma unroll
                    for (int q = 0; q < 8; q++)
                        *reinterpret_cast<float4*>(pp.y + o0 + 4 * q) =
                            make_float4(v[4 * q], v[4 * q + 1], v[4 * q + 2], v[4 * q + 3]);
                } else if (pp.y) {
#pragma unroll
                    for (int c = 0; c < 32; c++)
                        if (row0 + c >= vb && row0 + c < ve) pp.y[o0 + c] = v[c];
                }
            };
            auto release_acc = [&](uint32_t b = 0u) {
                // this warp's part of the accumulator is in registers: hand it back to the MMA issuer
                tc_fence_before();
                __syncwarp();
                if (lane == 0) arrive_lead(cempty(b));
            };
            // This warp's 128 accumulator values (SwiGLU: 64 gate + 64 up) into registers, and tensor
            // memory handed back. Chunked sums: the chunks arrive one after the other in the two
            // accumulators and are added here, in order, with round-to-nearest adds.
            auto drain = [&](uint32_t (&r)[MINE][32], uint32_t (&r2)[SWIGLU ? MINE : 1][32]) -> bool {
                if (!chunked) {
#pragma unroll
                    for (int i = 0; i < MINE; i++) {
                        const int ch = hsel * MINE + i;
                        tc_ld32(taddr + ch * 32, r[i]);
                        if (SWIGLU) tc_ld32(taddr + 128 + ch * 32, r2[SWIGLU ? i : 0]);
                    }
                    tc_wait_ld();
                    release_acc();
                    return true;
                }
                const int nchunks = (p.k_blocks + p.acc_chunk - 1) / p.acc_chunk;
#pragma unroll
                for (int i = 0; i < MINE; i++)
#pragma unroll
                    for (int j = 0; j < 32; j++) {
                        r[i][j] = 0u;
                        if (SWIGLU) r2[SWIGLU ? i : 0][j] = 0u;
                    }
#pragma unroll 1
                for (int c = 0; c < nchunks; c++) {
                    const uint32_t b = epi_chunk & 1u;
                    if (!mbar_wait(cfull(b), (epi_chunk >> 1) & 1u, 60)) {
                        if (lane == 0) atomicExch(p.status, ST_TIMEOUT_ACC_FULL);
                        return false;
                    }
                    tc_fence_after();
#pragma unroll
                    for (int i = 0; i < MINE; i++) {
                        const int ch = hsel * MINE + i;
                        uint32_t t[32];
                        tc_ld32(taddr + b * (uint32_t)BN + ch * 32, t);
                        tc_wait_ld();
#pragma unroll
                        for (int j = 0; j < 32; j++)
                            r[i][j] = __float_as_uint(__uint_as_float(r[i][j]) + __uint_as_float(t[j]));
                        if (SWIGLU) {
                            tc_ld32(taddr + b * (uint32_t)BN + 128 + ch * 32, t);
                            tc_wait_ld();
#pragma unroll
                            for (int j = 0; j < 32; j++)
                                r2[SWIGLU ? i : 0][j] = __float_as_uint(__uint_as_float(r2[SWIGLU ? i : 0][j]) + __uint_as_float(t[j]));
                        }
                    }
                    release_acc(b);
                    epi_chunk++;
                }
                return true;
            };
            const bool emit_q = pp.q_codes != nullptr && mt < p.tiles_m;
            if (staged || pp.q_codes != nullptr) {
                // Drain first: finish this warp's values and keep them as packed bf16 (16 registers
                // per chunk), release tensor memory so the next tile's MMAs can start, and only then
                // spend time on shared-memory staging and the tensor-map stores.
                uint32_t pk[MINE][16];
                {
                    uint32_t r[MINE][32], r2[SWIGLU ? MINE : 1][32];
                    if (!drain(r, r2)) break;
#pragma unroll
                    for (int i = 0; i < MINE; i++) {
                        float v[32];
                        compute(hsel * MINE + i, r[i], SWIGLU ? r2[SWIGLU ? i : 0] : r[i], v);
#pragma unroll
                        for (int c = 0; c < 16; c++) pk[i][c] = pack_bf16(v[2 * c], v[2 * c + 1]);
                    }
                }
                if (emit_q) {
                    // The output as the next linear's NVFP4 activations, quantised from the bf16
                    // values exactly as the stand-alone quantiser does (quotients by the Markstein
                    // sequence q0 = a*r, q = fma(fma(-q0, d, a), r, q0), which is the correctly
                    // rounded a / d when r is the correctly rounded 1 / d).
#pragma unroll
                    for (int j = 0; j < MINE / 2; j++) {
                        const long long col0 = (rbase[0] - pp.out_row0) + (long long)(hsel * MINE + 2 * j) * 32;
                        uint32_t sc = 0;
                        uint32_t cw[8];
#pragma unroll
                        for (int g = 0; g < 4; g++) {
                            float v[16];
                            float amax = 0.0f;
#pragma unroll
                            for (int i = 0; i < 8; i++) {
                                const uint32_t u = pk[2 * j + g / 2][(g % 2) * 8 + i];
                                v[2 * i] = __uint_as_float(u << 16);
                                v[2 * i + 1] = __uint_as_float(u & 0xffff0000u);
                                amax = fmaxf(amax, fmaxf(fabsf(v[2 * i]), fabsf(v[2 * i + 1])));
                            }
                            const uint32_t sb = f32_to_e4m3(__fdiv_rn(__fmul_rn(pp.q_divisor, amax), 6.0f));
                            uint32_t o0 = 0, o1 = 0;
                            if (sb != 0) {
                                const float ds = e4m3_to_f32(sb);
                                const float rc = __frcp_rn(ds);
#pragma unroll
                                for (int i = 0; i < 8; i++) {
                                    const float a0 = __fmul_rn(v[2 * i], pp.q_divisor);
                                    const float a1 = __fmul_rn(v[2 * i + 1], pp.q_divisor);
                                    float q0 = __fmul_rn(a0, rc), q1 = __fmul_rn(a1, rc);
                                    q0 = __fmaf_rn(__fmaf_rn(-q0, ds, a0), rc, q0);
                                    q1 = __fmaf_rn(__fmaf_rn(-q1, ds, a1), rc, q1);
                                    const uint32_t b = f32x2_to_e2m1x2(q0, q1) << (8 * (i & 3));
                                    if (i < 4) o0 |= b; else o1 |= b;
                                }
                            }
                            cw[2 * g] = o0;
                            cw[2 * g + 1] = o1;
                            sc |= sb << (8 * g);
                        }
                        if (col0 + 64 <= pp.q_ld) {
                            if (tok_ok) {
                                uint4* dst = reinterpret_cast<uint4*>(pp.q_codes + (token * pp.q_ld + col0) / 2);
                                dst[0] = make_uint4(cw[0], cw[1], cw[2], cw[3]);
                                dst[1] = make_uint4(cw[4], cw[5], cw[6], cw[7]);
                            }
                            // rows past m inside the last 128-row atom carry zero scales
                            *reinterpret_cast<uint32_t*>(pp.q_atoms + nvfp4_scale_offset(token, col0 / 16, pp.q_ld)) =
                                tok_ok ? sc : 0u;
                        }
                    }
                }
                if (staged) {
#pragma unroll
                for (int bx = 0; bx < MINE / 2; bx++) {
                    // the store that last read this half's 64-column box must be done with it
                    if (store_thread) asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");
                    asm volatile("bar.sync %0, 128;" ::"r"(bar_id) : "memory");
                    const uint32_t rowp = my_box + (uint32_t)row_in_tile * 128u;
#pragma unroll
                    for (int i2 = 0; i2 < 2; i2++) {
#pragma unroll
                        for (int q = 0; q < 4; q++) {
                            // 16-byte piece index XOR row % 8 (128-byte swizzle)
                            const uint4 w4 = make_uint4(pk[2 * bx + i2][4 * q], pk[2 * bx + i2][4 * q + 1],
                                                        pk[2 * bx + i2][4 * q + 2], pk[2 * bx + i2][4 * q + 3]);
                            const uint32_t piece = (uint32_t)(i2 * 4 + q);
                            sts16(rowp + ((piece ^ (uint32_t)(row_in_tile & 7)) << 4), w4);
                        }
                    }
                    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
                    asm volatile("bar.sync %0, 128;" ::"r"(bar_id) : "memory");
                    if (store_thread && any_token) {
                        // tensor parallel: the tile goes straight into the buffer of the rank that owns
                        // these token rows (a store over NVLink when that is not this rank)
                        const CUtensorMap* omap = &maps.out[t.pi];
                        int orow = mt * BM;
                        if (p.out_maps) {
                            const int owner = orow / p.rows_per_owner;
                            omap = p.out_maps + owner;
                            orow -= owner * p.rows_per_owner;
                        }
                        tma_store_2d(omap, my_box, (int)(rbase[0] - pp.out_row0) + (hsel * (MINE / 2) + bx) * 64, orow);
                        asm volatile("cp.async.bulk.commit_group;" ::: "memory");
                    }
                }
                }
            } else {
                uint32_t r[MINE][32], r2[SWIGLU ? MINE : 1][32];
                if (!drain(r, r2)) break;
#pragma unroll
                for (int i = 0; i < MINE; i++) {
                    float v[32];
                    compute(hsel * MINE + i, r[i], SWIGLU ? r2[SWIGLU ? i : 0] : r[i], v);
                    store_direct(hsel * MINE + i, v);
                }
            }
            acc_phase ^= 1u;
        }
        if (store_thread) {
            // all of this thread's tile stores are complete (written, not merely read from shared memory)
            asm volatile("cp.async.bulk.wait_group 0;" ::: "memory");
            if (p.sync.signal_phase >= 0) {
                asm volatile("fence.proxy.async.global;" ::: "memory");
                __threadfence_system();
            }
        }
    } else if (KIND == KIND_MXF4 && warp == 2) {
        // ---------------- scale producer: whole 512-byte atoms, x then the two W halves ----------------
        // (in a pair each CTA needs the scales of its own tokens and of all 256 weight rows)
        VX_REGS_ISSUE();
        {
            int stage = 0;
            uint32_t phase = 0;
            bool ok = true;
            const bool leader = elect_one();
            grid_dependency_wait();   // the activation scales come from the kernel ahead of this one ...
            ok = peers_ready(leader);  // ... or, tensor parallel, from every rank's norm
            for (int tile = unit; tile < num_tiles && ok; tile += units) {
                const TileAt t = tile_at(tile);
                const PartParams& pp = p.part[t.pi];
                const int mt = t.mt;
                const long long r0 = pp.b_row0[0] + (long long)t.nt * pp.b_tile_rows;
                const long long r1 = pp.b_row0[1] + (long long)t.nt * pp.b_tile_rows;
                const bool sf0 = r0 < pp.b_rows_total[0], sf1 = r1 < pp.b_rows_total[1];
                const bool sfx = mt < p.tiles_m;   // false only for a pair's second CTA past the last token tile
                for (int kb = 0; kb < p.k_blocks; kb++) {
                    if (!mbar_wait(sf_empty(stage), phase ^ 1u, 50)) {
                        if (leader) atomicExch(p.status, ST_TIMEOUT_SF);
                        ok = false;
                        break;
                    }
                    const uint32_t bytes = (uint32_t)min(4, p.k_steps - 4 * kb) * 512u;
                    const uint32_t ssfa = sf_ring + stage * SF_STAGE_BYTES, ssfb = ssfa + SFA_BYTES;
                    const long long atom = 4LL * kb;
                    if (leader) {
                        const uint32_t parts = (sfx ? 1u : 0u) + (sf0 ? 1u : 0u) + (sf1 ? 1u : 0u);
                        if (parts == 0) {
                            mbar_arrive(sf_full(stage));
                        } else {
                            mbar_arrive_expect_tx(sf_full(stage), bytes * parts);
                            if (sfx)
                                bulk_load_1d(ssfa, p.sfa + ((long long)mt * p.k_tiles64 + atom) * 512, bytes,
                                             sf_full(stage));
                            if (sf0)
                                bulk_load_1d(ssfb, pp.sfb[0] + ((r0 / 128) * p.k_tiles64 + atom) * 512, bytes,
                                             sf_full(stage));
                            if (sf1)
                                bulk_load_1d(ssfb + 4 * 512, pp.sfb[1] + ((r1 / 128) * p.k_tiles64 + atom) * 512,
                                             bytes, sf_full(stage));
                        }
                    }
                    if (++stage == SF_STAGES) {
                        stage = 0;
                        phase ^= 1u;
                    }
                }
            }
            if (!ok) __nanosleep(200000);
        }
    } else if (KIND == KIND_MXF4 && warp >= MOVER_WARP0) {
        // ---------------- scale movers: shared memory -> tensor memory through registers ----------------
        // Lane i of the warp serving lane quadrant q writes rows i, i+32, i+64, i+96 of each
        // 128-row atom: the 16 bytes of atom row i are the four 32-bit columns of that atom,
        // replicated in every quadrant as the block-scaled MMA reads them.
        VX_REGS_MOVER();
        const int quad = warp % 4;
        int stage = 0;
        uint32_t phase = 0;
        bool ok = true;
        for (int tile = unit; tile < num_tiles && ok; tile += units) {
            for (int kb = 0; kb < p.k_blocks; kb++) {
                if (!mbar_wait(sf_full(stage), phase, 50)) {
                    if (lane == 0) atomicExch(p.status, ST_TIMEOUT_SF);
                    ok = false;
                    break;
                }
                const uint32_t ssfa = sf_ring + stage * SF_STAGE_BYTES + (uint32_t)lane * 16u;
                uint32_t ra[16], rb[32];
#pragma unroll
                for (int j = 0; j < 4; j++) {
                    const uint4 a = lds16(ssfa + 512 * j);
                    ra[4 * j] = a.x; ra[4 * j + 1] = a.y; ra[4 * j + 2] = a.z; ra[4 * j + 3] = a.w;
                    const uint4 b0 = lds16(ssfa + SFA_BYTES + 512 * j);
                    const uint4 b1 = lds16(ssfa + SFA_BYTES + 2048 + 512 * j);
                    rb[8 * j] = b0.x; rb[8 * j + 1] = b0.y; rb[8 * j + 2] = b0.z; rb[8 * j + 3] = b0.w;
                    rb[8 * j + 4] = b1.x; rb[8 * j + 5] = b1.y; rb[8 * j + 6] = b1.z; rb[8 * j + 7] = b1.w;
                }
                // The stage is handed back to a writer of another proxy (the bulk copies of the scale
                // producer): the reads above have to be ordered ahead of that proxy's accesses before
                // the arrive, or a copy can land while a lane's load is still in flight. Measured on
                // B200 without this fence: a few percent of all tiles but a CTA's first came out with
                // one k-block's scales of the block four steps later, in single lane quadrants.
                asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
                __syncwarp();
                if (lane == 0) mbar_arrive(sf_empty(stage));
                // the MMAs that read this column set (SF_STAGES k-blocks ago) must have completed
                if (!mbar_wait(tsf_empty(stage), phase ^ 1u, 50)) {
                    if (lane == 0) atomicExch(p.status, ST_TIMEOUT_SF);
                    ok = false;
                    break;
                }
                tc_fence_after();
                const uint32_t tsf = tmem + ((uint32_t)(quad * 32) << 16) + TMEM_SF_COL + stage * TMEM_SF_SET;
                tc_st16(tsf, ra);
                tc_st32(tsf + 16, rb);
                tc_wait_st();
                tc_fence_before();
                __syncwarp();
                if (lane == 0) arrive_lead(tsf_full(stage));
                if (++stage == SF_STAGES) {
                    stage = 0;
                    phase ^= 1u;
                }
            }
        }
    }

    else if (KIND == KIND_BF16 && warp >= MOVER_WARP0) {
        // ---------------- converters (bf16 kind on stored bytes): byte ring -> bf16 W operand of the stage ----------------
        // FP8 rows: thread (row = ct / 4 + 16 j, piece = ct % 4) takes 16 stored bytes and writes 16
        // bf16 numbers, two 16-byte pieces of the row's 128-byte line at the places the 128-byte
        // swizzle puts them (piece index xor row % 8). An E4M3 byte re-labelled as bf16 is the value
        // times 2^-120, subnormals included; the bf16 multiply by 2^120 is exact.
        VX_REGS_MOVER();
        if (raw) {
            // Two groups of two warps take the k-blocks in turn, so that one group's wait, loads,
            // stores and fence overlap the other's (a single group's round trip per k-block was
            // longer than the k-block's MMAs).
            const int group = (warp - MOVER_WARP0) / 2;
            const int ct = (int)threadIdx.x - (MOVER_WARP0 + 2 * group) * 32;   // 0..63 within the group
            const int piece = ct % 4;
            bool ok = true;
            const __nv_bfloat162 up = __floats2bfloat162_rn(1.329227995784916e36f, 1.329227995784916e36f);   // 2^120
            long long it = 0;   // k-blocks since the kernel began (all tiles of this CTA)
            for (int tile = unit; tile < num_tiles && ok; tile += units) {
                for (int kb = 0; kb < p.k_blocks; kb++, it++) {
                    if ((int)(it & 1) != group) continue;
                    const int stage = (int)(it % OP_STAGES), rstage = (int)(it % RAW_STAGES);
                    const uint32_t phase = (uint32_t)(it / OP_STAGES) & 1u, rphase = (uint32_t)(it / RAW_STAGES) & 1u;
                    if (!mbar_wait(raw_full(rstage), rphase, 20) || !mbar_wait(op_empty(stage), phase ^ 1u, 20)) {
                        if (lane == 0) atomicExch(p.status, ST_TIMEOUT_FULL);
                        ok = false;
                        break;
                    }
                    const uint32_t src = sf_ring + rstage * RAW_STAGE_BYTES;
                    const uint32_t dstb = base + stage * OP_STAGE_BYTES + A_BYTES;
#pragma unroll 2
                    for (int j = 0; j < 8; j++) {
                        const int row = ct / 4 + 16 * j;
                        const uint4 q = lds16(src + row * 64 + piece * 16);
                        const uint32_t w[4] = {q.x, q.y, q.z, q.w};
                        uint32_t o[8];
#pragma unroll
                        for (int i = 0; i < 4; i++) {
                            const uint32_t odd = ((w[i] >> 4) & 0x07F007F0u) | (w[i] & 0x80008000u);   // bytes 1, 3
                            const uint32_t v = w[i] << 8;
                            const uint32_t even = ((v >> 4) & 0x07F007F0u) | (v & 0x80008000u);        // bytes 0, 2
                            uint32_t lo = __byte_perm(even, odd, 0x5410u), hi = __byte_perm(even, odd, 0x7632u);
                            __nv_bfloat162 a = __hmul2(*reinterpret_cast<__nv_bfloat162*>(&lo), up);
                            __nv_bfloat162 b = __hmul2(*reinterpret_cast<__nv_bfloat162*>(&hi), up);
                            o[2 * i] = *reinterpret_cast<uint32_t*>(&a);
                            o[2 * i + 1] = *reinterpret_cast<uint32_t*>(&b);
                        }
                        const uint32_t line = dstb + row * 128;
                        sts16(line + (((2 * piece) ^ (row & 7)) << 4), make_uint4(o[0], o[1], o[2], o[3]));
                        sts16(line + (((2 * piece + 1) ^ (row & 7)) << 4), make_uint4(o[4], o[5], o[6], o[7]));
                    }
                    // the MMA (asynchronous proxy) reads what these generic-proxy stores wrote, and the
                    // next bulk copy into the byte stage follows the loads above
                    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
                    __syncwarp();
                    if (lane == 0) {
                        mbar_arrive(op_full(stage));
                        mbar_arrive(raw_empty(rstage));
                    }
                }
            }
        }
    }

    else if (warp < 4) {
        VX_REGS_ISSUE();       // warps without a role in this form of the kernel
    } else {
        VX_REGS_MOVER();
    }
#undef VX_REGS_ISSUE
#undef VX_REGS_MOVER
#undef VX_REGS_EPILOGUE

    // Nobody leaves while the partner may still signal this CTA's barriers or read its shared memory.
    tc_fence_before();
    __syncthreads();
    if (CG == 2) cluster_sync_all();
    if (warp == 1) {
        if (CG == 2)
            asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"((uint32_t)TMEM_COLS)
                         : "memory");
        else
            asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"((uint32_t)TMEM_COLS)
                         : "memory");
    }
    // Tensor parallel: every CTA's stores are complete behind the barrier above; the last CTA of the
    // grid to get here tells every rank that this rank's partial sums have landed.
    if (threadIdx.x == 0) tp_signal(p.sync, gridDim.x);
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

int gemm_make_map_u8(CUtensorMap* map, const void* ptr, long long rows, long long row_bytes, int box_rows) {
    if (!encode_fn()) return VELOX_ERR_UNSUPPORTED;
    const cuuint64_t dims[2] = {(cuuint64_t)row_bytes, (cuuint64_t)rows};
    const cuuint64_t strides[1] = {(cuuint64_t)row_bytes};
    const cuuint32_t box[2] = {128u, (cuuint32_t)box_rows};
    const cuuint32_t estr[2] = {1, 1};
    CUresult r = encode_fn()(map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void*>(ptr), dims, strides, box, estr,
                             CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                             CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r == CUDA_SUCCESS ? 0 : VELOX_ERR_UNSUPPORTED;
}

// Output maps of a tensor-parallel row-split linear: map o covers the [rows_per_owner, cols] bf16
// buffer at ptrs[o] (this rank's slot in rank o's memory). Encoded here, copied to `maps_dev`
// (n x 128 bytes of device memory, 64-byte aligned) on the current stream.
int gemm_make_rs_maps(void* maps_dev, const unsigned long long* ptrs, int n, int rows_per_owner, long long cols) {
    if (!encode_fn() || n < 1 || n > VX_MAX_PEERS || !maps_dev || (reinterpret_cast<uintptr_t>(maps_dev) & 63))
        return VELOX_ERR_UNSUPPORTED;
    CUtensorMap maps[VX_MAX_PEERS];
    for (int o = 0; o < n; o++) {
        const cuuint64_t dims[2] = {(cuuint64_t)cols, (cuuint64_t)rows_per_owner};
        const cuuint64_t strides[1] = {(cuuint64_t)cols * 2};
        const cuuint32_t box[2] = {64u, 128u};
        const cuuint32_t estr[2] = {1, 1};
        if (encode_fn()(&maps[o], CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, reinterpret_cast<void*>(ptrs[o]), dims, strides,
                        box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                        CU_TENSOR_MAP_L2_PROMOTION_NONE, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
            return VELOX_ERR_UNSUPPORTED;
    }
    // pageable source: the copy has read `maps` by the time the call returns
    cudaError_t e = cudaMemcpyAsync(maps_dev, maps, sizeof(CUtensorMap) * n, cudaMemcpyHostToDevice, stream());
    return e == cudaSuccess ? 0 : (int)e;
}

// Stored bytes of a row-major matrix [rows, row_bytes] as 128-row x 64-byte boxes, no swizzle (the
// byte ring of the bf16 kind's in-kernel conversion).
static int make_raw_map(CUtensorMap* map, const void* ptr, long long rows, long long row_bytes) {
    const cuuint64_t dims[2] = {(cuuint64_t)row_bytes, (cuuint64_t)rows};
    const cuuint64_t strides[1] = {(cuuint64_t)row_bytes};
    const cuuint32_t box[2] = {64u, 128u};
    const cuuint32_t estr[2] = {1, 1};
    CUresult r = encode_fn()(map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void*>(ptr), dims, strides, box, estr,
                             CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                             CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r == CUDA_SUCCESS ? 0 : VELOX_ERR_UNSUPPORTED;
}

// Tensor map over the bf16 output columns [col, col + out_cols) of a part's yb, for whole-tile
// stores. Leaves tma_store at 0 when the output is not bf16-only or not 16-byte friendly.
static void make_out_map(CUtensorMap* map, int m, PartParams& pp, long long out_cols, long long first_row) {
    pp.tma_store = 0;
    if (!pp.yb || pp.y || pp.ld % 8 != 0 || pp.col % 8 != 0 || first_row % 8 != 0) return;
    uint16_t* basep = pp.yb + pp.col;
    if (reinterpret_cast<uintptr_t>(basep) & 15) return;
    const cuuint64_t dims[2] = {(cuuint64_t)out_cols, (cuuint64_t)m};
    const cuuint64_t strides[1] = {(cuuint64_t)pp.ld * 2};
    const cuuint32_t box[2] = {64u, 128u};
    const cuuint32_t estr[2] = {1, 1};
    if (encode_fn()(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, basep, dims, strides, box, estr,
                    CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_NONE,
                    CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS)
        pp.tma_store = 1;
}

static int sm_count() {
    static int sms[64] = {};
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 148;
    if (sms[dev] == 0) {
        int n = 0;
        cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev);
        sms[dev] = n > 0 ? n : 148;
    }
    return sms[dev];
}

template <int KIND, bool SWIGLU, int CG>
static int launch_cfg(const CUtensorMap& a, const GemmMaps& maps, GemmParams& p, int sms) {
    auto kern = gemm_kernel<KIND, SWIGLU, CG>;
    constexpr int smem = Plan<CG>::SMEM_BYTES;
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
    if (e != cudaSuccess) return (int)e;
    int tiles = 0;
    for (int i = 0; i < p.nparts; i++) {
        tiles += ((p.tiles_m + CG - 1) / CG) * p.part[i].tiles_n;
        p.part[i].tile_end = tiles;
    }
    cudaLaunchConfig_t cfg{};
    cfg.blockDim = dim3(GEMM_THREADS);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream();
    cudaLaunchAttribute attr[2];
    int units = sms / CG;
    cfg.attrs = attr;
    cfg.numAttrs = 0;
    if (CG == 2) {
        attr[0].id = cudaLaunchAttributeClusterDimension;
        attr[0].val.clusterDim.x = 2;
        attr[0].val.clusterDim.y = 1;
        attr[0].val.clusterDim.z = 1;
        cfg.numAttrs = 1;
        // pairs that can be resident at once (GPCs with an odd SM count leave one SM out)
        static int max_pairs[2] = {0, 0};
        int& mp = max_pairs[SWIGLU ? 1 : 0];
        if (mp == 0) {
            cfg.gridDim = dim3(2 * (sms / 2));
            int n = 0;
            if (cudaOccupancyMaxActiveClusters(&n, kern, &cfg) != cudaSuccess || n <= 0) n = sms / 2;
            cudaGetLastError();
            mp = n;
        }
        units = mp < sms / 2 ? mp : sms / 2;
    }
    if (tiles < units) units = tiles;
    cfg.gridDim = dim3(units * CG);
    if (p.early) {
        // early start: CTAs may become resident while the kernel ahead in the stream drains; they
        // fetch weights and wait for that kernel before reading or writing anything it touches
        attr[cfg.numAttrs].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[cfg.numAttrs].val.programmaticStreamSerializationAllowed = 1;
        cfg.numAttrs++;
    }
    e = cudaLaunchKernelEx(&cfg, kern, a, maps, p);
    if (e != cudaSuccess) return (int)e;
    return launch_status();
}

// out_cols / first_row per part: the view's width and the parent row its output column 0 stands for.
template <int KIND>
static int launch(bool swiglu, const CUtensorMap& a, GemmMaps& maps, GemmParams& p, const long long* out_cols,
                  const long long* first_row) {
    for (int i = 0; i < p.nparts; i++) {
        maps.out[i] = a;   // a valid map even where none is used
        if (p.out_maps)
            p.part[i].tma_store = 1;   // every tile is stored through the owner's map
        else
            make_out_map(&maps.out[i], p.m, p.part[i], out_cols[i], first_row[i]);
    }
    // (entries no tile refers to still have to be valid maps; the SwiGLU form uses b[0] and b[1])
    for (int i = swiglu && p.nparts < 2 ? 2 : p.nparts; i < MAX_PARTS; i++) maps.b[i] = maps.b[0];
    for (int i = p.nparts; i < MAX_PARTS; i++) maps.out[i] = a;
    const int sms = sm_count();
    TimedRegion timed(KIND == KIND_MXF4 ? TIMED_GEMM_FP4 : KIND == KIND_F8 ? TIMED_GEMM_FP8 : TIMED_GEMM_BF16);
    // More than one token tile: CTA pairs (256 tokens per unit, half the W traffic per CTA).
    const bool pair = p.tiles_m > 1;
    if (swiglu) return pair ? launch_cfg<KIND, true, 2>(a, maps, p, sms) : launch_cfg<KIND, true, 1>(a, maps, p, sms);
    return pair ? launch_cfg<KIND, false, 2>(a, maps, p, sms) : launch_cfg<KIND, false, 1>(a, maps, p, sms);
}

// Device addresses of the status word and of the signalling ticket, per device ordinal (a
// __device__ variable has one instance per device).
__device__ unsigned int g_gemm_tp_ticket = 0;
static std::mutex g_sym_mu;
static int* status_ptr() {
    static int* ptrs[64] = {};
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return nullptr;
    std::lock_guard<std::mutex> lock(g_sym_mu);
    if (!ptrs[dev] && cudaGetSymbolAddress(reinterpret_cast<void**>(&ptrs[dev]), g_gemm_status) != cudaSuccess) {
        cudaGetLastError();
        return nullptr;
    }
    return ptrs[dev];
}
static unsigned int* ticket_ptr() {
    static unsigned int* ptrs[64] = {};
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return nullptr;
    std::lock_guard<std::mutex> lock(g_sym_mu);
    if (!ptrs[dev] && cudaGetSymbolAddress(reinterpret_cast<void**>(&ptrs[dev]), g_gemm_tp_ticket) != cudaSuccess) {
        cudaGetLastError();
        return nullptr;
    }
    return ptrs[dev];
}

int gemm_status_sync() {
    int v = -1;
    if (cudaMemcpyFromSymbol(&v, g_gemm_status, sizeof(int)) != cudaSuccess) return -1;
    return v;
}

int gemm_status_reset() {
    const int zero = 0;
    const unsigned int uzero = 0;
    cudaError_t e = cudaMemcpyToSymbol(g_gemm_status, &zero, sizeof(int));
    if (e == cudaSuccess) e = cudaMemcpyToSymbol(g_gemm_tp_ticket, &uzero, sizeof(unsigned int));
    return (int)e;
}

static void common_params(GemmParams& p, int m) {
    p.m = m;
    p.tiles_m = (m + BM - 1) / BM;
    p.nparts = 1;
    p.status = status_ptr();
    p.alpha = 1.0f;
    p.acc_chunk = 0;
    p.raw_fmt = 0;
    p.sync.wait_phase = p.sync.signal_phase = -1;
    static const bool early = getenv("VELOX_SM100_NO_EARLY_START") == nullptr;
    p.early = early ? 1 : 0;
}

// One NVFP4 view (or a gate / up pair) as part `pi` of a block-scaled launch: W geometry on parent
// row coordinates rounded down to a scale tile, outputs, and the optional NVFP4 producer epilogue.
static int nvfp4_part(const LinearArgs& a, GemmParams& p, GemmMaps& maps, int pi) {
    const velox_sm100_view& w = a.w;
    const bool sw = a.swiglu != 0;
    const velox_sm100_view& w1 = sw ? a.up : a.w;
    const long long k = w.k;
    PartParams& pp = p.part[pi];
    if (w.format != VELOX_FMT_NVFP4 || w1.format != VELOX_FMT_NVFP4) return VELOX_ERR_UNSUPPORTED;
    if (sw && (w.row_begin - w1.row_begin) % 128 != 0) return VELOX_ERR_UNSUPPORTED;
    pp.y = a.y;
    pp.yb = a.yb;
    pp.ld = a.ld;
    pp.col = a.col;
    const velox_sm100_view* hv[2] = {&w, &w1};
    for (int h = 0; h < 2; h++) {
        const velox_sm100_view& v = *hv[h];
        const long long plane = align256(v.n * k / 2);
        pp.sfb[h] = v.w + plane;
        pp.wdiv[h] = reinterpret_cast<const float*>(v.w + plane + v.n * k / 16);
        pp.b_rows_total[h] = v.n;
        pp.valid_begin[h] = v.row_begin;
        pp.valid_end[h] = v.row_begin + v.rows;
    }
    const long long base0 = w.row_begin / 128 * 128;
    if (sw) {
        pp.b_row0[0] = base0;
        pp.b_row0[1] = w1.row_begin - (w.row_begin - base0);
        pp.b_tile_rows = 128;
        pp.tiles_n = (int)((w.row_begin + w.rows - base0 + 127) / 128);
    } else {
        pp.b_row0[0] = base0;
        pp.b_row0[1] = base0 + 128;
        pp.b_tile_rows = 256;
        pp.tiles_n = (int)((w.row_begin + w.rows - base0 + 255) / 256);
    }
    pp.out_row0 = w.row_begin;
    if (a.qo_codes) {
        // whole 64-column pieces of whole rows of the quantised matrix, starting at column 0
        if (!a.qo_atoms || !(a.qo_divisor > 0.0f) || a.col != 0 || w.row_begin % 128 != 0 || w.rows % 64 != 0 ||
            (a.y != nullptr))
            return VELOX_ERR_UNSUPPORTED;
        pp.q_codes = a.qo_codes;
        pp.q_atoms = a.qo_atoms;
        pp.q_divisor = a.qo_divisor;
        pp.q_ld = w.rows;
    }
    int rc;
    if (sw) {
        if ((rc = make_map(&maps.b[0], w.w, false, w.n, k / 2)) != 0) return rc;
        if ((rc = make_map(&maps.b[1], w1.w, false, w1.n, k / 2)) != 0) return rc;
    } else {
        if ((rc = make_map(&maps.b[pi], w.w, false, w.n, k / 2)) != 0) return rc;
    }
    return 0;
}

// Several NVFP4 views of one width reading the same pre-quantised activations, as one launch: the
// tiles of the views are numbered one view after the other and walked by one persistent grid
// (Backend::linears, crates/velox-core/src/backend.rs:938-958, for the FP4 activation twins).
int gemm_linears_q4(const LinearArgs* parts, int n, float divisor, const velox_sm100_tp_sync* sync) {
    if (!gemm_available() || n < 1 || n > MAX_PARTS) return VELOX_ERR_UNSUPPORTED;
    const LinearArgs& a0 = parts[0];
    const long long k = a0.w.k;
    if (k % 64 != 0 || a0.m < 1 || !a0.q_codes || !a0.q_atoms) return VELOX_ERR_UNSUPPORTED;
    GemmParams p{};
    common_params(p, a0.m);
    if (!p.status) return VELOX_ERR_UNSUPPORTED;
    p.nparts = n;
    p.k_steps = (int)(k / 64);
    p.k_elems_per_block = 128;
    p.k_tiles64 = (int)(k / 64);
    p.k_blocks = (p.k_steps + 3) / 4;
    p.a_k_blocks = p.k_blocks;
    p.sfa = a0.q_atoms;
    p.alpha = 1.0f / divisor;
    int rc = tp_sync_fill(&p.sync, sync, ticket_ptr(), p.status);
    if (rc != 0) return rc;
    if (p.sync.signal_phase >= 0) return VELOX_ERR_UNSUPPORTED;   // only the scattering linear signals
    GemmMaps maps;
    CUtensorMap ma;
    long long out_cols[MAX_PARTS], first_row[MAX_PARTS];
    for (int i = 0; i < n; i++) {
        const LinearArgs& a = parts[i];
        if (a.swiglu || a.rs_maps || a.w.k != k || a.m != a0.m || a.q_codes != a0.q_codes || a.q_atoms != a0.q_atoms)
            return VELOX_ERR_UNSUPPORTED;
        if ((rc = nvfp4_part(a, p, maps, i)) != 0) return rc;
        out_cols[i] = a.w.rows;
        first_row[i] = a.w.row_begin;
    }
    if ((rc = make_map(&ma, a0.q_codes, false, a0.m, k / 2)) != 0) return rc;
    return launch<KIND_MXF4>(false, ma, maps, p, out_cols, first_row);
}

int gemm_linear(const LinearArgs& a, int act, float divisor) {
    if (!gemm_available()) return VELOX_ERR_UNSUPPORTED;
    const velox_sm100_view& w = a.w;
    const long long k = w.k;
    if (k % 64 != 0 || a.m < 1) return VELOX_ERR_UNSUPPORTED;
    const bool sw = a.swiglu != 0;
    const velox_sm100_view& w1 = sw ? a.up : a.w;

    GemmParams p{};
    common_params(p, a.m);
    if (!p.status) return VELOX_ERR_UNSUPPORTED;
    PartParams& pp = p.part[0];
    pp.y = a.y;
    pp.yb = a.yb;
    pp.ld = a.ld;
    pp.col = a.col;

    CUtensorMap ma;
    GemmMaps maps;
    int rc;
    if ((rc = tp_sync_fill(&p.sync, a.sync, ticket_ptr(), p.status)) != 0) return rc;
    if (a.sync && act != VELOX_ACT_NVFP4) return VELOX_ERR_UNSUPPORTED;

    if (act == VELOX_ACT_NVFP4) {
        const int mp = p.tiles_m * BM;
        const uint8_t* codes = a.q_codes;
        const uint8_t* atoms = a.q_atoms;
        if ((rc = nvfp4_part(a, p, maps, 0)) != 0) return rc;
        if (!codes || !atoms) {
            // no producer has quantised x already: do it here, into scratch
            uint8_t* c = static_cast<uint8_t*>(scratch(SCRATCH_ACT_CODES, (size_t)a.m * k / 2));
            uint8_t* s = static_cast<uint8_t*>(scratch(SCRATCH_ACT_SCALES, (size_t)mp * k / 16));
            if (!c || !s) return (int)cudaErrorMemoryAllocation;
            rc = quantize_act_nvfp4(a.x, a.xb, a.m, k, divisor, c, s);
            if (rc != 0) return rc;
            codes = c;
            atoms = s;
        }
        p.k_steps = (int)(k / 64);
        p.k_elems_per_block = 128;
        p.k_tiles64 = (int)(k / 64);
        p.sfa = atoms;
        p.alpha = 1.0f / divisor;
        if (a.rs_maps) {
            // whole tiles of whole rows into per-owner buffers: nothing ragged
            if (a.y || a.yb || a.qo_codes || a.col != 0 || w.row_begin != 0 || w.rows % 256 != 0 ||
                a.rs_rows_per_owner < 128 || a.rs_rows_per_owner % 128 != 0 || a.m % a.rs_rows_per_owner != 0)
                return VELOX_ERR_UNSUPPORTED;
            p.out_maps = static_cast<const CUtensorMap*>(a.rs_maps);
            p.rows_per_owner = a.rs_rows_per_owner;
        } else if (p.sync.signal_phase >= 0) {
            return VELOX_ERR_UNSUPPORTED;   // only the scattering linear signals
        }
        if ((rc = make_map(&ma, codes, false, a.m, k / 2)) != 0) return rc;
        p.k_blocks = (p.k_steps + 3) / 4;
        p.a_k_blocks = p.k_blocks;
        const long long oc = w.rows, fr = w.row_begin;
        return launch<KIND_MXF4>(sw, ma, maps, p, &oc, &fr);
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
            pp.col_scale[h] = reinterpret_cast<const uint16_t*>(v.w + align256(v.n * k));
            pp.b_rows_total[h] = v.n;
            pp.valid_begin[h] = v.row_begin;
            pp.valid_end[h] = v.row_begin + v.rows;
        }
        pp.b_row0[0] = w.row_begin;
        pp.b_row0[1] = sw ? w1.row_begin : w.row_begin + 128;
        pp.b_tile_rows = sw ? 128 : 256;
        pp.tiles_n = (int)((w.rows + pp.b_tile_rows - 1) / pp.b_tile_rows);
        pp.out_row0 = w.row_begin;
        if ((rc = make_map(&ma, codes, false, a.m, k)) != 0) return rc;
        if ((rc = make_map(&maps.b[0], w.w, false, w.n, k)) != 0) return rc;
        if ((rc = make_map(&maps.b[1], w1.w, false, w1.n, k)) != 0) return rc;
        p.k_blocks = (p.k_steps + 3) / 4;
        p.a_k_blocks = p.k_blocks;
        if (p.k_blocks > 4) p.acc_chunk = 4;   // (see the bf16 kind below: sums of 512 products, then f32 adds)
        const long long oc = w.rows, fr = 0;
        return launch<KIND_F8>(sw, ma, maps, p, &oc, &fr);
    }

    if (act != VELOX_ACT_BF16) return VELOX_ERR_UNSUPPORTED;
    // bf16 activations x weights dequantised to bf16 in scratch (view rows only, row 0 = row_begin).
    // Q4_K values are not bf16 numbers: they go in as three bf16 terms side by side along K
    // ([rows, 3k]: bf16(v), bf16 of what that dropped, bf16 of what is left; together the f32 value
    // exactly), each multiplied by the same activations, which the producer re-reads for every
    // third. Two terms (2^-17) were not enough for the 2e-4 conformance bound on sums that cancel.
    const bool split = w.format == VELOX_FMT_GGML_Q4_K;
    const long long kw = split ? 3 * k : k;
    // FP8 rows above one token tile (CTA pairs): no scratch at all; the kernel converts the stored
    // bytes on their way into the operand stage.
    const bool raw = w.format == VELOX_FMT_FP8_ROW_BF16 && a.m > BM && k % 64 == 0 &&
                     (!sw || w1.format == VELOX_FMT_FP8_ROW_BF16);
    uint16_t* wq = nullptr;
    if (!raw) {
        const size_t wbytes = (size_t)w.rows * kw * 2;
        wq = static_cast<uint16_t*>(scratch(SCRATCH_WEIGHT_BF16, wbytes * (sw ? 2 : 1)));
        if (!wq) return (int)cudaErrorMemoryAllocation;
        if ((rc = dequant_rows_bf16(&w, wq, kw, split ? k : 0)) != 0) return rc;
        if (sw && (rc = dequant_rows_bf16(&w1, wq + (size_t)w.rows * kw, kw, split ? k : 0)) != 0) return rc;
    }
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
    // The tensor cores' running f32 sum truncates, and over a long K that bias reaches the fourth
    // digit of sums that cancel (Q4_K blocks with values up to 30 at K = 2560, FP8 rows at K = 8192):
    // four k-blocks per accumulator, the chunks added by the epilogue with ordinary f32 adds (eight
    // k-blocks per chunk failed the bound on the K = 8192 case).
    if (kw > 4 * 64) p.acc_chunk = 4;
    const velox_sm100_view* hv[2] = {&w, &w1};
    if ((rc = make_map(&ma, xb, true, a.m, k)) != 0) return rc;
    if (raw) {
        // parent coordinates, as in the FP8 kind: the maps describe the stored code planes
        p.raw_fmt = 1;
        for (int h = 0; h < 2; h++) {
            const velox_sm100_view& v = *hv[h];
            pp.col_scale[h] = reinterpret_cast<const uint16_t*>(v.w + align256(v.n * k));
            pp.b_rows_total[h] = v.n;
            pp.valid_begin[h] = v.row_begin;
            pp.valid_end[h] = v.row_begin + v.rows;
        }
        pp.b_row0[0] = w.row_begin;
        pp.b_row0[1] = sw ? w1.row_begin : w.row_begin + 128;
        pp.out_row0 = w.row_begin;
        if ((rc = make_raw_map(&maps.b[0], w.w, w.n, k)) != 0) return rc;
        if ((rc = make_raw_map(&maps.b[1], w1.w, w1.n, k)) != 0) return rc;
    } else {
        for (int h = 0; h < 2; h++) {
            const velox_sm100_view& v = *hv[h];
            if (v.format == VELOX_FMT_NVFP4)
                pp.wdiv[h] = reinterpret_cast<const float*>(v.w + align256(v.n * k / 2) + v.n * k / 16);
            if (v.format == VELOX_FMT_FP8_ROW_BF16)
                pp.col_scale[h] = reinterpret_cast<const uint16_t*>(v.w + align256(v.n * k)) + v.row_begin;
            pp.b_rows_total[h] = v.rows;
            pp.valid_begin[h] = 0;
            pp.valid_end[h] = v.rows;
        }
        pp.b_row0[0] = 0;
        pp.b_row0[1] = sw ? 0 : 128;
        pp.out_row0 = 0;
        if ((rc = make_map(&maps.b[0], wq, true, w.rows, kw)) != 0) return rc;
        if ((rc = make_map(&maps.b[1], sw ? wq + (size_t)w.rows * kw : wq, true, w.rows, kw)) != 0) return rc;
    }
    pp.b_tile_rows = sw ? 128 : 256;
    pp.tiles_n = (int)((w.rows + pp.b_tile_rows - 1) / pp.b_tile_rows);
    p.k_blocks = (p.k_steps + 3) / 4;
    const long long oc = w.rows, fr = 0;
    return launch<KIND_BF16>(sw, ma, maps, p, &oc, &fr);
}

}  // namespace vx

// ---- prefill linear for callers that cannot allocate ------------------------------------------------
//
// The NVFP4 prefill path needs room for the quantised activations (codes and scale atoms). The
// regular entry points take it from grow-only cudaMalloc'd scratch; this one keeps it in a fixed
// array that is part of the library image, so nothing is allocated at any point.

namespace vx {

constexpr size_t STATIC_SCRATCH_BYTES = 8u << 20;  // 8 MiB per device, held until the process exits
static __device__ __align__(256) uint8_t g_static_act_scratch[STATIC_SCRATCH_BYTES];

// Device address of the array, per device ordinal. In host code the array's name is only a handle
// for the runtime, not an address a kernel can use, so it is resolved once per device here.
static uint8_t* g_static_scratch_ptr[64] = {};
static int* g_static_status_ptr[64] = {};
static std::mutex g_static_mu;

static int static_scratch_setup(int dev, uint8_t** scratch_out, int** status_out) {
    std::lock_guard<std::mutex> lock(g_static_mu);
    if (!g_static_scratch_ptr[dev]) {
        void* ptr = nullptr;
        cudaError_t e = cudaGetSymbolAddress(&ptr, g_static_act_scratch);
        if (e != cudaSuccess) return (int)e;
        void* st = nullptr;
        e = cudaGetSymbolAddress(&st, g_gemm_status);
        if (e != cudaSuccess) return (int)e;
        g_static_scratch_ptr[dev] = static_cast<uint8_t*>(ptr);
        g_static_status_ptr[dev] = static_cast<int*>(st);
    }
    *scratch_out = g_static_scratch_ptr[dev];
    *status_out = g_static_status_ptr[dev];
    return 0;
}

}  // namespace vx

extern "C" int velox_sm100_linear_nvfp4_a4_static(const uint16_t* xb, const velox_sm100_view* view, int m,
                                                  float* y, uint16_t* yb) {
    using namespace vx;
    if (!xb || (!y && !yb) || m <= 0) return VELOX_ERR_SHAPE;
    int rc = check_view(view);
    if (rc != 0) return rc;
    const velox_sm100_view& w = *view;
    if (w.format != VELOX_FMT_NVFP4 || w.policy != VELOX_POLICY_ALLOW_A4 || !(w.divisor > 0.0f) || m <= 16)
        return VELOX_ERR_UNSUPPORTED;
    if (!gemm_available()) return VELOX_ERR_UNSUPPORTED;
    const long long k = w.k;
    const int tiles_m = (m + BM - 1) / BM;
    const size_t code_bytes = ((size_t)m * k / 2 + 255) / 256 * 256;
    const size_t atom_bytes = (size_t)tiles_m * BM * k / 16;
    if (code_bytes + atom_bytes > STATIC_SCRATCH_BYTES) return VELOX_ERR_STATIC_SCRATCH;

    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return (int)e;
    if (dev < 0 || dev >= 64) return VELOX_ERR_UNSUPPORTED;
    uint8_t* scratch_base = nullptr;
    int* status = nullptr;
    if ((rc = static_scratch_setup(dev, &scratch_base, &status)) != 0) return rc;
    uint8_t* codes = scratch_base;
    uint8_t* atoms = scratch_base + code_bytes;
    // Every byte the GEMM reads is rewritten here: codes of rows < m, and the scale atoms of all
    // tiles_m * 128 rows (zeros past m). Nothing left over from an earlier call is consumed.
    if ((rc = quantize_act_nvfp4_untimed(xb, m, k, w.divisor, codes, atoms)) != 0) return rc;

    GemmParams p{};
    p.m = m;
    p.tiles_m = tiles_m;
    p.nparts = 1;
    p.status = status;
    p.sync.wait_phase = p.sync.signal_phase = -1;
    p.k_steps = (int)(k / 64);
    p.k_blocks = (p.k_steps + 3) / 4;
    p.a_k_blocks = p.k_blocks;
    p.k_elems_per_block = 128;
    p.k_tiles64 = (int)(k / 64);
    p.sfa = atoms;
    p.alpha = 1.0f / w.divisor;
    LinearArgs a{};
    a.w = w;
    a.m = m;
    a.y = y;
    a.yb = yb;
    a.ld = w.rows;
    a.col = 0;
    GemmMaps maps;
    CUtensorMap ma;
    if ((rc = nvfp4_part(a, p, maps, 0)) != 0) return rc;
    if ((rc = make_map(&ma, codes, false, m, k / 2)) != 0) return rc;
    for (int i = 1; i < MAX_PARTS; i++) maps.b[i] = maps.b[0];
    for (int i = 0; i < MAX_PARTS; i++) maps.out[i] = ma;
    make_out_map(&maps.out[0], m, p.part[0], w.rows, w.row_begin);
    int sms = 0;
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
    if (sms <= 0) sms = 148;
    const int tiles = p.tiles_m * p.part[0].tiles_n;
    p.part[0].tile_end = tiles;
    auto kern = gemm_kernel<KIND_MXF4, false, 1>;
    e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, Plan<1>::SMEM_BYTES);
    if (e != cudaSuccess) return (int)e;
    kern<<<tiles < sms ? tiles : sms, GEMM_THREADS, Plan<1>::SMEM_BYTES, stream()>>>(ma, maps, p);
    return launch_status();
}
