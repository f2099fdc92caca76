// Decode and small-batch linear (m <= 64 tokens) on the tensor cores: NVFP4 weights (block-scaled MMA) and FP8 rows.
//
// Decode is a byte stream: 0.5625 B per weight, every byte once. The SIMT/mma.sync GEMV spends
// about 1.6 issue slots per weight on unpacking (E2M1 -> f16, times the block scale) and is bound
// by instruction issue near half the copy rate. Here nothing is unpacked: a persistent CTA per SM
// streams 128-row x 256-k tiles of the stored codes (16 KB, one tensor-map box) and their four
// 512-byte scale atoms into shared memory, and tcgen05.mma kind::mxf4nvf4 consumes them as they
// are - weight rows are the MMA M operand (128), the tokens the N operand (16 or 64, zero padded), the
// activations NVFP4 with the view's per-tensor divisor (ActQuant::Nvfp4, which the view's AllowA4
// policy admits at any m). An MMA of this shape takes a few tens of cycles, so a CTA is idle
// unless bytes arrive: the ring (eight stages of 18 KB, or 24 KB with 64 token columns) is what sets
// the speed.
//
// Work is cut by bytes, not by tiles: the (tile, k-block) steps of the whole matrix are laid end to
// end and every CTA takes an equal contiguous run of them, so a run starts and ends inside tiles.
// A CTA that holds only part of a tile's K parks f32 partial sums; the CTA that arrives last at
// the tile adds the parts in K order, so the result does not depend on arrival order. Roles:
//   warp 0      operand producer (TMA: W codes box + the x codes box, 16 or 64 rows);
//   warp 1      MMA issuer (one elected lane), accumulators double-buffered in tensor memory;
//   warp 2      scale producer (bulk copies of whole atoms, W then x);
//   warps 4-7   epilogue: tcgen05.ld, K-split fix-up, per-tensor factors, optional silu(gate)*up, and
//               optionally the result as the next linear's NVFP4 input; one rolled code instance,
//               because this code runs once or twice per CTA and cold instruction lines cost as
//               much as memory round trips;
//   warps 8-11  scale movers: shared memory -> tensor memory (tcgen05.st), one per lane quadrant.
// FP8-E4M3 rows with FP8-row activations (ActQuant::Fp8Row, views that admit it) take the same
// route without the scale roles: kind::f8f6f4, 128 k per stage, the bf16 row scale and the f32
// token scale applied in the epilogue.
// Every mbarrier wait is bounded; a wait that gives up records a code in the status word.
//
// Reference counterpart: linear_gemv_vec_kernel, crates/velox-cuda/kernels/portable_model.cu:1448-1626.
#include <cstdlib>
#include <mutex>

#include "common.cuh"
#include "gemm.cuh"
#include "kernels.cuh"
#include "tcgen.cuh"

namespace vx {

constexpr int DT_STAGES = 8;
constexpr int DT_W_BYTES = 128 * 128;   // 128 weight rows x 128 bytes (256 k)
constexpr int DT_SF_STAGE_BYTES = 2048 + 2048;   // four W atoms, four x atoms
constexpr int DT_THREADS = 384;
constexpr int DT_TMEM_COLS = 512;
constexpr int DT_SF_SET = 32;        // per set: 16 columns of W scales, 16 of x scales

// Sizes that depend on the token capacity NT of a launch (the MMA N extent): 16 for decode proper,
// 64 for small batches (speculative decode, short prefills), which are still a weight stream.
template <int NT>
struct DtPlan {
    static constexpr int X_BYTES = NT * 128;                    // NT token rows x 128 bytes
    static constexpr int STAGE_BYTES = DT_W_BYTES + X_BYTES;    // 18 KB / 24 KB
    static constexpr int OFF_SF = DT_STAGES * STAGE_BYTES;
    static constexpr int OFF_BARS = OFF_SF + DT_STAGES * DT_SF_STAGE_BYTES;
    static constexpr int SMEM_BYTES = OFF_BARS + 1024 + 512;
    static constexpr int ACC_COLS = 2 * NT;                     // per buffer: NT token columns for each of two passes
    static constexpr int SF_COL = 2 * ACC_COLS;                 // scale sets follow the two accumulator buffers
    static_assert(SF_COL + DT_STAGES * DT_SF_SET <= DT_TMEM_COLS, "tensor memory plan");
    static_assert(SMEM_BYTES <= 232448, "shared memory plan");
};

constexpr int DT_MAX_PARTS = 3;   // views served by one launch (q, k, v of one input)

// Where one view's results go.
struct DtOut {
    long long valid_begin, valid_end;   // rows of the view, parent coordinates
    float* y;
    uint16_t* yb;
    long long ld, col;
    uint8_t* q_codes;            // optional: the result also (or only) as NVFP4 activations [m, q_ld / 2] ...
    uint8_t* q_atoms;            // ... with their scale atoms, for the next linear
    float q_divisor;
    long long q_ld;
};

struct DtParams {
    int m;
    int k_blocks, k_steps;
    long long k_tiles64;
    // Plain form: up to three views of the same width sharing the activations, their 128-row tiles
    // numbered one view after the other. SwiGLU form: entries 0 and 1 are gate and up of one
    // output (out[0]), walked as two passes over the same tile index.
    int nparts;
    int part_tiles[DT_MAX_PARTS];
    long long tile0[DT_MAX_PARTS];      // first 128-row tile (parent coordinates)
    const uint8_t* sfw[DT_MAX_PARTS];
    const float* wdiv[DT_MAX_PARTS];
    DtOut out[DT_MAX_PARTS];
    int tiles;                   // all parts together
    long long per_cta;           // (tile, k-block) steps per CTA; CTA c takes steps [c * per_cta, (c + 1) * per_cta)
    const uint8_t* sfx;
    float alpha;                 // 1 / activation divisor
    const uint16_t* rowscale[DT_MAX_PARTS];   // FP8 rows: bf16 scale per weight row
    const float* tokscale;                     // FP8 rows: f32 scale per token
    float* partial;              // [CTAs][2][V][NT/16][128][16]: a CTA's first and last run can be partial tiles
    int* tickets;                // [tiles], zero between launches
    int* status;
};

__device__ int g_gemv_tc_status = 0;

template <bool SWIGLU, int KIND, int NT>
__global__ void __launch_bounds__(DT_THREADS, 1)
gemv_nvfp4_tc_kernel(const __grid_constant__ CUtensorMap map_w0, const __grid_constant__ CUtensorMap map_w1,
                     const __grid_constant__ CUtensorMap map_w2, const __grid_constant__ CUtensorMap map_x,
                     const DtParams p) {
    constexpr int V = SWIGLU ? 2 : 1;
    using PL = DtPlan<NT>;
    constexpr int DT_STAGE_BYTES = PL::STAGE_BYTES;
    constexpr int DT_ACC_COLS = PL::ACC_COLS;
    constexpr int DT_SF_COL = PL::SF_COL;
    extern __shared__ uint8_t smem_raw[];
    const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    const uint32_t sf_ring = base + PL::OFF_SF;
    const uint32_t bars = base + PL::OFF_BARS;
    auto op_full = [&](int s) { return bars + 8u * s; };
    auto op_empty = [&](int s) { return bars + 8u * (DT_STAGES + s); };
    auto sf_full = [&](int s) { return bars + 8u * (2 * DT_STAGES + s); };
    auto sf_empty = [&](int s) { return bars + 8u * (3 * DT_STAGES + s); };
    auto tsf_full = [&](int s) { return bars + 8u * (4 * DT_STAGES + s); };
    auto tsf_empty = [&](int s) { return bars + 8u * (5 * DT_STAGES + s); };
    auto acc_full = [&](int b) { return bars + 8u * (6 * DT_STAGES + b); };
    auto acc_empty = [&](int b) { return bars + 8u * (6 * DT_STAGES + 2 + b); };
    const uint32_t tmem_slot = bars + 8u * (6 * DT_STAGES + 4);
    const uint32_t flag_slot = tmem_slot + 8u;   // "this CTA finishes the tile", shared by the epilogue warps
    uint32_t* tmem_slot_ptr = reinterpret_cast<uint32_t*>(smem_raw + (tmem_slot - smem_u32(smem_raw)));
    volatile uint32_t* flag_ptr = reinterpret_cast<volatile uint32_t*>(smem_raw + (flag_slot - smem_u32(smem_raw)));

    const int warp = threadIdx.x / 32, lane = threadIdx.x % 32;

    // A kernel launched after this one with early start allowed may begin as CTAs here retire.
    if (threadIdx.x == 0) grid_launch_dependents();

    if (threadIdx.x == 0) {
        for (int s = 0; s < DT_STAGES; s++) {
            mbar_init(op_full(s), 1);
            mbar_init(op_empty(s), 1);
            mbar_init(sf_full(s), 1);
            mbar_init(sf_empty(s), 4);
            mbar_init(tsf_full(s), 4);
            mbar_init(tsf_empty(s), 1);
        }
        for (int b = 0; b < 2; b++) {
            mbar_init(acc_full(b), 1);
            mbar_init(acc_empty(b), 4);
        }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("prefetch.tensormap [%0];" ::"l"(&map_w0) : "memory");
        asm volatile("prefetch.tensormap [%0];" ::"l"(&map_w1) : "memory");
        asm volatile("prefetch.tensormap [%0];" ::"l"(&map_w2) : "memory");
        asm volatile("prefetch.tensormap [%0];" ::"l"(&map_x) : "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(tmem_slot),
                     "r"((uint32_t)DT_TMEM_COLS)
                     : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = *tmem_slot_ptr;

    // This CTA's run of steps, walked tile by tile: each piece is (tile, k-blocks [kb0, kb1)).
    const long long total_steps = (long long)p.tiles * p.k_blocks;
    const long long u_begin = (long long)blockIdx.x * p.per_cta;
    const long long u_end = u_begin + p.per_cta < total_steps ? u_begin + p.per_cta : total_steps;
    struct Piece { int tile, kb0, kb1; };
    auto piece_at = [&](long long u) {
        Piece q;
        q.tile = (int)(u / p.k_blocks);
        q.kb0 = (int)(u % p.k_blocks);
        const long long left = u_end - u;
        q.kb1 = q.kb0 + left < p.k_blocks ? (int)(q.kb0 + left) : p.k_blocks;
        return q;
    };

    // which view a tile belongs to, and its index among that view's tiles (plain form)
    auto part_of = [&](int tile, int& local) {
        int part = 0;
        local = tile;
        while (part + 1 < p.nparts && local >= p.part_tiles[part]) {
            local -= p.part_tiles[part];
            part++;
        }
        return part;
    };

    if (warp == 0) {
        // ---------------- operand producer ----------------
        int stage = 0;
        uint32_t phase = 0;
        bool ok = true;
        const bool leader = elect_one();
        // The weights do not depend on the kernel before this one, the activations do: the first
        // ring pass requests its weight boxes at once, then waits for the preceding grid (a
        // no-op unless this launch was allowed to start early) and adds the activation boxes.
        int issued = 0, pend_kb[DT_STAGES];
        bool waited = false;
        auto after_dependency = [&]() {
            grid_dependency_wait();
            if (leader)
                for (int i = 0; i < issued; i++)
                    tma_load_2d(base + i * DT_STAGE_BYTES + DT_W_BYTES, &map_x, op_full(i), pend_kb[i] * 128, 0);
            waited = true;
        };
        for (long long u = u_begin; u < u_end && ok;) {
            const Piece pc = piece_at(u);
            const int tile = pc.tile, kb0 = pc.kb0, kb1 = pc.kb1;
            u += kb1 - kb0;
            for (int v = 0; v < V && ok; v++) {
                int lt = tile;
                const int idx = SWIGLU ? v : part_of(tile, lt);
                const int row0 = (int)((p.tile0[idx] + lt) * 128);
                const CUtensorMap* mw = idx == 0 ? &map_w0 : idx == 1 ? &map_w1 : &map_w2;
                for (int kb = kb0; kb < kb1; kb++) {
                    if (!waited && issued == DT_STAGES) after_dependency();
                    if (!mbar_wait(op_empty(stage), phase ^ 1u, 20)) {
                        if (leader) atomicExch(p.status, 21);
                        ok = false;
                        break;
                    }
                    const uint32_t sw = base + stage * DT_STAGE_BYTES;
                    if (leader) {
                        mbar_arrive_expect_tx(op_full(stage), DT_STAGE_BYTES);
                        tma_load_2d(sw, mw, op_full(stage), kb * 128, row0);
                        if (waited) tma_load_2d(sw + DT_W_BYTES, &map_x, op_full(stage), kb * 128, 0);
                    }
                    if (!waited) pend_kb[issued++] = kb;
                    if (++stage == DT_STAGES) {
                        stage = 0;
                        phase ^= 1u;
                    }
                }
            }
        }
        if (!waited) after_dependency();
        if (!ok) __nanosleep(200000);   // let copies already in flight land before the CTA exits
    } else if (warp == 1) {
        // ---------------- MMA issuer ----------------
        int stage = 0;
        uint32_t phase = 0;
        bool ok = true;
        const bool leader = elect_one();
        // M = 128, N = NT, E2M1 x E2M1 with UE4M3 block scales, K-major operands, f32 accumulate
        const uint32_t shape = ((uint32_t)(NT >> 3) << 17) | ((uint32_t)(128 >> 4) << 24);
        const uint32_t idesc = KIND == KIND_MXF4 ? ((1u << 7) | (1u << 10) | shape)   // E2M1 x E2M1, UE4M3 scales
                                                 : ((1u << 4) | shape);                // E4M3 x E4M3 -> f32
        int n = 0;
        for (long long u = u_begin; u < u_end && ok; n++) {
            const Piece pc = piece_at(u);
            const int kb0 = pc.kb0, kb1 = pc.kb1;
            u += kb1 - kb0;
            const int buf = n & 1;
            if (!mbar_wait(acc_empty(buf), ((uint32_t)(n >> 1) & 1u) ^ 1u)) {
                if (leader) atomicExch(p.status, 22);
                break;
            }
            for (int v = 0; v < V && ok; v++) {
                const uint32_t d = tmem + buf * DT_ACC_COLS + v * NT;
                for (int kb = kb0; kb < kb1; kb++) {
                    if (!mbar_wait(op_full(stage), phase) || (KIND == KIND_MXF4 && !mbar_wait(tsf_full(stage), phase))) {
                        if (leader) atomicExch(p.status, 23);
                        ok = false;
                        break;
                    }
                    tc_fence_after();
                    const int steps = min(4, p.k_steps - 4 * kb);
                    const uint32_t sw = base + stage * DT_STAGE_BYTES;
                    const uint64_t da = smem_desc_sw128(sw), db = smem_desc_sw128(sw + DT_W_BYTES);
                    const uint32_t tsf = tmem + DT_SF_COL + stage * DT_SF_SET;
                    if (leader) {
                        for (int j = 0; j < steps; j++)
                            tc_mma<KIND, 1>(d, da + 2u * j, db + 2u * j, idesc, (kb != kb0 || j != 0) ? 1u : 0u,
                                                 tsf + 4 * j, tsf + 16 + 4 * j);
                        tc_commit(op_empty(stage));
                        if (KIND == KIND_MXF4) tc_commit(tsf_empty(stage));
                    }
                    if (++stage == DT_STAGES) {
                        stage = 0;
                        phase ^= 1u;
                    }
                }
            }
            if (ok && leader) tc_commit(acc_full(buf));
        }
    } else if (KIND == KIND_MXF4 && warp == 2) {
        // ---------------- scale producer ----------------
        // (weight atoms at once, activation atoms after the preceding grid, as the operand producer)
        int stage = 0;
        uint32_t phase = 0;
        bool ok = true;
        const bool leader = elect_one();
        int issued = 0, pend_kb[DT_STAGES];
        bool waited = false;
        auto x_atoms = [&](int st, int kb) {
            const uint32_t bytes = (uint32_t)min(4, p.k_steps - 4 * kb) * 512u;
            bulk_load_1d(sf_ring + st * DT_SF_STAGE_BYTES + 2048, p.sfx + 4LL * kb * 512, bytes, sf_full(st));
        };
        auto after_dependency = [&]() {
            grid_dependency_wait();
            if (leader)
                for (int i = 0; i < issued; i++) x_atoms(i, pend_kb[i]);
            waited = true;
        };
        for (long long u = u_begin; u < u_end && ok;) {
            const Piece pc = piece_at(u);
            const int tile = pc.tile, kb0 = pc.kb0, kb1 = pc.kb1;
            u += kb1 - kb0;
            for (int v = 0; v < V && ok; v++) {
                int lt = tile;
                const int idx = SWIGLU ? v : part_of(tile, lt);
                const uint8_t* wsf = p.sfw[idx] + (p.tile0[idx] + lt) * p.k_tiles64 * 512;
                for (int kb = kb0; kb < kb1; kb++) {
                    if (!waited && issued == DT_STAGES) after_dependency();
                    if (!mbar_wait(sf_empty(stage), phase ^ 1u, 50)) {
                        if (leader) atomicExch(p.status, 24);
                        ok = false;
                        break;
                    }
                    const uint32_t bytes = (uint32_t)min(4, p.k_steps - 4 * kb) * 512u;
                    const uint32_t dst = sf_ring + stage * DT_SF_STAGE_BYTES;
                    if (leader) {
                        mbar_arrive_expect_tx(sf_full(stage), 2 * bytes);
                        bulk_load_1d(dst, wsf + 4LL * kb * 512, bytes, sf_full(stage));
                        if (waited) x_atoms(stage, kb);
                    }
                    if (!waited) pend_kb[issued++] = kb;
                    if (++stage == DT_STAGES) {
                        stage = 0;
                        phase ^= 1u;
                    }
                }
            }
        }
        if (!waited) after_dependency();
        if (!ok) __nanosleep(200000);
    } else if (KIND == KIND_MXF4 && warp >= 8) {
        // ---------------- scale movers ----------------
        // Lane i of the warp serving lane quadrant q writes atom rows i, i+32, i+64, i+96: the 16
        // bytes of atom row i are that atom's four 32-bit columns, replicated in every quadrant.
        const int quad = warp % 4;
        int stage = 0;
        uint32_t phase = 0;
        bool ok = true;
        {
            // one pass over this CTA's steps: the ring does not care where tiles begin
            const long long count = (u_end > u_begin ? u_end - u_begin : 0) * V;
            for (long long i = 0; i < count; i++) {
                if (!mbar_wait(sf_full(stage), phase, 50)) {
                    if (lane == 0) atomicExch(p.status, 25);
                    ok = false;
                    break;
                }
                const uint32_t src = sf_ring + stage * DT_SF_STAGE_BYTES + (uint32_t)lane * 16u;
                uint32_t ra[16], rb[16];
#pragma unroll
                for (int j = 0; j < 4; j++) {
                    const uint4 a = lds16(src + 512 * j);
                    const uint4 b = lds16(src + 2048 + 512 * j);
                    ra[4 * j] = a.x; ra[4 * j + 1] = a.y; ra[4 * j + 2] = a.z; ra[4 * j + 3] = a.w;
                    rb[4 * j] = b.x; rb[4 * j + 1] = b.y; rb[4 * j + 2] = b.z; rb[4 * j + 3] = b.w;
                }
                // the stage goes back to a writer of the async proxy (bulk copies): order these
                // generic-proxy reads ahead of it before the arrive (a copy landing while a lane's
                // load was in flight corrupted scales in the prefill GEMM, which shares this scheme)
                asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
                __syncwarp();
                if (lane == 0) mbar_arrive(sf_empty(stage));
                // the MMAs that read this column set one ring pass ago must have completed
                if (!mbar_wait(tsf_empty(stage), phase ^ 1u, 50)) {
                    if (lane == 0) atomicExch(p.status, 26);
                    ok = false;
                    break;
                }
                tc_fence_after();
                const uint32_t tsf = tmem + ((uint32_t)(quad * 32) << 16) + DT_SF_COL + stage * DT_SF_SET;
                tc_st16(tsf, ra);
                tc_st16(tsf + 16, rb);
                tc_wait_st();
                tc_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive(tsf_full(stage));
                if (++stage == DT_STAGES) {
                    stage = 0;
                    phase ^= 1u;
                }
            }
        }
    } else if (warp >= 4 && warp < 8) {
        // ---------------- epilogue ----------------
        const int quad = warp % 4;
        const int row_in_tile = quad * 32 + lane;
        int n = 0;
        for (long long u = u_begin; u < u_end; n++) {
            const Piece pc = piece_at(u);
            const int tile = pc.tile;
            const bool whole = pc.kb0 == 0 && pc.kb1 == p.k_blocks;
            const bool first_piece = u == u_begin;
            u += pc.kb1 - pc.kb0;
            const int buf = n & 1;
            if (!mbar_wait(acc_full(buf), (uint32_t)(n >> 1) & 1u, 60)) {
                if (lane == 0) atomicExch(p.status, 27);
                break;
            }
            tc_fence_after();
            const uint32_t taddr = tmem + ((uint32_t)(quad * 32) << 16) + buf * DT_ACC_COLS;
            constexpr int NC = NT / 16;                         // token chunks of 16 accumulator columns
            const int chunks = (p.m + 15) / 16;                 // ... of which this many hold tokens

            int lt = tile;
            const int idx = SWIGLU ? 0 : part_of(tile, lt);
            const DtOut& o = p.out[idx];
            const long long row = (p.tile0[idx] + lt) * 128 + row_in_tile;
            const bool row_ok = row >= o.valid_begin && row < o.valid_end;
            const long long o0 = o.col + (row - o.valid_begin);
            float f0, f1 = 0.0f;
            if (KIND == KIND_MXF4) {
                f0 = p.alpha / *p.wdiv[idx];
                if (SWIGLU) f1 = p.alpha / *p.wdiv[1];
            } else {
                // row scales; the matching up row sits at the same offset from its view's start
                f0 = row_ok ? bf16_bits_to_f32(p.rowscale[idx][row]) : 0.0f;
                if (SWIGLU) f1 = row_ok ? bf16_bits_to_f32(p.rowscale[1][(p.tile0[1] + lt) * 128 + row_in_tile]) : 0.0f;
            }
            auto release_acc = [&]() {
                tc_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive(acc_empty(buf));
            };
            // The code below runs once or twice per CTA, so it is written for few instructions
            // rather than few cycles: fetching a cold instruction line costs about as much as a
            // trip to memory, and an unrolled 16-token body was most of this kernel's per-token
            // cost. Loops are kept rolled; the per-token values go through a small local array.
            const size_t slot_floats = (size_t)V * NC * 128 * 16;
            const long long t0 = (long long)tile * p.k_blocks, t1 = t0 + p.k_blocks;
            const int c_first = (int)(t0 / p.per_cta), c_last = (int)((t1 - 1) / p.per_cta);
            if (!whole) {
                // Part of a tile's K: park the partial sums; the CTA that arrives last at the tile adds
                // the pieces in K order (which is CTA order) and finishes. The tile's pieces belong to
                // CTAs c_first .. c_last; a CTA's piece of a tile is its first piece exactly when its
                // run starts inside that tile, otherwise it is its last.
                float* mine = p.partial + ((size_t)blockIdx.x * 2 + (first_piece ? 0 : 1)) * slot_floats;
#pragma unroll 1
                for (int c = 0; c < chunks; c++) {
                    uint32_t r[V][16];
#pragma unroll
                    for (int v = 0; v < V; v++) tc_ld16(taddr + v * NT + c * 16, r[v]);
                    tc_wait_ld();
#pragma unroll
                    for (int v = 0; v < V; v++) {
                        uint4* dstp = reinterpret_cast<uint4*>(mine + (((size_t)v * NC + c) * 128 + row_in_tile) * 16);
#pragma unroll
                        for (int q = 0; q < 4; q++)
                            dstp[q] = make_uint4(r[v][4 * q], r[v][4 * q + 1], r[v][4 * q + 2], r[v][4 * q + 3]);
                    }
                }
                release_acc();
                __threadfence();
                asm volatile("bar.sync 1, 128;" ::: "memory");
                if (warp == 4 && lane == 0) {
                    const int prev = atomicAdd(p.tickets + tile, 1);
                    const bool last = prev == c_last - c_first;
                    if (last) p.tickets[tile] = 0;   // back to zero for the next launch
                    *flag_ptr = last ? 1u : 0u;
                }
                asm volatile("bar.sync 1, 128;" ::: "memory");
                const bool finish = *flag_ptr != 0u;
                asm volatile("bar.sync 1, 128;" ::: "memory");   // the flag is read before it is rewritten
                if (!finish) continue;
                __threadfence();
            }

            float* const oy = o.y;
            uint16_t* const oyb = o.yb;
            const long long old = o.ld;
            uint8_t* const oq_codes = o.q_codes;
            uint8_t* const oq_atoms = o.q_atoms;
            const float oq_div = o.q_divisor;
            const long long oq_ld = o.q_ld;
#pragma unroll 1
            for (int c = 0; c < chunks; c++) {
                float sum[V][16];   // tokens 16 c .. 16 c + 15 of this lane's weight row
                if (whole) {
                    uint32_t r[V][16];
#pragma unroll
                    for (int v = 0; v < V; v++) tc_ld16(taddr + v * NT + c * 16, r[v]);
                    tc_wait_ld();
                    if (c == chunks - 1) release_acc();
#pragma unroll
                    for (int v = 0; v < V; v++)
#pragma unroll
                        for (int j = 0; j < 16; j++) sum[v][j] = __uint_as_float(r[v][j]);
                } else {
#pragma unroll
                    for (int v = 0; v < V; v++)
#pragma unroll
                        for (int j = 0; j < 16; j++) sum[v][j] = 0.0f;
                    // several CTAs' slots per pass, so that their loads are in flight together
                    constexpr int B = V == 1 ? 4 : 2;
#pragma unroll 1
                    for (int cta0 = c_first; cta0 <= c_last; cta0 += B) {
                        float4 t[B][V][4];
#pragma unroll
                        for (int b = 0; b < B; b++) {
                            const int cta = cta0 + b <= c_last ? cta0 + b : c_last;   // (a repeat is not added)
                            const int slot = (long long)cta * p.per_cta >= t0 ? 0 : 1;
                            const float* theirs = p.partial + ((size_t)cta * 2 + slot) * slot_floats;
#pragma unroll
                            for (int v = 0; v < V; v++) {
                                const float4* src = reinterpret_cast<const float4*>(
                                    theirs + (((size_t)v * NC + c) * 128 + row_in_tile) * 16);
#pragma unroll
                                for (int q = 0; q < 4; q++) t[b][v][q] = __ldcg(src + q);
                            }
                        }
#pragma unroll
                        for (int b = 0; b < B; b++)
                            if (cta0 + b <= c_last) {
#pragma unroll
                                for (int v = 0; v < V; v++)
#pragma unroll
                                    for (int q = 0; q < 4; q++) {
                                        sum[v][4 * q] += t[b][v][q].x;
                                        sum[v][4 * q + 1] += t[b][v][q].y;
                                        sum[v][4 * q + 2] += t[b][v][q].z;
                                        sum[v][4 * q + 3] += t[b][v][q].w;
                                    }
                            }
                    }
                }
                const int ntok = p.m - c * 16 < 16 ? p.m - c * 16 : 16;   // uniform across the warp
                // Four tokens per pass of a rolled loop: a lone warp issues a dependent instruction
                // every few cycles, so the body is kept short and its four tokens independent.
                const long long tok0 = (long long)(c * 16) * old + o0;
#pragma unroll 1
                for (int g = 0; g < 4 && g * 4 < ntok; g++) {
                    float a[V][4];
#pragma unroll
                    for (int v = 0; v < V; v++)
#pragma unroll
                        for (int i = 0; i < 4; i++)
                            a[v][i] = g == 0 ? sum[v][i] : g == 1 ? sum[v][4 + i] : g == 2 ? sum[v][8 + i] : sum[v][12 + i];
                    const long long at = tok0 + (long long)(g * 4) * old;
#pragma unroll
                    for (int i = 0; i < 4; i++) {
                        if (g * 4 + i >= ntok) break;
                        const int j = c * 16 + g * 4 + i;
                        float val = a[0][i] * f0;
                        if (KIND != KIND_MXF4) val *= p.tokscale[j];
                        if (SWIGLU) {
                            float u = a[V - 1][i] * f1;
                            if (KIND != KIND_MXF4) u *= p.tokscale[j];
                            val = val / (1.0f + __expf(-val)) * u;
                        }
                        if (row_ok) {
                            if (oy) oy[at + i * old] = val;
                            if (oyb) oyb[at + i * old] = bf16_bits(val);
                        }
                        if (oq_codes) {
                            // The same value as the next linear's NVFP4 input: sixteen consecutive
                            // outputs of a token sit in sixteen consecutive lanes (the host side only
                            // allows views that start on a scale tile and hold whole groups).
                            const float vb = row_ok ? round_bf16(val) : 0.0f;
                            float amax = fabsf(vb);
#pragma unroll
                            for (int off = 8; off >= 1; off >>= 1)
                                amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, off));
                            const uint32_t sb = f32_to_e4m3(__fdiv_rn(__fmul_rn(oq_div, amax), 6.0f));
                            const float q = sb ? __fdiv_rn(__fmul_rn(vb, oq_div), e4m3_to_f32(sb)) : 0.0f;
                            const float qn = __shfl_down_sync(0xffffffffu, q, 1);
                            if (row_ok) {
                                if ((lane & 1) == 0)
                                    oq_codes[((long long)j * oq_ld + o0) / 2] = (uint8_t)f32x2_to_e2m1x2(q, qn);
                                if ((lane & 15) == 0) oq_atoms[nvfp4_scale_offset(j, o0 / 16, oq_ld)] = (uint8_t)sb;
                            }
                        }
                    }
                }
            }
        }
    }

    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem), "r"((uint32_t)DT_TMEM_COLS)
                     : "memory");
    }
}

// ---- host side ----

static std::mutex g_gemv_tc_mu;
static int* gemv_tc_status_ptr() {
    static int* ptrs[64] = {};
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return nullptr;
    std::lock_guard<std::mutex> lock(g_gemv_tc_mu);
    if (!ptrs[dev]) cudaGetSymbolAddress(reinterpret_cast<void**>(&ptrs[dev]), g_gemv_tc_status);
    return ptrs[dev];
}

// Arrival counters of the K-split fix-up: zeroed when (re)allocated, returned to zero by the kernel.
// One array per device, shared by every launch: launches on a device must be stream-ordered.
static int* g_gemv_tc_ticket_ptrs[64] = {};
static size_t g_gemv_tc_ticket_caps[64] = {};
static int* gemv_tc_tickets(size_t count) {
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return nullptr;
    std::lock_guard<std::mutex> lock(g_gemv_tc_mu);
    if (count > g_gemv_tc_ticket_caps[dev]) {
        const size_t n = count < 4096 ? 4096 : count * 2;
        int* q = nullptr;
        if (cudaMalloc(&q, n * sizeof(int)) != cudaSuccess) {
            cudaGetLastError();
            return nullptr;
        }
        if (cudaMemsetAsync(q, 0, n * sizeof(int), stream()) != cudaSuccess) return nullptr;
        g_gemv_tc_ticket_ptrs[dev] = q;   // the old block stays allocated: queued work may still use it
        g_gemv_tc_ticket_caps[dev] = n;
    }
    return g_gemv_tc_ticket_ptrs[dev];
}

// Clears the status word and the arrival counters (a launch that gave up leaves them non-zero).
// The caller has synchronised the device.
int gemv_tc_status_reset() {
    const int zero = 0;
    cudaError_t e = cudaMemcpyToSymbol(g_gemv_tc_status, &zero, sizeof(int));
    if (e != cudaSuccess) return (int)e;
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 0;
    std::lock_guard<std::mutex> lock(g_gemv_tc_mu);
    if (g_gemv_tc_ticket_ptrs[dev])
        e = cudaMemset(g_gemv_tc_ticket_ptrs[dev], 0, g_gemv_tc_ticket_caps[dev] * sizeof(int));
    return (int)e;
}

int gemv_tc_status_sync() {
    int v = -1;
    if (cudaMemcpyFromSymbol(&v, g_gemv_tc_status, sizeof(int)) != cudaSuccess) return -1;
    return v;
}

// One launch for `n` views of the same parent width that read the same activations (n = 1 is the
// plain linear; the fused SwiGLU pair is a single LinearArgs with swiglu set and n = 1). `act` is
// VELOX_ACT_NVFP4 (NVFP4 views, `divisor`) or VELOX_ACT_FP8_ROW (FP8-row views).
int gemv_tc_parts(const LinearArgs* parts, int n, int act, float divisor) {
    if (!gemm_available() || n < 1 || n > DT_MAX_PARTS) return VELOX_ERR_UNSUPPORTED;
    const LinearArgs& a = parts[0];
    const bool sw = a.swiglu != 0;
    const bool f8 = act == VELOX_ACT_FP8_ROW;
    if (!f8 && act != VELOX_ACT_NVFP4) return VELOX_ERR_UNSUPPORTED;
    if (sw && n != 1) return VELOX_ERR_UNSUPPORTED;
    const long long k = a.w.k;
    if (a.m < 1 || a.m > 64) return VELOX_ERR_UNSUPPORTED;
    const int nt = a.m <= 16 ? 16 : 64;   // token capacity of the launch
    if (f8 ? (k % 128 != 0 || a.q_codes) : (k % 64 != 0 || !(divisor > 0.0f))) return VELOX_ERR_UNSUPPORTED;

    DtParams p{};
    const uint8_t* codes = a.q_codes;
    int rc;
    if (f8) {
        uint8_t* c = static_cast<uint8_t*>(scratch(SCRATCH_ACT_CODES, (size_t)a.m * k));
        float* sc = static_cast<float*>(scratch(SCRATCH_ACT_SCALES, 64 * sizeof(float)));
        if (!c || !sc) return (int)cudaErrorMemoryAllocation;
        if ((rc = quantize_act_fp8row(a.x, a.xb, a.m, k, c, sc)) != 0) return rc;
        codes = c;
        p.tokscale = sc;
        p.k_steps = (int)(k / 32);
    } else {
        const uint8_t* atoms = a.q_atoms;
        if (!codes || !atoms) {
            uint8_t* c = static_cast<uint8_t*>(scratch(SCRATCH_ACT_CODES, (size_t)a.m * k / 2));
            uint8_t* s = static_cast<uint8_t*>(scratch(SCRATCH_ACT_SCALES, (size_t)128 * k / 16));
            if (!c || !s) return (int)cudaErrorMemoryAllocation;
            if ((rc = quantize_act_nvfp4(a.x, a.xb, a.m, k, divisor, c, s)) != 0) return rc;
            codes = c;
            atoms = s;
        }
        p.sfx = atoms;
        p.alpha = 1.0f / divisor;
        p.k_steps = (int)(k / 64);
    }
    const long long row_bytes = f8 ? k : k / 2;
    p.m = a.m;
    p.k_blocks = (p.k_steps + 3) / 4;
    p.k_tiles64 = k / 64;
    p.status = gemv_tc_status_ptr();
    if (!p.status) return VELOX_ERR_UNSUPPORTED;

    CUtensorMap mw[DT_MAX_PARTS], mx;
    auto set_weights = [&](int i, const velox_sm100_view& v) -> int {
        if (v.format != (f8 ? VELOX_FMT_FP8_ROW_BF16 : VELOX_FMT_NVFP4) || v.k != k ||
            (reinterpret_cast<uintptr_t>(v.w) & 15))
            return VELOX_ERR_UNSUPPORTED;
        p.tile0[i] = v.row_begin / 128;
        if (f8) {
            p.rowscale[i] = reinterpret_cast<const uint16_t*>(v.w + align256(v.n * k));
        } else {
            p.sfw[i] = v.w + align256(v.n * k / 2);
            p.wdiv[i] = reinterpret_cast<const float*>(p.sfw[i] + v.n * k / 16);
        }
        return gemm_make_map_u8(&mw[i], v.w, v.n, row_bytes, 128);
    };
    auto set_out = [&](int i, const LinearArgs& l) -> int {
        const velox_sm100_view& v = l.w;
        DtOut& o = p.out[i];
        o.valid_begin = v.row_begin;
        o.valid_end = v.row_begin + v.rows;
        o.y = l.y;
        o.yb = l.yb;
        o.ld = l.ld;
        o.col = l.col;
        if (l.qo_codes) {
            // whole 16-wide groups of whole rows of the quantised matrix, starting at column 0
            if (f8 || !l.qo_atoms || !(l.qo_divisor > 0.0f) || l.col != 0 || v.row_begin % 128 != 0 ||
                v.rows % 64 != 0 || l.y)
                return VELOX_ERR_UNSUPPORTED;
            o.q_codes = l.qo_codes;
            o.q_atoms = l.qo_atoms;
            o.q_divisor = l.qo_divisor;
            o.q_ld = v.rows;
        }
        return 0;
    };
    if (sw) {
        if ((a.w.row_begin - a.up.row_begin) % 128 != 0) return VELOX_ERR_UNSUPPORTED;
        if ((rc = set_weights(0, a.w)) != 0 || (rc = set_weights(1, a.up)) != 0 || (rc = set_out(0, a)) != 0) return rc;
        mw[2] = mw[0];
        p.nparts = 1;
        p.part_tiles[0] = (int)((a.w.row_begin + a.w.rows - 1) / 128 - a.w.row_begin / 128 + 1);
        p.tiles = p.part_tiles[0];
    } else {
        for (int i = 0; i < n; i++) {
            const LinearArgs& l = parts[i];
            if (l.swiglu || l.m != a.m) return VELOX_ERR_UNSUPPORTED;
            if ((rc = set_weights(i, l.w)) != 0 || (rc = set_out(i, l)) != 0) return rc;
            p.part_tiles[i] = (int)((l.w.row_begin + l.w.rows - 1) / 128 - l.w.row_begin / 128 + 1);
            p.tiles += p.part_tiles[i];
        }
        for (int i = n; i < DT_MAX_PARTS; i++) mw[i] = mw[0];
        p.nparts = n;
    }
    if ((rc = gemm_make_map_u8(&mx, codes, a.m, row_bytes, nt)) != 0) return rc;

    static int sms = 0;
    if (sms == 0) {
        int dev = 0;
        cudaGetDevice(&dev);
        cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
        if (sms <= 0) sms = 148;
    }
    // Equal runs of (tile, k-block) steps per CTA, at least two steps each.
    const long long total_steps = (long long)p.tiles * p.k_blocks;
    long long grid_l = total_steps / 2 < 1 ? 1 : total_steps / 2;
    if (grid_l > sms) grid_l = sms;
    p.per_cta = (total_steps + grid_l - 1) / grid_l;
    const int grid = (int)((total_steps + p.per_cta - 1) / p.per_cta);
    {
        const size_t per_slot = (size_t)(sw ? 2 : 1) * 128 * nt * sizeof(float);
        p.partial = static_cast<float*>(scratch(SCRATCH_Y_F32, (size_t)grid * 2 * per_slot));
        p.tickets = gemv_tc_tickets((size_t)p.tiles);
        if (!p.partial || !p.tickets) return (int)cudaErrorMemoryAllocation;
    }

    cudaError_t e;
    TimedRegion timed(TIMED_GEMV);
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = dim3(grid);
    cfg.blockDim = dim3(DT_THREADS);
    cfg.dynamicSmemBytes = nt == 16 ? DtPlan<16>::SMEM_BYTES : DtPlan<64>::SMEM_BYTES;
    cfg.stream = stream();
    // Early start: this kernel's CTAs may become resident while the kernel before it in the
    // stream is still finishing; they fetch weights, and wait for that kernel before touching
    // anything it wrote (grid_dependency_wait in the producers).
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    static const bool early = getenv("VELOX_SM100_NO_EARLY_START") == nullptr;
    cfg.attrs = attr;
    cfg.numAttrs = early ? 1 : 0;
    auto go = [&](auto kern) {
        cudaError_t err =
            cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)cfg.dynamicSmemBytes);
        if (err != cudaSuccess) return err;
        return cudaLaunchKernelEx(&cfg, kern, mw[0], mw[1], mw[2], mx, p);
    };
    if (nt == 16) {
        if (f8)
            e = sw ? go(gemv_nvfp4_tc_kernel<true, KIND_F8, 16>) : go(gemv_nvfp4_tc_kernel<false, KIND_F8, 16>);
        else
            e = sw ? go(gemv_nvfp4_tc_kernel<true, KIND_MXF4, 16>) : go(gemv_nvfp4_tc_kernel<false, KIND_MXF4, 16>);
    } else {
        if (f8)
            e = sw ? go(gemv_nvfp4_tc_kernel<true, KIND_F8, 64>) : go(gemv_nvfp4_tc_kernel<false, KIND_F8, 64>);
        else
            e = sw ? go(gemv_nvfp4_tc_kernel<true, KIND_MXF4, 64>) : go(gemv_nvfp4_tc_kernel<false, KIND_MXF4, 64>);
    }
    if (e != cudaSuccess) return (int)e;
    return launch_status();
}

int gemv_nvfp4_tc_parts(const LinearArgs* parts, int n, float divisor) {
    return gemv_tc_parts(parts, n, VELOX_ACT_NVFP4, divisor);
}

int gemv_tc(const LinearArgs& a, int act, float divisor) { return gemv_tc_parts(&a, 1, act, divisor); }

}  // namespace vx
