/*
 * velox_sm100 — C ABI of the B200 (sm_100a) quantized-linear kernel set for velox-inferer.
 *
 * These are the `extern "C"` launchers a `velox-variant` crate binds for the `Backend` linear
 * family on NVFP4, FP8-E4M3-per-row and GGML Q4_K weights. Conventions follow the reference's
 * launchers (crates/velox-cuda/kernels/velox_common.cuh:13-14, crates/velox-cuda/src/lib.rs:85-112):
 *
 *   return 0        success (work queued on the launch stream; nothing is synchronised)
 *   return  > 0     a cudaError_t
 *   return -1       VELOX_ERR_UNSUPPORTED: shape/format this kernel set does not serve; the
 *                   caller falls back to the portable path
 *   return -2       VELOX_ERR_SHAPE: arguments the reference's check::linear would reject
 *                   (crates/velox-core/src/check.rs:100-131); the Rust side raises Error::Shape
 *                   before the call, so a binding never sees this code in practice
 *
 * All pointers are device pointers unless stated. Weight pointers address the parent payload in
 * its stored layout (crates/velox-core/src/format.rs:147-160), 256-byte aligned as cudaMalloc
 * returns it. Buffers are borrowed for the duration of the queued work.
 *
 * Streams: like the reference's launchers (per-thread default stream, no stream argument) the
 * launch stream is implicit: cudaStreamPerThread unless the calling thread chose another with
 * velox_sm100_set_stream. Launchers do not synchronise, read back or allocate, except for
 * grow-only private scratch on first use of a larger size (the reference's VeloxScratch rule,
 * velox_common.cuh:49-70).
 *
 * One stream per device at a time. The scratch is one set of pools per device, shared by every
 * call: quantised activations, dequantised bf16 weights, the f32 partial sums and arrival counters
 * of the K-split decode kernels, the words that elect a launch's last CTA. Two calls whose kernels
 * can run at the same time on one device (different streams, or different threads with their
 * per-thread streams) would overwrite each other's scratch and give wrong results without any
 * error. Keep all calls on a device stream-ordered, as the reference's engine does (its scratch
 * carries the same rule: "engine work is serialized", velox_common.cuh:49-70). The entry points
 * that take pre-quantised activations (the _q4 family) at prefill width use no scratch.
 */
#ifndef VELOX_SM100_H
#define VELOX_SM100_H

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define VELOX_ERR_UNSUPPORTED (-1)
#define VELOX_ERR_SHAPE (-2)
/* velox_sm100_linear_nvfp4_a4_static only: the call needs more than the fixed scratch array holds. */
#define VELOX_ERR_STATIC_SCRATCH (-3)
#define VELOX_SM100_STATIC_SCRATCH_BYTES (8u << 20)

/* Weight format codes: crates/velox-cuda/src/portable.rs:197-216. */
#define VELOX_FMT_FP8_ROW_BF16 2
#define VELOX_FMT_NVFP4 3
#define VELOX_FMT_GGML_Q4_K 17

/* ActPolicy (crates/velox-core/src/backend.rs:757-780). */
#define VELOX_POLICY_A16_ONLY 0
#define VELOX_POLICY_ALLOW_A8 1
#define VELOX_POLICY_ALLOW_A4 2

/* ActQuant (crates/velox-core/src/backend.rs:786-806). */
#define VELOX_ACT_EXACT 0
#define VELOX_ACT_BF16 1
#define VELOX_ACT_FP8_ROW 2
#define VELOX_ACT_NVFP4 3

/* WeightView (crates/velox-core/src/backend.rs:826-895): rows [row_begin, row_begin+rows) of an
 * encoded parent [n, k]. `policy`/`divisor` carry the view's ActPolicy. */
typedef struct velox_sm100_view {
    const uint8_t* w;
    int32_t format;
    int32_t policy;
    int64_t n;
    int64_t k;
    int64_t row_begin;
    int32_t rows;
    float divisor;
} velox_sm100_view;

/* LinearPart + LinearDst (backend.rs:847-867): one view written to columns [col, col+rows) of a
 * destination with row stride ld. */
typedef struct velox_sm100_part {
    velox_sm100_view view;
    float* y;
    int64_t ld;
    int64_t col;
} velox_sm100_part;

/* Library / build information. Returns the ABI version (1). */
int velox_sm100_abi_version(void);

/* Debug aid with no counterpart in the reference: synchronises the device and returns the status
 * word of the kernels that wait on something: 0, or the code of the first bounded wait that gave up
 * (1-5: an mbarrier inside a tensor-core kernel; 6: a peer's flag in a tensor-parallel step). The
 * kernel then went on without what it waited for and its output is meaningless. The word is sticky
 * until velox_sm100_debug_status_reset. Never call either on a hot path. */
int velox_sm100_debug_status(void);
/* Synchronises the device, then clears the status words and the per-device counters a kernel that
 * gave up may have left non-zero (arrival tickets of the K-split fix-up, last-CTA tickets). */
int velox_sm100_debug_status_reset(void);

/* Kernel launches issued through this library since it was loaded (host counter). No counterpart
 * in the reference; the benchmark reports it. */
long long velox_sm100_launch_count(void);

/* CUDA-event timing of the main kernels, the counterpart of the reference's VELOX_GPU_TIMING
 * (crates/velox-cuda/src/timing.rs:1-97). While enabled every timed kernel is bracketed by an
 * event pair on its launch stream (do not enable it while capturing a CUDA graph).
 * velox_sm100_timing_collect synchronises the device and returns, per class, the summed kernel
 * milliseconds and the launch count since the last collect. Classes: 0 GEMV, 1 GEMM NVFP4,
 * 2 GEMM FP8, 3 GEMM bf16, 4 activation quantiser, 5 weight dequantiser, 6 the norms that write
 * NVFP4 activations (and the tensor-parallel finish). A kernel's time includes what it spends
 * waiting for peers' flags. `classes` >= 7. */
int velox_sm100_timing_enable(int on);
int velox_sm100_timing_collect(double* ms_by_class, long long* count_by_class, int classes);

/* Launch stream of the calling thread (a cudaStream_t); NULL restores cudaStreamPerThread.
 * Replaces nothing in the reference: its launchers always use the per-thread default stream
 * (crates/velox-build/src/lib.rs:120-129). */
int velox_sm100_set_stream(void* stream);

/* The rounding `linear` applies to x for this view at m rows (Backend::linear_act,
 * backend.rs:933-937; CudaKernels::linear_act, crates/velox-cuda/src/lib.rs:578). Returns a
 * VELOX_ACT_* code (>= 0) or a negative error. For VELOX_ACT_NVFP4, *divisor_out (host pointer,
 * may be NULL) receives the divisor. Never rounds further than the view's policy allows. */
int velox_sm100_linear_act(const velox_sm100_view* view, int m, float* divisor_out);

/* y[m, rows] = x[m, k] . W^T with the view's policy fixed to A16Only. Same signature as
 * velox_portable_linear (crates/velox-cuda/src/portable.rs:81-91; kernels/portable_model.cu:1899). */
int velox_sm100_linear(const float* x, const uint8_t* w, int format, long long n, long long k,
                       long long row_begin, int rows, int m, float* y);

/* Backend::linear for a view with an activation policy (backend.rs:925-932). yb (may be NULL)
 * receives the bf16 RNE twin of y, bit for bit. */
int velox_sm100_linear_view(const float* x, const velox_sm100_view* view, int m, float* y,
                            uint16_t* yb);

/* Backend::linear_bf16 (backend.rs:1011-1021): the same result from x's bf16 twin. Served where
 * velox_sm100_linear_act reports VELOX_ACT_BF16 (Backend::takes_bf16). y and yb: either may be
 * NULL, not both. */
int velox_sm100_linear_bf16(const uint16_t* xb, const velox_sm100_view* view, int m, float* y,
                            uint16_t* yb);

/* NVFP4 prefill linear that allocates nothing. It has no counterpart in the reference.
 *
 * For whom: hosts that may not call cudaMalloc while they run the model - a server whose memory
 * planner has already handed every byte of the device to weights, KV cache and workspaces, a
 * real-time loop that must not take the allocator's lock, a process whose allocations are
 * audited or capped. The regular entry points keep the quantised activations of the tensor-core
 * path (E2M1 codes and their scale atoms) in scratch that they cudaMalloc on first use and grow
 * when a larger call arrives; this one keeps them in a fixed 8 MiB array inside the library
 * image (VELOX_SM100_STATIC_SCRATCH_BYTES; every GPU that loads the library carries it until the
 * process ends) and calls no cudaMalloc, cudaFree or other allocating routine, ever.
 *
 * Serves an NVFP4 view whose policy is AllowA4 at m > 16 on the prefill GEMM, activations rounded as
 * VELOX_ACT_NVFP4 with the view's divisor: the bits velox_sm100_linear_bf16 gives wherever it takes
 * the GEMM too (m > 64 always; 17..64 unless its cost model streams the shape). Anything else returns
 * VELOX_ERR_UNSUPPORTED. The call needs align256(m*k/2) + ceil(m/128)*128*k/16 bytes of the
 * array (m = 2048, k = 5120: 5.9 MiB); a larger call returns VELOX_ERR_STATIC_SCRATCH and does
 * nothing.
 *
 * The first call on each device looks up the array's device address (cudaGetSymbolAddress, with
 * that device current): make that first call before starting any stream capture.
 * All calls on a device share the one array. Each call rewrites every byte it later reads, so
 * contents left by an earlier call are harmless, but two calls whose kernels can run at the same
 * time (different streams, or different threads) race on it: keep such calls on one stream. */
int velox_sm100_linear_nvfp4_a4_static(const uint16_t* xb, const velox_sm100_view* view, int m,
                                       float* y, uint16_t* yb);

/* Backend::linear_swiglu (backend.rs:1102-1118): out[r][i] = silu(x_r . gate_i) * (x_r . up_i).
 * gate and up: same width, format and k; any two views (adjacent in one parent in either order,
 * or separate parents). Fused: no intermediate [m, 2w] buffer. outb (may be NULL): bf16 twin. */
int velox_sm100_linear_swiglu(const float* x, const velox_sm100_view* gate,
                              const velox_sm100_view* up, int m, float* out, uint16_t* outb);

/* Backend::linear_swiglu_twin (backend.rs:1034-1048): the same from x's bf16 twin. */
int velox_sm100_linear_swiglu_bf16(const uint16_t* xb, const velox_sm100_view* gate,
                                   const velox_sm100_view* up, int m, float* out, uint16_t* outb);

/* The rounding linear_swiglu applies (Backend::linear_swiglu_act, backend.rs:1130-1141). */
int velox_sm100_linear_swiglu_act(const velox_sm100_view* gate, const velox_sm100_view* up, int m,
                                  float* divisor_out);

/* Backend::linears (backend.rs:938-958): several views of one x, each into a column range of its
 * destination. `parts` is a HOST array. x may be NULL when xb (bf16 twin) is given and every
 * part rounds to bf16. */
int velox_sm100_linears(const float* x, const uint16_t* xb, const velox_sm100_part* parts,
                        int nparts, int m);

/* Backend::embed / embed_from (crates/velox-core/src/backend.rs:1142-1160): out[t, :] = the exact
 * decode of row row_begin + ids[t] of the parent [n, k]; a row that does not exist gives zeros (ids
 * written on the device are not checked by the host). `ids` is a device array. Same signature as
 * velox_portable_embed (crates/velox-cuda/src/portable.rs:92-101; kernels
 * crates/velox-cuda/kernels/portable_model.cu:485-575). k must be a multiple of 16. */
int velox_sm100_embed(const uint32_t* ids, int count, const uint8_t* w, int format, long long n, long long k,
                      long long row_begin, float* out);

/* Backend::matmul (backend.rs:1550-1564): y[m, n] = x[m, k] . w[n, k]^T, all f32, f32 accumulation.
 * Same signature as velox_portable_matmul (crates/velox-cuda/src/portable.rs:19-26; kernel
 * crates/velox-cuda/kernels/portable.cu:13-28). */
int velox_sm100_matmul(const float* x, const float* w, float* y, int m, int n, int k);

/* Exact decode of a view to f32 [rows, k]: the values format::decode_rows produces
 * (crates/velox-core/src/format.rs:426-490), bit for bit. */
int velox_sm100_dequant_rows(const velox_sm100_view* view, float* out);

/* Activation quantisers, bit-exact with quant::quantize_activations (crates/velox-core/src/quant.rs:63-96).
 * fp8row: codes [m, k] E4M3, scales[m] = amax/448. nvfp4: codes [m, k/2] (two E2M1 per byte, low
 * nibble first), scale bytes in the weight format's 128x4 swizzled atoms (format.rs:345-354)
 * over ceil(m/128)*128 rows. */
int velox_sm100_quantize_act_fp8row(const float* x, int m, long long k, uint8_t* codes,
                                    float* scales);
int velox_sm100_quantize_act_nvfp4(const float* x, int m, long long k, float divisor,
                                   uint8_t* codes, uint8_t* scale_atoms);

/* NVFP4 weight construction on the device (round-to-nearest-even converters of quant.rs:9-59,
 * layout and divisor convention of format::encode_nvfp4, format.rs:385-423). `amax` is max|w|
 * over the matrix. Used to build benchmark-sized synthetic weights. */
int velox_sm100_encode_nvfp4(const float* w, long long n, long long k, float amax,
                             uint8_t* payload);

/* Elementwise neighbours of the path. Signatures as the portable launchers
 * (crates/velox-cuda/src/portable.rs:19-66; kernels/portable.cu:109-115, 1519-1550). */
int velox_sm100_swiglu(const float* src, long long rows, int src_cols, int gate, int up, int width,
                       float* out);
int velox_sm100_silu_mul(float* gate, const float* up, long long len);
int velox_sm100_add(float* acc, const float* x, long long len);
/* Backend::add_rms_norm_twin (backend.rs:968-983): acc += x (x may be NULL: plain rms_norm of
 * acc); y = rms_norm(acc) * (offset + weight); yb (may be NULL) = bf16 twin of y. */
int velox_sm100_add_rms_norm_twin(float* acc, const float* x, const float* weight, float* y,
                                  uint16_t* yb, int rows, int dim, float eps, int offset);
/* FP4 activation twins, the counterpart for NVFP4 of the reference's int8 twins
 * (Backend::add_rms_norm_q8 / linear_q8 / linear_swiglu_q8, backend.rs:1050-1100): the norm also
 * writes its result as the activation blob the FP4 tensor-core linears read - E2M1 codes [rows,
 * dim/2] and E4M3 scale atoms over ceil(rows/128)*128 rows, quantised from the bf16-rounded values
 * with `divisor` exactly as quant::quantize_activations(Nvfp4{divisor}) does - so the projections
 * that follow run without a quantisation pass. velox_sm100_linear_q4 / _swiglu_q4 take that blob
 * in place of x; they serve NVFP4 views whose policy is AllowA4 with the same divisor, at any m
 * (tensor-core decode kernel up to 16 tokens and for small batches it streams faster, prefill GEMM
 * otherwise), and return
 * VELOX_ERR_UNSUPPORTED otherwise (use the bf16 entry points then). */
int velox_sm100_add_rms_norm_q4(float* acc, const float* x, const uint16_t* xb, const float* weight,
                                uint16_t* yb, uint8_t* codes, uint8_t* atoms, int rows, int dim, float eps,
                                int offset, float divisor);
int velox_sm100_linear_q4(const uint8_t* codes, const uint8_t* atoms, float divisor,
                          const velox_sm100_view* view, int m, float* y, uint16_t* yb);
int velox_sm100_linear_swiglu_q4(const uint8_t* codes, const uint8_t* atoms, float divisor,
                                 const velox_sm100_view* gate, const velox_sm100_view* up, int m, float* out,
                                 uint16_t* outb);

/* The FP4 linears as producers of the next linear's FP4 input: the result, rounded to bf16, is
 * quantised in the kernel's epilogue with `out_divisor` into out_codes [m, rows/2] and out_atoms
 * (scale atoms over ceil(m/128)*128 rows; the scales of rows past m are zero after a prefill call
 * and left as they were after a decode call, whose consumers do not read them) - for rows < m bit
 * for bit what velox_sm100_quantize_act_nvfp4 makes of the bf16 output - and also stored as bf16 when yb / outb
 * is not NULL. Same conditions as the _q4 entry points, and the view must start on a 128-row scale
 * tile and hold a multiple of 64 rows; VELOX_ERR_UNSUPPORTED otherwise. */
int velox_sm100_linear_q4_to_q4(const uint8_t* codes, const uint8_t* atoms, float divisor,
                                const velox_sm100_view* view, int m, uint16_t* yb, uint8_t* out_codes,
                                uint8_t* out_atoms, float out_divisor);
int velox_sm100_linear_swiglu_q4_to_q4(const uint8_t* codes, const uint8_t* atoms, float divisor,
                                       const velox_sm100_view* gate, const velox_sm100_view* up, int m,
                                       uint16_t* outb, uint8_t* out_codes, uint8_t* out_atoms,
                                       float out_divisor);

/* Several views of one width reading the same FP4 activations, each with its own destination: the
 * q4 form of Backend::linears (backend.rs:938-958, 1001-1048). yb may be NULL when out_codes is
 * given (the result then exists only as the next linear's FP4 input). Up to three views run as one
 * launch, at decode sizes on the streaming kernel and at prefill sizes on the GEMM (one persistent
 * grid walks the tiles of all views); more views, or views the kernels group differently, run as
 * one launch each. */
typedef struct {
    velox_sm100_view view;
    uint16_t* yb;          /* [m, view.rows] bf16, or NULL */
    uint8_t* out_codes;    /* optional: see velox_sm100_linear_q4_to_q4 */
    uint8_t* out_atoms;
    float out_divisor;
} velox_sm100_part_q4;
int velox_sm100_linears_q4(const uint8_t* codes, const uint8_t* atoms, float divisor,
                           const velox_sm100_part_q4* parts, int nparts, int m);

/* Tensor parallelism over one node (no counterpart in the reference, which is single-device).
 * Token rows are owned by ranks in equal blocks of `rows_per_owner` (a multiple of 128). Buffers
 * named "_ptrs" are arrays, one entry per rank, of device addresses valid on the calling GPU
 * (peer mappings of symmetric allocations).
 *
 * Ordering between ranks needs no barrier kernels: a kernel whose output other ranks read raises a
 * flag on every rank when its last CTA is done, and a kernel that reads such data polls its own
 * rank's flags before its first read. velox_sm100_tp_sync describes both for one launch:
 *   flag_tables[r]   rank r's flag table as mapped on this GPU (entry [rank] is this rank's own):
 *                    `phases` rows of 8 32-bit words, zero when allocated, never reset;
 *   epoch            device address of this rank's 32-bit step counter; velox_sm100_tp_step_begin
 *                    adds one at the start of every step (every rank runs the same steps);
 *   wait_phase       row to wait on: the launch starts reading once flag_tables[rank][row][src] has
 *                    reached the epoch for every src < n; -1: no wait;
 *   signal_phase     row to raise: when the launch's stores are complete the epoch is written to
 *                    flag_tables[d][row][rank] for every d < n; -1: no signal.
 * A wait gives up after a wall-clock limit (2 s; velox_sm100_tp_set_wait_limit_ms), records code 6
 * in the status word (velox_sm100_debug_status) and the kernel runs on and exits normally: a rank
 * that never arrives costs the others a bounded delay and a reported error, not a hang.
 * All launches of a step must be issued on one stream per rank.
 *
 *  - velox_sm100_tp_make_maps: output maps for a row-split linear. slot_ptrs[o] is this rank's
 *    [rows_per_owner, cols] bf16 slot in rank o's memory; maps_dev receives n x 128 bytes.
 *  - velox_sm100_tp_linears_q4 / _tp_linear_swiglu_q4_to_q4: velox_sm100_linears_q4 /
 *    velox_sm100_linear_swiglu_q4_to_q4 at prefill width (m > 16) that wait for `sync` before
 *    reading the activation blob (every rank's norm has written its rows).
 *  - velox_sm100_tp_linear_q4_scatter: linear_q4 whose bf16 result tiles are stored by the GEMM
 *    epilogue straight into the owners' slots (the reduce-scatter's data movement, fused into the
 *    linear), then signals. The view must be a whole parent with a multiple of 256 rows, m a
 *    multiple of rows_per_owner, m > 16.
 *  - velox_sm100_tp_norm_q4: waits; acc (this rank's rows, f32) += the nslots slots in order; rms
 *    norm; the result as NVFP4 codes and scale atoms at rows row0.. of every rank's blob (the
 *    all-gather, fused into the norm); signals. nslots = 0: no addend.
 *  - velox_sm100_tp_finish: waits; acc += the slots; acc as bf16 at rows row0.. of every rank's
 *    output; signals.
 *  - velox_sm100_tp_wait: a one-thread kernel that only waits (the end of a step: every rank's
 *    output rows are in place).
 *  - velox_sm100_tp_barrier: a one-warp kernel that raises row signal_phase (= wait_phase) on every
 *    rank and then waits on it, all ranks side by side: a barrier between two phases as a launch
 *    of its own, for steps whose kernels run without `sync` (the data kernels then carry no
 *    waits; same bounded wait, same status). Launched with early start allowed; the launch behind
 *    it may start early too and is ordered by its own wait for this kernel.
 *  - velox_sm100_tp_signal: a one-thread kernel that only signals (tests).
 * `sync` may be NULL everywhere except tp_wait / tp_signal (single rank, or the caller orders the
 * ranks itself). */
typedef struct velox_sm100_tp_sync {
    unsigned long long flag_tables[8];
    unsigned long long epoch;
    int32_t n, rank;
    int32_t wait_phase, signal_phase;
} velox_sm100_tp_sync;
int velox_sm100_tp_step_begin(unsigned int* epoch);
int velox_sm100_tp_wait(const velox_sm100_tp_sync* sync);
int velox_sm100_tp_barrier(const velox_sm100_tp_sync* sync);
int velox_sm100_tp_signal(const velox_sm100_tp_sync* sync);
int velox_sm100_tp_set_wait_limit_ms(int ms);
int velox_sm100_tp_make_maps(void* maps_dev, const unsigned long long* slot_ptrs, int n, int rows_per_owner,
                             long long cols);
int velox_sm100_tp_linears_q4(const uint8_t* codes, const uint8_t* atoms, float divisor,
                              const velox_sm100_part_q4* parts, int nparts, int m, const velox_sm100_tp_sync* sync);
int velox_sm100_tp_linear_swiglu_q4_to_q4(const uint8_t* codes, const uint8_t* atoms, float divisor,
                                          const velox_sm100_view* gate, const velox_sm100_view* up, int m,
                                          uint16_t* outb, uint8_t* out_codes, uint8_t* out_atoms, float out_divisor,
                                          const velox_sm100_tp_sync* sync);
int velox_sm100_tp_linear_q4_scatter(const uint8_t* codes, const uint8_t* atoms, float divisor,
                                     const velox_sm100_view* view, int m, const void* maps_dev, int rows_per_owner,
                                     const velox_sm100_tp_sync* sync);
int velox_sm100_tp_norm_q4(float* acc, const uint16_t* slots, int nslots, long long slot_stride, const float* weight,
                           const unsigned long long* codes_ptrs, const unsigned long long* atoms_ptrs, int ndst,
                           long long row0, int rows, int dim, float eps, int offset, float divisor,
                           const velox_sm100_tp_sync* sync);
int velox_sm100_tp_finish(float* acc, const uint16_t* slots, int nslots, long long slot_stride,
                          const unsigned long long* out_ptrs, int ndst, long long row0, int rows, int dim,
                          const velox_sm100_tp_sync* sync);

/* The same with a bf16 addend (the all-reduced partial sums of a row-split projection): acc += xb,
 * then the norm. No counterpart in the reference, which has no tensor parallelism. */
int velox_sm100_add_bf16_rms_norm_twin(float* acc, const uint16_t* xb, const float* weight, float* y,
                                       uint16_t* yb, int rows, int dim, float eps, int offset);
int velox_sm100_add_bf16(float* acc, const uint16_t* xb, long long len);
/* f32 -> bf16 twin (RNE), as velox_bf16_bits (velox_common.cuh:74-82). */
int velox_sm100_bf16_twin(const float* x, uint16_t* xb, long long len);

#ifdef __cplusplus
}
#endif
#endif
