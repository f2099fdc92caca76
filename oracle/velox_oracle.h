/*
 * TEST INFRASTRUCTURE ONLY. CPU restatement of velox-inferer's quantized-linear oracle.
 *
 * This is the checker the CUDA path is compared against. Only tests, the smoke check and the
 * benchmark's CPU-baseline leg may load it; the product library never links or calls it.
 *
 * Each function cites the reference source (path within the velox-inferer project) whose
 * arithmetic it follows. All single-precision steps are kept in the reference's order and the
 * file is compiled with -ffp-contract=off so no fused multiply-add changes a rounding.
 *
 * Parity status: pinned against the reference's own known-answer tests (E4M3/E2M1/bf16 values,
 * payload sizes, the NVFP4 encode/decode fixed point, the scale-swizzle permutation, E4M3 and
 * E2M1 round-to-nearest-even tables, the gguf-py Q4_K known answer, matmul_small and
 * linear_bf16_matches_matmul). The reference is Rust and cannot be executed in this build
 * environment, so pinning is through those vectors only.
 */
#ifndef VELOX_ORACLE_H
#define VELOX_ORACLE_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* Format codes shared with the kernels: crates/velox-cuda/src/portable.rs:197-216. */
#define VO_FMT_F32 0
#define VO_FMT_BF16 1
#define VO_FMT_FP8_ROW_BF16 2
#define VO_FMT_NVFP4 3
#define VO_FMT_GGML_Q4_K 17

/* ActQuant kinds: crates/velox-core/src/backend.rs:786-806. */
#define VO_ACT_EXACT 0
#define VO_ACT_BF16 1
#define VO_ACT_FP8_ROW 2
#define VO_ACT_NVFP4 3

/* --- scalar converters ------------------------------------------------------------------- */
float vo_bf16_to_f32(uint16_t bits);          /* format.rs:306-308 */
uint16_t vo_f32_to_bf16(float v);             /* format.rs:311-317 */
float vo_f16_to_f32(uint16_t h);              /* format.rs:179-195 */
uint16_t vo_f32_to_f16(float v);              /* RNE; used only by this repo's Q4_K quantiser */
float vo_e4m3fn_to_f32(uint8_t b);            /* format.rs:320-332 */
float vo_e2m1_to_f32(uint8_t c);              /* format.rs:335-343 */
uint8_t vo_f32_to_e4m3fn_lower(float x);      /* format.rs:357-379 (ties to the lower code) */
uint8_t vo_f32_to_e4m3fn(float x);            /* quant.rs:11-41 (RNE, saturating) */
uint8_t vo_f32_to_e2m1(float x);              /* quant.rs:43-59 (RNE, saturating) */

/* --- layout ------------------------------------------------------------------------------- */
size_t vo_align256(size_t x);                                   /* format.rs:175-177 */
size_t vo_nvfp4_scale_offset(size_t n, size_t g, size_t k);     /* format.rs:345-354 */
/* 0 when the shape is legal for the format, -2 otherwise. format.rs:117-145 */
int vo_check_shape(int fmt, size_t n, size_t k);
size_t vo_payload_bytes(int fmt, size_t n, size_t k);           /* format.rs:147-160 */

/* --- decoders ----------------------------------------------------------------------------- */
void vo_q4k_decode_block(const uint8_t* x, float* y);           /* ggml.rs:159-169, 196-210 */
/* format.rs:426-490. Returns 0, or -2 for a shape error. out is [rows, k]. */
int vo_decode_rows(int fmt, const uint8_t* payload, size_t payload_len, size_t n, size_t k,
                   size_t row_begin, size_t rows, float* out);

/* --- encoders ----------------------------------------------------------------------------- */
/* The reference's own NVFP4 encoder (ties to the lower code): format.rs:385-423. */
void vo_encode_nvfp4_ref(const float* x, size_t n, size_t k, uint8_t* out);
/* The benchmark's construction: same layout and divisor convention, but E4M3 block scales and
 * E2M1 codes rounded to nearest even with the quant.rs converters. */
void vo_encode_nvfp4_rne(const float* x, size_t n, size_t k, uint8_t* out);
/* fp8_e4m3fn_row_bf16: scale_r = bf16(amax_r / 448), code = e4m3_rne(w / scale_r). Layout
 * format.rs:151, 460-467. */
void vo_encode_fp8_row(const float* x, size_t n, size_t k, uint8_t* out);
/* This repo's own Q4_K quantiser (the reference has a decoder only): min/max affine per 32-value
 * sub-block, 6-bit sub-scales against per-super-block f16 d/dmin. Any legal block is valid. */
void vo_encode_q4k(const float* x, size_t n, size_t k, uint8_t* out);

/* --- activation rounding: quant.rs:63-96 --------------------------------------------------- */
void vo_quantize_activations(float* x, size_t rows, size_t k, int act, float divisor);
/* Codes and scales of the same roundings, for comparing a device quantiser bit for bit.
 * fp8: codes [rows,k], scales[rows] (amax/448). nvfp4: codes packed two per byte low nibble
 * first [rows,k/2], scale bytes row-major [rows,k/16]. */
void vo_act_codes_fp8(const float* x, size_t rows, size_t k, uint8_t* codes, float* scales);
void vo_act_codes_nvfp4(const float* x, size_t rows, size_t k, float divisor, uint8_t* codes,
                        uint8_t* scales);

/* --- ops: crates/velox-cpu/src/lib.rs ------------------------------------------------------ */
/* y[m,n] = x[m,k] . w[n,k]^T, f64 accumulation (lib.rs:31-36, 128-145). */
void vo_matmul(const float* x, const float* w, float* y, size_t m, size_t n, size_t k,
               int threads);
/* lib.rs:147-164 with check::linear (check.rs:100-131). Returns 0 or -2 (shape). threads > 1
 * splits output rows across threads; every output keeps its own summation order. */
int vo_linear(const float* x, size_t x_len, const uint8_t* payload, size_t payload_len, int fmt,
              size_t n, size_t k, size_t row_begin, size_t rows, size_t m, float* y, size_t y_len,
              int threads);
void vo_silu_mul(float* gate, const float* up, size_t len);                     /* lib.rs:224-230 */
void vo_swiglu(const float* src, size_t rows, size_t src_cols, size_t gate, size_t up,
               size_t width, float* out);                                       /* lib.rs:688-707 */
void vo_add(float* acc, const float* x, size_t len);
void vo_rms_norm(const float* x, const float* weight, float* y, size_t rows, size_t dim,
                 float eps, int offset);                                        /* lib.rs:188-207 */

/* --- generators used by the reference's tests ---------------------------------------------- */
/* xorshift generator: crates/velox-core/src/rng.rs:3-27. */
typedef struct { uint64_t s; } vo_rng;
void vo_rng_new(vo_rng* r, uint64_t seed);
uint64_t vo_rng_next(vo_rng* r);
float vo_rng_uniform(vo_rng* r);
void vo_rng_vec(vo_rng* r, size_t len, float scale, float* out);
/* A random legal encoding: crates/velox-conformance/src/lib.rs:114-199 (NVFP4, FP8 row, Q4_K). */
int vo_random_weight(vo_rng* r, int fmt, size_t n, size_t k, uint8_t* out);
/* SplitMix64 block bytes of the gguf-py known-answer test: ggml.rs:4450-4485. Writes
 * 512/256 * 144 bytes for Q4_K. */
void vo_kat_q4k_blocks(uint64_t seed, uint8_t* out);

/* --- error metrics -------------------------------------------------------------------------- */
double vo_max_err(const float* got, const float* want, size_t len);   /* conformance lib.rs:43-58 */
double vo_rms(const float* v, size_t len);
double vo_max_abs_diff(const float* got, const float* want, size_t len);

#ifdef __cplusplus
}
#endif
#endif
