// Internal launcher declarations shared by the C-ABI dispatcher (api.cu).
#pragma once

#include <stdint.h>

#include "../../include/velox_sm100.h"

namespace vx {

// One projection of a decode/verify GEMV or of the generic fallback.
struct LinearArgs {
    velox_sm100_view w;      // gate view for the fused SwiGLU form
    velox_sm100_view up;     // used when swiglu != 0
    int swiglu;
    const float* x;          // [m, k] f32, or NULL
    const uint16_t* xb;      // [m, k] bf16 twin, or NULL (one of x / xb is set)
    int round_x;             // round f32 x to bf16 on load (ActQuant::Bf16)
    int m;
    float* y;                // may be NULL when yb is set
    uint16_t* yb;            // bf16 twin of y, may be NULL
    const uint8_t* q_codes;  // activations already quantised to NVFP4 (codes [m, k/2]) ...
    const uint8_t* q_atoms;  // ... and their scale atoms; both NULL unless the caller has them
    uint8_t* qo_codes;       // optional: the result also (or only) as NVFP4 activations for the
    uint8_t* qo_atoms;       // next linear, quantised with qo_divisor (FP4 tensor-core path only)
    float qo_divisor;
    const void* rs_maps;     // optional (tensor parallel): per-owner output maps in device memory, and
    int rs_rows_per_owner;   // the token rows each owner holds; replaces y / yb
    long long ld;            // row stride of y / yb in elements
    long long col;           // first column written
    const velox_sm100_tp_sync* sync;  // optional (tensor parallel): flags to wait for / to raise
};

int dequant_rows_f32(const velox_sm100_view* v, float* out);
// out[t] = exact decode of parent row v->row_begin + ids[t] (zeros for rows that do not exist).
int embed_rows_f32(const velox_sm100_view* v, const uint32_t* ids, int count, float* out);
// y[m, n] = x[m, k] . w[n, k]^T, all f32.
int matmul_f32(const float* x, const float* w, float* y, int m, int n, int k);
// lo_offset > 0: also write the two bf16 remainder terms of each value, lo_offset and 2 lo_offset elements after it.
int dequant_rows_bf16(const velox_sm100_view* v, uint16_t* out, long long ld_out, long long lo_offset);

// Memory-bound path, m <= 16, k % 64 == 0.
int gemv(const LinearArgs& a);
// NVFP4 only: inner products on the tensor cores (mma.sync); k % 128 == 0.
int gemv_nvfp4_mma(const LinearArgs& a);
// NVFP4 only: TMA-staged weight stream + mma.sync; k % 128 == 0. The preferred decode kernel.
int gemv_nvfp4_tma(const LinearArgs& a);
int gemv_status_sync();
int gemv_tc_status_sync();
int gemv_status_reset();
int gemv_tc_status_reset();
int tp_status_sync();
int tp_status_reset();
// Any shape, any m: one warp per output row, per-element decode. Slow but total.
int linear_generic(const LinearArgs& a);

int quantize_act_fp8row(const float* x, const uint16_t* xb, int m, long long k, uint8_t* codes,
                        float* scales);
int quantize_act_nvfp4(const float* x, const uint16_t* xb, int m, long long k, float divisor,
                       uint8_t* codes, uint8_t* scale_atoms);
int quantize_act_nvfp4_untimed(const uint16_t* xb, int m, long long k, float divisor, uint8_t* codes,
                               uint8_t* scale_atoms);
int encode_nvfp4(const float* w, long long n, long long k, float amax, uint8_t* payload);

int swiglu(const float* src, long long rows, int src_cols, int gate, int up, int width, float* out);
int silu_mul(float* gate, const float* up, long long len);
int add(float* acc, const float* x, long long len);
int add_bf16(float* acc, const uint16_t* xb, long long len);
// acc += x (f32) or xb (bf16) when given, then the norm of acc.
int add_rms_norm_twin(float* acc, const float* x, const uint16_t* xb, const float* weight, float* y,
                      uint16_t* yb, int rows, int dim, float eps, int offset);
int bf16_twin(const float* x, uint16_t* xb, long long len);
// Q4_K decode on the warp-level tensor-core MMA (plain form, m <= 16, k % 256 == 0); else VELOX_ERR_UNSUPPORTED.
int gemv_q4k_mma(const LinearArgs& a);
// FP8-row decode with bf16 activations on the same MMA (m <= 16, k % 64 == 0); else VELOX_ERR_UNSUPPORTED.
int gemv_fp8_mma(const LinearArgs& a);
int sp_norm_q4(float* acc, const uint16_t* slots, int nslots, long long slot_stride, const float* weight,
               uint8_t* const* codes, uint8_t* const* atoms, int ndst, long long row0, int rows, int dim, float eps,
               int offset, float divisor, const velox_sm100_tp_sync* sync);
int sp_finish(float* acc, const uint16_t* slots, int nslots, long long slot_stride, uint16_t* const* out, int ndst,
              long long row0, int rows, int dim, const velox_sm100_tp_sync* sync);
int add_rms_norm_q4(float* acc, const float* x, const uint16_t* xb, const float* weight, uint16_t* yb,
                    uint8_t* codes, uint8_t* atoms, int rows, int dim, float eps, int offset, float divisor);

}  // namespace vx
