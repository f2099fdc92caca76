// Weight-view decoders.
//
// dequant_rows_f32: the values format::decode_rows produces (crates/velox-core/src/format.rs:426-490,
// Q4_K crates/velox-core/src/ggml.rs:196-210), bit for bit: every f32 step is issued with an
// explicit round-to-nearest intrinsic so the compiler cannot fuse a multiply into an add, and the
// NVFP4 per-tensor divisor is an IEEE division as in the reference.
//
// dequant_rows_bf16: the operand the bf16 tensor-core GEMM multiplies. NVFP4 -> e2m1*e4m3 (six
// significant bits: exact in bf16; the 1/divisor factor is applied to the f32 accumulator), FP8 ->
// the E4M3 value (exact; the row scale is applied to the accumulator), Q4_K -> the decoded value
// as three bf16 terms (bf16(v), bf16 of the remainder, bf16 of what is left of that) laid side by
// side along K, so the GEMM's f32 accumulation sees the f32 value exactly.
#include "common.cuh"
#include "kernels.cuh"

namespace vx {

// One thread decodes 16 consecutive k of one row. With `ids` the rows are gathered: output row i is
// parent row row_begin + ids[i], or zeros where that row does not exist (ids written on the device
// are not checked by the host), which is Backend::embed (crates/velox-core/src/backend.rs:1142-1160;
// reference kernels crates/velox-cuda/kernels/portable_model.cu:485-575).
template <int FMT, typename OUT>
__global__ void __launch_bounds__(256)
dequant_rows_kernel(const uint8_t* __restrict__ w, long long n, long long k, long long row_begin,
                    int rows, OUT* __restrict__ out, long long ld_out, long long lo_offset,
                    const uint32_t* __restrict__ ids) {
    const long long groups_per_row = k / 16;
    const long long total = (long long)rows * groups_per_row;
    for (long long idx = blockIdx.x * (long long)blockDim.x + threadIdx.x; idx < total;
         idx += (long long)gridDim.x * blockDim.x) {
        const long long i = idx / groups_per_row;
        const long long g = idx % groups_per_row;
        const long long r = row_begin + (ids ? (long long)ids[i] : i);
        float v[16];
        if (ids && (r < 0 || r >= n)) {
#pragma unroll
            for (int j = 0; j < 16; j++) v[j] = 0.0f;
        } else if (FMT == VELOX_FMT_NVFP4) {
            const long long scale_plane = align256(n * k / 2);
            const uint2 codes = *reinterpret_cast<const uint2*>(w + (r * k + g * 16) / 2);
            const float scale = e4m3_to_f32(w[scale_plane + nvfp4_scale_offset(r, g, k)]);
            const float divisor = *reinterpret_cast<const float*>(w + scale_plane + n * k / 16);
#pragma unroll
            for (int j = 0; j < 16; j++) {
                const uint32_t word = j < 8 ? codes.x : codes.y;
                const float m = e2m1_to_f32((word >> (4 * (j & 7))) & 0xfu);
                const float p = __fmul_rn(m, scale);
                v[j] = sizeof(OUT) == 4 ? __fdiv_rn(p, divisor) : p;
            }
        } else if (FMT == VELOX_FMT_FP8_ROW_BF16) {
            const uint4 codes = *reinterpret_cast<const uint4*>(w + r * k + g * 16);
            const uint32_t sbits = *reinterpret_cast<const unsigned short*>(w + align256(n * k) + 2 * r);
            const float scale = bf16_bits_to_f32(sbits);
            const uint32_t words[4] = {codes.x, codes.y, codes.z, codes.w};
#pragma unroll
            for (int j = 0; j < 16; j++) {
                const float c = e4m3_to_f32((words[j >> 2] >> (8 * (j & 3))) & 0xffu);
                v[j] = sizeof(OUT) == 4 ? __fmul_rn(c, scale) : c;
            }
        } else {  // Q4_K: block = d | dmin | scales[12] | qs[128]
            const long long blocks = k / 256;
            const long long b = g / 16;
            const int sub = (int)(g % 16) / 2;      // sub-block of 32 values
            const int half16 = (int)(g % 2);        // which 16 of the 32
            const uint8_t* blk = w + (r * blocks + b) * 144;
            const float d = f16_bits_to_f32(*reinterpret_cast<const unsigned short*>(blk));
            const float dmin = f16_bits_to_f32(*reinterpret_cast<const unsigned short*>(blk + 2));
            uint32_t sc, mn;
            q4k_scale_min(sub, blk + 4, sc, mn);
            const float d1 = __fmul_rn(d, (float)sc);
            const float m1 = __fmul_rn(dmin, (float)mn);
            const uint4 qs = *reinterpret_cast<const uint4*>(blk + 16 + 32 * (sub / 2) + 16 * half16);
            const uint32_t words[4] = {qs.x, qs.y, qs.z, qs.w};
            const int shift = (sub & 1) ? 4 : 0;
#pragma unroll
            for (int j = 0; j < 16; j++) {
                const uint32_t q = (words[j >> 2] >> (8 * (j & 3) + shift)) & 0xfu;
                v[j] = __fsub_rn(__fmul_rn(d1, (float)q), m1);
            }
        }
        OUT* o = out + i * ld_out + g * 16;
        if (sizeof(OUT) == 4) {
            float4* o4 = reinterpret_cast<float4*>(o);
#pragma unroll
            for (int j = 0; j < 4; j++) o4[j] = make_float4(v[4 * j], v[4 * j + 1], v[4 * j + 2], v[4 * j + 3]);
        } else {
            uint32_t packed[8];
#pragma unroll
            for (int j = 0; j < 8; j++)
                packed[j] = (uint32_t)bf16_bits(v[2 * j]) | ((uint32_t)bf16_bits(v[2 * j + 1]) << 16);
            uint4* o4 = reinterpret_cast<uint4*>(o);
            o4[0] = make_uint4(packed[0], packed[1], packed[2], packed[3]);
            o4[1] = make_uint4(packed[4], packed[5], packed[6], packed[7]);
            if (lo_offset > 0) {
                // second and third bf16 term: what the roundings before dropped (each difference is
                // exact in f32; three terms of eight bits hold the 24-bit value)
                uint32_t third[8];
#pragma unroll
                for (int j = 0; j < 8; j++) {
                    const float r0 = v[2 * j] - round_bf16(v[2 * j]);
                    const float r1 = v[2 * j + 1] - round_bf16(v[2 * j + 1]);
                    packed[j] = (uint32_t)bf16_bits(r0) | ((uint32_t)bf16_bits(r1) << 16);
                    third[j] = (uint32_t)bf16_bits(r0 - round_bf16(r0)) | ((uint32_t)bf16_bits(r1 - round_bf16(r1)) << 16);
                }
                uint4* t4 = reinterpret_cast<uint4*>(o + 2 * lo_offset);
                t4[0] = make_uint4(third[0], third[1], third[2], third[3]);
                t4[1] = make_uint4(third[4], third[5], third[6], third[7]);
                uint4* l4 = reinterpret_cast<uint4*>(o + lo_offset);
                l4[0] = make_uint4(packed[0], packed[1], packed[2], packed[3]);
                l4[1] = make_uint4(packed[4], packed[5], packed[6], packed[7]);
            }
        }
    }
}

template <typename OUT>
static int launch_dequant(const velox_sm100_view* v, OUT* out, long long ld_out, long long lo_offset,
                          const uint32_t* ids = nullptr, int count = 0) {
    if (v->k % 16 != 0 || (reinterpret_cast<uintptr_t>(v->w) & 15)) return VELOX_ERR_UNSUPPORTED;   // 16-byte loads
    const int rows = ids ? count : v->rows;
    const long long total = (long long)rows * (v->k / 16);
    long long blocks = (total + 255) / 256;
    if (blocks > 148 * 16) blocks = 148 * 16;
    if (blocks < 1) blocks = 1;
    cudaStream_t s = stream();
    TimedRegion timed(TIMED_DEQUANT);
    switch (v->format) {
        case VELOX_FMT_NVFP4:
            dequant_rows_kernel<VELOX_FMT_NVFP4, OUT><<<(unsigned)blocks, 256, 0, s>>>(
                v->w, v->n, v->k, v->row_begin, rows, out, ld_out, lo_offset, ids);
            break;
        case VELOX_FMT_FP8_ROW_BF16:
            dequant_rows_kernel<VELOX_FMT_FP8_ROW_BF16, OUT><<<(unsigned)blocks, 256, 0, s>>>(
                v->w, v->n, v->k, v->row_begin, rows, out, ld_out, lo_offset, ids);
            break;
        case VELOX_FMT_GGML_Q4_K:
            dequant_rows_kernel<VELOX_FMT_GGML_Q4_K, OUT><<<(unsigned)blocks, 256, 0, s>>>(
                v->w, v->n, v->k, v->row_begin, rows, out, ld_out, lo_offset, ids);
            break;
        default:
            return VELOX_ERR_UNSUPPORTED;
    }
    return launch_status();
}

int dequant_rows_f32(const velox_sm100_view* v, float* out) { return launch_dequant<float>(v, out, v->k, 0); }

int embed_rows_f32(const velox_sm100_view* v, const uint32_t* ids, int count, float* out) {
    return launch_dequant<float>(v, out, v->k, 0, ids, count);
}

int dequant_rows_bf16(const velox_sm100_view* v, uint16_t* out, long long ld_out, long long lo_offset) {
    return launch_dequant<uint16_t>(v, out, ld_out, lo_offset);
}

}  // namespace vx
