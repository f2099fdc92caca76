/*
 * TEST INFRASTRUCTURE ONLY: see velox_oracle.h. CPU restatement of velox-inferer's oracle for
 * the quantized-linear path. Compile with -ffp-contract=off (the Makefile does): the reference
 * does every single-precision step as a separate rounding.
 */
#include "velox_oracle.h"

#include <math.h>
#include <stdlib.h>
#include <string.h>
#ifdef _OPENMP
#include <omp.h>
#endif

/* ---------------------------------------------------------------------------------------------
 * scalar converters
 * ------------------------------------------------------------------------------------------- */

static float bits_f32(uint32_t u) {
    float f;
    memcpy(&f, &u, 4);
    return f;
}
static uint32_t f32_bits(float f) {
    uint32_t u;
    memcpy(&u, &f, 4);
    return u;
}

/* format.rs:306-308 */
float vo_bf16_to_f32(uint16_t bits) { return bits_f32((uint32_t)bits << 16); }

/* format.rs:311-317: round to nearest even, NaN kept quiet. */
uint16_t vo_f32_to_bf16(float v) {
    uint32_t b = f32_bits(v);
    if (v != v) return (uint16_t)((b >> 16) | 0x40);
    return (uint16_t)((b + 0x7fffu + ((b >> 16) & 1u)) >> 16);
}

/* format.rs:179-195 */
float vo_f16_to_f32(uint16_t h) {
    float sign = (h & 0x8000) ? -1.0f : 1.0f;
    int e = (h >> 10) & 0x1f;
    float m = (float)(h & 0x3ff);
    if (e == 0) return sign * m * ldexpf(1.0f, -24);
    if (e == 31) return m == 0.0f ? sign * INFINITY : NAN;
    return sign * (1.0f + m / 1024.0f) * ldexpf(1.0f, e - 15);
}

/* f32 -> binary16, round to nearest even, overflow to infinity. Not in the reference's linear
 * path; the Q4_K quantiser below needs it to store d and dmin. */
uint16_t vo_f32_to_f16(float v) {
    uint32_t b = f32_bits(v);
    uint16_t sign = (uint16_t)((b >> 16) & 0x8000);
    uint32_t a = b & 0x7fffffffu;
    if (a > 0x7f800000u) return sign | 0x7e00;
    if (a >= 0x47800000u) return sign | 0x7c00; /* >= 65536: inf (65520.. rounds to inf below) */
    float af = bits_f32(a);
    if (af < ldexpf(1.0f, -14)) {
        /* subnormal: step 2^-24 */
        float q = rintf(af * ldexpf(1.0f, 24));
        return sign | (uint16_t)q; /* q == 1024 lands on the smallest normal */
    }
    int e;
    frexpf(af, &e); /* af = f * 2^e, f in [0.5, 1) */
    e -= 1;         /* af in [2^e, 2^(e+1)) */
    float q = rintf((af / ldexpf(1.0f, e) - 1.0f) * 1024.0f);
    int qi = (int)q;
    if (qi == 1024) {
        qi = 0;
        e += 1;
    }
    if (e > 15) return sign | 0x7c00;
    return sign | (uint16_t)(((e + 15) << 10) | qi);
}

/* format.rs:320-332: E4M3FN, bias 7, no infinities, 0x7f / 0xff are NaN. */
float vo_e4m3fn_to_f32(uint8_t b) {
    float sign = (b & 0x80) ? -1.0f : 1.0f;
    int e = (b >> 3) & 0xf;
    float m = (float)(b & 7);
    if (e == 15 && (b & 7) == 7) return NAN;
    if (e == 0) return sign * m * ldexpf(1.0f, -9);
    return sign * (1.0f + m / 8.0f) * ldexpf(1.0f, e - 7);
}

/* format.rs:335-343 */
float vo_e2m1_to_f32(uint8_t c) {
    static const float V[8] = {0.0f, 0.5f, 1.0f, 1.5f, 2.0f, 3.0f, 4.0f, 6.0f};
    float v = V[c & 7];
    return (c & 8) ? -v : v;
}

/* format.rs:357-379: nearest non-negative code, saturating at 448, ties to the lower code. */
uint8_t vo_f32_to_e4m3fn_lower(float x) {
    if (!(x > 0.0f)) return 0;
    uint8_t lo = 0, hi = 0x7e;
    if (x >= vo_e4m3fn_to_f32(hi)) return hi;
    while (hi - lo > 1) {
        uint8_t mid = (uint8_t)(lo + (hi - lo) / 2);
        if (vo_e4m3fn_to_f32(mid) <= x)
            lo = mid;
        else
            hi = mid;
    }
    return (x - vo_e4m3fn_to_f32(lo) <= vo_e4m3fn_to_f32(hi) - x) ? lo : hi;
}

/* floor(log2(a)) for finite a > 0, exact. The reference computes log2().floor() and then repairs
 * an off-by-one, which lands on this value (quant.rs:21-30). */
static int floor_log2f(float a) {
    int e;
    frexpf(a, &e);
    return e - 1;
}

/* quant.rs:11-41: round to nearest even, saturating to +-448; NaN -> 0x7f. */
uint8_t vo_f32_to_e4m3fn(float x) {
    if (x != x) return 0x7f;
    uint8_t sign = signbit(x) ? 0x80 : 0;
    float a = fabsf(x);
    uint8_t code;
    if (a < ldexpf(1.0f, -6)) {
        code = (uint8_t)rintf(a * 512.0f);
    } else if (isinf(a)) {
        code = 0x7e;
    } else {
        int e = floor_log2f(a);
        int q = (int)rintf((a / ldexpf(1.0f, e) - 1.0f) * 8.0f);
        if (q == 8) {
            e += 1;
            q = 0;
        }
        if (e > 8) {
            code = 0x7e;
        } else {
            int c = ((e + 7) << 3) | q;
            code = (uint8_t)(c < 0x7e ? c : 0x7e);
        }
    }
    return sign | code;
}

/* quant.rs:43-59: round to nearest even, saturating to +-6. */
uint8_t vo_f32_to_e2m1(float x) {
    uint8_t sign = signbit(x) ? 8 : 0;
    float a = fabsf(x);
    uint8_t code;
    if (a != a) {
        code = 7;
    } else if (a < 1.0f) {
        code = (uint8_t)rintf(a * 2.0f);
    } else if (a < 2.0f) {
        code = (uint8_t)(2 + (uint8_t)rintf((a - 1.0f) * 2.0f));
    } else if (a < 4.0f) {
        code = (uint8_t)(4 + (uint8_t)rintf(a - 2.0f));
    } else {
        float r = rintf((a - 4.0f) * 0.5f);
        unsigned v = r >= 250.0f ? 255u : 6u + (unsigned)r; /* saturating_add on u8 */
        code = (uint8_t)(v < 7 ? v : 7);
    }
    return sign | code;
}

/* ---------------------------------------------------------------------------------------------
 * layout
 * ------------------------------------------------------------------------------------------- */

size_t vo_align256(size_t x) { return (x + 255) / 256 * 256; }

/* format.rs:345-354 */
size_t vo_nvfp4_scale_offset(size_t n, size_t g, size_t k) {
    size_t k_tiles = k / 64;
    size_t row_tile = n / 128, row_inner = n % 128;
    size_t scale_tile = g / 4, scale_lane = g % 4;
    return (row_tile * k_tiles + scale_tile) * 512 + (row_inner % 32) * 16 + (row_inner / 32) * 4 +
           scale_lane;
}

/* format.rs:117-145 */
int vo_check_shape(int fmt, size_t n, size_t k) {
    if (n == 0 || k == 0) return -2;
    if (fmt == VO_FMT_NVFP4 && (n % 128 != 0 || k % 64 != 0)) return -2;
    if (fmt == VO_FMT_GGML_Q4_K && k % 256 != 0) return -2;
    if (fmt != VO_FMT_F32 && fmt != VO_FMT_BF16 && fmt != VO_FMT_FP8_ROW_BF16 &&
        fmt != VO_FMT_NVFP4 && fmt != VO_FMT_GGML_Q4_K)
        return -2;
    return 0;
}

/* format.rs:147-160 */
size_t vo_payload_bytes(int fmt, size_t n, size_t k) {
    switch (fmt) {
        case VO_FMT_F32: return n * k * 4;
        case VO_FMT_BF16: return n * k * 2;
        case VO_FMT_FP8_ROW_BF16: return vo_align256(n * k) + 2 * n;
        case VO_FMT_NVFP4: return vo_align256(n * k / 2) + n * k / 16 + 4;
        case VO_FMT_GGML_Q4_K: return n * (k / 256) * 144;
        default: return 0;
    }
}

/* ---------------------------------------------------------------------------------------------
 * decoders
 * ------------------------------------------------------------------------------------------- */

/* ggml.rs:159-169 */
static void scale_min_k4(int j, const uint8_t* q, uint8_t* sc, uint8_t* mn) {
    if (j < 4) {
        *sc = q[j] & 63;
        *mn = q[j + 4] & 63;
    } else {
        *sc = (uint8_t)((q[j + 4] & 0xf) | ((q[j - 4] >> 6) << 4));
        *mn = (uint8_t)((q[j + 4] >> 4) | ((q[j] >> 6) << 4));
    }
}

/* ggml.rs:196-210: block = d | dmin | scales[12] | qs[128]. */
void vo_q4k_decode_block(const uint8_t* x, float* y) {
    float d = vo_f16_to_f32((uint16_t)(x[0] | (x[1] << 8)));
    float min = vo_f16_to_f32((uint16_t)(x[2] | (x[3] << 8)));
    const uint8_t* scales = x + 4;
    for (int c = 0; c < 4; c++) {
        const uint8_t* q = x + 16 + 32 * c;
        uint8_t sc1, m1, sc2, m2;
        scale_min_k4(2 * c, scales, &sc1, &m1);
        scale_min_k4(2 * c + 1, scales, &sc2, &m2);
        float d1 = d * (float)sc1, mm1 = min * (float)m1;
        float d2 = d * (float)sc2, mm2 = min * (float)m2;
        for (int l = 0; l < 32; l++) {
            y[64 * c + l] = d1 * (float)(q[l] & 0xf) - mm1;
            y[64 * c + 32 + l] = d2 * (float)(q[l] >> 4) - mm2;
        }
    }
}

/* format.rs:426-490 */
int vo_decode_rows(int fmt, const uint8_t* payload, size_t payload_len, size_t n, size_t k,
                   size_t row_begin, size_t rows, float* out) {
    if (vo_check_shape(fmt, n, k) != 0) return -2;
    if (payload_len < vo_payload_bytes(fmt, n, k) || row_begin + rows > n) return -2;
    for (size_t i = 0; i < rows; i++) {
        size_t r = row_begin + i;
        float* o = out + i * k;
        switch (fmt) {
            case VO_FMT_F32:
                memcpy(o, payload + r * k * 4, k * 4);
                break;
            case VO_FMT_BF16:
                for (size_t c = 0; c < k; c++) {
                    const uint8_t* p = payload + (r * k + c) * 2;
                    o[c] = vo_bf16_to_f32((uint16_t)(p[0] | (p[1] << 8)));
                }
                break;
            case VO_FMT_FP8_ROW_BF16: {
                size_t so = vo_align256(n * k) + 2 * r;
                float scale = vo_bf16_to_f32((uint16_t)(payload[so] | (payload[so + 1] << 8)));
                for (size_t c = 0; c < k; c++) o[c] = vo_e4m3fn_to_f32(payload[r * k + c]) * scale;
                break;
            }
            case VO_FMT_NVFP4: {
                size_t scale_plane = vo_align256(n * k / 2);
                size_t div_off = scale_plane + n * k / 16;
                float divisor;
                memcpy(&divisor, payload + div_off, 4);
                for (size_t c = 0; c < k; c++) {
                    uint8_t byte = payload[(r * k + c) / 2];
                    uint8_t code = (c % 2 == 0) ? (byte & 0xf) : (byte >> 4);
                    float scale = vo_e4m3fn_to_f32(
                        payload[scale_plane + vo_nvfp4_scale_offset(r, c / 16, k)]);
                    o[c] = vo_e2m1_to_f32(code) * scale / divisor;
                }
                break;
            }
            case VO_FMT_GGML_Q4_K: {
                size_t rb = k / 256 * 144;
                for (size_t b = 0; b < k / 256; b++)
                    vo_q4k_decode_block(payload + r * rb + b * 144, o + b * 256);
                break;
            }
            default:
                return -2;
        }
    }
    return 0;
}

/* ---------------------------------------------------------------------------------------------
 * encoders
 * ------------------------------------------------------------------------------------------- */

static void put_nibble(uint8_t* out, size_t idx, uint8_t code) {
    out[idx / 2] |= (idx % 2 == 0) ? code : (uint8_t)(code << 4);
}

/* format.rs:385-423: divisor 448*6/amax, per 16 values an E4M3 scale of amax16/6*divisor, each
 * value the nearest E2M1 magnitude of |x|/step with ties to the lower one. */
void vo_encode_nvfp4_ref(const float* x, size_t n, size_t k, uint8_t* out) {
    static const float MAG[8] = {0.0f, 0.5f, 1.0f, 1.5f, 2.0f, 3.0f, 4.0f, 6.0f};
    float amax = 0.0f;
    for (size_t i = 0; i < n * k; i++) amax = fmaxf(amax, fabsf(x[i]));
    float divisor = amax > 0.0f ? 448.0f * 6.0f / amax : 1.0f;
    size_t scale_plane = vo_align256(n * k / 2);
    memset(out, 0, scale_plane + n * k / 16 + 4);
    for (size_t r = 0; r < n; r++) {
        for (size_t g = 0; g < k / 16; g++) {
            const float* blk = x + r * k + g * 16;
            float bmax = 0.0f;
            for (int j = 0; j < 16; j++) bmax = fmaxf(bmax, fabsf(blk[j]));
            uint8_t sc = vo_f32_to_e4m3fn_lower(bmax / 6.0f * divisor);
            out[scale_plane + vo_nvfp4_scale_offset(r, g, k)] = sc;
            float step = vo_e4m3fn_to_f32(sc) / divisor;
            if (step <= 0.0f) continue;
            for (int j = 0; j < 16; j++) {
                float v = blk[j];
                float q = fminf(fabsf(v) / step, 6.0f);
                uint8_t code = 0;
                for (int c = 1; c < 8; c++)
                    if (q - MAG[c - 1] > MAG[c] - q) code = (uint8_t)c;
                if (v < 0.0f && code != 0) code |= 8;
                put_nibble(out, r * k + g * 16 + (size_t)j, code);
            }
        }
    }
    memcpy(out + scale_plane + n * k / 16, &divisor, 4);
}

/* Benchmark construction: as above but with the RNE converters of quant.rs, in the operation
 * order of the activation quantiser (quant.rs:81-96): s = e4m3(divisor*amax16/6),
 * code = e2m1(w*divisor/e4m3(s)). */
void vo_encode_nvfp4_rne(const float* x, size_t n, size_t k, uint8_t* out) {
    float amax = 0.0f;
    for (size_t i = 0; i < n * k; i++) amax = fmaxf(amax, fabsf(x[i]));
    float divisor = amax > 0.0f ? 448.0f * 6.0f / amax : 1.0f;
    size_t scale_plane = vo_align256(n * k / 2);
    memset(out, 0, scale_plane + n * k / 16 + 4);
#pragma omp parallel for schedule(static)
    for (size_t r = 0; r < n; r++) {
        for (size_t g = 0; g < k / 16; g++) {
            const float* blk = x + r * k + g * 16;
            float bmax = 0.0f;
            for (int j = 0; j < 16; j++) bmax = fmaxf(bmax, fabsf(blk[j]));
            uint8_t sc = vo_f32_to_e4m3fn(divisor * bmax / 6.0f);
            out[scale_plane + vo_nvfp4_scale_offset(r, g, k)] = sc;
            float ds = vo_e4m3fn_to_f32(sc);
            if (sc == 0) continue;
            for (int j = 0; j < 16; j += 2) {
                uint8_t lo = vo_f32_to_e2m1(blk[j] * divisor / ds);
                uint8_t hi = vo_f32_to_e2m1(blk[j + 1] * divisor / ds);
                out[(r * k + g * 16 + (size_t)j) / 2] = (uint8_t)(lo | (hi << 4));
            }
        }
    }
    memcpy(out + scale_plane + n * k / 16, &divisor, 4);
}

void vo_encode_fp8_row(const float* x, size_t n, size_t k, uint8_t* out) {
    size_t plane = vo_align256(n * k);
    memset(out, 0, plane + 2 * n);
#pragma omp parallel for schedule(static)
    for (size_t r = 0; r < n; r++) {
        float amax = 0.0f;
        for (size_t c = 0; c < k; c++) amax = fmaxf(amax, fabsf(x[r * k + c]));
        uint16_t sb = vo_f32_to_bf16(amax / 448.0f);
        float scale = vo_bf16_to_f32(sb);
        out[plane + 2 * r] = (uint8_t)(sb & 0xff);
        out[plane + 2 * r + 1] = (uint8_t)(sb >> 8);
        for (size_t c = 0; c < k; c++) {
            float q = scale > 0.0f ? x[r * k + c] / scale : 0.0f;
            out[r * k + c] = vo_f32_to_e4m3fn(q);
        }
    }
}

static int clampi(int v, int lo, int hi) { return v < lo ? lo : (v > hi ? hi : v); }

void vo_encode_q4k(const float* x, size_t n, size_t k, uint8_t* out) {
    size_t blocks = k / 256;
#pragma omp parallel for schedule(static)
    for (size_t r = 0; r < n; r++) {
        for (size_t b = 0; b < blocks; b++) {
            const float* v = x + r * k + b * 256;
            uint8_t* blk = out + (r * blocks + b) * 144;
            float sub_scale[8], sub_min[8];
            float max_scale = 0.0f, max_min = 0.0f;
            for (int j = 0; j < 8; j++) {
                float lo = 0.0f, hi = 0.0f;
                for (int l = 0; l < 32; l++) {
                    lo = fminf(lo, v[32 * j + l]);
                    hi = fmaxf(hi, v[32 * j + l]);
                }
                sub_min[j] = -lo;
                sub_scale[j] = (hi - lo) / 15.0f;
                max_scale = fmaxf(max_scale, sub_scale[j]);
                max_min = fmaxf(max_min, sub_min[j]);
            }
            uint16_t dh = vo_f32_to_f16(max_scale / 63.0f);
            uint16_t mh = vo_f32_to_f16(max_min / 63.0f);
            float d = vo_f16_to_f32(dh), dmin = vo_f16_to_f32(mh);
            uint8_t sc[8], mn[8];
            for (int j = 0; j < 8; j++) {
                sc[j] = (uint8_t)(d > 0.0f ? clampi((int)rintf(sub_scale[j] / d), 0, 63) : 0);
                mn[j] = (uint8_t)(dmin > 0.0f ? clampi((int)rintf(sub_min[j] / dmin), 0, 63) : 0);
            }
            memset(blk, 0, 144);
            blk[0] = (uint8_t)(dh & 0xff);
            blk[1] = (uint8_t)(dh >> 8);
            blk[2] = (uint8_t)(mh & 0xff);
            blk[3] = (uint8_t)(mh >> 8);
            uint8_t* s = blk + 4;
            for (int j = 0; j < 4; j++) {
                s[j] = (uint8_t)((sc[j] & 63) | ((sc[j + 4] >> 4) << 6));
                s[j + 4] = (uint8_t)((mn[j] & 63) | ((mn[j + 4] >> 4) << 6));
                s[j + 8] = (uint8_t)((sc[j + 4] & 0xf) | ((mn[j + 4] & 0xf) << 4));
            }
            for (int c = 0; c < 4; c++) {
                for (int half = 0; half < 2; half++) {
                    int j = 2 * c + half;
                    float dj = d * (float)sc[j], mj = dmin * (float)mn[j];
                    for (int l = 0; l < 32; l++) {
                        int q = dj > 0.0f ? clampi((int)rintf((v[32 * j + l] + mj) / dj), 0, 15) : 0;
                        blk[16 + 32 * c + l] |= (uint8_t)(half == 0 ? q : (q << 4));
                    }
                }
            }
        }
    }
}

/* ---------------------------------------------------------------------------------------------
 * activation rounding: quant.rs:63-96
 * ------------------------------------------------------------------------------------------- */

void vo_quantize_activations(float* x, size_t rows, size_t k, int act, float divisor) {
    size_t total = rows * k;
    switch (act) {
        case VO_ACT_EXACT:
            break;
        case VO_ACT_BF16:
            for (size_t i = 0; i < total; i++) x[i] = vo_bf16_to_f32(vo_f32_to_bf16(x[i]));
            break;
        case VO_ACT_FP8_ROW:
            for (size_t r = 0; r < rows; r++) {
                float* row = x + r * k;
                float amax = 0.0f;
                for (size_t c = 0; c < k; c++) amax = fmaxf(amax, fabsf(row[c]));
                float scale = amax / 448.0f;
                float inv = scale > 0.0f ? 1.0f / scale : 0.0f;
                for (size_t c = 0; c < k; c++)
                    row[c] = vo_e4m3fn_to_f32(vo_f32_to_e4m3fn(row[c] * inv)) * scale;
            }
            break;
        case VO_ACT_NVFP4:
            /* chunks of 16 over the whole buffer (k % 16 == 0 wherever this is used) */
            for (size_t g = 0; g + 16 <= total; g += 16) {
                float* grp = x + g;
                float amax = 0.0f;
                for (int j = 0; j < 16; j++) amax = fmaxf(amax, fabsf(grp[j]));
                uint8_t s = vo_f32_to_e4m3fn(divisor * amax / 6.0f);
                float ds = vo_e4m3fn_to_f32(s);
                for (int j = 0; j < 16; j++) {
                    if (s == 0) {
                        grp[j] = 0.0f;
                    } else {
                        uint8_t code = vo_f32_to_e2m1(grp[j] * divisor / ds);
                        grp[j] = (float)((double)vo_e2m1_to_f32(code) * (double)ds /
                                         (double)divisor);
                    }
                }
            }
            break;
        default:
            break;
    }
}

void vo_act_codes_fp8(const float* x, size_t rows, size_t k, uint8_t* codes, float* scales) {
    for (size_t r = 0; r < rows; r++) {
        const float* row = x + r * k;
        float amax = 0.0f;
        for (size_t c = 0; c < k; c++) amax = fmaxf(amax, fabsf(row[c]));
        float scale = amax / 448.0f;
        float inv = scale > 0.0f ? 1.0f / scale : 0.0f;
        scales[r] = scale;
        for (size_t c = 0; c < k; c++) codes[r * k + c] = vo_f32_to_e4m3fn(row[c] * inv);
    }
}

void vo_act_codes_nvfp4(const float* x, size_t rows, size_t k, float divisor, uint8_t* codes,
                        uint8_t* scales) {
    memset(codes, 0, rows * k / 2);
    for (size_t g = 0; g < rows * k / 16; g++) {
        const float* grp = x + g * 16;
        float amax = 0.0f;
        for (int j = 0; j < 16; j++) amax = fmaxf(amax, fabsf(grp[j]));
        uint8_t s = vo_f32_to_e4m3fn(divisor * amax / 6.0f);
        float ds = vo_e4m3fn_to_f32(s);
        scales[g] = s;
        if (s == 0) continue;
        for (int j = 0; j < 16; j++)
            put_nibble(codes, g * 16 + (size_t)j, vo_f32_to_e2m1(grp[j] * divisor / ds));
    }
}

/* ---------------------------------------------------------------------------------------------
 * ops: crates/velox-cpu/src/lib.rs
 * ------------------------------------------------------------------------------------------- */

/* lib.rs:31-36 */
static double dot(const float* a, const float* b, size_t k) {
    double s = 0.0;
    for (size_t i = 0; i < k; i++) s += (double)a[i] * (double)b[i];
    return s;
}

static int use_threads(int threads) {
#ifdef _OPENMP
    if (threads <= 0) return omp_get_max_threads();
    return threads;
#else
    (void)threads;
    return 1;
#endif
}

/* lib.rs:128-145 */
void vo_matmul(const float* x, const float* w, float* y, size_t m, size_t n, size_t k,
               int threads) {
    int t = use_threads(threads);
    (void)t;
#pragma omp parallel for schedule(static) num_threads(t)
    for (size_t j = 0; j < n; j++)
        for (size_t i = 0; i < m; i++) y[i * n + j] = (float)dot(x + i * k, w + j * k, k);
}

/* lib.rs:147-164 after check::linear (check.rs:100-131). */
int vo_linear(const float* x, size_t x_len, const uint8_t* payload, size_t payload_len, int fmt,
              size_t n, size_t k, size_t row_begin, size_t rows, size_t m, float* y, size_t y_len,
              int threads) {
    if (m == 0) return -2;
    if (vo_check_shape(fmt, n, k) != 0) return -2;
    if (rows == 0 || row_begin + rows > n) return -2;
    if ((payload_len + 3) / 4 < (vo_payload_bytes(fmt, n, k) + 3) / 4) return -2;
    if (x_len < m * k || y_len < m * rows) return -2;
    int t = use_threads(threads);
    (void)t;
    int bad = 0;
    /* Decode and multiply row by row: the same values and the same per-output summation order
     * as decoding the whole view first. */
#pragma omp parallel num_threads(t)
    {
        float* wd = (float*)malloc(k * sizeof(float));
#pragma omp for schedule(static)
        for (size_t j = 0; j < rows; j++) {
            if (!wd || vo_decode_rows(fmt, payload, payload_len, n, k, row_begin + j, 1, wd) != 0) {
                bad = 1;
                continue;
            }
            for (size_t i = 0; i < m; i++) y[i * rows + j] = (float)dot(x + i * k, wd, k);
        }
        free(wd);
    }
    return bad ? -2 : 0;
}

/* lib.rs:38-44, 224-230 */
void vo_silu_mul(float* gate, const float* up, size_t len) {
    for (size_t i = 0; i < len; i++) {
        double g = (double)gate[i];
        double s = g * (1.0 / (1.0 + exp(-g)));
        gate[i] = (float)(s * (double)up[i]);
    }
}

/* lib.rs:688-707 */
void vo_swiglu(const float* src, size_t rows, size_t src_cols, size_t gate, size_t up,
               size_t width, float* out) {
    for (size_t r = 0; r < rows; r++)
        for (size_t i = 0; i < width; i++) {
            double g = (double)src[r * src_cols + gate + i];
            double u = (double)src[r * src_cols + up + i];
            out[r * width + i] = (float)(g / (1.0 + exp(-g)) * u);
        }
}

void vo_add(float* acc, const float* x, size_t len) {
    for (size_t i = 0; i < len; i++) acc[i] += x[i];
}

/* lib.rs:188-207 */
void vo_rms_norm(const float* x, const float* weight, float* y, size_t rows, size_t dim,
                 float eps, int offset) {
    double off = offset ? 1.0 : 0.0;
    for (size_t r = 0; r < rows; r++) {
        const float* xr = x + r * dim;
        double ms = 0.0;
        for (size_t c = 0; c < dim; c++) ms += (double)xr[c] * (double)xr[c];
        ms /= (double)dim;
        double inv = 1.0 / sqrt(ms + (double)eps);
        for (size_t c = 0; c < dim; c++)
            y[r * dim + c] = (float)((double)xr[c] * inv * (off + (double)weight[c]));
    }
}

/* ---------------------------------------------------------------------------------------------
 * generators of the reference's tests
 * ------------------------------------------------------------------------------------------- */

/* rng.rs:6-8 */
void vo_rng_new(vo_rng* r, uint64_t seed) { r->s = (seed * 0x9E3779B97F4A7C15ull) | 1ull; }

/* rng.rs:10-17 */
uint64_t vo_rng_next(vo_rng* r) {
    uint64_t x = r->s;
    x ^= x << 13;
    x ^= x >> 7;
    x ^= x << 17;
    r->s = x;
    return x;
}

/* rng.rs:20-22 */
float vo_rng_uniform(vo_rng* r) {
    return ((float)(vo_rng_next(r) >> 40) / (float)(1ull << 24)) * 2.0f - 1.0f;
}

void vo_rng_vec(vo_rng* r, size_t len, float scale, float* out) {
    for (size_t i = 0; i < len; i++) out[i] = vo_rng_uniform(r) * scale;
}

static uint8_t rng_byte(vo_rng* r) { return (uint8_t)(vo_rng_next(r) >> 56); }

/* conformance lib.rs:114-199 */
int vo_random_weight(vo_rng* r, int fmt, size_t n, size_t k, uint8_t* out) {
    size_t total = vo_payload_bytes(fmt, n, k);
    memset(out, 0, total);
    if (fmt == VO_FMT_FP8_ROW_BF16) {
        for (size_t i = 0; i < n * k; i++) {
            uint8_t b = rng_byte(r);
            out[i] = ((b & 0x7f) == 0x7f) ? (uint8_t)(b & 0xfe) : b;
        }
        size_t plane = vo_align256(n * k);
        for (size_t i = 0; i < n; i++) {
            float scale = 0.001f + 0.01f * (vo_rng_uniform(r) + 1.0f);
            uint16_t sb = vo_f32_to_bf16(scale);
            out[plane + 2 * i] = (uint8_t)(sb & 0xff);
            out[plane + 2 * i + 1] = (uint8_t)(sb >> 8);
        }
        return 0;
    }
    if (fmt == VO_FMT_NVFP4) {
        for (size_t i = 0; i < n * k / 2; i++) out[i] = rng_byte(r);
        size_t plane = vo_align256(n * k / 2);
        for (size_t i = 0; i < n * k / 16; i++) {
            /* argument order as the reference evaluates it: exponent byte first */
            uint8_t e = rng_byte(r);
            uint8_t m = rng_byte(r);
            out[plane + i] = (uint8_t)((((e % 8) + 4) << 3) | (m & 7));
        }
        float d = 96.0f;
        memcpy(out + plane + n * k / 16, &d, 4);
        return 0;
    }
    if (fmt == VO_FMT_GGML_Q4_K) {
        size_t blocks = n * (k / 256);
        for (size_t b = 0; b < blocks; b++) {
            uint8_t* blk = out + b * 144;
            uint8_t bytes[144];
            uint16_t scales[3];
            for (int i = 0; i < 144; i++) bytes[i] = rng_byte(r);
            for (int i = 0; i < 3; i++) {
                uint64_t e = 6 + vo_rng_next(r) % 4;
                uint64_t m = vo_rng_next(r) % 1024;
                scales[i] = (uint16_t)((e << 10) | m);
            }
            memcpy(blk, bytes, 144);
            /* ggml.rs:460-481 with scale_fields(Q4K) = [0, 2] */
            blk[0] = (uint8_t)(scales[0] & 0xff);
            blk[1] = (uint8_t)(scales[0] >> 8);
            blk[2] = (uint8_t)(scales[1] & 0xff);
            blk[3] = (uint8_t)(scales[1] >> 8);
        }
        return 0;
    }
    return -1;
}

/* ggml.rs:4450-4485 for Q4_K (scale fields at bytes 0 and 2). */
void vo_kat_q4k_blocks(uint64_t seed, uint8_t* out) {
    uint64_t s = seed;
#define SM_NEXT(dst)                                   \
    do {                                               \
        s += 0x9E3779B97F4A7C15ull;                    \
        uint64_t z = s;                                \
        z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;   \
        z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;   \
        (dst) = z ^ (z >> 31);                         \
    } while (0)
    size_t size = 144, count = 2;
    for (size_t i = 0; i < count * size; i++) {
        uint64_t v;
        SM_NEXT(v);
        out[i] = (uint8_t)v;
    }
    for (size_t b = 0; b < count; b++) {
        for (int f = 0; f < 2; f++) {
            uint64_t a, c;
            SM_NEXT(a);
            SM_NEXT(c);
            uint16_t h = (uint16_t)(((8 + a % 3) << 10) | (c % 1024));
            out[b * size + 2 * (size_t)f] = (uint8_t)(h & 0xff);
            out[b * size + 2 * (size_t)f + 1] = (uint8_t)(h >> 8);
        }
    }
#undef SM_NEXT
}

/* ---------------------------------------------------------------------------------------------
 * error metrics
 * ------------------------------------------------------------------------------------------- */

/* conformance lib.rs:43-58 */
double vo_max_err(const float* got, const float* want, size_t len) {
    double m = 0.0;
    for (size_t i = 0; i < len; i++) {
        double e = fabs((double)got[i] - (double)want[i]) / (1.0 + fabs((double)want[i]));
        if (e != e) return INFINITY;
        if (e > m) m = e;
    }
    return m;
}

double vo_rms(const float* v, size_t len) {
    double s = 0.0;
    for (size_t i = 0; i < len; i++) s += (double)v[i] * (double)v[i];
    return len ? sqrt(s / (double)len) : 0.0;
}

double vo_max_abs_diff(const float* got, const float* want, size_t len) {
    double m = 0.0;
    for (size_t i = 0; i < len; i++) {
        double e = fabs((double)got[i] - (double)want[i]);
        if (e != e) return INFINITY;
        if (e > m) m = e;
    }
    return m;
}
