// Activation quantisers for the tensor-core GEMM operands, and the NVFP4 weight constructor.
// Every step is the single-precision operation, in the order, that quant::quantize_activations
// performs on the host (crates/velox-core/src/quant.rs:63-96), so codes and scales agree bit for
// bit; the final conversions are the hardware cvt.rn.satfinite the reference's converters restate
// (quant.rs:9-59).
#include "common.cuh"
#include "kernels.cuh"

namespace vx {

__device__ __forceinline__ float load_act(const float* x, const uint16_t* xb, long long i) {
    return xb ? bf16_bits_to_f32(xb[i]) : x[i];
}

// Fp8Row: scale = amax / 448, inv = 1 / scale, code = e4m3(x * inv). One block per row.
__global__ void __launch_bounds__(256)
quantize_fp8row_kernel(const float* __restrict__ x, const uint16_t* __restrict__ xb, long long k,
                       uint8_t* __restrict__ codes, float* __restrict__ scales) {
    __shared__ float red[8];
    const long long row = blockIdx.x;
    if (threadIdx.x == 0) grid_launch_dependents();   // the linear behind this may start fetching weights
    grid_dependency_wait();                           // (launched early itself: x, and readers of the old codes)
    float amax = 0.0f;
    for (long long c = threadIdx.x; c < k; c += blockDim.x)
        amax = fmaxf(amax, fabsf(load_act(x, xb, row * k + c)));
    amax = warp_max(amax);
    if (threadIdx.x % VX_WARP == 0) red[threadIdx.x / VX_WARP] = amax;
    __syncthreads();
    amax = red[0];
#pragma unroll
    for (int i = 1; i < 8; i++) amax = fmaxf(amax, red[i]);
    const float scale = __fdiv_rn(amax, 448.0f);
    const float inv = scale > 0.0f ? __fdiv_rn(1.0f, scale) : 0.0f;
    if (threadIdx.x == 0) scales[row] = scale;
    for (long long c = threadIdx.x; c < k; c += blockDim.x)
        codes[row * k + c] = (uint8_t)f32_to_e4m3(__fmul_rn(load_act(x, xb, row * k + c), inv));
}

// Nvfp4{divisor}: per 16 values s = e4m3(divisor * amax / 6), code = e2m1(x * divisor / e4m3(s)).
// One thread per group. Rows m..rows_padded get zero scales and codes so whole scale atoms are
// defined.
__global__ void __launch_bounds__(256)
quantize_nvfp4_kernel(const float* __restrict__ x, const uint16_t* __restrict__ xb, int m,
                      int rows_padded, long long k, float divisor, uint8_t* __restrict__ codes,
                      uint8_t* __restrict__ scale_atoms) {
    const long long groups = k / 16;
    const long long total = (long long)rows_padded * groups;
    if (threadIdx.x == 0) grid_launch_dependents();   // the linear behind this may start fetching weights
    grid_dependency_wait();                           // (launched early itself: x, and readers of the old codes)
    for (long long idx = blockIdx.x * (long long)blockDim.x + threadIdx.x; idx < total;
         idx += (long long)gridDim.x * blockDim.x) {
        const long long row = idx / groups, g = idx % groups;
        uint32_t out[2] = {0, 0};
        uint32_t s = 0;
        if (row < m) {
            float v[16];
            const long long base = row * k + g * 16;
            if (xb) {
                const uint4 a = *reinterpret_cast<const uint4*>(xb + base);
                const uint4 b = *reinterpret_cast<const uint4*>(xb + base + 8);
                const uint32_t u[8] = {a.x, a.y, a.z, a.w, b.x, b.y, b.z, b.w};
#pragma unroll
                for (int i = 0; i < 8; i++) {
                    v[2 * i] = __uint_as_float(u[i] << 16);
                    v[2 * i + 1] = __uint_as_float(u[i] & 0xffff0000u);
                }
            } else {
#pragma unroll
                for (int i = 0; i < 4; i++) {
                    const float4 f = *reinterpret_cast<const float4*>(x + base + 4 * i);
                    v[4 * i] = f.x; v[4 * i + 1] = f.y; v[4 * i + 2] = f.z; v[4 * i + 3] = f.w;
                }
            }
            float amax = 0.0f;
#pragma unroll
            for (int i = 0; i < 16; i++) amax = fmaxf(amax, fabsf(v[i]));
            s = f32_to_e4m3(__fdiv_rn(__fmul_rn(divisor, amax), 6.0f));
            if (s != 0) {
                const float ds = e4m3_to_f32(s);
#pragma unroll
                for (int i = 0; i < 8; i++) {
                    const float lo = __fdiv_rn(__fmul_rn(v[2 * i], divisor), ds);
                    const float hi = __fdiv_rn(__fmul_rn(v[2 * i + 1], divisor), ds);
                    out[i >> 2] |= f32x2_to_e2m1x2(lo, hi) << (8 * (i & 3));
                }
            }
            *reinterpret_cast<uint2*>(codes + base / 2) = make_uint2(out[0], out[1]);
        }
        scale_atoms[nvfp4_scale_offset(row, g, k)] = (uint8_t)s;
    }
}

// NVFP4 weight payload from f32 [n, k]: divisor = 448*6/amax (format.rs:392), block scales and
// codes as the activation quantiser above with that divisor, written in the stored layout.
__global__ void __launch_bounds__(256)
encode_nvfp4_kernel(const float* __restrict__ w, long long n, long long k, float divisor,
                    uint8_t* __restrict__ payload) {
    const long long groups = k / 16;
    const long long total = n * groups;
    const long long scale_plane = align256(n * k / 2);
    if (blockIdx.x == 0 && threadIdx.x == 0)
        *reinterpret_cast<float*>(payload + scale_plane + n * k / 16) = divisor;
    for (long long idx = blockIdx.x * (long long)blockDim.x + threadIdx.x; idx < total;
         idx += (long long)gridDim.x * blockDim.x) {
        const long long row = idx / groups, g = idx % groups;
        const long long base = row * k + g * 16;
        float v[16];
#pragma unroll
        for (int i = 0; i < 4; i++) {
            const float4 f = *reinterpret_cast<const float4*>(w + base + 4 * i);
            v[4 * i] = f.x; v[4 * i + 1] = f.y; v[4 * i + 2] = f.z; v[4 * i + 3] = f.w;
        }
        float amax = 0.0f;
#pragma unroll
        for (int i = 0; i < 16; i++) amax = fmaxf(amax, fabsf(v[i]));
        const uint32_t s = f32_to_e4m3(__fdiv_rn(__fmul_rn(divisor, amax), 6.0f));
        uint32_t out[2] = {0, 0};
        if (s != 0) {
            const float ds = e4m3_to_f32(s);
#pragma unroll
            for (int i = 0; i < 8; i++) {
                const float lo = __fdiv_rn(__fmul_rn(v[2 * i], divisor), ds);
                const float hi = __fdiv_rn(__fmul_rn(v[2 * i + 1], divisor), ds);
                out[i >> 2] |= f32x2_to_e2m1x2(lo, hi) << (8 * (i & 3));
            }
        }
        *reinterpret_cast<uint2*>(payload + base / 2) = make_uint2(out[0], out[1]);
        payload[scale_plane + nvfp4_scale_offset(row, g, k)] = (uint8_t)s;
    }
}

static unsigned grid_for(long long total) {
    long long b = (total + 255) / 256;
    if (b > 148 * 16) b = 148 * 16;
    return (unsigned)(b < 1 ? 1 : b);
}

int quantize_act_fp8row(const float* x, const uint16_t* xb, int m, long long k, uint8_t* codes,
                        float* scales) {
    if (m < 1 || k < 1) return VELOX_ERR_SHAPE;
    TimedRegion timed(TIMED_ACT_QUANT);
    EarlyLaunch l((unsigned)m, 256u);
    const cudaError_t e = cudaLaunchKernelEx(&l.cfg, quantize_fp8row_kernel, x, xb, k, codes, scales);
    note_launch();
    return e != cudaSuccess ? (int)e : (int)cudaGetLastError();
}

int quantize_act_nvfp4(const float* x, const uint16_t* xb, int m, long long k, float divisor,
                       uint8_t* codes, uint8_t* scale_atoms) {
    if (m < 1 || k < 64 || k % 64 != 0) return VELOX_ERR_SHAPE;
    const int rows_padded = (m + 127) / 128 * 128;
    TimedRegion timed(TIMED_ACT_QUANT);
    EarlyLaunch l(grid_for((long long)rows_padded * (k / 16)), 256u);
    const cudaError_t e = cudaLaunchKernelEx(&l.cfg, quantize_nvfp4_kernel, x, xb, m, rows_padded, k, divisor, codes,
                                             scale_atoms);
    note_launch();
    return e != cudaSuccess ? (int)e : (int)cudaGetLastError();
}

// The same launch without the optional event timing (which creates events): for callers that must
// not allocate anything.
int quantize_act_nvfp4_untimed(const uint16_t* xb, int m, long long k, float divisor, uint8_t* codes,
                               uint8_t* scale_atoms) {
    if (m < 1 || k < 64 || k % 64 != 0) return VELOX_ERR_SHAPE;
    const int rows_padded = (m + 127) / 128 * 128;
    quantize_nvfp4_kernel<<<grid_for((long long)rows_padded * (k / 16)), 256, 0, stream()>>>(
        nullptr, xb, m, rows_padded, k, divisor, codes, scale_atoms);
    return launch_status();
}

int encode_nvfp4(const float* w, long long n, long long k, float amax, uint8_t* payload) {
    if (n < 128 || n % 128 != 0 || k < 64 || k % 64 != 0) return VELOX_ERR_SHAPE;
    const float divisor = amax > 0.0f ? 448.0f * 6.0f / amax : 1.0f;
    encode_nvfp4_kernel<<<grid_for(n * (k / 16)), 256, 0, stream()>>>(w, n, k, divisor, payload);
    return launch_status();
}

}  // namespace vx
