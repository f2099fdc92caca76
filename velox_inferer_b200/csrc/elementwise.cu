// Elementwise neighbours of the linear path: the unfused SwiGLU the composed form uses, the
// residual add, RMS norm with its bf16 twin, and the twin conversion. f32 arithmetic; the oracle
// computes these in f64 (crates/velox-cpu/src/lib.rs:188-230, 688-707), results agree to f32
// rounding. Reference kernels: crates/velox-cuda/kernels/portable.cu:109-115, 1519-1550;
// portable_model.cu:2011-2022.
#include "common.cuh"
#include "kernels.cuh"

namespace vx {

static unsigned grid_1d(long long n, int block) {
    long long g = (n + block - 1) / block;
    if (g > 148LL * 32) g = 148LL * 32;
    return (unsigned)(g < 1 ? 1 : g);
}

__device__ __forceinline__ float silu(float g) { return g / (1.0f + expf(-g)); }

__global__ void swiglu_kernel(const float* __restrict__ src, long long rows, int src_cols, int gate,
                              int up, int width, float* __restrict__ out) {
    const long long total = rows * width;
    for (long long idx = blockIdx.x * (long long)blockDim.x + threadIdx.x; idx < total;
         idx += (long long)gridDim.x * blockDim.x) {
        const long long r = idx / width;
        const int i = (int)(idx % width);
        const float g = src[r * src_cols + gate + i];
        const float u = src[r * src_cols + up + i];
        out[idx] = silu(g) * u;
    }
}

__global__ void silu_mul_kernel(float* __restrict__ gate, const float* __restrict__ up, long long len) {
    for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < len;
         i += (long long)gridDim.x * blockDim.x)
        gate[i] = silu(gate[i]) * up[i];
}

__global__ void add_kernel(float* __restrict__ acc, const float* __restrict__ x, long long len) {
    for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < len;
         i += (long long)gridDim.x * blockDim.x)
        acc[i] += x[i];
}

__global__ void bf16_twin_kernel(const float* __restrict__ x, uint16_t* __restrict__ xb, long long len) {
    for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < len;
         i += (long long)gridDim.x * blockDim.x)
        xb[i] = bf16_bits(x[i]);
}

// One block per row: acc += x (when x is given), y = acc * rsqrt(mean(acc^2) + eps) * (offset + weight).
__global__ void __launch_bounds__(256)
add_rms_norm_twin_kernel(float* __restrict__ acc, const float* __restrict__ x,
                         const uint16_t* __restrict__ xb, const float* __restrict__ weight,
                         float* __restrict__ y,
                         uint16_t* __restrict__ yb, int dim, float eps, float offset) {
    __shared__ float red[8];
    const long long base = (long long)blockIdx.x * dim;
    float ss = 0.0f;
    for (int c = threadIdx.x; c < dim; c += blockDim.x) {
        float v = acc[base + c];
        if (x) {
            v += x[base + c];
            acc[base + c] = v;
        } else if (xb) {
            v += bf16_bits_to_f32(xb[base + c]);
            acc[base + c] = v;
        }
        ss = fmaf(v, v, ss);
    }
    ss = warp_sum(ss);
    if (threadIdx.x % VX_WARP == 0) red[threadIdx.x / VX_WARP] = ss;
    __syncthreads();
    float total = 0.0f;
#pragma unroll
    for (int i = 0; i < 8; i++) total += red[i];
    const float inv = 1.0f / sqrtf(total / (float)dim + eps);
    for (int c = threadIdx.x; c < dim; c += blockDim.x) {
        const float v = acc[base + c] * inv * (offset + weight[c]);
        if (y) y[base + c] = v;
        if (yb) yb[base + c] = bf16_bits(v);
    }
}

// The norm above that also writes its result as NVFP4 activations (E2M1 codes + E4M3 scale atoms,
// quantised from the bf16-rounded values exactly as quantize_nvfp4_kernel does), so the projections
// that follow read them without a quantisation pass of their own. The counterpart, for FP4, of the
// reference's add_rms_norm_q8 (crates/velox-core/src/backend.rs:1061-1077). Blocks past `rows`
// (up to the next multiple of 128) only zero their scale bytes so whole atoms are defined.
__global__ void __launch_bounds__(256)
add_rms_norm_q4_kernel(float* __restrict__ acc, const float* __restrict__ x, const uint16_t* __restrict__ xb,
                       const float* __restrict__ weight, uint16_t* __restrict__ yb, uint8_t* __restrict__ codes,
                       uint8_t* __restrict__ atoms, int rows, int dim, float eps, float offset, float divisor) {
    __shared__ float red[8];
    const long long row = blockIdx.x;
    const int groups = dim / 16;
    if (threadIdx.x == 0) grid_launch_dependents();   // a decode linear behind this may start fetching weights
    if (row >= rows) {
        for (int g = threadIdx.x; g < groups; g += blockDim.x) atoms[nvfp4_scale_offset(row, g, dim)] = 0;
        return;
    }
    const long long base = row * dim;
    float ss = 0.0f;
    for (int c = threadIdx.x; c < dim; c += blockDim.x) {
        float v = acc[base + c];
        if (x) {
            v += x[base + c];
            acc[base + c] = v;
        } else if (xb) {
            v += bf16_bits_to_f32(xb[base + c]);
            acc[base + c] = v;
        }
        ss = fmaf(v, v, ss);
    }
    ss = warp_sum(ss);
    if (threadIdx.x % VX_WARP == 0) red[threadIdx.x / VX_WARP] = ss;
    __syncthreads();
    float total = 0.0f;
#pragma unroll
    for (int i = 0; i < 8; i++) total += red[i];
    const float inv = 1.0f / sqrtf(total / (float)dim + eps);
    for (int g = threadIdx.x; g < groups; g += blockDim.x) {
        float v[16];
        float amax = 0.0f;
#pragma unroll
        for (int i = 0; i < 16; i++) {
            const int c = g * 16 + i;
            v[i] = round_bf16(acc[base + c] * inv * (offset + weight[c]));
            amax = fmaxf(amax, fabsf(v[i]));
        }
        if (yb) {
            uint32_t pk[8];
#pragma unroll
            for (int i = 0; i < 8; i++)
                pk[i] = (__float_as_uint(v[2 * i]) >> 16) | (__float_as_uint(v[2 * i + 1]) & 0xffff0000u);
            uint4* o = reinterpret_cast<uint4*>(yb + base + g * 16);
            o[0] = make_uint4(pk[0], pk[1], pk[2], pk[3]);
            o[1] = make_uint4(pk[4], pk[5], pk[6], pk[7]);
        }
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
        *reinterpret_cast<uint2*>(codes + (base + g * 16) / 2) = make_uint2(out[0], out[1]);
        atoms[nvfp4_scale_offset(row, g, dim)] = (uint8_t)s;
    }
}

int add_rms_norm_q4(float* acc, const float* x, const uint16_t* xb, const float* weight, uint16_t* yb,
                    uint8_t* codes, uint8_t* atoms, int rows, int dim, float eps, int offset, float divisor) {
    if (rows < 1 || dim < 64 || dim % 64 != 0 || !(divisor > 0.0f)) return VELOX_ERR_SHAPE;
    const int rows_padded = (rows + 127) / 128 * 128;
    add_rms_norm_q4_kernel<<<(unsigned)rows_padded, 256, 0, stream()>>>(acc, x, xb, weight, yb, codes, atoms, rows,
                                                                         dim, eps, offset ? 1.0f : 0.0f, divisor);
    return launch_status();
}

int swiglu(const float* src, long long rows, int src_cols, int gate, int up, int width, float* out) {
    if (rows < 1 || width < 1 || gate < 0 || up < 0 || gate + width > src_cols || up + width > src_cols)
        return VELOX_ERR_SHAPE;
    swiglu_kernel<<<grid_1d(rows * width, 256), 256, 0, stream()>>>(src, rows, src_cols, gate, up, width, out);
    return launch_status();
}

int silu_mul(float* gate, const float* up, long long len) {
    if (len < 1) return 0;
    silu_mul_kernel<<<grid_1d(len, 256), 256, 0, stream()>>>(gate, up, len);
    return launch_status();
}

int add(float* acc, const float* x, long long len) {
    if (len < 1) return 0;
    add_kernel<<<grid_1d(len, 256), 256, 0, stream()>>>(acc, x, len);
    return launch_status();
}

int bf16_twin(const float* x, uint16_t* xb, long long len) {
    if (len < 1) return 0;
    bf16_twin_kernel<<<grid_1d(len, 256), 256, 0, stream()>>>(x, xb, len);
    return launch_status();
}

__global__ void add_bf16_kernel(float* __restrict__ acc, const uint16_t* __restrict__ xb, long long len) {
    for (long long i = blockIdx.x * (long long)blockDim.x + threadIdx.x; i < len;
         i += (long long)gridDim.x * blockDim.x)
        acc[i] += bf16_bits_to_f32(xb[i]);
}

int add_bf16(float* acc, const uint16_t* xb, long long len) {
    if (len < 1) return 0;
    add_bf16_kernel<<<grid_1d(len, 256), 256, 0, stream()>>>(acc, xb, len);
    return launch_status();
}

int add_rms_norm_twin(float* acc, const float* x, const uint16_t* xb, const float* weight, float* y,
                      uint16_t* yb, int rows, int dim, float eps, int offset) {
    if (rows < 1 || dim < 1) return VELOX_ERR_SHAPE;
    add_rms_norm_twin_kernel<<<(unsigned)rows, 256, 0, stream()>>>(acc, x, xb, weight, y, yb, dim, eps,
                                                                  offset ? 1.0f : 0.0f);
    return launch_status();
}

}  // namespace vx
