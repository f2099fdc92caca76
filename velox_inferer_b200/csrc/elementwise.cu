// Elementwise neighbours of the linear path: the unfused SwiGLU the composed form uses, the
// residual add, RMS norm with its bf16 twin, and the twin conversion. f32 arithmetic; the oracle
// computes these in f64 (crates/velox-cpu/src/lib.rs:188-230, 688-707), results agree to f32
// rounding. Reference kernels: crates/velox-cuda/kernels/portable.cu:109-115, 1519-1550;
// portable_model.cu:2011-2022.
#include <cstdlib>

#include "common.cuh"
#include "kernels.cuh"
#include "tpsync.cuh"

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

// Where the norm's NVFP4 output goes: one blob, or the same rows of the blob on every rank of a
// tensor-parallel group (peer pointers into symmetric memory; plain stores over NVLink).
struct Q4Dest {
    uint8_t* codes[VX_MAX_PEERS];
    uint8_t* atoms[VX_MAX_PEERS];
    int n;
};

// The same for rows of at most ITERS * 1024 values, kept in registers between the two passes: a
// thread owns four consecutive values per 1024-wide slice (coalesced 128-bit accesses), four
// neighbouring lanes own a 16-wide scale group, and the quotients use the Markstein sequence
// (q0 = a*r, q = fma(fma(-q0, d, a), r, q0), the correctly rounded a / d for r = rn(1 / d)), so the
// bytes written are those of the kernel above.
//
// Sequence-parallel form: `acc` holds only this rank's rows; the addend is the sum, in slot order,
// of `nslots` bf16 partial-sum slots (one per source rank, `slot_stride` values apart), and the
// output row lands at row `row0 + row` of every destination blob.
template <int ITERS, int MAXT>
__global__ void __launch_bounds__(MAXT)
add_rms_norm_q4_rows_kernel(float* __restrict__ acc, const float* __restrict__ x, const uint16_t* __restrict__ xb,
                            int nslots, long long slot_stride, const float* __restrict__ weight,
                            uint16_t* __restrict__ yb, const Q4Dest dst, long long row0, int rows, int dim,
                            float eps, float offset, float divisor, const __grid_constant__ TpSync sync) {
    __shared__ float red[32];
    const int T = (int)blockDim.x;   // a multiple of 32, at most 1024
    const long long row = blockIdx.x;
    if (threadIdx.x == 0) grid_launch_dependents();   // a decode linear behind this may start fetching weights
    grid_dependency_wait();   // (returns at once unless the launch allowed an early start)
    if (sync.wait_phase >= 0) {
        // tensor parallel: the partial-sum slots are complete once every rank's linear has said so
        if (threadIdx.x == 0) tp_wait_flags(sync);
        __syncthreads();
    }
    if (row >= rows) {
        for (int g = threadIdx.x; g < dim / 16; g += blockDim.x)
            for (int d = 0; d < dst.n; d++) dst.atoms[d][nvfp4_scale_offset(row0 + row, g, dim)] = 0;
        if (sync.signal_phase >= 0) {
            __syncthreads();
            if (threadIdx.x == 0) tp_signal(sync, gridDim.x);
        }
        return;
    }
    const long long base = row * dim;
    float4 v[ITERS];
    float4 part[ITERS];   // sum of the partial-sum slots (sequence-parallel form), added to the row once
    auto sum_slots = [&](int it, const float4& f, bool first) {
        if (first) {
            part[it] = f;
        } else {
            part[it].x += f.x; part[it].y += f.y; part[it].z += f.z; part[it].w += f.w;
        }
    };
    float ss = 0.0f;
    // All loads of the row are issued before anything is stored back: a store to acc between them
    // would order the later loads behind it (same array) and cost one memory round trip per slice.
#pragma unroll
    for (int it = 0; it < ITERS; it++) {
        const int c = (it * T + (int)threadIdx.x) * 4;
        v[it] = c < dim ? __ldcs(reinterpret_cast<const float4*>(acc + base + c)) : make_float4(0.0f, 0.0f, 0.0f, 0.0f);
    }
    if (x) {
        float4 t[ITERS];
#pragma unroll
        for (int it = 0; it < ITERS; it++) {
            const int c = (it * T + (int)threadIdx.x) * 4;
            t[it] = c < dim ? __ldcs(reinterpret_cast<const float4*>(x + base + c)) : make_float4(0.0f, 0.0f, 0.0f, 0.0f);
        }
#pragma unroll
        for (int it = 0; it < ITERS; it++) {
            v[it].x += t[it].x; v[it].y += t[it].y; v[it].z += t[it].z; v[it].w += t[it].w;
        }
    } else if (xb) {
        // slots are fetched four at a time (their loads in flight together) and added in slot order
        for (int s0 = 0; s0 < nslots; s0 += 4) {
            uint2 t[4][ITERS];
#pragma unroll
            for (int j = 0; j < 4; j++)
#pragma unroll
                for (int it = 0; it < ITERS; it++) {
                    const int c = (it * T + (int)threadIdx.x) * 4;
                    t[j][it] = (c < dim && s0 + j < nslots)
                                   ? __ldcs(reinterpret_cast<const uint2*>(xb + (s0 + j) * slot_stride + base + c))
                                   : make_uint2(0u, 0u);
                }
#pragma unroll
            for (int j = 0; j < 4; j++) {
                if (s0 + j >= nslots) break;
#pragma unroll
                for (int it = 0; it < ITERS; it++) {
                    const float4 f = make_float4(__uint_as_float(t[j][it].x << 16), __uint_as_float(t[j][it].x & 0xffff0000u),
                                                 __uint_as_float(t[j][it].y << 16), __uint_as_float(t[j][it].y & 0xffff0000u));
                    if (nslots == 1) {
                        // a single addend goes in as it is; several are summed first
                        v[it].x += f.x; v[it].y += f.y; v[it].z += f.z; v[it].w += f.w;
                    } else {
                        sum_slots(it, f, s0 + j == 0);
                    }
                }
            }
        }
        if (nslots > 1) {
#pragma unroll
            for (int it = 0; it < ITERS; it++) {
                v[it].x += part[it].x; v[it].y += part[it].y; v[it].z += part[it].z; v[it].w += part[it].w;
            }
        }
    }
    if (x || xb) {
#pragma unroll
        for (int it = 0; it < ITERS; it++) {
            const int c = (it * T + (int)threadIdx.x) * 4;
            if (c < dim) __stcs(reinterpret_cast<float4*>(acc + base + c), v[it]);
        }
    }
#pragma unroll
    for (int it = 0; it < ITERS; it++) {
        // the order of the reference's running sum does not survive any parallel reduction; this
        // one matches add_rms_norm_twin's up to the f32 rounding of the partial sums
        ss = fmaf(v[it].x, v[it].x, ss); ss = fmaf(v[it].y, v[it].y, ss);
        ss = fmaf(v[it].z, v[it].z, ss); ss = fmaf(v[it].w, v[it].w, ss);
    }
    ss = warp_sum(ss);
    if (threadIdx.x % VX_WARP == 0) red[threadIdx.x / VX_WARP] = ss;
    __syncthreads();
    // the warps' sums go through the same shuffle tree as in the persistent forms below, so that a
    // row gives the same bits whichever of these kernels takes it
    const float total = warp_sum((int)(threadIdx.x % VX_WARP) < T / VX_WARP ? red[threadIdx.x % VX_WARP] : 0.0f);
    const float inv = 1.0f / sqrtf(total / (float)dim + eps);
    const long long obase = (row0 + row) * dim;
#pragma unroll
    for (int it = 0; it < ITERS; it++) {
        const int c = (it * T + (int)threadIdx.x) * 4;
        const bool in = c < dim;
        float n[4] = {0.0f, 0.0f, 0.0f, 0.0f};
        if (in) {
            const float4 w = *reinterpret_cast<const float4*>(weight + c);
            n[0] = round_bf16(v[it].x * inv * (offset + w.x));
            n[1] = round_bf16(v[it].y * inv * (offset + w.y));
            n[2] = round_bf16(v[it].z * inv * (offset + w.z));
            n[3] = round_bf16(v[it].w * inv * (offset + w.w));
            if (yb)
                *reinterpret_cast<uint2*>(yb + base + c) =
                    make_uint2((__float_as_uint(n[0]) >> 16) | (__float_as_uint(n[1]) & 0xffff0000u),
                               (__float_as_uint(n[2]) >> 16) | (__float_as_uint(n[3]) & 0xffff0000u));
        }
        float amax = fmaxf(fmaxf(fabsf(n[0]), fabsf(n[1])), fmaxf(fabsf(n[2]), fabsf(n[3])));
        amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 1));
        amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 2));
        const uint32_t sb = f32_to_e4m3(__fdiv_rn(__fmul_rn(divisor, amax), 6.0f));
        uint32_t out = 0;
        if (sb != 0) {
            const float ds = e4m3_to_f32(sb);
            const float rc = __frcp_rn(ds);
            float q[4];
#pragma unroll
            for (int i = 0; i < 4; i++) {
                const float a = __fmul_rn(n[i], divisor);
                const float q0 = __fmul_rn(a, rc);
                q[i] = __fmaf_rn(__fmaf_rn(-q0, ds, a), rc, q0);
            }
            out = f32x2_to_e2m1x2(q[0], q[1]) | (f32x2_to_e2m1x2(q[2], q[3]) << 8);
        }
        // two more shuffles gather a lane quad's four code bytes pairs so that one lane stores 8 bytes
        const uint32_t o1 = __shfl_down_sync(0xffffffffu, out, 1);
        const uint32_t o2 = __shfl_down_sync(0xffffffffu, out, 2);
        const uint32_t o3 = __shfl_down_sync(0xffffffffu, out, 3);
        if (in && (threadIdx.x & 3) == 0) {
            const uint2 pk = make_uint2((out & 0xffffu) | (o1 << 16), (o2 & 0xffffu) | (o3 << 16));
            const long long soff = nvfp4_scale_offset(row0 + row, c / 16, dim);
            for (int d = 0; d < dst.n; d++) {
                *reinterpret_cast<uint2*>(dst.codes[d] + (obase + c) / 2) = pk;
                dst.atoms[d][soff] = (uint8_t)sb;
            }
        }
    }
    if (sync.signal_phase >= 0) {
        // this row is in place on every rank: the last block of the grid raises this rank's flag there
        __syncthreads();
        if (threadIdx.x == 0) tp_signal(sync, gridDim.x);
    }
}

// The hot form of the norm above (one bf16 addend or none, one destination, rows of dim / 8 threads
// x two 128-bit slices): persistent blocks walk the rows and request the next row's values before
// they finish the current one, so loads stay in flight across the reduction barrier and the
// stores. Same arithmetic, same bytes written.
template <int MAXT, int MINB>
__global__ void __launch_bounds__(MAXT, MINB)
add_rms_norm_q4_stream_kernel(float* __restrict__ acc, const uint16_t* __restrict__ xb,
                              const float* __restrict__ weight, uint16_t* __restrict__ yb,
                              uint8_t* __restrict__ codes, uint8_t* __restrict__ atoms, int rows, int rows_padded,
                              int dim, float eps, float offset, float divisor) {
    __shared__ float red[2][32];
    const int T = (int)blockDim.x, tid = (int)threadIdx.x;
    const int c0 = tid * 4, c1 = (T + tid) * 4;     // this thread's two slices of every row
    if (tid == 0) grid_launch_dependents();          // a linear behind this may start fetching weights
    grid_dependency_wait();   // launched with early start allowed: everything it reads comes from the kernel ahead
    float4 a0 = make_float4(0.f, 0.f, 0.f, 0.f), a1 = a0;
    uint2 b0 = make_uint2(0u, 0u), b1 = b0;
    auto fetch = [&](long long r) {
        const long long base = r * dim;
        a0 = __ldcs(reinterpret_cast<const float4*>(acc + base + c0));
        a1 = __ldcs(reinterpret_cast<const float4*>(acc + base + c1));
        if (xb) {
            b0 = __ldcs(reinterpret_cast<const uint2*>(xb + base + c0));
            b1 = __ldcs(reinterpret_cast<const uint2*>(xb + base + c1));
        }
    };
    long long row = blockIdx.x;
    if (row < rows) fetch(row);
    int par = 0;
    for (; row < rows_padded; row += gridDim.x, par ^= 1) {
        if (row >= rows) {   // rows that only complete the last 128-row scale tile
            for (int g = tid; g < dim / 16; g += T) atoms[nvfp4_scale_offset(row, g, dim)] = 0;
            continue;
        }
        float4 v[2] = {a0, a1};
        const uint2 t[2] = {b0, b1};
        const long long next = row + gridDim.x;
        if (next < rows) fetch(next);   // in flight while this row is finished
        const long long base = row * dim;
        if (xb) {
#pragma unroll
            for (int it = 0; it < 2; it++) {
                v[it].x += __uint_as_float(t[it].x << 16); v[it].y += __uint_as_float(t[it].x & 0xffff0000u);
                v[it].z += __uint_as_float(t[it].y << 16); v[it].w += __uint_as_float(t[it].y & 0xffff0000u);
            }
            __stcs(reinterpret_cast<float4*>(acc + base + c0), v[0]);
            __stcs(reinterpret_cast<float4*>(acc + base + c1), v[1]);
        }
        float ss = 0.0f;
#pragma unroll
        for (int it = 0; it < 2; it++) {
            ss = fmaf(v[it].x, v[it].x, ss); ss = fmaf(v[it].y, v[it].y, ss);
            ss = fmaf(v[it].z, v[it].z, ss); ss = fmaf(v[it].w, v[it].w, ss);
        }
        ss = warp_sum(ss);
        if (tid % VX_WARP == 0) red[par][tid / VX_WARP] = ss;
        __syncthreads();
        // every warp adds the warps' sums with one shuffle tree (a serial loop over up to 32 shared
        // words is several hundred cycles of dependent latency per row)
        float total = warp_sum((tid % VX_WARP) < T / VX_WARP ? red[par][tid % VX_WARP] : 0.0f);
        const float inv = 1.0f / sqrtf(total / (float)dim + eps);
#pragma unroll
        for (int it = 0; it < 2; it++) {
            const int c = it ? c1 : c0;
            const float4 w = __ldg(reinterpret_cast<const float4*>(weight + c));   // L1-resident after the first row
            float n[4];
            n[0] = round_bf16(v[it].x * inv * (offset + w.x));
            n[1] = round_bf16(v[it].y * inv * (offset + w.y));
            n[2] = round_bf16(v[it].z * inv * (offset + w.z));
            n[3] = round_bf16(v[it].w * inv * (offset + w.w));
            if (yb)
                *reinterpret_cast<uint2*>(yb + base + c) =
                    make_uint2((__float_as_uint(n[0]) >> 16) | (__float_as_uint(n[1]) & 0xffff0000u),
                               (__float_as_uint(n[2]) >> 16) | (__float_as_uint(n[3]) & 0xffff0000u));
            float amax = fmaxf(fmaxf(fabsf(n[0]), fabsf(n[1])), fmaxf(fabsf(n[2]), fabsf(n[3])));
            amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 1));
            amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 2));
            const uint32_t sb = f32_to_e4m3(__fdiv_rn(__fmul_rn(divisor, amax), 6.0f));
            uint32_t out = 0;
            if (sb != 0) {
                const float ds = e4m3_to_f32(sb);
                const float rc = __frcp_rn(ds);
                float q[4];
#pragma unroll
                for (int i = 0; i < 4; i++) {
                    const float a = __fmul_rn(n[i], divisor);
                    const float q0 = __fmul_rn(a, rc);
                    q[i] = __fmaf_rn(__fmaf_rn(-q0, ds, a), rc, q0);
                }
                out = f32x2_to_e2m1x2(q[0], q[1]) | (f32x2_to_e2m1x2(q[2], q[3]) << 8);
            }
            const uint32_t o1 = __shfl_down_sync(0xffffffffu, out, 1);
            const uint32_t o2 = __shfl_down_sync(0xffffffffu, out, 2);
            const uint32_t o3 = __shfl_down_sync(0xffffffffu, out, 3);
            if ((tid & 3) == 0) {
                *reinterpret_cast<uint2*>(codes + (base + c) / 2) =
                    make_uint2((out & 0xffffu) | (o1 << 16), (o2 & 0xffffu) | (o3 << 16));
                atoms[nvfp4_scale_offset(row, c / 16, dim)] = (uint8_t)sb;
            }
        }
    }
}

// The sequence-parallel norm in the same persistent, fetch-ahead form: NS partial-sum slots added in
// slot order, the NVFP4 row written at row0 + row of every destination blob. (One block per SM:
// a rank owns few rows and the slots' values take the registers.)
// QUAD (rows and row0 multiples of 128): a block takes the four rows q, q + 32, q + 64, q + 96 of a
// 128-row tile, whose scale bytes share one 16-byte piece of every scale atom; the pieces are put
// together in shared memory and go to each destination as 16-byte stores instead of sixteen
// single bytes, which is what a link between GPUs wants.
template <int NS, bool QUAD>
__global__ void __launch_bounds__(1024, 1)
sp_norm_q4_stream_kernel(float* __restrict__ acc, const uint16_t* __restrict__ slots, long long slot_stride,
                         const float* __restrict__ weight, const Q4Dest dst, long long row0, int rows, int dim,
                         float eps, float offset, float divisor, const __grid_constant__ TpSync sync) {
    __shared__ float red[2][32];
    __shared__ __align__(16) uint8_t quad_scales[QUAD ? 128 : 1][16];   // [atom along K][4 rows x 4 groups]
    const int T = (int)blockDim.x, tid = (int)threadIdx.x;
    const int c0 = tid * 4, c1 = (T + tid) * 4;
    if (tid == 0) grid_launch_dependents();
    grid_dependency_wait();   // launched with early start allowed: everything it reads comes from the kernel ahead
    if (sync.wait_phase >= 0) {
        // the partial-sum slots are complete once every rank's row-split linear has said so
        if (tid == 0) tp_wait_flags(sync);
        __syncthreads();
    }
    float4 a0 = make_float4(0.f, 0.f, 0.f, 0.f), a1 = a0;
    uint2 b0[NS], b1[NS];
    auto fetch = [&](long long r) {
        const long long base = r * dim;
        a0 = __ldcs(reinterpret_cast<const float4*>(acc + base + c0));
        a1 = __ldcs(reinterpret_cast<const float4*>(acc + base + c1));
#pragma unroll
        for (int sl = 0; sl < NS; sl++) {
            b0[sl] = __ldcs(reinterpret_cast<const uint2*>(slots + sl * slot_stride + base + c0));
            b1[sl] = __ldcs(reinterpret_cast<const uint2*>(slots + sl * slot_stride + base + c1));
        }
    };
    // the i-th row of this block
    const long long quad_first = (long long)(blockIdx.x / 32) * 128 + blockIdx.x % 32;
    auto row_at = [&](int i) { return QUAD ? quad_first + 32LL * i : (long long)blockIdx.x + (long long)i * gridDim.x; };
    if (row_at(0) < rows) fetch(row_at(0));
    int par = 0;
    for (int ri = 0; (!QUAD || ri < 4) && row_at(ri) < rows; ri++, par ^= 1) {
        const long long row = row_at(ri);
        float4 v[2] = {a0, a1};
        float4 part[2];
#pragma unroll
        for (int it = 0; it < 2; it++) {
#pragma unroll
            for (int sl = 0; sl < NS; sl++) {
                const uint2 t = it ? b1[sl] : b0[sl];
                const float4 f = make_float4(__uint_as_float(t.x << 16), __uint_as_float(t.x & 0xffff0000u),
                                             __uint_as_float(t.y << 16), __uint_as_float(t.y & 0xffff0000u));
                if (sl == 0) {
                    part[it] = f;
                } else {
                    part[it].x += f.x; part[it].y += f.y; part[it].z += f.z; part[it].w += f.w;
                }
            }
        }
        const long long next = row_at(ri + 1);
        if ((!QUAD || ri < 3) && next < rows) fetch(next);   // in flight while this row is finished
        const long long base = row * dim, obase = (row0 + row) * dim;
#pragma unroll
        for (int it = 0; it < 2; it++) {
            v[it].x += part[it].x; v[it].y += part[it].y; v[it].z += part[it].z; v[it].w += part[it].w;
        }
        __stcs(reinterpret_cast<float4*>(acc + base + c0), v[0]);
        __stcs(reinterpret_cast<float4*>(acc + base + c1), v[1]);
        float ss = 0.0f;
#pragma unroll
        for (int it = 0; it < 2; it++) {
            ss = fmaf(v[it].x, v[it].x, ss); ss = fmaf(v[it].y, v[it].y, ss);
            ss = fmaf(v[it].z, v[it].z, ss); ss = fmaf(v[it].w, v[it].w, ss);
        }
        ss = warp_sum(ss);
        if (tid % VX_WARP == 0) red[par][tid / VX_WARP] = ss;
        __syncthreads();
        const float total = warp_sum((tid % VX_WARP) < T / VX_WARP ? red[par][tid % VX_WARP] : 0.0f);
        const float inv = 1.0f / sqrtf(total / (float)dim + eps);
#pragma unroll
        for (int it = 0; it < 2; it++) {
            const int c = it ? c1 : c0;
            const float4 w = __ldg(reinterpret_cast<const float4*>(weight + c));
            float n[4];
            n[0] = round_bf16(v[it].x * inv * (offset + w.x));
            n[1] = round_bf16(v[it].y * inv * (offset + w.y));
            n[2] = round_bf16(v[it].z * inv * (offset + w.z));
            n[3] = round_bf16(v[it].w * inv * (offset + w.w));
            float amax = fmaxf(fmaxf(fabsf(n[0]), fabsf(n[1])), fmaxf(fabsf(n[2]), fabsf(n[3])));
            amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 1));
            amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 2));
            const uint32_t sb = f32_to_e4m3(__fdiv_rn(__fmul_rn(divisor, amax), 6.0f));
            uint32_t out = 0;
            if (sb != 0) {
                const float ds = e4m3_to_f32(sb);
                const float rc = __frcp_rn(ds);
                float q[4];
#pragma unroll
                for (int i = 0; i < 4; i++) {
                    const float a = __fmul_rn(n[i], divisor);
                    const float q0 = __fmul_rn(a, rc);
                    q[i] = __fmaf_rn(__fmaf_rn(-q0, ds, a), rc, q0);
                }
                out = f32x2_to_e2m1x2(q[0], q[1]) | (f32x2_to_e2m1x2(q[2], q[3]) << 8);
            }
            const uint32_t o1 = __shfl_down_sync(0xffffffffu, out, 1);
            const uint32_t o2 = __shfl_down_sync(0xffffffffu, out, 2);
            const uint32_t o3 = __shfl_down_sync(0xffffffffu, out, 3);
            if ((tid & 3) == 0) {
                const uint2 pk = make_uint2((out & 0xffffu) | (o1 << 16), (o2 & 0xffffu) | (o3 << 16));
                const long long soff = nvfp4_scale_offset(row0 + row, c / 16, dim);
                for (int d = 0; d < dst.n; d++) {
                    *reinterpret_cast<uint2*>(dst.codes[d] + (obase + c) / 2) = pk;
                    if (!QUAD) dst.atoms[d][soff] = (uint8_t)sb;
                }
                if (QUAD) quad_scales[c / 64][ri * 4 + (c / 16) % 4] = (uint8_t)sb;
            }
        }
    }
    if (QUAD) {
        __syncthreads();
        if (tid < dim / 64) {
            const uint4 piece = *reinterpret_cast<const uint4*>(quad_scales[tid]);
            const long long off = (((row0 + quad_first) / 128) * (dim / 64) + tid) * 512 + (quad_first % 32) * 16;
            for (int d = 0; d < dst.n; d++) *reinterpret_cast<uint4*>(dst.atoms[d] + off) = piece;
        }
    }
    if (sync.signal_phase >= 0) {
        // this block's rows are in place on every rank: the last block of the grid raises the flag
        __syncthreads();
        if (tid == 0) tp_signal(sync, gridDim.x);
    }
}

// x_own += sum of the slots, then the rows as bf16 to every destination (the last step of a
// sequence-parallel stack: residual add and all-gather of the result in one pass).
__global__ void __launch_bounds__(256)
sp_finish_kernel(float* __restrict__ acc, const uint16_t* __restrict__ slots, int nslots, long long slot_stride,
                 const Q4Dest dst, long long row0, long long len, int dim, const __grid_constant__ TpSync sync) {
    if (threadIdx.x == 0) grid_launch_dependents();
    grid_dependency_wait();
    if (sync.wait_phase >= 0) {
        if (threadIdx.x == 0) tp_wait_flags(sync);
        __syncthreads();
    }
    for (long long i = (blockIdx.x * (long long)blockDim.x + threadIdx.x) * 4; i < len;
         i += (long long)gridDim.x * blockDim.x * 4) {
        float4 a = *reinterpret_cast<const float4*>(acc + i);
        float4 t = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
        for (int sl = 0; sl < nslots; sl++) {
            const uint2 b = *reinterpret_cast<const uint2*>(slots + sl * slot_stride + i);
            t.x += __uint_as_float(b.x << 16); t.y += __uint_as_float(b.x & 0xffff0000u);
            t.z += __uint_as_float(b.y << 16); t.w += __uint_as_float(b.y & 0xffff0000u);
        }
        a.x += t.x; a.y += t.y; a.z += t.z; a.w += t.w;
        *reinterpret_cast<float4*>(acc + i) = a;
        const uint2 pk = make_uint2((uint32_t)bf16_bits(a.x) | ((uint32_t)bf16_bits(a.y) << 16),
                                    (uint32_t)bf16_bits(a.z) | ((uint32_t)bf16_bits(a.w) << 16));
        for (int d = 0; d < dst.n; d++)
            *reinterpret_cast<uint2*>(reinterpret_cast<uint16_t*>(dst.codes[d]) + row0 * dim + i) = pk;
    }
    if (sync.signal_phase >= 0) {
        __syncthreads();
        if (threadIdx.x == 0) tp_signal(sync, gridDim.x);
    }
}


static int launch_norm_q4(float* acc, const float* x, const uint16_t* xb, int nslots, long long slot_stride,
                          const float* weight, uint16_t* yb, const Q4Dest& dst, long long row0, int rows,
                          int rows_padded, int dim, float eps, int offset, float divisor, const TpSync& sync) {
    const float off = offset ? 1.0f : 0.0f;
    TimedRegion timed(TIMED_NORM);
    cudaError_t e;
    if (dim % 256 == 0) {
        // one block per row with dim / 8 threads: two 128-bit slices per thread, many warps in flight
        EarlyLaunch l((unsigned)rows_padded, (unsigned)(dim / 8));
        e = cudaLaunchKernelEx(&l.cfg, add_rms_norm_q4_rows_kernel<2, 1024>, acc, x, xb, nslots, slot_stride, weight, yb,
                               dst, row0, rows, dim, eps, off, divisor, sync);
    } else if (dim <= 2048) {
        EarlyLaunch l((unsigned)rows_padded, 256u);
        e = cudaLaunchKernelEx(&l.cfg, add_rms_norm_q4_rows_kernel<2, 256>, acc, x, xb, nslots, slot_stride, weight, yb,
                               dst, row0, rows, dim, eps, off, divisor, sync);
    } else {
        EarlyLaunch l((unsigned)rows_padded, 256u);
        e = cudaLaunchKernelEx(&l.cfg, add_rms_norm_q4_rows_kernel<8, 256>, acc, x, xb, nslots, slot_stride, weight, yb,
                               dst, row0, rows, dim, eps, off, divisor, sync);
    }
    if (e != cudaSuccess) return (int)e;
    return launch_status();
}

int add_rms_norm_q4(float* acc, const float* x, const uint16_t* xb, const float* weight, uint16_t* yb,
                    uint8_t* codes, uint8_t* atoms, int rows, int dim, float eps, int offset, float divisor) {
    if (rows < 1 || dim < 64 || dim % 64 != 0 || !(divisor > 0.0f)) return VELOX_ERR_SHAPE;
    const int rows_padded = (rows + 127) / 128 * 128;
    const bool aligned = ((reinterpret_cast<uintptr_t>(acc) | reinterpret_cast<uintptr_t>(x) |
                           reinterpret_cast<uintptr_t>(weight)) & 15) == 0 &&
                         ((reinterpret_cast<uintptr_t>(xb) | reinterpret_cast<uintptr_t>(yb) |
                           reinterpret_cast<uintptr_t>(codes)) & 7) == 0;
    if (aligned && !x && dim % 256 == 0 && dim <= 8192) {
        static int sms = 0;
        if (sms == 0) {
            int dev = 0;
            cudaGetDevice(&dev);
            cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
            if (sms <= 0) sms = 148;
        }
        // register budgets chosen so that about 1300-1500 threads are resident per SM: the loads of
        // the next rows in flight are what hides the row-wide reduction barrier
        const int threads = dim / 8;
        const float off = offset ? 1.0f : 0.0f;
        // early start allowed: the launch overlaps the tail of the kernel ahead (the kernel waits
        // for it before its first load)
        cudaLaunchConfig_t cfg{};
        cfg.blockDim = dim3(threads);
        cfg.stream = stream();
        cudaLaunchAttribute attr[1];
        attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[0].val.programmaticStreamSerializationAllowed = 1;
        static const bool early = getenv("VELOX_SM100_NO_EARLY_START") == nullptr;
        cfg.attrs = attr;
        cfg.numAttrs = early ? 1 : 0;
        auto go = [&](auto kern, int per_sm) {
            int blocks = sms * per_sm;
            if (blocks > rows_padded) blocks = rows_padded;
            cfg.gridDim = dim3(blocks);
            return cudaLaunchKernelEx(&cfg, kern, acc, xb, weight, yb, codes, atoms, rows, rows_padded, dim, eps, off,
                                      divisor);
        };
        cudaError_t e;
        TimedRegion timed(TIMED_NORM);
        if (threads <= 256)
            e = go(add_rms_norm_q4_stream_kernel<256, 6>, 6);
        else if (threads <= 512)
            e = go(add_rms_norm_q4_stream_kernel<512, 3>, 3);
        else if (threads <= 768)
            e = go(add_rms_norm_q4_stream_kernel<768, 2>, 2);
        else
            e = go(add_rms_norm_q4_stream_kernel<1024, 1>, 1);
        if (e != cudaSuccess) return (int)e;
        return launch_status();
    }
    if (aligned && dim <= 8192) {
        Q4Dest dst{};
        dst.codes[0] = codes;
        dst.atoms[0] = atoms;
        dst.n = 1;
        TpSync none{};
        none.wait_phase = none.signal_phase = -1;
        return launch_norm_q4(acc, x, xb, 1, 0, weight, yb, dst, 0, rows, rows_padded, dim, eps, offset, divisor, none);
    }
    add_rms_norm_q4_kernel<<<(unsigned)rows_padded, 256, 0, stream()>>>(acc, x, xb, weight, yb, codes, atoms, rows,
                                                                         dim, eps, offset ? 1.0f : 0.0f, divisor);
    return launch_status();
}

int sp_norm_q4(float* acc, const uint16_t* slots, int nslots, long long slot_stride, const float* weight,
               uint8_t* const* codes, uint8_t* const* atoms, int ndst, long long row0, int rows, int dim, float eps,
               int offset, float divisor, const velox_sm100_tp_sync* sync) {
    if (rows < 1 || rows % 128 != 0 || row0 % 128 != 0 || dim < 64 || dim % 64 != 0 || dim > 8192 ||
        !(divisor > 0.0f) || ndst < 1 || ndst > VX_MAX_PEERS || nslots < 0 || (nslots > 0 && !slots))
        return VELOX_ERR_SHAPE;
    Q4Dest dst{};
    for (int d = 0; d < ndst; d++) {
        dst.codes[d] = codes[d];
        dst.atoms[d] = atoms[d];
    }
    dst.n = ndst;
    TpSync ts;
    const int src = tp_sync_fill_elementwise(&ts, sync);
    if (src != 0) return src;
    const bool aligned = ((reinterpret_cast<uintptr_t>(acc) | reinterpret_cast<uintptr_t>(weight)) & 15) == 0 &&
                         (reinterpret_cast<uintptr_t>(slots) & 7) == 0 && slot_stride % 4 == 0;
    if (aligned && dim % 256 == 0 && (nslots == 2 || nslots == 4 || nslots == 8)) {
        static int sms = 0;
        if (sms == 0) {
            int dev = 0;
            cudaGetDevice(&dev);
            cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
            if (sms <= 0) sms = 148;
        }
        const int blocks = rows < sms ? rows : sms;
        const float off = offset ? 1.0f : 0.0f;
        TimedRegion timed(TIMED_NORM);
        EarlyLaunch l((unsigned)blocks, (unsigned)(dim / 8));
        cudaError_t e;
        // whole 128-row scale tiles (what a rank of a tensor-parallel group owns): four rows per block
        const bool quad = rows % 128 == 0 && row0 % 128 == 0 && dim <= 8192;
        if (quad) l.cfg.gridDim = dim3((unsigned)(rows / 4));
        if (quad && nslots == 2)
            e = cudaLaunchKernelEx(&l.cfg, sp_norm_q4_stream_kernel<2, true>, acc, slots, slot_stride, weight, dst, row0, rows,
                                   dim, eps, off, divisor, ts);
        else if (quad && nslots == 4)
            e = cudaLaunchKernelEx(&l.cfg, sp_norm_q4_stream_kernel<4, true>, acc, slots, slot_stride, weight, dst, row0, rows,
                                   dim, eps, off, divisor, ts);
        else if (quad)
            e = cudaLaunchKernelEx(&l.cfg, sp_norm_q4_stream_kernel<8, true>, acc, slots, slot_stride, weight, dst, row0, rows,
                                   dim, eps, off, divisor, ts);
        else if (nslots == 2)
            e = cudaLaunchKernelEx(&l.cfg, sp_norm_q4_stream_kernel<2, false>, acc, slots, slot_stride, weight, dst, row0, rows,
                                   dim, eps, off, divisor, ts);
        else if (nslots == 4)
            e = cudaLaunchKernelEx(&l.cfg, sp_norm_q4_stream_kernel<4, false>, acc, slots, slot_stride, weight, dst, row0, rows,
                                   dim, eps, off, divisor, ts);
        else
            e = cudaLaunchKernelEx(&l.cfg, sp_norm_q4_stream_kernel<8, false>, acc, slots, slot_stride, weight, dst, row0, rows,
                                   dim, eps, off, divisor, ts);
        if (e != cudaSuccess) return (int)e;
        return launch_status();
    }
    return launch_norm_q4(acc, nullptr, nslots > 0 ? slots : nullptr, nslots, slot_stride, weight, nullptr, dst, row0,
                          rows, rows, dim, eps, offset, divisor, ts);
}

int sp_finish(float* acc, const uint16_t* slots, int nslots, long long slot_stride, uint16_t* const* out, int ndst,
              long long row0, int rows, int dim, const velox_sm100_tp_sync* sync) {
    if (rows < 1 || dim % 4 != 0 || ndst < 1 || ndst > VX_MAX_PEERS || nslots < 1 || !slots) return VELOX_ERR_SHAPE;
    Q4Dest dst{};
    for (int d = 0; d < ndst; d++) dst.codes[d] = reinterpret_cast<uint8_t*>(out[d]);
    dst.n = ndst;
    const long long len = (long long)rows * dim;
    TpSync ts;
    const int src = tp_sync_fill_elementwise(&ts, sync);
    if (src != 0) return src;
    TimedRegion timed(TIMED_NORM);
    EarlyLaunch l(grid_1d(len / 4, 256), 256u);
    const cudaError_t e = cudaLaunchKernelEx(&l.cfg, sp_finish_kernel, acc, slots, nslots, slot_stride, dst, row0, len, dim, ts);
    if (e != cudaSuccess) return (int)e;
    return launch_status();
}

// y[m, n] = x[m, k] . w[n, k]^T in f32 (Backend::matmul, crates/velox-core/src/backend.rs:1550-1564;
// reference kernel: one warp per output, crates/velox-cuda/kernels/portable.cu:13-28). A 64 x 64
// output tile per block of 256 threads, 16-wide k slices staged in shared memory (k-major, so a
// thread's four rows / four columns are one 16-byte load), a 4 x 4 register block per thread and
// f32 fused multiply-adds in ascending k: each output is one f32 running sum.
__global__ void __launch_bounds__(256)
matmul_f32_kernel(const float* __restrict__ x, const float* __restrict__ w, float* __restrict__ y, int m, int n, int k) {
    __shared__ __align__(16) float xs[16][64 + 4];
    __shared__ __align__(16) float ws[16][64 + 4];
    const int tx = threadIdx.x % 16, ty = threadIdx.x / 16;
    const long long row0 = (long long)blockIdx.y * 64, col0 = (long long)blockIdx.x * 64;
    float acc[4][4] = {};
    for (int k0 = 0; k0 < k; k0 += 16) {
        for (int i = threadIdx.x; i < 64 * 16; i += 256) {
            const int r = i / 16, c = i % 16;
            xs[c][r] = (row0 + r < m && k0 + c < k) ? x[(row0 + r) * k + k0 + c] : 0.0f;
            ws[c][r] = (col0 + r < n && k0 + c < k) ? w[(col0 + r) * k + k0 + c] : 0.0f;
        }
        __syncthreads();
#pragma unroll
        for (int c = 0; c < 16; c++) {
            const float4 a = *reinterpret_cast<const float4*>(&xs[c][ty * 4]);
            const float4 b = *reinterpret_cast<const float4*>(&ws[c][tx * 4]);
            const float av[4] = {a.x, a.y, a.z, a.w}, bv[4] = {b.x, b.y, b.z, b.w};
#pragma unroll
            for (int i = 0; i < 4; i++)
#pragma unroll
                for (int j = 0; j < 4; j++) acc[i][j] = fmaf(av[i], bv[j], acc[i][j]);
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < 4; i++)
#pragma unroll
        for (int j = 0; j < 4; j++) {
            const long long r = row0 + ty * 4 + i, c = col0 + tx * 4 + j;
            if (r < m && c < n) y[r * n + c] = acc[i][j];
        }
}

int matmul_f32(const float* x, const float* w, float* y, int m, int n, int k) {
    if (m < 1 || n < 1 || k < 1) return VELOX_ERR_SHAPE;
    const dim3 grid((unsigned)((n + 63) / 64), (unsigned)((m + 63) / 64));
    if (grid.y > 65535) return VELOX_ERR_UNSUPPORTED;
    matmul_f32_kernel<<<grid, 256, 0, stream()>>>(x, w, y, m, n, k);
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
