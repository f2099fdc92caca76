// C ABI of the sm_100a quantized-linear kernel set (declared in include/velox_sm100.h): argument
// checks as the reference's check::linear (crates/velox-core/src/check.rs:100-131), kernel
// selection by (format, policy, m, k), and the launch-stream / scratch state the launchers share.
#include <atomic>
#include <cstdlib>
#include <cstring>
#include <mutex>
#include <vector>

#include "common.cuh"
#include "gemm.cuh"
#include "kernels.cuh"

namespace vx {

static thread_local cudaStream_t g_stream = cudaStreamPerThread;
cudaStream_t stream() { return g_stream; }
void set_stream(cudaStream_t s) { g_stream = s ? s : cudaStreamPerThread; }

struct Pool {
    void* ptr = nullptr;
    size_t cap = 0;
};
static std::mutex g_scratch_mu;
static Pool g_pools[64][SCRATCH_SLOTS];

void* scratch(ScratchSlot slot, size_t bytes) {
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return nullptr;
    std::lock_guard<std::mutex> lock(g_scratch_mu);
    Pool& p = g_pools[dev][slot];
    if (bytes > p.cap) {
        size_t n = p.cap * 2 > bytes ? p.cap * 2 : bytes;
        if (n < (1u << 20)) n = 1u << 20;
        void* q = nullptr;
        if (cudaMalloc(&q, n) != cudaSuccess) {
            cudaGetLastError();
            return nullptr;
        }
        p.ptr = q;  // the old buffer is kept alive: queued work or a captured graph may use it
        p.cap = n;
    }
    return p.ptr;
}

static std::atomic<long long> g_launches{0};
void note_launch() { g_launches.fetch_add(1, std::memory_order_relaxed); }

struct TimedPair {
    cudaEvent_t a, b;
    int cls;
};
static std::mutex g_timing_mu;
static bool g_timing_on = false;
static std::vector<TimedPair> g_timed;

TimedRegion::TimedRegion(int cls) : slot(-1) {
    if (!g_timing_on) return;
    std::lock_guard<std::mutex> lock(g_timing_mu);
    TimedPair t;
    t.cls = cls;
    if (cudaEventCreate(&t.a) != cudaSuccess || cudaEventCreate(&t.b) != cudaSuccess) return;
    cudaEventRecord(t.a, stream());
    g_timed.push_back(t);
    slot = (int)g_timed.size() - 1;
}

TimedRegion::~TimedRegion() {
    if (slot < 0) return;
    std::lock_guard<std::mutex> lock(g_timing_mu);
    cudaEventRecord(g_timed[slot].b, stream());
}

int check_view(const velox_sm100_view* v) {
    if (!v || !v->w) return VELOX_ERR_SHAPE;
    // (the per-tensor divisor and the row scales are read as aligned words by every kernel)
    if (reinterpret_cast<uintptr_t>(v->w) & 3) return VELOX_ERR_UNSUPPORTED;
    if (v->n <= 0 || v->k <= 0) return VELOX_ERR_SHAPE;
    switch (v->format) {
        case VELOX_FMT_NVFP4:
            if (v->n % 128 != 0 || v->k % 64 != 0) return VELOX_ERR_SHAPE;
            break;
        case VELOX_FMT_FP8_ROW_BF16:
            break;
        case VELOX_FMT_GGML_Q4_K:
            if (v->k % 256 != 0) return VELOX_ERR_SHAPE;
            break;
        default:
            return VELOX_ERR_UNSUPPORTED;
    }
    if (v->rows <= 0 || v->row_begin < 0 || v->row_begin + v->rows > v->n) return VELOX_ERR_SHAPE;
    return 0;
}

enum Path { PATH_GEMV, PATH_GEMV_TC, PATH_GEMM_A4, PATH_GEMM_A8, PATH_GEMM_BF16, PATH_GENERIC };

struct Plan {
    Path path;
    int act;
    float divisor;
};

// Kernel and activation rounding for one view at m rows. The rounding never exceeds the view's
// policy (crates/velox-conformance/src/lib.rs:64-74): bf16 is always permitted; FP8 rows need
// AllowA8 or AllowA4; NVFP4 activations need AllowA4 and use its divisor.
static int device_sms() {
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

// 17 <= m <= 64: true where the byte-balanced streaming kernel is expected to beat the GEMM. Both
// models are per-SM rates measured on B200, scaled by the SM count of the device at hand: a CTA of
// the GEMM streams the K of its tile at about 68 GB/s, the streaming kernel moves about 32 GB/s per
// SM with every SM busy, plus 3 us of fixed cost and 0.35 us per token of fix-up and stores.
static bool small_batch_streams(const velox_sm100_view& v, int m) {
    const int sms = device_sms();
    const double row_bytes = v.format == VELOX_FMT_NVFP4 ? 0.5625 * (double)v.k : (double)v.k;
    const long long gemm_tiles = (v.rows + 255) / 256;
    const double gemm_us = (double)((gemm_tiles + sms - 1) / sms) * 256.0 * row_bytes / 68e3;
    const double stream_us = (double)v.rows * row_bytes / (31.8e3 * sms) + 3.0 + 0.35 * m;
    return gemm_us > stream_us;
}

static Plan plan_for(const velox_sm100_view& v, int m) {
    Plan p{PATH_GENERIC, VELOX_ACT_EXACT, 0.0f};
    if (v.k % 64 != 0) return p;
    // Every fast path reads the payload with 16-byte accesses (tensor maps, vector loads). A payload
    // that does not start on such a boundary (cudaMalloc gives 256) is still a legal view: it takes
    // the per-element kernel, and linear_act says so up front.
    if (reinterpret_cast<uintptr_t>(v.w) & 15) return p;
    if (m <= 16) {
        // Decode. Where the view admits NVFP4 activations the stored bytes go to the block-scaled
        // tensor cores as they are; otherwise bf16 activations and the unpacking GEMV.
        if (v.format == VELOX_FMT_NVFP4 && v.policy == VELOX_POLICY_ALLOW_A4 && v.divisor > 0.0f && gemm_available()) {
            p.path = PATH_GEMV_TC;
            p.act = VELOX_ACT_NVFP4;
            p.divisor = v.divisor;
            return p;
        }
        // FP8 rows at decode width keep bf16 activations whatever the policy admits: the warp-MMA
        // kernel that re-labels E4M3 bytes as bf16 ([14336, 4096]: 15 us at 1 to 8 tokens, 19 at 16)
        // beats the FP8 quantiser launch plus the block-scaled tensor-core kernel (21 to 25 us),
        // and rounds less.
        p.path = PATH_GEMV;
        p.act = VELOX_ACT_BF16;
        return p;
    }
    if (!gemm_available()) return p;
    // Small batches (17 to 64 tokens) are still a weight stream. The GEMM gives a 256-row tile to one
    // CTA, which then streams the whole K of those rows by itself: few tiles with a long K leave most
    // of the machine idle. The streaming kernel cuts the same bytes evenly over all SMs but pays per
    // token in its fix-up and stores. Measured models of both (microseconds) pick the kernel; the
    // rounding is the same either way.
    if (m <= 64 && small_batch_streams(v, m)) {
        if (v.format == VELOX_FMT_NVFP4 && v.policy == VELOX_POLICY_ALLOW_A4 && v.divisor > 0.0f) {
            p.path = PATH_GEMV_TC;
            p.act = VELOX_ACT_NVFP4;
            p.divisor = v.divisor;
            return p;
        }
        if (v.format == VELOX_FMT_FP8_ROW_BF16 && v.policy != VELOX_POLICY_A16_ONLY && v.k % 128 == 0) {
            p.path = PATH_GEMV_TC;
            p.act = VELOX_ACT_FP8_ROW;
            return p;
        }
    }
    if (v.format == VELOX_FMT_NVFP4 && v.policy == VELOX_POLICY_ALLOW_A4 && v.divisor > 0.0f) {
        p.path = PATH_GEMM_A4;
        p.act = VELOX_ACT_NVFP4;
        p.divisor = v.divisor;
        return p;
    }
    if (v.format == VELOX_FMT_FP8_ROW_BF16 && v.policy != VELOX_POLICY_A16_ONLY && v.k % 128 == 0) {
        p.path = PATH_GEMM_A8;
        p.act = VELOX_ACT_FP8_ROW;
        return p;
    }
    p.path = PATH_GEMM_BF16;
    p.act = VELOX_ACT_BF16;
    return p;
}

// The fused tensor-core SwiGLU pairs column c of the gate tile with column c of the up tile; with
// NVFP4 scale tiles that needs both views at the same offset inside a 128-row tile. Otherwise the
// pair runs on the bf16 path, which has no such constraint.
static Plan plan_swiglu(const velox_sm100_view& both, const velox_sm100_view& gate,
                        const velox_sm100_view& up, int m) {
    Plan p = plan_for(both, m);
    if (reinterpret_cast<uintptr_t>(up.w) & 15) return Plan{PATH_GENERIC, VELOX_ACT_EXACT, 0.0f};
    if ((p.path == PATH_GEMM_A4 || p.path == PATH_GEMV_TC) && (gate.row_begin - up.row_begin) % 128 != 0) {
        p.path = p.path == PATH_GEMV_TC && m <= 16 ? PATH_GEMV : PATH_GEMM_BF16;
        p.act = VELOX_ACT_BF16;
        p.divisor = 0.0f;
    }
    return p;
}

static int run(const LinearArgs& a, const Plan& p) {
    int rc = VELOX_ERR_UNSUPPORTED;
    switch (p.path) {
        case PATH_GEMV:
            rc = gemv(a);
            break;
        case PATH_GEMV_TC:
            rc = gemv_tc(a, p.act, p.divisor);
            // (a small batch the streaming kernel declines has the same rounding on the GEMM)
            if (rc == VELOX_ERR_UNSUPPORTED && a.m > 16) rc = gemm_linear(a, p.act, p.divisor);
            break;
        case PATH_GEMM_A4:
        case PATH_GEMM_A8:
        case PATH_GEMM_BF16:
            rc = gemm_linear(a, p.act, p.divisor);
            break;
        default:
            break;
    }
    if (rc == VELOX_ERR_UNSUPPORTED) {
        LinearArgs g = a;
        g.round_x = p.act == VELOX_ACT_BF16;
        if (p.act == VELOX_ACT_FP8_ROW || p.act == VELOX_ACT_NVFP4) return VELOX_ERR_UNSUPPORTED;
        rc = linear_generic(g);
    }
    return rc;
}

static int linear_common(const float* x, const uint16_t* xb, const velox_sm100_view* view, int m,
                         float* y, uint16_t* yb, long long ld, long long col,
                         const uint8_t* q_codes = nullptr, const uint8_t* q_atoms = nullptr,
                         uint8_t* qo_codes = nullptr, uint8_t* qo_atoms = nullptr, float qo_divisor = 0.0f,
                         const void* rs_maps = nullptr, int rs_rows = 0, const velox_sm100_tp_sync* sync = nullptr) {
    if (m <= 0 || (!x && !xb && !q_codes) || (!y && !yb && !qo_codes && !rs_maps)) return VELOX_ERR_SHAPE;
    int rc = check_view(view);
    if (rc != 0) return rc;
    LinearArgs a{};
    a.w = *view;
    a.swiglu = 0;
    a.x = x;
    a.xb = xb;
    a.m = m;
    a.y = y;
    a.yb = yb;
    a.ld = ld;
    a.col = col;
    a.q_codes = q_codes;
    a.q_atoms = q_atoms;
    a.qo_codes = qo_codes;
    a.qo_atoms = qo_atoms;
    a.qo_divisor = qo_divisor;
    a.rs_maps = rs_maps;
    a.rs_rows_per_owner = rs_rows;
    a.sync = sync;
    Plan p = plan_for(*view, m);
    // the scattering epilogue is the GEMM's (same rounding as the small-batch streaming kernel)
    if (rs_maps && m > 16 && p.path == PATH_GEMV_TC && p.act == VELOX_ACT_NVFP4) p.path = PATH_GEMM_A4;
    if ((rs_maps || sync) && p.path != PATH_GEMM_A4) return VELOX_ERR_UNSUPPORTED;
    // pre-quantised input: the FP4 tensor-core paths only; and quantised output: the FP4 tensor-core paths only
    if (q_codes && p.path != PATH_GEMM_A4 && p.path != PATH_GEMV_TC) return VELOX_ERR_UNSUPPORTED;
    if (qo_codes && p.path != PATH_GEMM_A4 && p.path != PATH_GEMV_TC) return VELOX_ERR_UNSUPPORTED;
    return run(a, p);
}

static int swiglu_common(const float* x, const uint16_t* xb, const velox_sm100_view* gate,
                         const velox_sm100_view* up, int m, float* out, uint16_t* outb,
                         const uint8_t* q_codes = nullptr, const uint8_t* q_atoms = nullptr,
                         uint8_t* qo_codes = nullptr, uint8_t* qo_atoms = nullptr, float qo_divisor = 0.0f,
                         const velox_sm100_tp_sync* sync = nullptr) {
    if (m <= 0 || (!x && !xb && !q_codes) || (!out && !outb && !qo_codes)) return VELOX_ERR_SHAPE;
    int rc = check_view(gate);
    if (rc != 0) return rc;
    rc = check_view(up);
    if (rc != 0) return rc;
    // backend.rs:2329-2334
    if (up->rows != gate->rows || up->k != gate->k) return VELOX_ERR_SHAPE;
    if (up->format != gate->format) return VELOX_ERR_UNSUPPORTED;
    LinearArgs a{};
    a.w = *gate;
    a.up = *up;
    a.swiglu = 1;
    a.x = x;
    a.xb = xb;
    a.m = m;
    a.y = out;
    a.yb = outb;
    a.ld = gate->rows;
    a.col = 0;
    velox_sm100_view both = *gate;  // the stricter of the two policies (ActPolicy::meet)
    if (up->policy != gate->policy || up->divisor != gate->divisor) {
        both.policy = (gate->policy == VELOX_POLICY_A16_ONLY || up->policy == VELOX_POLICY_A16_ONLY)
                          ? VELOX_POLICY_A16_ONLY
                          : VELOX_POLICY_ALLOW_A8;
    }
    a.w.policy = a.up.policy = both.policy;
    a.q_codes = q_codes;
    a.q_atoms = q_atoms;
    a.qo_codes = qo_codes;
    a.qo_atoms = qo_atoms;
    a.qo_divisor = qo_divisor;
    a.sync = sync;
    Plan p = plan_swiglu(both, *gate, *up, m);
    // (a launch that waits for peers is the GEMM's; same rounding as the small-batch streaming kernel)
    if (sync && m > 16 && p.path == PATH_GEMV_TC && p.act == VELOX_ACT_NVFP4) p.path = PATH_GEMM_A4;
    if (sync && p.path != PATH_GEMM_A4) return VELOX_ERR_UNSUPPORTED;
    if (q_codes && p.path != PATH_GEMM_A4 && p.path != PATH_GEMV_TC) return VELOX_ERR_UNSUPPORTED;
    if (qo_codes && p.path != PATH_GEMM_A4 && p.path != PATH_GEMV_TC) return VELOX_ERR_UNSUPPORTED;
    return run(a, p);
}

}  // namespace vx

using namespace vx;

extern "C" {

int velox_sm100_abi_version(void) { return 1; }

int velox_sm100_set_stream(void* s) {
    set_stream(reinterpret_cast<cudaStream_t>(s));
    return 0;
}

int velox_sm100_linear_act(const velox_sm100_view* view, int m, float* divisor_out) {
    if (m <= 0) return VELOX_ERR_SHAPE;
    int rc = check_view(view);
    if (rc != 0) return rc;
    const Plan p = plan_for(*view, m);
    if (divisor_out) *divisor_out = p.divisor;
    return p.act;
}

int velox_sm100_linear_swiglu_act(const velox_sm100_view* gate, const velox_sm100_view* up, int m,
                                  float* divisor_out) {
    if (m <= 0) return VELOX_ERR_SHAPE;
    int rc = check_view(gate);
    if (rc != 0) return rc;
    rc = check_view(up);
    if (rc != 0) return rc;
    velox_sm100_view both = *gate;
    if (up->policy != gate->policy || up->divisor != gate->divisor) {
        both.policy = (gate->policy == VELOX_POLICY_A16_ONLY || up->policy == VELOX_POLICY_A16_ONLY)
                          ? VELOX_POLICY_A16_ONLY
                          : VELOX_POLICY_ALLOW_A8;
    }
    const Plan p = plan_swiglu(both, *gate, *up, m);
    if (divisor_out) *divisor_out = p.divisor;
    return p.act;
}

int velox_sm100_debug_status(void) {
    const int a = gemm_status_sync();
    if (a != 0) return a;
    const int b = gemv_status_sync();
    if (b != 0) return b;
    const int c = gemv_tc_status_sync();
    return c != 0 ? c : tp_status_sync();
}

int velox_sm100_debug_status_reset(void) {
    cudaError_t e = cudaDeviceSynchronize();
    if (e != cudaSuccess) return (int)e;
    int rc = gemm_status_reset();
    if (rc == 0) rc = gemv_status_reset();
    if (rc == 0) rc = gemv_tc_status_reset();
    if (rc == 0) rc = tp_status_reset();
    return rc;
}

long long velox_sm100_launch_count(void) { return g_launches.load(std::memory_order_relaxed); }

int velox_sm100_timing_enable(int on) {
    std::lock_guard<std::mutex> lock(g_timing_mu);
    g_timing_on = on != 0;
    return 0;
}

int velox_sm100_timing_collect(double* ms_by_class, long long* count_by_class, int classes) {
    if (!ms_by_class || !count_by_class || classes < TIMED_CLASSES) return VELOX_ERR_SHAPE;
    cudaError_t e = cudaDeviceSynchronize();
    if (e != cudaSuccess) return (int)e;
    std::lock_guard<std::mutex> lock(g_timing_mu);
    for (int i = 0; i < classes; i++) {
        ms_by_class[i] = 0.0;
        count_by_class[i] = 0;
    }
    for (TimedPair& t : g_timed) {
        float ms = 0.0f;
        if (cudaEventElapsedTime(&ms, t.a, t.b) == cudaSuccess) {
            ms_by_class[t.cls] += ms;
            count_by_class[t.cls] += 1;
        }
        cudaEventDestroy(t.a);
        cudaEventDestroy(t.b);
    }
    g_timed.clear();
    return 0;
}

int velox_sm100_linear(const float* x, const uint8_t* w, int format, long long n, long long k,
                       long long row_begin, int rows, int m, float* y) {
    velox_sm100_view v{};
    v.w = w;
    v.format = format;
    v.policy = VELOX_POLICY_A16_ONLY;
    v.n = n;
    v.k = k;
    v.row_begin = row_begin;
    v.rows = rows;
    return linear_common(x, nullptr, &v, m, y, nullptr, rows, 0);
}

int velox_sm100_linear_view(const float* x, const velox_sm100_view* view, int m, float* y,
                            uint16_t* yb) {
    if (!view) return VELOX_ERR_SHAPE;
    return linear_common(x, nullptr, view, m, y, yb, view->rows, 0);
}

int velox_sm100_linear_bf16(const uint16_t* xb, const velox_sm100_view* view, int m, float* y,
                            uint16_t* yb) {
    if (!view) return VELOX_ERR_SHAPE;
    return linear_common(nullptr, xb, view, m, y, yb, view->rows, 0);
}

int velox_sm100_linear_swiglu(const float* x, const velox_sm100_view* gate,
                              const velox_sm100_view* up, int m, float* out, uint16_t* outb) {
    return swiglu_common(x, nullptr, gate, up, m, out, outb);
}

int velox_sm100_linear_swiglu_bf16(const uint16_t* xb, const velox_sm100_view* gate,
                                   const velox_sm100_view* up, int m, float* out, uint16_t* outb) {
    return swiglu_common(nullptr, xb, gate, up, m, out, outb);
}

int velox_sm100_linears(const float* x, const uint16_t* xb, const velox_sm100_part* parts,
                        int nparts, int m) {
    if (!parts || nparts <= 0) return VELOX_ERR_SHAPE;
    for (int i = 0; i < nparts; i++) {
        const velox_sm100_part& p = parts[i];
        // backend.rs:2286-2294: the column range must fit the destination's row stride
        if (p.col < 0 || p.col + p.view.rows > p.ld || !p.y) return VELOX_ERR_SHAPE;
        int rc = check_view(&p.view);
        if (rc != 0) return rc;
    }
    for (int i = 0; i < nparts; i++) {
        const velox_sm100_part& p = parts[i];
        // A part that rounds to bf16 reads the twin when the caller has one.
        const Plan pl = plan_for(p.view, m);
        const bool twin = xb && (pl.act == VELOX_ACT_BF16 || !x);
        int rc = linear_common(twin ? nullptr : x, twin ? xb : nullptr, &p.view, m, p.y, nullptr,
                               p.ld, p.col);
        if (rc != 0) return rc;
    }
    return 0;
}

int velox_sm100_dequant_rows(const velox_sm100_view* view, float* out) {
    int rc = check_view(view);
    if (rc != 0) return rc;
    if (!out) return VELOX_ERR_SHAPE;
    return dequant_rows_f32(view, out);
}

int velox_sm100_embed(const uint32_t* ids, int count, const uint8_t* w, int format, long long n, long long k,
                      long long row_begin, float* out) {
    if (!ids || !out || count < 0) return VELOX_ERR_SHAPE;
    if (count == 0) return 0;
    velox_sm100_view v{};
    v.w = w;
    v.format = format;
    v.policy = VELOX_POLICY_A16_ONLY;
    v.n = n;
    v.k = k;
    v.row_begin = row_begin;
    v.rows = 1;     // (check::embed: the table is rows [row_begin, n) of the parent; ids index into it)
    if (row_begin < 0 || row_begin >= n) return VELOX_ERR_SHAPE;
    int rc = check_view(&v);
    if (rc != 0) return rc;
    return embed_rows_f32(&v, ids, count, out);
}

int velox_sm100_matmul(const float* x, const float* w, float* y, int m, int n, int k) {
    if (!x || !w || !y) return VELOX_ERR_SHAPE;
    return matmul_f32(x, w, y, m, n, k);
}

int velox_sm100_quantize_act_fp8row(const float* x, int m, long long k, uint8_t* codes,
                                    float* scales) {
    if (!x || !codes || !scales) return VELOX_ERR_SHAPE;
    return quantize_act_fp8row(x, nullptr, m, k, codes, scales);
}

int velox_sm100_quantize_act_nvfp4(const float* x, int m, long long k, float divisor,
                                   uint8_t* codes, uint8_t* scale_atoms) {
    if (!x || !codes || !scale_atoms || !(divisor > 0.0f)) return VELOX_ERR_SHAPE;
    return quantize_act_nvfp4(x, nullptr, m, k, divisor, codes, scale_atoms);
}

int velox_sm100_encode_nvfp4(const float* w, long long n, long long k, float amax,
                             uint8_t* payload) {
    if (!w || !payload) return VELOX_ERR_SHAPE;
    return encode_nvfp4(w, n, k, amax, payload);
}

int velox_sm100_swiglu(const float* src, long long rows, int src_cols, int gate, int up, int width,
                       float* out) {
    return swiglu(src, rows, src_cols, gate, up, width, out);
}

int velox_sm100_silu_mul(float* gate, const float* up, long long len) { return silu_mul(gate, up, len); }

int velox_sm100_add(float* acc, const float* x, long long len) { return add(acc, x, len); }

int velox_sm100_add_rms_norm_twin(float* acc, const float* x, const float* weight, float* y,
                                  uint16_t* yb, int rows, int dim, float eps, int offset) {
    if (!acc || !weight || (!y && !yb)) return VELOX_ERR_SHAPE;
    return add_rms_norm_twin(acc, x, nullptr, weight, y, yb, rows, dim, eps, offset);
}

int velox_sm100_add_bf16_rms_norm_twin(float* acc, const uint16_t* xb, const float* weight, float* y,
                                       uint16_t* yb, int rows, int dim, float eps, int offset) {
    if (!acc || !xb || !weight || (!y && !yb)) return VELOX_ERR_SHAPE;
    return add_rms_norm_twin(acc, nullptr, xb, weight, y, yb, rows, dim, eps, offset);
}

int velox_sm100_add_rms_norm_q4(float* acc, const float* x, const uint16_t* xb, const float* weight,
                                uint16_t* yb, uint8_t* codes, uint8_t* atoms, int rows, int dim, float eps,
                                int offset, float divisor) {
    if (!acc || !weight || !codes || !atoms) return VELOX_ERR_SHAPE;
    return add_rms_norm_q4(acc, x, xb, weight, yb, codes, atoms, rows, dim, eps, offset, divisor);
}

int velox_sm100_linear_q4(const uint8_t* codes, const uint8_t* atoms, float divisor,
                          const velox_sm100_view* view, int m, float* y, uint16_t* yb) {
    if (!view || !codes || !atoms) return VELOX_ERR_SHAPE;
    if (view->policy != VELOX_POLICY_ALLOW_A4 || view->divisor != divisor) return VELOX_ERR_UNSUPPORTED;
    return linear_common(nullptr, nullptr, view, m, y, yb, view->rows, 0, codes, atoms);
}

int velox_sm100_linear_swiglu_q4(const uint8_t* codes, const uint8_t* atoms, float divisor,
                                 const velox_sm100_view* gate, const velox_sm100_view* up, int m, float* out,
                                 uint16_t* outb) {
    if (!gate || !up || !codes || !atoms) return VELOX_ERR_SHAPE;
    if (gate->policy != VELOX_POLICY_ALLOW_A4 || gate->divisor != divisor || up->policy != VELOX_POLICY_ALLOW_A4 ||
        up->divisor != divisor)
        return VELOX_ERR_UNSUPPORTED;
    return swiglu_common(nullptr, nullptr, gate, up, m, out, outb, codes, atoms);
}

int velox_sm100_linear_q4_to_q4(const uint8_t* codes, const uint8_t* atoms, float divisor,
                                const velox_sm100_view* view, int m, uint16_t* yb, uint8_t* out_codes,
                                uint8_t* out_atoms, float out_divisor) {
    if (!view || !codes || !atoms || !out_codes || !out_atoms) return VELOX_ERR_SHAPE;
    if (view->policy != VELOX_POLICY_ALLOW_A4 || view->divisor != divisor) return VELOX_ERR_UNSUPPORTED;
    return linear_common(nullptr, nullptr, view, m, nullptr, yb, view->rows, 0, codes, atoms, out_codes, out_atoms,
                         out_divisor);
}

int velox_sm100_linear_swiglu_q4_to_q4(const uint8_t* codes, const uint8_t* atoms, float divisor,
                                       const velox_sm100_view* gate, const velox_sm100_view* up, int m,
                                       uint16_t* outb, uint8_t* out_codes, uint8_t* out_atoms,
                                       float out_divisor) {
    if (!gate || !up || !codes || !atoms || !out_codes || !out_atoms) return VELOX_ERR_SHAPE;
    if (gate->policy != VELOX_POLICY_ALLOW_A4 || gate->divisor != divisor || up->policy != VELOX_POLICY_ALLOW_A4 ||
        up->divisor != divisor)
        return VELOX_ERR_UNSUPPORTED;
    return swiglu_common(nullptr, nullptr, gate, up, m, nullptr, outb, codes, atoms, out_codes, out_atoms,
                         out_divisor);
}

static int linears_q4_common(const uint8_t* codes, const uint8_t* atoms, float divisor,
                             const velox_sm100_part_q4* parts, int nparts, int m, const velox_sm100_tp_sync* sync) {
    if (!codes || !atoms || !parts || nparts < 1 || m <= 0) return VELOX_ERR_SHAPE;
    for (int i = 0; i < nparts; i++) {
        const velox_sm100_part_q4& q = parts[i];
        int rc = check_view(&q.view);
        if (rc != 0) return rc;
        if (!q.yb && !q.out_codes) return VELOX_ERR_SHAPE;
        if (q.view.policy != VELOX_POLICY_ALLOW_A4 || q.view.divisor != divisor || q.view.k != parts[0].view.k)
            return VELOX_ERR_UNSUPPORTED;
    }
    auto args_of = [&](const velox_sm100_part_q4& q) {
        LinearArgs l{};
        l.w = q.view;
        l.m = m;
        l.yb = q.yb;
        l.ld = q.view.rows;
        l.col = 0;
        l.q_codes = codes;
        l.q_atoms = atoms;
        l.qo_codes = q.out_codes;
        l.qo_atoms = q.out_atoms;
        l.qo_divisor = q.out_divisor;
        l.sync = sync;
        return l;
    };
    // Up to three views as one launch: the streaming kernel where every view would take it (decode,
    // and small batches of views it streams faster), the GEMM where every view would take that.
    if (nparts <= 3) {
        bool all_stream = !sync, all_gemm = m > 16;
        for (int i = 0; i < nparts; i++) {
            const Path path = plan_for(parts[i].view, m).path;
            all_stream = all_stream && path == PATH_GEMV_TC;
            all_gemm = all_gemm && (path == PATH_GEMM_A4 || (sync && path == PATH_GEMV_TC));
        }
        LinearArgs l[3];
        for (int i = 0; i < nparts; i++) l[i] = args_of(parts[i]);
        if (all_stream && m <= 16) {
            const int rc = gemv_nvfp4_tc_parts(l, nparts, divisor);
            if (rc != VELOX_ERR_UNSUPPORTED) return rc;
        } else if (all_gemm) {
            const int rc = gemm_linears_q4(l, nparts, divisor, sync);
            if (rc != VELOX_ERR_UNSUPPORTED) return rc;
        }
    }
    if (sync) return VELOX_ERR_UNSUPPORTED;
    for (int i = 0; i < nparts; i++) {
        const Plan p = plan_for(parts[i].view, m);
        if (p.path != PATH_GEMM_A4 && p.path != PATH_GEMV_TC) return VELOX_ERR_UNSUPPORTED;
        const int rc = run(args_of(parts[i]), p);
        if (rc != 0) return rc;
    }
    return 0;
}

int velox_sm100_linears_q4(const uint8_t* codes, const uint8_t* atoms, float divisor,
                           const velox_sm100_part_q4* parts, int nparts, int m) {
    return linears_q4_common(codes, atoms, divisor, parts, nparts, m, nullptr);
}

int velox_sm100_tp_linears_q4(const uint8_t* codes, const uint8_t* atoms, float divisor,
                              const velox_sm100_part_q4* parts, int nparts, int m, const velox_sm100_tp_sync* sync) {
    return linears_q4_common(codes, atoms, divisor, parts, nparts, m, sync);
}

int velox_sm100_tp_linear_swiglu_q4_to_q4(const uint8_t* codes, const uint8_t* atoms, float divisor,
                                          const velox_sm100_view* gate, const velox_sm100_view* up, int m,
                                          uint16_t* outb, uint8_t* out_codes, uint8_t* out_atoms, float out_divisor,
                                          const velox_sm100_tp_sync* sync) {
    if (!gate || !up || !codes || !atoms || !out_codes || !out_atoms) return VELOX_ERR_SHAPE;
    if (gate->policy != VELOX_POLICY_ALLOW_A4 || gate->divisor != divisor || up->policy != VELOX_POLICY_ALLOW_A4 ||
        up->divisor != divisor)
        return VELOX_ERR_UNSUPPORTED;
    return swiglu_common(nullptr, nullptr, gate, up, m, nullptr, outb, codes, atoms, out_codes, out_atoms,
                         out_divisor, sync);
}

int velox_sm100_tp_make_maps(void* maps_dev, const unsigned long long* slot_ptrs, int n, int rows_per_owner,
                             long long cols) {
    return gemm_make_rs_maps(maps_dev, slot_ptrs, n, rows_per_owner, cols);
}

int velox_sm100_tp_linear_q4_scatter(const uint8_t* codes, const uint8_t* atoms, float divisor,
                                     const velox_sm100_view* view, int m, const void* maps_dev, int rows_per_owner,
                                     const velox_sm100_tp_sync* sync) {
    if (!view || !codes || !atoms || !maps_dev) return VELOX_ERR_SHAPE;
    if (view->policy != VELOX_POLICY_ALLOW_A4 || view->divisor != divisor) return VELOX_ERR_UNSUPPORTED;
    return linear_common(nullptr, nullptr, view, m, nullptr, nullptr, view->rows, 0, codes, atoms, nullptr, nullptr,
                         0.0f, maps_dev, rows_per_owner, sync);
}

int velox_sm100_tp_norm_q4(float* acc, const uint16_t* slots, int nslots, long long slot_stride, const float* weight,
                           const unsigned long long* codes_ptrs, const unsigned long long* atoms_ptrs, int ndst,
                           long long row0, int rows, int dim, float eps, int offset, float divisor,
                           const velox_sm100_tp_sync* sync) {
    if (!acc || !weight || !codes_ptrs || !atoms_ptrs || ndst < 1 || ndst > VX_MAX_PEERS) return VELOX_ERR_SHAPE;
    uint8_t* c[VX_MAX_PEERS];
    uint8_t* s[VX_MAX_PEERS];
    for (int d = 0; d < ndst; d++) {
        c[d] = reinterpret_cast<uint8_t*>(codes_ptrs[d]);
        s[d] = reinterpret_cast<uint8_t*>(atoms_ptrs[d]);
        if (!c[d] || !s[d]) return VELOX_ERR_SHAPE;
    }
    return sp_norm_q4(acc, slots, nslots, slot_stride, weight, c, s, ndst, row0, rows, dim, eps, offset, divisor, sync);
}

int velox_sm100_tp_finish(float* acc, const uint16_t* slots, int nslots, long long slot_stride,
                          const unsigned long long* out_ptrs, int ndst, long long row0, int rows, int dim,
                          const velox_sm100_tp_sync* sync) {
    if (!acc || !slots || !out_ptrs || ndst < 1 || ndst > VX_MAX_PEERS) return VELOX_ERR_SHAPE;
    uint16_t* o[VX_MAX_PEERS];
    for (int d = 0; d < ndst; d++) {
        o[d] = reinterpret_cast<uint16_t*>(out_ptrs[d]);
        if (!o[d]) return VELOX_ERR_SHAPE;
    }
    return sp_finish(acc, slots, nslots, slot_stride, o, ndst, row0, rows, dim, sync);
}

int velox_sm100_add_bf16(float* acc, const uint16_t* xb, long long len) {
    if (!acc || !xb) return VELOX_ERR_SHAPE;
    return add_bf16(acc, xb, len);
}

int velox_sm100_bf16_twin(const float* x, uint16_t* xb, long long len) { return bf16_twin(x, xb, len); }

}  // extern "C"
