// Tensor-parallel step control: the step counter, the kernel that only waits for peers' flags, and
// the host half of the flag protocol (see tpsync.cuh). No counterpart in the reference, which runs
// on one device; the status-word convention is that of its launchers
// (crates/velox-cuda/src/lib.rs:85-112).
#include <atomic>
#include <mutex>

#include "common.cuh"
#include "kernels.cuh"
#include "tpsync.cuh"

namespace vx {

static std::atomic<unsigned long long> g_wait_limit_ns{2000000000ull};

unsigned long long tp_wait_limit_ns() { return g_wait_limit_ns.load(std::memory_order_relaxed); }

int tp_sync_fill(TpSync* out, const velox_sm100_tp_sync* sync, unsigned int* ticket, int* status) {
    TpSync s{};
    s.wait_phase = s.signal_phase = -1;
    if (sync) {
        if (sync->n < 1 || sync->n > VX_MAX_PEERS || sync->rank < 0 || sync->rank >= sync->n || !sync->epoch ||
            !ticket || !status)
            return VELOX_ERR_SHAPE;
        for (int i = 0; i < sync->n; i++) {
            if (!sync->flag_tables[i] || (sync->flag_tables[i] & 3)) return VELOX_ERR_SHAPE;
            s.flags[i] = sync->flag_tables[i];
        }
        s.epoch = reinterpret_cast<const unsigned int*>(sync->epoch);
        s.ticket = ticket;
        s.status = status;
        s.limit_ns = tp_wait_limit_ns();
        s.n = sync->n;
        s.rank = sync->rank;
        s.wait_phase = sync->wait_phase;
        s.signal_phase = sync->signal_phase;
    }
    *out = s;
    return 0;
}

__device__ int g_tp_status = 0;
__device__ unsigned int g_tp_ticket = 0;

__global__ void tp_step_begin_kernel(unsigned int* epoch) { *epoch += 1u; }

// One thread: the end-of-step barrier (waits for every rank's "output rows written" flag), and the
// kernel a test uses to see a wait run out.
__global__ void tp_wait_kernel(const TpSync s) {
    tp_wait_flags(s);
}

// One thread: raises this rank's flag on every rank without any data (used by tests).
__global__ void tp_signal_kernel(const TpSync s) {
    tp_signal(s, 1u);
}

// A barrier between two phases of the step as a kernel of its own (one warp): lane r raises this
// rank's flag on rank r with a release store (the writes of the kernels ahead in the stream come
// before it) and then waits, bounded like every wait here, for rank r's flag on this rank. The ranks
// are served side by side, so the barrier costs one round trip over the links, not one per rank.
__global__ void tp_barrier_kernel(const TpSync s) {
    const int r = (int)threadIdx.x;
    // Launched with early start allowed, and lets the launch behind it start early too: the warp is
    // resident while the kernel ahead drains, and the next kernel sets itself up (and requests its
    // weights) while this one waits for the peers. The wait below is what orders the data: it
    // returns once the kernel ahead has completed and its writes, remote ones included, are done.
    if (r == 0) grid_launch_dependents();
    grid_dependency_wait();
    if (r < s.n) {
        const unsigned int want = *reinterpret_cast<const volatile unsigned int*>(s.epoch);
        const long long at = (long long)s.wait_phase * TP_FLAG_STRIDE;
        asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(reinterpret_cast<unsigned int*>(s.flags[r]) + at + s.rank),
                     "r"(want)
                     : "memory");
        const unsigned int* mine = reinterpret_cast<const unsigned int*>(s.flags[s.rank]) + at + r;
        const unsigned long long t0 = tp_timer_ns();
        unsigned int spins = 0, seen;
        for (;;) {
            asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(seen) : "l"(mine) : "memory");
            if ((int)(seen - want) >= 0) break;
            if ((++spins & 63u) == 0 && tp_timer_ns() - t0 > s.limit_ns) {
                atomicExch(s.status, ST_TIMEOUT_PEER);
                break;
            }
        }
    }
    __syncwarp();
}

static std::mutex g_tp_mu;
static int* tp_status_ptr() {
    static int* ptrs[64] = {};
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return nullptr;
    std::lock_guard<std::mutex> lock(g_tp_mu);
    if (!ptrs[dev] && cudaGetSymbolAddress(reinterpret_cast<void**>(&ptrs[dev]), g_tp_status) != cudaSuccess) {
        cudaGetLastError();
        return nullptr;
    }
    return ptrs[dev];
}
static unsigned int* tp_ticket_ptr() {
    static unsigned int* ptrs[64] = {};
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return nullptr;
    std::lock_guard<std::mutex> lock(g_tp_mu);
    if (!ptrs[dev] && cudaGetSymbolAddress(reinterpret_cast<void**>(&ptrs[dev]), g_tp_ticket) != cudaSuccess) {
        cudaGetLastError();
        return nullptr;
    }
    return ptrs[dev];
}

int tp_status_sync() {
    int v = -1;
    if (cudaMemcpyFromSymbol(&v, g_tp_status, sizeof(int)) != cudaSuccess) return -1;
    return v;
}

int tp_status_reset() {
    const int zero = 0;
    const unsigned int uzero = 0;
    cudaError_t e = cudaMemcpyToSymbol(g_tp_status, &zero, sizeof(int));
    if (e == cudaSuccess) e = cudaMemcpyToSymbol(g_tp_ticket, &uzero, sizeof(unsigned int));
    return (int)e;
}

// The elementwise kernels of the step (norm, finish) report through the same words.
int tp_sync_fill_elementwise(TpSync* out, const velox_sm100_tp_sync* sync) {
    return tp_sync_fill(out, sync, sync ? tp_ticket_ptr() : nullptr, sync ? tp_status_ptr() : nullptr);
}

}  // namespace vx

using namespace vx;

extern "C" {

int velox_sm100_tp_set_wait_limit_ms(int ms) {
    if (ms < 1 || ms > 60000) return VELOX_ERR_SHAPE;
    g_wait_limit_ns.store((unsigned long long)ms * 1000000ull, std::memory_order_relaxed);
    return 0;
}

int velox_sm100_tp_step_begin(unsigned int* epoch) {
    if (!epoch || (reinterpret_cast<uintptr_t>(epoch) & 3)) return VELOX_ERR_SHAPE;
    tp_step_begin_kernel<<<1, 1, 0, stream()>>>(epoch);
    return launch_status();
}

int velox_sm100_tp_wait(const velox_sm100_tp_sync* sync) {
    if (!sync || sync->wait_phase < 0) return VELOX_ERR_SHAPE;
    TpSync s;
    int rc = tp_sync_fill_elementwise(&s, sync);
    if (rc != 0) return rc;
    s.signal_phase = -1;
    tp_wait_kernel<<<1, 1, 0, stream()>>>(s);
    return launch_status();
}

int velox_sm100_tp_barrier(const velox_sm100_tp_sync* sync) {
    if (!sync || sync->wait_phase < 0 || sync->signal_phase != sync->wait_phase) return VELOX_ERR_SHAPE;
    TpSync s;
    int rc = tp_sync_fill_elementwise(&s, sync);
    if (rc != 0) return rc;
    EarlyLaunch l(1u, 32u);
    const cudaError_t e = cudaLaunchKernelEx(&l.cfg, tp_barrier_kernel, s);
    note_launch();
    return e != cudaSuccess ? (int)e : (int)cudaGetLastError();
}

int velox_sm100_tp_signal(const velox_sm100_tp_sync* sync) {
    if (!sync || sync->signal_phase < 0) return VELOX_ERR_SHAPE;
    TpSync s;
    int rc = tp_sync_fill_elementwise(&s, sync);
    if (rc != 0) return rc;
    s.wait_phase = -1;
    tp_signal_kernel<<<1, 1, 0, stream()>>>(s);
    return launch_status();
}

}  // extern "C"
