// Cross-GPU ordering of the tensor-parallel step without barrier kernels: a kernel that produces
// data other ranks read publishes a step counter in a flag table on every rank when its last CTA is
// done; a kernel that consumes such data polls its own rank's table before its first read.
//
// A table is `phases` rows of VX_MAX_PEERS 32-bit words (row = a point of the step, column = the
// rank that signals), zero when allocated and never reset: the value written is the rank's step
// counter ("epoch"), which velox_sm100_tp_step_begin increments once per step, and a waiter accepts
// any value that has reached its own epoch. Every wait is bounded by a wall-clock limit; a wait
// that runs out records ST_TIMEOUT_PEER in the kernel family's status word and the kernel goes on
// and exits normally (its output is then meaningless, which the status word says).
//
// The reference has no tensor parallelism; its convention followed here is the launcher status /
// sticky-error path (crates/velox-cuda/src/lib.rs:85-112).
#pragma once

#include "common.cuh"

namespace vx {

constexpr int TP_FLAG_STRIDE = VX_MAX_PEERS;   // words per row of a flag table
constexpr int ST_TIMEOUT_PEER = 6;             // a peer's flag did not arrive within the limit

struct TpSync {
    unsigned long long flags[VX_MAX_PEERS];   // every rank's table as mapped on this GPU; [rank] is this rank's own
    const unsigned int* epoch;                // this rank's step counter (device memory)
    unsigned int* ticket;                     // elects the last CTA of a signalling launch; zero between launches
    int* status;
    unsigned long long limit_ns;
    int n, rank;
    int wait_phase, signal_phase;             // rows of the table; -1 = none
};

__device__ __forceinline__ unsigned int ld_relaxed_sys_u32(const unsigned int* p) {
    unsigned int v;
    asm volatile("ld.relaxed.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}

__device__ __forceinline__ void st_relaxed_sys_u32(unsigned int* p, unsigned int v) {
    asm volatile("st.relaxed.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}

__device__ __forceinline__ unsigned long long tp_timer_ns() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
    return t;
}

// Called by one thread, after the kernel's dependency on the launch ahead of it is resolved:
// returns once every rank's flag in row wait_phase has reached this step's epoch, or false after
// limit_ns with the status word set. The polls are relaxed loads; one system-scope fence after the
// last of them orders everything this thread (and, behind a barrier, its CTA) reads afterwards
// behind the peers' writes that preceded their flags.
static __device__ __noinline__ bool tp_wait_flags(const TpSync& s) {
    if (s.wait_phase < 0 || s.n <= 0) return true;
    const unsigned int want = *reinterpret_cast<const volatile unsigned int*>(s.epoch);
    const unsigned int* row =
        reinterpret_cast<const unsigned int*>(s.flags[s.rank]) + (long long)s.wait_phase * TP_FLAG_STRIDE;
    const unsigned long long t0 = tp_timer_ns();
    bool ok = true;
    for (int src = 0; src < s.n && ok; src++) {
        unsigned int spins = 0;
        while ((int)(ld_relaxed_sys_u32(row + src) - want) < 0) {
            __nanosleep(32);
            if ((++spins & 63u) == 0 && tp_timer_ns() - t0 > s.limit_ns) {
                atomicExch(s.status, ST_TIMEOUT_PEER);
                ok = false;
                break;
            }
        }
    }
    __threadfence_system();
    return ok;
}

// Called by one thread of every CTA, behind a CTA-wide barrier that follows the CTA's last store
// (and the completion of its bulk stores): each CTA makes its writes visible system-wide and takes
// a ticket; the CTA that takes the last one writes the epoch into row signal_phase, column rank, of
// every rank's table (relaxed stores behind one fence: a release store per peer would serialise a
// round trip over the links for each of them).
static __device__ __noinline__ void tp_signal(const TpSync& s, unsigned int ctas) {
    if (s.signal_phase < 0 || s.n <= 0) return;
    __threadfence_system();
    const unsigned int t = atomicAdd(s.ticket, 1u);
    if (t + 1u != ctas) return;
    atomicExch(s.ticket, 0u);
    __threadfence_system();
    const unsigned int e = *reinterpret_cast<const volatile unsigned int*>(s.epoch);
    for (int d = 0; d < s.n; d++)
        st_relaxed_sys_u32(reinterpret_cast<unsigned int*>(s.flags[d]) + (long long)s.signal_phase * TP_FLAG_STRIDE + s.rank, e);
}

// Host side: the C-ABI description of a launch's waits and signals, completed with the library's
// own words (ticket, status, limit). `sync` may be NULL: no waits, no signals.
int tp_sync_fill(TpSync* out, const velox_sm100_tp_sync* sync, unsigned int* ticket, int* status);
unsigned long long tp_wait_limit_ns();
// The same with the words of the step's elementwise kernels (norm, finish, wait).
int tp_sync_fill_elementwise(TpSync* out, const velox_sm100_tp_sync* sync);

}  // namespace vx
