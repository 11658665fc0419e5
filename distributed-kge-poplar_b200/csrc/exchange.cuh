// Flag-based synchronisation of the exchange steps of a training step, folded into the kernels
// that produce and consume the exchanged data.
//
// A step has four hand-overs between processes (one process per GPU): the tail rows
// (src/poplar_kge.cpp:680-681), their gradients (the backward of the same all-to-all), the partial
// gradients of the dense parameters, and the updated dense parameters (the reduce-scatter /
// all-gather pair of src/pag/pag.cpp:980-994).  The producer of each writes straight into the
// consumers' memory over NVLink; what remains is to tell the consumer that the data has arrived.
// Instead of a barrier kernel between producer and consumer,
//   - the last block of the producing kernel to finish publishes a new epoch of that hand-over
//     into every process's flag array (exchange_signal), and
//   - every block of the consuming kernel waits until all processes' flags have reached the
//     epoch this process has itself published (exchange_wait) before it reads.
// All processes run the same sequence of kernels, so "the epoch I have published" is the epoch
// to wait for.  Waits are bounded: on expiry the block records which process was missing in the
// status word and goes on; once the word is set no later wait spins again, and the host turns
// the word into an error after the run.
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>

namespace kge {

enum ExchangeKind : int { XCHG_TAILS = 0, XCHG_TAIL_GRADS = 1, XCHG_DENSE_PARTIALS = 2, XCHG_DENSE_PARAMS = 3, XCHG_KINDS = 4 };
constexpr int kMaxProcesses = 64;
// A process's flag array: [1 + XCHG_KINDS][kMaxProcesses] words; row 0 belongs to the plain barrier kernel.
constexpr size_t kFlagWords = (size_t)(1 + XCHG_KINDS) * kMaxProcesses;

struct ExchangeSync {
    unsigned* const* peer_flags;  // [world] every process's flag array (peer-visible memory)
    unsigned* epochs;             // [XCHG_KINDS] epochs this process has published (device memory of its own)
    unsigned* counters;           // [XCHG_KINDS] blocks of the publishing kernel that have finished
    unsigned* status;             // device error word
    int rank, world;
    unsigned max_spins;            // a wait gives up after this many polls ...
    unsigned long long timeout_ns; // ... or this long, whichever comes first
    // Optional time stamps (nanoseconds of the GPU's global timer), [kTraceSlots][XCHG_KINDS][3]:
    // when this process published an epoch, and when its first consuming block began and ended
    // its wait for that epoch; slot = epoch % kTraceSlots.  Null: no stamps.
    unsigned long long* trace;
};
constexpr int kTraceSlots = 256;

#ifdef __CUDACC__
__device__ __forceinline__ unsigned long long global_timer_ns() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}

// Called by every thread of every block of the producing kernel once the block's writes have been
// issued (contains __syncthreads).  `total_blocks` = blocks of the grid.
__device__ __forceinline__ void exchange_signal(const ExchangeSync& s, int kind, unsigned total_blocks) {
    if (s.world <= 1 || kind < 0) return;
    __syncthreads();  // the block's writes are ordered before thread 0's fence, which is cumulative
    if (threadIdx.x == 0 && threadIdx.y == 0 && threadIdx.z == 0) {
        __threadfence();  // release at device scope: pairs with the last block's fence after the counter
        const unsigned done = atomicAdd(&s.counters[kind], 1u) + 1u;
        if (done == total_blocks) {
            __threadfence_system();  // everything that happened before, on any SM, precedes the flags for any observer
            s.counters[kind] = 0;
            const unsigned epoch = *reinterpret_cast<volatile unsigned*>(&s.epochs[kind]) + 1u;
            *reinterpret_cast<volatile unsigned*>(&s.epochs[kind]) = epoch;
            for (int p = 0; p < s.world; ++p)
                *reinterpret_cast<volatile unsigned*>(s.peer_flags[p] + (size_t)(1 + kind) * kMaxProcesses + s.rank) = epoch;
            if (s.trace) s.trace[((size_t)(epoch % kTraceSlots) * XCHG_KINDS + kind) * 3 + 0] = global_timer_ns();
        }
    }
}

__device__ __forceinline__ unsigned load_acquire_system(const unsigned* p) {
    unsigned v;
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}

// Called by every thread of every block of the consuming kernel before it reads exchanged data
// (contains __syncthreads; the block needs at least `world` threads).  Thread t reads process t's
// flag with acquire semantics at system scope; the barrier passes that on to the block.
__device__ __forceinline__ void exchange_wait(const ExchangeSync& s, int kind) {
    if (s.world <= 1 || kind < 0) return;
    const int t = threadIdx.x + blockDim.x * (threadIdx.y + blockDim.y * threadIdx.z);
    if (t < s.world) {
        const unsigned want = __ldcg(&s.epochs[kind]);
        const bool stamp = s.trace && t == 0 && blockIdx.x == 0 && blockIdx.y == 0 && blockIdx.z == 0;
        if (stamp) s.trace[((size_t)(want % kTraceSlots) * XCHG_KINDS + kind) * 3 + 1] = global_timer_ns();
        const unsigned* flag = s.peer_flags[s.rank] + (size_t)(1 + kind) * kMaxProcesses + t;
        if ((int)(load_acquire_system(flag) - want) < 0 && __ldcg(s.status) == 0) {
            // bounded by the GPU's global timer (and by a count, should the timer not advance)
            const unsigned long long deadline = global_timer_ns() + s.timeout_ns;
            unsigned spins = 0;
            while ((int)(load_acquire_system(flag) - want) < 0) {
                if (++spins > s.max_spins || ((spins & 63u) == 0 && global_timer_ns() > deadline)) {
                    atomicExch(s.status, 1u + (unsigned)t);
                    break;
                }
                __nanosleep(20);
            }
        }
    }
    __syncthreads();
    if (s.trace && t == 0 && blockIdx.x == 0 && blockIdx.y == 0 && blockIdx.z == 0)  // all processes' flags have arrived
        s.trace[((size_t)(__ldcg(&s.epochs[kind]) % kTraceSlots) * XCHG_KINDS + kind) * 3 + 2] = global_timer_ns();
}

// The two halves as kernels of their own, for producers and consumers that have no fused form.
static __global__ void k_exchange_signal(ExchangeSync s, int kind) {
    asm volatile("griddepcontrol.wait;" ::: "memory");
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    exchange_signal(s, kind, 1u);
}
static __global__ void k_exchange_wait(ExchangeSync s, int kind) {
    asm volatile("griddepcontrol.wait;" ::: "memory");
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    exchange_wait(s, kind);
}
#endif

}  // namespace kge
