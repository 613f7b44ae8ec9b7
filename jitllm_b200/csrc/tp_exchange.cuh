// Small-message exchanges between the GPUs of a tensor-parallel group, done by one kernel per
// exchange over peer memory (plain stores into the other GPUs' inboxes through NVLink, plain loads
// from this GPU's own inbox) instead of a library collective: at decode sizes (a few KB to a few
// hundred KB) a collective's fixed cost is several times the cost of the data movement.
#pragma once
#include <cuda_runtime.h>

#include <cstddef>
#include <cstdint>

namespace jl {

constexpr int kTpMaxRanks = 8;

// Every GPU owns one inbox; all ranks map all inboxes. Words are packets {payload, sequence}: an
// aligned 8-byte store lands whole, so a reader that sees the sequence number it waits for also
// sees the payload, and no fence or separate flag is needed. Two slots alternate by sequence
// parity: a peer can be at most one exchange ahead of this GPU, so it never overwrites a packet
// that is still to be read.
struct TpInboxes {
    uint2 *of[kTpMaxRanks];  // of[r]: rank r's inbox as addressable from this GPU (own at [rank])
};

struct TpReduceArgs {
    const float *part;  // this GPU's partial sums [count]
    float *x;           // residual stream [count]: x += sum over ranks of part
    TpInboxes inbox;
    size_t base;        // packet offset of the reduce region inside an inbox
    size_t cap;         // packets per (slot, source rank) in that region
    int tp, rank, count;
    unsigned *ctr;      // [0] sequence of the next exchange (starts at 1), [1] CTA arrivals
    int *status;
    unsigned long long timeout_ns;
};

struct TpBestArgs {
    const float *logits;  // [n][l_vocab] this GPU's vocabulary shard
    const int32_t *local; // [n] first maximum inside the shard
    int32_t *out;         // [n] first maximum over the whole vocabulary
    const uint8_t *active;
    TpInboxes inbox;
    size_t base, cap;     // the arg-max region: 2 packets per row
    int tp, rank, n, l_vocab;
    unsigned *ctr;
    int *status;
    unsigned long long timeout_ns;
};

cudaError_t tp_push_reduce_launch(const TpReduceArgs &a, cudaStream_t stream, bool programmatic);
cudaError_t tp_push_best_launch(const TpBestArgs &a, cudaStream_t stream, bool programmatic);

#ifdef __CUDACC__
// ---- device side of the exchange, shared by the exchange kernels and the mat-vec epilogue -------
namespace tpx {

__device__ __forceinline__ void store_packet(uint2 *p, uint32_t payload, uint32_t seq) {
    asm volatile("st.volatile.global.v2.u32 [%0], {%1, %2};" ::"l"(p), "r"(payload), "r"(seq) : "memory");
}
__device__ __forceinline__ uint2 load_packet(const uint2 *p) {
    uint2 v;
    asm volatile("ld.volatile.global.v2.u32 {%0, %1}, [%2];" : "=r"(v.x), "=r"(v.y) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ unsigned long long global_ns() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
    return t;
}
// Waits for the packet with sequence `seq`; gives up after timeout_ns (a peer that stopped), records
// that in *status (value 1 = a bounded device-side wait gave up) and returns 0 so that the kernel still ends.
__device__ __forceinline__ uint32_t wait_packet(const uint2 *p, uint32_t seq, unsigned long long t0,
                                                unsigned long long timeout_ns, int *status) {
    for (unsigned spins = 0;; ++spins) {
        const uint2 v = load_packet(p);
        if (v.y == seq) return v.x;
        if ((spins & 255u) == 255u) {
            if (global_ns() - t0 > timeout_ns) {
                atomicExch(status, 1);
                return 0u;
            }
            __nanosleep(64);
        }
    }
}
// Once a wait has run out the group is out of step: later exchanges of the same step do not wait
// again, so that a step with a stopped peer costs one time-out, not one per exchange.
__device__ __forceinline__ unsigned long long patience(const int *status, unsigned long long timeout_ns) {
    return *reinterpret_cast<const volatile int *>(status) == 0 ? timeout_ns : 0ull;
}

}  // namespace tpx
#endif

// The sequence number after `seq`. Two inbox slots alternate by its lowest bit and 0 means "never
// written", so the step from 0xFFFFFFFF must skip 0 and still change parity: it goes to 2.
__host__ __device__ inline unsigned tp_next_sequence(unsigned seq) { return seq + 1u == 0u ? 2u : seq + 1u; }

}  // namespace jl
