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

// The sequence number after `seq`. Two inbox slots alternate by its lowest bit and 0 means "never
// written", so the step from 0xFFFFFFFF must skip 0 and still change parity: it goes to 2.
__host__ __device__ inline unsigned tp_next_sequence(unsigned seq) { return seq + 1u == 0u ? 2u : seq + 1u; }

}  // namespace jl
