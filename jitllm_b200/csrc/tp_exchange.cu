#include "tp_exchange.cuh"

#include "common.cuh"

namespace jl {
namespace {

using namespace tpx;

static_assert(kDevTimeout == 1 && kDevOk == 0, "tpx::wait_packet and tpx::patience spell the status values out");

// The last CTA to finish moves the sequence on. Every CTA has read it by then.
__device__ __forceinline__ void advance_sequence(unsigned *ctr, unsigned seq) {
    __syncthreads();
    if (threadIdx.x == 0) {
        __threadfence();
        const unsigned arrived = atomicAdd(&ctr[1], 1u);
        if (arrived == gridDim.x - 1) {
            ctr[1] = 0u;
            __threadfence();
            *reinterpret_cast<volatile unsigned *>(&ctr[0]) = tp_next_sequence(seq);
        }
    }
}

constexpr int kExchangeThreads = 128;

// One element per thread: push this GPU's partial sum to every peer, collect the peers' partial
// sums of the same element, add them in rank order (every GPU computes the same bits) into x.
__global__ void __launch_bounds__(kExchangeThreads) tp_push_reduce_kernel(const TpReduceArgs a) {
    pdl_wait();
    pdl_launch_dependents();
    const unsigned long long t0 = global_ns();
    const unsigned long long limit = patience(a.status, a.timeout_ns);
    const unsigned seq = *reinterpret_cast<volatile unsigned *>(&a.ctr[0]);
    const size_t slot = seq & 1u;
    const int i = blockIdx.x * kExchangeThreads + threadIdx.x;
    if (i < a.count) {
        const float mine = a.part[i];
        const size_t out_at = a.base + (slot * a.tp + a.rank) * a.cap + i;
        for (int k = 1; k < a.tp; ++k) {
            const int r = (a.rank + k) % a.tp;  // every GPU starts with a different peer
            store_packet(a.inbox.of[r] + out_at, __float_as_uint(mine), seq);
        }
        const uint2 *own = a.inbox.of[a.rank] + a.base + slot * a.tp * a.cap + i;
        float sum = 0.f;
        for (int r = 0; r < a.tp; ++r) {
            const float v = r == a.rank ? mine
                                        : __uint_as_float(wait_packet(own + size_t(r) * a.cap, seq, t0, limit, a.status));
            sum = r == 0 ? v : sum + v;
        }
        a.x[i] = a.x[i] + sum;
    }
    advance_sequence(a.ctr, seq);
}

// One row per thread: push (best logit, global index) of this GPU's vocabulary shard, collect the
// peers', keep the largest value and among equals the lowest index.
__global__ void __launch_bounds__(kExchangeThreads) tp_push_best_kernel(const TpBestArgs a) {
    pdl_wait();
    pdl_launch_dependents();
    const unsigned long long t0 = global_ns();
    const unsigned long long limit = patience(a.status, a.timeout_ns);
    const unsigned seq = *reinterpret_cast<volatile unsigned *>(&a.ctr[0]);
    const size_t slot = seq & 1u;
    const int r = blockIdx.x * kExchangeThreads + threadIdx.x;
    if (r < a.n) {
        const int li = a.local[r];
        const float lv = a.logits[size_t(r) * a.l_vocab + li];
        const int gi = li + a.rank * a.l_vocab;
        const size_t out_at = a.base + (slot * a.tp + a.rank) * a.cap + 2 * size_t(r);
        for (int k = 1; k < a.tp; ++k) {
            const int p = (a.rank + k) % a.tp;
            store_packet(a.inbox.of[p] + out_at, __float_as_uint(lv), seq);
            store_packet(a.inbox.of[p] + out_at + 1, uint32_t(gi), seq);
        }
        const uint2 *own = a.inbox.of[a.rank] + a.base + slot * a.tp * a.cap + 2 * size_t(r);
        float bv = lv;
        int bi = gi;
        for (int p = 0; p < a.tp; ++p) {
            if (p == a.rank) continue;
            const float v = __uint_as_float(wait_packet(own + size_t(p) * a.cap, seq, t0, limit, a.status));
            const int i = int(wait_packet(own + size_t(p) * a.cap + 1, seq, t0, limit, a.status));
            if (v > bv || (v == bv && i < bi)) {
                bv = v;
                bi = i;
            }
        }
        if (a.active == nullptr || a.active[r] != 0) a.out[r] = bi;
    }
    advance_sequence(a.ctr, seq);
}

template <typename Args>
cudaError_t launch(void (*kernel)(const Args), const Args &a, int items, cudaStream_t stream, bool programmatic) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((items + kExchangeThreads - 1) / kExchangeThreads);
    cfg.blockDim = dim3(kExchangeThreads);
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = programmatic ? 1 : 0;
    return cudaLaunchKernelEx(&cfg, kernel, a);
}

}  // namespace

cudaError_t tp_push_reduce_launch(const TpReduceArgs &a, cudaStream_t stream, bool programmatic) {
    if (a.tp < 2 || a.tp > kTpMaxRanks || a.count <= 0 || size_t(a.count) > a.cap) return cudaErrorInvalidValue;
    return launch(tp_push_reduce_kernel, a, a.count, stream, programmatic);
}

cudaError_t tp_push_best_launch(const TpBestArgs &a, cudaStream_t stream, bool programmatic) {
    if (a.tp < 2 || a.tp > kTpMaxRanks || a.n <= 0 || 2 * size_t(a.n) > a.cap) return cudaErrorInvalidValue;
    return launch(tp_push_best_kernel, a, a.n, stream, programmatic);
}

}  // namespace jl
