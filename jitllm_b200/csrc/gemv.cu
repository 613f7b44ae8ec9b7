// Dequant-fused quantised matrix-vector product for single-token decode on sm_100a.
//
// What it computes: FloatTensor.matmul of the reference (tensor/standard/FloatTensor.java:123-125)
// for Q8_0 / Q4_0 / Q4_K weights kept in GGUF block layout, optionally with the RMSNorm of the
// input (inference/op/CpuOperations.java:55-73), a residual add (:369-371), SwiGLU over a
// gate/up pair (:255-260) or the greedy argmax (inference/Logits.java:49-60) folded in.
//
// How: the kernel is HBM-bound, so the design goal is "every weight byte crosses HBM once, in
// large aligned bursts, with few issue slots spent per weight, and as little fixed time per launch
// as possible":
//   * one CTA per SM: 16 consumer warps and one producer warp. The producer warp does nothing but
//     issue 1-D bulk async copies (cp.async.bulk, the TMA engine) of weight rows into per-warp
//     rings of shared-memory stages, completing on mbarriers; consumers hand stages back through a
//     second set of mbarriers. The producer starts before the grid dependency is resolved, so under
//     programmatic dependent launch the weight stream runs while the previous kernel drains.
//   * activations: quantised once per CTA into two signed 8-bit digits per element with one scale
//     per 32 elements (16-bit fixed point per block), so the inner product of 4 weights is
//     2 dp4a instructions on the packed integer weights. Integer sums are exact; block results are
//     scaled and accumulated in fp32.
//   * a consumer warp owns one 2048-column chunk of the activation (a lane: 64 elements, in
//     registers for the whole launch) and walks the rows of its group; the warps that hold the
//     other chunks of the same rows leave their partial sums in shared memory and one thread per
//     row adds them in chunk order, applies the RMS factor, residual, SwiGLU or arg-max and stores.
//     Every sum has a fixed order: results do not vary from run to run.
//   * a CTA's rows are one contiguous range, so its output is written in one coalesced burst.
#include "gemv_core.cuh"

#include <climits>
#include <cstdlib>

namespace jl {

JL_TRACE_DEFINE_BIND(gemv_trace_bind)

namespace {

constexpr int kThreads = kGemvThreads;
constexpr int kWarps = kGemvConsumerWarps;
constexpr int kConsumers = kWarps * 32;
constexpr int kBarBytes = 2 * kWarps * kGemvMaxStages * 8 + 128;  // full + empty barriers, then the RMS barrier
constexpr int kScratchFloats = 64;                          // RMS partials, RMS factor, arg-max fold
constexpr int kHeaderBytes = kBarBytes + kScratchFloats * 4;
constexpr int kPartialFloatsMax = 4096;
constexpr int kBarStaged = 1;     // consumers + producer warp: the activation is staged
constexpr int kBarConsumers = 2;  // consumers only: a phase's partial sums are complete / consumed

__device__ __forceinline__ void mbar_arrive_u32(uint32_t bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ bool mbar_test_wait_u32(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(bar), "r"(parity)
        : "memory");
    return ok != 0;
}
__device__ __forceinline__ bool mbar_wait_bounded_u32(uint32_t bar, uint32_t parity, uint32_t limit = (1u << 16)) {
    for (uint32_t i = 0; i < limit; ++i) {
        uint32_t ok;
        asm volatile(
            "{\n\t.reg .pred p;\n\t"
            "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n\t"
            "selp.u32 %0, 1, 0, p;\n\t}"
            : "=r"(ok)
            : "r"(bar), "r"(parity), "r"(kSuspendHintNs)
            : "memory");
        if (ok) return true;
    }
    return false;
}

// Which matrix and row a job of a plain launch is: jobs number the rows of the segments one
// after another.
__device__ __forceinline__ void locate(const GemvArgs &a, int job, int &seg, int &row) {
    seg = 0;
    row = job;
    if (row >= a.seg[0].rows) {
        row -= a.seg[0].rows;
        seg = 1;
        if (a.nseg > 2 && row >= a.seg[1].rows) {
            row -= a.seg[1].rows;
            seg = 2;
        }
    }
}

// A group's walk over its jobs [0, nj), stage by stage. The rows of a stage are consecutive rows of
// one matrix (one contiguous piece of memory, one bulk copy), at most S of them, and never straddle
// the end of a matrix or of a phase. The producer and the consumers of a group run the same walk
// and so agree on every stage.
template <int MODE, int S>
struct StageWalk {
    int k, nj, phase_end, pj;
    int seg, row, seg_left;
    __device__ __forceinline__ void init(const GemvArgs &a, int first_job, int njobs_of_group, int phase_jobs) {
        k = 0;
        nj = njobs_of_group;
        pj = phase_jobs;
        phase_end = min(nj, pj);
        seg = 0;
        row = first_job;
        seg_left = nj;
        if (MODE == kGemvPlain && nj > 0) {
            locate(a, first_job, seg, row);
            seg_left = a.seg[seg].rows - row;
        }
    }
    __device__ __forceinline__ bool done() const { return k >= nj; }
    __device__ __forceinline__ int rows() const { return min(min(S, phase_end - k), seg_left); }
    __device__ __forceinline__ void advance(const GemvArgs &a, int n) {
        k += n;
        row += n;
        if (MODE == kGemvPlain) {
            seg_left -= n;
            if (seg_left == 0 && k < nj) {
                ++seg;
                row = 0;
                seg_left = a.seg[seg].rows;
            }
        }
        if (k == phase_end) phase_end = min(nj, phase_end + pj);
    }
};

template <int TYPE, int MODE>
__global__ void __launch_bounds__(kThreads, 1) gemv_kernel(const GemvArgs a, const GemvPlan pl) {
    extern __shared__ __align__(128) uint8_t smem[];
    constexpr int CB = Fmt<TYPE>::chunk_bytes;
    constexpr int S = Fmt<TYPE>::streams;               // rows per stage
    constexpr int SPJ = (MODE == kGemvGateUp) ? 2 : 1;  // row streams per job
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int trace = trace_begin(kTraceGemv);
    JL_TRACE_MODE_LOCAL;
    if (a.active != nullptr && *a.active == 0) {
        // Still wait: a grid that finished without waiting would let its successor run ahead of
        // the grid before this one.
        pdl_wait();
        return;
    }
    const int nunits = a.cols / 64;
    const int nchunks = pl.nchunks, G = pl.groups, D = pl.stages, PJ = pl.phase_jobs;
    const uint32_t rowb = Fmt<TYPE>::row_bytes(nunits);
    const uint32_t stage_bytes = S * rowb;
    const int total_jobs = (MODE == kGemvGateUp) ? a.seg[0].rows
                                                 : a.seg[0].rows + (a.nseg > 1 ? a.seg[1].rows : 0) +
                                                       (a.nseg > 2 ? a.seg[2].rows : 0);
    const int job0 = gemv_split(total_jobs, blockIdx.x, gridDim.x);
    const int njobs = gemv_split(total_jobs, blockIdx.x + 1, gridDim.x) - job0;

    const uint32_t full_u32 = smem_u32(smem);  // [group][stage], then the same for "empty"
    const uint32_t empty_u32 = full_u32 + kWarps * kGemvMaxStages * 8;
    const uint32_t rms_bar_u32 = full_u32 + 2 * kWarps * kGemvMaxStages * 8;
    float *scratch = reinterpret_cast<float *>(smem + kBarBytes);
    float *sx = reinterpret_cast<float *>(smem + pl.off_x);
    const uint32_t planes_u32 = smem_u32(smem + pl.off_x) + uint32_t(x_scales_bytes(a.cols));
    float *partial = reinterpret_cast<float *>(smem + pl.off_partial);
    const uint32_t ring_u32 = smem_u32(smem + pl.off_ring);

    // One barrier per thread: a single thread initialising all of them would take a microsecond that
    // every launch of the chain would have to wait for.
    if (tid < G * D) {
        const int g = tid / D, s = tid - g * D;
        mbar_init(reinterpret_cast<uint64_t *>(smem) + g * kGemvMaxStages + s, 1);
        mbar_init(reinterpret_cast<uint64_t *>(smem) + (kWarps + g) * kGemvMaxStages + s, nchunks);
        if (tid == 0) mbar_init(reinterpret_cast<uint64_t *>(smem) + 2 * kWarps * kGemvMaxStages, 1);
        mbar_fence_init();
        fence_proxy_async();
    }
    __syncthreads();
    // The next kernel of the chain may be scheduled as soon as SMs free up; whatever it does before
    // its own griddepcontrol.wait touches weights only.
    pdl_launch_dependents();

    if (warp == kWarps) {
        // ---------------------------------------------------------------- producer warp
        // Lane g feeds the ring of group g: one bulk copy per stage, the stage's rows being one
        // contiguous piece of the matrix. Nothing here reads what an earlier kernel wrote.
        if (njobs == 0) return;
        const int g = lane;
        int gs = 0, nj = 0;
        if (g < G) {
            gs = gemv_split(njobs, g, G);
            nj = gemv_split(njobs, g + 1, G) - gs;
        }
        const uint32_t my_full = full_u32 + uint32_t(g) * kGemvMaxStages * 8;
        const uint32_t my_empty = empty_u32 + uint32_t(g) * kGemvMaxStages * 8;
        const uint32_t my_ring = ring_u32 + uint32_t(g) * D * stage_bytes;
        const uint64_t policy = policy_evict_first();
        StageWalk<MODE, S> walk;
        walk.init(a, job0 + gs, nj, PJ);
        int which = 0, slot = 0, use = 0;
        uint32_t idle = 0;
        bool failed = false, joined = false;
        while (true) {
            if (!joined && (idle > 0 || !__any_sync(0xffffffffu, !walk.done()))) {
                // Every ring is full (or all copies are out): nothing to do until the consumers, which
                // are staging the activation, start to hand stages back. Meet them at their barrier
                // and take the one serial piece of the RMSNorm off their hands: the reference
                // narrows 1.0 / Math.sqrt(ss) from double once.
                joined = true;
                named_bar_sync(kBarStaged, kThreads);
                if (a.norm_w != nullptr && lane == 0) {
                    float tot = 0.f;
#pragma unroll
                    for (int w = 0; w < kWarps; ++w) tot += scratch[w];
                    float ms = tot / static_cast<float>(a.cols);
                    ms += a.eps;
                    scratch[kWarps] = static_cast<float>(1.0 / sqrt(static_cast<double>(ms)));
                    mbar_arrive_u32(rms_bar_u32);  // release: the consumers wait on it before they read
                }
                __syncwarp();
            }
            const bool want = !walk.done();
            if (!__any_sync(0xffffffffu, want)) break;
            bool can = false;
            if (want) can = use == 0 || mbar_test_wait_u32(my_empty + slot * 8, uint32_t(use - 1) & 1u);
            if (can) {
                const int n = walk.rows();
                const uint8_t *src = a.seg[MODE == kGemvGateUp ? which : walk.seg].w + size_t(walk.row) * rowb;
                fence_proxy_async();
                mbar_expect_tx_u32(my_full + slot * 8, uint32_t(n) * rowb);
                bulk_g2s_hint_u32(my_ring + slot * stage_bytes, src, uint32_t(n) * rowb, my_full + slot * 8, policy);
                if (SPJ == 2) {
                    which ^= 1;
                    if (which == 0) walk.advance(a, n);
                } else {
                    walk.advance(a, n);
                }
                if (++slot == D) {
                    slot = 0;
                    ++use;
                }
            }
            if (__any_sync(0xffffffffu, can)) {
                idle = 0;
            } else {
                // Every ring is full: stay off the issue ports for a moment. Bounded (about two
                // seconds) so that a consumer that never hands a stage back cannot hang the GPU.
                if (++idle > (1u << 24)) {
                    failed = true;
                    break;
                }
                __nanosleep(100);
            }
        }
        if (failed && lane == 0) atomicExch(a.status, kDevTimeout);
        return;
    }

    // -------------------------------------------------------------------- consumer warps
    const bool norm = a.norm_w != nullptr;
    const int n4 = a.cols / 4;
    float best_v = -INFINITY;
    int best_i = INT_MAX;
    bool failed = false;
    if (njobs > 0) {
        float4 wpre[kStageDeep];
        if (norm) {
#pragma unroll
            for (int k = 0; k < kStageDeep; ++k) {
                const int i = k * kConsumers + tid;
                wpre[k] = i < n4 ? reinterpret_cast<const float4 *>(a.norm_w)[i] : make_float4(0.f, 0.f, 0.f, 0.f);
            }
        }
        pdl_wait();
        trace_mark(trace, 2);
        trace_word(trace, 6, trace_latest_exit());
#ifdef JL_TRACE
        // class of this launch for the per-CTA cells: 0 QKV, 1 output projection, 2 gate/up, 3 down, 4 vocabulary
        const int tcls = MODE == kGemvGateUp ? 2 : (a.argmax_val != nullptr ? 4 : (a.nseg == 3 ? 0 : (a.cols > 8192 ? 3 : 1)));
        if (tid == 0) trace_cta_word(tcls, 3, trace_now());
#endif
#ifdef JL_TRACE
        float ssq = stage_activation_core<kConsumers>(a.x, a.norm_w, wpre, a.cols, tid, sx, planes_u32, tcls);
        if (tid == 0) trace_cta_word(tcls, 5, trace_now());
#else
        float ssq = stage_activation_core<kConsumers>(a.x, a.norm_w, wpre, a.cols, tid, sx, planes_u32);
#endif
        if (norm) {
            ssq = warp_sum(ssq);
            if (lane == 0) scratch[warp] = ssq;
        }
        named_bar_sync(kBarStaged, kThreads);  // the producer warp joins: it computes the RMS factor
        trace_mark(trace, 3);
#ifdef JL_TRACE
        if (tid == 0) {
            unsigned smid;
            asm volatile("mov.u32 %0, %%smid;" : "=r"(smid));
            trace_cta_word(tcls, 0, trace_now());
            trace_cta_word(tcls, 2, smid);
        }
#endif

        const int c = warp % nchunks, g = warp / nchunks;
        int gs = 0, nj = 0;
        if (g < G) {
            gs = gemv_split(njobs, g, G);
            nj = gemv_split(njobs, g + 1, G) - gs;
        }
        const int unit = c * 32 + lane;
        const bool lane_on = unit < nunits;
        UnitX x;
        if (nj > 0 && lane_on) {
            load_unit_x(planes_u32, smem_u32(sx), nunits, unit, x);
        } else {
#pragma unroll
            for (int m = 0; m < kDigits; ++m)
#pragma unroll
                for (int i = 0; i < 8; ++i) x.a[m][i] = x.b[m][i] = 0;
            x.sa = x.sb = x.ma = x.mb = 0.f;
        }
        const uint32_t my_full = full_u32 + uint32_t(g) * kGemvMaxStages * 8;
        const uint32_t my_empty = empty_u32 + uint32_t(g) * kGemvMaxStages * 8;
        const uint32_t my_ring = ring_u32 + uint32_t(g) * D * stage_bytes + uint32_t(c) * CB;
        const int slots = G * PJ * SPJ;  // partial sums per chunk
        const int nphases = ((njobs + G - 1) / G + PJ - 1) / PJ;
        // The residual this thread will add in the (only) epilogue, fetched now so that its trip to
        // L2 is over by then.
        float res_pre = 0.f;
        if (MODE == kGemvPlain && nphases == 1 && tid < G * PJ) {
            const int eg = tid / PJ, jl = tid - eg * PJ;
            const int lj = gemv_split(njobs, eg, G) + jl;
            if (lj < gemv_split(njobs, eg + 1, G)) {
                int seg, row;
                locate(a, job0 + lj, seg, row);
                if (a.seg[seg].res != nullptr) res_pre = __ldcg(a.seg[seg].res + row);
            }
        }
        int slot = 0;
        uint32_t parity = 0;
#ifdef JL_TRACE
        long long t_wait = 0;
        const long long t_loop0 = clock64();
#endif
        StageWalk<MODE, S> walk;
        walk.init(a, job0 + gs, nj, PJ);
        for (int ph = 0; ph < nphases; ++ph) {
            const int k_end = min(nj, (ph + 1) * PJ);
            while (walk.k < k_end) {
                const int k = walk.k;
                const int n = walk.rows();
                // The stages of this step: one, or for a gate/up launch the gate rows' stage and the up
                // rows' stage. All of their rows are multiplied before anything is reduced, so that the
                // dot products of up to four rows overlap and one transposed reduction serves them all.
                constexpr int NV = S * SPJ;
                uint32_t stage[SPJ];
#pragma unroll
                for (int which = 0; which < SPJ; ++which) {
                    if (!failed) {
#ifdef JL_TRACE
                        const long long t_w0 = clock64();
#endif
                        bool ok;
                        if (JL_TRACE_MODE(2)) {
                            ok = false;
                            for (uint32_t sp = 0; sp < (1u << 26) && !ok; ++sp) ok = mbar_test_wait_u32(my_full + slot * 8, parity);
                        } else {
                            ok = mbar_wait_bounded_u32(my_full + slot * 8, parity);
                        }
                        ok = __all_sync(0xffffffffu, ok);
                        failed = !ok;
#ifdef JL_TRACE
                        t_wait += clock64() - t_w0;
#endif
                    }
                    stage[which] = my_ring + slot * stage_bytes;
                    if (!failed && which + 1 < SPJ) {  // the second stage sits in the next slot; both are released below
                        if (++slot == D) {
                            slot = 0;
                            parity ^= 1u;
                        }
                    }
                }
                if (failed) {  // keep walking so that every barrier below is still reached
                    walk.advance(a, n);
                    continue;
                }
                float acc[NV];
#pragma unroll
                for (int which = 0; which < SPJ; ++which)
#pragma unroll
                    for (int i = 0; i < S; ++i)
                        acc[which * S + i] = (lane_on && i < n && !JL_TRACE_MODE(1)) ? unit_dot<TYPE>(stage[which] + i * rowb, lane, x) : 0.f;
                __syncwarp();
                if (lane == 0) {
                    if (SPJ == 2) mbar_arrive_u32(my_empty + (slot == 0 ? D - 1 : slot - 1) * 8);
                    mbar_arrive_u32(my_empty + slot * 8);
                }
                if (++slot == D) {
                    slot = 0;
                    parity ^= 1u;
                }
                // partial sums of this step: row i of matrix `which` at dst[i * SPJ + which]
                float *dst = partial + size_t(c) * slots + (g * PJ + (k - ph * PJ)) * SPJ;
                if constexpr (NV == 4) {
                    // Four values reduced together: after the exchanges over lane bits 4 and 3 each
                    // quarter of the warp holds one of them; lanes 0, 8, 16, 24 end up with the sums.
                    const bool b4 = (lane & 16) != 0, b3 = (lane & 8) != 0;
                    float k0 = b4 ? acc[2] : acc[0], k1 = b4 ? acc[3] : acc[1];
                    const float s0 = b4 ? acc[0] : acc[2], s1 = b4 ? acc[1] : acc[3];
                    k0 += __shfl_xor_sync(0xffffffffu, s0, 16);
                    k1 += __shfl_xor_sync(0xffffffffu, s1, 16);
                    float keep = b3 ? k1 : k0;
                    const float send = b3 ? k0 : k1;
                    keep += __shfl_xor_sync(0xffffffffu, send, 8);
#pragma unroll
                    for (int o = 4; o > 0; o >>= 1) keep += __shfl_xor_sync(0xffffffffu, keep, o);
                    // quarter q = lane / 8 holds acc[q] = (which = q / S, row i = q % S)
                    const int q = lane >> 3;
                    if ((lane & 7) == 0 && (q % S) < n) dst[(q % S) * SPJ + q / S] = keep;
                } else if constexpr (NV == 2) {
                    // Both values reduced together: lanes 0-15 end up with the first, lanes 16-31 with the second.
                    const bool up = (lane & 16) != 0;
                    float keep = up ? acc[1] : acc[0];
                    const float send = up ? acc[0] : acc[1];
                    keep += __shfl_xor_sync(0xffffffffu, send, 16);
#pragma unroll
                    for (int o = 8; o > 0; o >>= 1) keep += __shfl_xor_sync(0xffffffffu, keep, o);
                    const int q = lane >> 4;  // value index: (which, row) = (q / S, q % S)
                    if ((lane & 15) == 0 && (q % S) < n) dst[(q % S) * SPJ + q / S] = keep;
                } else {
                    const float tot = warp_sum(acc[0]);
                    if (lane == 0) dst[0] = tot;
                }
                walk.advance(a, n);
            }
#ifdef JL_TRACE
            if (ph == 0)
                trace_word(trace, 7, (static_cast<unsigned long long>(t_wait) << 32) |
                                         static_cast<unsigned long long>((clock64() - t_loop0) & 0xffffffffll));
#endif
            named_bar_sync(kBarConsumers, kConsumers);
            // One thread per job: add the chunks in order, finish, store.
            unsigned tp_seq = 0;
            unsigned long long tp_t0 = 0, tp_limit = 0;
            if (MODE == kGemvPlain && a.tpr.tp > 1) {
                tp_seq = *reinterpret_cast<volatile unsigned *>(&a.tpr.ctr[0]);  // moves on only after every CTA is done
                tp_t0 = tpx::global_ns();
                tp_limit = tpx::patience(a.status, a.tpr.timeout_ns);
            }
            if (norm && ph == 0 && !mbar_wait_bounded_u32(rms_bar_u32, 0)) failed = true;
            const float rms = norm ? scratch[kWarps] : 1.0f;
            for (int idx = tid; idx < G * PJ; idx += kConsumers) {
                const int eg = idx / PJ, jl = idx - eg * PJ;
                const int egs = gemv_split(njobs, eg, G), ege = gemv_split(njobs, eg + 1, G);
                const int lj = egs + ph * PJ + jl;  // job within this CTA
                if (lj >= ege) continue;
                const float *pp = partial + size_t(idx) * SPJ;
                if (MODE == kGemvGateUp) {
                    float gt = 0.f, ut = 0.f;
                    for (int cc = 0; cc < nchunks; ++cc) {
                        gt += pp[size_t(cc) * slots];
                        ut += pp[size_t(cc) * slots + 1];
                    }
                    gt *= rms;
                    ut *= rms;
                    const float silu = gt / (1.0f + expf(-gt));
                    a.seg[0].y[job0 + lj] = silu * ut;
                } else {
                    float v = 0.f;
                    for (int cc = 0; cc < nchunks; ++cc) v += pp[size_t(cc) * slots];
                    v *= rms;
                    int seg, row;
                    locate(a, job0 + lj, seg, row);
                    if (a.tpr.tp > 1) {
                        // Row-parallel projection under tensor parallelism: v is this GPU's share of the
                        // row. Push it to the peers, collect theirs, add in rank order.
                        const GemvTpReduce &t = a.tpr;
                        const size_t at = size_t(t.row_offset) + row;
                        const size_t slot_at = t.base + size_t(tp_seq & 1u) * t.tp * t.cap;
                        for (int k = 1; k < t.tp; ++k) {
                            const int r = (t.rank + k) % t.tp;  // every GPU starts with a different peer
                            tpx::store_packet(t.inbox.of[r] + slot_at + size_t(t.rank) * t.cap + at, __float_as_uint(v), tp_seq);
                        }
                        const uint2 *own = t.inbox.of[t.rank] + slot_at + at;
                        float sum = 0.f;
                        for (int r = 0; r < t.tp; ++r) {
                            const float pv = r == t.rank ? v
                                                         : __uint_as_float(tpx::wait_packet(own + size_t(r) * t.cap, tp_seq, tp_t0,
                                                                                            tp_limit, a.status));
                            sum = r == 0 ? pv : sum + pv;
                        }
                        v = sum;
                    }
                    if (a.seg[seg].res != nullptr) v = (nphases == 1 ? res_pre : a.seg[seg].res[row]) + v;
                    a.seg[seg].y[row] = v;
                    if (v > best_v || (v == best_v && row < best_i)) {
                        best_v = v;
                        best_i = row;
                    }
                }
            }
            if (ph + 1 < nphases) named_bar_sync(kBarConsumers, kConsumers);  // partials are reused
        }
        trace_mark(trace, 4);
#ifdef JL_TRACE
        if (tid == 0) trace_cta_word(tcls, 1, trace_now());
#endif
        if (failed) {
            // Give copies already in flight a bounded chance to land before this CTA's shared memory
            // is released, then report; the host turns the status word into an error.
            if (g < G)
                for (int s = 0; s < D; ++s) mbar_wait_bounded_u32(my_full + s * 8, 0, 16);
            if (lane == 0) atomicExch(a.status, kDevTimeout);
        }
    } else {
        pdl_wait();
    }

    if (MODE == kGemvPlain && a.tpr.tp > 1) {
        // The last CTA to finish moves the exchange's sequence number on; every CTA has read it by then.
        named_bar_sync(kBarConsumers, kConsumers);
        if (tid == 0) {
            const unsigned seq = *reinterpret_cast<volatile unsigned *>(&a.tpr.ctr[0]);
            __threadfence();
            const unsigned arrived = atomicAdd(&a.tpr.ctr[1], 1u);
            if (arrived == gridDim.x - 1) {
                a.tpr.ctr[1] = 0u;
                __threadfence();
                *reinterpret_cast<volatile unsigned *>(&a.tpr.ctr[0]) = tp_next_sequence(seq);
            }
        }
    }
    if (a.argmax_val != nullptr) {
        // Warp, block, then grid reduction of (value, first index).
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float ov = __shfl_xor_sync(0xffffffffu, best_v, o);
            const int oi = __shfl_xor_sync(0xffffffffu, best_i, o);
            if (ov > best_v || (ov == best_v && oi < best_i)) {
                best_v = ov;
                best_i = oi;
            }
        }
        float *bv = scratch + 32;
        int *bi = reinterpret_cast<int *>(scratch + 48);
        if (lane == 0) {
            bv[warp] = best_v;
            bi[warp] = best_i;
        }
        named_bar_sync(kBarConsumers, kConsumers);
        if (tid == 0) {
            float v = bv[0];
            int i = bi[0];
            for (int w = 1; w < kWarps; ++w)
                if (bv[w] > v || (bv[w] == v && bi[w] < i)) {
                    v = bv[w];
                    i = bi[w];
                }
            a.argmax_val[blockIdx.x] = v;
            a.argmax_idx[blockIdx.x] = i;
            __threadfence();
            const unsigned prev = atomicAdd(a.argmax_count, 1u);
            if (prev == gridDim.x - 1) {
                __threadfence();
                float fv = -INFINITY;
                int fi = INT_MAX;
                for (unsigned b = 0; b < gridDim.x; ++b) {
                    const float ov = __ldcg(a.argmax_val + b);
                    const int oi = __ldcg(a.argmax_idx + b);
                    if (ov > fv || (ov == fv && oi < fi)) {
                        fv = ov;
                        fi = oi;
                    }
                }
                // Logits.argmax starts from index 0 and only moves on a strictly greater value.
                *a.out_token = (fi == INT_MAX) ? 0 : fi;
                *a.argmax_count = 0u;
            }
        }
    }
    trace_mark(trace, 5);
    if (tid == 0) trace_cta_exit();
}

template <int TYPE, int MODE>
cudaError_t configure_one() {
    return cudaFuncSetAttribute(gemv_kernel<TYPE, MODE>, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024);
}

template <int TYPE, int MODE>
cudaError_t launch_one(const GemvArgs &args, const GemvPlan &plan, cudaStream_t stream, bool programmatic) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(plan.grid);
    cfg.blockDim = dim3(kThreads);
    cfg.dynamicSmemBytes = plan.smem_bytes;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = programmatic ? 1 : 0;
    return cudaLaunchKernelEx(&cfg, gemv_kernel<TYPE, MODE>, args, plan);
}

template <int TYPE>
cudaError_t launch_mode(const GemvArgs &a, const GemvPlan &p, cudaStream_t s, bool pdl) {
    if (a.mode == kGemvGateUp) return launch_one<TYPE, kGemvGateUp>(a, p, s, pdl);
    return launch_one<TYPE, kGemvPlain>(a, p, s, pdl);
}

template <int TYPE>
cudaError_t configure_type() {
    cudaError_t e;
    if ((e = configure_one<TYPE, kGemvPlain>()) != cudaSuccess) return e;
    return configure_one<TYPE, kGemvGateUp>();
}

}  // namespace

bool gemv_plan(int type, int cols, int total_rows, int mode, int sm_count, GemvPlan *out) {
    if (!gemv_takes(type, cols) || cols > kGemvMaxCols || total_rows <= 0) return false;
    const size_t rowb = size_t(gemv_row_bytes(type, cols));
    const size_t stage = gemv_rows_per_stage(type) * rowb;
    const int spj = mode == kGemvGateUp ? 2 : 1;
    const int jobs = total_rows / spj;
    GemvPlan p = {};
    p.grid = sm_count;
    p.nchunks = (cols + kGemvChunkCols - 1) / kGemvChunkCols;
    p.groups = kGemvConsumerWarps / p.nchunks;
    // Jobs per group between two epilogues: all of a CTA's rows when their partial sums fit (they do
    // for every decode shape), otherwise as many as fit, in several phases.
    const int per_cta = (jobs + p.grid - 1) / p.grid;
    const int per_group = (per_cta + p.groups - 1) / p.groups;
    int pj = kPartialFloatsMax / (p.nchunks * p.groups * spj);
    if (pj < 1) return false;
    if (per_group < pj) pj = per_group;
    p.phase_jobs = pj;
    p.off_x = kHeaderBytes;
    p.off_partial = p.off_x + int(x_region_bytes(cols));
    p.off_ring = int(align_up(size_t(p.off_partial) + size_t(p.nchunks) * p.groups * pj * spj * 4, 128));
    const size_t budget = 227 * 1024;
    if (size_t(p.off_ring) + size_t(p.groups) * 2 * stage > budget) return false;
    int s = int((budget - p.off_ring) / (size_t(p.groups) * stage));
    if (s > kGemvMaxStages) s = kGemvMaxStages;
    p.stages = s;
    p.smem_bytes = size_t(p.off_ring) + size_t(p.groups) * s * stage;
    *out = p;
    return true;
}

cudaError_t gemv_configure() {
    cudaError_t e;
    if ((e = configure_type<kQ4_K>()) != cudaSuccess) return e;
    if ((e = configure_type<kQ4_0>()) != cudaSuccess) return e;
    if ((e = configure_type<kQ6_K>()) != cudaSuccess) return e;
    if ((e = configure_type<kQ5_K>()) != cudaSuccess) return e;
    if ((e = configure_type<kQ4_1>()) != cudaSuccess) return e;
    return configure_type<kQ8_0>();
}

cudaError_t gemv_launch(const GemvArgs &args, const GemvPlan &plan, cudaStream_t stream, bool programmatic) {
    switch (args.type) {
        case kQ4_K: return launch_mode<kQ4_K>(args, plan, stream, programmatic);
        case kQ4_0: return launch_mode<kQ4_0>(args, plan, stream, programmatic);
        case kQ8_0: return launch_mode<kQ8_0>(args, plan, stream, programmatic);
        case kQ6_K: return launch_mode<kQ6_K>(args, plan, stream, programmatic);
        case kQ5_K: return launch_mode<kQ5_K>(args, plan, stream, programmatic);
        case kQ4_1: return launch_mode<kQ4_1>(args, plan, stream, programmatic);
        default: return cudaErrorInvalidValue;
    }
}

}  // namespace jl
