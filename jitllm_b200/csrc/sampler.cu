// Temperature / top-p sampling on the device: a cluster of eight CTAs per batch row turns the row of
// logits the vocabulary projection left in device memory into a token id, so that a non-greedy decode
// step returns 4 bytes per sequence instead of the whole row (513 KB at a 128 256-token vocabulary).
//
// What it computes is the reference's sampler chain, inference/sampler/Sampler.java:63-110:
//   scores /= temperature; softmaxInPlace (tensor/standard/FloatTensor.java:248-256: max, (float) Math.exp(f - max),
//   sum, divide); then CategoricalSampler.sampleToken (CategoricalSampler.java:13-25) or
//   ToppSampler.sampleToken (ToppSampler.java:46-103): largest first until the running sum exceeds topp,
//   r = u * that sum, first candidate whose running sum exceeds r.
// The random number u comes from the caller (the reference draws rng.nextFloat(1f) once per call): the
// generator stays on the host. As in the reference the row is overwritten (with e = exp(score - max)). The
// exponential is expf (within 2 units in the last place of the reference's (float) Math.exp): a double-precision
// exp cost 130 us per row of 128 256 tokens, and a last-bit difference in e is two orders of magnitude below the
// rounding of the reference's own fp32 running sums.
//
// How. Everything is done on e, not on e / sum: dividing by a positive constant keeps the order, and
// "running sum of p exceeds t" is "running sum of e exceeds t * sum". The reference's cut-off (candidates with
// p >= (1 - topp) / (n - 1)) is an optimisation without effect on the result - all the elements below it
// together hold less than 1 - topp, so the running sum passes topp before it reaches them - and is not needed.
// Nothing is sorted: "the element where the running sum, largest first, crosses t" is found by descending the
// binary32 bit pattern of e (non-negative floats order like their bits) 11 + 11 + 9 bits at a time: each CTA
// builds a histogram (count and sum per bucket) of its eighth of the row over the elements that match the
// prefix found so far, the cluster's first CTA adds the eight histograms through distributed shared memory,
// scans from the top to the bucket where the sum crosses, and hands the result back. Sums are exact integers
// (e x 2^40 in 64 bits), so the result does not depend on the order of the additions: the same row and the
// same u give the same token on every run, and ties go in index order. Against the reference's sequential
// fp32 sums this differs only when r falls within rounding of a boundary of the cumulative distribution
// (at 128 256 tokens that rounding is about 1e-5).
#include "sampler.cuh"

#include "common.cuh"

namespace jl {

namespace {

constexpr int kCluster = 8;
constexpr int kSampleThreads = 1024;
constexpr int kSampleWarps = kSampleThreads / 32;
constexpr int kBuckets = 2048;
constexpr int kKeep = 16;  // elements a thread keeps in registers between the passes (8 x 1024 x 16 = 131 072 per row)

__device__ __forceinline__ unsigned long long to_fixed(float e) {
    return static_cast<unsigned long long>(__float2ull_rz(e * 1099511627776.0f));  // exact scaling by 2^40
}

struct Pick {  // what a scan of a merged histogram found
    unsigned long long above;  // mass strictly before the chosen bucket (largest first)
    unsigned long long bsum;   // mass of the chosen bucket
    unsigned bcnt;             // elements in it
    int bucket;                // -1: the running sum never exceeds the target
    unsigned long long total;  // first level only: the mass of the whole row
};

struct SampleSmem {
    // this CTA's histogram of the current level: the sum of a bucket in three 32-bit limbs of 14 bits each
    // (a slice has at most 2^16 elements of 41 bits), because shared memory adds 32-bit words natively while a
    // 64-bit addition there is a compare-and-swap loop that many warps on a few buckets keep retrying
    unsigned hlimb[3][kBuckets];
    unsigned hcnt[kBuckets];
    unsigned long long g1sum[kBuckets];  // first CTA only: the merged first-level histogram (used three times)
    unsigned g1cnt[kBuckets];
    unsigned long long wsum[kSampleWarps];
    unsigned wcnt[kSampleWarps];
    float wred[kSampleWarps];
    // one slot per CTA of the cluster, written by its owner into every CTA's copy
    float cmax[kCluster];
    unsigned long long csum[kCluster];
    unsigned long long ccnt[kCluster];
    Pick pick;  // written by the first CTA into every CTA's copy
    float fval;
    int ival;
};

__device__ __forceinline__ uint32_t cluster_ctarank() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}
__device__ __forceinline__ void cluster_sync() {
    asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
template <typename T>
__device__ __forceinline__ uint32_t remote_addr(T *local, uint32_t rank) {
    uint32_t remote;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"(smem_u32(local)), "r"(rank));
    return remote;
}
__device__ __forceinline__ void st_remote_u64(unsigned long long *local, uint32_t rank, unsigned long long v) {
    asm volatile("st.shared::cluster.u64 [%0], %1;" ::"r"(remote_addr(local, rank)), "l"(v) : "memory");
}
__device__ __forceinline__ void st_remote_u32(unsigned *local, uint32_t rank, unsigned v) {
    asm volatile("st.shared::cluster.u32 [%0], %1;" ::"r"(remote_addr(local, rank)), "r"(v) : "memory");
}
// (No memory clobber: these loads follow a cluster barrier and are independent of one another, so that the
// compiler may keep all of a thread's loads in flight together: a round trip to another SM's shared memory
// is a few hundred nanoseconds.)
__device__ __forceinline__ unsigned ld_remote_u32(unsigned *local, uint32_t rank) {
    unsigned v;
    asm volatile("ld.shared::cluster.u32 %0, [%1];" : "=r"(v) : "r"(remote_addr(local, rank)));
    return v;
}

__device__ __forceinline__ float block_max(float v, SampleSmem &sm) {
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    if ((threadIdx.x & 31) == 0) sm.wred[threadIdx.x >> 5] = v;
    __syncthreads();
    if (threadIdx.x < 32) {
        float w = sm.wred[threadIdx.x];
        for (int o = 16; o > 0; o >>= 1) w = fmaxf(w, __shfl_xor_sync(0xffffffffu, w, o));
        if (threadIdx.x == 0) sm.fval = w;
    }
    __syncthreads();
    const float r = sm.fval;
    __syncthreads();
    return r;
}

__device__ __forceinline__ void hist_clear(SampleSmem &sm, int nb) {
    for (int b = threadIdx.x; b < nb; b += kSampleThreads) {
        sm.hlimb[0][b] = sm.hlimb[1][b] = sm.hlimb[2][b] = 0u;
        sm.hcnt[b] = 0u;
    }
}

// Adds one element to this CTA's histogram: four 32-bit shared-memory additions. (Grouping the lanes of a warp
// by bucket first, with __match_any_sync and __reduce_add_sync, was tried: the match costs several hundred
// instructions and the kernel spent its time resolving its branches.)
__device__ __forceinline__ void hist_add(SampleSmem &sm, int bucket, unsigned long long fx) {
    if (bucket < 0) return;
    atomicAdd(&sm.hlimb[0][bucket], unsigned(fx & 0x3FFFull));
    atomicAdd(&sm.hlimb[1][bucket], unsigned((fx >> 14) & 0x3FFFull));
    atomicAdd(&sm.hlimb[2][bucket], unsigned(fx >> 28));
    atomicAdd(&sm.hcnt[bucket], 1u);
}

// The first kKeep elements of a thread (element lo + rd * 1024 + tid for round rd) stay in registers after the
// exponential pass, so the later passes of a row of up to 131 072 tokens read nothing from memory.
__device__ void hist_pass(const float *e, const float (&kept)[kKeep], int lo, int hi, unsigned prefix, int known, int bits,
                          SampleSmem &sm) {
    const int nb = 1 << bits, shift = 31 - known - bits;
    hist_clear(sm, nb);
    __syncthreads();
    const int rounds = (hi - lo + kSampleThreads - 1) / kSampleThreads;
#pragma unroll
    for (int rd = 0; rd < kKeep; ++rd) {
        if (rd >= rounds) break;  // uniform over the CTA
        const int i = lo + rd * kSampleThreads + threadIdx.x;
        int bucket = -1;
        unsigned long long fx = 0ull;
        if (i < hi) {
            const float v = kept[rd];
            const unsigned key = __float_as_uint(v);
            if ((key >> (31 - known)) == prefix) {
                bucket = int((key >> shift) & unsigned(nb - 1));
                fx = to_fixed(v);
            }
        }
        hist_add(sm, bucket, fx);
    }
    for (int rd = kKeep; rd < rounds; ++rd) {
        const int i = lo + rd * kSampleThreads + threadIdx.x;
        int bucket = -1;
        unsigned long long fx = 0ull;
        if (i < hi) {
            const float v = e[i];
            const unsigned key = __float_as_uint(v);
            if ((key >> (31 - known)) == prefix) {
                bucket = int((key >> shift) & unsigned(nb - 1));
                fx = to_fixed(v);
            }
        }
        hist_add(sm, bucket, fx);
    }
    __syncthreads();
}

// First CTA only: scans a histogram (buckets from the top) for the bucket where `above + running sum` first
// exceeds `target`, and writes the result into every CTA's copy of `pick`. `merge`: add the eight CTAs'
// histograms on the fly (and keep the sums in g1 when `keep`); otherwise scan g1.
// `frac` >= 0 (first level only): the target is that fraction of the row's total mass, which this scan also finds.
__device__ void scan_and_publish(SampleSmem &sm, int bits, bool merge, bool keep, unsigned long long above,
                                 unsigned long long target, double frac) {
    const int tid = threadIdx.x, lane = tid & 31;
    const int nb = 1 << bits;
    const int per = (nb + kSampleThreads - 1) / kSampleThreads;  // 2 or 1
    unsigned long long s[2] = {0ull, 0ull};
    unsigned c[2] = {0u, 0u};
    for (int k = 0; k < per; ++k) {
        const int b = nb - 1 - (tid * per + k);
        if (b < 0) continue;
        if (merge) {
            unsigned t0[kCluster], t1[kCluster], t2[kCluster], tc[kCluster];
#pragma unroll
            for (uint32_t r = 0; r < kCluster; ++r) {
                t0[r] = ld_remote_u32(&sm.hlimb[0][b], r);
                t1[r] = ld_remote_u32(&sm.hlimb[1][b], r);
                t2[r] = ld_remote_u32(&sm.hlimb[2][b], r);
                tc[r] = ld_remote_u32(&sm.hcnt[b], r);
            }
#pragma unroll
            for (uint32_t r = 0; r < kCluster; ++r) {
                s[k] += static_cast<unsigned long long>(t0[r]) + (static_cast<unsigned long long>(t1[r]) << 14) +
                        (static_cast<unsigned long long>(t2[r]) << 28);
                c[k] += tc[r];
            }
            if (keep) {
                sm.g1sum[b] = s[k];
                sm.g1cnt[b] = c[k];
            }
        } else {
            s[k] = sm.g1sum[b];
            c[k] = sm.g1cnt[b];
        }
    }
    const unsigned long long mine = s[0] + s[1];
    unsigned long long incl = mine;
    for (int o = 1; o < 32; o <<= 1) {
        const unsigned long long up = __shfl_up_sync(0xffffffffu, incl, o);
        if (lane >= o) incl += up;
    }
    if (lane == 31) sm.wsum[tid >> 5] = incl;
    if (tid == 0) sm.ival = -1;
    __syncthreads();
    unsigned long long run = above + incl - mine;
    for (int w = 0; w < (tid >> 5); ++w) run += sm.wsum[w];
    unsigned long long total = above;
    for (int w = 0; w < kSampleWarps; ++w) total += sm.wsum[w];
    if (frac >= 0.0) target = static_cast<unsigned long long>(frac * static_cast<double>(total));
    Pick p = {0ull, 0ull, 0u, -1, total};
    bool found = false;
    for (int k = 0; k < per; ++k) {
        const int b = nb - 1 - (tid * per + k);
        if (b < 0) break;
        if (!found && run <= target && run + s[k] > target && c[k] > 0u) {  // exactly one bucket satisfies this
            p.above = run;
            p.bsum = s[k];
            p.bcnt = c[k];
            p.bucket = b;
            found = true;
        }
        run += s[k];
    }
    if (found) sm.ival = tid;
    __syncthreads();
    const int owner = sm.ival;
    if (owner < 0 && tid == 0) p.above = total;  // never exceeds the target: report the whole mass
    if (tid == (owner < 0 ? 0 : owner)) {
        for (uint32_t r = 0; r < kCluster; ++r) {
            st_remote_u64(&sm.pick.above, r, p.above);
            st_remote_u64(&sm.pick.bsum, r, p.bsum);
            st_remote_u32(&sm.pick.bcnt, r, p.bcnt);
            st_remote_u32(reinterpret_cast<unsigned *>(&sm.pick.bucket), r, unsigned(p.bucket));
            st_remote_u64(&sm.pick.total, r, p.total);
        }
    }
    __syncthreads();
}

struct Crossing {
    bool found;
    unsigned key;             // bit pattern of the element where the running sum crosses
    unsigned rank;            // its 1-based rank among the elements with that key, in index order
    unsigned long long mass;  // running sum up to and including it (found), or the whole mass (not found)
    unsigned long long total; // the row's whole mass (when the first level was scanned with a fraction)
};

// The whole descent for one target. `first_level_ready`: the merged first-level histogram is already in the
// first CTA's g1; otherwise this CTA's first-level histogram has just been built in hsum / hcnt. Every CTA
// of the cluster calls this with the same arguments.
// `frac` >= 0: the target is that fraction of the row's mass (known only after the first level's scan).
__device__ Crossing find_crossing(const float *e, const float (&kept)[kKeep], int lo, int hi, unsigned long long target, double frac,
                                  bool first_level_ready, uint32_t crank, SampleSmem &sm) {
    Crossing c = {false, 0u, 0u, 0ull, 0ull};
    const int level_bits[3] = {11, 11, 9};
    unsigned prefix = 0u;
    unsigned long long above = 0ull;
    int known = 0;
    Pick pk = {0ull, 0ull, 0u, -1};
    for (int lv = 0; lv < 3; ++lv) {
        const bool reuse = lv == 0 && first_level_ready;
        if (lv > 0) hist_pass(e, kept, lo, hi, prefix, known, level_bits[lv], sm);
        if (!reuse) cluster_sync();  // every CTA's histogram of this level is complete
        if (crank == 0) scan_and_publish(sm, level_bits[lv], !reuse, lv == 0, above, target, lv == 0 ? frac : -1.0);
        cluster_sync();  // the result is in every CTA's `pick`; the histograms may be cleared again
        pk = sm.pick;
        if (lv == 0) {
            c.total = pk.total;
            if (frac >= 0.0) target = static_cast<unsigned long long>(frac * static_cast<double>(pk.total));
        }
        if (pk.bucket < 0) {
            c.mass = pk.above;
            return c;
        }
        above = pk.above;
        prefix = (prefix << level_bits[lv]) | unsigned(pk.bucket);
        known += level_bits[lv];
    }
    // All elements of the last bucket share one key, hence one value: how many of them are needed.
    const unsigned long long each = pk.bsum / pk.bcnt;
    const unsigned long long need = target - above;  // above <= target < above + bsum
    unsigned rank = unsigned(need / each) + 1u;
    if (rank > pk.bcnt) rank = pk.bcnt;
    c.found = true;
    c.key = prefix;
    c.rank = rank;
    c.mass = above + each * rank;
    return c;
}

// One value per CTA (slices are in index order) into every CTA's `slots`; returns what comes before this CTA's.
__device__ unsigned long long cluster_exclusive(unsigned long long mine, unsigned long long *slots, uint32_t crank) {
    if (threadIdx.x < kCluster) st_remote_u64(&slots[crank], threadIdx.x, mine);
    cluster_sync();
    unsigned long long before = 0ull;
    for (uint32_t r = 0; r < crank; ++r) before += slots[r];
    return before;
}

__global__ void __launch_bounds__(kSampleThreads) sample_rows_kernel(float *logits, int vocab, const uint8_t *active,
                                                                     float temperature, float topp, const float *uniforms,
                                                                     const int32_t *greedy, int32_t *out) {
    extern __shared__ __align__(16) uint8_t sample_smem_raw[];
    SampleSmem &sm = *reinterpret_cast<SampleSmem *>(sample_smem_raw);
    const int row = blockIdx.y, tid = threadIdx.x, lane = tid & 31;
    const uint32_t crank = cluster_ctarank();
    if (active != nullptr && active[row] == 0) {  // the whole cluster leaves together
        if (tid == 0 && crank == 0) out[row] = -1;
        return;
    }
    float *e = logits + size_t(row) * vocab;
    const int n = vocab;
    const int per_cta = ((n + kCluster - 1) / kCluster + 3) & ~3;
    const int lo = min(n, int(crank) * per_cta), hi = min(n, lo + per_cta);
    // scores / temperature and their maximum over the row: the step's arg-max kernel has already found where
    // the maximum sits (greedy may alias out: it is read here, out is written at the very end)
    float mx;
    if (greedy != nullptr) {
        mx = __fdiv_rn(e[greedy[row]], temperature);
        cluster_sync();  // everybody has read it before anybody overwrites the row below
    } else {
        mx = -INFINITY;
        for (int i = lo + tid; i < hi; i += kSampleThreads) mx = fmaxf(mx, __fdiv_rn(e[i], temperature));
        mx = block_max(mx, sm);
        if (tid < kCluster)
            asm volatile("st.shared::cluster.f32 [%0], %1;" ::"r"(remote_addr(&sm.cmax[crank], uint32_t(tid))), "f"(mx) : "memory");
        cluster_sync();
        mx = sm.cmax[0];
        for (int r = 1; r < kCluster; ++r) mx = fmaxf(mx, sm.cmax[r]);
    }
    // e = exp(score - max) in place, and (for the nucleus sampler) this CTA's first-level histogram of it in the same pass
    const bool nucleus_mode = topp > 0.0f && topp < 1.0f;
    hist_clear(sm, kBuckets);
    __syncthreads();
    float kept[kKeep];
    {
        const int rounds = (hi - lo + kSampleThreads - 1) / kSampleThreads;
        float raw[kKeep];
#pragma unroll
        for (int rd = 0; rd < kKeep; ++rd) {  // all of a thread's loads in flight together
            const int i = lo + rd * kSampleThreads + tid;
            raw[rd] = (rd < rounds && i < hi) ? e[i] : 0.f;
        }
#pragma unroll
        for (int rd = 0; rd < kKeep; ++rd) {
            kept[rd] = 0.f;
            if (rd >= rounds) continue;  // uniform over the CTA
            const int i = lo + rd * kSampleThreads + tid;
            int bucket = -1;
            unsigned long long fx = 0ull;
            if (i < hi) {
                const float v = expf(__fsub_rn(__fdiv_rn(raw[rd], temperature), mx));
                e[i] = v;
                kept[rd] = v;
                bucket = nucleus_mode ? int(__float_as_uint(v) >> 20) : -1;
                fx = to_fixed(v);
            }
            hist_add(sm, bucket, fx);
        }
        for (int rd = kKeep; rd < rounds; ++rd) {
            const int i = lo + rd * kSampleThreads + tid;
            int bucket = -1;
            unsigned long long fx = 0ull;
            if (i < hi) {
                const float v = expf(__fsub_rn(__fdiv_rn(e[i], temperature), mx));
                e[i] = v;
                bucket = nucleus_mode ? int(__float_as_uint(v) >> 20) : -1;
                fx = to_fixed(v);
            }
            hist_add(sm, bucket, fx);
        }
    }
    __syncthreads();
    const float u = uniforms[row];
    if (!nucleus_mode) {
        // CategoricalSampler: first index whose running sum (index order) exceeds u * sum.
        const int chunk = (hi - lo + kSampleThreads - 1) / kSampleThreads;
        const int tlo = min(hi, lo + tid * chunk), thi = min(hi, tlo + chunk);
        unsigned long long mine = 0ull;
        for (int i = tlo; i < thi; ++i) mine += to_fixed(e[i]);
        unsigned long long incl = mine;
        for (int o = 1; o < 32; o <<= 1) {
            const unsigned long long up = __shfl_up_sync(0xffffffffu, incl, o);
            if (lane >= o) incl += up;
        }
        if (lane == 31) sm.wsum[tid >> 5] = incl;
        __syncthreads();
        unsigned long long cta_total = 0ull;
        for (int w = 0; w < kSampleWarps; ++w) cta_total += sm.wsum[w];
        unsigned long long before = cluster_exclusive(cta_total, sm.csum, crank);
        unsigned long long total = 0ull;
        for (int r = 0; r < kCluster; ++r) total += sm.csum[r];
        const unsigned long long target =
            static_cast<unsigned long long>(static_cast<double>(u) * static_cast<double>(total));  // cdf > u  <=>  running e > u * sum
        for (int w = 0; w < (tid >> 5); ++w) before += sm.wsum[w];
        before += incl - mine;
        if (before <= target && before + mine > target) {
            unsigned long long run = before;
            for (int i = tlo; i < thi; ++i) {
                run += to_fixed(e[i]);
                if (run > target) {
                    out[row] = i;
                    break;
                }
            }
        }
        if (crank == kCluster - 1 && tid == kSampleThreads - 1 && target >= total) out[row] = n - 1;  // CategoricalSampler.java:24
        cluster_sync();  // nobody leaves while its shared memory may still be written
        return;
    }
    // ToppSampler. Stage 1: where the running sum, largest first, exceeds topp * sum (the first scan also yields the
    // sum and leaves the merged first-level histogram with the first CTA).
    const Crossing nucleus = find_crossing(e, kept, lo, hi, 0ull, static_cast<double>(topp), false, crank, sm);
    const unsigned long long total = nucleus.total;
    // Stage 2: r = u * (that running sum as a probability), ToppSampler.java:92, and where the running sum exceeds it.
    const float mass_p = static_cast<float>(static_cast<double>(nucleus.mass) / static_cast<double>(total));
    const float r = __fmul_rn(u, mass_p);
    unsigned long long t2 = static_cast<unsigned long long>(static_cast<double>(r) * static_cast<double>(total));
    if (nucleus.mass > 0ull && t2 >= nucleus.mass) t2 = nucleus.mass - 1ull;  // u * mass rounded up to the mass: its last element
    const Crossing pick = find_crossing(e, kept, lo, hi, t2, -1.0, true, crank, sm);
    const Crossing use = pick.found ? pick : nucleus;
    if (use.found) {
        // The rank-th element (index order) with exactly this key.
        const int chunk = (hi - lo + kSampleThreads - 1) / kSampleThreads;
        const int tlo = min(hi, lo + tid * chunk), thi = min(hi, tlo + chunk);
        unsigned mine = 0u;
        for (int i = tlo; i < thi; ++i) mine += (__float_as_uint(e[i]) == use.key) ? 1u : 0u;
        unsigned incl = mine;
        for (int o = 1; o < 32; o <<= 1) {
            const unsigned up = __shfl_up_sync(0xffffffffu, incl, o);
            if (lane >= o) incl += up;
        }
        if (lane == 31) sm.wcnt[tid >> 5] = incl;
        __syncthreads();
        unsigned cta_total = 0u;
        for (int w = 0; w < kSampleWarps; ++w) cta_total += sm.wcnt[w];
        unsigned before = unsigned(cluster_exclusive(cta_total, sm.ccnt, crank));
        for (int w = 0; w < (tid >> 5); ++w) before += sm.wcnt[w];
        before += incl - mine;
        if (before < use.rank && use.rank <= before + mine) {
            unsigned seen = before;
            for (int i = tlo; i < thi; ++i)
                if (__float_as_uint(e[i]) == use.key && ++seen == use.rank) {
                    out[row] = i;
                    break;
                }
        }
    } else if (crank == 0 && tid == 0) {
        out[row] = 0;  // cannot happen (the maximum itself has e = 1); keeps the output defined
    }
    cluster_sync();  // nobody leaves while its shared memory may still be read or written
}

}  // namespace

cudaError_t sample_rows_configure() {
    return cudaFuncSetAttribute(sample_rows_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, int(sizeof(SampleSmem)));
}

cudaError_t sample_rows_launch(float *logits, int vocab, int width, const uint8_t *active, float temperature, float topp,
                               const float *uniforms, const int32_t *greedy, int32_t *out, cudaStream_t stream) {
    if (logits == nullptr || uniforms == nullptr || out == nullptr || vocab < 2 || width < 1 || !(temperature > 0.0f))
        return cudaErrorInvalidValue;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(kCluster, unsigned(width));
    cfg.blockDim = dim3(kSampleThreads);
    cfg.dynamicSmemBytes = sizeof(SampleSmem);
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = kCluster;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    return cudaLaunchKernelEx(&cfg, sample_rows_kernel, logits, vocab, active, temperature, topp, uniforms, greedy, out);
}

}  // namespace jl
