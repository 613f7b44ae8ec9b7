// Per-layer kernels around the matrix products (see ops.cuh).
#include "ops.cuh"

#include <cuda_fp16.h>

namespace jl {

JL_TRACE_DEFINE_BIND(ops_trace_bind)

namespace {

// ---- embedding -------------------------------------------------------------------------------
__global__ void embedding_kernel(int type, const uint8_t *table, const int32_t *tokens,
                                 const uint8_t *active, float *x, int dim) {
    const int row = blockIdx.y;
    const bool on = active == nullptr || active[row] != 0;
    pdl_wait();
    pdl_launch_dependents();
    if (!on) return;
    const int token = tokens[row];
    for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < dim; i += gridDim.x * blockDim.x)
        x[size_t(row) * dim + i] = decode_any(type, table, int64_t(token) * dim + i);
}

// ---- dequant ---------------------------------------------------------------------------------
__global__ void dequant_kernel(int type, const uint8_t *blocks, int64_t n, float *out) {
    const int64_t stride = int64_t(gridDim.x) * blockDim.x;
    for (int64_t i = int64_t(blockIdx.x) * blockDim.x + threadIdx.x; i < n; i += stride)
        out[i] = decode_any(type, blocks, i);
}

// Q6_K super-blocks (210 bytes) copied into slots of kQ6_KPadded bytes, the tail zeroed: the layout the tensor-core
// kernel's 2-D tensor map needs (rows that are 16-byte multiples). 16-bit pieces: the source is 2-byte aligned.
__global__ void pad_q6k_kernel(const uint8_t *src, uint8_t *dst, size_t nblocks) {
    constexpr int kHalfWords = kQ6_KPadded / 2;
    const size_t total = nblocks * kHalfWords, stride = size_t(gridDim.x) * blockDim.x;
    for (size_t i = size_t(blockIdx.x) * blockDim.x + threadIdx.x; i < total; i += stride) {
        const size_t blk = i / kHalfWords;
        const int w = int(i - blk * kHalfWords);
        const unsigned short v = w < kQ6_KBytes / 2 ? reinterpret_cast<const unsigned short *>(src + blk * kQ6_KBytes)[w] : 0;
        reinterpret_cast<unsigned short *>(dst + blk * kQ6_KPadded)[w] = v;
    }
}

__global__ void fill_kernel(uint32_t *buf, size_t words, uint32_t value) {
    const size_t stride = size_t(gridDim.x) * blockDim.x;
    for (size_t i = size_t(blockIdx.x) * blockDim.x + threadIdx.x; i < words; i += stride)
        buf[i] = value;
}

__global__ void advance_kernel(int32_t *tokens, int32_t *positions, const int32_t *sampled,
                               const uint8_t *active, int32_t *history, int32_t *step_counter,
                               int width) {
    pdl_wait();
    pdl_launch_dependents();
    const int b = threadIdx.x;
    const int step = *step_counter;
    __syncthreads();
    if (b < width) {
        const bool on = active[b] != 0;
        const int32_t tok = on ? sampled[b] : -1;
        history[size_t(step) * width + b] = tok;
        if (on) {
            tokens[b] = tok;
            positions[b] += 1;
        }
    }
    if (b == 0) *step_counter = step + 1;
}

__device__ __forceinline__ int64_t kv_offset(const KvGeom &g, int slot, int pos, int layer) {
    const int blk = pos / g.block_tokens;
    const int within = pos - blk * g.block_tokens;
    const int64_t phys = g.block_table[int64_t(slot) * g.blocks_per_slot + blk];
    const int64_t block_stride = int64_t(g.layers) * g.block_tokens * g.kv_dim;
    return phys * block_stride + int64_t(layer) * g.block_tokens * g.kv_dim +
           int64_t(within) * g.kv_dim;
}

// The row kernels below take part in chains of programmatic dependent launches: each lets the next
// kernel start its preamble at once (a matrix-matrix kernel then streams its first weights while this
// one runs) and waits for the kernel before it. Every CTA waits, also one that then has nothing to do:
// a grid whose CTAs left without waiting would count as complete while its predecessor still runs,
// and the next kernel's wait covers only its own predecessor. The embedding and the advance kernel
// wait before they release: whatever starts after them may read the step's positions at once.
__global__ void add_rows_kernel(float *x, const float *y, size_t total) {
    pdl_launch_dependents();
    pdl_wait();
    const size_t stride = size_t(gridDim.x) * blockDim.x;
    for (size_t i = size_t(blockIdx.x) * blockDim.x + threadIdx.x; i < total; i += stride) x[i] = x[i] + y[i];
}

// Four consecutive activations as binary16 hi and lo parts (x = hi + lo), the tensor-core path's
// activation format. Inside each group of four the pairs are (x0, x2) and (x1, x3): the weight
// conversion gets the nibbles of bytes 0 and 2 of a word with one logic operation, and a sum over K
// does not care about the order as long as both operands use the same one.
__device__ __forceinline__ void split4_store(const float4 v, uint2 *hi, uint2 *lo) {
    const __half2 h0 = __floats2half2_rn(v.x, v.z), h1 = __floats2half2_rn(v.y, v.w);
    const float2 b0 = __half22float2(h0), b1 = __half22float2(h1);
    const __half2 l0 = __floats2half2_rn(v.x - b0.x, v.z - b0.y), l1 = __floats2half2_rn(v.y - b1.x, v.w - b1.y);
    *hi = make_uint2(*reinterpret_cast<const uint32_t *>(&h0), *reinterpret_cast<const uint32_t *>(&h1));
    *lo = make_uint2(*reinterpret_cast<const uint32_t *>(&l0), *reinterpret_cast<const uint32_t *>(&l1));
}

__global__ void split_rows_kernel(const float4 *x, size_t total4, uint2 *hi, uint2 *lo) {
    pdl_launch_dependents();
    pdl_wait();
    const size_t stride = size_t(gridDim.x) * blockDim.x;
    for (size_t i = size_t(blockIdx.x) * blockDim.x + threadIdx.x; i < total4; i += stride) {
        split4_store(x[i], hi + i, lo + i);
    }
}

__global__ void tp_pack_best_kernel(const float *logits, const int32_t *idx, int l_vocab, int index_offset, int n,
                                    float *best) {
    const int r = blockIdx.x * blockDim.x + threadIdx.x;
    if (r >= n) return;
    const int i = idx[r];
    best[2 * r] = logits[size_t(r) * l_vocab + i];
    best[2 * r + 1] = static_cast<float>(i + index_offset);  // vocabulary indices are exact in fp32
}

__global__ void tp_pick_best_kernel(const float *all, int ranks, int n, const uint8_t *active, int32_t *out) {
    const int r = blockIdx.x * blockDim.x + threadIdx.x;
    if (r >= n || (active != nullptr && active[r] == 0)) return;
    float bv = -INFINITY;
    int bi = 0x7fffffff;
    for (int k = 0; k < ranks; ++k) {
        const float v = all[(size_t(k) * n + r) * 2];
        const int i = static_cast<int>(all[(size_t(k) * n + r) * 2 + 1]);
        if (v > bv || (v == bv && i < bi)) {
            bv = v;
            bi = i;
        }
    }
    out[r] = bi == 0x7fffffff ? 0 : bi;
}

// ---- row-wise operators for the matrix-matrix path ---------------------------------------------
// One CTA per row. The row is read once, as float4 batches held in registers (all loads issued
// before the first use: one L2 round trip, not one per element), and the same registers feed the
// output pass. Optionally also writes the row as binary16 hi / lo parts (x = hi + lo), the
// activation format of the tensor-core path.
constexpr int kNormThreads = 256;
constexpr int kNormBatch = 8;  // float4 per thread per batch: rows up to 8192 in one batch

__global__ void __launch_bounds__(kNormThreads) rmsnorm_rows_kernel(const float *x, const float *w, float eps, float *out,
                                                                    int dim, const uint8_t *active, uint2 *hi, uint2 *lo) {
    const int row = blockIdx.x;
    const int trace = trace_begin(kTraceRows);
    trace_word(trace, 7, 1);
    pdl_launch_dependents();
    pdl_wait();
    if (active != nullptr && active[row] == 0) return;
    __shared__ float part[9];
    const int n4 = dim / 4;
    const float4 *xr = reinterpret_cast<const float4 *>(x + size_t(row) * dim);
    const float4 *w4 = reinterpret_cast<const float4 *>(w);
    float4 v[kNormBatch];
#pragma unroll
    for (int k = 0; k < kNormBatch; ++k) {
        const int i = k * kNormThreads + threadIdx.x;
        v[k] = i < n4 ? xr[i] : make_float4(0.f, 0.f, 0.f, 0.f);
    }
    float s = 0.f;
#pragma unroll
    for (int k = 0; k < kNormBatch; ++k) s += v[k].x * v[k].x + v[k].y * v[k].y + v[k].z * v[k].z + v[k].w * v[k].w;
    for (int i = kNormBatch * kNormThreads + threadIdx.x; i < n4; i += kNormThreads) {
        const float4 u = xr[i];
        s += u.x * u.x + u.y * u.y + u.z * u.z + u.w * u.w;
    }
    s = warp_sum(s);
    if ((threadIdx.x & 31) == 0) part[threadIdx.x >> 5] = s;
    __syncthreads();
    if (threadIdx.x == 0) {
        float tot = 0.f;
        for (int i = 0; i < kNormThreads / 32; ++i) tot += part[i];
        float ms = tot / static_cast<float>(dim);
        ms += eps;
        part[8] = static_cast<float>(1.0 / sqrt(static_cast<double>(ms)));
    }
    __syncthreads();
    const float ss = part[8];
    float4 *o4 = reinterpret_cast<float4 *>(out + size_t(row) * dim);
    uint2 *hr = hi != nullptr ? hi + size_t(row) * n4 : nullptr;
    uint2 *lr = lo != nullptr ? lo + size_t(row) * n4 : nullptr;
    auto emit = [&](int i, float4 u) {
        const float4 g = w4[i];
        float4 r;
        r.x = __fmul_rn(g.x, __fmul_rn(ss, u.x));
        r.y = __fmul_rn(g.y, __fmul_rn(ss, u.y));
        r.z = __fmul_rn(g.z, __fmul_rn(ss, u.z));
        r.w = __fmul_rn(g.w, __fmul_rn(ss, u.w));
        o4[i] = r;
        if (hr != nullptr) split4_store(r, hr + i, lr + i);
    };
#pragma unroll
    for (int k = 0; k < kNormBatch; ++k) {
        const int i = k * kNormThreads + threadIdx.x;
        if (i < n4) emit(i, v[k]);
    }
    for (int i = kNormBatch * kNormThreads + threadIdx.x; i < n4; i += kNormThreads) emit(i, xr[i]);
}

// Four elements per thread per step (row lengths are multiples of 256, so float4 never straddles).
__global__ void swiglu_rows_kernel(float4 *g, const float4 *u, size_t total4, uint2 *hi, uint2 *lo) {
    const int trace = trace_begin(kTraceRows);
    trace_word(trace, 7, 2);
    pdl_launch_dependents();
    pdl_wait();
    const size_t stride = size_t(gridDim.x) * blockDim.x;
    for (size_t i = size_t(blockIdx.x) * blockDim.x + threadIdx.x; i < total4; i += stride) {
        const float4 v = g[i], w = u[i];
        float4 r;
        r.x = (v.x / (1.0f + expf(-v.x))) * w.x;
        r.y = (v.y / (1.0f + expf(-v.y))) * w.y;
        r.z = (v.z / (1.0f + expf(-v.z))) * w.z;
        r.w = (v.w / (1.0f + expf(-v.w))) * w.w;
        g[i] = r;
        if (hi != nullptr) split4_store(r, hi + i, lo + i);
    }
}

__global__ void kv_append_kernel(const float *k, const float *v, const float *rope_cos, const float *rope_sin,
                                 const int32_t *positions, const int32_t *slots, const uint8_t *active,
                                 KvGeom kv, int layer, int head_dim) {
    const int row = blockIdx.x;
    pdl_launch_dependents();
    pdl_wait();
    if (active != nullptr && active[row] == 0) return;
    const int pos = positions[row], slot = slots[row];
    const int64_t off = kv_offset(kv, slot, pos, layer);
    const float *kr = k + size_t(row) * kv.kv_dim, *vr = v + size_t(row) * kv.kv_dim;
    const int half = head_dim / 2;
    for (int p = threadIdx.x; p < kv.kv_dim / 2; p += blockDim.x) {
        const int i = p % half;
        const float cr = rope_cos[size_t(pos) * half + i], ci = rope_sin[size_t(pos) * half + i];
        const float v0 = kr[2 * p], v1 = kr[2 * p + 1];
        kv.kpool[off + 2 * p] = __float2half_rn(__fsub_rn(__fmul_rn(v0, cr), __fmul_rn(v1, ci)));
        kv.kpool[off + 2 * p + 1] = __float2half_rn(__fadd_rn(__fmul_rn(v0, ci), __fmul_rn(v1, cr)));
        kv.vpool[off + 2 * p] = __float2half_rn(vr[2 * p]);
        kv.vpool[off + 2 * p + 1] = __float2half_rn(vr[2 * p + 1]);
    }
}

__global__ void argmax_rows_kernel(const float *logits, int vocab, const uint8_t *active, int32_t *out) {
    const int row = blockIdx.x;
    pdl_launch_dependents();
    pdl_wait();
    if (active != nullptr && active[row] == 0) return;
    const float *lr = logits + size_t(row) * vocab;
    float bv = -INFINITY;
    int bi = 0x7fffffff;
    for (int i = threadIdx.x; i < vocab; i += blockDim.x) {
        const float v = lr[i];
        if (v > bv) {  // strided scan visits indices in increasing order per thread
            bv = v;
            bi = i;
        }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
        const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
        if (ov > bv || (ov == bv && oi < bi)) {
            bv = ov;
            bi = oi;
        }
    }
    __shared__ float sv[32];
    __shared__ int si[32];
    if ((threadIdx.x & 31) == 0) {
        sv[threadIdx.x >> 5] = bv;
        si[threadIdx.x >> 5] = bi;
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        for (int w = 1; w < int(blockDim.x >> 5); ++w)
            if (sv[w] > bv || (sv[w] == bv && si[w] < bi)) {
                bv = sv[w];
                bi = si[w];
            }
        out[row] = bi == 0x7fffffff ? 0 : bi;
    }
}

// ---- RoPE + KV append + paged decode attention -------------------------------------------------

// Sixteen warps per CTA (eight when the G query heads of a KV head hold more state per thread than
// 512 threads leave registers for). A warp takes eight keys per iteration: four lanes share a key for the
// q.k products (each lane a quarter of the head dimension), while for the p.v sums every lane owns
// head_dim / 32 output dimensions of all eight keys.
// Wide launches (many rows) use eight warps as well: two or three CTAs then share an SM and the whole
// grid is resident at once.
template <int HD, int G, bool WIDE = false>
struct AttnShape {
    static constexpr int threads = (WIDE || G * HD > 512) ? 256 : 512;
    static constexpr int warps = threads / 32;
    static constexpr int keys = 8;
    static constexpr int dk = HD / 4;       // dimensions of a key one lane multiplies
    static constexpr int qpad = dk + 4;     // quarter stride of q in shared memory: no bank conflicts
};
constexpr int kAttnMaxCluster = 8;      // CTAs of one cluster share a (row, KV head) and fold through shared memory
constexpr int kAttnMaxFold = 8;         // clusters per (row, KV head) at most: their fold goes through global memory
constexpr int kAttnKeysPerCluster = 1024;  // short contexts use one cluster, so nothing crosses global memory
constexpr int kAttnPages = 264;         // page bases kept in shared memory (4096 keys of 16-token pages, and margin)

__device__ __forceinline__ uint32_t cluster_rank() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}
// Clusters actually used for n keys: short contexts use one, so that the fold stays on chip; the
// launch grid is sized for the maximum and surplus clusters leave at once.
__device__ __forceinline__ int clusters_for(int n, int ncl_max) {
    return max(1, min(ncl_max, (n + kAttnKeysPerCluster - 1) / kAttnKeysPerCluster));
}

__device__ __forceinline__ void st_cluster_f32(float *local, uint32_t rank, float v) {
    uint32_t remote;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"(smem_u32(local)), "r"(rank));
    asm volatile("st.shared::cluster.f32 [%0], %1;" ::"r"(remote), "f"(v) : "memory");
}

template <int HD, int G, bool WIDE>
struct AttnSmem {
    float q[G][4][AttnShape<HD, G, WIDE>::qpad];
    float red[AttnShape<HD, G, WIDE>::warps][G][HD + 2];
    float part[kAttnMaxCluster][G][HD + 2];  // in the cluster's first CTA: every CTA's result
    float wgt[G][kAttnMaxFold];
    float inv_l[G];
    float rope[2][HD / 2];    // cos and sin of this row's position
    alignas(16) uint32_t knew[HD / 2];    // the new key, rotated and rounded: binary16 pairs as they go to the page
    alignas(16) uint32_t vnew[HD / 2];    // the new value, rounded
    long long page_base[kAttnPages];
    int is_last;
};

// One CTA = (split of the position range, KV head, batch row); `csize` consecutive splits form a
// thread-block cluster. The G query heads that share the KV head are processed together so each
// K/V row is read once. What it computes is CpuOperations.rope + appendKeyValue + attention
// (inference/op/CpuOperations.java:94-204) with the softmax evaluated online; K and V are rounded
// to binary16 on append exactly as ArrayHalfFloatTensor.setFloat does
// (tensor/standard/ArrayHalfFloatTensor.java:33-40).
//
// Decode launches (a.append != 0: every row is its own sequence and position pos is the only key
// this step adds) read everything that no kernel of this step writes -- position, slot, block
// table, RoPE row and the first batch of old K/V rows -- before waiting for the kernel that
// produces q, k and v, so that memory latency overlaps that kernel's tail. The new key never
// comes back from the pool: the warp that appends it uses the rounded values it just wrote.
// positions[] and slots[] are written by the host before the step or by advance_kernel, and the
// kernel that follows advance_kernel releases its dependents only after it has itself waited, so
// no kernel of a step starts before advance_kernel has completed.
//
// Folding: the warps of a CTA fold in its shared memory; the CTAs of a cluster store their results
// into the shared memory of the cluster's first CTA, which folds them; only when a context is long
// enough to use several clusters do their results meet in global memory, where the last cluster
// to arrive folds them.
// One attention output element, and its binary16 hi / lo parts at the element's place in the tensor-core
// path's operand order when the launch asks for them.
__device__ __forceinline__ void attn_store(const AttnArgs &a, size_t row, int k, float v) {
    a.out[row * a.dim + k] = v;
    if (a.out_hi != nullptr) {
        const int p = (k & ~3) | ((k & 1) << 1) | ((k >> 1) & 1);
        const __half h = __float2half_rn(v);
        static_cast<__half *>(a.out_hi)[row * a.dim + p] = h;
        static_cast<__half *>(a.out_lo)[row * a.dim + p] = __float2half_rn(v - __half2float(h));
    }
}

template <int HD, int G, bool WIDE>
__global__ void __launch_bounds__(AttnShape<HD, G, WIDE>::threads, WIDE ? 2 : 1)
    attn_decode_kernel(const AttnArgs a, const int csize) {
    constexpr int VEC = HD / 32;
    constexpr int UN = AttnShape<HD, G, WIDE>::keys;
    constexpr int kAttnThreads = AttnShape<HD, G, WIDE>::threads, kAttnWarps = AttnShape<HD, G, WIDE>::warps;
    extern __shared__ __align__(16) uint8_t attn_smem_raw[];
    AttnSmem<HD, G, WIDE> &sm = *reinterpret_cast<AttnSmem<HD, G, WIDE> *>(attn_smem_raw);
    const int split = blockIdx.x, kvh = blockIdx.y, b = blockIdx.z;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int trace = trace_begin(kTraceAttn);
    pdl_launch_dependents();
    const bool on = a.active == nullptr || a.active[b] != 0;
    const bool dec = a.append != 0;
    int pos = 0, slot = 0;
    if (on && dec) {
        pos = a.positions[b];
        slot = a.slots[b];
    }
    if (!dec) {
        pdl_wait();
        if (on) {
            pos = a.positions[b];
            slot = a.slots[b];
        }
    }
    const int n_old = dec ? pos : pos + 1;  // keys that come from the pool
    const int ncl_max = a.nsplit / csize;
    const int ncl = clusters_for(max(n_old, 1), ncl_max);
    const int cl = split / csize;
    if (!on || cl >= ncl) {  // whole clusters leave; still in step with the chain of launches
        if (dec) pdl_wait();
        return;
    }
    const int nsplit = ncl * csize;
    const uint32_t crank = csize > 1 ? cluster_rank() : 0u;
    // First half of a cluster barrier whose second half sits just before the stores into the first
    // CTA's shared memory: that CTA must have started before anybody writes there.
    if (csize > 1) asm volatile("barrier.cluster.arrive.relaxed.aligned;" ::: "memory");

    const int chunk = (n_old + nsplit - 1) / nsplit;
    const int start = min(n_old, split * chunk);
    const int end = min(n_old, start + chunk);
    // Page bases of this CTA's key range.
    const int bt = a.kv.block_tokens;
    const int first_page = start / bt;
    const int npages = end > start ? (end - 1) / bt - first_page + 1 : 0;
    const int64_t block_stride = int64_t(a.kv.layers) * bt * a.kv.kv_dim;
    for (int pg = tid; pg < npages && pg < kAttnPages; pg += kAttnThreads) {
        const int64_t phys = a.kv.block_table[int64_t(slot) * a.kv.blocks_per_slot + first_page + pg];
        sm.page_base[pg] = phys * block_stride + int64_t(a.layer) * bt * a.kv.kv_dim + int64_t(kvh) * HD;
    }
    // The RoPE row of this position (the tables never change) goes to shared memory now, so that
    // nothing after the wait below has to fetch it.
    for (int i = tid; i < HD; i += kAttnThreads)
        sm.rope[i / (HD / 2)][i % (HD / 2)] = (i < HD / 2 ? a.rope_cos : a.rope_sin)[size_t(pos) * (HD / 2) + i % (HD / 2)];
    __syncthreads();
    // Each warp takes a contiguous run of keys so that consecutive keys share a page. The new key
    // of a decode launch goes to the last warp of the first CTA, behind that warp's old keys.
    constexpr int DK = AttnShape<HD, G, WIDE>::dk;
    const int per_warp = (end - start + kAttnWarps - 1) / kAttnWarps;
    const int w0 = min(end, start + warp * per_warp);
    const int w1 = min(end, w0 + per_warp);
    const int extra = (dec && split == 0 && warp == kAttnWarps - 1) ? 1 : 0;
    const int ku = lane >> 2, qd = lane & 3;  // this lane's key of the batch and quarter of its dimensions
    auto key_base = [&](int t) -> int64_t {
        const int pg = t / bt - first_page;
        const int64_t base = (pg < kAttnPages) ? int64_t(sm.page_base[pg])
                                               : kv_offset(a.kv, slot, t, a.layer) - int64_t(t % bt) * a.kv.kv_dim + int64_t(kvh) * HD;
        return base + int64_t(t % bt) * a.kv.kv_dim;
    };
    uint4 kq[DK / 8];    // this lane's quarter of its key, as stored (binary16)
    uint32_t vq[UN][VEC / 2];  // this lane's output dimensions of the batch's eight values
    auto load_batch = [&](int t0) {
        if (t0 + ku < w1) {
            const uint4 *kp = reinterpret_cast<const uint4 *>(a.kv.kpool + key_base(t0 + ku) + qd * DK);
#pragma unroll
            for (int i = 0; i < DK / 8; ++i) kq[i] = kp[i];
        } else {
#pragma unroll
            for (int i = 0; i < DK / 8; ++i) kq[i] = make_uint4(0u, 0u, 0u, 0u);
        }
#pragma unroll
        for (int u = 0; u < UN; ++u) {
            if (t0 + u < w1) {
                const uint32_t *vp = reinterpret_cast<const uint32_t *>(a.kv.vpool + key_base(t0 + u) + lane * VEC);
#pragma unroll
                for (int j = 0; j < VEC / 2; ++j) vq[u][j] = vp[j];
            } else {
#pragma unroll
                for (int j = 0; j < VEC / 2; ++j) vq[u][j] = 0u;
            }
        }
    };
    const float *cr = sm.rope[0], *ci = sm.rope[1];
    if (dec) {
        load_batch(w0);
        pdl_wait();
    }
    trace_mark(trace, 2);
    trace_word(trace, 6, trace_latest_exit());
    for (int idx = tid; idx < G * (HD / 2); idx += kAttnThreads) {
        const int g = idx / (HD / 2), i = idx - g * (HD / 2);
        const float *qh = a.q + size_t(b) * a.dim + size_t(kvh * G + g) * HD;
        const float v0 = qh[2 * i], v1 = qh[2 * i + 1];
        const int d0 = 2 * i;
        sm.q[g][d0 / DK][d0 % DK] = __fsub_rn(__fmul_rn(v0, cr[i]), __fmul_rn(v1, ci[i]));
        sm.q[g][d0 / DK][d0 % DK + 1] = __fadd_rn(__fmul_rn(v0, ci[i]), __fmul_rn(v1, cr[i]));
    }
    if (dec && split == 0) {
        // The new key of this step: rotate k, round k and v to fp16 as the append does, write them to
        // the page and keep the rounded pairs in shared memory for the warp that attends to them. The
        // threads that do this are the upper ones, so that it runs beside the staging of q above.
        const int64_t off = kv_offset(a.kv, slot, pos, a.layer) + int64_t(kvh) * HD;
        const float *kh = a.k + size_t(b) * a.kv.kv_dim + size_t(kvh) * HD;
        const float *vh = a.v + size_t(b) * a.kv.kv_dim + size_t(kvh) * HD;
        for (int idx = kAttnThreads - 1 - tid; idx < HD; idx += kAttnThreads) {
            const int i = idx % (HD / 2);
            __half2 h;
            if (idx < HD / 2) {
                const float v0 = kh[2 * i], v1 = kh[2 * i + 1];
                h = __halves2half2(__float2half_rn(__fsub_rn(__fmul_rn(v0, cr[i]), __fmul_rn(v1, ci[i]))),
                                   __float2half_rn(__fadd_rn(__fmul_rn(v0, ci[i]), __fmul_rn(v1, cr[i]))));
                sm.knew[i] = *reinterpret_cast<const uint32_t *>(&h);
                *reinterpret_cast<__half2 *>(a.kv.kpool + off + 2 * i) = h;
            } else {
                h = __halves2half2(__float2half_rn(vh[2 * i]), __float2half_rn(vh[2 * i + 1]));
                sm.vnew[i] = *reinterpret_cast<const uint32_t *>(&h);
                *reinterpret_cast<__half2 *>(a.kv.vpool + off + 2 * i) = h;
            }
        }
    }
    __syncthreads();
    trace_mark(trace, 3);

    float m[G], l[G], acc[G][VEC];
#pragma unroll
    for (int g = 0; g < G; ++g) {
        m[g] = -INFINITY;
        l[g] = 0.f;
#pragma unroll
        for (int j = 0; j < VEC; ++j) acc[g][j] = 0.f;
    }
    const float inv_sqrt = 1.0f / sqrtf(static_cast<float>(HD));
    const int w1x = w1 + extra;
    for (int t0 = w0; t0 < w1x; t0 += UN) {
        if (!(dec && t0 == w0)) load_batch(t0);
        if (extra && w1 - t0 < UN && w1 >= t0) {
            // The new key sits in this batch: its rounded pairs are in shared memory.
            if (ku == w1 - t0) {
#pragma unroll
                for (int i = 0; i < DK / 8; ++i)
                    kq[i] = *reinterpret_cast<const uint4 *>(&sm.knew[qd * (DK / 2) + 4 * i]);
            }
#pragma unroll
            for (int u = 0; u < UN; ++u)
                if (t0 + u == w1) {
#pragma unroll
                    for (int j = 0; j < VEC / 2; ++j) vq[u][j] = sm.vnew[lane * (VEC / 2) + j];
                }
        }
        // q.k: this lane's quarter of its key against the same quarter of every query head.
        float s[G];
#pragma unroll
        for (int g = 0; g < G; ++g) s[g] = 0.f;
#pragma unroll
        for (int i = 0; i < DK / 8; ++i) {
            const uint32_t w[4] = {kq[i].x, kq[i].y, kq[i].z, kq[i].w};
            float kf[8];
#pragma unroll
            for (int h = 0; h < 4; ++h) {
                const float2 f = __half22float2(*reinterpret_cast<const __half2 *>(&w[h]));
                kf[2 * h] = f.x;
                kf[2 * h + 1] = f.y;
            }
#pragma unroll
            for (int g = 0; g < G; ++g) {
                const float4 qa = *reinterpret_cast<const float4 *>(&sm.q[g][qd][8 * i]);
                const float4 qb = *reinterpret_cast<const float4 *>(&sm.q[g][qd][8 * i + 4]);
                s[g] += qa.x * kf[0] + qa.y * kf[1] + qa.z * kf[2] + qa.w * kf[3] + qb.x * kf[4] + qb.y * kf[5] +
                        qb.z * kf[6] + qb.w * kf[7];
            }
        }
        const bool valid = t0 + ku < w1x;
#pragma unroll
        for (int g = 0; g < G; ++g) {
            float sg = s[g];
            sg += __shfl_xor_sync(0xffffffffu, sg, 1);
            sg += __shfl_xor_sync(0xffffffffu, sg, 2);
            sg = valid ? sg * inv_sqrt : -INFINITY;
            float mn = sg;
            mn = fmaxf(mn, __shfl_xor_sync(0xffffffffu, mn, 4));
            mn = fmaxf(mn, __shfl_xor_sync(0xffffffffu, mn, 8));
            mn = fmaxf(mn, __shfl_xor_sync(0xffffffffu, mn, 16));
            mn = fmaxf(mn, m[g]);  // finite: the batch has at least one valid key
            const float corr = expf(m[g] - mn);
            const float p = expf(sg - mn);  // exp(-inf) = 0 for masked keys
            float psum = p;
            psum += __shfl_xor_sync(0xffffffffu, psum, 4);
            psum += __shfl_xor_sync(0xffffffffu, psum, 8);
            psum += __shfl_xor_sync(0xffffffffu, psum, 16);
            l[g] = l[g] * corr + psum;
            m[g] = mn;
#pragma unroll
            for (int j = 0; j < VEC; ++j) acc[g][j] *= corr;
#pragma unroll
            for (int u = 0; u < UN; ++u) {
                const float pu = __shfl_sync(0xffffffffu, p, 4 * u);
#pragma unroll
                for (int j = 0; j < VEC / 2; ++j) {
                    const float2 f = __half22float2(*reinterpret_cast<const __half2 *>(&vq[u][j]));
                    acc[g][2 * j] += pu * f.x;
                    acc[g][2 * j + 1] += pu * f.y;
                }
            }
        }
    }
#pragma unroll
    for (int g = 0; g < G; ++g) {
#pragma unroll
        for (int j = 0; j < VEC; ++j) sm.red[warp][g][lane * VEC + j] = acc[g][j];
        if (lane == 0) {
            sm.red[warp][g][HD] = m[g];
            sm.red[warp][g][HD + 1] = l[g];
        }
    }
    __syncthreads();
    trace_mark(trace, 4);

    // Fold the warps of this CTA (a warp without keys has m = -inf, l = 0 and weighs nothing) and
    // hand the result to the cluster's first CTA.
    if (csize > 1) asm volatile("barrier.cluster.wait.aligned;" ::: "memory");
    for (int idx = tid; idx < G * HD; idx += kAttnThreads) {
        const int g = idx / HD, d = idx - g * HD;
        float M = -INFINITY;
#pragma unroll
        for (int w = 0; w < kAttnWarps; ++w) M = fmaxf(M, sm.red[w][g][HD]);
        float val = 0.f, L = 0.f;
#pragma unroll
        for (int w = 0; w < kAttnWarps; ++w) {
            const float mw = sm.red[w][g][HD];
            const float wgt = (mw == -INFINITY) ? 0.f : expf(mw - M);
            val += sm.red[w][g][d] * wgt;
            L += sm.red[w][g][HD + 1] * wgt;
        }
        if (crank == 0) {
            sm.part[0][g][d] = val;
            if (d == 0) {
                sm.part[0][g][HD] = M;
                sm.part[0][g][HD + 1] = L;
            }
        } else {
            st_cluster_f32(&sm.part[crank][g][d], 0, val);
            if (d == 0) {
                st_cluster_f32(&sm.part[crank][g][HD], 0, M);
                st_cluster_f32(&sm.part[crank][g][HD + 1], 0, L);
            }
        }
    }
    if (csize > 1) {
        asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
        if (crank != 0) {
            if (tid == 0) trace_cta_exit();
            return;  // the stores above are ordered before the arrival; nobody reads this CTA's memory
        }
        asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
    } else {
        __syncthreads();
    }
    const size_t pstride = size_t(HD + 2);
    for (int idx = tid; idx < G * HD; idx += kAttnThreads) {
        const int g = idx / HD, d = idx - g * HD;
        float M = -INFINITY;
#pragma unroll
        for (int r = 0; r < kAttnMaxCluster; ++r)
            if (r < csize) M = fmaxf(M, sm.part[r][g][HD]);
        float val = 0.f, L = 0.f;
#pragma unroll
        for (int r = 0; r < kAttnMaxCluster; ++r) {
            if (r < csize) {
                const float mr = sm.part[r][g][HD];
                const float wgt = (mr == -INFINITY) ? 0.f : expf(mr - M);
                val += sm.part[r][g][d] * wgt;
                L += sm.part[r][g][HD + 1] * wgt;
            }
        }
        const int h = kvh * G + g;
        if (ncl == 1) {
            attn_store(a, size_t(b), h * HD + d, val / L);
        } else {
            float *p = a.partial + ((size_t(b) * a.heads + h) * ncl_max + cl) * pstride;
            p[d] = val;
            if (d == 0) {
                p[HD] = M;
                p[HD + 1] = L;
            }
        }
    }
    if (ncl == 1) {
        trace_mark(trace, 5);
        if (tid == 0) trace_cta_exit();
        return;
    }

    // Several clusters: the last of them to finish folds their results.
    __threadfence();
    __syncthreads();
    if (tid == 0) {
        const unsigned prev = atomicAdd(a.counters + size_t(b) * a.kv_heads + kvh, 1u);
        sm.is_last = (prev == unsigned(ncl) - 1u);
    }
    __syncthreads();
    if (!sm.is_last) return;
    __threadfence();
    for (int idx = tid; idx < G * kAttnMaxFold; idx += kAttnThreads) {
        const int g = idx / kAttnMaxFold, s = idx - g * kAttnMaxFold;
        const float *p = a.partial + (size_t(b) * a.heads + kvh * G + g) * ncl_max * pstride;
        sm.wgt[g][s] = s < ncl ? __ldcg(p + s * pstride + HD) : -INFINITY;
    }
    __syncthreads();
    if (tid < G) {
        const int g = tid;
        const float *p = a.partial + (size_t(b) * a.heads + kvh * G + g) * ncl_max * pstride;
        float M = -INFINITY;
        for (int s = 0; s < ncl; ++s) M = fmaxf(M, sm.wgt[g][s]);
        float L = 0.f;
        for (int s = 0; s < ncl; ++s) {
            const float msv = sm.wgt[g][s];
            const float w = (msv == -INFINITY) ? 0.f : expf(msv - M);
            sm.wgt[g][s] = w;
            L += __ldcg(p + s * pstride + HD + 1) * w;
        }
        sm.inv_l[g] = 1.0f / L;
    }
    __syncthreads();
    for (int idx = tid; idx < G * HD; idx += kAttnThreads) {
        const int g = idx / HD, d = idx - g * HD;
        const float *p = a.partial + (size_t(b) * a.heads + kvh * G + g) * ncl_max * pstride + d;
        float ld[kAttnMaxFold];
#pragma unroll
        for (int u = 0; u < kAttnMaxFold; ++u) ld[u] = u < ncl ? __ldcg(p + u * pstride) : 0.f;
        float val = 0.f;
#pragma unroll
        for (int u = 0; u < kAttnMaxFold; ++u)
            if (u < ncl) val += ld[u] * sm.wgt[g][u];
        attn_store(a, size_t(b), (kvh * G + g) * HD + d, val * sm.inv_l[g]);
    }
    if (tid == 0) a.counters[size_t(b) * a.kv_heads + kvh] = 0u;
}

// nsplit = cluster size * clusters per (row, KV head); the cluster size is the largest power of two
// up to 8 that divides it.
int attention_cluster_size(int nsplit) {
    int c = 1;
    while (c < kAttnMaxCluster && nsplit % (2 * c) == 0) c *= 2;
    return c;
}

template <int HD, int G, bool WIDE>
cudaError_t attn_launch_w(const AttnArgs &a, int width, cudaStream_t stream, bool programmatic) {
    const int csize = attention_cluster_size(a.nsplit);
    if (a.nsplit / csize > kAttnMaxFold || (G * HD) % csize != 0) return cudaErrorInvalidValue;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(a.nsplit, a.kv_heads, width);
    cfg.blockDim = dim3(AttnShape<HD, G, WIDE>::threads);
    cfg.dynamicSmemBytes = sizeof(AttnSmem<HD, G, WIDE>);
    cfg.stream = stream;
    cudaLaunchAttribute attr[2];
    int na = 0;
    if (programmatic) {
        attr[na].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[na].val.programmaticStreamSerializationAllowed = 1;
        ++na;
    }
    if (csize > 1) {
        attr[na].id = cudaLaunchAttributeClusterDimension;
        attr[na].val.clusterDim.x = csize;
        attr[na].val.clusterDim.y = 1;
        attr[na].val.clusterDim.z = 1;
        ++na;
    }
    cfg.attrs = attr;
    cfg.numAttrs = na;
    return cudaLaunchKernelEx(&cfg, attn_decode_kernel<HD, G, WIDE>, a, csize);
}

template <int HD, int G>
cudaError_t attn_launch_t(const AttnArgs &a, int width, cudaStream_t stream, bool programmatic) {
    return width >= 4 ? attn_launch_w<HD, G, true>(a, width, stream, programmatic)
                      : attn_launch_w<HD, G, false>(a, width, stream, programmatic);
}

// ---- prompt attention: a tile of query rows against the pages on the tensor cores -------------------
// The rows of one prompt chunk all belong to one sequence and their keys are already in the pages, so a
// CTA can share every key: it takes 16 * RW consecutive rows and the G query heads of one KV head (one warp
// per head and 16-row block), walks the keys in tiles of 64 staged in shared memory, and keeps the running
// maximum, the running sum and the 16 x HD output of its rows in registers (online softmax). Products are
// mma.sync m16n8k16 with fp32 accumulation: S = Q K^T with the rotated query split into two binary16 parts
// (hi + lo, 22 significant bits; the keys are binary16 in the pages anyway), O += P V with the probabilities
// rounded to binary16 (they are in [0, 1]). Function of the reference's tensor-core prompt attention
// (backend/tornado/layers/TensorCoreBatchAttention.java:227-366), not its code; the arithmetic it must match
// is inference/op/CpuOperations.java:94-235 (score = q.k / sqrt(d), softmax, weighted sum of values).
template <int HD, int G>
struct PromptShape {
    // eight warps: 32 query rows per CTA at four query heads per KV head (16 measured 4-9 % slower on long prompts:
    // a staged key / value tile serves twice the rows); the kernel's ~210 registers rule out sixteen
    static constexpr int warps = G >= 8 ? G : 8;
    static constexpr int rw = warps / G;      // 16-row blocks per CTA
    static constexpr int tq = 16 * rw;        // query rows per CTA
    static constexpr int tk = 64;             // keys per tile
    static constexpr int ld = HD + 8;         // padded row of a staged tile, in binary16 elements
    static constexpr int pages = 1024;        // page bases kept in shared memory (16 K keys of 16-token pages)
    static constexpr int tile_halves = tk * ld;
    // two buffers of a key tile and a value tile each, then the page bases
    static constexpr int smem_bytes = 2 * 2 * tile_halves * 2 + pages * 8;
};

__device__ __forceinline__ void cp_async_16(uint32_t dst_smem, const void *src) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst_smem), "l"(src) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
__device__ __forceinline__ void cp_async_wait_all() { asm volatile("cp.async.wait_group 0;" ::: "memory"); }

__device__ __forceinline__ void mma_16816(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

template <int HD, int G>
__global__ void __launch_bounds__(PromptShape<HD, G>::warps * 32)
    attn_prompt_kernel(const AttnArgs a, int n) {
    using P = PromptShape<HD, G>;
    constexpr int TK = P::tk, LD = P::ld, KS = HD / 16, NB = TK / 8, DB = HD / 8, PS = TK / 16;
    extern __shared__ __align__(16) uint8_t prompt_smem[];
    __half *tiles = reinterpret_cast<__half *>(prompt_smem);  // [buffer][K | V][TK][LD]
    int64_t *page_base = reinterpret_cast<int64_t *>(prompt_smem + 2 * 2 * P::tile_halves * 2);
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int g = warp % G, rb = warp / G;
    const int kvh = blockIdx.y, head = kvh * G + g;
    const int cta_row0 = blockIdx.x * P::tq;
    const int qr = lane >> 2, qc = lane & 3;  // this lane's row of a block (and qr + 8) and column pair
    pdl_launch_dependents();
    pdl_wait();
    const int slot = a.slots[cta_row0];
    // The two rows of this lane, their positions (-1: no such row, or an inactive one: every key is masked).
    int row[2], pos[2];
#pragma unroll
    for (int h = 0; h < 2; ++h) {
        row[h] = cta_row0 + rb * 16 + qr + 8 * h;
        const bool on = row[h] < n && (a.active == nullptr || a.active[row[h]] != 0);
        pos[h] = on ? a.positions[row[h]] : -1;
    }
    // Keys this CTA needs: up to the largest position among its rows.
    int last = -1;
    for (int r = cta_row0; r < min(n, cta_row0 + P::tq); ++r)
        if (a.active == nullptr || a.active[r] != 0) last = max(last, a.positions[r]);
    // This warp's query block, rotated (inference/op/CpuOperations.java:94-147 applies RoPE to q before the
    // scores), as A fragments: hi and lo binary16 parts.
    uint32_t qhi[KS][4], qlo[KS][4];
#pragma unroll
    for (int k = 0; k < KS; ++k) {
#pragma unroll
        for (int f = 0; f < 4; ++f) {
            const int h = f & 1, d0 = 16 * k + 8 * (f >> 1) + 2 * qc;  // a0: row, a1: row + 8, a2 / a3: columns + 8
            float x0 = 0.f, x1 = 0.f;
            if (pos[h] >= 0) {
                const float *qh = a.q + size_t(row[h]) * a.dim + size_t(head) * HD;
                const float v0 = qh[d0], v1 = qh[d0 + 1];
                const float cr = a.rope_cos[size_t(pos[h]) * (HD / 2) + d0 / 2], ci = a.rope_sin[size_t(pos[h]) * (HD / 2) + d0 / 2];
                x0 = __fsub_rn(__fmul_rn(v0, cr), __fmul_rn(v1, ci));
                x1 = __fadd_rn(__fmul_rn(v0, ci), __fmul_rn(v1, cr));
            }
            const __half2 hi = __floats2half2_rn(x0, x1);
            const float2 back = __half22float2(hi);
            const __half2 lo = __floats2half2_rn(x0 - back.x, x1 - back.y);
            qhi[k][f] = *reinterpret_cast<const uint32_t *>(&hi);
            qlo[k][f] = *reinterpret_cast<const uint32_t *>(&lo);
        }
    }
    float o[DB][4];
#pragma unroll
    for (int db = 0; db < DB; ++db) o[db][0] = o[db][1] = o[db][2] = o[db][3] = 0.f;
    float m[2] = {-INFINITY, -INFINITY}, l[2] = {0.f, 0.f};
    const float inv_sqrt = 1.0f / sqrtf(static_cast<float>(HD));
    int wl = max(pos[0], pos[1]);  // the largest position among this warp's 16 rows
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) wl = max(wl, __shfl_xor_sync(0xffffffffu, wl, off));
    // Where each page of this sequence starts (for this layer and KV head), once per CTA.
    const int bt = a.kv.block_tokens;
    {
        const int64_t block_stride = int64_t(a.kv.layers) * bt * a.kv.kv_dim;
        const int npages = last >= 0 ? last / bt + 1 : 0;
        for (int pg = tid; pg < min(npages, P::pages); pg += P::warps * 32) {
            const int64_t phys = a.kv.block_table[int64_t(slot) * a.kv.blocks_per_slot + pg];
            page_base[pg] = phys * block_stride + int64_t(a.layer) * bt * a.kv.kv_dim + int64_t(kvh) * HD;
        }
    }
    __syncthreads();
    const uint32_t tiles_u32 = static_cast<uint32_t>(__cvta_generic_to_shared(tiles));
    // Keys and values t0 .. t0 + 63 of this KV head into buffer `buf`, as asynchronous 16-byte copies (past
    // the last key: zeros), so that the next tile travels while this one is multiplied.
    auto stage = [&](int t0, int buf) {
        constexpr int kChunks = TK * HD / 8;
        for (int c = tid; c < 2 * kChunks; c += P::warps * 32) {
            const int which = c >= kChunks, cc = which ? c - kChunks : c;
            const int key = cc / (HD / 8), part = cc % (HD / 8);
            const uint32_t dst = tiles_u32 + uint32_t(((buf * 2 + which) * P::tile_halves + key * LD + part * 8) * 2);
            const int t = t0 + key;
            if (t <= last) {
                const int pg = t / bt;
                const int64_t base = pg < P::pages ? page_base[pg] : kv_offset(a.kv, slot, t - t % bt, a.layer) + int64_t(kvh) * HD;
                cp_async_16(dst, (which ? a.kv.vpool : a.kv.kpool) + base + int64_t(t % bt) * a.kv.kv_dim + part * 8);
            } else {
                asm volatile("st.shared.v4.b32 [%0], {%1, %1, %1, %1};" ::"r"(dst), "r"(0u) : "memory");
            }
        }
        cp_async_commit();
    };
    if (last >= 0) stage(0, 0);
    for (int t0 = 0, it = 0; t0 <= last; t0 += TK, ++it) {
        const int buf = it & 1;
        cp_async_wait_all();  // this thread's copies of tile `it`
        __syncthreads();      // everybody's copies have landed, and everybody is done with tile it - 1
        if (t0 + TK <= last) stage(t0 + TK, buf ^ 1);
        if (t0 > wl) continue;  // every key of this tile lies after this warp's rows
        const __half (*ks)[LD] = reinterpret_cast<const __half (*)[LD]>(tiles + (buf * 2) * P::tile_halves);
        const uint32_t vs_u32 = tiles_u32 + uint32_t((buf * 2 + 1) * P::tile_halves * 2);
        // S = Q K^T for 16 rows x 64 keys.
        float sacc[NB][4];
#pragma unroll
        for (int nb = 0; nb < NB; ++nb) sacc[nb][0] = sacc[nb][1] = sacc[nb][2] = sacc[nb][3] = 0.f;
#pragma unroll
        for (int k = 0; k < KS; ++k) {
#pragma unroll
            for (int nb = 0; nb < NB; ++nb) {
                const uint32_t b0 = *reinterpret_cast<const uint32_t *>(&ks[nb * 8 + qr][16 * k + 2 * qc]);
                const uint32_t b1 = *reinterpret_cast<const uint32_t *>(&ks[nb * 8 + qr][16 * k + 8 + 2 * qc]);
                mma_16816(sacc[nb], qhi[k], b0, b1);
                mma_16816(sacc[nb], qlo[k], b0, b1);
            }
        }
        // Scale, mask what lies after each row's position, and fold the tile into the running softmax.
        float tmax[2] = {-INFINITY, -INFINITY};
#pragma unroll
        for (int nb = 0; nb < NB; ++nb) {
#pragma unroll
            for (int c = 0; c < 4; ++c) {
                const int h = c >> 1, key = t0 + nb * 8 + 2 * qc + (c & 1);
                const float v = key <= pos[h] ? sacc[nb][c] * inv_sqrt : -INFINITY;
                sacc[nb][c] = v;
                tmax[h] = fmaxf(tmax[h], v);
            }
        }
        float corr[2];
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            tmax[h] = fmaxf(tmax[h], __shfl_xor_sync(0xffffffffu, tmax[h], 1));
            tmax[h] = fmaxf(tmax[h], __shfl_xor_sync(0xffffffffu, tmax[h], 2));
            const float mn = fmaxf(m[h], tmax[h]);
            corr[h] = (mn == -INFINITY) ? 1.0f : expf(m[h] - mn);  // exp(-inf) = 0 on the first tile
            m[h] = mn;
            l[h] *= corr[h];
        }
        uint32_t pa[PS][4];
#pragma unroll
        for (int nb = 0; nb < NB; ++nb) {
            float pv[4];
#pragma unroll
            for (int c = 0; c < 4; ++c) {
                const int h = c >> 1;
                pv[c] = (m[h] == -INFINITY) ? 0.f : expf(sacc[nb][c] - m[h]);  // exp(-inf) = 0 for masked keys
                l[h] += pv[c];
            }
            const __half2 p01 = __floats2half2_rn(pv[0], pv[1]), p23 = __floats2half2_rn(pv[2], pv[3]);
            pa[nb >> 1][(nb & 1) * 2] = *reinterpret_cast<const uint32_t *>(&p01);
            pa[nb >> 1][(nb & 1) * 2 + 1] = *reinterpret_cast<const uint32_t *>(&p23);
        }
#pragma unroll
        for (int db = 0; db < DB; ++db) {
            o[db][0] *= corr[0];
            o[db][1] *= corr[0];
            o[db][2] *= corr[1];
            o[db][3] *= corr[1];
        }
        // O += P V: the values come out of shared memory transposed (ldmatrix.trans), 16 keys x 8 dimensions a time.
#pragma unroll
        for (int j = 0; j < PS; ++j) {
#pragma unroll
            for (int db = 0; db < DB; ++db) {
                uint32_t b0, b1;
                const uint32_t addr = vs_u32 + uint32_t(((16 * j + (lane & 15)) * LD + db * 8) * 2);
                asm volatile("ldmatrix.sync.aligned.m8n8.x2.trans.shared.b16 {%0, %1}, [%2];" : "=r"(b0), "=r"(b1) : "r"(addr));
                mma_16816(o[db], pa[j], b0, b1);
            }
        }
    }
    // The running sums were kept per lane: add the four lanes of a row, then write out / l.
#pragma unroll
    for (int h = 0; h < 2; ++h) {
        l[h] += __shfl_xor_sync(0xffffffffu, l[h], 1);
        l[h] += __shfl_xor_sync(0xffffffffu, l[h], 2);
    }
#pragma unroll
    for (int db = 0; db < DB; ++db) {
#pragma unroll
        for (int c = 0; c < 4; ++c) {
            const int h = c >> 1;
            if (pos[h] >= 0) attn_store(a, size_t(row[h]), head * HD + db * 8 + 2 * qc + (c & 1), o[db][c] / l[h]);
        }
    }
}

template <int HD, int G>
cudaError_t attn_prompt_launch_t(const AttnArgs &a, int n, cudaStream_t stream, bool programmatic) {
    using P = PromptShape<HD, G>;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((n + P::tq - 1) / P::tq, a.kv_heads);
    cfg.blockDim = dim3(P::warps * 32);
    cfg.dynamicSmemBytes = P::smem_bytes;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = programmatic ? 1 : 0;
    return cudaLaunchKernelEx(&cfg, attn_prompt_kernel<HD, G>, a, n);
}

template <int HD>
cudaError_t attn_prompt_launch_hd(const AttnArgs &a, int n, cudaStream_t s, bool pdl) {
    switch (a.heads / a.kv_heads) {
        case 1: return attn_prompt_launch_t<HD, 1>(a, n, s, pdl);
        case 2: return attn_prompt_launch_t<HD, 2>(a, n, s, pdl);
        case 4: return attn_prompt_launch_t<HD, 4>(a, n, s, pdl);
        case 8: return attn_prompt_launch_t<HD, 8>(a, n, s, pdl);
        default: return cudaErrorInvalidValue;
    }
}

// ---- decode attention for wide batches: the query heads of a KV head as the rows of an MMA tile ---------------
// One CTA per (batch row, KV head). The G query heads that share the KV head are rows 0..G-1 of the 16-row A
// operand (the other rows are zero), so the scores of all heads against 64 keys are 16 mma.sync per key tile
// and warp instead of a few thousand scalar multiply-adds, and the kernel runs at the speed the pages arrive.
// The four warps share the staged key / value tiles (cp.async, one tile ahead, as in the prompt kernel) and
// split each tile's 64 keys four ways; each keeps its own running maximum, sum and output, merged at the end.
// The step's own key and value (rotated, rounded to binary16 as the append does) are written to the page and
// dropped into the staged tile by the CTA itself, so nothing else has to run before it.
// Arithmetic: inference/op/CpuOperations.java:94-235, as attn_decode_kernel.
template <int HD, int G>
struct BatchAttnShape {
    static constexpr int warps = 4;
    static constexpr int tk = 64;       // keys per tile: sixteen per warp
    static constexpr int depth = 3;     // tile buffers: two tiles in flight while one is used
    static constexpr int ld = HD + 8;
    static constexpr int pages = 256;   // page bases kept in shared memory (4 K keys of 16-token pages)
    static constexpr int tile_halves = tk * ld;
    static constexpr int merge_floats = warps * G * (HD + 2);  // overlays the tiles once the keys are done
    static constexpr int smem_bytes = depth * 2 * tile_halves * 2 + pages * 8;  // two CTAs per SM at HD = 128
    static_assert(merge_floats * 4 <= depth * 2 * tile_halves * 2, "the merge area overlays the tile buffers");
};

template <int HD, int G>
__global__ void __launch_bounds__(BatchAttnShape<HD, G>::warps * 32, 2)
    attn_batch_kernel(const AttnArgs a) {
    using P = BatchAttnShape<HD, G>;
    constexpr int TK = P::tk, LD = P::ld, KS = HD / 16, DB = HD / 8, NBUF = P::depth;
    constexpr int PARTS = HD / 8;                       // 16-byte chunks per key row
    constexpr int KEYS_PER_PASS = P::warps * 32 / PARTS;  // key rows one pass of the CTA's threads covers
    extern __shared__ __align__(16) uint8_t batch_smem[];
    __half *tiles = reinterpret_cast<__half *>(batch_smem);  // [buffer][K | V][TK][LD]
    int64_t *page_base = reinterpret_cast<int64_t *>(batch_smem + NBUF * 2 * P::tile_halves * 2);
    float *merge = reinterpret_cast<float *>(batch_smem);  // after the last tile
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int kvh = blockIdx.x, b = blockIdx.y;
    const int qr = lane >> 2, qc = lane & 3;
    const bool on = a.active == nullptr || a.active[b] != 0;
    const int trace = trace_begin(kTraceAttn);
    pdl_launch_dependents();
    // positions, slots and the block table are not written by anything in this step (see attn_decode_kernel)
    const int pos = on ? a.positions[b] : -1;
    const int slot = on ? a.slots[b] : 0;
    const int bt = a.kv.block_tokens;
    if (on) {
        const int64_t block_stride = int64_t(a.kv.layers) * bt * a.kv.kv_dim;
        for (int pg = tid; pg < min(pos / bt + 1, P::pages); pg += P::warps * 32) {
            const int64_t phys = a.kv.block_table[int64_t(slot) * a.kv.blocks_per_slot + pg];
            page_base[pg] = phys * block_stride + int64_t(a.layer) * bt * a.kv.kv_dim + int64_t(kvh) * HD;
        }
    }
    __syncthreads();
    const uint32_t tiles_u32 = static_cast<uint32_t>(__cvta_generic_to_shared(tiles));
    auto key_offset = [&](int t) -> int64_t {
        const int pg = t / bt;
        const int64_t base = pg < P::pages ? page_base[pg] : kv_offset(a.kv, slot, t - t % bt, a.layer) + int64_t(kvh) * HD;
        return base + int64_t(t % bt) * a.kv.kv_dim;
    };
    // Keys 0 .. pos - 1 come from the pages (this step's key, position pos, is written below). A thread copies the
    // same 16-byte part of every KEYS_PER_PASS-th key row, of the key tile and of the value tile.
    const int part = tid % PARTS, key_first = tid / PARTS;
    auto stage = [&](int t0, int buf) {
#pragma unroll
        for (int key = key_first; key < TK; key += KEYS_PER_PASS) {
            const uint32_t dk = tiles_u32 + uint32_t(((buf * 2) * P::tile_halves + key * LD + part * 8) * 2);
            const uint32_t dv = dk + uint32_t(P::tile_halves * 2);
            const int t = t0 + key;
            if (t < pos) {
                const int64_t off = key_offset(t) + part * 8;
                cp_async_16(dk, a.kv.kpool + off);
                cp_async_16(dv, a.kv.vpool + off);
            } else {
                asm volatile("st.shared.v4.b32 [%0], {%1, %1, %1, %1};" ::"r"(dk), "r"(0u) : "memory");
                asm volatile("st.shared.v4.b32 [%0], {%1, %1, %1, %1};" ::"r"(dv), "r"(0u) : "memory");
            }
        }
        cp_async_commit();
    };
    const int ntiles = on ? pos / TK + 1 : 0;
    // old keys: in flight while the kernel ahead finishes (one commit group per tile slot, empty ones included,
    // so that "all but the newest NBUF - 2 groups" always means "the tile about to be used")
#pragma unroll
    for (int p = 0; p < NBUF - 1; ++p) {
        if (p < ntiles) stage(p * TK, p);
        else cp_async_commit();
    }
    pdl_wait();
    trace_mark(trace, 2);
    if (!on) return;
    // The G heads' queries, rotated, as rows 0..G-1 of the A operand (hi and lo binary16 parts); rows G..15 are zero.
    uint32_t qhi[KS][2], qlo[KS][2];  // a0 and a2 of each K step: a1 / a3 (rows 8..15) are zero
    const float *cr = a.rope_cos + size_t(pos) * (HD / 2), *ci = a.rope_sin + size_t(pos) * (HD / 2);
#pragma unroll
    for (int k = 0; k < KS; ++k) {
#pragma unroll
        for (int f = 0; f < 2; ++f) {
            const int d0 = 16 * k + 8 * f + 2 * qc;
            float x0 = 0.f, x1 = 0.f;
            if (qr < G) {
                const float *qh = a.q + size_t(b) * a.dim + size_t(kvh * G + qr) * HD;
                const float v0 = qh[d0], v1 = qh[d0 + 1];
                x0 = __fsub_rn(__fmul_rn(v0, cr[d0 / 2]), __fmul_rn(v1, ci[d0 / 2]));
                x1 = __fadd_rn(__fmul_rn(v0, ci[d0 / 2]), __fmul_rn(v1, cr[d0 / 2]));
            }
            const __half2 hi = __floats2half2_rn(x0, x1);
            const float2 back = __half22float2(hi);
            const __half2 lo = __floats2half2_rn(x0 - back.x, x1 - back.y);
            qhi[k][f] = *reinterpret_cast<const uint32_t *>(&hi);
            qlo[k][f] = *reinterpret_cast<const uint32_t *>(&lo);
        }
    }
    float o[DB][4];
#pragma unroll
    for (int db = 0; db < DB; ++db) o[db][0] = o[db][1] = o[db][2] = o[db][3] = 0.f;
    float m = -INFINITY, l = 0.f;  // of row qr (a head when qr < G)
    const float inv_sqrt = 1.0f / sqrtf(static_cast<float>(HD));
    trace_mark(trace, 3);
    for (int it = 0; it < ntiles; ++it) {
        const int t0 = it * TK, buf = it % NBUF;
        asm volatile("cp.async.wait_group %0;" ::"n"(NBUF - 2) : "memory");  // this thread's copies of tile `it`
        __syncthreads();  // everybody's copies of it have landed, and everybody is done with tile it - 1
        if (it + NBUF - 1 < ntiles) stage((it + NBUF - 1) * TK, (it + NBUF - 1) % NBUF);  // into the buffer tile it - 1 used
        else cp_async_commit();
        __half *kt = tiles + (buf * 2) * P::tile_halves, *vt = tiles + (buf * 2 + 1) * P::tile_halves;
        if (it == ntiles - 1) {
            // This step's key and value: rotate k, round both to binary16, into the page and into the tile.
            const int64_t off = key_offset(pos);
            const float *kh = a.k + size_t(b) * a.kv.kv_dim + size_t(kvh) * HD;
            const float *vh = a.v + size_t(b) * a.kv.kv_dim + size_t(kvh) * HD;
            for (int idx = tid; idx < HD; idx += P::warps * 32) {
                const int i = idx % (HD / 2);
                __half2 h;
                if (idx < HD / 2) {
                    const float v0 = kh[2 * i], v1 = kh[2 * i + 1];
                    h = __halves2half2(__float2half_rn(__fsub_rn(__fmul_rn(v0, cr[i]), __fmul_rn(v1, ci[i]))),
                                       __float2half_rn(__fadd_rn(__fmul_rn(v0, ci[i]), __fmul_rn(v1, cr[i]))));
                    *reinterpret_cast<__half2 *>(kt + (pos - t0) * LD + 2 * i) = h;
                    *reinterpret_cast<__half2 *>(a.kv.kpool + off + 2 * i) = h;
                } else {
                    h = __halves2half2(__float2half_rn(vh[2 * i]), __float2half_rn(vh[2 * i + 1]));
                    *reinterpret_cast<__half2 *>(vt + (pos - t0) * LD + 2 * i) = h;
                    *reinterpret_cast<__half2 *>(a.kv.vpool + off + 2 * i) = h;
                }
            }
            __syncthreads();
        }
        const int k0 = 16 * warp;  // this warp's sixteen keys of the tile
        if (t0 + k0 > pos) continue;
        // S = Q K^T: 16 rows (heads) x 16 keys; separate accumulators for the hi and the lo part of q, so that
        // four chains of MMAs run side by side
        float sh[2][4] = {{0.f, 0.f, 0.f, 0.f}, {0.f, 0.f, 0.f, 0.f}}, sl[2][4] = {{0.f, 0.f, 0.f, 0.f}, {0.f, 0.f, 0.f, 0.f}};
#pragma unroll
        for (int k = 0; k < KS; ++k) {
            const uint32_t ah[4] = {qhi[k][0], 0u, qhi[k][1], 0u}, al[4] = {qlo[k][0], 0u, qlo[k][1], 0u};
#pragma unroll
            for (int nb = 0; nb < 2; ++nb) {
                const uint32_t b0 = *reinterpret_cast<const uint32_t *>(kt + (k0 + nb * 8 + qr) * LD + 16 * k + 2 * qc);
                const uint32_t b1 = *reinterpret_cast<const uint32_t *>(kt + (k0 + nb * 8 + qr) * LD + 16 * k + 8 + 2 * qc);
                mma_16816(sh[nb], ah, b0, b1);
                mma_16816(sl[nb], al, b0, b1);
            }
        }
        // rows 0..7 are c0 / c1 of each lane: scale, mask the keys after pos, fold into the running soft-max
        float sv[2][2];
        float tmax = -INFINITY;
#pragma unroll
        for (int nb = 0; nb < 2; ++nb)
#pragma unroll
            for (int c = 0; c < 2; ++c) {
                sv[nb][c] = (t0 + k0 + nb * 8 + 2 * qc + c <= pos) ? (sh[nb][c] + sl[nb][c]) * inv_sqrt : -INFINITY;
                tmax = fmaxf(tmax, sv[nb][c]);
            }
        tmax = fmaxf(tmax, __shfl_xor_sync(0xffffffffu, tmax, 1));
        tmax = fmaxf(tmax, __shfl_xor_sync(0xffffffffu, tmax, 2));
        const float mn = fmaxf(m, tmax);
        const float corr = (mn == -INFINITY) ? 1.0f : expf(m - mn);
        m = mn;
        l *= corr;
        uint32_t pa[4] = {0u, 0u, 0u, 0u};  // a0 (keys 0-7) and a2 (keys 8-15) of rows 0..7; a1 / a3 (rows 8..15) stay zero
#pragma unroll
        for (int nb = 0; nb < 2; ++nb) {
            const float p0 = (m == -INFINITY) ? 0.f : expf(sv[nb][0] - m), p1 = (m == -INFINITY) ? 0.f : expf(sv[nb][1] - m);
            l += p0 + p1;
            const __half2 ph = __floats2half2_rn(p0, p1);
            pa[2 * nb] = *reinterpret_cast<const uint32_t *>(&ph);
        }
        const uint32_t vt_u32 = tiles_u32 + uint32_t((buf * 2 + 1) * P::tile_halves * 2);
#pragma unroll
        for (int db = 0; db < DB; ++db) {
            o[db][0] *= corr;
            o[db][1] *= corr;
            uint32_t b0, b1;
            const uint32_t addr = vt_u32 + uint32_t(((k0 + (lane & 15)) * LD + db * 8) * 2);
            asm volatile("ldmatrix.sync.aligned.m8n8.x2.trans.shared.b16 {%0, %1}, [%2];" : "=r"(b0), "=r"(b1) : "r"(addr));
            mma_16816(o[db], pa, b0, b1);
        }
    }
    // Merge the four warps (each saw a quarter of every tile's keys): per head the maxima, sums and outputs.
    trace_mark(trace, 4);
    l += __shfl_xor_sync(0xffffffffu, l, 1);
    l += __shfl_xor_sync(0xffffffffu, l, 2);
    asm volatile("cp.async.wait_group 0;" ::: "memory");
    __syncthreads();  // everybody is done with the tiles: their memory becomes the merge area
    if (qr < G) {
        float *mine = merge + (warp * G + qr) * (HD + 2);
#pragma unroll
        for (int db = 0; db < DB; ++db) {
            mine[db * 8 + 2 * qc] = o[db][0];
            mine[db * 8 + 2 * qc + 1] = o[db][1];
        }
        if (qc == 0) {
            mine[HD] = m;
            mine[HD + 1] = l;
        }
    }
    __syncthreads();
    for (int idx = tid; idx < G * HD; idx += P::warps * 32) {
        const int g = idx / HD, d = idx - g * HD;
        float M = -INFINITY;
#pragma unroll
        for (int w = 0; w < P::warps; ++w) M = fmaxf(M, merge[(w * G + g) * (HD + 2) + HD]);
        float val = 0.f, L = 0.f;
#pragma unroll
        for (int w = 0; w < P::warps; ++w) {
            const float *pw = merge + (w * G + g) * (HD + 2);
            const float wgt = (pw[HD] == -INFINITY) ? 0.f : expf(pw[HD] - M);
            val += pw[d] * wgt;
            L += pw[HD + 1] * wgt;
        }
        attn_store(a, size_t(b), (kvh * G + g) * HD + d, val / L);
    }
    trace_mark(trace, 5);
}

template <int HD, int G>
cudaError_t attn_batch_launch_t(const AttnArgs &a, int width, cudaStream_t stream, bool programmatic) {
    using P = BatchAttnShape<HD, G>;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(a.kv_heads, width);
    cfg.blockDim = dim3(P::warps * 32);
    cfg.dynamicSmemBytes = P::smem_bytes;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = programmatic ? 1 : 0;
    return cudaLaunchKernelEx(&cfg, attn_batch_kernel<HD, G>, a);
}

template <int HD>
cudaError_t attn_batch_launch_hd(const AttnArgs &a, int width, cudaStream_t s, bool pdl) {
    switch (a.heads / a.kv_heads) {
        case 1: return attn_batch_launch_t<HD, 1>(a, width, s, pdl);
        case 2: return attn_batch_launch_t<HD, 2>(a, width, s, pdl);
        case 4: return attn_batch_launch_t<HD, 4>(a, width, s, pdl);
        case 8: return attn_batch_launch_t<HD, 8>(a, width, s, pdl);
        default: return cudaErrorInvalidValue;
    }
}

template <int HD>
cudaError_t attn_launch_hd(const AttnArgs &a, int width, cudaStream_t s, bool pdl) {
    switch (a.heads / a.kv_heads) {
        case 1: return attn_launch_t<HD, 1>(a, width, s, pdl);
        case 2: return attn_launch_t<HD, 2>(a, width, s, pdl);
        case 4: return attn_launch_t<HD, 4>(a, width, s, pdl);
        case 8: return attn_launch_t<HD, 8>(a, width, s, pdl);
        default: return cudaErrorInvalidValue;
    }
}

}  // namespace

namespace {
template <int HD, int G>
cudaError_t attn_configure_t() {
    const cudaError_t ep = cudaFuncSetAttribute(attn_prompt_kernel<HD, G>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                                PromptShape<HD, G>::smem_bytes);
    if (ep != cudaSuccess) return ep;
    const cudaError_t eb = cudaFuncSetAttribute(attn_batch_kernel<HD, G>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                                BatchAttnShape<HD, G>::smem_bytes);
    if (eb != cudaSuccess) return eb;
    const cudaError_t e = cudaFuncSetAttribute(attn_decode_kernel<HD, G, false>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                               int(sizeof(AttnSmem<HD, G, false>)));
    if (e != cudaSuccess) return e;
    return cudaFuncSetAttribute(attn_decode_kernel<HD, G, true>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                int(sizeof(AttnSmem<HD, G, true>)));
}
template <int HD>
cudaError_t attn_configure_hd() {
    cudaError_t e;
    if ((e = attn_configure_t<HD, 1>()) != cudaSuccess) return e;
    if ((e = attn_configure_t<HD, 2>()) != cudaSuccess) return e;
    if ((e = attn_configure_t<HD, 4>()) != cudaSuccess) return e;
    return attn_configure_t<HD, 8>();
}
}  // namespace

cudaError_t attention_configure() {
    const cudaError_t e = attn_configure_hd<128>();
    return e != cudaSuccess ? e : attn_configure_hd<64>();
}

size_t attention_partial_floats(int width, int heads, int nsplit, int head_dim) {
    return size_t(width) * heads * nsplit * (head_dim + 2);
}

int attention_splits(int sm_count, int width, int kv_heads) {
    // About two CTAs per SM over the whole launch: first a cluster of up to 8 per (row, KV head),
    // then up to kAttnMaxFold clusters.
    const int per = (2 * sm_count) / (width * kv_heads);
    int c = 1;
    while (c < kAttnMaxCluster && 2 * c <= per) c *= 2;
    int ncl = per / c;
    if (ncl < 1) ncl = 1;
    if (ncl > 4) ncl = 4;
    return c * ncl;
}

cudaError_t attention_launch(const AttnArgs &a, int width, cudaStream_t stream, bool programmatic) {
    if (a.head_dim == 128) return attn_launch_hd<128>(a, width, stream, programmatic);
    if (a.head_dim == 64) return attn_launch_hd<64>(a, width, stream, programmatic);
    return cudaErrorInvalidValue;
}

cudaError_t attention_batch_launch(const AttnArgs &a, int width, cudaStream_t stream, bool programmatic) {
    if (a.head_dim == 128) return attn_batch_launch_hd<128>(a, width, stream, programmatic);
    if (a.head_dim == 64) return attn_batch_launch_hd<64>(a, width, stream, programmatic);
    return cudaErrorInvalidValue;
}

cudaError_t attention_prompt_launch(const AttnArgs &a, int n, cudaStream_t stream, bool programmatic) {
    if (a.head_dim == 128) return attn_prompt_launch_hd<128>(a, n, stream, programmatic);
    if (a.head_dim == 64) return attn_prompt_launch_hd<64>(a, n, stream, programmatic);
    return cudaErrorInvalidValue;
}

cudaError_t embedding_launch(int type, const uint8_t *table, const int32_t *tokens,
                             const uint8_t *active, float *x, int dim, int width,
                             cudaStream_t stream, bool programmatic) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((dim + 255) / 256, width);
    cfg.blockDim = dim3(256);
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = programmatic ? 1 : 0;
    return cudaLaunchKernelEx(&cfg, embedding_kernel, type, table, tokens, active, x, dim);
}

cudaError_t pad_q6k_launch(const uint8_t *src, uint8_t *dst, size_t nblocks, cudaStream_t stream) {
    if (nblocks == 0) return cudaSuccess;
    const size_t want = (nblocks * (kQ6_KPadded / 2) + 255) / 256;
    pad_q6k_kernel<<<unsigned(want < 148 * 32 ? want : 148 * 32), 256, 0, stream>>>(src, dst, nblocks);
    return cudaGetLastError();
}

cudaError_t dequant_launch(int type, const uint8_t *blocks, int64_t n, float *out,
                           cudaStream_t stream) {
    if (n <= 0) return cudaSuccess;
    int64_t blocks_needed = (n + 255) / 256;
    int grid = static_cast<int>(blocks_needed < 148 * 16 ? blocks_needed : 148 * 16);
    dequant_kernel<<<grid, 256, 0, stream>>>(type, blocks, n, out);
    return cudaGetLastError();
}

cudaError_t advance_launch(int32_t *tokens, int32_t *positions, const int32_t *sampled,
                           const uint8_t *active, int32_t *history, int32_t *step_counter, int width,
                           cudaStream_t stream, bool programmatic) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(1);
    cfg.blockDim = dim3(256);
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = programmatic ? 1 : 0;
    return cudaLaunchKernelEx(&cfg, advance_kernel, tokens, positions, sampled, active, history,
                              step_counter, width);
}

// One launch configuration for the row kernels, with or without the programmatic-dependent-launch attribute.
struct RowLaunch {
    cudaLaunchConfig_t cfg = {};
    cudaLaunchAttribute attr[1] = {};
    RowLaunch(int grid, int block, cudaStream_t stream, bool programmatic) {
        cfg.gridDim = dim3(unsigned(grid));
        cfg.blockDim = dim3(unsigned(block));
        cfg.stream = stream;
        attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[0].val.programmaticStreamSerializationAllowed = 1;
        cfg.attrs = attr;
        cfg.numAttrs = programmatic ? 1 : 0;
    }
};

cudaError_t rmsnorm_rows_launch(const float *x, const float *w, float eps, float *out, int dim, int n,
                                const uint8_t *active, cudaStream_t stream, void *hi, void *lo, bool programmatic) {
    RowLaunch l(n, kNormThreads, stream, programmatic);
    return cudaLaunchKernelEx(&l.cfg, rmsnorm_rows_kernel, x, w, eps, out, dim, active, static_cast<uint2 *>(hi),
                              static_cast<uint2 *>(lo));
}

cudaError_t swiglu_rows_launch(float *g, const float *u, int hidden, int n, cudaStream_t stream, void *hi, void *lo,
                               bool programmatic) {
    const size_t total4 = size_t(hidden) * n / 4;
    const int grid = static_cast<int>((total4 + 255) / 256 < 148 * 8 ? (total4 + 255) / 256 : 148 * 8);
    RowLaunch l(grid, 256, stream, programmatic);
    return cudaLaunchKernelEx(&l.cfg, swiglu_rows_kernel, reinterpret_cast<float4 *>(g), reinterpret_cast<const float4 *>(u),
                              total4, static_cast<uint2 *>(hi), static_cast<uint2 *>(lo));
}

cudaError_t kv_append_launch(const float *k, const float *v, const float *rope_cos, const float *rope_sin,
                             const int32_t *positions, const int32_t *slots, const uint8_t *active,
                             KvGeom kv, int layer, int head_dim, int n, cudaStream_t stream, bool programmatic) {
    RowLaunch l(n, 256, stream, programmatic);
    return cudaLaunchKernelEx(&l.cfg, kv_append_kernel, k, v, rope_cos, rope_sin, positions, slots, active, kv, layer, head_dim);
}

cudaError_t argmax_rows_launch(const float *logits, int vocab, int n, const uint8_t *active, int32_t *out,
                               cudaStream_t stream, bool programmatic) {
    RowLaunch l(n, 1024, stream, programmatic);
    return cudaLaunchKernelEx(&l.cfg, argmax_rows_kernel, logits, vocab, active, out);
}

cudaError_t add_rows_launch(float *x, const float *y, size_t total, cudaStream_t stream, bool programmatic) {
    const int grid = static_cast<int>((total + 1023) / 1024 < 148 * 8 ? (total + 1023) / 1024 : 148 * 8);
    RowLaunch l(grid, 256, stream, programmatic);
    return cudaLaunchKernelEx(&l.cfg, add_rows_kernel, x, y, total);
}

cudaError_t split_rows_launch(const float *x, size_t total, void *hi, void *lo, cudaStream_t stream, bool programmatic) {
    const size_t total4 = total / 4;  // row lengths are multiples of 256
    const int grid = static_cast<int>((total4 + 255) / 256 < 148 * 8 ? (total4 + 255) / 256 : 148 * 8);
    RowLaunch l(grid, 256, stream, programmatic);
    return cudaLaunchKernelEx(&l.cfg, split_rows_kernel, reinterpret_cast<const float4 *>(x), total4, static_cast<uint2 *>(hi),
                              static_cast<uint2 *>(lo));
}

cudaError_t tp_pack_best_launch(const float *logits, const int32_t *idx, int l_vocab, int index_offset, int n,
                                float *best, cudaStream_t stream) {
    tp_pack_best_kernel<<<(n + 127) / 128, 128, 0, stream>>>(logits, idx, l_vocab, index_offset, n, best);
    return cudaGetLastError();
}

cudaError_t tp_pick_best_launch(const float *all, int ranks, int n, const uint8_t *active, int32_t *out,
                                cudaStream_t stream) {
    tp_pick_best_kernel<<<(n + 127) / 128, 128, 0, stream>>>(all, ranks, n, active, out);
    return cudaGetLastError();
}

cudaError_t fill_launch(uint32_t *buf, size_t words, uint32_t value, cudaStream_t stream) {
    fill_kernel<<<148 * 8, 256, 0, stream>>>(buf, words, value);
    return cudaGetLastError();
}

}  // namespace jl
