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

__global__ void add_rows_kernel(float *x, const float *y, size_t total) {
    const size_t stride = size_t(gridDim.x) * blockDim.x;
    for (size_t i = size_t(blockIdx.x) * blockDim.x + threadIdx.x; i < total; i += stride) x[i] = x[i] + y[i];
}

__global__ void split_rows_kernel(const float4 *x, size_t total4, uint2 *hi, uint2 *lo) {
    const size_t stride = size_t(gridDim.x) * blockDim.x;
    for (size_t i = size_t(blockIdx.x) * blockDim.x + threadIdx.x; i < total4; i += stride) {
        const float4 v = x[i];
        const __half2 h0 = __floats2half2_rn(v.x, v.y), h1 = __floats2half2_rn(v.z, v.w);
        const float2 b0 = __half22float2(h0), b1 = __half22float2(h1);
        const __half2 l0 = __floats2half2_rn(v.x - b0.x, v.y - b0.y), l1 = __floats2half2_rn(v.z - b1.x, v.w - b1.y);
        hi[i] = make_uint2(*reinterpret_cast<const uint32_t *>(&h0), *reinterpret_cast<const uint32_t *>(&h1));
        lo[i] = make_uint2(*reinterpret_cast<const uint32_t *>(&l0), *reinterpret_cast<const uint32_t *>(&l1));
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
        if (hr != nullptr) {
            const __half2 h0 = __floats2half2_rn(r.x, r.y), h1 = __floats2half2_rn(r.z, r.w);
            const float2 b0 = __half22float2(h0), b1 = __half22float2(h1);
            const __half2 l0 = __floats2half2_rn(r.x - b0.x, r.y - b0.y), l1 = __floats2half2_rn(r.z - b1.x, r.w - b1.y);
            hr[i] = make_uint2(*reinterpret_cast<const uint32_t *>(&h0), *reinterpret_cast<const uint32_t *>(&h1));
            lr[i] = make_uint2(*reinterpret_cast<const uint32_t *>(&l0), *reinterpret_cast<const uint32_t *>(&l1));
        }
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
    const size_t stride = size_t(gridDim.x) * blockDim.x;
    for (size_t i = size_t(blockIdx.x) * blockDim.x + threadIdx.x; i < total4; i += stride) {
        const float4 v = g[i], w = u[i];
        float4 r;
        r.x = (v.x / (1.0f + expf(-v.x))) * w.x;
        r.y = (v.y / (1.0f + expf(-v.y))) * w.y;
        r.z = (v.z / (1.0f + expf(-v.z))) * w.z;
        r.w = (v.w / (1.0f + expf(-v.w))) * w.w;
        g[i] = r;
        if (hi != nullptr) {
            const __half2 h0 = __floats2half2_rn(r.x, r.y), h1 = __floats2half2_rn(r.z, r.w);
            const float2 b0 = __half22float2(h0), b1 = __half22float2(h1);
            const __half2 l0 = __floats2half2_rn(r.x - b0.x, r.y - b0.y), l1 = __floats2half2_rn(r.z - b1.x, r.w - b1.y);
            hi[i] = make_uint2(*reinterpret_cast<const uint32_t *>(&h0), *reinterpret_cast<const uint32_t *>(&h1));
            lo[i] = make_uint2(*reinterpret_cast<const uint32_t *>(&l0), *reinterpret_cast<const uint32_t *>(&l1));
        }
    }
}

__global__ void kv_append_kernel(const float *k, const float *v, const float *rope_cos, const float *rope_sin,
                                 const int32_t *positions, const int32_t *slots, const uint8_t *active,
                                 KvGeom kv, int layer, int head_dim) {
    const int row = blockIdx.x;
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

constexpr int kAttnThreads = 256;
constexpr int kAttnWarps = kAttnThreads / 32;
constexpr int kAttnMaxSplit = 32;
constexpr int kAttnMinKeysPerSplit = 64;

// Number of splits actually used for n keys: short contexts use few CTAs so that the fold at the
// end stays small; the launch grid is sized for the maximum and surplus CTAs leave at once.
__device__ __forceinline__ int splits_for(int n, int nsplit_max) {
    const int want = (n + kAttnMinKeysPerSplit - 1) / kAttnMinKeysPerSplit;
    return max(1, min(nsplit_max, want));
}

// One CTA = (split of the position range, KV head, batch row). The G query heads that share the
// KV head are processed together so each K/V row is read once. What it computes is
// CpuOperations.rope + appendKeyValue + attention (inference/op/CpuOperations.java:94-204) with
// the softmax evaluated online; K and V are rounded to binary16 on append exactly as
// ArrayHalfFloatTensor.setFloat does (tensor/standard/ArrayHalfFloatTensor.java:33-40).
template <int HD, int G>
__global__ void __launch_bounds__(kAttnThreads) attn_decode_kernel(const AttnArgs a) {
    constexpr int VEC = HD / 32;
    constexpr int UN = 4;  // keys per warp iteration, loaded before any of them is used
    const int split = blockIdx.x, kvh = blockIdx.y, b = blockIdx.z;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int trace = trace_begin(kTraceAttn);
    const bool on = a.active == nullptr || a.active[b] != 0;
    pdl_wait();
    pdl_launch_dependents();
    trace_mark(trace, 2);
    const int pos = on ? a.positions[b] : 0;
    const int slot = on ? a.slots[b] : 0;
    const int n = pos + 1;
    const int nsplit = splits_for(n, a.nsplit);
    if (!on || split >= nsplit) return;

    __shared__ float q_s[G][HD];
    __shared__ float red[kAttnWarps][G][HD + 2];
    __shared__ float wgt_s[G][kAttnMaxSplit];
    __shared__ float inv_l[G];
    __shared__ int64_t page_base[kAttnMaxSplit * 0 + 40];
    __shared__ int is_last;

    const int chunk = (n + nsplit - 1) / nsplit;
    const int start = split * chunk;
    const int end = min(n, start + chunk);
    // Page bases of this CTA's key range (at most chunk/block_tokens + 2 pages).
    const int bt = a.kv.block_tokens;
    const int first_page = start / bt;
    const int npages = end > start ? (end - 1) / bt - first_page + 1 : 0;
    const int64_t block_stride = int64_t(a.kv.layers) * bt * a.kv.kv_dim;
    for (int pg = tid; pg < npages && pg < 40; pg += kAttnThreads) {
        const int64_t phys = a.kv.block_table[int64_t(slot) * a.kv.blocks_per_slot + first_page + pg];
        page_base[pg] = phys * block_stride + int64_t(a.layer) * bt * a.kv.kv_dim + int64_t(kvh) * HD;
    }
    const float *cr = a.rope_cos + size_t(pos) * (HD / 2);
    const float *ci = a.rope_sin + size_t(pos) * (HD / 2);
    for (int idx = tid; idx < G * (HD / 2); idx += kAttnThreads) {
        const int g = idx / (HD / 2), i = idx - g * (HD / 2);
        const float *qh = a.q + size_t(b) * a.dim + size_t(kvh * G + g) * HD;
        const float v0 = qh[2 * i], v1 = qh[2 * i + 1];
        q_s[g][2 * i] = __fsub_rn(__fmul_rn(v0, cr[i]), __fmul_rn(v1, ci[i]));
        q_s[g][2 * i + 1] = __fadd_rn(__fmul_rn(v0, ci[i]), __fmul_rn(v1, cr[i]));
    }
    if (a.append && start <= pos && pos < end) {
        // This CTA owns the new position: rotate k, round k and v to fp16, append to the page.
        const int64_t off = kv_offset(a.kv, slot, pos, a.layer) + int64_t(kvh) * HD;
        const float *kh = a.k + size_t(b) * a.kv.kv_dim + size_t(kvh) * HD;
        const float *vh = a.v + size_t(b) * a.kv.kv_dim + size_t(kvh) * HD;
        for (int i = tid; i < HD / 2; i += kAttnThreads) {
            const float v0 = kh[2 * i], v1 = kh[2 * i + 1];
            const float r0 = __fsub_rn(__fmul_rn(v0, cr[i]), __fmul_rn(v1, ci[i]));
            const float r1 = __fadd_rn(__fmul_rn(v0, ci[i]), __fmul_rn(v1, cr[i]));
            a.kv.kpool[off + 2 * i] = __float2half_rn(r0);
            a.kv.kpool[off + 2 * i + 1] = __float2half_rn(r1);
            a.kv.vpool[off + 2 * i] = __float2half_rn(vh[2 * i]);
            a.kv.vpool[off + 2 * i + 1] = __float2half_rn(vh[2 * i + 1]);
        }
    }
    __syncthreads();

    float m[G], l[G], acc[G][VEC], qr[G][VEC];
#pragma unroll
    for (int g = 0; g < G; ++g) {
        m[g] = -INFINITY;
        l[g] = 0.f;
#pragma unroll
        for (int j = 0; j < VEC; ++j) {
            acc[g][j] = 0.f;
            qr[g][j] = q_s[g][lane * VEC + j];
        }
    }
    const float inv_sqrt = 1.0f / sqrtf(static_cast<float>(HD));
    // Each warp takes a contiguous run of keys so that consecutive keys share a page.
    const int per_warp = (end - start + kAttnWarps - 1) / kAttnWarps;
    const int w0 = start + warp * per_warp;
    const int w1 = min(end, w0 + per_warp);
    for (int t0 = w0; t0 < w1; t0 += UN) {
        float kf[UN][VEC], vf[UN][VEC];
#pragma unroll
        for (int u = 0; u < UN; ++u) {
            const int t = min(t0 + u, w1 - 1);  // the tail repeats the last key; masked below
            const int pg = t / bt - first_page;
            const int64_t base = (pg < 40) ? page_base[pg] : kv_offset(a.kv, slot, t, a.layer) - int64_t(t % bt) * a.kv.kv_dim + int64_t(kvh) * HD;
            const int64_t off = base + int64_t(t % bt) * a.kv.kv_dim + lane * VEC;
            load_halfs<VEC>(a.kv.kpool + off, kf[u]);
            load_halfs<VEC>(a.kv.vpool + off, vf[u]);
        }
#pragma unroll
        for (int g = 0; g < G; ++g) {
            float s[UN];
#pragma unroll
            for (int u = 0; u < UN; ++u) {
                float d = 0.f;
#pragma unroll
                for (int j = 0; j < VEC; ++j) d += qr[g][j] * kf[u][j];
                s[u] = d;
            }
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) {
#pragma unroll
                for (int u = 0; u < UN; ++u) s[u] += __shfl_xor_sync(0xffffffffu, s[u], o);
            }
            float mn = m[g];
#pragma unroll
            for (int u = 0; u < UN; ++u) {
                s[u] = (t0 + u < w1) ? s[u] * inv_sqrt : -INFINITY;
                mn = fmaxf(mn, s[u]);
            }
            const float corr = expf(m[g] - mn);
            float psum = 0.f;
#pragma unroll
            for (int j = 0; j < VEC; ++j) acc[g][j] *= corr;
#pragma unroll
            for (int u = 0; u < UN; ++u) {
                const float p = expf(s[u] - mn);  // exp(-inf) = 0 for masked keys
                psum += p;
#pragma unroll
                for (int j = 0; j < VEC; ++j) acc[g][j] += p * vf[u][j];
            }
            l[g] = l[g] * corr + psum;
            m[g] = mn;
        }
    }
#pragma unroll
    for (int g = 0; g < G; ++g) {
#pragma unroll
        for (int j = 0; j < VEC; ++j) red[warp][g][lane * VEC + j] = acc[g][j];
        if (lane == 0) {
            red[warp][g][HD] = m[g];
            red[warp][g][HD + 1] = l[g];
        }
    }
    __syncthreads();

    const size_t pstride = size_t(HD + 2);
    for (int idx = tid; idx < G * HD; idx += kAttnThreads) {
        const int g = idx / HD, d = idx - g * HD;
        float M = -INFINITY;
#pragma unroll
        for (int w = 0; w < kAttnWarps; ++w) M = fmaxf(M, red[w][g][HD]);
        float val = 0.f, L = 0.f;
#pragma unroll
        for (int w = 0; w < kAttnWarps; ++w) {
            const float mw = red[w][g][HD];
            const float wgt = (mw == -INFINITY) ? 0.f : expf(mw - M);
            val += red[w][g][d] * wgt;
            L += red[w][g][HD + 1] * wgt;
        }
        const int h = kvh * G + g;
        if (nsplit == 1) {
            a.out[size_t(b) * a.dim + size_t(h) * HD + d] = val / L;
        } else {
            float *p = a.partial + ((size_t(b) * a.heads + h) * a.nsplit + split) * pstride;
            p[d] = val;
            if (d == 0) {
                p[HD] = M;
                p[HD + 1] = L;
            }
        }
    }
    if (nsplit == 1) return;

    // The last CTA of this (row, KV head) to finish folds the splits together.
    __threadfence();
    __syncthreads();
    if (tid == 0) {
        const unsigned prev = atomicAdd(a.counters + size_t(b) * a.kv_heads + kvh, 1u);
        is_last = (prev == unsigned(nsplit) - 1u);
    }
    __syncthreads();
    if (!is_last) return;
    __threadfence();
    // Fold weights first (one thread per (head, split)), then every output element sums its
    // splits with the loads issued four at a time.
    for (int idx = tid; idx < G * kAttnMaxSplit; idx += kAttnThreads) {
        const int g = idx / kAttnMaxSplit, s = idx - g * kAttnMaxSplit;
        const float *p = a.partial + (size_t(b) * a.heads + kvh * G + g) * a.nsplit * pstride;
        wgt_s[g][s] = s < nsplit ? __ldcg(p + s * pstride + HD) : -INFINITY;
    }
    __syncthreads();
    if (tid < G) {
        const int g = tid;
        const float *p = a.partial + (size_t(b) * a.heads + kvh * G + g) * a.nsplit * pstride;
        float M = -INFINITY;
        for (int s = 0; s < nsplit; ++s) M = fmaxf(M, wgt_s[g][s]);
        float L = 0.f;
        for (int s = 0; s < nsplit; ++s) {
            const float ms = wgt_s[g][s];
            const float w = (ms == -INFINITY) ? 0.f : expf(ms - M);
            wgt_s[g][s] = w;
            L += __ldcg(p + s * pstride + HD + 1) * w;
        }
        inv_l[g] = 1.0f / L;
    }
    __syncthreads();
    // Each thread owns G*HD/threads outputs and walks the splits eight at a time, so that all of a
    // batch's loads are in flight together (the fold is pure L2 latency otherwise).
    constexpr int kOuts = (G * HD + kAttnThreads - 1) / kAttnThreads;
    float val[kOuts];
#pragma unroll
    for (int j = 0; j < kOuts; ++j) val[j] = 0.f;
    for (int s0 = 0; s0 < nsplit; s0 += 8) {
        float ld[kOuts][8];
#pragma unroll
        for (int j = 0; j < kOuts; ++j) {
            const int idx = tid + j * kAttnThreads;
            const int g = idx / HD, d = idx - g * HD;
            const float *p = a.partial + (size_t(b) * a.heads + kvh * G + g) * a.nsplit * pstride + d;
#pragma unroll
            for (int u = 0; u < 8; ++u)
                ld[j][u] = (idx < G * HD && s0 + u < nsplit) ? __ldcg(p + (s0 + u) * pstride) : 0.f;
        }
#pragma unroll
        for (int j = 0; j < kOuts; ++j) {
            const int idx = tid + j * kAttnThreads;
            const int g = min(idx / HD, G - 1);
#pragma unroll
            for (int u = 0; u < 8; ++u)
                if (s0 + u < nsplit) val[j] += ld[j][u] * wgt_s[g][s0 + u];
        }
    }
#pragma unroll
    for (int j = 0; j < kOuts; ++j) {
        const int idx = tid + j * kAttnThreads;
        if (idx < G * HD) {
            const int g = idx / HD, d = idx - g * HD;
            a.out[size_t(b) * a.dim + size_t(kvh * G + g) * HD + d] = val[j] * inv_l[g];
        }
    }
    if (tid == 0) a.counters[size_t(b) * a.kv_heads + kvh] = 0u;
}

template <int HD, int G>
cudaError_t attn_launch_t(const AttnArgs &a, int width, cudaStream_t stream, bool programmatic) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(a.nsplit, a.kv_heads, width);
    cfg.blockDim = dim3(kAttnThreads);
    cfg.dynamicSmemBytes = 0;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = programmatic ? 1 : 0;
    return cudaLaunchKernelEx(&cfg, attn_decode_kernel<HD, G>, a);
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

cudaError_t attention_configure() { return cudaSuccess; }

size_t attention_partial_floats(int width, int heads, int nsplit, int head_dim) {
    return size_t(width) * heads * nsplit * (head_dim + 2);
}

cudaError_t attention_launch(const AttnArgs &a, int width, cudaStream_t stream, bool programmatic) {
    if (a.head_dim == 128) return attn_launch_hd<128>(a, width, stream, programmatic);
    if (a.head_dim == 64) return attn_launch_hd<64>(a, width, stream, programmatic);
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

cudaError_t rmsnorm_rows_launch(const float *x, const float *w, float eps, float *out, int dim, int n,
                                const uint8_t *active, cudaStream_t stream, void *hi, void *lo) {
    rmsnorm_rows_kernel<<<n, kNormThreads, 0, stream>>>(x, w, eps, out, dim, active, static_cast<uint2 *>(hi),
                                                        static_cast<uint2 *>(lo));
    return cudaGetLastError();
}

cudaError_t swiglu_rows_launch(float *g, const float *u, int hidden, int n, cudaStream_t stream, void *hi, void *lo) {
    const size_t total4 = size_t(hidden) * n / 4;
    const int grid = static_cast<int>((total4 + 255) / 256 < 148 * 8 ? (total4 + 255) / 256 : 148 * 8);
    swiglu_rows_kernel<<<grid, 256, 0, stream>>>(reinterpret_cast<float4 *>(g), reinterpret_cast<const float4 *>(u), total4,
                                                 static_cast<uint2 *>(hi), static_cast<uint2 *>(lo));
    return cudaGetLastError();
}

cudaError_t kv_append_launch(const float *k, const float *v, const float *rope_cos, const float *rope_sin,
                             const int32_t *positions, const int32_t *slots, const uint8_t *active,
                             KvGeom kv, int layer, int head_dim, int n, cudaStream_t stream) {
    kv_append_kernel<<<n, 256, 0, stream>>>(k, v, rope_cos, rope_sin, positions, slots, active, kv, layer,
                                            head_dim);
    return cudaGetLastError();
}

cudaError_t argmax_rows_launch(const float *logits, int vocab, int n, const uint8_t *active, int32_t *out,
                               cudaStream_t stream) {
    argmax_rows_kernel<<<n, 1024, 0, stream>>>(logits, vocab, active, out);
    return cudaGetLastError();
}

cudaError_t add_rows_launch(float *x, const float *y, size_t total, cudaStream_t stream) {
    const int grid = static_cast<int>((total + 1023) / 1024 < 148 * 8 ? (total + 1023) / 1024 : 148 * 8);
    add_rows_kernel<<<grid, 256, 0, stream>>>(x, y, total);
    return cudaGetLastError();
}

cudaError_t split_rows_launch(const float *x, size_t total, void *hi, void *lo, cudaStream_t stream) {
    const size_t total4 = total / 4;  // row lengths are multiples of 256
    const int grid = static_cast<int>((total4 + 255) / 256 < 148 * 8 ? (total4 + 255) / 256 : 148 * 8);
    split_rows_kernel<<<grid, 256, 0, stream>>>(reinterpret_cast<const float4 *>(x), total4, static_cast<uint2 *>(hi),
                                                static_cast<uint2 *>(lo));
    return cudaGetLastError();
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
