// Persistent per-token decode kernel for a single sequence on sm_100a.
//
// One cooperative launch per token, one CTA of 16 warps per SM. The kernel walks the operator
// sequence of InferenceCore.forwardJava (backend/cpu/InferenceCore.java:72-141 of the reference):
// embedding, then per layer RMSNorm+QKV, RoPE+KV append+attention, output projection+residual,
// RMSNorm+gate/up+SwiGLU, down projection+residual, and finally RMSNorm+vocabulary+arg-max.
// Dependent operators are separated by a grid barrier instead of a kernel boundary.
//
// Why: at batch 1 a matrix of the 8B model is 2-66 MB, i.e. 0.4-10 us of HBM time, and a kernel
// boundary costs several microseconds of launch, prologue, pipeline fill and tail during which
// HBM idles. Here every warp owns a ring of shared-memory slots that lane 0 keeps filled with 1-D
// bulk async copies (TMA) of the row chunks the warp will need next. The request stream does not
// stop at operator boundaries (weights do not depend on activations), so while a CTA waits at a
// barrier or stages the next activation vector, the weights of the next operator are already
// landing in its rings.
//
// Work split inside a matrix-vector operator: rows are divided evenly over CTAs (contiguous
// ranges), and inside a CTA the (row, 2048-column chunk) items are divided evenly over the warps
// in chunk-major order, so a warp re-reads its activation digits from shared memory only when
// the chunk changes. Chunk partial sums meet in shared memory and are added in chunk order, which
// keeps results independent of timing.
#include "token_kernel.cuh"

#include <climits>

#include "gemv_core.cuh"

namespace jl {

namespace {

constexpr int kTokThreads = 512;
constexpr int kTokWarps = kTokThreads / 32;
constexpr int kTokMaxSlots = 16;
constexpr int kBarBytes = kTokWarps * kTokMaxSlots * 8;  // 2048
constexpr int kScratchBytes = 256;
constexpr int kPartialFloats = 4096;
constexpr int kMaxLayers = 128;
constexpr unsigned kGridSpinLimit = 4u << 20;

__device__ __forceinline__ unsigned long long gtime() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
    return t;
}

// A matrix-vector operator, rebuilt from the layer table whenever needed.
struct GemvDesc {
    const uint8_t *w[3];
    int rows[3];
    int nseg;
    int cols;
    int rows_total;  // gate/up: rows of one of the two matrices
    int gateup;
};

// Per-warp producer cursor and ring position; lives in shared memory so that lane 0's request
// bookkeeping does not occupy registers in the arithmetic loop.
struct WarpState {
    const uint8_t *w[3];
    int rows[3];
    int g;  // matrix-vector operator index: 4*layer + {0 qkv, 1 out, 2 gate/up, 3 down}, 4*L = vocab
    int chunk, rl, e, left;
    int r_lo, rows_cnt, nunits, entries;
    unsigned rowb;
    int c_slot, c_parity;
    int pad[3];
};
static_assert(sizeof(WarpState) == 96, "WarpState layout");

__host__ __device__ inline size_t stage_region_bytes(int max_cols) {
    return x_region_bytes(max_cols) + size_t(kPartialFloats) * 4;
}
__host__ __device__ inline size_t attn_region_bytes(int hd, int g) {
    return size_t(g) * hd * 4 + size_t(kTokWarps) * g * (hd + 2) * 4 + 512;
}
__host__ __device__ inline size_t layer_table_bytes(int n_layers) {
    return align_up(size_t(n_layers) * sizeof(TokLayer), 128);
}
__host__ __device__ inline size_t header_bytes(int n_layers) {
    return kBarBytes + kScratchBytes + kTokWarps * sizeof(WarpState) + layer_table_bytes(n_layers);
}

// Arrive + bounded wait on a monotonically increasing counter. After a timeout the status word
// is set and later barriers return at once, so the kernel always terminates.
__device__ __forceinline__ void grid_sync(unsigned *counter, unsigned target, int *status) {
    __syncthreads();
    if (threadIdx.x == 0) {
        __threadfence();
        atomicAdd(counter, 1u);
        unsigned v = 0;
        if (*reinterpret_cast<volatile int *>(status) == kDevOk) {
            unsigned spins = 0;
            for (;;) {
                asm volatile("ld.acquire.gpu.u32 %0, [%1];" : "=r"(v) : "l"(counter) : "memory");
                if (v >= target) break;
                if (++spins > kGridSpinLimit) {
                    atomicExch(status, kDevTimeout);
                    break;
                }
            }
        }
    }
    __syncthreads();
}

__device__ __forceinline__ GemvDesc describe(const TokArgs &a, const TokLayer *layers, int g) {
    GemvDesc d = {};
    const int l = g >> 2, which = g & 3;
    if (l >= a.n_layers) {  // vocabulary projection
        d.w[0] = a.wcls;
        d.rows[0] = a.vocab;
        d.nseg = 1;
        d.cols = a.dim;
        d.rows_total = a.vocab;
        return d;
    }
    const TokLayer &L = layers[l];
    if (which == 0) {
        d.w[0] = L.wq; d.w[1] = L.wk; d.w[2] = L.wv;
        d.rows[0] = a.dim; d.rows[1] = a.kv_dim; d.rows[2] = a.kv_dim;
        d.nseg = 3;
        d.cols = a.dim;
        d.rows_total = a.dim + 2 * a.kv_dim;
    } else if (which == 1) {
        d.w[0] = L.wo;
        d.rows[0] = a.dim;
        d.nseg = 1;
        d.cols = a.dim;
        d.rows_total = a.dim;
    } else if (which == 2) {
        d.w[0] = L.w1; d.w[1] = L.w3;
        d.rows[0] = a.hidden; d.rows[1] = a.hidden;
        d.nseg = 2;
        d.cols = a.dim;
        d.rows_total = a.hidden;
        d.gateup = 1;
    } else {
        d.w[0] = L.w2;
        d.rows[0] = a.dim;
        d.nseg = 1;
        d.cols = a.hidden;
        d.rows_total = a.dim;
    }
    return d;
}

struct OpRange {
    int r_lo, rows_cnt;  // this CTA's rows
    int i_lo, i_hi;      // this warp's items, item = chunk * rows_cnt + local row
    int nchunks, nunits;
};

__device__ __forceinline__ OpRange op_range(int rows_total, int cols, int cta, int ncta, int warp) {
    OpRange r;
    r.nunits = cols / 64;
    r.nchunks = (r.nunits + 31) / 32;
    r.r_lo = int((long long)rows_total * cta / ncta);
    const int r_hi = int((long long)rows_total * (cta + 1) / ncta);
    r.rows_cnt = r_hi - r.r_lo;
    const int items = r.rows_cnt * r.nchunks;
    r.i_lo = items * warp / kTokWarps;
    r.i_hi = items * (warp + 1) / kTokWarps;
    return r;
}

// Lane 0: moves the warp's producer cursor to the next operator in which it has items.
template <int TYPE>
__device__ __noinline__ void producer_next_op(const TokArgs &a, const TokLayer *layers, WarpState *ws,
                                              int n_gemv, int warp) {
    for (int g = ws->g + 1; g < n_gemv; ++g) {
        const GemvDesc d = describe(a, layers, g);
        const OpRange r = op_range(d.rows_total, d.cols, blockIdx.x, gridDim.x, warp);
        if (r.i_hi > r.i_lo) {
            ws->g = g;
            ws->w[0] = d.w[0]; ws->w[1] = d.w[1]; ws->w[2] = d.w[2];
            ws->rows[0] = d.rows[0]; ws->rows[1] = d.rows[1]; ws->rows[2] = d.rows[2];
            ws->left = r.i_hi - r.i_lo;
            ws->chunk = r.i_lo / r.rows_cnt;
            ws->rl = r.i_lo - ws->chunk * r.rows_cnt;
            ws->e = 0;
            ws->r_lo = r.r_lo;
            ws->rows_cnt = r.rows_cnt;
            ws->nunits = r.nunits;
            ws->entries = d.gateup ? 2 : 1;
            ws->rowb = unsigned(r.nunits) * Fmt<TYPE>::unit_bytes;
            return;
        }
    }
    ws->g = n_gemv;
    ws->left = 0;
}

// Lane 0: requests the next ring entry (one row chunk) into `slot`. Requires ws->left > 0.
template <int TYPE>
__device__ __forceinline__ void produce(const TokArgs &a, const TokLayer *layers, WarpState *ws,
                                        uint64_t *bars, uint8_t *ring, int slot, uint64_t policy,
                                        int n_gemv, int warp) {
    constexpr int CB = Fmt<TYPE>::chunk_bytes;
    constexpr int UB = Fmt<TYPE>::unit_bytes;
    const int chunk = ws->chunk, rl = ws->rl, e = ws->e;
    int seg = e, row = ws->r_lo + rl;
    if (ws->entries == 1) {
        seg = 0;
        if (row >= ws->rows[0] && ws->w[1] != nullptr) {
            row -= ws->rows[0];
            seg = 1;
            if (row >= ws->rows[1]) {
                row -= ws->rows[1];
                seg = 2;
            }
        }
    }
    const int nun = min(32, ws->nunits - chunk * 32);
    const uint32_t bytes = uint32_t(nun) * UB;
    const uint8_t *src = ws->w[seg] + size_t(row) * ws->rowb + size_t(chunk) * CB;
    mbar_expect_tx(bars + slot, bytes);
    bulk_g2s_hint(ring + size_t(slot) * CB, src, bytes, bars + slot, policy);
    if (e + 1 < ws->entries) {
        ws->e = e + 1;
        return;
    }
    ws->e = 0;
    const int left = ws->left - 1;
    ws->left = left;
    if (rl + 1 == ws->rows_cnt) {
        ws->rl = 0;
        ws->chunk = chunk + 1;
    } else {
        ws->rl = rl + 1;
    }
    if (left == 0) producer_next_op<TYPE>(a, layers, ws, n_gemv, warp);
}

struct Epilogue {
    float *y[3];
    const float *res;  // nullable; only with one segment
    int track_argmax;
};

// One matrix-vector operator: stage the activation, consume this warp's items, fold the chunk
// partial sums and write the results.
template <int TYPE>
__device__ __noinline__ void gemv_phase(const TokArgs &a, const GemvDesc &d, const float *x,
                                        const float *norm_w, const Epilogue &ep, uint8_t *smem,
                                        int max_cols, int work_bytes, int ns, int n_gemv,
                                        unsigned long long *prof) {
    constexpr int CB = Fmt<TYPE>::chunk_bytes;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int cta = blockIdx.x, ncta = gridDim.x;
    uint64_t *bars = reinterpret_cast<uint64_t *>(smem) + warp * kTokMaxSlots;
    float *scratch = reinterpret_cast<float *>(smem + kBarBytes);
    WarpState *ws = reinterpret_cast<WarpState *>(smem + kBarBytes + kScratchBytes) + warp;
    const TokLayer *layers = reinterpret_cast<const TokLayer *>(smem + kBarBytes + kScratchBytes +
                                                                kTokWarps * sizeof(WarpState));
    uint8_t *work = smem + header_bytes(a.n_layers);
    float *sx = reinterpret_cast<float *>(work);
    float *sumx = sx + max_cols / 32;
    uint8_t *limbs = work + align_up(size_t(max_cols) / 32 * 8, 128);
    float *partial = reinterpret_cast<float *>(limbs + align_up(size_t(max_cols) * kLimbs, 128));
    uint8_t *ring = work + work_bytes + size_t(warp) * ns * CB;
    const uint32_t ring_u32 = smem_u32(ring), limbs_u32 = smem_u32(limbs);
    const uint32_t sx_u32 = smem_u32(sx), sumx_u32 = smem_u32(sumx);
    const uint64_t policy = policy_evict_first();

    const OpRange r = op_range(d.rows_total, d.cols, cta, ncta, warp);
    const int entries = d.gateup ? 2 : 1;
    stage_activation_core<kTokThreads>(x, norm_w, a.eps, d.cols, scratch, sx, sumx, limbs_u32);
    __syncthreads();
    if (prof) prof[1] = gtime();

    if (r.i_hi > r.i_lo) {
        int c_slot = ws->c_slot;
        uint32_t c_parity = uint32_t(ws->c_parity);
        int chunk = r.i_lo / r.rows_cnt;
        int rl = r.i_lo - chunk * r.rows_cnt;
        int cur_chunk = -1;
        UnitX ux;
        bool lane_on = false;
        bool failed = false;
        for (int i = r.i_lo; i < r.i_hi && !failed; ++i) {
            if (chunk != cur_chunk) {
                cur_chunk = chunk;
                const int unit = chunk * 32 + lane;
                lane_on = unit < r.nunits;
                if (lane_on) load_unit_x(limbs_u32, sx_u32, sumx_u32, r.nunits, unit, ux);
            }
            float v0 = 0.f, v1 = 0.f;
            for (int e = 0; e < entries; ++e) {
                bool ok = mbar_wait_bounded(bars + c_slot, c_parity);
                ok = __all_sync(0xffffffffu, ok);
                if (!ok) {
                    failed = true;
                    break;
                }
                float v = 0.f;
                if (lane_on) v = unit_dot<TYPE>(ring_u32 + uint32_t(c_slot) * CB, lane, ux);
                if (e == 0) v0 = v; else v1 = v;
                __syncwarp();
                if (lane == 0 && ws->left > 0) {
                    fence_proxy_async();
                    produce<TYPE>(a, layers, ws, bars, ring, c_slot, policy, n_gemv, warp);
                }
                if (++c_slot == ns) {
                    c_slot = 0;
                    c_parity ^= 1u;
                }
            }
            v0 = warp_sum(v0);
            if (entries == 2) v1 = warp_sum(v1);
            if (lane == 0) {
                partial[chunk * r.rows_cnt + rl] = v0;
                if (entries == 2) partial[(r.nchunks + chunk) * r.rows_cnt + rl] = v1;
            }
            if (++rl == r.rows_cnt) {
                rl = 0;
                ++chunk;
            }
        }
        if (lane == 0) {
            ws->c_slot = c_slot;
            ws->c_parity = int(c_parity);
        }
        if (failed && lane == 0) atomicExch(a.status, kDevTimeout);
    }
    __syncthreads();
    if (prof) prof[2] = gtime();

    // Chunk sums in chunk order, then the operator's epilogue.
    float best_v = -INFINITY;
    int best_i = INT_MAX;
    for (int idx = tid; idx < r.rows_cnt; idx += kTokThreads) {
        float s0 = 0.f;
        for (int c = 0; c < r.nchunks; ++c) s0 += partial[c * r.rows_cnt + idx];
        const int grow = r.r_lo + idx;
        if (d.gateup) {
            float s1 = 0.f;
            for (int c = 0; c < r.nchunks; ++c) s1 += partial[(r.nchunks + c) * r.rows_cnt + idx];
            const float silu = s0 / (1.0f + expf(-s0));
            ep.y[0][grow] = silu * s1;
        } else {
            int seg = 0, row = grow;
            if (d.nseg > 1 && row >= d.rows[0]) {
                row -= d.rows[0];
                seg = 1;
                if (d.nseg > 2 && row >= d.rows[1]) {
                    row -= d.rows[1];
                    seg = 2;
                }
            }
            float val = s0;
            if (ep.res != nullptr) val = __ldcg(ep.res + row) + val;
            ep.y[seg][row] = val;
            if (val > best_v || (val == best_v && row < best_i)) {
                best_v = val;
                best_i = row;
            }
        }
    }
    if (ep.track_argmax) {
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float ov = __shfl_xor_sync(0xffffffffu, best_v, o);
            const int oidx = __shfl_xor_sync(0xffffffffu, best_i, o);
            if (ov > best_v || (ov == best_v && oidx < best_i)) {
                best_v = ov;
                best_i = oidx;
            }
        }
        int *si = reinterpret_cast<int *>(scratch + 32);
        if (lane == 0) {
            scratch[warp] = best_v;
            si[warp] = best_i;
        }
        __syncthreads();
        if (tid == 0) {
            float fv = scratch[0];
            int fi = si[0];
            for (int w = 1; w < kTokWarps; ++w)
                if (scratch[w] > fv || (scratch[w] == fv && si[w] < fi)) {
                    fv = scratch[w];
                    fi = si[w];
                }
            a.amax_val[cta] = fv;
            a.amax_idx[cta] = fi;
        }
    }
    if (prof) prof[3] = gtime();
}

template <int HD, int G>
__device__ __noinline__ void attention_phase(const TokArgs &a, int layer, int pos, int slot, int nsplit,
                                             uint8_t *work) {
    constexpr int VEC = HD / 32;
    constexpr int UN = (G >= 8) ? 2 : 4;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int cta = blockIdx.x;
    const int kvh = cta % a.kv_heads, split = cta / a.kv_heads;
    if (split >= nsplit) return;
    float(*q_s)[HD] = reinterpret_cast<float(*)[HD]>(work);
    float(*red)[G][HD + 2] = reinterpret_cast<float(*)[G][HD + 2]>(work + size_t(G) * HD * 4);
    const int n = pos + 1;
    const int kv_dim = a.kv.kv_dim;
    const float *cr = a.rope_cos + size_t(pos) * (HD / 2);
    const float *ci = a.rope_sin + size_t(pos) * (HD / 2);
    for (int idx = tid; idx < G * (HD / 2); idx += kTokThreads) {
        const int g = idx / (HD / 2), i = idx - g * (HD / 2);
        const float2 qv = __ldcg(reinterpret_cast<const float2 *>(a.q + size_t(kvh * G + g) * HD) + i);
        q_s[g][2 * i] = __fsub_rn(__fmul_rn(qv.x, cr[i]), __fmul_rn(qv.y, ci[i]));
        q_s[g][2 * i + 1] = __fadd_rn(__fmul_rn(qv.x, ci[i]), __fmul_rn(qv.y, cr[i]));
    }
    const int chunk = (n + nsplit - 1) / nsplit;
    const int start = split * chunk;
    const int end = min(n, start + chunk);
    const int bt = a.kv.block_tokens;
    const int64_t block_stride = int64_t(a.kv.layers) * bt * kv_dim;
    const int64_t layer_off = int64_t(layer) * bt * kv_dim + int64_t(kvh) * HD;
    const int32_t *table = a.kv.block_table + int64_t(slot) * a.kv.blocks_per_slot;
    if (start <= pos && pos < end) {
        const int64_t off = int64_t(table[pos / bt]) * block_stride + layer_off + int64_t(pos % bt) * kv_dim;
        const float *kh = a.k + size_t(kvh) * HD;
        const float *vh = a.v + size_t(kvh) * HD;
        for (int i = tid; i < HD / 2; i += kTokThreads) {
            const float2 kvv = __ldcg(reinterpret_cast<const float2 *>(kh) + i);
            const float2 vvv = __ldcg(reinterpret_cast<const float2 *>(vh) + i);
            const float r0 = __fsub_rn(__fmul_rn(kvv.x, cr[i]), __fmul_rn(kvv.y, ci[i]));
            const float r1 = __fadd_rn(__fmul_rn(kvv.x, ci[i]), __fmul_rn(kvv.y, cr[i]));
            *reinterpret_cast<__half2 *>(a.kv.kpool + off + 2 * i) =
                __halves2half2(__float2half_rn(r0), __float2half_rn(r1));
            *reinterpret_cast<__half2 *>(a.kv.vpool + off + 2 * i) =
                __halves2half2(__float2half_rn(vvv.x), __float2half_rn(vvv.y));
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
    const int per_warp = (end - start + kTokWarps - 1) / kTokWarps;
    const int w0 = start + warp * per_warp;
    const int w1 = min(end, w0 + per_warp);
    for (int t0 = w0; t0 < w1; t0 += UN) {
        float kf[UN][VEC], vf[UN][VEC];
#pragma unroll
        for (int u = 0; u < UN; ++u) {
            const int t = min(t0 + u, w1 - 1);
            const int64_t off = int64_t(table[t / bt]) * block_stride + layer_off +
                                int64_t(t % bt) * kv_dim + lane * VEC;
            load_halfs<VEC>(a.kv.kpool + off, kf[u]);
            load_halfs<VEC>(a.kv.vpool + off, vf[u]);
        }
#pragma unroll
        for (int g = 0; g < G; ++g) {
            float s[UN];
#pragma unroll
            for (int u = 0; u < UN; ++u) {
                float dsum = 0.f;
#pragma unroll
                for (int j = 0; j < VEC; ++j) dsum += qr[g][j] * kf[u][j];
                s[u] = dsum;
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
                const float p = expf(s[u] - mn);
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
    for (int idx = tid; idx < G * HD; idx += kTokThreads) {
        const int g = idx / HD, dd = idx - g * HD;
        float M = -INFINITY;
#pragma unroll
        for (int w = 0; w < kTokWarps; ++w) M = fmaxf(M, red[w][g][HD]);
        float val = 0.f, L = 0.f;
#pragma unroll
        for (int w = 0; w < kTokWarps; ++w) {
            const float mw = red[w][g][HD];
            const float wgt = (mw == -INFINITY) ? 0.f : expf(mw - M);
            val += red[w][g][dd] * wgt;
            L += red[w][g][HD + 1] * wgt;
        }
        const int h = kvh * G + g;
        if (nsplit == 1) {
            a.xb[size_t(h) * HD + dd] = val / L;
        } else {
            float *p = a.partial + (size_t(h) * a.max_splits + split) * pstride;
            p[dd] = val;
            if (dd == 0) {
                p[HD] = M;
                p[HD + 1] = L;
            }
        }
    }
}

template <int HD>
__device__ __noinline__ void attention_fold(const TokArgs &a, int nsplit) {
    // CTA h folds head h: every thread recomputes the (tiny) split weights, then one output each.
    const int h = blockIdx.x;
    if (h >= a.heads) return;
    const size_t pstride = size_t(HD + 2);
    const float *p = a.partial + size_t(h) * a.max_splits * pstride;
    for (int d = threadIdx.x; d < HD; d += kTokThreads) {
        float M = -INFINITY;
        for (int s = 0; s < nsplit; ++s) M = fmaxf(M, __ldcg(p + s * pstride + HD));
        float val = 0.f, L = 0.f;
        for (int s = 0; s < nsplit; ++s) {
            const float ms = __ldcg(p + s * pstride + HD);
            const float w = (ms == -INFINITY) ? 0.f : expf(ms - M);
            val += __ldcg(p + s * pstride + d) * w;
            L += __ldcg(p + s * pstride + HD + 1) * w;
        }
        a.xb[size_t(h) * HD + d] = val / L;
    }
}

template <int TYPE, int HD, int G>
__global__ void __launch_bounds__(kTokThreads, 1)
token_kernel(const TokArgs a, const int ns, const int max_cols, const int work_bytes) {
    extern __shared__ __align__(128) uint8_t smem[];
    constexpr int CB = Fmt<TYPE>::chunk_bytes;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int cta = blockIdx.x, ncta = gridDim.x;

    uint64_t *bars = reinterpret_cast<uint64_t *>(smem) + warp * kTokMaxSlots;
    WarpState *ws = reinterpret_cast<WarpState *>(smem + kBarBytes + kScratchBytes) + warp;
    TokLayer *layers = reinterpret_cast<TokLayer *>(smem + kBarBytes + kScratchBytes +
                                                    kTokWarps * sizeof(WarpState));
    uint8_t *work = smem + header_bytes(a.n_layers);
    uint8_t *ring = work + work_bytes + size_t(warp) * ns * CB;

    // Layer table into shared memory (9 pointers per layer).
    {
        const uint64_t *src = reinterpret_cast<const uint64_t *>(a.layers);
        uint64_t *dst = reinterpret_cast<uint64_t *>(layers);
        const int words = a.n_layers * int(sizeof(TokLayer) / 8);
        for (int i = tid; i < words; i += kTokThreads) dst[i] = src[i];
    }
    __syncthreads();

    const int n_gemv = 4 * a.n_layers + (a.with_logits ? 1 : 0);
    const uint64_t policy = policy_evict_first();
    if (lane == 0) {
        for (int s = 0; s < ns; ++s) mbar_init(bars + s, 1);
        mbar_fence_init();
        fence_proxy_async();
        ws->g = -1;
        ws->c_slot = 0;
        ws->c_parity = 0;
        producer_next_op<TYPE>(a, layers, ws, n_gemv, warp);
        for (int s = 0; s < ns && ws->left > 0; ++s)
            produce<TYPE>(a, layers, ws, bars, ring, s, policy, n_gemv, warp);
    }
    __syncwarp();

    const int pos = a.positions[0];
    const int slot = a.slots[0];
    const int n_keys = pos + 1;
    const int nsplit = (n_keys <= 256) ? 1 : min(a.max_splits, (n_keys + 127) / 128);
    unsigned syncs = 0;
    unsigned long long *prof0 = (a.profile != nullptr && cta == 0 && tid == 0) ? a.profile : nullptr;

    // ---- embedding
    {
        if (prof0) prof0[0] = gtime();
        const int token = a.tokens[0];
        for (int i = cta * kTokThreads + tid; i < a.dim; i += ncta * kTokThreads)
            a.x[i] = decode_any(a.emb_type, a.emb, int64_t(token) * a.dim + i);
        if (prof0) prof0[3] = gtime();
        grid_sync(a.barrier, ++syncs * ncta, a.status);
        if (prof0) prof0[4] = gtime();
    }
    for (int l = 0; l < a.n_layers; ++l) {
        unsigned long long *pf = prof0 ? prof0 + (1 + 6 * l) * 5 : nullptr;
        {   // RMSNorm + QKV
            if (pf) pf[0] = gtime();
            const GemvDesc d = describe(a, layers, 4 * l);
            const Epilogue ep = {{a.q, a.k, a.v}, nullptr, 0};
            gemv_phase<TYPE>(a, d, a.x, layers[l].attn_norm, ep, smem, max_cols, work_bytes, ns, n_gemv, pf);
            grid_sync(a.barrier, ++syncs * ncta, a.status);
            if (pf) pf[4] = gtime();
        }
        {   // RoPE + KV append + attention
            if (pf) pf[5] = gtime();
            attention_phase<HD, G>(a, l, pos, slot, nsplit, work);
            if (pf) pf[8] = gtime();
            grid_sync(a.barrier, ++syncs * ncta, a.status);
            if (pf) pf[9] = gtime();
            if (nsplit > 1) {
                if (pf) pf[10] = gtime();
                attention_fold<HD>(a, nsplit);
                if (pf) pf[13] = gtime();
                grid_sync(a.barrier, ++syncs * ncta, a.status);
                if (pf) pf[14] = gtime();
            }
        }
        {   // output projection + residual
            if (pf) pf[15] = gtime();
            const GemvDesc d = describe(a, layers, 4 * l + 1);
            const Epilogue ep = {{a.x, nullptr, nullptr}, a.x, 0};
            gemv_phase<TYPE>(a, d, a.xb, nullptr, ep, smem, max_cols, work_bytes, ns, n_gemv,
                             pf ? pf + 15 : nullptr);
            grid_sync(a.barrier, ++syncs * ncta, a.status);
            if (pf) pf[19] = gtime();
        }
        {   // RMSNorm + gate/up + SwiGLU
            if (pf) pf[20] = gtime();
            const GemvDesc d = describe(a, layers, 4 * l + 2);
            const Epilogue ep = {{a.hb, nullptr, nullptr}, nullptr, 0};
            gemv_phase<TYPE>(a, d, a.x, layers[l].ffn_norm, ep, smem, max_cols, work_bytes, ns, n_gemv,
                             pf ? pf + 20 : nullptr);
            grid_sync(a.barrier, ++syncs * ncta, a.status);
            if (pf) pf[24] = gtime();
        }
        {   // down projection + residual
            if (pf) pf[25] = gtime();
            const GemvDesc d = describe(a, layers, 4 * l + 3);
            const Epilogue ep = {{a.x, nullptr, nullptr}, a.x, 0};
            gemv_phase<TYPE>(a, d, a.hb, nullptr, ep, smem, max_cols, work_bytes, ns, n_gemv,
                             pf ? pf + 25 : nullptr);
            grid_sync(a.barrier, ++syncs * ncta, a.status);
            if (pf) pf[29] = gtime();
        }
    }
    if (a.with_logits) {
        unsigned long long *pf = prof0 ? prof0 + (1 + 6 * a.n_layers) * 5 : nullptr;
        if (pf) pf[0] = gtime();
        const GemvDesc d = describe(a, layers, 4 * a.n_layers);
        const Epilogue ep = {{a.logits, nullptr, nullptr}, nullptr, 1};
        gemv_phase<TYPE>(a, d, a.x, a.out_norm, ep, smem, max_cols, work_bytes, ns, n_gemv, pf);
        grid_sync(a.barrier, ++syncs * ncta, a.status);
        if (pf) pf[4] = gtime();
        if (cta == 0 && tid == 0) {
            float fv = -INFINITY;
            int fi = INT_MAX;
            for (int b = 0; b < ncta; ++b) {
                const float ov = __ldcg(a.amax_val + b);
                const int oidx = __ldcg(a.amax_idx + b);
                if (ov > fv || (ov == fv && oidx < fi)) {
                    fv = ov;
                    fi = oidx;
                }
            }
            const int tok = (fi == INT_MAX) ? 0 : fi;
            *a.out_token = tok;
            if (a.advance) {
                const int step = *a.step_counter;
                a.history[step] = tok;
                a.tokens[0] = tok;
                a.positions[0] = pos + 1;
                *a.step_counter = step + 1;
            }
        }
    }
}

template <int TYPE, int HD, int G>
cudaError_t configure_tok() {
    return cudaFuncSetAttribute(token_kernel<TYPE, HD, G>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                227 * 1024);
}

struct TokPlan {
    int ns;
    int work_bytes;
    size_t smem;
};

bool plan_tok(int type, int hd, int g, int max_cols, int n_layers, TokPlan *p) {
    if (!is_quant(type) || max_cols <= 0 || max_cols % 256 != 0 || n_layers > kMaxLayers) return false;
    const int cb = 32 * (type == kQ8_0 ? kUnitBytesQ8 : kUnitBytesQ4);
    size_t work = stage_region_bytes(max_cols);
    const size_t attn = attn_region_bytes(hd, g);
    if (attn > work) work = attn;
    work = align_up(work, 128);
    const size_t fixed = header_bytes(n_layers) + work;
    const size_t limit = 226 * 1024;
    if (fixed + size_t(kTokWarps) * 2 * cb > limit) return false;
    int ns = int((limit - fixed) / (size_t(kTokWarps) * cb));
    if (ns > kTokMaxSlots) ns = kTokMaxSlots;
    p->ns = ns;
    p->work_bytes = int(work);
    p->smem = fixed + size_t(kTokWarps) * ns * cb;
    return true;
}

template <int TYPE, int HD, int G>
cudaError_t launch_tok(const TokArgs &args, const TokPlan &plan, int max_cols, int sm_count,
                       cudaStream_t stream) {
    TokArgs a = args;
    int ns = plan.ns, mc = max_cols, wb = plan.work_bytes;
    void *params[] = {&a, &ns, &mc, &wb};
    return cudaLaunchCooperativeKernel(reinterpret_cast<void *>(token_kernel<TYPE, HD, G>), dim3(sm_count),
                                       dim3(kTokThreads), params, plan.smem, stream);
}

template <int TYPE>
cudaError_t launch_tok_type(int hd, int g, const TokArgs &a, const TokPlan &p, int mc, int sms,
                            cudaStream_t s) {
    if (hd == 128 && g == 4) return launch_tok<TYPE, 128, 4>(a, p, mc, sms, s);
    if (hd == 64 && g == 4) return launch_tok<TYPE, 64, 4>(a, p, mc, sms, s);
    if (hd == 128 && g == 8) return launch_tok<TYPE, 128, 8>(a, p, mc, sms, s);
    if (hd == 64 && g == 2) return launch_tok<TYPE, 64, 2>(a, p, mc, sms, s);
    return cudaErrorInvalidValue;
}

template <int TYPE>
cudaError_t configure_tok_type() {
    cudaError_t e;
    if ((e = configure_tok<TYPE, 128, 4>()) != cudaSuccess) return e;
    if ((e = configure_tok<TYPE, 64, 4>()) != cudaSuccess) return e;
    if ((e = configure_tok<TYPE, 128, 8>()) != cudaSuccess) return e;
    if ((e = configure_tok<TYPE, 64, 2>()) != cudaSuccess) return e;
    return cudaSuccess;
}

}  // namespace

bool token_kernel_supported(int type, int head_dim, int group, int dim, int hidden, int kv_dim,
                            int vocab, int heads, int kv_heads, int n_layers, int sm_count) {
    const bool geom = (head_dim == 128 && (group == 4 || group == 8)) ||
                      (head_dim == 64 && (group == 4 || group == 2));
    if (!geom || sm_count <= 0 || heads > sm_count || kv_heads > sm_count) return false;
    TokPlan p;
    const int max_cols = dim > hidden ? dim : hidden;
    if (!plan_tok(type, head_dim, group, max_cols, n_layers, &p)) return false;
    auto fits = [&](int rows_total, int cols, int entries) {
        const long long rows_cta = (rows_total + sm_count - 1) / sm_count + 1;
        const int nchunks = (cols / 64 + 31) / 32;
        return rows_cta * nchunks * entries <= kPartialFloats;
    };
    return fits(dim + 2 * kv_dim, dim, 1) && fits(hidden, dim, 2) && fits(dim, hidden, 1) &&
           fits(vocab, dim, 1);
}

int token_kernel_op_count(int n_layers) { return 2 + 6 * n_layers; }

cudaError_t token_kernel_configure() {
    cudaError_t e;
    if ((e = configure_tok_type<kQ4_K>()) != cudaSuccess) return e;
    if ((e = configure_tok_type<kQ4_0>()) != cudaSuccess) return e;
    if ((e = configure_tok_type<kQ8_0>()) != cudaSuccess) return e;
    return cudaSuccess;
}

cudaError_t token_kernel_launch(int type, int head_dim, int group, const TokArgs &args, int sm_count,
                                cudaStream_t stream) {
    TokPlan p;
    const int max_cols = args.dim > args.hidden ? args.dim : args.hidden;
    if (!plan_tok(type, head_dim, group, max_cols, args.n_layers, &p)) return cudaErrorInvalidValue;
    switch (type) {
        case kQ4_K: return launch_tok_type<kQ4_K>(head_dim, group, args, p, max_cols, sm_count, stream);
        case kQ4_0: return launch_tok_type<kQ4_0>(head_dim, group, args, p, max_cols, sm_count, stream);
        case kQ8_0: return launch_tok_type<kQ8_0>(head_dim, group, args, p, max_cols, sm_count, stream);
        default: return cudaErrorInvalidValue;
    }
}

}  // namespace jl
