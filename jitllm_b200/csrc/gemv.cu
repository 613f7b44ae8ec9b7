// Dequant-fused quantised matrix-vector product for single-token decode on sm_100a.
//
// What it computes: FloatTensor.matmul of the reference (tensor/standard/FloatTensor.java:123-125)
// for Q8_0 / Q4_0 / Q4_K weights kept in GGUF block layout, optionally with the RMSNorm of the
// input (inference/op/CpuOperations.java:55-73), a residual add (:369-371), SwiGLU over a
// gate/up pair (:255-260) or the greedy argmax (inference/Logits.java:49-60) folded in.
//
// How: the kernel is HBM-bound, so the design goal is "every weight byte crosses HBM once, in
// large aligned bursts, with few issue slots spent per weight":
//   * weights: each warp owns a ring of shared-memory stages that one lane fills with 1-D bulk
//     async copies (cp.async.bulk, the TMA engine) completing on an mbarrier; a stage holds the
//     same 2048-column chunk of R consecutive rows. No registers are tied up by loads in flight.
//   * activations: quantised once per CTA into three signed 7-bit digits per element
//     (x ~ s_blk * (a1*2^14 + a2*2^7 + a3), error <= 2^-21 of the block maximum, i.e. at the
//     level of fp32 rounding itself) so that the inner product of 4 weights is 3 dp4a
//     instructions on the packed integer weights instead of 4 unpack + 4 convert + 4 FMA.
//     Integer sums are exact; block results are scaled and accumulated in fp32.
//   * a lane works on a 64-element unit (a Q4_K nibble pair of sub-blocks, or two Q4_0 / Q8_0
//     blocks) and keeps its activation digits in registers across the R rows of the tile.
//   * the kernel prefetches its first stages before griddepcontrol.wait, so under programmatic
//     dependent launch the weight stream of kernel N+1 starts while kernel N drains.
#include "gemv_core.cuh"

#include <climits>
#include <cstdlib>

namespace jl {

namespace {

constexpr int kThreads = 512;
constexpr int kWarps = kThreads / 32;
constexpr int kMaxStages = 16;
constexpr int kHeaderBytes = 2176;  // mbarriers (16 warps x 16 stages x 8 B) + 128 B scratch
struct SmemLayout {
    uint64_t *bars;
    float *scratch;  // 32 floats
    float *sx, *sumx;
    uint8_t *limbs;
    uint8_t *ring;
};

__device__ __forceinline__ SmemLayout carve(uint8_t *smem, int cols) {
    SmemLayout l;
    l.bars = reinterpret_cast<uint64_t *>(smem);
    l.scratch = reinterpret_cast<float *>(smem + 2048);
    l.sx = reinterpret_cast<float *>(smem + kHeaderBytes);
    l.sumx = l.sx + cols / 32;
    l.limbs = smem + kHeaderBytes + align_up(size_t(cols) / 32 * 8, 128);
    l.ring = smem + kHeaderBytes + x_region_bytes(cols);
    return l;
}

__device__ void stage_activation(const GemvArgs &a, const SmemLayout &sm) {
    stage_activation_core<kThreads>(a.x, a.norm_w, a.eps, a.cols, sm.scratch, sm.sx, sm.sumx,
                                    smem_u32(sm.limbs));
}

template <int TYPE, int R, int MODE>
__global__ void __launch_bounds__(kThreads, 1) gemv_kernel(const GemvArgs a, const int stages) {
    extern __shared__ __align__(128) uint8_t smem[];
    constexpr int NR = (MODE == kGemvGateUp) ? 2 * R : R;
    constexpr int CB = Fmt<TYPE>::chunk_bytes;
    constexpr int UB = Fmt<TYPE>::unit_bytes;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int nunits = a.cols / 64;
    const int nchunks = (nunits + 31) / 32;
    const size_t rowb = size_t(a.cols) / 64 * UB;
    if (a.active != nullptr && *a.active == 0) {
        // Still wait: a grid that finished without waiting would let its successor run ahead of
        // the grid before this one.
        pdl_wait();
        return;
    }
    const SmemLayout sm = carve(smem, a.cols);
    const int stage_bytes = NR * CB;
    uint8_t *my_ring = sm.ring + size_t(warp) * stages * stage_bytes;
    uint64_t *my_bars = sm.bars + warp * kMaxStages;
    const uint32_t ring_u32 = smem_u32(my_ring);
    const uint32_t limbs_u32 = smem_u32(sm.limbs), sx_u32 = smem_u32(sm.sx), sumx_u32 = smem_u32(sm.sumx);

    // Tiles of R rows, numbered segment after segment; gate/up tiles pair the same rows.
    const int nseg_tiled = (MODE == kGemvGateUp) ? 1 : a.nseg;
    const int t0 = (a.seg[0].rows + R - 1) / R;
    const int t1 = nseg_tiled > 1 ? (a.seg[1].rows + R - 1) / R : 0;
    const int t2 = nseg_tiled > 2 ? (a.seg[2].rows + R - 1) / R : 0;
    const int total_tiles = t0 + t1 + t2;
    const int total_warps = kWarps * gridDim.x;
    const int wg = warp * gridDim.x + blockIdx.x;
    const int n_my = total_tiles > wg ? (total_tiles - wg - 1) / total_warps + 1 : 0;
    const int n_items = n_my * nchunks;

    auto locate = [&](int tile, int &seg, int &row0) {
        seg = 0;
        if (tile >= t0) {
            tile -= t0;
            seg = 1;
            if (tile >= t1) {
                tile -= t1;
                seg = 2;
            }
        }
        row0 = tile * R;
    };
    const uint64_t policy = policy_evict_first();
    // Producer cursor (lane 0): the next item to request, advanced incrementally; source pointers
    // move by one chunk per item and are recomputed only when the cursor enters a new tile.
    int p_tile = wg, p_cc = 0, p_seg = 0, p_row0 = 0, p_issued = 0, p_rows = 0;
    const uint8_t *p_src0 = nullptr, *p_src1 = nullptr;
    auto enter_tile = [&]() {
        locate(p_tile, p_seg, p_row0);
        p_rows = min(R, a.seg[p_seg].rows - p_row0);
        p_src0 = a.seg[p_seg].w + size_t(p_row0) * rowb;
        if (MODE == kGemvGateUp) p_src1 = a.seg[1].w + size_t(p_row0) * rowb;
    };
    if (n_items > 0) enter_tile();
    const uint32_t bars_u32 = smem_u32(my_bars);
    const uint32_t last_bytes = uint32_t(nunits - (nchunks - 1) * 32) * UB;
    auto issue = [&](int s) {  // lane 0 only
        const uint32_t bytes = p_cc == nchunks - 1 ? last_bytes : uint32_t(CB);
        const uint32_t stage = ring_u32 + uint32_t(s) * stage_bytes;
        const uint32_t bar = bars_u32 + uint32_t(s) * 8u;
        mbar_expect_tx_u32(bar, bytes * p_rows * (MODE == kGemvGateUp ? 2 : 1));
        const uint8_t *src0 = p_src0, *src1 = p_src1;
#pragma unroll
        for (int r = 0; r < R; ++r) {
            if (r < p_rows) {
                bulk_g2s_hint_u32(stage + r * CB, src0, bytes, bar, policy);
                if (MODE == kGemvGateUp) bulk_g2s_hint_u32(stage + (R + r) * CB, src1, bytes, bar, policy);
                src0 += rowb;
                if (MODE == kGemvGateUp) src1 += rowb;
            }
        }
        ++p_issued;
        p_src0 += CB;
        if (MODE == kGemvGateUp) p_src1 += CB;
        if (++p_cc == nchunks) {
            p_cc = 0;
            p_tile += total_warps;
            if (p_tile < total_tiles) enter_tile();
        }
    };

    if (lane == 0) {
        for (int s = 0; s < stages; ++s) mbar_init(my_bars + s, 1);
        mbar_fence_init();
        fence_proxy_async();
        const int first = a.debug == 2 ? 0 : min(stages, n_items);
        for (int it = 0; it < first; ++it) issue(it);
    }
    __syncwarp();

    // Everything above touches only weights, which no earlier kernel writes.
    pdl_wait();
    stage_activation(a, sm);
    __syncthreads();
    pdl_launch_dependents();

    float acc[NR];
#pragma unroll
    for (int r = 0; r < NR; ++r) acc[r] = 0.f;
    float best_v = -INFINITY;
    int best_i = INT_MAX;
    bool failed = false;
    int cc = 0, tk = 0, s = 0;
    uint32_t parity = 0;
    for (int it = 0; it < n_items; ++it) {
        bool ok = a.debug == 2 ? true : mbar_wait_bounded(my_bars + s, parity);
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) {
            failed = true;
            break;
        }
        const uint32_t stage = ring_u32 + uint32_t(s) * stage_bytes;
        const int unit = cc * 32 + lane;
        if (unit < nunits && a.debug != 1) {
            UnitX x;
            load_unit_x(limbs_u32, sx_u32, sumx_u32, nunits, unit, x);
#pragma unroll
            for (int r = 0; r < NR; ++r) acc[r] += unit_dot<TYPE>(stage + r * CB, lane, x);
        }
        __syncwarp();
        if (lane == 0 && p_issued < n_items && a.debug != 2) {
            fence_proxy_async();
            issue(s);
        }
        if (++s == stages) {
            s = 0;
            parity ^= 1u;
        }
        if (++cc == nchunks) {
            cc = 0;
            int seg, row0;
            locate(wg + tk * total_warps, seg, row0);
            ++tk;
            const int nrows = min(R, a.seg[seg].rows - row0);
#pragma unroll
            for (int r = 0; r < NR; ++r) acc[r] = warp_sum(acc[r]);
            if (MODE == kGemvGateUp) {
#pragma unroll
                for (int r = 0; r < R; ++r) {
                    if (r < nrows && lane == r) {
                        const float g = acc[r], u = acc[R + r];
                        const float silu = g / (1.0f + expf(-g));
                        a.seg[0].y[row0 + r] = silu * u;
                    }
                }
            } else {
#pragma unroll
                for (int r = 0; r < R; ++r) {
                    if (r < nrows) {
                        float v = acc[r];
                        if (a.seg[seg].res != nullptr) v = a.seg[seg].res[row0 + r] + v;
                        if (lane == r) a.seg[seg].y[row0 + r] = v;
                        if (v > best_v || (v == best_v && row0 + r < best_i)) {
                            best_v = v;
                            best_i = row0 + r;
                        }
                    }
                }
            }
#pragma unroll
            for (int r = 0; r < NR; ++r) acc[r] = 0.f;
        }
    }
    if (failed) {
        // Give copies already in flight a bounded chance to land before this CTA's shared memory
        // is released, then report; the host turns the status word into an error.
        for (int s = 0; s < stages; ++s) mbar_wait_bounded(my_bars + s, 0, 16);
        if (lane == 0) atomicExch(a.status, kDevTimeout);
    }

    if (a.argmax_val != nullptr) {
        // Block-level then grid-level reduction of (value, first index).
        __syncthreads();
        float *bv = sm.scratch;
        int *bi = reinterpret_cast<int *>(sm.scratch + kWarps);
        if (lane == 0) {
            bv[warp] = best_v;
            bi[warp] = best_i;
        }
        __syncthreads();
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
}

template <int TYPE, int R, int MODE>
cudaError_t configure_one() {
    return cudaFuncSetAttribute(gemv_kernel<TYPE, R, MODE>,
                                cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024);
}

template <int TYPE, int R, int MODE>
cudaError_t launch_one(const GemvArgs &args, const GemvPlan &plan, cudaStream_t stream,
                       bool programmatic) {
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
    return cudaLaunchKernelEx(&cfg, gemv_kernel<TYPE, R, MODE>, args, plan.stages);
}

template <int TYPE, int MODE>
cudaError_t launch_r(const GemvArgs &a, const GemvPlan &p, cudaStream_t s, bool pdl) {
    switch (p.rows_per_tile) {
        case 4: return launch_one<TYPE, 4, MODE>(a, p, s, pdl);
        case 2: return launch_one<TYPE, 2, MODE>(a, p, s, pdl);
        default: return launch_one<TYPE, 1, MODE>(a, p, s, pdl);
    }
}
template <int TYPE>
cudaError_t launch_mode(const GemvArgs &a, const GemvPlan &p, cudaStream_t s, bool pdl) {
    if (a.mode == kGemvGateUp) {
        // Gate/up tiles hold twice the rows; height 4 is not instantiated for them.
        if (p.rows_per_tile == 2) return launch_one<TYPE, 2, kGemvGateUp>(a, p, s, pdl);
        return launch_one<TYPE, 1, kGemvGateUp>(a, p, s, pdl);
    }
    return launch_r<TYPE, kGemvPlain>(a, p, s, pdl);
}

template <int TYPE>
cudaError_t configure_type() {
    cudaError_t e;
    if ((e = configure_one<TYPE, 1, kGemvPlain>()) != cudaSuccess) return e;
    if ((e = configure_one<TYPE, 2, kGemvPlain>()) != cudaSuccess) return e;
    if ((e = configure_one<TYPE, 4, kGemvPlain>()) != cudaSuccess) return e;
    if ((e = configure_one<TYPE, 1, kGemvGateUp>()) != cudaSuccess) return e;
    if ((e = configure_one<TYPE, 2, kGemvGateUp>()) != cudaSuccess) return e;
    return cudaSuccess;
}

}  // namespace

bool gemv_plan(int type, int cols, int total_rows, int mode, int sm_count, GemvPlan *out) {
    if (!is_quant(type) || cols <= 0 || cols % 256 != 0 || total_rows <= 0) return false;
    const int chunk = 32 * (type == kQ8_0 ? kUnitBytesQ8 : kUnitBytesQ4);
    const size_t fixed = kHeaderBytes + x_region_bytes(cols);
    // One CTA of 16 warps per SM; most of the SM's shared memory goes to the weight rings.
    static const int env_kb = [] {
        const char *v = getenv("JITLLM_B200_GEMV_SMEM_KB");
        return v ? atoi(v) : 0;
    }();
    size_t budget = size_t(env_kb > 0 ? env_kb : 208) * 1024;
    if (budget > 224 * 1024) budget = 224 * 1024;
    if (fixed + size_t(kWarps) * 2 * chunk > budget) budget = 224 * 1024;
    if (fixed + size_t(kWarps) * 2 * chunk > budget) return false;
    static const int env_mult = [] {
        const char *v = getenv("JITLLM_B200_GEMV_GRID_MULT");
        return v ? atoi(v) : 1;
    }();
    static const int env_r = [] {
        const char *v = getenv("JITLLM_B200_GEMV_ROWS");
        return v ? atoi(v) : 0;
    }();
    const int grid = sm_count * (env_mult > 0 ? env_mult : 1);
    const int warps = grid * kWarps;
    const int mult = (mode == kGemvGateUp) ? 2 : 1;
    int best_r = 1, best_s = 0;
    int rmax = (mode == kGemvGateUp) ? 2 : 4;
    if (env_r > 0 && env_r < rmax) rmax = env_r;
    for (int r = rmax; r >= 1; r >>= 1) {
        // Taller tiles reuse the activation registers more, but leave warps idle on short matrices.
        if (r > 1 && (total_rows / mult + r - 1) / r < warps) continue;
        const size_t stage = size_t(r) * mult * chunk;
        int s = static_cast<int>((budget - fixed) / (size_t(kWarps) * stage));
        if (s > kMaxStages) s = kMaxStages;
        if (s >= 2) {
            best_r = r;
            best_s = s;
            break;
        }
    }
    if (best_s < 2) {
        const size_t stage = size_t(mult) * chunk;
        best_r = 1;
        best_s = static_cast<int>((budget - fixed) / (size_t(kWarps) * stage));
        if (best_s > kMaxStages) best_s = kMaxStages;
        if (best_s < 2) return false;
    }
    out->rows_per_tile = best_r;
    out->stages = best_s;
    out->grid = grid;
    out->smem_bytes = fixed + size_t(kWarps) * best_s * best_r * mult * chunk;
    return true;
}

cudaError_t gemv_configure() {
    cudaError_t e;
    if ((e = configure_type<kQ4_K>()) != cudaSuccess) return e;
    if ((e = configure_type<kQ4_0>()) != cudaSuccess) return e;
    if ((e = configure_type<kQ8_0>()) != cudaSuccess) return e;
    return cudaSuccess;
}

cudaError_t gemv_launch(const GemvArgs &args, const GemvPlan &plan, cudaStream_t stream,
                        bool programmatic) {
    switch (args.type) {
        case kQ4_K: return launch_mode<kQ4_K>(args, plan, stream, programmatic);
        case kQ4_0: return launch_mode<kQ4_0>(args, plan, stream, programmatic);
        case kQ8_0: return launch_mode<kQ8_0>(args, plan, stream, programmatic);
        default: return cudaErrorInvalidValue;
    }
}

}  // namespace jl
