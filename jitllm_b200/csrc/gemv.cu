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
#include "gemv.cuh"

#include <climits>
#include <cstdlib>

namespace jl {

namespace {

constexpr int kThreads = 512;
constexpr int kWarps = kThreads / 32;
constexpr int kMaxStages = 16;
constexpr int kHeaderBytes = 2176;  // mbarriers (16 warps x 16 stages x 8 B) + 128 B scratch
constexpr int kUnitBytesQ4 = 36;   // 64 elements: Q4_K 144/4, Q4_0 2*18
constexpr int kUnitBytesQ8 = 68;   // 64 elements: Q8_0 2*34

template <int TYPE>
struct Fmt {
    static constexpr int unit_bytes = (TYPE == kQ8_0) ? kUnitBytesQ8 : kUnitBytesQ4;
    static constexpr int chunk_bytes = 32 * unit_bytes;  // 32 lanes x one unit
};

__device__ __forceinline__ int dp4a_u8s8(uint32_t a, int b, int c) {
    int d;
    asm("dp4a.u32.s32 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(c));
    return d;
}
__device__ __forceinline__ int dp4a_s8s8(int a, int b, int c) {
    int d;
    asm("dp4a.s32.s32 %0, %1, %2, %3;" : "=r"(d) : "r"(a), "r"(b), "r"(c));
    return d;
}

// Activation digits of one 64-element unit: [digit][word], words 0..7 = first 32-block.
struct UnitX {
    int a[kLimbs][8];
    int b[kLimbs][8];
    float sa, sb;    // block scales
    float ma, mb;    // block sums of the quantised activation (s * sum X)
};

// ---- one unit of one row: returns sum_{64 el} w * x -------------------------------------------

// Q4_K: the unit is nibble pair p of super-block (lane/4): 32 qs bytes whose low nibbles are
// sub-block 2p and high nibbles sub-block 2p+1 (tensor/standard/Q4_KFloatTensor.java:88-122).
__device__ __forceinline__ float unit_q4_k(const uint8_t *chunk, int lane, const UnitX &x) {
    const uint8_t *sb = chunk + (lane >> 2) * kQ4_KBytes;
    const int p = lane & 3;
    const uint4 hdr = *reinterpret_cast<const uint4 *>(sb);
    const uint4 q0 = *reinterpret_cast<const uint4 *>(sb + 16 + p * 32);
    const uint4 q1 = *reinterpret_cast<const uint4 *>(sb + 32 + p * 32);
    const float d = half_bits_to_float(hdr.x & 0xFFFFu);
    const float dmin = half_bits_to_float(hdr.x >> 16);
    // 6-bit scales / mins of all eight sub-blocks as bytes: sub-blocks 0-3 in *A, 4-7 in *B.
    const uint32_t scA = hdr.y & 0x3F3F3F3Fu, mA = hdr.z & 0x3F3F3F3Fu;
    const uint32_t scB = (hdr.w & 0x0F0F0F0Fu) | ((hdr.y >> 2) & 0x30303030u);
    const uint32_t mB = ((hdr.w >> 4) & 0x0F0F0F0Fu) | ((hdr.z >> 2) & 0x30303030u);
    const int sh = (p & 1) * 16;
    const uint32_t scw = ((p < 2) ? scA : scB) >> sh;
    const uint32_t mw = ((p < 2) ? mA : mB) >> sh;
    const float sc0 = static_cast<float>(scw & 0xFFu), sc1 = static_cast<float>((scw >> 8) & 0xFFu);
    const float m0 = static_cast<float>(mw & 0xFFu), m1 = static_cast<float>((mw >> 8) & 0xFFu);

    const uint32_t qw[8] = {q0.x, q0.y, q0.z, q0.w, q1.x, q1.y, q1.z, q1.w};
    int l0 = 0, l1 = 0, l2 = 0, h0 = 0, h1 = 0, h2 = 0;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        const uint32_t lo = qw[i] & 0x0F0F0F0Fu;
        const uint32_t hi = qw[i] & 0xF0F0F0F0u;  // 16 * nibble; folded back below
        l0 = dp4a_u8s8(lo, x.a[0][i], l0);
        l1 = dp4a_u8s8(lo, x.a[1][i], l1);
        l2 = dp4a_u8s8(lo, x.a[2][i], l2);
        h0 = dp4a_u8s8(hi, x.b[0][i], h0);
        h1 = dp4a_u8s8(hi, x.b[1][i], h1);
        h2 = dp4a_u8s8(hi, x.b[2][i], h2);
    }
    const int tl = l0 * 16384 + l1 * 128 + l2;
    const int th = h0 * 1024 + h1 * 8 + (h2 >> 4);  // exact: every h is a multiple of 16
    float r = (d * sc0) * x.sa * static_cast<float>(tl) - (dmin * m0) * x.ma;
    r += (d * sc1) * x.sb * static_cast<float>(th) - (dmin * m1) * x.mb;
    return r;
}

// Q4_0: the unit is two 18-byte blocks = 9 aligned words; block A's nibbles straddle word
// boundaries by two bytes (tensor/standard/Q4_0FloatTensor.java:56-79: w = (q - 8) * d).
__device__ __forceinline__ float unit_q4_0(const uint8_t *chunk, int lane, const UnitX &x) {
    const uint32_t *wp = reinterpret_cast<const uint32_t *>(chunk) + lane * 9;
    uint32_t w[9];
#pragma unroll
    for (int i = 0; i < 9; ++i) w[i] = wp[i];
    const float dA = half_bits_to_float(w[0] & 0xFFFFu);
    const float dB = half_bits_to_float(w[4] >> 16);
    int l0 = 0, l1 = 0, l2 = 0, h0 = 0, h1 = 0, h2 = 0;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const uint32_t q = __funnelshift_r(w[i], w[i + 1], 16);
        const uint32_t lo = q & 0x0F0F0F0Fu, hi = q & 0xF0F0F0F0u;
        l0 = dp4a_u8s8(lo, x.a[0][i], l0);
        l1 = dp4a_u8s8(lo, x.a[1][i], l1);
        l2 = dp4a_u8s8(lo, x.a[2][i], l2);
        h0 = dp4a_u8s8(hi, x.a[0][4 + i], h0);
        h1 = dp4a_u8s8(hi, x.a[1][4 + i], h1);
        h2 = dp4a_u8s8(hi, x.a[2][4 + i], h2);
    }
    const int tA = (l0 * 16384 + l1 * 128 + l2) + (h0 * 1024 + h1 * 8 + (h2 >> 4));
    l0 = l1 = l2 = h0 = h1 = h2 = 0;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const uint32_t q = w[5 + i];
        const uint32_t lo = q & 0x0F0F0F0Fu, hi = q & 0xF0F0F0F0u;
        l0 = dp4a_u8s8(lo, x.b[0][i], l0);
        l1 = dp4a_u8s8(lo, x.b[1][i], l1);
        l2 = dp4a_u8s8(lo, x.b[2][i], l2);
        h0 = dp4a_u8s8(hi, x.b[0][4 + i], h0);
        h1 = dp4a_u8s8(hi, x.b[1][4 + i], h1);
        h2 = dp4a_u8s8(hi, x.b[2][4 + i], h2);
    }
    const int tB = (l0 * 16384 + l1 * 128 + l2) + (h0 * 1024 + h1 * 8 + (h2 >> 4));
    float r = dA * (x.sa * static_cast<float>(tA) - 8.0f * x.ma);
    r += dB * (x.sb * static_cast<float>(tB) - 8.0f * x.mb);
    return r;
}

// Q8_0: two 34-byte blocks = 17 aligned words (tensor/standard/Q8_0FloatTensor.java:53-61).
__device__ __forceinline__ float unit_q8_0(const uint8_t *chunk, int lane, const UnitX &x) {
    const uint32_t *wp = reinterpret_cast<const uint32_t *>(chunk) + lane * 17;
    uint32_t w[17];
#pragma unroll
    for (int i = 0; i < 17; ++i) w[i] = wp[i];
    const float dA = half_bits_to_float(w[0] & 0xFFFFu);
    const float dB = half_bits_to_float(w[8] >> 16);
    int a0 = 0, a1 = 0, a2 = 0, b0 = 0, b1 = 0, b2 = 0;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        const int qa = static_cast<int>(__funnelshift_r(w[i], w[i + 1], 16));
        const int qb = static_cast<int>(w[9 + i]);
        a0 = dp4a_s8s8(qa, x.a[0][i], a0);
        a1 = dp4a_s8s8(qa, x.a[1][i], a1);
        a2 = dp4a_s8s8(qa, x.a[2][i], a2);
        b0 = dp4a_s8s8(qb, x.b[0][i], b0);
        b1 = dp4a_s8s8(qb, x.b[1][i], b1);
        b2 = dp4a_s8s8(qb, x.b[2][i], b2);
    }
    // |a0| can reach 2^18, so the 2^14 digit weight is applied in floating point.
    const float fA = static_cast<float>(a0) * 16384.0f + static_cast<float>(a1 * 128 + a2);
    const float fB = static_cast<float>(b0) * 16384.0f + static_cast<float>(b1 * 128 + b2);
    return (dA * x.sa) * fA + (dB * x.sb) * fB;
}

template <int TYPE>
__device__ __forceinline__ float unit_dot(const uint8_t *chunk, int lane, const UnitX &x) {
    if constexpr (TYPE == kQ4_K) return unit_q4_k(chunk, lane, x);
    if constexpr (TYPE == kQ4_0) return unit_q4_0(chunk, lane, x);
    return unit_q8_0(chunk, lane, x);
}

struct SmemLayout {
    uint64_t *bars;
    float *scratch;  // 32 floats
    float *sx, *sumx;
    uint8_t *limbs;
    uint8_t *ring;
};

__host__ __device__ inline size_t align_up(size_t v, size_t a) { return (v + a - 1) / a * a; }
__host__ __device__ inline size_t x_region_bytes(int cols) {
    return align_up(size_t(cols) / 32 * 8, 128) + align_up(size_t(cols) * kLimbs, 128);
}

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

// Quantises the activation vector (optionally RMS-normalised first) into digit planes in shared
// memory. Layout of the planes: 16-byte cell index ((digit*4 + quarter) * nunits + unit), so that
// the 32 lanes of a warp, working on 32 consecutive units, read consecutive cells.
//
// A thread handles float4 pieces; the eight lanes that hold one 32-element block agree on the
// block maximum with three shuffles. Loads are issued eight deep before anything depends on them,
// so the whole vector costs about one L2 round trip rather than one per block.
__device__ __forceinline__ uint32_t pack4(int b0, int b1, int b2, int b3) {
    return (uint32_t(b0) & 0xFFu) | ((uint32_t(b1) & 0xFFu) << 8) | ((uint32_t(b2) & 0xFFu) << 16) |
           (uint32_t(b3) << 24);
}

__device__ void stage_activation(const GemvArgs &a, const SmemLayout &sm) {
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int cols = a.cols, nunits = cols / 64, n4 = cols / 4;
    const float4 *x4 = reinterpret_cast<const float4 *>(a.x);
    const float4 *w4 = reinterpret_cast<const float4 *>(a.norm_w);
    const bool norm = a.norm_w != nullptr;
    float ss = 1.0f;
    if (norm) {
        float part = 0.f;
#pragma unroll 4
        for (int i = tid; i < n4; i += kThreads) {
            const float4 v = x4[i];
            part += v.x * v.x + v.y * v.y + v.z * v.z + v.w * v.w;
        }
        part = warp_sum(part);
        if (lane == 0) sm.scratch[warp] = part;
        __syncthreads();
        float tot = 0.f;
#pragma unroll
        for (int w = 0; w < kWarps; ++w) tot += sm.scratch[w];
        float ms = tot / static_cast<float>(cols);
        ms += a.eps;
        ss = static_cast<float>(1.0 / sqrt(static_cast<double>(ms)));
    }
    constexpr int kDeep = 8;
    const size_t plane = size_t(4) * nunits * 16;
    for (int base = 0; base < n4; base += kThreads * kDeep) {
        float4 v[kDeep];
#pragma unroll
        for (int k = 0; k < kDeep; ++k) {
            const int i = base + k * kThreads + tid;
            v[k] = i < n4 ? x4[i] : make_float4(0.f, 0.f, 0.f, 0.f);
        }
        if (norm) {
#pragma unroll
            for (int k = 0; k < kDeep; ++k) {
                const int i = base + k * kThreads + tid;
                const float4 w = i < n4 ? w4[i] : make_float4(0.f, 0.f, 0.f, 0.f);
                v[k].x = __fmul_rn(w.x, __fmul_rn(ss, v[k].x));
                v[k].y = __fmul_rn(w.y, __fmul_rn(ss, v[k].y));
                v[k].z = __fmul_rn(w.z, __fmul_rn(ss, v[k].z));
                v[k].w = __fmul_rn(w.w, __fmul_rn(ss, v[k].w));
            }
        }
#pragma unroll
        for (int k = 0; k < kDeep; ++k) {
            const int i = base + k * kThreads + tid;  // float4 index; 8 consecutive = one block
            float amax = fmaxf(fmaxf(fabsf(v[k].x), fabsf(v[k].y)), fmaxf(fabsf(v[k].z), fabsf(v[k].w)));
            amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 1));
            amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 2));
            amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 4));
            const float inv = amax > 0.f ? kLimbRange / amax : 0.f;
            int X[4] = {__float2int_rn(v[k].x * inv), __float2int_rn(v[k].y * inv),
                        __float2int_rn(v[k].z * inv), __float2int_rn(v[k].w * inv)};
            int d1[4], d2[4], d3[4], sum = 0;
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                X[j] = max(-1040000, min(1040000, X[j]));
                sum += X[j];
                d3[j] = ((X[j] + 64) & 127) - 64;
                const int X1 = (X[j] - d3[j]) >> 7;
                d2[j] = ((X1 + 64) & 127) - 64;
                d1[j] = (X1 - d2[j]) >> 7;
            }
            sum += __shfl_xor_sync(0xffffffffu, sum, 1);
            sum += __shfl_xor_sync(0xffffffffu, sum, 2);
            sum += __shfl_xor_sync(0xffffffffu, sum, 4);
            if (i < n4) {
                const int e = i * 4;
                const int unit = e >> 6, within = e & 63, quarter = within >> 4, byte = within & 15;
                uint8_t *cell = sm.limbs + (size_t(quarter) * nunits + unit) * 16 + byte;
                *reinterpret_cast<uint32_t *>(cell) = pack4(d1[0], d1[1], d1[2], d1[3]);
                *reinterpret_cast<uint32_t *>(cell + plane) = pack4(d2[0], d2[1], d2[2], d2[3]);
                *reinterpret_cast<uint32_t *>(cell + 2 * plane) = pack4(d3[0], d3[1], d3[2], d3[3]);
                if ((i & 7) == 0) {
                    const float s = amax / kLimbRange;
                    sm.sx[i >> 3] = s;
                    sm.sumx[i >> 3] = s * static_cast<float>(sum);
                }
            }
        }
    }
}

__device__ __forceinline__ void load_unit_x(const SmemLayout &sm, int nunits, int unit, UnitX &x) {
    const size_t plane = size_t(4) * nunits * 16;
#pragma unroll
    for (int m = 0; m < kLimbs; ++m) {
        const uint8_t *base = sm.limbs + m * plane + size_t(unit) * 16;
        const int4 c0 = *reinterpret_cast<const int4 *>(base);
        const int4 c1 = *reinterpret_cast<const int4 *>(base + size_t(nunits) * 16);
        const int4 c2 = *reinterpret_cast<const int4 *>(base + size_t(nunits) * 32);
        const int4 c3 = *reinterpret_cast<const int4 *>(base + size_t(nunits) * 48);
        x.a[m][0] = c0.x; x.a[m][1] = c0.y; x.a[m][2] = c0.z; x.a[m][3] = c0.w;
        x.a[m][4] = c1.x; x.a[m][5] = c1.y; x.a[m][6] = c1.z; x.a[m][7] = c1.w;
        x.b[m][0] = c2.x; x.b[m][1] = c2.y; x.b[m][2] = c2.z; x.b[m][3] = c2.w;
        x.b[m][4] = c3.x; x.b[m][5] = c3.y; x.b[m][6] = c3.z; x.b[m][7] = c3.w;
    }
    const float2 s = *reinterpret_cast<const float2 *>(sm.sx + 2 * unit);
    const float2 m = *reinterpret_cast<const float2 *>(sm.sumx + 2 * unit);
    x.sa = s.x; x.sb = s.y; x.ma = m.x; x.mb = m.y;
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
    // Producer cursor (lane 0): the next item to request, advanced incrementally.
    int p_tile = wg, p_cc = 0, p_seg = 0, p_row0 = 0, p_issued = 0;
    locate(p_tile, p_seg, p_row0);
    auto issue = [&](int s) {  // lane 0 only
        const int nun = min(32, nunits - p_cc * 32);
        const uint32_t bytes = uint32_t(nun) * UB;
        const int nrows = min(R, a.seg[p_seg].rows - p_row0);
        uint8_t *stage = my_ring + size_t(s) * stage_bytes;
        uint64_t *bar = my_bars + s;
        mbar_expect_tx(bar, bytes * nrows * (MODE == kGemvGateUp ? 2 : 1));
        const uint8_t *src = a.seg[p_seg].w + size_t(p_row0) * rowb + size_t(p_cc) * CB;
        for (int r = 0; r < nrows; ++r) {
            bulk_g2s_hint(stage + r * CB, src + size_t(r) * rowb, bytes, bar, policy);
            if (MODE == kGemvGateUp)
                bulk_g2s_hint(stage + (R + r) * CB,
                              a.seg[1].w + size_t(p_row0 + r) * rowb + size_t(p_cc) * CB, bytes, bar,
                              policy);
        }
        ++p_issued;
        if (++p_cc == nchunks) {
            p_cc = 0;
            p_tile += total_warps;
            if (p_tile < total_tiles) locate(p_tile, p_seg, p_row0);
        }
    };

    if (lane == 0) {
        for (int s = 0; s < stages; ++s) mbar_init(my_bars + s, 1);
        mbar_fence_init();
        fence_proxy_async();
        const int first = min(stages, n_items);
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
        bool ok = mbar_wait_bounded(my_bars + s, parity);
        ok = __all_sync(0xffffffffu, ok);
        if (!ok) {
            failed = true;
            break;
        }
        const uint8_t *stage = my_ring + size_t(s) * stage_bytes;
        const int unit = cc * 32 + lane;
        if (unit < nunits) {
            UnitX x;
            load_unit_x(sm, nunits, unit, x);
#pragma unroll
            for (int r = 0; r < NR; ++r) acc[r] += unit_dot<TYPE>(stage + r * CB, lane, x);
        }
        __syncwarp();
        if (lane == 0 && p_issued < n_items) {
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
