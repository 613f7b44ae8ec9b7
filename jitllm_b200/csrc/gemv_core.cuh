// Device-side core of the quantised matrix-vector product, shared by the per-operator kernel
// (gemv.cu) and the persistent per-token kernel (token_kernel.cu): block formats as integer dot
// products against three signed 7-bit digits of the activation, and the activation staging.
#pragma once

#include "gemv.cuh"

namespace jl {

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
__device__ __forceinline__ float unit_q4_k(uint32_t chunk, int lane, const UnitX &x) {
    const uint32_t sb = chunk + (lane >> 2) * kQ4_KBytes;
    const int p = lane & 3;
    const uint4 hdr = lds128(sb);
    const uint4 q0 = lds128(sb + 16 + p * 32);
    const uint4 q1 = lds128(sb + 32 + p * 32);
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
__device__ __forceinline__ float unit_q4_0(uint32_t chunk, int lane, const UnitX &x) {
    const uint32_t wp = chunk + lane * 36;
    uint32_t w[9];
#pragma unroll
    for (int i = 0; i < 9; ++i) w[i] = lds32(wp + 4 * i);
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
__device__ __forceinline__ float unit_q8_0(uint32_t chunk, int lane, const UnitX &x) {
    const uint32_t wp = chunk + lane * 68;
    uint32_t w[17];
#pragma unroll
    for (int i = 0; i < 17; ++i) w[i] = lds32(wp + 4 * i);
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
__device__ __forceinline__ float unit_dot(uint32_t chunk, int lane, const UnitX &x) {
    if constexpr (TYPE == kQ4_K) return unit_q4_k(chunk, lane, x);
    if constexpr (TYPE == kQ4_0) return unit_q4_0(chunk, lane, x);
    return unit_q8_0(chunk, lane, x);
}

__host__ __device__ inline size_t align_up(size_t v, size_t a) { return (v + a - 1) / a * a; }
__host__ __device__ inline size_t x_region_bytes(int cols) {
    return align_up(size_t(cols) / 32 * 8, 128) + align_up(size_t(cols) * kLimbs, 128);
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

// The activation is read with ld.global.cg: inside the persistent kernel it was written by other
// SMs moments earlier and must not be served from a stale L1 line.
// scratch: NTHREADS/32 + 1 floats of shared memory; sx / sumx: cols/32 floats each; limbs_u32: shared
// address of the 3*cols-byte digit planes. Contains a __syncthreads when norm_w != nullptr; the
// caller synchronises before the planes are read.
template <int NTHREADS>
__device__ __forceinline__ void stage_activation_core(const float *x, const float *norm_w, float eps,
                                                      int cols, float *scratch, float *sx_p,
                                                      float *sumx_p, uint32_t limbs_u32) {
    constexpr int kThreads = NTHREADS, kWarps = NTHREADS / 32;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int nunits = cols / 64, n4 = cols / 4;
    const float4 *x4 = reinterpret_cast<const float4 *>(x);
    const float4 *w4 = reinterpret_cast<const float4 *>(norm_w);
    const bool norm = norm_w != nullptr;
    constexpr int kDeep = 8;
    const uint32_t plane = 64u * nunits;
    // First batch of the vector; when the whole vector fits in one batch (dim <= 16384 with 512
    // threads) the RMS pass reuses these registers instead of a second trip to L2.
    float4 v[kDeep];
#pragma unroll
    for (int k = 0; k < kDeep; ++k) {
        const int i = k * kThreads + tid;
        v[k] = i < n4 ? __ldcg(x4 + i) : make_float4(0.f, 0.f, 0.f, 0.f);
    }
    float ss = 1.0f;
    if (norm) {
        float part = 0.f;
#pragma unroll
        for (int k = 0; k < kDeep; ++k)
            part += v[k].x * v[k].x + v[k].y * v[k].y + v[k].z * v[k].z + v[k].w * v[k].w;
#pragma unroll 4
        for (int i = kThreads * kDeep + tid; i < n4; i += kThreads) {
            const float4 u = __ldcg(x4 + i);
            part += u.x * u.x + u.y * u.y + u.z * u.z + u.w * u.w;
        }
        part = warp_sum(part);
        if (lane == 0) scratch[warp] = part;
        __syncthreads();
        if (tid == 0) {
            // One thread does the double-precision reciprocal square root (the reference narrows
            // 1.0 / Math.sqrt(ss) once); FP64 throughput is far too low to have every thread do it.
            float tot = 0.f;
#pragma unroll
            for (int w = 0; w < kWarps; ++w) tot += scratch[w];
            float ms = tot / static_cast<float>(cols);
            ms += eps;
            scratch[kWarps] = static_cast<float>(1.0 / sqrt(static_cast<double>(ms)));
        }
        __syncthreads();
        ss = scratch[kWarps];
    }
    for (int base = 0; base < n4; base += kThreads * kDeep) {
        if (base > 0) {
#pragma unroll
            for (int k = 0; k < kDeep; ++k) {
                const int i = base + k * kThreads + tid;
                v[k] = i < n4 ? __ldcg(x4 + i) : make_float4(0.f, 0.f, 0.f, 0.f);
            }
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
            if (base + k * kThreads >= n4) break;  // uniform: nothing left for any thread
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
                const uint32_t cell = limbs_u32 + (uint32_t(quarter) * nunits + unit) * 16 + byte;
                sts32(cell, pack4(d1[0], d1[1], d1[2], d1[3]));
                sts32(cell + plane, pack4(d2[0], d2[1], d2[2], d2[3]));
                sts32(cell + 2 * plane, pack4(d3[0], d3[1], d3[2], d3[3]));
                if ((i & 7) == 0) {
                    const float s = amax / kLimbRange;
                    sx_p[i >> 3] = s;
                    sumx_p[i >> 3] = s * static_cast<float>(sum);
                }
            }
        }
    }
}

__device__ __forceinline__ void load_unit_x(uint32_t limbs, uint32_t sx, uint32_t sumx, int nunits,
                                            int unit, UnitX &x) {
    const uint32_t plane = 64u * nunits;
    const uint32_t q = 16u * nunits;
#pragma unroll
    for (int m = 0; m < kLimbs; ++m) {
        const uint32_t base = limbs + m * plane + 16u * unit;
        const uint4 c0 = lds128(base), c1 = lds128(base + q), c2 = lds128(base + 2 * q),
                    c3 = lds128(base + 3 * q);
        x.a[m][0] = c0.x; x.a[m][1] = c0.y; x.a[m][2] = c0.z; x.a[m][3] = c0.w;
        x.a[m][4] = c1.x; x.a[m][5] = c1.y; x.a[m][6] = c1.z; x.a[m][7] = c1.w;
        x.b[m][0] = c2.x; x.b[m][1] = c2.y; x.b[m][2] = c2.z; x.b[m][3] = c2.w;
        x.b[m][4] = c3.x; x.b[m][5] = c3.y; x.b[m][6] = c3.z; x.b[m][7] = c3.w;
    }
    const uint2 s = lds64(sx + 8u * unit), m = lds64(sumx + 8u * unit);
    x.sa = __uint_as_float(s.x); x.sb = __uint_as_float(s.y);
    x.ma = __uint_as_float(m.x); x.mb = __uint_as_float(m.y);
}


}  // namespace jl
