// Device-side core of the quantised matrix-vector product: the three block formats as integer dot
// products against two signed 8-bit digits of the activation, and the activation staging.
#pragma once

#include "gemv.cuh"

namespace jl {

constexpr int kUnitBytesQ4 = 36;   // 64 elements: Q4_K 144/4, Q4_0 2*18
constexpr int kUnitBytesQ8 = 68;   // 64 elements: Q8_0 2*34

template <int TYPE>
struct Fmt {
    // bytes of 256 columns: one super-block (Q4_K, Q5_K, Q6_K) or eight blocks (Q4_0, Q4_1, Q8_0). A 64-element
    // unit is a quarter of that; for Q5_K and Q6_K it is no byte range of its own (the high bits sit apart).
    static constexpr int group_bytes = TYPE == kQ8_0   ? 8 * kQ8_0Bytes
                                       : TYPE == kQ6_K ? kQ6_KPadded  // read from the copy with padded super-blocks
                                       : TYPE == kQ5_K ? kQ5_KBytes
                                       : TYPE == kQ4_1 ? 8 * kQ4_1Bytes
                                                       : kQ4_KBytes;  // Q4_K, and Q4_0: 8 x 18
    static constexpr int unit_bytes = group_bytes / 4;   // meaningful for Q8_0, Q4_0, Q4_1, Q4_K
    static constexpr int chunk_bytes = 8 * group_bytes;  // 32 lanes x one unit = 2048 columns
    static constexpr int streams = (TYPE == kQ8_0) ? 1 : 2;  // rows per stage (gemv_rows_per_stage)
    // bytes of one row of nunits 64-element units
    __host__ __device__ static constexpr uint32_t row_bytes(int nunits) { return uint32_t(nunits / 4) * group_bytes; }
};
static_assert(Fmt<kQ4_K>::unit_bytes == kUnitBytesQ4 && Fmt<kQ4_0>::unit_bytes == kUnitBytesQ4 &&
                  Fmt<kQ8_0>::unit_bytes == kUnitBytesQ8, "unit sizes");

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

// Activation digits of one 64-element unit: [digit][word]; a = first 32-element block, b = second.
struct UnitX {
    int a[kDigits][8];
    int b[kDigits][8];
    float sa, sb;    // block scales
    float ma, mb;    // block sums of the quantised activation (scale * sum of the integers)
};

// ---- one unit of one row: returns sum_{64 el} w * x -------------------------------------------

// Q4_K: the unit is nibble pair p of super-block (lane/4): 32 qs bytes whose low nibbles are
// sub-block 2p and high nibbles sub-block 2p+1 (tensor/standard/Q4_KFloatTensor.java:88-122).
// The 6-bit scale and minimum of the two sub-blocks are cut out of the 12 packed bytes with
// selectors that depend on p only, so they cost the same for every lane.
__device__ __forceinline__ float unit_q4_k(uint32_t chunk, int lane, const UnitX &x) {
    const uint32_t sb = chunk + (lane >> 2) * kQ4_KBytes;
    const int p = lane & 3;
    const uint4 hdr = lds128(sb);
    const uint4 q0 = lds128(sb + 16 + p * 32);
    const uint4 q1 = lds128(sb + 32 + p * 32);
    const float d = half_bits_to_float(hdr.x & 0xFFFFu);
    const float dmin = half_bits_to_float(hdr.x >> 16);
    // Sub-blocks 0-3: scale = y byte & 63, minimum = z byte & 63. Sub-blocks 4-7: low four bits from
    // w (scale: low nibble, minimum: high nibble), top two bits from the top of the y / z bytes.
    const bool upper = p >= 2;
    const int sh = (p & 1) * 16;
    const uint32_t lo_mask = upper ? 0x0F0Fu : 0x3F3Fu;
    const uint32_t hi_mask = upper ? 0x3030u : 0u;
    const uint32_t sc2 = (((upper ? hdr.w : hdr.y) >> sh) & lo_mask) | ((hdr.y >> (sh + 2)) & hi_mask);
    const uint32_t m2 = (((upper ? (hdr.w >> 4) : hdr.z) >> sh) & lo_mask) | ((hdr.z >> (sh + 2)) & hi_mask);
    const int sc0 = sc2 & 0xFFu, sc1 = sc2 >> 8;
    const float m0 = static_cast<float>(m2 & 0xFFu), m1 = static_cast<float>(m2 >> 8);

    const uint32_t qw[8] = {q0.x, q0.y, q0.z, q0.w, q1.x, q1.y, q1.z, q1.w};
    int l0 = 0, l1 = 0, h0 = 0, h1 = 0;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        const uint32_t lo = qw[i] & 0x0F0F0F0Fu;
        const uint32_t hi = qw[i] & 0xF0F0F0F0u;  // 16 * nibble; folded back below
        l0 = dp4a_u8s8(lo, x.a[0][i], l0);
        l1 = dp4a_u8s8(lo, x.a[1][i], l1);
        h0 = dp4a_u8s8(hi, x.b[0][i], h0);
        h1 = dp4a_u8s8(hi, x.b[1][i], h1);
    }
    // |sum q*X| <= 15 * 32639 * 32 < 2^24 and times a 6-bit scale < 2^31: exact in integers.
    const int tl = l0 * 256 + l1;
    const int th = (h0 * 256 + h1) >> 4;  // exact: every h is a multiple of 16
    const float dots = x.sa * static_cast<float>(sc0 * tl) + x.sb * static_cast<float>(sc1 * th);
    const float mins = m0 * x.ma + m1 * x.mb;
    return d * dots - dmin * mins;
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
    int l0 = 0, l1 = 0, h0 = 0, h1 = 0;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const uint32_t q = __funnelshift_r(w[i], w[i + 1], 16);
        const uint32_t lo = q & 0x0F0F0F0Fu, hi = q & 0xF0F0F0F0u;
        l0 = dp4a_u8s8(lo, x.a[0][i], l0);
        l1 = dp4a_u8s8(lo, x.a[1][i], l1);
        h0 = dp4a_u8s8(hi, x.a[0][4 + i], h0);
        h1 = dp4a_u8s8(hi, x.a[1][4 + i], h1);
    }
    const int tA = (l0 * 256 + l1) + ((h0 * 256 + h1) >> 4);
    l0 = l1 = h0 = h1 = 0;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const uint32_t q = w[5 + i];
        const uint32_t lo = q & 0x0F0F0F0Fu, hi = q & 0xF0F0F0F0u;
        l0 = dp4a_u8s8(lo, x.b[0][i], l0);
        l1 = dp4a_u8s8(lo, x.b[1][i], l1);
        h0 = dp4a_u8s8(hi, x.b[0][4 + i], h0);
        h1 = dp4a_u8s8(hi, x.b[1][4 + i], h1);
    }
    const int tB = (l0 * 256 + l1) + ((h0 * 256 + h1) >> 4);
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
    int a0 = 0, a1 = 0, b0 = 0, b1 = 0;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        const int qa = static_cast<int>(__funnelshift_r(w[i], w[i + 1], 16));
        const int qb = static_cast<int>(w[9 + i]);
        a0 = dp4a_s8s8(qa, x.a[0][i], a0);
        a1 = dp4a_s8s8(qa, x.a[1][i], a1);
        b0 = dp4a_s8s8(qb, x.b[0][i], b0);
        b1 = dp4a_s8s8(qb, x.b[1][i], b1);
    }
    // |a0| <= 128 * 128 * 32 = 2^19, so 256 * a0 + a1 stays below 2^28: exact in integers.
    const float fA = static_cast<float>(a0 * 256 + a1);
    const float fB = static_cast<float>(b0 * 256 + b1);
    return (dA * x.sa) * fA + (dB * x.sb) * fB;
}

// Q6_K (tensor/standard/Q6_KFloatTensor.java:64-117), read from the copy whose 210-byte super-blocks are padded to
// kQ6_KPadded bytes (made at upload: rows become whole 16-byte pieces for the bulk copies, and every field is
// word-aligned). The unit is quarter p of super-block (lane/4): half h = p / 2 of the block, groups 2u and 2u + 1 of
// that half with u = p & 1 -- the low (u = 0) or high (u = 1) nibbles of the half's 64 ql bytes, bits 4u..4u+3 of its
// 32 qh bytes, four signed byte scales (one per 16 elements), the block's d. The six-bit value v becomes the signed
// byte 4 * (v - 32) as (v ^ 32) << 2 -- flipping bit 5 is v - 32 in six-bit two's complement and the shift moves its
// sign into bit 7 -- so the integer dot products are exact and four times too large.
__device__ __forceinline__ float unit_q6_k(uint32_t chunk, int lane, const UnitX &x) {
    const uint32_t sb = chunk + (lane >> 2) * kQ6_KPadded;
    const int p = lane & 3, h = p >> 1, u = p & 1;
    const uint4 h0 = lds128(sb + 128 + 32 * h), h1 = lds128(sb + 144 + 32 * h);
    const uint32_t qh[8] = {h0.x >> (4 * u), h0.y >> (4 * u), h0.z >> (4 * u), h0.w >> (4 * u),
                            h1.x >> (4 * u), h1.y >> (4 * u), h1.z >> (4 * u), h1.w >> (4 * u)};  // bits 0-1, 2-3: the groups
    const uint32_t sc4 = lds32(sb + 192 + 8 * h + 4 * u) ^ 0x80808080u;  // signed scales, biased by 128
    const float d = half_bits_to_float(lds32(sb + 208) & 0xFFFFu);
    int acc[4][2] = {{0, 0}, {0, 0}, {0, 0}, {0, 0}};  // [16-element scale group][digit]
#pragma unroll
    for (int q = 0; q < 4; ++q) {  // four words of ql per load: words 0-7 the first group, 8-15 the second
        const uint4 l4 = lds128(sb + 64 * h + 16 * q);
        const uint32_t lw[4] = {l4.x, l4.y, l4.z, l4.w};
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int i = 4 * q + j;
            const uint32_t nib = (lw[j] >> (4 * u)) & 0x0F0F0F0Fu;
            const uint32_t top = i < 8 ? (qh[i] << 4) : (qh[i - 8] << 2);
            const uint32_t w4 = ((nib | (top & 0x30303030u)) ^ 0x20202020u) << 2;
            const int g = i >> 2;
            if (i < 8) {
                acc[g][0] = dp4a_s8s8(int(w4), x.a[0][i], acc[g][0]);
                acc[g][1] = dp4a_s8s8(int(w4), x.a[1][i], acc[g][1]);
            } else {
                acc[g][0] = dp4a_s8s8(int(w4), x.b[0][i - 8], acc[g][0]);
                acc[g][1] = dp4a_s8s8(int(w4), x.b[1][i - 8], acc[g][1]);
            }
        }
    }
    // |acc| <= 16 * 128 * 128 = 2^18, so 256 * acc[.][0] + acc[.][1] stays below 2^27: exact in integers.
    float t[4];
#pragma unroll
    for (int g = 0; g < 4; ++g) t[g] = static_cast<float>(acc[g][0] * 256 + acc[g][1]);
    const float s0 = __uint_as_float(__byte_perm(sc4, 0x4B000000u, 0x7540u)) - 8388736.0f;  // byte - 128, no conversion
    const float s1 = __uint_as_float(__byte_perm(sc4, 0x4B000000u, 0x7541u)) - 8388736.0f;
    const float s2 = __uint_as_float(__byte_perm(sc4, 0x4B000000u, 0x7542u)) - 8388736.0f;
    const float s3 = __uint_as_float(__byte_perm(sc4, 0x4B000000u, 0x7543u)) - 8388736.0f;
    return (0.25f * d) * (x.sa * (s0 * t[0] + s1 * t[1]) + x.sb * (s2 * t[2] + s3 * t[3]));
}

// Q5_K (tensor/standard/Q5_KFloatTensor.java:87-127): Q4_K's layout with 32 bytes of fifth bits between the header
// and the nibbles: the unit is nibble pair p of super-block (lane/4); bit 2p of qh byte j is the fifth bit of
// element j of sub-block 2p (low nibbles), bit 2p + 1 that of sub-block 2p + 1 (high nibbles).
__device__ __forceinline__ float unit_q5_k(uint32_t chunk, int lane, const UnitX &x) {
    const uint32_t sb = chunk + (lane >> 2) * kQ5_KBytes;
    const int p = lane & 3;
    const uint4 hdr = lds128(sb);
    const uint4 h0 = lds128(sb + 16), h1 = lds128(sb + 32);
    const uint4 q0 = lds128(sb + 48 + p * 32), q1 = lds128(sb + 64 + p * 32);
    const float d = half_bits_to_float(hdr.x & 0xFFFFu);
    const float dmin = half_bits_to_float(hdr.x >> 16);
    const bool upper = p >= 2;  // the packed 6-bit scales and minima: as in unit_q4_k
    const int sh = (p & 1) * 16;
    const uint32_t lo_mask = upper ? 0x0F0Fu : 0x3F3Fu;
    const uint32_t hi_mask = upper ? 0x3030u : 0u;
    const uint32_t sc2 = (((upper ? hdr.w : hdr.y) >> sh) & lo_mask) | ((hdr.y >> (sh + 2)) & hi_mask);
    const uint32_t m2 = (((upper ? (hdr.w >> 4) : hdr.z) >> sh) & lo_mask) | ((hdr.z >> (sh + 2)) & hi_mask);
    const int sc0 = sc2 & 0xFFu, sc1 = sc2 >> 8;
    const float m0 = static_cast<float>(m2 & 0xFFu), m1 = static_cast<float>(m2 >> 8);
    const uint32_t qw[8] = {q0.x, q0.y, q0.z, q0.w, q1.x, q1.y, q1.z, q1.w};
    const uint32_t hw[8] = {h0.x, h0.y, h0.z, h0.w, h1.x, h1.y, h1.z, h1.w};
    int l0 = 0, l1 = 0, h0s = 0, h1s = 0;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        const uint32_t fifth = hw[i] >> (2 * p);
        const uint32_t lo = (qw[i] & 0x0F0F0F0Fu) | ((fifth << 4) & 0x10101010u);
        const uint32_t hi = ((qw[i] >> 4) & 0x0F0F0F0Fu) | ((fifth << 3) & 0x10101010u);
        l0 = dp4a_u8s8(lo, x.a[0][i], l0);
        l1 = dp4a_u8s8(lo, x.a[1][i], l1);
        h0s = dp4a_u8s8(hi, x.b[0][i], h0s);
        h1s = dp4a_u8s8(hi, x.b[1][i], h1s);
    }
    // |sum q*X| <= 31 * 128 * 32 < 2^17 per digit, 256 * l0 + l1 < 2^25, times a 6-bit scale < 2^31: exact in integers.
    const float dots = x.sa * static_cast<float>(sc0 * (l0 * 256 + l1)) + x.sb * static_cast<float>(sc1 * (h0s * 256 + h1s));
    const float mins = m0 * x.ma + m1 * x.mb;
    return d * dots - dmin * mins;
}

// Q4_1 (tensor/standard/Q4_1FloatTensor.java:76-99: w = q * d + m, q unsigned): the unit is two 20-byte blocks = ten
// aligned words, each block a word of (d, m) and four words of nibbles (low nibbles elements 0-15, high 16-31).
__device__ __forceinline__ float unit_q4_1(uint32_t chunk, int lane, const UnitX &x) {
    const uint32_t wp = chunk + lane * 40;
    uint32_t w[10];
#pragma unroll
    for (int i = 0; i < 10; ++i) w[i] = lds32(wp + 4 * i);
    int l0 = 0, l1 = 0, h0 = 0, h1 = 0;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const uint32_t lo = w[1 + i] & 0x0F0F0F0Fu, hi = (w[1 + i] >> 4) & 0x0F0F0F0Fu;
        l0 = dp4a_u8s8(lo, x.a[0][i], l0);
        l1 = dp4a_u8s8(lo, x.a[1][i], l1);
        h0 = dp4a_u8s8(hi, x.a[0][4 + i], h0);
        h1 = dp4a_u8s8(hi, x.a[1][4 + i], h1);
    }
    const float tA = static_cast<float>((l0 + h0) * 256 + (l1 + h1));
    l0 = l1 = h0 = h1 = 0;
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const uint32_t lo = w[6 + i] & 0x0F0F0F0Fu, hi = (w[6 + i] >> 4) & 0x0F0F0F0Fu;
        l0 = dp4a_u8s8(lo, x.b[0][i], l0);
        l1 = dp4a_u8s8(lo, x.b[1][i], l1);
        h0 = dp4a_u8s8(hi, x.b[0][4 + i], h0);
        h1 = dp4a_u8s8(hi, x.b[1][4 + i], h1);
    }
    const float tB = static_cast<float>((l0 + h0) * 256 + (l1 + h1));
    float r = half_bits_to_float(w[0] & 0xFFFFu) * (x.sa * tA) + half_bits_to_float(w[0] >> 16) * x.ma;
    r += half_bits_to_float(w[5] & 0xFFFFu) * (x.sb * tB) + half_bits_to_float(w[5] >> 16) * x.mb;
    return r;
}

template <int TYPE>
__device__ __forceinline__ float unit_dot(uint32_t chunk, int lane, const UnitX &x) {
    if constexpr (TYPE == kQ6_K) return unit_q6_k(chunk, lane, x);
    if constexpr (TYPE == kQ5_K) return unit_q5_k(chunk, lane, x);
    if constexpr (TYPE == kQ4_1) return unit_q4_1(chunk, lane, x);
    if constexpr (TYPE == kQ4_K) return unit_q4_k(chunk, lane, x);
    if constexpr (TYPE == kQ4_0) return unit_q4_0(chunk, lane, x);
    return unit_q8_0(chunk, lane, x);
}

__host__ __device__ inline size_t align_up(size_t v, size_t a) { return (v + a - 1) / a * a; }
// Shared-memory bytes of the staged activation: block scales (one float per 32 elements), then
// kDigits planes of one byte per element.
__host__ __device__ inline size_t x_scales_bytes(int cols) { return align_up(size_t(cols) / 32 * 4, 128); }
__host__ __device__ inline size_t x_region_bytes(int cols) {
    return x_scales_bytes(cols) + align_up(size_t(cols) * kDigits, 128);
}

__device__ __forceinline__ uint32_t pack4(int b0, int b1, int b2, int b3) {
    return (uint32_t(b0) & 0xFFu) | ((uint32_t(b1) & 0xFFu) << 8) | ((uint32_t(b2) & 0xFFu) << 16) |
           (uint32_t(b3) << 24);
}

__device__ __forceinline__ void named_bar_sync(int id, int threads) {
    asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(threads) : "memory");
}

// Quantises the activation vector into digit planes in shared memory; NTHREADS threads (tid
// 0..NTHREADS-1) take part and nothing is synchronised here. With norm_w the vector quantised is
// norm_w * x and the sum of x^2 over this thread's elements is returned: the RMS factor is a
// scalar, so the caller multiplies the finished dot products by it instead of every element.
//
// Layout of the planes: 16-byte cell index ((digit*4 + quarter) * nunits + unit), so that the 32
// lanes of a warp, working on 32 consecutive units, read consecutive cells. A thread handles
// float4 pieces; the eight lanes that hold one 32-element block agree on the block maximum with
// three shuffles. wpre: the first KD float4 of norm_w for this thread, loaded by the caller before
// it waited for the producing kernel (weights are never written by a kernel).
constexpr int kStageDeep = 8;
template <int NTHREADS>
__device__ __forceinline__ float stage_activation_core(const float *x, const float *norm_w, const float4 *wpre,
                                                       int cols, int tid, float *sx_p, uint32_t planes_u32,
                                                       int trace_cls = -1) {
    const int nunits = cols / 64, n4 = cols / 4;
    const float4 *x4 = reinterpret_cast<const float4 *>(x);
    const float4 *w4 = reinterpret_cast<const float4 *>(norm_w);
    const bool norm = norm_w != nullptr;
    const uint32_t plane = 64u * nunits;
    float ssq = 0.f;
    for (int base = 0; base < n4; base += NTHREADS * kStageDeep) {
        float4 v[kStageDeep];
#pragma unroll
        for (int k = 0; k < kStageDeep; ++k) {
            const int i = base + k * NTHREADS + tid;
            // ld.global.cg: the vector was written by other SMs moments ago.
            v[k] = i < n4 ? __ldcg(x4 + i) : make_float4(0.f, 0.f, 0.f, 0.f);
        }
#ifdef JL_TRACE
        if (tid == 0 && trace_cls >= 0 && base == 0) {
            if (v[0].x == 12345.678f) trace_cta_word(trace_cls, 7, 1);  // make the stamp wait for the data
            trace_cta_word(trace_cls, 4, trace_now());
        }
#endif
        if (norm) {
#pragma unroll
            for (int k = 0; k < kStageDeep; ++k) {
                const int i = base + k * NTHREADS + tid;
                float4 w = make_float4(0.f, 0.f, 0.f, 0.f);
                if (base == 0) w = wpre[k];
                else if (i < n4) w = w4[i];
                ssq += v[k].x * v[k].x + v[k].y * v[k].y + v[k].z * v[k].z + v[k].w * v[k].w;
                v[k].x *= w.x; v[k].y *= w.y; v[k].z *= w.z; v[k].w *= w.w;
            }
        }
#pragma unroll
        for (int k = 0; k < kStageDeep; ++k) {
            if (base + k * NTHREADS >= n4) break;  // uniform: nothing left for any thread
            const int i = base + k * NTHREADS + tid;  // float4 index; 8 consecutive = one block
            float amax = fmaxf(fmaxf(fabsf(v[k].x), fabsf(v[k].y)), fmaxf(fabsf(v[k].z), fabsf(v[k].w)));
            amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 1));
            amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 2));
            amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 4));
            const float inv = amax > 0.f ? __fdividef(kDigitRange, amax) : 0.f;
            int X[4] = {__float2int_rn(v[k].x * inv), __float2int_rn(v[k].y * inv),
                        __float2int_rn(v[k].z * inv), __float2int_rn(v[k].w * inv)};
            int d1[4], d2[4];
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                X[j] = max(-32639, min(32639, X[j]));
                d1[j] = (X[j] + 128) >> 8;       // floor: the low digit lands in [-128, 127]
                d2[j] = X[j] - (d1[j] << 8);
            }
            if (i < n4) {
                const int e = i * 4;
                const int unit = e >> 6, within = e & 63, quarter = within >> 4, byte = within & 15;
                const uint32_t cell = planes_u32 + (uint32_t(quarter) * nunits + unit) * 16 + byte;
                sts32(cell, pack4(d1[0], d1[1], d1[2], d1[3]));
                sts32(cell + plane, pack4(d2[0], d2[1], d2[2], d2[3]));
                if ((i & 7) == 0) sx_p[i >> 3] = amax * (1.0f / kDigitRange);
            }
        }
    }
    return ssq;
}

// This lane's unit of the staged activation, from shared memory into registers. The block sums the
// 4-bit formats need (their codes carry an offset) are formed here from the digits: once per launch
// and lane, instead of three more shuffles per block while every warp waits for the staging.
__device__ __forceinline__ void load_unit_x(uint32_t planes, uint32_t sx, int nunits, int unit, UnitX &x) {
    const uint32_t plane = 64u * nunits;
    const uint32_t q = 16u * nunits;
#pragma unroll
    for (int m = 0; m < kDigits; ++m) {
        const uint32_t base = planes + m * plane + 16u * unit;
        const uint4 c0 = lds128(base), c1 = lds128(base + q), c2 = lds128(base + 2 * q),
                    c3 = lds128(base + 3 * q);
        x.a[m][0] = c0.x; x.a[m][1] = c0.y; x.a[m][2] = c0.z; x.a[m][3] = c0.w;
        x.a[m][4] = c1.x; x.a[m][5] = c1.y; x.a[m][6] = c1.z; x.a[m][7] = c1.w;
        x.b[m][0] = c2.x; x.b[m][1] = c2.y; x.b[m][2] = c2.z; x.b[m][3] = c2.w;
        x.b[m][4] = c3.x; x.b[m][5] = c3.y; x.b[m][6] = c3.z; x.b[m][7] = c3.w;
    }
    const uint2 s = lds64(sx + 8u * unit);
    x.sa = __uint_as_float(s.x); x.sb = __uint_as_float(s.y);
    int a1 = 0, a2 = 0, b1 = 0, b2 = 0;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        a1 = dp4a_s8s8(0x01010101, x.a[0][i], a1);
        a2 = dp4a_s8s8(0x01010101, x.a[1][i], a2);
        b1 = dp4a_s8s8(0x01010101, x.b[0][i], b1);
        b2 = dp4a_s8s8(0x01010101, x.b[1][i], b2);
    }
    x.ma = x.sa * static_cast<float>(a1 * 256 + a2);
    x.mb = x.sb * static_cast<float>(b1 * 256 + b2);
}

}  // namespace jl
