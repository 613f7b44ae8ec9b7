// GGUF block formats kept in their on-disk layout (format/GGMLType.java:7,13,18-20 of the
// reference): geometry constants and element-exact device decoders.
#pragma once

#include "common.cuh"

namespace jl {

enum : int { kF32 = 0, kF16 = 1, kQ4_0 = 2, kQ4_1 = 3, kQ8_0 = 8, kQ4_K = 12, kQ5_K = 13, kQ6_K = 14 };

constexpr int kQ8_0Block = 32, kQ8_0Bytes = 34;
constexpr int kQ4_0Block = 32, kQ4_0Bytes = 18;
constexpr int kQ4_KBlock = 256, kQ4_KBytes = 144;
// The formats real mixed-precision files add (format/GGMLType.java:8,21-30): decoded element-exactly and
// multiplied by the stand-alone operators; the model's step kernels take the three above.
constexpr int kQ4_1Block = 32, kQ4_1Bytes = 20;
constexpr int kQ5_KBlock = 256, kQ5_KBytes = 176;
constexpr int kQ6_KBlock = 256, kQ6_KBytes = 210;
// The tensor-core kernel fetches 128-row tiles through a 2-D tensor map, whose rows must be 16-byte multiples: it reads
// Q6_K matrices from a second copy with every super-block padded to this size (made on upload, same bytes, zero fill).
constexpr int kQ6_KPadded = 224;

// Every format packs 256 consecutive elements into a 16-byte-aligned group:
// Q4_K 144 B (one super-block), Q4_0 8 x 18 = 144 B, Q8_0 8 x 34 = 272 B.
__host__ __device__ inline int64_t row_bytes(int type, int64_t cols) {
    switch (type) {
        case kF32: return cols * 4;
        case kF16: return cols * 2;
        case kQ8_0: return cols / kQ8_0Block * kQ8_0Bytes;
        case kQ4_0: return cols / kQ4_0Block * kQ4_0Bytes;
        case kQ4_K: return cols / kQ4_KBlock * kQ4_KBytes;
        case kQ4_1: return cols / kQ4_1Block * kQ4_1Bytes;
        case kQ5_K: return cols / kQ5_KBlock * kQ5_KBytes;
        case kQ6_K: return cols / kQ6_KBlock * kQ6_KBytes;
        default: return -1;
    }
}
__host__ __device__ inline bool is_quant(int type) {
    return type == kQ8_0 || type == kQ4_0 || type == kQ4_K;
}

// Q4_1, Q5_K, Q6_K: block formats outside the model's step kernels.
__host__ __device__ inline bool is_extra_quant(int type) {
    return type == kQ4_1 || type == kQ5_K || type == kQ6_K;
}
__host__ __device__ inline int block_elements(int type) {
    return (type == kQ4_K || type == kQ5_K || type == kQ6_K) ? 256 : 32;
}

__device__ __forceinline__ float f16_at(const uint8_t *p) {
    return half_bits_to_float(uint32_t(p[0]) | (uint32_t(p[1]) << 8));
}

// Element-exact decoders: the same binary32 operations in the same order as the reference's
// FloatTensor.getFloat, with explicit round-to-nearest intrinsics so nothing is contracted to FMA.
// tensor/standard/Q8_0FloatTensor.java:53-61
__device__ __forceinline__ float decode_q8_0(const uint8_t *data, int64_t index) {
    const uint8_t *blk = data + (index / kQ8_0Block) * kQ8_0Bytes;
    int q = static_cast<int8_t>(blk[2 + index % kQ8_0Block]);
    return __fmul_rn(static_cast<float>(q), f16_at(blk));
}
// tensor/standard/Q4_0FloatTensor.java:56-79
__device__ __forceinline__ float decode_q4_0(const uint8_t *data, int64_t index) {
    const uint8_t *blk = data + (index / kQ4_0Block) * kQ4_0Bytes;
    int w = static_cast<int>(index % kQ4_0Block);
    int q = w < 16 ? (blk[2 + w] & 0x0F) : (blk[2 + w - 16] >> 4);
    return __fmul_rn(static_cast<float>(q - 8), f16_at(blk));
}
// tensor/standard/Q4_KFloatTensor.java:68-122: ((d * sc) * q) - (dmin * m)
__device__ __forceinline__ float decode_q4_k(const uint8_t *data, int64_t index) {
    const uint8_t *blk = data + (index / kQ4_KBlock) * kQ4_KBytes;
    int within = static_cast<int>(index % kQ4_KBlock);
    float d = f16_at(blk), dmin = f16_at(blk + 2);
    const uint8_t *s = blk + 4, *qs = blk + 16;
    int pair = within >> 6, pos = within & 63;
    int sub = pair * 2 + (pos >> 5);
    int byte = qs[pair * 32 + (pos & 31)];
    int q = (pos < 32) ? (byte & 0xF) : (byte >> 4);
    int sc, m;
    if (sub < 4) {
        sc = s[sub] & 63;
        m = s[sub + 4] & 63;
    } else {
        sc = (s[sub + 4] & 0xF) | ((s[sub - 4] >> 6) << 4);
        m = (s[sub + 4] >> 4) | ((s[sub] >> 6) << 4);
    }
    float t = __fmul_rn(__fmul_rn(d, static_cast<float>(sc)), static_cast<float>(q));
    return __fsub_rn(t, __fmul_rn(dmin, static_cast<float>(m)));
}
// getScaleK4 / getMinK4 (tensor/standard/Q4_KFloatTensor.java:68-86, the same packing in Q5_KFloatTensor.java:64-84)
__device__ __forceinline__ int k4_scale(int j, const uint8_t *s) {
    return j < 4 ? (s[j] & 63) : ((s[j + 4] & 0xF) | ((s[j - 4] >> 6) << 4));
}
__device__ __forceinline__ int k4_min(int j, const uint8_t *s) {
    return j < 4 ? (s[j + 4] & 63) : ((s[j + 4] >> 4) | ((s[j] >> 6) << 4));
}
// tensor/standard/Q4_1FloatTensor.java:76-99: nibble * scale + min, unsigned nibble
__device__ __forceinline__ float decode_q4_1(const uint8_t *data, int64_t index) {
    const uint8_t *blk = data + (index / kQ4_1Block) * kQ4_1Bytes;
    const int w = static_cast<int>(index % kQ4_1Block);
    const int nibble = w < 16 ? (blk[4 + w] & 0x0F) : (blk[4 + w - 16] >> 4);
    return __fadd_rn(__fmul_rn(static_cast<float>(nibble), f16_at(blk)), f16_at(blk + 2));
}
// tensor/standard/Q5_KFloatTensor.java:87-127: ((d * sc) * q) - (dmin * m), q = nibble + 16 * fifth bit
__device__ __forceinline__ float decode_q5_k(const uint8_t *data, int64_t index) {
    const uint8_t *blk = data + (index / kQ5_KBlock) * kQ5_KBytes;
    const int within = static_cast<int>(index % kQ5_KBlock);
    const float d = f16_at(blk), dmin = f16_at(blk + 2);
    const uint8_t *s = blk + 4, *qh = blk + 16, *qs = blk + 48;
    const int pair = within >> 6, pos = within & 63, hi = pos >> 5, p = pos & 31;
    const int sub = pair * 2 + hi;
    const int byte = qs[pair * 32 + p];
    const int q = (hi ? (byte >> 4) : (byte & 0xF)) + (((qh[p] >> sub) & 1) << 4);
    const float t = __fmul_rn(__fmul_rn(d, static_cast<float>(k4_scale(sub, s))), static_cast<float>(q));
    return __fsub_rn(t, __fmul_rn(dmin, static_cast<float>(k4_min(sub, s))));
}
// tensor/standard/Q6_KFloatTensor.java:64-117: (d * scale) * (q - 32)
__device__ __forceinline__ float decode_q6_k(const uint8_t *data, int64_t index) {
    const uint8_t *blk = data + (index / kQ6_KBlock) * kQ6_KBytes;
    const int within = static_cast<int>(index % kQ6_KBlock);
    const int half = within >> 7, group = (within >> 5) & 3, p = within & 31;
    const int lo = blk[half * 64 + (group & 1) * 32 + p];
    const int q = ((group < 2 ? (lo & 0xF) : (lo >> 4)) | (((blk[128 + half * 32 + p] >> (2 * group)) & 3) << 4)) - 32;
    const int sc = static_cast<int8_t>(blk[192 + half * 8 + 2 * group + (p >> 4)]);
    return __fmul_rn(__fmul_rn(f16_at(blk + 208), static_cast<float>(sc)), static_cast<float>(q));
}
__device__ __forceinline__ float decode_any(int type, const uint8_t *data, int64_t index) {
    switch (type) {
        case kQ8_0: return decode_q8_0(data, index);
        case kQ4_0: return decode_q4_0(data, index);
        case kQ4_K: return decode_q4_k(data, index);
        case kQ4_1: return decode_q4_1(data, index);
        case kQ5_K: return decode_q5_k(data, index);
        case kQ6_K: return decode_q6_k(data, index);
        case kF16: return __half2float(reinterpret_cast<const __half *>(data)[index]);
        default: return reinterpret_cast<const float *>(data)[index];
    }
}

}  // namespace jl
