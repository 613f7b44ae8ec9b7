/*
 * CPU oracle for the jitLLM Llama hot path -- TEST INFRASTRUCTURE, NOT PRODUCT CODE.
 * See jl_oracle.h for scope, parity status and the citation convention.
 *
 * Build: gcc -O2 -ffp-contract=off -fopenmp -shared -fPIC (see Makefile). -ffast-math must never
 * be used here: every sum below is written in the order the Java code performs it.
 */
#include "jl_oracle.h"

#include <math.h>
#include <stdlib.h>
#include <string.h>
#ifdef _OPENMP
#include <omp.h>
#endif

static int g_vector_bits = 0;
static int g_threads = 0;

void orc_set_vector_bits(int bits) { g_vector_bits = (bits == 128 || bits == 256) ? bits : 0; }
int orc_get_vector_bits(void) { return g_vector_bits; }
void orc_set_threads(int n) { g_threads = n; }
int orc_get_threads(void) {
#ifdef _OPENMP
    return g_threads > 0 ? g_threads : omp_get_num_procs();
#else
    return 1;
#endif
}

/* ---------------------------------------------------------------- fp16 <-> fp32 */

/* Float.float16ToFloat: exact widening, subnormals kept, NaN payload shifted. */
float orc_f16_to_f32(uint16_t h) {
    uint32_t sign = (uint32_t)(h & 0x8000u) << 16;
    uint32_t exp = (h >> 10) & 0x1Fu;
    uint32_t man = h & 0x3FFu;
    uint32_t bits;
    if (exp == 0) {
        if (man == 0) {
            bits = sign;
        } else { /* subnormal: normalise */
            int e = -1;
            do {
                man <<= 1;
                e++;
            } while ((man & 0x400u) == 0);
            man &= 0x3FFu;
            bits = sign | ((uint32_t)(127 - 15 - e) << 23) | (man << 13);
        }
    } else if (exp == 31) {
        bits = sign | 0x7F800000u | (man << 13);
    } else {
        bits = sign | ((exp + 127 - 15) << 23) | (man << 13);
    }
    float f;
    memcpy(&f, &bits, 4);
    return f;
}

/* Float.floatToFloat16: round to nearest even, overflow to infinity, subnormals produced. */
uint16_t orc_f32_to_f16(float f) {
    uint32_t x;
    memcpy(&x, &f, 4);
    uint16_t sign = (uint16_t)((x >> 16) & 0x8000u);
    uint32_t absx = x & 0x7FFFFFFFu;
    if (absx > 0x7F800000u) { /* NaN stays NaN: top 10 payload bits kept, the rest OR-ed in */
        return (uint16_t)(sign | 0x7C00u | ((x & 0x007FE000u) >> 13) | ((x & 0x00001FF0u) >> 4) |
                          (x & 0x0000000Fu));
    }
    if (absx >= 0x477FF000u) { /* >= 65520 rounds to infinity */
        return (uint16_t)(sign | 0x7C00u);
    }
    if (absx < 0x33000001u) { /* <= 2^-25: rounds to zero (tie at exactly 2^-25 goes to even=0) */
        return sign;
    }
    int32_t e = (int32_t)(absx >> 23) - 127;
    uint32_t m = (absx & 0x007FFFFFu) | 0x00800000u;
    int shift; /* bits dropped from the 24-bit significand */
    int32_t he;
    if (e < -14) { /* subnormal half */
        shift = 13 + (-14 - e);
        he = 0;
    } else {
        shift = 13;
        he = e + 15;
    }
    uint32_t kept = m >> shift;
    uint32_t rem = m & ((1u << shift) - 1u);
    uint32_t half = 1u << (shift - 1);
    if (rem > half || (rem == half && (kept & 1u))) kept++;
    uint32_t out;
    if (he == 0) {
        out = kept; /* may carry into exponent 1: correct by construction */
    } else {
        out = ((uint32_t)he << 10) + (kept - 0x400u); /* carry propagates into the exponent */
    }
    return (uint16_t)(sign | out);
}

/* ---------------------------------------------------------------- block formats */

#define Q8_0_BLOCK 32
#define Q8_0_BYTES 34
#define Q4_0_BLOCK 32
#define Q4_0_BYTES 18
#define Q4_K_BLOCK 256
#define Q4_K_BYTES 144
#define Q4_1_BLOCK 32
#define Q4_1_BYTES 20
#define Q5_K_BLOCK 256
#define Q5_K_BYTES 176
#define Q6_K_BLOCK 256
#define Q6_K_BYTES 210

static inline uint16_t rd16(const uint8_t *p) { return (uint16_t)(p[0] | (p[1] << 8)); }

size_t orc_row_bytes(int type, int64_t cols) {
    switch (type) {
    case ORC_F32: return (size_t)cols * 4;
    case ORC_F16: return (size_t)cols * 2;
    case ORC_Q8_0: return (size_t)(cols / Q8_0_BLOCK) * Q8_0_BYTES;
    case ORC_Q4_0: return (size_t)(cols / Q4_0_BLOCK) * Q4_0_BYTES;
    case ORC_Q4_K: return (size_t)(cols / Q4_K_BLOCK) * Q4_K_BYTES;
    case ORC_Q4_1: return (size_t)(cols / Q4_1_BLOCK) * Q4_1_BYTES;
    case ORC_Q5_K: return (size_t)(cols / Q5_K_BLOCK) * Q5_K_BYTES;
    case ORC_Q6_K: return (size_t)(cols / Q6_K_BLOCK) * Q6_K_BYTES;
    default: return 0;
    }
}

/* Q8_0FloatTensor.getFloat, tensor/standard/Q8_0FloatTensor.java:53-61: quant * scale. */
static inline float q8_0_get(const uint8_t *data, int64_t index) {
    int64_t b = index / Q8_0_BLOCK;
    int w = (int)(index % Q8_0_BLOCK);
    const uint8_t *blk = data + b * Q8_0_BYTES;
    int8_t quant = (int8_t)blk[2 + w];
    float scale = orc_f16_to_f32(rd16(blk));
    return (float)quant * scale;
}

/* Q4_0FloatTensor.getFloat, tensor/standard/Q4_0FloatTensor.java:56-79. */
static inline float q4_0_get(const uint8_t *data, int64_t index) {
    int64_t b = index / Q4_0_BLOCK;
    int w = (int)(index % Q4_0_BLOCK);
    const uint8_t *blk = data + b * Q4_0_BYTES;
    float scale = orc_f16_to_f32(rd16(blk));
    int8_t quant;
    if (w < Q4_0_BLOCK / 2) {
        quant = (int8_t)(blk[2 + w] & 0x0F);
    } else {
        quant = (int8_t)((blk[2 + w - Q4_0_BLOCK / 2] >> 4) & 0x0F);
    }
    quant = (int8_t)(quant - 8);
    return (float)quant * scale;
}

/* getScaleK4 / getMinK4, tensor/standard/Q4_KFloatTensor.java:68-86. */
static inline int q4k_scale(int j, const uint8_t *s) {
    return j < 4 ? (s[j] & 63) : ((s[j + 4] & 0xF) | ((s[j - 4] >> 6) << 4));
}
static inline int q4k_min(int j, const uint8_t *s) {
    return j < 4 ? (s[j + 4] & 63) : ((s[j + 4] >> 4) | ((s[j] >> 6) << 4));
}

/* Q4_KFloatTensor.getFloat, tensor/standard/Q4_KFloatTensor.java:88-122:
 * ((d * sc) * q) - (dmin * m), evaluated left to right in binary32, no contraction. */
static inline float q4_k_get(const uint8_t *data, int64_t index) {
    int64_t b = index / Q4_K_BLOCK;
    int within = (int)(index % Q4_K_BLOCK);
    const uint8_t *blk = data + b * Q4_K_BYTES;
    float d = orc_f16_to_f32(rd16(blk));
    float dmin = orc_f16_to_f32(rd16(blk + 2));
    const uint8_t *scales = blk + 4;
    const uint8_t *qs = blk + 16;
    int pair = within / 64, pos = within % 64;
    int sub, q;
    if (pos < 32) {
        sub = pair * 2;
        q = qs[pair * 32 + pos] & 0xF;
    } else {
        sub = pair * 2 + 1;
        q = (qs[pair * 32 + pos - 32] >> 4) & 0xF;
    }
    int sc = q4k_scale(sub, scales);
    int m = q4k_min(sub, scales);
    float t = d * (float)sc;
    t = t * (float)q;
    float u = dmin * (float)m;
    return t - u;
}

/* Q4_1FloatTensor.getFloat, tensor/standard/Q4_1FloatTensor.java:76-99: block = fp16 scale, fp16
 * minimum, 16 bytes of nibbles packed like Q4_0; nibble * scale + min with an unsigned nibble
 * (product rounded, then the sum: Java does not contract). */
static inline float q4_1_get(const uint8_t *data, int64_t index) {
    const uint8_t *blk = data + (index / Q4_1_BLOCK) * Q4_1_BYTES;
    int w = (int)(index % Q4_1_BLOCK);
    float scale = orc_f16_to_f32(rd16(blk));
    float min = orc_f16_to_f32(rd16(blk + 2));
    int nibble = w < 16 ? (blk[4 + w] & 0x0F) : ((blk[4 + w - 16] >> 4) & 0x0F);
    float t = (float)nibble * scale;
    return t + min;
}

/* Q5_KFloatTensor.getFloat, tensor/standard/Q5_KFloatTensor.java:87-127: block = d, dmin, 12 bytes of
 * 6-bit scales / minima packed as in Q4_K, 32 bytes qh (fifth bits), 128 bytes qs (low four bits).
 * Element e of pair p = e / 64: low nibble (e % 64 < 32) of qs[32 p + e % 32] with bit 2p of
 * qh[e % 32], or high nibble with bit 2p + 1; ((d * sc) * q) - (dmin * m). */
static inline float q5_k_get(const uint8_t *data, int64_t index) {
    const uint8_t *blk = data + (index / Q5_K_BLOCK) * Q5_K_BYTES;
    int within = (int)(index % Q5_K_BLOCK);
    float d = orc_f16_to_f32(rd16(blk));
    float dmin = orc_f16_to_f32(rd16(blk + 2));
    const uint8_t *scales = blk + 4, *qh = blk + 16, *qs = blk + 48;
    int pair = within / 64, pos = within % 64;
    int sub, q, high;
    if (pos < 32) {
        sub = pair * 2;
        q = qs[pair * 32 + pos] & 0xF;
        high = (qh[pos] >> (pair * 2)) & 1;
    } else {
        sub = pair * 2 + 1;
        q = (qs[pair * 32 + pos - 32] >> 4) & 0xF;
        high = (qh[pos - 32] >> (pair * 2 + 1)) & 1;
    }
    q += high * 16;
    float t = d * (float)q4k_scale(sub, scales);
    t = t * (float)q;
    float u = dmin * (float)q4k_min(sub, scales);
    return t - u;
}

/* Q6_KFloatTensor.getFloat, tensor/standard/Q6_KFloatTensor.java:64-117: block = 128 bytes ql, 64 bytes
 * qh, 16 signed byte scales, fp16 d. Half h = e / 128, group g = (e % 128) / 32, position p = e % 32:
 * low four bits from ql[64 h + 32 (g & 1) + p] (low nibble for g < 2, high nibble otherwise), top two
 * bits from qh[32 h + p] >> 2 g, value minus 32; scale index 8 h + 2 g + p / 16;
 * (d * scale) * q left to right. */
static inline float q6_k_get(const uint8_t *data, int64_t index) {
    const uint8_t *blk = data + (index / Q6_K_BLOCK) * Q6_K_BYTES;
    int within = (int)(index % Q6_K_BLOCK);
    float d = orc_f16_to_f32(rd16(blk + 208));
    int half = within / 128, in_half = within % 128;
    int group = in_half / 32, pos = in_half % 32;
    const uint8_t *ql = blk + half * 64, *qh = blk + 128 + half * 32;
    const int8_t *sc = (const int8_t *)(blk + 192 + half * 8);
    int lo = ql[(group & 1) * 32 + pos];
    lo = group < 2 ? (lo & 0xF) : (lo >> 4);
    int q = (lo | (((qh[pos] >> (2 * group)) & 3) << 4)) - 32;
    float t = d * (float)sc[pos / 16 + 2 * group];
    return t * (float)q;
}

float orc_get_float(int type, const void *data, int64_t index) {
    const uint8_t *p = (const uint8_t *)data;
    switch (type) {
    case ORC_F32: return ((const float *)data)[index];
    case ORC_F16: return orc_f16_to_f32(((const uint16_t *)data)[index]);
    case ORC_Q8_0: return q8_0_get(p, index);
    case ORC_Q4_0: return q4_0_get(p, index);
    case ORC_Q4_K: return q4_k_get(p, index);
    case ORC_Q4_1: return q4_1_get(p, index);
    case ORC_Q5_K: return q5_k_get(p, index);
    case ORC_Q6_K: return q6_k_get(p, index);
    default: return NAN;
    }
}

/* Whole-block decoders: the same values as the per-element getters, produced a block at a time
 * so that the dot products below do not redo the header decode per element. */
static void decode_span(int type, const uint8_t *data, int64_t first, int64_t n, float *out) {
    if (type == ORC_Q8_0 && first % Q8_0_BLOCK == 0 && n % Q8_0_BLOCK == 0) {
        const uint8_t *blk = data + (first / Q8_0_BLOCK) * Q8_0_BYTES;
        for (int64_t b = 0; b < n / Q8_0_BLOCK; b++, blk += Q8_0_BYTES) {
            float scale = orc_f16_to_f32(rd16(blk));
            for (int i = 0; i < 32; i++) out[b * 32 + i] = (float)(int8_t)blk[2 + i] * scale;
        }
    } else if (type == ORC_Q4_0 && first % Q4_0_BLOCK == 0 && n % Q4_0_BLOCK == 0) {
        const uint8_t *blk = data + (first / Q4_0_BLOCK) * Q4_0_BYTES;
        for (int64_t b = 0; b < n / Q4_0_BLOCK; b++, blk += Q4_0_BYTES) {
            float scale = orc_f16_to_f32(rd16(blk));
            for (int i = 0; i < 16; i++) {
                out[b * 32 + i] = (float)((int)(blk[2 + i] & 0x0F) - 8) * scale;
                out[b * 32 + 16 + i] = (float)((int)(blk[2 + i] >> 4) - 8) * scale;
            }
        }
    } else if (type == ORC_Q4_K && first % Q4_K_BLOCK == 0 && n % Q4_K_BLOCK == 0) {
        const uint8_t *blk = data + (first / Q4_K_BLOCK) * Q4_K_BYTES;
        for (int64_t b = 0; b < n / Q4_K_BLOCK; b++, blk += Q4_K_BYTES) {
            float d = orc_f16_to_f32(rd16(blk));
            float dmin = orc_f16_to_f32(rd16(blk + 2));
            const uint8_t *scales = blk + 4, *qs = blk + 16;
            for (int sub = 0; sub < 8; sub++) {
                float ds = d * (float)q4k_scale(sub, scales);
                float mm = dmin * (float)q4k_min(sub, scales);
                const uint8_t *q = qs + (sub / 2) * 32;
                float *o = out + b * 256 + sub * 32;
                if ((sub & 1) == 0)
                    for (int i = 0; i < 32; i++) o[i] = ds * (float)(q[i] & 0xF) - mm;
                else
                    for (int i = 0; i < 32; i++) o[i] = ds * (float)(q[i] >> 4) - mm;
            }
        }
    } else {
        for (int64_t i = 0; i < n; i++) out[i] = orc_get_float(type, data, first + i);
    }
}

void orc_dequant(int type, const void *data, int64_t n, float *out) {
    const uint8_t *p = (const uint8_t *)data;
    int64_t chunk = 1 << 16;
#pragma omp parallel for schedule(static) num_threads(orc_get_threads())
    for (int64_t c = 0; c < (n + chunk - 1) / chunk; c++) {
        int64_t first = c * chunk;
        int64_t len = n - first < chunk ? n - first : chunk;
        decode_span(type, p, first, len, out + first);
    }
}

/* ---------------------------------------------------------------- dot products */

/* FloatTensor.scalarDot, tensor/standard/FloatTensor.java:110-117:
 * result += thiz.getFloat(i) * that.getFloat(i), strictly sequential, product rounded first. */
static float scalar_dot(int type, const uint8_t *data, int64_t off, const float *x, int64_t size) {
    float result = 0.f;
    float buf[256];
    int64_t j = 0;
    while (j < size) {
        int64_t n = size - j < 256 ? size - j : 256;
        decode_span(type, data, off + j, n, buf);
        for (int64_t i = 0; i < n; i++) {
            float p = buf[i] * x[j + i];
            result += p;
        }
        j += n;
    }
    return result;
}

/* FloatVector.reduceLanes(ADD): lanes added in index order starting from lane 0 (what both
 * HotSpot's ordered float reduction and the library's scalar fallback do). */
static float reduce_lanes(const float *val, int lanes) {
    float r = val[0];
    for (int i = 1; i < lanes; i++) r += val[i];
    return r;
}

/* Q8_0FloatTensor.vectorDot, tensor/standard/Q8_0FloatTensor.java:142-229.
 * 256-bit: per block, lane l: ((x[l]*w[l] + x[8+l]*w[8+l]) + x[16+l]*w[16+l]) + x[24+l]*w[24+l],
 * then val = fma(sum, scale, val). 128-bit: two halves of 16, four lanes each. */
static float q8_0_vector_dot(const uint8_t *data, int64_t off, const float *x, int64_t size,
                             int bits) {
    float result = 0.f;
    int64_t j = 0;
    int64_t align = (-off) & (Q8_0_BLOCK - 1);
    if (align > size) align = size;
    if (align > 0) {
        result += scalar_dot(ORC_Q8_0, data, off, x, align);
        j += align;
    }
    int lanes = bits / 32;
    float val[8] = {0};
    const uint8_t *blk = data + ((off + j) / Q8_0_BLOCK) * Q8_0_BYTES;
    int64_t upper = size / Q8_0_BLOCK * Q8_0_BLOCK;
    for (; j < upper; j += Q8_0_BLOCK, blk += Q8_0_BYTES) {
        float scale = orc_f16_to_f32(rd16(blk));
        const int8_t *w = (const int8_t *)(blk + 2);
        if (bits == 256) {
            for (int l = 0; l < 8; l++) {
                float s0 = x[j + l] * (float)w[l];
                float s1 = x[j + 8 + l] * (float)w[8 + l];
                float s2 = x[j + 16 + l] * (float)w[16 + l];
                float s3 = x[j + 24 + l] * (float)w[24 + l];
                float s = ((s0 + s1) + s2) + s3;
                val[l] = fmaf(s, scale, val[l]);
            }
        } else {
            for (int i = 0; i < 2; i++) {
                for (int l = 0; l < 4; l++) {
                    float s0 = x[j + i * 16 + l] * (float)w[i * 16 + l];
                    float s1 = x[j + i * 16 + 4 + l] * (float)w[i * 16 + 4 + l];
                    float s2 = x[j + i * 16 + 8 + l] * (float)w[i * 16 + 8 + l];
                    float s3 = x[j + i * 16 + 12 + l] * (float)w[i * 16 + 12 + l];
                    float s = ((s0 + s1) + s2) + s3;
                    val[l] = fmaf(s, scale, val[l]);
                }
            }
        }
    }
    result += reduce_lanes(val, lanes);
    if (j < size) result += scalar_dot(ORC_Q8_0, data, off + j, x + j, size - j);
    return result;
}

/* Q4_0FloatTensor.vectorDot, tensor/standard/Q4_0FloatTensor.java:92-174.
 * lo = (byte & 0xF) - 8 covers elements 0..15, hi = (byte >>> 4) - 8 covers 16..31. */
static float q4_0_vector_dot(const uint8_t *data, int64_t off, const float *x, int64_t size,
                             int bits) {
    float result = 0.f;
    int64_t j = 0;
    int64_t align = (-off) & (Q4_0_BLOCK - 1);
    if (align > size) align = size;
    if (align > 0) {
        result += scalar_dot(ORC_Q4_0, data, off, x, align);
        j += align;
    }
    int lanes = bits / 32;
    float val[8] = {0};
    const uint8_t *blk = data + ((off + j) / Q4_0_BLOCK) * Q4_0_BYTES;
    int64_t upper = size / Q4_0_BLOCK * Q4_0_BLOCK;
    for (; j < upper; j += Q4_0_BLOCK, blk += Q4_0_BYTES) {
        float scale = orc_f16_to_f32(rd16(blk));
        float w[32];
        for (int i = 0; i < 16; i++) {
            w[i] = (float)((int)(blk[2 + i] & 0xF) - 8);
            w[16 + i] = (float)((int)(blk[2 + i] >> 4) - 8);
        }
        if (bits == 256) {
            for (int l = 0; l < 8; l++) {
                float s0 = x[j + l] * w[l];
                float s1 = x[j + 8 + l] * w[8 + l];
                float s2 = x[j + 16 + l] * w[16 + l];
                float s3 = x[j + 24 + l] * w[24 + l];
                float s = ((s0 + s1) + s2) + s3;
                val[l] = fmaf(s, scale, val[l]);
            }
        } else {
            for (int i = 0; i < 2; i++) {
                for (int l = 0; l < 4; l++) {
                    float s0 = x[j + (i * 4 + 0) * 4 + l] * w[i * 16 + l];
                    float s1 = x[j + (i * 4 + 1) * 4 + l] * w[i * 16 + 4 + l];
                    float s2 = x[j + (i * 4 + 2) * 4 + l] * w[i * 16 + 8 + l];
                    float s3 = x[j + (i * 4 + 3) * 4 + l] * w[i * 16 + 12 + l];
                    float s = ((s0 + s1) + s2) + s3;
                    val[l] = fmaf(s, scale, val[l]);
                }
            }
        }
    }
    result += reduce_lanes(val, lanes);
    if (j < size) result += scalar_dot(ORC_Q4_0, data, off + j, x + j, size - j);
    return result;
}

/* Q4_1FloatTensor.vectorDot, tensor/standard/Q4_1FloatTensor.java:110-192: per block the lanes carry
 * the products with the unsigned nibbles and the plain sum of the activations;
 * val = fma(products, scale, val), then val = fma(activations, min, val). */
static float q4_1_vector_dot(const uint8_t *data, int64_t off, const float *x, int64_t size, int bits) {
    float result = 0.f;
    int64_t j = 0;
    int64_t align = (-off) & (Q4_1_BLOCK - 1);
    if (align > size) align = size;
    if (align > 0) {
        result += scalar_dot(ORC_Q4_1, data, off, x, align);
        j += align;
    }
    int lanes = bits / 32;
    float val[8] = {0};
    const uint8_t *blk = data + ((off + j) / Q4_1_BLOCK) * Q4_1_BYTES;
    int64_t upper = size / Q4_1_BLOCK * Q4_1_BLOCK;
    for (; j < upper; j += Q4_1_BLOCK, blk += Q4_1_BYTES) {
        float scale = orc_f16_to_f32(rd16(blk));
        float min = orc_f16_to_f32(rd16(blk + 2));
        float w[32];
        for (int i = 0; i < 16; i++) {
            w[i] = (float)(blk[4 + i] & 0xF);
            w[16 + i] = (float)(blk[4 + i] >> 4);
        }
        if (bits == 256) {
            for (int l = 0; l < 8; l++) {
                float x0 = x[j + l], x1 = x[j + 8 + l], x2 = x[j + 16 + l], x3 = x[j + 24 + l];
                float s0 = x0 * w[l], s1 = x1 * w[8 + l], s2 = x2 * w[16 + l], s3 = x3 * w[24 + l];
                float products = ((s0 + s1) + s2) + s3;
                float activations = ((x0 + x1) + x2) + x3;
                val[l] = fmaf(products, scale, val[l]);
                val[l] = fmaf(activations, min, val[l]);
            }
        } else {
            for (int i = 0; i < 2; i++) {
                for (int l = 0; l < 4; l++) {
                    float x0 = x[j + (i * 4 + 0) * 4 + l], x1 = x[j + (i * 4 + 1) * 4 + l];
                    float x2 = x[j + (i * 4 + 2) * 4 + l], x3 = x[j + (i * 4 + 3) * 4 + l];
                    float s0 = x0 * w[i * 16 + l], s1 = x1 * w[i * 16 + 4 + l];
                    float s2 = x2 * w[i * 16 + 8 + l], s3 = x3 * w[i * 16 + 12 + l];
                    float products = ((s0 + s1) + s2) + s3;
                    float activations = ((x0 + x1) + x2) + x3;
                    val[l] = fmaf(products, scale, val[l]);
                    val[l] = fmaf(activations, min, val[l]);
                }
            }
        }
    }
    result += reduce_lanes(val, lanes);
    if (j < size) result += scalar_dot(ORC_Q4_1, data, off + j, x + j, size - j);
    return result;
}

float orc_dot(int type, const void *data, int64_t this_offset, const float *x, int64_t size) {
    const uint8_t *p = (const uint8_t *)data;
    /* Q8_0FloatTensor.java:90-99, Q4_0FloatTensor.java:82-88: vector path only for 128/256-bit
     * species; Q4_KFloatTensor.java:125-127 and everything else: scalarDot. */
    if (g_vector_bits != 0) {
        if (type == ORC_Q8_0) return q8_0_vector_dot(p, this_offset, x, size, g_vector_bits);
        if (type == ORC_Q4_0) return q4_0_vector_dot(p, this_offset, x, size, g_vector_bits);
        if (type == ORC_Q4_1) return q4_1_vector_dot(p, this_offset, x, size, g_vector_bits);
    }
    return scalar_dot(type, p, this_offset, x, size);
}

/* Eight rows at a time for the scalar mode: each row's sum is still strictly sequential in k
 * (mul rounded, then add), the eight independent rows are what the compiler may vectorise. */
#define RB 8
static void scalar_rows8(int type, const uint8_t *w, size_t row_bytes, const float *x, float *out,
                         int cols, int nrows) {
    float acc[RB] = {0};
    float buf[RB][256];
    float tb[256][RB];
    for (int c0 = 0; c0 < cols; c0 += 256) {
        int n = cols - c0 < 256 ? cols - c0 : 256;
        for (int r = 0; r < RB; r++) {
            if (r < nrows)
                decode_span(type, w + (size_t)r * row_bytes, c0, n, buf[r]);
            else
                memset(buf[r], 0, sizeof(float) * (size_t)n);
        }
        for (int k = 0; k < n; k++)
            for (int r = 0; r < RB; r++) tb[k][r] = buf[r][k];
        for (int k = 0; k < n; k++) {
            float xv = x[c0 + k];
            for (int r = 0; r < RB; r++) {
                float p = tb[k][r] * xv;
                acc[r] += p;
            }
        }
    }
    for (int r = 0; r < nrows; r++) out[r] = acc[r];
}

static void matmul_rows(int type, const uint8_t *w, const float *x, float *out, int r0, int r1,
                        int cols) {
    size_t rb = orc_row_bytes(type, cols);
    /* Q5_KFloatTensor.java:129-131 and Q6_KFloatTensor.java:119-121 always take scalarDot, like Q4_K. */
    int always_scalar = type == ORC_Q4_K || type == ORC_Q5_K || type == ORC_Q6_K;
    int blocked = (type == ORC_Q8_0 || type == ORC_Q4_0 || type == ORC_Q4_1 || always_scalar) &&
                  (g_vector_bits == 0 || always_scalar);
    if (blocked) {
        for (int r = r0; r < r1; r += RB) {
            int n = r1 - r < RB ? r1 - r : RB;
            scalar_rows8(type, w + (size_t)r * rb, rb, x, out + r, cols, n);
        }
    } else {
        for (int r = r0; r < r1; r++) out[r] = orc_dot(type, w, (int64_t)r * cols, x, cols);
    }
}

/* FloatTensor.matmul, tensor/standard/FloatTensor.java:123-125: one task per output row. */
void orc_matmul(int type, const void *w, const float *x, float *out, int rows, int cols) {
    const uint8_t *p = (const uint8_t *)w;
    int chunk = 64;
    int nchunks = (rows + chunk - 1) / chunk;
#pragma omp parallel for schedule(dynamic, 1) num_threads(orc_get_threads())
    for (int c = 0; c < nchunks; c++) {
        int r0 = c * chunk, r1 = r0 + chunk < rows ? r0 + chunk : rows;
        matmul_rows(type, p, x, out, r0, r1, cols);
    }
}

/* FloatTensor.matmul(context, that[], out[], dim0, dim1), FloatTensor.java:127-140. */
void orc_matmul_batch(int type, const void *w, const float *x, float *out, int rows, int cols,
                      int n) {
    const uint8_t *p = (const uint8_t *)w;
    int chunk = 64;
    int nchunks = (rows + chunk - 1) / chunk;
#pragma omp parallel for schedule(dynamic, 1) collapse(2) num_threads(orc_get_threads())
    for (int b = 0; b < n; b++) {
        for (int c = 0; c < nchunks; c++) {
            int r0 = c * chunk, r1 = r0 + chunk < rows ? r0 + chunk : rows;
            matmul_rows(type, p, x + (size_t)b * cols, out + (size_t)b * rows, r0, r1, cols);
        }
    }
}

/* ---------------------------------------------------------------- layer operations */

/* CpuOperations.rmsNorm, inference/op/CpuOperations.java:55-73. */
void orc_rmsnorm(float *out, const float *x, const float *weight, int size, float eps) {
    float ss = 0.f;
    for (int i = 0; i < size; i++) {
        float p = x[i] * x[i];
        ss = ss + p;
    }
    ss /= (float)size;
    ss += eps;
    ss = (float)(1.0 / sqrt((double)ss));
    for (int i = 0; i < size; i++) {
        float t = ss * x[i];
        out[i] = weight[i] * t;
    }
}

/* CpuOperations.rope, inference/op/CpuOperations.java:94-116: interleaved pairs. */
void orc_rope(float *q, float *k, const float *cr, const float *ci, int position, int dim,
              int kv_dim, int head_size) {
    for (int i = 0; i < dim; i += 2) {
        int hd = i % head_size;
        float fcr = cr[position * (head_size / 2) + hd / 2];
        float fci = ci[position * (head_size / 2) + hd / 2];
        int rotn = i < kv_dim ? 2 : 1;
        for (int v = 0; v < rotn; v++) {
            float *vec = v == 0 ? q : k;
            float v0 = vec[i], v1 = vec[i + 1];
            float a = v0 * fcr, b = v1 * fci;
            float c = v0 * fci, d = v1 * fcr;
            vec[i] = a - b;
            vec[i + 1] = c + d;
        }
    }
}

/* CpuOperations.swiGLU, inference/op/CpuOperations.java:255-260. */
void orc_swiglu(float *gate, const float *up, int n) {
    for (int i = 0; i < n; i++) {
        float v = gate[i];
        float e = (float)(1.0 + exp((double)(-v)));
        gate[i] = v / e;
    }
    for (int i = 0; i < n; i++) gate[i] = gate[i] * up[i];
}

/* Logits.argmax, inference/Logits.java:49-60: strict >, first index wins. */
int orc_argmax(const float *logits, int n) {
    int mi = 0;
    float mv = -INFINITY;
    for (int i = 0; i < n; i++) {
        if (logits[i] > mv) {
            mv = logits[i];
            mi = i;
        }
    }
    return mi;
}

/* RopeFrequencies.precomputeFreqsCis, model/loader/RopeFrequencies.java:14-54 (no scaling). */
void orc_rope_tables(int context_length, int head_size, double theta, float *cr, float *ci) {
    size_t n = 0;
    for (int pos = 0; pos < context_length; pos++) {
        for (int i = 0; i < head_size; i += 2) {
            float freq = (float)(1.0 / pow(theta, i / (double)head_size));
            float val = (float)pos * freq;
            cr[n] = (float)cos((double)val);
            ci[n] = (float)sin((double)val);
            n++;
        }
    }
}

/* CpuOperations.attention with AttentionShape.uniform, inference/op/CpuOperations.java:149-204;
 * scores via FloatTensor.scalarDot (ArrayFloatTensor does not override dot), softmax as
 * FloatTensor.softmaxInPlace (FloatTensor.java:248-256), weighted sum as saxpyInPlace in t order. */
void orc_attention(const float *q, const uint16_t *kcache, const uint16_t *vcache, float *att,
                   float *out, int position, int heads, int kv_mul, int head_size, int kv_dim,
                   int context_length) {
    float sqrt_hs = (float)sqrt((double)head_size);
#pragma omp parallel for schedule(static) num_threads(orc_get_threads())
    for (int h = 0; h < heads; h++) {
        const float *qh = q + (size_t)h * head_size;
        float *a = att + (size_t)h * context_length;
        for (int t = 0; t <= position; t++) {
            const uint16_t *kt = kcache + (size_t)t * kv_dim + (size_t)(h / kv_mul) * head_size;
            float score = 0.f;
            for (int i = 0; i < head_size; i++) {
                float p = qh[i] * orc_f16_to_f32(kt[i]);
                score += p;
            }
            a[t] = score / sqrt_hs;
        }
        float mx = -INFINITY;
        for (int t = 0; t <= position; t++) mx = a[t] > mx ? a[t] : mx; /* Float::max */
        for (int t = 0; t <= position; t++) a[t] = (float)exp((double)(a[t] - mx));
        float sum = 0.f;
        for (int t = 0; t <= position; t++) sum += a[t];
        for (int t = 0; t <= position; t++) a[t] = a[t] / sum;
        float *o = out + (size_t)h * head_size;
        for (int i = 0; i < head_size; i++) o[i] = 0.f;
        for (int t = 0; t <= position; t++) {
            const uint16_t *vt = vcache + (size_t)t * kv_dim + (size_t)(h / kv_mul) * head_size;
            float w = a[t];
            for (int i = 0; i < head_size; i++) {
                float p = w * orc_f16_to_f32(vt[i]);
                o[i] = p + o[i];
            }
        }
    }
}

/* KvBlockAddress.offset, backend/tornado/kernels/KvBlockAddress.java:59-71, plus the layer term
 * of layerOffset (:52-54); 64-bit so that pools beyond 2^31 elements address correctly. */
int64_t orc_kv_offset(const int32_t *block_table, int slot, int pos, int layer, int kv_dim,
                      int block_size, int max_blocks_per_slot, int num_layers) {
    int64_t block_stride = (int64_t)num_layers * block_size * kv_dim;
    int64_t layer_off = (int64_t)layer * block_size * kv_dim;
    int32_t phys = block_table[(int64_t)slot * max_blocks_per_slot + pos / block_size];
    return (int64_t)phys * block_stride + layer_off + (int64_t)(pos % block_size) * kv_dim;
}

/* ---------------------------------------------------------------- whole model */

enum {
    ROLE_TOKEN_EMBEDDING = 0,
    ROLE_ATTENTION_NORM = 1,
    ROLE_ATTENTION_QUERY = 2,
    ROLE_ATTENTION_KEY = 3,
    ROLE_ATTENTION_VALUE = 4,
    ROLE_ATTENTION_OUTPUT = 5,
    ROLE_FFN_NORM = 6,
    ROLE_FFN_GATE = 7,
    ROLE_FFN_UP = 8,
    ROLE_FFN_DOWN = 9,
    ROLE_OUTPUT_NORM = 10,
    ROLE_OUTPUT = 11,
    ROLE_COUNT = 12
};

struct orc_model {
    orc_config cfg;
    orc_tensor global[ROLE_COUNT];
    orc_tensor *layer[ROLE_COUNT];
    float *rope_cr, *rope_ci;
};

struct orc_state {
    const orc_model *m;
    float *x, *xb, *xb2, *q, *k, *v, *hb, *hb2, *att, *logits;
    uint16_t **kcache, **vcache; /* [layer][ctx*kvDim], fp16: State.allocateKeyValue default */
};

orc_model *orc_model_create(const orc_config *cfg) {
    orc_model *m = (orc_model *)calloc(1, sizeof(orc_model));
    m->cfg = *cfg;
    for (int r = 0; r < ROLE_COUNT; r++)
        m->layer[r] = (orc_tensor *)calloc((size_t)cfg->layers, sizeof(orc_tensor));
    size_t n = (size_t)cfg->ctx_len * (cfg->head_dim / 2);
    m->rope_cr = (float *)malloc(n * sizeof(float));
    m->rope_ci = (float *)malloc(n * sizeof(float));
    orc_rope_tables(cfg->ctx_len, cfg->head_dim, (double)cfg->theta, m->rope_cr, m->rope_ci);
    return m;
}

void orc_model_free(orc_model *m) {
    if (!m) return;
    for (int r = 0; r < ROLE_COUNT; r++) free(m->layer[r]);
    free(m->rope_cr);
    free(m->rope_ci);
    free(m);
}

int orc_model_set_tensor(orc_model *m, int role, int layer, int type, const void *data) {
    if (role < 0 || role >= ROLE_COUNT) return -1;
    orc_tensor t = {type, data};
    if (layer < 0)
        m->global[role] = t;
    else if (layer < m->cfg.layers)
        m->layer[role][layer] = t;
    else
        return -1;
    return 0;
}

void orc_model_set_rope(orc_model *m, const float *cr, const float *ci) {
    size_t n = (size_t)m->cfg.ctx_len * (m->cfg.head_dim / 2);
    memcpy(m->rope_cr, cr, n * sizeof(float));
    memcpy(m->rope_ci, ci, n * sizeof(float));
}
const float *orc_model_rope_cos(const orc_model *m) { return m->rope_cr; }
const float *orc_model_rope_sin(const orc_model *m) { return m->rope_ci; }

orc_state *orc_state_create(const orc_model *m) {
    const orc_config *c = &m->cfg;
    int kv_dim = c->kv_heads * c->head_dim;
    orc_state *s = (orc_state *)calloc(1, sizeof(orc_state));
    s->m = m;
    s->x = (float *)calloc((size_t)c->dim, 4);
    s->xb = (float *)calloc((size_t)c->dim, 4);
    s->xb2 = (float *)calloc((size_t)c->dim, 4);
    s->q = (float *)calloc((size_t)c->dim, 4);
    s->k = (float *)calloc((size_t)kv_dim, 4);
    s->v = (float *)calloc((size_t)kv_dim, 4);
    s->hb = (float *)calloc((size_t)c->hidden, 4);
    s->hb2 = (float *)calloc((size_t)c->hidden, 4);
    s->att = (float *)calloc((size_t)c->heads * c->ctx_len, 4);
    s->logits = (float *)calloc((size_t)c->vocab, 4);
    s->kcache = (uint16_t **)calloc((size_t)c->layers, sizeof(uint16_t *));
    s->vcache = (uint16_t **)calloc((size_t)c->layers, sizeof(uint16_t *));
    for (int l = 0; l < c->layers; l++) {
        s->kcache[l] = (uint16_t *)calloc((size_t)c->ctx_len * kv_dim, 2);
        s->vcache[l] = (uint16_t *)calloc((size_t)c->ctx_len * kv_dim, 2);
    }
    return s;
}

void orc_state_free(orc_state *s) {
    if (!s) return;
    for (int l = 0; l < s->m->cfg.layers; l++) {
        free(s->kcache[l]);
        free(s->vcache[l]);
    }
    free(s->kcache);
    free(s->vcache);
    free(s->x);
    free(s->xb);
    free(s->xb2);
    free(s->q);
    free(s->k);
    free(s->v);
    free(s->hb);
    free(s->hb2);
    free(s->att);
    free(s->logits);
    free(s);
}

static void layers_forward(const orc_model *m, orc_state *s, int token, int position) {
    const orc_config *c = &m->cfg;
    int dim = c->dim, hs = c->head_dim;
    int kv_dim = (c->dim * c->kv_heads) / c->heads;
    int kv_mul = c->heads / c->kv_heads;
    /* CpuOperations.embeddingLookup (:30-32): row copy through getFloat. */
    const orc_tensor *emb = &m->global[ROLE_TOKEN_EMBEDDING];
    decode_span(emb->type, (const uint8_t *)emb->data, (int64_t)token * dim, dim, s->x);

    for (int l = 0; l < c->layers; l++) {
        const orc_tensor *wq = &m->layer[ROLE_ATTENTION_QUERY][l];
        const orc_tensor *wk = &m->layer[ROLE_ATTENTION_KEY][l];
        const orc_tensor *wv = &m->layer[ROLE_ATTENTION_VALUE][l];
        const orc_tensor *wo = &m->layer[ROLE_ATTENTION_OUTPUT][l];
        const orc_tensor *w1 = &m->layer[ROLE_FFN_GATE][l];
        const orc_tensor *w3 = &m->layer[ROLE_FFN_UP][l];
        const orc_tensor *w2 = &m->layer[ROLE_FFN_DOWN][l];
        orc_rmsnorm(s->xb, s->x, (const float *)m->layer[ROLE_ATTENTION_NORM][l].data, dim, c->eps);
        orc_matmul(wq->type, wq->data, s->xb, s->q, dim, dim);
        orc_matmul(wk->type, wk->data, s->xb, s->k, kv_dim, dim);
        orc_matmul(wv->type, wv->data, s->xb, s->v, kv_dim, dim);
        orc_rope(s->q, s->k, m->rope_cr, m->rope_ci, position, dim, kv_dim, hs);
        /* appendKeyValue (:137-147) into an ArrayHalfFloatTensor: floatToFloat16 on write. */
        for (int i = 0; i < kv_dim; i++) {
            s->kcache[l][(size_t)position * kv_dim + i] = orc_f32_to_f16(s->k[i]);
            s->vcache[l][(size_t)position * kv_dim + i] = orc_f32_to_f16(s->v[i]);
        }
        orc_attention(s->q, s->kcache[l], s->vcache[l], s->att, s->xb, position, c->heads, kv_mul,
                      hs, kv_dim, c->ctx_len);
        orc_matmul(wo->type, wo->data, s->xb, s->xb2, dim, dim);
        for (int i = 0; i < dim; i++) s->x[i] = s->x[i] + s->xb2[i]; /* residualAdd :369-371 */
        orc_rmsnorm(s->xb, s->x, (const float *)m->layer[ROLE_FFN_NORM][l].data, dim, c->eps);
        orc_matmul(w1->type, w1->data, s->xb, s->hb, c->hidden, dim);
        orc_matmul(w3->type, w3->data, s->xb, s->hb2, c->hidden, dim);
        orc_swiglu(s->hb, s->hb2, c->hidden);
        orc_matmul(w2->type, w2->data, s->hb, s->xb, dim, c->hidden);
        for (int i = 0; i < dim; i++) s->x[i] = s->x[i] + s->xb[i];
    }
}

void orc_forward_no_logits(const orc_model *m, orc_state *s, int token, int position) {
    layers_forward(m, s, token, position);
}

/* InferenceCore.forwardJava, backend/cpu/InferenceCore.java:72-141. */
const float *orc_forward(const orc_model *m, orc_state *s, int token, int position) {
    const orc_config *c = &m->cfg;
    layers_forward(m, s, token, position);
    orc_rmsnorm(s->x, s->x, (const float *)m->global[ROLE_OUTPUT_NORM].data, c->dim, c->eps);
    /* absent output.weight => tied to the embedding, model/loader/AbstractModelLoader.java:255-266 */
    const orc_tensor *wcls = m->global[ROLE_OUTPUT].data ? &m->global[ROLE_OUTPUT]
                                                          : &m->global[ROLE_TOKEN_EMBEDDING];
    orc_matmul(wcls->type, wcls->data, s->x, s->logits, c->vocab, c->dim);
    return s->logits;
}

const float *orc_state_buffer(const orc_state *s, const char *name) {
    if (!strcmp(name, "x")) return s->x;
    if (!strcmp(name, "xb")) return s->xb;
    if (!strcmp(name, "xb2")) return s->xb2;
    if (!strcmp(name, "q")) return s->q;
    if (!strcmp(name, "k")) return s->k;
    if (!strcmp(name, "v")) return s->v;
    if (!strcmp(name, "hb")) return s->hb;
    if (!strcmp(name, "hb2")) return s->hb2;
    if (!strcmp(name, "att")) return s->att;
    if (!strcmp(name, "logits")) return s->logits;
    return NULL;
}
const uint16_t *orc_state_kcache(const orc_state *s, int layer) { return s->kcache[layer]; }
const uint16_t *orc_state_vcache(const orc_state *s, int layer) { return s->vcache[layer]; }

/* ---- sampler chain (inference/sampler/Sampler.java:63-110) ------------------------------------------------ */

typedef struct {
    float p;
    int idx;
} orc_cand;

static int orc_cand_desc(const void *a, const void *b) {
    const orc_cand *x = (const orc_cand *)a, *y = (const orc_cand *)b;
    if (x->p > y->p) return -1;
    if (x->p < y->p) return 1;
    return x->idx < y->idx ? -1 : (x->idx > y->idx ? 1 : 0);
}

int orc_sample(float *logits, int n, float temperature, float topp, float u, float *margin) {
    if (margin) *margin = 1.0f;
    if (temperature == 0.0f) { /* Sampler.java:66-68, Logits.java:49-60: first index of the maximum */
        int best = 0;
        for (int i = 1; i < n; ++i)
            if (logits[i] > logits[best]) best = i;
        return best;
    }
    /* Sampler.java:97-99: divideInPlace(temperature), softmaxInPlace (FloatTensor.java:240-256) */
    for (int i = 0; i < n; ++i) logits[i] = logits[i] / temperature;
    float mx = logits[0];
    for (int i = 1; i < n; ++i)
        if (logits[i] > mx) mx = logits[i];
    for (int i = 0; i < n; ++i) logits[i] = (float)exp((double)(logits[i] - mx));
    float sum = 0.0f;
    for (int i = 0; i < n; ++i) sum += logits[i];
    for (int i = 0; i < n; ++i) logits[i] = logits[i] / sum;
    if (topp <= 0.0f || topp >= 1.0f) { /* CategoricalSampler.java:13-25 */
        float cdf = 0.0f, best = 1.0f;
        int tok = n - 1, found = 0;
        for (int i = 0; i < n; ++i) {
            cdf += logits[i];
            if (!found && u < cdf) {
                tok = i;
                found = 1;
            }
            const float gap = fabsf(cdf - u);
            if (gap < best) best = gap;
        }
        if (margin) *margin = best;
        return tok;
    }
    /* ToppSampler.java:46-64: candidates at or above (1 - topp) / (n - 1) */
    const float cutoff = (1.0f - topp) / (float)(n - 1);
    orc_cand *c = (orc_cand *)malloc(sizeof(orc_cand) * (size_t)n);
    int n0 = 0;
    for (int i = 0; i < n; ++i)
        if (logits[i] >= cutoff) {
            c[n0].p = logits[i];
            c[n0].idx = i;
            ++n0;
        }
    /* ToppSampler.java:70-89: largest first until the running sum exceeds topp */
    qsort(c, (size_t)n0, sizeof(orc_cand), orc_cand_desc);
    float cumulative = 0.0f;
    int last = n0 - 1;
    for (int i = 0; i < n0; ++i) {
        cumulative += c[i].p;
        if (cumulative > topp) {
            last = i;
            break;
        }
    }
    /* ToppSampler.java:91-102 */
    const float r = u * cumulative;
    float cdf = 0.0f, best = 1.0f;
    int tok = c[last].idx, found = 0;
    for (int i = 0; i <= last; ++i) {
        cdf += c[i].p;
        if (!found && r < cdf) {
            tok = c[i].idx;
            found = 1;
        }
        const float gap = fabsf(cdf - r) / cumulative;
        if (gap < best) best = gap;
    }
    /* how close the nucleus boundary itself was to topp */
    {
        float run = 0.0f;
        for (int i = 0; i < n0 && i <= last + 1; ++i) {
            run += c[i].p;
            const float gap = fabsf(run - topp);
            if (gap < best && i >= last - 1) best = gap;
        }
    }
    if (margin) *margin = best;
    free(c);
    return tok;
}
