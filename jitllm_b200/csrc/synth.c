/*
 * Seeded synthetic weights in GGUF block formats (host code, no GPU).
 *
 * The reference ships decoders only (its fixtures use random payloads,
 * src/test/java/org/beehive/jitllm/backend/tornado/Qwen35SyntheticModel.java:123-170), so the
 * float -> Q8_0 / Q4_0 / Q4_K encoders here are written from the block definitions
 * (format/GGMLType.java:7,13,18-20 and the decoders in tensor/standard). Any encoder is valid
 * for parity work: parity is defined on the bytes both sides read.
 *
 * Values: i.i.d. N(0, std) from a counter-based generator, so a tensor is a pure function of
 * (seed, element index) and can be produced in parallel and in pieces.
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>
#ifdef _OPENMP
#include <omp.h>
#endif

enum { T_F32 = 0, T_Q4_0 = 2, T_Q8_0 = 8, T_Q4_K = 12 };

static inline uint64_t mix64(uint64_t z) {
    z += 0x9E3779B97F4A7C15ull;
    z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
    z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
    return z ^ (z >> 31);
}

/* Two standard normals from one 64-bit hash (Box-Muller). */
static inline void normal_pair(uint64_t seed, uint64_t pair_index, float *a, float *b) {
    uint64_t h = mix64(seed ^ mix64(pair_index));
    float u1 = ((float)(uint32_t)(h >> 40) + 1.0f) * (1.0f / 16777217.0f); /* (0,1) */
    float u2 = (float)(uint32_t)((h >> 8) & 0xFFFFFFu) * (1.0f / 16777216.0f);
    float r = sqrtf(-2.0f * logf(u1));
    float t = 6.28318530717958647692f * u2;
    *a = r * cosf(t);
    *b = r * sinf(t);
}

static void fill_span(float *out, int64_t first, int64_t n, uint64_t seed, float std) {
    /* `first` is even for every caller (block boundaries). */
    for (int64_t i = 0; i < n; i += 2) {
        float a, b;
        normal_pair(seed, (uint64_t)(first + i) >> 1, &a, &b);
        out[i] = a * std;
        if (i + 1 < n) out[i + 1] = b * std;
    }
}

/* binary32 -> binary16, round to nearest even (subnormals kept, overflow to infinity). */
static uint16_t to_half(float f) {
    uint32_t x;
    memcpy(&x, &f, 4);
    uint16_t sign = (uint16_t)((x >> 16) & 0x8000u);
    uint32_t ax = x & 0x7FFFFFFFu;
    if (ax >= 0x7F800000u) return (uint16_t)(sign | 0x7C00u | (ax > 0x7F800000u ? 0x200u : 0));
    if (ax >= 0x477FF000u) return (uint16_t)(sign | 0x7C00u);
    if (ax < 0x33000001u) return sign;
    int e = (int)(ax >> 23) - 127;
    uint32_t m = (ax & 0x7FFFFFu) | 0x800000u;
    int shift = e < -14 ? 13 + (-14 - e) : 13;
    uint32_t kept = m >> shift, rem = m & ((1u << shift) - 1u), half = 1u << (shift - 1);
    if (rem > half || (rem == half && (kept & 1u))) kept++;
    uint32_t out = e < -14 ? kept : (((uint32_t)(e + 15) << 10) + (kept - 0x400u));
    return (uint16_t)(sign | out);
}
static float from_half(uint16_t h) {
    uint32_t s = (uint32_t)(h & 0x8000u) << 16, e = (h >> 10) & 0x1F, m = h & 0x3FF, bits;
    if (e == 0) {
        if (!m) bits = s;
        else {
            int k = -1;
            do { m <<= 1; k++; } while (!(m & 0x400u));
            bits = s | ((uint32_t)(112 - k) << 23) | ((m & 0x3FFu) << 13);
        }
    } else if (e == 31) bits = s | 0x7F800000u | (m << 13);
    else bits = s | ((e + 112) << 23) | (m << 13);
    float f;
    memcpy(&f, &bits, 4);
    return f;
}

/* Q8_0: d = amax / 127, q = round(x / d). */
static void enc_q8_0(const float *x, uint8_t *blk) {
    float amax = 0.f;
    for (int i = 0; i < 32; i++) amax = fmaxf(amax, fabsf(x[i]));
    float d = amax / 127.0f;
    uint16_t hd = to_half(d);
    float id = d > 0.f ? 1.0f / d : 0.f;
    blk[0] = (uint8_t)(hd & 0xFF);
    blk[1] = (uint8_t)(hd >> 8);
    for (int i = 0; i < 32; i++) {
        int q = (int)lrintf(x[i] * id);
        q = q > 127 ? 127 : (q < -127 ? -127 : q);
        blk[2 + i] = (uint8_t)(int8_t)q;
    }
}

/* Q4_0: d = (value of largest magnitude) / -8, q = clamp(round(x / d) + 8, 0, 15);
 * element i in the low nibble of byte i, element i + 16 in the high nibble. */
static void enc_q4_0(const float *x, uint8_t *blk) {
    float amax = 0.f, vmax = 0.f;
    for (int i = 0; i < 32; i++)
        if (fabsf(x[i]) > amax) {
            amax = fabsf(x[i]);
            vmax = x[i];
        }
    float d = vmax / -8.0f;
    uint16_t hd = to_half(d);
    float id = d != 0.f ? 1.0f / d : 0.f;
    blk[0] = (uint8_t)(hd & 0xFF);
    blk[1] = (uint8_t)(hd >> 8);
    for (int i = 0; i < 16; i++) {
        int lo = (int)lrintf(x[i] * id) + 8, hi = (int)lrintf(x[i + 16] * id) + 8;
        lo = lo < 0 ? 0 : (lo > 15 ? 15 : lo);
        hi = hi < 0 ? 0 : (hi > 15 ? 15 : hi);
        blk[2 + i] = (uint8_t)(lo | (hi << 4));
    }
}

/* Q4_K: per 32-element sub-block an affine grid x ~ scale*q - min (q in 0..15, min >= 0);
 * scales and mins quantised to 6 bits against the super-block's fp16 d and dmin; 12 packed
 * scale bytes in the layout Q4_KFloatTensor.getScaleK4/getMinK4 unpack. */
static void enc_q4_k(const float *x, uint8_t *blk) {
    float scale[8], mn[8];
    float max_scale = 0.f, max_min = 0.f;
    for (int j = 0; j < 8; j++) {
        float lo = x[j * 32], hi = x[j * 32];
        for (int i = 1; i < 32; i++) {
            lo = fminf(lo, x[j * 32 + i]);
            hi = fmaxf(hi, x[j * 32 + i]);
        }
        if (lo > 0.f) lo = 0.f; /* the format stores -min as a non-negative quantity */
        scale[j] = (hi - lo) / 15.0f;
        mn[j] = -lo;
        max_scale = fmaxf(max_scale, scale[j]);
        max_min = fmaxf(max_min, mn[j]);
    }
    uint16_t hd = to_half(max_scale / 63.0f), hm = to_half(max_min / 63.0f);
    float d = from_half(hd), dmin = from_half(hm);
    uint8_t sc[8], mm[8];
    for (int j = 0; j < 8; j++) {
        int s = d > 0.f ? (int)lrintf(scale[j] / d) : 0;
        int m = dmin > 0.f ? (int)lrintf(mn[j] / dmin) : 0;
        sc[j] = (uint8_t)(s > 63 ? 63 : (s < 0 ? 0 : s));
        mm[j] = (uint8_t)(m > 63 ? 63 : (m < 0 ? 0 : m));
    }
    blk[0] = (uint8_t)(hd & 0xFF);
    blk[1] = (uint8_t)(hd >> 8);
    blk[2] = (uint8_t)(hm & 0xFF);
    blk[3] = (uint8_t)(hm >> 8);
    uint8_t *s = blk + 4;
    for (int j = 0; j < 4; j++) {
        s[j] = (uint8_t)((sc[j] & 63) | ((sc[j + 4] >> 4) << 6));
        s[j + 4] = (uint8_t)((mm[j] & 63) | ((mm[j + 4] >> 4) << 6));
        s[j + 8] = (uint8_t)((sc[j + 4] & 0xF) | ((mm[j + 4] & 0xF) << 4));
    }
    uint8_t *qs = blk + 16;
    for (int p = 0; p < 4; p++) {
        float d0 = d * sc[2 * p], m0 = dmin * mm[2 * p];
        float d1 = d * sc[2 * p + 1], m1 = dmin * mm[2 * p + 1];
        float i0 = d0 > 0.f ? 1.0f / d0 : 0.f, i1 = d1 > 0.f ? 1.0f / d1 : 0.f;
        for (int i = 0; i < 32; i++) {
            int lo = (int)lrintf((x[p * 64 + i] + m0) * i0);
            int hi = (int)lrintf((x[p * 64 + 32 + i] + m1) * i1);
            lo = lo < 0 ? 0 : (lo > 15 ? 15 : lo);
            hi = hi < 0 ? 0 : (hi > 15 ? 15 : hi);
            qs[p * 32 + i] = (uint8_t)(lo | (hi << 4));
        }
    }
}

static int block_elems(int type) { return type == T_Q4_K ? 256 : 32; }
static int block_bytes(int type) { return type == T_Q4_K ? 144 : (type == T_Q8_0 ? 34 : 18); }

int64_t jls_tensor_bytes(int type, int64_t n) {
    if (type == T_F32) return n * 4;
    if (type != T_Q4_0 && type != T_Q8_0 && type != T_Q4_K) return -1;
    if (n % block_elems(type)) return -1;
    return n / block_elems(type) * block_bytes(type);
}

/* Quantises n floats (a whole number of blocks) into dst. Returns 0, or -1 on a bad argument. */
int jls_quantize(int type, const float *src, int64_t n, void *dst, int threads) {
    if (jls_tensor_bytes(type, n) < 0 || type == T_F32) return -1;
    const int be = block_elems(type), bb = block_bytes(type);
    const int64_t nb = n / be;
    uint8_t *out = (uint8_t *)dst;
#ifdef _OPENMP
    if (threads <= 0) threads = omp_get_num_procs();
#endif
#pragma omp parallel for schedule(static) num_threads(threads)
    for (int64_t b = 0; b < nb; b++) {
        if (type == T_Q8_0) enc_q8_0(src + b * be, out + b * bb);
        else if (type == T_Q4_0) enc_q4_0(src + b * be, out + b * bb);
        else enc_q4_k(src + b * be, out + b * bb);
    }
    return 0;
}

/* n floats of N(0, std) for stream `seed`, starting at element `first` (even). */
int jls_fill_normal(float *out, int64_t first, int64_t n, uint64_t seed, float std, int threads) {
    if (first & 1) return -1;
    const int64_t chunk = 1 << 14;
    const int64_t nchunks = (n + chunk - 1) / chunk;
#ifdef _OPENMP
    if (threads <= 0) threads = omp_get_num_procs();
#endif
#pragma omp parallel for schedule(static) num_threads(threads)
    for (int64_t c = 0; c < nchunks; c++) {
        int64_t o = c * chunk, len = n - o < chunk ? n - o : chunk;
        fill_span(out + o, first + o, len, seed, std);
    }
    return 0;
}

/* Generates and encodes a whole tensor of n elements without materialising it in fp32. */
int jls_synth_tensor(int type, int64_t n, uint64_t seed, float std, void *dst, int threads) {
    if (jls_tensor_bytes(type, n) < 0) return -1;
    if (type == T_F32) return jls_fill_normal((float *)dst, 0, n, seed, std, threads);
    const int be = block_elems(type), bb = block_bytes(type);
    const int64_t nb = n / be;
    const int64_t group = 64; /* blocks per task */
    const int64_t ngroups = (nb + group - 1) / group;
    uint8_t *out = (uint8_t *)dst;
#ifdef _OPENMP
    if (threads <= 0) threads = omp_get_num_procs();
#endif
#pragma omp parallel for schedule(static) num_threads(threads)
    for (int64_t g = 0; g < ngroups; g++) {
        float buf[256];
        int64_t b0 = g * group, b1 = b0 + group < nb ? b0 + group : nb;
        for (int64_t b = b0; b < b1; b++) {
            fill_span(buf, b * be, be, seed, std);
            if (type == T_Q8_0) enc_q8_0(buf, out + b * bb);
            else if (type == T_Q4_0) enc_q4_0(buf, out + b * bb);
            else enc_q4_k(buf, out + b * bb);
        }
    }
    return 0;
}
