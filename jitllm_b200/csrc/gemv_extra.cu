// Matrix-vector product for the block formats that real mixed-precision GGUF files add to the three the
// model's step kernels take: Q4_1 (tensor/standard/Q4_1FloatTensor.java:76-99 of the reference), Q5_K
// (Q5_KFloatTensor.java:87-127) and Q6_K (Q6_KFloatTensor.java:64-117). The weights stay in their on-disk
// layout; every lane unpacks eight or sixteen weights of a 256-element group from a few aligned words and
// multiplies them with the activation row held in shared memory, in binary32:
//
//   Q4_1  sum_i x_i (d q_i + m)                 = d * sum q_i x_i + m * sum x_i            per 32-element block
//   Q5_K  sum_i x_i (d sc q_i - dmin mn)        = d sc * sum q_i x_i - dmin mn * sum x_i   per 32-element sub-block
//   Q6_K  sum_i x_i (d sc (q_i - 32))           = d * sum_g sc_g * sum (q_i - 32) x_i      per 16-element scale group
//
// One warp per row, eight rows per CTA in flight, the activation staged once per CTA. The kernel is bound by
// instruction issue, not by memory latency (about eight instructions per weight: byte -> float without the
// slow integer conversion is a permute and a subtraction, then the multiply-add; requesting rows into L2 ahead
// of the loads changed nothing): 2.0-2.7 TB/s on a 128256 x 4096 matrix. Integer dot products against an
// 8-bit activation, as the model's own mat-vec does them, are the next step. This is the
// stand-alone operator behind jl_gemv / jl_gemv_dev (HBM-bound: every weight byte is read once); it is
// not wired into the decode step.
#include "gemv_extra.cuh"

namespace jl {
namespace {

constexpr int kExtraWarps = 8;
constexpr int kExtraThreads = kExtraWarps * 32;

__device__ __forceinline__ uint32_t ldg_u16(const uint8_t *p) {
    return uint32_t(__ldg(reinterpret_cast<const unsigned short *>(p)));
}
__device__ __forceinline__ uint32_t ldg_u32(const uint8_t *p) { return __ldg(reinterpret_cast<const uint32_t *>(p)); }

// Byte k of `word` as a float, minus `bias`, without an integer-to-float conversion (those issue at a fraction of
// the FMA rate): the byte becomes the low mantissa bits of 2^23, and one subtraction leaves byte - bias exactly.
template <int K>
__device__ __forceinline__ float byte_to_float(uint32_t word, float bias_plus_2p23) {
    return __uint_as_float(__byte_perm(word, 0x4B000000u, 0x7540u + K)) - bias_plus_2p23;
}
constexpr float k2p23 = 8388608.0f;

// Four bytes of `v`, each minus `bias`, against four floats.
__device__ __forceinline__ float dot4(uint32_t v, const float4 x, float acc, float bias_plus_2p23 = k2p23) {
    acc = fmaf(byte_to_float<0>(v, bias_plus_2p23), x.x, acc);
    acc = fmaf(byte_to_float<1>(v, bias_plus_2p23), x.y, acc);
    acc = fmaf(byte_to_float<2>(v, bias_plus_2p23), x.z, acc);
    return fmaf(byte_to_float<3>(v, bias_plus_2p23), x.w, acc);
}

// ---- Q6_K: half a warp per 210-byte super-block; lane = (half h, bytes 4q..4q+3): 4 positions x 4 groups ----
// (210-byte blocks are only 2-byte aligned, hence the 16-bit loads.)
__device__ __forceinline__ uint32_t ldg_2x16(const uint8_t *p) { return ldg_u16(p) | (ldg_u16(p + 2) << 16); }
__device__ __forceinline__ float superblock_q6_k(const uint8_t *blk, const float *xs, const float *, int lane16) {
    const int h = lane16 >> 3, q4 = (lane16 & 7) * 4;
    const uint32_t ql0 = ldg_2x16(blk + h * 64 + q4);
    const uint32_t ql1 = ldg_2x16(blk + h * 64 + 32 + q4);
    const uint32_t qh = ldg_2x16(blk + 128 + h * 32 + q4);
    const uint8_t *scp = blk + 192 + h * 8 + (q4 >> 4);
    // the four signed scales of this lane's groups, biased by 128 into unsigned bytes of one word
    const uint32_t sc4 = (uint32_t(__ldg(scp)) | (uint32_t(__ldg(scp + 2)) << 8) | (uint32_t(__ldg(scp + 4)) << 16) |
                          (uint32_t(__ldg(scp + 6)) << 24)) ^ 0x80808080u;
    const float d = half_bits_to_float(ldg_u16(blk + 208));
    // six-bit values of the four positions, one group per word: nibble | two bits of qh << 4
    const uint32_t v0 = (ql0 & 0x0F0F0F0Fu) | ((qh << 4) & 0x30303030u);
    const uint32_t v1 = (ql1 & 0x0F0F0F0Fu) | ((qh << 2) & 0x30303030u);
    const uint32_t v2 = ((ql0 >> 4) & 0x0F0F0F0Fu) | (qh & 0x30303030u);
    const uint32_t v3 = ((ql1 >> 4) & 0x0F0F0F0Fu) | ((qh >> 2) & 0x30303030u);
    const float *xp = xs + h * 128 + q4;
    constexpr float kBias = k2p23 + 32.0f;  // value - 32
    const float s0 = dot4(v0, *reinterpret_cast<const float4 *>(xp), 0.f, kBias);
    const float s1 = dot4(v1, *reinterpret_cast<const float4 *>(xp + 32), 0.f, kBias);
    const float s2 = dot4(v2, *reinterpret_cast<const float4 *>(xp + 64), 0.f, kBias);
    const float s3 = dot4(v3, *reinterpret_cast<const float4 *>(xp + 96), 0.f, kBias);
    constexpr float kScBias = k2p23 + 128.0f;
    float t = byte_to_float<0>(sc4, kScBias) * s0;
    t = fmaf(byte_to_float<1>(sc4, kScBias), s1, t);
    t = fmaf(byte_to_float<2>(sc4, kScBias), s2, t);
    t = fmaf(byte_to_float<3>(sc4, kScBias), s3, t);
    return d * t;
}

// ---- Q5_K: half a warp per super-block; lane = (nibble pair p, bytes 8j..8j+7): low nibbles are sub-block 2p,
// high nibbles 2p+1; xsum holds the sum of every 32 activations (the minimum's factor), added by one lane per pair.
__device__ __forceinline__ float superblock_q5_k(const uint8_t *blk, const float *xs, const float *xsum, int lane16) {
    const int p = lane16 >> 2, j8 = (lane16 & 3) * 8;
    const uint4 hdr = __ldg(reinterpret_cast<const uint4 *>(blk));  // d, dmin, 12 bytes of packed scales / minima
    const uint2 qs = __ldg(reinterpret_cast<const uint2 *>(blk + 48 + p * 32 + j8));
    const uint2 qh = __ldg(reinterpret_cast<const uint2 *>(blk + 16 + j8));
    const float d = half_bits_to_float(hdr.x & 0xFFFFu), dmin = half_bits_to_float(hdr.x >> 16);
    // Scale and minimum of sub-blocks 2p and 2p + 1 from the 12 packed bytes (hdr.y = bytes 0-3, hdr.z = 4-7,
    // hdr.w = 8-11): below sub-block 4 the low six bits of byte j / byte j + 4; from 4 on the low / high nibble
    // of byte j + 4 with the top two bits of byte j - 4 / byte j.
    const bool upper = p >= 2;
    const int sh = (p & 1) * 16;
    const uint32_t lo_mask = upper ? 0x0F0Fu : 0x3F3Fu;
    const uint32_t hi_mask = upper ? 0x3030u : 0u;
    const uint32_t sc2 = (((upper ? hdr.w : hdr.y) >> sh) & lo_mask) | ((hdr.y >> (sh + 2)) & hi_mask);
    const uint32_t m2 = (((upper ? (hdr.w >> 4) : hdr.z) >> sh) & lo_mask) | ((hdr.z >> (sh + 2)) & hi_mask);
    // five-bit values, four to a word: nibble | fifth bit << 4 (bit 2p of the qh byte for the low nibble, 2p + 1 for the high)
    const int b = 2 * p;
    const uint32_t lo_a = (qs.x & 0x0F0F0F0Fu) | (((qh.x >> b) << 4) & 0x10101010u);
    const uint32_t lo_b = (qs.y & 0x0F0F0F0Fu) | (((qh.y >> b) << 4) & 0x10101010u);
    const uint32_t hi_a = ((qs.x >> 4) & 0x0F0F0F0Fu) | (((qh.x >> b) << 3) & 0x10101010u);
    const uint32_t hi_b = ((qs.y >> 4) & 0x0F0F0F0Fu) | (((qh.y >> b) << 3) & 0x10101010u);
    const float *xl = xs + p * 64 + j8, *xh = xl + 32;
    float ql = dot4(lo_a, *reinterpret_cast<const float4 *>(xl), 0.f);
    ql = dot4(lo_b, *reinterpret_cast<const float4 *>(xl + 4), ql);
    float qhi = dot4(hi_a, *reinterpret_cast<const float4 *>(xh), 0.f);
    qhi = dot4(hi_b, *reinterpret_cast<const float4 *>(xh + 4), qhi);
    float r = d * (byte_to_float<0>(sc2, k2p23) * ql + byte_to_float<1>(sc2, k2p23) * qhi);
    if (j8 == 0) r -= dmin * (byte_to_float<0>(m2, k2p23) * xsum[2 * p] + byte_to_float<1>(m2, k2p23) * xsum[2 * p + 1]);
    return r;
}

// ---- Q4_1: eight 20-byte blocks per 256 elements; lane = (block, bytes 4j..4j+3) ----
__device__ __forceinline__ float group_q4_1(const uint8_t *grp, const float *xs, const float *xsum, int lane) {
    const int b = lane >> 2, j4 = (lane & 3) * 4;
    const uint8_t *blk = grp + b * kQ4_1Bytes;
    const uint32_t hdr = ldg_u32(blk);
    const uint32_t qs = ldg_u32(blk + 4 + j4);
    const float *xl = xs + b * 32 + j4;
    float dot = dot4(qs & 0x0F0F0F0Fu, *reinterpret_cast<const float4 *>(xl), 0.f);
    dot = dot4((qs >> 4) & 0x0F0F0F0Fu, *reinterpret_cast<const float4 *>(xl + 16), dot);
    float r = half_bits_to_float(hdr & 0xFFFFu) * dot;
    if (j4 == 0) r = fmaf(half_bits_to_float(hdr >> 16), xsum[b], r);
    return r;
}

template <int TYPE>
__global__ void __launch_bounds__(kExtraThreads) gemv_extra_kernel(const uint8_t *__restrict__ w, const float *__restrict__ x,
                                                                   float *__restrict__ y, int rows, int cols) {
    extern __shared__ __align__(16) float xs[];  // the activation row, then the sum of every 32 of its elements
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    x += size_t(blockIdx.y) * cols;
    y += size_t(blockIdx.y) * rows;
    float *xsum = xs + cols;
    constexpr int kGroupBytes = TYPE == kQ6_K ? kQ6_KBytes : (TYPE == kQ5_K ? kQ5_KBytes : 8 * kQ4_1Bytes);
    const int groups = cols >> 8;
    const size_t rb = size_t(groups) * kGroupBytes;
    const int row_step = gridDim.x * kExtraWarps;
    for (int i = tid * 4; i < cols; i += kExtraThreads * 4)
        *reinterpret_cast<float4 *>(xs + i) = __ldg(reinterpret_cast<const float4 *>(x + i));
    __syncthreads();
    if constexpr (TYPE != kQ6_K) {
        for (int blk = warp; blk < (cols >> 5); blk += kExtraWarps) {
            const float v = warp_sum(xs[blk * 32 + lane]);
            if (lane == 0) xsum[blk] = v;
        }
        __syncthreads();
    }
    for (int row = blockIdx.x * kExtraWarps + warp; row < rows; row += row_step) {
        const uint8_t *wr = w + size_t(row) * rb;
        float acc = 0.f;
        if constexpr (TYPE == kQ5_K || TYPE == kQ6_K) {
            // half a warp per super-block: two super-blocks per iteration (cols / 256 may be odd)
            const int half = lane >> 4, lane16 = lane & 15;
#pragma unroll 2
            for (int g = half; g < groups; g += 2) {
                const uint8_t *grp = wr + size_t(g) * kGroupBytes;
                if constexpr (TYPE == kQ6_K) acc += superblock_q6_k(grp, xs + g * 256, nullptr, lane16);
                else acc += superblock_q5_k(grp, xs + g * 256, xsum + g * 8, lane16);
            }
        } else {
#pragma unroll 2
            for (int g = 0; g < groups; ++g) acc += group_q4_1(wr + size_t(g) * kGroupBytes, xs + g * 256, xsum + g * 8, lane);
        }
        acc = warp_sum(acc);
        if (lane == 0) y[row] = acc;
    }
}

template <int TYPE>
cudaError_t launch_type(const uint8_t *w, const float *x, float *y, int rows, int cols, int n, int sm_count,
                        cudaStream_t stream) {
    const int per_cta = (rows + kExtraWarps - 1) / kExtraWarps;
    const int cap = (sm_count > 0 ? sm_count : 148) * 4;
    dim3 grid(unsigned(per_cta < cap ? per_cta : cap), unsigned(n));
    gemv_extra_kernel<TYPE><<<grid, kExtraThreads, size_t(cols) * 4 + size_t(cols / 32) * 4, stream>>>(w, x, y, rows, cols);
    return cudaGetLastError();
}

}  // namespace

cudaError_t gemv_extra_configure() {
    cudaError_t e;
    const int bytes = kGemvExtraMaxCols * 4 + kGemvExtraMaxCols / 32 * 4;
    if ((e = cudaFuncSetAttribute(gemv_extra_kernel<kQ4_1>, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes)) != cudaSuccess)
        return e;
    if ((e = cudaFuncSetAttribute(gemv_extra_kernel<kQ5_K>, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes)) != cudaSuccess)
        return e;
    return cudaFuncSetAttribute(gemv_extra_kernel<kQ6_K>, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes);
}

cudaError_t gemv_extra_launch(int type, const uint8_t *w, const float *x, float *y, int rows, int cols, int n, int sm_count,
                              cudaStream_t stream) {
    if (w == nullptr || x == nullptr || y == nullptr || rows <= 0 || n <= 0 || n > 65535 || cols <= 0 || cols % 256 != 0 ||
        cols > kGemvExtraMaxCols)
        return cudaErrorInvalidValue;
    switch (type) {
        case kQ4_1: return launch_type<kQ4_1>(w, x, y, rows, cols, n, sm_count, stream);
        case kQ5_K: return launch_type<kQ5_K>(w, x, y, rows, cols, n, sm_count, stream);
        case kQ6_K: return launch_type<kQ6_K>(w, x, y, rows, cols, n, sm_count, stream);
        default: return cudaErrorInvalidValue;
    }
}

}  // namespace jl
