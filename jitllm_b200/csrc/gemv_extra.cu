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
// One warp per row of W, eight rows per CTA in flight, one, two or four activation rows staged per CTA (a batch
// or a prompt chunk re-uses every unpacked weight for that many rows). The kernel is bound by instruction issue and
// the L1 data pipe, not by memory latency (about eight instructions per weight: byte -> float without the slow
// integer conversion is a permute and a subtraction, then the multiply-add; narrow global loads because 210-byte
// blocks are only 2-byte aligned; requesting rows into L2 ahead of the loads changed nothing): 2.0-2.7 TB/s on a
// 128256 x 4096 matrix. A variant that kept the activation as 8-bit digits in registers (a column slice per warp,
// dp4a, partial sums meeting in shared memory) had a quarter fewer instructions and no shared-memory reads in its
// row loop, and was 1.4-2.2x slower: with a slice per warp too few bytes are in flight per SM.
//
// Where this kernel runs: a few rows (up to seven of the stand-alone operator, up to three of a model step) of a
// Q6_K matrix whose rows are not a whole number of 16-byte pieces. Other single rows go through the model's own
// mat-vec kernel (gemv.cu: whole rows by bulk copies, integer dot products), which reaches 0.7-0.9 of the HBM rate on
// these formats, and batches through the tensor-core kernel. It was the first kernel for these formats and stays as
// the one that takes any row length.
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

// Four bytes of `v`, each minus `bias`, as floats.
__device__ __forceinline__ void bytes4(uint32_t v, float *out, float bias_plus_2p23 = k2p23) {
    out[0] = byte_to_float<0>(v, bias_plus_2p23);
    out[1] = byte_to_float<1>(v, bias_plus_2p23);
    out[2] = byte_to_float<2>(v, bias_plus_2p23);
    out[3] = byte_to_float<3>(v, bias_plus_2p23);
}
__device__ __forceinline__ float dot4f(const float *w, const float4 x, float acc) {
    acc = fmaf(w[0], x.x, acc);
    acc = fmaf(w[1], x.y, acc);
    acc = fmaf(w[2], x.z, acc);
    return fmaf(w[3], x.w, acc);
}
__device__ __forceinline__ float4 lds4(const float *p) { return *reinterpret_cast<const float4 *>(p); }

// Every unpacker turns its lane's weights into floats once and then visits the NB activation rows the CTA holds
// (row r of the group at xs + r * xstride, its 32-element sums at xsum + r * sstride), adding into acc[r]: the
// unpacking, which is most of the work, is paid once for NB rows of a batch or a prompt chunk.

// ---- Q6_K: half a warp per 210-byte super-block; lane = (half h, bytes 4q..4q+3): 4 positions x 4 groups ----
// (210-byte blocks are only 2-byte aligned, hence the 16-bit loads.)
__device__ __forceinline__ uint32_t ldg_2x16(const uint8_t *p) { return ldg_u16(p) | (ldg_u16(p + 2) << 16); }
template <int NB>
__device__ __forceinline__ void superblock_q6_k(const uint8_t *blk, const float *xs, int xstride, const float *, int, int lane16,
                                                float (&acc)[NB]) {
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
    float wq[16], sc[4];
    constexpr float kBias = k2p23 + 32.0f;  // value - 32
    bytes4((ql0 & 0x0F0F0F0Fu) | ((qh << 4) & 0x30303030u), wq, kBias);
    bytes4((ql1 & 0x0F0F0F0Fu) | ((qh << 2) & 0x30303030u), wq + 4, kBias);
    bytes4(((ql0 >> 4) & 0x0F0F0F0Fu) | (qh & 0x30303030u), wq + 8, kBias);
    bytes4(((ql1 >> 4) & 0x0F0F0F0Fu) | ((qh >> 2) & 0x30303030u), wq + 12, kBias);
    bytes4(sc4, sc, k2p23 + 128.0f);
#pragma unroll
    for (int g = 0; g < 4; ++g) sc[g] *= d;
    const float *xp = xs + h * 128 + q4;
#pragma unroll
    for (int r = 0; r < NB; ++r, xp += xstride) {
        float t = sc[0] * dot4f(wq, lds4(xp), 0.f);
        t = fmaf(sc[1], dot4f(wq + 4, lds4(xp + 32), 0.f), t);
        t = fmaf(sc[2], dot4f(wq + 8, lds4(xp + 64), 0.f), t);
        acc[r] += fmaf(sc[3], dot4f(wq + 12, lds4(xp + 96), 0.f), t);
    }
}

// ---- Q5_K: half a warp per super-block; lane = (nibble pair p, bytes 8j..8j+7): low nibbles are sub-block 2p,
// high nibbles 2p+1; xsum holds the sum of every 32 activations (the minimum's factor), added by one lane per pair.
template <int NB>
__device__ __forceinline__ void superblock_q5_k(const uint8_t *blk, const float *xs, int xstride, const float *xsum, int sstride,
                                                int lane16, float (&acc)[NB]) {
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
    const float sc_lo = d * byte_to_float<0>(sc2, k2p23), sc_hi = d * byte_to_float<1>(sc2, k2p23);
    const float mn_lo = dmin * byte_to_float<0>(m2, k2p23), mn_hi = dmin * byte_to_float<1>(m2, k2p23);
    // five-bit values, four to a word: nibble | fifth bit << 4 (bit 2p of the qh byte for the low nibble, 2p + 1 for the high)
    const int b = 2 * p;
    float lo[8], hi[8];
    bytes4((qs.x & 0x0F0F0F0Fu) | (((qh.x >> b) << 4) & 0x10101010u), lo);
    bytes4((qs.y & 0x0F0F0F0Fu) | (((qh.y >> b) << 4) & 0x10101010u), lo + 4);
    bytes4(((qs.x >> 4) & 0x0F0F0F0Fu) | (((qh.x >> b) << 3) & 0x10101010u), hi);
    bytes4(((qs.y >> 4) & 0x0F0F0F0Fu) | (((qh.y >> b) << 3) & 0x10101010u), hi + 4);
    const float *xl = xs + p * 64 + j8;
    const float *sp = xsum + 2 * p;
#pragma unroll
    for (int r = 0; r < NB; ++r, xl += xstride, sp += sstride) {
        const float ql = dot4f(lo + 4, lds4(xl + 4), dot4f(lo, lds4(xl), 0.f));
        const float qhi = dot4f(hi + 4, lds4(xl + 36), dot4f(hi, lds4(xl + 32), 0.f));
        float t = fmaf(sc_hi, qhi, sc_lo * ql);
        if (j8 == 0) t -= fmaf(mn_hi, sp[1], mn_lo * sp[0]);
        acc[r] += t;
    }
}

// ---- Q4_1: eight 20-byte blocks per 256 elements; lane = (block, bytes 4j..4j+3) ----
template <int NB>
__device__ __forceinline__ void group_q4_1(const uint8_t *grp, const float *xs, int xstride, const float *xsum, int sstride, int lane,
                                           float (&acc)[NB]) {
    const int b = lane >> 2, j4 = (lane & 3) * 4;
    const uint8_t *blk = grp + b * kQ4_1Bytes;
    const uint32_t hdr = ldg_u32(blk);
    const uint32_t qs = ldg_u32(blk + 4 + j4);
    const float d = half_bits_to_float(hdr & 0xFFFFu), m = half_bits_to_float(hdr >> 16);
    float lo[4], hi[4];
    bytes4(qs & 0x0F0F0F0Fu, lo);
    bytes4((qs >> 4) & 0x0F0F0F0Fu, hi);
    const float *xl = xs + b * 32 + j4;
    const float *sp = xsum + b;
#pragma unroll
    for (int r = 0; r < NB; ++r, xl += xstride, sp += sstride) {
        float t = d * dot4f(hi, lds4(xl + 16), dot4f(lo, lds4(xl), 0.f));
        if (j4 == 0) t = fmaf(m, sp[0], t);
        acc[r] += t;
    }
}

// Grid: x = CTAs over the rows of W (eight warps, one row each per pass), y = groups of NB activation rows.
template <int TYPE, int NB>
__global__ void __launch_bounds__(kExtraThreads) gemv_extra_kernel(const uint8_t *__restrict__ w, const float *__restrict__ x,
                                                                   float *__restrict__ y, int rows, int cols, int n) {
    extern __shared__ __align__(16) float xs[];  // NB activation rows, then the sums of every 32 of their elements
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int b0 = blockIdx.y * NB;
    float *xsum = xs + NB * cols;
    const int nsum = cols >> 5;
    constexpr int kGroupBytes = TYPE == kQ6_K ? kQ6_KBytes : (TYPE == kQ5_K ? kQ5_KBytes : 8 * kQ4_1Bytes);
    const int groups = cols >> 8;
    const size_t rb = size_t(groups) * kGroupBytes;
    const int row_step = gridDim.x * kExtraWarps;
#pragma unroll
    for (int r = 0; r < NB; ++r) {
        const bool live = b0 + r < n;  // rows past the batch are zeros: their results are not stored
        const float *xr = x + size_t(live ? b0 + r : b0) * cols;
        for (int i = tid * 4; i < cols; i += kExtraThreads * 4)
            *reinterpret_cast<float4 *>(xs + r * cols + i) =
                live ? __ldg(reinterpret_cast<const float4 *>(xr + i)) : make_float4(0.f, 0.f, 0.f, 0.f);
    }
    __syncthreads();
    if constexpr (TYPE != kQ6_K) {
        for (int blk = warp; blk < NB * nsum; blk += kExtraWarps) {
            const float v = warp_sum(xs[blk * 32 + lane]);  // row r's sums at xsum + r * nsum: rows are whole blocks
            if (lane == 0) xsum[blk] = v;
        }
        __syncthreads();
    }
    for (int row = blockIdx.x * kExtraWarps + warp; row < rows; row += row_step) {
        const uint8_t *wr = w + size_t(row) * rb;
        float acc[NB];
#pragma unroll
        for (int r = 0; r < NB; ++r) acc[r] = 0.f;
        if constexpr (TYPE == kQ5_K || TYPE == kQ6_K) {
            // half a warp per super-block: two super-blocks per iteration (cols / 256 may be odd)
            const int half = lane >> 4, lane16 = lane & 15;
#pragma unroll 2
            for (int g = half; g < groups; g += 2) {
                const uint8_t *grp = wr + size_t(g) * kGroupBytes;
                if constexpr (TYPE == kQ6_K) superblock_q6_k<NB>(grp, xs + g * 256, cols, nullptr, 0, lane16, acc);
                else superblock_q5_k<NB>(grp, xs + g * 256, cols, xsum + g * 8, nsum, lane16, acc);
            }
        } else {
#pragma unroll 2
            for (int g = 0; g < groups; ++g)
                group_q4_1<NB>(wr + size_t(g) * kGroupBytes, xs + g * 256, cols, xsum + g * 8, nsum, lane, acc);
        }
#pragma unroll
        for (int r = 0; r < NB; ++r) {
            const float v = warp_sum(acc[r]);
            if (lane == 0 && b0 + r < n) y[size_t(b0 + r) * rows + row] = v;
        }
    }
}

constexpr size_t extra_smem(int nb, int cols) { return size_t(nb) * (size_t(cols) * 4 + size_t(cols / 32) * 4); }
// Activation rows per CTA: as many of 4 / 2 / 1 as the batch has and as leave room for three CTAs per SM.
constexpr size_t kExtraSmemBudget = 72 * 1024;

template <int TYPE, int NB>
cudaError_t launch_nb(const uint8_t *w, const float *x, float *y, int rows, int cols, int n, int sm_count, cudaStream_t stream) {
    const int per_cta = (rows + kExtraWarps - 1) / kExtraWarps;
    const int cap = (sm_count > 0 ? sm_count : 148) * 4;
    dim3 grid(unsigned(per_cta < cap ? per_cta : cap), unsigned((n + NB - 1) / NB));
    gemv_extra_kernel<TYPE, NB><<<grid, kExtraThreads, extra_smem(NB, cols), stream>>>(w, x, y, rows, cols, n);
    return cudaGetLastError();
}

template <int TYPE>
cudaError_t launch_type(const uint8_t *w, const float *x, float *y, int rows, int cols, int n, int sm_count,
                        cudaStream_t stream) {
    if (n >= 4 && extra_smem(4, cols) <= kExtraSmemBudget) return launch_nb<TYPE, 4>(w, x, y, rows, cols, n, sm_count, stream);
    if (n >= 2 && extra_smem(2, cols) <= kExtraSmemBudget) return launch_nb<TYPE, 2>(w, x, y, rows, cols, n, sm_count, stream);
    return launch_nb<TYPE, 1>(w, x, y, rows, cols, n, sm_count, stream);
}

template <int TYPE>
cudaError_t configure_type() {
    cudaError_t e;
    if ((e = cudaFuncSetAttribute(gemv_extra_kernel<TYPE, 1>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                  int(extra_smem(1, kGemvExtraMaxCols)))) != cudaSuccess)
        return e;
    if ((e = cudaFuncSetAttribute(gemv_extra_kernel<TYPE, 2>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                  int(kExtraSmemBudget))) != cudaSuccess)
        return e;
    return cudaFuncSetAttribute(gemv_extra_kernel<TYPE, 4>, cudaFuncAttributeMaxDynamicSharedMemorySize, int(kExtraSmemBudget));
}

}  // namespace

cudaError_t gemv_extra_configure() {
    cudaError_t e;
    if ((e = configure_type<kQ4_1>()) != cudaSuccess) return e;
    if ((e = configure_type<kQ5_K>()) != cudaSuccess) return e;
    return configure_type<kQ6_K>();
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
