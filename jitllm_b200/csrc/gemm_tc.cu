// Quantised matrix-matrix product on the 5th-generation tensor cores (tcgen05) for batched prefill
// and wide decode batches: Y[n][rows] = X[n][cols] . W[rows][cols]^T, W in GGUF block layout.
// What it computes: FloatTensor.matmul(context, that[], out[], dim0, dim1)
// (tensor/standard/FloatTensor.java:127-140 of the reference), n independent mat-vecs.
//
// Shape of the kernel: a CTA owns a 128-row x NT-token output tile; the accumulator lives in
// tensor memory (128 lanes x NT fp32 columns). Per 128-column K step all 256 threads build the
// operands in shared memory in the canonical K-major 128-byte-swizzled layout:
//   A = weights dequantised element-exactly in fp32 ((d*sc)*q - dmin*m etc.), rounded to fp16;
//   B = activations split as x = hi + lo with hi, lo fp16 (22 significant bits), so the only
//       rounding left is the fp16 rounding of the weights (rel-L2 ~3e-4 per product, inside the
//       1e-3 bar; the reference's own tensor-core prefill feeds single fp16 operands).
// One elected thread issues tcgen05.mma (M=128, N=NT, K=16) for the hi and lo operand, commits to
// an mbarrier, and the next K step is built while the tensor core works (two stages).
// The epilogue reads the accumulator with tcgen05.ld and writes fp32 (optionally + residual).
#include "gemm_tc.cuh"

#include "formats.cuh"

namespace jl {

namespace {

constexpr int kGemmThreads = 256;
constexpr int kTileM = 128;   // weight rows per CTA
constexpr int kStageK = 128;  // columns per pipeline stage (two 64-column swizzle atoms)

__device__ __forceinline__ void tmem_alloc(uint32_t *dst_smem, uint32_t ncols) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(dst_smem)),
                 "r"(ncols)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t ncols) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
__device__ __forceinline__ void tc_fence_before() {
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void tc_fence_after() {
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
}
// D[tmem] (+)= A[smem] * B[smem]; fp16 operands, fp32 accumulate.
__device__ __forceinline__ void umma_f16(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                         uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
        : "memory");
}
__device__ __forceinline__ void umma_commit(uint64_t *bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar))
                 : "memory");
}
// 32 lanes x 16 consecutive fp32 columns of the accumulator into registers.
__device__ __forceinline__ void tmem_ld16(uint32_t taddr, float (&v)[16]) {
    uint32_t r[16];
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
          "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
        : "r"(taddr));
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
    for (int i = 0; i < 16; ++i) v[i] = __uint_as_float(r[i]);
}

// Shared-memory matrix descriptor: K-major, 128-byte swizzle, rows of 64 fp16 (128 B), groups of
// eight rows 1024 B apart; `addr` is the shared address of the first element of the K slice.
__device__ __forceinline__ uint64_t smem_desc_sw128(uint32_t addr) {
    uint64_t d = 0;
    d |= uint64_t((addr >> 4) & 0x3FFFu);  // start address, 16-byte units
    d |= uint64_t(1) << 16;                // leading byte offset (unused for swizzled K-major)
    d |= uint64_t(1024 >> 4) << 32;        // stride byte offset between 8-row groups
    d |= uint64_t(1) << 46;                // descriptor version for sm_100
    d |= uint64_t(2) << 61;                // SWIZZLE_128B
    return d;
}
// Instruction descriptor: D fp32, A and B fp16, both K-major, M = 128, N = n.
__host__ __device__ constexpr uint32_t instr_desc_f16(int n) {
    return (1u << 4) | (uint32_t(n >> 3) << 17) | (uint32_t(kTileM >> 4) << 24);
}

// 16-byte chunk c of row r inside a [rows][64 fp16] swizzled tile.
__device__ __forceinline__ uint32_t sw128_offset(int r, int c) { return uint32_t(r) * 128u + uint32_t((c ^ (r & 7)) << 4); }

__device__ __forceinline__ uint32_t pack_half2(float a, float b) {
    const __half2 h = __halves2half2(__float2half_rn(a), __float2half_rn(b));
    return *reinterpret_cast<const uint32_t *>(&h);
}

// 64 consecutive weights of one row (columns k0 .. k0+63, k0 a multiple of 64), element-exact in
// fp32 like the reference's getFloat, then rounded to fp16 into eight 16-byte chunks.
template <int TYPE>
__device__ __forceinline__ void dequant64_to_half(const uint8_t *row, int k0, uint4 (&out)[8]) {
    float w[64];
    if constexpr (TYPE == kQ4_K) {
        const uint8_t *sb = row + size_t(k0 >> 8) * kQ4_KBytes;
        const int p = (k0 >> 6) & 3;
        const uint4 hdr = *reinterpret_cast<const uint4 *>(sb);
        const uint4 q0 = *reinterpret_cast<const uint4 *>(sb + 16 + p * 32);
        const uint4 q1 = *reinterpret_cast<const uint4 *>(sb + 32 + p * 32);
        const float d = half_bits_to_float(hdr.x & 0xFFFFu), dmin = half_bits_to_float(hdr.x >> 16);
        const uint32_t scA = hdr.y & 0x3F3F3F3Fu, mA = hdr.z & 0x3F3F3F3Fu;
        const uint32_t scB = (hdr.w & 0x0F0F0F0Fu) | ((hdr.y >> 2) & 0x30303030u);
        const uint32_t mB = ((hdr.w >> 4) & 0x0F0F0F0Fu) | ((hdr.z >> 2) & 0x30303030u);
        const int sh = (p & 1) * 16;
        const uint32_t scw = ((p < 2) ? scA : scB) >> sh, mw = ((p < 2) ? mA : mB) >> sh;
        const float ds0 = __fmul_rn(d, float(scw & 0xFFu)), ds1 = __fmul_rn(d, float((scw >> 8) & 0xFFu));
        const float mm0 = __fmul_rn(dmin, float(mw & 0xFFu)), mm1 = __fmul_rn(dmin, float((mw >> 8) & 0xFFu));
        const uint32_t qw[8] = {q0.x, q0.y, q0.z, q0.w, q1.x, q1.y, q1.z, q1.w};
#pragma unroll
        for (int i = 0; i < 8; ++i) {
#pragma unroll
            for (int b = 0; b < 4; ++b) {
                const uint32_t byte = (qw[i] >> (8 * b)) & 0xFFu;
                w[i * 4 + b] = __fsub_rn(__fmul_rn(ds0, float(byte & 0xFu)), mm0);
                w[32 + i * 4 + b] = __fsub_rn(__fmul_rn(ds1, float(byte >> 4)), mm1);
            }
        }
    } else if constexpr (TYPE == kQ4_0) {
        const uint32_t *wp = reinterpret_cast<const uint32_t *>(row + size_t(k0 >> 6) * 36);
        uint32_t v[9];
#pragma unroll
        for (int i = 0; i < 9; ++i) v[i] = wp[i];
        const float dA = half_bits_to_float(v[0] & 0xFFFFu), dB = half_bits_to_float(v[4] >> 16);
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const uint32_t qa = __funnelshift_r(v[i], v[i + 1], 16), qb = v[5 + i];
#pragma unroll
            for (int b = 0; b < 4; ++b) {
                const int a8 = (qa >> (8 * b)) & 0xFF, b8 = (qb >> (8 * b)) & 0xFF;
                w[i * 4 + b] = __fmul_rn(float((a8 & 0xF) - 8), dA);
                w[16 + i * 4 + b] = __fmul_rn(float((a8 >> 4) - 8), dA);
                w[32 + i * 4 + b] = __fmul_rn(float((b8 & 0xF) - 8), dB);
                w[48 + i * 4 + b] = __fmul_rn(float((b8 >> 4) - 8), dB);
            }
        }
    } else {
        const uint32_t *wp = reinterpret_cast<const uint32_t *>(row + size_t(k0 >> 6) * 68);
        uint32_t v[17];
#pragma unroll
        for (int i = 0; i < 17; ++i) v[i] = wp[i];
        const float dA = half_bits_to_float(v[0] & 0xFFFFu), dB = half_bits_to_float(v[8] >> 16);
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            const uint32_t qa = __funnelshift_r(v[i], v[i + 1], 16), qb = v[9 + i];
#pragma unroll
            for (int b = 0; b < 4; ++b) {
                w[i * 4 + b] = __fmul_rn(float(int8_t((qa >> (8 * b)) & 0xFF)), dA);
                w[32 + i * 4 + b] = __fmul_rn(float(int8_t((qb >> (8 * b)) & 0xFF)), dB);
            }
        }
    }
#pragma unroll
    for (int c = 0; c < 8; ++c) {
        out[c].x = pack_half2(w[8 * c + 0], w[8 * c + 1]);
        out[c].y = pack_half2(w[8 * c + 2], w[8 * c + 3]);
        out[c].z = pack_half2(w[8 * c + 4], w[8 * c + 5]);
        out[c].w = pack_half2(w[8 * c + 6], w[8 * c + 7]);
    }
}

template <int NT>
struct GemmSmem {
    static constexpr int a_sub = kTileM * 128;  // one 64-column atom of A: 16 KB
    static constexpr int b_sub = NT * 128;      // one 64-column atom of B
    static constexpr int stage = 2 * a_sub + 4 * b_sub;  // A(2 atoms) + B hi (2) + B lo (2)
    static constexpr int total = 2 * stage + 1024 /*alignment slack*/ + 64 /*barriers, tmem ptr*/;
};

template <int TYPE, int NT>
__global__ void __launch_bounds__(kGemmThreads, 1) gemm_tc_kernel(const GemmArgs a) {
    extern __shared__ uint8_t smem_raw[];
    using S = GemmSmem<NT>;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    // 1024-byte aligned base: the swizzle pattern is a function of the shared address.
    uint8_t *base = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint64_t *bars = reinterpret_cast<uint64_t *>(base + 2 * S::stage);  // [0,1] stage free, [2] unused
    uint32_t *tmem_ptr = reinterpret_cast<uint32_t *>(base + 2 * S::stage + 32);
    constexpr uint32_t tmem_cols = NT < 32 ? 32 : NT;

    const int row0 = blockIdx.x * kTileM;
    const int tok0 = blockIdx.y * NT;
    const size_t rowb = size_t(row_bytes(TYPE, a.cols));
    const int nk = a.cols / kStageK;

    if (warp == 0) tmem_alloc(tmem_ptr, tmem_cols);
    if (tid == 0) {
        mbar_init(bars + 0, 1);
        mbar_init(bars + 1, 1);
        mbar_fence_init();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_d = *tmem_ptr;
    constexpr uint32_t idesc = instr_desc_f16(NT);

    // Operand-building roles: thread t dequantises 64 columns (atom t>>7) of weight row t&127.
    const int a_row = tid & 127, a_atom = tid >> 7;
    const int grow = row0 + a_row;
    const uint8_t *wrow = a.w + size_t(min(grow, a.rows - 1)) * rowb;
    bool failed = false;
    uint32_t free_parity[2] = {0, 0};

    for (int it = 0; it < nk; ++it) {
        const int s = it & 1;
        uint8_t *st = base + size_t(s) * S::stage;
        if (it >= 2) {
            // The tensor core must be done reading this stage (commit of iteration it-2).
            bool ok = mbar_wait_bounded(bars + s, free_parity[s]);
            free_parity[s] ^= 1u;
            if (!ok) failed = true;
        }
        if (__syncthreads_or(failed)) {
            failed = true;
            break;
        }
        const int k0 = it * kStageK;
        {   // A: one atom line per thread
            uint4 chunks[8];
            dequant64_to_half<TYPE>(wrow, k0 + a_atom * 64, chunks);
            uint8_t *tile = st + size_t(a_atom) * S::a_sub;
            const bool valid = grow < a.rows;
#pragma unroll
            for (int c = 0; c < 8; ++c)
                *reinterpret_cast<uint4 *>(tile + sw128_offset(a_row, c)) = valid ? chunks[c] : make_uint4(0, 0, 0, 0);
        }
        // B: 16-byte chunks of eight activations, hi and lo parts
        for (int ch = tid; ch < NT * 16; ch += kGemmThreads) {
            const int t = ch >> 4, kc = ch & 15;
            const int atom = kc >> 3, c = kc & 7;
            float x[8];
            const int tok = tok0 + t;
            if (tok < a.n) {
                const float4 *src = reinterpret_cast<const float4 *>(a.x + size_t(tok) * a.cols + k0 + kc * 8);
                const float4 u0 = src[0], u1 = src[1];
                x[0] = u0.x; x[1] = u0.y; x[2] = u0.z; x[3] = u0.w;
                x[4] = u1.x; x[5] = u1.y; x[6] = u1.z; x[7] = u1.w;
            } else {
#pragma unroll
                for (int i = 0; i < 8; ++i) x[i] = 0.f;
            }
            float lo[8];
#pragma unroll
            for (int i = 0; i < 8; ++i) lo[i] = x[i] - __half2float(__float2half_rn(x[i]));
            const uint32_t off = sw128_offset(t, c);
            uint8_t *bh = st + 2 * S::a_sub + size_t(atom) * S::b_sub;
            uint8_t *bl = bh + 2 * S::b_sub;
            *reinterpret_cast<uint4 *>(bh + off) = make_uint4(pack_half2(x[0], x[1]), pack_half2(x[2], x[3]),
                                                             pack_half2(x[4], x[5]), pack_half2(x[6], x[7]));
            *reinterpret_cast<uint4 *>(bl + off) = make_uint4(pack_half2(lo[0], lo[1]), pack_half2(lo[2], lo[3]),
                                                             pack_half2(lo[4], lo[5]), pack_half2(lo[6], lo[7]));
        }
        // Generic-proxy writes -> visible to the tensor core's (async proxy) reads.
        fence_proxy_async();
        tc_fence_before();
        __syncthreads();
        if (tid == 0) {
            tc_fence_after();
            const uint32_t a_addr = smem_u32(st);
            const uint32_t bh_addr = smem_u32(st + 2 * S::a_sub);
            const uint32_t bl_addr = bh_addr + 2 * S::b_sub;
#pragma unroll
            for (int atom = 0; atom < 2; ++atom) {
#pragma unroll
                for (int k16 = 0; k16 < 4; ++k16) {
                    const uint64_t da = smem_desc_sw128(a_addr + atom * S::a_sub + k16 * 32);
                    const uint64_t dbh = smem_desc_sw128(bh_addr + atom * S::b_sub + k16 * 32);
                    const uint64_t dbl = smem_desc_sw128(bl_addr + atom * S::b_sub + k16 * 32);
                    umma_f16(tmem_d, da, dbh, idesc, (it > 0 || atom > 0 || k16 > 0) ? 1u : 0u);
                    umma_f16(tmem_d, da, dbl, idesc, 1u);
                }
            }
            umma_commit(bars + s);  // arrives when every MMA issued so far has completed
        }
    }

    // Wait for the last commit (covers all earlier MMAs), then read the accumulator.
    if (!failed && nk > 0) {
        const int s = (nk - 1) & 1;
        if (!mbar_wait_bounded(bars + s, free_parity[s])) failed = true;
    }
    failed = __syncthreads_or(failed);
    tc_fence_after();
    if (!failed && warp < 4) {
        const int row = row0 + warp * 32 + lane;  // TMEM lane = output row of the tile
#pragma unroll 1
        for (int c0 = 0; c0 < NT; c0 += 16) {
            float v[16];
            tmem_ld16(tmem_d + (uint32_t(warp * 32) << 16) + uint32_t(c0), v);
            if (row < a.rows) {
#pragma unroll
                for (int j = 0; j < 16; ++j) {
                    const int tok = tok0 + c0 + j;
                    if (tok < a.n) {
                        float out = v[j];
                        if (a.res != nullptr) out = a.res[size_t(tok) * a.rows + row] + out;
                        a.y[size_t(tok) * a.rows + row] = out;
                    }
                }
            }
        }
    }
    if (failed && tid == 0) atomicExch(a.status, kDevTimeout);
    tc_fence_before();
    __syncthreads();
    if (warp == 0) tmem_dealloc(tmem_d, tmem_cols);
}

template <int TYPE, int NT>
cudaError_t launch_nt(const GemmArgs &a, cudaStream_t stream) {
    dim3 grid((a.rows + kTileM - 1) / kTileM, (a.n + NT - 1) / NT);
    gemm_tc_kernel<TYPE, NT><<<grid, kGemmThreads, GemmSmem<NT>::total, stream>>>(a);
    return cudaGetLastError();
}

template <int TYPE>
cudaError_t launch_type(const GemmArgs &a, cudaStream_t stream) {
    if (a.n <= 16) return launch_nt<TYPE, 16>(a, stream);
    if (a.n <= 32) return launch_nt<TYPE, 32>(a, stream);
    if (a.n <= 64) return launch_nt<TYPE, 64>(a, stream);
    return launch_nt<TYPE, 128>(a, stream);
}

template <int TYPE>
cudaError_t configure_type() {
    cudaError_t e;
    if ((e = cudaFuncSetAttribute(gemm_tc_kernel<TYPE, 16>, cudaFuncAttributeMaxDynamicSharedMemorySize, GemmSmem<16>::total)) != cudaSuccess) return e;
    if ((e = cudaFuncSetAttribute(gemm_tc_kernel<TYPE, 32>, cudaFuncAttributeMaxDynamicSharedMemorySize, GemmSmem<32>::total)) != cudaSuccess) return e;
    if ((e = cudaFuncSetAttribute(gemm_tc_kernel<TYPE, 64>, cudaFuncAttributeMaxDynamicSharedMemorySize, GemmSmem<64>::total)) != cudaSuccess) return e;
    return cudaFuncSetAttribute(gemm_tc_kernel<TYPE, 128>, cudaFuncAttributeMaxDynamicSharedMemorySize, GemmSmem<128>::total);
}

}  // namespace

cudaError_t gemm_tc_configure() {
    cudaError_t e;
    if ((e = configure_type<kQ4_K>()) != cudaSuccess) return e;
    if ((e = configure_type<kQ4_0>()) != cudaSuccess) return e;
    return configure_type<kQ8_0>();
}

cudaError_t gemm_tc_launch(const GemmArgs &a, cudaStream_t stream) {
    if (a.cols <= 0 || a.cols % 256 != 0 || a.rows <= 0 || a.n <= 0) return cudaErrorInvalidValue;
    switch (a.type) {
        case kQ4_K: return launch_type<kQ4_K>(a, stream);
        case kQ4_0: return launch_type<kQ4_0>(a, stream);
        case kQ8_0: return launch_type<kQ8_0>(a, stream);
        default: return cudaErrorInvalidValue;
    }
}

}  // namespace jl
