// Quantised matrix-matrix product on the 5th-generation tensor cores (tcgen05) for batched decode
// and chunked prefill: Y[n][rows] = X[n][cols] . W[rows][cols]^T, W in GGUF block layout.
// What it computes: FloatTensor.matmul(context, that[], out[], dim0, dim1)
// (tensor/standard/FloatTensor.java:127-140 of the reference), n independent mat-vecs.
//
// Shape of the kernel. A CTA owns a 128-row x NT-token output tile over a range of columns (the
// grid's z axis splits the columns so that small matrices still fill the GPU); the accumulator
// lives in tensor memory (128 lanes x NT fp32 columns).
//   * Weight bytes arrive exactly once, as they are stored: 128 threads each request their row's
//     next 256 columns (144 or 272 bytes) with a bulk async copy (the TMA engine) into a ring of
//     raw stages, completing on an mbarrier. Nothing waits on global-memory latency.
//   * All 512 threads turn a raw half-stage (128 columns) into the A operand: weights dequantised
//     element-exactly in fp32 ((d*sc)*q - dmin*m etc., as the reference's getFloat), rounded once
//     to fp16, stored K-major with the 128-byte swizzle the tensor core expects.
//   * B = activations split as x = hi + lo with hi, lo fp16 (22 significant bits), so the only
//     rounding left is the fp16 rounding of the weights (rel-L2 ~3e-4 per product, inside the
//     1e-3 bar; the reference's own tensor-core prefill feeds single fp16 operands).
//   * One thread issues tcgen05.mma (M=128, N=NT, K=16) for hi and lo and commits to an mbarrier;
//     the next operands are built while the tensor core works (two operand stages).
//   * Epilogue: tcgen05.ld by all warps; with split columns the partial tile goes to a workspace
//     and the CTA that arrives last at the tile's counter adds the partials in split order (so the
//     result does not depend on which CTA finished first), adds the residual and writes Y.
// Every wait is bounded; a wait that runs out sets the status word and the CTA leaves.
#include "gemm_tc.cuh"

#include "formats.cuh"

#include <cuda.h>

#include <cstring>

namespace jl {

namespace {

constexpr int kGemmThreads = 512;
constexpr int kTileM = 128;    // weight rows per CTA
constexpr int kStageK = 128;   // columns per operand stage (two 64-column swizzle atoms)
constexpr int kRawK = 256;     // columns per raw stage (one Q4_K super-block per row)
constexpr int kMaxSplit = 8;

// One box of a 2-D tensor map into shared memory; x counts 32-bit words along a row (x * 4 bytes is
// a multiple of 16 for every raw stage: 144- and 272-byte steps), y counts rows.
__device__ __forceinline__ void tma_load_2d(void *dst_smem, const CUtensorMap *map, int x, int y, uint64_t *bar,
                                            uint64_t policy) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes.L2::cache_hint "
        "[%0], [%1, {%2, %3}], [%4], %5;" ::"r"(smem_u32(dst_smem)),
        "l"(map), "r"(x), "r"(y), "r"(smem_u32(bar)), "l"(policy)
        : "memory");
}

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


template <int TYPE>
struct RawFmt {
    static constexpr int row_bytes = (TYPE == kQ8_0) ? 272 : 144;  // 256 columns of one row
    static constexpr int stages = (TYPE == kQ8_0) ? 2 : 3;
    static constexpr int stage_bytes = kTileM * row_bytes;
};

// 32 consecutive weights of one row out of a raw stage in shared memory: `row_u32` is the shared
// address of the row's 256-column slice, `unit` the 64-column unit inside it (0..3), `half` the
// 32-column half of the unit. Element-exact in fp32, then rounded to fp16 into four 16-byte chunks.
template <int TYPE>
__device__ __forceinline__ void dequant32_to_half(uint32_t row_u32, int unit, int half, uint4 (&out)[4]) {
    float w[32];
    if constexpr (TYPE == kQ4_K) {
        // tensor/standard/Q4_KFloatTensor.java:68-122: unit p holds sub-blocks 2p (low nibbles) and
        // 2p+1 (high nibbles) of the same 32 bytes.
        const uint4 hdr = lds128(row_u32);
        const uint4 q0 = lds128(row_u32 + 16 + unit * 32);
        const uint4 q1 = lds128(row_u32 + 32 + unit * 32);
        const float d = half_bits_to_float(hdr.x & 0xFFFFu), dmin = half_bits_to_float(hdr.x >> 16);
        uint32_t scw, mw;
        if (unit < 2) {
            scw = hdr.y & 0x3F3F3F3Fu;
            mw = hdr.z & 0x3F3F3F3Fu;
        } else {
            scw = (hdr.w & 0x0F0F0F0Fu) | ((hdr.y >> 2) & 0x30303030u);
            mw = ((hdr.w >> 4) & 0x0F0F0F0Fu) | ((hdr.z >> 2) & 0x30303030u);
        }
        const int sh = (unit & 1) * 16 + half * 8;
        const float ds = __fmul_rn(d, float((scw >> sh) & 0xFFu));
        const float mm = __fmul_rn(dmin, float((mw >> sh) & 0xFFu));
        const uint32_t qw[8] = {q0.x, q0.y, q0.z, q0.w, q1.x, q1.y, q1.z, q1.w};
        const int nib = half * 4;
#pragma unroll
        for (int i = 0; i < 8; ++i) {
#pragma unroll
            for (int b = 0; b < 4; ++b) {
                const uint32_t q = (qw[i] >> (8 * b + nib)) & 0xFu;
                w[i * 4 + b] = __fsub_rn(__fmul_rn(ds, float(q)), mm);
            }
        }
    } else if constexpr (TYPE == kQ4_0) {
        // tensor/standard/Q4_0FloatTensor.java:56-79: a unit is two 18-byte blocks; element i < 16
        // is the low nibble of byte i, element i >= 16 the high nibble of byte i - 16.
        const uint32_t base = row_u32 + unit * 36 + half * 16;
        uint32_t t[5];
#pragma unroll
        for (int i = 0; i < 5; ++i) t[i] = lds32(base + 4 * i);
        const float d = half_bits_to_float(half == 0 ? (t[0] & 0xFFFFu) : (t[0] >> 16));
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const uint32_t q = half == 0 ? __funnelshift_r(t[i], t[i + 1], 16) : t[1 + i];
#pragma unroll
            for (int b = 0; b < 4; ++b) {
                const int byte = (q >> (8 * b)) & 0xFF;
                w[i * 4 + b] = __fmul_rn(float((byte & 0xF) - 8), d);
                w[16 + i * 4 + b] = __fmul_rn(float((byte >> 4) - 8), d);
            }
        }
    } else {
        // tensor/standard/Q8_0FloatTensor.java:53-61: a unit is two 34-byte blocks.
        const uint32_t base = row_u32 + unit * 68 + half * 32;
        uint32_t t[9];
#pragma unroll
        for (int i = 0; i < 9; ++i) t[i] = lds32(base + 4 * i);
        const float d = half_bits_to_float(half == 0 ? (t[0] & 0xFFFFu) : (t[0] >> 16));
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            const uint32_t q = half == 0 ? __funnelshift_r(t[i], t[i + 1], 16) : t[1 + i];
#pragma unroll
            for (int b = 0; b < 4; ++b) w[i * 4 + b] = __fmul_rn(float(int8_t((q >> (8 * b)) & 0xFF)), d);
        }
    }
#pragma unroll
    for (int c = 0; c < 4; ++c) {
        out[c].x = pack_half2(w[8 * c + 0], w[8 * c + 1]);
        out[c].y = pack_half2(w[8 * c + 2], w[8 * c + 3]);
        out[c].z = pack_half2(w[8 * c + 4], w[8 * c + 5]);
        out[c].w = pack_half2(w[8 * c + 6], w[8 * c + 7]);
    }
}

template <int TYPE, int NT>
struct GemmSmem {
    static constexpr int a_sub = kTileM * 128;         // one 64-column atom of A: 16 KB
    static constexpr int b_sub = NT * 128;             // one 64-column atom of B
    static constexpr int a_stage = 2 * a_sub;
    static constexpr int b_stage = 4 * b_sub;          // hi (2 atoms) + lo (2 atoms)
    static constexpr int a_off = 0;
    static constexpr int b_off = 2 * a_stage;
    static constexpr int raw_off = b_off + 2 * b_stage;
    static constexpr int bar_off = raw_off + RawFmt<TYPE>::stages * RawFmt<TYPE>::stage_bytes;
    static constexpr int total = bar_off + 128 + 1024 /*alignment slack*/;
};
static_assert(GemmSmem<kQ8_0, 64>::total <= 227 * 1024, "shared memory budget");

struct TileRef {
    int seg, row0, row_offset;  // segment, first row inside it, rows of the segments before it
};

__device__ __forceinline__ TileRef locate_tile(const GemmArgs &a, int tile) {
    TileRef t = {0, 0, 0};
    for (int s = 0; s < a.nseg; ++s) {
        const int tiles = (a.seg[s].rows + kTileM - 1) / kTileM;
        if (tile < tiles) {
            t.seg = s;
            t.row0 = tile * kTileM;
            return t;
        }
        tile -= tiles;
        t.row_offset += a.seg[s].rows;
    }
    return t;
}

template <int TYPE, int NT>
__global__ void __launch_bounds__(kGemmThreads, 1)
    gemm_tc_kernel(const GemmArgs a, const __grid_constant__ CUtensorMap tm0, const __grid_constant__ CUtensorMap tm1,
                   const __grid_constant__ CUtensorMap tm2) {
    extern __shared__ uint8_t smem_raw[];
    using S = GemmSmem<TYPE, NT>;
    using R = RawFmt<TYPE>;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    // 1024-byte aligned base: the swizzle pattern is a function of the shared address.
    uint8_t *base = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint64_t *a_free = reinterpret_cast<uint64_t *>(base + S::bar_off);  // [2]
    uint64_t *raw_full = a_free + 2;                                      // [R::stages]
    uint32_t *tmem_ptr = reinterpret_cast<uint32_t *>(base + S::bar_off + 64);
    uint32_t *last_flag = tmem_ptr + 1;
    constexpr uint32_t tmem_cols = NT < 32 ? 32 : NT;

    const TileRef tile = locate_tile(a, blockIdx.x);
    const GemmSeg seg = a.seg[tile.seg];
    const int tok0 = blockIdx.y * NT;
    const int ksplit = gridDim.z, split = blockIdx.z;
    const size_t rowb = size_t(row_bytes(TYPE, a.cols));
    const int raw_total = a.cols / kRawK;
    const int raw_begin = int(int64_t(raw_total) * split / ksplit);
    const int raw_end = int(int64_t(raw_total) * (split + 1) / ksplit);
    const int n_raw = raw_end - raw_begin;
    const int n_a = 2 * n_raw;

    if (warp == 0) tmem_alloc(tmem_ptr, tmem_cols);
    if (tid == 0) {
        mbar_init(a_free + 0, 1);
        mbar_init(a_free + 1, 1);
        for (int s = 0; s < R::stages; ++s) mbar_init(raw_full + s, 1);
        mbar_fence_init();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_d = *tmem_ptr;
    constexpr uint32_t idesc = instr_desc_f16(NT);

    // Raw producer role (one thread): a raw stage is one 2-D TMA box of 128 rows x 256 columns;
    // rows past the end of the matrix arrive as zeros.
    const CUtensorMap *tmap = tile.seg == 0 ? &tm0 : (tile.seg == 1 ? &tm1 : &tm2);
    const uint64_t policy = policy_evict_first();
    auto request_raw = [&](int i) {
        uint64_t *bar = raw_full + (i % R::stages);
        mbar_expect_tx(bar, R::stage_bytes);
        tma_load_2d(base + S::raw_off + (i % R::stages) * R::stage_bytes, tmap, (raw_begin + i) * (R::row_bytes / 4),
                    tile.row0, bar, policy);
    };
    if (tid == 0) {
        fence_proxy_async();
        for (int i = 0; i < R::stages && i < n_raw; ++i) request_raw(i);
    }

    // Operand-building role: thread t dequantises 32 columns of weight row t & 127.
    const int a_row = tid & 127, a_q = tid >> 7;  // a_q: which 32-column quarter of the 128
    const int a_atom = a_q >> 1, a_half = a_q & 1;
    const bool a_valid = tile.row0 + a_row < seg.rows;
    constexpr int kBChunks = NT * 16;  // 16-byte chunks of eight activations per operand stage
    constexpr int kBPerThread = (kBChunks + kGemmThreads - 1) / kGemmThreads;
    bool failed = false;

    for (int it = 0; it < n_a; ++it) {
        const int s = it & 1, j = it & 1, ri = it >> 1;
        const int k0 = (raw_begin + ri) * kRawK + j * kStageK;
        // Activations first: their global loads are in flight while the weights are dequantised.
        float4 xv[kBPerThread][2];
#pragma unroll
        for (int u = 0; u < kBPerThread; ++u) {
            const int ch = tid + u * kGemmThreads;
            const int t = ch >> 4, kc = ch & 15;
            const int tok = tok0 + t;
            if (ch < kBChunks && tok < a.n) {
                const float4 *src = reinterpret_cast<const float4 *>(a.x + size_t(tok) * a.cols + k0 + kc * 8);
                xv[u][0] = __ldg(src);
                xv[u][1] = __ldg(src + 1);
            } else {
                xv[u][0] = xv[u][1] = make_float4(0.f, 0.f, 0.f, 0.f);
            }
        }
        bool ok = true;
        if (j == 0) ok = mbar_wait_bounded(raw_full + (ri % R::stages), uint32_t(ri / R::stages) & 1u);
        if (ok && it >= 2) ok = mbar_wait_bounded(a_free + s, uint32_t((it - 2) >> 1) & 1u);
        if (ok) {
            tc_fence_after();
            uint8_t *a_st = base + S::a_off + s * S::a_stage;
            uint8_t *b_st = base + S::b_off + s * S::b_stage;
            if (!(a.debug & 1)) {
                uint4 chunks[4];
                const uint32_t row_u32 = smem_u32(base + S::raw_off + (ri % R::stages) * R::stage_bytes) +
                                         uint32_t(a_row) * R::row_bytes;
                dequant32_to_half<TYPE>(row_u32, 2 * j + a_atom, a_half, chunks);
                uint8_t *tile_a = a_st + size_t(a_atom) * S::a_sub;
#pragma unroll
                for (int c = 0; c < 4; ++c)
                    *reinterpret_cast<uint4 *>(tile_a + sw128_offset(a_row, a_half * 4 + c)) =
                        a_valid ? chunks[c] : make_uint4(0, 0, 0, 0);
            }
#pragma unroll
            for (int u = 0; u < kBPerThread; ++u) {
                const int ch = tid + u * kGemmThreads;
                if (ch < kBChunks && !(a.debug & 2)) {
                    const int t = ch >> 4, kc = ch & 15;
                    const int atom = kc >> 3, c = kc & 7;
                    const float x[8] = {xv[u][0].x, xv[u][0].y, xv[u][0].z, xv[u][0].w,
                                        xv[u][1].x, xv[u][1].y, xv[u][1].z, xv[u][1].w};
                    float lo[8];
#pragma unroll
                    for (int i = 0; i < 8; ++i) lo[i] = x[i] - __half2float(__float2half_rn(x[i]));
                    const uint32_t off = sw128_offset(t, c);
                    uint8_t *bh = b_st + size_t(atom) * S::b_sub;
                    uint8_t *bl = bh + 2 * S::b_sub;
                    *reinterpret_cast<uint4 *>(bh + off) = make_uint4(pack_half2(x[0], x[1]), pack_half2(x[2], x[3]),
                                                                     pack_half2(x[4], x[5]), pack_half2(x[6], x[7]));
                    *reinterpret_cast<uint4 *>(bl + off) = make_uint4(pack_half2(lo[0], lo[1]), pack_half2(lo[2], lo[3]),
                                                                     pack_half2(lo[4], lo[5]), pack_half2(lo[6], lo[7]));
                }
            }
        }
        // Generic-proxy writes -> visible to the tensor core's (async proxy) reads.
        fence_proxy_async();
        tc_fence_before();
        if (__syncthreads_or(!ok)) {
            failed = true;
            break;
        }
        if (tid == 0) {
            tc_fence_after();
            const uint32_t a_addr = smem_u32(base + S::a_off + s * S::a_stage);
            const uint32_t bh_addr = smem_u32(base + S::b_off + s * S::b_stage);
            const uint32_t bl_addr = bh_addr + 2 * S::b_sub;
#pragma unroll
            for (int atom = 0; atom < 2; ++atom) {
#pragma unroll
                for (int k16 = 0; k16 < 4; ++k16) {
                    const uint64_t da = smem_desc_sw128(a_addr + atom * S::a_sub + k16 * 32);
                    const uint64_t dbh = smem_desc_sw128(bh_addr + atom * S::b_sub + k16 * 32);
                    const uint64_t dbl = smem_desc_sw128(bl_addr + atom * S::b_sub + k16 * 32);
                    if (a.debug & 4) continue;
                    umma_f16(tmem_d, da, dbh, idesc, (it > 0 || atom > 0 || k16 > 0) ? 1u : 0u);
                    umma_f16(tmem_d, da, dbl, idesc, 1u);
                }
            }
            umma_commit(a_free + s);  // arrives when every MMA issued so far has completed
        }
        // Both halves of the raw stage have been read by every thread (they all passed the
        // barrier above): hand it back to the copy engine.
        if (j == 1 && tid == 0 && ri + R::stages < n_raw) {
            fence_proxy_async();
            request_raw(ri + R::stages);
        }
    }

    // Wait for the last commit (covers all earlier MMAs), then read the accumulator.
    if (!failed && n_a > 0) {
        if (!mbar_wait_bounded(a_free + ((n_a - 1) & 1), uint32_t((n_a - 1) >> 1) & 1u)) failed = true;
    }
    failed = __syncthreads_or(failed);
    tc_fence_after();
    // TMEM lane = output row of the tile; warp w reads lanes 32*(w%4) and the 16-column group w/4.
    const int lane_grp = warp & 3, col_grp = warp >> 2;
    const int row = tile.row0 + lane_grp * 32 + lane;
    size_t total_rows = 0;
    for (int sgi = 0; sgi < a.nseg; ++sgi) total_rows += size_t(a.seg[sgi].rows);
    const size_t grow = size_t(tile.row_offset) + row;
    if (!failed && col_grp * 16 < NT && n_a > 0) {
        float v[16];
        tmem_ld16(tmem_d + (uint32_t(lane_grp * 32) << 16) + uint32_t(col_grp * 16), v);
        if (row < seg.rows) {
#pragma unroll
            for (int jc = 0; jc < 16; ++jc) {
                const int tok = tok0 + col_grp * 16 + jc;
                if (tok < a.n) {
                    if (ksplit == 1) {
                        float out = v[jc];
                        if (seg.res != nullptr) out = seg.res[size_t(tok) * seg.rows + row] + out;
                        seg.y[size_t(tok) * seg.rows + row] = out;
                    } else {
                        a.scratch[(size_t(split) * a.n + tok) * total_rows + grow] = v[jc];
                    }
                }
            }
        }
    }
    if (ksplit > 1 && !failed) {
        // The CTA that arrives last adds the partial tiles in split order.
        __threadfence();
        __syncthreads();
        unsigned *counter = a.counters + (blockIdx.y * gridDim.x + blockIdx.x);
        if (tid == 0) {
            const unsigned prev = atomicAdd(counter, 1u);
            *last_flag = prev == unsigned(ksplit) - 1u ? 1u : 0u;
        }
        __syncthreads();
        if (*last_flag != 0u) {
            __threadfence();
            const int ntok = min(NT, a.n - tok0);
            for (int idx = tid; idx < ntok * kTileM; idx += kGemmThreads) {
                const int t = idx >> 7, r = idx & 127;
                const int orow = tile.row0 + r;
                if (orow >= seg.rows) continue;
                const int tok = tok0 + t;
                float sum = 0.f;
                for (int sp = 0; sp < ksplit; ++sp) {
                    const float pv = __ldcg(a.scratch + (size_t(sp) * a.n + tok) * total_rows + tile.row_offset + orow);
                    sum = sp == 0 ? pv : sum + pv;
                }
                if (seg.res != nullptr) sum = seg.res[size_t(tok) * seg.rows + orow] + sum;
                seg.y[size_t(tok) * seg.rows + orow] = sum;
            }
            if (tid == 0) *counter = 0u;
        }
    }
    if (failed && tid == 0) atomicExch(a.status, kDevTimeout);
    tc_fence_before();
    __syncthreads();
    if (warp == 0) tmem_dealloc(tmem_d, tmem_cols);
}

// Column splits: enough CTAs to fill the GPU's last wave, at least two raw stages per CTA, and
// no more than the workspace holds.
int choose_split(const GemmArgs &a, int tiles, int n_tiles, int nt) {
    if (a.scratch == nullptr || a.counters == nullptr || tiles * n_tiles > a.counters_len) return 1;
    const int sms = a.sm_count > 0 ? a.sm_count : 148;
    const int raw_total = a.cols / kRawK;
    size_t total_rows = 0;
    for (int s = 0; s < a.nseg; ++s) total_rows += size_t(a.seg[s].rows);
    const int work = tiles * n_tiles;
    if (work >= 4 * sms) return 1;
    int best = 1;
    double best_eff = 0.0;
    for (int ks = 1; ks <= kMaxSplit; ++ks) {
        if (raw_total / ks < 2) break;
        if (size_t(ks) * a.n * total_rows > a.scratch_floats && ks > 1) break;
        const double waves = double(work) * ks / sms;
        const double eff = waves / double((long long)(waves + 0.999999));
        // a later (larger) split must be clearly better to be worth its workspace traffic
        if (eff > best_eff * 1.08) {
            best_eff = eff;
            best = ks;
        }
    }
    (void)nt;
    return best;
}

template <int TYPE, int NT>
cudaError_t launch_nt(const GemmArgs &a, cudaStream_t stream) {
    int tiles = 0;
    for (int s = 0; s < a.nseg; ++s) tiles += (a.seg[s].rows + kTileM - 1) / kTileM;
    const int n_tiles = (a.n + NT - 1) / NT;
    const int ks = choose_split(a, tiles, n_tiles, NT);
    dim3 grid(tiles, n_tiles, ks);
    CUtensorMap maps[3];
    for (int s = 0; s < 3; ++s) {
        const GemmTensorMap *m = a.seg[s < a.nseg ? s : 0].tmap;
        memcpy(&maps[s], m->bytes, sizeof(CUtensorMap));
    }
    gemm_tc_kernel<TYPE, NT><<<grid, kGemmThreads, GemmSmem<TYPE, NT>::total, stream>>>(a, maps[0], maps[1], maps[2]);
    return cudaGetLastError();
}

template <int TYPE>
cudaError_t launch_type(const GemmArgs &a, cudaStream_t stream) {
    if (a.n <= 16) return launch_nt<TYPE, 16>(a, stream);
    if (a.n <= 32) return launch_nt<TYPE, 32>(a, stream);
    return launch_nt<TYPE, 64>(a, stream);
}

template <int TYPE, int NT>
cudaError_t configure_nt() {
    return cudaFuncSetAttribute(gemm_tc_kernel<TYPE, NT>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                GemmSmem<TYPE, NT>::total);
}

template <int TYPE>
cudaError_t configure_type() {
    cudaError_t e;
    if ((e = configure_nt<TYPE, 16>()) != cudaSuccess) return e;
    if ((e = configure_nt<TYPE, 32>()) != cudaSuccess) return e;
    return configure_nt<TYPE, 64>();
}

}  // namespace

cudaError_t gemm_make_tensor_map(GemmTensorMap *out, const void *w_dev, int type, int64_t rows, int64_t cols) {
    static_assert(sizeof(CUtensorMap) == sizeof(GemmTensorMap), "descriptor size");
    if (!out || !w_dev || !is_quant(type) || rows <= 0 || cols <= 0 || cols % kRawK != 0) return cudaErrorInvalidValue;
    typedef CUresult (*EncodeFn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *,
                                 const cuuint64_t *, const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave,
                                 CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
    static EncodeFn encode = nullptr;
    if (encode == nullptr) {
        void *fn = nullptr;
        cudaDriverEntryPointQueryResult q;
        cudaError_t e = cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &q);
        if (e != cudaSuccess) return e;
        if (q != cudaDriverEntryPointSuccess || fn == nullptr) return cudaErrorNotSupported;
        encode = reinterpret_cast<EncodeFn>(fn);
    }
    const uint64_t rowb = uint64_t(row_bytes(type, cols));
    const uint32_t raw_bytes = type == kQ8_0 ? 272u : 144u;
    const cuuint64_t gdim[2] = {rowb / 4, cuuint64_t(rows)};
    const cuuint64_t gstride[1] = {rowb};
    const cuuint32_t box[2] = {raw_bytes / 4, cuuint32_t(kTileM)};
    const cuuint32_t estride[2] = {1, 1};
    CUtensorMap map;
    const CUresult r = encode(&map, CU_TENSOR_MAP_DATA_TYPE_UINT32, 2, const_cast<void *>(w_dev), gdim, gstride, box,
                              estride, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE,
                              CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return cudaErrorInvalidValue;
    memcpy(out->bytes, &map, sizeof map);
    return cudaSuccess;
}

cudaError_t gemm_tc_configure() {
    cudaError_t e;
    if ((e = configure_type<kQ4_K>()) != cudaSuccess) return e;
    if ((e = configure_type<kQ4_0>()) != cudaSuccess) return e;
    return configure_type<kQ8_0>();
}

cudaError_t gemm_tc_launch(const GemmArgs &a, cudaStream_t stream) {
    if (a.cols <= 0 || a.cols % 256 != 0 || a.n <= 0 || a.nseg < 1 || a.nseg > 3) return cudaErrorInvalidValue;
    for (int s = 0; s < a.nseg; ++s)
        if (a.seg[s].rows <= 0 || a.seg[s].w == nullptr || a.seg[s].y == nullptr || a.seg[s].tmap == nullptr)
            return cudaErrorInvalidValue;
    switch (a.type) {
        case kQ4_K: return launch_type<kQ4_K>(a, stream);
        case kQ4_0: return launch_type<kQ4_0>(a, stream);
        case kQ8_0: return launch_type<kQ8_0>(a, stream);
        default: return cudaErrorInvalidValue;
    }
}

}  // namespace jl
