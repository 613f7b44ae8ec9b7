// Quantised matrix-matrix product on the 5th-generation tensor cores (tcgen05) for batched decode
// and chunked prefill: Y[n][rows] = X[n][cols] . W[rows][cols]^T, W in GGUF block layout.
// What it computes: FloatTensor.matmul(context, that[], out[], dim0, dim1)
// (tensor/standard/FloatTensor.java:127-140 of the reference), n independent mat-vecs.
//
// Shape of the kernel. One persistent CTA per SM. The work is the list of (128-row tile, NT-token
// tile, 256-column raw stage) triples in that order, cut into equal contiguous ranges, one per
// CTA, so every SM gets the same number of weight bytes whatever the matrix shape (with fewer tiles
// than SMs the ranges are aligned to tiles). Inside a CTA four roles run concurrently and meet only
// at mbarriers:
//   * warp 17, one thread: requests each raw stage (128 rows x 256 columns of quantised bytes, as
//     stored) as one 2-D TMA box into a ring; rows past the end of the matrix arrive as zeros.
//   * warp 18, one thread: requests the B operand of every stage, NT rows of the activations' hi part
//     and NT rows of their lo part (x = hi + lo, both fp16: 22 significant bits; written by the
//     kernels that produce the activations) as swizzled TMA boxes, stacked along N so that one MMA
//     covers both. Entry points without such a buffer convert fp32 activations in warps 0-15.
//   * warps 0-15: turn raw half-stages (128 columns) into the A operand -- weights rounded once to
//     fp16 (Q4_0 / Q8_0: integer code times the block's fp16 scale in half2 arithmetic, which is
//     exactly the fp16 rounding of the reference's fp32 product; Q4_K: (d*sc)*q - dmin*m in fp32
//     with the last two steps fused, then rounded) -- and store it into tensor memory with
//     tcgen05.st (lane = weight row, 64 columns per stage). Two groups of eight warps take alternate
//     stages, one 64-column unit per thread. The only rounding left is the fp16 rounding of the
//     weights (rel-L2 ~3e-4 per product, inside the 1e-3 bar; the reference's own tensor-core
//     prefill feeds single fp16 operands).
//   * warp 16, one thread: issues tcgen05.mma (M=128, N=2*NT, K=16; A from tensor memory, B from
//     shared memory) into the tensor-memory accumulator and commits to the barriers that free the
//     operand stage / publish the finished accumulator.
//   Warps 0-15 also run the epilogue (tcgen05.ld). A CTA whose range covers a whole output tile
//   writes it; where a range ends inside a tile the partial goes to a per-CTA slot and the CTA
//   that arrives last at the tile's counter adds the partials in CTA order (the result does not
//   depend on which CTA finished first), adds the residual and writes Y.
// Every wait is bounded; a wait that runs out sets the status word and the CTA winds down.
#include "gemm_tc.cuh"

#include "formats.cuh"

#include <cuda.h>
#include <cuda_fp16.h>

#include <cstring>

namespace jl {

JL_TRACE_DEFINE_BIND(gemm_trace_bind)

namespace {

// Which bounded wait the kernel uses (a build-time experiment switch).
#define GEMM_WAIT mbar_poll_bounded

constexpr int kConvertWarps = 16;
constexpr int kConvertThreads = kConvertWarps * 32;
constexpr int kGemmThreads = kConvertThreads + 96;  // + tensor-core issue warp + two copy-request warps
constexpr int kTileM = 128;    // weight rows per tile
constexpr int kStageK = 128;   // columns per operand stage (two 64-column swizzle atoms)
constexpr int kRawK = 256;     // columns per raw stage (one Q4_K super-block per row)

__device__ __forceinline__ void mbar_arrive(uint64_t *bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
// Barrier among the conversion warps only, on an mbarrier so that the wait is bounded like every
// other wait here: lane 0 of each warp arrives, everybody waits for the phase to flip.
__device__ __forceinline__ bool convert_warps_sync(uint64_t *bar, int &phase) {
    __syncwarp();
    if ((threadIdx.x & 31) == 0) mbar_arrive(bar);
    const bool ok = GEMM_WAIT(bar, uint32_t(phase) & 1u);
    ++phase;
    return ok;
}

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

__device__ __forceinline__ void tma_load_2d_plain(void *dst_smem, const CUtensorMap *map, int x, int y, uint64_t *bar) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
        ::"r"(smem_u32(dst_smem)), "l"(map), "r"(x), "r"(y), "r"(smem_u32(bar))
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
// D[tmem] (+)= A * B; fp16 operands, fp32 accumulate, A in tensor memory: lane = row, one 32-bit column =
// two consecutive K elements (even K in the low half), eight columns per K = 16 step; B in shared memory.
// The eight MMAs of one operand stage (K = 128: two 64-column atoms of four K = 16 steps) and the commit
// that hands the stage back, issued by one elected lane while the whole warp stays converged: every
// operand is warp-uniform, so the addresses and descriptors can stay in the uniform datapath instead of
// being moved there one by one in front of each MMA. The shared-memory descriptor is given as its two
// 32-bit words; KBm is the descriptor's address step of MMA m, in 16-byte units.
template <int KB1, int KB2, int KB3, int KB4, int KB5, int KB6, int KB7>
__device__ __forceinline__ void umma_stage_f16_tmem_a(uint32_t d_tmem, uint32_t a_tmem, uint32_t b_desc_lo, uint32_t b_desc_hi,
                                                      uint32_t idesc, uint32_t free_bar, uint32_t accumulate_first) {
    asm volatile(
        "{\n\t"
        ".reg .pred pe, pacc, pone;\n\t"
        ".reg .b64 bd;\n\t"
        ".reg .b32 lo, ac;\n\t"
        "elect.sync _|pe, 0xffffffff;\n\t"
        "setp.ne.b32 pacc, %6, 0;\n\t"
        "setp.eq.b32 pone, 0, 0;\n\t"
        "mov.b64 bd, {%2, %3};\n\t"
        "@pe tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], bd, %4, pacc;\n\t"
        "add.u32 lo, %2, %7;\n\t add.u32 ac, %1, 8;\n\t mov.b64 bd, {lo, %3};\n\t"
        "@pe tcgen05.mma.cta_group::1.kind::f16 [%0], [ac], bd, %4, pone;\n\t"
        "add.u32 lo, %2, %8;\n\t add.u32 ac, %1, 16;\n\t mov.b64 bd, {lo, %3};\n\t"
        "@pe tcgen05.mma.cta_group::1.kind::f16 [%0], [ac], bd, %4, pone;\n\t"
        "add.u32 lo, %2, %9;\n\t add.u32 ac, %1, 24;\n\t mov.b64 bd, {lo, %3};\n\t"
        "@pe tcgen05.mma.cta_group::1.kind::f16 [%0], [ac], bd, %4, pone;\n\t"
        "add.u32 lo, %2, %10;\n\t add.u32 ac, %1, 32;\n\t mov.b64 bd, {lo, %3};\n\t"
        "@pe tcgen05.mma.cta_group::1.kind::f16 [%0], [ac], bd, %4, pone;\n\t"
        "add.u32 lo, %2, %11;\n\t add.u32 ac, %1, 40;\n\t mov.b64 bd, {lo, %3};\n\t"
        "@pe tcgen05.mma.cta_group::1.kind::f16 [%0], [ac], bd, %4, pone;\n\t"
        "add.u32 lo, %2, %12;\n\t add.u32 ac, %1, 48;\n\t mov.b64 bd, {lo, %3};\n\t"
        "@pe tcgen05.mma.cta_group::1.kind::f16 [%0], [ac], bd, %4, pone;\n\t"
        "add.u32 lo, %2, %13;\n\t add.u32 ac, %1, 56;\n\t mov.b64 bd, {lo, %3};\n\t"
        "@pe tcgen05.mma.cta_group::1.kind::f16 [%0], [ac], bd, %4, pone;\n\t"
        "@pe tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%5];\n\t"
        "}"
        ::"r"(d_tmem), "r"(a_tmem), "r"(b_desc_lo), "r"(b_desc_hi), "r"(idesc), "r"(free_bar), "r"(accumulate_first),
          "n"(KB1), "n"(KB2), "n"(KB3), "n"(KB4), "n"(KB5), "n"(KB6), "n"(KB7)
        : "memory");
}
// A commit by one elected lane of a converged warp.
__device__ __forceinline__ void umma_commit_elect(uint32_t bar) {
    asm volatile(
        "{\n\t.reg .pred pe;\n\t"
        "elect.sync _|pe, 0xffffffff;\n\t"
        "@pe tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];\n\t}"
        ::"r"(bar) : "memory");
}
__device__ __forceinline__ void mbar_arrive_u32(uint32_t bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
// mbar_poll_bounded on a shared-window address.
__device__ __forceinline__ bool mbar_poll_bounded_u32(uint32_t bar, uint32_t parity, uint32_t limit = (1u << 24)) {
    for (uint32_t i = 0; i < limit; ++i) {
        uint32_t ok;
        asm volatile(
            "{\n\t.reg .pred p;\n\t"
            "mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
            "selp.u32 %0, 1, 0, p;\n\t}"
            : "=r"(ok)
            : "r"(bar), "r"(parity)
            : "memory");
        if (ok != 0) return true;
        __nanosleep(40);
    }
    return false;
}
// 16 consecutive 32-bit columns of this thread's lane.
__device__ __forceinline__ void tmem_st16(uint32_t taddr, const uint32_t (&r)[16]) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16};"
        ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]),
        "r"(r[9]), "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15])
        : "memory");
}
__device__ __forceinline__ void tmem_wait_st() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }
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

// Shared-memory matrix descriptor of the B operand: K-major, 128-byte swizzle, rows of 64 fp16
// (128 B), groups of eight rows 1024 B apart. Low word: bits 0-13 the start address in 16-byte
// units, bit 16 the (unused) leading byte offset; high word: bits 0-13 the stride between 8-row
// groups in 16-byte units (1024 >> 4), bit 14 the descriptor version for sm_100, bits 29-31 the
// swizzle mode (2 = 128 bytes). The issuing thread keeps the low word as a running value.
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
    static constexpr int row_bytes = TYPE == kQ8_0   ? 272  // 256 columns of one row
                                     : TYPE == kQ6_K ? kQ6_KPadded
                                     : TYPE == kQ5_K ? kQ5_KBytes
                                     : TYPE == kQ4_1 ? 8 * kQ4_1Bytes
                                                     : 144;
    static constexpr int stage_bytes = kTileM * row_bytes;
};

// Two bytes of v (selected by sel) as half2 {1024 + byte, 1024 + byte}: 0x64xx is 1024 + xx in fp16.
__device__ __forceinline__ __half2 bytes_to_half2_plus1024(uint32_t v, uint32_t sel) {
    uint32_t r;
    asm("prmt.b32 %0, %1, %2, %3;" : "=r"(r) : "r"(v), "r"(0x64646464u), "r"(sel));
    return *reinterpret_cast<const __half2 *>(&r);
}
__device__ __forceinline__ uint32_t h2_bits(__half2 h) { return *reinterpret_cast<const uint32_t *>(&h); }

// Operand order. Inside every group of four consecutive K elements the tensor-memory columns (and the
// activation rows, see the in-kernel activation conversion below and split4_store in ops.cu) hold
// the pairs (k0, k2) and (k1, k3): a sum over K does not care about the order as long as both
// operands agree, and the bytes 0 and 2 of a 32-bit word come out together with one logic operation.

// What a thread keeps of its 64-weight unit between the two 32-weight halves it converts.
template <int TYPE>
struct UnitRegs;

template <>
struct UnitRegs<kQ4_K> {
    uint32_t qw[8];         // the unit's 32 bytes: low nibbles = first half, high nibbles = second
    __half2 d2;             // the super-block scale, exact (it is stored as binary16)
    __half2 sc2[2], off2[2];  // per half: the 6-bit scale as a number, and -base * scale
    __half2 chi2[2], clo2[2];  // per half: -dmin * m as an exact binary16 pair (17 significant bits)
};
template <>
struct UnitRegs<kQ4_0> {
    uint32_t t[9];  // two 18-byte blocks
};
template <>
struct UnitRegs<kQ8_0> {
    uint32_t base;  // shared address of the unit (two 34-byte blocks); its halves are loaded one at a time
};
template <>
struct UnitRegs<kQ5_K> {
    uint32_t qw[8];            // as Q4_K
    __half2 d2;
    __half2 sc2[2], off2[2];
    __half2 chi2[2], clo2[2];
    uint32_t qh_at;            // shared address of the super-block's 32 bytes of fifth bits (read again per half)
    int shift;                 // bit of those bytes that belongs to the unit's low nibbles (the high nibbles' is the next)
};
template <>
struct UnitRegs<kQ4_1> {
    uint32_t t[10];  // two 20-byte blocks: (d, m), 16 bytes of nibbles, twice
};
template <>
struct UnitRegs<kQ6_K> {
    uint32_t blk;   // shared address of the (padded) super-block; the unit's halves are loaded one at a time
    int unit;
    __half2 d2;     // the super-block scale, exact (it is stored as binary16)
};

__device__ __forceinline__ __half2 u32_as_half2(uint32_t v) { return *reinterpret_cast<const __half2 *>(&v); }

// Loads a unit: `row_u32` is the shared address of the row's 256-column slice of a raw stage, `unit`
// the 64-column unit inside it (0..3).
template <int TYPE>
__device__ __forceinline__ void unit_load(uint32_t row_u32, int unit, UnitRegs<TYPE> &r) {
    if constexpr (TYPE == kQ4_K || TYPE == kQ5_K) {
        // tensor/standard/Q4_KFloatTensor.java:68-122: unit p holds sub-blocks 2p (low nibbles) and
        // 2p+1 (high nibbles) of the same 32 bytes; w = (d*sc)*q - dmin*m. Q5_K (Q5_KFloatTensor.java:87-127) is
        // the same with 32 bytes of fifth bits between the header and the nibbles.
        constexpr int kNibbles = TYPE == kQ5_K ? 48 : 16;
        const uint4 hdr = lds128(row_u32);
        const uint4 q0 = lds128(row_u32 + kNibbles + unit * 32);
        const uint4 q1 = lds128(row_u32 + kNibbles + 16 + unit * 32);
        if constexpr (TYPE == kQ5_K) {
            r.qh_at = row_u32 + 16;
            r.shift = 2 * unit;
        }
        r.qw[0] = q0.x; r.qw[1] = q0.y; r.qw[2] = q0.z; r.qw[3] = q0.w;
        r.qw[4] = q1.x; r.qw[5] = q1.y; r.qw[6] = q1.z; r.qw[7] = q1.w;
        r.d2 = u32_as_half2(__byte_perm(hdr.x, 0u, 0x1010));
        const float dmin = half_bits_to_float(hdr.x >> 16);
        uint32_t scw, mw;
        if (unit < 2) {
            scw = hdr.y & 0x3F3F3F3Fu;
            mw = hdr.z & 0x3F3F3F3Fu;
        } else {
            scw = (hdr.w & 0x0F0F0F0Fu) | ((hdr.y >> 2) & 0x30303030u);
            mw = ((hdr.w >> 4) & 0x0F0F0F0Fu) | ((hdr.z >> 2) & 0x30303030u);
        }
        const int sh = (unit & 1) * 16;
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            // 0x6400 | n is 1024 + n in binary16: the 6-bit scale and minimum become numbers without
            // the conversion unit.
            const uint32_t scb = (scw >> (sh + 8 * h)) & 0xFFu, mb = (mw >> (sh + 8 * h)) & 0xFFu;
            const __half2 k1024 = u32_as_half2(0x64006400u);
            r.sc2[h] = __hsub2(u32_as_half2(0x64006400u | scb | (scb << 16)), k1024);
            r.off2[h] = __hmul2(r.sc2[h], u32_as_half2(h == 0 ? 0xE400E400u : 0xD400D400u));  // * -1024, * -64: exact
            const float c = -__fmul_rn(dmin, __half2float(__low2half(__hsub2(u32_as_half2(0x64006400u | mb), k1024))));
            const __half chi = __float2half_rn(c);
            const __half clo = __float2half_rn(c - __half2float(chi));  // exact: c has 17 significant bits
            r.chi2[h] = __half2half2(chi);
            r.clo2[h] = __half2half2(clo);
        }
    } else if constexpr (TYPE == kQ4_0) {
        const uint32_t base = row_u32 + unit * 36;
#pragma unroll
        for (int i = 0; i < 9; ++i) r.t[i] = lds32(base + 4 * i);
    } else if constexpr (TYPE == kQ4_1) {
        const uint32_t base = row_u32 + unit * 40;
#pragma unroll
        for (int i = 0; i < 10; ++i) r.t[i] = lds32(base + 4 * i);
    } else if constexpr (TYPE == kQ6_K) {
        r.blk = row_u32;
        r.unit = unit;
        const uint32_t dw = lds32(row_u32 + 208) & 0xFFFFu;
        r.d2 = u32_as_half2(dw | (dw << 16));
    } else {
        r.base = row_u32 + unit * 68;
    }
}

// 32 of the unit's 64 consecutive weights as 16 tensor-memory columns, each weight rounded to binary16:
// `half` 0 = the first 32 weights, 1 = the next 32. The two halves are converted and stored one after
// the other so that only 16 results are live.
template <int TYPE>
__device__ __forceinline__ void unit_convert(const UnitRegs<TYPE> &r, int half, uint32_t (&out)[16]) {
    if constexpr (TYPE == kQ4_K) {
        // The conversion runs on the floating-point pipe, two weights per instruction: one logic
        // operation drops two nibbles into the mantissas of a binary16 pair (0x6400 | q = 1024 + q for
        // the low nibbles, 0x5400 | (q << 4) = 64 + q for the high ones, both exact), one fused
        // multiply-add makes t = sc * q out of it (an integer below 1024: exact), a second one
        // d * t + c_hi rounds once, and the last addition brings in c_lo, the 6 bits of dmin * m that
        // c_hi cannot hold. The result is within two binary16 roundings of d * sc * q - dmin * m.
        const uint32_t mask = half == 0 ? 0x000F000Fu : 0x00F000F0u, magic = half == 0 ? 0x64006400u : 0x54005400u;
        const __half2 sc2 = r.sc2[half], off2 = r.off2[half], chi2 = r.chi2[half], clo2 = r.clo2[half];
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            const __half2 e = u32_as_half2((r.qw[i] & mask) | magic);         // bytes 0 and 2 of the word
            const __half2 o = u32_as_half2(((r.qw[i] >> 8) & mask) | magic);  // bytes 1 and 3
            const __half2 we = __hadd2(__hfma2(r.d2, __hfma2(sc2, e, off2), chi2), clo2);
            const __half2 wo = __hadd2(__hfma2(r.d2, __hfma2(sc2, o, off2), chi2), clo2);
            out[2 * i] = h2_bits(we);
            out[2 * i + 1] = h2_bits(wo);
        }
    } else if constexpr (TYPE == kQ5_K) {
        // As Q4_K, with the fifth bit dropped into the same mantissa: 1024 + q (low nibbles: bit 4) or 64 + q (high
        // nibbles, whose mantissa unit is 1/16: bit 8). sc * q stays below 2048, exact in binary16.
        const uint32_t mask = half == 0 ? 0x000F000Fu : 0x00F000F0u, magic = half == 0 ? 0x64006400u : 0x54005400u;
        const __half2 sc2 = r.sc2[half], off2 = r.off2[half], chi2 = r.chi2[half], clo2 = r.clo2[half];
        const uint4 f0 = lds128(r.qh_at), f1 = lds128(r.qh_at + 16);
        const uint32_t fw[8] = {f0.x, f0.y, f0.z, f0.w, f1.x, f1.y, f1.z, f1.w};
        const int fs = r.shift + half;
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            const uint32_t f = fw[i] >> fs;  // bit 0 of every byte: the fifth bit of that weight
            const uint32_t fe = half == 0 ? ((f << 4) & 0x00100010u) : ((f << 8) & 0x01000100u);  // bytes 0 and 2
            const uint32_t fo = half == 0 ? ((f >> 4) & 0x00100010u) : (f & 0x01000100u);          // bytes 1 and 3
            const __half2 e = u32_as_half2((r.qw[i] & mask) | fe | magic);
            const __half2 o = u32_as_half2(((r.qw[i] >> 8) & mask) | fo | magic);
            const __half2 we = __hadd2(__hfma2(r.d2, __hfma2(sc2, e, off2), chi2), clo2);
            const __half2 wo = __hadd2(__hfma2(r.d2, __hfma2(sc2, o, off2), chi2), clo2);
            out[2 * i] = h2_bits(we);
            out[2 * i + 1] = h2_bits(wo);
        }
    } else if constexpr (TYPE == kQ4_1) {
        // tensor/standard/Q4_1FloatTensor.java:76-99: a unit is two 20-byte blocks; w = q * d + m with an unsigned
        // nibble, one fused multiply-add on exact inputs.
        const uint32_t hdr = r.t[5 * half];
        const __half2 d2 = u32_as_half2(__byte_perm(hdr, 0u, 0x1010)), m2 = u32_as_half2(__byte_perm(hdr, 0u, 0x3232));
        const __half2 off = __float2half2_rn(1024.0f);
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const uint32_t q = r.t[5 * half + 1 + i];
            const uint32_t l4 = q & 0x0F0F0F0Fu, h4 = (q >> 4) & 0x0F0F0F0Fu;
            out[2 * i] = h2_bits(__hfma2(__hsub2(bytes_to_half2_plus1024(l4, 0x4240u), off), d2, m2));
            out[2 * i + 1] = h2_bits(__hfma2(__hsub2(bytes_to_half2_plus1024(l4, 0x4341u), off), d2, m2));
            out[8 + 2 * i] = h2_bits(__hfma2(__hsub2(bytes_to_half2_plus1024(h4, 0x4240u), off), d2, m2));
            out[8 + 2 * i + 1] = h2_bits(__hfma2(__hsub2(bytes_to_half2_plus1024(h4, 0x4341u), off), d2, m2));
        }
    } else if constexpr (TYPE == kQ6_K) {
        // tensor/standard/Q6_KFloatTensor.java:64-117. Unit p = 2h + u of the super-block: half h, the groups 2u
        // (this call's half 0) and 2u + 1 (half 1) of 32 weights: nibble u of ql[64 h + 32 half + j], bits
        // 4u + 2 half .. +1 of qh[32 h + j], one signed byte scale per 16 weights; w = d * scale * (v - 32).
        // v - 32 is exact in binary16; d * scale has up to 18 significant bits and is applied as an exact
        // binary16 pair (hi, lo): w = (v - 32) * hi + (v - 32) * lo, one rounding apart from the small lo product.
        const int h = r.unit >> 1, u = r.unit & 1;
        const uint32_t ql_at = r.blk + 64 * h + 32 * half, qh_at = r.blk + 128 + 32 * h;
        const uint32_t scw = lds32(r.blk + 192 + 8 * h + 4 * u) >> (16 * half);  // bytes 0, 1: this half's two scales
        const float d = __half2float(__low2half(r.d2));
        __half2 hi2[2], lo2[2];
#pragma unroll
        for (int k = 0; k < 2; ++k) {
            const float ds = __fmul_rn(d, static_cast<float>(static_cast<int>(static_cast<int8_t>((scw >> (8 * k)) & 0xFFu))));
            const __half hi = __float2half_rn(ds);
            hi2[k] = __half2half2(hi);
            lo2[k] = __half2half2(__float2half_rn(ds - __half2float(hi)));
        }
        const __half2 off = __float2half2_rn(1056.0f);  // 1024 of the byte trick + 32
        const int qsh = 4 * u + 2 * half;
#pragma unroll
        for (int q = 0; q < 2; ++q) {  // four words at a time: one 16-byte load of each plane, one scale
            const uint4 l4 = lds128(ql_at + 16 * q), h4 = lds128(qh_at + 16 * q);
            const uint32_t lw[4] = {l4.x, l4.y, l4.z, l4.w}, hw[4] = {h4.x, h4.y, h4.z, h4.w};
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const uint32_t v = ((lw[i] >> (4 * u)) & 0x0F0F0F0Fu) | (((hw[i] >> qsh) << 4) & 0x30303030u);
                const __half2 e = __hsub2(bytes_to_half2_plus1024(v, 0x4240u), off);
                const __half2 o = __hsub2(bytes_to_half2_plus1024(v, 0x4341u), off);
                out[8 * q + 2 * i] = h2_bits(__hfma2(e, hi2[q], __hmul2(e, lo2[q])));
                out[8 * q + 2 * i + 1] = h2_bits(__hfma2(o, hi2[q], __hmul2(o, lo2[q])));
            }
        }
    } else if constexpr (TYPE == kQ4_0) {
        // tensor/standard/Q4_0FloatTensor.java:56-79: a unit is two 18-byte blocks; element i < 16
        // is the low nibble of byte i, element i >= 16 the high nibble of byte i - 16; w = (q-8)*d.
        // (q-8) is exact in fp16 and d is fp16, so one half-precision multiply rounds exactly like
        // the reference's fp32 product narrowed to fp16.
        const uint32_t dbits = half == 0 ? (r.t[0] & 0xFFFFu) : (r.t[4] >> 16);
        const __half2 d2 = u32_as_half2(dbits | (dbits << 16));
        const __half2 off = __float2half2_rn(1032.0f);
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const uint32_t q = half == 0 ? __funnelshift_r(r.t[i], r.t[i + 1], 16) : r.t[5 + i];
            const uint32_t l4 = q & 0x0F0F0F0Fu, h4 = (q >> 4) & 0x0F0F0F0Fu;
            out[2 * i] = h2_bits(__hmul2(__hsub2(bytes_to_half2_plus1024(l4, 0x4240u), off), d2));
            out[2 * i + 1] = h2_bits(__hmul2(__hsub2(bytes_to_half2_plus1024(l4, 0x4341u), off), d2));
            out[8 + 2 * i] = h2_bits(__hmul2(__hsub2(bytes_to_half2_plus1024(h4, 0x4240u), off), d2));
            out[8 + 2 * i + 1] = h2_bits(__hmul2(__hsub2(bytes_to_half2_plus1024(h4, 0x4341u), off), d2));
        }
    } else {
        // tensor/standard/Q8_0FloatTensor.java:53-61: a unit is two 34-byte blocks; w = q * d, again
        // one exact-input half-precision multiply.
        const uint32_t base = r.base + half * 32;
        uint32_t t[9];
#pragma unroll
        for (int i = 0; i < 9; ++i) t[i] = lds32(base + 4 * i);
        const uint32_t dbits = half == 0 ? (t[0] & 0xFFFFu) : (t[0] >> 16);
        const __half2 d2 = u32_as_half2(dbits | (dbits << 16));
        const __half2 off = __float2half2_rn(1152.0f);  // 1024 + the 128 added by the sign flip
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            const uint32_t q = (half == 0 ? __funnelshift_r(t[i], t[i + 1], 16) : t[1 + i]) ^ 0x80808080u;
            out[2 * i] = h2_bits(__hmul2(__hsub2(bytes_to_half2_plus1024(q, 0x4240u), off), d2));
            out[2 * i + 1] = h2_bits(__hmul2(__hsub2(bytes_to_half2_plus1024(q, 0x4341u), off), d2));
        }
    }
}

// Tensor-memory columns: the accumulator (hi and lo partial products side by side, 2*NT columns)
// and behind it the A operand stages of 64 columns (128 K elements) each.
constexpr uint32_t kTmemCols = 512;
constexpr uint32_t kTmemAStageCols = kStageK / 2;
template <int NT>
struct TmemPlan {
    static constexpr uint32_t a_stage0 = NT <= 64 ? 128 : 256;
    static constexpr int a_stages = int((kTmemCols - a_stage0) / kTmemAStageCols);  // 6, or 4 for NT = 128
};

template <int TYPE, int NT>
struct GemmSmem {
    static constexpr int b_sub = 2 * NT * 128;         // one 64-column atom of B: hi rows, then lo rows
    static constexpr int b_stage = 2 * b_sub;
    static constexpr int bar_bytes = 384;               // barriers, the tensor-memory address and two flags
#ifdef JL_TRACE_EVENTS
    static constexpr int log_bytes = 4096;              // event-log build: a log of 512 words, copied out at the end
#else
    static constexpr int log_bytes = 0;
#endif
    static constexpr int budget = 227 * 1024 - 1024 /*alignment slack*/ - bar_bytes - log_bytes;
    // Operand stages: the A half lives in tensor memory (six stages fit beside the accumulator), the
    // B half in shared memory. Several stages must be in flight to hide the round trip
    // conversion -> MMA -> commit -> stage free again. They come first; two raw stages are the
    // least the raw ring works with.
    static constexpr int fit = (budget - 2 * RawFmt<TYPE>::stage_bytes) / b_stage;
    static constexpr int stages = fit >= TmemPlan<NT>::a_stages ? TmemPlan<NT>::a_stages : fit;
    // Raw stages take what is left, up to three: a raw stage is requested when its slot is handed
    // back and needed that many iterations later. Deeper rings measured slower: every CTA requests
    // its whole ring at kernel start, and the first stage then lands behind that burst.
    static constexpr int raw_fit = (budget - stages * b_stage) / RawFmt<TYPE>::stage_bytes;
    static constexpr int raw_stages = raw_fit > 3 ? 3 : raw_fit;
    static constexpr int raw_bytes = raw_stages * RawFmt<TYPE>::stage_bytes;
    static constexpr int b_off = 0;
    static constexpr int raw_off = stages * b_stage;
    static constexpr int bar_off = raw_off + raw_bytes;
    static constexpr int log_off = bar_off + bar_bytes;
    static constexpr int total = log_off + log_bytes + 1024;
};
static_assert((2 * 6 + 2 * 8 + 3) * 8 + 64 <= GemmSmem<kQ4_K, 32>::bar_bytes, "barrier block");
static_assert(GemmSmem<kQ8_0, 64>::total <= 227 * 1024 && GemmSmem<kQ4_K, 64>::total <= 227 * 1024 &&
                  GemmSmem<kQ4_K, 16>::total <= 227 * 1024 && GemmSmem<kQ8_0, 32>::total <= 227 * 1024,
              "shared memory budget");
static_assert(GemmSmem<kQ6_K, 16>::total <= 227 * 1024 && GemmSmem<kQ6_K, 32>::total <= 227 * 1024 &&
                  GemmSmem<kQ6_K, 64>::total <= 227 * 1024 && GemmSmem<kQ6_K, 128>::total <= 227 * 1024 &&
                  GemmSmem<kQ6_K, 64>::stages >= 3 && GemmSmem<kQ6_K, 128>::stages >= 2 && GemmSmem<kQ6_K, 128>::raw_stages >= 2,
              "Q6_K (padded super-blocks) budget");
static_assert(GemmSmem<kQ8_0, 64>::stages >= 3 && GemmSmem<kQ8_0, 128>::stages >= 2 &&
                  GemmSmem<kQ8_0, 128>::total <= 227 * 1024 && GemmSmem<kQ4_K, 128>::total <= 227 * 1024,
              "pipeline depth");

struct TileRef {
    int seg, row0;
};

__device__ __forceinline__ TileRef locate_tile(const GemmArgs &a, int tile) {
    TileRef t = {0, 0};
    for (int s = 0; s < a.nseg; ++s) {
        const int tiles = (a.seg[s].rows + kTileM - 1) / kTileM;
        if (tile < tiles || s == a.nseg - 1) {
            t.seg = s;
            t.row0 = tile * kTileM;
            return t;
        }
        tile -= tiles;
    }
    return t;
}

// The contiguous range of the flattened work list that CTA c owns.
// (The launcher refuses work lists with total * ctas >= 2^32, so the arithmetic stays in 32 bits: a
// 64-bit division costs about a hundred instructions, and these run at every tile end.)
__device__ __forceinline__ int range_lo(int total, int c, int ctas) {
    return int(uint32_t(total) * uint32_t(c) / uint32_t(ctas));
}
__device__ __forceinline__ int cta_of(int total, int f, int ctas) {
    int c = int(uint32_t(f) * uint32_t(ctas) / uint32_t(total));
    while (c + 1 < ctas && range_lo(total, c + 1, ctas) <= f) ++c;
    while (c > 0 && range_lo(total, c, ctas) > f) --c;
    return c;
}

// Adds the partial tiles of one output tile in CTA order and writes the result. Kept out of line so
// that its registers (every contributor's load is issued before the first add: the fold costs about
// one L2 round trip per item instead of one per contributor) do not weigh on the conversion loop.
template <int NT>
__device__ __noinline__ void fold_partials(const GemmArgs &a, const GemmSeg &seg, int row0, int tok0, int c_first, int c_last,
                                           int tid) {
    const int ntok = min(NT, a.n - tok0);
    const int ncontrib = c_last - c_first + 1;
    const size_t slot_floats = size_t(kTileM) * NT;
    for (int item = tid; item < ntok * (kTileM / 4); item += kConvertThreads) {
        const int t = item >> 5, rr = (item & 31) * 4;
        float4 pv[8];
#pragma unroll
        for (int k = 0; k < 8; ++k) {
            if (k < ncontrib) {
                const int c = c_first + k;
                const int which = k == 0 ? 1 : 0;  // only the first contributor's range starts before the tile
                pv[k] = __ldcg(reinterpret_cast<const float4 *>(a.scratch + (size_t(c) * 2 + which) * slot_floats +
                                                                t * kTileM + rr));
            } else {
                pv[k] = make_float4(0.f, 0.f, 0.f, 0.f);
            }
        }
        float4 sum = pv[0];
#pragma unroll
        for (int k = 1; k < 8; ++k) {
            if (k < ncontrib) {
                sum.x += pv[k].x;
                sum.y += pv[k].y;
                sum.z += pv[k].z;
                sum.w += pv[k].w;
            }
        }
        for (int c = c_first + 8; c <= c_last; ++c) {  // more than eight contributors: rare
            const int which = 0;
            const float4 more = __ldcg(reinterpret_cast<const float4 *>(a.scratch + (size_t(c) * 2 + which) * slot_floats +
                                                                        t * kTileM + rr));
            sum.x += more.x;
            sum.y += more.y;
            sum.z += more.z;
            sum.w += more.w;
        }
        const int tok = tok0 + t;
        const float s4[4] = {sum.x, sum.y, sum.z, sum.w};
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            const int orow = row0 + rr + e;
            if (orow < seg.rows) {
                float out = s4[e];
                if (seg.res != nullptr) out = seg.res[size_t(tok) * seg.rows + orow] + out;
                seg.y[size_t(tok) * seg.rows + orow] = out;
            }
        }
    }
}

template <int TYPE, int NT, bool XT>
__global__ void __launch_bounds__(kGemmThreads, 1)
    gemm_tc_kernel(const GemmArgs a, const __grid_constant__ CUtensorMap tm0, const __grid_constant__ CUtensorMap tm1,
                   const __grid_constant__ CUtensorMap tm2, const __grid_constant__ CUtensorMap tmx) {
    extern __shared__ uint8_t smem_raw[];
    using S = GemmSmem<TYPE, NT>;
    using R = RawFmt<TYPE>;
    constexpr int RS = S::raw_stages;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int trace = trace_begin(kTraceGemm);
    JL_TRACE_MODE_LOCAL;
    // 1024-byte aligned base: the swizzle pattern is a function of the shared address.
    uint8_t *base = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    constexpr int ST = S::stages;
    // The per-stage event log of CTA 0 is a build of its own (-DJL_TRACE -DJL_TRACE_EVENTS): its bookkeeping costs
    // registers that the timeline build would have to spill.
#ifdef JL_TRACE_EVENTS
    unsigned long long *slog = reinterpret_cast<unsigned long long *>(base + S::log_off);
    const bool logging = blockIdx.x == 0 && a.nseg == 2;
    if (tid < 512) slog[tid] = 0ull;
#define SLOG(idx, cond) do { if (logging && (cond)) slog[(idx)] = static_cast<unsigned long long>(clock64()); } while (0)
#else
#define SLOG(idx, cond) do { } while (0)
#endif
    uint64_t *a_free = reinterpret_cast<uint64_t *>(base + S::bar_off);  // [ST] tensor core done with operand stage
    uint64_t *a_full = a_free + ST;                                       // [ST] operand stage written
    uint64_t *raw_full = a_full + ST;                                     // [RS] raw bytes landed
    uint64_t *raw_empty = raw_full + RS;                                  // [RS] raw bytes consumed
    uint64_t *acc_full = raw_empty + RS;                                  // accumulator finished
    uint64_t *acc_empty = acc_full + 1;                                   // accumulator read out
    uint64_t *fix_bar = acc_empty + 1;                                    // conversion warps' own barrier
    uint32_t *tmem_ptr = reinterpret_cast<uint32_t *>(base + S::bar_off + S::bar_bytes - 16);
    volatile uint32_t *fold_flags = reinterpret_cast<uint32_t *>(base + S::bar_off + S::bar_bytes - 64);  // two sets of four
    volatile uint32_t *abort_flag = tmem_ptr + 2;
    constexpr uint32_t tmem_cols = kTmemCols;

    int tiles = 0;
    for (int s = 0; s < a.nseg; ++s) tiles += (a.seg[s].rows + kTileM - 1) / kTileM;
    const int n_tiles = (a.n + NT - 1) / NT;
    const int raw_total = a.cols / kRawK;
    const int total = tiles * n_tiles * raw_total;
    const int ctas = gridDim.x;
    const int lo = range_lo(total, blockIdx.x, ctas), hi = range_lo(total, blockIdx.x + 1, ctas);

    if (warp == kConvertWarps) tmem_alloc(tmem_ptr, tmem_cols);
    if (tid == 0) {
        for (int s = 0; s < ST; ++s) {
            mbar_init(a_free + s, 1);
            mbar_init(a_full + s, kConvertWarps / 2 + (XT ? 1 : 0));  // one group of eight warps per stage
        }
        for (int s = 0; s < RS; ++s) {
            mbar_init(raw_full + s, 1);
            mbar_init(raw_empty + s, kConvertWarps);
        }
        mbar_init(acc_full, 1);
        mbar_init(acc_empty, kConvertWarps);
        mbar_init(fix_bar, kConvertWarps);
        mbar_fence_init();
        *abort_flag = 0u;
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_d = *tmem_ptr;
    trace_mark(trace, 2);
    // The next kernel may start its preamble now; what of this kernel depends on the one before it
    // (activations, residuals, the outputs and the partial-tile workspace it writes) waits below:
    // the activation-copy thread and the conversion warps do, the weight-copy thread does not.
    pdl_launch_dependents();
#ifdef JL_TRACE
    unsigned tw_raw = 0, tw_free = 0, tw_acc = 0, tw_epi = 0, tw_pub = 0, tw_cvt = 0;
#endif

    if (warp == kConvertWarps + 1) {
        // ---- copy requests -------------------------------------------------------------------
        if (lane == 0) {
            const uint64_t policy = policy_evict_first();
            fence_proxy_async();
            int i = 0, cur_u = -1;
            TileRef tr = {0, 0};
            int u = lo / raw_total, r = lo - u * raw_total - 1;
            for (int f = lo; f < hi && *abort_flag == 0u; ++f, ++i) {
                if (++r == raw_total) {
                    r = 0;
                    ++u;
                }
                if (u != cur_u) {
                    cur_u = u;
                    tr = locate_tile(a, u / n_tiles);
                }
                const int st = i % RS;
                if (i >= RS && !GEMM_WAIT(raw_empty + st, uint32_t(i / RS - 1) & 1u)) {
                    *abort_flag = 1u;
                    atomicExch(a.status, kDevTimeout);
                    break;
                }
                SLOG(300 + (i - 4), i >= 4 && i < 12);
                const CUtensorMap *tmap = tr.seg == 0 ? &tm0 : (tr.seg == 1 ? &tm1 : &tm2);
                if (JL_TRACE_MODE(8)) {  // trace build, timing experiment: no copy at all, the stage is declared full
                    mbar_arrive(raw_full + st);
                    continue;
                }
                mbar_expect_tx(raw_full + st, R::stage_bytes);
                tma_load_2d(base + S::raw_off + st * R::stage_bytes, tmap, r * (R::row_bytes / 4), tr.row0,
                            raw_full + st, policy);
            }
        }
    } else if (warp == kConvertWarps + 2) {
        // ---- activation tiles by TMA (pre-split binary16 hi / lo rows), one request set per operand stage
        if (lane == 0 && XT) {
            pdl_wait();
            int i = 0;
            int u = lo / raw_total, r = lo - u * raw_total - 1;
            for (int f = lo; f < hi && *abort_flag == 0u; ++f, ++i) {
                if (++r == raw_total) {
                    r = 0;
                    ++u;
                }
                const int tok0 = (u % n_tiles) * NT;
                bool ok = true;
                for (int j = 0; j < 2 && ok; ++j) {
                    const int q = 2 * i + j, s = q % ST;
                    if (q >= ST) ok = GEMM_WAIT(a_free + s, uint32_t(q / ST - 1) & 1u);
                    if (!ok) break;
                    uint8_t *b_st = base + S::b_off + s * S::b_stage;
                    const int k0 = r * kRawK + j * kStageK;
                    SLOG(320 + (q - 8), q >= 8 && q < 24);
                    if (JL_TRACE_MODE(64)) {  // trace build, timing experiment: no activation copy
                        mbar_arrive(a_full + s);
                        continue;
                    }
                    mbar_expect_tx(a_full + s, S::b_stage);
#pragma unroll
                    for (int atom = 0; atom < 2; ++atom) {
                        tma_load_2d_plain(b_st + atom * S::b_sub, &tmx, k0 + atom * 64, tok0, a_full + s);
                        tma_load_2d_plain(b_st + atom * S::b_sub + NT * 128, &tmx, k0 + atom * 64, a.x_lo_row + tok0,
                                          a_full + s);
                    }
                }
                if (!ok) {
                    *abort_flag = 1u;
                    atomicExch(a.status, kDevTimeout);
                    break;
                }
            }
        }
    } else if (warp == kConvertWarps) {
        // ---- tensor-core issue ---------------------------------------------------------------
        // An operand stage is only handed back (a_free) once its eight MMAs are issued, so this
        // warp's instruction count per stage is on the kernel's critical path: it shares its scheduler
        // with four conversion warps that are always ready to issue. The loop carries the stage index,
        // the barrier parity, the tensor-memory column and the descriptor's address word as running
        // values, the descriptor's constant upper word is built once, and the whole warp runs the loop
        // converged (one elected lane issues), so every operand is warp-uniform.
        {
            constexpr uint32_t idesc = instr_desc_f16(2 * NT);
            constexpr uint32_t desc_hi = uint32_t(1024 >> 4) | (1u << 14) | (2u << 29);  // SBO, version, 128-byte swizzle
            constexpr uint32_t b_step = uint32_t(S::b_stage >> 4);
            constexpr int kAtom = S::b_sub >> 4;  // descriptor step between the two 64-column atoms
            const uint32_t a_col0 = tmem_d + TmemPlan<NT>::a_stage0;
            const uint32_t b_lo0 = ((smem_u32(base + S::b_off) >> 4) & 0x3FFFu) | (1u << 16);
            const uint32_t full0 = smem_u32(a_full), free0 = smem_u32(a_free), acc_full_u32 = smem_u32(acc_full);
            int s = 0, done = 0;
#ifdef JL_TRACE_EVENTS
            int qlog = 0;
#endif
            uint32_t parity = 0, a_col = a_col0, b_lo = b_lo0;
            bool ok = true;
            int f = lo;
            while (f < hi && ok && *abort_flag == 0u) {
                const int u_lo = f / raw_total * raw_total;
                const int seg_end = u_lo + raw_total < hi ? u_lo + raw_total : hi;
                const int nstage = 2 * (seg_end - f);  // operand stages of this CTA's share of the tile
#ifdef JL_TRACE
                const unsigned tm2_ = unsigned(clock());
#endif
                if (done > 0) ok = GEMM_WAIT(acc_empty, uint32_t(done - 1) & 1u);
#ifdef JL_TRACE
                tw_cvt += unsigned(clock()) - tm2_;
#endif
                for (int k = 0; k < nstage && ok; ++k) {
#ifdef JL_TRACE
                    const unsigned tm0_ = unsigned(clock());
#endif
                    ok = mbar_poll_bounded_u32(full0 + 8u * uint32_t(s), parity);
#ifdef JL_TRACE
                    tw_pub += unsigned(clock()) - tm0_;
#endif
                    if (!ok) break;
                    SLOG(256 + (qlog - 8) * 2, lane == 0 && qlog >= 8 && qlog < 24);
                    __syncwarp();  // elect.sync below names every lane
                    tc_fence_after();
                    umma_stage_f16_tmem_a<2, 4, 6, kAtom, kAtom + 2, kAtom + 4, kAtom + 6>(
                        tmem_d, a_col, b_lo, desc_hi, idesc, free0 + 8u * uint32_t(s), k == 0 ? 0u : 1u);
                    SLOG(256 + (qlog - 8) * 2 + 1, lane == 0 && qlog >= 8 && qlog < 24);
#ifdef JL_TRACE_EVENTS
                    ++qlog;
#endif
                    if (++s == ST) {
                        s = 0;
                        parity ^= 1u;
                        a_col = a_col0;
                        b_lo = b_lo0;
                    } else {
                        a_col += kTmemAStageCols;
                        b_lo += b_step;
                    }
                }
                if (!ok) break;
                __syncwarp();
                umma_commit_elect(acc_full_u32);
                ++done;
                f = seg_end;
            }
            if (!ok && lane == 0) {
                *abort_flag = 1u;
                atomicExch(a.status, kDevTimeout);
            }
#ifdef JL_TRACE
            if (lane == 0) {
                trace_cta_word(4, 0, static_cast<unsigned long long>(tw_pub));  // issue warp: waits for full operand stages
                trace_cta_word(4, 1, static_cast<unsigned long long>(tw_cvt));  // ... and for the accumulator to be read out
            }
#endif
        }
    } else {
        // ---- operand conversion and epilogue (warps 0-15) -------------------------------------
        // Two groups of eight warps take alternate operand stages (group 0 the first 128 columns of
        // every raw stage, group 1 the second): a thread converts a whole 64-column unit of its row,
        // so block headers, scale unpacking and barrier traffic are paid once per 64 weights.
        // Converting weights depends on nothing the kernel ahead produces: with pre-split activations these warps fill
        // the operand ring first and wait for that kernel only before their first epilogue (results, residuals,
        // the partial-tile workspace). When they convert the activations themselves they wait here.
        bool waited = false;
        if (!XT) {
            pdl_wait();
            waited = true;
        }
        constexpr int kGroupThreads = kConvertThreads / 2;
        const int grp = warp >> 3, g_tid = tid & (kGroupThreads - 1);
        const int a_row = g_tid & 127, a_unit = g_tid >> 7;  // a_unit: which 64-column unit of the 128
        constexpr int kBChunks = NT * 16;  // 16-byte chunks of eight activations per operand stage
        // converting activations inside the kernel (no pre-split buffer) is kept for tiles up to 64 tokens
        constexpr int kBPerThread = (!XT && NT <= 64) ? (kBChunks + kGroupThreads - 1) / kGroupThreads : 0;
        const int lane_grp = warp & 3, col_grp = warp >> 2;  // epilogue: TMEM lanes 32*lane_grp, columns 16*col_grp
        int i = 0, done = 0, fix_phase = 0, fold_turn = 0;
        TileRef tr = {0, 0};
        int tok0 = 0;
        bool ok = true;
        // An operand stage is published (a_full) one stage late: the tensor-memory stores of stage i
        // are waited for after stage i + 1 has been converted, when they have long landed, instead
        // of right after they were issued. With fewer than three operand stages the stage that has
        // to become free next would be the unpublished one, so there the stage is published at once.
        constexpr bool kDefer = ST >= 3;
        int pending = -1;
        const uint32_t raw_full0 = smem_u32(raw_full), raw_empty0 = smem_u32(raw_empty);
        const uint32_t a_free0 = smem_u32(a_free), a_full0 = smem_u32(a_full);
        auto publish = [&]() {
            if (pending < 0) return;
            tmem_wait_st();
            tc_fence_before();
            if (!XT) fence_proxy_async();
            __syncwarp();
            if (lane == 0) mbar_arrive_u32(a_full0 + 8u * uint32_t(pending));
            pending = -1;
        };
        // The loop's indices are running values (raw ring slot and parity, this group's operand stage
        // and how often it has wrapped): with four conversion warps on every scheduler, scalar
        // bookkeeping between two conversions costs several cycles per instruction.
        const uint32_t raw_row0 = smem_u32(base + S::raw_off) + uint32_t(a_row) * R::row_bytes;
        // this thread's row is TMEM lane a_row (its warp may touch lanes 32 * (warp % 4) ..); its 64
        // weights are columns a_unit * 32 .. + 31 of the operand stage
        const uint32_t tm_col0 = tmem_d + (uint32_t(a_row & ~31) << 16) + TmemPlan<NT>::a_stage0 + uint32_t(a_unit) * 32u;
        int st = 0, s = grp % ST, rev = grp / ST;
        uint32_t raw_par = 0;
        int f = lo;
        while (f < hi && ok && *abort_flag == 0u) {
            const int u = f / raw_total;
            const int u_lo = u * raw_total;
            const int seg_end = u_lo + raw_total < hi ? u_lo + raw_total : hi;
            const int nraw = seg_end - f;
            int r = f - u_lo;
            tr = locate_tile(a, u / n_tiles);
            tok0 = (u % n_tiles) * NT;
          for (int it = 0; it < nraw && *abort_flag == 0u; ++it, ++r, ++i) {
#ifdef JL_TRACE
            const unsigned tq0 = unsigned(clock());
#endif
#ifdef JL_TRACE_EVENTS
            const bool lgw = (tid == 0 || tid == 256 || tid == 96) && i >= 4 && i < 12;
            const int lg = (tid == 0 ? 0 : (tid == 256 ? 80 : 160)) + (i - 4) * 10;
            SLOG(lg, lgw);
#endif
            ok = mbar_poll_bounded_u32(raw_full0 + 8u * uint32_t(st), raw_par);
#ifdef JL_TRACE
            tw_raw += unsigned(clock()) - tq0;
            SLOG(lg + 1, lgw);
            if (i == 0) trace_mark(trace, 3);
#endif
            if (!ok) break;
            const uint32_t row_u32 = raw_row0 + uint32_t(st) * R::stage_bytes;
            {
                const int j = grp;
                const int k0 = r * kRawK + j * kStageK;
                // Activations first: their loads are in flight while the weights are converted.
                float4 xv[kBPerThread > 0 ? kBPerThread : 1][2];
#pragma unroll
                for (int uu = 0; uu < kBPerThread; ++uu) {
                    const int ch = g_tid + uu * kGroupThreads;
                    const int t = ch >> 4, kc = ch & 15;
                    const int tok = tok0 + t;
                    if (ch < kBChunks && tok < a.n) {
                        const float4 *src = reinterpret_cast<const float4 *>(a.x + size_t(tok) * a.cols + k0 + kc * 8);
                        xv[uu][0] = __ldg(src);
                        xv[uu][1] = __ldg(src + 1);
                    } else {
                        xv[uu][0] = xv[uu][1] = make_float4(0.f, 0.f, 0.f, 0.f);
                    }
                }
#ifdef JL_TRACE
                const unsigned tq1 = unsigned(clock());
#endif
                if (rev > 0) ok = mbar_poll_bounded_u32(a_free0 + 8u * uint32_t(s), uint32_t(rev - 1) & 1u);
#ifdef JL_TRACE
                tw_free += unsigned(clock()) - tq1;
                SLOG(lg + 2, lgw);
#endif
                if (ok) {
                uint8_t *b_st = base + S::b_off + s * S::b_stage;
                if (!JL_TRACE_MODE(1)) {  // always true outside the trace build
                    tc_fence_after();  // the stage's previous MMAs are complete (a_free): order the store after them
                    const uint32_t col0 = tm_col0 + uint32_t(s) * kTmemAStageCols;
#ifdef JL_TRACE
                    const unsigned tq4 = unsigned(clock());
#endif
                    publish();  // the previous stage of this group: its stores were issued a whole conversion ago
#ifdef JL_TRACE
                    const unsigned tq5 = unsigned(clock());
                    tw_pub += tq5 - tq4;
#endif
                    // (Rows past the end of a matrix, in its bottom tile, need no care: the copy engine
                    // fills them with zero bytes, which every format converts to zero weights.)
                    SLOG(lg + 5, lgw);
                    UnitRegs<TYPE> unit_regs;
                    unit_load<TYPE>(row_u32, 2 * j + a_unit, unit_regs);
#ifdef JL_TRACE_EVENTS
                    if (logging && lgw) {  // the stamp waits for the header arithmetic
                        if constexpr (TYPE == kQ4_K) {
                            if (h2_bits(unit_regs.clo2[1]) == 0x12345678u) slog[500] = 1;
                        }
                        slog[lg + 6] = static_cast<unsigned long long>(clock64());
                    }
#endif
#pragma unroll
                    for (int hf = 0; hf < 2; ++hf) {
                        uint32_t cols[16];
                        unit_convert<TYPE>(unit_regs, hf, cols);
#ifdef JL_TRACE_EVENTS
                        if (logging && lgw) {
                            if (cols[15] == 0x12345678u) slog[501] = 1;
                            slog[lg + 7 + hf] = static_cast<unsigned long long>(clock64());
                        }
#endif
                        tmem_st16(col0 + 16u * hf, cols);
                    }
#ifdef JL_TRACE
                    tw_cvt += unsigned(clock()) - tq5;
                    SLOG(lg + 3, lgw);
#endif
                } else {
                    publish();
                }
#pragma unroll
                for (int uu = 0; uu < kBPerThread; ++uu) {
                    const int ch = g_tid + uu * kGroupThreads;
                    if (ch < kBChunks && !JL_TRACE_MODE(2)) {
                        const int t = ch >> 4, kc = ch & 15;
                        const int atom = kc >> 3, c = kc & 7;
                        const float x[8] = {xv[uu][0].x, xv[uu][0].y, xv[uu][0].z, xv[uu][0].w,
                                            xv[uu][1].x, xv[uu][1].y, xv[uu][1].z, xv[uu][1].w};
                        float xl[8];
#pragma unroll
                        for (int e = 0; e < 8; ++e) xl[e] = x[e] - __half2float(__float2half_rn(x[e]));
                        const uint32_t off = sw128_offset(t, c);
                        uint8_t *bh = b_st + size_t(atom) * S::b_sub;
                        uint8_t *bl = bh + NT * 128;  // the lo rows follow the hi rows of the same atom
                        // pairs (k0, k2), (k1, k3) inside every group of four: the operand order
                        *reinterpret_cast<uint4 *>(bh + off) = make_uint4(pack_half2(x[0], x[2]), pack_half2(x[1], x[3]),
                                                                         pack_half2(x[4], x[6]), pack_half2(x[5], x[7]));
                        *reinterpret_cast<uint4 *>(bl + off) = make_uint4(pack_half2(xl[0], xl[2]), pack_half2(xl[1], xl[3]),
                                                                         pack_half2(xl[4], xl[6]), pack_half2(xl[5], xl[7]));
                    }
                }
                // Generic-proxy writes to shared memory (the B operand, when converted here) must be
                // visible to the tensor core's async-proxy reads; the A operand went to tensor memory:
                // both are settled in publish().
                pending = s;
                if (!kDefer) publish();
                s += 2;
                if (s >= ST) {
                    s -= ST;
                    ++rev;
                }
                }
            }
            if (!ok) break;
            // This warp has read both halves of the raw stage: hand its share back.
            __syncwarp();
            if (lane == 0) mbar_arrive_u32(raw_empty0 + 8u * uint32_t(st));
            SLOG(lg + 4, lgw);
            if (++st == RS) {
                st = 0;
                raw_par ^= 1u;
            }
          }
            if (!ok || *abort_flag != 0u) break;
            // ---- this CTA's share of output tile u is complete -----------------------------------
            const int seg_begin = u_lo > lo ? u_lo : lo;
            const bool whole = seg_begin == u_lo && seg_end == u_lo + raw_total;
            const GemmSeg seg = a.seg[tr.seg];
            publish();  // the accumulator cannot finish before the last stage is published
            if (!waited) {
                pdl_wait();
                waited = true;
            }
#ifdef JL_TRACE
            const unsigned tq2 = unsigned(clock());
#endif
            ok = GEMM_WAIT(acc_full, uint32_t(done) & 1u);
#ifdef JL_TRACE
            tw_acc += unsigned(clock()) - tq2;
            const unsigned tq3 = unsigned(clock());
#endif
            if (!ok) break;
            ++done;
            tc_fence_after();
            // partial slot: 0 if this CTA's range starts inside the tile, 1 if it only ends inside it
            float *slot = a.scratch + (size_t(blockIdx.x) * 2 + (seg_begin > u_lo ? 0 : 1)) * (size_t(kTileM) * NT);
#pragma unroll
            for (int cg = col_grp; cg * 16 < NT; cg += 4) {
                float v[16], vl[16];
                tmem_ld16(tmem_d + (uint32_t(lane_grp * 32) << 16) + uint32_t(cg * 16), v);
                tmem_ld16(tmem_d + (uint32_t(lane_grp * 32) << 16) + uint32_t(NT + cg * 16), vl);
#pragma unroll
                for (int jc = 0; jc < 16; ++jc) v[jc] += vl[jc];
                const int rr = lane_grp * 32 + lane;
                const int row = tr.row0 + rr;
#pragma unroll
                for (int jc = 0; jc < 16; ++jc) {
                    const int t = cg * 16 + jc;
                    const int tok = tok0 + t;
                    if (whole) {
                        if (row < seg.rows && tok < a.n) {
                            float out = v[jc];
                            if (seg.res != nullptr) out = seg.res[size_t(tok) * seg.rows + row] + out;
                            seg.y[size_t(tok) * seg.rows + row] = out;
                        }
                    } else {
                        slot[t * kTileM + rr] = v[jc];
                    }
                }
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(acc_empty);
            if (!whole) {
                // The CTA that arrives last adds the partial tiles in CTA order. The barrier orders
                // every thread's partial stores before thread 0's fence, which is cumulative.
                // Thread 0 alone works out who contributes (integer divisions) and leaves the answer
                // in one of two sets of flag words, taken in turn, so that a set is not rewritten
                // while a slower warp still reads it.
                ok = convert_warps_sync(fix_bar, fix_phase);
                if (!ok) break;
                volatile uint32_t *fl = fold_flags + 4 * (fold_turn & 1);
                ++fold_turn;
                if (tid == 0) {
                    const int c_first = cta_of(total, u_lo, ctas), c_last = cta_of(total, u_lo + raw_total - 1, ctas);
                    __threadfence();
                    const unsigned prev = atomicAdd(a.counters + u, 1u);
                    fl[1] = uint32_t(c_first);
                    fl[2] = uint32_t(c_last);
                    fl[0] = prev == unsigned(c_last - c_first) ? 1u : 0u;
                }
                ok = convert_warps_sync(fix_bar, fix_phase);
                if (!ok) break;
                if (fl[0] != 0u) {
                    __threadfence();
                    fold_partials<NT>(a, seg, tr.row0, tok0, int(fl[1]), int(fl[2]), tid);
                    if (tid == 0) a.counters[u] = 0u;
                }
            }
#ifdef JL_TRACE
            tw_epi += unsigned(clock()) - tq3;
#endif
            f = seg_end;
        }
#ifdef JL_TRACE
        trace_mark(trace, 4);
        trace_word(trace, 6, (static_cast<unsigned long long>(tw_raw) << 32) | static_cast<unsigned long long>(tw_free));
        trace_word(trace, 7, (static_cast<unsigned long long>(tw_acc) << 32) | static_cast<unsigned long long>(tw_epi));
        if (tid == 0) {  // this CTA's own sums, in the per-CTA cells
            trace_cta_word(5, 0, static_cast<unsigned long long>(tw_pub));
            trace_cta_word(5, 1, static_cast<unsigned long long>(tw_cvt));
            trace_cta_word(5, 2, static_cast<unsigned long long>(tw_raw));
            trace_cta_word(5, 3, static_cast<unsigned long long>(tw_free));
            trace_cta_word(5, 4, static_cast<unsigned long long>(tw_acc));
            trace_cta_word(5, 5, static_cast<unsigned long long>(tw_epi));
            trace_cta_word(5, 6, static_cast<unsigned long long>(i));
        }
#endif
        if (!ok && lane == 0) {
            *abort_flag = 1u;
            atomicExch(a.status, kDevTimeout);
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == kConvertWarps) tmem_dealloc(tmem_d, tmem_cols);
#ifdef JL_TRACE_EVENTS
    if (logging && tid < 512) trace_log(tid, slog[tid]);
#endif
    trace_mark(trace, 5);
}

template <int TYPE, int NT>
cudaError_t launch_nt(const GemmArgs &a, cudaStream_t stream) {
    int tiles = 0;
    for (int s = 0; s < a.nseg; ++s) tiles += (a.seg[s].rows + kTileM - 1) / kTileM;
    const int n_tiles = (a.n + NT - 1) / NT;
    const long long total = (long long)tiles * n_tiles * (a.cols / kRawK);
    const int sms = a.sm_count > 0 ? a.sm_count : 148;
    long long ctas = total / 2 < sms ? total / 2 : sms;  // at least two raw stages per CTA
    if (ctas < 1) ctas = 1;
    // Fewer output tiles than SMs: a whole number of CTAs per tile, so that each CTA's range lies
    // inside one tile and it takes part in one partial-tile fold instead of two.
    const long long units = (long long)tiles * n_tiles;
    if (units < ctas && ctas / units >= 1) {
        long long per = ctas / units;
        const int raw_total = a.cols / kRawK;
        if (per > raw_total / 2) per = raw_total / 2 > 0 ? raw_total / 2 : 1;
        ctas = units * per;
    }
    if (total * ctas >= (1ll << 32)) return cudaErrorInvalidValue;  // the kernel's work-list arithmetic is 32-bit
    if (a.scratch == nullptr || a.counters == nullptr || tiles * n_tiles > a.counters_len ||
        size_t(ctas) * 2 * kTileM * NT > a.scratch_floats)
        return cudaErrorInvalidValue;
    CUtensorMap maps[4];
    for (int s = 0; s < 3; ++s) memcpy(&maps[s], a.seg[s < a.nseg ? s : 0].tmap->bytes, sizeof(CUtensorMap));
    memcpy(&maps[3], (a.xmap != nullptr ? a.xmap : a.seg[0].tmap)->bytes, sizeof(CUtensorMap));
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(unsigned(ctas));
    cfg.blockDim = dim3(kGemmThreads);
    cfg.dynamicSmemBytes = GemmSmem<TYPE, NT>::total;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = a.programmatic ? 1 : 0;
    if (a.xmap != nullptr) return cudaLaunchKernelEx(&cfg, gemm_tc_kernel<TYPE, NT, true>, a, maps[0], maps[1], maps[2], maps[3]);
    return cudaLaunchKernelEx(&cfg, gemm_tc_kernel<TYPE, NT, false>, a, maps[0], maps[1], maps[2], maps[3]);
}

template <int TYPE>
cudaError_t launch_type(const GemmArgs &a, cudaStream_t stream) {
    if (a.n <= 16) return launch_nt<TYPE, 16>(a, stream);
    if (a.n <= 32) return launch_nt<TYPE, 32>(a, stream);
    if (a.n <= 64 || a.xmap == nullptr) return launch_nt<TYPE, 64>(a, stream);
    return launch_nt<TYPE, 128>(a, stream);
}

template <int TYPE, int NT>
cudaError_t configure_nt() {
    cudaError_t e = cudaFuncSetAttribute(gemm_tc_kernel<TYPE, NT, true>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         GemmSmem<TYPE, NT>::total);
    if (e != cudaSuccess) return e;
    return cudaFuncSetAttribute(gemm_tc_kernel<TYPE, NT, false>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                GemmSmem<TYPE, NT>::total);
}

template <int TYPE>
cudaError_t configure_type() {
    cudaError_t e;
    if ((e = configure_nt<TYPE, 16>()) != cudaSuccess) return e;
    if ((e = configure_nt<TYPE, 32>()) != cudaSuccess) return e;
    if ((e = configure_nt<TYPE, 64>()) != cudaSuccess) return e;
    return configure_nt<TYPE, 128>();
}

}  // namespace

cudaError_t gemm_make_tensor_map(GemmTensorMap *out, const void *w_dev, int type, int64_t rows, int64_t cols) {
    static_assert(sizeof(CUtensorMap) == sizeof(GemmTensorMap), "descriptor size");
    // (a Q6_K matrix is passed as its padded copy: kQ6_KPadded bytes per super-block)
    if (!out || !w_dev || !(is_quant(type) || is_extra_quant(type)) || rows <= 0 || cols <= 0 || cols % kRawK != 0)
        return cudaErrorInvalidValue;
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
    const uint32_t raw_bytes = type == kQ8_0   ? 272u
                               : type == kQ6_K ? uint32_t(kQ6_KPadded)
                               : type == kQ5_K ? uint32_t(kQ5_KBytes)
                               : type == kQ4_1 ? uint32_t(8 * kQ4_1Bytes)
                                               : 144u;
    const uint64_t rowb = type == kQ6_K ? uint64_t(cols / kRawK) * kQ6_KPadded : uint64_t(row_bytes(type, cols));
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

int gemm_token_tile(int n) { return n <= 16 ? 16 : (n <= 32 ? 32 : (n <= 64 ? 64 : 128)); }  // with pre-split activations

cudaError_t gemm_make_activation_map(GemmTensorMap *out, const void *x16_dev, int64_t row_cap, int64_t cols, int nt) {
    if (!out || !x16_dev || row_cap <= 0 || cols <= 0 || cols % 64 != 0 || (nt != 16 && nt != 32 && nt != 64 && nt != 128))
        return cudaErrorInvalidValue;
    typedef CUresult (*EncodeFn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *,
                                 const cuuint64_t *, const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave,
                                 CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
    void *fn = nullptr;
    cudaDriverEntryPointQueryResult q;
    cudaError_t e = cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &q);
    if (e != cudaSuccess) return e;
    if (q != cudaDriverEntryPointSuccess || fn == nullptr) return cudaErrorNotSupported;
    const cuuint64_t gdim[2] = {cuuint64_t(cols), cuuint64_t(2 * row_cap)};
    const cuuint64_t gstride[1] = {cuuint64_t(cols) * 2};
    const cuuint32_t box[2] = {64, cuuint32_t(nt)};  // 64 binary16 = one 128-byte swizzle row
    const cuuint32_t estride[2] = {1, 1};
    CUtensorMap map;
    const CUresult r = reinterpret_cast<EncodeFn>(fn)(&map, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, const_cast<void *>(x16_dev),
                                                      gdim, gstride, box, estride, CU_TENSOR_MAP_INTERLEAVE_NONE,
                                                      CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                                                      CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return cudaErrorInvalidValue;
    memcpy(out->bytes, &map, sizeof map);
    return cudaSuccess;
}

cudaError_t gemm_tc_configure() {
    cudaError_t e;
    if ((e = configure_type<kQ4_K>()) != cudaSuccess) return e;
    if ((e = configure_type<kQ4_0>()) != cudaSuccess) return e;
    if ((e = configure_type<kQ6_K>()) != cudaSuccess) return e;
    if ((e = configure_type<kQ5_K>()) != cudaSuccess) return e;
    if ((e = configure_type<kQ4_1>()) != cudaSuccess) return e;
    return configure_type<kQ8_0>();
}

cudaError_t gemm_tc_launch(const GemmArgs &a, cudaStream_t stream) {
    if (a.cols <= 0 || a.cols % 256 != 0 || a.n <= 0 || a.nseg < 1 || a.nseg > 3) return cudaErrorInvalidValue;
    int tiles = 0;
    for (int s = 0; s < a.nseg; ++s) {
        if (a.seg[s].rows <= 0 || a.seg[s].w == nullptr || a.seg[s].y == nullptr || a.seg[s].tmap == nullptr)
            return cudaErrorInvalidValue;
        tiles += (a.seg[s].rows + kTileM - 1) / kTileM;
    }
    // One arrival counter per output tile: very tall products go in token slabs that fit the counters.
    int slab = a.n;
    if (a.counters_len > 0 && tiles <= a.counters_len) {
        const int max_tiles_n = a.counters_len / tiles;
        const int widest = a.xmap != nullptr ? 128 : 64;  // the token tile launch_type will pick for a tall product
        if ((a.n + widest - 1) / widest > max_tiles_n) slab = max_tiles_n * widest;
    }
    if (a.xmap != nullptr && slab < a.n) return cudaErrorInvalidValue;  // pre-split activations: one slab only
    for (int t0 = 0; t0 < a.n; t0 += slab) {
        GemmArgs part = a;
        part.n = a.n - t0 < slab ? a.n - t0 : slab;
        part.x = a.x + size_t(t0) * a.cols;
        for (int s = 0; s < a.nseg; ++s) {
            part.seg[s].y = a.seg[s].y + size_t(t0) * a.seg[s].rows;
            if (a.seg[s].res != nullptr) part.seg[s].res = a.seg[s].res + size_t(t0) * a.seg[s].rows;
        }
        cudaError_t e;
        switch (a.type) {
            case kQ4_K: e = launch_type<kQ4_K>(part, stream); break;
            case kQ4_0: e = launch_type<kQ4_0>(part, stream); break;
            case kQ8_0: e = launch_type<kQ8_0>(part, stream); break;
            case kQ6_K: e = launch_type<kQ6_K>(part, stream); break;
            case kQ5_K: e = launch_type<kQ5_K>(part, stream); break;
            case kQ4_1: e = launch_type<kQ4_1>(part, stream); break;
            default: return cudaErrorInvalidValue;
        }
        if (e != cudaSuccess) return e;
    }
    return cudaSuccess;
}

}  // namespace jl
