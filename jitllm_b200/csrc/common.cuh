// Shared device helpers for the sm_100a kernels: mbarrier + bulk-async-copy (TMA) wrappers with
// bounded waits, programmatic-dependent-launch controls, warp reductions.
#pragma once

#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace jl {

constexpr int kWarp = 32;

// Device-side status word values (written by kernels, read by the host after a step).
enum : int { kDevOk = 0, kDevTimeout = 1, kDevBadArg = 2 };

__device__ __forceinline__ uint32_t smem_u32(const void *p) {
    return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

// ---- mbarrier -------------------------------------------------------------------------------
__device__ __forceinline__ void mbar_init(uint64_t *bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void mbar_fence_init() {
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t *bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)),
                 "r"(bytes)
                 : "memory");
}
// try_wait may block in hardware for up to the hinted time, so a waiting warp does not spend
// issue slots polling.
constexpr uint32_t kSuspendHintNs = 20000;
__device__ __forceinline__ bool mbar_try_wait(uint64_t *bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(smem_u32(bar)), "r"(parity), "r"(kSuspendHintNs)
        : "memory");
    return ok != 0;
}
// Bounded wait: gives up after `limit` polls (each poll may itself suspend for a
// hardware-defined time), so a copy that never lands cannot hang the GPU.
__device__ __forceinline__ bool mbar_wait_bounded(uint64_t *bar, uint32_t parity,
                                                  uint32_t limit = (1u << 16)) {
    for (uint32_t i = 0; i < limit; ++i) {
        if (mbar_try_wait(bar, parity)) return true;
    }
    return false;
}

// Polling wait without the suspend hint, for waits that are expected to end within a microsecond
// or two and sit on a kernel's critical path: test_wait never parks the thread, so the waiter
// continues on the cycle the phase flips. Bounded like the other wait (about a second of polls).
__device__ __forceinline__ bool mbar_test_wait(uint64_t *bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(smem_u32(bar)), "r"(parity)
        : "memory");
    return ok != 0;
}
__device__ __forceinline__ bool mbar_spin_bounded(uint64_t *bar, uint32_t parity, uint32_t limit = (1u << 26)) {
    for (uint32_t i = 0; i < limit; ++i) {
        if (mbar_test_wait(bar, parity)) return true;
    }
    return false;
}
// Polling with a short sleep between polls: a waiting warp stays off the issue ports (a spinning warp
// takes slots from the warps that share its scheduler) and still notices the flip within ~50 ns.
__device__ __forceinline__ bool mbar_poll_bounded(uint64_t *bar, uint32_t parity, uint32_t limit = (1u << 24)) {
    for (uint32_t i = 0; i < limit; ++i) {
        if (mbar_test_wait(bar, parity)) return true;
        __nanosleep(40);
    }
    return false;
}

// ---- bulk async copy global -> shared (TMA engine, 1-D, no multicast) -------------------------
// dst and src 16-byte aligned, bytes a multiple of 16.
__device__ __forceinline__ void bulk_g2s(void *dst_smem, const void *src_gmem, uint32_t bytes,
                                         uint64_t *bar) {
    asm volatile(
        "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
        ::"r"(smem_u32(dst_smem)),
        "l"(src_gmem), "r"(bytes), "r"(smem_u32(bar))
        : "memory");
}
// Same with an L2 evict-first hint for data that is streamed once per step (weights).
__device__ __forceinline__ uint64_t policy_evict_first() {
    uint64_t pol;
    asm volatile("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;" : "=l"(pol));
    return pol;
}
__device__ __forceinline__ void bulk_g2s_hint(void *dst_smem, const void *src_gmem, uint32_t bytes,
                                              uint64_t *bar, uint64_t policy) {
    asm volatile(
        "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes.L2::cache_hint "
        "[%0], [%1], %2, [%3], %4;" ::"r"(smem_u32(dst_smem)),
        "l"(src_gmem), "r"(bytes), "r"(smem_u32(bar)), "l"(policy)
        : "memory");
}
// Same, with the shared-memory addresses already in their 32-bit form (no conversion per copy).
__device__ __forceinline__ void bulk_g2s_hint_u32(uint32_t dst_smem, const void *src_gmem, uint32_t bytes,
                                                  uint32_t bar_smem, uint64_t policy) {
    asm volatile(
        "cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes.L2::cache_hint "
        "[%0], [%1], %2, [%3], %4;" ::"r"(dst_smem),
        "l"(src_gmem), "r"(bytes), "r"(bar_smem), "l"(policy)
        : "memory");
}
__device__ __forceinline__ void mbar_expect_tx_u32(uint32_t bar_smem, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar_smem), "r"(bytes) : "memory");
}
__device__ __forceinline__ void fence_proxy_async() {
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}

// ---- explicit shared-memory loads (32-bit shared addresses, never generic) ---------------------
__device__ __forceinline__ uint4 lds128(uint32_t addr) {
    uint4 v;
    asm volatile("ld.shared.v4.u32 {%0, %1, %2, %3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
                 : "r"(addr));
    return v;
}
__device__ __forceinline__ uint2 lds64(uint32_t addr) {
    uint2 v;
    asm volatile("ld.shared.v2.u32 {%0, %1}, [%2];" : "=r"(v.x), "=r"(v.y) : "r"(addr));
    return v;
}
__device__ __forceinline__ uint32_t lds32(uint32_t addr) {
    uint32_t v;
    asm volatile("ld.shared.u32 %0, [%1];" : "=r"(v) : "r"(addr));
    return v;
}
__device__ __forceinline__ void sts32(uint32_t addr, uint32_t v) {
    asm volatile("st.shared.u32 [%0], %1;" ::"r"(addr), "r"(v) : "memory");
}

// ---- programmatic dependent launch ------------------------------------------------------------
// No-ops when the kernel was launched without the programmatic-serialization attribute.
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_launch_dependents() {
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
}

// ---- launch-timeline stamps (trace build only) ---------------------------------------------------
// With -DJL_TRACE the first CTA of every launch claims a record in a device buffer and stamps it
// with %globaltimer at a few points; without it these are empty inline functions, so the default
// library carries no tracing code at all. Each translation unit has its own copy of the buffer
// pointer, bound from the host by JL_TRACE_DEFINE_BIND's function.
constexpr int kTraceWords = 8;  // kernel id, five stamps, two free words
enum : int { kTraceGemv = 1, kTraceAttn = 2, kTraceEmbed = 3, kTraceAdvance = 4, kTraceGemm = 5, kTraceRows = 6,
             kTraceExchange = 7 };
#ifdef JL_TRACE
static __device__ unsigned long long *g_trace_buf;
static __device__ unsigned g_trace_cap;
static __device__ int g_trace_mode;  // experiment switches of the trace build (0 = none)
__device__ __forceinline__ unsigned long long trace_now() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
    return t;
}
// Thread 0 of CTA (0,0,0) claims the next record; every other thread gets -1.
__device__ __forceinline__ int trace_begin(int kernel_id) {
    if (threadIdx.x != 0 || blockIdx.x != 0 || blockIdx.y != 0 || blockIdx.z != 0 || g_trace_buf == nullptr) return -1;
    const unsigned slot = static_cast<unsigned>(atomicAdd(g_trace_buf, 1ull));
    if (slot >= g_trace_cap) return -1;
    unsigned long long *r = g_trace_buf + kTraceWords * (1 + size_t(slot));
    r[0] = static_cast<unsigned long long>(kernel_id);
    r[1] = trace_now();
    return static_cast<int>(slot);
}
__device__ __forceinline__ void trace_mark(int slot, int word) {
    if (slot >= 0) g_trace_buf[kTraceWords * (1 + size_t(slot)) + word] = trace_now();
}
__device__ __forceinline__ void trace_word(int slot, int word, unsigned long long v) {
    if (slot >= 0) g_trace_buf[kTraceWords * (1 + size_t(slot)) + word] = v;
}
// Every CTA calls this from one thread when it is done: word 1 of the header keeps the latest exit
// of any CTA so far, which the next kernel reads once its grid dependency is resolved.
__device__ __forceinline__ void trace_cta_exit() {
    if (g_trace_buf != nullptr) atomicMax(g_trace_buf + 1, trace_now());
}
__device__ __forceinline__ unsigned long long trace_latest_exit() {
    return g_trace_buf != nullptr ? __ldcg(g_trace_buf + 1) : 0ull;
}
// Per-CTA cells behind the records (kTraceCtaWords words for each of the first 1024 CTAs of the
// latest launch that writes them): how evenly the CTAs of one launch finish.
constexpr int kTraceCtaWords = 8;
constexpr int kTraceCtaMax = 160, kTraceClasses = 6;  // cells: [class of launch][CTA][word]
__device__ __forceinline__ void trace_cta_word(int cls, int word, unsigned long long v) {
    if (g_trace_buf != nullptr && blockIdx.x < kTraceCtaMax && cls < kTraceClasses)
        g_trace_buf[kTraceWords * (1 + size_t(g_trace_cap)) + (size_t(cls) * kTraceCtaMax + blockIdx.x) * kTraceCtaWords + word] = v;
}
// An event log of CTA 0 in the cells no CTA owns (rows 148..159 of every class: 576 words).
__device__ __forceinline__ void trace_log(int idx, unsigned long long v) {
    if (g_trace_buf == nullptr || blockIdx.x != 0 || idx < 0 || idx >= kTraceClasses * 96) return;
    const int cls = idx / 96, rem = idx % 96;
    g_trace_buf[kTraceWords * (1 + size_t(g_trace_cap)) + (size_t(cls) * kTraceCtaMax + 148 + rem / 8) * kTraceCtaWords + rem % 8] = v;
}
#define JL_TRACE_DEFINE_BIND(fn)                                                              \
    cudaError_t fn(unsigned long long *buf, unsigned cap, int mode) {                        \
        cudaError_t e_ = cudaMemcpyToSymbol(g_trace_buf, &buf, sizeof buf);                   \
        if (e_ == cudaSuccess) e_ = cudaMemcpyToSymbol(g_trace_mode, &mode, sizeof mode);     \
        return e_ != cudaSuccess ? e_ : cudaMemcpyToSymbol(g_trace_cap, &cap, sizeof cap);    \
    }
// The experiment switches, read once per kernel into a local named trace_mode (JL_TRACE_MODE_LOCAL):
// a test of the global inside a loop would put a global load on the path it is meant to time.
#define JL_TRACE_MODE_LOCAL const int trace_mode = g_trace_mode
#define JL_TRACE_MODE(bit) ((trace_mode & (bit)) != 0)
#else
__device__ __forceinline__ int trace_begin(int) { return -1; }
__device__ __forceinline__ void trace_mark(int, int) {}
__device__ __forceinline__ void trace_word(int, int, unsigned long long) {}
__device__ __forceinline__ void trace_cta_exit() {}
__device__ __forceinline__ unsigned long long trace_latest_exit() { return 0ull; }
__device__ __forceinline__ void trace_cta_word(int, int, unsigned long long) {}
__device__ __forceinline__ void trace_log(int, unsigned long long) {}
#define JL_TRACE_DEFINE_BIND(fn) \
    cudaError_t fn(unsigned long long *, unsigned, int) { return cudaSuccess; }
#define JL_TRACE_MODE_LOCAL constexpr int trace_mode = 0
#define JL_TRACE_MODE(bit) ((trace_mode & (bit)) != 0)
#endif

// ---- arithmetic helpers -----------------------------------------------------------------------
__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}

__device__ __forceinline__ float half_bits_to_float(uint32_t h16) {
    return __half2float(__ushort_as_half(static_cast<unsigned short>(h16)));
}

// VEC (2 or 4) consecutive binary16 values widened to binary32.
template <int VEC>
__device__ __forceinline__ void load_halfs(const __half *p, float (&f)[VEC]) {
    if constexpr (VEC == 4) {
        const uint2 u = *reinterpret_cast<const uint2 *>(p);
        const __half2 a = *reinterpret_cast<const __half2 *>(&u.x);
        const __half2 b = *reinterpret_cast<const __half2 *>(&u.y);
        const float2 fa = __half22float2(a), fb = __half22float2(b);
        f[0] = fa.x; f[1] = fa.y; f[2] = fb.x; f[3] = fb.y;
    } else {
        const __half2 a = *reinterpret_cast<const __half2 *>(p);
        const float2 fa = __half22float2(a);
        f[0] = fa.x; f[1] = fa.y;
    }
}

}  // namespace jl
