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
