// Micro-benchmark behind the mat-vec kernel's staging rule: how fast one GPU reads HBM through rings
// of 1-D bulk copies (cp.async.bulk completing on mbarriers, as the mat-vec kernel's weight rings
// do) as a function of the copy size, the number of rings per CTA, who issues the copies (every
// consumer warp for itself, or one producer warp for all) and how the copies are dealt to the warps,
// next to plain 128-bit loads. One CTA per SM, nothing is computed: consumers wait for a stage and
// hand it back. Build: python -m jitllm_b200.build --microbench; run: jitllm_b200/lib/bulk_copy_bench [GiB].
#include <cuda_runtime.h>
#include <cstdio>
#include <cstdlib>
#include <cstdint>
#include <vector>
#define CK(x) do { cudaError_t e_ = (x); if (e_ != cudaSuccess) { printf("CUDA error %s at %d\n", cudaGetErrorString(e_), __LINE__); exit(1);} } while (0)

__device__ __forceinline__ uint32_t smem_u32(const void *p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) { asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count)); }
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) { asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory"); }
__device__ __forceinline__ void mbar_arrive(uint32_t bar) { asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory"); }
__device__ __forceinline__ bool mbar_try(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile("{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n\tselp.u32 %0, 1, 0, p;\n\t}" : "=r"(ok) : "r"(bar), "r"(parity), "r"(20000u) : "memory");
    return ok != 0;
}
__device__ __forceinline__ bool mbar_test(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile("{\n\t.reg .pred p;\n\tmbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}" : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
    return ok != 0;
}
__device__ __forceinline__ bool wait_b(uint32_t bar, uint32_t parity) { for (uint32_t i = 0; i < (1u << 16); ++i) if (mbar_try(bar, parity)) return true; return false; }
__device__ __forceinline__ void bulk(uint32_t dst, const void *src, uint32_t bytes, uint32_t bar, uint64_t pol, int hint) {
    if (hint)
        asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes.L2::cache_hint [%0], [%1], %2, [%3], %4;" ::"r"(dst), "l"(src), "r"(bytes), "r"(bar), "l"(pol) : "memory");
    else
        asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(dst), "l"(src), "r"(bytes), "r"(bar) : "memory");
}

// mode 0: every consumer warp's lane 0 issues its own copies. mode 1: a producer warp (last warp) feeds all rings.
// layout 0: copy i belongs to warp (w * grid + cta) round-robin over the grid. layout 1: each warp a contiguous range.
__global__ void __launch_bounds__(544, 1) stream_kernel(const uint8_t *src, long long ncopies, int cb, int depth, int nw, int mode, int layout, int hint, int touch, unsigned *sink, int *err) {
    extern __shared__ __align__(128) uint8_t smem[];
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const uint32_t bars = smem_u32(smem);              // full[nw][depth], empty[nw][depth]
    const uint32_t ring = bars + 4096;
    if (tid == 0) {
        for (int i = 0; i < nw * depth; ++i) { mbar_init(bars + i * 8, 1); mbar_init(bars + 2048 + i * 8, 1); }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    __syncthreads();
    uint64_t pol;
    asm volatile("createpolicy.fractional.L2::evict_first.b64 %0, 1.0;" : "=l"(pol));
    const long long total_warps = (long long)nw * gridDim.x;
    auto first = [&](int w) -> long long { return layout == 0 ? (long long)w * gridDim.x + blockIdx.x : ((long long)blockIdx.x * nw + w) * ((ncopies + total_warps - 1) / total_warps); };
    auto count = [&](int w) -> long long {
        if (layout == 0) { long long f = (long long)w * gridDim.x + blockIdx.x; return f < ncopies ? (ncopies - f - 1) / total_warps + 1 : 0; }
        long long per = (ncopies + total_warps - 1) / total_warps, f = ((long long)blockIdx.x * nw + w) * per;
        return f >= ncopies ? 0 : (f + per <= ncopies ? per : ncopies - f);
    };
    const long long stride = layout == 0 ? total_warps : 1;
    if (mode == 1 && warp == nw) {
        // producer warp: lane l feeds ring l (nw <= 32)
        const int w = lane;
        long long n = w < nw ? count(w) : 0, f = w < nw ? first(w) : 0, j = 0;
        int slot = 0, use = 0; unsigned idle = 0;
        while (true) {
            bool want = j < n;
            if (!__any_sync(0xffffffffu, want)) break;
            bool can = false;
            if (want) can = use == 0 || mbar_test(bars + 2048 + (w * depth + slot) * 8, (use - 1) & 1);
            if (can) {
                asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
                mbar_expect_tx(bars + (w * depth + slot) * 8, cb);
                bulk(ring + (w * depth + slot) * cb, src + (f + j * stride) * cb, cb, bars + (w * depth + slot) * 8, pol, hint);
                ++j; if (++slot == depth) { slot = 0; ++use; }
            }
            if (__any_sync(0xffffffffu, can)) idle = 0; else { if (++idle > (1u << 22)) { *err = 1; break; } __nanosleep(100); }
        }
        return;
    }
    if (warp >= nw) return;
    const long long n = count(warp), f = first(warp);
    const uint32_t myfull = bars + warp * depth * 8, myempty = bars + 2048 + warp * depth * 8, myring = ring + warp * depth * cb;
    unsigned acc = 0;
    if (mode == 0) {
        long long issued = 0;
        if (lane == 0) for (; issued < depth && issued < n; ++issued) { mbar_expect_tx(myfull + issued * 8, cb); bulk(myring + issued * cb, src + (f + issued * stride) * cb, cb, myfull + issued * 8, pol, hint); }
        int slot = 0; uint32_t par = 0;
        for (long long j = 0; j < n; ++j) {
            if (!wait_b(myfull + slot * 8, par)) { *err = 2; break; }
            if (touch) { for (int o = lane * 16; o < cb; o += 512) { uint4 v; asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(myring + slot * cb + o)); acc ^= v.x ^ v.y ^ v.z ^ v.w; } }
            __syncwarp();
            if (lane == 0 && issued < n) { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); mbar_expect_tx(myfull + slot * 8, cb); bulk(myring + slot * cb, src + (f + issued * stride) * cb, cb, myfull + slot * 8, pol, hint); ++issued; }
            if (++slot == depth) { slot = 0; par ^= 1; }
        }
    } else {
        int slot = 0; uint32_t par = 0;
        for (long long j = 0; j < n; ++j) {
            if (!wait_b(myfull + slot * 8, par)) { *err = 2; break; }
            if (touch) { for (int o = lane * 16; o < cb; o += 512) { uint4 v; asm volatile("ld.shared.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "r"(myring + slot * cb + o)); acc ^= v.x ^ v.y ^ v.z ^ v.w; } }
            __syncwarp();
            if (lane == 0) mbar_arrive(myempty + slot * 8);
            if (++slot == depth) { slot = 0; par ^= 1; }
        }
    }
    if (acc == 0x12345678u) *sink = acc;
}

// plain loads: each thread 16 B, U loads in flight, grid-stride
template <int U>
__global__ void __launch_bounds__(512) ldg_kernel(const uint4 *src, long long n16, unsigned *sink) {
    unsigned acc = 0;
    const long long stride = (long long)gridDim.x * blockDim.x;
    long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    for (; i + (U - 1) * stride < n16; i += U * stride) {
        uint4 v[U];
#pragma unroll
        for (int u = 0; u < U; ++u) v[u] = __ldcs(src + i + u * stride);
#pragma unroll
        for (int u = 0; u < U; ++u) acc ^= v[u].x ^ v[u].y ^ v[u].z ^ v[u].w;
    }
    for (; i < n16; i += stride) { uint4 v = __ldcs(src + i); acc ^= v.x ^ v.y; }
    if (acc == 0x12345678u) *sink = acc;
}

int main(int argc, char **argv) {
    const size_t bytes = (size_t)(argc > 1 ? atof(argv[1]) : 2.0) * (1u << 30);
    uint8_t *buf; unsigned *sink; int *err;
    CK(cudaMalloc(&buf, bytes)); CK(cudaMalloc(&sink, 4)); CK(cudaMalloc(&err, 4));
    CK(cudaMemset(buf, 1, bytes)); CK(cudaMemset(err, 0, 4));
    cudaEvent_t e0, e1; CK(cudaEventCreate(&e0)); CK(cudaEventCreate(&e1));
    int sms = 0; CK(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, 0));
    CK(cudaFuncSetAttribute(stream_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024));
    auto time_it = [&](auto launch, const char *name) {
        float best = 1e9;
        for (int r = 0; r < 4; ++r) { CK(cudaEventRecord(e0)); launch(); CK(cudaEventRecord(e1)); CK(cudaEventSynchronize(e1)); float ms; CK(cudaEventElapsedTime(&ms, e0, e1)); if (r > 0 && ms < best) best = ms; }
        CK(cudaGetLastError());
        int h = 0; CK(cudaMemcpy(&h, err, 4, cudaMemcpyDeviceToHost));
        printf("%-60s %8.1f GB/s  (%.3f ms)%s\n", name, bytes / best / 1e6, best, h ? "  ERR" : ""); fflush(stdout);
    };
    char name[256];
    for (int mult : {4, 8}) { snprintf(name, sizeof name, "ldg U=8 grid=%dx148 x512", mult); time_it([&] { ldg_kernel<8><<<sms * mult, 512>>>((const uint4 *)buf, bytes / 16, sink); }, name); }
    snprintf(name, sizeof name, "ldg U=4 grid=4x148 x512"); time_it([&] { ldg_kernel<4><<<sms * 4, 512>>>((const uint4 *)buf, bytes / 16, sink); }, name);
    struct Cfg { int cb, nw, mode, layout, hint, touch; };
    std::vector<Cfg> cfgs;
    for (int cb : {1152, 2304, 4608, 9216, 18432}) for (int mode : {0, 1}) for (int layout : {0, 1}) cfgs.push_back({cb, 16, mode, layout, 1, 0});
    cfgs.push_back({1152, 16, 0, 0, 0, 0}); cfgs.push_back({4608, 16, 0, 0, 0, 0}); cfgs.push_back({4608, 16, 1, 1, 0, 0});
    cfgs.push_back({1152, 16, 0, 0, 1, 1}); cfgs.push_back({4608, 16, 0, 0, 1, 1}); cfgs.push_back({4608, 16, 1, 1, 1, 1});
    cfgs.push_back({4608, 8, 0, 0, 1, 0}); cfgs.push_back({4608, 8, 1, 1, 1, 0}); cfgs.push_back({9216, 4, 0, 0, 1, 0}); cfgs.push_back({9216, 4, 1, 1, 1, 0});
    cfgs.push_back({1152, 32, 0, 0, 1, 0}); cfgs.push_back({2304, 32, 0, 0, 1, 0});
    for (auto c : cfgs) {
        int depth = (int)((200 * 1024) / ((size_t)c.nw * c.cb)); if (depth > 16) depth = 16; if (depth < 2) continue;
        if (c.nw * depth > 256) depth = 256 / c.nw;
        size_t smem = 4096 + (size_t)c.nw * depth * c.cb;
        long long ncopies = bytes / c.cb;
        int threads = (c.nw + (c.mode == 1 ? 1 : 0)) * 32;
        snprintf(name, sizeof name, "bulk cb=%5d warps=%2d depth=%2d %s %s hint=%d touch=%d", c.cb, c.nw, depth, c.mode ? "producer-warp" : "self-issue   ", c.layout ? "blocked    " : "interleaved", c.hint, c.touch);
        time_it([&] { stream_kernel<<<sms, threads, smem>>>(buf, ncopies, c.cb, depth, c.nw, c.mode, c.layout, c.hint, c.touch, sink, err); }, name);
    }
    return 0;
}
