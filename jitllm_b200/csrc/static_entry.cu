// Allocation-free entry point: quantised matrix-vector product with the greedy arg-max folded in,
// using scratch memory that is part of the library image instead of memory obtained at run time.
//
// Who needs this: callers that must not (or cannot) allocate device memory when they call -- a
// serving loop whose memory was carved up once at start-up and which treats any later cudaMalloc
// as a fault, code running between cudaStreamBeginCapture and EndCapture (allocation is not
// allowed there), or a host that hands this library pre-allocated buffers from its own pool and
// expects it to stay inside them. The caller still passes every input and output; only the
// kernel's cross-CTA scratch (per-CTA partial maxima, their indices and an arrival counter) comes
// from the file-scope array below.
#include "../../include/jitllm_b200.h"

#include <cstdio>
#include <mutex>
#include <string>

#include "gemv.cuh"

using namespace jl;

namespace {

// Scratch for at most kStaticMaxCtas CTAs: value + index per CTA, then the counter and a status
// word. 8 KiB + 256 B per GPU that loads the library, held until the process exits.
constexpr int kStaticMaxCtas = 1024;
constexpr size_t kStaticScratchBytes = size_t(kStaticMaxCtas) * 8 + 256;
static __device__ __align__(256) unsigned char g_static_scratch[kStaticScratchBytes];

constexpr int kMaxDevices = 64;
std::mutex g_mu;
unsigned char *g_scratch_addr[kMaxDevices] = {};  // device address of the array, per device
thread_local std::string g_static_error;

int static_fail(int code, const char *fmt, const char *detail) {
    char buf[512];
    snprintf(buf, sizeof buf, fmt, detail);
    g_static_error = buf;
    return code;
}

}  // namespace

extern "C" {

const char *jl_static_last_error(void) { return g_static_error.c_str(); }

int32_t jl_gemv_argmax_static(int32_t ggml_type, int64_t rows, int64_t cols, const void *w_dev,
                              const float *x_dev, const float *norm_w_dev, float rms_eps, float *y_dev,
                              int32_t *token_dev, void *stream) {
    if (!w_dev || !x_dev || !y_dev || !token_dev)
        return static_fail(JL_ERR_INVALID, "GPUL-CFG-002: %s", "w_dev, x_dev, y_dev and token_dev must not be NULL");
    if (!is_quant(ggml_type))
        return static_fail(JL_ERR_UNSUPPORTED, "GPUL-CFG-002: unsupported: %s", "GGML type (Q4_0, Q8_0, Q4_K only)");
    if (rows <= 0 || rows > INT32_MAX || cols <= 0 || cols % 256 != 0 || cols > INT32_MAX)
        return static_fail(JL_ERR_INVALID, "GPUL-CFG-002: %s",
                           "rows must be in 1..2^31-1 and cols a positive multiple of 256");
    // The kernel fetches weights with 16-byte bulk copies and the vectors with 16-byte loads; a
    // pointer that breaks that would fault on the device, so it is refused here, before any launch.
    if (reinterpret_cast<uintptr_t>(w_dev) % 16 != 0 || reinterpret_cast<uintptr_t>(x_dev) % 16 != 0 ||
        reinterpret_cast<uintptr_t>(norm_w_dev) % 16 != 0)
        return static_fail(JL_ERR_INVALID, "GPUL-CFG-002: %s", "w_dev, x_dev and norm_w_dev must be 16-byte aligned");
    if (reinterpret_cast<uintptr_t>(y_dev) % 4 != 0 || reinterpret_cast<uintptr_t>(token_dev) % 4 != 0)
        return static_fail(JL_ERR_INVALID, "GPUL-CFG-002: %s", "y_dev and token_dev must be 4-byte aligned");
    int device = -1;
    cudaError_t e = cudaGetDevice(&device);
    if (e != cudaSuccess || device < 0)
        return static_fail(JL_ERR_CUDA, "CUDA: no current device (%s)", cudaGetErrorString(e));
    if (device >= kMaxDevices)
        return static_fail(JL_ERR_UNSUPPORTED, "GPUL-CFG-002: unsupported: %s", "device ordinal beyond 63");
    unsigned char *scratch = nullptr;
    {
        // Set-up, once per device, with that device current: the array's name is only a host-side
        // stand-in; the address a kernel can use has to be asked for.
        std::lock_guard<std::mutex> lock(g_mu);
        if (g_scratch_addr[device] == nullptr) {
            void *p = nullptr;
            e = cudaGetSymbolAddress(&p, g_static_scratch);
            if (e != cudaSuccess)
                return static_fail(JL_ERR_CUDA, "CUDA: cudaGetSymbolAddress failed: %s", cudaGetErrorString(e));
            e = gemv_configure();
            if (e != cudaSuccess)
                return static_fail(JL_ERR_CUDA, "CUDA: kernel set-up failed: %s", cudaGetErrorString(e));
            g_scratch_addr[device] = static_cast<unsigned char *>(p);
        }
        scratch = g_scratch_addr[device];
    }
    int sm_count = 0;
    e = cudaDeviceGetAttribute(&sm_count, cudaDevAttrMultiProcessorCount, device);
    if (e != cudaSuccess) return static_fail(JL_ERR_CUDA, "CUDA: %s", cudaGetErrorString(e));
    GemvPlan plan;
    if (!gemv_plan(ggml_type, int(cols), int(rows), kGemvPlain, sm_count, &plan))
        return static_fail(JL_ERR_UNSUPPORTED, "GPUL-CFG-002: unsupported: %s",
                           "no launch plan for this many columns (shared memory)");
    if (plan.grid > kStaticMaxCtas)
        return static_fail(JL_ERR_UNSUPPORTED, "GPUL-CFG-002: unsupported: %s",
                           "launch needs more CTAs than the static scratch holds (1024)");
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    // Layout: [0, 4N) values, [4N, 8N) indices, then counter and status. The counter and status
    // must start at zero; the array keeps whatever the previous call left.
    float *vals = reinterpret_cast<float *>(scratch);
    int *idxs = reinterpret_cast<int *>(scratch + size_t(kStaticMaxCtas) * 4);
    unsigned *counter = reinterpret_cast<unsigned *>(scratch + size_t(kStaticMaxCtas) * 8);
    int *status = reinterpret_cast<int *>(scratch + size_t(kStaticMaxCtas) * 8 + 128);
    e = cudaMemsetAsync(scratch + size_t(kStaticMaxCtas) * 8, 0, 256, s);
    if (e != cudaSuccess) return static_fail(JL_ERR_CUDA, "CUDA: %s", cudaGetErrorString(e));
    GemvArgs a = {};
    a.nseg = 1;
    a.seg[0] = {static_cast<const uint8_t *>(w_dev), y_dev, nullptr, int(rows)};
    a.cols = int(cols);
    a.type = ggml_type;
    a.mode = kGemvPlain;
    a.x = x_dev;
    a.norm_w = norm_w_dev;
    a.eps = rms_eps;
    a.argmax_val = vals;
    a.argmax_idx = idxs;
    a.argmax_count = counter;
    a.out_token = token_dev;
    a.status = status;
    e = gemv_launch(a, plan, s, false);
    if (e != cudaSuccess)
        return static_fail(JL_ERR_CUDA, "CUDA: launch failed: %s", cudaGetErrorString(e));
    return JL_OK;
}

int32_t jl_static_status(void *stream) {
    int device = -1;
    cudaError_t e = cudaGetDevice(&device);
    if (e != cudaSuccess || device < 0 || device >= kMaxDevices)
        return static_fail(JL_ERR_CUDA, "CUDA: no current device (%s)", cudaGetErrorString(e));
    unsigned char *scratch = nullptr;
    {
        std::lock_guard<std::mutex> lock(g_mu);
        scratch = g_scratch_addr[device];
    }
    if (scratch == nullptr)
        return static_fail(JL_ERR_STATE, "GPUL-CFG-002: %s", "jl_gemv_argmax_static has not run on this device");
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    int status = 0;
    e = cudaMemcpyAsync(&status, scratch + size_t(kStaticMaxCtas) * 8 + 128, sizeof status, cudaMemcpyDeviceToHost, s);
    if (e == cudaSuccess) e = cudaStreamSynchronize(s);
    if (e != cudaSuccess) return static_fail(JL_ERR_CUDA, "CUDA: %s", cudaGetErrorString(e));
    if (status == kDevTimeout)
        return static_fail(JL_ERR_TIMEOUT, "GPUL-RUN-001: %s",
                           "the kernel gave up waiting for an asynchronous copy; y_dev and token_dev are not valid");
    return JL_OK;
}

}  // extern "C"
