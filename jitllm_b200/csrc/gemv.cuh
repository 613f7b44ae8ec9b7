// Decode-time quantised matrix-vector product: interface between the engine and gemv.cu.
#pragma once

#include "formats.cuh"

namespace jl {

// One weight matrix of a fused launch (Q, K and V share one launch; gate and up share one).
struct GemvSeg {
    const uint8_t *w;  // device, GGUF block layout, rows x cols
    float *y;          // device, rows
    const float *res;  // nullable: y[row] = res[row] + dot (may alias y)
    int rows;
};

enum GemvMode : int { kGemvPlain = 0, kGemvGateUp = 1 };

struct GemvArgs {
    GemvSeg seg[3];
    int nseg;
    int cols;  // multiple of 256
    int type;  // kQ8_0 / kQ4_0 / kQ4_K
    int mode;
    const float *x;       // cols floats
    const float *norm_w;  // nullable: y = W . (norm_w * (rsqrt(mean(x^2)+eps) * x))
    float eps;
    const uint8_t *active;  // nullable: a zero byte turns the whole launch into a no-op
    // Greedy argmax over the rows of seg[0] fused into the epilogue (nullable = off).
    float *argmax_val;       // gridDim.x partial maxima
    int *argmax_idx;         // gridDim.x partial indices
    unsigned *argmax_count;  // zero on entry, zero again on exit
    int *out_token;
    int *status;  // device status word, see common.cuh
    int debug;    // 0 normal; 1 = stream only (no arithmetic); 2 = arithmetic only (no copies)
};

struct GemvPlan {
    int rows_per_tile;  // 1, 2 or 4
    int stages;
    int grid;
    size_t smem_bytes;
};

// Chooses tile height, pipeline depth and shared-memory size for one launch shape.
bool gemv_plan(int type, int cols, int total_rows, int mode, int sm_count, GemvPlan *out);
// Sets the dynamic shared memory attribute of every instantiation; once per process per device.
cudaError_t gemv_configure();
cudaError_t gemv_launch(const GemvArgs &args, const GemvPlan &plan, cudaStream_t stream,
                        bool programmatic);

// Number of int8 digits an activation is split into (7 bits each) before the integer dot.
constexpr int kLimbs = 3;
constexpr float kLimbRange = 1040000.0f;  // |X| <= 63*2^14 + 63*2^7 + 63 stays in digit range

}  // namespace jl
