// Matrix-vector product for Q4_1, Q5_K and Q6_K weights (the stand-alone operator; see gemv_extra.cu).
#pragma once

#include "formats.cuh"

namespace jl {

// The activation row is staged in shared memory: at most this many columns.
constexpr int kGemvExtraMaxCols = 49152;

// Sets the dynamic shared memory attribute of every instantiation; once per process per device.
cudaError_t gemv_extra_configure();
// y[b][r] = sum_c W[r][c] * x[b][c] for b < n; w in GGUF block layout (rows x cols, 256-byte aligned), x and y
// 16-byte aligned device pointers, cols a multiple of 256.
cudaError_t gemv_extra_launch(int type, const uint8_t *w, const float *x, float *y, int rows, int cols, int n, int sm_count,
                              cudaStream_t stream);

}  // namespace jl
