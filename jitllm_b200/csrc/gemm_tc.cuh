// Tensor-core (tcgen05) quantised matrix-matrix product: interface.
#pragma once

#include "common.cuh"

namespace jl {

struct GemmArgs {
    const uint8_t *w;  // device, GGUF block layout, rows x cols
    int type;          // kQ8_0 / kQ4_0 / kQ4_K
    int rows, cols;    // cols a multiple of 256
    const float *x;    // device, n x cols
    int n;
    float *y;          // device, n x rows
    const float *res;  // nullable: y = res + W.x (may alias y)
    int *status;       // device status word
};

// Sets the shared-memory attribute of every instantiation (call once, outside stream capture).
cudaError_t gemm_tc_configure();
cudaError_t gemm_tc_launch(const GemmArgs &args, cudaStream_t stream);

}  // namespace jl
