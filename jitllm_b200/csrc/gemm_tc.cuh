// Tensor-core (tcgen05) quantised matrix-matrix product: interface.
#pragma once

#include "common.cuh"

namespace jl {

// Opaque 128-byte TMA descriptor of one weight matrix (a CUtensorMap): rows x row-bytes as 32-bit
// words, fetched in boxes of 128 rows x 256 columns. Built once per matrix by gemm_make_tensor_map.
struct alignas(64) GemmTensorMap {
    unsigned char bytes[128];
};
cudaError_t gemm_make_tensor_map(GemmTensorMap *out, const void *w_dev, int type, int64_t rows, int64_t cols);
// TMA descriptor of a pre-split activation buffer: binary16 [2 * row_cap][cols] (the hi rows, then
// the lo rows), fetched in swizzled boxes of nt rows x 64 columns; nt is 16, 32, 64 or 128.
cudaError_t gemm_make_activation_map(GemmTensorMap *out, const void *x16_dev, int64_t row_cap, int64_t cols, int nt);
int gemm_token_tile(int n);  // the nt the kernel will use for n rows

struct GemmSeg {
    const uint8_t *w;  // device, GGUF block layout, rows x cols
    const GemmTensorMap *tmap;  // host pointer, copied into the launch parameters
    float *y;          // device, n x rows
    const float *res;  // nullable: y = res + W.x (may alias y)
    int rows;
};

// Up to three matrices that share the input (Q/K/V, gate/up) go in one launch.
struct GemmArgs {
    GemmSeg seg[3];
    int nseg;
    int type;        // kQ8_0 / kQ4_0 / kQ4_K
    int cols;        // a multiple of 256
    const float *x;  // device, n x cols (used when xmap is NULL: converted inside the kernel)
    const GemmTensorMap *xmap;  // host pointer or NULL: pre-split activations for this launch's token tile
    int x_lo_row;    // first row of the lo half in that buffer (its row_cap)
    int n;
    int *status;     // device status word
    // Split-K workspace (nullable: then every CTA walks the whole row): partial tiles
    // [split][n][total rows] and one arrival counter per output tile, zero between launches.
    float *scratch;
    size_t scratch_floats;
    unsigned *counters;
    int counters_len;
    int sm_count;
    // Launch with the programmatic-dependent-launch attribute: the kernel's preamble and the first
    // weight copies (weights depend on no kernel) run while the kernel before it drains; everything
    // that reads activations or writes results waits for that kernel first.
    bool programmatic;
};

// Sets the shared-memory attribute of every instantiation (call once, outside stream capture).
cudaError_t gemm_tc_configure();
cudaError_t gemm_tc_launch(const GemmArgs &args, cudaStream_t stream);
cudaError_t gemm_trace_bind(unsigned long long *buf, unsigned cap, int mode);

}  // namespace jl
