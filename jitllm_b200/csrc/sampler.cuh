// Device-side temperature / top-p sampling of the rows of logits a decode step left in device memory.
#pragma once
#include <cuda_runtime.h>

#include <cstdint>

namespace jl {

// out[r] = the token the reference's sampler chain (inference/sampler/Sampler.java:63-110) picks from row r of
// logits[width][vocab] for temperature > 0, nucleus threshold topp (outside (0,1): plain categorical sampling)
// and the uniform random number uniforms[r] in [0,1); -1 for rows whose active flag is 0. The rows are
// `greedy` (nullable; may alias out): the index of each row's maximum, which spares a pass. The rows are
// overwritten with exp(score - max), as the reference overwrites its logits. A cluster of eight CTAs per row.
// Sets the kernel's shared-memory attribute (call once per device, outside stream capture).
cudaError_t sample_rows_configure();
cudaError_t sample_rows_launch(float *logits, int vocab, int width, const uint8_t *active, float temperature, float topp,
                               const float *uniforms, const int32_t *greedy, int32_t *out, cudaStream_t stream);

}  // namespace jl
