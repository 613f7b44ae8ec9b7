// Per-layer kernels around the matrix products: embedding lookup, RoPE + KV page append + paged
// decode attention, block dequantisation.
#pragma once

#include "formats.cuh"

namespace jl {

// Geometry of the paged fp16 KV store (backend/tornado/kernels/KvBlockAddress.java:59-71 of the
// reference): element offset = table[slot*blocks_per_slot + pos/block_tokens] * block_stride
//   + layer * block_tokens * kv_dim + (pos % block_tokens) * kv_dim + c, 64-bit here.
struct KvGeom {
    __half *kpool, *vpool;
    const int32_t *block_table;
    int blocks_per_slot, block_tokens, layers, kv_dim;
};

struct AttnArgs {
    const float *q, *k, *v;  // [width][dim], [width][kv_dim]: projections before RoPE
    float *out;              // [width][dim]
    // Optional: the same rows as binary16 hi and lo parts (out = hi + lo) in the tensor-core path's operand
    // order (pairs (k0, k2), (k1, k3) inside every four), [width][dim] each, for the output projection.
    void *out_hi, *out_lo;
    const float *rope_cos, *rope_sin;  // [ctx][head_dim/2]
    const int32_t *positions, *slots;
    const uint8_t *active;
    KvGeom kv;
    int layer, heads, kv_heads, head_dim, dim;
    int nsplit;  // from attention_splits()
    int append;  // 1: the CTA owning the new position rotates k and appends k,v; 0: pages already hold it
    float *partial;     // scratch [width][heads][nsplit][head_dim + 2]
    unsigned *counters; // scratch [width][kv_heads], zero between launches
};

cudaError_t attention_configure();
cudaError_t attention_launch(const AttnArgs &a, int width, cudaStream_t stream, bool programmatic);
// The rows of one prompt chunk (all of one sequence, their keys already in the pages; append = 0): tiles of
// query rows against tiles of keys on the tensor cores instead of one walk over the pages per row.
cudaError_t attention_prompt_launch(const AttnArgs &a, int n, cudaStream_t stream, bool programmatic);
// A decode batch of at least four rows (one sequence per row, append = 1): one CTA per (row, KV head) with the
// query heads as the rows of a tensor-core tile; rotates and appends the step's own key and value itself.
cudaError_t attention_batch_launch(const AttnArgs &a, int width, cudaStream_t stream, bool programmatic);
size_t attention_partial_floats(int width, int heads, int nsplit, int head_dim);
// Key-range splits per (row, KV head) for a launch of `width` rows: cluster size times clusters.
int attention_splits(int sm_count, int width, int kv_heads);

// x[row] = getFloat of embedding row tokens[row] (inference/op/CpuOperations.java:30-32).
cudaError_t embedding_launch(int type, const uint8_t *table, const int32_t *tokens,
                             const uint8_t *active, float *x, int dim, int width,
                             cudaStream_t stream, bool programmatic);

// out[i] = getFloat(i), element-exact.
// Copies nblocks Q6_K super-blocks into slots of kQ6_KPadded bytes (see formats.cuh).
cudaError_t pad_q6k_launch(const uint8_t *src, uint8_t *dst, size_t nblocks, cudaStream_t stream);
cudaError_t dequant_launch(int type, const uint8_t *blocks, int64_t n, float *out,
                           cudaStream_t stream);

// After a step: feeds each active row's sampled token back as its next input, advances its
// position and appends the token to history[step][row] (step counter kept on the device).
cudaError_t advance_launch(int32_t *tokens, int32_t *positions, const int32_t *sampled,
                           const uint8_t *active, int32_t *history, int32_t *step_counter, int width,
                           cudaStream_t stream, bool programmatic);

// Row-wise operators for the matrix-matrix (prefill / wide batch) path.
// out[r] = w * (rsqrt(mean(x[r]^2) + eps) * x[r])   (inference/op/CpuOperations.java:55-73)
// hi / lo: optional binary16 split of the result (x = hi + lo), contiguous [n][dim] each.
cudaError_t rmsnorm_rows_launch(const float *x, const float *w, float eps, float *out, int dim, int n,
                                const uint8_t *active, cudaStream_t stream, void *hi = nullptr, void *lo = nullptr,
                                bool programmatic = false);
// g[r] = silu(g[r]) * u[r]                          (inference/op/CpuOperations.java:255-260)
// hi / lo: optional binary16 split of the result (x = hi + lo), contiguous [n][hidden] each.
cudaError_t swiglu_rows_launch(float *g, const float *u, int hidden, int n, cudaStream_t stream, void *hi = nullptr,
                               void *lo = nullptr, bool programmatic = false);
// RoPE on k, then k and v rounded to fp16 into the page of (slot, position) of every row
// (inference/op/CpuOperations.java:94-147).
cudaError_t kv_append_launch(const float *k, const float *v, const float *rope_cos, const float *rope_sin,
                             const int32_t *positions, const int32_t *slots, const uint8_t *active,
                             KvGeom kv, int layer, int head_dim, int n, cudaStream_t stream, bool programmatic = false);
// out[r] = first index of the maximum of logits[r]  (inference/Logits.java:49-60)
cudaError_t argmax_rows_launch(const float *logits, int vocab, int n, const uint8_t *active, int32_t *out,
                               cudaStream_t stream, bool programmatic = false);

// x[i] += y[i]
cudaError_t add_rows_launch(float *x, const float *y, size_t total, cudaStream_t stream, bool programmatic = false);
// x = hi + lo with hi, lo binary16 (22 significant bits): the tensor-core path's activation format.
cudaError_t split_rows_launch(const float *x, size_t total, void *hi, void *lo, cudaStream_t stream,
                              bool programmatic = false);
// (programmatic: launch with the programmatic-dependent-launch attribute; the row kernels always wait for
// the kernel before them and release the one after them at their start.)
// best[r] = (logits[r][idx[r]], idx[r] + index_offset) for the n rows of this GPU's vocabulary shard.
cudaError_t tp_pack_best_launch(const float *logits, const int32_t *idx, int l_vocab, int index_offset, int n,
                                float *best, cudaStream_t stream);
// out[r] = index of the best of the gathered pairs all[rank][r], lowest index on ties.
cudaError_t tp_pick_best_launch(const float *all, int ranks, int n, const uint8_t *active, int32_t *out,
                                cudaStream_t stream);

cudaError_t ops_trace_bind(unsigned long long *buf, unsigned cap, int mode);

cudaError_t fill_launch(uint32_t *buf, size_t words, uint32_t value, cudaStream_t stream);

}  // namespace jl
