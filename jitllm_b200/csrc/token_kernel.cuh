// Persistent per-token decode kernel for a single sequence: interface.
#pragma once

#include "gemv.cuh"
#include "ops.cuh"

namespace jl {

// Device pointers of one transformer layer (all matrices share one quantisation type).
struct TokLayer {
    const uint8_t *wq, *wk, *wv, *wo, *w1, *w3, *w2;
    const float *attn_norm, *ffn_norm;
};

struct TokArgs {
    const TokLayer *layers;  // device array, n_layers entries
    int n_layers;
    int with_logits;  // 0: stop after the last layer (prompt ingestion)
    int dim, hidden, kv_dim, vocab;
    float eps;
    // embedding and output
    const uint8_t *emb;
    int emb_type;
    const uint8_t *wcls;
    const float *out_norm;
    // per-step state (row 0 of the engine's step buffers)
    int32_t *tokens;
    int32_t *positions;
    const int32_t *slots;
    int32_t *out_token;
    int32_t *history;
    int32_t *step_counter;
    int advance;
    float *x, *q, *k, *v, *xb, *hb, *logits;
    // attention
    KvGeom kv;
    const float *rope_cos, *rope_sin;
    int heads, kv_heads;
    float *partial;  // [heads][max_splits][head_dim + 2]
    int max_splits;
    // arg-max scratch, one entry per CTA
    float *amax_val;
    int *amax_idx;
    // grid barrier counter (zero at launch) and the device status word
    unsigned *barrier;
    int *status;
    // nullable: CTA 0 writes five globaltimer stamps per operator (start, staged, consumed,
    // reduced, past the barrier); operators are numbered 1 + 6*layer + {0 qkv, 1 attention, 2 fold,
    // 3 output projection, 4 gate/up, 5 down}, 0 = embedding, last = vocabulary
    unsigned long long *profile;
};

// True when the persistent kernel can run this model (supported head geometry, shared memory
// large enough, per-CTA partial sums fit).
bool token_kernel_supported(int type, int head_dim, int group, int dim, int hidden, int kv_dim,
                            int vocab, int heads, int kv_heads, int n_layers, int sm_count);
cudaError_t token_kernel_configure();
int token_kernel_op_count(int n_layers);
// Cooperative launch, one CTA per SM.
cudaError_t token_kernel_launch(int type, int head_dim, int group, const TokArgs &args, int sm_count,
                                cudaStream_t stream);

}  // namespace jl
