/*
 * CPU oracle for the jitLLM Llama hot path -- TEST INFRASTRUCTURE, NOT PRODUCT CODE.
 *
 * A plain-C restatement of jitLLM's CPU ("numerical reference") path, used only as the checker in
 * tests, the smoke check and the CPU-baseline leg of the benchmark. The CUDA library never calls
 * it and has no CPU fallback.
 *
 * Parity status: PINNED against the reference's own known-answer tests (Q4_0 specification bytes,
 * fp16 rounding known answers, the documented KV page-address formula, ArrayHalfFloatTensor
 * values) and against an independent numpy restatement on java.util.Random-seeded blocks; the
 * reference JVM itself cannot run in this environment (no JDK), so end-to-end logits rest on this
 * restatement.
 *
 * Every function cites the reference file:line it follows. Paths are relative to
 * src/main/java/org/beehive/jitllm/ in the reference project.
 *
 * Java semantics reproduced: IEEE binary32 with no FMA contraction (build with
 * -ffp-contract=off) except the explicit FloatVector.fma in the vector dot products; (float)
 * narrowing of double sqrt/exp/cos/sin/pow; Float.floatToFloat16 = round-to-nearest-even with
 * subnormals.
 */
#ifndef JL_ORACLE_H
#define JL_ORACLE_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* GGML type ids, format/GGMLType.java:7,13,18-20 (same numbering as the GGUF file format). */
enum { ORC_F32 = 0, ORC_F16 = 1, ORC_Q4_0 = 2, ORC_Q4_1 = 3, ORC_Q8_0 = 8, ORC_Q4_K = 12, ORC_Q5_K = 13, ORC_Q6_K = 14 };

/* Summation mode of the quantised dot products, tensor/standard/FloatTensor.java:22-36:
 * 0 = scalar sequential (also what a 512-bit host gets), 128 / 256 = FloatVector lanes. */
void orc_set_vector_bits(int bits);
int orc_get_vector_bits(void);
void orc_set_threads(int n); /* 0 = all cores; Parallel.parallelFor uses the common pool */
int orc_get_threads(void);

/* Float.float16ToFloat / Float.floatToFloat16 (JDK 20+). */
float orc_f16_to_f32(uint16_t h);
uint16_t orc_f32_to_f16(float f);

/* Block geometry. */
size_t orc_row_bytes(int type, int64_t cols);

/* getFloat of element `index`: Q8_0FloatTensor.java:53-61, Q4_0FloatTensor.java:56-79,
 * Q4_KFloatTensor.java:68-122. */
float orc_get_float(int type, const void *data, int64_t index);
void orc_dequant(int type, const void *data, int64_t n, float *out);

/* FloatTensor.dot for one row (FloatTensor.java:110-121 and the per-format overrides). */
float orc_dot(int type, const void *data, int64_t this_offset, const float *x, int64_t size);
/* FloatTensor.matmul (FloatTensor.java:123-125): out[r] = dot(row r, x). */
void orc_matmul(int type, const void *w, const float *x, float *out, int rows, int cols);
/* Batch form (FloatTensor.java:127-140): n independent activation vectors, x[n][cols]. */
void orc_matmul_batch(int type, const void *w, const float *x, float *out, int rows, int cols,
                      int n);

/* inference/op/CpuOperations.java */
void orc_rmsnorm(float *out, const float *x, const float *weight, int size, float eps); /* :55-73 */
void orc_rope(float *q, float *k, const float *cr, const float *ci, int position, int dim,
              int kv_dim, int head_size);                                   /* :94-116 */
void orc_swiglu(float *gate, const float *up, int n);                      /* :255-260 */
int orc_argmax(const float *logits, int n); /* inference/Logits.java:49-60 */
/* model/loader/RopeFrequencies.java:14-54 with ropeScaling=false. */
void orc_rope_tables(int context_length, int head_size, double theta, float *cr, float *ci);
/* Attention over an fp16 cache [pos][kvDim] of one layer, CpuOperations.java:149-204. */
void orc_attention(const float *q, const uint16_t *kcache, const uint16_t *vcache, float *att,
                   float *out, int position, int heads, int kv_mul, int head_size, int kv_dim,
                   int context_length);

/* KV page addressing, backend/tornado/kernels/KvBlockAddress.java:59-71. */
int64_t orc_kv_offset(const int32_t *block_table, int slot, int pos, int layer, int kv_dim,
                      int block_size, int max_blocks_per_slot, int num_layers);

/* ---- whole model: backend/cpu/InferenceCore.java:72-141 ---- */
typedef struct {
    int dim, hidden, layers, heads, kv_heads, head_dim, vocab, ctx_len;
    float eps;
    float theta;
} orc_config;

typedef struct {
    int type;         /* ORC_* */
    const void *data; /* borrowed */
} orc_tensor;

typedef struct orc_model orc_model;
typedef struct orc_state orc_state;

orc_model *orc_model_create(const orc_config *cfg);
void orc_model_free(orc_model *m);
/* role ids are those of include/jitllm_b200.h (JL_ROLE_*); layer = -1 for global tensors. */
int orc_model_set_tensor(orc_model *m, int role, int layer, int type, const void *data);
/* tables as Java's RopeFrequencies would compute them (done in orc_model_create); readable so
 * that both sides of a parity test consume the same table bits. */
/* Replaces the tables (the reference's forward pass reads whatever tables its weights hold). */
void orc_model_set_rope(orc_model *m, const float *cr, const float *ci);
const float *orc_model_rope_cos(const orc_model *m);
const float *orc_model_rope_sin(const orc_model *m);

orc_state *orc_state_create(const orc_model *m);
void orc_state_free(orc_state *s);
/* forwardJava: returns the logits buffer (vocab floats) owned by the state. */
const float *orc_forward(const orc_model *m, orc_state *s, int token, int position);
/* Same without final norm / logits: one row of batchForwardJavaPrefill
 * (backend/cpu/InferenceCoreBatchPrefillDecode.java:43-192), which is numerically the per-token
 * layer stack. */
void orc_forward_no_logits(const orc_model *m, orc_state *s, int token, int position);
/* Intermediate buffers for per-op parity checks. */
const float *orc_state_buffer(const orc_state *s, const char *name);
const uint16_t *orc_state_kcache(const orc_state *s, int layer);
const uint16_t *orc_state_vcache(const orc_state *s, int layer);

/* The sampler chain of inference/sampler/Sampler.java:63-110 for one row of logits (modified in place, as
 * the reference does): temperature 0 = arg-max (first index of the maximum, inference/Logits.java:49-60);
 * otherwise scores /= temperature, softmaxInPlace (tensor/standard/FloatTensor.java:248-256: max, (float)
 * Math.exp(f - max), sequential fp32 sum, divide), then CategoricalSampler.sampleToken
 * (CategoricalSampler.java:13-25) when topp is outside (0,1), else ToppSampler.sampleToken
 * (ToppSampler.java:46-103). `u` is what rng.nextFloat(1f) returned for this call: the random generator
 * itself (RandomGeneratorFactory.getDefault()) stays on the caller's side.
 * Order among equal probabilities: the reference's heap leaves it to its sift order; here ties are taken in
 * index order (lowest first). When `margin` is not NULL it receives how far, relative to the nucleus mass (or to
 * 1 for the categorical sampler), the scaled random number was from the nearest boundary of the cumulative
 * distribution: a sampler that sums in another order may differ only when this is within rounding. */
int orc_sample(float *logits, int n, float temperature, float topp, float u, float *margin);

#ifdef __cplusplus
}
#endif
#endif
