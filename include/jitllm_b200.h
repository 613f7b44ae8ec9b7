/*
 * jitllm_b200 -- C ABI of the B200 (sm_100a) CUDA library that stands in for jitLLM's TornadoVM
 * TaskGraph + kernel layer on the Llama decode / prefill hot path.
 *
 * Plain pointers and sizes only; every function returns a jl_status (0 = OK) and leaves a
 * human-readable message, prefixed with the reference's diagnostic code (GPUL-CFG-002,
 * GPUL-MEM-001, ...; runtime/diagnostics/DiagnosticCode.java:26-60), retrievable through
 * jl_last_error(). There is no CPU fallback: without a usable CUDA device jl_init fails.
 *
 * Ownership: the caller owns every host buffer (the mmapped GGUF slices, token arrays, output
 * arrays); the library copies what it needs and owns all device memory until jl_destroy. This is
 * the contract of lowering/InvocationBoundary.java:6-24 ("results copied out into session-owned
 * storage").
 *
 * Threading: one jl_ctx per model per GPU; calls on one context must be serialised by the
 * caller, as runtime/batch/BatchExecutor.java:17-18 and InvocationBoundary.java:13-21 already
 * require of the code this replaces.
 *
 * Reference paths below are relative to src/main/java/org/beehive/jitllm/.
 */
#ifndef JITLLM_B200_H
#define JITLLM_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef struct jl_ctx jl_ctx;
typedef struct jl_tensor jl_tensor;

typedef enum {
    JL_OK = 0,
    JL_ERR_INVALID = 1,     /* GPUL-CFG-002: bad argument / unsupported combination */
    JL_ERR_OOM = 2,         /* GPUL-MEM-001: device memory exhausted */
    JL_ERR_CUDA = 3,        /* a CUDA runtime call failed */
    JL_ERR_STATE = 4,       /* GPUL-LIFE-001: call out of order (no model, no KV store, closed) */
    JL_ERR_TIMEOUT = 5,     /* a bounded device-side wait gave up */
    JL_ERR_UNSUPPORTED = 6  /* GPUL-CFG-002: format or shape this build does not handle */
} jl_status;

/* GGML type ids as stored in GGUF (format/GGMLType.java:7-30). Q4_0, Q8_0 and Q4_K matrices run on the fused
 * single-row kernels and the tensor-core kernel. Q4_1, Q5_K and Q6_K, which mixed-precision files add for some
 * tensors, are decoded element-exactly and run on the same kernels (Q6_K from a second copy on the device whose
 * super-blocks are padded to 224 bytes). One GPU only. */
typedef enum {
    JL_F32 = 0, JL_F16 = 1, JL_Q4_0 = 2, JL_Q4_1 = 3, JL_Q8_0 = 8, JL_Q4_K = 12, JL_Q5_K = 13, JL_Q6_K = 14
} jl_ggml_type;

/* Tensor roles: the subset of runtime/tensor/TensorRole.java:17-59 a Llama file uses; this is
 * the key of TornadoWeights.tensor(role, layer) (inference/weights/tornado/TornadoWeights.java:95-109). */
typedef enum {
    JL_ROLE_TOKEN_EMBEDDING = 0,
    JL_ROLE_ATTENTION_NORM = 1,
    JL_ROLE_ATTENTION_QUERY = 2,
    JL_ROLE_ATTENTION_KEY = 3,
    JL_ROLE_ATTENTION_VALUE = 4,
    JL_ROLE_ATTENTION_OUTPUT = 5,
    JL_ROLE_FFN_NORM = 6,
    JL_ROLE_FFN_GATE = 7,
    JL_ROLE_FFN_UP = 8,
    JL_ROLE_FFN_DOWN = 9,
    JL_ROLE_OUTPUT_NORM = 10,
    JL_ROLE_OUTPUT = 11,
    JL_ROLE_COUNT = 12
} jl_tensor_role;

/* model/llama/LlamaConfiguration.java:5-16 plus the tensor-parallel placement of this GPU. */
typedef struct {
    int32_t dim, hidden, layers, heads, kv_heads, head_dim, vocab, ctx_len;
    float rms_eps;
    int32_t tied_embeddings; /* 1: no output.weight, logits use token_embd (AbstractModelLoader.java:255-266) */
    int32_t max_batch;       /* widest BatchSlots this context will be asked to decode */
    int32_t tp_rank, tp_size; /* 0,1 for a single GPU */
} jl_model_desc;

/* Counters for a MetricsSink adapter (runtime/metrics/MetricsSink.java;
 * backend/tornado/TornadoMetricsReporter.java:52-78). */
typedef struct {
    uint64_t decode_calls, prefill_calls, kernel_launches;
    uint64_t h2d_bytes, d2h_bytes;
    uint64_t weight_bytes, kv_bytes, workspace_bytes;
    float last_step_ms; /* device time of the last jl_decode / jl_prefill, CUDA events */
} jl_counters;

/* ---- lifecycle: replaces TornadoVMMasterPlan.initializeTornadoVMPlan / freeTornadoExecutionPlan
 * (backend/tornado/TornadoVMMasterPlan.java:59-83,131-180). */
int32_t jl_init(int32_t device_id, jl_ctx **out);
int32_t jl_destroy(jl_ctx *ctx);
/* Message of the last failing call on this context (ctx == NULL: last failing jl_init). */
const char *jl_last_error(jl_ctx *ctx);

/* ---- weights: replaces the device half of ModelLoader.loadTornadoTensorNative
 * (model/loader/ModelLoader.java:246-290). Bytes stay in GGUF block layout on the device. */
int32_t jl_model_create(jl_ctx *ctx, const jl_model_desc *desc);
int32_t jl_upload_tensor(jl_ctx *ctx, int32_t role, int32_t layer, int32_t ggml_type, int64_t rows,
                         int64_t cols, const void *host_bytes, size_t nbytes);
/* RoPE tables as computed by model/loader/RopeFrequencies.java:14-54, [ctx_len][head_dim/2]. */
int32_t jl_upload_rope(jl_ctx *ctx, const float *cos_table, const float *sin_table, int64_t n);
/* Checks that every tensor of every layer is present and builds the per-step launch plan;
 * replaces forceCopyInReadOnlyData + createExecutionPlan (TornadoVMMasterPlan.java:131-180). */
int32_t jl_model_finalize(jl_ctx *ctx);

/* ---- paged KV store: replaces backend/tornado/kv/TornadoKvStore.java behind
 * runtime/kv/KvStorageFactory.create(KvStorageRequest) (runtime/kv/KvStorageRequest.java:5-12).
 * One extra, never-leased scratch block is allocated for UNMAPPED (-1) table entries. */
int32_t jl_kv_create(jl_ctx *ctx, int32_t total_blocks, int32_t blocks_per_slot, int32_t max_slots,
                     int32_t block_size_tokens, int32_t fp16_key_value);
/* KvStorage.publishBlockTable (TornadoKvStore.java publishBlockTable): n must equal
 * max_slots * blocks_per_slot. */
int32_t jl_kv_publish_block_table(jl_ctx *ctx, const int32_t *table, int64_t n);
int64_t jl_kv_bytes_per_block(jl_ctx *ctx);
/* Fills both pools, scratch block included, with one binary16 bit pattern. The reference's
 * verification runs poison the cache with NaN (0x7E00) before a sequence so that any read of a
 * page the sequence has not written shows up in the logits (docs/architecture/verification.md:427-431). */
int32_t jl_kv_fill(jl_ctx *ctx, uint16_t half_bits);
/* Test / checkpoint access to one position's K or V row (kv_dim halfs) of a layer. */
int32_t jl_kv_read_row(jl_ctx *ctx, int32_t which /*0=K,1=V*/, int32_t slot, int32_t layer,
                       int32_t pos, uint16_t *out_halfs);

/* ---- the step: replaces TornadoVMMasterPlan.tornadoVMForwardDecode(position)
 * (backend/tornado/TornadoVMMasterPlanSingleToken.java:134-171) for width 1 and
 * BatchExecutor.decodeStep(BatchSlots) (backend/tornado/batch/TornadoBatchExecutor.java:294-347)
 * for width > 1. Arrays have `width` entries; inactive slots are skipped and get token -1.
 * out_tokens: greedy argmax, first index on ties (inference/Logits.java:49-60).
 * out_logits: NULL, or width * vocab floats. */
int32_t jl_decode(jl_ctx *ctx, int32_t width, const int32_t *tokens, const int32_t *positions,
                  const int32_t *kv_slots, const uint8_t *active, int32_t *out_tokens,
                  float *out_logits);
/* Temperature / top-p sampling of the rows of logits the last jl_decode(width) left on the device, in place of
 * copying them out: replaces the host-side chain Sampler.selectSampler builds for temperature != 0
 * (inference/sampler/Sampler.java:63-110: scores / temperature, softmax, then CategoricalSampler.java:13-25 when
 * topp is outside (0,1), else ToppSampler.java:46-103). uniforms[b] is what the caller's generator returned for
 * this call (rng.nextFloat(1f)); rows that were inactive in the decode get -1. The rows of logits are consumed
 * (overwritten, as the reference's in-place softmax does), so out_logits of that decode must have been taken
 * before. last_step_ms reports this call alone. Not available under tensor parallelism. */
int32_t jl_sample(jl_ctx *ctx, int32_t width, float temperature, float topp, const float *uniforms,
                  int32_t *out_tokens);
/* n_steps greedy steps without a host round trip between them: each active row's sampled token is
 * fed back on the device and its position advances (the device-side sampling the reference turns
 * on with -Djitllm.deviceSample, inference/TokenGenerationLoop.java:111-128, carried one step
 * further). out_history receives n_steps * width token ids, step-major; inactive rows get -1. */
int32_t jl_generate(jl_ctx *ctx, int32_t width, const int32_t *tokens, const int32_t *positions,
                    const int32_t *kv_slots, const uint8_t *active, int32_t n_steps,
                    int32_t *out_history);
/* Replaces BatchPrefillDecodePlan.tornadoVMForwardBatchPrefill (backend/tornado/
 * BatchPrefillDecodePlan.java:12-64): n prompt tokens of one sequence at start_pos.., KV pages
 * written, no logits (backend/cpu/InferenceCoreBatchPrefillDecode.java:189-191). */
int32_t jl_prefill(jl_ctx *ctx, int32_t kv_slot, const int32_t *tokens, int32_t start_pos,
                   int32_t n);
/* Reads a named per-step buffer ("x","q","k","v","xb","hb","logits") of batch row `row` after a
 * step; for per-operation parity tests. */
int32_t jl_debug_read(jl_ctx *ctx, const char *name, int32_t row, float *out, int64_t n);

/* ---- standalone operators (the sweep of quantised GEMV/GEMM shapes) */
/* Host blocks in, host floats out: element-exact FloatTensor.getFloat
 * (tensor/standard/Q8_0FloatTensor.java:53-61, Q4_0FloatTensor.java:56-79, Q4_KFloatTensor.java:88-122, and the
 * formats mixed-precision files add: Q4_1FloatTensor.java:76-99, Q5_KFloatTensor.java:87-127,
 * Q6_KFloatTensor.java:64-117). ggml_type: Q4_0=2, Q4_1=3, Q8_0=8, Q4_K=12, Q5_K=13, Q6_K=14. */
int32_t jl_dequant(jl_ctx *ctx, int32_t ggml_type, const void *blocks, int64_t n_elements,
                   float *out);
/* y[n][rows] = W[rows][cols] . x[n][cols]; FloatTensor.matmul (tensor/standard/FloatTensor.java:123-140).
 * Host buffers; copies are part of the call. The same six types as jl_dequant; at most 32768 columns. */
int32_t jl_gemv(jl_ctx *ctx, int32_t ggml_type, int64_t rows, int64_t cols, const void *w_host,
                const float *x_host, int32_t n, float *y_host);
/* Device-resident form: upload once, multiply many times. x_dev / y_dev are device pointers. */
int32_t jl_tensor_upload(jl_ctx *ctx, int32_t ggml_type, int64_t rows, int64_t cols,
                         const void *host_bytes, size_t nbytes, jl_tensor **out);
int32_t jl_tensor_free(jl_ctx *ctx, jl_tensor *t);
int32_t jl_gemv_dev(jl_ctx *ctx, const jl_tensor *w, const float *x_dev, int32_t n, float *y_dev);

/* ---- plumbing */
void *jl_device_alloc(jl_ctx *ctx, size_t nbytes);
int32_t jl_device_free(jl_ctx *ctx, void *p);
int32_t jl_memcpy_h2d(jl_ctx *ctx, void *dst_dev, const void *src_host, size_t nbytes);
int32_t jl_memcpy_d2h(jl_ctx *ctx, void *dst_host, const void *src_dev, size_t nbytes);
int32_t jl_synchronize(jl_ctx *ctx);
/* The cudaStream_t every launch of this context goes to. */
void *jl_stream(jl_ctx *ctx);
/* CUDA-event stopwatch on that stream. */
int32_t jl_timer_start(jl_ctx *ctx);
int32_t jl_timer_stop(jl_ctx *ctx, float *elapsed_ms);
/* Launches one operator of the loaded model `iters` times on successive layers (wrapping) with
 * the step workspace as input and output, for per-kernel timing: op 0 = RMSNorm+QKV, 1 = attention
 * output projection, 2 = RMSNorm+gate/up+SwiGLU, 3 = down projection, 4 = RMSNorm+vocabulary,
 * 5 = RoPE + KV append + attention of row 0 at the position the last step left on the device.
 * The measuring counterpart of backend/tornado/bench/SyntheticKernelBench.java:87-161. */
int32_t jl_bench_op(jl_ctx *ctx, int32_t op, int32_t first_layer, int32_t iters);
/* Launch timeline of the kernels this context enqueues (no counterpart in the reference; its
 * closest relative is the TornadoVM profiler seam, backend/tornado/TornadoMetricsReporter.java:52-64).
 * Only the trace build of the library (compiled with -DJL_TRACE) records anything; the default build
 * returns JL_ERR_UNSUPPORTED. Call with out == NULL to arm and clear the buffer (returns its capacity
 * in records); after some steps call with room for 8 * max_records words: every launch leaves one
 * record written by its first CTA -- kernel id, then nanosecond stamps (entry, grid dependency
 * resolved, inputs staged, main loop done, exit) and two kernel-specific words. Returns the number
 * of records copied. */
int32_t jl_debug_trace(jl_ctx *ctx, uint64_t *out, int32_t max_records);
int32_t jl_get_counters(jl_ctx *ctx, jl_counters *out);
/* Overwrites a 256 MiB scratch buffer (larger than L2) so that the next kernel starts cold. */
int32_t jl_flush_l2(jl_ctx *ctx);

/* ---- tensor parallelism (the reference has none; the nearest seam is the plan's per-layer task
 * graphs, backend/tornado/layers/LogitsQ8_0Layer.java:40-56 and docs/architecture/execution.md,
 * which run on one device). One context per GPU, one process per context. With tp_size > 1 in
 * jl_model_desc the host uploads this rank's shard of every matrix: rows [r*R/tp, (r+1)*R/tp) of
 * wq, wk, wv, w1 (gate), w3 (up) and the vocabulary matrix; columns [r*C/tp, (r+1)*C/tp) of wo and
 * w2 (down), cut on 256-column boundaries so that quantised super-blocks stay whole; norms, RoPE
 * tables and the token embedding in full. Each step then sums the two row-parallel partial results
 * per layer with an NCCL all-reduce on the context's stream and picks the token as the first
 * maximum over the ranks' vocabulary shards.
 * jl_tp_unique_id: rank 0 fills id128 (128 bytes, an ncclUniqueId) for the host to broadcast.
 * jl_tp_init: every rank, after jl_model_create and before jl_model_finalize; collective.
 * nccl_path: the NCCL shared library to bind at run time, or NULL for "libnccl.so.2". */
int32_t jl_tp_unique_id(jl_ctx *ctx, const char *nccl_path, void *id128);
int32_t jl_tp_init(jl_ctx *ctx, const char *nccl_path, const void *id128, int32_t rank, int32_t size);
/* How the ranks exchange the small per-step messages (partial sums of up to 16 rows, the best token
 * of each vocabulary shard) after jl_model_finalize: 0 = single GPU, 1 = NCCL collectives, 2 = one
 * kernel per exchange over peer memory (stores into the other GPUs' inboxes through NVLink; inboxes
 * shared by CUDA IPC between processes), 3 = as 2, with the all-reduce that follows the output and
 * down projections done by the mat-vec kernel's own epilogue (JITLLM_B200_TP_FUSE=0 gives 2 back).
 * Modes 2 and 3 are chosen when every rank could map every inbox;
 * jl_tp_exchange_note says why not otherwise. JITLLM_B200_TP_PUSH=0 forces mode 1. A rank that
 * waits longer than JITLLM_B200_TP_TIMEOUT_MS (default 5000) for a peer's message gives up and the
 * step returns JL_ERR_TIMEOUT; the group is then out of step and must be torn down. Larger
 * messages (prefill chunks, wide batches) always go through NCCL. */
int32_t jl_tp_exchange_mode(jl_ctx *ctx);
/* Self-test of the bounded wait (no counterpart in the reference): runs one two-rank peer exchange in
 * which the second rank is a local buffer that nobody writes, with the given patience (1..2000 ms).
 * The kernel gives up, the call returns JL_ERR_TIMEOUT, and the context stays usable. */
int32_t jl_debug_peer_wait_timeout(jl_ctx *ctx, int32_t timeout_ms);
const char *jl_tp_exchange_note(jl_ctx *ctx);
/* The peer exchange's sequence counter after `seq` (host-side mirror of the device rule, for tests; no
 * counterpart in the reference): consecutive exchanges use inbox slots of opposite parity, also
 * across the wrap of the 32-bit counter, and 0 ("never written") is never produced. Needs no GPU. */
uint32_t jl_debug_tp_next_sequence(uint32_t seq);

/* ---- native GGUF reader (replaces the Java-side parse and per-tensor Panama copies:
 * format/GGUF.java:60-110,123-165, model/loader/LlamaModelLoader.java:49-67,125-188,
 * model/loader/ModelLoader.java:246-290). jl_gguf_open maps the file and parses header, metadata and
 * tensor infos; jl_gguf_describe fills the model description from the llama.* keys (max_batch 1,
 * single GPU: adjust before use) and the RoPE base; jl_gguf_upload does jl_model_create, uploads
 * every tensor from the mapping (under tensor parallelism only this rank's slice, cut as described
 * at jl_tp_init) and the RoPE tables (rope_cos / rope_sin, or computed with the reference's formula
 * when NULL); the caller then calls jl_tp_init (tensor parallel) and jl_model_finalize. Errors:
 * jl_gguf_last_error(). Tokenizer metadata is skipped, not interpreted. */
typedef struct jl_gguf jl_gguf;
int32_t jl_gguf_open(const char *path, jl_gguf **out);
int32_t jl_gguf_describe(const jl_gguf *g, jl_model_desc *desc, float *rope_theta, int64_t *n_tensors);
int32_t jl_gguf_upload(jl_ctx *ctx, const jl_gguf *g, int32_t max_batch, int32_t tp_rank, int32_t tp_size,
                       const float *rope_cos, const float *rope_sin, int64_t rope_n);
void jl_gguf_close(jl_gguf *g);
const char *jl_gguf_last_error(void);

/* ---- allocation-free operator (no counterpart in the reference: its kernels take whatever
 * scratch the TornadoVM runtime allocates for them).
 * y_dev[rows] = W . x (x optionally RMS-normalised with norm_w_dev / rms_eps first) and
 * *token_dev = index of the first maximum of y, for callers that may not allocate device memory
 * at call time (memory carved up once at start-up, a stream being captured, a host-owned pool).
 * Every buffer is the caller's; the kernel's cross-CTA scratch is an 8.25 KiB array inside the
 * library image (held by every GPU that loads the library, until exit), enough for 1024 CTAs.
 * Calls no cudaMalloc / cudaFree. The first call on a device looks up the array's device address
 * and sets kernel attributes -- make that call outside any stream capture. All calls share the
 * array: calls whose kernels overlap on the GPU (different streams) race on it; serialise them.
 * Shapes whose launch would need more than 1024 CTAs, more than 32768 columns, or more shared
 * memory than one SM has, are rejected with JL_ERR_UNSUPPORTED. w_dev: rows x cols in GGUF block
 * layout. w_dev, x_dev and norm_w_dev must be 16-byte aligned, y_dev and token_dev 4-byte aligned;
 * anything else is refused with JL_ERR_INVALID before a kernel is launched.
 * Errors: jl_static_last_error(). The call returns as soon as the kernel is enqueued, so a wait
 * that ran out inside the kernel (every device-side wait is bounded) cannot show in its return
 * value: jl_static_status(stream) synchronises the stream, reads the status word of the latest
 * call on the current device from the static array (a 4-byte copy, no allocation) and returns
 * JL_ERR_TIMEOUT if that kernel gave up, in which case y_dev and token_dev hold nothing valid. */
int32_t jl_gemv_argmax_static(int32_t ggml_type, int64_t rows, int64_t cols, const void *w_dev,
                              const float *x_dev, const float *norm_w_dev, float rms_eps, float *y_dev,
                              int32_t *token_dev, void *stream);
int32_t jl_static_status(void *stream);
const char *jl_static_last_error(void);

#ifdef __cplusplus
}
#endif
#endif
