// Context, device-resident model, paged KV store, the decode step and the C ABI of
// include/jitllm_b200.h. Host-side logic only; the kernels live in gemv.cu / ops.cu.
#include "../../include/jitllm_b200.h"

#include <dlfcn.h>

#include <set>

#include <cstdarg>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <map>
#include <string>
#include <vector>

#include "gemv.cuh"
#include "ops.cuh"
#include "sampler.cuh"
#include "gemm_tc.cuh"
#include "tp_exchange.cuh"

#include <unistd.h>

#include <nvtx3/nvToolsExt.h>

using namespace jl;

namespace {

thread_local std::string g_init_error;

struct DevTensor {
    uint8_t *data = nullptr;
    int type = -1;
    int64_t rows = 0, cols = 0;
    size_t bytes = 0;
    bool has_tmap = false;  // quantised with whole 256-column groups: usable by the tensor-core path
    GemmTensorMap tmap = {};
    // Q6_K only: the copy with padded super-blocks that the tensor map describes (formats.cuh); owned like `data`.
    uint8_t *padded = nullptr;
    size_t padded_bytes = 0;
    // What the mat-vec kernel reads: the padded copy of a Q6_K matrix, else the matrix as uploaded.
    const uint8_t *mv() const { return padded != nullptr ? padded : data; }
};

// Frees a tensor's device memory (both copies) and leaves it empty.
void release_tensor(DevTensor *t) {
    if (t->data) cudaFree(t->data);
    if (t->padded) cudaFree(t->padded);
    *t = DevTensor();
}

struct StepGraph {
    cudaGraphExec_t exec = nullptr;
    uint64_t launches = 0;
};

}  // namespace

struct jl_tensor {
    DevTensor t;
};

struct jl_ctx {
    int device = 0;
    int sm_count = 148;
    cudaStream_t stream = nullptr;
    cudaEvent_t ev0 = nullptr, ev1 = nullptr, tev0 = nullptr, tev1 = nullptr;
    std::string err;
    bool use_graph = true, use_pdl = true;

    bool has_model = false, finalized = false;
    // The model holds a Q4_1 / Q5_K / Q6_K matrix, or Q/K/V (gate/up) of different types: every step, single rows
    // included, takes the row path, whose projections are launched one matrix at a time.
    bool mixed = false;
    jl_model_desc desc = {};
    int kv_dim = 0;
    DevTensor global[JL_ROLE_COUNT];
    std::vector<DevTensor> layer[JL_ROLE_COUNT];
    float *rope_cos = nullptr, *rope_sin = nullptr;

    // paged KV
    bool has_kv = false;
    __half *kpool = nullptr, *vpool = nullptr;
    int32_t *block_table = nullptr;
    int total_blocks = 0, blocks_per_slot = 0, max_slots = 0, block_tokens = 0;
    std::vector<int32_t> host_table;

    // per-step workspace, [max_batch] rows each
    float *x = nullptr, *q = nullptr, *k = nullptr, *v = nullptr, *xb = nullptr, *hb = nullptr,
          *logits = nullptr;
    int32_t *d_tokens = nullptr, *d_positions = nullptr, *d_slots = nullptr, *d_out = nullptr;
    uint8_t *d_active = nullptr;
    float *att_partial = nullptr;
    unsigned *att_count = nullptr;
    float *amax_val = nullptr;
    int *amax_idx = nullptr;
    unsigned *amax_count = nullptr;
    int *d_status = nullptr;
    int attn_nsplit = 1;
    // tensor-parallel placement: local (per-GPU) extents of the sharded dimensions
    int tp_rank = 0, tp_size = 1;
    int l_heads = 0, l_kv_heads = 0, l_qdim = 0, l_hidden = 0, l_vocab = 0;
    // activations of the tensor-core path, pre-split into binary16 hi / lo rows, and their TMA
    // descriptors per token-tile size (16, 32, 64): [0] xb as rows of dim, [1] xb as rows of the
    // local query width, [2] hb as rows of the local hidden width
    void *xb16 = nullptr, *hb16 = nullptr;
    GemmTensorMap xmaps[3][4] = {};
    GemmTensorMap wcls_slice_tmap = {};  // tied embeddings under tensor parallelism: this GPU's rows
    float *gemm_scratch = nullptr;       // split-column partial tiles of the tensor-core path
    size_t gemm_scratch_floats = 0;
    unsigned *gemm_counters = nullptr;   // one arrival counter per output tile, zero between launches
    float *part = nullptr;      // row-parallel partial sums before the all-reduce, [row_cap][dim]
    float *best = nullptr;      // local (value, index) of the arg-max and the gathered pairs
    // peer-memory exchange (tp_exchange.cuh): this GPU's inbox, every rank's inbox as mapped here
    uint2 *tp_inbox = nullptr;
    TpInboxes tp_peers = {};
    bool tp_peer_ipc[kTpMaxRanks] = {};  // mapped with cudaIpcOpenMemHandle (to be closed)
    unsigned *tp_ctr = nullptr;          // [0,1] reduce sequence / arrivals, [2,3] arg-max
    bool tp_push = false;
    size_t tp_reduce_cap = 0, tp_best_cap = 0;
    unsigned long long tp_timeout_ns = 5000000000ull;
    std::string tp_note;                 // why the peer-memory path is off, if it is
    std::set<int> tp_warm;        // step shapes that have run once uncaptured
    float *logits_all = nullptr;  // [rank][row][l_vocab], only when the host asks for logits
    void *nccl_lib = nullptr;   // dlopen handle
    void *nccl_comm = nullptr;  // ncclComm_t
    int row_cap = 1;        // rows the step buffers hold: max(max_batch, prefill chunk)
    float *hb2 = nullptr;   // second FFN buffer of the matrix-matrix path (up projection)
    int32_t *d_history = nullptr, *d_step = nullptr;
    size_t history_cap = 0;
    unsigned long long *d_trace = nullptr;  // launch-timeline records (trace build only)
    float *d_uniforms = nullptr;            // jl_sample: one random number per row
    int batch_attn_min_pairs = 0;           // (rows x KV heads) from which decode batches use attention_batch_launch
    int logits_rows = 0;                    // rows of ctx->logits the last jl_decode left valid
    // pinned host staging: tokens | positions | slots | out | active | status
    int32_t *h_stage = nullptr;

    std::map<int, StepGraph> graphs;  // key: width
    uint32_t *flush_buf = nullptr;
    size_t flush_words = 0;
    std::vector<void *> user_allocs;
    jl_counters counters = {};
};

namespace {

int fail(jl_ctx *ctx, int code, const char *fmt, ...) {
    char buf[1024];
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(buf, sizeof buf, fmt, ap);
    va_end(ap);
    const char *prefix = "";
    switch (code) {
        case JL_ERR_INVALID: prefix = "GPUL-CFG-002: "; break;
        case JL_ERR_UNSUPPORTED: prefix = "GPUL-CFG-002: unsupported: "; break;
        case JL_ERR_OOM: prefix = "GPUL-MEM-001: "; break;
        case JL_ERR_STATE: prefix = "GPUL-LIFE-001: "; break;
        case JL_ERR_TIMEOUT: prefix = "device wait timed out: "; break;
        case JL_ERR_CUDA: prefix = "CUDA: "; break;
        default: break;
    }
    std::string msg = std::string(prefix) + buf;
    if (ctx)
        ctx->err = msg;
    else
        g_init_error = msg;
    return code;
}

#define JL_CUDA(ctx, call)                                                                   \
    do {                                                                                     \
        cudaError_t e_ = (call);                                                             \
        if (e_ != cudaSuccess) {                                                             \
            int code_ = (e_ == cudaErrorMemoryAllocation) ? JL_ERR_OOM : JL_ERR_CUDA;        \
            return fail(ctx, code_, "%s failed: %s", #call, cudaGetErrorString(e_));         \
        }                                                                                    \
    } while (0)

#define JL_REQUIRE(ctx, cond, code, ...) \
    do {                                 \
        if (!(cond)) return fail(ctx, code, __VA_ARGS__); \
    } while (0)

int dev_alloc(jl_ctx *ctx, void **p, size_t bytes) {
    cudaError_t e = cudaMalloc(p, bytes ? bytes : 16);
    if (e != cudaSuccess) {
        cudaGetLastError();
        return fail(ctx, e == cudaErrorMemoryAllocation ? JL_ERR_OOM : JL_ERR_CUDA,
                    "device allocation of %zu bytes failed: %s", bytes, cudaGetErrorString(e));
    }
    return JL_OK;
}


// ---- NCCL, bound at run time (the library itself does not link against it) ---------------------
constexpr int kGemmCounters = 16384;
constexpr size_t kGemmScratchFloats = size_t(16) << 20;  // 64 MiB

struct NcclId {
    char b[128];
};
struct NcclApi {
    int (*GetUniqueId)(NcclId *);
    int (*CommInitRank)(void **, int, NcclId, int);
    int (*AllReduce)(const void *, void *, size_t, int, int, void *, cudaStream_t);
    int (*AllGather)(const void *, void *, size_t, int, void *, cudaStream_t);
    int (*CommDestroy)(void *);
    const char *(*GetErrorString)(int);
};
NcclApi g_nccl = {};
constexpr int kNcclFloat32 = 7, kNcclSum = 0;

int nccl_bind(jl_ctx *ctx, const char *path) {
    if (ctx->nccl_lib) return JL_OK;
    void *h = dlopen(path && *path ? path : "libnccl.so.2", RTLD_NOW | RTLD_GLOBAL);
    if (!h) return fail(ctx, JL_ERR_STATE, "cannot load NCCL (%s)", dlerror());
    g_nccl.GetUniqueId = reinterpret_cast<decltype(g_nccl.GetUniqueId)>(dlsym(h, "ncclGetUniqueId"));
    g_nccl.CommInitRank = reinterpret_cast<decltype(g_nccl.CommInitRank)>(dlsym(h, "ncclCommInitRank"));
    g_nccl.AllReduce = reinterpret_cast<decltype(g_nccl.AllReduce)>(dlsym(h, "ncclAllReduce"));
    g_nccl.AllGather = reinterpret_cast<decltype(g_nccl.AllGather)>(dlsym(h, "ncclAllGather"));
    g_nccl.CommDestroy = reinterpret_cast<decltype(g_nccl.CommDestroy)>(dlsym(h, "ncclCommDestroy"));
    g_nccl.GetErrorString = reinterpret_cast<decltype(g_nccl.GetErrorString)>(dlsym(h, "ncclGetErrorString"));
    if (!g_nccl.GetUniqueId || !g_nccl.CommInitRank || !g_nccl.AllReduce || !g_nccl.AllGather ||
        !g_nccl.CommDestroy || !g_nccl.GetErrorString) {
        dlclose(h);
        return fail(ctx, JL_ERR_STATE, "the NCCL library at '%s' lacks a required symbol", path ? path : "");
    }
    ctx->nccl_lib = h;
    return JL_OK;
}

// Sum of `count` floats over the tensor-parallel group, in place, on the context's stream.
int tp_all_reduce(jl_ctx *ctx, float *buf, size_t count) {
    const int rc = g_nccl.AllReduce(buf, buf, count, kNcclFloat32, kNcclSum, ctx->nccl_comm, ctx->stream);
    if (rc != 0) return fail(ctx, JL_ERR_CUDA, "ncclAllReduce failed: %s", g_nccl.GetErrorString(rc));
    return JL_OK;
}

bool env_flag(const char *name, bool dflt) {
    const char *v = getenv(name);
    if (!v || !*v) return dflt;
    return !(v[0] == '0' || v[0] == 'n' || v[0] == 'N' || v[0] == 'f' || v[0] == 'F');
}

// stand_alone: a matrix for jl_gemv / jl_gemv_dev, which also take Q4_1, Q5_K and Q6_K; the model's tensors
// (jl_upload_tensor) are held to the formats the step kernels read.
int check_shape(jl_ctx *ctx, int type, int64_t rows, int64_t cols, size_t nbytes, bool stand_alone = false) {
    JL_REQUIRE(ctx, rows > 0 && cols > 0, JL_ERR_INVALID, "rows and cols must be positive, got %lld x %lld",
               (long long)rows, (long long)cols);
    if (is_extra_quant(type) && !stand_alone)
        return fail(ctx, JL_ERR_UNSUPPORTED,
                    "GGML type %d (Q4_1=3, Q5_K=13, Q6_K=14) is decoded and multiplied by jl_dequant / jl_gemv only; "
                    "model tensors must be F32=0, F16=1, Q4_0=2, Q8_0=8 or Q4_K=12", type);
    JL_REQUIRE(ctx, type == kF32 || type == kF16 || is_quant(type) || is_extra_quant(type), JL_ERR_UNSUPPORTED,
               "GGML type %d (supported: F32=0, F16=1, Q4_0=2, Q8_0=8, Q4_K=12)", type);
    if (is_quant(type) || is_extra_quant(type))
        JL_REQUIRE(ctx, cols % 256 == 0, JL_ERR_UNSUPPORTED,
                   "quantised rows must be a multiple of 256 columns, got %lld", (long long)cols);
    const int64_t need = rows * row_bytes(type, cols);
    JL_REQUIRE(ctx, int64_t(nbytes) == need, JL_ERR_INVALID,
               "tensor of %lld x %lld type %d needs %lld bytes, got %zu", (long long)rows,
               (long long)cols, type, (long long)need, nbytes);
    return JL_OK;
}

int upload(jl_ctx *ctx, DevTensor *t, int type, int64_t rows, int64_t cols, const void *host,
           size_t nbytes) {
    if (t->data) {
        ctx->counters.weight_bytes -= t->bytes + t->padded_bytes;
        release_tensor(t);
    }
    void *p = nullptr;
    int rc = dev_alloc(ctx, &p, nbytes);
    if (rc) return rc;
    cudaError_t e = cudaMemcpyAsync(p, host, nbytes, cudaMemcpyHostToDevice, ctx->stream);
    if (e == cudaSuccess) e = cudaStreamSynchronize(ctx->stream);
    if (e != cudaSuccess) {
        cudaFree(p);
        return fail(ctx, JL_ERR_CUDA, "weight upload failed: %s", cudaGetErrorString(e));
    }
    t->data = static_cast<uint8_t *>(p);
    t->type = type;
    t->rows = rows;
    t->cols = cols;
    t->bytes = nbytes;
    t->has_tmap = false;
    if ((is_quant(type) || type == kQ4_1 || type == kQ5_K) && cols % 256 == 0) {
        e = gemm_make_tensor_map(&t->tmap, p, type, rows, cols);
        if (e != cudaSuccess) {
            cudaFree(p);
            *t = DevTensor();
            return fail(ctx, JL_ERR_CUDA, "TMA descriptor for a %lld x %lld matrix failed: %s", (long long)rows,
                        (long long)cols, cudaGetErrorString(e));
        }
        t->has_tmap = true;
    } else if (type == kQ6_K && cols % 256 == 0) {
        // The tensor-core kernel reads Q6_K from a copy with padded super-blocks (its tensor map needs rows of
        // 16-byte multiples); the mat-vec kernels and the embedding lookup keep reading the original.
        const size_t nblocks = size_t(rows) * size_t(cols / 256);
        void *pp = nullptr;
        if ((rc = dev_alloc(ctx, &pp, nblocks * kQ6_KPadded))) {
            release_tensor(t);
            return rc;
        }
        t->padded = static_cast<uint8_t *>(pp);
        t->padded_bytes = nblocks * kQ6_KPadded;
        e = pad_q6k_launch(t->data, t->padded, nblocks, ctx->stream);
        if (e == cudaSuccess) e = cudaStreamSynchronize(ctx->stream);
        if (e == cudaSuccess) e = gemm_make_tensor_map(&t->tmap, pp, type, rows, cols);
        if (e != cudaSuccess) {
            release_tensor(t);
            return fail(ctx, JL_ERR_CUDA, "padded copy of a %lld x %lld Q6_K matrix failed: %s", (long long)rows,
                        (long long)cols, cudaGetErrorString(e));
        }
        t->has_tmap = true;
        ctx->counters.kernel_launches++;
    }
    ctx->counters.weight_bytes += nbytes + t->padded_bytes;
    ctx->counters.h2d_bytes += nbytes;
    return JL_OK;
}

void drop_graphs(jl_ctx *ctx) {
    for (auto &kv : ctx->graphs)
        if (kv.second.exec) cudaGraphExecDestroy(kv.second.exec);
    ctx->graphs.clear();
}

// The per-step workspace jl_model_finalize allocates (step buffers, tensor-parallel inboxes and
// mappings, token history): released before a model is finalised again -- uploading a tensor after
// a finalize puts the model back into the "not finalised" state -- and with the model.
void free_workspace(jl_ctx *ctx) {
    drop_graphs(ctx);
    void *bufs[] = {ctx->x,        ctx->q,        ctx->k,      ctx->v,         ctx->xb,           ctx->hb,
                    ctx->hb2,      ctx->logits,   ctx->d_tokens, ctx->d_positions, ctx->d_slots,  ctx->d_out,
                    ctx->d_active, ctx->att_partial, ctx->att_count, ctx->amax_val, ctx->amax_idx, ctx->amax_count};
    for (void *b : bufs)
        if (b) cudaFree(b);
    ctx->x = ctx->q = ctx->k = ctx->v = ctx->xb = ctx->hb = ctx->hb2 = ctx->logits = nullptr;
    ctx->d_tokens = ctx->d_positions = ctx->d_slots = ctx->d_out = nullptr;
    ctx->d_active = nullptr;
    ctx->att_partial = nullptr;
    ctx->att_count = nullptr;
    ctx->amax_val = nullptr;
    ctx->amax_idx = nullptr;
    ctx->amax_count = nullptr;
    if (ctx->xb16) cudaFree(ctx->xb16);
    if (ctx->hb16) cudaFree(ctx->hb16);
    ctx->xb16 = ctx->hb16 = nullptr;
    if (ctx->part) cudaFree(ctx->part);
    if (ctx->best) cudaFree(ctx->best);
    if (ctx->logits_all) cudaFree(ctx->logits_all);
    ctx->part = ctx->best = ctx->logits_all = nullptr;
    for (int r = 0; r < kTpMaxRanks; ++r) {
        if (ctx->tp_peer_ipc[r] && ctx->tp_peers.of[r]) cudaIpcCloseMemHandle(ctx->tp_peers.of[r]);
        ctx->tp_peer_ipc[r] = false;
        ctx->tp_peers.of[r] = nullptr;
    }
    if (ctx->tp_inbox) cudaFree(ctx->tp_inbox);
    if (ctx->tp_ctr) cudaFree(ctx->tp_ctr);
    ctx->tp_inbox = nullptr;
    ctx->tp_ctr = nullptr;
    ctx->tp_push = false;
    ctx->tp_warm.clear();
    if (ctx->d_history) cudaFree(ctx->d_history);
    if (ctx->d_step) cudaFree(ctx->d_step);
    ctx->d_history = ctx->d_step = nullptr;
    ctx->history_cap = 0;
    if (ctx->h_stage) cudaFreeHost(ctx->h_stage);
    ctx->h_stage = nullptr;
    ctx->counters.workspace_bytes = 0;
    ctx->finalized = false;
}

void free_model(jl_ctx *ctx) {
    free_workspace(ctx);
    for (int r = 0; r < JL_ROLE_COUNT; ++r) {
        release_tensor(&ctx->global[r]);
        for (auto &t : ctx->layer[r]) release_tensor(&t);
        ctx->layer[r].clear();
    }
    if (ctx->rope_cos) cudaFree(ctx->rope_cos);
    if (ctx->rope_sin) cudaFree(ctx->rope_sin);
    ctx->rope_cos = ctx->rope_sin = nullptr;
    ctx->counters.weight_bytes = 0;
    ctx->has_model = false;
}

void free_kv(jl_ctx *ctx) {
    drop_graphs(ctx);
    if (ctx->kpool) cudaFree(ctx->kpool);
    if (ctx->vpool) cudaFree(ctx->vpool);
    if (ctx->block_table) cudaFree(ctx->block_table);
    ctx->kpool = ctx->vpool = nullptr;
    ctx->block_table = nullptr;
    ctx->has_kv = false;
    ctx->counters.kv_bytes = 0;
}

// The vocabulary projection of this GPU: output.weight, or -- tied embeddings -- this GPU's row
// range of the (replicated) embedding table.
DevTensor wcls_of(const jl_ctx *ctx) {
    if (ctx->global[JL_ROLE_OUTPUT].data) return ctx->global[JL_ROLE_OUTPUT];
    DevTensor t = ctx->global[JL_ROLE_TOKEN_EMBEDDING];
    if (ctx->tp_size > 1) {
        const size_t rb = size_t(row_bytes(t.type, t.cols));
        t.data += size_t(ctx->tp_rank) * ctx->l_vocab * rb;
        t.rows = ctx->l_vocab;
        t.bytes = size_t(ctx->l_vocab) * rb;
        if (t.has_tmap) t.tmap = ctx->wcls_slice_tmap;
    }
    return t;
}

// One quantised matrix-vector launch for batch row `row`.
int launch_gemv(jl_ctx *ctx, GemvArgs &a, int total_rows, uint64_t *launches) {
    GemvPlan plan;
    if (!gemv_plan(a.type, a.cols, total_rows, a.mode, ctx->sm_count, &plan))
        return fail(ctx, JL_ERR_UNSUPPORTED, "no launch plan for type %d with %d columns", a.type,
                    a.cols);
    a.status = ctx->d_status;
    cudaError_t e = gemv_launch(a, plan, ctx->stream, ctx->use_pdl);
    if (e != cudaSuccess)
        return fail(ctx, JL_ERR_CUDA, "matrix-vector launch failed: %s", cudaGetErrorString(e));
    ++*launches;
    return JL_OK;
}

// Sets up the peer-memory exchange: allocates this GPU's inbox, trades addresses with the other
// ranks (an IPC handle between processes, the plain pointer inside one process) over the NCCL group
// and maps theirs. Any rank failing turns the path off on all ranks, which then keep using NCCL.
struct TpPeerInfo {
    cudaIpcMemHandle_t handle;  // 64 bytes
    unsigned long long ptr;
    long long pid;
    int device;
    int ok;
};
static_assert(sizeof(TpPeerInfo) % 4 == 0, "gathered as 32-bit words");

int tp_push_setup(jl_ctx *ctx) {
    ctx->tp_push = false;
    ctx->tp_note.clear();
    if (!env_flag("JITLLM_B200_TP_PUSH", true)) {
        ctx->tp_note = "disabled by JITLLM_B200_TP_PUSH";
        return JL_OK;
    }
    if (const char *v = getenv("JITLLM_B200_TP_TIMEOUT_MS")) ctx->tp_timeout_ns = 1000000ull * strtoull(v, nullptr, 10);
    const int tp = ctx->tp_size;
    JL_REQUIRE(ctx, tp <= kTpMaxRanks, JL_ERR_UNSUPPORTED, "at most %d tensor-parallel ranks", kTpMaxRanks);
    // reduce region: up to 16 rows of the residual stream; arg-max region: 2 packets per row
    ctx->tp_reduce_cap = size_t(16) * ctx->desc.dim;
    ctx->tp_best_cap = 2 * size_t(ctx->row_cap);
    const size_t packets = 2 * size_t(tp) * (ctx->tp_reduce_cap + ctx->tp_best_cap);
    int rc;
    // A failure on this rank alone must not leave the others waiting in the gathers below: from here
    // on a local failure only clears `local_ok`, which travels to every rank as ok = 0 and turns the
    // path off everywhere. (The gather buffer itself is the one exception: without it this rank
    // cannot take part at all, and the error is returned.)
    float *d_info = nullptr;  // [1 + tp] records: own, then the gathered ones
    if ((rc = dev_alloc(ctx, reinterpret_cast<void **>(&d_info), (1 + tp) * sizeof(TpPeerInfo)))) return rc;
    bool local_ok = dev_alloc(ctx, reinterpret_cast<void **>(&ctx->tp_inbox), packets * sizeof(uint2)) == JL_OK &&
                    dev_alloc(ctx, reinterpret_cast<void **>(&ctx->tp_ctr), 4 * sizeof(unsigned)) == JL_OK;
    if (local_ok) {
        const unsigned ctr0[4] = {1u, 0u, 1u, 0u};
        cudaError_t e = cudaMemsetAsync(ctx->tp_inbox, 0, packets * sizeof(uint2), ctx->stream);
        if (e == cudaSuccess) e = cudaMemcpyAsync(ctx->tp_ctr, ctr0, sizeof ctr0, cudaMemcpyHostToDevice, ctx->stream);
        if (e == cudaSuccess) e = cudaStreamSynchronize(ctx->stream);
        local_ok = e == cudaSuccess;
        cudaGetLastError();
        if (local_ok) ctx->counters.workspace_bytes += packets * sizeof(uint2);
    }
    if (!local_ok) ctx->tp_note = "this rank could not allocate its inbox";

    TpPeerInfo mine = {};
    mine.ptr = reinterpret_cast<unsigned long long>(ctx->tp_inbox);
    mine.pid = static_cast<long long>(getpid());
    mine.device = ctx->device;
    mine.ok = local_ok && cudaIpcGetMemHandle(&mine.handle, ctx->tp_inbox) == cudaSuccess ? 1 : 0;
    cudaGetLastError();
    const size_t words = sizeof(TpPeerInfo) / 4;
    std::vector<TpPeerInfo> all(tp);
    auto gather = [&]() -> int {
        cudaError_t e = cudaMemcpyAsync(d_info, &mine, sizeof mine, cudaMemcpyHostToDevice, ctx->stream);
        if (e != cudaSuccess) return fail(ctx, JL_ERR_CUDA, "%s", cudaGetErrorString(e));
        const int nrc = g_nccl.AllGather(d_info, d_info + words, words, kNcclFloat32, ctx->nccl_comm, ctx->stream);
        if (nrc != 0) return fail(ctx, JL_ERR_CUDA, "ncclAllGather failed: %s", g_nccl.GetErrorString(nrc));
        e = cudaMemcpyAsync(all.data(), d_info + words, tp * sizeof(TpPeerInfo), cudaMemcpyDeviceToHost, ctx->stream);
        if (e == cudaSuccess) e = cudaStreamSynchronize(ctx->stream);
        if (e != cudaSuccess) return fail(ctx, JL_ERR_CUDA, "%s", cudaGetErrorString(e));
        return JL_OK;
    };
    rc = gather();
    // map the peers' inboxes
    bool ok = rc == JL_OK;
    for (int r = 0; ok && r < tp; ++r) ok = all[r].ok == 1;
    if (rc == JL_OK && !ok && ctx->tp_note.empty()) ctx->tp_note = "a rank could not export its inbox";
    for (int r = 0; ok && r < tp; ++r) {
        if (r == ctx->tp_rank) {
            ctx->tp_peers.of[r] = ctx->tp_inbox;
            continue;
        }
        if (all[r].pid == mine.pid) {  // same process: peer access and the pointer itself
            int can = 0;
            cudaDeviceCanAccessPeer(&can, ctx->device, all[r].device);
            cudaError_t e = can ? cudaDeviceEnablePeerAccess(all[r].device, 0) : cudaErrorInvalidDevice;
            if (e == cudaErrorPeerAccessAlreadyEnabled) e = cudaSuccess;
            cudaGetLastError();
            if (e != cudaSuccess) {
                ok = false;
                ctx->tp_note = std::string("no peer access: ") + cudaGetErrorString(e);
                break;
            }
            ctx->tp_peers.of[r] = reinterpret_cast<uint2 *>(all[r].ptr);
        } else {
            void *p = nullptr;
            cudaError_t e = cudaIpcOpenMemHandle(&p, all[r].handle, cudaIpcMemLazyEnablePeerAccess);
            cudaGetLastError();
            if (e != cudaSuccess) {
                ok = false;
                ctx->tp_note = std::string("cudaIpcOpenMemHandle failed: ") + cudaGetErrorString(e);
                break;
            }
            ctx->tp_peers.of[r] = static_cast<uint2 *>(p);
            ctx->tp_peer_ipc[r] = true;
        }
    }
    // agree: the path is on only if every rank mapped every inbox (this also orders the zeroing
    // of every inbox before anyone's first push)
    if (rc == JL_OK) {
        mine.ok = ok ? 1 : 0;
        rc = gather();
        for (int r = 0; rc == JL_OK && ok && r < tp; ++r) ok = all[r].ok == 1;
    }
    cudaFree(d_info);
    if (rc) return rc;
    if (!ok && ctx->tp_note.empty()) ctx->tp_note = "another rank could not map the inboxes";
    ctx->tp_push = ok;
    return JL_OK;
}

// Whether the mat-vec kernel itself does the all-reduce of a row-parallel projection (its epilogue
// pushes partial rows to the peers and collects theirs): needs the peer-memory path.
bool tp_fused(const jl_ctx *ctx) {
    static const bool want = env_flag("JITLLM_B200_TP_FUSE", true);
    return want && ctx->tp_size > 1 && ctx->tp_push && size_t(ctx->desc.dim) <= ctx->tp_reduce_cap;
}
void tp_fill_reduce(const jl_ctx *ctx, GemvArgs &a, int batch_row) {
    a.tpr.inbox = ctx->tp_peers;
    a.tpr.base = 0;
    a.tpr.cap = ctx->tp_reduce_cap;
    a.tpr.tp = ctx->tp_size;
    a.tpr.rank = ctx->tp_rank;
    a.tpr.row_offset = batch_row * ctx->desc.dim;
    a.tpr.ctr = ctx->tp_ctr;
    a.tpr.timeout_ns = ctx->tp_timeout_ns;
}

// Row-parallel epilogue under tensor parallelism: all-reduce the partial projections of `n` rows
// and add the sum into the residual stream (one NCCL all-reduce per sublayer).
int tp_reduce_into_x(jl_ctx *ctx, int n, uint64_t *launches) {
    const size_t count = size_t(n) * ctx->desc.dim;
    if (ctx->tp_push && count <= ctx->tp_reduce_cap) {
        TpReduceArgs a = {};
        a.part = ctx->part;
        a.x = ctx->x;
        a.inbox = ctx->tp_peers;
        a.base = 0;
        a.cap = ctx->tp_reduce_cap;
        a.tp = ctx->tp_size;
        a.rank = ctx->tp_rank;
        a.count = int(count);
        a.ctr = ctx->tp_ctr;
        a.status = ctx->d_status;
        a.timeout_ns = ctx->tp_timeout_ns;
        cudaError_t e = tp_push_reduce_launch(a, ctx->stream, ctx->use_pdl);
        if (e != cudaSuccess) return fail(ctx, JL_ERR_CUDA, "peer reduce launch failed: %s", cudaGetErrorString(e));
        ++*launches;
        return JL_OK;
    }
    int rc = tp_all_reduce(ctx, ctx->part, count);
    if (rc) return rc;
    cudaError_t e = add_rows_launch(ctx->x, ctx->part, size_t(n) * ctx->desc.dim, ctx->stream, ctx->use_pdl);
    if (e != cudaSuccess) return fail(ctx, JL_ERR_CUDA, "residual add launch failed: %s", cudaGetErrorString(e));
    ++*launches;
    return JL_OK;
}

// Each GPU holds the arg-max of its vocabulary shard; gather (value, global index) pairs and keep
// the best, first index on ties (inference/Logits.java:49-60).
int tp_global_argmax(jl_ctx *ctx, int n, uint64_t *launches) {
    if (ctx->tp_push && 2 * size_t(n) <= ctx->tp_best_cap) {
        TpBestArgs a = {};
        a.logits = ctx->logits;
        a.local = ctx->d_out;
        a.out = ctx->d_out;
        a.active = ctx->d_active;
        a.inbox = ctx->tp_peers;
        a.base = 2 * size_t(ctx->tp_size) * ctx->tp_reduce_cap;
        a.cap = ctx->tp_best_cap;
        a.tp = ctx->tp_size;
        a.rank = ctx->tp_rank;
        a.n = n;
        a.l_vocab = ctx->l_vocab;
        a.ctr = ctx->tp_ctr + 2;
        a.status = ctx->d_status;
        a.timeout_ns = ctx->tp_timeout_ns;
        cudaError_t e = tp_push_best_launch(a, ctx->stream, ctx->use_pdl);
        if (e != cudaSuccess) return fail(ctx, JL_ERR_CUDA, "peer arg-max launch failed: %s", cudaGetErrorString(e));
        ++*launches;
        return JL_OK;
    }
    float *local = ctx->best, *all = ctx->best + 2 * size_t(ctx->row_cap);
    cudaError_t e = tp_pack_best_launch(ctx->logits, ctx->d_out, ctx->l_vocab, ctx->tp_rank * ctx->l_vocab, n,
                                        local, ctx->stream);
    if (e != cudaSuccess) return fail(ctx, JL_ERR_CUDA, "arg-max pack launch failed: %s", cudaGetErrorString(e));
    ++*launches;
    const int rc = g_nccl.AllGather(local, all, size_t(2) * n, kNcclFloat32, ctx->nccl_comm, ctx->stream);
    if (rc != 0) return fail(ctx, JL_ERR_CUDA, "ncclAllGather failed: %s", g_nccl.GetErrorString(rc));
    e = tp_pick_best_launch(all, ctx->tp_size, n, ctx->d_active, ctx->d_out, ctx->stream);
    if (e != cudaSuccess) return fail(ctx, JL_ERR_CUDA, "arg-max pick launch failed: %s", cudaGetErrorString(e));
    ++*launches;
    return JL_OK;
}

// NVTX ranges around the sublayers of a step while it is enqueued (or captured into its graph), so
// that a timeline tool shows "L3.attention" / "L3.ffn" instead of a run of anonymous launches: the
// build's counterpart of the reference's per-task-graph profiler names
// (backend/tornado/TornadoMetricsReporter.java:52-78). Off unless JITLLM_B200_NVTX=1.
struct NvtxRange {
    bool on;
    NvtxRange(const char *what, int layer) {
        static const bool enabled = env_flag("JITLLM_B200_NVTX", false);
        on = enabled;
        if (on) {
            char name[48];
            if (layer >= 0) snprintf(name, sizeof name, "L%d.%s", layer, what);
            else snprintf(name, sizeof name, "%s", what);
            nvtxRangePushA(name);
        }
    }
    void next(const char *what, int layer) {
        if (!on) return;
        nvtxRangePop();
        char name[48];
        if (layer >= 0) snprintf(name, sizeof name, "L%d.%s", layer, what);
        else snprintf(name, sizeof name, "%s", what);
        nvtxRangePushA(name);
    }
    ~NvtxRange() {
        if (on) nvtxRangePop();
    }
};

int attn_splits_for_width(const jl_ctx *ctx, int width) {
    return attention_splits(ctx->sm_count, width, ctx->l_kv_heads);
}

// One tensor-core launch over up to three matrices that share the input rows.
// in_kind: which pre-split activation buffer x is mirrored in (0 xb by dim, 1 xb by the local query
// width, 2 hb by the local hidden width), or -1 to let the kernel convert x itself.
// Matrices the fused single-row step can multiply: F32 norm rows aside, what gemv_plan accepts.
bool fused_path_takes(const DevTensor &t) {
    if (!is_extra_quant(t.type)) return true;
    return gemv_takes(t.type, t.cols) && t.cols <= kGemvMaxCols && (t.type != kQ6_K || t.padded != nullptr);
}

// Batches of at least this many rows, and prompt chunks, take the tensor-core projections.
int gemm_min_width() {
    static const int v = [] { const char *e = getenv("JITLLM_B200_GEMM_MIN_WIDTH"); return e ? atoi(e) : 4; }();
    return v;
}

// How the row path multiplies n rows by one matrix: the mat-vec kernel row by row (narrow steps of a model whose gate
// and up projections differ in type, which keeps it off the fused single-row step), else the tensor-core kernel
// (Q6_K through its padded copy).
enum RowsVia { kViaGemv, kViaGemm };
RowsVia rows_via(const jl_ctx *ctx, const DevTensor &, int n) {
    return ctx->mixed && n < gemm_min_width() ? kViaGemv : kViaGemm;
}

int launch_gemm_segs(jl_ctx *ctx, const DevTensor *const *w, float *const *y, const float *const *res, int nseg,
                     const float *x, int n, uint64_t *launches, int in_kind = -1, bool presplit = false);

int launch_gemm(jl_ctx *ctx, const DevTensor &w, const float *x, int n, float *y, const float *res,
                uint64_t *launches, int in_kind = -1, bool presplit = false) {
    const DevTensor *ws[1] = {&w};
    float *ys[1] = {y};
    const float *rs[1] = {res};
    return launch_gemm_segs(ctx, ws, ys, rs, 1, x, n, launches, in_kind, presplit);
}

// Several matrices of one type against the same rows (Q, K, V; gate, up) in one launch where one kernel takes them
// all, else one matrix at a time.
int launch_gemm_segs(jl_ctx *ctx, const DevTensor *const *w, float *const *y, const float *const *res, int nseg,
                     const float *x, int n, uint64_t *launches, int in_kind, bool presplit) {
    const RowsVia via = rows_via(ctx, *w[0], n);
    bool alike = true;
    for (int s = 1; s < nseg; ++s) alike = alike && w[s]->type == w[0]->type && rows_via(ctx, *w[s], n) == via;
    if (!alike) {
        for (int s = 0; s < nseg; ++s) {
            int rc = launch_gemm(ctx, *w[s], x, n, y[s], res != nullptr ? res[s] : nullptr, launches, in_kind, presplit);
            if (rc) return rc;
        }
        return JL_OK;
    }
    if (via == kViaGemv) {
        // A mixed-format model takes the row path for narrow steps too: there the mat-vec kernel serves better,
        // one launch per row (plain mode: the norm, SwiGLU and arg-max around it are row kernels on this path;
        // the residual stays in its epilogue).
        int total = 0;
        for (int s = 0; s < nseg; ++s) total += int(w[s]->rows);
        for (int b = 0; b < n; ++b) {
            GemvArgs a = {};
            a.nseg = nseg;
            for (int s = 0; s < nseg; ++s)
                a.seg[s] = {w[s]->mv(), y[s] + size_t(b) * w[s]->rows,
                            res != nullptr && res[s] != nullptr ? res[s] + size_t(b) * w[s]->rows : nullptr, int(w[s]->rows)};
            a.cols = int(w[0]->cols);
            a.type = w[0]->type;
            a.mode = kGemvPlain;
            a.x = x + size_t(b) * w[0]->cols;
            int rc = launch_gemv(ctx, a, total, launches);
            if (rc) return rc;
        }
        return JL_OK;
    }
    GemmArgs g = {};
    if (in_kind >= 0 && ctx->xb16 != nullptr && n <= ctx->row_cap) {
        if (!presplit) {  // otherwise the producing kernel already wrote the hi / lo rows
            const int cols = int(w[0]->cols);
            char *buf = static_cast<char *>(in_kind == 2 ? ctx->hb16 : ctx->xb16);
            cudaError_t e = split_rows_launch(x, size_t(n) * cols, buf, buf + size_t(ctx->row_cap) * cols * 2, ctx->stream,
                                              ctx->use_pdl);
            if (e != cudaSuccess) return fail(ctx, JL_ERR_CUDA, "activation split launch failed: %s", cudaGetErrorString(e));
            ++*launches;
        }
        const int nt = gemm_token_tile(n);
        g.xmap = &ctx->xmaps[in_kind][nt == 16 ? 0 : (nt == 32 ? 1 : (nt == 64 ? 2 : 3))];
        g.x_lo_row = ctx->row_cap;
    }
    g.nseg = nseg;
    for (int s = 0; s < nseg; ++s) {
        if (!w[s]->has_tmap) return fail(ctx, JL_ERR_UNSUPPORTED, "matrix-matrix product needs a quantised matrix");
        g.seg[s] = {w[s]->data, &w[s]->tmap, y[s], res ? res[s] : nullptr, int(w[s]->rows)};
    }
    g.type = w[0]->type;
    g.cols = int(w[0]->cols);
    g.x = x;
    g.n = n;
    g.status = ctx->d_status;
    g.scratch = ctx->gemm_scratch;
    g.scratch_floats = ctx->gemm_scratch_floats;
    g.counters = ctx->gemm_counters;
    g.counters_len = kGemmCounters;
    g.sm_count = ctx->sm_count;
    g.programmatic = ctx->use_pdl;
    cudaError_t e = gemm_tc_launch(g, ctx->stream);
    if (e != cudaSuccess) return fail(ctx, JL_ERR_CUDA, "matrix-matrix launch failed: %s", cudaGetErrorString(e));
    ++*launches;
    return JL_OK;
}

#define JL_LAUNCH(ctx, call, what)                                                            \
    do {                                                                                      \
        cudaError_t e_ = (call);                                                              \
        if (e_ != cudaSuccess) return fail(ctx, JL_ERR_CUDA, what " launch failed: %s", cudaGetErrorString(e_)); \
        ++*launches;                                                                          \
    } while (0)

// The step for n rows on the tensor-core path (chunked prompt ingestion, wide decode batches):
// the same operator order as enqueue_step, with every projection one matrix-matrix launch and
// the element-wise operators as row kernels. Row r uses tokens[r], positions[r], slots[r].
// own_sequences: every row is a different sequence (a decode batch), so the attention kernel can
// rotate and append each row's K/V itself; rows of one prompt chunk need all appends done first.
int enqueue_rows_step(jl_ctx *ctx, int n, bool with_logits, bool advance, uint64_t *launches, bool own_sequences) {
    const jl_model_desc &d = ctx->desc;
    const int dim = d.dim, kv_dim = ctx->kv_dim;
    const DevTensor &emb = ctx->global[JL_ROLE_TOKEN_EMBEDDING];
    const KvGeom kvg = {ctx->kpool, ctx->vpool, ctx->block_table, ctx->blocks_per_slot, ctx->block_tokens,
                        d.layers, kv_dim};
    JL_LAUNCH(ctx, embedding_launch(emb.type, emb.data, ctx->d_tokens, ctx->d_active, ctx->x, dim, n, ctx->stream, ctx->use_pdl),
              "embedding");
    int rc;
    // The attention kernel writes its rows in the output projection's operand format as well, when
    // that projection will read the pre-split buffer (see launch_gemm_segs).
    const bool attn_presplit = ctx->xb16 != nullptr && n <= ctx->row_cap;
    for (int l = 0; l < d.layers; ++l) {
        const float *attn_norm = reinterpret_cast<const float *>(ctx->layer[JL_ROLE_ATTENTION_NORM][l].data);
        const float *ffn_norm = reinterpret_cast<const float *>(ctx->layer[JL_ROLE_FFN_NORM][l].data);
        NvtxRange range("attention", l);
        JL_LAUNCH(ctx, rmsnorm_rows_launch(ctx->x, attn_norm, d.rms_eps, ctx->xb, dim, n, ctx->d_active, ctx->stream, ctx->xb16,
                                           static_cast<char *>(ctx->xb16) + size_t(ctx->row_cap) * dim * 2, ctx->use_pdl),
                  "rmsnorm");
        {
            const DevTensor *ws[3] = {&ctx->layer[JL_ROLE_ATTENTION_QUERY][l], &ctx->layer[JL_ROLE_ATTENTION_KEY][l],
                                      &ctx->layer[JL_ROLE_ATTENTION_VALUE][l]};
            float *ys[3] = {ctx->q, ctx->k, ctx->v};
            if ((rc = launch_gemm_segs(ctx, ws, ys, nullptr, 3, ctx->xb, n, launches, 0, true))) return rc;
        }
        if (!own_sequences)
            JL_LAUNCH(ctx, kv_append_launch(ctx->k, ctx->v, ctx->rope_cos, ctx->rope_sin, ctx->d_positions, ctx->d_slots,
                                            ctx->d_active, kvg, l, d.head_dim, n, ctx->stream, ctx->use_pdl),
                      "kv append");
        {
            AttnArgs a = {};
            a.q = ctx->q;
            a.k = ctx->k;
            a.v = ctx->v;
            a.out = ctx->xb;
            a.rope_cos = ctx->rope_cos;
            a.rope_sin = ctx->rope_sin;
            a.positions = ctx->d_positions;
            a.slots = ctx->d_slots;
            a.active = ctx->d_active;
            a.kv = kvg;
            a.layer = l;
            a.heads = ctx->l_heads;
            a.kv_heads = ctx->l_kv_heads;
            a.head_dim = d.head_dim;
            a.dim = ctx->l_qdim;
            a.nsplit = attn_splits_for_width(ctx, n);
            a.append = own_sequences ? 1 : 0;
            a.partial = ctx->att_partial;
            a.counters = ctx->att_count;
            if (attn_presplit) {  // the output projection reads these rows as binary16 hi / lo parts
                a.out_hi = ctx->xb16;
                a.out_lo = static_cast<char *>(ctx->xb16) + size_t(ctx->row_cap) * ctx->l_qdim * 2;
            }
            // A prompt chunk (one sequence, keys appended above) goes through the tiled kernel; decode
            // batches (one sequence per row) and very short chunks walk the pages row by row.
            static const int tiled_min = [] { const char *v = getenv("JITLLM_B200_PROMPT_ATTN_MIN_ROWS"); return v ? atoi(v) : 8; }();
            if (!own_sequences && n >= tiled_min)
                JL_LAUNCH(ctx, attention_prompt_launch(a, n, ctx->stream, ctx->use_pdl), "prompt attention");
            else if (own_sequences && n >= 4 && n * ctx->l_kv_heads >= ctx->batch_attn_min_pairs)
                // enough (row, KV head) pairs to fill the GPU with one CTA each: the tensor-core walk; narrower
                // batches keep the kernel that splits a sequence's keys over a cluster of CTAs
                JL_LAUNCH(ctx, attention_batch_launch(a, n, ctx->stream, ctx->use_pdl), "batch attention");
            else
                JL_LAUNCH(ctx, attention_launch(a, n, ctx->stream, ctx->use_pdl), "attention");
        }
        if (ctx->tp_size > 1) {
            if ((rc = launch_gemm(ctx, ctx->layer[JL_ROLE_ATTENTION_OUTPUT][l], ctx->xb, n, ctx->part, nullptr, launches, 1, attn_presplit))) return rc;
            if ((rc = tp_reduce_into_x(ctx, n, launches))) return rc;
        } else if ((rc = launch_gemm(ctx, ctx->layer[JL_ROLE_ATTENTION_OUTPUT][l], ctx->xb, n, ctx->x, ctx->x, launches, 1, attn_presplit))) {
            return rc;
        }
        range.next("ffn", l);
        JL_LAUNCH(ctx, rmsnorm_rows_launch(ctx->x, ffn_norm, d.rms_eps, ctx->xb, dim, n, ctx->d_active, ctx->stream, ctx->xb16,
                                           static_cast<char *>(ctx->xb16) + size_t(ctx->row_cap) * dim * 2, ctx->use_pdl),
                  "rmsnorm");
        {
            const DevTensor *ws[2] = {&ctx->layer[JL_ROLE_FFN_GATE][l], &ctx->layer[JL_ROLE_FFN_UP][l]};
            float *ys[2] = {ctx->hb, ctx->hb2};
            if ((rc = launch_gemm_segs(ctx, ws, ys, nullptr, 2, ctx->xb, n, launches, 0, true))) return rc;
        }
        JL_LAUNCH(ctx, swiglu_rows_launch(ctx->hb, ctx->hb2, ctx->l_hidden, n, ctx->stream, ctx->hb16,
                                          static_cast<char *>(ctx->hb16) + size_t(ctx->row_cap) * ctx->l_hidden * 2, ctx->use_pdl),
                  "swiglu");
        if (ctx->tp_size > 1) {
            if ((rc = launch_gemm(ctx, ctx->layer[JL_ROLE_FFN_DOWN][l], ctx->hb, n, ctx->part, nullptr, launches, 2, true))) return rc;
            if ((rc = tp_reduce_into_x(ctx, n, launches))) return rc;
        } else if ((rc = launch_gemm(ctx, ctx->layer[JL_ROLE_FFN_DOWN][l], ctx->hb, n, ctx->x, ctx->x, launches, 2, true))) {
            return rc;
        }
    }
    if (with_logits) {
        const float *out_norm = reinterpret_cast<const float *>(ctx->global[JL_ROLE_OUTPUT_NORM].data);
        JL_LAUNCH(ctx, rmsnorm_rows_launch(ctx->x, out_norm, d.rms_eps, ctx->xb, dim, n, ctx->d_active, ctx->stream, ctx->xb16,
                                           static_cast<char *>(ctx->xb16) + size_t(ctx->row_cap) * dim * 2, ctx->use_pdl),
                  "rmsnorm");
        if ((rc = launch_gemm(ctx, wcls_of(ctx), ctx->xb, n, ctx->logits, nullptr, launches, 0, true))) return rc;
        JL_LAUNCH(ctx, argmax_rows_launch(ctx->logits, ctx->l_vocab, n, ctx->d_active, ctx->d_out, ctx->stream, ctx->use_pdl),
                  "argmax");
        if (ctx->tp_size > 1 && (rc = tp_global_argmax(ctx, n, launches))) return rc;
    }
    if (advance)
        JL_LAUNCH(ctx, advance_launch(ctx->d_tokens, ctx->d_positions, ctx->d_out, ctx->d_active, ctx->d_history,
                                      ctx->d_step, n, ctx->stream, ctx->use_pdl),
                  "advance");
    return JL_OK;
}

// Enqueues the kernels of one decode step for `width` batch rows on ctx->stream.
// Order of operations per layer: backend/cpu/InferenceCore.java:72-141 of the reference.
int enqueue_step(jl_ctx *ctx, int width, bool with_logits, bool advance, uint64_t *launches) {
    const jl_model_desc &d = ctx->desc;
    const int dim = d.dim, kv_dim = ctx->kv_dim, hidden = ctx->l_hidden, qdim = ctx->l_qdim;
    const bool tp = ctx->tp_size > 1;
    const bool fused = tp_fused(ctx);
    const DevTensor &emb = ctx->global[JL_ROLE_TOKEN_EMBEDDING];
    cudaError_t e = embedding_launch(emb.type, emb.data, ctx->d_tokens, ctx->d_active, ctx->x, dim,
                                     width, ctx->stream, false);
    if (e != cudaSuccess)
        return fail(ctx, JL_ERR_CUDA, "embedding launch failed: %s", cudaGetErrorString(e));
    ++*launches;
    int rc;
    for (int l = 0; l < d.layers; ++l) {
        const DevTensor &wq = ctx->layer[JL_ROLE_ATTENTION_QUERY][l];
        const DevTensor &wk = ctx->layer[JL_ROLE_ATTENTION_KEY][l];
        const DevTensor &wv = ctx->layer[JL_ROLE_ATTENTION_VALUE][l];
        const DevTensor &wo = ctx->layer[JL_ROLE_ATTENTION_OUTPUT][l];
        const DevTensor &w1 = ctx->layer[JL_ROLE_FFN_GATE][l];
        const DevTensor &w3 = ctx->layer[JL_ROLE_FFN_UP][l];
        const DevTensor &w2 = ctx->layer[JL_ROLE_FFN_DOWN][l];
        const float *attn_norm =
            reinterpret_cast<const float *>(ctx->layer[JL_ROLE_ATTENTION_NORM][l].data);
        const float *ffn_norm =
            reinterpret_cast<const float *>(ctx->layer[JL_ROLE_FFN_NORM][l].data);
        NvtxRange range("attention", l);
        const bool qkv_alike = wk.type == wq.type && wv.type == wq.type;
        for (int b = 0; b < width; ++b) {
            GemvArgs a = {};
            a.cols = dim;
            a.mode = kGemvPlain;
            a.x = ctx->x + size_t(b) * dim;
            a.norm_w = attn_norm;
            a.eps = d.rms_eps;
            a.active = ctx->d_active + b;
            const GemvSeg segs[3] = {{wq.mv(), ctx->q + size_t(b) * qdim, nullptr, int(wq.rows)},
                                     {wk.mv(), ctx->k + size_t(b) * kv_dim, nullptr, int(wk.rows)},
                                     {wv.mv(), ctx->v + size_t(b) * kv_dim, nullptr, int(wv.rows)}};
            if (qkv_alike) {
                a.nseg = 3;
                a.seg[0] = segs[0];
                a.seg[1] = segs[1];
                a.seg[2] = segs[2];
                a.type = wq.type;
                if ((rc = launch_gemv(ctx, a, int(wq.rows + wk.rows + wv.rows), launches))) return rc;
            } else {
                // mixed-precision files keep the value projection in another format: one launch per matrix, each
                // normalising the row again
                const int types[3] = {wq.type, wk.type, wv.type};
                for (int i = 0; i < 3; ++i) {
                    a.nseg = 1;
                    a.seg[0] = segs[i];
                    a.type = types[i];
                    if ((rc = launch_gemv(ctx, a, segs[i].rows, launches))) return rc;
                }
            }
        }
        {
            AttnArgs a = {};
            a.q = ctx->q;
            a.k = ctx->k;
            a.v = ctx->v;
            a.out = ctx->xb;
            a.rope_cos = ctx->rope_cos;
            a.rope_sin = ctx->rope_sin;
            a.positions = ctx->d_positions;
            a.slots = ctx->d_slots;
            a.active = ctx->d_active;
            a.kv = {ctx->kpool, ctx->vpool, ctx->block_table, ctx->blocks_per_slot,
                    ctx->block_tokens, d.layers, kv_dim};
            a.layer = l;
            a.heads = ctx->l_heads;
            a.kv_heads = ctx->l_kv_heads;
            a.head_dim = d.head_dim;
            a.dim = qdim;
            a.nsplit = attn_splits_for_width(ctx, width);
            a.append = 1;
            a.partial = ctx->att_partial;
            a.counters = ctx->att_count;
            e = attention_launch(a, width, ctx->stream, ctx->use_pdl);
            if (e != cudaSuccess)
                return fail(ctx, JL_ERR_CUDA, "attention launch failed: %s", cudaGetErrorString(e));
            ++*launches;
        }
        for (int b = 0; b < width; ++b) {
            GemvArgs a = {};
            a.nseg = 1;
            float *xr = ctx->x + size_t(b) * dim;
            if (tp && !fused)
                a.seg[0] = {wo.mv(), ctx->part + size_t(b) * dim, nullptr, int(wo.rows)};
            else
                a.seg[0] = {wo.mv(), xr, xr, int(wo.rows)};
            if (fused) tp_fill_reduce(ctx, a, b);
            a.cols = int(wo.cols);
            a.type = wo.type;
            a.mode = kGemvPlain;
            a.x = ctx->xb + size_t(b) * qdim;
            a.active = ctx->d_active + b;
            if ((rc = launch_gemv(ctx, a, int(wo.rows), launches))) return rc;
        }
        if (tp && !fused && (rc = tp_reduce_into_x(ctx, width, launches))) return rc;
        range.next("ffn", l);
        for (int b = 0; b < width; ++b) {
            GemvArgs a = {};
            a.nseg = 2;
            a.seg[0] = {w1.mv(), ctx->hb + size_t(b) * hidden, nullptr, int(w1.rows)};
            a.seg[1] = {w3.mv(), nullptr, nullptr, int(w3.rows)};
            a.cols = dim;
            a.type = w1.type;
            a.mode = kGemvGateUp;
            a.x = ctx->x + size_t(b) * dim;
            a.norm_w = ffn_norm;
            a.eps = d.rms_eps;
            a.active = ctx->d_active + b;
            if ((rc = launch_gemv(ctx, a, int(w1.rows + w3.rows), launches))) return rc;
        }
        for (int b = 0; b < width; ++b) {
            GemvArgs a = {};
            a.nseg = 1;
            float *xr = ctx->x + size_t(b) * dim;
            if (tp && !fused)
                a.seg[0] = {w2.mv(), ctx->part + size_t(b) * dim, nullptr, int(w2.rows)};
            else
                a.seg[0] = {w2.mv(), xr, xr, int(w2.rows)};
            if (fused) tp_fill_reduce(ctx, a, b);
            a.cols = int(w2.cols);
            a.type = w2.type;
            a.mode = kGemvPlain;
            a.x = ctx->hb + size_t(b) * hidden;
            a.active = ctx->d_active + b;
            if ((rc = launch_gemv(ctx, a, int(w2.rows), launches))) return rc;
        }
        if (tp && !fused && (rc = tp_reduce_into_x(ctx, width, launches))) return rc;
    }
    if (with_logits) {
        NvtxRange range("logits", -1);
        const DevTensor wc = wcls_of(ctx);
        for (int b = 0; b < width; ++b) {
            GemvArgs a = {};
            a.nseg = 1;
            a.seg[0] = {wc.mv(), ctx->logits + size_t(b) * ctx->l_vocab, nullptr, int(wc.rows)};
            a.cols = dim;
            a.type = wc.type;
            a.mode = kGemvPlain;
            a.x = ctx->x + size_t(b) * dim;
            a.norm_w = reinterpret_cast<const float *>(ctx->global[JL_ROLE_OUTPUT_NORM].data);
            a.eps = d.rms_eps;
            a.active = ctx->d_active + b;
            a.argmax_val = ctx->amax_val + size_t(b) * 4 * ctx->sm_count;
            a.argmax_idx = ctx->amax_idx + size_t(b) * 4 * ctx->sm_count;
            a.argmax_count = ctx->amax_count + b;
            a.out_token = ctx->d_out + b;
            if ((rc = launch_gemv(ctx, a, int(wc.rows), launches))) return rc;
        }
        if (tp && (rc = tp_global_argmax(ctx, width, launches))) return rc;
    }
    if (advance) {
        e = advance_launch(ctx->d_tokens, ctx->d_positions, ctx->d_out, ctx->d_active, ctx->d_history,
                           ctx->d_step, width, ctx->stream, ctx->use_pdl);
        if (e != cudaSuccess)
            return fail(ctx, JL_ERR_CUDA, "advance launch failed: %s", cudaGetErrorString(e));
        ++*launches;
    }
    return JL_OK;
}

// Runs one step: replays the captured graph for this width, capturing it on first use.
int run_step(jl_ctx *ctx, int width, bool with_logits, bool advance = false) {
    const bool rows_path = width >= gemm_min_width() || ctx->mixed;
    const int key = width * 8 + (with_logits ? 1 : 0) + (advance ? 2 : 0) + (rows_path ? 4 : 0);
    uint64_t launches = 0;
    // Under tensor parallelism the first step of each shape runs uncaptured, so that NCCL sets up
    // its channels and buffers outside a capture; later steps replay a graph that holds the
    // collectives too (JITLLM_B200_TP_GRAPH=0 keeps them all uncaptured).
    static const bool tp_graph = env_flag("JITLLM_B200_TP_GRAPH", true);
    const bool eager = !ctx->use_graph || (ctx->tp_size > 1 && (!tp_graph || ctx->tp_warm.insert(key).second));
    if (eager) {
        int rc = rows_path ? enqueue_rows_step(ctx, width, with_logits, advance, &launches, true)
                           : enqueue_step(ctx, width, with_logits, advance, &launches);
        ctx->counters.kernel_launches += launches;
        return rc;
    }
    auto it = ctx->graphs.find(key);
    if (it == ctx->graphs.end()) {
        cudaGraph_t graph = nullptr;
        JL_CUDA(ctx, cudaStreamBeginCapture(ctx->stream, cudaStreamCaptureModeThreadLocal));
        int rc = rows_path ? enqueue_rows_step(ctx, width, with_logits, advance, &launches, true)
                           : enqueue_step(ctx, width, with_logits, advance, &launches);
        cudaError_t e = cudaStreamEndCapture(ctx->stream, &graph);
        if (rc) {
            if (graph) cudaGraphDestroy(graph);
            return rc;
        }
        if (e != cudaSuccess)
            return fail(ctx, JL_ERR_CUDA, "graph capture failed: %s", cudaGetErrorString(e));
        StepGraph sg;
        e = cudaGraphInstantiate(&sg.exec, graph, 0);
        cudaGraphDestroy(graph);
        if (e != cudaSuccess)
            return fail(ctx, e == cudaErrorMemoryAllocation ? JL_ERR_OOM : JL_ERR_CUDA,
                        "graph instantiation failed: %s", cudaGetErrorString(e));
        sg.launches = launches;
        it = ctx->graphs.emplace(key, sg).first;
    }
    JL_CUDA(ctx, cudaGraphLaunch(it->second.exec, ctx->stream));
    ctx->counters.kernel_launches += it->second.launches;
    return JL_OK;
}

int check_status(jl_ctx *ctx) {
    int st = ctx->h_stage[5 * ctx->row_cap];
    if (st == kDevTimeout) {
        cudaMemsetAsync(ctx->d_status, 0, sizeof(int), ctx->stream);
        return fail(ctx, JL_ERR_TIMEOUT, "a kernel gave up waiting for an asynchronous copy");
    }
    return JL_OK;
}

}  // namespace

// =================================================================================== C ABI

extern "C" {

int32_t jl_init(int32_t device_id, jl_ctx **out) {
    if (!out) return fail(nullptr, JL_ERR_INVALID, "out must not be NULL");
    *out = nullptr;
    int count = 0;
    cudaError_t e = cudaGetDeviceCount(&count);
    if (e != cudaSuccess || count == 0) {
        cudaGetLastError();
        return fail(nullptr, JL_ERR_CUDA,
                    "no usable CUDA device (%s); this library has no CPU fallback",
                    e != cudaSuccess ? cudaGetErrorString(e) : "device count is 0");
    }
    if (device_id < 0 || device_id >= count)
        return fail(nullptr, JL_ERR_INVALID, "device %d out of range (0..%d)", device_id, count - 1);
    cudaDeviceProp prop;
    JL_CUDA(nullptr, cudaSetDevice(device_id));
    JL_CUDA(nullptr, cudaGetDeviceProperties(&prop, device_id));
    if (prop.major != 10)
        return fail(nullptr, JL_ERR_UNSUPPORTED,
                    "device %d is sm_%d%d; this build carries sm_100a code only", device_id,
                    prop.major, prop.minor);
    jl_ctx *ctx = new jl_ctx();
    ctx->device = device_id;
    ctx->sm_count = prop.multiProcessorCount;
    ctx->use_graph = env_flag("JITLLM_B200_GRAPH", true);
    ctx->use_pdl = env_flag("JITLLM_B200_PDL", true);
    {
        // enough (row, KV head) pairs to give most SMs a CTA of their own: the tensor-core walk of
        // attention_batch_launch; narrower batches keep the kernel that splits a sequence's keys over a cluster
        const char *v = getenv("JITLLM_B200_BATCH_ATTN_MIN_PAIRS");
        ctx->batch_attn_min_pairs = v ? atoi(v) : (3 * ctx->sm_count) / 4;
    }
    e = cudaStreamCreateWithFlags(&ctx->stream, cudaStreamNonBlocking);
    if (e == cudaSuccess) e = cudaEventCreate(&ctx->ev0);
    if (e == cudaSuccess) e = cudaEventCreate(&ctx->ev1);
    if (e == cudaSuccess) e = cudaEventCreate(&ctx->tev0);
    if (e == cudaSuccess) e = cudaEventCreate(&ctx->tev1);
    if (e == cudaSuccess) e = gemv_configure();
    if (e == cudaSuccess) e = attention_configure();
    if (e == cudaSuccess) e = gemm_tc_configure();
    if (e == cudaSuccess) e = cudaMalloc(reinterpret_cast<void **>(&ctx->d_status), sizeof(int));
    if (e == cudaSuccess) e = cudaMemset(ctx->d_status, 0, sizeof(int));
    if (e == cudaSuccess) e = cudaMalloc(reinterpret_cast<void **>(&ctx->gemm_scratch), kGemmScratchFloats * 4);
    if (e == cudaSuccess) ctx->gemm_scratch_floats = kGemmScratchFloats;
    if (e == cudaSuccess) e = cudaMalloc(reinterpret_cast<void **>(&ctx->gemm_counters), kGemmCounters * sizeof(unsigned));
    if (e == cudaSuccess) e = cudaMemset(ctx->gemm_counters, 0, kGemmCounters * sizeof(unsigned));
    if (e != cudaSuccess) {
        int rc = fail(nullptr, JL_ERR_CUDA, "context set-up failed: %s", cudaGetErrorString(e));
        jl_destroy(ctx);
        return rc;
    }
    *out = ctx;
    return JL_OK;
}

int32_t jl_destroy(jl_ctx *ctx) {
    if (!ctx) return JL_OK;
    cudaSetDevice(ctx->device);
    if (ctx->stream) cudaStreamSynchronize(ctx->stream);
    free_model(ctx);
    free_kv(ctx);
    if (ctx->nccl_comm) g_nccl.CommDestroy(ctx->nccl_comm);
    ctx->nccl_comm = nullptr;
    for (void *p : ctx->user_allocs) cudaFree(p);
    if (ctx->flush_buf) cudaFree(ctx->flush_buf);
    if (ctx->d_status) cudaFree(ctx->d_status);
    if (ctx->gemm_scratch) cudaFree(ctx->gemm_scratch);
    if (ctx->gemm_counters) cudaFree(ctx->gemm_counters);
    if (ctx->ev0) cudaEventDestroy(ctx->ev0);
    if (ctx->ev1) cudaEventDestroy(ctx->ev1);
    if (ctx->tev0) cudaEventDestroy(ctx->tev0);
    if (ctx->tev1) cudaEventDestroy(ctx->tev1);
    if (ctx->stream) cudaStreamDestroy(ctx->stream);
    delete ctx;
    return JL_OK;
}

const char *jl_last_error(jl_ctx *ctx) { return ctx ? ctx->err.c_str() : g_init_error.c_str(); }

int32_t jl_tp_exchange_mode(jl_ctx *ctx) {
    if (!ctx || ctx->tp_size <= 1) return 0;
    return ctx->tp_push ? (tp_fused(ctx) ? 3 : 2) : 1;
}

const char *jl_tp_exchange_note(jl_ctx *ctx) { return ctx ? ctx->tp_note.c_str() : ""; }

int32_t jl_tp_unique_id(jl_ctx *ctx, const char *nccl_path, void *id128) {
    if (!ctx) return JL_ERR_INVALID;
    JL_REQUIRE(ctx, id128 != nullptr, JL_ERR_INVALID, "id128 must not be NULL");
    int rc = nccl_bind(ctx, nccl_path);
    if (rc) return rc;
    NcclId id;
    const int nrc = g_nccl.GetUniqueId(&id);
    if (nrc != 0) return fail(ctx, JL_ERR_CUDA, "ncclGetUniqueId failed: %s", g_nccl.GetErrorString(nrc));
    memcpy(id128, id.b, sizeof id.b);
    return JL_OK;
}

int32_t jl_tp_init(jl_ctx *ctx, const char *nccl_path, const void *id128, int32_t rank, int32_t size) {
    if (!ctx) return JL_ERR_INVALID;
    JL_REQUIRE(ctx, id128 != nullptr, JL_ERR_INVALID, "id128 must not be NULL");
    JL_REQUIRE(ctx, size >= 2 && rank >= 0 && rank < size, JL_ERR_INVALID,
               "tensor-parallel rank %d of %d is not valid (size must be at least 2)", rank, size);
    JL_REQUIRE(ctx, ctx->nccl_comm == nullptr, JL_ERR_STATE, "the tensor-parallel group is already set up");
    JL_REQUIRE(ctx, !ctx->has_model || (ctx->tp_rank == rank && ctx->tp_size == size), JL_ERR_INVALID,
               "rank %d of %d does not match the model description (%d of %d)", rank, size, ctx->tp_rank,
               ctx->tp_size);
    int rc = nccl_bind(ctx, nccl_path);
    if (rc) return rc;
    cudaSetDevice(ctx->device);
    NcclId id;
    memcpy(id.b, id128, sizeof id.b);
    void *comm = nullptr;
    const int nrc = g_nccl.CommInitRank(&comm, size, id, rank);
    if (nrc != 0) return fail(ctx, JL_ERR_CUDA, "ncclCommInitRank failed: %s", g_nccl.GetErrorString(nrc));
    ctx->nccl_comm = comm;
    return JL_OK;
}

int32_t jl_model_create(jl_ctx *ctx, const jl_model_desc *desc) {
    if (!ctx) return JL_ERR_INVALID;
    JL_REQUIRE(ctx, desc != nullptr, JL_ERR_INVALID, "desc must not be NULL");
    const jl_model_desc &d = *desc;
    JL_REQUIRE(ctx, d.dim > 0 && d.hidden > 0 && d.layers > 0 && d.heads > 0 && d.kv_heads > 0 &&
                        d.head_dim > 0 && d.vocab > 0 && d.ctx_len > 0,
               JL_ERR_INVALID, "every model dimension must be positive");
    JL_REQUIRE(ctx, d.heads % d.kv_heads == 0, JL_ERR_INVALID,
               "heads (%d) must be a multiple of kv_heads (%d)", d.heads, d.kv_heads);
    JL_REQUIRE(ctx, d.heads * d.head_dim == d.dim, JL_ERR_UNSUPPORTED,
               "heads * head_dim (%d) must equal dim (%d) for the Llama layout", d.heads * d.head_dim,
               d.dim);
    JL_REQUIRE(ctx, d.head_dim == 64 || d.head_dim == 128, JL_ERR_UNSUPPORTED,
               "head_dim %d (supported: 64, 128)", d.head_dim);
    const int gq = d.heads / d.kv_heads;
    JL_REQUIRE(ctx, gq == 1 || gq == 2 || gq == 4 || gq == 8, JL_ERR_UNSUPPORTED,
               "heads / kv_heads = %d (supported: 1, 2, 4, 8)", gq);
    JL_REQUIRE(ctx, d.dim % 256 == 0 && d.hidden % 256 == 0, JL_ERR_UNSUPPORTED,
               "dim and hidden must be multiples of 256");
    JL_REQUIRE(ctx, d.max_batch >= 1 && d.max_batch <= 256, JL_ERR_INVALID,
               "max_batch must be in 1..256, got %d", d.max_batch);
    const int tp = d.tp_size < 1 ? 1 : d.tp_size;
    JL_REQUIRE(ctx, d.tp_rank >= 0 && d.tp_rank < tp, JL_ERR_INVALID, "tensor parallel rank %d outside 0..%d",
               d.tp_rank, tp - 1);
    JL_REQUIRE(ctx, d.heads % tp == 0 && d.kv_heads % tp == 0 && d.vocab % tp == 0 &&
                        (d.dim / tp) % 256 == 0 && d.dim % tp == 0 && d.hidden % (tp * 256) == 0,
               JL_ERR_UNSUPPORTED,
               "tensor parallel degree %d must divide heads, kv_heads and vocab, and leave dim/tp and "
               "hidden/tp multiples of 256 (column shards cut on quantisation group boundaries)",
               tp);
    {
        const int lg = (d.heads / tp) / (d.kv_heads / tp);
        JL_REQUIRE(ctx, lg == gq, JL_ERR_INVALID, "inconsistent head grouping under tensor parallelism (%d)", lg);
    }
    cudaSetDevice(ctx->device);
    free_model(ctx);
    ctx->desc = d;
    if (ctx->desc.tp_size < 1) ctx->desc.tp_size = 1;
    ctx->tp_size = ctx->desc.tp_size;
    ctx->tp_rank = d.tp_rank;
    ctx->l_heads = d.heads / ctx->tp_size;
    ctx->l_kv_heads = d.kv_heads / ctx->tp_size;
    ctx->l_qdim = ctx->l_heads * d.head_dim;
    ctx->l_hidden = d.hidden / ctx->tp_size;
    ctx->l_vocab = d.vocab / ctx->tp_size;
    ctx->kv_dim = ctx->l_kv_heads * d.head_dim;  // local: KV pages hold this GPU's KV heads only
    for (int r = 0; r < JL_ROLE_COUNT; ++r) ctx->layer[r].assign(d.layers, DevTensor());
    ctx->has_model = true;
    return JL_OK;
}

int32_t jl_upload_tensor(jl_ctx *ctx, int32_t role, int32_t layer, int32_t ggml_type, int64_t rows,
                         int64_t cols, const void *host_bytes, size_t nbytes) {
    if (!ctx) return JL_ERR_INVALID;
    JL_REQUIRE(ctx, ctx->has_model, JL_ERR_STATE, "jl_model_create must come first");
    JL_REQUIRE(ctx, role >= 0 && role < JL_ROLE_COUNT, JL_ERR_INVALID, "unknown tensor role %d", role);
    JL_REQUIRE(ctx, host_bytes != nullptr, JL_ERR_INVALID, "host_bytes must not be NULL");
    const jl_model_desc &d = ctx->desc;
    const bool per_layer = !(role == JL_ROLE_TOKEN_EMBEDDING || role == JL_ROLE_OUTPUT_NORM ||
                             role == JL_ROLE_OUTPUT);
    if (per_layer)
        JL_REQUIRE(ctx, layer >= 0 && layer < d.layers, JL_ERR_INVALID, "layer %d out of range 0..%d",
                   layer, d.layers - 1);
    int64_t er = 0, ec = 0;
    bool norm = false;
    switch (role) {
        case JL_ROLE_TOKEN_EMBEDDING: er = d.vocab; ec = d.dim; break;
        // Under tensor parallelism the caller uploads this GPU's shard: column-parallel matrices
        // (Q, K, V, gate, up, output) lose rows, row-parallel ones (attention output, down) columns.
        case JL_ROLE_OUTPUT: er = ctx->l_vocab; ec = d.dim; break;
        case JL_ROLE_ATTENTION_QUERY: er = ctx->l_qdim; ec = d.dim; break;
        case JL_ROLE_ATTENTION_KEY:
        case JL_ROLE_ATTENTION_VALUE: er = ctx->kv_dim; ec = d.dim; break;
        case JL_ROLE_ATTENTION_OUTPUT: er = d.dim; ec = ctx->l_qdim; break;
        case JL_ROLE_FFN_GATE:
        case JL_ROLE_FFN_UP: er = ctx->l_hidden; ec = d.dim; break;
        case JL_ROLE_FFN_DOWN: er = d.dim; ec = ctx->l_hidden; break;
        default: er = 1; ec = d.dim; norm = true; break;
    }
    JL_REQUIRE(ctx, rows == er && cols == ec, JL_ERR_INVALID,
               "role %d expects %lld x %lld, got %lld x %lld", role, (long long)er, (long long)ec,
               (long long)rows, (long long)cols);
    if (norm)
        JL_REQUIRE(ctx, ggml_type == kF32, JL_ERR_UNSUPPORTED, "norm weights must be F32, got type %d",
                   ggml_type);
    else
        JL_REQUIRE(ctx, is_quant(ggml_type) || (is_extra_quant(ggml_type) && ctx->tp_size == 1), JL_ERR_UNSUPPORTED,
                   "matrix role %d must be Q8_0, Q4_0 or Q4_K (on one GPU also Q4_1, Q5_K or Q6_K), got type %d", role,
                   ggml_type);
    int rc = check_shape(ctx, ggml_type, rows, cols, nbytes, /*stand_alone=*/true);
    if (rc) return rc;
    cudaSetDevice(ctx->device);
    drop_graphs(ctx);
    ctx->finalized = false;
    DevTensor *t = per_layer ? &ctx->layer[role][layer] : &ctx->global[role];
    return upload(ctx, t, ggml_type, rows, cols, host_bytes, nbytes);
}

int32_t jl_upload_rope(jl_ctx *ctx, const float *cos_table, const float *sin_table, int64_t n) {
    if (!ctx) return JL_ERR_INVALID;
    JL_REQUIRE(ctx, ctx->has_model, JL_ERR_STATE, "jl_model_create must come first");
    const int64_t need = int64_t(ctx->desc.ctx_len) * (ctx->desc.head_dim / 2);
    JL_REQUIRE(ctx, cos_table && sin_table && n == need, JL_ERR_INVALID,
               "RoPE tables must hold ctx_len * head_dim / 2 = %lld floats, got %lld",
               (long long)need, (long long)n);
    cudaSetDevice(ctx->device);
    if (!ctx->rope_cos) {
        int rc;
        if ((rc = dev_alloc(ctx, reinterpret_cast<void **>(&ctx->rope_cos), n * 4))) return rc;
        if ((rc = dev_alloc(ctx, reinterpret_cast<void **>(&ctx->rope_sin), n * 4))) return rc;
    }
    JL_CUDA(ctx, cudaMemcpyAsync(ctx->rope_cos, cos_table, n * 4, cudaMemcpyHostToDevice, ctx->stream));
    JL_CUDA(ctx, cudaMemcpyAsync(ctx->rope_sin, sin_table, n * 4, cudaMemcpyHostToDevice, ctx->stream));
    JL_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
    ctx->counters.h2d_bytes += n * 8;
    return JL_OK;
}

int32_t jl_model_finalize(jl_ctx *ctx) {
    if (!ctx) return JL_ERR_INVALID;
    JL_REQUIRE(ctx, ctx->has_model, JL_ERR_STATE, "jl_model_create must come first");
    const jl_model_desc &d = ctx->desc;
    JL_REQUIRE(ctx, ctx->global[JL_ROLE_TOKEN_EMBEDDING].data, JL_ERR_STATE, "token embedding missing");
    JL_REQUIRE(ctx, ctx->global[JL_ROLE_OUTPUT_NORM].data, JL_ERR_STATE, "output norm missing");
    JL_REQUIRE(ctx, d.tied_embeddings || ctx->global[JL_ROLE_OUTPUT].data, JL_ERR_STATE,
               "output.weight missing and embeddings are not tied");
    JL_REQUIRE(ctx, ctx->rope_cos != nullptr, JL_ERR_STATE, "RoPE tables missing");
    cudaSetDevice(ctx->device);
    if (ctx->x != nullptr) {
        // Finalised before, then a tensor was replaced: the old workspace goes first. (Under tensor
        // parallelism every rank must then finalise again: setting up the peer exchange is collective.)
        JL_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
        free_workspace(ctx);
    }
    if (ctx->tp_size > 1 && !ctx->global[JL_ROLE_OUTPUT].data) {
        const DevTensor &emb = ctx->global[JL_ROLE_TOKEN_EMBEDDING];
        if (emb.has_tmap) {
            const size_t rb = size_t(row_bytes(emb.type, emb.cols));
            JL_CUDA(ctx, gemm_make_tensor_map(&ctx->wcls_slice_tmap, emb.data + size_t(ctx->tp_rank) * ctx->l_vocab * rb,
                                              emb.type, ctx->l_vocab, emb.cols));
        }
    }
    bool mixed = false;
    static const int per_layer_roles[] = {JL_ROLE_ATTENTION_NORM,  JL_ROLE_ATTENTION_QUERY,
                                          JL_ROLE_ATTENTION_KEY,   JL_ROLE_ATTENTION_VALUE,
                                          JL_ROLE_ATTENTION_OUTPUT, JL_ROLE_FFN_NORM,
                                          JL_ROLE_FFN_GATE,        JL_ROLE_FFN_UP,
                                          JL_ROLE_FFN_DOWN};
    for (int l = 0; l < d.layers; ++l) {
        for (int r : per_layer_roles)
            JL_REQUIRE(ctx, ctx->layer[r][l].data, JL_ERR_STATE, "layer %d is missing tensor role %d", l, r);
        // The fused single-row kernels want every matrix in a format the mat-vec kernel reads (Q6_K among them
        // where rows are whole 16-byte pieces) and gate and up alike; a layer that is not makes the whole model
        // take the row path (one GPU only). Q, K and V of different types are launched one by one.
        if (ctx->layer[JL_ROLE_FFN_GATE][l].type != ctx->layer[JL_ROLE_FFN_UP][l].type) mixed = true;
        for (int r : per_layer_roles)
            if (!fused_path_takes(ctx->layer[r][l])) mixed = true;
    }
    // (a table that only serves the embedding kernel may have any type)
    if (ctx->global[JL_ROLE_OUTPUT].data ? !fused_path_takes(ctx->global[JL_ROLE_OUTPUT])
                                         : !fused_path_takes(ctx->global[JL_ROLE_TOKEN_EMBEDDING]))
        mixed = true;
    JL_REQUIRE(ctx, !mixed || ctx->tp_size == 1, JL_ERR_UNSUPPORTED,
               "tensor parallelism needs Q, K, V (gate, up) of one type per layer and no Q4_1 / Q5_K / Q6_K matrices");
    ctx->mixed = mixed;
    if (ctx->finalized) return JL_OK;
    cudaSetDevice(ctx->device);
    const size_t B = d.max_batch;
    // Rows per prompt chunk (JITLLM_B200_PREFILL_CHUNK: a multiple of 128 between 128 and 2048; default 512). A chunk's
    // attention walks all earlier keys again, so fewer, larger chunks ingest long prompts faster; the step buffers
    // grow with it.
    static const int kPrefillChunk = [] {
        const char *v = getenv("JITLLM_B200_PREFILL_CHUNK");
        const int c = v ? atoi(v) : 512;
        return c >= 128 && c <= 2048 && c % 128 == 0 ? c : 512;
    }();
    ctx->row_cap = d.max_batch > kPrefillChunk ? d.max_batch : kPrefillChunk;
    const size_t R = ctx->row_cap;
    int rc;
    size_t ws = 0;
    auto alloc = [&](void **p, size_t bytes) {
        ws += bytes;
        return dev_alloc(ctx, p, bytes);
    };
    // Key-range splits per launch width: a single row has (pos+1) keys to spread over ~2 CTAs per
    // SM; wide launches already fill the grid with rows.
    size_t max_row_splits = 1;
    for (int w = 1; w <= int(R); ++w) {
        const size_t v = size_t(w) * size_t(attn_splits_for_width(ctx, w));
        if (v > max_row_splits) max_row_splits = v;
    }
    ctx->attn_nsplit = attn_splits_for_width(ctx, 1);
    if ((rc = alloc(reinterpret_cast<void **>(&ctx->x), R * d.dim * 4))) return rc;
    if ((rc = alloc(reinterpret_cast<void **>(&ctx->q), R * ctx->l_qdim * 4))) return rc;
    if ((rc = alloc(reinterpret_cast<void **>(&ctx->k), R * ctx->kv_dim * 4))) return rc;
    if ((rc = alloc(reinterpret_cast<void **>(&ctx->v), R * ctx->kv_dim * 4))) return rc;
    if ((rc = alloc(reinterpret_cast<void **>(&ctx->xb), R * d.dim * 4))) return rc;
    if ((rc = alloc(reinterpret_cast<void **>(&ctx->hb), R * ctx->l_hidden * 4))) return rc;
    if ((rc = alloc(reinterpret_cast<void **>(&ctx->hb2), R * ctx->l_hidden * 4))) return rc;
    if ((rc = alloc(reinterpret_cast<void **>(&ctx->logits), B * ctx->l_vocab * 4))) return rc;
    {
        if ((rc = alloc(&ctx->xb16, 2 * R * d.dim * 2))) return rc;
        if ((rc = alloc(&ctx->hb16, 2 * R * ctx->l_hidden * 2))) return rc;
        const int nts[4] = {16, 32, 64, 128};
        for (int i = 0; i < 4; ++i) {
            JL_CUDA(ctx, gemm_make_activation_map(&ctx->xmaps[0][i], ctx->xb16, R, d.dim, nts[i]));
            JL_CUDA(ctx, gemm_make_activation_map(&ctx->xmaps[1][i], ctx->xb16, R, ctx->l_qdim, nts[i]));
            JL_CUDA(ctx, gemm_make_activation_map(&ctx->xmaps[2][i], ctx->hb16, R, ctx->l_hidden, nts[i]));
        }
    }
    if (ctx->tp_size > 1) {
        JL_REQUIRE(ctx, ctx->nccl_comm != nullptr, JL_ERR_STATE, "jl_tp_init must come before jl_model_finalize");
        if ((rc = alloc(reinterpret_cast<void **>(&ctx->part), R * d.dim * 4))) return rc;
        if ((rc = alloc(reinterpret_cast<void **>(&ctx->logits_all), B * d.vocab * 4))) return rc;
        JL_CUDA(ctx, cudaMemsetAsync(ctx->part, 0, R * d.dim * 4, ctx->stream));
        if ((rc = tp_push_setup(ctx))) return rc;
        if ((rc = alloc(reinterpret_cast<void **>(&ctx->best), (2 * R + 2 * R * ctx->tp_size) * 4))) return rc;
    }
    if ((rc = alloc(reinterpret_cast<void **>(&ctx->d_tokens), R * 4))) return rc;
    if ((rc = alloc(reinterpret_cast<void **>(&ctx->d_positions), R * 4))) return rc;
    if ((rc = alloc(reinterpret_cast<void **>(&ctx->d_slots), R * 4))) return rc;
    if ((rc = alloc(reinterpret_cast<void **>(&ctx->d_out), R * 4))) return rc;
    if ((rc = alloc(reinterpret_cast<void **>(&ctx->d_active), R))) return rc;
    if ((rc = alloc(reinterpret_cast<void **>(&ctx->att_partial),
                    max_row_splits * ctx->l_heads * (d.head_dim + 2) * 4)))
        return rc;
    if ((rc = alloc(reinterpret_cast<void **>(&ctx->att_count), R * ctx->l_kv_heads * 4))) return rc;
    if ((rc = alloc(reinterpret_cast<void **>(&ctx->amax_val), B * ctx->sm_count * 16))) return rc;
    if ((rc = alloc(reinterpret_cast<void **>(&ctx->amax_idx), B * ctx->sm_count * 16))) return rc;
    if ((rc = alloc(reinterpret_cast<void **>(&ctx->amax_count), B * 4))) return rc;
    JL_CUDA(ctx, cudaMemsetAsync(ctx->att_count, 0, R * ctx->l_kv_heads * 4, ctx->stream));
    JL_CUDA(ctx, cudaMemsetAsync(ctx->d_out, 0, R * 4, ctx->stream));
    JL_CUDA(ctx, cudaMemsetAsync(ctx->amax_count, 0, B * 4, ctx->stream));
    JL_CUDA(ctx, cudaMemsetAsync(ctx->d_active, 0, R, ctx->stream));
    JL_CUDA(ctx, cudaMallocHost(reinterpret_cast<void **>(&ctx->h_stage), (5 * R + 1) * 4));
    JL_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
    ctx->counters.workspace_bytes = ws;
    ctx->finalized = true;
    return JL_OK;
}

int32_t jl_kv_create(jl_ctx *ctx, int32_t total_blocks, int32_t blocks_per_slot, int32_t max_slots,
                     int32_t block_size_tokens, int32_t fp16_key_value) {
    if (!ctx) return JL_ERR_INVALID;
    JL_REQUIRE(ctx, ctx->has_model, JL_ERR_STATE, "jl_model_create must come first");
    // runtime/kv/KvStorageRequest.java:5-12: every pool dimension must be positive.
    JL_REQUIRE(ctx, total_blocks > 0 && blocks_per_slot > 0 && max_slots > 0 && block_size_tokens > 0,
               JL_ERR_INVALID,
               "every key/value pool dimension must be positive, got totalBlocks=%d blocksPerSlot=%d "
               "maxSlots=%d blockSizeTokens=%d",
               total_blocks, blocks_per_slot, max_slots, block_size_tokens);
    JL_REQUIRE(ctx, fp16_key_value != 0, JL_ERR_UNSUPPORTED, "fp32 key/value pages; the pool is fp16");
    cudaSetDevice(ctx->device);
    free_kv(ctx);
    const jl_model_desc &d = ctx->desc;
    // One block beyond the leasable range is the scratch block for UNMAPPED entries.
    const size_t elems = size_t(total_blocks + 1) * d.layers * block_size_tokens * ctx->kv_dim;
    int rc;
    if ((rc = dev_alloc(ctx, reinterpret_cast<void **>(&ctx->kpool), elems * 2))) return rc;
    if ((rc = dev_alloc(ctx, reinterpret_cast<void **>(&ctx->vpool), elems * 2))) {
        free_kv(ctx);
        return rc;
    }
    const size_t entries = size_t(max_slots) * blocks_per_slot;
    if ((rc = dev_alloc(ctx, reinterpret_cast<void **>(&ctx->block_table), entries * 4))) {
        free_kv(ctx);
        return rc;
    }
    JL_CUDA(ctx, cudaMemsetAsync(ctx->kpool, 0, elems * 2, ctx->stream));
    JL_CUDA(ctx, cudaMemsetAsync(ctx->vpool, 0, elems * 2, ctx->stream));
    ctx->total_blocks = total_blocks;
    ctx->blocks_per_slot = blocks_per_slot;
    ctx->max_slots = max_slots;
    ctx->block_tokens = block_size_tokens;
    ctx->host_table.assign(entries, total_blocks);  // everything unmapped -> scratch
    JL_CUDA(ctx, cudaMemcpyAsync(ctx->block_table, ctx->host_table.data(), entries * 4,
                                 cudaMemcpyHostToDevice, ctx->stream));
    JL_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
    ctx->counters.kv_bytes = elems * 4 + entries * 4;
    ctx->has_kv = true;
    return JL_OK;
}

int32_t jl_kv_publish_block_table(jl_ctx *ctx, const int32_t *table, int64_t n) {
    if (!ctx) return JL_ERR_INVALID;
    JL_REQUIRE(ctx, ctx->has_kv, JL_ERR_STATE, "this KV store is closed");
    const int64_t entries = int64_t(ctx->max_slots) * ctx->blocks_per_slot;
    JL_REQUIRE(ctx, table != nullptr && n == entries, JL_ERR_INVALID,
               "block table shape changed: manager has %lld entries, the device mirror has %lld",
               (long long)n, (long long)entries);
    for (int64_t i = 0; i < n; ++i) {
        const int32_t entry = table[i];
        JL_REQUIRE(ctx, entry >= -1 && entry < ctx->total_blocks, JL_ERR_INVALID,
                   "block table entry %lld = %d is outside the pool of %d blocks", (long long)i, entry,
                   ctx->total_blocks);
        ctx->host_table[i] = entry < 0 ? ctx->total_blocks : entry;  // UNMAPPED -> scratch block
    }
    cudaSetDevice(ctx->device);
    JL_CUDA(ctx, cudaMemcpyAsync(ctx->block_table, ctx->host_table.data(), n * 4,
                                 cudaMemcpyHostToDevice, ctx->stream));
    JL_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
    ctx->counters.h2d_bytes += n * 4;
    return JL_OK;
}

int32_t jl_kv_fill(jl_ctx *ctx, uint16_t half_bits) {
    if (!ctx) return JL_ERR_INVALID;
    JL_REQUIRE(ctx, ctx->has_kv, JL_ERR_STATE, "jl_kv_create must come first");
    cudaSetDevice(ctx->device);
    const size_t elems = size_t(ctx->total_blocks + 1) * ctx->desc.layers * ctx->block_tokens * ctx->kv_dim;
    const uint32_t word = uint32_t(half_bits) | (uint32_t(half_bits) << 16);
    JL_CUDA(ctx, fill_launch(reinterpret_cast<uint32_t *>(ctx->kpool), elems / 2, word, ctx->stream));
    JL_CUDA(ctx, fill_launch(reinterpret_cast<uint32_t *>(ctx->vpool), elems / 2, word, ctx->stream));
    JL_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
    return JL_OK;
}

int64_t jl_kv_bytes_per_block(jl_ctx *ctx) {
    if (!ctx || !ctx->has_kv) return 0;
    return 2LL * ctx->kv_dim * ctx->block_tokens * ctx->desc.layers * 2LL;
}

int32_t jl_kv_read_row(jl_ctx *ctx, int32_t which, int32_t slot, int32_t layer, int32_t pos,
                       uint16_t *out_halfs) {
    if (!ctx) return JL_ERR_INVALID;
    JL_REQUIRE(ctx, ctx->has_kv, JL_ERR_STATE, "this KV store is closed");
    JL_REQUIRE(ctx, out_halfs && slot >= 0 && slot < ctx->max_slots && layer >= 0 &&
                        layer < ctx->desc.layers && pos >= 0 &&
                        pos < ctx->blocks_per_slot * ctx->block_tokens,
               JL_ERR_INVALID, "slot/layer/pos out of range");
    const int64_t phys = ctx->host_table[size_t(slot) * ctx->blocks_per_slot + pos / ctx->block_tokens];
    const int64_t off = phys * (int64_t(ctx->desc.layers) * ctx->block_tokens * ctx->kv_dim) +
                        int64_t(layer) * ctx->block_tokens * ctx->kv_dim +
                        int64_t(pos % ctx->block_tokens) * ctx->kv_dim;
    cudaSetDevice(ctx->device);
    const __half *pool = which == 0 ? ctx->kpool : ctx->vpool;
    JL_CUDA(ctx, cudaMemcpyAsync(out_halfs, pool + off, size_t(ctx->kv_dim) * 2, cudaMemcpyDeviceToHost,
                                 ctx->stream));
    JL_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
    return JL_OK;
}

static int validate_rows(jl_ctx *ctx, int width, const int32_t *tokens, const int32_t *positions,
                         const int32_t *kv_slots, const uint8_t *active) {
    const jl_model_desc &d = ctx->desc;
    const int capacity = ctx->blocks_per_slot * ctx->block_tokens;
    for (int b = 0; b < width; ++b) {
        if (active && !active[b]) continue;
        JL_REQUIRE(ctx, tokens[b] >= 0 && tokens[b] < d.vocab, JL_ERR_INVALID,
                   "row %d: token %d outside vocabulary of %d", b, tokens[b], d.vocab);
        JL_REQUIRE(ctx, positions[b] >= 0 && positions[b] < d.ctx_len && positions[b] < capacity,
                   JL_ERR_INVALID, "row %d: position %d outside context %d / slot capacity %d", b,
                   positions[b], d.ctx_len, capacity);
        JL_REQUIRE(ctx, kv_slots[b] >= 0 && kv_slots[b] < ctx->max_slots, JL_ERR_INVALID,
                   "row %d: kv slot %d outside 0..%d", b, kv_slots[b], ctx->max_slots - 1);
        for (int c = b + 1; c < width; ++c)
            JL_REQUIRE(ctx, (active && !active[c]) || kv_slots[c] != kv_slots[b], JL_ERR_INVALID,
                       "rows %d and %d share kv slot %d in one step", b, c, kv_slots[b]);
    }
    return JL_OK;
}

int32_t jl_decode(jl_ctx *ctx, int32_t width, const int32_t *tokens, const int32_t *positions,
                  const int32_t *kv_slots, const uint8_t *active, int32_t *out_tokens,
                  float *out_logits) {
    if (!ctx) return JL_ERR_INVALID;
    JL_REQUIRE(ctx, ctx->finalized, JL_ERR_STATE, "jl_model_finalize must come first");
    JL_REQUIRE(ctx, ctx->has_kv, JL_ERR_STATE, "jl_kv_create must come first");
    JL_REQUIRE(ctx, width >= 1 && width <= ctx->desc.max_batch, JL_ERR_INVALID,
               "a batch is fixed width: got %d, this context was sized for 1..%d", width,
               ctx->desc.max_batch);
    JL_REQUIRE(ctx, tokens && positions && kv_slots && out_tokens, JL_ERR_INVALID,
               "tokens, positions, kv_slots and out_tokens must not be NULL");
    int rc = validate_rows(ctx, width, tokens, positions, kv_slots, active);
    if (rc) return rc;
    cudaSetDevice(ctx->device);
    const size_t B = ctx->row_cap;
    int32_t *h_tok = ctx->h_stage, *h_pos = h_tok + B, *h_slot = h_pos + B, *h_out = h_slot + B;
    uint8_t *h_act = reinterpret_cast<uint8_t *>(h_out + B);
    int32_t *h_status = ctx->h_stage + 5 * B;
    for (int b = 0; b < width; ++b) {
        const bool on = !active || active[b];
        h_tok[b] = on ? tokens[b] : 0;
        h_pos[b] = on ? positions[b] : 0;
        h_slot[b] = on ? kv_slots[b] : 0;
        h_act[b] = on ? 1 : 0;
    }
    bool any = false;
    for (int b = 0; b < width; ++b) any = any || h_act[b];
    if (!any) {
        for (int b = 0; b < width; ++b) out_tokens[b] = -1;
        return JL_OK;
    }
    JL_CUDA(ctx, cudaEventRecord(ctx->ev0, ctx->stream));
    JL_CUDA(ctx, cudaMemcpyAsync(ctx->d_tokens, h_tok, width * 4, cudaMemcpyHostToDevice, ctx->stream));
    JL_CUDA(ctx, cudaMemcpyAsync(ctx->d_positions, h_pos, width * 4, cudaMemcpyHostToDevice, ctx->stream));
    JL_CUDA(ctx, cudaMemcpyAsync(ctx->d_slots, h_slot, width * 4, cudaMemcpyHostToDevice, ctx->stream));
    JL_CUDA(ctx, cudaMemcpyAsync(ctx->d_active, h_act, width, cudaMemcpyHostToDevice, ctx->stream));
    if ((rc = run_step(ctx, width, true, false))) return rc;
    JL_CUDA(ctx, cudaMemcpyAsync(h_out, ctx->d_out, width * 4, cudaMemcpyDeviceToHost, ctx->stream));
    JL_CUDA(ctx, cudaMemcpyAsync(h_status, ctx->d_status, 4, cudaMemcpyDeviceToHost, ctx->stream));
    std::vector<float> gathered;
    if (out_logits && ctx->tp_size > 1) {
        // Every rank holds [row][l_vocab]; gather them as [rank][row][l_vocab] and let the host
        // interleave them into rows of the full vocabulary after the synchronise.
        const size_t shard = size_t(width) * ctx->l_vocab;
        gathered.resize(shard * ctx->tp_size);
        const int nrc = g_nccl.AllGather(ctx->logits, ctx->logits_all, shard, kNcclFloat32, ctx->nccl_comm,
                                         ctx->stream);
        if (nrc != 0) return fail(ctx, JL_ERR_CUDA, "ncclAllGather failed: %s", g_nccl.GetErrorString(nrc));
        JL_CUDA(ctx, cudaMemcpyAsync(gathered.data(), ctx->logits_all, shard * ctx->tp_size * 4,
                                     cudaMemcpyDeviceToHost, ctx->stream));
    } else if (out_logits) {
        JL_CUDA(ctx, cudaMemcpyAsync(out_logits, ctx->logits, size_t(width) * ctx->desc.vocab * 4,
                                     cudaMemcpyDeviceToHost, ctx->stream));
    }
    JL_CUDA(ctx, cudaEventRecord(ctx->ev1, ctx->stream));
    JL_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
    if ((rc = check_status(ctx))) return rc;
    for (int b = 0; b < width; ++b) out_tokens[b] = h_act[b] ? h_out[b] : -1;
    if (out_logits && ctx->tp_size > 1) {
        for (int k = 0; k < ctx->tp_size; ++k)
            for (int b = 0; b < width; ++b)
                memcpy(out_logits + size_t(b) * ctx->desc.vocab + size_t(k) * ctx->l_vocab,
                       gathered.data() + (size_t(k) * width + b) * ctx->l_vocab, size_t(ctx->l_vocab) * 4);
    }
    cudaEventElapsedTime(&ctx->counters.last_step_ms, ctx->ev0, ctx->ev1);
    ctx->logits_rows = width;
    ctx->counters.decode_calls++;
    ctx->counters.h2d_bytes += width * 13;
    ctx->counters.d2h_bytes += width * 4 + 4 + (out_logits ? size_t(width) * ctx->desc.vocab * 4 : 0);
    return JL_OK;
}

int32_t jl_sample(jl_ctx *ctx, int32_t width, float temperature, float topp, const float *uniforms, int32_t *out_tokens) {
    if (!ctx) return JL_ERR_INVALID;
    JL_REQUIRE(ctx, ctx->finalized && ctx->has_kv, JL_ERR_STATE, "jl_model_finalize and jl_kv_create must come first");
    JL_REQUIRE(ctx, uniforms && out_tokens, JL_ERR_INVALID, "uniforms and out_tokens must not be NULL");
    JL_REQUIRE(ctx, temperature > 0.0f, JL_ERR_INVALID,
               "temperature must be positive: temperature 0 is greedy decoding, which jl_decode already returns");
    JL_REQUIRE(ctx, ctx->tp_size == 1, JL_ERR_UNSUPPORTED,
               "device-side sampling needs the whole row of logits on one GPU: not available under tensor parallelism");
    JL_REQUIRE(ctx, width >= 1 && width == ctx->logits_rows, JL_ERR_STATE,
               "jl_sample(width = %d) must follow a jl_decode of the same width (last: %d rows of logits)", width,
               ctx->logits_rows);
    for (int b = 0; b < width; ++b)
        JL_REQUIRE(ctx, uniforms[b] >= 0.0f && uniforms[b] < 1.0f, JL_ERR_INVALID, "uniforms[%d] = %g outside [0, 1)", b,
                   double(uniforms[b]));
    cudaSetDevice(ctx->device);
    if (!ctx->d_uniforms) {
        int rc = dev_alloc(ctx, reinterpret_cast<void **>(&ctx->d_uniforms), size_t(ctx->row_cap) * 4);
        if (rc) return rc;
        ctx->user_allocs.push_back(ctx->d_uniforms);  // released with the context
        JL_CUDA(ctx, sample_rows_configure());
    }
    float *h_u = reinterpret_cast<float *>(ctx->h_stage);
    int32_t *h_out = ctx->h_stage + 3 * size_t(ctx->row_cap);
    memcpy(h_u, uniforms, size_t(width) * 4);
    JL_CUDA(ctx, cudaEventRecord(ctx->ev0, ctx->stream));
    JL_CUDA(ctx, cudaMemcpyAsync(ctx->d_uniforms, h_u, size_t(width) * 4, cudaMemcpyHostToDevice, ctx->stream));
    cudaError_t e = sample_rows_launch(ctx->logits, ctx->desc.vocab, width, ctx->d_active, temperature, topp, ctx->d_uniforms,
                                       ctx->d_out, ctx->d_out, ctx->stream);  // d_out: the step's arg-max in, the sample out
    if (e != cudaSuccess) return fail(ctx, JL_ERR_CUDA, "sampling launch failed: %s", cudaGetErrorString(e));
    ctx->counters.kernel_launches += 1;
    JL_CUDA(ctx, cudaMemcpyAsync(h_out, ctx->d_out, size_t(width) * 4, cudaMemcpyDeviceToHost, ctx->stream));
    JL_CUDA(ctx, cudaEventRecord(ctx->ev1, ctx->stream));
    JL_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
    for (int b = 0; b < width; ++b) out_tokens[b] = h_out[b];
    cudaEventElapsedTime(&ctx->counters.last_step_ms, ctx->ev0, ctx->ev1);
    ctx->logits_rows = 0;  // the rows now hold exp(score - max), not logits
    ctx->counters.h2d_bytes += size_t(width) * 4;
    ctx->counters.d2h_bytes += size_t(width) * 4;
    return JL_OK;
}

int32_t jl_prefill(jl_ctx *ctx, int32_t kv_slot, const int32_t *tokens, int32_t start_pos, int32_t n) {
    if (!ctx) return JL_ERR_INVALID;
    JL_REQUIRE(ctx, ctx->finalized, JL_ERR_STATE, "jl_model_finalize must come first");
    JL_REQUIRE(ctx, ctx->has_kv, JL_ERR_STATE, "jl_kv_create must come first");
    JL_REQUIRE(ctx, tokens != nullptr && n >= 0 && start_pos >= 0, JL_ERR_INVALID,
               "tokens must not be NULL, n and start_pos must not be negative");
    if (n == 0) return JL_OK;
    cudaSetDevice(ctx->device);
    const size_t B = ctx->row_cap;
    int32_t *h_tok = ctx->h_stage, *h_pos = h_tok + B, *h_slot = h_pos + B, *h_out = h_slot + B;
    uint8_t *h_act = reinterpret_cast<uint8_t *>(h_out + B);
    int32_t *h_status = ctx->h_stage + 5 * B;
    JL_CUDA(ctx, cudaEventRecord(ctx->ev0, ctx->stream));
    {
        const int32_t first = tokens[0], last_pos = start_pos + n - 1;
        const uint8_t on = 1;
        int rc = validate_rows(ctx, 1, &first, &last_pos, &kv_slot, &on);
        if (rc) return rc;
        for (int i = 0; i < n; ++i)
            JL_REQUIRE(ctx, tokens[i] >= 0 && tokens[i] < ctx->desc.vocab, JL_ERR_INVALID,
                       "prompt token %d = %d outside vocabulary of %d", i, tokens[i], ctx->desc.vocab);
    }
    static const int rows_min = [] { const char *v = getenv("JITLLM_B200_GEMM_MIN_WIDTH"); return v ? atoi(v) : 4; }();
    // Chunks of up to row_cap tokens through the tensor-core path (every projection one
    // matrix-matrix launch, as TornadoBatchPrefillPass does per chunk,
    // backend/tornado/TornadoBatchPrefillPass.java:104-141); a short tail goes token by token.
    // The values are those of batchForwardJavaPrefill: the per-token layer stack, no logits.
    int done = 0;
    while (done < n) {
        int chunk = n - done;
        if (chunk > ctx->row_cap) chunk = ctx->row_cap;
        if (chunk < rows_min) chunk = 1;
        for (int i = 0; i < chunk; ++i) {
            h_tok[i] = tokens[done + i];
            h_pos[i] = start_pos + done + i;
            h_slot[i] = kv_slot;
            h_act[i] = 1;
        }
        JL_CUDA(ctx, cudaMemcpyAsync(ctx->d_tokens, h_tok, chunk * 4, cudaMemcpyHostToDevice, ctx->stream));
        JL_CUDA(ctx, cudaMemcpyAsync(ctx->d_positions, h_pos, chunk * 4, cudaMemcpyHostToDevice, ctx->stream));
        JL_CUDA(ctx, cudaMemcpyAsync(ctx->d_slots, h_slot, chunk * 4, cudaMemcpyHostToDevice, ctx->stream));
        JL_CUDA(ctx, cudaMemcpyAsync(ctx->d_active, h_act, chunk, cudaMemcpyHostToDevice, ctx->stream));
        int rc;
        if (chunk == 1) {
            rc = run_step(ctx, 1, false, false);
        } else {
            uint64_t launches = 0;
            rc = enqueue_rows_step(ctx, chunk, false, false, &launches, false);
            ctx->counters.kernel_launches += launches;
        }
        if (rc) return rc;
        // The staging words are reused by the next chunk's copies.
        JL_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
        done += chunk;
    }
    JL_CUDA(ctx, cudaMemcpyAsync(h_status, ctx->d_status, 4, cudaMemcpyDeviceToHost, ctx->stream));
    JL_CUDA(ctx, cudaEventRecord(ctx->ev1, ctx->stream));
    JL_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
    int rc = check_status(ctx);
    if (rc) return rc;
    cudaEventElapsedTime(&ctx->counters.last_step_ms, ctx->ev0, ctx->ev1);
    ctx->counters.prefill_calls++;
    ctx->counters.h2d_bytes += size_t(n) * 13;
    return JL_OK;
}

int32_t jl_generate(jl_ctx *ctx, int32_t width, const int32_t *tokens, const int32_t *positions,
                    const int32_t *kv_slots, const uint8_t *active, int32_t n_steps,
                    int32_t *out_history) {
    if (!ctx) return JL_ERR_INVALID;
    JL_REQUIRE(ctx, ctx->finalized, JL_ERR_STATE, "jl_model_finalize must come first");
    JL_REQUIRE(ctx, ctx->has_kv, JL_ERR_STATE, "jl_kv_create must come first");
    JL_REQUIRE(ctx, width >= 1 && width <= ctx->desc.max_batch, JL_ERR_INVALID,
               "a batch is fixed width: got %d, this context was sized for 1..%d", width,
               ctx->desc.max_batch);
    JL_REQUIRE(ctx, tokens && positions && kv_slots && out_history && n_steps >= 0, JL_ERR_INVALID,
               "NULL argument or negative step count");
    if (n_steps == 0) return JL_OK;
    int rc = validate_rows(ctx, width, tokens, positions, kv_slots, active);
    if (rc) return rc;
    const int capacity = ctx->blocks_per_slot * ctx->block_tokens;
    for (int b = 0; b < width; ++b) {
        if (active && !active[b]) continue;
        const int last = positions[b] + n_steps - 1;
        JL_REQUIRE(ctx, last < ctx->desc.ctx_len && last < capacity, JL_ERR_INVALID,
                   "row %d: %d steps from position %d run past context %d / slot capacity %d", b,
                   n_steps, positions[b], ctx->desc.ctx_len, capacity);
    }
    cudaSetDevice(ctx->device);
    const size_t need = size_t(n_steps) * width;
    if (need > ctx->history_cap) {
        drop_graphs(ctx);  // captured graphs hold the old history pointer
        if (ctx->d_history) cudaFree(ctx->d_history);
        ctx->d_history = nullptr;
        ctx->history_cap = 0;
        if ((rc = dev_alloc(ctx, reinterpret_cast<void **>(&ctx->d_history), need * 4))) return rc;
        ctx->history_cap = need;
    }
    if (!ctx->d_step && (rc = dev_alloc(ctx, reinterpret_cast<void **>(&ctx->d_step), 4))) return rc;
    const size_t B = ctx->row_cap;
    int32_t *h_tok = ctx->h_stage, *h_pos = h_tok + B, *h_slot = h_pos + B, *h_out = h_slot + B;
    uint8_t *h_act = reinterpret_cast<uint8_t *>(h_out + B);
    int32_t *h_status = ctx->h_stage + 5 * B;
    for (int b = 0; b < width; ++b) {
        const bool on = !active || active[b];
        h_tok[b] = on ? tokens[b] : 0;
        h_pos[b] = on ? positions[b] : 0;
        h_slot[b] = on ? kv_slots[b] : 0;
        h_act[b] = on ? 1 : 0;
    }
    bool any = false;
    for (int b = 0; b < width; ++b) any = any || h_act[b];
    if (!any) {
        for (size_t i = 0; i < need; ++i) out_history[i] = -1;
        return JL_OK;
    }
    JL_CUDA(ctx, cudaEventRecord(ctx->ev0, ctx->stream));
    JL_CUDA(ctx, cudaMemcpyAsync(ctx->d_tokens, h_tok, width * 4, cudaMemcpyHostToDevice, ctx->stream));
    JL_CUDA(ctx, cudaMemcpyAsync(ctx->d_positions, h_pos, width * 4, cudaMemcpyHostToDevice, ctx->stream));
    JL_CUDA(ctx, cudaMemcpyAsync(ctx->d_slots, h_slot, width * 4, cudaMemcpyHostToDevice, ctx->stream));
    JL_CUDA(ctx, cudaMemcpyAsync(ctx->d_active, h_act, width, cudaMemcpyHostToDevice, ctx->stream));
    JL_CUDA(ctx, cudaMemsetAsync(ctx->d_step, 0, 4, ctx->stream));
    for (int s = 0; s < n_steps; ++s)
        if ((rc = run_step(ctx, width, true, true))) return rc;
    JL_CUDA(ctx, cudaMemcpyAsync(out_history, ctx->d_history, need * 4, cudaMemcpyDeviceToHost, ctx->stream));
    JL_CUDA(ctx, cudaMemcpyAsync(h_status, ctx->d_status, 4, cudaMemcpyDeviceToHost, ctx->stream));
    JL_CUDA(ctx, cudaEventRecord(ctx->ev1, ctx->stream));
    JL_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
    if ((rc = check_status(ctx))) return rc;
    cudaEventElapsedTime(&ctx->counters.last_step_ms, ctx->ev0, ctx->ev1);
    ctx->counters.decode_calls += n_steps;
    ctx->counters.h2d_bytes += width * 13;
    ctx->counters.d2h_bytes += need * 4 + 4;
    return JL_OK;
}

int32_t jl_debug_trace(jl_ctx *ctx, uint64_t *out, int32_t max_records) {
    if (!ctx) return JL_ERR_INVALID;
#ifndef JL_TRACE
    (void)out;
    (void)max_records;
    return fail(ctx, JL_ERR_UNSUPPORTED, "this build of the library records no launch timeline (build with --trace)");
#else
    constexpr unsigned kCap = 16384;
    cudaSetDevice(ctx->device);
    if (!out) {  // arm: later launches record stamps
        if (!ctx->d_trace) {
            int rc = dev_alloc(ctx, reinterpret_cast<void **>(&ctx->d_trace), (size_t(kCap + 1) * kTraceWords + kTraceClasses * kTraceCtaMax * kTraceCtaWords) * 8);
            if (rc) return rc;
            ctx->user_allocs.push_back(ctx->d_trace);  // released with the context
            const char *mv = getenv("JITLLM_B200_TRACE_MODE");
            const int mode = mv ? atoi(mv) : 0;
            JL_CUDA(ctx, gemv_trace_bind(ctx->d_trace, kCap, mode));
            JL_CUDA(ctx, ops_trace_bind(ctx->d_trace, kCap, mode));
            JL_CUDA(ctx, gemm_trace_bind(ctx->d_trace, kCap, mode));
        }
        JL_CUDA(ctx, cudaMemsetAsync(ctx->d_trace, 0, (size_t(kCap + 1) * kTraceWords + kTraceClasses * kTraceCtaMax * kTraceCtaWords) * 8, ctx->stream));
        JL_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
        return int32_t(kCap);
    }
    JL_REQUIRE(ctx, ctx->d_trace != nullptr, JL_ERR_STATE, "the trace was not armed");
    unsigned long long n = 0;
    JL_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
    JL_CUDA(ctx, cudaMemcpy(&n, ctx->d_trace, 8, cudaMemcpyDeviceToHost));
    if (n > kCap) n = kCap;
    if (n > (unsigned long long)max_records) n = max_records;
    if (max_records < 0) {  // the per-CTA cells of the latest launch instead of the records
        JL_CUDA(ctx, cudaMemcpy(out, ctx->d_trace + size_t(kCap + 1) * kTraceWords, kTraceClasses * kTraceCtaMax * kTraceCtaWords * 8, cudaMemcpyDeviceToHost));
        return kTraceClasses * kTraceCtaMax;
    }
    JL_CUDA(ctx, cudaMemcpy(out, ctx->d_trace + kTraceWords, size_t(n) * kTraceWords * 8, cudaMemcpyDeviceToHost));
    return int32_t(n);
#endif
}

int32_t jl_bench_op(jl_ctx *ctx, int32_t op, int32_t first_layer, int32_t iters) {
    if (!ctx) return JL_ERR_INVALID;
    JL_REQUIRE(ctx, ctx->finalized, JL_ERR_STATE, "jl_model_finalize must come first");
    JL_REQUIRE(ctx, op >= 0 && op <= 5 && iters >= 0 && first_layer >= 0, JL_ERR_INVALID,
               "op must be 0..5 (qkv, attn-out, gate/up, down, vocabulary, attention)");
    JL_REQUIRE(ctx, op != 5 || ctx->has_kv, JL_ERR_STATE, "the attention operator needs jl_kv_create first");
    cudaSetDevice(ctx->device);
    const jl_model_desc &d = ctx->desc;
    uint64_t launches = 0;
    for (int i = 0; i < iters; ++i) {
        const int l = (first_layer + i) % d.layers;
        if (op == 5) {
            // Row 0 at the position and slot the last step left on the device: rotates and appends
            // whatever the q/k/v buffers hold, then attends over the slot's pages of layer l.
            AttnArgs t = {};
            t.q = ctx->q;
            t.k = ctx->k;
            t.v = ctx->v;
            t.out = ctx->xb;
            t.rope_cos = ctx->rope_cos;
            t.rope_sin = ctx->rope_sin;
            t.positions = ctx->d_positions;
            t.slots = ctx->d_slots;
            t.active = nullptr;
            t.kv = {ctx->kpool, ctx->vpool, ctx->block_table, ctx->blocks_per_slot, ctx->block_tokens, d.layers,
                    ctx->kv_dim};
            t.layer = l;
            t.heads = ctx->l_heads;
            t.kv_heads = ctx->l_kv_heads;
            t.head_dim = d.head_dim;
            t.dim = ctx->l_qdim;
            t.nsplit = attn_splits_for_width(ctx, 1);
            t.append = 1;
            t.partial = ctx->att_partial;
            t.counters = ctx->att_count;
            cudaError_t e = attention_launch(t, 1, ctx->stream, ctx->use_pdl);
            if (e != cudaSuccess) return fail(ctx, JL_ERR_CUDA, "attention launch failed: %s", cudaGetErrorString(e));
            ++launches;
            continue;
        }
        GemvArgs a = {};
        a.cols = d.dim;
        a.mode = kGemvPlain;
        a.eps = d.rms_eps;
        int total = 0;
        if (op == 0) {
            const DevTensor &wq = ctx->layer[JL_ROLE_ATTENTION_QUERY][l];
            const DevTensor &wk = ctx->layer[JL_ROLE_ATTENTION_KEY][l];
            const DevTensor &wv = ctx->layer[JL_ROLE_ATTENTION_VALUE][l];
            a.nseg = 3;
            a.seg[0] = {wq.mv(), ctx->q, nullptr, int(wq.rows)};
            a.seg[1] = {wk.mv(), ctx->k, nullptr, int(wk.rows)};
            a.seg[2] = {wv.mv(), ctx->v, nullptr, int(wv.rows)};
            a.type = wq.type;
            a.x = ctx->x;
            a.norm_w = reinterpret_cast<const float *>(ctx->layer[JL_ROLE_ATTENTION_NORM][l].data);
            total = int(wq.rows + wk.rows + wv.rows);
        } else if (op == 1) {
            const DevTensor &wo = ctx->layer[JL_ROLE_ATTENTION_OUTPUT][l];
            a.nseg = 1;
            a.seg[0] = {wo.mv(), ctx->tp_size > 1 ? ctx->part : ctx->q, nullptr, int(wo.rows)};
            a.cols = int(wo.cols);
            a.type = wo.type;
            a.x = ctx->xb;
            total = int(wo.rows);
        } else if (op == 2) {
            const DevTensor &w1 = ctx->layer[JL_ROLE_FFN_GATE][l];
            const DevTensor &w3 = ctx->layer[JL_ROLE_FFN_UP][l];
            a.nseg = 2;
            a.seg[0] = {w1.mv(), ctx->hb, nullptr, int(w1.rows)};
            a.seg[1] = {w3.mv(), nullptr, nullptr, int(w3.rows)};
            a.type = w1.type;
            a.mode = kGemvGateUp;
            a.x = ctx->x;
            a.norm_w = reinterpret_cast<const float *>(ctx->layer[JL_ROLE_FFN_NORM][l].data);
            total = int(w1.rows + w3.rows);
        } else if (op == 3) {
            const DevTensor &w2 = ctx->layer[JL_ROLE_FFN_DOWN][l];
            a.nseg = 1;
            a.seg[0] = {w2.mv(), ctx->tp_size > 1 ? ctx->part : ctx->q, nullptr, int(w2.rows)};
            a.cols = int(w2.cols);
            a.type = w2.type;
            a.x = ctx->hb;
            total = int(w2.rows);
        } else {
            const DevTensor wc = wcls_of(ctx);
            a.nseg = 1;
            a.seg[0] = {wc.mv(), ctx->logits, nullptr, int(wc.rows)};
            a.type = wc.type;
            a.x = ctx->x;
            a.norm_w = reinterpret_cast<const float *>(ctx->global[JL_ROLE_OUTPUT_NORM].data);
            total = int(wc.rows);
        }
        int rc = launch_gemv(ctx, a, total, &launches);
        if (rc) return rc;
    }
    ctx->counters.kernel_launches += launches;
    return JL_OK;
}

int32_t jl_debug_read(jl_ctx *ctx, const char *name, int32_t row, float *out, int64_t n) {
    if (!ctx) return JL_ERR_INVALID;
    JL_REQUIRE(ctx, ctx->finalized, JL_ERR_STATE, "jl_model_finalize must come first");
    JL_REQUIRE(ctx, name && out && row >= 0 && row < ctx->desc.max_batch, JL_ERR_INVALID,
               "bad name, out or row");
    const jl_model_desc &d = ctx->desc;
    const float *src = nullptr;
    int64_t width = 0;
    if (!strcmp(name, "x")) { src = ctx->x; width = d.dim; }
    else if (!strcmp(name, "q")) { src = ctx->q; width = ctx->l_qdim; }
    else if (!strcmp(name, "k")) { src = ctx->k; width = ctx->kv_dim; }
    else if (!strcmp(name, "v")) { src = ctx->v; width = ctx->kv_dim; }
    else if (!strcmp(name, "xb")) { src = ctx->xb; width = d.dim; }
    else if (!strcmp(name, "hb")) { src = ctx->hb; width = ctx->l_hidden; }
    else if (!strcmp(name, "logits")) { src = ctx->logits; width = ctx->l_vocab; }
    JL_REQUIRE(ctx, src != nullptr, JL_ERR_INVALID, "unknown buffer '%s'", name);
    JL_REQUIRE(ctx, n >= 0 && n <= width, JL_ERR_INVALID, "buffer '%s' has %lld floats per row", name,
               (long long)width);
    cudaSetDevice(ctx->device);
    JL_CUDA(ctx, cudaMemcpyAsync(out, src + size_t(row) * width, n * 4, cudaMemcpyDeviceToHost, ctx->stream));
    JL_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
    return JL_OK;
}

// ---- standalone operators ---------------------------------------------------------------------

int32_t jl_dequant(jl_ctx *ctx, int32_t ggml_type, const void *blocks, int64_t n_elements, float *out) {
    if (!ctx) return JL_ERR_INVALID;
    JL_REQUIRE(ctx, n_elements >= 0, JL_ERR_INVALID, "n_elements must not be negative");
    if (n_elements == 0) return JL_OK;
    JL_REQUIRE(ctx, blocks && out, JL_ERR_INVALID, "blocks and out must not be NULL");
    JL_REQUIRE(ctx, is_quant(ggml_type) || is_extra_quant(ggml_type), JL_ERR_UNSUPPORTED,
               "GGML type %d (supported: Q4_0=2, Q4_1=3, Q8_0=8, Q4_K=12, Q5_K=13, Q6_K=14)", ggml_type);
    const int blk = block_elements(ggml_type);
    JL_REQUIRE(ctx, n_elements % blk == 0, JL_ERR_INVALID,
               "n_elements (%lld) must be a whole number of %d-element blocks", (long long)n_elements, blk);
    cudaSetDevice(ctx->device);
    const size_t in_bytes = size_t(row_bytes(ggml_type, n_elements));
    void *d_in = nullptr, *d_out = nullptr;
    int rc;
    if ((rc = dev_alloc(ctx, &d_in, in_bytes))) return rc;
    if ((rc = dev_alloc(ctx, &d_out, size_t(n_elements) * 4))) {
        cudaFree(d_in);
        return rc;
    }
    cudaError_t e = cudaMemcpyAsync(d_in, blocks, in_bytes, cudaMemcpyHostToDevice, ctx->stream);
    if (e == cudaSuccess)
        e = dequant_launch(ggml_type, static_cast<uint8_t *>(d_in), n_elements,
                           static_cast<float *>(d_out), ctx->stream);
    if (e == cudaSuccess)
        e = cudaMemcpyAsync(out, d_out, size_t(n_elements) * 4, cudaMemcpyDeviceToHost, ctx->stream);
    if (e == cudaSuccess) e = cudaStreamSynchronize(ctx->stream);
    cudaFree(d_in);
    cudaFree(d_out);
    if (e != cudaSuccess) return fail(ctx, JL_ERR_CUDA, "dequant failed: %s", cudaGetErrorString(e));
    ctx->counters.kernel_launches++;
    ctx->counters.h2d_bytes += in_bytes;
    ctx->counters.d2h_bytes += size_t(n_elements) * 4;
    return JL_OK;
}

int32_t jl_tensor_upload(jl_ctx *ctx, int32_t ggml_type, int64_t rows, int64_t cols,
                         const void *host_bytes, size_t nbytes, jl_tensor **out) {
    if (!ctx) return JL_ERR_INVALID;
    JL_REQUIRE(ctx, out != nullptr && host_bytes != nullptr, JL_ERR_INVALID, "NULL argument");
    *out = nullptr;
    JL_REQUIRE(ctx, is_quant(ggml_type) || is_extra_quant(ggml_type), JL_ERR_UNSUPPORTED,
               "GGML type %d (supported: Q4_0=2, Q4_1=3, Q8_0=8, Q4_K=12, Q5_K=13, Q6_K=14)", ggml_type);
    int rc = check_shape(ctx, ggml_type, rows, cols, nbytes, /*stand_alone=*/true);
    if (rc) return rc;
    JL_REQUIRE(ctx, rows <= INT32_MAX && cols <= INT32_MAX, JL_ERR_UNSUPPORTED, "matrix too large");
    cudaSetDevice(ctx->device);
    jl_tensor *t = new jl_tensor();
    rc = upload(ctx, &t->t, ggml_type, rows, cols, host_bytes, nbytes);
    if (rc) {
        delete t;
        return rc;
    }
    *out = t;
    return JL_OK;
}

int32_t jl_tensor_free(jl_ctx *ctx, jl_tensor *t) {
    if (!ctx || !t) return JL_OK;
    cudaSetDevice(ctx->device);
    cudaStreamSynchronize(ctx->stream);
    if (t->t.data) {
        ctx->counters.weight_bytes -= t->t.bytes + t->t.padded_bytes;
        release_tensor(&t->t);
    }
    delete t;
    return JL_OK;
}

int32_t jl_gemv_dev(jl_ctx *ctx, const jl_tensor *w, const float *x_dev, int32_t n, float *y_dev) {
    if (!ctx) return JL_ERR_INVALID;
    JL_REQUIRE(ctx, w && x_dev && y_dev, JL_ERR_INVALID, "NULL argument");
    JL_REQUIRE(ctx, n >= 0, JL_ERR_INVALID, "n must not be negative");
    // The kernels read activation rows with 16-byte loads (rows are a multiple of 256 floats long, so
    // every row of an aligned buffer is aligned); a pointer that breaks that would fault on the device.
    JL_REQUIRE(ctx, reinterpret_cast<uintptr_t>(x_dev) % 16 == 0 && reinterpret_cast<uintptr_t>(y_dev) % 16 == 0,
               JL_ERR_INVALID, "x_dev and y_dev must be 16-byte aligned");
    cudaSetDevice(ctx->device);
    uint64_t launches = 0;
    static const int gemm_min_n = [] { const char *v = getenv("JITLLM_B200_GEMM_MIN_N"); return v ? atoi(v) : 8; }();
    if (n >= gemm_min_n && w->t.has_tmap) {
        // Wide enough for the tensor cores: one tcgen05 matrix-matrix launch.
        int rc = launch_gemm(ctx, w->t, x_dev, n, y_dev, nullptr, &launches);
        ctx->counters.kernel_launches += launches;
        return rc;
    }
    for (int b = 0; b < n; ++b) {
        GemvArgs a = {};
        a.nseg = 1;
        a.seg[0] = {w->t.mv(), y_dev + size_t(b) * w->t.rows, nullptr, int(w->t.rows)};
        a.cols = int(w->t.cols);
        a.type = w->t.type;
        a.mode = kGemvPlain;
        a.x = x_dev + size_t(b) * w->t.cols;
        int rc = launch_gemv(ctx, a, int(w->t.rows), &launches);
        if (rc) return rc;
    }
    ctx->counters.kernel_launches += launches;
    return JL_OK;
}

int32_t jl_gemv(jl_ctx *ctx, int32_t ggml_type, int64_t rows, int64_t cols, const void *w_host,
                const float *x_host, int32_t n, float *y_host) {
    if (!ctx) return JL_ERR_INVALID;
    JL_REQUIRE(ctx, w_host && x_host && y_host, JL_ERR_INVALID, "NULL argument");
    JL_REQUIRE(ctx, n >= 0, JL_ERR_INVALID, "n must not be negative");
    JL_REQUIRE(ctx, is_quant(ggml_type) || is_extra_quant(ggml_type), JL_ERR_UNSUPPORTED,
               "GGML type %d (supported: Q4_0=2, Q4_1=3, Q8_0=8, Q4_K=12, Q5_K=13, Q6_K=14)", ggml_type);
    JL_REQUIRE(ctx, rows > 0 && cols > 0 && cols % 256 == 0, JL_ERR_UNSUPPORTED,
               "rows must be positive and cols a positive multiple of 256");
    if (n == 0) return JL_OK;
    jl_tensor *t = nullptr;
    int rc = jl_tensor_upload(ctx, ggml_type, rows, cols, w_host, size_t(rows * row_bytes(ggml_type, cols)), &t);
    if (rc) return rc;
    void *dx = nullptr, *dy = nullptr;
    if ((rc = dev_alloc(ctx, &dx, size_t(n) * cols * 4)) || (rc = dev_alloc(ctx, &dy, size_t(n) * rows * 4))) {
        if (dx) cudaFree(dx);
        jl_tensor_free(ctx, t);
        return rc;
    }
    cudaError_t e = cudaMemcpyAsync(dx, x_host, size_t(n) * cols * 4, cudaMemcpyHostToDevice, ctx->stream);
    if (e == cudaSuccess) {
        rc = jl_gemv_dev(ctx, t, static_cast<float *>(dx), n, static_cast<float *>(dy));
        if (!rc) e = cudaMemcpyAsync(y_host, dy, size_t(n) * rows * 4, cudaMemcpyDeviceToHost, ctx->stream);
    }
    int32_t status = 0;
    if (e == cudaSuccess) e = cudaMemcpyAsync(&status, ctx->d_status, 4, cudaMemcpyDeviceToHost, ctx->stream);
    if (e == cudaSuccess) e = cudaStreamSynchronize(ctx->stream);
    cudaFree(dx);
    cudaFree(dy);
    jl_tensor_free(ctx, t);
    if (rc) return rc;
    if (e != cudaSuccess) return fail(ctx, JL_ERR_CUDA, "matrix-vector product failed: %s", cudaGetErrorString(e));
    if (status == kDevTimeout) {
        cudaMemset(ctx->d_status, 0, 4);
        return fail(ctx, JL_ERR_TIMEOUT, "a kernel gave up waiting for an asynchronous copy");
    }
    ctx->counters.h2d_bytes += size_t(n) * cols * 4;
    ctx->counters.d2h_bytes += size_t(n) * rows * 4;
    return JL_OK;
}

// ---- plumbing ---------------------------------------------------------------------------------

void *jl_device_alloc(jl_ctx *ctx, size_t nbytes) {
    if (!ctx) return nullptr;
    cudaSetDevice(ctx->device);
    void *p = nullptr;
    if (dev_alloc(ctx, &p, nbytes)) return nullptr;
    ctx->user_allocs.push_back(p);
    return p;
}

int32_t jl_device_free(jl_ctx *ctx, void *p) {
    if (!ctx || !p) return JL_OK;
    cudaSetDevice(ctx->device);
    for (size_t i = 0; i < ctx->user_allocs.size(); ++i)
        if (ctx->user_allocs[i] == p) {
            cudaStreamSynchronize(ctx->stream);
            cudaFree(p);
            ctx->user_allocs.erase(ctx->user_allocs.begin() + i);
            return JL_OK;
        }
    return fail(ctx, JL_ERR_INVALID, "pointer was not allocated by jl_device_alloc");
}

int32_t jl_memcpy_h2d(jl_ctx *ctx, void *dst_dev, const void *src_host, size_t nbytes) {
    if (!ctx) return JL_ERR_INVALID;
    cudaSetDevice(ctx->device);
    JL_CUDA(ctx, cudaMemcpyAsync(dst_dev, src_host, nbytes, cudaMemcpyHostToDevice, ctx->stream));
    JL_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
    ctx->counters.h2d_bytes += nbytes;
    return JL_OK;
}

int32_t jl_memcpy_d2h(jl_ctx *ctx, void *dst_host, const void *src_dev, size_t nbytes) {
    if (!ctx) return JL_ERR_INVALID;
    cudaSetDevice(ctx->device);
    JL_CUDA(ctx, cudaMemcpyAsync(dst_host, src_dev, nbytes, cudaMemcpyDeviceToHost, ctx->stream));
    JL_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
    ctx->counters.d2h_bytes += nbytes;
    return JL_OK;
}

int32_t jl_synchronize(jl_ctx *ctx) {
    if (!ctx) return JL_ERR_INVALID;
    cudaSetDevice(ctx->device);
    JL_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
    return JL_OK;
}

void *jl_stream(jl_ctx *ctx) { return ctx ? static_cast<void *>(ctx->stream) : nullptr; }

int32_t jl_timer_start(jl_ctx *ctx) {
    if (!ctx) return JL_ERR_INVALID;
    cudaSetDevice(ctx->device);
    JL_CUDA(ctx, cudaEventRecord(ctx->tev0, ctx->stream));
    return JL_OK;
}

int32_t jl_timer_stop(jl_ctx *ctx, float *elapsed_ms) {
    if (!ctx || !elapsed_ms) return JL_ERR_INVALID;
    cudaSetDevice(ctx->device);
    JL_CUDA(ctx, cudaEventRecord(ctx->tev1, ctx->stream));
    JL_CUDA(ctx, cudaEventSynchronize(ctx->tev1));
    JL_CUDA(ctx, cudaEventElapsedTime(elapsed_ms, ctx->tev0, ctx->tev1));
    return JL_OK;
}

int32_t jl_get_counters(jl_ctx *ctx, jl_counters *out) {
    if (!ctx || !out) return JL_ERR_INVALID;
    *out = ctx->counters;
    return JL_OK;
}

int32_t jl_flush_l2(jl_ctx *ctx) {
    if (!ctx) return JL_ERR_INVALID;
    cudaSetDevice(ctx->device);
    if (!ctx->flush_buf) {
        ctx->flush_words = size_t(256) * 1024 * 1024 / 4;  // 256 MiB > 126 MB of L2
        int rc = dev_alloc(ctx, reinterpret_cast<void **>(&ctx->flush_buf), ctx->flush_words * 4);
        if (rc) return rc;
    }
    JL_CUDA(ctx, fill_launch(ctx->flush_buf, ctx->flush_words, 0u, ctx->stream));
    return JL_OK;
}

uint32_t jl_debug_tp_next_sequence(uint32_t seq) { return tp_next_sequence(seq); }

int32_t jl_debug_peer_wait_timeout(jl_ctx *ctx, int32_t timeout_ms) {
    if (!ctx) return JL_ERR_INVALID;
    JL_REQUIRE(ctx, timeout_ms >= 1 && timeout_ms <= 2000, JL_ERR_INVALID, "timeout_ms must be 1..2000");
    cudaSetDevice(ctx->device);
    // A two-rank exchange in which this GPU is rank 0 and "rank 1" is a local buffer nobody writes:
    // the kernel pushes, waits for packets that never come, gives up after timeout_ms and says so.
    constexpr int kCount = 256;
    const size_t cap = kCount;
    const size_t inbox_packets = 2 * 2 * cap;  // [slot][source rank][cap]
    char *buf = nullptr;
    const size_t bytes = 2 * inbox_packets * sizeof(uint2) + 2 * kCount * sizeof(float) + 4 * sizeof(unsigned);
    int rc = dev_alloc(ctx, reinterpret_cast<void **>(&buf), bytes);
    if (rc) return rc;
    cudaError_t e = cudaMemsetAsync(buf, 0, bytes, ctx->stream);
    TpReduceArgs a = {};
    a.inbox.of[0] = reinterpret_cast<uint2 *>(buf);
    a.inbox.of[1] = reinterpret_cast<uint2 *>(buf) + inbox_packets;
    a.part = reinterpret_cast<float *>(buf + 2 * inbox_packets * sizeof(uint2));
    a.x = const_cast<float *>(a.part) + kCount;
    a.ctr = reinterpret_cast<unsigned *>(a.x + kCount);
    a.base = 0;
    a.cap = cap;
    a.tp = 2;
    a.rank = 0;
    a.count = kCount;
    a.status = ctx->d_status;
    a.timeout_ns = 1000000ull * unsigned(timeout_ms);
    const unsigned ctr0[4] = {1u, 0u, 0u, 0u};
    if (e == cudaSuccess) e = cudaMemcpyAsync(a.ctr, ctr0, sizeof ctr0, cudaMemcpyHostToDevice, ctx->stream);
    if (e == cudaSuccess) e = tp_push_reduce_launch(a, ctx->stream, false);
    int status = 0;
    if (e == cudaSuccess) e = cudaMemcpyAsync(&status, ctx->d_status, sizeof status, cudaMemcpyDeviceToHost, ctx->stream);
    if (e == cudaSuccess) e = cudaStreamSynchronize(ctx->stream);
    if (e == cudaSuccess) e = cudaMemsetAsync(ctx->d_status, 0, sizeof(int), ctx->stream);
    if (e == cudaSuccess) e = cudaStreamSynchronize(ctx->stream);
    cudaFree(buf);
    if (e != cudaSuccess) return fail(ctx, JL_ERR_CUDA, "peer wait self-test failed: %s", cudaGetErrorString(e));
    ctx->counters.kernel_launches += 1;
    if (status == kDevTimeout) return fail(ctx, JL_ERR_TIMEOUT, "a peer did not answer within %d ms", timeout_ms);
    return JL_OK;
}

}  // extern "C"
