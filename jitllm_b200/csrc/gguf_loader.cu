// Native GGUF reader: maps a GGUF v2/v3 file, finds the Llama metadata and the weight tensors, and
// hands every tensor (or, under tensor parallelism, this GPU's slice of it) straight from the
// mapping to jl_upload_tensor. It stands where the reference parses the file in Java and copies
// tensors through Panama segments (format/GGUF.java:60-110 header and tensor infos, :123-165
// tensor mapping; model/loader/LlamaModelLoader.java:49-67 metadata keys, :125-188 tensor names;
// model/loader/ModelLoader.java:246-290 device copies).
#include "../../include/jitllm_b200.h"

#include <fcntl.h>
#include <sys/mman.h>
#include <sys/stat.h>
#include <unistd.h>

#include <cmath>
#include <cstdio>
#include <cstring>
#include <map>
#include <string>
#include <vector>

namespace {

thread_local std::string g_gguf_error;

int gguf_fail(int code, const std::string &msg) {
    g_gguf_error = msg;
    return code;
}

struct TensorInfo {
    int type = -1;
    uint64_t dims[4] = {1, 1, 1, 1};
    uint32_t n_dims = 0;
    uint64_t offset = 0;  // relative to the data section
};

}  // namespace

struct jl_gguf {
    int fd = -1;
    const uint8_t *map = nullptr;
    size_t size = 0;
    uint32_t version = 0;
    uint64_t alignment = 32;
    uint64_t data_offset = 0;
    std::map<std::string, double> numbers;       // every scalar metadata value
    std::map<std::string, std::string> strings;  // every string metadata value
    std::map<std::string, uint64_t> array_len;   // "<key>.length" of the reference's metadata map
    std::map<std::string, TensorInfo> tensors;
};

namespace {

struct Cursor {
    const uint8_t *p, *end;
    bool ok = true;
    template <typename T>
    T get() {
        T v{};
        if (size_t(end - p) < sizeof(T)) {
            ok = false;
            return v;
        }
        memcpy(&v, p, sizeof(T));
        p += sizeof(T);
        return v;
    }
    std::string str() {
        const uint64_t n = get<uint64_t>();
        if (!ok || uint64_t(end - p) < n) {
            ok = false;
            return std::string();
        }
        std::string s(reinterpret_cast<const char *>(p), size_t(n));
        p += n;
        return s;
    }
};

// gguf_metadata_value_type: 0 u8, 1 i8, 2 u16, 3 i16, 4 u32, 5 i32, 6 f32, 7 bool, 8 string, 9 array,
// 10 u64, 11 i64, 12 f64.
bool read_scalar(Cursor &c, uint32_t type, double *out) {
    switch (type) {
        case 0: *out = c.get<uint8_t>(); return c.ok;
        case 1: *out = c.get<int8_t>(); return c.ok;
        case 2: *out = c.get<uint16_t>(); return c.ok;
        case 3: *out = c.get<int16_t>(); return c.ok;
        case 4: *out = c.get<uint32_t>(); return c.ok;
        case 5: *out = c.get<int32_t>(); return c.ok;
        case 6: *out = c.get<float>(); return c.ok;
        case 7: *out = c.get<uint8_t>(); return c.ok;
        case 10: *out = double(c.get<uint64_t>()); return c.ok;
        case 11: *out = double(c.get<int64_t>()); return c.ok;
        case 12: *out = c.get<double>(); return c.ok;
        default: return false;
    }
}

bool read_value(Cursor &c, jl_gguf *g, const std::string &key, uint32_t type) {
    if (type == 8) {
        g->strings[key] = c.str();
        return c.ok;
    }
    if (type == 9) {
        const uint32_t et = c.get<uint32_t>();
        const uint64_t n = c.get<uint64_t>();
        if (!c.ok) return false;
        g->array_len[key] = n;
        for (uint64_t i = 0; i < n; ++i) {
            if (et == 8) {
                c.str();
            } else if (et == 9) {
                return false;  // nested arrays do not occur in model files
            } else {
                double ignored;
                if (!read_scalar(c, et, &ignored)) return false;
            }
            if (!c.ok) return false;
        }
        return true;
    }
    double v;
    if (!read_scalar(c, type, &v)) return false;
    g->numbers[key] = v;
    return true;
}

int64_t type_row_bytes(int type, uint64_t cols) {
    switch (type) {
        case JL_F32: return int64_t(cols) * 4;
        case JL_F16: return int64_t(cols) * 2;
        case JL_Q4_0: return int64_t(cols / 32) * 18;
        case JL_Q8_0: return int64_t(cols / 32) * 34;
        case JL_Q4_K: return int64_t(cols / 256) * 144;
        case JL_Q4_1: return int64_t(cols / 32) * 20;
        case JL_Q5_K: return int64_t(cols / 256) * 176;
        case JL_Q6_K: return int64_t(cols / 256) * 210;
        default: return -1;
    }
}

}  // namespace

extern "C" {

const char *jl_gguf_last_error(void) { return g_gguf_error.c_str(); }

void jl_gguf_close(jl_gguf *g) {
    if (!g) return;
    if (g->map) munmap(const_cast<uint8_t *>(g->map), g->size);
    if (g->fd >= 0) close(g->fd);
    delete g;
}

int32_t jl_gguf_open(const char *path, jl_gguf **out) {
    if (!path || !out) return gguf_fail(JL_ERR_INVALID, "GPUL-CFG-002: path and out must not be NULL");
    *out = nullptr;
    jl_gguf *g = new jl_gguf();
    g->fd = open(path, O_RDONLY);
    struct stat st;
    if (g->fd < 0 || fstat(g->fd, &st) != 0 || st.st_size < 24) {
        jl_gguf_close(g);
        return gguf_fail(JL_ERR_INVALID, std::string("GPUL-CFG-002: cannot open GGUF file ") + path);
    }
    g->size = size_t(st.st_size);
    void *m = mmap(nullptr, g->size, PROT_READ, MAP_PRIVATE, g->fd, 0);
    if (m == MAP_FAILED) {
        g->map = nullptr;
        jl_gguf_close(g);
        return gguf_fail(JL_ERR_OOM, std::string("cannot map ") + path);
    }
    g->map = static_cast<const uint8_t *>(m);
    Cursor c{g->map, g->map + g->size};
    const uint32_t magic = c.get<uint32_t>();
    g->version = c.get<uint32_t>();
    if (magic != 0x46554747u || (g->version != 2 && g->version != 3)) {
        jl_gguf_close(g);
        return gguf_fail(JL_ERR_UNSUPPORTED, "GPUL-CFG-002: unsupported: not a GGUF v2/v3 file");
    }
    const uint64_t n_tensors = c.get<uint64_t>(), n_kv = c.get<uint64_t>();
    for (uint64_t i = 0; c.ok && i < n_kv; ++i) {
        const std::string key = c.str();
        const uint32_t type = c.get<uint32_t>();
        if (!c.ok || !read_value(c, g, key, type)) c.ok = false;
    }
    for (uint64_t i = 0; c.ok && i < n_tensors; ++i) {
        const std::string name = c.str();
        TensorInfo t;
        t.n_dims = c.get<uint32_t>();
        if (!c.ok || t.n_dims > 4) {
            c.ok = false;
            break;
        }
        for (uint32_t d = 0; d < t.n_dims; ++d) t.dims[d] = c.get<uint64_t>();
        t.type = int(c.get<uint32_t>());
        t.offset = c.get<uint64_t>();
        g->tensors[name] = t;
    }
    if (!c.ok) {
        jl_gguf_close(g);
        return gguf_fail(JL_ERR_INVALID, "GPUL-CFG-002: truncated or malformed GGUF header");
    }
    if (g->numbers.count("general.alignment")) g->alignment = uint64_t(g->numbers["general.alignment"]);
    if (g->alignment == 0 || (g->alignment & (g->alignment - 1)) != 0) {
        jl_gguf_close(g);
        return gguf_fail(JL_ERR_INVALID, "GPUL-CFG-002: general.alignment must be a power of two");
    }
    const uint64_t pos = uint64_t(c.p - g->map);
    g->data_offset = (pos + g->alignment - 1) / g->alignment * g->alignment;
    // every tensor must lie inside the file
    for (const auto &kv : g->tensors) {
        const TensorInfo &t = kv.second;
        const int64_t rb = type_row_bytes(t.type, t.dims[0]);
        if (rb < 0) continue;  // a type this library does not use; refused only if a needed tensor has it
        // Every product and sum below can wrap in a crafted file, and a wrapped value would pass the
        // comparison with the file size: each step is checked.
        uint64_t rows = 0, bytes = 0, end = 0;
        const bool overflow = __builtin_mul_overflow(uint64_t(t.dims[1]), uint64_t(t.dims[2]), &rows) ||
                              __builtin_mul_overflow(rows, uint64_t(t.dims[3]), &rows) ||
                              __builtin_mul_overflow(uint64_t(rb), rows, &bytes) ||
                              __builtin_add_overflow(uint64_t(g->data_offset), uint64_t(t.offset), &end) ||
                              __builtin_add_overflow(end, bytes, &end);
        if (overflow || t.offset % g->alignment != 0 || end > g->size) {
            const std::string msg = "GPUL-CFG-002: tensor '" + kv.first + "' lies outside the file or is misaligned";
            jl_gguf_close(g);  // frees the map the name lives in: the message is built first
            return gguf_fail(JL_ERR_INVALID, msg);
        }
    }
    *out = g;
    return JL_OK;
}

int32_t jl_gguf_describe(const jl_gguf *g, jl_model_desc *desc, float *rope_theta, int64_t *n_tensors) {
    if (!g || !desc) return gguf_fail(JL_ERR_INVALID, "GPUL-CFG-002: NULL argument");
    auto num = [&](const char *key, double dflt, bool required, bool *missing) {
        auto it = g->numbers.find(key);
        if (it != g->numbers.end()) return it->second;
        if (required) *missing = true;
        return dflt;
    };
    auto arch = g->strings.find("general.architecture");
    if (arch != g->strings.end() && arch->second != "llama")
        return gguf_fail(JL_ERR_UNSUPPORTED, "GPUL-CFG-002: unsupported: architecture '" + arch->second + "' (llama only)");
    bool missing = false;
    jl_model_desc d = {};
    d.dim = int(num("llama.embedding_length", 0, true, &missing));
    d.hidden = int(num("llama.feed_forward_length", 0, true, &missing));
    d.layers = int(num("llama.block_count", 0, true, &missing));
    d.heads = int(num("llama.attention.head_count", 0, true, &missing));
    d.kv_heads = int(num("llama.attention.head_count_kv", d.heads, false, &missing));
    d.ctx_len = int(num("llama.context_length", 0, true, &missing));
    d.rms_eps = float(num("llama.attention.layer_norm_rms_epsilon", 1e-5, false, &missing));
    if (g->numbers.count("llama.vocab_size")) {
        d.vocab = int(g->numbers.at("llama.vocab_size"));
    } else if (g->array_len.count("tokenizer.ggml.tokens")) {
        d.vocab = int(g->array_len.at("tokenizer.ggml.tokens"));
    } else {
        missing = true;
    }
    if (missing || d.heads <= 0) return gguf_fail(JL_ERR_INVALID, "GPUL-CFG-002: a required llama.* metadata key is missing");
    d.head_dim = d.dim / d.heads;
    d.tied_embeddings = g->tensors.count("output.weight") ? 0 : 1;
    d.max_batch = 1;
    d.tp_rank = 0;
    d.tp_size = 1;
    *desc = d;
    if (rope_theta) *rope_theta = float(num("llama.rope.freq_base", 10000.0, false, &missing));
    if (n_tensors) *n_tensors = int64_t(g->tensors.size());
    return JL_OK;
}

}  // extern "C"

namespace {

struct RoleName {
    int role;
    const char *name;  // printf pattern with the layer number for per-layer roles
    bool per_layer;
    int split;  // 0 replicated, 1 by rows, 2 by columns (tensor parallelism)
};

const RoleName kRoles[] = {
    {JL_ROLE_TOKEN_EMBEDDING, "token_embd.weight", false, 0},
    {JL_ROLE_OUTPUT_NORM, "output_norm.weight", false, 0},
    {JL_ROLE_OUTPUT, "output.weight", false, 1},
    {JL_ROLE_ATTENTION_NORM, "blk.%d.attn_norm.weight", true, 0},
    {JL_ROLE_ATTENTION_QUERY, "blk.%d.attn_q.weight", true, 1},
    {JL_ROLE_ATTENTION_KEY, "blk.%d.attn_k.weight", true, 1},
    {JL_ROLE_ATTENTION_VALUE, "blk.%d.attn_v.weight", true, 1},
    {JL_ROLE_ATTENTION_OUTPUT, "blk.%d.attn_output.weight", true, 2},
    {JL_ROLE_FFN_NORM, "blk.%d.ffn_norm.weight", true, 0},
    {JL_ROLE_FFN_GATE, "blk.%d.ffn_gate.weight", true, 1},
    {JL_ROLE_FFN_UP, "blk.%d.ffn_up.weight", true, 1},
    {JL_ROLE_FFN_DOWN, "blk.%d.ffn_down.weight", true, 2},
};

// One tensor, or this rank's slice of it: rows [r*R/tp, (r+1)*R/tp) as a byte range of the mapping,
// columns [r*C/tp, (r+1)*C/tp) gathered row by row (whole 256-column groups, so blocks stay whole).
int upload_one(jl_ctx *ctx, const jl_gguf *g, const RoleName &rn, int layer, const std::string &name, int tp_rank,
               int tp_size, bool optional) {
    auto it = g->tensors.find(name);
    if (it == g->tensors.end())
        return optional ? JL_OK : gguf_fail(JL_ERR_INVALID, "GPUL-CFG-002: tensor '" + name + "' is missing");
    const TensorInfo &t = it->second;
    const uint64_t cols = t.dims[0], rows = t.n_dims >= 2 ? t.dims[1] : 1;
    const int64_t rb = type_row_bytes(t.type, cols);
    if (rb < 0) return gguf_fail(JL_ERR_UNSUPPORTED, "GPUL-CFG-002: unsupported: GGML type of '" + name + "'");
    const uint8_t *src = g->map + g->data_offset + t.offset;
    int rc;
    if (tp_size <= 1 || rn.split == 0) {
        rc = jl_upload_tensor(ctx, rn.role, layer, t.type, int64_t(rows), int64_t(cols), src, size_t(rb) * rows);
    } else if (rn.split == 1) {
        const uint64_t lr = rows / tp_size;
        rc = jl_upload_tensor(ctx, rn.role, layer, t.type, int64_t(lr), int64_t(cols), src + size_t(tp_rank) * lr * rb,
                              size_t(rb) * lr);
    } else {
        const uint64_t lc = cols / tp_size;
        if (cols % tp_size != 0 || lc % 256 != 0)
            return gguf_fail(JL_ERR_INVALID, "GPUL-CFG-002: '" + name + "' cannot be cut into whole 256-column groups per GPU");
        const int64_t lrb = type_row_bytes(t.type, lc);
        std::vector<uint8_t> slice(size_t(lrb) * rows);
        for (uint64_t r = 0; r < rows; ++r)
            memcpy(slice.data() + r * lrb, src + r * rb + size_t(tp_rank) * lrb, size_t(lrb));
        rc = jl_upload_tensor(ctx, rn.role, layer, t.type, int64_t(rows), int64_t(lc), slice.data(), slice.size());
    }
    if (rc != JL_OK) return gguf_fail(rc, std::string("upload of '") + name + "' failed: " + jl_last_error(ctx));
    return JL_OK;
}

}  // namespace

extern "C" int32_t jl_gguf_upload(jl_ctx *ctx, const jl_gguf *g, int32_t max_batch, int32_t tp_rank, int32_t tp_size,
                                  const float *rope_cos, const float *rope_sin, int64_t rope_n) {
    if (!ctx || !g) return gguf_fail(JL_ERR_INVALID, "GPUL-CFG-002: NULL argument");
    jl_model_desc d;
    float theta = 10000.f;
    int rc = jl_gguf_describe(g, &d, &theta, nullptr);
    if (rc) return rc;
    d.max_batch = max_batch;
    d.tp_rank = tp_rank;
    d.tp_size = tp_size < 1 ? 1 : tp_size;
    if ((rc = jl_model_create(ctx, &d))) return gguf_fail(rc, std::string("jl_model_create: ") + jl_last_error(ctx));
    char name[96];
    for (const RoleName &rn : kRoles) {
        if (!rn.per_layer) {
            const bool optional = rn.role == JL_ROLE_OUTPUT;  // tied embeddings: no output.weight
            if ((rc = upload_one(ctx, g, rn, -1, rn.name, tp_rank, d.tp_size, optional))) return rc;
            continue;
        }
        for (int l = 0; l < d.layers; ++l) {
            snprintf(name, sizeof name, rn.name, l);
            if ((rc = upload_one(ctx, g, rn, l, name, tp_rank, d.tp_size, false))) return rc;
        }
    }
    if (rope_cos != nullptr && rope_sin != nullptr) {
        rc = jl_upload_rope(ctx, rope_cos, rope_sin, rope_n);
    } else {
        // The table of RopeFrequencies.precomputeFreqsCis without scaling
        // (model/loader/RopeFrequencies.java:14-54): freq narrowed to binary32, the angle pos * freq in
        // binary32, cos / sin in double then narrowed. The C library's last bit may differ from the
        // JVM's; a host that wants the CPU path's exact table passes it in.
        const int half = d.head_dim / 2;
        std::vector<float> cr(size_t(d.ctx_len) * half), ci(cr.size());
        for (int pos = 0; pos < d.ctx_len; ++pos) {
            for (int i = 0; i < half; ++i) {
                const float freq = float(1.0 / pow(double(theta), double(2 * i) / double(d.head_dim)));
                const float val = float(pos) * freq;
                cr[size_t(pos) * half + i] = float(cos(double(val)));
                ci[size_t(pos) * half + i] = float(sin(double(val)));
            }
        }
        rc = jl_upload_rope(ctx, cr.data(), ci.data(), int64_t(cr.size()));
    }
    if (rc) return gguf_fail(rc, std::string("jl_upload_rope: ") + jl_last_error(ctx));
    return JL_OK;
}
