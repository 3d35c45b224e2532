// GGUF v3 reader and model loader: real model files straight into HBM.
//
// The parser follows yule-core/src/gguf.rs:271-431 check for check — magic, version 3 only, caps on
// tensor / key-value / string / array / dimension counts before anything is allocated, bounds-checked
// reads, the data section at the next multiple of `general.alignment` (32 by default), every tensor
// inside the file, no two tensors overlapping — and the model description follows
// GgufFile::to_loaded_model (gguf.rs:493-586) plus the derivations of GpuTransformerRunner::new
// (yule-infer/src/gpu_runner.rs:86-122).  The loader uploads the raw tensor bytes the way
// upload_weights does (gpu_runner.rs:171-254), through two pinned staging buffers and asynchronous
// copies, and hands them to the runner by GGUF tensor name.

#include <fcntl.h>
#include <sys/mman.h>
#include <sys/stat.h>
#include <unistd.h>

#include <algorithm>
#include <cmath>
#include <cstdio>
#include <cstring>
#include <string>
#include <unordered_map>
#include <vector>

#include "internal.h"

namespace {

constexpr uint32_t kMagic = 0x46554747u;  // "GGUF", little endian
constexpr uint64_t kMaxString = 1024 * 1024, kMaxTensors = 100000, kMaxKv = 100000, kMaxArray = 10000000;
constexpr uint32_t kMaxDims = 8;

enum ValueType : uint32_t { U8 = 0, I8, U16, I16, U32, I32, F32, BOOL, STRING, ARRAY, U64, I64, F64 };

struct Value {
    uint32_t type = 0;
    uint64_t u = 0;   // unsigned and bool
    int64_t i = 0;    // signed
    double f = 0;     // floats
    std::string s;    // string
    uint32_t elem_type = 0;  // arrays: only the element type and the length are kept
    uint64_t len = 0;
};

struct TensorEntry {
    std::string name;
    uint32_t n_dims = 0;
    uint64_t shape[kMaxDims] = {};
    uint32_t type = 0;
    uint64_t offset = 0, size_bytes = 0;
};

// block size and bytes per block of every GGML type id the reference knows (yule-core/src/dtype.rs:13-190)
bool type_layout(uint32_t id, uint32_t *block, uint32_t *bytes) {
    struct Row {
        uint32_t id, block, bytes;
    };
    static const Row rows[] = {{0, 1, 4},     {1, 1, 2},    {2, 32, 18},   {3, 32, 20},   {6, 32, 22},   {7, 32, 24},   {8, 32, 34},
                               {9, 32, 36},   {10, 256, 84}, {11, 256, 110}, {12, 256, 144}, {13, 256, 176}, {14, 256, 210},
                               {15, 256, 292}, {16, 256, 66}, {17, 256, 74},  {18, 256, 98},  {19, 256, 50},  {20, 32, 18},
                               {21, 256, 110}, {22, 256, 82}, {23, 256, 136}, {24, 1, 1},     {25, 1, 2},     {26, 1, 4},
                               {27, 1, 8},    {28, 1, 8},   {29, 256, 56},  {30, 1, 2},     {34, 256, 54},  {35, 256, 66}};
    for (const Row &r : rows)
        if (r.id == id) {
            *block = r.block;
            *bytes = r.bytes;
            return true;
        }
    return false;
}

struct Cursor {
    const uint8_t *data;
    size_t size, pos = 0;
    bool ok = true;
    template <typename T>
    T read() {
        T v{};
        if (!ok || size - pos < sizeof(T) || pos > size) {
            ok = false;
            return v;
        }
        memcpy(&v, data + pos, sizeof(T));
        pos += sizeof(T);
        return v;
    }
    bool read_string(std::string *out, std::string *err) {
        const uint64_t len = read<uint64_t>();
        if (!ok) {
            *err = "unexpected end of file";
            return false;
        }
        if (len > kMaxString) {
            *err = "string length " + std::to_string(len) + " exceeds maximum " + std::to_string(kMaxString);
            return false;
        }
        if (size - pos < len) {
            ok = false;
            *err = "unexpected end of file";
            return false;
        }
        out->assign(reinterpret_cast<const char *>(data + pos), (size_t)len);
        pos += (size_t)len;
        return true;
    }
};

}  // namespace

struct yule_gguf {
    const uint8_t *data = nullptr;
    size_t size = 0;
    bool mapped = false;
    uint32_t version = 0;
    std::unordered_map<std::string, Value> meta;
    std::vector<std::string> meta_order;
    std::vector<TensorEntry> tensors;
    uint64_t data_offset = 0, alignment = 32;

    const Value *get(const std::string &key) const {
        auto it = meta.find(key);
        return it == meta.end() ? nullptr : &it->second;
    }
    // the widening rules of GgufValue::as_u32 / as_f64 / as_str (gguf.rs:53-103)
    bool get_u32(const std::string &key, uint32_t *out) const {
        const Value *v = get(key);
        if (!v) return false;
        if (v->type == U32 || v->type == U8 || v->type == U16) {
            *out = (uint32_t)v->u;
            return true;
        }
        if (v->type == I32 && v->i >= 0) {
            *out = (uint32_t)v->i;
            return true;
        }
        return false;
    }
    bool get_f64(const std::string &key, double *out) const {
        const Value *v = get(key);
        if (!v || (v->type != F64 && v->type != F32)) return false;
        *out = v->f;
        return true;
    }
    const char *get_str(const std::string &key) const {
        const Value *v = get(key);
        return (v && v->type == STRING) ? v->s.c_str() : nullptr;
    }
    const TensorEntry *find_tensor(const std::string &name) const {
        for (const TensorEntry &t : tensors)
            if (t.name == name) return &t;
        return nullptr;
    }
};

namespace {

using yule::fail;

bool read_value(Cursor &c, uint32_t type, Value *v, std::string *err, int depth = 0) {
    v->type = type;
    switch (type) {
        case U8: v->u = c.read<uint8_t>(); break;
        case I8: v->i = c.read<int8_t>(); break;
        case U16: v->u = c.read<uint16_t>(); break;
        case I16: v->i = c.read<int16_t>(); break;
        case U32: v->u = c.read<uint32_t>(); break;
        case I32: v->i = c.read<int32_t>(); break;
        case F32: v->f = c.read<float>(); break;
        case BOOL: v->u = c.read<uint8_t>() != 0; break;
        case STRING: return c.read_string(&v->s, err);
        case U64: v->u = c.read<uint64_t>(); break;
        case I64: v->i = c.read<int64_t>(); break;
        case F64: v->f = c.read<double>(); break;
        case ARRAY: {
            v->elem_type = c.read<uint32_t>();
            v->len = c.read<uint64_t>();
            if (!c.ok) break;
            if (v->len > kMaxArray) {
                *err = "array length " + std::to_string(v->len) + " exceeds maximum " + std::to_string(kMaxArray);
                return false;
            }
            if (depth > 4) {
                *err = "arrays nested too deeply";
                return false;
            }
            Value scratch;
            for (uint64_t i = 0; i < v->len; i++)
                if (!read_value(c, v->elem_type, &scratch, err, depth + 1)) return false;
            break;
        }
        default: *err = "unknown GGUF value type: " + std::to_string(type); return false;
    }
    if (!c.ok) {
        *err = "unexpected end of file";
        return false;
    }
    return true;
}

int32_t parse(yule_gguf *g) {
    Cursor c{g->data, g->size};
    std::string err;
    const uint32_t magic = c.read<uint32_t>();
    if (!c.ok) return fail(YULE_ERR_PARSE, "gguf: file of %zu bytes is too small for a header", g->size);
    if (magic != kMagic) return fail(YULE_ERR_PARSE, "gguf: invalid magic: expected 0x%08x, got 0x%08x", kMagic, magic);
    g->version = c.read<uint32_t>();
    if (!c.ok) return fail(YULE_ERR_PARSE, "gguf: truncated header");
    if (g->version != 3) return fail(YULE_ERR_PARSE, "gguf: unsupported version %u", g->version);
    const uint64_t n_tensors = c.read<uint64_t>();
    const uint64_t n_kv = c.read<uint64_t>();
    if (!c.ok) return fail(YULE_ERR_PARSE, "gguf: truncated header");
    if (n_tensors > kMaxTensors)
        return fail(YULE_ERR_PARSE, "gguf: tensor count %llu exceeds maximum %llu", (unsigned long long)n_tensors,
                    (unsigned long long)kMaxTensors);
    if (n_kv > kMaxKv)
        return fail(YULE_ERR_PARSE, "gguf: KV count %llu exceeds maximum %llu", (unsigned long long)n_kv, (unsigned long long)kMaxKv);
    for (uint64_t i = 0; i < n_kv; i++) {
        std::string key;
        if (!c.read_string(&key, &err)) return fail(YULE_ERR_PARSE, "gguf: failed to read KV key %llu: %s", (unsigned long long)i, err.c_str());
        const uint32_t type = c.read<uint32_t>();
        Value v;
        if (!c.ok || !read_value(c, type, &v, &err))
            return fail(YULE_ERR_PARSE, "gguf: failed to read KV value for '%s': %s", key.c_str(), c.ok ? err.c_str() : "unexpected end of file");
        if (!g->meta.count(key)) g->meta_order.push_back(key);
        g->meta[key] = std::move(v);
    }
    g->tensors.reserve((size_t)n_tensors);
    for (uint64_t i = 0; i < n_tensors; i++) {
        TensorEntry t;
        if (!c.read_string(&t.name, &err))
            return fail(YULE_ERR_PARSE, "gguf: failed to read tensor %llu name: %s", (unsigned long long)i, err.c_str());
        t.n_dims = c.read<uint32_t>();
        if (!c.ok) return fail(YULE_ERR_PARSE, "gguf: truncated tensor info");
        if (t.n_dims > kMaxDims)
            return fail(YULE_ERR_PARSE, "gguf: tensor '%s' has %u dimensions, max is %u", t.name.c_str(), t.n_dims, kMaxDims);
        uint64_t elements = 1;
        for (uint32_t d = 0; d < t.n_dims; d++) {
            t.shape[d] = c.read<uint64_t>();
            if (t.shape[d] != 0 && elements > UINT64_MAX / t.shape[d])
                return fail(YULE_ERR_PARSE, "gguf: invalid tensor shape for '%s': shape overflow", t.name.c_str());
            elements *= t.shape[d];
        }
        t.type = c.read<uint32_t>();
        t.offset = c.read<uint64_t>();
        if (!c.ok) return fail(YULE_ERR_PARSE, "gguf: truncated tensor info");
        uint32_t block = 0, bytes = 0;
        if (!type_layout(t.type, &block, &bytes)) return fail(YULE_ERR_PARSE, "gguf: unknown GGUF dtype: %u", t.type);
        const uint64_t blocks = (elements + block - 1) / block;
        if (blocks > UINT64_MAX / bytes) return fail(YULE_ERR_PARSE, "gguf: invalid tensor shape for '%s': size overflow", t.name.c_str());
        t.size_bytes = blocks * bytes;
        g->tensors.push_back(std::move(t));
    }
    uint32_t align = 32;
    g->get_u32("general.alignment", &align);
    if (align == 0) return fail(YULE_ERR_PARSE, "gguf: general.alignment is 0");
    g->alignment = align;
    g->data_offset = ((uint64_t)c.pos + align - 1) / align * align;
    for (const TensorEntry &t : g->tensors) {
        const uint64_t abs = g->data_offset + t.offset;
        if (abs < t.offset || abs + t.size_bytes < abs || abs + t.size_bytes > g->size)
            return fail(YULE_ERR_PARSE, "gguf: tensor '%s' out of bounds: offset %llu + %llu bytes in a file of %zu", t.name.c_str(),
                        (unsigned long long)abs, (unsigned long long)t.size_bytes, g->size);
    }
    std::vector<const TensorEntry *> sorted;
    for (const TensorEntry &t : g->tensors) sorted.push_back(&t);
    std::sort(sorted.begin(), sorted.end(), [](const TensorEntry *a, const TensorEntry *b) { return a->offset < b->offset; });
    for (size_t i = 1; i < sorted.size(); i++)
        if (sorted[i - 1]->offset + sorted[i - 1]->size_bytes > sorted[i]->offset)
            return fail(YULE_ERR_PARSE, "gguf: overlapping tensors: '%s' [%llu..%llu] overlaps '%s' [%llu..]", sorted[i - 1]->name.c_str(),
                        (unsigned long long)sorted[i - 1]->offset, (unsigned long long)(sorted[i - 1]->offset + sorted[i - 1]->size_bytes),
                        sorted[i]->name.c_str(), (unsigned long long)sorted[i]->offset);
    return YULE_OK;
}

}  // namespace

extern "C" {

int32_t yule_gguf_parse(const void *data, size_t size, yule_gguf **out) {
    if (!data || !out) return fail(YULE_ERR_INVALID_ARGUMENT, "null argument");
    yule_gguf *g = new yule_gguf();
    g->data = static_cast<const uint8_t *>(data);
    g->size = size;
    int32_t rc = parse(g);
    if (rc) {
        delete g;
        return rc;
    }
    *out = g;
    return YULE_OK;
}

int32_t yule_gguf_open(const char *path, yule_gguf **out) {
    if (!path || !out) return fail(YULE_ERR_INVALID_ARGUMENT, "null argument");
    const int fd = open(path, O_RDONLY);
    if (fd < 0) return fail(YULE_ERR_PARSE, "gguf: cannot open '%s': %s", path, strerror(errno));
    struct stat st;
    if (fstat(fd, &st) != 0 || st.st_size < 24) {
        close(fd);
        return fail(YULE_ERR_PARSE, "gguf: '%s' is too small for a header", path);
    }
    void *map = mmap(nullptr, (size_t)st.st_size, PROT_READ, MAP_PRIVATE, fd, 0);
    close(fd);  // the mapping keeps the file
    if (map == MAP_FAILED) return fail(YULE_ERR_PARSE, "gguf: mmap of '%s' failed: %s", path, strerror(errno));
    yule_gguf *g = new yule_gguf();
    g->data = static_cast<const uint8_t *>(map);
    g->size = (size_t)st.st_size;
    g->mapped = true;
    int32_t rc = parse(g);
    if (rc) {
        munmap(map, g->size);
        delete g;
        return rc;
    }
    *out = g;
    return YULE_OK;
}

int32_t yule_gguf_close(yule_gguf *g) {
    if (!g) return YULE_OK;
    if (g->mapped) munmap(const_cast<uint8_t *>(g->data), g->size);
    delete g;
    return YULE_OK;
}

int32_t yule_gguf_summary(const yule_gguf *g, uint32_t *version, uint64_t *n_tensors, uint64_t *n_kv, uint64_t *data_offset,
                          uint64_t *alignment) {
    if (!g) return fail(YULE_ERR_INVALID_ARGUMENT, "null gguf");
    if (version) *version = g->version;
    if (n_tensors) *n_tensors = g->tensors.size();
    if (n_kv) *n_kv = g->meta.size();
    if (data_offset) *data_offset = g->data_offset;
    if (alignment) *alignment = g->alignment;
    return YULE_OK;
}

int32_t yule_gguf_tensor(const yule_gguf *g, uint64_t index, yule_gguf_tensor_info *out) {
    if (!g || !out) return fail(YULE_ERR_INVALID_ARGUMENT, "null argument");
    if (index >= g->tensors.size()) return fail(YULE_ERR_OUT_OF_BOUNDS, "tensor index %llu of %zu", (unsigned long long)index, g->tensors.size());
    const TensorEntry &t = g->tensors[(size_t)index];
    out->name = t.name.c_str();
    out->n_dims = t.n_dims;
    for (uint32_t d = 0; d < kMaxDims; d++) out->shape[d] = d < t.n_dims ? t.shape[d] : 0;
    out->gguf_type = t.type;
    out->offset = t.offset;
    out->size_bytes = t.size_bytes;
    out->data = g->data + g->data_offset + t.offset;
    return YULE_OK;
}

int32_t yule_gguf_find_tensor(const yule_gguf *g, const char *name, uint64_t *index) {
    if (!g || !name || !index) return fail(YULE_ERR_INVALID_ARGUMENT, "null argument");
    for (size_t i = 0; i < g->tensors.size(); i++)
        if (g->tensors[i].name == name) {
            *index = i;
            return YULE_OK;
        }
    return fail(YULE_ERR_MISSING_TENSOR, "tensor not found: %s", name);
}

int32_t yule_gguf_meta_u32(const yule_gguf *g, const char *key, uint32_t *out) {
    if (!g || !key || !out) return fail(YULE_ERR_INVALID_ARGUMENT, "null argument");
    return g->get_u32(key, out) ? YULE_OK : fail(YULE_ERR_INVALID_ARGUMENT, "gguf: no unsigned value under '%s'", key);
}

int32_t yule_gguf_meta_f64(const yule_gguf *g, const char *key, double *out) {
    if (!g || !key || !out) return fail(YULE_ERR_INVALID_ARGUMENT, "null argument");
    return g->get_f64(key, out) ? YULE_OK : fail(YULE_ERR_INVALID_ARGUMENT, "gguf: no float value under '%s'", key);
}

int32_t yule_gguf_meta_str(const yule_gguf *g, const char *key, const char **out) {
    if (!g || !key || !out) return fail(YULE_ERR_INVALID_ARGUMENT, "null argument");
    *out = g->get_str(key);
    return *out ? YULE_OK : fail(YULE_ERR_INVALID_ARGUMENT, "gguf: no string value under '%s'", key);
}

// to_loaded_model (gguf.rs:493-586) followed by the derivations of GpuTransformerRunner::new
// (gpu_runner.rs:86-122): head_dim = dim / heads, ff_dim from blk.0.ffn_gate.weight's second
// dimension (else ceil(dim·8/3/256)·256), eps 1e-5 and theta 1e4 when the file has none.
int32_t yule_gguf_runner_config(const yule_gguf *g, uint32_t max_seq_len_cap, yule_runner_config *cfg) {
    if (!g || !cfg) return fail(YULE_ERR_INVALID_ARGUMENT, "null argument");
    const char *arch = g->get_str("general.architecture");
    const std::string prefix = arch ? arch : "unknown";
    // The dense transformer path of yule-infer/src/model_runner.rs with its variants: Llama / Mistral (sliding
    // window), Phi (partial RoPE), Qwen (Q/K/V bias), Gemma (norm offset, embedding scale, GeGLU, post-norms,
    // softcaps), and the mixture-of-experts FFN (model_runner.rs:813-958).  The non-transformer architectures are
    // refused rather than mis-computed.
    const bool is_gemma = prefix == "gemma" || prefix == "gemma2";
    const bool is_phi = prefix == "phi" || prefix == "phi2" || prefix == "phi3";
    const bool is_qwen = prefix == "qwen" || prefix == "qwen2";
    if (prefix != "llama" && prefix != "mistral" && !is_qwen && !is_gemma && !is_phi)
        return fail(YULE_ERR_INVALID_ARGUMENT, "gguf: architecture '%s' is outside the dense decode path of this backend", prefix.c_str());
    // mixture of experts (model_runner.rs:395-397): expert_count > 0 switches every layer's FFN to the routed form
    uint32_t experts = 0, experts_used = 0;
    g->get_u32(prefix + ".expert_count", &experts);
    g->get_u32(prefix + ".expert_used_count", &experts_used);
    if (experts == 0 && (g->find_tensor("blk.0.ffn_gate_exps.weight") || g->find_tensor("blk.0.ffn_gate.0.weight")))
        return fail(YULE_ERR_INVALID_ARGUMENT, "gguf: mixture-of-experts tensors present but no %s.expert_count", prefix.c_str());
    if (experts > 0 && (experts > 256 || experts_used == 0 || experts_used > experts))
        return fail(YULE_ERR_INVALID_ARGUMENT, "gguf: mixture of experts with %u experts, %u used per token", experts, experts_used);
    if (is_phi && !g->find_tensor("blk.0.attn_q.weight"))
        return fail(YULE_ERR_INVALID_ARGUMENT, "gguf: this file has a packed attn_qkv tensor; the runner reads separate attn_q / attn_k / attn_v");
    memset(cfg, 0, sizeof(*cfg));
    uint32_t ctx = 4096, heads = 0, kv = 0;
    g->get_u32(prefix + ".context_length", &ctx);
    g->get_u32(prefix + ".embedding_length", &cfg->dim);
    g->get_u32(prefix + ".attention.head_count", &heads);
    kv = heads;
    g->get_u32(prefix + ".attention.head_count_kv", &kv);
    g->get_u32(prefix + ".block_count", &cfg->n_layers);
    cfg->n_heads = heads;
    cfg->n_kv_heads = kv;
    if (!g->get_u32("tokenizer.ggml.vocab_size", &cfg->vocab_size)) {
        const Value *toks = g->get("tokenizer.ggml.tokens");
        if (toks && toks->type == ARRAY) cfg->vocab_size = (uint32_t)toks->len;
    }
    if (!cfg->vocab_size) {  // files without a tokenizer section: the embedding table's row count
        const TensorEntry *emb = g->find_tensor("token_embd.weight");
        if (emb && emb->n_dims == 2) cfg->vocab_size = (uint32_t)emb->shape[1];
    }
    if (!cfg->dim || !heads || !kv || !cfg->n_layers || !cfg->vocab_size || cfg->dim % heads || heads % kv)
        return fail(YULE_ERR_INVALID_ARGUMENT, "gguf: incomplete model description (dim %u, heads %u, kv heads %u, layers %u, vocab %u)",
                    cfg->dim, heads, kv, cfg->n_layers, cfg->vocab_size);
    cfg->head_dim = cfg->dim / heads;
    const TensorEntry *gate = g->find_tensor("blk.0.ffn_gate.weight");
    cfg->ff_dim = (gate && gate->n_dims == 2) ? (uint32_t)gate->shape[1] : (uint32_t)(std::ceil(cfg->dim * 8.0 / 3.0 / 256.0) * 256);
    if (experts > 0) {
        // model_runner.rs:399-407: the packed tensor holds all experts' rows, a per-expert tensor one expert's
        cfg->n_experts = experts;
        cfg->n_experts_used = experts_used;
        const TensorEntry *packed = g->find_tensor("blk.0.ffn_gate_exps.weight"), *one = g->find_tensor("blk.0.ffn_gate.0.weight");
        if (packed && packed->n_dims == 2)
            cfg->ff_dim = (uint32_t)(packed->shape[1] / experts);
        else if (one && one->n_dims == 2)
            cfg->ff_dim = (uint32_t)one->shape[1];
    }
    // model_runner.rs:414-417: 1e-6 for Phi / Qwen / Gemma, 1e-5 otherwise, when the file has no epsilon
    double eps = (is_phi || is_qwen || is_gemma) ? 1e-6 : 1e-5, theta = 10000.0;
    g->get_f64(prefix + ".attention.layer_norm_rms_epsilon", &eps);
    g->get_f64(prefix + ".rope.freq_base", &theta);
    cfg->norm_eps = (float)eps;
    cfg->rope_freq_base = (float)theta;
    cfg->max_seq_len = (max_seq_len_cap && max_seq_len_cap < ctx) ? max_seq_len_cap : ctx;
    cfg->fused = 1;
    // variants (gguf.rs:553-560, model_runner.rs:417-460)
    uint32_t v = 0;
    if (g->get_u32(prefix + ".attention.sliding_window", &v)) cfg->sliding_window = v;
    if (g->get_u32(prefix + ".rope.dimension_count", &v) && v < cfg->head_dim) cfg->rotary_dim = v;
    double cap = 0.0;
    if (g->get_f64(prefix + ".attn_logit_softcapping", &cap)) cfg->logit_softcap = (float)cap;
    if (g->get_f64(prefix + ".attention.attn_logit_softcapping", &cap)) cfg->attn_logit_softcap = (float)cap;
    if (is_gemma) {
        cfg->norm_weight_offset = 1.0f;
        cfg->geglu = 1;
    }
    if (cfg->rotary_dim % 2) return fail(YULE_ERR_INVALID_ARGUMENT, "gguf: odd rope.dimension_count %u", cfg->rotary_dim);
    // The CPU runner switches to a streaming KV cache (sink tokens + half-context window) from 8192 positions
    // (model_runner.rs:458, :468-481); this backend keeps the flat cache, so longer contexts are capped there.
    if (cfg->max_seq_len >= 8192) cfg->max_seq_len = 8191;
    return YULE_OK;
}

// Creates a runner for the model in `g` on `ctx` and uploads its tensors: raw bytes for the
// matrices, f32 or f16 bytes for the norm weights (the runner converts f16 norms itself).
int32_t yule_cuda_runner_load_gguf(yule_cuda_ctx *ctx, const yule_gguf *g, uint32_t max_seq_len_cap, uint32_t fused,
                                   yule_cuda_runner **out_runner) {
    using namespace yule;
    if (!ctx || !g || !out_runner) return fail(YULE_ERR_INVALID_ARGUMENT, "null argument");
    yule_runner_config cfg;
    int32_t rc = yule_gguf_runner_config(g, max_seq_len_cap, &cfg);
    if (rc) return rc;
    cfg.fused = fused ? 1 : 0;
    YULE_CUDA_TRY(cudaSetDevice(ctx->device));
    yule_cuda_runner *r = nullptr;
    if ((rc = yule_cuda_runner_create(ctx, &cfg, &r))) return rc;

    constexpr size_t kStage = 32u << 20;
    uint8_t *stage[2] = {nullptr, nullptr};
    cudaEvent_t done[2] = {nullptr, nullptr};
    auto cleanup = [&](int32_t code) {
        cudaStreamSynchronize(ctx->stream);
        for (int b = 0; b < 2; b++) {
            if (stage[b]) cudaFreeHost(stage[b]);
            if (done[b]) cudaEventDestroy(done[b]);
        }
        if (code) yule_cuda_runner_destroy(r);
        return code;
    };
    for (int b = 0; b < 2; b++) {
        if (cudaMallocHost((void **)&stage[b], kStage) != cudaSuccess || cudaEventCreateWithFlags(&done[b], cudaEventDisableTiming) != cudaSuccess)
            return cleanup(fail(YULE_ERR_OUT_OF_MEMORY, "gguf: cannot allocate the pinned staging buffers"));
    }
    int which = 0;
    auto upload = [&](const char *name, bool required) -> int32_t {
        const TensorEntry *t = g->find_tensor(name);
        if (!t) return required ? fail(YULE_ERR_MISSING_TENSOR, "tensor not found: %s", name) : YULE_OK;
        if (!is_quantized(t->type) && t->type != YULE_DTYPE_F32 && t->type != YULE_DTYPE_F16)
            return fail(YULE_ERR_UNSUPPORTED_DTYPE, "unsupported dtype for CUDA qmv: GGUF type %u (tensor %s)", t->type, name);
        yule_buffer h = 0;
        int32_t urc = yule_cuda_allocate(ctx, (size_t)t->size_bytes, &h);
        if (urc) return urc;
        runner_adopt_buffer(r, h);  // freed with the runner
        Buffer buf;
        if (!ctx->find(h, &buf, name)) return YULE_ERR_UNKNOWN_BUFFER;
        const uint8_t *src = g->data + g->data_offset + t->offset;
        for (uint64_t off = 0; off < t->size_bytes; off += kStage) {
            const size_t n = (size_t)std::min<uint64_t>(kStage, t->size_bytes - off);
            YULE_CUDA_TRY(cudaEventSynchronize(done[which]));  // the previous copy out of this buffer
            memcpy(stage[which], src + off, n);
            YULE_CUDA_TRY(cudaMemcpyAsync((uint8_t *)buf.ptr + off, stage[which], n, cudaMemcpyHostToDevice, ctx->stream));
            YULE_CUDA_TRY(cudaEventRecord(done[which], ctx->stream));
            which ^= 1;
        }
        return yule_cuda_runner_set_tensor(r, name, h, t->type);
    };
    if ((rc = upload("token_embd.weight", true)) || (rc = upload("output_norm.weight", true)) || (rc = upload("output.weight", false)))
        return cleanup(rc);
    static const char *per_layer[] = {"attn_norm.weight", "attn_q.weight",   "attn_k.weight",  "attn_v.weight",   "attn_output.weight",
                                      "ffn_norm.weight"};
    static const char *dense_ffn[] = {"ffn_gate.weight", "ffn_up.weight", "ffn_down.weight"};
    // optional tensors of the variants (weight_loader.rs:203-218)
    static const char *per_layer_optional[] = {"attn_q.bias", "attn_k.bias", "attn_v.bias", "attn_post_norm.weight", "ffn_post_norm.weight"};
    for (uint32_t l = 0; l < cfg.n_layers; l++) {
        char name[96];
        for (const char *suffix : per_layer) {
            snprintf(name, sizeof(name), "blk.%u.%s", l, suffix);
            if ((rc = upload(name, true))) return cleanup(rc);
        }
        for (const char *suffix : per_layer_optional) {
            snprintf(name, sizeof(name), "blk.%u.%s", l, suffix);
            if ((rc = upload(name, false))) return cleanup(rc);
        }
        if (cfg.n_experts == 0) {
            for (const char *suffix : dense_ffn) {
                snprintf(name, sizeof(name), "blk.%u.%s", l, suffix);
                if ((rc = upload(name, true))) return cleanup(rc);
            }
        } else {
            // the router, then the experts: packed tensors if the file has them, else one tensor per expert
            // (weight_loader.rs:222-260)
            snprintf(name, sizeof(name), "blk.%u.ffn_gate_inp.weight", l);
            if ((rc = upload(name, true))) return cleanup(rc);
            snprintf(name, sizeof(name), "blk.%u.ffn_gate_exps.weight", l);
            if (g->find_tensor(name)) {
                for (const char *proj : {"gate", "up", "down"}) {
                    snprintf(name, sizeof(name), "blk.%u.ffn_%s_exps.weight", l, proj);
                    if ((rc = upload(name, true))) return cleanup(rc);
                }
            } else {
                for (uint32_t e = 0; e < cfg.n_experts; e++)
                    for (const char *proj : {"gate", "up", "down"}) {
                        snprintf(name, sizeof(name), "blk.%u.ffn_%s.%u.weight", l, proj, e);
                        if ((rc = upload(name, true))) return cleanup(rc);
                    }
            }
        }
    }
    rc = cleanup(YULE_OK);
    *out_runner = r;
    return rc;
}

}  // extern "C"
