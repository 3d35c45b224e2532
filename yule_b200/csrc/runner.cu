// runner.cu — forward-pass runner over the C ABI: Yule's `ModelRunner` trait
// (yule-infer/src/model_runner.rs:12-17) for the Llama-family dense path, issuing the op
// sequence of GpuTransformerRunner::forward (yule-infer/src/gpu_runner.rs:296-695).
//
// Two modes (yule_runner_config::fused):
//   0  one kernel per reference dispatch, launched one by one with the position passed by value;
//      the embedding row is dequantised on the device instead of on the CPU (gpu_runner.rs:309-343).
//   1  the same arithmetic with the RMSNorm/Rope/KV-copy/Add dispatches folded into neighbouring
//      kernels, position and token read from device memory, and the whole token step replayed
//      from one CUDA graph.

#include <cmath>
#include <cstdlib>
#include <cstring>
#include <initializer_list>
#include <string>
#include <utility>

#include "internal.h"

using namespace yule;

namespace {

struct Tensor {
    Buffer buf;
    yule_buffer handle = 0;
    uint32_t type = 0;
    bool set = false;
};

struct Layer {
    Tensor attn_norm, attn_q, attn_k, attn_v, attn_output, ffn_norm, ffn_gate, ffn_up, ffn_down;
    // optional tensors of the architecture variants (yule-infer/src/weight_loader.rs:203-218)
    Tensor q_bias, k_bias, v_bias, attn_post_norm, ffn_post_norm;
    const float *attn_norm_f32 = nullptr, *ffn_norm_f32 = nullptr;
    const float *q_bias_f32 = nullptr, *k_bias_f32 = nullptr, *v_bias_f32 = nullptr;
    const float *attn_post_norm_f32 = nullptr, *ffn_post_norm_f32 = nullptr;
    yule_buffer k_cache_h = 0, v_cache_h = 0;
    float *k_cache = nullptr, *v_cache = nullptr;
    // mixture of experts (weight_loader.rs:222-260): the router, then the experts packed in one tensor per projection
    // or one tensor per expert
    Tensor ffn_gate_inp, ffn_gate_exps, ffn_up_exps, ffn_down_exps;
    std::vector<Tensor> gate_e, up_e, down_e;
    const float *router_f32 = nullptr;  // the router as fp32 when the file holds it as F32 / F16
};

}  // namespace

struct yule_cuda_runner {
    yule_cuda_ctx *ctx = nullptr;
    yule_runner_config cfg{};
    std::vector<Layer> layers;
    Tensor token_embd, output_norm, output;
    const float *output_norm_f32 = nullptr;
    std::vector<yule_buffer> owned;  // everything the runner allocated, freed on destroy

    yule_buffer hidden_h = 0, logits_h = 0;
    float *hidden = nullptr, *residual = nullptr, *normed = nullptr, *q = nullptr, *k_tmp = nullptr,
          *v_tmp = nullptr, *attn_out = nullptr, *attn_proj = nullptr, *gate = nullptr, *up = nullptr,
          *ffn_out = nullptr, *logits = nullptr;
    float *moe_logits = nullptr, *moe_w = nullptr;  // mixture of experts: router logits / probabilities, weights of the chosen experts
    uint32_t *moe_sel = nullptr, *h_moe_sel = nullptr;  // the chosen experts (device, pinned host)
    float *rope_cos = nullptr, *rope_sin = nullptr;  // [max_seq_len][head_dim/2], device
    float *attn_scratch = nullptr;  // partial results of the split-KV attention
    uint32_t *attn_tickets = nullptr;
    uint32_t attn_splits = 1;
    bool attn_gqa = false;
    // tensor parallelism with the peer-memory exchange: offsets (floats) of the gathered buffers inside
    // the exchange region
    bool xchg = false;
    size_t x_attn_out = 0, x_hidden = 0, x_gate = 0, x_logits = 0;
    size_t x_pair_hidden = 0, x_pair_gate = 0, x_pair_attn = 0;  // (value, epoch) pair copies (2 floats per element)
    uint32_t *d_state = nullptr;    // [0] token, [1] position, [2] tokens processed since creation
    uint32_t *d_history = nullptr;  // greedy pick made after each position
    uint32_t *h_pinned = nullptr;   // staging for token ids (pinned)
    size_t h_pinned_cap = 0;
    float *h_logits = nullptr;      // pinned landing buffer of the logits read-back (a copy into pageable memory is staged by the driver, slower)

    // Batched prefill on the tensor-core GEMM: chunk buffers, allocated on first use
    uint32_t pf_chunk = 0, pf_splits = 1;
    float *pf_x = nullptr, *pf_q = nullptr, *pf_k = nullptr, *pf_v = nullptr, *pf_att = nullptr, *pf_gate = nullptr,
          *pf_up = nullptr, *pf_attn_scratch = nullptr, *pf_norm = nullptr;
    uint32_t *pf_tokens = nullptr, *pf_tickets = nullptr;

    // Batched decode: `bd_batch` independent sequences advancing one token per step, each with its own KV
    // caches and position; every linear is one GEMM over the batch (the chunk buffers above hold the rows).
    uint32_t bd_batch = 0, bd_rows = 0;  // sequences; rows the GEMMs run over (at least 8)
    std::vector<float *> bd_k, bd_v;     // per layer [batch][max_seq_len][kv_dim]
    float *bd_logits = nullptr;          // [bd_rows][vocab]
    uint32_t *bd_tokens = nullptr, *bd_pos = nullptr, *bd_step = nullptr, *bd_history = nullptr, *bd_prompts = nullptr;
    size_t bd_prompts_cap = 0;
    std::vector<uint32_t> bd_host_pos;
    uint32_t bd_host_step = 0;
    cudaGraphExec_t bd_graph = nullptr;
    uint32_t bd_graph_kernels = 0;

    // tensor parallelism of the GEMM-driven paths (chunked prefill, batched decode): the row matrices that are
    // gathered live in the exchange region (offsets in floats), their exchanges count epochs on a device word
    size_t xb_x = 0, xb_att = 0, xb_gate = 0, xb_up = 0, xb_logits = 0;
    uint32_t xb_rows = 0, xb_logit_rows = 0;  // rows those regions were sized for
    uint32_t *d_btick = nullptr;
    uint32_t *d_seq = nullptr;  // sampled generation: every token of the sequence so far (prompt and picks)

    uint32_t pos = 0;
    bool fused = false;
    bool pdl = true;  // programmatic dependent launch between the kernels of the graph
    uint32_t graph_kernels = 0;  // kernels replayed per graph launch
    bool finalized = false;
    bool created = false;  // yule_cuda_runner_create ran to its end
    bool have_next_token = false;  // d_state[0] holds the greedy continuation
    cudaGraphExec_t graph_exec = nullptr;
    // fused = 2: the token step as one persistent kernel (decode_mega.cu) where the model allows it
    bool mega_wanted = false, mega_tried = false;
    MegaHandle *mega = nullptr;
    std::string mega_why;  // why the persistent kernel does not cover this model (empty when it does)
};

namespace yule {
void runner_adopt_buffer(yule_cuda_runner *r, yule_buffer h) { r->owned.push_back(h); }
}  // namespace yule

namespace {

int32_t alloc_f32(yule_cuda_runner *r, size_t n, float **out, yule_buffer *handle_out = nullptr) {
    yule_buffer h;
    int32_t rc = yule_cuda_allocate(r->ctx, n * sizeof(float), &h);
    if (rc) return rc;
    Buffer b;
    if (!r->ctx->find(h, &b, "runner scratch")) return YULE_ERR_UNKNOWN_BUFFER;
    r->owned.push_back(h);
    *out = (float *)b.ptr;
    if (handle_out) *handle_out = h;
    return YULE_OK;
}

Tensor *slot_for(yule_cuda_runner *r, const char *name) {
    if (!strcmp(name, "token_embd.weight")) return &r->token_embd;
    if (!strcmp(name, "output_norm.weight")) return &r->output_norm;
    if (!strcmp(name, "output.weight")) return &r->output;
    unsigned layer = 0;
    char rest[64];
    if (sscanf(name, "blk.%u.%63s", &layer, rest) != 2 || layer >= r->cfg.n_layers) return nullptr;
    Layer &L = r->layers[layer];
    struct {
        const char *n;
        Tensor *t;
    } slots[] = {{"attn_norm.weight", &L.attn_norm},     {"attn_q.weight", &L.attn_q},
                 {"attn_k.weight", &L.attn_k},           {"attn_v.weight", &L.attn_v},
                 {"attn_output.weight", &L.attn_output}, {"ffn_norm.weight", &L.ffn_norm},
                 {"ffn_gate.weight", &L.ffn_gate},       {"ffn_up.weight", &L.ffn_up},
                 {"ffn_down.weight", &L.ffn_down},       {"attn_q.bias", &L.q_bias},
                 {"attn_k.bias", &L.k_bias},             {"attn_v.bias", &L.v_bias},
                 {"attn_post_norm.weight", &L.attn_post_norm}, {"ffn_post_norm.weight", &L.ffn_post_norm}};
    for (auto &s : slots)
        if (!strcmp(rest, s.n)) return s.t;
    if (r->cfg.n_experts) {
        struct {
            const char *n;
            Tensor *t;
        } moe[] = {{"ffn_gate_inp.weight", &L.ffn_gate_inp}, {"ffn_gate_exps.weight", &L.ffn_gate_exps},
                   {"ffn_up_exps.weight", &L.ffn_up_exps}, {"ffn_down_exps.weight", &L.ffn_down_exps}};
        for (auto &s : moe)
            if (!strcmp(rest, s.n)) return s.t;
        // one tensor per expert: "ffn_gate.E.weight" (weight_loader.rs:228-244)
        unsigned e = 0;
        char which[16], tail[16];
        if (sscanf(rest, "ffn_%15[a-z].%u.%15s", which, &e, tail) == 3 && !strcmp(tail, "weight") && e < r->cfg.n_experts) {
            std::vector<Tensor> *arr = !strcmp(which, "gate") ? &L.gate_e : !strcmp(which, "up") ? &L.up_e : !strcmp(which, "down") ? &L.down_e : nullptr;
            if (arr) {
                if (arr->size() < r->cfg.n_experts) arr->resize(r->cfg.n_experts);
                return &(*arr)[e];
            }
        }
    }
    return nullptr;
}

int32_t check_matrix(const Tensor &t, const char *what, uint32_t layer, uint64_t rows, uint64_t cols) {
    if (!t.set) return fail(YULE_ERR_MISSING_TENSOR, "tensor not found: %s (layer %u)", what, layer);
    if (!is_quantized(t.type))
        return fail(YULE_ERR_UNSUPPORTED_DTYPE, "unsupported dtype for GPU qmv: GGUF type %u (%s)", t.type, what);
    if (cols % block_size(t.type))
        return fail(YULE_ERR_INVALID_ARGUMENT, "%s: %llu columns is not a multiple of the block size", what,
                    (unsigned long long)cols);
    size_t need = tensor_bytes(t.type, rows, cols);
    if (t.buf.size < need)
        return fail(YULE_ERR_OUT_OF_BOUNDS, "%s (layer %u) holds %zu bytes, %zu needed", what, layer, t.buf.size, need);
    return YULE_OK;
}

// Norm weights and biases arrive as F32 or F16 (gpu_runner.rs:183-211 converts on the host; model_runner.rs:259-273,
// :295-310 read both); F16 ones are expanded once on the device.  `offset` is Gemma's norm weight offset
// (model_runner.rs:273: w[i] + offset, formed in f32 exactly as there).
int32_t vector_as_f32(yule_cuda_runner *r, const Tensor &t, const char *what, uint32_t layer, uint32_t n, float offset,
                      const float **out) {
    if (!t.set) return fail(YULE_ERR_MISSING_TENSOR, "tensor not found: %s (layer %u)", what, layer);
    if (t.type != YULE_DTYPE_F32 && t.type != YULE_DTYPE_F16) return fail(YULE_ERR_UNSUPPORTED_DTYPE, "%s must be F32 or F16", what);
    if (t.buf.size < (size_t)n * (t.type == YULE_DTYPE_F32 ? 4 : 2)) return fail(YULE_ERR_OUT_OF_BOUNDS, "%s too small", what);
    if (t.type == YULE_DTYPE_F32 && offset == 0.f) {
        *out = (const float *)t.buf.ptr;
        return YULE_OK;
    }
    float *dst;
    int32_t rc = alloc_f32(r, n, &dst);
    if (rc) return rc;
    uint64_t cnt = 0;
    cudaError_t e = cudaSuccess;
    const float *src = (const float *)t.buf.ptr;
    if (t.type == YULE_DTYPE_F16) {
        e = launch_dequantize((const uint8_t *)t.buf.ptr, YULE_DTYPE_F16, n, dst, r->ctx->stream, &cnt);
        src = dst;
    }
    if (e == cudaSuccess && offset != 0.f) e = launch_elementwise(kElemAddScalar, src, nullptr, dst, n, offset, r->ctx->stream, &cnt);
    r->ctx->launches.fetch_add(cnt);
    if (e != cudaSuccess) return fail_cuda(e, "norm / bias weight conversion");
    *out = dst;
    return YULE_OK;
}
int32_t norm_as_f32(yule_cuda_runner *r, const Tensor &t, const char *what, uint32_t layer, const float **out) {
    return vector_as_f32(r, t, what, layer, r->cfg.dim, r->cfg.norm_weight_offset, out);
}

// Any architecture variant that changes the op sequence (everything except partial RoPE, which lives in the
// RoPE table, and the norm offset, which lives in the converted norm weights).
bool has_bias(const yule_cuda_runner *r) {
    for (const Layer &L : r->layers)
        if (L.q_bias.set || L.k_bias.set || L.v_bias.set) return true;
    return false;
}
bool has_post_norms(const yule_cuda_runner *r) {
    for (const Layer &L : r->layers)
        if (L.attn_post_norm.set || L.ffn_post_norm.set) return true;
    return false;
}
bool is_variant(const yule_cuda_runner *r) {
    const yule_runner_config &c = r->cfg;
    return c.sliding_window || c.attn_logit_softcap != 0.f || c.logit_softcap != 0.f || c.norm_weight_offset != 0.f || c.geglu ||
           c.n_experts != 0 || has_bias(r) || has_post_norms(r);
}

struct Step {
    yule_cuda_runner *r;
    bool pdl = false;
    uint64_t n = 0;
    cudaError_t err = cudaSuccess;
    void ok(cudaError_t e) {
        if (err == cudaSuccess && e != cudaSuccess) err = e;
    }
    // Weights of the kernel(s) that will run next; the tensor-pipe matvecs prefetch them into L2.
    const void *next_w[2] = {nullptr, nullptr};
    uint64_t next_bytes[2] = {0, 0};
    void then(const Tensor *a, const Tensor *b = nullptr) {
        const Tensor *ts[2] = {a, b};
        // measured neutral-to-slightly-negative on the TinyLlama-size step, so off unless asked for
        static const bool enabled = knob("YULE_CUDA_PREFETCH") && atoi(knob("YULE_CUDA_PREFETCH")) != 0;
        if (!enabled) ts[0] = ts[1] = nullptr;
        for (int i = 0; i < 2; i++) {
            const Tensor *t = ts[i];
            next_w[i] = nullptr;
            next_bytes[i] = 0;
            if (!t || !t->set) continue;
            // the bytes the next kernel will actually read: the planar copy when there is one
            next_w[i] = t->buf.planar ? (const void *)t->buf.planar : t->buf.ptr;
            next_bytes[i] = t->buf.planar ? q6k_planar_bytes(t->buf.planar_blocks / (t->buf.planar_cols / 256), t->buf.planar_cols) - 256 : t->buf.size;
        }
    }
    // norm_w set: RMSNorm of x folded into the matvec (only valid when fusable(w, cols) holds)
    void qmv(const Tensor &w, const float *x, float *out, uint32_t rows, uint32_t cols, const float *residual = nullptr,
             const float *norm_w = nullptr, const TpFuse *tp = nullptr) {
        QmvArgs a;
        if (tp) a.tp = *tp;
        a.w = (const uint8_t *)w.buf.ptr;
        a.x = x;
        a.out = out;
        a.n_rows = rows;
        a.n_cols = cols;
        a.type = w.type;
        a.batch = 1;
        a.x_stride = cols;
        a.out_stride = rows;
        a.residual = residual;
        a.pdl = pdl;
        a.planar = w.buf.planar;
        a.norm_w = norm_w;
        a.eps = r->cfg.norm_eps;
        a.status = r->ctx->device_status;
        a.wait_cycles = r->ctx->wait_cycles;
        for (int i = 0; i < 2; i++) {
            a.next_w[i] = next_w[i];
            a.next_bytes[i] = next_bytes[i];
        }
        ok(launch_qmv(a, r->ctx->prop.multiProcessorCount, r->ctx->stream, &n));
    }
};

// Mode 0: one kernel per reference dispatch, token and position baked into the launches as host
// values (gpu_runner.rs:296-695 in order; the embedding row is dequantised on the device).
cudaError_t enqueue_forward_by_value(yule_cuda_runner *r, uint32_t token, uint32_t pos, uint64_t *launches) {
    const yule_runner_config &c = r->cfg;
    cudaStream_t s = r->ctx->stream;
    const uint32_t dim = c.dim, hd = c.head_dim, qdim = c.n_heads * hd, kvdim = c.n_kv_heads * hd, ff = c.ff_dim;
    Step st{r};
    st.ok(launch_embed_gather((const uint8_t *)r->token_embd.buf.ptr, r->token_embd.type, dim, token, nullptr,
                              r->hidden, s, &st.n));
    // Gemma: embeddings scaled by sqrt(dim) (model_runner.rs:568-574)
    if (c.norm_weight_offset > 0.f) st.ok(launch_elementwise(kElemScale, r->hidden, nullptr, r->hidden, dim, sqrtf((float)dim), s, &st.n));
    // RoPE angles of this position; with partial RoPE only the first rotary_dim/2 pairs turn (cos 1, sin 0 beyond)
    RopeAngles ang;
    const uint32_t half = hd / 2, rot = (c.rotary_dim && c.rotary_dim < hd) ? c.rotary_dim : hd;
    for (uint32_t i = 0; i < half; i++) {
        if (i < rot / 2) {
            float freq = 1.0f / powf(c.rope_freq_base, 2.0f * (float)i / (float)rot);
            float theta = (float)pos * freq;
            ang.cos[i] = cosf(theta);
            ang.sin[i] = sinf(theta);
        } else {
            ang.cos[i] = 1.0f;
            ang.sin[i] = 0.0f;
        }
    }
    for (uint32_t l = 0; l < c.n_layers; l++) {
        Layer &L = r->layers[l];
        st.ok(cudaMemcpyAsync(r->residual, r->hidden, (size_t)dim * 4, cudaMemcpyDeviceToDevice, s));
        st.ok(launch_rms_norm(r->hidden, L.attn_norm_f32, r->normed, dim, c.norm_eps, s, &st.n));
        st.qmv(L.attn_q, r->normed, r->q, qdim, dim);
        st.qmv(L.attn_k, r->normed, r->k_tmp, kvdim, dim);
        st.qmv(L.attn_v, r->normed, r->v_tmp, kvdim, dim);
        // Q/K/V bias (model_runner.rs:640-651)
        if (L.q_bias_f32) st.ok(launch_elementwise(kElemAddVec, r->q, L.q_bias_f32, r->q, qdim, 0.f, s, &st.n));
        if (L.k_bias_f32) st.ok(launch_elementwise(kElemAddVec, r->k_tmp, L.k_bias_f32, r->k_tmp, kvdim, 0.f, s, &st.n));
        if (L.v_bias_f32) st.ok(launch_elementwise(kElemAddVec, r->v_tmp, L.v_bias_f32, r->v_tmp, kvdim, 0.f, s, &st.n));
        st.ok(launch_rope_angles(r->q, r->k_tmp, hd, c.n_heads, c.n_kv_heads, ang, s, &st.n));
        const size_t off = (size_t)pos * kvdim;
        st.ok(cudaMemcpyAsync(L.k_cache + off, r->k_tmp, (size_t)kvdim * 4, cudaMemcpyDeviceToDevice, s));
        st.ok(cudaMemcpyAsync(L.v_cache + off, r->v_tmp, (size_t)kvdim * 4, cudaMemcpyDeviceToDevice, s));
        st.ok(launch_multihead_attention(r->q, L.k_cache, L.v_cache, r->attn_out, hd, pos + 1, nullptr, pos + 1,
                                         c.n_heads, c.n_kv_heads, kvdim, s, &st.n, false, c.sliding_window, c.attn_logit_softcap));
        st.qmv(L.attn_output, r->attn_out, r->attn_proj, dim, qdim);
        // post-attention norm (Gemma2, model_runner.rs:764-779)
        if (L.attn_post_norm_f32) {
            st.ok(launch_rms_norm(r->attn_proj, L.attn_post_norm_f32, r->ffn_out, dim, c.norm_eps, s, &st.n));
            st.ok(launch_add(r->residual, r->ffn_out, r->hidden, dim, s, &st.n));
        } else {
            st.ok(launch_add(r->residual, r->attn_proj, r->hidden, dim, s, &st.n));
        }
        st.ok(cudaMemcpyAsync(r->residual, r->hidden, (size_t)dim * 4, cudaMemcpyDeviceToDevice, s));
        st.ok(launch_rms_norm(r->hidden, L.ffn_norm_f32, r->normed, dim, c.norm_eps, s, &st.n));
        if (c.n_experts) {
            // Mixture of experts (model_runner.rs:813-958).  Router, softmax, the n_experts_used most probable
            // experts and their renormalised weights on the device; the chosen indices come back to the host (a few
            // bytes per layer), which picks the experts' weights; their SwiGLU FFNs are summed with the device-side
            // weights in the order of decreasing probability, as the CPU runner does.
            if (L.router_f32)
                st.ok(launch_matvec_f32(L.router_f32, r->normed, r->moe_logits, c.n_experts, dim, s, &st.n));
            else
                st.qmv(L.ffn_gate_inp, r->normed, r->moe_logits, c.n_experts, dim);
            st.ok(launch_moe_route(r->moe_logits, c.n_experts, c.n_experts_used, r->moe_sel, r->moe_w, s, &st.n));
            st.ok(cudaMemcpyAsync(r->h_moe_sel, r->moe_sel, (size_t)c.n_experts_used * 4, cudaMemcpyDeviceToHost, s));
            st.ok(cudaMemsetAsync(r->ffn_out, 0, (size_t)dim * 4, s));
            if (st.err == cudaSuccess) st.ok(cudaStreamSynchronize(s));
            for (uint32_t k = 0; k < c.n_experts_used && st.err == cudaSuccess; k++) {
                const uint32_t e = r->h_moe_sel[k] < c.n_experts ? r->h_moe_sel[k] : 0;
                Tensor g, u, d;
                if (!L.gate_e.empty() && L.gate_e[e].set) {
                    g = L.gate_e[e];
                    u = L.up_e[e];
                    d = L.down_e[e];
                } else {
                    // packed: expert e is the e-th of n_experts equal slices of each tensor (:890-918)
                    auto slice = [&](const Tensor &t, uint64_t rows, uint64_t cols) {
                        Tensor o = t;
                        const size_t bytes = tensor_bytes(t.type, rows, cols);
                        o.buf.ptr = (char *)t.buf.ptr + (size_t)e * bytes;
                        o.buf.size = bytes;
                        o.buf.planar = nullptr;  // a planar copy, if any, belongs to the whole tensor
                        return o;
                    };
                    g = slice(L.ffn_gate_exps, ff, dim);
                    u = slice(L.ffn_up_exps, ff, dim);
                    d = slice(L.ffn_down_exps, dim, ff);
                }
                st.qmv(g, r->normed, r->gate, ff, dim);
                st.qmv(u, r->normed, r->up, ff, dim);
                st.ok(launch_silu_mul(r->gate, r->up, r->gate, ff, s, &st.n));  // always SwiGLU here (:876-881)
                st.qmv(d, r->gate, r->attn_proj, dim, ff);
                st.ok(launch_axpy_dev(r->moe_w + k, r->attn_proj, r->ffn_out, dim, s, &st.n));  // ffn_out += w_k · expert_out
            }
        } else {
        st.qmv(L.ffn_gate, r->normed, r->gate, ff, dim);
        st.qmv(L.ffn_up, r->normed, r->up, ff, dim);
        if (c.geglu)  // model_runner.rs:974-978
            st.ok(launch_elementwise(kElemGeluMul, r->gate, r->up, r->gate, ff, 0.f, s, &st.n));
        else
            st.ok(launch_silu_mul(r->gate, r->up, r->gate, ff, s, &st.n));
        st.qmv(L.ffn_down, r->gate, r->ffn_out, dim, ff);
        }
        // post-FFN norm (Gemma2, model_runner.rs:985-999)
        if (L.ffn_post_norm_f32) {
            st.ok(launch_rms_norm(r->ffn_out, L.ffn_post_norm_f32, r->attn_proj, dim, c.norm_eps, s, &st.n));
            st.ok(launch_add(r->residual, r->attn_proj, r->hidden, dim, s, &st.n));
        } else {
            st.ok(launch_add(r->residual, r->ffn_out, r->hidden, dim, s, &st.n));
        }
    }
    st.ok(launch_rms_norm(r->hidden, r->output_norm_f32, r->normed, dim, c.norm_eps, s, &st.n));
    const Tensor &out_w = r->output.set ? r->output : r->token_embd;
    st.qmv(out_w, r->normed, r->logits, c.vocab_size, dim);
    // final logit softcap (Gemma2, model_runner.rs:1027-1032)
    if (c.logit_softcap != 0.f) st.ok(launch_elementwise(kElemSoftcap, r->logits, nullptr, r->logits, c.vocab_size, c.logit_softcap, s, &st.n));
    *launches += st.n;
    return st.err;
}

// Mode 1: the same token step with the small dispatches folded into the matvecs, token and
// position read from d_state so that one captured graph serves every position, and every launch
// marked for programmatic dependent launch.
//   embed → per layer { [RMSNorm + Q/K/V] → [RoPE + KV write] → attention → [o-proj + residual]
//                       → [RMSNorm + gate/up + SiLU·mul] → [down + residual] }
//         → [RMSNorm + output] → [argmax + history + position advance]
// Brackets are single kernels when the matrices involved are Q4_K; other formats fall back to a
// separate RMSNorm / SiLU·mul kernel around the per-matrix matvec.
cudaError_t enqueue_forward_graph(yule_cuda_runner *r, uint64_t *launches) {
    const yule_runner_config &c = r->cfg;
    cudaStream_t s = r->ctx->stream;
    const int sms = r->ctx->prop.multiProcessorCount;
    const bool pdl = r->pdl;
    const uint32_t dim = c.dim, hd = c.head_dim, qdim = c.n_heads * hd, kvdim = c.n_kv_heads * hd, ff = c.ff_dim;
    // Tensor parallelism: this rank computes rows [R*n/N, (R+1)*n/N) of every matrix — its heads, its
    // slice of the FFN, its slice of the vocabulary — into its slice of the full-size activation
    // buffers, which are then all-gathered in place.
    const uint32_t N = r->ctx->tp_world ? r->ctx->tp_world : 1, R = r->ctx->tp_rank;
    const uint32_t qdim_l = qdim / N, kvdim_l = kvdim / N, ff_l = ff / N, dim_l = dim / N, vocab_l = c.vocab_size / N;
    const uint32_t heads_l = c.n_heads / N, kvh_l = c.n_kv_heads / N;
    Step st{r};
    st.pdl = pdl;
    // All-gather number `k` of layer `layer` (k = 4: the logits).  With the peer exchange each gather
    // has its own flag slot and an epoch derived from the token counter in d_state[2].
    const uint32_t epochs_per_token = 4 * c.n_layers + 1;
    const bool skip_gather = knob("YULE_CUDA_SKIP") && (strtoul(knob("YULE_CUDA_SKIP"), nullptr, 0) & 512);
    auto gather = [&](float *buf, size_t x_off, uint32_t per_rank, uint32_t layer, uint32_t k) {
        if (N <= 1 || skip_gather) return;
        if (r->xchg)
            st.ok(tp_exchange(r->ctx, x_off, per_rank, k, r->d_state + 2, epochs_per_token, k == 4 ? 4 * c.n_layers : 4 * layer + k,
                              pdl, &st.n));
        else
            st.ok(tp_all_gather_inplace(r->ctx, buf, per_rank));
    };
    const uint32_t *tok_ptr = r->d_state, *pos_ptr = r->d_state + 1;
    // Timing aid: YULE_CUDA_SKIP is a bit mask of kernel classes to leave out of the graph (results
    // are then meaningless); the time that disappears is that class's cost inside the real step.
    const unsigned skip = knob("YULE_CUDA_SKIP") ? (unsigned)strtoul(knob("YULE_CUDA_SKIP"), nullptr, 0) : 0u;
    auto all_q4k = [&](std::initializer_list<const Tensor *> ts, uint32_t cols) {
        for (const Tensor *t : ts)
            if (t->type != YULE_DTYPE_Q4_K) return false;
        return q4k_mma_supported(cols, 1);
    };
    // Matrices that can share one launch of the tensor-pipe kernel: all Q4_K, or (single GPU) all Q5_K.
    auto all_mma = [&](std::initializer_list<const Tensor *> ts, uint32_t cols) {
        if (all_q4k(ts, cols)) return true;
        if (N > 1) return false;
        for (const Tensor *t : ts)
            if (t->type != YULE_DTYPE_Q5_K || (reinterpret_cast<uintptr_t>(t->buf.ptr) & 15)) return false;
        return q4k_mma_supported(cols, 1);
    };
    // Tensor parallelism folded into the Q4_K matvecs: when both the kernel that produces a gathered vector
    // and the one that consumes it are the Q4_K tensor-pipe kernel, the producer stores (value, epoch) pairs
    // straight into every rank's pair buffer as its rows are reduced and the consumer polls the pairs while it
    // stages x: no exchange launch, no fence, no flag.  YULE_TP_FUSE=0 keeps the exchange kernel everywhere.
    // (the folded exchange assumes the Llama op sequence: a variant model takes the exchange kernel everywhere)
    const bool tp_fuse = N > 1 && r->xchg && !skip_gather && !is_variant(r) && !(knob("YULE_TP_FUSE") && atoi(knob("YULE_TP_FUSE")) == 0);
    auto is_q4k_mma = [&](const Tensor &t, uint32_t cols) { return t.type == YULE_DTYPE_Q4_K && q4k_mma_supported(cols, 1); };
    auto epoch_index = [&](uint32_t layer, uint32_t k) { return k == 4 ? 4 * c.n_layers : 4 * layer + k; };
    auto push_of = [&](size_t pair_off, uint32_t per_rank, uint32_t layer, uint32_t k) {
        TpFuse f;
        tp_fuse_push(r->ctx, pair_off, per_rank, r->d_state + 2, epochs_per_token, epoch_index(layer, k), &f);
        return f;
    };
    auto add_wait = [&](TpFuse &f, size_t pair_off, uint32_t layer, uint32_t k) {
        tp_fuse_wait(r->ctx, pair_off, r->d_state + 2, epochs_per_token, epoch_index(layer, k), &f);
    };
    // which gathers are folded: 0 after attention (grouped-query kernel, consumer o-proj),
    // 1 after o-proj (consumer gate/up), 2 after gate/up (consumer down),
    // 3 after down (consumer: next layer's Q/K/V, or the output matrix after the last layer)
    auto folded = [&](uint32_t layer, uint32_t k) {
        if (!tp_fuse) return false;
        const Layer &L = r->layers[layer];
        const Tensor &ow = r->output.set ? r->output : r->token_embd;
        if (k == 0) return r->attn_gqa && attn_decode_supported(hd) && is_q4k_mma(L.attn_output, qdim);
        if (k == 1) return is_q4k_mma(L.attn_output, qdim) && all_q4k({&L.ffn_gate, &L.ffn_up}, dim);
        if (k == 2) return all_q4k({&L.ffn_gate, &L.ffn_up}, dim) && is_q4k_mma(L.ffn_down, ff);
        if (k == 3) {
            if (!is_q4k_mma(L.ffn_down, ff)) return false;
            if (layer + 1 < c.n_layers) {
                const Layer &Nx = r->layers[layer + 1];
                return all_q4k({&Nx.attn_q, &Nx.attn_k, &Nx.attn_v}, dim);
            }
            return all_q4k({&ow}, dim);
        }
        return false;
    };
    // x → (optional RMSNorm) → up to three Q4_K matrices in one launch
    auto fused = [&](std::initializer_list<std::pair<const Tensor *, std::pair<float *, uint32_t>>> segs, const float *x,
                     uint32_t cols, const float *norm_w, const float *residual, bool pair, const TpFuse *tp = nullptr) {
        Q4kFused f;
        if (tp) f.tp = *tp;
        uint32_t i = 0;
        f.q5 = segs.begin()->first->type == YULE_DTYPE_Q5_K;
        for (auto &sg : segs) {
            f.w[i] = (const uint8_t *)sg.first->buf.ptr;
            f.out[i] = sg.second.first;
            f.rows[i] = sg.second.second;
            f.out_stride[i] = sg.second.second;
            i++;
        }
        f.n_seg = i;
        f.x = x;
        f.x_stride = cols;
        f.n_cols = cols;
        f.batch = 1;
        f.norm_w = norm_w;
        f.eps = c.norm_eps;
        f.residual = residual;
        f.swiglu_pair = pair;
        f.pdl = pdl;
        f.status = r->ctx->device_status;
        f.wait_cycles = r->ctx->wait_cycles;
        for (int k = 0; k < 2; k++) {
            f.next_w[k] = st.next_w[k];
            f.next_bytes[k] = st.next_bytes[k];
        }
        st.ok(launch_q4k_mma(f, sms, s, &st.n));
    };

    if (!(skip & 256))
        st.ok(launch_embed_gather((const uint8_t *)r->token_embd.buf.ptr, r->token_embd.type, dim, 0, tok_ptr,
                                  r->hidden, s, &st.n, pdl));
    // Gemma: embeddings scaled by sqrt(dim) (model_runner.rs:568-574)
    if (c.norm_weight_offset > 0.f)
        st.ok(launch_elementwise(kElemScale, r->hidden, nullptr, r->hidden, dim, sqrtf((float)dim), s, &st.n, pdl));
    for (uint32_t l = 0; l < c.n_layers; l++) {
        Layer &L = r->layers[l];
        const Tensor &out_w_ = r->output.set ? r->output : r->token_embd;
        st.then(&L.attn_output);  // while Q/K/V and attention run, o-proj's weights come in
        if (skip & 1) {
        } else if (all_mma({&L.attn_q, &L.attn_k, &L.attn_v}, dim)) {
            TpFuse tq;
            if (l > 0 && folded(l - 1, 3)) add_wait(tq, r->x_pair_hidden, l - 1, 3);
            fused({{&L.attn_q, {r->q, qdim_l}}, {&L.attn_k, {r->k_tmp, kvdim_l}}, {&L.attn_v, {r->v_tmp, kvdim_l}}},
                  r->hidden, dim, L.attn_norm_f32, nullptr, false, &tq);
        } else {
            st.ok(launch_rms_norm(r->hidden, L.attn_norm_f32, r->normed, dim, c.norm_eps, s, &st.n, pdl));
            st.qmv(L.attn_q, r->normed, r->q, qdim_l, dim);
            st.qmv(L.attn_k, r->normed, r->k_tmp, kvdim_l, dim);
            st.qmv(L.attn_v, r->normed, r->v_tmp, kvdim_l, dim);
        }
        // Q/K/V bias (model_runner.rs:640-651); tensor parallelism: this rank's rows of each
        if (L.q_bias_f32) st.ok(launch_elementwise(kElemAddVec, r->q, L.q_bias_f32 + (size_t)R * qdim_l, r->q, qdim_l, 0.f, s, &st.n, pdl));
        if (L.k_bias_f32) st.ok(launch_elementwise(kElemAddVec, r->k_tmp, L.k_bias_f32 + (size_t)R * kvdim_l, r->k_tmp, kvdim_l, 0.f, s, &st.n, pdl));
        if (L.v_bias_f32) st.ok(launch_elementwise(kElemAddVec, r->v_tmp, L.v_bias_f32 + (size_t)R * kvdim_l, r->v_tmp, kvdim_l, 0.f, s, &st.n, pdl));
        float *attn_out_l = r->attn_out + (size_t)R * qdim_l;
        if (attn_decode_supported(hd)) {
            // Rope dispatch + both KV copies + MultiheadAttn in one launch
            AttnDecode a;
            a.q = r->q;
            a.k_new = r->k_tmp;
            a.v_new = r->v_tmp;
            a.k_cache = L.k_cache;
            a.v_cache = L.v_cache;
            a.cos_table = r->rope_cos;
            a.sin_table = r->rope_sin;
            a.pos_ptr = pos_ptr;
            a.out = attn_out_l;
            a.scratch = r->attn_scratch;
            a.tickets = r->attn_tickets;
            a.hd = hd;
            a.n_heads = heads_l;
            a.n_kv_heads = kvh_l;
            a.kv_stride = kvdim_l;
            a.n_splits = r->attn_splits;
            a.gqa = r->attn_gqa;
            a.max_seq_len = c.max_seq_len;
            a.min_chunk = knob("YULE_CUDA_ATTN_MIN_CHUNK") ? (uint32_t)atoi(knob("YULE_CUDA_ATTN_MIN_CHUNK")) : 32;
            a.pdl = pdl;
            a.window = c.sliding_window;
            a.softcap = c.attn_logit_softcap;
            if (folded(l, 0)) a.tp = push_of(r->x_pair_attn, qdim_l, l, 0);
            if (!(skip & 4)) st.ok(launch_attn_decode(a, s, &st.n));
        } else {
            if (!(skip & 2))
                st.ok(launch_rope_kv_write(r->q, r->k_tmp, r->v_tmp, L.k_cache, L.v_cache, r->rope_cos, r->rope_sin,
                                           pos_ptr, hd, heads_l, kvh_l, s, &st.n, pdl));
            if (!(skip & 4))
                st.ok(launch_multihead_attention(r->q, L.k_cache, L.v_cache, attn_out_l, hd, 0, pos_ptr, c.max_seq_len,
                                                 heads_l, kvh_l, kvdim_l, s, &st.n, pdl, c.sliding_window, c.attn_logit_softcap));
        }
        if (!folded(l, 0)) gather(r->attn_out, r->x_attn_out, qdim_l, l, 0);
        float *hidden_l = r->hidden + (size_t)R * dim_l;
        // hidden = hidden + W_o · attn_out (the Add dispatch folded into the matvec epilogue)
        st.then(&L.ffn_gate, &L.ffn_up);
        {
            TpFuse to;
            if (folded(l, 1)) to = push_of(r->x_pair_hidden, dim_l, l, 1);
            if (folded(l, 0)) add_wait(to, r->x_pair_attn, l, 0);
            if (L.attn_post_norm_f32) {
                // post-attention norm (Gemma2, model_runner.rs:764-779): project, normalise, then add the residual
                st.qmv(L.attn_output, r->attn_out, r->attn_proj, dim, qdim);
                st.ok(launch_rms_norm(r->attn_proj, L.attn_post_norm_f32, r->ffn_out, dim, c.norm_eps, s, &st.n, pdl));
                st.ok(launch_elementwise(kElemAddVec, r->hidden, r->ffn_out, r->hidden, dim, 0.f, s, &st.n, pdl));
            } else if (!(skip & 8)) {
                st.qmv(L.attn_output, r->attn_out, hidden_l, dim_l, qdim, hidden_l, nullptr, &to);
            }
        }
        if (!folded(l, 1)) gather(r->hidden, r->x_hidden, dim_l, l, 1);
        st.then(&L.ffn_down);
        if (skip & 16) {
        } else if (!c.geglu && all_mma({&L.ffn_gate, &L.ffn_up}, dim)) {
            TpFuse tg;
            if (folded(l, 2)) tg = push_of(r->x_pair_gate, ff_l, l, 2);
            if (folded(l, 1)) add_wait(tg, r->x_pair_hidden, l, 1);
            fused({{&L.ffn_gate, {r->gate + (size_t)R * ff_l, ff_l}}, {&L.ffn_up, {r->up, ff_l}}}, r->hidden, dim,
                  L.ffn_norm_f32, nullptr, true, &tg);
        } else {
            st.ok(launch_rms_norm(r->hidden, L.ffn_norm_f32, r->normed, dim, c.norm_eps, s, &st.n, pdl));
            st.qmv(L.ffn_gate, r->normed, r->gate + (size_t)R * ff_l, ff_l, dim);
            st.qmv(L.ffn_up, r->normed, r->up, ff_l, dim);
            if (c.geglu)  // model_runner.rs:974-978
                st.ok(launch_elementwise(kElemGeluMul, r->gate + (size_t)R * ff_l, r->up, r->gate + (size_t)R * ff_l, ff_l, 0.f, s, &st.n, pdl));
            else
                st.ok(launch_silu_mul(r->gate + (size_t)R * ff_l, r->up, r->gate + (size_t)R * ff_l, ff_l, s, &st.n, pdl));
        }
        if (!folded(l, 2)) gather(r->gate, r->x_gate, ff_l, l, 2);
        // during down-proj: the next layer's Q and K/V (or the output matrix after the last layer)
        if (l + 1 < c.n_layers)
            st.then(&r->layers[l + 1].attn_q, &r->layers[l + 1].attn_k);
        else
            st.then(&out_w_);
        {
            TpFuse td;
            if (folded(l, 3)) td = push_of(r->x_pair_hidden, dim_l, l, 3);
            if (folded(l, 2)) add_wait(td, r->x_pair_gate, l, 2);
            if (L.ffn_post_norm_f32) {
                // post-FFN norm (Gemma2, model_runner.rs:985-999)
                st.qmv(L.ffn_down, r->gate, r->ffn_out, dim, ff);
                st.ok(launch_rms_norm(r->ffn_out, L.ffn_post_norm_f32, r->attn_proj, dim, c.norm_eps, s, &st.n, pdl));
                st.ok(launch_elementwise(kElemAddVec, r->hidden, r->attn_proj, r->hidden, dim, 0.f, s, &st.n, pdl));
            } else if (!(skip & 32)) {
                st.qmv(L.ffn_down, r->gate, hidden_l, dim_l, ff, hidden_l, nullptr, &td);
            }
        }
        if (!folded(l, 3)) gather(r->hidden, r->x_hidden, dim_l, l, 3);
    }
    st.then(nullptr);
    const Tensor &out_w = r->output.set ? r->output : r->token_embd;
    if (skip & 64) {
    } else if (all_mma({&out_w}, dim)) {
        TpFuse tw;
        if (c.n_layers && folded(c.n_layers - 1, 3)) add_wait(tw, r->x_pair_hidden, c.n_layers - 1, 3);
        fused({{&out_w, {r->logits + (size_t)R * vocab_l, vocab_l}}}, r->hidden, dim, r->output_norm_f32, nullptr, false, &tw);
    } else if (out_w.type == YULE_DTYPE_Q6_K && out_w.buf.planar && q6k_mma_supported(dim)) {
        st.qmv(out_w, r->hidden, r->logits + (size_t)R * vocab_l, vocab_l, dim, nullptr, r->output_norm_f32);
    } else {
        st.ok(launch_rms_norm(r->hidden, r->output_norm_f32, r->normed, dim, c.norm_eps, s, &st.n, pdl));
        st.qmv(out_w, r->normed, r->logits + (size_t)R * vocab_l, vocab_l, dim);
    }
    gather(r->logits, r->x_logits, vocab_l, 0, 4);
    // final logit softcap (Gemma2, model_runner.rs:1027-1032)
    if (c.logit_softcap != 0.f)
        st.ok(launch_elementwise(kElemSoftcap, r->logits, nullptr, r->logits, c.vocab_size, c.logit_softcap, s, &st.n, pdl));
    if (!(skip & 128)) st.ok(launch_argmax(r->logits, c.vocab_size, r->d_state, r->d_history, s, &st.n, pdl));
    *launches += st.n;
    return st.err;
}

int32_t finalize(yule_cuda_runner *r) {
    if (r->finalized) return YULE_OK;
    const yule_runner_config &c = r->cfg;
    const uint32_t N = r->ctx->tp_world ? r->ctx->tp_world : 1;
    // rows this rank holds of each matrix (all of them when single-GPU); input widths stay global
    const uint32_t dim = c.dim, hd = c.head_dim, qdim_in = c.n_heads * hd, ff_in = c.ff_dim;
    const uint32_t qdim = qdim_in / N, kvdim = c.n_kv_heads * hd / N, ff = ff_in / N, dim_rows = dim / N,
                   vocab_rows = c.vocab_size / N;
    int32_t rc;
    if (N > 1 && !r->output.set)
        return fail(YULE_ERR_MISSING_TENSOR, "tensor parallelism needs output.weight (a tied embedding cannot be row-sharded)");
    if (N > 1 && has_post_norms(r))
        return fail(YULE_ERR_INVALID_ARGUMENT, "tensor parallelism does not cover the post-attention / post-FFN norms (they need the whole projected vector)");
    if (!r->token_embd.set) return fail(YULE_ERR_MISSING_TENSOR, "tensor not found: token_embd.weight");
    {
        uint32_t bs = block_size(r->token_embd.type);
        if (bs == 0 || dim % bs) return fail(YULE_ERR_UNSUPPORTED_DTYPE, "token_embd dtype %u unsupported", r->token_embd.type);
        size_t need = (size_t)c.vocab_size * (dim / bs) * block_bytes(r->token_embd.type);
        if (r->token_embd.buf.size < need) return fail(YULE_ERR_OUT_OF_BOUNDS, "token_embd.weight too small");
    }
    if ((rc = norm_as_f32(r, r->output_norm, "output_norm.weight", 0, &r->output_norm_f32))) return rc;
    if (r->output.set) {
        if ((rc = check_matrix(r->output, "output.weight", 0, vocab_rows, dim))) return rc;
    } else if ((rc = check_matrix(r->token_embd, "token_embd.weight (as output)", 0, c.vocab_size, dim))) {
        return rc;
    }
    for (uint32_t l = 0; l < c.n_layers; l++) {
        Layer &L = r->layers[l];
        if ((rc = norm_as_f32(r, L.attn_norm, "attn_norm.weight", l, &L.attn_norm_f32))) return rc;
        if ((rc = norm_as_f32(r, L.ffn_norm, "ffn_norm.weight", l, &L.ffn_norm_f32))) return rc;
        if (L.attn_post_norm.set && (rc = norm_as_f32(r, L.attn_post_norm, "attn_post_norm.weight", l, &L.attn_post_norm_f32))) return rc;
        if (L.ffn_post_norm.set && (rc = norm_as_f32(r, L.ffn_post_norm, "ffn_post_norm.weight", l, &L.ffn_post_norm_f32))) return rc;
        if (L.q_bias.set && (rc = vector_as_f32(r, L.q_bias, "attn_q.bias", l, qdim_in, 0.f, &L.q_bias_f32))) return rc;
        if (L.k_bias.set && (rc = vector_as_f32(r, L.k_bias, "attn_k.bias", l, c.n_kv_heads * hd, 0.f, &L.k_bias_f32))) return rc;
        if (L.v_bias.set && (rc = vector_as_f32(r, L.v_bias, "attn_v.bias", l, c.n_kv_heads * hd, 0.f, &L.v_bias_f32))) return rc;
        if ((rc = check_matrix(L.attn_q, "attn_q.weight", l, qdim, dim))) return rc;
        if ((rc = check_matrix(L.attn_k, "attn_k.weight", l, kvdim, dim))) return rc;
        if ((rc = check_matrix(L.attn_v, "attn_v.weight", l, kvdim, dim))) return rc;
        if ((rc = check_matrix(L.attn_output, "attn_output.weight", l, dim_rows, qdim_in))) return rc;
        if (c.n_experts) {
            // router: F32 / F16 (expanded to fp32 once) or a block format; experts: per expert or packed
            if (!L.ffn_gate_inp.set) return fail(YULE_ERR_MISSING_TENSOR, "tensor not found: ffn_gate_inp.weight (layer %u)", l);
            if (L.ffn_gate_inp.type == YULE_DTYPE_F32 || L.ffn_gate_inp.type == YULE_DTYPE_F16) {
                if ((rc = vector_as_f32(r, L.ffn_gate_inp, "ffn_gate_inp.weight", l, c.n_experts * dim, 0.f, &L.router_f32))) return rc;
            } else if ((rc = check_matrix(L.ffn_gate_inp, "ffn_gate_inp.weight", l, c.n_experts, dim))) {
                return rc;
            }
            const bool per_expert = !L.gate_e.empty();
            if (per_expert) {
                if (L.up_e.size() < c.n_experts || L.down_e.size() < c.n_experts || L.gate_e.size() < c.n_experts)
                    return fail(YULE_ERR_MISSING_TENSOR, "layer %u: expert tensors missing", l);
                for (uint32_t e = 0; e < c.n_experts; e++)
                    if ((rc = check_matrix(L.gate_e[e], "ffn_gate.E.weight", l, ff, dim)) || (rc = check_matrix(L.up_e[e], "ffn_up.E.weight", l, ff, dim)) ||
                        (rc = check_matrix(L.down_e[e], "ffn_down.E.weight", l, dim, ff)))
                        return rc;
            } else if ((rc = check_matrix(L.ffn_gate_exps, "ffn_gate_exps.weight", l, (uint64_t)c.n_experts * ff, dim)) ||
                       (rc = check_matrix(L.ffn_up_exps, "ffn_up_exps.weight", l, (uint64_t)c.n_experts * ff, dim)) ||
                       (rc = check_matrix(L.ffn_down_exps, "ffn_down_exps.weight", l, (uint64_t)c.n_experts * dim, ff))) {
                return rc;
            }
            continue;
        }
        if ((rc = check_matrix(L.ffn_gate, "ffn_gate.weight", l, ff, dim))) return rc;
        if ((rc = check_matrix(L.ffn_up, "ffn_up.weight", l, ff, dim))) return rc;
        if ((rc = check_matrix(L.ffn_down, "ffn_down.weight", l, dim_rows, ff_in))) return rc;
    }
    // Device-side planar copies for the formats whose fast kernel wants one (Q6_K).
    auto prepare = [&](Tensor &t, uint32_t rows, uint32_t cols) -> int32_t {
        if (!t.set || t.type != YULE_DTYPE_Q6_K) return YULE_OK;
        int32_t prc = yule_cuda_prepare_weights(r->ctx, t.handle, t.type, rows, cols);
        if (prc) return prc;
        if (!r->ctx->find(t.handle, &t.buf, "prepared tensor")) return YULE_ERR_UNKNOWN_BUFFER;
        return YULE_OK;
    };
    if ((rc = prepare(r->output.set ? r->output : r->token_embd, vocab_rows, dim))) return rc;
    for (uint32_t l = 0; l < c.n_layers; l++) {
        Layer &L = r->layers[l];
        if ((rc = prepare(L.attn_q, qdim, dim)) || (rc = prepare(L.attn_k, kvdim, dim)) ||
            (rc = prepare(L.attn_v, kvdim, dim)) || (rc = prepare(L.attn_output, dim_rows, qdim_in)) ||
            (rc = prepare(L.ffn_gate, ff, dim)) || (rc = prepare(L.ffn_up, ff, dim)) ||
            (rc = prepare(L.ffn_down, dim_rows, ff_in)))
            return rc;
    }
    r->finalized = true;
    return YULE_OK;
}

// fused = 2: describes the model to the persistent decode kernel.  A model it does not cover keeps the
// multi-kernel graph (the reason is kept for yule_cuda_runner_token_step_kind).
int32_t setup_mega(yule_cuda_runner *r) {
    const yule_runner_config &c = r->cfg;
    if (is_variant(r)) {
        r->mega_why = "architecture variant";
        return YULE_OK;
    }
    MegaModel m;
    m.dim = c.dim;
    m.head_dim = c.head_dim;
    m.n_heads = c.n_heads;
    m.n_kv_heads = c.n_kv_heads;
    m.ff_dim = c.ff_dim;
    m.vocab = c.vocab_size;
    m.n_layers = c.n_layers;
    m.max_seq_len = c.max_seq_len;
    m.eps = c.norm_eps;
    auto tensor = [](const Tensor &t, uint32_t cols) {
        MegaTensor o;
        o.type = t.type;
        // Q6_K travels as its row-planar copy (finalize() built it); a Q6_K tensor without one is not covered
        o.ptr = t.type == YULE_DTYPE_Q6_K ? (t.buf.planar && t.buf.planar_cols == cols ? (const uint8_t *)t.buf.planar : nullptr)
                                          : (const uint8_t *)t.buf.ptr;
        return o;
    };
    const uint32_t qdim = c.n_heads * c.head_dim;
    m.embd = (const uint8_t *)r->token_embd.buf.ptr;
    m.embd_type = r->token_embd.type;
    m.output = tensor(r->output.set ? r->output : r->token_embd, c.dim);
    m.output_norm = r->output_norm_f32;
    m.layers.resize(c.n_layers);
    for (uint32_t l = 0; l < c.n_layers; l++) {
        const Layer &L = r->layers[l];
        MegaLayer &M = m.layers[l];
        M.q = tensor(L.attn_q, c.dim);
        M.k = tensor(L.attn_k, c.dim);
        M.v = tensor(L.attn_v, c.dim);
        M.o = tensor(L.attn_output, qdim);
        M.gate = tensor(L.ffn_gate, c.dim);
        M.up = tensor(L.ffn_up, c.dim);
        M.down = tensor(L.ffn_down, c.ff_dim);
        M.attn_norm = L.attn_norm_f32;
        M.ffn_norm = L.ffn_norm_f32;
        M.k_cache = L.k_cache;
        M.v_cache = L.v_cache;
    }
    m.rope_cos = r->rope_cos;
    m.rope_sin = r->rope_sin;
    m.state = r->d_state;
    m.history = r->d_history;
    m.logits = r->logits;
    m.status = r->ctx->device_status;
    m.wait_cycles = r->ctx->wait_cycles;
    m.sm_count = r->ctx->prop.multiProcessorCount;
    const size_t bytes = mega_workspace_bytes(m, &r->mega_why);
    if (!bytes) return YULE_OK;
    float *ws = nullptr;
    int32_t rc = alloc_f32(r, (bytes + 3) / 4, &ws);  // zero-filled
    if (rc) return rc;
    cudaError_t e = mega_setup(m, ws, r->ctx->stream, &r->mega);
    if (e != cudaSuccess) {
        r->mega = nullptr;
        return fail_cuda(e, "persistent decode kernel set-up");
    }
    r->mega_why.clear();
    return YULE_OK;
}

int32_t ensure_graph(yule_cuda_runner *r) {
    if (r->graph_exec) return YULE_OK;
    cudaStream_t s = r->ctx->stream;
    YULE_CUDA_TRY(cudaStreamSynchronize(s));
    if (r->mega_wanted && !r->mega_tried) {
        r->mega_tried = true;
        int32_t rc = setup_mega(r);
        if (rc) return rc;
    }
    // With the persistent kernel the graph is that one launch: cooperative first, and if the capture or the
    // instantiation refuses the attribute, an ordinary launch of the same grid (one CTA per SM; its waits are bounded).
    const bool plain_first = knob("YULE_MEGA_COOP") && atoi(knob("YULE_MEGA_COOP")) == 0;  // timing aid: skip the cooperative attempt
    for (int attempt = plain_first ? 1 : 0; attempt < (r->mega ? 2 : 1); attempt++) {
        cudaGraph_t graph = nullptr;
        if (r->mega) mega_set_cooperative(r->mega, attempt == 0);
        YULE_CUDA_TRY(cudaStreamBeginCapture(s, cudaStreamCaptureModeRelaxed));
        uint64_t n = 0;
        cudaError_t e = r->mega ? mega_launch(r->mega, s, &n) : enqueue_forward_graph(r, &n);
        cudaError_t e2 = cudaStreamEndCapture(s, &graph);
        if (e == cudaSuccess && e2 == cudaSuccess) {
            e = cudaGraphInstantiate(&r->graph_exec, graph, 0);
            cudaGraphDestroy(graph);
            if (e == cudaSuccess) {
                r->graph_kernels = (uint32_t)n;
                return YULE_OK;
            }
            r->graph_exec = nullptr;
            cudaGetLastError();
            if (r->mega && attempt == 0) continue;
            return fail_cuda(e, "cudaGraphInstantiate");
        }
        if (graph) cudaGraphDestroy(graph);
        cudaGetLastError();
        if (r->mega && attempt == 0) continue;
        return fail_cuda(e != cudaSuccess ? e : e2, "graph capture of the token step");
    }
    return YULE_OK;
}

inline uint32_t graph_kernels(const yule_cuda_runner *r) { return r->graph_kernels; }
inline bool is_fused(const yule_cuda_runner *r) { return r->fused; }

int32_t ensure_pinned(yule_cuda_runner *r, size_t n_words) {
    if (r->h_pinned_cap >= n_words) return YULE_OK;
    if (r->h_pinned) cudaFreeHost(r->h_pinned);
    r->h_pinned = nullptr;
    r->h_pinned_cap = 0;
    size_t cap = n_words < 4096 ? 4096 : n_words;
    YULE_CUDA_TRY(cudaMallocHost((void **)&r->h_pinned, cap * sizeof(uint32_t)));
    r->h_pinned_cap = cap;
    return YULE_OK;
}

// ── batched prefill ─────────────────────────────────────────────────────────────────────────
// The reference feeds a prompt one token at a time through the decode path
// (yule-infer/src/gpu_runner.rs:146-160).  Here the prompt goes through the layers in chunks of up
// to 512 tokens: every linear is one tensor-core GEMM over the chunk, so the weights cross HBM once
// per chunk instead of once per token.  It fills the KV caches only; the caller runs the last prompt
// token through the ordinary token step, which produces the logits and the greedy pick.

// Tensor-parallel runs read the device status word every this many tokens and stop enqueuing once a bounded
// wait has given up (the waits themselves return at once after the first failure).
constexpr uint32_t kStatusCheckTokens = 32;
constexpr uint32_t kPrefillChunk = 512, kPrefillMinTokens = 16, kPrefillMinChunk = 256;
// Up to this many live rows a pass over the layers runs its linears on the batched matvec kernels (two to four rows
// per pass over the weights, about the time of one) instead of the GEMM, whose fixed cost per launch is several
// matvec passes.
constexpr uint32_t kRowsMatvecMax = 12;

uint32_t prefill_chunk_size(const yule_cuda_runner *r) {
    uint32_t c = knob("YULE_CUDA_PREFILL_CHUNK") ? (uint32_t)atoi(knob("YULE_CUDA_PREFILL_CHUNK")) : kPrefillChunk;
    c = c < 8 ? 8 : c;
    return c < r->cfg.max_seq_len ? c : r->cfg.max_seq_len;
}

// Single GPU, graph mode, grouped-query attention kernel available, every linear of every layer in a
// block format with a column count the GEMM takes (multiples of 256), and a context short enough
// for the attention kernel's score buffer at eight splits.
bool prefill_batched_ok(const yule_cuda_runner *r) {
    const yule_runner_config &c = r->cfg;
    if (knob("YULE_CUDA_BATCH_PREFILL") && atoi(knob("YULE_CUDA_BATCH_PREFILL")) == 0) return false;
    if (!r->fused || !r->attn_gqa) return false;
    if (r->ctx->tp_world > 1 && (!r->xchg || !r->xb_rows)) return false;  // needs the peer exchange with its row matrices
    if (is_variant(r)) return false;  // the chunked path implements the Llama op sequence only
    if (!qgemm_supported(YULE_DTYPE_Q4_K, c.dim, 8) || !qgemm_supported(YULE_DTYPE_Q4_K, c.ff_dim, 8) ||
        !qgemm_supported(YULE_DTYPE_Q4_K, c.n_heads * c.head_dim, 8))
        return false;
    for (const Layer &L : r->layers)
        for (const Tensor *t : {&L.attn_q, &L.attn_k, &L.attn_v, &L.attn_output, &L.ffn_gate, &L.ffn_up, &L.ffn_down})
            if (!is_quantized(t->type)) return false;
    const uint32_t splits = c.max_seq_len / 1024 < 1 ? 1 : (c.max_seq_len / 1024 > 8 ? 8 : c.max_seq_len / 1024);
    const size_t score_bytes = (size_t)(c.n_heads / c.n_kv_heads) * ((c.max_seq_len + splits - 1) / splits + 4) * 4;
    return score_bytes <= 96 * 1024;
}

// Row buffers of the GEMM-driven paths (chunked prefill, batched decode), allocated on first use.  Under tensor
// parallelism the matrices that are gathered (x, attention output, gate, up) live in the exchange region, which
// every peer maps; q / k / v hold this rank's heads only.
int32_t ensure_chunk_buffers(yule_cuda_runner *r) {
    const yule_runner_config &c = r->cfg;
    const uint32_t N = r->ctx->tp_world > 1 ? r->ctx->tp_world : 1;
    const uint32_t dim = c.dim, hd = c.head_dim, qdim = c.n_heads * hd, kvdim = c.n_kv_heads * hd, ff = c.ff_dim;
    int32_t rc;
    if (!r->pf_chunk) {
        uint32_t C = prefill_chunk_size(r);
        if (N > 1 && C > r->xb_rows) C = r->xb_rows;
        r->pf_splits = c.max_seq_len / 1024 < 1 ? 1 : (c.max_seq_len / 1024 > 8 ? 8 : c.max_seq_len / 1024);
        float *tok_f = nullptr, *tick_f = nullptr, *bt = nullptr;
        if (N > 1) {
            float *base = r->ctx->tp_peer_base[r->ctx->tp_rank];
            r->pf_x = base + r->xb_x;
            r->pf_att = base + r->xb_att;
            r->pf_gate = base + r->xb_gate;
            r->pf_up = base + r->xb_up;
            if ((rc = alloc_f32(r, 4, &bt))) return rc;
            r->d_btick = (uint32_t *)bt;
        } else if ((rc = alloc_f32(r, (size_t)C * dim, &r->pf_x)) || (rc = alloc_f32(r, (size_t)C * qdim, &r->pf_att)) ||
                   (rc = alloc_f32(r, (size_t)C * ff, &r->pf_gate)) || (rc = alloc_f32(r, (size_t)C * ff, &r->pf_up))) {
            return rc;
        }
        if ((rc = alloc_f32(r, (size_t)C * (qdim / N), &r->pf_q)) || (rc = alloc_f32(r, (size_t)C * (kvdim / N), &r->pf_k)) ||
            (rc = alloc_f32(r, (size_t)C * (kvdim / N), &r->pf_v)) || (rc = alloc_f32(r, C, &tok_f)) ||
            (rc = alloc_f32(r, (size_t)C * c.n_heads, &tick_f)) ||
            (rc = alloc_f32(r, (size_t)C * attn_scratch_floats(c.n_heads / N, r->pf_splits, hd) + 4, &r->pf_attn_scratch)) ||
            (rc = alloc_f32(r, (size_t)kRowsMatvecMax * dim, &r->pf_norm)))
            return rc;
        r->pf_tokens = (uint32_t *)tok_f;
        r->pf_tickets = (uint32_t *)tick_f;  // zero-filled by the allocator; the kernel leaves them at zero
        r->pf_chunk = C;
    }
    const uint32_t C = r->pf_chunk;
    const uint32_t widest = ff > qdim ? (ff > dim ? ff : dim) : (qdim > dim ? qdim : dim);
    if ((rc = ensure_gemm_scratch(r->ctx, qgemm_scratch_bytes(C, widest)))) return rc;
    return ensure_pinned(r, C);
}

// One pass of `m` rows through every layer with one GEMM per linear: the body shared by the chunked prefill
// (rows = consecutive positions of one sequence) and the batched decode step (rows = the current tokens of
// `n_live` sequences, each at its own position of its own caches).  Tensor parallelism: every GEMM computes this
// rank's output rows into its column block of the full-width matrix, which is then exchanged with the peers
// (row-matrix form of the peer-store exchange; epochs count on d_btick, flag slots 5..7).
struct RowsPass {
    uint32_t m = 0;            // rows the GEMMs run over
    uint32_t n_live = 0;       // rows that carry a token (RoPE, KV write and attention touch only these)
    const uint32_t *tokens = nullptr;
    bool batch = false;        // false: prefill at positions pos0 .. pos0 + n_live − 1 of the runner's caches
    uint32_t pos0 = 0;
};

cudaError_t enqueue_rows_pass(yule_cuda_runner *r, const RowsPass &ps, uint64_t *launches) {
    const yule_runner_config &c = r->cfg;
    yule_cuda_ctx *ctx = r->ctx;
    cudaStream_t s = ctx->stream;
    const uint32_t N = ctx->tp_world > 1 ? ctx->tp_world : 1, R = N > 1 ? ctx->tp_rank : 0;
    const uint32_t dim = c.dim, hd = c.head_dim, qdim = c.n_heads * hd, kvdim = c.n_kv_heads * hd, ff = c.ff_dim;
    const uint32_t qdim_l = qdim / N, kvdim_l = kvdim / N, ff_l = ff / N, dim_l = dim / N, vocab_l = c.vocab_size / N;
    const uint32_t m = ps.m;
    const int sms = ctx->prop.multiProcessorCount;
    const size_t cache_stride = (size_t)c.max_seq_len * kvdim_l;
    cudaError_t err = cudaSuccess;
    auto ok = [&](cudaError_t e) {
        if (err == cudaSuccess && e != cudaSuccess) err = e;
    };
    auto xprep = [&](const float *x, uint32_t cols, const float *norm_w, const float *gate) {
        QGemm g;
        g.type = YULE_DTYPE_Q4_K;
        g.x = x;
        g.gate = gate;
        g.norm_w = norm_w;
        g.eps = c.norm_eps;
        g.x_stride = cols;
        g.n_cols = cols;
        g.n_tokens = m;
        g.scratch = ctx->gemm_scratch;
        g.pdl = true;  // starts under the tail of its predecessor; reads and writes only after the dependency wait
        ok(launch_qgemm_xprep(g, s, launches));
    };
    // `rows` output rows of this rank, written at `out` with `stride` floats between the rows of the result.  Matrices
    // of one format that read the same re-laid-out rows and add no residual (Q/K/V; gate/up) wait in `gq` and go out
    // as one launch, whose row tiles run over all of them.
    QGemm gq;
    bool gq_open = false;
    bool share_mm = true;
    if (const char *k = knob("YULE_GEMM_SHARE")) share_mm = atoi(k) != 0;
    auto mm_flush = [&]() {
        if (!gq_open) return;
        ok(launch_qgemm_mm(gq, sms, s, launches));
        gq_open = false;
    };
    auto mm = [&](const Tensor &t, uint32_t rows, uint32_t cols, float *out, uint32_t stride, const float *residual) {
        if (gq_open && share_mm && !residual && gq.type == t.type && gq.n_cols == cols && gq.n_more < 2) {
            const uint32_t i = gq.n_more++;
            gq.w_more[i] = (const uint8_t *)t.buf.ptr;
            gq.out_more[i] = out;
            gq.n_rows_more[i] = rows;
            gq.out_stride_more[i] = stride;
            return;
        }
        mm_flush();
        gq = QGemm();
        gq.w = (const uint8_t *)t.buf.ptr;
        gq.type = t.type;
        gq.out = out;
        gq.residual = residual;
        gq.n_rows = rows;
        gq.n_cols = cols;
        gq.n_tokens = m;
        gq.out_stride = stride;
        gq.scratch = ctx->gemm_scratch;
        gq.status = ctx->device_status;
        gq.pdl = true;  // barrier set-up, TMEM allocation and the first weight copies overlap with the re-layout before it
        gq_open = true;
        if (residual) mm_flush();
    };
    // Few live rows: the same sequence of linears on the matvec kernels.  `prep` leaves the rows the next linears read
    // in `act`: normed rows in a buffer of their own, SwiGLU in place, anything else where it is.
    bool mv = ps.n_live <= kRowsMatvecMax;
    if (const char *k = knob("YULE_ROWS_MATVEC")) mv = mv && atoi(k) != 0;
    // The matrices that read the same rows (Q/K/V; gate/up) are collected and launched together by `flush`: as one
    // launch with the RMSNorm folded into its staging where the batched kernel allows it, else one by one behind a
    // separate RMSNorm kernel.
    const float *act = nullptr, *act_norm = nullptr;
    QmvArgs pending[3];
    uint32_t n_pending = 0;
    auto flush = [&]() {
        mm_flush();
        if (n_pending == 0) return;
        for (uint32_t i = 0; i < n_pending; i++) pending[i].norm_w = act_norm;
        if (act_norm && !kquant_batch_can_share(pending, n_pending)) {
            ok(launch_rms_norm_rows(act, act_norm, r->pf_norm, pending[0].n_cols, ps.n_live, c.norm_eps, s, launches));
            for (uint32_t i = 0; i < n_pending; i++) {
                pending[i].x = r->pf_norm;
                pending[i].norm_w = nullptr;
            }
        }
        if (kquant_batch_can_share(pending, n_pending))
            ok(launch_kquant_batch_shared(pending, n_pending, sms, s, launches));
        else
            for (uint32_t i = 0; i < n_pending; i++) ok(launch_qmv(pending[i], sms, s, launches));
        n_pending = 0;
    };
    auto prep = [&](float *x, uint32_t cols, const float *norm_w, const float *gate) {
        flush();
        if (!mv) {
            xprep(x, cols, norm_w, gate);
            return;
        }
        if (gate) ok(launch_silu_mul(gate, x, x, ps.n_live * cols, s, launches, true));  // SwiGLU in place
        act = x;
        act_norm = norm_w;
    };
    auto lin = [&](const Tensor &t, uint32_t rows, uint32_t cols, float *out, uint32_t stride, const float *residual) {
        if (!mv) {
            mm(t, rows, cols, out, stride, residual);
            return;
        }
        if (n_pending == 3) flush();
        QmvArgs a = {};
        a.w = (const uint8_t *)t.buf.ptr;
        a.x = act;
        a.out = out;
        a.n_rows = rows;
        a.n_cols = cols;
        a.type = t.type;
        a.batch = ps.n_live;
        a.x_stride = cols;
        a.out_stride = stride;
        a.residual = residual;
        a.eps = c.norm_eps;
        if (t.type == YULE_DTYPE_Q6_K && t.buf.planar && t.buf.planar_cols == cols) a.planar = t.buf.planar;
        a.status = ctx->device_status;
        a.wait_cycles = ctx->wait_cycles;
        a.pdl = true;  // set-up and the first weight copies run under the tail of the kernel before; the rows are read after the wait
        pending[n_pending++] = a;
    };
    const uint32_t epochs_per_tick = 5 * c.n_layers + 1;
    uint32_t xchg_index = 0;
    auto exchange = [&](size_t offset, uint32_t per_rank, uint32_t stride) {
        flush();
        if (N > 1) ok(tp_exchange(ctx, offset, per_rank, 5 + xchg_index % 3, r->d_btick, epochs_per_tick, xchg_index, false, launches, m, stride));
        xchg_index++;
    };
    if (N > 1) ok(launch_advance_rows(nullptr, r->d_btick, 0, s, launches));  // a new tick for this pass's exchanges
    ok(launch_embed_gather_batch((const uint8_t *)r->token_embd.buf.ptr, r->token_embd.type, dim, ps.tokens, ps.n_live, r->pf_x, s, launches));
    for (uint32_t l = 0; l < c.n_layers; l++) {
        Layer &L = r->layers[l];
        // attention block: RMSNorm folded into the re-layout, Q/K/V share it; this rank's heads only
        prep(r->pf_x, dim, L.attn_norm_f32, nullptr);
        lin(L.attn_q, qdim_l, dim, r->pf_q, qdim_l, nullptr);
        lin(L.attn_k, kvdim_l, dim, r->pf_k, kvdim_l, nullptr);
        lin(L.attn_v, kvdim_l, dim, r->pf_v, kvdim_l, nullptr);
        flush();
        AttnDecode a;
        if (ps.batch) {
            ok(launch_rope_kv_write_batch(r->pf_q, r->pf_k, r->pf_v, r->bd_k[l], r->bd_v[l], r->rope_cos, r->rope_sin, 0, ps.n_live, hd,
                                          c.n_heads / N, c.n_kv_heads / N, s, launches, r->bd_pos, cache_stride));
            a.k_cache = r->bd_k[l];
            a.v_cache = r->bd_v[l];
            a.pos_ptr = r->bd_pos;
            a.pos_per_query = true;
            a.kv_batch_stride = cache_stride;
        } else {
            ok(launch_rope_kv_write_batch(r->pf_q, r->pf_k, r->pf_v, L.k_cache, L.v_cache, r->rope_cos, r->rope_sin, ps.pos0, ps.n_live, hd,
                                          c.n_heads / N, c.n_kv_heads / N, s, launches));
            a.k_cache = L.k_cache;
            a.v_cache = L.v_cache;
            a.seq_len = ps.pos0 + 1;  // query z attends to positions [0, pos0 + z]
        }
        a.q = r->pf_q;
        a.out = r->pf_att + (size_t)R * qdim_l;
        a.scratch = r->pf_attn_scratch;
        a.tickets = r->pf_tickets;
        a.hd = hd;
        a.n_heads = c.n_heads / N;
        a.n_kv_heads = c.n_kv_heads / N;
        a.kv_stride = kvdim_l;
        a.n_splits = r->pf_splits;
        a.max_seq_len = c.max_seq_len;
        a.min_chunk = kPrefillMinChunk;
        a.gqa = true;
        a.n_tokens = ps.n_live;
        a.q_stride = qdim_l;
        a.out_stride = qdim;
        ok(launch_attn_decode(a, s, launches));
        exchange(r->xb_att, qdim_l, qdim);
        prep(r->pf_att, qdim, nullptr, nullptr);
        lin(L.attn_output, dim_l, qdim, r->pf_x + (size_t)R * dim_l, dim, r->pf_x + (size_t)R * dim_l);  // x += Wo · attention
        exchange(r->xb_x, dim_l, dim);
        // feed-forward block: RMSNorm folded in, gate/up share the re-layout, SwiGLU folded into the next one
        prep(r->pf_x, dim, L.ffn_norm_f32, nullptr);
        lin(L.ffn_gate, ff_l, dim, r->pf_gate + (size_t)R * ff_l, ff, nullptr);
        lin(L.ffn_up, ff_l, dim, r->pf_up + (size_t)R * ff_l, ff, nullptr);
        exchange(r->xb_gate, ff_l, ff);
        exchange(r->xb_up, ff_l, ff);
        prep(r->pf_up, ff, nullptr, r->pf_gate);
        lin(L.ffn_down, dim_l, ff, r->pf_x + (size_t)R * dim_l, dim, r->pf_x + (size_t)R * dim_l);  // x += Wdown · (silu(gate) · up)
        exchange(r->xb_x, dim_l, dim);
    }
    if (ps.batch) {
        const Tensor &out_w = r->output.set ? r->output : r->token_embd;
        prep(r->pf_x, dim, r->output_norm_f32, nullptr);
        lin(out_w, vocab_l, dim, r->bd_logits + (size_t)R * vocab_l, c.vocab_size, nullptr);
        exchange(r->xb_logits, vocab_l, c.vocab_size);
        flush();
        ok(launch_argmax_rows(r->bd_logits, c.vocab_size, ps.n_live, r->bd_tokens, r->bd_pos, r->bd_step, r->bd_history, c.max_seq_len + 1, s, launches));
        ok(launch_advance_rows(r->bd_pos, r->bd_step, ps.n_live, s, launches));
    }
    flush();
    return err;
}

int32_t prefill_batched(yule_cuda_runner *r, const uint32_t *tokens, uint32_t n) {
    yule_cuda_ctx *ctx = r->ctx;
    cudaStream_t s = ctx->stream;
    int32_t rc;
    if ((rc = ensure_chunk_buffers(r))) return rc;
    const uint32_t C = r->pf_chunk;
    uint64_t launches = 0;
    struct Guard {
        yule_cuda_ctx *ctx;
        uint64_t *n;
        ~Guard() { ctx->launches.fetch_add(*n); }
    } guard{ctx, &launches};
    for (uint32_t c0 = 0; c0 < n; c0 += C) {
        const uint32_t m = n - c0 < C ? n - c0 : C;
        YULE_CUDA_TRY(cudaStreamSynchronize(s));  // the staging words of the previous chunk may still be in flight
        for (uint32_t i = 0; i < m; i++) r->h_pinned[i] = tokens[c0 + i];
        YULE_CUDA_TRY(cudaMemcpyAsync(r->pf_tokens, r->h_pinned, (size_t)m * 4, cudaMemcpyHostToDevice, s));
        RowsPass ps;
        ps.m = m;
        ps.n_live = m;
        ps.tokens = r->pf_tokens;
        ps.pos0 = r->pos + c0;
        cudaError_t e = enqueue_rows_pass(r, ps, &launches);
        if (e != cudaSuccess) return fail_cuda(e, "batched prefill");
        // tensor parallelism: a peer that stopped answering is noticed per chunk
        if (r->xchg && (rc = yule_cuda_synchronize(ctx))) return rc;
    }
    r->pos += n;
    r->have_next_token = false;
    return YULE_OK;
}

// ── batched decode ──────────────────────────────────────────────────────────────────────────
// `batch` independent sequences, one new token each per step.  The reference decodes one sequence at a time
// (yule-infer/src/lib.rs:169-216 drives ModelRunner::decode_step); per sequence the arithmetic here is the
// chunked prefill's — every linear one tensor-core GEMM over the rows, so the weights cross HBM once per step
// instead of once per sequence — with row b at its own position of its own KV caches.

bool batch_decode_ok(const yule_cuda_runner *r) { return prefill_batched_ok(r); }

// Enqueues one step: tokens in bd_tokens, positions in bd_pos (device).  Leaves the logits in bd_logits, the greedy
// picks in bd_tokens / bd_history, and moves positions and step counter on.
cudaError_t enqueue_batch_step(yule_cuda_runner *r, uint64_t *launches) {
    RowsPass ps;
    ps.m = r->bd_rows;
    ps.n_live = r->bd_batch;
    ps.tokens = r->bd_tokens;
    ps.batch = true;
    return enqueue_rows_pass(r, ps, launches);
}

int32_t ensure_batch_state(yule_cuda_runner *r, uint32_t batch) {
    const yule_runner_config &c = r->cfg;
    if (!batch_decode_ok(r))
        return fail(YULE_ERR_INVALID_ARGUMENT, "batched decode needs a runner created with fused = 1 (under tensor parallelism: with "
                                               "the peer exchange), block-quantised linears with column counts in multiples of 256 "
                                               "and the Llama op sequence");
    int32_t rc = ensure_chunk_buffers(r);
    if (rc) return rc;
    if (batch == 0 || batch > r->pf_chunk) return fail(YULE_ERR_INVALID_ARGUMENT, "batch %u outside 1..%u", batch, r->pf_chunk);
    if (r->bd_batch == batch) return YULE_OK;
    if (r->bd_batch) return fail(YULE_ERR_INVALID_ARGUMENT, "this runner decodes batches of %u sequences; %u asked for", r->bd_batch, batch);
    const uint32_t tpw = r->ctx->tp_world > 1 ? r->ctx->tp_world : 1;
    const uint32_t kvdim = c.n_kv_heads * c.head_dim / tpw;  // this rank's KV heads
    const uint32_t rows = batch < 8 ? 8 : batch;  // the GEMM works on at least eight rows; the extra ones stay unused
    if (tpw > 1 && rows > r->xb_logit_rows)
        return fail(YULE_ERR_INVALID_ARGUMENT, "tensor-parallel batched decode takes at most %u sequences", r->xb_logit_rows);
    r->bd_k.assign(c.n_layers, nullptr);
    r->bd_v.assign(c.n_layers, nullptr);
    for (uint32_t l = 0; l < c.n_layers; l++)
        if ((rc = alloc_f32(r, (size_t)batch * c.max_seq_len * kvdim, &r->bd_k[l])) ||
            (rc = alloc_f32(r, (size_t)batch * c.max_seq_len * kvdim, &r->bd_v[l])))
            return rc;
    float *tok = nullptr, *pos = nullptr, *step = nullptr, *hist = nullptr;
    if (tpw > 1)
        r->bd_logits = r->ctx->tp_peer_base[r->ctx->tp_rank] + r->xb_logits;  // gathered: lives in the exchange region
    else if ((rc = alloc_f32(r, (size_t)rows * c.vocab_size, &r->bd_logits)))
        return rc;
    if ((rc = alloc_f32(r, rows, &tok)) ||
        (rc = alloc_f32(r, rows, &pos)) || (rc = alloc_f32(r, 4, &step)) ||
        (rc = alloc_f32(r, (size_t)batch * (c.max_seq_len + 1), &hist)))
        return rc;
    r->bd_tokens = (uint32_t *)tok;
    r->bd_pos = (uint32_t *)pos;
    r->bd_step = (uint32_t *)step;
    r->bd_history = (uint32_t *)hist;
    r->bd_host_pos.assign(batch, 0);
    r->bd_host_step = 0;
    r->bd_batch = batch;
    r->bd_rows = rows;
    return YULE_OK;
}

int32_t ensure_batch_graph(yule_cuda_runner *r) {
    if (r->bd_graph) return YULE_OK;
    cudaStream_t s = r->ctx->stream;
    cudaGraph_t graph = nullptr;
    YULE_CUDA_TRY(cudaStreamSynchronize(s));
    YULE_CUDA_TRY(cudaStreamBeginCapture(s, cudaStreamCaptureModeRelaxed));
    uint64_t n = 0;
    cudaError_t e = enqueue_batch_step(r, &n);
    cudaError_t e2 = cudaStreamEndCapture(s, &graph);
    if (e != cudaSuccess || e2 != cudaSuccess) {
        if (graph) cudaGraphDestroy(graph);
        cudaGetLastError();
        return fail_cuda(e != cudaSuccess ? e : e2, "graph capture of the batched decode step");
    }
    e = cudaGraphInstantiate(&r->bd_graph, graph, 0);
    cudaGraphDestroy(graph);
    if (e != cudaSuccess) return fail_cuda(e, "cudaGraphInstantiate");
    r->bd_graph_kernels = (uint32_t)n;
    return YULE_OK;
}

// One token through the model; logits stay on the device.
int32_t step(yule_cuda_runner *r, uint32_t token, bool token_from_device) {
    const yule_runner_config &c = r->cfg;
    if (r->pos >= c.max_seq_len) return fail(YULE_ERR_CONTEXT_LENGTH, "context length exceeded");
    if (!token_from_device && token >= c.vocab_size)
        return fail(YULE_ERR_INVALID_ARGUMENT, "token %u outside the vocabulary (%u)", token, c.vocab_size);
    cudaStream_t s = r->ctx->stream;
    if (!is_fused(r)) {
        uint64_t n = 0;
        cudaError_t e = enqueue_forward_by_value(r, token, r->pos, &n);
        r->ctx->launches.fetch_add(n);
        if (e != cudaSuccess) return fail_cuda(e, "token step");
    } else {
        int32_t rc = ensure_graph(r);
        if (rc) return rc;
        if (!token_from_device) {
            // h_pinned[0..1] = {token, pos}: the position is rewritten too, so a reset() or a
            // failed step cannot leave the device counter out of step with the host's.
            YULE_CUDA_TRY(cudaStreamSynchronize(s));  // staging words may still be in flight
            r->h_pinned[0] = token;
            r->h_pinned[1] = r->pos;
            YULE_CUDA_TRY(cudaMemcpyAsync(r->d_state, r->h_pinned, 8, cudaMemcpyHostToDevice, s));
        }
        YULE_CUDA_TRY(cudaGraphLaunch(r->graph_exec, s));
        r->ctx->launches.fetch_add(graph_kernels(r));
    }
    r->pos += 1;
    r->have_next_token = is_fused(r);
    return YULE_OK;
}

int32_t read_logits(yule_cuda_runner *r, float *logits_out) {
    if (!logits_out) return YULE_OK;
    cudaStream_t s = r->ctx->stream;
    const size_t bytes = (size_t)r->cfg.vocab_size * 4;
    if (!r->h_logits) YULE_CUDA_TRY(cudaMallocHost((void **)&r->h_logits, bytes));
    YULE_CUDA_TRY(cudaMemcpyAsync(r->h_logits, r->logits, bytes, cudaMemcpyDeviceToHost, s));
    YULE_CUDA_TRY(cudaStreamSynchronize(s));
    memcpy(logits_out, r->h_logits, bytes);
    return r->xchg ? yule_cuda_synchronize(r->ctx) : YULE_OK;  // reports a peer that never arrived
}

}  // namespace

extern "C" {

// Offsets (in floats) inside a rank's exchange region of the tensor-parallel runner: the four gathered
// activation vectors, then their (value, epoch) pair copies (two floats per element, 16-byte aligned), then the
// total.  Rank r's slice of a gathered vector of n elements is [r·n/world, (r+1)·n/world) of it, of a pair copy
// twice that; the layout itself does not depend on the world size.
int32_t yule_cuda_tp_exchange_layout(const yule_runner_config *cfg, uint64_t out_offsets[8]) {
    if (!cfg || !out_offsets) return fail(YULE_ERR_INVALID_ARGUMENT, "null argument");
    const uint64_t qdim = (uint64_t)cfg->n_heads * cfg->head_dim;
    out_offsets[0] = 0;                                                   // attention output, qdim
    out_offsets[1] = out_offsets[0] + qdim;                               // hidden, dim
    out_offsets[2] = out_offsets[1] + cfg->dim;                           // gate (SwiGLU output), ff_dim
    out_offsets[3] = out_offsets[2] + cfg->ff_dim;                        // logits, vocab_size
    out_offsets[4] = (out_offsets[3] + cfg->vocab_size + 3) & ~(uint64_t)3;  // pairs of hidden, 2·dim
    out_offsets[5] = out_offsets[4] + 2 * (uint64_t)cfg->dim;             // pairs of gate, 2·ff_dim
    out_offsets[6] = out_offsets[5] + 2 * (uint64_t)cfg->ff_dim;          // pairs of the attention output, 2·qdim
    out_offsets[7] = out_offsets[6] + 2 * qdim;                           // floats in all
    return YULE_OK;
}

int32_t yule_cuda_runner_create(yule_cuda_ctx *ctx, const yule_runner_config *cfg, yule_cuda_runner **out_runner) {
    if (!ctx || !cfg || !out_runner) return fail(YULE_ERR_INVALID_ARGUMENT, "null argument");
    *out_runner = nullptr;
    YULE_CUDA_TRY(cudaSetDevice(ctx->device));
    const yule_runner_config &c = *cfg;
    if (!c.dim || !c.n_layers || !c.n_heads || !c.n_kv_heads || !c.head_dim || !c.vocab_size || !c.ff_dim ||
        !c.max_seq_len)
        return fail(YULE_ERR_INVALID_ARGUMENT, "runner config has a zero field");
    if (c.n_heads % c.n_kv_heads) return fail(YULE_ERR_INVALID_ARGUMENT, "n_heads must be a multiple of n_kv_heads");
    if (c.head_dim % 2 || c.head_dim > 256) return fail(YULE_ERR_INVALID_ARGUMENT, "head_dim must be even and <= 256");
    if (c.rotary_dim % 2) return fail(YULE_ERR_INVALID_ARGUMENT, "rotary_dim must be even");
    if (c.attn_logit_softcap < 0.f || c.logit_softcap < 0.f) return fail(YULE_ERR_INVALID_ARGUMENT, "softcaps must be positive (0 = none)");
    if (c.dim % 32 || c.ff_dim % 32 || (c.n_heads * c.head_dim) % 32)
        return fail(YULE_ERR_INVALID_ARGUMENT, "dim, ff_dim and n_heads*head_dim must be multiples of 32");
    const uint32_t tpw = ctx->tp_world ? ctx->tp_world : 1;
    if (tpw > 1) {
        if (!c.fused) return fail(YULE_ERR_INVALID_ARGUMENT, "tensor parallelism needs a runner created with fused = 1");
        if (c.n_heads % tpw || c.n_kv_heads % tpw || c.dim % tpw || c.ff_dim % tpw || c.vocab_size % tpw ||
            (c.dim / tpw) % 8 || (c.ff_dim / tpw) % 8 || (c.vocab_size / tpw) % 8)
            return fail(YULE_ERR_INVALID_ARGUMENT, "model dimensions do not split evenly over %u ranks", tpw);
    }
    if (c.n_experts) {
        if (c.n_experts > 256 || c.n_experts_used == 0 || c.n_experts_used > c.n_experts)
            return fail(YULE_ERR_INVALID_ARGUMENT, "mixture of experts: %u experts, %u used per token", c.n_experts, c.n_experts_used);
        if (tpw > 1) return fail(YULE_ERR_INVALID_ARGUMENT, "tensor parallelism does not cover mixture-of-experts models");
    }
    auto *r = new yule_cuda_runner();
    r->ctx = ctx;
    r->cfg = c;
    // a mixture-of-experts model runs one kernel per dispatch: its expert choice passes through the host
    r->fused = c.fused != 0 && c.n_experts == 0;
    r->mega_wanted = c.fused == 2 && tpw <= 1 && !(knob("YULE_CUDA_MEGA") && atoi(knob("YULE_CUDA_MEGA")) == 0);
    if (const char *e = knob("YULE_CUDA_PDL")) r->pdl = atoi(e) != 0;
    r->layers.resize(c.n_layers);
    const uint32_t hd = c.head_dim, qdim = c.n_heads * hd, kvdim = c.n_kv_heads * hd;
    int32_t rc = YULE_OK;
    auto A = [&](size_t n, float **p, yule_buffer *h = nullptr) {
        if (rc == YULE_OK) rc = alloc_f32(r, n, p, h);
    };
    const bool use_xchg = tpw > 1 && !(knob("YULE_TP_NCCL") && atoi(knob("YULE_TP_NCCL")) != 0);
    if (use_xchg) {
        // gathered activations live in one region that every peer maps
        uint64_t lay[8];
        yule_cuda_tp_exchange_layout(&c, lay);
        r->x_attn_out = lay[0];
        r->x_hidden = lay[1];
        r->x_gate = lay[2];
        r->x_logits = lay[3];
        r->x_pair_hidden = lay[4];
        r->x_pair_gate = lay[5];
        r->x_pair_attn = lay[6];
        float *base = nullptr;
        // behind the vectors of the token step: the row matrices of the GEMM-driven paths (chunked prefill, batched
        // decode) — x, attention output, gate and up for a chunk of rows, and the logits of a decode batch
        const uint32_t pf_rows = prefill_chunk_size(r) < 8 ? 8 : prefill_chunk_size(r);
        const uint32_t logit_rows = 64;
        size_t at = ((size_t)lay[7] + 3) & ~(size_t)3;
        r->xb_x = at;
        at += (size_t)pf_rows * c.dim;
        r->xb_att = at;
        at += (size_t)pf_rows * qdim;
        r->xb_gate = at;
        at += (size_t)pf_rows * c.ff_dim;
        r->xb_up = at;
        at += (size_t)pf_rows * c.ff_dim;
        r->xb_logits = at;
        at += (size_t)logit_rows * c.vocab_size;
        r->xb_rows = pf_rows;
        r->xb_logit_rows = logit_rows;
        rc = tp_setup_exchange(ctx, at, &base);
        if (rc == YULE_OK) {
            r->xchg = true;
            r->attn_out = base + r->x_attn_out;
            r->hidden = base + r->x_hidden;
            r->gate = base + r->x_gate;
            r->logits = base + r->x_logits;
        }
    } else {
        A(c.dim, &r->hidden, &r->hidden_h);
    }
    A(c.dim, &r->residual);
    if (c.n_experts) {
        float *sel_f = nullptr;
        A(c.n_experts, &r->moe_logits);
        A(c.n_experts_used, &r->moe_w);
        A(c.n_experts_used, &sel_f);
        r->moe_sel = (uint32_t *)sel_f;
        if (rc == YULE_OK && cudaMallocHost((void **)&r->h_moe_sel, (size_t)c.n_experts_used * 4) != cudaSuccess) {
            cudaGetLastError();
            rc = fail(YULE_ERR_OUT_OF_MEMORY, "pinned host allocation for the expert choice failed");
        }
    }
    A(c.dim, &r->normed);
    const uint32_t kvdim_l = kvdim / tpw;  // this rank's KV heads
    A(qdim / tpw, &r->q);
    A(kvdim_l, &r->k_tmp);
    A(kvdim_l, &r->v_tmp);
    if (!use_xchg) A(qdim, &r->attn_out);
    A(c.dim, &r->attn_proj);
    if (!use_xchg) A(c.ff_dim, &r->gate);
    A(c.ff_dim, &r->up);
    A(c.dim, &r->ffn_out);
    if (!use_xchg) A(c.vocab_size, &r->logits, &r->logits_h);
    const size_t half = hd / 2;
    A((size_t)c.max_seq_len * half, &r->rope_cos);
    A((size_t)c.max_seq_len * half, &r->rope_sin);
    float *tmp = nullptr;
    r->attn_gqa = attn_gqa_supported(hd, c.n_heads, c.n_kv_heads) && !(knob("YULE_CUDA_ATTN_GQA") && atoi(knob("YULE_CUDA_ATTN_GQA")) == 0);
    r->attn_splits = r->attn_gqa ? attn_gqa_pick_splits(c.n_kv_heads / (ctx->tp_world > 1 ? ctx->tp_world : 1), c.max_seq_len,
                                                        ctx->prop.multiProcessorCount)
                                 : attn_pick_splits(c.n_heads, c.max_seq_len, ctx->prop.multiProcessorCount);
    A(attn_scratch_floats(c.n_heads, r->attn_splits, hd) + 4, &r->attn_scratch);
    A(c.n_heads, &tmp);
    r->attn_tickets = (uint32_t *)tmp;  // zero-filled by the allocator
    A(4, &tmp);
    r->d_state = (uint32_t *)tmp;
    A((size_t)c.max_seq_len + 1, &tmp);
    r->d_history = (uint32_t *)tmp;
    for (uint32_t l = 0; l < c.n_layers && rc == YULE_OK; l++) {
        A((size_t)c.max_seq_len * kvdim_l, &r->layers[l].k_cache, &r->layers[l].k_cache_h);
        A((size_t)c.max_seq_len * kvdim_l, &r->layers[l].v_cache, &r->layers[l].v_cache_h);
    }
    if (rc == YULE_OK) rc = ensure_pinned(r, 4096);
    if (rc == YULE_OK) {
        // RoPE table with the CPU runner's recipe (model_runner.rs:78-99): f32 powf / sin / cos of
        // the host libm, so rotations match it bit for bit.
        std::vector<float> hc((size_t)c.max_seq_len * half), hs((size_t)c.max_seq_len * half);
        // partial RoPE (model_runner.rs:430-434, :502): only the first rotary_dim/2 pairs of a head turn, with
        // frequencies formed over rotary_dim; the other pairs get the identity rotation (x·1 − y·0 is x exactly)
        const size_t rot = (c.rotary_dim && c.rotary_dim < hd) ? c.rotary_dim : hd;
        for (size_t p = 0; p < c.max_seq_len; p++)
            for (size_t i = 0; i < half; i++) {
                if (i < rot / 2) {
                    float freq = 1.0f / powf(c.rope_freq_base, 2.0f * (float)i / (float)rot);
                    float theta = (float)p * freq;
                    hc[p * half + i] = cosf(theta);
                    hs[p * half + i] = sinf(theta);
                } else {
                    hc[p * half + i] = 1.0f;
                    hs[p * half + i] = 0.0f;
                }
            }
        cudaError_t e = cudaMemcpyAsync(r->rope_cos, hc.data(), hc.size() * 4, cudaMemcpyHostToDevice, ctx->stream);
        if (e == cudaSuccess)
            e = cudaMemcpyAsync(r->rope_sin, hs.data(), hs.size() * 4, cudaMemcpyHostToDevice, ctx->stream);
        if (e == cudaSuccess) e = cudaStreamSynchronize(ctx->stream);
        if (e != cudaSuccess) rc = fail_cuda(e, "rope table upload");
    }
    if (rc != YULE_OK) {
        yule_cuda_runner_destroy(r);
        return rc;
    }
    r->created = true;
    *out_runner = r;
    return YULE_OK;
}

int32_t yule_cuda_runner_destroy(yule_cuda_runner *r) {
    if (!r) return YULE_OK;
    cudaSetDevice(r->ctx->device);
    cudaStreamSynchronize(r->ctx->stream);
    if (r->graph_exec) cudaGraphExecDestroy(r->graph_exec);
    if (r->bd_graph) cudaGraphExecDestroy(r->bd_graph);
    if (r->mega) mega_destroy(r->mega);
    if (r->h_logits) cudaFreeHost(r->h_logits);
    if (r->h_moe_sel) cudaFreeHost(r->h_moe_sel);
    if (r->h_pinned) cudaFreeHost(r->h_pinned);
    for (yule_buffer h : r->owned) yule_cuda_free(r->ctx, h);
    // collective: every rank destroys its runner at the same point (a runner whose creation failed half-way leaves
    // the region to the context, which frees it without a rendezvous)
    if (r->xchg && r->created) tp_release_exchange(r->ctx);
    delete r;
    return YULE_OK;
}

int32_t yule_cuda_runner_set_tensor(yule_cuda_runner *r, const char *name, yule_buffer handle, uint32_t gguf_type) {
    if (!r || !name) return fail(YULE_ERR_INVALID_ARGUMENT, "null argument");
    Tensor *t = slot_for(r, name);
    if (!t) return fail(YULE_ERR_INVALID_ARGUMENT, "tensor name not used by this runner: %s", name);
    Buffer b;
    if (!r->ctx->find(handle, &b, name)) return YULE_ERR_UNKNOWN_BUFFER;
    if (block_size(gguf_type) == 0) return fail(YULE_ERR_UNSUPPORTED_DTYPE, "GGUF type %u not supported (%s)", gguf_type, name);
    t->buf = b;
    t->handle = handle;
    t->type = gguf_type;
    t->set = true;
    r->finalized = false;
    if (r->graph_exec) {  // pointers are baked into the graph
        cudaGraphExecDestroy(r->graph_exec);
        r->graph_exec = nullptr;
    }
    if (r->mega) {
        mega_destroy(r->mega);
        r->mega = nullptr;
    }
    r->mega_tried = false;
    if (r->bd_graph) {
        cudaGraphExecDestroy(r->bd_graph);
        r->bd_graph = nullptr;
    }
    return YULE_OK;
}

int32_t yule_cuda_runner_prefill(yule_cuda_runner *r, const uint32_t *tokens, uint32_t n_tokens, float *logits_out) {
    if (!r || (n_tokens && !tokens)) return fail(YULE_ERR_INVALID_ARGUMENT, "null argument");
    YULE_CUDA_TRY(cudaSetDevice(r->ctx->device));
    int32_t rc = finalize(r);
    if (rc) return rc;
    if ((uint64_t)r->pos + n_tokens > r->cfg.max_seq_len) return fail(YULE_ERR_CONTEXT_LENGTH, "context length exceeded");
    uint32_t first = 0;
    if (n_tokens >= kPrefillMinTokens && prefill_batched_ok(r)) {
        for (uint32_t i = 0; i < n_tokens; i++)
            if (tokens[i] >= r->cfg.vocab_size)
                return fail(YULE_ERR_INVALID_ARGUMENT, "token %u outside the vocabulary (%u)", tokens[i], r->cfg.vocab_size);
        // all but the last token in chunks on the GEMM path; the last one yields the logits
        if ((rc = prefill_batched(r, tokens, n_tokens - 1))) return rc;
        first = n_tokens - 1;
    }
    for (uint32_t i = first; i < n_tokens; i++)
        if ((rc = step(r, tokens[i], false))) return rc;
    return n_tokens ? read_logits(r, logits_out) : YULE_OK;
}

int32_t yule_cuda_runner_decode_step(yule_cuda_runner *r, uint32_t token, float *logits_out) {
    if (!r) return fail(YULE_ERR_INVALID_ARGUMENT, "null runner");
    YULE_CUDA_TRY(cudaSetDevice(r->ctx->device));
    int32_t rc = finalize(r);
    if (rc) return rc;
    if ((rc = step(r, token, false))) return rc;
    return read_logits(r, logits_out);
}

int32_t yule_cuda_runner_reset(yule_cuda_runner *r) {
    if (!r) return fail(YULE_ERR_INVALID_ARGUMENT, "null runner");
    r->pos = 0;
    r->have_next_token = false;
    return YULE_OK;
}

int32_t yule_cuda_runner_step_kind(yule_cuda_runner *r, uint32_t *out_kind) {
    if (!r || !out_kind) return fail(YULE_ERR_INVALID_ARGUMENT, "null argument");
    YULE_CUDA_TRY(cudaSetDevice(r->ctx->device));
    int32_t rc = finalize(r);
    if (rc) return rc;
    if (is_fused(r) && (rc = ensure_graph(r))) return rc;
    *out_kind = !is_fused(r) ? 0u : (r->mega ? 2u : 1u);
    return YULE_OK;
}

int32_t yule_cuda_runner_selftest_bounded_wait(yule_cuda_runner *r, uint64_t budget_cycles) {
    if (!r) return fail(YULE_ERR_INVALID_ARGUMENT, "null runner");
    uint32_t kind = 0;
    int32_t rc = yule_cuda_runner_step_kind(r, &kind);
    if (rc) return rc;
    if (kind != 2) return fail(YULE_ERR_INVALID_ARGUMENT, "the self-test needs a runner whose token step is the persistent kernel");
    cudaStream_t s = r->ctx->stream;
    YULE_CUDA_TRY(cudaStreamSynchronize(s));
    // a valid token and position for the garbage step
    r->h_pinned[0] = 0;
    r->h_pinned[1] = 0;
    YULE_CUDA_TRY(cudaMemcpyAsync(r->d_state, r->h_pinned, 8, cudaMemcpyHostToDevice, s));
    uint64_t n = 0;
    cudaError_t e = mega_launch_selftest(r->mega, budget_cycles ? (long long)budget_cycles : r->ctx->wait_cycles, s, &n);
    r->ctx->launches.fetch_add(n);
    r->pos = 0;
    r->have_next_token = false;
    return e == cudaSuccess ? yule_cuda_synchronize(r->ctx) : fail_cuda(e, "bounded-wait self-test launch");
}

int32_t yule_cuda_runner_position(yule_cuda_runner *r, uint32_t *out_pos) {
    if (!r || !out_pos) return fail(YULE_ERR_INVALID_ARGUMENT, "null argument");
    *out_pos = r->pos;
    return YULE_OK;
}

int32_t yule_cuda_runner_generate_greedy(yule_cuda_runner *r, const uint32_t *prompt, uint32_t n_prompt,
                                         uint32_t n_generate, uint32_t *out_tokens) {
    if (!r || (n_prompt && !prompt) || (n_generate && !out_tokens)) return fail(YULE_ERR_INVALID_ARGUMENT, "null argument");
    YULE_CUDA_TRY(cudaSetDevice(r->ctx->device));
    if (!is_fused(r)) return fail(YULE_ERR_INVALID_ARGUMENT, "generate_greedy needs a runner created with fused = 1");
    int32_t rc = finalize(r);
    if (rc) return rc;
    if ((rc = ensure_graph(r))) return rc;
    const yule_runner_config &c = r->cfg;
    if ((uint64_t)r->pos + n_prompt + n_generate > c.max_seq_len)
        return fail(YULE_ERR_CONTEXT_LENGTH, "context length exceeded");
    if (n_prompt == 0 && n_generate && !r->have_next_token)
        return fail(YULE_ERR_INVALID_ARGUMENT, "nothing to continue from: feed a prompt first");
    cudaStream_t s = r->ctx->stream;
    if (n_prompt) {
        for (uint32_t i = 0; i < n_prompt; i++)
            if (prompt[i] >= c.vocab_size) return fail(YULE_ERR_INVALID_ARGUMENT, "token %u outside the vocabulary", prompt[i]);
        uint32_t first = 0;
        if (n_prompt >= kPrefillMinTokens && prefill_batched_ok(r)) {
            // all but the last prompt token in chunks on the GEMM path (KV caches only)
            if ((rc = prefill_batched(r, prompt, n_prompt - 1))) return rc;
            first = n_prompt - 1;
        }
        const uint32_t rest = n_prompt - first;
        if ((rc = ensure_pinned(r, 2 * (size_t)rest))) return rc;
        YULE_CUDA_TRY(cudaStreamSynchronize(s));
        for (uint32_t i = 0; i < rest; i++) {
            r->h_pinned[2 * i] = prompt[first + i];
            r->h_pinned[2 * i + 1] = r->pos + i;
        }
        for (uint32_t i = 0; i < rest; i++) {
            YULE_CUDA_TRY(cudaMemcpyAsync(r->d_state, r->h_pinned + 2 * i, 8, cudaMemcpyHostToDevice, s));
            YULE_CUDA_TRY(cudaGraphLaunch(r->graph_exec, s));
            // tensor parallelism: a peer that stopped answering is noticed here, not after the whole prompt
            if (r->xchg && (i % kStatusCheckTokens) == kStatusCheckTokens - 1 && (rc = yule_cuda_synchronize(r->ctx))) return rc;
        }
        r->ctx->launches.fetch_add((uint64_t)graph_kernels(r) * rest);
        r->pos += rest;
        r->have_next_token = true;
    }
    if (n_generate) {
        // Token g is the pick made after position first+g-1, i.e. d_history[first + g - 1]; each
        // replay consumes the previous pick from d_state[0] without touching the host.
        const uint32_t first = r->pos;
        for (uint32_t g = 0; g < n_generate; g++) {
            YULE_CUDA_TRY(cudaGraphLaunch(r->graph_exec, s));
            if (r->xchg && (g % kStatusCheckTokens) == kStatusCheckTokens - 1 && (rc = yule_cuda_synchronize(r->ctx))) return rc;
        }
        r->ctx->launches.fetch_add((uint64_t)graph_kernels(r) * n_generate);
        r->pos += n_generate;
        YULE_CUDA_TRY(cudaMemcpyAsync(out_tokens, r->d_history + first - 1, (size_t)n_generate * 4,
                                      cudaMemcpyDeviceToHost, s));
    }
    YULE_CUDA_TRY(cudaStreamSynchronize(s));
    return r->xchg ? yule_cuda_synchronize(r->ctx) : YULE_OK;  // reports a peer that never arrived
}

float yule_cuda_sampling_random_value(uint64_t seed, uint32_t index) {
    // SplitMix64 of (seed, index); the top 24 bits over 2^24, the mapping of the reference's csprng_f32
    // (yule-infer/src/sampler.rs:212-220)
    uint64_t z = seed + 0x9E3779B97F4A7C15ull * ((uint64_t)index + 1);
    z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
    z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
    z ^= z >> 31;
    return (float)(uint32_t)(z >> 40) / 16777216.0f;
}

int32_t yule_cuda_runner_generate_sampled(yule_cuda_runner *r, const uint32_t *prompt, uint32_t n_prompt, uint32_t n_generate,
                                          const yule_sampling_params *params, uint64_t seed, uint32_t *out_tokens) {
    if (!r || !prompt || !params || (n_generate && !out_tokens)) return fail(YULE_ERR_INVALID_ARGUMENT, "null argument");
    if (n_prompt == 0) return fail(YULE_ERR_INVALID_ARGUMENT, "sampled generation needs a prompt");
    YULE_CUDA_TRY(cudaSetDevice(r->ctx->device));
    if (!is_fused(r)) return fail(YULE_ERR_INVALID_ARGUMENT, "generate_sampled needs a runner created with fused = 1");
    if (r->pos != 0) return fail(YULE_ERR_INVALID_ARGUMENT, "generate_sampled starts a sequence: reset the runner first");
    int32_t rc = finalize(r);
    if (rc) return rc;
    if ((rc = ensure_graph(r))) return rc;
    const yule_runner_config &c = r->cfg;
    if ((uint64_t)n_prompt + n_generate > c.max_seq_len) return fail(YULE_ERR_CONTEXT_LENGTH, "context length exceeded");
    if ((rc = ensure_sampler_scratch(r->ctx, 2 * (size_t)c.vocab_size + 4))) return rc;
    if (!r->d_seq) {
        float *p = nullptr;
        if ((rc = alloc_f32(r, (size_t)c.max_seq_len + 1, &p))) return rc;
        r->d_seq = (uint32_t *)p;
    }
    cudaStream_t s = r->ctx->stream;
    // the prompt: KV caches and the logits after its last token, exactly as generate_greedy feeds it
    uint32_t dummy = 0;
    if ((rc = yule_cuda_runner_generate_greedy(r, prompt, n_prompt, 0, &dummy))) return rc;
    YULE_CUDA_TRY(cudaMemcpyAsync(r->d_seq, prompt, (size_t)n_prompt * 4, cudaMemcpyHostToDevice, s));
    uint64_t launches = 0;
    cudaError_t e = cudaSuccess;
    for (uint32_t g = 0; g < n_generate && e == cudaSuccess; g++) {
        SampleArgs a;
        a.logits = r->logits;
        a.n = c.vocab_size;
        a.temperature = params->temperature;
        a.top_p = params->top_p;
        a.top_k = params->top_k;
        a.min_p = params->min_p;
        a.repetition_penalty = params->repetition_penalty;
        a.previous = r->d_seq;
        a.n_previous = n_prompt + g;
        a.r = yule_cuda_sampling_random_value(seed, g);
        a.scratch = r->ctx->sampler_scratch;
        a.out_token = reinterpret_cast<uint32_t *>(r->ctx->sampler_scratch + 2 * (size_t)c.vocab_size);
        a.append_to = r->d_seq;
        a.feed_state = r->d_state;  // the token step reads its input token here
        e = launch_sample(a, s, &launches);
        if (e == cudaSuccess) e = cudaGraphLaunch(r->graph_exec, s);
    }
    r->ctx->launches.fetch_add(launches + (uint64_t)graph_kernels(r) * n_generate);
    if (e != cudaSuccess) return fail_cuda(e, "sampled generation");
    r->pos += n_generate;
    if (n_generate)
        YULE_CUDA_TRY(cudaMemcpyAsync(out_tokens, r->d_seq + n_prompt, (size_t)n_generate * 4, cudaMemcpyDeviceToHost, s));
    YULE_CUDA_TRY(cudaStreamSynchronize(s));
    return r->xchg ? yule_cuda_synchronize(r->ctx) : YULE_OK;
}

int32_t yule_cuda_runner_reset_batch(yule_cuda_runner *r) {
    if (!r) return fail(YULE_ERR_INVALID_ARGUMENT, "null runner");
    for (auto &p : r->bd_host_pos) p = 0;
    r->bd_host_step = 0;
    return YULE_OK;
}

int32_t yule_cuda_runner_decode_batch(yule_cuda_runner *r, const uint32_t *tokens, uint32_t batch, float *logits_out) {
    if (!r || !tokens) return fail(YULE_ERR_INVALID_ARGUMENT, "null argument");
    YULE_CUDA_TRY(cudaSetDevice(r->ctx->device));
    int32_t rc = finalize(r);
    if (rc) return rc;
    if ((rc = ensure_batch_state(r, batch))) return rc;
    const yule_runner_config &c = r->cfg;
    for (uint32_t b = 0; b < batch; b++) {
        if (tokens[b] >= c.vocab_size) return fail(YULE_ERR_INVALID_ARGUMENT, "token %u outside the vocabulary (%u)", tokens[b], c.vocab_size);
        if (r->bd_host_pos[b] >= c.max_seq_len) return fail(YULE_ERR_CONTEXT_LENGTH, "context length exceeded");
    }
    if ((rc = ensure_batch_graph(r))) return rc;
    cudaStream_t s = r->ctx->stream;
    if ((rc = ensure_pinned(r, 2 * (size_t)batch + 1))) return rc;
    YULE_CUDA_TRY(cudaStreamSynchronize(s));  // staging words may still be in flight
    // tokens, positions and the step are rewritten from the host's copy, so a reset or a failed step cannot
    // leave the device counters out of step with it
    for (uint32_t b = 0; b < batch; b++) {
        r->h_pinned[b] = tokens[b];
        r->h_pinned[batch + b] = r->bd_host_pos[b];
    }
    r->h_pinned[2 * batch] = r->bd_host_step;
    YULE_CUDA_TRY(cudaMemcpyAsync(r->bd_tokens, r->h_pinned, (size_t)batch * 4, cudaMemcpyHostToDevice, s));
    YULE_CUDA_TRY(cudaMemcpyAsync(r->bd_pos, r->h_pinned + batch, (size_t)batch * 4, cudaMemcpyHostToDevice, s));
    YULE_CUDA_TRY(cudaMemcpyAsync(r->bd_step, r->h_pinned + 2 * batch, 4, cudaMemcpyHostToDevice, s));
    YULE_CUDA_TRY(cudaGraphLaunch(r->bd_graph, s));
    r->ctx->launches.fetch_add(r->bd_graph_kernels);
    for (auto &p : r->bd_host_pos) p += 1;
    r->bd_host_step += 1;
    if (logits_out) YULE_CUDA_TRY(cudaMemcpyAsync(logits_out, r->bd_logits, (size_t)batch * c.vocab_size * 4, cudaMemcpyDeviceToHost, s));
    YULE_CUDA_TRY(cudaStreamSynchronize(s));
    return yule_cuda_synchronize(r->ctx);
}

int32_t yule_cuda_runner_generate_greedy_batch(yule_cuda_runner *r, const uint32_t *prompts, uint32_t batch, uint32_t n_prompt,
                                               uint32_t n_generate, uint32_t *out_tokens) {
    if (!r || !prompts || (n_generate && !out_tokens)) return fail(YULE_ERR_INVALID_ARGUMENT, "null argument");
    if (n_prompt == 0) return fail(YULE_ERR_INVALID_ARGUMENT, "every sequence needs at least one prompt token");
    YULE_CUDA_TRY(cudaSetDevice(r->ctx->device));
    int32_t rc = finalize(r);
    if (rc) return rc;
    if ((rc = ensure_batch_state(r, batch))) return rc;
    const yule_runner_config &c = r->cfg;
    if ((uint64_t)n_prompt + n_generate > c.max_seq_len) return fail(YULE_ERR_CONTEXT_LENGTH, "context length exceeded");
    for (size_t i = 0; i < (size_t)batch * n_prompt; i++)
        if (prompts[i] >= c.vocab_size) return fail(YULE_ERR_INVALID_ARGUMENT, "token %u outside the vocabulary", prompts[i]);
    if ((rc = ensure_batch_graph(r))) return rc;
    cudaStream_t s = r->ctx->stream;
    // prompts to the device, position-major, so that step i takes its tokens with one small device copy
    const size_t n_words = (size_t)batch * n_prompt;
    if (r->bd_prompts_cap < n_words) {
        float *pw = nullptr;
        if ((rc = alloc_f32(r, n_words, &pw))) return rc;
        r->bd_prompts = (uint32_t *)pw;
        r->bd_prompts_cap = n_words;
    }
    if ((rc = ensure_pinned(r, n_words + batch + 1))) return rc;
    YULE_CUDA_TRY(cudaStreamSynchronize(s));
    for (uint32_t i = 0; i < n_prompt; i++)
        for (uint32_t b = 0; b < batch; b++) r->h_pinned[(size_t)i * batch + b] = prompts[(size_t)b * n_prompt + i];
    for (uint32_t b = 0; b <= batch; b++) r->h_pinned[n_words + b] = 0;  // positions and step start at zero
    YULE_CUDA_TRY(cudaMemcpyAsync(r->bd_prompts, r->h_pinned, n_words * 4, cudaMemcpyHostToDevice, s));
    YULE_CUDA_TRY(cudaMemcpyAsync(r->bd_pos, r->h_pinned + n_words, (size_t)batch * 4, cudaMemcpyHostToDevice, s));
    YULE_CUDA_TRY(cudaMemcpyAsync(r->bd_step, r->h_pinned + n_words + batch, 4, cudaMemcpyHostToDevice, s));
    for (uint32_t i = 0; i < n_prompt + n_generate; i++) {
        // prompt steps take their tokens from the prompt; afterwards each step consumes the previous step's picks
        if (i < n_prompt)
            YULE_CUDA_TRY(cudaMemcpyAsync(r->bd_tokens, r->bd_prompts + (size_t)i * batch, (size_t)batch * 4, cudaMemcpyDeviceToDevice, s));
        YULE_CUDA_TRY(cudaGraphLaunch(r->bd_graph, s));
    }
    r->ctx->launches.fetch_add((uint64_t)r->bd_graph_kernels * (n_prompt + n_generate));
    // token g of sequence b is the pick made after position n_prompt − 1 + g
    const size_t hist_stride = (size_t)c.max_seq_len + 1;
    for (uint32_t b = 0; b < batch && n_generate; b++)
        YULE_CUDA_TRY(cudaMemcpyAsync(out_tokens + (size_t)b * n_generate, r->bd_history + b * hist_stride + n_prompt - 1,
                                      (size_t)n_generate * 4, cudaMemcpyDeviceToHost, s));
    YULE_CUDA_TRY(cudaStreamSynchronize(s));
    for (auto &p : r->bd_host_pos) p = n_prompt + n_generate;
    r->bd_host_step = n_prompt + n_generate;
    return yule_cuda_synchronize(r->ctx);
}

int32_t yule_cuda_runner_buffer(yule_cuda_runner *r, uint32_t which, uint32_t layer, yule_buffer *out_handle) {
    if (!r || !out_handle) return fail(YULE_ERR_INVALID_ARGUMENT, "null argument");
    switch (which) {
        case 0:
        case 3:
            if (r->xchg) return fail(YULE_ERR_INVALID_ARGUMENT, "hidden/logits live in the peer exchange region, not in a buffer");
            *out_handle = which == 0 ? r->hidden_h : r->logits_h;
            return YULE_OK;
        case 1:
        case 2:
            if (layer >= r->cfg.n_layers) return fail(YULE_ERR_INVALID_ARGUMENT, "layer %u out of range", layer);
            *out_handle = which == 1 ? r->layers[layer].k_cache_h : r->layers[layer].v_cache_h;
            return YULE_OK;
        default: return fail(YULE_ERR_INVALID_ARGUMENT, "unknown buffer selector %u", which);
    }
}

}  // extern "C"
