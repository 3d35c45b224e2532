// api.cu — context, buffer table and the trait-level entry points of libyule_cuda.so.
//
// Mirrors CudaBackend (yule-gpu/src/cuda/mod.rs:14-329) and CudaMemoryManager
// (yule-gpu/src/cuda/memory.rs:10-154): opaque u64 handles, zero-filled allocations, byte-typed
// copies, every op enqueued on one stream.  Unlike the reference there is no runtime nvcc and no
// PTX cache (cuda/kernels.rs:145-186): the sm_100a kernels are compiled into this library.

#include <cmath>
#include <cstring>

#include <cstdlib>

#include "internal.h"

namespace yule {

static thread_local char g_err[512] = "";

const char *knob(const char *name) {
    static const bool debug = [] {
        const char *d = getenv("YULE_CUDA_DEBUG");
        return d && atoi(d) != 0;
    }();
    return debug ? getenv(name) : nullptr;
}

int32_t fail(int32_t code, const char *fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_err, sizeof(g_err), fmt, ap);
    va_end(ap);
    return code;
}

int32_t fail_cuda(cudaError_t e, const char *what) {
    int32_t code = (e == cudaErrorMemoryAllocation) ? YULE_ERR_OUT_OF_MEMORY : YULE_ERR_CUDA;
    return fail(code, "cuda: %s failed: %s (%s)", what, cudaGetErrorName(e), cudaGetErrorString(e));
}

// Grows the context's GEMM scratch.  Not while a graph is being captured: allocation is not a
// stream operation, so the caller must have run one call of this size before capturing.
int32_t ensure_gemm_scratch(yule_cuda_ctx *ctx, size_t bytes) {
    std::lock_guard<std::mutex> lock(ctx->mu);
    if (ctx->gemm_scratch_bytes >= bytes) return YULE_OK;
    if (ctx->capturing)
        return fail(YULE_ERR_INVALID_ARGUMENT, "the GEMM scratch (%zu bytes) cannot grow during graph capture", bytes);
    YULE_CUDA_TRY(cudaStreamSynchronize(ctx->stream));
    if (ctx->gemm_scratch) ctx->retired_scratch.push_back(ctx->gemm_scratch);  // graphs captured earlier may still use it
    ctx->gemm_scratch = nullptr;
    ctx->gemm_scratch_bytes = 0;
    cudaError_t e = cudaMalloc(&ctx->gemm_scratch, bytes);
    if (e != cudaSuccess) {
        cudaGetLastError();
        return fail(YULE_ERR_OUT_OF_MEMORY, "cuda allocation of %zu bytes of GEMM scratch failed", bytes);
    }
    // the scratch opens with the split-column tickets of the GEMM, which the kernels expect (and leave) at zero
    e = cudaMemset(ctx->gemm_scratch, 0, bytes < kGemmTicketBytes ? bytes : kGemmTicketBytes);
    if (e != cudaSuccess) return fail_cuda(e, "cudaMemset of the GEMM tickets");
    ctx->gemm_scratch_bytes = bytes;
    return YULE_OK;
}

int32_t ensure_sampler_scratch(yule_cuda_ctx *ctx, size_t n_floats) {
    if (ctx->sampler_scratch_floats >= n_floats) return YULE_OK;
    if (ctx->capturing) return fail(YULE_ERR_INVALID_ARGUMENT, "the sampler scratch cannot grow during graph capture");
    YULE_CUDA_TRY(cudaStreamSynchronize(ctx->stream));
    if (ctx->sampler_scratch) ctx->retired_scratch.push_back(ctx->sampler_scratch);
    ctx->sampler_scratch = nullptr;
    ctx->sampler_scratch_floats = 0;
    if (cudaMalloc((void **)&ctx->sampler_scratch, n_floats * sizeof(float)) != cudaSuccess) {
        cudaGetLastError();
        return fail(YULE_ERR_OUT_OF_MEMORY, "cuda allocation of %zu bytes of sampler scratch failed", n_floats * sizeof(float));
    }
    ctx->sampler_scratch_floats = n_floats;
    return YULE_OK;
}

}  // namespace yule

using namespace yule;

bool yule_cuda_ctx::find(yule_buffer h, Buffer *out, const char *what) {
    std::lock_guard<std::mutex> lock(mu);
    auto it = buffers.find(h);
    if (it == buffers.end()) {
        fail(YULE_ERR_UNKNOWN_BUFFER, "unknown buffer %llu (%s)", (unsigned long long)h, what);
        return false;
    }
    *out = it->second;
    return true;
}

// Also ends the chain of programmatic dependent launches: only qmv_common re-arms it, after a matvec.
#define CTX_GUARD(ctx)                                                        \
    if (!(ctx)) return fail(YULE_ERR_INVALID_ARGUMENT, "null context");       \
    const bool _pdl_chain = (ctx)->pdl_chain;                                 \
    (void)_pdl_chain;                                                         \
    (ctx)->pdl_chain = false;                                                 \
    const int _chain_n = (ctx)->chain_n;                                      \
    (void)_chain_n;                                                           \
    (ctx)->chain_n = 0;                                                       \
    YULE_CUDA_TRY(cudaSetDevice((ctx)->device))

#define FIND(ctx, handle, var)  \
    Buffer var;                 \
    if (!(ctx)->find(handle, &var, #handle)) return YULE_ERR_UNKNOWN_BUFFER

#define NEED_BYTES(buf, bytes, what)                                                              \
    if ((size_t)(bytes) > (buf).size)                                                             \
    return fail(YULE_ERR_OUT_OF_BOUNDS, "%s needs %zu bytes but buffer holds %zu", what,          \
                (size_t)(bytes), (buf).size)

#define LAUNCHED(ctx, call)                                   \
    do {                                                      \
        uint64_t _n = 0;                                      \
        cudaError_t _e = (call);                              \
        (ctx)->launches.fetch_add(_n);                        \
        if (_e != cudaSuccess) return fail_cuda(_e, #call);   \
    } while (0)

extern "C" {

const char *yule_cuda_last_error(void) { return g_err; }

int32_t yule_cuda_is_available(void) {
    int n = 0;
    if (cudaGetDeviceCount(&n) != cudaSuccess) {
        cudaGetLastError();
        return 0;
    }
    return n > 0 ? 1 : 0;
}

int32_t yule_cuda_create(int32_t ordinal, yule_cuda_ctx **out_ctx) {
    if (!out_ctx) return fail(YULE_ERR_INVALID_ARGUMENT, "null out_ctx");
    *out_ctx = nullptr;
    int n = 0;
    cudaError_t e = cudaGetDeviceCount(&n);
    if (e != cudaSuccess || n == 0) {
        cudaGetLastError();
        return fail(YULE_ERR_CUDA, "no CUDA device available (this backend has no CPU fallback)");
    }
    if (ordinal < 0 || ordinal >= n)
        return fail(YULE_ERR_INVALID_ARGUMENT, "device ordinal %d out of range (have %d)", ordinal, n);
    YULE_CUDA_TRY(cudaSetDevice(ordinal));
    auto *ctx = new yule_cuda_ctx();
    ctx->device = ordinal;
    e = cudaGetDeviceProperties(&ctx->prop, ordinal);
    if (e == cudaSuccess) e = cudaStreamCreateWithFlags(&ctx->stream, cudaStreamNonBlocking);
    if (e == cudaSuccess) e = cudaMalloc(&ctx->device_status, sizeof(int));
    if (e == cudaSuccess) e = cudaMemset(ctx->device_status, 0, sizeof(int));
    if (e != cudaSuccess) {
        delete ctx;
        return fail_cuda(e, "context setup");
    }
    if (ctx->prop.major < 10) {
        int major = ctx->prop.major, minor = ctx->prop.minor;
        cudaStreamDestroy(ctx->stream);
        cudaFree(ctx->device_status);
        delete ctx;
        return fail(YULE_ERR_CUDA, "device is sm_%d%d; this library carries sm_100a kernels only", major,
                    minor);
    }
    *out_ctx = ctx;
    return YULE_OK;
}

int32_t yule_cuda_destroy(yule_cuda_ctx *ctx) {
    if (!ctx) return YULE_OK;
    cudaSetDevice(ctx->device);
    cudaStreamSynchronize(ctx->stream);
    tp_destroy(ctx);
    for (auto &kv : ctx->buffers) {
        cudaFree(kv.second.ptr);
        if (kv.second.planar) cudaFree(kv.second.planar);
    }
    for (auto ev : ctx->events) cudaEventDestroy(ev);
    for (auto &g : ctx->graphs)
        if (g.exec) cudaGraphExecDestroy(g.exec);
    if (ctx->flush_buf) cudaFree(ctx->flush_buf);
    if (ctx->attn_scratch) cudaFree(ctx->attn_scratch);
    if (ctx->attn_tickets) cudaFree(ctx->attn_tickets);
    if (ctx->device_status) cudaFree(ctx->device_status);
    if (ctx->gemm_scratch) cudaFree(ctx->gemm_scratch);
    for (void *p : ctx->retired_scratch) cudaFree(p);
    if (ctx->sampler_scratch) cudaFree(ctx->sampler_scratch);
    cudaStreamDestroy(ctx->stream);
    delete ctx;
    return YULE_OK;
}

int32_t yule_cuda_device_info(yule_cuda_ctx *ctx, char *name_buf, size_t name_cap, uint64_t *memory_bytes,
                              uint32_t *compute_units) {
    CTX_GUARD(ctx);
    if (name_buf && name_cap) {
        strncpy(name_buf, ctx->prop.name, name_cap - 1);
        name_buf[name_cap - 1] = 0;
    }
    if (memory_bytes) *memory_bytes = (uint64_t)ctx->prop.totalGlobalMem;
    if (compute_units) *compute_units = (uint32_t)ctx->prop.multiProcessorCount;
    return YULE_OK;
}

int32_t yule_cuda_allocate(yule_cuda_ctx *ctx, size_t size_bytes, yule_buffer *out_handle) {
    CTX_GUARD(ctx);
    if (!out_handle) return fail(YULE_ERR_INVALID_ARGUMENT, "null out_handle");
    Buffer b;
    b.size = size_bytes;
    // Rounded up so that a 16-byte vector load starting inside the buffer never leaves it.
    b.capacity = ((size_bytes + 255) / 256) * 256 + 256;
    cudaError_t e = cudaMalloc(&b.ptr, b.capacity);
    if (e != cudaSuccess) {
        cudaGetLastError();
        return fail(YULE_ERR_OUT_OF_MEMORY, "cuda allocation of %zu bytes failed: %s", size_bytes,
                    cudaGetErrorString(e));
    }
    YULE_CUDA_TRY(cudaMemsetAsync(b.ptr, 0, b.capacity, ctx->stream));
    std::lock_guard<std::mutex> lock(ctx->mu);
    uint64_t h = ctx->next_handle++;
    ctx->buffers[h] = b;
    *out_handle = h;
    return YULE_OK;
}

int32_t yule_cuda_free(yule_cuda_ctx *ctx, yule_buffer handle) {
    CTX_GUARD(ctx);
    Buffer b;
    {
        std::lock_guard<std::mutex> lock(ctx->mu);
        auto it = ctx->buffers.find(handle);
        if (it == ctx->buffers.end())
            return fail(YULE_ERR_UNKNOWN_BUFFER, "unknown buffer %llu (free)", (unsigned long long)handle);
        b = it->second;
        ctx->buffers.erase(it);
    }
    // Work already enqueued may still read the buffer.
    YULE_CUDA_TRY(cudaStreamSynchronize(ctx->stream));
    YULE_CUDA_TRY(cudaFree(b.ptr));
    if (b.planar) YULE_CUDA_TRY(cudaFree(b.planar));
    return YULE_OK;
}

// A write to a buffer invalidates the planar copy made from its old contents.
static int32_t drop_planar(yule_cuda_ctx *ctx, yule_buffer h) {
    uint8_t *planar = nullptr;
    {
        std::lock_guard<std::mutex> lock(ctx->mu);
        auto it = ctx->buffers.find(h);
        if (it == ctx->buffers.end() || !it->second.planar) return YULE_OK;
        planar = it->second.planar;
        it->second.planar = nullptr;
        it->second.planar_blocks = 0;
        it->second.planar_cols = 0;
    }
    YULE_CUDA_TRY(cudaStreamSynchronize(ctx->stream));
    YULE_CUDA_TRY(cudaFree(planar));
    return YULE_OK;
}

static bool is_pinned_host(const void *p) {
    cudaPointerAttributes attr;
    if (cudaPointerGetAttributes(&attr, p) != cudaSuccess) {
        cudaGetLastError();
        return false;
    }
    return attr.type == cudaMemoryTypeHost;
}

int32_t yule_cuda_copy_to_device(yule_cuda_ctx *ctx, const void *data, size_t len, yule_buffer dst) {
    CTX_GUARD(ctx);
    FIND(ctx, dst, d);
    if (len && !data) return fail(YULE_ERR_INVALID_ARGUMENT, "null data");
    size_t n = len < d.size ? len : d.size;
    if (n == 0) return YULE_OK;
    if (d.planar) {
        int32_t rc = drop_planar(ctx, dst);
        if (rc) return rc;
    }
    YULE_CUDA_TRY(cudaMemcpyAsync(d.ptr, data, n, cudaMemcpyHostToDevice, ctx->stream));
    // A pageable source has been staged when the call returns; a pinned one has not, and the
    // caller's slice is only borrowed for the duration of this call.
    if (is_pinned_host(data)) YULE_CUDA_TRY(cudaStreamSynchronize(ctx->stream));
    return YULE_OK;
}

int32_t yule_cuda_copy_from_device(yule_cuda_ctx *ctx, yule_buffer src, void *data, size_t len) {
    CTX_GUARD(ctx);
    FIND(ctx, src, s);
    if (len && !data) return fail(YULE_ERR_INVALID_ARGUMENT, "null data");
    size_t n = len < s.size ? len : s.size;
    if (n) YULE_CUDA_TRY(cudaMemcpyAsync(data, s.ptr, n, cudaMemcpyDeviceToHost, ctx->stream));
    YULE_CUDA_TRY(cudaStreamSynchronize(ctx->stream));
    return YULE_OK;
}

int32_t yule_cuda_copy_buffer_offset(yule_cuda_ctx *ctx, yule_buffer src, yule_buffer dst, size_t src_offset,
                                     size_t dst_offset, size_t size) {
    CTX_GUARD(ctx);
    FIND(ctx, src, s);
    FIND(ctx, dst, d);
    if (src_offset > s.size || size > s.size - src_offset)
        return fail(YULE_ERR_OUT_OF_BOUNDS, "copy reads [%zu, %zu) of a %zu-byte buffer", src_offset,
                    src_offset + size, s.size);
    if (dst_offset > d.size || size > d.size - dst_offset)
        return fail(YULE_ERR_OUT_OF_BOUNDS, "copy writes [%zu, %zu) of a %zu-byte buffer", dst_offset,
                    dst_offset + size, d.size);
    if (size == 0) return YULE_OK;
    if (d.planar) {
        int32_t rc = drop_planar(ctx, dst);
        if (rc) return rc;
    }
    YULE_CUDA_TRY(cudaMemcpyAsync((char *)d.ptr + dst_offset, (const char *)s.ptr + src_offset, size,
                                  cudaMemcpyDeviceToDevice, ctx->stream));
    return YULE_OK;
}

int32_t yule_cuda_copy_buffer(yule_cuda_ctx *ctx, yule_buffer src, yule_buffer dst, size_t size) {
    return yule_cuda_copy_buffer_offset(ctx, src, dst, 0, 0, size);
}

int32_t yule_cuda_synchronize(yule_cuda_ctx *ctx) {
    CTX_GUARD(ctx);
    YULE_CUDA_TRY(cudaStreamSynchronize(ctx->stream));
    int status = 0;
    YULE_CUDA_TRY(cudaMemcpy(&status, ctx->device_status, sizeof(int), cudaMemcpyDeviceToHost));
    if (status != 0) {
        cudaMemset(ctx->device_status, 0, sizeof(int));
        // a GEMM that gave up may have left tickets of its column split behind: the next launch expects zeros
        if (ctx->gemm_scratch) cudaMemset(ctx->gemm_scratch, 0, ctx->gemm_scratch_bytes < kGemmTicketBytes ? ctx->gemm_scratch_bytes : kGemmTicketBytes);
        return fail(YULE_ERR_DEVICE_STATUS, "a device-side bounded wait gave up (status word %d)", status);
    }
    return YULE_OK;
}

int32_t yule_cuda_set_wait_budget(yule_cuda_ctx *ctx, uint64_t cycles) {
    CTX_GUARD(ctx);
    ctx->wait_cycles = cycles ? (long long)(cycles > (1ull << 62) ? (1ull << 62) : cycles) : kDefaultWaitCycles;
    return YULE_OK;
}

// ── compute ────────────────────────────────────────────────────────────────────────────────

int32_t yule_cuda_matmul(yule_cuda_ctx *ctx, yule_buffer a, yule_buffer b, yule_buffer out, uint32_t m,
                         uint32_t n, uint32_t k) {
    (void)n;
    CTX_GUARD(ctx);
    FIND(ctx, a, A);
    FIND(ctx, b, B);
    FIND(ctx, out, O);
    NEED_BYTES(A, (size_t)m * k * 4, "matmul a");
    NEED_BYTES(B, (size_t)k * 4, "matmul b");
    NEED_BYTES(O, (size_t)m * 4, "matmul out");
    if (m == 0) return YULE_OK;
    LAUNCHED(ctx, launch_matvec_f32((const float *)A.ptr, (const float *)B.ptr, (float *)O.ptr, m, k,
                                    ctx->stream, &_n));
    return YULE_OK;
}

int32_t yule_cuda_softmax(yule_cuda_ctx *ctx, yule_buffer input, yule_buffer output, uint32_t size) {
    CTX_GUARD(ctx);
    FIND(ctx, input, I);
    FIND(ctx, output, O);
    NEED_BYTES(I, (size_t)size * 4, "softmax input");
    NEED_BYTES(O, (size_t)size * 4, "softmax output");
    if (size == 0) return YULE_OK;
    LAUNCHED(ctx, launch_softmax((const float *)I.ptr, (float *)O.ptr, size, ctx->stream, &_n));
    return YULE_OK;
}

int32_t yule_cuda_rms_norm(yule_cuda_ctx *ctx, yule_buffer input, yule_buffer weight, yule_buffer output,
                           uint32_t size, float eps) {
    CTX_GUARD(ctx);
    FIND(ctx, input, I);
    FIND(ctx, weight, W);
    FIND(ctx, output, O);
    NEED_BYTES(I, (size_t)size * 4, "rms_norm input");
    NEED_BYTES(W, (size_t)size * 4, "rms_norm weight");
    NEED_BYTES(O, (size_t)size * 4, "rms_norm output");
    if (size == 0) return YULE_OK;
    LAUNCHED(ctx, launch_rms_norm((const float *)I.ptr, (const float *)W.ptr, (float *)O.ptr, size, eps,
                                  ctx->stream, &_n));
    return YULE_OK;
}

int32_t yule_cuda_rope(yule_cuda_ctx *ctx, yule_buffer q, yule_buffer k, uint32_t pos, uint32_t head_dim,
                       float freq_base, uint32_t n_heads_q, uint32_t n_heads_k) {
    CTX_GUARD(ctx);
    FIND(ctx, q, Q);
    FIND(ctx, k, K);
    if (head_dim == 0 || head_dim % 2 || head_dim > 256)
        return fail(YULE_ERR_INVALID_ARGUMENT, "rope head_dim %u must be even and at most 256", head_dim);
    NEED_BYTES(Q, (size_t)n_heads_q * head_dim * 4, "rope q");
    NEED_BYTES(K, (size_t)n_heads_k * head_dim * 4, "rope k");
    // Angles are evaluated on the host in f32 with the platform libm — the recipe of the CPU
    // runner's RopeTable (yule-infer/src/model_runner.rs:78-99) — so the rotation matches it bit
    // for bit; device powf/sinf/cosf differ from libm in the last place.
    RopeAngles ang;
    uint32_t half = head_dim / 2;
    for (uint32_t i = 0; i < half; i++) {
        float freq = 1.0f / powf(freq_base, 2.0f * (float)i / (float)head_dim);
        float theta = (float)pos * freq;
        ang.cos[i] = cosf(theta);
        ang.sin[i] = sinf(theta);
    }
    LAUNCHED(ctx, launch_rope_angles((float *)Q.ptr, (float *)K.ptr, head_dim, n_heads_q, n_heads_k, ang,
                                     ctx->stream, &_n));
    return YULE_OK;
}

int32_t yule_cuda_silu(yule_cuda_ctx *ctx, yule_buffer input, yule_buffer output, uint32_t size) {
    CTX_GUARD(ctx);
    FIND(ctx, input, I);
    FIND(ctx, output, O);
    NEED_BYTES(I, (size_t)size * 4, "silu input");
    NEED_BYTES(O, (size_t)size * 4, "silu output");
    if (size == 0) return YULE_OK;
    LAUNCHED(ctx, launch_silu_mul((const float *)I.ptr, (const float *)O.ptr, (float *)O.ptr, size,
                                  ctx->stream, &_n));
    return YULE_OK;
}

int32_t yule_cuda_element_mul(yule_cuda_ctx *ctx, yule_buffer a, yule_buffer b, yule_buffer output,
                              uint32_t size) {
    CTX_GUARD(ctx);
    FIND(ctx, a, A);
    FIND(ctx, b, B);
    FIND(ctx, output, O);
    NEED_BYTES(A, (size_t)size * 4, "element_mul a");
    NEED_BYTES(B, (size_t)size * 4, "element_mul b");
    NEED_BYTES(O, (size_t)size * 4, "element_mul output");
    if (size == 0) return YULE_OK;
    LAUNCHED(ctx, launch_silu_mul((const float *)A.ptr, (const float *)B.ptr, (float *)O.ptr, size,
                                  ctx->stream, &_n));
    return YULE_OK;
}

int32_t yule_cuda_add(yule_cuda_ctx *ctx, yule_buffer a, yule_buffer b, yule_buffer output, uint32_t size) {
    CTX_GUARD(ctx);
    FIND(ctx, a, A);
    FIND(ctx, b, B);
    FIND(ctx, output, O);
    NEED_BYTES(A, (size_t)size * 4, "add a");
    NEED_BYTES(B, (size_t)size * 4, "add b");
    NEED_BYTES(O, (size_t)size * 4, "add output");
    if (size == 0) return YULE_OK;
    LAUNCHED(ctx, launch_add((const float *)A.ptr, (const float *)B.ptr, (float *)O.ptr, size, ctx->stream,
                             &_n));
    return YULE_OK;
}

int32_t yule_cuda_attn_score(yule_cuda_ctx *ctx, yule_buffer q, yule_buffer k_cache, yule_buffer scores,
                             uint32_t head_dim, uint32_t seq_len, uint32_t head_offset, uint32_t kv_offset,
                             uint32_t kv_stride) {
    CTX_GUARD(ctx);
    FIND(ctx, q, Q);
    FIND(ctx, k_cache, K);
    FIND(ctx, scores, S);
    if (seq_len == 0) return YULE_OK;
    NEED_BYTES(Q, ((size_t)head_offset + head_dim) * 4, "attn_score q");
    NEED_BYTES(K, ((size_t)(seq_len - 1) * kv_stride + kv_offset + head_dim) * 4, "attn_score k_cache");
    NEED_BYTES(S, (size_t)seq_len * 4, "attn_score scores");
    LAUNCHED(ctx, launch_attn_score((const float *)Q.ptr, (const float *)K.ptr, (float *)S.ptr, head_dim,
                                    seq_len, head_offset, kv_offset, kv_stride, ctx->stream, &_n));
    return YULE_OK;
}

int32_t yule_cuda_attn_value(yule_cuda_ctx *ctx, yule_buffer weights, yule_buffer v_cache, yule_buffer output,
                             uint32_t head_dim, uint32_t seq_len, uint32_t kv_offset, uint32_t kv_stride,
                             uint32_t out_offset) {
    CTX_GUARD(ctx);
    FIND(ctx, weights, W);
    FIND(ctx, v_cache, V);
    FIND(ctx, output, O);
    NEED_BYTES(W, (size_t)seq_len * 4, "attn_value weights");
    if (seq_len)
        NEED_BYTES(V, ((size_t)(seq_len - 1) * kv_stride + kv_offset + head_dim) * 4, "attn_value v_cache");
    NEED_BYTES(O, ((size_t)out_offset + head_dim) * 4, "attn_value output");
    if (head_dim == 0) return YULE_OK;
    LAUNCHED(ctx, launch_attn_value((const float *)W.ptr, (const float *)V.ptr, (float *)O.ptr, head_dim,
                                    seq_len, kv_offset, kv_stride, out_offset, ctx->stream, &_n));
    return YULE_OK;
}

// From how many activation rows the tcgen05 GEMM beats ceil(batch / 4) passes of the matvec kernels
// (measured on 1024x4096 .. 128256x4096): the exact Q4_K kernel from 16 (from 32 on matrices of up to 8M weights,
// where four passes of the batched matvec cost less than the GEMM's fixed part), the generic kernel of the other
// formats from 32, except Q5_K (tensor-pipe matvec at 3.5 us per row against a 195 us GEMM) from 64; from 8 where the
// rows are too long for a batched matvec kernel to hold its activation image.  YULE_GEMM_MIN_BATCH overrides all of
// them (at least 8).
static uint32_t gemm_min_batch(const QmvArgs &a) {
    if (const char *e = knob("YULE_GEMM_MIN_BATCH")) {
        const int v = atoi(e);
        return v < 8 ? 8u : (uint32_t)v;
    }
    const bool tuned = a.type == YULE_DTYPE_Q4_K || a.type == YULE_DTYPE_Q6_K || a.type == YULE_DTYPE_Q8_0 || a.type == YULE_DTYPE_Q4_0;
    if (tuned && a.batch >= 8 && kquant_batch_width(a) < 2 && q8q4_ring_batch_width(a) < 2) return 8u;
    if (a.type == YULE_DTYPE_Q4_K) return (uint64_t)a.n_rows * a.n_cols <= (8ull << 20) ? 32u : 16u;
    return a.type == YULE_DTYPE_Q5_K ? 64u : 32u;
}

static int32_t qmv_common(yule_cuda_ctx *ctx, yule_buffer weights, size_t weight_offset, yule_buffer input,
                          yule_buffer output, uint32_t n_rows, uint32_t n_cols, uint32_t type, uint32_t batch,
                          uint32_t x_stride, uint32_t out_stride) {
    CTX_GUARD(ctx);
    if (!is_quantized(type))
        return fail(YULE_ERR_UNSUPPORTED_DTYPE, "unsupported dtype for CUDA qmv: GGUF type %u", type);
    uint32_t bs = block_size(type);
    if (n_cols == 0 || n_cols % bs)
        return fail(YULE_ERR_INVALID_ARGUMENT, "n_cols %u is not a multiple of the block size %u", n_cols, bs);
    if (batch == 0 || x_stride < n_cols || out_stride < n_rows || x_stride % 4)
        return fail(YULE_ERR_INVALID_ARGUMENT, "bad batch/stride (batch %u, x_stride %u, out_stride %u)", batch,
                    x_stride, out_stride);
    uint32_t align = (type == YULE_DTYPE_Q4_K) ? 16 : 2;
    if (weight_offset % align)
        return fail(YULE_ERR_INVALID_ARGUMENT, "weight offset %zu is not a multiple of %u", weight_offset, align);
    FIND(ctx, weights, W);
    FIND(ctx, input, X);
    FIND(ctx, output, O);
    size_t wbytes = tensor_bytes(type, n_rows, n_cols);
    if (weight_offset > W.size || wbytes > W.size - weight_offset)
        return fail(YULE_ERR_OUT_OF_BOUNDS, "quantized_matmul weights need [%zu, %zu) of a %zu-byte buffer",
                    weight_offset, weight_offset + wbytes, W.size);
    NEED_BYTES(X, ((size_t)(batch - 1) * x_stride + n_cols) * 4, "quantized_matmul input");
    NEED_BYTES(O, ((size_t)(batch - 1) * out_stride + n_rows) * 4, "quantized_matmul output");
    if (n_rows == 0) return YULE_OK;
    QmvArgs a;
    a.w = (const uint8_t *)W.ptr + weight_offset;
    a.x = (const float *)X.ptr;
    a.out = (float *)O.ptr;
    a.n_rows = n_rows;
    a.n_cols = n_cols;
    a.type = type;
    a.batch = batch;
    a.x_stride = x_stride;
    a.out_stride = out_stride;
    if (type == YULE_DTYPE_Q6_K && W.planar && weight_offset == 0 && W.planar_cols == n_cols &&
        W.planar_blocks == (uint64_t)n_rows * (n_cols / 256))
        a.planar = W.planar;
    if (batch >= 8 && batch >= gemm_min_batch(a) && qgemm_supported(type, n_cols, batch)) {
        // enough activation rows: one pass over the weights on the tcgen05 GEMM
        int32_t rc = ensure_gemm_scratch(ctx, qgemm_scratch_bytes(batch, n_cols));
        if (rc) return rc;
        QGemm g;
        g.w = a.w;
        g.type = type;
        g.x = a.x;
        g.out = a.out;
        g.n_rows = n_rows;
        g.n_cols = n_cols;
        g.n_tokens = batch;
        g.x_stride = x_stride;
        g.out_stride = out_stride;
        g.scratch = ctx->gemm_scratch;
        g.status = ctx->device_status;
        LAUNCHED(ctx, launch_qgemm(g, ctx->prop.multiProcessorCount, ctx->stream, &_n));
        return YULE_OK;
    }
    // Consecutive matvec calls overlap through programmatic dependent launch.  The kernels read their weights
    // before the dependency wait, so the chain is used only when the previous call on this context was a matvec
    // too and no call that may still be running writes what this one reads as weights.  When its activations
    // are not such an output either (Q, K and V from one normed vector; gate and up), nothing this kernel reads
    // depends on its predecessors: only its stores are ordered behind them (late wait).
    const char *w_lo = (const char *)a.w, *w_hi = w_lo + wbytes;
    const char *x_lo = (const char *)X.ptr, *x_hi = x_lo + ((size_t)(batch - 1) * x_stride + n_cols) * 4;
    const char *o_lo = (const char *)O.ptr, *o_hi = o_lo + ((size_t)(batch - 1) * out_stride + n_rows) * 4;
    bool w_hazard = false, x_hazard = false;
    ctx->chain_n = _chain_n;  // (the guard above ended the chain for every other entry point)
    for (int i = 0; i < ctx->chain_n; i++) {
        w_hazard = w_hazard || (w_lo < ctx->chain_hi[i] && ctx->chain_lo[i] < w_hi);
        x_hazard = x_hazard || (x_lo < ctx->chain_hi[i] && ctx->chain_lo[i] < x_hi);
    }
    a.pdl = _pdl_chain && !w_hazard;
    a.late_wait = a.pdl && !x_hazard && ctx->chain_n < yule_cuda_ctx::kChainRanges;
    a.status = ctx->device_status;
    a.wait_cycles = ctx->wait_cycles;
    LAUNCHED(ctx, launch_qmv(a, ctx->prop.multiProcessorCount, ctx->stream, &_n));
    ctx->pdl_chain = true;
    if (!a.late_wait) ctx->chain_n = 0;  // this kernel waits for all its predecessors before it reads or writes
    bool listed = false;
    for (int i = 0; i < ctx->chain_n; i++) listed = listed || (ctx->chain_lo[i] <= o_lo && o_hi <= ctx->chain_hi[i]);
    if (!listed) {
        ctx->chain_lo[ctx->chain_n] = o_lo;
        ctx->chain_hi[ctx->chain_n] = o_hi;
        ctx->chain_n++;
    }
    return YULE_OK;
}

int32_t yule_cuda_quantized_matmul(yule_cuda_ctx *ctx, yule_buffer weights, yule_buffer input,
                                   yule_buffer output, uint32_t n_rows, uint32_t n_cols, uint32_t gguf_type) {
    return qmv_common(ctx, weights, 0, input, output, n_rows, n_cols, gguf_type, 1, n_cols, n_rows);
}

int32_t yule_cuda_quantized_matmul_at(yule_cuda_ctx *ctx, yule_buffer weights, size_t weight_offset,
                                      yule_buffer input, yule_buffer output, uint32_t n_rows, uint32_t n_cols,
                                      uint32_t gguf_type) {
    return qmv_common(ctx, weights, weight_offset, input, output, n_rows, n_cols, gguf_type, 1, n_cols, n_rows);
}

int32_t yule_cuda_quantized_matmul_batched(yule_cuda_ctx *ctx, yule_buffer weights, yule_buffer input,
                                           yule_buffer output, uint32_t n_rows, uint32_t n_cols,
                                           uint32_t gguf_type, uint32_t batch, uint32_t x_stride,
                                           uint32_t out_stride) {
    return qmv_common(ctx, weights, 0, input, output, n_rows, n_cols, gguf_type, batch, x_stride, out_stride);
}

int32_t yule_cuda_prepare_weights(yule_cuda_ctx *ctx, yule_buffer weights, uint32_t gguf_type, uint32_t n_rows,
                                  uint32_t n_cols) {
    CTX_GUARD(ctx);
    if (!is_quantized(gguf_type))
        return fail(YULE_ERR_UNSUPPORTED_DTYPE, "unsupported dtype for CUDA qmv: GGUF type %u", gguf_type);
    if (n_cols == 0 || n_cols % block_size(gguf_type))
        return fail(YULE_ERR_INVALID_ARGUMENT, "n_cols %u is not a multiple of the block size", n_cols);
    FIND(ctx, weights, W);
    NEED_BYTES(W, tensor_bytes(gguf_type, n_rows, n_cols), "prepare_weights");
    if (gguf_type != YULE_DTYPE_Q6_K || !q6k_mma_supported(n_cols) || n_rows == 0) return YULE_OK;
    const uint64_t n_blocks = (uint64_t)n_rows * (n_cols / 256);
    if (W.planar && W.planar_blocks == n_blocks && W.planar_cols == n_cols) return YULE_OK;
    if (W.planar) {
        int32_t rc = drop_planar(ctx, weights);
        if (rc) return rc;
    }
    uint8_t *planar = nullptr;
    cudaError_t e = cudaMalloc((void **)&planar, q6k_planar_bytes(n_rows, n_cols));
    if (e != cudaSuccess) {
        cudaGetLastError();
        return fail(YULE_ERR_OUT_OF_MEMORY, "cuda allocation of the planar Q6_K copy (%zu bytes) failed",
                    q6k_planar_bytes(n_rows, n_cols));
    }
    {
        uint64_t _n = 0;
        e = launch_q6k_repack((const uint8_t *)W.ptr, planar, n_rows, n_cols, ctx->stream, &_n);
        ctx->launches.fetch_add(_n);
    }
    if (e != cudaSuccess) {
        cudaFree(planar);
        return fail_cuda(e, "Q6_K repack");
    }
    std::lock_guard<std::mutex> lock(ctx->mu);
    auto it = ctx->buffers.find(weights);
    if (it == ctx->buffers.end()) {
        cudaFree(planar);
        return fail(YULE_ERR_UNKNOWN_BUFFER, "buffer freed during prepare_weights");
    }
    it->second.planar = planar;
    it->second.planar_blocks = n_blocks;
    it->second.planar_cols = n_cols;
    return YULE_OK;
}

int32_t yule_cuda_dequantize(yule_cuda_ctx *ctx, yule_buffer weights, uint32_t gguf_type, uint64_t n_blocks,
                             yule_buffer out_f32) {
    CTX_GUARD(ctx);
    if (!is_quantized(gguf_type) && gguf_type != YULE_DTYPE_F16 && gguf_type != YULE_DTYPE_F32)
        return fail(YULE_ERR_UNSUPPORTED_DTYPE, "dequant not implemented for GGUF type %u", gguf_type);
    FIND(ctx, weights, W);
    FIND(ctx, out_f32, O);
    NEED_BYTES(W, n_blocks * block_bytes(gguf_type), "dequantize weights");
    NEED_BYTES(O, n_blocks * block_size(gguf_type) * 4, "dequantize output");
    if (n_blocks == 0) return YULE_OK;
    LAUNCHED(ctx, launch_dequantize((const uint8_t *)W.ptr, gguf_type, n_blocks, (float *)O.ptr, ctx->stream,
                                    &_n));
    return YULE_OK;
}

int32_t yule_cuda_multihead_attention(yule_cuda_ctx *ctx, yule_buffer q, yule_buffer k_cache, yule_buffer v_cache,
                                      yule_buffer out, uint32_t head_dim, uint32_t seq_len, uint32_t n_heads,
                                      uint32_t n_kv_heads, uint32_t kv_stride) {
    CTX_GUARD(ctx);
    if (n_kv_heads == 0 || n_heads == 0 || n_heads % n_kv_heads || head_dim == 0 || seq_len == 0)
        return fail(YULE_ERR_INVALID_ARGUMENT, "bad attention shape (heads %u, kv heads %u, head_dim %u, seq %u)",
                    n_heads, n_kv_heads, head_dim, seq_len);
    if (head_dim > 256) return fail(YULE_ERR_INVALID_ARGUMENT, "head_dim %u above 256", head_dim);
    FIND(ctx, q, Q);
    FIND(ctx, k_cache, K);
    FIND(ctx, v_cache, V);
    FIND(ctx, out, O);
    size_t kv_need = ((size_t)(seq_len - 1) * kv_stride + (size_t)n_kv_heads * head_dim) * 4;
    NEED_BYTES(Q, (size_t)n_heads * head_dim * 4, "attention q");
    NEED_BYTES(K, kv_need, "attention k_cache");
    NEED_BYTES(V, kv_need, "attention v_cache");
    NEED_BYTES(O, (size_t)n_heads * head_dim * 4, "attention out");
    if (attn_decode_supported(head_dim) && kv_stride % 4 == 0) {
        // split over positions; the partial results live in a context-owned scratch grown on demand
        AttnDecode a;
        a.gqa = attn_gqa_supported(head_dim, n_heads, n_kv_heads) && seq_len >= 512;
        a.n_splits = a.gqa ? attn_gqa_pick_splits(n_kv_heads, seq_len, ctx->prop.multiProcessorCount)
                           : attn_pick_splits(n_heads, seq_len, ctx->prop.multiProcessorCount);
        const size_t need = attn_scratch_floats(n_heads, a.n_splits, head_dim);
        {
            std::lock_guard<std::mutex> lock(ctx->mu);
            if (a.n_splits > 1 && (ctx->attn_scratch_floats < need || ctx->attn_tickets_n < n_heads)) {
                YULE_CUDA_TRY(cudaStreamSynchronize(ctx->stream));
                if (ctx->capturing)
                    return fail(YULE_ERR_INVALID_ARGUMENT, "the attention scratch cannot grow during graph capture: run the call once outside the capture first");
                // graphs captured earlier may still replay into the old blocks: retire them, do not free them
                if (ctx->attn_scratch) ctx->retired_scratch.push_back(ctx->attn_scratch);
                if (ctx->attn_tickets) ctx->retired_scratch.push_back(ctx->attn_tickets);
                ctx->attn_scratch = nullptr;
                ctx->attn_tickets = nullptr;
                ctx->attn_scratch_floats = ctx->attn_tickets_n = 0;
                YULE_CUDA_TRY(cudaMalloc((void **)&ctx->attn_scratch, need * sizeof(float)));
                YULE_CUDA_TRY(cudaMalloc((void **)&ctx->attn_tickets, (size_t)n_heads * sizeof(uint32_t)));
                YULE_CUDA_TRY(cudaMemsetAsync(ctx->attn_tickets, 0, (size_t)n_heads * sizeof(uint32_t), ctx->stream));
                ctx->attn_scratch_floats = need;
                ctx->attn_tickets_n = n_heads;
            }
            a.scratch = ctx->attn_scratch;
            a.tickets = ctx->attn_tickets;
        }
        a.q = (const float *)Q.ptr;
        a.k_cache = (float *)K.ptr;
        a.v_cache = (float *)V.ptr;
        a.seq_len = seq_len;
        a.out = (float *)O.ptr;
        a.hd = head_dim;
        a.n_heads = n_heads;
        a.n_kv_heads = n_kv_heads;
        a.kv_stride = kv_stride;
        a.max_seq_len = seq_len;
        LAUNCHED(ctx, launch_attn_decode(a, ctx->stream, &_n));
        return YULE_OK;
    }
    LAUNCHED(ctx, launch_multihead_attention((const float *)Q.ptr, (const float *)K.ptr, (const float *)V.ptr,
                                             (float *)O.ptr, head_dim, seq_len, nullptr, seq_len, n_heads,
                                             n_kv_heads, kv_stride, ctx->stream, &_n));
    return YULE_OK;
}

int32_t yule_cuda_embed_gather(yule_cuda_ctx *ctx, yule_buffer table, uint32_t gguf_type, uint32_t dim,
                               uint32_t token, yule_buffer out) {
    CTX_GUARD(ctx);
    uint32_t bs = block_size(gguf_type);
    if (bs == 0) return fail(YULE_ERR_UNSUPPORTED_DTYPE, "embedding dtype %u not supported", gguf_type);
    if (dim == 0 || dim % bs) return fail(YULE_ERR_INVALID_ARGUMENT, "dim %u not a multiple of block size %u", dim, bs);
    FIND(ctx, table, T);
    FIND(ctx, out, O);
    size_t row_bytes = (size_t)(dim / bs) * block_bytes(gguf_type);
    NEED_BYTES(T, ((size_t)token + 1) * row_bytes, "embedding table");
    NEED_BYTES(O, (size_t)dim * 4, "embedding out");
    LAUNCHED(ctx, launch_embed_gather((const uint8_t *)T.ptr, gguf_type, dim, token, nullptr, (float *)O.ptr,
                                      ctx->stream, &_n));
    return YULE_OK;
}

// ── graph capture / replay ─────────────────────────────────────────────────────────────────

int32_t yule_cuda_graph_begin(yule_cuda_ctx *ctx) {
    CTX_GUARD(ctx);
    if (ctx->capturing) return fail(YULE_ERR_INVALID_ARGUMENT, "graph capture already in progress");
    YULE_CUDA_TRY(cudaStreamBeginCapture(ctx->stream, cudaStreamCaptureModeRelaxed));
    ctx->capturing = true;
    ctx->launches_at_capture_begin = ctx->launches.load();
    return YULE_OK;
}

int32_t yule_cuda_graph_end(yule_cuda_ctx *ctx, uint32_t *out_graph_id) {
    CTX_GUARD(ctx);
    if (!ctx->capturing) return fail(YULE_ERR_INVALID_ARGUMENT, "no graph capture in progress");
    ctx->capturing = false;
    cudaGraph_t graph = nullptr;
    cudaError_t e = cudaStreamEndCapture(ctx->stream, &graph);
    // Captured launches did not run; they count each time the graph is replayed.
    uint64_t captured = ctx->launches.load() - ctx->launches_at_capture_begin;
    ctx->launches.fetch_sub(captured);
    if (e != cudaSuccess) {
        if (graph) cudaGraphDestroy(graph);
        return fail_cuda(e, "cudaStreamEndCapture");
    }
    if (!out_graph_id) {
        cudaGraphDestroy(graph);
        return fail(YULE_ERR_INVALID_ARGUMENT, "null out_graph_id");
    }
    yule_cuda_ctx::Graph g;
    e = cudaGraphInstantiate(&g.exec, graph, 0);
    cudaGraphDestroy(graph);
    if (e != cudaSuccess) return fail_cuda(e, "cudaGraphInstantiate");
    g.kernels = captured;
    std::lock_guard<std::mutex> lock(ctx->mu);
    ctx->graphs.push_back(g);
    *out_graph_id = (uint32_t)ctx->graphs.size() - 1;
    return YULE_OK;
}

int32_t yule_cuda_graph_launch(yule_cuda_ctx *ctx, uint32_t graph_id) {
    CTX_GUARD(ctx);
    yule_cuda_ctx::Graph g;
    {
        std::lock_guard<std::mutex> lock(ctx->mu);
        if (graph_id >= ctx->graphs.size() || !ctx->graphs[graph_id].exec)
            return fail(YULE_ERR_INVALID_ARGUMENT, "unknown graph %u", graph_id);
        g = ctx->graphs[graph_id];
    }
    YULE_CUDA_TRY(cudaGraphLaunch(g.exec, ctx->stream));
    ctx->launches.fetch_add(g.kernels);
    return YULE_OK;
}

int32_t yule_cuda_graph_destroy(yule_cuda_ctx *ctx, uint32_t graph_id) {
    CTX_GUARD(ctx);
    YULE_CUDA_TRY(cudaStreamSynchronize(ctx->stream));
    std::lock_guard<std::mutex> lock(ctx->mu);
    if (graph_id >= ctx->graphs.size() || !ctx->graphs[graph_id].exec)
        return fail(YULE_ERR_INVALID_ARGUMENT, "unknown graph %u", graph_id);
    cudaGraphExecDestroy(ctx->graphs[graph_id].exec);
    ctx->graphs[graph_id].exec = nullptr;
    return YULE_OK;
}

// Sampler::sample_with_history (yule-infer/src/sampler.rs:17-136) on the device.
int32_t yule_cuda_sample(yule_cuda_ctx *ctx, yule_buffer logits, uint32_t n, const yule_sampling_params *params,
                         yule_buffer previous_tokens, uint32_t n_previous, float random_value, uint32_t *out_token) {
    CTX_GUARD(ctx);
    if (!params || !out_token) return fail(YULE_ERR_INVALID_ARGUMENT, "null argument");
    if (n == 0) return fail(YULE_ERR_INVALID_ARGUMENT, "empty logits");  // sampler.rs:19-21
    if (!(random_value >= 0.0f && random_value < 1.0f)) return fail(YULE_ERR_INVALID_ARGUMENT, "the random value must lie in [0, 1)");
    FIND(ctx, logits, L);
    NEED_BYTES(L, (size_t)n * 4, "sample logits");
    const uint32_t *prev = nullptr;
    if (n_previous) {
        FIND(ctx, previous_tokens, P);
        NEED_BYTES(P, (size_t)n_previous * 4, "sample previous tokens");
        prev = (const uint32_t *)P.ptr;
    }
    int32_t rc = ensure_sampler_scratch(ctx, 2 * (size_t)n + 4);
    if (rc) return rc;
    SampleArgs a;
    a.logits = (const float *)L.ptr;
    a.n = n;
    a.temperature = params->temperature;
    a.top_p = params->top_p;
    a.top_k = params->top_k;
    a.min_p = params->min_p;
    a.repetition_penalty = params->repetition_penalty;
    a.previous = prev;
    a.n_previous = n_previous;
    a.r = random_value;
    a.scratch = ctx->sampler_scratch;
    a.out_token = reinterpret_cast<uint32_t *>(ctx->sampler_scratch + 2 * (size_t)n);
    LAUNCHED(ctx, launch_sample(a, ctx->stream, &_n));
    YULE_CUDA_TRY(cudaMemcpyAsync(out_token, a.out_token, 4, cudaMemcpyDeviceToHost, ctx->stream));
    YULE_CUDA_TRY(cudaStreamSynchronize(ctx->stream));
    return YULE_OK;
}

// ── timing helpers ─────────────────────────────────────────────────────────────────────────

int32_t yule_cuda_event_record(yule_cuda_ctx *ctx, uint32_t *out_event_id) {
    CTX_GUARD(ctx);
    if (!out_event_id) return fail(YULE_ERR_INVALID_ARGUMENT, "null out_event_id");
    cudaEvent_t ev;
    YULE_CUDA_TRY(cudaEventCreate(&ev));
    YULE_CUDA_TRY(cudaEventRecord(ev, ctx->stream));
    std::lock_guard<std::mutex> lock(ctx->mu);
    ctx->events.push_back(ev);
    *out_event_id = (uint32_t)ctx->events.size() - 1;
    return YULE_OK;
}

int32_t yule_cuda_event_elapsed_ms(yule_cuda_ctx *ctx, uint32_t start_id, uint32_t end_id, float *out_ms) {
    CTX_GUARD(ctx);
    cudaEvent_t a, b;
    {
        std::lock_guard<std::mutex> lock(ctx->mu);
        if (start_id >= ctx->events.size() || end_id >= ctx->events.size())
            return fail(YULE_ERR_INVALID_ARGUMENT, "unknown event id");
        a = ctx->events[start_id];
        b = ctx->events[end_id];
    }
    YULE_CUDA_TRY(cudaEventSynchronize(b));
    YULE_CUDA_TRY(cudaEventElapsedTime(out_ms, a, b));
    return YULE_OK;
}

int32_t yule_cuda_event_reset(yule_cuda_ctx *ctx) {
    CTX_GUARD(ctx);
    YULE_CUDA_TRY(cudaStreamSynchronize(ctx->stream));
    std::lock_guard<std::mutex> lock(ctx->mu);
    for (auto ev : ctx->events) cudaEventDestroy(ev);
    ctx->events.clear();
    return YULE_OK;
}

int32_t yule_cuda_flush_l2(yule_cuda_ctx *ctx) {
    CTX_GUARD(ctx);
    if (!ctx->flush_buf) {
        // Twice the L2 size, so that nothing of an earlier kernel's inputs survives.
        size_t bytes = (size_t)ctx->prop.l2CacheSize * 2;
        if (bytes < ((size_t)256 << 20)) bytes = (size_t)256 << 20;
        YULE_CUDA_TRY(cudaMalloc(&ctx->flush_buf, bytes));
        ctx->flush_bytes = bytes;
    }
    LAUNCHED(ctx, launch_fill_bytes(ctx->flush_buf, ctx->flush_bytes, 0, ctx->stream, &_n));
    return YULE_OK;
}

int32_t yule_cuda_launch_count(yule_cuda_ctx *ctx, uint64_t *out_count) {
    if (!ctx || !out_count) return fail(YULE_ERR_INVALID_ARGUMENT, "null argument");
    *out_count = ctx->launches.load();
    return YULE_OK;
}

}  // extern "C"
