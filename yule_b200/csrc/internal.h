// internal.h — shared declarations of libyule_cuda.so (context, buffer table, kernel launchers).
#pragma once

#include <cuda_runtime.h>


#include <atomic>
#include <cstdarg>
#include <cstdint>
#include <cstdio>
#include <mutex>
#include <string>
#include <unordered_map>
#include <vector>

#include "../../include/yule_cuda.h"

#ifdef __CUDACC__
// Programmatic dependent launch: a kernel launched with the attribute may start while its
// predecessor drains; everything it reads that the predecessor wrote must come after the wait.
// Both are no-ops for a normal launch.
__device__ __forceinline__ void yule_pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
__device__ __forceinline__ void yule_pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
// Asks L2 to fetch [p, p + bytes) from HBM without waiting for it (p 16-byte aligned, bytes a
// multiple of 16).  Used by a matvec to pull in the weights of the kernel that runs after it,
// so HBM keeps streaming across the dependency between the two.
__device__ __forceinline__ void yule_prefetch_l2(const void *p, uint32_t bytes) {
    asm volatile("cp.async.bulk.prefetch.L2.global [%0], %1;" ::"l"(p), "r"(bytes) : "memory");
}
// Each CTA takes an equal 16-byte-granular slice of [base, base + bytes) and prefetches it in
// pieces of at most 32 KB from one thread.
__device__ __forceinline__ void yule_prefetch_l2_slice(const void *base, uint64_t bytes) {
    if (!base || threadIdx.x != 0) return;
    const uint64_t per = ((bytes / gridDim.x) + 15) & ~(uint64_t)15;
    uint64_t lo = (uint64_t)blockIdx.x * per;
    uint64_t hi = lo + per < bytes ? lo + per : (bytes & ~(uint64_t)15);
    for (; lo < hi; lo += 32768) {
        const uint64_t n = hi - lo < 32768 ? hi - lo : 32768;
        yule_prefetch_l2(reinterpret_cast<const char *>(base) + lo, (uint32_t)n);
    }
}
#endif

namespace yule {

// Values of the device status word (yule_cuda_ctx::device_status): which bounded wait gave up.
constexpr int kStatusPeerTimeout = 2;   // tensor parallelism: a peer's (value, epoch) pairs or flag never arrived
constexpr int kStatusGemmTimeout = 3;   // tcgen05 GEMM: an mbarrier of its pipeline never completed
constexpr int kStatusRingTimeout = 4;   // matvec: a bulk copy into the shared-memory ring never completed
// Default budget of a bounded wait, in SM clock cycles (~1 s): far beyond any real skew between ranks,
// short enough to report a lost peer.  yule_cuda_set_wait_budget changes it per context.
constexpr long long kDefaultWaitCycles = 2000000000LL;

struct Buffer {
    void *ptr = nullptr;
    size_t size = 0;      // bytes the caller asked for
    size_t capacity = 0;  // bytes allocated (rounded up, so 16-byte over-reads stay in bounds)
    // Optional row-planar device copy of a Q6_K tensor held in this buffer (yule_cuda_prepare_weights);
    // dropped whenever the buffer is written.
    uint8_t *planar = nullptr;
    uint64_t planar_blocks = 0;
    uint32_t planar_cols = 0;  // the copy is laid out row by row, so it belongs to one (rows, cols) shape
};

// Tuning and timing knobs (YULE_QMV_*, YULE_GEMM_*, YULE_CUDA_*, YULE_TP_*) are read from the environment only
// when the process runs with YULE_CUDA_DEBUG=1; a production process ignores them, so no environment
// variable can change routing or results.  Returns the variable's value or null.
const char *knob(const char *name);

// Sets the calling thread's error text and returns `code`.
int32_t fail(int32_t code, const char *fmt, ...);
int32_t fail_cuda(cudaError_t e, const char *what);

#define YULE_CUDA_TRY(expr)                                   \
    do {                                                      \
        cudaError_t _e = (expr);                              \
        if (_e != cudaSuccess) return fail_cuda(_e, #expr);   \
    } while (0)

}  // namespace yule

struct yule_cuda_ctx {
    int device = 0;
    cudaStream_t stream = nullptr;
    cudaDeviceProp prop{};
    std::mutex mu;
    std::unordered_map<uint64_t, yule::Buffer> buffers;
    uint64_t next_handle = 1;
    std::vector<cudaEvent_t> events;
    struct Graph {
        cudaGraphExec_t exec = nullptr;
        uint64_t kernels = 0;
    };
    std::vector<Graph> graphs;
    bool capturing = false;
    uint64_t launches_at_capture_begin = 0;
    void *flush_buf = nullptr;
    size_t flush_bytes = 0;
    // tensor parallelism (tp.cu): NCCL communicator of this rank, or null when single-GPU
    void *tp_comm = nullptr;
    uint32_t tp_rank = 0, tp_world = 1;
    float *tp_peer_base[8] = {};  // exchange regions: own allocation at [tp_rank], peers' mappings elsewhere
    size_t tp_flag_offset = 0, tp_xchg_floats = 0;
    // scratch of the split-KV attention entry point, grown on demand
    float *attn_scratch = nullptr;
    size_t attn_scratch_floats = 0;
    uint32_t *attn_tickets = nullptr;
    size_t attn_tickets_n = 0;
    // activation tiles of the tensor-core GEMM (qgemm_tc.cu), grown on demand
    void *gemm_scratch = nullptr;
    size_t gemm_scratch_bytes = 0;
    // scratch of the device sampler (sampler.cu): probabilities and occurrence counts, plus one word for the pick
    float *sampler_scratch = nullptr;
    size_t sampler_scratch_floats = 0;
    // Scratch blocks that were outgrown.  A CUDA graph captured earlier (the runner's steps, a caller's batch)
    // may still replay into them, so they are kept until the context is destroyed instead of being freed.
    std::vector<void *> retired_scratch;
    std::atomic<uint64_t> launches{0};
    // Word the kernels with bounded waits write when they give up; read by synchronize.
    int *device_status = nullptr;
    long long wait_cycles = yule::kDefaultWaitCycles;  // budget of every bounded device-side wait
    // Programmatic dependent launch between consecutive matvec calls of the trait API: allowed only when the
    // previous operation enqueued on the stream was one of this library's kernels, and its output does not
    // overlap the weights of the call being launched (weights are read before the dependency wait).
    bool pdl_chain = false;
    // Outputs of the matvec calls of the current chain that may still be running when the next one starts:
    // a kernel that waits for its predecessor before reading anything settles everything before it, a kernel
    // whose stores alone wait (late wait) does not.
    static constexpr int kChainRanges = 8;
    const char *chain_lo[kChainRanges] = {}, *chain_hi[kChainRanges] = {};
    int chain_n = 0;

    // Looks a handle up under the lock; returns false (and sets the error) when unknown.
    bool find(yule_buffer h, yule::Buffer *out, const char *what);
};

namespace yule {

// The four formats with tuned matvec and tensor-core GEMM kernels.
inline bool is_tuned_format(uint32_t t) {
    return t == YULE_DTYPE_Q4_0 || t == YULE_DTYPE_Q8_0 || t == YULE_DTYPE_Q4_K || t == YULE_DTYPE_Q6_K;
}
// Every block format the kernels can read: the tuned four plus the formats that run through the
// element-wise matvec (Yule's own GPU backends reject those, yule-gpu/src/cuda/mod.rs:303-307).
inline bool is_quantized(uint32_t t) {
    switch (t) {
        case YULE_DTYPE_Q4_1: case YULE_DTYPE_Q5_0: case YULE_DTYPE_Q5_1: case YULE_DTYPE_Q8_1:
        case YULE_DTYPE_Q2_K: case YULE_DTYPE_Q3_K: case YULE_DTYPE_Q5_K: return true;
        default: return is_tuned_format(t);
    }
}
inline uint32_t block_size(uint32_t t) {  // yule-core/src/dtype.rs:99-118
    switch (t) {
        case YULE_DTYPE_F32: case YULE_DTYPE_F16: return 1;
        case YULE_DTYPE_Q4_0: case YULE_DTYPE_Q8_0: case YULE_DTYPE_Q4_1: case YULE_DTYPE_Q5_0:
        case YULE_DTYPE_Q5_1: case YULE_DTYPE_Q8_1: return 32;
        case YULE_DTYPE_Q4_K: case YULE_DTYPE_Q6_K: case YULE_DTYPE_Q2_K: case YULE_DTYPE_Q3_K:
        case YULE_DTYPE_Q5_K: return 256;
        default: return 0;
    }
}
inline uint32_t block_bytes(uint32_t t) {  // yule-core/src/dtype.rs:62-96
    switch (t) {
        case YULE_DTYPE_F32: return 4;
        case YULE_DTYPE_F16: return 2;
        case YULE_DTYPE_Q4_0: return 18;
        case YULE_DTYPE_Q8_0: return 34;
        case YULE_DTYPE_Q4_K: return 144;
        case YULE_DTYPE_Q6_K: return 210;
        case YULE_DTYPE_Q4_1: return 20;
        case YULE_DTYPE_Q5_0: return 22;
        case YULE_DTYPE_Q5_1: return 24;
        case YULE_DTYPE_Q8_1: return 36;
        case YULE_DTYPE_Q2_K: return 84;
        case YULE_DTYPE_Q3_K: return 110;
        case YULE_DTYPE_Q5_K: return 176;
        default: return 0;
    }
}
inline size_t tensor_bytes(uint32_t t, uint64_t n_rows, uint64_t n_cols) {
    return (size_t)(n_rows * (n_cols / block_size(t)) * block_bytes(t));
}

// ── kernel launchers (raw device pointers; arguments already validated) ──────────────────────
// Each returns the cudaError_t of the launch and adds the kernels it launched to *launches.

// Tensor parallelism folded into a matvec (set-up in tp.cu), flag-in-data form.  A gathered vector has, next
// to its plain copy, a copy of (value, epoch) pairs in every rank's exchange region.  Producer side: as each
// output row is reduced the kernel stores the pair, one 8-byte store, into every rank's pair buffer (its own
// included).  Consumer side: the kernel that reads the gathered vector reads the pairs and polls — for a
// bounded time, reporting through `status` — until every pair it needs carries the epoch of that exchange.
// No fence, no flag word, no ticket: an exchange costs one NVLink store latency.
// epoch = *tick · epochs_per_tick + index + 1 (never 0: the buffers start zeroed).
struct TpFuse {
    uint32_t world = 1, rank = 0;
    const uint32_t *tick = nullptr;
    uint32_t epochs_per_tick = 0;
    int *status = nullptr;
    long long wait_cycles = kDefaultWaitCycles;  // budget of the consumer's polling
    bool push = false;               // producer
    uint32_t push_index = 0;
    uint2 *pair_out[8] = {};         // rank p's pair buffer at this rank's slice (every rank, this one too)
    bool wait = false;               // consumer
    uint32_t wait_index = 0;
    const uint2 *pair_in = nullptr;  // this rank's pair buffer of the whole gathered vector
};

struct QmvArgs {
    const uint8_t *w;   // raw GGUF blocks, row-major
    const float *x;     // [batch][x_stride]
    float *out;         // [batch][out_stride]
    uint32_t n_rows, n_cols, type, batch, x_stride, out_stride;
    // Optional fused prologue/epilogue used by the runner (null when unused):
    const float *residual = nullptr;  // out[row] = residual[row] + dot   (o-proj / down-proj)
    bool pdl = false;                 // programmatic dependent launch
    // With pdl: none of this call's inputs (x, residual) is written by the previous kernel of the stream, so
    // only this kernel's stores have to wait for it (Q4_K / Q6_K tensor-pipe kernels; ignored elsewhere).
    bool late_wait = false;
    const uint8_t *planar = nullptr;  // Q6_K: planar copy of the same tensor, when one was prepared
    const float *norm_w = nullptr;    // RMSNorm prologue (planar Q6_K and Q4_K paths only)
    float eps = 0.f;
    const void *next_w[2] = {nullptr, nullptr};  // tensor-pipe paths: weights to prefetch into L2
    uint64_t next_bytes[2] = {0, 0};
    TpFuse tp;                        // Q4_K tensor-pipe path only
    int *status = nullptr;            // device status word for bounded waits inside the kernels, or null
    long long wait_cycles = kDefaultWaitCycles;
};
cudaError_t launch_qmv(const QmvArgs &a, int sm_count, cudaStream_t s, uint64_t *launches);
// Q8_0 / Q4_0 on the tensor pipe from a shared-memory ring (qmv_q8q4_ring.cu): n_cols a multiple of 256, weights and
// activations 16-byte aligned, one activation vector.
bool q8q4_ring_supported(const QmvArgs &a);
cudaError_t launch_q8q4_ring(const QmvArgs &a, int sm_count, cudaStream_t s, uint64_t *launches);
// The same kernels over two to four activation vectors per pass: the number of vectors one pass can take for this
// call (0: not supported), and one pass over the first `nb` vectors of `a`.
uint32_t q8q4_ring_batch_width(const QmvArgs &a);
cudaError_t launch_q8q4_ring_batch(const QmvArgs &a, uint32_t nb, int sm_count, cudaStream_t s, uint64_t *launches);

// Q4_K and Q6_K (row-planar copy) over two to four activation vectors per pass (qmv_kquant_batch.cu): the number of
// vectors one pass can take for this call (0: not supported), and one pass over the first `nb` vectors of `a`.
uint32_t kquant_batch_width(const QmvArgs &a);
cudaError_t launch_kquant_batch(const QmvArgs &a, uint32_t nb, int sm_count, cudaStream_t s, uint64_t *launches);
// Up to three matrices that read the same activation rows (Q/K/V; gate/up) as ONE launch per pass of four vectors, with
// the optional RMSNorm prologue (norm_w / eps of the arguments): whether the arguments allow it, and the launch.
bool kquant_batch_can_share(const QmvArgs *segs, uint32_t n_seg);
cudaError_t launch_kquant_batch_shared(const QmvArgs *segs, uint32_t n_seg, int sm_count, cudaStream_t s, uint64_t *launches);

// Quantised GEMM on tcgen05 for eight or more activation rows (qgemm_tc.cu): an activation
// re-layout kernel followed by the persistent GEMM.  `scratch` holds qgemm_scratch_bytes().
struct QGemm {
    const uint8_t *w = nullptr;  // Q4_K blocks, row-major
    uint32_t type = 0;
    const float *x = nullptr;    // [n_tokens][x_stride]
    const float *gate = nullptr;    // prologue: x ← silu(gate) · x (same layout as x), or null
    const float *norm_w = nullptr;  // prologue: RMSNorm with these weights, or null
    float eps = 0.f;
    float *out = nullptr;           // [n_tokens][out_stride]
    const float *residual = nullptr;  // added to out (same layout), or null
    uint32_t n_rows = 0, n_cols = 0, n_tokens = 0, x_stride = 0, out_stride = 0;
    // Further matrices of the same type and row length applied to the same activations in the same launch (Q/K/V,
    // gate/up); residual must then be null.
    uint32_t n_more = 0;
    const uint8_t *w_more[2] = {nullptr, nullptr};
    float *out_more[2] = {nullptr, nullptr};
    uint32_t n_rows_more[2] = {0, 0}, out_stride_more[2] = {0, 0};
    void *scratch = nullptr;
    int *status = nullptr;  // the context's device status word
    bool pdl = false;
};
// The scratch opens with the work area of the GEMM's column split: tickets (zero between launches), then one block of
// partial results per work item; the activation tiles follow.
constexpr size_t kGemmTicketBytes = 8192;
constexpr uint32_t kGemmSplitMaxItems = 160;
constexpr size_t kGemmSplitBytes = kGemmTicketBytes + (size_t)kGemmSplitMaxItems * 128 * 128 * sizeof(float);
int32_t ensure_gemm_scratch(yule_cuda_ctx *ctx, size_t bytes);
// Adds a buffer to the set the runner frees when it is destroyed (runner.cu).
void runner_adopt_buffer(yule_cuda_runner *r, yule_buffer h);
bool qgemm_supported(uint32_t type, uint32_t n_cols, uint32_t n_tokens);
size_t qgemm_scratch_bytes(uint32_t n_tokens, uint32_t n_cols);
cudaError_t launch_qgemm(const QGemm &g, int sm_count, cudaStream_t s, uint64_t *launches);
// The two halves of launch_qgemm, for matrices that share their activations (Q/K/V, gate/up):
// one re-layout, then one GEMM per matrix with the same n_tokens, n_cols and scratch.
cudaError_t launch_qgemm_xprep(const QGemm &g, cudaStream_t s, uint64_t *launches);
cudaError_t launch_qgemm_mm(const QGemm &g, int sm_count, cudaStream_t s, uint64_t *launches);

// Q4_K tensor-pipe matvec with the neighbouring ops folded in (qmv_q4k_mma.cu).
struct Q4kFused {
    const uint8_t *w[3] = {nullptr, nullptr, nullptr};  // up to three matrices sharing x
    float *out[3] = {nullptr, nullptr, nullptr};
    uint32_t rows[3] = {0, 0, 0};
    uint32_t out_stride[3] = {0, 0, 0};
    uint32_t n_seg = 1;
    const float *x = nullptr;  // [batch][x_stride]
    uint32_t x_stride = 0, n_cols = 0, batch = 1;
    const float *norm_w = nullptr;    // RMSNorm prologue on x when set
    float eps = 0.f;
    const float *residual = nullptr;  // out[0] += residual when set
    bool swiglu_pair = false;         // w[0], w[1] = gate, up → out[0] = SiLU(gate)·up
    bool q5 = false;                  // the matrices are Q5_K (176-byte super-blocks), 16-byte aligned
    bool pdl = false;                 // programmatic dependent launch
    bool late_wait = false;           // with pdl: inputs do not come from the previous kernel; only the stores wait for it
    const void *next_w[2] = {nullptr, nullptr};  // weights of the kernel(s) that follow: prefetched into L2
    uint64_t next_bytes[2] = {0, 0};
    TpFuse tp;                        // pushes out[0] to the peers / waits for a gathered x
    int *status = nullptr;            // device status word for the kernel's own bounded waits, or null
    long long wait_cycles = kDefaultWaitCycles;
};
bool q4k_mma_supported(uint32_t n_cols, uint32_t batch);
// Routes to the shared-memory-ring kernel (qmv_q4k_ring.cu) when it takes the case, else to the
// register-streaming kernel of qmv_q4k_mma.cu.
cudaError_t launch_q4k_mma(const Q4kFused &f, int sm_count, cudaStream_t s, uint64_t *launches);
bool q4k_ring_supported(const Q4kFused &f);
cudaError_t launch_q4k_ring(const Q4kFused &f, int sm_count, cudaStream_t s, uint64_t *launches);

// Q6_K tensor-pipe matvec over the row-planar device copy of a tensor (qmv_q6k_ring.cu).
struct Q6kPlanar {
    const uint8_t *planar = nullptr;  // per row: ql | qh | scales | d of all its blocks, built by launch_q6k_repack
    float *out = nullptr;
    uint32_t n_rows = 0, n_cols = 0;
    const float *x = nullptr;
    const float *norm_w = nullptr;    // RMSNorm prologue on x when set
    float eps = 0.f;
    const float *residual = nullptr;  // out += residual when set
    bool pdl = false;
    bool late_wait = false;           // with pdl: inputs do not come from the previous kernel; only the stores wait for it
    const void *next_w[2] = {nullptr, nullptr};  // unused by the ring kernel (its successor fetches its own weights early)
    uint64_t next_bytes[2] = {0, 0};
    int *status = nullptr;            // device status word for the kernel's bounded waits, or null
    long long wait_cycles = kDefaultWaitCycles;
};
size_t q6k_planar_bytes(uint64_t n_rows, uint32_t n_cols);
cudaError_t launch_q6k_repack(const uint8_t *raw, uint8_t *planar, uint64_t n_rows, uint32_t n_cols, cudaStream_t s,
                              uint64_t *launches);
bool q6k_mma_supported(uint32_t n_cols);
// Shared-memory-ring kernel (qmv_q6k_ring.cu): the kernel of calls whose inputs do not depend on the previous
// kernel (late wait), which overlap with it on the same SMs.
cudaError_t launch_q6k_mma(const Q6kPlanar &f, int sm_count, cudaStream_t s, uint64_t *launches);
// Register-streaming kernel (qmv_q6k_mma.cu): the kernel of dependent chains.
bool q6k_stream_supported(uint32_t n_cols);
cudaError_t launch_q6k_stream(const Q6kPlanar &f, int sm_count, cudaStream_t s, uint64_t *launches);

// Tensor parallelism (tp.cu).
struct NcclId {
    char internal[128];
};
cudaError_t tp_all_gather_inplace(yule_cuda_ctx *ctx, float *buf, size_t count_per_rank);
void tp_destroy(yule_cuda_ctx *ctx);
// Peer-memory exchange: the same all-gather as stores into every peer's mapped buffer plus epoch flags.
int32_t tp_setup_exchange(yule_cuda_ctx *ctx, size_t n_floats, float **out_base);
bool tp_has_exchange(const yule_cuda_ctx *ctx);
int32_t tp_release_exchange(yule_cuda_ctx *ctx);  // collective over the ranks; called when a tensor-parallel runner is destroyed
// Fill the producer / consumer half of a TpFuse for exchange `index` of a gathered vector whose pair buffer
// starts at pair_offset_floats inside the exchange region (2 floats per element, rank r's slice at element
// r·per_rank).
void tp_fuse_push(const yule_cuda_ctx *ctx, size_t pair_offset_floats, uint32_t per_rank, const uint32_t *tick,
                  uint32_t epochs_per_tick, uint32_t index, TpFuse *f);
void tp_fuse_wait(const yule_cuda_ctx *ctx, size_t pair_offset_floats, const uint32_t *tick, uint32_t epochs_per_tick,
                  uint32_t index, TpFuse *f);
// n_rows > 1: the buffer is a matrix [n_rows][row_stride] (floats) and each rank owns a column block of every row.
cudaError_t tp_exchange(yule_cuda_ctx *ctx, size_t buf_offset_floats, uint32_t per_rank, uint32_t slot,
                        const uint32_t *tick, uint32_t epochs_per_tick, uint32_t epoch_index, bool pdl, uint64_t *launches,
                        uint32_t n_rows = 1, size_t row_stride = 0);

// Launch helper shared by every kernel: optional programmatic-dependent-launch attribute.
template <typename... KArgs, typename... Args>
inline cudaError_t launch_kernel(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t s,
                                 bool pdl, Args... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = s;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = pdl ? 1 : 0;
    return cudaLaunchKernelEx(&cfg, kernel, KArgs(args)...);
}

cudaError_t launch_dequantize(const uint8_t *w, uint32_t type, uint64_t n_blocks, float *out,
                              cudaStream_t s, uint64_t *launches);
// Row `*token_ptr` (device) or `token` (when token_ptr is null) of a [vocab][dim] table.
cudaError_t launch_embed_gather(const uint8_t *table, uint32_t type, uint32_t dim, uint32_t token,
                                const uint32_t *token_ptr, float *out, cudaStream_t s,
                                uint64_t *launches, bool pdl = false);

cudaError_t launch_embed_gather_batch(const uint8_t *table, uint32_t type, uint32_t dim, const uint32_t *tokens,
                                      uint32_t n_tokens, float *out, cudaStream_t s, uint64_t *launches);
cudaError_t launch_rope_kv_write_batch(float *q, const float *k, const float *v, float *k_cache, float *v_cache,
                                       const float *cos_table, const float *sin_table, uint32_t pos0, uint32_t n_tokens,
                                       uint32_t head_dim, uint32_t n_heads, uint32_t n_kv_heads, cudaStream_t s,
                                       uint64_t *launches, const uint32_t *row_pos = nullptr, size_t cache_stride = 0);
// Batched decode: greedy pick per row of [batch][n] logits (ties to the highest index) into tokens[b] and
// history[b * history_stride + step[0]]; then every position and the step counter move on by one.
cudaError_t launch_argmax_rows(const float *v, uint32_t n, uint32_t batch, uint32_t *tokens, uint32_t *pos, uint32_t *step,
                               uint32_t *history, uint32_t history_stride, cudaStream_t s, uint64_t *launches);
cudaError_t launch_advance_rows(uint32_t *pos, uint32_t *step, uint32_t batch, cudaStream_t s, uint64_t *launches);

cudaError_t launch_matvec_f32(const float *a, const float *b, float *out, uint32_t m, uint32_t k,
                              cudaStream_t s, uint64_t *launches);
cudaError_t launch_softmax(const float *in, float *out, uint32_t n, cudaStream_t s, uint64_t *launches);
// Mixture-of-experts router: softmax of the n_exp logits in `probs` (in place), the n_used most probable experts and
// their renormalised weights.  out[i] += (*w) · x[i] with the weight read on the device.
cudaError_t launch_moe_route(float *probs, uint32_t n_exp, uint32_t n_used, uint32_t *sel, float *w, cudaStream_t s, uint64_t *launches);
cudaError_t launch_axpy_dev(const float *w, const float *x, float *out, uint32_t n, cudaStream_t s, uint64_t *launches);
// `rows` contiguous rows of n elements, one CTA each.
cudaError_t launch_rms_norm_rows(const float *in, const float *w, float *out, uint32_t n, uint32_t rows, float eps, cudaStream_t s,
                                 uint64_t *launches);
cudaError_t launch_rms_norm(const float *in, const float *w, float *out, uint32_t n, float eps,
                            cudaStream_t s, uint64_t *launches, bool pdl = false);
// cos/sin hold head_dim/2 entries for this position (host-computed), passed by value.
struct RopeAngles {
    float cos[128];
    float sin[128];
};
cudaError_t launch_rope_angles(float *q, float *k, uint32_t head_dim, uint32_t n_heads_q,
                               uint32_t n_heads_k, const RopeAngles &ang, cudaStream_t s,
                               uint64_t *launches);
cudaError_t launch_silu_mul(const float *gate, const float *up, float *out, uint32_t n, cudaStream_t s,
                            uint64_t *launches, bool pdl = false);
cudaError_t launch_add(const float *a, const float *b, float *out, uint32_t n, cudaStream_t s,
                       uint64_t *launches);
cudaError_t launch_attn_score(const float *q, const float *k_cache, float *scores, uint32_t hd,
                              uint32_t seq_len, uint32_t head_offset, uint32_t kv_offset,
                              uint32_t kv_stride, cudaStream_t s, uint64_t *launches);
cudaError_t launch_attn_value(const float *w, const float *v_cache, float *out, uint32_t hd,
                              uint32_t seq_len, uint32_t kv_offset, uint32_t kv_stride,
                              uint32_t out_offset, cudaStream_t s, uint64_t *launches);
// seq_len_ptr (device, value = position; attends to position+1 entries) overrides seq_len when set.
cudaError_t launch_multihead_attention(const float *q, const float *k_cache, const float *v_cache,
                                       float *out, uint32_t hd, uint32_t seq_len,
                                       const uint32_t *pos_ptr, uint32_t max_seq_len, uint32_t n_heads,
                                       uint32_t n_kv_heads, uint32_t kv_stride, cudaStream_t s,
                                       uint64_t *launches, bool pdl = false, uint32_t window = 0, float softcap = 0.f);
// Element-wise pieces of the architecture variants (glue.cu): out[i] = f(a[i], b[i], v); b may be null for the
// one-input ops.
enum { kElemAddScalar = 0, kElemScale = 1, kElemSoftcap = 2, kElemGeluMul = 3, kElemAddVec = 4 };
cudaError_t launch_elementwise(int op, const float *a, const float *b, float *out, uint32_t n, float v, cudaStream_t s,
                               uint64_t *launches, bool pdl = false);
// Split-KV decode attention, optionally fused with RoPE and the KV-cache append (attention.cu).
struct AttnDecode {
    const float *q = nullptr;       // [n_heads][hd]
    const float *k_new = nullptr;   // fused mode: un-rotated K row of the current token, else null
    const float *v_new = nullptr;
    float *k_cache = nullptr, *v_cache = nullptr;
    const float *cos_table = nullptr, *sin_table = nullptr;  // fused mode: RoPE table [max_seq][hd/2]
    const uint32_t *pos_ptr = nullptr;  // position in device memory (graph replay), else seq_len is used
    uint32_t seq_len = 0;
    float *out = nullptr;
    float *scratch = nullptr;       // attn_scratch_floats(n_heads, n_splits, hd) floats
    uint32_t *tickets = nullptr;    // n_heads words, zero before the first launch
    uint32_t hd = 0, n_heads = 0, n_kv_heads = 0, kv_stride = 0, n_splits = 1, max_seq_len = 0;
    uint32_t min_chunk = 0;  // fewest positions a split is worth (0: one per thread of the CTA)
    bool pdl = false;
    // Prefill: n_tokens > 1 runs one query per blockIdx.z; query z sits at position seq_len - 1 + z,
    // its q and out rows are q_stride / out_stride floats apart (grouped-query kernel, not fused).
    uint32_t n_tokens = 1, q_stride = 0, out_stride = 0;
    // Batched decode: query z is the current token of sequence z — its position is pos_ptr[z] and its caches lie
    // z * kv_batch_stride floats after k_cache / v_cache (grouped-query kernel, not fused).
    bool pos_per_query = false;
    size_t kv_batch_stride = 0;
    TpFuse tp;               // grouped-query kernel: tensor parallelism, output pushed as (value, epoch) pairs
    uint32_t window = 0;     // sliding window (yule-infer/src/model_runner.rs:688-696): positions < pos − window are not attended; 0 = none
    float softcap = 0.f;     // attention logit softcap (:716-721): score = cap · tanh(score / cap); 0 = none
    bool gqa = false;        // grouped-query kernel: one CTA per (KV head, split); n_splits from attn_gqa_pick_splits
};
bool attn_gqa_supported(uint32_t hd, uint32_t n_heads, uint32_t n_kv_heads);
uint32_t attn_gqa_pick_splits(uint32_t n_kv_heads, uint32_t max_seq_len, int sm_count);
size_t attn_scratch_floats(uint32_t n_heads, uint32_t n_splits, uint32_t hd);
uint32_t attn_pick_splits(uint32_t n_heads, uint32_t seq_len_hint, int sm_count);
bool attn_decode_supported(uint32_t hd);
cudaError_t launch_attn_decode(const AttnDecode &a, cudaStream_t s, uint64_t *launches);

// Runner kernels that read the position from device memory (graph-replayable).
cudaError_t launch_rope_kv_write(float *q, const float *k_tmp, const float *v_tmp, float *k_cache,
                                 float *v_cache, const float *cos_table, const float *sin_table,
                                 const uint32_t *pos_ptr, uint32_t head_dim, uint32_t n_heads,
                                 uint32_t n_kv_heads, cudaStream_t s, uint64_t *launches, bool pdl = false);
// Greedy pick (ties to the highest index) into state[0]; when history is set also records it at
// history[state[1]] and advances state[1].
cudaError_t launch_argmax(const float *v, uint32_t n, uint32_t *state, uint32_t *history, cudaStream_t s,
                          uint64_t *launches, bool pdl = false);
cudaError_t launch_fill_bytes(void *p, size_t n, int value, cudaStream_t s, uint64_t *launches);

// Token sampler on the device (sampler.cu; yule-infer/src/sampler.rs:17-136).
struct SampleArgs {
    const float *logits = nullptr;
    uint32_t n = 0;
    float temperature = 0.7f, top_p = 0.9f, min_p = 0.05f, repetition_penalty = 1.1f;  // SamplingParams::default
    uint32_t top_k = 40;
    const uint32_t *previous = nullptr;  // tokens seen so far, device memory
    uint32_t n_previous = 0;
    float r = 0.f;                       // uniform random value in [0, 1)
    float *scratch = nullptr;            // 2 * n floats
    uint32_t *out_token = nullptr;       // device word that receives the pick
    uint32_t *append_to = nullptr;       // optional: the pick also goes to append_to[n_previous]
    uint32_t *feed_state = nullptr;      // optional: the pick also goes to feed_state[0]
};
cudaError_t launch_sample(const SampleArgs &a, cudaStream_t s, uint64_t *launches);
int32_t ensure_sampler_scratch(yule_cuda_ctx *ctx, size_t n_floats);

// Tiled 2-D tensor map (qgemm_tc.cu); `out` points to a CUtensorMap (128 bytes, 64-byte aligned).
cudaError_t encode_tensor_map_2d(const void *base, uint32_t elem_bytes, uint64_t inner, uint64_t n_rows, uint64_t row_stride_bytes,
                                 uint32_t box_inner, uint32_t box_rows, void *out);

cudaError_t cached_tensor_map_2d(const void *base, uint32_t elem_bytes, uint64_t inner, uint64_t n_rows, uint64_t row_stride_bytes,
                                 uint32_t box_inner, uint32_t box_rows, void *out);

// Persistent decode kernel (decode_mega.cu): the whole token step of a dense Llama-family model in one cooperative
// launch.  Covers: one GPU, no architecture variant, Q4_K attn_q/k/v and ffn_gate/up, Q4_K or Q6_K (row-planar copy)
// attn_output / ffn_down / output matrix, grouped-query head shapes that were instantiated.
struct MegaTensor {
    const uint8_t *ptr = nullptr;  // raw Q4_K rows, or the row-planar copy of a Q6_K tensor
    uint32_t type = 0;
};
struct MegaLayer {
    MegaTensor q, k, v, o, gate, up, down;
    const float *attn_norm = nullptr, *ffn_norm = nullptr;
    float *k_cache = nullptr, *v_cache = nullptr;
};
struct MegaModel {
    uint32_t dim = 0, head_dim = 0, n_heads = 0, n_kv_heads = 0, ff_dim = 0, vocab = 0, n_layers = 0, max_seq_len = 0;
    float eps = 0.f;
    const uint8_t *embd = nullptr;  // token_embd, any block format
    uint32_t embd_type = 0;
    MegaTensor output;
    const float *output_norm = nullptr;
    std::vector<MegaLayer> layers;
    const float *rope_cos = nullptr, *rope_sin = nullptr;
    uint32_t *state = nullptr, *history = nullptr;  // {token, position, tokens so far}; picks by position
    float *logits = nullptr;
    int *status = nullptr;
    long long wait_cycles = kDefaultWaitCycles;
    int sm_count = 0;
};
struct MegaHandle;
// Bytes of zero-filled device memory the kernel needs for this model, or 0 with the reason when it does not cover it.
size_t mega_workspace_bytes(const MegaModel &m, std::string *why);
cudaError_t mega_setup(const MegaModel &m, void *workspace, cudaStream_t s, MegaHandle **out);
void mega_set_cooperative(MegaHandle *h, bool on);
void mega_set_wait_cycles(MegaHandle *h, long long cycles);
cudaError_t mega_launch(const MegaHandle *h, cudaStream_t s, uint64_t *launches);
cudaError_t mega_launch_selftest(const MegaHandle *h, long long budget, cudaStream_t s, uint64_t *launches);
void mega_destroy(MegaHandle *h);

}  // namespace yule
