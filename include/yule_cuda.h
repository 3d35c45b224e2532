/*
 * yule_cuda.h — C ABI of libyule_cuda.so, a B200 (sm_100a) compute backend for Yule.
 *
 * The library is the device side of Yule's `ComputeBackend` trait
 * (yule-gpu/src/lib.rs:21-132).  A Rust shim maps each trait method onto the
 * entry point of the same name below; `BufferHandle(u64)` (lib.rs:135) crosses
 * unchanged as `yule_buffer`, `DType` crosses as its GGUF type id
 * (yule-core/src/dtype.rs:13-58, :155-190), and every failure comes back as a
 * nonzero status whose text (`yule_cuda_last_error`) the shim wraps in
 * `YuleError::Gpu(String)` (yule-core/src/error.rs:44).
 *
 * Conventions
 *   - Every entry point returns int32 status; 0 is success.  No exception or
 *     abort crosses the boundary.
 *   - All entry points are thread-safe (`ComputeBackend: Send + Sync`, every
 *     method takes `&self`).  Work is enqueued on one stream per context, so
 *     ordering between calls is call order; only copy_from_device,
 *     synchronize, destroy and the runner's logits read-back block the host.
 *   - Buffers are owned by the context, zero-filled on allocation
 *     (yule-gpu/src/cuda/memory.rs:26) and addressed only by handle; sizes and
 *     offsets are checked against the allocation, a bad handle is an error and
 *     never undefined behaviour.
 *   - Quantized weights are raw GGUF tensor bytes, unmodified
 *     (yule-infer/src/gpu_runner.rs:176-181).
 *   - There is no CPU fallback: without a CUDA device `yule_cuda_create` fails.
 */
#ifndef YULE_CUDA_H
#define YULE_CUDA_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef struct yule_cuda_ctx yule_cuda_ctx;
typedef struct yule_cuda_runner yule_cuda_runner;
typedef uint64_t yule_buffer; /* yule-gpu/src/lib.rs:135 BufferHandle(pub u64) */

/* Status codes (nonzero ⇒ YuleError::Gpu(last_error)). */
enum {
    YULE_OK = 0,
    YULE_ERR_INVALID_ARGUMENT = 1,
    YULE_ERR_UNKNOWN_BUFFER = 2,   /* cuda/memory.rs "unknown buffer" */
    YULE_ERR_OUT_OF_BOUNDS = 3,
    YULE_ERR_UNSUPPORTED_DTYPE = 4, /* cuda/mod.rs:303-307 */
    YULE_ERR_CUDA = 5,
    YULE_ERR_OUT_OF_MEMORY = 6,
    YULE_ERR_DEVICE_STATUS = 7,    /* a bounded device-side wait gave up */
    YULE_ERR_CONTEXT_LENGTH = 8,   /* gpu_runner.rs:305-307 "context length exceeded" */
    YULE_ERR_MISSING_TENSOR = 9,
    YULE_ERR_PARSE = 10            /* a model file was rejected (yule-core/src/error.rs: InvalidMagic, UnsupportedVersion,
                                      Parse, InvalidTensorShape, TensorOutOfBounds); the message names which */
};

/* GGUF type ids accepted where a dtype is asked for (dtype.rs:155-190).  Q4_0, Q8_0, Q4_K and
 * Q6_K have tuned matvec and GEMM kernels; the other block formats (which Yule's own GPU backends
 * refuse, yule-gpu/src/cuda/mod.rs:303-307) dequantise bit-exactly and run through slower matvecs. */
enum {
    YULE_DTYPE_F32 = 0,
    YULE_DTYPE_F16 = 1,
    YULE_DTYPE_Q4_0 = 2,
    YULE_DTYPE_Q4_1 = 3,
    YULE_DTYPE_Q5_0 = 6,
    YULE_DTYPE_Q5_1 = 7,
    YULE_DTYPE_Q8_0 = 8,
    YULE_DTYPE_Q8_1 = 9,
    YULE_DTYPE_Q2_K = 10,
    YULE_DTYPE_Q3_K = 11,
    YULE_DTYPE_Q4_K = 12,
    YULE_DTYPE_Q5_K = 13,
    YULE_DTYPE_Q6_K = 14
};

/* Text of the calling thread's most recent failure (UTF-8, NUL-terminated,
 * valid until that thread's next failing call). */
const char *yule_cuda_last_error(void);

/* ── lifecycle: CudaBackend::is_available / new / Drop / device_info
 *    (yule-gpu/src/cuda/mod.rs:20-58, cuda/device.rs:5-77) ─────────────── */
int32_t yule_cuda_is_available(void); /* 1 when a CUDA device answers, else 0 */
int32_t yule_cuda_create(int32_t device_ordinal, yule_cuda_ctx **out_ctx);
int32_t yule_cuda_destroy(yule_cuda_ctx *ctx);
int32_t yule_cuda_device_info(yule_cuda_ctx *ctx, char *name_buf, size_t name_cap,
                              uint64_t *memory_bytes, uint32_t *compute_units);

/* ── memory: ComputeBackend::allocate / free / copy_* / synchronize
 *    (lib.rs:24-25, :69-80; cuda/memory.rs:10-154) ─────────────────────── */
int32_t yule_cuda_allocate(yule_cuda_ctx *ctx, size_t size_bytes, yule_buffer *out_handle);
int32_t yule_cuda_free(yule_cuda_ctx *ctx, yule_buffer handle);
/* Copies min(len, allocation) bytes like the reference's slice semantics. */
int32_t yule_cuda_copy_to_device(yule_cuda_ctx *ctx, const void *data, size_t len, yule_buffer dst);
int32_t yule_cuda_copy_from_device(yule_cuda_ctx *ctx, yule_buffer src, void *data, size_t len);
int32_t yule_cuda_copy_buffer(yule_cuda_ctx *ctx, yule_buffer src, yule_buffer dst, size_t size);
int32_t yule_cuda_copy_buffer_offset(yule_cuda_ctx *ctx, yule_buffer src, yule_buffer dst,
                                     size_t src_offset, size_t dst_offset, size_t size);
int32_t yule_cuda_synchronize(yule_cuda_ctx *ctx);
/* Budget, in SM clock cycles, of every bounded device-side wait launched from this
 * context afterwards (peer pairs and flags of the tensor-parallel exchange, the
 * shared-memory ring of the matvec, the GEMM pipeline).  A wait that runs out
 * writes the context's status word; every later wait of the same context returns
 * at once, and the next synchronize / runner call returns YULE_ERR_DEVICE_STATUS.
 * 0 restores the default (about one second).  No counterpart in the reference,
 * which has no device-side waits (cuda/mod.rs synchronises on the host). */
int32_t yule_cuda_set_wait_budget(yule_cuda_ctx *ctx, uint64_t cycles);
/* Self-test of the give-up path: runs one kernel whose bounded wait cannot be
 * satisfied (which = 0: the Q4_K matvec polling for a gathered vector's pairs;
 * 1: the exchange kernel polling for a peer's flag; the "peer" is memory of this
 * GPU that nothing writes), with a budget of budget_cycles (0: the context's).
 * The kernel returns normally; the call returns YULE_ERR_DEVICE_STATUS, which is
 * the expected result, and the context stays usable.  No counterpart in the
 * reference. */
int32_t yule_cuda_selftest_bounded_wait(yule_cuda_ctx *ctx, uint32_t which, uint64_t budget_cycles);

/* ── compute: the trait's numeric methods with the semantics of the
 *    reference's own GPU backends (cuda/mod.rs:95-328, vulkan/mod.rs) ───── */

/* lib.rs:26 matmul — kernels/cuda/matmul.cu:4-32: out[row] = dot(A[row,0..k], b)
 * for row < m; `n` is carried but unused, as in the reference kernel. */
int32_t yule_cuda_matmul(yule_cuda_ctx *ctx, yule_buffer a, yule_buffer b, yule_buffer out,
                         uint32_t m, uint32_t n, uint32_t k);
/* lib.rs:35 softmax — kernels/cuda/softmax.cu:3-45 (max-subtracted). */
int32_t yule_cuda_softmax(yule_cuda_ctx *ctx, yule_buffer input, yule_buffer output, uint32_t size);
/* lib.rs:36 rms_norm — kernels/cuda/rms_norm.cu:4-36: x * rsqrt(mean(x^2)+eps) * w. */
int32_t yule_cuda_rms_norm(yule_cuda_ctx *ctx, yule_buffer input, yule_buffer weight,
                           yule_buffer output, uint32_t size, float eps);
/* lib.rs:44 rope — kernels/cuda/rope.cu:3-49: interleaved pairs (2i,2i+1) of
 * every Q and K head rotated in place by pos * base^(-2i/head_dim). */
int32_t yule_cuda_rope(yule_cuda_ctx *ctx, yule_buffer q, yule_buffer k, uint32_t pos,
                       uint32_t head_dim, float freq_base, uint32_t n_heads_q, uint32_t n_heads_k);
/* lib.rs:54 silu — cuda/mod.rs:173-188: output = SiLU(input) * output. */
int32_t yule_cuda_silu(yule_cuda_ctx *ctx, yule_buffer input, yule_buffer output, uint32_t size);
/* lib.rs:55 element_mul — cuda/mod.rs:190-208: output = SiLU(a) * b. */
int32_t yule_cuda_element_mul(yule_cuda_ctx *ctx, yule_buffer a, yule_buffer b, yule_buffer output,
                              uint32_t size);
/* lib.rs:62 add — kernels/cuda/add.cu:2-11. */
int32_t yule_cuda_add(yule_cuda_ctx *ctx, yule_buffer a, yule_buffer b, yule_buffer output,
                      uint32_t size);
/* lib.rs:83 attn_score — kernels/cuda/attn_score.cu:3-33: scores[t] =
 * dot(q[head_offset..+hd], K[t*kv_stride+kv_offset..]) / sqrt(hd); offsets and
 * strides count floats. */
int32_t yule_cuda_attn_score(yule_cuda_ctx *ctx, yule_buffer q, yule_buffer k_cache,
                             yule_buffer scores, uint32_t head_dim, uint32_t seq_len,
                             uint32_t head_offset, uint32_t kv_offset, uint32_t kv_stride);
/* lib.rs:100 attn_value — kernels/cuda/attn_value.cu:3-33: out[out_offset+d] =
 * sum_t weights[t] * V[t*kv_stride+kv_offset+d]. */
int32_t yule_cuda_attn_value(yule_cuda_ctx *ctx, yule_buffer weights, yule_buffer v_cache,
                             yule_buffer output, uint32_t head_dim, uint32_t seq_len,
                             uint32_t kv_offset, uint32_t kv_stride, uint32_t out_offset);
/* lib.rs:119 quantized_matmul — cuda/mod.rs:289-328 + kernels/cuda/qmv_*.cu:
 * out[row] = sum over blocks of dot(dequant(W[row, block]), x[block]).
 * gguf_type is any block format of the YULE_DTYPE_* list above: the reference's
 * GPU backends take 2 (Q4_0), 8 (Q8_0), 12 (Q4_K) and 14 (Q6_K) and reject the
 * rest (cuda/mod.rs:303-307); here Q4_1, Q5_0, Q5_1, Q8_1, Q2_K, Q3_K and Q5_K
 * are accepted too.  n_cols must be a multiple of the format's block size. */
int32_t yule_cuda_quantized_matmul(yule_cuda_ctx *ctx, yule_buffer weights, yule_buffer input,
                                   yule_buffer output, uint32_t n_rows, uint32_t n_cols,
                                   uint32_t gguf_type);

/* ── sampling: Sampler::sample_with_history (yule-infer/src/sampler.rs:17-136) on the device ── */
typedef struct yule_sampling_params { /* SamplingParams, yule-infer/src/lib.rs:65-84 */
    float temperature;        /* <= 0 or 1: no scaling (sampler.rs:41) */
    float top_p;              /* >= 1: off */
    uint32_t top_k;           /* 0 or >= n: off; keeps the probabilities >= sorted[k] of the descending order */
    float repetition_penalty; /* 1: off; applied once per earlier occurrence of a token */
    float min_p;              /* <= 0: off */
} yule_sampling_params;
/* One pick from `n` logits held in a device buffer.  previous_tokens (n_previous words, device buffer; ignored
 * when n_previous is 0) is the token list the repetition penalty looks at.  random_value in [0, 1) takes the
 * place of the reference's CSPRNG draw (sampler.rs:212-220), so a call is reproducible.  The steps and their
 * order are the reference's; sums are formed as trees instead of left to right, which can move a pick only when
 * random_value lies within rounding distance of a boundary of the cumulative distribution. */
int32_t yule_cuda_sample(yule_cuda_ctx *ctx, yule_buffer logits, uint32_t n, const yule_sampling_params *params,
                         yule_buffer previous_tokens, uint32_t n_previous, float random_value, uint32_t *out_token);

/* ── additive entry points (not trait methods; each equals a sequence of
 *    trait calls, so the plain trait stays sufficient) ──────────────────── */

/* `batch` activation vectors against one weight read: input is
 * [batch][x_stride] floats, output [batch][out_stride] floats.  Same per-row
 * arithmetic as quantized_matmul.  Small batches go through the matvec kernels
 * four vectors at a time (Q4_K, Q6_K, Q8_0, Q4_0: four vectors share the
 * tensor-core instructions of one, so a pass costs about one vector's time);
 * from 16 vectors of Q4_K (32 on matrices of up to 8M weights), 64 of Q5_K, or
 * 32 of the other block formats (n_cols a multiple of 256), the tcgen05 GEMM
 * takes one pass over the weights.
 * The GEMM keeps its activation tiles in a scratch owned by the context, grown
 * on demand; growing is not possible while a graph is being captured, so run
 * one call of the largest batch before yule_cuda_graph_begin. */
int32_t yule_cuda_quantized_matmul_batched(yule_cuda_ctx *ctx, yule_buffer weights,
                                           yule_buffer input, yule_buffer output, uint32_t n_rows,
                                           uint32_t n_cols, uint32_t gguf_type, uint32_t batch,
                                           uint32_t x_stride, uint32_t out_stride);
/* Same as quantized_matmul but the weight tensor starts `weight_offset` bytes
 * into its buffer (a multiple of 2; 16 for Q4_K) — what a row-sharded rank or a
 * ring of tensor copies in one allocation needs. */
int32_t yule_cuda_quantized_matmul_at(yule_cuda_ctx *ctx, yule_buffer weights, size_t weight_offset,
                                      yule_buffer input, yule_buffer output, uint32_t n_rows,
                                      uint32_t n_cols, uint32_t gguf_type);
/* Optional, once per weight tensor: lets the library keep a device-side copy of the tensor in the
 * layout its fastest kernel wants (today: Q6_K regrouped into 16-byte-aligned planes, same byte
 * count).  Later quantized_matmul calls on the same handle, type and shape use it.  Writing to the
 * buffer drops the copy.  A no-op for formats that need none.  Results are unchanged. */
int32_t yule_cuda_prepare_weights(yule_cuda_ctx *ctx, yule_buffer weights, uint32_t gguf_type,
                                  uint32_t n_rows, uint32_t n_cols);
/* dequant_block over a whole tensor (yule-core/src/dequant.rs:1232): n_blocks
 * raw blocks → n_blocks*block_size floats.  Results are bit-identical to
 * yule-core's scalar dequantisers. */
int32_t yule_cuda_dequantize(yule_cuda_ctx *ctx, yule_buffer weights, uint32_t gguf_type,
                             uint64_t n_blocks, yule_buffer out_f32);
/* The MultiheadAttn dispatch of the GPU runner (gpu_runner.rs:477-499,
 * shaders/multihead_attn.comp): for every head h, kv head h/(n_heads/n_kv_heads):
 * scores → softmax → weighted V sum over positions [0, seq_len). */
int32_t yule_cuda_multihead_attention(yule_cuda_ctx *ctx, yule_buffer q, yule_buffer k_cache,
                                      yule_buffer v_cache, yule_buffer out, uint32_t head_dim,
                                      uint32_t seq_len, uint32_t n_heads, uint32_t n_kv_heads,
                                      uint32_t kv_stride);
/* multihead_attention for callers that must not allocate device memory when they call: a host that
 * sealed its process before inference (Yule's sandbox is applied first, and the driver requests
 * behind cudaMalloc may then be denied), an embedder whose device-memory budget is already handed
 * out, or a decode loop that may not wait on the allocator's lock.  This entry point has no
 * counterpart in the reference.  Same arguments and results as yule_cuda_multihead_attention, but
 * the scratch for the position splits is a fixed array inside the library image (2.02 MiB of
 * partial sums plus 512 bytes of counters, held by every GPU that loads the library until the
 * process exits) instead of a buffer the context grows on demand; neither this call nor anything
 * it calls uses cudaMalloc / cudaFree.
 *   Limits: at most 128 heads, head_dim <= 256 with 256 % (head_dim / 4) == 0, kv_stride a multiple
 *   of 4; anything larger is refused with YULE_ERR_INVALID_ARGUMENT and a message naming the limit.
 *   First use on a device looks up the array's device address; make that first call before you
 *   open any stream capture.
 *   All calls share the one array: two calls whose kernels overlap on the GPU (different contexts
 *   or streams on the same device) race on it — issue them one after the other. */
int32_t yule_cuda_multihead_attention_static(yule_cuda_ctx *ctx, yule_buffer q, yule_buffer k_cache,
                                             yule_buffer v_cache, yule_buffer out, uint32_t head_dim,
                                             uint32_t seq_len, uint32_t n_heads, uint32_t n_kv_heads,
                                             uint32_t kv_stride);
/* Embedding row `token` of a [vocab][dim] table of any supported dtype (F32,
 * F16 or a quantized format) dequantised to `out` — the step the reference GPU
 * runner does on the CPU (gpu_runner.rs:309-343). */
int32_t yule_cuda_embed_gather(yule_cuda_ctx *ctx, yule_buffer table, uint32_t gguf_type,
                               uint32_t dim, uint32_t token, yule_buffer out);

/* Record a sequence of this context's compute/copy_buffer calls once and replay it: between
 * graph_begin and graph_end the calls are captured into a CUDA graph instead of executed (the
 * blocking entry points — copy_from_device, synchronize, free, destroy — must not be called
 * in between).  graph_launch enqueues one replay on the context's stream.  This is the
 * single-submit batching of the reference's Vulkan runner (begin_batch / submit_batch,
 * yule-gpu/src/vulkan/mod.rs:108-174) in CUDA terms. */
int32_t yule_cuda_graph_begin(yule_cuda_ctx *ctx);
int32_t yule_cuda_graph_end(yule_cuda_ctx *ctx, uint32_t *out_graph_id);
int32_t yule_cuda_graph_launch(yule_cuda_ctx *ctx, uint32_t graph_id);
int32_t yule_cuda_graph_destroy(yule_cuda_ctx *ctx, uint32_t graph_id);

/* Stream-ordered timing without any other CUDA binding: record returns an
 * event id on the context's stream; elapsed gives milliseconds between two
 * recorded events after waiting for the second. */
int32_t yule_cuda_event_record(yule_cuda_ctx *ctx, uint32_t *out_event_id);
int32_t yule_cuda_event_elapsed_ms(yule_cuda_ctx *ctx, uint32_t start_id, uint32_t end_id,
                                   float *out_ms);
int32_t yule_cuda_event_reset(yule_cuda_ctx *ctx);
/* Overwrites a context-owned scratch larger than L2 so that the next kernel
 * finds its inputs in HBM, not in cache. */
int32_t yule_cuda_flush_l2(yule_cuda_ctx *ctx);
/* Number of kernels this library has launched on the context so far. */
int32_t yule_cuda_launch_count(yule_cuda_ctx *ctx, uint64_t *out_count);

/* ── tensor parallelism over output rows (no counterpart in the reference, which is single-device):
 *    one process and one context per GPU; rank 0 creates a 128-byte rendezvous id, the caller
 *    carries it to the other ranks, every rank calls tp_init before creating its runner.  A runner
 *    created on such a context expects each matrix to hold only this rank's rows
 *    [rank*n/world, (rank+1)*n/world) (a byte slice of the raw tensor) and all-gathers the
 *    activations over NCCL.  n_heads, n_kv_heads, dim, ff_dim and vocab_size must be multiples of
 *    the world size. ── */
int32_t yule_cuda_tp_unique_id(uint8_t *out_id128);
int32_t yule_cuda_tp_init(yule_cuda_ctx *ctx, uint32_t rank, uint32_t world, const uint8_t *id128);
/* In-place all-gather of fp32 on the context's stream: rank r's count_per_rank floats already sit
 * at offset r*count_per_rank of the buffer; afterwards every rank holds every slice. */
int32_t yule_cuda_tp_all_gather(yule_cuda_ctx *ctx, yule_buffer buffer, size_t count_per_rank);

/* ── forward-pass runner: the `ModelRunner` trait
 *    (yule-infer/src/model_runner.rs:12-17) issued in the op order of
 *    GpuTransformerRunner::forward (yule-infer/src/gpu_runner.rs:296-695) ── */
typedef struct {
    uint32_t dim, n_layers, n_heads, n_kv_heads, head_dim, vocab_size, ff_dim, max_seq_len;
    float norm_eps, rope_freq_base;
    /* 0: one kernel per reference dispatch (RmsNorm, Qmv, Rope, KV copy,
     *    MultiheadAttn, Add, SiluMul), launched one by one.
     * 1: fused kernels replayed from a CUDA graph (same arithmetic per row).
     * 2: as 1, with the token step as ONE persistent kernel where the model allows it (one GPU, the Llama op
     *    sequence, Q4_K attn_q/k/v and ffn_gate/up, Q4_K or Q6_K attn_output / ffn_down / output matrix,
     *    grouped-query head shapes 64 or 128 wide); any other model runs as with 1.
     *    yule_cuda_runner_step_kind tells which one a runner uses. */
    uint32_t fused;
    /* Architecture variants of the dense path, as RunnerConfig derives them from the file
     * (yule-infer/src/model_runner.rs:417-460); all zero = the Llama default.  The reference's GPU runner drops
     * them (gpu_runner.rs implements the Llama path only); its CPU runner is the contract.
     * Optional tensors go with them: "blk.N.attn_{q,k,v}.bias" (F32 / F16; :640-651) and Gemma2's
     * "blk.N.attn_post_norm.weight" / "blk.N.ffn_post_norm.weight" (:764-779, :985-999). */
    uint32_t rotary_dim;         /* partial RoPE: rotated prefix of every head (:430-434); 0 or >= head_dim = all of it */
    uint32_t sliding_window;     /* attention sees positions >= pos - window (:688-696); 0 = none */
    float attn_logit_softcap;    /* score = cap * tanh(score / cap) before the softmax (:716-721); 0 = none */
    float logit_softcap;         /* the same on the final logits (:1027-1032); 0 = none */
    float norm_weight_offset;    /* Gemma: norms use (w + offset), embeddings are scaled by sqrt(dim) (:246-275, :568-574) */
    uint32_t geglu;              /* Gemma: gelu(gate) * up instead of SiLU(gate) * up (:974-978) */
    /* Mixture of experts (:395-397, :813-958): n_experts > 0 replaces the dense FFN of every layer by a router
     * ("blk.N.ffn_gate_inp.weight", [n_experts][dim], F32 / F16 or a block format), a softmax over its logits, the
     * n_experts_used most probable experts (ties: lower index first) with their probabilities renormalised, and the
     * weighted sum of those experts' SwiGLU FFNs.  Expert weights: packed, "blk.N.ffn_{gate,up,down}_exps.weight"
     * (expert e = the e-th of n_experts equal slices), or one tensor per expert, "blk.N.ffn_{gate,up,down}.E.weight".
     * Such a runner works in mode 0 (one kernel per dispatch, the chosen expert indices read back once per layer). */
    uint32_t n_experts, n_experts_used;
} yule_runner_config;

int32_t yule_cuda_runner_create(yule_cuda_ctx *ctx, const yule_runner_config *cfg,
                                yule_cuda_runner **out_runner);
int32_t yule_cuda_runner_destroy(yule_cuda_runner *runner);
/* Register an uploaded tensor under its GGUF name ("token_embd.weight",
 * "blk.%u.attn_q.weight", "output_norm.weight", …; gpu_runner.rs:171-254).
 * Norm weights are F32 or F16; matrices are any block format of the enum above. */
int32_t yule_cuda_runner_set_tensor(yule_cuda_runner *runner, const char *name, yule_buffer handle,
                                    uint32_t gguf_type);
/* ModelRunner::prefill — token-by-token forward (gpu_runner.rs:703-709);
 * logits (vocab_size floats, host memory) of the last token. */
int32_t yule_cuda_runner_prefill(yule_cuda_runner *runner, const uint32_t *tokens, uint32_t n_tokens,
                                 float *logits_out);
/* ModelRunner::decode_step (gpu_runner.rs:711-713). */
int32_t yule_cuda_runner_decode_step(yule_cuda_runner *runner, uint32_t token, float *logits_out);
/* ModelRunner::reset (gpu_runner.rs:715-719). */
int32_t yule_cuda_runner_reset(yule_cuda_runner *runner);
int32_t yule_cuda_runner_position(yule_cuda_runner *runner, uint32_t *out_pos);
/* How this runner executes a token step: 0 one kernel per dispatch, 1 fused kernels in a CUDA graph, 2 one
 * persistent kernel.  Builds the step (weights must be set) so that the answer is final. */
int32_t yule_cuda_runner_step_kind(yule_cuda_runner *runner, uint32_t *out_kind);
/* Self-test of the persistent kernel's bounded waits (step kind 2 only): runs the token kernel once with every
 * consumer expecting epochs that no producer writes, with a budget of budget_cycles (0: the context's).  The
 * kernel returns normally; the call returns YULE_ERR_DEVICE_STATUS, which is the expected result.  Token and
 * position are left as they were; the activations and the KV rows of the current position hold garbage
 * afterwards, so reset the runner before using it again. */
int32_t yule_cuda_runner_selftest_bounded_wait(yule_cuda_runner *runner, uint64_t budget_cycles);
/* Greedy generation with the argmax on the device (ties resolve to the highest
 * index, yule-infer/src/sampler.rs:150-163): feeds `prompt`, then emits
 * n_generate tokens into out_tokens.  Only token ids cross the bus. */
int32_t yule_cuda_runner_generate_greedy(yule_cuda_runner *runner, const uint32_t *prompt,
                                         uint32_t n_prompt, uint32_t n_generate,
                                         uint32_t *out_tokens);
/* Layout of a rank's exchange region under tensor parallelism, in floats: out_offsets[0..3] the gathered
 * attention output / hidden / gate / logits vectors, [4..6] the (value, epoch) pair copies of hidden / gate /
 * attention output, [7] the total.  Host arithmetic only (no device needed).  No counterpart in the reference,
 * which has no multi-device path. */
int32_t yule_cuda_tp_exchange_layout(const yule_runner_config *cfg, uint64_t out_offsets[8]);
/* Batched decode: `batch` independent sequences, one new token each per call, every sequence with its own
 * KV caches and position (all start at 0; reset_batch rewinds them).  Per sequence the result is that of
 * decode_step on a runner of its own (the reference serves one sequence per ModelRunner,
 * yule-infer/src/lib.rs:169-216); across the batch every linear is one GEMM, so the weights are read once
 * per step.  Single GPU, fused = 1, Llama op sequence, n_cols in multiples of 256; the first call fixes the
 * batch size of the runner.  logits_out: [batch][vocab_size] floats or null. */
int32_t yule_cuda_runner_decode_batch(yule_cuda_runner *runner, const uint32_t *tokens, uint32_t batch, float *logits_out);
int32_t yule_cuda_runner_reset_batch(yule_cuda_runner *runner);
/* Greedy generation for a batch, picks made on the device: prompts is [batch][n_prompt] (equal lengths),
 * out_tokens [batch][n_generate]; token g of a sequence is the pick made after its position
 * n_prompt - 1 + g (ties to the highest index, sampler.rs:150-163). */
int32_t yule_cuda_runner_generate_greedy_batch(yule_cuda_runner *runner, const uint32_t *prompts, uint32_t batch,
                                               uint32_t n_prompt, uint32_t n_generate, uint32_t *out_tokens);
/* Sampled generation: as generate_greedy, but every pick after the prompt is made by the device sampler
 * (yule_cuda_sample's arithmetic) over all tokens so far, prompt included (yule-infer/src/lib.rs:194-204), and fed
 * back without leaving the device.  The random values come from a counter-based generator seeded with `seed`
 * (pick g uses value g of the stream), so equal seeds give equal streams. */
int32_t yule_cuda_runner_generate_sampled(yule_cuda_runner *runner, const uint32_t *prompt, uint32_t n_prompt,
                                          uint32_t n_generate, const yule_sampling_params *params, uint64_t seed,
                                          uint32_t *out_tokens);
/* The random value pick g of a sampled generation uses: a function of (seed, g) only, in [0, 1). */
float yule_cuda_sampling_random_value(uint64_t seed, uint32_t index);
/* Device buffers of the runner for layer-by-layer checks: which = 0 hidden,
 * 1 K cache of `layer`, 2 V cache of `layer`, 3 logits. */
int32_t yule_cuda_runner_buffer(yule_cuda_runner *runner, uint32_t which, uint32_t layer,
                                yule_buffer *out_handle);

/* ── GGUF v3 files (yule-core/src/gguf.rs:271-431, yule-infer/src/weight_loader.rs:19-38,
 *    yule-infer/src/gpu_runner.rs:171-254) ─────────────────────────────────
 * The reader needs no GPU.  It applies the reference's checks: magic, version 3
 * only, at most 100 000 tensors and key-value pairs, strings up to 1 MiB, arrays
 * up to 10 M elements, at most 8 dimensions, shape overflow, every tensor inside
 * the file, no two tensors overlapping; the data section starts at the next
 * multiple of general.alignment (32 when absent).  Any violation is
 * YULE_ERR_PARSE with a message. */
typedef struct yule_gguf yule_gguf;

typedef struct yule_gguf_tensor_info {
    const char *name;       /* owned by the yule_gguf */
    uint32_t n_dims;
    uint64_t shape[8];      /* GGUF order: shape[0] is the row length, shape[1] the row count */
    uint32_t gguf_type;
    uint64_t offset;        /* from the start of the data section */
    uint64_t size_bytes;
    const uint8_t *data;    /* the tensor's bytes inside the mapped (or caller-owned) file image */
} yule_gguf_tensor_info;

/* Maps the file read-only and parses it (GgufParser::parse_file). */
int32_t yule_gguf_open(const char *path, yule_gguf **out);
/* Parses an image the caller keeps alive until yule_gguf_close (GgufParser::parse_bytes). */
int32_t yule_gguf_parse(const void *data, size_t size, yule_gguf **out);
int32_t yule_gguf_close(yule_gguf *g);
/* Any out pointer may be null. */
int32_t yule_gguf_summary(const yule_gguf *g, uint32_t *version, uint64_t *n_tensors, uint64_t *n_kv,
                          uint64_t *data_offset, uint64_t *alignment);
int32_t yule_gguf_tensor(const yule_gguf *g, uint64_t index, yule_gguf_tensor_info *out);
int32_t yule_gguf_find_tensor(const yule_gguf *g, const char *name, uint64_t *index);
/* Metadata with the widening rules of GgufValue::as_u32 / as_f64 / as_str. */
int32_t yule_gguf_meta_u32(const yule_gguf *g, const char *key, uint32_t *out);
int32_t yule_gguf_meta_f64(const yule_gguf *g, const char *key, double *out);
int32_t yule_gguf_meta_str(const yule_gguf *g, const char *key, const char **out);
/* The runner configuration of the model in the file: GgufFile::to_loaded_model
 * (gguf.rs:493-586) plus the derivations of GpuTransformerRunner::new
 * (gpu_runner.rs:86-122).  max_seq_len = min(context_length, max_seq_len_cap)
 * when the cap is non-zero.  Llama-family architectures only. */
int32_t yule_gguf_runner_config(const yule_gguf *g, uint32_t max_seq_len_cap, yule_runner_config *cfg);
/* Creates a runner and uploads every tensor it needs from the file image through
 * pinned staging buffers and asynchronous copies (upload_weights,
 * gpu_runner.rs:171-254).  The runner owns the device buffers. */
int32_t yule_cuda_runner_load_gguf(yule_cuda_ctx *ctx, const yule_gguf *g, uint32_t max_seq_len_cap, uint32_t fused,
                                   yule_cuda_runner **out_runner);

#ifdef __cplusplus
}
#endif
#endif /* YULE_CUDA_H */
