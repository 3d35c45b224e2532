// glue.cu — the small f32 ops of the decode step: RMSNorm, RoPE, SiLU·mul, add, softmax, dense
// matvec, per-head score/value, the fused all-heads attention, argmax.
//
// Each kernel states which reference dispatch it stands for (yule-gpu/kernels/cuda/*.cu and
// yule-gpu/shaders/multihead_attn.comp); the arithmetic per output element is the same, only the
// order of the f32 partial sums differs (tree instead of 256-slot shared-memory ladder).

#include <cfloat>

#include "internal.h"

namespace yule {

namespace {

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}

// Block-wide sum / max for up to 1024 threads; `red` holds 32 floats.
__device__ __forceinline__ float block_sum(float v, float *red) {
    const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5, nw = (blockDim.x + 31) >> 5;
    v = warp_sum(v);
    __syncthreads();
    if (lane == 0) red[wid] = v;
    __syncthreads();
    float t = (lane < nw) ? red[lane] : 0.f;
    return warp_sum(t);
}
__device__ __forceinline__ float block_max(float v, float *red) {
    const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5, nw = (blockDim.x + 31) >> 5;
    v = warp_max(v);
    __syncthreads();
    if (lane == 0) red[wid] = v;
    __syncthreads();
    float t = (lane < nw) ? red[lane] : -FLT_MAX;
    return warp_max(t);
}

// kernels/cuda/matmul.cu:4-32 — one warp per output row.
__global__ void matvec_f32_kernel(const float *__restrict__ a, const float *__restrict__ b, float *__restrict__ out,
                                  uint32_t m, uint32_t k) {
    const uint32_t warp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    const int lane = threadIdx.x & 31;
    if (warp >= m) return;
    const float *row = a + (size_t)warp * k;
    float acc = 0.f;
    for (uint32_t i = lane; i < k; i += 32) acc = fmaf(row[i], b[i], acc);
    acc = warp_sum(acc);
    if (lane == 0) out[warp] = acc;
}

// Router of a mixture-of-experts layer (yule-infer/src/model_runner.rs:827-854): softmax over the n_exp router logits
// (left in `probs`), the n_used most probable experts in order of decreasing probability (equal probabilities: lower
// index first, as the CPU runner's stable sort leaves them) and their probabilities renormalised to sum 1.  A handful
// of values: one thread.
__global__ void moe_route_kernel(float *__restrict__ probs, uint32_t n_exp, uint32_t n_used, uint32_t *__restrict__ sel,
                                 float *__restrict__ w) {
    if (threadIdx.x != 0 || blockIdx.x != 0) return;
    float mx = -INFINITY;
    for (uint32_t i = 0; i < n_exp; i++) mx = fmaxf(mx, probs[i]);
    float sum = 0.f;
    for (uint32_t i = 0; i < n_exp; i++) {
        const float e = expf(probs[i] - mx);
        probs[i] = e;
        sum += e;
    }
    const float inv = 1.0f / sum;
    for (uint32_t i = 0; i < n_exp; i++) probs[i] *= inv;
    uint32_t picked[8] = {0, 0, 0, 0, 0, 0, 0, 0};  // n_exp <= 256
    float sel_sum = 0.f;
    for (uint32_t k = 0; k < n_used; k++) {
        int best = -1;
        for (uint32_t i = 0; i < n_exp; i++) {
            if ((picked[i >> 5] >> (i & 31)) & 1u) continue;
            if (best < 0 || probs[i] > probs[best]) best = (int)i;
        }
        picked[best >> 5] |= 1u << (best & 31);
        sel[k] = (uint32_t)best;
        sel_sum += probs[best];
    }
    const float inv_sel = 1.0f / sel_sum;
    for (uint32_t k = 0; k < n_used; k++) w[k] = probs[sel[k]] * inv_sel;
}

// out[i] += (*w) · x[i], the product and the sum rounded separately (model_runner.rs:950-952).
__global__ void axpy_dev_kernel(const float *__restrict__ w, const float *__restrict__ x, float *__restrict__ out, uint32_t n) {
    const uint32_t i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) out[i] = __fadd_rn(out[i], __fmul_rn(*w, x[i]));
}

// kernels/cuda/softmax.cu:3-45 — single CTA, max-subtracted.
__global__ void softmax_kernel(const float *__restrict__ in, float *__restrict__ out, uint32_t n) {
    __shared__ float red[32];
    float mx = -FLT_MAX;
    for (uint32_t i = threadIdx.x; i < n; i += blockDim.x) mx = fmaxf(mx, in[i]);
    mx = block_max(mx, red);
    float sum = 0.f;
    for (uint32_t i = threadIdx.x; i < n; i += blockDim.x) {
        float e = expf(in[i] - mx);
        out[i] = e;
        sum += e;
    }
    sum = block_sum(sum, red);
    const float inv = 1.0f / sum;
    for (uint32_t i = threadIdx.x; i < n; i += blockDim.x) out[i] *= inv;
}

// kernels/cuda/rms_norm.cu:4-36.  1/sqrt (not rsqrt.approx) so the scale matches the CPU
// runner's `1.0 / (ss / n + eps).sqrt()` (yule-infer/src/model_runner.rs:254-258).
__global__ void rms_norm_kernel(const float *__restrict__ in, const float *__restrict__ w, float *__restrict__ out,
                                uint32_t n, float eps) {
    yule_pdl_launch_dependents();
    yule_pdl_wait();
    __shared__ float red[32];
    in += (size_t)blockIdx.x * n;  // one CTA per row
    out += (size_t)blockIdx.x * n;
    float ss = 0.f;
    for (uint32_t i = threadIdx.x; i < n; i += blockDim.x) ss = fmaf(in[i], in[i], ss);
    ss = block_sum(ss, red);
    const float inv = 1.0f / sqrtf(ss / (float)n + eps);
    for (uint32_t i = threadIdx.x; i < n; i += blockDim.x) out[i] = in[i] * inv * w[i];
}

// kernels/cuda/rope.cu:3-49 with the angles supplied by the host.
__global__ void rope_angles_kernel(float *__restrict__ q, float *__restrict__ k, uint32_t head_dim, uint32_t n_heads_q,
                                   uint32_t n_heads_k, RopeAngles ang) {
    const uint32_t half = head_dim / 2;
    const uint32_t idx = blockIdx.x * blockDim.x + threadIdx.x;
    const uint32_t total_q = n_heads_q * half, total_k = n_heads_k * half;
    if (idx >= total_q + total_k) return;
    float *base = idx < total_q ? q : k;
    const uint32_t r = idx < total_q ? idx : idx - total_q;
    const uint32_t pair = r % half, head = r / half;
    float *p = base + (size_t)head * head_dim + 2 * pair;
    const float c = ang.cos[pair], s = ang.sin[pair];
    const float x0 = p[0], x1 = p[1];
    // Products and differences rounded separately, as the CPU code does (no contraction).
    p[0] = __fsub_rn(__fmul_rn(x0, c), __fmul_rn(x1, s));
    p[1] = __fadd_rn(__fmul_rn(x0, s), __fmul_rn(x1, c));
}

// Runner variant: RoPE on Q in place, RoPE on the new K row, and both K and V rows written
// straight into the caches at the position read from device memory — the Rope dispatch plus the
// two offset copies of yule-infer/src/gpu_runner.rs:422-470 in one launch.
__global__ void rope_kv_write_kernel(float *__restrict__ q, const float *__restrict__ k_tmp,
                                     const float *__restrict__ v_tmp, float *__restrict__ k_cache,
                                     float *__restrict__ v_cache, const float *__restrict__ cos_table,
                                     const float *__restrict__ sin_table, const uint32_t *__restrict__ pos_ptr,
                                     uint32_t head_dim, uint32_t n_heads, uint32_t n_kv_heads) {
    yule_pdl_launch_dependents();
    yule_pdl_wait();
    const uint32_t pos = *pos_ptr;
    const uint32_t half = head_dim / 2;
    const uint32_t kv_stride = n_kv_heads * head_dim;
    const uint32_t total_q = n_heads * half, total_k = n_kv_heads * half;
    const uint32_t idx = blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= total_q + total_k) return;
    const bool is_q = idx < total_q;
    const uint32_t r = is_q ? idx : idx - total_q;
    const uint32_t pair = r % half, head = r / half;
    const float c = cos_table[(size_t)pos * half + pair], s = sin_table[(size_t)pos * half + pair];
    const size_t off = (size_t)head * head_dim + 2 * pair;
    const float *src = is_q ? q + off : k_tmp + off;
    const float x0 = src[0], x1 = src[1];
    const float y0 = __fsub_rn(__fmul_rn(x0, c), __fmul_rn(x1, s));
    const float y1 = __fadd_rn(__fmul_rn(x0, s), __fmul_rn(x1, c));
    if (is_q) {
        q[off] = y0;
        q[off + 1] = y1;
    } else {
        float *kd = k_cache + (size_t)pos * kv_stride + off;
        kd[0] = y0;
        kd[1] = y1;
        float *vd = v_cache + (size_t)pos * kv_stride + off;
        vd[0] = v_tmp[off];
        vd[1] = v_tmp[off + 1];
    }
}

// Batched form for prefill: token slot z = blockIdx.y sits at position pos0 + z; q[z] is rotated in
// place, k[z] is rotated into the K cache row of its position and v[z] copied into the V cache.
// Batched decode uses the same kernel with `row_pos` set: slot z is then the current token of sequence z, at
// position row_pos[z] of that sequence's own cache (caches `cache_stride` floats apart).
__global__ void rope_kv_write_batch_kernel(float *__restrict__ q, const float *__restrict__ k, const float *__restrict__ v,
                                           float *__restrict__ k_cache, float *__restrict__ v_cache,
                                           const float *__restrict__ cos_table, const float *__restrict__ sin_table,
                                           uint32_t pos0, uint32_t head_dim, uint32_t n_heads, uint32_t n_kv_heads,
                                           const uint32_t *__restrict__ row_pos, size_t cache_stride) {
    const uint32_t z = blockIdx.y, pos = row_pos ? row_pos[z] : pos0 + z;
    if (row_pos) {
        k_cache += (size_t)z * cache_stride;
        v_cache += (size_t)z * cache_stride;
    }
    const uint32_t half = head_dim / 2;
    const uint32_t kv_stride = n_kv_heads * head_dim, q_stride = n_heads * head_dim;
    const uint32_t total_q = n_heads * half, total_k = n_kv_heads * half;
    const uint32_t idx = blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= total_q + total_k) return;
    const bool is_q = idx < total_q;
    const uint32_t r = is_q ? idx : idx - total_q;
    const uint32_t pair = r % half, head = r / half;
    const float c = cos_table[(size_t)pos * half + pair], sn = sin_table[(size_t)pos * half + pair];
    const size_t off = (size_t)head * head_dim + 2 * pair;
    const float *src = is_q ? q + (size_t)z * q_stride + off : k + (size_t)z * kv_stride + off;
    const float x0 = src[0], x1 = src[1];
    const float y0 = __fsub_rn(__fmul_rn(x0, c), __fmul_rn(x1, sn));
    const float y1 = __fadd_rn(__fmul_rn(x0, sn), __fmul_rn(x1, c));
    if (is_q) {
        q[(size_t)z * q_stride + off] = y0;
        q[(size_t)z * q_stride + off + 1] = y1;
    } else {
        float *kd = k_cache + (size_t)pos * kv_stride + off;
        kd[0] = y0;
        kd[1] = y1;
        float *vd = v_cache + (size_t)pos * kv_stride + off;
        vd[0] = v[(size_t)z * kv_stride + off];
        vd[1] = v[(size_t)z * kv_stride + off + 1];
    }
}

// kernels/cuda/silu_mul.cu:3-14.
__global__ void silu_mul_kernel(const float *__restrict__ gate, const float *__restrict__ up, float *__restrict__ out,
                                uint32_t n) {
    yule_pdl_launch_dependents();
    yule_pdl_wait();
    const uint32_t i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    const float x = gate[i];
    out[i] = (x / (1.0f + expf(-x))) * up[i];
}

// Element-wise pieces of the architecture variants of yule-infer/src/model_runner.rs: out[i] = f(a[i], b[i], v).
//   kAddScalar   a + v                      norm weights with Gemma's offset (:246-275: w[i] + offset)
//   kScale       a * v                      Gemma's embedding scale sqrt(dim) (:568-574)
//   kSoftcap     v * tanh(a / v)            final logit softcap (:1027-1032)
//   kGeluMul     gelu(a) * b                GeGLU (:312-314, :974-978), gelu in its tanh form
//   kAddVec      a + b                      Q/K/V bias (:295-310), residual after a post-norm (:781-783)
enum ElemOp { kAddScalar, kScale, kSoftcap, kGeluMul, kAddVec };
template <int OP>
__global__ void elementwise_kernel(const float *__restrict__ a, const float *__restrict__ b, float *__restrict__ out, uint32_t n,
                                   float v) {
    yule_pdl_launch_dependents();
    yule_pdl_wait();
    const uint32_t i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    const float x = a[i];
    float r;
    if (OP == kAddScalar) {
        r = x + v;
    } else if (OP == kScale) {
        r = x * v;
    } else if (OP == kSoftcap) {
        r = v * tanhf(x / v);
    } else if (OP == kGeluMul) {
        r = (x * 0.5f * (1.0f + tanhf(0.7978846f * (x + 0.044715f * x * x * x)))) * b[i];
    } else {
        r = x + b[i];
    }
    out[i] = r;
}

// kernels/cuda/add.cu:2-11.
__global__ void add_kernel(const float *__restrict__ a, const float *__restrict__ b, float *__restrict__ out, uint32_t n) {
    const uint32_t i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) out[i] = a[i] + b[i];
}

// kernels/cuda/attn_score.cu:3-33 — one warp per position.
__global__ void attn_score_kernel(const float *__restrict__ q, const float *__restrict__ k_cache,
                                  float *__restrict__ scores, uint32_t hd, uint32_t seq_len, uint32_t head_offset,
                                  uint32_t kv_offset, uint32_t kv_stride) {
    const uint32_t t = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    const int lane = threadIdx.x & 31;
    if (t >= seq_len) return;
    const float *kp = k_cache + (size_t)t * kv_stride + kv_offset;
    float acc = 0.f;
    for (uint32_t d = lane; d < hd; d += 32) acc = fmaf(q[head_offset + d], kp[d], acc);
    acc = warp_sum(acc);
    if (lane == 0) scores[t] = acc / sqrtf((float)hd);
}

// kernels/cuda/attn_value.cu:3-33 — one thread per output dimension.
__global__ void attn_value_kernel(const float *__restrict__ w, const float *__restrict__ v_cache, float *__restrict__ out,
                                  uint32_t hd, uint32_t seq_len, uint32_t kv_offset, uint32_t kv_stride,
                                  uint32_t out_offset) {
    const uint32_t d = blockIdx.x * blockDim.x + threadIdx.x;
    if (d >= hd) return;
    float acc = 0.f;
    for (uint32_t t = 0; t < seq_len; t++) acc = fmaf(w[t], v_cache[(size_t)t * kv_stride + kv_offset + d], acc);
    out[out_offset + d] = acc;
}

// shaders/multihead_attn.comp (the MultiheadAttn dispatch, gpu_runner.rs:477-499): one CTA per
// head; scores for all positions in shared memory → max-subtracted softmax → weighted V sum.
// The sequence length is position+1 read from device memory when pos_ptr is set, so the same
// launch can be replayed from a CUDA graph at every position.
constexpr int kAttnThreads = 256;
__global__ void __launch_bounds__(kAttnThreads)
multihead_attention_kernel(const float *__restrict__ q, const float *__restrict__ k_cache,
                           const float *__restrict__ v_cache, float *__restrict__ out, uint32_t hd, uint32_t seq_len_arg,
                           const uint32_t *__restrict__ pos_ptr, uint32_t n_heads, uint32_t n_kv_heads,
                           uint32_t kv_stride, uint32_t window, float softcap) {
    extern __shared__ __align__(16) float sm[];
    __shared__ float red[32];
    yule_pdl_launch_dependents();
    yule_pdl_wait();
    const uint32_t seq_len = pos_ptr ? (*pos_ptr + 1) : seq_len_arg;
    const uint32_t head = blockIdx.x;
    const uint32_t kv_head = head / (n_heads / n_kv_heads);
    float *qs = sm;                 // hd floats
    float *scores = sm + hd;        // seq_len floats
    float *partial = scores + seq_len;  // (kAttnThreads / hd_lanes) × hd floats, see below
    const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5;
    const float scale = 1.0f / sqrtf((float)hd);
    // sliding window (yule-infer/src/model_runner.rs:688-696): positions before pos − window are masked to −inf
    // there, i.e. carry no weight; here they are simply not visited
    // With a softcap as well the reference caps after masking, and cap·tanh(−inf / cap) = −cap is a finite score:
    // masked positions then keep a small weight, so they are visited and given exactly that score.
    const uint32_t pos = seq_len - 1;
    const uint32_t first_visible = (window && pos >= window) ? pos - window : 0;
    const uint32_t begin = softcap != 0.f ? 0u : first_visible;

    for (uint32_t d = threadIdx.x; d < hd; d += blockDim.x) qs[d] = q[(size_t)head * hd + d];
    __syncthreads();

    // scores: one warp per position, lanes across head_dim (coalesced K rows)
    float mx = -FLT_MAX;
    for (uint32_t t = begin + wid; t < seq_len; t += kAttnThreads / 32) {
        const float *kp = k_cache + (size_t)t * kv_stride + (size_t)kv_head * hd;
        float acc = 0.f;
        for (uint32_t d = lane; d < hd; d += 32) acc = fmaf(qs[d], kp[d], acc);
        acc = warp_sum(acc) * scale;
        if (softcap != 0.f) acc = t < first_visible ? -softcap : softcap * tanhf(acc / softcap);  // attention logit softcap (:716-721)
        if (lane == 0) scores[t] = acc;
        mx = fmaxf(mx, acc);
    }
    mx = block_max(mx, red);  // also orders the score writes before the reads below

    float sum = 0.f;
    for (uint32_t t = begin + threadIdx.x; t < seq_len; t += blockDim.x) {
        float e = expf(scores[t] - mx);
        scores[t] = e;
        sum += e;
    }
    sum = block_sum(sum, red);
    const float inv = 1.0f / sum;

    // weighted V: thread (slice, d) sums positions slice, slice+n_slices, … for dimension d
    const uint32_t n_slices = kAttnThreads / hd ? kAttnThreads / hd : 1;
    const uint32_t d = threadIdx.x % hd, slice = threadIdx.x / hd;
    float acc = 0.f;
    if (slice < n_slices && threadIdx.x < n_slices * hd) {
        for (uint32_t t = begin + slice; t < seq_len; t += n_slices)
            acc = fmaf(scores[t] * inv, v_cache[(size_t)t * kv_stride + (size_t)kv_head * hd + d], acc);
        partial[slice * hd + d] = acc;
    }
    __syncthreads();
    for (uint32_t dd = threadIdx.x; dd < hd; dd += blockDim.x) {
        float o = 0.f;
        for (uint32_t s2 = 0; s2 < n_slices; s2++) o += partial[s2 * hd + dd];
        out[(size_t)head * hd + dd] = o;
    }
}

// Greedy pick with ties to the highest index (yule-infer/src/sampler.rs:150-163) into state[0];
// with `history` the pick is also logged at history[position] and the position (state[1]) is
// advanced, so the next graph replay continues the sequence without the host.
__global__ void argmax_kernel(const float *__restrict__ v, uint32_t n, uint32_t *__restrict__ state,
                              uint32_t *__restrict__ history) {
    yule_pdl_launch_dependents();
    yule_pdl_wait();
    __shared__ float bv[32];
    __shared__ uint32_t bi[32];
    float best = -FLT_MAX;
    uint32_t idx = 0;
    bool any = false;
    // eight loads in flight per thread (the logits sit in L2; one load at a time is all latency)
    for (uint32_t base = threadIdx.x; base < n; base += blockDim.x * 8) {
        float x[8];
#pragma unroll
        for (int k = 0; k < 8; k++) {
            const uint32_t i = base + k * blockDim.x;
            x[k] = i < n ? v[i] : 0.f;
        }
#pragma unroll
        for (int k = 0; k < 8; k++) {
            const uint32_t i = base + k * blockDim.x;
            if (i < n && (!any || x[k] >= best)) {
                best = x[k];
                idx = i;
                any = true;
            }
        }
    }
    if (!any) best = -FLT_MAX;
    const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5, nw = blockDim.x >> 5;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        float ob = __shfl_xor_sync(0xffffffffu, best, o);
        uint32_t oi = __shfl_xor_sync(0xffffffffu, idx, o);
        if (ob > best || (ob == best && oi > idx)) {
            best = ob;
            idx = oi;
        }
    }
    if (lane == 0) {
        bv[wid] = best;
        bi[wid] = idx;
    }
    __syncthreads();
    if (wid == 0) {
        best = lane < nw ? bv[lane] : -FLT_MAX;
        idx = lane < nw ? bi[lane] : 0;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            float ob = __shfl_xor_sync(0xffffffffu, best, o);
            uint32_t oi = __shfl_xor_sync(0xffffffffu, idx, o);
            if (ob > best || (ob == best && oi > idx)) {
                best = ob;
                idx = oi;
            }
        }
        if (lane == 0) {
            state[0] = idx;
            if (history) {
                const uint32_t pos = state[1];
                history[pos] = idx;
                state[1] = pos + 1;
                state[2] += 1;  // token counter that reset() never rewinds (epochs of the peer exchange)
            }
        }
    }
}

// Batched decode: row b = blockIdx.x of [batch][n] logits → tokens[b] (ties to the highest index, as above),
// logged at history[b * history_stride + step[0]]; block 0 advances every sequence's position and the step.
__global__ void argmax_rows_kernel(const float *__restrict__ v, uint32_t n, uint32_t *__restrict__ tokens, uint32_t *__restrict__ pos,
                                   uint32_t *__restrict__ step, uint32_t *__restrict__ history, uint32_t history_stride) {
    __shared__ float bv[32];
    __shared__ uint32_t bi[32];
    const float *row = v + (size_t)blockIdx.x * n;
    float best = -FLT_MAX;
    uint32_t idx = 0;
    bool any = false;
    for (uint32_t i = threadIdx.x; i < n; i += blockDim.x) {
        const float x = row[i];
        if (!any || x >= best) {
            best = x;
            idx = i;
            any = true;
        }
    }
    if (!any) best = -FLT_MAX;
    const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5, nw = blockDim.x >> 5;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        float ob = __shfl_xor_sync(0xffffffffu, best, o);
        uint32_t oi = __shfl_xor_sync(0xffffffffu, idx, o);
        if (ob > best || (ob == best && oi > idx)) {
            best = ob;
            idx = oi;
        }
    }
    if (lane == 0) {
        bv[wid] = best;
        bi[wid] = idx;
    }
    __syncthreads();
    if (wid == 0) {
        best = lane < nw ? bv[lane] : -FLT_MAX;
        idx = lane < nw ? bi[lane] : 0;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            float ob = __shfl_xor_sync(0xffffffffu, best, o);
            uint32_t oi = __shfl_xor_sync(0xffffffffu, idx, o);
            if (ob > best || (ob == best && oi > idx)) {
                best = ob;
                idx = oi;
            }
        }
        if (lane == 0) {
            tokens[blockIdx.x] = idx;
            if (history) history[(size_t)blockIdx.x * history_stride + step[0]] = idx;
        }
    }
}
// After the picks of a step: every sequence moves one position on.
__global__ void advance_rows_kernel(uint32_t *__restrict__ pos, uint32_t *__restrict__ step, uint32_t batch) {
    const uint32_t i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i < batch) pos[i] += 1;
    if (i == 0) step[0] += 1;
}

__global__ void fill_bytes_kernel(uint4 *__restrict__ p, size_t n16, uint32_t v) {
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n16; i += (size_t)gridDim.x * blockDim.x)
        p[i] = make_uint4(v, v, v, v);
}

}  // namespace

cudaError_t launch_matvec_f32(const float *a, const float *b, float *out, uint32_t m, uint32_t k, cudaStream_t s,
                              uint64_t *launches) {
    matvec_f32_kernel<<<(m + 7) / 8, 256, 0, s>>>(a, b, out, m, k);
    *launches += 1;
    return cudaGetLastError();
}
cudaError_t launch_moe_route(float *probs, uint32_t n_exp, uint32_t n_used, uint32_t *sel, float *w, cudaStream_t s, uint64_t *launches) {
    if (n_exp == 0 || n_exp > 256 || n_used == 0 || n_used > n_exp) return cudaErrorInvalidValue;
    moe_route_kernel<<<1, 32, 0, s>>>(probs, n_exp, n_used, sel, w);
    *launches += 1;
    return cudaGetLastError();
}
cudaError_t launch_axpy_dev(const float *w, const float *x, float *out, uint32_t n, cudaStream_t s, uint64_t *launches) {
    axpy_dev_kernel<<<(n + 255) / 256, 256, 0, s>>>(w, x, out, n);
    *launches += 1;
    return cudaGetLastError();
}
cudaError_t launch_softmax(const float *in, float *out, uint32_t n, cudaStream_t s, uint64_t *launches) {
    softmax_kernel<<<1, 1024, 0, s>>>(in, out, n);
    *launches += 1;
    return cudaGetLastError();
}
cudaError_t launch_rms_norm(const float *in, const float *w, float *out, uint32_t n, float eps, cudaStream_t s,
                            uint64_t *launches, bool pdl) {
    *launches += 1;
    return launch_kernel(rms_norm_kernel, dim3(1), dim3(1024), 0, s, pdl, in, w, out, n, eps);
}
cudaError_t launch_rms_norm_rows(const float *in, const float *w, float *out, uint32_t n, uint32_t rows, float eps, cudaStream_t s,
                                 uint64_t *launches) {
    if (rows == 0) return cudaSuccess;
    *launches += 1;
    return launch_kernel(rms_norm_kernel, dim3(rows), dim3(1024), 0, s, true, in, w, out, n, eps);
}
cudaError_t launch_rope_angles(float *q, float *k, uint32_t head_dim, uint32_t n_heads_q, uint32_t n_heads_k,
                               const RopeAngles &ang, cudaStream_t s, uint64_t *launches) {
    uint32_t total = (n_heads_q + n_heads_k) * (head_dim / 2);
    if (total == 0) return cudaSuccess;
    rope_angles_kernel<<<(total + 255) / 256, 256, 0, s>>>(q, k, head_dim, n_heads_q, n_heads_k, ang);
    *launches += 1;
    return cudaGetLastError();
}
cudaError_t launch_rope_kv_write(float *q, const float *k_tmp, const float *v_tmp, float *k_cache, float *v_cache,
                                 const float *cos_table, const float *sin_table, const uint32_t *pos_ptr,
                                 uint32_t head_dim, uint32_t n_heads, uint32_t n_kv_heads, cudaStream_t s,
                                 uint64_t *launches, bool pdl) {
    uint32_t total = (n_heads + n_kv_heads) * (head_dim / 2);
    *launches += 1;
    return launch_kernel(rope_kv_write_kernel, dim3((total + 255) / 256), dim3(256), 0, s, pdl, q, k_tmp, v_tmp, k_cache,
                         v_cache, cos_table, sin_table, pos_ptr, head_dim, n_heads, n_kv_heads);
}
cudaError_t launch_rope_kv_write_batch(float *q, const float *k, const float *v, float *k_cache, float *v_cache,
                                       const float *cos_table, const float *sin_table, uint32_t pos0, uint32_t n_tokens,
                                       uint32_t head_dim, uint32_t n_heads, uint32_t n_kv_heads, cudaStream_t s,
                                       uint64_t *launches, const uint32_t *row_pos, size_t cache_stride) {
    uint32_t total = (n_heads + n_kv_heads) * (head_dim / 2);
    *launches += 1;
    rope_kv_write_batch_kernel<<<dim3((total + 255) / 256, n_tokens), 256, 0, s>>>(q, k, v, k_cache, v_cache, cos_table, sin_table,
                                                                                  pos0, head_dim, n_heads, n_kv_heads, row_pos,
                                                                                  cache_stride);
    return cudaGetLastError();
}
cudaError_t launch_silu_mul(const float *gate, const float *up, float *out, uint32_t n, cudaStream_t s,
                            uint64_t *launches, bool pdl) {
    *launches += 1;
    return launch_kernel(silu_mul_kernel, dim3((n + 255) / 256), dim3(256), 0, s, pdl, gate, up, out, n);
}
cudaError_t launch_add(const float *a, const float *b, float *out, uint32_t n, cudaStream_t s, uint64_t *launches) {
    add_kernel<<<(n + 255) / 256, 256, 0, s>>>(a, b, out, n);
    *launches += 1;
    return cudaGetLastError();
}
cudaError_t launch_attn_score(const float *q, const float *k_cache, float *scores, uint32_t hd, uint32_t seq_len,
                              uint32_t head_offset, uint32_t kv_offset, uint32_t kv_stride, cudaStream_t s,
                              uint64_t *launches) {
    attn_score_kernel<<<(seq_len + 7) / 8, 256, 0, s>>>(q, k_cache, scores, hd, seq_len, head_offset, kv_offset,
                                                        kv_stride);
    *launches += 1;
    return cudaGetLastError();
}
cudaError_t launch_attn_value(const float *w, const float *v_cache, float *out, uint32_t hd, uint32_t seq_len,
                              uint32_t kv_offset, uint32_t kv_stride, uint32_t out_offset, cudaStream_t s,
                              uint64_t *launches) {
    attn_value_kernel<<<(hd + 127) / 128, 128, 0, s>>>(w, v_cache, out, hd, seq_len, kv_offset, kv_stride, out_offset);
    *launches += 1;
    return cudaGetLastError();
}
cudaError_t launch_multihead_attention(const float *q, const float *k_cache, const float *v_cache, float *out,
                                       uint32_t hd, uint32_t seq_len, const uint32_t *pos_ptr, uint32_t max_seq_len,
                                       uint32_t n_heads, uint32_t n_kv_heads, uint32_t kv_stride, cudaStream_t s,
                                       uint64_t *launches, bool pdl, uint32_t window, float softcap) {
    uint32_t n_slices = kAttnThreads / hd ? kAttnThreads / hd : 1;
    size_t smem = ((size_t)hd + max_seq_len + (size_t)n_slices * hd) * sizeof(float);
    if (smem > 200 * 1024) return cudaErrorInvalidValue;
    if (smem > 48 * 1024) {
        cudaError_t e = cudaFuncSetAttribute(multihead_attention_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                             (int)smem);
        if (e != cudaSuccess) return e;
    }
    *launches += 1;
    return launch_kernel(multihead_attention_kernel, dim3(n_heads), dim3(kAttnThreads), smem, s, pdl, q, k_cache,
                         v_cache, out, hd, seq_len, pos_ptr, n_heads, n_kv_heads, kv_stride, window, softcap);
}
cudaError_t launch_elementwise(int op, const float *a, const float *b, float *out, uint32_t n, float v, cudaStream_t s,
                               uint64_t *launches, bool pdl) {
    if (n == 0) return cudaSuccess;
    *launches += 1;
    const dim3 grid((n + 255) / 256), block(256);
    switch (op) {
        case kAddScalar: return launch_kernel(elementwise_kernel<kAddScalar>, grid, block, 0, s, pdl, a, b, out, n, v);
        case kScale: return launch_kernel(elementwise_kernel<kScale>, grid, block, 0, s, pdl, a, b, out, n, v);
        case kSoftcap: return launch_kernel(elementwise_kernel<kSoftcap>, grid, block, 0, s, pdl, a, b, out, n, v);
        case kGeluMul: return launch_kernel(elementwise_kernel<kGeluMul>, grid, block, 0, s, pdl, a, b, out, n, v);
        default: return launch_kernel(elementwise_kernel<kAddVec>, grid, block, 0, s, pdl, a, b, out, n, v);
    }
}
cudaError_t launch_argmax(const float *v, uint32_t n, uint32_t *state, uint32_t *history, cudaStream_t s,
                          uint64_t *launches, bool pdl) {
    *launches += 1;
    return launch_kernel(argmax_kernel, dim3(1), dim3(1024), 0, s, pdl, v, n, state, history);
}
cudaError_t launch_argmax_rows(const float *v, uint32_t n, uint32_t batch, uint32_t *tokens, uint32_t *pos, uint32_t *step,
                               uint32_t *history, uint32_t history_stride, cudaStream_t s, uint64_t *launches) {
    argmax_rows_kernel<<<batch, 1024, 0, s>>>(v, n, tokens, pos, step, history, history_stride);
    *launches += 1;
    return cudaGetLastError();
}
cudaError_t launch_advance_rows(uint32_t *pos, uint32_t *step, uint32_t batch, cudaStream_t s, uint64_t *launches) {
    advance_rows_kernel<<<batch ? (batch + 255) / 256 : 1, 256, 0, s>>>(pos, step, batch);  // batch 0: only the counter moves
    *launches += 1;
    return cudaGetLastError();
}
cudaError_t launch_fill_bytes(void *p, size_t n, int value, cudaStream_t s, uint64_t *launches) {
    uint32_t v = (uint32_t)(value & 0xFF) * 0x01010101u;
    fill_bytes_kernel<<<148 * 8, 256, 0, s>>>((uint4 *)p, n / 16, v);
    *launches += 1;
    return cudaGetLastError();
}

}  // namespace yule
