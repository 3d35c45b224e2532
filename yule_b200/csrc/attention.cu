// attention.cu — GQA decode attention over the flat fp32 KV cache, split over positions.
//
// What it computes is the per-head loop of yule-infer/src/model_runner.rs:672-758 (equivalently
// the MultiheadAttn dispatch, yule-gpu/shaders/multihead_attn.comp): for head h with KV head
// h / (n_heads / n_kv_heads),
//     s_t = (q_h · K[t]) / sqrt(hd),  p = softmax(s) (max-subtracted),  o_h = Σ_t p_t · V[t].
// In the runner's graph it also does the work of the Rope dispatch and the two KV-cache copies
// (yule-infer/src/gpu_runner.rs:422-470): q and the new k row are rotated here with the
// host-built cos/sin table, and the new K/V rows are written to the caches.
//
// Grid (n_heads, n_splits): CTA (h, s) handles positions [s·chunk, (s+1)·chunk).  One thread per
// position computes a whole score (q is broadcast from shared memory; no shuffles), then the CTA
// forms its local max / sum-of-exponentials / weighted V sum.  With more than one split the
// partial triples go to a scratch area and the CTA that arrives last for a head (a ticket from one
// atomicAdd — nobody waits for anybody) merges them in split order, the standard log-sum-exp
// merge of yule-gpu/shaders/flash_decode_reduce.comp.

#include <cfloat>

#include "internal.h"

namespace yule {

namespace {

constexpr int kThreads = 256;

__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}
__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}

struct AttnParams {
    // inputs
    const float *q;        // [n_heads][hd]; rotated here when cos_table is set
    const float *k_new;    // [n_kv][hd] un-rotated K row of the current token (fused mode) or null
    const float *v_new;    // [n_kv][hd] V row of the current token (fused mode) or null
    float *k_cache;        // [max_seq][kv_stride]
    float *v_cache;
    const float *cos_table, *sin_table;  // [max_seq][hd/2] or null
    const uint32_t *pos_ptr;             // device position (fused / graph mode) or null
    uint32_t seq_len;                    // used when pos_ptr is null
    float *out;                          // [n_heads][hd]
    float *scratch;                      // [n_heads][n_splits][hd + 2] partial (m, l, acc)
    uint32_t *tickets;                   // [n_heads], zero between launches
    uint32_t hd, n_heads, n_kv_heads, kv_stride, n_splits, max_chunk, min_chunk;
    uint32_t q_stride, out_stride;       // floats between the q / out rows of consecutive queries (blockIdx.z)
    uint32_t pos_per_query;              // batched decode: query z sits at pos_ptr[z] of its own caches
    size_t kv_batch_stride;              // floats between the caches of consecutive queries (batched decode)
    uint32_t window;                     // sliding window (model_runner.rs:688-696), 0 = none
    float softcap;                       // attention logit softcap (model_runner.rs:716-721), 0 = none
    TpFuse tp;                           // tensor parallelism: the output also goes out as (value, epoch) pairs
};

__global__ void __launch_bounds__(kThreads) attn_decode_kernel(const AttnParams p) {
    extern __shared__ __align__(16) float sm[];
    __shared__ float red[2 * (kThreads / 32)];
    __shared__ uint32_t s_last;
    yule_pdl_launch_dependents();
    yule_pdl_wait();

    const uint32_t hd = p.hd, hd4 = hd / 4;
    const uint32_t head = blockIdx.x, split = blockIdx.y;
    const uint32_t group = p.n_heads / p.n_kv_heads, kvh = head / group;
    const uint32_t pos = p.pos_ptr ? *p.pos_ptr : p.seq_len - 1;
    const uint32_t seq = pos + 1;
    const bool fused = p.k_new != nullptr;
    // splits actually used at this sequence length: at least 256 positions each (one per thread);
    // the rest exit.  Short sequences therefore take the single-CTA path with no merge step.
    // Sliding window: the reference masks positions t < pos − window to −inf once pos >= window; they then carry
    // no weight, so the splits simply cover [begin, seq) instead of [0, seq).  With an attention softcap as well
    // the reference caps after masking (model_runner.rs:688-721), and cap·tanh(−inf / cap) is −cap, a finite
    // score: masked positions then keep a (small) weight, so they are visited and given exactly that score.
    const uint32_t first_visible = (p.window && pos >= p.window) ? pos - p.window : 0;
    const uint32_t begin = p.softcap != 0.f ? 0u : first_visible;
    const uint32_t span = seq - begin;
    uint32_t eff = (span + p.min_chunk - 1) / p.min_chunk;
    eff = eff < 1 ? 1 : (eff > p.n_splits ? p.n_splits : eff);
    if (split >= eff) return;
    const uint32_t chunk = (span + eff - 1) / eff;
    const uint32_t lo = begin + (split * chunk < span ? split * chunk : span);
    const uint32_t hi = lo + chunk < seq ? lo + chunk : seq;
    const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5;

    float *qs = sm;                 // hd: the (rotated) query of this head
    float *kcur = qs + hd;          // hd: rotated K row of the current token (fused mode)
    float *scores = kcur + hd;      // max_chunk
    float *partial = scores + p.max_chunk;  // n_slices × hd

    // q (and the new k row) with RoPE: pairs (2i, 2i+1) rotated by the table entry of this position,
    // products and sums rounded separately as in apply_rope (model_runner.rs:277-293)
    for (uint32_t i = threadIdx.x; i < hd / 2; i += kThreads) {
        float q0 = p.q[(size_t)head * hd + 2 * i], q1 = p.q[(size_t)head * hd + 2 * i + 1];
        if (p.cos_table) {
            const float c = p.cos_table[(size_t)pos * (hd / 2) + i], s = p.sin_table[(size_t)pos * (hd / 2) + i];
            const float r0 = __fsub_rn(__fmul_rn(q0, c), __fmul_rn(q1, s));
            const float r1 = __fadd_rn(__fmul_rn(q0, s), __fmul_rn(q1, c));
            q0 = r0;
            q1 = r1;
            if (fused) {
                const float k0 = p.k_new[(size_t)kvh * hd + 2 * i], k1 = p.k_new[(size_t)kvh * hd + 2 * i + 1];
                kcur[2 * i] = __fsub_rn(__fmul_rn(k0, c), __fmul_rn(k1, s));
                kcur[2 * i + 1] = __fadd_rn(__fmul_rn(k0, s), __fmul_rn(k1, c));
            }
        } else if (fused) {
            kcur[2 * i] = p.k_new[(size_t)kvh * hd + 2 * i];
            kcur[2 * i + 1] = p.k_new[(size_t)kvh * hd + 2 * i + 1];
        }
        qs[2 * i] = q0;
        qs[2 * i + 1] = q1;
    }
    __syncthreads();

    // The first head of each GQA group, in the split that owns the current position, appends the
    // new K and V rows to the caches (readers of this launch take them from k_new / v_new).
    if (fused && head % group == 0 && pos >= lo && pos < hi) {
        for (uint32_t d = threadIdx.x; d < hd; d += kThreads) {
            p.k_cache[(size_t)pos * p.kv_stride + (size_t)kvh * hd + d] = kcur[d];
            p.v_cache[(size_t)pos * p.kv_stride + (size_t)kvh * hd + d] = p.v_new[(size_t)kvh * hd + d];
        }
    }

    // scores: one thread per position
    const float scale = 1.0f / sqrtf((float)hd);
    float mx = -FLT_MAX;
    for (uint32_t t = lo + threadIdx.x; t < hi; t += kThreads) {
        const float4 *kp = (fused && t == pos) ? reinterpret_cast<const float4 *>(kcur)
                                               : reinterpret_cast<const float4 *>(p.k_cache + (size_t)t * p.kv_stride + (size_t)kvh * hd);
        const float4 *qp = reinterpret_cast<const float4 *>(qs);
        float a0 = 0.f, a1 = 0.f, a2 = 0.f, a3 = 0.f;
        for (uint32_t i = 0; i < hd4; i++) {
            const float4 k = kp[i], q = qp[i];
            a0 = fmaf(q.x, k.x, a0);
            a1 = fmaf(q.y, k.y, a1);
            a2 = fmaf(q.z, k.z, a2);
            a3 = fmaf(q.w, k.w, a3);
        }
        float sc = ((a0 + a1) + (a2 + a3)) * scale;
        if (p.softcap != 0.f) sc = t < first_visible ? -p.softcap : p.softcap * tanhf(sc / p.softcap);
        scores[t - lo] = sc;
        mx = fmaxf(mx, sc);
    }
    mx = warp_max(mx);
    if (lane == 0) red[wid] = mx;
    __syncthreads();
    mx = -FLT_MAX;
#pragma unroll
    for (int i = 0; i < kThreads / 32; i++) mx = fmaxf(mx, red[i]);

    float sum = 0.f;
    for (uint32_t t = lo + threadIdx.x; t < hi; t += kThreads) {
        const float e = expf(scores[t - lo] - mx);
        scores[t - lo] = e;
        sum += e;
    }
    sum = warp_sum(sum);
    if (lane == 0) red[kThreads / 32 + wid] = sum;
    __syncthreads();
    sum = 0.f;
#pragma unroll
    for (int i = 0; i < kThreads / 32; i++) sum += red[kThreads / 32 + i];

    // Σ_t e_t · V[t]: thread (slice, d4) takes positions slice, slice + n_slices, … for 4 dimensions
    const uint32_t n_slices = kThreads / hd4;
    const uint32_t d4 = threadIdx.x % hd4, slice = threadIdx.x / hd4;
    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
    if (slice < n_slices) {
        for (uint32_t t = lo + slice; t < hi; t += n_slices) {
            const float4 *vp = (fused && t == pos) ? reinterpret_cast<const float4 *>(p.v_new + (size_t)kvh * hd)
                                                   : reinterpret_cast<const float4 *>(p.v_cache + (size_t)t * p.kv_stride + (size_t)kvh * hd);
            const float4 v = vp[d4];
            const float e = scores[t - lo];
            acc.x = fmaf(e, v.x, acc.x);
            acc.y = fmaf(e, v.y, acc.y);
            acc.z = fmaf(e, v.z, acc.z);
            acc.w = fmaf(e, v.w, acc.w);
        }
        reinterpret_cast<float4 *>(partial)[slice * hd4 + d4] = acc;
    }
    __syncthreads();
    float o = 0.f;  // thread d < hd: this split's un-normalised output for dimension d
    if (threadIdx.x < hd)
        for (uint32_t s2 = 0; s2 < n_slices; s2++) o += partial[s2 * hd + threadIdx.x];

    if (eff == 1) {
        if (threadIdx.x < hd) p.out[(size_t)head * hd + threadIdx.x] = o * (1.0f / sum);
        return;
    }

    // publish (m, l, acc) of this split, then take a ticket; the last CTA of the head merges
    float *mine = p.scratch + ((size_t)head * p.n_splits + split) * (hd + 2);
    if (threadIdx.x < hd) mine[2 + threadIdx.x] = o;
    if (threadIdx.x == 0) {
        mine[0] = lo < hi ? mx : -FLT_MAX;
        mine[1] = lo < hi ? sum : 0.f;
    }
    __threadfence();
    __syncthreads();
    if (threadIdx.x == 0) s_last = (atomicAdd(&p.tickets[head], 1u) == eff - 1) ? 1u : 0u;
    __syncthreads();
    if (!s_last) return;
    __threadfence();
    // __ldcg: these words were written by other SMs; read them from L2, not from a stale L1 line.
    // All loads are issued before any is used (one L2 round trip, not one per split).
    const float *all = p.scratch + (size_t)head * p.n_splits * (hd + 2);
    constexpr int kMaxSplits = 16;
    float ms[kMaxSplits], ls[kMaxSplits], os[kMaxSplits];
#pragma unroll
    for (int s2 = 0; s2 < kMaxSplits; s2++) {
        const bool live = (uint32_t)s2 < eff;
        ms[s2] = live ? __ldcg(all + s2 * (hd + 2)) : -FLT_MAX;
        ls[s2] = live ? __ldcg(all + s2 * (hd + 2) + 1) : 0.f;
        os[s2] = (live && threadIdx.x < hd) ? __ldcg(all + s2 * (hd + 2) + 2 + threadIdx.x) : 0.f;
    }
    float M = -FLT_MAX;
#pragma unroll
    for (int s2 = 0; s2 < kMaxSplits; s2++) M = fmaxf(M, ms[s2]);
    float L = 0.f, O = 0.f;
#pragma unroll
    for (int s2 = 0; s2 < kMaxSplits; s2++) {
        const float w = ls[s2] > 0.f ? expf(ms[s2] - M) : 0.f;  // empty split: no weight
        L = fmaf(ls[s2], w, L);
        O = fmaf(os[s2], w, O);
    }
    if (threadIdx.x < hd) p.out[(size_t)head * hd + threadIdx.x] = O * (1.0f / L);
    if (threadIdx.x == 0) p.tickets[head] = 0;  // ready for the next launch on this stream
}


// ── grouped-query variant ───────────────────────────────────────────────────────────────────
// Grid (n_kv_heads, n_splits): CTA (kv, s) serves all GROUP query heads that share KV head kv, so a
// K or V row leaves HBM once per token instead of once per query head.  Scores: eight lanes per
// position, each lane reading 16 contiguous bytes per step, so one load instruction of a warp covers
// four rows in whole 128-byte lines.  Up to 64 splits keep every SM busy at long contexts; the last
// CTA of a KV head (ticket) merges the splits of its GROUP heads.
constexpr int kGqaMaxSplits = 64;

// Tensor parallelism: element o of this rank's slice of the attention output as a (value, epoch) pair into
// every rank's pair buffer, one 8-byte store each (the reader polls the pairs; see TpFuse).
__device__ __noinline__ void tp_push_value(const TpFuse &tp, size_t o, float v) {
    const uint32_t epoch = *tp.tick * tp.epochs_per_tick + tp.push_index + 1u;
    for (uint32_t pp = 0; pp < tp.world; pp++)
        asm volatile("st.volatile.global.v2.u32 [%0], {%1, %2};" ::"l"(tp.pair_out[pp] + o), "r"(__float_as_uint(v)), "r"(epoch) : "memory");
}

// TP = true only for launches of a tensor-parallel runner that also push (value, epoch) pairs.
template <int GROUP, int HD, bool TP>
__global__ void __launch_bounds__(kThreads) attn_decode_gqa_kernel(const __grid_constant__ AttnParams p) {
    constexpr int J = HD / 32;                               // 16-byte steps per lane and row
    constexpr int GH = (GROUP * J > 16) ? (16 / J) : GROUP;  // query heads scored per pass over K
    constexpr int HD4 = HD / 4;
    constexpr int NSL = kThreads / HD4;                      // position slices of the V pass
    constexpr int NOUT = (GROUP * HD + kThreads - 1) / kThreads;
    extern __shared__ __align__(16) float sm[];
    __shared__ uint32_t s_last;
    yule_pdl_launch_dependents();
    yule_pdl_wait();

    const uint32_t kvh = blockIdx.x, split = blockIdx.y, head0 = kvh * GROUP;
    // prefill: query z of the launch sits z positions further on and has its own rows and scratch
    const uint32_t z = blockIdx.z;
    const uint32_t pos = p.pos_ptr ? (p.pos_per_query ? p.pos_ptr[z] : *p.pos_ptr) : p.seq_len - 1 + z;
    float *const k_cache = p.k_cache + (size_t)z * p.kv_batch_stride;
    float *const v_cache = p.v_cache + (size_t)z * p.kv_batch_stride;
    const float *q_in = p.q + (size_t)z * p.q_stride;
    float *out_z = p.out + (size_t)z * p.out_stride;
    float *scratch_z = p.scratch + (size_t)z * p.n_heads * p.n_splits * (HD + 2);
    uint32_t *tickets_z = p.tickets + (size_t)z * p.n_heads;
    const uint32_t seq = pos + 1;
    const bool fused = p.k_new != nullptr;
    // Sliding window: the reference masks positions t < pos − window to −inf once pos >= window; they then carry
    // no weight, so the splits simply cover [begin, seq) instead of [0, seq).  With an attention softcap as well
    // the reference caps after masking (model_runner.rs:688-721), and cap·tanh(−inf / cap) is −cap, a finite
    // score: masked positions then keep a (small) weight, so they are visited and given exactly that score.
    const uint32_t first_visible = (p.window && pos >= p.window) ? pos - p.window : 0;
    const uint32_t begin = p.softcap != 0.f ? 0u : first_visible;
    const uint32_t span = seq - begin;
    uint32_t eff = (span + p.min_chunk - 1) / p.min_chunk;
    eff = eff < 1 ? 1 : (eff > p.n_splits ? p.n_splits : eff);
    if (split >= eff) return;
    const uint32_t chunk = (span + eff - 1) / eff;
    const uint32_t lo = begin + (split * chunk < span ? split * chunk : span);
    const uint32_t hi = lo + chunk < seq ? lo + chunk : seq;
    const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5;

    float *qs = sm;                               // GROUP × HD rotated queries
    float *kcur = qs + GROUP * HD;                // HD: rotated K row of the current token
    float *ml = kcur + HD;                        // (max, sum) per head, 16 floats
    float *scores = ml + 16;                      // GROUP × max_chunk
    float *partial = scores + (size_t)GROUP * p.max_chunk;  // NSL × GROUP × HD
    float *mrg = partial + (size_t)NSL * GROUP * HD;        // merge: 2 × GROUP × kGqaMaxSplits

    // The first K tile does not depend on the query: its loads go out before the RoPE prologue.
    const int qtr = lane >> 3, l8 = lane & 7;
    auto k_row = [&](uint32_t tb) {
        const uint32_t t = tb + wid * 4 + qtr;
        return k_cache + (size_t)(t < hi ? t : lo) * p.kv_stride + (size_t)kvh * HD + l8 * 4;
    };
    float4 kv_next[J];
    if (lo < hi) {
        const float *kp = k_row(lo);
#pragma unroll
        for (int j = 0; j < J; j++) kv_next[j] = *reinterpret_cast<const float4 *>(kp + j * 32);
    }

    // RoPE as in apply_rope (model_runner.rs:277-293): products and sums rounded separately
    for (uint32_t idx = threadIdx.x; idx < GROUP * (HD / 2); idx += kThreads) {
        const uint32_t h = idx / (HD / 2), i = idx % (HD / 2);
        float q0 = q_in[(size_t)(head0 + h) * HD + 2 * i], q1 = q_in[(size_t)(head0 + h) * HD + 2 * i + 1];
        if (p.cos_table) {
            const float c = p.cos_table[(size_t)pos * (HD / 2) + i], sn = p.sin_table[(size_t)pos * (HD / 2) + i];
            const float r0 = __fsub_rn(__fmul_rn(q0, c), __fmul_rn(q1, sn));
            const float r1 = __fadd_rn(__fmul_rn(q0, sn), __fmul_rn(q1, c));
            q0 = r0;
            q1 = r1;
            if (fused && h == 0) {
                const float k0 = p.k_new[(size_t)kvh * HD + 2 * i], k1 = p.k_new[(size_t)kvh * HD + 2 * i + 1];
                kcur[2 * i] = __fsub_rn(__fmul_rn(k0, c), __fmul_rn(k1, sn));
                kcur[2 * i + 1] = __fadd_rn(__fmul_rn(k0, sn), __fmul_rn(k1, c));
            }
        } else if (fused && h == 0) {
            kcur[2 * i] = p.k_new[(size_t)kvh * HD + 2 * i];
            kcur[2 * i + 1] = p.k_new[(size_t)kvh * HD + 2 * i + 1];
        }
        qs[h * HD + 2 * i] = q0;
        qs[h * HD + 2 * i + 1] = q1;
    }
    __syncthreads();

    // the split that owns the current position appends the new K and V rows (readers of this launch
    // take that row from kcur / v_new, never from the cache)
    if (fused && pos >= lo && pos < hi) {
        for (uint32_t d = threadIdx.x; d < HD; d += kThreads) {
            k_cache[(size_t)pos * p.kv_stride + (size_t)kvh * HD + d] = kcur[d];
            v_cache[(size_t)pos * p.kv_stride + (size_t)kvh * HD + d] = p.v_new[(size_t)kvh * HD + d];
        }
    }

    // scores; the loads of tile i+1 are in flight while tile i is multiplied
    const float scale = 1.0f / sqrtf((float)HD);
#pragma unroll 1
    for (int h0 = 0; h0 < GROUP; h0 += GH) {
        float4 qr[GH][J];
#pragma unroll
        for (int h = 0; h < GH; h++)
#pragma unroll
            for (int j = 0; j < J; j++) qr[h][j] = *reinterpret_cast<const float4 *>(qs + (h0 + h) * HD + j * 32 + l8 * 4);
        if (h0 > 0 && lo < hi) {
            const float *kp = k_row(lo);
#pragma unroll
            for (int j = 0; j < J; j++) kv_next[j] = *reinterpret_cast<const float4 *>(kp + j * 32);
        }
        for (uint32_t tb = lo; tb < hi; tb += 32) {
            const uint32_t t = tb + wid * 4 + qtr;
            const bool valid = t < hi;
            float4 kv[J];
#pragma unroll
            for (int j = 0; j < J; j++) kv[j] = kv_next[j];
            if (tb + 32 < hi) {
                const float *kp = k_row(tb + 32);
#pragma unroll
                for (int j = 0; j < J; j++) kv_next[j] = *reinterpret_cast<const float4 *>(kp + j * 32);
            }
            if (fused && t == pos) {
#pragma unroll
                for (int j = 0; j < J; j++) kv[j] = *reinterpret_cast<const float4 *>(kcur + j * 32 + l8 * 4);
            }
            float d[GH];
#pragma unroll
            for (int h = 0; h < GH; h++) {
                float a0 = 0.f, a1 = 0.f;
#pragma unroll
                for (int j = 0; j < J; j++) {
                    a0 = fmaf(qr[h][j].x, kv[j].x, a0);
                    a1 = fmaf(qr[h][j].y, kv[j].y, a1);
                    a0 = fmaf(qr[h][j].z, kv[j].z, a0);
                    a1 = fmaf(qr[h][j].w, kv[j].w, a1);
                }
                d[h] = a0 + a1;
            }
#pragma unroll
            for (int h = 0; h < GH; h++) {
                d[h] += __shfl_xor_sync(0xffffffffu, d[h], 4);
                d[h] += __shfl_xor_sync(0xffffffffu, d[h], 2);
                d[h] += __shfl_xor_sync(0xffffffffu, d[h], 1);
            }
            if (valid && l8 == 0) {
#pragma unroll
                for (int h = 0; h < GH; h++) {
                    float sc = d[h] * scale;
                    if (p.softcap != 0.f) sc = t < first_visible ? -p.softcap : p.softcap * tanhf(sc / p.softcap);
                    scores[(size_t)(h0 + h) * p.max_chunk + (t - lo)] = sc;
                }
            }
        }
    }
    __syncthreads();

    // softmax statistics: one warp per head
    for (int h = wid; h < GROUP; h += kThreads / 32) {
        float *sc = scores + (size_t)h * p.max_chunk;
        float mx = -FLT_MAX;
        for (uint32_t i = lane; i < hi - lo; i += 32) mx = fmaxf(mx, sc[i]);
        mx = warp_max(mx);
        float sum = 0.f;
        for (uint32_t i = lane; i < hi - lo; i += 32) {
            const float e = expf(sc[i] - mx);
            sc[i] = e;
            sum += e;
        }
        sum = warp_sum(sum);
        if (lane == 0) {
            ml[2 * h] = mx;
            ml[2 * h + 1] = sum;
        }
    }
    __syncthreads();

    // Σ_t e_t · V[t] for all GROUP heads from one read of V
    const uint32_t d4 = threadIdx.x % HD4, slice = threadIdx.x / HD4;
    float4 acc[GROUP];
#pragma unroll
    for (int h = 0; h < GROUP; h++) acc[h] = make_float4(0.f, 0.f, 0.f, 0.f);
    auto v_row = [&](uint32_t t) {
        return (fused && t == pos) ? reinterpret_cast<const float4 *>(p.v_new + (size_t)kvh * HD) + d4
                                   : reinterpret_cast<const float4 *>(v_cache + (size_t)t * p.kv_stride + (size_t)kvh * HD) + d4;
    };
    uint32_t t = lo + slice;
    for (; t + 3 * NSL < hi; t += 4 * NSL) {  // four rows in flight
        float4 v[4];
#pragma unroll
        for (int u = 0; u < 4; u++) v[u] = *v_row(t + u * NSL);
#pragma unroll
        for (int u = 0; u < 4; u++)
#pragma unroll
            for (int h = 0; h < GROUP; h++) {
                const float e = scores[(size_t)h * p.max_chunk + (t + u * NSL - lo)];
                acc[h].x = fmaf(e, v[u].x, acc[h].x);
                acc[h].y = fmaf(e, v[u].y, acc[h].y);
                acc[h].z = fmaf(e, v[u].z, acc[h].z);
                acc[h].w = fmaf(e, v[u].w, acc[h].w);
            }
    }
    for (; t < hi; t += NSL) {
        const float4 v = *v_row(t);
#pragma unroll
        for (int h = 0; h < GROUP; h++) {
            const float e = scores[(size_t)h * p.max_chunk + (t - lo)];
            acc[h].x = fmaf(e, v.x, acc[h].x);
            acc[h].y = fmaf(e, v.y, acc[h].y);
            acc[h].z = fmaf(e, v.z, acc[h].z);
            acc[h].w = fmaf(e, v.w, acc[h].w);
        }
    }
#pragma unroll
    for (int h = 0; h < GROUP; h++) reinterpret_cast<float4 *>(partial)[((size_t)slice * GROUP + h) * HD4 + d4] = acc[h];
    __syncthreads();
    float o[NOUT];
#pragma unroll
    for (int k = 0; k < NOUT; k++) {
        const uint32_t idx = threadIdx.x + k * kThreads;  // (head, dimension)
        o[k] = 0.f;
        if (idx < GROUP * HD) {
            const uint32_t h = idx / HD, dd = idx % HD;
            for (uint32_t s2 = 0; s2 < NSL; s2++) o[k] += partial[((size_t)s2 * GROUP + h) * HD + dd];
        }
    }

    if (eff == 1) {
#pragma unroll
        for (int k = 0; k < NOUT; k++) {
            const uint32_t idx = threadIdx.x + k * kThreads;
            if (idx < GROUP * HD) {
                const float val = o[k] * (1.0f / ml[2 * (idx / HD) + 1]);
                out_z[(size_t)head0 * HD + idx] = val;
                if (TP && p.tp.push) tp_push_value(p.tp, (size_t)head0 * HD + idx, val);
            }
        }
        return;
    }

    // publish (m, l, acc) per head, take a ticket; the last CTA of this KV head merges.
    // Scratch: accumulators [head][split][HD], then the (m, l) pairs [head][split][2].
    float *stats = scratch_z + (size_t)p.n_heads * p.n_splits * HD;
#pragma unroll
    for (int k = 0; k < NOUT; k++) {
        const uint32_t idx = threadIdx.x + k * kThreads;
        if (idx < GROUP * HD) {
            const uint32_t h = idx / HD, dd = idx % HD;
            scratch_z[((size_t)(head0 + h) * p.n_splits + split) * HD + dd] = o[k];
        }
    }
    if (threadIdx.x < GROUP) {
        float *mine = stats + ((size_t)(head0 + threadIdx.x) * p.n_splits + split) * 2;
        mine[0] = lo < hi ? ml[2 * threadIdx.x] : -FLT_MAX;
        mine[1] = lo < hi ? ml[2 * threadIdx.x + 1] : 0.f;
    }
    __threadfence();
    __syncthreads();
    if (threadIdx.x == 0) s_last = (atomicAdd(&tickets_z[kvh], 1u) == eff - 1) ? 1u : 0u;
    __syncthreads();
    if (!s_last) return;
    __threadfence();
    // (m, l) of every (head, split): one load per thread, then the weights exp(m - M) in shared memory
    float *mm = mrg, *ww = mrg + GROUP * kGqaMaxSplits;
    for (uint32_t i = threadIdx.x; i < GROUP * eff; i += kThreads) {
        const uint32_t h = i / eff, s2 = i % eff;
        const float2 st = __ldcg(reinterpret_cast<const float2 *>(stats + ((size_t)(head0 + h) * p.n_splits + s2) * 2));
        mm[h * kGqaMaxSplits + s2] = st.x;
        ww[h * kGqaMaxSplits + s2] = st.y;
    }
    __syncthreads();
    if (threadIdx.x < GROUP) {
        const uint32_t h = threadIdx.x;
        float M = -FLT_MAX;
        for (uint32_t s2 = 0; s2 < eff; s2++) M = fmaxf(M, mm[h * kGqaMaxSplits + s2]);
        float L = 0.f;
        for (uint32_t s2 = 0; s2 < eff; s2++) {
            const float l = ww[h * kGqaMaxSplits + s2];
            const float w = l > 0.f ? expf(mm[h * kGqaMaxSplits + s2] - M) : 0.f;  // empty split: no weight
            L = fmaf(l, w, L);
            ww[h * kGqaMaxSplits + s2] = w;
        }
        ml[2 * h + 1] = L;
    }
    __syncthreads();
    // Weighted sum of the splits' accumulators: thread (slice, head, d4) takes splits slice,
    // slice + MS, … as 16-byte loads, sixteen in flight; the slices meet in shared memory.
    constexpr int NV = GROUP * HD4;                         // float4 outputs of this KV head
    constexpr int MS = NV >= kThreads ? 1 : kThreads / NV;  // split slices
    constexpr int NVT = (NV + kThreads - 1) / kThreads;     // outputs per thread when MS == 1
    float4 *red4 = reinterpret_cast<float4 *>(partial);     // MS × NV float4 (fits: MS·NV ≤ max(NV, 256))
#pragma unroll
    for (int k = 0; k < NVT; k++) {
        const uint32_t vi = (threadIdx.x % (MS > 1 ? NV : kThreads)) + k * kThreads;
        const uint32_t msl = MS > 1 ? threadIdx.x / NV : 0;
        if (vi < (uint32_t)NV) {
            const uint32_t h = vi / HD4, c4 = vi % HD4;
            const float4 *src = reinterpret_cast<const float4 *>(scratch_z + (size_t)(head0 + h) * p.n_splits * HD) + c4;
            const float *wh = ww + h * kGqaMaxSplits;
            float4 O = make_float4(0.f, 0.f, 0.f, 0.f);
            uint32_t s2 = msl;
            for (; s2 + 15 * MS < eff; s2 += 16 * MS) {
                float4 v[16];
#pragma unroll
                for (int u = 0; u < 16; u++) v[u] = __ldcg(src + (size_t)(s2 + u * MS) * HD4);
#pragma unroll
                for (int u = 0; u < 16; u++) {
                    const float w = wh[s2 + u * MS];
                    O.x = fmaf(v[u].x, w, O.x);
                    O.y = fmaf(v[u].y, w, O.y);
                    O.z = fmaf(v[u].z, w, O.z);
                    O.w = fmaf(v[u].w, w, O.w);
                }
            }
            for (; s2 < eff; s2 += MS) {
                const float4 v = __ldcg(src + (size_t)s2 * HD4);
                const float w = wh[s2];
                O.x = fmaf(v.x, w, O.x);
                O.y = fmaf(v.y, w, O.y);
                O.z = fmaf(v.z, w, O.z);
                O.w = fmaf(v.w, w, O.w);
            }
            red4[(size_t)msl * NV + vi] = O;
        }
    }
    __syncthreads();
    for (uint32_t vi = threadIdx.x; vi < (uint32_t)NV; vi += kThreads) {
        float4 O = red4[vi];
        for (int m2 = 1; m2 < MS; m2++) {
            const float4 v = red4[(size_t)m2 * NV + vi];
            O.x += v.x;
            O.y += v.y;
            O.z += v.z;
            O.w += v.w;
        }
        const float inv = 1.0f / ml[2 * (vi / HD4) + 1];
        const float4 res = make_float4(O.x * inv, O.y * inv, O.z * inv, O.w * inv);
        reinterpret_cast<float4 *>(out_z + (size_t)head0 * HD)[vi] = res;
        if (TP && p.tp.push) {
            const size_t o0 = (size_t)head0 * HD + 4 * (size_t)vi;
            tp_push_value(p.tp, o0, res.x);
            tp_push_value(p.tp, o0 + 1, res.y);
            tp_push_value(p.tp, o0 + 2, res.z);
            tp_push_value(p.tp, o0 + 3, res.w);
        }
    }
    if (threadIdx.x == 0) tickets_z[kvh] = 0;  // ready for the next launch on this stream
}

template <int GROUP, int HD>
cudaError_t launch_gqa_variant(const AttnParams &p, size_t smem, bool pdl, cudaStream_t s, uint32_t n_tokens = 1) {
    auto kern = p.tp.push ? attn_decode_gqa_kernel<GROUP, HD, true> : attn_decode_gqa_kernel<GROUP, HD, false>;
    if (smem > 48 * 1024) {
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return e;
    }
    return launch_kernel(kern, dim3(p.n_kv_heads, p.n_splits, n_tokens), dim3(kThreads), smem, s, pdl, p);
}

}  // namespace

size_t attn_scratch_floats(uint32_t n_heads, uint32_t n_splits, uint32_t hd) {
    return (size_t)n_heads * n_splits * (hd + 2);
}

uint32_t attn_pick_splits(uint32_t n_heads, uint32_t seq_len_hint, int sm_count) {
    uint32_t s = (2u * (uint32_t)sm_count) / (n_heads ? n_heads : 1);
    s = s < 1 ? 1 : (s > 16 ? 16 : s);
    const uint32_t by_len = (seq_len_hint + kThreads - 1) / kThreads;  // at least 256 positions per split
    if (by_len < s) s = by_len < 1 ? 1 : by_len;
    return s;
}

bool attn_gqa_supported(uint32_t hd, uint32_t n_heads, uint32_t n_kv_heads) {
    if (!n_kv_heads || n_heads % n_kv_heads) return false;
    const uint32_t g = n_heads / n_kv_heads;
    return (hd == 64 || hd == 128) && (g == 1 || g == 2 || g == 4 || g == 8);
}

// Splits for the grouped-query kernel: one wave of CTAs, at least 32 positions each at the longest
// context, at most 64.
uint32_t attn_gqa_pick_splits(uint32_t n_kv_heads, uint32_t max_seq_len, int sm_count) {
    uint32_t s = (2u * (uint32_t)sm_count) / (n_kv_heads ? n_kv_heads : 1);  // one wave at two CTAs per SM
    const uint32_t by_len = (max_seq_len + 31) / 32;
    if (by_len < s) s = by_len;
    return s < 1 ? 1 : (s > (uint32_t)kGqaMaxSplits ? (uint32_t)kGqaMaxSplits : s);
}

bool attn_decode_supported(uint32_t hd) { return hd % 4 == 0 && hd >= 4 && hd <= 256 && kThreads % (hd / 4) == 0; }

cudaError_t launch_attn_decode(const AttnDecode &a, cudaStream_t s, uint64_t *launches) {
    AttnParams p = {};
    p.q = a.q;
    p.k_new = a.k_new;
    p.v_new = a.v_new;
    p.k_cache = a.k_cache;
    p.v_cache = a.v_cache;
    p.cos_table = a.cos_table;
    p.sin_table = a.sin_table;
    p.pos_ptr = a.pos_ptr;
    p.seq_len = a.seq_len;
    p.out = a.out;
    p.scratch = a.scratch;
    p.tickets = a.tickets;
    p.hd = a.hd;
    p.n_heads = a.n_heads;
    p.n_kv_heads = a.n_kv_heads;
    p.kv_stride = a.kv_stride;
    p.n_splits = a.n_splits;
    p.window = a.window;
    p.softcap = a.softcap;
    p.pos_per_query = a.pos_per_query ? 1u : 0u;
    p.kv_batch_stride = a.kv_batch_stride;
    if ((a.pos_per_query || a.kv_batch_stride) && !a.gqa) return cudaErrorInvalidValue;
    if (a.gqa) {
        if (!attn_gqa_supported(a.hd, a.n_heads, a.n_kv_heads) || a.n_splits > (uint32_t)kGqaMaxSplits) return cudaErrorInvalidValue;
        const uint32_t g = a.n_heads / a.n_kv_heads;
        uint32_t mc = (a.max_seq_len + a.n_splits - 1) / a.n_splits;
        p.min_chunk = a.min_chunk ? a.min_chunk : 32;
        if (mc < p.min_chunk) mc = p.min_chunk;
        p.max_chunk = ((mc + 3) / 4) * 4;
        const uint32_t nsl = kThreads / (a.hd / 4);
        const size_t smem = ((size_t)g * a.hd + a.hd + 16 + (size_t)g * p.max_chunk + (size_t)nsl * g * a.hd +
                             2 * (size_t)g * kGqaMaxSplits) * sizeof(float);
        if (smem > 200 * 1024) return cudaErrorInvalidValue;
        *launches += 1;
        p.q_stride = a.q_stride;
        p.out_stride = a.out_stride;
        p.tp = a.tp;
        // several queries per launch read the caches only; a device position is one per query then (batched decode)
        if (a.n_tokens > 1 && (a.k_new || (a.pos_ptr && !a.pos_per_query))) return cudaErrorInvalidValue;
#define YULE_GQA_CASE(G, H) if (g == G && a.hd == H) return launch_gqa_variant<G, H>(p, smem, a.pdl, s, a.n_tokens)
        YULE_GQA_CASE(1, 64); YULE_GQA_CASE(2, 64); YULE_GQA_CASE(4, 64); YULE_GQA_CASE(8, 64);
        YULE_GQA_CASE(1, 128); YULE_GQA_CASE(2, 128); YULE_GQA_CASE(4, 128); YULE_GQA_CASE(8, 128);
#undef YULE_GQA_CASE
        return cudaErrorInvalidValue;
    }
    // A split holds at most max(256, ceil(max_seq / n_splits)) scores (fewer, larger splits are only
    // used while they stay at 256 positions or less).  A multiple of 4 keeps the float4 area behind
    // the scores 16-byte aligned.
    uint32_t mc = (a.max_seq_len + a.n_splits - 1) / a.n_splits;
    p.min_chunk = a.min_chunk ? a.min_chunk : kThreads;
    if (mc < p.min_chunk) mc = p.min_chunk;
    p.max_chunk = ((mc + 3) / 4) * 4;
    const uint32_t n_slices = kThreads / (a.hd / 4);
    const size_t smem = ((size_t)2 * a.hd + p.max_chunk + (size_t)n_slices * a.hd) * sizeof(float);
    if (smem > 200 * 1024) return cudaErrorInvalidValue;
    if (smem > 48 * 1024) {
        cudaError_t e = cudaFuncSetAttribute(attn_decode_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return e;
    }
    *launches += 1;
    return launch_kernel(attn_decode_kernel, dim3(a.n_heads, a.n_splits), dim3(kThreads), smem, s, a.pdl, p);
}

}  // namespace yule

// ── allocation-free variant ─────────────────────────────────────────────────────────────────
// Some hosts cannot allocate device memory at call time: a process that sealed itself before
// inference (Yule applies a seccomp / Landlock / Job Object sandbox first, and the driver calls
// behind cudaMalloc may then be refused), an embedder running under a fixed device-memory budget it
// has already handed out, or a decode loop that may not take the allocator's lock.  For them the
// split-KV scratch lives in the library image itself: two file-scope __device__ arrays of a fixed,
// modest size that every GPU which loads the library holds until the process exits.

namespace yule {
namespace {

constexpr uint32_t kStaticMaxHeads = 128;
constexpr uint32_t kStaticMaxSplits = 16;
constexpr uint32_t kStaticMaxHeadDim = 256;
// 128 heads x 16 splits x (256 + 2) floats = 528 384 floats = 2.02 MiB, plus 512 bytes of tickets
constexpr size_t kStaticScratchFloats = (size_t)kStaticMaxHeads * kStaticMaxSplits * (kStaticMaxHeadDim + 2);

static __device__ __align__(256) float g_attn_static_scratch[kStaticScratchFloats];
static __device__ __align__(256) uint32_t g_attn_static_tickets[kStaticMaxHeads];

// In host code the two names above are only stand-ins; the device addresses come from
// cudaGetSymbolAddress, asked once per device with that device current.
struct StaticAddrs {
    float *scratch = nullptr;
    uint32_t *tickets = nullptr;
};
constexpr int kMaxDevices = 64;
StaticAddrs g_static_addrs[kMaxDevices];
std::mutex g_static_mu;

cudaError_t static_addresses(int device, StaticAddrs *out) {
    if (device < 0 || device >= kMaxDevices) return cudaErrorInvalidDevice;
    std::lock_guard<std::mutex> lock(g_static_mu);
    StaticAddrs &a = g_static_addrs[device];
    if (!a.scratch) {
        float *sp = nullptr;
        uint32_t *tp = nullptr;
        cudaError_t e = cudaGetSymbolAddress((void **)&sp, g_attn_static_scratch);
        if (e != cudaSuccess) return e;
        e = cudaGetSymbolAddress((void **)&tp, g_attn_static_tickets);
        if (e != cudaSuccess) return e;
        a.scratch = sp;
        a.tickets = tp;
    }
    *out = a;
    return cudaSuccess;
}

}  // namespace
}  // namespace yule

extern "C" int32_t yule_cuda_multihead_attention_static(yule_cuda_ctx *ctx, yule_buffer q, yule_buffer k_cache,
                                                        yule_buffer v_cache, yule_buffer out, uint32_t head_dim,
                                                        uint32_t seq_len, uint32_t n_heads, uint32_t n_kv_heads,
                                                        uint32_t kv_stride) {
    using namespace yule;
    if (!ctx) return fail(YULE_ERR_INVALID_ARGUMENT, "null context");
    YULE_CUDA_TRY(cudaSetDevice(ctx->device));
    if (n_kv_heads == 0 || n_heads == 0 || n_heads % n_kv_heads || head_dim == 0 || seq_len == 0)
        return fail(YULE_ERR_INVALID_ARGUMENT, "bad attention shape (heads %u, kv heads %u, head_dim %u, seq %u)", n_heads,
                    n_kv_heads, head_dim, seq_len);
    if (!attn_decode_supported(head_dim) || kv_stride % 4)
        return fail(YULE_ERR_INVALID_ARGUMENT,
                    "multihead_attention_static needs head_dim with 256 %% (head_dim / 4) == 0 and kv_stride %% 4 == 0 "
                    "(got head_dim %u, kv_stride %u)", head_dim, kv_stride);
    const uint32_t n_splits = attn_pick_splits(n_heads, seq_len, ctx->prop.multiProcessorCount);
    if (n_heads > kStaticMaxHeads || n_splits > kStaticMaxSplits || head_dim > kStaticMaxHeadDim ||
        attn_scratch_floats(n_heads, n_splits, head_dim) > kStaticScratchFloats)
        return fail(YULE_ERR_INVALID_ARGUMENT,
                    "multihead_attention_static: %u heads x head_dim %u exceeds the built-in scratch (at most %u heads, "
                    "head_dim %u, %zu floats); use yule_cuda_multihead_attention", n_heads, head_dim, kStaticMaxHeads,
                    kStaticMaxHeadDim, kStaticScratchFloats);
    Buffer Q, K, V, O;
    if (!ctx->find(q, &Q, "q") || !ctx->find(k_cache, &K, "k_cache") || !ctx->find(v_cache, &V, "v_cache") ||
        !ctx->find(out, &O, "out"))
        return YULE_ERR_UNKNOWN_BUFFER;
    const size_t kv_need = ((size_t)(seq_len - 1) * kv_stride + (size_t)n_kv_heads * head_dim) * 4;
    const size_t q_need = (size_t)n_heads * head_dim * 4;
    if (Q.size < q_need || O.size < q_need || K.size < kv_need || V.size < kv_need)
        return fail(YULE_ERR_OUT_OF_BOUNDS, "attention buffers too small for %u heads x %u over %u positions", n_heads,
                    head_dim, seq_len);
    StaticAddrs addrs;
    cudaError_t e = static_addresses(ctx->device, &addrs);
    if (e != cudaSuccess) return fail_cuda(e, "cudaGetSymbolAddress of the built-in attention scratch");
    // The array keeps whatever the last call left.  Partial results are fully rewritten before they
    // are read; the tickets must start at zero, so clear them (a failed earlier launch may not have).
    YULE_CUDA_TRY(cudaMemsetAsync(addrs.tickets, 0, (size_t)n_heads * sizeof(uint32_t), ctx->stream));
    AttnDecode a;
    a.q = (const float *)Q.ptr;
    a.k_cache = (float *)K.ptr;
    a.v_cache = (float *)V.ptr;
    a.seq_len = seq_len;
    a.out = (float *)O.ptr;
    a.scratch = addrs.scratch;
    a.tickets = addrs.tickets;
    a.hd = head_dim;
    a.n_heads = n_heads;
    a.n_kv_heads = n_kv_heads;
    a.kv_stride = kv_stride;
    a.n_splits = n_splits;
    a.max_seq_len = seq_len;
    uint64_t n = 0;
    e = launch_attn_decode(a, ctx->stream, &n);
    ctx->launches.fetch_add(n);
    if (e != cudaSuccess) return fail_cuda(e, "multihead_attention_static launch");
    return YULE_OK;
}

