// attn_gqa.cuh — the grouped-query split-KV decode attention as a device function, shared by the attention
// kernels (attention.cu) and the persistent decode kernel (decode_mega.cu).
// Include inside namespace yule { namespace { … } }.
#pragma once

#include "pair_wait.cuh"

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
    int *status;                         // bounded waits of the pair inputs (persistent decode kernel)
    long long wait_cycles;
};

// What differs between the units of work that share one AttnParams: the query of the launch (blockIdx.z) in the
// attention kernels, the layer in the persistent decode kernel.
struct AttnUnit {
    float *k_cache, *v_cache;
    uint32_t *tickets;   // [n_kv_heads] of this query, zero between uses
    float *scratch;      // split partials of this query
    const float *q_in;   // [n_heads][HD], or null when the inputs are pairs
    const uint2 *q_pairs, *k_pairs, *v_pairs;
    uint32_t in_epoch;
    uint32_t pos;
    unsigned long long *prof;  // timing aid of the persistent kernel (three stamps), or null
};

// ── grouped-query variant ───────────────────────────────────────────────────────────────────
// Grid (n_kv_heads, n_splits): CTA (kv, s) serves all GROUP query heads that share KV head kv, so a
// K or V row leaves HBM once per token instead of once per query head.  Scores: eight lanes per
// position, each lane reading 16 contiguous bytes per step, so one load instruction of a warp covers
// four rows in whole 128-byte lines.  Up to 64 splits keep every SM busy at long contexts; the last
// CTA of a KV head (ticket) merges the splits of its GROUP heads.
constexpr int kGqaMaxSplits = 64;

// The end of a unit: `o` holds this split's unnormalised output sums (element tid + k·kThreads of the
// [GROUP][HD] block of this KV head), `ml` (shared memory) its (max, Σexp) per head.  One split: normalise and store.
// Several: publish (sums, max, Σexp), take a ticket; the last unit of the KV head merges all splits and stores.
//   work  shared memory: max(GROUP·HD/4, kThreads) float4 for the merge, then 2·GROUP·kGqaMaxSplits floats
template <int GROUP, int HD, class Sync, class Store>
__device__ __forceinline__ void attn_gqa_finish(const AttnParams &p, float *scratch_z, uint32_t *tickets_z, uint32_t kvh, uint32_t split,
                                                uint32_t eff, bool nonempty, uint32_t tid, const float (&o)[(GROUP * HD + kThreads - 1) / kThreads],
                                                float *ml, float *work, uint32_t *s_last, Sync sync, Store store) {
    constexpr int HD4 = HD / 4;
    constexpr int NOUT = (GROUP * HD + kThreads - 1) / kThreads;
    const uint32_t head0 = kvh * GROUP;
    float *partial = work;
    float *mrg = work + 4 * (GROUP * HD4 > kThreads ? GROUP * HD4 : kThreads);
    if (eff == 1) {
#pragma unroll
        for (int k = 0; k < NOUT; k++) {
            const uint32_t idx = tid + k * kThreads;
            if (idx < GROUP * HD) {
                const float val = o[k] * (1.0f / ml[2 * (idx / HD) + 1]);
                store((uint32_t)(head0 * HD + idx), val);
            }
        }
        return;
    }

    // publish (m, l, acc) per head, take a ticket; the last CTA of this KV head merges.
    // Scratch: accumulators [head][split][HD], then the (m, l) pairs [head][split][2].
    float *stats = scratch_z + (size_t)p.n_heads * p.n_splits * HD;
#pragma unroll
    for (int k = 0; k < NOUT; k++) {
        const uint32_t idx = tid + k * kThreads;
        if (idx < GROUP * HD) {
            const uint32_t h = idx / HD, dd = idx % HD;
            scratch_z[((size_t)(head0 + h) * p.n_splits + split) * HD + dd] = o[k];
        }
    }
    if (tid < GROUP) {
        float *mine = stats + ((size_t)(head0 + tid) * p.n_splits + split) * 2;
        mine[0] = nonempty ? ml[2 * tid] : -FLT_MAX;
        mine[1] = nonempty ? ml[2 * tid + 1] : 0.f;
    }
    __threadfence();
    sync();
    if (tid == 0) *s_last = (atomicAdd(&tickets_z[kvh], 1u) == eff - 1) ? 1u : 0u;
    sync();
    if (!*s_last) return;
    __threadfence();
    // (m, l) of every (head, split): one load per thread, then the weights exp(m - M) in shared memory
    float *mm = mrg, *ww = mrg + GROUP * kGqaMaxSplits;
    for (uint32_t i = tid; i < GROUP * eff; i += kThreads) {
        const uint32_t h = i / eff, s2 = i % eff;
        const float2 st = __ldcg(reinterpret_cast<const float2 *>(stats + ((size_t)(head0 + h) * p.n_splits + s2) * 2));
        mm[h * kGqaMaxSplits + s2] = st.x;
        ww[h * kGqaMaxSplits + s2] = st.y;
    }
    sync();
    if (tid < GROUP) {
        const uint32_t h = tid;
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
    sync();
    // Weighted sum of the splits' accumulators: thread (slice, head, d4) takes splits slice,
    // slice + MS, … as 16-byte loads, sixteen in flight; the slices meet in shared memory.
    constexpr int NV = GROUP * HD4;                         // float4 outputs of this KV head
    constexpr int MS = NV >= kThreads ? 1 : kThreads / NV;  // split slices
    constexpr int NVT = (NV + kThreads - 1) / kThreads;     // outputs per thread when MS == 1
    float4 *red4 = reinterpret_cast<float4 *>(partial);     // MS × NV float4 (fits: MS·NV ≤ max(NV, 256))
#pragma unroll
    for (int k = 0; k < NVT; k++) {
        const uint32_t vi = (tid % (MS > 1 ? NV : kThreads)) + k * kThreads;
        const uint32_t msl = MS > 1 ? tid / NV : 0;
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
    sync();
    for (uint32_t vi = tid; vi < (uint32_t)NV; vi += kThreads) {
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
        const uint32_t o0 = head0 * HD + 4 * vi;
        store(o0, res.x);
        store(o0 + 1, res.y);
        store(o0 + 2, res.z);
        store(o0 + 3, res.w);
    }
    if (tid == 0) tickets_z[kvh] = 0;  // ready for the next launch on this stream
}
// One (KV head, split) unit of work, by 256 threads (`tid` 0..255) that can meet at `sync()`.
//   PAIRS  the query and the new K / V rows arrive as (value, epoch) pairs that are polled (persistent decode
//          kernel); otherwise they are plain floats written by an earlier kernel.
//   sm     dynamic shared memory of the unit (attn_gqa_smem_floats), s_last one more word
//   store  store(i, v): element i of the [n_heads][HD] output of this query
template <int GROUP, int HD, bool PAIRS, class Sync, class Store>
__device__ __forceinline__ void attn_gqa_unit(const AttnParams &p, const AttnUnit &au, uint32_t kvh, uint32_t split, uint32_t tid,
                                              float *sm, uint32_t *s_last, Sync sync, Store store) {
    constexpr int J = HD / 32;                               // 16-byte steps per lane and row
    // query heads scored per pass over K: 16 float4 of queries in registers, 8 inside the persistent kernel (which
    // has 128 registers per thread for everything and a tiny L1 behind its shared-memory carve-out: it must not spill)
    constexpr int QREGS = PAIRS ? 8 : 16;
    constexpr int GH = (GROUP * J > QREGS) ? (QREGS / J) : GROUP;
    constexpr int HD4 = HD / 4;
    constexpr int NSL = kThreads / HD4;                      // position slices of the V pass
    constexpr int NOUT = (GROUP * HD + kThreads - 1) / kThreads;
    const uint32_t head0 = kvh * GROUP;
    const uint32_t pos = au.pos;
    float *const k_cache = au.k_cache;
    float *const v_cache = au.v_cache;
    const float *q_in = au.q_in;
    float *scratch_z = au.scratch;
    uint32_t *tickets_z = au.tickets;
    const uint32_t seq = pos + 1;
    const bool fused = PAIRS || p.k_new != nullptr;
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
    const int lane = tid & 31, wid = tid >> 5;

    float *qs = sm;                               // GROUP × HD rotated queries
    float *kcur = qs + GROUP * HD;                // HD: rotated K row of the current token
    float *vcur = kcur + HD;                      // HD: V row of the current token
    float *ml = vcur + HD;                        // (max, sum) per head, 16 floats
    float *scores = ml + 16;                      // GROUP × max_chunk
    float *partial = scores + (size_t)GROUP * p.max_chunk;  // NSL × GROUP × HD
    // (the merge of attn_gqa_finish works in `partial` and the 2 × GROUP × kGqaMaxSplits floats behind it)

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

    // RoPE as in apply_rope (model_runner.rs:277-293): products and sums rounded separately.
    // Pair inputs: every load of this thread goes out before the first one is checked (an L2 round trip each).
    constexpr int QIT = (GROUP * (HD / 2) + kThreads - 1) / kThreads;
    uint2 pq[QIT][2] = {}, pk[2] = {}, pv = {};
    // the rotation of this thread's pairs: plain loads, asked for before the polled ones (which nothing may overtake)
    float rot_c[QIT], rot_s[QIT];
#pragma unroll
    for (int it = 0; it < QIT; it++) {
        const uint32_t idx = tid + it * kThreads;
        rot_c[it] = 1.f;
        rot_s[it] = 0.f;
        if (p.cos_table && idx < GROUP * (HD / 2)) {
            rot_c[it] = p.cos_table[(size_t)pos * (HD / 2) + idx % (HD / 2)];
            rot_s[it] = p.sin_table[(size_t)pos * (HD / 2) + idx % (HD / 2)];
        }
    }
    if (PAIRS) {
#pragma unroll
        for (int it = 0; it < QIT; it++) {
            const uint32_t idx = tid + it * kThreads;
            if (idx < GROUP * (HD / 2)) {
                pq[it][0] = pair_peek(au.q_pairs + (size_t)head0 * HD + 2 * idx);
                pq[it][1] = pair_peek(au.q_pairs + (size_t)head0 * HD + 2 * idx + 1);
            }
        }
        if (tid < HD / 2) {
            pk[0] = pair_peek(au.k_pairs + (size_t)kvh * HD + 2 * tid);
            pk[1] = pair_peek(au.k_pairs + (size_t)kvh * HD + 2 * tid + 1);
        }
        if (tid < HD) pv = pair_peek(au.v_pairs + (size_t)kvh * HD + tid);
    }
    auto k_at = [&](size_t i) {
        if (!PAIRS) return p.k_new[i];
        return pair_settle(pk[i & 1], au.k_pairs + i, au.in_epoch, p.status, p.wait_cycles);  // i = kvh·HD + 2·tid + {0, 1}
    };
    auto v_at = [&](size_t i) {
        if (!PAIRS) return p.v_new[i];
        return pair_settle(pv, au.v_pairs + i, au.in_epoch, p.status, p.wait_cycles);  // i = kvh·HD + tid
    };
#pragma unroll
    for (int it = 0; it < QIT; it++) {
        const uint32_t idx = tid + it * kThreads;
        if (idx >= GROUP * (HD / 2)) break;
        const uint32_t h = idx / (HD / 2), i = idx % (HD / 2);
        const size_t qi = (size_t)(head0 + h) * HD + 2 * i;
        float q0 = PAIRS ? pair_settle(pq[it][0], au.q_pairs + qi, au.in_epoch, p.status, p.wait_cycles) : q_in[qi];
        float q1 = PAIRS ? pair_settle(pq[it][1], au.q_pairs + qi + 1, au.in_epoch, p.status, p.wait_cycles) : q_in[qi + 1];
        if (p.cos_table) {
            const float c = rot_c[it], sn = rot_s[it];
            const float r0 = __fsub_rn(__fmul_rn(q0, c), __fmul_rn(q1, sn));
            const float r1 = __fadd_rn(__fmul_rn(q0, sn), __fmul_rn(q1, c));
            q0 = r0;
            q1 = r1;
            if (fused && h == 0) {
                const float k0 = k_at((size_t)kvh * HD + 2 * i), k1 = k_at((size_t)kvh * HD + 2 * i + 1);
                kcur[2 * i] = __fsub_rn(__fmul_rn(k0, c), __fmul_rn(k1, sn));
                kcur[2 * i + 1] = __fadd_rn(__fmul_rn(k0, sn), __fmul_rn(k1, c));
            }
        } else if (fused && h == 0) {
            kcur[2 * i] = k_at((size_t)kvh * HD + 2 * i);
            kcur[2 * i + 1] = k_at((size_t)kvh * HD + 2 * i + 1);
        }
        qs[h * HD + 2 * i] = q0;
        qs[h * HD + 2 * i + 1] = q1;
    }
    if (fused)
        for (uint32_t d = tid; d < HD; d += kThreads) vcur[d] = v_at((size_t)kvh * HD + d);
    sync();

    // the split that owns the current position appends the new K and V rows (readers of this launch
    // take that row from kcur / v_new, never from the cache)
    if (fused && pos >= lo && pos < hi) {
        for (uint32_t d = tid; d < HD; d += kThreads) {
            k_cache[(size_t)pos * p.kv_stride + (size_t)kvh * HD + d] = kcur[d];
            v_cache[(size_t)pos * p.kv_stride + (size_t)kvh * HD + d] = vcur[d];
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
    sync();

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
    sync();

    // Σ_t e_t · V[t] for all GROUP heads from one read of V
    const uint32_t d4 = tid % HD4, slice = tid / HD4;
    float4 acc[GROUP];
#pragma unroll
    for (int h = 0; h < GROUP; h++) acc[h] = make_float4(0.f, 0.f, 0.f, 0.f);
    auto v_row = [&](uint32_t t) {
        return (fused && t == pos) ? reinterpret_cast<const float4 *>(vcur) + d4
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
    sync();
    float o[NOUT];
#pragma unroll
    for (int k = 0; k < NOUT; k++) {
        const uint32_t idx = tid + k * kThreads;  // (head, dimension)
        o[k] = 0.f;
        if (idx < GROUP * HD) {
            const uint32_t h = idx / HD, dd = idx % HD;
            for (uint32_t s2 = 0; s2 < NSL; s2++) o[k] += partial[((size_t)s2 * GROUP + h) * HD + dd];
        }
    }

    attn_gqa_finish<GROUP, HD>(p, scratch_z, tickets_z, kvh, split, eff, lo < hi, tid, o, ml, partial, s_last, sync, store);
}

// ── the same unit with its keys and values staged in shared memory ──────────────────────────────────────────────
// For the persistent decode kernel, where a phase costs latency rather than bandwidth and registers are scarce.
// The K and V rows of the unit's positions are brought into shared memory by 16-byte asynchronous copies, all in
// flight at once and issued before the unit waits for its query (they do not depend on it); scores, soft-max and
// the weighted sum then run out of shared memory, C positions per pass, with a running (max, Σexp) across passes.
// Inputs are (value, epoch) pairs; plain Llama attention (no window, no soft-cap).  Splits, tickets, merge and
// output are those of attn_gqa_unit.
constexpr size_t attn_staged_smem_floats(int hpu, int hd) {
    const int c = 4096 / hd;
    const size_t front = (size_t)hpu * hd + 2 * hd + 32 + (size_t)hpu * c;
    const size_t kv = (size_t)c * (hd + 4) + (size_t)c * hd;
    const size_t nv = (size_t)hpu * hd / 4;
    const size_t work = 4 * (nv > (size_t)kThreads ? nv : (size_t)kThreads) + 2 * (size_t)hpu * kGqaMaxSplits;
    return front + (kv > work ? kv : work);
}

// A unit serves GROUP consecutive query heads (unit index `uh`: heads uh·GROUP …) that share KV head `kvh`; the
// persistent kernel uses GROUP = 1 (a unit per query head: at the contexts where a phase is latency-bound the
// passes of eight heads in one CTA cost more than reading the K / V rows, which sit in L2, eight times).
template <int GROUP, int HD, int NT, class SyncAll, class Sync, class Store>
__device__ __forceinline__ void attn_unit_staged(const AttnParams &p, const AttnUnit &au, uint32_t uh, uint32_t kvh, uint32_t split,
                                                 uint32_t tid, float *sm, uint32_t *s_last, SyncAll sync_all, Sync sync, Store store) {
    // NT threads (tid 0..NT-1, meeting at sync_all) run the passes; the first kThreads of them (meeting at sync)
    // publish / merge / store.
    constexpr int C = 4096 / HD;  // positions per pass
    constexpr int KP = HD + 4;    // row pitch of K in shared memory (floats): rows 16 bytes apart in bank terms
    constexpr int HD4 = HD / 4;
    constexpr int LP = NT / C;    // lanes per position in the score step, 8 dimensions each
    static_assert(LP * 8 == HD && LP <= 32, "eight dimensions per lane");
    constexpr int NOUT = (GROUP * HD + kThreads - 1) / kThreads;
    constexpr int NACC = (GROUP * HD + NT - 1) / NT;
    constexpr int QIT = (GROUP * (HD / 2) + NT - 1) / NT;
    const uint32_t head0 = uh * GROUP, pos = au.pos, seq = pos + 1;
    uint32_t eff = (seq + p.min_chunk - 1) / p.min_chunk;
    eff = eff < 1 ? 1 : (eff > p.n_splits ? p.n_splits : eff);
    if (split >= eff) return;
    const uint32_t chunk = (seq + eff - 1) / eff;
    const uint32_t lo = split * chunk < seq ? split * chunk : seq;
    const uint32_t hi = lo + chunk < seq ? lo + chunk : seq;
    const int lane = tid & 31, wid = tid >> 5;

    float *qs = sm;                  // GROUP × HD rotated queries
    float *kcur = qs + GROUP * HD;   // rotated K row of the current token
    float *vcur = kcur + HD;         // V row of the current token
    float *ml = vcur + HD;           // running (max, Σexp) per head
    float *alpha = ml + 16;          // rescale factor of the pass, per head
    float *sc = alpha + 16;          // GROUP × C scores, then weights
    float *Ks = sc + GROUP * C;      // C × KP
    float *Vs = Ks + C * KP;         // C × HD
    float *k_cache = au.k_cache, *v_cache = au.v_cache;

    // the rows of positions [p0, p0 + n) except the current one (which never comes from the cache)
    auto stage_rows = [&](uint32_t p0, uint32_t n) {
        for (uint32_t idx = tid; idx < n * HD4; idx += NT) {
            const uint32_t t = idx / HD4, j = idx % HD4;
            if (p0 + t == pos) continue;
            const size_t src = (size_t)(p0 + t) * p.kv_stride + (size_t)kvh * HD + 4 * j;
            asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"((uint32_t)__cvta_generic_to_shared(Ks + t * KP + 4 * j)),
                         "l"(k_cache + src)
                         : "memory");
            asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"((uint32_t)__cvta_generic_to_shared(Vs + t * HD + 4 * j)),
                         "l"(v_cache + src)
                         : "memory");
        }
        asm volatile("cp.async.commit_group;" ::: "memory");
    };
    if (lo < hi) stage_rows(lo, hi - lo < (uint32_t)C ? hi - lo : (uint32_t)C);

    // query and new K / V rows: rotation factors first (plain loads), then every pair load, then the checks
    float rot_c[QIT], rot_s[QIT];
    uint2 pq[QIT][2] = {}, pk[2] = {}, pv = {};
#pragma unroll
    for (int it = 0; it < QIT; it++) {
        const uint32_t idx = tid + it * NT;
        rot_c[it] = 1.f;
        rot_s[it] = 0.f;
        if (p.cos_table && idx < GROUP * (HD / 2)) {
            rot_c[it] = p.cos_table[(size_t)pos * (HD / 2) + idx % (HD / 2)];
            rot_s[it] = p.sin_table[(size_t)pos * (HD / 2) + idx % (HD / 2)];
        }
    }
#pragma unroll
    for (int it = 0; it < QIT; it++) {
        const uint32_t idx = tid + it * NT;
        if (idx < GROUP * (HD / 2)) {
            pq[it][0] = pair_peek(au.q_pairs + (size_t)head0 * HD + 2 * idx);
            pq[it][1] = pair_peek(au.q_pairs + (size_t)head0 * HD + 2 * idx + 1);
        }
    }
    if (tid < HD / 2) {
        pk[0] = pair_peek(au.k_pairs + (size_t)kvh * HD + 2 * tid);
        pk[1] = pair_peek(au.k_pairs + (size_t)kvh * HD + 2 * tid + 1);
    }
    // the V row is fetched by the threads at the far end, which have no query pair to fetch
    const uint32_t vt = NT - 1 - tid;
    if (vt < HD) pv = pair_peek(au.v_pairs + (size_t)kvh * HD + vt);
    // RoPE as in apply_rope (model_runner.rs:277-293): products and sums rounded separately
#pragma unroll
    for (int it = 0; it < QIT; it++) {
        const uint32_t idx = tid + it * NT;
        if (idx >= GROUP * (HD / 2)) break;
        const size_t qi = (size_t)head0 * HD + 2 * idx;
        const float q0 = pair_settle(pq[it][0], au.q_pairs + qi, au.in_epoch, p.status, p.wait_cycles);
        const float q1 = pair_settle(pq[it][1], au.q_pairs + qi + 1, au.in_epoch, p.status, p.wait_cycles);
        const float c = rot_c[it], sn = rot_s[it];
        qs[2 * idx] = __fsub_rn(__fmul_rn(q0, c), __fmul_rn(q1, sn));
        qs[2 * idx + 1] = __fadd_rn(__fmul_rn(q0, sn), __fmul_rn(q1, c));
        if (idx < HD / 2) {  // head 0 of the group: this thread also rotates the new K row
            const size_t ki = (size_t)kvh * HD + 2 * idx;
            const float k0 = pair_settle(pk[0], au.k_pairs + ki, au.in_epoch, p.status, p.wait_cycles);
            const float k1 = pair_settle(pk[1], au.k_pairs + ki + 1, au.in_epoch, p.status, p.wait_cycles);
            kcur[2 * idx] = __fsub_rn(__fmul_rn(k0, c), __fmul_rn(k1, sn));
            kcur[2 * idx + 1] = __fadd_rn(__fmul_rn(k0, sn), __fmul_rn(k1, c));
        }
    }
    if (vt < HD) vcur[vt] = pair_settle(pv, au.v_pairs + (size_t)kvh * HD + vt, au.in_epoch, p.status, p.wait_cycles);
    if (tid < GROUP) {
        ml[2 * tid] = -FLT_MAX;
        ml[2 * tid + 1] = 0.f;
    }
    sync_all();
    if (au.prof && tid == 0) asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(au.prof[1]));  // inputs settled
    // the split that owns the current position appends the new K and V rows
    if (pos >= lo && pos < hi) {
        for (uint32_t d = tid; d < HD; d += NT) {
            k_cache[(size_t)pos * p.kv_stride + (size_t)kvh * HD + d] = kcur[d];
            v_cache[(size_t)pos * p.kv_stride + (size_t)kvh * HD + d] = vcur[d];
        }
    }

    const float scale = 1.0f / sqrtf((float)HD);
    float acc[NACC];
#pragma unroll
    for (int k = 0; k < NACC; k++) acc[k] = 0.f;
    for (uint32_t p0 = lo; p0 < hi; p0 += C) {
        const uint32_t n = hi - p0 < (uint32_t)C ? hi - p0 : (uint32_t)C;
        if (p0 != lo) stage_rows(p0, n);
        asm volatile("cp.async.wait_group 0;" ::: "memory");
        if (pos >= p0 && pos < p0 + n)
            for (uint32_t d = tid; d < HD; d += NT) {
                Ks[(pos - p0) * KP + d] = kcur[d];
                Vs[(pos - p0) * HD + d] = vcur[d];
            }
        sync_all();
        // scores: LP lanes per position, eight dimensions each
        {
            const uint32_t tp = tid / LP, part = tid % LP;
            const float *kr = Ks + (tp < n ? tp : 0u) * KP + part * 8;
            const float4 k0 = *reinterpret_cast<const float4 *>(kr), k1 = *reinterpret_cast<const float4 *>(kr + 4);
#pragma unroll
            for (int h = 0; h < GROUP; h++) {
                const float *qr = qs + h * HD + part * 8;
                const float4 q0 = *reinterpret_cast<const float4 *>(qr), q1 = *reinterpret_cast<const float4 *>(qr + 4);
                float a0 = q0.x * k0.x, a1 = q0.y * k0.y;
                a0 = fmaf(q0.z, k0.z, a0);
                a1 = fmaf(q0.w, k0.w, a1);
                a0 = fmaf(q1.x, k1.x, a0);
                a1 = fmaf(q1.y, k1.y, a1);
                a0 = fmaf(q1.z, k1.z, a0);
                a1 = fmaf(q1.w, k1.w, a1);
                float dsum = a0 + a1;
#pragma unroll
                for (int o = 1; o < LP; o <<= 1) dsum += __shfl_xor_sync(0xffffffffu, dsum, o);
                if (part == 0 && tp < n) sc[h * C + tp] = dsum * scale;
            }
        }
        sync_all();
        // running soft-max: one warp per head
        for (int h = wid; h < GROUP; h += NT / 32) {
            float *s = sc + h * C;
            float mx = -FLT_MAX;
            for (uint32_t i = lane; i < n; i += 32) mx = fmaxf(mx, s[i]);
            mx = warp_max(mx);
            const float m_old = ml[2 * h], m_new = fmaxf(m_old, mx);
            float sum = 0.f;
            for (uint32_t i = lane; i < n; i += 32) {
                const float e = expf(s[i] - m_new);
                s[i] = e;
                sum += e;
            }
            sum = warp_sum(sum);
            if (lane == 0) {
                const float a = expf(m_old - m_new);  // 0 on the first pass
                alpha[h] = a;
                ml[2 * h] = m_new;
                ml[2 * h + 1] = fmaf(ml[2 * h + 1], a, sum);
            }
        }
        sync_all();
        // Σ_t weight_t · V[t].  With at least NT outputs every thread owns NACC (head, dimension) outputs; with fewer, PG
        // threads share an output (positions pg, pg + PG, …) and meet in shared memory (the K rows are done with).
        if (GROUP * HD >= NT) {
#pragma unroll
            for (int k = 0; k < NACC; k++) {
                const uint32_t idx = tid + k * NT;
                if (idx < GROUP * HD) {
                    const uint32_t h = idx / HD, d = idx % HD;
                    const float *w = sc + h * C;
                    const float *v = Vs + d;
                    float a = acc[k] * alpha[h], b = 0.f;
                    uint32_t t = 0;
                    for (; t + 4 <= n; t += 4) {
                        const float4 w4 = *reinterpret_cast<const float4 *>(w + t);
                        a = fmaf(w4.x, v[(size_t)t * HD], a);
                        b = fmaf(w4.y, v[(size_t)(t + 1) * HD], b);
                        a = fmaf(w4.z, v[(size_t)(t + 2) * HD], a);
                        b = fmaf(w4.w, v[(size_t)(t + 3) * HD], b);
                    }
                    for (; t < n; t++) a = fmaf(w[t], v[(size_t)t * HD], a);
                    acc[k] = a + b;
                }
            }
        } else {
            constexpr int NVO = GROUP * HD, PG = NT / (NVO > NT ? NT : NVO);
            const uint32_t idx = tid % NVO, pg = tid / NVO;
            const uint32_t h = idx / HD, d = idx % HD;
            float a = 0.f;
            for (uint32_t t = pg; t < n; t += PG) a = fmaf(sc[h * C + t], Vs[(size_t)t * HD + d], a);
            Ks[pg * NVO + idx] = a;
            sync_all();
            if (tid < (uint32_t)NVO) {
                float sum = 0.f;
#pragma unroll
                for (int g2 = 0; g2 < PG; g2++) sum += Ks[g2 * NVO + tid];
                acc[0] = fmaf(acc[0], alpha[h], sum);
            }
        }
        sync_all();  // before the next pass (or the hand-over) reuses the rows and the scores
        if (au.prof && tid == 0 && p0 == lo) asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(au.prof[2]));  // first pass done
    }
    if (au.prof && tid == 0) asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(au.prof[3]));  // all passes done
    // hand the sums to the first kThreads threads, which finish the unit
#pragma unroll
    for (int k = 0; k < NACC; k++) {
        const uint32_t idx = tid + k * NT;
        if (idx < GROUP * HD) Vs[idx] = acc[k];
    }
    sync_all();
    if (tid >= (uint32_t)kThreads) return;
    float o[NOUT];
#pragma unroll
    for (int k = 0; k < NOUT; k++) {
        const uint32_t idx = tid + k * kThreads;
        o[k] = idx < GROUP * HD ? Vs[idx] : 0.f;
    }
    attn_gqa_finish<GROUP, HD>(p, au.scratch, au.tickets, uh, split, eff, lo < hi, tid, o, ml, Ks, s_last, sync, store);
}
