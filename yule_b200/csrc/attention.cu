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

#include "attn_gqa.cuh"

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
    extern __shared__ __align__(16) float sm[];
    __shared__ uint32_t s_last;
    yule_pdl_launch_dependents();
    yule_pdl_wait();
    // prefill: query z of the launch sits z positions further on and has its own rows and scratch
    const uint32_t z = blockIdx.z;
    AttnUnit au;
    au.pos = p.pos_ptr ? (p.pos_per_query ? p.pos_ptr[z] : *p.pos_ptr) : p.seq_len - 1 + z;
    au.k_cache = p.k_cache + (size_t)z * p.kv_batch_stride;
    au.v_cache = p.v_cache + (size_t)z * p.kv_batch_stride;
    au.q_in = p.q + (size_t)z * p.q_stride;
    au.scratch = p.scratch + (size_t)z * p.n_heads * p.n_splits * (HD + 2);
    au.tickets = p.tickets + (size_t)z * p.n_heads;
    au.q_pairs = au.k_pairs = au.v_pairs = nullptr;
    au.in_epoch = 0;
    au.prof = nullptr;
    float *out_z = p.out + (size_t)z * p.out_stride;
    attn_gqa_unit<GROUP, HD, false>(
        p, au, blockIdx.x, blockIdx.y, threadIdx.x, sm, &s_last, [] { __syncthreads(); },
        [&](uint32_t i, float v) {
            out_z[i] = v;
            if (TP && p.tp.push) tp_push_value(p.tp, i, v);
        });
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
        const size_t smem = ((size_t)g * a.hd + 2 * a.hd + 16 + (size_t)g * p.max_chunk + (size_t)nsl * g * a.hd +
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

