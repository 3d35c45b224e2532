// sampler.cu — Yule's token sampler on the device (yule-infer/src/sampler.rs:17-136): repetition penalty,
// temperature, softmax, top-k, min-p, top-p, renormalisation and the inverse-CDF pick, in one kernel, so that a
// sampled decode loop moves neither the vocabulary-sized logits nor the pick across the bus.
//
// One CTA of 1024 threads walks the vocabulary in strides; every step of the reference is a phase between
// CTA barriers.  What the reference does with sorts is done with radix selection over the bit patterns of the
// (non-negative) probabilities:
//   top-k   the threshold `sorted[k]` of the descending order (sampler.rs:58-70) is the value of rank k: four
//           passes over 8-bit digits with a 256-bin count histogram;
//   top-p   the shortest descending prefix whose mass reaches top_p (sampler.rs:83-118): the same descent with
//           per-bin sums, accumulated as 2^-44 fixed point in 64-bit integers so that the result does not
//           depend on the order in which threads add; equal probabilities at the boundary are taken in index
//           order (the reference's unstable sort leaves that order open).
// The random number is an argument (the reference draws it from the OS CSPRNG, sampler.rs:212-220): the host
// supplies it, which also makes a sampled run reproducible.
// Differences from the CPU code are confined to the order of floating-point additions (tree instead of
// sequential sums) and the device's expf; they can move a pick only when the random value falls within
// rounding distance of a boundary of the cumulative distribution.

#include <cfloat>

#include "internal.h"

namespace yule {

namespace {

constexpr int kSampThreads = 1024;
constexpr float kFixScale = 17592186044416.0f;  // 2^44

__device__ __forceinline__ float block_reduce_max(float v, float *red) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    __syncthreads();
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = v;
    __syncthreads();
    v = red[threadIdx.x & 31];
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}
__device__ __forceinline__ float block_reduce_sum(float v, float *red) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    __syncthreads();
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = v;
    __syncthreads();
    v = red[threadIdx.x & 31];
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}
// Inclusive scan of one value per thread over the CTA (warp scans, then the warp totals).
__device__ __forceinline__ float block_scan_inclusive(float v, float *red, float *total) {
    const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
        const float t = __shfl_up_sync(0xffffffffu, v, o);
        if (lane >= o) v += t;
    }
    __syncthreads();
    if (lane == 31) red[wid] = v;
    __syncthreads();
    float w = red[lane];
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
        const float t = __shfl_up_sync(0xffffffffu, w, o);
        if (lane >= o) w += t;
    }
    const float before = __shfl_sync(0xffffffffu, w, wid > 0 ? wid - 1 : 0);
    *total = __shfl_sync(0xffffffffu, w, 31);
    return v + (wid > 0 ? before : 0.f);
}
__device__ __forceinline__ uint32_t block_scan_inclusive_u32(uint32_t v, uint32_t *red, uint32_t *total) {
    const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
        const uint32_t t = __shfl_up_sync(0xffffffffu, v, o);
        if (lane >= o) v += t;
    }
    __syncthreads();
    if (lane == 31) red[wid] = v;
    __syncthreads();
    uint32_t w = red[lane];
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
        const uint32_t t = __shfl_up_sync(0xffffffffu, w, o);
        if (lane >= o) w += t;
    }
    const uint32_t before = __shfl_sync(0xffffffffu, w, wid > 0 ? wid - 1 : 0);
    *total = __shfl_sync(0xffffffffu, w, 31);
    return v + (wid > 0 ? before : 0u);
}

// The logit of token i after the repetition penalty (once per earlier occurrence, sampler.rs:26-38) and the
// temperature (sampler.rs:41-46).
__device__ __forceinline__ float adjusted_logit(const float *logits, const uint32_t *counts, uint32_t i, float penalty,
                                                bool penalise, float inv_t, bool scale) {
    float l = logits[i];
    if (penalise)
        for (uint32_t c = counts[i]; c > 0; c--) l = l > 0.0f ? l / penalty : l * penalty;
    if (scale) l *= inv_t;
    return l;
}

struct SampleParams {
    const float *logits;
    uint32_t n;
    float temperature, top_p, min_p, repetition_penalty;
    uint32_t top_k;
    const uint32_t *previous;  // tokens seen so far (prompt and picks)
    uint32_t n_previous;
    float r;                   // uniform random value in [0, 1)
    float *probs;              // scratch, n floats
    uint32_t *counts;          // scratch, n words
    uint32_t *out_token;       // the pick
    uint32_t *append_to;       // when set: the pick is also stored at append_to[n_previous] (the running token list)
    uint32_t *feed_state;      // when set: the pick is also stored at feed_state[0] (the runner's next input token)
};

__global__ void __launch_bounds__(kSampThreads) sample_kernel(const SampleParams p) {
    __shared__ float red[32];
    __shared__ uint32_t redu[32];
    __shared__ unsigned long long hsum[256];
    __shared__ uint32_t hcnt[256];
    __shared__ uint32_t s_prefix, s_rank, s_take, s_first;
    __shared__ unsigned long long s_carry;
    const uint32_t n = p.n, tid = threadIdx.x;
    const bool penalise = p.repetition_penalty != 1.0f && p.n_previous > 0;
    const bool scale = p.temperature > 0.0f && p.temperature != 1.0f;
    const float inv_t = scale ? 1.0f / p.temperature : 1.0f;

    // occurrences of every token among the previous ones
    if (penalise) {
        for (uint32_t i = tid; i < n; i += kSampThreads) p.counts[i] = 0;
        __syncthreads();
        for (uint32_t j = tid; j < p.n_previous; j += kSampThreads) {
            const uint32_t t = p.previous[j];
            if (t < n) atomicAdd(&p.counts[t], 1u);
        }
        __threadfence_block();
        __syncthreads();
    }
    // softmax (sampler.rs:49-55)
    float mx = -FLT_MAX;
    for (uint32_t i = tid; i < n; i += kSampThreads) {
        const float l = adjusted_logit(p.logits, p.counts, i, p.repetition_penalty, penalise, inv_t, scale);
        p.probs[i] = l;
        mx = fmaxf(mx, l);
    }
    mx = block_reduce_max(mx, red);
    float sum = 0.f;
    for (uint32_t i = tid; i < n; i += kSampThreads) {
        const float e = expf(p.probs[i] - mx);
        p.probs[i] = e;
        sum += e;
    }
    sum = block_reduce_sum(sum, red);
    const float inv_sum = 1.0f / sum;
    float max_prob = 0.f;
    for (uint32_t i = tid; i < n; i += kSampThreads) {
        const float q = p.probs[i] * inv_sum;
        p.probs[i] = q;
        max_prob = fmaxf(max_prob, q);
    }
    __syncthreads();

    // top-k (sampler.rs:58-70): keep probs >= the value of rank k in descending order
    if (p.top_k > 0 && p.top_k < n) {
        if (tid == 0) {
            s_prefix = 0;
            s_rank = p.top_k;
        }
        for (int pass = 0; pass < 4; pass++) {
            const int shift = 24 - 8 * pass;
            if (tid < 256) hcnt[tid] = 0;
            __syncthreads();
            const uint32_t prefix = s_prefix, mask = pass == 0 ? 0u : 0xFFFFFFFFu << (shift + 8);
            for (uint32_t i = tid; i < n; i += kSampThreads) {
                const uint32_t b = __float_as_uint(p.probs[i]);
                if ((b & mask) == prefix) atomicAdd(&hcnt[(b >> shift) & 255u], 1u);
            }
            __syncthreads();
            if (tid == 0) {
                uint32_t rank = s_rank, d = 255;
                for (;; d--) {
                    if (rank < hcnt[d]) break;
                    rank -= hcnt[d];
                    if (d == 0) break;
                }
                s_rank = rank;
                s_prefix = prefix | (d << shift);
            }
            __syncthreads();
        }
        const float threshold = __uint_as_float(s_prefix);
        for (uint32_t i = tid; i < n; i += kSampThreads)
            if (!(p.probs[i] >= threshold)) p.probs[i] = 0.f;
        __syncthreads();
    }
    // min-p (sampler.rs:73-80): the largest probability survives top-k, so the maximum taken above still holds
    if (p.min_p > 0.0f) {
        max_prob = block_reduce_max(max_prob, red);
        const float thr = max_prob * p.min_p;
        for (uint32_t i = tid; i < n; i += kSampThreads)
            if (!(p.probs[i] >= thr)) p.probs[i] = 0.f;
        __syncthreads();
    }
    // top-p (sampler.rs:83-118)
    if (p.top_p < 1.0f) {
        const unsigned long long want = (unsigned long long)(p.top_p * kFixScale);
        if (tid == 0) {
            s_prefix = 0;
            s_carry = 0;
            s_take = 0xFFFFFFFFu;  // ties to keep at the boundary value; all of them unless the descent says otherwise
        }
        bool all_in = false;
        for (int pass = 0; pass < 4 && !all_in; pass++) {
            const int shift = 24 - 8 * pass;
            if (tid < 256) {
                hsum[tid] = 0;
                hcnt[tid] = 0;
            }
            __syncthreads();
            const uint32_t prefix = s_prefix, mask = pass == 0 ? 0u : 0xFFFFFFFFu << (shift + 8);
            for (uint32_t i = tid; i < n; i += kSampThreads) {
                const float q = p.probs[i];
                const uint32_t b = __float_as_uint(q);
                if ((b & mask) == prefix) {
                    atomicAdd(&hsum[(b >> shift) & 255u], (unsigned long long)(q * kFixScale));
                    atomicAdd(&hcnt[(b >> shift) & 255u], 1u);
                }
            }
            __syncthreads();
            if (tid == 0) {
                unsigned long long carry = s_carry;
                uint32_t d = 255;
                bool crossed = false;
                for (;; d--) {
                    if (carry + hsum[d] >= want && hcnt[d] > 0) {
                        crossed = true;
                        break;
                    }
                    carry += hsum[d];
                    if (d == 0) break;
                }
                if (!crossed) {
                    s_rank = 0xFFFFFFFFu;  // the mass never reaches top_p: every token stays (the reference never breaks)
                } else {
                    s_rank = 0;
                    s_carry = carry;
                    s_prefix = prefix | (d << shift);
                    if (pass == 3) {
                        // hcnt[d] tokens share the boundary value v: the first m of them (index order) complete the nucleus
                        const unsigned long long v = hcnt[d] ? hsum[d] / hcnt[d] : 0;
                        unsigned long long need = want > carry ? want - carry : 0;
                        uint32_t m = v ? (uint32_t)((need + v - 1) / v) : 1u;
                        if (m < 1) m = 1;
                        if (m > hcnt[d]) m = hcnt[d];
                        s_take = m;
                    }
                }
            }
            __syncthreads();
            all_in = s_rank == 0xFFFFFFFFu;
        }
        if (!all_in) {
            const uint32_t vb = s_prefix, take = s_take;
            uint32_t seen = 0;  // boundary-valued tokens before this chunk
            for (uint32_t base = 0; base < n; base += kSampThreads) {
                const uint32_t i = base + tid;
                const uint32_t b = i < n ? __float_as_uint(p.probs[i]) : 0u;
                const uint32_t is_tie = (i < n && b == vb) ? 1u : 0u;
                uint32_t total;
                const uint32_t incl = block_scan_inclusive_u32(is_tie, redu, &total);
                if (i < n) {
                    const bool keep = b > vb || (is_tie && seen + incl <= take);
                    if (!keep) p.probs[i] = 0.f;
                }
                seen += total;
                __syncthreads();
            }
        }
    }
    // renormalise (sampler.rs:121-130)
    float total = 0.f;
    for (uint32_t i = tid; i < n; i += kSampThreads) total += p.probs[i];
    total = block_reduce_sum(total, red);
    uint32_t pick;
    if (!(total > 0.0f)) {
        // nothing left: argmax of the adjusted logits, ties to the highest index (sampler.rs:123-125, :150-163)
        float best = -FLT_MAX;
        uint32_t idx = 0;
        bool any = false;
        for (uint32_t i = tid; i < n; i += kSampThreads) {
            const float l = adjusted_logit(p.logits, p.counts, i, p.repetition_penalty, penalise, inv_t, scale);
            if (!any || l >= best) {
                best = l;
                idx = i;
                any = true;
            }
        }
        const float bmax = block_reduce_max(any ? best : -FLT_MAX, red);
        __syncthreads();
        if (tid == 0) s_first = 0;
        __syncthreads();
        if (any && best == bmax) atomicMax(&s_first, idx);
        __syncthreads();
        pick = s_first;
    } else {
        // inverse CDF in index order (sampler.rs:166-183): the first token whose running sum reaches r, else the last
        const float inv_total = 1.0f / total;
        if (tid == 0) s_first = n - 1;
        __syncthreads();
        float carry = 0.f;
        for (uint32_t base = 0; base < n; base += kSampThreads) {
            const uint32_t i = base + tid;
            const float q = i < n ? p.probs[i] * inv_total : 0.f;
            float chunk_total;
            const float incl = block_scan_inclusive(q, red, &chunk_total);
            if (i < n && carry + incl >= p.r) atomicMin(&s_first, i);
            carry += chunk_total;
            __syncthreads();
            if (s_first != n - 1 || carry >= p.r) break;  // uniform across the CTA: found in this chunk
        }
        __syncthreads();
        pick = s_first;
    }
    if (tid == 0) {
        *p.out_token = pick;
        if (p.append_to) p.append_to[p.n_previous] = pick;
        if (p.feed_state) p.feed_state[0] = pick;
    }
}

}  // namespace

cudaError_t launch_sample(const SampleArgs &a, cudaStream_t s, uint64_t *launches) {
    SampleParams p;
    p.logits = a.logits;
    p.n = a.n;
    p.temperature = a.temperature;
    p.top_p = a.top_p;
    p.min_p = a.min_p;
    p.repetition_penalty = a.repetition_penalty;
    p.top_k = a.top_k;
    p.previous = a.previous;
    p.n_previous = a.n_previous;
    p.r = a.r;
    p.probs = a.scratch;
    p.counts = reinterpret_cast<uint32_t *>(a.scratch + a.n);
    p.out_token = a.out_token;
    p.append_to = a.append_to;
    p.feed_state = a.feed_state;
    if (a.n == 0) return cudaErrorInvalidValue;
    sample_kernel<<<1, kSampThreads, 0, s>>>(p);
    *launches += 1;
    return cudaGetLastError();
}

}  // namespace yule
