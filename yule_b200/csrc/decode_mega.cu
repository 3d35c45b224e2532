// decode_mega.cu — one persistent kernel per decoded token.
//
// The token step of GpuTransformerRunner::forward (yule-infer/src/gpu_runner.rs:296-695) is a chain of
// about five dependent matvec-sized dispatches per layer.  As separate kernels each link of that chain
// pays a launch boundary and a cold start of its weight stream; at the TinyLlama shape those fixed costs are
// several times the time HBM needs for the bytes.  This kernel runs the whole chain in one cooperative launch of
// one 512-thread CTA per SM (two groups of eight warps):
//
//   * Weights.  Every group owns a ring of shared-memory slots, each filled by one tiled TMA copy per plane of a
//     stage (16 rows × 8 super-blocks of raw Q4_K rows, or of the row-planar Q6_K records).  The sequence of stages
//     a group will consume — over every matvec of the token — is a list built on the host, so the warp that
//     releases a slot last refills it with the stage `slots` ahead, whatever phase that stage belongs to: the weight
//     stream never stops at a phase boundary, and a phase's first weights are in shared memory before its input is.
//   * Activations.  A vector that one phase produces and the next consumes lives in global memory as
//     (value, epoch) pairs.  A producer stores each finished row as one 8-byte pair; a consumer polls the pairs while
//     it builds its shared-memory image of x, so "the data has arrived" and "the data" are the same load.  The epoch
//     is token counter × (phases + 1) + phase + 1: no flag is ever reset, and there is no grid barrier.
//     A pair buffer is overwritten only by a phase whose CTAs have, through the vectors they polled, transitively
//     waited for every reader of the previous contents.
//   * Phases.  embedding row → per layer { RMSNorm + Q/K/V, RoPE + KV append + attention (a unit per query head and
//     split, K / V rows staged in shared memory), o-proj + residual, RMSNorm + gate/up + SiLU·mul (a CTA's two groups
//     take the gate and the up tile of the same rows), down + residual (the groups split the column chunks of a
//     tile) } → RMSNorm + output matrix with a running arg-max → pick (ties to the highest index,
//     yule-infer/src/sampler.rs:150-163), history and position advance.
//   * Arithmetic is that of the tensor-pipe matvec kernels (qmv_q4k_ring.cu, qmv_q6k_ring.cu) and of the
//     grouped-query attention kernel (attention.cu), whose device code this file includes.
//   * Registers and L1.  With 224 KB of the SM given to shared memory L1 is tiny: a register spill, or a descriptor
//     read from global memory, is an L2 round trip.  The kernel compiles without spills (128 registers per thread)
//     and keeps its phase table, job counts and stage lists in shared memory; pointers into shared memory are
//     derived where they are used rather than carried through the phase loop.
//
// Every wait (copy, pair) is bounded; the first one that runs out records a status word and every later wait
// returns at once, so a failed step ends in microseconds and the host reads the status.  No thread leaves the
// kernel early: all CTA- and group-wide barriers are reached whatever happened.

#include <cfloat>
#include <cstring>
#include <mutex>
#include <string>
#include <vector>

#include <cuda.h>
#include <cuda_fp16.h>

#include "internal.h"
#include "dequant_device.cuh"

namespace yule {

namespace {

#include "ring_common.cuh"
#include "pair_wait.cuh"
namespace q4 {
#include "q4k_mma_common.cuh"
#include "q4k_ring_common.cuh"
}  // namespace q4
namespace q6 {
#include "q6k_ring_common.cuh"
}  // namespace q6
#include "attn_gqa.cuh"

constexpr int kMegaThreads = 512;
constexpr uint32_t kSlotBytes = 28672;  // a ring slot holds one stage of either format
constexpr int kMegaMaxSlots = 3;
constexpr uint32_t kMegaMinChunk = 256;  // positions per attention split
static_assert(q4::kStageBytes <= kSlotBytes && q6::kStageBytes <= kSlotBytes, "slot holds a stage of either format");
static_assert(q4::kThreadsCta == kMegaThreads && q6::kThreadsCta == kMegaThreads, "staging code assumes this CTA size");
constexpr size_t kMegaSmemMax = 227 * 1024;

enum : uint32_t { kPhEmbed = 0, kPhQ4K = 1, kPhQ6K = 2, kPhAttn = 3, kPhPick = 4 };
enum : uint32_t { kVecHidden = 0, kVecQ, kVecK, kVecV, kVecAtt, kVecGate, kVecCount, kVecLogits = 100 };
constexpr uint32_t kNoPhase = 0xFFFFFFFFu;

// One phase of the token.  The table is built on the host, lives in global memory and is copied into shared
// memory by every CTA when the kernel starts: the walk over a group's stage sequence crosses phases all the time,
// and with the shared-memory carve-out this kernel needs, L1 is too small to keep anything else close.
struct Phase {
    uint64_t ptr[3];      // matvec: the matrices sharing x (raw Q4_K rows / row-planar Q6_K records); attention: K cache, V cache, tickets
    const float *norm_w;  // RMSNorm weights folded into the staging of x, or null
    uint32_t kind;        // kind | pair << 8 | k-split << 9 | chunks << 16   (chunks: stages per (job, matrix))
    uint32_t n_tiles;     // 16-row jobs (pair: of one matrix); pick: records to read
    uint32_t x_phase;     // the phase that wrote the input vector
    uint32_t res_phase;   // the phase that wrote the hidden state added to the rows, or kNoPhase
    uint32_t n_prod;      // groups (attention: KV heads, embedding: CTAs) that announce their output in this phase
    uint32_t n_cols;
    uint32_t rows[3];
    uint32_t vecs;        // input vector | output vector of matrix 0 << 8 | of matrix 1 << 16 | of matrix 2 << 24
    uint32_t n_seg;
    uint32_t pad;
};
static_assert(sizeof(Phase) == 80, "copied to shared memory 16 bytes at a time");
__device__ __forceinline__ uint32_t ph_kind(const Phase &P) { return P.kind & 0xFFu; }
__device__ __forceinline__ bool ph_pair(const Phase &P) { return (P.kind & 0x100u) != 0; }
__device__ __forceinline__ bool ph_ksplit(const Phase &P) { return (P.kind & 0x200u) != 0; }
__device__ __forceinline__ bool ph_cta_jobs(const Phase &P) { return (P.kind & 0x300u) != 0; }  // tiles dealt to CTAs, the two groups share a tile
__device__ __forceinline__ uint32_t ph_chunks(const Phase &P) { return P.kind >> 16; }
// k-split phase: chunks [0, ph_split_at) go to group 0, the rest to group 1
__device__ __forceinline__ uint32_t ph_split_at(const Phase &P) { return (ph_chunks(P) + 1u) / 2u; }
__device__ __forceinline__ bool ph_matvec(const Phase &P) { return ph_kind(P) == kPhQ4K || ph_kind(P) == kPhQ6K; }

struct MegaParams {
    const Phase *phases;
    uint32_t n_phases;
    uint2 *vec[kVecCount];
    float *logits;
    uint2 *best;     // [groups of the grid][2]: (value, epoch), (index, epoch)
    uint32_t *hint;  // [phase] producers that have issued their stores, summed over all tokens so far
    uint32_t *tick;  // tokens this kernel has processed (epochs and hint targets count from it)
    unsigned long long *prof;  // timing aid: [CTA][phase] %globaltimer when the CTA entered the phase, or null
    uint32_t *state, *history;
    const uint8_t *embd;
    uint32_t embd_type, dim;
    uint64_t embd_row_bytes;
    AttnParams attn;  // the fields that do not change from layer to layer
    uint32_t attn_units;
    uint32_t slots, scratch_bytes, hot_bytes;
    const uint32_t *lists;     // [groups of the grid][list_stride] stage sequences (see stage_entry)
    const uint32_t *list_len;  // [groups of the grid]
    uint32_t list_stride;
    uint32_t use_hints;  // consumers wait for the producers' count before they read the pairs (see hint_wait)
    float eps;
    int *status;
    long long wait_cycles;
    // Self-test of the bounded waits: consumers expect epochs that no producer writes, so every wait runs out (once:
    // the first one records the status, the others return at once); the pick then only advances the token counter.
    uint32_t epoch_skew;
    uint32_t dbg;  // timing aid (debug knob): 1 leaves the multiplications out, 2 the refills of the ring (results are garbage then)
};

// fixed part of the shared memory, after ring, phase scratch and the phase table
constexpr uint32_t kFxZero = 0, kFxInvScale = 1024, kFxRed = 1040, kFxPartial = 1296, kFxBest = 5392, kFxBars = 5648,
                   kFxCnt = 5696, kFxLast = 5720, kFxPick = 5728, kFxPairBuf = 5888, kFxBytes = 6016;

__device__ __forceinline__ void pair_store(uint2 *p, uint32_t v, uint32_t epoch) {
    asm volatile("st.volatile.global.v2.u32 [%0], {%1, %2};" ::"l"(p), "r"(v), "r"(epoch) : "memory");
}

// "Probably complete": optional.  Each producer counts itself in a per-phase word once its stores are issued, one
// thread per consumer CTA polls that word, and only then do the others read the pairs (which still carry their
// own epoch, so a store that lags behind the count is simply polled a little longer).  Bounded like every wait.
__device__ __forceinline__ void hint_wait(const uint32_t *h, uint32_t target, int *status, long long budget) {
    long long t0 = 0;
    for (uint32_t it = 0;; it++) {
        uint32_t v;
        asm volatile("ld.volatile.global.u32 %0, [%1];" : "=r"(v) : "l"(h) : "memory");
        if ((int32_t)(v - target) >= 0) return;
        if (it == 0) t0 = clock64();
        if ((it & 15u) != 15u) continue;
        if (*reinterpret_cast<volatile int *>(status) != 0) return;
        if (clock64() - t0 >= budget) {
            atomicCAS(status, 0, kStatusPeerTimeout);
            return;
        }
    }
}
__device__ __forceinline__ unsigned long long global_ns() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}

// Jobs of a group in a phase.  Tiles are dealt round-robin to the groups of the grid, except where the two groups of
// a CTA share a tile and meet in shared memory: a pair phase (SiLU(gate)·up: group 0 multiplies the gate tile, group 1
// the up tile of the same rows; 352 tiles over 148 CTAs is three rounds of one stage, over 296 groups as gate+up jobs
// it was two rounds of two) and a k-split phase (a matrix with few tiles and several chunks of columns, like the
// down projection: the groups take half of the chunks each and group 0 adds the two partial sums).
__device__ __forceinline__ uint32_t my_tiles_of(const Phase &P, uint32_t group) {
    if (!ph_matvec(P)) return 0u;
    const uint32_t G = gridDim.x;
    const uint32_t first = ph_cta_jobs(P) ? blockIdx.x : blockIdx.x + group * G, stride = ph_cta_jobs(P) ? G : 2u * G;
    return P.n_tiles > first ? (P.n_tiles - first + stride - 1) / stride : 0u;
}
// A group's stage sequence over the whole token is a list built on the host (it depends on the model and the
// grid only) and copied into shared memory: entry = phase | matrix << 10 | chunk << 12 | tile within the matrix << 18.
__host__ __device__ inline uint32_t stage_entry(uint32_t ph, uint32_t seg, uint32_t chunk, uint32_t tile) {
    return ph | (seg << 10) | (chunk << 12) | (tile << 18);
}

// One tiled TMA load: box of the tensor map at element coordinates (x, y) into shared memory, bytes counted on `bar`.
// The source is this GPU's own memory; no multicast.
__device__ __forceinline__ void tma_load_2d(uint32_t dst, uint64_t map, uint32_t x, uint32_t y, uint32_t bar) {
    asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];" ::"r"(dst),
                 "l"(map), "r"(bar), "r"(x), "r"(y)
                 : "memory");
}

// Copies of one stage, by one thread.  A stage is one box per plane: issuing a copy instruction per row (16 for a
// Q4_K stage, 64 for a Q6_K stage) costs the issuing warp 0.7 / 2.3 µs, and its group waits for it at the end of the job.
// The boxes are as wide as the shared-memory row pitches, so the padding between rows comes with the copy (what
// lies beyond the eight super-blocks of a row chunk — the next block, the next row or zeros — is never read);
// rows past the end of the matrix arrive as zeros.
__device__ __forceinline__ void mega_issue(const Phase *hot, uint32_t entry, uint32_t dst, uint32_t bar) {
    const Phase &P = hot[entry & 0x3FFu];
    const uint32_t seg = (entry >> 10) & 3u;
    const uint32_t row0 = (entry >> 18) * 16u, blk0 = ((entry >> 12) & 0x3Fu) * 8u;
    const uint64_t maps = P.ptr[seg];  // CUtensorMap (128 bytes each): one for Q4_K, four planes for Q6_K; 8-byte elements
    if (ph_kind(P) == kPhQ4K) {
        mbar_arrive_expect_tx(bar, q4::kStageBytes);
        tma_load_2d(dst, maps, blk0 * 18u, row0, bar);
    } else {
        mbar_arrive_expect_tx(bar, q6::kStageBytes);
        tma_load_2d(dst + q6::kQlOff, maps, blk0 * 16u, row0, bar);
        tma_load_2d(dst + q6::kQhOff, maps + 128, blk0 * 8u, row0, bar);
        tma_load_2d(dst + q6::kScOff, maps + 256, blk0 * 2u, row0, bar);
        tma_load_2d(dst + q6::kDOff, maps + 384, blk0 / 4u, row0, bar);
    }
}

__device__ __forceinline__ void mega_group_barrier(int group) {
    asm volatile("bar.sync %0, %1;" ::"r"(1 + group), "r"(256) : "memory");
}

__device__ __forceinline__ bool better(float v, uint32_t i, float bv, uint32_t bi) { return v > bv || (v == bv && i > bi); }

__device__ __forceinline__ uint4 ld_pairs2(const uint2 *p) {
    uint4 q;
    asm volatile("ld.volatile.global.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(q.x), "=r"(q.y), "=r"(q.z), "=r"(q.w) : "l"(p) : "memory");
    return q;
}

// Builds the shared-memory image of x for one matvec phase from the (value, epoch) pairs of the vector, by the
// whole CTA: optional RMSNorm, power-of-two normalisation, fp16 hi/lo split, per-sub-block sums — the arithmetic
// of stage_activations in q4k_mma_common.cuh / q6k_ring_common.cuh, ordered for latency and for registers (this
// kernel has 128 per thread and must not spill: behind its shared-memory carve-out L1 is tiny, a spill is an L2
// round trip).  The norm weights (static) are requested before any waiting.  A thread's first 8 columns stay in
// registers between the reduction and the conversion; further chunks (vectors longer than 4096) wait in shared
// memory, in the 32 bytes of the image that the same thread later overwrites with their converted form.
// `hint`: see hint_wait.  Starts with a CTA barrier (the previous users of the scratch are done).
__device__ __forceinline__ void mega_stage(const bool Q6, unsigned char *scratch, const uint2 *xp, uint32_t x_epoch, uint32_t n_cols,
                                           const float *__restrict__ norm_w, float eps, float *red, float *inv_scale_out,
                                           const uint32_t *hint, uint32_t hint_target, int *status, long long budget,
                                           unsigned long long *prof) {
    const uint32_t tid = threadIdx.x;
    const int lane = tid & 31, wid = tid >> 5;
    const uint32_t c0 = tid * 8u;
    float gw[8], a[8];
    if (norm_w && c0 < n_cols) {
        *reinterpret_cast<float4 *>(gw) = *reinterpret_cast<const float4 *>(norm_w + c0);
        *reinterpret_cast<float4 *>(gw + 4) = *reinterpret_cast<const float4 *>(norm_w + c0 + 4);
    }
    if (hint && tid == 0) hint_wait(hint, hint_target, status, budget);
    __syncthreads();
    // the two 16-byte homes of columns c..c+7 in the image
    const size_t plane = q6::x_plane_bytes(n_cols) + 64;
    auto homes = [&](uint32_t c, uint4 *&h0, uint4 *&h1) {
        if (!Q6) {
            // fragment order of q4k_mma_common.cuh: B operands of word pairs, hi part and lo part 4 uint4 apart
            const uint32_t blk = c >> 8, tt = (c >> 6) & 3, h = (c >> 5) & 1, wp = (c >> 3) & 3;
            h0 = reinterpret_cast<uint4 *>(scratch) + ((blk * 2 + h) * 4 + wp) * 8 + tt;
            h1 = h0 + 4;
        } else {
            // column order with 8 halves of padding after every 128 columns (q6k_ring_common.cuh): hi plane, lo plane
            const uint32_t pc = c + 8 * (c >> 7);
            h0 = reinterpret_cast<uint4 *>(scratch + 2 * (size_t)pc);
            h1 = reinterpret_cast<uint4 *>(scratch + plane + 2 * (size_t)pc);
        }
    };
    float ss = 0.f, mx = 0.f;
    auto reduce8 = [&](const float(&v)[8], const float(&w)[8]) {
#pragma unroll
        for (int i = 0; i < 8; i++) {
            ss = fmaf(v[i], v[i], ss);
            mx = fmaxf(mx, fabsf(norm_w ? v[i] * w[i] : v[i]));
        }
    };
    // eight columns from the pairs of the vector: the four loads go out together, then they are checked
    auto load_x = [&](uint32_t c, float(&v)[8]) {
        uint4 q[4];
#pragma unroll
        for (int i = 0; i < 4; i++) q[i] = ld_pairs2(xp + c + 2 * i);
        bool ok = true;
#pragma unroll
        for (int i = 0; i < 4; i++) ok = ok && q[i].y == x_epoch && q[i].w == x_epoch;
        if (ok) {
#pragma unroll
            for (int i = 0; i < 4; i++) {
                v[2 * i] = __uint_as_float(q[i].x);
                v[2 * i + 1] = __uint_as_float(q[i].z);
            }
        } else {
            q4::tp_load8(xp + c, x_epoch, status, budget, v);
        }
    };
    if (c0 < n_cols) {
        load_x(c0, a);
        reduce8(a, gw);
    }
    if (prof && tid == 0) prof[1] = global_ns();  // this thread's part of x has arrived
    for (uint32_t c = c0 + kMegaThreads * 8u; c < n_cols; c += kMegaThreads * 8u) {
        float v[8], w[8];
        load_x(c, v);
        if (norm_w) {
            *reinterpret_cast<float4 *>(w) = *reinterpret_cast<const float4 *>(norm_w + c);
            *reinterpret_cast<float4 *>(w + 4) = *reinterpret_cast<const float4 *>(norm_w + c + 4);
        }
        reduce8(v, w);
        uint4 *h0, *h1;
        homes(c, h0, h1);
        *h0 = make_uint4(__float_as_uint(v[0]), __float_as_uint(v[1]), __float_as_uint(v[2]), __float_as_uint(v[3]));
        *h1 = make_uint4(__float_as_uint(v[4]), __float_as_uint(v[5]), __float_as_uint(v[6]), __float_as_uint(v[7]));
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        ss += __shfl_xor_sync(0xffffffffu, ss, o);
        mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
    }
    if (lane == 0) {
        red[wid] = ss;
        red[32 + wid] = mx;
    }
    __syncthreads();
    ss = 0.f;
    mx = 0.f;
#pragma unroll
    for (int i = 0; i < kMegaThreads / 32; i++) {
        ss += red[i];
        mx = fmaxf(mx, red[32 + i]);
    }
    // RMSNorm scale exactly as the CPU runner forms it: 1 / sqrt(ss / n + eps) (yule-infer/src/model_runner.rs:254-258)
    const float inv_rms = norm_w ? 1.0f / sqrtf(ss / (float)n_cols + eps) : 1.0f;
    mx *= inv_rms;
    // 2^e with max|x|·2^e in [2^13, 2^14); exponent clamped so both 2^e and 2^-e stay finite normals
    int eb = (int)((__float_as_uint(mx) >> 23) & 0xFFu);
    if (mx == 0.f || eb == 0xFF) eb = 127 + 13;
    int se = 127 + 13 - (eb - 127);
    se = se < 1 ? 1 : (se > 253 ? 253 : se);
    const float scale = __uint_as_float((uint32_t)se << 23);
    if (tid == 0) inv_scale_out[0] = __uint_as_float((uint32_t)(254 - se) << 23);
    auto convert8 = [&](uint32_t c, float(&v)[8], const float(&w)[8]) {
        if (norm_w) {
            // x * inv * w, rounded in that order (yule-infer/src/model_runner.rs:273)
#pragma unroll
            for (int i = 0; i < 8; i++) v[i] = v[i] * inv_rms * w[i];
        }
        __half hi[8], lo[8];
#pragma unroll
        for (int i = 0; i < 8; i++) {
            v[i] *= scale;  // exact (power of two)
            hi[i] = __float2half_rn(v[i]);
            lo[i] = __float2half_rn(v[i] - __half2float(hi[i]));
        }
        float s8 = ((v[0] + v[1]) + (v[2] + v[3])) + ((v[4] + v[5]) + (v[6] + v[7]));
        uint4 *h0, *h1;
        homes(c, h0, h1);
        if (!Q6) {
            *h0 = make_uint4(q4::h2_as_u32(__halves2half2(hi[0], hi[2])), q4::h2_as_u32(__halves2half2(hi[1], hi[3])),
                             q4::h2_as_u32(__halves2half2(hi[4], hi[6])), q4::h2_as_u32(__halves2half2(hi[5], hi[7])));
            *h1 = make_uint4(q4::h2_as_u32(__halves2half2(lo[0], lo[2])), q4::h2_as_u32(__halves2half2(lo[1], lo[3])),
                             q4::h2_as_u32(__halves2half2(lo[4], lo[6])), q4::h2_as_u32(__halves2half2(lo[5], lo[7])));
            s8 += __shfl_xor_sync(0xffffffffu, s8, 1);  // Σ over 32 columns: 4 consecutive lanes hold one sub-block
            s8 += __shfl_xor_sync(0xffffffffu, s8, 2);
            if ((lane & 3) == 0) reinterpret_cast<float *>(scratch + (size_t)4 * n_cols)[c >> 5] = s8;
        } else {
            *h0 = make_uint4(q4::h2_as_u32(__halves2half2(hi[0], hi[1])), q4::h2_as_u32(__halves2half2(hi[2], hi[3])),
                             q4::h2_as_u32(__halves2half2(hi[4], hi[5])), q4::h2_as_u32(__halves2half2(hi[6], hi[7])));
            *h1 = make_uint4(q4::h2_as_u32(__halves2half2(lo[0], lo[1])), q4::h2_as_u32(__halves2half2(lo[2], lo[3])),
                             q4::h2_as_u32(__halves2half2(lo[4], lo[5])), q4::h2_as_u32(__halves2half2(lo[6], lo[7])));
            s8 += __shfl_xor_sync(0xffffffffu, s8, 1);  // two consecutive lanes hold one 16-column scale group
            if ((lane & 1) == 0) reinterpret_cast<float *>(scratch + 2 * plane)[c >> 4] = -32.0f * s8;
        }
    };
    // n_cols is a multiple of 256, so whole warps are in or out of every step (the shuffles are safe)
    if (c0 < n_cols) convert8(c0, a, gw);
    for (uint32_t c = c0 + kMegaThreads * 8u; c < n_cols; c += kMegaThreads * 8u) {
        float v[8], w[8];
        uint4 *h0, *h1;
        homes(c, h0, h1);
        const uint4 r0 = *h0, r1 = *h1;
        v[0] = __uint_as_float(r0.x), v[1] = __uint_as_float(r0.y), v[2] = __uint_as_float(r0.z), v[3] = __uint_as_float(r0.w);
        v[4] = __uint_as_float(r1.x), v[5] = __uint_as_float(r1.y), v[6] = __uint_as_float(r1.z), v[7] = __uint_as_float(r1.w);
        if (norm_w) {
            *reinterpret_cast<float4 *>(w) = *reinterpret_cast<const float4 *>(norm_w + c);
            *reinterpret_cast<float4 *>(w + 4) = *reinterpret_cast<const float4 *>(norm_w + c + 4);
        }
        convert8(c, v, w);
    }
    __syncthreads();
    if (prof && tid == 0) prof[2] = global_ns();  // image complete
}

// The dynamic shared memory of the kernel: fixed part (constant offsets), phase table with the per-group job counts
// and stage lists, phase scratch, the two rings.  Pointers into it are derived where they are used instead of being
// carried through the phase loop: registers are what this kernel is short of.
extern __shared__ __align__(128) unsigned char mega_smem[];
__device__ __forceinline__ Phase *sm_hot() { return reinterpret_cast<Phase *>(mega_smem + kFxBytes); }
__device__ __forceinline__ unsigned short *sm_mt(const MegaParams &p, int group) {
    return reinterpret_cast<unsigned short *>(mega_smem + kFxBytes + (size_t)p.n_phases * sizeof(Phase)) + group * p.n_phases;
}
__device__ __forceinline__ uint32_t *sm_list(const MegaParams &p, int group) {
    return reinterpret_cast<uint32_t *>(mega_smem + kFxBytes + (size_t)p.n_phases * (sizeof(Phase) + 4)) + group * p.list_stride;
}
__device__ __forceinline__ unsigned char *sm_scratch(const MegaParams &p) { return mega_smem + kFxBytes + p.hot_bytes; }
__device__ __forceinline__ unsigned char *sm_ring(const MegaParams &p, int group) {
    return mega_smem + kFxBytes + p.hot_bytes + p.scratch_bytes + (size_t)group * p.slots * kSlotBytes;
}
__device__ __forceinline__ uint4 *sm_zero() { return reinterpret_cast<uint4 *>(mega_smem + kFxZero); }
__device__ __forceinline__ float *sm_partial(int group) { return reinterpret_cast<float *>(mega_smem + kFxPartial) + group * 512; }
__device__ __forceinline__ float *sm_bestv(int group) { return reinterpret_cast<float *>(mega_smem + kFxBest) + group * 32; }
__device__ __forceinline__ uint32_t *sm_cnt(int group) { return reinterpret_cast<uint32_t *>(mega_smem + kFxCnt) + group * kMegaMaxSlots; }
__device__ __forceinline__ uint32_t sm_bar0(int group) { return smem_u32(mega_smem + kFxBars) + (uint32_t)group * kMegaMaxSlots * 8u; }

// What the consume loop of a phase keeps across iterations: where the group is in its ring.
struct RingPos {
    uint32_t slot, parity, n;  // n: stages of the token consumed so far
};

// One matvec phase of one group: consumes this group's stages of phase `ph` in order, finishes each 16-row job
// (cross-warp sum, scale, SiLU·up or residual, pair store or logits + running arg-max) and refills the ring.
// Separate instantiations per format keep the lane constants of the other format out of the loop.
template <bool Q6>
__device__ __forceinline__ void mega_consume(const MegaParams &p, uint32_t ph, RingPos &rp, uint32_t tick, uint2 res_pre) {
    const uint32_t tid = threadIdx.x, gt = tid & 255u;
    const int lane = tid & 31, group = tid >> 8, wid = (tid >> 5) & 7;
    const int g = lane >> 2, t = lane & 3;
    const uint32_t gi = blockIdx.x + (uint32_t)group * gridDim.x, stride = 2u * gridDim.x;
    const uint32_t S = p.slots, total = p.list_len[gi];
    const Phase *hot = sm_hot();
    const unsigned short *mt = sm_mt(p, group);
    const uint32_t *list = sm_list(p, group);
    unsigned char *ring = sm_ring(p, group);
    const uint32_t ring_u32 = smem_u32(ring), bar0 = sm_bar0(group);
    uint32_t *cnt = sm_cnt(group);
    const unsigned char *scratch = sm_scratch(p);
    const uint4 *zero = sm_zero();
    float *partial = sm_partial(group), *bestv = sm_bestv(group);
    const float invs = reinterpret_cast<const float *>(mega_smem + kFxInvScale)[0];
    const uint32_t epoch0 = tick * (p.n_phases + 1u), epoch = epoch0 + ph + 1u;
    const Phase &P = hot[ph];
    const uint32_t bpr = P.n_cols >> 8, chunks = ph_chunks(P);
    const bool pair = ph_pair(P), ksplit = ph_ksplit(P), shared_tile = pair || ksplit;
    const uint32_t my_tiles = mt[ph];
    const uint32_t tile0 = shared_tile ? blockIdx.x : gi, tile_step = shared_tile ? gridDim.x : stride;
    const uint32_t c_begin = (ksplit && group == 1) ? ph_split_at(P) : 0u, c_end = (ksplit && group == 0) ? ph_split_at(P) : chunks;
    const bool has_res = P.res_phase != kNoPhase;
    // lane constants (B column n = g is live only for g = t (hi part) and g = t + 4 (lo part))
    const bool feeds = (g & 3) == t;
    const int u = t & 1;
    const bool first_half = t < 2;  // lanes that charge the per-sub-block offsets (mins / −32·Σx) once
    // Q4_K image: fragments, then per-sub-block sums.  Q6_K image: hi plane, lo plane, −32·Σx.
    const size_t plane = q6::x_plane_bytes(P.n_cols) + 64;
    const unsigned char *bsrc = Q6 ? (feeds ? scratch + ((g >> 2) ? plane : 0) + 2 * ((128 + 8) * (t >> 1) + 16 * u) : reinterpret_cast<const unsigned char *>(zero))
                                   : (feeds ? scratch + 16 * ((g >> 2) * 4 + t) : reinterpret_cast<const unsigned char *>(zero));
    const uint32_t bstride = feeds ? (Q6 ? 2u * 2u * (128 + 8) : 64u * 16u) : 0u;  // bytes per super-block
    const unsigned char *ssrc = Q6 ? (first_half ? scratch + 2 * plane + 4 * (8 * u) : reinterpret_cast<const unsigned char *>(zero))
                                   : scratch + (size_t)4 * P.n_cols + 4 * (4 * u);
    const uint32_t sstride = Q6 ? (first_half ? 64u : 0u) : 32u;  // bytes per super-block

    float acc0 = 0.f, acc1 = 0.f;
    const uint32_t rr = gt >> 3, w2 = gt & 7u;  // finishing threads (gt < 128): row of the tile, lane of the eight that add up a row
    // Releases the slot just consumed when some later stage of the token will reuse it; the warp that releases it last
    // refills it (one thread: a stage is one tiled copy per plane).
    auto release = [&](uint32_t n_stage, uint32_t slot_used) {
        if (n_stage + S < total) {
            __syncwarp();
            if (lane == 0) {
                __threadfence_block();
                const bool last = (atomicAdd(&cnt[slot_used], 1u) & 7u) == 7u;
                if (last && !(p.dbg & 2u)) mega_issue(hot, list[n_stage + S], ring_u32 + slot_used * kSlotBytes, bar0 + 8 * slot_used);
            }
            __syncwarp();
        }
    };
    for (uint32_t k = 0; k < my_tiles; k++) {
        // where this job's rows go: worked out before the multiplications, off the path from the last one to the stores
        uint32_t seg = pair ? (uint32_t)group : 0u, tile = tile0 + k * tile_step;
        if (!pair)
            while (seg + 1 < P.n_seg && tile >= (P.rows[seg] + 15u) / 16u) {
                tile -= (P.rows[seg] + 15u) / 16u;
                seg++;
            }
        const uint32_t row = tile * 16u + rr;
        const bool mine = gt < 128u && w2 == 0 && row < P.rows[seg];
        const uint32_t ov = (P.vecs >> (8 + 8 * (pair ? 0u : seg))) & 0xFFu;
        if (k > 0 && has_res && mine) res_pre = pair_peek(p.vec[kVecHidden] + row);  // settled in the epilogue
        uint32_t last_n = 0, last_slot = 0;
        for (uint32_t c = c_begin; c < c_end; c++) {
            const uint32_t bar = bar0 + 8 * rp.slot;
            if (!(p.dbg & 2u)) ring_wait(bar, rp.parity, p.status, p.wait_cycles);  // a wait that gave up has recorded it; go on with what is there
            const uint32_t blk0 = c * 8u;
            const uint32_t nblk = bpr - blk0 < 8u ? bpr - blk0 : 8u;
            if ((uint32_t)wid < nblk && !(p.dbg & 1u)) {
                const unsigned char *st = ring + (size_t)rp.slot * kSlotBytes;
                const uint32_t blk = blk0 + wid;
                if (!Q6) {
                    const unsigned char *r0 = st + (uint32_t)g * q4::kRowPitch + (uint32_t)wid * 144u;
                    q4::consume_block_smem(r0, r0 + 8 * q4::kRowPitch, reinterpret_cast<const uint4 *>(bsrc + (size_t)blk * bstride),
                                           reinterpret_cast<const float *>(ssrc + (size_t)blk * sstride), u, t, first_half, acc0, acc1);
                } else {
                    const int h6 = t >> 1;
                    q6::consume_block_smem(st + q6::kQlOff + (uint32_t)g * q6::kQlPitch + (uint32_t)wid * 128u + 64u * h6 + 16u * u,
                                           st + q6::kQhOff + (uint32_t)g * q6::kQhPitch + (uint32_t)wid * 64u + 32u * h6 + 16u * u,
                                           st + q6::kScOff + (uint32_t)g * q6::kScPitch + (uint32_t)wid * 16u,
                                           st + q6::kDOff + (uint32_t)g * q6::kDPitch + (uint32_t)wid * 2u,
                                           reinterpret_cast<const __half *>(bsrc + (size_t)blk * bstride), feeds ? 32u : 0u,
                                           reinterpret_cast<const float *>(ssrc + (size_t)blk * sstride), u, acc0, acc1);
                }
            }
            // the last stage of a job is released after the job's rows are on their way (below)
            if (c + 1 < c_end) {
                release(rp.n, rp.slot);
            } else {
                last_n = rp.n;
                last_slot = rp.slot;
            }
            rp.n++;
            if (++rp.slot == S) {
                rp.slot = 0;
                rp.parity ^= 1u;
            }
        }
        // the tile's rows are complete in this warp: sum the four column groups, park the 16 row sums
        {
            float v0 = acc0, v1 = acc1;
            v0 += __shfl_xor_sync(0xffffffffu, v0, 1);
            v1 += __shfl_xor_sync(0xffffffffu, v1, 1);
            v0 += __shfl_xor_sync(0xffffffffu, v0, 2);
            v1 += __shfl_xor_sync(0xffffffffu, v1, 2);
            float *part = partial + (size_t)(k & 1u) * 256;
            if (t == 0) {
                part[wid * 16 + g] = v0;
                part[wid * 16 + g + 8] = v1;
            }
            acc0 = acc1 = 0.f;
        }
        // job complete: one group barrier, then 128 threads finish the 16 rows (eight lanes per row add the eight warps'
        // sums in a fixed tree).  The two partial buffers alternate between jobs, so the next job's sums cannot overtake
        // these reads (a warp passes the next barrier only after the first four warps have finished here).
        mega_group_barrier(group);
        if (gt < 128u) {
            const uint32_t nwu = bpr < 8u ? bpr : 8u;
            float s0 = w2 < nwu ? partial[(size_t)(k & 1u) * 256 + w2 * 16 + rr] : 0.f;
#pragma unroll
            for (int o = 1; o < 8; o <<= 1) s0 += __shfl_xor_sync(0xffffffffu, s0, o);
            s0 *= invs;
            if (shared_tile) {
                // group 1 hands its sums to group 0 through shared memory: the finishing warps of the two groups (256
                // threads; both groups run the same number of jobs here) meet at a barrier of their own, the other warps
                // go on with the next job
                float *pairbuf = reinterpret_cast<float *>(mega_smem + kFxPairBuf) + (k & 1u) * 16;
                if (group == 1 && mine) pairbuf[rr] = s0;
                asm volatile("bar.sync 3, 256;" ::: "memory");
                if (group == 0 && mine) {
                    const float other = pairbuf[rr];
                    if (pair) {
                        s0 = (s0 / (1.0f + expf(-s0))) * other;  // silu_mul.cu: x / (1 + exp(−x)) * up
                    } else {
                        s0 += other;
                        if (has_res)
                            s0 += pair_settle(res_pre, p.vec[kVecHidden] + row, epoch0 + P.res_phase + 1u + p.epoch_skew, p.status, p.wait_cycles);
                    }
                    pair_store(p.vec[ov] + row, __float_as_uint(s0), epoch);
                }
            } else if (mine) {
                if (has_res) s0 += pair_settle(res_pre, p.vec[kVecHidden] + row, epoch0 + P.res_phase + 1u + p.epoch_skew, p.status, p.wait_cycles);
                if (ov == kVecLogits) {
                    p.logits[row] = s0;
                    // running arg-max of the rows this lane finishes; rows come in rising order: ties go to the highest index
                    if (s0 >= bestv[rr]) {
                        bestv[rr] = s0;
                        reinterpret_cast<uint32_t *>(bestv)[16 + rr] = row;
                    }
                } else {
                    pair_store(p.vec[ov] + row, __float_as_uint(s0), epoch);
                }
            }
        }
        release(last_n, last_slot);
    }
}

template <int HD>
__global__ void __launch_bounds__(kMegaThreads, 1) decode_token_kernel(const __grid_constant__ MegaParams p) {
    const uint32_t tid = threadIdx.x;
    const int lane = tid & 31, group = tid >> 8;
    const uint32_t gt = tid & 255u;  // thread within the group
    const uint32_t NP = p.n_phases;
    const uint32_t pos = p.state[1], tick = *p.tick;

    // the phase table, the zero region, the arg-max slots and the ring barriers; one CTA barrier before anybody uses them
    {
        const uint4 *src = reinterpret_cast<const uint4 *>(p.phases);
        uint4 *dst = reinterpret_cast<uint4 *>(sm_hot());
        for (uint32_t i = tid; i < NP * (uint32_t)(sizeof(Phase) / 16); i += kMegaThreads) dst[i] = src[i];
    }
    if (tid < 64) sm_zero()[tid] = make_uint4(0u, 0u, 0u, 0u);
    if (gt < 16) {
        sm_bestv(group)[gt] = -FLT_MAX;
        reinterpret_cast<uint32_t *>(sm_bestv(group))[16 + gt] = 0u;
    }
    if (gt == 0) {
        for (int i = 0; i < kMegaMaxSlots; i++) {
            mbar_init(sm_bar0(group) + 8 * i, 1);
            sm_cnt(group)[i] = 0;
        }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    }
    __syncthreads();

    // this group's job count per phase, its stage list, and its first copies
    {
        const uint32_t gi = blockIdx.x + (uint32_t)group * gridDim.x;
        const uint32_t total = p.list_len[gi];
        const Phase *hot = sm_hot();
        unsigned short *mt = sm_mt(p, group);
        uint32_t *list = sm_list(p, group);
        for (uint32_t i = gt; i < NP; i += 256u) mt[i] = (unsigned short)my_tiles_of(hot[i], (uint32_t)group);
        for (uint32_t i = gt; i < total; i += 256u) list[i] = p.lists[(size_t)gi * p.list_stride + i];
        mega_group_barrier(group);
        if (gt == 0)
            for (uint32_t n = 0; n < p.slots && n < total; n++)
                mega_issue(hot, list[n], smem_u32(sm_ring(p, group)) + n * kSlotBytes, sm_bar0(group) + 8 * n);
    }

    RingPos rp = {0u, 0u, 0u};

    for (uint32_t ph = 0; ph < NP; ph++) {
        const Phase *hot = sm_hot();
        const uint32_t kind = ph_kind(hot[ph]);
        const uint32_t epoch0 = tick * (NP + 1u);  // phase ph writes with epoch0 + ph + 1
        const uint32_t epoch = epoch0 + ph + 1u;
        const uint32_t x_phase = hot[ph].x_phase;
        const uint32_t x_epoch = epoch0 + x_phase + 1u + p.epoch_skew;
        const uint32_t *hints = p.use_hints ? p.hint : nullptr;
        if (p.prof && tid == 0) p.prof[((size_t)blockIdx.x * (NP + 1u) + ph) * 4] = global_ns();  // entering phase ph

        if (kind == kPhEmbed) {
            // embedding row of the token (gpu_runner.rs:309-343 does this on the CPU and uploads it)
            const uint32_t c = blockIdx.x * kMegaThreads + tid;
            if (c < p.dim)
                pair_store(p.vec[kVecHidden] + c,
                           __float_as_uint(dequant_elem(p.embd + (uint64_t)p.state[0] * p.embd_row_bytes, p.embd_type, c)), epoch);
            if (hints && blockIdx.x * kMegaThreads < p.dim) {
                __syncthreads();
                if (tid == 0) atomicAdd(p.hint + ph, 1u);
            }
            continue;
        }

        if (kind == kPhAttn) {
            if (blockIdx.x >= p.attn_units) continue;
            if (hints && tid == 0) hint_wait(hints + x_phase, (tick + 1u) * hot[x_phase].n_prod, p.status, p.wait_cycles);
            __syncthreads();  // Q/K/V are there; and both groups have left the image of x that this scratch overlays
            {
                // a unit per (query head, split); all sixteen warps run its passes, group 0 then publishes / merges / stores
                bool stored = false;
                const uint32_t n_splits = p.attn.n_splits;
                const uint32_t head = blockIdx.x / n_splits;
                AttnUnit au;
                au.k_cache = reinterpret_cast<float *>(hot[ph].ptr[0]);
                au.v_cache = reinterpret_cast<float *>(hot[ph].ptr[1]);
                au.tickets = reinterpret_cast<uint32_t *>(hot[ph].ptr[2]);
                au.scratch = p.attn.scratch;
                au.q_in = nullptr;
                au.q_pairs = p.vec[kVecQ];
                au.k_pairs = p.vec[kVecK];
                au.v_pairs = p.vec[kVecV];
                au.in_epoch = x_epoch;
                au.pos = pos;
                au.prof = p.prof ? p.prof + ((size_t)blockIdx.x * (NP + 1u) + ph) * 4 : nullptr;
                uint2 *outp = p.vec[kVecAtt];
                attn_unit_staged<1, HD, kMegaThreads>(
                    p.attn, au, head, head / (p.attn.n_heads / p.attn.n_kv_heads), blockIdx.x % n_splits, tid,
                    reinterpret_cast<float *>(sm_scratch(p)), reinterpret_cast<uint32_t *>(mega_smem + kFxLast), [] { __syncthreads(); },
                    [] { mega_group_barrier(0); },
                    [&](uint32_t idx, float v) {
                        pair_store(outp + idx, __float_as_uint(v), epoch);
                        stored = true;
                    });
                if (hints && group == 0) {
                    // the unit that wrote this KV head's output (thread 0 takes part in those stores) announces it
                    mega_group_barrier(0);
                    if (gt == 0 && stored) atomicAdd(p.hint + ph, 1u);
                }
            }
            continue;
        }

        if (kind == kPhPick) {
            // by CTA 0: arg-max over the groups' records (ties to the highest index), then what argmax_kernel does at the
            // end of the multi-kernel token step
            if (blockIdx.x != 0) continue;
            float *pickv = reinterpret_cast<float *>(mega_smem + kFxPick);
            uint32_t *picki = reinterpret_cast<uint32_t *>(mega_smem + kFxPick + 64);
            if (hints && tid == 0) hint_wait(hints + x_phase, (tick + 1u) * hot[x_phase].n_prod, p.status, p.wait_cycles);
            __syncthreads();
            float bv = -FLT_MAX;
            uint32_t bi = 0;
            if (tid < hot[ph].n_tiles) {
                const uint2 q0 = pair_peek(p.best + 2 * tid), q1 = pair_peek(p.best + 2 * tid + 1);
                bv = pair_settle(q0, p.best + 2 * tid, x_epoch, p.status, p.wait_cycles);
                bi = __float_as_uint(pair_settle(q1, p.best + 2 * tid + 1, x_epoch, p.status, p.wait_cycles));
            }
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) {
                const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
                const uint32_t oi = __shfl_xor_sync(0xffffffffu, bi, o);
                if (better(ov, oi, bv, bi)) {
                    bv = ov;
                    bi = oi;
                }
            }
            if (lane == 0) {
                pickv[tid >> 5] = bv;
                picki[tid >> 5] = bi;
            }
            __syncthreads();
            if (tid < 32) {
                bv = lane < kMegaThreads / 32 ? pickv[lane] : -FLT_MAX;
                bi = lane < kMegaThreads / 32 ? picki[lane] : 0u;
#pragma unroll
                for (int o = 16; o > 0; o >>= 1) {
                    const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
                    const uint32_t oi = __shfl_xor_sync(0xffffffffu, bi, o);
                    if (better(ov, oi, bv, bi)) {
                        bv = ov;
                        bi = oi;
                    }
                }
                if (lane == 0) {
                    if (p.epoch_skew == 0u) {
                        p.state[0] = bi;
                        p.history[pos] = bi;
                        p.state[1] = pos + 1u;
                    }
                    p.state[2] += 1u;  // token counter of the runner (argmax_kernel keeps it too)
                    *p.tick = tick + 1u;
                }
            }
            continue;
        }

        // ── matvec phase ─────────────────────────────────────────────────────────────────────────
        if (hot[ph].n_tiles <= blockIdx.x) continue;  // neither group of this CTA has a job here
        const uint32_t gi = blockIdx.x + (uint32_t)group * gridDim.x;
        // the hidden-state value this lane will add to the row of its first job: requested before anything else (it was
        // complete long ago), settled in the epilogue
        uint2 res_pre = make_uint2(0u, 0u);
        if (hot[ph].res_phase != kNoPhase && gt < 128u && (gt & 7u) == 0u) {
            const uint32_t row = (ph_cta_jobs(hot[ph]) ? blockIdx.x : gi) * 16u + (gt >> 3);
            if (row < hot[ph].rows[0]) res_pre = pair_peek(p.vec[kVecHidden] + row);
        }
        {
            const uint32_t *hw = hints ? hints + x_phase : nullptr;
            const uint32_t target = (tick + 1u) * hot[x_phase].n_prod;
            const uint2 *xp = p.vec[hot[ph].vecs & 0xFFu];
            mega_stage(kind == kPhQ6K, sm_scratch(p), xp, x_epoch, hot[ph].n_cols, hot[ph].norm_w, p.eps,
                       reinterpret_cast<float *>(mega_smem + kFxRed), reinterpret_cast<float *>(mega_smem + kFxInvScale), hw, target, p.status,
                       p.wait_cycles, p.prof ? p.prof + ((size_t)blockIdx.x * (NP + 1u) + ph) * 4 : nullptr);
        }
        if (!ph_cta_jobs(hot[ph]) && hot[ph].n_tiles <= gi) continue;  // this group has no job in the phase (it only helped with the staging)
        if (kind == kPhQ4K)
            mega_consume<false>(p, ph, rp, tick, res_pre);
        else
            mega_consume<true>(p, ph, rp, tick, res_pre);
        if (p.prof && tid == 0) p.prof[((size_t)blockIdx.x * (NP + 1u) + ph) * 4 + 3] = global_ns();  // group 0's jobs done
        const bool to_logits = ((hot[ph].vecs >> 8) & 0xFFu) == kVecLogits;
        if (hints && !to_logits && !(ph_cta_jobs(hot[ph]) && group == 1)) {
            // every store of this group in this phase has been issued: announce it
            mega_group_barrier(group);
            if (gt == 0) atomicAdd(p.hint + ph, 1u);
        }
        if (to_logits) {
            // this group's arg-max over the rows it produced, as two pairs for the pick phase
            const float *bestv = sm_bestv(group);
            mega_group_barrier(group);
            if (gt == 0) {
                float bv = bestv[0];
                uint32_t bi = reinterpret_cast<const uint32_t *>(bestv)[16];
                for (int i = 1; i < 16; i++) {
                    const float v = bestv[i];
                    const uint32_t vi = reinterpret_cast<const uint32_t *>(bestv)[16 + i];
                    if (better(v, vi, bv, bi)) {
                        bv = v;
                        bi = vi;
                    }
                }
                pair_store(p.best + 2 * gi, __float_as_uint(bv), epoch);
                pair_store(p.best + 2 * gi + 1, bi, epoch);
                if (hints) atomicAdd(p.hint + ph, 1u);
            }
        }
    }
    if (p.prof && tid == 0) p.prof[((size_t)blockIdx.x * (NP + 1u) + NP) * 4] = global_ns();
}

}  // namespace

// ── host side ────────────────────────────────────────────────────────────────────────────────────

struct MegaHandle {
    MegaParams params;
    size_t smem = 0;
    uint32_t grid = 0;
    uint32_t group = 0, hd = 0;
    bool cooperative = true;
    std::vector<Phase> phases;
};

namespace {

struct MegaDims {
    uint32_t grid, n_splits, max_chunk, slots, scratch_bytes, hot_bytes, n_phases;
    size_t smem;
    size_t off_phases, off_vec[kVecCount], off_best, off_scratch, off_tickets, off_hint, off_tick, off_prof, off_maps, off_lists, off_list_len, total;
    uint32_t n_maps, list_stride;
};

bool tensor_ok(const MegaTensor &t, bool allow_q6) {
    if (!t.ptr || (reinterpret_cast<uintptr_t>(t.ptr) & 15)) return false;
    return t.type == YULE_DTYPE_Q4_K || (allow_q6 && t.type == YULE_DTYPE_Q6_K);
}

bool variant_built(uint32_t hd) { return hd == 64 || hd == 128; }

size_t q4_image_bytes(uint32_t n_cols) { return (size_t)4 * n_cols + 2 * (size_t)(n_cols / 8); }
size_t q6_image_bytes(uint32_t n_cols) { return 2 * (q6::x_plane_bytes(n_cols) + 64) + (size_t)(n_cols / 16) * 4; }

bool mega_dims(const MegaModel &m, MegaDims *d, std::string *why) {
    auto no = [&](const char *s) {
        if (why) *why = s;
        return false;
    };
    if (!m.n_layers || m.layers.size() != m.n_layers) return no("no layers");
    if (!m.n_kv_heads || m.n_heads % m.n_kv_heads) return no("head counts");
    const uint32_t hd = m.head_dim;
    if (!variant_built(hd)) return no("no instantiation for this head dimension");
    const uint32_t dim = m.dim, qdim = m.n_heads * hd, kvdim = m.n_kv_heads * hd, ff = m.ff_dim;
    if (dim % 256 || qdim % 256 || ff % 256) return no("row lengths must be multiples of 256");
    if (m.sm_count < 1 || 2 * m.sm_count > kMegaThreads) return no("SM count");
    for (const MegaLayer &L : m.layers) {
        if (!tensor_ok(L.q, false) || !tensor_ok(L.k, false) || !tensor_ok(L.v, false)) return no("attn_q/k/v must be Q4_K");
        if (!tensor_ok(L.gate, false) || !tensor_ok(L.up, false)) return no("ffn_gate/up must be Q4_K");
        if (!tensor_ok(L.o, true) || !tensor_ok(L.down, true)) return no("attn_output / ffn_down must be Q4_K or Q6_K");
        if (!L.attn_norm || !L.ffn_norm || !L.k_cache || !L.v_cache) return no("layer pointers");
    }
    if (!tensor_ok(m.output, true) || !m.output_norm || !m.embd) return no("output matrix must be Q4_K or Q6_K");
    const uint32_t G = (uint32_t)m.sm_count;
    d->grid = G;
    uint32_t ns = G / m.n_heads;  // a unit per (query head, split)
    // A split is at least kMegaMinChunk positions: below that one unit per KV head is faster than several plus the
    // merge (a ticket, a fence and two more L2 round trips), since a phase here costs latency, not bandwidth.
    const uint32_t by_len = (m.max_seq_len + kMegaMinChunk - 1) / kMegaMinChunk;
    if (by_len < ns) ns = by_len;
    if (ns > (uint32_t)kGqaMaxSplits) ns = kGqaMaxSplits;
    if (ns < 1) return no("more query heads than SMs");
    d->n_splits = ns;
    uint32_t mc = (m.max_seq_len + ns - 1) / ns;
    if (mc < kMegaMinChunk) mc = kMegaMinChunk;
    d->max_chunk = ((mc + 3) / 4) * 4;
    const size_t attn_bytes = attn_staged_smem_floats(1, (int)hd) * sizeof(float);
    size_t scratch = attn_bytes;
    auto image = [&](const MegaTensor &t, uint32_t cols) {
        const size_t b = t.type == YULE_DTYPE_Q4_K ? q4_image_bytes(cols) : q6_image_bytes(cols);
        if (b > scratch) scratch = b;
    };
    for (const MegaLayer &L : m.layers) {
        image(L.q, dim);
        image(L.o, qdim);
        image(L.gate, dim);
        image(L.down, ff);
    }
    image(m.output, dim);
    scratch = (scratch + 127) & ~(size_t)127;
    d->scratch_bytes = (uint32_t)scratch;
    d->n_phases = 1 + 5 * m.n_layers + 2;
    if (d->n_phases >= 0xFFFFu) return no("too many layers");
    if (d->n_phases >= 1024u) return no("too many layers");
    // the longest stage list is that of group 0
    {
        auto tiles = [](uint32_t rows) { return (rows + 15) / 16; };
        auto chunks = [](uint32_t cols) { return (cols / 256 + 7) / 8; };
        auto mine = [&](uint32_t n_tiles) { return (n_tiles + 2 * G - 1) / (2 * G); };
        auto mine_cta = [&](uint32_t n_tiles) { return (n_tiles + G - 1) / G; };  // pair phases: a CTA's groups share the tile
        const uint32_t per_layer = mine(tiles(qdim) + 2 * tiles(kvdim)) * chunks(dim) + mine(tiles(dim)) * chunks(qdim) +
                                   mine_cta(tiles(ff)) * chunks(dim) + mine(tiles(dim)) * chunks(ff);
        const uint32_t longest = per_layer * m.n_layers + mine(tiles(m.vocab)) * chunks(dim);
        d->list_stride = (longest + 3) & ~3u;
        if (chunks(dim) > 64 || chunks(ff) > 64 || chunks(qdim) > 64 || tiles(m.vocab) >= (1u << 14) || tiles(ff) >= (1u << 14) ||
            tiles(qdim) + 2 * tiles(kvdim) >= (1u << 14))
            return no("matrix too large for the stage list encoding");
    }
    const size_t hot = ((size_t)d->n_phases * (sizeof(Phase) + 2 * sizeof(unsigned short)) + 2 * (size_t)d->list_stride * sizeof(uint32_t) + 127) &
                       ~(size_t)127;
    d->hot_bytes = (uint32_t)hot;
    if (scratch + hot + kFxBytes + 2 * 2 * (size_t)kSlotBytes > kMegaSmemMax) return no("activation image too large for two ring slots per group");
    uint32_t slots = (uint32_t)((kMegaSmemMax - scratch - hot - kFxBytes) / (2 * (size_t)kSlotBytes));
    if (slots > (uint32_t)kMegaMaxSlots) slots = kMegaMaxSlots;
    // Where it pays off.  The kernel wins where a token is a chain of short, latency-bound steps (TinyLlama class:
    // 0.65 against 0.76 ms per token); where the steps are long enough to be bound by the weight stream (8B class:
    // rows of 4096 / 14336 columns, whose image of x leaves room for two ring slots only) the multi-kernel graph with
    // the streaming kernels is faster (2.2 against 3.0 ms per token), so such models keep it.
    if (slots < (uint32_t)kMegaMaxSlots) return no("model too wide for the persistent kernel to pay off");
    d->slots = slots;
    d->smem = (size_t)2 * slots * kSlotBytes + scratch + hot + kFxBytes;
    // workspace layout
    size_t off = 0;
    auto take = [&](size_t bytes) {
        const size_t o = off;
        off += (bytes + 255) & ~(size_t)255;
        return o;
    };
    d->off_phases = take((size_t)d->n_phases * sizeof(Phase));
    const uint32_t vlen[kVecCount] = {dim, qdim, kvdim, kvdim, qdim, ff};
    for (uint32_t i = 0; i < kVecCount; i++) d->off_vec[i] = take((size_t)vlen[i] * sizeof(uint2));
    d->off_best = take((size_t)2 * G * 2 * sizeof(uint2));
    d->off_scratch = take(((size_t)m.n_heads * ns * (hd + 2) + 4) * sizeof(float));
    d->off_tickets = take((size_t)m.n_layers * m.n_heads * sizeof(uint32_t));
    d->off_hint = take((size_t)d->n_phases * sizeof(uint32_t));
    d->off_tick = take(sizeof(uint32_t));
    auto maps_of = [](const MegaTensor &t) { return t.type == YULE_DTYPE_Q4_K ? 1u : 4u; };
    d->n_maps = maps_of(m.output);
    for (const MegaLayer &L : m.layers) d->n_maps += 5 + maps_of(L.o) + maps_of(L.down);
    d->off_maps = take((size_t)d->n_maps * sizeof(CUtensorMap));
    d->off_lists = take((size_t)2 * G * d->list_stride * sizeof(uint32_t));
    d->off_list_len = take((size_t)2 * G * sizeof(uint32_t));
    d->off_prof = take((size_t)G * (d->n_phases + 1) * 4 * sizeof(unsigned long long));
    d->total = off;
    (void)kvdim;
    return true;
}

template <int HD>
cudaError_t launch_variant(const MegaHandle &h, cudaStream_t s) {
    auto kern = decode_token_kernel<HD>;
    static bool attr_done[64] = {};
    static std::mutex mu;
    {
        int dev = 0;
        cudaError_t e = cudaGetDevice(&dev);
        if (e != cudaSuccess) return e;
        std::lock_guard<std::mutex> lock(mu);
        if (dev < 0 || dev >= 64 || !attr_done[dev]) {
            e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kMegaSmemMax);
            if (e != cudaSuccess) return e;
            if (dev >= 0 && dev < 64) attr_done[dev] = true;
        }
    }
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(h.grid);
    cfg.blockDim = dim3(kMegaThreads);
    cfg.dynamicSmemBytes = h.smem;
    cfg.stream = s;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeCooperative;  // every CTA resident at once: they wait for one another's data
    attr[0].val.cooperative = 1;
    cfg.attrs = attr;
    cfg.numAttrs = h.cooperative ? 1 : 0;
    return cudaLaunchKernelEx(&cfg, kern, h.params);
}

}  // namespace

size_t mega_workspace_bytes(const MegaModel &m, std::string *why) {
    MegaDims d;
    if (!mega_dims(m, &d, why)) return 0;
    return d.total;
}

cudaError_t mega_setup(const MegaModel &m, void *workspace, cudaStream_t s, MegaHandle **out) {
    MegaDims d;
    if (!mega_dims(m, &d, nullptr)) return cudaErrorInvalidValue;
    MegaHandle *h = new MegaHandle();
    unsigned char *ws = static_cast<unsigned char *>(workspace);
    const uint32_t hd = m.head_dim, group = m.n_heads / m.n_kv_heads;
    const uint32_t dim = m.dim, qdim = m.n_heads * hd, kvdim = m.n_kv_heads * hd, ff = m.ff_dim;
    const uint32_t G = d.grid;
    uint32_t *tickets = reinterpret_cast<uint32_t *>(ws + d.off_tickets);

    std::vector<CUtensorMap> maps;
    maps.reserve(d.n_maps);
    cudaError_t map_err = cudaSuccess;
    auto blank = [](uint32_t kind) {
        Phase P;
        memset(&P, 0, sizeof(P));
        P.kind = kind;
        P.res_phase = kNoPhase;
        return P;
    };
    auto matvec = [&](std::initializer_list<MegaTensor> ts, std::initializer_list<uint32_t> rows, uint32_t cols, bool pair, uint32_t x_vec,
                      uint32_t x_phase, const float *norm_w, std::initializer_list<uint32_t> outs, uint32_t res_phase) {
        Phase P = blank(ts.begin()->type == YULE_DTYPE_Q4_K ? kPhQ4K : kPhQ6K);
        uint32_t i = 0;
        const uint32_t bpr = cols / 256;
        for (const MegaTensor &t : ts) {
            // tensor maps of this matrix (8-byte elements): boxes as wide as the shared-memory row pitches
            const uint32_t n_rows = *(rows.begin() + i);
            P.ptr[i++] = reinterpret_cast<uint64_t>(ws + d.off_maps) + maps.size() * sizeof(CUtensorMap);
            if (t.type == YULE_DTYPE_Q4_K) {
                maps.emplace_back();
                if (map_err == cudaSuccess)
                    map_err = encode_tensor_map_2d(t.ptr, 8, (uint64_t)bpr * 18, n_rows, (uint64_t)bpr * 144, q4::kRowPitch / 8, 16, &maps.back());
            } else {
                const uint64_t rec = q6::row_record_bytes(bpr);
                const uint64_t off[4] = {0, (uint64_t)bpr * 128, (uint64_t)bpr * 192, (uint64_t)bpr * 208};
                const uint64_t len[4] = {(uint64_t)bpr * 128, (uint64_t)bpr * 64, (uint64_t)bpr * 16, q6::d_section_bytes(bpr)};
                const uint32_t pitch[4] = {q6::kQlPitch, q6::kQhPitch, q6::kScPitch, q6::kDPitch};
                for (int pl = 0; pl < 4; pl++) {
                    maps.emplace_back();
                    if (map_err == cudaSuccess)
                        map_err = encode_tensor_map_2d(t.ptr + off[pl], 8, len[pl] / 8, n_rows, rec, pitch[pl] / 8, 16, &maps.back());
                }
            }
        }
        P.n_seg = i;
        i = 0;
        uint32_t tiles = 0;
        for (uint32_t r : rows) {
            P.rows[i] = r;
            if (!pair || i == 0) tiles += (r + 15) / 16;
            i++;
        }
        P.vecs = x_vec;
        i = 0;
        for (uint32_t o : outs) P.vecs |= o << (8 + 8 * i++);
        const uint32_t n_chunks = (cols / 256 + 7) / 8;
        // few tiles and several chunks of columns: the two groups of a CTA split the chunks of a tile between them
        const bool ksplit = !pair && P.n_seg == 1 && n_chunks >= 2 && tiles <= G && *outs.begin() != kVecLogits;
        P.kind |= (pair ? 0x100u : 0u) | (ksplit ? 0x200u : 0u) | (n_chunks << 16);
        P.n_cols = cols;
        P.n_tiles = tiles;
        P.x_phase = x_phase;
        P.norm_w = norm_w;
        P.res_phase = res_phase;
        P.n_prod = (pair || ksplit) ? (tiles < G ? tiles : G) : (tiles < 2 * G ? tiles : 2 * G);
        h->phases.push_back(P);
        return (uint32_t)h->phases.size() - 1;
    };
    {
        Phase P = blank(kPhEmbed);
        P.n_prod = (dim + kMegaThreads - 1) / kMegaThreads;
        h->phases.push_back(P);
    }
    uint32_t last_hidden = 0;
    for (uint32_t l = 0; l < m.n_layers; l++) {
        const MegaLayer &L = m.layers[l];
        const uint32_t ph_qkv = matvec({L.q, L.k, L.v}, {qdim, kvdim, kvdim}, dim, false, kVecHidden, last_hidden, L.attn_norm,
                                       {kVecQ, kVecK, kVecV}, kNoPhase);
        Phase A = blank(kPhAttn);
        A.ptr[0] = reinterpret_cast<uint64_t>(L.k_cache);
        A.ptr[1] = reinterpret_cast<uint64_t>(L.v_cache);
        A.ptr[2] = reinterpret_cast<uint64_t>(tickets + (size_t)l * m.n_heads);
        A.x_phase = ph_qkv;
        A.n_prod = m.n_heads;
        h->phases.push_back(A);
        const uint32_t ph_att = (uint32_t)h->phases.size() - 1;
        const uint32_t ph_o = matvec({L.o}, {dim}, qdim, false, kVecAtt, ph_att, nullptr, {kVecHidden}, last_hidden);
        const uint32_t ph_gu = matvec({L.gate, L.up}, {ff, ff}, dim, true, kVecHidden, ph_o, L.ffn_norm, {kVecGate, kVecGate}, kNoPhase);
        last_hidden = matvec({L.down}, {dim}, ff, false, kVecGate, ph_gu, nullptr, {kVecHidden}, ph_o);
    }
    const uint32_t ph_out = matvec({m.output}, {m.vocab}, dim, false, kVecHidden, last_hidden, m.output_norm, {kVecLogits}, kNoPhase);
    {
        Phase P = blank(kPhPick);
        const uint32_t tiles = (m.vocab + 15) / 16;
        P.n_tiles = tiles < 2 * G ? tiles : 2 * G;
        P.x_phase = ph_out;
        h->phases.push_back(P);
    }
    if (h->phases.size() != d.n_phases || maps.size() != d.n_maps || map_err != cudaSuccess) {
        delete h;
        return map_err != cudaSuccess ? map_err : cudaErrorInvalidValue;
    }
    // every group's stage sequence
    std::vector<uint32_t> lists((size_t)2 * G * d.list_stride, 0u), list_len(2 * G, 0u);
    for (uint32_t gi = 0; gi < 2 * G; gi++) {
        uint32_t n = 0;
        for (uint32_t ph = 0; ph < d.n_phases; ph++) {
            const Phase &P = h->phases[ph];
            const uint32_t kind = P.kind & 0xFFu;
            if (kind != kPhQ4K && kind != kPhQ6K) continue;
            const bool pair = (P.kind & 0x100u) != 0, ksplit = (P.kind & 0x200u) != 0, shared_tile = pair || ksplit;
            const uint32_t n_chunks = P.kind >> 16, split_at = (n_chunks + 1) / 2, grp = gi / G;
            // pair / k-split phase: tiles go to the CTAs; group 0 takes the gate tile (or the first half of the chunks),
            // group 1 the up tile of the same rows (or the second half)
            const uint32_t c_begin = (ksplit && grp == 1) ? split_at : 0, c_end = (ksplit && grp == 0) ? split_at : n_chunks;
            for (uint32_t tile = shared_tile ? gi % G : gi; tile < P.n_tiles; tile += shared_tile ? G : 2 * G) {
                uint32_t seg = pair ? grp : 0, t = tile;
                if (!shared_tile)
                    while (seg + 1 < P.n_seg && t >= (P.rows[seg] + 15) / 16) {
                        t -= (P.rows[seg] + 15) / 16;
                        seg++;
                    }
                for (uint32_t c = c_begin; c < c_end; c++) {
                    if (n >= d.list_stride) {
                        delete h;
                        return cudaErrorInvalidValue;
                    }
                    lists[(size_t)gi * d.list_stride + n++] = stage_entry(ph, seg, c, t);
                }
            }
        }
        list_len[gi] = n;
    }
    {
        cudaError_t me = cudaMemcpyAsync(ws + d.off_lists, lists.data(), lists.size() * sizeof(uint32_t), cudaMemcpyHostToDevice, s);
        if (me == cudaSuccess) me = cudaMemcpyAsync(ws + d.off_list_len, list_len.data(), list_len.size() * sizeof(uint32_t), cudaMemcpyHostToDevice, s);
        if (me == cudaSuccess) me = cudaStreamSynchronize(s);  // the host vectors go out of scope
        if (me != cudaSuccess) {
            delete h;
            return me;
        }
    }
    {
        cudaError_t me = cudaMemcpyAsync(ws + d.off_maps, maps.data(), maps.size() * sizeof(CUtensorMap), cudaMemcpyHostToDevice, s);
        if (me == cudaSuccess) me = cudaStreamSynchronize(s);  // `maps` goes out of scope
        if (me != cudaSuccess) {
            delete h;
            return me;
        }
    }
    cudaError_t e = cudaMemcpyAsync(ws + d.off_phases, h->phases.data(), h->phases.size() * sizeof(Phase), cudaMemcpyHostToDevice, s);
    if (e == cudaSuccess) e = cudaStreamSynchronize(s);
    if (e != cudaSuccess) {
        delete h;
        return e;
    }
    MegaParams &p = h->params;
    memset(&p, 0, sizeof(p));
    p.phases = reinterpret_cast<const Phase *>(ws + d.off_phases);
    p.n_phases = d.n_phases;
    for (uint32_t i = 0; i < kVecCount; i++) p.vec[i] = reinterpret_cast<uint2 *>(ws + d.off_vec[i]);
    p.logits = m.logits;
    p.best = reinterpret_cast<uint2 *>(ws + d.off_best);
    p.hint = reinterpret_cast<uint32_t *>(ws + d.off_hint);
    p.tick = reinterpret_cast<uint32_t *>(ws + d.off_tick);
    p.prof = knob("YULE_MEGA_PROF") ? reinterpret_cast<unsigned long long *>(ws + d.off_prof) : nullptr;
    p.state = m.state;
    p.history = m.history;
    p.embd = m.embd;
    p.embd_type = m.embd_type;
    p.dim = dim;
    p.embd_row_bytes = (uint64_t)(dim / block_size(m.embd_type)) * block_bytes(m.embd_type);
    AttnParams &a = p.attn;
    a.cos_table = m.rope_cos;
    a.sin_table = m.rope_sin;
    a.scratch = reinterpret_cast<float *>(ws + d.off_scratch);
    a.hd = hd;
    a.n_heads = m.n_heads;
    a.n_kv_heads = m.n_kv_heads;
    a.kv_stride = kvdim;
    a.n_splits = d.n_splits;
    a.max_chunk = d.max_chunk;
    a.min_chunk = kMegaMinChunk;
    a.status = m.status;
    a.wait_cycles = m.wait_cycles;
    p.attn_units = m.n_heads * d.n_splits;
    p.slots = d.slots;
    p.scratch_bytes = d.scratch_bytes;
    p.hot_bytes = d.hot_bytes;
    p.lists = reinterpret_cast<const uint32_t *>(ws + d.off_lists);
    p.list_len = reinterpret_cast<const uint32_t *>(ws + d.off_list_len);
    p.list_stride = d.list_stride;
    p.dbg = knob("YULE_MEGA_DBG") ? (uint32_t)atoi(knob("YULE_MEGA_DBG")) : 0u;
    p.use_hints = (knob("YULE_MEGA_HINTS") && atoi(knob("YULE_MEGA_HINTS")) != 0) ? 1u : 0u;
    p.eps = m.eps;
    p.status = m.status;
    p.wait_cycles = m.wait_cycles;
    h->smem = d.smem;
    h->grid = d.grid;
    h->group = group;
    h->hd = hd;
    *out = h;
    return cudaSuccess;
}

void mega_set_cooperative(MegaHandle *h, bool on) { h->cooperative = on; }
void mega_set_wait_cycles(MegaHandle *h, long long cycles) {
    h->params.wait_cycles = cycles;
    h->params.attn.wait_cycles = cycles;
}

cudaError_t mega_launch(const MegaHandle *h, cudaStream_t s, uint64_t *launches) {
    cudaError_t e = cudaErrorInvalidValue;
    if (h->hd == 64) e = launch_variant<64>(*h, s);
    if (h->hd == 128) e = launch_variant<128>(*h, s);
    if (e == cudaSuccess) *launches += 1;
    return e;
}

// One launch with skewed epochs (see MegaParams::epoch_skew) and a budget of its own; the caller synchronises
// and reads the status word.
cudaError_t mega_launch_selftest(const MegaHandle *h, long long budget, cudaStream_t s, uint64_t *launches) {
    MegaHandle t = *h;
    t.params.epoch_skew = 0x40000000u;
    t.params.wait_cycles = budget;
    t.params.attn.wait_cycles = budget;
    return mega_launch(&t, s, launches);
}

void mega_destroy(MegaHandle *h) {
    // timing aid (YULE_MEGA_PROF=<file> in a debug process): the stamps of the last token, with the phase kinds
    const char *path = knob("YULE_MEGA_PROF");
    if (h && h->params.prof && path) {
        const size_t n = (size_t)h->grid * (h->params.n_phases + 1) * 4;
        std::vector<unsigned long long> stamps(n);
        if (cudaMemcpy(stamps.data(), h->params.prof, n * 8, cudaMemcpyDeviceToHost) == cudaSuccess) {
            if (FILE *f = fopen(path, "wb")) {
                const uint32_t hdr[2] = {h->grid, h->params.n_phases};
                fwrite(hdr, 4, 2, f);
                for (const Phase &P : h->phases) {
                    const uint32_t kind = P.kind & 0xFFu;
                    fwrite(&kind, 4, 1, f);
                }
                fwrite(stamps.data(), 8, n, f);
                fclose(f);
            }
        }
    }
    delete h;
}

}  // namespace yule
