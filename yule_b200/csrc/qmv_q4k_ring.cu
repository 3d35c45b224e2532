// qmv_q4k_ring.cu — Q4_K fused dequantise + matvec (one activation vector), weights staged through a
// shared-memory ring by bulk copies.
//
// Same arithmetic as qmv_q4k_mma.cu (yule-core/src/dequant.rs:929-972 on the tensor pipe: unscaled
// nibbles as fp16 subnormals, x split into fp16 hi/lo, fp32 accumulation, scales applied in fp32) and
// the same fused prologue / epilogue (RMSNorm, up to three matrices sharing x, SiLU(gate)·up, residual,
// tensor-parallel pairs).  What differs is how the bytes travel and what a CTA costs:
//
//   * Raw super-blocks go HBM → shared memory with 1-D `cp.async.bulk` copies, one per row of a stage
//     (16 rows × up to 8 super-blocks), completion counted by an mbarrier per stage.  The copies of the
//     first stages are issued before `griddepcontrol.wait`: a matvec launched with programmatic dependent
//     launch has its weights in flight (or already landed) while its predecessor is still computing;
//     only the activation read waits for the predecessor.
//   * No weights live in registers between iterations, so the kernel fits in 64 registers per thread
//     and, for the usual shapes, in half an SM's shared memory: predecessor and successor are resident
//     on the same SM at the same time, which is what makes the early copies possible.
//   * Rows in shared memory are 16 bytes further apart than in HBM (pitch 1168 B for 1152 B of blocks):
//     the 16-byte fragment reads of the eight row-lanes of a quarter warp fall into distinct banks.
//
// Schedule.  A CTA has two groups of 8 warps.  Tiles of 16 rows are dealt round-robin to the groups of
// the grid (in pair mode a job is the gate tile followed by the up tile of the same rows).  A job is
// `chunks` stages per matrix; warp w of the group multiplies super-block 8·chunk + w of all 16 rows.
// A stage slot is released by the eight warps through a counter; the warp that releases it last issues
// the copies of the stage that will reuse it, so nobody ever waits for an "empty" signal.
// Every wait on a copy is bounded: when it runs out the group records kStatusRingTimeout and leaves.

#include <cstdlib>

#include <cuda.h>
#include <cuda_fp16.h>

#include "internal.h"

namespace yule {

namespace {

#include "q4k_mma_common.cuh"
#include "q4k_ring_common.cuh"
#include "ring_common.cuh"

constexpr int kMaxStages = 6;                                       // per group
constexpr size_t kHalfSmSmem = 115712;                              // (228 KB − 2 × 1 KB reserved) / 2
constexpr size_t kFullSmSmem = 227 * 1024;
constexpr size_t kRingPartialBytes = (size_t)kGroups * 2 * 2 * kWarps * 16 * sizeof(float);  // [group][buffer][matrix][warp][row]

struct Q4kRingParams {
    // One tiled view per matrix (8-byte elements, box = 16 rows x the shared-memory row pitch): a stage is ONE copy
    // instruction.  A copy per row (16 per stage) cost the issuing warp about 0.7 µs, on the critical path of its group.
    CUtensorMap map[3];
    const uint8_t *w[3];
    float *out[3];
    uint32_t seg_tiles[3];
    uint32_t seg_rows[3];
    uint32_t n_seg;
    uint32_t n_tiles;  // jobs: 16-row tiles over all segments (pair mode: tiles of one matrix)
    uint32_t pair;
    const float *x;
    uint32_t n_cols;
    const float *norm_w;
    float eps;
    const float *residual;
    uint32_t stages;  // ring depth per group
    uint32_t chunks;  // stages per (tile, matrix) = ceil(super-blocks per row / 8)
    int *status;      // device status word, or null
    long long wait_cycles;
    uint32_t late_wait;  // inputs are not written by the previous kernel: only the stores wait for it
    TpFuse tp;
    unsigned long long *prof;  // timing aid (PROF instantiation only): [launch % 64][CTA][group][8] clock stamps
    uint32_t prof_launch;
};
constexpr int kProfLaunches = 64, kProfCtas = 304, kProfWords = 16;

struct RingSmem {
    unsigned char *ring;  // [group][stage][row][kRowPitch]
    SmemLayout x;         // activation image (xb, sb, sf, zb, inv_scale, red); `partial` unused
    float *partial;
    uint64_t *bars;       // [group][kMaxStages] "stage full"
    uint32_t *cnt;        // [group][kMaxStages] releases so far
};

__host__ __device__ inline size_t ring_fixed_bytes(uint32_t n_cols) {
    size_t off = xb_bytes(n_cols, 1) + 2 * sb_bytes(n_cols, 1);
    off = (off + 15) & ~(size_t)15;
    off += kZeroBytes + 16 /*inv_scale*/ + 64 * sizeof(float) /*red*/ + kRingPartialBytes;
    off += (size_t)kGroups * kMaxStages * (8 + 4);
    return (off + 127) & ~(size_t)127;
}
__host__ __device__ inline size_t ring_smem_bytes(uint32_t n_cols, uint32_t stages) {
    return (size_t)kGroups * stages * kStageBytes + ring_fixed_bytes(n_cols);
}

__device__ __forceinline__ RingSmem carve_ring(unsigned char *base, uint32_t n_cols, uint32_t stages) {
    RingSmem s;
    s.ring = base;
    size_t off = (size_t)kGroups * stages * kStageBytes;
    s.x.xb = reinterpret_cast<uint4 *>(base + off);
    off += xb_bytes(n_cols, 1);
    s.x.sb = reinterpret_cast<uint32_t *>(base + off);
    off += sb_bytes(n_cols, 1);
    s.x.sf = reinterpret_cast<float *>(base + off);
    off += sb_bytes(n_cols, 1);
    off = (off + 15) & ~(size_t)15;
    s.x.zb = reinterpret_cast<uint4 *>(base + off);
    off += kZeroBytes;
    s.x.inv_scale = reinterpret_cast<float *>(base + off);
    off += 16;
    s.x.red = reinterpret_cast<float *>(base + off);
    off += 64 * sizeof(float);
    s.x.partial = nullptr;
    s.partial = reinterpret_cast<float *>(base + off);
    off += kRingPartialBytes;
    s.bars = reinterpret_cast<uint64_t *>(base + off);
    off += (size_t)kGroups * kMaxStages * 8;
    s.cnt = reinterpret_cast<uint32_t *>(base + off);
    return s;
}

// Position in a group's stage sequence: job k (tile first_tile + k·tile_stride), matrix q, chunk c.
struct Cur {
    uint32_t k, q, c;
};
__device__ __forceinline__ void cur_advance(Cur &u, uint32_t by, uint32_t chunks, uint32_t nq) {
    u.c += by;
    while (u.c >= chunks) {
        u.c -= chunks;
        if (++u.q == nq) {
            u.q = 0;
            u.k++;
        }
    }
}
// Segment and tile-within-segment of job k.
__device__ __forceinline__ void locate_job(const Q4kRingParams &p, uint32_t tile, uint32_t q, uint32_t &seg, uint32_t &seg_tile) {
    seg = 0;
    if (p.pair) {
        seg = q;
    } else {
        while (seg + 1 < p.n_seg && tile >= p.seg_tiles[seg]) {
            tile -= p.seg_tiles[seg];
            seg++;
        }
    }
    seg_tile = tile;
}

// Issues the copy of one stage; called by a whole (converged) warp, done by its first lane.  The box is as wide as the
// shared-memory row pitch, so the padding between rows comes with the copy (what lies beyond the eight super-blocks of
// the chunk — the next block, the next row or zeros — is never read); rows past the end of the matrix arrive as zeros.
__device__ __forceinline__ void issue_stage(const Q4kRingParams &p, const Cur &u, uint32_t first_tile, uint32_t tile_stride,
                                            uint32_t bpr, uint32_t dst, uint32_t bar, int lane) {
    (void)bpr;
    if (lane == 0) {
        uint32_t seg, tile;
        locate_job(p, first_tile + u.k * tile_stride, u.q, seg, tile);
        mbar_arrive_expect_tx(bar, kStageBytes);
        asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];" ::"r"(dst),
                     "l"(reinterpret_cast<uint64_t>(&p.map[seg])), "r"(bar), "r"(u.c * kStageBlocks * 18u), "r"(tile * kStageRows)
                     : "memory");
    }
    __syncwarp();
}

__device__ __forceinline__ void ring_group_barrier(int group) {
    asm volatile("bar.sync %0, %1;" ::"r"(1 + group), "r"(kWarps * 32) : "memory");
}

// Activation staging by one 8-warp group, without any CTA-wide barrier.  Warp w multiplies super-blocks
// w, w+8, … of every tile, so it converts exactly those 256-column slices of x (lane l: columns 8l..8l+7 of
// each) into the fragment image, reads back only what it wrote, and needs the other warps only for the two
// scalars that depend on all of x (Σx² for RMSNorm, max|x| for the power-of-two scale): one named barrier.
// Both groups of a CTA write the same bytes to the same places of the shared image; neither reads the
// other's.  Returns 2^-e (the factor that undoes the scale).
template <bool TP>
__device__ __forceinline__ float stage_x_group(const SmemLayout &sm, const float *__restrict__ x, uint32_t bpr,
                                               const float *__restrict__ norm_w, float eps, uint32_t n_cols, int group, int wid,
                                               int lane, const uint2 *pairs, uint32_t pair_epoch, int *status, long long budget) {
    constexpr int KC = 2;  // slices kept in registers between the reduction and the conversion
    const uint32_t tid = threadIdx.x & (kWarps * 32 - 1);
    if (tid < 64) sm.zb[tid] = make_uint4(0u, 0u, 0u, 0u);
    float cache[KC][8];
    float ss = 0.f, mx = 0.f;
    auto load8 = [&](uint32_t c, float (&a)[8]) {
        if (TP && pairs) {
            tp_load8(pairs + c, pair_epoch, status, budget, a);
            return;
        }
        *reinterpret_cast<float4 *>(a) = *reinterpret_cast<const float4 *>(x + c);
        *reinterpret_cast<float4 *>(a + 4) = *reinterpret_cast<const float4 *>(x + c + 4);
    };
    auto reduce8 = [&](uint32_t c, const float (&a)[8]) {
        float gw[8];
        if (norm_w) {
            *reinterpret_cast<float4 *>(gw) = *reinterpret_cast<const float4 *>(norm_w + c);
            *reinterpret_cast<float4 *>(gw + 4) = *reinterpret_cast<const float4 *>(norm_w + c + 4);
        }
#pragma unroll
        for (int i = 0; i < 8; i++) {
            ss = fmaf(a[i], a[i], ss);
            mx = fmaxf(mx, fabsf(norm_w ? a[i] * gw[i] : a[i]));
        }
    };
#pragma unroll
    for (int i = 0; i < KC; i++) {
        const uint32_t b = (uint32_t)wid + 8u * i;
        if (b < bpr) {
            load8(b * 256u + lane * 8u, cache[i]);
            reduce8(b * 256u + lane * 8u, cache[i]);
        }
    }
    for (uint32_t b = (uint32_t)wid + 8u * KC; b < bpr; b += 8u) {
        float a[8];
        load8(b * 256u + lane * 8u, a);
        reduce8(b * 256u + lane * 8u, a);
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        ss += __shfl_xor_sync(0xffffffffu, ss, o);
        mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
    }
    float *red = sm.red + group * 16;
    if (lane == 0) {
        red[wid] = ss;
        red[8 + wid] = mx;
    }
    ring_group_barrier(group);
    {
        const float4 s0 = *reinterpret_cast<const float4 *>(red), s1 = *reinterpret_cast<const float4 *>(red + 4);
        const float4 m0 = *reinterpret_cast<const float4 *>(red + 8), m1 = *reinterpret_cast<const float4 *>(red + 12);
        ss = ((((((s0.x + s0.y) + s0.z) + s0.w) + s1.x) + s1.y) + s1.z) + s1.w;  // fixed order: both groups get the same bits
        mx = fmaxf(fmaxf(fmaxf(m0.x, m0.y), fmaxf(m0.z, m0.w)), fmaxf(fmaxf(m1.x, m1.y), fmaxf(m1.z, m1.w)));
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
    auto convert8 = [&](uint32_t c, float (&a)[8]) {
        if (norm_w) {
            float gw[8];
            *reinterpret_cast<float4 *>(gw) = *reinterpret_cast<const float4 *>(norm_w + c);
            *reinterpret_cast<float4 *>(gw + 4) = *reinterpret_cast<const float4 *>(norm_w + c + 4);
            // x * inv * w, rounded in that order (yule-infer/src/model_runner.rs:273)
#pragma unroll
            for (int i = 0; i < 8; i++) a[i] = a[i] * inv_rms * gw[i];
        }
        __half hi[8], lo[8];
#pragma unroll
        for (int i = 0; i < 8; i++) {
            a[i] *= scale;  // exact (power of two)
            hi[i] = __float2half_rn(a[i]);
            lo[i] = __float2half_rn(a[i] - __half2float(hi[i]));
        }
        float s8 = ((a[0] + a[1]) + (a[2] + a[3])) + ((a[4] + a[5]) + (a[6] + a[7]));
        const uint32_t blk = c >> 8, tt = (c >> 6) & 3, h = (c >> 5) & 1, wp = (c >> 3) & 3;
        const uint32_t idx = ((blk * 2 + h) * 4 + wp) * 8 + tt;
        sm.xb[idx] = make_uint4(h2_as_u32(__halves2half2(hi[0], hi[2])), h2_as_u32(__halves2half2(hi[1], hi[3])),
                                h2_as_u32(__halves2half2(hi[4], hi[6])), h2_as_u32(__halves2half2(hi[5], hi[7])));
        sm.xb[idx + 4] = make_uint4(h2_as_u32(__halves2half2(lo[0], lo[2])), h2_as_u32(__halves2half2(lo[1], lo[3])),
                                    h2_as_u32(__halves2half2(lo[4], lo[6])), h2_as_u32(__halves2half2(lo[5], lo[7])));
        // Σ over 32 columns: 4 consecutive lanes hold one sub-block
        s8 += __shfl_xor_sync(0xffffffffu, s8, 1);
        s8 += __shfl_xor_sync(0xffffffffu, s8, 2);
        if ((lane & 3) == 0) sm.sf[c >> 5] = s8;
    };
#pragma unroll
    for (int i = 0; i < KC; i++) {
        const uint32_t b = (uint32_t)wid + 8u * i;
        if (b < bpr) convert8(b * 256u + lane * 8u, cache[i]);
    }
    for (uint32_t b = (uint32_t)wid + 8u * KC; b < bpr; b += 8u) {
        float a[8];
        load8(b * 256u + lane * 8u, a);
        convert8(b * 256u + lane * 8u, a);
    }
    __syncwarp();
    return __uint_as_float((uint32_t)(254 - se) << 23);
}


template <bool TP, bool PROF>
__global__ void __launch_bounds__(kThreadsCta, 2)
qmv_q4k_ring_kernel(const __grid_constant__ Q4kRingParams p) {
    extern __shared__ __align__(128) unsigned char smem_raw[];
    unsigned long long *prof = nullptr;
    if (PROF) {
        prof = p.prof + (((size_t)(p.prof_launch % kProfLaunches) * kProfCtas + blockIdx.x) * kGroups + (threadIdx.x >> 8)) * kProfWords;
        if ((threadIdx.x & 255) == 0) {
            uint32_t smid;
            asm volatile("mov.u32 %0, %%smid;" : "=r"(smid));
            prof[0] = clock64();
            prof[7] = smid;
        }
    }
    yule_pdl_launch_dependents();

    const int lane = threadIdx.x & 31;
    const int group = threadIdx.x >> 8, wid = (threadIdx.x >> 5) & (kWarps - 1);
    const int g = lane >> 2, t = lane & 3;
    const uint32_t bpr = p.n_cols / 256;
    const uint32_t nq = p.pair ? 2u : 1u;
    const uint32_t G = gridDim.x;
    const uint32_t first_tile = blockIdx.x + group * G, tile_stride = kGroups * G;
    const uint32_t my_tiles = p.n_tiles > first_tile ? (p.n_tiles - first_tile + tile_stride - 1) / tile_stride : 0;
    const uint32_t S = p.stages, chunks = p.chunks;
    const uint32_t total = my_tiles * nq * chunks;  // stages this group consumes

    const RingSmem sm = carve_ring(smem_raw, p.n_cols, S);
    unsigned char *ring = sm.ring + (size_t)group * S * kStageBytes;
    const uint32_t ring_u32 = smem_u32(ring);
    const uint32_t bar0 = smem_u32(sm.bars + group * kMaxStages);
    uint32_t *cnt = sm.cnt + group * kMaxStages;

    // Warp 0 of each group sets the group's barriers up and starts the first copies; the other warps see
    // both through the group barrier of the activation staging, which they pass before their first wait.
    if (total == 0) return;  // a group without tiles takes no part in anything below
    if (wid == 0) {
        if (lane == 0) {
            for (int i = 0; i < kMaxStages; i++) {
                mbar_init(bar0 + 8 * i, 1);
                cnt[i] = 0;
            }
            asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        }
        __syncwarp();
        Cur u = {0u, 0u, 0u};
        for (uint32_t n = 0; n < S && n < total; n++) {
            issue_stage(p, u, first_tile, tile_stride, bpr, ring_u32 + n * kStageBytes, bar0 + 8 * n, lane);
            cur_advance(u, 1, chunks, nq);
        }
    }

    if (PROF && (threadIdx.x & 255) == 0) prof[1] = clock64();
    if (!p.late_wait) yule_pdl_wait();  // the activations (and the residual) come from the previous kernel
    if (PROF && (threadIdx.x & 255) == 0) prof[2] = clock64();
    const float inv_scale =
        TP ? stage_x_group<true>(sm.x, p.x, bpr, p.norm_w, p.eps, p.n_cols, group, wid, lane, p.tp.wait ? p.tp.pair_in : nullptr,
                                 p.tp.wait ? *p.tp.tick * p.tp.epochs_per_tick + p.tp.wait_index + 1u : 0u, p.tp.status, p.tp.wait_cycles)
           : stage_x_group<false>(sm.x, p.x, bpr, p.norm_w, p.eps, p.n_cols, group, wid, lane, nullptr, 0u, nullptr, 0);
    if (PROF && (threadIdx.x & 255) == 0) prof[3] = clock64();

    // B column n = g is live only for g = t (hi part) and g = t + 4 (lo part); the other lanes read zeros
    const bool feeds = (g & 3) == t;
    const uint4 *sub_base = feeds ? sm.x.xb + (g >> 2) * 4 + t : sm.x.zb;
    const uint32_t sub_stride = feeds ? 64u : 0u;
    const int u = t & 1;
    const bool charge_mins = t < 2;
    const uint32_t n_warps_used = bpr < (uint32_t)kWarps ? bpr : (uint32_t)kWarps;
    float *part_base = sm.partial + (size_t)group * (2 * 2 * kWarps * 16);

    Cur cu = {0u, 0u, 0u};
    float acc0 = 0.f, acc1 = 0.f;
    uint32_t slot = 0, phase = 0;
    for (uint32_t n = 0; n < total; n++) {
        const uint32_t bar = bar0 + 8 * slot;
        if (!ring_wait(bar, phase, p.status, p.wait_cycles)) return;  // all eight warps of the group wait on the same copy
        if (PROF && n == 0 && (threadIdx.x & 255) == 0) prof[4] = clock64();
        const uint32_t blk0 = cu.c * kStageBlocks;
        const uint32_t nblk = bpr - blk0 < (uint32_t)kStageBlocks ? bpr - blk0 : (uint32_t)kStageBlocks;
        if ((uint32_t)wid < nblk) {
            const unsigned char *r0 = ring + (size_t)slot * kStageBytes + (uint32_t)g * kRowPitch + (uint32_t)wid * 144u;
            const uint32_t blk = blk0 + wid;
            consume_block_smem(r0, r0 + 8 * kRowPitch, sub_base + (size_t)blk * sub_stride, sm.x.sf + (size_t)blk * 8 + 4 * u, u, t,
                               charge_mins, acc0, acc1);
        }
        if (PROF && n == 0 && (threadIdx.x & 255) == 0) prof[8] = clock64();
        // release the slot (only when some later stage will reuse it); the warp that releases it last refills it
        if (n + S < total) {
            __syncwarp();
            uint32_t last = 0;
            if (lane == 0) {
                __threadfence_block();
                last = ((atomicAdd(&cnt[slot], 1u) & (kWarps - 1)) == kWarps - 1) ? 1u : 0u;
            }
            last = __shfl_sync(0xffffffffu, last, 0);
            if (last) {
                Cur nx = cu;
                cur_advance(nx, S, chunks, nq);
                issue_stage(p, nx, first_tile, tile_stride, bpr, ring_u32 + slot * kStageBytes, bar, lane);
            }
        }
        if (PROF && n == 0 && (threadIdx.x & 255) == 0) prof[9] = clock64();
        if (cu.c + 1 == chunks) {
            // this matrix's rows are complete in this warp: sum the four column groups, park the 16 row sums
            float v0 = acc0, v1 = acc1;
            v0 += __shfl_xor_sync(0xffffffffu, v0, 1);
            v1 += __shfl_xor_sync(0xffffffffu, v1, 1);
            v0 += __shfl_xor_sync(0xffffffffu, v0, 2);
            v1 += __shfl_xor_sync(0xffffffffu, v1, 2);
            float *part = part_base + (size_t)(cu.k & 1u) * (2 * kWarps * 16) + (size_t)cu.q * (kWarps * 16);
            if (t == 0) {
                part[wid * 16 + g] = v0;
                part[wid * 16 + g + 8] = v1;
            }
            acc0 = acc1 = 0.f;
            if (cu.q + 1 == nq) {
                // job complete: one barrier, then 128 threads finish the 16 rows — eight lanes per row fetch the
                // eight warps' sums and add them in a fixed tree.  The partial buffers alternate between jobs,
                // so the next job's sums cannot overtake these reads (a warp passes the next barrier only
                // after the first four warps have finished here).
                const uint32_t tid = threadIdx.x & (kWarps * 32 - 1);
                uint32_t seg = 0, tile = 0;
                if (tid < 128u) locate_job(p, first_tile + cu.k * tile_stride, 0, seg, tile);
                if (PROF && cu.k == 0 && (threadIdx.x & 255) == 0) prof[10] = clock64();
                if (p.late_wait) yule_pdl_wait();  // the previous kernel is settled before our stores
                ring_group_barrier(group);
                if (PROF && cu.k == 0 && (threadIdx.x & 255) == 0) prof[11] = clock64();
                if (tid < 128u) {
                    const uint32_t rr = tid >> 3, w2 = tid & 7u;
                    const float *pb = part_base + (size_t)(cu.k & 1u) * (2 * kWarps * 16);
                    float s0 = w2 < n_warps_used ? pb[w2 * 16 + rr] : 0.f;
                    float s1 = (p.pair && w2 < n_warps_used) ? pb[(kWarps + w2) * 16 + rr] : 0.f;
#pragma unroll
                    for (int o = 1; o < 8; o <<= 1) {
                        s0 += __shfl_xor_sync(0xffffffffu, s0, o);
                        s1 += __shfl_xor_sync(0xffffffffu, s1, o);
                    }
                    const uint32_t row = tile * kStageRows + rr;
                    if (w2 == 0 && row < p.seg_rows[seg]) {
                        s0 *= inv_scale;
                        if (p.pair) {
                            // silu_mul.cu: x / (1 + exp(−x)) * up
                            s1 *= inv_scale;
                            s0 = (s0 / (1.0f + expf(-s0))) * s1;
                        } else if (seg == 0 && p.residual) {
                            s0 += p.residual[row];
                        }
                        p.out[seg][row] = s0;
                        if (TP && p.tp.push && seg == 0) tp_push_value(p.tp, row, s0);
                    }
                }
                if (PROF && cu.k == 0 && (threadIdx.x & 255) == 0) prof[12] = clock64();
            }
        }
        cur_advance(cu, 1, chunks, nq);
        if (++slot == S) {
            slot = 0;
            phase ^= 1u;
        }
    }
    if (PROF && (threadIdx.x & 255) == 0) {
        prof[5] = clock64();
        prof[6] = total;
    }
}

// Timing aid (YULE_QMV_PROF=<file> in a debug process): clock stamps of every CTA of the last 64 launches,
// written to the file when the process ends.
unsigned long long *g_prof_dev = nullptr;
uint32_t g_prof_launches = 0;
std::string g_prof_path;
void prof_dump() {
    if (!g_prof_dev) return;
    const size_t n = (size_t)kProfLaunches * kProfCtas * kGroups * kProfWords;
    std::vector<unsigned long long> h(n);
    if (cudaMemcpy(h.data(), g_prof_dev, n * 8, cudaMemcpyDeviceToHost) != cudaSuccess) return;
    if (FILE *f = fopen(g_prof_path.c_str(), "wb")) {
        fwrite(&g_prof_launches, 4, 1, f);
        fwrite(h.data(), 8, n, f);
        fclose(f);
    }
}

template <bool TP, bool PROF = false>
cudaError_t launch_ring_variant(const Q4kRingParams &p, uint32_t grid, size_t smem, bool pdl, cudaStream_t s) {
    auto kern = qmv_q4k_ring_kernel<TP, PROF>;
    // the opt-in for large dynamic shared memory is a per-device attribute
    static bool attr_done[64] = {};
    static std::mutex mu;
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return e;
    {
        std::lock_guard<std::mutex> lock(mu);
        if (dev < 0 || dev >= 64 || !attr_done[dev]) {
            e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kFullSmSmem);
            if (e != cudaSuccess) return e;
            if (dev >= 0 && dev < 64) attr_done[dev] = true;
        }
    }
    return launch_kernel(kern, dim3(grid), dim3(kThreadsCta), smem, s, pdl, p);
}

}  // namespace

bool q4k_ring_supported(const Q4kFused &f) {
    if (f.q5 || f.batch != 1 || f.n_cols == 0 || f.n_cols % 256) return false;
    if (f.x_stride != f.n_cols && f.batch > 1) return false;
    for (uint32_t i = 0; i < f.n_seg; i++) {
        if (reinterpret_cast<uintptr_t>(f.w[i]) & 15) return false;
        if (f.out_stride[i] != f.rows[i] && f.batch > 1) return false;
    }
    if (reinterpret_cast<uintptr_t>(f.x) & 15) return false;
    return ring_smem_bytes(f.n_cols, 2) <= kFullSmSmem;
}

cudaError_t launch_q4k_ring(const Q4kFused &f, int sm_count, cudaStream_t s, uint64_t *launches) {
    Q4kRingParams p = {};
    for (uint32_t i = 0; i < f.n_seg; i++) {
        const uint32_t bpr_i = f.n_cols / 256;
        cudaError_t me = cached_tensor_map_2d(f.w[i], 8, (uint64_t)bpr_i * 18, f.rows[i], (uint64_t)bpr_i * 144, kRowPitch / 8, kStageRows, &p.map[i]);
        if (me != cudaSuccess) return me;
    }
    const bool pair = f.swiglu_pair;
    uint32_t n_tiles = 0;
    for (uint32_t i = 0; i < f.n_seg; i++) {
        p.w[i] = f.w[i];
        p.out[i] = f.out[i];
        p.seg_rows[i] = f.rows[i];
        p.seg_tiles[i] = (f.rows[i] + kStageRows - 1) / kStageRows;
        if (!pair || i == 0) n_tiles += p.seg_tiles[i];
    }
    if (n_tiles == 0) return cudaSuccess;
    p.n_seg = f.n_seg;
    p.n_tiles = n_tiles;
    p.pair = pair ? 1 : 0;
    p.x = f.x;
    p.n_cols = f.n_cols;
    p.norm_w = f.norm_w;
    p.eps = f.eps;
    p.residual = f.residual;
    p.status = f.status;
    p.wait_cycles = f.wait_cycles;
    p.late_wait = (f.pdl && f.late_wait) ? 1u : 0u;
    p.tp = f.tp;
    const uint32_t bpr = f.n_cols / 256;
    p.chunks = (bpr + kStageBlocks - 1) / kStageBlocks;
    // Grid: every group gets whole jobs, one CTA per SM: the other half of each SM is where the neighbouring
    // launches run (measured: two CTAs of one launch per SM are slower than one CTA each of two launches).
    uint32_t max_ctas = (uint32_t)sm_count;
    if (const char *k = knob("YULE_QMV_RING_CTAS")) max_ctas = (uint32_t)atoi(k) > 0 ? (uint32_t)atoi(k) : max_ctas;
    uint32_t grid = (n_tiles + kGroups - 1) / kGroups;
    if (grid > max_ctas) grid = max_ctas;
    // Ring depth: what fits in half an SM next to the activation image, at least two stages per group (then
    // the CTA may need more than half an SM), no more than a group will ever consume.
    const size_t fixed = ring_fixed_bytes(f.n_cols);
    uint32_t stages = fixed + 2 * (size_t)kGroups * kStageBytes <= kHalfSmSmem
                          ? (uint32_t)((kHalfSmSmem - fixed) / ((size_t)kGroups * kStageBytes))
                          : (uint32_t)((kFullSmSmem - fixed) / ((size_t)kGroups * kStageBytes));
    if (stages > (uint32_t)kMaxStages) stages = kMaxStages;
    const uint32_t jobs_per_group = (n_tiles + kGroups * grid - 1) / (kGroups * grid);
    const uint32_t need = jobs_per_group * (pair ? 2u : 1u) * p.chunks;
    if (stages > need) stages = need;
    if (stages < 1) return cudaErrorInvalidValue;
    p.stages = stages;
    const size_t smem = ring_smem_bytes(f.n_cols, stages);
    cudaError_t e;
    if (const char *path = knob("YULE_QMV_PROF")) {
        if (!g_prof_dev) {
            const size_t n = (size_t)kProfLaunches * kProfCtas * kGroups * kProfWords;
            if (cudaMalloc((void **)&g_prof_dev, n * 8) != cudaSuccess) return cudaErrorMemoryAllocation;
            cudaMemset(g_prof_dev, 0, n * 8);
            g_prof_path = path;
            atexit(prof_dump);
        }
        p.prof = g_prof_dev;
        p.prof_launch = g_prof_launches++;
        if (grid > (uint32_t)kProfCtas) return cudaErrorInvalidValue;
        e = launch_ring_variant<false, true>(p, grid, smem, f.pdl, s);
    } else {
        e = (f.tp.push || f.tp.wait) ? launch_ring_variant<true>(p, grid, smem, f.pdl, s)
                                     : launch_ring_variant<false>(p, grid, smem, f.pdl, s);
    }
    if (e != cudaSuccess) return e;
    *launches += 1;
    return cudaSuccess;
}

}  // namespace yule
