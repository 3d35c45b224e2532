// qmv_q4k_mma.cu — Q4_K fused dequantise + matvec on the tensor pipe, with the neighbouring
// element-wise ops of the decode step folded in.
//
// Why tensor cores for a matvec: at 0.5625 bytes per weight, HBM delivers ~11.6 T weights/s; the
// SIMT route (extract nibble, convert, FMA ≈ 3–4 issue slots per weight) needs more issue slots
// than the SMs have, so it is ALU-bound below the memory roofline.  `mma.sync.m16n8k16` takes the
// multiply-accumulate off the issue budget and leaves ~1.9 slots per weight (unpack + scale).
//
// Exactness.  The contract is yule-core/src/dequant.rs:929-972:
//     sum += (d*sc_s) * Σ_l q_l x_l − (dmin*mn_s) * Σ_l x_l        per 32-column sub-block s.
// Operands are fed to the tensor core without rounding:
//   A (weights)  q·sc_s as fp16 — an integer ≤ 15·63 = 945, exact.  Built from the packed nibbles
//                as (1024+q)·sc − 1024·sc in one fp16 FMA (exact: the product fits in the FMA's
//                internal precision and the result is an integer < 2048).
//   B (x)        x·2^e split into hi = fp16(x·2^e) and lo = fp16(x·2^e − hi): two columns of the
//                8-wide B tile, summed after the MMA.  2^e normalises max|x| to [2^13, 2^14) so
//                neither overflow nor fp16 subnormals cost precision (error ≤ 2^-22 relative).
//   accumulate   fp32 in the MMA; d, dmin and 2^-e are applied in fp32 afterwards.
//   mins         one extra MMA per super-block: A = mn_s, B = Σ_l x_l of each sub-block (hi/lo).
// What differs from the CPU code is only the order of the fp32 additions.
//
// Mapping.  A CTA of 8 warps owns ROWS (16 or 8) consecutive rows; warp w takes super-blocks
// w, w+8, … of those rows.  Lane (g = lane/4, t = lane%4) holds rows g and g+8 and the 64-column
// group t of the super-block: 32 bytes of qs per row plus the 16-byte header — all 16-byte
// loads, issued for the warp's first super-block before anything else, the next super-block's
// while the current one is being multiplied.  The k index of the MMA is a free permutation
// (A and B agree on it), so nibbles go straight from the loaded words into fragments.
// Cross-warp sums go through 2 KB of shared memory in a fixed order (deterministic).
//
// Fused around the matvec (each replaces a dispatch of yule-infer/src/gpu_runner.rs:296-695):
//   prologue  RMSNorm of x (rms_norm.cu) computed per CTA while the weight loads are in flight;
//   segments  up to three matrices sharing x in one launch (Q/K/V);
//   epilogue  + residual (add.cu), or SiLU(gate)·up (silu_mul.cu) for a gate/up pair.
// Programmatic dependent launch: weights do not depend on the previous kernel, so their loads are
// issued before `griddepcontrol.wait`; only the activation read waits.

#include <cstdlib>

#include <cuda_fp16.h>

#include "internal.h"

namespace yule {

namespace {

constexpr int kWarps = 8;  // warps per group: one per super-block slot of a tile

__device__ __forceinline__ uint4 ld_stream_u4(const uint4 *p) {
    uint4 v;
    // L1-allocating on purpose: neighbouring 16-byte pieces share 32-byte sectors, and the second
    // request then merges with the first in L1 instead of going to L2 again.
    asm volatile("ld.global.nc.L1::evict_first.v4.u32 {%0,%1,%2,%3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
                 : "l"(p));
    return v;
}
__device__ __forceinline__ uint2 ld_stream_u2(const void *p) {
    uint2 v;
    asm volatile("ld.global.nc.L1::evict_first.v2.u32 {%0,%1}, [%2];" : "=r"(v.x), "=r"(v.y) : "l"(p));
    return v;
}

__device__ __forceinline__ void mma_16816(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                          uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

__device__ __forceinline__ uint32_t h2_as_u32(__half2 h) { return *reinterpret_cast<uint32_t *>(&h); }
__device__ __forceinline__ __half2 u32_as_h2(uint32_t u) { return *reinterpret_cast<__half2 *>(&u); }

// The three 16-byte pieces one lane needs from one super-block of one row.
// Q5_K (dequant.rs:297-338) adds the 32 bytes of fifth bits that sit between header and nibbles:
// bit s of byte l belongs to sub-block s, column l.  All four lanes of a row need all 32 bytes;
// each keeps a quarter (bytes 8t..8t+7) and hands words out by shuffle when the block is used.
struct BlockLoads {
    uint4 hdr, qa, qb;
    uint2 f;  // Q5_K only
};

template <int NR, bool Q5>  // rows per lane: 2 (ROWS = 16) or 1 (ROWS = 8)
__device__ __forceinline__ void issue_loads(BlockLoads (&ld)[NR], const uint4 *const (&rowp)[NR], uint32_t blk, int t) {
#pragma unroll
    for (int r = 0; r < NR; r++) {
        const uint4 *bp = rowp[r] + (size_t)blk * (Q5 ? 11 : 9);
        ld[r].hdr = ld_stream_u4(bp);
        if (Q5) ld[r].f = ld_stream_u2(reinterpret_cast<const uint2 *>(bp + 1) + t);
        ld[r].qa = ld_stream_u4(bp + (Q5 ? 3 : 1) + 2 * t);
        ld[r].qb = ld_stream_u4(bp + (Q5 ? 4 : 2) + 2 * t);
    }
}

// Fifth bits of the four columns of word wi for this lane's group t, moved to bit 0 of each byte:
// `.x` for the low-nibble sub-block 2t, `.y` for the high-nibble sub-block 2t+1.
// Word wi of the 32 bytes of fifth bits: it lives in lane (wi >> 1) of this row's quad; every lane of
// the warp takes part in the shuffle.
template <bool Q5>
__device__ __forceinline__ uint32_t fifth_word(const BlockLoads &b, int wi) {
    if (!Q5) return 0u;
    return __shfl_sync(0xFFFFFFFFu, (wi & 1) ? b.f.y : b.f.x, wi >> 1, 4);
}
template <bool Q5>
__device__ __forceinline__ uint2 fifth_of(const BlockLoads &b, int wi, int t) {
    if (!Q5) return make_uint2(0u, 0u);
    const uint32_t f = fifth_word<Q5>(b, wi) >> (2 * t);
    return make_uint2(f & 0x01010101u, (f >> 1) & 0x01010101u);
}

// Word wi (0..7) of the lane's 32 bytes of qs; wi is a compile-time constant after unrolling.
__device__ __forceinline__ uint32_t word_of(const BlockLoads &b, int wi) {
    switch (wi) {
        case 0: return b.qa.x;
        case 1: return b.qa.y;
        case 2: return b.qa.z;
        case 3: return b.qa.w;
        case 4: return b.qb.x;
        case 5: return b.qb.y;
        case 6: return b.qb.z;
        default: return b.qb.w;
    }
}

// Per-row constants of one super-block for this lane's 64-column group t.
struct RowScales {
    __half2 sc_lo, c_lo;  // low nibbles:  (1024+q)*sc_lo + c_lo          = q*sc[2t]
    __half2 sc_hi, c_hi;  // high nibbles: (1024+16q)*(sc/16) + (−64 sc)  = q*sc[2t+1]
    uint32_t mn;          // half2 {mn[2t], mn[2t+1]}
    float d, dmin;  // dmin carries the 2^6 that the stored column sums lack
};

// 6-bit scale/min unpack of yule-core/src/dequant.rs:176-190 for sub-blocks 2t and 2t+1, two
// bytes at a time.
__device__ __forceinline__ RowScales unpack_scales(const uint4 &hdr, int t) {
    const int sh = 16 * (t & 1);
    const uint32_t a0 = (hdr.y >> sh) & 0xFFFFu, a1 = (hdr.z >> sh) & 0xFFFFu, a2 = (hdr.w >> sh) & 0xFFFFu;
    uint32_t sc2, mn2;
    if (t < 2) {
        sc2 = a0 & 0x3F3Fu;
        mn2 = a1 & 0x3F3Fu;
    } else {
        sc2 = (a2 & 0x0F0Fu) | ((a0 >> 2) & 0x3030u);
        mn2 = ((a2 >> 4) & 0x0F0Fu) | ((a1 >> 2) & 0x3030u);
    }
    // bytes {v0, v1} → half2 {1024+v0, 1024+v1} → minus 1024
    const __half2 k1024 = __float2half2_rn(1024.0f);
    const __half2 sc = __hsub2(u32_as_h2(__byte_perm(sc2, 0x64u, 0x4140)), k1024);
    const __half2 mn = __hsub2(u32_as_h2(__byte_perm(mn2, 0x64u, 0x4140)), k1024);
    RowScales r;
    r.sc_lo = __low2half2(sc);
    r.c_lo = __hmul2(r.sc_lo, __float2half2_rn(-1024.0f));
    const __half2 sch = __high2half2(sc);
    r.sc_hi = __hmul2(sch, __float2half2_rn(0.0625f));
    r.c_hi = __hmul2(sch, __float2half2_rn(-64.0f));
    r.mn = h2_as_u32(mn);
    r.d = __half2float(__ushort_as_half((unsigned short)(hdr.x & 0xFFFFu)));
    r.dmin = 64.0f * __half2float(__ushort_as_half((unsigned short)(hdr.x >> 16)));  // sums are stored as Σ·2^-6
    return r;
}

// One word = 4 bytes = 4 low-nibble weights (columns c..c+3) + 4 high-nibble weights (c+32..).
// Fragment halves pair bytes (0,2) and (1,3); B is laid out to match.
// A fifth bit (Q5_K) is +16: mantissa bit 4 of 1024+q, bit 8 of 1024+16q; 31·63 < 2048 stays exact.
__device__ __forceinline__ void word_to_frags(uint32_t w, const RowScales &s, uint2 fifth, uint32_t &lo02, uint32_t &lo13,
                                              uint32_t &hi02, uint32_t &hi13) {
    const uint32_t magic = 0x64006400u;
    const uint32_t w8 = w >> 8;
    const uint32_t f_lo02 = (fifth.x & 0x00010001u) << 4, f_lo13 = ((fifth.x >> 8) & 0x00010001u) << 4;
    const uint32_t f_hi02 = (fifth.y & 0x00010001u) << 8, f_hi13 = ((fifth.y >> 8) & 0x00010001u) << 8;
    lo02 = h2_as_u32(__hfma2(u32_as_h2((w & 0x000F000Fu) | magic | f_lo02), s.sc_lo, s.c_lo));
    lo13 = h2_as_u32(__hfma2(u32_as_h2((w8 & 0x000F000Fu) | magic | f_lo13), s.sc_lo, s.c_lo));
    hi02 = h2_as_u32(__hfma2(u32_as_h2((w & 0x00F000F0u) | magic | f_hi02), s.sc_hi, s.c_hi));
    hi13 = h2_as_u32(__hfma2(u32_as_h2((w8 & 0x00F000F0u) | magic | f_hi13), s.sc_hi, s.c_hi));
}

// Shared-memory image of the activations for one CTA.  Per vector v:
//   xb[v]  uint4 index ((blk*2 + h)*4 + wp)*8 + part*4 + t  — for super-block blk, nibble half h
//          (0 = columns of the low nibbles), word pair wp, part (0 = hi, 1 = lo) and 64-column
//          group t: the B fragments of words 2wp and 2wp+1, i.e. halves
//          {x[c], x[c+2], x[c+1], x[c+3], x[c+4], x[c+6], x[c+5], x[c+7]}, c = 256 blk + 64 t + 32 h + 8 wp.
//          The eight (part, t) combinations a warp reads at once are 128 contiguous bytes.
//   sb[v]  half2 index (blk*2 + part)*4 + t = 2^-6 · {Σ sub-block 2t, Σ sub-block 2t+1}
//   inv_scale[v] = 2^-e
//   sf[v]  float index c/32 = Σ of the 32 columns (scaled by 2^e), for the batch-1 path
//   zb     64 zeroed uint4: B fragments of lanes that feed an all-zero column
struct SmemLayout {
    uint4 *xb;
    uint32_t *sb;
    float *sf;
    uint4 *zb;
    float *inv_scale;
    float *partial;  // [2 groups][kRoundSlots][kWarps][4 vectors][16 rows]
    float *red;      // reduction scratch, 2 × 32 floats
};

constexpr int kGroups = 2;       // independent 8-warp groups per CTA
constexpr int kRoundSlots = 8;   // (tile, matrix) slots whose partial sums a group holds at once

__host__ __device__ inline size_t xb_bytes(uint32_t n_cols, uint32_t nb) { return (size_t)nb * n_cols * 4; }
__host__ __device__ inline size_t sb_bytes(uint32_t n_cols, uint32_t nb) { return (size_t)nb * (n_cols / 32) * 4; }
constexpr size_t kZeroBytes = 64 * sizeof(uint4);
constexpr size_t kPartialBytes = (size_t)kGroups * kRoundSlots * kWarps * 4 * 16 * sizeof(float);

__device__ __forceinline__ SmemLayout carve(unsigned char *base, uint32_t n_cols, uint32_t nb) {
    SmemLayout s;
    size_t off = 0;
    s.xb = reinterpret_cast<uint4 *>(base);
    off += xb_bytes(n_cols, nb);
    s.sb = reinterpret_cast<uint32_t *>(base + off);
    off += sb_bytes(n_cols, nb);
    s.sf = reinterpret_cast<float *>(base + off);
    off += sb_bytes(n_cols, nb);
    off = (off + 15) & ~(size_t)15;
    s.zb = reinterpret_cast<uint4 *>(base + off);
    off += kZeroBytes;
    s.inv_scale = reinterpret_cast<float *>(base + off);
    off += 4 * sizeof(float);
    s.partial = reinterpret_cast<float *>(base + off);
    off += kPartialBytes;
    s.red = reinterpret_cast<float *>(base + off);
    return s;
}

size_t smem_bytes(uint32_t n_cols, uint32_t nb) {
    size_t off = xb_bytes(n_cols, nb) + 2 * sb_bytes(n_cols, nb);
    off = (off + 15) & ~(size_t)15;
    return off + kZeroBytes + 4 * sizeof(float) + kPartialBytes + 64 * sizeof(float) + 16;
}

constexpr int kThreadsCta = kGroups * kWarps * 32;  // 512

// Kept out of line: the tensor-parallel path must not cost the single-GPU kernels registers.
__device__ __noinline__ void tp_push_value(const TpFuse &tp, size_t o, float v) {
    const uint2 pair = make_uint2(__float_as_uint(v), *tp.tick * tp.epochs_per_tick + tp.push_index + 1u);
    for (uint32_t pp = 0; pp < tp.world; pp++)  // one 8-byte store each
        asm volatile("st.volatile.global.v2.u32 [%0], {%1, %2};" ::"l"(tp.pair_out[pp] + o), "r"(pair.x), "r"(pair.y) : "memory");
}
// Eight consecutive elements of a gathered vector from its (value, epoch) pairs: polls until all eight
// carry `epoch` (bounded: a lost peer becomes a status word, not a hung GPU).
__device__ __forceinline__ void tp_load8(const uint2 *pairs, uint32_t epoch, int *status, float (&a)[8]) {
    long long t0 = 0;
    for (uint32_t it = 0;; it++) {
        uint4 q[4];
        // one 16-byte load per two pairs: value and epoch of a pair must come from the same access
#pragma unroll
        for (int i = 0; i < 4; i++)
            asm volatile("ld.volatile.global.v4.u32 {%0, %1, %2, %3}, [%4];"
                         : "=r"(q[i].x), "=r"(q[i].y), "=r"(q[i].z), "=r"(q[i].w)
                         : "l"(pairs + 2 * i)
                         : "memory");
        bool ok = true;
#pragma unroll
        for (int i = 0; i < 4; i++) ok = ok && q[i].y == epoch && q[i].w == epoch;
        if (!ok) {
            if (it == 0) t0 = clock64();
            if ((it & 63u) != 63u || clock64() - t0 < 4000000000LL) continue;
            atomicExch(status, 2);
        }
#pragma unroll
        for (int i = 0; i < 4; i++) {
            a[2 * i] = __uint_as_float(q[i].x);
            a[2 * i + 1] = __uint_as_float(q[i].z);
        }
        return;
    }
}

// Stage NB activation vectors: optional RMSNorm, power-of-two normalisation, hi/lo split,
// fragment order, per-32-column sums.  Each thread owns groups of 8 consecutive columns; the first
// kCache groups (16 K columns per CTA) stay in registers between the reduction pass and the
// conversion pass, so x is fetched from L2 only once; longer vectors re-read the remainder.
constexpr int kCache = 4;

template <bool TP>
__device__ __forceinline__ void stage_activations(const SmemLayout &sm, const float *__restrict__ x, uint32_t x_stride,
                                                  uint32_t n_cols, uint32_t nb, const float *__restrict__ norm_w,
                                                  float eps, const uint2 *pairs = nullptr, uint32_t pair_epoch = 0,
                                                  int *status = nullptr) {
    const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5;
    constexpr int NW = kThreadsCta / 32;
    if (threadIdx.x < 64) sm.zb[threadIdx.x] = make_uint4(0u, 0u, 0u, 0u);
    for (uint32_t v = 0; v < nb; v++) {
        const float *xv = x + (size_t)v * x_stride;
        float cache[kCache][8];
        float ss = 0.f, mx = 0.f;
        auto load8 = [&](uint32_t c, float (&a)[8]) {
            if (TP && pairs) {  // tensor parallelism: the vector arrives as (value, epoch) pairs stored by all ranks
                tp_load8(pairs + c, pair_epoch, status, a);
                return;
            }
            *reinterpret_cast<float4 *>(a) = *reinterpret_cast<const float4 *>(xv + c);
            *reinterpret_cast<float4 *>(a + 4) = *reinterpret_cast<const float4 *>(xv + c + 4);
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
        for (int k = 0; k < kCache; k++) {
            const uint32_t c = (threadIdx.x + k * kThreadsCta) * 8;
            if (c < n_cols) {
                load8(c, cache[k]);
                reduce8(c, cache[k]);
            }
        }
        for (uint32_t c = (threadIdx.x + kCache * kThreadsCta) * 8; c < n_cols; c += kThreadsCta * 8) {
            float a[8];
            load8(c, a);
            reduce8(c, a);
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            ss += __shfl_xor_sync(0xffffffffu, ss, o);
            mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
        }
        __syncthreads();  // previous vector's readers of `red` are done
        if (lane == 0) {
            sm.red[wid] = ss;
            sm.red[32 + wid] = mx;
        }
        __syncthreads();
        ss = 0.f;
        mx = 0.f;
#pragma unroll
        for (int i = 0; i < NW; i++) {
            ss += sm.red[i];
            mx = fmaxf(mx, sm.red[32 + i]);
        }
        // RMSNorm scale exactly as the CPU runner forms it: 1 / sqrt(ss / n + eps)
        const float inv_rms = norm_w ? 1.0f / sqrtf(ss / (float)n_cols + eps) : 1.0f;
        mx *= inv_rms;
        // 2^e with max|x|·2^e in [2^13, 2^14); exponent clamped so both 2^e and 2^-e stay finite normals
        int eb = (int)((__float_as_uint(mx) >> 23) & 0xFFu);
        if (mx == 0.f || eb == 0xFF) eb = 127 + 13;
        int se = 127 + 13 - (eb - 127);
        se = se < 1 ? 1 : (se > 253 ? 253 : se);
        const float scale = __uint_as_float((uint32_t)se << 23);
        const float inv_scale = __uint_as_float((uint32_t)(254 - se) << 23);
        if (threadIdx.x == 0) sm.inv_scale[v] = inv_scale;
        uint4 *xb = sm.xb + (size_t)v * (n_cols / 4);
        __half *sbh = reinterpret_cast<__half *>(sm.sb + (size_t)v * (n_cols / 32));
        float *sf = sm.sf + (size_t)v * (n_cols / 32);
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
            const uint32_t blk = c >> 8, t = (c >> 6) & 3, h = (c >> 5) & 1, wp = (c >> 3) & 3;
            const uint32_t idx = ((blk * 2 + h) * 4 + wp) * 8 + t;
            xb[idx] = make_uint4(h2_as_u32(__halves2half2(hi[0], hi[2])), h2_as_u32(__halves2half2(hi[1], hi[3])),
                                 h2_as_u32(__halves2half2(hi[4], hi[6])), h2_as_u32(__halves2half2(hi[5], hi[7])));
            xb[idx + 4] = make_uint4(h2_as_u32(__halves2half2(lo[0], lo[2])), h2_as_u32(__halves2half2(lo[1], lo[3])),
                                     h2_as_u32(__halves2half2(lo[4], lo[6])), h2_as_u32(__halves2half2(lo[5], lo[7])));
            // Σ over 32 columns: 4 consecutive threads hold one sub-block
            s8 += __shfl_xor_sync(0xffffffffu, s8, 1);
            s8 += __shfl_xor_sync(0xffffffffu, s8, 2);
            if ((lane & 3) == 0) {
                sf[c >> 5] = s8;
                // 32 values below 2^14 can sum to 2^19: keep Σ·2^-6 (exact) so fp16 cannot overflow;
                // unpack_scales folds the 2^6 back into dmin
                s8 *= 0.015625f;
                const __half sh = __float2half_rn(s8);
                const uint32_t sub = (c >> 5) & 7;  // sub-block within the super-block
                const uint32_t hidx = ((blk * 2 + 0) * 4 + (sub >> 1)) * 2 + (sub & 1);
                sbh[hidx] = sh;
                sbh[hidx + 8] = __float2half_rn(s8 - __half2float(sh));  // part 1 sits 4 half2 further on
            }
        };
        // n_cols is a multiple of 256, so whole warps are in or out of every step (the shuffles are safe)
#pragma unroll
        for (int k = 0; k < kCache; k++) {
            const uint32_t c = (threadIdx.x + k * kThreadsCta) * 8;
            if (c < n_cols) convert8(c, cache[k]);
        }
        for (uint32_t c = (threadIdx.x + kCache * kThreadsCta) * 8; c < n_cols; c += kThreadsCta * 8) {
            float a[8];
            load8(c, a);
            convert8(c, a);
        }
    }
    __syncthreads();
}

// Multiply one super-block (this lane's rows × 64-column group) into the running sums.
template <int NR, bool Q5>
__device__ __forceinline__ void consume_block(const BlockLoads (&ld)[NR], uint32_t blk, int t, const uint4 *xb_lane,
                                              const uint32_t *sb_lane, float (&acc)[NR][2]) {
    RowScales rs[NR];
#pragma unroll
    for (int r = 0; r < NR; r++) rs[r] = unpack_scales(ld[r].hdr, t);

    // two independent accumulator chains (low-nibble and high-nibble MMAs)
    float dl[4] = {0.f, 0.f, 0.f, 0.f}, dh[4] = {0.f, 0.f, 0.f, 0.f}, dm[4] = {0.f, 0.f, 0.f, 0.f};
    const uint4 *bp = xb_lane + (size_t)blk * 64;  // 2 halves × 4 word pairs × 8 lanes-groups
#pragma unroll
    for (int wp = 0; wp < 4; wp++) {
        const uint4 bl = bp[wp * 8], bh = bp[32 + wp * 8];
#pragma unroll
        for (int e = 0; e < 2; e++) {
            const int wi = 2 * wp + e;
            uint32_t lo02[2], lo13[2], hi02[2], hi13[2];
#pragma unroll
            for (int r = 0; r < NR; r++) {
                const uint32_t w = word_of(ld[r], wi);
                word_to_frags(w, rs[r], fifth_of<Q5>(ld[r], wi, t), lo02[r], lo13[r], hi02[r], hi13[r]);
            }
            if (NR == 1) lo02[1] = lo13[1] = hi02[1] = hi13[1] = 0u;
            mma_16816(dl, lo02[0], lo02[1], lo13[0], lo13[1], e ? bl.z : bl.x, e ? bl.w : bl.y);
            mma_16816(dh, hi02[0], hi02[1], hi13[0], hi13[1], e ? bh.z : bh.x, e ? bh.w : bh.y);
        }
    }
    // mins: k slots 2t, 2t+1 carry sub-blocks 2t, 2t+1; the other slots are zero
    const uint32_t sx = sb_lane[(size_t)blk * 8];
    mma_16816(dm, rs[0].mn, NR == 2 ? rs[NR - 1].mn : 0u, 0u, 0u, sx, 0u);
    acc[0][0] = fmaf(rs[0].d, dl[0] + dh[0], acc[0][0]);
    acc[0][0] = fmaf(-rs[0].dmin, dm[0], acc[0][0]);
    acc[0][1] = fmaf(rs[0].d, dl[1] + dh[1], acc[0][1]);
    acc[0][1] = fmaf(-rs[0].dmin, dm[1], acc[0][1]);
    if (NR == 2) {
        acc[NR - 1][0] = fmaf(rs[NR - 1].d, dl[2] + dh[2], acc[NR - 1][0]);
        acc[NR - 1][0] = fmaf(-rs[NR - 1].dmin, dm[2], acc[NR - 1][0]);
        acc[NR - 1][1] = fmaf(rs[NR - 1].d, dl[3] + dh[3], acc[NR - 1][1]);
        acc[NR - 1][1] = fmaf(-rs[NR - 1].dmin, dm[3], acc[NR - 1][1]);
    }
}

// ── batch-1 path: sub-blocks in the N dimension ─────────────────────────────────────────────
// B column n = 4·part + t' carries x (part 0 = hi, 1 = lo) only at the k slots that lane t' feeds,
// zeros elsewhere.  Those slots belong to one sub-block (2t' for the low-nibble MMA, 2t'+1 for the
// high-nibble one), so D[row][n] is that sub-block's Σ q·x whatever the k order — and the weights
// go in unscaled: the nibble's bits are used as an fp16 subnormal (q·2^-24, or 16q·2^-24 for a
// high nibble), one AND per pair of weights.  Lane (g, t) ends up with columns 2t, 2t+1 =
// groups 2u, 2u+1 (u = t&1) of part t>>1, i.e. sub-blocks 4u..4u+3, and applies their scales.
struct RowScalesF {
    float sc[4];  // sc[4u + i] · d · 2^24 (i even: low-nibble MMAs) or · d · 2^20 (i odd)
    float mn[4];  // mn[4u + i] · dmin, zero in the lanes of the lo part (mins are charged once)
};

template <bool Q5>
__device__ __forceinline__ RowScalesF unpack_scales_f(const uint4 &hdr, int u, bool charge_mins) {
    uint32_t sc4, mn4;  // four 6-bit values each, one per byte (dequant.rs:176-190)
    if (u == 0) {
        sc4 = hdr.y & 0x3F3F3F3Fu;
        mn4 = hdr.z & 0x3F3F3F3Fu;
    } else {
        sc4 = (hdr.w & 0x0F0F0F0Fu) | ((hdr.y >> 2) & 0x30303030u);
        mn4 = ((hdr.w >> 4) & 0x0F0F0F0Fu) | ((hdr.z >> 2) & 0x30303030u);
    }
    const float d = __half2float(__ushort_as_half((unsigned short)(hdr.x & 0xFFFFu)));
    const float dmin = charge_mins ? __half2float(__ushort_as_half((unsigned short)(hdr.x >> 16))) : 0.f;
    // Q5_K operands carry q·2^-24 in both halves; Q4_K's high nibbles stay in place (16q·2^-24)
    const float d24 = d * 16777216.0f, d20 = Q5 ? d24 : d * 1048576.0f;
    const float k23 = 8388608.0f;
    RowScalesF r;
    r.sc[0] = (__uint_as_float(__byte_perm(sc4, 0x4B000000u, 0x7440)) - k23) * d24;
    r.sc[1] = (__uint_as_float(__byte_perm(sc4, 0x4B000000u, 0x7441)) - k23) * d20;
    r.sc[2] = (__uint_as_float(__byte_perm(sc4, 0x4B000000u, 0x7442)) - k23) * d24;
    r.sc[3] = (__uint_as_float(__byte_perm(sc4, 0x4B000000u, 0x7443)) - k23) * d20;
    r.mn[0] = (__uint_as_float(__byte_perm(mn4, 0x4B000000u, 0x7440)) - k23) * dmin;
    r.mn[1] = (__uint_as_float(__byte_perm(mn4, 0x4B000000u, 0x7441)) - k23) * dmin;
    r.mn[2] = (__uint_as_float(__byte_perm(mn4, 0x4B000000u, 0x7442)) - k23) * dmin;
    r.mn[3] = (__uint_as_float(__byte_perm(mn4, 0x4B000000u, 0x7443)) - k23) * dmin;
    return r;
}

template <int NR, bool Q5>
__device__ __forceinline__ void consume_block_subcol(const BlockLoads (&ld)[NR], const uint4 *bp, const float *sfp, int u,
                                                     int t, bool charge_mins, float (&acc)[NR][2]) {
    float dl[4] = {0.f, 0.f, 0.f, 0.f}, dh[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
    for (int wp = 0; wp < 4; wp++) {
        const uint4 bl = bp[wp * 8], bh = bp[32 + wp * 8];
#pragma unroll
        for (int e = 0; e < 2; e++) {
            const int wi = 2 * wp + e;
            uint32_t lo02[2], lo13[2], hi02[2], hi13[2];
#pragma unroll
            for (int r = 0; r < NR; r++) {
                const uint32_t w = word_of(ld[r], wi), w8 = w >> 8;
                if (Q5) {
                    // four 5-bit values per register first (nibble | fifth bit << 4), then one byte
                    // permute per operand: both halves of the word are q·2^-24 (no factor 16 on the
                    // high nibbles, see unpack_scales_f)
                    const uint32_t f = fifth_word<Q5>(ld[r], wi) >> (2 * t);
                    const uint32_t cl = (w & 0x0F0F0F0Fu) | ((f << 4) & 0x10101010u);
                    const uint32_t ch = ((w >> 4) & 0x0F0F0F0Fu) | ((f << 3) & 0x10101010u);
                    lo02[r] = __byte_perm(cl, 0u, 0x4240);
                    lo13[r] = __byte_perm(cl, 0u, 0x4341);
                    hi02[r] = __byte_perm(ch, 0u, 0x4240);
                    hi13[r] = __byte_perm(ch, 0u, 0x4341);
                } else {
                    lo02[r] = w & 0x000F000Fu;
                    lo13[r] = w8 & 0x000F000Fu;
                    hi02[r] = w & 0x00F000F0u;
                    hi13[r] = w8 & 0x00F000F0u;
                }
            }
            if (NR == 1) lo02[1] = lo13[1] = hi02[1] = hi13[1] = 0u;
            mma_16816(dl, lo02[0], lo02[1], lo13[0], lo13[1], e ? bl.z : bl.x, e ? bl.w : bl.y);
            mma_16816(dh, hi02[0], hi02[1], hi13[0], hi13[1], e ? bh.z : bh.x, e ? bh.w : bh.y);
        }
    }
    const float4 sx = *reinterpret_cast<const float4 *>(sfp);  // Σx of sub-blocks 4u..4u+3
#pragma unroll
    for (int r = 0; r < NR; r++) {
        const RowScalesF rs = unpack_scales_f<Q5>(ld[r].hdr, u, charge_mins);
        float a = acc[r][0];
        a = fmaf(rs.sc[0], dl[2 * r + 0], a);
        a = fmaf(rs.sc[1], dh[2 * r + 0], a);
        a = fmaf(rs.sc[2], dl[2 * r + 1], a);
        a = fmaf(rs.sc[3], dh[2 * r + 1], a);
        float m = rs.mn[0] * sx.x;
        m = fmaf(rs.mn[1], sx.y, m);
        m = fmaf(rs.mn[2], sx.z, m);
        m = fmaf(rs.mn[3], sx.w, m);
        acc[r][0] = a - m;
    }
}

struct Q4kMmaParams {
    const uint8_t *w[3];    // segment weight tensors (raw Q4_K blocks)
    float *out[3];          // segment outputs, [batch][out_stride[s]]
    uint32_t seg_tiles[3];  // row tiles per segment
    uint32_t seg_rows[3];
    uint32_t out_stride[3];
    uint32_t n_seg;
    uint32_t n_tiles;       // tiles over all segments (pair mode: tiles of one matrix)
    uint32_t pair;          // 1: w[0], w[1] are gate and up over the same rows → out[0] = SiLU(gate)·up
    const float *x;         // [batch][x_stride]
    uint32_t x_stride, n_cols, batch;
    const float *norm_w;    // RMSNorm weights for the prologue, or null
    float eps;
    const float *residual;  // added to segment 0's output, or null (same layout as out[0])
    const void *next_w[2];  // weights of the following kernel(s), prefetched into L2
    uint64_t next_bytes[2];
    TpFuse tp;              // tensor parallelism: push out[0] to the peers / wait for the gathered x
};

__device__ __forceinline__ void group_barrier(int group) {
    asm volatile("bar.sync %0, %1;" ::"r"(1 + group), "r"(kWarps * 32) : "memory");
}

// Walks one warp's units in order: tile index k (of its group), matrix q (pair mode), super-block
// slot j; the row pointers are recomputed only when the tile or matrix changes.
template <int ROWS, bool Q5>
struct UnitCursor {
    static constexpr int NR = ROWS / 8;
    uint32_t k, q, j;
    const uint4 *rowp[NR];

    __device__ __forceinline__ void locate(const Q4kMmaParams &p, uint32_t first_tile, uint32_t tile_stride, uint32_t bpr,
                                           int g) {
        uint32_t tile = first_tile + k * tile_stride, seg = 0;
        if (p.pair) {
            seg = q;
        } else {
            while (seg + 1 < p.n_seg && tile >= p.seg_tiles[seg]) {
                tile -= p.seg_tiles[seg];
                seg++;
            }
        }
        const uint32_t n_rows = p.seg_rows[seg];
#pragma unroll
        for (int r = 0; r < NR; r++) {
            uint32_t row = tile * ROWS + g + 8 * r;
            row = row < n_rows ? row : n_rows - 1;  // clamp: the load stays in bounds, the result is dropped
            rowp[r] = reinterpret_cast<const uint4 *>(p.w[seg] + (size_t)row * bpr * (Q5 ? 176 : 144));
        }
    }
    __device__ __forceinline__ void advance(const Q4kMmaParams &p, uint32_t first_tile, uint32_t tile_stride, uint32_t bpr,
                                            int g, uint32_t nbw, uint32_t nq) {
        if (++j == nbw) {
            j = 0;
            if (++q == nq) {
                q = 0;
                k++;
            }
            locate(p, first_tile, tile_stride, bpr, g);
        }
    }
};

// Persistent kernel, one CTA per SM: CTA c owns tiles c, c+G, c+2G, … (G = gridDim.x), dealt
// alternately to its two 8-warp groups, so every SM gets the same number of tiles (±1) and at any
// moment the grid streams one contiguous region of the tensor.  Within a tile, warp w of the
// group multiplies super-blocks w, w+8, …; a warp's (tile, matrix, super-block) units form one
// sequence that is prefetched DEPTH units ahead.  In pair mode a tile is the gate rows followed by
// the same rows of up.  The activations are staged once per CTA.
// TP = true only for launches of a tensor-parallel runner that push or poll (value, epoch) pairs: the
// single-GPU instantiations carry none of that code.
template <int ROWS, int DEPTH, bool SUBCOL, bool TP, bool Q5>
__global__ void __launch_bounds__(kThreadsCta, 1)
qmv_q4k_mma_kernel(const __grid_constant__ Q4kMmaParams p) {
    constexpr int NR = ROWS / 8;
    extern __shared__ __align__(16) unsigned char smem_raw[];
    yule_pdl_launch_dependents();

    const int lane = threadIdx.x & 31;
    const int group = threadIdx.x >> 8, wid = (threadIdx.x >> 5) & (kWarps - 1);
    const int g = lane >> 2, t = lane & 3;
    const uint32_t bpr = p.n_cols / 256;
    const uint32_t nbw = bpr > (uint32_t)wid ? (bpr - wid + kWarps - 1) / kWarps : 0;  // super-blocks per tile for this warp
    const uint32_t nq = p.pair ? 2 : 1;
    const uint32_t G = gridDim.x;
    // tiles of this CTA: blockIdx.x + i*G; group takes i = group, group + 2, …
    const uint32_t first_tile = blockIdx.x + group * G, tile_stride = kGroups * G;
    const uint32_t my_tiles = p.n_tiles > first_tile ? (p.n_tiles - first_tile + tile_stride - 1) / tile_stride : 0;
    const uint32_t tiles_per_round = kRoundSlots / nq;

    const SmemLayout sm = carve(smem_raw, p.n_cols, p.batch);
    float *partial = sm.partial + (size_t)group * kRoundSlots * kWarps * 4 * 16;

    UnitCursor<ROWS, Q5> ld_cur;
    ld_cur.k = ld_cur.q = ld_cur.j = 0;
    const uint32_t total_units = my_tiles * nq * nbw;
    uint32_t issued = 0;
    BlockLoads buf[DEPTH][NR];
    if (total_units) {
        ld_cur.locate(p, first_tile, tile_stride, bpr, g);
#pragma unroll
        for (int i = 0; i < DEPTH; i++) {
            if (issued < total_units) {
                issue_loads<NR, Q5>(buf[i], ld_cur.rowp, wid + kWarps * ld_cur.j, t);
                issued++;
                if (issued < total_units) ld_cur.advance(p, first_tile, tile_stride, bpr, g, nbw, nq);
            }
        }
    }

    // Own weight loads are in flight; start HBM on the next kernel's weights too, then wait for
    // the kernel that produced the activations.
    yule_prefetch_l2_slice(p.next_w[0], p.next_bytes[0]);
    yule_prefetch_l2_slice(p.next_w[1], p.next_bytes[1]);
    yule_pdl_wait();
    // tensor parallelism: x may arrive as (value, epoch) pairs stored by all ranks
    if (TP)
        stage_activations<true>(sm, p.x, p.x_stride, p.n_cols, p.batch, p.norm_w, p.eps, p.tp.wait ? p.tp.pair_in : nullptr,
                                p.tp.wait ? *p.tp.tick * p.tp.epochs_per_tick + p.tp.wait_index + 1u : 0u, p.tp.status);
    else
        stage_activations<false>(sm, p.x, p.x_stride, p.n_cols, p.batch, p.norm_w, p.eps);
    // B column n = g: vector n/2, part n%2.  Lanes whose vector does not exist read vector 0;
    // their output columns are never looked at.
    const uint32_t vec = (uint32_t)(g >> 1) < p.batch ? (g >> 1) : 0;
    const uint4 *xb_lane = sm.xb + (size_t)vec * (p.n_cols / 4) + (g & 1) * 4 + t;
    const uint32_t *sb_lane = sm.sb + (size_t)vec * (p.n_cols / 32) + (g & 1) * 4 + t;
    // batch-1 path: lane (g, t) feeds column g; that column is live only for g = t (hi part) and
    // g = t + 4 (lo part), every other lane reads zeros
    const bool feeds = (g & 3) == t;
    const uint4 *sub_base = feeds ? sm.xb + (g >> 2) * 4 + t : sm.zb;
    const uint32_t sub_stride = feeds ? 64u : 0u;
    const int u = t & 1;
    const bool charge_mins = t < 2;

    // Cross-warp sums of the tiles [k0, k0+kn) of this group, then the epilogue.  Every warp of
    // the group calls this once per round.
    auto finish_round = [&](uint32_t k0, uint32_t kn) {
        group_barrier(group);
        const uint32_t n_warps_used = bpr < (uint32_t)kWarps ? bpr : kWarps;
        const uint32_t tid = threadIdx.x & (kWarps * 32 - 1);
        for (uint32_t idx = tid; idx < kn * 64; idx += kWarps * 32) {
            const uint32_t kk = idx >> 6, v = (idx >> 4) & 3, rr = idx & 15;
            if (v >= p.batch || rr >= ROWS) continue;
            uint32_t tile = first_tile + (k0 + kk) * tile_stride, seg = 0;
            if (!p.pair) {
                while (seg + 1 < p.n_seg && tile >= p.seg_tiles[seg]) {
                    tile -= p.seg_tiles[seg];
                    seg++;
                }
            }
            const uint32_t row = tile * ROWS + rr;
            if (row >= p.seg_rows[seg]) continue;
            const float inv_scale = sm.inv_scale[v];
            float sums[2] = {0.f, 0.f};
            for (uint32_t q = 0; q < nq; q++) {
                const uint32_t sl = kk * nq + q;
                float sacc = 0.f;  // fixed order over the warps: deterministic
                if (SUBCOL) {
                    // the four t lanes hold (hi, lo) × (sub-blocks 0..3, 4..7): one vector, four addends
                    for (uint32_t w2 = 0; w2 < n_warps_used; w2++)
#pragma unroll
                        for (int tt = 0; tt < 4; tt++) sacc += partial[((sl * kWarps + w2) * 4 + tt) * 16 + rr];
                } else {
                    for (uint32_t w2 = 0; w2 < n_warps_used; w2++) sacc += partial[((sl * kWarps + w2) * 4 + v) * 16 + rr];
                }
                sums[q] = sacc * inv_scale;
            }
            const size_t o = (size_t)v * p.out_stride[seg] + row;
            if (p.pair) {
                // silu_mul.cu: x / (1 + exp(−x)) * up
                sums[0] = (sums[0] / (1.0f + expf(-sums[0]))) * sums[1];
            } else if (seg == 0 && p.residual) {
                sums[0] += p.residual[o];
            }
            p.out[seg][o] = sums[0];
            if (TP && p.tp.push && seg == 0) tp_push_value(p.tp, o, sums[0]);  // the same row into every peer's copy
        }
        group_barrier(group);
    };

    if (nbw == 0) {
        // more warps than super-blocks per row: this warp only helps with the reductions
        for (uint32_t k0 = 0; k0 < my_tiles; k0 += tiles_per_round)
            finish_round(k0, (my_tiles - k0) < tiles_per_round ? (my_tiles - k0) : tiles_per_round);
    } else {

    float acc[NR][2];
#pragma unroll
    for (int r = 0; r < NR; r++) acc[r][0] = acc[r][1] = 0.f;
    uint32_t k0 = 0, kn = my_tiles < tiles_per_round ? my_tiles : tiles_per_round;
    uint32_t in_slot = 0, slot = 0;  // super-blocks done in the current (tile, matrix); slots done in the round
    // unit n lives in buf[n % DEPTH]; the loop is unrolled by DEPTH so the ring index is static
    for (uint32_t base = 0; base < total_units; base += DEPTH) {
#pragma unroll
        for (int i = 0; i < DEPTH; i++) {
            if (base + i < total_units) {
                if (SUBCOL) {
                    const uint32_t blk = wid + kWarps * in_slot;
                    consume_block_subcol<NR, Q5>(buf[i], sub_base + (size_t)blk * sub_stride, sm.sf + (size_t)blk * 8 + 4 * u,
                                                 u, t, charge_mins, acc);
                } else {
                    consume_block<NR, Q5>(buf[i], wid + kWarps * in_slot, t, xb_lane, sb_lane, acc);
                }
                if (issued < total_units) {
                    issue_loads<NR, Q5>(buf[i], ld_cur.rowp, wid + kWarps * ld_cur.j, t);
                    issued++;
                    if (issued < total_units) ld_cur.advance(p, first_tile, tile_stride, bpr, g, nbw, nq);
                }
                if (++in_slot == nbw) {
                    // lane (g, t) holds, for vector t, rows g (and g+8): hi-column + lo-column sums
#pragma unroll
                    for (int r = 0; r < NR; r++) {
                        partial[((slot * kWarps + wid) * 4 + t) * 16 + g + 8 * r] = acc[r][0] + acc[r][1];
                        acc[r][0] = acc[r][1] = 0.f;
                    }
                    in_slot = 0;
                    if (++slot == kn * nq) {
                        finish_round(k0, kn);
                        k0 += kn;
                        kn = (my_tiles - k0) < tiles_per_round ? (my_tiles - k0) : tiles_per_round;
                        slot = 0;
                    }
                }
            }
        }
    }
    }  // nbw != 0

}

template <int ROWS, int DEPTH, bool SUBCOL, bool Q5 = false, bool TP = false>
cudaError_t launch_variant(const Q4kMmaParams &p, int sm_count, size_t smem, bool pdl, cudaStream_t s) {
    if (!TP && !Q5 && (p.tp.push || p.tp.wait))
        return launch_variant<ROWS, DEPTH, SUBCOL, false, true>(p, sm_count, smem, pdl, s);
    auto kern = qmv_q4k_mma_kernel<ROWS, DEPTH, SUBCOL, TP, Q5>;
    // per instantiation: the opt-in for large dynamic shared memory
    static bool attr_done = false;
    static std::mutex mu;
    {
        std::lock_guard<std::mutex> lock(mu);
        if (!attr_done) {
            cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
            if (e != cudaSuccess) return e;
            attr_done = true;
        }
    }
    // one CTA per SM; fewer when there are not enough tiles to give every group one
    uint32_t grid = (uint32_t)sm_count;
    const uint32_t want = (p.n_tiles + kGroups - 1) / kGroups;
    if (grid > want) grid = want;
    return launch_kernel(kern, dim3(grid), dim3(kThreadsCta), smem, s, pdl, p);
}

}  // namespace

bool q4k_mma_supported(uint32_t n_cols, uint32_t batch) {
    return n_cols % 256 == 0 && batch >= 1 && batch <= 4 && smem_bytes(n_cols, batch) <= 200 * 1024;
}

cudaError_t launch_q4k_mma(const Q4kFused &f, int sm_count, cudaStream_t s, uint64_t *launches) {
    Q4kMmaParams p = {};
    const bool pair = f.swiglu_pair;
    uint32_t total_rows = 0;
    for (uint32_t i = 0; i < f.n_seg; i++) total_rows += f.rows[i];
    // 16-row tiles use the whole MMA; 8-row tiles (half of each MMA idle) only when 16-row tiles
    // would leave warp groups without work.
    const uint32_t rows_for_grid = pair ? 2 * f.rows[0] : total_rows;
    // Tile height.  16-row tiles use the whole MMA and half the instructions per byte of 8-row tiles; they win
    // as soon as they keep about 60 % of the warp groups busy (measured: 4096 rows, 256 tiles for 296 groups,
    // 10-25 % faster with 16; 2048 rows, 128 tiles, faster with 8).  YULE_QMV_ROWS forces one (timing aid).
    const uint32_t n_groups = (uint32_t)kGroups * (uint32_t)sm_count;
    int tile_rows = ((rows_for_grid / 16) * 10 >= n_groups * 6) ? 16 : 8;
    if (const char *force = getenv("YULE_QMV_ROWS")) tile_rows = atoi(force) == 8 ? 8 : (atoi(force) == 16 ? 16 : tile_rows);
    uint32_t n_tiles = 0;
    for (uint32_t i = 0; i < f.n_seg; i++) {
        p.w[i] = f.w[i];
        p.out[i] = f.out[i];
        p.seg_rows[i] = f.rows[i];
        p.seg_tiles[i] = (f.rows[i] + tile_rows - 1) / tile_rows;
        p.out_stride[i] = f.out_stride[i];
        if (!pair || i == 0) n_tiles += p.seg_tiles[i];
    }
    p.n_seg = f.n_seg;
    p.n_tiles = n_tiles;
    p.pair = pair ? 1 : 0;
    p.x = f.x;
    p.x_stride = f.x_stride;
    p.n_cols = f.n_cols;
    p.batch = f.batch;
    p.norm_w = f.norm_w;
    p.eps = f.eps;
    p.residual = f.residual;
    p.tp = f.tp;
    for (int i = 0; i < 2; i++) {
        p.next_w[i] = f.next_w[i];
        p.next_bytes[i] = f.next_bytes[i];
    }
    if (n_tiles == 0) return cudaSuccess;
    const size_t smem = smem_bytes(f.n_cols, f.batch);
    cudaError_t e;
    if (f.q5 && (f.tp.push || f.tp.wait)) return cudaErrorInvalidValue;  // the exchange is built for Q4_K only
    if (f.q5 && f.batch == 1)
        e = tile_rows == 8 ? launch_variant<8, 4, true, true>(p, sm_count, smem, f.pdl, s)
                           : launch_variant<16, 2, true, true>(p, sm_count, smem, f.pdl, s);
    else if (f.q5)
        e = tile_rows == 8 ? launch_variant<8, 4, false, true>(p, sm_count, smem, f.pdl, s)
                           : launch_variant<16, 2, false, true>(p, sm_count, smem, f.pdl, s);
    else if (f.batch == 1)
        e = tile_rows == 8 ? launch_variant<8, 4, true>(p, sm_count, smem, f.pdl, s)
                           : launch_variant<16, 2, true>(p, sm_count, smem, f.pdl, s);
    else
        e = tile_rows == 8 ? launch_variant<8, 4, false>(p, sm_count, smem, f.pdl, s)
                           : launch_variant<16, 2, false>(p, sm_count, smem, f.pdl, s);
    if (e != cudaSuccess) return e;
    *launches += 1;
    return cudaSuccess;
}

}  // namespace yule
