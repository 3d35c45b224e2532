// Quantised GEMM on the 5th-generation tensor cores (tcgen05, accumulators in TMEM):
//
//     out[n][r] = Σ_k W[r][k] · x[n][k]        W: Q4_K blocks, x: N ≥ 8 fp32 activation rows
//
// This is the prefill / batched-decode counterpart of the matvec kernels: the weights cross HBM
// once per pass over up to 128 activation rows instead of once per four.  The reference runs
// prefill as one matvec chain per token (yule-infer/src/gpu_runner.rs:146-160); the arithmetic
// contract is the same fp32 dot product.
//
// Operands.  A Q4_K weight is d·sc·q − dmin·m with a 4-bit q, 6-bit sc and m per 32 columns and
// fp16 d, dmin per 256.  The tensor core multiplies the exact integers: the W operand of a stage is
// sc·q (≤ 945, exact in fp16), the 64-column partial sums are drained from TMEM after every stage
// and multiplied by that row's d in fp32 on the way into register accumulators.  The min term is one
// more MMA per super-block, (m of the 8 sub-blocks) × (per-sub-block sums of x), drained with −dmin.
// Activations are fp32, which tcgen05 cannot take: each row is scaled by a power of two that puts
// its largest element in [2¹³, 2¹⁴) and split into fp16 hi + lo (22 significant bits); two MMAs per
// 16 columns, W·x_hi and W·x_lo (up to 64 activation rows one MMA against both terms side by side as
// one operand of twice the rows).  The tensor core adds into its fp32 accumulator with truncation, a
// bias that grows with the chain length; draining after every stage keeps a chain at 8 MMAs and
// leaves the long sum to ordinary round-to-nearest fp32.  The result matches the fp32 matvec to
// fp32 rounding.
//
// Work items: (row tile, activation tile) pairs; when these are few (small matrices, tensor-parallel
// shards, few activation rows) the super-blocks of a row are split into up to 16 parts, one item each,
// whose scaled partial sums the last drain warp of a (tile, warp) to finish adds up in the order of
// the parts.
//
// One CTA per SM, 20 warps, persistent over the work items:
//   warps 0-7   drain warps: tcgen05.ld of their 32 TMEM lanes × half of the columns after every
//               stage, FMA by d (and −dmin) into registers; at the end of a tile scale, residual, store
//   warp  8     one thread: bulk copies (TMA engine) of the pre-arranged activation tiles
//   warps 9, 11 one thread each: tcgen05.mma issue, even stages from one, odd stages from the other
//               (a single thread issues about one MMA per 63 cycles, less than the tensor core
//               takes); warp 9 also owns the TMEM allocation
//   warp  10    one thread: tiled TMA loads (cp.async.bulk.tensor.2d) of the raw Q4_K bytes, one
//               128-row × 144-byte box per super-block, four boxes in flight (two at 128 activation
//               rows, where the room goes to a third operand stage; three at 32); rows past the end of
//               the matrix arrive as zeros
//   warps 12-19 unpack Q4_K from that shared-memory copy → fp16 sc·q in the operand layout (about
//               1.4 instructions per weight)
// A stage is a 128-row × 64-column slab of W (16 KB) plus the matching hi and lo slabs of x; the last
// stage of a super-block also carries the 4 KB m slab and the sub-block sums of x.  At 32 activation rows
// a stage is two such column groups (a chain of eight MMAs, as at 128 rows, and half the hand-offs per
// column), and three raw boxes are in flight.
// One launch can run over up to three matrices that read the same activations (Q/K/V; gate/up): their row
// tiles are numbered one after the other.
// Operands use the no-swizzle K-major core-matrix layout: 8 rows × 16 bytes per core matrix,
// core matrices of one 8-column step contiguous along the rows.  Inside a core-matrix row the eight
// columns sit in the order 0,2,1,3,4,6,5,7 (the order in which nibble pairs fall out of a 32-bit
// word); both operands use it, so the products pair up correctly.
//
// Every wait is bounded: a pipeline that stops making progress sets the context's status word,
// raises the CTA's abort flag, lets all roles fall through to the common exit and frees its TMEM.

#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <functional>
#include <type_traits>
#include <unordered_map>

#include <cuda.h>
#include <cuda_fp16.h>

#include "dequant_device.cuh"
#include "internal.h"

namespace yule {
namespace {

constexpr int kBM = 128;  // rows of W per tile = TMEM lanes
constexpr int kBK = 64;   // columns per stage (a quarter of a super-block)
constexpr int kEpiWarps = 8, kProdWarps = 8;
constexpr int kLoaderWarp = kEpiWarps, kMmaWarp = kEpiWarps + 1, kRawWarp = kEpiWarps + 2, kMmaWarp2 = kEpiWarps + 3,
              kFirstProdWarp = kEpiWarps + 4;
constexpr int kGemmThreads = (kEpiWarps + 4 + kProdWarps) * 32;  // 640
constexpr int kMaxStages = 6;
#ifndef YULE_GEMM_RAW_SLOTS
#define YULE_GEMM_RAW_SLOTS 4
#endif
constexpr int kRawSlots = YULE_GEMM_RAW_SLOTS;                       // super-blocks of raw Q4_K bytes in flight per CTA (at most)
// At 128 activation rows a stage is 56 KB: two raw slots instead of four make room for a third stage, which together
// with the third accumulator set lets the unpacking, MMA-issuing and drain roles overlap.
// At 32 rows a stage is two column groups wide (53 KB): three raw slots leave room for three of them.
#ifndef YULE_GEMM_WIDE_32
#define YULE_GEMM_WIDE_32 1   // two column groups per stage at 32 activation rows
#endif
#ifndef YULE_GEMM_RAW_SLOTS_32
#define YULE_GEMM_RAW_SLOTS_32 (YULE_GEMM_WIDE_32 ? 3 : 4)
#endif
__host__ __device__ constexpr uint32_t raw_slots_for(uint32_t bn) {
    return bn >= 128 ? 2u : (bn <= 32 ? (uint32_t)YULE_GEMM_RAW_SLOTS_32 : (uint32_t)(kRawSlots < 4 ? kRawSlots : 4));
}
// 64-column groups of W per stage.  The exact kernel at 32 activation rows takes two: its MMAs are narrow and its
// drains short, so the waits, fences and barrier arrivals of a stage, not its work, set the pace, and a stage of
// twice the columns halves them.  A chain is then eight MMAs (one per 16 columns against hi | lo), the same length as
// at 128 rows.
__host__ __device__ constexpr uint32_t groups_per_stage(uint32_t bn, bool generic) {
    return (YULE_GEMM_WIDE_32 && !generic && bn <= 32) ? 2u : 1u;
}
constexpr uint32_t kRawBytes = kBM * 144;          // one super-block of 128 rows: 18 KB
constexpr uint32_t kABytes = kBM * kBK * 2;  // the W slab of a stage: 16 KB
constexpr float kSumScale = 1.0f / 32.0f;     // the sub-block sums of x are stored divided by 32
constexpr float kGenericWScale = 1024.f;      // generic kernel: weights are scaled by 2^10 before the fp16 hi/lo split
constexpr uint32_t kAmBytes = kBM * 16 * 2;  // the m slab of a super-block: 128 rows × 16 columns, 4 KB
constexpr long long kWaitCycles = 2000000000LL;  // ~1 s: far beyond any real stall

// Cycle counters of CTA 0's roles (YULE_GEMM_PROF=1 prints them after the launch): a timing aid, compiled in only
// with -DYULE_GEMM_PROFILE (its counters cost the drain warps registers they do not have to spare).
#ifdef YULE_GEMM_PROFILE
constexpr bool kProfile = true;
#else
constexpr bool kProfile = false;
#endif
__device__ long long g_gemm_prof[16];

constexpr int kGemmSegs = 3;  // matrices that share their activation tiles (Q/K/V; gate/up) in one launch
struct GemmMaps {
    CUtensorMap m[kGemmSegs];  // exact kernel: tiled view of each weight matrix
};
struct GemmParams {
    const uint8_t *w[kGemmSegs];  // blocks, row-major, per matrix
    const __half *xb;      // activation tiles written by gemm_xprep_kernel
    const float *oscale;   // per (padded) activation row: 1 / row scale
    float *out[kGemmSegs]; // [n_tokens][out_stride] per matrix
    const float *residual; // added to the results of matrix 0 (same layout; single-matrix launches only) or null
    uint32_t n_rows[kGemmSegs], out_stride[kGemmSegs];
    uint32_t mt0[kGemmSegs + 1];  // first row tile of each matrix in the launch's numbering; [n_seg] = n_mtiles
    uint32_t n_seg;
    uint32_t n_cols, n_tokens;
    uint32_t bn;           // activation rows per tile: 32, 64 or 128
    uint32_t n_mtiles, n_ntiles, stages;
    uint32_t ksplit, sb_per;  // split of the columns: `ksplit` work items per tile, `sb_per` super-blocks each (the last may be shorter)
    float *split_part;        // ksplit > 1: per work item a [bn][128] block of partial results
    uint32_t *split_tickets;  // ksplit > 1: per (tile, drain warp) the number of items that have stored theirs; left at zero
    uint32_t type;         // GGUF type id of the weights (generic kernel)
    uint64_t w_row_bytes;  // bytes of one row of the weight tensor
    uint32_t unit_bytes;   // generic kernel: bytes of 256 columns of one row
    uint32_t raw_stride;   // generic kernel: shared-memory row stride of the raw copy (an odd multiple of 16 bytes)
    uint32_t raw_chunks;   // generic kernel: 16-byte chunks copied per row and unit
    uint32_t raw_ring_bytes;  // generic kernel: two slots of 128 rows
    float out_scale;       // generic kernel: 1 / kGenericWScale; exact kernel: 1
    uint32_t prof;         // timing aid: record cycle counters of CTA 0
    uint32_t skip;         // timing aid (YULE_GEMM_SKIP, bits): 1 no unpacking, 2 no MMAs, 4 no draining, 8 no activation copies,
                           // 64 no weight copies, 256 the MMA threads wait for their own commits; results meaningless
    int *status;
};

__device__ __forceinline__ uint32_t smem_u32(const void *p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void mbar_arrive_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(bar), "r"(parity)
        : "memory");
    return ok != 0;
}
// Bounded wait.  False: the CTA is giving up (this thread ran out of time, or another did).
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile int *abort_flag, int *status) {
    if (mbar_try_wait(bar, parity)) return true;
    const long long t0 = clock64();
    for (uint32_t it = 1;; it++) {
        if (mbar_try_wait(bar, parity)) return true;
        if ((it & 255u) == 0u) {
            if (*abort_flag) return false;
            if (clock64() - t0 > kWaitCycles) {
                *abort_flag = 1;
                atomicExch(status, kStatusGemmTimeout);
                return false;
            }
        }
    }
}

__device__ __forceinline__ void fence_async_smem() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }

// Shared-memory operand descriptor, K-major, no swizzle: lbo = bytes between the two core
// matrices of a 16-column step, sbo = bytes between 8-row groups.  Bit 46 is the descriptor
// version of this architecture.
__device__ __forceinline__ uint64_t smem_desc(uint32_t addr, uint32_t lbo, uint32_t sbo) {
    return (uint64_t)((addr & 0x3FFFFu) >> 4) | ((uint64_t)(lbo >> 4) << 16) | ((uint64_t)(sbo >> 4) << 32) | (1ull << 46);
}

// D[tmem] (+)= A[smem] · B[smem], fp16 operands, fp32 accumulate, one CTA.
__device__ __forceinline__ void umma_f16(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
        : "memory");
}
// The same with the accumulate flag known at compile time (an immediate: no register, a predicate ptxas can fold).
template <int ACC>
__device__ __forceinline__ void umma_f16_c(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "n"(ACC)
        : "memory");
}
// The mbarrier gets one arrival when every MMA issued so far by this thread has completed.
__device__ __forceinline__ void umma_commit(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}

// The same load without the wait: the registers hold the values only after tmem_ld_wait().
__device__ __forceinline__ void tmem_ld16_issue(uint32_t taddr, uint32_t *v) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
        : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]), "=r"(v[8]),
          "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15])
        : "r"(taddr)
        : "memory");
}
__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void tmem_ld16(uint32_t taddr, uint32_t (&v)[16]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
        : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]), "=r"(v[8]),
          "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15])
        : "r"(taddr)
        : "memory");
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}

// The eight 6-bit scales and mins of a super-block from its 12 packed bytes
// (yule-core/src/dequant.rs:165-176), four per word, one byte each.
struct ScalesMins {
    uint32_t sc_lo, sc_hi, m_lo, m_hi;  // sub-blocks 0-3 and 4-7
};
__device__ __forceinline__ ScalesMins q4k_scales_mins(uint32_t s0, uint32_t s1, uint32_t s2) {
    ScalesMins r;
    r.sc_lo = s0 & 0x3F3F3F3Fu;
    r.m_lo = s1 & 0x3F3F3F3Fu;
    r.sc_hi = (s2 & 0x0F0F0F0Fu) | ((s0 >> 2) & 0x30303030u);
    r.m_hi = ((s2 >> 4) & 0x0F0F0F0Fu) | ((s1 >> 2) & 0x30303030u);
    return r;
}
// fp16 pair (1024 + a, 1024 + b) from two bytes: 0x6400 | v is the half 1024 + v for v < 1024
__device__ __forceinline__ uint32_t biased_pair(uint32_t word, uint32_t selector) { return __byte_perm(word, 0x64646464u, selector); }
__device__ __forceinline__ __half2 as_half2(uint32_t v) { return *reinterpret_cast<const __half2 *>(&v); }
__device__ __forceinline__ uint32_t as_u32(__half2 v) { return *reinterpret_cast<const uint32_t *>(&v); }

// Eight consecutive weights (columns col0 .. col0+7 of a 256-column unit, col0 a multiple of 8) from a
// 2-byte-aligned copy of the unit's blocks, with the arithmetic of the per-element routines
// (dequant_device.cuh): one header decode per call instead of one per weight.
__device__ __forceinline__ void dequant8_unit(const unsigned char *unit, uint32_t type, uint32_t col0, float (&v)[8]) {
    auto u16_at = [&](uint32_t byte_off) { return (uint32_t) * reinterpret_cast<const unsigned short *>(unit + byte_off); };
    if (type == YULE_DTYPE_Q8_0) {
        const uint32_t b = (col0 >> 5) * 34, i0 = col0 & 31u;
        const float d = f16_bits_to_f32(u16_at(b));
#pragma unroll
        for (int k = 0; k < 4; k++) {
            const uint32_t w = u16_at(b + 2 + i0 + 2 * k);
            v[2 * k] = __fmul_rn((float)(int)(signed char)(w & 0xFFu), d);
            v[2 * k + 1] = __fmul_rn((float)(int)(signed char)(w >> 8), d);
        }
    } else if (type == YULE_DTYPE_Q4_0) {
        const uint32_t b = (col0 >> 5) * 18, i0 = col0 & 31u;
        const float d = f16_bits_to_f32(u16_at(b));
#pragma unroll
        for (int k = 0; k < 2; k++) {
            const uint32_t w = u16_at(b + 2 + i0 / 2 + 2 * k);  // two bytes = four weights: low nibble first
#pragma unroll
            for (int q = 0; q < 4; q++) v[4 * k + q] = __fmul_rn(__fsub_rn((float)((w >> (4 * q)) & 0xFu), 8.0f), d);
        }
    } else if (type == YULE_DTYPE_Q6_K) {
        const uint32_t h = col0 >> 7, r = col0 & 127u, g = r >> 5, l0 = r & 31u;
        const float d = f16_bits_to_f32(u16_at(208));
        const uint32_t scw = u16_at(192 + 8 * h + 2 * g);  // the two scales of this 32-column group
        const float ds = __fmul_rn(d, (float)(int)(signed char)((l0 >> 4) ? (scw >> 8) : (scw & 0xFFu)));
#pragma unroll
        for (int k = 0; k < 4; k++) {
            const uint32_t ql = u16_at(64 * h + 32 * (g & 1u) + l0 + 2 * k) >> (4 * (g >> 1));
            const uint32_t qh = u16_at(128 + 32 * h + l0 + 2 * k) >> (2 * g);
            const int q0 = (int)((ql & 0xFu) | ((qh & 3u) << 4)) - 32;
            const int q1 = (int)(((ql >> 8) & 0xFu) | (((qh >> 8) & 3u) << 4)) - 32;
            v[2 * k] = __fmul_rn(ds, (float)q0);
            v[2 * k + 1] = __fmul_rn(ds, (float)q1);
        }
    } else if (type == YULE_DTYPE_Q5_K) {
        // dequant.rs:297-338: eight columns of sub-block s; nibbles of group s/2, fifth bits in bit s of qh
        const uint32_t s = col0 >> 5, l0 = col0 & 31u;
        uint32_t sc, mn;
        if (s < 4) {
            sc = unit[4 + s] & 63u;
            mn = unit[8 + s] & 63u;
        } else {
            sc = (unit[8 + s] & 0xFu) | ((unit[s] >> 6) << 4);
            mn = (unit[8 + s] >> 4) | ((unit[4 + s] >> 6) << 4);
        }
        const float ds = __fmul_rn(f16_bits_to_f32(u16_at(0)), (float)sc);
        const float dm = __fmul_rn(f16_bits_to_f32(u16_at(2)), (float)mn);
#pragma unroll
        for (int k = 0; k < 4; k++) {
            const uint32_t ql = u16_at(48 + 32 * (s >> 1) + l0 + 2 * k) >> (4 * (s & 1u));
            const uint32_t qh = u16_at(16 + l0 + 2 * k) >> s;
            const uint32_t q0 = (ql & 0xFu) | ((qh & 1u) << 4), q1 = ((ql >> 8) & 0xFu) | (((qh >> 8) & 1u) << 4);
            v[2 * k] = __fsub_rn(__fmul_rn((float)q0, ds), dm);
            v[2 * k + 1] = __fsub_rn(__fmul_rn((float)q1, ds), dm);
        }
    } else if (type == YULE_DTYPE_Q2_K) {
        // dequant.rs:196-214: (d*scale)*q - dmin*min, sub-blocks of 16
        const uint32_t sm = unit[col0 >> 4];
        const float ds = __fmul_rn(f16_bits_to_f32(u16_at(80)), (float)(sm & 0xFu));
        const float dm = __fmul_rn(f16_bits_to_f32(u16_at(82)), (float)(sm >> 4));
        const uint32_t qs = u16_at(16 + (col0 >> 2));
#pragma unroll
        for (int k = 0; k < 8; k++) v[k] = __fsub_rn(__fmul_rn(ds, (float)((qs >> (2 * k)) & 3u)), dm);
    } else if (type == YULE_DTYPE_Q3_K) {
        // dequant.rs:219-251: 6-bit scale centred at 32, 3-bit weight centred at 4
        const uint32_t j = col0 >> 4;
        const uint32_t lo4 = j < 8 ? (unit[96 + j] & 0xFu) : (unit[88 + j] >> 4);
        const uint32_t hi2 = (unit[104 + (j >> 2)] >> (2 * (j & 3u))) & 3u;
        const float ds = __fmul_rn(f16_bits_to_f32(u16_at(108)), (float)((int)(lo4 | (hi2 << 4)) - 32));
        const uint32_t qs = u16_at(32 + (col0 >> 2)), hm = unit[col0 >> 3];
#pragma unroll
        for (int k = 0; k < 8; k++)
            v[k] = __fmul_rn(ds, (float)((int)(((qs >> (2 * k)) & 3u) | (((hm >> k) & 1u) << 2)) - 4));
    } else if (type == YULE_DTYPE_Q8_1) {
        const uint32_t b = (col0 >> 5) * 36, i0 = col0 & 31u;
        const float d = f16_bits_to_f32(u16_at(b));
#pragma unroll
        for (int k = 0; k < 4; k++) {
            const uint32_t w = u16_at(b + 4 + i0 + 2 * k);
            v[2 * k] = __fmul_rn((float)(int)(signed char)(w & 0xFFu), d);
            v[2 * k + 1] = __fmul_rn((float)(int)(signed char)(w >> 8), d);
        }
    } else if (type == YULE_DTYPE_Q4_1 || type == YULE_DTYPE_Q5_0 || type == YULE_DTYPE_Q5_1) {
        // dequant.rs:91-138: optional minimum m after d, optional 32 fifth bits before the nibbles
        const bool has_m = type != YULE_DTYPE_Q5_0, has_qh = type != YULE_DTYPE_Q4_1;
        const uint32_t bb = type == YULE_DTYPE_Q4_1 ? 20u : type == YULE_DTYPE_Q5_0 ? 22u : 24u;
        const uint32_t b = (col0 >> 5) * bb, i0 = col0 & 31u;
        const uint32_t qh_off = has_m ? 4u : 2u, qs_off = qh_off + (has_qh ? 4u : 0u);
        const float d = f16_bits_to_f32(u16_at(b));
        const float m = has_m ? f16_bits_to_f32(u16_at(b + 2)) : 0.f;
        const uint32_t qh = has_qh ? unit[b + qh_off + (i0 >> 3)] : 0u;
        const uint32_t qs = u16_at(b + qs_off + (i0 >> 1)) | (u16_at(b + qs_off + (i0 >> 1) + 2) << 16);
#pragma unroll
        for (int k = 0; k < 8; k++) {
            const float q = (float)(((qs >> (4 * k)) & 0xFu) | (((qh >> k) & 1u) << 4));
            v[k] = has_m ? __fadd_rn(__fmul_rn(q, d), m) : __fmul_rn(__fsub_rn(q, 16.0f), d);
        }
    } else {
#pragma unroll
        for (int i = 0; i < 8; i++) v[i] = dequant_elem(unit, type, col0 + i);
    }
}

// Position in the stage ring without a runtime division (an integer division runs on the same
// slow pipe as the half conversions): slot and phase parity, advanced once per stage.
struct RingPos {
    uint32_t s = 0, ph = 0;
    __device__ __forceinline__ void advance(uint32_t stages) {
        if (++s == stages) {
            s = 0;
            ph ^= 1u;
        }
    }
};

// A work item: tile (row tile x activation tile) and the range of super-blocks [sb0, sb1) of its columns.
struct Item {
    uint32_t tile, ks, mt, nt, sb0, sb1, seg;  // mt: row tile inside matrix `seg`
};
__device__ __forceinline__ Item decode_item(const GemmParams &p, uint32_t item, uint32_t bpr) {
    Item r;
    r.tile = item / p.ksplit;
    r.ks = item - r.tile * p.ksplit;
    r.mt = r.tile / p.n_ntiles;
    r.nt = r.tile - r.mt * p.n_ntiles;
    r.seg = 0;
    while (r.seg + 1 < p.n_seg && r.mt >= p.mt0[r.seg + 1]) r.seg++;
    r.mt -= p.mt0[r.seg];
    r.sb0 = r.ks * p.sb_per;
    r.sb1 = r.sb0 + p.sb_per < bpr ? r.sb0 + p.sb_per : bpr;
    return r;
}
// The (work item, super-block) pairs of this CTA in the order every role goes through them.
struct UnitWalk {
    uint32_t item, sb, sb1, mt, seg;
    bool live;
    __device__ __forceinline__ void load(const GemmParams &p, uint32_t n_items, uint32_t bpr) {
        live = item < n_items;
        if (live) {
            const Item it = decode_item(p, item, bpr);
            sb = it.sb0;
            sb1 = it.sb1;
            mt = it.mt;
            seg = it.seg;
        }
    }
    __device__ __forceinline__ void start(const GemmParams &p, uint32_t n_items, uint32_t bpr) {
        item = blockIdx.x;
        load(p, n_items, bpr);
    }
    __device__ __forceinline__ void next(const GemmParams &p, uint32_t n_items, uint32_t bpr) {
        if (++sb == sb1) {
            item += gridDim.x;
            load(p, n_items, bpr);
        }
    }
};

// One row's share of a super-block: the 16-byte header (d, dmin, packed scales) and this thread's
// 16 of the 32 quant bytes of each of the four 64-column groups.
struct RowBlock {
    uint4 hdr;
    uint4 q[4];
};

// GENERIC = false: the Q4_K kernel with exact integer operands.  GENERIC = true: any block format;
// the producers dequantise to fp32 exactly as the CPU code does and split the value, scaled by 2^10,
// into fp16 hi + lo; three MMAs per 16 columns (W_hi·x_hi, W_hi·x_lo, W_lo·x_hi); no raw-block ring.
template <int BN, bool GENERIC>
struct Tile {
    // Up to 64 activation rows the hi and lo terms of the activations sit side by side as one operand of 2·BN rows:
    // one MMA per 16 columns instead of two (an MMA reads its 4 KB of W from shared memory whatever its width, which
    // is what a narrow MMA costs), the two products land in neighbouring accumulator columns and the drain adds them.
    static constexpr bool MERGED = BN <= 64;
    // TMEM accumulator sets in flight.  Up to 64 rows every set has its own min accumulator.  At 128 rows the min
    // accumulator (written by one MMA per super-block, read by the drain of that stage) is shared by all sets, which
    // leaves room for three main accumulators instead of two: the MMA of stage i + 3 waits for the drain of stage i,
    // which is after the drain of any earlier min term.  With two sets the issue-then-drain cycle of a set (about
    // 600 cycles each at 128 rows) bounded a stage at 750 cycles whatever the other buffers.
    static constexpr bool SHARED_MIN = BN == 128;
    static constexpr uint32_t NBUF = BN == 32 ? 4 : (SHARED_MIN ? (GENERIC ? 4 : 3) : 2);
    static constexpr uint32_t kMainCols = MERGED ? 2 * BN : BN;
    static constexpr uint32_t kBufCols = SHARED_MIN ? kMainCols : kMainCols + BN;  // main (+ min) accumulator of a set
    static constexpr uint32_t kMinBase = SHARED_MIN ? 3 * kMainCols : kMainCols;   // shared: column 384; else behind the set's main
    static constexpr uint32_t kTmemCols = 512;               // allocated as a power of two
    static constexpr uint32_t CW = BN / 2;                   // columns per drain warp
    static constexpr uint32_t kXHalfBytes = BN * kBK * 2;    // one fp16 term of the activation slab
    static constexpr uint32_t kBmBytes = BN * 16 * 2;        // sub-block sums of x: BN rows × (8 hi + 8 lo)
    static constexpr uint32_t KG = groups_per_stage(BN, GENERIC);  // 64-column groups per stage
    static constexpr uint32_t SPB = 4 / KG;                        // stages per super-block
    // stage (exact):   W (KG groups) | m | KG × (x_hi | x_lo) | sums   (everything after m arrives in one bulk copy)
    // stage (generic): W_hi | W_lo | x_hi | x_lo
    static constexpr uint32_t kOffAm = KG * kABytes, kOffX = GENERIC ? 2 * kABytes : KG * kABytes + kAmBytes;
    static constexpr uint32_t kOffSums = kOffX + KG * 2 * kXHalfBytes;
    static constexpr uint32_t kStageBytes = kOffSums + (GENERIC ? 0u : kBmBytes);
    static constexpr uint32_t kRaw = raw_slots_for(BN);
    static constexpr uint32_t kRawRingBytes = GENERIC ? 0u : kRaw * kRawBytes;  // generic: sized at launch
    // activation tiles in global memory, per (activation tile, super-block): four (hi, lo) slabs, then the sums
    static constexpr uint32_t kSuperBytes = 8 * kXHalfBytes + kBmBytes;
};

template <int BN, bool GENERIC>
__global__ void __launch_bounds__(kGemmThreads, 1) qgemm_tc_kernel(const __grid_constant__ GemmParams p, const __grid_constant__ GemmMaps w_maps) {
    using T = Tile<BN, GENERIC>;
    constexpr uint32_t NBUF = T::NBUF, CW = T::CW, kXHalfBytes = T::kXHalfBytes, kStageBytes = T::kStageBytes;
    extern __shared__ __align__(128) unsigned char smem[];
    yule_pdl_launch_dependents();
    const uint32_t skip = kProfile ? p.skip : 0u;  // the timing aids exist only in profiling builds
    const long long t_entry = (kProfile && p.prof) ? clock64() : 0;
    const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    unsigned char *tail = smem + (size_t)p.stages * kStageBytes;
    unsigned char *raw = tail;                               // kRawSlots boxes of raw Q4_K bytes
    uint64_t *bars = reinterpret_cast<uint64_t *>(tail + (GENERIC ? p.raw_ring_bytes : T::kRawRingBytes));  // full[6] empty[6] acc_full[4] acc_empty[4] raw_full[4] raw_empty[4]
    const uint32_t bar_full = smem_u32(bars), bar_empty = bar_full + 8 * kMaxStages;
    const uint32_t bar_acc_full = bar_empty + 8 * kMaxStages, bar_acc_empty = bar_acc_full + 32;
    const uint32_t bar_raw_full = bar_acc_empty + 32, bar_raw_empty = bar_raw_full + 8 * kRawSlots;
    uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(bars + 2 * kMaxStages + 8 + 2 * kRawSlots);
    volatile int *abort_flag = reinterpret_cast<volatile int *>(tmem_slot + 1);
    volatile uint32_t *mma_progress = reinterpret_cast<volatile uint32_t *>(tmem_slot + 2);  // per MMA thread: stages seen full

    if (threadIdx.x == 0) {
        for (uint32_t s = 0; s < p.stages; s++) {
            mbar_init(bar_full + 8 * s, kProdWarps + 1);  // one arrival per producer warp + the loader's expect_tx
            mbar_init(bar_empty + 8 * s, 1);              // tcgen05.commit
        }
        for (uint32_t b = 0; b < NBUF; b++) {
            mbar_init(bar_acc_full + 8 * b, 1);
            mbar_init(bar_acc_empty + 8 * b, kEpiWarps);
        }
        for (uint32_t b = 0; b < T::kRaw; b++) {
            mbar_init(bar_raw_full + 8 * b, 1);            // the loader's expect_tx
            mbar_init(bar_raw_empty + 8 * b, kProdWarps);  // every producer warp is done with the box
        }
        *abort_flag = 0;
        mma_progress[0] = mma_progress[1] = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        fence_async_smem();
    }
    if (warp == kMmaWarp) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(T::kTmemCols)
                     : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    const uint32_t n_items = p.n_mtiles * p.n_ntiles * p.ksplit;
    const uint32_t bpr = p.n_cols / 256;  // super-blocks per row

    if (warp == kLoaderWarp) {
        if (lane == 0) {
            yule_pdl_wait();  // the activation tiles come from the kernel before this one
            uint32_t it = 0;
            RingPos ring;
            bool ok = true;
            for (uint32_t item = blockIdx.x; item < n_items && ok; item += gridDim.x) {
                const Item wi = decode_item(p, item, bpr);
                const unsigned char *src = reinterpret_cast<const unsigned char *>(p.xb) + (size_t)wi.nt * bpr * T::kSuperBytes;
                for (uint32_t kb = T::SPB * wi.sb0; kb < T::SPB * wi.sb1; kb++, it++, ring.advance(p.stages)) {
                    const uint32_t s = ring.s, ph = ring.ph;
                    if (!mbar_wait(bar_empty + 8 * s, ph ^ 1u, abort_flag, p.status)) {
                        ok = false;
                        break;
                    }
                    const uint32_t g = kb % T::SPB;
                    const uint32_t bytes = T::KG * 2 * kXHalfBytes + ((!GENERIC && g == T::SPB - 1) ? T::kBmBytes : 0u);  // the sums ride with the last stage
                    const uint32_t dst = smem_u32(smem + (size_t)s * kStageBytes + T::kOffX);
                    if (skip & 8u) {
                        mbar_arrive(bar_full + 8 * s);
                        continue;
                    }
                    mbar_arrive_expect_tx(bar_full + 8 * s, bytes);
                    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(dst),
                                 "l"(src + (size_t)(kb / T::SPB) * T::kSuperBytes + (size_t)g * T::KG * 2 * kXHalfBytes), "r"(bytes),
                                 "r"(bar_full + 8 * s)
                                 : "memory");
                }
            }
        }
    } else if (warp == kMmaWarp || warp == kMmaWarp2) {
        if (lane == 0) {
            const uint32_t parity_of_mine = warp == kMmaWarp ? 0u : 1u;  // this thread issues the stages with it % 2 == parity
            // fp16 × fp16 → fp32, both operands K-major, M = 128, N = BN
            constexpr uint32_t idesc = (1u << 4) | ((uint32_t)(BN >> 3) << 17) | ((uint32_t)(kBM >> 4) << 24);
            [[maybe_unused]] constexpr uint32_t idesc2 = (1u << 4) | ((uint32_t)((2 * BN) >> 3) << 17) | ((uint32_t)(kBM >> 4) << 24);  // N = 2·BN
            constexpr uint32_t x_lbo = BN * 16;  // bytes of one 8-column step of an activation slab (of its hi or lo rows)
            uint32_t it = 0;
            bool ok = true;
            RingPos ring;
            long long tw0 = 0, tw1 = 0, ti = 0, tc = 0;
            const long long tstart = (kProfile && p.prof) ? clock64() : 0;
            for (uint32_t item = blockIdx.x; item < n_items && ok; item += gridDim.x) {
                const Item wi = decode_item(p, item, bpr);
                for (uint32_t kb = T::SPB * wi.sb0; kb < T::SPB * wi.sb1; kb++, it++, ring.advance(p.stages)) {
                    const bool mine = (it & 1u) == parity_of_mine;  // the threads alternate stages
                    const uint32_t s = ring.s, ph = ring.ph;
                    const uint32_t buf = it % NBUF, aph = (it / NBUF) & 1u;
                    const long long c0 = (kProfile && p.prof) ? clock64() : 0;
                    if (mine && !(skip & 16u) && !mbar_wait(bar_acc_empty + 8 * buf, aph ^ 1u, abort_flag, p.status)) {
                        ok = false;
                        break;
                    }
                    if (!mine) continue;
                    const long long c1 = (kProfile && p.prof) ? clock64() : 0;
                    // A parity wait only tells phase k of a barrier from phase k - 1.  The previous use of this
                    // stage may belong to the other thread: wait until it has seen that phase complete, so that
                    // this thread never asks for a phase two ahead of the barrier's.
                    if (it >= p.stages && ((it - p.stages) & 1u) != parity_of_mine) {
                        const long long t0 = clock64();
                        while (mma_progress[parity_of_mine ^ 1u] < it - p.stages + 1) {
                            if (*abort_flag || clock64() - t0 > kWaitCycles) {
                                *abort_flag = 1;
                                atomicExch(p.status, kStatusGemmTimeout);
                                ok = false;
                                break;
                            }
                        }
                        if (!ok) break;
                    }
                    if (!mbar_wait(bar_full + 8 * s, ph, abort_flag, p.status)) {
                        ok = false;
                        break;
                    }
                    mma_progress[parity_of_mine] = it + 1;
                    const long long c2 = (kProfile && p.prof) ? clock64() : 0;
                    tw0 += c1 - c0;
                    tw1 += c2 - c1;
                    tc_fence_after();
                    const uint32_t d_main = tmem_base + buf * T::kBufCols;
                    [[maybe_unused]] const uint32_t d_min = T::SHARED_MIN ? tmem_base + T::kMinBase : d_main + T::kMinBase;
                    const uint32_t a = smem_u32(smem + (size_t)s * kStageBytes);
                    const uint32_t x_hi = a + T::kOffX;
                    // One descriptor per operand and stage; the 16-column steps are constants added to its address field (the
                    // issuing thread's own instruction stream, not the tensor pipe, bounded the MMA rate).
                    const uint64_t da0 = smem_desc(a, 2048, 128);
                    const uint64_t db0 = T::MERGED ? smem_desc(x_hi, 2 * x_lbo, 128) : smem_desc(x_hi, x_lbo, 128);
                    auto step = [&](auto k16c) {
                        constexpr uint32_t k16 = decltype(k16c)::value;
                        const uint64_t da = da0 + (uint64_t)((k16 * 4096u) >> 4);
                        if constexpr (T::MERGED) {
                            // rows [0, BN) of an 8-column step are the hi terms, rows [BN, 2·BN) the lo terms
                            const uint64_t db = db0 + (uint64_t)((k16 * 4u * x_lbo) >> 4);
                            umma_f16_c<(k16 != 0)>(d_main, da, db, idesc2);  // every stage starts a fresh accumulator
                            if (GENERIC)  // the lo term of the weights against the hi term of the activations: the first BN rows
                                umma_f16_c<1>(d_main, da + (uint64_t)(kABytes >> 4), db, idesc);
                        } else {
                            const uint64_t dbh = db0 + (uint64_t)((k16 * 2u * x_lbo) >> 4);
                            umma_f16_c<(k16 != 0)>(d_main, da, dbh, idesc);  // every stage starts a fresh accumulator
                            umma_f16_c<1>(d_main, da, dbh + (uint64_t)(kXHalfBytes >> 4), idesc);
                            if (GENERIC)  // the lo term of the weights against the hi term of the activations
                                umma_f16_c<1>(d_main, da + (uint64_t)(kABytes >> 4), dbh, idesc);
                        }
                    };
                    if (!(skip & 2u)) {
                        step(std::integral_constant<uint32_t, 0>{});
                        step(std::integral_constant<uint32_t, 1>{});
                        step(std::integral_constant<uint32_t, 2>{});
                        step(std::integral_constant<uint32_t, 3>{});
                        if constexpr (T::KG == 2) {  // the second group's slabs follow the first's in both operands
                            step(std::integral_constant<uint32_t, 4>{});
                            step(std::integral_constant<uint32_t, 5>{});
                            step(std::integral_constant<uint32_t, 6>{});
                            step(std::integral_constant<uint32_t, 7>{});
                        }
                    }
                    if (!GENERIC && kb % T::SPB == T::SPB - 1)  // Σ_s m_s · (sum of x over sub-block s), hi and lo sums side by side
                        umma_f16(d_min, smem_desc(a + T::kOffAm, 2048, 128), smem_desc(a + T::kOffSums, x_lbo, 128), idesc, 0u);
                    const long long c3 = (kProfile && p.prof) ? clock64() : 0;
                    umma_commit(bar_empty + 8 * s);       // the slabs may be overwritten once these MMAs are done
                    if (!(skip & 32u)) umma_commit(bar_acc_full + 8 * buf);  // and the accumulators may be drained
                    if (skip & 256u) mbar_wait(bar_empty + 8 * s, ph, abort_flag, p.status);  // timing aid: the commit's own latency, charged to `commit`
                    const long long c4 = (kProfile && p.prof) ? clock64() : 0;
                    ti += c3 - c2;
                    tc += c4 - c3;
                }
            }
            if ((kProfile && p.prof) && blockIdx.x == 0 && warp == kMmaWarp) {
                g_gemm_prof[0] = clock64() - tstart;
                g_gemm_prof[1] = tw0;
                g_gemm_prof[2] = tw1;
                g_gemm_prof[3] = ti;
                g_gemm_prof[4] = tc;
                g_gemm_prof[5] = it;
            }
        }
    } else if (warp == kRawWarp) {
        if (!GENERIC && lane == 0) {
            UnitWalk walk;
            walk.start(p, n_items, bpr);
            for (uint32_t u = 0; walk.live; u++, walk.next(p, n_items, bpr)) {
                const uint32_t slot = u % T::kRaw, ph = (u / T::kRaw) & 1u;
                if (!mbar_wait(bar_raw_empty + 8 * slot, ph ^ 1u, abort_flag, p.status)) break;
                const uint32_t x = walk.sb * 144u, y = walk.mt * kBM;  // byte column (a multiple of 16), first row
                if (skip & 64u) {  // timing aid: no raw bytes
                    mbar_arrive(bar_raw_full + 8 * slot);
                    continue;
                }
                mbar_arrive_expect_tx(bar_raw_full + 8 * slot, kRawBytes);
                asm volatile(
                    "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];" ::"r"(
                        smem_u32(raw + (size_t)slot * kRawBytes)),
                    "l"(reinterpret_cast<uint64_t>(&w_maps.m[walk.seg])), "r"(bar_raw_full + 8 * slot), "r"(x), "r"(y)
                    : "memory");
            }
        }
    } else if (warp >= kFirstProdWarp) {
        const uint32_t ptid = threadIdx.x - kFirstProdWarp * 32;  // 0..255
        const uint32_t r = ptid & 127u, hf = ptid >> 7;           // row of the tile, which 16 bytes of the 32
        if (GENERIC) {
            // Any block format.  The eight producer warps copy a 256-column unit of the raw bytes of the tile's 128
            // rows into one of two shared-memory slots with 16-byte cp.async from the aligned address at or below
            // each row's unit start (the blocks themselves are only 2-byte aligned), always one unit ahead of the
            // one being unpacked; thread (r, hf) then dequantises columns [32·hf, 32·hf + 32) of every stage for
            // row r from that copy with the arithmetic of the bit-exact per-element routines, scales by 2^10 and
            // splits into fp16 hi + lo.
            const uint32_t in_core = (r >> 3) * 128 + (r & 7u) * 16;
            const uint32_t ub = p.unit_bytes, rstride = p.raw_stride, c16 = p.raw_chunks;
            const uint32_t slot_bytes = kBM * rstride;
            auto unit_start = [&](const UnitWalk &w, uint32_t tile_row) {  // address of row `tile_row`'s bytes of the unit
                uint32_t grow = w.mt * kBM + tile_row;
                grow = grow < p.n_rows[w.seg] ? grow : p.n_rows[w.seg] - 1;
                return reinterpret_cast<uintptr_t>(p.w[w.seg]) + (size_t)grow * p.w_row_bytes + (size_t)w.sb * ub;
            };
            auto copy_unit = [&](const UnitWalk &w, uint32_t u) {
                if (w.live) {
                    const uint32_t dst0 = smem_u32(raw + (size_t)(u & 1u) * slot_bytes);
                    uint32_t row = 0, c = ptid;
                    while (c >= c16) {
                        c -= c16;
                        row++;
                    }
                    for (uint32_t e = ptid; e < kBM * c16; e += 256) {
                        const uintptr_t src = (unit_start(w, row) & ~(uintptr_t)15) + (size_t)c * 16;
                        asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst0 + row * rstride + c * 16), "l"(src) : "memory");
                        c += 256;
                        while (c >= c16) {
                            c -= c16;
                            row++;
                        }
                    }
                }
                asm volatile("cp.async.commit_group;" ::: "memory");  // one group per unit, empty past the end
            };
            RingPos ring;
            bool ok = true;
            UnitWalk cur, ahead;  // the unit being unpacked and the one being copied
            cur.start(p, n_items, bpr);
            ahead = cur;
            copy_unit(ahead, 0);
            for (uint32_t u = 0; cur.live && ok; u++, cur = ahead) {
                ahead.next(p, n_items, bpr);
                copy_unit(ahead, u + 1);
                asm volatile("cp.async.wait_group 1;" ::: "memory");   // this thread's copies of unit u have landed
                asm volatile("bar.sync 2, 256;" ::: "memory");         // and everyone else's
                const bool live = cur.mt * kBM + r < p.n_rows[cur.seg];
                const unsigned char *rawrow = raw + (size_t)(u & 1u) * slot_bytes + (size_t)r * rstride + (unit_start(cur, r) & 15u);
                for (uint32_t g = 0; g < 4 && ok; g++, ring.advance(p.stages)) {
                    if (!mbar_wait(bar_empty + 8 * ring.s, ring.ph ^ 1u, abort_flag, p.status)) {
                        ok = false;
                        break;
                    }
                    unsigned char *a_hi = smem + (size_t)ring.s * kStageBytes, *a_lo = a_hi + kABytes;
#pragma unroll 1
                    for (uint32_t c8 = 0; c8 < 4; c8++) {
                        const uint32_t col0 = g * kBK + hf * 32 + c8 * 8;  // column inside the unit
                        float v[8];
                        dequant8_unit(rawrow, p.type, col0, v);
#pragma unroll
                        for (int i = 0; i < 8; i++) v[i] = live ? v[i] * kGenericWScale : 0.f;
                        // positions 0..7 of the 16 bytes hold columns 0,2,1,3,4,6,5,7 (the order of the activation tiles)
                        const float o[8] = {v[0], v[2], v[1], v[3], v[4], v[6], v[5], v[7]};
                        uint32_t h[4], l[4];
#pragma unroll
                        for (int i = 0; i < 4; i++) {
                            const __half2 hh = __floats2half2_rn(o[2 * i], o[2 * i + 1]);
                            const float2 back = __half22float2(hh);
                            h[i] = as_u32(hh);
                            l[i] = as_u32(__floats2half2_rn(o[2 * i] - back.x, o[2 * i + 1] - back.y));
                        }
                        const uint32_t kc = hf * 4 + c8;
                        *reinterpret_cast<uint4 *>(a_hi + kc * 2048 + in_core) = make_uint4(h[0], h[1], h[2], h[3]);
                        *reinterpret_cast<uint4 *>(a_lo + kc * 2048 + in_core) = make_uint4(l[0], l[1], l[2], l[3]);
                    }
                    fence_async_smem();
                    __syncwarp();
                    if (lane == 0) mbar_arrive(bar_full + 8 * ring.s);
                }
                asm volatile("bar.sync 2, 256;" ::: "memory");  // the slot may be overwritten by unit u + 2
            }
            asm volatile("cp.async.wait_group 0;" ::: "memory");
        } else {
        uint32_t it = 0;
        bool ok = true;
        const uint32_t in_core = (r >> 3) * 128 + (r & 7u) * 16;
        const __half2 k1024 = __half2half2(__ushort_as_half(0x6400)), kneg1024 = __half2half2(__ushort_as_half(0xE400));
        RingPos ring;
        long long pw = 0, pk = 0, pf = 0;
        const long long pstart = (kProfile && p.prof) ? clock64() : 0;
        // the four stages of one super-block
        auto unpack_block = [&](const RowBlock &cur) {
            const ScalesMins sm = q4k_scales_mins(cur.hdr.y, cur.hdr.z, cur.hdr.w);
#pragma unroll
            for (uint32_t g = 0; g < 4; g++, it++) {
                const uint32_t s = ring.s, ph = ring.ph;
                const bool opens = g % T::KG == 0, closes = g % T::KG == T::KG - 1;  // first / last group of its stage
                // scales of sub-blocks 2g (low nibbles) and 2g + 1 (high nibbles) as fp16 pairs (sc, sc)
                const uint32_t scw = g < 2 ? sm.sc_lo : sm.sc_hi, j0 = (2 * g) & 3u;
                const __half2 sc0 = __hsub2(as_half2(biased_pair(scw, 0x4040u + j0 * 0x0101u)), k1024);
                const __half2 sc1 = __hsub2(as_half2(biased_pair(scw, 0x4040u + (j0 + 1) * 0x0101u)), k1024);
                const __half2 nb0 = __hmul2(sc0, kneg1024), nb1 = __hmul2(sc1, kneg1024);  // −1024·sc ≥ −64512: exact
                const long long c0 = (kProfile && p.prof) ? clock64() : 0;
                if (opens && !mbar_wait(bar_empty + 8 * s, ph ^ 1u, abort_flag, p.status)) {
                    ok = false;
                    return;
                }
                const long long c1 = (kProfile && p.prof) ? clock64() : 0;
                pw += c1 - c0;
                unsigned char *stage = smem + (size_t)s * kStageBytes, *a = stage + (g % T::KG) * kABytes;
                // byte b of the 32 holds column b (low nibble, sub-block 2g) and column 32 + b (high nibble)
                const uint32_t qw[4] = {cur.q[g].x, cur.q[g].y, cur.q[g].z, cur.q[g].w};
#pragma unroll
                for (int half8 = 0; half8 < 2; half8++) {
                    if (skip & 1u) break;
                    const uint32_t w0 = qw[2 * half8], w1 = qw[2 * half8 + 1];
                    const uint32_t kc_lo = hf * 2 + half8;  // 8-column step of the low-nibble columns
                    // (1024 + q)·sc − 1024·sc = q·sc, exact; pairs are bytes (0, 2) and (1, 3) of a word
                    auto mul = [&](uint32_t nib_pair, __half2 sc, __half2 nb) {
                        return as_u32(__hfma2(as_half2((nib_pair & 0x000F000Fu) | 0x64006400u), sc, nb));
                    };
                    uint4 lo, hi;
                    lo.x = mul(w0, sc0, nb0);
                    lo.y = mul(w0 >> 8, sc0, nb0);
                    lo.z = mul(w1, sc0, nb0);
                    lo.w = mul(w1 >> 8, sc0, nb0);
                    hi.x = mul(w0 >> 4, sc1, nb1);
                    hi.y = mul(w0 >> 12, sc1, nb1);
                    hi.z = mul(w1 >> 4, sc1, nb1);
                    hi.w = mul(w1 >> 12, sc1, nb1);
                    *reinterpret_cast<uint4 *>(a + kc_lo * 2048 + in_core) = lo;
                    *reinterpret_cast<uint4 *>(a + (4 + kc_lo) * 2048 + in_core) = hi;
                }
                if (g == 3) {
                    // the eight mins of the super-block, twice: columns 0-7 meet the hi sums, 8-15 the lo sums
                    uint4 m;
                    m.x = as_u32(__hsub2(as_half2(biased_pair(sm.m_lo, 0x5140u)), k1024));
                    m.y = as_u32(__hsub2(as_half2(biased_pair(sm.m_lo, 0x5342u)), k1024));
                    m.z = as_u32(__hsub2(as_half2(biased_pair(sm.m_hi, 0x5140u)), k1024));
                    m.w = as_u32(__hsub2(as_half2(biased_pair(sm.m_hi, 0x5342u)), k1024));
                    *reinterpret_cast<uint4 *>(stage + T::kOffAm + hf * 2048 + in_core) = m;
                }
                const long long c2 = (kProfile && p.prof) ? clock64() : 0;
                if (closes) {
                    fence_async_smem();  // generic-proxy stores → visible to the tensor core's reads
                    __syncwarp();
                    if (lane == 0) mbar_arrive(bar_full + 8 * s);
                    ring.advance(p.stages);
                }
                const long long c3 = (kProfile && p.prof) ? clock64() : 0;
                pk += c2 - c1;
                pf += c3 - c2;
            }
        };
        UnitWalk walk;
        walk.start(p, n_items, bpr);
        for (uint32_t u = 0; walk.live && ok; u++, walk.next(p, n_items, bpr)) {
            const uint32_t slot = u % T::kRaw, ph = (u / T::kRaw) & 1u;
            if (!mbar_wait(bar_raw_full + 8 * slot, ph, abort_flag, p.status)) break;
            // row r of the box: 144 bytes; rows are 36 words apart, so eight lanes cover all 32 banks
            const unsigned char *bp = raw + (size_t)slot * kRawBytes + r * 144u;
            RowBlock cur;
            cur.hdr = *reinterpret_cast<const uint4 *>(bp);
#pragma unroll
            for (int g = 0; g < 4; g++) cur.q[g] = *reinterpret_cast<const uint4 *>(bp + 16 + g * 32 + hf * 16);
            unpack_block(cur);
            __syncwarp();
            if (lane == 0) mbar_arrive(bar_raw_empty + 8 * slot);  // this warp is done with the box
        }
        if ((kProfile && p.prof) && blockIdx.x == 0 && ptid == 0) {
            g_gemm_prof[6] = clock64() - pstart;
            g_gemm_prof[7] = pw;
            g_gemm_prof[8] = pk;
            g_gemm_prof[9] = pf;
        }
        }  // exact Q4_K producer
    } else {
        // drain warp: TMEM lanes [32·(warp % 4), +32) = rows of the tile, columns [CW·(warp / 4), +CW)
        const long long t_ready = (kProfile && p.prof) ? clock64() : 0;
        yule_pdl_wait();
        const uint32_t lane_base = (warp & 3u) * 32u, col_base = (warp >> 2) * CW;
        uint32_t it = 0;
        bool ok = true;
        long long dw = 0, t_loop_end = 0;
        const long long dstart = (kProfile && p.prof) ? clock64() : 0;
        for (uint32_t item = blockIdx.x; item < n_items && ok; item += gridDim.x) {
            const Item wi = decode_item(p, item, bpr);
            const uint32_t mt = wi.mt, nt = wi.nt;
            const uint32_t row = mt * kBM + lane_base + lane;
            const uint8_t *rowp = p.w[wi.seg] + (size_t)(row < p.n_rows[wi.seg] ? row : p.n_rows[wi.seg] - 1) * bpr * 144;
            float acc[CW];
#pragma unroll
            for (uint32_t j = 0; j < CW; j++) acc[j] = 0.f;
            uint32_t dd_cur = 0, dd_next = GENERIC ? 0u : __ldg(reinterpret_cast<const uint32_t *>(rowp + (size_t)wi.sb0 * 144));  // (d, dmin) of the first super-block
            const uint32_t kb_end = T::SPB * wi.sb1;
            for (uint32_t kb = T::SPB * wi.sb0; kb < kb_end; kb++, it++) {
                if (skip & 32u) break;
                const uint32_t buf = it % NBUF, aph = (it / NBUF) & 1u;
                if (!GENERIC && kb % T::SPB == 0u) {  // new super-block: take its (d, dmin), ask for the next one's
                    dd_cur = dd_next;
                    if (kb + T::SPB < kb_end) dd_next = __ldg(reinterpret_cast<const uint32_t *>(rowp + (size_t)(kb / T::SPB + 1) * 144));
                }
                const float2 dd = GENERIC ? make_float2(1.f, 0.f) : __half22float2(as_half2(dd_cur));
                const long long c0 = (kProfile && p.prof) ? clock64() : 0;
                if (!mbar_wait(bar_acc_full + 8 * buf, aph, abort_flag, p.status)) {
                    ok = false;
                    break;
                }
                if ((kProfile && p.prof)) dw += clock64() - c0;
                tc_fence_after();
                const uint32_t t_main = tmem_base + (lane_base << 16) + buf * T::kBufCols + col_base;
                if constexpr (T::MERGED) {
                    // all the loads of the stage in flight together, one wait
                    uint32_t v[CW], vl[CW];
                    if (!(skip & 4u)) {
#pragma unroll
                        for (uint32_t c0 = 0; c0 < CW; c0 += 16) {
                            tmem_ld16_issue(t_main + c0, v + c0);
                            tmem_ld16_issue(t_main + BN + c0, vl + c0);  // the products with the lo terms
                        }
                        tmem_ld_wait();
#pragma unroll
                        for (uint32_t j = 0; j < CW; j++) acc[j] = fmaf(dd.x, __uint_as_float(v[j]) + __uint_as_float(vl[j]), acc[j]);
                    }
                } else {
#pragma unroll
                    for (uint32_t c0 = 0; c0 < CW; c0 += 16) {
                        if (skip & 4u) break;
                        uint32_t v[16];
                        tmem_ld16(t_main + c0, v);
#pragma unroll
                        for (int j = 0; j < 16; j++) acc[c0 + j] = fmaf(dd.x, __uint_as_float(v[j]), acc[c0 + j]);
                    }
                }
                if (!GENERIC && kb % T::SPB == T::SPB - 1) {  // the stage that ends a super-block carries the min term
#pragma unroll
                    for (uint32_t c0 = 0; c0 < CW; c0 += 16) {
                        uint32_t v[16];
                        tmem_ld16((T::SHARED_MIN ? tmem_base + (lane_base << 16) + col_base : t_main) + T::kMinBase + c0, v);
#pragma unroll
                        for (int j = 0; j < 16; j++) acc[c0 + j] = fmaf(-dd.y * (1.0f / kSumScale), __uint_as_float(v[j]), acc[c0 + j]);
                    }
                }
                tc_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive(bar_acc_empty + 8 * buf);
            }
            if (!ok) break;
            if ((kProfile && p.prof)) t_loop_end = clock64();
            const uint32_t n0 = nt * BN + col_base;
            if (p.ksplit > 1) {
                // This item covers a part of the columns.  Every drain warp stores its block of scaled partial sums, then
                // takes a ticket of its (tile, warp); the warp that finds all the other parts stored adds them in the
                // order of the parts (its own included, so the sum does not depend on who came last) and writes the result.
                float *mine = p.split_part + (size_t)item * (BN * kBM) + lane_base + lane;
#pragma unroll
                for (uint32_t c0 = 0; c0 < CW; c0 += 16) {
                    const float osc = lane < 16 ? p.oscale[n0 + c0 + lane] : 0.f;
#pragma unroll
                    for (int j = 0; j < 16; j++) {
                        const float sc = __shfl_sync(0xffffffffu, osc, j);
                        __stcg(mine + (size_t)(col_base + c0 + j) * kBM, acc[c0 + j] * sc * p.out_scale);
                    }
                }
                __threadfence();
                __syncwarp();
                uint32_t ticket = 0;
                uint32_t *tk = p.split_tickets + (size_t)wi.tile * kEpiWarps + warp;
                if (lane == 0) {
                    ticket = atomicAdd(tk, 1u);
                    if (ticket == p.ksplit - 1) *tk = 0;  // left at zero for the next launch
                }
                ticket = __shfl_sync(0xffffffffu, ticket, 0);
                if (ticket != p.ksplit - 1) continue;
                __threadfence();
                const float *parts = p.split_part + (size_t)(wi.tile * p.ksplit) * (BN * kBM) + (size_t)col_base * kBM + lane_base + lane;
#pragma unroll
                for (uint32_t j = 0; j < CW; j++) acc[j] = 0.f;
                // the loads of up to KS parts are in flight together; the additions keep the order of the parts
                constexpr uint32_t KS = CW <= 16 ? 4 : (CW <= 32 ? 2 : 1);
#pragma unroll 1
                for (uint32_t ks0 = 0; ks0 < p.ksplit; ks0 += KS, parts += KS * BN * kBM) {
                    float v[KS][CW];
#pragma unroll
                    for (uint32_t q = 0; q < KS; q++)
#pragma unroll
                        for (uint32_t j = 0; j < CW; j++)
                            v[q][j] = ks0 + q < p.ksplit ? __ldcg(parts + (size_t)q * (BN * kBM) + (size_t)j * kBM) : 0.f;
#pragma unroll
                    for (uint32_t q = 0; q < KS; q++)
#pragma unroll
                        for (uint32_t j = 0; j < CW; j++) acc[j] += v[q][j];
                }
#pragma unroll
                for (uint32_t j = 0; j < CW; j++) {
                    const uint32_t n = n0 + j;
                    if (row < p.n_rows[wi.seg] && n < p.n_tokens) {
                        const size_t o = (size_t)n * p.out_stride[wi.seg] + row;
                        p.out[wi.seg][o] = p.residual ? acc[j] + p.residual[o] : acc[j];
                    }
                }
                continue;
            }
#pragma unroll
            for (uint32_t c0 = 0; c0 < CW; c0 += 16) {
                const float osc = lane < 16 ? p.oscale[n0 + c0 + lane] : 0.f;  // padded to whole tiles
#pragma unroll
                for (int j = 0; j < 16; j++) {
                    const float sc = __shfl_sync(0xffffffffu, osc, j);
                    const uint32_t n = n0 + c0 + j;
                    if (row < p.n_rows[wi.seg] && n < p.n_tokens) {
                        float val = acc[c0 + j] * sc * p.out_scale;
                        const size_t o = (size_t)n * p.out_stride[wi.seg] + row;
                        if (p.residual) val += p.residual[o];
                        p.out[wi.seg][o] = val;
                    }
                }
            }
        }
        if ((kProfile && p.prof) && blockIdx.x == 0 && threadIdx.x == 0) {
            g_gemm_prof[10] = clock64() - dstart;
            g_gemm_prof[11] = dw;
            g_gemm_prof[12] = t_ready - t_entry;
            g_gemm_prof[13] = dstart - t_ready;
            g_gemm_prof[14] = clock64() - t_loop_end;
        }
    }

    // common exit: nothing of this CTA may still be in flight when its TMEM and shared memory go
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    if (*abort_flag) {
        // gave up: let copies and MMAs that were already issued drain before the resources are freed
        const long long t0 = clock64();
        while (clock64() - t0 < 2000000LL) {
        }
        __syncthreads();
    }
    if (warp == kMmaWarp) {
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(T::kTmemCols) : "memory");
    }
    if ((kProfile && p.prof) && blockIdx.x == 0 && threadIdx.x == 0) g_gemm_prof[15] = clock64() - t_entry;
}

// Activation rows → the GEMM's operand tiles, one CTA per (padded) row: power-of-two row scale,
// fp16 hi/lo split, the column order of the W operand inside every group of eight, and the
// per-32-column sums for the min term.  Optional prologues: RMSNorm (out = x · inv · w as in
// yule-infer/src/model_runner.rs:254-263) or SwiGLU (silu(gate) · x, kernels/cuda/silu_mul.cu:3-14).
struct XprepParams {
    const float *x;
    const float *gate;    // when set: y = silu(gate) · x
    const float *norm_w;  // when set: y = x · inv_rms · norm_w
    float eps;
    uint32_t x_stride, n_tokens, n_cols, bn;
    unsigned char *xb;
    float *oscale;
};

// One CTA of 1024 threads per row; a thread keeps its 8·CHUNKS columns in registers from the single read of the row
// to the stores, so a row of up to 8192·CHUNKS columns costs one round trip to memory and two block reductions
// whatever its length.
constexpr int kXprepThreads = 1024;
template <int CHUNKS>
__global__ void __launch_bounds__(kXprepThreads) gemm_xprep_kernel(const XprepParams p) {
    yule_pdl_launch_dependents();
    yule_pdl_wait();
    __shared__ float red[32];
    const uint32_t n = blockIdx.x, nt = n / p.bn, r = n % p.bn;
    const uint32_t bpr = p.n_cols / 256;
    const uint32_t x_half_bytes = p.bn * kBK * 2, bm_bytes = p.bn * 32, super_bytes = 8 * x_half_bytes + bm_bytes;
    const uint32_t core = ((r >> 3) * 64 + (r & 7u) * 8) * 2;  // byte offset of this row inside an 8-column step
    // 16 bytes of columns [k0, k0 + 8): term 0 = hi, 1 = lo
    auto slab16 = [&](uint32_t k0, uint32_t term) {
        const uint32_t sb = k0 >> 8, g = (k0 >> 6) & 3u, kc = (k0 >> 3) & 7u;
        if (p.bn <= 64)  // hi and lo rows of an 8-column step side by side (one operand of 2·bn rows)
            return p.xb + ((size_t)nt * bpr + sb) * super_bytes + (size_t)(2 * g) * x_half_bytes + (2 * kc + term) * (p.bn * 16) + core;
        return p.xb + ((size_t)nt * bpr + sb) * super_bytes + (size_t)(2 * g + term) * x_half_bytes + kc * (p.bn * 16) + core;
    };
    // the two bytes of sub-block s (of super-block sb) in the sums slab: column s (hi) or 8 + s (lo)
    auto sum_slot = [&](uint32_t sb, uint32_t s, uint32_t term) {
        return reinterpret_cast<__half *>(p.xb + ((size_t)nt * bpr + sb) * super_bytes + 8 * (size_t)x_half_bytes +
                                          term * (p.bn * 16) + core) + s;
    };
    if (n >= p.n_tokens) {  // padding row of the last tile
        for (uint32_t k0 = threadIdx.x * 8; k0 < p.n_cols; k0 += kXprepThreads * 8) {
            *reinterpret_cast<uint4 *>(slab16(k0, 0)) = make_uint4(0, 0, 0, 0);
            *reinterpret_cast<uint4 *>(slab16(k0, 1)) = make_uint4(0, 0, 0, 0);
            if ((k0 & 31u) == 0) {
                *sum_slot(k0 >> 8, (k0 >> 5) & 7u, 0) = __ushort_as_half(0);
                *sum_slot(k0 >> 8, (k0 >> 5) & 7u, 1) = __ushort_as_half(0);
            }
        }
        if (threadIdx.x == 0) p.oscale[n] = 0.f;
        return;
    }
    const float *x = p.x + (size_t)n * p.x_stride;
    const float *gate = p.gate ? p.gate + (size_t)n * p.x_stride : nullptr;
    auto block_reduce = [&](float v, bool is_max) {
        for (int o = 16; o > 0; o >>= 1) {
            const float other = __shfl_xor_sync(0xffffffffu, v, o);
            v = is_max ? fmaxf(v, other) : v + other;
        }
        __syncthreads();
        if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = v;
        __syncthreads();
        v = red[0];
        for (int i = 1; i < kXprepThreads / 32; i++) v = is_max ? fmaxf(v, red[i]) : v + red[i];
        return v;
    };
    // rows start on a 16-byte boundary when the stride is a multiple of four floats; otherwise scalar loads
    const bool vec = ((reinterpret_cast<uintptr_t>(x) | (gate ? reinterpret_cast<uintptr_t>(gate) : 0)) & 15u) == 0;
    float v[CHUNKS][8];
#pragma unroll
    for (int c = 0; c < CHUNKS; c++) {
        const uint32_t k0 = ((uint32_t)c * kXprepThreads + threadIdx.x) * 8;
        if (k0 < p.n_cols) {
            if (vec) {
                const float4 a = *reinterpret_cast<const float4 *>(x + k0), b = *reinterpret_cast<const float4 *>(x + k0 + 4);
                v[c][0] = a.x, v[c][1] = a.y, v[c][2] = a.z, v[c][3] = a.w, v[c][4] = b.x, v[c][5] = b.y, v[c][6] = b.z, v[c][7] = b.w;
            } else {
#pragma unroll
                for (int i = 0; i < 8; i++) v[c][i] = x[k0 + i];
            }
        } else {
#pragma unroll
            for (int i = 0; i < 8; i++) v[c][i] = 0.f;
        }
    }
    if (p.norm_w) {
        float ss = 0.f;
#pragma unroll
        for (int c = 0; c < CHUNKS; c++)
#pragma unroll
            for (int i = 0; i < 8; i++) ss = fmaf(v[c][i], v[c][i], ss);
        ss = block_reduce(ss, false);
        const float inv = 1.0f / sqrtf(ss / (float)p.n_cols + p.eps);
#pragma unroll
        for (int c = 0; c < CHUNKS; c++) {
            const uint32_t k0 = ((uint32_t)c * kXprepThreads + threadIdx.x) * 8;
            if (k0 < p.n_cols) {
#pragma unroll
                for (int i = 0; i < 8; i++) v[c][i] = v[c][i] * inv * p.norm_w[k0 + i];
            }
        }
    }
    if (gate) {
#pragma unroll
        for (int c = 0; c < CHUNKS; c++) {
            const uint32_t k0 = ((uint32_t)c * kXprepThreads + threadIdx.x) * 8;
            if (k0 < p.n_cols) {
#pragma unroll
                for (int i = 0; i < 8; i++) {
                    const float gt = gate[k0 + i];
                    v[c][i] = (gt / (1.0f + expf(-gt))) * v[c][i];
                }
            }
        }
    }
    float amax = 0.f;
#pragma unroll
    for (int c = 0; c < CHUNKS; c++)
#pragma unroll
        for (int i = 0; i < 8; i++) amax = fmaxf(amax, fabsf(v[c][i]));
    amax = block_reduce(amax, true);
    // power of two that puts the largest element in [2^13, 2^14)
    float scale = 1.f;
    if (amax > 1e-30f && amax < 1e30f) {
        int ex;
        frexpf(amax, &ex);  // amax = m · 2^ex, m in [0.5, 1)
        scale = ldexpf(1.f, 14 - ex);
    }
    if (threadIdx.x == 0) p.oscale[n] = 1.0f / scale;
#pragma unroll
    for (int c = 0; c < CHUNKS; c++) {
        const uint32_t k0 = ((uint32_t)c * kXprepThreads + threadIdx.x) * 8;
        if (k0 >= p.n_cols) break;  // whole groups of four threads (32 columns) leave together
        float sum = 0.f;
#pragma unroll
        for (int i = 0; i < 8; i++) {
            v[c][i] *= scale;
            sum += v[c][i];
        }
        // positions 0..7 of the 16 bytes hold columns 0,2,1,3,4,6,5,7
        const float o[8] = {v[c][0], v[c][2], v[c][1], v[c][3], v[c][4], v[c][6], v[c][5], v[c][7]};
        uint32_t h[4], l[4];
#pragma unroll
        for (int i = 0; i < 4; i++) {
            const __half2 hh = __floats2half2_rn(o[2 * i], o[2 * i + 1]);
            const float2 back = __half22float2(hh);
            h[i] = as_u32(hh);
            l[i] = as_u32(__floats2half2_rn(o[2 * i] - back.x, o[2 * i + 1] - back.y));
        }
        *reinterpret_cast<uint4 *>(slab16(k0, 0)) = make_uint4(h[0], h[1], h[2], h[3]);
        *reinterpret_cast<uint4 *>(slab16(k0, 1)) = make_uint4(l[0], l[1], l[2], l[3]);
        // four consecutive threads cover one 32-column sub-block
        sum += __shfl_xor_sync(0xffffffffu, sum, 1);
        sum += __shfl_xor_sync(0xffffffffu, sum, 2);
        if ((threadIdx.x & 3u) == 0) {
            sum *= kSumScale;  // 32 elements of up to 2^14 each: keep the sum inside fp16's range
            const __half sh = __float2half_rn(sum);
            *sum_slot(k0 >> 8, (k0 >> 5) & 7u, 0) = sh;
            *sum_slot(k0 >> 8, (k0 >> 5) & 7u, 1) = __float2half_rn(sum - __half2float(sh));
        }
    }
}

// 2-D view of a Q4_K matrix for the TMA engine: bytes along a row, rows; box = one super-block
// (144 bytes) of 128 rows.  Rows past the end read as zeros (a block of zeros dequantises to 0).
cudaError_t encode_weight_map(const uint8_t *w, uint32_t n_rows, uint32_t n_cols, CUtensorMap *out) {
    const uint64_t row_bytes = (uint64_t)(n_cols / 256) * 144;
    return cached_tensor_map_2d(w, 1, row_bytes, n_rows, row_bytes, 144, kBM, out);  // one driver call per (tensor, shape), not per launch
}

uint32_t pick_bn(uint32_t n_tokens) { return n_tokens <= 32 ? 32 : (n_tokens <= 64 ? 64 : 128); }

}  // namespace

// The same through a per-process cache: a map depends on the address and the shape only, and encoding one costs a
// driver call, which the matvec entry points would otherwise pay on every launch.
cudaError_t cached_tensor_map_2d(const void *base, uint32_t elem_bytes, uint64_t inner, uint64_t n_rows, uint64_t row_stride_bytes,
                                 uint32_t box_inner, uint32_t box_rows, void *out) {
    struct Key {
        const void *base;
        uint64_t inner, n_rows, stride;
        uint32_t elem, box_inner, box_rows;
        bool operator==(const Key &o) const {
            return base == o.base && inner == o.inner && n_rows == o.n_rows && stride == o.stride && elem == o.elem &&
                   box_inner == o.box_inner && box_rows == o.box_rows;
        }
    };
    struct Hash {
        size_t operator()(const Key &k) const {
            size_t h = std::hash<const void *>()(k.base);
            for (uint64_t v : {k.inner, k.n_rows, k.stride, (uint64_t)k.elem, (uint64_t)k.box_inner, (uint64_t)k.box_rows})
                h = h * 0x9E3779B97F4A7C15ull + std::hash<uint64_t>()(v);
            return h;
        }
    };
    static std::unordered_map<Key, CUtensorMap, Hash> cache;
    static std::mutex mu;
    const Key key{base, inner, n_rows, row_stride_bytes, elem_bytes, box_inner, box_rows};
    std::lock_guard<std::mutex> lock(mu);
    auto it = cache.find(key);
    if (it == cache.end()) {
        CUtensorMap m;
        cudaError_t e = encode_tensor_map_2d(base, elem_bytes, inner, n_rows, row_stride_bytes, box_inner, box_rows, &m);
        if (e != cudaSuccess) return e;
        if (cache.size() >= 16384) cache.clear();
        it = cache.emplace(key, m).first;
    }
    memcpy(out, &it->second, sizeof(CUtensorMap));
    return cudaSuccess;
}

// Tiled 2-D tensor map over rows of `elem_bytes`-sized elements (1 or 8): `inner` elements per row, `n_rows` rows
// `row_stride_bytes` apart (a multiple of 16; base 16-byte aligned), box of box_inner x box_rows elements, no
// swizzle, out-of-range elements read as zeros.  `out` is a CUtensorMap.
cudaError_t encode_tensor_map_2d(const void *base, uint32_t elem_bytes, uint64_t inner, uint64_t n_rows, uint64_t row_stride_bytes,
                                 uint32_t box_inner, uint32_t box_rows, void *out) {
    typedef CUresult (*EncodeFn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *, const cuuint64_t *,
                                 const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave, CUtensorMapSwizzle,
                                 CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
    static EncodeFn encode = nullptr;
    static std::mutex mu;
    {
        std::lock_guard<std::mutex> lock(mu);
        if (!encode) {
            void *fn = nullptr;
            cudaDriverEntryPointQueryResult qres;
            cudaError_t e = cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &qres);
            if (e != cudaSuccess) return e;
            if (qres != cudaDriverEntryPointSuccess || !fn) return cudaErrorNotSupported;
            encode = reinterpret_cast<EncodeFn>(fn);
        }
    }
    if (elem_bytes != 1 && elem_bytes != 8) return cudaErrorInvalidValue;
    const cuuint64_t dims[2] = {inner, n_rows};
    const cuuint64_t strides[1] = {row_stride_bytes};
    const cuuint32_t box[2] = {box_inner, box_rows};
    const cuuint32_t estr[2] = {1, 1};
    CUresult r = encode(static_cast<CUtensorMap *>(out), elem_bytes == 1 ? CU_TENSOR_MAP_DATA_TYPE_UINT8 : CU_TENSOR_MAP_DATA_TYPE_UINT64, 2,
                        const_cast<void *>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE,
                        CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r == CUDA_SUCCESS ? cudaSuccess : cudaErrorInvalidValue;
}

// Q4_K runs on the exact-integer kernel; Q6_K, Q8_0 and Q4_0 on the generic one (YULE_GEMM_GENERIC=1
// sends Q4_K there too, for comparison).  The activation tiles are laid out per 256 columns.
bool qgemm_supported(uint32_t type, uint32_t n_cols, uint32_t n_tokens) {
    return is_quantized(type) && n_cols % 256 == 0 && n_cols > 0 && n_cols <= 65536 && n_tokens >= 1;
}

size_t qgemm_scratch_bytes(uint32_t n_tokens, uint32_t n_cols) {
    const uint32_t bn = pick_bn(n_tokens);
    const size_t padded = (size_t)((n_tokens + bn - 1) / bn) * bn;
    return kGemmSplitBytes + padded * n_cols * 4 + padded * (n_cols / 256) * 32 + padded * sizeof(float) + 512;
}

cudaError_t launch_qgemm_xprep(const QGemm &g, cudaStream_t s, uint64_t *launches) {
    if (!qgemm_supported(g.type, g.n_cols, g.n_tokens)) return cudaErrorInvalidValue;
    const uint32_t bn = pick_bn(g.n_tokens);
    const uint32_t n_ntiles = (g.n_tokens + bn - 1) / bn, padded = n_ntiles * bn;
    unsigned char *xb = reinterpret_cast<unsigned char *>(g.scratch) + kGemmSplitBytes;
    const size_t tiles_bytes = (size_t)padded * g.n_cols * 4 + (size_t)padded * (g.n_cols / 256) * 32;
    float *oscale = reinterpret_cast<float *>(xb + ((tiles_bytes + 255) & ~(size_t)255));

    XprepParams xp = {};
    xp.x = g.x;
    xp.gate = g.gate;
    xp.norm_w = g.norm_w;
    xp.eps = g.eps;
    xp.x_stride = g.x_stride;
    xp.n_tokens = g.n_tokens;
    xp.n_cols = g.n_cols;
    xp.bn = bn;
    xp.xb = xb;
    xp.oscale = oscale;
    cudaError_t e;
    if (g.n_cols <= 8192)
        e = launch_kernel(gemm_xprep_kernel<1>, dim3(padded), dim3(kXprepThreads), 0, s, g.pdl, xp);
    else if (g.n_cols <= 16384)
        e = launch_kernel(gemm_xprep_kernel<2>, dim3(padded), dim3(kXprepThreads), 0, s, g.pdl, xp);
    else if (g.n_cols <= 32768)
        e = launch_kernel(gemm_xprep_kernel<4>, dim3(padded), dim3(kXprepThreads), 0, s, g.pdl, xp);
    else if (g.n_cols <= 65536)
        e = launch_kernel(gemm_xprep_kernel<8>, dim3(padded), dim3(kXprepThreads), 0, s, g.pdl, xp);
    else
        return cudaErrorInvalidValue;
    if (e != cudaSuccess) return e;
    *launches += 1;
    return cudaSuccess;
}

cudaError_t launch_qgemm_mm(const QGemm &g, int sm_count, cudaStream_t s, uint64_t *launches) {
    if (!qgemm_supported(g.type, g.n_cols, g.n_tokens) || g.n_rows == 0) return cudaErrorInvalidValue;
    if (g.n_more > (uint32_t)kGemmSegs - 1 || (g.n_more && g.residual)) return cudaErrorInvalidValue;
    const uint32_t bn = pick_bn(g.n_tokens);
    const uint32_t n_ntiles = (g.n_tokens + bn - 1) / bn, padded = n_ntiles * bn;
    unsigned char *xb = reinterpret_cast<unsigned char *>(g.scratch) + kGemmSplitBytes;
    const size_t tiles_bytes = (size_t)padded * g.n_cols * 4 + (size_t)padded * (g.n_cols / 256) * 32;
    float *oscale = reinterpret_cast<float *>(xb + ((tiles_bytes + 255) & ~(size_t)255));
    cudaError_t e;
    GemmParams p = {};
    p.xb = reinterpret_cast<const __half *>(xb);
    p.oscale = oscale;
    p.residual = g.residual;
    p.n_cols = g.n_cols;
    p.n_tokens = g.n_tokens;
    p.bn = bn;
    p.n_seg = 1 + g.n_more;
    for (uint32_t i = 0; i < p.n_seg; i++) {
        p.w[i] = i ? g.w_more[i - 1] : g.w;
        p.out[i] = i ? g.out_more[i - 1] : g.out;
        p.n_rows[i] = i ? g.n_rows_more[i - 1] : g.n_rows;
        p.out_stride[i] = i ? g.out_stride_more[i - 1] : g.out_stride;
        if (!p.w[i] || !p.out[i] || p.n_rows[i] == 0) return cudaErrorInvalidValue;
        p.mt0[i + 1] = p.mt0[i] + (p.n_rows[i] + kBM - 1) / kBM;
    }
    for (uint32_t i = p.n_seg; i < (uint32_t)kGemmSegs; i++) p.mt0[i + 1] = p.mt0[p.n_seg];
    p.n_mtiles = p.mt0[p.n_seg];
    p.n_ntiles = n_ntiles;
    // Few tiles and long rows: the columns of a tile are split over several CTAs (whole super-blocks, at least four
    // per part), whose partial results the last one to finish adds up in a fixed order.
    p.ksplit = 1;
    p.sb_per = g.n_cols / 256;
    {
        const uint32_t base = p.n_mtiles * p.n_ntiles, bpr = g.n_cols / 256;
        uint32_t want = 1;
        if (base * 2 <= (uint32_t)sm_count && bpr >= 8) {
            want = (uint32_t)sm_count / base;
            if (want > bpr / 4) want = bpr / 4;
            if (want > 16) want = 16;
        }
        if (const char *k = knob("YULE_GEMM_KSPLIT")) want = (uint32_t)atoi(k) > 0 ? (uint32_t)atoi(k) : want;
        if (want > bpr) want = bpr;
        while (want > 1 && base * want > kGemmSplitMaxItems) want--;
        if (want > 1) {
            p.sb_per = (bpr + want - 1) / want;
            p.ksplit = (bpr + p.sb_per - 1) / p.sb_per;
        }
        p.split_tickets = reinterpret_cast<uint32_t *>(g.scratch);
        p.split_part = reinterpret_cast<float *>(reinterpret_cast<unsigned char *>(g.scratch) + kGemmTicketBytes);
    }
    const bool generic = g.type != YULE_DTYPE_Q4_K || (knob("YULE_GEMM_GENERIC") && atoi(knob("YULE_GEMM_GENERIC")));
    const uint32_t kg = groups_per_stage(bn, generic);
    const uint32_t stage_bytes = generic ? 2 * kABytes + 2 * bn * kBK * 2 : kg * kABytes + kAmBytes + kg * 2 * bn * kBK * 2 + bn * 32;
    p.unit_bytes = 256 / block_size(g.type) * block_bytes(g.type);
    p.raw_chunks = (p.unit_bytes + 14 + 15) / 16;      // covers the unit from any 2-byte-aligned start
    p.raw_stride = (p.raw_chunks | 1u) * 16;            // an odd multiple of 16 bytes
    p.raw_ring_bytes = (2 * kBM * p.raw_stride + 127u) & ~127u;
    const size_t raw_ring = generic ? p.raw_ring_bytes : (size_t)raw_slots_for(bn) * kRawBytes;
    uint32_t stages = (uint32_t)((220u * 1024u - (raw_ring + 512u)) / stage_bytes);
    if (stages < 2) return cudaErrorInvalidValue;
    p.stages = stages > (uint32_t)kMaxStages ? (uint32_t)kMaxStages : stages;
    p.type = g.type;
    p.w_row_bytes = (uint64_t)(g.n_cols / block_size(g.type)) * block_bytes(g.type);
    p.out_scale = generic ? 1.0f / kGenericWScale : 1.0f;
    p.status = g.status;
    p.prof = (kProfile && knob("YULE_GEMM_PROF")) ? 1u : 0u;
    p.skip = (kProfile && knob("YULE_GEMM_SKIP")) ? (uint32_t)atoi(knob("YULE_GEMM_SKIP")) : 0u;
    const size_t tail_bytes = raw_ring + (2 * kMaxStages + 8 + 2 * kRawSlots) * 8 + 32;
    const size_t smem = (size_t)p.stages * stage_bytes + tail_bytes;
    GemmMaps w_maps;
    memset(&w_maps, 0, sizeof(w_maps));
    if (!generic) {
        for (uint32_t i = 0; i < p.n_seg; i++) {
            e = encode_weight_map(p.w[i], p.n_rows[i], g.n_cols, &w_maps.m[i]);
            if (e != cudaSuccess) return e;
        }
    }
    uint32_t grid = p.n_mtiles * p.n_ntiles * p.ksplit;
    if (grid > (uint32_t)sm_count) grid = (uint32_t)sm_count;
    auto launch = [&](auto kern) {
        cudaError_t e2 = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, 222 * 1024);
        if (e2 != cudaSuccess) return e2;
        return launch_kernel(kern, dim3(grid), dim3(kGemmThreads), smem, s, g.pdl, p, w_maps);
    };
    if (generic)
        e = bn == 32 ? launch(qgemm_tc_kernel<32, true>) : (bn == 64 ? launch(qgemm_tc_kernel<64, true>) : launch(qgemm_tc_kernel<128, true>));
    else
        e = bn == 32 ? launch(qgemm_tc_kernel<32, false>) : (bn == 64 ? launch(qgemm_tc_kernel<64, false>) : launch(qgemm_tc_kernel<128, false>));
    if (e != cudaSuccess) return e;
    *launches += 1;
    if (p.prof) {
        cudaStreamCaptureStatus cs = cudaStreamCaptureStatusNone;
        cudaStreamIsCapturing(s, &cs);
        if (cs == cudaStreamCaptureStatusNone && cudaStreamSynchronize(s) == cudaSuccess) {
            long long h[16];
            if (cudaMemcpyFromSymbol(h, g_gemm_prof, sizeof(h)) == cudaSuccess)
                fprintf(stderr,
                        "[qgemm prof, CTA 0, cycles] mma: total %lld wait_acc_empty %lld wait_full %lld issue %lld commit %lld stages %lld | "
                        "producer: total %lld wait_empty %lld unpack %lld fence+arrive %lld | drain: total %lld wait_acc_full %lld | "
                        "set-up %lld wait for the re-layout %lld epilogue %lld kernel %lld\n",
                        h[0], h[1], h[2], h[3], h[4], h[5], h[6], h[7], h[8], h[9], h[10], h[11], h[12], h[13], h[14], h[15]);
        }
    }
    return cudaSuccess;
}

cudaError_t launch_qgemm(const QGemm &g, int sm_count, cudaStream_t s, uint64_t *launches) {
    if (g.n_rows == 0) return cudaErrorInvalidValue;
    cudaError_t e = launch_qgemm_xprep(g, s, launches);
    if (e != cudaSuccess) return e;
    QGemm mm = g;
    mm.pdl = true;  // behind the re-layout of its own activations: only the weight copies run ahead of it
    return launch_qgemm_mm(mm, sm_count, s, launches);
}

}  // namespace yule
