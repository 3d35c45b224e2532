// Quantised GEMM on the 5th-generation tensor cores (tcgen05, accumulators in TMEM):
//
//     out[n][r] = Σ_k W[r][k] · x[n][k]        W: Q4_K blocks, x: N ≥ 8 fp32 activation rows
//
// This is the prefill / batched-decode counterpart of the matvec kernels: the weights cross HBM
// once per pass over up to 128 activation rows instead of once per four.  The reference runs
// prefill as one matvec chain per token (yule-infer/src/gpu_runner.rs:146-160); the arithmetic
// contract is the same fp32 dot product.
//
// Precision.  tcgen05 has no fp32 operand type, so both operands are split into two fp16 terms,
// v = hi + lo with hi = fp16(v) and lo = fp16(v − hi) (22 significant bits), and three products
// are accumulated in fp32: W_hi·x_hi + W_hi·x_lo + W_lo·x_hi (the lo·lo term is below 2⁻²² of the
// result).  Weights are scaled by 2¹⁰ and every activation row by a power of two that puts its
// largest element in [2¹³, 2¹⁴), so that the lo terms stay in fp16's normal range; the epilogue
// multiplies the exact inverse back in.
//
// The tensor core adds into its fp32 accumulator with truncation, a bias that grows with the length
// of the accumulation chain.  So a TMEM accumulator only ever holds one 64-column stage (12 MMAs);
// the epilogue warps drain it after every stage and keep the running sums in registers, added with
// ordinary round-to-nearest fp32.
//
// One CTA per SM, 18 warps, persistent over (row tile, activation tile) pairs:
//   warps 0-7   drain warps: tcgen05.ld of their 32 TMEM lanes × half of the columns after every
//               stage, running sums in registers; at the end of a tile scale, residual, store
//   warp  8     one thread: bulk copies (TMA engine) of the pre-arranged activation tiles
//   warp  9     one thread: tcgen05.mma issue; the warp also owns the TMEM allocation
//   warps 10-17 dequantise Q4_K → fp16 hi/lo straight into the shared-memory operand layout,
//               with the blocks of the next two super-blocks already on their way from HBM
// A stage is a 128-row × 64-column slab of W (hi and lo, 32 KB) plus the matching slab of x.
// Operands use the no-swizzle K-major core-matrix layout: 8 rows × 16 bytes per core matrix,
// core matrices of one 8-column step contiguous along the rows.
//
// Every wait is bounded: a pipeline that stops making progress sets the context's status word,
// raises the CTA's abort flag, lets all roles fall through to the common exit and frees its TMEM.

#include <cuda_fp16.h>

#include "internal.h"

namespace yule {
namespace {

constexpr int kBM = 128;  // rows of W per tile = TMEM lanes
constexpr int kBK = 64;   // columns per stage (a quarter of a super-block)
constexpr int kEpiWarps = 8, kProdWarps = 8;
constexpr int kLoaderWarp = kEpiWarps, kMmaWarp = kEpiWarps + 1, kFirstProdWarp = kEpiWarps + 2;
constexpr int kGemmThreads = (kEpiWarps + 2 + kProdWarps) * 32;  // 576
constexpr int kMaxStages = 6;
constexpr uint32_t kAHalfBytes = kBM * kBK * 2;  // one fp16 term of the W slab: 16 KB
constexpr float kWScale = 1024.f;
constexpr long long kWaitCycles = 2000000000LL;  // ~1 s: far beyond any real stall
constexpr int kStatusGemmTimeout = 3;

struct GemmParams {
    const uint8_t *w;      // Q4_K blocks, row-major
    const __half *xb;      // activation tiles written by gemm_xprep_kernel
    const float *oscale;   // per (padded) activation row: 1 / (row scale · kWScale)
    float *out;            // [n_tokens][out_stride]
    const float *residual; // added to out (same layout) or null
    uint32_t n_rows, n_cols, n_tokens, out_stride;
    uint32_t bn;           // activation rows per tile: 32, 64 or 128
    uint32_t n_mtiles, n_ntiles, stages;
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
// The mbarrier gets one arrival when every MMA issued so far by this thread has completed.
__device__ __forceinline__ void umma_commit(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}

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

// 6-bit scale and min of sub-block j from the 12 packed bytes (yule-core/src/dequant.rs:165-176).
__device__ __forceinline__ void q4k_scale_min(uint32_t s0, uint32_t s1, uint32_t s2, uint32_t j, uint32_t *sc, uint32_t *mn) {
    auto byte_of = [&](uint32_t i) {
        const uint32_t w = i < 4 ? s0 : (i < 8 ? s1 : s2);
        return (w >> (8 * (i & 3))) & 0xFFu;
    };
    if (j < 4) {
        *sc = byte_of(j) & 63u;
        *mn = byte_of(j + 4) & 63u;
    } else {
        *sc = (byte_of(j + 4) & 0xFu) | ((byte_of(j - 4) >> 6) << 4);
        *mn = (byte_of(j + 4) >> 4) | ((byte_of(j) >> 6) << 4);
    }
}

// Eight weights q·ds − dm (q = the low nibble of each byte of w0, w1) as fp16 hi and lo terms.
__device__ __forceinline__ void dequant8(uint32_t w0, uint32_t w1, float ds, float dm, uint4 *hi, uint4 *lo) {
    float v[8];
#pragma unroll
    for (int b = 0; b < 4; b++) {
        // 0x4B000000 | q is the float 2²³ + q: the subtraction is exact
        v[b] = fmaf(__uint_as_float(__byte_perm(w0, 0x4B000000u, 0x7440 + b)) - 8388608.f, ds, -dm);
        v[4 + b] = fmaf(__uint_as_float(__byte_perm(w1, 0x4B000000u, 0x7440 + b)) - 8388608.f, ds, -dm);
    }
    uint32_t h[4], l[4];
#pragma unroll
    for (int i = 0; i < 4; i++) {
        const __half2 hh = __floats2half2_rn(v[2 * i], v[2 * i + 1]);
        const float2 back = __half22float2(hh);
        const __half2 ll = __floats2half2_rn(v[2 * i] - back.x, v[2 * i + 1] - back.y);
        h[i] = *reinterpret_cast<const uint32_t *>(&hh);
        l[i] = *reinterpret_cast<const uint32_t *>(&ll);
    }
    *hi = make_uint4(h[0], h[1], h[2], h[3]);
    *lo = make_uint4(l[0], l[1], l[2], l[3]);
}

// One row's share of a super-block: the 16-byte header (d, dmin, packed scales) and this thread's
// 16 of the 32 quant bytes of each of the four 64-column groups.
struct RowBlock {
    uint4 hdr;
    uint4 q[4];
};

template <int BN>
__global__ void __launch_bounds__(kGemmThreads, 1) qgemm_q4k_tc_kernel(const GemmParams p) {
    constexpr uint32_t NBUF = BN <= 64 ? 4 : 2;            // TMEM accumulators in flight
    constexpr uint32_t kTmemCols = NBUF * BN;              // 128 or 256: a power of two ≥ 32
    constexpr uint32_t CW = BN / 2;                        // columns per drain warp
    constexpr uint32_t kXHalfBytes = BN * kBK * 2;         // one fp16 term of the activation slab
    constexpr uint32_t kStageBytes = 2 * kAHalfBytes + 2 * kXHalfBytes;
    extern __shared__ __align__(128) unsigned char smem[];
    yule_pdl_launch_dependents();
    const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    unsigned char *tail = smem + (size_t)p.stages * kStageBytes;
    uint64_t *bars = reinterpret_cast<uint64_t *>(tail);     // full[6] empty[6] acc_full[4] acc_empty[4]
    const uint32_t bar_full = smem_u32(bars), bar_empty = bar_full + 8 * kMaxStages;
    const uint32_t bar_acc_full = bar_empty + 8 * kMaxStages, bar_acc_empty = bar_acc_full + 32;
    uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(bars + 2 * kMaxStages + 8);
    volatile int *abort_flag = reinterpret_cast<volatile int *>(tmem_slot + 1);

    if (threadIdx.x == 0) {
        for (uint32_t s = 0; s < p.stages; s++) {
            mbar_init(bar_full + 8 * s, kProdWarps + 1);  // one arrival per producer warp + the loader's expect_tx
            mbar_init(bar_empty + 8 * s, 1);              // tcgen05.commit
        }
        for (uint32_t b = 0; b < NBUF; b++) {
            mbar_init(bar_acc_full + 8 * b, 1);
            mbar_init(bar_acc_empty + 8 * b, kEpiWarps);
        }
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        fence_async_smem();
    }
    if (warp == kMmaWarp) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(kTmemCols)
                     : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    const uint32_t n_tiles = p.n_mtiles * p.n_ntiles;
    const uint32_t n_kb = p.n_cols / kBK;
    const uint32_t bpr = p.n_cols / 256;  // super-blocks per row

    if (warp == kLoaderWarp) {
        if (lane == 0) {
            yule_pdl_wait();  // the activation tiles come from the kernel before this one
            uint32_t it = 0;
            bool ok = true;
            for (uint32_t tile = blockIdx.x; tile < n_tiles && ok; tile += gridDim.x) {
                const uint32_t nt = tile % p.n_ntiles;
                const unsigned char *src = reinterpret_cast<const unsigned char *>(p.xb) + (size_t)nt * n_kb * 2 * kXHalfBytes;
                for (uint32_t kb = 0; kb < n_kb; kb++, it++) {
                    const uint32_t s = it % p.stages, ph = (it / p.stages) & 1u;
                    if (!mbar_wait(bar_empty + 8 * s, ph ^ 1u, abort_flag, p.status)) {
                        ok = false;
                        break;
                    }
                    const uint32_t dst = smem_u32(smem + (size_t)s * kStageBytes + 2 * kAHalfBytes);
                    mbar_arrive_expect_tx(bar_full + 8 * s, 2 * kXHalfBytes);
                    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(dst),
                                 "l"(src + (size_t)kb * 2 * kXHalfBytes), "r"(2 * kXHalfBytes), "r"(bar_full + 8 * s)
                                 : "memory");
                }
            }
        }
    } else if (warp == kMmaWarp) {
        if (lane == 0) {
            // fp16 × fp16 → fp32, both operands K-major, M = 128, N = BN
            constexpr uint32_t idesc = (1u << 4) | ((uint32_t)(BN >> 3) << 17) | ((uint32_t)(kBM >> 4) << 24);
            constexpr uint32_t x_lbo = BN * 16;  // bytes of one 8-column step of the activation slab
            uint32_t it = 0;
            bool ok = true;
            for (uint32_t tile = blockIdx.x; tile < n_tiles && ok; tile += gridDim.x) {
                for (uint32_t kb = 0; kb < n_kb; kb++, it++) {
                    const uint32_t s = it % p.stages, ph = (it / p.stages) & 1u;
                    const uint32_t buf = it % NBUF, aph = (it / NBUF) & 1u;
                    if (!mbar_wait(bar_acc_empty + 8 * buf, aph ^ 1u, abort_flag, p.status) ||
                        !mbar_wait(bar_full + 8 * s, ph, abort_flag, p.status)) {
                        ok = false;
                        break;
                    }
                    tc_fence_after();
                    const uint32_t d_tmem = tmem_base + buf * BN;
                    const uint32_t a_hi = smem_u32(smem + (size_t)s * kStageBytes), a_lo = a_hi + kAHalfBytes;
                    const uint32_t x_hi = a_lo + kAHalfBytes, x_lo = x_hi + kXHalfBytes;
#pragma unroll
                    for (uint32_t k16 = 0; k16 < kBK / 16; k16++) {
                        const uint64_t da_hi = smem_desc(a_hi + k16 * 4096, 2048, 128), da_lo = smem_desc(a_lo + k16 * 4096, 2048, 128);
                        const uint64_t dx_hi = smem_desc(x_hi + k16 * 2 * x_lbo, x_lbo, 128), dx_lo = smem_desc(x_lo + k16 * 2 * x_lbo, x_lbo, 128);
                        umma_f16(d_tmem, da_hi, dx_hi, idesc, k16 != 0u);  // every stage starts a fresh accumulator
                        umma_f16(d_tmem, da_hi, dx_lo, idesc, 1u);
                        umma_f16(d_tmem, da_lo, dx_hi, idesc, 1u);
                    }
                    umma_commit(bar_empty + 8 * s);       // the slabs may be overwritten once these MMAs are done
                    umma_commit(bar_acc_full + 8 * buf);  // and the accumulator may be drained
                }
            }
        }
    } else if (warp >= kFirstProdWarp) {
        const uint32_t ptid = threadIdx.x - kFirstProdWarp * 32;  // 0..255
        const uint32_t r = ptid & 127u, hf = ptid >> 7;           // row of the tile, which 16 bytes of the 32
        const uint32_t my_tiles = n_tiles > blockIdx.x ? (n_tiles - blockIdx.x + gridDim.x - 1) / gridDim.x : 0;
        const uint32_t n_units = my_tiles * bpr;  // (tile, super-block) pairs of this CTA, in order
        auto load_block = [&](uint32_t u, RowBlock &b) {
            if (u >= n_units) return;
            const uint32_t tile = blockIdx.x + (u / bpr) * gridDim.x, sb = u % bpr;
            uint32_t row = (tile / p.n_ntiles) * kBM + r;
            row = row < p.n_rows ? row : p.n_rows - 1;  // clamp: stays in bounds, the result is dropped
            const uint8_t *bp = p.w + ((size_t)row * bpr + sb) * 144;
            b.hdr = __ldg(reinterpret_cast<const uint4 *>(bp));
#pragma unroll
            for (int g = 0; g < 4; g++) b.q[g] = __ldg(reinterpret_cast<const uint4 *>(bp + 16 + g * 32 + hf * 16));
        };
        RowBlock cur, nxt, nxt2;
        load_block(0, cur);
        load_block(1, nxt);
        uint32_t it = 0;
        bool ok = true;
        const uint32_t in_core = (r >> 3) * 128 + (r & 7u) * 16;
        for (uint32_t u = 0; u < n_units && ok; u++) {
            load_block(u + 2, nxt2);
            const float2 dd = __half22float2(*reinterpret_cast<const __half2 *>(&cur.hdr.x));
#pragma unroll
            for (uint32_t g = 0; g < 4; g++, it++) {
                const uint32_t s = it % p.stages, ph = (it / p.stages) & 1u;
                uint32_t sc0, mn0, sc1, mn1;
                q4k_scale_min(cur.hdr.y, cur.hdr.z, cur.hdr.w, 2 * g, &sc0, &mn0);
                q4k_scale_min(cur.hdr.y, cur.hdr.z, cur.hdr.w, 2 * g + 1, &sc1, &mn1);
                const float ds0 = dd.x * (float)sc0 * kWScale, dm0 = dd.y * (float)mn0 * kWScale;
                const float ds1 = dd.x * (float)sc1 * kWScale, dm1 = dd.y * (float)mn1 * kWScale;
                if (!mbar_wait(bar_empty + 8 * s, ph ^ 1u, abort_flag, p.status)) {
                    ok = false;
                    break;
                }
                unsigned char *a_hi = smem + (size_t)s * kStageBytes, *a_lo = a_hi + kAHalfBytes;
                // byte b of the 32 holds column b (low nibble, sub-block 2g) and column 32 + b (high nibble)
                const uint32_t qw[4] = {cur.q[g].x, cur.q[g].y, cur.q[g].z, cur.q[g].w};
#pragma unroll
                for (int half8 = 0; half8 < 2; half8++) {
                    const uint32_t w0 = qw[2 * half8], w1 = qw[2 * half8 + 1];
                    uint4 hi, lo;
                    const uint32_t kc_lo = hf * 2 + half8;  // 8-column step of the low-nibble columns
                    dequant8(w0 & 0x0F0F0F0Fu, w1 & 0x0F0F0F0Fu, ds0, dm0, &hi, &lo);
                    *reinterpret_cast<uint4 *>(a_hi + kc_lo * 2048 + in_core) = hi;
                    *reinterpret_cast<uint4 *>(a_lo + kc_lo * 2048 + in_core) = lo;
                    dequant8((w0 >> 4) & 0x0F0F0F0Fu, (w1 >> 4) & 0x0F0F0F0Fu, ds1, dm1, &hi, &lo);
                    *reinterpret_cast<uint4 *>(a_hi + (4 + kc_lo) * 2048 + in_core) = hi;
                    *reinterpret_cast<uint4 *>(a_lo + (4 + kc_lo) * 2048 + in_core) = lo;
                }
                fence_async_smem();  // generic-proxy stores → visible to the tensor core's reads
                __syncwarp();
                if (lane == 0) mbar_arrive(bar_full + 8 * s);
            }
            cur = nxt;
            nxt = nxt2;
        }
    } else {
        // drain warp: TMEM lanes [32·(warp % 4), +32) = rows of the tile, columns [CW·(warp / 4), +CW)
        yule_pdl_wait();
        const uint32_t lane_base = (warp & 3u) * 32u, col_base = (warp >> 2) * CW;
        uint32_t it = 0;
        bool ok = true;
        for (uint32_t tile = blockIdx.x; tile < n_tiles && ok; tile += gridDim.x) {
            const uint32_t mt = tile / p.n_ntiles, nt = tile % p.n_ntiles;
            float acc[CW];
#pragma unroll
            for (uint32_t j = 0; j < CW; j++) acc[j] = 0.f;
            for (uint32_t kb = 0; kb < n_kb; kb++, it++) {
                const uint32_t buf = it % NBUF, aph = (it / NBUF) & 1u;
                if (!mbar_wait(bar_acc_full + 8 * buf, aph, abort_flag, p.status)) {
                    ok = false;
                    break;
                }
                tc_fence_after();
#pragma unroll
                for (uint32_t c0 = 0; c0 < CW; c0 += 16) {
                    uint32_t v[16];
                    tmem_ld16(tmem_base + (lane_base << 16) + buf * BN + col_base + c0, v);
#pragma unroll
                    for (int j = 0; j < 16; j++) acc[c0 + j] += __uint_as_float(v[j]);
                }
                tc_fence_before();
                __syncwarp();
                if (lane == 0) mbar_arrive(bar_acc_empty + 8 * buf);
            }
            if (!ok) break;
            const uint32_t row = mt * kBM + lane_base + lane;
            const uint32_t n0 = nt * BN + col_base;
#pragma unroll
            for (uint32_t c0 = 0; c0 < CW; c0 += 16) {
                const float osc = lane < 16 ? p.oscale[n0 + c0 + lane] : 0.f;  // padded to whole tiles
#pragma unroll
                for (int j = 0; j < 16; j++) {
                    const float sc = __shfl_sync(0xffffffffu, osc, j);
                    const uint32_t n = n0 + c0 + j;
                    if (row < p.n_rows && n < p.n_tokens) {
                        float val = acc[c0 + j] * sc;
                        const size_t o = (size_t)n * p.out_stride + row;
                        if (p.residual) val += p.residual[o];
                        p.out[o] = val;
                    }
                }
            }
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
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(kTmemCols) : "memory");
    }
}

// Activation rows → fp16 hi/lo tiles in the operand layout of the GEMM, one CTA per (padded) row.
// Optional prologues: RMSNorm (out = x · inv · w as in yule-infer/src/model_runner.rs:254-263) or
// SwiGLU (silu(gate) · x, kernels/cuda/silu_mul.cu:3-14).
struct XprepParams {
    const float *x;
    const float *gate;    // when set: y = silu(gate) · x
    const float *norm_w;  // when set: y = x · inv_rms · norm_w
    float eps;
    uint32_t x_stride, n_tokens, n_cols, bn;
    __half *xb;
    float *oscale;
};

__global__ void __launch_bounds__(256) gemm_xprep_kernel(const XprepParams p) {
    yule_pdl_launch_dependents();
    yule_pdl_wait();
    __shared__ float red[32];
    const uint32_t n = blockIdx.x, nt = n / p.bn, r = n % p.bn;
    const uint32_t n_kb = p.n_cols / kBK;
    const size_t half_elems = (size_t)p.bn * kBK;  // halves per fp16 term of one slab
    auto slab = [&](uint32_t kb, uint32_t term) { return p.xb + ((size_t)(nt * n_kb + kb) * 2 + term) * half_elems; };
    auto in_slab = [&](uint32_t kk) { return ((kk >> 3) * (p.bn / 8) + (r >> 3)) * 64 + (r & 7u) * 8; };
    if (n >= p.n_tokens) {  // padding row of the last tile
        for (uint32_t k0 = threadIdx.x * 8; k0 < p.n_cols; k0 += 256 * 8) {
            const uint32_t kb = k0 / kBK, off = in_slab(k0 % kBK);
            *reinterpret_cast<uint4 *>(slab(kb, 0) + off) = make_uint4(0, 0, 0, 0);
            *reinterpret_cast<uint4 *>(slab(kb, 1) + off) = make_uint4(0, 0, 0, 0);
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
        for (int i = 1; i < 8; i++) v = is_max ? fmaxf(v, red[i]) : v + red[i];
        return v;
    };
    float inv = 1.f;
    if (p.norm_w) {
        float ss = 0.f;
        for (uint32_t i = threadIdx.x; i < p.n_cols; i += 256) ss = fmaf(x[i], x[i], ss);
        ss = block_reduce(ss, false);
        inv = 1.0f / sqrtf(ss / (float)p.n_cols + p.eps);
    }
    auto value = [&](uint32_t i) {
        float v = x[i];
        if (p.norm_w) v = v * inv * p.norm_w[i];
        if (gate) {
            const float gt = gate[i];
            v = (gt / (1.0f + expf(-gt))) * v;
        }
        return v;
    };
    float amax = 0.f;
    for (uint32_t i = threadIdx.x; i < p.n_cols; i += 256) amax = fmaxf(amax, fabsf(value(i)));
    amax = block_reduce(amax, true);
    // power of two that puts the largest element in [2^13, 2^14)
    float scale = 1.f;
    if (amax > 1e-30f && amax < 1e30f) {
        int ex;
        frexpf(amax, &ex);  // amax = m · 2^ex, m in [0.5, 1)
        scale = ldexpf(1.f, 14 - ex);
    }
    if (threadIdx.x == 0) p.oscale[n] = (1.0f / scale) / kWScale;
    for (uint32_t k0 = threadIdx.x * 8; k0 < p.n_cols; k0 += 256 * 8) {
        uint32_t h[4], l[4];
#pragma unroll
        for (int i = 0; i < 4; i++) {
            const float v0 = value(k0 + 2 * i) * scale, v1 = value(k0 + 2 * i + 1) * scale;
            const __half2 hh = __floats2half2_rn(v0, v1);
            const float2 back = __half22float2(hh);
            const __half2 ll = __floats2half2_rn(v0 - back.x, v1 - back.y);
            h[i] = *reinterpret_cast<const uint32_t *>(&hh);
            l[i] = *reinterpret_cast<const uint32_t *>(&ll);
        }
        const uint32_t kb = k0 / kBK, off = in_slab(k0 % kBK);
        *reinterpret_cast<uint4 *>(slab(kb, 0) + off) = make_uint4(h[0], h[1], h[2], h[3]);
        *reinterpret_cast<uint4 *>(slab(kb, 1) + off) = make_uint4(l[0], l[1], l[2], l[3]);
    }
}

uint32_t pick_bn(uint32_t n_tokens) { return n_tokens <= 32 ? 32 : (n_tokens <= 64 ? 64 : 128); }

}  // namespace

bool qgemm_supported(uint32_t type, uint32_t n_cols, uint32_t n_tokens) {
    return type == YULE_DTYPE_Q4_K && n_cols % 256 == 0 && n_cols > 0 && n_tokens >= 1;
}

size_t qgemm_scratch_bytes(uint32_t n_tokens, uint32_t n_cols) {
    const uint32_t bn = pick_bn(n_tokens);
    const size_t padded = (size_t)((n_tokens + bn - 1) / bn) * bn;
    return padded * n_cols * 4 + padded * sizeof(float) + 256;
}

cudaError_t launch_qgemm(const QGemm &g, int sm_count, cudaStream_t s, uint64_t *launches) {
    if (!qgemm_supported(g.type, g.n_cols, g.n_tokens) || g.n_rows == 0) return cudaErrorInvalidValue;
    const uint32_t bn = pick_bn(g.n_tokens);
    const uint32_t n_ntiles = (g.n_tokens + bn - 1) / bn, padded = n_ntiles * bn;
    __half *xb = reinterpret_cast<__half *>(g.scratch);
    float *oscale = reinterpret_cast<float *>(reinterpret_cast<unsigned char *>(g.scratch) + (((size_t)padded * g.n_cols * 4 + 255) & ~(size_t)255));

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
    cudaError_t e = launch_kernel(gemm_xprep_kernel, dim3(padded), dim3(256), 0, s, g.pdl, xp);
    if (e != cudaSuccess) return e;
    *launches += 1;

    GemmParams p = {};
    p.w = g.w;
    p.xb = xb;
    p.oscale = oscale;
    p.out = g.out;
    p.residual = g.residual;
    p.n_rows = g.n_rows;
    p.n_cols = g.n_cols;
    p.n_tokens = g.n_tokens;
    p.out_stride = g.out_stride;
    p.bn = bn;
    p.n_mtiles = (g.n_rows + kBM - 1) / kBM;
    p.n_ntiles = n_ntiles;
    const uint32_t stage_bytes = 2 * kAHalfBytes + 2 * bn * kBK * 2;
    uint32_t stages = (200u * 1024u) / stage_bytes;
    p.stages = stages > (uint32_t)kMaxStages ? (uint32_t)kMaxStages : stages;
    p.status = g.status;
    const size_t smem = (size_t)p.stages * stage_bytes + (2 * kMaxStages + 8) * 8 + 16;
    uint32_t grid = p.n_mtiles * p.n_ntiles;
    if (grid > (uint32_t)sm_count) grid = (uint32_t)sm_count;
    auto launch = [&](auto kern) {
        cudaError_t e2 = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, 210 * 1024);
        if (e2 != cudaSuccess) return e2;
        return launch_kernel(kern, dim3(grid), dim3(kGemmThreads), smem, s, g.pdl, p);
    };
    e = bn == 32 ? launch(qgemm_q4k_tc_kernel<32>) : (bn == 64 ? launch(qgemm_q4k_tc_kernel<64>) : launch(qgemm_q4k_tc_kernel<128>));
    if (e != cudaSuccess) return e;
    *launches += 1;
    return cudaSuccess;
}

}  // namespace yule
