// qmv_q8q4_ring.cu — Q8_0 and Q4_0 fused dequantise + matvec on the tensor pipe, raw blocks staged through a
// shared-memory ring by tiled TMA copies: a kernel for one activation vector and one for two to four per pass.
//
// Contract: yule-core/src/dequant.rs:902-926 — per 32-weight block, sum += d · Σ q·x with q the signed byte
// (Q8_0) or nibble − 8 (Q4_0, byte j of a block holding weights 2j in its low and 2j+1 in its high nibble).
//
// The blocks are 34 and 18 bytes long and only 2-byte aligned in the GGUF stream, which rules out wide global
// loads.  A row, however, is 16-byte aligned whenever n_cols is a multiple of 256 (8 blocks = 272 or 144 bytes),
// and so is every run of eight 128-column groups of it: 16 rows of such runs go HBM → shared memory as one tiled
// copy (cp.async.bulk.tensor.2d + mbarrier, issued before `griddepcontrol.wait`), and the odd alignment is dealt
// with there — aligned 32-bit shared-memory loads and a funnel shift by 0 or 16 bits.
//
// Tensor-core formulation (the same ideas as qmv_q4k_mma.cu):
//   A  the quant as an fp16 subnormal, exact: the byte + 128 (Q8_0: one XOR, two PRMT per four weights) or the
//      nibble in place (Q4_0: one AND per pair of weights; high nibbles carry a factor 16);
//   B  x·2^e split into fp16 hi / lo; lane t of a quad owns block t of a 128-column group, and B column
//      n = 4·part + t' carries x only at the k slots lane t' feeds, so D[row][n] is the Σ q·x of one block;
//   the −128 / −8 offsets: Σ (q − c)·x = Σ q·x − c·Σx with the per-block Σx staged with the activations;
//   d and the power-of-two factors are applied in fp32.  Only the order of fp32 additions differs from the CPU.
//
// Schedule: that of qmv_q4k_ring.cu — two groups of 8 warps per CTA, 16-row tiles dealt round-robin, a stage is
// 16 rows × eight (Q8_0) or sixteen (Q4_0) 128-column groups (one or two per warp), slots refilled by the warp that releases them last, every
// wait bounded.  Activation staging is per group (each warp converts the columns it multiplies).

#include <cuda.h>
#include <cuda_fp16.h>

#include "internal.h"

namespace yule {

namespace {

constexpr int kWarps = 8;
constexpr int kGroups = 2;
constexpr int kThreadsCta = kGroups * kWarps * 32;
constexpr int kStageRows = 16;
// 128-column groups per warp and stage: one of Q8_0 (136 bytes per row), two of Q4_0 (72 bytes per row), so that a
// stage row is about 1.1 KB in both formats and the per-stage bookkeeping is spread over the same amount of work
constexpr int kMaxStages = 6;      // per group
constexpr size_t kHalfSmSmem = 115712;
constexpr size_t kFullSmSmem = 227 * 1024;

template <bool Q8>
struct Fmt {
    static constexpr uint32_t kBlockBytes = Q8 ? 34 : 18;
    static constexpr uint32_t kSgBytes = 4 * kBlockBytes;                  // 136 / 72
    static constexpr int kSgsPerWarp = Q8 ? 1 : 2;
    static constexpr uint32_t kStageSgs = kWarps * kSgsPerWarp;            // 8 / 16 groups per stage row
    static constexpr uint32_t kRowPitch = kStageSgs * kSgBytes + 16;       // 1104 / 1168
    static constexpr uint32_t kStageBytes = kStageRows * kRowPitch;        // 17 664 / 18 688
};

__device__ __forceinline__ void mma_16816(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3,
                                          uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t h2_as_u32(__half2 h) { return *reinterpret_cast<uint32_t *>(&h); }
__device__ __forceinline__ uint32_t smem_u32(const void *p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
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
__device__ __forceinline__ bool ring_wait(uint32_t bar, uint32_t parity, int *status, long long budget) {
    if (mbar_try_wait(bar, parity)) return true;
    const long long t0 = clock64();
    for (uint32_t it = 1;; it++) {
        if (mbar_try_wait(bar, parity)) return true;
        if ((it & 255u) == 0u && clock64() - t0 > budget) {
            if (status) atomicCAS(status, 0, kStatusRingTimeout);
            return false;
        }
    }
}
__device__ __forceinline__ void ring_group_barrier(int group) {
    asm volatile("bar.sync %0, %1;" ::"r"(1 + group), "r"(kWarps * 32) : "memory");
}

// Shared-memory image of the activations, per 128-column group s, 8-column run m (0..15 within the group, i.e.
// block t = m / 4, run m % 4) and part (0 = hi, 1 = lo): one uint4 of four half2 B operands at index
//     ((s·4 + m%4)·2 + part)·4 + t
// so that the eight lanes that feed an MMA (block t = 0..3 × part) read 128 contiguous bytes.  Its four half2:
//   Q8_0  {x0,x1} {x2,x3} {x4,x5} {x6,x7}   (word 2j of a block ↔ .x,.y ; word 2j+1 ↔ .z,.w)
//   Q4_0  {x0,x4} {x2,x6} {x1,x5} {x3,x7}   (low nibbles ↔ .x,.y ; high nibbles ↔ .z,.w of the same word)
// sf[c/32] is Σ of the 32 scaled activations of block c/32; zb is 1 KB of zeros for the lanes whose B column is
// empty.
struct XImage {
    uint4 *xb;
    float *sf;
    uint4 *zb;
    float *red;
};
struct RingSmem {
    unsigned char *ring;
    XImage x;
    float *partial;  // [group][buffer][warp][row]
    uint64_t *bars;
    uint32_t *cnt;
};
constexpr size_t kPartialBytes = (size_t)kGroups * 2 * kWarps * 16 * sizeof(float);
__host__ __device__ inline size_t ring_fixed_bytes(uint32_t n_cols) {
    size_t off = (size_t)n_cols * 4 + (size_t)(n_cols / 32) * 4;
    off = (off + 15) & ~(size_t)15;
    off += 1024 + 64 * sizeof(float) + kPartialBytes + (size_t)kGroups * kMaxStages * (8 + 4);
    return (off + 127) & ~(size_t)127;
}
__device__ __forceinline__ RingSmem carve(unsigned char *base, uint32_t n_cols, size_t ring_bytes) {
    RingSmem s;
    s.ring = base;
    size_t off = ring_bytes;
    s.x.xb = reinterpret_cast<uint4 *>(base + off);
    off += (size_t)n_cols * 4;
    s.x.sf = reinterpret_cast<float *>(base + off);
    off += (size_t)(n_cols / 32) * 4;
    off = (off + 15) & ~(size_t)15;
    s.x.zb = reinterpret_cast<uint4 *>(base + off);
    off += 1024;
    s.x.red = reinterpret_cast<float *>(base + off);
    off += 64 * sizeof(float);
    s.partial = reinterpret_cast<float *>(base + off);
    off += kPartialBytes;
    s.bars = reinterpret_cast<uint64_t *>(base + off);
    off += (size_t)kGroups * kMaxStages * 8;
    s.cnt = reinterpret_cast<uint32_t *>(base + off);
    return s;
}

// Activation staging by one 8-warp group: warp w converts the 128-column groups w, w+8, … (the ones it multiplies),
// lane l the four columns 4l..4l+3 of each; one named barrier for the power-of-two scale (max|x| over the whole
// vector).  Both groups of a CTA write the same bytes to the same places; neither reads the other's.
// Returns 2^-e.
template <bool Q8>
__device__ __forceinline__ float stage_x_group(const XImage &sm, const float *__restrict__ x, uint32_t n_sg, int group, int wid,
                                               int lane) {
    constexpr int KC = 4;  // groups kept in registers between the two passes
    const uint32_t tid = threadIdx.x & (kWarps * 32 - 1);
    if (tid < 64) sm.zb[tid] = make_uint4(0u, 0u, 0u, 0u);
    float4 cache[KC];
    float mx = 0.f;
#pragma unroll
    for (int i = 0; i < KC; i++) {
        const uint32_t s = (uint32_t)wid + 8u * i;
        if (s < n_sg) {
            cache[i] = *reinterpret_cast<const float4 *>(x + s * 128u + lane * 4u);
            mx = fmaxf(mx, fmaxf(fmaxf(fabsf(cache[i].x), fabsf(cache[i].y)), fmaxf(fabsf(cache[i].z), fabsf(cache[i].w))));
        }
    }
    for (uint32_t s = (uint32_t)wid + 8u * KC; s < n_sg; s += 8u) {
        const float4 a = *reinterpret_cast<const float4 *>(x + s * 128u + lane * 4u);
        mx = fmaxf(mx, fmaxf(fmaxf(fabsf(a.x), fabsf(a.y)), fmaxf(fabsf(a.z), fabsf(a.w))));
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
    float *red = sm.red + group * 8;
    if (lane == 0) red[wid] = mx;
    ring_group_barrier(group);
    {
        const float4 m0 = *reinterpret_cast<const float4 *>(red), m1 = *reinterpret_cast<const float4 *>(red + 4);
        mx = fmaxf(fmaxf(fmaxf(m0.x, m0.y), fmaxf(m0.z, m0.w)), fmaxf(fmaxf(m1.x, m1.y), fmaxf(m1.z, m1.w)));
    }
    // 2^e with max|x|·2^e in [2^13, 2^14); exponent clamped so both 2^e and 2^-e stay finite normals
    int eb = (int)((__float_as_uint(mx) >> 23) & 0xFFu);
    if (mx == 0.f || eb == 0xFF) eb = 127 + 13;
    int se = 127 + 13 - (eb - 127);
    se = se < 1 ? 1 : (se > 253 ? 253 : se);
    const float scale = __uint_as_float((uint32_t)se << 23);
    auto convert = [&](uint32_t s, float4 a) {
        a.x *= scale;  // exact (power of two)
        a.y *= scale;
        a.z *= scale;
        a.w *= scale;
        const __half h0 = __float2half_rn(a.x), h1 = __float2half_rn(a.y), h2 = __float2half_rn(a.z), h3 = __float2half_rn(a.w);
        const __half l0 = __float2half_rn(a.x - __half2float(h0)), l1 = __float2half_rn(a.y - __half2float(h1)),
                     l2 = __float2half_rn(a.z - __half2float(h2)), l3 = __float2half_rn(a.w - __half2float(h3));
        // two neighbouring lanes hold one 8-column run: the even lane its columns 0..3, the odd lane 4..7
        uint32_t hi_a, hi_b, lo_a, lo_b;  // this lane's two half2 of the hi part, of the lo part
        if (Q8) {
            hi_a = h2_as_u32(__halves2half2(h0, h1));
            hi_b = h2_as_u32(__halves2half2(h2, h3));
            lo_a = h2_as_u32(__halves2half2(l0, l1));
            lo_b = h2_as_u32(__halves2half2(l2, l3));
        } else {
            // wanted: {x0,x4} {x2,x6} {x1,x5} {x3,x7}: every half2 pairs a column of the even lane with one of the odd lane
            const uint32_t mine_h02 = h2_as_u32(__halves2half2(h0, h2)), mine_h13 = h2_as_u32(__halves2half2(h1, h3));
            const uint32_t mine_l02 = h2_as_u32(__halves2half2(l0, l2)), mine_l13 = h2_as_u32(__halves2half2(l1, l3));
            const uint32_t oth_h02 = __shfl_xor_sync(0xffffffffu, mine_h02, 1), oth_h13 = __shfl_xor_sync(0xffffffffu, mine_h13, 1);
            const uint32_t oth_l02 = __shfl_xor_sync(0xffffffffu, mine_l02, 1), oth_l13 = __shfl_xor_sync(0xffffffffu, mine_l13, 1);
            // even lane (columns 0..3) builds {x0,x4} {x2,x6}; odd lane (columns 4..7) builds {x1,x5} {x3,x7}
            if ((lane & 1) == 0) {
                hi_a = __byte_perm(mine_h02, oth_h02, 0x5410);  // {x0, x4}
                hi_b = __byte_perm(mine_h02, oth_h02, 0x7632);  // {x2, x6}
                lo_a = __byte_perm(mine_l02, oth_l02, 0x5410);
                lo_b = __byte_perm(mine_l02, oth_l02, 0x7632);
            } else {
                hi_a = __byte_perm(oth_h13, mine_h13, 0x5410);  // {x1, x5}
                hi_b = __byte_perm(oth_h13, mine_h13, 0x7632);  // {x3, x7}
                lo_a = __byte_perm(oth_l13, mine_l13, 0x5410);
                lo_b = __byte_perm(oth_l13, mine_l13, 0x7632);
            }
        }
        const uint32_t m = (uint32_t)lane >> 1, t = m >> 2, run = m & 3u;
        const uint32_t idx = ((s * 4 + run) * 2) * 4 + t;  // hi part; the lo part sits 4 uint4 further on
        uint2 *dst_hi = reinterpret_cast<uint2 *>(sm.xb + idx) + (lane & 1);
        uint2 *dst_lo = reinterpret_cast<uint2 *>(sm.xb + idx + 4) + (lane & 1);
        *dst_hi = make_uint2(hi_a, hi_b);
        *dst_lo = make_uint2(lo_a, lo_b);
        // Σ over the 32 columns of a block: eight consecutive lanes
        float s4 = (a.x + a.y) + (a.z + a.w);
        s4 += __shfl_xor_sync(0xffffffffu, s4, 1);
        s4 += __shfl_xor_sync(0xffffffffu, s4, 2);
        s4 += __shfl_xor_sync(0xffffffffu, s4, 4);
        if ((lane & 7) == 0) sm.sf[s * 4 + (lane >> 3)] = s4;
    };
#pragma unroll
    for (int i = 0; i < KC; i++) {
        const uint32_t s = (uint32_t)wid + 8u * i;
        if (s < n_sg) convert(s, cache[i]);
    }
    for (uint32_t s = (uint32_t)wid + 8u * KC; s < n_sg; s += 8u) convert(s, *reinterpret_cast<const float4 *>(x + s * 128u + lane * 4u));
    __syncwarp();
    return __uint_as_float((uint32_t)(254 - se) << 23);
}

struct RingParams {
    CUtensorMap map;  // tiled view of the matrix (8-byte elements, box = 16 rows x the shared-memory row pitch): one copy per stage
    const uint8_t *w;
    float *out;
    uint32_t n_rows, n_cols, n_tiles;
    const float *x;
    const float *residual;
    uint32_t stages, chunks;
    int *status;
    long long wait_cycles;
    uint32_t late_wait;
    uint32_t sg_off;  // first 128-column group of the rows this launch covers (the batched kernel may take a range of the columns)
};

template <bool Q8>
__device__ __forceinline__ void issue_stage(const RingParams &p, uint32_t tile, uint32_t chunk, uint32_t n_sg, uint32_t dst,
                                            uint32_t bar, int lane) {
    // One tiled copy per stage, by the first lane (a copy per row, 16 per stage, cost the issuing warp about 0.7 µs on
    // the critical path of its group).  The box is as wide as the shared-memory row pitch; what lies beyond the chunk's
    // groups is never read, rows past the end of the matrix arrive as zeros.
    using F = Fmt<Q8>;
    (void)n_sg;
    if (lane == 0) {
        mbar_arrive_expect_tx(bar, F::kStageBytes);
        asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];" ::"r"(dst),
                     "l"(reinterpret_cast<uint64_t>(&p.map)), "r"(bar), "r"((p.sg_off + chunk * F::kStageSgs) * (F::kSgBytes / 8u)), "r"(tile * kStageRows)
                     : "memory");
    }
    __syncwarp();
}

// The 32-bit word `i` of the quants of a block whose bytes start at `qs` (2-byte aligned) in shared memory.
__device__ __forceinline__ uint32_t quant_word(const unsigned char *qs_aligned, uint32_t shift, int i) {
    const uint32_t lo = *reinterpret_cast<const uint32_t *>(qs_aligned + 4 * i);
    const uint32_t hi = *reinterpret_cast<const uint32_t *>(qs_aligned + 4 * i + 4);
    return __funnelshift_r(lo, hi, shift);
}

// One 128-column group of rows g and g+8: this lane's block t of it.
//   r0      the group's bytes of row g in the ring (row g+8 is 8 row pitches further on)
//   bp      this lane's B source for the group (image index of run 0, part and t folded in), or the zero region
//   sfp     Σx of the two blocks whose sums this lane finishes (or zeros for the lanes of the lo part)
template <bool Q8>
__device__ __forceinline__ void consume_sg(const unsigned char *r0, int t, const uint4 *bp, uint32_t bstride, const float *sfp, int u,
                                           float &acc0, float &acc1) {
    using F = Fmt<Q8>;
    const unsigned char *blk0 = r0 + (uint32_t)t * F::kBlockBytes, *blk1 = blk0 + 8 * F::kRowPitch;
    const uint32_t addr = (uint32_t)(size_t)(blk0 + 2);  // both rows share the alignment (the pitch is a multiple of 4)
    const uint32_t shift = (addr & 3u) * 8u;
    const unsigned char *q0 = blk0 + 2 - (addr & 3u), *q1 = blk1 + 2 - (addr & 3u);
    float dl[4] = {0.f, 0.f, 0.f, 0.f}, dh[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
    for (int run = 0; run < 4; run++) {
        const uint4 b = bp[run * bstride];
        if (Q8) {
            // words 2·run and 2·run+1: bytes + 128 as fp16 subnormals, pairs {b0,b1} and {b2,b3}
#pragma unroll
            for (int e = 0; e < 2; e++) {
                const uint32_t w0 = quant_word(q0, shift, 2 * run + e) ^ 0x80808080u, w1 = quant_word(q1, shift, 2 * run + e) ^ 0x80808080u;
                mma_16816(dl, __byte_perm(w0, 0u, 0x4140), __byte_perm(w1, 0u, 0x4140), __byte_perm(w0, 0u, 0x4342),
                          __byte_perm(w1, 0u, 0x4342), e ? b.z : b.x, e ? b.w : b.y);
            }
        } else {
            // word `run`: low nibbles {0,4} {2,6} in place, high nibbles {1,5} {3,7} with their factor 16
            const uint32_t w0 = quant_word(q0, shift, run), w1 = quant_word(q1, shift, run);
            const uint32_t w08 = w0 >> 8, w18 = w1 >> 8;
            mma_16816(dl, w0 & 0x000F000Fu, w1 & 0x000F000Fu, w08 & 0x000F000Fu, w18 & 0x000F000Fu, b.x, b.y);
            mma_16816(dh, w0 & 0x00F000F0u, w1 & 0x00F000F0u, w08 & 0x00F000F0u, w18 & 0x00F000F0u, b.z, b.w);
        }
    }
    // columns 2t and 2t+1 of D are blocks 2u and 2u+1 of this lane's part; scales of those blocks, both rows
    const float2 sx = *reinterpret_cast<const float2 *>(sfp);
    const float k24 = 16777216.0f, k20 = 1048576.0f, off = Q8 ? -128.0f : -8.0f;
#pragma unroll
    for (int r = 0; r < 2; r++) {
        const unsigned char *rb = r0 + (uint32_t)r * 8 * F::kRowPitch + (uint32_t)(2 * u) * F::kBlockBytes;
        const float d_a = __half2float(__ushort_as_half(*reinterpret_cast<const unsigned short *>(rb)));
        const float d_b = __half2float(__ushort_as_half(*reinterpret_cast<const unsigned short *>(rb + F::kBlockBytes)));
        float va = fmaf(dl[2 * r], k24, off * sx.x), vb = fmaf(dl[2 * r + 1], k24, off * sx.y);
        if (!Q8) {
            va = fmaf(dh[2 * r], k20, va);
            vb = fmaf(dh[2 * r + 1], k20, vb);
        }
        const float add = fmaf(d_a, va, d_b * vb);
        if (r)
            acc1 += add;
        else
            acc0 += add;
    }
}

template <bool Q8>
__global__ void __launch_bounds__(kThreadsCta, 2)
qmv_q8q4_ring_kernel(const __grid_constant__ RingParams p) {
    using F = Fmt<Q8>;
    extern __shared__ __align__(128) unsigned char smem_raw[];
    yule_pdl_launch_dependents();

    const int lane = threadIdx.x & 31;
    const int group = threadIdx.x >> 8, wid = (threadIdx.x >> 5) & (kWarps - 1);
    const int g = lane >> 2, t = lane & 3;
    const uint32_t n_sg = p.n_cols / 128;
    const uint32_t G = gridDim.x;
    const uint32_t first_tile = blockIdx.x + group * G, tile_stride = kGroups * G;
    const uint32_t my_tiles = p.n_tiles > first_tile ? (p.n_tiles - first_tile + tile_stride - 1) / tile_stride : 0;
    const uint32_t S = p.stages, chunks = p.chunks;
    const uint32_t total = my_tiles * chunks;
    if (total == 0) return;  // a group without tiles takes no part in anything below

    const RingSmem sm = carve(smem_raw, p.n_cols, (size_t)kGroups * S * F::kStageBytes);
    unsigned char *ring = sm.ring + (size_t)group * S * F::kStageBytes;
    const uint32_t ring_u32 = smem_u32(ring);
    const uint32_t bar0 = smem_u32(sm.bars + group * kMaxStages);
    uint32_t *cnt = sm.cnt + group * kMaxStages;

    // Warp 0 of each group sets the group's barriers up and starts the first copies; the other warps see both
    // through the group barrier of the activation staging, which they pass before their first wait.
    if (wid == 0) {
        if (lane == 0) {
            for (int i = 0; i < kMaxStages; i++) {
                mbar_init(bar0 + 8 * i, 1);
                cnt[i] = 0;
            }
            asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        }
        __syncwarp();
        uint32_t k = 0, c = 0;
        for (uint32_t n = 0; n < S && n < total; n++) {
            issue_stage<Q8>(p, first_tile + k * tile_stride, c, n_sg, ring_u32 + n * F::kStageBytes, bar0 + 8 * n, lane);
            if (++c == chunks) {
                c = 0;
                k++;
            }
        }
    }

    if (!p.late_wait) yule_pdl_wait();  // the activations (and the residual) come from the previous kernel
    const float inv_scale = stage_x_group<Q8>(sm.x, p.x, n_sg, group, wid, lane);

    // B column n = g is live only for g = t (hi part) and g = t + 4 (lo part); the other lanes read zeros
    const bool feeds = (g & 3) == t;
    const uint4 *b_base = feeds ? sm.x.xb + (g >> 2) * 4 + t : sm.x.zb;
    const uint32_t b_sg = feeds ? 32u : 0u, b_run = feeds ? 8u : 0u;  // uint4 per 128-column group / per 8-column run
    // D columns 2t, 2t+1 of this lane: blocks 2u, 2u+1 (u = t & 1) of part t >> 1; the offset term is charged once,
    // by the lanes of the hi part
    const int u = t & 1;
    const bool charge = t < 2;
    const float *sf_base = charge ? sm.x.sf + 2 * u : reinterpret_cast<const float *>(sm.x.zb);
    const uint32_t sf_sg = charge ? 4u : 0u;
    const uint32_t n_warps_used = n_sg < (uint32_t)kWarps ? n_sg : (uint32_t)kWarps;
    float *part_base = sm.partial + (size_t)group * (2 * kWarps * 16);

    uint32_t ck = 0, cc = 0;
    float acc0 = 0.f, acc1 = 0.f;
    uint32_t slot = 0, phase = 0;
    for (uint32_t n = 0; n < total; n++) {
        const uint32_t bar = bar0 + 8 * slot;
        if (!ring_wait(bar, phase, p.status, p.wait_cycles)) return;  // all eight warps of the group wait on the same copy
        const uint32_t sg0 = cc * F::kStageSgs;
        const uint32_t nsg = n_sg - sg0 < F::kStageSgs ? n_sg - sg0 : F::kStageSgs;
#pragma unroll
        for (int j = 0; j < F::kSgsPerWarp; j++) {
            const uint32_t local = (uint32_t)wid + (uint32_t)kWarps * j;  // groups ≡ wid (mod 8): the ones this warp staged x for
            if (local < nsg) {
                const uint32_t s = sg0 + local;
                const unsigned char *r0 = ring + (size_t)slot * F::kStageBytes + (uint32_t)g * F::kRowPitch + local * F::kSgBytes;
                consume_sg<Q8>(r0, t, b_base + (size_t)s * b_sg, b_run, sf_base + (size_t)s * sf_sg, u, acc0, acc1);
            }
        }
        if (n + S < total) {
            __syncwarp();
            uint32_t last = 0;
            if (lane == 0) {
                __threadfence_block();
                last = ((atomicAdd(&cnt[slot], 1u) & (kWarps - 1)) == kWarps - 1) ? 1u : 0u;
            }
            last = __shfl_sync(0xffffffffu, last, 0);
            if (last) {
                uint32_t nk = ck, nc = cc + S;
                while (nc >= chunks) {
                    nc -= chunks;
                    nk++;
                }
                issue_stage<Q8>(p, first_tile + nk * tile_stride, nc, n_sg, ring_u32 + slot * F::kStageBytes, bar, lane);
            }
        }
        if (cc + 1 == chunks) {
            float v0 = acc0, v1 = acc1;
            v0 += __shfl_xor_sync(0xffffffffu, v0, 1);
            v1 += __shfl_xor_sync(0xffffffffu, v1, 1);
            v0 += __shfl_xor_sync(0xffffffffu, v0, 2);
            v1 += __shfl_xor_sync(0xffffffffu, v1, 2);
            float *part = part_base + (size_t)(ck & 1u) * (kWarps * 16);
            if (t == 0) {
                part[wid * 16 + g] = v0;
                part[wid * 16 + g + 8] = v1;
            }
            acc0 = acc1 = 0.f;
            if (p.late_wait) yule_pdl_wait();  // the previous kernel is settled before our stores
            ring_group_barrier(group);
            const uint32_t tid = threadIdx.x & (kWarps * 32 - 1);
            if (tid < 128u) {
                // eight lanes per row fetch the eight warps' sums and add them in a fixed tree
                const uint32_t rr = tid >> 3, w2 = tid & 7u;
                float sacc = w2 < n_warps_used ? part[w2 * 16 + rr] : 0.f;
#pragma unroll
                for (int o = 1; o < 8; o <<= 1) sacc += __shfl_xor_sync(0xffffffffu, sacc, o);
                const uint32_t row = (first_tile + ck * tile_stride) * kStageRows + rr;
                if (w2 == 0 && row < p.n_rows) {
                    sacc *= inv_scale;
                    if (p.residual) sacc += p.residual[row];
                    p.out[row] = sacc;
                }
            }
            cc = 0;
            ck++;
        } else {
            cc++;
        }
        if (++slot == S) {
            slot = 0;
            phase ^= 1u;
        }
    }
}

// ── two to four activation vectors per pass ──────────────────────────────────────────────────────────────────
//
// Same ring, same stages, another use of the MMA's eight B columns: column 2v is the hi term of vector v, column
// 2v + 1 its lo term, and one MMA covers 16 weights of ONE block (its k slots are permuted so that lane t owns four
// consecutive quant bytes: one 32-bit word per row and MMA).  D[row][2v], D[row][2v+1] of the two MMAs of a block
// are the Σ q·x of that block for vector v; lane (g, t) holds them for rows g, g + 8 and vector t, adds the offset
// term (−128 or −8 times the block's Σx, staged with the activations) and multiplies by the row's d in fp32.  The
// tensor pipe does the same number of MMAs per weight as for one vector, so up to four vectors cost about the time
// of one.  Each vector has its own power-of-two scale.
//
// Shared-memory image of the activations: per 16-weight chunk (block b of group s, MMA j: chunk (4s + b)·2 + j)
// and B column n = 2v + part, four entries t of 8 bytes = the four halves lane t multiplies:
//   Q8_0  chunk j of a block = its weights 16j + 4t .. 16j + 4t + 3 for t = 0..3 (the four lanes of a quad read 16
//         contiguous bytes of a row, and the eight rows of an MMA sit at distinct multiples of 16 bytes mod 128:
//         no bank conflicts; lane t at byte 8t, the first version, had them two ways)
//   Q4_0  word t of a block holds its weights 8t..8t+7 (byte j: weight 2j low, 2j+1 high); chunk 0 = the low
//         nibbles, entry t = weights 8t, 8t+4, 8t+2, 8t+6; chunk 1 = the high nibbles, entry t = 8t+1, 8t+5, 8t+3,
//         8t+7 (the order in which the nibbles of a word fall into the A registers)
// A chunk is nb·64 bytes; the 8 x nb lanes that feed an MMA read it as one contiguous run.  sfb[(4s + b)·4 + v]
// is c·2^-24·Σx of block b for vector v (c = −128 or −8).
struct BatchParams {
    RingParams r;
    uint32_t nb, x_stride, out_stride;
};

struct BatchSmem {
    unsigned char *ring;
    unsigned char *xb;  // n_cols/16 chunks of nb·64 bytes
    float *sfb;         // n_cols/32 blocks x 4
    unsigned char *zb;  // 256 bytes of zeros
    float *red;         // [group][warp][4]
    float *partial;     // [group][buffer][warp][16 rows][4 vectors]
    uint64_t *bars;
    uint32_t *cnt;
};
constexpr size_t kBatchPartialBytes = (size_t)kGroups * 2 * kWarps * 64 * sizeof(float);
__host__ __device__ inline size_t batch_fixed_bytes(uint32_t n_cols, uint32_t nb) {
    size_t off = (size_t)n_cols * 4 * nb + (size_t)(n_cols / 32) * 16;
    off += 256 + (size_t)kGroups * kWarps * 4 * sizeof(float) + kBatchPartialBytes + (size_t)kGroups * kMaxStages * (8 + 4);
    return (off + 127) & ~(size_t)127;
}
__device__ __forceinline__ BatchSmem batch_carve(unsigned char *base, uint32_t n_cols, uint32_t nb, size_t ring_bytes) {
    BatchSmem s;
    s.ring = base;
    size_t off = ring_bytes;
    s.xb = base + off;
    off += (size_t)n_cols * 4 * nb;
    s.sfb = reinterpret_cast<float *>(base + off);
    off += (size_t)(n_cols / 32) * 16;
    s.zb = base + off;
    off += 256;
    s.red = reinterpret_cast<float *>(base + off);
    off += (size_t)kGroups * kWarps * 4 * sizeof(float);
    s.partial = reinterpret_cast<float *>(base + off);
    off += kBatchPartialBytes;
    s.bars = reinterpret_cast<uint64_t *>(base + off);
    off += (size_t)kGroups * kMaxStages * 8;
    s.cnt = reinterpret_cast<uint32_t *>(base + off);
    return s;
}

__device__ __forceinline__ void mma_16816_z(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%10,%10,%10};"
        : "=f"(d[0]), "=f"(d[1]), "=f"(d[2]), "=f"(d[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1), "f"(0.f));
}

// Activation staging by the whole CTA for `nb` vectors: warp W (0..15) converts the 128-column groups W, W+16, … of
// every vector, lane l the four columns 4l..4l+3; two CTA barriers (the per-vector power-of-two scales, then the
// finished image).  Returns 2^-e of vector `want` (the one this thread stores at the end of a tile).
template <bool Q8>
__device__ __forceinline__ float stage_x_batch(const BatchSmem &sm, const float *__restrict__ x, uint32_t x_stride, uint32_t nb,
                                               uint32_t n_sg, int lane, uint32_t want) {
    constexpr int KC = 2;  // groups per vector kept in registers between the two passes (all of them up to 4096 columns)
    constexpr uint32_t kAllWarps = kGroups * kWarps;
    const uint32_t W = threadIdx.x >> 5;
    if (threadIdx.x < 64) reinterpret_cast<uint32_t *>(sm.zb)[threadIdx.x] = 0u;
    float4 cache[4][KC];
    float mx[4] = {0.f, 0.f, 0.f, 0.f};
    auto amax4 = [](float4 a) { return fmaxf(fmaxf(fabsf(a.x), fabsf(a.y)), fmaxf(fabsf(a.z), fabsf(a.w))); };
#pragma unroll
    for (int v = 0; v < 4; v++) {
        if ((uint32_t)v < nb) {
            const float *xv = x + (size_t)v * x_stride;
#pragma unroll
            for (int i = 0; i < KC; i++) {
                const uint32_t s = W + kAllWarps * i;
                if (s < n_sg) cache[v][i] = *reinterpret_cast<const float4 *>(xv + s * 128u + lane * 4u);
            }
        }
    }
#pragma unroll
    for (int v = 0; v < 4; v++) {
        if ((uint32_t)v < nb) {
            const float *xv = x + (size_t)v * x_stride;
#pragma unroll
            for (int i = 0; i < KC; i++)
                if (W + kAllWarps * i < n_sg) mx[v] = fmaxf(mx[v], amax4(cache[v][i]));
            for (uint32_t s = W + kAllWarps * KC; s < n_sg; s += kAllWarps)
                mx[v] = fmaxf(mx[v], amax4(*reinterpret_cast<const float4 *>(xv + s * 128u + lane * 4u)));
        }
    }
#pragma unroll
    for (int v = 0; v < 4; v++)
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) mx[v] = fmaxf(mx[v], __shfl_xor_sync(0xffffffffu, mx[v], o));
    float4 *red = reinterpret_cast<float4 *>(sm.red);
    if (lane == 0) red[W] = make_float4(mx[0], mx[1], mx[2], mx[3]);
    __syncthreads();
    {
        float4 m = red[0];
#pragma unroll
        for (uint32_t w = 1; w < kAllWarps; w++) {
            const float4 o = red[w];
            m.x = fmaxf(m.x, o.x), m.y = fmaxf(m.y, o.y), m.z = fmaxf(m.z, o.z), m.w = fmaxf(m.w, o.w);
        }
        mx[0] = m.x, mx[1] = m.y, mx[2] = m.z, mx[3] = m.w;
    }
    float scale[4], inv_want = 1.f;
#pragma unroll
    for (int v = 0; v < 4; v++) {
        // 2^e with max|x|·2^e in [2^13, 2^14); exponent clamped so both 2^e and 2^-e stay finite normals
        int eb = (int)((__float_as_uint(mx[v]) >> 23) & 0xFFu);
        if (mx[v] == 0.f || eb == 0xFF) eb = 127 + 13;
        int se = 127 + 13 - (eb - 127);
        se = se < 1 ? 1 : (se > 253 ? 253 : se);
        scale[v] = __uint_as_float((uint32_t)se << 23);
        if ((uint32_t)v == want) inv_want = __uint_as_float((uint32_t)(254 - se) << 23);
    }
    const uint32_t chunk_bytes = nb * 64u;
    const float off = (Q8 ? -128.0f : -8.0f) * 5.9604644775390625e-08f;  // c · 2^-24
    const uint32_t b = (uint32_t)lane >> 3, m = (uint32_t)lane & 7u;
    auto convert = [&](uint32_t s, uint32_t v, float4 a, float sc) {
        a.x *= sc;  // exact (power of two)
        a.y *= sc;
        a.z *= sc;
        a.w *= sc;
        uint2 hi, lo;
        if (Q8) {
            const __half2 h01 = __floats2half2_rn(a.x, a.y), h23 = __floats2half2_rn(a.z, a.w);
            const float2 b01 = __half22float2(h01), b23 = __half22float2(h23);
            hi = make_uint2(h2_as_u32(h01), h2_as_u32(h23));
            lo = make_uint2(h2_as_u32(__floats2half2_rn(a.x - b01.x, a.y - b01.y)), h2_as_u32(__floats2half2_rn(a.z - b23.x, a.w - b23.y)));
        } else {
            // two neighbouring lanes hold the eight weights of a word: the even lane builds the entry of the low nibbles
            // {x0,x4} {x2,x6}, the odd lane that of the high nibbles {x1,x5} {x3,x7}
            const __half2 h02 = __floats2half2_rn(a.x, a.z), h13 = __floats2half2_rn(a.y, a.w);
            const float2 b02 = __half22float2(h02), b13 = __half22float2(h13);
            const uint32_t mine_h02 = h2_as_u32(h02), mine_h13 = h2_as_u32(h13);
            const uint32_t mine_l02 = h2_as_u32(__floats2half2_rn(a.x - b02.x, a.z - b02.y)),
                           mine_l13 = h2_as_u32(__floats2half2_rn(a.y - b13.x, a.w - b13.y));
            const bool even = (m & 1u) == 0;
            // each lane needs one pair of the other: the even lane the other's {x4,x6}, the odd lane the other's {x1,x3}
            const uint32_t oth_h = __shfl_xor_sync(0xffffffffu, even ? mine_h13 : mine_h02, 1);
            const uint32_t oth_l = __shfl_xor_sync(0xffffffffu, even ? mine_l13 : mine_l02, 1);
            if (even) {
                hi = make_uint2(__byte_perm(mine_h02, oth_h, 0x5410), __byte_perm(mine_h02, oth_h, 0x7632));
                lo = make_uint2(__byte_perm(mine_l02, oth_l, 0x5410), __byte_perm(mine_l02, oth_l, 0x7632));
            } else {
                hi = make_uint2(__byte_perm(oth_h, mine_h13, 0x5410), __byte_perm(oth_h, mine_h13, 0x7632));
                lo = make_uint2(__byte_perm(oth_l, mine_l13, 0x5410), __byte_perm(oth_l, mine_l13, 0x7632));
            }
        }
        // Q8_0: chunk j of a block = its weights 16j..16j+15, lane m % 4 of it; Q4_0: the lane pair m / 2 built entry m / 2
        // of chunk 0 (even lane) and of chunk 1 (odd lane)
        const uint32_t chunk = (s * 4 + b) * 2 + (Q8 ? (m >> 2) : (m & 1u)), t = Q8 ? (m & 3u) : (m >> 1);
        unsigned char *dst = sm.xb + (size_t)chunk * chunk_bytes + (2 * v) * 32u + t * 8u;
        *reinterpret_cast<uint2 *>(dst) = hi;
        *reinterpret_cast<uint2 *>(dst + 32) = lo;
        // Σ over the 32 columns of a block: eight consecutive lanes
        float s4 = (a.x + a.y) + (a.z + a.w);
        s4 += __shfl_xor_sync(0xffffffffu, s4, 1);
        s4 += __shfl_xor_sync(0xffffffffu, s4, 2);
        s4 += __shfl_xor_sync(0xffffffffu, s4, 4);
        if (m == 0) sm.sfb[(s * 4 + b) * 4 + v] = s4 * off;
    };
#pragma unroll
    for (int v = 0; v < 4; v++) {
        if ((uint32_t)v < nb) {
            const float *xv = x + (size_t)v * x_stride;
#pragma unroll
            for (int i = 0; i < KC; i++) {
                const uint32_t s = W + kAllWarps * i;
                if (s < n_sg) convert(s, v, cache[v][i], scale[v]);
            }
            for (uint32_t s = W + kAllWarps * KC; s < n_sg; s += kAllWarps)
                convert(s, v, *reinterpret_cast<const float4 *>(xv + s * 128u + lane * 4u), scale[v]);
        } else {
            for (uint32_t s = W; s < n_sg; s += kAllWarps)
                if (m == 0) sm.sfb[(s * 4 + b) * 4 + v] = 0.f;
        }
    }
    __syncthreads();
    return inv_want;
}

// Block B (0..3, a compile-time constant: it fixes the alignment of the quants) of one 128-column group, rows g and g+8.
template <bool Q8, int B>
__device__ __forceinline__ void consume_block_batch(const unsigned char *r0, int t, const unsigned char *bp, uint32_t chunk_stride,
                                                    const float *sfp, float &acc0, float &acc1) {
    using F = Fmt<Q8>;
    const unsigned char *blk0 = r0 + B * F::kBlockBytes, *blk1 = blk0 + 8 * F::kRowPitch;
    // the quants start 2 bytes into the block: 4-byte aligned for odd B, 2 bytes past a word for even B
    constexpr bool kShift = (B & 1) == 0;
    const uint32_t lane_off = 4u * t;
    const unsigned char *q0 = blk0 + (kShift ? 0 : 2) + lane_off, *q1 = blk1 + (kShift ? 0 : 2) + lane_off;
    auto word = [&](const unsigned char *q, int i) {
        const uint32_t *w = reinterpret_cast<const uint32_t *>(q);
        return kShift ? __funnelshift_r(w[i], w[i + 1], 16) : w[i];
    };
    float d[4];
    if (Q8) {
#pragma unroll
        for (int j = 0; j < 2; j++) {
            const uint32_t w0 = word(q0, 4 * j) ^ 0x80808080u, w1 = word(q1, 4 * j) ^ 0x80808080u;
            const uint2 b = *reinterpret_cast<const uint2 *>(bp + j * chunk_stride);
            const uint32_t a0 = __byte_perm(w0, 0u, 0x4140), a1 = __byte_perm(w1, 0u, 0x4140), a2 = __byte_perm(w0, 0u, 0x4342),
                           a3 = __byte_perm(w1, 0u, 0x4342);
            if (j == 0)
                mma_16816_z(d, a0, a1, a2, a3, b.x, b.y);
            else
                mma_16816(d, a0, a1, a2, a3, b.x, b.y);
        }
    } else {
        const uint32_t w0 = word(q0, 0), w1 = word(q1, 0);
        const uint2 blo = *reinterpret_cast<const uint2 *>(bp), bhi = *reinterpret_cast<const uint2 *>(bp + chunk_stride);
        mma_16816_z(d, w0 & 0x000F000Fu, w1 & 0x000F000Fu, (w0 >> 8) & 0x000F000Fu, (w1 >> 8) & 0x000F000Fu, blo.x, blo.y);
        mma_16816(d, (w0 >> 4) & 0x000F000Fu, (w1 >> 4) & 0x000F000Fu, (w0 >> 12) & 0x000F000Fu, (w1 >> 12) & 0x000F000Fu, bhi.x, bhi.y);
    }
    const float sx = *sfp;
    const float d0 = __half2float(__ushort_as_half(*reinterpret_cast<const unsigned short *>(blk0)));
    const float d1 = __half2float(__ushort_as_half(*reinterpret_cast<const unsigned short *>(blk1)));
    acc0 = fmaf(d0, (d[0] + d[1]) + sx, acc0);
    acc1 = fmaf(d1, (d[2] + d[3]) + sx, acc1);
}

template <bool Q8>
__global__ void __launch_bounds__(kThreadsCta, 1)
qmv_q8q4_ring_batch_kernel(const __grid_constant__ BatchParams bpm) {
    using F = Fmt<Q8>;
    const RingParams &p = bpm.r;
    extern __shared__ __align__(128) unsigned char smem_raw[];
    yule_pdl_launch_dependents();

    const int lane = threadIdx.x & 31;
    const int group = threadIdx.x >> 8, wid = (threadIdx.x >> 5) & (kWarps - 1);
    const int g = lane >> 2, t = lane & 3;
    const uint32_t nb = bpm.nb;
    const uint32_t n_sg = p.n_cols / 128;
    const uint32_t G = gridDim.x;
    const uint32_t first_tile = blockIdx.x + group * G, tile_stride = kGroups * G;
    const uint32_t my_tiles = p.n_tiles > first_tile ? (p.n_tiles - first_tile + tile_stride - 1) / tile_stride : 0;
    const uint32_t S = p.stages, chunks = p.chunks;
    const uint32_t total = my_tiles * chunks;  // 0: this group only helps with the activations

    const BatchSmem sm = batch_carve(smem_raw, p.n_cols, nb, (size_t)kGroups * S * F::kStageBytes);
    unsigned char *ring = sm.ring + (size_t)group * S * F::kStageBytes;
    const uint32_t ring_u32 = smem_u32(ring);
    const uint32_t bar0 = smem_u32(sm.bars + group * kMaxStages);
    uint32_t *cnt = sm.cnt + group * kMaxStages;

    if (wid == 0 && total != 0) {
        if (lane == 0) {
            for (int i = 0; i < kMaxStages; i++) {
                mbar_init(bar0 + 8 * i, 1);
                cnt[i] = 0;
            }
            asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        }
        __syncwarp();
        uint32_t k = 0, c = 0;
        for (uint32_t n = 0; n < S && n < total; n++) {
            issue_stage<Q8>(p, first_tile + k * tile_stride, c, n_sg, ring_u32 + n * F::kStageBytes, bar0 + 8 * n, lane);
            if (++c == chunks) {
                c = 0;
                k++;
            }
        }
    }

    if (!p.late_wait) yule_pdl_wait();  // the activations (and the residual) come from the previous kernel
    const uint32_t tid = threadIdx.x & (kWarps * 32 - 1);
    const float inv_scale = stage_x_batch<Q8>(sm, p.x, bpm.x_stride, nb, n_sg, lane, tid >> 4);
    if (total == 0) return;

    // B column n = g carries vector g / 2 (hi for even g, lo for odd); columns past 2·nb read zeros
    const bool feeds = (uint32_t)g < 2 * nb;
    const unsigned char *b_base = feeds ? sm.xb + g * 32 + t * 8 : sm.zb;
    const uint32_t chunk_stride = feeds ? nb * 64u : 0u;
    const bool charge = (uint32_t)t < nb;  // this lane's D columns belong to vector t
    const float *sf_base = charge ? sm.sfb + t : reinterpret_cast<const float *>(sm.zb);
    const uint32_t sf_blk = charge ? 4u : 0u;
    const uint32_t n_warps_used = n_sg < (uint32_t)kWarps ? n_sg : (uint32_t)kWarps;
    float *part_base = sm.partial + (size_t)group * (2 * kWarps * 64);

    uint32_t ck = 0, cc = 0;
    float acc0 = 0.f, acc1 = 0.f;
    uint32_t slot = 0, phase = 0;
    for (uint32_t n = 0; n < total; n++) {
        const uint32_t bar = bar0 + 8 * slot;
        if (!ring_wait(bar, phase, p.status, p.wait_cycles)) return;
        const uint32_t sg0 = cc * F::kStageSgs;
        const uint32_t nsg = n_sg - sg0 < F::kStageSgs ? n_sg - sg0 : F::kStageSgs;
#pragma unroll
        for (int j = 0; j < F::kSgsPerWarp; j++) {
            const uint32_t local = (uint32_t)wid + (uint32_t)kWarps * j;
            if (local < nsg) {
                const uint32_t s = sg0 + local;
                const unsigned char *r0 = ring + (size_t)slot * F::kStageBytes + (uint32_t)g * F::kRowPitch + local * F::kSgBytes;
                const unsigned char *bp = b_base + (size_t)(s * 8) * chunk_stride;
                const float *sfp = sf_base + (size_t)(s * 4) * sf_blk;
                consume_block_batch<Q8, 0>(r0, t, bp, chunk_stride, sfp, acc0, acc1);
                consume_block_batch<Q8, 1>(r0, t, bp + 2 * chunk_stride, chunk_stride, sfp + sf_blk, acc0, acc1);
                consume_block_batch<Q8, 2>(r0, t, bp + 4 * chunk_stride, chunk_stride, sfp + 2 * sf_blk, acc0, acc1);
                consume_block_batch<Q8, 3>(r0, t, bp + 6 * chunk_stride, chunk_stride, sfp + 3 * sf_blk, acc0, acc1);
            }
        }
        if (n + S < total) {
            __syncwarp();
            uint32_t last = 0;
            if (lane == 0) {
                __threadfence_block();
                last = ((atomicAdd(&cnt[slot], 1u) & (kWarps - 1)) == kWarps - 1) ? 1u : 0u;
            }
            last = __shfl_sync(0xffffffffu, last, 0);
            if (last) {
                uint32_t nk = ck, nc = cc + S;
                while (nc >= chunks) {
                    nc -= chunks;
                    nk++;
                }
                issue_stage<Q8>(p, first_tile + nk * tile_stride, nc, n_sg, ring_u32 + slot * F::kStageBytes, bar, lane);
            }
        }
        if (cc + 1 == chunks) {
            float *part = part_base + (size_t)(ck & 1u) * (kWarps * 64);
            part[wid * 64 + g * 4 + t] = acc0;
            part[wid * 64 + (g + 8) * 4 + t] = acc1;
            acc0 = acc1 = 0.f;
            if (p.late_wait) yule_pdl_wait();  // the previous kernel is settled before our stores
            ring_group_barrier(group);
            if (tid < 16u * nb) {
                // thread (vector v, row r): the eight warps' sums in a fixed order
                const uint32_t v = tid >> 4, rr = tid & 15u;
                float sacc = 0.f;
                for (uint32_t w2 = 0; w2 < n_warps_used; w2++) sacc += part[w2 * 64 + rr * 4 + v];
                const uint32_t row = (first_tile + ck * tile_stride) * kStageRows + rr;
                if (row < p.n_rows) {
                    sacc = (sacc * 16777216.0f) * inv_scale;
                    const size_t o = (size_t)v * bpm.out_stride + row;
                    if (p.residual) sacc += p.residual[o];
                    p.out[o] = sacc;
                }
            }
            cc = 0;
            ck++;
        } else {
            cc++;
        }
        if (++slot == S) {
            slot = 0;
            phase ^= 1u;
        }
    }
}

template <bool Q8>
cudaError_t launch_variant(const QmvArgs &a, int sm_count, cudaStream_t s) {
    using F = Fmt<Q8>;
    RingParams p = {};
    {
        const uint64_t row_bytes = (uint64_t)(a.n_cols / 128) * F::kSgBytes;
        cudaError_t me = cached_tensor_map_2d(a.w, 8, row_bytes / 8, a.n_rows, row_bytes, F::kRowPitch / 8, kStageRows, &p.map);
        if (me != cudaSuccess) return me;
    }
    p.w = a.w;
    p.out = a.out;
    p.n_rows = a.n_rows;
    p.n_cols = a.n_cols;
    p.n_tiles = (a.n_rows + kStageRows - 1) / kStageRows;
    p.x = a.x;
    p.residual = a.residual;
    p.status = a.status;
    p.wait_cycles = a.wait_cycles;
    p.late_wait = (a.pdl && a.late_wait) ? 1u : 0u;
    const uint32_t n_sg = a.n_cols / 128;
    p.chunks = (n_sg + F::kStageSgs - 1) / F::kStageSgs;
    uint32_t max_ctas = 2u * (uint32_t)sm_count;
    if (const char *k = knob("YULE_QMV_RING_CTAS")) max_ctas = (uint32_t)atoi(k) > 0 ? (uint32_t)atoi(k) : max_ctas;
    uint32_t grid = (p.n_tiles + kGroups - 1) / kGroups;
    if (grid > max_ctas) grid = max_ctas;
    const size_t fixed = ring_fixed_bytes(a.n_cols);
    const size_t per_stage = (size_t)kGroups * F::kStageBytes;
    uint32_t stages = fixed + 2 * per_stage <= kHalfSmSmem ? (uint32_t)((kHalfSmSmem - fixed) / per_stage)
                                                           : (uint32_t)((kFullSmSmem - fixed) / per_stage);
    if (stages > (uint32_t)kMaxStages) stages = kMaxStages;
    const uint32_t jobs_per_group = (p.n_tiles + kGroups * grid - 1) / (kGroups * grid);
    const uint32_t need = jobs_per_group * p.chunks;
    if (stages > need) stages = need;
    if (stages < 1) return cudaErrorInvalidValue;
    p.stages = stages;
    const size_t smem = (size_t)stages * per_stage + fixed;
    auto kern = qmv_q8q4_ring_kernel<Q8>;
    static bool attr_done[64] = {};  // the opt-in for large dynamic shared memory is a per-device attribute
    static std::mutex mu;
    {
        int dev = 0;
        cudaError_t e = cudaGetDevice(&dev);
        if (e != cudaSuccess) return e;
        std::lock_guard<std::mutex> lock(mu);
        if (dev < 0 || dev >= 64 || !attr_done[dev]) {
            e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kFullSmSmem);
            if (e != cudaSuccess) return e;
            if (dev >= 0 && dev < 64) attr_done[dev] = true;
        }
    }
    return launch_kernel(kern, dim3(grid), dim3(kThreadsCta), smem, s, a.pdl, p);
}

// One launch over the columns [128·sg_off, 128·sg_off + part_cols) of every row; `residual` is added to its results.
template <bool Q8>
cudaError_t launch_batch_variant(const QmvArgs &a, uint32_t nb, uint32_t stages, uint32_t sg_off, uint32_t part_cols, const float *residual,
                                 int sm_count, cudaStream_t s) {
    using F = Fmt<Q8>;
    BatchParams bp = {};
    RingParams &p = bp.r;
    {
        const uint64_t row_bytes = (uint64_t)(a.n_cols / 128) * F::kSgBytes;
        cudaError_t me = cached_tensor_map_2d(a.w, 8, row_bytes / 8, a.n_rows, row_bytes, F::kRowPitch / 8, kStageRows, &p.map);
        if (me != cudaSuccess) return me;
    }
    p.w = a.w;
    p.out = a.out;
    p.n_rows = a.n_rows;
    p.n_cols = part_cols;
    p.sg_off = sg_off;
    p.n_tiles = (a.n_rows + kStageRows - 1) / kStageRows;
    p.x = a.x + (size_t)sg_off * 128;
    p.residual = residual;
    p.status = a.status;
    p.wait_cycles = a.wait_cycles;
    p.late_wait = (a.pdl && a.late_wait) ? 1u : 0u;
    bp.nb = nb;
    bp.x_stride = a.x_stride;
    bp.out_stride = a.out_stride;
    const uint32_t n_sg = part_cols / 128;
    p.chunks = (n_sg + F::kStageSgs - 1) / F::kStageSgs;
    uint32_t grid = (p.n_tiles + kGroups - 1) / kGroups;
    if (grid > (uint32_t)sm_count) grid = (uint32_t)sm_count;
    const uint32_t jobs_per_group = (p.n_tiles + kGroups * grid - 1) / (kGroups * grid);
    const uint32_t need = jobs_per_group * p.chunks;
    if (stages > need) stages = need;
    p.stages = stages;
    const size_t smem = (size_t)stages * kGroups * F::kStageBytes + batch_fixed_bytes(part_cols, nb);
    auto kern = qmv_q8q4_ring_batch_kernel<Q8>;
    static bool attr_done[64] = {};  // the opt-in for large dynamic shared memory is a per-device attribute
    static std::mutex mu;
    {
        int dev = 0;
        cudaError_t e = cudaGetDevice(&dev);
        if (e != cudaSuccess) return e;
        std::lock_guard<std::mutex> lock(mu);
        if (dev < 0 || dev >= 64 || !attr_done[dev]) {
            e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kFullSmSmem);
            if (e != cudaSuccess) return e;
            if (dev >= 0 && dev < 64) attr_done[dev] = true;
        }
    }
    return launch_kernel(kern, dim3(grid), dim3(kThreadsCta), smem, s, a.pdl, bp);
}

// Ring slots per group that fit beside the activation image of `nb` vectors.
uint32_t batch_stages(uint32_t type, uint32_t n_cols, uint32_t nb) {
    const size_t stage = type == YULE_DTYPE_Q8_0 ? Fmt<true>::kStageBytes : Fmt<false>::kStageBytes;
    const size_t fixed = batch_fixed_bytes(n_cols, nb);
    if (fixed + (size_t)kGroups * stage > kFullSmSmem) return 0;
    const size_t st = (kFullSmSmem - fixed) / ((size_t)kGroups * stage);
    return st > (size_t)kMaxStages ? (uint32_t)kMaxStages : (uint32_t)st;
}

// Columns one launch covers for `nb` vectors: all of them if their activation image leaves room for three ring slots
// per group, else the largest multiple of a stage's columns that does; rows longer than that take several launches,
// each adding its columns' share to the result of the one before.  0: nothing fits.
uint32_t batch_part_cols(uint32_t type, uint32_t n_cols, uint32_t nb) {
    if (batch_stages(type, n_cols, nb) >= 3) return n_cols;
    const uint32_t step = 128u * (type == YULE_DTYPE_Q8_0 ? Fmt<true>::kStageSgs : Fmt<false>::kStageSgs);
    uint32_t best = 0;
    for (uint32_t c = step; c < n_cols; c += step)
        if (batch_stages(type, c, nb) >= 3) best = c;
    return best >= 4096 ? best : 0;  // shorter parts would be mostly launch overhead
}

}  // namespace

uint32_t q8q4_ring_batch_width(const QmvArgs &a) {
    if (a.type != YULE_DTYPE_Q8_0 && a.type != YULE_DTYPE_Q4_0) return 0;
    if (a.batch < 2 || a.n_cols == 0 || a.n_cols % 256 || a.n_rows == 0 || a.x_stride % 4) return 0;
    if ((reinterpret_cast<uintptr_t>(a.w) & 15) || (reinterpret_cast<uintptr_t>(a.x) & 15)) return 0;
    // the widest pass whose image fits whole; for longer rows the widest that fits in parts
    for (uint32_t nb = a.batch < 4 ? a.batch : 4; nb >= 2; nb--)
        if (batch_part_cols(a.type, a.n_cols, nb) == a.n_cols) return nb;
    for (uint32_t nb = a.batch < 4 ? a.batch : 4; nb >= 2; nb--)
        if (batch_part_cols(a.type, a.n_cols, nb) != 0) return nb;
    return 0;
}

cudaError_t launch_q8q4_ring_batch(const QmvArgs &a, uint32_t nb, int sm_count, cudaStream_t s, uint64_t *launches) {
    if (nb < 2 || nb > 4) return cudaErrorInvalidValue;
    const uint32_t part = batch_part_cols(a.type, a.n_cols, nb);
    if (part == 0) return cudaErrorInvalidValue;
    const bool q8 = a.type == YULE_DTYPE_Q8_0;
    const uint32_t step = 128u * (q8 ? Fmt<true>::kStageSgs : Fmt<false>::kStageSgs);
    const uint32_t n_parts = (a.n_cols + part - 1) / part;
    const uint32_t stages_total = (a.n_cols + step - 1) / step;
    uint32_t col = 0;
    for (uint32_t i = 0; i < n_parts; i++) {  // parts of equal length (in stages)
        const uint32_t st = stages_total / n_parts + (i < stages_total % n_parts ? 1u : 0u);
        uint32_t cols = st * step;
        if (col + cols > a.n_cols) cols = a.n_cols - col;
        const uint32_t stages = batch_stages(a.type, cols, nb);
        const float *residual = i == 0 ? a.residual : a.out;  // later parts add to what the earlier ones stored
        cudaError_t e = q8 ? launch_batch_variant<true>(a, nb, stages, col / 128, cols, residual, sm_count, s)
                           : launch_batch_variant<false>(a, nb, stages, col / 128, cols, residual, sm_count, s);
        if (e != cudaSuccess) return e;
        *launches += 1;
        col += cols;
    }
    return cudaSuccess;
}

bool q8q4_ring_supported(const QmvArgs &a) {
    if (a.type != YULE_DTYPE_Q8_0 && a.type != YULE_DTYPE_Q4_0) return false;
    if (a.batch != 1 || a.n_cols == 0 || a.n_cols % 256 || a.n_rows == 0) return false;
    if ((reinterpret_cast<uintptr_t>(a.w) & 15) || (reinterpret_cast<uintptr_t>(a.x) & 15)) return false;
    const size_t smallest = ring_fixed_bytes(a.n_cols) + (size_t)kGroups * (a.type == YULE_DTYPE_Q8_0 ? Fmt<true>::kStageBytes : Fmt<false>::kStageBytes);
    return smallest <= kFullSmSmem;
}

cudaError_t launch_q8q4_ring(const QmvArgs &a, int sm_count, cudaStream_t s, uint64_t *launches) {
    cudaError_t e = a.type == YULE_DTYPE_Q8_0 ? launch_variant<true>(a, sm_count, s) : launch_variant<false>(a, sm_count, s);
    if (e == cudaSuccess) *launches += 1;
    return e;
}

}  // namespace yule
