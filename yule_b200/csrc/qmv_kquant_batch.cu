// qmv_kquant_batch.cu — Q4_K and Q6_K fused dequantise + matvec over two to four activation vectors per pass, on
// the tensor pipe, weights staged through a shared-memory ring by tiled TMA copies.
//
// Contract: yule-core/src/dequant.rs:902-1009 per vector — Q4_K: Σ over 32-weight sub-blocks of d·sc·Σ q·x −
// dmin·m·Σx; Q6_K (row-planar device copy of the tensor): Σ over 16-weight scale groups of d·sc·Σ (q − 32)·x.
//
// Formulation.  One `mma.sync.m16n8k16` covers 16 weights of ONE scale group (Q6_K) or half a sub-block (Q4_K) of
// 16 rows; its eight B columns are the hi and lo fp16 terms of up to four activation vectors (column 2v: hi of
// vector v, 2v + 1: lo), so the tensor pipe does as many MMAs per weight as the one-vector kernels and the extra
// vectors ride along.  A operands are the quants as fp16 subnormals (exact): lane t of a quad owns four consecutive
// quant bytes of the group, `v & 0x00FF00FF` and `(v >> 8) & 0x00FF00FF` are its two A registers (k slots 2t, 2t+1
// = bytes 0, 2; k slots 2t+8, 2t+9 = bytes 1, 3), and the activation image holds x in that order.  Lane (g, t)
// receives D[g][2t], D[g][2t+1], D[g+8][…]: the Σ q·x of rows g, g + 8 against vector t; it adds hi + lo, the
// offset term (Q6_K: −32·Σx of the group; Q4_K: −dmin·m·Σx of the sub-block) and multiplies by d·sc in fp32.
// Only the order of the fp32 additions differs from the CPU.
//
// Schedule: the one of the one-vector ring kernels (qmv_q4k_ring.cu, qmv_q6k_ring.cu) — one CTA of two 8-warp
// groups per SM, 16-row tiles dealt round-robin over the groups, a stage = 16 rows × 8 super-blocks (one per warp),
// slots refilled by the warp that releases them last, every wait bounded.  The activation image (all vectors) is
// built once per CTA.

#include <cuda.h>
#include <cuda_fp16.h>

#include <mutex>

#include "internal.h"

namespace yule {

namespace {

constexpr int kWarps = 8;
constexpr int kGroups = 2;
constexpr int kThreadsCta = kGroups * kWarps * 32;
constexpr int kStageRows = 16;
constexpr int kStageBlocks = kWarps;  // super-blocks per row in a stage
constexpr int kMaxStages = 6;         // per group
constexpr size_t kFullSmSmem = 227 * 1024;

// Q4_K stage: 16 rows of eight raw 144-byte super-blocks (+16 bytes of padding: the pitch is ≡ 16 mod 128).
constexpr uint32_t kQ4RowPitch = kStageBlocks * 144 + 16, kQ4StageBytes = kStageRows * kQ4RowPitch;  // 18 688
// Q6_K stage: four planes (low nibbles, high bit pairs, scales, d) of the row-planar copy
constexpr uint32_t kQlPitch = kStageBlocks * 128 + 32, kQhPitch = kStageBlocks * 64 + 64, kScPitch = kStageBlocks * 16 + 16, kDPitch = 16;
constexpr uint32_t kQlOff = 0, kQhOff = kQlOff + kStageRows * kQlPitch, kScOff = kQhOff + kStageRows * kQhPitch,
                   kDOff = kScOff + kStageRows * kScPitch, kQ6StageBytes = kDOff + kStageRows * kDPitch;  // 28 672
template <bool Q6>
__host__ __device__ constexpr uint32_t stage_bytes() {
    return Q6 ? kQ6StageBytes : kQ4StageBytes;
}

__host__ __device__ inline uint32_t d_section_bytes(uint32_t bpr) { return (bpr * 2 + 15) & ~15u; }
__host__ __device__ inline size_t row_record_bytes(uint32_t bpr) { return (size_t)bpr * 208 + d_section_bytes(bpr); }

#include "ring_common.cuh"

__device__ __forceinline__ void mma_16816(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
__device__ __forceinline__ void mma_16816_z(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%10,%10,%10,%10};"
        : "=f"(d[0]), "=f"(d[1]), "=f"(d[2]), "=f"(d[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1), "f"(0.f));
}
__device__ __forceinline__ uint32_t h2_as_u32(__half2 h) { return *reinterpret_cast<uint32_t *>(&h); }
__device__ __forceinline__ void ring_group_barrier(int group) {
    asm volatile("bar.sync %0, %1;" ::"r"(1 + group), "r"(kWarps * 32) : "memory");
}
// Byte `i` (0..3) of `w` as a float, for bytes that hold an unsigned value: 2^23 + b as fp32 bits, minus 2^23.
template <int I>
__device__ __forceinline__ float byte_to_float(uint32_t w) {
    return __uint_as_float(__byte_perm(w, 0x4B000000u, 0x7440 + I)) - 8388608.0f;
}

constexpr int kMaxSegs = 3;  // matrices that share their activations (Q/K/V; gate/up) in one launch
struct KBatchParams {
    CUtensorMap map[kMaxSegs][4];  // per matrix — Q4_K: [0] = the raw tensor; Q6_K: the four planes of the row-planar copy
    float *out[kMaxSegs];
    uint32_t n_rows[kMaxSegs], out_stride[kMaxSegs];
    uint32_t tile0[kMaxSegs + 1];  // first 16-row tile of each matrix in the launch's tile numbering; [n_seg] = n_tiles
    uint32_t n_seg;
    const float *x;
    const float *residual;  // added to the results of matrix 0 (single-matrix launches only)
    const float *norm_w;    // RMSNorm prologue: the rows are x · inv_rms · norm_w (yule-infer/src/model_runner.rs:254-263), or null
    float eps;
    uint32_t n_cols, n_tiles, stages, chunks;
    uint32_t nb, x_stride, late_wait;
    uint32_t blk_off;  // first super-block of the rows this launch covers (a launch takes a range of the columns)
    int *status;
    long long wait_cycles;
};

// Shared memory: ring | activation image | per-chunk sums | zeros | reduction scratch | partial sums | barriers.
// Image: per 16-column chunk c (columns 16c..16c+15) and B column n = 2v + part, four entries t of 8 bytes: the halves
// of columns 16c + 4t + {0, 2, 1, 3}.  A chunk is nb·64 bytes.  sfb[4c + v] = 2^-24 · Σ of the chunk's scaled x.
struct KBatchSmem {
    unsigned char *ring, *xb;
    float *sfb;
    unsigned char *zb;
    float *red, *partial;
    uint64_t *bars;
    uint32_t *cnt;
};
constexpr size_t kPartialBytes = (size_t)kGroups * 2 * kWarps * 64 * sizeof(float);
__host__ __device__ inline size_t fixed_bytes(uint32_t n_cols, uint32_t nb) {
    size_t off = (size_t)n_cols * 4 * nb + (size_t)(n_cols / 16) * 16;
    off += 256 + 2 * (size_t)kGroups * kWarps * 4 * sizeof(float) + kPartialBytes + (size_t)kGroups * kMaxStages * (8 + 4);
    return (off + 127) & ~(size_t)127;
}
__device__ __forceinline__ KBatchSmem carve(unsigned char *base, uint32_t n_cols, uint32_t nb, size_t ring_bytes) {
    KBatchSmem s;
    s.ring = base;
    size_t off = ring_bytes;
    s.xb = base + off;
    off += (size_t)n_cols * 4 * nb;
    s.sfb = reinterpret_cast<float *>(base + off);
    off += (size_t)(n_cols / 16) * 16;
    s.zb = base + off;
    off += 256;
    s.red = reinterpret_cast<float *>(base + off);
    off += 2 * (size_t)kGroups * kWarps * 4 * sizeof(float);
    s.partial = reinterpret_cast<float *>(base + off);
    off += kPartialBytes;
    s.bars = reinterpret_cast<uint64_t *>(base + off);
    off += (size_t)kGroups * kMaxStages * 8;
    s.cnt = reinterpret_cast<uint32_t *>(base + off);
    return s;
}

template <bool Q6>
__device__ __forceinline__ void issue_stage(const KBatchParams &p, uint32_t tile, uint32_t chunk, uint32_t dst, uint32_t bar, int lane) {
    // Tiled copies by the first lane; every box is as wide as its plane's shared-memory row pitch (what lies beyond the
    // eight super-blocks is never read), rows past the end of the matrix arrive as zeros.
    if (lane == 0) {
        uint32_t seg = 0;
        while (seg + 1 < p.n_seg && tile >= p.tile0[seg + 1]) seg++;
        const uint32_t row0 = (tile - p.tile0[seg]) * kStageRows, blk0 = p.blk_off + chunk * kStageBlocks;
        mbar_arrive_expect_tx(bar, stage_bytes<Q6>());
        auto box = [&](uint32_t off, const CUtensorMap *m, uint32_t x) {
            asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];" ::"r"(
                             dst + off),
                         "l"(reinterpret_cast<uint64_t>(m)), "r"(bar), "r"(x), "r"(row0)
                         : "memory");
        };
        if (Q6) {
            box(kQlOff, &p.map[seg][0], blk0 * 16u);
            box(kQhOff, &p.map[seg][1], blk0 * 8u);
            box(kScOff, &p.map[seg][2], blk0 * 2u);
            box(kDOff, &p.map[seg][3], blk0 / 4u);
        } else {
            box(0, &p.map[seg][0], blk0 * 18u);
        }
    }
    __syncwarp();
}

// Activation staging by the whole CTA: warp W (0..15) converts the 128-column groups W, W+16, … of every vector, lane
// l the four columns 4l..4l+3; two CTA barriers (the per-vector power-of-two scales, then the finished image).
// Returns 2^-e of vector `want`.
__device__ __forceinline__ float stage_x(const KBatchSmem &sm, const float *__restrict__ x, uint32_t x_stride, uint32_t nb, uint32_t n_sg,
                                         int lane, uint32_t want, const float *__restrict__ norm_w, float eps) {
    constexpr int KC = 2;  // groups per vector kept in registers between the two passes (all of them up to 4096 columns)
    constexpr uint32_t kAllWarps = kGroups * kWarps;
    const uint32_t W = threadIdx.x >> 5;
    if (threadIdx.x < 64) reinterpret_cast<uint32_t *>(sm.zb)[threadIdx.x] = 0u;
    float4 cache[4][KC];
    float mx[4] = {0.f, 0.f, 0.f, 0.f}, ss[4] = {0.f, 0.f, 0.f, 0.f};
    // With the RMSNorm prologue the image holds x · inv_rms · w: max |x · w| and Σx² are reduced together, the
    // vector's 1/rms enters the maximum afterwards.
    auto wts = [&](uint32_t s) { return norm_w ? *reinterpret_cast<const float4 *>(norm_w + s * 128u + lane * 4u) : make_float4(1.f, 1.f, 1.f, 1.f); };
    auto amax4 = [](float4 a, float4 g) { return fmaxf(fmaxf(fabsf(a.x * g.x), fabsf(a.y * g.y)), fmaxf(fabsf(a.z * g.z), fabsf(a.w * g.w))); };
    auto sq4 = [](float4 a, float acc) { return fmaf(a.w, a.w, fmaf(a.z, a.z, fmaf(a.y, a.y, fmaf(a.x, a.x, acc)))); };
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
                if (W + kAllWarps * i < n_sg) {
                    mx[v] = fmaxf(mx[v], amax4(cache[v][i], wts(W + kAllWarps * i)));
                    ss[v] = sq4(cache[v][i], ss[v]);
                }
            for (uint32_t s = W + kAllWarps * KC; s < n_sg; s += kAllWarps) {
                const float4 a = *reinterpret_cast<const float4 *>(xv + s * 128u + lane * 4u);
                mx[v] = fmaxf(mx[v], amax4(a, wts(s)));
                ss[v] = sq4(a, ss[v]);
            }
        }
    }
#pragma unroll
    for (int v = 0; v < 4; v++)
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            mx[v] = fmaxf(mx[v], __shfl_xor_sync(0xffffffffu, mx[v], o));
            ss[v] += __shfl_xor_sync(0xffffffffu, ss[v], o);
        }
    float4 *red = reinterpret_cast<float4 *>(sm.red);
    if (lane == 0) {
        red[W] = make_float4(mx[0], mx[1], mx[2], mx[3]);
        red[kAllWarps + W] = make_float4(ss[0], ss[1], ss[2], ss[3]);
    }
    __syncthreads();
    float inv_rms[4] = {1.f, 1.f, 1.f, 1.f};
    {
        float4 m = red[0], q = red[kAllWarps];
#pragma unroll
        for (uint32_t w = 1; w < kAllWarps; w++) {
            const float4 o = red[w], o2 = red[kAllWarps + w];
            m.x = fmaxf(m.x, o.x), m.y = fmaxf(m.y, o.y), m.z = fmaxf(m.z, o.z), m.w = fmaxf(m.w, o.w);
            q.x += o2.x, q.y += o2.y, q.z += o2.z, q.w += o2.w;
        }
        mx[0] = m.x, mx[1] = m.y, mx[2] = m.z, mx[3] = m.w;
        if (norm_w) {
            // 1 / sqrt(Σx² / n + eps), as the CPU runner forms it (model_runner.rs:254-258)
            const float n = (float)(n_sg * 128u);
            inv_rms[0] = 1.0f / sqrtf(q.x / n + eps), inv_rms[1] = 1.0f / sqrtf(q.y / n + eps);
            inv_rms[2] = 1.0f / sqrtf(q.z / n + eps), inv_rms[3] = 1.0f / sqrtf(q.w / n + eps);
#pragma unroll
            for (int v = 0; v < 4; v++) mx[v] *= inv_rms[v];
        }
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
    auto convert = [&](uint32_t s, uint32_t v, float4 a, float sc) {
        if (norm_w) {
            const float4 g = wts(s);
            const float ir = inv_rms[v];
            a.x = a.x * ir * g.x, a.y = a.y * ir * g.y, a.z = a.z * ir * g.z, a.w = a.w * ir * g.w;
        }
        a.x *= sc;  // exact (power of two)
        a.y *= sc;
        a.z *= sc;
        a.w *= sc;
        const __half2 h02 = __floats2half2_rn(a.x, a.z), h13 = __floats2half2_rn(a.y, a.w);
        const float2 b02 = __half22float2(h02), b13 = __half22float2(h13);
        const uint2 hi = make_uint2(h2_as_u32(h02), h2_as_u32(h13));
        const uint2 lo = make_uint2(h2_as_u32(__floats2half2_rn(a.x - b02.x, a.z - b02.y)), h2_as_u32(__floats2half2_rn(a.y - b13.x, a.w - b13.y)));
        const uint32_t chunk = s * 8 + ((uint32_t)lane >> 2), t = (uint32_t)lane & 3u;
        unsigned char *dst = sm.xb + (size_t)chunk * chunk_bytes + (2 * v) * 32u + t * 8u;
        *reinterpret_cast<uint2 *>(dst) = hi;
        *reinterpret_cast<uint2 *>(dst + 32) = lo;
        // Σ over the 16 columns of a chunk: four consecutive lanes
        float s4 = (a.x + a.y) + (a.z + a.w);
        s4 += __shfl_xor_sync(0xffffffffu, s4, 1);
        s4 += __shfl_xor_sync(0xffffffffu, s4, 2);
        if (t == 0) sm.sfb[chunk * 4 + v] = s4 * 5.9604644775390625e-08f;
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
                if ((lane & 3) == 0) sm.sfb[(s * 8 + ((uint32_t)lane >> 2)) * 4 + v] = 0.f;
        }
    }
    __syncthreads();
    return inv_want;
}

// One Q4_K super-block of rows g and g+8.
//   r0          the block's 144 bytes of row g in the ring (row g+8: 8 row pitches further on)
//   bp, cs      this lane's B source of the block's first chunk and the chunk stride (zeros / 0 for idle columns)
//   sfp, sfs    this lane's chunk sums of the block's first chunk and their stride in floats (zeros / 0)
__device__ __forceinline__ void consume_q4k(const unsigned char *r0, int t, const unsigned char *bp, uint32_t cs, const float *sfp,
                                            uint32_t sfs, float &acc0, float &acc1) {
    const unsigned char *r1 = r0 + 8 * kQ4RowPitch;
    const uint4 h0 = *reinterpret_cast<const uint4 *>(r0), h1 = *reinterpret_cast<const uint4 *>(r1);
    // d·sc and dmin·m of the eight sub-blocks of both rows (yule-core/src/dequant.rs:165-176: 6-bit scales and mins)
    float dsc[2][8], dmn[2][8];
#pragma unroll
    for (int r = 0; r < 2; r++) {
        const uint4 h = r ? h1 : h0;
        const float2 dd = __half22float2(*reinterpret_cast<const __half2 *>(&h.x));
        const uint32_t sc_lo = h.y & 0x3F3F3F3Fu, mn_lo = h.z & 0x3F3F3F3Fu;
        const uint32_t sc_hi = (h.w & 0x0F0F0F0Fu) | ((h.y >> 2) & 0x30303030u), mn_hi = ((h.w >> 4) & 0x0F0F0F0Fu) | ((h.z >> 2) & 0x30303030u);
        dsc[r][0] = dd.x * byte_to_float<0>(sc_lo), dsc[r][1] = dd.x * byte_to_float<1>(sc_lo);
        dsc[r][2] = dd.x * byte_to_float<2>(sc_lo), dsc[r][3] = dd.x * byte_to_float<3>(sc_lo);
        dsc[r][4] = dd.x * byte_to_float<0>(sc_hi), dsc[r][5] = dd.x * byte_to_float<1>(sc_hi);
        dsc[r][6] = dd.x * byte_to_float<2>(sc_hi), dsc[r][7] = dd.x * byte_to_float<3>(sc_hi);
        dmn[r][0] = dd.y * byte_to_float<0>(mn_lo), dmn[r][1] = dd.y * byte_to_float<1>(mn_lo);
        dmn[r][2] = dd.y * byte_to_float<2>(mn_lo), dmn[r][3] = dd.y * byte_to_float<3>(mn_lo);
        dmn[r][4] = dd.y * byte_to_float<0>(mn_hi), dmn[r][5] = dd.y * byte_to_float<1>(mn_hi);
        dmn[r][6] = dd.y * byte_to_float<2>(mn_hi), dmn[r][7] = dd.y * byte_to_float<3>(mn_hi);
    }
#pragma unroll
    for (int jj = 0; jj < 4; jj++) {
        // 32 bytes: low nibbles = sub-block 2jj, high nibbles = sub-block 2jj + 1; this lane's word of each half
        const uint32_t wa0 = *reinterpret_cast<const uint32_t *>(r0 + 16 + 32 * jj + 4 * t);
        const uint32_t wb0 = *reinterpret_cast<const uint32_t *>(r0 + 16 + 32 * jj + 16 + 4 * t);
        const uint32_t wa1 = *reinterpret_cast<const uint32_t *>(r1 + 16 + 32 * jj + 4 * t);
        const uint32_t wb1 = *reinterpret_cast<const uint32_t *>(r1 + 16 + 32 * jj + 16 + 4 * t);
#pragma unroll
        for (int nib = 0; nib < 2; nib++) {
            const int s = 2 * jj + nib;
            const uint2 ba = *reinterpret_cast<const uint2 *>(bp + (2 * s) * cs), bb = *reinterpret_cast<const uint2 *>(bp + (2 * s + 1) * cs);
            const uint32_t a0 = wa0 >> (4 * nib), a1 = wa1 >> (4 * nib), b0 = wb0 >> (4 * nib), b1 = wb1 >> (4 * nib);
            float d[4];
            mma_16816_z(d, a0 & 0x000F000Fu, a1 & 0x000F000Fu, (a0 >> 8) & 0x000F000Fu, (a1 >> 8) & 0x000F000Fu, ba.x, ba.y);
            mma_16816(d, b0 & 0x000F000Fu, b1 & 0x000F000Fu, (b0 >> 8) & 0x000F000Fu, (b1 >> 8) & 0x000F000Fu, bb.x, bb.y);
            const float sx = sfp[(2 * s) * sfs] + sfp[(2 * s + 1) * sfs];
            acc0 = fmaf(dsc[0][s], d[0] + d[1], acc0);
            acc1 = fmaf(dsc[1][s], d[2] + d[3], acc1);
            acc0 = fmaf(-dmn[0][s], sx, acc0);
            acc1 = fmaf(-dmn[1][s], sx, acc1);
        }
    }
}

// One Q6_K super-block (slot `w` of the stage `st`) of rows g and g+8 (dequant.rs:343-373: weight 128h + 32j + l has
// its low nibble in ql[64h + 32(j&1) + l] (high half of the byte for j ≥ 2), bits 2j..2j+1 of qh[32h + l] above it,
// scale 8h + 2j + l/16).
__device__ __forceinline__ void consume_q6k(const unsigned char *st, int g, int w, int t, const unsigned char *bp, uint32_t cs, const float *sfp,
                                            uint32_t sfs, float &acc0, float &acc1) {
    const unsigned char *ql0 = st + kQlOff + g * kQlPitch + w * 128, *ql1 = ql0 + 8 * kQlPitch;
    const unsigned char *qh0 = st + kQhOff + g * kQhPitch + w * 64, *qh1 = qh0 + 8 * kQhPitch;
    const unsigned char *sc0 = st + kScOff + g * kScPitch + w * 16, *sc1 = sc0 + 8 * kScPitch;
    const unsigned char *d0 = st + kDOff + g * kDPitch + w * 2, *d1 = d0 + 8 * kDPitch;
    // d·sc of the sixteen scale groups of both rows: signed bytes → float via (b ^ 0x80) − 128
    float dsc[2][16];
#pragma unroll
    for (int r = 0; r < 2; r++) {
        const float d = __half2float(__ushort_as_half(*reinterpret_cast<const unsigned short *>(r ? d1 : d0)));
        const uint4 sw = *reinterpret_cast<const uint4 *>(r ? sc1 : sc0);
        const uint32_t wds[4] = {sw.x ^ 0x80808080u, sw.y ^ 0x80808080u, sw.z ^ 0x80808080u, sw.w ^ 0x80808080u};
#pragma unroll
        for (int i = 0; i < 4; i++) {
            dsc[r][4 * i + 0] = d * (byte_to_float<0>(wds[i]) - 128.0f);
            dsc[r][4 * i + 1] = d * (byte_to_float<1>(wds[i]) - 128.0f);
            dsc[r][4 * i + 2] = d * (byte_to_float<2>(wds[i]) - 128.0f);
            dsc[r][4 * i + 3] = d * (byte_to_float<3>(wds[i]) - 128.0f);
        }
    }
#pragma unroll
    for (int h = 0; h < 2; h++) {
#pragma unroll
        for (int u = 0; u < 2; u++) {
            // l = 16u + 4t .. 16u + 4t + 3 of half h: one word of each nibble plane half and of the bit-pair plane, per row
            const uint32_t qa0 = *reinterpret_cast<const uint32_t *>(ql0 + 64 * h + 16 * u + 4 * t);
            const uint32_t qb0 = *reinterpret_cast<const uint32_t *>(ql0 + 64 * h + 32 + 16 * u + 4 * t);
            const uint32_t hh0 = *reinterpret_cast<const uint32_t *>(qh0 + 32 * h + 16 * u + 4 * t);
            const uint32_t qa1 = *reinterpret_cast<const uint32_t *>(ql1 + 64 * h + 16 * u + 4 * t);
            const uint32_t qb1 = *reinterpret_cast<const uint32_t *>(ql1 + 64 * h + 32 + 16 * u + 4 * t);
            const uint32_t hh1 = *reinterpret_cast<const uint32_t *>(qh1 + 32 * h + 16 * u + 4 * t);
            uint32_t v0[4], v1[4];
            v0[0] = (qa0 & 0x0F0F0F0Fu) | ((hh0 << 4) & 0x30303030u);
            v0[1] = (qb0 & 0x0F0F0F0Fu) | ((hh0 << 2) & 0x30303030u);
            v0[2] = ((qa0 >> 4) & 0x0F0F0F0Fu) | (hh0 & 0x30303030u);
            v0[3] = ((qb0 >> 4) & 0x0F0F0F0Fu) | ((hh0 >> 2) & 0x30303030u);
            v1[0] = (qa1 & 0x0F0F0F0Fu) | ((hh1 << 4) & 0x30303030u);
            v1[1] = (qb1 & 0x0F0F0F0Fu) | ((hh1 << 2) & 0x30303030u);
            v1[2] = ((qa1 >> 4) & 0x0F0F0F0Fu) | (hh1 & 0x30303030u);
            v1[3] = ((qb1 >> 4) & 0x0F0F0F0Fu) | ((hh1 >> 2) & 0x30303030u);
#pragma unroll
            for (int j = 0; j < 4; j++) {
                const int grp = 8 * h + 2 * j + u;  // scale group = chunk of the super-block
                const uint2 b = *reinterpret_cast<const uint2 *>(bp + grp * cs);
                float d[4];
                mma_16816_z(d, v0[j] & 0x00FF00FFu, v1[j] & 0x00FF00FFu, (v0[j] >> 8) & 0x00FF00FFu, (v1[j] >> 8) & 0x00FF00FFu, b.x, b.y);
                const float off = -32.0f * sfp[grp * sfs];
                acc0 = fmaf(dsc[0][grp], (d[0] + d[1]) + off, acc0);
                acc1 = fmaf(dsc[1][grp], (d[2] + d[3]) + off, acc1);
            }
        }
    }
}

template <bool Q6>
__global__ void __launch_bounds__(kThreadsCta, 1)
qmv_kquant_batch_kernel(const __grid_constant__ KBatchParams p) {
    constexpr uint32_t kStageBytes = stage_bytes<Q6>();
    extern __shared__ __align__(128) unsigned char smem_raw[];
    yule_pdl_launch_dependents();

    const int lane = threadIdx.x & 31;
    const int group = threadIdx.x >> 8, wid = (threadIdx.x >> 5) & (kWarps - 1);
    const int g = lane >> 2, t = lane & 3;
    const uint32_t nb = p.nb;
    const uint32_t bpr = p.n_cols / 256;
    const uint32_t G = gridDim.x;
    const uint32_t first_tile = blockIdx.x + group * G, tile_stride = kGroups * G;
    const uint32_t my_tiles = p.n_tiles > first_tile ? (p.n_tiles - first_tile + tile_stride - 1) / tile_stride : 0;
    const uint32_t S = p.stages, chunks = p.chunks;
    const uint32_t total = my_tiles * chunks;  // 0: this group only helps with the activations

    const KBatchSmem sm = carve(smem_raw, p.n_cols, nb, (size_t)kGroups * S * kStageBytes);
    unsigned char *ring = sm.ring + (size_t)group * S * kStageBytes;
    const uint32_t ring_u32 = smem_u32(ring);
    const uint32_t bar0 = smem_u32(sm.bars + group * kMaxStages);
    uint32_t *cnt = sm.cnt + group * kMaxStages;

    // Warp 0 of each group sets the group's barriers up and starts the first copies; the other warps see both through
    // the CTA barriers of the activation staging, which they pass before their first wait.
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
            issue_stage<Q6>(p, first_tile + k * tile_stride, c, ring_u32 + n * kStageBytes, bar0 + 8 * n, lane);
            if (++c == chunks) {
                c = 0;
                k++;
            }
        }
    }

    if (!p.late_wait) yule_pdl_wait();  // the activations (and the residual) come from the previous kernel
    const uint32_t tid = threadIdx.x & (kWarps * 32 - 1);
    const float inv_scale = stage_x(sm, p.x, p.x_stride, nb, p.n_cols / 128, lane, tid >> 4, p.norm_w, p.eps);
    if (total == 0) return;

    // B column n = g carries vector g / 2 (hi for even g, lo for odd); columns past 2·nb read zeros
    const bool feeds = (uint32_t)g < 2 * nb;
    const unsigned char *b_base = feeds ? sm.xb + g * 32 + t * 8 : sm.zb;
    const uint32_t cs = feeds ? nb * 64u : 0u;
    const bool charge = (uint32_t)t < nb;  // this lane's D columns belong to vector t
    const float *sf_base = charge ? sm.sfb + t : reinterpret_cast<const float *>(sm.zb);
    const uint32_t sfs = charge ? 4u : 0u;
    const uint32_t n_warps_used = bpr < (uint32_t)kWarps ? bpr : (uint32_t)kWarps;
    float *part_base = sm.partial + (size_t)group * (2 * kWarps * 64);

    uint32_t ck = 0, cc = 0;
    float acc0 = 0.f, acc1 = 0.f;
    uint32_t slot = 0, phase = 0;
    for (uint32_t n = 0; n < total; n++) {
        const uint32_t bar = bar0 + 8 * slot;
        if (!ring_wait(bar, phase, p.status, p.wait_cycles)) return;  // all eight warps of the group wait on the same copy
        const uint32_t blk = cc * kStageBlocks + (uint32_t)wid;  // this warp's super-block of the row
        if (blk < bpr) {
            const unsigned char *st = ring + (size_t)slot * kStageBytes;
            const unsigned char *bp = b_base + (size_t)(blk * 16) * cs;
            const float *sfp = sf_base + (size_t)(blk * 16) * sfs;
            if (Q6)
                consume_q6k(st, g, wid, t, bp, cs, sfp, sfs, acc0, acc1);
            else
                consume_q4k(st + (uint32_t)g * kQ4RowPitch + (uint32_t)wid * 144u, t, bp, cs, sfp, sfs, acc0, acc1);
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
                issue_stage<Q6>(p, first_tile + nk * tile_stride, nc, ring_u32 + slot * kStageBytes, bar, lane);
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
                const uint32_t tile = first_tile + ck * tile_stride;
                uint32_t seg = 0;
                while (seg + 1 < p.n_seg && tile >= p.tile0[seg + 1]) seg++;
                const uint32_t row = (tile - p.tile0[seg]) * kStageRows + rr;
                if (row < p.n_rows[seg]) {
                    sacc = (sacc * 16777216.0f) * inv_scale;
                    const size_t o = (size_t)v * p.out_stride[seg] + row;
                    if (p.residual) sacc += p.residual[o];
                    p.out[seg][o] = sacc;
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

// Ring slots per group that fit beside the activation image of `nb` vectors.
uint32_t batch_stages(bool q6, uint32_t n_cols, uint32_t nb) {
    const size_t stage = q6 ? kQ6StageBytes : kQ4StageBytes;
    const size_t fixed = fixed_bytes(n_cols, nb);
    if (fixed + (size_t)kGroups * stage > kFullSmSmem) return 0;
    const size_t st = (kFullSmSmem - fixed) / ((size_t)kGroups * stage);
    return st > (size_t)kMaxStages ? (uint32_t)kMaxStages : (uint32_t)st;
}

// One launch over the columns [256·blk_off, 256·blk_off + part_cols) of every row of `n_seg` matrices that share their
// activations (same type, columns, vectors); `residual` is added to the results (single matrix only).
template <bool Q6>
cudaError_t launch_variant(const QmvArgs *segs, uint32_t n_seg, uint32_t nb, uint32_t stages, uint32_t blk_off, uint32_t part_cols,
                           const float *residual, int sm_count, cudaStream_t s) {
    const QmvArgs &a = segs[0];
    KBatchParams p = {};
    const uint32_t bpr = a.n_cols / 256;
    p.n_seg = n_seg;
    uint32_t tiles = 0;
    for (uint32_t i = 0; i < n_seg; i++) {
        const QmvArgs &g = segs[i];
        if (Q6) {
            const uint64_t rec = row_record_bytes(bpr);
            const uint64_t off[4] = {0, (uint64_t)bpr * 128, (uint64_t)bpr * 192, (uint64_t)bpr * 208};
            const uint64_t len[4] = {(uint64_t)bpr * 128, (uint64_t)bpr * 64, (uint64_t)bpr * 16, d_section_bytes(bpr)};
            const uint32_t pitch[4] = {kQlPitch, kQhPitch, kScPitch, kDPitch};
            for (int pl = 0; pl < 4; pl++) {
                cudaError_t me = cached_tensor_map_2d(g.planar + off[pl], 8, len[pl] / 8, g.n_rows, rec, pitch[pl] / 8, kStageRows, &p.map[i][pl]);
                if (me != cudaSuccess) return me;
            }
        } else {
            const uint64_t row_bytes = (uint64_t)bpr * 144;
            cudaError_t me = cached_tensor_map_2d(g.w, 8, row_bytes / 8, g.n_rows, row_bytes, kQ4RowPitch / 8, kStageRows, &p.map[i][0]);
            if (me != cudaSuccess) return me;
        }
        p.out[i] = g.out;
        p.n_rows[i] = g.n_rows;
        p.out_stride[i] = g.out_stride;
        p.tile0[i] = tiles;
        tiles += (g.n_rows + kStageRows - 1) / kStageRows;
    }
    for (uint32_t i = n_seg; i <= (uint32_t)kMaxSegs; i++) p.tile0[i] = tiles;
    p.x = a.x + (size_t)blk_off * 256;
    p.residual = residual;
    p.norm_w = a.norm_w;
    p.eps = a.eps;
    p.n_cols = part_cols;
    p.blk_off = blk_off;
    p.n_tiles = tiles;
    p.chunks = (part_cols / 256 + kStageBlocks - 1) / kStageBlocks;
    p.nb = nb;
    p.x_stride = a.x_stride;
    p.late_wait = (a.pdl && a.late_wait) ? 1u : 0u;
    p.status = a.status;
    p.wait_cycles = a.wait_cycles;
    uint32_t grid = (p.n_tiles + kGroups - 1) / kGroups;
    if (grid > (uint32_t)sm_count) grid = (uint32_t)sm_count;
    const uint32_t jobs_per_group = (p.n_tiles + kGroups * grid - 1) / (kGroups * grid);
    const uint32_t need = jobs_per_group * p.chunks;
    if (stages > need) stages = need;
    p.stages = stages;
    const size_t smem = (size_t)stages * kGroups * stage_bytes<Q6>() + fixed_bytes(part_cols, nb);
    auto kern = qmv_kquant_batch_kernel<Q6>;
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

// Columns one launch covers for `nb` vectors: all of them if their activation image leaves room for enough ring slots
// (three per group for Q4_K, two for Q6_K), else the largest multiple of a stage's 2048 columns that does; rows longer
// than that take several launches, each adding its columns' share to the result of the one before.  0: nothing fits.
uint32_t part_cols_for(bool q6, uint32_t n_cols, uint32_t nb) {
    const uint32_t want = q6 ? 2u : 3u;
    if (batch_stages(q6, n_cols, nb) >= want) return n_cols;
    const uint32_t step = kStageBlocks * 256;
    uint32_t best = 0;
    for (uint32_t c = step; c < n_cols; c += step)
        if (batch_stages(q6, c, nb) >= want) best = c;
    return best >= 2 * step ? best : 0;  // shorter parts would be mostly launch overhead
}

}  // namespace

uint32_t kquant_batch_width(const QmvArgs &a) {
    const bool q6 = a.type == YULE_DTYPE_Q6_K;
    if (!q6 && a.type != YULE_DTYPE_Q4_K) return 0;
    if (q6 && !a.planar) return 0;
    if (a.batch < 2 || a.n_cols == 0 || a.n_cols % 256 || a.n_rows == 0 || a.x_stride % 4) return 0;
    if (a.tp.push || a.tp.wait) return 0;  // fused exchanges stay with the one-vector kernels
    if ((reinterpret_cast<uintptr_t>(q6 ? (const void *)a.planar : (const void *)a.w) & 15) || (reinterpret_cast<uintptr_t>(a.x) & 15)) return 0;
    // the widest pass whose image fits whole; for longer rows the widest that fits in parts of at least two stages
    for (uint32_t nb = a.batch < 4 ? a.batch : 4; nb >= 2; nb--)
        if (part_cols_for(q6, a.n_cols, nb) == a.n_cols) return nb;
    if (a.norm_w) return 0;  // the RMSNorm prologue needs the whole row in one launch
    for (uint32_t nb = a.batch < 4 ? a.batch : 4; nb >= 2; nb--)
        if (part_cols_for(q6, a.n_cols, nb) != 0) return nb;
    return 0;
}

// Matrices that share their activations (Q/K/V, gate/up) as one launch: same format, columns, vectors, prologue.
bool kquant_batch_can_share(const QmvArgs *segs, uint32_t n_seg) {
    if (n_seg < 1 || n_seg > (uint32_t)kMaxSegs) return false;
    const QmvArgs &a = segs[0];
    const uint32_t nb = kquant_batch_width(a);
    if (nb < 2) return false;
    if (part_cols_for(a.type == YULE_DTYPE_Q6_K, a.n_cols, nb) != a.n_cols) return false;  // rows that need several launches: one matrix at a time
    for (uint32_t i = 1; i < n_seg; i++) {
        const QmvArgs &g = segs[i];
        if (g.type != a.type || g.n_cols != a.n_cols || g.x != a.x || g.batch != a.batch || g.x_stride != a.x_stride || g.norm_w != a.norm_w ||
            g.residual || a.residual || kquant_batch_width(g) != nb)
            return false;
    }
    return true;
}

cudaError_t launch_kquant_batch_shared(const QmvArgs *segs, uint32_t n_seg, int sm_count, cudaStream_t s, uint64_t *launches) {
    if (!kquant_batch_can_share(segs, n_seg)) return cudaErrorInvalidValue;
    // passes of up to four vectors over all the matrices
    const QmvArgs &a = segs[0];
    const bool q6 = a.type == YULE_DTYPE_Q6_K;
    uint32_t done = 0;
    while (done < a.batch) {
        QmvArgs part[kMaxSegs];
        for (uint32_t i = 0; i < n_seg; i++) {
            part[i] = segs[i];
            part[i].x = segs[i].x + (size_t)done * segs[i].x_stride;
            part[i].out = segs[i].out + (size_t)done * segs[i].out_stride;
            part[i].residual = segs[i].residual ? segs[i].residual + (size_t)done * segs[i].out_stride : nullptr;
            part[i].batch = a.batch - done;
        }
        const uint32_t nb = kquant_batch_width(part[0]);
        if (nb < 2) {  // one vector left: the one-vector kernels, matrix by matrix
            for (uint32_t i = 0; i < n_seg; i++) {
                cudaError_t e = launch_qmv(part[i], sm_count, s, launches);
                if (e != cudaSuccess) return e;
            }
            return cudaSuccess;
        }
        const uint32_t stages = batch_stages(q6, a.n_cols, nb);
        cudaError_t e = q6 ? launch_variant<true>(part, n_seg, nb, stages, 0, a.n_cols, part[0].residual, sm_count, s)
                           : launch_variant<false>(part, n_seg, nb, stages, 0, a.n_cols, part[0].residual, sm_count, s);
        if (e != cudaSuccess) return e;
        *launches += 1;
        done += nb;
    }
    return cudaSuccess;
}

cudaError_t launch_kquant_batch(const QmvArgs &a, uint32_t nb, int sm_count, cudaStream_t s, uint64_t *launches) {
    const bool q6 = a.type == YULE_DTYPE_Q6_K;
    if (nb < 2 || nb > 4) return cudaErrorInvalidValue;
    const uint32_t part = part_cols_for(q6, a.n_cols, nb);
    if (part == 0) return cudaErrorInvalidValue;
    // parts of equal length (in stages) rather than full parts and a short tail
    const uint32_t step = kStageBlocks * 256;
    const uint32_t n_parts = (a.n_cols + part - 1) / part;
    const uint32_t stages_total = (a.n_cols + step - 1) / step;
    uint32_t col = 0;
    for (uint32_t i = 0; i < n_parts; i++) {
        const uint32_t st = stages_total / n_parts + (i < stages_total % n_parts ? 1u : 0u);
        uint32_t cols = st * step;
        if (col + cols > a.n_cols) cols = a.n_cols - col;
        const uint32_t stages = batch_stages(q6, cols, nb);
        const float *residual = i == 0 ? a.residual : a.out;  // later parts add to what the earlier ones stored
        cudaError_t e = q6 ? launch_variant<true>(&a, 1, nb, stages, col / 256, cols, residual, sm_count, s)
                           : launch_variant<false>(&a, 1, nb, stages, col / 256, cols, residual, sm_count, s);
        if (e != cudaSuccess) return e;
        *launches += 1;
        col += cols;
    }
    return cudaSuccess;
}

}  // namespace yule
