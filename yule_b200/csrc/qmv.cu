// qmv.cu — fused dequantise + dot matvec kernels over raw GGUF blocks, plus the standalone
// dequantiser and the embedding-row gather.
//
// Arithmetic contract (what the CPU code being replaced computes):
//   Q4_K  yule-core/src/dequant.rs:929-972   sum += (d*sc)*Σ q·x − (dmin*mn)*Σ x   per 32-column sub-block
//   Q6_K  yule-core/src/dequant.rs:976-1009  sum += d*sc*(q−32)*x                  per weight, 16-column scales
//   Q4_0  yule-core/src/dequant.rs:902-913   (Σ (nib−8)·x)*d, nibble i in byte i/2 (even=low, odd=high)
//   Q8_0  yule-core/src/dequant.rs:916-926   (Σ q·x)*d
// All accumulation is fp32; integer fields are turned into floats exactly (bit-spliced into a
// float or half whose value is 2^k + n, then one exact subtraction), never rounded.
//
// Data layout: weights stay exactly as in the GGUF file — row-major blocks, row r at byte
// r * (n_cols/block_size) * block_bytes.  The activation vector(s) are staged once per CTA into
// shared memory together with per-32-column sums (the Σx that every row of a Q4_K matrix shares).

#include <cuda_fp16.h>

#include "internal.h"
#include "dequant_device.cuh"

namespace yule {

namespace {

constexpr int kThreads = 256;
constexpr int kWarps = kThreads / 32;


// Streaming 128-bit load: weights are read exactly once, so keep them out of L1.
__device__ __forceinline__ uint4 ld_stream_u4(const uint4 *p) {
    uint4 v;
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
                 : "l"(p));
    return v;
}
__device__ __forceinline__ uint32_t ld_stream_u16(const uint8_t *p) {
    unsigned short v;
    asm volatile("ld.global.nc.u16 %0, [%1];" : "=h"(v) : "l"(p));
    return v;
}
__device__ __forceinline__ uint32_t ld_stream_u8(const uint8_t *p) {
    uint32_t v;
    asm volatile("ld.global.nc.u8 %0, [%1];" : "=r"(v) : "l"(p));
    return v;
}

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}

// byte `i` (0..11) of the 12 packed scale bytes held in three little-endian words.
__device__ __forceinline__ uint32_t scale_byte(uint32_t a, uint32_t b, uint32_t c, int i) {
    uint32_t w = (i < 4) ? a : ((i < 8) ? b : c);
    return (w >> (8 * (i & 3))) & 0xFFu;
}
// yule-core/src/dequant.rs:176-190 for one sub-block index s.
__device__ __forceinline__ void q4k_scale_min(uint32_t a, uint32_t b, uint32_t c, int s, uint32_t *sc,
                                              uint32_t *mn) {
    if (s < 4) {
        *sc = scale_byte(a, b, c, s) & 63u;
        *mn = scale_byte(a, b, c, s + 4) & 63u;
    } else {
        uint32_t hi = scale_byte(a, b, c, s + 4);
        *sc = (hi & 0xFu) | ((scale_byte(a, b, c, s - 4) >> 6) << 4);
        *mn = (hi >> 4) | ((scale_byte(a, b, c, s) >> 6) << 4);
    }
}

// Eight nibbles of one word → exact floats.  Low nibble of byte i → lo[i], high nibble → hi[i].
// (n | 0x6400) read as a half is 1024+n; (16n | 0x6400) is 1024+16n; one exact half op removes
// the offset.
// `bit_lo` / `bit_hi` carry a fifth bit per byte (bit 0 of each byte, Q5_K): +16 on the low-nibble
// value is mantissa bit 4 of 1024+n, +16 on the high-nibble value is bit 8 of 1024+16n.
__device__ __forceinline__ void nibbles_to_float(uint32_t w, float lo[4], float hi[4], uint32_t bit_lo = 0,
                                                 uint32_t bit_hi = 0) {
    const uint32_t magic = 0x64006400u;
    uint32_t w8 = w >> 8;
    uint32_t l02 = (w & 0x000F000Fu) | magic | ((bit_lo & 0x00010001u) << 4);
    uint32_t l13 = (w8 & 0x000F000Fu) | magic | (((bit_lo >> 8) & 0x00010001u) << 4);
    uint32_t h02 = (w & 0x00F000F0u) | magic | ((bit_hi & 0x00010001u) << 8);
    uint32_t h13 = (w8 & 0x00F000F0u) | magic | (((bit_hi >> 8) & 0x00010001u) << 8);
    const __half2 k1024 = __float2half2_rn(1024.0f);
    const __half2 k16th = __float2half2_rn(0.0625f);
    const __half2 k64 = __float2half2_rn(-64.0f);
    float2 a = __half22float2(__hsub2(*reinterpret_cast<__half2 *>(&l02), k1024));
    float2 b = __half22float2(__hsub2(*reinterpret_cast<__half2 *>(&l13), k1024));
    float2 c = __half22float2(__hfma2(*reinterpret_cast<__half2 *>(&h02), k16th, k64));
    float2 d = __half22float2(__hfma2(*reinterpret_cast<__half2 *>(&h13), k16th, k64));
    lo[0] = a.x; lo[2] = a.y; lo[1] = b.x; lo[3] = b.y;
    hi[0] = c.x; hi[2] = c.y; hi[1] = d.x; hi[3] = d.y;
}

// Byte k of `v` (0..255) minus `offset` as an exact float: splice the byte into the mantissa of
// 2^23, subtract 2^23 + offset.
template <int K>
__device__ __forceinline__ float byte_to_float(uint32_t v, float two23_plus_offset) {
    return __uint_as_float(__byte_perm(v, 0x4B000000u, 0x7440 | K)) - two23_plus_offset;
}

// ── activation staging ──────────────────────────────────────────────────────────────────────
// xs: NB vectors of n_cols floats, optionally padded by 4 floats per 32 (PAD) so that lanes
// that each own one 32-column block hit distinct banks; xsum: NB × n_cols/32 sums.
template <int NB, bool PAD>
__device__ __forceinline__ void stage_x(const float *__restrict__ x, uint32_t x_stride, uint32_t n_cols,
                                        float *xs, float *xsum, bool want_sums) {
    const uint32_t vstride = PAD ? (n_cols / 32) * 36 : n_cols;
    for (uint32_t i = threadIdx.x * 4; i < n_cols; i += blockDim.x * 4) {
#pragma unroll
        for (int b = 0; b < NB; b++) {
            float4 v = *reinterpret_cast<const float4 *>(x + (size_t)b * x_stride + i);
            uint32_t o = PAD ? (i / 32) * 36 + (i % 32) : i;
            *reinterpret_cast<float4 *>(xs + b * vstride + o) = v;
        }
    }
    __syncthreads();
    if (want_sums) {
        // one warp per 32-column group: lane i reads element i (no bank conflicts), shuffle tree
        const uint32_t n_sb = n_cols / 32;
        const int lane = threadIdx.x & 31;
        for (uint32_t s = threadIdx.x >> 5; s < n_sb * NB; s += blockDim.x >> 5) {
            uint32_t b = s / n_sb, sb = s % n_sb;
            float v = xs[b * vstride + (PAD ? sb * 36 : sb * 32) + lane];
            v = warp_sum(v);
            if (lane == 0) xsum[s] = v;
        }
        __syncthreads();
    }
}

// ── Q4_K ────────────────────────────────────────────────────────────────────────────────────
// Eight lanes share one 144-byte super-block: every lane reads the 16-byte header (one
// broadcast transaction) and one 16-byte slice of qs — 16 low-nibble columns and the 16
// high-nibble columns 32 further on.  A warp covers four consecutive super-blocks (576
// contiguous bytes) per step and walks one row; rows are dealt round-robin to warps.
// Q5: the 176-byte Q5_K super-block (dequant.rs:297-338) — same header, then 32 bytes of fifth
// bits (bit s of qh[l] belongs to sub-block s, column l) before the 128 bytes of nibbles.
template <int NB, bool Q5 = false>
__global__ void __launch_bounds__(kThreads)
qmv_q4k_kernel(const uint8_t *__restrict__ w, const float *__restrict__ x, float *__restrict__ out,
               uint32_t n_rows, uint32_t n_cols, uint32_t x_stride, uint32_t out_stride,
               const float *__restrict__ residual) {
    extern __shared__ __align__(16) float smem[];
    yule_pdl_launch_dependents();
    yule_pdl_wait();
    float *xs = smem;
    float *xsum = smem + (size_t)NB * n_cols;
    stage_x<NB, false>(x, x_stride, n_cols, xs, xsum, true);

    const uint32_t bpr = n_cols / 256;
    const uint32_t n_sb = n_cols / 32;
    const int lane = threadIdx.x & 31;
    const int sub = lane >> 3;  // which of the 4 super-blocks of this step
    const int j = lane & 7;     // which 16-byte slice of qs
    const int g = j >> 1;       // group of 64 columns
    const uint32_t warp = blockIdx.x * kWarps + (threadIdx.x >> 5);
    const uint32_t n_warps = gridDim.x * kWarps;

    for (uint32_t row = warp; row < n_rows; row += n_warps) {
        constexpr int kU4 = Q5 ? 11 : 9;  // 16-byte words per super-block
        const uint4 *rowp = reinterpret_cast<const uint4 *>(w + (size_t)row * bpr * (kU4 * 16));
        float acc[NB];
#pragma unroll
        for (int b = 0; b < NB; b++) acc[b] = 0.f;

        for (uint32_t blk0 = 0; blk0 < bpr; blk0 += 4) {
            const uint32_t blk = blk0 + sub;
            if (blk < bpr) {
                const uint4 *bp = rowp + (size_t)blk * kU4;
                const uint4 hdr = __ldg(bp);
                const uint4 q = ld_stream_u4(bp + (Q5 ? 3 : 1) + j);
                uint4 fifth = make_uint4(0, 0, 0, 0);
                if (Q5) fifth = __ldg(bp + 1 + (j & 1));
                const float d = f16_bits_to_f32(hdr.x & 0xFFFFu);
                const float dmin = f16_bits_to_f32(hdr.x >> 16);
                uint32_t sc0, mn0, sc1, mn1;
                q4k_scale_min(hdr.y, hdr.z, hdr.w, 2 * g, &sc0, &mn0);
                q4k_scale_min(hdr.y, hdr.z, hdr.w, 2 * g + 1, &sc1, &mn1);
                const float s0 = d * (float)sc0, s1 = d * (float)sc1;
                const float m0 = dmin * (float)mn0, m1 = dmin * (float)mn1;

                float lo[16], hi[16];
                const int sh = 2 * g;
                nibbles_to_float(q.x, lo + 0, hi + 0, fifth.x >> sh, fifth.x >> (sh + 1));
                nibbles_to_float(q.y, lo + 4, hi + 4, fifth.y >> sh, fifth.y >> (sh + 1));
                nibbles_to_float(q.z, lo + 8, hi + 8, fifth.z >> sh, fifth.z >> (sh + 1));
                nibbles_to_float(q.w, lo + 12, hi + 12, fifth.w >> sh, fifth.w >> (sh + 1));

                const uint32_t col = blk * 256 + 64 * g + 16 * (j & 1);
#pragma unroll
                for (int b = 0; b < NB; b++) {
                    const float4 *xl = reinterpret_cast<const float4 *>(xs + (size_t)b * n_cols + col);
                    const float4 *xh = reinterpret_cast<const float4 *>(xs + (size_t)b * n_cols + col + 32);
                    float dl = 0.f, dh = 0.f;
#pragma unroll
                    for (int v = 0; v < 4; v++) {
                        float4 a = xl[v], c = xh[v];
                        dl = fmaf(lo[4 * v + 0], a.x, dl);
                        dl = fmaf(lo[4 * v + 1], a.y, dl);
                        dl = fmaf(lo[4 * v + 2], a.z, dl);
                        dl = fmaf(lo[4 * v + 3], a.w, dl);
                        dh = fmaf(hi[4 * v + 0], c.x, dh);
                        dh = fmaf(hi[4 * v + 1], c.y, dh);
                        dh = fmaf(hi[4 * v + 2], c.z, dh);
                        dh = fmaf(hi[4 * v + 3], c.w, dh);
                    }
                    float t = fmaf(s0, dl, s1 * dh);
                    if ((j & 1) == 0) {
                        // The Σx of a whole 32-column sub-block is charged once, by the even lane.
                        const float *sx = xsum + (size_t)b * n_sb + blk * 8 + 2 * g;
                        t -= fmaf(m0, sx[0], m1 * sx[1]);
                    }
                    acc[b] += t;
                }
            }
        }
#pragma unroll
        for (int b = 0; b < NB; b++) {
            float v = warp_sum(acc[b]);
            if (lane == 0) {
                if (residual) v += residual[(size_t)b * out_stride + row];
                out[(size_t)b * out_stride + row] = v;
            }
        }
    }
}

// ── Q6_K ────────────────────────────────────────────────────────────────────────────────────
// Sixteen lanes share one 210-byte super-block; lane (h, i) owns columns 128h + 32g + 4i..4i+3
// for g = 0..3: two 4-byte pieces of ql, one of qh, the four scales of its 16-column groups.
// Blocks are only 2-byte aligned, so the pieces are fetched as 16-bit halves.
__device__ __forceinline__ uint32_t ld_u32_as_halves(const uint8_t *p) {
    return ld_stream_u16(p) | (ld_stream_u16(p + 2) << 16);
}

template <int NB>
__global__ void __launch_bounds__(kThreads)
qmv_q6k_kernel(const uint8_t *__restrict__ w, const float *__restrict__ x, float *__restrict__ out,
               uint32_t n_rows, uint32_t n_cols, uint32_t x_stride, uint32_t out_stride,
               const float *__restrict__ residual) {
    extern __shared__ __align__(16) float smem[];
    yule_pdl_launch_dependents();
    yule_pdl_wait();
    float *xs = smem;
    stage_x<NB, false>(x, x_stride, n_cols, xs, nullptr, false);

    const uint32_t bpr = n_cols / 256;
    const int lane = threadIdx.x & 31;
    const int sub = lane >> 4;      // which of the 2 super-blocks of this step
    const int h = (lane >> 3) & 1;  // half of the super-block (128 columns)
    const int i = lane & 7;         // columns 4i..4i+3 within each 32-column group
    const uint32_t warp = blockIdx.x * kWarps + (threadIdx.x >> 5);
    const uint32_t n_warps = gridDim.x * kWarps;

    for (uint32_t row = warp; row < n_rows; row += n_warps) {
        const uint8_t *rowp = w + (size_t)row * bpr * 210;
        float acc[NB];
#pragma unroll
        for (int b = 0; b < NB; b++) acc[b] = 0.f;

        for (uint32_t blk0 = 0; blk0 < bpr; blk0 += 2) {
            const uint32_t blk = blk0 + sub;
            if (blk < bpr) {
                const uint8_t *bp = rowp + (size_t)blk * 210;
                const uint32_t ql0 = ld_u32_as_halves(bp + 64 * h + 4 * i);
                const uint32_t ql1 = ld_u32_as_halves(bp + 64 * h + 32 + 4 * i);
                const uint32_t qh = ld_u32_as_halves(bp + 128 + 32 * h + 4 * i);
                const float d = f16_bits_to_f32(ld_stream_u16(bp + 208));
                const uint8_t *scp = bp + 192 + 8 * h + (i >> 2);
                float ds[4];
#pragma unroll
                for (int g = 0; g < 4; g++) ds[g] = d * (float)(int)(signed char)ld_stream_u8(scp + 2 * g);

                uint32_t qv[4];
                qv[0] = (ql0 & 0x0F0F0F0Fu) | ((qh << 4) & 0x30303030u);
                qv[1] = (ql1 & 0x0F0F0F0Fu) | ((qh << 2) & 0x30303030u);
                qv[2] = ((ql0 >> 4) & 0x0F0F0F0Fu) | (qh & 0x30303030u);
                qv[3] = ((ql1 >> 4) & 0x0F0F0F0Fu) | ((qh >> 2) & 0x30303030u);

                const float kOff = 8388608.0f + 32.0f;  // 2^23 + 32: yields q − 32 exactly
                const uint32_t col = blk * 256 + 128 * h + 4 * i;
#pragma unroll
                for (int b = 0; b < NB; b++) {
                    float t = 0.f;
#pragma unroll
                    for (int g = 0; g < 4; g++) {
                        const float4 a = *reinterpret_cast<const float4 *>(xs + (size_t)b * n_cols + col + 32 * g);
                        float s = byte_to_float<0>(qv[g], kOff) * a.x;
                        s = fmaf(byte_to_float<1>(qv[g], kOff), a.y, s);
                        s = fmaf(byte_to_float<2>(qv[g], kOff), a.z, s);
                        s = fmaf(byte_to_float<3>(qv[g], kOff), a.w, s);
                        t = fmaf(ds[g], s, t);
                    }
                    acc[b] += t;
                }
            }
        }
#pragma unroll
        for (int b = 0; b < NB; b++) {
            float v = warp_sum(acc[b]);
            if (lane == 0) {
                if (residual) v += residual[(size_t)b * out_stride + row];
                out[(size_t)b * out_stride + row] = v;
            }
        }
    }
}

// ── Q8_0 / Q4_0 ─────────────────────────────────────────────────────────────────────────────
// One lane per 32-weight block (34 or 18 bytes, 2-byte aligned): a warp step covers 32
// consecutive blocks, i.e. 1088 or 576 contiguous bytes.  Activations sit in shared memory with
// a 4-float pad after every 32 so the 32 lanes' float4 reads fall into distinct banks.
template <int NB, bool IS_Q8>
__global__ void __launch_bounds__(kThreads)
qmv_q32_kernel(const uint8_t *__restrict__ w, const float *__restrict__ x, float *__restrict__ out,
               uint32_t n_rows, uint32_t n_cols, uint32_t x_stride, uint32_t out_stride,
               const float *__restrict__ residual) {
    extern __shared__ __align__(16) float smem[];
    yule_pdl_launch_dependents();
    yule_pdl_wait();
    float *xs = smem;
    stage_x<NB, true>(x, x_stride, n_cols, xs, nullptr, false);

    constexpr int BB = IS_Q8 ? 34 : 18;
    const uint32_t bpr = n_cols / 32;
    const uint32_t vstride = bpr * 36;
    const int lane = threadIdx.x & 31;
    const uint32_t warp = blockIdx.x * kWarps + (threadIdx.x >> 5);
    const uint32_t n_warps = gridDim.x * kWarps;

    for (uint32_t row = warp; row < n_rows; row += n_warps) {
        const uint8_t *rowp = w + (size_t)row * bpr * BB;
        float acc[NB];
#pragma unroll
        for (int b = 0; b < NB; b++) acc[b] = 0.f;

        for (uint32_t blk = lane; blk < bpr; blk += 32) {
            const uint8_t *bp = rowp + (size_t)blk * BB;
            const float d = f16_bits_to_f32(ld_stream_u16(bp));
            float s[NB];
#pragma unroll
            for (int b = 0; b < NB; b++) s[b] = 0.f;
            if (IS_Q8) {
                const float kOff = 8388608.0f + 128.0f;  // (q ^ 0x80) is q + 128 as an unsigned byte
#pragma unroll
                for (int v = 0; v < 8; v++) {
                    uint32_t q4 = (ld_stream_u16(bp + 2 + 4 * v) | (ld_stream_u16(bp + 4 + 4 * v) << 16)) ^ 0x80808080u;
                    float f0 = byte_to_float<0>(q4, kOff), f1 = byte_to_float<1>(q4, kOff);
                    float f2 = byte_to_float<2>(q4, kOff), f3 = byte_to_float<3>(q4, kOff);
#pragma unroll
                    for (int b = 0; b < NB; b++) {
                        const float4 a = *reinterpret_cast<const float4 *>(xs + b * vstride + blk * 36 + 4 * v);
                        s[b] = fmaf(f0, a.x, s[b]);
                        s[b] = fmaf(f1, a.y, s[b]);
                        s[b] = fmaf(f2, a.z, s[b]);
                        s[b] = fmaf(f3, a.w, s[b]);
                    }
                }
            } else {
                const float kOff = 8388608.0f + 8.0f;  // nibble − 8
#pragma unroll
                for (int v = 0; v < 8; v++) {
                    // 16 bits = columns 4v..4v+3 in nibble order (low nibble of a byte comes first)
                    uint32_t q = ld_stream_u16(bp + 2 + 2 * v);
                    float f0 = __uint_as_float(0x4B000000u | (q & 0xFu)) - kOff;
                    float f1 = __uint_as_float(0x4B000000u | ((q >> 4) & 0xFu)) - kOff;
                    float f2 = __uint_as_float(0x4B000000u | ((q >> 8) & 0xFu)) - kOff;
                    float f3 = __uint_as_float(0x4B000000u | (q >> 12)) - kOff;
#pragma unroll
                    for (int b = 0; b < NB; b++) {
                        const float4 a = *reinterpret_cast<const float4 *>(xs + b * vstride + blk * 36 + 4 * v);
                        s[b] = fmaf(f0, a.x, s[b]);
                        s[b] = fmaf(f1, a.y, s[b]);
                        s[b] = fmaf(f2, a.z, s[b]);
                        s[b] = fmaf(f3, a.w, s[b]);
                    }
                }
            }
#pragma unroll
            for (int b = 0; b < NB; b++) acc[b] = fmaf(s[b], d, acc[b]);
        }
#pragma unroll
        for (int b = 0; b < NB; b++) {
            float v = warp_sum(acc[b]);
            if (lane == 0) {
                if (residual) v += residual[(size_t)b * out_stride + row];
                out[(size_t)b * out_stride + row] = v;
            }
        }
    }
}

// ── formats without a tuned kernel ──────────────────────────────────────────────────────────
// Eight consecutive weights of a row (columns 8·run .. 8·run+7, inside one sub-block of every
// format) with 16-bit loads: one header decode per call.  Rows start 2-byte aligned and every block
// size is even, so the 16-bit loads are aligned.  Same arithmetic as the per-element decoders.
template <uint32_t TYPE>
__device__ __forceinline__ void dequant8_row(const uint8_t *rowp, uint32_t run, float (&v)[8]) {
    if (TYPE == YULE_DTYPE_Q8_1) {
        const uint8_t *bp = rowp + (size_t)(run >> 2) * 36;
        const float d = f16_bits_to_f32(ld_stream_u16(bp));
#pragma unroll
        for (int k = 0; k < 4; k++) {
            const uint32_t w = ld_stream_u16(bp + 4 + (run & 3u) * 8 + 2 * k);
            v[2 * k] = (float)(int)(signed char)(w & 0xFFu) * d;
            v[2 * k + 1] = (float)(int)(signed char)(w >> 8) * d;
        }
    } else if (TYPE == YULE_DTYPE_Q4_1 || TYPE == YULE_DTYPE_Q5_0 || TYPE == YULE_DTYPE_Q5_1) {
        constexpr uint32_t BB = TYPE == YULE_DTYPE_Q4_1 ? 20 : TYPE == YULE_DTYPE_Q5_0 ? 22 : 24;
        constexpr bool HAS_M = TYPE != YULE_DTYPE_Q5_0, HAS_QH = TYPE != YULE_DTYPE_Q4_1;
        constexpr uint32_t QH = HAS_M ? 4 : 2, QS = QH + (HAS_QH ? 4 : 0);
        const uint8_t *bp = rowp + (size_t)(run >> 2) * BB;
        const uint32_t part = run & 3u;  // which 8 of the block's 32 weights
        const float d = f16_bits_to_f32(ld_stream_u16(bp));
        const float m = HAS_M ? f16_bits_to_f32(ld_stream_u16(bp + 2)) : 0.f;
        const uint32_t qh = HAS_QH ? ld_stream_u8(bp + QH + part) : 0u;
        const uint32_t qs = ld_stream_u16(bp + QS + part * 4) | (ld_stream_u16(bp + QS + part * 4 + 2) << 16);
#pragma unroll
        for (int k = 0; k < 8; k++) {
            const float q = (float)(((qs >> (4 * k)) & 0xFu) | (((qh >> k) & 1u) << 4));
            v[k] = HAS_M ? fmaf(q, d, m) : (q - 16.0f) * d;
        }
    } else if (TYPE == YULE_DTYPE_Q2_K) {
        const uint8_t *bp = rowp + (size_t)(run >> 5) * 84;
        const uint32_t i0 = (run & 31u) * 8;
        const uint32_t sm = ld_stream_u8(bp + (i0 >> 4));
        const float ds = f16_bits_to_f32(ld_stream_u16(bp + 80)) * (float)(sm & 0xFu);
        const float dm = f16_bits_to_f32(ld_stream_u16(bp + 82)) * (float)(sm >> 4);
        const uint32_t qs = ld_stream_u16(bp + 16 + (i0 >> 2));
#pragma unroll
        for (int k = 0; k < 8; k++) v[k] = fmaf(ds, (float)((qs >> (2 * k)) & 3u), -dm);
    } else if (TYPE == YULE_DTYPE_Q3_K) {
        const uint8_t *bp = rowp + (size_t)(run >> 5) * 110;
        const uint32_t i0 = (run & 31u) * 8, j = i0 >> 4;
        const uint32_t lo4 = j < 8 ? (ld_stream_u8(bp + 96 + j) & 0xFu) : (ld_stream_u8(bp + 88 + j) >> 4);
        const uint32_t hi2 = (ld_stream_u8(bp + 104 + (j >> 2)) >> (2 * (j & 3u))) & 3u;
        const float ds = f16_bits_to_f32(ld_stream_u16(bp + 108)) * (float)((int)(lo4 | (hi2 << 4)) - 32);
        const uint32_t qs = ld_stream_u16(bp + 32 + (i0 >> 2));
        const uint32_t hm = ld_stream_u8(bp + (i0 >> 3));
#pragma unroll
        for (int k = 0; k < 8; k++)
            v[k] = ds * (float)((int)(((qs >> (2 * k)) & 3u) | (((hm >> k) & 1u) << 2)) - 4);
    } else {
#pragma unroll
        for (int k = 0; k < 8; k++) v[k] = dequant_row_elem<TYPE>(rowp, run * 8 + k);
    }
}

// One warp per row, a lane per run of 8 consecutive columns (inside one sub-block of every
// format, so the scale decode is shared by the 8 weights), accumulated in f32.  Correct for any
// row length that is a multiple of the block size; not tuned: narrow loads and a scalar decode
// keep it far below the HBM roofline.
template <int NB, uint32_t TYPE>
__global__ void __launch_bounds__(kThreads)
qmv_elem_kernel(const uint8_t *__restrict__ w, const float *__restrict__ x, float *__restrict__ out,
                uint32_t n_rows, uint32_t n_cols, uint32_t x_stride, uint32_t out_stride,
                const float *__restrict__ residual) {
    extern __shared__ __align__(16) float smem[];
    yule_pdl_launch_dependents();
    yule_pdl_wait();
    float *xs = smem;
    stage_x<NB, false>(x, x_stride, n_cols, xs, nullptr, false);

    constexpr uint32_t BS = (TYPE == YULE_DTYPE_Q2_K || TYPE == YULE_DTYPE_Q3_K || TYPE == YULE_DTYPE_Q5_K) ? 256 : 32;
    constexpr uint32_t BB = TYPE == YULE_DTYPE_Q4_1 ? 20 : TYPE == YULE_DTYPE_Q5_0 ? 22 : TYPE == YULE_DTYPE_Q5_1 ? 24
                          : TYPE == YULE_DTYPE_Q8_1 ? 36 : TYPE == YULE_DTYPE_Q2_K ? 84 : TYPE == YULE_DTYPE_Q3_K ? 110 : 176;
    const size_t row_bytes = (size_t)(n_cols / BS) * BB;
    const uint32_t n_runs = n_cols / 8;
    const int lane = threadIdx.x & 31;
    const uint32_t warp = blockIdx.x * kWarps + (threadIdx.x >> 5);
    const uint32_t n_warps = gridDim.x * kWarps;

    for (uint32_t row = warp; row < n_rows; row += n_warps) {
        const uint8_t *rowp = w + (size_t)row * row_bytes;
        float acc[NB];
#pragma unroll
        for (int b = 0; b < NB; b++) acc[b] = 0.f;
        for (uint32_t run = lane; run < n_runs; run += 32) {
            float wv[8];
            dequant8_row<TYPE>(rowp, run, wv);
#pragma unroll
            for (int b = 0; b < NB; b++) {
                const float4 a0 = *reinterpret_cast<const float4 *>(xs + (size_t)b * n_cols + run * 8);
                const float4 a1 = *reinterpret_cast<const float4 *>(xs + (size_t)b * n_cols + run * 8 + 4);
                float s = acc[b];
                s = fmaf(wv[0], a0.x, s);
                s = fmaf(wv[1], a0.y, s);
                s = fmaf(wv[2], a0.z, s);
                s = fmaf(wv[3], a0.w, s);
                s = fmaf(wv[4], a1.x, s);
                s = fmaf(wv[5], a1.y, s);
                s = fmaf(wv[6], a1.z, s);
                s = fmaf(wv[7], a1.w, s);
                acc[b] = s;
            }
        }
#pragma unroll
        for (int b = 0; b < NB; b++) {
            float v = warp_sum(acc[b]);
            if (lane == 0) {
                if (residual) v += residual[(size_t)b * out_stride + row];
                out[(size_t)b * out_stride + row] = v;
            }
        }
    }
}

// ── launch plumbing ─────────────────────────────────────────────────────────────────────────

using QmvKernel = void (*)(const uint8_t *, const float *, float *, uint32_t, uint32_t, uint32_t, uint32_t,
                           const float *);

// `aligned`: the weights start on a 16-byte boundary (the Q5_K kernel reads 16-byte words).
template <int NB>
QmvKernel pick_kernel(uint32_t type, bool aligned) {
    if (type == YULE_DTYPE_Q5_K && aligned) return qmv_q4k_kernel<NB, true>;
    switch (type) {
        case YULE_DTYPE_Q4_K: return qmv_q4k_kernel<NB>;
        case YULE_DTYPE_Q6_K: return qmv_q6k_kernel<NB>;
        case YULE_DTYPE_Q8_0: return qmv_q32_kernel<NB, true>;
        case YULE_DTYPE_Q4_0: return qmv_q32_kernel<NB, false>;
        case YULE_DTYPE_Q4_1: return qmv_elem_kernel<NB, YULE_DTYPE_Q4_1>;
        case YULE_DTYPE_Q5_0: return qmv_elem_kernel<NB, YULE_DTYPE_Q5_0>;
        case YULE_DTYPE_Q5_1: return qmv_elem_kernel<NB, YULE_DTYPE_Q5_1>;
        case YULE_DTYPE_Q8_1: return qmv_elem_kernel<NB, YULE_DTYPE_Q8_1>;
        case YULE_DTYPE_Q2_K: return qmv_elem_kernel<NB, YULE_DTYPE_Q2_K>;
        case YULE_DTYPE_Q3_K: return qmv_elem_kernel<NB, YULE_DTYPE_Q3_K>;
        case YULE_DTYPE_Q5_K: return qmv_elem_kernel<NB, YULE_DTYPE_Q5_K>;
        default: return nullptr;
    }
}

size_t qmv_smem_bytes(uint32_t type, uint32_t n_cols, int nb) {
    size_t per_vec;
    if (type == YULE_DTYPE_Q4_K || type == YULE_DTYPE_Q5_K)
        per_vec = (size_t)n_cols + n_cols / 32;
    else if (type == YULE_DTYPE_Q6_K || !is_tuned_format(type))
        per_vec = n_cols;
    else
        per_vec = (size_t)(n_cols / 32) * 36;
    return per_vec * nb * sizeof(float);
}

constexpr size_t kMaxSmem = 200 * 1024;

}  // namespace

cudaError_t launch_qmv(const QmvArgs &a, int sm_count, cudaStream_t s, uint64_t *launches) {
    // Q4_K / Q6_K, several vectors: two to four per pass of the batched ring kernel (YULE_QMV_KBATCH=0: the older paths);
    // a single left-over vector goes through the one-vector routing below
    if (a.batch >= 2 && kquant_batch_width(a) >= 2 && !(knob("YULE_QMV_KBATCH") && atoi(knob("YULE_QMV_KBATCH")) == 0)) {
        uint32_t done = 0;
        while (done < a.batch) {
            QmvArgs part = a;
            part.x = a.x + (size_t)done * a.x_stride;
            part.out = a.out + (size_t)done * a.out_stride;
            part.residual = a.residual ? a.residual + (size_t)done * a.out_stride : nullptr;
            part.batch = a.batch - done;
            const uint32_t nb = kquant_batch_width(part);
            if (nb < 2) return launch_qmv(part, sm_count, s, launches);  // one vector left
            cudaError_t e = launch_kquant_batch(part, nb, sm_count, s, launches);
            if (e != cudaSuccess) return e;
            done += nb;
        }
        return cudaSuccess;
    }
    const bool q5_mma = a.type == YULE_DTYPE_Q5_K && (reinterpret_cast<uintptr_t>(a.w) & 15) == 0 && !a.tp.push && !a.tp.wait;
    if ((a.type == YULE_DTYPE_Q4_K || q5_mma) && q4k_mma_supported(a.n_cols, 1)) {
        // tensor-pipe path, up to four activation vectors per pass over the weights
        uint32_t done = 0;
        while (done < a.batch) {
            uint32_t nb = a.batch - done < 4 ? a.batch - done : 4;
            while (!q4k_mma_supported(a.n_cols, nb)) nb--;
            Q4kFused f;
            f.w[0] = a.w;
            f.out[0] = a.out + (size_t)done * a.out_stride;
            f.rows[0] = a.n_rows;
            f.out_stride[0] = a.out_stride;
            f.n_seg = 1;
            f.q5 = q5_mma;
            f.x = a.x + (size_t)done * a.x_stride;
            f.x_stride = a.x_stride;
            f.n_cols = a.n_cols;
            f.batch = nb;
            f.residual = a.residual ? a.residual + (size_t)done * a.out_stride : nullptr;
            f.norm_w = a.norm_w;
            f.eps = a.eps;
            f.pdl = a.pdl;
            f.late_wait = a.late_wait;
            f.tp = a.tp;
            f.status = a.status;
            f.wait_cycles = a.wait_cycles;
            for (int i = 0; i < 2; i++) {
                f.next_w[i] = a.next_w[i];
                f.next_bytes[i] = a.next_bytes[i];
            }
            cudaError_t e = launch_q4k_mma(f, sm_count, s, launches);
            if (e != cudaSuccess) return e;
            done += nb;
        }
        return cudaSuccess;
    }
    if (a.type == YULE_DTYPE_Q6_K && a.planar && a.batch > 1 && a.batch <= 8 && q6k_mma_supported(a.n_cols) && q6k_stream_supported(a.n_cols)) {
        // rows too long for the batched kernel's activation image: one pass of the one-vector kernel per vector
        for (uint32_t b = 0; b < a.batch; b++) {
            QmvArgs one = a;
            one.x = a.x + (size_t)b * a.x_stride;
            one.out = a.out + (size_t)b * a.out_stride;
            one.residual = a.residual ? a.residual + (size_t)b * a.out_stride : nullptr;
            one.batch = 1;
            cudaError_t e = launch_qmv(one, sm_count, s, launches);
            if (e != cudaSuccess) return e;
        }
        return cudaSuccess;
    }
    if (a.type == YULE_DTYPE_Q6_K && a.planar && a.batch == 1 && q6k_mma_supported(a.n_cols) && q6k_stream_supported(a.n_cols)) {
        Q6kPlanar f;
        f.planar = a.planar;
        f.out = a.out;
        f.n_rows = a.n_rows;
        f.n_cols = a.n_cols;
        f.x = a.x;
        f.norm_w = a.norm_w;
        f.eps = a.eps;
        f.residual = a.residual;
        f.pdl = a.pdl;
        f.late_wait = a.late_wait;
        f.status = a.status;
        f.wait_cycles = a.wait_cycles;
        // independent call → ring kernel (overlaps with its predecessor; measured against the streaming kernel: 5.1 / 6.7 µs at
        // 4096x4096, 12.7 / 14.5 at 14336x4096, 93 / 91 at 128256x4096); dependent chain or very long matrix → streaming kernel
        bool ring = a.pdl && a.late_wait && (a.n_rows + 15) / 16 <= 8u * (uint32_t)sm_count;
        if (const char *k = knob("YULE_QMV_RING")) ring = atoi(k) != 0;
        return ring ? launch_q6k_mma(f, sm_count, s, launches) : launch_q6k_stream(f, sm_count, s, launches);
    }
    // Q8_0 / Q4_0, one vector, 256-column multiples: the tensor-pipe ring kernel (YULE_QMV_Q8Q4_RING=0: the SIMT kernel)
    if (q8q4_ring_supported(a) && !(knob("YULE_QMV_Q8Q4_RING") && atoi(knob("YULE_QMV_Q8Q4_RING")) == 0))
        return launch_q8q4_ring(a, sm_count, s, launches);
    // Q8_0 / Q4_0, several vectors: two to four per pass of the batched ring kernel, a single left-over vector on the
    // one-vector kernel
    if (q8q4_ring_batch_width(a) >= 2 && !(knob("YULE_QMV_Q8Q4_RING") && atoi(knob("YULE_QMV_Q8Q4_RING")) == 0)) {
        uint32_t done = 0;
        while (done < a.batch) {
            QmvArgs part = a;
            part.x = a.x + (size_t)done * a.x_stride;
            part.out = a.out + (size_t)done * a.out_stride;
            part.residual = a.residual ? a.residual + (size_t)done * a.out_stride : nullptr;
            part.batch = a.batch - done;
            const uint32_t nb = q8q4_ring_batch_width(part);
            cudaError_t e;
            if (nb >= 2) {
                e = launch_q8q4_ring_batch(part, nb, sm_count, s, launches);
                done += nb;
            } else {
                part.batch = 1;
                if (!q8q4_ring_supported(part)) break;  // the SIMT kernels below take the rest
                e = launch_q8q4_ring(part, sm_count, s, launches);
                done += 1;
            }
            if (e != cudaSuccess) return e;
        }
        if (done == a.batch) return cudaSuccess;
        QmvArgs rest = a;
        rest.x = a.x + (size_t)done * a.x_stride;
        rest.out = a.out + (size_t)done * a.out_stride;
        rest.residual = a.residual ? a.residual + (size_t)done * a.out_stride : nullptr;
        rest.batch = a.batch - done;
        return launch_qmv(rest, sm_count, s, launches);
    }
    if (qmv_smem_bytes(a.type, a.n_cols, 1) > kMaxSmem) return cudaErrorInvalidValue;
    uint32_t done = 0;
    while (done < a.batch) {
        int nb = 1;
        uint32_t left = a.batch - done;
        if (left >= 4 && qmv_smem_bytes(a.type, a.n_cols, 4) <= kMaxSmem)
            nb = 4;
        else if (left >= 2 && qmv_smem_bytes(a.type, a.n_cols, 2) <= kMaxSmem)
            nb = 2;
        const bool aligned = (reinterpret_cast<uintptr_t>(a.w) & 15) == 0;
        QmvKernel k = nb == 4 ? pick_kernel<4>(a.type, aligned) : nb == 2 ? pick_kernel<2>(a.type, aligned)
                                                                           : pick_kernel<1>(a.type, aligned);
        if (!k) return cudaErrorInvalidValue;
        size_t smem = qmv_smem_bytes(a.type, a.n_cols, nb);
        // attribute and occupancy are per (kernel, smem): remember the last answer per kernel
        struct Cached {
            QmvKernel k = nullptr;
            size_t smem = 0;
            int occ = 0;
        };
        static Cached cache[48];
        static std::mutex cache_mu;
        int occ = 0;
        {
            std::lock_guard<std::mutex> lock(cache_mu);
            Cached *slot = nullptr;
            for (auto &c : cache)
                if (c.k == k || c.k == nullptr) {
                    slot = &c;
                    break;
                }
            if (slot && slot->k == k && slot->smem == smem) {
                occ = slot->occ;
            } else {
                cudaError_t e = cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kMaxSmem);
                if (e != cudaSuccess) return e;
                e = cudaOccupancyMaxActiveBlocksPerMultiprocessor(&occ, k, kThreads, smem);
                if (e != cudaSuccess) return e;
                if (occ < 1) occ = 1;
                if (slot) {
                    slot->k = k;
                    slot->smem = smem;
                    slot->occ = occ;
                }
            }
        }
        uint32_t max_ctas = (uint32_t)(sm_count * occ);
        uint32_t want = (a.n_rows + kWarps - 1) / kWarps;
        uint32_t grid = want < max_ctas ? want : max_ctas;
        cudaError_t e = launch_kernel(k, dim3(grid), dim3(kThreads), smem, s, a.pdl, a.w,
                                      a.x + (size_t)done * a.x_stride, a.out + (size_t)done * a.out_stride, a.n_rows,
                                      a.n_cols, a.x_stride, a.out_stride,
                                      a.residual ? a.residual + (size_t)done * a.out_stride : (const float *)nullptr);
        if (e != cudaSuccess) return e;
        *launches += 1;
        done += nb;
    }
    return cudaSuccess;
}

// ── standalone dequantiser (bit-exact with yule-core/src/dequant.rs) ────────────────────────
namespace {


__global__ void dequantize_kernel(const uint8_t *__restrict__ data, uint32_t type, uint64_t n, float *__restrict__ out) {
    for (uint64_t i = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (uint64_t)gridDim.x * blockDim.x)
        out[i] = dequant_elem(data, type, i);
}

__global__ void embed_gather_kernel(const uint8_t *__restrict__ table, uint32_t type, uint32_t dim, uint32_t token,
                                    const uint32_t *__restrict__ token_ptr, uint64_t row_bytes,
                                    float *__restrict__ out) {
    yule_pdl_launch_dependents();
    yule_pdl_wait();
    const uint32_t tok = token_ptr ? *token_ptr : token;
    const uint8_t *row = table + (uint64_t)tok * row_bytes;
    for (uint32_t i = blockIdx.x * blockDim.x + threadIdx.x; i < dim; i += gridDim.x * blockDim.x)
        out[i] = dequant_elem(row, type, i);
}

// Rows tokens[0..n) of a [vocab][dim] table into out[n][dim]; blockIdx.y is the token slot.
__global__ void embed_gather_batch_kernel(const uint8_t *__restrict__ table, uint32_t type, uint32_t dim,
                                          const uint32_t *__restrict__ tokens, uint64_t row_bytes, float *__restrict__ out) {
    const uint8_t *row = table + (uint64_t)tokens[blockIdx.y] * row_bytes;
    float *o = out + (size_t)blockIdx.y * dim;
    for (uint32_t i = blockIdx.x * blockDim.x + threadIdx.x; i < dim; i += gridDim.x * blockDim.x) o[i] = dequant_elem(row, type, i);
}

}  // namespace

cudaError_t launch_embed_gather_batch(const uint8_t *table, uint32_t type, uint32_t dim, const uint32_t *tokens,
                                      uint32_t n_tokens, float *out, cudaStream_t s, uint64_t *launches) {
    uint64_t row_bytes = (uint64_t)(dim / block_size(type)) * block_bytes(type);
    *launches += 1;
    embed_gather_batch_kernel<<<dim3((dim + 255) / 256, n_tokens), 256, 0, s>>>(table, type, dim, tokens, row_bytes, out);
    return cudaGetLastError();
}

cudaError_t launch_dequantize(const uint8_t *w, uint32_t type, uint64_t n_blocks, float *out, cudaStream_t s,
                              uint64_t *launches) {
    uint64_t n = n_blocks * block_size(type);
    uint64_t grid = (n + 255) / 256;
    if (grid > 148 * 16) grid = 148 * 16;
    dequantize_kernel<<<(uint32_t)grid, 256, 0, s>>>(w, type, n, out);
    *launches += 1;
    return cudaGetLastError();
}

cudaError_t launch_embed_gather(const uint8_t *table, uint32_t type, uint32_t dim, uint32_t token,
                                const uint32_t *token_ptr, float *out, cudaStream_t s, uint64_t *launches, bool pdl) {
    uint64_t row_bytes = (uint64_t)(dim / block_size(type)) * block_bytes(type);
    *launches += 1;
    return launch_kernel(embed_gather_kernel, dim3((dim + 255) / 256), dim3(256), 0, s, pdl, table, type, dim, token,
                         token_ptr, row_bytes, out);
}

}  // namespace yule
