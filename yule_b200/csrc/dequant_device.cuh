// Per-element dequantisation of the block formats, bit-exact with yule-core/src/dequant.rs
// (each product and difference rounded separately, in the reference's order).  Shared by the
// whole-tensor dequantise / embedding kernels (qmv.cu) and the generic GEMM producer (qgemm_tc.cu).
#pragma once

#include <cstdint>

#include <cuda_fp16.h>

#include "../../include/yule_cuda.h"

namespace yule {
namespace {

__device__ __forceinline__ float f16_bits_to_f32(uint32_t bits) {
    // cvt.f32.f16 is exact for every finite half, subnormals included.
    return __half2float(__ushort_as_half((unsigned short)bits));
}

// Element i of a Q4_K super-block — dequant.rs:260-290.  d*sc, dmin*mn and q*(d*sc) are exact
// in f32, so the single rounding of the subtraction is the only one, as on the CPU.
__device__ __forceinline__ float dequant_q4k_elem(const uint8_t *bp, int i) {
    const float d = f16_bits_to_f32(bp[0] | (bp[1] << 8));
    const float dmin = f16_bits_to_f32(bp[2] | (bp[3] << 8));
    const int jg = i >> 6, hi = (i >> 5) & 1, l = i & 31;
    const int s = 2 * jg + hi;
    const uint8_t *q = bp + 4;
    uint32_t sc, mn;
    if (s < 4) {
        sc = q[s] & 63;
        mn = q[s + 4] & 63;
    } else {
        sc = (q[s + 4] & 0xF) | ((q[s - 4] >> 6) << 4);
        mn = (q[s + 4] >> 4) | ((q[s] >> 6) << 4);
    }
    const uint32_t nib = (bp[16 + 32 * jg + l] >> (4 * hi)) & 0xF;
    return __fsub_rn(__fmul_rn((float)nib, __fmul_rn(d, (float)sc)), __fmul_rn(dmin, (float)mn));
}

// Element i of a Q6_K super-block — dequant.rs:346-372, evaluated (d*sc)*q.
__device__ __forceinline__ float dequant_q6k_elem(const uint8_t *bp, int i) {
    const float d = f16_bits_to_f32(bp[208] | (bp[209] << 8));
    const int h = i >> 7, r = i & 127, g = r >> 5, l = r & 31;
    const uint32_t low4 = (bp[64 * h + l + 32 * (g & 1)] >> (4 * (g >> 1))) & 0xF;
    const uint32_t high2 = (bp[128 + 32 * h + l] >> (2 * g)) & 3;
    const int q = (int)(low4 | (high2 << 4)) - 32;
    const int sc = (int)(signed char)bp[192 + 8 * h + (l >> 4) + 2 * g];
    return __fmul_rn(__fmul_rn(d, (float)sc), (float)q);
}

// dequant.rs:77-86 (interleaved nibbles) and :142-150.
__device__ __forceinline__ float dequant_q4_0_elem(const uint8_t *bp, int i) {
    const float d = f16_bits_to_f32(bp[0] | (bp[1] << 8));
    const uint32_t byte = bp[2 + (i >> 1)];
    const uint32_t nib = (i & 1) ? (byte >> 4) : (byte & 0xF);
    return __fmul_rn(__fsub_rn((float)nib, 8.0f), d);
}
__device__ __forceinline__ float dequant_q8_0_elem(const uint8_t *bp, int i) {
    const float d = f16_bits_to_f32(bp[0] | (bp[1] << 8));
    return __fmul_rn((float)(int)(signed char)bp[2 + i], d);
}

// ── formats without a tuned kernel (Yule's CPU runner handles them, its GPU backends do not) ──
__device__ __forceinline__ uint32_t nibble_of(const uint8_t *qs, int i) {
    const uint32_t byte = qs[i >> 1];
    return (i & 1) ? (byte >> 4) : (byte & 0xF);
}
// dequant.rs:91-101: nibble*d + m, product and sum rounded separately.
__device__ __forceinline__ float dequant_q4_1_elem(const uint8_t *bp, int i) {
    const float d = f16_bits_to_f32(bp[0] | (bp[1] << 8)), m = f16_bits_to_f32(bp[2] | (bp[3] << 8));
    return __fadd_rn(__fmul_rn((float)nibble_of(bp + 4, i), d), m);
}
// dequant.rs:106-119: fifth bit from the 32-bit qh word.
__device__ __forceinline__ float dequant_q5_0_elem(const uint8_t *bp, int i) {
    const float d = f16_bits_to_f32(bp[0] | (bp[1] << 8));
    const uint32_t hi = (bp[2 + (i >> 3)] >> (i & 7)) & 1;
    const uint32_t q = (hi << 4) | nibble_of(bp + 6, i);
    return __fmul_rn(__fsub_rn((float)q, 16.0f), d);
}
// dequant.rs:124-138
__device__ __forceinline__ float dequant_q5_1_elem(const uint8_t *bp, int i) {
    const float d = f16_bits_to_f32(bp[0] | (bp[1] << 8)), m = f16_bits_to_f32(bp[2] | (bp[3] << 8));
    const uint32_t hi = (bp[4 + (i >> 3)] >> (i & 7)) & 1;
    const uint32_t q = (hi << 4) | nibble_of(bp + 8, i);
    return __fadd_rn(__fmul_rn((float)q, d), m);
}
// dequant.rs:156-165: the f16 sum at offset 2 is not used.
__device__ __forceinline__ float dequant_q8_1_elem(const uint8_t *bp, int i) {
    const float d = f16_bits_to_f32(bp[0] | (bp[1] << 8));
    return __fmul_rn((float)(int)(signed char)bp[4 + i], d);
}
// dequant.rs:196-214: (d*scale)*q - dmin*min, sixteen sub-blocks of 16.
__device__ __forceinline__ float dequant_q2k_elem(const uint8_t *bp, int i) {
    const float d = f16_bits_to_f32(bp[80] | (bp[81] << 8)), dmin = f16_bits_to_f32(bp[82] | (bp[83] << 8));
    const uint32_t s = bp[i >> 4];
    const uint32_t q = (bp[16 + (i >> 2)] >> (2 * (i & 3))) & 3;
    return __fsub_rn(__fmul_rn(__fmul_rn(d, (float)(s & 0xF)), (float)q), __fmul_rn(dmin, (float)(s >> 4)));
}
// dequant.rs:219-251: 6-bit scales centred at 32, 3-bit weights centred at 4, (d*sc)*q.
__device__ __forceinline__ float dequant_q3k_elem(const uint8_t *bp, int i) {
    const float d = f16_bits_to_f32(bp[108] | (bp[109] << 8));
    const int j = i >> 4;
    const uint32_t lo4 = j < 8 ? (bp[96 + j] & 0xF) : (bp[96 + j - 8] >> 4);
    const uint32_t hi2 = (bp[104 + (j >> 2)] >> (2 * (j & 3))) & 3;
    const int sc = (int)(lo4 | (hi2 << 4)) - 32;
    const uint32_t lo = (bp[32 + (i >> 2)] >> (2 * (i & 3))) & 3;
    const uint32_t hi = (bp[i >> 3] >> (i & 7)) & 1;
    const int q = (int)(lo | (hi << 2)) - 4;
    return __fmul_rn(__fmul_rn(d, (float)sc), (float)q);
}
// dequant.rs:297-338: Q4_K's scales and nibble groups plus one high bit per weight from qh.
__device__ __forceinline__ float dequant_q5k_elem(const uint8_t *bp, int i) {
    const float d = f16_bits_to_f32(bp[0] | (bp[1] << 8));
    const float dmin = f16_bits_to_f32(bp[2] | (bp[3] << 8));
    const int jg = i >> 6, hi = (i >> 5) & 1, l = i & 31;
    const int s = 2 * jg + hi;
    const uint8_t *q = bp + 4;
    uint32_t sc, mn;
    if (s < 4) {
        sc = q[s] & 63;
        mn = q[s + 4] & 63;
    } else {
        sc = (q[s + 4] & 0xF) | ((q[s - 4] >> 6) << 4);
        mn = (q[s + 4] >> 4) | ((q[s] >> 6) << 4);
    }
    const uint32_t nib = (bp[48 + 32 * jg + l] >> (4 * hi)) & 0xF;
    const uint32_t q5 = nib + (((bp[16 + l] >> s) & 1) << 4);
    return __fsub_rn(__fmul_rn((float)q5, __fmul_rn(d, (float)sc)), __fmul_rn(dmin, (float)mn));
}

// Element i of a row in one of those formats (i < row length).
template <uint32_t TYPE>
__device__ __forceinline__ float dequant_row_elem(const uint8_t *row, uint32_t i) {
    if (TYPE == YULE_DTYPE_Q4_1) return dequant_q4_1_elem(row + (size_t)(i >> 5) * 20, i & 31);
    if (TYPE == YULE_DTYPE_Q5_0) return dequant_q5_0_elem(row + (size_t)(i >> 5) * 22, i & 31);
    if (TYPE == YULE_DTYPE_Q5_1) return dequant_q5_1_elem(row + (size_t)(i >> 5) * 24, i & 31);
    if (TYPE == YULE_DTYPE_Q8_1) return dequant_q8_1_elem(row + (size_t)(i >> 5) * 36, i & 31);
    if (TYPE == YULE_DTYPE_Q2_K) return dequant_q2k_elem(row + (size_t)(i >> 8) * 84, i & 255);
    if (TYPE == YULE_DTYPE_Q3_K) return dequant_q3k_elem(row + (size_t)(i >> 8) * 110, i & 255);
    return dequant_q5k_elem(row + (size_t)(i >> 8) * 176, i & 255);
}

__device__ __forceinline__ float dequant_elem(const uint8_t *data, uint32_t type, uint64_t idx) {
    switch (type) {
        case YULE_DTYPE_Q4_K: return dequant_q4k_elem(data + (idx >> 8) * 144, (int)(idx & 255));
        case YULE_DTYPE_Q6_K: return dequant_q6k_elem(data + (idx >> 8) * 210, (int)(idx & 255));
        case YULE_DTYPE_Q4_0: return dequant_q4_0_elem(data + (idx >> 5) * 18, (int)(idx & 31));
        case YULE_DTYPE_Q8_0: return dequant_q8_0_elem(data + (idx >> 5) * 34, (int)(idx & 31));
        case YULE_DTYPE_Q4_1: return dequant_q4_1_elem(data + (idx >> 5) * 20, (int)(idx & 31));
        case YULE_DTYPE_Q5_0: return dequant_q5_0_elem(data + (idx >> 5) * 22, (int)(idx & 31));
        case YULE_DTYPE_Q5_1: return dequant_q5_1_elem(data + (idx >> 5) * 24, (int)(idx & 31));
        case YULE_DTYPE_Q8_1: return dequant_q8_1_elem(data + (idx >> 5) * 36, (int)(idx & 31));
        case YULE_DTYPE_Q2_K: return dequant_q2k_elem(data + (idx >> 8) * 84, (int)(idx & 255));
        case YULE_DTYPE_Q3_K: return dequant_q3k_elem(data + (idx >> 8) * 110, (int)(idx & 255));
        case YULE_DTYPE_Q5_K: return dequant_q5k_elem(data + (idx >> 8) * 176, (int)(idx & 255));
        case YULE_DTYPE_F16: return f16_bits_to_f32(data[2 * idx] | (data[2 * idx + 1] << 8));
        default: return reinterpret_cast<const float *>(data)[idx];
    }
}

}  // namespace
}  // namespace yule
