// Per-element dequantisation of the four block formats, bit-exact with yule-core/src/dequant.rs
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

__device__ __forceinline__ float dequant_elem(const uint8_t *data, uint32_t type, uint64_t idx) {
    switch (type) {
        case YULE_DTYPE_Q4_K: return dequant_q4k_elem(data + (idx >> 8) * 144, (int)(idx & 255));
        case YULE_DTYPE_Q6_K: return dequant_q6k_elem(data + (idx >> 8) * 210, (int)(idx & 255));
        case YULE_DTYPE_Q4_0: return dequant_q4_0_elem(data + (idx >> 5) * 18, (int)(idx & 31));
        case YULE_DTYPE_Q8_0: return dequant_q8_0_elem(data + (idx >> 5) * 34, (int)(idx & 31));
        case YULE_DTYPE_F16: return f16_bits_to_f32(data[2 * idx] | (data[2 * idx + 1] << 8));
        default: return reinterpret_cast<const float *>(data)[idx];
    }
}

}  // namespace
}  // namespace yule
