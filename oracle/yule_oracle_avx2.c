/*
 * yule_oracle_avx2.c — yule-core/src/simd/avx2.rs restated with the same
 * AVX2/FMA intrinsics.  TEST INFRASTRUCTURE ONLY (see yule_oracle.h); this is
 * also the CPU kernel that the timed baseline runs.
 *
 * Compile with -mavx2 -mfma -O2 -ffp-contract=off: the only fused
 * multiply-adds are the explicit _mm256_fmadd_ps calls, as in the Rust.
 */
#include "yule_oracle.h"

#include <immintrin.h>
#include <string.h>

int yo_have_avx2(void) {
    /* simd/mod.rs:26 is_x86_feature_detected!("avx2") && ("fma") */
    return __builtin_cpu_supports("avx2") && __builtin_cpu_supports("fma");
}

/* avx2.rs:9-19: (lo128 + hi128) → add upper pair onto lower pair → add lane 1
 * onto lane 0. */
static inline float hsum_avx2(__m256 v) {
    __m128 hi128 = _mm256_extractf128_ps(v, 1);
    __m128 lo128 = _mm256_castps256_ps128(v);
    __m128 sum128 = _mm_add_ps(lo128, hi128);
    __m128 hi64 = _mm_movehl_ps(sum128, sum128);
    __m128 sum64 = _mm_add_ps(sum128, hi64);
    __m128 hi32 = _mm_shuffle_ps(sum64, sum64, 0x55);
    __m128 sum32 = _mm_add_ss(sum64, hi32);
    return _mm_cvtss_f32(sum32);
}

static inline float rd_f16(const uint8_t *p, size_t off) {
    return yo_f16_to_f32((uint16_t)(p[off] | ((uint16_t)p[off + 1] << 8)));
}

/* avx2.rs:39-56: four groups of 8 int8 → i32 → f32, fmadd into one acc. */
float yo_vec_dot_q8_0_avx2(const uint8_t *block, const float *act) {
    float d = rd_f16(block, 0);
    const uint8_t *qs = block + 2;
    __m256 acc = _mm256_setzero_ps();
    for (int g = 0; g < 4; g++) {
        int off = g * 8;
        __m128i qi = _mm_loadl_epi64((const __m128i *)(qs + off));
        __m256 fl = _mm256_cvtepi32_ps(_mm256_cvtepi8_epi32(qi));
        __m256 a = _mm256_loadu_ps(act + off);
        acc = _mm256_fmadd_ps(fl, a, acc);
    }
    return hsum_avx2(acc) * d;
}

/* avx2.rs:60-83: nibbles unpacked one by one into an 8-float stack array
 * (interleaved order), minus 8.0, fmadd. */
float yo_vec_dot_q4_0_avx2(const uint8_t *block, const float *act) {
    float d = rd_f16(block, 0);
    const uint8_t *qs = block + 2;
    __m256 bias = _mm256_set1_ps(8.0f);
    __m256 acc = _mm256_setzero_ps();
    for (int g = 0; g < 4; g++) {
        int off = g * 4;
        float w[8];
        for (int i = 0; i < 4; i++) {
            uint8_t byte = qs[off + i];
            w[2 * i] = (float)(byte & 0x0F);
            w[2 * i + 1] = (float)(byte >> 4);
        }
        __m256 wv = _mm256_sub_ps(_mm256_loadu_ps(w), bias);
        __m256 a = _mm256_loadu_ps(act + g * 8);
        acc = _mm256_fmadd_ps(wv, a, acc);
    }
    return hsum_avx2(acc) * d;
}

/* avx2.rs:103-152: the Rust-intrinsic Q4_K kernel used when the assembly
 * kernel was not built (build.rs:9-16: no clang found). */
float yo_vec_dot_q4_k_avx2_rust(const uint8_t *block, const float *act) {
    float d = rd_f16(block, 0);
    float dmin = rd_f16(block, 2);
    uint8_t sc[8], mn[8];
    yo_extract_q4k_scales_mins(block + 4, sc, mn);
    float sum = 0.0f;
    for (int j = 0; j < 4; j++) {
        const uint8_t *ql = block + 16 + 32 * j;
        __m256 dot_acc = _mm256_setzero_ps();
        __m256 sum_acc = _mm256_setzero_ps();
        for (int g = 0; g < 4; g++) {
            int off = g * 8;
            float w[8];
            for (int l = 0; l < 8; l++)
                w[l] = (float)(ql[off + l] & 0xF);
            __m256 wv = _mm256_loadu_ps(w);
            __m256 a = _mm256_loadu_ps(act + 64 * j + off);
            dot_acc = _mm256_fmadd_ps(wv, a, dot_acc);
            sum_acc = _mm256_add_ps(sum_acc, a);
        }
        sum += d * (float)sc[2 * j] * hsum_avx2(dot_acc) -
               dmin * (float)mn[2 * j] * hsum_avx2(sum_acc);

        dot_acc = _mm256_setzero_ps();
        sum_acc = _mm256_setzero_ps();
        for (int g = 0; g < 4; g++) {
            int off = g * 8;
            float w[8];
            for (int l = 0; l < 8; l++)
                w[l] = (float)(ql[off + l] >> 4);
            __m256 wv = _mm256_loadu_ps(w);
            __m256 a = _mm256_loadu_ps(act + 64 * j + 32 + off);
            dot_acc = _mm256_fmadd_ps(wv, a, dot_acc);
            sum_acc = _mm256_add_ps(sum_acc, a);
        }
        sum += d * (float)sc[2 * j + 1] * hsum_avx2(dot_acc) -
               dmin * (float)mn[2 * j + 1] * hsum_avx2(sum_acc);
    }
    return sum;
}

/* avx2.rs:306-337: the "AVX2" Q6_K kernel is the scalar loop. */
float yo_vec_dot_q6_k_avx2(const uint8_t *block, const float *act) {
    return yo_vec_dot_q6_k(block, act);
}
