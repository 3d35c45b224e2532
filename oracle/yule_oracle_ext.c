/* CPU restatement of Yule's remaining K-quant and legacy block formats (Q4_1, Q5_0, Q5_1, Q8_1,
 * Q2_K, Q3_K, Q5_K): per-block dequantisation and the scalar fused dot products, each f32
 * operation in the reference's order.  Test infrastructure only, like the rest of this folder.
 * Pinned by the known-answer tests of yule-core/src/dequant.rs:1405-1565,1598-1611. */
#include "yule_oracle.h"

#include <string.h>

static inline float ext_f16(const uint8_t *p, size_t off) {
    return yo_f16_to_f32((uint16_t)(p[off] | (p[off + 1] << 8)));
}
static inline uint32_t ext_u32(const uint8_t *p) {
    return (uint32_t)p[0] | ((uint32_t)p[1] << 8) | ((uint32_t)p[2] << 16) | ((uint32_t)p[3] << 24);
}
static inline int nibble_at(const uint8_t *qs, int i) { return (i & 1) ? (qs[i / 2] >> 4) : (qs[i / 2] & 0x0F); }

/* dequant.rs:91-101 */
void yo_dequant_q4_1(const uint8_t *b, float *out) {
    float d = ext_f16(b, 0), m = ext_f16(b, 2);
    for (int i = 0; i < 32; i++)
        out[i] = (float)nibble_at(b + 4, i) * d + m;
}

/* dequant.rs:106-119 */
void yo_dequant_q5_0(const uint8_t *b, float *out) {
    float d = ext_f16(b, 0);
    uint32_t qh = ext_u32(b + 2);
    for (int i = 0; i < 32; i++) {
        int q = (int)(((qh >> i) & 1) << 4) | nibble_at(b + 6, i);
        out[i] = ((float)q - 16.0f) * d;
    }
}

/* dequant.rs:124-138 */
void yo_dequant_q5_1(const uint8_t *b, float *out) {
    float d = ext_f16(b, 0), m = ext_f16(b, 2);
    uint32_t qh = ext_u32(b + 4);
    for (int i = 0; i < 32; i++) {
        int q = (int)(((qh >> i) & 1) << 4) | nibble_at(b + 8, i);
        out[i] = (float)q * d + m;
    }
}

/* dequant.rs:156-165 */
void yo_dequant_q8_1(const uint8_t *b, float *out) {
    float d = ext_f16(b, 0);
    for (int i = 0; i < 32; i++)
        out[i] = (float)(int8_t)b[4 + i] * d;
}

/* dequant.rs:196-214 */
void yo_dequant_q2_k(const uint8_t *b, float *out) {
    float d = ext_f16(b, 80), dmin = ext_f16(b, 82);
    for (int sb = 0; sb < 16; sb++) {
        float scale = (float)(b[sb] & 0x0F), mn = (float)(b[sb] >> 4);
        for (int k = 0; k < 16; k++) {
            int wi = sb * 16 + k;
            float q = (float)((b[16 + wi / 4] >> (2 * (wi % 4))) & 3);
            out[wi] = d * scale * q - dmin * mn;
        }
    }
}

/* dequant.rs:223-236: sixteen 6-bit scales, centred at 32 */
static void q3k_scales(const uint8_t *b, int8_t *scales) {
    for (int j = 0; j < 16; j++) {
        int lo = j < 8 ? (b[96 + j] & 0x0F) : (b[96 + j - 8] >> 4);
        int hi = (b[104 + j / 4] >> (2 * (j % 4))) & 3;
        scales[j] = (int8_t)((lo | (hi << 4)) - 32);
    }
}
static inline int q3k_q(const uint8_t *b, int wi) {
    int lo = (b[32 + wi / 4] >> (2 * (wi % 4))) & 3;
    int hi = (b[wi / 8] >> (wi % 8)) & 1;
    return (lo | (hi << 2)) - 4;
}

/* dequant.rs:219-251 */
void yo_dequant_q3_k(const uint8_t *b, float *out) {
    float d = ext_f16(b, 108);
    int8_t scales[16];
    q3k_scales(b, scales);
    for (int sb = 0; sb < 16; sb++) {
        float sc = (float)scales[sb];
        for (int k = 0; k < 16; k++) {
            int wi = sb * 16 + k;
            out[wi] = d * sc * (float)q3k_q(b, wi);
        }
    }
}

/* dequant.rs:297-338 */
void yo_dequant_q5_k(const uint8_t *b, float *out) {
    float d = ext_f16(b, 0), dmin = ext_f16(b, 2);
    uint8_t sc[8], mn[8];
    yo_extract_q4k_scales_mins(b + 4, sc, mn);
    const uint8_t *qh = b + 16;
    for (int j = 0; j < 4; j++) {
        const uint8_t *ql = b + 48 + 32 * j;
        for (int h = 0; h < 2; h++) {
            int is = 2 * j + h;
            float ds = d * (float)sc[is], ms = dmin * (float)mn[is];
            uint8_t u = (uint8_t)(1u << is);
            for (int l = 0; l < 32; l++) {
                int q = (h ? (ql[l] >> 4) : (ql[l] & 0xF)) + ((qh[l] & u) ? 16 : 0);
                out[64 * j + 32 * h + l] = (float)q * ds - ms;
            }
        }
    }
}

/* dequant.rs:1143-1157 */
float yo_vec_dot_q4_1(const uint8_t *b, const float *act) {
    float d = ext_f16(b, 0), m = ext_f16(b, 2), sum = 0.0f, act_sum = 0.0f;
    for (int i = 0; i < 32; i++) {
        sum += (float)nibble_at(b + 4, i) * act[i];
        act_sum += act[i];
    }
    return d * sum + m * act_sum;
}

/* dequant.rs:1160-1174 */
float yo_vec_dot_q5_0(const uint8_t *b, const float *act) {
    float d = ext_f16(b, 0), sum = 0.0f;
    uint32_t qh = ext_u32(b + 2);
    for (int i = 0; i < 32; i++) {
        int q = (int)(((qh >> i) & 1) << 4) | nibble_at(b + 6, i);
        sum += ((float)q - 16.0f) * act[i];
    }
    return sum * d;
}

/* dequant.rs:1177-1194 */
float yo_vec_dot_q5_1(const uint8_t *b, const float *act) {
    float d = ext_f16(b, 0), m = ext_f16(b, 2), sum = 0.0f, act_sum = 0.0f;
    uint32_t qh = ext_u32(b + 4);
    for (int i = 0; i < 32; i++) {
        int q = (int)(((qh >> i) & 1) << 4) | nibble_at(b + 8, i);
        sum += (float)q * act[i];
        act_sum += act[i];
    }
    return d * sum + m * act_sum;
}

/* dequant.rs:1197-1207 */
float yo_vec_dot_q8_1(const uint8_t *b, const float *act) {
    float d = ext_f16(b, 0), sum = 0.0f;
    for (int i = 0; i < 32; i++)
        sum += (float)(int8_t)b[4 + i] * act[i];
    return sum * d;
}

/* dequant.rs:1013-1041 */
float yo_vec_dot_q2_k(const uint8_t *b, const float *act) {
    float d = ext_f16(b, 80), dmin = ext_f16(b, 82), sum = 0.0f;
    for (int sb = 0; sb < 16; sb++) {
        float scale = (float)(b[sb] & 0x0F), mn = (float)(b[sb] >> 4), dot = 0.0f, act_sum = 0.0f;
        for (int k = 0; k < 16; k++) {
            int wi = sb * 16 + k;
            float q = (float)((b[16 + wi / 4] >> (2 * (wi % 4))) & 3);
            dot += q * act[wi];
            act_sum += act[wi];
        }
        sum += d * scale * dot - dmin * mn * act_sum;
    }
    return sum;
}

/* dequant.rs:1045-1084 */
float yo_vec_dot_q3_k(const uint8_t *b, const float *act) {
    float d = ext_f16(b, 108), sum = 0.0f;
    int8_t scales[16];
    q3k_scales(b, scales);
    for (int sb = 0; sb < 16; sb++) {
        float sc = (float)scales[sb], dot = 0.0f;
        for (int k = 0; k < 16; k++) {
            int wi = sb * 16 + k;
            dot += (float)q3k_q(b, wi) * act[wi];
        }
        sum += d * sc * dot;
    }
    return sum;
}

/* dequant.rs:1088-1140 */
float yo_vec_dot_q5_k(const uint8_t *b, const float *act) {
    float d = ext_f16(b, 0), dmin = ext_f16(b, 2), sum = 0.0f;
    uint8_t sc[8], mn[8];
    yo_extract_q4k_scales_mins(b + 4, sc, mn);
    const uint8_t *qh = b + 16;
    for (int j = 0; j < 4; j++) {
        const uint8_t *ql = b + 48 + 32 * j;
        for (int h = 0; h < 2; h++) {
            int is = 2 * j + h;
            float scale = d * (float)sc[is], mnv = dmin * (float)mn[is], dot = 0.0f, asum = 0.0f;
            uint8_t u = (uint8_t)(1u << is);
            for (int l = 0; l < 32; l++) {
                int q = (h ? (ql[l] >> 4) : (ql[l] & 0xF)) + ((qh[l] & u) ? 16 : 0);
                dot += (float)q * act[64 * j + 32 * h + l];
                asum += act[64 * j + 32 * h + l];
            }
            sum += scale * dot - mnv * asum;
        }
    }
    return sum;
}

int yo_ext_dequant_block(int type, const uint8_t *block, float *out) {
    switch (type) {
    case YO_Q4_1: yo_dequant_q4_1(block, out); return 0;
    case YO_Q5_0: yo_dequant_q5_0(block, out); return 0;
    case YO_Q5_1: yo_dequant_q5_1(block, out); return 0;
    case YO_Q8_1: yo_dequant_q8_1(block, out); return 0;
    case YO_Q2_K: yo_dequant_q2_k(block, out); return 0;
    case YO_Q3_K: yo_dequant_q3_k(block, out); return 0;
    case YO_Q5_K: yo_dequant_q5_k(block, out); return 0;
    default: return -1;
    }
}

int yo_ext_vec_dot_block(int type, const uint8_t *block, const float *act, float *out) {
    switch (type) {
    case YO_Q4_1: *out = yo_vec_dot_q4_1(block, act); return 0;
    case YO_Q5_0: *out = yo_vec_dot_q5_0(block, act); return 0;
    case YO_Q5_1: *out = yo_vec_dot_q5_1(block, act); return 0;
    case YO_Q8_1: *out = yo_vec_dot_q8_1(block, act); return 0;
    case YO_Q2_K: *out = yo_vec_dot_q2_k(block, act); return 0;
    case YO_Q3_K: *out = yo_vec_dot_q3_k(block, act); return 0;
    case YO_Q5_K: *out = yo_vec_dot_q5_k(block, act); return 0;
    default: return -1;
    }
}
