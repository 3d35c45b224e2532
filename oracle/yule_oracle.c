/*
 * yule_oracle.c — scalar CPU restatement of Yule's quantized-inference path.
 *
 * TEST INFRASTRUCTURE ONLY (see yule_oracle.h).  Each function names the Yule
 * source lines whose arithmetic — including the order of every f32 operation —
 * it reproduces.  Compile with -O2 -ffp-contract=off -fno-fast-math.
 */
#define _GNU_SOURCE
#include "yule_oracle.h"

#include <math.h>
#include <pthread.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>
#include <unistd.h>

/* ───────────────────────── format registry ───────────────────────── */

/* yule-core/src/dtype.rs:99-118 */
int yo_block_size(int type) {
    switch (type) {
    case YO_F32:
    case YO_F16:
        return 1;
    case YO_Q4_0:
    case YO_Q4_1:
    case YO_Q5_0:
    case YO_Q5_1:
    case YO_Q8_0:
    case YO_Q8_1:
        return 32;
    case YO_Q2_K:
    case YO_Q3_K:
    case YO_Q4_K:
    case YO_Q5_K:
    case YO_Q6_K:
        return 256;
    default:
        return 0;
    }
}

/* yule-core/src/dtype.rs:62-96 */
int yo_block_bytes(int type) {
    switch (type) {
    case YO_F32:
        return 4;
    case YO_F16:
        return 2;
    case YO_Q4_0:
        return 18;
    case YO_Q8_0:
        return 34;
    case YO_Q4_K:
        return 144;
    case YO_Q6_K:
        return 210;
    case YO_Q4_1:
        return 20;
    case YO_Q5_0:
        return 22;
    case YO_Q5_1:
        return 24;
    case YO_Q8_1:
        return 36;
    case YO_Q2_K:
        return 84;
    case YO_Q3_K:
        return 110;
    case YO_Q5_K:
        return 176;
    default:
        return 0;
    }
}

/* ───────────────────────── f16 → f32 ───────────────────────── */

static inline float bits_to_f32(uint32_t b) {
    float f;
    memcpy(&f, &b, 4);
    return f;
}

/* yule-core/src/dequant.rs:20-49: sign/exponent/mantissa split, subnormals
 * renormalised by shifting, inf/NaN keep the mantissa payload << 13. */
float yo_f16_to_f32(uint16_t h) {
    uint32_t sign = (uint32_t)(h >> 15) & 1u;
    uint32_t ex = (uint32_t)(h >> 10) & 0x1Fu;
    uint32_t man = (uint32_t)h & 0x3FFu;
    if (ex == 0) {
        if (man == 0)
            return bits_to_f32(sign << 31);
        int32_t e = -14;
        while ((man & 0x400u) == 0) {
            man <<= 1;
            e -= 1;
        }
        man &= 0x3FFu;
        uint32_t fe = (uint32_t)(e + 127) & 0xFFu;
        return bits_to_f32((sign << 31) | (fe << 23) | (man << 13));
    }
    if (ex == 31)
        return bits_to_f32((sign << 31) | (0xFFu << 23) | (man << 13));
    uint32_t fe = (uint32_t)((int32_t)ex - 15 + 127);
    return bits_to_f32((sign << 31) | (fe << 23) | (man << 13));
}

/* dequant.rs:59 read_f16 */
static inline float rd_f16(const uint8_t *p, size_t off) {
    uint16_t b = (uint16_t)(p[off] | ((uint16_t)p[off + 1] << 8));
    return yo_f16_to_f32(b);
}

/* ───────────────────────── block dequantisers ───────────────────────── */

/* dequant.rs:77-86 — nibble i lives in byte i/2; even i = low nibble, odd i =
 * high nibble (Yule's interleaved order, not ggml's split order). */
void yo_dequant_q4_0(const uint8_t *block, float *out) {
    float d = rd_f16(block, 0);
    for (int i = 0; i < 32; i++) {
        uint8_t byte = block[2 + i / 2];
        uint8_t nib = (i % 2 == 0) ? (uint8_t)(byte & 0x0F) : (uint8_t)(byte >> 4);
        out[i] = ((float)nib - 8.0f) * d;
    }
}

/* dequant.rs:142-150 */
void yo_dequant_q8_0(const uint8_t *block, float *out) {
    float d = rd_f16(block, 0);
    for (int i = 0; i < 32; i++) {
        int8_t q = (int8_t)block[2 + i];
        out[i] = (float)q * d;
    }
}

/* dequant.rs:176-190 */
void yo_extract_q4k_scales_mins(const uint8_t *q, uint8_t *sc, uint8_t *mn) {
    for (int j = 0; j < 4; j++) {
        sc[j] = q[j] & 63;
        mn[j] = q[j + 4] & 63;
    }
    for (int j = 4; j < 8; j++) {
        sc[j] = (uint8_t)((q[j + 4] & 0xF) | ((q[j - 4] >> 6) << 4));
        mn[j] = (uint8_t)((q[j + 4] >> 4) | ((q[j] >> 6) << 4));
    }
}

/* dequant.rs:260-290: d@0, dmin@2, scales@4..16, qs@16..144; group j of 64
 * weights takes low nibbles of qs[32j..32j+32) then high nibbles. */
void yo_dequant_q4_k(const uint8_t *block, float *out) {
    float d = rd_f16(block, 0);
    float dmin = rd_f16(block, 2);
    uint8_t sc[8], mn[8];
    yo_extract_q4k_scales_mins(block + 4, sc, mn);
    for (int j = 0; j < 4; j++) {
        const uint8_t *qs = block + 16 + 32 * j;
        float scale0 = d * (float)sc[2 * j];
        float min0 = dmin * (float)mn[2 * j];
        for (int l = 0; l < 32; l++)
            out[64 * j + l] = (float)(qs[l] & 0x0F) * scale0 - min0;
        float scale1 = d * (float)sc[2 * j + 1];
        float min1 = dmin * (float)mn[2 * j + 1];
        for (int l = 0; l < 32; l++)
            out[64 * j + 32 + l] = (float)(qs[l] >> 4) * scale1 - min1;
    }
}

/* dequant.rs:346-372: ql@0..128, qh@128..192, int8 scales@192..208, d@208.
 * Value is evaluated left to right: (d * sc) * q. */
void yo_dequant_q6_k(const uint8_t *block, float *out) {
    float d = rd_f16(block, 208);
    const uint8_t *sc = block + 192;
    for (int half = 0; half < 2; half++) {
        const uint8_t *ql = block + half * 64;
        const uint8_t *qh = block + 128 + half * 32;
        int ob = half * 128, sb = half * 8;
        for (int l = 0; l < 32; l++) {
            int is = l / 16;
            int8_t q1 = (int8_t)((ql[l] & 0xF) | ((qh[l] & 3) << 4)) - 32;
            int8_t q2 = (int8_t)((ql[l + 32] & 0xF) | (((qh[l] >> 2) & 3) << 4)) - 32;
            int8_t q3 = (int8_t)((ql[l] >> 4) | (((qh[l] >> 4) & 3) << 4)) - 32;
            int8_t q4 = (int8_t)((ql[l + 32] >> 4) | (((qh[l] >> 6) & 3) << 4)) - 32;
            out[ob + l] = d * (float)(int8_t)sc[sb + is] * (float)q1;
            out[ob + l + 32] = d * (float)(int8_t)sc[sb + is + 2] * (float)q2;
            out[ob + l + 64] = d * (float)(int8_t)sc[sb + is + 4] * (float)q3;
            out[ob + l + 96] = d * (float)(int8_t)sc[sb + is + 6] * (float)q4;
        }
    }
}

/* dequant.rs:1232-1275 restricted to the formats on the hot path. */
int yo_dequant_block(int type, const uint8_t *block, float *out) {
    switch (type) {
    case YO_Q4_0:
        yo_dequant_q4_0(block, out);
        return 0;
    case YO_Q8_0:
        yo_dequant_q8_0(block, out);
        return 0;
    case YO_Q4_K:
        yo_dequant_q4_k(block, out);
        return 0;
    case YO_Q6_K:
        yo_dequant_q6_k(block, out);
        return 0;
    case YO_F16:
        out[0] = rd_f16(block, 0);
        return 0;
    case YO_F32:
        memcpy(out, block, 4);
        return 0;
    default:
        return yo_ext_dequant_block(type, block, out);
    }
}

int yo_dequant_tensor(int type, const uint8_t *data, size_t n_blocks, float *out) {
    int bs = yo_block_size(type), bb = yo_block_bytes(type);
    if (bs == 0)
        return -1;
    for (size_t b = 0; b < n_blocks; b++)
        if (yo_dequant_block(type, data + b * (size_t)bb, out + b * (size_t)bs))
            return -1;
    return 0;
}

/* ───────────────────────── scalar fused dots ───────────────────────── */

/* dequant.rs:902-913 */
float yo_vec_dot_q4_0(const uint8_t *block, const float *act) {
    float d = rd_f16(block, 0);
    float sum = 0.0f;
    for (int i = 0; i < 32; i++) {
        uint8_t byte = block[2 + i / 2];
        uint8_t nib = (i % 2 == 0) ? (uint8_t)(byte & 0x0F) : (uint8_t)(byte >> 4);
        sum += ((float)nib - 8.0f) * act[i];
    }
    return sum * d;
}

/* dequant.rs:916-926 */
float yo_vec_dot_q8_0(const uint8_t *block, const float *act) {
    float d = rd_f16(block, 0);
    float sum = 0.0f;
    for (int i = 0; i < 32; i++) {
        int8_t q = (int8_t)block[2 + i];
        sum += (float)q * act[i];
    }
    return sum * d;
}

/* dequant.rs:929-972: per sub-block `sum += scale*Σq·x − min*Σx`, all sums
 * sequential in f32. */
float yo_vec_dot_q4_k(const uint8_t *block, const float *act) {
    float d = rd_f16(block, 0);
    float dmin = rd_f16(block, 2);
    uint8_t sc[8], mn[8];
    yo_extract_q4k_scales_mins(block + 4, sc, mn);
    float sum = 0.0f;
    for (int j = 0; j < 4; j++) {
        const uint8_t *qs = block + 16 + 32 * j;
        float scale0 = d * (float)sc[2 * j];
        float min0 = dmin * (float)mn[2 * j];
        float sb_sum = 0.0f, min_sum = 0.0f;
        for (int l = 0; l < 32; l++) {
            sb_sum += (float)(qs[l] & 0x0F) * act[64 * j + l];
            min_sum += act[64 * j + l];
        }
        sum += scale0 * sb_sum - min0 * min_sum;

        float scale1 = d * (float)sc[2 * j + 1];
        float min1 = dmin * (float)mn[2 * j + 1];
        sb_sum = 0.0f;
        min_sum = 0.0f;
        for (int l = 0; l < 32; l++) {
            sb_sum += (float)(qs[l] >> 4) * act[64 * j + 32 + l];
            min_sum += act[64 * j + 32 + l];
        }
        sum += scale1 * sb_sum - min1 * min_sum;
    }
    return sum;
}

/* dequant.rs:976-1009: `sum += d * sc * q * act`, evaluated left to right,
 * four terms per l in the order q1,q2,q3,q4. */
float yo_vec_dot_q6_k(const uint8_t *block, const float *act) {
    float d = rd_f16(block, 208);
    const uint8_t *sc = block + 192;
    float sum = 0.0f;
    for (int half = 0; half < 2; half++) {
        const uint8_t *ql = block + half * 64;
        const uint8_t *qh = block + 128 + half * 32;
        int ab = half * 128, sb = half * 8;
        for (int l = 0; l < 32; l++) {
            int is = l / 16;
            int8_t q1 = (int8_t)((ql[l] & 0xF) | ((qh[l] & 3) << 4)) - 32;
            int8_t q2 = (int8_t)((ql[l + 32] & 0xF) | (((qh[l] >> 2) & 3) << 4)) - 32;
            int8_t q3 = (int8_t)((ql[l] >> 4) | (((qh[l] >> 4) & 3) << 4)) - 32;
            int8_t q4 = (int8_t)((ql[l + 32] >> 4) | (((qh[l] >> 6) & 3) << 4)) - 32;
            sum += d * (float)(int8_t)sc[sb + is] * (float)q1 * act[ab + l];
            sum += d * (float)(int8_t)sc[sb + is + 2] * (float)q2 * act[ab + l + 32];
            sum += d * (float)(int8_t)sc[sb + is + 4] * (float)q3 * act[ab + l + 64];
            sum += d * (float)(int8_t)sc[sb + is + 6] * (float)q4 * act[ab + l + 96];
        }
    }
    return sum;
}

/* ───────────────────────── SIMD dispatch ───────────────────────── */

static yo_q4k_asm_fn g_q4k_asm = NULL;
void yo_set_q4k_asm(yo_q4k_asm_fn fn) { g_q4k_asm = fn; }
int yo_has_q4k_asm(void) { return g_q4k_asm != NULL; }

/* simd/mod.rs:38-47 + avx2.rs:23-37 + scalar.rs. */
int yo_vec_dot_block(int type, const uint8_t *block, const float *act, int simd, float *out) {
    if (simd != YO_SCALAR && yo_have_avx2()) {
        switch (type) {
        case YO_Q8_0:
            *out = yo_vec_dot_q8_0_avx2(block, act);
            return 0;
        case YO_Q4_0:
            *out = yo_vec_dot_q4_0_avx2(block, act);
            return 0;
        case YO_Q4_K:
            if (simd == YO_AVX2_ASM && g_q4k_asm)
                *out = g_q4k_asm(block, act); /* avx2.rs:88-93 has_asm_kernels arm */
            else
                *out = yo_vec_dot_q4_k_avx2_rust(block, act);
            return 0;
        case YO_Q6_K:
            *out = yo_vec_dot_q6_k_avx2(block, act);
            return 0;
        default:
            break;
        }
    }
    switch (type) {
    case YO_Q4_0:
        *out = yo_vec_dot_q4_0(block, act);
        return 0;
    case YO_Q8_0:
        *out = yo_vec_dot_q8_0(block, act);
        return 0;
    case YO_Q4_K:
        *out = yo_vec_dot_q4_k(block, act);
        return 0;
    case YO_Q6_K:
        *out = yo_vec_dot_q6_k(block, act);
        return 0;
    default:
        return yo_ext_vec_dot_block(type, block, act, out);
    }
}

/* ───────────────────────── qmv ───────────────────────── */

int yo_hardware_threads(void) {
    long n = sysconf(_SC_NPROCESSORS_ONLN);
    return n > 0 ? (int)n : 1;
}

typedef struct {
    int type, simd, bs, bb;
    const uint8_t *w;
    const float *x;
    float *out;
    size_t row_begin, row_end, bpr, n_rows;
} qmv_job;

/* model_runner.rs:104-133: T0 prefetch of the next block (perf only). */
static inline void prefetch_next(const uint8_t *w, size_t row_off, size_t row, size_t b, size_t bpr,
                                 size_t bb, size_t n_rows) {
    size_t next;
    if (b + 1 < bpr)
        next = row_off + (b + 1) * bb;
    else if (row + 1 < n_rows)
        next = (row + 1) * bpr * bb;
    else
        return;
    __builtin_prefetch(w + next, 0, 3);
    if (bb > 64)
        __builtin_prefetch(w + next + 64, 0, 3);
}

static void qmv_rows(const qmv_job *j) {
    for (size_t row = j->row_begin; row < j->row_end; row++) {
        float sum = 0.0f;
        size_t row_off = row * j->bpr * (size_t)j->bb;
        for (size_t b = 0; b < j->bpr; b++) {
            const uint8_t *block = j->w + row_off + b * (size_t)j->bb;
            const float *act = j->x + b * (size_t)j->bs;
            prefetch_next(j->w, row_off, row, b, j->bpr, (size_t)j->bb, j->n_rows);
            float v = 0.0f;
            yo_vec_dot_block(j->type, block, act, j->simd, &v);
            sum += v;
        }
        j->out[row] = sum;
    }
}

static void *qmv_thread(void *p) {
    qmv_rows((const qmv_job *)p);
    return NULL;
}

/* model_runner.rs:152-244: rows split into ceil(n_rows / n_threads) chunks,
 * one freshly spawned thread per chunk per call when n_rows >= 128 and more
 * than one hardware thread exists; otherwise the sequential loop. */
int yo_qmv(int type, const uint8_t *w, const float *x, float *out, size_t n_rows, size_t n_cols,
           int n_threads, int simd) {
    int bs = yo_block_size(type), bb = yo_block_bytes(type);
    if (bs <= 1)
        return -1;
    if (n_threads <= 0)
        n_threads = yo_hardware_threads();
    qmv_job base = {type, simd, bs, bb, w, x, out, 0, n_rows, n_cols / (size_t)bs, n_rows};
    if (n_rows >= 128 && n_threads > 1) {
        size_t chunk = (n_rows + (size_t)n_threads - 1) / (size_t)n_threads;
        size_t n_chunks = (n_rows + chunk - 1) / chunk;
        pthread_t *tid = (pthread_t *)malloc(n_chunks * sizeof(pthread_t));
        qmv_job *jobs = (qmv_job *)malloc(n_chunks * sizeof(qmv_job));
        for (size_t c = 0; c < n_chunks; c++) {
            jobs[c] = base;
            jobs[c].row_begin = c * chunk;
            jobs[c].row_end = (c + 1) * chunk < n_rows ? (c + 1) * chunk : n_rows;
            pthread_create(&tid[c], NULL, qmv_thread, &jobs[c]);
        }
        for (size_t c = 0; c < n_chunks; c++)
            pthread_join(tid[c], NULL);
        free(tid);
        free(jobs);
    } else {
        qmv_rows(&base);
    }
    return 0;
}

/* ───────────────────────── glue ops ───────────────────────── */

/* model_runner.rs:246-275 */
void yo_rms_norm(const float *x, const float *w, size_t n, float eps, float offset, float *out) {
    float ss = 0.0f;
    for (size_t i = 0; i < n; i++)
        ss += x[i] * x[i];
    float inv = 1.0f / sqrtf(ss / (float)n + eps);
    for (size_t i = 0; i < n; i++)
        out[i] = x[i] * inv * (w[i] + offset);
}

/* model_runner.rs:78-99: freq = 1 / base^(2i/rotary_dim), theta = pos*freq,
 * all in f32 with the platform libm (Rust's powf/sin_cos call it too). */
void yo_rope_table(size_t max_seq_len, size_t rotary_dim, float freq_base, float *cos_out,
                   float *sin_out) {
    size_t half = rotary_dim / 2;
    for (size_t pos = 0; pos < max_seq_len; pos++) {
        for (size_t i = 0; i < half; i++) {
            float freq = 1.0f / powf(freq_base, 2.0f * (float)i / (float)rotary_dim);
            float theta = (float)pos * freq;
            cos_out[pos * half + i] = cosf(theta);
            sin_out[pos * half + i] = sinf(theta);
        }
    }
}

/* model_runner.rs:277-293: interleaved pairs (2i, 2i+1). */
void yo_apply_rope(float *vec, size_t vec_len, size_t pos, size_t head_dim, size_t half,
                   const float *cos_t, const float *sin_t) {
    size_t n_heads = vec_len / head_dim;
    size_t base = pos * half;
    for (size_t h = 0; h < n_heads; h++) {
        size_t ho = h * head_dim;
        for (size_t i = 0; i < half; i++) {
            float c = cos_t[base + i], s = sin_t[base + i];
            float x0 = vec[ho + 2 * i], x1 = vec[ho + 2 * i + 1];
            vec[ho + 2 * i] = x0 * c - x1 * s;
            vec[ho + 2 * i + 1] = x0 * s + x1 * c;
        }
    }
}

/* model_runner.rs:723-733 */
void yo_softmax(float *s, size_t n) {
    float mx = -INFINITY;
    for (size_t i = 0; i < n; i++)
        mx = fmaxf(mx, s[i]);
    float sum = 0.0f;
    for (size_t i = 0; i < n; i++) {
        s[i] = expf(s[i] - mx);
        sum += s[i];
    }
    float inv = 1.0f / sum;
    for (size_t i = 0; i < n; i++)
        s[i] *= inv;
}

/* model_runner.rs:672-758, flat cache (no streaming cache).  A masked score is -inf, so it contributes
 * exp(-inf) = 0 to the softmax and 0 * v to the output, exactly as in the reference. */
void yo_attention_ex(const float *q, const float *k_cache, const float *v_cache, float *attn_out,
                     float *scores, size_t n_heads, size_t n_kv_heads, size_t hd, size_t seq_len,
                     size_t sliding_window, float softcap) {
    size_t group = n_heads / n_kv_heads;
    size_t kv_stride = n_kv_heads * hd;
    size_t pos = seq_len - 1;
    float scale = 1.0f / sqrtf((float)hd);
    memset(attn_out, 0, n_heads * hd * sizeof(float));
    for (size_t h = 0; h < n_heads; h++) {
        size_t kv_h = h / group;
        const float *qh = q + h * hd;
        for (size_t t = 0; t < seq_len; t++) {
            if (sliding_window && pos >= sliding_window && t < pos - sliding_window) {
                scores[t] = -INFINITY;
                continue;
            }
            const float *kh = k_cache + t * kv_stride + kv_h * hd;
            float dot = 0.0f;
            for (size_t d = 0; d < hd; d++)
                dot += qh[d] * kh[d];
            scores[t] = dot * scale;
        }
        if (softcap != 0.0f)
            for (size_t t = 0; t < seq_len; t++)
                scores[t] = softcap * tanhf(scores[t] / softcap);
        yo_softmax(scores, seq_len);
        float *oh = attn_out + h * hd;
        for (size_t t = 0; t < seq_len; t++) {
            float w = scores[t];
            const float *vh = v_cache + t * kv_stride + kv_h * hd;
            for (size_t d = 0; d < hd; d++)
                oh[d] += w * vh[d];
        }
    }
}

void yo_attention(const float *q, const float *k_cache, const float *v_cache, float *attn_out,
                  float *scores, size_t n_heads, size_t n_kv_heads, size_t hd, size_t seq_len) {
    yo_attention_ex(q, k_cache, v_cache, attn_out, scores, n_heads, n_kv_heads, hd, seq_len, 0, 0.0f);
}

/* model_runner.rs:968-972 */
void yo_swiglu(float *gate, const float *up, size_t n) {
    for (size_t i = 0; i < n; i++) {
        float sig = 1.0f / (1.0f + expf(-gate[i]));
        gate[i] = gate[i] * sig * up[i];
    }
}

/* sampler.rs:140-163: `is_better` is the sign test of (v - best) >= 0, so an
 * equal value replaces the incumbent and ties resolve to the highest index. */
uint32_t yo_argmax(const float *v, size_t n) {
    if (n == 0)
        return 0;
    uint32_t best = 0;
    float bv = v[0];
    for (size_t i = 1; i < n; i++) {
        float diff = v[i] - bv;
        uint32_t bits;
        memcpy(&bits, &diff, 4);
        if ((bits >> 31) == 0) {
            best = (uint32_t)i;
            bv = v[i];
        }
    }
    return best;
}

/* ───────────────────────── TransformerRunner ───────────────────────── */

typedef struct {
    const uint8_t *data;
    size_t n_bytes;
    int type;
} yo_tensor;

typedef struct {
    yo_tensor attn_norm, attn_q, attn_k, attn_v, attn_output, ffn_norm, ffn_gate, ffn_up, ffn_down;
    /* optional (weight_loader.rs:203-218): Qwen2 Q/K/V biases, Gemma2 post-norms */
    yo_tensor attn_q_bias, attn_k_bias, attn_v_bias, attn_post_norm, ffn_post_norm;
    /* mixture of experts (weight_loader.rs:222-260): the router, the experts packed in one tensor per projection
     * or one tensor per expert ("ffn_gate.E.weight") */
    yo_tensor ffn_gate_inp, ffn_gate_exps, ffn_up_exps, ffn_down_exps;
    yo_tensor *gate_e, *up_e, *down_e; /* n_experts each, or NULL */
} yo_layer;

struct yo_model {
    yo_model_config cfg;
    int mod_on;
    yo_tensor token_embd, output_norm, output;
    yo_layer *layers;
    float **k_cache, **v_cache;
    float *hidden, *residual, *normed, *q, *k, *v, *attn_out, *attn_proj, *scores, *gate, *up,
        *ffn_out, *normw, *post_tmp, *router, *expert_out;
    float *rope_cos, *rope_sin;
    uint32_t pos;
    /* Mixture-of-Depths bookkeeping (mixture_of_depths.rs:28-67) */
    uint64_t mod_total_tokens, mod_layers_skipped;
    uint8_t *mod_layer_computed;
};

static float *falloc(size_t n) { return (float *)calloc(n ? n : 1, sizeof(float)); }

yo_model *yo_model_create(const yo_model_config *cfg) {
    yo_model *m = (yo_model *)calloc(1, sizeof(yo_model));
    m->cfg = *cfg;
    /* model_runner.rs:463: mod_enabled = n_layers >= 32 */
    m->mod_on = cfg->mod_enabled < 0 ? (cfg->n_layers >= 32) : cfg->mod_enabled;
    size_t L = cfg->n_layers, dim = cfg->dim, hd = cfg->head_dim;
    size_t kv_len = (size_t)cfg->max_seq_len * cfg->n_kv_heads * hd;
    m->layers = (yo_layer *)calloc(L, sizeof(yo_layer));
    m->k_cache = (float **)calloc(L, sizeof(float *));
    m->v_cache = (float **)calloc(L, sizeof(float *));
    for (size_t l = 0; l < L; l++) {
        m->k_cache[l] = falloc(kv_len);
        m->v_cache[l] = falloc(kv_len);
    }
    m->hidden = falloc(dim);
    m->residual = falloc(dim);
    m->normed = falloc(dim);
    m->normw = falloc(dim);
    m->post_tmp = falloc(dim);
    m->q = falloc((size_t)cfg->n_heads * hd);
    m->k = falloc((size_t)cfg->n_kv_heads * hd);
    m->v = falloc((size_t)cfg->n_kv_heads * hd);
    m->attn_out = falloc((size_t)cfg->n_heads * hd);
    m->attn_proj = falloc(dim);
    m->scores = falloc(cfg->max_seq_len);
    m->gate = falloc(cfg->ff_dim);
    m->up = falloc(cfg->ff_dim);
    m->ffn_out = falloc(dim);
    m->router = falloc(cfg->n_experts);
    m->expert_out = falloc(dim);
    if (cfg->n_experts)
        for (size_t l = 0; l < L; l++) {
            m->layers[l].gate_e = (yo_tensor *)calloc(cfg->n_experts, sizeof(yo_tensor));
            m->layers[l].up_e = (yo_tensor *)calloc(cfg->n_experts, sizeof(yo_tensor));
            m->layers[l].down_e = (yo_tensor *)calloc(cfg->n_experts, sizeof(yo_tensor));
        }
    /* model_runner.rs:430-434: a rotary dimension below head_dim rotates only that prefix of every head */
    size_t rot = (cfg->rotary_dim && cfg->rotary_dim < hd) ? cfg->rotary_dim : hd;
    size_t half = rot / 2;
    m->rope_cos = falloc((size_t)cfg->max_seq_len * half);
    m->rope_sin = falloc((size_t)cfg->max_seq_len * half);
    yo_rope_table(cfg->max_seq_len, rot, cfg->rope_freq_base, m->rope_cos, m->rope_sin);
    m->mod_layer_computed = (uint8_t *)malloc(L ? L : 1);
    memset(m->mod_layer_computed, 1, L ? L : 1);
    return m;
}

void yo_model_destroy(yo_model *m) {
    if (!m)
        return;
    for (size_t l = 0; l < m->cfg.n_layers; l++) {
        free(m->k_cache[l]);
        free(m->v_cache[l]);
    }
    free(m->k_cache);
    free(m->v_cache);
    for (size_t l = 0; l < m->cfg.n_layers; l++) {
        free(m->layers[l].gate_e);
        free(m->layers[l].up_e);
        free(m->layers[l].down_e);
    }
    free(m->router);
    free(m->expert_out);
    free(m->layers);
    free(m->hidden);
    free(m->residual);
    free(m->normed);
    free(m->normw);
    free(m->post_tmp);
    free(m->q);
    free(m->k);
    free(m->v);
    free(m->attn_out);
    free(m->attn_proj);
    free(m->scores);
    free(m->gate);
    free(m->up);
    free(m->ffn_out);
    free(m->rope_cos);
    free(m->rope_sin);
    free(m->mod_layer_computed);
    free(m);
}

int yo_model_set_tensor(yo_model *m, const char *name, const uint8_t *data, size_t n_bytes,
                        int type) {
    yo_tensor t = {data, n_bytes, type};
    if (!strcmp(name, "token_embd.weight")) {
        m->token_embd = t;
        return 0;
    }
    if (!strcmp(name, "output_norm.weight")) {
        m->output_norm = t;
        return 0;
    }
    if (!strcmp(name, "output.weight")) {
        m->output = t;
        return 0;
    }
    unsigned layer = 0;
    char rest[64];
    if (sscanf(name, "blk.%u.%63s", &layer, rest) == 2 && layer < m->cfg.n_layers) {
        yo_layer *l = &m->layers[layer];
        struct {
            const char *n;
            yo_tensor *t;
        } slots[] = {{"attn_norm.weight", &l->attn_norm},     {"attn_q.weight", &l->attn_q},
                     {"attn_k.weight", &l->attn_k},           {"attn_v.weight", &l->attn_v},
                     {"attn_output.weight", &l->attn_output}, {"ffn_norm.weight", &l->ffn_norm},
                     {"ffn_gate.weight", &l->ffn_gate},       {"ffn_up.weight", &l->ffn_up},
                     {"ffn_down.weight", &l->ffn_down},       {"attn_q.bias", &l->attn_q_bias},
                     {"attn_k.bias", &l->attn_k_bias},        {"attn_v.bias", &l->attn_v_bias},
                     {"attn_post_norm.weight", &l->attn_post_norm},
                     {"ffn_post_norm.weight", &l->ffn_post_norm},
                     {"ffn_gate_inp.weight", &l->ffn_gate_inp},
                     {"ffn_gate_exps.weight", &l->ffn_gate_exps},
                     {"ffn_up_exps.weight", &l->ffn_up_exps},
                     {"ffn_down_exps.weight", &l->ffn_down_exps}};
        for (size_t i = 0; i < sizeof(slots) / sizeof(slots[0]); i++)
            if (!strcmp(rest, slots[i].n)) {
                *slots[i].t = t;
                return 0;
            }
        /* one tensor per expert: "ffn_gate.E.weight" (weight_loader.rs:228-244) */
        unsigned e = 0;
        char which[16], tail[16];
        if (l->gate_e && sscanf(rest, "ffn_%15[a-z].%u.%15s", which, &e, tail) == 3 && !strcmp(tail, "weight") &&
            e < m->cfg.n_experts) {
            yo_tensor *arr = !strcmp(which, "gate") ? l->gate_e : !strcmp(which, "up") ? l->up_e : !strcmp(which, "down") ? l->down_e : NULL;
            if (arr) {
                arr[e] = t;
                return 0;
            }
        }
    }
    return -1;
}

/* model_runner.rs:259-273: norm weights are F32 or F16 in the file. */
static int norm_weights(const yo_tensor *t, size_t n, float *out) {
    if (!t->data)
        return -1;
    if (t->type == YO_F32)
        memcpy(out, t->data, n * 4);
    else
        for (size_t i = 0; i < n; i++)
            out[i] = rd_f16(t->data, 2 * i);
    return 0;
}

static int model_qmv(const yo_model *m, const yo_tensor *t, const float *x, size_t n_cols,
                     float *out, size_t n_rows) {
    if (!t->data)
        return -1;
    return yo_qmv(t->type, t->data, x, out, n_rows, n_cols, m->cfg.n_threads, m->cfg.simd);
}

/* The router's matvec (model_runner.rs:819-825 through qmv, :152-244): block formats as everywhere; F32 / F16 are
 * "blocks" of one weight, i.e. a plain left-to-right fp32 sum of w * x. */
static int router_mv(const yo_model *m, const yo_tensor *t, const float *x, size_t n_cols, float *out, size_t n_rows) {
    if (!t->data)
        return -1;
    if (t->type != YO_F32 && t->type != YO_F16)
        return model_qmv(m, t, x, n_cols, out, n_rows);
    for (size_t r = 0; r < n_rows; r++) {
        float sum = 0.0f;
        for (size_t i = 0; i < n_cols; i++) {
            float w;
            if (t->type == YO_F32)
                memcpy(&w, t->data + 4 * (r * n_cols + i), 4);
            else
                w = rd_f16(t->data, 2 * (r * n_cols + i));
            sum += w * x[i];
        }
        out[r] = sum;
    }
    return 0;
}

/* model_runner.rs:827-854 (and its test :1138-1186): softmax over the router logits, experts ordered by probability
 * (stable sort, descending: equal probabilities keep index order), the first n_used renormalised to sum 1.
 * `probs` holds the logits on entry and the probabilities on return. */
void yo_moe_route(float *probs, size_t n_exp, size_t n_used, uint32_t *selected, float *weights) {
    float max_r = -INFINITY;
    for (size_t i = 0; i < n_exp; i++)
        max_r = probs[i] > max_r ? probs[i] : max_r;
    float sum_r = 0.0f;
    for (size_t i = 0; i < n_exp; i++) {
        probs[i] = expf(probs[i] - max_r);
        sum_r += probs[i];
    }
    float inv_r = 1.0f / sum_r;
    for (size_t i = 0; i < n_exp; i++)
        probs[i] *= inv_r;
    /* stable insertion sort of the indices by descending probability */
    uint32_t order[256];
    if (n_exp > 256)
        n_exp = 256;
    for (size_t i = 0; i < n_exp; i++) {
        size_t j = i;
        while (j > 0 && probs[order[j - 1]] < probs[i]) {
            order[j] = order[j - 1];
            j--;
        }
        order[j] = (uint32_t)i;
    }
    float selected_sum = 0.0f;
    for (size_t k = 0; k < n_used; k++)
        selected_sum += probs[order[k]];
    float inv_sel = 1.0f / selected_sum;
    for (size_t k = 0; k < n_used; k++) {
        selected[k] = order[k];
        weights[k] = probs[order[k]] * inv_sel;
    }
}

/* model_runner.rs:295-310: F32 or F16 bias added element by element. */
static void add_bias(float *v, size_t n, const yo_tensor *b) {
    for (size_t i = 0; i < n; i++) {
        float x;
        if (b->type == YO_F32)
            memcpy(&x, b->data + 4 * i, 4);
        else
            x = rd_f16(b->data, 2 * i);
        v[i] += x;
    }
}

/* model_runner.rs:312-314 */
static float gelu_tanh(float x) {
    return x * 0.5f * (1.0f + tanhf(0.7978846f * (x + 0.044715f * x * x * x)));
}
float yo_gelu(float x) { return gelu_tanh(x); }

/* mixture_of_depths.rs:113-117 */
static float activation_norm(const float *h, size_t n) {
    float ss = 0.0f;
    for (size_t i = 0; i < n; i++)
        ss += h[i] * h[i];
    return sqrtf(ss / (float)n);
}

/* mixture_of_depths.rs:82-111 with MoDConfig::default (:17-25). */
static int should_skip_layer(const float *hidden, size_t dim, size_t layer, size_t n_layers,
                             uint64_t tokens_seen, size_t skipped_this_token) {
    const float skip_threshold = 0.1f, max_skip_ratio = 0.5f;
    const uint64_t warmup_tokens = 10;
    if (tokens_seen < warmup_tokens)
        return 0;
    if (layer == 0 || layer == n_layers - 1)
        return 0;
    size_t max_skips = (size_t)((float)n_layers * max_skip_ratio);
    if (skipped_this_token >= max_skips)
        return 0;
    return activation_norm(hidden, dim) < skip_threshold;
}

/* model_runner.rs:533-1036: the dense path with its architecture variants (Q/K/V bias, partial RoPE, sliding
 * window, Gemma norm offset / embedding scale / GeGLU / post-norms / softcaps) and the mixture-of-experts FFN;
 * flat KV cache. */
int yo_model_forward(yo_model *m, uint32_t token, float *logits) {
    const yo_model_config *c = &m->cfg;
    size_t dim = c->dim, hd = c->head_dim, n_heads = c->n_heads, n_kv = c->n_kv_heads;
    size_t kv_stride = n_kv * hd, ff = c->ff_dim, pos = m->pos;
    if (pos >= c->max_seq_len)
        return -2;

    /* 1. token embedding (:543-566) */
    if (!m->token_embd.data)
        return -1;
    size_t row_bytes = m->token_embd.n_bytes / c->vocab_size;
    const uint8_t *tok = m->token_embd.data + (size_t)token * row_bytes;
    if (m->token_embd.type == YO_F32) {
        memcpy(m->hidden, tok, dim * 4);
    } else {
        int bs = yo_block_size(m->token_embd.type), bb = yo_block_bytes(m->token_embd.type);
        for (size_t b = 0; b < dim / (size_t)bs; b++)
            if (yo_dequant_block(m->token_embd.type, tok + b * (size_t)bb, m->hidden + b * (size_t)bs))
                return -1;
    }

    /* Gemma: embeddings scaled by sqrt(dim) (:568-574) */
    const float norm_off = c->norm_weight_offset;
    if (norm_off > 0.0f) {
        float sc = sqrtf((float)dim);
        for (size_t i = 0; i < dim; i++)
            m->hidden[i] *= sc;
    }
    size_t rot = (c->rotary_dim && c->rotary_dim < hd) ? c->rotary_dim : hd;

    size_t seq_len = pos + 1;
    if (m->mod_on)
        m->mod_total_tokens += 1; /* MoDStats::new_token (:581-583) */

    for (size_t layer = 0; layer < c->n_layers; layer++) {
        yo_layer *L = &m->layers[layer];
        memcpy(m->residual, m->hidden, dim * 4);

        /* Mixture-of-Depths (:594-618) */
        if (m->mod_on) {
            size_t skipped = 0;
            for (size_t i = 0; i < layer; i++)
                skipped += m->mod_layer_computed[i] ? 0 : 1;
            if (should_skip_layer(m->hidden, dim, layer, c->n_layers, m->mod_total_tokens,
                                  skipped)) {
                m->mod_layer_computed[layer] = 0;
                m->mod_layers_skipped += 1;
                continue;
            }
            m->mod_layer_computed[layer] = 1;
        }

        if (norm_weights(&L->attn_norm, dim, m->normw))
            return -1;
        yo_rms_norm(m->hidden, m->normw, dim, c->norm_eps, norm_off, m->normed);

        if (model_qmv(m, &L->attn_q, m->normed, dim, m->q, n_heads * hd) ||
            model_qmv(m, &L->attn_k, m->normed, dim, m->k, kv_stride) ||
            model_qmv(m, &L->attn_v, m->normed, dim, m->v, kv_stride))
            return -1;
        /* Q/K/V bias (:640-651) */
        if (L->attn_q_bias.data)
            add_bias(m->q, n_heads * hd, &L->attn_q_bias);
        if (L->attn_k_bias.data)
            add_bias(m->k, kv_stride, &L->attn_k_bias);
        if (L->attn_v_bias.data)
            add_bias(m->v, kv_stride, &L->attn_v_bias);

        yo_apply_rope(m->q, n_heads * hd, pos, hd, rot / 2, m->rope_cos, m->rope_sin);
        yo_apply_rope(m->k, kv_stride, pos, hd, rot / 2, m->rope_cos, m->rope_sin);

        memcpy(m->k_cache[layer] + pos * kv_stride, m->k, kv_stride * 4);
        memcpy(m->v_cache[layer] + pos * kv_stride, m->v, kv_stride * 4);

        yo_attention_ex(m->q, m->k_cache[layer], m->v_cache[layer], m->attn_out, m->scores, n_heads,
                        n_kv, hd, seq_len, c->sliding_window, c->attn_logit_softcap);

        if (model_qmv(m, &L->attn_output, m->attn_out, n_heads * hd, m->attn_proj, dim))
            return -1;
        /* post-attention norm (Gemma2, :764-779) */
        if (L->attn_post_norm.data) {
            memcpy(m->post_tmp, m->attn_proj, dim * 4);
            if (norm_weights(&L->attn_post_norm, dim, m->normw))
                return -1;
            yo_rms_norm(m->post_tmp, m->normw, dim, c->norm_eps, norm_off, m->attn_proj);
        }
        for (size_t i = 0; i < dim; i++)
            m->hidden[i] = m->residual[i] + m->attn_proj[i];

        memcpy(m->residual, m->hidden, dim * 4);
        if (norm_weights(&L->ffn_norm, dim, m->normw))
            return -1;
        yo_rms_norm(m->hidden, m->normw, dim, c->norm_eps, norm_off, m->normed);

        if (c->n_experts > 0) {
            /* mixture of experts (:813-958): router, top-k, the selected experts' SwiGLU FFNs weighted and summed */
            size_t n_exp = c->n_experts, n_used = c->n_experts_used;
            if (n_used == 0 || n_used > n_exp || n_exp > 256)
                return -1;
            if (router_mv(m, &L->ffn_gate_inp, m->normed, dim, m->router, n_exp))
                return -1;
            uint32_t sel[256];
            float wsel[256];
            yo_moe_route(m->router, n_exp, n_used, sel, wsel);
            memset(m->ffn_out, 0, dim * 4);
            for (size_t k = 0; k < n_used; k++) {
                size_t e = sel[k];
                yo_tensor g, u, d;
                if (L->gate_e && L->gate_e[e].data) {
                    g = L->gate_e[e];
                    u = L->up_e[e];
                    d = L->down_e[e];
                    if (!u.data || !d.data)
                        return -1;
                } else if (L->ffn_gate_exps.data) {
                    /* packed: expert e is the e-th of n_exp equal slices of each tensor (:890-918) */
                    if (!L->ffn_up_exps.data || !L->ffn_down_exps.data)
                        return -1;
                    size_t gb = L->ffn_gate_exps.n_bytes / n_exp, ub = L->ffn_up_exps.n_bytes / n_exp, db = L->ffn_down_exps.n_bytes / n_exp;
                    g = (yo_tensor){L->ffn_gate_exps.data + e * gb, gb, L->ffn_gate_exps.type};
                    u = (yo_tensor){L->ffn_up_exps.data + e * ub, ub, L->ffn_up_exps.type};
                    d = (yo_tensor){L->ffn_down_exps.data + e * db, db, L->ffn_down_exps.type};
                } else {
                    return -1;
                }
                if (model_qmv(m, &g, m->normed, dim, m->gate, ff) || model_qmv(m, &u, m->normed, dim, m->up, ff))
                    return -1;
                /* always SwiGLU here (:876-881), written as gate * sigmoid(gate) * up */
                for (size_t i = 0; i < ff; i++) {
                    float sigmoid = 1.0f / (1.0f + expf(-m->gate[i]));
                    m->gate[i] = m->gate[i] * sigmoid * m->up[i];
                }
                if (model_qmv(m, &d, m->gate, ff, m->expert_out, dim))
                    return -1;
                for (size_t i = 0; i < dim; i++)
                    m->ffn_out[i] += wsel[k] * m->expert_out[i];
            }
        } else {
        if (model_qmv(m, &L->ffn_gate, m->normed, dim, m->gate, ff) ||
            model_qmv(m, &L->ffn_up, m->normed, dim, m->up, ff))
            return -1;
        if (c->geglu) { /* :974-978 */
            for (size_t i = 0; i < ff; i++)
                m->gate[i] = gelu_tanh(m->gate[i]) * m->up[i];
        } else {
            yo_swiglu(m->gate, m->up, ff);
        }
        if (model_qmv(m, &L->ffn_down, m->gate, ff, m->ffn_out, dim))
            return -1;
        }
        /* post-FFN norm (Gemma2, :985-999) */
        if (L->ffn_post_norm.data) {
            memcpy(m->post_tmp, m->ffn_out, dim * 4);
            if (norm_weights(&L->ffn_post_norm, dim, m->normw))
                return -1;
            yo_rms_norm(m->post_tmp, m->normw, dim, c->norm_eps, norm_off, m->ffn_out);
        }
        for (size_t i = 0; i < dim; i++)
            m->hidden[i] = m->residual[i] + m->ffn_out[i];
    }

    if (norm_weights(&m->output_norm, dim, m->normw))
        return -1;
    yo_rms_norm(m->hidden, m->normw, dim, c->norm_eps, norm_off, m->normed);
    /* gpu_runner.rs:214-215 and weight_loader: output falls back to token_embd */
    const yo_tensor *out_t = m->output.data ? &m->output : &m->token_embd;
    if (model_qmv(m, out_t, m->normed, dim, logits, c->vocab_size))
        return -1;
    /* final logit softcap (Gemma2, :1027-1032) */
    if (c->logit_softcap != 0.0f)
        for (size_t i = 0; i < c->vocab_size; i++)
            logits[i] = c->logit_softcap * tanhf(logits[i] / c->logit_softcap);
    m->pos += 1;
    return 0;
}

void yo_model_reset(yo_model *m) { m->pos = 0; }
uint32_t yo_model_pos(const yo_model *m) { return m->pos; }
uint64_t yo_model_layers_skipped(const yo_model *m) { return m->mod_layers_skipped; }
const float *yo_model_hidden(const yo_model *m) { return m->hidden; }
const float *yo_model_k_cache(const yo_model *m, uint32_t layer) { return m->k_cache[layer]; }
const float *yo_model_v_cache(const yo_model *m, uint32_t layer) { return m->v_cache[layer]; }
