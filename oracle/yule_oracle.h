/*
 * yule_oracle.h — CPU restatement of Yule's quantized-inference arithmetic.
 *
 * TEST INFRASTRUCTURE ONLY.  This library is the checker that the CUDA
 * backend's results are compared against; nothing in the shipped package may
 * link, import or call it.  Every function cites the file:line of the Yule
 * source it follows (paths relative to the Yule repository root).
 *
 * Parity status: pinned against the known-answer vectors of Yule's own tests
 * (f16 KATs, Q4_0/Q8_0 dequant + dot KATs, the xorshift AVX2-vs-scalar
 * recipes, trait-level RoPE/attention/Q4_0-matvec KATs) and, for the Q4_K
 * block dot, against Yule's own assembly kernel q4k_gemv_avx2.S built
 * unmodified into oracle/_ref/.  No Yule test fixes a Q4_K or Q6_K *value*
 * or a full-forward logit vector, so for those the restatement of the cited
 * lines is the pin.
 *
 * Build: -O2 -ffp-contract=off -fno-fast-math so that sums round like the
 * Rust code (Rust never contracts a*b+c into an FMA on its own).
 */
#ifndef YULE_ORACLE_H
#define YULE_ORACLE_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* GGUF type ids == yule-core/src/dtype.rs:13-58 discriminants. */
enum {
    YO_F32 = 0,
    YO_F16 = 1,
    YO_Q4_0 = 2,
    YO_Q4_1 = 3,
    YO_Q5_0 = 6,
    YO_Q5_1 = 7,
    YO_Q8_0 = 8,
    YO_Q8_1 = 9,
    YO_Q2_K = 10,
    YO_Q3_K = 11,
    YO_Q4_K = 12,
    YO_Q5_K = 13,
    YO_Q6_K = 14,
};

/* SIMD dispatch level of yule-core/src/simd/mod.rs:20-47. */
enum {
    YO_SCALAR = 0,   /* dequant.rs scalar fused dots                          */
    YO_AVX2 = 1,     /* simd/avx2.rs, Q4_K through its Rust-intrinsic fallback */
    YO_AVX2_ASM = 2, /* simd/avx2.rs, Q4_K through kernels/q4k_gemv_avx2.S     */
};

int yo_block_size(int type);  /* dtype.rs:99-118  */
int yo_block_bytes(int type); /* dtype.rs:62-96   */

float yo_f16_to_f32(uint16_t bits);                                       /* dequant.rs:20-49   */
void yo_extract_q4k_scales_mins(const uint8_t *q12, uint8_t *sc8, uint8_t *mn8); /* :176-190 */
void yo_dequant_q4_0(const uint8_t *block, float *out);                   /* dequant.rs:77-86   */
void yo_dequant_q8_0(const uint8_t *block, float *out);                   /* dequant.rs:142-150 */
void yo_dequant_q4_k(const uint8_t *block, float *out);                   /* dequant.rs:260-290 */
void yo_dequant_q6_k(const uint8_t *block, float *out);                   /* dequant.rs:346-372 */
int yo_dequant_block(int type, const uint8_t *block, float *out);         /* dequant.rs:1232    */
/* yule_oracle_ext.c: the formats the reference's GPU backends reject but its CPU runner handles. */
void yo_dequant_q4_1(const uint8_t *block, float *out); /* dequant.rs:91-101  */
void yo_dequant_q5_0(const uint8_t *block, float *out); /* dequant.rs:106-119 */
void yo_dequant_q5_1(const uint8_t *block, float *out); /* dequant.rs:124-138 */
void yo_dequant_q8_1(const uint8_t *block, float *out); /* dequant.rs:156-165 */
void yo_dequant_q2_k(const uint8_t *block, float *out); /* dequant.rs:196-214 */
void yo_dequant_q3_k(const uint8_t *block, float *out); /* dequant.rs:219-251 */
void yo_dequant_q5_k(const uint8_t *block, float *out); /* dequant.rs:297-338 */
float yo_vec_dot_q4_1(const uint8_t *block, const float *act); /* dequant.rs:1143-1157 */
float yo_vec_dot_q5_0(const uint8_t *block, const float *act); /* dequant.rs:1160-1174 */
float yo_vec_dot_q5_1(const uint8_t *block, const float *act); /* dequant.rs:1177-1194 */
float yo_vec_dot_q8_1(const uint8_t *block, const float *act); /* dequant.rs:1197-1207 */
float yo_vec_dot_q2_k(const uint8_t *block, const float *act); /* dequant.rs:1013-1041 */
float yo_vec_dot_q3_k(const uint8_t *block, const float *act); /* dequant.rs:1045-1084 */
float yo_vec_dot_q5_k(const uint8_t *block, const float *act); /* dequant.rs:1088-1140 */
int yo_ext_dequant_block(int type, const uint8_t *block, float *out);
int yo_ext_vec_dot_block(int type, const uint8_t *block, const float *act, float *out);
int yo_dequant_tensor(int type, const uint8_t *data, size_t n_blocks, float *out);

float yo_vec_dot_q4_0(const uint8_t *block, const float *act); /* dequant.rs:902-913  */
float yo_vec_dot_q8_0(const uint8_t *block, const float *act); /* dequant.rs:916-926  */
float yo_vec_dot_q4_k(const uint8_t *block, const float *act); /* dequant.rs:929-972  */
float yo_vec_dot_q6_k(const uint8_t *block, const float *act); /* dequant.rs:976-1009 */

/* simd/avx2.rs restated with the same intrinsics (file yule_oracle_avx2.c). */
int yo_have_avx2(void);
float yo_vec_dot_q8_0_avx2(const uint8_t *block, const float *act);      /* avx2.rs:39-56   */
float yo_vec_dot_q4_0_avx2(const uint8_t *block, const float *act);      /* avx2.rs:60-83   */
float yo_vec_dot_q4_k_avx2_rust(const uint8_t *block, const float *act); /* avx2.rs:103-152 */
float yo_vec_dot_q6_k_avx2(const uint8_t *block, const float *act);      /* avx2.rs:306-337 */

/* Hand the oracle the entry point of Yule's own assembly kernel
 * (kernels/mod.rs:22), loaded by the caller from oracle/_ref/. */
typedef float (*yo_q4k_asm_fn)(const uint8_t *weights, const float *activations);
void yo_set_q4k_asm(yo_q4k_asm_fn fn);
int yo_has_q4k_asm(void);

/* simd::vec_dot (simd/mod.rs:38-47) → dequant::vec_dot_block (dequant.rs:1279). */
int yo_vec_dot_block(int type, const uint8_t *block, const float *act, int simd, float *out);

/* yule-infer/src/model_runner.rs:152-244.  n_threads <= 0 means "all hardware
 * threads" (available_parallelism).  Returns 0, or -1 on a bad type. */
int yo_qmv(int type, const uint8_t *w, const float *x, float *out, size_t n_rows, size_t n_cols,
           int n_threads, int simd);
int yo_hardware_threads(void);

/* model_runner.rs:246-275 with f32 weights. */
void yo_rms_norm(const float *x, const float *w, size_t n, float eps, float offset, float *out);
/* model_runner.rs:78-99 — cos/sin laid out [pos][half]. */
void yo_rope_table(size_t max_seq_len, size_t rotary_dim, float freq_base, float *cos_out,
                   float *sin_out);
/* model_runner.rs:277-293. */
void yo_apply_rope(float *vec, size_t vec_len, size_t pos, size_t head_dim, size_t half,
                   const float *cos_t, const float *sin_t);
/* softmax as written inline in model_runner.rs:723-733. */
void yo_softmax(float *s, size_t n);
/* model_runner.rs:672-758 for one token: all heads, flat fp32 cache. */
void yo_attention(const float *q, const float *k_cache, const float *v_cache, float *attn_out,
                  float *scores_scratch, size_t n_heads, size_t n_kv_heads, size_t head_dim,
                  size_t seq_len);
/* The same with the sliding-window mask (:688-696; window 0 = none) and the attention logit softcap
 * (:716-721; cap 0 = none). */
void yo_attention_ex(const float *q, const float *k_cache, const float *v_cache, float *attn_out,
                     float *scores_scratch, size_t n_heads, size_t n_kv_heads, size_t head_dim,
                     size_t seq_len, size_t sliding_window, float softcap);
/* model_runner.rs:968-972: gate[i] = gate[i]*sigmoid(gate[i])*up[i]. */
void yo_swiglu(float *gate, const float *up, size_t n);
/* model_runner.rs:312-314: the tanh form of GELU used by GeGLU. */
float yo_gelu(float x);
/* yule-infer/src/sampler.rs:150-163 — argmax with `>=`, so ties go to the
 * highest index. */
uint32_t yo_argmax(const float *v, size_t n);

/* ── sampler (yule-infer/src/sampler.rs), yule_oracle_sampler.c ── */
float yo_ct_gte(float a, float b);                                  /* sampler.rs:141-147 */
uint32_t yo_sample_ct(const float *probs, size_t n, float r);      /* sampler.rs:166-183 */
/* sampler.rs:17-136 with the random value supplied by the caller; -1 on empty logits. */
int64_t yo_sample(const float *logits, size_t n, float temperature, float top_p, uint32_t top_k, float min_p,
                  float repetition_penalty, const uint32_t *previous, size_t n_previous, float r);

/* ── whole forward pass: TransformerRunner (model_runner.rs:533-1036) ── */
typedef struct {
    uint32_t dim, n_layers, n_heads, n_kv_heads, head_dim, vocab_size, ff_dim, max_seq_len;
    float norm_eps, rope_freq_base;
    int32_t mod_enabled; /* -1: as the reference (n_layers >= 32, model_runner.rs:463); 0/1 force */
    int32_t simd;        /* YO_SCALAR / YO_AVX2 / YO_AVX2_ASM */
    int32_t n_threads;   /* <= 0: all hardware threads */
    /* Architecture variants of the dense path (RunnerConfig, model_runner.rs:25-58); zero = the Llama default. */
    uint32_t rotary_dim;       /* partial RoPE: rotated prefix of each head (model_runner.rs:430-434, :502); 0 = head_dim */
    uint32_t sliding_window;   /* attention sees positions t >= pos - w once pos >= w (:688-696); 0 = none */
    float attn_logit_softcap;  /* scores = cap * tanh(scores / cap) before the softmax (:716-721); 0 = none */
    float logit_softcap;       /* the same on the final logits (:1027-1032); 0 = none */
    float norm_weight_offset;  /* Gemma: norm weights are (w + 1) and embeddings are scaled by sqrt(dim) (:246-275, :568-574) */
    int32_t geglu;             /* Gemma: gelu(gate) * up instead of SiLU (:312-314, :974-978) */
    uint32_t n_experts;        /* mixture of experts (:395-397, :813-958): experts per layer, 0 = dense FFN */
    uint32_t n_experts_used;   /* experts evaluated per token */
} yo_model_config;

typedef struct yo_model yo_model;

/* Router of the mixture-of-experts FFN (model_runner.rs:827-854): `probs` holds n_exp logits on entry, their softmax
 * on return; selected[k], weights[k] (k < n_used) are the chosen experts in order of decreasing probability and their
 * renormalised weights. */
void yo_moe_route(float *probs, size_t n_exp, size_t n_used, uint32_t *selected, float *weights);

yo_model *yo_model_create(const yo_model_config *cfg);
void yo_model_destroy(yo_model *m);
/* name is the GGUF tensor name ("blk.3.attn_q.weight", "token_embd.weight",
 * "output_norm.weight", ...).  data is borrowed, not copied. */
int yo_model_set_tensor(yo_model *m, const char *name, const uint8_t *data, size_t n_bytes,
                        int type);
/* One token through every layer; writes vocab_size logits.  Returns 0, -1 on a
 * missing tensor, -2 on "context length exceeded". */
int yo_model_forward(yo_model *m, uint32_t token, float *logits);
void yo_model_reset(yo_model *m); /* model_runner.rs:1087-1092 (MoD token count survives) */
uint32_t yo_model_pos(const yo_model *m);
uint64_t yo_model_layers_skipped(const yo_model *m);
/* Copies of internal state for layer-by-layer comparisons. */
const float *yo_model_hidden(const yo_model *m);
const float *yo_model_k_cache(const yo_model *m, uint32_t layer);
const float *yo_model_v_cache(const yo_model *m, uint32_t layer);

#ifdef __cplusplus
}
#endif
#endif
