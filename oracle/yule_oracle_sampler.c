/*
 * yule_oracle_sampler.c — CPU restatement of Yule's token sampler (yule-infer/src/sampler.rs).
 *
 * TEST INFRASTRUCTURE ONLY (see yule_oracle.h).  The reference draws its random number from the OS CSPRNG
 * (sampler.rs:212-220); here it is a parameter, so that a result can be reproduced and compared.
 * Pinned to the reference's own known answers: ct_gte (:175-187 tests :229-234), argmax (:236-240),
 * sample_ct (:242-251).  The composition of the steps is pinned by restatement only.
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#include "yule_oracle.h"

/* sampler.rs:141-147: 1.0 when a >= b by the sign bit of (a - b), else 0.0 */
float yo_ct_gte(float a, float b) {
    float diff = a - b;
    uint32_t bits;
    memcpy(&bits, &diff, 4);
    return (float)(1u - (bits >> 31));
}

/* sampler.rs:166-183: first index whose running sum reaches r; the last token when none does */
uint32_t yo_sample_ct(const float *probs, size_t n, float r) {
    float cumulative = 0.0f, found = 0.0f;
    uint32_t selected = (uint32_t)(n - 1);
    for (size_t i = 0; i < n; i++) {
        cumulative += probs[i];
        float crossed = yo_ct_gte(cumulative, r);
        float first_cross = crossed * (1.0f - found);
        uint32_t m = ((uint32_t)first_cross) & 1u; /* blend_u32, :187-190 */
        selected = selected * (1u - m) + (uint32_t)i * m;
        found = found * (1.0f - crossed) + 1.0f * crossed; /* blend_f32, :193-197 */
    }
    return selected;
}

static int cmp_desc(const void *a, const void *b) {
    float x = *(const float *)a, y = *(const float *)b;
    return (x < y) - (x > y);
}
typedef struct {
    uint32_t idx;
    float p;
} ip;
/* descending by probability; equal probabilities keep index order (the reference's sort_unstable_by leaves
 * the order of ties unspecified, :84-87) */
static int cmp_ip_desc(const void *a, const void *b) {
    const ip *x = (const ip *)a, *y = (const ip *)b;
    if (x->p != y->p)
        return (x->p < y->p) - (x->p > y->p);
    return (x->idx > y->idx) - (x->idx < y->idx);
}

/* sampler.rs:17-136 with the random value r supplied by the caller.  Returns -1 on empty logits. */
int64_t yo_sample(const float *logits_in, size_t n, float temperature, float top_p, uint32_t top_k, float min_p,
                  float repetition_penalty, const uint32_t *previous, size_t n_previous, float r) {
    if (n == 0)
        return -1;
    float *logits = (float *)malloc(n * sizeof(float));
    float *probs = (float *)malloc(n * sizeof(float));
    memcpy(logits, logits_in, n * sizeof(float));
    /* repetition penalty, once per occurrence (:26-38) */
    if (repetition_penalty != 1.0f && n_previous) {
        for (size_t j = 0; j < n_previous; j++) {
            size_t idx = previous[j];
            if (idx < n) {
                if (logits[idx] > 0.0f)
                    logits[idx] /= repetition_penalty;
                else
                    logits[idx] *= repetition_penalty;
            }
        }
    }
    /* temperature (:41-46) */
    if (temperature > 0.0f && temperature != 1.0f) {
        float inv_t = 1.0f / temperature;
        for (size_t i = 0; i < n; i++)
            logits[i] *= inv_t;
    }
    /* softmax (:49-55) */
    float mx = -INFINITY;
    for (size_t i = 0; i < n; i++)
        mx = fmaxf(mx, logits[i]);
    float sum = 0.0f;
    for (size_t i = 0; i < n; i++) {
        probs[i] = expf(logits[i] - mx);
        sum += probs[i];
    }
    float inv_sum = 1.0f / sum;
    for (size_t i = 0; i < n; i++)
        probs[i] *= inv_sum;
    /* top-k (:58-70): the threshold is sorted[k] of the descending order */
    if (top_k > 0 && (size_t)top_k < n) {
        float *sorted = (float *)malloc(n * sizeof(float));
        memcpy(sorted, probs, n * sizeof(float));
        qsort(sorted, n, sizeof(float), cmp_desc);
        float threshold = sorted[top_k];
        for (size_t i = 0; i < n; i++)
            probs[i] *= yo_ct_gte(probs[i], threshold);
        free(sorted);
    }
    /* min_p (:73-80) */
    if (min_p > 0.0f) {
        float max_prob = 0.0f;
        for (size_t i = 0; i < n; i++)
            max_prob = fmaxf(max_prob, probs[i]);
        float thr = max_prob * min_p;
        for (size_t i = 0; i < n; i++)
            probs[i] *= yo_ct_gte(probs[i], thr);
    }
    /* top-p (:83-118): tokens in descending order until the running sum reaches top_p, that token included */
    if (top_p < 1.0f) {
        ip *ord = (ip *)malloc(n * sizeof(ip));
        for (size_t i = 0; i < n; i++) {
            ord[i].idx = (uint32_t)i;
            ord[i].p = probs[i];
        }
        qsort(ord, n, sizeof(ip), cmp_ip_desc);
        uint8_t *in_nucleus = (uint8_t *)calloc(n, 1);
        float cumulative = 0.0f;
        for (size_t i = 0; i < n; i++) {
            cumulative += ord[i].p;
            in_nucleus[ord[i].idx] = 1;
            if (cumulative >= top_p)
                break;
        }
        for (size_t i = 0; i < n; i++)
            if (!in_nucleus[i])
                probs[i] = 0.0f;
        free(in_nucleus);
        free(ord);
    }
    /* renormalise (:121-130); nothing left: argmax of the (penalised, scaled) logits */
    float total = 0.0f;
    for (size_t i = 0; i < n; i++)
        total += probs[i];
    int64_t out;
    if (total <= 0.0f) {
        out = yo_argmax(logits, n);
    } else {
        float inv_total = 1.0f / total;
        for (size_t i = 0; i < n; i++)
            probs[i] *= inv_total;
        out = yo_sample_ct(probs, n, r);
    }
    free(logits);
    free(probs);
    return out;
}
