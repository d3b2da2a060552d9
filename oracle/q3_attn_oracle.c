/* q3_attn_oracle.c - see q3_attn_oracle.h. TEST INFRASTRUCTURE ONLY.
 *
 * Plain C restatement of the sera.c attention-path kernels with double
 * accumulation. Each function names the reference lines it follows.
 */
#include "q3_attn_oracle.h"

#include <math.h>
#include <stdlib.h>
#include <string.h>

#ifdef _OPENMP
#include <omp.h>
#endif

int q3o_threads(void) {
#ifdef _OPENMP
    return omp_get_max_threads();
#else
    return 1;
#endif
}

void q3o_set_threads(int n) {
#ifdef _OPENMP
    if (n > 0) omp_set_num_threads(n);
#else
    (void)n;
#endif
}

/* src/q3_forward.cu:1128-1130 */
void q3o_inv_freq(double theta, uint32_t head_dim, float *inv_freq) {
    for (uint32_t i = 0; i < head_dim / 2; i++)
        inv_freq[i] = (float)(1.0 / pow(theta, (double)(2 * i) / (double)head_dim));
}

/* src/q3_forward.cu:117-148; tests/test_q3_forward_primitives.cu:46-56 */
void q3o_rms_norm(const float *input, const float *weight, uint32_t rows,
                  uint32_t width, float epsilon, float *output) {
#pragma omp parallel for schedule(static)
    for (int64_t r = 0; r < (int64_t)rows; r++) {
        const float *in = input + (size_t)r * width;
        float *out = output + (size_t)r * width;
        double sum = 0.0;
        for (uint32_t i = 0; i < width; i++) sum += (double)in[i] * (double)in[i];
        const double inv = 1.0 / sqrt(sum / (double)width + (double)epsilon);
        for (uint32_t i = 0; i < width; i++)
            out[i] = (float)((double)in[i] * inv * (double)weight[i]);
    }
}

static void rope_row(float *row, uint32_t head_dim, uint32_t position,
                     const float *inv_freq) {
    const uint32_t half = head_dim / 2;
    for (uint32_t p = 0; p < half; p++) {
        /* fp32 product, as the reference forms it (src/q3_forward.cu:199). */
        const float angle = (float)position * inv_freq[p];
        const double c = cos((double)angle), s = sin((double)angle);
        const double x = row[p], y = row[half + p];
        row[p] = (float)(x * c - y * s);
        row[half + p] = (float)(x * s + y * c);
    }
}

/* src/q3_forward.cu:181-209 (scalar base) and :380-410 (per-token positions) */
void q3o_rope(float *q, float *k, uint32_t tokens, uint32_t n_heads,
              uint32_t n_kv_heads, uint32_t head_dim, uint32_t position_base,
              const uint32_t *token_positions, const float *inv_freq) {
#pragma omp parallel for schedule(static)
    for (int64_t t = 0; t < (int64_t)tokens; t++) {
        const uint32_t position =
            token_positions ? token_positions[t] : position_base + (uint32_t)t;
        for (uint32_t h = 0; h < n_heads; h++)
            rope_row(q + ((size_t)t * n_heads + h) * head_dim, head_dim,
                     position, inv_freq);
        for (uint32_t h = 0; h < n_kv_heads; h++)
            rope_row(k + ((size_t)t * n_kv_heads + h) * head_dim, head_dim,
                     position, inv_freq);
    }
}

/* One (query row) x (two key segments) softmax-weighted sum. seg*_k / seg*_v
 * point at the kv_head's first element of key 0; consecutive keys are `row`
 * floats apart. scores is scratch for n0+n1 doubles. */
static void attend_row(const float *q_row, uint32_t head_dim, float scale,
                       const float *seg0_k, const float *seg0_v, uint32_t n0,
                       const float *seg1_k, const float *seg1_v, uint32_t n1,
                       size_t row, double *scores, float *out_row) {
    const uint32_t n = n0 + n1;
    double max_score = -INFINITY;
    for (uint32_t j = 0; j < n; j++) {
        const float *k_row = j < n0 ? seg0_k + (size_t)j * row
                                    : seg1_k + (size_t)(j - n0) * row;
        double dot = 0.0;
        for (uint32_t d = 0; d < head_dim; d++)
            dot += (double)q_row[d] * (double)k_row[d];
        const double s = dot * (double)scale;
        scores[j] = s;
        if (s > max_score) max_score = s;
    }
    double acc[512];
    for (uint32_t d = 0; d < head_dim; d++) acc[d] = 0.0;
    double den = 0.0;
    for (uint32_t j = 0; j < n; j++) {
        const float *v_row = j < n0 ? seg0_v + (size_t)j * row
                                    : seg1_v + (size_t)(j - n0) * row;
        const double p = exp(scores[j] - max_score);
        den += p;
        for (uint32_t d = 0; d < head_dim; d++) acc[d] += p * (double)v_row[d];
    }
    for (uint32_t d = 0; d < head_dim; d++) out_row[d] = (float)(acc[d] / den);
}

/* src/q3_forward.cu:218-290 */
void q3o_attention(const float *q, const float *k_rows, const float *v_rows,
                   uint32_t tokens, uint32_t n_heads, uint32_t n_kv_heads,
                   uint32_t head_dim, uint32_t position_base,
                   uint32_t kv_length, float scale, float *out) {
    if (head_dim > 512 || n_kv_heads == 0) return;
    const uint32_t group = n_heads / n_kv_heads;
    const size_t row = (size_t)n_kv_heads * head_dim;
    const int64_t work = (int64_t)tokens * n_heads;
#pragma omp parallel
    {
        double *scores =
            (double *)malloc(((size_t)position_base + tokens + 1) * sizeof(double));
#pragma omp for schedule(dynamic, 8)
        for (int64_t w = 0; w < work; w++) {
            const uint32_t t = (uint32_t)(w / n_heads);
            const uint32_t h = (uint32_t)(w % n_heads);
            const uint32_t visible = position_base + t + 1;
            if (visible > kv_length) continue; /* :244 */
            const uint32_t kv_head = h / group;
            attend_row(q + ((size_t)t * n_heads + h) * head_dim, head_dim, scale,
                       k_rows + (size_t)kv_head * head_dim,
                       v_rows + (size_t)kv_head * head_dim, visible, NULL, NULL,
                       0, row, scores,
                       out + ((size_t)t * n_heads + h) * head_dim);
        }
        free(scores);
    }
}

/* src/q3_forward.cu:418-525 */
void q3o_attention_segmented(
    const float *q, const float *prefix_k, const float *prefix_v,
    uint32_t prefix_len, uint32_t prefix_capacity, const float *suffix_k,
    const float *suffix_v, uint32_t suffix_capacity, uint32_t suffix_num_layers,
    uint32_t suffix_layer, const uint32_t *token_branch,
    const uint32_t *token_local_pos, uint32_t tokens, uint32_t n_heads,
    uint32_t n_kv_heads, uint32_t head_dim, float scale, float *out) {
    if (head_dim > 512 || n_kv_heads == 0) return;
    const uint32_t group = n_heads / n_kv_heads;
    const size_t row = (size_t)n_kv_heads * head_dim;
    const size_t prefix_layer_base = (size_t)suffix_layer * prefix_capacity * row;
    const int64_t work = (int64_t)tokens * n_heads;
#pragma omp parallel
    {
        double *scores = (double *)malloc(
            ((size_t)prefix_len + suffix_capacity + 1) * sizeof(double));
#pragma omp for schedule(dynamic, 8)
        for (int64_t w = 0; w < work; w++) {
            const uint32_t t = (uint32_t)(w / n_heads);
            const uint32_t h = (uint32_t)(w % n_heads);
            const uint32_t kv_head = h / group;
            const uint32_t b = token_branch[t];
            const uint32_t lp = token_local_pos[t];
            const size_t branch_base =
                ((size_t)b * suffix_num_layers + suffix_layer) * suffix_capacity * row;
            attend_row(q + ((size_t)t * n_heads + h) * head_dim, head_dim, scale,
                       prefix_k + prefix_layer_base + (size_t)kv_head * head_dim,
                       prefix_v + prefix_layer_base + (size_t)kv_head * head_dim,
                       prefix_len,
                       suffix_k + branch_base + (size_t)kv_head * head_dim,
                       suffix_v + branch_base + (size_t)kv_head * head_dim,
                       lp + 1, row, scores,
                       out + ((size_t)t * n_heads + h) * head_dim);
        }
        free(scores);
    }
}

/* src/q3_forward.cu:529-550 */
void q3o_kv_scatter(float *suffix_k, float *suffix_v, const float *k_src,
                    const float *v_src, const uint32_t *token_branch,
                    const uint32_t *token_local_pos, uint32_t tokens,
                    uint32_t row, uint32_t suffix_capacity, uint32_t num_layers,
                    uint32_t layer) {
    for (uint32_t t = 0; t < tokens; t++) {
        const size_t dst =
            ((size_t)token_branch[t] * num_layers + layer) * suffix_capacity * row +
            (size_t)token_local_pos[t] * row;
        memcpy(suffix_k + dst, k_src + (size_t)t * row, (size_t)row * sizeof(float));
        memcpy(suffix_v + dst, v_src + (size_t)t * row, (size_t)row * sizeof(float));
    }
}

void q3o_attention_decode(const float *q, const float *k_rows,
                          const float *v_rows, uint32_t ctx, uint32_t n_heads,
                          uint32_t n_kv_heads, uint32_t head_dim, float scale,
                          float *out) {
    if (ctx == 0) return;
    q3o_attention(q, k_rows, v_rows, 1, n_heads, n_kv_heads, head_dim, ctx - 1,
                  ctx, scale, out);
}
