/* q3_attn_oracle.h - CPU restatement of the sera.c Qwen3-32B attention path.
 *
 * TEST INFRASTRUCTURE ONLY. Nothing in the shipped library links, loads or
 * calls this file; it exists so the parity tests, the smoke check and the
 * timed CPU baseline have something independent of the CUDA kernels to
 * compare against.
 *
 * Every function restates one function of the reference (path inside the
 * sera.c project given beside each declaration). Accumulation is in double
 * and sin/cos/exp use the precise libm routines, so the oracle is the
 * "fp32 reference" the tolerance of the path is quoted against.
 *
 * Pinning: the oracle is checked (a) against golden vectors produced by the
 * HuggingFace Qwen3 functions the reference's Python oracle calls
 * (tests/golden/make_golden_hf.py), and (b) against the reference's own CUDA
 * kernels compiled from its sources and run on the GPU box (oracle/_ref,
 * tests/golden/make_golden_refkernels.py).
 */
#ifndef Q3_ATTN_ORACLE_H
#define Q3_ATTN_ORACLE_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* inv_freq[i] = 1 / theta^(2i/head_dim), computed in double, stored fp32.
 * Reference: src/q3_forward.cu:1128-1130. */
void q3o_inv_freq(double theta, uint32_t head_dim, float *inv_freq);

/* out = x * (1/sqrt(mean(x^2)+eps)) * w, row by row. In-place allowed.
 * Reference: src/q3_forward.cu:117-148 (kernel) and
 * tests/test_q3_forward_primitives.cu:46-56 (the reference's own CPU loop). */
void q3o_rms_norm(const float *input, const float *weight, uint32_t rows,
                  uint32_t width, float epsilon, float *output);

/* NeoX half-split RoPE on q [T][n_heads][D] and k [T][n_kv_heads][D], in
 * place. angle = (float)position * inv_freq[p] is formed in fp32 exactly as
 * the reference does; cos/sin of that fp32 angle are evaluated in double.
 * position = position_base + token when token_positions is NULL.
 * Reference: src/q3_forward.cu:181-209, :380-410 and
 * tests/test_q3_forward_primitives.cu:58-85. */
void q3o_rope(float *q, float *k, uint32_t tokens, uint32_t n_heads,
              uint32_t n_kv_heads, uint32_t head_dim, uint32_t position_base,
              const uint32_t *token_positions, const float *inv_freq);

/* Causal GQA attention of `tokens` query rows over a K/V slab whose rows are
 * [position][n_kv_heads][D]; token t sees keys 0..position_base+t.
 * Rows with position_base+t+1 > kv_length are left untouched (reference
 * behaviour). Reference: src/q3_forward.cu:218-290. */
void q3o_attention(const float *q, const float *k_rows, const float *v_rows,
                   uint32_t tokens, uint32_t n_heads, uint32_t n_kv_heads,
                   uint32_t head_dim, uint32_t position_base,
                   uint32_t kv_length, float scale, float *out);

/* Two-segment attention [shared prefix 0..P-1 | own branch suffix 0..lp].
 * Argument meaning identical to q3_cuda_attention_segmented.
 * Reference: src/q3_forward.cu:418-525. */
void q3o_attention_segmented(
    const float *q, const float *prefix_k, const float *prefix_v,
    uint32_t prefix_len, uint32_t prefix_capacity, const float *suffix_k,
    const float *suffix_v, uint32_t suffix_capacity, uint32_t suffix_num_layers,
    uint32_t suffix_layer, const uint32_t *token_branch,
    const uint32_t *token_local_pos, uint32_t tokens, uint32_t n_heads,
    uint32_t n_kv_heads, uint32_t head_dim, float scale, float *out);

/* Scatter packed K/V rows into the per-branch suffix arena
 * [branch][layer][suffix_capacity][row]. Reference: src/q3_forward.cu:529-550. */
void q3o_kv_scatter(float *suffix_k, float *suffix_v, const float *k_src,
                    const float *v_src, const uint32_t *token_branch,
                    const uint32_t *token_local_pos, uint32_t tokens,
                    uint32_t row, uint32_t suffix_capacity, uint32_t num_layers,
                    uint32_t layer);

/* Single-query attention over a gathered context (decode): q [n_heads][D],
 * keys/values [ctx][n_kv_heads][D]. Same arithmetic as q3o_attention with one
 * token at position ctx-1. */
void q3o_attention_decode(const float *q, const float *k_rows,
                          const float *v_rows, uint32_t ctx, uint32_t n_heads,
                          uint32_t n_kv_heads, uint32_t head_dim, float scale,
                          float *out);

/* Number of OpenMP threads the oracle will use (1 when built without it). */
int q3o_threads(void);
void q3o_set_threads(int n);

#ifdef __cplusplus
}
#endif

#endif /* Q3_ATTN_ORACLE_H */
