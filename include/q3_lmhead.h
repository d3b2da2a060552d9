/* q3_lmhead.h - C ABI of the consumer of the attention path's last rows: the
 * last-row gather and the batched selected-row LM head of the packed decision
 * forward, rebuilt for B200 (sm_100a).
 *
 * In the reference both are file-static kernels inside its forward
 * (gather_last_rows_kernel, src/q3_forward.cu:553-564, launched :1866-1872;
 * candidate_logits_batched_kernel, :566-607, launched :1884-1894) followed by a
 * host softmax/argmax (src/q3_decide.cu:517-553). Here they are exported with
 * the same argument meaning, plus one fused launch that does both and the
 * per-branch argmax. Conventions: device pointers, `void *stream` is a
 * cudaStream_t, nothing synchronises or allocates, `bool` + error buffer.
 */
#ifndef Q3_LMHEAD_B200_H
#define Q3_LMHEAD_B200_H

#include <stdbool.h>
#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* out[b][0..hidden) = src[branch_offsets[b + 1] - 1][0..hidden): the hidden
 * state of the last packed token of every branch (ref: src/q3_forward.cu:553-564).
 * branch_offsets: device array of branch_count + 1 packed-token offsets. */
bool q3_cuda_gather_last_rows(const float *src, const uint32_t *branch_offsets,
                              uint32_t branch_count, uint32_t hidden, float *out,
                              void *stream, char *error, size_t error_len);

/* logits[b * candidate_count + c] = row(candidate_ids[b * candidate_count + c])
 * of the quantised output weight (qtype 12 = Q4_K, 14 = Q6_K, rows of
 * hidden_size / 256 blocks) dotted with hidden_per_branch[b]
 * (ref: src/q3_forward.cu:566-607). Ids >= vocab_size are an error the kernel
 * reports by writing NaN for that logit. */
bool q3_cuda_candidate_logits_batched(const float *hidden_per_branch, const void *weight,
                                      uint32_t qtype, uint32_t hidden_size,
                                      uint32_t vocab_size, const uint32_t *candidate_ids,
                                      uint32_t candidate_count, uint32_t branch_count,
                                      float *logits, void *stream, char *error,
                                      size_t error_len);

/* Both steps and the decision in one launch (no counterpart in the reference,
 * which gathers, computes logits, copies them to the host and takes the
 * argmax there): rows are read straight from the packed hidden states
 * `hidden_rows` [tokens][hidden_size]; best[b] = index in 0..candidate_count
 * of the largest logit of branch b (first one on ties); `best` may be NULL. */
bool q3_cuda_candidate_head(const float *hidden_rows, const uint32_t *branch_offsets,
                            const void *weight, uint32_t qtype, uint32_t hidden_size,
                            uint32_t vocab_size, const uint32_t *candidate_ids,
                            uint32_t candidate_count, uint32_t branch_count, float *logits,
                            uint32_t *best, void *stream, char *error, size_t error_len);

#ifdef __cplusplus
}
#endif

#endif /* Q3_LMHEAD_B200_H */
