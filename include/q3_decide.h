/* q3_decide.h - the decision-batch entry point of the sera.c runtime on the
 * B200 attention path: one call that validates a batch of private suffix
 * branches, packs them, runs the packed suffix pass layer by layer over
 * [shared prefix | own suffix], scores each branch's candidates with the
 * selected-row LM head, synchronises once and fills the results.
 *
 * The types q3_decision_item / q3_decision_batch / q3_decision_result /
 * q3_decide_stats and q3_decide_result_softmax are the reference's
 * (ref: src/q3_decide.h:28-86,153); q3_decide_run keeps the reference's
 * validation, packing, error messages and result semantics
 * (ref: src/q3_decide.cu:369-553). What differs: the runtime is the attention
 * runtime of q3_attn.h, and everything of the model that is not the attention
 * slice (embedding, projections, MLP, final norm) stays with the caller, who
 * hands in per-layer q/k/v buffers and a hook that is called between layers -
 * the reference reaches those parts through its own q3_forward_run_packed.
 */
#ifndef Q3_DECIDE_B200_H
#define Q3_DECIDE_B200_H

#include <stdbool.h>
#include <stddef.h>
#include <stdint.h>

#include "q3_attn.h"

#ifdef __cplusplus
extern "C" {
#endif

#define Q3_MAX_BRANCHES Q3_PACK_MAX_BRANCHES
/* ref: src/q3_forward.h:206 */
#define Q3_MAX_CANDIDATES 30u

/* ref: src/q3_decide.h:28-34 - one decision question: a private suffix plus
 * the candidate rows to score. `tokens` is handed to the caller's hook
 * untouched (this library never embeds); only token_count matters here. */
typedef struct {
    uint32_t branch;               /* handle from q3_branch_acquire            */
    const uint32_t *tokens;        /* suffix token ids, host                   */
    uint32_t token_count;
    const uint32_t *candidate_ids; /* [candidate_count], host                  */
    uint32_t candidate_count;
} q3_decision_item;

/* ref: src/q3_decide.h:36-39 */
typedef struct {
    const q3_decision_item *items;
    uint32_t count;                /* B: 1..Q3_MAX_BRANCHES                    */
} q3_decision_batch;

/* ref: src/q3_decide.h:43-48 */
typedef struct {
    uint32_t predicted_index;      /* argmax over this branch's candidates     */
    uint32_t candidate_count;
    float logits[Q3_MAX_CANDIDATES];
    float probabilities[Q3_MAX_CANDIDATES];
} q3_decision_result;

/* ref: src/q3_decide.h:50-86, field for field. The reference fills the
 * counters with literals (cuda_allocations = 0, host_syncs = 1); here they are
 * measured: differences of the runtime's counters across the call. Timings are
 * CUDA-event times of the two phases of this call. Fields that belong to the
 * reference's cold path (prefix_prefill_ms, branch_create_ms, cold / warm
 * totals, accuracy) are left 0 for the caller to fill. */
typedef struct q3_decide_stats {
    double prefix_prefill_ms;
    double branch_create_ms;
    double suffix_forward_ms;
    double candidate_head_ms;
    double cold_total_ms;
    double warm_total_ms;

    double suffix_questions_per_s;
    double warm_ms_per_question;

    size_t prefix_kv_bytes_physical;
    size_t expected_prefix_kv_bytes;
    size_t suffix_kv_bytes;
    size_t workspace_bytes;
    size_t peak_cuda_bytes;

    uint64_t prefix_allocations;   /* 0: prefix pages come from the pool       */
    uint64_t prefix_bytes;
    uint64_t prefix_copy_calls;    /* 0: the prefix is never copied            */
    uint64_t prefix_copy_bytes;
    uint64_t suffix_allocations;   /* 0: branch pages come from the pool       */
    uint64_t suffix_bytes;

    uint64_t cuda_allocations;     /* measured; 0 in a warm batch              */
    uint64_t cuda_frees;
    uint64_t host_syncs;           /* measured; 1 in a warm batch              */

    uint64_t kernel_launches_per_batch;
    uint64_t kernel_launches_per_question;

    uint32_t batch;
    uint32_t suffix_tokens_total;

    uint32_t accuracy_matches;
    uint32_t accuracy_total;
} q3_decide_stats;

/* The caller's side of the packed forward. All device pointers; q/k/v and
 * attn_out are arrays of num_layers pointers (bf16 [tokens][heads][128] in
 * packed branch order, attn_out fp32 when the runtime was created with
 * out_fp32). Layers 0..num_layers-1 run in order on the runtime's stream;
 * after layer l, `between_layers` (optional) is called with that stream so the
 * caller can queue the rest of the layer - output projection, MLP, the next
 * layer's q/k/v - before layer l+1 reads its buffers. After the last hook,
 * `final_hidden` must hold the final-norm hidden rows fp32 [tokens][hidden_size]
 * from which the head reads each branch's last row
 * (ref: gather_last_rows_kernel + candidate_logits_batched_kernel,
 * src/q3_forward.cu:553-607). */
typedef struct {
    uint32_t num_layers;
    const void *const *q;
    const void *const *k;
    const void *const *v;
    void *const *attn_out;
    bool (*between_layers)(void *user, uint32_t layer_done, const uint32_t *packed_token_ids,
                           uint32_t tokens, void *stream);
    void *user;
    const float *final_hidden;
    uint32_t hidden_size;
    const void *lm_head;           /* quantised output weight rows               */
    uint32_t lm_head_qtype;        /* 12 = Q4_K, 14 = Q6_K                       */
    uint32_t vocab_size;
} q3_decide_model_io;

/* ref: src/q3_decide.h:147-150, src/q3_decide.cu:369-553. Validates as the
 * reference does (same messages), packs tight (no padding rows), runs the
 * layers, the candidate head (logits and per-branch argmax in one launch),
 * synchronises ONCE and fills results[0..batch->count-1] with logits, host
 * softmax probabilities and predicted_index. The staging buffers live in the
 * branch set and grow once: a warm batch (same or smaller shape than an earlier
 * one) performs no allocation and exactly one host synchronisation, which
 * `stats` (optional) reports as measured. */
bool q3_decide_run(q3_attn_runtime *runtime, q3_prefix_kv *prefix, q3_branch_set *set,
                   const q3_decision_batch *batch, const q3_decide_model_io *model,
                   q3_decision_result *results, q3_decide_stats *stats, char *error,
                   size_t error_len);

/* ref: src/q3_decide.h:153 - softmax over one result's candidate logits. */
void q3_decide_result_softmax(q3_decision_result *result);

#ifdef __cplusplus
}
#endif

#endif /* Q3_DECIDE_B200_H */
