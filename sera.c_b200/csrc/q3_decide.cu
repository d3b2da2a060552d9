/* q3_decide.cu - q3_decide_run on the paged attention runtime: validation,
 * packing and result handling of the reference's decision-batch entry point
 * (ref: src/q3_decide.cu:369-553), driving q3_suffix_attention_layer per layer
 * and the fused candidate head. Host code only.
 */
#include "q3_internal.h"

#include <math.h>

#include <new>

#include "q3_decide.h"
#include "q3_lmhead.h"

/* Scratch of q3_decide_run, owned by the branch set, grown once: the staged
 * descriptors (shared with the plan path), candidate ids / logits / argmax on
 * the device with pinned mirrors, and the phase events. */
struct q3_decide_state {
    q3_stage *stage;
    q3_pack_plan plan;            /* borrows `stage` */
    uint8_t *host;                /* pinned */
    uint8_t *dev;
    size_t bytes;
    cudaEvent_t uploaded;         /* the copy out of `host` (ids, offsets) was consumed */
    cudaEvent_t ev[3];            /* layers begin / head begin / head end */
    bool events_ready;
    std::vector<uint32_t> token_ids;
    std::vector<q3_suffix_item> items;
};

void q3_decide_state_destroy(q3_branch_set *set) {
    q3_decide_state *d = set->decide;
    if (!d) return;
    q3_attn_runtime *rt = set->prefix->rt;
    if (rt->stream) cudaStreamSynchronize(rt->stream);
    q3_stage_destroy(d->stage);
    if (d->events_ready) {
        cudaEventDestroy(d->uploaded);
        for (int i = 0; i < 3; i++) cudaEventDestroy(d->ev[i]);
    }
    if (d->host) cudaFreeHost(d->host);
    if (d->dev) {
        cudaFree(d->dev);
        rt->n_free++;
    }
    delete d;
    set->decide = nullptr;
}

static q3_decide_state *decide_state(q3_branch_set *set, size_t need, char *error,
                                     size_t error_len) {
    q3_attn_runtime *rt = set->prefix->rt;
    q3_decide_state *d = set->decide;
    if (!d) {
        d = new (std::nothrow) q3_decide_state();
        if (!d) {
            q3_fail(error, error_len, "q3_decide_run: allocation failed");
            return NULL;
        }
        d->stage = q3_stage_create(rt, error, error_len);
        d->host = d->dev = nullptr;
        d->bytes = 0;
        d->events_ready = false;
        if (!d->stage) {
            delete d;
            return NULL;
        }
        bool ok = cudaEventCreateWithFlags(&d->uploaded, cudaEventDisableTiming) == cudaSuccess;
        for (int i = 0; i < 3 && ok; i++) ok = cudaEventCreate(&d->ev[i]) == cudaSuccess;
        if (!ok) {
            q3_stage_destroy(d->stage);
            delete d;
            q3_fail(error, error_len, "q3_decide_run: event creation failed");
            return NULL;
        }
        d->events_ready = true;
        set->decide = d;
    }
    if (need > d->bytes) {
        /* growth is set-up (counted): a warm batch never gets here */
        cudaStreamSynchronize(rt->stream);
        rt->n_sync++;
        if (d->host) cudaFreeHost(d->host);
        if (d->dev) {
            cudaFree(d->dev);
            rt->n_free++;
        }
        d->host = d->dev = nullptr;
        d->bytes = 0;
        const size_t cap = need + need / 2;
        if (cudaHostAlloc((void **)&d->host, cap, cudaHostAllocDefault) != cudaSuccess ||
            cudaMalloc((void **)&d->dev, cap) != cudaSuccess) {
            q3_fail(error, error_len, "q3_decide_run: allocation failed");
            return NULL;
        }
        rt->n_alloc++;
        rt->workspace_bytes += cap;
        d->bytes = cap;
    }
    return d;
}

extern "C" void q3_decide_result_softmax(q3_decision_result *result) {
    if (!result || result->candidate_count == 0 ||
        result->candidate_count > Q3_MAX_CANDIDATES)
        return;
    const uint32_t n = result->candidate_count;
    float mx = result->logits[0];
    for (uint32_t i = 1; i < n; i++) mx = fmaxf(mx, result->logits[i]);
    float sum = 0.f;
    for (uint32_t i = 0; i < n; i++) {
        result->probabilities[i] = expf(result->logits[i] - mx);
        sum += result->probabilities[i];
    }
    if (sum > 0.f)
        for (uint32_t i = 0; i < n; i++) result->probabilities[i] /= sum;
}

extern "C" bool q3_decide_run(q3_attn_runtime *runtime, q3_prefix_kv *prefix,
                              q3_branch_set *set, const q3_decision_batch *batch,
                              const q3_decide_model_io *model, q3_decision_result *results,
                              q3_decide_stats *stats, char *error, size_t error_len) {
    q3_clear_error(error, error_len);
    if (!runtime || !prefix || !set || !batch || !batch->items || !results || !model ||
        !model->q || !model->k || !model->v || !model->attn_out || !model->final_hidden ||
        !model->lm_head || model->num_layers == 0)
        return q3_fail(error, error_len, "q3_decide_run: invalid argument");
    const uint32_t B = batch->count;
    if (B == 0 || B > Q3_MAX_BRANCHES || B > set->max_branches)
        return q3_fail(error, error_len, "q3_decide_run: bad branch count");
    if (!prefix->sealed) return q3_fail(error, error_len, "q3_decide_run: prefix not sealed");
    if (prefix->rt != runtime)
        return q3_fail(error, error_len, "q3_decide_run: prefix belongs to another runtime");
    if (model->num_layers > runtime->cfg.num_layers)
        return q3_fail(error, error_len, "q3_decide_run: more layers than the runtime holds");
    /* one uniform candidate count for the whole batch: the head writes a dense
     * [B, K] tile (ref: src/q3_decide.cu:396-402) */
    const uint32_t K = batch->items[0].candidate_count;
    if (K == 0 || K > Q3_MAX_CANDIDATES)
        return q3_fail(error, error_len, "q3_decide_run: bad candidate count");
    uint64_t packed = 0;
    for (uint32_t b = 0; b < B; b++) {
        const q3_decision_item *item = &batch->items[b];
        if (!item->tokens || item->token_count == 0 || item->token_count > set->max_suffix ||
            !item->candidate_ids || item->candidate_count != K)
            return q3_fail(error, error_len, "q3_decide_run: invalid decision item");
        if (item->branch >= set->max_branches)
            return q3_fail(error, error_len, "q3_decide_run: invalid branch handle");
        packed += item->token_count;
    }
    if (packed > runtime->cfg.max_tokens)
        return q3_fail(error, error_len,
                       "q3_decide_run: packed batch exceeds runtime capacity");
    if (!q3_use_device(runtime, error, error_len)) return false;

    const uint64_t alloc0 = runtime->n_alloc, free0 = runtime->n_free;
    const uint64_t sync0 = runtime->n_sync, launch0 = runtime->n_launch;

    /* device scratch: [candidate ids B*K | branch offsets B+1 | logits B*K | best B] */
    auto al = [](size_t x) { return (x + 15) & ~(size_t)15; };
    const size_t o_ids = 0;
    const size_t o_off = al(o_ids + (size_t)B * K * 4);
    const size_t o_log = al(o_off + (size_t)(B + 1) * 4);
    const size_t o_best = al(o_log + (size_t)B * K * 4);
    const size_t need = al(o_best + (size_t)B * 4);
    q3_decide_state *d = decide_state(set, need, error, error_len);
    if (!d) return false;

    /* packing, exactly the reference's (ref: src/q3_decide.cu:440-464) */
    d->items.resize(B);
    d->token_ids.resize(packed);
    {
        size_t cursor = 0;
        for (uint32_t b = 0; b < B; b++) {
            const q3_decision_item *item = &batch->items[b];
            d->items[b].branch = item->branch;
            d->items[b].token_count = item->token_count;
            for (uint32_t j = 0; j < item->token_count; j++)
                d->token_ids[cursor + j] = item->tokens[j];
            cursor += item->token_count;
        }
    }
    if (!q3_pack_plan_build(&d->plan, d->stage, prefix, set, d->items.data(), B,
                            "q3_decide_run", error, error_len))
        return false;
    /* the previous batch's copy out of the pinned mirror was consumed long ago */
    if (cudaEventQuery(d->uploaded) != cudaSuccess) {
        cudaEventSynchronize(d->uploaded);
        runtime->n_sync++;
    }
    uint32_t *h_ids = (uint32_t *)(d->host + o_ids);
    uint32_t *h_off = (uint32_t *)(d->host + o_off);
    for (uint32_t b = 0; b < B; b++)
        for (uint32_t k = 0; k < K; k++) h_ids[b * K + k] = batch->items[b].candidate_ids[k];
    memcpy(h_off, d->plan.branch_offsets.data(), (size_t)(B + 1) * 4);
    cudaError_t e = cudaMemcpyAsync(d->dev, d->host, o_log, cudaMemcpyHostToDevice,
                                    runtime->stream);
    if (e == cudaSuccess) e = cudaEventRecord(d->uploaded, runtime->stream);
    if (e == cudaSuccess) e = cudaEventRecord(d->ev[0], runtime->stream);
    if (e != cudaSuccess) return q3_fail_cuda(error, error_len, "q3_decide_run: upload", e);

    /* the packed suffix pass: two launches per layer */
    for (uint32_t l = 0; l < model->num_layers; l++) {
        if (!model->q[l] || !model->k[l] || !model->v[l] || !model->attn_out[l])
            return q3_fail(error, error_len, "q3_decide_run: missing layer buffer");
        if (!q3_suffix_attention_layer(&d->plan, l, model->q[l], model->k[l], model->v[l],
                                       model->attn_out[l], error, error_len))
            return false;
        if (model->between_layers &&
            !model->between_layers(model->user, l, d->token_ids.data(), d->plan.tokens,
                                   (void *)runtime->stream))
            return q3_fail(error, error_len, "q3_decide_run: the caller's layer hook failed");
    }
    cudaEventRecord(d->ev[1], runtime->stream);

    /* last-row gather + selected-row head + per-branch argmax: one launch */
    float *logits_dev = (float *)(d->dev + o_log);
    uint32_t *best_dev = (uint32_t *)(d->dev + o_best);
    if (!q3_cuda_candidate_head(model->final_hidden, (const uint32_t *)(d->dev + o_off),
                                model->lm_head, model->lm_head_qtype, model->hidden_size,
                                model->vocab_size, (const uint32_t *)(d->dev + o_ids), K, B,
                                logits_dev, best_dev, (void *)runtime->stream, error,
                                error_len))
        return false;
    runtime->n_launch++;
    cudaEventRecord(d->ev[2], runtime->stream);
    e = cudaMemcpyAsync(d->host + o_log, d->dev + o_log, need - o_log, cudaMemcpyDeviceToHost,
                        runtime->stream);
    if (e != cudaSuccess) return q3_fail_cuda(error, error_len, "q3_decide_run: logits copy", e);

    /* the one explicit measurement-boundary sync (ref: src/q3_decide.cu:499-500) */
    if (!q3_attn_synchronize(runtime, error, error_len)) return false;

    const float *h_log = (const float *)(d->host + o_log);
    const uint32_t *h_best = (const uint32_t *)(d->host + o_best);
    for (uint32_t b = 0; b < B; b++) {
        q3_decision_result *r = &results[b];
        r->candidate_count = K;
        for (uint32_t k = 0; k < K; k++) r->logits[k] = h_log[b * K + k];
        q3_decide_result_softmax(r);
        r->predicted_index = h_best[b] < K ? h_best[b] : 0;
    }

    if (stats) {
        memset(stats, 0, sizeof(*stats));
        float ms = 0.f;
        if (cudaEventElapsedTime(&ms, d->ev[0], d->ev[1]) == cudaSuccess)
            stats->suffix_forward_ms = ms;
        if (cudaEventElapsedTime(&ms, d->ev[1], d->ev[2]) == cudaSuccess)
            stats->candidate_head_ms = ms;
        const q3_attn_config &c = runtime->cfg;
        stats->prefix_kv_bytes_physical = q3_prefix_kv_bytes(prefix);
        /* the paged pool holds f16: half the reference's fp32 figure */
        stats->expected_prefix_kv_bytes =
            q3_kv_bytes_for_tokens(prefix->token_count, c.num_layers, c.n_kv_heads, Q3_D) / 2;
        stats->suffix_kv_bytes = q3_branch_set_kv_bytes(set);
        stats->workspace_bytes = runtime->workspace_bytes;
        stats->prefix_bytes = q3_prefix_kv_bytes(prefix);
        stats->suffix_bytes = q3_branch_set_kv_bytes(set);
        stats->prefix_allocations = q3_prefix_allocations(prefix);
        stats->prefix_copy_bytes = q3_prefix_copy_bytes(prefix);
        stats->cuda_allocations = runtime->n_alloc - alloc0;
        stats->cuda_frees = runtime->n_free - free0;
        stats->host_syncs = runtime->n_sync - sync0;
        stats->kernel_launches_per_batch = runtime->n_launch - launch0;
        stats->kernel_launches_per_question = stats->kernel_launches_per_batch / B;
        stats->batch = B;
        stats->suffix_tokens_total = d->plan.tokens;
        if (stats->suffix_forward_ms + stats->candidate_head_ms > 0.0) {
            stats->warm_total_ms = stats->suffix_forward_ms + stats->candidate_head_ms;
            stats->warm_ms_per_question = stats->warm_total_ms / B;
            stats->suffix_questions_per_s = 1e3 * B / stats->warm_total_ms;
        }
    }
    return true;
}
