/* q3_attn.h - C ABI of the B200 (sm_100a) attention path for the sera.c
 * Qwen3-32B runtime: QK-RMSNorm + RoPE + paged f16 KV write, causal GQA
 * prefill, shared-prefix + packed-suffix attention, paged decode.
 *
 * Part 1 keeps the reference's primitive surface symbol for symbol (fp32
 * device pointers, void* stream, never synchronises) so the reference's own
 * run_layer / run_layer_packed and its tests link against this library
 * unchanged. Part 2 is the native path (bf16 activations, paged f16 KV,
 * tcgen05 kernels) behind the same conventions: bool / NULL / -1 on failure
 * plus a caller-supplied error buffer that is cleared on entry, opaque
 * handles, no allocation and no host synchronisation in the warm path.
 *
 * Citations "ref:" are paths inside the sera.c project.
 */
#ifndef Q3_ATTN_H
#define Q3_ATTN_H

#include <stdbool.h>
#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* ======================================================================
 * Part 1 - reference-identical surface (fp32, contiguous KV slabs)
 * ====================================================================== */

/* ref: src/q3_forward.h:82-91 - contiguous fp32 KV cache
 * [layer][capacity][kv_heads][head_dim]. */
typedef struct q3_kv_cache q3_kv_cache;

q3_kv_cache *q3_kv_cache_init(uint32_t num_layers, uint32_t num_kv_heads,
                              uint32_t head_dim, uint32_t capacity,
                              char *error, size_t error_len);
bool q3_kv_cache_reserve(q3_kv_cache *kv, uint32_t capacity,
                         char *error, size_t error_len);
void q3_kv_cache_reset(q3_kv_cache *kv);
void q3_kv_cache_destroy(q3_kv_cache *kv);
uint32_t q3_kv_cache_length(const q3_kv_cache *kv);
/* ref: src/q3_forward.h:278-281 - header that borrows slabs it does not own. */
q3_kv_cache *q3_kv_cache_alias(float *k, float *v, uint32_t num_layers,
                               uint32_t num_kv_heads, uint32_t head_dim,
                               uint32_t capacity, uint32_t length,
                               char *error, size_t error_len);
/* Not in the reference header: the reference advances `length` inside
 * q3_forward_run_range (ref: src/q3_forward.cu:1423); a caller that drives the
 * primitives layer by layer needs to do the same. */
void q3_kv_cache_advance(q3_kv_cache *kv, uint32_t tokens);
/* Device bases of the slabs, for a caller that appends rows itself
 * (ref: src/q3_forward.cu:1268-1278 does this with two cudaMemcpyAsync). */
float *q3_kv_cache_k(const q3_kv_cache *kv);
float *q3_kv_cache_v(const q3_kv_cache *kv);

/* ref: src/q3_forward.h:177-179, kernel src/q3_forward.cu:117-148 */
bool q3_cuda_rms_norm(const float *input, const float *weight, uint32_t rows,
                      uint32_t width, float epsilon, float *output,
                      void *stream, char *error, size_t error_len);
/* ref: src/q3_forward.h:185-187, kernel src/q3_forward.cu:181-209 */
bool q3_cuda_rope(float *q, float *k, uint32_t tokens, uint32_t n_heads,
                  uint32_t n_kv_heads, uint32_t head_dim, uint32_t position_base,
                  const float *inv_freq, void *stream, char *error, size_t error_len);
/* ref: src/q3_forward.h:252-256, kernel src/q3_forward.cu:380-410 */
bool q3_cuda_rope_positions(float *q, float *k, uint32_t tokens,
                            uint32_t n_heads, uint32_t n_kv_heads,
                            uint32_t head_dim, const uint32_t *token_positions,
                            const float *inv_freq, void *stream, char *error,
                            size_t error_len);
/* ref: src/q3_forward.h:188-192, kernel src/q3_forward.cu:218-290.
 * kv == NULL: keys are the call's own k/v rows; else the cache slab of
 * `layer`, visible length kv->length + tokens. */
bool q3_cuda_attention(const float *q, const float *k, const float *v,
                       uint32_t tokens, uint32_t n_heads, uint32_t n_kv_heads,
                       uint32_t head_dim, uint32_t position_base,
                       q3_kv_cache *kv, uint32_t layer, float scale, float *out,
                       void *stream, char *error, size_t error_len);
/* ref: src/q3_forward.h:262-272, kernel src/q3_forward.cu:418-525.
 * token_branch / token_local_pos must be DEVICE pointers (the reference hands
 * its kernels host malloc memory, which only works on unified-memory parts). */
bool q3_cuda_attention_segmented(const float *q, const float *prefix_k,
                                 const float *prefix_v, uint32_t prefix_len,
                                 uint32_t prefix_capacity, const float *suffix_k,
                                 const float *suffix_v, uint32_t suffix_capacity,
                                 uint32_t suffix_num_layers,
                                 uint32_t suffix_layer,
                                 const uint32_t *token_branch,
                                 const uint32_t *token_local_pos, uint32_t tokens,
                                 uint32_t n_heads, uint32_t n_kv_heads,
                                 uint32_t head_dim, float scale, float *out,
                                 void *stream, char *error, size_t error_len);
/* The two attention entries above through the tensor-core kernel (not in the
 * reference). After q3_cuda_attention_native_init(device, max_tokens,
 * max_kv_tokens, n_heads, n_kv_heads) - the one place this surface allocates:
 * an f16 page pool for max_kv_tokens keys, a query workspace, schedule staging -
 * a call with head_dim 128, 8 query heads per KV head, scale = 128^-0.5 and
 * sizes within those limits converts q and the visible K/V slab rows to f16,
 * runs attention_tc_kernel and writes fp32 `out`, on the caller's stream and
 * without synchronising. q3_cuda_attention_segmented additionally needs
 * token_branch / token_local_pos in memory the HOST can read (pageable, pinned
 * or managed - where the reference's own caller keeps them), because the launch
 * schedule is built on the host; with device-only descriptors, or any other
 * geometry, the exact fp32 kernels run as before. Operands are rounded to f16
 * on this path (agreement with the fp32 kernels about 1e-3, not 1e-4).
 * q3_cuda_attention_last_path() names the path of the last call ("tensor-core"
 * or "simt"); q3_cuda_attention_native_synchronize synchronises the last
 * caller stream used and reports a bounded device wait that gave up. */
bool q3_cuda_attention_native_init(int device, uint32_t max_tokens, uint32_t max_kv_tokens,
                                   uint32_t n_heads, uint32_t n_kv_heads, char *error,
                                   size_t error_len);
void q3_cuda_attention_native_shutdown(int device);
const char *q3_cuda_attention_last_path(void);
bool q3_cuda_attention_native_synchronize(int device, char *error, size_t error_len);

/* The reference's kv_scatter_kernel is file-static (ref: src/q3_forward.cu:529-550,
 * launched at :1507-1515); exported here so run_layer_packed's scatter step has
 * a symbol to call. Same argument meaning as the kernel. */
bool q3_cuda_kv_scatter(float *suffix_k, float *suffix_v, const float *k_src,
                        const float *v_src, const uint32_t *token_branch,
                        const uint32_t *token_local_pos, uint32_t tokens,
                        uint32_t row, uint32_t suffix_capacity,
                        uint32_t num_layers, uint32_t layer, void *stream,
                        char *error, size_t error_len);
/* ref: src/q3_decide.h:89-90 - fp32 K+V bytes of the reference's layout. */
size_t q3_kv_bytes_for_tokens(uint32_t tokens, uint32_t num_layers,
                              uint32_t num_kv_heads, uint32_t head_dim);

/* ======================================================================
 * Part 2 - native paged path (bf16 activations, f16 KV pages, sm_100a)
 * ====================================================================== */

#define Q3_PAGE_TOKENS 16u
/* ref: src/q3_forward.h:205 has 32; raised because the benchmark
 * configurations pack up to 128 branches. Still enforced. */
#define Q3_PACK_MAX_BRANCHES 1024u
/* ref: src/q3_decide.h:25 */
#define Q3_DEFAULT_SUFFIX_CAP 512u
#define Q3_NO_PAGE 0xFFFFFFFFu

/* Stands where q3_forward_runtime stands in the reference
 * (ref: src/q3_forward.h:94-100): one stream, geometry, grow-once workspace.
 * Also owns the KV page pool and the RoPE table. */
typedef struct q3_attn_runtime q3_attn_runtime;

typedef struct {
    uint32_t num_layers;
    uint32_t n_heads;        /* query heads held by THIS runtime (shard)      */
    uint32_t n_kv_heads;     /* KV heads held by THIS runtime; n_heads = 8 *  */
    uint32_t head_dim;       /* must be 128                                   */
    float rms_eps;           /* ref: 1e-6                                     */
    double rope_theta;       /* ref: 1e6                                      */
    uint32_t max_positions;  /* RoPE table rows                               */
    uint32_t max_tokens;     /* query tokens per call (workspace size)        */
    uint32_t num_pages;      /* KV pool size in 16-token pages                */
    uint32_t out_fp32;       /* 0: attention output is bf16 (native); 1: fp32,
                                the reference's dtype, used to measure the
                                kernels' own error without output rounding     */
    int device;
} q3_attn_config;

q3_attn_runtime *q3_attn_create(const q3_attn_config *config, char *error,
                                size_t error_len);
void q3_attn_destroy(q3_attn_runtime *rt);
/* [head_dim] fp32 HOST weights shared by all heads of a layer
 * (ref: src/q3_forward.cu:1246-1253). Default is all ones. */
bool q3_attn_set_qk_norm(q3_attn_runtime *rt, uint32_t layer,
                         const float *q_norm_weight, const float *k_norm_weight,
                         char *error, size_t error_len);
void *q3_attn_stream(const q3_attn_runtime *rt);
/* ref: src/q3_forward.h:163-164 - the explicit measurement-boundary sync. */
bool q3_attn_synchronize(q3_attn_runtime *rt, char *error, size_t error_len);
/* After q3_attn_synchronize reported that a kernel gave up a bounded wait:
 * queues, on the runtime's stream, the clearing of the status word and of the
 * arrival counters that launch may have left part-way. Required before the
 * runtime is used again; results of the launch that timed out are undefined. */
bool q3_attn_reset_status(q3_attn_runtime *rt, char *error, size_t error_len);

typedef struct {
    uint64_t cuda_allocations;   /* since create; constant in the warm path   */
    uint64_t cuda_frees;
    uint64_t host_syncs;
    uint64_t kernel_launches;
    uint64_t pages_total;
    uint64_t pages_free;
    uint64_t pool_bytes;         /* K + V                                     */
    uint64_t workspace_bytes;
    uint32_t device_status;      /* nonzero: a bounded device wait gave up    */
} q3_attn_stats;
void q3_attn_get_stats(const q3_attn_runtime *rt, q3_attn_stats *stats);

/* Per-kernel device times, the counterpart of the reference's phase events
 * (ref: q3_forward_stats qk_norm_ms/rope_ms/attention_ms, src/q3_forward.h:50-75;
 * events at src/q3_forward.cu:1205-1285). When enabled, every launch is
 * bracketed by an event pair on the runtime's stream (up to `max_launches`
 * pairs, created here, none in the warm path). q3_attn_phase_times
 * synchronises the stream, SUMS the pairs recorded since the last call per
 * phase, and rewinds. Phases: 0 fused norm+rope+KV write, 1 tensor-core
 * attention, 2 waits for the other ranks' rows (q3_attn_wait_gathered: the
 * part of the output exchange that is not hidden), 3 paged decode (+ its merge). */
bool q3_attn_enable_timing(q3_attn_runtime *rt, uint32_t max_launches, char *error,
                           size_t error_len);
bool q3_attn_phase_times(q3_attn_runtime *rt, double ms_out[4],
                         uint64_t launches_out[4], char *error, size_t error_len);

/* --- paged KV: page pool ------------------------------------------- *
 * Physical layout, K and V alike: [layer][kv_head][page][16 tokens][128] f16,
 * so one page of one head is 4 KiB contiguous and a KV-head shard is a
 * contiguous slice. A page id names the same slot in every layer and head.
 * Logical addressing is the reference's: position p of a sequence lives in
 * page_table[p / 16], slot p % 16. */
bool q3_pages_alloc(q3_attn_runtime *rt, uint32_t count, uint32_t *pages_out,
                    char *error, size_t error_len);
void q3_pages_free(q3_attn_runtime *rt, const uint32_t *pages, uint32_t count);
/* Device bases of the pools (tests fill / read pages through these). */
void *q3_pages_k(const q3_attn_runtime *rt);
void *q3_pages_v(const q3_attn_runtime *rt);

/* --- shared prefix (ref: src/q3_decide.h:96-116) --------------------- */
typedef struct q3_prefix_kv q3_prefix_kv;
typedef struct q3_branch_set q3_branch_set;

q3_prefix_kv *q3_prefix_create(q3_attn_runtime *rt, uint32_t capacity_tokens,
                               char *error, size_t error_len);
/* Use caller-chosen physical pages (e.g. a permuted table) instead of taking
 * them from the free list. `pages` holds ceil(capacity/16) ids. */
q3_prefix_kv *q3_prefix_create_with_pages(q3_attn_runtime *rt,
                                          uint32_t capacity_tokens,
                                          const uint32_t *pages, char *error,
                                          size_t error_len);
/* One layer of the prefill: fused QK-RMSNorm + RoPE + KV write of `tokens`
 * rows at positions [token_count, token_count + tokens), then causal GQA
 * attention over positions 0..token_count+tokens-1. q/k/v/out are bf16 device
 * [tokens][n_heads|n_kv_heads][128]. Replaces the attention slice of
 * run_layer (ref: src/q3_forward.cu:1244-1286). */
bool q3_prefix_prefill_layer(q3_prefix_kv *prefix, uint32_t layer,
                             const void *q, const void *k, const void *v,
                             uint32_t tokens, void *out, char *error,
                             size_t error_len);
/* After all layers of a chunk: token_count += tokens
 * (ref: src/q3_forward.cu:1423). */
bool q3_prefix_advance(q3_prefix_kv *prefix, uint32_t tokens, char *error,
                       size_t error_len);
/* Declare `token_count` positions already resident (KV written by the caller
 * straight into the pages). */
bool q3_prefix_set_resident(q3_prefix_kv *prefix, uint32_t token_count,
                            char *error, size_t error_len);
bool q3_prefix_seal(q3_prefix_kv *prefix, char *error, size_t error_len);
void q3_prefix_destroy(q3_prefix_kv *prefix);
uint32_t q3_prefix_token_count(const q3_prefix_kv *prefix);
size_t q3_prefix_kv_bytes(const q3_prefix_kv *prefix);
uint64_t q3_prefix_copy_bytes(const q3_prefix_kv *prefix);   /* stays 0 */
uint64_t q3_prefix_allocations(const q3_prefix_kv *prefix);  /* stays 0: pool */
const uint32_t *q3_prefix_page_table(const q3_prefix_kv *prefix);  /* host */

/* --- branch set (ref: src/q3_decide.h:118-139) ----------------------- *
 * max_branches * ceil(max_suffix/16) pages taken once; acquire / reset /
 * release are descriptor-only. */
q3_branch_set *q3_branch_set_create(q3_prefix_kv *prefix, uint32_t max_branches,
                                    uint32_t max_suffix_tokens, char *error,
                                    size_t error_len);
int32_t q3_branch_acquire(q3_branch_set *set, char *error, size_t error_len);
void q3_branch_reset(q3_branch_set *set, int32_t branch);
void q3_branch_release(q3_branch_set *set, int32_t branch);
void q3_branch_set_destroy(q3_branch_set *set);
size_t q3_branch_set_kv_bytes(const q3_branch_set *set);
uint32_t q3_branch_set_max_branches(const q3_branch_set *set);
uint32_t q3_branch_set_max_suffix(const q3_branch_set *set);
const uint32_t *q3_branch_set_page_table(const q3_branch_set *set); /* host [B][pages] */
uint32_t q3_branch_set_pages_per_branch(const q3_branch_set *set);

/* --- packed suffix pass (ref: src/q3_decide.h:28-40, packing at
 *     src/q3_decide.cu:440-464, view at src/q3_forward.h:213-229) -------- */
typedef struct {
    uint32_t branch;        /* handle from q3_branch_acquire */
    uint32_t token_count;   /* suffix tokens of this branch  */
} q3_suffix_item;

/* Host-side packing exactly as q3_decide_run does it: tight, branch b occupies
 * [branch_offsets[b], branch_offsets[b+1]); token_positions = prefix_len + j.
 * Pure host function (no CUDA). Arrays are caller-allocated:
 * token_* hold sum(token_count) entries, branch_offsets count+1. Returns the
 * packed total, or -1 on an invalid item. */
int64_t q3_pack_suffix_host(const q3_suffix_item *items, uint32_t count,
                            uint32_t prefix_len, uint32_t max_branches,
                            uint32_t max_suffix, uint32_t *token_positions,
                            uint32_t *token_branch, uint32_t *token_local_pos,
                            uint32_t *branch_offsets, char *error,
                            size_t error_len);

/* A staged, device-resident q3_pack_view plus the launch schedule derived from
 * it. Built once per batch, reused by every layer; building it is the only
 * place the packed path touches host memory. */
typedef struct q3_pack_plan q3_pack_plan;
q3_pack_plan *q3_pack_plan_create(q3_prefix_kv *prefix, q3_branch_set *set,
                                  const q3_suffix_item *items, uint32_t count,
                                  char *error, size_t error_len);
void q3_pack_plan_destroy(q3_pack_plan *plan);
uint32_t q3_pack_plan_tokens(const q3_pack_plan *plan);
/* Host copies of the descriptors, for inspection. */
const uint32_t *q3_pack_plan_token_positions(const q3_pack_plan *plan);
const uint32_t *q3_pack_plan_token_branch(const q3_pack_plan *plan);
const uint32_t *q3_pack_plan_token_local_pos(const q3_pack_plan *plan);
const uint32_t *q3_pack_plan_branch_offsets(const q3_pack_plan *plan);

/* One layer of the packed suffix pass: fused QK-RMSNorm + RoPE at
 * token_positions + KV write into each token's own branch pages, then
 * attention over [shared prefix pages | own branch suffix 0..lp].
 * Replaces the attention slice of run_layer_packed
 * (ref: src/q3_forward.cu:1489-1526). q/k/v/out: bf16 device, packed order. */
bool q3_suffix_attention_layer(q3_pack_plan *plan, uint32_t layer,
                               const void *q, const void *k, const void *v,
                               void *out, char *error, size_t error_len);

/* --- head-sharded runs: attention + output all-gather ------------------- *
 * New (the reference is single-device). With the KV heads sharded over the
 * GPUs of one box, every rank needs all heads' outputs after a layer.
 * `gathered[r]` is the base of rank r's buffer [n_ranks][tokens][n_heads][128]
 * (bf16, or fp32 with out_fp32), mapped into this process (peer memory over
 * NVLink). The call writes this rank's rows into slot `rank` of its own buffer
 * and queues, on a side stream, copy-engine copies of that slot into slot
 * `rank` of every other rank's buffer (no SM is used, so the next layer's
 * kernels keep the whole GPU), followed by the flags: `flags[r]` is rank r's
 * array of n_ranks uint32 (peer mapped, zero-initialised) and `seq` is
 * published in flags[r][rank] for every r. q3_attn_wait_gathered queues a
 * bounded device-side wait until this rank's flags all reached `seq`, i.e. its
 * gathered buffer holds that layer from every rank (timeout: status bit 2,
 * reported by q3_attn_synchronize). seq must increase; comparisons wrap. */
#define Q3_MAX_GATHER_RANKS 8u
typedef struct {
    uint32_t n_ranks;
    uint32_t rank;
    void *gathered[Q3_MAX_GATHER_RANKS];
    uint32_t *flags[Q3_MAX_GATHER_RANKS];
} q3_gather_peers;
bool q3_suffix_attention_layer_gathered(q3_pack_plan *plan, uint32_t layer,
                                        const void *q, const void *k, const void *v,
                                        const q3_gather_peers *gather, uint32_t seq,
                                        char *error, size_t error_len);
bool q3_attn_wait_gathered(q3_attn_runtime *rt, const q3_gather_peers *gather,
                           uint32_t seq, char *error, size_t error_len);
/* Every `seq` above is offset on the device by a per-runtime counter that
 * starts at 0; this queues `counter += count` on the runtime's stream. A step
 * recorded into a graph passes step-relative sequence numbers (1..L) and ends
 * with q3_attn_gather_advance(rt, L), after the waits of its last layers, so
 * that every replay publishes fresh numbers. All ranks must advance alike. */
bool q3_attn_gather_advance(q3_attn_runtime *rt, uint32_t count, char *error,
                            size_t error_len);

/* --- sealed prefixes kept across requests -------------------------------- *
 * The reference creates, prefills and destroys the prefix once per request
 * (ref: src/q3_systemone.cu:498-523, 740-741). With pages a sealed prefix is a
 * page table, so it can outlive the request: the cache keeps sealed prefixes
 * under a caller-chosen key (e.g. a hash of the prompt's token ids), hands them
 * out by reference count and evicts the least recently used unreferenced ones;
 * their pages return to the pool's free list and are reused without any
 * allocation. Host code only. */
typedef struct q3_prefix_cache q3_prefix_cache;
typedef struct {
    uint64_t hits, misses, inserts, evictions;
    uint32_t entries;
    uint32_t pages_held;
} q3_prefix_cache_stats;
q3_prefix_cache *q3_prefix_cache_create(q3_attn_runtime *rt, uint32_t max_entries,
                                        char *error, size_t error_len);
/* Destroys every prefix it still holds. */
void q3_prefix_cache_destroy(q3_prefix_cache *cache);
/* Hit (same key and token count): one more reference, returns the prefix.
 * Miss: NULL - the caller prefills a new prefix and inserts it. */
q3_prefix_kv *q3_prefix_cache_acquire(q3_prefix_cache *cache, uint64_t key,
                                      uint32_t token_count);
/* Gives a sealed prefix to the cache (the cache destroys it on eviction); the
 * caller keeps one reference, as after an acquire. At max_entries the least
 * recently used unreferenced entry is evicted first. */
bool q3_prefix_cache_insert(q3_prefix_cache *cache, uint64_t key, q3_prefix_kv *prefix,
                            char *error, size_t error_len);
bool q3_prefix_cache_release(q3_prefix_cache *cache, q3_prefix_kv *prefix, char *error,
                             size_t error_len);
/* Evicts unreferenced entries, least recently used first, until the pool has
 * `pages_needed` free pages or nothing more can go; returns the number evicted. */
uint32_t q3_prefix_cache_make_room(q3_prefix_cache *cache, uint32_t pages_needed);
/* 1 while the cache holds `prefix` (an evicted prefix no longer exists). */
int q3_prefix_cache_holds(const q3_prefix_cache *cache, const q3_prefix_kv *prefix);
void q3_prefix_cache_get_stats(const q3_prefix_cache *cache, q3_prefix_cache_stats *out);

/* --- replaying a fixed sequence of layer calls as one CUDA graph --------- *
 * The reference notes CUDA-graph capture of the 64-layer stack as the natural
 * next step of its launch plumbing (ref: docs/M3.md, src/q3_forward.cu:1588-1651
 * launches every layer eagerly). Between begin and end, the layer calls of this
 * header (device-pointer variants, including the gathered one) are recorded
 * instead of executed; q3_attn_graph_launch replays them on the runtime's
 * stream with the same pointers. Per-kernel timing is suspended while
 * recording. The host-buffer entry point cannot be recorded. */
typedef struct q3_attn_graph q3_attn_graph;
bool q3_attn_graph_begin(q3_attn_runtime *rt, char *error, size_t error_len);
q3_attn_graph *q3_attn_graph_end(q3_attn_runtime *rt, char *error, size_t error_len);
bool q3_attn_graph_launch(q3_attn_graph *graph, char *error, size_t error_len);
void q3_attn_graph_destroy(q3_attn_graph *graph);

/* --- paged decode: many independent sequences, one query token each --- */
typedef struct q3_decode_plan q3_decode_plan;
/* Host arrays: ctx_lens[num_seqs]; CSR page lists page_indptr[num_seqs+1],
 * page_indices[page_indptr[num_seqs]]. */
q3_decode_plan *q3_decode_plan_create(q3_attn_runtime *rt,
                                      const uint32_t *ctx_lens,
                                      const uint32_t *page_indptr,
                                      const uint32_t *page_indices,
                                      uint32_t num_seqs, char *error,
                                      size_t error_len);
void q3_decode_plan_destroy(q3_decode_plan *plan);
/* q [num_seqs][n_heads][128] bf16. If k_new/v_new are non-NULL the new token's
 * K/V (bf16 [num_seqs][n_kv_heads][128]) are normalised, roped and written at
 * position ctx_len and the query sees ctx_len + 1 keys; otherwise it sees
 * ctx_len keys. The query is normalised and roped at position ctx_len. */
bool q3_decode_attention_layer(q3_decode_plan *plan, uint32_t layer,
                               const void *q, const void *k_new,
                               const void *v_new, void *out, char *error,
                               size_t error_len);

/* --- decode without any allocation ------------------------------------ *
 * No counterpart in the reference. For callers that cannot allocate device
 * memory when they need attention (a server that gave the whole heap to its own
 * arena, a process under a no-cudaMalloc-after-start-up rule, a plugin that
 * must not re-enter the host's allocator): the split-KV partials of the decode
 * kernel live in a fixed array inside the library (about 8.5 MB per GPU, held
 * until the process exits) instead of a runtime-owned buffer. The call
 * allocates nothing, on host or device, and needs no q3_attn_runtime: every
 * buffer is the caller's.
 *   q_f16        [num_seqs][n_heads][128] f16, already normalised and roped
 *                (e.g. by q3_cuda_qknorm_rope_kvwrite)
 *   k_pages/v_pages  one layer of a page pool, [n_kv_heads][num_pages][16][128] f16
 *   ctx_lens, page_indptr, page_indices, work, seq_work_begin: DEVICE arrays;
 *                work / seq_work_begin are produced on the host by
 *                q3_decode_work_host and copied by the caller
 *   out_bf16     [num_seqs][n_heads][128] bf16
 * Limit: n_work * n_kv_heads <= Q3_DECODE_NOALLOC_MAX_SLOTS, else the call
 * fails with a message. The first call on each device looks up the array's
 * device address (safe from several host threads); make that call before any
 * stream capture. All calls share the array: two calls that overlap on the GPU
 * race. Nothing in it needs clearing (every slot a call reads was written by
 * that call). The pools are the caller's: slots past ctx_len in a sequence's
 * last page are multiplied by an exact 0 and must therefore hold finite values
 * (a zero-initialised pool does). Every ctx_len must be >= 1. The kernel's waits
 * are bounded; q3_cuda_attention_decode_noalloc_status tells whether one gave
 * up (the rows of that call are then undefined). */
#define Q3_DECODE_NOALLOC_MAX_SLOTS 2048u
typedef struct {
    uint32_t seq;
    uint32_t page_begin;
    uint32_t page_end;
    uint32_t slot;
} q3_decode_work_item;
/* Pure host: cut sequences into chunks of at most 64 pages. work_out holds up
 * to max_work items, seq_work_begin_out num_seqs + 1 entries. Returns the
 * number of work items, or -1. */
int64_t q3_decode_work_host(const uint32_t *ctx_lens, uint32_t num_seqs,
                            q3_decode_work_item *work_out, uint32_t max_work,
                            uint32_t *seq_work_begin_out, char *error, size_t error_len);
bool q3_cuda_attention_decode_noalloc(
    const void *q_f16, const void *k_pages, const void *v_pages, uint32_t num_pages,
    const uint32_t *ctx_lens, const uint32_t *page_indptr, const uint32_t *page_indices,
    const q3_decode_work_item *work, uint32_t n_work, const uint32_t *seq_work_begin,
    uint32_t num_seqs, uint32_t n_heads, uint32_t n_kv_heads, void *out_bf16,
    void *stream, char *error, size_t error_len);
/* Copies the current device's status word of the entry above into *status_out
 * (host memory), clears it and synchronises `stream`: 0 = every wait of the
 * calls queued so far on that stream completed; nonzero = one gave up. Also
 * allocates nothing. No counterpart in the reference. */
bool q3_cuda_attention_decode_noalloc_status(uint32_t *status_out, void *stream,
                                             char *error, size_t error_len);

/* --- low-level fused KV write (new kernel; replaces ref a1+a2/a3+a5/a8:
 *     two rms_norm launches, rope, and the append / scatter) -------------- *
 * Per token t: rope position rope_pos[t], destination page dst_page[t] and
 * slot dst_slot[t] (device arrays). Writes K,V pages and the normalised,
 * roped query as f16 into q_out [tokens][n_heads][128] (may be NULL with
 * q == NULL). k/v may be NULL to transform only q. */
bool q3_cuda_qknorm_rope_kvwrite(q3_attn_runtime *rt, uint32_t layer,
                                 const void *q, const void *k, const void *v,
                                 uint32_t tokens, const uint32_t *rope_pos,
                                 const uint32_t *dst_page,
                                 const uint32_t *dst_slot, void *q_out,
                                 char *error, size_t error_len);

/* Host-buffer entry for callers whose activations live in (pinned) host
 * memory: copies q/k/v in, runs q3_suffix_attention_layer, copies `out` back.
 * Successive calls are pipelined over three device slots and two copy streams,
 * so the copy-in of the next layer and the copy-out of the previous one overlap
 * the kernels. Does not synchronise: `out_host` is valid, and q/k/v may be
 * reused, after q3_attn_synchronize. */
bool q3_suffix_attention_layer_host(q3_pack_plan *plan, uint32_t layer,
                                    const void *q_host, const void *k_host,
                                    const void *v_host, void *out_host,
                                    char *error, size_t error_len);
/* The same for head-sharded runs: copies q/k/v in, runs
 * q3_suffix_attention_layer_gathered (rows into this rank's slot of its own
 * gathered buffer, copies to the other ranks and flags queued behind them) and
 * copies this rank's rows [tokens][n_heads][128] back to `out_host`. The
 * caller alternates two gathered buffers from layer to layer and waits
 * (q3_attn_wait_gathered) exactly as with the device-pointer call. */
bool q3_suffix_attention_layer_gathered_host(q3_pack_plan *plan, uint32_t layer,
                                             const void *q_host, const void *k_host,
                                             const void *v_host,
                                             const q3_gather_peers *gather, uint32_t seq,
                                             void *out_host, char *error,
                                             size_t error_len);

/* --- the layer with its q/k/v projection fused in ------------------------- *
 * The reference's layer drivers run three quantised linears, then rms_norm on
 * q and k, rope, and the KV append or scatter (ref: src/q3_forward.cu:1214-1278
 * and :1462-1516): q, k and v are written by the linears and read again by the
 * next five steps. Here the projection's epilogue normalises, rotates and
 * writes - queries as f16 into the attention kernel's Q buffer, keys and values
 * into their pages - so q, k and v never exist as tensors: two launches per
 * layer (projection, attention).
 *   weights  three resident Q4_K tensors [heads*128][hidden], all in the GGUF
 *            order (Q3_QUANT_Q4_K = 12) or all in the tiled order of
 *            q3_cuda_q4k_linear_pack (include/q3_q4_linear.h); other types are
 *            refused with a message - project them with q3_cuda_q4k_linear_f16
 *            and call the plain layer entry;
 *   x_f16    the layer's input rows after the attention norm, f16
 *            [tokens][hidden], device memory, 16-byte aligned;
 * everything else as q3_prefix_prefill_layer / q3_suffix_attention_layer.
 * q3_cuda_q4k_linear_init must have been called on this device. */
typedef struct {
    const void *wq, *wk, *wv;
    uint32_t qtype_q, qtype_k, qtype_v;
    uint32_t hidden;
} q3_qkv_weights;
bool q3_prefix_prefill_layer_projected(q3_prefix_kv *prefix, uint32_t layer,
                                       const q3_qkv_weights *weights, const void *x_f16,
                                       uint32_t tokens, void *out, char *error,
                                       size_t error_len);
bool q3_suffix_attention_layer_projected(q3_pack_plan *plan, uint32_t layer,
                                         const q3_qkv_weights *weights, const void *x_f16,
                                         void *out, char *error, size_t error_len);

/* --- diagnostics: the launch schedule (pure host, no CUDA) ---------------- *
 * The tensor-core attention kernel is launched with one CTA per SM; the host
 * cuts the launch into segments = (32-token tile, KV head, range of 128-key
 * tiles) so that every CTA streams the same number of key tiles. This call
 * builds that schedule for a packed batch described by per-token branch and
 * local position (a plain causal sequence: branch 0, lp = absolute position,
 * shared_len 0) and reports it. `lockstep` selects whole-item waves followed by
 * a stream-K tail (used when the shared KV would not stay in L2 under the
 * staggered access of pure stream-K). No counterpart in the reference, whose grid is
 * one warp per (token, head) (ref: src/q3_forward.cu:815-819). */
typedef struct {
    uint32_t cta;
    uint32_t tok0;
    uint32_t kv_head;
    uint32_t tile_begin;
    uint32_t tile_end;
    uint32_t shared_tiles;
    int32_t partial_slot;
} q3_sched_segment_info;
typedef struct {
    uint32_t grid;
    uint32_t n_segments;
    uint32_t n_cut_items;
    uint32_t n_slots;
    uint64_t total_key_tiles;
} q3_sched_summary;
bool q3_schedule_describe(uint32_t tokens, uint32_t n_kv_heads, uint32_t shared_len,
                          const uint32_t *row_tag, const uint32_t *row_lp,
                          uint32_t pages_per_branch, uint32_t n_branches,
                          uint32_t num_ctas, uint32_t max_slots, bool lockstep,
                          q3_sched_summary *summary, q3_sched_segment_info *segments,
                          uint32_t max_segments, char *error, size_t error_len);

/* Which of the two assignments of key tiles to CTAs a packed batch gets
 * (plans built after the call). AUTO: lockstep waves when the shared KV of the
 * runtime's heads is larger than L2 holds comfortably, stream-K otherwise.
 * Both give the same rows up to the rounding of the partial combination; the
 * knob exists for tuning and so that tests can run either on any shape. */
#define Q3_SCHED_AUTO 0u
#define Q3_SCHED_STREAMK 1u
#define Q3_SCHED_LOCKSTEP 2u
bool q3_attn_set_schedule_policy(q3_attn_runtime *rt, uint32_t policy, char *error,
                                 size_t error_len);

const char *q3_attn_version(void);

#ifdef __cplusplus
}
#endif

#endif /* Q3_ATTN_H */
