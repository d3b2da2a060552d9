/* q3_internal.h - private structs shared by the translation units of
 * libq3attn. Nothing here is part of the C ABI (include/q3_attn.h is). */
#ifndef Q3_INTERNAL_H
#define Q3_INTERNAL_H

#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include <stdint.h>
#include <stdio.h>
#include <string.h>

#include <vector>

#include "q3_attn.h"
#include "q3_sched.h"

#define Q3_D 128u          /* head_dim the kernels are specialised for     */
#define Q3_G 8u            /* query heads per KV head                       */
#define Q3_PAGE 16u        /* tokens per KV page                            */

/* device_status bits (set by kernels whose bounded waits gave up) */
#define Q3_STATUS_WAIT_TIMEOUT 1u
#define Q3_STATUS_GATHER_TIMEOUT 2u

static inline void q3_clear_error(char *error, size_t error_len) {
    if (error && error_len) error[0] = '\0';
}

static inline bool q3_fail(char *error, size_t error_len, const char *msg) {
    if (error && error_len) {
        error[0] = '\0';
        snprintf(error, error_len, "%s", msg);
    }
    return false;
}

static inline bool q3_fail_cuda(char *error, size_t error_len, const char *what,
                                cudaError_t code) {
    if (error && error_len) {
        error[0] = '\0';
        snprintf(error, error_len, "%s: %s", what, cudaGetErrorString(code));
    }
    return false;
}

/* Read the launch status right after a launch, as the reference does
 * (ref: src/q3_forward.cu:632-636). */
#define Q3_LAUNCH_CHECK(what)                                             \
    do {                                                                  \
        cudaError_t q3_code_ = cudaGetLastError();                        \
        if (q3_code_ != cudaSuccess)                                      \
            return q3_fail_cuda(error, error_len, (what), q3_code_);      \
    } while (0)

struct q3_attn_runtime {
    q3_attn_config cfg;
    cudaStream_t stream;
    int num_sms;

    __half *k_pool;   /* [L][Hkv][num_pages][16][128] */
    __half *v_pool;
    CUtensorMap k_map; /* 2-D {128, L*Hkv*num_pages*16}, box {64,16}, SW128 */
    CUtensorMap v_map;
    CUtensorMap k_map_tile; /* same tensor, box {64,128}: eight consecutive pages in one copy */
    CUtensorMap v_map_page; /* 3-D {64, rows, 2 halves}, box {64,16,2}: a page's two halves in one copy */
    std::vector<uint32_t> free_pages;

    float *qk_norm_w;  /* device [L][2][128] */
    float2 *rope_table; /* device [max_positions][64] (cos, sin) */
    __half *q2;        /* workspace [max_tokens][n_heads][128] */

    /* stream-K partial accumulators, sized for 2 slots per SM */
    float *part_o;     /* [slots][256][128] */
    float2 *part_ml;   /* [slots][256] (max in log2 units, sum) */
    uint32_t part_slots;
    uint32_t *fix_counters; /* [part_slots][8] arrival counters, zero between launches */

    /* decode split partials */
    float *dec_o;      /* [dec_slots][8][128] */
    float2 *dec_ml;    /* [dec_slots][8] */
    uint32_t dec_slots;

    uint32_t *status_dev;
    uint32_t *gather_epoch_dev;  /* added to every gather sequence number on the device */
    uint32_t *status_host; /* pinned mirror, refreshed by q3_attn_synchronize */

    /* pinned staging for the host-buffer entry point (grow-once) */
    void *host_stage;
    size_t host_stage_bytes;
    void *dev_stage;
    size_t dev_stage_bytes;      /* per slot */
    /* the host-buffer entry pipelines three slots over two copy streams */
    cudaStream_t h2d_stream, d2h_stream;
    cudaEvent_t ev_in[3], ev_compute[3], ev_out[3];
    bool copy_ready;
    uint64_t host_calls;
    /* head-sharded runs: copies of this rank's rows to the other ranks */
    cudaStream_t gather_stream;
    cudaEvent_t ev_gather[4];
    bool gather_ready;
    uint64_t gather_calls;
    /* stream capture (q3_attn_graph_*) */
    bool capturing;
    bool capture_used_gather;
    uint64_t capture_launches;

    uint64_t n_alloc, n_free, n_sync, n_launch;
    uint64_t workspace_bytes;
    uint32_t sched_policy;       /* Q3_SCHED_AUTO / _STREAMK / _LOCKSTEP */

    /* optional per-kernel timing: event pairs recorded around launches, read
     * after a synchronize (the reference brackets its phases the same way,
     * ref: src/q3_forward.cu:1205-1285,1759-1822) */
    bool timing_on;
    std::vector<cudaEvent_t> ev;      /* pairs: [2i] start, [2i+1] stop */
    std::vector<uint8_t> ev_phase;    /* phase of pair i */
    size_t ev_used;                   /* pairs recorded */
};

enum { Q3_PHASE_KVWRITE = 0, Q3_PHASE_ATTENTION = 1, Q3_PHASE_GATHER_WAIT = 2,
       Q3_PHASE_DECODE = 3, Q3_PHASE_COUNT = 4 };

static inline void q3_phase_begin(q3_attn_runtime *rt, int phase) {
    if (rt->timing_on && !rt->capturing && rt->ev_used < rt->ev_phase.size()) {
        rt->ev_phase[rt->ev_used] = (uint8_t)phase;
        cudaEventRecord(rt->ev[2 * rt->ev_used], rt->stream);
    }
}
static inline void q3_phase_end(q3_attn_runtime *rt) {
    if (rt->timing_on && !rt->capturing && rt->ev_used < rt->ev_phase.size()) {
        cudaEventRecord(rt->ev[2 * rt->ev_used + 1], rt->stream);
        rt->ev_used++;
    }
}

struct q3_attn_graph {
    q3_attn_runtime *rt;
    cudaGraph_t graph;
    cudaGraphExec_t exec;
    uint64_t launches;   /* kernels per replay */
};

struct q3_prefix_kv {
    q3_attn_runtime *rt;
    uint32_t capacity;
    uint32_t token_count;
    bool sealed;
    bool owns_pages;
    std::vector<uint32_t> pages; /* ceil(capacity/16) physical page ids */
    /* staged descriptors for prefill chunks (grow-once, device + pinned) */
    struct q3_stage *stage;
};

struct q3_branch_set {
    q3_prefix_kv *prefix;
    uint32_t max_branches;
    uint32_t max_suffix;
    uint32_t pages_per_branch;
    uint32_t live;
    std::vector<uint8_t> in_use;
    std::vector<uint32_t> pages; /* [max_branches][pages_per_branch] */
    struct q3_decide_state *decide; /* scratch of q3_decide_run, created on first use */
};

/* Device-resident descriptors + schedule of one attention launch. */
struct q3_stage {
    q3_attn_runtime *rt;
    void *host;        /* pinned */
    void *dev;
    size_t bytes;      /* capacity of both */
    /* device views into `dev`, valid after q3_stage_upload */
    const uint32_t *rope_pos, *dst_page, *dst_slot;
    const uint32_t *row_tag, *row_lp;
    const uint32_t *page_ids;
    const q3_run *runs;
    const q3_segment *segments;
    const uint32_t *cta_seg_begin;
    uint32_t tokens, n_shared_pages, shared_len, grid;
    cudaEvent_t uploaded;  /* recorded after the last upload from `host` */
    bool has_uploaded;
    /* prefill chunks: which (base, tokens) the staged schedule describes */
    bool chunk_valid;
    uint32_t chunk_base, chunk_tokens;
};

struct q3_pack_plan {
    q3_prefix_kv *prefix;
    q3_branch_set *set;
    uint32_t tokens, branches;
    std::vector<uint32_t> token_positions, token_branch, token_local_pos,
        branch_offsets;
    q3_stage *stage;
};

struct q3_decode_plan {
    q3_attn_runtime *rt;
    uint32_t num_seqs;
    uint32_t n_work;     /* (sequence, chunk) work items per KV head */
    uint32_t chunk_pages;
    bool can_append;     /* every sequence has a page slot for one more token */
    bool has_empty;      /* some sequence has ctx_len 0 (needs an appended token) */
    void *dev;
    const uint32_t *ctx_lens, *page_indptr, *page_indices;
    const uint32_t *rope_pos, *dst_page, *dst_slot;
    const q3_decode_work *work;
    const uint32_t *seq_work_begin; /* [num_seqs+1] */
};

/* --- cross-file helpers ------------------------------------------------- */
q3_stage *q3_stage_create(q3_attn_runtime *rt, char *error, size_t error_len);
void q3_stage_destroy(q3_stage *st);
/* Serialise a host schedule into the stage's pinned buffer and queue the copy
 * on the runtime's stream. Grows the buffers when needed (counted). */
bool q3_stage_upload(q3_stage *st, const q3_schedule &sched,
                     const std::vector<uint32_t> &rope_pos,
                     const std::vector<uint32_t> &dst_page,
                     const std::vector<uint32_t> &dst_slot,
                     char *error, size_t error_len);

bool q3_pack_plan_build(q3_pack_plan *plan, q3_stage *stage, q3_prefix_kv *prefix,
                        q3_branch_set *set, const q3_suffix_item *items, uint32_t count,
                        const char *who, char *error, size_t error_len);
void q3_decide_state_destroy(q3_branch_set *set);
/* fp32 surface through the tensor-core kernel (q3_fp32_native.cu): return true
 * when the call was taken (*ok = its outcome), false when it does not apply */
bool q3_fp32_native_attention(const float *q, const float *k_src, const float *v_src,
                              uint32_t tokens, uint32_t n_heads, uint32_t n_kv_heads,
                              uint32_t head_dim, uint32_t position_base, uint32_t kv_length,
                              float scale, float *out, void *stream, bool *ok, char *error,
                              size_t error_len);
bool q3_fp32_native_segmented(const float *q, const float *prefix_k, const float *prefix_v,
                              uint32_t prefix_len, const float *suffix_k,
                              const float *suffix_v, uint32_t suffix_capacity,
                              uint32_t suffix_num_layers, uint32_t suffix_layer,
                              const uint32_t *token_branch, const uint32_t *token_local_pos,
                              uint32_t tokens, uint32_t n_heads, uint32_t n_kv_heads,
                              uint32_t head_dim, float scale, float *out, void *stream,
                              bool *ok, char *error, size_t error_len);

bool q3_launch_kvwrite(q3_attn_runtime *rt, uint32_t layer, const void *q,
                       const void *k, const void *v, uint32_t tokens,
                       const uint32_t *rope_pos, const uint32_t *dst_page,
                       const uint32_t *dst_slot, void *q_out, char *error,
                       size_t error_len);
bool q3_launch_attention(q3_attn_runtime *rt, uint32_t layer,
                         const q3_stage *st, void *out_bf16, char *error,
                         size_t error_len);
bool q3_launch_gather_signal(q3_attn_runtime *rt, const q3_gather_peers *g, uint32_t seq,
                             cudaStream_t stream, char *error, size_t error_len);
bool q3_launch_gather_advance(q3_attn_runtime *rt, uint32_t count, char *error,
                              size_t error_len);
bool q3_launch_gather_wait(q3_attn_runtime *rt, const q3_gather_peers *g, uint32_t seq,
                           char *error, size_t error_len);
bool q3_launch_decode(q3_attn_runtime *rt, uint32_t layer,
                      const q3_decode_plan *plan, bool with_new_token,
                      void *out_bf16, char *error, size_t error_len);

bool q3_prepare_attention_kernel(char *error, size_t error_len);
bool q3_prepare_decode_kernel(char *error, size_t error_len);
/* q3_q4k_linear.cu: the q/k/v projection with norm + RoPE + page write as its
 * epilogue. All pointers are device pointers. */
struct q3_qkv_fused_args {
    const void *wq, *wk, *wv;   /* [n_q_heads*128][hidden], [n_kv_heads*128][hidden] x 2 */
    uint32_t qtype;             /* Q4_K in GGUF or tiled order, the same for all three */
    uint32_t hidden;
    uint32_t n_q_heads, n_kv_heads;
    const void *x_f16;          /* [tokens][hidden] */
    uint32_t tokens;
    const float *norm_w;        /* [2][128] of the layer */
    float eps;
    const void *rope_table;     /* float2 [position][64] */
    const uint32_t *rope_pos, *dst_page, *dst_slot;
    void *q_out;                /* f16 [tokens][n_q_heads][128] */
    void *k_pool, *v_pool;      /* the layer's pages: f16 [kv head][page][16][128] */
    uint32_t num_pages;
};
bool q3_launch_qkv_fused(const q3_qkv_fused_args *a, cudaStream_t stream, char *error,
                         size_t error_len);
bool q3_prepare_kvwrite_kernel(char *error, size_t error_len);

/* Entry points make the runtime's device current: a host that drives several
 * GPUs from one thread would otherwise launch on whichever device it left. */
static inline bool q3_use_device(const q3_attn_runtime *rt, char *error, size_t error_len) {
    cudaError_t e = cudaSetDevice(rt->cfg.device);
    if (e != cudaSuccess) return q3_fail_cuda(error, error_len, "cudaSetDevice", e);
    return true;
}

bool q3_encode_tmap_2d(CUtensorMap *map, const void *base, uint64_t inner,
                       uint64_t rows, uint32_t box_inner, uint32_t box_rows,
                       char *error, size_t error_len);
bool q3_encode_tmap_bytes_2d(CUtensorMap *map, const void *base, uint64_t row_bytes,
                             uint64_t rows, uint32_t box_bytes, uint32_t box_rows,
                             char *error, size_t error_len);
bool q3_encode_tmap_page(CUtensorMap *map, const void *base, uint64_t rows, char *error,
                         size_t error_len);
bool q3_encode_tmap_q(CUtensorMap *map, const void *base, uint32_t n_heads,
                      uint32_t tokens, char *error, size_t error_len);

#endif /* Q3_INTERNAL_H */
