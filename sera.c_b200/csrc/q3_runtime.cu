/* q3_runtime.cu - host side of the native paged attention path: runtime,
 * KV page pool and free list, shared prefix, branch set, suffix packing,
 * descriptor staging. Mirrors the object model of the reference's
 * src/q3_decide.cu (prefix / branch set / packing) and the runtime shell of
 * src/q3_forward.cu (stream, grow-once workspace, counters), re-based on a
 * paged f16 pool. No kernel lives in this file.
 */
#include "q3_internal.h"

#include <math.h>
#include <stdlib.h>

#include <algorithm>
#include <new>

/* ---------------------------------------------------------------------- */
/* counted allocation helpers                                              */
/* ---------------------------------------------------------------------- */

static cudaError_t rt_malloc(q3_attn_runtime *rt, void **p, size_t bytes) {
    cudaError_t e = cudaMalloc(p, bytes);
    if (e == cudaSuccess) {
        rt->n_alloc++;
        rt->workspace_bytes += bytes;
    }
    return e;
}

static void rt_free(q3_attn_runtime *rt, void *p) {
    if (p) {
        cudaFree(p);
        rt->n_free++;
    }
}

/* ---------------------------------------------------------------------- */
/* TMA descriptors                                                         */
/* ---------------------------------------------------------------------- */

typedef CUresult (*encode_tiled_fn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t,
                                    void *, const cuuint64_t *, const cuuint64_t *,
                                    const cuuint32_t *, const cuuint32_t *,
                                    CUtensorMapInterleave, CUtensorMapSwizzle,
                                    CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static encode_tiled_fn get_encode_fn() {
    static encode_tiled_fn fn = nullptr;
    if (!fn) {
        void *p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault,
                                    &q) == cudaSuccess &&
            q == cudaDriverEntryPointSuccess)
            fn = (encode_tiled_fn)p;
    }
    return fn;
}

/* 2-D f16 tensor {inner, rows}, row pitch inner*2 bytes, 128-byte swizzle. */
bool q3_encode_tmap_2d(CUtensorMap *map, const void *base, uint64_t inner,
                       uint64_t rows, uint32_t box_inner, uint32_t box_rows,
                       char *error, size_t error_len) {
    encode_tiled_fn fn = get_encode_fn();
    if (!fn) return q3_fail(error, error_len, "cuTensorMapEncodeTiled unavailable");
    cuuint64_t dims[2] = {inner, rows};
    cuuint64_t strides[1] = {inner * 2};
    cuuint32_t box[2] = {box_inner, box_rows};
    cuuint32_t estr[2] = {1, 1};
    CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, (void *)base, dims,
                    strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                    CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                    CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) {
        if (error && error_len)
            snprintf(error, error_len, "cuTensorMapEncodeTiled failed (%d)", (int)r);
        return false;
    }
    return true;
}

/* 2-D byte tensor {row_bytes, rows}, no swizzle: rows of packed quantised
 * blocks. box_bytes and row_bytes must be multiples of 16. */
bool q3_encode_tmap_bytes_2d(CUtensorMap *map, const void *base, uint64_t row_bytes,
                             uint64_t rows, uint32_t box_bytes, uint32_t box_rows,
                             char *error, size_t error_len) {
    encode_tiled_fn fn = get_encode_fn();
    if (!fn) return q3_fail(error, error_len, "cuTensorMapEncodeTiled unavailable");
    cuuint64_t dims[2] = {row_bytes, rows};
    cuuint64_t strides[1] = {row_bytes};
    cuuint32_t box[2] = {box_bytes, box_rows};
    cuuint32_t estr[2] = {1, 1};
    CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, (void *)base, dims, strides, box,
                    estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE,
                    CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) {
        if (error && error_len)
            snprintf(error, error_len, "cuTensorMapEncodeTiled(bytes) failed (%d)", (int)r);
        return false;
    }
    return true;
}

/* Query workspace [tokens][n_heads][128] f16 viewed as {128, n_heads, tokens};
 * box {64, 8, 16}: 16 tokens x 8 heads of one KV group, half a head row. */
/* A page pool [rows][128] f16 seen as {64 columns, rows, 2 column halves}: the
 * stride of the third dimension (128 B) is smaller than that of the second
 * (256 B), which the encoder accepts. One box {64, 16, 2} is a whole page,
 * written as [half][16 rows][128 B] - byte for byte what the two 64-column
 * boxes of the 2-D map write into two consecutive 2 KiB blocks. */
bool q3_encode_tmap_page(CUtensorMap *map, const void *base, uint64_t rows, char *error,
                         size_t error_len) {
    encode_tiled_fn fn = get_encode_fn();
    if (!fn) return q3_fail(error, error_len, "cuTensorMapEncodeTiled unavailable");
    cuuint64_t dims[3] = {64, rows, 2};
    cuuint64_t strides[2] = {Q3_D * 2, 128};
    cuuint32_t box[3] = {64, Q3_PAGE, 2};
    cuuint32_t estr[3] = {1, 1, 1};
    CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 3, (void *)base, dims, strides, box,
                    estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                    CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) {
        if (error && error_len)
            snprintf(error, error_len, "cuTensorMapEncodeTiled(page) failed (%d)", (int)r);
        return false;
    }
    return true;
}

bool q3_encode_tmap_q(CUtensorMap *map, const void *base, uint32_t n_heads,
                      uint32_t tokens, char *error, size_t error_len) {
    encode_tiled_fn fn = get_encode_fn();
    if (!fn) return q3_fail(error, error_len, "cuTensorMapEncodeTiled unavailable");
    cuuint64_t dims[3] = {Q3_D, n_heads, tokens};
    cuuint64_t strides[2] = {Q3_D * 2, (cuuint64_t)n_heads * Q3_D * 2};
    cuuint32_t box[3] = {64, Q3_G, 16};
    cuuint32_t estr[3] = {1, 1, 1};
    CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 3, (void *)base, dims,
                    strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                    CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                    CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) {
        if (error && error_len)
            snprintf(error, error_len, "cuTensorMapEncodeTiled(q) failed (%d)", (int)r);
        return false;
    }
    return true;
}

/* ---------------------------------------------------------------------- */
/* runtime                                                                 */
/* ---------------------------------------------------------------------- */

extern "C" const char *q3_attn_version(void) { return "q3attn-b200 0.1 (sm_100a)"; }

extern "C" q3_attn_runtime *q3_attn_create(const q3_attn_config *config,
                                           char *error, size_t error_len) {
    q3_clear_error(error, error_len);
    if (!config) {
        q3_fail(error, error_len, "q3_attn_create: null config");
        return NULL;
    }
    const q3_attn_config &c = *config;
    if (c.head_dim != Q3_D || c.n_kv_heads == 0 || c.n_heads != c.n_kv_heads * Q3_G ||
        c.num_layers == 0 || c.max_tokens == 0 || c.num_pages == 0 ||
        c.max_positions == 0) {
        q3_fail(error, error_len,
                "q3_attn_create: unsupported geometry (need head_dim 128, "
                "n_heads == 8 * n_kv_heads, nonzero sizes)");
        return NULL;
    }
    const uint64_t pool_rows =
        (uint64_t)c.num_layers * c.n_kv_heads * c.num_pages * Q3_PAGE;
    if (pool_rows >= (1ull << 31)) {
        q3_fail(error, error_len, "q3_attn_create: page pool too large for one tensor map");
        return NULL;
    }
    int count = 0;
    if (cudaGetDeviceCount(&count) != cudaSuccess || count == 0) {
        q3_fail(error, error_len, "q3_attn_create: no CUDA device (this library has no CPU path)");
        return NULL;
    }
    if (cudaSetDevice(c.device) != cudaSuccess) {
        q3_fail(error, error_len, "q3_attn_create: cudaSetDevice failed");
        return NULL;
    }
    cudaDeviceProp prop;
    cudaGetDeviceProperties(&prop, c.device);
    if (prop.major != 10) {
        q3_fail(error, error_len,
                "q3_attn_create: kernels are built for sm_100a only; device is not compute 10.x");
        return NULL;
    }
    q3_attn_runtime *rt = new (std::nothrow) q3_attn_runtime();
    if (!rt) {
        q3_fail(error, error_len, "q3_attn_create: allocation failed");
        return NULL;
    }
    rt->cfg = c;
    rt->num_sms = prop.multiProcessorCount;
    rt->stream = nullptr;
    rt->k_pool = rt->v_pool = nullptr;
    rt->qk_norm_w = nullptr;
    rt->rope_table = nullptr;
    rt->q2 = nullptr;
    rt->part_o = nullptr;
    rt->part_ml = nullptr;
    rt->fix_counters = nullptr;
    rt->dec_o = nullptr;
    rt->dec_ml = nullptr;
    rt->dec_slots = 0;
    rt->status_dev = nullptr;
    rt->gather_epoch_dev = nullptr;
    rt->status_host = nullptr;
    rt->host_stage = rt->dev_stage = nullptr;
    rt->host_stage_bytes = rt->dev_stage_bytes = 0;
    rt->h2d_stream = rt->d2h_stream = nullptr;
    rt->copy_ready = false;
    rt->host_calls = 0;
    rt->gather_stream = nullptr;
    rt->gather_ready = false;
    rt->gather_calls = 0;
    rt->capturing = false;
    rt->capture_used_gather = false;
    rt->capture_launches = 0;
    rt->n_alloc = rt->n_free = rt->n_sync = rt->n_launch = 0;
    rt->workspace_bytes = 0;
    rt->sched_policy = Q3_SCHED_AUTO;
    rt->timing_on = false;
    rt->ev_used = 0;

    const size_t pool_bytes = (size_t)pool_rows * Q3_D * sizeof(__half);
    const size_t q2_bytes = (size_t)c.max_tokens * c.n_heads * Q3_D * sizeof(__half);
    rt->part_slots = 2u * (uint32_t)rt->num_sms + 2u;
    const size_t part_o_bytes = (size_t)rt->part_slots * 256 * Q3_D * sizeof(float);
    const size_t part_ml_bytes = (size_t)rt->part_slots * 256 * sizeof(float2);
    const size_t w_bytes = (size_t)c.num_layers * 2 * Q3_D * sizeof(float);
    const size_t rope_bytes = (size_t)c.max_positions * 64 * sizeof(float2);
    bool ok = cudaStreamCreateWithFlags(&rt->stream, cudaStreamNonBlocking) == cudaSuccess;
    ok = ok && rt_malloc(rt, (void **)&rt->k_pool, pool_bytes) == cudaSuccess;
    ok = ok && rt_malloc(rt, (void **)&rt->v_pool, pool_bytes) == cudaSuccess;
    ok = ok && rt_malloc(rt, (void **)&rt->q2, q2_bytes) == cudaSuccess;
    ok = ok && rt_malloc(rt, (void **)&rt->part_o, part_o_bytes) == cudaSuccess;
    ok = ok && rt_malloc(rt, (void **)&rt->part_ml, part_ml_bytes) == cudaSuccess;
    ok = ok && rt_malloc(rt, (void **)&rt->fix_counters,
                         (size_t)rt->part_slots * 8 * sizeof(uint32_t)) == cudaSuccess;
    ok = ok && rt_malloc(rt, (void **)&rt->qk_norm_w, w_bytes) == cudaSuccess;
    ok = ok && rt_malloc(rt, (void **)&rt->rope_table, rope_bytes) == cudaSuccess;
    ok = ok && rt_malloc(rt, (void **)&rt->status_dev, sizeof(uint32_t)) == cudaSuccess;
    ok = ok && rt_malloc(rt, (void **)&rt->gather_epoch_dev, sizeof(uint32_t)) == cudaSuccess;
    ok = ok && cudaHostAlloc((void **)&rt->status_host, sizeof(uint32_t),
                             cudaHostAllocDefault) == cudaSuccess;
    if (!ok) {
        q3_fail(error, error_len, "q3_attn_create: device allocation failed");
        q3_attn_destroy(rt);
        return NULL;
    }
    rt->workspace_bytes -= 2 * pool_bytes; /* pool reported separately */
    *rt->status_host = 0;
    /* Stale f16 bit patterns in never-written page slots are multiplied by an
     * exact 0 probability; they must therefore be finite. */
    cudaMemsetAsync(rt->k_pool, 0, pool_bytes, rt->stream);
    cudaMemsetAsync(rt->v_pool, 0, pool_bytes, rt->stream);
    cudaMemsetAsync(rt->q2, 0, q2_bytes, rt->stream);
    cudaMemsetAsync(rt->status_dev, 0, sizeof(uint32_t), rt->stream);
    cudaMemsetAsync(rt->gather_epoch_dev, 0, sizeof(uint32_t), rt->stream);
    cudaMemsetAsync(rt->fix_counters, 0, (size_t)rt->part_slots * 8 * sizeof(uint32_t),
                    rt->stream);

    /* QK-norm weights default to 1 (ref: synthetic configs use weight 1). */
    {
        std::vector<float> ones((size_t)c.num_layers * 2 * Q3_D, 1.0f);
        cudaMemcpyAsync(rt->qk_norm_w, ones.data(), w_bytes, cudaMemcpyHostToDevice,
                        rt->stream);
        cudaStreamSynchronize(rt->stream);
    }
    /* RoPE table. The reference forms angle = (float)position * inv_freq[p] in
     * fp32 (ref: src/q3_forward.cu:199, inv_freq from :1128-1130) and takes
     * cosf/sinf of it; the table holds the correctly rounded cos/sin of that
     * same fp32 angle, so large positions do not depend on fast-math
     * intrinsics. */
    {
        std::vector<float2> table((size_t)c.max_positions * 64);
        float inv_freq[64];
        for (uint32_t i = 0; i < 64; i++)
            inv_freq[i] = (float)(1.0 / pow(c.rope_theta, (double)(2 * i) / (double)Q3_D));
        for (uint32_t pos = 0; pos < c.max_positions; pos++)
            for (uint32_t i = 0; i < 64; i++) {
                const float angle = (float)pos * inv_freq[i];
                table[(size_t)pos * 64 + i] =
                    make_float2((float)cos((double)angle), (float)sin((double)angle));
            }
        cudaMemcpyAsync(rt->rope_table, table.data(), rope_bytes,
                        cudaMemcpyHostToDevice, rt->stream);
        cudaStreamSynchronize(rt->stream);
    }
    if (!q3_encode_tmap_2d(&rt->k_map, rt->k_pool, Q3_D, pool_rows, 64, Q3_PAGE, error,
                           error_len) ||
        !q3_encode_tmap_2d(&rt->v_map, rt->v_pool, Q3_D, pool_rows, 64, Q3_PAGE, error,
                           error_len) ||
        !q3_encode_tmap_2d(&rt->k_map_tile, rt->k_pool, Q3_D, pool_rows, 64, 8 * Q3_PAGE, error,
                           error_len) ||
        !q3_encode_tmap_page(&rt->v_map_page, rt->v_pool, pool_rows, error, error_len)) {
        q3_attn_destroy(rt);
        return NULL;
    }
    if (!q3_prepare_attention_kernel(error, error_len) ||
        !q3_prepare_decode_kernel(error, error_len) ||
        !q3_prepare_kvwrite_kernel(error, error_len)) {
        q3_attn_destroy(rt);
        return NULL;
    }
    rt->free_pages.resize(c.num_pages);
    for (uint32_t i = 0; i < c.num_pages; i++) rt->free_pages[i] = c.num_pages - 1 - i;
    if (cudaGetLastError() != cudaSuccess) {
        q3_fail(error, error_len, "q3_attn_create: initialisation failed");
        q3_attn_destroy(rt);
        return NULL;
    }
    return rt;
}

extern "C" void q3_attn_destroy(q3_attn_runtime *rt) {
    if (!rt) return;
    if (rt->stream) cudaStreamSynchronize(rt->stream);
    rt_free(rt, rt->k_pool);
    rt_free(rt, rt->v_pool);
    rt_free(rt, rt->q2);
    rt_free(rt, rt->part_o);
    rt_free(rt, rt->part_ml);
    rt_free(rt, rt->fix_counters);
    rt_free(rt, rt->dec_o);
    rt_free(rt, rt->dec_ml);
    rt_free(rt, rt->qk_norm_w);
    rt_free(rt, rt->rope_table);
    rt_free(rt, rt->status_dev);
    rt_free(rt, rt->gather_epoch_dev);
    rt_free(rt, rt->dev_stage);
    for (cudaEvent_t e : rt->ev) cudaEventDestroy(e);
    if (rt->gather_ready) {
        cudaStreamSynchronize(rt->gather_stream);
        for (int i = 0; i < 4; i++) cudaEventDestroy(rt->ev_gather[i]);
        cudaStreamDestroy(rt->gather_stream);
    }
    if (rt->copy_ready) {
        cudaStreamSynchronize(rt->h2d_stream);
        cudaStreamSynchronize(rt->d2h_stream);
        for (int i = 0; i < 3; i++) {
            cudaEventDestroy(rt->ev_in[i]);
            cudaEventDestroy(rt->ev_compute[i]);
            cudaEventDestroy(rt->ev_out[i]);
        }
        cudaStreamDestroy(rt->h2d_stream);
        cudaStreamDestroy(rt->d2h_stream);
    }
    if (rt->host_stage) cudaFreeHost(rt->host_stage);
    if (rt->status_host) cudaFreeHost(rt->status_host);
    if (rt->stream) cudaStreamDestroy(rt->stream);
    delete rt;
}

extern "C" bool q3_attn_set_qk_norm(q3_attn_runtime *rt, uint32_t layer,
                                    const float *q_norm_weight,
                                    const float *k_norm_weight, char *error,
                                    size_t error_len) {
    q3_clear_error(error, error_len);
    if (!rt || !q_norm_weight || !k_norm_weight || layer >= rt->cfg.num_layers)
        return q3_fail(error, error_len, "q3_attn_set_qk_norm: invalid argument");
    float *dst = rt->qk_norm_w + (size_t)layer * 2 * Q3_D;
    cudaError_t e = cudaMemcpyAsync(dst, q_norm_weight, Q3_D * sizeof(float),
                                    cudaMemcpyHostToDevice, rt->stream);
    if (e == cudaSuccess)
        e = cudaMemcpyAsync(dst + Q3_D, k_norm_weight, Q3_D * sizeof(float),
                            cudaMemcpyHostToDevice, rt->stream);
    if (e == cudaSuccess) e = cudaStreamSynchronize(rt->stream); /* set-up time */
    if (e != cudaSuccess)
        return q3_fail_cuda(error, error_len, "q3_attn_set_qk_norm", e);
    return true;
}

extern "C" bool q3_attn_set_schedule_policy(q3_attn_runtime *rt, uint32_t policy,
                                            char *error, size_t error_len) {
    q3_clear_error(error, error_len);
    if (!rt || policy > Q3_SCHED_LOCKSTEP)
        return q3_fail(error, error_len, "q3_attn_set_schedule_policy: invalid argument");
    rt->sched_policy = policy;
    return true;
}

extern "C" void *q3_attn_stream(const q3_attn_runtime *rt) {
    return rt ? (void *)rt->stream : NULL;
}

extern "C" bool q3_attn_synchronize(q3_attn_runtime *rt, char *error,
                                    size_t error_len) {
    q3_clear_error(error, error_len);
    if (!rt) return q3_fail(error, error_len, "q3_attn_synchronize: null runtime");
    cudaMemcpyAsync(rt->status_host, rt->status_dev, sizeof(uint32_t),
                    cudaMemcpyDeviceToHost, rt->stream);
    cudaError_t e = cudaStreamSynchronize(rt->stream);
    if (e == cudaSuccess && rt->copy_ready) e = cudaStreamSynchronize(rt->d2h_stream);
    if (e == cudaSuccess && rt->gather_ready) e = cudaStreamSynchronize(rt->gather_stream);
    rt->n_sync++;
    if (e != cudaSuccess)
        return q3_fail_cuda(error, error_len, "q3_attn_synchronize", e);
    if (*rt->status_host != 0) {
        if (error && error_len)
            snprintf(error, error_len,
                     "q3_attn_synchronize: a kernel gave up a bounded wait (status 0x%x)",
                     *rt->status_host);
        return false;
    }
    return true;
}

extern "C" bool q3_attn_reset_status(q3_attn_runtime *rt, char *error, size_t error_len) {
    q3_clear_error(error, error_len);
    if (!rt) return q3_fail(error, error_len, "q3_attn_reset_status: null runtime");
    if (!q3_use_device(rt, error, error_len)) return false;
    /* A launch that gave up a wait may have left arrival counters of cut items
     * part-way: clear them together with the status word, in stream order. */
    cudaError_t e = cudaMemsetAsync(rt->fix_counters, 0,
                                    (size_t)rt->part_slots * 8 * sizeof(uint32_t), rt->stream);
    if (e == cudaSuccess) e = cudaMemsetAsync(rt->status_dev, 0, sizeof(uint32_t), rt->stream);
    if (e != cudaSuccess) return q3_fail_cuda(error, error_len, "q3_attn_reset_status", e);
    *rt->status_host = 0;
    return true;
}

extern "C" bool q3_attn_enable_timing(q3_attn_runtime *rt, uint32_t max_launches,
                                      char *error, size_t error_len) {
    q3_clear_error(error, error_len);
    if (!rt || max_launches == 0)
        return q3_fail(error, error_len, "q3_attn_enable_timing: invalid argument");
    while (rt->ev.size() < 2 * (size_t)max_launches) {
        cudaEvent_t e;
        if (cudaEventCreate(&e) != cudaSuccess)
            return q3_fail(error, error_len, "q3_attn_enable_timing: cudaEventCreate failed");
        rt->ev.push_back(e);
    }
    rt->ev_phase.assign(rt->ev.size() / 2, 0);
    rt->ev_used = 0;
    rt->timing_on = true;
    return true;
}

extern "C" bool q3_attn_phase_times(q3_attn_runtime *rt, double ms_out[4],
                                    uint64_t launches_out[4], char *error,
                                    size_t error_len) {
    q3_clear_error(error, error_len);
    if (!rt || !ms_out || !launches_out)
        return q3_fail(error, error_len, "q3_attn_phase_times: invalid argument");
    for (int i = 0; i < Q3_PHASE_COUNT; i++) {
        ms_out[i] = 0.0;
        launches_out[i] = 0;
    }
    cudaError_t e = cudaStreamSynchronize(rt->stream);
    rt->n_sync++;
    if (e != cudaSuccess) return q3_fail_cuda(error, error_len, "q3_attn_phase_times", e);
    for (size_t i = 0; i < rt->ev_used; i++) {
        float ms = 0.f;
        if (cudaEventElapsedTime(&ms, rt->ev[2 * i], rt->ev[2 * i + 1]) != cudaSuccess)
            return q3_fail(error, error_len, "q3_attn_phase_times: cudaEventElapsedTime failed");
        ms_out[rt->ev_phase[i]] += ms;
        launches_out[rt->ev_phase[i]]++;
    }
    rt->ev_used = 0;
    return true;
}

extern "C" void q3_attn_get_stats(const q3_attn_runtime *rt, q3_attn_stats *stats) {
    if (!stats) return;
    memset(stats, 0, sizeof(*stats));
    if (!rt) return;
    stats->cuda_allocations = rt->n_alloc;
    stats->cuda_frees = rt->n_free;
    stats->host_syncs = rt->n_sync;
    stats->kernel_launches = rt->n_launch;
    stats->pages_total = rt->cfg.num_pages;
    stats->pages_free = rt->free_pages.size();
    stats->pool_bytes = 2ull * rt->cfg.num_layers * rt->cfg.n_kv_heads *
                        rt->cfg.num_pages * Q3_PAGE * Q3_D * sizeof(__half);
    stats->workspace_bytes = rt->workspace_bytes;
    stats->device_status = rt->status_host ? *rt->status_host : 0;
}

/* ---------------------------------------------------------------------- */
/* page pool                                                               */
/* ---------------------------------------------------------------------- */

extern "C" bool q3_pages_alloc(q3_attn_runtime *rt, uint32_t count,
                               uint32_t *pages_out, char *error, size_t error_len) {
    q3_clear_error(error, error_len);
    if (!rt || (!pages_out && count))
        return q3_fail(error, error_len, "q3_pages_alloc: invalid argument");
    if (rt->free_pages.size() < count)
        return q3_fail(error, error_len, "q3_pages_alloc: page pool exhausted");
    for (uint32_t i = 0; i < count; i++) {
        pages_out[i] = rt->free_pages.back();
        rt->free_pages.pop_back();
    }
    return true;
}

extern "C" void q3_pages_free(q3_attn_runtime *rt, const uint32_t *pages,
                              uint32_t count) {
    if (!rt || !pages) return;
    for (uint32_t i = 0; i < count; i++)
        if (pages[i] < rt->cfg.num_pages) rt->free_pages.push_back(pages[i]);
}

extern "C" void *q3_pages_k(const q3_attn_runtime *rt) { return rt ? rt->k_pool : NULL; }
extern "C" void *q3_pages_v(const q3_attn_runtime *rt) { return rt ? rt->v_pool : NULL; }

/* ---------------------------------------------------------------------- */
/* descriptor staging                                                      */
/* ---------------------------------------------------------------------- */

q3_stage *q3_stage_create(q3_attn_runtime *rt, char *error, size_t error_len) {
    q3_stage *st = new (std::nothrow) q3_stage();
    if (!st) {
        q3_fail(error, error_len, "stage: allocation failed");
        return NULL;
    }
    memset(st, 0, sizeof(*st));
    st->rt = rt;
    return st;
}

void q3_stage_destroy(q3_stage *st) {
    if (!st) return;
    /* the copy that last used the pinned buffer may still be queued */
    if (st->rt && st->rt->stream) cudaStreamSynchronize(st->rt->stream);
    if (st->has_uploaded) cudaEventDestroy(st->uploaded);
    if (st->host) cudaFreeHost(st->host);
    if (st->dev) rt_free(st->rt, st->dev);
    delete st;
}

template <typename T>
static size_t put(uint8_t *base, size_t off, const std::vector<T> &v, const T **dev_view,
                  const uint8_t *dev_base) {
    off = (off + 15) & ~(size_t)15;
    if (base && !v.empty()) memcpy(base + off, v.data(), v.size() * sizeof(T));
    if (dev_view) *dev_view = (const T *)(dev_base + off);
    return off + v.size() * sizeof(T);
}

bool q3_stage_upload(q3_stage *st, const q3_schedule &s,
                     const std::vector<uint32_t> &rope_pos,
                     const std::vector<uint32_t> &dst_page,
                     const std::vector<uint32_t> &dst_slot, char *error,
                     size_t error_len) {
    q3_attn_runtime *rt = st->rt;
    /* pass 1: size */
    size_t need = 0;
    need = put<uint32_t>(nullptr, need, rope_pos, nullptr, nullptr);
    need = put<uint32_t>(nullptr, need, dst_page, nullptr, nullptr);
    need = put<uint32_t>(nullptr, need, dst_slot, nullptr, nullptr);
    need = put<uint32_t>(nullptr, need, s.row_tag, nullptr, nullptr);
    need = put<uint32_t>(nullptr, need, s.row_lp, nullptr, nullptr);
    need = put<uint32_t>(nullptr, need, s.page_ids, nullptr, nullptr);
    need = put<q3_run>(nullptr, need, s.runs, nullptr, nullptr);
    need = put<q3_segment>(nullptr, need, s.segments, nullptr, nullptr);
    need = put<uint32_t>(nullptr, need, s.cta_seg_begin, nullptr, nullptr);
    need += 64;
    if (need > st->bytes) {
        cudaStreamSynchronize(rt->stream); /* growth is set-up, not warm path */
        if (st->host) cudaFreeHost(st->host);
        if (st->dev) rt_free(rt, st->dev);
        st->host = st->dev = nullptr;
        st->bytes = 0;
        const size_t cap = need + need / 2;
        if (cudaHostAlloc(&st->host, cap, cudaHostAllocDefault) != cudaSuccess ||
            rt_malloc(rt, &st->dev, cap) != cudaSuccess)
            return q3_fail(error, error_len, "stage: allocation failed");
        st->bytes = cap;
    } else if (st->has_uploaded && cudaEventQuery(st->uploaded) != cudaSuccess) {
        /* the pinned buffer is rewritten below: the previous upload from it
         * must have been consumed (normally long ago: no wait, no sync counted) */
        cudaEventSynchronize(st->uploaded);
        rt->n_sync++;
    }
    uint8_t *h = (uint8_t *)st->host;
    const uint8_t *d = (const uint8_t *)st->dev;
    size_t off = 0;
    off = put<uint32_t>(h, off, rope_pos, &st->rope_pos, d);
    off = put<uint32_t>(h, off, dst_page, &st->dst_page, d);
    off = put<uint32_t>(h, off, dst_slot, &st->dst_slot, d);
    off = put<uint32_t>(h, off, s.row_tag, &st->row_tag, d);
    off = put<uint32_t>(h, off, s.row_lp, &st->row_lp, d);
    off = put<uint32_t>(h, off, s.page_ids, &st->page_ids, d);
    off = put<q3_run>(h, off, s.runs, &st->runs, d);
    off = put<q3_segment>(h, off, s.segments, &st->segments, d);
    off = put<uint32_t>(h, off, s.cta_seg_begin, &st->cta_seg_begin, d);
    st->tokens = s.tokens;
    st->n_shared_pages = s.n_shared_pages;
    st->shared_len = s.shared_len;
    st->grid = s.grid;
    cudaError_t e = cudaMemcpyAsync(st->dev, st->host, off, cudaMemcpyHostToDevice,
                                    rt->stream);
    if (e != cudaSuccess) return q3_fail_cuda(error, error_len, "stage: upload", e);
    if (!st->has_uploaded) {
        if (cudaEventCreateWithFlags(&st->uploaded, cudaEventDisableTiming) != cudaSuccess)
            return q3_fail(error, error_len, "stage: event creation failed");
        st->has_uploaded = true;
    }
    cudaEventRecord(st->uploaded, rt->stream);
    return true;
}

/* ---------------------------------------------------------------------- */
/* shared prefix (ref: src/q3_decide.cu:61-184)                            */
/* ---------------------------------------------------------------------- */

static q3_prefix_kv *prefix_new(q3_attn_runtime *rt, uint32_t capacity_tokens,
                                const uint32_t *pages, char *error,
                                size_t error_len, const char *who) {
    q3_clear_error(error, error_len);
    if (!rt || capacity_tokens == 0) {
        if (error && error_len) snprintf(error, error_len, "%s: invalid argument", who);
        return NULL;
    }
    if (capacity_tokens > rt->cfg.max_positions) {
        if (error && error_len)
            snprintf(error, error_len, "%s: capacity exceeds max_positions", who);
        return NULL;
    }
    q3_prefix_kv *p = new (std::nothrow) q3_prefix_kv();
    if (!p) {
        if (error && error_len) snprintf(error, error_len, "%s: allocation failed", who);
        return NULL;
    }
    p->rt = rt;
    p->capacity = capacity_tokens;
    p->token_count = 0;
    p->sealed = false;
    p->stage = nullptr;
    const uint32_t n = (capacity_tokens + Q3_PAGE - 1) / Q3_PAGE;
    p->pages.resize(n);
    if (pages) {
        p->owns_pages = false;
        for (uint32_t i = 0; i < n; i++) {
            if (pages[i] >= rt->cfg.num_pages) {
                if (error && error_len)
                    snprintf(error, error_len, "%s: page id out of range", who);
                delete p;
                return NULL;
            }
            p->pages[i] = pages[i];
        }
    } else {
        p->owns_pages = true;
        if (!q3_pages_alloc(rt, n, p->pages.data(), error, error_len)) {
            delete p;
            return NULL;
        }
    }
    p->stage = q3_stage_create(rt, error, error_len);
    if (!p->stage) {
        if (p->owns_pages) q3_pages_free(rt, p->pages.data(), n);
        delete p;
        return NULL;
    }
    return p;
}

extern "C" q3_prefix_kv *q3_prefix_create(q3_attn_runtime *rt,
                                          uint32_t capacity_tokens, char *error,
                                          size_t error_len) {
    return prefix_new(rt, capacity_tokens, NULL, error, error_len, "q3_prefix_create");
}

extern "C" q3_prefix_kv *q3_prefix_create_with_pages(q3_attn_runtime *rt,
                                                     uint32_t capacity_tokens,
                                                     const uint32_t *pages,
                                                     char *error, size_t error_len) {
    if (!pages) {
        q3_clear_error(error, error_len);
        q3_fail(error, error_len, "q3_prefix_create_with_pages: invalid argument");
        return NULL;
    }
    return prefix_new(rt, capacity_tokens, pages, error, error_len,
                      "q3_prefix_create_with_pages");
}

/* Validation and the chunk's schedule, shared by the two prefill entries. */
static q3_stage *prefill_prepare(q3_prefix_kv *prefix, uint32_t layer, uint32_t tokens,
                                 char *error, size_t error_len) {
    q3_attn_runtime *rt = prefix->rt;
    if (!q3_use_device(rt, error, error_len)) return NULL;
    if (prefix->sealed) {
        q3_fail(error, error_len, "q3_prefix_prefill_layer: prefix already sealed");
        return NULL;
    }
    if (layer >= rt->cfg.num_layers) {
        q3_fail(error, error_len, "q3_prefix_prefill_layer: layer out of range");
        return NULL;
    }
    if ((uint64_t)prefix->token_count + tokens > prefix->capacity) {
        q3_fail(error, error_len, "q3_prefix_prefill_layer: token_count exceeds capacity");
        return NULL;
    }
    if (tokens > rt->cfg.max_tokens) {
        q3_fail(error, error_len,
                "q3_prefix_prefill_layer: token_count exceeds runtime capacity");
        return NULL;
    }
    q3_stage *st = prefix->stage;
    const uint32_t base = prefix->token_count;
    /* The schedule depends only on (base, tokens): built for the first layer
     * of a chunk and reused by the others. */
    if (!st->chunk_valid || st->chunk_base != base || st->chunk_tokens != tokens) {
        std::vector<uint32_t> pos(tokens), dpage(tokens), dslot(tokens), tag(tokens, 0);
        for (uint32_t t = 0; t < tokens; t++) {
            pos[t] = base + t;
            dpage[t] = prefix->pages[(base + t) / Q3_PAGE];
            dslot[t] = (base + t) % Q3_PAGE;
        }
        q3_schedule s;
        std::vector<uint32_t> no_shared;
        if (!q3_build_schedule(s, tokens, rt->cfg.n_kv_heads, 0, no_shared, tag.data(),
                               pos.data(), prefix->pages, (uint32_t)prefix->pages.size(),
                               (uint32_t)rt->num_sms, rt->part_slots, false, error,
                               error_len))
            return NULL;
        if (!q3_stage_upload(st, s, pos, dpage, dslot, error, error_len)) return NULL;
        st->chunk_valid = true;
        st->chunk_base = base;
        st->chunk_tokens = tokens;
    }
    return st;
}

extern "C" bool q3_prefix_prefill_layer(q3_prefix_kv *prefix, uint32_t layer,
                                        const void *q, const void *k,
                                        const void *v, uint32_t tokens, void *out,
                                        char *error, size_t error_len) {
    q3_clear_error(error, error_len);
    if (!prefix || !q || !k || !v || !out || tokens == 0)
        return q3_fail(error, error_len, "q3_prefix_prefill_layer: invalid argument");
    q3_attn_runtime *rt = prefix->rt;
    q3_stage *st = prefill_prepare(prefix, layer, tokens, error, error_len);
    if (!st) return false;
    if (!q3_launch_kvwrite(rt, layer, q, k, v, tokens, st->rope_pos, st->dst_page,
                           st->dst_slot, rt->q2, error, error_len))
        return false;
    return q3_launch_attention(rt, layer, st, out, error, error_len);
}

/* The q/k/v projection of the layer with norm + RoPE + page write as its
 * epilogue, then attention: two launches, and q, k, v never exist as tensors. */
static bool projected_layer(q3_attn_runtime *rt, uint32_t layer, const q3_qkv_weights *w,
                            const void *x_f16, uint32_t tokens, const q3_stage *st, void *out,
                            char *error, size_t error_len) {
    const q3_attn_config &c = rt->cfg;
    if (w->qtype_q != w->qtype_k || w->qtype_q != w->qtype_v)
        return q3_fail(error, error_len,
                       "fused q/k/v projection: the three weights must have one quantisation "
                       "type and layout (project them one by one otherwise)");
    const size_t layer_off = (size_t)layer * c.n_kv_heads * c.num_pages * Q3_PAGE * Q3_D;
    q3_qkv_fused_args a;
    a.wq = w->wq;
    a.wk = w->wk;
    a.wv = w->wv;
    a.qtype = w->qtype_q;
    a.hidden = w->hidden;
    a.n_q_heads = c.n_heads;
    a.n_kv_heads = c.n_kv_heads;
    a.x_f16 = x_f16;
    a.tokens = tokens;
    a.norm_w = rt->qk_norm_w + (size_t)layer * 2 * Q3_D;
    a.eps = c.rms_eps;
    a.rope_table = rt->rope_table;
    a.rope_pos = st->rope_pos;
    a.dst_page = st->dst_page;
    a.dst_slot = st->dst_slot;
    a.q_out = rt->q2;
    a.k_pool = rt->k_pool + layer_off;
    a.v_pool = rt->v_pool + layer_off;
    a.num_pages = c.num_pages;
    q3_phase_begin(rt, Q3_PHASE_KVWRITE);
    const bool ok = q3_launch_qkv_fused(&a, rt->stream, error, error_len);
    q3_phase_end(rt);
    if (!ok) return false;
    rt->n_launch++;
    return q3_launch_attention(rt, layer, st, out, error, error_len);
}

extern "C" bool q3_prefix_prefill_layer_projected(q3_prefix_kv *prefix, uint32_t layer,
                                                  const q3_qkv_weights *weights,
                                                  const void *x_f16, uint32_t tokens,
                                                  void *out, char *error, size_t error_len) {
    q3_clear_error(error, error_len);
    if (!prefix || !weights || !weights->wq || !weights->wk || !weights->wv || !x_f16 ||
        !out || tokens == 0)
        return q3_fail(error, error_len,
                       "q3_prefix_prefill_layer_projected: invalid argument");
    q3_stage *st = prefill_prepare(prefix, layer, tokens, error, error_len);
    if (!st) return false;
    return projected_layer(prefix->rt, layer, weights, x_f16, tokens, st, out, error,
                           error_len);
}

extern "C" bool q3_suffix_attention_layer_projected(q3_pack_plan *plan, uint32_t layer,
                                                    const q3_qkv_weights *weights,
                                                    const void *x_f16, void *out,
                                                    char *error, size_t error_len) {
    q3_clear_error(error, error_len);
    if (!plan || !weights || !weights->wq || !weights->wk || !weights->wv || !x_f16 || !out)
        return q3_fail(error, error_len,
                       "q3_suffix_attention_layer_projected: invalid argument");
    q3_attn_runtime *rt = plan->prefix->rt;
    if (!q3_use_device(rt, error, error_len)) return false;
    if (layer >= rt->cfg.num_layers)
        return q3_fail(error, error_len,
                       "q3_suffix_attention_layer_projected: layer out of range");
    return projected_layer(rt, layer, weights, x_f16, plan->tokens, plan->stage, out, error,
                           error_len);
}

extern "C" bool q3_prefix_advance(q3_prefix_kv *prefix, uint32_t tokens,
                                  char *error, size_t error_len) {
    q3_clear_error(error, error_len);
    if (!prefix) return q3_fail(error, error_len, "q3_prefix_advance: null prefix");
    if (prefix->sealed)
        return q3_fail(error, error_len, "q3_prefix_advance: prefix already sealed");
    if ((uint64_t)prefix->token_count + tokens > prefix->capacity)
        return q3_fail(error, error_len, "q3_prefix_advance: exceeds capacity");
    prefix->token_count += tokens;
    prefix->stage->chunk_valid = false;
    return true;
}

extern "C" bool q3_prefix_set_resident(q3_prefix_kv *prefix, uint32_t token_count,
                                       char *error, size_t error_len) {
    q3_clear_error(error, error_len);
    if (!prefix) return q3_fail(error, error_len, "q3_prefix_set_resident: null prefix");
    if (prefix->sealed)
        return q3_fail(error, error_len, "q3_prefix_set_resident: prefix already sealed");
    if (token_count > prefix->capacity)
        return q3_fail(error, error_len, "q3_prefix_set_resident: exceeds capacity");
    prefix->token_count = token_count;
    prefix->stage->chunk_valid = false;
    return true;
}

extern "C" bool q3_prefix_seal(q3_prefix_kv *prefix, char *error, size_t error_len) {
    q3_clear_error(error, error_len);
    if (!prefix) return q3_fail(error, error_len, "q3_prefix_seal: null prefix");
    if (prefix->token_count == 0)
        return q3_fail(error, error_len, "q3_prefix_seal: prefix is empty");
    prefix->sealed = true;
    return true;
}

extern "C" void q3_prefix_destroy(q3_prefix_kv *prefix) {
    if (!prefix) return;
    q3_stage_destroy(prefix->stage);
    if (prefix->owns_pages)
        q3_pages_free(prefix->rt, prefix->pages.data(), (uint32_t)prefix->pages.size());
    delete prefix;
}

extern "C" uint32_t q3_prefix_token_count(const q3_prefix_kv *prefix) {
    return prefix ? prefix->token_count : 0;
}

extern "C" size_t q3_prefix_kv_bytes(const q3_prefix_kv *prefix) {
    if (!prefix) return 0;
    const q3_attn_config &c = prefix->rt->cfg;
    return 2 * (size_t)c.num_layers * prefix->pages.size() * Q3_PAGE * c.n_kv_heads *
           Q3_D * sizeof(__half);
}

extern "C" uint64_t q3_prefix_copy_bytes(const q3_prefix_kv *prefix) {
    (void)prefix;
    return 0;
}

extern "C" uint64_t q3_prefix_allocations(const q3_prefix_kv *prefix) {
    (void)prefix;
    return 0;
}

extern "C" const uint32_t *q3_prefix_page_table(const q3_prefix_kv *prefix) {
    return prefix ? prefix->pages.data() : NULL;
}

/* ---------------------------------------------------------------------- */
/* branch set (ref: src/q3_decide.cu:191-347)                              */
/* ---------------------------------------------------------------------- */

extern "C" q3_branch_set *q3_branch_set_create(q3_prefix_kv *prefix,
                                               uint32_t max_branches,
                                               uint32_t max_suffix_tokens,
                                               char *error, size_t error_len) {
    q3_clear_error(error, error_len);
    if (!prefix || max_branches == 0 || max_suffix_tokens == 0 ||
        max_branches > Q3_PACK_MAX_BRANCHES) {
        q3_fail(error, error_len, "q3_branch_set_create: invalid argument");
        return NULL;
    }
    q3_branch_set *set = new (std::nothrow) q3_branch_set();
    if (!set) {
        q3_fail(error, error_len, "q3_branch_set_create: allocation failed");
        return NULL;
    }
    set->prefix = prefix;
    set->max_branches = max_branches;
    set->max_suffix = max_suffix_tokens;
    set->pages_per_branch = (max_suffix_tokens + Q3_PAGE - 1) / Q3_PAGE;
    set->live = 0;
    set->decide = nullptr;
    set->in_use.assign(max_branches, 0);
    set->pages.resize((size_t)max_branches * set->pages_per_branch);
    if (!q3_pages_alloc(prefix->rt, (uint32_t)set->pages.size(), set->pages.data(),
                        error, error_len)) {
        delete set;
        return NULL;
    }
    return set;
}

extern "C" int32_t q3_branch_acquire(q3_branch_set *set, char *error,
                                     size_t error_len) {
    q3_clear_error(error, error_len);
    if (!set) {
        q3_fail(error, error_len, "q3_branch_acquire: null set");
        return -1;
    }
    for (uint32_t b = 0; b < set->max_branches; b++)
        if (!set->in_use[b]) {
            set->in_use[b] = 1;
            set->live++;
            return (int32_t)b;
        }
    q3_fail(error, error_len, "q3_branch_acquire: branch limit exceeded");
    return -1;
}

extern "C" void q3_branch_reset(q3_branch_set *set, int32_t branch) {
    /* Descriptor only, as in the reference: a branch's suffix length lives in
     * the caller's item (ref: src/q3_decide.cu:296-301). */
    (void)set;
    (void)branch;
}

extern "C" void q3_branch_release(q3_branch_set *set, int32_t branch) {
    if (!set || branch < 0 || (uint32_t)branch >= set->max_branches) return;
    if (set->in_use[branch]) {
        set->in_use[branch] = 0;
        set->live--;
    }
}

extern "C" void q3_branch_set_destroy(q3_branch_set *set) {
    if (!set) return;
    q3_decide_state_destroy(set);
    q3_pages_free(set->prefix->rt, set->pages.data(), (uint32_t)set->pages.size());
    delete set;
}

extern "C" size_t q3_branch_set_kv_bytes(const q3_branch_set *set) {
    if (!set) return 0;
    const q3_attn_config &c = set->prefix->rt->cfg;
    return 2 * (size_t)c.num_layers * set->pages.size() * Q3_PAGE * c.n_kv_heads * Q3_D *
           sizeof(__half);
}

extern "C" uint32_t q3_branch_set_max_branches(const q3_branch_set *set) {
    return set ? set->max_branches : 0;
}
extern "C" uint32_t q3_branch_set_max_suffix(const q3_branch_set *set) {
    return set ? set->max_suffix : 0;
}
extern "C" const uint32_t *q3_branch_set_page_table(const q3_branch_set *set) {
    return set ? set->pages.data() : NULL;
}
extern "C" uint32_t q3_branch_set_pages_per_branch(const q3_branch_set *set) {
    return set ? set->pages_per_branch : 0;
}

/* ---------------------------------------------------------------------- */
/* suffix packing (ref: src/q3_decide.cu:369-480)                          */
/* ---------------------------------------------------------------------- */

extern "C" int64_t q3_pack_suffix_host(const q3_suffix_item *items, uint32_t count,
                                       uint32_t prefix_len, uint32_t max_branches,
                                       uint32_t max_suffix,
                                       uint32_t *token_positions,
                                       uint32_t *token_branch,
                                       uint32_t *token_local_pos,
                                       uint32_t *branch_offsets, char *error,
                                       size_t error_len) {
    q3_clear_error(error, error_len);
    if (!items || !token_positions || !token_branch || !token_local_pos ||
        !branch_offsets) {
        q3_fail(error, error_len, "q3_pack_suffix_host: invalid argument");
        return -1;
    }
    if (count == 0 || count > Q3_PACK_MAX_BRANCHES || count > max_branches) {
        q3_fail(error, error_len, "q3_pack_suffix_host: bad branch count");
        return -1;
    }
    uint32_t cursor = 0;
    for (uint32_t b = 0; b < count; b++) {
        const q3_suffix_item *item = &items[b];
        if (item->token_count == 0 || item->token_count > max_suffix) {
            q3_fail(error, error_len, "q3_pack_suffix_host: invalid decision item");
            return -1;
        }
        if (item->branch >= max_branches) {
            q3_fail(error, error_len, "q3_pack_suffix_host: invalid branch handle");
            return -1;
        }
        branch_offsets[b] = cursor;
        for (uint32_t j = 0; j < item->token_count; j++) {
            const uint32_t t = cursor + j;
            token_branch[t] = item->branch;
            token_local_pos[t] = j;
            /* the suffix continues right after the shared prefix, identically
             * for every branch (ref: src/q3_decide.cu:455-457) */
            token_positions[t] = prefix_len + j;
        }
        cursor += item->token_count;
    }
    branch_offsets[count] = cursor;
    return (int64_t)cursor;
}

/* Staggered stream-K access keeps the shared KV of ALL local heads live at
 * once; when that exceeds what L2 holds comfortably, walk items in lockstep. */
static bool q3_prefers_lockstep(const q3_attn_runtime *rt, uint32_t shared_len) {
    if (rt->sched_policy == Q3_SCHED_STREAMK) return false;
    if (rt->sched_policy == Q3_SCHED_LOCKSTEP) return true;
    const uint64_t kv_bytes = (uint64_t)((shared_len + Q3_PAGE - 1) / Q3_PAGE) * 2 * 4096 *
                              rt->cfg.n_kv_heads;
    return kv_bytes > (48ull << 20);
}

/* Pack `items` and stage descriptors + schedule into `stage` (grow-once).
 * Shared by q3_pack_plan_create and q3_decide_run, which keeps its stage in
 * the branch set so that a warm batch allocates nothing. */
bool q3_pack_plan_build(q3_pack_plan *plan, q3_stage *stage, q3_prefix_kv *prefix,
                        q3_branch_set *set, const q3_suffix_item *items, uint32_t count,
                        const char *who, char *error, size_t error_len) {
    char msg[160];
    auto fail = [&](const char *what) {
        snprintf(msg, sizeof(msg), "%s: %s", who, what);
        return q3_fail(error, error_len, msg);
    };
    if (!prefix->sealed) return fail("prefix not sealed");
    if (set->prefix != prefix) return fail("branch set belongs to another prefix");
    q3_attn_runtime *rt = prefix->rt;
    uint64_t total = 0;
    for (uint32_t b = 0; b < count; b++) total += items[b].token_count;
    if (count == 0 || total == 0) return fail("bad branch count");
    if (total > rt->cfg.max_tokens) return fail("packed batch exceeds runtime capacity");
    if ((uint64_t)prefix->token_count + set->max_suffix > rt->cfg.max_positions)
        return fail("suffix positions exceed max_positions");
    plan->prefix = prefix;
    plan->set = set;
    plan->branches = count;
    plan->stage = stage;
    plan->token_positions.resize(total);
    plan->token_branch.resize(total);
    plan->token_local_pos.resize(total);
    plan->branch_offsets.resize(count + 1);
    const int64_t packed = q3_pack_suffix_host(
        items, count, prefix->token_count, set->max_branches, set->max_suffix,
        plan->token_positions.data(), plan->token_branch.data(),
        plan->token_local_pos.data(), plan->branch_offsets.data(), error, error_len);
    if (packed < 0) return false;
    plan->tokens = (uint32_t)packed;
    std::vector<uint32_t> dpage(plan->tokens), dslot(plan->tokens);
    for (uint32_t t = 0; t < plan->tokens; t++) {
        const uint32_t b = plan->token_branch[t], lp = plan->token_local_pos[t];
        dpage[t] = set->pages[(size_t)b * set->pages_per_branch + lp / Q3_PAGE];
        dslot[t] = lp % Q3_PAGE;
    }
    q3_schedule s;
    return q3_build_schedule(s, plan->tokens, rt->cfg.n_kv_heads, prefix->token_count,
                             prefix->pages, plan->token_branch.data(),
                             plan->token_local_pos.data(), set->pages,
                             set->pages_per_branch, (uint32_t)rt->num_sms, rt->part_slots,
                             q3_prefers_lockstep(rt, prefix->token_count), error,
                             error_len) &&
           q3_stage_upload(stage, s, plan->token_positions, dpage, dslot, error, error_len);
}

extern "C" q3_pack_plan *q3_pack_plan_create(q3_prefix_kv *prefix,
                                             q3_branch_set *set,
                                             const q3_suffix_item *items,
                                             uint32_t count, char *error,
                                             size_t error_len) {
    q3_clear_error(error, error_len);
    if (!prefix || !set || !items) {
        q3_fail(error, error_len, "q3_pack_plan_create: invalid argument");
        return NULL;
    }
    q3_pack_plan *plan = new (std::nothrow) q3_pack_plan();
    q3_stage *stage = plan ? q3_stage_create(prefix->rt, error, error_len) : nullptr;
    if (!plan || !stage) {
        if (!plan) q3_fail(error, error_len, "q3_pack_plan_create: allocation failed");
        delete plan;
        return NULL;
    }
    if (!q3_pack_plan_build(plan, stage, prefix, set, items, count, "q3_pack_plan_create",
                            error, error_len)) {
        q3_stage_destroy(stage);
        delete plan;
        return NULL;
    }
    return plan;
}

extern "C" void q3_pack_plan_destroy(q3_pack_plan *plan) {
    if (!plan) return;
    q3_stage_destroy(plan->stage);
    delete plan;
}

extern "C" uint32_t q3_pack_plan_tokens(const q3_pack_plan *plan) {
    return plan ? plan->tokens : 0;
}
extern "C" const uint32_t *q3_pack_plan_token_positions(const q3_pack_plan *plan) {
    return plan ? plan->token_positions.data() : NULL;
}
extern "C" const uint32_t *q3_pack_plan_token_branch(const q3_pack_plan *plan) {
    return plan ? plan->token_branch.data() : NULL;
}
extern "C" const uint32_t *q3_pack_plan_token_local_pos(const q3_pack_plan *plan) {
    return plan ? plan->token_local_pos.data() : NULL;
}
extern "C" const uint32_t *q3_pack_plan_branch_offsets(const q3_pack_plan *plan) {
    return plan ? plan->branch_offsets.data() : NULL;
}

extern "C" bool q3_suffix_attention_layer(q3_pack_plan *plan, uint32_t layer,
                                          const void *q, const void *k,
                                          const void *v, void *out, char *error,
                                          size_t error_len) {
    q3_clear_error(error, error_len);
    if (!plan || !q || !k || !v || !out)
        return q3_fail(error, error_len, "q3_suffix_attention_layer: invalid argument");
    q3_attn_runtime *rt = plan->prefix->rt;
    if (!q3_use_device(rt, error, error_len)) return false;
    if (layer >= rt->cfg.num_layers)
        return q3_fail(error, error_len, "q3_suffix_attention_layer: layer out of range");
    const q3_stage *st = plan->stage;
    if (!q3_launch_kvwrite(rt, layer, q, k, v, plan->tokens, st->rope_pos, st->dst_page,
                           st->dst_slot, rt->q2, error, error_len))
        return false;
    return q3_launch_attention(rt, layer, st, out, error, error_len);
}

extern "C" bool q3_suffix_attention_layer_gathered(q3_pack_plan *plan, uint32_t layer,
                                                   const void *q, const void *k,
                                                   const void *v,
                                                   const q3_gather_peers *gather,
                                                   uint32_t seq, char *error,
                                                   size_t error_len) {
    q3_clear_error(error, error_len);
    if (!plan || !q || !k || !v || !gather || gather->n_ranks == 0 ||
        gather->n_ranks > Q3_MAX_GATHER_RANKS || gather->rank >= gather->n_ranks)
        return q3_fail(error, error_len,
                       "q3_suffix_attention_layer_gathered: invalid argument");
    for (uint32_t d = 0; d < gather->n_ranks; d++)
        if (!gather->gathered[d] || !gather->flags[d])
            return q3_fail(error, error_len,
                           "q3_suffix_attention_layer_gathered: invalid argument");
    q3_attn_runtime *rt = plan->prefix->rt;
    if (!q3_use_device(rt, error, error_len)) return false;
    if (layer >= rt->cfg.num_layers)
        return q3_fail(error, error_len,
                       "q3_suffix_attention_layer_gathered: layer out of range");
    const q3_stage *st = plan->stage;
    const size_t slot_bytes =
        (size_t)plan->tokens * rt->cfg.n_heads * Q3_D * (rt->cfg.out_fp32 ? 4 : 2);
    void *local = (uint8_t *)gather->gathered[gather->rank] + slot_bytes * gather->rank;
    if (!q3_launch_kvwrite(rt, layer, q, k, v, plan->tokens, st->rope_pos, st->dst_page,
                           st->dst_slot, rt->q2, error, error_len))
        return false;
    /* The kernels write this rank's slot of its own gathered buffer. The copies
     * to the other ranks go through the copy engines on a side stream (NVLink,
     * no SM involved), overlapped with the next layer's kernels; the flags are
     * published after them on the same stream. (Storing the rows into peer
     * memory from the attention epilogue was measured and dropped: scattered
     * 16-byte remote stores stalled the softmax warps, 450 us instead of 250 us
     * per layer at 8 GPUs.) */
    if (!q3_launch_attention(rt, layer, st, local, error, error_len)) return false;
    if (!rt->gather_ready) {
        bool ok = cudaStreamCreateWithFlags(&rt->gather_stream, cudaStreamNonBlocking) ==
                  cudaSuccess;
        for (int i = 0; i < 4 && ok; i++)
            ok = cudaEventCreateWithFlags(&rt->ev_gather[i], cudaEventDisableTiming) ==
                 cudaSuccess;
        if (!ok)
            return q3_fail(error, error_len,
                           "q3_suffix_attention_layer_gathered: stream set-up failed");
        rt->gather_ready = true;
    }
    if (rt->capturing) rt->capture_used_gather = true;
    cudaEvent_t ev = rt->ev_gather[rt->gather_calls++ % 4];
    cudaError_t e = cudaEventRecord(ev, rt->stream);
    if (e == cudaSuccess) e = cudaStreamWaitEvent(rt->gather_stream, ev, 0);
    for (uint32_t d = 0; d < gather->n_ranks && e == cudaSuccess; d++)
        if (d != gather->rank)
            e = cudaMemcpyAsync((uint8_t *)gather->gathered[d] + slot_bytes * gather->rank,
                                local, slot_bytes, cudaMemcpyDeviceToDevice,
                                rt->gather_stream);
    if (e != cudaSuccess)
        return q3_fail_cuda(error, error_len, "q3_suffix_attention_layer_gathered: copy", e);
    return q3_launch_gather_signal(rt, gather, seq, rt->gather_stream, error, error_len);
}

extern "C" bool q3_attn_wait_gathered(q3_attn_runtime *rt, const q3_gather_peers *gather,
                                      uint32_t seq, char *error, size_t error_len) {
    q3_clear_error(error, error_len);
    if (!rt || !gather || gather->n_ranks == 0 || gather->n_ranks > Q3_MAX_GATHER_RANKS ||
        gather->rank >= gather->n_ranks || !gather->flags[gather->rank])
        return q3_fail(error, error_len, "q3_attn_wait_gathered: invalid argument");
    return q3_launch_gather_wait(rt, gather, seq, error, error_len);
}

extern "C" bool q3_attn_gather_advance(q3_attn_runtime *rt, uint32_t count, char *error,
                                       size_t error_len) {
    q3_clear_error(error, error_len);
    if (!rt) return q3_fail(error, error_len, "q3_attn_gather_advance: null runtime");
    return q3_launch_gather_advance(rt, count, error, error_len);
}

extern "C" bool q3_cuda_qknorm_rope_kvwrite(q3_attn_runtime *rt, uint32_t layer,
                                            const void *q, const void *k,
                                            const void *v, uint32_t tokens,
                                            const uint32_t *rope_pos,
                                            const uint32_t *dst_page,
                                            const uint32_t *dst_slot, void *q_out,
                                            char *error, size_t error_len) {
    q3_clear_error(error, error_len);
    if (!rt || tokens == 0 || !rope_pos || (!q && !k) || (q && !q_out) ||
        ((k || v) && (!k || !v || !dst_page || !dst_slot)))
        return q3_fail(error, error_len, "q3_cuda_qknorm_rope_kvwrite: invalid argument");
    if (layer >= rt->cfg.num_layers)
        return q3_fail(error, error_len, "q3_cuda_qknorm_rope_kvwrite: layer out of range");
    return q3_launch_kvwrite(rt, layer, q, k, v, tokens, rope_pos, dst_page, dst_slot,
                             q_out, error, error_len);
}

/* ---------------------------------------------------------------------- */
/* host-buffer entry                                                       */
/* ---------------------------------------------------------------------- */

/* Shared by the two host-buffer entries; gather == NULL: plain layer call. */
static bool host_layer(q3_pack_plan *plan, uint32_t layer, const void *q_host,
                       const void *k_host, const void *v_host, void *out_host,
                       const q3_gather_peers *gather, uint32_t seq, char *error,
                       size_t error_len) {
    q3_clear_error(error, error_len);
    if (!plan || !q_host || !k_host || !v_host || !out_host)
        return q3_fail(error, error_len,
                       "q3_suffix_attention_layer_host: invalid argument");
    q3_attn_runtime *rt = plan->prefix->rt;
    if (rt->capturing)
        return q3_fail(error, error_len,
                       "q3_suffix_attention_layer_host: cannot be recorded into a graph");
    const size_t qb = (size_t)plan->tokens * rt->cfg.n_heads * Q3_D * 2;
    const size_t kb = (size_t)plan->tokens * rt->cfg.n_kv_heads * Q3_D * 2;
    const size_t ob = rt->cfg.out_fp32 ? 2 * qb : qb;
    const size_t need = (qb + ob + 2 * kb + 255) & ~(size_t)255;
    if (!rt->copy_ready) {
        /* set-up, once: two copy streams and the events that order the slots */
        bool ok = cudaStreamCreateWithFlags(&rt->h2d_stream, cudaStreamNonBlocking) == cudaSuccess &&
                  cudaStreamCreateWithFlags(&rt->d2h_stream, cudaStreamNonBlocking) == cudaSuccess;
        for (int i = 0; i < 3 && ok; i++)
            ok = cudaEventCreateWithFlags(&rt->ev_in[i], cudaEventDisableTiming) == cudaSuccess &&
                 cudaEventCreateWithFlags(&rt->ev_compute[i], cudaEventDisableTiming) == cudaSuccess &&
                 cudaEventCreateWithFlags(&rt->ev_out[i], cudaEventDisableTiming) == cudaSuccess;
        if (!ok)
            return q3_fail(error, error_len,
                           "q3_suffix_attention_layer_host: stream set-up failed");
        rt->copy_ready = true;
    }
    if (need > rt->dev_stage_bytes) {
        cudaStreamSynchronize(rt->stream);
        cudaStreamSynchronize(rt->h2d_stream);
        cudaStreamSynchronize(rt->d2h_stream);
        rt_free(rt, rt->dev_stage);
        rt->dev_stage = nullptr;
        rt->dev_stage_bytes = 0;
        if (rt_malloc(rt, &rt->dev_stage, 3 * need) != cudaSuccess)
            return q3_fail(error, error_len,
                           "q3_suffix_attention_layer_host: allocation failed");
        rt->dev_stage_bytes = need;
        rt->host_calls = 0;
    }
    /* Slot i%3: copy-in (h2d stream) -> kernels (runtime stream) -> copy-out
     * (d2h stream). The copy-in of call i+1 and the copy-out of call i-1 run
     * while call i computes. A slot is reused only after its copy-out. */
    const uint32_t slot = (uint32_t)(rt->host_calls % 3);
    const bool reused = rt->host_calls >= 3;
    rt->host_calls++;
    uint8_t *d = (uint8_t *)rt->dev_stage + (size_t)slot * rt->dev_stage_bytes;
    void *dq = d, *dk = d + qb, *dv = d + qb + kb, *dout = d + qb + 2 * kb;
    cudaError_t e = cudaSuccess;
    if (reused) e = cudaStreamWaitEvent(rt->h2d_stream, rt->ev_out[slot], 0);
    if (e == cudaSuccess)
        e = cudaMemcpyAsync(dq, q_host, qb, cudaMemcpyHostToDevice, rt->h2d_stream);
    if (e == cudaSuccess)
        e = cudaMemcpyAsync(dk, k_host, kb, cudaMemcpyHostToDevice, rt->h2d_stream);
    if (e == cudaSuccess)
        e = cudaMemcpyAsync(dv, v_host, kb, cudaMemcpyHostToDevice, rt->h2d_stream);
    if (e == cudaSuccess) e = cudaEventRecord(rt->ev_in[slot], rt->h2d_stream);
    if (e == cudaSuccess) e = cudaStreamWaitEvent(rt->stream, rt->ev_in[slot], 0);
    if (e != cudaSuccess)
        return q3_fail_cuda(error, error_len, "q3_suffix_attention_layer_host: H2D", e);
    const void *result = dout;
    if (gather) {
        /* The rows land in this rank's slot of its own gathered buffer, which
         * the caller alternates between two buffers: the copy-out of the call
         * two back read the buffer this call overwrites. */
        if (rt->host_calls >= 3)
            e = cudaStreamWaitEvent(rt->stream, rt->ev_out[(slot + 1) % 3], 0);
        if (e != cudaSuccess)
            return q3_fail_cuda(error, error_len, "q3_suffix_attention_layer_host: order", e);
        if (!q3_suffix_attention_layer_gathered(plan, layer, dq, dk, dv, gather, seq, error,
                                                error_len))
            return false;
        result = (const uint8_t *)gather->gathered[gather->rank] + ob * gather->rank;
    } else if (!q3_suffix_attention_layer(plan, layer, dq, dk, dv, dout, error, error_len)) {
        return false;
    }
    e = cudaEventRecord(rt->ev_compute[slot], rt->stream);
    if (e == cudaSuccess) e = cudaStreamWaitEvent(rt->d2h_stream, rt->ev_compute[slot], 0);
    if (e == cudaSuccess)
        e = cudaMemcpyAsync(out_host, result, ob, cudaMemcpyDeviceToHost, rt->d2h_stream);
    if (e == cudaSuccess) e = cudaEventRecord(rt->ev_out[slot], rt->d2h_stream);
    if (e != cudaSuccess)
        return q3_fail_cuda(error, error_len, "q3_suffix_attention_layer_host: D2H", e);
    return true;
}

extern "C" bool q3_suffix_attention_layer_host(q3_pack_plan *plan, uint32_t layer,
                                               const void *q_host,
                                               const void *k_host,
                                               const void *v_host, void *out_host,
                                               char *error, size_t error_len) {
    return host_layer(plan, layer, q_host, k_host, v_host, out_host, NULL, 0, error,
                      error_len);
}

extern "C" bool q3_suffix_attention_layer_gathered_host(
    q3_pack_plan *plan, uint32_t layer, const void *q_host, const void *k_host,
    const void *v_host, const q3_gather_peers *gather, uint32_t seq, void *out_host,
    char *error, size_t error_len) {
    if (!gather) {
        q3_clear_error(error, error_len);
        return q3_fail(error, error_len,
                       "q3_suffix_attention_layer_gathered_host: invalid argument");
    }
    return host_layer(plan, layer, q_host, k_host, v_host, out_host, gather, seq, error,
                      error_len);
}

/* ---------------------------------------------------------------------- */
/* graph capture of a sequence of layer calls                              */
/* ---------------------------------------------------------------------- */

extern "C" bool q3_attn_graph_begin(q3_attn_runtime *rt, char *error, size_t error_len) {
    q3_clear_error(error, error_len);
    if (!rt) return q3_fail(error, error_len, "q3_attn_graph_begin: null runtime");
    if (rt->capturing) return q3_fail(error, error_len, "q3_attn_graph_begin: already recording");
    if (!q3_use_device(rt, error, error_len)) return false;
    cudaError_t e = cudaStreamBeginCapture(rt->stream, cudaStreamCaptureModeRelaxed);
    if (e != cudaSuccess) return q3_fail_cuda(error, error_len, "q3_attn_graph_begin", e);
    rt->capturing = true;
    rt->capture_used_gather = false;
    rt->capture_launches = rt->n_launch;
    return true;
}

extern "C" q3_attn_graph *q3_attn_graph_end(q3_attn_runtime *rt, char *error,
                                            size_t error_len) {
    q3_clear_error(error, error_len);
    if (!rt || !rt->capturing) {
        q3_fail(error, error_len, "q3_attn_graph_end: not recording");
        return NULL;
    }
    cudaError_t e = cudaSuccess;
    if (rt->capture_used_gather) {
        /* join the side stream back, or the capture has unjoined work */
        cudaEvent_t ev = rt->ev_gather[rt->gather_calls++ % 4];
        e = cudaEventRecord(ev, rt->gather_stream);
        if (e == cudaSuccess) e = cudaStreamWaitEvent(rt->stream, ev, 0);
    }
    cudaGraph_t graph = nullptr;
    cudaError_t e2 = cudaStreamEndCapture(rt->stream, &graph);
    rt->capturing = false;
    if (e == cudaSuccess) e = e2;
    if (e != cudaSuccess || !graph) {
        q3_fail_cuda(error, error_len, "q3_attn_graph_end", e);
        if (graph) cudaGraphDestroy(graph);
        return NULL;
    }
    q3_attn_graph *g = new (std::nothrow) q3_attn_graph();
    if (!g) {
        cudaGraphDestroy(graph);
        q3_fail(error, error_len, "q3_attn_graph_end: allocation failed");
        return NULL;
    }
    g->rt = rt;
    g->graph = graph;
    g->exec = nullptr;
    g->launches = rt->n_launch - rt->capture_launches;
    rt->n_launch = rt->capture_launches;   /* nothing ran while recording */
    e = cudaGraphInstantiate(&g->exec, graph, 0);
    if (e != cudaSuccess) {
        q3_fail_cuda(error, error_len, "q3_attn_graph_end: instantiate", e);
        cudaGraphDestroy(graph);
        delete g;
        return NULL;
    }
    return g;
}

extern "C" bool q3_attn_graph_launch(q3_attn_graph *g, char *error, size_t error_len) {
    q3_clear_error(error, error_len);
    if (!g || !g->exec) return q3_fail(error, error_len, "q3_attn_graph_launch: null graph");
    if (g->rt->capturing)
        return q3_fail(error, error_len, "q3_attn_graph_launch: runtime is recording");
    if (!q3_use_device(g->rt, error, error_len)) return false;
    cudaError_t e = cudaGraphLaunch(g->exec, g->rt->stream);
    if (e != cudaSuccess) return q3_fail_cuda(error, error_len, "q3_attn_graph_launch", e);
    g->rt->n_launch += g->launches;
    return true;
}

extern "C" void q3_attn_graph_destroy(q3_attn_graph *g) {
    if (!g) return;
    if (g->rt && g->rt->stream) cudaStreamSynchronize(g->rt->stream);
    if (g->exec) cudaGraphExecDestroy(g->exec);
    if (g->graph) cudaGraphDestroy(g->graph);
    delete g;
}

/* ---------------------------------------------------------------------- */
/* decode plan                                                             */
/* ---------------------------------------------------------------------- */

extern "C" q3_decode_plan *q3_decode_plan_create(q3_attn_runtime *rt,
                                                 const uint32_t *ctx_lens,
                                                 const uint32_t *page_indptr,
                                                 const uint32_t *page_indices,
                                                 uint32_t num_seqs, char *error,
                                                 size_t error_len) {
    q3_clear_error(error, error_len);
    if (!rt || !ctx_lens || !page_indptr || !page_indices || num_seqs == 0) {
        q3_fail(error, error_len, "q3_decode_plan_create: invalid argument");
        return NULL;
    }
    if (num_seqs > rt->cfg.max_tokens) {
        q3_fail(error, error_len, "q3_decode_plan_create: more sequences than max_tokens");
        return NULL;
    }
    const uint32_t n_idx = page_indptr[num_seqs];
    std::vector<uint32_t> pos(num_seqs), dpage(num_seqs), dslot(num_seqs);
    bool can_append = true;
    for (uint32_t s = 0; s < num_seqs; s++) {
        const uint32_t have = page_indptr[s + 1] - page_indptr[s];
        if (page_indptr[s + 1] < page_indptr[s] ||
            (uint64_t)have * Q3_PAGE < ctx_lens[s] || ctx_lens[s] >= rt->cfg.max_positions) {
            q3_fail(error, error_len, "q3_decode_plan_create: page list shorter than context");
            return NULL;
        }
        pos[s] = ctx_lens[s];
        /* slot for an appended token, when the page list has room for it */
        const uint32_t pi = ctx_lens[s] / Q3_PAGE;
        dpage[s] = pi < have ? page_indices[page_indptr[s] + pi] : Q3_NO_PAGE;
        dslot[s] = ctx_lens[s] % Q3_PAGE;
        if (pi >= have) can_append = false;
    }
    for (uint32_t i = 0; i < n_idx; i++)
        if (page_indices[i] >= rt->cfg.num_pages) {
            q3_fail(error, error_len, "q3_decode_plan_create: page id out of range");
            return NULL;
        }
    q3_decode_plan *plan = new (std::nothrow) q3_decode_plan();
    if (!plan) {
        q3_fail(error, error_len, "q3_decode_plan_create: allocation failed");
        return NULL;
    }
    memset(plan, 0, sizeof(*plan));
    plan->rt = rt;
    plan->num_seqs = num_seqs;
    plan->can_append = can_append;
    plan->has_empty = false;
    for (uint32_t s = 0; s < num_seqs; s++)
        if (ctx_lens[s] == 0) plan->has_empty = true;
    /* Chunks of 64 pages (1024 keys, 256 KiB of K+V per head): long enough to
     * amortise the pipeline fill, short enough to balance ragged contexts. */
    plan->chunk_pages = 64;
    std::vector<q3_decode_work> work;
    std::vector<uint32_t> seq_work_begin;
    q3_build_decode_work(ctx_lens, num_seqs, 1, plan->chunk_pages, work, seq_work_begin);
    plan->n_work = (uint32_t)work.size();

    auto al = [](size_t x) { return (x + 15) & ~(size_t)15; };
    size_t off = 0;
    const size_t o_ctx = off;  off = al(off + num_seqs * 4);
    const size_t o_ptr = off;  off = al(off + (num_seqs + 1) * 4);
    const size_t o_idx = off;  off = al(off + (size_t)n_idx * 4);
    const size_t o_pos = off;  off = al(off + num_seqs * 4);
    const size_t o_dp = off;   off = al(off + num_seqs * 4);
    const size_t o_ds = off;   off = al(off + num_seqs * 4);
    const size_t o_wk = off;   off = al(off + work.size() * sizeof(q3_decode_work));
    const size_t o_swb = off;  off = al(off + (num_seqs + 1) * 4);
    std::vector<uint8_t> host(off);
    memcpy(&host[o_ctx], ctx_lens, num_seqs * 4);
    memcpy(&host[o_ptr], page_indptr, (num_seqs + 1) * 4);
    memcpy(&host[o_idx], page_indices, (size_t)n_idx * 4);
    memcpy(&host[o_pos], pos.data(), num_seqs * 4);
    memcpy(&host[o_dp], dpage.data(), num_seqs * 4);
    memcpy(&host[o_ds], dslot.data(), num_seqs * 4);
    memcpy(&host[o_wk], work.data(), work.size() * sizeof(q3_decode_work));
    memcpy(&host[o_swb], seq_work_begin.data(), (num_seqs + 1) * 4);
    const uint32_t need_slots = plan->n_work * rt->cfg.n_kv_heads;
    bool ok = rt_malloc(rt, &plan->dev, off) == cudaSuccess;
    if (ok && need_slots > rt->dec_slots) {
        cudaStreamSynchronize(rt->stream);
        rt_free(rt, rt->dec_o);
        rt_free(rt, rt->dec_ml);
        rt->dec_o = nullptr;
        rt->dec_ml = nullptr;
        rt->dec_slots = 0;
        ok = rt_malloc(rt, (void **)&rt->dec_o,
                       (size_t)need_slots * Q3_G * Q3_D * sizeof(float)) == cudaSuccess &&
             rt_malloc(rt, (void **)&rt->dec_ml,
                       (size_t)need_slots * Q3_G * sizeof(float2)) == cudaSuccess;
        if (ok) rt->dec_slots = need_slots;
    }
    if (ok)
        ok = cudaMemcpyAsync(plan->dev, host.data(), off, cudaMemcpyHostToDevice,
                             rt->stream) == cudaSuccess &&
             cudaStreamSynchronize(rt->stream) == cudaSuccess; /* plan build is set-up */
    if (!ok) {
        q3_fail(error, error_len, "q3_decode_plan_create: device allocation failed");
        rt_free(rt, plan->dev);
        delete plan;
        return NULL;
    }
    const uint8_t *d = (const uint8_t *)plan->dev;
    plan->ctx_lens = (const uint32_t *)(d + o_ctx);
    plan->page_indptr = (const uint32_t *)(d + o_ptr);
    plan->page_indices = (const uint32_t *)(d + o_idx);
    plan->rope_pos = (const uint32_t *)(d + o_pos);
    plan->dst_page = (const uint32_t *)(d + o_dp);
    plan->dst_slot = (const uint32_t *)(d + o_ds);
    plan->work = (const q3_decode_work *)(d + o_wk);
    plan->seq_work_begin = (const uint32_t *)(d + o_swb);
    return plan;
}

extern "C" void q3_decode_plan_destroy(q3_decode_plan *plan) {
    if (!plan) return;
    if (plan->rt && plan->rt->stream) cudaStreamSynchronize(plan->rt->stream);
    rt_free(plan->rt, plan->dev);
    delete plan;
}

extern "C" bool q3_decode_attention_layer(q3_decode_plan *plan, uint32_t layer,
                                          const void *q, const void *k_new,
                                          const void *v_new, void *out, char *error,
                                          size_t error_len) {
    q3_clear_error(error, error_len);
    if (!plan || !q || !out || ((k_new == NULL) != (v_new == NULL)))
        return q3_fail(error, error_len, "q3_decode_attention_layer: invalid argument");
    q3_attn_runtime *rt = plan->rt;
    if (!q3_use_device(rt, error, error_len)) return false;
    if (layer >= rt->cfg.num_layers)
        return q3_fail(error, error_len, "q3_decode_attention_layer: layer out of range");
    if (!k_new && plan->has_empty)
        return q3_fail(error, error_len,
                       "q3_decode_attention_layer: a sequence has no context and no new token");
    if (k_new && !plan->can_append)
        return q3_fail(error, error_len,
                       "q3_decode_attention_layer: a sequence has no page for the new token");
    if (!q3_launch_kvwrite(rt, layer, q, k_new, v_new, plan->num_seqs, plan->rope_pos,
                           plan->dst_page, plan->dst_slot, rt->q2, error, error_len))
        return false;
    return q3_launch_decode(rt, layer, plan, k_new != NULL, out, error, error_len);
}
