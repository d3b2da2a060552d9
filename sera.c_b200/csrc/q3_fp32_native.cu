/* q3_fp32_native.cu - the reference's fp32 attention entry points
 * (q3_cuda_attention, q3_cuda_attention_segmented; ref: src/q3_forward.h:188-192,
 * 262-272) routed through the tensor-core kernel, so that a caller that keeps
 * the reference's fp32 slab layout and links against this library unchanged
 * gets the fast path.
 *
 * Opt-in: q3_cuda_attention_native_init reserves, once, a hidden one-layer
 * attention runtime (f16 page pool, query workspace, schedule staging). A call
 * then (1) converts q to f16 and the visible K/V slab rows to f16 pages of
 * that pool, (2) builds and stages the launch schedule on the host, (3) runs
 * attention_tc_kernel with fp32 output straight into the caller's buffer -
 * all on the caller's stream, without synchronising. Calls that do not fit
 * (other geometry or scale, capacity, descriptors that the host cannot read)
 * fall through to the exact fp32 SIMT kernels of q3_compat_fp32.cu.
 * Operands are rounded to f16 on this path: results agree with the fp32
 * kernels to about 1e-3, not 1e-4.
 */
#include "q3_internal.h"

#include <math.h>

#include <algorithm>
#include <new>

namespace {

struct NativeCtx {
    q3_attn_runtime *rt;
    q3_stage *stage;
    cudaStream_t own_stream;
    uint32_t max_kv_tokens;
};
NativeCtx g_ctx[64];
const char *g_last_path = "simt";

__global__ void __launch_bounds__(256)
f32_to_f16_kernel(const float4 *__restrict__ src, uint2 *__restrict__ dst, size_t n4) {
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n4) return;
    const float4 f = src[i];
    const __half2 a = __floats2half2_rn(f.x, f.y), b = __floats2half2_rn(f.z, f.w);
    dst[i] = make_uint2(*reinterpret_cast<const uint32_t *>(&a),
                        *reinterpret_cast<const uint32_t *>(&b));
}

/* One block per (row, list entry): rows [0, rows[i]) of the slab of entry i
 * go to pages first_page + ids[i] * ppb + row / 16 of every KV head; the
 * remaining slots of the entry's pages are zeroed (they are multiplied by a
 * probability of exactly 0 and must be finite). */
__global__ void __launch_bounds__(256)
slab_rows_to_pages_kernel(const float *__restrict__ k_slab, const float *__restrict__ v_slab,
                          size_t entry_stride, const uint32_t *__restrict__ ids,
                          const uint32_t *__restrict__ rows, uint32_t first_page,
                          uint32_t ppb, __half *__restrict__ k_pool,
                          __half *__restrict__ v_pool, uint32_t n_kv, uint32_t num_pages) {
    const uint32_t r = blockIdx.x, i = blockIdx.y;
    const uint32_t id = ids ? ids[i] : 0u;
    const bool live = r < (rows ? rows[i] : 0xFFFFFFFFu);
    const size_t src_off = (size_t)id * entry_stride + (size_t)r * n_kv * Q3_D;
    for (uint32_t e = threadIdx.x * 4; e < n_kv * Q3_D; e += blockDim.x * 4) {
        const uint32_t h = e / Q3_D, d = e % Q3_D;
        float4 kf = make_float4(0.f, 0.f, 0.f, 0.f), vf = kf;
        if (live) {
            kf = *reinterpret_cast<const float4 *>(k_slab + src_off + e);
            vf = *reinterpret_cast<const float4 *>(v_slab + src_off + e);
        }
        const size_t dst = (((size_t)h * num_pages + first_page + id * ppb + r / Q3_PAGE) *
                                Q3_PAGE + r % Q3_PAGE) * Q3_D + d;
        const __half2 k0 = __floats2half2_rn(kf.x, kf.y), k1 = __floats2half2_rn(kf.z, kf.w);
        const __half2 v0 = __floats2half2_rn(vf.x, vf.y), v1 = __floats2half2_rn(vf.z, vf.w);
        *reinterpret_cast<uint2 *>(k_pool + dst) =
            make_uint2(*reinterpret_cast<const uint32_t *>(&k0),
                       *reinterpret_cast<const uint32_t *>(&k1));
        *reinterpret_cast<uint2 *>(v_pool + dst) =
            make_uint2(*reinterpret_cast<const uint32_t *>(&v0),
                       *reinterpret_cast<const uint32_t *>(&v1));
    }
}

/* Can the host dereference this pointer? (pageable, pinned or managed memory) */
bool host_readable(const void *p) {
    cudaPointerAttributes a;
    if (cudaPointerGetAttributes(&a, p) != cudaSuccess) {
        cudaGetLastError();
        return false;
    }
    return a.type == cudaMemoryTypeUnregistered || a.type == cudaMemoryTypeHost ||
           a.type == cudaMemoryTypeManaged;
}

NativeCtx *current_ctx(uint32_t n_heads, uint32_t n_kv_heads, uint32_t head_dim, float scale,
                       uint32_t tokens) {
    int dev = -1;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return nullptr;
    NativeCtx *c = &g_ctx[dev];
    if (!c->rt) return nullptr;
    const q3_attn_config &cfg = c->rt->cfg;
    if (head_dim != Q3_D || n_heads != cfg.n_heads || n_kv_heads != cfg.n_kv_heads ||
        tokens > cfg.max_tokens)
        return nullptr;
    const float want = 1.0f / sqrtf((float)Q3_D);
    if (fabsf(scale - want) > 1e-6f * want) return nullptr;
    return c;
}

bool convert_q(NativeCtx *c, const float *q, uint32_t tokens, cudaStream_t st, char *error,
               size_t error_len) {
    const size_t n4 = (size_t)tokens * c->rt->cfg.n_heads * Q3_D / 4;
    f32_to_f16_kernel<<<(unsigned)((n4 + 255) / 256), 256, 0, st>>>(
        reinterpret_cast<const float4 *>(q), reinterpret_cast<uint2 *>(c->rt->q2), n4);
    Q3_LAUNCH_CHECK("q3_cuda_attention: query conversion launch failed");
    return true;
}

}  // namespace

extern "C" bool q3_cuda_attention_native_init(int device, uint32_t max_tokens,
                                              uint32_t max_kv_tokens, uint32_t n_heads,
                                              uint32_t n_kv_heads, char *error,
                                              size_t error_len) {
    q3_clear_error(error, error_len);
    if (device < 0 || device >= 64 || max_tokens == 0 || max_kv_tokens == 0)
        return q3_fail(error, error_len, "q3_cuda_attention_native_init: invalid argument");
    NativeCtx *c = &g_ctx[device];
    if (c->rt) return q3_fail(error, error_len,
                              "q3_cuda_attention_native_init: already initialised");
    q3_attn_config cfg;
    memset(&cfg, 0, sizeof(cfg));
    cfg.num_layers = 1;
    cfg.n_heads = n_heads;
    cfg.n_kv_heads = n_kv_heads;
    cfg.head_dim = Q3_D;
    cfg.rms_eps = 1e-6f;
    cfg.rope_theta = 1e6;
    cfg.max_positions = 1;          /* norm and rope are the caller's own fp32 calls */
    cfg.max_tokens = max_tokens;
    /* every branch may start a page of its own: one spare page per 16 rows */
    cfg.num_pages = (max_kv_tokens + Q3_PAGE - 1) / Q3_PAGE + Q3_PACK_MAX_BRANCHES;
    cfg.out_fp32 = 1;
    cfg.device = device;
    c->rt = q3_attn_create(&cfg, error, error_len);
    if (!c->rt) return false;
    c->stage = q3_stage_create(c->rt, error, error_len);
    if (!c->stage) {
        q3_attn_destroy(c->rt);
        c->rt = nullptr;
        return false;
    }
    c->own_stream = c->rt->stream;
    c->max_kv_tokens = max_kv_tokens;
    return true;
}

extern "C" void q3_cuda_attention_native_shutdown(int device) {
    if (device < 0 || device >= 64 || !g_ctx[device].rt) return;
    NativeCtx *c = &g_ctx[device];
    cudaDeviceSynchronize();
    c->rt->stream = c->own_stream;
    q3_stage_destroy(c->stage);
    q3_attn_destroy(c->rt);
    c->rt = nullptr;
    c->stage = nullptr;
}

extern "C" const char *q3_cuda_attention_last_path(void) { return g_last_path; }

extern "C" bool q3_cuda_attention_native_synchronize(int device, char *error,
                                                     size_t error_len) {
    q3_clear_error(error, error_len);
    if (device < 0 || device >= 64 || !g_ctx[device].rt)
        return q3_fail(error, error_len,
                       "q3_cuda_attention_native_synchronize: not initialised");
    return q3_attn_synchronize(g_ctx[device].rt, error, error_len);
}

/* Returns true when the call was taken (*ok tells how it went); false = not
 * applicable, the caller runs its fp32 kernel. */
bool q3_fp32_native_attention(const float *q, const float *k_src, const float *v_src,
                              uint32_t tokens, uint32_t n_heads, uint32_t n_kv_heads,
                              uint32_t head_dim, uint32_t position_base, uint32_t kv_length,
                              float scale, float *out, void *stream, bool *ok, char *error,
                              size_t error_len) {
    g_last_path = "simt";
    NativeCtx *c = current_ctx(n_heads, n_kv_heads, head_dim, scale, tokens);
    const uint32_t visible = position_base + tokens;     /* keys the last row sees */
    if (!c || visible > kv_length || visible > c->max_kv_tokens) return false;
    q3_attn_runtime *rt = c->rt;
    cudaStream_t st = (cudaStream_t)stream;
    rt->stream = st;
    *ok = false;
    const uint32_t n_pages = (visible + Q3_PAGE - 1) / Q3_PAGE;
    std::vector<uint32_t> tag(tokens, 0u), lp(tokens), table(n_pages), none;
    for (uint32_t t = 0; t < tokens; t++) lp[t] = position_base + t;
    for (uint32_t i = 0; i < n_pages; i++) table[i] = i;
    std::vector<uint32_t> ids(1, 0u), rows(1, visible);
    q3_schedule s;
    if (!q3_build_schedule(s, tokens, n_kv_heads, 0, none, tag.data(), lp.data(), table, n_pages,
                           (uint32_t)rt->num_sms, rt->part_slots, false, error, error_len) ||
        !q3_stage_upload(c->stage, s, ids, rows, none, error, error_len))
        return true;
    if (!convert_q(c, q, tokens, st, error, error_len)) return true;
    slab_rows_to_pages_kernel<<<dim3(n_pages * Q3_PAGE, 1), 256, 0, st>>>(
        k_src, v_src, 0, c->stage->rope_pos, c->stage->dst_page, 0, n_pages, rt->k_pool,
        rt->v_pool, n_kv_heads, rt->cfg.num_pages);
    if (cudaGetLastError() != cudaSuccess) {
        q3_fail(error, error_len, "q3_cuda_attention: KV conversion launch failed");
        return true;
    }
    *ok = q3_launch_attention(rt, 0, c->stage, out, error, error_len);
    if (*ok) g_last_path = "tensor-core";
    return true;
}

bool q3_fp32_native_segmented(const float *q, const float *prefix_k, const float *prefix_v,
                              uint32_t prefix_len, const float *suffix_k,
                              const float *suffix_v, uint32_t suffix_capacity,
                              uint32_t suffix_num_layers, uint32_t suffix_layer,
                              const uint32_t *token_branch, const uint32_t *token_local_pos,
                              uint32_t tokens, uint32_t n_heads, uint32_t n_kv_heads,
                              uint32_t head_dim, float scale, float *out, void *stream,
                              bool *ok, char *error, size_t error_len) {
    g_last_path = "simt";
    NativeCtx *c = current_ctx(n_heads, n_kv_heads, head_dim, scale, tokens);
    /* the schedule is built on the host: the descriptors must be readable here
     * (the reference's own caller keeps them in host memory) */
    if (!c || !host_readable(token_branch) || !host_readable(token_local_pos)) return false;
    q3_attn_runtime *rt = c->rt;
    uint32_t n_tags = 0, max_rows = 0;
    for (uint32_t t = 0; t < tokens; t++) {
        n_tags = std::max(n_tags, token_branch[t] + 1);
        max_rows = std::max(max_rows, token_local_pos[t] + 1);
    }
    if (n_tags > Q3_PACK_MAX_BRANCHES || max_rows > suffix_capacity) return false;
    const uint32_t npp = (prefix_len + Q3_PAGE - 1) / Q3_PAGE;
    const uint32_t ppb = (max_rows + Q3_PAGE - 1) / Q3_PAGE;
    if ((uint64_t)npp + (uint64_t)n_tags * ppb > rt->cfg.num_pages) return false;
    cudaStream_t st = (cudaStream_t)stream;
    rt->stream = st;
    *ok = false;
    std::vector<uint32_t> shared(npp), table((size_t)n_tags * ppb), none;
    for (uint32_t i = 0; i < npp; i++) shared[i] = i;
    for (size_t i = 0; i < table.size(); i++) table[i] = npp + (uint32_t)i;
    /* rows to convert per branch present: 0 .. its largest local position */
    std::vector<uint32_t> used(n_tags, 0u), ids(1, 0u), rows(1, prefix_len);   /* [0]: prefix */
    for (uint32_t t = 0; t < tokens; t++)
        used[token_branch[t]] = std::max(used[token_branch[t]], token_local_pos[t] + 1);
    for (uint32_t b = 0; b < n_tags; b++)
        if (used[b]) {
            ids.push_back(b);
            rows.push_back(used[b]);
        }
    q3_schedule s;
    if (!q3_build_schedule(s, tokens, n_kv_heads, prefix_len, shared, token_branch,
                           token_local_pos, table, ppb, (uint32_t)rt->num_sms, rt->part_slots,
                           (uint64_t)npp * 2 * 4096 * n_kv_heads > (48ull << 20), error,
                           error_len) ||
        !q3_stage_upload(c->stage, s, ids, rows, none, error, error_len))
        return true;
    if (!convert_q(c, q, tokens, st, error, error_len)) return true;
    const size_t row = (size_t)n_kv_heads * Q3_D;
    if (npp)
        slab_rows_to_pages_kernel<<<dim3(npp * Q3_PAGE, 1), 256, 0, st>>>(
            prefix_k, prefix_v, 0, c->stage->rope_pos, c->stage->dst_page, 0, npp, rt->k_pool,
            rt->v_pool, n_kv_heads, rt->cfg.num_pages);
    /* suffix: branch b, layer `suffix_layer`: rows at ((b * L + layer) * capacity) * row */
    slab_rows_to_pages_kernel<<<dim3(ppb * Q3_PAGE, (unsigned)ids.size() - 1), 256, 0, st>>>(
        suffix_k + (size_t)suffix_layer * suffix_capacity * row,
        suffix_v + (size_t)suffix_layer * suffix_capacity * row,
        (size_t)suffix_num_layers * suffix_capacity * row, c->stage->rope_pos + 1,
        c->stage->dst_page + 1, npp, ppb, rt->k_pool, rt->v_pool, n_kv_heads,
        rt->cfg.num_pages);
    if (cudaGetLastError() != cudaSuccess) {
        q3_fail(error, error_len, "q3_cuda_attention_segmented: KV conversion launch failed");
        return true;
    }
    *ok = q3_launch_attention(rt, 0, c->stage, out, error, error_len);
    if (*ok) g_last_path = "tensor-core";
    return true;
}
