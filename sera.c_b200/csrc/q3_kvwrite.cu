/* q3_kvwrite.cu - fused QK-RMSNorm + RoPE + paged KV write.
 *
 * One launch replaces five steps of the reference's layer drivers
 * (ref: src/q3_forward.cu:1244-1278 and :1489-1516): rms_norm on q, rms_norm
 * on k, rope / rope_positions, and the KV append (two cudaMemcpyAsync) or
 * kv_scatter_kernel. Arithmetic per row is the reference's:
 *   inv = 1/sqrt(mean(x^2) + eps);  x' = x * inv * w            (:117-148)
 *   (a, b) = (x'[d], x'[d+64]);  a' = a c - b s;  b' = a s + b c  (:199-208)
 * with c, s = cos/sin of the fp32 angle (float)pos * inv_freq[d], read from a
 * host-built table so that positions of tens of thousands stay accurate.
 *
 * HBM-bound. Each head row (128 values) is handled by 8 lanes; a lane loads
 * 2 x 16 B (elements 8s..8s+7 and 64+8s..64+8s+7, so both members of every
 * rotary pair sit in the same lane) and stores 2 x 16 B of f16.
 * Algorithmic bytes per token: (64+8+8)*128*2 read + 64*128*2 (q out)
 * + 2*8*128*2 (K,V pages) written = 40,960 B at the full geometry.
 */
#include "q3_internal.h"

namespace {

__device__ __forceinline__ void unpack_bf16x8(const uint4 &u, float *f) {
    const __nv_bfloat162 *p = reinterpret_cast<const __nv_bfloat162 *>(&u);
#pragma unroll
    for (int i = 0; i < 4; i++) {
        const float2 t = __bfloat1622float2(p[i]);
        f[2 * i] = t.x;
        f[2 * i + 1] = t.y;
    }
}

__device__ __forceinline__ uint4 pack_f16x8(const float *f) {
    uint4 u;
    __half2 *p = reinterpret_cast<__half2 *>(&u);
#pragma unroll
    for (int i = 0; i < 4; i++) p[i] = __floats2half2_rn(f[2 * i], f[2 * i + 1]);
    return u;
}

__global__ void __launch_bounds__(256)
qknorm_rope_kvwrite_kernel(const __nv_bfloat16 *__restrict__ q,
                           const __nv_bfloat16 *__restrict__ k,
                           const __nv_bfloat16 *__restrict__ v, uint32_t tokens,
                           uint32_t n_heads, uint32_t n_kv_heads,
                           const float *__restrict__ norm_w /* [2][128] */, float eps,
                           const float2 *__restrict__ rope_table,
                           const uint32_t *__restrict__ rope_pos,
                           const uint32_t *__restrict__ dst_page,
                           const uint32_t *__restrict__ dst_slot,
                           __half *__restrict__ q_out, __half *__restrict__ k_pool_layer,
                           __half *__restrict__ v_pool_layer, uint32_t num_pages,
                           uint32_t q_rows, uint32_t kv_rows) {
    const uint32_t rows_per_token = q_rows + 2 * kv_rows;
    const uint64_t gid = (uint64_t)blockIdx.x * blockDim.x + threadIdx.x;
    const uint32_t sub = (uint32_t)(gid & 7u);
    const uint64_t row = gid >> 3;
    if (row >= (uint64_t)tokens * rows_per_token) return;
    const uint32_t t = (uint32_t)(row / rows_per_token);
    const uint32_t r = (uint32_t)(row % rows_per_token);

    const __nv_bfloat16 *src;
    __half *dst;
    const float *w = nullptr;
    if (r < q_rows) {
        src = q + ((size_t)t * n_heads + r) * Q3_D;
        dst = q_out + ((size_t)t * n_heads + r) * Q3_D;
        w = norm_w;
    } else {
        const uint32_t h = (r - q_rows) % n_kv_heads;
        const bool is_k = (r - q_rows) < kv_rows;
        const uint32_t page = dst_page[t];
        if (page == Q3_NO_PAGE) return;
        const size_t off =
            (((size_t)h * num_pages + page) * Q3_PAGE + dst_slot[t]) * Q3_D;
        src = (is_k ? k : v) + ((size_t)t * n_kv_heads + h) * Q3_D;
        dst = (is_k ? k_pool_layer : v_pool_layer) + off;
        if (is_k) w = norm_w + Q3_D;
    }
    const uint4 lo_raw = *reinterpret_cast<const uint4 *>(src + 8 * sub);
    const uint4 hi_raw = *reinterpret_cast<const uint4 *>(src + 64 + 8 * sub);
    float lo[8], hi[8];
    unpack_bf16x8(lo_raw, lo);
    unpack_bf16x8(hi_raw, hi);
    if (w) {
        float ss = 0.f;
#pragma unroll
        for (int i = 0; i < 8; i++) ss += lo[i] * lo[i] + hi[i] * hi[i];
        /* the 8 lanes of a row take the same path; other rows of the warp may
         * be V rows (no norm) or past the end, so the mask names this row only */
        const unsigned gmask = 0xFFu << (threadIdx.x & 24u);
        ss += __shfl_xor_sync(gmask, ss, 1);
        ss += __shfl_xor_sync(gmask, ss, 2);
        ss += __shfl_xor_sync(gmask, ss, 4);
        const float inv = 1.0f / sqrtf(ss * (1.0f / (float)Q3_D) + eps);
        const float2 *cs = rope_table + (size_t)rope_pos[t] * 64 + 8 * sub;
#pragma unroll
        for (int i = 0; i < 8; i++) {
            const float a = lo[i] * inv * w[8 * sub + i];
            const float b = hi[i] * inv * w[64 + 8 * sub + i];
            const float2 c = cs[i];
            lo[i] = a * c.x - b * c.y;
            hi[i] = a * c.y + b * c.x;
        }
    }
    *reinterpret_cast<uint4 *>(dst + 8 * sub) = pack_f16x8(lo);
    *reinterpret_cast<uint4 *>(dst + 64 + 8 * sub) = pack_f16x8(hi);
}

}  // namespace

bool q3_launch_kvwrite(q3_attn_runtime *rt, uint32_t layer, const void *q,
                       const void *k, const void *v, uint32_t tokens,
                       const uint32_t *rope_pos, const uint32_t *dst_page,
                       const uint32_t *dst_slot, void *q_out, char *error,
                       size_t error_len) {
    const q3_attn_config &c = rt->cfg;
    const uint32_t q_rows = q ? c.n_heads : 0;
    const uint32_t kv_rows = k ? c.n_kv_heads : 0;
    const uint64_t threads = (uint64_t)tokens * (q_rows + 2 * kv_rows) * 8;
    if (threads == 0) return true;
    const size_t layer_off = (size_t)layer * c.n_kv_heads * c.num_pages * Q3_PAGE * Q3_D;
    const unsigned grid = (unsigned)((threads + 255) / 256);
    q3_phase_begin(rt, Q3_PHASE_KVWRITE);
    qknorm_rope_kvwrite_kernel<<<grid, 256, 0, rt->stream>>>(
        (const __nv_bfloat16 *)q, (const __nv_bfloat16 *)k, (const __nv_bfloat16 *)v,
        tokens, c.n_heads, c.n_kv_heads, rt->qk_norm_w + (size_t)layer * 2 * Q3_D,
        c.rms_eps, rt->rope_table, rope_pos, dst_page, dst_slot, (__half *)q_out,
        rt->k_pool + layer_off, rt->v_pool + layer_off, c.num_pages, q_rows, kv_rows);
    q3_phase_end(rt);
    Q3_LAUNCH_CHECK("qknorm_rope_kvwrite launch failed");
    rt->n_launch++;
    return true;
}
