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
 * HBM-bound. Persistent CTAs stream one token's rows at a time into shared
 * memory with bulk async copies, four tokens ahead, so the bytes in flight do
 * not depend on registers or occupancy; eight consumer warps take 8 lanes per
 * row: a lane holds elements 8s..8s+7 and 64+8s..64+8s+7, so both members of
 * every rotary pair sit in the same lane.
 * Algorithmic bytes per token: (64+8+8)*128*2 read + 64*128*2 (q out)
 * + 2*8*128*2 (K,V pages) written = 40,960 B at the full geometry.
 */
#include "q3_internal.h"
#include "q3_ptx.cuh"

#include <algorithm>

namespace {

/* packed fp32 pairs (one issue slot for two lanes of arithmetic): the kernel is
 * bound by instruction issue once its loads are staged through shared memory */
typedef unsigned long long f32x2;
__device__ __forceinline__ f32x2 pk2(float x, float y) {
    f32x2 r;
    asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(x), "f"(y));
    return r;
}
__device__ __forceinline__ void upk2(f32x2 v, float &x, float &y) {
    asm("mov.b64 {%0, %1}, %2;" : "=f"(x), "=f"(y) : "l"(v));
}
__device__ __forceinline__ f32x2 mul2(f32x2 a, f32x2 b) {
    f32x2 d;
    asm("mul.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b));
    return d;
}
__device__ __forceinline__ f32x2 fma2(f32x2 a, f32x2 b, f32x2 c) {
    f32x2 d;
    asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(d) : "l"(a), "l"(b), "l"(c));
    return d;
}
/* 8 bf16 -> 4 packed fp32 pairs (a bf16 is the upper half of an fp32) */
__device__ __forceinline__ void unpack_bf16x8_2(const uint4 &u, f32x2 *f) {
    const uint32_t w[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
    for (int i = 0; i < 4; i++)
        f[i] = pk2(__uint_as_float(w[i] << 16), __uint_as_float(w[i] & 0xFFFF0000u));
}
__device__ __forceinline__ uint4 pack_f16x8_2(const f32x2 *f) {
    uint4 u;
    __half2 *p = reinterpret_cast<__half2 *>(&u);
#pragma unroll
    for (int i = 0; i < 4; i++) {
        float x, y;
        upk2(f[i], x, y);
        p[i] = __floats2half2_rn(x, y);
    }
    return u;
}

constexpr uint32_t kWriteThreads = 288;      /* 8 consumer warps + 1 producer warp */
constexpr uint32_t kWriteStages = 4;

/* Shared memory of one CTA: kWriteStages slots of one token's rows
 * [q rows | k rows | v rows] (bf16, 256 B per row), then the barriers. */
struct WriteBarriers {
    uint64_t full[kWriteStages], empty[kWriteStages];
    uint32_t abort_flag;
};

/* Per-token values a consumer lane needs besides the row data. */
struct TokenInfo {
    f32x2 cosv[4], sinv[4];      /* elements (2i, 2i+1) of this lane's 8 */
    f32x2 nsinv[4];              /* -sin */
    uint32_t page, slot;
};
/* The indices of a token: two dependent loads sit between a token number and
 * its rotary factors, so the first is issued one group ahead. */
struct TokenIndex {
    uint32_t pos, page, slot;
};
__device__ __forceinline__ TokenIndex load_token_index(uint32_t t, bool with_kv,
                                                       const uint32_t *__restrict__ rope_pos,
                                                       const uint32_t *__restrict__ dst_page,
                                                       const uint32_t *__restrict__ dst_slot) {
    TokenIndex ix;
    ix.pos = rope_pos[t];
    ix.page = Q3_NO_PAGE;
    ix.slot = 0;
    if (with_kv) {
        ix.page = dst_page[t];
        ix.slot = dst_slot[t];
    }
    return ix;
}
__device__ __forceinline__ void load_token_factors(TokenInfo &ti, const TokenIndex &ix,
                                                   uint32_t sub,
                                                   const float2 *__restrict__ rope_table) {
    const float4 *c4 =
        reinterpret_cast<const float4 *>(rope_table + (size_t)ix.pos * 64 + 8 * sub);
#pragma unroll
    for (int i = 0; i < 4; i++) {
        const float4 f = c4[i];             /* (cos, sin) of elements 2i and 2i+1 */
        ti.cosv[i] = pk2(f.x, f.z);
        ti.sinv[i] = pk2(f.y, f.w);
        ti.nsinv[i] = pk2(-f.y, -f.w);
    }
    ti.page = ix.page;
    ti.slot = ix.slot;
}
__device__ __forceinline__ void load_token_info(TokenInfo &ti, uint32_t t, uint32_t sub,
                                                bool with_kv,
                                                const float2 *__restrict__ rope_table,
                                                const uint32_t *__restrict__ rope_pos,
                                                const uint32_t *__restrict__ dst_page,
                                                const uint32_t *__restrict__ dst_slot) {
    const float4 *c4 =
        reinterpret_cast<const float4 *>(rope_table + (size_t)rope_pos[t] * 64 + 8 * sub);
#pragma unroll
    for (int i = 0; i < 4; i++) {
        const float4 f = c4[i];             /* (cos, sin) of elements 2i and 2i+1 */
        ti.cosv[i] = pk2(f.x, f.z);
        ti.sinv[i] = pk2(f.y, f.w);
        ti.nsinv[i] = pk2(-f.y, -f.w);
    }
    ti.page = Q3_NO_PAGE;
    ti.slot = 0;
    if (with_kv) {
        ti.page = dst_page[t];
        ti.slot = dst_slot[t];
    }
}

/* Persistent CTAs over groups of `group` consecutive tokens (group * rows per
 * token = at most 80 rows: one token at the full geometry, eight at one local
 * KV head), group g = blockIdx.x, += gridDim.x. The producer warp streams each
 * group's rows into shared memory with bulk async copies (the query rows of
 * consecutive tokens are contiguous), kWriteStages groups ahead, so the bytes
 * in flight do not depend on registers or occupancy; the consumer warps
 * normalise, rotate and store. With one token per group the token's rotary
 * factors are fetched one group ahead. */
__global__ void __launch_bounds__(kWriteThreads, 2)
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
                           uint32_t q_rows, uint32_t kv_rows, uint32_t group,
                           uint32_t *status) {
    extern __shared__ __align__(128) uint8_t wsmem[];
    const uint32_t rows = q_rows + 2 * kv_rows;          /* per token */
    const uint32_t slot_bytes = group * rows * 256u;
    const uint32_t n_groups = (tokens + group - 1) / group;
    WriteBarriers *bar = reinterpret_cast<WriteBarriers *>(wsmem + kWriteStages * slot_bytes);
    const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31u;
    if (threadIdx.x == 0) {
        for (uint32_t s = 0; s < kWriteStages; s++) {
            q3ptx::mbar_init(&bar->full[s], 1);
            q3ptx::mbar_init(&bar->empty[s], 8);     /* one arrival per consumer warp */
        }
        bar->abort_flag = 0;
        q3ptx::fence_mbar_init();
    }
    __syncthreads();

    if (warp == 8) {
        /* ---------------- producer ----------------
         * slot layout: [group x q rows | group x k rows | group x v rows] */
        if (lane == 0) {
            uint32_t n = 0;
            for (uint32_t g = blockIdx.x; g < n_groups; g += gridDim.x, n++) {
                const uint32_t s = n % kWriteStages;
                if (n >= kWriteStages &&
                    !q3ptx::mbar_wait(&bar->empty[s], ((n / kWriteStages) - 1u) & 1u)) {
                    atomicExch(&bar->abort_flag, 1u);
                    break;
                }
                const uint32_t t0 = g * group;
                const uint32_t nt = min(group, tokens - t0);
                uint8_t *dst = wsmem + s * slot_bytes;
                q3ptx::mbar_arrive_expect_tx(&bar->full[s], nt * rows * 256u);
                if (q_rows)
                    q3ptx::bulk_load(dst, q + (size_t)t0 * n_heads * Q3_D, nt * q_rows * 256u,
                                     &bar->full[s]);
                if (kv_rows) {
                    q3ptx::bulk_load(dst + group * q_rows * 256u,
                                     k + (size_t)t0 * n_kv_heads * Q3_D, nt * kv_rows * 256u,
                                     &bar->full[s]);
                    q3ptx::bulk_load(dst + group * (q_rows + kv_rows) * 256u,
                                     v + (size_t)t0 * n_kv_heads * Q3_D, nt * kv_rows * 256u,
                                     &bar->full[s]);
                }
            }
        }
    } else {
        /* ---------------- consumers: 8 lanes per row, 32 rows per pass ------- */
        const uint32_t sub = lane & 7u;
        const uint32_t row_in_pass = warp * 4u + (lane >> 3);
        f32x2 wq_lo[4], wq_hi[4];
        {
            const float4 *w4 = reinterpret_cast<const float4 *>(norm_w);
#pragma unroll
            for (int i = 0; i < 2; i++) {
                const float4 a = w4[2 * sub + i], b = w4[16 + 2 * sub + i];
                wq_lo[2 * i] = pk2(a.x, a.y); wq_lo[2 * i + 1] = pk2(a.z, a.w);
                wq_hi[2 * i] = pk2(b.x, b.y); wq_hi[2 * i + 1] = pk2(b.z, b.w);
            }
        }
        const bool single = group == 1;
        TokenIndex next = {0u, Q3_NO_PAGE, 0u};
        if (single && blockIdx.x < n_groups)
            next = load_token_index(blockIdx.x, kv_rows != 0, rope_pos, dst_page, dst_slot);
        uint32_t n = 0;
        bool alive = true;
        for (uint32_t g = blockIdx.x; g < n_groups && alive; g += gridDim.x, n++) {
            const uint32_t s = n % kWriteStages;
            const uint32_t t0 = g * group;
            const uint32_t nt = min(group, tokens - t0);
            TokenInfo ti;
            if (single) {
                load_token_factors(ti, next, sub, rope_table);   /* lands during the wait below */
                if (g + gridDim.x < n_groups)      /* one group ahead: off the critical path */
                    next = load_token_index(g + gridDim.x, kv_rows != 0, rope_pos, dst_page,
                                            dst_slot);
            }
            alive = q3ptx::mbar_wait(&bar->full[s], (n / kWriteStages) & 1u);
            alive = __all_sync(0xffffffffu, alive);
            if (!alive) {
                if (lane == 0) atomicExch(&bar->abort_flag, 1u);
                break;
            }
            const uint8_t *src = wsmem + s * slot_bytes;
            /* rows of the slot in order: all query rows, all K rows, all V rows */
            const uint32_t slot_rows = group * rows;
            for (uint32_t r0 = 0; r0 < slot_rows; r0 += 32) {
                const uint32_t r = r0 + row_in_pass;
                uint32_t kind, tt, h;           /* kind: 0 q, 1 k, 2 v */
                if (r < group * q_rows) {
                    kind = 0; tt = r / max(q_rows, 1u); h = r - tt * q_rows;
                } else if (r < group * (q_rows + kv_rows)) {
                    const uint32_t x = r - group * q_rows;
                    kind = 1; tt = x / max(kv_rows, 1u); h = x - tt * kv_rows;
                } else {
                    const uint32_t x = r - group * (q_rows + kv_rows);
                    kind = 2; tt = x / max(kv_rows, 1u); h = x - tt * kv_rows;
                }
                const bool have = r < slot_rows && tt < nt;
                uint4 lo_raw = make_uint4(0, 0, 0, 0), hi_raw = make_uint4(0, 0, 0, 0);
                if (have) {
                    lo_raw = *reinterpret_cast<const uint4 *>(src + r * 256u + 16u * sub);
                    hi_raw = *reinterpret_cast<const uint4 *>(src + r * 256u + 128u + 16u * sub);
                    if (!single)
                        load_token_info(ti, t0 + tt, sub, kind != 0, rope_table, rope_pos,
                                        dst_page, dst_slot);
                }
                f32x2 lo[4], hi[4];
                unpack_bf16x8_2(lo_raw, lo);
                unpack_bf16x8_2(hi_raw, hi);
                float ss;
                {
                    f32x2 acc = mul2(lo[0], lo[0]);
#pragma unroll
                    for (int e = 1; e < 4; e++) acc = fma2(lo[e], lo[e], acc);
#pragma unroll
                    for (int e = 0; e < 4; e++) acc = fma2(hi[e], hi[e], acc);
                    float s0, s1;
                    upk2(acc, s0, s1);
                    ss = s0 + s1;
                }
                ss += __shfl_xor_sync(0xffffffffu, ss, 1);
                ss += __shfl_xor_sync(0xffffffffu, ss, 2);
                ss += __shfl_xor_sync(0xffffffffu, ss, 4);
                if (!have) continue;
                if (kind && ti.page == Q3_NO_PAGE) continue;
                if (kind < 2) {
                    const float inv = 1.0f / sqrtf(ss * (1.0f / (float)Q3_D) + eps);
                    const f32x2 inv2 = pk2(inv, inv);
                    f32x2 wl[4], wh[4];
                    if (kind == 1) {      /* K rows are one in ten: weights from L1 */
                        const float4 *w4 = reinterpret_cast<const float4 *>(norm_w + Q3_D);
#pragma unroll
                        for (int i = 0; i < 2; i++) {
                            const float4 a = w4[2 * sub + i], b = w4[16 + 2 * sub + i];
                            wl[2 * i] = pk2(a.x, a.y); wl[2 * i + 1] = pk2(a.z, a.w);
                            wh[2 * i] = pk2(b.x, b.y); wh[2 * i + 1] = pk2(b.z, b.w);
                        }
                    } else {
#pragma unroll
                        for (int i = 0; i < 4; i++) {
                            wl[i] = wq_lo[i];
                            wh[i] = wq_hi[i];
                        }
                    }
#pragma unroll
                    for (int e = 0; e < 4; e++) {
                        /* x' = x * inv * w;  (a, b) -> (a c - b s, a s + b c) */
                        const f32x2 a = mul2(mul2(lo[e], inv2), wl[e]);
                        const f32x2 c = mul2(mul2(hi[e], inv2), wh[e]);
                        lo[e] = fma2(a, ti.cosv[e], mul2(c, ti.nsinv[e]));
                        hi[e] = fma2(a, ti.sinv[e], mul2(c, ti.cosv[e]));
                    }
                }
                __half *dst =
                    kind == 0 ? q_out + ((size_t)(t0 + tt) * n_heads + h) * Q3_D
                              : (kind == 1 ? k_pool_layer : v_pool_layer) +
                                    (((size_t)h * num_pages + ti.page) * Q3_PAGE + ti.slot) * Q3_D;
                *reinterpret_cast<uint4 *>(dst + 8 * sub) = pack_f16x8_2(lo);
                *reinterpret_cast<uint4 *>(dst + 64 + 8 * sub) = pack_f16x8_2(hi);
            }
            __syncwarp();
            if (lane == 0) q3ptx::mbar_arrive(&bar->empty[s]);
        }
    }
    __syncthreads();
    if (threadIdx.x == 0 && bar->abort_flag) atomicOr(status, Q3_STATUS_WAIT_TIMEOUT);
}

}  // namespace

/* Per device, at runtime creation: opt in to the dynamic shared memory of the
 * staging ring (4 tokens x 80 rows x 256 B at the full geometry). */
bool q3_prepare_kvwrite_kernel(char *error, size_t error_len) {
    cudaError_t e = cudaFuncSetAttribute(qknorm_rope_kvwrite_kernel,
                                         cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         (int)(kWriteStages * 80u * 256u + 1024u));
    if (e != cudaSuccess)
        return q3_fail_cuda(error, error_len, "kvwrite: shared memory opt-in", e);
    return true;
}

bool q3_launch_kvwrite(q3_attn_runtime *rt, uint32_t layer, const void *q,
                       const void *k, const void *v, uint32_t tokens,
                       const uint32_t *rope_pos, const uint32_t *dst_page,
                       const uint32_t *dst_slot, void *q_out, char *error,
                       size_t error_len) {
    const q3_attn_config &c = rt->cfg;
    const uint32_t q_rows = q ? c.n_heads : 0;
    const uint32_t kv_rows = k ? c.n_kv_heads : 0;
    if (tokens == 0 || q_rows + kv_rows == 0) return true;
    if ((((uintptr_t)q | (uintptr_t)k | (uintptr_t)v | (uintptr_t)q_out) & 15u) != 0)
        return q3_fail(error, error_len,
                       "qknorm_rope_kvwrite: q, k, v and q_out must be 16-byte aligned");
    if (c.n_kv_heads > 8)
        return q3_fail(error, error_len, "qknorm_rope_kvwrite: more than 8 local KV heads");
    const size_t layer_off = (size_t)layer * c.n_kv_heads * c.num_pages * Q3_PAGE * Q3_D;
    const uint32_t rows = q_rows + 2 * kv_rows;
    const uint32_t group = std::max(1u, 80u / rows);     /* tokens staged together */
    const uint32_t smem = kWriteStages * group * rows * 256u + sizeof(WriteBarriers) + 128u;
    const uint32_t n_groups = (tokens + group - 1) / group;
    const unsigned grid = (unsigned)std::min<uint64_t>(n_groups, 2ull * (uint64_t)rt->num_sms);
    q3_phase_begin(rt, Q3_PHASE_KVWRITE);
    qknorm_rope_kvwrite_kernel<<<grid, kWriteThreads, smem, rt->stream>>>(
        (const __nv_bfloat16 *)q, (const __nv_bfloat16 *)k, (const __nv_bfloat16 *)v,
        tokens, c.n_heads, c.n_kv_heads, rt->qk_norm_w + (size_t)layer * 2 * Q3_D,
        c.rms_eps, rt->rope_table, rope_pos, dst_page, dst_slot, (__half *)q_out,
        rt->k_pool + layer_off, rt->v_pool + layer_off, c.num_pages, q_rows, kv_rows, group,
        rt->status_dev);
    q3_phase_end(rt);
    Q3_LAUNCH_CHECK("qknorm_rope_kvwrite launch failed");
    rt->n_launch++;
    return true;
}
