/* q3_attn_decode.cu - paged decode attention: many independent sequences, one
 * query token each, f16 KV in 16-token pages (the reference's q3_cuda_attention
 * with tokens == 1 over a cache, ref: src/q3_forward.cu:218-290,722-755, on a
 * paged pool).
 *
 * HBM-bound: 8 query rows per KV head against up to 16K keys, 8 FLOP per KV
 * byte. The design is therefore about keeping pages in flight:
 *   - every sequence is cut into chunks of <= 64 pages (split-KV); a CTA owns
 *     one (chunk, KV head) and writes either the final bf16 rows (single
 *     chunk) or fp32 partials + (max, sum) that decode_merge_kernel combines
 *     with log-sum-exp;
 *   - one producer warp streams K and V pages with TMA (128-byte swizzle, two
 *     2 KiB boxes per page per operand) through a 3-stage ring of 4 pages
 *     (32 KiB per stage; two CTAs per SM keep ~128 KiB in flight per SM);
 *   - four consumer warps take one page each: S = Q K^T and O += P V with
 *     mma.sync m16n8k16 (rows 8..15 of the M tile are padding; tensor-core
 *     rate is irrelevant here), ldmatrix reads the swizzled pages without
 *     bank conflicts, online softmax in registers with quad shuffles.
 * Algorithmic bytes: every K and V page of the context once (4 KiB per page
 * per head per operand) + q in + out.
 */
#include "q3_internal.h"
#include "q3_ptx.cuh"

#include <mutex>

using namespace q3ptx;

namespace {

constexpr uint32_t kDecStages = 3;
constexpr uint32_t kDecTilePages = 4;
constexpr uint32_t kDecStageBytes = kDecTilePages * 2 * 4096; /* K + V */
constexpr uint32_t kDecThreads = 160;
constexpr uint32_t kDecSmemRing = kDecStages * kDecStageBytes;
/* The per-warp partials (O + (m,l)) are combined through the ring's first
 * bytes once every page has been consumed, so two CTAs fit in one SM. */
constexpr uint32_t kDecSmemCombine = 4 * 8 * 132 * 4 + 4 * 8 * 8;
static_assert(kDecSmemCombine <= kDecSmemRing, "combine buffer aliases the ring");
constexpr uint32_t kDecSmemTotal = kDecSmemRing + 256 + 1024;

struct DecodeParams {
    const q3_decode_work *work;
    const uint32_t *seq_work_begin;
    const uint32_t *ctx_lens;
    const uint32_t *page_indptr;
    const uint32_t *page_indices;
    const __half *q2;          /* [seqs][n_heads][128] normalised, roped */
    uint32_t n_heads, n_kv_heads, num_pages;
    uint32_t pool_row_base, pool_rows_total;
    uint32_t extra_token;
    float scale_log2;
    uint32_t out_fp32;
    void *out;
    float *part_o;             /* [work*Hkv + h][8][128] */
    float2 *part_ml;           /* [work*Hkv + h][8] */
    uint32_t *status;
};

__device__ __forceinline__ void ldsm_x4(uint32_t addr, uint32_t &r0, uint32_t &r1,
                                        uint32_t &r2, uint32_t &r3) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3)
                 : "r"(addr));
}
__device__ __forceinline__ void ldsm_x4_t(uint32_t addr, uint32_t &r0, uint32_t &r1,
                                          uint32_t &r2, uint32_t &r3) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3)
                 : "r"(addr));
}
__device__ __forceinline__ void mma16816(float *c, uint32_t a0, uint32_t a1, uint32_t a2,
                                         uint32_t a3, uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 "
        "{%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
__device__ __forceinline__ float dec_exp2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

__global__ void __launch_bounds__(kDecThreads, 2)
decode_attention_kernel(const __grid_constant__ CUtensorMap k_map,
                        const __grid_constant__ CUtensorMap v_map, const DecodeParams p) {
    extern __shared__ uint8_t smem_raw[];
    uint8_t *smem = (uint8_t *)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    float *comb_o = reinterpret_cast<float *>(smem);
    float2 *comb_ml = reinterpret_cast<float2 *>(smem + 4 * 8 * 132 * 4);
    uint64_t *full = reinterpret_cast<uint64_t *>(smem + kDecSmemRing);
    uint64_t *empty = full + kDecStages;
    uint32_t *abort_flag = reinterpret_cast<uint32_t *>(empty + kDecStages);

    const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31u;
    const q3_decode_work w = p.work[blockIdx.x];
    const uint32_t h = blockIdx.y;
    const uint32_t n_keys = p.ctx_lens[w.seq] + p.extra_token;
    /* The work list may have been cut for one more key than this call sees
     * (a plan serves calls with and without an appended token): never touch a
     * page that holds no visible key, it may lie past the sequence's list. */
    const uint32_t page_end = min(w.page_end, (n_keys + Q3_PAGE - 1) / Q3_PAGE);
    const uint32_t n_pages = page_end > w.page_begin ? page_end - w.page_begin : 0u;
    const uint32_t n_tiles = (n_pages + kDecTilePages - 1) / kDecTilePages;

    if (threadIdx.x == 0) {
        for (uint32_t s = 0; s < kDecStages; s++) {
            mbar_init(&full[s], 1);
            mbar_init(&empty[s], 4);
        }
        *abort_flag = 0;
        fence_mbar_init();
    }
    __syncthreads();

    if (warp == 4) {
        /* ---------------- producer ---------------- */
        const uint32_t *pages = p.page_indices + p.page_indptr[w.seq] + w.page_begin;
        bool alive = true;
        for (uint32_t t = 0; t < n_tiles && alive; t++) {
            const uint32_t stage = t % kDecStages, ph = (t / kDecStages) & 1u;
            const uint32_t pi = t * kDecTilePages + lane;
            const bool have = lane < kDecTilePages && pi < n_pages;
            const uint32_t page = have ? pages[pi] : 0u;
            for (uint32_t i = 0; i < Q3_WAIT_POLLS; i++) {
                alive = mbar_try_wait(&empty[stage], ph ^ 1u);
                if (alive) break;
            }
            alive = __all_sync(0xffffffffu, alive);
            if (!alive) {
                if (lane == 0) atomicExch(abort_flag, 1u);
                break;
            }
            const uint32_t live = min(kDecTilePages, n_pages - t * kDecTilePages);
            if (lane == 0) mbar_arrive_expect_tx(&full[stage], live * 8192u);
            __syncwarp();
            if (have) {
                const int32_t row = (int32_t)(p.pool_row_base +
                                              (h * p.num_pages + page) * Q3_PAGE);
                uint8_t *kd = smem + stage * kDecStageBytes + lane * 4096u;
                uint8_t *vd = kd + kDecTilePages * 4096u;
                tma_load_2d(kd, &k_map, 0, row, &full[stage]);
                tma_load_2d(kd + 2048, &k_map, 64, row, &full[stage]);
                tma_load_2d(vd, &v_map, 0, row, &full[stage]);
                tma_load_2d(vd + 2048, &v_map, 64, row, &full[stage]);
            }
        }
        __syncthreads(); /* ring drained: consumers reuse it for the combine */
    } else {
        /* ---------------- consumers: warp `warp` takes page `warp` of a tile ---- */
        const uint32_t g = lane >> 2;       /* query head row 0..7 */
        const uint32_t tq = lane & 3u;
        /* A fragments of Q for the 8 k-steps: a0 = (row g, d 16ks+2tq..), a2 = (+8) */
        uint32_t qa0[8], qa2[8];
        {
            const __half *qrow =
                p.q2 + ((size_t)w.seq * p.n_heads + h * Q3_G + g) * Q3_D;
#pragma unroll
            for (uint32_t ks = 0; ks < 8; ks++) {
                qa0[ks] = *reinterpret_cast<const uint32_t *>(qrow + ks * 16 + 2 * tq);
                qa2[ks] = *reinterpret_cast<const uint32_t *>(qrow + ks * 16 + 8 + 2 * tq);
            }
        }
        float o[16][4];
#pragma unroll
        for (uint32_t i = 0; i < 16; i++) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f;
        float m_run = -INFINITY, l_run = 0.f;
        const float c = p.scale_log2;
        /* ldmatrix lane addressing inside a swizzled page half:
         *   K (non-transposed): matrix j = lane/8; key = (j/2)*8 + lane%8; chunk += j&1
         *   V (transposed):     matrix j = lane/8; key = (j&1)*8 + lane%8; chunk += j/2 */
        const uint32_t lm = lane >> 3, lr = lane & 7u;
        const uint32_t k_key = (lm >> 1) * 8 + lr, k_csel = lm & 1u;
        const uint32_t v_key = (lm & 1u) * 8 + lr, v_csel = lm >> 1;
        bool alive = true;
        for (uint32_t t = 0; t < n_tiles && alive; t++) {
            const uint32_t stage = t % kDecStages, ph = (t / kDecStages) & 1u;
            for (uint32_t i = 0; i < Q3_WAIT_POLLS; i++) {
                alive = mbar_try_wait(&full[stage], ph);
                if (alive || ((i & 255u) == 255u && *(volatile uint32_t *)abort_flag)) break;
            }
            alive = __all_sync(0xffffffffu, alive);
            if (!alive) {
                if (lane == 0) atomicExch(abort_flag, 1u);
                break;
            }
            const uint32_t pi = t * kDecTilePages + warp;
            if (pi < n_pages) {
                const uint32_t kbase = smem_u32(smem + stage * kDecStageBytes + warp * 4096u);
                const uint32_t vbase = kbase + kDecTilePages * 4096u;
                /* S = Q K^T for the 16 keys of the page */
                float s0[4] = {0.f, 0.f, 0.f, 0.f}, s1[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
                for (uint32_t ks = 0; ks < 8; ks++) {
                    const uint32_t chunk = (2 * ks + k_csel) & 7u;
                    const uint32_t addr = kbase + (ks >> 2) * 2048u + k_key * 128u +
                                          ((chunk ^ (k_key & 7u)) << 4);
                    uint32_t b0, b1, b2, b3;
                    ldsm_x4(addr, b0, b1, b2, b3);
                    mma16816(s0, qa0[ks], 0u, qa2[ks], 0u, b0, b1);
                    mma16816(s1, qa0[ks], 0u, qa2[ks], 0u, b2, b3);
                }
                /* mask keys past the context, online softmax for row g */
                const uint32_t key0 = (w.page_begin + pi) * Q3_PAGE + 2 * tq;
                if (key0 >= n_keys) s0[0] = -INFINITY;
                if (key0 + 1 >= n_keys) s0[1] = -INFINITY;
                if (key0 + 8 >= n_keys) s1[0] = -INFINITY;
                if (key0 + 9 >= n_keys) s1[1] = -INFINITY;
                float mx = fmaxf(fmaxf(s0[0], s0[1]), fmaxf(s1[0], s1[1]));
                mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
                mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
                const float m_new = fmaxf(m_run, mx);
                const float m_use = m_new == -INFINITY ? 0.f : m_new;
                const float alpha = dec_exp2((m_run - m_use) * c);
                const float neg = -m_use * c;
                const float p00 = dec_exp2(fmaf(s0[0], c, neg));
                const float p01 = dec_exp2(fmaf(s0[1], c, neg));
                const float p10 = dec_exp2(fmaf(s1[0], c, neg));
                const float p11 = dec_exp2(fmaf(s1[1], c, neg));
                l_run = l_run * alpha + (p00 + p01 + p10 + p11);
                m_run = m_new;
                const __half2 pa = __floats2half2_rn(p00, p01);
                const __half2 pb = __floats2half2_rn(p10, p11);
                const uint32_t a0 = *reinterpret_cast<const uint32_t *>(&pa);
                const uint32_t a2 = *reinterpret_cast<const uint32_t *>(&pb);
#pragma unroll
                for (uint32_t nt = 0; nt < 16; nt += 2) {
                    o[nt][0] *= alpha;
                    o[nt][1] *= alpha;
                    o[nt + 1][0] *= alpha;
                    o[nt + 1][1] *= alpha;
                    const uint32_t chunk = (nt + v_csel) & 7u;
                    const uint32_t addr = vbase + (nt >> 3) * 2048u + v_key * 128u +
                                          ((chunk ^ (v_key & 7u)) << 4);
                    uint32_t b0, b1, b2, b3;
                    ldsm_x4_t(addr, b0, b1, b2, b3);
                    mma16816(o[nt], a0, 0u, a2, 0u, b0, b1);
                    mma16816(o[nt + 1], a0, 0u, a2, 0u, b2, b3);
                }
            }
            __syncwarp();
            if (lane == 0) mbar_arrive(&empty[stage]);
        }
        /* per-warp partial -> shared memory (over the drained ring) */
        __syncthreads();
        l_run += __shfl_xor_sync(0xffffffffu, l_run, 1);
        l_run += __shfl_xor_sync(0xffffffffu, l_run, 2);
        float *wo = comb_o + (warp * 8 + g) * 132;
#pragma unroll
        for (uint32_t nt = 0; nt < 16; nt++) {
            wo[nt * 8 + 2 * tq] = o[nt][0];
            wo[nt * 8 + 2 * tq + 1] = o[nt][1];
        }
        if (tq == 0) comb_ml[warp * 8 + g] = make_float2(m_run, l_run);
    }
    __syncthreads();
    if (threadIdx.x == 0 && *abort_flag) atomicOr(p.status, Q3_STATUS_WAIT_TIMEOUT);
    if (threadIdx.x < 128) {
        /* combine the 4 warps: thread = (row, 8 consecutive d) */
        const uint32_t r = threadIdx.x >> 4, d0 = (threadIdx.x & 15u) * 8;
        const float c = p.scale_log2;
        float M = -INFINITY;
#pragma unroll
        for (uint32_t wi = 0; wi < 4; wi++) M = fmaxf(M, comb_ml[wi * 8 + r].x);
        float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
        float den = 0.f;
#pragma unroll
        for (uint32_t wi = 0; wi < 4; wi++) {
            const float2 ml = comb_ml[wi * 8 + r];
            const float wgt = ml.x == -INFINITY ? 0.f : dec_exp2((ml.x - M) * c);
            den += wgt * ml.y;
            const float *src = comb_o + (wi * 8 + r) * 132 + d0;
#pragma unroll
            for (uint32_t i = 0; i < 8; i++) acc[i] += wgt * src[i];
        }
        const bool single = p.seq_work_begin[w.seq + 1] - p.seq_work_begin[w.seq] == 1;
        if (single && p.out_fp32) {
            const float inv = den > 0.f ? 1.0f / den : 0.f;   /* no visible key: zeros */
            float *dst = reinterpret_cast<float *>(p.out) +
                         ((size_t)w.seq * p.n_heads + h * Q3_G + r) * Q3_D + d0;
            *reinterpret_cast<float4 *>(dst) =
                make_float4(acc[0] * inv, acc[1] * inv, acc[2] * inv, acc[3] * inv);
            *reinterpret_cast<float4 *>(dst + 4) =
                make_float4(acc[4] * inv, acc[5] * inv, acc[6] * inv, acc[7] * inv);
        } else if (single) {
            const float inv = den > 0.f ? 1.0f / den : 0.f;
            uint4 u;
            __nv_bfloat162 *hh = reinterpret_cast<__nv_bfloat162 *>(&u);
#pragma unroll
            for (uint32_t i = 0; i < 4; i++)
                hh[i] = __floats2bfloat162_rn(acc[2 * i] * inv, acc[2 * i + 1] * inv);
            *reinterpret_cast<uint4 *>(
                reinterpret_cast<__nv_bfloat16 *>(p.out) +
                ((size_t)w.seq * p.n_heads + h * Q3_G + r) * Q3_D + d0) = u;
        } else {
            /* the partial slot is the work item's index (the merge kernel walks
             * seq_work_begin the same way); a caller-written `slot` field is
             * not trusted with an index into the fixed scratch */
            const size_t slot = (size_t)blockIdx.x * p.n_kv_heads + h;
            float *dst = p.part_o + (slot * 8 + r) * Q3_D + d0;
            *reinterpret_cast<float4 *>(dst) = make_float4(acc[0], acc[1], acc[2], acc[3]);
            *reinterpret_cast<float4 *>(dst + 4) = make_float4(acc[4], acc[5], acc[6], acc[7]);
            if ((threadIdx.x & 15u) == 0)
                p.part_ml[slot * 8 + r] = make_float2(M == -INFINITY ? -INFINITY : M * c, den);
        }
    }
}

/* One warp per (sequence, query head): combine that sequence's chunks. */
__global__ void __launch_bounds__(256)
decode_merge_kernel(const uint32_t *__restrict__ seq_work_begin, uint32_t num_seqs,
                    uint32_t n_heads, uint32_t n_kv_heads,
                    const float *__restrict__ part_o, const float2 *__restrict__ part_ml,
                    uint32_t out_fp32, void *__restrict__ out) {
    const uint32_t gw = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    const uint32_t lane = threadIdx.x & 31u;
    if (gw >= num_seqs * n_heads) return;
    const uint32_t seq = gw / n_heads, head = gw % n_heads;
    const uint32_t wb = seq_work_begin[seq], we = seq_work_begin[seq + 1];
    if (we - wb <= 1) return; /* written directly by the attention kernel */
    const uint32_t h = head / Q3_G, r = head % Q3_G;
    float M = -INFINITY;
    for (uint32_t i = wb; i < we; i++)
        M = fmaxf(M, part_ml[((size_t)i * n_kv_heads + h) * 8 + r].x);
    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
    float den = 0.f;
    for (uint32_t i = wb; i < we; i++) {
        const size_t row = ((size_t)i * n_kv_heads + h) * 8 + r;
        const float2 ml = part_ml[row];
        const float wgt = ml.x == -INFINITY ? 0.f : exp2f(ml.x - M);
        den += wgt * ml.y;
        const float4 o = *reinterpret_cast<const float4 *>(part_o + row * Q3_D + lane * 4);
        acc.x += wgt * o.x;
        acc.y += wgt * o.y;
        acc.z += wgt * o.z;
        acc.w += wgt * o.w;
    }
    const float inv = den > 0.f ? 1.0f / den : 0.f;
    const size_t off = ((size_t)seq * n_heads + head) * Q3_D + lane * 4;
    if (out_fp32) {
        *reinterpret_cast<float4 *>(reinterpret_cast<float *>(out) + off) =
            make_float4(acc.x * inv, acc.y * inv, acc.z * inv, acc.w * inv);
        return;
    }
    __nv_bfloat162 lo = __floats2bfloat162_rn(acc.x * inv, acc.y * inv);
    __nv_bfloat162 hi = __floats2bfloat162_rn(acc.z * inv, acc.w * inv);
    uint2 u;
    u.x = *reinterpret_cast<uint32_t *>(&lo);
    u.y = *reinterpret_cast<uint32_t *>(&hi);
    *reinterpret_cast<uint2 *>(reinterpret_cast<__nv_bfloat16 *>(out) + off) = u;
}

}  // namespace

/* Per device, at runtime creation: opt in to the large dynamic shared memory. */
bool q3_prepare_decode_kernel(char *error, size_t error_len) {
    cudaError_t e = cudaFuncSetAttribute(decode_attention_kernel,
                                         cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         (int)kDecSmemTotal);
    if (e != cudaSuccess)
        return q3_fail_cuda(error, error_len, "decode: shared memory opt-in", e);
    return true;
}

bool q3_launch_decode(q3_attn_runtime *rt, uint32_t layer, const q3_decode_plan *plan,
                      bool with_new_token, void *out_bf16, char *error,
                      size_t error_len) {
    const q3_attn_config &c = rt->cfg;
    DecodeParams p;
    p.work = plan->work;
    p.seq_work_begin = plan->seq_work_begin;
    p.ctx_lens = plan->ctx_lens;
    p.page_indptr = plan->page_indptr;
    p.page_indices = plan->page_indices;
    p.q2 = rt->q2;
    p.n_heads = c.n_heads;
    p.n_kv_heads = c.n_kv_heads;
    p.num_pages = c.num_pages;
    p.pool_row_base = layer * c.n_kv_heads * c.num_pages * Q3_PAGE;
    p.pool_rows_total = c.num_layers * c.n_kv_heads * c.num_pages * Q3_PAGE;
    p.extra_token = with_new_token ? 1u : 0u;
    p.scale_log2 = (1.0f / sqrtf((float)Q3_D)) * 1.4426950408889634f;
    p.out_fp32 = c.out_fp32;
    p.out = out_bf16;
    p.part_o = rt->dec_o;
    p.part_ml = rt->dec_ml;
    p.status = rt->status_dev;
    dim3 grid(plan->n_work, c.n_kv_heads);
    q3_phase_begin(rt, Q3_PHASE_DECODE);
    decode_attention_kernel<<<grid, kDecThreads, kDecSmemTotal, rt->stream>>>(
        rt->k_map, rt->v_map, p);
    q3_phase_end(rt);
    Q3_LAUNCH_CHECK("decode_attention launch failed");
    rt->n_launch++;
    if (plan->n_work > plan->num_seqs) {
        const uint32_t warps = plan->num_seqs * c.n_heads;
        q3_phase_begin(rt, Q3_PHASE_DECODE);
        decode_merge_kernel<<<(warps * 32 + 255) / 256, 256, 0, rt->stream>>>(
            plan->seq_work_begin, plan->num_seqs, c.n_heads, c.n_kv_heads, rt->dec_o,
            rt->dec_ml, c.out_fp32, out_bf16);
        q3_phase_end(rt);
        Q3_LAUNCH_CHECK("decode_merge launch failed");
        rt->n_launch++;
    }
    return true;
}

/* ------------------------------------------------------------------------
 * Allocation-free decode entry point.
 *
 * Some hosts may not allocate device memory at the time they need attention:
 * a serving loop that has handed the whole device heap to its own arena, code
 * running under a memory budget that forbids cudaMalloc after start-up, or a
 * plugin loaded into a process whose allocator must not be re-entered. For
 * them the split-KV partials live in the fixed arrays below instead of a
 * buffer the runtime would allocate. Every GPU that loads this library holds
 * these arrays (about 8.5 MB) until the process exits.
 * ------------------------------------------------------------------------ */
#define Q3_NOALLOC_SLOTS Q3_DECODE_NOALLOC_MAX_SLOTS

static __device__ __align__(256) float q3_noalloc_part_o[(size_t)Q3_NOALLOC_SLOTS * Q3_G * Q3_D];
static __device__ __align__(256) float2 q3_noalloc_part_ml[(size_t)Q3_NOALLOC_SLOTS * Q3_G];
static __device__ __align__(256) uint32_t q3_noalloc_status[64];

namespace {
struct NoallocDevice {
    bool ready;
    float *part_o;
    float2 *part_ml;
    uint32_t *status;
};
NoallocDevice g_noalloc[64];
std::mutex g_noalloc_mutex;   /* first-call set-up may race between host threads */

/* Looks up the scratch addresses of the current device once. */
bool noalloc_device(NoallocDevice **out, const char *who, char *error, size_t error_len) {
    int dev = -1;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) {
        if (error && error_len) snprintf(error, error_len, "%s: no current device", who);
        return false;
    }
    std::lock_guard<std::mutex> lock(g_noalloc_mutex);
    NoallocDevice &nd = g_noalloc[dev];
    if (!nd.ready) {
        /* The array names are host-side stand-ins, not device addresses; ask the
         * runtime for the addresses once, with this device current. */
        cudaError_t e = cudaGetSymbolAddress((void **)&nd.part_o, q3_noalloc_part_o);
        if (e == cudaSuccess)
            e = cudaGetSymbolAddress((void **)&nd.part_ml, q3_noalloc_part_ml);
        if (e == cudaSuccess)
            e = cudaGetSymbolAddress((void **)&nd.status, q3_noalloc_status);
        if (e == cudaSuccess)
            e = cudaFuncSetAttribute(decode_attention_kernel,
                                     cudaFuncAttributeMaxDynamicSharedMemorySize,
                                     (int)kDecSmemTotal);
        if (e != cudaSuccess) {
            if (error && error_len)
                snprintf(error, error_len, "%s: device set-up: %s", who, cudaGetErrorString(e));
            return false;
        }
        nd.ready = true;
    }
    *out = &nd;
    return true;
}
}  // namespace

static_assert(sizeof(q3_decode_work_item) == sizeof(q3_decode_work),
              "public and internal work items must have one layout");

extern "C" int64_t q3_decode_work_host(const uint32_t *ctx_lens, uint32_t num_seqs,
                                       q3_decode_work_item *work_out, uint32_t max_work,
                                       uint32_t *seq_work_begin_out, char *error,
                                       size_t error_len) {
    q3_clear_error(error, error_len);
    if (!ctx_lens || !work_out || !seq_work_begin_out || num_seqs == 0) {
        q3_fail(error, error_len, "q3_decode_work_host: invalid argument");
        return -1;
    }
    for (uint32_t s = 0; s < num_seqs; s++)
        if (ctx_lens[s] == 0) {
            q3_fail(error, error_len, "q3_decode_work_host: a sequence has no context");
            return -1;
        }
    std::vector<q3_decode_work> work;
    std::vector<uint32_t> swb;
    q3_build_decode_work(ctx_lens, num_seqs, 0, 64, work, swb);
    if (work.size() > max_work) {
        q3_fail(error, error_len, "q3_decode_work_host: work list does not fit");
        return -1;
    }
    memcpy(work_out, work.data(), work.size() * sizeof(q3_decode_work));
    memcpy(seq_work_begin_out, swb.data(), swb.size() * sizeof(uint32_t));
    return (int64_t)work.size();
}

extern "C" bool q3_cuda_attention_decode_noalloc(
    const void *q_f16, const void *k_pages, const void *v_pages, uint32_t num_pages,
    const uint32_t *ctx_lens, const uint32_t *page_indptr, const uint32_t *page_indices,
    const q3_decode_work_item *work, uint32_t n_work, const uint32_t *seq_work_begin,
    uint32_t num_seqs, uint32_t n_heads, uint32_t n_kv_heads, void *out_bf16,
    void *stream, char *error, size_t error_len) {
    q3_clear_error(error, error_len);
    if (!q_f16 || !k_pages || !v_pages || !ctx_lens || !page_indptr || !page_indices ||
        !work || !seq_work_begin || !out_bf16 || num_seqs == 0 || n_work < num_seqs ||
        num_pages == 0 || n_kv_heads == 0 || n_heads != n_kv_heads * Q3_G)
        return q3_fail(error, error_len, "q3_cuda_attention_decode_noalloc: invalid argument");
    if ((uint64_t)n_work * n_kv_heads > Q3_NOALLOC_SLOTS) {
        if (error && error_len)
            snprintf(error, error_len,
                     "q3_cuda_attention_decode_noalloc: %u work items x %u KV heads exceed the "
                     "fixed scratch of %u slots",
                     n_work, n_kv_heads, (unsigned)Q3_NOALLOC_SLOTS);
        return false;
    }
    const uint64_t rows = (uint64_t)n_kv_heads * num_pages * Q3_PAGE;
    if (rows >= (1ull << 31))
        return q3_fail(error, error_len, "q3_cuda_attention_decode_noalloc: pool too large");
    NoallocDevice *ndp = nullptr;
    if (!noalloc_device(&ndp, "q3_cuda_attention_decode_noalloc", error, error_len)) return false;
    NoallocDevice &nd = *ndp;
    CUtensorMap k_map, v_map;   /* host-side encoding, no device memory involved */
    if (!q3_encode_tmap_2d(&k_map, k_pages, Q3_D, rows, 64, Q3_PAGE, error, error_len) ||
        !q3_encode_tmap_2d(&v_map, v_pages, Q3_D, rows, 64, Q3_PAGE, error, error_len))
        return false;
    DecodeParams p;
    p.work = reinterpret_cast<const q3_decode_work *>(work);
    p.seq_work_begin = seq_work_begin;
    p.ctx_lens = ctx_lens;
    p.page_indptr = page_indptr;
    p.page_indices = page_indices;
    p.q2 = (const __half *)q_f16;
    p.n_heads = n_heads;
    p.n_kv_heads = n_kv_heads;
    p.num_pages = num_pages;
    p.pool_row_base = 0;
    p.pool_rows_total = (uint32_t)rows;
    p.extra_token = 0;
    p.scale_log2 = (1.0f / sqrtf((float)Q3_D)) * 1.4426950408889634f;
    p.out_fp32 = 0;
    p.out = out_bf16;
    p.part_o = nd.part_o;
    p.part_ml = nd.part_ml;
    p.status = nd.status;
    dim3 grid(n_work, n_kv_heads);
    decode_attention_kernel<<<grid, kDecThreads, kDecSmemTotal, (cudaStream_t)stream>>>(
        k_map, v_map, p);
    Q3_LAUNCH_CHECK("q3_cuda_attention_decode_noalloc: launch failed");
    if (n_work > num_seqs) {
        const uint32_t warps = num_seqs * n_heads;
        decode_merge_kernel<<<(warps * 32 + 255) / 256, 256, 0, (cudaStream_t)stream>>>(
            seq_work_begin, num_seqs, n_heads, n_kv_heads, nd.part_o, nd.part_ml, 0u,
            out_bf16);
        Q3_LAUNCH_CHECK("q3_cuda_attention_decode_noalloc: merge launch failed");
    }
    return true;
}

extern "C" bool q3_cuda_attention_decode_noalloc_status(uint32_t *status_out, void *stream,
                                                        char *error, size_t error_len) {
    q3_clear_error(error, error_len);
    if (!status_out)
        return q3_fail(error, error_len,
                       "q3_cuda_attention_decode_noalloc_status: invalid argument");
    NoallocDevice *nd = nullptr;
    if (!noalloc_device(&nd, "q3_cuda_attention_decode_noalloc_status", error, error_len))
        return false;
    cudaStream_t st = (cudaStream_t)stream;
    cudaError_t e = cudaMemcpyAsync(status_out, nd->status, sizeof(uint32_t),
                                    cudaMemcpyDeviceToHost, st);
    if (e == cudaSuccess) e = cudaMemsetAsync(nd->status, 0, sizeof(uint32_t), st);
    if (e == cudaSuccess) e = cudaStreamSynchronize(st);
    if (e != cudaSuccess)
        return q3_fail_cuda(error, error_len, "q3_cuda_attention_decode_noalloc_status", e);
    return true;
}
