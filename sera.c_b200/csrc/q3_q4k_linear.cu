/* q3_q4k_linear.cu - resident Q4_K weight x activation on the sm_100a tensor
 * cores (tcgen05, accumulators in tensor memory).
 *
 *   out[token][feature] = sum_k W[feature][k] * x[token][k]
 *
 * W stays in its 144-byte Q4_K blocks in HBM (ref: src/q3_quant.h:24-33). A CTA
 * owns a tile of MT*128 tokens x 128 features and walks K in steps of 64:
 *
 *   warp 0      TMA producer of the activation tiles (f16, 128-byte swizzle)
 *   warp 1      allocates tensor memory, issues tcgen05.mma (one thread)
 *   warp 2      TMA producer of the raw weight bytes: per 256 k one box of
 *               128 rows x 144 bytes (one Q4_K block per feature row)
 *   warps 4..   dequantise, one group of 4 warps per operand stage: thread =
 *               feature row; per k-step 64 quants -> 64 f16 written straight
 *               into the swizzled K-major operand layout the MMA reads;
 *               afterwards two of the groups drain the accumulators
 *
 * A k-step of 64 is exactly one 32-byte group of a block: its low nibbles are
 * elements 0..31, its high nibbles elements 32..63 (ref: src/q3_quant.c:57-76),
 * each half with its own 6-bit scale and min (ref: src/q3_quant.c:44-55).
 * Operand rounding: scale = f16(d*sc), offset = f16(dmin*m), element =
 * f16(fma(q, scale, -offset)); activations are f16; accumulation is fp32.
 *
 * Every wait is bounded: on expiry the CTA raises its abort flag, all roles
 * drain, the status word gets bit 0 and tensor memory is released.
 */
#include <cuda.h>
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdio.h>
#include <string.h>

#include "q3_internal.h"
#include "q3_ptx.cuh"
#include "q3_q4_linear.h"

namespace {
using namespace q3ptx;

constexpr uint32_t kTileBytes = 128 * 64 * 2;      /* one 128 x 64 f16 operand tile */
constexpr uint32_t kRawRowBytes = Q3_QUANT_Q4_K_BLOCK_BYTES;
constexpr uint32_t kRawBytes = 128 * kRawRowBytes; /* 128 feature rows, one block each */
constexpr uint32_t kRawStages = 2;
constexpr uint32_t kMaxStages = 6;

template <uint32_t MT>
struct Layout {
    /* activation ring: deep enough to cover the TMA latency; weight-operand
     * ring: one stage per dequantising warp group */
    static constexpr uint32_t kXStages = MT == 1 ? 6u : 4u;
    static constexpr uint32_t kBStages = 3u;
    static constexpr uint32_t kDequantThreads = 128u * kBStages;
    static constexpr uint32_t kThreads = 128u + kDequantThreads;
    static constexpr uint32_t kX = 0;
    static constexpr uint32_t kB = kX + kXStages * MT * kTileBytes;
    static constexpr uint32_t kRaw = kB + kBStages * kTileBytes;
    static constexpr uint32_t kMisc = kRaw + kRawStages * kRawBytes;
    static constexpr uint32_t kTotal = kMisc + 256 + 1024; /* + alignment slack */
    static constexpr uint32_t kTmemCols = MT * 128;
};

struct Misc {
    uint64_t raw_full[kRawStages], raw_empty[kRawStages];
    uint64_t x_full[kMaxStages], x_empty[kMaxStages];
    uint64_t b_full[kMaxStages], b_empty[kMaxStages];
    uint64_t acc_full;
    uint32_t tmem_base;
    uint32_t abort_flag;
};
static_assert(sizeof(Misc) <= 256, "Misc must fit its slot");

struct LinearParams {
    void *out;
    uint32_t M, N, K;
    uint32_t out_type;
    uint32_t *status;
};

__device__ __forceinline__ bool wait_or_abort(uint64_t *bar, uint32_t parity, Misc *misc) {
    for (uint32_t i = 0; i < Q3_WAIT_POLLS; i++) {
        if (mbar_try_wait(bar, parity)) return true;
        if ((i & 255u) == 255u && *(volatile uint32_t *)&misc->abort_flag) return false;
    }
    atomicExch(&misc->abort_flag, 1u);
    return false;
}

/* `pair` holds two quant bytes in its 16-bit lanes (bits 0-7 of each lane).
 * Low nibbles: 0x6400 | q is the f16 1024 + q. High nibbles: 0x5400 | (q << 4)
 * is the f16 64 + q (one ulp there is 1/16). Subtracting the bias is exact;
 * the result is f16(fma(q, scale, -offset)) for both lanes. */
__device__ __forceinline__ uint32_t dequant_lo(uint32_t pair, __half2 scale,
                                               __half2 neg_offset) {
    uint32_t b = (pair & 0x000F000Fu) | 0x64006400u;
    const __half2 bias = __half2half2(__ushort_as_half((unsigned short)0x6400));
    __half2 h = __hfma2(__hsub2(*reinterpret_cast<__half2 *>(&b), bias), scale, neg_offset);
    return *reinterpret_cast<uint32_t *>(&h);
}
__device__ __forceinline__ uint32_t dequant_hi(uint32_t pair, __half2 scale,
                                               __half2 neg_offset) {
    uint32_t b = (pair & 0x00F000F0u) | 0x54005400u;
    const __half2 bias = __half2half2(__ushort_as_half((unsigned short)0x5400));
    __half2 h = __hfma2(__hsub2(*reinterpret_cast<__half2 *>(&b), bias), scale, neg_offset);
    return *reinterpret_cast<uint32_t *>(&h);
}

__device__ __forceinline__ void store_out32(const LinearParams &p, size_t off,
                                            const uint32_t *v) {
    const float *f = reinterpret_cast<const float *>(v);
    if (p.out_type == Q3_OUT_F32) {
        float4 *dst = reinterpret_cast<float4 *>(static_cast<float *>(p.out) + off);
#pragma unroll
        for (uint32_t i = 0; i < 8; i++)
            dst[i] = make_float4(f[4 * i], f[4 * i + 1], f[4 * i + 2], f[4 * i + 3]);
    } else if (p.out_type == Q3_OUT_BF16) {
        uint4 *dst = reinterpret_cast<uint4 *>(static_cast<__nv_bfloat16 *>(p.out) + off);
#pragma unroll
        for (uint32_t i = 0; i < 4; i++) {
            __nv_bfloat162 a = __floats2bfloat162_rn(f[8 * i], f[8 * i + 1]);
            __nv_bfloat162 b = __floats2bfloat162_rn(f[8 * i + 2], f[8 * i + 3]);
            __nv_bfloat162 c = __floats2bfloat162_rn(f[8 * i + 4], f[8 * i + 5]);
            __nv_bfloat162 d = __floats2bfloat162_rn(f[8 * i + 6], f[8 * i + 7]);
            dst[i] = make_uint4(*reinterpret_cast<uint32_t *>(&a),
                                *reinterpret_cast<uint32_t *>(&b),
                                *reinterpret_cast<uint32_t *>(&c),
                                *reinterpret_cast<uint32_t *>(&d));
        }
    } else {
        uint4 *dst = reinterpret_cast<uint4 *>(static_cast<__half *>(p.out) + off);
#pragma unroll
        for (uint32_t i = 0; i < 4; i++) {
            __half2 a = __floats2half2_rn(f[8 * i], f[8 * i + 1]);
            __half2 b = __floats2half2_rn(f[8 * i + 2], f[8 * i + 3]);
            __half2 c = __floats2half2_rn(f[8 * i + 4], f[8 * i + 5]);
            __half2 d = __floats2half2_rn(f[8 * i + 6], f[8 * i + 7]);
            dst[i] = make_uint4(*reinterpret_cast<uint32_t *>(&a),
                                *reinterpret_cast<uint32_t *>(&b),
                                *reinterpret_cast<uint32_t *>(&c),
                                *reinterpret_cast<uint32_t *>(&d));
        }
    }
}

template <uint32_t MT>
__global__ void __launch_bounds__(Layout<MT>::kThreads, 1)
q4k_linear_tc_kernel(const __grid_constant__ CUtensorMap x_map,
                     const __grid_constant__ CUtensorMap w_map, const LinearParams p) {
    using L = Layout<MT>;
    extern __shared__ uint8_t smem_raw[];
    uint8_t *smem = (uint8_t *)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    Misc *misc = reinterpret_cast<Misc *>(smem + L::kMisc);
    const uint32_t warp = threadIdx.x >> 5;
    const uint32_t lane = threadIdx.x & 31u;
    const uint32_t m0 = blockIdx.x * (MT * 128u);
    const uint32_t n0 = blockIdx.y * 128u;
    const uint32_t n_super = p.K / Q3_QUANT_QK_K;   /* Q4_K blocks per feature row */
    const uint32_t n_kt = n_super * 4u;             /* k-steps of 64 */

    if (threadIdx.x == 0) {
        for (uint32_t s = 0; s < kRawStages; s++) {
            mbar_init(&misc->raw_full[s], 1);
            mbar_init(&misc->raw_empty[s], L::kDequantThreads);
        }
        for (uint32_t s = 0; s < L::kXStages; s++) {
            mbar_init(&misc->x_full[s], 1);
            mbar_init(&misc->x_empty[s], 1);
        }
        for (uint32_t s = 0; s < L::kBStages; s++) {
            mbar_init(&misc->b_full[s], 128);
            mbar_init(&misc->b_empty[s], 1);
        }
        mbar_init(&misc->acc_full, 1);
        misc->abort_flag = 0;
        fence_mbar_init();
    }
    if (warp == 1) {
        tmem_alloc(&misc->tmem_base, L::kTmemCols);
        tmem_relinquish();
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = misc->tmem_base;

    if (warp == 0) {
        /* ============ activation tiles ============ */
        if (lane == 0) {
            prefetch_tmap(&x_map);
            bool alive = true;
            for (uint32_t kt = 0; kt < n_kt && alive; kt++) {
                const uint32_t s = kt % L::kXStages, use = kt / L::kXStages;
                if (use > 0) alive = wait_or_abort(&misc->x_empty[s], (use - 1) & 1u, misc);
                if (!alive) break;
                mbar_arrive_expect_tx(&misc->x_full[s], MT * kTileBytes);
#pragma unroll
                for (uint32_t mt = 0; mt < MT; mt++)
                    tma_load_2d(smem + L::kX + (s * MT + mt) * kTileBytes, &x_map,
                                (int32_t)(kt * 64u), (int32_t)(m0 + mt * 128u),
                                &misc->x_full[s]);
            }
        }
        __syncwarp();
    } else if (warp == 2) {
        /* ============ raw Q4_K blocks ============ */
        if (lane == 0) {
            prefetch_tmap(&w_map);
            bool alive = true;
            for (uint32_t sb = 0; sb < n_super && alive; sb++) {
                const uint32_t rs = sb % kRawStages, use = sb / kRawStages;
                if (use > 0) alive = wait_or_abort(&misc->raw_empty[rs], (use - 1) & 1u, misc);
                if (!alive) break;
                mbar_arrive_expect_tx(&misc->raw_full[rs], kRawBytes);
                tma_load_2d(smem + L::kRaw + rs * kRawBytes, &w_map,
                            (int32_t)(sb * kRawRowBytes), (int32_t)n0, &misc->raw_full[rs]);
            }
        }
        __syncwarp();
    } else if (warp == 1) {
        /* ============ MMA issuer ============ */
        if (elect_one()) {
            constexpr uint32_t idesc = umma_idesc_f16(128, 128, false);
            const uint32_t x_addr = smem_u32(smem + L::kX);
            const uint32_t b_addr = smem_u32(smem + L::kB);
            bool alive = true;
            for (uint32_t kt = 0; kt < n_kt; kt++) {
                const uint32_t s = kt % L::kXStages, bs = kt % L::kBStages;
                alive = wait_or_abort(&misc->x_full[s], (kt / L::kXStages) & 1u, misc) &&
                        wait_or_abort(&misc->b_full[bs], (kt / L::kBStages) & 1u, misc);
                if (!alive) break;
                tc_fence_after();
#pragma unroll
                for (uint32_t kk = 0; kk < 4; kk++) {
#pragma unroll
                    for (uint32_t mt = 0; mt < MT; mt++)
                        umma_ss(tmem + mt * 128u,
                                umma_desc(x_addr + (s * MT + mt) * kTileBytes + kk * 32u, 16, 1024),
                                umma_desc(b_addr + bs * kTileBytes + kk * 32u, 16, 1024), idesc,
                                (kt | kk) != 0u);
                }
                umma_commit(&misc->x_empty[s]);
                umma_commit(&misc->b_empty[bs]);
            }
            if (alive) umma_commit(&misc->acc_full);
        }
        __syncwarp();
    } else if (warp >= 4) {
        /* ============ dequantise, then drain the accumulators ============
         * Group g (128 threads, one per feature row) owns operand stage g and
         * converts k-steps g, g + kBStages, ...: the groups work on different
         * k-steps at the same time, which hides the latency of one step's
         * wait -> load -> convert -> store -> fence -> arrive chain. */
        const uint32_t dq = threadIdx.x - 128u;
        const uint32_t row = dq & 127u;
        const uint32_t group = dq >> 7;
        const uint32_t swz = row & 7u;
        uint8_t *brow = smem + L::kB + group * kTileBytes + row * 128u;
        const uint8_t *blk = nullptr;
        uint4 hdr = make_uint4(0, 0, 0, 0);
        float dd = 0.f, dm = 0.f;
        uint32_t cur_sb = 0xffffffffu;
        bool alive = true;
        for (uint32_t kt = group, use = 0; kt < n_kt; kt += L::kBStages, use++) {
            const uint32_t sb = kt >> 2, j = kt & 3u;
            if (sb != cur_sb) {
                if (cur_sb != 0xffffffffu) mbar_arrive(&misc->raw_empty[cur_sb % kRawStages]);
                const uint32_t rs = sb % kRawStages;
                alive = wait_or_abort(&misc->raw_full[rs], (sb / kRawStages) & 1u, misc);
                alive = __all_sync(0xffffffffu, alive);
                if (!alive) break;
                cur_sb = sb;
                blk = smem + L::kRaw + rs * kRawBytes + row * kRawRowBytes;
                hdr = *reinterpret_cast<const uint4 *>(blk);
                dd = __half2float(__ushort_as_half((unsigned short)(hdr.x & 0xffffu)));
                dm = __half2float(__ushort_as_half((unsigned short)(hdr.x >> 16)));
            }
            /* sub-blocks 2j (low nibbles) and 2j+1 (high nibbles); scales bytes
             * 0-3 = hdr.y, 4-7 = hdr.z, 8-11 = hdr.w */
            const uint32_t bsh = (j & 1u) * 16u;
            uint32_t sc_lo, mn_lo, sc_hi, mn_hi;
            if (j < 2) {
                const uint32_t a = hdr.y >> bsh, b = hdr.z >> bsh;
                sc_lo = a & 63u;
                mn_lo = b & 63u;
                sc_hi = (a >> 8) & 63u;
                mn_hi = (b >> 8) & 63u;
            } else {
                const uint32_t a = hdr.y >> bsh, b = hdr.z >> bsh, c = hdr.w >> bsh;
                sc_lo = (c & 0xFu) | (((a & 0xffu) >> 6) << 4);
                mn_lo = ((c & 0xffu) >> 4) | (((b & 0xffu) >> 6) << 4);
                sc_hi = ((c >> 8) & 0xFu) | ((((a >> 8) & 0xffu) >> 6) << 4);
                mn_hi = (((c >> 8) & 0xffu) >> 4) | ((((b >> 8) & 0xffu) >> 6) << 4);
            }
            const __half2 scale_lo = __float2half2_rn(dd * (float)sc_lo);
            const __half2 scale_hi = __float2half2_rn(dd * (float)sc_hi);
            const __half2 noff_lo = __hneg2(__float2half2_rn(dm * (float)mn_lo));
            const __half2 noff_hi = __hneg2(__float2half2_rn(dm * (float)mn_hi));

            if (use > 0) alive = wait_or_abort(&misc->b_empty[group], (use - 1) & 1u, misc);
            alive = __all_sync(0xffffffffu, alive);
            if (!alive) break;
            const uint4 qa = *reinterpret_cast<const uint4 *>(blk + 16u + 32u * j);
            const uint4 qb = *reinterpret_cast<const uint4 *>(blk + 32u + 32u * j);
            const uint32_t w[8] = {qa.x, qa.y, qa.z, qa.w, qb.x, qb.y, qb.z, qb.w};
#pragma unroll
            for (uint32_t c = 0; c < 4; c++) {
                /* quant bytes 8c..8c+7: low nibbles -> elements 8c.., chunk c;
                 * high nibbles -> elements 32+8c.., chunk 4+c */
                uint32_t lo[4], hi[4];
#pragma unroll
                for (uint32_t u = 0; u < 2; u++) {
                    const uint32_t p01 = __byte_perm(w[2 * c + u], 0u, 0x4140);
                    const uint32_t p23 = __byte_perm(w[2 * c + u], 0u, 0x4342);
                    lo[2 * u] = dequant_lo(p01, scale_lo, noff_lo);
                    lo[2 * u + 1] = dequant_lo(p23, scale_lo, noff_lo);
                    hi[2 * u] = dequant_hi(p01, scale_hi, noff_hi);
                    hi[2 * u + 1] = dequant_hi(p23, scale_hi, noff_hi);
                }
                *reinterpret_cast<uint4 *>(brow + ((c ^ swz) * 16u)) =
                    make_uint4(lo[0], lo[1], lo[2], lo[3]);
                *reinterpret_cast<uint4 *>(brow + (((4u + c) ^ swz) * 16u)) =
                    make_uint4(hi[0], hi[1], hi[2], hi[3]);
            }
            fence_proxy_async();
            mbar_arrive(&misc->b_full[group]);
        }
        if (alive && cur_sb != 0xffffffffu) mbar_arrive(&misc->raw_empty[cur_sb % kRawStages]);

        if (group < 2) {
            if (alive) alive = wait_or_abort(&misc->acc_full, 0u, misc);
            alive = __all_sync(0xffffffffu, alive);
            if (alive) {
                tc_fence_after();
                const uint32_t quarter = warp & 3u;      /* tensor-memory lanes 32*quarter.. */
                const uint32_t mt = MT == 2 ? group : 0u;
                const uint32_t col0 = MT == 2 ? 0u : group * 64u;
                const uint32_t n_chunks = MT == 2 ? 4u : 2u;
                const uint32_t token = m0 + mt * 128u + quarter * 32u + lane;
                const uint32_t taddr = tmem + ((quarter * 32u) << 16) + mt * 128u + col0;
                for (uint32_t ch = 0; ch < n_chunks; ch++) {
                    uint32_t v[32];
                    tmem_ld32(taddr + ch * 32u, v);
                    tmem_wait_ld();
                    if (token < p.M)
                        store_out32(p, (size_t)token * p.N + n0 + col0 + ch * 32u, v);
                }
            }
        }
    }

    tc_fence_before();
    __syncthreads();
    if (threadIdx.x == 0 && misc->abort_flag) atomicOr(p.status, 1u);
    if (warp == 1) tmem_dealloc(tmem, L::kTmemCols);
}

/* fp32 -> f16, 8 elements per thread (n is a multiple of 256: K is). */
__global__ void f32_to_f16_kernel(const float *__restrict__ in, __half *__restrict__ out,
                                  size_t n8) {
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n8) return;
    const float4 a = reinterpret_cast<const float4 *>(in)[2 * i];
    const float4 b = reinterpret_cast<const float4 *>(in)[2 * i + 1];
    __half2 h0 = __floats2half2_rn(a.x, a.y), h1 = __floats2half2_rn(a.z, a.w);
    __half2 h2 = __floats2half2_rn(b.x, b.y), h3 = __floats2half2_rn(b.z, b.w);
    reinterpret_cast<uint4 *>(out)[i] =
        make_uint4(*reinterpret_cast<uint32_t *>(&h0), *reinterpret_cast<uint32_t *>(&h1),
                   *reinterpret_cast<uint32_t *>(&h2), *reinterpret_cast<uint32_t *>(&h3));
}

static __device__ uint32_t q3_linear_status_word;

/* process-wide state, as in the reference (src/q3_q4_linear.cu:36-44) */
struct LinearState {
    bool initialized = false;
    int device = -1;
    size_t workspace_bytes = 0;
    void *workspace = nullptr;
    size_t workspace_attached = 0;
    uint32_t *status_dev = nullptr;
    cudaEvent_t ev_begin = nullptr, ev_mid = nullptr, ev_end = nullptr;
    bool timed_convert = false;
};
LinearState g;

size_t arena_bytes(size_t max_tokens, int64_t max_k) {
    const size_t b = max_tokens * (size_t)(max_k > 0 ? max_k : 0) * sizeof(__half);
    return (b + 255) & ~(size_t)255;
}

/* MT = 2 (256 tokens per CTA) halves the dequantisation work and the weight
 * operand traffic per FLOP; MT = 1 is for batches of at most 128 tokens or
 * when it needs less time (waves of 128-token tiles cost half as much). */
uint32_t choose_mt(uint32_t M, uint32_t N, int sm_count) {
    if (M <= 128) return 1;
    const uint64_t t1 = (uint64_t)((M + 127) / 128) * (N / 128);
    const uint64_t t2 = (uint64_t)((M + 255) / 256) * (N / 128);
    const uint64_t w1 = (t1 + sm_count - 1) / sm_count;        /* waves of cost 1 */
    const uint64_t w2 = 2 * ((t2 + sm_count - 1) / sm_count);  /* waves of cost 2 */
    return w2 <= w1 + w1 / 8 ? 2 : 1;
}

bool launch_linear(const q3_q4_linear_geometry *geo, const void *weight, const void *x_f16,
                   size_t tokens, void *out, uint32_t out_type, cudaStream_t stream,
                   char *error, size_t error_len) {
    const uint32_t M = (uint32_t)tokens, N = (uint32_t)geo->N, K = (uint32_t)geo->K;
    if (geo->qtype != Q3_QUANT_Q4_K)
        return q3_fail(error, error_len,
                       "q3_q4_linear: only Q4_K weights are implemented (Q6_K is not)");
    if (K % Q3_QUANT_QK_K || N % 128u)
        return q3_fail(error, error_len,
                       "q3_q4_linear: K must be a multiple of 256 and N of 128");
    if (((uintptr_t)weight | (uintptr_t)x_f16 | (uintptr_t)out) & 15u)
        return q3_fail(error, error_len, "q3_q4_linear: pointers must be 16-byte aligned");
    CUtensorMap x_map, w_map;
    if (!q3_encode_tmap_2d(&x_map, x_f16, K, M, 64, 128, error, error_len)) return false;
    if (!q3_encode_tmap_bytes_2d(&w_map, weight, (uint64_t)(K / Q3_QUANT_QK_K) * kRawRowBytes,
                                 N, kRawRowBytes, 128, error, error_len))
        return false;
    LinearParams p;
    p.out = out;
    p.M = M;
    p.N = N;
    p.K = K;
    p.out_type = out_type;
    p.status = g.status_dev;
    int sms = 148;
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, g.device);
    if (choose_mt(M, N, sms) == 2) {
        dim3 grid((M + 255) / 256, N / 128);
        q4k_linear_tc_kernel<2><<<grid, Layout<2>::kThreads, Layout<2>::kTotal, stream>>>(x_map, w_map, p);
    } else {
        dim3 grid((M + 127) / 128, N / 128);
        q4k_linear_tc_kernel<1><<<grid, Layout<1>::kThreads, Layout<1>::kTotal, stream>>>(x_map, w_map, p);
    }
    Q3_LAUNCH_CHECK("q4k_linear_tc launch failed");
    return true;
}

}  // namespace

extern "C" bool q3_q4_linear_bind_geometry(uint32_t qtype, uint32_t gguf_rows_dim0,
                                           uint32_t gguf_cols_dim1,
                                           q3_q4_linear_geometry *out, char *error,
                                           size_t error_len) {
    q3_clear_error(error, error_len);
    if (!out) return q3_fail(error, error_len, "q3_q4_linear: null geometry");
    memset(out, 0, sizeof(*out));
    if (qtype != Q3_QUANT_Q4_K && qtype != Q3_QUANT_Q6_K)
        return q3_fail(error, error_len, "q3_q4_linear: weight is neither Q4_K nor Q6_K");
    const uint64_t K = gguf_rows_dim0, N = gguf_cols_dim1;
    if (K == 0 || N == 0) return q3_fail(error, error_len, "q3_q4_linear: degenerate geometry");
    if (K % Q3_QUANT_QK_K) {
        if (error && error_len)
            snprintf(error, error_len, "q3_q4_linear: K=%llu must be a multiple of %d",
                     (unsigned long long)K, Q3_QUANT_QK_K);
        return false;
    }
    if (K > INT32_MAX || N > INT32_MAX)
        return q3_fail(error, error_len, "q3_q4_linear: geometry exceeds int32");
    out->K = (int32_t)K;
    out->N = (int32_t)N;
    out->M = 0;
    out->qtype = qtype;
    out->weight_bytes = N * (K / Q3_QUANT_QK_K) *
                        (qtype == Q3_QUANT_Q6_K ? 210u : (uint64_t)Q3_QUANT_Q4_K_BLOCK_BYTES);
    return true;
}

extern "C" bool q3_cuda_q4k_linear_init(int device, size_t max_tokens, int64_t max_features,
                                        int64_t max_k, char *error, size_t error_len) {
    q3_clear_error(error, error_len);
    (void)max_features;
    if (device < 0) return q3_fail(error, error_len, "q3_q4_linear: invalid device index");
    const size_t need = arena_bytes(max_tokens, max_k);
    if (g.initialized && g.device == device) {
        if (need > g.workspace_bytes) g.workspace_bytes = need;   /* never shrinks */
        return true;
    }
    int count = 0;
    if (cudaGetDeviceCount(&count) != cudaSuccess || count == 0)
        return q3_fail(error, error_len, "q3_q4_linear: no CUDA device");
    cudaError_t e = cudaSetDevice(device);
    if (e != cudaSuccess) return q3_fail_cuda(error, error_len, "q3_q4_linear: cudaSetDevice", e);
    e = cudaFuncSetAttribute(q4k_linear_tc_kernel<1>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                             (int)Layout<1>::kTotal);
    if (e == cudaSuccess)
        e = cudaFuncSetAttribute(q4k_linear_tc_kernel<2>,
                                 cudaFuncAttributeMaxDynamicSharedMemorySize,
                                 (int)Layout<2>::kTotal);
    if (e == cudaSuccess) e = cudaGetSymbolAddress((void **)&g.status_dev, q3_linear_status_word);
    if (e == cudaSuccess) e = cudaMemset(g.status_dev, 0, sizeof(uint32_t));
    if (e == cudaSuccess && !g.ev_begin) {
        e = cudaEventCreate(&g.ev_begin);
        if (e == cudaSuccess) e = cudaEventCreate(&g.ev_mid);
        if (e == cudaSuccess) e = cudaEventCreate(&g.ev_end);
    }
    if (e != cudaSuccess) return q3_fail_cuda(error, error_len, "q3_q4_linear: set-up", e);
    g.device = device;
    g.workspace_bytes = need;
    g.workspace = nullptr;
    g.workspace_attached = 0;
    g.initialized = true;
    return true;
}

extern "C" size_t q3_cuda_q4k_linear_workspace_bytes(void) { return g.workspace_bytes; }

extern "C" bool q3_cuda_q4k_linear_set_workspace(void *device_ptr, size_t bytes, char *error,
                                                 size_t error_len) {
    q3_clear_error(error, error_len);
    if (!device_ptr || bytes < g.workspace_bytes || ((uintptr_t)device_ptr & 15u)) {
        if (error && error_len)
            snprintf(error, error_len, "q3_q4_linear: workspace too small (%zu < %zu)", bytes,
                     g.workspace_bytes);
        return false;
    }
    g.workspace = device_ptr;
    g.workspace_attached = bytes;
    return true;
}

extern "C" const char *q3_cuda_q4k_linear_path_for_batch(size_t token_count) {
    (void)token_count;
    return "TC";
}

extern "C" bool q3_cuda_q4k_linear(const q3_q4_linear_geometry *geometry, const void *weight,
                                   const float *device_input, size_t token_count,
                                   float *device_output, void *stream,
                                   q3_q4_linear_stats *stats, char *error, size_t error_len) {
    q3_clear_error(error, error_len);
    if (!geometry || !weight || !device_input || !device_output)
        return q3_fail(error, error_len, "q3_q4_linear: null argument");
    if (!g.initialized) return q3_fail(error, error_len, "q3_q4_linear: not initialized");
    if (token_count == 0 || token_count > INT32_MAX)
        return q3_fail(error, error_len, "q3_q4_linear: bad token count");
    if (geometry->N <= 0 || geometry->K <= 0)
        return q3_fail(error, error_len, "q3_q4_linear: unresolved geometry");
    const size_t need = token_count * (size_t)geometry->K * sizeof(__half);
    if (!g.workspace || need > g.workspace_attached)
        return q3_fail(error, error_len,
                       "q3_q4_linear: workspace missing or too small for this batch");
    if (stats) {
        memset(stats, 0, sizeof(*stats));
        stats->weight_bytes = geometry->weight_bytes;
        stats->kernel_launches = 2;
        stats->activation_read_bytes = token_count * (size_t)geometry->K * sizeof(float);
        stats->activation_write_bytes = token_count * (size_t)geometry->N * sizeof(float);
    }
    cudaStream_t st = (cudaStream_t)stream;
    cudaEventRecord(g.ev_begin, st);
    const size_t n8 = token_count * (size_t)geometry->K / 8;
    f32_to_f16_kernel<<<(unsigned)((n8 + 255) / 256), 256, 0, st>>>(
        device_input, static_cast<__half *>(g.workspace), n8);
    Q3_LAUNCH_CHECK("q3_q4_linear: activation conversion launch failed");
    cudaEventRecord(g.ev_mid, st);
    if (!launch_linear(geometry, weight, g.workspace, token_count, device_output, Q3_OUT_F32,
                       st, error, error_len))
        return false;
    cudaEventRecord(g.ev_end, st);
    g.timed_convert = true;
    return true;
}

extern "C" void q3_cuda_q4k_linear_read_stats(q3_q4_linear_stats *stats, void *stream) {
    (void)stream;
    if (!stats || !g.initialized || !g.timed_convert) return;
    float a = 0.f, b = 0.f;
    if (cudaEventElapsedTime(&a, g.ev_begin, g.ev_mid) == cudaSuccess)
        stats->activation_quant_ms = a;
    if (cudaEventElapsedTime(&b, g.ev_mid, g.ev_end) == cudaSuccess) stats->kernel_ms = b;
    stats->total_ms = (double)a + (double)b;
}

extern "C" bool q3_cuda_q4k_linear_f16(const q3_q4_linear_geometry *geometry,
                                       const void *weight, const void *x_f16,
                                       size_t token_count, void *out, uint32_t out_type,
                                       void *stream, char *error, size_t error_len) {
    q3_clear_error(error, error_len);
    if (!geometry || !weight || !x_f16 || !out)
        return q3_fail(error, error_len, "q3_q4_linear: null argument");
    if (!g.initialized) return q3_fail(error, error_len, "q3_q4_linear: not initialized");
    if (token_count == 0 || token_count > INT32_MAX)
        return q3_fail(error, error_len, "q3_q4_linear: bad token count");
    if (geometry->N <= 0 || geometry->K <= 0)
        return q3_fail(error, error_len, "q3_q4_linear: unresolved geometry");
    if (out_type > Q3_OUT_F16) return q3_fail(error, error_len, "q3_q4_linear: bad output type");
    return launch_linear(geometry, weight, x_f16, token_count, out, out_type,
                         (cudaStream_t)stream, error, error_len);
}

extern "C" bool q3_cuda_q4k_linear_status(void *stream, uint32_t *status, char *error,
                                          size_t error_len) {
    q3_clear_error(error, error_len);
    if (!status) return q3_fail(error, error_len, "q3_q4_linear: null argument");
    if (!g.initialized) return q3_fail(error, error_len, "q3_q4_linear: not initialized");
    cudaError_t e = cudaStreamSynchronize((cudaStream_t)stream);
    if (e == cudaSuccess)
        e = cudaMemcpy(status, g.status_dev, sizeof(uint32_t), cudaMemcpyDeviceToHost);
    if (e != cudaSuccess) return q3_fail_cuda(error, error_len, "q3_q4_linear: status read", e);
    return true;
}
