/* q3_q4k_linear.cu - resident Q4_K weight x activation on the sm_100a tensor
 * cores (tcgen05, accumulators and the weight operand in tensor memory).
 *
 *   out[token][feature] = sum_k W[feature][k] * x[token][k]
 *
 * W stays in its 144-byte Q4_K blocks in HBM (ref: src/q3_quant.h:24-33). A CTA
 * owns 128 features x NT tokens (NT <= 256) and walks K in steps of 64. The MMA
 * runs transposed: D[feature][token] += W[feature][k] * x[token][k], M = 128
 * features (tensor-memory lanes), N = NT tokens, with
 *   A = W tile, dequantised to f16 by the CTA's warps and stored straight
 *       into tensor memory (tcgen05.st; thread = feature row = lane), and
 *   B = x tile [NT tokens][64 k] f16 in shared memory (TMA, 128-byte swizzle).
 * Keeping the weight operand out of shared memory matters: with both operands
 * in shared memory this kernel was bound by shared-memory bandwidth (operand
 * stores + TMA writes + MMA reads were about 240 B/clk at full tensor rate).
 *
 *   warp 0      TMA producer of the activation tiles
 *   warp 1      allocates tensor memory, issues tcgen05.mma (one thread)
 *   warp 2      TMA producer of the raw weight bytes: per 256 k one box of
 *               128 rows x 144 bytes (one Q4_K block per feature row)
 *   warps 4-15  three groups of four warps dequantise: group g takes k-steps
 *               g, g+3, ...; thread = feature row; 64 quants -> 32 packed f16
 *               registers -> tcgen05.st; afterwards all of them drain D
 *
 * A k-step of 64 is exactly one 32-byte group of a block: its low nibbles are
 * elements 0..31, its high nibbles elements 32..63 (ref: src/q3_quant.c:57-76),
 * each half with its own 6-bit scale and min (ref: src/q3_quant.c:44-55).
 * Operand rounding: scale = f16(d*sc), offset = f16(dmin*m), element =
 * f16(fma(q, scale, -offset)); activations are f16; accumulation is fp32.
 *
 * A second instantiation serves the q/k/v projection of a layer (three weights,
 * a feature tile = one head): its drain normalises and rotates the heads and
 * writes f16 queries and K/V pages instead of an output tensor (FusedEpilogue).
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

/* q3_q4k_small.cu */
#define Q3_Q4K_SMALL_BATCH 16u
bool q3_launch_q4k_small(const void *weight, const void *x_f16, uint32_t M, uint32_t N,
                         uint32_t K, void *out, uint32_t out_type, cudaStream_t stream,
                         char *error, size_t error_len);

/* q3_q4k_mmvq.cu */
#define Q3_MMVQ_MAX_BATCH 8u
size_t q3_q4k_mmvq_workspace_bytes(size_t tokens, size_t k);
bool q3_launch_q4k_generic(uint32_t qtype, const void *weight, const void *x_f16, uint32_t M,
                           uint32_t N, uint32_t K, void *out, uint32_t out_type,
                           cudaStream_t stream, char *error, size_t error_len);
bool q3_launch_q4k_mmvq(const void *weight, const float *x, uint32_t M, uint32_t N, uint32_t K,
                        float *out, void *workspace, cudaStream_t stream, char *error,
                        size_t error_len);

namespace {
using namespace q3ptx;

/* Per weight format: bytes of one block as it sits in shared memory. Q6_K
 * blocks are 210 bytes (not a multiple of 16, so TMA cannot fetch them from
 * the GGUF order); they exist only in the tiled layout, padded to 224. */
template <uint32_t QT> struct Fmt;
template <> struct Fmt<4> { static constexpr uint32_t kRowBytes = 144; };
template <> struct Fmt<6> { static constexpr uint32_t kRowBytes = 224; };
constexpr uint32_t kRawStages = 2;
constexpr uint32_t kMaxTokens = 256;               /* token tile = MMA N */
constexpr uint32_t kXStageBytes = kMaxTokens * 128; /* [256 tokens][64 k] f16 */
constexpr uint32_t kXStages = 5;
constexpr uint32_t kAStages = 6;                   /* weight operand stages in tensor memory */
constexpr uint32_t kGroups = 3;                    /* dequantising warp groups */
constexpr uint32_t kThreads = 128 + 128 * kGroups;
constexpr uint32_t kColD = 0;                      /* D: 128 lanes x 256 fp32 columns */
constexpr uint32_t kColA = 256;                    /* A stage: 128 lanes x 32 columns (64 f16) */
constexpr uint32_t kTmemCols = 512;
constexpr uint32_t kSmemX = 0;
constexpr uint32_t kSmemRaw = kSmemX + kXStages * kXStageBytes;
constexpr uint32_t kStageTokens = 16;               /* fused epilogue: tokens staged per group */
constexpr uint32_t kStageBytes = kStageTokens * 128 * 4;
template <uint32_t QT, bool FUSED = false>
struct Smem {
    static constexpr uint32_t kRowBytes = Fmt<QT>::kRowBytes;
    static constexpr uint32_t kRawBytes = 128 * kRowBytes;   /* 128 feature rows, one block each */
    static constexpr uint32_t kTiledRows = kRawBytes / 256;  /* tiled layout: a chunk in rows of 256 B */
    static constexpr uint32_t kStage = kSmemRaw + kRawStages * kRawBytes;  /* fused epilogue only */
    static constexpr uint32_t kMisc = kStage + (FUSED ? kGroups * kStageBytes : 0u);
    static constexpr uint32_t kTotal = kMisc + 512 + 1024;   /* + alignment slack */
};
static_assert(Smem<6>::kTotal <= 227 * 1024, "shared memory budget");
static_assert(Smem<4, true>::kTotal <= 227 * 1024, "shared memory budget of the fused kernel");
static_assert(kColA + kAStages * 32 <= kTmemCols, "tensor memory budget");
static_assert(kAStages % kGroups == 0, "a group must come back to its own stages");

struct Misc {
    uint64_t raw_full[kRawStages], raw_empty[kRawStages];
    uint64_t x_full[kXStages], x_empty[kXStages];
    uint64_t a_full[kAStages], a_empty[kAStages];
    uint64_t acc_full, d_free;
    uint64_t stage_full[kGroups], stage_empty[kGroups];   /* fused epilogue: staging hand-over */
    uint32_t tmem_base;
    uint32_t abort_flag;
};
static_assert(sizeof(Misc) <= 512, "Misc must fit its slot");

/* Fused epilogue of the q/k/v projection (ref: the five steps after the three
 * linears in run_layer / run_layer_packed, src/q3_forward.cu:1244-1278 and
 * :1489-1516): a feature tile of 128 is one head; query and key heads are
 * RMS-normalised and rotated, all three are written as f16 - queries into the
 * attention kernel's Q buffer, keys and values into their pages. */
struct FusedEpilogue {
    uint32_t seg_end[3];      /* feature tiles: [0, e0) query heads, [e0, e1) key, [e1, e2) value */
    uint32_t n_q_heads;
    const float *norm_w;      /* [2][128]: query weights, key weights */
    float eps;
    const float2 *rope_table; /* [position][64] (cos, sin) of the pair (d, d + 64) */
    const uint32_t *rope_pos, *dst_page, *dst_slot;
    __half *q_out;            /* [tokens][n_q_heads][128] */
    __half *k_pool, *v_pool;  /* this layer: [kv head][page][16][128] */
    uint32_t num_pages;
};

struct LinearParams {
    void *out;
    uint32_t M, N, K;
    uint32_t NT;          /* tokens per CTA: multiple of 16, <= 256 */
    uint32_t w_tiled;     /* weight in the tiled layout of q3_cuda_q4k_linear_pack */
    uint32_t out_type;
    uint32_t *status;
    FusedEpilogue f;      /* read by the fused instantiation only */
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

/* One k-step (64 elements) of one Q4_K block -> 32 packed f16 pairs, element
 * order. j = 32-byte quant group of the block (ref: src/q3_quant.c:44-76). */
__device__ __forceinline__ void convert_q4(const uint8_t *blk, uint32_t j, uint32_t *v) {
    const uint4 hdr = *reinterpret_cast<const uint4 *>(blk);
    const float dd = __half2float(__ushort_as_half((unsigned short)(hdr.x & 0xffffu)));
    const float dm = __half2float(__ushort_as_half((unsigned short)(hdr.x >> 16)));
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
    const uint4 qa = *reinterpret_cast<const uint4 *>(blk + 16u + 32u * j);
    const uint4 qb = *reinterpret_cast<const uint4 *>(blk + 32u + 32u * j);
    const uint32_t w[8] = {qa.x, qa.y, qa.z, qa.w, qb.x, qb.y, qb.z, qb.w};
    /* register i = elements (2i, 2i+1) of the k-step: low nibbles of the 32
     * quant bytes are elements 0..31, high nibbles elements 32..63 */
#pragma unroll
    for (uint32_t u = 0; u < 8; u++) {
        const uint32_t p01 = __byte_perm(w[u], 0u, 0x4140);
        const uint32_t p23 = __byte_perm(w[u], 0u, 0x4342);
        v[2 * u] = dequant_lo(p01, scale_lo, noff_lo);
        v[2 * u + 1] = dequant_lo(p23, scale_lo, noff_lo);
        v[16 + 2 * u] = dequant_hi(p01, scale_hi, noff_hi);
        v[16 + 2 * u + 1] = dequant_hi(p23, scale_hi, noff_hi);
    }
}

/* Q6_K: `nib` holds two quant bytes in its 16-bit lanes already shifted so that
 * the wanted nibble is in bits 0-3, `hb4` the two high-bit bytes shifted so that
 * the wanted 2 bits are in bits 4-5. 0x6400 | q is the f16 1024 + q; the value
 * is f16((q - 32) * scale). */
__device__ __forceinline__ uint32_t dequant6(uint32_t nib, uint32_t hb4, __half2 scale) {
    uint32_t b = (nib & 0x000F000Fu) | (hb4 & 0x00300030u) | 0x64006400u;
    const __half2 bias = __half2half2(__ushort_as_half((unsigned short)0x6420)); /* 1056 */
    __half2 h = __hmul2(__hsub2(*reinterpret_cast<__half2 *>(&b), bias), scale);
    return *reinterpret_cast<uint32_t *>(&h);
}

/* One k-step (64 elements) of one Q6_K block (ql[128] | qh[64] | scales[16] int8
 * | d, ref: src/q3_quant.c:78-103). k-step j lies in half h = j / 2 of the block;
 * its first 32 elements take the nibbles of ql[64h + l], its last 32 those of
 * ql[64h + 32 + l] (low nibbles for even j, high for odd), both with 2 more bits
 * from qh[32h + l]; one int8 scale per 16 elements. */
__device__ __forceinline__ void convert_q6(const uint8_t *blk, uint32_t j, uint32_t *v) {
    const uint32_t h = j >> 1, odd = j & 1u;
    const float d = __half2float(
        __ushort_as_half(*reinterpret_cast<const unsigned short *>(blk + 208)));
    const uint32_t sc4 = *reinterpret_cast<const uint32_t *>(blk + 192u + 8u * h + 4u * odd);
    const __half2 s_a0 = __float2half2_rn(d * (float)(int8_t)(sc4 & 0xffu));
    const __half2 s_a1 = __float2half2_rn(d * (float)(int8_t)((sc4 >> 8) & 0xffu));
    const __half2 s_b0 = __float2half2_rn(d * (float)(int8_t)((sc4 >> 16) & 0xffu));
    const __half2 s_b1 = __float2half2_rn(d * (float)(int8_t)(sc4 >> 24));
    const uint4 *ql = reinterpret_cast<const uint4 *>(blk + 64u * h);
    const uint4 *qh = reinterpret_cast<const uint4 *>(blk + 128u + 32u * h);
    const uint32_t nsh = 4u * odd;          /* nibble select */
    const uint32_t sh_a = 4u * odd;         /* high bits of the first 32 elements */
    const uint32_t sh_b = 4u * odd + 2u;    /* ... of the last 32 */
#pragma unroll
    for (uint32_t c = 0; c < 2; c++) {
        const uint4 a4 = ql[c], b4 = ql[2 + c], h4 = qh[c];
        const uint32_t wa[4] = {a4.x, a4.y, a4.z, a4.w};
        const uint32_t wb[4] = {b4.x, b4.y, b4.z, b4.w};
        const uint32_t wh[4] = {h4.x, h4.y, h4.z, h4.w};
        const __half2 sa = c == 0 ? s_a0 : s_a1;
        const __half2 sb = c == 0 ? s_b0 : s_b1;
#pragma unroll
        for (uint32_t i = 0; i < 4; i++) {
            const uint32_t u = 4 * c + i;   /* quant bytes 4u .. 4u+3 */
            const uint32_t a01 = __byte_perm(wa[i], 0u, 0x4140) >> nsh;
            const uint32_t a23 = __byte_perm(wa[i], 0u, 0x4342) >> nsh;
            const uint32_t b01 = __byte_perm(wb[i], 0u, 0x4140) >> nsh;
            const uint32_t b23 = __byte_perm(wb[i], 0u, 0x4342) >> nsh;
            const uint32_t h01 = __byte_perm(wh[i], 0u, 0x4140) << 4;
            const uint32_t h23 = __byte_perm(wh[i], 0u, 0x4342) << 4;
            v[2 * u] = dequant6(a01, h01 >> sh_a, sa);
            v[2 * u + 1] = dequant6(a23, h23 >> sh_a, sa);
            v[16 + 2 * u] = dequant6(b01, h01 >> sh_b, sb);
            v[16 + 2 * u + 1] = dequant6(b23, h23 >> sh_b, sb);
        }
    }
}

/* One output row segment: 32 token columns of one feature (lane) - the 32 lanes
 * of a warp store 32 consecutive features of one token per instruction. */
__device__ __forceinline__ void store_chunk(const LinearParams &p, const uint32_t *v,
                                            uint32_t m0, uint32_t t0, uint32_t feature) {
#pragma unroll
    for (uint32_t i = 0; i < 32; i++) {
        const uint32_t t = t0 + i;
        const uint32_t token = m0 + t;
        if (t < p.NT && token < p.M) {
            const size_t off = (size_t)token * p.N + feature;
            const float f = __uint_as_float(v[i]);
            if (p.out_type == Q3_OUT_F32)
                static_cast<float *>(p.out)[off] = f;
            else if (p.out_type == Q3_OUT_BF16)
                static_cast<__nv_bfloat16 *>(p.out)[off] = __float2bfloat16_rn(f);
            else
                static_cast<__half *>(p.out)[off] = __float2half_rn(f);
        }
    }
}

/* Persistent: CTA b computes output tiles b, b + gridDim.x, ... (tile = token
 * tile fastest, then feature tile). All rings run on counters that continue
 * across tiles, so the producers and the dequantising groups flow from one
 * tile into the next; only the accumulator D is single: a tile's first MMA
 * waits until every thread has read the previous tile's D out of tensor
 * memory (d_free). A group reads D after it has already converted its next two
 * k-steps, so the MMA has operands to go on with while the rows are stored. */
template <uint32_t QT, bool FUSED>
__global__ void __launch_bounds__(kThreads, 1)
q4k_linear_tc_kernel(const __grid_constant__ CUtensorMap x_map,
                     const __grid_constant__ CUtensorMap w_map,
                     const __grid_constant__ CUtensorMap w_map1,
                     const __grid_constant__ CUtensorMap w_map2, const LinearParams p) {
    constexpr uint32_t kRawRowBytes = Smem<QT>::kRowBytes;
    constexpr uint32_t kRawBytes = Smem<QT>::kRawBytes;
    constexpr uint32_t kTiledRows = Smem<QT>::kTiledRows;
    extern __shared__ uint8_t smem_raw[];
    uint8_t *smem = (uint8_t *)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    Misc *misc = reinterpret_cast<Misc *>(smem + Smem<QT, FUSED>::kMisc);
    const uint32_t warp = threadIdx.x >> 5;
    const uint32_t lane = threadIdx.x & 31u;
    const uint32_t n_super = p.K / Q3_QUANT_QK_K;   /* Q4_K blocks per feature row */
    const uint32_t n_kt = n_super * 4u;             /* k-steps of 64 per tile */
    const uint32_t n_tok_tiles = (p.M + p.NT - 1u) / p.NT;
    const uint32_t n_tiles = n_tok_tiles * (p.N / 128u);
    const uint32_t n_my = blockIdx.x < n_tiles
                              ? (n_tiles - blockIdx.x + gridDim.x - 1u) / gridDim.x : 0u;

    if (threadIdx.x == 0) {
        for (uint32_t s = 0; s < kRawStages; s++) {
            mbar_init(&misc->raw_full[s], 1);
            mbar_init(&misc->raw_empty[s], 128 * kGroups);
        }
        for (uint32_t s = 0; s < kXStages; s++) {
            mbar_init(&misc->x_full[s], 1);
            mbar_init(&misc->x_empty[s], 1);
        }
        for (uint32_t s = 0; s < kAStages; s++) {
            mbar_init(&misc->a_full[s], 128);
            mbar_init(&misc->a_empty[s], 1);
        }
        mbar_init(&misc->acc_full, 1);
        mbar_init(&misc->d_free, 128 * kGroups);
        for (uint32_t s = 0; s < kGroups; s++) {
            mbar_init(&misc->stage_full[s], 128);
            mbar_init(&misc->stage_empty[s], 128);
        }
        misc->abort_flag = 0;
        fence_mbar_init();
    }
    if (warp == 1) {
        tmem_alloc(&misc->tmem_base, kTmemCols);
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
            uint32_t g = 0;   /* k-steps issued by this CTA so far */
            for (uint32_t ti = 0; ti < n_my && alive; ti++) {
                const uint32_t tile = blockIdx.x + ti * gridDim.x;
                const uint32_t m0 = (tile % n_tok_tiles) * p.NT;
                for (uint32_t kt = 0; kt < n_kt; kt++, g++) {
                    const uint32_t s = g % kXStages, use = g / kXStages;
                    if (use > 0) alive = wait_or_abort(&misc->x_empty[s], (use - 1) & 1u, misc);
                    if (!alive) break;
                    mbar_arrive_expect_tx(&misc->x_full[s], p.NT * 128u);
                    tma_load_2d(smem + kSmemX + s * kXStageBytes, &x_map, (int32_t)(kt * 64u),
                                (int32_t)m0, &misc->x_full[s]);
                }
            }
        }
        __syncwarp();
    } else if (warp == 2) {
        /* ============ raw Q4_K blocks ============ */
        if (lane == 0) {
            prefetch_tmap(&w_map);
            if (FUSED) {
                prefetch_tmap(&w_map1);
                prefetch_tmap(&w_map2);
            }
            bool alive = true;
            uint32_t g = 0;   /* super-blocks issued so far */
            for (uint32_t ti = 0; ti < n_my && alive; ti++) {
                const uint32_t tile = blockIdx.x + ti * gridDim.x;
                uint32_t ft = tile / n_tok_tiles;      /* feature tile */
                const CUtensorMap *wm = &w_map;
                if (FUSED) {                           /* q, k and v are three tensors */
                    if (ft >= p.f.seg_end[1]) {
                        wm = &w_map2;
                        ft -= p.f.seg_end[1];
                    } else if (ft >= p.f.seg_end[0]) {
                        wm = &w_map1;
                        ft -= p.f.seg_end[0];
                    }
                }
                const uint32_t n0 = ft * 128u;
                for (uint32_t sb = 0; sb < n_super; sb++, g++) {
                    const uint32_t rs = g % kRawStages, use = g / kRawStages;
                    if (use > 0)
                        alive = wait_or_abort(&misc->raw_empty[rs], (use - 1) & 1u, misc);
                    if (!alive) break;
                    mbar_arrive_expect_tx(&misc->raw_full[rs], kRawBytes);
                    if (p.w_tiled)   /* 18432 contiguous bytes = 72 rows of 256 */
                        tma_load_2d(smem + kSmemRaw + rs * kRawBytes, wm, 0,
                                    (int32_t)(((n0 / 128u) * n_super + sb) * kTiledRows),
                                    &misc->raw_full[rs]);
                    else
                        tma_load_2d(smem + kSmemRaw + rs * kRawBytes, wm,
                                    (int32_t)(sb * kRawRowBytes), (int32_t)n0,
                                    &misc->raw_full[rs]);
                }
            }
        }
        __syncwarp();
    } else if (warp == 1) {
        /* ============ MMA issuer ============ */
        if (elect_one()) {
            const uint32_t idesc = umma_idesc_f16(128, p.NT, false);
            const uint32_t x_addr = smem_u32(smem + kSmemX);
            bool alive = true;
            uint32_t g = 0;
            for (uint32_t ti = 0; ti < n_my && alive; ti++) {
                if (ti > 0) {
                    alive = wait_or_abort(&misc->d_free, (ti - 1) & 1u, misc);
                    if (!alive) break;
                    tc_fence_after();
                }
                for (uint32_t kt = 0; kt < n_kt; kt++, g++) {
                    const uint32_t sx = g % kXStages, sa = g % kAStages;
                    alive = wait_or_abort(&misc->x_full[sx], (g / kXStages) & 1u, misc) &&
                            wait_or_abort(&misc->a_full[sa], (g / kAStages) & 1u, misc);
                    if (!alive) break;
                    tc_fence_after();
#pragma unroll
                    for (uint32_t kk = 0; kk < 4; kk++)
                        umma_ts(tmem + kColD, tmem + kColA + sa * 32u + kk * 8u,
                                umma_desc(x_addr + sx * kXStageBytes + kk * 32u, 16, 1024),
                                idesc, (kt | kk) != 0u);
                    umma_commit(&misc->x_empty[sx]);
                    umma_commit(&misc->a_empty[sa]);
                }
                if (alive) umma_commit(&misc->acc_full);
            }
        }
        __syncwarp();
    } else if (warp >= 4) {
        /* ============ dequantise into tensor memory; drain D ============
         * Group g (128 threads, one per feature row) converts this CTA's
         * k-steps g, g+3, ... (counted across tiles): the groups work on
         * different k-steps at the same time, which hides the latency of one
         * step's wait -> load -> convert -> store chain. */
        const uint32_t dq = threadIdx.x - 128u;
        const uint32_t row = dq & 127u;              /* feature row = tensor-memory lane */
        const uint32_t group = dq >> 7;
        const uint32_t lane_base = ((warp & 3u) * 32u) << 16;
        const uint32_t n_chunks = (p.NT + 31u) / 32u;
        const uint8_t *blk = nullptr;
        uint32_t cur_sb = 0xffffffffu;
        bool alive = true;

        uint32_t stored = 0xffffffffu;   /* A stage whose store is issued but not yet published */
        auto publish = [&]() {
            if (stored != 0xffffffffu) {
                tmem_wait_st();
                tc_fence_before();
                mbar_arrive(&misc->a_full[stored]);
                stored = 0xffffffffu;
            }
        };

        /* Fused epilogue: the group's 32-token chunks of D go through a staging
         * buffer of 16 tokens x 128 features (fp32) so that a warp can work
         * along a token's head: lane l holds features 2l, 2l+1, 64+2l, 65+2l -
         * both members of two rotary pairs. Arithmetic per row as in the
         * stand-alone kernel (q3_kvwrite.cu), on the fp32 accumulator instead
         * of a bf16 copy of it. */
        uint32_t stage_use = 0;
        auto drain_fused = [&](uint32_t ti) {
            publish();
            if (alive) alive = wait_or_abort(&misc->acc_full, ti & 1u, misc);
            alive = __all_sync(0xffffffffu, alive);
            if (!alive) return;
            tc_fence_after();
            const uint32_t tile = blockIdx.x + ti * gridDim.x;
            const uint32_t m0 = (tile % n_tok_tiles) * p.NT;
            uint32_t head = tile / n_tok_tiles, kind = 0;     /* 0 query, 1 key, 2 value */
            if (head >= p.f.seg_end[1]) {
                kind = 2;
                head -= p.f.seg_end[1];
            } else if (head >= p.f.seg_end[0]) {
                kind = 1;
                head -= p.f.seg_end[0];
            }
            float2 w_lo = make_float2(1.f, 1.f), w_hi = make_float2(1.f, 1.f);
            if (kind < 2) {
                w_lo = *reinterpret_cast<const float2 *>(p.f.norm_w + kind * 128u + 2u * lane);
                w_hi = *reinterpret_cast<const float2 *>(p.f.norm_w + kind * 128u + 64u + 2u * lane);
            }
            float *stg = reinterpret_cast<float *>(smem + Smem<QT, FUSED>::kStage +
                                                   group * kStageBytes);
            const uint32_t wig = warp & 3u;      /* warp within the group */
            bool released = false;
            for (uint32_t ch = group; ch < n_chunks && alive; ch += kGroups) {
                uint32_t v[32];
                tmem_ld32(tmem + lane_base + kColD + ch * 32u, v);
                tmem_wait_ld();
                if (ch + kGroups >= n_chunks) {      /* last chunk of this thread: release D */
                    tc_fence_before();
                    mbar_arrive(&misc->d_free);
                    released = true;
                }
#pragma unroll
                for (uint32_t hf = 0; hf < 2; hf++) {
                    /* this warp's four tokens: position and page, in flight during
                     * the staging hand-over below */
                    uint32_t pos[4], page[4], slot[4];
#pragma unroll
                    for (uint32_t tt = 0; tt < 4; tt++) {
                        const uint32_t tl = ch * 32u + hf * kStageTokens + wig * 4u + tt;
                        const uint32_t token = m0 + tl;
                        const bool ok = tl < p.NT && token < p.M;
                        pos[tt] = ok && kind < 2 ? p.f.rope_pos[token] : 0u;
                        page[tt] = ok ? (kind ? p.f.dst_page[token] : 0u) : Q3_NO_PAGE;
                        slot[tt] = ok && kind ? p.f.dst_slot[token] : 0u;
                    }
                    if (stage_use > 0)
                        alive = wait_or_abort(&misc->stage_empty[group], (stage_use - 1u) & 1u, misc);
                    alive = __all_sync(0xffffffffu, alive);
                    if (!alive) break;
#pragma unroll
                    for (uint32_t i = 0; i < kStageTokens; i++)
                        stg[i * 128u + row] = __uint_as_float(v[hf * kStageTokens + i]);
                    mbar_arrive(&misc->stage_full[group]);
                    alive = wait_or_abort(&misc->stage_full[group], stage_use & 1u, misc);
                    alive = __all_sync(0xffffffffu, alive);
                    if (!alive) break;
                    float4 cs[4];
                    if (kind < 2) {
#pragma unroll
                        for (uint32_t tt = 0; tt < 4; tt++)
                            cs[tt] = *reinterpret_cast<const float4 *>(
                                p.f.rope_table + (size_t)pos[tt] * 64u + 2u * lane);
                    }
#pragma unroll
                    for (uint32_t tt = 0; tt < 4; tt++) {
                        const uint32_t t16 = wig * 4u + tt;
                        float2 a = *reinterpret_cast<const float2 *>(stg + t16 * 128u + 2u * lane);
                        float2 b = *reinterpret_cast<const float2 *>(stg + t16 * 128u + 64u + 2u * lane);
                        if (kind < 2) {
                            float ss = a.x * a.x + a.y * a.y + b.x * b.x + b.y * b.y;
#pragma unroll
                            for (uint32_t o = 16; o; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
                            const float inv = 1.0f / sqrtf(ss * (1.0f / 128.0f) + p.f.eps);
                            /* x' = x * inv * w;  (a, b) -> (a c - b s, a s + b c) */
                            const float ax = a.x * inv * w_lo.x, ay = a.y * inv * w_lo.y;
                            const float bx = b.x * inv * w_hi.x, by = b.y * inv * w_hi.y;
                            a.x = fmaf(ax, cs[tt].x, -bx * cs[tt].y);
                            b.x = fmaf(ax, cs[tt].y, bx * cs[tt].x);
                            a.y = fmaf(ay, cs[tt].z, -by * cs[tt].w);
                            b.y = fmaf(ay, cs[tt].w, by * cs[tt].z);
                        }
                        if (page[tt] != Q3_NO_PAGE) {
                            const uint32_t token = m0 + ch * 32u + hf * kStageTokens + t16;
                            __half *dst =
                                kind == 0
                                    ? p.f.q_out + ((size_t)token * p.f.n_q_heads + head) * 128u
                                    : (kind == 1 ? p.f.k_pool : p.f.v_pool) +
                                          (((size_t)head * p.f.num_pages + page[tt]) * Q3_PAGE +
                                           slot[tt]) * 128u;
                            *reinterpret_cast<__half2 *>(dst + 2u * lane) = __floats2half2_rn(a.x, a.y);
                            *reinterpret_cast<__half2 *>(dst + 64u + 2u * lane) = __floats2half2_rn(b.x, b.y);
                        }
                    }
                    mbar_arrive(&misc->stage_empty[group]);
                    stage_use++;
                }
            }
            if (!released) {
                tc_fence_before();
                mbar_arrive(&misc->d_free);
            }
        };

        /* Read this thread's share of tile ti's D, release D, store the rows. */
        auto drain = [&](uint32_t ti) {
            if (FUSED) {
                drain_fused(ti);
                return;
            }
            publish();
            if (alive) alive = wait_or_abort(&misc->acc_full, ti & 1u, misc);
            alive = __all_sync(0xffffffffu, alive);
            if (!alive) return;
            tc_fence_after();
            const uint32_t tile = blockIdx.x + ti * gridDim.x;
            const uint32_t m0 = (tile % n_tok_tiles) * p.NT;
            const uint32_t feature = (tile / n_tok_tiles) * 128u + row;
            uint32_t ch = group;
            for (; ch + kGroups < n_chunks; ch += kGroups) {
                uint32_t v[32];
                tmem_ld32(tmem + lane_base + kColD + ch * 32u, v);
                tmem_wait_ld();
                store_chunk(p, v, m0, ch * 32u, feature);
            }
            /* last chunk of this thread: release D before storing */
            uint32_t v[32];
            const bool mine = ch < n_chunks;
            if (mine) {
                tmem_ld32(tmem + lane_base + kColD + ch * 32u, v);
                tmem_wait_ld();
            }
            tc_fence_before();
            mbar_arrive(&misc->d_free);
            if (mine) store_chunk(p, v, m0, ch * 32u, feature);
        };

        const uint32_t total = n_my * n_kt;
        uint32_t cur_ti = 0, pending = 0xffffffffu, ahead = 0;
        for (uint32_t g = group; g < total && alive; g += kGroups) {
            const uint32_t ti = g / n_kt;
            if (ti != cur_ti) {
                if (pending != 0xffffffffu) drain(pending);   /* (only for very short K) */
                pending = cur_ti;
                ahead = 0;
                cur_ti = ti;
                if (!alive) break;
            }
            const uint32_t sb = g >> 2, j = g & 3u;   /* n_kt is a multiple of 4 */
            if (sb != cur_sb) {
                if (cur_sb != 0xffffffffu) mbar_arrive(&misc->raw_empty[cur_sb % kRawStages]);
                const uint32_t rs = sb % kRawStages;
                alive = wait_or_abort(&misc->raw_full[rs], (sb / kRawStages) & 1u, misc);
                alive = __all_sync(0xffffffffu, alive);
                if (!alive) break;
                cur_sb = sb;
                blk = smem + kSmemRaw + rs * kRawBytes + row * kRawRowBytes;
            }
            uint32_t v[32];
            if constexpr (QT == 4) convert_q4(blk, j, v);
            else convert_q6(blk, j, v);
            /* The store of the previous step has had this step's conversion
             * time to retire: publish it now, then issue this step's store and
             * go on without waiting for it. */
            publish();
            const uint32_t sa = g % kAStages, use = g / kAStages;
            if (use > 0) alive = wait_or_abort(&misc->a_empty[sa], (use - 1) & 1u, misc);
            alive = __all_sync(0xffffffffu, alive);
            if (!alive) break;
            tc_fence_after();
            tmem_st32(tmem + lane_base + kColA + sa * 32u, v);
            stored = sa;
            if (pending != 0xffffffffu && ++ahead == 2) {
                drain(pending);
                pending = 0xffffffffu;
            }
        }
        if (alive) publish();
        if (alive && cur_sb != 0xffffffffu) mbar_arrive(&misc->raw_empty[cur_sb % kRawStages]);
        if (pending != 0xffffffffu) drain(pending);
        if (n_my > 0) drain(n_my - 1);
    }

    tc_fence_before();
    __syncthreads();
    if (threadIdx.x == 0 && misc->abort_flag) atomicOr(p.status, 1u);
    if (warp == 1) tmem_dealloc(tmem, kTmemCols);
}

/* GGUF row-major blocks -> tiled: chunk (feature tile, super-block) holds the 128
 * blocks of its rows back to back. One thread per 16 bytes. */
__global__ void q4k_pack_kernel(const uint4 *__restrict__ src, uint4 *__restrict__ dst,
                                uint32_t n_rows, uint32_t n_super) {
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    const size_t total = (size_t)n_rows * n_super * 9u;
    if (i >= total) return;
    const uint32_t part = (uint32_t)(i % 9u);
    const size_t blk = i / 9u;
    const uint32_t sb = (uint32_t)(blk % n_super);
    const uint32_t row = (uint32_t)(blk / n_super);
    const size_t chunk = (size_t)(row / 128u) * n_super + sb;
    dst[(chunk * 128u + (row % 128u)) * 9u + part] = src[i];
}

/* Q6_K: GGUF row-major 210-byte blocks -> tiled chunks of 128 slots of 224 bytes
 * (block + 14 zero bytes). One thread per block, 2-byte granularity (the source
 * is only 2-byte aligned). */
__global__ void q6k_pack_kernel(const uint16_t *__restrict__ src, uint16_t *__restrict__ dst,
                                uint32_t n_rows, uint32_t n_super) {
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= (size_t)n_rows * n_super) return;
    const uint32_t sb = (uint32_t)(i % n_super);
    const uint32_t row = (uint32_t)(i / n_super);
    const size_t chunk = (size_t)(row / 128u) * n_super + sb;
    const uint16_t *s = src + i * 105u;
    uint16_t *d = dst + (chunk * 128u + (row % 128u)) * 112u;
    for (uint32_t w = 0; w < 105u; w++) d[w] = s[w];
    for (uint32_t w = 105u; w < 112u; w++) d[w] = 0;
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

/* Tokens per CTA (the MMA N, any multiple of 16 up to 256): the whole batch
 * when it fits one tile; otherwise the size that minimises
 * waves x (NT + 32) - a wave lasts as long as its token tile, and the +32
 * stands for the per-tile work that does not shrink with NT (dequantisation,
 * pipeline fill, drain). */
uint32_t choose_token_tile(uint32_t M, uint32_t N, int sm_count) {
    if (M <= kMaxTokens) return (M + 15u) & ~15u;
    uint32_t best = kMaxTokens;
    uint64_t best_cost = ~0ull;
    for (uint32_t nt = kMaxTokens; nt >= 96; nt -= 16) {
        const uint64_t tiles = (uint64_t)((M + nt - 1) / nt) * (N / 128);
        const uint64_t cost = ((tiles + sm_count - 1) / sm_count) * (nt + 32ull);
        if (cost < best_cost) {
            best_cost = cost;
            best = nt;
        }
    }
    return best;
}

bool launch_linear(const q3_q4_linear_geometry *geo, const void *weight, const void *x_f16,
                   size_t tokens, void *out, uint32_t out_type, cudaStream_t stream,
                   char *error, size_t error_len) {
    const uint32_t M = (uint32_t)tokens, N = (uint32_t)geo->N, K = (uint32_t)geo->K;
    /* GGUF-order Q6_K (210-byte blocks cannot be fetched by TMA) and feature
     * counts off the 128 grid: the plain kernel, so that no caller of the
     * reference's entry point is refused where the reference runs. Re-laying a
     * Q6_K weight out once with q3_cuda_q4k_linear_pack gives the tile kernel. */
    if (geo->qtype == Q3_QUANT_Q6_K || (geo->qtype == Q3_QUANT_Q4_K && (N % 128u) != 0))
        return q3_launch_q4k_generic(geo->qtype, weight, x_f16, M, N, K, out, out_type, stream,
                                     error, error_len);
    if (geo->qtype != Q3_QUANT_Q4_K && geo->qtype != Q3_QUANT_Q4_K_TILED &&
        geo->qtype != Q3_QUANT_Q6_K_TILED)
        return q3_fail(error, error_len, "q3_q4_linear: weight is neither Q4_K nor Q6_K");
    if (K % Q3_QUANT_QK_K || N % 128u)
        return q3_fail(error, error_len,
                       "q3_q4_linear: K must be a multiple of 256 and N of 128");
    if (((uintptr_t)weight | (uintptr_t)x_f16 | (uintptr_t)out) & 15u)
        return q3_fail(error, error_len, "q3_q4_linear: pointers must be 16-byte aligned");
    if (geo->qtype == Q3_QUANT_Q4_K && M <= Q3_Q4K_SMALL_BATCH)
        return q3_launch_q4k_small(weight, x_f16, M, N, K, out, out_type, stream, error,
                                   error_len);
    int sms = 148;
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, g.device);
    LinearParams p = {};
    p.out = out;
    p.M = M;
    p.N = N;
    p.K = K;
    p.NT = choose_token_tile(M, N, sms);
    p.out_type = out_type;
    p.status = g.status_dev;
    const bool q6 = geo->qtype == Q3_QUANT_Q6_K_TILED;
    p.w_tiled = geo->qtype != Q3_QUANT_Q4_K ? 1u : 0u;
    CUtensorMap x_map, w_map;
    if (!q3_encode_tmap_2d(&x_map, x_f16, K, M, 64, p.NT, error, error_len)) return false;
    const uint32_t slot = q6 ? Smem<6>::kRowBytes : Smem<4>::kRowBytes;
    const uint64_t row_bytes = (uint64_t)(K / Q3_QUANT_QK_K) * slot;
    if (p.w_tiled) {
        if (!q3_encode_tmap_bytes_2d(&w_map, weight, 256, row_bytes * N / 256, 256,
                                     q6 ? Smem<6>::kTiledRows : Smem<4>::kTiledRows, error,
                                     error_len))
            return false;
    } else if (!q3_encode_tmap_bytes_2d(&w_map, weight, row_bytes, N, slot, 128, error,
                                        error_len)) {
        return false;
    }
    const uint32_t n_tiles = ((M + p.NT - 1) / p.NT) * (N / 128);
    const uint32_t grid = n_tiles < (uint32_t)sms ? n_tiles : (uint32_t)sms;
    if (q6)
        q4k_linear_tc_kernel<6, false><<<grid, kThreads, Smem<6>::kTotal, stream>>>(
            x_map, w_map, w_map, w_map, p);
    else
        q4k_linear_tc_kernel<4, false><<<grid, kThreads, Smem<4>::kTotal, stream>>>(
            x_map, w_map, w_map, w_map, p);
    Q3_LAUNCH_CHECK("q4k_linear_tc launch failed");
    return true;
}

}  // namespace

/* The q/k/v projection with the norm + rotation + page write as its epilogue:
 * one launch over the feature tiles of the three weights (Q4_K, all in the
 * GGUF order or all in the tiled order), a head per tile. */
bool q3_launch_qkv_fused(const q3_qkv_fused_args *a, cudaStream_t stream, char *error,
                         size_t error_len) {
    if (!g.initialized)
        return q3_fail(error, error_len, "q3_q4_linear: not initialized");
    if (a->qtype != Q3_QUANT_Q4_K && a->qtype != Q3_QUANT_Q4_K_TILED)
        return q3_fail(error, error_len,
                       "fused q/k/v projection: weights must be Q4_K (GGUF or tiled order)");
    if (a->hidden == 0 || a->hidden % Q3_QUANT_QK_K)
        return q3_fail(error, error_len,
                       "fused q/k/v projection: hidden size must be a multiple of 256");
    if (((uintptr_t)a->wq | (uintptr_t)a->wk | (uintptr_t)a->wv | (uintptr_t)a->x_f16) & 15u)
        return q3_fail(error, error_len,
                       "fused q/k/v projection: pointers must be 16-byte aligned");
    int sms = 148;
    cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, g.device);
    const uint32_t heads = a->n_q_heads + 2u * a->n_kv_heads;
    LinearParams p = {};
    p.out = nullptr;
    p.M = a->tokens;
    p.N = heads * 128u;
    p.K = a->hidden;
    p.NT = choose_token_tile(p.M, p.N, sms);
    p.out_type = Q3_OUT_F16;
    p.status = g.status_dev;
    p.w_tiled = a->qtype == Q3_QUANT_Q4_K_TILED ? 1u : 0u;
    p.f.seg_end[0] = a->n_q_heads;
    p.f.seg_end[1] = a->n_q_heads + a->n_kv_heads;
    p.f.seg_end[2] = heads;
    p.f.n_q_heads = a->n_q_heads;
    p.f.norm_w = a->norm_w;
    p.f.eps = a->eps;
    p.f.rope_table = (const float2 *)a->rope_table;
    p.f.rope_pos = a->rope_pos;
    p.f.dst_page = a->dst_page;
    p.f.dst_slot = a->dst_slot;
    p.f.q_out = (__half *)a->q_out;
    p.f.k_pool = (__half *)a->k_pool;
    p.f.v_pool = (__half *)a->v_pool;
    p.f.num_pages = a->num_pages;
    CUtensorMap x_map, w_map[3];
    if (!q3_encode_tmap_2d(&x_map, a->x_f16, p.K, p.M, 64, p.NT, error, error_len)) return false;
    const uint32_t slot = Smem<4>::kRowBytes;
    const uint64_t row_bytes = (uint64_t)(p.K / Q3_QUANT_QK_K) * slot;
    const void *w[3] = {a->wq, a->wk, a->wv};
    const uint64_t n[3] = {a->n_q_heads * 128ull, a->n_kv_heads * 128ull, a->n_kv_heads * 128ull};
    for (int i = 0; i < 3; i++) {
        const bool ok = p.w_tiled
                            ? q3_encode_tmap_bytes_2d(&w_map[i], w[i], 256, row_bytes * n[i] / 256,
                                                      256, Smem<4>::kTiledRows, error, error_len)
                            : q3_encode_tmap_bytes_2d(&w_map[i], w[i], row_bytes, n[i], slot, 128,
                                                      error, error_len);
        if (!ok) return false;
    }
    const uint32_t n_tiles = ((p.M + p.NT - 1) / p.NT) * heads;
    const uint32_t grid = n_tiles < (uint32_t)sms ? n_tiles : (uint32_t)sms;
    q4k_linear_tc_kernel<4, true><<<grid, kThreads, Smem<4, true>::kTotal, stream>>>(
        x_map, w_map[0], w_map[1], w_map[2], p);
    Q3_LAUNCH_CHECK("fused q/k/v projection launch failed");
    return true;
}

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
    e = cudaFuncSetAttribute(q4k_linear_tc_kernel<4, false>,
                             cudaFuncAttributeMaxDynamicSharedMemorySize, (int)Smem<4>::kTotal);
    if (e == cudaSuccess)
        e = cudaFuncSetAttribute(q4k_linear_tc_kernel<6, false>,
                                 cudaFuncAttributeMaxDynamicSharedMemorySize,
                                 (int)Smem<6>::kTotal);
    if (e == cudaSuccess)
        e = cudaFuncSetAttribute(q4k_linear_tc_kernel<4, true>,
                                 cudaFuncAttributeMaxDynamicSharedMemorySize,
                                 (int)Smem<4, true>::kTotal);
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
    return token_count <= Q3_MMVQ_MAX_BATCH ? "MMVQ" : "TC";
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
    const bool mmvq = token_count <= Q3_MMVQ_MAX_BATCH && geometry->qtype == Q3_QUANT_Q4_K &&
                      geometry->N % 128 == 0 && (((uintptr_t)weight | (uintptr_t)device_input |
                                                  (uintptr_t)device_output) & 15u) == 0;
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
    if (mmvq) {
        /* the reference's small-batch arithmetic: 8-bit activations, integer dots
         * (its workspace need is below the f16 copy's, checked above) */
        cudaEventRecord(g.ev_mid, st);
        if (!q3_launch_q4k_mmvq(weight, device_input, (uint32_t)token_count,
                                (uint32_t)geometry->N, (uint32_t)geometry->K, device_output,
                                g.workspace, st, error, error_len))
            return false;
        cudaEventRecord(g.ev_end, st);
        g.timed_convert = true;
        return true;
    }
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

extern "C" size_t q3_q4_linear_packed_bytes(const q3_q4_linear_geometry *geometry) {
    if (!geometry || geometry->N <= 0 || geometry->K <= 0) return 0;
    const size_t blocks = (size_t)geometry->N * ((size_t)geometry->K / Q3_QUANT_QK_K);
    if (geometry->qtype == Q3_QUANT_Q4_K) return blocks * Smem<4>::kRowBytes;
    if (geometry->qtype == Q3_QUANT_Q6_K) return blocks * Smem<6>::kRowBytes;
    return 0;
}

extern "C" bool q3_cuda_q4k_linear_pack(const q3_q4_linear_geometry *geometry,
                                        const void *weight, void *tiled,
                                        q3_q4_linear_geometry *tiled_geometry, void *stream,
                                        char *error, size_t error_len) {
    q3_clear_error(error, error_len);
    if (!geometry || !weight || !tiled || !tiled_geometry)
        return q3_fail(error, error_len, "q3_q4_linear: null argument");
    if (geometry->qtype != Q3_QUANT_Q4_K && geometry->qtype != Q3_QUANT_Q6_K)
        return q3_fail(error, error_len,
                       "q3_q4_linear: pack takes a Q4_K or Q6_K weight in GGUF order");
    if (geometry->N <= 0 || geometry->K <= 0 || geometry->N % 128 || geometry->K % Q3_QUANT_QK_K)
        return q3_fail(error, error_len,
                       "q3_q4_linear: K must be a multiple of 256 and N of 128");
    const bool q6 = geometry->qtype == Q3_QUANT_Q6_K;
    if (((uintptr_t)tiled & 15u) || ((uintptr_t)weight & (q6 ? 1u : 15u)))
        return q3_fail(error, error_len, "q3_q4_linear: misaligned pointer");
    const uint32_t n_super = (uint32_t)geometry->K / Q3_QUANT_QK_K;
    if (q6) {
        const size_t total = (size_t)geometry->N * n_super;
        q6k_pack_kernel<<<(unsigned)((total + 255) / 256), 256, 0, (cudaStream_t)stream>>>(
            static_cast<const uint16_t *>(weight), static_cast<uint16_t *>(tiled),
            (uint32_t)geometry->N, n_super);
    } else {
        const size_t total = (size_t)geometry->N * n_super * 9u;
        q4k_pack_kernel<<<(unsigned)((total + 255) / 256), 256, 0, (cudaStream_t)stream>>>(
            static_cast<const uint4 *>(weight), static_cast<uint4 *>(tiled),
            (uint32_t)geometry->N, n_super);
    }
    Q3_LAUNCH_CHECK("q3_q4_linear: pack launch failed");
    *tiled_geometry = *geometry;
    tiled_geometry->qtype = q6 ? Q3_QUANT_Q6_K_TILED : Q3_QUANT_Q4_K_TILED;
    tiled_geometry->weight_bytes = q3_q4_linear_packed_bytes(geometry);
    return true;
}

extern "C" bool q3_q4_linear_plan(uint32_t tokens, uint32_t n_features, uint32_t sm_count,
                                  q3_q4_linear_plan_info *out, char *error,
                                  size_t error_len) {
    q3_clear_error(error, error_len);
    if (!out || tokens == 0 || n_features == 0 || n_features % 128u || sm_count == 0)
        return q3_fail(error, error_len, "q3_q4_linear_plan: invalid argument");
    out->token_tile = choose_token_tile(tokens, n_features, (int)sm_count);
    out->tiles = ((tokens + out->token_tile - 1) / out->token_tile) * (n_features / 128u);
    out->ctas = out->tiles < sm_count ? out->tiles : sm_count;
    out->tiles_per_cta_max = (out->tiles + out->ctas - 1) / out->ctas;
    return true;
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
