/* q3_lmhead.cu - last-row gather and selected-row LM head (see q3_lmhead.h).
 *
 * The work is tiny (branches x candidates rows of 2.9-4.2 KB against one
 * hidden vector each), so the design goal is one launch and coalesced reads:
 * one CTA per branch, one warp per candidate at a time, a lane per 32-element
 * sub-block of the row; the branch's hidden vector is staged in shared memory
 * once and reused by all candidates.
 */
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <math.h>
#include <stdint.h>

#include "q3_internal.h"
#include "q3_lmhead.h"

namespace {

constexpr uint32_t kWarps = 8;
constexpr uint32_t kQ4Block = 144, kQ6Block = 210;

__device__ __forceinline__ float half_bits(const uint8_t *p) {
    return __half2float(__ushort_as_half((unsigned short)(p[0] | (p[1] << 8))));
}

/* 32 consecutive elements (sub-block `sub` of 8) of one Q4_K block times h
 * (ref: src/q3_quant.c:44-76). */
__device__ __forceinline__ float dot_q4_sub(const uint8_t *blk, uint32_t sub, const float *h) {
    const float d = half_bits(blk), dmin = half_bits(blk + 2);
    const uint8_t *s = blk + 4;
    uint32_t sc, mn;
    if (sub < 4) {
        sc = s[sub] & 63u;
        mn = s[sub + 4] & 63u;
    } else {
        sc = (s[sub + 4] & 0xFu) | ((s[sub - 4] >> 6) << 4);
        mn = (s[sub + 4] >> 4) | ((s[sub] >> 6) << 4);
    }
    const float d1 = d * (float)sc, m1 = dmin * (float)mn;
    const uint8_t *q = blk + 16 + 32u * (sub >> 1);
    const uint32_t shift = (sub & 1u) * 4u;
    float acc = 0.f;
#pragma unroll 8
    for (uint32_t l = 0; l < 32; l++)
        acc += (d1 * (float)((q[l] >> shift) & 0xFu) - m1) * h[l];
    return acc;
}

/* 32 consecutive elements (unit `sub` of 8: half = sub / 4, group = sub % 4) of
 * one Q6_K block times h (ref: src/q3_quant.c:78-103). */
__device__ __forceinline__ float dot_q6_sub(const uint8_t *blk, uint32_t sub, const float *h) {
    const uint32_t half = sub >> 2, grp = sub & 3u;
    const uint8_t *ql = blk + 64u * half + ((grp & 1u) ? 32u : 0u);
    const uint8_t *qh = blk + 128 + 32u * half;
    const int8_t *sc = reinterpret_cast<const int8_t *>(blk + 192 + 8u * half + 2u * grp);
    const float d = half_bits(blk + 208);
    const uint32_t nib = (grp >> 1) * 4u, hs = grp * 2u;
    float acc = 0.f;
#pragma unroll 8
    for (uint32_t l = 0; l < 32; l++) {
        const int q = (int)(((ql[l] >> nib) & 0xFu) | (((qh[l] >> hs) & 3u) << 4)) - 32;
        acc += d * (float)sc[l >> 4] * (float)q * h[l];
    }
    return acc;
}

__global__ void gather_last_rows_kernel(const float *__restrict__ src,
                                        const uint32_t *__restrict__ branch_offsets,
                                        uint32_t hidden, float *__restrict__ out) {
    const uint32_t b = blockIdx.x;
    const uint32_t last = branch_offsets[b + 1] - 1u;
    const float4 *row = reinterpret_cast<const float4 *>(src + (size_t)last * hidden);
    float4 *dst = reinterpret_cast<float4 *>(out + (size_t)b * hidden);
    for (uint32_t i = threadIdx.x; i < hidden / 4; i += blockDim.x) dst[i] = row[i];
}

/* One CTA per branch. row_of_branch: NULL -> hidden is [branches][hidden_size];
 * else the packed offsets (the branch's row is offsets[b+1]-1). */
__global__ void __launch_bounds__(kWarps * 32)
candidate_head_kernel(const float *__restrict__ hidden, const uint32_t *__restrict__ offsets,
                      const uint8_t *__restrict__ weight, uint32_t qtype, uint32_t hidden_size,
                      uint32_t vocab_size, const uint32_t *__restrict__ candidate_ids,
                      uint32_t candidate_count, float *__restrict__ logits,
                      uint32_t *__restrict__ best) {
    extern __shared__ float h_sm[];
    const uint32_t b = blockIdx.x;
    const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31u;
    const size_t row = offsets ? (size_t)(offsets[b + 1] - 1u) : (size_t)b;
    const float4 *src = reinterpret_cast<const float4 *>(hidden + row * hidden_size);
    for (uint32_t i = threadIdx.x; i < hidden_size / 4; i += blockDim.x)
        reinterpret_cast<float4 *>(h_sm)[i] = src[i];
    __syncthreads();
    const uint32_t n_blocks = hidden_size / 256u;
    const uint32_t block_bytes = qtype == 12u ? kQ4Block : kQ6Block;
    for (uint32_t c = warp; c < candidate_count; c += kWarps) {
        const uint32_t id = candidate_ids[(size_t)b * candidate_count + c];
        float acc = 0.f;
        if (id < vocab_size) {
            const uint8_t *wrow = weight + (size_t)id * n_blocks * block_bytes;
            for (uint32_t u = lane; u < n_blocks * 8u; u += 32u) {
                const uint8_t *blk = wrow + (size_t)(u >> 3) * block_bytes;
                const float *h = h_sm + u * 32u;
                acc += qtype == 12u ? dot_q4_sub(blk, u & 7u, h) : dot_q6_sub(blk, u & 7u, h);
            }
        } else {
            acc = NAN;
        }
        for (uint32_t off = 16; off; off >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, off);
        if (lane == 0) logits[(size_t)b * candidate_count + c] = acc;
    }
    if (best) {
        __syncthreads();
        if (threadIdx.x == 0) {
            uint32_t arg = 0;
            float top = logits[(size_t)b * candidate_count];
            for (uint32_t c = 1; c < candidate_count; c++) {
                const float v = logits[(size_t)b * candidate_count + c];
                if (v > top) {
                    top = v;
                    arg = c;
                }
            }
            best[b] = arg;
        }
    }
}

bool launch_head(const float *hidden, const uint32_t *offsets, const void *weight,
                 uint32_t qtype, uint32_t hidden_size, uint32_t vocab_size,
                 const uint32_t *candidate_ids, uint32_t candidate_count,
                 uint32_t branch_count, float *logits, uint32_t *best, void *stream,
                 const char *who, char *error, size_t error_len) {
    if (!hidden || !weight || !candidate_ids || !logits || branch_count == 0 ||
        candidate_count == 0 || hidden_size == 0 || hidden_size % 256u || vocab_size == 0) {
        if (error && error_len) snprintf(error, error_len, "%s: invalid argument", who);
        return false;
    }
    if (qtype != 12u && qtype != 14u) {
        if (error && error_len)
            snprintf(error, error_len, "%s: weight is neither Q4_K nor Q6_K", who);
        return false;
    }
    const size_t smem = (size_t)hidden_size * sizeof(float);
    if (smem > 48 * 1024) {
        if (error && error_len)
            snprintf(error, error_len, "%s: hidden_size above 12288 is not supported", who);
        return false;
    }
    candidate_head_kernel<<<branch_count, kWarps * 32, smem, (cudaStream_t)stream>>>(
        hidden, offsets, static_cast<const uint8_t *>(weight), qtype, hidden_size, vocab_size,
        candidate_ids, candidate_count, logits, best);
    Q3_LAUNCH_CHECK("candidate head launch failed");
    return true;
}

}  // namespace

extern "C" bool q3_cuda_gather_last_rows(const float *src, const uint32_t *branch_offsets,
                                         uint32_t branch_count, uint32_t hidden, float *out,
                                         void *stream, char *error, size_t error_len) {
    q3_clear_error(error, error_len);
    if (!src || !branch_offsets || !out || branch_count == 0 || hidden == 0 || hidden % 4u)
        return q3_fail(error, error_len, "q3_cuda_gather_last_rows: invalid argument");
    gather_last_rows_kernel<<<branch_count, 256, 0, (cudaStream_t)stream>>>(src, branch_offsets,
                                                                           hidden, out);
    Q3_LAUNCH_CHECK("gather_last_rows launch failed");
    return true;
}

extern "C" bool q3_cuda_candidate_logits_batched(
    const float *hidden_per_branch, const void *weight, uint32_t qtype, uint32_t hidden_size,
    uint32_t vocab_size, const uint32_t *candidate_ids, uint32_t candidate_count,
    uint32_t branch_count, float *logits, void *stream, char *error, size_t error_len) {
    q3_clear_error(error, error_len);
    return launch_head(hidden_per_branch, NULL, weight, qtype, hidden_size, vocab_size,
                       candidate_ids, candidate_count, branch_count, logits, NULL, stream,
                       "q3_cuda_candidate_logits_batched", error, error_len);
}

extern "C" bool q3_cuda_candidate_head(const float *hidden_rows, const uint32_t *branch_offsets,
                                       const void *weight, uint32_t qtype,
                                       uint32_t hidden_size, uint32_t vocab_size,
                                       const uint32_t *candidate_ids, uint32_t candidate_count,
                                       uint32_t branch_count, float *logits, uint32_t *best,
                                       void *stream, char *error, size_t error_len) {
    q3_clear_error(error, error_len);
    if (!branch_offsets)
        return q3_fail(error, error_len, "q3_cuda_candidate_head: invalid argument");
    return launch_head(hidden_rows, branch_offsets, weight, qtype, hidden_size, vocab_size,
                       candidate_ids, candidate_count, branch_count, logits, best, stream,
                       "q3_cuda_candidate_head", error, error_len);
}
