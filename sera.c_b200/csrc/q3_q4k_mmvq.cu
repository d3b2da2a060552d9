/* q3_q4k_mmvq.cu - the reference's small-batch arithmetic for the Q4_K linear:
 * activations quantised to 8 bits per 32 elements, integer dot products.
 *
 * For at most 8 tokens the reference takes its MMVQ path (ref:
 * src/q3_q4_linear.cu:140-142, 198-206): the fp32 activations become Q8_1 blocks
 * (per 32 elements d = max|x| / 127 stored as f16, q = round(x / d)) and every
 * output is
 *     sum over blocks of  d * sum_i d8_i * (sc_i * sum q4*q8)
 *                        - dmin * sum_i d8_i * (m_i * sum q8)
 * over the eight 32-element sub-blocks i of a block. This file computes exactly
 * that (its own kernels; only the arithmetic is the reference's), so that
 * q3_cuda_q4k_linear gives the reference's small-batch results up to fp32
 * summation order, and - being integer work on packed nibbles - runs at the
 * speed of the weight bytes instead of the nibble -> f16 conversion.
 *
 * One warp per four feature rows (every 8-bit activation word it reads serves
 * all four). A lane takes one 16-byte piece of a block's quants (8 lanes per
 * block, 4 blocks per warp step): its low nibbles are 16 elements of sub-block
 * 2j, its high nibbles 16 elements of sub-block 2j+1.
 */
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "q3_internal.h"
#include "q3_q4_linear.h"

namespace {

/* x [tokens][K] fp32 -> q [tokens][K] int8, d8 [tokens][K/32] (f16-rounded) and
 * s16 [tokens][K/16]: the sum of the 8-bit values of every 16 elements (the
 * constant part of a Q4_K sub-block multiplies it). One warp per 32 elements. */
__global__ void quantize_q8_kernel(const float *__restrict__ x, int8_t *__restrict__ q,
                                   float *__restrict__ d8, int16_t *__restrict__ s16,
                                   size_t n_blocks) {
    const size_t blk = (size_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (blk >= n_blocks) return;
    const uint32_t lane = threadIdx.x & 31u;
    const float xi = x[blk * 32u + lane];
    float amax = fabsf(xi);
#pragma unroll
    for (uint32_t o = 16; o; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
    const float d = amax / 127.0f;
    const int qi = amax == 0.0f ? 0 : (int)roundf(xi / d);
    q[blk * 32u + lane] = (int8_t)qi;
    int s = qi;
#pragma unroll
    for (uint32_t o = 8; o; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
    if ((lane & 15u) == 0) s16[blk * 2u + (lane >> 4)] = (int16_t)s;
    if (lane == 0) d8[blk] = __half2float(__float2half_rn(d));
}

constexpr uint32_t kRows = 4;    /* feature rows per warp: one read of the activations serves all */

template <uint32_t MTOK>
__global__ void __launch_bounds__(128)
q4k_mmvq_kernel(const uint8_t *__restrict__ weight, const int8_t *__restrict__ q8,
                const float *__restrict__ d8, const int16_t *__restrict__ s16,
                float *__restrict__ out, uint32_t M, uint32_t N, uint32_t K) {
    const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31u;
    const uint32_t n0 = (blockIdx.x * 4u + warp) * kRows;
    if (n0 >= N) return;
    const uint32_t n_super = K / 256u;
    const size_t row_bytes = (size_t)n_super * 144u;
    const uint8_t *row0 = weight + (size_t)n0 * row_bytes;
    const uint32_t c = lane & 7u;            /* 16-byte piece of the block's 128 quant bytes */
    const uint32_t j = c >> 1, span = c & 1u;
    const uint32_t bsh = (j & 1u) * 16u;
    float acc[MTOK][kRows];
#pragma unroll
    for (uint32_t m = 0; m < MTOK; m++)
#pragma unroll
        for (uint32_t r = 0; r < kRows; r++) acc[m][r] = 0.f;

    for (uint32_t b = lane >> 3; b < n_super; b += 4u) {
        uint4 hdr[kRows], qs[kRows];
#pragma unroll
        for (uint32_t r = 0; r < kRows; r++) {
            const uint8_t *blk = row0 + r * row_bytes + (size_t)b * 144u;
            hdr[r] = *reinterpret_cast<const uint4 *>(blk);
            qs[r] = *reinterpret_cast<const uint4 *>(blk + 16u + 16u * c);
        }
        /* per row: d*sc and dmin*m of sub-blocks 2j (low nibbles) and 2j+1 (high) */
        float ds_lo[kRows], ds_hi[kRows], dm_lo[kRows], dm_hi[kRows];
#pragma unroll
        for (uint32_t r = 0; r < kRows; r++) {
            const float d = __half2float(__ushort_as_half((unsigned short)(hdr[r].x & 0xffffu)));
            const float dmin = __half2float(__ushort_as_half((unsigned short)(hdr[r].x >> 16)));
            uint32_t sc_lo, mn_lo, sc_hi, mn_hi;       /* ref: src/q3_quant.c:44-55 */
            if (j < 2) {
                const uint32_t a = hdr[r].y >> bsh, bb = hdr[r].z >> bsh;
                sc_lo = a & 63u;
                mn_lo = bb & 63u;
                sc_hi = (a >> 8) & 63u;
                mn_hi = (bb >> 8) & 63u;
            } else {
                const uint32_t a = hdr[r].y >> bsh, bb = hdr[r].z >> bsh, cc = hdr[r].w >> bsh;
                sc_lo = (cc & 0xFu) | (((a & 0xffu) >> 6) << 4);
                mn_lo = ((cc & 0xffu) >> 4) | (((bb & 0xffu) >> 6) << 4);
                sc_hi = ((cc >> 8) & 0xFu) | ((((a >> 8) & 0xffu) >> 6) << 4);
                mn_hi = (((cc >> 8) & 0xffu) >> 4) | ((((bb >> 8) & 0xffu) >> 6) << 4);
            }
            ds_lo[r] = d * (float)sc_lo;
            ds_hi[r] = d * (float)sc_hi;
            dm_lo[r] = dmin * (float)mn_lo;
            dm_hi[r] = dmin * (float)mn_hi;
        }
        /* first of the 16 low-nibble elements; the high nibbles are 32 further */
        const uint32_t e_lo = b * 256u + 64u * j + 16u * span;
#pragma unroll
        for (uint32_t m = 0; m < MTOK; m++) {
            if (m >= M) break;
            const int8_t *qm = q8 + (size_t)m * K;
            const uint4 ul = *reinterpret_cast<const uint4 *>(qm + e_lo);
            const uint4 uh = *reinterpret_cast<const uint4 *>(qm + e_lo + 32u);
            const uint32_t u_lo[4] = {ul.x, ul.y, ul.z, ul.w};
            const uint32_t u_hi[4] = {uh.x, uh.y, uh.z, uh.w};
            const float *dm = d8 + (size_t)m * (K / 32u) + b * 8u + 2u * j;
            const int16_t *sm = s16 + (size_t)m * (K / 16u) + (e_lo >> 4);
            const float d_lo = dm[0], d_hi = dm[1];
            const float s_lo = (float)sm[0], s_hi = (float)sm[2];
#pragma unroll
            for (uint32_t r = 0; r < kRows; r++) {
                const uint32_t w[4] = {qs[r].x, qs[r].y, qs[r].z, qs[r].w};
                int dot_lo = 0, dot_hi = 0;
#pragma unroll
                for (uint32_t i = 0; i < 4; i++) {
                    dot_lo = __dp4a((int)(w[i] & 0x0F0F0F0Fu), (int)u_lo[i], dot_lo);
                    dot_hi = __dp4a((int)((w[i] >> 4) & 0x0F0F0F0Fu), (int)u_hi[i], dot_hi);
                }
                acc[m][r] += d_lo * (ds_lo[r] * (float)dot_lo - dm_lo[r] * s_lo) +
                             d_hi * (ds_hi[r] * (float)dot_hi - dm_hi[r] * s_hi);
            }
        }
    }
#pragma unroll
    for (uint32_t m = 0; m < MTOK; m++)
#pragma unroll
        for (uint32_t r = 0; r < kRows; r++) {
            float v = acc[m][r];
#pragma unroll
            for (uint32_t o = 16; o; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
            if (lane == 0 && m < M) out[(size_t)m * N + n0 + r] = v;
        }
}

}  // namespace

size_t q3_q4k_mmvq_workspace_bytes(size_t tokens, size_t k) {
    return tokens * k + tokens * (k / 32u) * sizeof(float) + tokens * (k / 16u) * sizeof(int16_t);
}

/* fp32 activations, Q4_K weight in GGUF order, 1..8 tokens, fp32 output.
 * workspace: q3_q4k_mmvq_workspace_bytes(tokens, K) bytes, 16-byte aligned. */
bool q3_launch_q4k_mmvq(const void *weight, const float *x, uint32_t M, uint32_t N, uint32_t K,
                        float *out, void *workspace, cudaStream_t stream, char *error,
                        size_t error_len) {
    int8_t *q8 = static_cast<int8_t *>(workspace);
    float *d8 = reinterpret_cast<float *>(q8 + (size_t)M * K);
    int16_t *s16 = reinterpret_cast<int16_t *>(d8 + (size_t)M * (K / 32u));
    const size_t n_blocks = (size_t)M * K / 32u;
    quantize_q8_kernel<<<(unsigned)((n_blocks + 7) / 8), 256, 0, stream>>>(x, q8, d8, s16,
                                                                          n_blocks);
    Q3_LAUNCH_CHECK("q8 activation quantisation launch failed");
    const unsigned grid = (N + 4u * kRows - 1u) / (4u * kRows);   /* N is a multiple of 128 */
    const uint8_t *w = static_cast<const uint8_t *>(weight);
    if (M == 1)
        q4k_mmvq_kernel<1><<<grid, 128, 0, stream>>>(w, q8, d8, s16, out, M, N, K);
    else if (M <= 2)
        q4k_mmvq_kernel<2><<<grid, 128, 0, stream>>>(w, q8, d8, s16, out, M, N, K);
    else if (M <= 4)
        q4k_mmvq_kernel<4><<<grid, 128, 0, stream>>>(w, q8, d8, s16, out, M, N, K);
    else
        q4k_mmvq_kernel<8><<<grid, 128, 0, stream>>>(w, q8, d8, s16, out, M, N, K);
    Q3_LAUNCH_CHECK("q4k_mmvq launch failed");
    return true;
}
