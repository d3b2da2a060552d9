/* q3_q4k_generic.cu - plain (non-TMA) quantised linear for the weights and
 * shapes the tile kernels do not take, so that a caller of the reference's
 * q3_cuda_q4k_linear is never refused where the reference runs
 * (ref: src/q3_q4_linear.cu:149-228 accepts Q4_K and Q6_K in GGUF order at any
 * feature count, on its vector and its matrix path):
 *   - Q6_K in GGUF order (210-byte blocks are not 16-byte multiples, so TMA
 *     cannot fetch them; some attn_v / ffn_down tensors of a Q4_K_M file and
 *     output.weight are Q6_K),
 *   - Q4_K with a feature count that is not a multiple of 128.
 * One warp per output feature, eight tokens per pass; a lane dequantises a
 * 32-element sub-block (Q4_K) or 32 elements of a 128-element half (Q6_K) in
 * fp32, exactly the block semantics of ref: src/q3_quant.c:18-103. Bound by
 * the weight bytes at small batches; at large batches the weight is re-read
 * once per eight tokens (from L2), which is what makes it the slow path.
 */
#include "q3_internal.h"
#include "q3_q4_linear.h"

namespace {

constexpr uint32_t kTok = 8;    /* tokens per pass */

__device__ __forceinline__ void q4k_scale_min(const uint8_t *scales, uint32_t j, uint32_t &sc,
                                              uint32_t &mn) {
    if (j < 4) {
        sc = scales[j] & 63u;
        mn = scales[j + 4] & 63u;
    } else {
        sc = (scales[j + 4] & 0x0Fu) | ((scales[j - 4] >> 6) << 4);
        mn = (scales[j + 4] >> 4) | ((scales[j] >> 6) << 4);
    }
}

/* out[token][n] = sum_k W[n][k] x[token][k]; x f16 [M][K]; W rows of K/256 blocks. */
template <int QT>
__global__ void __launch_bounds__(256)
q4k_generic_kernel(const uint8_t *__restrict__ w, const __half *__restrict__ x, uint32_t M,
                   uint32_t N, uint32_t K, void *__restrict__ out, uint32_t out_type) {
    const uint32_t n = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    const uint32_t lane = threadIdx.x & 31u;
    if (n >= N) return;
    constexpr uint32_t kBlock = QT == 4 ? 144u : 210u;
    const uint32_t nb = K / 256u;
    const uint8_t *row = w + (size_t)n * nb * kBlock;
    for (uint32_t t0 = 0; t0 < M; t0 += kTok) {
        float acc[kTok];
#pragma unroll
        for (uint32_t t = 0; t < kTok; t++) acc[t] = 0.f;
        /* 8 groups of 32 elements per block; lane = (block parity.., group): a warp
         * walks 4 blocks at a time, lane / 8 = block within the four, lane % 8 = group */
        for (uint32_t b0 = 0; b0 < nb; b0 += 4) {
            const uint32_t b = b0 + (lane >> 3), gidx = lane & 7u;
            if (b >= nb) continue;
            const uint8_t *blk = row + (size_t)b * kBlock;
            float wv[32];
            if (QT == 4) {
                /* ref: src/q3_quant.c dequantize_row_q4_K: d, dmin (f16), 12 scale bytes,
                 * 128 quant bytes; group g of 32: low nibbles of bytes 32*(g/2).. for even
                 * g, high nibbles for odd g */
                const float d = __half2float(*reinterpret_cast<const __half *>(blk));
                const float dmin = __half2float(*reinterpret_cast<const __half *>(blk + 2));
                uint32_t sc, mn;
                q4k_scale_min(blk + 4, gidx, sc, mn);
                const float ds = d * (float)sc, dm = dmin * (float)mn;
                const uint8_t *qs = blk + 16 + 32u * (gidx >> 1);
#pragma unroll
                for (uint32_t i = 0; i < 32; i++) {
                    const uint32_t qv = (gidx & 1u) ? (qs[i] >> 4) : (qs[i] & 0x0Fu);
                    wv[i] = ds * (float)qv - dm;
                }
            } else {
                /* ref: src/q3_quant.c dequantize_row_q6_K: ql[128], qh[64], scales[16]
                 * (int8), d (f16). Half hh = g/4 of 128 elements; within it quarter
                 * qq = g%4 covers elements 32*qq..: ql byte l (+32 for qq odd), low
                 * nibble for qq < 2 else high; qh bits 2*qq; scale index 8*hh + 2*qq + l/16 */
                const uint32_t hh = gidx >> 2, qq = gidx & 3u;
                const uint8_t *ql = blk + 64u * hh + ((qq & 1u) ? 32u : 0u);
                const uint8_t *qh = blk + 128 + 32u * hh;
                const int8_t *scs = reinterpret_cast<const int8_t *>(blk + 192) + 8u * hh + 2u * qq;
                const float d = __half2float(*reinterpret_cast<const __half *>(blk + 208));
#pragma unroll
                for (uint32_t l = 0; l < 32; l++) {
                    const uint32_t lo = (qq < 2) ? (ql[l] & 0x0Fu) : (ql[l] >> 4);
                    const uint32_t hi = (qh[l] >> (2u * qq)) & 3u;
                    const int qv = (int)(lo | (hi << 4)) - 32;
                    wv[l] = d * (float)scs[l >> 4] * (float)qv;
                }
            }
            const uint32_t k0 = b * 256u + gidx * 32u;
#pragma unroll
            for (uint32_t t = 0; t < kTok; t++) {
                if (t0 + t >= M) break;
                const uint4 *xp = reinterpret_cast<const uint4 *>(x + (size_t)(t0 + t) * K + k0);
                float s = 0.f;
#pragma unroll
                for (uint32_t c = 0; c < 4; c++) {
                    const uint4 u = xp[c];
                    const __half2 *h2 = reinterpret_cast<const __half2 *>(&u);
#pragma unroll
                    for (uint32_t e = 0; e < 4; e++) {
                        const float2 f = __half22float2(h2[e]);
                        s += wv[c * 8 + 2 * e] * f.x + wv[c * 8 + 2 * e + 1] * f.y;
                    }
                }
                acc[t] += s;
            }
        }
#pragma unroll
        for (uint32_t t = 0; t < kTok; t++) {
            float v = acc[t];
#pragma unroll
            for (uint32_t o = 16; o; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
            if (lane == 0 && t0 + t < M) {
                const size_t idx = (size_t)(t0 + t) * N + n;
                if (out_type == Q3_OUT_F32) reinterpret_cast<float *>(out)[idx] = v;
                else if (out_type == Q3_OUT_BF16)
                    reinterpret_cast<__nv_bfloat16 *>(out)[idx] = __float2bfloat16_rn(v);
                else reinterpret_cast<__half *>(out)[idx] = __float2half_rn(v);
            }
        }
    }
}

}  // namespace

bool q3_launch_q4k_generic(uint32_t qtype, const void *weight, const void *x_f16, uint32_t M,
                           uint32_t N, uint32_t K, void *out, uint32_t out_type,
                           cudaStream_t stream, char *error, size_t error_len) {
    if (K % 256u) return q3_fail(error, error_len, "q3_q4_linear: K must be a multiple of 256");
    if ((uintptr_t)x_f16 & 15u)
        return q3_fail(error, error_len, "q3_q4_linear: activations must be 16-byte aligned");
    const unsigned grid = (unsigned)(((uint64_t)N * 32 + 255) / 256);
    if (qtype == Q3_QUANT_Q4_K)
        q4k_generic_kernel<4><<<grid, 256, 0, stream>>>((const uint8_t *)weight,
                                                        (const __half *)x_f16, M, N, K, out,
                                                        out_type);
    else
        q4k_generic_kernel<6><<<grid, 256, 0, stream>>>((const uint8_t *)weight,
                                                        (const __half *)x_f16, M, N, K, out,
                                                        out_type);
    Q3_LAUNCH_CHECK("q4k_generic launch failed");
    return true;
}
