/* q3_q4k_small.cu - the Q4_K linear for small batches (at most 32 tokens).
 *
 * The tile kernel of q3_q4k_linear.cu is built for batches that keep the
 * tcgen05 pipe busy; for a handful of tokens its per-CTA dequantisation
 * pipeline is the limit (36 us for the q/k/v weight, whose 29.5 MB take 4.5 us
 * of HBM time). This kernel is the weight-bandwidth-bound counterpart (the
 * reference has one too: MMVQ below 9 tokens, src/q3_q4_linear.cu:140-142): every
 * warp owns 8 feature rows and walks all of K; the lanes dequantise their
 * nibbles straight into the B fragment of mma.sync.m16n8k16 (tokens are the M
 * dimension, one 16-token tile), the activations of the current 256 k sit in
 * shared memory for the CTA's four warps, and the next block's bytes are in
 * flight while the current one is multiplied. Measured on the q/k/v weight:
 * 27-29 us for 1-16 tokens against 33-36 us for the tile kernel; both are far
 * from the 4.5 us of HBM time because the nibble -> f16 conversion alone costs
 * about two ALU instructions per weight element (a variant that dealt K out to
 * the warps of a CTA and read the activations through L1 was faster for one
 * token, 23.6 us, and slower for sixteen, 47 us).
 *
 * k is permuted inside each group of 16 (thread t of a quad takes elements
 * 4t..4t+3 for its two B registers) so that a lane reads one 32-bit word of
 * quants per k-step pair; A is read from shared memory with the same
 * permutation, so the product is unchanged.
 * Operand rounding is that of the tile kernel: scale = f16(d*sc), offset =
 * f16(dmin*m), element = f16(fma(q, scale, -offset)), fp32 accumulation.
 */
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "q3_internal.h"
#include "q3_q4_linear.h"

namespace {

constexpr uint32_t kWarps = 4;                 /* 32 features per CTA */
constexpr uint32_t kRowHalfs = 256 + 16;       /* 544-byte rows: conflict-free 8-byte reads */

__device__ __forceinline__ uint32_t deq_lo(uint32_t pair, __half2 scale, __half2 neg_offset) {
    uint32_t b = (pair & 0x000F000Fu) | 0x64006400u;
    const __half2 bias = __half2half2(__ushort_as_half((unsigned short)0x6400));
    __half2 h = __hfma2(__hsub2(*reinterpret_cast<__half2 *>(&b), bias), scale, neg_offset);
    return *reinterpret_cast<uint32_t *>(&h);
}
__device__ __forceinline__ uint32_t deq_hi(uint32_t pair, __half2 scale, __half2 neg_offset) {
    uint32_t b = (pair & 0x00F000F0u) | 0x54005400u;
    const __half2 bias = __half2half2(__ushort_as_half((unsigned short)0x5400));
    __half2 h = __hfma2(__hsub2(*reinterpret_cast<__half2 *>(&b), bias), scale, neg_offset);
    return *reinterpret_cast<uint32_t *>(&h);
}

__device__ __forceinline__ void mma16816(float *c, const uint32_t *a, uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 "
        "{%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, {%0, %1, %2, %3};"
        : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

/* The 12 words a lane needs from one Q4_K block of its row: the 16-byte header
 * and, per 32-byte quant group j, the words at bytes 4t and 16 + 4t. */
struct BlockWords {
    uint4 hdr;
    uint32_t q[8];
};

__device__ __forceinline__ BlockWords load_block(const uint8_t *blk, uint32_t t) {
    BlockWords w;
    w.hdr = *reinterpret_cast<const uint4 *>(blk);
#pragma unroll
    for (uint32_t j = 0; j < 4; j++) {
        w.q[2 * j] = *reinterpret_cast<const uint32_t *>(blk + 16u + 32u * j + 4u * t);
        w.q[2 * j + 1] = *reinterpret_cast<const uint32_t *>(blk + 32u + 32u * j + 4u * t);
    }
    return w;
}

__device__ __forceinline__ void cp_async16(void *smem, const void *gmem) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(
                     (uint32_t)__cvta_generic_to_shared(smem)),
                 "l"(gmem)
                 : "memory");
}
__device__ __forceinline__ void cp_async_wait_all() {
    asm volatile("cp.async.wait_all;" ::: "memory");
}

/* One CTA = 32 feature rows (8 per warp); every warp walks all of K. The token
 * rows of the current 256 k are staged in shared memory once per CTA (double
 * buffered, cp.async one block ahead) and the next block's weight words are in
 * registers while the current one is multiplied. */
template <uint32_t MT>
__global__ void __launch_bounds__(kWarps * 32)
q4k_small_batch_kernel(const uint8_t *__restrict__ weight, const __half *__restrict__ x,
                       void *__restrict__ out, uint32_t M, uint32_t N, uint32_t K,
                       uint32_t out_type) {
    __shared__ __align__(16) __half xs[2][MT * 16][kRowHalfs];
    const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31u;
    const uint32_t g = lane >> 2, t = lane & 3u;
    const uint32_t n_super = K / 256u;
    const uint32_t n0 = blockIdx.x * (kWarps * 8u) + warp * 8u;
    const uint8_t *wrow = weight + (size_t)(n0 + g) * n_super * 144u;

    /* rows beyond the batch stay zero in both buffers */
    for (uint32_t i = threadIdx.x; i < 2u * MT * 16u * (kRowHalfs / 8u); i += blockDim.x)
        reinterpret_cast<uint4 *>(&xs[0][0][0])[i] = make_uint4(0, 0, 0, 0);
    __syncthreads();
    auto stage_x = [&](uint32_t sb) {
        /* 32 16-byte pieces per token row */
        for (uint32_t i = threadIdx.x; i < M * 32u; i += blockDim.x) {
            const uint32_t m = i >> 5, piece = i & 31u;
            cp_async16(&xs[sb & 1u][m][piece * 8u], x + (size_t)m * K + sb * 256u + piece * 8u);
        }
    };
    stage_x(0);
    BlockWords cur = load_block(wrow, t);

    float acc[MT][4];
#pragma unroll
    for (uint32_t mt = 0; mt < MT; mt++)
#pragma unroll
        for (uint32_t i = 0; i < 4; i++) acc[mt][i] = 0.f;

    for (uint32_t sb = 0; sb < n_super; sb++) {
        cp_async_wait_all();
        __syncthreads();                       /* chunk sb is in xs[sb & 1]; the other buffer is free */
        BlockWords nxt = cur;
        if (sb + 1 < n_super) {
            stage_x(sb + 1);
            nxt = load_block(wrow + (size_t)(sb + 1) * 144u, t);
        }
        const float dd = __half2float(__ushort_as_half((unsigned short)(cur.hdr.x & 0xffffu)));
        const float dm = __half2float(__ushort_as_half((unsigned short)(cur.hdr.x >> 16)));
        const __half(*xb)[kRowHalfs] = xs[sb & 1u];
#pragma unroll
        for (uint32_t j = 0; j < 4; j++) {
            /* sub-blocks 2j (low nibbles) and 2j+1 (high nibbles); scales bytes
             * 0-3 = hdr.y, 4-7 = hdr.z, 8-11 = hdr.w (ref: src/q3_quant.c:44-55) */
            const uint32_t bsh = (j & 1u) * 16u;
            uint32_t sc_lo, mn_lo, sc_hi, mn_hi;
            if (j < 2) {
                const uint32_t a = cur.hdr.y >> bsh, b = cur.hdr.z >> bsh;
                sc_lo = a & 63u;
                mn_lo = b & 63u;
                sc_hi = (a >> 8) & 63u;
                mn_hi = (b >> 8) & 63u;
            } else {
                const uint32_t a = cur.hdr.y >> bsh, b = cur.hdr.z >> bsh, c = cur.hdr.w >> bsh;
                sc_lo = (c & 0xFu) | (((a & 0xffu) >> 6) << 4);
                mn_lo = ((c & 0xffu) >> 4) | (((b & 0xffu) >> 6) << 4);
                sc_hi = ((c >> 8) & 0xFu) | ((((a >> 8) & 0xffu) >> 6) << 4);
                mn_hi = (((c >> 8) & 0xffu) >> 4) | ((((b >> 8) & 0xffu) >> 6) << 4);
            }
            const __half2 s_lo = __float2half2_rn(dd * (float)sc_lo);
            const __half2 s_hi = __float2half2_rn(dd * (float)sc_hi);
            const __half2 o_lo = __hneg2(__float2half2_rn(dm * (float)mn_lo));
            const __half2 o_hi = __hneg2(__float2half2_rn(dm * (float)mn_hi));
#pragma unroll
            for (uint32_t span = 0; span < 2; span++) {
                const uint32_t w = cur.q[2 * j + span];
                const uint32_t p01 = __byte_perm(w, 0u, 0x4140);
                const uint32_t p23 = __byte_perm(w, 0u, 0x4342);
                /* quant bytes 16*span + 4t .. +3: low nibbles are elements
                 * 64j + 16*span + 4t .., high nibbles the same + 32 */
                const uint32_t k_lo = 64u * j + 16u * span + 4u * t;
#pragma unroll
                for (uint32_t half = 0; half < 2; half++) {
                    const uint32_t b0 = half ? deq_hi(p01, s_hi, o_hi) : deq_lo(p01, s_lo, o_lo);
                    const uint32_t b1 = half ? deq_hi(p23, s_hi, o_hi) : deq_lo(p23, s_lo, o_lo);
                    const uint32_t kk = k_lo + 32u * half;
#pragma unroll
                    for (uint32_t mt = 0; mt < MT; mt++) {
                        const uint2 r0 = *reinterpret_cast<const uint2 *>(&xb[mt * 16u + g][kk]);
                        const uint2 r1 =
                            *reinterpret_cast<const uint2 *>(&xb[mt * 16u + g + 8u][kk]);
                        const uint32_t a[4] = {r0.x, r1.x, r0.y, r1.y};
                        mma16816(acc[mt], a, b0, b1);
                    }
                }
            }
        }
        cur = nxt;
    }

#pragma unroll
    for (uint32_t mt = 0; mt < MT; mt++)
#pragma unroll
        for (uint32_t r = 0; r < 2; r++) {
            const uint32_t token = mt * 16u + g + 8u * r;
            if (token >= M) continue;
            const size_t off = (size_t)token * N + n0 + 2u * t;
            const float c0 = acc[mt][2 * r], c1 = acc[mt][2 * r + 1];
            if (out_type == Q3_OUT_F32) {
                *reinterpret_cast<float2 *>(static_cast<float *>(out) + off) = make_float2(c0, c1);
            } else if (out_type == Q3_OUT_BF16) {
                *reinterpret_cast<__nv_bfloat162 *>(static_cast<__nv_bfloat16 *>(out) + off) =
                    __floats2bfloat162_rn(c0, c1);
            } else {
                *reinterpret_cast<__half2 *>(static_cast<__half *>(out) + off) =
                    __floats2half2_rn(c0, c1);
            }
        }
}

}  // namespace

/* Q4_K weight in GGUF order, 1..16 tokens (the template also covers 17..32). */
bool q3_launch_q4k_small(const void *weight, const void *x_f16, uint32_t M, uint32_t N,
                         uint32_t K, void *out, uint32_t out_type, cudaStream_t stream,
                         char *error, size_t error_len) {
    const dim3 grid(N / (kWarps * 8u));
    if (M <= 16)
        q4k_small_batch_kernel<1><<<grid, kWarps * 32, 0, stream>>>(
            static_cast<const uint8_t *>(weight), static_cast<const __half *>(x_f16), out, M, N,
            K, out_type);
    else
        q4k_small_batch_kernel<2><<<grid, kWarps * 32, 0, stream>>>(
            static_cast<const uint8_t *>(weight), static_cast<const __half *>(x_f16), out, M, N,
            K, out_type);
    Q3_LAUNCH_CHECK("q4k_small_batch launch failed");
    return true;
}
