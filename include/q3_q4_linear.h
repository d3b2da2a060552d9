/* q3_q4_linear.h - C ABI of the resident Q4_K linear (the projections on
 * either side of the attention path), rebuilt for B200 (sm_100a).
 *
 * Part 1 keeps the reference's interface symbol for symbol, so its callers
 * (run_layer / run_layer_packed, src/q3_forward.cu:1214-1242 and :1289-1296)
 * and its test (tests/test_q3_q4_linear.cu) link unchanged:
 *   ref: src/q3_q4_linear.h:24-119.
 * Where the reference quantises the fp32 activations to Q8_1 and runs integer
 * MMQ/MMVQ kernels, this library converts them to f16 and runs one tensor-core
 * kernel (tcgen05, fp32 accumulation in tensor memory) that dequantises the
 * Q4_K blocks into f16 operands held in tensor memory; the result is closer to
 * the exact fp32 product than the reference's (no activation quantisation).
 *
 * Part 2 is native: f16 activations in, bf16/f16/fp32 out, no conversion pass.
 *
 * Conventions as in the reference: device pointers, `void *stream` is a
 * cudaStream_t, nothing synchronises or allocates in the warm path, `bool` +
 * caller-supplied error buffer (cleared on entry), unsupported input fails
 * loudly - there is no slow fallback.
 */
#ifndef Q3_Q4_LINEAR_B200_H
#define Q3_Q4_LINEAR_B200_H

#include <stdbool.h>
#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* GGML type ids of the weights (ref: src/q3_quant.h:19-22). Q4_K runs from
 * the GGUF block order or from the tiled order of q3_cuda_q4k_linear_pack; Q6_K
 * (210-byte blocks, which TMA cannot fetch) only from the tiled order. */
enum { Q3_QUANT_Q4_K = 12, Q3_QUANT_Q6_K = 14 };
#define Q3_QUANT_QK_K 256
#define Q3_QUANT_Q4_K_BLOCK_BYTES 144

/* ---- part 1: the reference's surface (ref: src/q3_q4_linear.h) ---------- */

/* ref: src/q3_q4_linear.h:35-47 */
typedef struct {
    double total_ms;
    double activation_quant_ms;   /* here: the fp32 -> f16 conversion pass */
    double kernel_ms;
    uint64_t weight_bytes;
    uint64_t activation_read_bytes;
    uint64_t activation_write_bytes;
    uint64_t kernel_launches;
    uint64_t cuda_allocations;
    uint64_t host_syncs;
} q3_q4_linear_stats;

/* weight = [N, K] (N rows of K/256 blocks), input = [M, K], output = [M, N]
 * row-major: out[token * N + feature] (ref: src/q3_q4_linear.h:49-58 and the
 * note at src/q3_q4_linear.cu:178-183). */
typedef struct {
    int32_t M;
    int32_t N;
    int32_t K;
    uint32_t qtype;
    uint64_t weight_bytes;
} q3_q4_linear_geometry;

/* GGUF dim[0] = K (row length), dim[1] = N (row count); K must be a multiple
 * of 256 (ref: src/q3_q4_linear.h:60-72, src/q3_q4_linear.cu:47-91). */
bool q3_q4_linear_bind_geometry(uint32_t qtype, uint32_t gguf_rows_dim0,
                                uint32_t gguf_cols_dim1, q3_q4_linear_geometry *out,
                                char *error, size_t error_len);

/* One-time set-up per process: device, kernel attributes, the size of the
 * scratch arena (f16 copy of the largest activation batch). Repeated calls
 * only grow the requirement (ref: src/q3_q4_linear.h:74-80). */
bool q3_cuda_q4k_linear_init(int device, size_t max_tokens, int64_t max_features,
                             int64_t max_k, char *error, size_t error_len);
size_t q3_cuda_q4k_linear_workspace_bytes(void);
bool q3_cuda_q4k_linear_set_workspace(void *device_ptr, size_t bytes, char *error,
                                      size_t error_len);
/* Which arithmetic q3_cuda_q4k_linear applies to a batch. The reference answers
 * "MMVQ" (at most 8 tokens) or "MMQ"; this library answers "MMVQ" for the same
 * batches - the reference's own small-batch arithmetic: activations quantised
 * to 8 bits per 32 elements, integer dot products, bound by the weight bytes -
 * and "TC" above (f16 operands on the tensor cores). q3_cuda_q4k_linear_f16
 * never quantises activations: at most 16 tokens take an mma.sync kernel,
 * larger batches the tcgen05 tile kernel. */
const char *q3_cuda_q4k_linear_path_for_batch(size_t token_count);

/* Q4_K weight x fp32 activation -> fp32 output (ref: src/q3_q4_linear.h:93-108). */
bool q3_cuda_q4k_linear(const q3_q4_linear_geometry *geometry, const void *weight,
                        const float *device_input, size_t token_count,
                        float *device_output, void *stream, q3_q4_linear_stats *stats,
                        char *error, size_t error_len);
/* After the caller synchronised the stream (ref: src/q3_q4_linear.h:114-118). */
void q3_cuda_q4k_linear_read_stats(q3_q4_linear_stats *stats, void *stream);

/* ---- part 2: native entry (no counterpart in the reference) -------------- */

enum { Q3_OUT_F32 = 0, Q3_OUT_BF16 = 1, Q3_OUT_F16 = 2 };

/* One-time re-layout of a resident Q4_K or Q6_K weight: the 128 blocks that one
 * 128-feature tile needs for one 256-wide k range are stored back to back
 * (Q4_K: 128 x 144 = 18432 contiguous bytes; Q6_K: each 210-byte block padded
 * to 224, 28672 bytes), tile by tile, so that the kernel fetches them with one
 * dense TMA box. `tiled` must hold q3_q4_linear_packed_bytes(geometry) bytes;
 * `tiled_geometry` receives the geometry to pass with the tiled copy (qtype
 * Q3_QUANT_Q4_K_TILED / Q3_QUANT_Q6_K_TILED). Both linear entry points accept
 * Q4_K in either order and Q6_K in the tiled order only. The source may be
 * freed afterwards. */
#define Q3_QUANT_Q4_K_TILED (12u | (1u << 16))
#define Q3_QUANT_Q6_K_TILED (14u | (1u << 16))
size_t q3_q4_linear_packed_bytes(const q3_q4_linear_geometry *geometry);
bool q3_cuda_q4k_linear_pack(const q3_q4_linear_geometry *geometry, const void *weight,
                             void *tiled, q3_q4_linear_geometry *tiled_geometry,
                             void *stream, char *error, size_t error_len);

/* x: f16 [tokens][K] row-major (16-byte aligned); out: [tokens][N] of out_type.
 * One kernel launch, no workspace. q3_cuda_q4k_linear_init must have run on
 * this device. */
bool q3_cuda_q4k_linear_f16(const q3_q4_linear_geometry *geometry, const void *weight,
                            const void *x_f16, size_t token_count, void *out,
                            uint32_t out_type, void *stream, char *error,
                            size_t error_len);

/* Host-only: the launch shape the linear picks for a batch (tokens per CTA =
 * the MMA N dimension, a multiple of 16 up to 256; 128 features per tile;
 * persistent CTAs, tile t -> CTA t % ctas). Pure arithmetic, no CUDA call. */
typedef struct {
    uint32_t token_tile;
    uint32_t tiles;
    uint32_t ctas;
    uint32_t tiles_per_cta_max;
} q3_q4_linear_plan_info;
bool q3_q4_linear_plan(uint32_t tokens, uint32_t n_features, uint32_t sm_count,
                       q3_q4_linear_plan_info *out, char *error, size_t error_len);

/* Device status word of the linear kernels (bit 0: a bounded wait inside a
 * kernel gave up). Synchronises `stream`. */
bool q3_cuda_q4k_linear_status(void *stream, uint32_t *status, char *error,
                               size_t error_len);

#ifdef __cplusplus
}
#endif

#endif /* Q3_Q4_LINEAR_B200_H */
