/* q3_compat_fp32.cu - the reference's primitive surface, symbol for symbol
 * (ref: src/q3_forward.h:82-91,177-192,252-281): fp32 device pointers,
 * contiguous fp32 KV slabs, void* stream, never synchronises. These entry
 * points exist so the reference's own layer drivers and tests link against
 * this library unchanged; the tensor-core path is the paged one in
 * q3_attn_tc.cu. Same arithmetic as the reference kernels, with two
 * differences that do not change results beyond rounding: softmax is one pass
 * with a running maximum instead of two passes, and sin/cos are the precise
 * routines (this file is compiled without fast-math) so large positions stay
 * accurate.
 */
#include "q3_internal.h"

#include <stdlib.h>

struct q3_kv_cache {
    uint32_t num_layers;
    uint32_t num_kv_heads;
    uint32_t head_dim;
    uint32_t capacity;
    uint32_t length;
    float *k; /* [num_layers][capacity][num_kv_heads][head_dim] */
    float *v;
    bool owns_storage;
};

namespace {

/* ref: rms_norm_batched_kernel, src/q3_forward.cu:117-148. One warp per row. */
__global__ void __launch_bounds__(256)
rms_norm_rows_kernel(const float *__restrict__ input, const float *__restrict__ weight,
                     float *output, uint32_t rows, uint32_t width, float epsilon) {
    const uint32_t row = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    const uint32_t lane = threadIdx.x & 31u;
    if (row >= rows) return;
    const float *in = input + (size_t)row * width;
    float *out = output + (size_t)row * width;
    float sum = 0.f;
    for (uint32_t i = lane; i < width; i += 32) sum += in[i] * in[i];
    for (uint32_t o = 16; o; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
    const float inv = 1.0f / sqrtf(sum / (float)width + epsilon);
    for (uint32_t i = lane; i < width; i += 32) out[i] = in[i] * inv * weight[i];
}

/* ref: rope_kernel / rope_kernel_positions, src/q3_forward.cu:181-209,380-410 */
__global__ void __launch_bounds__(256)
rope_pairs_kernel(float *q, float *k, uint32_t tokens, uint32_t n_heads,
                  uint32_t n_kv_heads, uint32_t head_dim, uint32_t position_base,
                  const uint32_t *__restrict__ token_positions,
                  const float *__restrict__ inv_freq) {
    const uint32_t pairs = head_dim / 2;
    const size_t total = (size_t)tokens * (n_heads + n_kv_heads) * pairs;
    const size_t index = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (index >= total) return;
    const size_t pi = index % pairs;
    const size_t head = (index / pairs) % (n_heads + n_kv_heads);
    const size_t token = index / ((size_t)pairs * (n_heads + n_kv_heads));
    const bool is_q = head < n_heads;
    const uint32_t h = is_q ? (uint32_t)head : (uint32_t)(head - n_heads);
    const uint32_t heads = is_q ? n_heads : n_kv_heads;
    const uint32_t position =
        token_positions ? token_positions[token] : position_base + (uint32_t)token;
    const float angle = (float)position * inv_freq[pi];
    float s, c;
    sincosf(angle, &s, &c);
    float *tensor = is_q ? q : k;
    const size_t base = ((size_t)token * heads + h) * head_dim;
    const float x = tensor[base + pi], y = tensor[base + pairs + pi];
    tensor[base + pi] = x * c - y * s;
    tensor[base + pairs + pi] = x * s + y * c;
}

/* One warp per (token, head); keys of up to two segments; running max. */
__device__ __forceinline__ void walk_keys(const float *q_row, const float *k_rows,
                                          const float *v_rows, uint32_t n, size_t row,
                                          uint32_t dims_per_lane, uint32_t lane,
                                          float scale, float &m, float &den,
                                          float *acc) {
    for (uint32_t j = 0; j < n; j++) {
        const float *k_row = k_rows + (size_t)j * row;
        const float *v_row = v_rows + (size_t)j * row;
        float dot = 0.f;
        for (uint32_t i = 0; i < dims_per_lane; i++) {
            const uint32_t d = lane + i * 32;
            dot += q_row[d] * k_row[d];
        }
        for (uint32_t o = 16; o; o >>= 1) dot += __shfl_xor_sync(0xffffffffu, dot, o);
        const float s = dot * scale;
        const float m_new = fmaxf(m, s);
        const float alpha = expf(m - m_new);
        const float p = expf(s - m_new);
        den = den * alpha + p;
        for (uint32_t i = 0; i < dims_per_lane; i++)
            acc[i] = acc[i] * alpha + p * v_row[lane + i * 32];
        m = m_new;
    }
}

/* ref: attention_kernel, src/q3_forward.cu:218-290 */
__global__ void __launch_bounds__(32)
attention_fp32_kernel(const float *q, const float *k, const float *v, float *out,
                      uint32_t tokens, uint32_t n_heads, uint32_t n_kv_heads,
                      uint32_t head_dim, uint32_t position_base, uint32_t kv_length,
                      float scale) {
    const uint32_t token = blockIdx.x, head = blockIdx.y, lane = threadIdx.x;
    const uint32_t kv_head = head / (n_heads / n_kv_heads);
    const uint32_t visible = position_base + token + 1;
    if (visible > kv_length) return;
    const uint32_t dpl = head_dim / 32;
    float acc[8];
    for (uint32_t i = 0; i < dpl; i++) acc[i] = 0.f;
    float m = -INFINITY, den = 0.f;
    const size_t row = (size_t)n_kv_heads * head_dim;
    walk_keys(q + ((size_t)token * n_heads + head) * head_dim,
              k + (size_t)kv_head * head_dim, v + (size_t)kv_head * head_dim, visible, row,
              dpl, lane, scale, m, den, acc);
    float *out_row = out + ((size_t)token * n_heads + head) * head_dim;
    for (uint32_t i = 0; i < dpl; i++) out_row[lane + i * 32] = acc[i] / den;
}

/* ref: attention_segmented_kernel, src/q3_forward.cu:418-525 */
__global__ void __launch_bounds__(32)
attention_segmented_fp32_kernel(const float *q, float *out, uint32_t tokens,
                                uint32_t n_heads, uint32_t n_kv_heads, uint32_t head_dim,
                                float scale, const float *prefix_k, const float *prefix_v,
                                uint32_t prefix_len, uint32_t prefix_capacity,
                                const float *suffix_k, const float *suffix_v,
                                uint32_t suffix_capacity, uint32_t suffix_num_layers,
                                uint32_t suffix_layer, const uint32_t *token_branch,
                                const uint32_t *token_local_pos) {
    const uint32_t token = blockIdx.x, head = blockIdx.y, lane = threadIdx.x;
    const uint32_t kv_head = head / (n_heads / n_kv_heads);
    const size_t row = (size_t)n_kv_heads * head_dim;
    const uint32_t b = token_branch[token], lp = token_local_pos[token];
    const size_t branch_base =
        ((size_t)b * suffix_num_layers + suffix_layer) * suffix_capacity * row;
    const size_t prefix_base = (size_t)suffix_layer * prefix_capacity * row;
    const uint32_t dpl = head_dim / 32;
    float acc[8];
    for (uint32_t i = 0; i < dpl; i++) acc[i] = 0.f;
    float m = -INFINITY, den = 0.f;
    const float *q_row = q + ((size_t)token * n_heads + head) * head_dim;
    walk_keys(q_row, prefix_k + prefix_base + (size_t)kv_head * head_dim,
              prefix_v + prefix_base + (size_t)kv_head * head_dim, prefix_len, row, dpl,
              lane, scale, m, den, acc);
    walk_keys(q_row, suffix_k + branch_base + (size_t)kv_head * head_dim,
              suffix_v + branch_base + (size_t)kv_head * head_dim, lp + 1, row, dpl, lane,
              scale, m, den, acc);
    float *out_row = out + ((size_t)token * n_heads + head) * head_dim;
    for (uint32_t i = 0; i < dpl; i++) out_row[lane + i * 32] = acc[i] / den;
}

/* ref: kv_scatter_kernel, src/q3_forward.cu:529-550; 16 bytes per thread */
__global__ void __launch_bounds__(256)
kv_scatter_fp32_kernel(float *suffix_k, float *suffix_v, const float *k_src,
                       const float *v_src, const uint32_t *token_branch,
                       const uint32_t *token_local_pos, uint32_t tokens, uint32_t row,
                       uint32_t suffix_capacity, uint32_t num_layers, uint32_t layer) {
    const size_t index = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    const uint32_t row4 = row / 4;
    if (index >= (size_t)tokens * row4) return;
    const uint32_t token = (uint32_t)(index / row4), e = (uint32_t)(index % row4);
    const size_t dst = ((size_t)token_branch[token] * num_layers + layer) *
                           suffix_capacity * row +
                       (size_t)token_local_pos[token] * row;
    reinterpret_cast<float4 *>(suffix_k + dst)[e] =
        reinterpret_cast<const float4 *>(k_src + (size_t)token * row)[e];
    reinterpret_cast<float4 *>(suffix_v + dst)[e] =
        reinterpret_cast<const float4 *>(v_src + (size_t)token * row)[e];
}

}  // namespace

/* ---------------------------------------------------------------------- */

extern "C" bool q3_cuda_rms_norm(const float *input, const float *weight, uint32_t rows,
                                 uint32_t width, float epsilon, float *output,
                                 void *stream, char *error, size_t error_len) {
    q3_clear_error(error, error_len);
    if (!input || !weight || !output || rows == 0 || width == 0)
        return q3_fail(error, error_len, "q3_cuda_rms_norm: invalid argument");
    const unsigned grid = (unsigned)(((size_t)rows * 32 + 255) / 256);
    rms_norm_rows_kernel<<<grid, 256, 0, (cudaStream_t)stream>>>(input, weight, output,
                                                                  rows, width, epsilon);
    Q3_LAUNCH_CHECK("q3_cuda_rms_norm launch failed");
    return true;
}

static bool rope_common(float *q, float *k, uint32_t tokens, uint32_t n_heads,
                        uint32_t n_kv_heads, uint32_t head_dim, uint32_t position_base,
                        const uint32_t *token_positions, const float *inv_freq,
                        void *stream, char *error, size_t error_len, const char *who) {
    const size_t total = (size_t)tokens * (n_heads + n_kv_heads) * (head_dim / 2);
    const unsigned grid = (unsigned)((total + 255) / 256);
    rope_pairs_kernel<<<grid, 256, 0, (cudaStream_t)stream>>>(
        q, k, tokens, n_heads, n_kv_heads, head_dim, position_base, token_positions,
        inv_freq);
    Q3_LAUNCH_CHECK(who);
    return true;
}

extern "C" bool q3_cuda_rope(float *q, float *k, uint32_t tokens, uint32_t n_heads,
                             uint32_t n_kv_heads, uint32_t head_dim,
                             uint32_t position_base, const float *inv_freq, void *stream,
                             char *error, size_t error_len) {
    q3_clear_error(error, error_len);
    if (!q || !k || !inv_freq || tokens == 0 || head_dim == 0 || head_dim % 2 != 0)
        return q3_fail(error, error_len, "q3_cuda_rope: invalid argument");
    return rope_common(q, k, tokens, n_heads, n_kv_heads, head_dim, position_base, NULL,
                       inv_freq, stream, error, error_len, "q3_cuda_rope launch failed");
}

extern "C" bool q3_cuda_rope_positions(float *q, float *k, uint32_t tokens,
                                       uint32_t n_heads, uint32_t n_kv_heads,
                                       uint32_t head_dim,
                                       const uint32_t *token_positions,
                                       const float *inv_freq, void *stream, char *error,
                                       size_t error_len) {
    q3_clear_error(error, error_len);
    if (!q || !k || !inv_freq || !token_positions || tokens == 0 || head_dim == 0 ||
        head_dim % 2 != 0)
        return q3_fail(error, error_len, "q3_cuda_rope_positions: invalid argument");
    return rope_common(q, k, tokens, n_heads, n_kv_heads, head_dim, 0, token_positions,
                       inv_freq, stream, error, error_len,
                       "q3_cuda_rope_positions launch failed");
}

extern "C" bool q3_cuda_attention(const float *q, const float *k, const float *v,
                                  uint32_t tokens, uint32_t n_heads, uint32_t n_kv_heads,
                                  uint32_t head_dim, uint32_t position_base,
                                  q3_kv_cache *kv, uint32_t layer, float scale,
                                  float *out, void *stream, char *error,
                                  size_t error_len) {
    q3_clear_error(error, error_len);
    if (!q || !out || tokens == 0 || n_heads == 0 || n_kv_heads == 0 || head_dim == 0 ||
        head_dim % 32 != 0 || head_dim > 256 || n_heads % n_kv_heads != 0 ||
        (!kv && (!k || !v)))
        return q3_fail(error, error_len, "q3_cuda_attention: invalid argument");
    const float *k_src = k, *v_src = v;
    uint32_t kv_length = tokens;
    if (kv) {
        if (layer >= kv->num_layers)
            return q3_fail(error, error_len, "q3_cuda_attention: invalid argument");
        const size_t per_layer = (size_t)kv->capacity * n_kv_heads * head_dim;
        k_src = kv->k + (size_t)layer * per_layer;
        v_src = kv->v + (size_t)layer * per_layer;
        kv_length = kv->length + tokens;
    }
    {
        bool ok = false;
        if (q3_fp32_native_attention(q, k_src, v_src, tokens, n_heads, n_kv_heads, head_dim,
                                     position_base, kv_length, scale, out, stream, &ok, error,
                                     error_len))
            return ok;
    }
    dim3 grid(tokens, n_heads);
    attention_fp32_kernel<<<grid, 32, 0, (cudaStream_t)stream>>>(
        q, k_src, v_src, out, tokens, n_heads, n_kv_heads, head_dim, position_base,
        kv_length, scale);
    Q3_LAUNCH_CHECK("q3_cuda_attention launch failed");
    return true;
}

extern "C" bool q3_cuda_attention_segmented(
    const float *q, const float *prefix_k, const float *prefix_v, uint32_t prefix_len,
    uint32_t prefix_capacity, const float *suffix_k, const float *suffix_v,
    uint32_t suffix_capacity, uint32_t suffix_num_layers, uint32_t suffix_layer,
    const uint32_t *token_branch, const uint32_t *token_local_pos, uint32_t tokens,
    uint32_t n_heads, uint32_t n_kv_heads, uint32_t head_dim, float scale, float *out,
    void *stream, char *error, size_t error_len) {
    q3_clear_error(error, error_len);
    if (!q || !out || !prefix_k || !prefix_v || !suffix_k || !suffix_v || !token_branch ||
        !token_local_pos || tokens == 0 || n_heads == 0 || n_kv_heads == 0 ||
        head_dim == 0 || head_dim % 32 != 0 || head_dim > 256 ||
        n_heads % n_kv_heads != 0 || prefix_len > prefix_capacity ||
        suffix_num_layers == 0)
        return q3_fail(error, error_len, "q3_cuda_attention_segmented: invalid argument");
    if (suffix_layer < suffix_num_layers) {
        bool ok = false;
        /* the prefix slabs hold every layer: [layer][prefix_capacity][row] */
        const size_t pbase = (size_t)suffix_layer * prefix_capacity * n_kv_heads * head_dim;
        if (q3_fp32_native_segmented(q, prefix_k + pbase, prefix_v + pbase, prefix_len, suffix_k, suffix_v,
                                     suffix_capacity, suffix_num_layers, suffix_layer,
                                     token_branch, token_local_pos, tokens, n_heads,
                                     n_kv_heads, head_dim, scale, out, stream, &ok, error,
                                     error_len))
            return ok;
    }
    {
        /* the fp32 kernel dereferences the descriptors on the device: pageable
         * host memory would fault there (the reference hands its kernels such
         * memory, which only works on unified-memory parts) */
        cudaPointerAttributes a, b;
        const bool known = cudaPointerGetAttributes(&a, token_branch) == cudaSuccess &&
                           cudaPointerGetAttributes(&b, token_local_pos) == cudaSuccess;
        if (!known) cudaGetLastError();
        if (known && (a.type == cudaMemoryTypeUnregistered || b.type == cudaMemoryTypeUnregistered))
            return q3_fail(error, error_len,
                           "q3_cuda_attention_segmented: token_branch / token_local_pos are in "
                           "pageable host memory, which this device cannot read: pass device "
                           "copies, or enable the tensor-core path "
                           "(q3_cuda_attention_native_init), which reads them on the host");
    }
    dim3 grid(tokens, n_heads);
    attention_segmented_fp32_kernel<<<grid, 32, 0, (cudaStream_t)stream>>>(
        q, out, tokens, n_heads, n_kv_heads, head_dim, scale, prefix_k, prefix_v,
        prefix_len, prefix_capacity, suffix_k, suffix_v, suffix_capacity,
        suffix_num_layers, suffix_layer, token_branch, token_local_pos);
    Q3_LAUNCH_CHECK("q3_cuda_attention_segmented launch failed");
    return true;
}

extern "C" bool q3_cuda_kv_scatter(float *suffix_k, float *suffix_v, const float *k_src,
                                   const float *v_src, const uint32_t *token_branch,
                                   const uint32_t *token_local_pos, uint32_t tokens,
                                   uint32_t row, uint32_t suffix_capacity,
                                   uint32_t num_layers, uint32_t layer, void *stream,
                                   char *error, size_t error_len) {
    q3_clear_error(error, error_len);
    if (!suffix_k || !suffix_v || !k_src || !v_src || !token_branch || !token_local_pos ||
        tokens == 0 || row == 0 || row % 4 != 0 || num_layers == 0 || layer >= num_layers)
        return q3_fail(error, error_len, "q3_cuda_kv_scatter: invalid argument");
    const size_t total = (size_t)tokens * (row / 4);
    kv_scatter_fp32_kernel<<<(unsigned)((total + 255) / 256), 256, 0,
                             (cudaStream_t)stream>>>(suffix_k, suffix_v, k_src, v_src,
                                                     token_branch, token_local_pos, tokens,
                                                     row, suffix_capacity, num_layers, layer);
    Q3_LAUNCH_CHECK("q3_cuda_kv_scatter launch failed");
    return true;
}

/* ---- KV cache API (ref: src/q3_forward.cu:834-946) ---------------------- */

extern "C" q3_kv_cache *q3_kv_cache_init(uint32_t num_layers, uint32_t num_kv_heads,
                                         uint32_t head_dim, uint32_t capacity,
                                         char *error, size_t error_len) {
    q3_clear_error(error, error_len);
    if (num_layers == 0 || num_kv_heads == 0 || head_dim == 0 || capacity == 0) {
        q3_fail(error, error_len, "q3_kv_cache_init: invalid argument");
        return NULL;
    }
    q3_kv_cache *kv = (q3_kv_cache *)calloc(1, sizeof(q3_kv_cache));
    if (!kv) {
        q3_fail(error, error_len, "q3_kv_cache_init: allocation failed");
        return NULL;
    }
    kv->num_layers = num_layers;
    kv->num_kv_heads = num_kv_heads;
    kv->head_dim = head_dim;
    kv->capacity = capacity;
    kv->owns_storage = true;
    const size_t bytes =
        (size_t)capacity * num_kv_heads * head_dim * num_layers * sizeof(float);
    if (cudaMalloc(&kv->k, bytes) != cudaSuccess ||
        cudaMalloc(&kv->v, bytes) != cudaSuccess) {
        q3_fail(error, error_len, "q3_kv_cache_init: cudaMalloc failed");
        if (kv->k) cudaFree(kv->k);
        free(kv);
        cudaGetLastError();
        return NULL;
    }
    return kv;
}

extern "C" bool q3_kv_cache_reserve(q3_kv_cache *kv, uint32_t capacity, char *error,
                                    size_t error_len) {
    q3_clear_error(error, error_len);
    if (!kv) return q3_fail(error, error_len, "q3_kv_cache_reserve: null cache");
    if (capacity <= kv->capacity) return true;
    if (!kv->owns_storage)
        return q3_fail(error, error_len, "q3_kv_cache_reserve: cache borrows its storage");
    const size_t row = (size_t)kv->num_kv_heads * kv->head_dim;
    const size_t per_layer = (size_t)capacity * row;
    float *nk = NULL, *nv = NULL;
    if (cudaMalloc(&nk, per_layer * kv->num_layers * sizeof(float)) != cudaSuccess ||
        cudaMalloc(&nv, per_layer * kv->num_layers * sizeof(float)) != cudaSuccess) {
        if (nk) cudaFree(nk);
        cudaGetLastError();
        return q3_fail(error, error_len, "q3_kv_cache_reserve: cudaMalloc failed");
    }
    const size_t used = (size_t)kv->length * row * sizeof(float);
    for (uint32_t l = 0; l < kv->num_layers && used; l++) {
        cudaMemcpy(nk + l * per_layer, kv->k + (size_t)l * kv->capacity * row, used,
                   cudaMemcpyDeviceToDevice);
        cudaMemcpy(nv + l * per_layer, kv->v + (size_t)l * kv->capacity * row, used,
                   cudaMemcpyDeviceToDevice);
    }
    cudaDeviceSynchronize(); /* the old slabs may still be read by queued work */
    cudaFree(kv->k);
    cudaFree(kv->v);
    kv->k = nk;
    kv->v = nv;
    kv->capacity = capacity;
    return true;
}

extern "C" void q3_kv_cache_reset(q3_kv_cache *kv) {
    if (kv) kv->length = 0;
}

extern "C" void q3_kv_cache_destroy(q3_kv_cache *kv) {
    if (!kv) return;
    if (kv->owns_storage) {
        if (kv->k) cudaFree(kv->k);
        if (kv->v) cudaFree(kv->v);
    }
    free(kv);
}

extern "C" uint32_t q3_kv_cache_length(const q3_kv_cache *kv) {
    return kv ? kv->length : 0;
}

extern "C" q3_kv_cache *q3_kv_cache_alias(float *k, float *v, uint32_t num_layers,
                                          uint32_t num_kv_heads, uint32_t head_dim,
                                          uint32_t capacity, uint32_t length, char *error,
                                          size_t error_len) {
    q3_clear_error(error, error_len);
    if (!k || !v || num_layers == 0 || num_kv_heads == 0 || head_dim == 0 ||
        capacity == 0) {
        q3_fail(error, error_len, "q3_kv_cache_alias: invalid argument");
        return NULL;
    }
    q3_kv_cache *kv = (q3_kv_cache *)calloc(1, sizeof(q3_kv_cache));
    if (!kv) {
        q3_fail(error, error_len, "q3_kv_cache_alias: allocation failed");
        return NULL;
    }
    kv->num_layers = num_layers;
    kv->num_kv_heads = num_kv_heads;
    kv->head_dim = head_dim;
    kv->capacity = capacity;
    kv->length = length;
    kv->k = k;
    kv->v = v;
    kv->owns_storage = false;
    return kv;
}

extern "C" void q3_kv_cache_advance(q3_kv_cache *kv, uint32_t tokens) {
    if (kv && (uint64_t)kv->length + tokens <= kv->capacity) kv->length += tokens;
}

extern "C" float *q3_kv_cache_k(const q3_kv_cache *kv) { return kv ? kv->k : NULL; }
extern "C" float *q3_kv_cache_v(const q3_kv_cache *kv) { return kv ? kv->v : NULL; }

extern "C" size_t q3_kv_bytes_for_tokens(uint32_t tokens, uint32_t num_layers,
                                         uint32_t num_kv_heads, uint32_t head_dim) {
    const size_t row = (size_t)num_kv_heads * head_dim;
    return 2 * (size_t)num_layers * tokens * row * sizeof(float);
}
