// KV cache: allocation, token append (dense and compressed), reset and debug read-back.
//
// Device layout is head-major (see common.cuh). The append kernels fuse RoPE(K), the
// f32->f16 cast and, for compressed caches, the eviction of the ring slot being
// overwritten (copy K to the old region, quantise V to q4 with one f32 scale per
// (token, kv head)) into ONE launch per token; the reference spends up to four
// (cuda/kernels.cu:6108-6250).
#include <stdlib.h>
#include <string.h>

#include "common.cuh"
#include "kv_append.cuh"

namespace {

// Dense append: grid = kv_heads, block = hd/2 threads (one RoPE pair each).
// position < 0xffffffff: explicit; position_dev != null overrides; use_seq_map: append at seq_map[seq].
__global__ void dense_append_kernel(const float* __restrict__ k_in, const float* __restrict__ v_in,
                                    __half* __restrict__ K, __half* __restrict__ V, uint32_t* __restrict__ seq_map,
                                    uint32_t seq_id, uint32_t max_seq_len, uint32_t heads, uint32_t hd,
                                    uint32_t position, const uint32_t* __restrict__ position_dev, uint32_t rope_pos,
                                    uint32_t rope_from_position, uint32_t apply_rope, float freq_base,
                                    float freq_scale, uint32_t layout) {
    if (position_dev) position = *position_dev;
    if (position >= max_seq_len) return;
    if (rope_from_position) rope_pos = position;
    const uint32_t head = blockIdx.x;
    const uint32_t half = hd / 2u;
    const size_t row = kv_row_offset(seq_id, head, position, heads, max_seq_len, hd);
    for (uint32_t i = threadIdx.x; i < half; i += blockDim.x) {
        const uint32_t i0 = layout == 1u ? i : 2u * i;
        const uint32_t i1 = layout == 1u ? i + half : 2u * i + 1u;
        const float a = k_in[head * hd + i0], b = k_in[head * hd + i1];
        float c = 1.0f, s = 0.0f;
        if (apply_rope) rope_cs(rope_pos, i, hd, freq_base, freq_scale, &c, &s);
        K[row + i0] = __float2half_rn(apply_rope ? a * c - b * s : a);
        K[row + i1] = __float2half_rn(apply_rope ? a * s + b * c : b);
        V[row + i0] = __float2half_rn(v_in[head * hd + i0]);
        V[row + i1] = __float2half_rn(v_in[head * hd + i1]);
    }
    if ((hd & 1u) && threadIdx.x == 0) {  // odd head_dim: last element has no pair
        K[row + hd - 1u] = __float2half_rn(k_in[head * hd + hd - 1u]);
        V[row + hd - 1u] = __float2half_rn(v_in[head * hd + hd - 1u]);
    }
    if (head == 0 && threadIdx.x == 0) seq_map[seq_id] = position + 1u;
}

__global__ void dense_append_f16_kernel(const __half* __restrict__ k_in, const __half* __restrict__ v_in,
                                        __half* __restrict__ K, __half* __restrict__ V, uint32_t seq_id,
                                        uint32_t max_seq_len, uint32_t heads, uint32_t hd, uint32_t position) {
    const uint32_t head = blockIdx.x;
    const size_t row = kv_row_offset(seq_id, head, position, heads, max_seq_len, hd);
    for (uint32_t i = threadIdx.x; i < hd; i += blockDim.x) {
        K[row + i] = k_in[head * hd + i];
        V[row + i] = v_in[head * hd + i];
    }
}

// Compressed append (cuda/kernels.cu:2230-2311, 5691-5791): grid = kv_heads, block = 64 threads
// (hd/2 <= 64). If position >= R, the ring slot position % R still holds token position - R:
// move it to the old region first, then overwrite the slot with the new token.
__global__ void __launch_bounds__(64) compressed_append_kernel(
    const float* __restrict__ k_in, const float* __restrict__ v_in, M40llmKVCache kv, uint32_t seq_id,
    uint32_t position, float freq_base, float freq_scale, uint32_t layout) {
    __shared__ float red[32];
    kv_append_compressed_head(kv, seq_id, blockIdx.x, position, k_in + blockIdx.x * kv.head_dim,
                              v_in + blockIdx.x * kv.head_dim, freq_base, freq_scale, layout, red);
}

// Harness loader: staged tokens [count][heads][hd] f16 (reference logical layout) -> cache.
// grid = (count, heads), block = 64.
__global__ void __launch_bounds__(64) place_tokens_kernel(const __half* __restrict__ k_st,
                                                          const __half* __restrict__ v_st, M40llmKVCache kv,
                                                          uint32_t seq_id, uint32_t tok_begin, uint32_t final_len) {
    __shared__ float red[32];
    const uint32_t t = tok_begin + blockIdx.x;
    const uint32_t head = blockIdx.y;
    const uint32_t hd = kv.head_dim;
    const __half* ks = k_st + ((size_t)blockIdx.x * kv.num_heads + head) * hd;
    const __half* vs = v_st + ((size_t)blockIdx.x * kv.num_heads + head) * hd;
    if (!kv.compressed) {
        const size_t row = kv_row_offset(seq_id, head, t, kv.num_heads, kv.max_seq_len, hd);
        for (uint32_t i = threadIdx.x; i < hd; i += blockDim.x) {
            kv.d_k[row + i] = ks[i];
            kv.d_v[row + i] = vs[i];
        }
        return;
    }
    const uint32_t old_len = final_len > kv.recent_window ? final_len - kv.recent_window : 0u;
    if (t < old_len) {
        const size_t row = kv_row_offset(seq_id, head, t, kv.num_heads, kv.max_seq_len, hd);
        for (uint32_t i = threadIdx.x; i < hd; i += blockDim.x) kv.d_old_k[row + i] = ks[i];
        const size_t vec = ((size_t)seq_id * kv.num_heads + head) * (size_t)kv.max_seq_len + t;
        quantize_v_row_q4(vs, kv.d_q4_v + vec * (hd / 2u), kv.d_q4_scale + vec, hd, red);
    } else {
        const size_t row = kv_row_offset(seq_id, head, t % kv.recent_window, kv.num_heads, kv.recent_window, hd);
        for (uint32_t i = threadIdx.x; i < hd; i += blockDim.x) {
            kv.d_recent_k[row + i] = ks[i];
            kv.d_recent_v[row + i] = vs[i];
        }
    }
}

// One (token, kv head, slot) of a dense cache into the compressed cache. grid (seq_len, heads, slots), block 64.
__global__ void __launch_bounds__(64) compress_from_dense_kernel(M40llmKVCache dense, M40llmKVCache kv, uint32_t seq_len) {
    __shared__ float red[32];
    const uint32_t t = blockIdx.x, head = blockIdx.y, slot = blockIdx.z, hd = kv.head_dim;
    const size_t src = kv_row_offset(slot, head, t, dense.num_heads, dense.max_seq_len, hd);
    const uint32_t old_len = seq_len > kv.recent_window ? seq_len - kv.recent_window : 0u;
    if (t < old_len) {
        const size_t row = kv_row_offset(slot, head, t, kv.num_heads, kv.max_seq_len, hd);
        for (uint32_t i = threadIdx.x; i < hd; i += blockDim.x) kv.d_old_k[row + i] = dense.d_k[src + i];
        const size_t vec = ((size_t)slot * kv.num_heads + head) * (size_t)kv.max_seq_len + t;
        quantize_v_row_q4(dense.d_v + src, kv.d_q4_v + vec * (hd / 2u), kv.d_q4_scale + vec, hd, red);
    } else {
        const size_t row = kv_row_offset(slot, head, t % kv.recent_window, kv.num_heads, kv.recent_window, hd);
        for (uint32_t i = threadIdx.x; i < hd; i += blockDim.x) {
            kv.d_recent_k[row + i] = dense.d_k[src + i];
            kv.d_recent_v[row + i] = dense.d_v[src + i];
        }
    }
}

__global__ void fill_u32_kernel(uint32_t* p, uint32_t v, uint32_t n) {
    const uint32_t i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) p[i] = v;
}

template <typename T>
bool dev_alloc_zero(T** p, size_t count) {
    if (cudaMalloc((void**)p, count * sizeof(T)) != cudaSuccess) {
        cudaGetLastError();
        *p = nullptr;
        return false;
    }
    return cudaMemset(*p, 0, count * sizeof(T)) == cudaSuccess;
}

// The host reads the sequence's length to choose the slot of the new token (cuda/kernels.cu reads it with a blocking
// cudaMemcpy, which on the reference's blocking streams waits for an append still in flight). The streams here are
// non-blocking, so the read rides the decode stream, where every append writes the length, and waits for it: two
// appends issued back to back see each other.
int read_current_len(M40llmCudaContext* ctx, M40llmKVCache* kv, uint32_t seq_id, uint32_t* out) {
    cudaStream_t s = ctx->decode_stream;
    if (cudaMemcpyAsync(out, kv->d_seq_map + seq_id, sizeof(uint32_t), cudaMemcpyDeviceToHost, s) != cudaSuccess) return -1;
    return cudaStreamSynchronize(s) == cudaSuccess ? 0 : -1;
}

}  // namespace

extern "C" {

M40llmKVCache* m40llm_kvcache_create(M40llmCudaContext* ctx, uint32_t max_seq_len, uint32_t max_batch_size,
                                     uint32_t num_heads, uint32_t head_dim) {
    if (!ctx) return nullptr;
    if (m40_ensure_device(ctx) != 0) return nullptr;
    M40llmKVCache* kv = (M40llmKVCache*)calloc(1, sizeof(M40llmKVCache));
    if (!kv) return nullptr;
    kv->device_id = ctx->device_id;
    kv->max_seq_len = max_seq_len;
    kv->max_batch_size = max_batch_size;
    kv->num_heads = num_heads;
    kv->head_dim = head_dim;
    const size_t elems = (size_t)max_seq_len * max_batch_size * num_heads * head_dim;
    bool ok = dev_alloc_zero(&kv->d_k, elems ? elems : 1);
    ok = ok && dev_alloc_zero(&kv->d_v, elems ? elems : 1);
    ok = ok && dev_alloc_zero(&kv->d_seq_map, max_batch_size ? max_batch_size : 1);
    // zero-fill ran on the legacy stream; the context's non-blocking streams do not order against it
    ok = ok && cudaStreamSynchronize(cudaStreamLegacy) == cudaSuccess;
    if (!ok) {
        m40llm_kvcache_destroy(kv);
        return nullptr;
    }
    return kv;
}

M40llmKVCache* m40llm_kvcache_create_compressed(M40llmCudaContext* ctx, uint32_t max_seq_len, uint32_t max_batch_size,
                                                uint32_t num_heads, uint32_t head_dim, uint32_t recent_window,
                                                uint32_t block_size, uint32_t top_blocks, uint32_t representatives,
                                                uint32_t representative_policy, uint32_t exact_old_backing) {
    if (!ctx || recent_window == 0 || block_size == 0) return nullptr;
    // Only the FP16-K / q4-V backing (2) is implemented; q8 (1) and the summary-only form (0) belong to
    // modes outside the decode hot path. q4 needs head_dim 64 or 128 (cuda/kernels.cu:5370-5371).
    if (exact_old_backing != 2u) return nullptr;
    if (head_dim != 64 && head_dim != 128) return nullptr;
    if (m40_ensure_device(ctx) != 0) return nullptr;
    M40llmKVCache* kv = (M40llmKVCache*)calloc(1, sizeof(M40llmKVCache));
    if (!kv) return nullptr;
    kv->device_id = ctx->device_id;
    kv->max_seq_len = max_seq_len;
    kv->max_batch_size = max_batch_size;
    kv->num_heads = num_heads;
    kv->head_dim = head_dim;
    kv->compressed = 1;
    kv->recent_window = recent_window;
    kv->block_size = block_size;
    kv->top_blocks = top_blocks;
    kv->representatives = representatives;
    kv->representative_policy = representative_policy;
    kv->fp16_k_q4_v_backing = 1;
    const uint32_t old_capacity = max_seq_len > recent_window ? max_seq_len - recent_window : 0;
    kv->max_blocks = old_capacity == 0 ? 1 : (old_capacity + block_size - 1) / block_size;
    const size_t ept = (size_t)num_heads * head_dim;
    const size_t vectors = (size_t)max_seq_len * max_batch_size * num_heads;
    bool ok = dev_alloc_zero(&kv->d_recent_k, (size_t)max_batch_size * recent_window * ept);
    ok = ok && dev_alloc_zero(&kv->d_recent_v, (size_t)max_batch_size * recent_window * ept);
    ok = ok && dev_alloc_zero(&kv->d_old_k, vectors * head_dim);
    ok = ok && dev_alloc_zero(&kv->d_q4_v, vectors * (head_dim / 2));
    ok = ok && dev_alloc_zero(&kv->d_q4_scale, vectors);
    ok = ok && dev_alloc_zero(&kv->d_seq_map, max_batch_size ? max_batch_size : 1);
    // zero-fill ran on the legacy stream; the context's non-blocking streams do not order against it
    ok = ok && cudaStreamSynchronize(cudaStreamLegacy) == cudaSuccess;
    if (!ok) {
        m40llm_kvcache_destroy(kv);
        return nullptr;
    }
    return kv;
}

void m40llm_kvcache_destroy(M40llmKVCache* kv) {
    if (!kv) return;
    cudaSetDevice(kv->device_id);
    if (kv->d_k) cudaFree(kv->d_k);
    if (kv->d_v) cudaFree(kv->d_v);
    if (kv->d_seq_map) cudaFree(kv->d_seq_map);
    if (kv->d_recent_k) cudaFree(kv->d_recent_k);
    if (kv->d_recent_v) cudaFree(kv->d_recent_v);
    if (kv->d_old_k) cudaFree(kv->d_old_k);
    if (kv->d_q4_v) cudaFree(kv->d_q4_v);
    if (kv->d_q4_scale) cudaFree(kv->d_q4_scale);
    free(kv);
}

int m40llm_kvcache_reset(M40llmCudaContext* ctx, M40llmKVCache* kv) {
    if (!ctx || !kv) return -1;
    if (m40_ensure_device(ctx) != 0) return -2;
    cudaStream_t s = ctx->decode_stream;
    if (cudaMemsetAsync(kv->d_seq_map, 0, (size_t)kv->max_batch_size * sizeof(uint32_t), s) != cudaSuccess) return -3;
    if (kv->compressed) {
        const size_t ept = (size_t)kv->num_heads * kv->head_dim;
        const size_t vectors = (size_t)kv->max_seq_len * kv->max_batch_size * kv->num_heads;
        cudaMemsetAsync(kv->d_recent_k, 0, (size_t)kv->max_batch_size * kv->recent_window * ept * sizeof(__half), s);
        cudaMemsetAsync(kv->d_recent_v, 0, (size_t)kv->max_batch_size * kv->recent_window * ept * sizeof(__half), s);
        cudaMemsetAsync(kv->d_old_k, 0, vectors * kv->head_dim * sizeof(__half), s);
        cudaMemsetAsync(kv->d_q4_v, 0, vectors * (kv->head_dim / 2), s);
        cudaMemsetAsync(kv->d_q4_scale, 0, vectors * sizeof(float), s);
    }
    return cudaStreamSynchronize(s) == cudaSuccess ? 0 : -4;
}

int m40llm_kvcache_append_token(M40llmCudaContext* ctx, M40llmKVCache* kv, uint32_t seq_id, const void* k_dev,
                                const void* v_dev) {
    if (!ctx || !kv || !k_dev || !v_dev) return -1;
    if (seq_id >= kv->max_batch_size) return -2;
    if (m40_ensure_device(ctx) != 0 || !kv->d_k) return -3;
    uint32_t cur = 0;
    if (read_current_len(ctx, kv, seq_id, &cur) != 0) return -3;
    if (cur >= kv->max_seq_len) return -4;
    dense_append_f16_kernel<<<kv->num_heads, 128, 0, ctx->decode_stream>>>(
        (const __half*)k_dev, (const __half*)v_dev, kv->d_k, kv->d_v, seq_id, kv->max_seq_len, kv->num_heads,
        kv->head_dim, cur);
    M40_COUNT_LAUNCH(ctx);
    if (cudaGetLastError() != cudaSuccess) return -5;
    cur += 1;
    if (cudaMemcpyAsync(kv->d_seq_map + seq_id, &cur, sizeof(uint32_t), cudaMemcpyHostToDevice, ctx->decode_stream) !=
        cudaSuccess)
        return -7;
    return cudaStreamSynchronize(ctx->decode_stream) == cudaSuccess ? 0 : -6;
}

int m40llm_kvcache_append_token_f32_async(M40llmCudaContext* ctx, M40llmKVCache* kv, uint32_t seq_id,
                                          const void* k_dev_f32, const void* v_dev_f32) {
    if (!ctx || !kv || !k_dev_f32 || !v_dev_f32) return -1;
    if (seq_id >= kv->max_batch_size) return -2;
    if (m40_ensure_device(ctx) != 0 || !kv->d_k) return -3;
    uint32_t cur = 0;
    if (read_current_len(ctx, kv, seq_id, &cur) != 0) return -3;
    if (cur >= kv->max_seq_len) return -4;
    dense_append_kernel<<<kv->num_heads, 64, 0, ctx->decode_stream>>>(
        (const float*)k_dev_f32, (const float*)v_dev_f32, kv->d_k, kv->d_v, kv->d_seq_map, seq_id, kv->max_seq_len,
        kv->num_heads, kv->head_dim, cur, nullptr, 0u, 0u, 0u, 0.0f, 0.0f, 0u);
    M40_COUNT_LAUNCH(ctx);
    return cudaGetLastError() == cudaSuccess ? 0 : -5;
}

int m40llm_kvcache_append_token_f32(M40llmCudaContext* ctx, M40llmKVCache* kv, uint32_t seq_id, const void* k_dev_f32,
                                    const void* v_dev_f32) {
    const int rc = m40llm_kvcache_append_token_f32_async(ctx, kv, seq_id, k_dev_f32, v_dev_f32);
    if (rc != 0) return rc;
    return cudaStreamSynchronize(ctx->decode_stream) == cudaSuccess ? 0 : -7;
}

int m40llm_kvcache_append_token_f32_rope_k_layout_async(M40llmCudaContext* ctx, M40llmKVCache* kv, uint32_t seq_id,
                                                        const void* k_dev_f32, const void* v_dev_f32,
                                                        uint32_t past_len, float freq_base, float freq_scale,
                                                        uint32_t rope_layout) {
    if (!ctx || !kv || !k_dev_f32 || !v_dev_f32) return -1;
    if (seq_id >= kv->max_batch_size) return -2;
    if (kv->head_dim == 0 || kv->num_heads == 0) return -3;
    if (kv->head_dim % 2 != 0) return -4;
    if (m40_ensure_device(ctx) != 0 || !kv->d_k) return -5;
    uint32_t cur = 0;
    if (read_current_len(ctx, kv, seq_id, &cur) != 0) return -5;
    if (cur >= kv->max_seq_len) return -6;
    dense_append_kernel<<<kv->num_heads, 64, 0, ctx->decode_stream>>>(
        (const float*)k_dev_f32, (const float*)v_dev_f32, kv->d_k, kv->d_v, kv->d_seq_map, seq_id, kv->max_seq_len,
        kv->num_heads, kv->head_dim, cur, nullptr, past_len, 0u, 1u, freq_base, freq_scale, rope_layout);
    M40_COUNT_LAUNCH(ctx);
    return cudaGetLastError() == cudaSuccess ? 0 : -7;
}

int m40llm_kvcache_append_token_f32_rope_k_async(M40llmCudaContext* ctx, M40llmKVCache* kv, uint32_t seq_id,
                                                 const void* k_dev_f32, const void* v_dev_f32, uint32_t past_len,
                                                 float freq_base, float freq_scale) {
    return m40llm_kvcache_append_token_f32_rope_k_layout_async(ctx, kv, seq_id, k_dev_f32, v_dev_f32, past_len,
                                                               freq_base, freq_scale, 0u);
}

int m40llm_kvcache_append_token_f32_rope_k(M40llmCudaContext* ctx, M40llmKVCache* kv, uint32_t seq_id,
                                           const void* k_dev_f32, const void* v_dev_f32, uint32_t past_len,
                                           float freq_base, float freq_scale) {
    const int rc =
        m40llm_kvcache_append_token_f32_rope_k_async(ctx, kv, seq_id, k_dev_f32, v_dev_f32, past_len, freq_base, freq_scale);
    if (rc != 0) return rc;
    return cudaStreamSynchronize(ctx->decode_stream) == cudaSuccess ? 0 : -7;
}

int m40llm_kvcache_append_token_f32_rope_k_compressed_at_layout_async(M40llmCudaContext* ctx, M40llmKVCache* kv,
                                                                      uint32_t seq_id, const void* k_dev_f32,
                                                                      const void* v_dev_f32, uint32_t position,
                                                                      float freq_base, float freq_scale,
                                                                      uint32_t rope_layout) {
    if (!ctx || !kv || !k_dev_f32 || !v_dev_f32) return -1;
    if (!kv->compressed) return -2;
    if (seq_id >= kv->max_batch_size) return -3;
    if ((kv->head_dim != 64 && kv->head_dim != 128) || kv->num_heads == 0 || kv->recent_window == 0 ||
        kv->block_size == 0)
        return -4;
    if (position >= kv->max_seq_len) return -5;
    if (m40_ensure_device(ctx) != 0) return -1;
    compressed_append_kernel<<<kv->num_heads, 64, 0, ctx->decode_stream>>>(
        (const float*)k_dev_f32, (const float*)v_dev_f32, *kv, seq_id, position, freq_base, freq_scale, rope_layout);
    M40_COUNT_LAUNCH(ctx);
    return cudaGetLastError() == cudaSuccess ? 0 : -6;
}

int m40llm_kvcache_append_token_f32_rope_k_compressed_at_async(M40llmCudaContext* ctx, M40llmKVCache* kv,
                                                               uint32_t seq_id, const void* k_dev_f32,
                                                               const void* v_dev_f32, uint32_t position,
                                                               float freq_base, float freq_scale) {
    return m40llm_kvcache_append_token_f32_rope_k_compressed_at_layout_async(ctx, kv, seq_id, k_dev_f32, v_dev_f32,
                                                                             position, freq_base, freq_scale, 0u);
}

int m40llm_kvcache_append_token_f32_rope_k_at_layout_async(M40llmCudaContext* ctx, M40llmKVCache* kv, uint32_t seq_id,
                                                           const void* k_dev_f32, const void* v_dev_f32,
                                                           uint32_t position, uint32_t past_len, float freq_base,
                                                           float freq_scale, uint32_t rope_layout) {
    if (!ctx || !kv || !k_dev_f32 || !v_dev_f32) return -1;
    if (kv->compressed)
        return m40llm_kvcache_append_token_f32_rope_k_compressed_at_layout_async(
            ctx, kv, seq_id, k_dev_f32, v_dev_f32, position, freq_base, freq_scale, rope_layout);
    if (seq_id >= kv->max_batch_size) return -2;
    if (kv->head_dim == 0 || kv->num_heads == 0) return -3;
    if (kv->head_dim % 2 != 0) return -4;
    if (position >= kv->max_seq_len) return -5;
    (void)past_len;
    if (m40_ensure_device(ctx) != 0) return -1;
    dense_append_kernel<<<kv->num_heads, 64, 0, ctx->decode_stream>>>(
        (const float*)k_dev_f32, (const float*)v_dev_f32, kv->d_k, kv->d_v, kv->d_seq_map, seq_id, kv->max_seq_len,
        kv->num_heads, kv->head_dim, position, nullptr, 0u, 1u, 1u, freq_base, freq_scale, rope_layout);
    M40_COUNT_LAUNCH(ctx);
    return cudaGetLastError() == cudaSuccess ? 0 : -6;
}

int m40llm_kvcache_append_token_f32_rope_k_at_async(M40llmCudaContext* ctx, M40llmKVCache* kv, uint32_t seq_id,
                                                    const void* k_dev_f32, const void* v_dev_f32, uint32_t position,
                                                    uint32_t past_len, float freq_base, float freq_scale) {
    return m40llm_kvcache_append_token_f32_rope_k_at_layout_async(ctx, kv, seq_id, k_dev_f32, v_dev_f32, position,
                                                                  past_len, freq_base, freq_scale, 0u);
}

int m40llm_kvcache_append_token_f32_rope_k_position_dev_layout_async(M40llmCudaContext* ctx, M40llmKVCache* kv,
                                                                     uint32_t seq_id, const void* k_dev_f32,
                                                                     const void* v_dev_f32,
                                                                     const uint32_t* position_dev, float freq_base,
                                                                     float freq_scale, uint32_t rope_layout) {
    if (!ctx || !kv || !k_dev_f32 || !v_dev_f32 || !position_dev) return -1;
    if (seq_id >= kv->max_batch_size) return -2;
    if (kv->head_dim == 0 || kv->num_heads == 0) return -3;
    if (kv->head_dim % 2 != 0) return -4;
    if (m40_ensure_device(ctx) != 0 || !kv->d_k) return -5;
    dense_append_kernel<<<kv->num_heads, 64, 0, ctx->decode_stream>>>(
        (const float*)k_dev_f32, (const float*)v_dev_f32, kv->d_k, kv->d_v, kv->d_seq_map, seq_id, kv->max_seq_len,
        kv->num_heads, kv->head_dim, 0u, position_dev, 0u, 1u, 1u, freq_base, freq_scale, rope_layout);
    M40_COUNT_LAUNCH(ctx);
    return cudaGetLastError() == cudaSuccess ? 0 : -5;
}

int m40llm_kvcache_append_token_f32_rope_k_position_dev_async(M40llmCudaContext* ctx, M40llmKVCache* kv,
                                                              uint32_t seq_id, const void* k_dev_f32,
                                                              const void* v_dev_f32, const uint32_t* position_dev,
                                                              float freq_base, float freq_scale) {
    return m40llm_kvcache_append_token_f32_rope_k_position_dev_layout_async(ctx, kv, seq_id, k_dev_f32, v_dev_f32,
                                                                            position_dev, freq_base, freq_scale, 0u);
}

int m40llm_kvcache_debug_read_token(M40llmCudaContext* ctx, M40llmKVCache* kv, uint32_t seq_id, uint32_t token,
                                    void* out_k_f16, void* out_v_f16) {
    (void)ctx;
    if (!kv || !out_k_f16 || !out_v_f16) return -1;
    if (seq_id >= kv->max_batch_size) return -2;
    if (token >= kv->max_seq_len) return -3;
    if (!kv->d_k || !kv->d_v) return -4;
    cudaSetDevice(kv->device_id);
    const size_t row_bytes = (size_t)kv->head_dim * sizeof(__half);
    const size_t pitch = (size_t)kv->max_seq_len * row_bytes;
    const size_t off = kv_row_offset(seq_id, 0, token, kv->num_heads, kv->max_seq_len, kv->head_dim);
    if (cudaMemcpy2D(out_k_f16, row_bytes, kv->d_k + off, pitch, row_bytes, kv->num_heads, cudaMemcpyDeviceToHost) !=
        cudaSuccess)
        return -4;
    if (cudaMemcpy2D(out_v_f16, row_bytes, kv->d_v + off, pitch, row_bytes, kv->num_heads, cudaMemcpyDeviceToHost) !=
        cudaSuccess)
        return -5;
    return 0;
}

int m40llm_kvcache_debug_read_old_token(M40llmCudaContext* ctx, M40llmKVCache* kv, uint32_t seq_id, uint32_t token,
                                        void* out_k_f16, void* out_q4_v, float* out_scale) {
    if (!ctx || !kv || !out_k_f16 || !out_q4_v || !out_scale) return -1;
    if (!kv->compressed || !kv->d_old_k) return -16;
    if (seq_id >= kv->max_batch_size) return -2;
    if (token >= kv->max_seq_len) return -3;
    if (m40_ensure_device(ctx) != 0) return -1;
    if (cudaStreamSynchronize(ctx->decode_stream) != cudaSuccess) return -4;
    const uint32_t hd = kv->head_dim;
    const size_t off = kv_row_offset(seq_id, 0, token, kv->num_heads, kv->max_seq_len, hd);
    if (cudaMemcpy2D(out_k_f16, hd * 2, kv->d_old_k + off, (size_t)kv->max_seq_len * hd * 2, hd * 2, kv->num_heads,
                     cudaMemcpyDeviceToHost) != cudaSuccess)
        return -4;
    const size_t vec0 = ((size_t)seq_id * kv->num_heads) * (size_t)kv->max_seq_len + token;
    if (cudaMemcpy2D(out_q4_v, hd / 2, kv->d_q4_v + vec0 * (hd / 2), (size_t)kv->max_seq_len * (hd / 2), hd / 2,
                     kv->num_heads, cudaMemcpyDeviceToHost) != cudaSuccess)
        return -5;
    if (cudaMemcpy2D(out_scale, sizeof(float), kv->d_q4_scale + vec0, (size_t)kv->max_seq_len * sizeof(float),
                     sizeof(float), kv->num_heads, cudaMemcpyDeviceToHost) != cudaSuccess)
        return -6;
    return 0;
}

int m40llm_kvcache_debug_read_compressed_state(M40llmCudaContext* ctx, M40llmKVCache* kv, uint32_t seq_id,
                                               uint32_t* out_seq_len, uint32_t* out_block_counts,
                                               void* out_recent_k_f16, void* out_recent_v_f16,
                                               float* out_summary_k_acc, float* out_summary_v_acc,
                                               void* out_summary_k_f16, void* out_summary_v_f16, void* out_rep_k_f16,
                                               void* out_rep_v_f16, uint32_t* out_rep_positions) {
    if (!ctx) return -16;
    if (m40_ensure_device(ctx) != 0) return -17;
    if (!kv || !kv->compressed) return -1;
    if (seq_id >= kv->max_batch_size) return -2;
    if (!out_seq_len || !out_block_counts || !out_recent_k_f16 || !out_recent_v_f16 || !out_summary_k_acc ||
        !out_summary_v_acc || !out_summary_k_f16 || !out_summary_v_f16)
        return -3;
    if (cudaStreamSynchronize(ctx->decode_stream) != cudaSuccess) return -18;
    if (cudaStreamSynchronize(ctx->prefill_stream) != cudaSuccess) return -19;
    if (cudaMemcpy(out_seq_len, kv->d_seq_map + seq_id, sizeof(uint32_t), cudaMemcpyDeviceToHost) != cudaSuccess)
        return -4;
    const uint32_t old_len = *out_seq_len > kv->recent_window ? *out_seq_len - kv->recent_window : 0;
    for (uint32_t b = 0; b < kv->max_blocks; ++b) {
        const uint32_t start = b * kv->block_size;
        out_block_counts[b] = start >= old_len ? 0u : (old_len - start < kv->block_size ? old_len - start : kv->block_size);
    }
    // ring back to the reference's [slot][kv_head][d] order
    const uint32_t hd = kv->head_dim, R = kv->recent_window, H = kv->num_heads;
    for (uint32_t h = 0; h < H; ++h) {
        const size_t src = kv_row_offset(seq_id, h, 0, H, R, hd);
        if (cudaMemcpy2D((char*)out_recent_k_f16 + (size_t)h * hd * 2, (size_t)H * hd * 2, kv->d_recent_k + src,
                         hd * 2, hd * 2, R, cudaMemcpyDeviceToHost) != cudaSuccess)
            return -6;
        if (cudaMemcpy2D((char*)out_recent_v_f16 + (size_t)h * hd * 2, (size_t)H * hd * 2, kv->d_recent_v + src,
                         hd * 2, hd * 2, R, cudaMemcpyDeviceToHost) != cudaSuccess)
            return -7;
    }
    const size_t summary_elems = (size_t)kv->max_blocks * H * hd;
    memset(out_summary_k_acc, 0, summary_elems * sizeof(float));
    memset(out_summary_v_acc, 0, summary_elems * sizeof(float));
    memset(out_summary_k_f16, 0, summary_elems * 2);
    memset(out_summary_v_f16, 0, summary_elems * 2);
    if (kv->representatives > 0) {
        if (!out_rep_k_f16 || !out_rep_v_f16 || !out_rep_positions) return -12;
        memset(out_rep_k_f16, 0, summary_elems * kv->representatives * 2);
        memset(out_rep_v_f16, 0, summary_elems * kv->representatives * 2);
        memset(out_rep_positions, 0xff, (size_t)kv->max_blocks * kv->representatives * sizeof(uint32_t));
    }
    return 0;
}

int m40llm_kvcache_debug_write_range(M40llmCudaContext* ctx, M40llmKVCache* kv, uint32_t seq_id, uint32_t tok_begin,
                                     uint32_t count, const void* k_f16_host, const void* v_f16_host,
                                     uint32_t final_seq_len) {
    if (!ctx || !kv || !k_f16_host || !v_f16_host) return -1;
    if (seq_id >= kv->max_batch_size) return -2;
    if ((uint64_t)tok_begin + count > kv->max_seq_len || final_seq_len > kv->max_seq_len ||
        (uint64_t)tok_begin + count > final_seq_len)
        return -3;
    if (m40_ensure_device(ctx) != 0) return -1;
    cudaStream_t s = ctx->decode_stream;
    const size_t tok_bytes = (size_t)kv->num_heads * kv->head_dim * sizeof(__half);
    const uint32_t chunk_tokens = (uint32_t)(((size_t)32 << 20) / tok_bytes) ? (uint32_t)(((size_t)32 << 20) / tok_bytes) : 1u;
    __half* st = nullptr;
    const uint32_t first = count < chunk_tokens ? count : chunk_tokens;
    if (count > 0 && cudaMalloc((void**)&st, 2 * (size_t)first * tok_bytes) != cudaSuccess) {
        cudaGetLastError();
        return -4;
    }
    int rc = 0;
    for (uint32_t done = 0; done < count && rc == 0; done += chunk_tokens) {
        const uint32_t n = count - done < chunk_tokens ? count - done : chunk_tokens;
        __half* kst = st;
        __half* vst = st + (size_t)first * kv->num_heads * kv->head_dim;
        if (cudaMemcpyAsync(kst, (const char*)k_f16_host + (size_t)done * tok_bytes, (size_t)n * tok_bytes,
                            cudaMemcpyHostToDevice, s) != cudaSuccess ||
            cudaMemcpyAsync(vst, (const char*)v_f16_host + (size_t)done * tok_bytes, (size_t)n * tok_bytes,
                            cudaMemcpyHostToDevice, s) != cudaSuccess) {
            rc = -5;
            break;
        }
        dim3 grid(n, kv->num_heads);
        place_tokens_kernel<<<grid, 64, 0, s>>>(kst, vst, *kv, seq_id, tok_begin + done, final_seq_len);
        M40_COUNT_LAUNCH(ctx);
        if (cudaGetLastError() != cudaSuccess) rc = -6;
        if (cudaStreamSynchronize(s) != cudaSuccess) rc = -7;
    }
    if (rc == 0 && cudaMemcpyAsync(kv->d_seq_map + seq_id, &final_seq_len, sizeof(uint32_t), cudaMemcpyHostToDevice,
                                   s) != cudaSuccess)
        rc = -8;
    if (cudaStreamSynchronize(s) != cudaSuccess && rc == 0) rc = -7;
    if (st) cudaFree(st);
    return rc;
}

// Builds the compressed state of EVERY sequence slot from a dense cache holding `seq_len` tokens per slot
// (cuda/kernels.cu:7173-7231; the reference fills its recent ring and lossy summaries there). Here the state is what
// token-by-token appends would have left in the FP16-K / q4-V cache: tokens [0, seq_len - R) in the old region (K
// copied, V quantised to q4), the last min(seq_len, R) tokens in ring slot t % R, every sequence length = seq_len.
// Decode stream, synchronous like the reference.
int m40llm_kvcache_build_compressed_from_dense(M40llmCudaContext* ctx, M40llmKVCache* compressed,
                                               const M40llmKVCache* dense, uint32_t seq_len) {
    if (!ctx || !compressed || !dense) return -1;
    if (!compressed->compressed || dense->compressed) return -2;
    if (compressed->max_batch_size != dense->max_batch_size || compressed->num_heads != dense->num_heads ||
        compressed->head_dim != dense->head_dim)
        return -3;
    if (seq_len > compressed->max_seq_len || seq_len > dense->max_seq_len) return -4;
    if (!compressed->d_old_k || !compressed->d_q4_v || !compressed->d_q4_scale || !dense->d_k || !dense->d_v)
        return M40LLM_ERR_UNSUPPORTED;  // only the FP16-K / q4-V backing is built
    if (m40_ensure_device(ctx) != 0) return -1;
    cudaStream_t s = ctx->decode_stream;
    const size_t ring_elems = (size_t)compressed->max_batch_size * compressed->num_heads * compressed->recent_window * compressed->head_dim;
    if (cudaMemsetAsync(compressed->d_recent_k, 0, ring_elems * sizeof(__half), s) != cudaSuccess ||
        cudaMemsetAsync(compressed->d_recent_v, 0, ring_elems * sizeof(__half), s) != cudaSuccess)
        return -5;
    if (seq_len > 0) {
        dim3 grid(seq_len, compressed->num_heads, compressed->max_batch_size);
        compress_from_dense_kernel<<<grid, 64, 0, s>>>(*dense, *compressed, seq_len);
        M40_COUNT_LAUNCH(ctx);
    }
    fill_u32_kernel<<<(compressed->max_batch_size + 127) / 128, 128, 0, s>>>(compressed->d_seq_map, seq_len, compressed->max_batch_size);
    M40_COUNT_LAUNCH(ctx);
    if (cudaGetLastError() != cudaSuccess) return -5;
    return cudaStreamSynchronize(s) == cudaSuccess ? 0 : -6;
}

int m40llm_kvcache_build_q8_old_from_dense(M40llmCudaContext* ctx, M40llmKVCache* kv, uint32_t seq_id,
                                           uint32_t seq_len, uint32_t recent_window) {
    (void)seq_id; (void)seq_len; (void)recent_window;
    if (!ctx || !kv) return -1;
    return M40LLM_ERR_UNSUPPORTED;
}

int m40llm_kvcache_debug_attention_telemetry(M40llmCudaContext* ctx, const M40llmKVCache* kv, uint32_t mode,
                                             uint32_t seq_id, const void* d_q_f32, uint32_t q_heads, uint32_t seq_len,
                                             uint32_t recent_window, uint32_t block_size, uint32_t top_blocks,
                                             uint32_t needle_block, M40llmAttentionTelemetry* out) {
    (void)mode; (void)seq_id; (void)q_heads; (void)seq_len; (void)recent_window; (void)block_size; (void)top_blocks;
    (void)needle_block;
    if (!ctx || !kv || !d_q_f32 || !out) return -1;
    return M40LLM_ERR_UNSUPPORTED;
}

}  // extern "C"
