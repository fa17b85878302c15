// RMSNorm, RoPE, residual add, SwiGLU and the cast/dequant helpers.
// All are HBM/latency-bound streaming kernels: 128-bit loads where alignment allows,
// warp-shuffle reductions, one pass over the data.
#include "common.cuh"

namespace {

// ---------------------------------------------------------------- RMSNorm
// One CTA per row. y = x * rsqrt(mean(x^2) + eps) [* w]   (cuda/kernels.cu:736-807)
template <int WDTYPE>  // -1 none, 0 f16, 1 f32
__global__ void __launch_bounds__(256) rms_norm_kernel(const float* __restrict__ in, const void* __restrict__ w,
                                                       float* __restrict__ out, uint32_t dim, float eps) {
    __shared__ float red[8];
    const float* x = in + (size_t)blockIdx.x * dim;
    float* y = out + (size_t)blockIdx.x * dim;
    const bool vec = (dim % 4u == 0u) && ((((uintptr_t)x | (uintptr_t)y) & 15u) == 0u);
    float ss = 0.0f;
    if (vec) {
        const float4* x4 = reinterpret_cast<const float4*>(x);
        for (uint32_t i = threadIdx.x; i < dim / 4u; i += blockDim.x) {
            const float4 v = x4[i];
            ss += v.x * v.x + v.y * v.y + v.z * v.z + v.w * v.w;
        }
    } else {
        for (uint32_t i = threadIdx.x; i < dim; i += blockDim.x) ss += x[i] * x[i];
    }
    ss = warp_sum(ss);
    if ((threadIdx.x & 31u) == 0u) red[threadIdx.x >> 5] = ss;
    __syncthreads();
    float tot = 0.0f;
#pragma unroll
    for (int i = 0; i < 8; ++i) tot += red[i];
    const float scale = rsqrtf(tot / static_cast<float>(dim) + eps);
    for (uint32_t i = threadIdx.x; i < dim; i += blockDim.x) {
        float v = x[i] * scale;
        if (WDTYPE == 0) v *= __half2float(reinterpret_cast<const __half*>(w)[i]);
        if (WDTYPE == 1) v *= reinterpret_cast<const float*>(w)[i];
        y[i] = v;
    }
}

// ------------------------------------------------------------------- RoPE
// One thread per (row, head, pair). layout 0: (2i, 2i+1); layout 1: (i, i + hd/2)
// (cuda/kernels.cu:5570-5585, 7300-7332).
__global__ void rope_kernel(float* __restrict__ x, float* __restrict__ x2, uint32_t rows, uint32_t heads,
                            uint32_t head_dim, uint32_t past_len, const uint32_t* __restrict__ past_len_dev,
                            float freq_base, float freq_scale, uint32_t layout) {
    const uint32_t half = head_dim / 2u;
    const uint32_t pairs_per_row = heads * half;
    const uint32_t idx = blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= rows * pairs_per_row) return;
    if (past_len_dev) past_len = *past_len_dev;
    const uint32_t row = idx / pairs_per_row;
    const uint32_t pr = idx % pairs_per_row;
    const uint32_t head = pr / half;
    const uint32_t i = pr % half;
    float c, s;
    rope_cs(past_len + row, i, head_dim, freq_base, freq_scale, &c, &s);
    const size_t base = ((size_t)row * heads + head) * head_dim;
    const size_t i0 = base + (layout == 1u ? i : 2u * i);
    const size_t i1 = layout == 1u ? i0 + half : i0 + 1u;
    const float a = x[i0], b = x[i1];
    x[i0] = a * c - b * s;
    x[i1] = a * s + b * c;
    if (x2) {
        const float a2 = x2[i0], b2 = x2[i1];
        x2[i0] = a2 * c - b2 * s;
        x2[i1] = a2 * s + b2 * c;
    }
}

__global__ void residual_add_kernel(const float* __restrict__ a, const float* __restrict__ b, float* __restrict__ o,
                                    size_t n) {
    const size_t stride = (size_t)gridDim.x * blockDim.x;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride) o[i] = a[i] + b[i];
}

__global__ void swiglu_kernel(const float* __restrict__ g, const float* __restrict__ u, float* __restrict__ o,
                              size_t n) {
    const size_t stride = (size_t)gridDim.x * blockDim.x;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride) {
        const float x = g[i];
        o[i] = (x / (1.0f + expf(-x))) * u[i];
    }
}

__global__ void f16_to_f32_kernel(const __half* __restrict__ in, float* __restrict__ out, size_t n) {
    const size_t stride = (size_t)gridDim.x * blockDim.x;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride) out[i] = __half2float(in[i]);
}

// Q8_0: 34-byte blocks {f16 d; int8 qs[32]} (cuda/kernels.cu:856-867). 2-byte aligned only.
__global__ void q80_to_f32_kernel(const uint8_t* __restrict__ in, float* __restrict__ out, size_t n) {
    const size_t stride = (size_t)gridDim.x * blockDim.x;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride) {
        const uint8_t* blk = in + (i / 32u) * 34u;
        const float d = __half2float(*reinterpret_cast<const __half*>(blk));
        out[i] = d * static_cast<float>(static_cast<int8_t>(blk[2u + (i % 32u)]));
    }
}

inline int grid_for(size_t n, int threads, int sm_count) {
    size_t blocks = (n + threads - 1) / threads;
    const size_t cap = (size_t)sm_count * 16;
    if (blocks > cap) blocks = cap;
    if (blocks == 0) blocks = 1;
    return (int)blocks;
}

int rms_norm_launch(M40llmCudaContext* ctx, const void* in, const void* w, void* out, uint32_t rows, uint32_t dim,
                    float eps, int wdtype) {
    if (rows == 0) return 0;
    cudaGetLastError();
    const float* x = reinterpret_cast<const float*>(in);
    float* y = reinterpret_cast<float*>(out);
    if (wdtype < 0) rms_norm_kernel<-1><<<rows, 256, 0, ctx->decode_stream>>>(x, nullptr, y, dim, eps);
    else if (wdtype == 0) rms_norm_kernel<0><<<rows, 256, 0, ctx->decode_stream>>>(x, w, y, dim, eps);
    else rms_norm_kernel<1><<<rows, 256, 0, ctx->decode_stream>>>(x, w, y, dim, eps);
    M40_COUNT_LAUNCH(ctx);
    return cudaGetLastError() == cudaSuccess ? 0 : -2;
}

int rope_launch(M40llmCudaContext* ctx, float* x, float* x2, uint32_t rows, uint32_t heads, uint32_t head_dim,
                uint32_t past_len, const uint32_t* past_len_dev, float base, float scale, uint32_t layout) {
    const uint32_t total = rows * (heads * head_dim / 2u);
    if (total == 0) return 0;
    const int threads = 256;
    rope_kernel<<<(total + threads - 1) / threads, threads, 0, ctx->decode_stream>>>(
        x, x2, rows, heads, head_dim, past_len, past_len_dev, base, scale, layout);
    M40_COUNT_LAUNCH(ctx);
    return cudaGetLastError() == cudaSuccess ? 0 : -3;
}

}  // namespace

// Internal: weighted RMSNorm of `rows` rows on the decode stream (used by the fused prologue).
int m40_rms_norm_rows(M40llmCudaContext* ctx, const void* in, const void* w, void* out, uint32_t rows, uint32_t dim,
                      float eps, uint32_t wdtype) {
    return rms_norm_launch(ctx, in, w, out, rows, dim, eps, (int)wdtype);
}

extern "C" {

int m40llm_rms_norm_f32_async(M40llmCudaContext* ctx, const void* d_in, void* d_out, uint32_t rows, uint32_t dim,
                              float eps) {
    if (!ctx || !d_in || !d_out || dim == 0) return -1;
    if (m40_ensure_device(ctx) != 0) return -1;
    return rms_norm_launch(ctx, d_in, nullptr, d_out, rows, dim, eps, -1);
}

int m40llm_rms_norm_f32(M40llmCudaContext* ctx, const void* d_in, void* d_out, uint32_t rows, uint32_t dim, float eps) {
    const int rc = m40llm_rms_norm_f32_async(ctx, d_in, d_out, rows, dim, eps);
    if (rc != 0) return rc;
    return cudaStreamSynchronize(ctx->decode_stream) == cudaSuccess ? 0 : -3;
}

int m40llm_rms_norm_f32_weighted_async(M40llmCudaContext* ctx, const void* d_in, const void* d_weight, void* d_out,
                                       uint32_t rows, uint32_t dim, float eps, uint32_t weight_dtype) {
    if (!ctx || !d_in || !d_weight || !d_out || dim == 0) return -1;
    if (weight_dtype > 1) return -4;
    if (m40_ensure_device(ctx) != 0) return -1;
    return rms_norm_launch(ctx, d_in, d_weight, d_out, rows, dim, eps, (int)weight_dtype);
}

int m40llm_rms_norm_f32_weighted(M40llmCudaContext* ctx, const void* d_in, const void* d_weight, void* d_out,
                                 uint32_t rows, uint32_t dim, float eps, uint32_t weight_dtype) {
    const int rc = m40llm_rms_norm_f32_weighted_async(ctx, d_in, d_weight, d_out, rows, dim, eps, weight_dtype);
    if (rc != 0) return rc;
    return cudaStreamSynchronize(ctx->decode_stream) == cudaSuccess ? 0 : -3;
}

int m40llm_rope_f32_layout_async(M40llmCudaContext* ctx, float* d_q, float* d_k, uint32_t rows, uint32_t num_heads,
                                 uint32_t head_dim, uint32_t past_len, float freq_base, float freq_scale,
                                 uint32_t rope_layout) {
    if (!ctx || !d_q || !d_k || head_dim == 0 || num_heads == 0) return -1;
    if (head_dim % 2 != 0) return -2;
    if (m40_ensure_device(ctx) != 0) return -1;
    return rope_launch(ctx, d_q, d_k, rows, num_heads, head_dim, past_len, nullptr, freq_base, freq_scale,
                       rope_layout);
}

int m40llm_rope_f32_async(M40llmCudaContext* ctx, float* d_q, float* d_k, uint32_t rows, uint32_t num_heads,
                          uint32_t head_dim, uint32_t past_len, float freq_base, float freq_scale) {
    return m40llm_rope_f32_layout_async(ctx, d_q, d_k, rows, num_heads, head_dim, past_len, freq_base, freq_scale, 0u);
}

int m40llm_rope_f32(M40llmCudaContext* ctx, float* d_q, float* d_k, uint32_t rows, uint32_t num_heads,
                    uint32_t head_dim, uint32_t past_len, float freq_base, float freq_scale) {
    const int rc = m40llm_rope_f32_async(ctx, d_q, d_k, rows, num_heads, head_dim, past_len, freq_base, freq_scale);
    if (rc != 0) return rc;
    return cudaStreamSynchronize(ctx->decode_stream) == cudaSuccess ? 0 : -4;
}

int m40llm_rope_f32_inplace_layout_async(M40llmCudaContext* ctx, float* d_x, uint32_t rows, uint32_t num_heads,
                                         uint32_t head_dim, uint32_t past_len, float freq_base, float freq_scale,
                                         uint32_t rope_layout) {
    if (!ctx || !d_x || head_dim == 0 || num_heads == 0) return -1;
    if (head_dim % 2 != 0) return -2;
    if (m40_ensure_device(ctx) != 0) return -1;
    return rope_launch(ctx, d_x, nullptr, rows, num_heads, head_dim, past_len, nullptr, freq_base, freq_scale,
                       rope_layout);
}

int m40llm_rope_f32_inplace_async(M40llmCudaContext* ctx, float* d_x, uint32_t rows, uint32_t num_heads,
                                  uint32_t head_dim, uint32_t past_len, float freq_base, float freq_scale) {
    return m40llm_rope_f32_inplace_layout_async(ctx, d_x, rows, num_heads, head_dim, past_len, freq_base, freq_scale,
                                                0u);
}

int m40llm_rope_f32_inplace(M40llmCudaContext* ctx, float* d_x, uint32_t rows, uint32_t num_heads, uint32_t head_dim,
                            uint32_t past_len, float freq_base, float freq_scale) {
    const int rc = m40llm_rope_f32_inplace_async(ctx, d_x, rows, num_heads, head_dim, past_len, freq_base, freq_scale);
    if (rc != 0) return rc;
    return cudaStreamSynchronize(ctx->decode_stream) == cudaSuccess ? 0 : -4;
}

int m40llm_rope_f32_inplace_position_dev_layout_async(M40llmCudaContext* ctx, float* d_x, uint32_t rows,
                                                      uint32_t num_heads, uint32_t head_dim,
                                                      const uint32_t* past_len_dev, float freq_base, float freq_scale,
                                                      uint32_t rope_layout) {
    if (!ctx || !d_x || !past_len_dev || head_dim == 0 || num_heads == 0) return -1;
    if (head_dim % 2 != 0) return -2;
    if (m40_ensure_device(ctx) != 0) return -1;
    return rope_launch(ctx, d_x, nullptr, rows, num_heads, head_dim, 0, past_len_dev, freq_base, freq_scale,
                       rope_layout);
}

int m40llm_rope_f32_inplace_position_dev_async(M40llmCudaContext* ctx, float* d_x, uint32_t rows, uint32_t num_heads,
                                               uint32_t head_dim, const uint32_t* past_len_dev, float freq_base,
                                               float freq_scale) {
    return m40llm_rope_f32_inplace_position_dev_layout_async(ctx, d_x, rows, num_heads, head_dim, past_len_dev,
                                                             freq_base, freq_scale, 0u);
}

int m40llm_residual_add_f32_async(M40llmCudaContext* ctx, const void* d_a, const void* d_b, void* d_out, size_t n) {
    if (!ctx || !d_a || !d_b || !d_out) return -1;
    if (m40_ensure_device(ctx) != 0) return -2;
    if (n == 0) return 0;
    residual_add_kernel<<<grid_for(n, 256, ctx->sm_count), 256, 0, ctx->decode_stream>>>(
        reinterpret_cast<const float*>(d_a), reinterpret_cast<const float*>(d_b), reinterpret_cast<float*>(d_out), n);
    M40_COUNT_LAUNCH(ctx);
    return cudaGetLastError() == cudaSuccess ? 0 : -3;
}

int m40llm_residual_add_f32(M40llmCudaContext* ctx, const void* d_a, const void* d_b, void* d_out, size_t n) {
    const int rc = m40llm_residual_add_f32_async(ctx, d_a, d_b, d_out, n);
    if (rc != 0) return rc;
    return cudaStreamSynchronize(ctx->decode_stream) == cudaSuccess ? 0 : -4;
}

int m40llm_swiglu_f32_async(M40llmCudaContext* ctx, const void* d_gate, const void* d_up, void* d_out, size_t n) {
    if (!ctx || !d_gate || !d_up || !d_out) return -1;
    if (m40_ensure_device(ctx) != 0) return -2;
    if (n == 0) return 0;
    swiglu_kernel<<<grid_for(n, 256, ctx->sm_count), 256, 0, ctx->decode_stream>>>(
        reinterpret_cast<const float*>(d_gate), reinterpret_cast<const float*>(d_up), reinterpret_cast<float*>(d_out),
        n);
    M40_COUNT_LAUNCH(ctx);
    return cudaGetLastError() == cudaSuccess ? 0 : -3;
}

int m40llm_swiglu_f32(M40llmCudaContext* ctx, const void* d_gate, const void* d_up, void* d_out, size_t n) {
    const int rc = m40llm_swiglu_f32_async(ctx, d_gate, d_up, d_out, n);
    if (rc != 0) return rc;
    return cudaStreamSynchronize(ctx->decode_stream) == cudaSuccess ? 0 : -4;
}

int m40llm_f16_to_f32(M40llmCudaContext* ctx, const void* d_in_f16, void* d_out_f32, size_t n) {
    if (!ctx || !d_in_f16 || !d_out_f32) return -1;
    if (m40_ensure_device(ctx) != 0) return -4;
    cudaGetLastError();
    if (((uintptr_t)d_in_f16 % alignof(__half)) != 0) return -3;
    if (n == 0) return 0;
    f16_to_f32_kernel<<<grid_for(n, 256, ctx->sm_count), 256, 0, ctx->prefill_stream>>>(
        reinterpret_cast<const __half*>(d_in_f16), reinterpret_cast<float*>(d_out_f32), n);
    M40_COUNT_LAUNCH(ctx);
    if (cudaGetLastError() != cudaSuccess) return -2;
    return cudaStreamSynchronize(ctx->prefill_stream) == cudaSuccess ? 0 : -3;
}

int m40llm_q80_to_f32(M40llmCudaContext* ctx, const void* d_in_q80, void* d_out_f32, size_t n) {
    if (!ctx || !d_in_q80 || !d_out_f32) return -1;
    if (m40_ensure_device(ctx) != 0) return -4;
    if (n == 0) return 0;
    q80_to_f32_kernel<<<grid_for(n, 256, ctx->sm_count), 256, 0, ctx->prefill_stream>>>(
        reinterpret_cast<const uint8_t*>(d_in_q80), reinterpret_cast<float*>(d_out_f32), n);
    M40_COUNT_LAUNCH(ctx);
    if (cudaGetLastError() != cudaSuccess) return -2;
    return cudaStreamSynchronize(ctx->prefill_stream) == cudaSuccess ? 0 : -3;
}

}  // extern "C"
