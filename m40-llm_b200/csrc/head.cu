// Model-level ends of the decode step: token embedding gather, the logits head (output RMSNorm + lm_head
// projection) and greedy arg-max on the device, so that a whole token step can be captured in one CUDA graph and
// replayed without the per-token device-to-host copy of vocab x 4 bytes the reference makes
// (src/infer/logits.rs:57-116, src/sampling.rs:95-108, src/infer/embeddings.rs:80-140).
#include "common.cuh"
#include "gemm.cuh"
#include "gemm_tc.cuh"
#include "gemv_stream.cuh"

int m40_rms_norm_rows(M40llmCudaContext* ctx, const void* in, const void* w, void* out, uint32_t rows, uint32_t dim,
                      float eps, uint32_t wdtype);

namespace {

// out[r][:] = f32(table[ids[r]][:]); an id outside the table raises status bit 8 and yields zeros.
__global__ void __launch_bounds__(256) embed_rows_f16_kernel(const __half* __restrict__ table,
                                                             const uint32_t* __restrict__ ids, float* __restrict__ out,
                                                             uint32_t hidden, uint32_t vocab, uint32_t* status) {
    pdl_wait();
    pdl_trigger();
    const uint32_t r = blockIdx.x, id = ids[r];
    const bool ok = id < vocab;
    if (!ok && threadIdx.x == 0) atomicOr(status, 8u);
    const __half* src = table + (size_t)(ok ? id : 0u) * hidden;
    float* dst = out + (size_t)r * hidden;
    for (uint32_t i = threadIdx.x; i < hidden; i += blockDim.x) dst[i] = ok ? __half2float(src[i]) : 0.0f;
}

// Greedy choice per row: the first index of the largest value under strict '>' from -inf, so NaN is never chosen
// and an all-NaN / all -inf row yields 0 (src/sampling.rs:95-108). One CTA per row.
__global__ void __launch_bounds__(1024) argmax_rows_kernel(const float* __restrict__ x, uint32_t n,
                                                           uint32_t* __restrict__ out) {
    __shared__ float sv[32];
    __shared__ uint32_t si[32];
    pdl_wait();
    pdl_trigger();
    const float* row = x + (size_t)blockIdx.x * n;
    float bv = -INFINITY;
    uint32_t bi = 0xffffffffu;  // "none yet": any real candidate beats it
    for (uint32_t i = threadIdx.x; i < n; i += blockDim.x) {
        const float v = row[i];
        if (v > bv) bv = v, bi = i;  // ascending i per thread: the first maximum is kept
    }
    auto better = [](float v, uint32_t i, float bv2, uint32_t bi2) { return v > bv2 || (v == bv2 && i < bi2); };
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
        const uint32_t oi = __shfl_xor_sync(0xffffffffu, bi, o);
        if (better(ov, oi, bv, bi)) bv = ov, bi = oi;
    }
    const uint32_t lane = threadIdx.x & 31u, warp = threadIdx.x >> 5;
    if (lane == 0) sv[warp] = bv, si[warp] = bi;
    __syncthreads();
    if (warp == 0) {
        const uint32_t nw = (blockDim.x + 31u) / 32u;
        bv = lane < nw ? sv[lane] : -INFINITY;
        bi = lane < nw ? si[lane] : 0xffffffffu;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
            const uint32_t oi = __shfl_xor_sync(0xffffffffu, bi, o);
            if (better(ov, oi, bv, bi)) bv = ov, bi = oi;
        }
        if (lane == 0) out[blockIdx.x] = bi == 0xffffffffu ? 0u : bi;
    }
}

__global__ void advance_rows_kernel(uint32_t* __restrict__ positions, uint32_t* __restrict__ lens, uint32_t rows) {
    pdl_wait();
    pdl_trigger();
    const uint32_t r = blockIdx.x * blockDim.x + threadIdx.x;
    if (r < rows) {
        if (positions) positions[r] += 1u;
        if (lens) lens[r] += 1u;
    }
}

}  // namespace

extern "C" {

int m40llm_embed_tokens_f16_async(M40llmCudaContext* ctx, const void* d_table_f16, const uint32_t* d_token_ids,
                                  void* d_out_f32, uint32_t rows, uint32_t hidden, uint32_t vocab) {
    if (!ctx || !d_table_f16 || !d_token_ids || !d_out_f32) return -1;
    if (rows == 0 || hidden == 0 || vocab == 0) return -2;
    if (m40_ensure_device(ctx) != 0) return -1;
    const cudaError_t e = m40_launch_dependent(embed_rows_f16_kernel, dim3(rows), dim3(256), 0, ctx->decode_stream,
                                               (const __half*)d_table_f16, d_token_ids, (float*)d_out_f32, hidden,
                                               vocab, ctx->d_status);
    M40_COUNT_LAUNCH(ctx);
    return e == cudaSuccess && cudaGetLastError() == cudaSuccess ? 0 : -3;
}

int m40llm_logits_head_f32_async(M40llmCudaContext* ctx, const void* d_hidden_f32, const void* d_norm_w,
                                 uint32_t norm_w_dtype, float eps, const void* d_lm_head_f16, void* d_logits_f32,
                                 uint32_t rows, uint32_t hidden, uint32_t vocab) {
    if (!ctx || !d_hidden_f32 || !d_lm_head_f16 || !d_logits_f32) return -1;
    if (rows == 0 || hidden == 0 || vocab == 0) return -2;
    if (d_norm_w && norm_w_dtype > 1) return -4;
    if (m40_ensure_device(ctx) != 0) return -1;
    cudaStream_t s = ctx->decode_stream;
    const M40GemvNorm norm = {d_norm_w, norm_w_dtype == 1u ? 1 : 0, eps, nullptr};
    const M40GemvNorm* np = d_norm_w ? &norm : nullptr;
    if (rows == 1) {
        const M40GemvSeg seg = {d_lm_head_f16, nullptr, (float*)d_logits_f32, nullptr, nullptr, (int)vocab};
        const int rc = m40_gemv_stream(ctx, s, (const float*)d_hidden_f32, (int)hidden, M40_GEMV_F16, 0, 1, &seg, np);
        if (rc != 1) return rc;
    }
    const void* wp[1] = {d_lm_head_f16};
    if ((int)rows >= m40_tc_min_rows() && hidden % 4 == 0 && m40_gemm_tc_supported((int)rows, (int)hidden, 1, wp)) {
        const __half* w[1] = {(const __half*)d_lm_head_f16};
        const int n[1] = {(int)vocab};
        float* o[1] = {(float*)d_logits_f32};
        return m40_gemm_tc_f16(ctx, s, 1u, (const float*)d_hidden_f32, (int)rows, (int)hidden, 1, w, n, o, nullptr,
                               nullptr, 0, np);
    }
    const float* x = (const float*)d_hidden_f32;
    if (d_norm_w) {
        float* xn = (float*)m40_ensure_scratch(ctx, 1, (size_t)rows * hidden * sizeof(float), 1);
        if (!xn) return -5;
        const int rc = m40_rms_norm_rows(ctx, d_hidden_f32, d_norm_w, xn, rows, hidden, eps, norm_w_dtype);
        if (rc != 0) return rc;
        x = xn;
    }
    return m40_gemm_f32xf16_gguf(ctx, s, x, (const __half*)d_lm_head_f16, (float*)d_logits_f32, (int)rows, (int)vocab,
                                 (int)hidden, nullptr, nullptr);
}

int m40llm_argmax_f32_async(M40llmCudaContext* ctx, const void* d_values_f32, uint32_t rows, uint32_t n,
                            uint32_t* d_out_index) {
    if (!ctx || !d_values_f32 || !d_out_index) return -1;
    if (rows == 0 || n == 0) return -2;
    if (m40_ensure_device(ctx) != 0) return -1;
    const cudaError_t e = m40_launch_dependent(argmax_rows_kernel, dim3(rows), dim3(1024), 0, ctx->decode_stream,
                                               (const float*)d_values_f32, n, d_out_index);
    M40_COUNT_LAUNCH(ctx);
    return e == cudaSuccess && cudaGetLastError() == cudaSuccess ? 0 : -3;
}

int m40llm_advance_positions_async(M40llmCudaContext* ctx, uint32_t* d_positions, uint32_t* d_lens, uint32_t rows) {
    if (!ctx || (!d_positions && !d_lens)) return -1;
    if (rows == 0) return -2;
    if (m40_ensure_device(ctx) != 0) return -1;
    const cudaError_t e = m40_launch_dependent(advance_rows_kernel, dim3((rows + 127) / 128), dim3(128), 0,
                                               ctx->decode_stream, d_positions, d_lens, rows);
    M40_COUNT_LAUNCH(ctx);
    return e == cudaSuccess && cudaGetLastError() == cudaSuccess ? 0 : -3;
}

}  // extern "C"
