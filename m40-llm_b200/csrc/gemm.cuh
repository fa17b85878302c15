// Internal launch helpers of gemm.cu, shared with the fused layer paths.
#pragma once
#include "common.cuh"

// C[m][n] = sum_k A[m][k] * W[n][k] (+ bias[n]) (+ residual[m][n]); W f16 GGUF rows.
int m40_gemm_f32xf16_gguf(M40llmCudaContext* ctx, cudaStream_t s, const float* A, const __half* W, float* C, int M,
                          int N, int K, const float* bias, const float* residual);
int m40_gemm_dispatch_f16(M40llmCudaContext* ctx, cudaStream_t s, uint32_t stream_kind, const float* A,
                          const __half* W, float* C, int M, int N, int K, const float* bias, const float* residual);
// Same over Q8_0 rows (+ residual).
int m40_gemm_f32xq80_gguf(M40llmCudaContext* ctx, cudaStream_t s, const float* A, const uint8_t* W, float* C, int M,
                          int N, int K, const float* residual);
// hid[m][n] = silu(A.Wg[n]) * (A.Wu[n])
int m40_gate_up_swiglu_q80(M40llmCudaContext* ctx, cudaStream_t s, const float* A, const uint8_t* Wg,
                           const uint8_t* Wu, float* hid, int M, int F, int K);
int m40_gate_up_swiglu_f16(M40llmCudaContext* ctx, cudaStream_t s, const float* A, const __half* Wg, const __half* Wu,
                           float* hid, int M, int F, int K);

struct M40GemvNorm;
// SwiGLU FFN over Q8_0 (q80 != 0) or f16 weights with an optional RMSNorm folded into the batched path; returns 1
// when the norm could not be folded for this shape.
int m40_ffn_swiglu(M40llmCudaContext* ctx, uint32_t stream_kind, const void* d_x, const void* d_wg, const void* d_wu,
                   const void* d_wd, const void* d_residual, void* d_hid, void* d_out, uint32_t rows, uint32_t hidden,
                   uint32_t ffn, int q80, const M40GemvNorm* norm);

// Rows at which projections switch to the tcgen05 kernel (default 2; env M40LLM_TC_MIN_ROWS).
int m40_tc_min_rows();
