// Tensor-core (tcgen05) weight-streaming GEMM for batched decode rows; see gemm_tc.cu.
#pragma once
#include "common.cuh"
#include "gemv_stream.cuh"  // M40GemvNorm

// Optional tail of a three-problem (Wq | Wk | Wv) call: the epilogue applies RoPE (adjacent pairs) to q and k per row
// position, writes q, and appends k / v as f16 to a dense cache, instead of storing f32 k / v for a separate launch.
// Needs every N to be a multiple of 128 and of head_dim.
struct M40TcRopeAppend {
    const uint32_t* seq_ids;
    const uint32_t* positions;
    __half* d_k;
    __half* d_v;
    uint32_t* d_seq_map;
    uint32_t* status;
    uint32_t head_dim, kv_heads, max_seq_len, max_batch;
    float freq_base, freq_scale;
    const float* inv_freq;  // host-made inverse-frequency table [head_dim / 2] or null (see m40_rope_inv_freq)
};

// True when the tcgen05 path can take this problem set (2 <= M <= 256, K % 8 == 0, 16-byte aligned weights).
bool m40_gemm_tc_supported(int M, int K, int problems, const void* const* W);

// Up to three GGUF-layout f16 weight matrices W[p] ([N[p]][K]) applied to the same activations X [M][K] f32.
// mode 0: out[p][m][n] = X.W[p]^T (+ bias[p][n]) (+ residual[p][m][n]); bias / residual arrays or entries may be null.
// mode 1: two problems (gate, up) of equal N: out[0][m][n] = silu(X.Wg^T) * (X.Wu^T).
int m40_gemm_tc_f16(M40llmCudaContext* ctx, cudaStream_t s, uint32_t stream_kind, const float* X, int M, int K,
                    int problems, const __half* const* W, const int* N, float* const* out, const float* const* bias,
                    const float* const* residual, int mode, const M40GemvNorm* norm = nullptr,
                    const M40TcRopeAppend* rope = nullptr);
// `norm` (optional): RMSNorm applied to X while it is split into f16 hi/lo (saves the separate norm pass).

// Two Q8_0 tensor-core calls chained through the f16 hi | lo copies the second one consumes (gate|up -> down): the
// first call's epilogue writes its result already split, the second skips its split pass. Both calls request
// `scratch_bytes` of stream scratch; the split copies live at byte offset `act_off` (hi, then lo), past everything
// either call keeps in front of it.
struct M40TcChain {
    size_t scratch_bytes;
    size_t act_off;
    int write_split;  // this call: epilogue also writes out[0] as f16 hi | lo at act_off
    int read_split;   // this call: the activations are already split at act_off
};
// Scratch one Q8_0 tensor-core call needs: bytes of one f16 activation copy and of its partial tiles.
void m40_gemm_tc_q80_scratch(const M40llmCudaContext* ctx, int M, int K, int problems, const int* N, size_t* act_bytes,
                             size_t* part_bytes);

// Same over Q8_0 GGUF rows (K % 256 == 0, 2 <= M <= 64 per call). mode 0: out[p] = X.W[p]^T (+ residual[p]);
// mode 1: out[0] = silu(X.Wg^T) * (X.Wu^T).
bool m40_gemm_tc_q80_supported(int M, int K, int problems, const void* const* W);
int m40_gemm_tc_q80(M40llmCudaContext* ctx, cudaStream_t s, uint32_t stream_kind, const float* X, int M, int K,
                    int problems, const uint8_t* const* W, const int* N, float* const* out,
                    const float* const* residual, int mode, const M40GemvNorm* norm = nullptr,
                    const M40TcChain* chain = nullptr);
// The f32 -> f16 hi/lo split (with optional RMSNorm per row) shared by both tensor-core paths.
int m40_split_activations(M40llmCudaContext* ctx, cudaStream_t s, const float* X, __half* hi, __half* lo, int M, int K,
                          const M40GemvNorm* norm);
