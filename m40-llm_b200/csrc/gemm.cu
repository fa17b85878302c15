// GEMV / small-batch GEMM over streamed weights (f16 GGUF rows, Q8_0 GGUF rows, f16 row-major).
//
// These are HBM-bound at decode batch sizes: every weight byte is read once, activations
// come from L1/L2. The kernels stream weights with 128-bit no-allocate loads, keep several
// loads in flight per lane, accumulate in f32 and reduce with warp shuffles.
#include "common.cuh"
#include <stdlib.h>

#include "gemm.cuh"
#include "gemm_tc.cuh"
#include "gemv_stream.cuh"

int m40_tc_min_rows();

namespace {

__device__ __forceinline__ uint4 ldg_stream_u4(const void* p) {
    uint4 v;
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
                 : "l"(p));
    return v;
}

__device__ __forceinline__ float dot8_f16(const uint4& w, const float4& xa, const float4& xb) {
    const __half2* h = reinterpret_cast<const __half2*>(&w);
    const float2 w0 = __half22float2(h[0]), w1 = __half22float2(h[1]);
    const float2 w2 = __half22float2(h[2]), w3 = __half22float2(h[3]);
    float acc = xa.x * w0.x;
    acc = fmaf(xa.y, w0.y, acc);
    acc = fmaf(xa.z, w1.x, acc);
    acc = fmaf(xa.w, w1.y, acc);
    acc = fmaf(xb.x, w2.x, acc);
    acc = fmaf(xb.y, w2.y, acc);
    acc = fmaf(xb.z, w3.x, acc);
    acc = fmaf(xb.w, w3.y, acc);
    return acc;
}

// ---------------------------------------------------------------------------
// f16 GGUF rows: C[m][n] = sum_k A[m][k] * W[n][k].   (cuda/kernels.cu:5037-5052)
// One warp owns RW consecutive weight rows; lanes stride K in 16-byte pieces.
// MT activation rows are processed per pass over the weights.
// Requires K % 8 == 0 and 16-byte aligned A, W.
// ---------------------------------------------------------------------------
template <int MT, int RW>
__global__ void __launch_bounds__(256) gemv_f16_gguf_kernel(const float* __restrict__ A, const __half* __restrict__ W,
                                                            float* __restrict__ C, int M, int N, int K,
                                                            const float* __restrict__ bias,
                                                            const float* __restrict__ residual) {
    const int warp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    const int lane = threadIdx.x & 31;
    const int n0 = warp * RW;
    if (n0 >= N) return;
    for (int m0 = 0; m0 < M; m0 += MT) {
        float acc[MT][RW];
#pragma unroll
        for (int m = 0; m < MT; ++m)
#pragma unroll
            for (int r = 0; r < RW; ++r) acc[m][r] = 0.0f;
#pragma unroll 2
        for (int k = lane * 8; k < K; k += 256) {
            uint4 w[RW];
#pragma unroll
            for (int r = 0; r < RW; ++r) {
                const int n = n0 + r < N ? n0 + r : N - 1;
                w[r] = ldg_stream_u4(W + (size_t)n * K + k);
            }
#pragma unroll
            for (int m = 0; m < MT; ++m) {
                const int mm = m0 + m < M ? m0 + m : M - 1;
                const float4 xa = *reinterpret_cast<const float4*>(A + (size_t)mm * K + k);
                const float4 xb = *reinterpret_cast<const float4*>(A + (size_t)mm * K + k + 4);
#pragma unroll
                for (int r = 0; r < RW; ++r) acc[m][r] += dot8_f16(w[r], xa, xb);
            }
        }
#pragma unroll
        for (int m = 0; m < MT; ++m)
#pragma unroll
            for (int r = 0; r < RW; ++r) {
                const float v = warp_sum(acc[m][r]);
                if (lane == 0 && m0 + m < M && n0 + r < N) {
                    float o = v;
                    if (bias) o += bias[n0 + r];
                    if (residual) o += residual[(size_t)(m0 + m) * N + n0 + r];
                    C[(size_t)(m0 + m) * N + n0 + r] = o;
                }
            }
    }
}

// Scalar fallback for shapes/alignments the vector kernel does not take.
__global__ void gemm_f32xf16_gguf_naive_kernel(const float* __restrict__ A, const __half* __restrict__ W,
                                               float* __restrict__ C, int M, int N, int K,
                                               const float* __restrict__ bias, const float* __restrict__ residual) {
    const int warp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    const int lane = threadIdx.x & 31;
    if (warp >= M * N) return;
    const int m = warp / N, n = warp % N;
    float acc = 0.0f;
    for (int k = lane; k < K; k += 32) acc = fmaf(A[(size_t)m * K + k], __half2float(W[(size_t)n * K + k]), acc);
    acc = warp_sum(acc);
    if (lane == 0) {
        if (bias) acc += bias[n];
        if (residual) acc += residual[(size_t)m * N + n];
        C[(size_t)m * N + n] = acc;
    }
}

// ---------------------------------------------------------------------------
// Q8_0 GGUF rows: 34-byte blocks {f16 d; int8 q[32]}, value d*q (cuda/kernels.cu:856-867).
// C[m][n] = sum_k A[m][k] * d[n][k/32] * q[n][k].
// One warp per weight row; a lane owns 4 consecutive weights of a 128-weight slice, so the
// activation loads are fully coalesced float4s. Weight bytes are only 2-byte aligned in the
// raw GGUF layout, so they are fetched as two u16 loads (the warp still touches each sector once).
// MODE 0: plain; MODE 1: two weight matrices (gate, up) sharing x with the SwiGLU epilogue.
// ---------------------------------------------------------------------------
__device__ __forceinline__ void q80_unpack4(uint32_t q, float d, float* w) {
    // bytes -> exact floats: (q ^ 0x80) as unsigned u in [0,255]; 0x4B000000|u = 2^23 + u.
    const uint32_t u = q ^ 0x80808080u;
    const float magic = 8388608.0f + 128.0f;
    w[0] = (__uint_as_float(__byte_perm(u, 0x4B000000u, 0x7650)) - magic) * d;
    w[1] = (__uint_as_float(__byte_perm(u, 0x4B000000u, 0x7651)) - magic) * d;
    w[2] = (__uint_as_float(__byte_perm(u, 0x4B000000u, 0x7652)) - magic) * d;
    w[3] = (__uint_as_float(__byte_perm(u, 0x4B000000u, 0x7653)) - magic) * d;
}

template <int MT, int MODE>
__global__ void __launch_bounds__(256) gemv_q80_gguf_kernel(const float* __restrict__ A, const uint8_t* __restrict__ W,
                                                            const uint8_t* __restrict__ W2, float* __restrict__ C,
                                                            int M, int N, int K, const float* __restrict__ residual) {
    const int warp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    const int lane = threadIdx.x & 31;
    if (warp >= N) return;
    const size_t row_bytes = (size_t)(K / 32) * 34;
    const uint8_t* wr = W + (size_t)warp * row_bytes;
    const uint8_t* wr2 = MODE == 1 ? W2 + (size_t)warp * row_bytes : nullptr;
    const int sub = lane >> 3;        // which of the 4 blocks in a 128-weight slice
    const int part = (lane & 7) * 4;  // byte offset inside the block's 32 weights
    for (int m0 = 0; m0 < M; m0 += MT) {
        float acc[MT], acc2[MT];
#pragma unroll
        for (int m = 0; m < MT; ++m) acc[m] = acc2[m] = 0.0f;
#pragma unroll 4
        for (int k = 0; k < K; k += 128) {
            const size_t boff = (size_t)(k / 32 + sub) * 34;
            float w[4], w2[4];
            {
                const uint16_t* p = reinterpret_cast<const uint16_t*>(wr + boff);
                const float d = __half2float(__ushort_as_half(__ldg(p)));
                const uint32_t lo = __ldg(p + 1 + part / 2), hi = __ldg(p + 2 + part / 2);
                q80_unpack4(lo | (hi << 16), d, w);
            }
            if (MODE == 1) {
                const uint16_t* p = reinterpret_cast<const uint16_t*>(wr2 + boff);
                const float d = __half2float(__ushort_as_half(__ldg(p)));
                const uint32_t lo = __ldg(p + 1 + part / 2), hi = __ldg(p + 2 + part / 2);
                q80_unpack4(lo | (hi << 16), d, w2);
            }
#pragma unroll
            for (int m = 0; m < MT; ++m) {
                const int mm = m0 + m < M ? m0 + m : M - 1;
                const float4 x = *reinterpret_cast<const float4*>(A + (size_t)mm * K + k + lane * 4);
                acc[m] = fmaf(x.x, w[0], acc[m]);
                acc[m] = fmaf(x.y, w[1], acc[m]);
                acc[m] = fmaf(x.z, w[2], acc[m]);
                acc[m] = fmaf(x.w, w[3], acc[m]);
                if (MODE == 1) {
                    acc2[m] = fmaf(x.x, w2[0], acc2[m]);
                    acc2[m] = fmaf(x.y, w2[1], acc2[m]);
                    acc2[m] = fmaf(x.z, w2[2], acc2[m]);
                    acc2[m] = fmaf(x.w, w2[3], acc2[m]);
                }
            }
        }
#pragma unroll
        for (int m = 0; m < MT; ++m) {
            float v = warp_sum(acc[m]);
            float v2 = MODE == 1 ? warp_sum(acc2[m]) : 0.0f;
            if (lane == 0 && m0 + m < M) {
                if (MODE == 1) v = (v / (1.0f + expf(-v))) * v2;  // silu(gate) * up
                if (residual) v += residual[(size_t)(m0 + m) * N + warp];
                C[(size_t)(m0 + m) * N + warp] = v;
            }
        }
    }
}

// Generic Q8_0 fallback (K % 32 == 0 only): one warp per output, lane = weight within block.
__global__ void gemm_q80_naive_kernel(const float* __restrict__ A, const uint8_t* __restrict__ W,
                                      float* __restrict__ C, int M, int N, int K) {
    const int warp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    const int lane = threadIdx.x & 31;
    if (warp >= M * N) return;
    const int m = warp / N, n = warp % N;
    const uint8_t* wr = W + (size_t)n * (size_t)(K / 32) * 34;
    float acc = 0.0f;
    for (int kb = 0; kb < K / 32; ++kb) {
        const uint8_t* blk = wr + (size_t)kb * 34;
        const float d = __half2float(*reinterpret_cast<const __half*>(blk));
        acc = fmaf(A[(size_t)m * K + kb * 32 + lane], d * (float)(int8_t)blk[2 + lane], acc);
    }
    acc = warp_sum(acc);
    if (lane == 0) C[(size_t)m * N + n] = acc;
}

// f16 GGUF gate+up with SwiGLU epilogue: hid[m][n] = silu(x.Wg[n]) * (x.Wu[n]).
template <int MT>
__global__ void __launch_bounds__(256) gemv_f16_gate_up_kernel(const float* __restrict__ A,
                                                               const __half* __restrict__ Wg,
                                                               const __half* __restrict__ Wu, float* __restrict__ C,
                                                               int M, int N, int K) {
    const int warp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    const int lane = threadIdx.x & 31;
    if (warp >= N) return;
    for (int m0 = 0; m0 < M; m0 += MT) {
        float ag[MT], au[MT];
#pragma unroll
        for (int m = 0; m < MT; ++m) ag[m] = au[m] = 0.0f;
#pragma unroll 2
        for (int k = lane * 8; k < K; k += 256) {
            const uint4 wg = ldg_stream_u4(Wg + (size_t)warp * K + k);
            const uint4 wu = ldg_stream_u4(Wu + (size_t)warp * K + k);
#pragma unroll
            for (int m = 0; m < MT; ++m) {
                const int mm = m0 + m < M ? m0 + m : M - 1;
                const float4 xa = *reinterpret_cast<const float4*>(A + (size_t)mm * K + k);
                const float4 xb = *reinterpret_cast<const float4*>(A + (size_t)mm * K + k + 4);
                ag[m] += dot8_f16(wg, xa, xb);
                au[m] += dot8_f16(wu, xa, xb);
            }
        }
#pragma unroll
        for (int m = 0; m < MT; ++m) {
            const float g = warp_sum(ag[m]);
            const float u = warp_sum(au[m]);
            if (lane == 0 && m0 + m < M) C[(size_t)(m0 + m) * N + warp] = (g / (1.0f + expf(-g))) * u;
        }
    }
}

// ---------------------------------------------------------------------------
// Row-major B [K][N] (m40llm_gemm_f16xf16_f32 / f32xf16_f32, cuda/kernels.cu:4999-5032).
// C[m][n] = sum_k A[m][k] * B[k][n]. Columns are contiguous, so a lane owns 8 columns
// (16 bytes) and the K range of the CTA is split over its 16 thread rows; partial sums
// meet in shared memory. grid.y splits K further; split partials go to scratch and a
// second kernel adds them in a fixed order (deterministic, no atomics).
// ---------------------------------------------------------------------------
template <typename AT>
__device__ __forceinline__ float load_a(const AT* p);
template <>
__device__ __forceinline__ float load_a<float>(const float* p) { return *p; }
template <>
__device__ __forceinline__ float load_a<__half>(const __half* p) { return __half2float(*p); }

template <typename AT, int MT>
__global__ void __launch_bounds__(256) gemm_rowmajor_b_kernel(const AT* __restrict__ A, const __half* __restrict__ B,
                                                              float* __restrict__ out, int M, int N, int K,
                                                              int k_per_split, int m0) {
    __shared__ float red[16][MT][128 + 4];
    const int tx = threadIdx.x & 15;   // 16 lanes x 8 columns = 128 columns per CTA
    const int ty = threadIdx.x >> 4;   // 16 k-rows
    const int n = blockIdx.x * 128 + tx * 8;
    const int kb = blockIdx.y * k_per_split;
    const int ke = min(K, kb + k_per_split);
    float acc[MT][8];
#pragma unroll
    for (int m = 0; m < MT; ++m)
#pragma unroll
        for (int j = 0; j < 8; ++j) acc[m][j] = 0.0f;
    if (n < N) {
#pragma unroll 4
        for (int k = kb + ty; k < ke; k += 16) {
            const uint4 w = ldg_stream_u4(B + (size_t)k * N + n);
            const __half2* h = reinterpret_cast<const __half2*>(&w);
            float wf[8];
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const float2 f = __half22float2(h[j]);
                wf[2 * j] = f.x;
                wf[2 * j + 1] = f.y;
            }
#pragma unroll
            for (int m = 0; m < MT; ++m) {
                const int mm = m0 + m < M ? m0 + m : M - 1;
                const float a = load_a<AT>(A + (size_t)mm * K + k);
#pragma unroll
                for (int j = 0; j < 8; ++j) acc[m][j] = fmaf(a, wf[j], acc[m][j]);
            }
        }
    }
#pragma unroll
    for (int m = 0; m < MT; ++m)
#pragma unroll
        for (int j = 0; j < 8; ++j) red[ty][m][tx * 8 + j] = acc[m][j];
    __syncthreads();
    // 256 threads reduce MT*128 outputs over the 16 k-rows
    for (int o = threadIdx.x; o < MT * 128; o += 256) {
        const int m = o / 128, c = o % 128;
        float s = 0.0f;
#pragma unroll
        for (int r = 0; r < 16; ++r) s += red[r][m][c];
        const int nn = blockIdx.x * 128 + c;
        if (nn < N && m0 + m < M) out[((size_t)blockIdx.y * M + (m0 + m)) * N + nn] = s;
    }
}

__global__ void reduce_splits_kernel(const float* __restrict__ part, float* __restrict__ C, size_t mn, int splits) {
    const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= mn) return;
    float s = 0.0f;
    for (int p = 0; p < splits; ++p) s += part[(size_t)p * mn + i];
    C[i] = s;
}

template <typename AT>
__global__ void gemm_rowmajor_naive_kernel(const AT* __restrict__ A, const __half* __restrict__ B,
                                           float* __restrict__ C, __half* __restrict__ C16, int M, int N, int K) {
    const int n = blockIdx.x * blockDim.x + threadIdx.x;
    const int m = blockIdx.y;
    if (n >= N || m >= M) return;
    float acc = 0.0f;
    for (int k = 0; k < K; ++k) acc = fmaf(load_a<AT>(A + (size_t)m * K + k), __half2float(B[(size_t)k * N + n]), acc);
    if (C) C[(size_t)m * N + n] = acc;
    if (C16) C16[(size_t)m * N + n] = __float2half_rn(acc);
}

// A f32 [M,K] x Bt f32 (Bt[k*N+n]) -> C; the layout m40llm_materialize_* produces (kernels.cu:5217-5242).
__global__ void gemm_f32xf32_nt_kernel(const float* __restrict__ A, const float* __restrict__ Bt,
                                       float* __restrict__ C, int M, int N, int K) {
    const int n = blockIdx.x * blockDim.x + threadIdx.x;
    const int m = blockIdx.y;
    if (n >= N || m >= M) return;
    float acc = 0.0f;
    for (int k = 0; k < K; ++k) acc = fmaf(A[(size_t)m * K + k], Bt[(size_t)k * N + n], acc);
    C[(size_t)m * N + n] = acc;
}

__global__ void materialize_nt_kernel(const __half* __restrict__ B, float* __restrict__ Bt, int N, int K) {
    // tile transpose through shared memory so both sides are coalesced
    __shared__ float tile[32][33];
    const int k0 = blockIdx.x * 32, n0 = blockIdx.y * 32;
    for (int j = threadIdx.y; j < 32; j += blockDim.y) {
        const int n = n0 + j, k = k0 + threadIdx.x;
        tile[j][threadIdx.x] = (n < N && k < K) ? __half2float(B[(size_t)n * K + k]) : 0.0f;
    }
    __syncthreads();
    for (int j = threadIdx.y; j < 32; j += blockDim.y) {
        const int k = k0 + j, n = n0 + threadIdx.x;
        if (n < N && k < K) Bt[(size_t)k * N + n] = tile[threadIdx.x][j];
    }
}

bool aligned16(const void* p) { return (((uintptr_t)p) & 15u) == 0u; }

template <int RW>
int launch_gemv_f16(M40llmCudaContext* ctx, cudaStream_t s, const float* A, const __half* W, float* C, int M, int N,
                    int K, const float* bias, const float* residual) {
    const int warps = (N + RW - 1) / RW;
    const int blocks = (warps + 7) / 8;
    if (M == 1) gemv_f16_gguf_kernel<1, RW><<<blocks, 256, 0, s>>>(A, W, C, M, N, K, bias, residual);
    else if (M == 2) gemv_f16_gguf_kernel<2, RW><<<blocks, 256, 0, s>>>(A, W, C, M, N, K, bias, residual);
    else gemv_f16_gguf_kernel<4, RW><<<blocks, 256, 0, s>>>(A, W, C, M, N, K, bias, residual);
    M40_COUNT_LAUNCH(ctx);
    return cudaGetLastError() == cudaSuccess ? 0 : -2;
}

}  // namespace

// ------------------------------------------------------------------ internal API (gemm.cuh)
int m40_gemm_f32xf16_gguf(M40llmCudaContext* ctx, cudaStream_t s, const float* A, const __half* W, float* C, int M,
                          int N, int K, const float* bias, const float* residual) {
    if (M <= 0 || N <= 0 || K <= 0) return 0;
    if (M == 1) {  // one row: the bulk-copy streaming kernel, when the shape is one it takes
        const M40GemvSeg seg = {W, nullptr, C, bias, residual, N};
        const int rc = m40_gemv_stream(ctx, s, A, K, M40_GEMV_F16, 0, 1, &seg, nullptr);
        if (rc != 1) return rc;
    }
    if (K % 8 == 0 && aligned16(A) && aligned16(W)) {
        // Two rows per warp once there are enough rows to fill the machine with 256-thread CTAs.
        if (N >= ctx->sm_count * 16) return launch_gemv_f16<2>(ctx, s, A, W, C, M, N, K, bias, residual);
        return launch_gemv_f16<1>(ctx, s, A, W, C, M, N, K, bias, residual);
    }
    const long long warps = (long long)M * N;
    gemm_f32xf16_gguf_naive_kernel<<<(unsigned)((warps + 7) / 8), 256, 0, s>>>(A, W, C, M, N, K, bias, residual);
    M40_COUNT_LAUNCH(ctx);
    return cudaGetLastError() == cudaSuccess ? 0 : -2;
}

int m40_gemm_f32xq80_gguf(M40llmCudaContext* ctx, cudaStream_t s, const float* A, const uint8_t* W, float* C, int M,
                          int N, int K, const float* residual) {
    if (M <= 0 || N <= 0 || K <= 0) return 0;
    if (K % 32 != 0) return -2;
    if (M == 1) {
        const M40GemvSeg seg = {W, nullptr, C, nullptr, residual, N};
        const int rc = m40_gemv_stream(ctx, s, A, K, M40_GEMV_Q80, 0, 1, &seg, nullptr);
        if (rc != 1) return rc;
    }
    if (K % 128 == 0 && aligned16(A) && (((uintptr_t)W) & 1u) == 0u) {
        const int blocks = (N + 7) / 8;
        if (M == 1) gemv_q80_gguf_kernel<1, 0><<<blocks, 256, 0, s>>>(A, W, nullptr, C, M, N, K, residual);
        else if (M == 2) gemv_q80_gguf_kernel<2, 0><<<blocks, 256, 0, s>>>(A, W, nullptr, C, M, N, K, residual);
        else gemv_q80_gguf_kernel<4, 0><<<blocks, 256, 0, s>>>(A, W, nullptr, C, M, N, K, residual);
        M40_COUNT_LAUNCH(ctx);
        return cudaGetLastError() == cudaSuccess ? 0 : -2;
    }
    if (residual) return -2;
    const long long warps = (long long)M * N;
    gemm_q80_naive_kernel<<<(unsigned)((warps + 7) / 8), 256, 0, s>>>(A, W, C, M, N, K);
    M40_COUNT_LAUNCH(ctx);
    return cudaGetLastError() == cudaSuccess ? 0 : -2;
}

// Q8_0 projections for batched rows on the tensor cores, 64 rows per pass. Returns 1 when not applicable.
static int q80_tc_rows(M40llmCudaContext* ctx, cudaStream_t s, uint32_t stream_kind, const float* A, int M, int K,
                       int problems, const uint8_t* const* W, const int* N, float* const* out, const float* residual,
                       int mode, const M40GemvNorm* norm = nullptr, const M40TcChain* chain = nullptr) {
    const void* wp[3] = {W[0], problems > 1 ? W[1] : W[0], problems > 2 ? W[2] : W[0]};
    if (M < m40_tc_min_rows() || !m40_gemm_tc_q80_supported(M < 64 ? M : 64, K, problems, wp)) return 1;
    if (norm && norm->w && M % 64 == 1) return 1;  // a single trailing row would need the un-normalised path
    for (int m0 = 0; m0 < M; m0 += 64) {
        const int rows = M - m0 < 64 ? M - m0 : 64;
        if (rows < 2) {  // a single trailing row: CUDA-core kernel
            if (mode == 1) {
                const int rc1 = m40_gate_up_swiglu_q80(ctx, s, A + (size_t)m0 * K, W[0], W[1], out[0] + (size_t)m0 * N[0], 1, N[0], K);
                if (rc1 != 0) return rc1;
            } else {
                for (int p = 0; p < problems; ++p) {
                    const int rc1 = m40_gemm_f32xq80_gguf(ctx, s, A + (size_t)m0 * K, W[p], out[p] + (size_t)m0 * N[p], 1, N[p], K,
                                                          residual ? residual + (size_t)m0 * N[p] : nullptr);
                    if (rc1 != 0) return rc1;
                }
            }
            continue;
        }
        float* o[3];
        const float* r[3];
        for (int p = 0; p < problems; ++p) {
            o[p] = out[p] ? out[p] + (size_t)m0 * N[p] : nullptr;
            r[p] = residual ? residual + (size_t)m0 * N[p] : nullptr;
        }
        const int rc = m40_gemm_tc_q80(ctx, s, stream_kind, A + (size_t)m0 * K, rows, K, problems, W, N, o, r, mode, norm,
                                       M <= 64 ? chain : nullptr);
        if (rc != 0) return rc;
    }
    return 0;
}

int m40_gate_up_swiglu_q80(M40llmCudaContext* ctx, cudaStream_t s, const float* A, const uint8_t* Wg,
                           const uint8_t* Wu, float* hid, int M, int F, int K) {
    if (M == 1) {
        const M40GemvSeg seg = {Wg, Wu, hid, nullptr, nullptr, F};
        const int rc = m40_gemv_stream(ctx, s, A, K, M40_GEMV_Q80, 1, 1, &seg, nullptr);
        if (rc != 1) return rc;
    }
    if (K % 128 != 0 || !aligned16(A) || ((((uintptr_t)Wg) | ((uintptr_t)Wu)) & 1u) != 0u) return -2;
    const int blocks = (F + 7) / 8;
    if (M == 1) gemv_q80_gguf_kernel<1, 1><<<blocks, 256, 0, s>>>(A, Wg, Wu, hid, M, F, K, nullptr);
    else if (M == 2) gemv_q80_gguf_kernel<2, 1><<<blocks, 256, 0, s>>>(A, Wg, Wu, hid, M, F, K, nullptr);
    else gemv_q80_gguf_kernel<4, 1><<<blocks, 256, 0, s>>>(A, Wg, Wu, hid, M, F, K, nullptr);
    M40_COUNT_LAUNCH(ctx);
    return cudaGetLastError() == cudaSuccess ? 0 : -2;
}

int m40_gate_up_swiglu_f16(M40llmCudaContext* ctx, cudaStream_t s, const float* A, const __half* Wg, const __half* Wu,
                           float* hid, int M, int F, int K) {
    if (M == 1) {
        const M40GemvSeg seg = {Wg, Wu, hid, nullptr, nullptr, F};
        const int rc = m40_gemv_stream(ctx, s, A, K, M40_GEMV_F16, 1, 1, &seg, nullptr);
        if (rc != 1) return rc;
    }
    if (K % 8 != 0 || !aligned16(A) || !aligned16(Wg) || !aligned16(Wu)) return -2;
    const int blocks = (F + 7) / 8;
    if (M == 1) gemv_f16_gate_up_kernel<1><<<blocks, 256, 0, s>>>(A, Wg, Wu, hid, M, F, K);
    else if (M == 2) gemv_f16_gate_up_kernel<2><<<blocks, 256, 0, s>>>(A, Wg, Wu, hid, M, F, K);
    else gemv_f16_gate_up_kernel<4><<<blocks, 256, 0, s>>>(A, Wg, Wu, hid, M, F, K);
    M40_COUNT_LAUNCH(ctx);
    return cudaGetLastError() == cudaSuccess ? 0 : -2;
}

// Rows at which projections switch from the CUDA-core GEMV to the tcgen05 kernel.
int m40_tc_min_rows() {
    static int v = -1;
    if (v < 0) {
        const char* e = getenv("M40LLM_TC_MIN_ROWS");
        v = e ? atoi(e) : 2;
        if (v < 2) v = 2;
    }
    return v;
}

// Chooses the kernel for a GGUF-f16 projection by batch size: CUDA-core GEMV for one row (or when the
// shape does not fit the tensor-core kernel), the tcgen05 kernel for batched rows.
int m40_gemm_dispatch_f16(M40llmCudaContext* ctx, cudaStream_t s, uint32_t stream_kind, const float* A,
                          const __half* W, float* C, int M, int N, int K, const float* bias, const float* residual) {
    const void* wp[1] = {W};
    if (M >= m40_tc_min_rows() && m40_gemm_tc_supported(M, K, 1, wp)) {
        const __half* w[1] = {W};
        const int n[1] = {N};
        float* o[1] = {C};
        const float* b[1] = {bias};
        const float* r[1] = {residual};
        return m40_gemm_tc_f16(ctx, s, stream_kind, A, M, K, 1, w, n, o, b, r, 0);
    }
    return m40_gemm_f32xf16_gguf(ctx, s, A, W, C, M, N, K, bias, residual);
}

namespace {

template <typename AT>
int gemm_rowmajor_b(M40llmCudaContext* ctx, const AT* A, const __half* B, float* C, int M, int N, int K) {
    cudaStream_t s = ctx->prefill_stream;
    if (N % 8 != 0 || !aligned16(B)) {
        dim3 grid((N + 127) / 128, M);
        gemm_rowmajor_naive_kernel<AT><<<grid, 128, 0, s>>>(A, B, C, nullptr, M, N, K);
        M40_COUNT_LAUNCH(ctx);
        return cudaGetLastError() == cudaSuccess ? 0 : -2;
    }
    const int col_blocks = (N + 127) / 128;
    int splits = (ctx->sm_count * 2 + col_blocks - 1) / col_blocks;
    const int max_splits = (K + 255) / 256;
    if (splits > max_splits) splits = max_splits;
    if (splits < 1) splits = 1;
    const int k_per_split = (((K + splits - 1) / splits) + 15) / 16 * 16;
    splits = (K + k_per_split - 1) / k_per_split;
    float* out = C;
    if (splits > 1) {
        out = (float*)m40_ensure_scratch(ctx, 0, (size_t)splits * M * N * sizeof(float));
        if (!out) return -2;
    }
    dim3 grid(col_blocks, splits);
    for (int m0 = 0; m0 < M; m0 += 4) {
        const int mt = M - m0;
        if (mt >= 3) gemm_rowmajor_b_kernel<AT, 4><<<grid, 256, 0, s>>>(A, B, out, M, N, K, k_per_split, m0);
        else if (mt == 2) gemm_rowmajor_b_kernel<AT, 2><<<grid, 256, 0, s>>>(A, B, out, M, N, K, k_per_split, m0);
        else gemm_rowmajor_b_kernel<AT, 1><<<grid, 256, 0, s>>>(A, B, out, M, N, K, k_per_split, m0);
        M40_COUNT_LAUNCH(ctx);
    }
    if (splits > 1) {
        const size_t mn = (size_t)M * N;
        reduce_splits_kernel<<<(unsigned)((mn + 255) / 256), 256, 0, s>>>(out, C, mn, splits);
        M40_COUNT_LAUNCH(ctx);
    }
    return cudaGetLastError() == cudaSuccess ? 0 : -2;
}

}  // namespace

// The SwiGLU FFN (gate|up with the SiLU*up epilogue, then down + residual) over Q8_0 or f16 GGUF weights.
// `norm` (optional) is applied to x on the fly by the batched tensor-core path; returns 1 when a norm was asked for
// but the shape went to a path that cannot fold it (the caller then normalises explicitly and calls again).
int m40_ffn_swiglu(M40llmCudaContext* ctx, uint32_t stream_kind, const void* d_x, const void* d_wg, const void* d_wu,
                   const void* d_wd, const void* d_residual, void* d_hid, void* d_out, uint32_t rows, uint32_t hidden,
                   uint32_t ffn, int q80, const M40GemvNorm* norm) {
    cudaStream_t s = m40_stream(ctx, stream_kind);
    const bool want_norm = norm && norm->w;
    int rc;
    if (q80) {
        // One pass of up to 64 rows on the tensor cores: the SwiGLU epilogue hands the down projection its
        // activations already split into f16 hi | lo (one launch and one pass over hid fewer).
        M40TcChain first = {}, second = {};
        bool chained = false;
        {
            const void* wp[3] = {d_wg, d_wu, d_wd};
            if ((int)rows >= m40_tc_min_rows() && rows <= 64 && m40_gemm_tc_q80_supported((int)rows, (int)hidden, 2, wp) &&
                m40_gemm_tc_q80_supported((int)rows, (int)ffn, 1, wp + 2)) {
                const int n1[2] = {(int)ffn, (int)ffn}, n2[1] = {(int)hidden};
                size_t act1, part1, act2, part2;
                m40_gemm_tc_q80_scratch(ctx, (int)rows, (int)hidden, 2, n1, &act1, &part1);
                m40_gemm_tc_q80_scratch(ctx, (int)rows, (int)ffn, 1, n2, &act2, &part2);
                size_t front = 2 * act1 + part1;
                if (part2 > front) front = part2;
                front = (front + 1023) & ~(size_t)1023;
                first.scratch_bytes = second.scratch_bytes = front + 2 * act2;
                first.act_off = second.act_off = front;
                first.write_split = 1;
                second.read_split = 1;
                chained = true;
            }
        }
        {
            const uint8_t* w[2] = {(const uint8_t*)d_wg, (const uint8_t*)d_wu};
            const int n[2] = {(int)ffn, (int)ffn};
            float* o[2] = {(float*)d_hid, nullptr};
            rc = q80_tc_rows(ctx, s, stream_kind, (const float*)d_x, (int)rows, (int)hidden, 2, w, n, o, nullptr, 1, norm,
                             chained ? &first : nullptr);
        }
        if (rc == 1) {
            chained = false;
            if (want_norm) return 1;
            rc = m40_gate_up_swiglu_q80(ctx, s, (const float*)d_x, (const uint8_t*)d_wg, (const uint8_t*)d_wu,
                                        (float*)d_hid, (int)rows, (int)ffn, (int)hidden);
        }
        if (rc != 0) return rc;
        {
            const uint8_t* w[1] = {(const uint8_t*)d_wd};
            const int n[1] = {(int)hidden};
            float* o[1] = {(float*)d_out};
            rc = q80_tc_rows(ctx, s, stream_kind, (const float*)d_hid, (int)rows, (int)ffn, 1, w, n, o,
                             (const float*)d_residual, 0, nullptr, chained ? &second : nullptr);
        }
        if (rc != 1) return rc;
        return m40_gemm_f32xq80_gguf(ctx, s, (const float*)d_hid, (const uint8_t*)d_wd, (float*)d_out, (int)rows,
                                     (int)hidden, (int)ffn, (const float*)d_residual);
    }
    const void* wp[2] = {d_wg, d_wu};
    if ((int)rows >= m40_tc_min_rows() && m40_gemm_tc_supported((int)rows, (int)hidden, 2, wp)) {
        const __half* w[2] = {(const __half*)d_wg, (const __half*)d_wu};
        const int n[2] = {(int)ffn, (int)ffn};
        float* o[2] = {(float*)d_hid, nullptr};
        rc = m40_gemm_tc_f16(ctx, s, stream_kind, (const float*)d_x, (int)rows, (int)hidden, 2, w, n, o, nullptr, nullptr,
                             1, norm);
    } else {
        if (want_norm) return 1;
        rc = m40_gate_up_swiglu_f16(ctx, s, (const float*)d_x, (const __half*)d_wg, (const __half*)d_wu, (float*)d_hid,
                                    (int)rows, (int)ffn, (int)hidden);
    }
    if (rc != 0) return rc;
    return m40_gemm_dispatch_f16(ctx, s, stream_kind, (const float*)d_hid, (const __half*)d_wd, (float*)d_out, (int)rows,
                                 (int)hidden, (int)ffn, nullptr, (const float*)d_residual);
}

extern "C" {

int m40llm_gemm_f16xf16_f32(M40llmCudaContext* ctx, const void* d_A_f16, const void* d_B_f16, void* d_C_f32, int M,
                            int N, int K) {
    if (!ctx) return -1;
    if (!d_A_f16 || !d_B_f16 || !d_C_f32 || M <= 0 || N <= 0 || K <= 0) return -1;
    if (m40_ensure_device(ctx) != 0) return -1;
    const int rc = gemm_rowmajor_b<__half>(ctx, (const __half*)d_A_f16, (const __half*)d_B_f16, (float*)d_C_f32, M, N, K);
    if (rc != 0) return rc;
    return cudaStreamSynchronize(ctx->prefill_stream) == cudaSuccess ? 0 : -3;
}

int m40llm_gemm_f32xf16_f32(M40llmCudaContext* ctx, const void* d_A_f32, const void* d_B_f16, void* d_C_f32, int M,
                            int N, int K) {
    if (!ctx) return -1;
    if (!d_A_f32 || !d_B_f16 || !d_C_f32 || M <= 0 || N <= 0 || K <= 0) return -1;
    if (m40_ensure_device(ctx) != 0) return -1;
    const int rc = gemm_rowmajor_b<float>(ctx, (const float*)d_A_f32, (const __half*)d_B_f16, (float*)d_C_f32, M, N, K);
    if (rc != 0) return rc;
    return cudaStreamSynchronize(ctx->prefill_stream) == cudaSuccess ? 0 : -3;
}

int m40llm_gemm_f16_storage_f32_compute(M40llmCudaContext* ctx, const void* d_A, const void* d_B, void* d_C, int M,
                                        int N, int K) {
    if (!ctx) return -1;
    if (!d_A || !d_B || !d_C || M <= 0 || N <= 0 || K <= 0) return -1;
    if (m40_ensure_device(ctx) != 0) return -1;
    dim3 grid((N + 127) / 128, M);
    gemm_rowmajor_naive_kernel<__half><<<grid, 128, 0, ctx->prefill_stream>>>(
        (const __half*)d_A, (const __half*)d_B, nullptr, (__half*)d_C, M, N, K);
    M40_COUNT_LAUNCH(ctx);
    if (cudaGetLastError() != cudaSuccess) return -2;
    return cudaStreamSynchronize(ctx->prefill_stream) == cudaSuccess ? 0 : -3;
}

int m40llm_gemm_f32xf16_gguf_f32_async(M40llmCudaContext* ctx, const void* d_A_f32, const void* d_B_f16,
                                       void* d_C_f32, int M, int N, int K, uint32_t stream_kind) {
    if (!ctx || !d_A_f32 || !d_B_f16 || !d_C_f32) return -1;
    if (M <= 0 || N <= 0 || K <= 0) return -2;
    if (m40_ensure_device(ctx) != 0) return -1;
    cudaStream_t s = m40_stream(ctx, stream_kind);
    if (!s) return -4;
    return m40_gemm_dispatch_f16(ctx, s, stream_kind, (const float*)d_A_f32, (const __half*)d_B_f16, (float*)d_C_f32,
                                 M, N, K, nullptr, nullptr);
}

int m40llm_gemm_f32xf16_gguf_f32(M40llmCudaContext* ctx, const void* d_A_f32, const void* d_B_f16, void* d_C_f32,
                                 int M, int N, int K) {
    if (!ctx) return -1;
    const int rc = m40llm_gemm_f32xf16_gguf_f32_async(ctx, d_A_f32, d_B_f16, d_C_f32, M, N, K, 0u);
    if (rc != 0) return rc;
    return cudaStreamSynchronize(ctx->prefill_stream) == cudaSuccess ? 0 : -3;
}

int m40llm_gemm_f32xq80_gguf_f32_async(M40llmCudaContext* ctx, const void* d_A_f32, const void* d_B_q80,
                                       void* d_C_f32, int M, int N, int K, uint32_t stream_kind) {
    if (!ctx || !d_A_f32 || !d_B_q80 || !d_C_f32) return -1;
    if (M <= 0 || N <= 0 || K <= 0 || K % 32 != 0) return -2;
    if (m40_ensure_device(ctx) != 0) return -1;
    cudaStream_t s = m40_stream(ctx, stream_kind);
    if (!s) return -4;
    {
        const uint8_t* w[1] = {(const uint8_t*)d_B_q80};
        const int n[1] = {N};
        float* o[1] = {(float*)d_C_f32};
        const int rc = q80_tc_rows(ctx, s, stream_kind, (const float*)d_A_f32, M, K, 1, w, n, o, nullptr, 0);
        if (rc != 1) return rc;
    }
    return m40_gemm_f32xq80_gguf(ctx, s, (const float*)d_A_f32, (const uint8_t*)d_B_q80, (float*)d_C_f32, M, N, K,
                                 nullptr);
}

int m40llm_gemm_f32xf32_f32_async(M40llmCudaContext* ctx, const void* d_A_f32, const void* d_B_f32_colmajor_nt,
                                  void* d_C_f32, int M, int N, int K) {
    if (!ctx || !d_A_f32 || !d_B_f32_colmajor_nt || !d_C_f32) return -1;
    if (M <= 0 || N <= 0 || K <= 0) return -2;
    if (m40_ensure_device(ctx) != 0) return -1;
    dim3 grid((N + 127) / 128, M);
    gemm_f32xf32_nt_kernel<<<grid, 128, 0, ctx->prefill_stream>>>((const float*)d_A_f32,
                                                                   (const float*)d_B_f32_colmajor_nt,
                                                                   (float*)d_C_f32, M, N, K);
    M40_COUNT_LAUNCH(ctx);
    return cudaGetLastError() == cudaSuccess ? 0 : -3;
}

int m40llm_gemm_f32xf32_f32(M40llmCudaContext* ctx, const void* d_A_f32, const void* d_B_f32_colmajor_nt,
                            void* d_C_f32, int M, int N, int K) {
    const int rc = m40llm_gemm_f32xf32_f32_async(ctx, d_A_f32, d_B_f32_colmajor_nt, d_C_f32, M, N, K);
    if (rc != 0) return rc;
    return cudaStreamSynchronize(ctx->prefill_stream) == cudaSuccess ? 0 : -4;
}

int m40llm_materialize_gguf_f16_to_f32_colmajor_nt(M40llmCudaContext* ctx, const void* d_B_f16,
                                                   void* d_B_f32_colmajor_nt, int N, int K) {
    if (!ctx || !d_B_f16 || !d_B_f32_colmajor_nt) return -1;
    if (N <= 0 || K <= 0) return -2;
    if (m40_ensure_device(ctx) != 0) return -1;
    dim3 grid((K + 31) / 32, (N + 31) / 32), block(32, 8);
    materialize_nt_kernel<<<grid, block, 0, ctx->prefill_stream>>>((const __half*)d_B_f16,
                                                                   (float*)d_B_f32_colmajor_nt, N, K);
    M40_COUNT_LAUNCH(ctx);
    if (cudaGetLastError() != cudaSuccess) return -3;
    return cudaStreamSynchronize(ctx->prefill_stream) == cudaSuccess ? 0 : -4;
}

int m40llm_ffn_swiglu_q80_f32_async(M40llmCudaContext* ctx, const void* d_x_f32, const void* d_wg_q80,
                                    const void* d_wu_q80, const void* d_wd_q80, const void* d_residual_f32,
                                    void* d_hid_f32, void* d_out_f32, uint32_t rows, uint32_t hidden, uint32_t ffn,
                                    uint32_t stream_kind) {
    if (!ctx || !d_x_f32 || !d_wg_q80 || !d_wu_q80 || !d_wd_q80 || !d_hid_f32 || !d_out_f32) return -1;
    if (rows == 0 || hidden == 0 || ffn == 0 || hidden % 128 != 0 || ffn % 128 != 0) return -2;
    if (m40_ensure_device(ctx) != 0) return -1;
    if (!m40_stream(ctx, stream_kind)) return -4;
    return m40_ffn_swiglu(ctx, stream_kind, d_x_f32, d_wg_q80, d_wu_q80, d_wd_q80, d_residual_f32, d_hid_f32, d_out_f32,
                          rows, hidden, ffn, 1, nullptr);
}

int m40llm_ffn_swiglu_f16_f32_async(M40llmCudaContext* ctx, const void* d_x_f32, const void* d_wg_f16,
                                    const void* d_wu_f16, const void* d_wd_f16, const void* d_residual_f32,
                                    void* d_hid_f32, void* d_out_f32, uint32_t rows, uint32_t hidden, uint32_t ffn,
                                    uint32_t stream_kind) {
    if (!ctx || !d_x_f32 || !d_wg_f16 || !d_wu_f16 || !d_wd_f16 || !d_hid_f32 || !d_out_f32) return -1;
    if (rows == 0 || hidden == 0 || ffn == 0 || hidden % 8 != 0 || ffn % 8 != 0) return -2;
    if (m40_ensure_device(ctx) != 0) return -1;
    if (!m40_stream(ctx, stream_kind)) return -4;
    return m40_ffn_swiglu(ctx, stream_kind, d_x_f32, d_wg_f16, d_wu_f16, d_wd_f16, d_residual_f32, d_hid_f32, d_out_f32,
                          rows, hidden, ffn, 0, nullptr);
}

}  // extern "C"
