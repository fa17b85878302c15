// Internal interface of the single-row weight-streaming GEMV (gemv_stream.cu).
#pragma once
#include "common.cuh"

// One weight matrix of a grouped launch: out[n] = x . W[n] (+ bias[n]) (+ residual[n]), n < N.
// In gate/up mode W is the gate matrix and W2 the up matrix: out[n] = silu(x . W[n]) * (x . W2[n]).
struct M40GemvSeg {
    const void* W;
    const void* W2;
    float* out;
    const float* bias;
    const float* residual;
    int N;
};

// Optional RMSNorm applied to x on the fly (each CTA normalises its own copy): x <- x * rsqrt(mean(x^2)+eps) * w.
struct M40GemvNorm {
    const void* w;    // null: no normalisation
    int w_is_f32;     // 1: f32 weights, 0: f16
    float eps;
    float* xn_out;    // optional: CTA 0 also writes the normalised row here
};

enum { M40_GEMV_F16 = 0, M40_GEMV_Q80 = 1 };

// Streams up to three weight matrices that share one activation row x [K] (f32) in a single launch.
// Returns 0 when launched, 1 when the shape/alignment is not one this kernel takes (caller falls back),
// < 0 on a launch failure.
int m40_gemv_stream(M40llmCudaContext* ctx, cudaStream_t s, const float* x, int K, int fmt, int gate_up, int nseg,
                    const M40GemvSeg* segs, const M40GemvNorm* norm);
