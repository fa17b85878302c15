// Last-token (decode) GQA attention over the dense FP16 KV cache.
//
// Work decomposition (flash-decoding): one CTA per (sequence, kv head, KV split). A CTA
// serves ALL q heads of its kv head from one read of K and V (the reference launches one
// CTA per q head and re-reads K/V G times: cuda/kernels.cu:1493-1573). Splits write
// unnormalised partials (m, l, o[hd]) that a merge kernel combines; with one split the
// CTA normalises and writes the output itself.
//
// Semantics: softmax(q.K^T / sqrt(hd)) V over tokens [0, seq_len) with f16 storage and
// f32 arithmetic, equal to the reference's three-pass host form (src/cuda.rs:4561-4628)
// up to f32 summation order.
#include <stdlib.h>

#include "attention.cuh"
#include "common.cuh"

namespace {

// ---------------------------------------------------------------------------
// Generic kernel: any head_dim <= 256, any group size (processed GC heads at a time).
// Warp w of the CTA takes tokens t0+w, t0+w+4, ...; a lane owns dims lane, lane+32, ...
// This is the correctness path for shapes the tiled kernel does not take.
// ---------------------------------------------------------------------------
template <int DJ, int GC>
__global__ void __launch_bounds__(128) attn_decode_generic_kernel(DenseAttnArgs a) {
    extern __shared__ float sm[];
    const uint32_t split = blockIdx.x, kvh = blockIdx.y, row = blockIdx.z;
    const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31u;
    const uint32_t hd = a.hd, G = a.q_heads / a.kv_heads;
    uint32_t seq = 0, t0 = 0, t1 = 0;
    if (!attn_resolve_row(a, row, split, &seq, &t0, &t1)) {
        attn_write_rejected_row(a, row, split, kvh, a.write_partials || a.splits > 1);
        return;
    }
    const __half* Kh = a.K + kv_row_offset(seq, kvh, 0, a.kv_heads, a.max_seq_len, hd);
    const __half* Vh = a.V + kv_row_offset(seq, kvh, 0, a.kv_heads, a.max_seq_len, hd);
    float* sm_m = sm;                    // [4][GC]
    float* sm_l = sm + 4 * GC;           // [4][GC]
    float* sm_o = sm + 8 * GC;           // [4][GC][hd]
    for (uint32_t g0 = 0; g0 < G; g0 += GC) {
        float qr[GC][DJ], acc[GC][DJ], m[GC], l[GC];
#pragma unroll
        for (int g = 0; g < GC; ++g) {
            m[g] = -INFINITY;
            l[g] = 0.0f;
            const uint32_t h = kvh * G + g0 + g;
#pragma unroll
            for (int j = 0; j < DJ; ++j) {
                const uint32_t d = lane + 32u * j;
                qr[g][j] = (g0 + g < G && d < hd) ? a.q[((size_t)row * a.q_heads + h) * hd + d] : 0.0f;
                acc[g][j] = 0.0f;
            }
        }
        for (uint32_t t = t0 + warp; t < t1; t += 4u) {
            float kx[DJ], vx[DJ];
#pragma unroll
            for (int j = 0; j < DJ; ++j) {
                const uint32_t d = lane + 32u * j;
                kx[j] = d < hd ? __half2float(Kh[(size_t)t * hd + d]) : 0.0f;
                vx[j] = d < hd ? __half2float(Vh[(size_t)t * hd + d]) : 0.0f;
            }
#pragma unroll
            for (int g = 0; g < GC; ++g) {
                float dot = 0.0f;
#pragma unroll
                for (int j = 0; j < DJ; ++j) dot = fmaf(qr[g][j], kx[j], dot);
                const float s = warp_sum(dot) * a.inv_sqrt;
                const float mn = fmaxf(m[g], s);
                const float corr = expf(m[g] - mn);  // m = -inf on the first token: exp(-inf) = 0
                const float p = expf(s - mn);
                l[g] = l[g] * corr + p;
#pragma unroll
                for (int j = 0; j < DJ; ++j) acc[g][j] = fmaf(p, vx[j], acc[g][j] * corr);
                m[g] = mn;
            }
        }
        // combine the 4 warps
        __syncthreads();
#pragma unroll
        for (int g = 0; g < GC; ++g) {
            if (lane == 0) {
                sm_m[warp * GC + g] = m[g];
                sm_l[warp * GC + g] = l[g];
            }
#pragma unroll
            for (int j = 0; j < DJ; ++j) {
                const uint32_t d = lane + 32u * j;
                if (d < hd) sm_o[((size_t)warp * GC + g) * hd + d] = acc[g][j];
            }
        }
        __syncthreads();
        for (uint32_t idx = threadIdx.x; idx < GC * hd; idx += blockDim.x) {
            const uint32_t g = idx / hd, d = idx % hd;
            if (g0 + g >= G) continue;
            float M = -INFINITY;
#pragma unroll
            for (int w = 0; w < 4; ++w) M = fmaxf(M, sm_m[w * GC + g]);
            float L = 0.0f, O = 0.0f;
#pragma unroll
            for (int w = 0; w < 4; ++w) {
                const float mw = sm_m[w * GC + g];
                const float e = mw == -INFINITY ? 0.0f : expf(mw - M);
                L += sm_l[w * GC + g] * e;
                O += sm_o[((size_t)w * GC + g) * hd + d] * e;
            }
            const uint32_t h = kvh * G + g0 + g;
            if (a.write_partials || a.splits > 1) {
                const size_t pi = ((size_t)row * a.q_heads + h) * a.splits + split;
                if (d == 0) {
                    a.part_m[pi] = M;
                    a.part_l[pi] = L;
                }
                a.part_o[pi * hd + d] = O;
            } else {
                a.out[((size_t)row * a.q_heads + h) * hd + d] = O / (L > 0.0f ? L : 1.0f);
            }
        }
    }
}

// Merge split partials: grid (q_heads, rows), block 128.
__global__ void __launch_bounds__(128) attn_merge_kernel(const float* __restrict__ pm, const float* __restrict__ pl,
                                                         const float* __restrict__ po, float* __restrict__ out,
                                                         uint32_t q_heads, uint32_t hd, uint32_t splits,
                                                         size_t part_stride_m, size_t part_stride_o,
                                                         uint32_t strided) {
    // strided == 0: partials laid out [row][head][split]; strided == 1: [split][head] (rank-major, one row)
    const uint32_t h = blockIdx.x, row = blockIdx.y;
    float M = -INFINITY;
    for (uint32_t s = 0; s < splits; ++s) {
        const size_t i = strided ? (size_t)s * part_stride_m + h : ((size_t)row * q_heads + h) * splits + s;
        if (pl[i] > 0.0f) M = fmaxf(M, pm[i]);
    }
    float L = 0.0f;
    for (uint32_t s = 0; s < splits; ++s) {
        const size_t i = strided ? (size_t)s * part_stride_m + h : ((size_t)row * q_heads + h) * splits + s;
        if (pl[i] > 0.0f) L += pl[i] * expf(pm[i] - M);
    }
    const float inv = 1.0f / (L > 0.0f ? L : 1.0f);
    for (uint32_t d = threadIdx.x; d < hd; d += blockDim.x) {
        float O = 0.0f;
        for (uint32_t s = 0; s < splits; ++s) {
            const size_t i = strided ? (size_t)s * part_stride_m + h : ((size_t)row * q_heads + h) * splits + s;
            const size_t oi = strided ? ((size_t)s * part_stride_o + (size_t)h * hd + d) : (i * hd + d);
            if (pl[i] > 0.0f) O += po[oi] * expf(pm[i] - M);
        }
        out[((size_t)row * q_heads + h) * hd + d] = O * inv;
    }
}

// The same merge with the work spread over the CTA: split s's weight exp(m_s - M) is computed once by thread s,
// the output accumulation runs as 8 split groups x (hd/4) float4 lanes with independent loads, and the groups
// meet in shared memory in a fixed order. Takes hd % 4 == 0, hd <= 128, splits <= 256 and 16-byte aligned partials.
// With fold_m / fold_l given the result is left unnormalised and its (max, sum) are written too: the fold of one
// rank's splits into ONE triple per head for the split-K exchange.
__global__ void __launch_bounds__(256) attn_merge_wide_kernel(const float* __restrict__ pm, const float* __restrict__ pl,
                                                              const float* __restrict__ po, float* __restrict__ out,
                                                              uint32_t q_heads, uint32_t hd, uint32_t splits,
                                                              size_t part_stride_m, size_t part_stride_o,
                                                              uint32_t strided, float* __restrict__ fold_m = nullptr,
                                                              float* __restrict__ fold_l = nullptr) {
    __shared__ float sw[256];
    __shared__ float sred[8];
    __shared__ float4 sacc[8][32];
    pdl_wait();
    pdl_trigger();
    const uint32_t tid = threadIdx.x, lane = tid & 31u, warp = tid >> 5;
    const uint32_t h = blockIdx.x, row = blockIdx.y;
    const size_t base = ((size_t)row * q_heads + h) * splits;
    float m = -INFINITY, l = 0.0f;
    if (tid < splits) {
        const size_t i = strided ? (size_t)tid * part_stride_m + h : base + tid;
        l = pl[i];
        m = l > 0.0f ? pm[i] : -INFINITY;
    }
    float M = m;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) M = fmaxf(M, __shfl_xor_sync(0xffffffffu, M, o));
    if (lane == 0) sred[warp] = M;
    __syncthreads();
    M = sred[0];
#pragma unroll
    for (int i = 1; i < 8; ++i) M = fmaxf(M, sred[i]);
    const float e = l > 0.0f ? expf(m - M) : 0.0f;
    sw[tid] = e;
    float L = warp_sum(l * e);
    __syncthreads();  // everyone has read sred (max) before it is reused for the sum
    if (lane == 0) sred[warp] = L;
    __syncthreads();
    L = 0.0f;
#pragma unroll
    for (int i = 0; i < 8; ++i) L += sred[i];
    const float inv = fold_m ? 1.0f : 1.0f / (L > 0.0f ? L : 1.0f);
    if (fold_m && tid == 0) {
        fold_m[(size_t)row * q_heads + h] = M;
        fold_l[(size_t)row * q_heads + h] = L;
    }
    const uint32_t vl = hd / 4u;            // float4 lanes per split (<= 32)
    const uint32_t g = tid / 32u, v = lane;  // split group, float4 lane
    float4 acc = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
    if (v < vl) {
#pragma unroll 4
        for (uint32_t s = g; s < splits; s += 8u) {
            const float w = sw[s];
            const size_t oi = strided ? ((size_t)s * part_stride_o + (size_t)h * hd) : ((base + s) * hd);
            const float4 x = *reinterpret_cast<const float4*>(po + oi + 4u * v);
            if (w != 0.0f) {  // empty splits may hold anything
                acc.x = fmaf(w, x.x, acc.x);
                acc.y = fmaf(w, x.y, acc.y);
                acc.z = fmaf(w, x.z, acc.z);
                acc.w = fmaf(w, x.w, acc.w);
            }
        }
    }
    sacc[g][v] = acc;
    __syncthreads();
    if (g == 0 && v < vl) {
        float4 t = sacc[0][v];
#pragma unroll
        for (int i = 1; i < 8; ++i) {
            const float4 u = sacc[i][v];
            t.x += u.x, t.y += u.y, t.z += u.z, t.w += u.w;
        }
        t.x *= inv, t.y *= inv, t.z *= inv, t.w *= inv;
        *reinterpret_cast<float4*>(out + ((size_t)row * q_heads + h) * hd + 4u * v) = t;
    }
}

static bool merge_wide_ok(const float* o, const float* out, uint32_t hd, uint32_t splits, size_t stride_o) {
    return hd % 4u == 0u && hd <= 128u && splits <= 256u && stride_o % 4u == 0u &&
           ((((uintptr_t)o) | ((uintptr_t)out)) & 15u) == 0u;
}

// Fold split partials of one row into ONE unnormalised triple per head (split-K rank output).
// grid q_heads, block 128. In: [head][split] ; out: m[head], l[head], o[head][hd].
__global__ void __launch_bounds__(128) attn_fold_kernel(const float* __restrict__ pm, const float* __restrict__ pl,
                                                        const float* __restrict__ po, uint32_t hd, uint32_t splits,
                                                        float* __restrict__ om, float* __restrict__ ol,
                                                        float* __restrict__ oo) {
    const uint32_t h = blockIdx.x;
    float M = -INFINITY;
    for (uint32_t s = 0; s < splits; ++s)
        if (pl[(size_t)h * splits + s] > 0.0f) M = fmaxf(M, pm[(size_t)h * splits + s]);
    float L = 0.0f;
    for (uint32_t s = 0; s < splits; ++s) {
        const size_t i = (size_t)h * splits + s;
        if (pl[i] > 0.0f) L += pl[i] * expf(pm[i] - M);
    }
    for (uint32_t d = threadIdx.x; d < hd; d += blockDim.x) {
        float O = 0.0f;
        for (uint32_t s = 0; s < splits; ++s) {
            const size_t i = (size_t)h * splits + s;
            if (pl[i] > 0.0f) O += po[i * hd + d] * expf(pm[i] - M);
        }
        oo[(size_t)h * hd + d] = O;
    }
    if (threadIdx.x == 0) {
        om[h] = M;
        ol[h] = L;
    }
}

int launch_generic(M40llmCudaContext* ctx, const DenseAttnArgs& a, uint32_t rows) {
    dim3 grid(a.splits, a.kv_heads, rows);
    const uint32_t dj = (a.hd + 31u) / 32u;
    constexpr int GC = 4;
    const size_t smem = (size_t)(8 * GC + 4 * GC * a.hd) * sizeof(float);
    cudaStream_t s = ctx->decode_stream;
    if (dj <= 1) attn_decode_generic_kernel<1, GC><<<grid, 128, smem, s>>>(a);
    else if (dj <= 2) attn_decode_generic_kernel<2, GC><<<grid, 128, smem, s>>>(a);
    else if (dj <= 4) attn_decode_generic_kernel<4, GC><<<grid, 128, smem, s>>>(a);
    else attn_decode_generic_kernel<8, GC><<<grid, 128, smem, s>>>(a);
    M40_COUNT_LAUNCH(ctx);
    return cudaGetLastError() == cudaSuccess ? 0 : -4;
}

}  // namespace

// ------------------------------------------------------------------ internal API
void m40_attn_pick_chunk(const M40llmCudaContext* ctx, uint32_t rows, uint32_t kv_heads, uint32_t max_tokens,
                         uint32_t* chunk, uint32_t* splits) {
    // Aim for ~2 CTAs per SM over the whole launch (one resident wave: a single 8K-token sequence measured 4 us
    // faster per layer step with 256-token chunks than with 128-token ones, whose second wave is mostly ramp).
    // Chunks are fixed-size so that variable-length batches produce CTAs of equal cost (CTAs past a row's length
    // exit at once); never shorter than 128 tokens.
    static int min_chunk_env = -1, max_chunk_env = -1;
    if (min_chunk_env < 0) {
        const char* e = getenv("M40LLM_ATTN_MIN_CHUNK");
        min_chunk_env = e ? atoi(e) : 0;
        if (min_chunk_env < 64) min_chunk_env = 128;
        const char* x = getenv("M40LLM_ATTN_MAX_CHUNK");
        max_chunk_env = x ? atoi(x) : 0;
        if (max_chunk_env < min_chunk_env) max_chunk_env = 1024;
    }
    const uint64_t work = (uint64_t)rows * kv_heads * max_tokens;
    const uint64_t target = (uint64_t)ctx->sm_count * 2u;
    uint64_t c = (work + target - 1) / target;
    if (c < (uint64_t)min_chunk_env) c = (uint64_t)min_chunk_env;
    if (c > (uint64_t)max_chunk_env) c = (uint64_t)max_chunk_env;
    c = (c + 63) & ~(uint64_t)63;
    uint32_t s = (uint32_t)((max_tokens + c - 1) / c);
    if (s > 128u) {
        c = ((max_tokens + 127u) / 128u + 63u) & ~(uint64_t)63;
        s = (uint32_t)((max_tokens + c - 1) / c);
    }
    if (s < 1u) s = 1u;
    *chunk = (uint32_t)c;
    *splits = s;
}

int m40_attention_dense(M40llmCudaContext* ctx, const M40llmKVCache* kv, const M40DenseAttnCall& c) {
    DenseAttnArgs a;
    a.K = kv->d_k;
    a.V = kv->d_v;
    a.q = c.q;
    a.out = c.out;
    a.seq_ids = c.seq_ids;
    a.seq_lens = c.seq_lens;
    a.seq_len_dev = c.seq_len_dev;
    a.status = ctx->d_status;
    a.seq_id = c.seq_id;
    a.seq_len = c.seq_len;
    a.tok_begin = c.tok_begin;
    a.tok_end = c.tok_end;
    a.range_mode = c.range_mode;
    a.max_seq_len = kv->max_seq_len;
    a.max_batch = kv->max_batch_size;
    a.kv_heads = kv->num_heads;
    a.q_heads = c.q_heads;
    a.hd = kv->head_dim;
    a.inv_sqrt = attn_inv_sqrt(kv->head_dim);
    a.write_partials = c.partials_out ? 1u : 0u;
    uint32_t bound = c.token_bound ? c.token_bound : kv->max_seq_len;
    if (c.range_mode && c.tok_end - c.tok_begin < bound) bound = c.tok_end - c.tok_begin;
    if (bound == 0) bound = 1;
    m40_attn_pick_chunk(ctx, c.rows, kv->num_heads, bound, &a.chunk, &a.splits);
    if (a.splits > 1 || c.partials_out) {
        const size_t n = (size_t)c.rows * c.q_heads * a.splits;
        float* scratch = (float*)m40_ensure_scratch(ctx, 1, n * (2 + (size_t)a.hd) * sizeof(float));
        if (!scratch) return -4;
        a.part_m = scratch;
        a.part_l = scratch + n;
        a.part_o = scratch + 2 * n;
    } else {
        a.part_m = a.part_l = a.part_o = nullptr;
    }
    int rc = m40_attention_dense_tiled(ctx, a, c.rows);
    if (rc == 1) rc = launch_generic(ctx, a, c.rows);  // 1 = shape not taken by the tiled kernel
    if (rc != 0) return rc;
    if (c.partials_out) {
        return m40_attention_fold_partials(ctx, a.part_m, a.part_l, a.part_o, a.splits, c.q_heads, a.hd, c.part_m,
                                           c.part_l, c.part_o);
    }
    if (a.splits > 1) return m40_attention_merge_rows(ctx, a.part_m, a.part_l, a.part_o, a.splits, c.q_heads, a.hd, c.out, c.rows);
    return 0;
}

int m40_attention_merge_rows(M40llmCudaContext* ctx, const float* m, const float* l, const float* o, uint32_t splits,
                             uint32_t q_heads, uint32_t hd, float* out, uint32_t rows) {
    dim3 grid(q_heads, rows);
    if (merge_wide_ok(o, out, hd, splits, 0))
        m40_launch_dependent(attn_merge_wide_kernel, grid, dim3(256), 0, ctx->decode_stream, m, l, o, out, q_heads, hd,
                             splits, (size_t)0, (size_t)0, 0u, (float*)nullptr, (float*)nullptr);
    else
        attn_merge_kernel<<<grid, 128, 0, ctx->decode_stream>>>(m, l, o, out, q_heads, hd, splits, 0, 0, 0u);
    M40_COUNT_LAUNCH(ctx);
    return cudaGetLastError() == cudaSuccess ? 0 : -4;
}

int m40_attention_fold_partials(M40llmCudaContext* ctx, const float* m, const float* l, const float* o,
                                uint32_t splits, uint32_t q_heads, uint32_t hd, float* out_m, float* out_l,
                                float* out_o) {
    if (merge_wide_ok(o, out_o, hd, splits, 0))
        m40_launch_dependent(attn_merge_wide_kernel, dim3(q_heads, 1), dim3(256), 0, ctx->decode_stream, m, l, o, out_o, q_heads,
                             hd, splits, (size_t)0, (size_t)0, 0u, out_m, out_l);
    else
        attn_fold_kernel<<<q_heads, 128, 0, ctx->decode_stream>>>(m, l, o, hd, splits, out_m, out_l, out_o);
    M40_COUNT_LAUNCH(ctx);
    return cudaGetLastError() == cudaSuccess ? 0 : -4;
}

// m, l [part][...] with `stride_m` floats between parts, o with `stride_o` floats between parts.
static int merge_strided(M40llmCudaContext* ctx, const float* m, const float* l, const float* o, uint32_t parts,
                         uint32_t q_heads, uint32_t hd, float* out, size_t stride_m, size_t stride_o) {
    dim3 grid(q_heads, 1);
    if (merge_wide_ok(o, out, hd, parts, stride_o))
        attn_merge_wide_kernel<<<grid, 256, 0, ctx->decode_stream>>>(m, l, o, out, q_heads, hd, parts, stride_m, stride_o, 1u);
    else
        attn_merge_kernel<<<grid, 128, 0, ctx->decode_stream>>>(m, l, o, out, q_heads, hd, parts, stride_m, stride_o, 1u);
    M40_COUNT_LAUNCH(ctx);
    return cudaGetLastError() == cudaSuccess ? 0 : -4;
}

int m40_attention_merge(M40llmCudaContext* ctx, const float* m, const float* l, const float* o, uint32_t parts,
                        uint32_t q_heads, uint32_t hd, float* out) {
    return merge_strided(ctx, m, l, o, parts, q_heads, hd, out, (size_t)q_heads, (size_t)q_heads * hd);
}


extern "C" {

int m40llm_attention_last_token_f32_gqa_async(M40llmCudaContext* ctx, const M40llmKVCache* kv, uint32_t seq_id,
                                              const void* d_q_f32, uint32_t q_heads, uint32_t seq_len,
                                              void* d_out_f32) {
    if (!ctx || !kv || !d_q_f32 || !d_out_f32) return -1;
    if (seq_id >= kv->max_batch_size) return -2;
    if (seq_len == 0 || seq_len > kv->max_seq_len) return -3;
    if (q_heads == 0 || kv->num_heads == 0 || q_heads % kv->num_heads != 0) return -6;
    if (!kv->d_k || !kv->d_v || kv->head_dim == 0 || kv->head_dim > 256) return -4;
    if (m40_ensure_device(ctx) != 0) return -1;
    M40DenseAttnCall c = {};
    c.q = (const float*)d_q_f32;
    c.out = (float*)d_out_f32;
    c.seq_id = seq_id;
    c.seq_len = seq_len;
    c.token_bound = seq_len;
    c.rows = 1;
    c.q_heads = q_heads;
    return m40_attention_dense(ctx, kv, c);
}

int m40llm_attention_last_token_f32_gqa(M40llmCudaContext* ctx, const M40llmKVCache* kv, uint32_t seq_id,
                                        const void* d_q_f32, uint32_t q_heads, uint32_t seq_len, void* d_out_f32) {
    const int rc = m40llm_attention_last_token_f32_gqa_async(ctx, kv, seq_id, d_q_f32, q_heads, seq_len, d_out_f32);
    if (rc != 0) return rc;
    return cudaStreamSynchronize(ctx->decode_stream) == cudaSuccess ? 0 : -5;
}

int m40llm_attention_last_token_f32(M40llmCudaContext* ctx, const M40llmKVCache* kv, uint32_t seq_id,
                                    const void* d_q_f32, uint32_t seq_len, void* d_out_f32) {
    if (!ctx || !kv || !d_q_f32 || !d_out_f32) return -1;
    if (seq_id >= kv->max_batch_size) return -2;
    if (seq_len == 0 || seq_len > kv->max_seq_len) return -3;
    const int rc = m40llm_attention_last_token_f32_gqa_async(ctx, kv, seq_id, d_q_f32, kv->num_heads, seq_len, d_out_f32);
    if (rc != 0) return -4;
    return cudaStreamSynchronize(ctx->decode_stream) == cudaSuccess ? 0 : -5;
}

int m40llm_attention_last_token_f32_gqa_seq_len_dev_async(M40llmCudaContext* ctx, const M40llmKVCache* kv,
                                                          uint32_t seq_id, const void* d_q_f32, uint32_t q_heads,
                                                          const uint32_t* d_seq_len, void* d_out_f32) {
    if (!ctx || !kv || !d_q_f32 || !d_seq_len || !d_out_f32) return -1;
    if (seq_id >= kv->max_batch_size) return -2;
    if (q_heads == 0 || kv->num_heads == 0 || q_heads % kv->num_heads != 0) return -3;
    if (!kv->d_k || !kv->d_v || kv->head_dim == 0 || kv->head_dim > 256) return -4;
    if (m40_ensure_device(ctx) != 0) return -1;
    M40DenseAttnCall c = {};
    c.q = (const float*)d_q_f32;
    c.out = (float*)d_out_f32;
    c.seq_id = seq_id;
    c.seq_len_dev = d_seq_len;
    c.rows = 1;
    c.q_heads = q_heads;
    return m40_attention_dense(ctx, kv, c);
}

static int batched_impl(M40llmCudaContext* ctx, const M40llmKVCache* kv, const uint32_t* d_seq_ids,
                        const uint32_t* d_seq_lens, uint32_t batch_size, const void* d_q_f32, uint32_t q_heads,
                        void* d_out_f32, bool synchronize) {
    if (!ctx || !kv || !d_seq_ids || !d_seq_lens || !d_q_f32 || !d_out_f32) return -1;
    if (batch_size == 0) return -2;
    if (q_heads == 0 || kv->num_heads == 0 || q_heads % kv->num_heads != 0) return -3;
    if (!kv->d_k || !kv->d_v || kv->head_dim == 0 || kv->head_dim > 256) return -6;
    if (m40_ensure_device(ctx) != 0) return -1;
    M40DenseAttnCall c = {};
    c.q = (const float*)d_q_f32;
    c.out = (float*)d_out_f32;
    c.seq_ids = d_seq_ids;
    c.seq_lens = d_seq_lens;
    c.rows = batch_size;
    c.q_heads = q_heads;
    const int rc = m40_attention_dense(ctx, kv, c);
    if (rc != 0) return -4;
    if (synchronize) {
        // The reference validates ids/lengths on the host before launching (kernels.cu:4737-4754,
        // rc -8). Here rows are validated on the device and skipped; the synchronous form reports it.
        if (cudaStreamSynchronize(ctx->decode_stream) != cudaSuccess) return -5;
        uint32_t st = 0;
        if (cudaMemcpy(&st, ctx->d_status, sizeof(uint32_t), cudaMemcpyDeviceToHost) != cudaSuccess) return -7;
        if (st & 1u) {
            cudaMemset(ctx->d_status, 0, sizeof(uint32_t));
            cudaStreamSynchronize(cudaStreamLegacy);
            return -8;
        }
    }
    return 0;
}

int m40llm_attention_last_token_f32_gqa_batched(M40llmCudaContext* ctx, const M40llmKVCache* kv,
                                                const uint32_t* d_seq_ids, const uint32_t* d_seq_lens,
                                                uint32_t batch_size, const void* d_q_f32, uint32_t q_heads,
                                                void* d_out_f32) {
    return batched_impl(ctx, kv, d_seq_ids, d_seq_lens, batch_size, d_q_f32, q_heads, d_out_f32, true);
}

int m40llm_attention_last_token_f32_gqa_batched_async(M40llmCudaContext* ctx, const M40llmKVCache* kv,
                                                      const uint32_t* d_seq_ids, const uint32_t* d_seq_lens,
                                                      uint32_t batch_size, const void* d_q_f32, uint32_t q_heads,
                                                      void* d_out_f32) {
    return batched_impl(ctx, kv, d_seq_ids, d_seq_lens, batch_size, d_q_f32, q_heads, d_out_f32, false);
}

int m40llm_attention_last_token_f32_gqa_partial_async(M40llmCudaContext* ctx, const M40llmKVCache* kv,
                                                      uint32_t seq_id, const void* d_q_f32, uint32_t q_heads,
                                                      uint32_t tok_begin, uint32_t tok_end, void* d_m_f32,
                                                      void* d_l_f32, void* d_o_f32) {
    if (!ctx || !kv || !d_q_f32 || !d_m_f32 || !d_l_f32 || !d_o_f32) return -1;
    if (seq_id >= kv->max_batch_size) return -2;
    if (tok_begin > tok_end || tok_end > kv->max_seq_len) return -3;
    if (q_heads == 0 || kv->num_heads == 0 || q_heads % kv->num_heads != 0) return -6;
    if (!kv->d_k || !kv->d_v || kv->head_dim == 0 || kv->head_dim > 256) return -4;
    if (m40_ensure_device(ctx) != 0) return -1;
    M40DenseAttnCall c = {};
    c.q = (const float*)d_q_f32;
    c.seq_id = seq_id;
    c.seq_len = tok_end > 0 ? tok_end : 1;  // range mode clamps to [tok_begin, tok_end)
    c.tok_begin = tok_begin;
    c.tok_end = tok_end;
    c.range_mode = 1;
    c.rows = 1;
    c.q_heads = q_heads;
    c.partials_out = 1;
    c.part_m = (float*)d_m_f32;
    c.part_l = (float*)d_l_f32;
    c.part_o = (float*)d_o_f32;
    return m40_attention_dense(ctx, kv, c);
}

int m40llm_attention_merge_gathered_async(M40llmCudaContext* ctx, const void* d_triples_f32, uint32_t parts,
                                          uint32_t q_heads, uint32_t head_dim, void* d_out_f32) {
    if (!ctx || !d_triples_f32 || !d_out_f32) return -1;
    if (parts == 0 || q_heads == 0 || head_dim == 0) return -2;
    if (m40_ensure_device(ctx) != 0) return -1;
    const float* base = (const float*)d_triples_f32;
    const size_t stride = (size_t)q_heads * (2u + head_dim);
    return merge_strided(ctx, base, base + q_heads, base + 2u * (size_t)q_heads, parts, q_heads, head_dim,
                         (float*)d_out_f32, stride, stride);
}

int m40llm_attention_merge_partials_async(M40llmCudaContext* ctx, const void* d_m_f32, const void* d_l_f32,
                                          const void* d_o_f32, uint32_t parts, uint32_t q_heads, uint32_t head_dim,
                                          void* d_out_f32) {
    if (!ctx || !d_m_f32 || !d_l_f32 || !d_o_f32 || !d_out_f32) return -1;
    if (parts == 0 || q_heads == 0 || head_dim == 0) return -2;
    if (m40_ensure_device(ctx) != 0) return -1;
    return m40_attention_merge(ctx, (const float*)d_m_f32, (const float*)d_l_f32, (const float*)d_o_f32, parts,
                               q_heads, head_dim, (float*)d_out_f32);
}

// ---- modes outside the decode hot path: reference argument checks, then "unsupported" ----
int m40llm_attention_last_token_f32_gqa_dense_recent_async(M40llmCudaContext* ctx, const M40llmKVCache* kv,
                                                           uint32_t seq_id, const void* d_q_f32, uint32_t q_heads,
                                                           uint32_t seq_len, uint32_t recent_window, void* d_out_f32) {
    if (!ctx || !kv || !d_q_f32 || !d_out_f32) return -1;
    if (seq_id >= kv->max_batch_size) return -2;
    if (seq_len == 0 || seq_len > kv->max_seq_len) return -3;
    if (q_heads == 0 || kv->num_heads == 0 || q_heads % kv->num_heads != 0) return -4;
    if (recent_window == 0) return -6;
    return M40LLM_ERR_UNSUPPORTED;
}

}  // extern "C"
