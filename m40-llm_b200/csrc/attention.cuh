// Internal interface of the dense decode-attention path (attention.cu, attention_tiled.cu).
#pragma once
#include "common.cuh"

// Kernel argument block shared by the generic and the tiled kernels.
struct DenseAttnArgs {
    const __half* K;
    const __half* V;
    const float* q;            // [rows][q_heads][hd]
    float* out;                // [rows][q_heads][hd]
    const uint32_t* seq_ids;   // device [rows] or null (then seq_id)
    const uint32_t* seq_lens;  // device [rows] or null (then seq_len / seq_len_dev)
    const uint32_t* seq_len_dev;
    float* part_m;             // [rows][q_heads][splits]
    float* part_l;
    float* part_o;             // [rows][q_heads][splits][hd]
    uint32_t* status;
    uint32_t seq_id, seq_len;
    uint32_t tok_begin, tok_end;  // absolute token range when range_mode != 0
    uint32_t range_mode;
    uint32_t max_seq_len, max_batch, kv_heads, q_heads, hd, splits;
    uint32_t chunk;           // tokens per split (multiple of 64); split s covers [begin + s*chunk, +chunk)
    uint32_t write_partials;  // 1: always write (m,l,o) partials
    float inv_sqrt;
};

// Host-side description of one attention call.
struct M40DenseAttnCall {
    const float* q;
    float* out;
    const uint32_t* seq_ids;
    const uint32_t* seq_lens;
    const uint32_t* seq_len_dev;
    uint32_t seq_id, seq_len;
    uint32_t tok_begin, tok_end, range_mode;
    uint32_t token_bound;  // host-known upper bound of tokens per row (0 = cache capacity)
    uint32_t rows, q_heads;
    uint32_t partials_out;  // write one (m,l,o) triple per q head instead of the output
    float* part_m;
    float* part_l;
    float* part_o;
};

// Chooses the tokens-per-CTA chunk (multiple of 64) and the number of splits covering `max_tokens`.
void m40_attn_pick_chunk(const M40llmCudaContext* ctx, uint32_t rows, uint32_t kv_heads, uint32_t max_tokens,
                         uint32_t* chunk, uint32_t* splits);
int m40_attention_dense(M40llmCudaContext* ctx, const M40llmKVCache* kv, const M40DenseAttnCall& c);
int m40_attention_merge(M40llmCudaContext* ctx, const float* m, const float* l, const float* o, uint32_t parts,
                        uint32_t q_heads, uint32_t hd, float* out);
// Merge [row][head][split] partials into out [rows][q_heads][hd].
int m40_attention_merge_rows(M40llmCudaContext* ctx, const float* m, const float* l, const float* o, uint32_t splits,
                             uint32_t q_heads, uint32_t hd, float* out, uint32_t rows = 1);
// Fold [head][split] partials of one row into one unnormalised triple per head.
int m40_attention_fold_partials(M40llmCudaContext* ctx, const float* m, const float* l, const float* o,
                                uint32_t splits, uint32_t q_heads, uint32_t hd, float* out_m, float* out_l,
                                float* out_o);
// Returns 0 when launched, 1 when the shape is not one the tiled kernel takes, < 0 on launch failure.
int m40_attention_dense_tiled(M40llmCudaContext* ctx, const DenseAttnArgs& a, uint32_t rows);

// One launch for rows whose new token is appended in the same step: RoPE(q) -> q_out, RoPE(k) + f16 append of k / v,
// attention over the cache and the new token, split merge through distributed shared memory. Needs
// positions[r] + 1 == seq_lens[r]. Returns 0 when launched, 1 when the shape / device does not take it.
int m40_attention_fused_row(M40llmCudaContext* ctx, M40llmKVCache* kv, const float* q_raw, const float* k_new,
                            const float* v_new, const uint32_t* seq_ids, const uint32_t* positions,
                            const uint32_t* seq_lens, uint32_t rows, uint32_t q_heads, float freq_base,
                            float freq_scale, uint32_t layout, float* q_out, float* out);

// Token range of (row, split): shared by both kernels so partial layouts agree.
__device__ __forceinline__ bool attn_resolve_row(const DenseAttnArgs& a, uint32_t row, uint32_t split, uint32_t* seq,
                                                 uint32_t* t0, uint32_t* t1) {
    const uint32_t sid = a.seq_ids ? a.seq_ids[row] : a.seq_id;
    const uint32_t len = a.seq_lens ? a.seq_lens[row] : (a.seq_len_dev ? *a.seq_len_dev : a.seq_len);
    if (sid >= a.max_batch || len == 0 || len > a.max_seq_len) {
        if (a.seq_ids && a.status && threadIdx.x == 0 && split == 0 && blockIdx.y == 0) atomicOr(a.status, 1u);
        return false;
    }
    uint32_t b = 0, e = len;
    if (a.range_mode) {
        b = a.tok_begin;
        e = a.tok_end < len ? a.tok_end : len;
        if (b > e) b = e;
    }
    const uint32_t sb = b + split * a.chunk;
    uint32_t se = sb + a.chunk;
    if (se > e || se < sb) se = e;
    *seq = sid;
    *t0 = sb < e ? sb : e;
    *t1 = se > *t0 ? se : *t0;
    return true;
}

// A row whose sequence id or length is out of range reads no cache data. So that its output never depends on
// what the partial arena held before, every CTA of the row still leaves a defined result: an empty partial
// (l = 0, which the merge kernels turn into a zero row) when partials are in use, zeros in `out` otherwise.
__device__ __forceinline__ void attn_write_rejected_row(const DenseAttnArgs& a, uint32_t row, uint32_t split,
                                                        uint32_t kvh, bool partial) {
    const uint32_t G = a.q_heads / a.kv_heads;
    if (partial) {
        for (uint32_t i = threadIdx.x; i < G; i += blockDim.x) {
            const size_t pi = ((size_t)row * a.q_heads + kvh * G + i) * a.splits + split;
            a.part_m[pi] = -INFINITY;
            a.part_l[pi] = 0.0f;
        }
    } else {
        for (uint32_t i = threadIdx.x; i < G * a.hd; i += blockDim.x)
            a.out[((size_t)row * a.q_heads + kvh * G) * a.hd + i] = 0.0f;
    }
}
