// Fused attention prologue for a batch of decode rows:
//   xn = rmsnorm(x, w);  q,k,v = xn.Wq/Wk/Wv (+bias);  q <- rope(q, pos);
//   cache[seq][pos] <- f16(rope(k, pos)), f16(v)
// The reference issues this as 1 norm + 3 GEMMs + 3 bias adds + per-row rope and append launches
// with cross-stream waits between them (src/infer/forward.rs:307-421). Here it is five launches
// on the decode stream for any number of rows: the norm, three projections that share the
// normalised activations (bias folded into their epilogue), and one rope+append launch that
// covers every row, q head and kv head.
#include <stdlib.h>

#include "attention.cuh"
#include "common.cuh"
#include "gemm.cuh"
#include "gemm_tc.cuh"
#include "gemv_stream.cuh"
#include "kv_append.cuh"

namespace {

// grid (q_heads + kv_heads, rows), block 64.
__global__ void __launch_bounds__(64) rope_q_append_kv_rows_kernel(float* __restrict__ q, const float* __restrict__ k,
                                                                   const float* __restrict__ v, M40llmKVCache kv,
                                                                   const uint32_t* __restrict__ seq_ids,
                                                                   const uint32_t* __restrict__ positions,
                                                                   uint32_t q_heads, float freq_base, float freq_scale,
                                                                   uint32_t layout, uint32_t* status,
                                                                   const float* __restrict__ inv_freq) {
    __shared__ float red[32];
    pdl_wait();
    pdl_trigger();
    const uint32_t row = blockIdx.y, hsel = blockIdx.x;
    const uint32_t hd = kv.head_dim, half = hd / 2u;
    const uint32_t seq = seq_ids[row], pos = positions[row];
    if (seq >= kv.max_batch_size || pos >= kv.max_seq_len) {
        if (threadIdx.x == 0 && hsel == 0) atomicOr(status, 2u);
        return;
    }
    if (hsel < q_heads) {
        float* qh = q + ((size_t)row * q_heads + hsel) * hd;
        for (uint32_t i = threadIdx.x; i < half; i += blockDim.x) {
            const uint32_t i0 = layout == 1u ? i : 2u * i;
            const uint32_t i1 = layout == 1u ? i + half : 2u * i + 1u;
            float c, s;
            rope_cs(pos, i, hd, freq_base, freq_scale, &c, &s, inv_freq);
            const float a = qh[i0], b = qh[i1];
            qh[i0] = a * c - b * s;
            qh[i1] = a * s + b * c;
        }
        return;
    }
    const uint32_t kvh = hsel - q_heads;
    const float* kh = k + ((size_t)row * kv.num_heads + kvh) * hd;
    const float* vh = v + ((size_t)row * kv.num_heads + kvh) * hd;
    if (kv.compressed) kv_append_compressed_head(kv, seq, kvh, pos, kh, vh, freq_base, freq_scale, layout, red, inv_freq);
    else kv_append_dense_head(kv, seq, kvh, pos, kh, vh, freq_base, freq_scale, layout, inv_freq);
}

}  // namespace

int m40_rms_norm_rows(M40llmCudaContext* ctx, const void* in, const void* w, void* out, uint32_t rows, uint32_t dim,
                      float eps, uint32_t wdtype);

extern "C" int m40llm_qkv_rmsnorm_rope_append_async(M40llmCudaContext* ctx, M40llmKVCache* kv, const void* d_x_f32,
                                                    const void* d_norm_w, uint32_t norm_w_dtype, float eps,
                                                    const void* d_wq_f16, const void* d_wk_f16, const void* d_wv_f16,
                                                    const void* d_bq_f32, const void* d_bk_f32, const void* d_bv_f32,
                                                    const uint32_t* d_seq_ids, const uint32_t* d_positions,
                                                    uint32_t rows, uint32_t hidden, uint32_t q_heads, float freq_base,
                                                    float freq_scale, uint32_t rope_layout, void* d_q_out_f32) {
    if (!ctx || !kv || !d_x_f32 || !d_norm_w || !d_wq_f16 || !d_wk_f16 || !d_wv_f16 || !d_seq_ids || !d_positions ||
        !d_q_out_f32)
        return -1;
    if (rows == 0 || hidden == 0 || q_heads == 0 || kv->num_heads == 0 || q_heads % kv->num_heads != 0) return -2;
    if (norm_w_dtype > 1) return -4;
    if (kv->head_dim == 0 || kv->head_dim % 2 != 0) return -3;
    if (kv->compressed && kv->head_dim != 64 && kv->head_dim != 128) return -3;
    if (!kv->compressed && (!kv->d_k || !kv->d_v)) return -3;
    if (m40_ensure_device(ctx) != 0) return -1;
    const uint32_t hd = kv->head_dim, QD = q_heads * hd, KD = kv->num_heads * hd;
    // level-1 arena: the projections called below use the level-0 arena for their own temporaries
    const size_t need = (size_t)rows * ((size_t)hidden + 2 * (size_t)KD) * sizeof(float);
    float* scratch = (float*)m40_ensure_scratch(ctx, 1, need, 1);
    if (!scratch) return -5;
    float* xn = scratch;
    float* kbuf = xn + (size_t)rows * hidden;
    float* vbuf = kbuf + (size_t)rows * KD;
    cudaStream_t s = ctx->decode_stream;
    int rc = 1;
    if (rows == 1) {
        // one row: RMSNorm folded into a single streaming launch over Wq | Wk | Wv
        const M40GemvSeg segs[3] = {
            {d_wq_f16, nullptr, (float*)d_q_out_f32, (const float*)d_bq_f32, nullptr, (int)QD},
            {d_wk_f16, nullptr, kbuf, (const float*)d_bk_f32, nullptr, (int)KD},
            {d_wv_f16, nullptr, vbuf, (const float*)d_bv_f32, nullptr, (int)KD}};
        const M40GemvNorm norm = {d_norm_w, norm_w_dtype == 1u ? 1 : 0, eps, nullptr};
        rc = m40_gemv_stream(ctx, s, (const float*)d_x_f32, (int)hidden, M40_GEMV_F16, 0, 3, segs, &norm);
        if (rc < 0) return rc;
    }
    const void* wp[3] = {d_wq_f16, d_wk_f16, d_wv_f16};
    if (rc == 0) {
        // projections done above
    } else if ((int)rows >= m40_tc_min_rows() && m40_gemm_tc_supported((int)rows, (int)hidden, 3, wp) && hidden % 4 == 0) {
        // one tensor-core launch over Wq | Wk | Wv; the norm rides on the f16 split of the activations
        const __half* w[3] = {(const __half*)d_wq_f16, (const __half*)d_wk_f16, (const __half*)d_wv_f16};
        const int n[3] = {(int)QD, (int)KD, (int)KD};
        float* o[3] = {(float*)d_q_out_f32, kbuf, vbuf};
        const float* b[3] = {(const float*)d_bq_f32, (const float*)d_bk_f32, (const float*)d_bv_f32};
        const M40GemvNorm norm = {d_norm_w, norm_w_dtype == 1u ? 1 : 0, eps, nullptr};
        // dense cache, adjacent-pair RoPE, whole 128-column tiles per matrix: the projection's epilogue rotates and
        // appends, and no separate launch follows
        const bool tail_in_epilogue = !kv->compressed && rope_layout == 0u && QD % 128u == 0u && KD % 128u == 0u;
        const M40TcRopeAppend ra = {d_seq_ids, d_positions, (__half*)kv->d_k, (__half*)kv->d_v, kv->d_seq_map,
                                    ctx->d_status, hd, kv->num_heads, kv->max_seq_len, kv->max_batch_size,
                                    freq_base, freq_scale, m40_rope_inv_freq(ctx, freq_base, hd)};
        rc = m40_gemm_tc_f16(ctx, s, 1u, (const float*)d_x_f32, (int)rows, (int)hidden, 3, w, n, o, b, nullptr, 0, &norm,
                             tail_in_epilogue ? &ra : nullptr);
        if (rc != 0) return rc;
        if (tail_in_epilogue) return 0;
    } else if ((rc = m40_rms_norm_rows(ctx, d_x_f32, d_norm_w, xn, rows, hidden, eps, norm_w_dtype)) != 0) {
        return rc;
    } else {
        rc = m40_gemm_f32xf16_gguf(ctx, s, xn, (const __half*)d_wq_f16, (float*)d_q_out_f32, (int)rows, (int)QD,
                                   (int)hidden, (const float*)d_bq_f32, nullptr);
        if (rc != 0) return rc;
        rc = m40_gemm_f32xf16_gguf(ctx, s, xn, (const __half*)d_wk_f16, kbuf, (int)rows, (int)KD, (int)hidden,
                                   (const float*)d_bk_f32, nullptr);
        if (rc != 0) return rc;
        rc = m40_gemm_f32xf16_gguf(ctx, s, xn, (const __half*)d_wv_f16, vbuf, (int)rows, (int)KD, (int)hidden,
                                   (const float*)d_bv_f32, nullptr);
        if (rc != 0) return rc;
    }
    dim3 grid(q_heads + kv->num_heads, rows);
    const cudaError_t e = m40_launch_dependent(rope_q_append_kv_rows_kernel, grid, dim3(64), 0, s, (float*)d_q_out_f32,
                                               (const float*)kbuf, (const float*)vbuf, *kv, d_seq_ids, d_positions,
                                               q_heads, freq_base, freq_scale, rope_layout, ctx->d_status,
                                               m40_rope_inv_freq(ctx, freq_base, hd));
    M40_COUNT_LAUNCH(ctx);
    return e == cudaSuccess && cudaGetLastError() == cudaSuccess ? 0 : -6;
}

int m40llm_attention_last_token_f32_gqa_batched_async(M40llmCudaContext* ctx, const M40llmKVCache* kv,
                                                      const uint32_t* d_seq_ids, const uint32_t* d_seq_lens,
                                                      uint32_t batch_size, const void* d_q_f32, uint32_t q_heads,
                                                      void* d_out_f32);

// Steps 1-6 of the layer in one call (src/infer/forward.rs:307-470): the prologue above followed by the batched decode
// attention. One row on a dense cache takes two launches: the streaming Wq | Wk | Wv projection (norm and bias
// folded in) and the cluster kernel that rotates, appends, attends and merges. Everything else is the two entry
// points back to back.
extern "C" int m40llm_qkv_rope_append_attention_async(
    M40llmCudaContext* ctx, M40llmKVCache* kv, const void* d_x_f32, const void* d_norm_w, uint32_t norm_w_dtype, float eps,
    const void* d_wq_f16, const void* d_wk_f16, const void* d_wv_f16, const void* d_bq_f32, const void* d_bk_f32,
    const void* d_bv_f32, const uint32_t* d_seq_ids, const uint32_t* d_positions, const uint32_t* d_seq_lens, uint32_t rows,
    uint32_t hidden, uint32_t q_heads, float freq_base, float freq_scale, uint32_t rope_layout, void* d_q_out_f32,
    void* d_att_out_f32) {
    if (!ctx || !kv || !d_x_f32 || !d_norm_w || !d_wq_f16 || !d_wk_f16 || !d_wv_f16 || !d_seq_ids || !d_positions ||
        !d_seq_lens || !d_q_out_f32 || !d_att_out_f32)
        return -1;
    if (rows == 0 || hidden == 0 || q_heads == 0 || kv->num_heads == 0 || q_heads % kv->num_heads != 0) return -2;
    if (norm_w_dtype > 1) return -4;
    if (m40_ensure_device(ctx) != 0) return -1;
    const uint32_t hd = kv->head_dim, QD = q_heads * hd, KD = kv->num_heads * hd;
    // The cluster kernel saves two launches per layer, which is what counts while a sequence's K / V is a few MB
    // (1198 against 1087 tokens/s on a 22-layer stack at context 2048); with tens of MB to stream its 16 CTAs per kv
    // head fall behind the separate split + merge launches (87 against 82 us per layer step at context 8K). The
    // lengths live on the device, so the cache's capacity stands in for them.
    static long fused_row_max_bytes = -1;
    if (fused_row_max_bytes < 0) {
        const char* e = getenv("M40LLM_FUSED_ROW_MAX_KV_MB");
        fused_row_max_bytes = (e ? atol(e) : 8L) << 20;
    }
    const size_t kv_bytes = (size_t)kv->num_heads * kv->max_seq_len * hd * 4u;  // K and V rows of one sequence, f16
    const bool one_launch_attention = rows == 1 && !kv->compressed && kv->d_k && kv->d_v && (hd == 64 || hd == 128) &&
                                      q_heads / kv->num_heads <= 16 && kv_bytes <= (size_t)fused_row_max_bytes;
    if (one_launch_attention) {
        const size_t need = (size_t)rows * ((size_t)QD + 2 * (size_t)KD) * sizeof(float);
        float* scratch = (float*)m40_ensure_scratch(ctx, 1, need, 1);
        if (!scratch) return -5;
        float* qraw = scratch;
        float* kbuf = qraw + (size_t)rows * QD;
        float* vbuf = kbuf + (size_t)rows * KD;
        const M40GemvSeg segs[3] = {{d_wq_f16, nullptr, qraw, (const float*)d_bq_f32, nullptr, (int)QD},
                                    {d_wk_f16, nullptr, kbuf, (const float*)d_bk_f32, nullptr, (int)KD},
                                    {d_wv_f16, nullptr, vbuf, (const float*)d_bv_f32, nullptr, (int)KD}};
        const M40GemvNorm norm = {d_norm_w, norm_w_dtype == 1u ? 1 : 0, eps, nullptr};
        int rc = m40_gemv_stream(ctx, ctx->decode_stream, (const float*)d_x_f32, (int)hidden, M40_GEMV_F16, 0, 3, segs, &norm);
        if (rc < 0) return rc;
        if (rc == 0) {
            rc = m40_attention_fused_row(ctx, kv, qraw, kbuf, vbuf, d_seq_ids, d_positions, d_seq_lens, rows, q_heads,
                                         freq_base, freq_scale, rope_layout, (float*)d_q_out_f32, (float*)d_att_out_f32);
            if (rc <= 0) return rc;
            // the device does not take the cluster kernel: finish with the separate rope/append and attention launches
            dim3 grid(q_heads + kv->num_heads, rows);
            const cudaError_t ce = cudaMemcpyAsync(d_q_out_f32, qraw, (size_t)rows * QD * sizeof(float),
                                                   cudaMemcpyDeviceToDevice, ctx->decode_stream);
            if (ce != cudaSuccess) return -6;
            rope_q_append_kv_rows_kernel<<<grid, 64, 0, ctx->decode_stream>>>((float*)d_q_out_f32, kbuf, vbuf, *kv, d_seq_ids,
                                                                              d_positions, q_heads, freq_base, freq_scale,
                                                                              rope_layout, ctx->d_status,
                                                                              m40_rope_inv_freq(ctx, freq_base, hd));
            M40_COUNT_LAUNCH(ctx);
            if (cudaGetLastError() != cudaSuccess) return -6;
            return m40llm_attention_last_token_f32_gqa_batched_async(ctx, kv, d_seq_ids, d_seq_lens, rows, d_q_out_f32,
                                                                     q_heads, d_att_out_f32);
        }
        // the projection shape does not stream: the general prologue below handles it
    }
    const int rc = m40llm_qkv_rmsnorm_rope_append_async(ctx, kv, d_x_f32, d_norm_w, norm_w_dtype, eps, d_wq_f16, d_wk_f16,
                                                        d_wv_f16, d_bq_f32, d_bk_f32, d_bv_f32, d_seq_ids, d_positions, rows,
                                                        hidden, q_heads, freq_base, freq_scale, rope_layout, d_q_out_f32);
    if (rc != 0) return rc;
    if (kv->compressed) return M40LLM_ERR_UNSUPPORTED;  // compressed caches attend per row through their own entry point
    return m40llm_attention_last_token_f32_gqa_batched_async(ctx, kv, d_seq_ids, d_seq_lens, rows, d_q_out_f32, q_heads,
                                                             d_att_out_f32);
}

// Steps 9-13 of the layer (src/infer/forward.rs:470-667): x1 = x + att.Wo; xn = rmsnorm(x1) * w;
// hid = silu(xn.Wg) * (xn.Wu); out = x1 + hid.Wd. One row runs as three streaming launches (residuals folded into
// the stores, the norm folded into the gate/up launch); batched rows go through the tensor-core projections.
extern "C" int m40llm_attn_out_ffn_async(M40llmCudaContext* ctx, const void* d_att_f32, const void* d_wo_f16,
                                         const void* d_x_f32, const void* d_ffn_norm_w, uint32_t norm_w_dtype,
                                         float eps, const void* d_wg, const void* d_wu, const void* d_wd,
                                         uint32_t ffn_q80, void* d_x1_f32, void* d_hid_f32, void* d_out_f32,
                                         uint32_t rows, uint32_t hidden, uint32_t q_dim, uint32_t ffn) {
    if (!ctx || !d_att_f32 || !d_wo_f16 || !d_x_f32 || !d_ffn_norm_w || !d_wg || !d_wu || !d_wd || !d_x1_f32 ||
        !d_hid_f32 || !d_out_f32)
        return -1;
    if (rows == 0 || hidden == 0 || q_dim == 0 || ffn == 0) return -2;
    if (norm_w_dtype > 1) return -4;
    if (ffn_q80 ? (hidden % 128 != 0 || ffn % 128 != 0) : (hidden % 8 != 0 || ffn % 8 != 0)) return -2;
    if (m40_ensure_device(ctx) != 0) return -1;
    cudaStream_t s = ctx->decode_stream;
    // x1 = x + att.Wo (residual folded into the projection's store on every path)
    int rc = m40_gemm_dispatch_f16(ctx, s, 1u, (const float*)d_att_f32, (const __half*)d_wo_f16, (float*)d_x1_f32,
                                   (int)rows, (int)hidden, (int)q_dim, nullptr, (const float*)d_x_f32);
    if (rc != 0) return rc;
    if (rows == 1) {
        const int fmt = ffn_q80 ? M40_GEMV_Q80 : M40_GEMV_F16;
        const M40GemvSeg gu = {d_wg, d_wu, (float*)d_hid_f32, nullptr, nullptr, (int)ffn};
        const M40GemvNorm norm = {d_ffn_norm_w, norm_w_dtype == 1u ? 1 : 0, eps, nullptr};
        rc = m40_gemv_stream(ctx, s, (const float*)d_x1_f32, (int)hidden, fmt, 1, 1, &gu, &norm);
        if (rc < 0) return rc;
        if (rc == 0) {
            const M40GemvSeg dn = {d_wd, nullptr, (float*)d_out_f32, nullptr, (const float*)d_x1_f32, (int)hidden};
            rc = m40_gemv_stream(ctx, s, (const float*)d_hid_f32, (int)ffn, fmt, 0, 1, &dn, nullptr);
            if (rc < 0) return rc;
            if (rc == 0) return 0;
            // the down projection alone did not fit the streaming kernel: finish through the regular entry
            return ffn_q80 ? m40_gemm_f32xq80_gguf(ctx, s, (const float*)d_hid_f32, (const uint8_t*)d_wd,
                                                   (float*)d_out_f32, 1, (int)hidden, (int)ffn, (const float*)d_x1_f32)
                           : m40_gemm_f32xf16_gguf(ctx, s, (const float*)d_hid_f32, (const __half*)d_wd,
                                                   (float*)d_out_f32, 1, (int)hidden, (int)ffn, nullptr,
                                                   (const float*)d_x1_f32);
        }
    }
    const M40GemvNorm norm = {d_ffn_norm_w, norm_w_dtype == 1u ? 1 : 0, eps, nullptr};
    rc = m40_ffn_swiglu(ctx, 1u, d_x1_f32, d_wg, d_wu, d_wd, d_x1_f32, d_hid_f32, d_out_f32, rows, hidden, ffn,
                        ffn_q80 ? 1 : 0, &norm);
    if (rc != 1) return rc;
    // the shape went to a path that cannot fold the norm: normalise explicitly
    float* xn = (float*)m40_ensure_scratch(ctx, 1, (size_t)rows * hidden * sizeof(float), 1);
    if (!xn) return -5;
    rc = m40_rms_norm_rows(ctx, d_x1_f32, d_ffn_norm_w, xn, rows, hidden, eps, norm_w_dtype);
    if (rc != 0) return rc;
    return m40_ffn_swiglu(ctx, 1u, xn, d_wg, d_wu, d_wd, d_x1_f32, d_hid_f32, d_out_f32, rows, hidden, ffn,
                          ffn_q80 ? 1 : 0, nullptr);
}
