#include "decode_model.hpp"

#include <string.h>

namespace m40host {

DecodeModel::DecodeModel(M40llmCudaContext* ctx, const ModelConfig& cfg, const std::vector<LayerWeights>& layers,
                         const ModelHead& head, M40llmKVCache* kv, uint32_t sequences)
    : ctx_(ctx), cfg_(cfg), layers_(layers), head_(head), kv_(kv), seqs_(sequences) {
    if (!ctx || !kv || sequences == 0 || layers.empty() || !head.embeddings || !head.lm_head || head.vocab == 0) return;
    const size_t r = sequences, qd = (size_t)cfg.q_heads * cfg.head_dim, nl = layers.size();
    ok_ = m40llm_device_malloc(ctx, r * cfg.hidden * 4, &d_xa_) == 0 &&
          m40llm_device_malloc(ctx, r * cfg.hidden * 4, &d_xb_) == 0 &&
          m40llm_device_malloc(ctx, r * qd * 4, &d_q_) == 0 && m40llm_device_malloc(ctx, r * qd * 4, &d_att_) == 0 &&
          m40llm_device_malloc(ctx, r * cfg.hidden * 4, &d_x1_) == 0 &&
          m40llm_device_malloc(ctx, r * cfg.ffn * 4, &d_hid_) == 0 &&
          m40llm_device_malloc(ctx, r * head.vocab * 4, &d_logits_) == 0 &&
          m40llm_device_malloc(ctx, r * 4, &d_tokens_) == 0 && m40llm_device_malloc(ctx, r * 4, &d_pos_) == 0 &&
          m40llm_device_malloc(ctx, r * 4, &d_lens_) == 0 && m40llm_device_malloc(ctx, nl * r * 4, &d_slots_) == 0 &&
          m40llm_device_malloc(ctx, (size_t)kHistory * r * 4, &d_history_) == 0;
    if (!ok_) return;
    // slot of (sequence, layer) = sequence * layers + layer, laid out [layer][sequence] for the per-layer calls
    std::vector<uint32_t> slots(nl * r);
    for (size_t l = 0; l < nl; ++l)
        for (size_t s = 0; s < r; ++s) slots[l * r + s] = (uint32_t)(s * nl + l);
    ok_ = m40llm_memcpy_h2d(ctx, d_slots_, slots.data(), slots.size() * 4) == 0;
}

DecodeModel::~DecodeModel() {
    if (!ctx_) return;
    m40llm_stream_synchronize(ctx_, 1);
    if (graph_) m40llm_cuda_graph_destroy(graph_);
    void* bufs[] = {d_xa_, d_xb_, d_q_, d_att_, d_x1_, d_hid_, d_logits_, d_tokens_, d_pos_, d_lens_, d_slots_, d_history_};
    for (void* b : bufs)
        if (b) m40llm_device_free(ctx_, b);
}

int DecodeModel::fail(int rc, const char* step) {
    failed_step_ = step;
    return rc;
}

int DecodeModel::begin(const uint32_t* token_ids, const uint32_t* positions) {
    if (!ok_) return fail(-1, "not_initialised");
    int rc = m40llm_stream_synchronize(ctx_, 1);
    if (rc != 0) return fail(rc, "stream_synchronize");
    std::vector<uint32_t> lens(seqs_);
    for (uint32_t s = 0; s < seqs_; ++s) lens[s] = positions[s] + 1u;  // the new token is attended too
    if ((rc = m40llm_memcpy_h2d(ctx_, d_tokens_, token_ids, (size_t)seqs_ * 4)) != 0) return fail(rc, "upload_tokens");
    if ((rc = m40llm_memcpy_h2d(ctx_, d_pos_, positions, (size_t)seqs_ * 4)) != 0) return fail(rc, "upload_positions");
    if ((rc = m40llm_memcpy_h2d(ctx_, d_lens_, lens.data(), (size_t)seqs_ * 4)) != 0) return fail(rc, "upload_lens");
    return 0;
}

// One token for every sequence: embed -> layers (ping-pong between the two hidden buffers) -> logits -> arg-max into
// the token array (the next step's input) -> positions and lengths advance. The chosen ids are also appended to
// the history ring by a device-to-device copy so that a replayed graph leaves a trace per step.
int DecodeModel::enqueue_step() {
    const uint32_t H = cfg_.hidden, QD = cfg_.q_heads * cfg_.head_dim, r = seqs_;
    int rc = m40llm_embed_tokens_f16_async(ctx_, head_.embeddings, (const uint32_t*)d_tokens_, d_xa_, r, H, head_.vocab);
    if (rc != 0) return fail(rc, "embed_tokens");
    void *x = d_xa_, *y = d_xb_;
    for (size_t l = 0; l < layers_.size(); ++l) {
        const LayerWeights& w = layers_[l];
        const uint32_t* slots = (const uint32_t*)d_slots_ + l * r;
        rc = m40llm_qkv_rope_append_attention_async(ctx_, kv_, x, w.attn_norm, 1u, cfg_.rms_eps, w.wq, w.wk, w.wv, w.bq, w.bk,
                                                    w.bv, slots, (const uint32_t*)d_pos_, (const uint32_t*)d_lens_, r, H,
                                                    cfg_.q_heads, cfg_.rope_base, cfg_.rope_scale, cfg_.rope_layout, d_q_,
                                                    d_att_);
        if (rc != 0) return fail(rc, "qkv_rope_append_attention");
        rc = m40llm_attn_out_ffn_async(ctx_, d_att_, w.wo, x, w.ffn_norm, 1u, cfg_.rms_eps, w.wg, w.wu, w.wd,
                                       w.ffn_q80 ? 1u : 0u, d_x1_, d_hid_, y, r, H, QD, cfg_.ffn);
        if (rc != 0) return fail(rc, "attn_out_ffn");
        void* t = x;
        x = y;
        y = t;
    }
    rc = m40llm_logits_head_f32_async(ctx_, x, head_.output_norm, 1u, cfg_.rms_eps, head_.lm_head, d_logits_, r, H,
                                      head_.vocab);
    if (rc != 0) return fail(rc, "logits_head");
    rc = m40llm_argmax_f32_async(ctx_, d_logits_, r, head_.vocab, (uint32_t*)d_tokens_);
    if (rc != 0) return fail(rc, "argmax");
    rc = m40llm_advance_positions_async(ctx_, (uint32_t*)d_pos_, (uint32_t*)d_lens_, r);
    if (rc != 0) return fail(rc, "advance_positions");
    return 0;
}

int DecodeModel::generate(uint32_t steps, bool use_graph, uint32_t* out_ids, float* out_logits) {
    if (!ok_) return fail(-1, "not_initialised");
    if (steps == 0) return 0;
    if (out_ids && steps > kHistory) return fail(-2, "too_many_steps_for_history");
    int rc;
    for (uint32_t t = 0; t < steps; ++t) {
        const bool replay = use_graph && graph_ != nullptr;
        if (replay) {
            if ((rc = m40llm_cuda_graph_launch(ctx_, graph_, 1u)) != 0) return fail(rc, "graph_launch");
            ++graph_replays_;
        } else {
            uint64_t n0 = 0, n1 = 0;
            m40llm_context_launch_count(ctx_, &n0);
            if ((rc = enqueue_step()) != 0) return rc;
            m40llm_context_launch_count(ctx_, &n1);
            launches_per_step_ = n1 - n0;
        }
        // the ids chosen by this step, kept per step so that back-to-back replays leave a trace
        if (out_ids && (rc = m40llm_memcpy_d2d_async(ctx_, (char*)d_history_ + (size_t)t * seqs_ * 4, d_tokens_,
                                                     (size_t)seqs_ * 4, 1u)) != 0)
            return fail(rc, "history_copy");
        if (!replay && use_graph && !capture_tried_ && t + 1 < steps) {
            // the eager step sized every scratch arena; capture the same sequence once for all later tokens
            capture_tried_ = true;
            if ((rc = m40llm_stream_synchronize(ctx_, 1u)) != 0) return fail(rc, "sync_before_capture");
            if (m40llm_cuda_graph_begin_capture(ctx_, 1u) == 0) {
                rc = enqueue_step();
                if (rc != 0) {
                    m40llm_cuda_graph_cancel_capture(ctx_, 1u);
                    return rc;
                }
                M40llmCudaGraphExec* exec = nullptr;
                if (m40llm_cuda_graph_end_capture(ctx_, 1u, &exec) == 0 && exec) graph_ = exec;
            }
        }
    }
    if ((rc = m40llm_stream_synchronize(ctx_, 1u)) != 0) return fail(rc, "stream_synchronize");
    if (out_ids && (rc = m40llm_memcpy_d2h(ctx_, out_ids, d_history_, (size_t)steps * seqs_ * 4)) != 0)
        return fail(rc, "read_ids");
    if (out_logits && (rc = m40llm_memcpy_d2h(ctx_, out_logits, d_logits_, (size_t)seqs_ * head_.vocab * 4)) != 0)
        return fail(rc, "read_logits");
    uint32_t status = 0;
    if (m40llm_context_take_device_status(ctx_, &status) == 0 && status != 0) return fail(-(int)(1000 + status), "device_status");
    return 0;
}

}  // namespace m40host
