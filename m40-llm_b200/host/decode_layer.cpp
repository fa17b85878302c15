#include "decode_layer.hpp"

namespace m40host {

DecodeLayer::DecodeLayer(M40llmCudaContext* ctx, const ModelConfig& cfg, uint32_t max_rows)
    : ctx_(ctx), cfg_(cfg), max_rows_(max_rows) {
    const size_t qd = (size_t)cfg.q_heads * cfg.head_dim;
    const size_t r = max_rows;
    // workspace of src/infer/workspace.rs:60-126: dq, datt, d_x1, d_x1n, dhid (rows x dim, f32)
    ok_ = ctx && r > 0 && m40llm_device_malloc(ctx, r * qd * 4, &d_q_) == 0 &&
          m40llm_device_malloc(ctx, r * qd * 4, &d_att_) == 0 &&
          m40llm_device_malloc(ctx, r * cfg.hidden * 4, &d_x1_) == 0 &&
          m40llm_device_malloc(ctx, r * cfg.hidden * 4, &d_x1n_) == 0 &&
          m40llm_device_malloc(ctx, r * cfg.ffn * 4, &d_hid_) == 0 &&
          m40llm_device_malloc(ctx, r * cfg.hidden * 4, &d_xin_) == 0 &&
          m40llm_device_malloc(ctx, r * cfg.hidden * 4, &d_xout_) == 0;
}

DecodeLayer::~DecodeLayer() {
    if (!ctx_) return;
    m40llm_stream_synchronize(ctx_, 1);
    for (auto& g : graphs_) m40llm_cuda_graph_destroy(g.exec);
    m40llm_stream_synchronize(ctx_, 0);
    void* bufs[] = {d_q_, d_att_, d_x1_, d_x1n_, d_hid_, d_xin_, d_xout_, slots_[0].d_xin, slots_[0].d_xout,
                    slots_[1].d_xin, slots_[1].d_xout};
    for (void* b : bufs)
        if (b) m40llm_device_free(ctx_, b);
    for (Slot& sl : slots_) {
        if (sl.computed) m40llm_cuda_event_destroy(sl.computed);
        if (sl.arrived) m40llm_cuda_event_destroy(sl.arrived);
    }
}

int DecodeLayer::fail(int rc, const char* step) {
    failed_step_ = step;
    return rc;
}

int DecodeLayer::enqueue(M40llmKVCache* kv, const LayerWeights& w, const KvCompressionConfig& kvcfg,
                         const DecodeBatchPlan& plan, const CudaDecodeBatchPlan& dplan, const void* d_x, void* d_out) {
    const uint32_t rows = plan.batch_size();
    const uint32_t H = cfg_.hidden, QD = cfg_.q_heads * cfg_.head_dim;
    int rc;
    if (kvcfg.mode == KvCompressMode::Off) {
        // steps 1-6 in one call: at one row the RoPE, the append, the attention and its split merge are one kernel
        rc = m40llm_qkv_rope_append_attention_async(ctx_, kv, d_x, w.attn_norm, 1u, cfg_.rms_eps, w.wq, w.wk, w.wv, w.bq,
                                                    w.bk, w.bv, dplan.d_sequence_ids(), dplan.d_positions(),
                                                    dplan.d_sequence_lens(), rows, H, cfg_.q_heads, cfg_.rope_base,
                                                    cfg_.rope_scale, cfg_.rope_layout, d_q_, d_att_);
        if (rc != 0) return fail(rc, "qkv_rope_append_attention");
    } else {
        rc = m40llm_qkv_rmsnorm_rope_append_async(ctx_, kv, d_x, w.attn_norm, 1u, cfg_.rms_eps, w.wq, w.wk, w.wv, w.bq, w.bk,
                                                  w.bv, dplan.d_sequence_ids(), dplan.d_positions(), rows, H, cfg_.q_heads,
                                                  cfg_.rope_base, cfg_.rope_scale, cfg_.rope_layout, d_q_);
        if (rc != 0) return fail(rc, "qkv_rmsnorm_rope_append");
        // src/infer/kv.rs:562-575: the default compressed configuration goes to the FP16-K/q4-V direct entry point,
        // one call per row (each row has its own sequence and block selection)
        const auto& e = plan.entries();
        for (uint32_t r = 0; r < rows; ++r) {
            rc = m40llm_attention_last_token_f32_gqa_block_select_exact_fp16_k_q4_v_old_direct_async(
                ctx_, kv, e[r].sequence_id, (const char*)d_q_ + (size_t)r * QD * 4, cfg_.q_heads, e[r].kv_len,
                kvcfg.recent_window, kvcfg.block_size, kvcfg.top_blocks, (char*)d_att_ + (size_t)r * QD * 4);
            if (rc != 0) return fail(rc, "attention_block_select_exact_fp16_k_q4_v_old_direct");
        }
    }
    // steps 9-13 in one call: out-projection + residual, FFN norm, SwiGLU FFN + residual
    rc = m40llm_attn_out_ffn_async(ctx_, d_att_, w.wo, d_x, w.ffn_norm, 1u, cfg_.rms_eps, w.wg, w.wu, w.wd,
                                   w.ffn_q80 ? 1u : 0u, d_x1_, d_hid_, d_out, rows, H, QD, cfg_.ffn);
    if (rc != 0) return fail(rc, "attn_out_ffn");
    return 0;
}

int DecodeLayer::forward_device(M40llmKVCache* kv, const LayerWeights& w, const KvCompressionConfig& kvcfg,
                                const DecodeBatchPlan& plan, const CudaDecodeBatchPlan& dplan, const void* d_x,
                                void* d_out, bool use_graph) {
    if (!ok_) return fail(-1, "workspace");
    const uint32_t rows = plan.batch_size();
    if (rows == 0 || rows > max_rows_) return fail(-2, "rows");
    const std::string cfg_err = kvcfg.validate_b200_support(0xffffffffu, cfg_.head_dim);
    if (!cfg_err.empty()) {
        failed_step_ = cfg_err;
        return -3;
    }
    // Graph replay as in src/decode_session.rs:828-954: only with KV compression off (the compressed path takes
    // host-side lengths), keyed by the buffers baked into the captured launches; positions and lengths are read
    // from device memory, so one graph serves every step of the same batch.
    if (!use_graph || kvcfg.mode != KvCompressMode::Off) return enqueue(kv, w, kvcfg, plan, dplan, d_x, d_out);
    const GraphKey key{kv, w.wq, w.wg, d_x, d_out, dplan.d_sequence_ids(), rows};
    for (auto& g : graphs_) {
        if (g.key == key) {
            ++graph_replays_;
            const int rc = m40llm_cuda_graph_launch(ctx_, g.exec, 1u);
            return rc == 0 ? 0 : fail(rc, "graph_launch");
        }
    }
    // first sight of this configuration: run it eagerly once (sizes scratch arenas), then capture for next time
    int rc = enqueue(kv, w, kvcfg, plan, dplan, d_x, d_out);
    if (rc != 0) return rc;
    if ((rc = m40llm_stream_synchronize(ctx_, 1u)) != 0) return fail(rc, "sync_before_capture");
    if (m40llm_cuda_graph_begin_capture(ctx_, 1u) != 0) return 0;  // capture unavailable: stay eager
    // the captured pass rewrites the same cache slot with the same values, so it is safe to let it execute later
    rc = enqueue(kv, w, kvcfg, plan, dplan, d_x, d_out);
    M40llmCudaGraphExec* exec = nullptr;
    if (rc != 0) {
        m40llm_cuda_graph_cancel_capture(ctx_, 1u);
        return rc;
    }
    if (m40llm_cuda_graph_end_capture(ctx_, 1u, &exec) == 0 && exec) graphs_.push_back({key, exec});
    return 0;
}

int DecodeLayer::forward_host(M40llmKVCache* kv, const LayerWeights& w, const KvCompressionConfig& kvcfg,
                              const std::vector<DecodeRequestState>& requests, const float* x_host, float* out_host,
                              bool use_graph) {
    if (!ok_) return fail(-1, "workspace");
    DecodeBatchPlan plan;
    const std::string err = DecodeBatchPlan::from_requests(requests, &plan);
    if (!err.empty()) {
        failed_step_ = err;
        return -4;
    }
    const uint32_t rows = plan.batch_size();
    if (rows > max_rows_) return fail(-2, "rows");
    int rc = host_plan_dev_.upload(ctx_, plan);
    if (rc != 0) return fail(rc, "plan_upload");
    const size_t bytes = (size_t)rows * cfg_.hidden * 4;
    // everything rides the decode stream: activations in, the layer, the result out, then ONE synchronisation
    if ((rc = m40llm_memcpy_h2d_async(ctx_, d_xin_, x_host, bytes, 1u)) != 0) return fail(rc, "memcpy_h2d");
    if ((rc = forward_device(kv, w, kvcfg, plan, host_plan_dev_, d_xin_, d_xout_, use_graph)) != 0) return rc;
    if ((rc = m40llm_memcpy_d2h_async(ctx_, out_host, d_xout_, bytes, 1u)) != 0) return fail(rc, "memcpy_d2h");
    if ((rc = m40llm_stream_synchronize(ctx_, 1u)) != 0) return fail(rc, "stream_synchronize");
    return 0;
}

// staging buffers and events of a slot, made at its first use
int DecodeLayer::slot_ready(uint32_t slot) {
    Slot& sl = slots_[slot];
    if (sl.d_xin) return 0;
    const size_t bytes = (size_t)max_rows_ * cfg_.hidden * 4;
    int rc;
    if ((rc = m40llm_device_malloc(ctx_, bytes, &sl.d_xin)) != 0) return rc;
    if ((rc = m40llm_device_malloc(ctx_, bytes, &sl.d_xout)) != 0) return rc;
    if ((rc = m40llm_cuda_event_create(ctx_, &sl.computed)) != 0) return rc;
    return m40llm_cuda_event_create(ctx_, &sl.arrived);
}

int DecodeLayer::forward_host_begin(uint32_t slot, M40llmKVCache* kv, const LayerWeights& w,
                                    const KvCompressionConfig& kvcfg, const std::vector<DecodeRequestState>& requests,
                                    const float* x_host, bool use_graph) {
    if (!ok_) return fail(-1, "workspace");
    if (slot > 1) return fail(-2, "slot");
    Slot& sl = slots_[slot];
    if (sl.busy) return fail(-2, "slot_busy");
    DecodeBatchPlan plan;
    const std::string err = DecodeBatchPlan::from_requests(requests, &plan);
    if (!err.empty()) {
        failed_step_ = err;
        return -4;
    }
    const uint32_t rows = plan.batch_size();
    if (rows > max_rows_) return fail(-2, "rows");
    int rc = slot_ready(slot);
    if (rc != 0) return fail(rc, "slot_alloc");
    // the slot's previous step has been ended (its result arrived), so nothing reads its plan or staging any more
    if ((rc = sl.plan.upload(ctx_, plan, 0u, false)) != 0) return fail(rc, "plan_upload");
    const size_t bytes = (size_t)rows * cfg_.hidden * 4;
    if ((rc = m40llm_memcpy_h2d_async(ctx_, sl.d_xin, x_host, bytes, 0u)) != 0) return fail(rc, "memcpy_h2d");
    if ((rc = m40llm_stream_wait_for_stream(ctx_, 1u, 0u)) != 0) return fail(rc, "stream_wait_for_stream");
    if ((rc = forward_device(kv, w, kvcfg, plan, sl.plan, sl.d_xin, sl.d_xout, use_graph)) != 0) return rc;
    if ((rc = m40llm_cuda_event_record(ctx_, sl.computed, 1u)) != 0) return fail(rc, "event_record");
    sl.rows = rows;
    sl.busy = true;
    return 0;
}

int DecodeLayer::forward_host_end(uint32_t slot, float* out_host) {
    if (!ok_) return fail(-1, "workspace");
    if (slot > 1 || !slots_[slot].busy) return fail(-2, "slot");
    Slot& sl = slots_[slot];
    sl.busy = false;
    int rc;
    if ((rc = m40llm_stream_wait_event(ctx_, 0u, sl.computed)) != 0) return fail(rc, "stream_wait_event");
    if ((rc = m40llm_memcpy_d2h_async(ctx_, out_host, sl.d_xout, (size_t)sl.rows * cfg_.hidden * 4, 0u)) != 0)
        return fail(rc, "memcpy_d2h");
    if ((rc = m40llm_cuda_event_record(ctx_, sl.arrived, 0u)) != 0) return fail(rc, "event_record");
    if ((rc = m40llm_cuda_event_synchronize(ctx_, sl.arrived)) != 0) return fail(rc, "event_synchronize");
    return 0;
}

}  // namespace m40host
