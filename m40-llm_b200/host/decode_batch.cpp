#include "decode_batch.hpp"

namespace m40host {

std::string DecodeBatchPlan::from_requests(const std::vector<DecodeRequestState>& requests, DecodeBatchPlan* out) {
    DecodeBatchPlan plan;
    for (const auto& r : requests) {
        if (!r.active) continue;
        if (r.kv_len == 0) return "active request " + std::to_string(r.request_id) + " has zero kv_len";
        plan.entries_.push_back({r.request_id, r.sequence_id, r.kv_len, plan.entries_.size()});
    }
    if (plan.entries_.empty()) return "decode batch requires at least one active request";
    *out = plan;
    return "";
}

std::vector<uint32_t> DecodeBatchPlan::sequence_ids() const {
    std::vector<uint32_t> v;
    for (const auto& e : entries_) v.push_back(e.sequence_id);
    return v;
}

std::vector<uint32_t> DecodeBatchPlan::sequence_lens() const {
    std::vector<uint32_t> v;
    for (const auto& e : entries_) v.push_back(e.kv_len);
    return v;
}

long DecodeBatchPlan::batch_index_for_request(uint64_t request_id) const {
    for (const auto& e : entries_)
        if (e.request_id == request_id) return (long)e.batch_index;
    return -1;
}

long DecodeBatchPlan::output_offset_f32(uint64_t request_id, uint32_t q_heads, uint32_t head_dim) const {
    const long idx = batch_index_for_request(request_id);
    return idx < 0 ? -1 : idx * (long)q_heads * (long)head_dim;
}

CudaDecodeBatchPlan::~CudaDecodeBatchPlan() {
    if (ctx_) {
        m40llm_device_free(ctx_, d_ids_);
        m40llm_device_free(ctx_, d_lens_);
        m40llm_device_free(ctx_, d_pos_);
    }
}

int CudaDecodeBatchPlan::upload(M40llmCudaContext* ctx, const DecodeBatchPlan& plan) {
    const uint32_t n = plan.batch_size();
    if (n > capacity_ || ctx != ctx_) {
        if (ctx_) {
            m40llm_device_free(ctx_, d_ids_);
            m40llm_device_free(ctx_, d_lens_);
            m40llm_device_free(ctx_, d_pos_);
        }
        ctx_ = ctx;
        d_ids_ = d_lens_ = d_pos_ = nullptr;
        capacity_ = 0;
        int rc;
        if ((rc = m40llm_device_malloc(ctx, n * 4, (void**)&d_ids_)) != 0) return rc;
        if ((rc = m40llm_device_malloc(ctx, n * 4, (void**)&d_lens_)) != 0) return rc;
        if ((rc = m40llm_device_malloc(ctx, n * 4, (void**)&d_pos_)) != 0) return rc;
        capacity_ = n;
    }
    const std::vector<uint32_t> ids = plan.sequence_ids(), lens = plan.sequence_lens();
    std::vector<uint32_t> pos(n);
    for (uint32_t i = 0; i < n; ++i) pos[i] = lens[i] - 1;
    int rc;
    if ((rc = m40llm_memcpy_h2d(ctx, d_ids_, ids.data(), n * 4)) != 0) return rc;
    if ((rc = m40llm_memcpy_h2d(ctx, d_lens_, lens.data(), n * 4)) != 0) return rc;
    if ((rc = m40llm_memcpy_h2d(ctx, d_pos_, pos.data(), n * 4)) != 0) return rc;
    batch_ = n;
    return 0;
}

}  // namespace m40host
