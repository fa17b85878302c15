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
        m40llm_stream_synchronize(ctx_, 1u);
        m40llm_device_free(ctx_, d_ids_);
    }
}

// One stream-ordered copy of [ids | lens | positions] onto the decode stream: the kernels that read the plan are
// enqueued behind it on the same stream, so no host synchronisation is needed here.
int CudaDecodeBatchPlan::upload(M40llmCudaContext* ctx, const DecodeBatchPlan& plan, uint32_t stream_kind, bool sync_first) {
    const uint32_t n = plan.batch_size();
    if (n > capacity_ || ctx != ctx_) {
        if (ctx_) {
            m40llm_stream_synchronize(ctx_, 1u);
            m40llm_device_free(ctx_, d_ids_);
        }
        ctx_ = ctx;
        d_ids_ = d_lens_ = d_pos_ = nullptr;
        capacity_ = 0;
        const int rc = m40llm_device_malloc(ctx, (size_t)3 * n * 4, (void**)&d_ids_);
        if (rc != 0) return rc;
        capacity_ = n;
    }
    d_lens_ = d_ids_ + capacity_;
    d_pos_ = d_ids_ + 2 * (size_t)capacity_;
    // the previous copy out of the staging vector must have left it before it is overwritten
    int rc = sync_first ? m40llm_stream_synchronize(ctx, stream_kind) : 0;
    if (rc != 0) return rc;
    staging_.assign((size_t)3 * capacity_, 0u);
    const std::vector<uint32_t> ids = plan.sequence_ids(), lens = plan.sequence_lens();
    for (uint32_t i = 0; i < n; ++i) {
        staging_[i] = ids[i];
        staging_[capacity_ + i] = lens[i];
        staging_[2 * (size_t)capacity_ + i] = lens[i] - 1;
    }
    if ((rc = m40llm_memcpy_h2d_async(ctx, d_ids_, staging_.data(), staging_.size() * 4, stream_kind)) != 0) return rc;
    batch_ = n;
    return 0;
}

}  // namespace m40host
