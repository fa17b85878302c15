// Decode batch plan: active requests -> (sequence ids, kv lengths) in batch order, uploaded once per step.
// Host-side mirror of the reference's src/decode_batch.rs (DecodeBatchPlan :143-230, CudaDecodeBatchPlan :232-286).
#pragma once
#include <stdint.h>

#include <string>
#include <vector>

#include "../../include/m40llm_native.h"

namespace m40host {

struct DecodeRequestState {
    uint64_t request_id;
    uint32_t sequence_id;
    uint32_t kv_len;   // tokens in the cache INCLUDING the token decoded this step
    bool active;
};

struct DecodeBatchEntry {
    uint64_t request_id;
    uint32_t sequence_id;
    uint32_t kv_len;
    size_t batch_index;
};

class DecodeBatchPlan {
public:
    // Keeps active requests in order; error (non-empty) when none is active or one has kv_len == 0
    // (src/decode_batch.rs:150-181).
    static std::string from_requests(const std::vector<DecodeRequestState>& requests, DecodeBatchPlan* out);
    const std::vector<DecodeBatchEntry>& entries() const { return entries_; }
    uint32_t batch_size() const { return (uint32_t)entries_.size(); }
    std::vector<uint32_t> sequence_ids() const;
    std::vector<uint32_t> sequence_lens() const;
    // -1 when the request is not part of the batch (src/decode_batch.rs:207-228)
    long batch_index_for_request(uint64_t request_id) const;
    long output_offset_f32(uint64_t request_id, uint32_t q_heads, uint32_t head_dim) const;

private:
    std::vector<DecodeBatchEntry> entries_;
};

// Device copy of a plan (ids, lengths, positions = length - 1), owned through the C ABI's malloc/free.
class CudaDecodeBatchPlan {
public:
    CudaDecodeBatchPlan() = default;
    ~CudaDecodeBatchPlan();
    CudaDecodeBatchPlan(const CudaDecodeBatchPlan&) = delete;
    CudaDecodeBatchPlan& operator=(const CudaDecodeBatchPlan&) = delete;
    // 0 or the failing ABI return code. The copy rides `stream_kind` (1 = decode, 0 = prefill). The staging vector is
    // pageable, so the copy has left it when the call returns; `sync_first` additionally drains that stream before the
    // device block is rewritten (needed when kernels of an earlier step may still read it).
    int upload(M40llmCudaContext* ctx, const DecodeBatchPlan& plan, uint32_t stream_kind = 1u, bool sync_first = true);
    const uint32_t* d_sequence_ids() const { return d_ids_; }
    const uint32_t* d_sequence_lens() const { return d_lens_; }
    const uint32_t* d_positions() const { return d_pos_; }
    uint32_t batch_size() const { return batch_; }

private:
    M40llmCudaContext* ctx_ = nullptr;
    uint32_t *d_ids_ = nullptr, *d_lens_ = nullptr, *d_pos_ = nullptr;  // three views of one device block
    std::vector<uint32_t> staging_;  // [ids | lens | positions], alive until the stream has passed the copy
    uint32_t batch_ = 0, capacity_ = 0;
};

}  // namespace m40host
