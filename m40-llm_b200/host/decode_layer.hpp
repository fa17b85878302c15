// One decode layer over a batch of rows, issued through the m40llm C ABI only.
// Host-side mirror of the reference's layer driver: the 13-step sequence of
// src/infer/forward.rs:247-667 (forward_one_token_minimal_with_norms), its batched form
// src/infer/forward.rs:1729-2140, the attention-mode dispatch of src/infer/kv.rs:433-765 and the optional
// CUDA-graph replay of src/decode_session.rs:828-954. On this library the sequence is:
//   1. m40llm_qkv_rmsnorm_rope_append_async      (steps 1-5: norm, QKV (+bias), RoPE(q), RoPE(k)+append)
//   2. attention: dense batched, or block-select FP16-K/q4-V per row (step 6)
//   3. Wo projection, then x1 = x + y            (steps 7-8)
//   4. weighted RMSNorm                          (step 9)
//   5. SwiGLU FFN with residual epilogue          (steps 10-13), Q8_0 or f16 weights
#pragma once
#include <stdint.h>

#include <string>
#include <vector>

#include "../../include/m40llm_native.h"
#include "decode_batch.hpp"
#include "kv_compression.hpp"

namespace m40host {

// src/infer/types.rs:18-41 (the fields the layer math needs)
struct ModelConfig {
    uint32_t hidden = 0, q_heads = 0, kv_heads = 0, head_dim = 0, ffn = 0;
    float rms_eps = 1e-5f, rope_base = 10000.0f, rope_scale = 1.0f;
    uint32_t rope_layout = 0;  // 0 adjacent pairs (llama), 1 NeoX split-half (qwen)
};

// Device pointers of one layer's weights (GGUF layout [N][K]); owned by the caller.
struct LayerWeights {
    const void* attn_norm = nullptr;  // f32 [hidden]
    const void* ffn_norm = nullptr;   // f32 [hidden]
    const void *wq = nullptr, *wk = nullptr, *wv = nullptr, *wo = nullptr;  // f16
    const void *bq = nullptr, *bk = nullptr, *bv = nullptr;                 // f32 or null
    const void *wg = nullptr, *wu = nullptr, *wd = nullptr;                 // f16 or Q8_0 rows
    bool ffn_q80 = false;
};

class DecodeLayer {
public:
    DecodeLayer(M40llmCudaContext* ctx, const ModelConfig& cfg, uint32_t max_rows);
    ~DecodeLayer();
    DecodeLayer(const DecodeLayer&) = delete;
    DecodeLayer& operator=(const DecodeLayer&) = delete;
    bool ok() const { return ok_; }

    // Device in / device out: d_x, d_out f32 [rows][hidden]. Everything is enqueued on the decode stream.
    // Returns 0 or the first failing ABI return code; `failed_step` names it.
    int forward_device(M40llmKVCache* kv, const LayerWeights& w, const KvCompressionConfig& kvcfg,
                       const DecodeBatchPlan& plan, const CudaDecodeBatchPlan& dplan, const void* d_x, void* d_out,
                       bool use_graph);
    // Host in / host out (the end-to-end call): copies x and the plan to the device, runs the layer, copies the
    // result back and synchronises.
    int forward_host(M40llmKVCache* kv, const LayerWeights& w, const KvCompressionConfig& kvcfg,
                     const std::vector<DecodeRequestState>& requests, const float* x_host, float* out_host,
                     bool use_graph);
    // The same call in two halves, for two steps in flight (slot 0 or 1, each with its own staging buffers and plan):
    // `begin` copies the plan and x on the PREFILL stream, makes the decode stream wait for them and enqueues the layer;
    // `end` copies the slot's result back on the prefill stream behind the layer and blocks until it has arrived. A
    // caller that begins step i + 1 before it ends step i overlaps i + 1's upload and i's download with the compute
    // of the other step; the layer kernels themselves stay in order on the decode stream. A slot must be ended before
    // it is begun again.
    int forward_host_begin(uint32_t slot, M40llmKVCache* kv, const LayerWeights& w, const KvCompressionConfig& kvcfg,
                           const std::vector<DecodeRequestState>& requests, const float* x_host, bool use_graph);
    int forward_host_end(uint32_t slot, float* out_host);
    const std::string& failed_step() const { return failed_step_; }
    uint64_t graph_replays() const { return graph_replays_; }

private:
    int enqueue(M40llmKVCache* kv, const LayerWeights& w, const KvCompressionConfig& kvcfg,
                const DecodeBatchPlan& plan, const CudaDecodeBatchPlan& dplan, const void* d_x, void* d_out);
    int fail(int rc, const char* step);
    struct GraphKey {
        const void *kv, *wq, *wg, *x, *out, *ids;
        uint32_t rows;
        bool operator==(const GraphKey& o) const {
            return kv == o.kv && wq == o.wq && wg == o.wg && x == o.x && out == o.out && ids == o.ids && rows == o.rows;
        }
    };
    struct GraphEntry { GraphKey key; M40llmCudaGraphExec* exec; };

    M40llmCudaContext* ctx_;
    ModelConfig cfg_;
    uint32_t max_rows_;
    bool ok_ = false;
    void *d_q_ = nullptr, *d_att_ = nullptr, *d_x1_ = nullptr, *d_x1n_ = nullptr, *d_hid_ = nullptr;
    void *d_xin_ = nullptr, *d_xout_ = nullptr;  // staging for forward_host
    CudaDecodeBatchPlan host_plan_dev_;
    struct Slot {
        void *d_xin = nullptr, *d_xout = nullptr;
        CudaDecodeBatchPlan plan;
        M40llmCudaEvent *computed = nullptr, *arrived = nullptr;
        uint32_t rows = 0;
        bool busy = false;
    } slots_[2];
    int slot_ready(uint32_t slot);
    std::vector<GraphEntry> graphs_;
    std::string failed_step_;
    uint64_t graph_replays_ = 0;
};

}  // namespace m40host
