// Plain-C surface of the host mirror so that harnesses (ctypes) can drive it; every function returns 0 or a
// negative code and m40host_last_error() gives the text.
#include <string.h>

#include <string>

#include "decode_batch.hpp"
#include "decode_layer.hpp"
#include "decode_model.hpp"
#include "kv_compression.hpp"

using namespace m40host;

static thread_local std::string g_err;

extern "C" {

struct m40host_layer_cfg {
    uint32_t hidden, q_heads, kv_heads, head_dim, ffn, rope_layout;
    float rms_eps, rope_base, rope_scale;
};

struct m40host_weights {
    const void *attn_norm, *ffn_norm, *wq, *wk, *wv, *wo, *bq, *bk, *bv, *wg, *wu, *wd;
    uint32_t ffn_q80;
};

struct m40host_kv_cfg {
    uint32_t mode, recent_window, block_size, top_blocks, representatives, representative_policy, exact_old_backing,
        exact_old_attention;
};

static KvCompressionConfig to_cfg(const m40host_kv_cfg* c) {
    KvCompressionConfig k;
    k.mode = (KvCompressMode)c->mode;
    k.recent_window = c->recent_window;
    k.block_size = c->block_size;
    k.top_blocks = c->top_blocks;
    k.representatives = c->representatives;
    k.representative_policy = (KvRepresentativePolicy)c->representative_policy;
    k.exact_old_backing = (KvExactOldBacking)c->exact_old_backing;
    k.exact_old_attention = (KvExactOldAttention)c->exact_old_attention;
    return k;
}

const char* m40host_last_error(void) { return g_err.c_str(); }

void m40host_kv_cfg_default(m40host_kv_cfg* out) {
    const KvCompressionConfig k;
    *out = {(uint32_t)k.mode, k.recent_window, k.block_size, k.top_blocks, k.representatives,
            (uint32_t)k.representative_policy, (uint32_t)k.exact_old_backing, (uint32_t)k.exact_old_attention};
}

// which: 0 validate, 1 validate_runtime_support, 2 validate_b200_support
int m40host_kv_cfg_validate(const m40host_kv_cfg* c, uint32_t which, uint32_t max_seq_len, uint32_t head_dim) {
    const KvCompressionConfig k = to_cfg(c);
    g_err = which == 0 ? k.validate()
                       : (which == 1 ? k.validate_runtime_support(max_seq_len, head_dim)
                                     : k.validate_b200_support(max_seq_len, head_dim));
    return g_err.empty() ? 0 : -1;
}

// requests: n x {request_id, sequence_id, kv_len, active} as u64,u32,u32,u32 arrays. Outputs sized n.
int m40host_plan_from_requests(uint32_t n, const uint64_t* request_ids, const uint32_t* sequence_ids,
                               const uint32_t* kv_lens, const uint32_t* active, uint32_t* out_batch,
                               uint32_t* out_seq_ids, uint32_t* out_seq_lens, uint64_t* out_request_ids) {
    std::vector<DecodeRequestState> r;
    for (uint32_t i = 0; i < n; ++i) r.push_back({request_ids[i], sequence_ids[i], kv_lens[i], active[i] != 0});
    DecodeBatchPlan plan;
    g_err = DecodeBatchPlan::from_requests(r, &plan);
    if (!g_err.empty()) return -1;
    *out_batch = plan.batch_size();
    for (const auto& e : plan.entries()) {
        out_seq_ids[e.batch_index] = e.sequence_id;
        out_seq_lens[e.batch_index] = e.kv_len;
        out_request_ids[e.batch_index] = e.request_id;
    }
    return 0;
}

void* m40host_layer_create(M40llmCudaContext* ctx, const m40host_layer_cfg* c, uint32_t max_rows) {
    ModelConfig m;
    m.hidden = c->hidden; m.q_heads = c->q_heads; m.kv_heads = c->kv_heads; m.head_dim = c->head_dim; m.ffn = c->ffn;
    m.rope_layout = c->rope_layout; m.rms_eps = c->rms_eps; m.rope_base = c->rope_base; m.rope_scale = c->rope_scale;
    DecodeLayer* l = new DecodeLayer(ctx, m, max_rows);
    if (!l->ok()) {
        delete l;
        g_err = "workspace allocation failed";
        return nullptr;
    }
    return l;
}

void m40host_layer_destroy(void* layer) { delete (DecodeLayer*)layer; }

// The end-to-end call: host activations in, host activations out, one layer step for the active requests.
int m40host_layer_forward_host(void* layer, M40llmKVCache* kv, const m40host_weights* w, const m40host_kv_cfg* kc,
                               uint32_t n, const uint64_t* request_ids, const uint32_t* sequence_ids,
                               const uint32_t* kv_lens, const uint32_t* active, const float* x_host, float* out_host,
                               uint32_t use_graph) {
    DecodeLayer* l = (DecodeLayer*)layer;
    LayerWeights lw;
    lw.attn_norm = w->attn_norm; lw.ffn_norm = w->ffn_norm; lw.wq = w->wq; lw.wk = w->wk; lw.wv = w->wv; lw.wo = w->wo;
    lw.bq = w->bq; lw.bk = w->bk; lw.bv = w->bv; lw.wg = w->wg; lw.wu = w->wu; lw.wd = w->wd; lw.ffn_q80 = w->ffn_q80 != 0;
    std::vector<DecodeRequestState> r;
    for (uint32_t i = 0; i < n; ++i) r.push_back({request_ids[i], sequence_ids[i], kv_lens[i], active[i] != 0});
    const int rc = l->forward_host(kv, lw, to_cfg(kc), r, x_host, out_host, use_graph != 0);
    if (rc != 0) g_err = l->failed_step();
    return rc;
}

// The same call in two halves (two steps in flight, slot 0 or 1): see DecodeLayer::forward_host_begin / _end.
int m40host_layer_forward_host_begin(void* layer, uint32_t slot, M40llmKVCache* kv, const m40host_weights* w,
                                     const m40host_kv_cfg* kc, uint32_t n, const uint64_t* request_ids,
                                     const uint32_t* sequence_ids, const uint32_t* kv_lens, const uint32_t* active,
                                     const float* x_host, uint32_t use_graph) {
    DecodeLayer* l = (DecodeLayer*)layer;
    LayerWeights lw;
    lw.attn_norm = w->attn_norm; lw.ffn_norm = w->ffn_norm; lw.wq = w->wq; lw.wk = w->wk; lw.wv = w->wv; lw.wo = w->wo;
    lw.bq = w->bq; lw.bk = w->bk; lw.bv = w->bv; lw.wg = w->wg; lw.wu = w->wu; lw.wd = w->wd; lw.ffn_q80 = w->ffn_q80 != 0;
    std::vector<DecodeRequestState> r;
    for (uint32_t i = 0; i < n; ++i) r.push_back({request_ids[i], sequence_ids[i], kv_lens[i], active[i] != 0});
    const int rc = l->forward_host_begin(slot, kv, lw, to_cfg(kc), r, x_host, use_graph != 0);
    if (rc != 0) g_err = l->failed_step();
    return rc;
}

int m40host_layer_forward_host_end(void* layer, uint32_t slot, float* out_host) {
    DecodeLayer* l = (DecodeLayer*)layer;
    const int rc = l->forward_host_end(slot, out_host);
    if (rc != 0) g_err = l->failed_step();
    return rc;
}

uint64_t m40host_layer_graph_replays(void* layer) { return ((DecodeLayer*)layer)->graph_replays(); }


// ---- whole-model greedy decode (decode_model.hpp)
struct m40host_model_head {
    const void *embeddings, *output_norm, *lm_head;
    uint32_t vocab;
};

void* m40host_model_create(M40llmCudaContext* ctx, const m40host_layer_cfg* c, uint32_t n_layers,
                           const m40host_weights* layers, const m40host_model_head* head, M40llmKVCache* kv,
                           uint32_t sequences) {
    if (!ctx || !c || !layers || !head || !kv || n_layers == 0) {
        g_err = "m40host_model_create: null argument";
        return nullptr;
    }
    ModelConfig m;
    m.hidden = c->hidden, m.q_heads = c->q_heads, m.kv_heads = c->kv_heads, m.head_dim = c->head_dim, m.ffn = c->ffn;
    m.rope_layout = c->rope_layout, m.rms_eps = c->rms_eps, m.rope_base = c->rope_base, m.rope_scale = c->rope_scale;
    std::vector<LayerWeights> lw(n_layers);
    for (uint32_t i = 0; i < n_layers; ++i) {
        const m40host_weights& w = layers[i];
        lw[i].attn_norm = w.attn_norm, lw[i].ffn_norm = w.ffn_norm;
        lw[i].wq = w.wq, lw[i].wk = w.wk, lw[i].wv = w.wv, lw[i].wo = w.wo;
        lw[i].bq = w.bq, lw[i].bk = w.bk, lw[i].bv = w.bv;
        lw[i].wg = w.wg, lw[i].wu = w.wu, lw[i].wd = w.wd;
        lw[i].ffn_q80 = w.ffn_q80 != 0;
    }
    ModelHead h;
    h.embeddings = head->embeddings, h.output_norm = head->output_norm, h.lm_head = head->lm_head, h.vocab = head->vocab;
    DecodeModel* dm = new DecodeModel(ctx, m, lw, h, kv, sequences);
    if (!dm->ok()) {
        g_err = "m40host_model_create: device allocation failed or bad arguments";
        delete dm;
        return nullptr;
    }
    return dm;
}

void m40host_model_destroy(void* model) { delete (DecodeModel*)model; }

int m40host_model_begin(void* model, const uint32_t* token_ids, const uint32_t* positions) {
    DecodeModel* dm = (DecodeModel*)model;
    const int rc = dm->begin(token_ids, positions);
    if (rc != 0) g_err = "model begin failed at " + dm->failed_step() + " rc=" + std::to_string(rc);
    return rc;
}

int m40host_model_generate(void* model, uint32_t steps, uint32_t use_graph, uint32_t* out_ids, float* out_logits) {
    DecodeModel* dm = (DecodeModel*)model;
    const int rc = dm->generate(steps, use_graph != 0, out_ids, out_logits);
    if (rc != 0) g_err = "model generate failed at " + dm->failed_step() + " rc=" + std::to_string(rc);
    return rc;
}

uint64_t m40host_model_graph_replays(void* model) { return ((DecodeModel*)model)->graph_replays(); }
uint64_t m40host_model_launches_per_step(void* model) { return ((DecodeModel*)model)->launches_per_step(); }

}  // extern "C"
