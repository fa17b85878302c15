// Dense last-token GQA attention that never allocates.
//
// The regular entry point keeps its per-split (max, sum, out) partials in a context arena that grows with
// cudaMalloc on demand. Some callers cannot tolerate an allocating call at all: a serving loop that has handed
// every remaining byte of HBM to its KV pool (a late cudaMalloc would fail or fragment), and code that runs
// where the allocator must not be entered (inside another library's callback, or under a latency budget that
// an implicit device synchronisation by cudaMalloc/cudaFree would break). For them this file keeps the partials
// in a fixed array that is part of the loaded module: its storage exists as soon as the library is loaded on a
// device, so no call here creates or frees memory.
//
// Limits and sharing rules:
//   * the array holds M40_STATIC_ATTN_FLOATS floats (4 MiB); a call whose partials would not fit is rejected
//     with M40LLM_ERR_LIMIT and nothing is launched;
//   * every call on a device shares the one array. Nothing in it has to start at zero (each split writes its
//     triple before the merge reads it), so no clearing is needed; but two calls in flight at once on
//     different streams or contexts of the same device overwrite each other's partials: callers serialise them;
//   * the array's device address is looked up with cudaGetSymbolAddress the first time a device is used, with
//     that device current. That first call per device is the set-up call and should be made before any stream
//     capture begins. The first call per head shape on a device also raises that kernel's shared-memory limit
//     (cudaFuncSetAttribute; no allocation). Later calls only launch kernels;
//   * only the shapes of the tiled kernel are taken (head_dim 64 or 128, at most 16 q heads per kv head, q
//     8-byte aligned); others get M40LLM_ERR_UNSUPPORTED.
#include "attention.cuh"

#include <mutex>

#define M40_STATIC_ATTN_FLOATS (1u << 20)
#define M40_STATIC_MAX_DEVICES 64

static __device__ __align__(256) float g_static_attn_partials[M40_STATIC_ATTN_FLOATS];

namespace {
std::mutex g_lookup_mutex;
float* g_partials_addr[M40_STATIC_MAX_DEVICES] = {};

// Device address of the array on the context's device (looked up once per device, that device current).
int static_partials(M40llmCudaContext* ctx, float** out) {
    const int dev = ctx->device_id;
    if (dev < 0 || dev >= M40_STATIC_MAX_DEVICES) return M40LLM_ERR_LIMIT;
    std::lock_guard<std::mutex> lock(g_lookup_mutex);
    if (!g_partials_addr[dev]) {
        void* p = nullptr;
        const cudaError_t e = cudaGetSymbolAddress(&p, g_static_attn_partials);
        if (e != cudaSuccess || !p) {
            fprintf(stderr, "m40llm: cudaGetSymbolAddress(static attention partials) failed on device %d: %s\n", dev,
                    cudaGetErrorString(e));
            return M40LLM_ERR_SYMBOL;
        }
        g_partials_addr[dev] = (float*)p;
    }
    *out = g_partials_addr[dev];
    return 0;
}
}  // namespace

extern "C" int m40llm_attention_last_token_f32_gqa_static_async(M40llmCudaContext* ctx, const M40llmKVCache* kv,
                                                                uint32_t seq_id, const void* d_q_f32,
                                                                uint32_t q_heads, uint32_t seq_len,
                                                                void* d_out_f32) {
    if (!ctx || !kv || !d_q_f32 || !d_out_f32) return -1;
    if (seq_id >= kv->max_batch_size) return -2;
    if (seq_len == 0 || seq_len > kv->max_seq_len) return -3;
    if (q_heads == 0 || kv->num_heads == 0 || q_heads % kv->num_heads != 0) return -6;
    if (!kv->d_k || !kv->d_v) return -4;
    if (m40_ensure_device(ctx) != 0) return -1;

    DenseAttnArgs a = {};
    a.K = kv->d_k;
    a.V = kv->d_v;
    a.q = (const float*)d_q_f32;
    a.out = (float*)d_out_f32;
    a.status = ctx->d_status;
    a.seq_id = seq_id;
    a.seq_len = seq_len;
    a.max_seq_len = kv->max_seq_len;
    a.max_batch = kv->max_batch_size;
    a.kv_heads = kv->num_heads;
    a.q_heads = q_heads;
    a.hd = kv->head_dim;
    a.inv_sqrt = attn_inv_sqrt(kv->head_dim);
    m40_attn_pick_chunk(ctx, 1, kv->num_heads, seq_len, &a.chunk, &a.splits);

    // Looked up on every path (also when one split needs no partials) so that the first call on a device is
    // always the one that does the set-up.
    float* base = nullptr;
    const int lookup_rc = static_partials(ctx, &base);
    if (lookup_rc != 0) return lookup_rc;
    if (a.splits > 1) {
        const size_t n = (size_t)q_heads * a.splits;
        const size_t need = n * (2 + (size_t)a.hd);
        if (need > (size_t)M40_STATIC_ATTN_FLOATS) {
            fprintf(stderr,
                    "m40llm: static attention needs %zu floats of partials (q_heads %u x splits %u x (2 + head_dim %u)); "
                    "the fixed array holds %u\n",
                    need, q_heads, a.splits, a.hd, (unsigned)M40_STATIC_ATTN_FLOATS);
            return M40LLM_ERR_LIMIT;
        }
        a.part_m = base;
        a.part_l = base + n;
        a.part_o = base + 2 * n;
    }
    const int rc = m40_attention_dense_tiled(ctx, a, 1);
    if (rc == 1) return M40LLM_ERR_UNSUPPORTED;
    if (rc != 0) return rc;
    if (a.splits > 1)
        return m40_attention_merge_rows(ctx, a.part_m, a.part_l, a.part_o, a.splits, q_heads, a.hd, a.out, 1);
    return 0;
}
