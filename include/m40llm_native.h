/*
 * m40llm_native.h — C ABI of the B200 (sm_100a) native decode library.
 *
 * This is the drop-in boundary: the same `m40llm_*` symbols, argument order,
 * return-code convention (0 = ok, negative = the check that failed) and stream
 * semantics as the `extern "C"` block the reference host binds in
 * src/cuda.rs:87-682 (defined by cuda/kernels.cu in the reference). Each
 * declaration cites the reference definition it replaces.
 *
 * Conventions shared by every entry point:
 *   - `ctx` owns two streams: kind 0 = "prefill" (GEMMs, casts), kind 1 =
 *     "decode" (norm, rope, residual, swiglu, KV append, attention). `_async`
 *     entry points enqueue and return; the others also synchronise their stream.
 *   - All tensor arguments are raw device pointers owned by the caller.
 *   - The KV cache is opaque; its device layout is private to the library.
 *   - No C++ types, no exceptions, no torch types cross this boundary.
 */
#ifndef M40LLM_NATIVE_H
#define M40LLM_NATIVE_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef struct M40llmCudaContext M40llmCudaContext;
typedef struct M40llmKVCache M40llmKVCache;
typedef struct M40llmCudaGraphExec M40llmCudaGraphExec;
typedef struct M40llmCudaEvent M40llmCudaEvent;

/* Returned by entry points whose mode the B200 library does not implement
 * (lossy summary modes, q8 KV backing, staged gather, the persistent-kernel
 * prototype). The reference host maps any non-zero code to an error. */
#define M40LLM_ERR_UNSUPPORTED (-100)
/* Returned by the additive entry points when a size exceeds a documented limit. */
#define M40LLM_ERR_LIMIT (-101)
/* Returned by the allocation-free entry point when the address of its fixed device array cannot be looked up. */
#define M40LLM_ERR_SYMBOL (-102)

/* Telemetry structs, src/cuda.rs:46-85 <-> cuda/kernels.cu:84-115. */
typedef struct { float prob_mass, logit_max, logit_mean; uint32_t count; } M40llmAttentionGroupStats;
typedef struct { uint32_t group, block_index, token_position; float score, probability; } M40llmAttentionTopEntry;
typedef struct { uint32_t block_index; float prob_mass, logit_max, logit_mean; uint32_t count; } M40llmAttentionBlockMass;
typedef struct {
    M40llmAttentionGroupStats recent, selected_old_exact, summary, representatives, other;
    float needle_block_mass;
    M40llmAttentionBlockMass selected_block_masses[64];
    uint32_t selected_block_mass_count;
    M40llmAttentionTopEntry top_entries[8];
    uint32_t top_entry_count;
} M40llmAttentionTelemetry;

/* ------------------------------------------------------------------ lifecycle */
/* cuda/kernels.cu:366-474 (device_id < 0 = auto: first sm_100 device, else 0). */
M40llmCudaContext* m40llm_create_context(int device_id);
/* cuda/kernels.cu:8027-8042 */
void m40llm_destroy_context(M40llmCudaContext* ctx);
/* cuda/kernels.cu:1245-1263 */
int m40llm_current_device_props(char* name_buf, size_t buf_len, int* major, int* minor, int* device_id);
/* cuda/kernels.cu:302-319 */
int m40llm_device_malloc(M40llmCudaContext* ctx, size_t bytes, void** out_ptr);
int m40llm_device_free(M40llmCudaContext* ctx, void* ptr);
/* cuda/kernels.cu:321-355 */
int m40llm_memcpy_h2d(M40llmCudaContext* ctx, void* dst_device, const void* src_host, size_t bytes);
int m40llm_memcpy_d2h(M40llmCudaContext* ctx, void* dst_host, const void* src_device, size_t bytes);
int m40llm_memcpy_d2d_async(M40llmCudaContext* ctx, void* dst_device, const void* src_device, size_t bytes,
                            uint32_t stream_kind);
/* cuda/kernels.cu:357-364 */
int m40llm_validate_device_ptr(const void* ptr);
/* cuda/kernels.cu:1268-1292 */
int m40llm_upload_weights(M40llmCudaContext* ctx, const void* host_ptr, size_t num_bytes, void** out_device_ptr);
/* cuda/kernels.cu:476-514 */
int m40llm_stream_synchronize(M40llmCudaContext* ctx, uint32_t stream_kind);
int m40llm_stream_wait_for_stream(M40llmCudaContext* ctx, uint32_t waiting_stream_kind, uint32_t signal_stream_kind);
/* cuda/kernels.cu:516-626, 675-680 */
int m40llm_cuda_graph_begin_capture(M40llmCudaContext* ctx, uint32_t stream_kind);
int m40llm_cuda_graph_end_capture(M40llmCudaContext* ctx, uint32_t stream_kind, M40llmCudaGraphExec** out_graph);
int m40llm_cuda_graph_cancel_capture(M40llmCudaContext* ctx, uint32_t stream_kind);
int m40llm_cuda_graph_launch(M40llmCudaContext* ctx, M40llmCudaGraphExec* graph, uint32_t stream_kind);
int m40llm_cuda_graph_launch_timed_sync(M40llmCudaContext* ctx, M40llmCudaGraphExec* graph, uint32_t stream_kind,
                                        float* elapsed_ms);
void m40llm_cuda_graph_destroy(M40llmCudaGraphExec* graph);
/* cuda/kernels.cu:628-673 */
int m40llm_cuda_event_create(M40llmCudaContext* ctx, M40llmCudaEvent** out_event);
int m40llm_cuda_event_record(M40llmCudaContext* ctx, M40llmCudaEvent* event, uint32_t stream_kind);
int m40llm_cuda_event_elapsed_sync(M40llmCudaContext* ctx, M40llmCudaEvent* start, M40llmCudaEvent* stop,
                                   float* elapsed_ms);
void m40llm_cuda_event_destroy(M40llmCudaEvent* event);
/* Additive (no counterpart in cuda/kernels.cu): make a stream wait for a recorded event, and block the host on one.
 * With them a caller can keep two steps in flight: the next step's host-to-device copies on the prefill stream while
 * the decode stream computes, and a step's result copied back while the next one runs. 0, or -1 null argument,
 * -2 device, -3 / -4 the CUDA call failed. */
int m40llm_stream_wait_event(M40llmCudaContext* ctx, uint32_t waiting_stream_kind, M40llmCudaEvent* event);
int m40llm_cuda_event_synchronize(M40llmCudaContext* ctx, M40llmCudaEvent* event);

/* ---------------------------------------------------- elementwise (decode stream) */
/* cuda/kernels.cu:1049-1068 (kernel 736-768); sync form 1035-1047 */
int m40llm_rms_norm_f32_async(M40llmCudaContext* ctx, const void* d_in, void* d_out, uint32_t rows, uint32_t dim,
                              float eps);
int m40llm_rms_norm_f32(M40llmCudaContext* ctx, const void* d_in, void* d_out, uint32_t rows, uint32_t dim, float eps);
/* cuda/kernels.cu:1086-1127 (kernel 770-807); weight_dtype 0 = f16, 1 = f32; sync form 1070-1084 */
int m40llm_rms_norm_f32_weighted_async(M40llmCudaContext* ctx, const void* d_in, const void* d_weight, void* d_out,
                                       uint32_t rows, uint32_t dim, float eps, uint32_t weight_dtype);
int m40llm_rms_norm_f32_weighted(M40llmCudaContext* ctx, const void* d_in, const void* d_weight, void* d_out,
                                 uint32_t rows, uint32_t dim, float eps, uint32_t weight_dtype);
/* cuda/kernels.cu:7434-7456 (kernel 7258-7298); rope_layout 0 = adjacent pairs, 1 = NeoX split-half */
int m40llm_rope_f32_layout_async(M40llmCudaContext* ctx, float* d_q, float* d_k, uint32_t rows, uint32_t num_heads,
                                 uint32_t head_dim, uint32_t past_len, float freq_base, float freq_scale,
                                 uint32_t rope_layout);
/* cuda/kernels.cu:7402-7432 (adjacent-layout conveniences) */
int m40llm_rope_f32(M40llmCudaContext* ctx, float* d_q, float* d_k, uint32_t rows, uint32_t num_heads,
                    uint32_t head_dim, uint32_t past_len, float freq_base, float freq_scale);
int m40llm_rope_f32_async(M40llmCudaContext* ctx, float* d_q, float* d_k, uint32_t rows, uint32_t num_heads,
                          uint32_t head_dim, uint32_t past_len, float freq_base, float freq_scale);
/* cuda/kernels.cu:7488-7509 (kernel 7300-7332) */
int m40llm_rope_f32_inplace_layout_async(M40llmCudaContext* ctx, float* d_x, uint32_t rows, uint32_t num_heads,
                                         uint32_t head_dim, uint32_t past_len, float freq_base, float freq_scale,
                                         uint32_t rope_layout);
/* cuda/kernels.cu:7458-7486 */
int m40llm_rope_f32_inplace(M40llmCudaContext* ctx, float* d_x, uint32_t rows, uint32_t num_heads, uint32_t head_dim,
                            uint32_t past_len, float freq_base, float freq_scale);
int m40llm_rope_f32_inplace_async(M40llmCudaContext* ctx, float* d_x, uint32_t rows, uint32_t num_heads,
                                  uint32_t head_dim, uint32_t past_len, float freq_base, float freq_scale);
/* cuda/kernels.cu:7525-7546 (kernel 7334-7368): position read from device memory (graph replay) */
int m40llm_rope_f32_inplace_position_dev_layout_async(M40llmCudaContext* ctx, float* d_x, uint32_t rows,
                                                      uint32_t num_heads, uint32_t head_dim,
                                                      const uint32_t* past_len_dev, float freq_base, float freq_scale,
                                                      uint32_t rope_layout);
/* cuda/kernels.cu:7511-7523 */
int m40llm_rope_f32_inplace_position_dev_async(M40llmCudaContext* ctx, float* d_x, uint32_t rows, uint32_t num_heads,
                                               uint32_t head_dim, const uint32_t* past_len_dev, float freq_base,
                                               float freq_scale);
/* cuda/kernels.cu:1188-1207 (kernel 869-878); sync form 1175-1186 */
int m40llm_residual_add_f32_async(M40llmCudaContext* ctx, const void* d_a, const void* d_b, void* d_out, size_t n);
int m40llm_residual_add_f32(M40llmCudaContext* ctx, const void* d_a, const void* d_b, void* d_out, size_t n);
/* cuda/kernels.cu:1222-1241 (kernel 880-891); sync form 1209-1220 */
int m40llm_swiglu_f32_async(M40llmCudaContext* ctx, const void* d_gate, const void* d_up, void* d_out, size_t n);
int m40llm_swiglu_f32(M40llmCudaContext* ctx, const void* d_gate, const void* d_up, void* d_out, size_t n);
/* cuda/kernels.cu:1129-1158 (prefill stream, synchronous) */
int m40llm_f16_to_f32(M40llmCudaContext* ctx, const void* d_in_f16, void* d_out_f32, size_t n);
/* cuda/kernels.cu:1160-1173 (kernel 856-867): GGML Q8_0 {f16 d; int8 qs[32]} -> d*q */
int m40llm_q80_to_f32(M40llmCudaContext* ctx, const void* d_in_q80, void* d_out_f32, size_t n);

/* ------------------------------- GEMM / GEMV (prefill stream); C row-major [M,N] */
/* cuda/kernels.cu:5267-5302: A f16 [M,K] x B f16 [K,N] row-major -> C f32 (synchronous) */
int m40llm_gemm_f16xf16_f32(M40llmCudaContext* ctx, const void* d_A_f16, const void* d_B_f16, void* d_C_f32, int M,
                            int N, int K);
/* cuda/kernels.cu:5106-5155: A f32 x B f16 [K,N] row-major -> C f32 (synchronous) */
int m40llm_gemm_f32xf16_f32(M40llmCudaContext* ctx, const void* d_A_f32, const void* d_B_f16, void* d_C_f32, int M,
                            int N, int K);
/* cuda/kernels.cu:5158-5195: A f32 x B f16 GGUF layout (B[n*K+k]) -> C f32 (synchronous) */
int m40llm_gemm_f32xf16_gguf_f32(M40llmCudaContext* ctx, const void* d_A_f32, const void* d_B_f16, void* d_C_f32,
                                 int M, int N, int K);
/* cuda/kernels.cu:5217-5242: A f32 x Bt f32 (Bt[k*N+n]) -> C f32, asynchronous; sync form 5204-5215 */
int m40llm_gemm_f32xf32_f32_async(M40llmCudaContext* ctx, const void* d_A_f32, const void* d_B_f32_colmajor_nt,
                                  void* d_C_f32, int M, int N, int K);
int m40llm_gemm_f32xf32_f32(M40llmCudaContext* ctx, const void* d_A_f32, const void* d_B_f32_colmajor_nt,
                            void* d_C_f32, int M, int N, int K);
/* cuda/kernels.cu:5244-5263 (kernel 5056-5066): Bt[k*N+n] = f32(B[n*K+k]) */
int m40llm_materialize_gguf_f16_to_f32_colmajor_nt(M40llmCudaContext* ctx, const void* d_B_f16,
                                                   void* d_B_f32_colmajor_nt, int N, int K);
/* cuda/kernels.cu:5068-5103: f16 x f16 [K,N] -> f16, f32 accumulate (synchronous) */
int m40llm_gemm_f16_storage_f32_compute(M40llmCudaContext* ctx, const void* d_A, const void* d_B, void* d_C, int M,
                                        int N, int K);

/* ------------------------------------------------------------------ KV cache */
/* cuda/kernels.cu:5387-5433 */
M40llmKVCache* m40llm_kvcache_create(M40llmCudaContext* ctx, uint32_t max_seq_len, uint32_t max_batch_size,
                                     uint32_t num_heads, uint32_t head_dim);
/* cuda/kernels.cu:5435-5543; exact_old_backing 0 = dense, 1 = q8 (unsupported here), 2 = fp16-K/q4-V */
M40llmKVCache* m40llm_kvcache_create_compressed(M40llmCudaContext* ctx, uint32_t max_seq_len, uint32_t max_batch_size,
                                                uint32_t num_heads, uint32_t head_dim, uint32_t recent_window,
                                                uint32_t block_size, uint32_t top_blocks, uint32_t representatives,
                                                uint32_t representative_policy, uint32_t exact_old_backing);
/* cuda/kernels.cu:7233-7256 */
void m40llm_kvcache_destroy(M40llmKVCache* kv);
/* cuda/kernels.cu:6308-6358 */
int m40llm_kvcache_reset(M40llmCudaContext* ctx, M40llmKVCache* kv);
/* cuda/kernels.cu:5793-5823 (f16 inputs, synchronous) */
int m40llm_kvcache_append_token(M40llmCudaContext* ctx, M40llmKVCache* kv, uint32_t seq_id, const void* k_dev,
                                const void* v_dev);
/* cuda/kernels.cu:5837-5907; sync form 5825-5835 */
int m40llm_kvcache_append_token_f32_async(M40llmCudaContext* ctx, M40llmKVCache* kv, uint32_t seq_id,
                                          const void* k_dev_f32, const void* v_dev_f32);
int m40llm_kvcache_append_token_f32(M40llmCudaContext* ctx, M40llmKVCache* kv, uint32_t seq_id, const void* k_dev_f32,
                                    const void* v_dev_f32);
/* cuda/kernels.cu:5976-6029: RoPE(K, past_len) fused with the f16 cast, appended at the current length */
int m40llm_kvcache_append_token_f32_rope_k_layout_async(M40llmCudaContext* ctx, M40llmKVCache* kv, uint32_t seq_id,
                                                        const void* k_dev_f32, const void* v_dev_f32,
                                                        uint32_t past_len, float freq_base, float freq_scale,
                                                        uint32_t rope_layout);
/* cuda/kernels.cu:5947-5974 */
int m40llm_kvcache_append_token_f32_rope_k(M40llmCudaContext* ctx, M40llmKVCache* kv, uint32_t seq_id,
                                           const void* k_dev_f32, const void* v_dev_f32, uint32_t past_len,
                                           float freq_base, float freq_scale);
int m40llm_kvcache_append_token_f32_rope_k_async(M40llmCudaContext* ctx, M40llmKVCache* kv, uint32_t seq_id,
                                                 const void* k_dev_f32, const void* v_dev_f32, uint32_t past_len,
                                                 float freq_base, float freq_scale);
/* cuda/kernels.cu:6045-6093: write at an explicit position; compressed caches route to the ring/evict path */
int m40llm_kvcache_append_token_f32_rope_k_at_layout_async(M40llmCudaContext* ctx, M40llmKVCache* kv, uint32_t seq_id,
                                                           const void* k_dev_f32, const void* v_dev_f32,
                                                           uint32_t position, uint32_t past_len, float freq_base,
                                                           float freq_scale, uint32_t rope_layout);
/* cuda/kernels.cu:6031-6043 */
int m40llm_kvcache_append_token_f32_rope_k_at_async(M40llmCudaContext* ctx, M40llmKVCache* kv, uint32_t seq_id,
                                                    const void* k_dev_f32, const void* v_dev_f32, uint32_t position,
                                                    uint32_t past_len, float freq_base, float freq_scale);
/* cuda/kernels.cu:6108-6250 (ring write, eviction to f16 old K + q4 old V); adjacent form 6095-6106 */
int m40llm_kvcache_append_token_f32_rope_k_compressed_at_layout_async(M40llmCudaContext* ctx, M40llmKVCache* kv,
                                                                      uint32_t seq_id, const void* k_dev_f32,
                                                                      const void* v_dev_f32, uint32_t position,
                                                                      float freq_base, float freq_scale,
                                                                      uint32_t rope_layout);
int m40llm_kvcache_append_token_f32_rope_k_compressed_at_async(M40llmCudaContext* ctx, M40llmKVCache* kv,
                                                               uint32_t seq_id, const void* k_dev_f32,
                                                               const void* v_dev_f32, uint32_t position,
                                                               float freq_base, float freq_scale);
/* cuda/kernels.cu:6265-6306: position read from device memory (graph replay); adjacent form 6252-6263 */
int m40llm_kvcache_append_token_f32_rope_k_position_dev_layout_async(M40llmCudaContext* ctx, M40llmKVCache* kv,
                                                                     uint32_t seq_id, const void* k_dev_f32,
                                                                     const void* v_dev_f32,
                                                                     const uint32_t* position_dev, float freq_base,
                                                                     float freq_scale, uint32_t rope_layout);
int m40llm_kvcache_append_token_f32_rope_k_position_dev_async(M40llmCudaContext* ctx, M40llmKVCache* kv,
                                                              uint32_t seq_id, const void* k_dev_f32,
                                                              const void* v_dev_f32, const uint32_t* position_dev,
                                                              float freq_base, float freq_scale);
/* cuda/kernels.cu:6360-6379: one token's K and V, [kv_heads][head_dim] f16 each, to host */
int m40llm_kvcache_debug_read_token(M40llmCudaContext* ctx, M40llmKVCache* kv, uint32_t seq_id, uint32_t token,
                                    void* out_k_f16, void* out_v_f16);
/* cuda/kernels.cu:6381-6447. The summary/representative outputs belong to the lossy modes this
 * library does not maintain: they are written as zeros (positions 0xffffffff). */
int m40llm_kvcache_debug_read_compressed_state(M40llmCudaContext* ctx, M40llmKVCache* kv, uint32_t seq_id,
                                               uint32_t* out_seq_len, uint32_t* out_block_counts,
                                               void* out_recent_k_f16, void* out_recent_v_f16,
                                               float* out_summary_k_acc, float* out_summary_v_acc,
                                               void* out_summary_k_f16, void* out_summary_v_f16, void* out_rep_k_f16,
                                               void* out_rep_v_f16, uint32_t* out_rep_positions);
/* cuda/kernels.cu:6449-6677: host-visible result of the block selection for q head 0 (default policy) */
int m40llm_kvcache_debug_select_old_blocks(M40llmCudaContext* ctx, const M40llmKVCache* kv, uint32_t seq_id,
                                           const void* d_q_f32, uint32_t q_heads, uint32_t seq_len,
                                           uint32_t recent_window, uint32_t block_size, uint32_t top_blocks,
                                           uint32_t* out_blocks_host, float* out_scores_host, uint32_t* out_start_host,
                                           uint32_t* out_end_host, uint32_t* out_count, uint32_t max_out,
                                           uint32_t* out_total_old_blocks);
/* cuda/kernels.cu:6679-7036 — telemetry of the experimental modes: M40LLM_ERR_UNSUPPORTED */
int m40llm_kvcache_debug_attention_telemetry(M40llmCudaContext* ctx, const M40llmKVCache* kv, uint32_t mode,
                                             uint32_t seq_id, const void* d_q_f32, uint32_t q_heads, uint32_t seq_len,
                                             uint32_t recent_window, uint32_t block_size, uint32_t top_blocks,
                                             uint32_t needle_block, M40llmAttentionTelemetry* out);
/* cuda/kernels.cu:7173-7231 (src/cuda.rs:462-471) — builds the compressed state of every sequence slot from a dense
 * cache that holds seq_len tokens per slot: the last min(seq_len, recent_window) tokens in the ring (slot t % R), the
 * older ones in the FP16-K / q4-V old region (the state token-by-token appends would have left), every sequence length
 * = seq_len. Return codes as the reference: -2 wrong cache kinds, -3 shapes differ, -4 seq_len beyond a cache;
 * M40LLM_ERR_UNSUPPORTED for a compressed cache without the FP16-K / q4-V backing. Synchronous, decode stream. */
int m40llm_kvcache_build_compressed_from_dense(M40llmCudaContext* ctx, M40llmKVCache* compressed,
                                               const M40llmKVCache* dense, uint32_t seq_len);
/* cuda/kernels.cu:4089-4122 — q8 KV backing: M40LLM_ERR_UNSUPPORTED */
int m40llm_kvcache_build_q8_old_from_dense(M40llmCudaContext* ctx, M40llmKVCache* kv, uint32_t seq_id,
                                           uint32_t seq_len, uint32_t recent_window);

/* ------------------------ decode attention (decode stream); q/out f32 [q_heads*head_dim] */
/* cuda/kernels.cu:3837-3861 (MHA, synchronous) */
int m40llm_attention_last_token_f32(M40llmCudaContext* ctx, const M40llmKVCache* kv, uint32_t seq_id,
                                    const void* d_q_f32, uint32_t seq_len, void* d_out_f32);
/* cuda/kernels.cu:3879-3961; sync form 3863-3877 */
int m40llm_attention_last_token_f32_gqa_async(M40llmCudaContext* ctx, const M40llmKVCache* kv, uint32_t seq_id,
                                              const void* d_q_f32, uint32_t q_heads, uint32_t seq_len,
                                              void* d_out_f32);
int m40llm_attention_last_token_f32_gqa(M40llmCudaContext* ctx, const M40llmKVCache* kv, uint32_t seq_id,
                                        const void* d_q_f32, uint32_t q_heads, uint32_t seq_len, void* d_out_f32);
/* cuda/kernels.cu:3963-3987: seq_len read from device memory (graph replay) */
int m40llm_attention_last_token_f32_gqa_seq_len_dev_async(M40llmCudaContext* ctx, const M40llmKVCache* kv,
                                                          uint32_t seq_id, const void* d_q_f32, uint32_t q_heads,
                                                          const uint32_t* d_seq_len, void* d_out_f32);
/* cuda/kernels.cu:4694-4832: batched variable-length decode; q/out packed [batch][q_heads][head_dim].
 * Extension over the reference: any head_dim the single-sequence path accepts and no 8192-token cap. */
int m40llm_attention_last_token_f32_gqa_batched(M40llmCudaContext* ctx, const M40llmKVCache* kv,
                                                const uint32_t* d_seq_ids, const uint32_t* d_seq_lens,
                                                uint32_t batch_size, const void* d_q_f32, uint32_t q_heads,
                                                void* d_out_f32);
int m40llm_attention_last_token_f32_gqa_batched_async(M40llmCudaContext* ctx, const M40llmKVCache* kv,
                                                      const uint32_t* d_seq_ids, const uint32_t* d_seq_lens,
                                                      uint32_t batch_size, const void* d_q_f32, uint32_t q_heads,
                                                      void* d_out_f32);
/* cuda/kernels.cu:4025-4070 (kernel 1825-1983): block selection over a dense FP16 cache */
int m40llm_attention_last_token_f32_gqa_block_select_exact_async(M40llmCudaContext* ctx, const M40llmKVCache* kv,
                                                                 uint32_t seq_id, const void* d_q_f32,
                                                                 uint32_t q_heads, uint32_t seq_len,
                                                                 uint32_t recent_window, uint32_t block_size,
                                                                 uint32_t top_blocks, void* d_out_f32);
/* cuda/kernels.cu:4504-4577 (kernel 2832-3096): FP16 old K + q4 old V + FP16 recent ring */
int m40llm_attention_last_token_f32_gqa_block_select_exact_fp16_k_q4_v_old_direct_async(
    M40llmCudaContext* ctx, const M40llmKVCache* kv, uint32_t seq_id, const void* d_q_f32, uint32_t q_heads,
    uint32_t seq_len, uint32_t recent_window, uint32_t block_size, uint32_t top_blocks, void* d_out_f32);

/* Modes outside the decode hot path. The symbols exist so the reference host links;
 * each returns M40LLM_ERR_UNSUPPORTED after the reference's own argument checks.
 * cuda/kernels.cu:3989-4023, 4124-4174, 4176-4249, 4251-4340, 4342-4426, 4428-4502, 4579-4658, 4660-4692 */
int m40llm_attention_last_token_f32_gqa_dense_recent_async(M40llmCudaContext* ctx, const M40llmKVCache* kv,
                                                           uint32_t seq_id, const void* d_q_f32, uint32_t q_heads,
                                                           uint32_t seq_len, uint32_t recent_window, void* d_out_f32);
int m40llm_attention_last_token_f32_gqa_block_select_exact_staged_async(
    M40llmCudaContext* ctx, const M40llmKVCache* kv, uint32_t seq_id, const void* d_q_f32, uint32_t q_heads,
    uint32_t seq_len, uint32_t recent_window, uint32_t block_size, uint32_t top_blocks, void* d_out_f32);
int m40llm_attention_last_token_f32_gqa_block_select_exact_staged_with_buffers_async(
    M40llmCudaContext* ctx, const M40llmKVCache* kv, uint32_t seq_id, const void* d_q_f32, uint32_t q_heads,
    uint32_t seq_len, uint32_t recent_window, uint32_t block_size, uint32_t top_blocks, void* staged_k_dev,
    void* staged_v_dev, void* staged_positions_dev, void* staged_counts_dev, uint32_t staged_capacity_tokens,
    void* d_out_f32);
int m40llm_attention_last_token_f32_gqa_block_select_exact_staged_q8_old_with_buffers_async(
    M40llmCudaContext* ctx, const M40llmKVCache* kv, uint32_t seq_id, const void* d_q_f32, uint32_t q_heads,
    uint32_t seq_len, uint32_t recent_window, uint32_t block_size, uint32_t top_blocks, void* staged_k_dev,
    void* staged_v_dev, void* staged_positions_dev, void* staged_counts_dev, uint32_t staged_capacity_tokens,
    void* d_out_f32);
int m40llm_attention_last_token_f32_gqa_block_select_exact_staged_fp16_k_q4_v_old_with_buffers_async(
    M40llmCudaContext* ctx, const M40llmKVCache* kv, uint32_t seq_id, const void* d_q_f32, uint32_t q_heads,
    uint32_t seq_len, uint32_t recent_window, uint32_t block_size, uint32_t top_blocks, void* staged_k_dev,
    void* staged_v_dev, void* staged_positions_dev, void* staged_counts_dev, uint32_t staged_capacity_tokens,
    void* d_out_f32);
int m40llm_attention_last_token_f32_gqa_block_select_exact_q8_old_direct_async(
    M40llmCudaContext* ctx, const M40llmKVCache* kv, uint32_t seq_id, const void* d_q_f32, uint32_t q_heads,
    uint32_t seq_len, uint32_t recent_window, uint32_t block_size, uint32_t top_blocks, void* d_out_f32);
int m40llm_attention_last_token_f32_gqa_block_summary_lossy_async(
    M40llmCudaContext* ctx, const M40llmKVCache* kv, uint32_t seq_id, const void* d_q_f32, uint32_t q_heads,
    uint32_t seq_len, uint32_t recent_window, uint32_t block_size, uint32_t top_blocks, void* d_out_f32);
int m40llm_attention_last_token_f32_gqa_compressed_recent_only_async(M40llmCudaContext* ctx, const M40llmKVCache* kv,
                                                                     uint32_t seq_id, const void* d_q_f32,
                                                                     uint32_t q_heads, uint32_t seq_len,
                                                                     void* d_out_f32);
/* cuda/kernels.cu:3749-3835, 4834-4977 (src/cuda.rs:619-668) — packed variable-length causal prefill attention over f32
 * Q [total_q][q_heads][hd], K / V [total_kv][kv_heads][hd]: sequence b owns q rows [q_offsets[b], +q_lens[b]) and kv rows
 * [kv_offsets[b], +kv_lens[b]); q row i attends kv rows 0 .. kv_len - q_len + i. head_dim 64 or 128 (-9 otherwise, and
 * for pointers that are not 16-byte aligned); the lengths are validated on the host as in the reference (-8 for a zero
 * length, q_len > kv_len or kv_len > 8192). Prefill stream; the plain form synchronises it. */
int m40llm_attention_prefill_f32_gqa_varlen(M40llmCudaContext* ctx, const void* d_q_f32, const void* d_k_f32,
                                            const void* d_v_f32, const uint32_t* d_q_offsets,
                                            const uint32_t* d_kv_offsets, const uint32_t* d_q_lens,
                                            const uint32_t* d_kv_lens, uint32_t batch_size, uint32_t q_heads,
                                            uint32_t kv_heads, uint32_t head_dim, void* d_out_f32);
int m40llm_attention_prefill_f32_gqa_varlen_async(M40llmCudaContext* ctx, const void* d_q_f32, const void* d_k_f32,
                                                  const void* d_v_f32, const uint32_t* d_q_offsets,
                                                  const uint32_t* d_kv_offsets, const uint32_t* d_q_lens,
                                                  const uint32_t* d_kv_lens, uint32_t batch_size, uint32_t q_heads,
                                                  uint32_t kv_heads, uint32_t head_dim, void* d_out_f32);
/* cuda/kernels.cu:7927-8025 — the reference's resident kernel spins on host flags without a
 * bound; it is not built. All four return M40LLM_ERR_UNSUPPORTED. */
int m40llm_start_persistent_decode(M40llmCudaContext* ctx);
int m40llm_stop_persistent_decode(M40llmCudaContext* ctx);
int m40llm_persistent_decode_submit_vec(M40llmCudaContext* ctx, const void* d_in_f32, void* d_out_f32, uint32_t n,
                                        float scale, float bias, uint32_t iterations, uint32_t* out_command_id);
int m40llm_persistent_decode_poll(M40llmCudaContext* ctx, uint32_t* out_status, uint32_t* out_command_id);

/* =====================================================================
 * Additive entry points (no counterpart in the reference; the reference host
 * needs new `extern` lines to use them). Same conventions: int rc, ctx first.
 * ===================================================================== */

/* GEMV/GEMM over GGUF-layout f16 weights without the synchronise of
 * m40llm_gemm_f32xf16_gguf_f32; enqueued on `stream_kind`. Replaces the
 * materialise-to-FP32 + cublasSgemm default of src/infer/gemm.rs:245-362. */
int m40llm_gemm_f32xf16_gguf_f32_async(M40llmCudaContext* ctx, const void* d_A_f32, const void* d_B_f16,
                                       void* d_C_f32, int M, int N, int K, uint32_t stream_kind);
/* GEMV/GEMM over GGUF-layout Q8_0 rows (K % 32 == 0): C[m][n] = sum_k A[m][k] * d[n][k/32] * q[n][k].
 * Composition of m40llm_q80_to_f32 (kernels.cu:856-867) and the GGUF GEMM (kernels.cu:5037-5052). */
int m40llm_gemm_f32xq80_gguf_f32_async(M40llmCudaContext* ctx, const void* d_A_f32, const void* d_B_q80,
                                       void* d_C_f32, int M, int N, int K, uint32_t stream_kind);
/* The SwiGLU FFN over Q8_0 weights in two launches: hid = silu(x.Wg) * (x.Wu);
 * out = residual + hid.Wd (residual may be NULL). x [rows,H], hid scratch [rows,F], out [rows,H].
 * Composition of src/infer/gemm.rs:91-163 and kernels.cu:880-891, 869-878. */
int m40llm_ffn_swiglu_q80_f32_async(M40llmCudaContext* ctx, const void* d_x_f32, const void* d_wg_q80,
                                    const void* d_wu_q80, const void* d_wd_q80, const void* d_residual_f32,
                                    void* d_hid_f32, void* d_out_f32, uint32_t rows, uint32_t hidden, uint32_t ffn,
                                    uint32_t stream_kind);
/* The same FFN over f16 GGUF weights (the reference's production layout, src/infer/mapping.rs:218-231). */
int m40llm_ffn_swiglu_f16_f32_async(M40llmCudaContext* ctx, const void* d_x_f32, const void* d_wg_f16,
                                    const void* d_wu_f16, const void* d_wd_f16, const void* d_residual_f32,
                                    void* d_hid_f32, void* d_out_f32, uint32_t rows, uint32_t hidden, uint32_t ffn,
                                    uint32_t stream_kind);
/* Fused attention prologue for `rows` decode rows (steps 1-5 of src/infer/forward.rs:307-421):
 * xn = rmsnorm(x, w); q,k,v = xn.Wq/Wk/Wv (+ optional f32 biases); q <- rope(q, pos);
 * cache[seq][pos] <- f16(rope(k, pos)), f16(v). Row r uses seq_ids[r] and positions[r] (device u32 arrays).
 * q_out f32 [rows][q_heads*head_dim]. Dense or compressed cache. Decode stream. */
int m40llm_qkv_rmsnorm_rope_append_async(M40llmCudaContext* ctx, M40llmKVCache* kv, const void* d_x_f32,
                                         const void* d_norm_w, uint32_t norm_w_dtype, float eps, const void* d_wq_f16,
                                         const void* d_wk_f16, const void* d_wv_f16, const void* d_bq_f32,
                                         const void* d_bk_f32, const void* d_bv_f32, const uint32_t* d_seq_ids,
                                         const uint32_t* d_positions, uint32_t rows, uint32_t hidden,
                                         uint32_t q_heads, float freq_base, float freq_scale, uint32_t rope_layout,
                                         void* d_q_out_f32);
/* Fused second half of the layer for `rows` decode rows (steps 9-13 of src/infer/forward.rs:470-667):
 * x1 = x + att.Wo; xn = rmsnorm(x1, ffn_norm_w); hid = silu(xn.Wg) * (xn.Wu); out = x1 + hid.Wd.
 * att [rows][q_dim], x/x1/out [rows][hidden], hid [rows][ffn] (x1 and hid are caller-provided work buffers that hold
 * the intermediate values afterwards). Wo f16 GGUF rows; Wg/Wu/Wd Q8_0 (ffn_q80 != 0) or f16. norm_w_dtype: 0 f16,
 * 1 f32. Decode stream. */
int m40llm_attn_out_ffn_async(M40llmCudaContext* ctx, const void* d_att_f32, const void* d_wo_f16, const void* d_x_f32,
                              const void* d_ffn_norm_w, uint32_t norm_w_dtype, float eps, const void* d_wg,
                              const void* d_wu, const void* d_wd, uint32_t ffn_q80, void* d_x1_f32, void* d_hid_f32,
                              void* d_out_f32, uint32_t rows, uint32_t hidden, uint32_t q_dim, uint32_t ffn);
/* Steps 1-6 of the layer in one call (src/infer/forward.rs:307-470 issues them as norm, three GEMMs, bias adds, RoPE,
 * append and attention): m40llm_qkv_rmsnorm_rope_append_async followed by
 * m40llm_attention_last_token_f32_gqa_batched_async over d_seq_lens, with the same arguments and the same results in
 * d_q_out_f32 (q after RoPE), the cache and d_att_out_f32. Dense caches only (a compressed cache returns
 * M40LLM_ERR_UNSUPPORTED after the prologue: its attention is per row). With one row, head_dim 64 or 128 and at most
 * 16 q heads per kv head the whole of RoPE, append, attention and split merge is ONE kernel after the projection; that
 * path requires d_seq_lens[r] == d_positions[r] + 1 (the new token is the last attended one) and reports a row that
 * breaks it through status bit 1 with a zero output row. Decode stream. */
int m40llm_qkv_rope_append_attention_async(M40llmCudaContext* ctx, M40llmKVCache* kv, const void* d_x_f32,
                                           const void* d_norm_w, uint32_t norm_w_dtype, float eps,
                                           const void* d_wq_f16, const void* d_wk_f16, const void* d_wv_f16,
                                           const void* d_bq_f32, const void* d_bk_f32, const void* d_bv_f32,
                                           const uint32_t* d_seq_ids, const uint32_t* d_positions,
                                           const uint32_t* d_seq_lens, uint32_t rows, uint32_t hidden, uint32_t q_heads,
                                           float freq_base, float freq_scale, uint32_t rope_layout, void* d_q_out_f32,
                                           void* d_att_out_f32);
/* Split-K attention for one long sequence sharded over ranks: attends tokens [tok_begin, tok_end) of a dense
 * cache and writes the unnormalised triple per q head: m [q_heads], l [q_heads], o [q_heads][head_dim]. */
int m40llm_attention_last_token_f32_gqa_partial_async(M40llmCudaContext* ctx, const M40llmKVCache* kv,
                                                      uint32_t seq_id, const void* d_q_f32, uint32_t q_heads,
                                                      uint32_t tok_begin, uint32_t tok_end, void* d_m_f32,
                                                      void* d_l_f32, void* d_o_f32);
/* Merge `parts` triples laid out [part][q_heads] / [part][q_heads][head_dim] into out [q_heads*head_dim]. */
int m40llm_attention_merge_partials_async(M40llmCudaContext* ctx, const void* d_m_f32, const void* d_l_f32,
                                          const void* d_o_f32, uint32_t parts, uint32_t q_heads, uint32_t head_dim,
                                          void* d_out_f32);
/* Compressed-cache split-K, phase 1: scores of this rank's old blocks [block_begin, block_end) for every q head,
 * written to d_scores_f32 [q_heads][block_end-block_begin]. */
int m40llm_kvcache_score_old_blocks_async(M40llmCudaContext* ctx, const M40llmKVCache* kv, uint32_t seq_id,
                                          const void* d_q_f32, uint32_t q_heads, uint32_t seq_len,
                                          uint32_t block_begin, uint32_t block_end, void* d_scores_f32);
/* Phase 2: attend a caller-chosen block list (d_blocks u32 [q_heads][64], 0xffffffff = empty; only blocks inside
 * [block_begin, block_end) are read) plus, when include_recent != 0, the recent ring; writes triples as above. */
int m40llm_attention_compressed_selected_partial_async(M40llmCudaContext* ctx, const M40llmKVCache* kv,
                                                       uint32_t seq_id, const void* d_q_f32, uint32_t q_heads,
                                                       uint32_t seq_len, const uint32_t* d_blocks,
                                                       uint32_t block_begin, uint32_t block_end,
                                                       uint32_t include_recent, void* d_m_f32, void* d_l_f32,
                                                       void* d_o_f32);
/* Split-K selection, device side. m40llm_topk_pairs_async ranks the n candidate scores of every q head
 * (d_scores_f32 [q_heads][score_stride], candidate i = block index_base + i; n <= 4096) and writes the best top_n <= 64
 * as (f32 score, u32 block) pairs, descending, ties to the lower block, NaN and scores <= -1e30 never chosen, unused
 * slots (-1e30, 0xffffffff): d_pairs_out [q_heads][64][2] 32-bit words. That array is one rank's message of the
 * all-gather. m40llm_topk_merge_pairs_async applies the same rule to the gathered candidates d_pairs
 * [parts][q_heads][64][2] and writes the global block list d_blocks_out [q_heads][64] (the form
 * m40llm_attention_compressed_selected_partial_async takes) and, when given, the scores d_scores_out_f32
 * [q_heads][64]. The rule is the single-GPU selection's (cuda/kernels.cu:2861-2930), so every rank derives the
 * identical list without a further exchange. Decode stream, no host synchronisation. */
int m40llm_topk_pairs_async(M40llmCudaContext* ctx, const void* d_scores_f32, uint32_t q_heads, uint32_t n,
                            uint32_t score_stride, uint32_t index_base, uint32_t top_n, void* d_pairs_out);
int m40llm_topk_merge_pairs_async(M40llmCudaContext* ctx, const void* d_pairs, uint32_t parts, uint32_t q_heads,
                                  uint32_t top_n, uint32_t* d_blocks_out, void* d_scores_out_f32);
/* Merge of all-gathered triples that arrive as ONE message per rank: d_triples [parts][q_heads * (2 + head_dim)] with
 * each message laid out m [q_heads] | l [q_heads] | o [q_heads][head_dim]; out [q_heads * head_dim]. */
int m40llm_attention_merge_gathered_async(M40llmCudaContext* ctx, const void* d_triples_f32, uint32_t parts,
                                          uint32_t q_heads, uint32_t head_dim, void* d_out_f32);
/* Device-side result of the last block selection run on `ctx`: u32 [q_heads][64] block indices in
 * descending score order, 0xffffffff padded. Copies to host after synchronising the decode stream. */
int m40llm_kvcache_debug_last_selected_blocks(M40llmCudaContext* ctx, uint32_t q_heads, uint32_t* out_blocks_host,
                                              float* out_scores_host);
/* Harness loader: writes tokens [tok_begin, tok_begin+count) of sequence `seq_id` from host arrays in the
 * reference's logical layout [token][kv_head][head_dim] f16 (K already rotated). For a compressed cache the
 * tokens are placed exactly where token-by-token appends up to `final_seq_len` would have left them (old K,
 * q4 V quantised on device from the f16 V, ring slot t % R). Sets the sequence length to final_seq_len. */
int m40llm_kvcache_debug_write_range(M40llmCudaContext* ctx, M40llmKVCache* kv, uint32_t seq_id, uint32_t tok_begin,
                                     uint32_t count, const void* k_f16_host, const void* v_f16_host,
                                     uint32_t final_seq_len);
/* Reads back the compressed old region of one token: old K f16 [kv_heads][hd], q4 bytes [kv_heads][hd/2],
 * scales f32 [kv_heads] (host pointers). */
int m40llm_kvcache_debug_read_old_token(M40llmCudaContext* ctx, M40llmKVCache* kv, uint32_t seq_id, uint32_t token,
                                        void* out_k_f16, void* out_q4_v, float* out_scale);
/* Device error word of the context: bit 0 = a batched-attention row carried an out-of-range
 * sequence id or length and was skipped (no cache data is read for it and its output row is written as zeros,
 * whatever the number of splits). Reading clears it. */
int m40llm_context_take_device_status(M40llmCudaContext* ctx, uint32_t* out_status);
/* Stream-ordered host <-> device copies on one of the context's streams (the reference only has the synchronous
 * m40llm_memcpy_h2d / _d2h, cuda/kernels.cu). The host buffer must stay valid until the stream has passed the copy;
 * with pinned memory the call returns at once. */
int m40llm_memcpy_h2d_async(M40llmCudaContext* ctx, void* dst_device, const void* src_host, size_t bytes,
                            uint32_t stream_kind);
int m40llm_memcpy_d2h_async(M40llmCudaContext* ctx, void* dst_host, const void* src_device, size_t bytes,
                            uint32_t stream_kind);
/* Token embedding gather on the device: out[r][:] = f32(table[token_ids[r]][:]), table f16 [vocab][hidden]
 * (the reference gathers rows on the host and uploads them, src/infer/embeddings.rs:80-140). An id >= vocab yields a
 * zero row and raises bit 8 of the device status word. Decode stream. */
int m40llm_embed_tokens_f16_async(M40llmCudaContext* ctx, const void* d_table_f16, const uint32_t* d_token_ids,
                                  void* d_out_f32, uint32_t rows, uint32_t hidden, uint32_t vocab);
/* Logits head (src/infer/logits.rs:57-116): logits[r][v] = rmsnorm(hidden[r], norm_w) . lm_head[v], lm_head f16 GGUF
 * rows [vocab][hidden]; d_norm_w may be NULL (no output norm), norm_w_dtype 0 f16 / 1 f32. Decode stream; the logits
 * stay on the device. */
int m40llm_logits_head_f32_async(M40llmCudaContext* ctx, const void* d_hidden_f32, const void* d_norm_w,
                                 uint32_t norm_w_dtype, float eps, const void* d_lm_head_f16, void* d_logits_f32,
                                 uint32_t rows, uint32_t hidden, uint32_t vocab);
/* Greedy choice per row (Sampler::sample_greedy, src/sampling.rs:95-108): index of the first largest value under
 * strict '>' starting from -inf, so NaN is never chosen and a row without any value above -inf yields 0. */
int m40llm_argmax_f32_async(M40llmCudaContext* ctx, const void* d_values_f32, uint32_t rows, uint32_t n,
                            uint32_t* d_out_index);
/* positions[r] += 1 and lens[r] += 1 (either pointer may be NULL): lets a captured token step be replayed back to
 * back (the reference re-uploads these scalars per token, src/decode_session.rs:856-881). */
int m40llm_advance_positions_async(M40llmCudaContext* ctx, uint32_t* d_positions, uint32_t* d_lens, uint32_t rows);
/* No counterpart in the reference. Same contract as m40llm_attention_last_token_f32_gqa_async (dense cache, one
 * sequence, decode stream), but it never allocates or frees device or host memory: the per-split partials live in a
 * fixed 4 MiB device array that belongs to the loaded library. For callers that cannot take an allocating call (all
 * HBM already given to a KV pool; code that must not enter the allocator or its implicit device synchronisation).
 * The first call on each device looks up the array's address (cudaGetSymbolAddress) and should come before any
 * stream capture; the first call per head shape on a device also raises that kernel's shared-memory limit
 * (cudaFuncSetAttribute), which allocates nothing either. Returns M40LLM_ERR_LIMIT when
 * q_heads * splits * (2 + head_dim) floats exceed 2^20; M40LLM_ERR_UNSUPPORTED for head_dim other than 64/128, more
 * than 16 q heads per kv head, or a d_q_f32 that is not 8-byte aligned; M40LLM_ERR_SYMBOL when the array's address
 * cannot be looked up (a CUDA runtime failure, printed to stderr). All calls on a device share the array: calls
 * that overlap in time (other streams, other contexts) race and must be serialised. */
int m40llm_attention_last_token_f32_gqa_static_async(M40llmCudaContext* ctx, const M40llmKVCache* kv,
                                                     uint32_t seq_id, const void* d_q_f32, uint32_t q_heads,
                                                     uint32_t seq_len, void* d_out_f32);
/* Number of kernels this library has launched on `ctx` since creation (launch accounting for benchmarks). */
int m40llm_context_launch_count(M40llmCudaContext* ctx, uint64_t* out_count);
/* How many times a scratch arena of `ctx` has grown since creation. Growth happens only in eager (uncaptured)
 * calls; an arena that was outgrown stays allocated until the context is destroyed, so a CUDA graph captured
 * earlier keeps working on the memory it was captured with. A harness can watch this counter to see that a call
 * allocated. */
int m40llm_context_scratch_generation(M40llmCudaContext* ctx, uint64_t* out_generation);
/* The raw CUDA stream handle of a stream kind, for harnesses that time with their own events. */
int m40llm_context_stream_handle(M40llmCudaContext* ctx, uint32_t stream_kind, void** out_stream);

#ifdef __cplusplus
}
#endif
#endif /* M40LLM_NATIVE_H */
