// Context, streams, events, graphs and raw memory entry points of the C ABI.
// These are thin CUDA-runtime wrappers; their argument checks and return codes follow
// cuda/kernels.cu:302-680, 1245-1292, 8027-8042 of the reference.
#include <math.h>
#include <stdlib.h>
#include <string.h>

#include "common.cuh"

void* m40_ensure_scratch(M40llmCudaContext* ctx, uint32_t kind, size_t bytes, uint32_t level) {
    if (!ctx || kind > 1 || level > 1) return nullptr;
    if (ctx->scratch[kind][level] && ctx->scratch_bytes[kind][level] >= bytes) return ctx->scratch[kind][level];
    cudaStream_t s = m40_stream(ctx, kind);
    cudaStreamCaptureStatus cap = cudaStreamCaptureStatusNone;
    if (cudaStreamIsCapturing(s, &cap) != cudaSuccess || cap != cudaStreamCaptureStatusNone) return nullptr;
    // Grow at least geometrically so that the arenas retired below add up to less than the live one.
    size_t want = bytes < (size_t)(8u << 20) ? (size_t)(8u << 20) : bytes;
    if (want < 2 * ctx->scratch_bytes[kind][level]) want = 2 * ctx->scratch_bytes[kind][level];
    want = (want + ((size_t)1 << 20) - 1) & ~(((size_t)1 << 20) - 1);
    void* p = nullptr;
    if (cudaMalloc(&p, want) != cudaSuccess) {
        cudaGetLastError();
        return nullptr;
    }
    if (ctx->scratch[kind][level]) {
        // A CUDA graph captured earlier has the old arena's addresses baked into its kernel arguments and may be
        // replayed at any later time, so the old arena is retired, not freed: it stays valid (and private to
        // those graphs, which only ever use it consistently) until the context is destroyed.
        M40RetiredArena* r = (M40RetiredArena*)malloc(sizeof(M40RetiredArena));
        if (!r) {
            cudaFree(p);
            return nullptr;
        }
        r->ptr = ctx->scratch[kind][level];
        r->next = ctx->retired;
        ctx->retired = r;
    }
    ctx->scratch[kind][level] = p;
    ctx->scratch_bytes[kind][level] = want;
    ctx->scratch_generation++;
    return p;
}

const float* m40_rope_inv_freq(M40llmCudaContext* ctx, float freq_base, uint32_t head_dim) {
    if (!ctx || head_dim < 2 || head_dim > 512) return nullptr;
    for (uint32_t i = 0; i < ctx->rope_tables; ++i)
        if (ctx->rope_table_base[i] == freq_base && ctx->rope_table_hd[i] == head_dim) return ctx->d_rope_inv_freq[i];
    if (ctx->rope_tables >= 4) return nullptr;
    cudaStreamCaptureStatus cap = cudaStreamCaptureStatusNone;
    if (cudaStreamIsCapturing(ctx->decode_stream, &cap) != cudaSuccess || cap != cudaStreamCaptureStatusNone) return nullptr;
    float host[256];
    const uint32_t half = head_dim / 2u;
    for (uint32_t i = 0; i < half; ++i) {
        const float e = -2.0f * static_cast<float>(i) / static_cast<float>(head_dim);
        host[i] = static_cast<float>(pow(static_cast<double>(freq_base), static_cast<double>(e)));
    }
    float* d = nullptr;
    if (cudaMalloc(&d, half * sizeof(float)) != cudaSuccess) {
        cudaGetLastError();
        return nullptr;
    }
    if (cudaMemcpy(d, host, half * sizeof(float), cudaMemcpyHostToDevice) != cudaSuccess ||
        cudaStreamSynchronize(cudaStreamLegacy) != cudaSuccess) {
        cudaGetLastError();
        cudaFree(d);
        return nullptr;
    }
    const uint32_t slot = ctx->rope_tables++;
    ctx->d_rope_inv_freq[slot] = d;
    ctx->rope_table_base[slot] = freq_base;
    ctx->rope_table_hd[slot] = head_dim;
    return d;
}

extern "C" {

M40llmCudaContext* m40llm_create_context(int device_id) {
    int selected = device_id;
    if (device_id < 0) {
        // The reference auto-selects its target part (sm_52). Here the target is sm_100.
        selected = 0;
        int count = 0;
        if (cudaGetDeviceCount(&count) == cudaSuccess) {
            for (int i = 0; i < count; ++i) {
                int major = 0;
                if (cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, i) == cudaSuccess &&
                    major == 10) {
                    selected = i;
                    break;
                }
            }
        }
    }
    if (cudaSetDevice(selected) != cudaSuccess) {
        cudaGetLastError();
        return nullptr;
    }
    M40llmCudaContext* ctx = (M40llmCudaContext*)calloc(1, sizeof(M40llmCudaContext));
    if (!ctx) return nullptr;
    ctx->device_id = selected;
    if (cudaDeviceGetAttribute(&ctx->sm_count, cudaDevAttrMultiProcessorCount, selected) != cudaSuccess)
        ctx->sm_count = 148;
    int least = 0, greatest = 0;
    if (cudaDeviceGetStreamPriorityRange(&least, &greatest) == cudaSuccess) {
        ctx->prefill_priority = least;
        ctx->decode_priority = greatest;
    }
    bool ok = cudaStreamCreateWithPriority(&ctx->prefill_stream, cudaStreamNonBlocking, ctx->prefill_priority) ==
              cudaSuccess;
    ok = ok && cudaStreamCreateWithPriority(&ctx->decode_stream, cudaStreamNonBlocking, ctx->decode_priority) ==
                   cudaSuccess;
    ok = ok && cudaEventCreateWithFlags(&ctx->prefill_waits_decode_event, cudaEventDisableTiming) == cudaSuccess;
    ok = ok && cudaEventCreateWithFlags(&ctx->decode_waits_prefill_event, cudaEventDisableTiming) == cudaSuccess;
    ok = ok && cudaMalloc(&ctx->d_status, sizeof(uint32_t)) == cudaSuccess;
    ok = ok && cudaMemset(ctx->d_status, 0, sizeof(uint32_t)) == cudaSuccess;
    ctx->selected_capacity_heads = 256;
    ok = ok && cudaMalloc(&ctx->d_selected_blocks, (size_t)ctx->selected_capacity_heads * 64 * sizeof(uint32_t)) ==
                   cudaSuccess;
    ok = ok && cudaMalloc(&ctx->d_selected_scores, (size_t)ctx->selected_capacity_heads * 64 * sizeof(float)) ==
                   cudaSuccess;
    if (ok) {
        cudaMemset(ctx->d_selected_blocks, 0xff, (size_t)ctx->selected_capacity_heads * 64 * sizeof(uint32_t));
        cudaMemset(ctx->d_selected_scores, 0, (size_t)ctx->selected_capacity_heads * 64 * sizeof(float));
        ok = m40_ensure_scratch(ctx, 0, (size_t)32 << 20) != nullptr && m40_ensure_scratch(ctx, 1, (size_t)32 << 20) != nullptr;
        // the memsets above ran on the legacy stream, which the non-blocking streams do not order against
        ok = ok && cudaStreamSynchronize(cudaStreamLegacy) == cudaSuccess;
    }
    if (!ok) {
        cudaGetLastError();
        m40llm_destroy_context(ctx);
        return nullptr;
    }
    return ctx;
}

void m40llm_destroy_context(M40llmCudaContext* ctx) {
    if (!ctx) return;
    cudaSetDevice(ctx->device_id);
    if (ctx->prefill_stream) cudaStreamSynchronize(ctx->prefill_stream);
    if (ctx->decode_stream) cudaStreamSynchronize(ctx->decode_stream);
    for (int k = 0; k < 2; ++k)
        for (int l = 0; l < 2; ++l)
            if (ctx->scratch[k][l]) cudaFree(ctx->scratch[k][l]);
    for (uint32_t i = 0; i < ctx->rope_tables; ++i) cudaFree(ctx->d_rope_inv_freq[i]);
    while (ctx->retired) {
        M40RetiredArena* r = ctx->retired;
        ctx->retired = r->next;
        cudaFree(r->ptr);
        free(r);
    }
    if (ctx->d_status) cudaFree(ctx->d_status);
    if (ctx->d_selected_blocks) cudaFree(ctx->d_selected_blocks);
    if (ctx->d_selected_scores) cudaFree(ctx->d_selected_scores);
    if (ctx->prefill_waits_decode_event) cudaEventDestroy(ctx->prefill_waits_decode_event);
    if (ctx->decode_waits_prefill_event) cudaEventDestroy(ctx->decode_waits_prefill_event);
    if (ctx->prefill_stream) cudaStreamDestroy(ctx->prefill_stream);
    if (ctx->decode_stream) cudaStreamDestroy(ctx->decode_stream);
    cudaGetLastError();
    free(ctx);
}

int m40llm_current_device_props(char* name_buf, size_t buf_len, int* major, int* minor, int* device_id) {
    if (!name_buf || buf_len == 0 || !major || !minor || !device_id) return -1;
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess) return -2;
    cudaDeviceProp prop;
    if (cudaGetDeviceProperties(&prop, dev) != cudaSuccess) return -3;
    size_t n = strnlen(prop.name, sizeof(prop.name));
    if (buf_len <= n) n = buf_len - 1;
    memcpy(name_buf, prop.name, n);
    name_buf[n] = '\0';
    *major = prop.major;
    *minor = prop.minor;
    *device_id = dev;
    return 0;
}

int m40llm_device_malloc(M40llmCudaContext* ctx, size_t bytes, void** out_ptr) {
    if (!ctx || !out_ptr) return -1;
    if (m40_ensure_device(ctx) != 0) return -2;
    void* d = nullptr;
    if (cudaMalloc(&d, bytes) != cudaSuccess) {
        cudaGetLastError();
        return -3;
    }
    *out_ptr = d;
    return 0;
}

int m40llm_device_free(M40llmCudaContext* ctx, void* ptr) {
    if (!ctx) return -1;
    if (!ptr) return 0;
    if (m40_ensure_device(ctx) != 0) return -3;
    return cudaFree(ptr) == cudaSuccess ? 0 : -2;
}

int m40llm_memcpy_h2d(M40llmCudaContext* ctx, void* dst_device, const void* src_host, size_t bytes) {
    if (!ctx || !dst_device || !src_host) return -1;
    if (m40_ensure_device(ctx) != 0) return -3;
    if (cudaMemcpy(dst_device, src_host, bytes, cudaMemcpyHostToDevice) != cudaSuccess) return -2;
    // A copy from pageable memory returns once the data is staged, possibly before the DMA lands. The
    // context's streams are non-blocking (they do not order against the legacy stream the copy ran on),
    // so wait here: a kernel enqueued right after this call must see the bytes.
    return cudaStreamSynchronize(cudaStreamLegacy) == cudaSuccess ? 0 : -2;
}

int m40llm_memcpy_d2h(M40llmCudaContext* ctx, void* dst_host, const void* src_device, size_t bytes) {
    if (!ctx || !dst_host || !src_device) return -1;
    if (m40_ensure_device(ctx) != 0) return -3;
    return cudaMemcpy(dst_host, src_device, bytes, cudaMemcpyDeviceToHost) == cudaSuccess ? 0 : -2;
}

int m40llm_memcpy_d2d_async(M40llmCudaContext* ctx, void* dst_device, const void* src_device, size_t bytes,
                            uint32_t stream_kind) {
    if (!ctx || !dst_device || !src_device) return -1;
    if (m40_ensure_device(ctx) != 0) return -3;
    cudaStream_t s = m40_stream(ctx, stream_kind);
    if (!s) return -4;
    return cudaMemcpyAsync(dst_device, src_device, bytes, cudaMemcpyDeviceToDevice, s) == cudaSuccess ? 0 : -2;
}

int m40llm_memcpy_h2d_async(M40llmCudaContext* ctx, void* dst_device, const void* src_host, size_t bytes,
                            uint32_t stream_kind) {
    if (!ctx || !dst_device || !src_host) return -1;
    if (m40_ensure_device(ctx) != 0) return -3;
    cudaStream_t s = m40_stream(ctx, stream_kind);
    if (!s) return -4;
    return cudaMemcpyAsync(dst_device, src_host, bytes, cudaMemcpyHostToDevice, s) == cudaSuccess ? 0 : -2;
}

int m40llm_memcpy_d2h_async(M40llmCudaContext* ctx, void* dst_host, const void* src_device, size_t bytes,
                            uint32_t stream_kind) {
    if (!ctx || !dst_host || !src_device) return -1;
    if (m40_ensure_device(ctx) != 0) return -3;
    cudaStream_t s = m40_stream(ctx, stream_kind);
    if (!s) return -4;
    return cudaMemcpyAsync(dst_host, src_device, bytes, cudaMemcpyDeviceToHost, s) == cudaSuccess ? 0 : -2;
}

int m40llm_validate_device_ptr(const void* ptr) {
    if (!ptr) return -1;
    cudaPointerAttributes attr;
    if (cudaPointerGetAttributes(&attr, ptr) != cudaSuccess) {
        cudaGetLastError();
        return -2;
    }
    return attr.type == cudaMemoryTypeDevice ? 0 : -3;
}

int m40llm_upload_weights(M40llmCudaContext* ctx, const void* host_ptr, size_t num_bytes, void** out_device_ptr) {
    if (!ctx || !host_ptr || !out_device_ptr) return -1;
    if (m40_ensure_device(ctx) != 0) return -2;
    void* d = nullptr;
    if (cudaMalloc(&d, num_bytes) != cudaSuccess) {
        cudaGetLastError();
        return -2;
    }
    if (cudaMemcpy(d, host_ptr, num_bytes, cudaMemcpyHostToDevice) != cudaSuccess ||
        cudaStreamSynchronize(cudaStreamLegacy) != cudaSuccess) {
        cudaGetLastError();
        cudaFree(d);
        return -3;
    }
    *out_device_ptr = d;
    return 0;
}

int m40llm_stream_synchronize(M40llmCudaContext* ctx, uint32_t stream_kind) {
    if (!ctx) return -1;
    if (m40_ensure_device(ctx) != 0) return -2;
    cudaStream_t s = m40_stream(ctx, stream_kind);
    if (!s) return -3;
    return cudaStreamSynchronize(s) == cudaSuccess ? 0 : -4;
}

int m40llm_stream_wait_for_stream(M40llmCudaContext* ctx, uint32_t waiting_stream_kind, uint32_t signal_stream_kind) {
    if (!ctx) return -1;
    if (m40_ensure_device(ctx) != 0) return -2;
    cudaStream_t waiting = m40_stream(ctx, waiting_stream_kind);
    cudaStream_t signal = m40_stream(ctx, signal_stream_kind);
    if (!waiting || !signal) return -3;
    if (waiting_stream_kind == signal_stream_kind) return 0;
    cudaEvent_t ev = waiting_stream_kind == 0 ? ctx->prefill_waits_decode_event : ctx->decode_waits_prefill_event;
    if (!ev) return -4;
    if (cudaEventRecord(ev, signal) != cudaSuccess) return -5;
    if (cudaStreamWaitEvent(waiting, ev, 0) != cudaSuccess) return -6;
    return 0;
}

int m40llm_cuda_graph_begin_capture(M40llmCudaContext* ctx, uint32_t stream_kind) {
    if (!ctx) return -1;
    if (m40_ensure_device(ctx) != 0) return -2;
    cudaStream_t s = m40_stream(ctx, stream_kind);
    if (!s) return -3;
    return cudaStreamBeginCapture(s, cudaStreamCaptureModeRelaxed) == cudaSuccess ? 0 : -4;
}

int m40llm_cuda_graph_end_capture(M40llmCudaContext* ctx, uint32_t stream_kind, M40llmCudaGraphExec** out_graph) {
    if (!ctx || !out_graph) return -1;
    *out_graph = nullptr;
    if (m40_ensure_device(ctx) != 0) return -2;
    cudaStream_t s = m40_stream(ctx, stream_kind);
    if (!s) return -3;
    cudaGraph_t graph = nullptr;
    if (cudaStreamEndCapture(s, &graph) != cudaSuccess) {
        cudaGetLastError();
        return -4;
    }
    if (!graph) return -5;
    cudaGraphExec_t exec = nullptr;
    if (cudaGraphInstantiate(&exec, graph, 0) != cudaSuccess) {
        cudaGetLastError();
        cudaGraphDestroy(graph);
        return -6;
    }
    M40llmCudaGraphExec* w = (M40llmCudaGraphExec*)calloc(1, sizeof(M40llmCudaGraphExec));
    if (!w) {
        cudaGraphExecDestroy(exec);
        cudaGraphDestroy(graph);
        return -6;
    }
    w->graph = graph;
    w->exec = exec;
    *out_graph = w;
    return 0;
}

int m40llm_cuda_graph_cancel_capture(M40llmCudaContext* ctx, uint32_t stream_kind) {
    if (!ctx) return -1;
    if (m40_ensure_device(ctx) != 0) return -2;
    cudaStream_t s = m40_stream(ctx, stream_kind);
    if (!s) return -3;
    cudaGraph_t graph = nullptr;
    cudaError_t err = cudaStreamEndCapture(s, &graph);
    if (graph) cudaGraphDestroy(graph);
    if (err != cudaSuccess) cudaGetLastError();
    return err == cudaSuccess ? 0 : -4;
}

int m40llm_cuda_graph_launch(M40llmCudaContext* ctx, M40llmCudaGraphExec* graph, uint32_t stream_kind) {
    if (!ctx || !graph || !graph->exec) return -1;
    if (m40_ensure_device(ctx) != 0) return -2;
    cudaStream_t s = m40_stream(ctx, stream_kind);
    if (!s) return -3;
    return cudaGraphLaunch(graph->exec, s) == cudaSuccess ? 0 : -4;
}

int m40llm_cuda_graph_launch_timed_sync(M40llmCudaContext* ctx, M40llmCudaGraphExec* graph, uint32_t stream_kind,
                                        float* elapsed_ms) {
    if (!ctx || !graph || !graph->exec || !elapsed_ms) return -1;
    *elapsed_ms = 0.0f;
    if (m40_ensure_device(ctx) != 0) return -2;
    cudaStream_t s = m40_stream(ctx, stream_kind);
    if (!s) return -3;
    cudaEvent_t start = nullptr, stop = nullptr;
    if (cudaEventCreate(&start) != cudaSuccess) return -4;
    if (cudaEventCreate(&stop) != cudaSuccess) {
        cudaEventDestroy(start);
        return -5;
    }
    int rc = 0;
    if (cudaEventRecord(start, s) != cudaSuccess) rc = -6;
    else if (cudaGraphLaunch(graph->exec, s) != cudaSuccess) rc = -7;
    else if (cudaEventRecord(stop, s) != cudaSuccess) rc = -8;
    else if (cudaEventSynchronize(stop) != cudaSuccess) rc = -9;
    else if (cudaEventElapsedTime(elapsed_ms, start, stop) != cudaSuccess) rc = -10;
    cudaEventDestroy(stop);
    cudaEventDestroy(start);
    return rc;
}

void m40llm_cuda_graph_destroy(M40llmCudaGraphExec* graph) {
    if (!graph) return;
    if (graph->exec) cudaGraphExecDestroy(graph->exec);
    if (graph->graph) cudaGraphDestroy(graph->graph);
    free(graph);
}

int m40llm_cuda_event_create(M40llmCudaContext* ctx, M40llmCudaEvent** out_event) {
    if (!ctx || !out_event) return -1;
    *out_event = nullptr;
    if (m40_ensure_device(ctx) != 0) return -2;
    M40llmCudaEvent* w = (M40llmCudaEvent*)calloc(1, sizeof(M40llmCudaEvent));
    if (!w) return -3;
    if (cudaEventCreate(&w->event) != cudaSuccess) {
        free(w);
        return -3;
    }
    *out_event = w;
    return 0;
}

int m40llm_cuda_event_record(M40llmCudaContext* ctx, M40llmCudaEvent* event, uint32_t stream_kind) {
    if (!ctx || !event || !event->event) return -1;
    if (m40_ensure_device(ctx) != 0) return -2;
    cudaStream_t s = m40_stream(ctx, stream_kind);
    if (!s) return -3;
    return cudaEventRecord(event->event, s) == cudaSuccess ? 0 : -4;
}

int m40llm_stream_wait_event(M40llmCudaContext* ctx, uint32_t waiting_stream_kind, M40llmCudaEvent* event) {
    if (!ctx || !event || !event->event) return -1;
    if (m40_ensure_device(ctx) != 0) return -2;
    cudaStream_t s = m40_stream(ctx, waiting_stream_kind);
    if (!s) return -3;
    return cudaStreamWaitEvent(s, event->event, 0) == cudaSuccess ? 0 : -4;
}

int m40llm_cuda_event_synchronize(M40llmCudaContext* ctx, M40llmCudaEvent* event) {
    if (!ctx || !event || !event->event) return -1;
    if (m40_ensure_device(ctx) != 0) return -2;
    return cudaEventSynchronize(event->event) == cudaSuccess ? 0 : -3;
}

int m40llm_cuda_event_elapsed_sync(M40llmCudaContext* ctx, M40llmCudaEvent* start, M40llmCudaEvent* stop,
                                   float* elapsed_ms) {
    if (!ctx || !start || !stop || !start->event || !stop->event || !elapsed_ms) return -1;
    *elapsed_ms = 0.0f;
    if (m40_ensure_device(ctx) != 0) return -2;
    if (cudaEventSynchronize(stop->event) != cudaSuccess) return -3;
    return cudaEventElapsedTime(elapsed_ms, start->event, stop->event) == cudaSuccess ? 0 : -4;
}

void m40llm_cuda_event_destroy(M40llmCudaEvent* event) {
    if (!event) return;
    if (event->event) cudaEventDestroy(event->event);
    free(event);
}

int m40llm_context_take_device_status(M40llmCudaContext* ctx, uint32_t* out_status) {
    if (!ctx || !out_status) return -1;
    if (m40_ensure_device(ctx) != 0) return -2;
    if (cudaStreamSynchronize(ctx->decode_stream) != cudaSuccess) return -3;
    if (cudaMemcpy(out_status, ctx->d_status, sizeof(uint32_t), cudaMemcpyDeviceToHost) != cudaSuccess) return -4;
    if (*out_status != 0) {
        cudaMemset(ctx->d_status, 0, sizeof(uint32_t));
        cudaStreamSynchronize(cudaStreamLegacy);
    }
    return 0;
}

int m40llm_context_launch_count(M40llmCudaContext* ctx, uint64_t* out_count) {
    if (!ctx || !out_count) return -1;
    *out_count = (uint64_t)ctx->launches;
    return 0;
}

int m40llm_context_scratch_generation(M40llmCudaContext* ctx, uint64_t* out_generation) {
    if (!ctx || !out_generation) return -1;
    *out_generation = (uint64_t)ctx->scratch_generation;
    return 0;
}

int m40llm_context_stream_handle(M40llmCudaContext* ctx, uint32_t stream_kind, void** out_stream) {
    if (!ctx || !out_stream) return -1;
    cudaStream_t s = m40_stream(ctx, stream_kind);
    if (!s) return -3;
    *out_stream = (void*)s;
    return 0;
}

// ---- modes that are not part of the decode hot path: argument checks, then "unsupported" ----
int m40llm_start_persistent_decode(M40llmCudaContext* ctx) { return ctx ? M40LLM_ERR_UNSUPPORTED : -1; }
int m40llm_stop_persistent_decode(M40llmCudaContext* ctx) { return ctx ? M40LLM_ERR_UNSUPPORTED : -1; }
int m40llm_persistent_decode_submit_vec(M40llmCudaContext* ctx, const void* d_in_f32, void* d_out_f32, uint32_t n,
                                        float scale, float bias, uint32_t iterations, uint32_t* out_command_id) {
    (void)n; (void)scale; (void)bias; (void)iterations;
    if (!ctx || !d_in_f32 || !d_out_f32 || !out_command_id) return -1;
    return M40LLM_ERR_UNSUPPORTED;
}
int m40llm_persistent_decode_poll(M40llmCudaContext* ctx, uint32_t* out_status, uint32_t* out_command_id) {
    if (!ctx || !out_status || !out_command_id) return -1;
    return M40LLM_ERR_UNSUPPORTED;
}

}  // extern "C"

bool m40_pdl_enabled() {
    static int v = -1;
    if (v < 0) {
        const char* e = getenv("M40LLM_PDL");
        v = (e && e[0] == '0') ? 0 : 1;
    }
    return v != 0;
}
