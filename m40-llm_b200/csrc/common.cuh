// Internal definitions shared by the translation units of libm40llm_native.so.
// Nothing in this header is part of the C ABI (see include/m40llm_native.h).
#pragma once

#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdio.h>

#include "../../include/m40llm_native.h"

// ----------------------------------------------------------------------------
// Context: one device, two streams (0 = prefill, 1 = decode), two cross-stream
// events, a growable scratch arena and a device status word.
// Mirrors the handle of cuda/kernels.cu:25-37 in the reference.
// ----------------------------------------------------------------------------
struct M40RetiredArena {
    void* ptr;
    M40RetiredArena* next;
};

struct M40llmCudaContext {
    int device_id;
    int sm_count;
    cudaStream_t prefill_stream;
    cudaStream_t decode_stream;
    cudaEvent_t prefill_waits_decode_event;
    cudaEvent_t decode_waits_prefill_event;
    int prefill_priority;
    int decode_priority;
    // Scratch arenas, indexed [stream kind][level]. One set per stream kind so work on the two
    // streams never shares scratch; level 0 belongs to leaf operations (GEMM partials and
    // activation copies, attention partials), level 1 to composite operations that call leaf
    // operations while their own temporaries are live (the fused attention prologue).
    // Grown (never shrunk) outside of stream capture by m40_ensure_scratch(). An arena that was outgrown is kept
    // on the `retired` list until the context dies, because captured graphs may still point into it;
    // `scratch_generation` counts the growths.
    void* scratch[2][2];
    size_t scratch_bytes[2][2];
    M40RetiredArena* retired;
    unsigned long long scratch_generation;
    // Last block selection (u32 [q_heads][64] + f32 scores), for the debug read-back.
    uint32_t* d_selected_blocks;
    float* d_selected_scores;
    uint32_t selected_capacity_heads;
    // Device status word (bit 0: a batched-attention row was out of range and skipped).
    uint32_t* d_status;
    unsigned long long launches;
    // Inverse RoPE frequencies per (base, head_dim), made on the host (see m40_rope_inv_freq) and kept on the device.
    float* d_rope_inv_freq[4];
    float rope_table_base[4];
    uint32_t rope_table_hd[4];
    uint32_t rope_tables;
};


struct M40llmCudaGraphExec {
    cudaGraph_t graph;
    cudaGraphExec_t exec;
};

struct M40llmCudaEvent {
    cudaEvent_t event;
};

// ----------------------------------------------------------------------------
// KV cache. Logical layout in the reference is [seq][token][kv_head][d]
// (cuda/kernels.cu:5304-5312). The cache is opaque behind the ABI, so the device
// layout here is head-major: every (slot, kv_head) owns a contiguous
// [tokens][head_dim] matrix. One kv head's K (or V) stream is then a single
// contiguous run in HBM, which is what the decode-attention kernels stream.
//
//   dense       K, V        f16 [slot][kv_head][max_seq_len][hd]
//   compressed  recent_k/v  f16 [slot][kv_head][recent_window][hd]   (token t at t % R)
//               old_k       f16 [slot][kv_head][max_seq_len][hd]     (token t at t)
//               q4_v        u8  [slot][kv_head][max_seq_len][hd/2]
//               q4_scale    f32 [slot][kv_head][max_seq_len]
// ----------------------------------------------------------------------------
struct M40llmKVCache {
    int device_id;
    __half* d_k;
    __half* d_v;
    uint32_t* d_seq_map;  // [max_batch_size] tokens appended per sequence
    __half* d_recent_k;
    __half* d_recent_v;
    __half* d_old_k;
    uint8_t* d_q4_v;
    float* d_q4_scale;
    uint32_t max_seq_len;
    uint32_t max_batch_size;
    uint32_t num_heads;  // kv heads
    uint32_t head_dim;
    uint32_t compressed;
    uint32_t recent_window;
    uint32_t block_size;
    uint32_t max_blocks;
    uint32_t top_blocks;
    uint32_t representatives;
    uint32_t representative_policy;
    uint32_t fp16_k_q4_v_backing;
};

// element offset of (slot, head, token, 0) in a head-major [slot][head][tokens][hd] array
__host__ __device__ __forceinline__ size_t kv_row_offset(uint32_t slot, uint32_t head, uint32_t token,
                                                         uint32_t heads, uint32_t tokens, uint32_t hd) {
    return (((size_t)slot * heads + head) * (size_t)tokens + token) * (size_t)hd;
}

// ----------------------------------------------------------------------------
// Host helpers
// ----------------------------------------------------------------------------
static inline int m40_ensure_device(M40llmCudaContext* ctx) {
    if (!ctx) return -1;
    return cudaSetDevice(ctx->device_id) == cudaSuccess ? 0 : -2;
}

static inline cudaStream_t m40_stream(M40llmCudaContext* ctx, uint32_t kind) {
    if (!ctx) return nullptr;
    if (kind == 0) return ctx->prefill_stream;
    if (kind == 1) return ctx->decode_stream;
    return nullptr;
}

// Returns a scratch pointer of at least `bytes` for the given stream kind, growing the
// arena when needed. Growth allocates (cudaMalloc), so it must not happen during stream
// capture and returns null there: a configuration runs eagerly once before it is captured.
// The outgrown arena stays allocated (retired) so that graphs captured against it remain valid.
void* m40_ensure_scratch(M40llmCudaContext* ctx, uint32_t kind, size_t bytes, uint32_t level = 0);

#define M40_COUNT_LAUNCH(ctx) ((ctx)->launches++)

// ----------------------------------------------------------------------------
// Programmatic dependent launch. A kernel launched through m40_launch_dependent may start while its predecessor
// on the stream is still running; it must execute pdl_wait() before it reads anything the predecessor wrote and
// before its own first global write. Kernels call pdl_trigger() early so that their successor's CTAs are placed
// the moment resources free up. Both are no-ops for plain launches. M40LLM_PDL=0 turns the launch attribute off.
// ----------------------------------------------------------------------------
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_trigger() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

bool m40_pdl_enabled();

template <typename... KArgs, typename... Args>
static inline cudaError_t m40_launch_dependent(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem,
                                               cudaStream_t s, Args&&... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = s;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = m40_pdl_enabled() ? 1 : 0;
    return cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}

__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}

// RoPE angle: theta = float(pos)*freq_scale * powf(base, -2 i / hd)  (cuda/kernels.cu:7322-7327,
// CPU form tests/rmsnorm_rope.rs:43-76). At positions of 1e4..1e5 the angle reaches 1e4..1e5 rad, so one ulp of
// the inverse frequency moves sin/cos by ~1e-3. The host libm's powf is correctly rounded while the device powf
// is only good to a few ulp, so the inverse frequency is evaluated in double and rounded once: this makes the
// device angle equal to the host reference's angle instead of merely close to it.
__device__ __forceinline__ void rope_cs(uint32_t pos, uint32_t pair, uint32_t head_dim, float freq_base,
                                        float freq_scale, float* c, float* s, const float* inv_freq_table = nullptr) {
    const float p = static_cast<float>(pos) * freq_scale;
    float inv_freq;
    if (inv_freq_table) {  // the same value, made on the host (see m40_rope_inv_freq below)
        inv_freq = inv_freq_table[pair];
    } else {
        const float e = -2.0f * static_cast<float>(pair) / static_cast<float>(head_dim);
        inv_freq = static_cast<float>(pow(static_cast<double>(freq_base), static_cast<double>(e)));
    }
    const float theta = p * inv_freq;
    *c = cosf(theta);
    *s = sinf(theta);
}

// Device table of the head_dim / 2 inverse frequencies that rope_cs() evaluates per call: the same float-rounded
// values (the exponent in float, the power in double, rounded once), computed on the host where double precision is
// cheap. On this GPU a double-precision pow per rotation pair costs microseconds. Returns null when no table can be
// made right now (the stream is being captured and this pair of parameters was never seen eagerly; four pairs are
// kept per context): kernels then fall back to rope_cs().
const float* m40_rope_inv_freq(M40llmCudaContext* ctx, float freq_base, uint32_t head_dim);

// softmax scale as the reference kernels spell it (kernels.cu:2869) for 64/128, 1/sqrt otherwise (kernels.cu:1384)
__host__ __device__ __forceinline__ float attn_inv_sqrt(uint32_t head_dim) {
    return head_dim == 64u ? 0.125f : (head_dim == 128u ? 0.08838834764831845f : 1.0f / sqrtf((float)head_dim));
}
