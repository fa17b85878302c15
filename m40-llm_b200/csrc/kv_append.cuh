// Device-side building blocks of the KV append path, shared by the stand-alone append
// entry points (kvcache.cu) and the fused attention prologue (fused.cu).
#pragma once
#include "common.cuh"

// q4 pack of one pair, cuda/kernels.cu:2254-2258
__device__ __forceinline__ uint8_t pack_q4_pair(float a, float b, float scale) {
    const int qa = max(-7, min(7, (int)lrintf(a / scale)));
    const int qb = max(-7, min(7, (int)lrintf(b / scale)));
    return (uint8_t)((qa & 0x0f) | ((qb & 0x0f) << 4));
}

// Quantise one head's V row (f16, hd values) to q4 + scale. Called by all threads of a
// block whose threads [0, hd/2) each own one pair. `red` is shared scratch of >= 32 floats.
__device__ __forceinline__ void quantize_v_row_q4(const __half* __restrict__ v, uint8_t* __restrict__ q4,
                                                  float* __restrict__ scale_out, uint32_t hd, float* red) {
    const uint32_t tid = threadIdx.x;
    float v0 = 0.0f, v1 = 0.0f, mx = 0.0f;
    if (tid < hd / 2u) {
        const __half2 h = reinterpret_cast<const __half2*>(v)[tid];
        v0 = __low2float(h);
        v1 = __high2float(h);
        mx = fmaxf(fabsf(v0), fabsf(v1));
    }
    mx = warp_max(mx);
    if ((tid & 31u) == 0u) red[tid >> 5] = mx;
    __syncthreads();
    float m = 0.0f;
    for (uint32_t i = 0; i < (blockDim.x + 31u) / 32u; ++i) m = fmaxf(m, red[i]);
    const float scale = m > 0.0f ? m / 7.0f : 1.0f / 7.0f;
    if (tid == 0) *scale_out = scale;
    if (tid < hd / 2u) q4[tid] = pack_q4_pair(v0, v1, scale);
    __syncthreads();
}


// Compressed append of one (sequence, kv head, position), executed by a whole 64-thread block
// (cuda/kernels.cu:2230-2311, 5691-5791). If position >= R the ring slot position % R still
// holds token position - R: it moves to the old region (K copied, V quantised to q4) before
// the slot is overwritten with f16(RoPE(k)) and f16(v). k_in/v_in point at this head's hd floats.
__device__ __forceinline__ void kv_append_compressed_head(const M40llmKVCache& kv, uint32_t seq_id, uint32_t head,
                                                          uint32_t position, const float* __restrict__ k_in,
                                                          const float* __restrict__ v_in, float freq_base,
                                                          float freq_scale, uint32_t layout, float* red,
                                                          const float* inv_freq = nullptr) {
    const uint32_t hd = kv.head_dim, half = hd / 2u, R = kv.recent_window, heads = kv.num_heads;
    const uint32_t tid = threadIdx.x;
    const size_t ring_row = kv_row_offset(seq_id, head, position % R, heads, R, hd);
    if (position >= R) {
        const uint32_t old_pos = position - R;
        const size_t old_row = kv_row_offset(seq_id, head, old_pos, heads, kv.max_seq_len, hd);
        if (tid < half)
            reinterpret_cast<__half2*>(kv.d_old_k + old_row)[tid] =
                reinterpret_cast<const __half2*>(kv.d_recent_k + ring_row)[tid];
        const size_t vec = ((size_t)seq_id * heads + head) * (size_t)kv.max_seq_len + old_pos;
        quantize_v_row_q4(kv.d_recent_v + ring_row, kv.d_q4_v + vec * half, kv.d_q4_scale + vec, hd, red);
    }
    if (tid < half) {
        const uint32_t i0 = layout == 1u ? tid : 2u * tid;
        const uint32_t i1 = layout == 1u ? tid + half : 2u * tid + 1u;
        float c, s;
        rope_cs(position, tid, hd, freq_base, freq_scale, &c, &s, inv_freq);
        const float a = k_in[i0], b = k_in[i1];
        kv.d_recent_k[ring_row + i0] = __float2half_rn(a * c - b * s);
        kv.d_recent_k[ring_row + i1] = __float2half_rn(a * s + b * c);
        kv.d_recent_v[ring_row + i0] = __float2half_rn(v_in[i0]);
        kv.d_recent_v[ring_row + i1] = __float2half_rn(v_in[i1]);
    }
    if (head == 0 && tid == 0) kv.d_seq_map[seq_id] = position + 1u;
}

// Dense append of one (sequence, kv head, position) by a block of any size; head_dim even.
__device__ __forceinline__ void kv_append_dense_head(const M40llmKVCache& kv, uint32_t seq_id, uint32_t head,
                                                     uint32_t position, const float* __restrict__ k_in,
                                                     const float* __restrict__ v_in, float freq_base,
                                                     float freq_scale, uint32_t layout,
                                                     const float* inv_freq = nullptr) {
    const uint32_t hd = kv.head_dim, half = hd / 2u;
    const size_t row = kv_row_offset(seq_id, head, position, kv.num_heads, kv.max_seq_len, hd);
    for (uint32_t i = threadIdx.x; i < half; i += blockDim.x) {
        const uint32_t i0 = layout == 1u ? i : 2u * i;
        const uint32_t i1 = layout == 1u ? i + half : 2u * i + 1u;
        float c, s;
        rope_cs(position, i, hd, freq_base, freq_scale, &c, &s, inv_freq);
        const float a = k_in[i0], b = k_in[i1];
        kv.d_k[row + i0] = __float2half_rn(a * c - b * s);
        kv.d_k[row + i1] = __float2half_rn(a * s + b * c);
        kv.d_v[row + i0] = __float2half_rn(v_in[i0]);
        kv.d_v[row + i1] = __float2half_rn(v_in[i1]);
    }
    if (head == 0 && threadIdx.x == 0) kv.d_seq_map[seq_id] = position + 1u;
}
