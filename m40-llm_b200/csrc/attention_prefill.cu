// Packed variable-length prefill attention (causal, GQA) over f32 Q / K / V.
//
// Reference semantics (cuda/kernels.cu:3749-3835, host entry :4834-4977): sequence b owns q rows
// [q_offsets[b], +q_lens[b]) of Q [total_q][q_heads][hd] and kv rows [kv_offsets[b], +kv_lens[b]) of K, V
// [total_kv][kv_heads][hd]; q row i attends kv rows 0 .. kv_len - q_len + i; softmax scaled by 1/sqrt(hd); the
// reference runs one CTA per (q row, head) with a three-pass softmax in f32.
//
// Here K and V are first rounded to f16 once, by a streaming pass into stream scratch (every kv row is converted once,
// not once per q tile and q head). Then one CTA owns 64 q rows of one (sequence, q head) and walks the kv rows it may
// see in 64-row tiles, flash attention style: the f16 tiles arrive by cp.async into double-buffered, XOR-swizzled
// shared memory while the previous tile is being used, S = Q K^T and O += P V run on mma.sync m16n8k16 with f32
// accumulation (q split into f16 hi + lo so that the scores keep f32-level accuracy, P rounded to f16), and the
// softmax is online, base 2, in registers. Every kv row is read once per 64 q rows instead of once per q row.
#include "attention_mma.cuh"
#include "common.cuh"

namespace {
using namespace attn_mma;

constexpr int PF_TILE = 64;  // q rows per CTA and kv rows per tile

// K, V f32 [n8 * 8] -> f16, 8 values per thread and array.
__global__ void __launch_bounds__(256) prefill_pack_kv_kernel(const float* __restrict__ K, const float* __restrict__ V,
                                                              __half* __restrict__ Kh, __half* __restrict__ Vh, size_t n8) {
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n8; i += (size_t)gridDim.x * blockDim.x) {
        const float4 k0 = *reinterpret_cast<const float4*>(K + 8 * i), k1 = *reinterpret_cast<const float4*>(K + 8 * i + 4);
        const float4 v0 = *reinterpret_cast<const float4*>(V + 8 * i), v1 = *reinterpret_cast<const float4*>(V + 8 * i + 4);
        *reinterpret_cast<uint4*>(Kh + 8 * i) =
            make_uint4(pack_h2(k0.x, k0.y), pack_h2(k0.z, k0.w), pack_h2(k1.x, k1.y), pack_h2(k1.z, k1.w));
        *reinterpret_cast<uint4*>(Vh + 8 * i) =
            make_uint4(pack_h2(v0.x, v0.y), pack_h2(v0.z, v0.w), pack_h2(v1.x, v1.y), pack_h2(v1.z, v1.w));
    }
}

template <int HD>
__global__ void __launch_bounds__(128, 2) prefill_varlen_kernel(const float* __restrict__ Q, const __half* __restrict__ K,
                                                                const __half* __restrict__ V,
                                                                const uint32_t* __restrict__ q_offsets,
                                                                const uint32_t* __restrict__ kv_offsets,
                                                                const uint32_t* __restrict__ q_lens,
                                                                const uint32_t* __restrict__ kv_lens, uint32_t q_heads,
                                                                uint32_t kv_heads, float inv_sqrt, float* __restrict__ Out) {
    constexpr int KS = HD / 16;      // k-steps of Q K^T
    constexpr int NT = HD / 8;       // n8 tiles of the output
    constexpr int CHUNKS = HD / 8;   // 16-byte f16 pieces per row
    extern __shared__ __align__(128) __half pf_smem[];  // [2 buffers][K tile | V tile]
    constexpr uint32_t TILE_ELEMS = PF_TILE * HD;
    // the last q tiles of a sequence see the most kv rows: they are scheduled first (block index reversed)
    const uint32_t b = blockIdx.z, qh = blockIdx.y, r0 = (gridDim.x - 1u - blockIdx.x) * PF_TILE;
    const uint32_t q_len = q_lens[b], kv_len = kv_lens[b];
    if (r0 >= q_len || q_len == 0 || kv_len == 0 || q_len > kv_len) return;
    const uint32_t tid = threadIdx.x, warp = tid >> 5, lane = tid & 31u;
    const uint32_t g = lane >> 2, t4 = lane & 3u;
    const uint32_t kvh = qh / (q_heads / kv_heads);
    const size_t q_row0 = (size_t)q_offsets[b] + r0, kv_row0 = kv_offsets[b];
    const uint32_t shift = kv_len - q_len;  // q row i sees kv rows 0 .. shift + i
    // rows of this thread: r0 + warp * 16 + g and + 8
    const uint32_t row_a = r0 + warp * 16u + g, row_b = row_a + 8u;

    // ---- Q fragments (A operand), pre-scaled by 1/sqrt(hd) * log2(e), split into hi + lo f16
    uint32_t qhi[KS][4], qlo[KS][4];
    {
        const float qs = inv_sqrt * LOG2E;
        const float* qa = Q + ((q_row0 + warp * 16u + g) * q_heads + qh) * HD;
        const float* qb = qa + (size_t)8 * q_heads * HD;
#pragma unroll
        for (int ks = 0; ks < KS; ++ks) {
            const int k0 = ks * 16 + 2 * t4;
            float2 x0 = make_float2(0.f, 0.f), x1 = x0, x2 = x0, x3 = x0;
            if (row_a < q_len) {
                x0 = *reinterpret_cast<const float2*>(qa + k0);
                x2 = *reinterpret_cast<const float2*>(qa + k0 + 8);
            }
            if (row_b < q_len) {
                x1 = *reinterpret_cast<const float2*>(qb + k0);
                x3 = *reinterpret_cast<const float2*>(qb + k0 + 8);
            }
            split_h2(x0.x * qs, x0.y * qs, &qhi[ks][0], &qlo[ks][0]);
            split_h2(x1.x * qs, x1.y * qs, &qhi[ks][1], &qlo[ks][1]);
            split_h2(x2.x * qs, x2.y * qs, &qhi[ks][2], &qlo[ks][2]);
            split_h2(x3.x * qs, x3.y * qs, &qhi[ks][3], &qlo[ks][3]);
        }
    }
    float o[NT][4];
#pragma unroll
    for (int n = 0; n < NT; ++n) o[n][0] = o[n][1] = o[n][2] = o[n][3] = 0.0f;
    float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.0f, 0.0f};

    // kv rows this q tile may see: 0 .. shift + (last q row of the tile)
    const uint32_t last_q = min(r0 + PF_TILE, q_len) - 1u;
    const uint32_t kv_end = shift + last_q + 1u;
    const uint32_t n_tiles = (kv_end + PF_TILE - 1) / PF_TILE;
    // K and V rows of a tile: f16 global -> shared by cp.async (rows past the end repeat the last visible row: they are
    // masked below, and their bytes are finite)
    auto load_tile = [&](uint32_t tile, uint32_t buf) {
        const uint32_t base = tile * PF_TILE;
        __half* dK = pf_smem + (size_t)buf * 2 * TILE_ELEMS;
        __half* dV = dK + TILE_ELEMS;
#pragma unroll
        for (int c = 0; c < (PF_TILE * CHUNKS) / 128; ++c) {
            const uint32_t idx = c * 128 + tid;
            const uint32_t r = idx / CHUNKS, ch = idx % CHUNKS;
            const uint32_t dst = r * HD + ((ch ^ (r & 7u)) * 8);
            const uint32_t row = min(base + r, kv_end - 1u);
            const size_t src = ((kv_row0 + row) * kv_heads + kvh) * HD + ch * 8;
            cp_async16(dK + dst, K + src);
            cp_async16(dV + dst, V + src);
        }
        cp_async_commit();
    };
    load_tile(0, 0);
    for (uint32_t tile = 0; tile < n_tiles; ++tile) {
        const uint32_t base = tile * PF_TILE;
        cp_async_wait<0>();
        __syncthreads();  // this tile has landed for every thread, and the other buffer's tile has been consumed
        if (tile + 1 < n_tiles) load_tile(tile + 1, (tile + 1) & 1u);
        const __half* sK = pf_smem + (size_t)(tile & 1u) * 2 * TILE_ELEMS;
        const __half* sV = sK + TILE_ELEMS;
        // a warp whose 16 rows all sit before this tile's first kv row has nothing to add (causal)
        if (shift + min(r0 + warp * 16u + 15u, q_len - 1u) < base) continue;

        // ---- S = Q K^T: this warp's 16 rows against the tile's 64 kv rows (8 n-tiles of 8)
        float s[8][4];
#pragma unroll
        for (int j = 0; j < 8; ++j) s[j][0] = s[j][1] = s[j][2] = s[j][3] = 0.0f;
        {
            const uint32_t jm = lane >> 3;  // which 8x8 matrix this lane addresses
#pragma unroll
            for (int p = 0; p < 4; ++p) {
                const uint32_t r = p * 16 + (jm >> 1) * 8 + (lane & 7u);
#pragma unroll
                for (int ks = 0; ks < KS; ++ks) {
                    const uint32_t ch = ks * 2 + (jm & 1u);
                    uint32_t bb[4];
                    ldmatrix_x4(bb, sK + r * HD + ((ch ^ (r & 7u)) * 8));
                    mma16816(s[2 * p], qhi[ks][0], qhi[ks][1], qhi[ks][2], qhi[ks][3], bb[0], bb[1]);
                    mma16816(s[2 * p], qlo[ks][0], qlo[ks][1], qlo[ks][2], qlo[ks][3], bb[0], bb[1]);
                    mma16816(s[2 * p + 1], qhi[ks][0], qhi[ks][1], qhi[ks][2], qhi[ks][3], bb[2], bb[3]);
                    mma16816(s[2 * p + 1], qlo[ks][0], qlo[ks][1], qlo[ks][2], qlo[ks][3], bb[2], bb[3]);
                }
            }
        }
        // ---- causal mask and online softmax (base 2); c0, c1 belong to row_a, c2, c3 to row_b
        const uint32_t lim_a = row_a < q_len ? shift + row_a : 0u, lim_b = row_b < q_len ? shift + row_b : 0u;
        const bool live_a = row_a < q_len, live_b = row_b < q_len;
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            const uint32_t t = base + j * 8 + 2 * t4;
            if (!live_a || t > lim_a) s[j][0] = -INFINITY;
            if (!live_a || t + 1 > lim_a) s[j][1] = -INFINITY;
            if (!live_b || t > lim_b) s[j][2] = -INFINITY;
            if (!live_b || t + 1 > lim_b) s[j][3] = -INFINITY;
        }
        uint32_t pa[4][4];  // P as A fragments: [k-step of 16 kv rows][a0..a3]
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            float mx = -INFINITY;
#pragma unroll
            for (int j = 0; j < 8; ++j) mx = fmaxf(mx, fmaxf(s[j][2 * h], s[j][2 * h + 1]));
            mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
            mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
            const float m_new = fmaxf(m_run[h], mx);
            const float m_use = m_new == -INFINITY ? 0.0f : m_new;
            const float corr = fast_exp2(m_run[h] - m_use);
            float rs = 0.0f;
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                const float p0 = fast_exp2(s[j][2 * h] - m_use), p1 = fast_exp2(s[j][2 * h + 1] - m_use);
                rs += p0 + p1;
                // n-tile j = k-step j / 2, low (a0 / a1) or high (a2 / a3) half; row h picks a0 / a2 vs a1 / a3
                pa[j >> 1][(j & 1) * 2 + h] = pack_h2(p0, p1);
            }
            rs += __shfl_xor_sync(0xffffffffu, rs, 1);
            rs += __shfl_xor_sync(0xffffffffu, rs, 2);
            l_run[h] = l_run[h] * corr + rs;
            m_run[h] = m_new;
#pragma unroll
            for (int n = 0; n < NT; ++n) {
                o[n][2 * h] *= corr;
                o[n][2 * h + 1] *= corr;
            }
        }
        // ---- O += P V
        {
            const uint32_t jm = lane >> 3;
#pragma unroll
            for (int kk = 0; kk < 4; ++kk) {
                const uint32_t r = kk * 16 + (jm & 1u) * 8 + (lane & 7u);
#pragma unroll
                for (int nd = 0; nd < HD / 16; ++nd) {
                    const uint32_t ch = nd * 2 + (jm >> 1);
                    uint32_t bb[4];
                    ldmatrix_x4_trans(bb, sV + r * HD + ((ch ^ (r & 7u)) * 8));
                    mma16816(o[2 * nd], pa[kk][0], pa[kk][1], pa[kk][2], pa[kk][3], bb[0], bb[1]);
                    mma16816(o[2 * nd + 1], pa[kk][0], pa[kk][1], pa[kk][2], pa[kk][3], bb[2], bb[3]);
                }
            }
        }
    }
    // ---- normalise and store
    const float inv_a = 1.0f / (l_run[0] > 0.0f ? l_run[0] : 1.0f), inv_b = 1.0f / (l_run[1] > 0.0f ? l_run[1] : 1.0f);
    float* oa = Out + ((q_row0 + warp * 16u + g) * q_heads + qh) * HD;
    float* ob = oa + (size_t)8 * q_heads * HD;
#pragma unroll
    for (int n = 0; n < NT; ++n) {
        if (row_a < q_len) *reinterpret_cast<float2*>(oa + n * 8 + 2 * t4) = make_float2(o[n][0] * inv_a, o[n][1] * inv_a);
        if (row_b < q_len) *reinterpret_cast<float2*>(ob + n * 8 + 2 * t4) = make_float2(o[n][2] * inv_b, o[n][3] * inv_b);
    }
}

}  // namespace

extern "C" {

int m40llm_attention_prefill_f32_gqa_varlen_async(M40llmCudaContext* ctx, const void* d_q_f32, const void* d_k_f32,
                                                  const void* d_v_f32, const uint32_t* d_q_offsets,
                                                  const uint32_t* d_kv_offsets, const uint32_t* d_q_lens,
                                                  const uint32_t* d_kv_lens, uint32_t batch_size, uint32_t q_heads,
                                                  uint32_t kv_heads, uint32_t head_dim, void* d_out_f32) {
    if (!ctx || !d_q_f32 || !d_k_f32 || !d_v_f32 || !d_q_offsets || !d_kv_offsets || !d_q_lens || !d_kv_lens ||
        !d_out_f32)
        return -1;
    if (batch_size == 0) return -2;
    if (q_heads == 0 || kv_heads == 0 || q_heads % kv_heads != 0) return -3;
    if (head_dim != 64 && head_dim != 128) return -9;
    if (((((uintptr_t)d_q_f32) | ((uintptr_t)d_k_f32) | ((uintptr_t)d_v_f32) | ((uintptr_t)d_out_f32)) & 15u) != 0u) return -9;
    if (m40_ensure_device(ctx) != 0) return -1;
    cudaStream_t s = ctx->prefill_stream;
    // The grid needs the longest q run, and the reference validates every pair of lengths on the host
    // (kernels.cu:4861-4886): the lengths are read back behind whatever the prefill stream still holds.
    uint32_t* lens = (uint32_t*)malloc((size_t)batch_size * 3 * sizeof(uint32_t));
    if (!lens) return -7;
    int rc = 0;
    uint32_t max_q = 0;
    uint64_t total_kv = 0;  // rows of K / V the sequences reach: the extent of the f16 copies
    if (cudaMemcpyAsync(lens, d_q_lens, (size_t)batch_size * 4, cudaMemcpyDeviceToHost, s) != cudaSuccess ||
        cudaMemcpyAsync(lens + batch_size, d_kv_lens, (size_t)batch_size * 4, cudaMemcpyDeviceToHost, s) != cudaSuccess ||
        cudaMemcpyAsync(lens + 2 * batch_size, d_kv_offsets, (size_t)batch_size * 4, cudaMemcpyDeviceToHost, s) != cudaSuccess ||
        cudaStreamSynchronize(s) != cudaSuccess) {
        cudaGetLastError();
        rc = -7;
    }
    for (uint32_t i = 0; rc == 0 && i < batch_size; ++i) {
        const uint32_t ql = lens[i], kl = lens[batch_size + i];
        if (ql == 0 || kl == 0 || ql > kl || kl > 8192) rc = -8;
        if (ql > max_q) max_q = ql;
        const uint64_t end = (uint64_t)lens[2 * batch_size + i] + kl;
        if (end > total_kv) total_kv = end;
    }
    free(lens);
    if (rc != 0) return rc;
    // f16 copies of K and V in the prefill stream's scratch
    const size_t kv_elems = (size_t)total_kv * kv_heads * head_dim;
    __half* kh = (__half*)m40_ensure_scratch(ctx, 0, 2 * kv_elems * sizeof(__half));
    if (!kh) return -7;
    __half* vh = kh + kv_elems;
    {
        const size_t n8 = kv_elems / 8;
        const unsigned blocks = (unsigned)((n8 + 255) / 256 < (size_t)ctx->sm_count * 8 ? (n8 + 255) / 256 : (size_t)ctx->sm_count * 8);
        prefill_pack_kv_kernel<<<blocks ? blocks : 1u, 256, 0, s>>>((const float*)d_k_f32, (const float*)d_v_f32, kh, vh, n8);
        M40_COUNT_LAUNCH(ctx);
    }
    dim3 grid((max_q + PF_TILE - 1) / PF_TILE, q_heads, batch_size);
    const float inv_sqrt = attn_inv_sqrt(head_dim);
    const size_t smem = (size_t)2 * 2 * PF_TILE * head_dim * sizeof(__half);
    static unsigned long long configured = 0ull;
    const unsigned long long bit = 1ull << (ctx->device_id & 63);
    if (!(configured & bit)) {
        if (cudaFuncSetAttribute(prefill_varlen_kernel<128>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                 (int)(2 * 2 * PF_TILE * 128 * sizeof(__half))) != cudaSuccess)
            return -4;
        configured |= bit;
    }
    if (head_dim == 128)
        prefill_varlen_kernel<128><<<grid, 128, smem, s>>>((const float*)d_q_f32, kh, vh, d_q_offsets, d_kv_offsets, d_q_lens,
                                                           d_kv_lens, q_heads, kv_heads, inv_sqrt, (float*)d_out_f32);
    else
        prefill_varlen_kernel<64><<<grid, 128, smem, s>>>((const float*)d_q_f32, kh, vh, d_q_offsets, d_kv_offsets, d_q_lens,
                                                          d_kv_lens, q_heads, kv_heads, inv_sqrt, (float*)d_out_f32);
    M40_COUNT_LAUNCH(ctx);
    return cudaGetLastError() == cudaSuccess ? 0 : -4;
}

int m40llm_attention_prefill_f32_gqa_varlen(M40llmCudaContext* ctx, const void* d_q_f32, const void* d_k_f32,
                                            const void* d_v_f32, const uint32_t* d_q_offsets,
                                            const uint32_t* d_kv_offsets, const uint32_t* d_q_lens,
                                            const uint32_t* d_kv_lens, uint32_t batch_size, uint32_t q_heads,
                                            uint32_t kv_heads, uint32_t head_dim, void* d_out_f32) {
    const int rc = m40llm_attention_prefill_f32_gqa_varlen_async(ctx, d_q_f32, d_k_f32, d_v_f32, d_q_offsets, d_kv_offsets,
                                                                 d_q_lens, d_kv_lens, batch_size, q_heads, kv_heads, head_dim,
                                                                 d_out_f32);
    if (rc != 0) return rc;
    return cudaStreamSynchronize(ctx->prefill_stream) == cudaSuccess ? 0 : -5;
}

}  // extern "C"
