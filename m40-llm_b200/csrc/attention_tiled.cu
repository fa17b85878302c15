// Tiled decode attention for head_dim 64 and 128 (the shapes of every model configuration).
//
// One CTA (4 warps) owns (row, kv head, token chunk). It streams its K and V rows once through a
// multi-stage cp.async pipeline into XOR-swizzled shared memory (64-token tiles, 16-byte pieces,
// fully coalesced: in the head-major cache a kv head's rows are contiguous). All q heads of the
// kv head's group share that one read. The kernel is HBM-bound by design; the arithmetic runs on
// the tensor cores so that it stays out of the way of the memory pipeline:
//   S = Q K^T   mma.sync m16n8k16, rows = the group's q heads (padded to 16), q split into
//               f16 hi + lo parts so that scores keep f32-level accuracy;
//   softmax     online, base 2, per warp over its 16 tokens of the tile;
//   O += P V    mma.sync with P rounded to f16 (relative error <= 2^-11 per weight).
// Each warp keeps its own (m, l, O) and the four are merged once at the end, so the only CTA-wide
// synchronisation per tile is the pipeline hand-over.
#include "attention.cuh"
#include "attention_mma.cuh"

#include <cooperative_groups.h>

#include <atomic>

namespace cg = cooperative_groups;

namespace {

constexpr int TILE = 64;
using namespace attn_mma;

// Barrier over the 128 threads that stream one token range together: the whole CTA in the batched kernel, one of
// two warp groups (named barrier 1 or 2) in the one-launch row kernel.
struct CtaBarrier {
    __device__ __forceinline__ void sync() const { __syncthreads(); }
};
struct GroupBarrier {
    uint32_t id;
    __device__ __forceinline__ void sync() const { asm volatile("bar.sync %0, 128;" ::"r"(id) : "memory"); }
};

template <int HD, int STAGES_>
struct TiledCfgN {
    static constexpr int CHUNKS = HD / 8;                  // 16-byte pieces per row
    static constexpr int TILE_BYTES = TILE * HD * 2;       // one K (or V) tile
    static constexpr int STAGES = STAGES_;
    static constexpr int SMEM = STAGES * 2 * TILE_BYTES;
};
// The batched kernel keeps two CTAs per SM: 96 KB (hd 128) / 64 KB (hd 64).
template <int HD>
using TiledCfg = TiledCfgN<HD, HD == 128 ? 3 : 4>;

// One 64-token tile of K and V into stage `stage` (all 128 threads; rows past t1 repeat the last row and are masked
// by the consumer).
template <typename Cfg, int HD>
__device__ __forceinline__ void tiled_load_tile(const __half* Kh, const __half* Vh, __half* sK, __half* sV, uint32_t t0,
                                                uint32_t t1, uint32_t tile, uint32_t stage, uint32_t tid) {
    const uint32_t base = t0 + tile * TILE;
    __half* dK = sK + (size_t)stage * TILE * HD;
    __half* dV = sV + (size_t)stage * TILE * HD;
#pragma unroll
    for (int c = 0; c < (TILE * Cfg::CHUNKS) / 128; ++c) {
        const uint32_t idx = c * 128 + tid;
        const uint32_t r = idx / Cfg::CHUNKS, ch = idx % Cfg::CHUNKS;
        uint32_t tok = base + r;
        if (tok >= t1) tok = t1 - 1;  // rows past the end are masked later; keep the read in range
        const size_t src = (size_t)tok * HD + ch * 8;
        const uint32_t dst = r * HD + ((ch ^ (r & 7u)) * 8);
        cp_async16(dK + dst, Kh + src);
        cp_async16(dV + dst, Vh + src);
    }
}

// First STAGES - 1 tiles of [t0, t1) in flight (one commit group per stage, empty groups included).
template <typename Cfg, int HD>
__device__ __forceinline__ void tiled_prefetch(const __half* Kh, const __half* Vh, unsigned char* smem_raw, uint32_t t0,
                                               uint32_t t1, uint32_t tid) {
    __half* sK = reinterpret_cast<__half*>(smem_raw);
    __half* sV = reinterpret_cast<__half*>(smem_raw + Cfg::STAGES * Cfg::TILE_BYTES);
    const uint32_t n_tiles = (t1 - t0 + TILE - 1) / TILE;
#pragma unroll
    for (int s = 0; s < Cfg::STAGES - 1; ++s) {
        if ((uint32_t)s < n_tiles) tiled_load_tile<Cfg, HD>(Kh, Vh, sK, sV, t0, t1, s, s, tid);
        cp_async_commit();
    }
}

// Streams the tokens [t0, t1) of one kv head (tiled_prefetch must have been called) against the group's q heads and
// leaves every warp's (m, l, O) in shared memory: sm_m [4][16], sm_l [4][16], sm_o [4][16][HD] at the start of
// smem_raw (the pipeline buffers are dead by then); m is in the base-2 domain of the pre-scaled q. `q0` points at the
// group's first head ([G][HD] f32, global or shared), rows g >= G are zero. Ends with a CTA barrier.
template <typename Cfg, int HD, bool G_HI, typename Bar>
__device__ __forceinline__ void tiled_stream(const __half* Kh, const __half* Vh, unsigned char* smem_raw, uint32_t t0,
                                             uint32_t t1, const float* q0base, uint32_t G, float inv_sqrt, uint32_t tid,
                                             const Bar bar) {
    constexpr int KS = HD / 16;   // k-steps of Q K^T
    constexpr int NT = HD / 8;    // n8 tiles of the output
    __half* sK = reinterpret_cast<__half*>(smem_raw);
    __half* sV = reinterpret_cast<__half*>(smem_raw + Cfg::STAGES * Cfg::TILE_BYTES);
    const uint32_t warp = tid >> 5, lane = tid & 31u;
    const uint32_t g = lane >> 2, t4 = lane & 3u;

    // ---- Q fragments (A operand), pre-scaled by 1/sqrt(hd) * log2(e), split into hi + lo f16
    uint32_t qhi[KS][G_HI ? 4 : 2], qlo[KS][G_HI ? 4 : 2];
    {
        const float qs = inv_sqrt * LOG2E;
        const float* q0 = q0base + (size_t)g * HD;
        const float* q1 = q0 + (size_t)8 * HD;
#pragma unroll
        for (int ks = 0; ks < KS; ++ks) {
            const int k0 = ks * 16 + 2 * t4;
            float2 x0 = make_float2(0.f, 0.f), x2 = x0, x1 = x0, x3 = x0;
            if (g < G) {
                x0 = *reinterpret_cast<const float2*>(q0 + k0);
                x2 = *reinterpret_cast<const float2*>(q0 + k0 + 8);
            }
            split_h2(x0.x * qs, x0.y * qs, &qhi[ks][0], &qlo[ks][0]);
            split_h2(x2.x * qs, x2.y * qs, &qhi[ks][G_HI ? 2 : 1], &qlo[ks][G_HI ? 2 : 1]);
            if (G_HI) {
                if (g + 8 < G) {
                    x1 = *reinterpret_cast<const float2*>(q1 + k0);
                    x3 = *reinterpret_cast<const float2*>(q1 + k0 + 8);
                }
                split_h2(x1.x * qs, x1.y * qs, &qhi[ks][1], &qlo[ks][1]);
                split_h2(x3.x * qs, x3.y * qs, &qhi[ks][3], &qlo[ks][3]);
            }
        }
    }

    float o[NT][4];
#pragma unroll
    for (int n = 0; n < NT; ++n) o[n][0] = o[n][1] = o[n][2] = o[n][3] = 0.0f;
    float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.0f, 0.0f};

    const uint32_t n_tiles = (t1 - t0 + TILE - 1) / TILE;
    for (uint32_t tile = 0; tile < n_tiles; ++tile) {
        cp_async_wait<Cfg::STAGES - 2>();
        bar.sync();
        {
            const uint32_t nxt = tile + Cfg::STAGES - 1;
            if (nxt < n_tiles) tiled_load_tile<Cfg, HD>(Kh, Vh, sK, sV, t0, t1, nxt, nxt % Cfg::STAGES, tid);
            cp_async_commit();
        }
        const uint32_t stage = tile % Cfg::STAGES;
        const __half* tK = sK + (size_t)stage * TILE * HD;
        const __half* tV = sV + (size_t)stage * TILE * HD;

        // ---- S = Q K^T for this warp's 16 tokens
        float s0[4] = {0.f, 0.f, 0.f, 0.f}, s1[4] = {0.f, 0.f, 0.f, 0.f};
        {
            const uint32_t j = lane >> 3;  // which 8x8 matrix this lane addresses
            const uint32_t r = warp * 16 + (j >> 1) * 8 + (lane & 7u);
#pragma unroll
            for (int ks = 0; ks < KS; ++ks) {
                const uint32_t ch = ks * 2 + (j & 1u);
                uint32_t b[4];
                ldmatrix_x4(b, tK + r * HD + ((ch ^ (r & 7u)) * 8));
                const uint32_t a1h = G_HI ? qhi[ks][1] : 0u, a3h = G_HI ? qhi[ks][3] : 0u;
                const uint32_t a1l = G_HI ? qlo[ks][1] : 0u, a3l = G_HI ? qlo[ks][3] : 0u;
                const uint32_t a2h = qhi[ks][G_HI ? 2 : 1], a2l = qlo[ks][G_HI ? 2 : 1];
                mma16816(s0, qhi[ks][0], a1h, a2h, a3h, b[0], b[1]);
                mma16816(s0, qlo[ks][0], a1l, a2l, a3l, b[0], b[1]);
                mma16816(s1, qhi[ks][0], a1h, a2h, a3h, b[2], b[3]);
                mma16816(s1, qlo[ks][0], a1l, a2l, a3l, b[2], b[3]);
            }
        }
        // ---- mask tokens past the end, online softmax (base 2)
        const uint32_t tok0 = t0 + tile * TILE + warp * 16 + 2 * t4;
        if (tok0 >= t1) { s0[0] = -INFINITY; s0[2] = -INFINITY; }
        if (tok0 + 1 >= t1) { s0[1] = -INFINITY; s0[3] = -INFINITY; }
        if (tok0 + 8 >= t1) { s1[0] = -INFINITY; s1[2] = -INFINITY; }
        if (tok0 + 9 >= t1) { s1[1] = -INFINITY; s1[3] = -INFINITY; }
        uint32_t pa[4];
#pragma unroll
        for (int h = 0; h < (G_HI ? 2 : 1); ++h) {
            float mx = fmaxf(fmaxf(s0[2 * h], s0[2 * h + 1]), fmaxf(s1[2 * h], s1[2 * h + 1]));
            mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
            mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
            const float m_new = fmaxf(m_run[h], mx);
            const float m_use = m_new == -INFINITY ? 0.0f : m_new;
            const float corr = fast_exp2(m_run[h] - m_use);
            const float p00 = fast_exp2(s0[2 * h] - m_use), p01 = fast_exp2(s0[2 * h + 1] - m_use);
            const float p10 = fast_exp2(s1[2 * h] - m_use), p11 = fast_exp2(s1[2 * h + 1] - m_use);
            float rs = (p00 + p01) + (p10 + p11);
            rs += __shfl_xor_sync(0xffffffffu, rs, 1);
            rs += __shfl_xor_sync(0xffffffffu, rs, 2);
            l_run[h] = l_run[h] * corr + rs;
            m_run[h] = m_new;
#pragma unroll
            for (int n = 0; n < NT; ++n) {
                o[n][2 * h] *= corr;
                o[n][2 * h + 1] *= corr;
            }
            pa[h] = pack_h2(p00, p01);       // A[row g (+8h)][k = 2t, 2t+1]
            pa[2 + h] = pack_h2(p10, p11);   // A[row g (+8h)][k = 8+2t, 9+2t]
        }
        if (!G_HI) { pa[1] = 0u; pa[3] = 0u; }
        // ---- O += P V
        {
            const uint32_t j = lane >> 3;
            const uint32_t r = warp * 16 + (j & 1u) * 8 + (lane & 7u);
#pragma unroll
            for (int nd = 0; nd < HD / 16; ++nd) {
                const uint32_t ch = nd * 2 + (j >> 1);
                uint32_t b[4];
                ldmatrix_x4_trans(b, tV + r * HD + ((ch ^ (r & 7u)) * 8));
                mma16816(o[2 * nd], pa[0], pa[1], pa[2], pa[3], b[0], b[1]);
                mma16816(o[2 * nd + 1], pa[0], pa[1], pa[2], pa[3], b[2], b[3]);
            }
        }
    }
    cp_async_wait<0>();
    bar.sync();

    // ---- the four warps' partials through shared memory (reusing the pipeline buffers)
    float* sm_m = reinterpret_cast<float*>(smem_raw);  // [4][16]
    float* sm_l = sm_m + 64;                           // [4][16]
    float* sm_o = sm_l + 64;                           // [4][16][HD]
    if (t4 == 0) {
        sm_m[warp * 16 + g] = m_run[0];
        sm_l[warp * 16 + g] = l_run[0];
        sm_m[warp * 16 + g + 8] = G_HI ? m_run[1] : -INFINITY;
        sm_l[warp * 16 + g + 8] = G_HI ? l_run[1] : 0.0f;
    }
#pragma unroll
    for (int n = 0; n < NT; ++n) {
        float* dst = sm_o + ((size_t)warp * 16 + g) * HD + n * 8 + 2 * t4;
        dst[0] = o[n][0];
        dst[1] = o[n][1];
        if (G_HI) {
            dst[8 * HD] = o[n][2];
            dst[8 * HD + 1] = o[n][3];
        }
    }
    bar.sync();
}

// G_HI: the group has more than 8 q heads (rows 8..15 of the MMA are live).
template <int HD, bool G_HI>
__global__ void __launch_bounds__(128, 2) attn_decode_tiled_kernel(DenseAttnArgs a) {
    using Cfg = TiledCfg<HD>;
    extern __shared__ __align__(128) unsigned char smem_raw[];

    pdl_wait();     // q and the newest cache row come from the previous kernel
    pdl_trigger();
    const uint32_t split = blockIdx.x, kvh = blockIdx.y, row = blockIdx.z;
    const uint32_t tid = threadIdx.x;
    const uint32_t G = a.q_heads / a.kv_heads;
    uint32_t seq = 0, t0 = 0, t1 = 0;
    const bool partial = a.write_partials || a.splits > 1;
    if (!attn_resolve_row(a, row, split, &seq, &t0, &t1)) {
        attn_write_rejected_row(a, row, split, kvh, partial);
        return;
    }
    if (t0 >= t1) {  // nothing in this chunk: an empty partial (l = 0) that the merge ignores
        if (partial) {
            for (uint32_t i = tid; i < G; i += blockDim.x) {
                const size_t pi = ((size_t)row * a.q_heads + kvh * G + i) * a.splits + split;
                a.part_m[pi] = -INFINITY;
                a.part_l[pi] = 0.0f;
            }
        }
        return;
    }
    const __half* Kh = a.K + kv_row_offset(seq, kvh, 0, a.kv_heads, a.max_seq_len, HD);
    const __half* Vh = a.V + kv_row_offset(seq, kvh, 0, a.kv_heads, a.max_seq_len, HD);
    tiled_prefetch<Cfg, HD>(Kh, Vh, smem_raw, t0, t1, tid);
    tiled_stream<Cfg, HD, G_HI>(Kh, Vh, smem_raw, t0, t1, a.q + ((size_t)row * a.q_heads + kvh * G) * HD, G, a.inv_sqrt, tid,
                                CtaBarrier{});

    const float* sm_m = reinterpret_cast<const float*>(smem_raw);
    const float* sm_l = sm_m + 64;
    const float* sm_o = sm_l + 64;
    for (uint32_t idx = tid; idx < G * HD; idx += blockDim.x) {
        const uint32_t hh = idx / HD, d = idx % HD;
        float M = -INFINITY;
#pragma unroll
        for (int w = 0; w < 4; ++w) M = fmaxf(M, sm_m[w * 16 + hh]);
        float L = 0.0f, O = 0.0f;
#pragma unroll
        for (int w = 0; w < 4; ++w) {
            const float mw = sm_m[w * 16 + hh];
            const float e = mw == -INFINITY ? 0.0f : fast_exp2(mw - M);
            L += sm_l[w * 16 + hh] * e;
            O += sm_o[((size_t)w * 16 + hh) * HD + d] * e;
        }
        const uint32_t head = kvh * G + hh;
        if (partial) {
            const size_t pi = ((size_t)row * a.q_heads + head) * a.splits + split;
            if (d == 0) {
                a.part_m[pi] = M * LN2;  // back to the natural-log domain the merge kernels use
                a.part_l[pi] = L;
            }
            a.part_o[pi * HD + d] = O;
        } else {
            a.out[((size_t)row * a.q_heads + head) * HD + d] = O / (L > 0.0f ? L : 1.0f);
        }
    }
}

// ---------------------------------------------------------------------------------------------------------------
// Single-launch decode attention for rows whose new token is being appended in the same step: RoPE of q, RoPE of k +
// f16 append of k / v, attention over the cache and over the new token, and the merge of the token splits.
//
// One thread-block CLUSTER of CL CTAs owns (row, kv head); each CTA's two warp groups stream one slice each of the
// tokens already in the cache, [0, position), exactly as a CTA of the batched kernel does. The new token never makes the round trip through the
// cache: the last CTA of the cluster rotates k, stores the f16 rows for later steps and attends the f16-rounded values
// straight from shared memory as one more partial. The CL partial (m, l, O) triples then meet through distributed
// shared memory: every CTA reduces 1/CL of the outputs over its peers' triples and writes the normalised result. No
// partials in global memory, no merge launch, no rope / append launch.
//
// The rotation table (cos, sin per pair) costs a double-precision pow per pair; it is computed once per CTA while the
// first K/V tiles are already in flight.
// ---------------------------------------------------------------------------------------------------------------
struct FusedRowArgs {
    __half* K;
    __half* V;
    uint32_t* seq_map;
    const float* q_raw;   // [rows][q_heads][hd]  before RoPE
    const float* k_new;   // [rows][kv_heads][hd] before RoPE
    const float* v_new;   // [rows][kv_heads][hd]
    float* q_out;         // [rows][q_heads][hd]  after RoPE (what the separate prologue would have written)
    float* out;           // [rows][q_heads][hd]
    const uint32_t* seq_ids;
    const uint32_t* positions;
    const uint32_t* seq_lens;
    uint32_t* status;
    const float* inv_freq;  // [hd / 2] host-made table, or null: evaluate the power on the device
    uint32_t max_seq_len, max_batch, kv_heads, q_heads, layout;
    float freq_base, freq_scale, inv_sqrt;
};

constexpr int FUSED_CL = 16;  // CTAs per cluster (non-portable size; needs the opt-in attribute)
constexpr int FUSED_WG = 2;   // warp groups per CTA, each streaming its own half of the CTA's slice

// One CTA per SM: two warp groups with 96 KB of pipeline each. (A single group of four warps per CTA tops out near
// 20 GB/s, so 16 x kv_heads CTAs alone would leave most of HBM idle.)
template <int HD>
using FusedCfg = TiledCfgN<HD, HD == 128 ? 3 : 6>;

template <int HD, bool G_HI>
__global__ void __launch_bounds__(128 * FUSED_WG, 1) attn_decode_fused_row_kernel(FusedRowArgs a) {
    using Cfg = FusedCfg<HD>;
    constexpr uint32_t HALF = HD / 2;
    constexpr uint32_t NW = 4 * FUSED_WG;  // warps holding a partial
    extern __shared__ __align__(128) unsigned char smem_raw[];
    __shared__ float2 s_cs[HALF];                  // (cos, sin) per pair at this row's position
    __shared__ __align__(16) float s_q[16][HD];    // rotated q of the group (rows >= G stay zero)
    __shared__ float s_kn[HD], s_vn[HD];           // the new token's k (rotated) and v, rounded through f16
    __shared__ float s_new[16];                    // its score per q head, base-2 domain
    cg::cluster_group cluster = cg::this_cluster();
    const uint32_t rank = blockIdx.x, kvh = blockIdx.y, row = blockIdx.z;
    const uint32_t tid = threadIdx.x, warp = tid >> 5, lane = tid & 31u;
    const uint32_t wg = tid >> 7, gtid = tid & 127u;
    const uint32_t G = a.q_heads / a.kv_heads;

    pdl_wait();  // q, k, v of this step come from the projection kernel before this one
    pdl_trigger();
    const uint32_t seq = a.seq_ids[row], pos = a.positions[row], len = a.seq_lens[row];
    // every CTA of the cluster sees the same row, so this exit is taken by all of them or by none
    if (seq >= a.max_batch || pos >= a.max_seq_len || len != pos + 1u) {
        if (tid == 0 && rank == 0 && kvh == 0) atomicOr(a.status, seq >= a.max_batch || len != pos + 1u ? 1u : 2u);
        if (rank == 0)
            for (uint32_t i = tid; i < G * HD; i += blockDim.x) a.out[((size_t)row * a.q_heads + kvh * G) * HD + i] = 0.0f;
        return;
    }
    // tokens already in the cache: [0, pos), cut into CL x WG slices of whole 64-token tiles
    uint32_t chunk = (pos + FUSED_CL * FUSED_WG - 1) / (FUSED_CL * FUSED_WG);
    chunk = (chunk + TILE - 1) / TILE * TILE;
    const uint32_t t0 = min((rank * FUSED_WG + wg) * chunk, pos), t1 = min(t0 + chunk, pos);
    __half* Kh = a.K + kv_row_offset(seq, kvh, 0, a.kv_heads, a.max_seq_len, HD);
    __half* Vh = a.V + kv_row_offset(seq, kvh, 0, a.kv_heads, a.max_seq_len, HD);
    unsigned char* my_smem = smem_raw + (size_t)wg * Cfg::SMEM;
    tiled_prefetch<Cfg, HD>(Kh, Vh, my_smem, t0, t1, gtid);

    // ---- rotation table, rotated q, and (last CTA) the new token
    if (tid < HALF) {
        float c, sn;
        if (a.inv_freq) {  // the same angle as rope_cs, its power taken from the table
            const float theta = (static_cast<float>(pos) * a.freq_scale) * a.inv_freq[tid];
            c = cosf(theta);
            sn = sinf(theta);
        } else {
            rope_cs(pos, tid, HD, a.freq_base, a.freq_scale, &c, &sn);
        }
        s_cs[tid] = make_float2(c, sn);
    }
    for (uint32_t i = tid; i < 16 * HD; i += blockDim.x) (&s_q[0][0])[i] = 0.0f;
    __syncthreads();
    const float* qg = a.q_raw + ((size_t)row * a.q_heads + kvh * G) * HD;
    float* qo = a.q_out + ((size_t)row * a.q_heads + kvh * G) * HD;
    for (uint32_t idx = tid; idx < G * HALF; idx += blockDim.x) {
        const uint32_t hh = idx / HALF, i = idx % HALF;
        const uint32_t i0 = a.layout == 1u ? i : 2u * i, i1 = a.layout == 1u ? i + HALF : 2u * i + 1u;
        const float2 cs = s_cs[i];
        const float x = qg[hh * HD + i0], y = qg[hh * HD + i1];
        const float r0 = x * cs.x - y * cs.y, r1 = x * cs.y + y * cs.x;
        s_q[hh][i0] = r0;
        s_q[hh][i1] = r1;
        if (rank == 0) {
            qo[hh * HD + i0] = r0;
            qo[hh * HD + i1] = r1;
        }
    }
    const bool has_new = rank == FUSED_CL - 1;
    if (has_new && tid >= 128u && tid - 128u < HALF) {  // second warp group: the first is busy with q
        const uint32_t i = tid - 128u;
        const uint32_t i0 = a.layout == 1u ? i : 2u * i, i1 = a.layout == 1u ? i + HALF : 2u * i + 1u;
        const float* kn = a.k_new + ((size_t)row * a.kv_heads + kvh) * HD;
        const float* vn = a.v_new + ((size_t)row * a.kv_heads + kvh) * HD;
        const float2 cs = s_cs[i];
        const float x = kn[i0], y = kn[i1];
        const __half k0 = __float2half_rn(x * cs.x - y * cs.y), k1 = __float2half_rn(x * cs.y + y * cs.x);
        const __half v0 = __float2half_rn(vn[i0]), v1 = __float2half_rn(vn[i1]);
        const size_t rowoff = (size_t)pos * HD;
        Kh[rowoff + i0] = k0, Kh[rowoff + i1] = k1;
        Vh[rowoff + i0] = v0, Vh[rowoff + i1] = v1;
        s_kn[i0] = __half2float(k0), s_kn[i1] = __half2float(k1);
        s_vn[i0] = __half2float(v0), s_vn[i1] = __half2float(v1);
        if (kvh == 0 && i == 0) a.seq_map[seq] = pos + 1u;
    }
    __syncthreads();
    if (has_new) {  // score of the new token per q head, in the base-2 domain of the streamed scores
        for (uint32_t hh = warp; hh < G; hh += NW) {
            float dot = 0.0f;
            for (uint32_t d = lane; d < HD; d += 32u) dot = fmaf(s_q[hh][d], s_kn[d], dot);
            dot = warp_sum(dot);
            if (lane == 0) s_new[hh] = dot * (a.inv_sqrt * LOG2E);
        }
    }

    // ---- the cached tokens of this warp group's slice
    tiled_stream<Cfg, HD, G_HI>(Kh, Vh, my_smem, t0, t1, &s_q[0][0], G, a.inv_sqrt, gtid, GroupBarrier{1u + wg});
    __syncthreads();  // both groups' partials (and s_new) are in shared memory

    // ---- this CTA's triple per q head: c_m [16], c_l [16], c_o [16][HD] behind the first group's warp partials
    float* c_m = reinterpret_cast<float*>(smem_raw) + 128 + 4 * 16 * HD;
    float* c_l = c_m + 16;
    float* c_o = c_l + 16;
    for (uint32_t idx = tid; idx < G * HD; idx += blockDim.x) {
        const uint32_t hh = idx / HD, d = idx % HD;
        float M = has_new ? s_new[hh] : -INFINITY;
#pragma unroll
        for (uint32_t w = 0; w < NW; ++w) {
            const float* gm = reinterpret_cast<const float*>(smem_raw + (size_t)(w >> 2) * Cfg::SMEM);
            M = fmaxf(M, gm[(w & 3u) * 16 + hh]);
        }
        float L = 0.0f, O = 0.0f;
#pragma unroll
        for (uint32_t w = 0; w < NW; ++w) {
            const float* gm = reinterpret_cast<const float*>(smem_raw + (size_t)(w >> 2) * Cfg::SMEM);
            const float mw = gm[(w & 3u) * 16 + hh];
            const float e = mw == -INFINITY ? 0.0f : fast_exp2(mw - M);
            L += gm[64 + (w & 3u) * 16 + hh] * e;
            O += gm[128 + ((size_t)(w & 3u) * 16 + hh) * HD + d] * e;
        }
        if (has_new) {
            const float e = fast_exp2(s_new[hh] - M);
            L += e;
            O = fmaf(e, s_vn[d], O);
        }
        if (d == 0) {
            c_m[hh] = M;
            c_l[hh] = L;
        }
        c_o[hh * HD + d] = O;
    }
    cluster.sync();

    // ---- cluster merge: this CTA finishes outputs [rank * per, rank * per + per) of the group's G * HD
    const uint32_t per = (G * HD + FUSED_CL - 1) / FUSED_CL;
    for (uint32_t j = tid; j < per; j += blockDim.x) {
        const uint32_t idx = rank * per + j;
        if (idx >= G * HD) break;
        const uint32_t hh = idx / HD, d = idx % HD;
        float pm[FUSED_CL], pl[FUSED_CL], po[FUSED_CL];
#pragma unroll
        for (int c = 0; c < FUSED_CL; ++c) {  // all remote loads go out before any is used
            const float* rm = cluster.map_shared_rank(c_m, c);
            pm[c] = rm[hh];
            pl[c] = rm[16 + hh];
            po[c] = rm[32 + hh * HD + d];
        }
        float M = -INFINITY;
#pragma unroll
        for (int c = 0; c < FUSED_CL; ++c) M = fmaxf(M, pl[c] > 0.0f ? pm[c] : -INFINITY);
        float L = 0.0f, O = 0.0f;
#pragma unroll
        for (int c = 0; c < FUSED_CL; ++c) {
            const float e = pl[c] > 0.0f ? fast_exp2(pm[c] - M) : 0.0f;
            L = fmaf(pl[c], e, L);
            O = fmaf(po[c], e, O);
        }
        a.out[((size_t)row * a.q_heads + kvh * G + hh) * HD + d] = O / (L > 0.0f ? L : 1.0f);
    }
    cluster.sync();  // peers may still be reading this CTA's triples
}

template <int HD, bool G_HI>
int launch_fused_row(M40llmCudaContext* ctx, const FusedRowArgs& a, uint32_t rows) {
    auto kern = attn_decode_fused_row_kernel<HD, G_HI>;
    constexpr size_t smem = (size_t)FUSED_WG * FusedCfg<HD>::SMEM;
    static_assert(FusedCfg<HD>::SMEM >= (size_t)(128 + 4 * 16 * HD + 32 + 16 * HD) * sizeof(float),
                  "partials must fit one group's pipeline buffers");
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(FUSED_CL, a.kv_heads, rows);
    cfg.blockDim = dim3(128 * FUSED_WG);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = ctx->decode_stream;
    cudaLaunchAttribute attr[2];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = FUSED_CL;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[1].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    // per device: 0 = not tried, 1 = usable, 2 = this device cannot co-schedule such a cluster
    static std::atomic<unsigned char> state[64];
    const int dev = ctx->device_id & 63;
    unsigned char st = state[dev].load(std::memory_order_acquire);
    if (st == 0) {
        st = 2;
        if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) == cudaSuccess &&
            cudaFuncSetAttribute(kern, cudaFuncAttributeNonPortableClusterSizeAllowed, 1) == cudaSuccess) {
            int clusters = 0;
            cfg.numAttrs = 1;
            if (cudaOccupancyMaxActiveClusters(&clusters, kern, &cfg) == cudaSuccess && clusters >= 1) st = 1;
        }
        cudaGetLastError();
        state[dev].store(st, std::memory_order_release);
    }
    if (st != 1) return 1;
    cfg.numAttrs = m40_pdl_enabled() ? 2 : 1;
    const cudaError_t e = cudaLaunchKernelEx(&cfg, kern, a);
    M40_COUNT_LAUNCH(ctx);
    return e == cudaSuccess && cudaGetLastError() == cudaSuccess ? 0 : -4;
}

template <int HD, bool G_HI>
int launch(M40llmCudaContext* ctx, const DenseAttnArgs& a, uint32_t rows) {
    auto kern = attn_decode_tiled_kernel<HD, G_HI>;
    // per-device bit: the attribute is per device. Contexts on several threads may race to set it; setting it twice
    // is harmless, losing a bit is not, hence the atomic.
    static std::atomic<unsigned long long> configured{0ull};
    const unsigned long long bit = 1ull << (ctx->device_id & 63);
    if (!(configured.load(std::memory_order_acquire) & bit)) {
        if (cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, TiledCfg<HD>::SMEM) != cudaSuccess)
            return -4;
        configured.fetch_or(bit, std::memory_order_release);
    }
    dim3 grid(a.splits, a.kv_heads, rows);
    const cudaError_t e = m40_launch_dependent(kern, grid, dim3(128), (size_t)TiledCfg<HD>::SMEM, ctx->decode_stream, a);
    M40_COUNT_LAUNCH(ctx);
    return e == cudaSuccess && cudaGetLastError() == cudaSuccess ? 0 : -4;
}

}  // namespace

int m40_attention_dense_tiled(M40llmCudaContext* ctx, const DenseAttnArgs& a, uint32_t rows) {
    const uint32_t G = a.q_heads / a.kv_heads;
    if ((a.hd != 64 && a.hd != 128) || G > 16) return 1;
    if ((((uintptr_t)a.q) & 7u) != 0u) return 1;  // float2 loads of q
    if (a.hd == 128) return G > 8 ? launch<128, true>(ctx, a, rows) : launch<128, false>(ctx, a, rows);
    return G > 8 ? launch<64, true>(ctx, a, rows) : launch<64, false>(ctx, a, rows);
}

// Rows whose new token arrives with the call (q, k, v before RoPE; positions[r] + 1 == seq_lens[r]): rotates q (also
// written to q_out), appends k / v and attends, all in one launch. Returns 1 when the shape or the device does not
// take the cluster kernel (head_dim 64 / 128, at most 16 q heads per kv head, 8-byte aligned q).
int m40_attention_fused_row(M40llmCudaContext* ctx, M40llmKVCache* kv, const float* q_raw, const float* k_new,
                            const float* v_new, const uint32_t* seq_ids, const uint32_t* positions,
                            const uint32_t* seq_lens, uint32_t rows, uint32_t q_heads, float freq_base,
                            float freq_scale, uint32_t layout, float* q_out, float* out) {
    const uint32_t G = q_heads / kv->num_heads;
    if ((kv->head_dim != 64 && kv->head_dim != 128) || G > 16 || kv->compressed || !kv->d_k || !kv->d_v) return 1;
    FusedRowArgs a = {};
    a.K = kv->d_k;
    a.V = kv->d_v;
    a.seq_map = kv->d_seq_map;
    a.q_raw = q_raw;
    a.k_new = k_new;
    a.v_new = v_new;
    a.q_out = q_out;
    a.out = out;
    a.seq_ids = seq_ids;
    a.positions = positions;
    a.seq_lens = seq_lens;
    a.status = ctx->d_status;
    a.inv_freq = m40_rope_inv_freq(ctx, freq_base, kv->head_dim);
    a.max_seq_len = kv->max_seq_len;
    a.max_batch = kv->max_batch_size;
    a.kv_heads = kv->num_heads;
    a.q_heads = q_heads;
    a.layout = layout;
    a.freq_base = freq_base;
    a.freq_scale = freq_scale;
    a.inv_sqrt = attn_inv_sqrt(kv->head_dim);
    if (kv->head_dim == 128) return G > 8 ? launch_fused_row<128, true>(ctx, a, rows) : launch_fused_row<128, false>(ctx, a, rows);
    return G > 8 ? launch_fused_row<64, true>(ctx, a, rows) : launch_fused_row<64, false>(ctx, a, rows);
}
